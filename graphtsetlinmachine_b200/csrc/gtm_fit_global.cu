// Learning kernel with the model state in global memory (any model size; also the debug path).
#include "../../include/gtm_b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>

#include "gtm_handles.h"
#include "gtm_fit.cuh"

namespace gtm {

// Persistent learning kernel, state in global memory: the whole grid works on one graph at a time (online
// learning is sequential over graphs, tm.py:668-747); warps own clauses (clause c belongs to global warp c mod
// #warps for the whole launch, so automata and weights of a clause are only ever touched by one warp).  Per
// graph: layer evaluations separated by grid barriers (messages mix all clauses), one exchange of per-CTA vote
// partials, then clause-local feedback.  Serves any model size; also the debug path that keeps every layer.
template <int MAXSB, bool kBatchNodes>
__global__ void __launch_bounds__(512, 1) fit_kernel(DevModel m, DevGraphs g, EvalScratch sc, FitArgs a, int eval_only)
{
    extern __shared__ int s_mem[];   // [K] running partial, [K] totals, [K] targets, [K] thresholds
    int *s_sum = s_mem, *s_total = s_mem + m.K, *s_target = s_mem + 2 * m.K;
    float *s_thr = reinterpret_cast<float *>(s_mem + 3 * m.K);
    u32 *s_part = a.part_words > 0 ? reinterpret_cast<u32 *>(s_mem + ((4 * m.K + 3) & ~3)) : nullptr;   // message accumulation
    // small graphs (at most 32 nodes) are copied to shared memory once per step, and so are the message rows a layer
    // reads: a clause evaluation then waits for shared memory instead of for L2
    u32 *s_graph = a.gstage_words > 0 ? reinterpret_cast<u32 *>(s_mem + ((4 * m.K + 3) & ~3)) + max(a.part_words, 0) : nullptr;
    __shared__ u32 s_pack[16][kPackWords];
    __shared__ int s_next;                        // next clause of the CTA that gets its feedback
    __shared__ FitShared s_fs;
    fill_fit_shared(&s_fs, m, a);
    const int lane = threadIdx.x & 31;
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t layer_words = (size_t)a.max_nodes * m.MW;
    unsigned nb = a.barriers_done;           // barriers passed so far, see grid_barrier

    for (int k = threadIdx.x; k < m.K; k += blockDim.x) s_sum[k] = 0;
    for (int t = threadIdx.x; t < a.part_words; t += blockDim.x) s_part[t] = 0;
    __syncthreads();
    if (a.world > 1 && m.D > 1) {
        // clause-sharded start: every rank clears its own message buffers (peers will OR into them), then all ranks meet
        const size_t words = (size_t)(m.D - 1) * a.max_nodes * m.MW;
        for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < words; t += (size_t)gridDim.x * blockDim.x) {
            a.P_pair[0][t] = 0;
            a.P_pair[1][t] = 0;
        }
        if (!grid_barrier(a, ++nb)) return;
    }
    // the whole first warp of CTA 0 reads the clock (a warp-uniform branch: one timing lane would serialise against the
    // other 31 and count their instructions as its own); lane 0 reports
    const bool timer = a.timers != 0 && blockIdx.x == 0 && threadIdx.x < 32;
    long long t_eval = 0, t_bar = 0, t_tot = 0, t_fb = 0, t_clauses = 0, t_merge = 0, t_stage = 0, t0 = clock64(), t1;

    // Small graphs are staged one step ahead (two buffers), their sizes two steps ahead (a ring of three): the copies are
    // issued at the start of a step and have the whole step to land.  Fetched at the start of its own step instead, a
    // graph's dependent loads (index arrays, then rows) would queue behind the automaton write-back of the step before.
    __shared__ int s_size[3][4];                  // n, first node, first edge row, edge rows
    const u64 steps = (u64)a.epochs * (u64)a.count;
    int64_t e_cur = a.first, e_nxt = a.count > 1 ? a.first + 1 : a.first, e_nxt2 = a.count > 2 ? a.first + 2 : a.first;
    auto advance = [&](int64_t e) { return e + 1 < a.first + a.count ? e + 1 : a.first; };
    auto stage_fits = [&](const int *sz) {
        return s_graph != nullptr && sz[0] <= 32 && sz[0] * m.L0 <= kFitStageRowWords && (u32)sz[3] <= (u32)kFitStageEdges &&
               (u64)(u32)sz[2] + (u32)sz[3] <= g.total_edges;
    };
    auto fetch_sizes = [&](u64 st, int64_t e) {
        if (s_graph != nullptr && threadIdx.x < 4 && st < steps) {
            const u32 *src = threadIdx.x == 0 ? g.n_nodes : threadIdx.x == 1 ? g.node_index : threadIdx.x == 2 ? g.graph_edge0 : g.graph_edges;
            async_copy_word(reinterpret_cast<u32 *>(&s_size[(u32)st % 3u][threadIdx.x]), src + e);
        }
    };
    auto fetch_graph = [&](u64 st) {                // sizes of step st are in s_size[st % 3]
        if (s_graph == nullptr || st >= steps) return;
        const int *sz = s_size[(u32)st % 3u];
        if (!stage_fits(sz)) return;
        const int n = sz[0], base = sz[1], e0 = sz[2], ne = sz[3];
        u32 *st_x = s_graph + (st & 1) * kFitStageGraphWords, *st_t = st_x + kFitStageRowWords, *st_d = st_t + 32, *st_i = st_d + 32, *st_e = st_i + 32;
        for (int t = threadIdx.x; t < n * m.L0; t += blockDim.x) async_copy_word(st_x + t, g.X + (size_t)base * m.L0 + t);
        for (int t = threadIdx.x; t < n; t += blockDim.x) {
            async_copy_word(st_t + t, g.node_type + base + t);
            async_copy_word(st_d + t, g.degree + base + t);
            async_copy_word(st_i + t, g.edge_index + base + t);
        }
        for (int t = threadIdx.x; t < 2 * ne; t += blockDim.x) async_copy_word(st_e + t, g.edge + 2 * (size_t)e0 + t);
    };
    auto wait_copies = [&]() { asm volatile("cp.async.wait_all;" ::: "memory"); };
    fetch_sizes(0, e_cur);
    fetch_sizes(1, e_nxt);
    wait_copies();
    __syncthreads();
    fetch_graph(0);
    wait_copies();
    __syncthreads();

    int slot3 = 0;   // step % 3
    for (u64 step = 0; step < steps; ++step) {
        {
            const int64_t e = e_cur;
            const int par = (int)(step & 1);
            GraphView gv;
            u32 *P = par ? a.P_pair[1] : a.P_pair[0];
            const u32 *s_rows = nullptr;              // shared-memory copy of the message rows the current layer reads
            if (s_graph == nullptr || !stage_fits(s_size[slot3])) {
                gv = global_graph(g, e, m.L0);
            } else {
                // layout: [2] x (literal rows [kFitStageRowWords] | type, degree, CSR start [3][32] | edge rows [2*kFitStageEdges]) | message rows [D-1][32][MW]
                u32 *st_x = s_graph + par * kFitStageGraphWords, *st_t = st_x + kFitStageRowWords, *st_d = st_t + 32, *st_i = st_d + 32, *st_e = st_i + 32;
                gv.n = s_size[slot3][0];
                gv.X = st_x; gv.type = st_t; gv.degree = st_d; gv.eidx = st_i; gv.edge = st_e;
                gv.e_off = (u32)s_size[slot3][2]; gv.e_cnt = (u32)s_size[slot3][3];
                s_rows = s_graph + 2 * kFitStageGraphWords;
            }
            // staged (small) graphs: the CTAs merge their source-node marks and build the message rows themselves (flush_marks)
            const bool merged_marks = s_rows != nullptr && s_part != nullptr && (32 + kTransposedTypes) * (m.MW | 1) <= a.part_words;
            const u32 *rows_base = merged_marks ? s_rows : P;              // message rows [D-1][rows_nodes][MW] of this graph
            const int rows_nodes = merged_marks ? 32 : a.max_nodes;
            fetch_graph(step + 1);                    // lands in the other buffer while this step runs
            fetch_sizes(step + 2, e_nxt2);

            for (int d = 0; d < m.D; ++d) {
                const bool last = d == m.D - 1;
                if (d > 0) {
                    GTM_LAP(t_eval);
                    if (!grid_barrier(a, ++nb)) return;
                    GTM_LAP(t_bar);
                    if (d == 1) clear_next_messages(m, a, par ? a.P_pair[0] : a.P_pair[1], step + 1 < steps ? (int)g.n_nodes[e_nxt] : 0);
                    // the marks of the layer below are complete: this CTA's message rows from them
                    if (merged_marks) build_message_rows(P + (size_t)(d - 1) * layer_words, s_part, const_cast<u32 *>(s_rows) + (size_t)(d - 1) * 32 * m.MW, gv, m.MS, m.MW);
                }
                GTM_LAP(t_stage);
                ScatterTargets targets;
                targets.world = a.world;
                targets.rank = a.rank;
                targets.local_words = 0;
                targets.all = nullptr;
                targets.local = (!last && s_part != nullptr && ((gv.n + 31) & ~31) * (m.MW | 1) <= a.part_words) ? s_part : nullptr;
                #pragma unroll
                for (int r = 0; r < kMaxRanks; ++r) targets.base[r] = (par ? s_fs.P_peer[r][1] : s_fs.P_peer[r][0]) + (size_t)d * layer_words;
                for (int c = a.c_begin + gwarp; c < a.c_end; c += nwarps) {
                    const ClauseView cv = global_view(m, sc.n_inc, c);
                    if (c + nwarps < a.c_end) {       // the next clause's include words are on their way while this one is evaluated
                        const int Wd = d == 0 ? m.L0 : m.M;
                        const u32 *nxt = (d == 0 ? m.ta0 + (size_t)(c + nwarps) * m.SB * m.L0
                                                 : m.tam + ((size_t)(d - 1) * m.C + (c + nwarps)) * m.SB * m.M) + (size_t)(m.SB - 1) * Wd;
                        if (lane * 32 < Wd) asm volatile("prefetch.global.L2 [%0];" ::"l"(nxt + lane * 32));
                    }
                    const u32 any = eval_clause_layer<kBatchNodes>(m, gv, g.n_types, cv, c, d, d > 0 ? cno_row(sc, m.C, d - 1, c) : nullptr,
                                                      cno_row(sc, m.C, d, c),
                                                      d > 0 ? rows_base + (size_t)(d - 1) * rows_nodes * m.MW : nullptr,
                                                      last ? nullptr : &targets, lane);
                    if (last && any)
                        for (int k = lane; k < m.K; k += 32) atomicAdd(&s_sum[k], m.weights[(size_t)k * m.C + c]);
                }
                GTM_LAP(t_clauses);
                if (targets.local && merged_marks) {
                    __syncthreads();
                    flush_marks(targets, gv, m.MW);   // build_message_rows reuses and clears the buffer after the grid barrier
                    GTM_LAP(t_merge);
                } else if (targets.local) { // this CTA's share of the layer's messages, merged before the grid barrier
                    __syncthreads();
                    flush_messages(targets, gv, m.MS, m.MW);
                    __syncthreads();
                    for (int t = threadIdx.x; t < ((gv.n + 31) & ~31) * (m.MW | 1); t += blockDim.x) targets.local[t] = 0;
                    GTM_LAP(t_merge);
                }
            }
            __syncthreads();
            GTM_LAP(t_eval);
            if (!exchange_class_sums(a, step, par, a.tag_base + (u32)step + 1u, s_sum, s_total, m.K)) return;
            GTM_LAP(t_tot);
            if (!eval_only) {
                class_decision_inputs(m, s_total, a.Y + (size_t)e * m.K, s_target, s_thr);
                if (threadIdx.x == 0) s_next = 0;
                __syncthreads();
                // The CTA's clauses (those its warps evaluated) are handed out one at a time to whichever warp is free:
                // a clause with Type I feedback costs tens of Philox rounds, one without costs next to nothing, and a
                // fixed assignment leaves most warps waiting for the unluckiest one.  Everything a clause owns is in
                // global memory and was last written by this CTA before a CTA barrier.
                const int warps_cta = (int)(blockDim.x >> 5);
                const int rounds = (a.c_end - a.c_begin + nwarps - 1) / nwarps;
                while (true) {
                    int j = 0;
                    if (lane == 0) j = atomicAdd(&s_next, 1);
                    j = __shfl_sync(kFull, j, 0);
                    if (j >= rounds * warps_cta) break;
                    const int c = a.c_begin + (int)blockIdx.x * warps_cta + (j % warps_cta) + (j / warps_cta) * nwarps;
                    if (c >= a.c_end) continue;
                    const ClauseView cv = global_view(m, sc.n_inc, c);
                    clause_feedback<MAXSB>(m, gv, cv, a, cno_row(sc, m.C, m.D - 1, c), rows_base, rows_nodes, s_target, s_thr, c, lane,
                                           s_pack[threadIdx.x >> 5], s_fs.p_mask);
                }
            }
            wait_copies();
            __syncthreads();   // s_total is rewritten by the next graph; the next graph's copy is complete
            GTM_LAP(t_fb);
            e_cur = e_nxt; e_nxt = e_nxt2; e_nxt2 = advance(e_nxt2);
            slot3 = slot3 == 2 ? 0 : slot3 + 1;
        }
    }
    if (timer && threadIdx.x == 0) {
        a.phase_cycles[0] = (unsigned long long)t_eval; a.phase_cycles[1] = (unsigned long long)t_bar;
        a.phase_cycles[2] = (unsigned long long)t_tot; a.phase_cycles[3] = (unsigned long long)t_fb;
        a.phase_cycles[4] = (unsigned long long)t_clauses; a.phase_cycles[5] = (unsigned long long)t_merge;
        a.phase_cycles[6] = (unsigned long long)t_stage; a.phase_cycles[7] = 0;
    }
}

#undef GTM_LAP

}  // namespace gtm

const void *fit_global_kernel(int state_bits, bool batch_nodes)
{
    if (batch_nodes) return state_bits <= 8 ? (const void *)fit_kernel<8, true> : (const void *)fit_kernel<32, true>;
    return state_bits <= 8 ? (const void *)fit_kernel<8, false> : (const void *)fit_kernel<32, false>;
}
