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
    __shared__ FitShared s_fs;
    fill_fit_shared(&s_fs, m, a);
    const int lane = threadIdx.x & 31;
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t layer_words = (size_t)a.max_nodes * m.MW;
    unsigned arrivals = a.barrier_base;

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
        arrivals += gridDim.x * a.world;
        if (!grid_barrier(a, arrivals)) return;
    }
    const bool timer = a.timers != 0 && blockIdx.x == 0 && threadIdx.x == 0;
    long long t_eval = 0, t_bar = 0, t_tot = 0, t_fb = 0, t_clauses = 0, t_merge = 0, t_stage = 0, t0 = clock64(), t1;

    u64 step = 0;
    for (int ep = 0; ep < a.epochs; ++ep) {
        for (int64_t i = 0; i < a.count; ++i, ++step) {
            const int64_t e = a.first + i;
            const int par = (int)(step & 1);
            GraphView gv = global_graph(g, e, m.L0);
            u32 *P = par ? a.P_pair[1] : a.P_pair[0];
            const u32 *s_rows = nullptr;              // shared-memory copy of the message rows the current layer reads
            if (s_graph != nullptr) {
                // layout: literal rows [kFitStageRowWords] | type, degree, CSR start [3][32] | edge rows [2*kFitStageEdges] | message rows [32*MW]
                const u32 ge0 = g.graph_edge0[e], gne = g.graph_edges[e];
                if (gv.n <= 32 && gv.n * m.L0 <= kFitStageRowWords && gne <= (u32)kFitStageEdges && ge0 + gne <= g.total_edges) {
                    u32 *st_x = s_graph, *st_t = st_x + kFitStageRowWords, *st_d = st_t + 32, *st_i = st_d + 32, *st_e = st_i + 32;
                    for (int t = threadIdx.x; t < gv.n * m.L0; t += blockDim.x) st_x[t] = gv.X[t];
                    for (int t = threadIdx.x; t < gv.n; t += blockDim.x) { st_t[t] = gv.type[t]; st_d[t] = gv.degree[t]; st_i[t] = gv.eidx[t]; }
                    for (int t = threadIdx.x; t < 2 * (int)gne; t += blockDim.x) st_e[t] = g.edge[2 * (size_t)ge0 + t];
                    gv.X = st_x; gv.type = st_t; gv.degree = st_d; gv.eidx = st_i; gv.edge = st_e; gv.e_off = ge0; gv.e_cnt = gne;
                    s_rows = st_e + 2 * kFitStageEdges;
                    __syncthreads();
                }
            }

            for (int d = 0; d < m.D; ++d) {
                const bool last = d == m.D - 1;
                if (d > 0) {
                    GTM_LAP(t_eval);
                    arrivals += gridDim.x * a.world;
                    if (!grid_barrier(a, arrivals)) return;
                    GTM_LAP(t_bar);
                    if (d == 1) clear_next_messages(m, a, par ? a.P_pair[0] : a.P_pair[1], (int)g.n_nodes[i + 1 < a.count ? e + 1 : a.first]);
                    if (s_rows != nullptr) {          // the messages of the layer below are complete: this CTA's copy of them
                        u32 *dst = const_cast<u32 *>(s_rows);
                        const u32 *src = P + (size_t)(d - 1) * layer_words;
                        __syncthreads();              // the previous layer's readers are done
                        for (int t = threadIdx.x; t < gv.n * m.MW; t += blockDim.x) dst[t] = __ldcg(src + t);
                        __syncthreads();
                    }
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
                                                      d > 0 ? (s_rows != nullptr ? s_rows : P + (size_t)(d - 1) * layer_words) : nullptr,
                                                      last ? nullptr : &targets, lane);
                    if (last && any)
                        for (int k = lane; k < m.K; k += 32) atomicAdd(&s_sum[k], m.weights[(size_t)k * m.C + c]);
                }
                GTM_LAP(t_clauses);
                if (targets.local) {        // this CTA's share of the layer's messages, merged before the grid barrier
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
                __syncthreads();
                for (int c = a.c_begin + gwarp; c < a.c_end; c += nwarps) {
                    const ClauseView cv = global_view(m, sc.n_inc, c);
                    clause_feedback<MAXSB>(m, gv, cv, a, cno_row(sc, m.C, m.D - 1, c), P, s_target, s_thr, c, lane,
                                           s_pack[threadIdx.x >> 5], s_fs.p_mask);
                }
            }
            __syncthreads();   // s_total is rewritten by the next graph
            GTM_LAP(t_fb);
        }
    }
    if (timer) {
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
