// State-resident learning kernel and the launch logic of both learning kernels.
#include "../../include/gtm_b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>

#include "gtm_handles.h"
#include "gtm_fit.cuh"

const void *fit_global_kernel(int state_bits, bool batch_nodes);   // gtm_fit_global.cu

namespace gtm {

// Staging limits of the state-resident kernel: a graph is copied to shared memory one step ahead when it has at
// most kStageNodes nodes, kStageRowWords literal words and kStageEdges edge rows; larger graphs are read in place.
constexpr int kStageNodes = 256, kStageRowWords = 1536, kStageEdges = 512;
constexpr int kStageWords = kStageRowWords + 3 * kStageNodes + 2 * kStageEdges;
constexpr int kRecWords = 38;   // per clause and step: chosen node, Type-I classes, draw position (2), work items, feedback type (before the decisions: uniform) of 32 classes, bit offset of layer 0's first draw in its mask stream

// State-resident learning kernel.  Same schedule as fit_kernel, but everything a clause owns lives in the shared
// memory of the CTA that owns the clause for the whole launch: automaton planes of every layer, weights, message
// hypervector, draw counter, include count and the node-output words.  The graph of the NEXT step (rows, node
// types, CSR slice, targets) is copied into shared memory with cp.async while the current step runs, and the
// sizes of the step after that are fetched too, so that no step starts with a chain of dependent global loads.
// Per graph the remaining global traffic is the vote exchange and, for depth > 1, the merged marks and message rows.
// State is loaded at the start of the launch and written back at its end.
// One step (graph): copies of the next graph issued -> per layer: [grid barrier, message rows from the merged marks]
// evaluation of the CTA's clauses, marks sent -> votes published -> (narrow layers) node choice, decision uniforms
// and the first mask rounds while the votes travel -> votes collected -> decisions -> remaining masks and automaton
// updates as work items over all warps -> CTA barrier.
// Launch bounds: the register budget of 768 threads (85) is also that of two CTAs of 384 threads per SM; a CTA that has
// its SM to itself is launched with a warp per clause, up to 24.
//   shared memory: [K] vote partial | [K] totals | [2][K] targets | [3][4] graph sizes | [2] staged graphs |
//                  [warps] per-warp mask scratch | per-clause decision records, work-item offsets and pre-generated mask words |
//                  per owned clause: clause_words words =
//                  draw counter (2) | include count (1) | pad (1) | weights [K] | hypervector [MB] | node words [2][NC] | planes
template <int MAXSB, bool kBatchNodes, bool kOneLayer>
__global__ void __launch_bounds__(768, 1) fit_resident_kernel(DevModel m_in, DevGraphs g, FitArgs a)
{
    // kOneLayer: the depth is the compile-time constant 1, which removes the message passing, the grid barriers and the
    // message-layer feedback from the code (the one-layer variant is 40 % smaller; measured +13 % graphs/s on 2,500
    // clauses over single-node graphs).
    DevModel m = m_in;
    if (kOneLayer) m.D = 1;
    extern __shared__ __align__(16) int s_mem[];
    __shared__ FitShared s_fs;
    fill_fit_shared(&s_fs, m, a);
    const int KP = (m.K + 3) & ~3;
    int *s_sum = s_mem, *s_total = s_mem + KP, *s_y = s_mem + 2 * KP;      // s_y: [2][KP]
    int *s_target = s_mem + 4 * KP;
    float *s_thr = reinterpret_cast<float *>(s_mem + 5 * KP);
    int *s_size = s_mem + 6 * KP;                                           // [3][4]: n, first node, first edge row, edge rows
    u32 *s_stage = reinterpret_cast<u32 *>(s_size + 12);                    // [2][kStageWords]
    u32 *s_pack = s_stage + (a.stage ? 2 * kStageWords : 0);                                // [warps][kPackWords]
    int *s_rec = reinterpret_cast<int *>(s_pack + (blockDim.x >> 5) * kPackWords);       // [clauses_per_cta][kRecWords] decisions of the step
    int *s_item_off = s_rec + (size_t)a.clauses_per_cta * kRecWords;       // work-item table: entries, items, then (clause, first item) pairs
    u32 *s_pre = reinterpret_cast<u32 *>(s_item_off + 2 * a.clauses_per_cta + 2);   // [clauses_per_cta][pre_words]
    u32 *s_clauses = s_pre + (size_t)a.clauses_per_cta * a.pre_words;
    // one CTA learns the whole model: messages stay in shared memory, CTA barriers replace the grid-wide steps
    const bool solo = a.solo != 0;
    u32 *P_even = a.P_pair[0], *P_odd = a.P_pair[1];
    if (a.p_smem_words > 0) {
        P_even = s_clauses + (size_t)a.clauses_per_cta * a.clause_words;
        P_odd = P_even + a.p_smem_words;
        for (int t = threadIdx.x; t < 2 * a.p_smem_words; t += blockDim.x) P_even[t] = 0;
        if (threadIdx.x == 0) { s_fs.P_peer[0][0] = P_even; s_fs.P_peer[0][1] = P_odd; }
    }
    u32 *s_part = nullptr;      // message accumulation of one layer (clause-shared buffers are then touched once per word)
    if (a.part_words > 0) {
        s_part = s_clauses + (size_t)a.clauses_per_cta * a.clause_words;
        for (int t = threadIdx.x; t < a.part_words; t += blockDim.x) s_part[t] = 0;
    }
    // transposed copy of the current graph (graphs of 33..1024 nodes): literal rows, then node-type masks
    const int t_rows = 32 * max(m.L0, m.MW);
    u32 *s_T = s_clauses + (size_t)a.clauses_per_cta * a.clause_words + a.part_words + 2 * a.p_smem_words;
    // message rows [D-1][32][MW] that the CTA builds from the merged marks (graph sets of at most 32 nodes)
    u32 *s_rows = a.rows_words > 0 ? s_T + (a.t_stride > 0 ? (size_t)(t_rows + kTransposedTypes) * a.t_stride : 0) : nullptr;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int c_lo = min(a.c_end, a.c_begin + (int)blockIdx.x * a.clauses_per_cta), c_hi = min(a.c_end, c_lo + a.clauses_per_cta);
    const size_t layer_words = (size_t)a.max_nodes * m.MW;
    const int NC = a.NC;
    const u64 steps = (u64)a.epochs * (u64)a.count;
    unsigned nb = a.barriers_done;           // barriers passed so far, see grid_barrier
    unsigned nb_rank = 0;                    // and those among this rank's CTAs only, see rank_barrier

    auto view_of = [&](int c) {
        u32 *basep = s_clauses + (size_t)(c - c_lo) * a.clause_words;
        ClauseView cv;
        cv.pos = reinterpret_cast<u64 *>(basep);
        cv.n_inc = reinterpret_cast<int *>(basep + 2);
        cv.wgt = reinterpret_cast<int *>(basep + 4);
        cv.wstride = 1;
        cv.hv = basep + 4 + m.K;
        cv.ta0 = basep + 4 + m.K + m.MB + 2 * NC;
        cv.tam = cv.ta0 + (size_t)m.SB * m.L0;
        cv.tam_stride = (size_t)m.SB * m.M;
        return cv;
    };
    auto node_words = [&](int c, int d) { return s_clauses + (size_t)(c - c_lo) * a.clause_words + 4 + m.K + m.MB + (d & 1) * NC; };
    // graphs of the current step and of the two steps after it (wrapping at the end of every epoch)
    int64_t e_cur = a.first, e_nxt = a.count > 1 ? a.first + 1 : a.first;
    int64_t e_nxt2 = a.count > 2 ? a.first + 2 : (a.count == 2 ? a.first : a.first);
    auto advance = [&](int64_t e) { return e + 1 < a.first + a.count ? e + 1 : a.first; };
    auto fits = [&](const int *sz) { return a.stage != 0 && sz[0] <= kStageNodes && sz[0] * m.L0 <= kStageRowWords && sz[3] <= kStageEdges; };
    // sizes of the graph of step st -> s_size[st % 3]   (four independent loads)
    auto fetch_sizes = [&](u64 st, int64_t e) {
        if (threadIdx.x < 4 && st < steps) {
            const u32 *src = threadIdx.x == 0 ? g.n_nodes : threadIdx.x == 1 ? g.node_index : threadIdx.x == 2 ? g.graph_edge0 : g.graph_edges;
            async_copy_word(reinterpret_cast<u32 *>(s_size + (int)((u32)st % 3u) * 4 + threadIdx.x), src + e);
        }
    };
    // graph of step st (sizes already in s_size[st % 3]) -> s_stage[st & 1], targets -> s_y[st & 1]
    auto fetch_graph = [&](u64 st, int64_t e) {
        if (st >= steps) return;
        for (int k = threadIdx.x; k < m.K; k += blockDim.x)
            async_copy_word(reinterpret_cast<u32 *>(s_y + (st & 1) * KP + k), reinterpret_cast<const u32 *>(a.Y + (size_t)e * m.K + k));
        const int *sz = s_size + (int)((u32)st % 3u) * 4;
        if (!fits(sz)) return;
        const int n = sz[0], base = sz[1], e0 = sz[2], ne = sz[3];
        u32 *st_x = s_stage + (st & 1) * kStageWords, *st_t = st_x + kStageRowWords, *st_d = st_t + kStageNodes,
            *st_i = st_d + kStageNodes, *st_e = st_i + kStageNodes;
        for (int t = threadIdx.x; t < n * m.L0; t += blockDim.x) async_copy_word(st_x + t, g.X + (size_t)base * m.L0 + t);
        for (int t = threadIdx.x; t < n; t += blockDim.x) {
            async_copy_word(st_t + t, g.node_type + base + t);
            async_copy_word(st_d + t, g.degree + base + t);
            async_copy_word(st_i + t, g.edge_index + base + t);
        }
        for (int t = threadIdx.x; t < 2 * ne; t += blockDim.x) async_copy_word(st_e + t, g.edge + 2 * (size_t)e0 + t);
    };
    auto wait_copies = [&]() { asm volatile("cp.async.wait_all;" ::: "memory"); };

    // ---- state in ----
    for (int c = c_lo + warp; c < c_hi; c += nwarps) {
        ClauseView cv = view_of(c);
        if (lane == 0) { *cv.pos = m.draw_pos[c]; *cv.n_inc = 0; }
        for (int k = lane; k < m.K; k += 32) cv.wgt[k] = m.weights[(size_t)k * m.C + c];
        for (int b = lane; b < m.MB; b += 32) const_cast<u32 *>(cv.hv)[b] = m.hv[(size_t)c * m.MB + b];
        for (int l = 0; l < m.D; ++l) {
            const int total = m.SB * (l == 0 ? m.L0 : m.M);
            const u32 *src = l == 0 ? m.ta0 + (size_t)c * total : m.tam + ((size_t)(l - 1) * m.C + c) * total;
            u32 *dst = cv.ta(l);
            for (int t = lane; t < total; t += 32) dst[t] = src[t];
        }
    }
    for (int k = threadIdx.x; k < m.K; k += blockDim.x) s_sum[k] = 0;
    if (threadIdx.x == 0) { s_item_off[0] = 0; s_item_off[1] = 0; }
    fetch_sizes(0, e_cur);
    fetch_sizes(1, e_nxt);
    wait_copies();
    __syncthreads();
    fetch_graph(0, e_cur);
    wait_copies();
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
    const bool fine = timer && a.timers >= 2;     // timers == 2: slots 4..7 split the evaluation instead of the feedback
#define GTM_LAPE(acc) do { if (fine) { t1 = clock64(); acc += t1 - t0; t0 = t1; } } while (0)
#define GTM_LAPB(acc) do { if (timer && !fine) { t1 = clock64(); acc += t1 - t0; t0 = t1; } } while (0)
    long long t_eval = 0, t_bar = 0, t_tot = 0, t_fb = 0, t_x0 = 0, t_x1 = 0, t_x2 = 0, t_x3 = 0, t0 = clock64(), t1;

    int slot3 = 0;   // step % 3
    for (u64 step = 0; step < steps; ++step) {
        const int64_t e = e_cur;
        const int64_t i = e - a.first;
        const int par = (int)(step & 1);
        const int *sz = s_size + slot3 * 4;
        GraphView gv;
        gv.n = sz[0];
        if (fits(sz)) {
            const u32 *st_x = s_stage + par * kStageWords;
            gv.X = st_x; gv.type = st_x + kStageRowWords; gv.degree = gv.type + kStageNodes; gv.eidx = gv.degree + kStageNodes;
            gv.edge = gv.eidx + kStageNodes; gv.e_off = (u32)sz[2]; gv.e_cnt = (u32)sz[3];
        } else {
            const int base = sz[1];
            gv.X = g.X + (size_t)base * m.L0; gv.type = g.node_type + base; gv.degree = g.degree + base;
            gv.eidx = g.edge_index + base; gv.edge = g.edge; gv.e_off = 0; gv.e_cnt = g.total_edges;
        }
        u32 *P = par ? P_odd : P_even;
        const int *y = s_y + par * KP;
        TransposedGraph tg;
        tg.T = s_T; tg.TM = s_T + (size_t)t_rows * a.t_stride; tg.S = a.t_stride; tg.words = (gv.n + 31) >> 5;
        const bool transposed = kBatchNodes && a.t_stride > 0 && gv.n > 32 && tg.words <= a.t_stride && g.n_types <= kTransposedTypes;
        // larger graphs with a transposed copy: merged marks too; the destination rows are built in the local marks buffer
        // (via the transposed buffer as scratch), transposed from there, and written to global memory for the feedback
        const bool merged_large = kBatchNodes && !solo && transposed && s_part != nullptr && a.Q_pair[0] != nullptr && m.D > 1 &&
                                  (((gv.n + 31) & ~31) + kTransposedTypes) * (m.MW | 1) <= a.part_words;
        u32 *Q = par ? a.Q_pair[1] : a.Q_pair[0];
        // small graphs: the CTAs merge their source-node marks and build the message rows themselves (flush_marks)
        const bool merged_marks = !kBatchNodes && !solo && s_rows != nullptr && s_part != nullptr && gv.n <= 32 &&
                                  (32 + kTransposedTypes) * (m.MW | 1) <= a.part_words;
        const u32 *rows_base = merged_marks ? s_rows : merged_large ? Q : P;    // message rows [D-1][rows_nodes][MW] of this graph
        const int rows_nodes = merged_marks ? 32 : a.max_nodes;
        fetch_graph(step + 1, e_nxt);      // lands in the other stage buffer while this step runs
        fetch_sizes(step + 2, e_nxt2);
        GTM_LAPE(t_x0);

        for (int d = 0; d < m.D; ++d) {
            const bool last = d == m.D - 1;
            if (d > 0) {
                GTM_LAP(t_eval);
                if (solo) {
                    __syncthreads();
                } else {
                    if (!grid_barrier(a, ++nb)) return;
                }
                GTM_LAP(t_bar);
                if (d == 1) clear_next_messages(m, a, par ? P_even : P_odd, step + 1 < steps ? s_size[(slot3 == 2 ? 0 : slot3 + 1) * 4] : 0);
                if (merged_marks) build_message_rows(P + (size_t)(d - 1) * layer_words, s_part, s_rows + (size_t)(d - 1) * 32 * m.MW, gv, m.MS, m.MW);
                if (kBatchNodes && d == 1 && !solo && a.Q_pair[0] != nullptr) {
                    // the other parity's destination rows, last read in the step before this one, are cleared for the step
                    // after it - in every step, whichever way this step's graph passes its messages
                    u32 *Q_other = par ? a.Q_pair[0] : a.Q_pair[1];
                    const size_t words = (size_t)(m.D - 1) * layer_words;
                    for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < words; t += (size_t)gridDim.x * blockDim.x) Q_other[t] = 0;
                }
                if (merged_large) {
                    // the rank's CTAs build the layer's destination rows together, in global memory, and meet again
                    scatter_message_rows_share(P + (size_t)(d - 1) * layer_words, Q + (size_t)(d - 1) * layer_words, gv, m.MS, m.MW);
                    if (!rank_barrier(a, ++nb_rank)) return;
                }
                if (a.timers == 3) GTM_LAPE(t_x1);
            }
            if (transposed) {
                // this layer's literal rows, one bit per node: the graph's literals, or the messages of the layer below
                if (d == 0) {
                    build_transposed(gv.X, gv.n, m.L0, m.L0, tg);
                    build_type_masks(gv.type, gv.n, g.n_types, tg);
                } else if (merged_large) {
                    build_transposed(Q + (size_t)(d - 1) * layer_words, gv.n, m.MW, m.MW, tg);
                } else {
                    build_transposed(P + (size_t)(d - 1) * layer_words, gv.n, m.MW, m.MW, tg);
                }
                __syncthreads();
                if (a.timers == 3) GTM_LAPE(t_x2);
            }
            ScatterTargets targets;
            targets.world = a.world;
                targets.rank = a.rank;
            targets.local_words = transposed ? tg.words : 0;
            // the last kTransposedTypes rows of the buffer hold the marks of clauses that are true on every node of their type
            const int all_words = kTransposedTypes * (m.MW | 1);
            targets.local = (!last && s_part != nullptr && ((gv.n + 31) & ~31) * (m.MW | 1) + all_words <= a.part_words) ? s_part : nullptr;
            targets.all = (targets.local != nullptr && transposed) ? s_part + a.part_words - all_words : nullptr;
            #pragma unroll
                for (int r = 0; r < kMaxRanks; ++r) targets.base[r] = (par ? s_fs.P_peer[r][1] : s_fs.P_peer[r][0]) + (size_t)d * layer_words;
            for (int c = c_lo + warp; c < c_hi; c += nwarps) {
                const ClauseView cv = view_of(c);
                const u32 any = transposed
                    ? eval_clause_layer_transposed(m, gv, g.n_types, cv, c, d, d > 0 ? node_words(c, d - 1) : nullptr, node_words(c, d),
                                                   tg, last ? nullptr : &targets, lane)
                    : eval_clause_layer<kBatchNodes>(m, gv, g.n_types, cv, c, d, d > 0 ? node_words(c, d - 1) : nullptr, node_words(c, d),
                                                  d > 0 ? rows_base + (size_t)(d - 1) * rows_nodes * m.MW : nullptr,
                                                  last ? nullptr : &targets, lane);
                if (last && any)
                    for (int k = lane; k < m.K; k += 32) atomicAdd(&s_sum[k], cv.wgt[k]);
            }
            if (a.timers == 3) GTM_LAPE(t_x3); else GTM_LAPE(t_x1);
            if (targets.local && (merged_marks || merged_large)) {
                __syncthreads();
                flush_marks(targets, gv, m.MW);   // build_message_rows reuses and clears the buffer after the grid barrier
                if (merged_large) {               // ... larger graphs never come back to it: cleared here
                    __syncthreads();
                    for (int t = threadIdx.x; t < ((gv.n + 31) & ~31) * (m.MW | 1); t += blockDim.x) targets.local[t] = 0;
                }
                if (a.timers != 3) GTM_LAPE(t_x3);
            } else if (targets.local) {     // this CTA's share of the layer's messages, merged before the grid barrier
                __syncthreads();
                flush_messages(targets, gv, m.MS, m.MW);
                __syncthreads();
                for (int t = threadIdx.x; t < ((gv.n + 31) & ~31) * (m.MW | 1); t += blockDim.x) targets.local[t] = 0;
                if (a.timers != 3) GTM_LAPE(t_x3);
            }
        }
        __syncthreads();
        if (a.timers != 3) GTM_LAPE(t_x2);
        GTM_LAP(t_eval);
        if (solo) {
            for (int k = threadIdx.x; k < m.K; k += blockDim.x) {
                s_total[k] = s_sum[k];
                a.class_sum_tap[k] = s_sum[k];
                class_decision_input(m.T, s_sum[k], y[k], s_target + k, s_thr + k);
                s_sum[k] = 0;
            }
        } else {
            publish_votes(a, step, s_sum, m.K);
        }
        // Layer 0's masks come from a Bernoulli stream that starts at Philox block B0 = (position after the node choice + K)
        // >> 2: at or before the first mask draw whatever the decisions turn out to be, so that its first rounds - enough
        // for one Type-I class - can be generated before the class sums are known.
        const MaskProb mp0 = s_fs.p_mask[0];
        const float p0 = mp0.p;
        auto words0_of = [&](int npos, int off0) { return (npos > 0 && p0 < 1.0f) ? ((off0 + npos * m.L0 * 32 - 1) >> 5) + 1 : 0; };
        const int spec_rounds = (a.pre_words > 0 && p0 < 1.0f) ? (words0_of(1, m.K + 3) + 3) >> 2 : 0;
        if (a.pre_words > 0) {
            // in the shadow of the vote exchange: what the decisions need besides the class sums, and the speculative rounds
            for (int c = c_lo + warp; c < c_hi; c += nwarps) {
                const ClauseView cv = view_of(c);
                const PreDecision pd = clause_predecide(m, gv, cv, node_words(c, m.D - 1), c, lane);
                int *rec = s_rec + (size_t)(c - c_lo) * kRecWords;
                if (lane == 0) { rec[0] = pd.chosen; rec[2] = (int)(u32)pd.pos; rec[3] = (int)(u32)(pd.pos >> 32); }
                rec[5 + lane] = __float_as_int(pd.uni);
                const u64 B0 = (pd.pos + (u64)m.K) >> 2;
                for (int q = 0; q < spec_rounds; ++q)
                    generate_mask_round(m, c, B0, 4 * spec_rounds, q, s_pre + (size_t)(c - c_lo) * a.pre_words, lane, mp0);
            }
        }
        bool inputs_done = true;
        if (solo) {
            __syncthreads();
        } else {
            DecisionInputs di;
            di.y = y; di.target = s_target; di.thr = s_thr; di.T = m.T;
            if (!collect_votes(a, step, par, a.tag_base + (u32)step + 1u, s_total, m.K, di, &inputs_done)) return;
        }
        GTM_LAP(t_tot);
        if (!inputs_done) {
            class_decision_inputs(m, s_total, y, s_target, s_thr);
            __syncthreads();
        }
        if (a.pre_words > 0) {
            // cooperative feedback: decisions per clause, then every (clause, layer, round) of mask generation that is still
            // missing is a work item shared by all warps of the CTA, then the automaton updates per clause
            int any_items = 0;
            for (int c = c_lo + warp; c < c_hi; c += nwarps) {
                const ClauseView cv = view_of(c);
                int *rec = s_rec + (size_t)(c - c_lo) * kRecWords;
                PreDecision pd;
                pd.chosen = rec[0];
                pd.pos = (u64)(u32)rec[2] | ((u64)(u32)rec[3] << 32);
                pd.uni = __int_as_float(rec[5 + lane]);
                const u64 B0 = (pd.pos + (u64)m.K) >> 2;
                const Decision dec = clause_decide_finish(m, cv, a, pd, s_target, s_thr, c, lane);
                const int npos = __popc(__ballot_sync(kFull, dec.upd_lo > 0));
                const int off0 = (int)(dec.pos - 4 * B0);
                const int rounds0 = (words0_of(npos, off0) + 3) >> 2;
                int need = 4 * max(rounds0, spec_rounds), items = max(0, rounds0 - spec_rounds);
                u64 pos_l = dec.pos + (u64)npos * m.L0 * 32;
                for (int l = 1; l < m.D; ++l) {
                    need += npos * m.M + 1;
                    if (npos > 0 && s_fs.p_mask[l].p < 1.0f) items += (npos * m.M + ((pos_l & 3) ? 1 : 0) + 3) >> 2;
                    pos_l += (u64)npos * m.M * 32;
                }
                __syncwarp();
                if (lane == 0) {
                    rec[1] = npos;
                    rec[2] = (int)(u32)dec.pos; rec[3] = (int)(u32)(dec.pos >> 32);
                    const bool fits_pre = need <= a.pre_words;
                    rec[4] = fits_pre ? items : -1;                      // -1: does not fit, the clause generates on its own
                    rec[37] = off0;
                    // this clause's work items take the next `items` numbers; (clause, first number) goes to the item table
                    if (fits_pre && items > 0) {
                        const int slot = atomicAdd(&s_item_off[0], 1);
                        const int firsti = atomicAdd(&s_item_off[1], items);
                        s_item_off[2 + 2 * slot] = c - c_lo;
                        s_item_off[3 + 2 * slot] = firsti;
                    }
                }
                rec[5 + lane] = dec.upd_lo;
                any_items |= items;
            }
            // the work-item phase and its two CTA barriers only when some clause of the CTA has items
            any_items = __syncthreads_or(any_items > 0);
            GTM_LAPB(t_x0);
            GTM_LAPB(t_x1);
            if (any_items) {
                const int entries = s_item_off[0], total = s_item_off[1];
                for (int i = warp; i < total; i += nwarps) {
                    int ci = 0, firsti = 0;
                    for (int t = 0; t < entries; ++t) {                   // the entry whose range holds item i
                        const int f = s_item_off[3 + 2 * t];
                        if (f <= i && f >= firsti) { firsti = f; ci = s_item_off[2 + 2 * t]; }
                    }
                    const int *rec = s_rec + (size_t)ci * kRecWords;
                    const int npos = rec[1], off0 = rec[37];
                    const u64 pos = (u64)(u32)rec[2] | ((u64)(u32)rec[3] << 32);
                    const int rounds0 = (words0_of(npos, off0) + 3) >> 2;
                    int r = i - firsti;
                    u32 *dst = s_pre + (size_t)ci * a.pre_words;
                    if (r < rounds0 - spec_rounds) {
                        generate_mask_round(m, c_lo + ci, (pos - (u64)off0) >> 2, 4 * rounds0, spec_rounds + r, dst, lane, mp0);
                        continue;
                    }
                    r -= max(0, rounds0 - spec_rounds);
                    dst += 4 * max(rounds0, spec_rounds);
                    u64 pos_l = pos + (u64)npos * m.L0 * 32;
                    for (int l = 1; l < m.D; ++l) {
                        const int wneed = npos * m.M + ((pos_l & 3) ? 1 : 0);
                        const int rounds = s_fs.p_mask[l].p < 1.0f ? (wneed + 3) >> 2 : 0;
                        if (r < rounds) { generate_mask_round(m, c_lo + ci, pos_l >> 2, wneed, r, dst, lane, s_fs.p_mask[l]); break; }
                        r -= rounds;
                        dst += npos * m.M + 1;
                        pos_l += (u64)npos * m.M * 32;
                    }
                }
            }
            if (any_items) {
                __syncthreads();
                if (threadIdx.x == 0) { s_item_off[0] = 0; s_item_off[1] = 0; }     // next step's item table starts empty
            }
            GTM_LAPB(t_x2);
            for (int c = c_lo + warp; c < c_hi; c += nwarps) {
                const ClauseView cv = view_of(c);
                const int *rec = s_rec + (size_t)(c - c_lo) * kRecWords;
                Decision dec;
                dec.chosen = rec[0];
                dec.pos = (u64)(u32)rec[2] | ((u64)(u32)rec[3] << 32);
                dec.upd_lo = rec[5 + lane];
                const int rounds0 = (words0_of(rec[1], rec[37]) + 3) >> 2;
                clause_apply<MAXSB>(m, gv, cv, a, rows_base, rows_nodes, dec, rec[1], c, lane, s_pack + warp * kPackWords,
                                    rec[4] >= 0 ? s_pre + (size_t)(c - c_lo) * a.pre_words : nullptr, rec[37],
                                    4 * max(rounds0, spec_rounds), s_fs.p_mask);
            }
        } else if (m.K <= 32) {
            // wide layers: the clause's warp decides; the automaton updates are then work items of one (clause, layer,
            // 32-word stretch) each, shared by all warps of the CTA - a clause with Type I feedback costs tens of Philox
            // rounds per layer, one without costs nothing, and there are hardly more clauses than warps
            const int chunks0 = (m.L0 + 31) >> 5, chunksM = (m.M + 31) >> 5;
            for (int c = c_lo + warp; c < c_hi; c += nwarps) {
                const ClauseView cv = view_of(c);
                const Decision dec = clause_decide(m, gv, cv, a, node_words(c, m.D - 1), s_target, s_thr, c, lane);
                const int npos = __popc(__ballot_sync(kFull, dec.upd_lo > 0));
                const bool any_feedback = __ballot_sync(kFull, dec.upd_lo != 0) != 0;
                int *rec = s_rec + (size_t)(c - c_lo) * kRecWords;
                if (lane == 0) {
                    rec[0] = dec.chosen; rec[1] = npos;
                    rec[2] = (int)(u32)dec.pos; rec[3] = (int)(u32)(dec.pos >> 32);
                    *cv.pos = dec.pos + (any_feedback ? (u64)npos * (u64)(m.L0 + (m.D - 1) * m.M) * 32u : 0u);
                    if (any_feedback) {
                        const int slot = atomicAdd(&s_item_off[0], 1);
                        const int firsti = atomicAdd(&s_item_off[1], chunks0 + (m.D - 1) * chunksM);
                        s_item_off[2 + 2 * slot] = c - c_lo;
                        s_item_off[3 + 2 * slot] = firsti;
                    }
                }
                rec[5 + lane] = dec.upd_lo;
            }
            __syncthreads();
            const int entries = s_item_off[0], total = s_item_off[1];
            for (int i = warp; i < total; i += nwarps) {
                int ci = 0, firsti = 0;
                for (int t = 0; t < entries; ++t) {                   // the entry whose range holds item i
                    const int f = s_item_off[3 + 2 * t];
                    if (f <= i && f >= firsti) { firsti = f; ci = s_item_off[2 + 2 * t]; }
                }
                const int c = c_lo + ci;
                const ClauseView cv = view_of(c);
                const int *rec = s_rec + (size_t)ci * kRecWords;
                const int chosen = rec[0], npos = rec[1];
                const u64 pos = (u64)(u32)rec[2] | ((u64)(u32)rec[3] << 32);
                const int r = i - firsti;
                const int l = r < chunks0 ? 0 : 1 + (r - chunks0) / chunksM;
                const int g0 = 32 * (l == 0 ? r : (r - chunks0) % chunksM);
                const int W = l == 0 ? m.L0 : m.M;
                const u64 pos_l = pos + (l == 0 ? 0u : (u64)npos * (u64)(m.L0 + (l - 1) * m.M) * 32u);
                const bool clause_true = chosen != -1;
                const int node = clause_true ? chosen : 0;
                const u32 *row = l == 0 ? gv.X + (size_t)node * m.L0 : rows_base + ((size_t)(l - 1) * rows_nodes + node) * m.MW;
                layer_feedback<MAXSB>(m, c, l, cv.ta(l), rec[5 + lane], a.update, clause_true, *cv.n_inc <= m.max_included, row, l > 0,
                                      pos_l, g0, min(W, g0 + 32), lane, s_pack + warp * kPackWords, nullptr, 0, s_fs.p_mask[l]);
            }
            __syncthreads();
            if (threadIdx.x == 0) { s_item_off[0] = 0; s_item_off[1] = 0; }     // next step's item table starts empty
        } else {
            for (int c = c_lo + warp; c < c_hi; c += nwarps) {
                const ClauseView cv = view_of(c);
                clause_feedback<MAXSB>(m, gv, cv, a, node_words(c, m.D - 1), rows_base, rows_nodes, s_target, s_thr, c, lane, s_pack + warp * kPackWords, s_fs.p_mask);
            }
        }
        GTM_LAPB(t_x3);
        wait_copies();
        __syncthreads();   // next step's graph is complete; s_total and this step's stage buffer may be reused
        GTM_LAP(t_fb);
        e_cur = e_nxt; e_nxt = e_nxt2; e_nxt2 = advance(e_nxt2);
        slot3 = slot3 == 2 ? 0 : slot3 + 1;
    }

    // ---- state out ----
    for (int c = c_lo + warp; c < c_hi; c += nwarps) {
        ClauseView cv = view_of(c);
        if (lane == 0) m.draw_pos[c] = *cv.pos;
        for (int k = lane; k < m.K; k += 32) m.weights[(size_t)k * m.C + c] = cv.wgt[k];
        for (int l = 0; l < m.D; ++l) {
            const int total = m.SB * (l == 0 ? m.L0 : m.M);
            u32 *dst = l == 0 ? m.ta0 + (size_t)c * total : m.tam + ((size_t)(l - 1) * m.C + c) * total;
            const u32 *src = cv.ta(l);
            for (int t = lane; t < total; t += 32) dst[t] = src[t];
        }
    }
    if (timer && threadIdx.x == 0) {
        a.phase_cycles[0] = (unsigned long long)t_eval; a.phase_cycles[1] = (unsigned long long)t_bar;
        a.phase_cycles[2] = (unsigned long long)t_tot; a.phase_cycles[3] = (unsigned long long)t_fb;
        a.phase_cycles[4] = (unsigned long long)t_x0; a.phase_cycles[5] = (unsigned long long)t_x1;
        a.phase_cycles[6] = (unsigned long long)t_x2; a.phase_cycles[7] = (unsigned long long)t_x3;
    }
}
#undef GTM_LAP
#undef GTM_LAPE
#undef GTM_LAPB

}  // namespace gtm


int fit_grid_for_global_state(const DevModel &d, int sm_count, int block, int *grid_out)
{
    int per_sm = 0;
    const size_t smem = 4 * (size_t)d.K * sizeof(int);
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fit_global_kernel(d.SB, true), block, smem);
    if (e != cudaSuccess || per_sm < 1)
        return fail(GTM_ERR_CUDA, "learning kernel does not fit on this device: %s", cudaGetErrorString(e));
    const int warps_per_cta = block / 32;
    *grid_out = std::max(1, std::min(sm_count * std::min(per_sm, 2), (d.C + warps_per_cta - 1) / warps_per_cta));
    return GTM_OK;
}

static int words_for(int bits) { return (bits - 1) / 32 + 1; }

constexpr int kResidentThreads = 384;   // 12 warps when two CTAs share an SM; a CTA that has its SM to itself gets a warp per
                                        // clause, up to kResidentMaxWarps (the kernel's register budget is that of 768 threads)
constexpr int kResidentMaxWarps = 24;

// The state-resident kernel for the automaton width, with four-at-a-time node words for graph sets of more than 32 nodes per graph.
static const void *resident_kernel_for(int state_bits, int max_nodes, int depth)
{
    if (depth == 1) {
        if (max_nodes > 32) return state_bits <= 8 ? (const void *)fit_resident_kernel<8, true, true> : (const void *)fit_resident_kernel<32, true, true>;
        return state_bits <= 8 ? (const void *)fit_resident_kernel<8, false, true> : (const void *)fit_resident_kernel<32, false, true>;
    }
    if (max_nodes > 32) return state_bits <= 8 ? (const void *)fit_resident_kernel<8, true, false> : (const void *)fit_resident_kernel<32, true, false>;
    return state_bits <= 8 ? (const void *)fit_resident_kernel<8, false, false> : (const void *)fit_resident_kernel<32, false, false>;
}

// Shape of a state-resident launch, or grid == 0 when the model's state does not fit in shared memory.
struct ResidentPlan { int threads = kResidentThreads, grid = 0, clauses_per_cta = 0, clause_words = 0, pre_words = 0, solo = 0, p_smem_words = 0, part_words = 0, stage = 1, t_stride = 0, rows_words = 0; size_t smem = 0; };

static ResidentPlan plan_resident(const gtm_model *m, const gtm_dataset *ds, int n_clauses, bool solo_allowed)
{
    DevModel d = m->dm;
    d.C = n_clauses;   // clauses this rank learns
    ResidentPlan plan;
    const void *fn = resident_kernel_for(d.SB, ds->max_nodes, d.D);
    const int warps = kResidentThreads / 32;
    int words = 4 + d.K + d.MB + 2 * ds->NC + d.SB * (d.L0 + (d.D - 1) * d.M);
    words = (words + 3) & ~3;
    // cooperative mask generation: layers of at most 32 words, at most 32 classes; room for 8 Type-I classes per clause
    int pre_words = 0;
    if (d.K <= 32 && d.L0 <= 32 && (d.D == 1 || d.M <= 32)) pre_words = (std::min(d.K, 8) * (d.L0 + (d.D - 1) * d.M) + d.D + 9) & ~1;
    const size_t p_words = (size_t)(d.D - 1) * ds->max_nodes * d.MW;
    const size_t layer_bytes = (size_t)(((ds->max_nodes + 31) & ~31) + kTransposedTypes) * (d.MW | 1) * sizeof(u32);   // message bits of one layer: padded rows + per-type rows
    // transposed-graph buffer (graph sets of 33..1024 nodes per graph, few node types): rows of max(L0, MW) words plus type masks
    const int t_stride = ds->NC | 1;
    const size_t t_bytes = ((size_t)32 * std::max(d.L0, d.MW) + kTransposedTypes) * t_stride * sizeof(u32);
    const bool t_possible = ds->max_nodes > 32 && ds->NC <= 32 && t_bytes <= 96 * 1024;
    const bool part_possible = d.D > 1 && layer_bytes <= 72 * 1024;
    // preference: the transposed evaluation first (it is worth an occupancy step), then two CTAs per SM, then the message
    // accumulation buffer with and without the graph staging buffers, then staging alone
    for (int with_t = t_possible ? 1 : 0; with_t >= 0; --with_t)
    for (int per_sm = 2; per_sm >= 1; --per_sm) {
        for (int choice = part_possible ? 0 : 2; choice < 3; ++choice) {
            const int with_part = choice < 2, stage = choice != 1;
            int grid = std::max(1, std::min(per_sm * m->sm_count, (d.C + warps - 1) / warps));
            // more CTAs than SMs: then two on (nearly) every SM, with fewer clauses each, rather than two on some SMs and
            // one on the others - every step waits for the most loaded SM
            if (grid > m->sm_count) grid = std::min(per_sm * m->sm_count, d.C);
            int cpb = (d.C + grid - 1) / grid;
            if (m->opt_fit_block_clauses > 0) cpb = m->opt_fit_block_clauses;
            grid = (d.C + cpb - 1) / cpb;
            if (grid > per_sm * m->sm_count) continue;
            // one CTA per SM: a warp per clause where the CTA has more clauses than the usual twelve warps (two rounds of
            // clause work per phase otherwise); tried first, the usual size second
            for (int attempt = (per_sm == 1 && cpb > warps) ? 0 : 1; attempt < 2; ++attempt) {
            const int cta_warps = attempt == 0 ? std::min(kResidentMaxWarps, cpb) : warps;
            size_t smem = ((size_t)6 * ((d.K + 3) & ~3) + 12 + (stage ? 2 * (size_t)kStageWords : 0) + (size_t)cta_warps * kPackWords) * sizeof(int) +
                          ((size_t)cpb * kRecWords + 2 * (size_t)cpb + 2 + (size_t)cpb * pre_words) * sizeof(int) +
                          (size_t)cpb * words * sizeof(u32);
            // a model that one CTA learns alone needs no grid-wide step; its message buffers (two parities) then live in
            // shared memory, which they must fit (messages written with atomics to global memory would need a device-scope
            // acquire before they are read, i.e. the grid barrier)
            int solo = 0, p_smem_words = 0, part_words = 0, rows_words = 0;
            if (solo_allowed && grid == 1 && (d.D == 1 || smem + 2 * p_words * sizeof(u32) <= 96 * 1024)) {
                solo = 1;
                p_smem_words = (int)p_words;
                smem += 2 * p_words * sizeof(u32);
            } else if (with_part) {
                part_words = (int)(layer_bytes / sizeof(u32));
                smem += layer_bytes;
                if (ds->max_nodes <= 32) {      // merged marks: the message rows of all layers below the last live in the CTA
                    rows_words = (d.D - 1) * 32 * d.MW;
                    smem += (size_t)rows_words * sizeof(u32);
                }
            }
            if (with_t) smem += t_bytes;
            if (smem > 220 * 1024) continue;
            if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { cudaGetLastError(); continue; }
            int occ = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fn, 32 * cta_warps, smem) != cudaSuccess) { cudaGetLastError(); continue; }
            if ((long long)occ * m->sm_count < grid) continue;
            plan.threads = 32 * cta_warps;
            plan.grid = grid; plan.clauses_per_cta = cpb; plan.clause_words = words; plan.pre_words = pre_words; plan.smem = smem;
            plan.solo = solo; plan.p_smem_words = p_smem_words; plan.part_words = part_words; plan.stage = stage; plan.rows_words = rows_words;
            plan.t_stride = with_t ? t_stride : 0;
            return plan;
            }
        }
    }
    return plan;
}

static int shard_size(int C, int world) { return (C + world - 1) / world; }

// Bytes of one rank's vote exchange area: tagged slots [2][world][K], then the accumulators [4][K], all 64-bit
// (exchange_class_sums).
size_t exchange_bytes(int world, int K)
{
    return ((size_t)2 * world * K + (size_t)4 * K) * sizeof(unsigned long long);
}

int launch_fit(gtm_model *m, gtm_dataset *ds, int n_types, const int *Y_dev, int64_t first, int64_t count,
               int epochs, int eval_only)
{
    const DevModel &d = m->dm;
    FitComm &cm = ds->comm;
    const bool sharded = cm.world > 1 && !eval_only;
    if (sharded && !cm.connected) return fail(GTM_ERR_STATE, "clause sharding was prepared but the ranks are not connected (gtm_shard_connect)");
    if (sharded && cm.broken) return fail(GTM_ERR_STATE, "an earlier sharded fit timed out; prepare and connect the ranks again");
    DevGraphs g = ds->dg;
    g.n_types = n_types;
    EvalScratch sc = ds->fit_sc;
    FitArgs a;
    memset(&a, 0, sizeof a);
    a.Y = Y_dev; a.first = first; a.count = count; a.epochs = epochs;
    a.max_nodes = ds->max_nodes;
    a.error = m->error; a.clause_node = m->clause_node; a.update = m->update;
    a.class_sum_tap = m->class_sum_tap;
    a.phase_cycles = m->phase_cycles;
    a.timers = m->opt_fit_timers;
    a.wait_ns = (unsigned long long)m->opt_fit_wait_ms * 1000000ull;
    a.missing = eval_only ? 0 : m->opt_fit_missing_cta;
    a.NC = ds->NC;
    const size_t p_bytes = (size_t)std::max(1, d.D - 1) * ds->max_nodes * d.MW * sizeof(u32);
    GTM_CU(cudaMemsetAsync(m->error, 0, sizeof(int), m->stream));
    a.Q_pair[0] = ds->Q_pair[0]; a.Q_pair[1] = ds->Q_pair[1];
    a.barrier_rank = ds->rank_barrier;
    GTM_CU(cudaMemsetAsync(ds->rank_barrier, 0, sizeof(unsigned), m->stream));
    if (d.D > 1) {      // the rows of both parities start empty; each step clears the other parity's for the step after it
        GTM_CU(cudaMemsetAsync(ds->Q_pair[0], 0, p_bytes, m->stream));
        GTM_CU(cudaMemsetAsync(ds->Q_pair[1], 0, p_bytes, m->stream));
    }

    int grid, block, resident_threads = kResidentThreads;
    size_t smem;
    const void *fn;
    bool resident;
    if (sharded) {
        a.world = cm.world; a.rank = cm.rank;
        const int per = shard_size(d.C, cm.world);
        a.c_begin = std::min(d.C, cm.rank * per); a.c_end = std::min(d.C, a.c_begin + per);
        a.tag_base = cm.tag_base; a.barriers_done = cm.barriers_done;
        a.barrier_local = (unsigned *)((char *)cm.block + 128);
        for (int r = 0; r < cm.world; ++r) {
            char *base = (char *)cm.peer_block[r];
            a.barrier_peer[r] = (unsigned *)base;
            a.exchange_peer[r] = (unsigned long long *)(base + cm.exchange_off);
            a.P_peer[r][0] = (u32 *)(base + cm.P_off[0]);
            a.P_peer[r][1] = (u32 *)(base + cm.P_off[1]);
        }
        // the accumulators of the vote exchange start every launch at zero (they are this rank's own; the slots that
        // peers write keep their tags)
        GTM_CU(cudaMemsetAsync((char *)cm.block + cm.exchange_off + (size_t)2 * cm.world * d.K * sizeof(unsigned long long), 0,
                               (size_t)4 * d.K * sizeof(unsigned long long), m->stream));
        resident = cm.resident; grid = cm.grid; resident_threads = cm.threads;
        a.clauses_per_cta = cm.clauses_per_cta; a.clause_words = cm.clause_words; a.pre_words = cm.pre_words; a.part_words = cm.part_words; a.stage = cm.stage; a.t_stride = cm.t_stride; a.rows_words = cm.rows_words;
        smem = cm.smem;
    } else {
        a.world = 1; a.rank = 0; a.c_begin = 0; a.c_end = d.C;
        a.tag_base = 0; a.barriers_done = 0; a.barrier_local = nullptr;
        a.barrier_peer[0] = m->barrier; a.exchange_peer[0] = m->exchange;
        a.P_peer[0][0] = ds->P_pair[0]; a.P_peer[0][1] = ds->P_pair[1];
        GTM_CU(cudaMemsetAsync(m->barrier, 0, sizeof(unsigned), m->stream));
        GTM_CU(cudaMemsetAsync(m->exchange, 0, exchange_bytes(1, d.K), m->stream));
        if (d.D > 1) {
            GTM_CU(cudaMemsetAsync(ds->P_pair[0], 0, p_bytes, m->stream));
            GTM_CU(cudaMemsetAsync(ds->P_pair[1], 0, p_bytes, m->stream));
        }
        ResidentPlan plan;
        if (!eval_only && m->opt_fit_kernel != 1) plan = plan_resident(m, ds, d.C, true);
        if (m->opt_fit_kernel == 2 && !eval_only && plan.grid == 0)
            return fail(GTM_ERR_ARG, "the model's state does not fit in shared memory; the state-resident learning kernel cannot run");
        resident = plan.grid > 0;
        grid = resident ? plan.grid : m->fit_grid;
        a.clauses_per_cta = plan.clauses_per_cta; a.clause_words = plan.clause_words; a.pre_words = plan.pre_words;
        a.solo = plan.solo; a.p_smem_words = plan.p_smem_words; a.part_words = plan.part_words; a.stage = plan.stage; a.t_stride = plan.t_stride; a.rows_words = plan.rows_words;
        smem = plan.smem; resident_threads = plan.threads;
    }
    a.barrier = a.barrier_peer[a.rank]; a.exchange = a.exchange_peer[a.rank];
    a.P_pair[0] = a.P_peer[a.rank][0]; a.P_pair[1] = a.P_peer[a.rank][1];

    DevModel dm = d;
    if (resident) {
        fn = resident_kernel_for(d.SB, ds->max_nodes, d.D);
        block = resident_threads;
        // static and dynamic shared memory together may pass 48 KB well before the dynamic part alone does
        if (smem > 16 * 1024) GTM_CU(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        void *args[] = {&dm, &g, &a};
        GTM_CU(cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(block), args, smem, m->stream));
    } else {
        fn = fit_global_kernel(d.SB, ds->max_nodes > 32);
        block = m->fit_block;
        // one layer's messages are accumulated per CTA in shared memory when a layer takes at most 64 KB
        const size_t layer_bytes = (size_t)(((ds->max_nodes + 31) & ~31) + kTransposedTypes) * (d.MW | 1) * sizeof(u32);
        a.part_words = (!eval_only && d.D > 1 && layer_bytes <= 72 * 1024) ? (int)(layer_bytes / sizeof(u32)) : 0;
        // graph sets of at most 32 nodes per graph: the current graph (and the message rows a layer reads) in shared memory
        a.gstage_words = (!eval_only && ds->max_nodes <= 32) ? 2 * kFitStageGraphWords + std::max(1, d.D - 1) * 32 * d.MW : 0;
        smem = (size_t)((4 * d.K + 3) & ~3) * sizeof(int) + ((size_t)a.part_words + a.gstage_words) * sizeof(u32);
        // static and dynamic shared memory together may pass 48 KB well before the dynamic part alone does
        if (smem > 16 * 1024) GTM_CU(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        void *args[] = {&dm, &g, &sc, &a, &eval_only};
        GTM_CU(cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(block), args, smem, m->stream));
    }
    if (sharded) {   // what the counters and tags look like after this launch (the same on every rank)
        const unsigned long long steps = (unsigned long long)epochs * (unsigned long long)count;
        const unsigned long long barriers = (d.D > 1 ? 1ull : 0ull) + steps * (unsigned long long)(d.D - 1);
        cm.tag_base += (u32)steps;
        cm.barriers_done += (unsigned)barriers;
    }
    int err = 0;
    GTM_CU(cudaMemcpyAsync(&err, m->error, sizeof(int), cudaMemcpyDeviceToHost, m->stream));
    GTM_CU(cudaStreamSynchronize(m->stream));
    if (err) {
        if (sharded) cm.broken = true;
        return fail(GTM_ERR_TIMEOUT, "a bounded wait of the learning kernel (grid barrier or vote exchange) gave up");
    }
    return GTM_OK;
}

// ------------------------------------------------------------------------------------------ clause sharding
extern "C" int gtm_shard_range(gtm_model *m, int world, int rank, int *first_clause, int *n_clauses)
{
    if (!m || !first_clause || !n_clauses) return fail(GTM_ERR_ARG, "null argument");
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return fail(GTM_ERR_ARG, "world must be 1..%d and rank inside it", kMaxRanks);
    const int per = shard_size(m->dm.C, world);
    *first_clause = std::min(m->dm.C, rank * per);
    *n_clauses = std::min(m->dm.C, *first_clause + per) - *first_clause;
    return GTM_OK;
}

extern "C" int gtm_shard_prepare(gtm_model *m, gtm_dataset *ds, int world, int rank, unsigned char *handle_out)
{
    if (!m || !ds || ds->model != m || !handle_out) return fail(GTM_ERR_ARG, "null argument or dataset of another model");
    if (world < 2 || world > kMaxRanks || rank < 0 || rank >= world) return fail(GTM_ERR_ARG, "world must be 2..%d and rank inside it", kMaxRanks);
    GTM_CU(cudaSetDevice(m->cfg.device));
    const DevModel &d = m->dm;
    FitComm &cm = ds->comm;
    if (cm.block) return fail(GTM_ERR_STATE, "clause sharding is already prepared for this graph set");
    const int per = shard_size(d.C, world);
    // every rank derives the same launch shape from the shard size (the last shard may be shorter; it runs the same grid)
    ResidentPlan plan;
    if (m->opt_fit_kernel != 1) plan = plan_resident(m, ds, per, false);
    cm.resident = plan.grid > 0;
    if (cm.resident) {
        cm.grid = plan.grid; cm.threads = plan.threads; cm.clauses_per_cta = plan.clauses_per_cta; cm.clause_words = plan.clause_words;
        cm.pre_words = plan.pre_words; cm.part_words = plan.part_words; cm.stage = plan.stage; cm.t_stride = plan.t_stride; cm.rows_words = plan.rows_words; cm.smem = plan.smem;
    } else {
        const int warps = m->fit_block / 32;
        cm.grid = std::max(1, std::min(m->fit_grid, (per + warps - 1) / warps));
    }
    const size_t p_bytes = ((size_t)std::max(1, d.D - 1) * ds->max_nodes * d.MW * sizeof(u32) + 255) & ~(size_t)255;
    cm.exchange_off = 256;
    const size_t ex_bytes = (exchange_bytes(world, d.K) + 255) & ~(size_t)255;
    cm.P_off[0] = cm.exchange_off + ex_bytes;
    cm.P_off[1] = cm.P_off[0] + p_bytes;
    cm.bytes = cm.P_off[1] + p_bytes;
    GTM_CU(cudaMalloc(&cm.block, cm.bytes));
    GTM_CU(cudaMemset(cm.block, 0, cm.bytes));
    cm.world = world; cm.rank = rank;
    cm.peer_block[rank] = cm.block;
    cudaIpcMemHandle_t h;
    GTM_CU(cudaIpcGetMemHandle(&h, cm.block));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    memcpy(handle_out, &h, 64);
    return GTM_OK;
}

extern "C" int gtm_shard_connect(gtm_model *m, gtm_dataset *ds, const unsigned char *handles)
{
    if (!m || !ds || ds->model != m || !handles) return fail(GTM_ERR_ARG, "null argument or dataset of another model");
    FitComm &cm = ds->comm;
    if (!cm.block) return fail(GTM_ERR_STATE, "call gtm_shard_prepare first");
    GTM_CU(cudaSetDevice(m->cfg.device));
    for (int r = 0; r < cm.world; ++r) {
        if (r == cm.rank || cm.peer_block[r]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * 64, 64);
        GTM_CU(cudaIpcOpenMemHandle(&cm.peer_block[r], h, cudaIpcMemLazyEnablePeerAccess));
    }
    cm.connected = true;
    return GTM_OK;
}

void fit_comm_release(gtm_dataset *ds)
{
    FitComm &cm = ds->comm;
    for (int r = 0; r < cm.world; ++r)
        if (r != cm.rank && cm.peer_block[r]) cudaIpcCloseMemHandle(cm.peer_block[r]);
    if (cm.block) cudaFree(cm.block);
    cm = FitComm();
}
