// Kernels of the general path: state initialisation / layout conversion, CTA-per-graph scoring for any
// depth, and the persistent clause-parallel learning kernel.
#pragma once
#include "gtm_device.cuh"

namespace gtm {

// ------------------------------------------------------------------------------------------ state kernels
// kernels.py:638-664 / :622-636: weights = 1 - 2*(draw % 2), one draw per (clause, class) in class order;
// automata one step below include: planes 0..SB-2 all ones, include plane zero.
__global__ void init_weights_kernel(DevModel m)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= m.C) return;
    u64 pos = m.draw_pos[c];
    for (int k = 0; k < m.K; ++k) m.weights[(size_t)k * m.C + c] = 1 - 2 * (int)(draw_at(m, c, pos++) & 1u);
    m.draw_pos[c] = pos;
}

__global__ void init_planes_kernel(u32 *ta, int C, int SB, int W)
{
    const size_t total = (size_t)C * SB * W;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int b = (int)((i / W) % SB);
        ta[i] = b == SB - 1 ? 0u : kFull;
    }
}

// uint32[C][W][SB] (reference) <-> uint32[C][SB][W] (engine)
__global__ void planes_from_reference_kernel(const u32 *ref, u32 *ta, int C, int SB, int W)
{
    const size_t total = (size_t)C * SB * W;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int w = (int)(i % W), b = (int)((i / W) % SB);
        const size_t c = i / ((size_t)W * SB);
        ta[i] = ref[(c * W + w) * SB + b];
    }
}

__global__ void planes_to_reference_kernel(const u32 *ta, u32 *ref, int C, int SB, int W)
{
    const size_t total = (size_t)C * SB * W;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int w = (int)(i % W), b = (int)((i / W) % SB);
        const size_t c = i / ((size_t)W * SB);
        ref[(c * W + w) * SB + b] = ta[i];
    }
}

// Packed messages in the reference's clause_X layout uint32[n][M] from the positive halves (debug tap).
__global__ void expand_messages_kernel(const u32 *P, u32 *out, int n, int MS, int MW, int M)
{
    const int total = n * M;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int v = i / M, w = i % M;
        out[i] = msg_word(P + (size_t)v * MW, w, MS, MW);
    }
}

// ------------------------------------------------------------------------------- scoring, general path
// One CTA per graph (grid-stride), warps over clauses, lanes over the nodes of a node word.  Per-CTA scratch in
// global memory (L2-resident).  Serves every depth / graph size; the node-stream kernel in gtm_stream.cuh is
// the fast path for the shapes it covers.
struct ScoreArgs {
    int64_t first, count;
    int *class_sums;      // [count][K]
    int *clause_outputs;  // optional [count][C] (transform)
    int *node_outputs;    // optional [count][C][node_stride] per-node clause outputs of the last layer (transform_nodewise)
    int node_stride;
    size_t cno_stride, P_stride, ninc_stride;  // per-CTA scratch strides (elements)
    int part_words;       // > 0: shared-memory words (after the vote partial) that accumulate one layer's messages
    int t_stride;         // > 0: a transposed-graph buffer follows, with this (odd) row stride (TransposedGraph)
};

template <bool kBatchNodes>
__global__ void __launch_bounds__(kBatchNodes ? 512 : 256, kBatchNodes ? 1 : 5) score_graphs_kernel(DevModel m, DevGraphs g, EvalScratch sc0, ScoreArgs a)
{
    extern __shared__ int s_sum[];   // [K], then the message accumulation words
    u32 *s_part = a.part_words > 0 ? reinterpret_cast<u32 *>(s_sum + ((m.K + 3) & ~3)) : nullptr;
    u32 *s_T = reinterpret_cast<u32 *>(s_sum + ((m.K + 3) & ~3)) + max(a.part_words, 0);
    const int t_rows = 32 * max(m.L0, m.MW);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    EvalScratch sc = sc0;
    sc.cno += blockIdx.x * a.cno_stride;
    sc.P += blockIdx.x * a.P_stride;
    sc.n_inc += blockIdx.x * a.ninc_stride;
    const size_t layer_words = (size_t)sc.max_nodes * m.MW;

    for (int64_t i = blockIdx.x; i < a.count; i += gridDim.x) {
        const int64_t e = a.first + i;
        const GraphView gv = global_graph(g, e, m.L0);
        const int n = gv.n;
        for (int k = threadIdx.x; k < m.K; k += blockDim.x) s_sum[k] = 0;
        const int all_words = kTransposedTypes * (m.MW | 1);    // the buffer's last rows: marks of clauses true on every node of their type
        const bool part = s_part != nullptr && ((n + 31) & ~31) * (m.MW | 1) + all_words <= a.part_words;     // source-node message bits fit the shared buffer
        TransposedGraph tg;
        tg.T = s_T; tg.TM = s_T + (size_t)t_rows * a.t_stride; tg.S = a.t_stride; tg.words = (n + 31) >> 5;
        const bool transposed = kBatchNodes && a.t_stride > 0 && n > 32 && tg.words <= a.t_stride && g.n_types <= kTransposedTypes;
        if (m.D > 1) {
            const size_t rows = (size_t)n * m.MW;
            if (part) for (int t = threadIdx.x; t < a.part_words; t += blockDim.x) s_part[t] = 0;
            for (int d = 0; d < m.D - 1; ++d)
                for (size_t t = threadIdx.x; t < rows; t += blockDim.x) sc.P[(size_t)d * layer_words + t] = 0;
        }
        __syncthreads();
        for (int d = 0; d < m.D; ++d) {
            const bool last = d == m.D - 1;
            ScatterTargets targets;
            targets.world = 1;
            targets.rank = 0;
            targets.local = part && !last ? s_part : nullptr;
            targets.local_words = transposed ? tg.words : 0;
            targets.all = (targets.local != nullptr && transposed) ? s_part + a.part_words - all_words : nullptr;
            targets.base[0] = sc.P + (size_t)d * layer_words;
            if (transposed) {
                if (d == 0) {
                    build_transposed(gv.X, n, m.L0, m.L0, tg);
                    build_type_masks(gv.type, n, g.n_types, tg);
                } else {
                    build_transposed(sc.P + (size_t)(d - 1) * layer_words, n, m.MW, m.MW, tg);
                }
                __syncthreads();
            }
            for (int c = warp; c < m.C; c += nwarps) {
                const ClauseView cv = global_view(m, sc.n_inc, c);
                const u32 any = transposed
                    ? eval_clause_layer_transposed(m, gv, g.n_types, cv, c, d, d > 0 ? cno_row(sc, m.C, d - 1, c) : nullptr,
                                                   cno_row(sc, m.C, d, c), tg, last ? nullptr : &targets, lane)
                    : eval_clause_layer<kBatchNodes>(m, gv, g.n_types, cv, c, d, d > 0 ? cno_row(sc, m.C, d - 1, c) : nullptr,
                                                  cno_row(sc, m.C, d, c), d > 0 ? sc.P + (size_t)(d - 1) * layer_words : nullptr,
                                                  last ? nullptr : &targets, lane);
                if (last) {
                    if (any)
                        for (int k = lane; k < m.K; k += 32) atomicAdd(&s_sum[k], m.weights[(size_t)k * m.C + c]);
                    if (a.clause_outputs && lane == 0) a.clause_outputs[(size_t)i * m.C + c] = any != 0;
                }
            }
            __syncthreads();
            if (targets.local) {
                // every clause has marked its bits on the source nodes: one walk over the edges makes the layer's messages
                flush_messages(targets, gv, m.MS, m.MW);
                __syncthreads();
                for (int t = threadIdx.x; t < ((n + 31) & ~31) * (m.MW | 1); t += blockDim.x) s_part[t] = 0;
                __syncthreads();
            }
        }
        for (int k = threadIdx.x; k < m.K; k += blockDim.x) a.class_sums[(size_t)i * m.K + k] = s_sum[k];
        if (a.node_outputs) {
            // the last layer's node-output words, one int per (clause, node) as kernels.py:693-709 unpacks them
            const int stride = a.node_stride;
            for (size_t t = threadIdx.x; t < (size_t)m.C * stride; t += blockDim.x) {
                const int c = (int)(t / stride), v = (int)(t - (size_t)c * stride);
                const u32 word = v < n ? cno_row(sc, m.C, m.D - 1, c)[v >> 5] : 0u;
                a.node_outputs[((size_t)i * m.C + c) * stride + v] = (int)((word >> (v & 31)) & 1u);
            }
        }
        __syncthreads();
    }
}

// The same for small models on small graphs (at most 32 nodes): ONE WARP per graph, eight graphs per CTA in flight -
// a whole CTA per graph would leave most of its warps without a clause.  Scratch slices and the shared-memory words
// (vote partial, then message accumulation) are per warp; warp barriers replace the CTA barriers.
__global__ void __launch_bounds__(256, 5) score_small_graphs_kernel(DevModel m, DevGraphs g, EvalScratch sc0, ScoreArgs a)
{
    extern __shared__ int s_dyn[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int K4 = (m.K + 3) & ~3;
    int *s_sum = s_dyn + (size_t)warp * (K4 + a.part_words);
    u32 *s_part = a.part_words > 0 ? reinterpret_cast<u32 *>(s_sum + K4) : nullptr;
    const int64_t unit = (int64_t)blockIdx.x * nwarps + warp, units = (int64_t)gridDim.x * nwarps;
    EvalScratch sc = sc0;
    sc.cno += unit * a.cno_stride;
    sc.P += unit * a.P_stride;
    sc.n_inc += unit * a.ninc_stride;
    const size_t layer_words = (size_t)sc.max_nodes * m.MW;
    const int row_words = 32 * (m.MW | 1);                     // message-bit rows of a graph of at most 32 nodes

    for (int64_t i = unit; i < a.count; i += units) {
        const int64_t e = a.first + i;
        const GraphView gv = global_graph(g, e, m.L0);
        const int n = gv.n;
        for (int k = lane; k < m.K; k += 32) s_sum[k] = 0;
        const bool part = s_part != nullptr && n <= 32 && row_words <= a.part_words;
        if (m.D > 1) {
            if (part) for (int t = lane; t < row_words; t += 32) s_part[t] = 0;
            for (int d = 0; d < m.D - 1; ++d)
                for (int t = lane; t < n * m.MW; t += 32) sc.P[(size_t)d * layer_words + t] = 0;
        }
        __syncwarp();
        for (int d = 0; d < m.D; ++d) {
            const bool last = d == m.D - 1;
            ScatterTargets targets;
            targets.world = 1;
            targets.rank = 0;
            targets.local = part && !last ? s_part : nullptr;
            targets.local_words = 0;
            targets.all = nullptr;
            targets.base[0] = sc.P + (size_t)d * layer_words;
            for (int c = 0; c < m.C; ++c) {
                const ClauseView cv = global_view(m, sc.n_inc, c);
                const u32 any = eval_clause_layer<false>(m, gv, g.n_types, cv, c, d, d > 0 ? cno_row(sc, m.C, d - 1, c) : nullptr,
                                                         cno_row(sc, m.C, d, c), d > 0 ? sc.P + (size_t)(d - 1) * layer_words : nullptr,
                                                         last ? nullptr : &targets, lane);
                if (last) {
                    if (any)
                        for (int k = lane; k < m.K; k += 32) s_sum[k] += m.weights[(size_t)k * m.C + c];
                    if (a.clause_outputs && lane == 0) a.clause_outputs[(size_t)i * m.C + c] = any != 0;
                }
            }
            __syncwarp();
            if (targets.local) {
                flush_messages(targets, gv, m.MS, m.MW, lane, 32);
                __syncwarp();
                for (int t = lane; t < row_words; t += 32) s_part[t] = 0;
                __syncwarp();
            }
        }
        for (int k = lane; k < m.K; k += 32) a.class_sums[(size_t)i * m.K + k] = s_sum[k];
        if (a.node_outputs) {
            const int stride = a.node_stride;
            for (int t = lane; t < m.C * stride; t += 32) {
                const int c = t / stride, v = t - c * stride;
                const u32 word = v < n ? cno_row(sc, m.C, m.D - 1, c)[v >> 5] : 0u;
                a.node_outputs[((size_t)i * m.C + c) * stride + v] = (int)((word >> (v & 31)) & 1u);
            }
        }
        __syncwarp();
    }
}

}  // namespace gtm
