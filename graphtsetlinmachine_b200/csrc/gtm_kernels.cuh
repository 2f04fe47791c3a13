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
    size_t cno_stride, P_stride, ninc_stride;  // per-CTA scratch strides (elements)
};

__global__ void __launch_bounds__(256) score_graphs_kernel(DevModel m, DevGraphs g, EvalScratch sc0, ScoreArgs a)
{
    extern __shared__ int s_sum[];   // [K]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    EvalScratch sc = sc0;
    sc.cno += blockIdx.x * a.cno_stride;
    sc.P += blockIdx.x * a.P_stride;
    sc.n_inc += blockIdx.x * a.ninc_stride;

    for (int64_t i = blockIdx.x; i < a.count; i += gridDim.x) {
        const int64_t e = a.first + i;
        const int n = (int)g.n_nodes[e], base = (int)g.node_index[e];
        for (int k = threadIdx.x; k < m.K; k += blockDim.x) s_sum[k] = 0;
        if (m.D > 1) {
            const size_t rows = (size_t)n * m.MW;
            for (int d = 0; d < m.D - 1; ++d)
                for (size_t t = threadIdx.x; t < rows; t += blockDim.x) sc.P[(size_t)d * sc.max_nodes * m.MW + t] = 0;
        }
        __syncthreads();
        for (int d = 0; d < m.D; ++d) {
            const bool last = d == m.D - 1;
            for (int c = warp; c < m.C; c += nwarps) {
                const u32 any = eval_clause_layer(m, g, sc, c, d, n, base, lane, !last);
                if (last) {
                    if (any)
                        for (int k = lane; k < m.K; k += 32) atomicAdd(&s_sum[k], m.weights[(size_t)k * m.C + c]);
                    if (a.clause_outputs && lane == 0) a.clause_outputs[(size_t)i * m.C + c] = any != 0;
                }
            }
            __syncthreads();
        }
        for (int k = threadIdx.x; k < m.K; k += blockDim.x) a.class_sums[(size_t)i * m.K + k] = s_sum[k];
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------------ learning
struct FitArgs {
    const int *Y;           // [N][K] +-T targets, absolute graph ids
    int64_t first, count;
    int epochs;
    int *partial;           // [2][gridDim.x][K] per-CTA vote partials, ping-pong by graph parity
    u32 *P_pair[2];         // message buffers, ping-pong by graph parity ([D-1][max_nodes][MW] each)
    unsigned *barrier;      // monotonically increasing arrival counter (zeroed before launch)
    int *error;             // set to 1 when a bounded wait gave up
    int *clause_node;       // [C]    tap: selected node of the last graph (kernels.py:347-349)
    int *update;            // [K][C] feedback type (kernels.py:385-387); also the per-clause working copy
    int *class_sum_tap;     // [K]    class sums of the last graph
};

constexpr unsigned kSpinLimit = 1u << 24;

// Grid-wide barrier over co-resident CTAs (cooperative launch).  Arrival counter only grows; the wait is
// bounded: after kSpinLimit polls the CTA raises *error and gives up.  Returns false once any CTA gave up.
__device__ __forceinline__ bool grid_barrier(unsigned *counter, unsigned target, int *error)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
        unsigned spins = 0;
        while (true) {
            unsigned seen;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
            if (seen >= target) break;
            if (*(volatile int *)error) break;
            if (++spins > kSpinLimit) { atomicExch(error, 1); break; }
            __nanosleep(20);
        }
        __threadfence();
    }
    __syncthreads();
    return *(volatile int *)error == 0;
}

// Type I / II feedback of one clause on one layer (kernels.py:98-183), all classes in order.  The warp owns
// the clause; lanes hold one automaton word each (planes in registers), masks are made 32 draws at a time
// with one draw per lane and a ballot, so that bit b of a word's mask is the word's b-th draw exactly as in
// the reference's loop (kernels.py:158-162).  Returns the number of draws consumed.
template <int MAXSB>
__device__ __forceinline__ u64 layer_feedback(const DevModel &m, int c, int layer, const int *update,
                                              bool clause_true, bool within_budget, const u32 *row, bool row_is_msg,
                                              u64 pos0, int lane)
{
    const int W = layer == 0 ? m.L0 : m.M, SB = m.SB;
    u32 *ta = m.ta[layer] + (size_t)c * SB * W;
    const double p = 1.0 / (double)m.s[layer];
    const bool all_ones = p >= 1.0;          // every uniform is <= 1
    int positives = 0;
    for (int k = 0; k < m.K; ++k) positives += update[(size_t)k * m.C + c] > 0;

    for (int g0 = 0; g0 < W; g0 += 32) {
        const int w = g0 + lane;
        const bool mine = w < W;
        u32 pl[MAXSB];
#pragma unroll
        for (int b = 0; b < MAXSB; ++b) pl[b] = (b < SB && mine) ? ta[(size_t)b * W + w] : 0u;
        u32 x = 0;
        if (mine && clause_true) x = row_is_msg ? msg_word(row, w, m.MS, m.MW) : row[w];
        int rank = 0;
        for (int k = 0; k < m.K; ++k) {
            const int u = update[(size_t)k * m.C + c];
            if (u > 0) {
                u32 mask = kFull;
                if (!all_ones) {
                    const int lim = min(32, W - g0);
                    for (int ww = 0; ww < lim; ++ww) {
                        const u64 idx = pos0 + ((u64)rank * W + (g0 + ww)) * 32 + lane;
                        const bool hit = (double)to_uniform(draw_at(m, c, idx)) <= p;
                        const u32 bal = __ballot_sync(kFull, hit);
                        if (lane == ww) mask = bal;
                    }
                }
                if (clause_true && within_budget) {
                    automata_inc<MAXSB>(pl, SB, m.boost == 1 ? x : (x & ~mask));
                    automata_dec<MAXSB>(pl, SB, ~x & mask);
                } else {
                    automata_dec<MAXSB>(pl, SB, mask);
                }
                ++rank;
            } else if (u < 0 && clause_true) {
                u32 include = 0;
#pragma unroll
                for (int b = 0; b < MAXSB; ++b) if (b == SB - 1) include = pl[b];
                automata_inc<MAXSB>(pl, SB, ~x & ~include);
            }
        }
        if (mine) {
#pragma unroll
            for (int b = 0; b < MAXSB; ++b) if (b < SB) ta[(size_t)b * W + w] = pl[b];
        }
    }
    return (u64)positives * W * 32;
}

// Everything after the class sums for one clause (kernels.py:319-405 then :185-242), in the draw order of the
// reference: node selection, per-class decisions (+ weight move), layer-0 automata, message-layer automata.
template <int MAXSB>
__device__ __forceinline__ void clause_feedback(const DevModel &m, const DevGraphs &g, const EvalScratch &sc,
                                                const FitArgs &a, const int *s_total, const int *y, int c, int n,
                                                int base, int lane)
{
    const int slot = sc.cno_slots == 2 ? ((m.D - 1) & 1) : m.D - 1;
    const u32 *bits = sc.cno + ((size_t)slot * m.C + c) * sc.NC;
    const int words = (n + 31) >> 5;
    u64 pos = m.draw_pos[c];

    // 1. one true node, uniformly: the (draw % count)-th set bit in ascending node order
    int count = 0;
    for (int j = lane; j < words; j += 32) count += __popc(bits[j]);
    count = __reduce_add_sync(kFull, count);
    int chosen = -1;
    if (count > 0) {
        int rank = (int)(draw_at(m, c, pos++) % (u32)count);
        for (int j = 0; j < words; ++j) {
            const u32 wd = bits[j];
            const int pc = __popc(wd);
            if (rank < pc) { chosen = j * 32 + (int)__fns(wd, 0, rank + 1); break; }
            rank -= pc;
        }
    }
    const bool clause_true = chosen != -1;

    // 2. feedback type per class + weight move (all lanes compute the same; lane 0 stores)
    for (int k = 0; k < m.K; ++k) {
        int sum = s_total[k];
        sum = sum > m.T ? m.T : (sum < -m.T ? -m.T : sum);
        const int target = 1 - 2 * (sum > y[k]);
        int wgt = m.weights[(size_t)k * m.C + c];
        const int sign = (wgt >= 0) - (wgt < 0);
        const int err = abs(y[k] - sum);
        bool skip = false;
        if (target == -1) skip = (double)to_uniform(draw_at(m, c, pos++)) > m.q_keep;
        if (!skip) skip = (double)to_uniform(draw_at(m, c, pos++)) > 1.0 * err / (double)(2 * m.T);
        int upd = 0;
        if (!skip) {
            upd = target * sign;
            if (upd > 0 && clause_true && abs(wgt) < INT_MAX) wgt += sign;
            else if (upd < 0 && clause_true) wgt -= sign;
        }
        if (lane == 0) {
            a.update[(size_t)k * m.C + c] = upd;
            m.weights[(size_t)k * m.C + c] = wgt;
        }
    }
    __syncwarp();

    // 3./4. automata of every layer
    const bool within = sc.n_inc[c] <= m.max_included;
    const int node = clause_true ? chosen : 0;
    pos += layer_feedback<MAXSB>(m, c, 0, a.update, clause_true, within, g.X + (size_t)(base + node) * m.L0, false, pos, lane);
    for (int d = 1; d < m.D; ++d)
        pos += layer_feedback<MAXSB>(m, c, d, a.update, clause_true, within,
                                     sc.P + ((size_t)(d - 1) * sc.max_nodes + node) * m.MW, true, pos, lane);
    if (lane == 0) {
        m.draw_pos[c] = pos;
        a.clause_node[c] = chosen;
    }
}

// Persistent learning kernel: the whole grid works on one graph at a time (online learning is sequential over
// graphs, tm.py:668-747); warps own clauses (clause c belongs to global warp c mod #warps for the whole launch,
// so automata and weights of a clause are only ever touched by one warp).  Per graph: layer evaluations
// separated by grid barriers (messages mix all clauses), per-CTA vote partials, one more barrier, then
// clause-local feedback.  Buffers that the next graph overwrites while slow warps may still read them
// (messages, partials) alternate by graph parity.
template <int MAXSB>
__global__ void __launch_bounds__(512) fit_kernel(DevModel m, DevGraphs g, EvalScratch sc, FitArgs a, int eval_only)
{
    extern __shared__ int s_mem[];   // [K] running partial, [K] totals
    int *s_sum = s_mem, *s_total = s_mem + m.K;
    const int lane = threadIdx.x & 31;
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t gthread = blockIdx.x * (size_t)blockDim.x + threadIdx.x, gthreads = (size_t)gridDim.x * blockDim.x;
    unsigned arrivals = 0;

    for (int k = threadIdx.x; k < m.K; k += blockDim.x) s_sum[k] = 0;
    __syncthreads();

    u64 step = 0;
    for (int ep = 0; ep < a.epochs; ++ep) {
        for (int64_t i = 0; i < a.count; ++i, ++step) {
            const int64_t e = a.first + i;
            const int par = (int)(step & 1);
            const int n = (int)g.n_nodes[e], base = (int)g.node_index[e];
            sc.P = a.P_pair[par];

            for (int d = 0; d < m.D; ++d) {
                const bool last = d == m.D - 1;
                if (d > 0) {
                    arrivals += gridDim.x;
                    if (!grid_barrier(a.barrier, arrivals, a.error)) return;
                    if (d == 1) {
                        // clear the other parity's message rows for the graph after this one: every warp has
                        // finished the previous graph (the last reader), and the next writer comes after the
                        // remaining barriers of this graph
                        int64_t nxt = i + 1 < a.count ? e + 1 : a.first;
                        const size_t rows = (size_t)g.n_nodes[nxt] * m.MW;
                        for (int dd = 0; dd < m.D - 1; ++dd)
                            for (size_t t = gthread; t < rows; t += gthreads)
                                a.P_pair[par ^ 1][(size_t)dd * sc.max_nodes * m.MW + t] = 0;
                    }
                }
                for (int c = gwarp; c < m.C; c += nwarps) {
                    const u32 any = eval_clause_layer(m, g, sc, c, d, n, base, lane, !last);
                    if (last && any)
                        for (int k = lane; k < m.K; k += 32) atomicAdd(&s_sum[k], m.weights[(size_t)k * m.C + c]);
                }
            }
            __syncthreads();
            for (int k = threadIdx.x; k < m.K; k += blockDim.x) {
                a.partial[((size_t)par * gridDim.x + blockIdx.x) * m.K + k] = s_sum[k];
                s_sum[k] = 0;
            }
            arrivals += gridDim.x;
            if (!grid_barrier(a.barrier, arrivals, a.error)) return;
            for (int k = threadIdx.x; k < m.K; k += blockDim.x) {
                int tot = 0;
                for (unsigned b = 0; b < gridDim.x; ++b) tot += a.partial[((size_t)par * gridDim.x + b) * m.K + k];
                s_total[k] = tot;
                if (blockIdx.x == 0) a.class_sum_tap[k] = tot;
            }
            __syncthreads();
            if (!eval_only) {
                const int *y = a.Y + (size_t)e * m.K;
                for (int c = gwarp; c < m.C; c += nwarps)
                    clause_feedback<MAXSB>(m, g, sc, a, s_total, y, c, n, base, lane);
            }
            __syncthreads();   // s_total is rewritten by the next graph
        }
    }
}

}  // namespace gtm
