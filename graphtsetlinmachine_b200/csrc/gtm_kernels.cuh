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
// View of clause c in the global-memory state.
__device__ __forceinline__ ClauseView global_view(const DevModel &m, int *n_inc, int c)
{
    ClauseView cv;
    cv.ta0 = m.ta0 + (size_t)c * m.SB * m.L0;
    cv.tam_stride = (size_t)m.C * m.SB * m.M;
    cv.tam = m.tam + (size_t)c * m.SB * m.M;
    cv.wgt = m.weights + c;
    cv.wstride = m.C;
    cv.pos = m.draw_pos + c;
    cv.n_inc = n_inc + c;
    cv.hv = m.hv + (size_t)c * m.MB;
    return cv;
}

__device__ __forceinline__ u32 *cno_row(const EvalScratch &sc, int C, int d, int c)
{
    const int slot = sc.cno_slots == 2 ? (d & 1) : d;
    return sc.cno + ((size_t)slot * C + c) * sc.NC;
}

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
    const size_t layer_words = (size_t)sc.max_nodes * m.MW;

    for (int64_t i = blockIdx.x; i < a.count; i += gridDim.x) {
        const int64_t e = a.first + i;
        const GraphView gv = global_graph(g, e, m.L0);
        const int n = gv.n;
        for (int k = threadIdx.x; k < m.K; k += blockDim.x) s_sum[k] = 0;
        if (m.D > 1) {
            const size_t rows = (size_t)n * m.MW;
            for (int d = 0; d < m.D - 1; ++d)
                for (size_t t = threadIdx.x; t < rows; t += blockDim.x) sc.P[(size_t)d * layer_words + t] = 0;
        }
        __syncthreads();
        for (int d = 0; d < m.D; ++d) {
            const bool last = d == m.D - 1;
            for (int c = warp; c < m.C; c += nwarps) {
                const ClauseView cv = global_view(m, sc.n_inc, c);
                const u32 any = eval_clause_layer(m, gv, g.n_types, cv, c, d, d > 0 ? cno_row(sc, m.C, d - 1, c) : nullptr,
                                                  cno_row(sc, m.C, d, c), d > 0 ? sc.P + (size_t)(d - 1) * layer_words : nullptr,
                                                  last ? nullptr : sc.P + (size_t)d * layer_words, lane);
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
    unsigned long long *exchange;   // [2][gridDim.x][K] (vote partial << 32 | step tag), ping-pong by graph parity
    u32 *P_pair[2];         // message buffers, ping-pong by graph parity ([D-1][max_nodes][MW] each)
    int max_nodes;
    unsigned *barrier;      // monotonically increasing arrival counter (zeroed before launch)
    int *error;             // set to 1 when a bounded wait gave up
    int *clause_node;       // [C]    tap: selected node of the last graph (kernels.py:347-349)
    int *update;            // [K][C] feedback type (kernels.py:385-387)
    int *class_sum_tap;     // [K]    class sums of the last graph
    unsigned long long *phase_cycles;   // [4] SM cycles CTA 0 spent in: evaluation, barriers, vote exchange, feedback
    // state-resident kernel only
    int clauses_per_cta;
    int clause_words;       // shared-memory words per clause
    int NC;                 // node words of the largest graph
};

constexpr unsigned kSpinLimit = 1u << 22;

// Grid-wide barrier over co-resident CTAs (cooperative launch).  The arrival counter only grows; arrival is a
// release, the poll an acquire, so no separate fences are needed.  The wait is bounded: after kSpinLimit polls
// the CTA raises *error and gives up.  Returns false once any CTA gave up.
__device__ __forceinline__ bool grid_barrier(unsigned *counter, unsigned target, int *error)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
        unsigned spins = 0;
        while (true) {
            unsigned seen;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
            if (seen >= target) break;
            if (*(volatile int *)error) break;
            if (++spins > kSpinLimit) { atomicExch(error, 1); break; }
        }
    }
    __syncthreads();
    return *(volatile int *)error == 0;
}

// Class sums of one graph from per-CTA vote partials, in one round: every CTA publishes its K partials as 64-bit
// words that carry the step tag next to the value (an aligned 8-byte store is single-copy atomic, so a reader that
// sees the tag sees the value), then every CTA reads all gridDim.x*K words, eight independent loads per thread in
// flight, re-polling only words whose tag is still old.  Slots alternate by graph parity: a slot is rewritten two
// steps later, which its owner can only reach after every CTA has read the current step.
// Call with s_sum complete (after a __syncthreads); leaves totals in s_total, clears s_sum.  Bounded polls.
__device__ __forceinline__ bool exchange_class_sums(unsigned long long *slots, int par, u32 tag, int *s_sum, int *s_total,
                                                    int K, int *error, int *tap)
{
    volatile unsigned long long *all = slots + (size_t)par * gridDim.x * K;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        all[(size_t)blockIdx.x * K + k] = ((unsigned long long)(u32)s_sum[k] << 32) | tag;
        s_sum[k] = 0;
        s_total[k] = 0;
    }
    __syncthreads();
    const int total = (int)gridDim.x * K;
    for (int t0 = threadIdx.x; t0 < total; t0 += 8 * blockDim.x) {
        unsigned long long v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int t = t0 + j * blockDim.x;
            v[j] = t < total ? all[t] : (unsigned long long)tag;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int t = t0 + j * blockDim.x;
            if (t >= total) continue;
            unsigned spins = 0;
            while ((u32)v[j] != tag) {
                if (++spins > kSpinLimit || *(volatile int *)error) { atomicExch(error, 1); break; }
                v[j] = all[t];
            }
            atomicAdd(&s_total[t % K], (int)(u32)(v[j] >> 32));
        }
    }
    __syncthreads();
    if (tap && blockIdx.x == 0)
        for (int k = threadIdx.x; k < K; k += blockDim.x) tap[k] = s_total[k];
    return *(volatile int *)error == 0;
}

// Four consecutive draws of a clause stream: Philox block `block` (draws 4*block .. 4*block+3), or the
// recorded words at those positions.
__device__ __forceinline__ void draw4_at(const DevModel &m, int clause, u64 block, u32 out[4])
{
    if (m.recorded) {
        const u32 *rec = m.recorded + (u64)clause * m.recorded_len;
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = rec[(4 * block + i) % m.recorded_len];
        return;
    }
    philox4x32_10((u32)block, (u32)(block >> 32), (u32)clause, 0u, m.seed_lo, m.seed_hi, out);
}

// One round of Bernoulli bits for Type I masks.  Lane l takes Philox block `first_block + 32*round + l`, i.e.
// 4 consecutive draws; the warp's 128 outcomes are packed, in draw order, into 4 words returned in every lane:
// bit t of the packed stream = [uniform(draw 4*first_block + 128*round + t) <= p]  (kernels.py:158-162 makes
// bit b of a word's mask from the word's b-th draw; the caller aligns words to the stream with a funnel shift).
__device__ __forceinline__ u32 bernoulli_nibbles(const DevModel &m, int clause, u64 block, float p, int lane)
{
    u32 o[4];
    draw4_at(m, clause, block, o);
    u32 nib = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) nib |= (to_uniform(o[i]) <= p ? 1u : 0u) << i;
    return nib << (4 * (lane & 7));
}

__device__ __forceinline__ void bernoulli_round(const DevModel &m, int clause, u64 first_block, int round, float p,
                                                int lane, u32 (&words)[4])
{
    const u32 mine = __reduce_or_sync(0xffu << (lane & 24), bernoulli_nibbles(m, clause, first_block + (u64)round * 32 + lane, p, lane));
#pragma unroll
    for (int i = 0; i < 4; ++i) words[i] = __shfl_sync(kFull, mine, 8 * i);
}

constexpr int kPackWords = 264;   // per-warp scratch: packed Bernoulli words of up to 8 positive classes x 32 words + 1

// Type I / II feedback of one clause on one layer (kernels.py:98-183), all classes in order.  The warp owns
// the clause; lanes hold one automaton word each (planes in registers).  `upd_lo` holds the feedback type of
// class `lane` (classes 0..31); further classes are read back from `update`.  Layers of at most 32 words take the
// packed Bernoulli words of up to 8 classes at a time through `pack` (per-warp shared scratch), two Philox rounds
// in flight per step; wider layers generate them class by class.  Returns the draws consumed.
template <int MAXSB>
__device__ __forceinline__ u64 layer_feedback(const DevModel &m, int c, int layer, u32 *ta, int upd_lo, const int *update,
                                              bool clause_true, bool within_budget, const u32 *row, bool row_is_msg,
                                              u64 pos0, int lane, u32 *pack)
{
    const int W = layer == 0 ? m.L0 : m.M, SB = m.SB;
    const float p = m.p_mask[layer];
    const bool all_ones = p >= 1.0f;         // every uniform is <= 1
    const u64 first_block = pos0 >> 2;
    const int shift = (int)(pos0 & 3);       // the layer's first draw sits `shift` bits into the packed stream
    int positives = 0;

    for (int g0 = 0; g0 < W; g0 += 32) {
        const int w = g0 + lane;
        const bool mine = w < W;
        const int wend = min(W, g0 + 32);
        u32 pl[MAXSB];
#pragma unroll
        for (int b = 0; b < MAXSB; ++b) pl[b] = (b < SB && mine) ? ta[(size_t)b * W + w] : 0u;
        u32 x = 0;
        if (mine && clause_true) x = row_is_msg ? msg_word(row, w, m.MS, m.MW) : row[w];
        int rank = 0, cached = -1;
        bool dirty = false;
        u32 sw[4] = {0, 0, 0, 0};
        for (int kb = 0; kb < m.K; kb += 32) {
            const int vals = kb == 0 ? upd_lo : (kb + lane < m.K ? update[(size_t)(kb + lane) * m.C + c] : 0);
            const int kn = min(32, m.K - kb);
            const u32 posmask = __ballot_sync(kFull, vals > 0 && lane < kn);
            for (int k8 = 0; k8 < kn; k8 += 8) {
                const int npos8 = __popc((posmask >> k8) & 0xffu);
                const bool packed = W <= 32 && npos8 > 0 && !all_ones;
                if (packed) {
                    // packed-stream words rank*W .. (rank+npos8)*W [+1 when the stream is not word-aligned]
                    const int j0 = rank * W, j1 = (rank + npos8) * W - (shift ? 0 : 1);
                    __syncwarp();
                    for (int q = j0 >> 2; q <= j1 >> 2; q += 2) {
                        const u32 na = bernoulli_nibbles(m, c, first_block + (u64)q * 32 + lane, p, lane);
                        const u32 nb = bernoulli_nibbles(m, c, first_block + (u64)(q + 1) * 32 + lane, p, lane);
                        const u32 wa = __reduce_or_sync(0xffu << (lane & 24), na);
                        const u32 wb = __reduce_or_sync(0xffu << (lane & 24), nb);
                        if ((lane & 7) == 0) {
                            const int ja = 4 * q + (lane >> 3) - j0, jb = ja + 4;
                            if (ja >= 0 && ja <= j1 - j0) pack[ja] = wa;
                            if (jb >= 0 && jb <= j1 - j0) pack[jb] = wb;
                        }
                    }
                    __syncwarp();
                }
                int local = 0;
                for (int kk = k8; kk < min(kn, k8 + 8); ++kk) {
                    const int u = __shfl_sync(kFull, vals, kk);
                    if (u > 0) {
                        u32 mask = kFull;
                        if (packed) {
                            const u32 lo = mine ? pack[local * W + lane] : 0u;
                            const u32 hi = (mine && shift) ? pack[local * W + lane + 1] : 0u;
                            mask = __funnelshift_r(lo, hi, shift);
                            ++local;
                        } else if (!all_ones) {
                            const int j0 = rank * W + g0;                        // packed-stream word of lane 0's mask
                            const int j1 = rank * W + wend - (shift ? 0 : 1);    // last packed word needed
                            u32 lo = 0, hi = 0;
                            for (int q = j0 >> 2; q <= j1 >> 2; ++q) {
                                if (q != cached) { bernoulli_round(m, c, first_block, q, p, lane, sw); cached = q; }
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const int rel = 4 * q + i - j0;
                                    if (rel == lane) lo = sw[i];
                                    if (rel - 1 == lane) hi = sw[i];
                                }
                            }
                            mask = __funnelshift_r(lo, hi, shift);
                        }
                        if (clause_true && within_budget) {
                            automata_inc<MAXSB>(pl, SB, m.boost == 1 ? x : (x & ~mask));
                            automata_dec<MAXSB>(pl, SB, ~x & mask);
                        } else {
                            automata_dec<MAXSB>(pl, SB, mask);
                        }
                        ++rank;
                        dirty = true;
                    } else if (u < 0 && clause_true) {
                        u32 include = 0;
#pragma unroll
                        for (int b = 0; b < MAXSB; ++b) if (b == SB - 1) include = pl[b];
                        automata_inc<MAXSB>(pl, SB, ~x & ~include);
                        dirty = true;
                    }
                }
            }
        }
        positives = rank;
        if (mine && dirty) {
#pragma unroll
            for (int b = 0; b < MAXSB; ++b) if (b < SB) ta[(size_t)b * W + w] = pl[b];
        }
    }
    return (u64)positives * W * 32;
}

// Per-class quantities of the feedback decision that do not depend on the clause (kernels.py:373-384): computed
// once per CTA and graph.  target = +1 / -1; thr = rd(1.0 * |y - clamp(sum)| / (2T)) as a float (see DevModel).
__device__ __forceinline__ void class_decision_inputs(const DevModel &m, const int *s_total, const int *y, int *s_target,
                                                      float *s_thr)
{
    for (int k = threadIdx.x; k < m.K; k += blockDim.x) {
        int sum = s_total[k];
        sum = sum > m.T ? m.T : (sum < -m.T ? -m.T : sum);
        const int yk = y[k];
        s_target[k] = 1 - 2 * (sum > yk);
        s_thr[k] = __double2float_rd(1.0 * abs(yk - sum) / (double)(2 * m.T));
    }
}

// Everything after the class sums for one clause (kernels.py:319-405 then :185-242), in the draw order of the
// reference: node selection, per-class decisions (+ weight move), layer-0 automata, message-layer automata.
// Lane-parallel throughout: node words, classes (16 per pass: both possible uniforms of every class are drawn at
// once, lanes 0..31 = the pass's next 32 draws, and a short uniform scan replays the reference's short-circuit
// order on them) and automaton words are spread over lanes; nothing per class goes through global memory.
// `bits` = the clause's node-output words of the last layer; `P` = message rows [D-1][max_nodes][MW].
template <int MAXSB>
__device__ __forceinline__ void clause_feedback(const DevModel &m, const GraphView &gv, const ClauseView &cv,
                                                const FitArgs &a, const u32 *bits, const u32 *P, const int *s_target,
                                                const float *s_thr, int c, int lane, u32 *pack)
{
    const int words = (gv.n + 31) >> 5;
    u64 pos = *cv.pos;
    const int n_inc = *cv.n_inc;

    // 1. one true node, uniformly: the (draw % count)-th set bit in ascending node order
    int count = 0;
    for (int j = lane; j < words; j += 32) count += __popc(bits[j]);
    count = __reduce_add_sync(kFull, count);
    int chosen = -1;
    if (count > 0) {
        int rank = count == 1 ? 0 : (int)(draw_at(m, c, pos) % (u32)count);   // x % 1 == 0 whatever the draw
        ++pos;
        for (int jb = 0; jb < words; jb += 32) {
            const u32 wd = jb + lane < words ? bits[jb + lane] : 0u;
            const int pc = __popc(wd);
            int incl = pc;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int t = __shfl_up_sync(kFull, incl, d);
                if (lane >= d) incl += t;
            }
            const int total = __shfl_sync(kFull, incl, 31);
            if (rank < total) {
                const u32 has = __ballot_sync(kFull, rank >= incl - pc && rank < incl);
                const int src = __ffs(has) - 1;
                const u32 swd = __shfl_sync(kFull, wd, src);
                const int before = __shfl_sync(kFull, incl - pc, src);
                chosen = (jb + src) * 32 + (int)__fns(swd, 0, rank - before + 1);
                break;
            }
            rank -= total;
        }
    }
    const bool clause_true = chosen != -1;

    // 2. feedback type per class + weight move
    int upd_lo = 0;
    for (int kb = 0; kb < m.K; kb += 16) {
        const int kn = min(16, m.K - kb);
        const float uni = to_uniform(draw_at(m, c, pos + lane));     // only the first (at most 2*kn) are consumed
        int wgt = 0, sign = 1;
        if (lane < kn) {
            wgt = cv.wgt[(size_t)(kb + lane) * cv.wstride];
            sign = (wgt >= 0) - (wgt < 0);
        }
        int used = 0;
        for (int kk = 0; kk < kn; ++kk) {
            const int t = s_target[kb + kk];
            bool skip = false;
            if (t == -1) skip = __shfl_sync(kFull, uni, used++) > m.q_keep_f;
            if (!skip) skip = __shfl_sync(kFull, uni, used++) > s_thr[kb + kk];
            const int upd = skip ? 0 : t * __shfl_sync(kFull, sign, kk);
            if (lane == kk) {
                if (upd > 0 && clause_true && abs(wgt) < INT_MAX) wgt += sign;
                else if (upd < 0 && clause_true) wgt -= sign;
                a.update[(size_t)(kb + kk) * m.C + c] = upd;
                if (upd != 0 && clause_true) cv.wgt[(size_t)(kb + kk) * cv.wstride] = wgt;
            }
            if (kb + kk < 32 && lane == kb + kk) upd_lo = upd;
        }
        pos += used;
    }
    if (m.K > 32) __syncwarp();   // classes beyond 31 are read back from a.update

    // 3./4. automata of every layer
    const bool within = n_inc <= m.max_included;
    const int node = clause_true ? chosen : 0;
    pos += layer_feedback<MAXSB>(m, c, 0, cv.ta(0), upd_lo, a.update, clause_true, within,
                                 gv.X + (size_t)node * m.L0, false, pos, lane, pack);
    for (int d = 1; d < m.D; ++d)
        pos += layer_feedback<MAXSB>(m, c, d, cv.ta(d), upd_lo, a.update, clause_true, within,
                                     P + ((size_t)(d - 1) * a.max_nodes + node) * m.MW, true, pos, lane, pack);
    if (lane == 0) {
        *cv.pos = pos;
        a.clause_node[c] = chosen;
    }
}

// Message rows of the OTHER parity are cleared for the graph after this one: every warp has finished the previous
// graph (the last reader), and the next writer comes after the remaining synchronisations of this graph.
__device__ __forceinline__ void clear_next_messages(const DevModel &m, const DevGraphs &g, const FitArgs &a, int par,
                                                    int64_t i, int64_t e)
{
    const size_t gthread = blockIdx.x * (size_t)blockDim.x + threadIdx.x, gthreads = (size_t)gridDim.x * blockDim.x;
    const int64_t nxt = i + 1 < a.count ? e + 1 : a.first;
    const size_t rows = (size_t)g.n_nodes[nxt] * m.MW;
    for (int dd = 0; dd < m.D - 1; ++dd)
        for (size_t t = gthread; t < rows; t += gthreads) a.P_pair[par ^ 1][(size_t)dd * a.max_nodes * m.MW + t] = 0;
}

#define GTM_LAP(acc) do { if (timer) { t1 = clock64(); acc += t1 - t0; t0 = t1; } } while (0)

// Persistent learning kernel, state in global memory: the whole grid works on one graph at a time (online
// learning is sequential over graphs, tm.py:668-747); warps own clauses (clause c belongs to global warp c mod
// #warps for the whole launch, so automata and weights of a clause are only ever touched by one warp).  Per
// graph: layer evaluations separated by grid barriers (messages mix all clauses), one exchange of per-CTA vote
// partials, then clause-local feedback.  Serves any model size; also the debug path that keeps every layer.
template <int MAXSB>
__global__ void __launch_bounds__(512, 1) fit_kernel(DevModel m, DevGraphs g, EvalScratch sc, FitArgs a, int eval_only)
{
    extern __shared__ int s_mem[];   // [K] running partial, [K] totals, [K] targets, [K] thresholds
    int *s_sum = s_mem, *s_total = s_mem + m.K, *s_target = s_mem + 2 * m.K;
    float *s_thr = reinterpret_cast<float *>(s_mem + 3 * m.K);
    __shared__ u32 s_pack[16][kPackWords];
    const int lane = threadIdx.x & 31;
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t layer_words = (size_t)a.max_nodes * m.MW;
    unsigned arrivals = 0;

    for (int k = threadIdx.x; k < m.K; k += blockDim.x) s_sum[k] = 0;
    __syncthreads();
    const bool timer = blockIdx.x == 0 && threadIdx.x == 0;
    long long t_eval = 0, t_bar = 0, t_tot = 0, t_fb = 0, t0 = clock64(), t1;

    u64 step = 0;
    for (int ep = 0; ep < a.epochs; ++ep) {
        for (int64_t i = 0; i < a.count; ++i, ++step) {
            const int64_t e = a.first + i;
            const int par = (int)(step & 1);
            const GraphView gv = global_graph(g, e, m.L0);
            u32 *P = a.P_pair[par];

            for (int d = 0; d < m.D; ++d) {
                const bool last = d == m.D - 1;
                if (d > 0) {
                    GTM_LAP(t_eval);
                    arrivals += gridDim.x;
                    if (!grid_barrier(a.barrier, arrivals, a.error)) return;
                    GTM_LAP(t_bar);
                    if (d == 1) clear_next_messages(m, g, a, par, i, e);
                }
                for (int c = gwarp; c < m.C; c += nwarps) {
                    const ClauseView cv = global_view(m, sc.n_inc, c);
                    const u32 any = eval_clause_layer(m, gv, g.n_types, cv, c, d, d > 0 ? cno_row(sc, m.C, d - 1, c) : nullptr,
                                                      cno_row(sc, m.C, d, c), d > 0 ? P + (size_t)(d - 1) * layer_words : nullptr,
                                                      last ? nullptr : P + (size_t)d * layer_words, lane);
                    if (last && any)
                        for (int k = lane; k < m.K; k += 32) atomicAdd(&s_sum[k], m.weights[(size_t)k * m.C + c]);
                }
            }
            __syncthreads();
            GTM_LAP(t_eval);
            if (!exchange_class_sums(a.exchange, par, (u32)step + 1u, s_sum, s_total, m.K, a.error, a.class_sum_tap)) return;
            GTM_LAP(t_tot);
            if (!eval_only) {
                class_decision_inputs(m, s_total, a.Y + (size_t)e * m.K, s_target, s_thr);
                __syncthreads();
                for (int c = gwarp; c < m.C; c += nwarps) {
                    const ClauseView cv = global_view(m, sc.n_inc, c);
                    clause_feedback<MAXSB>(m, gv, cv, a, cno_row(sc, m.C, m.D - 1, c), P, s_target, s_thr, c, lane,
                                           s_pack[threadIdx.x >> 5]);
                }
            }
            __syncthreads();   // s_total is rewritten by the next graph
            GTM_LAP(t_fb);
        }
    }
    if (timer) {
        a.phase_cycles[0] = (unsigned long long)t_eval; a.phase_cycles[1] = (unsigned long long)t_bar;
        a.phase_cycles[2] = (unsigned long long)t_tot; a.phase_cycles[3] = (unsigned long long)t_fb;
    }
}

// Staging limits of the state-resident kernel: a graph is copied to shared memory one step ahead when it has at
// most kStageNodes nodes, kStageRowWords literal words and kStageEdges edge rows; larger graphs are read in place.
constexpr int kStageNodes = 256, kStageRowWords = 1536, kStageEdges = 512;
constexpr int kStageWords = kStageRowWords + 3 * kStageNodes + 2 * kStageEdges;

__device__ __forceinline__ void async_copy_word(u32 *smem_dst, const u32 *global_src)
{
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(global_src) : "memory");
}

// State-resident learning kernel.  Same schedule as fit_kernel, but everything a clause owns lives in the shared
// memory of the CTA that owns the clause for the whole launch: automaton planes of every layer, weights, message
// hypervector, draw counter, include count and the node-output words.  The graph of the NEXT step (rows, node
// types, CSR slice, targets) is copied into shared memory with cp.async while the current step runs, and the
// sizes of the step after that are fetched too, so that no step starts with a chain of dependent global loads.
// Per graph the remaining global traffic is the vote exchange and, for depth > 1, the message rows.
// State is loaded at the start of the launch and written back at its end.
//   shared memory: [K] vote partial | [K] totals | [2][K] targets | [3][4] graph sizes | [2] staged graphs |
//                  per owned clause: clause_words words =
//                  draw counter (2) | include count (1) | pad (1) | weights [K] | hypervector [MB] | node words [2][NC] | planes
template <int MAXSB>
__global__ void __launch_bounds__(384, 2) fit_resident_kernel(DevModel m, DevGraphs g, FitArgs a)
{
    extern __shared__ __align__(16) int s_mem[];
    const int KP = (m.K + 3) & ~3;
    int *s_sum = s_mem, *s_total = s_mem + KP, *s_y = s_mem + 2 * KP;      // s_y: [2][KP]
    int *s_target = s_mem + 4 * KP;
    float *s_thr = reinterpret_cast<float *>(s_mem + 5 * KP);
    int *s_size = s_mem + 6 * KP;                                           // [3][4]: n, first node, first edge row, edge rows
    u32 *s_stage = reinterpret_cast<u32 *>(s_size + 12);                    // [2][kStageWords]
    u32 *s_pack = s_stage + 2 * kStageWords;                                // [12][kPackWords]
    u32 *s_clauses = s_pack + 12 * kPackWords;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int c_lo = blockIdx.x * a.clauses_per_cta, c_hi = min(m.C, c_lo + a.clauses_per_cta);
    const size_t layer_words = (size_t)a.max_nodes * m.MW;
    const int NC = a.NC;
    const u64 steps = (u64)a.epochs * (u64)a.count;
    unsigned arrivals = 0;

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
    auto fits = [&](const int *sz) { return sz[0] <= kStageNodes && sz[0] * m.L0 <= kStageRowWords && sz[3] <= kStageEdges; };
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
    fetch_sizes(0, e_cur);
    fetch_sizes(1, e_nxt);
    wait_copies();
    __syncthreads();
    fetch_graph(0, e_cur);
    wait_copies();
    __syncthreads();
    const bool timer = blockIdx.x == 0 && threadIdx.x == 0;
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
            gv.edge = gv.eidx + kStageNodes; gv.e_off = (u32)sz[2];
        } else {
            const int base = sz[1];
            gv.X = g.X + (size_t)base * m.L0; gv.type = g.node_type + base; gv.degree = g.degree + base;
            gv.eidx = g.edge_index + base; gv.edge = g.edge; gv.e_off = 0;
        }
        u32 *P = a.P_pair[par];
        const int *y = s_y + par * KP;
        GTM_LAP(t_x0);
        fetch_graph(step + 1, e_nxt);      // lands in the other stage buffer while this step runs
        fetch_sizes(step + 2, e_nxt2);
        GTM_LAP(t_x1);

        for (int d = 0; d < m.D; ++d) {
            const bool last = d == m.D - 1;
            if (d > 0) {
                GTM_LAP(t_eval);
                arrivals += gridDim.x;
                if (!grid_barrier(a.barrier, arrivals, a.error)) return;
                GTM_LAP(t_bar);
                if (d == 1) clear_next_messages(m, g, a, par, i, e);
            }
            for (int c = c_lo + warp; c < c_hi; c += nwarps) {
                const ClauseView cv = view_of(c);
                const u32 any = eval_clause_layer(m, gv, g.n_types, cv, c, d, d > 0 ? node_words(c, d - 1) : nullptr, node_words(c, d),
                                                  d > 0 ? P + (size_t)(d - 1) * layer_words : nullptr,
                                                  last ? nullptr : P + (size_t)d * layer_words, lane);
                if (last && any)
                    for (int k = lane; k < m.K; k += 32) atomicAdd(&s_sum[k], cv.wgt[k]);
            }
        }
        GTM_LAP(t_x2);
        __syncthreads();
        GTM_LAP(t_eval);
        if (!exchange_class_sums(a.exchange, par, (u32)step + 1u, s_sum, s_total, m.K, a.error, a.class_sum_tap)) return;
        GTM_LAP(t_tot);
        class_decision_inputs(m, s_total, y, s_target, s_thr);
        __syncthreads();
        for (int c = c_lo + warp; c < c_hi; c += nwarps) {
            const ClauseView cv = view_of(c);
            clause_feedback<MAXSB>(m, gv, cv, a, node_words(c, m.D - 1), P, s_target, s_thr, c, lane, s_pack + warp * kPackWords);
        }
        GTM_LAP(t_x3);
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
    if (timer) {
        a.phase_cycles[0] = (unsigned long long)t_eval; a.phase_cycles[1] = (unsigned long long)t_bar;
        a.phase_cycles[2] = (unsigned long long)t_tot; a.phase_cycles[3] = (unsigned long long)t_fb;
        a.phase_cycles[4] = (unsigned long long)t_x0; a.phase_cycles[5] = (unsigned long long)t_x1;
        a.phase_cycles[6] = (unsigned long long)t_x2; a.phase_cycles[7] = (unsigned long long)t_x3;
    }
}
#undef GTM_LAP

}  // namespace gtm
