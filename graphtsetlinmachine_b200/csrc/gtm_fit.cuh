// Device code shared by the two learning kernels: vote exchange, grid barrier, per-clause feedback.
#pragma once
#include <climits>

#include "gtm_device.cuh"

namespace gtm {

// ------------------------------------------------------------------------------------------------ learning
struct FitArgs {
    const int *Y;           // [N][K] +-T targets, absolute graph ids
    int64_t first, count;
    int epochs;
    unsigned long long *exchange;   // this rank's vote exchange area, see exchange_class_sums
    u32 *P_pair[2];         // message buffers, ping-pong by graph parity ([D-1][max_nodes][MW] each)
    u32 *Q_pair[2];         // [D-1][max_nodes][MW] destination message rows by graph parity, which the CTAs of the rank build
                            // together from the merged marks (graphs of more than 32 nodes, scatter_message_rows_share)
    unsigned *barrier_rank; // arrival counter of the barriers among this rank's CTAs only (zeroed before launch)
    int max_nodes;
    unsigned *barrier;      // monotonically increasing arrival counter: all CTAs (one GPU, zeroed before launch) or one arrival
                            // per rank and barrier (clause-sharded fit), see grid_barrier
    int *error;             // set to 1 when a bounded wait gave up
    int *clause_node;       // [C]    tap: selected node of the last graph (kernels.py:347-349)
    int *update;            // [K][C] feedback type (kernels.py:385-387)
    int *class_sum_tap;     // [K]    class sums of the last graph
    unsigned long long *phase_cycles;   // [4] SM cycles CTA 0 spent in: evaluation, barriers, vote exchange, feedback
    // state-resident kernel only
    int clauses_per_cta;
    int clause_words;       // shared-memory words per clause
    int NC;                 // node words of the largest graph
    int pre_words;          // words per clause for pre-generated Type-I masks (0 = every clause generates its own)
    int t_stride;           // > 0: the CTA has a transposed-graph buffer with this (odd) row stride, see TransposedGraph
    int timers;             // CTA 0 accumulates phase cycle counts (gtm_debug_fit_phase_cycles); off by default: the reads sit on the critical path
    int stage;              // the state-resident kernel has its two graph staging buffers (0: every graph is read in place)
    int part_words;         // > 0: shared-memory words per CTA that accumulate one layer's messages before they are merged
    int gstage_words;       // global-state kernel: shared-memory words for a copy of the current (small) graph, 0 = none
    int rows_words;         // state-resident kernel, graph sets of at most 32 nodes: shared-memory words for the message rows
                            // [D-1][32][MW] that the CTA builds from the merged marks (build_message_rows), 0 = none
    int solo;               // one CTA learns the whole model: CTA barriers replace the grid barrier and the vote exchange
    int p_smem_words;       // solo and depth > 1: message buffers (words per parity) live in that CTA's shared memory
    // clause sharding over GPUs (one process per GPU): this rank learns clauses [c_begin, c_end); votes, message bits
    // and barrier arrivals go to every rank's buffers through peer pointers.  world == 1: everything is local.
    unsigned long long wait_ns;   // budget of one device-side wait (grid barrier, vote exchange)
    int missing;            // test hook: every wait expects this many arrivals more than there are CTAs, so it runs out
    int world, rank;
    int c_begin, c_end;
    u32 tag_base;           // step tags of this launch are tag_base + step + 1
    unsigned barriers_done; // barriers of earlier launches on these counters (clause-sharded fit; 0 on one GPU)
    unsigned *barrier_local; // this rank's local arrival counter (clause-sharded fit), see grid_barrier
    unsigned long long *exchange_peer[kMaxRanks];   // the exchange areas of all ranks
    unsigned *barrier_peer[kMaxRanks];
    u32 *P_peer[kMaxRanks][2];
};

// Every device-side wait (grid barrier, vote exchange) is bounded by wall time: FitArgs::wait_ns, set from the model
// option "fit_wait_ms".  A wait that runs out raises *error; the kernel then returns and the host reports GTM_ERR_TIMEOUT.
struct WaitClock {
    unsigned long long t0 = 0;
    unsigned spins = 0;
    // true when the budget is used up; reads the clock only every 64 polls
    __device__ __forceinline__ bool expired(unsigned long long budget_ns)
    {
        if ((++spins & 63u) != 0) return false;
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (t0 == 0) { t0 = now; return false; }
        return now - t0 > budget_ns;
    }
};

// Barrier number `nb` (counted from 1) over all co-resident CTAs of all ranks (cooperative launch per rank; the ranks of
// a clause-sharded fit run the same step sequence).  Counters only grow; targets are compared wrap-safely.
//   One GPU: every CTA adds one arrival to the counter (release) and polls it (acquire) until it reads nb * gridDim.x;
//   the host zeroes the counter before every launch.
//   Several GPUs, two levels: every CTA arrives on its own rank's LOCAL counter with one answering atomic (release at
//   system scope: the CTA's marks may sit in peers' memory); the CTA whose arrival completes the rank's count for this
//   barrier adds one arrival to the GLOBAL counter of every rank (release, system scope), and every CTA polls its own
//   rank's global counter until it reads nb * world.  A peer's counter thus receives one remote atomic per rank and
//   barrier instead of one per CTA (measured at 8 GPUs: the flat form spent tens of microseconds per barrier in remote
//   atomics).  Both counters count over all launches of the shard set (nb continues from FitArgs::barriers_done).
// The wait is bounded (WaitClock): when it runs out the CTA raises *error and gives up.  Returns false once any CTA gave up.
__device__ __forceinline__ bool grid_barrier(const FitArgs &a, unsigned nb)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        WaitClock clock;
        if (a.world == 1) {
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(a.barrier) : "memory");
            const unsigned expected = nb * (gridDim.x + (unsigned)a.missing);        // test hook: an arrival that never comes
            while (true) {
                unsigned seen;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.barrier) : "memory");
                if ((int)(seen - expected) >= 0) break;
                if (*(volatile int *)a.error) break;
                if (clock.expired(a.wait_ns)) { atomicExch(a.error, 1); break; }
            }
        } else {
            unsigned before;
            asm volatile("atom.acq_rel.sys.global.add.u32 %0, [%1], 1;" : "=r"(before) : "l"(a.barrier_local) : "memory");
            if (before + 1u == nb * (gridDim.x + (unsigned)a.missing)) {
#pragma unroll
                for (int r = 0; r < kMaxRanks; ++r)      // constant indices: kernel parameters must not be indexed dynamically
                    if (r < a.world) asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(a.barrier_peer[r]) : "memory");
            }
            const unsigned expected = nb * (unsigned)a.world;
            while (true) {
                unsigned seen;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.barrier) : "memory");
                if ((int)(seen - expected) >= 0) break;
                if (*(volatile int *)a.error) break;
                if (clock.expired(a.wait_ns)) { atomicExch(a.error, 1); break; }
            }
        }
    }
    __syncthreads();
    return *(volatile int *)a.error == 0;
}

// Barrier number `nb` (counted from 1 in every launch) among the CTAs of this rank only: what they exchange lives in
// this GPU's memory, so device scope is enough and no other GPU is involved.  Bounded like every other wait.
__device__ __forceinline__ bool rank_barrier(const FitArgs &a, unsigned nb)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        WaitClock clock;
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(a.barrier_rank) : "memory");
        const unsigned expected = nb * (gridDim.x + (unsigned)a.missing);            // test hook: an arrival that never comes
        while (true) {
            unsigned seen;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.barrier_rank) : "memory");
            if ((int)(seen - expected) >= 0) break;
            if (*(volatile int *)a.error) break;
            if (clock.expired(a.wait_ns)) { atomicExch(a.error, 1); break; }
        }
    }
    __syncthreads();
    return *(volatile int *)a.error == 0;
}

// Per-class quantities of the feedback decision that do not depend on the clause (kernels.py:373-384):
// target = +1 / -1; thr = rd(1.0 * |y - clamp(sum)| / (2T)) as a float (see DevModel).
__device__ __forceinline__ void class_decision_input(int T, int sum, int yk, int *target, float *thr)
{
    sum = sum > T ? T : (sum < -T ? -T : sum);
    *target = 1 - 2 * (sum > yk);
    *thr = __double2float_rd(1.0 * abs(yk - sum) / (double)(2 * T));
}

// Where collect_votes leaves the per-class decision inputs of a single-GPU fit (the thread that reads a class sum
// computes them on the spot, which saves the CTA a pass and a barrier); y == nullptr: not wanted.
struct DecisionInputs {
    const int *y;
    int *target;
    float *thr;
    int T;
};

// Class sums of one graph from per-CTA vote partials.
//   Inside a rank, one atomic and one poll: every CTA adds, per class, ONE 64-bit word to the rank's accumulator of the
//   step - arrival count in bits 48..63, its partial plus 2^31 (never negative) in bits 0..47 - and then polls the K
//   accumulators until the count field says that every CTA has added; the class sum is the low field minus count * 2^31.
//   No arrival counter, no second round trip: the wait ends one atomic and one load after the last CTA's votes.
//   There are four accumulator sets, used by step mod 4.  CTA 0 clears the set of step+2 before it adds at `step`: that
//   set was last read at step-2, and every CTA finished reading step-2 before it added at step-1, which CTA 0 has seen
//   complete; the next add to it comes from a CTA that has seen step+1 complete, i.e. CTA 0's add of step+1, a release
//   that follows the clearing store in the same thread.  The host zeroes all sets before every launch.
//   Between ranks (clause-sharded fit): CTA 0 of every rank publishes its rank's sums as K 64-bit words that carry the
//   step tag next to the value (an aligned 8-byte store is single-copy atomic, also through a peer pointer, so a reader
//   that sees the tag sees the value) into slot [parity][own rank] of EVERY rank, and all CTAs poll the slots of the
//   other ranks.  Parities alternate by step: a slot is written again two steps later, which its writer can only reach
//   after every CTA of every rank has read the current step.
// Layout of `exchange` (8-byte units): slots [2][world][K], then the accumulators [4][K].
// Call with s_sum complete (after a __syncthreads); leaves totals in s_total, clears s_sum.  Bounded polls.
// First half: this CTA's votes go out (and CTA 0 clears the accumulators of the step after next).  Whatever the CTA
// does between the two halves runs in the shadow of the exchange.
__device__ __forceinline__ void publish_votes(const FitArgs &a, unsigned long long step, int *s_sum, int K)
{
    unsigned long long *acc_base = a.exchange + (size_t)2 * a.world * K;
    unsigned long long *acc = acc_base + (size_t)(step & 3) * K;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        if (blockIdx.x == 0) acc_base[(size_t)((step + 2) & 3) * K + k] = 0;
        const unsigned long long word = (1ull << 48) + (1ull << 31) + (unsigned long long)(long long)s_sum[k];
        asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(acc + k), "l"(word) : "memory");
        s_sum[k] = 0;
    }
}

// Second half: wait for all votes of the step; totals in s_total (valid after the closing CTA barrier), and with them the
// decision inputs when `di` asks for them and there is one GPU (returns with *di_done set then).
__device__ __forceinline__ bool collect_votes(const FitArgs &a, unsigned long long step, int par, u32 tag, int *s_total, int K,
                                              const DecisionInputs &di, bool *di_done)
{
    *di_done = di.y != nullptr && a.world == 1;
    unsigned long long *acc = a.exchange + (size_t)2 * a.world * K + (size_t)(step & 3) * K;
    const unsigned long long want = (unsigned long long)gridDim.x + (unsigned long long)a.missing;   // test hook: a CTA that never adds
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        unsigned long long v;
        WaitClock clock;
        while (true) {
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(acc + k) : "memory");
            if ((v >> 48) >= want) break;
            if (clock.expired(a.wait_ns) || *(volatile int *)a.error) { atomicExch(a.error, 1); break; }
        }
        const int mine = (int)(long long)((v & 0xffffffffffffull) - ((v >> 48) << 31));
        s_total[k] = mine;
        if (*di_done) class_decision_input(di.T, mine, di.y[k], di.target + k, di.thr + k);
        if (a.world > 1 && blockIdx.x == 0) {
            const unsigned long long out = ((unsigned long long)(u32)mine << 32) | tag;
            const size_t slot = ((size_t)par * a.world + a.rank) * K + k;
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
                if (r < a.world && r != a.rank) *(volatile unsigned long long *)(a.exchange_peer[r] + slot) = out;
        }
    }
    if (a.world > 1) {
        __syncthreads();
        volatile unsigned long long *slots = a.exchange + (size_t)par * a.world * K;
        for (int t = threadIdx.x; t < a.world * K; t += blockDim.x) {
            if (t / K == a.rank) continue;
            unsigned long long v = slots[t];
            WaitClock clock;
            while ((u32)v != tag) {
                if (clock.expired(a.wait_ns) || *(volatile int *)a.error) { atomicExch(a.error, 1); break; }
                v = slots[t];
            }
            atomicAdd(&s_total[t % K], (int)(u32)(v >> 32));
        }
    }
    __syncthreads();
    if (blockIdx.x == 0)
        for (int k = threadIdx.x; k < K; k += blockDim.x) a.class_sum_tap[k] = s_total[k];
    return *(volatile int *)a.error == 0;
}

__device__ __forceinline__ bool exchange_class_sums(const FitArgs &a, unsigned long long step, int par, u32 tag, int *s_sum,
                                                    int *s_total, int K)
{
    publish_votes(a, step, s_sum, K);
    DecisionInputs none;
    none.y = nullptr; none.target = nullptr; none.thr = nullptr; none.T = 0;
    bool done;
    return collect_votes(a, step, par, tag, s_total, K, none, &done);
}

// Four consecutive draws of a clause stream: Philox block `block` (draws 4*block .. 4*block+3), or the
// recorded words at those positions.
__device__ __forceinline__ void draw4_at(const DevModel &m, int clause, u64 block, u32 out[4])
{
    const uint4 o = draw_block(m.recorded, m.recorded_len, m.seed_lo, m.seed_hi, (u32)clause, block);
    out[0] = o.x; out[1] = o.y; out[2] = o.z; out[3] = o.w;
}

// One round of Bernoulli bits for Type I masks.  Lane l takes Philox block `first_block + 32*round + l`, i.e.
// 4 consecutive draws; the warp's 128 outcomes are packed, in draw order, into 4 words returned in every lane:
// bit t of the packed stream = [uniform(draw 4*first_block + 128*round + t) <= p]  (kernels.py:158-162 makes
// bit b of a word's mask from the word's b-th draw; the caller aligns words to the stream with a funnel shift).
// Type-I mask probability of a layer: p = rd(1/s) and the number of 32-bit draws x whose uniform is <= p.  to_uniform is
// monotone in x (conversion, exact scaling, one rounded addition), so [to_uniform(x) <= p] == [x < count] for every x:
// one integer compare per draw instead of a conversion, a multiplication, an addition and a float compare.
struct MaskProb {
    float p;
    u32 count;      // meaningless when p >= 1 (every draw passes; callers test p first)
};

__device__ __forceinline__ MaskProb mask_prob(float p)
{
    MaskProb mp;
    mp.p = p;
    // largest x with to_uniform(x) <= p, by bisection (to_uniform(0) = 2^-33; count = 0 when even that exceeds p)
    unsigned long long lo = 0, hi = 0xffffffffull;
    if (!(to_uniform(0u) <= p)) { mp.count = 0; return mp; }
    while (lo < hi) {
        const unsigned long long mid = (lo + hi + 1) >> 1;
        if (to_uniform((u32)mid) <= p) lo = mid; else hi = mid - 1;
    }
    mp.count = (u32)(lo + 1);       // wraps to 0 only when p >= 1, which callers never ask for
    return mp;
}

__device__ __forceinline__ u32 bernoulli_nibbles(const DevModel &m, int clause, u64 block, MaskProb p, int lane)
{
    u32 o[4];
    draw4_at(m, clause, block, o);
    u32 nib = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) nib |= (o[i] < p.count ? 1u : 0u) << i;
    return nib << (4 * (lane & 7));
}

// Graph copy of the global-state learning kernel: literal rows, per-node arrays of up to 32 nodes, edge rows.
constexpr int kFitStageRowWords = 2560, kFitStageEdges = 384;
constexpr int kFitStageGraphWords = kFitStageRowWords + 3 * 32 + 2 * kFitStageEdges;

// One word, global -> shared, asynchronously (completion: cp.async.wait_all).
__device__ __forceinline__ void async_copy_word(u32 *smem_dst, const u32 *global_src)
{
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(global_src) : "memory");
}

constexpr int kPackWords = 264;   // per-warp scratch: packed Bernoulli words of up to 8 positive classes x 32 words + 1

// Type I / II feedback of one clause on one layer (kernels.py:98-183), all classes in order.  The warp owns
// the clause; lanes hold one automaton word each (planes in registers).  `upd_lo` holds the feedback type of
// class `lane` (classes 0..31); further classes are read back from `update`.  Masks come from `pre` when the CTA
// generated the layer's packed Bernoulli words beforehand (generate_mask_round; the layer's first draw is bit `pre_off`
// of that stream); otherwise the words of up to 8 classes at a time are generated into `pack` (per-warp shared scratch),
// two Philox rounds in flight per step.  Words [g_begin, g_end) of the layer are updated (a multiple of 32
// apart: a wide layer can be split over several warps, every word's masks depend on the layer's first draw only).
// Returns the draws the whole layer consumes.
template <int MAXSB>
__device__ __forceinline__ u64 layer_feedback(const DevModel &m, int c, int layer, u32 *ta, int upd_lo, const int *update,
                                              bool clause_true, bool within_budget, const u32 *row, bool row_is_msg,
                                              u64 pos0, int g_begin, int g_end, int lane, u32 *pack, const u32 *pre, int pre_off,
                                              MaskProb p)
{
    const int W = layer == 0 ? m.L0 : m.M, SB = m.SB;
    const bool all_ones = p.p >= 1.0f;       // every uniform is <= 1
    const u64 first_block = pos0 >> 2;
    const int shift = (int)(pos0 & 3);       // the layer's first draw sits `shift` bits into the packed stream
    int positives = 0;

    for (int g0 = g_begin; g0 < g_end; g0 += 32) {
        const int w = g0 + lane;
        const bool mine = w < W;
        const int wend = min(W, g0 + 32);
        u32 pl[MAXSB];
#pragma unroll
        for (int b = 0; b < plane_bound<MAXSB>(SB); ++b) pl[b] = (b < SB && mine) ? ta[(size_t)b * W + w] : 0u;
        u32 x = 0;
        if (mine && clause_true) x = row_is_msg ? msg_word(row, w, m.MS, m.MW) : row[w];
        int rank = 0;
        bool dirty = false;
        for (int kb = 0; kb < m.K; kb += 32) {
            const int vals = kb == 0 ? upd_lo : (kb + lane < m.K ? update[(size_t)(kb + lane) * m.C + c] : 0);
            const int kn = min(32, m.K - kb);
            const u32 posmask = __ballot_sync(kFull, vals > 0 && lane < kn);
            for (int k8 = 0; k8 < kn; k8 += 8) {
                const int npos8 = __popc((posmask >> k8) & 0xffu);
                const bool packed = pre == nullptr && npos8 > 0 && !all_ones;
                if (packed) {
                    // The masks of these classes for words [g0, wend) go through `pack`, two Philox rounds in flight per
                    // step.  A layer of at most 32 words: stream words rank*W .. (rank+npos8)*W [+1 when the stream is not
                    // word-aligned] in one run.  A wider layer: class by class, 33 words apart in `pack`, stream words
                    // r*W + g0 .. r*W + wend [+1].
                    __syncwarp();
                    const int runs = W <= 32 ? 1 : npos8;
                    for (int cls = 0; cls < runs; ++cls) {
                        const int j0 = (rank + cls) * W + g0;
                        const int j1 = (W <= 32 ? (rank + npos8) * W : (rank + cls) * W + wend) - (shift ? 0 : 1);
                        u32 *dst = pack + cls * 33;
                        for (int q = j0 >> 2; q <= j1 >> 2; q += 2) {
                            const u32 na = bernoulli_nibbles(m, c, first_block + (u64)q * 32 + lane, p, lane);
                            const u32 nb = bernoulli_nibbles(m, c, first_block + (u64)(q + 1) * 32 + lane, p, lane);
                            const u32 wa = __reduce_or_sync(0xffu << (lane & 24), na);
                            const u32 wb = __reduce_or_sync(0xffu << (lane & 24), nb);
                            if ((lane & 7) == 0) {
                                const int ja = 4 * q + (lane >> 3) - j0, jb = ja + 4;
                                if (ja >= 0 && ja <= j1 - j0) dst[ja] = wa;
                                if (jb >= 0 && jb <= j1 - j0) dst[jb] = wb;
                            }
                        }
                    }
                    __syncwarp();
                }
                int local = 0;
                u32 todo = (__ballot_sync(kFull, vals != 0 && lane < kn) >> k8) & 0xffu;    // classes with feedback, in order
                while (todo) {
                    const int kk = k8 + __ffs(todo) - 1;
                    todo &= todo - 1;
                    const int u = __shfl_sync(kFull, vals, kk);
                    if (u > 0) {
                        u32 mask = kFull;
                        if (pre != nullptr && !all_ones) {
                            // words generated beforehand (generate_mask_round): the layer's first draw sits pre_off bits
                            // into `pre`, rank r's word w follows 32 * (r * W + w) bits later
                            const int at = (pre_off >> 5) + rank * W + lane, sh = pre_off & 31;
                            const u32 lo = mine ? pre[at] : 0u;
                            const u32 hi = (mine && sh) ? pre[at + 1] : 0u;
                            mask = __funnelshift_r(lo, hi, sh);
                        } else if (packed) {
                            const u32 *src = pack + (W <= 32 ? local * W : local * 33);
                            const u32 lo = mine ? src[lane] : 0u;
                            const u32 hi = (mine && shift) ? src[lane + 1] : 0u;
                            mask = __funnelshift_r(lo, hi, shift);
                            ++local;
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
                        for (int b = 0; b < plane_bound<MAXSB>(SB); ++b) if (b == SB - 1) include = pl[b];
                        automata_inc<MAXSB>(pl, SB, ~x & ~include);
                        dirty = true;
                    }
                }
            }
        }
        positives = rank;
        if (mine && dirty) {
#pragma unroll
            for (int b = 0; b < plane_bound<MAXSB>(SB); ++b) if (b < SB) ta[(size_t)b * W + w] = pl[b];
        }
    }
    return (u64)positives * W * 32;
}

// Per-class quantities of the feedback decision that do not depend on the clause (kernels.py:373-384): computed
// once per CTA and graph.  target = +1 / -1; thr = rd(1.0 * |y - clamp(sum)| / (2T)) as a float (see DevModel).
__device__ __forceinline__ void class_decision_inputs(const DevModel &m, const int *s_total, const int *y, int *s_target,
                                                      float *s_thr)
{
    for (int k = threadIdx.x; k < m.K; k += blockDim.x) class_decision_input(m.T, s_total[k], y[k], s_target + k, s_thr + k);
}

// Everything after the class sums for one clause (kernels.py:319-405 then :185-242), in the draw order of the
// reference: node selection, per-class decisions (+ weight move), layer-0 automata, message-layer automata.
// Lane-parallel throughout: node words, classes (16 per pass: both possible uniforms of every class are drawn at
// once, lanes 0..31 = the pass's next 32 draws, and a short uniform scan replays the reference's short-circuit
// order on them) and automaton words are spread over lanes; nothing per class goes through global memory.
// `bits` = the clause's node-output words of the last layer; `P` = message rows [D-1][p_nodes][MW].
struct Decision {
    int chosen;   // selected true node or -1
    int upd_lo;   // feedback type of class `lane` (classes 0..31)
    u64 pos;      // stream position after node choice and decisions = first mask draw of layer 0
};

// The part of the decision that does not depend on the class sums: the node choice and the uniforms of the first 16
// classes.  A kernel runs it while the vote exchange is under way.
struct PreDecision {
    int chosen;   // selected true node or -1
    u64 pos;      // stream position after the node choice
    float uni;    // uniform of draw pos + lane
};

__device__ __forceinline__ PreDecision clause_predecide(const DevModel &m, const GraphView &gv, const ClauseView &cv,
                                                        const u32 *bits, int c, int lane)
{
    const int words = (gv.n + 31) >> 5;
    u64 pos = *cv.pos;

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
    PreDecision pd;
    pd.chosen = chosen;
    pd.pos = pos;
    pd.uni = to_uniform(draw_at(m, c, pos + lane));     // only the first (at most 2 * min(K, 16)) are consumed
    return pd;
}

__device__ __forceinline__ Decision clause_decide_finish(const DevModel &m, const ClauseView &cv, const FitArgs &a,
                                                         const PreDecision &pd, const int *s_target, const float *s_thr,
                                                         int c, int lane)
{
    const int chosen = pd.chosen;
    u64 pos = pd.pos;
    const bool clause_true = chosen != -1;

    // 2. feedback type per class + weight move, 16 classes per pass, one class per lane.
    //    Class k reads its first uniform at offset o_k = k + #{j < k : negative target and its first uniform kept it},
    //    which is the reference's short-circuit order (kernels.py:384).  The offsets are the unique fixed point of that
    //    recurrence; it is found by re-evaluating all lanes until the set of kept classes stops changing (one more
    //    round than there are kept negative classes, usually two).
    int upd_lo = 0;
    for (int kb = 0; kb < m.K; kb += 16) {
        const int kn = min(16, m.K - kb);
        const float uni = kb == 0 ? pd.uni : to_uniform(draw_at(m, c, pos + lane));     // only the first (at most 2*kn) are consumed
        const bool mine = lane < kn;
        int wgt = 0, sign = 1, t = 1;
        float thr = 0.0f;
        if (mine) {
            wgt = cv.wgt[(size_t)(kb + lane) * cv.wstride];
            sign = (wgt >= 0) - (wgt < 0);
            t = s_target[kb + lane];
            thr = s_thr[kb + lane];
        }
        const u32 below = (1u << lane) - 1u;
        u32 kept = 0, seen;
        int off;
        do {
            seen = kept;
            off = lane + __popc(kept & below);
            const float u1 = __shfl_sync(kFull, uni, off & 31);
            kept = __ballot_sync(kFull, mine && t == -1 && !(u1 > m.q_keep_f));
        } while (kept != seen);
        const float u1 = __shfl_sync(kFull, uni, off & 31);
        const float u2 = __shfl_sync(kFull, uni, (off + 1) & 31);
        // negative target: dropped when the first uniform exceeds q/(K-1), else decided by the second; positive
        // target: decided by its only uniform
        const bool skip = t == -1 ? ((u1 > m.q_keep_f) || (u2 > thr)) : (u1 > thr);
        const int upd = (mine && !skip) ? t * sign : 0;
        if (mine) {
            if (upd > 0 && clause_true && abs(wgt) < INT_MAX) wgt += sign;
            else if (upd < 0 && clause_true) wgt -= sign;
            a.update[(size_t)(kb + lane) * m.C + c] = upd;
            if (upd != 0 && clause_true) cv.wgt[(size_t)(kb + lane) * cv.wstride] = wgt;
        }
        if (kb == 0) upd_lo = upd;                                    // classes 0..15 sit in lanes 0..15
        else if (kb == 16) { const int moved = __shfl_sync(kFull, upd, lane & 15); if (lane >= 16) upd_lo = moved; }
        pos += kn + __popc(kept);
    }
    if (m.K > 32) __syncwarp();   // classes beyond 31 are read back from a.update
    if (lane == 0) a.clause_node[c] = chosen;
    Decision dec;
    dec.chosen = chosen; dec.upd_lo = upd_lo; dec.pos = pos;
    return dec;
}

__device__ __forceinline__ Decision clause_decide(const DevModel &m, const GraphView &gv, const ClauseView &cv,
                                                  const FitArgs &a, const u32 *bits, const int *s_target,
                                                  const float *s_thr, int c, int lane)
{
    const PreDecision pd = clause_predecide(m, gv, cv, bits, c, lane);
    return clause_decide_finish(m, cv, a, pd, s_target, s_thr, c, lane);
}

// 3./4. automata of every layer.  `pre`, when given, holds the pre-generated packed words of all layers back to back:
// layer 0 in the first pre0_words words, its first draw at bit pre0_off (the stream may have been started before the
// decisions were known, see PreDecision); layer l >= 1 in npos*W_l + 1 words that start at the Philox block of its
// first draw.
template <int MAXSB>
__device__ __forceinline__ void clause_apply(const DevModel &m, const GraphView &gv, const ClauseView &cv, const FitArgs &a,
                                             const u32 *P, int p_nodes, const Decision &dec, int npos, int c, int lane,
                                             u32 *pack, const u32 *pre, int pre0_off, int pre0_words, const MaskProb *p_mask)
{
    const bool clause_true = dec.chosen != -1;
    if (m.K <= 32 && __ballot_sync(kFull, dec.upd_lo != 0) == 0) {      // no feedback for this clause: nothing drawn, nothing changes
        if (lane == 0) *cv.pos = dec.pos;
        return;
    }
    const bool within = *cv.n_inc <= m.max_included;
    const int node = clause_true ? dec.chosen : 0;
    u64 pos = dec.pos;
#pragma unroll 1
    for (int d = 0; d < m.D; ++d) {
        const u32 *row = d == 0 ? gv.X + (size_t)node * m.L0 : P + ((size_t)(d - 1) * p_nodes + node) * m.MW;
        const int off = d == 0 ? pre0_off : (int)(pos & 3);
        pos += layer_feedback<MAXSB>(m, c, d, cv.ta(d), dec.upd_lo, a.update, clause_true, within, row, d > 0, pos, 0,
                                     d == 0 ? m.L0 : m.M, lane, pack, pre, off, p_mask[d]);
        if (pre) pre += d == 0 ? pre0_words : npos * m.M + 1;
    }
    if (lane == 0) *cv.pos = pos;
}

template <int MAXSB>
__device__ __forceinline__ void clause_feedback(const DevModel &m, const GraphView &gv, const ClauseView &cv,
                                                const FitArgs &a, const u32 *bits, const u32 *P, int p_nodes,
                                                const int *s_target, const float *s_thr, int c, int lane, u32 *pack,
                                                const MaskProb *p_mask)
{
    const Decision dec = clause_decide(m, gv, cv, a, bits, s_target, s_thr, c, lane);
    clause_apply<MAXSB>(m, gv, cv, a, P, p_nodes, dec, 0, c, lane, pack, nullptr, 0, 0, p_mask);
}

// Round q of a packed Bernoulli stream that starts at Philox block `first_block`: the warp's 32 blocks
// first_block + 32q .. + 31 give 128 outcomes [uniform <= p], in draw order, = words 4q .. 4q+3 of the stream; words
// below `need` are written to dst.
__device__ __forceinline__ void generate_mask_round(const DevModel &m, int c, u64 first_block, int need, int q, u32 *dst,
                                                    int lane, MaskProb p)
{
    const u32 nib = bernoulli_nibbles(m, c, first_block + (u64)q * 32 + lane, p, lane);
    const u32 word = __reduce_or_sync(0xffu << (lane & 24), nib);
    const int j = 4 * q + (lane >> 3);
    if ((lane & 7) == 0 && j < need) dst[j] = word;
}

// Per-layer constants and peer pointers that the kernels index at run time are copied from the kernel parameters
// to shared memory once (constant indices here): a dynamically indexed parameter array would be spilled to local
// memory and every access to it could miss the small L1 that is left beside the shared-memory carve-out.
struct FitShared {
    MaskProb p_mask[kMaxDepth];
    u32 *P_peer[kMaxRanks][2];
};

__device__ __forceinline__ void fill_fit_shared(FitShared *fs, const DevModel &m, const FitArgs &a)
{
    if (threadIdx.x == 0) {
#pragma unroll
        for (int l = 0; l < kMaxDepth; ++l) fs->p_mask[l] = mask_prob(m.p_mask[l]);
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) { fs->P_peer[r][0] = a.P_peer[r][0]; fs->P_peer[r][1] = a.P_peer[r][1]; }
    }
}

// Message rows of the OTHER parity are cleared for the graph after this one: every warp has finished the previous
// graph (the last reader), and the next writer comes after the remaining synchronisations of this graph.
__device__ __forceinline__ void clear_next_messages(const DevModel &m, const FitArgs &a, u32 *P_other, int next_nodes)
{
    const size_t gthread = blockIdx.x * (size_t)blockDim.x + threadIdx.x, gthreads = (size_t)gridDim.x * blockDim.x;
    const size_t rows = (size_t)next_nodes * m.MW;
    for (int dd = 0; dd < m.D - 1; ++dd)
        for (size_t t = gthread; t < rows; t += gthreads) P_other[(size_t)dd * a.max_nodes * m.MW + t] = 0;
}

#define GTM_LAP(acc) do { if (timer) { t1 = clock64(); acc += t1 - t0; t0 = t1; } } while (0)

}  // namespace gtm
