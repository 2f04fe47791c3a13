// Tile scoring: batched inference for any depth on graph sets whose graphs have at most 128 nodes.
//
// The reference evaluates one graph at a time with five kernels per message layer (tm.py:563-662 driving
// kernels.py:407-615).  Here a persistent CTA takes a TILE of consecutive whole graphs (32*TNC node slots, graphs
// never straddle a 128-slot "quad") and keeps everything of the tile in shared memory for all layers:
//
//   1. the tile's literal rows - one contiguous piece of X - arrive through a bulk asynchronous copy
//      (cp.async.bulk, completion on an mbarrier) and are transposed into XT[literal][node word]
//      (bit i of word j = that literal on node slot 32j+i);
//   2. layer 0: a thread evaluates one clause on a PAIR of quads, r = type/valid mask AND the rows of the clause's
//      INCLUDED literals (one 128-bit shared load per literal and 128 nodes), leaving as soon as r is empty; an empty
//      clause is true (kernels.py:443-460).  The included-literal lists are rebuilt from the include planes whenever
//      the automata changed and are stored interleaved per 32 clauses, so that a warp reads them with coalesced loads;
//   3. clauses that are still true somewhere go to a survivor list (clause, node bits) and OR their node bits into the
//      rows of their hypervector bits in a bit-major mark buffer (one 128-bit OR per hypervector bit and quad); later
//      layers only visit survivors, which is what "layer d is ANDed with layer d-1" (kernels.py:525-527) comes to;
//   4. the marks are transposed to node-major rows (the message each node SENDS), one pass over the tile's edges ORs
//      them, rotated by the edge type ((hv + type) mod MS, kernels.py:581), into the destination rows, and those are
//      transposed back into PT[message bit][node word] and its complement (the negated message literals), the literal
//      rows of the next layer;
//   5. after the last layer, per graph and warp, the weights of the clauses that fired are summed over the warp with
//      redux.sync and added to the graph's class sums in shared memory (kernels.py:279-317, unclamped).
//
// Shared memory: one buffer of literal rows (transposed literals, then transposed messages) and one that serves as
// staging area, mark buffer and destination rows in turn.  Global scratch: the survivor lists (L2 traffic
// proportional to the clauses that are still true).
#include "../../include/gtm_b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <vector>

#include "gtm_tile.h"

namespace gtm {

constexpr int kTileThreads = 512;
constexpr int kTileMaxK = 16;
constexpr int kTileMaxTypes = 8;
constexpr int kTileMaxGraphs = 512;   // graphs per tile: their vote accumulators and node masks live in shared memory
constexpr int kQuadNodes = 128;
constexpr unsigned long long kTileWaitNs = 500ull * 1000ull * 1000ull;   // bound of one wait for a bulk copy: 0.5 s

// ------------------------------------------------------------------------------------------- list building
__device__ __forceinline__ const u32 *include_plane(const DevModel &m, int layer, int c)
{
    return layer == 0 ? m.ta0 + ((size_t)c * m.SB + (m.SB - 1)) * m.L0
                      : m.tam + (((size_t)(layer - 1) * m.C + c) * m.SB + (m.SB - 1)) * m.M;
}

// Row of bit p in a transposed buffer whose source rows have W words: bit b of word w lives in row b*W + w (so that
// the threads that transpose adjacent words write adjacent rows).  Layer 0: row(l) for literal l (both polarities of a
// feature are literals of their own, graphs.py:150-159).  Message layers: rows 0 .. 32*MW-1 hold the message bits, rows
// 32*MW .. 64*MW-1 their complements - literal l >= MS of a message layer is the complement of message bit l - MS
// (kernels.py:544-545).  After the literal rows come four rows of ones (list padding, one per residue class).
__device__ __forceinline__ int tile_row(int p, int W) { return (p & 31) * W + (p >> 5); }
constexpr int kTilePadRows = 4;
__host__ __device__ __forceinline__ int tile_literal_rows(int layer, int L0, int MW) { return layer == 0 ? 32 * L0 : 64 * MW; }

// Visits the rows of the included literals of a clause layer.
template <class F>
__device__ __forceinline__ void tile_for_each_included(const DevModel &m, int layer, int c, F f)
{
    const int W = layer == 0 ? m.L0 : m.M;
    const u32 last = layer == 0 ? m.lit_mask : m.msg_mask;
    const u32 *inc = include_plane(m, layer, c);
    for (int w = 0; w < W; ++w) {
        u32 bits = inc[w] & (w == W - 1 ? last : kFull);
        while (bits) {
            const int l = 32 * w + __ffs(bits) - 1;
            bits &= bits - 1;
            if (layer == 0) f(tile_row(l, m.L0));
            else f(l < m.MS ? tile_row(l, m.MW) : 32 * m.MW + tile_row(l - m.MS, m.MW));
        }
    }
}

// The list of the clause at position p of its layer's order (see tile_fill_kernel) is arranged so that its entry e
// names a row of residue class (p + e) mod 4 (row number mod 4), with
// padding rows where a class runs dry: the eight lanes that share a shared-memory wavefront of a 128-bit load hold
// eight consecutive positions, so at every step they read rows of four different classes, which with 32-byte rows
// (tiles of 8 node words) and the two quads taken in opposite order by the two halves are eight different bank
// groups - no bank conflicts, whatever literals the clauses include.  A list therefore takes as many groups of
// four entries as its fullest class has rows: cnt[c].
__global__ void tile_count_kernel(DevModel m, int layer, int *cnt)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= m.C) return;
    int n0 = 0, n1 = 0, n2 = 0, n3 = 0;
    tile_for_each_included(m, layer, c, [&](int row) {
        const int r = row & 3;
        n0 += r == 0; n1 += r == 1; n2 += r == 2; n3 += r == 3;
    });
    cnt[c] = max(max(n0, n1), max(n2, n3));
}

// Clauses are evaluated in an order of their own per layer: by decreasing list length (`order[p]` = clause at position
// p), so that the 32 clauses a warp takes together have lists of about the same length and no lane waits long for
// the longest.  The lists of the 32 clauses of a block of positions are stored interleaved - group g of position p is
// the 8-byte element blk_off[p / 32] + 32*g + p % 32 - so that the warp fetches group g of all of them with one
// coalesced 256-byte load; a block takes 32 * (its longest list) elements.  Order and offsets are made on the host
// (tile_model_refresh).
__global__ void tile_fill_kernel(DevModel m, int layer, const int *order, const int *cnt, const int *blk_off,
                                 unsigned short *list, int *Wt, int KROW, u32 *hvm)
{
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= m.C) return;
    const int c = order[p];
    const int groups = cnt[c], pad = tile_literal_rows(layer, m.L0, m.MW);
    // entry e (four per group) of this position's list: element blk_off + 32*(e/4) + lane, slot e%4
    unsigned short *base = list + ((size_t)blk_off[p >> 5] + (p & 31)) * 4;
    auto slot = [&](int e) -> unsigned short & { return base[(size_t)(e >> 2) * 128 + (e & 3)]; };
    // padding first: entry e belongs to class (p + e) mod 4; a row of ones has no effect on an AND
    for (int e = 0; e < 4 * groups; ++e) slot(e) = (unsigned short)(pad + ((p + e) & 3));
    int s0 = 0, s1 = 0, s2 = 0, s3 = 0;
    tile_for_each_included(m, layer, c, [&](int row) {
        const int r = row & 3;
        const int k = r == 0 ? s0++ : r == 1 ? s1++ : r == 2 ? s2++ : s3++;
        slot(4 * k + ((r - p) & 3)) = (unsigned short)row;        // the k-th entry of class r
    });
    if (layer == 0) {
        for (int k = 0; k < KROW; ++k) Wt[(size_t)c * KROW + k] = k < m.K ? m.weights[(size_t)k * m.C + c] : 0;
        for (int b = 0; b < m.MB; ++b) hvm[(size_t)c * m.MB + b] = m.hv[(size_t)c * m.MB + b] % (u32)m.MS;
    }
}

// -------------------------------------------------------------------------------------------------- scoring
struct TileArgs {
    const int *tile_graph;              // first graph of every tile, or NULL: every tile holds graphs_per_tile graphs
    const unsigned short *gpos;         // first node slot of every graph in its tile, or NULL (uniform sets)
    int uniform_n, graphs_per_tile;
    int tile_lo, tile_hi;               // tiles [tile_lo, tile_hi)
    int64_t first, count;               // graphs written: [first, first+count)
    int64_t n_graphs;
    int *class_sums;                    // [count][K]
    unsigned *tile_counter;             // dynamic tile scheduler (zeroed before launch)
    int TNC, PS, words_a, words_b, stage_rows, gmax;
    int rot_step;                       // message transposition: block column j is read rotated by (rot_step * j) & 31
    const TileLayer *layers;            // [D]
    const int *Wt;
    int KROW;
    const u32 *hvm;
    uint4 *surv_r;                      // [grid][2][quad pairs][C][2] node bits of every clause on the pair's two quads after a layer
    int *error;                         // raised (2) when the wait for a bulk copy gave up
};

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint4 tile_lds128(unsigned addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// ---- bulk asynchronous copy global -> shared with completion on an mbarrier (plain form: this CTA's own shared
// memory, this GPU's own global memory, no multicast) ----
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void bulk_copy_to_shared(unsigned dst, const void *src, unsigned bytes, unsigned bar)
{
    // earlier generic-proxy accesses to the destination (ordered before this thread by a CTA barrier) precede the copy
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Bounded wait for phase `parity` of the barrier: polls without blocking and gives up after kTileWaitNs of wall
// time (a bulk copy of a few kilobytes takes microseconds); false when it gave up.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity)
{
    unsigned long long t0 = 0;
    for (unsigned spins = 0;; ++spins) {
        unsigned done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((spins & 63u) == 63u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > kTileWaitNs) return false;
        }
    }
}

// r &= two rows of one quad (128-bit shared loads at a0 and a1).
__device__ __forceinline__ void tile_and_rows(uint4 &r, unsigned a0, unsigned a1)
{
    const uint4 x0 = tile_lds128(a0), x1 = tile_lds128(a1);
    r.x &= x0.x & x1.x; r.y &= x0.y & x1.y; r.z &= x0.z & x1.z; r.w &= x0.w & x1.w;
}

// Node bits of the warp's 32 clauses (lane = clause) on a PAIR of quads after ANDing the rows of their included
// literals.  lp: the lane's first list element (elements of one clause are 32 apart, see tile_fill_kernel);
// groups: its list length in groups of four rows (0 for a lane without a clause); pad4: four padding rows of the lane's
// residue classes, packed like a list element; t0 / t1: shared addresses, in row 0, of the quad this lane takes first /
// second (r0 / r1 are its node bits; lanes 4..7 of every eight take the pair in the opposite order, see
// tile_count_kernel); a row is `1 << rowshift` bytes; `two`: the pair has a second quad (warp-uniform).
// Called by all lanes of the warp, which stay in lockstep - that is what keeps their loads free of bank conflicts: the
// trip count is the warp's, a lane whose list has ended reads padding rows (all ones), a lane whose bits are all gone
// keeps reading its rows (a load costs nothing extra while the other lanes of its wavefront load anyway), and the warp
// leaves together when no lane has work left.  The next group's row numbers are fetched while the current group's
// rows are read.
__device__ __forceinline__ void tile_eval(uint4 &r0, uint4 &r1, const uint2 *lp, int groups, uint2 pad4, unsigned t0,
                                          unsigned t1, int rowshift, bool two)
{
    const int longest = __reduce_max_sync(kFull, groups);
    const unsigned keep = 0xffffu << rowshift;
    uint2 next = pad4;
    if (groups > 0) next = __ldg(lp);
#pragma unroll 1
    for (int gI = 0; gI < longest; ++gI) {
        const bool busy = gI < groups && (r0.x | r0.y | r0.z | r0.w | r1.x | r1.y | r1.z | r1.w) != 0;
        if (!__any_sync(kFull, busy)) return;
        const uint2 four = next;
        next = pad4;
        if (gI + 1 < groups) next = __ldg(lp + 32 * (gI + 1));
        const unsigned o0 = (four.x << rowshift) & keep, o1 = (four.x >> (16 - rowshift)) & keep,
                       o2 = (four.y << rowshift) & keep, o3 = (four.y >> (16 - rowshift)) & keep;
        tile_and_rows(r0, t0 + o0, t0 + o1);
        if (two) tile_and_rows(r1, t1 + o0, t1 + o1);
        tile_and_rows(r0, t0 + o2, t0 + o3);
        if (two) tile_and_rows(r1, t1 + o2, t1 + o3);
    }
}

// Bits [lo, lo+n) of a 128-bit quad.
__device__ __forceinline__ uint4 quad_mask(int lo, int n)
{
    u32 wd[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int a = min(32, max(0, lo - 32 * i)), b = min(32, max(0, lo + n - 32 * i));
        const u32 below_b = b >= 32 ? kFull : (1u << b) - 1u, below_a = a >= 32 ? kFull : (1u << a) - 1u;
        wd[i] = below_b & ~below_a;
    }
    return make_uint4(wd[0], wd[1], wd[2], wd[3]);
}

template <int KP>
__global__ void __launch_bounds__(kTileThreads, 2) tile_score_kernel(DevModel m, DevGraphs g, TileArgs a)
{
    extern __shared__ __align__(16) u32 s_dyn[];
    const int TNC = a.TNC, TN = TNC * 32, Q = TNC >> 2, PS = a.PS;
    const int rowshift = 31 - __clz(TNC * 4);
    u32 *bufA = s_dyn;                                              // literal rows / message rows, swapping roles
    u32 *bufB = bufA + a.words_a;                                   // staging of X / message rows, swapping roles
    u32 *TMV = bufB + a.words_b;                                    // [kTileMaxTypes][TNC] valid nodes of each type
    u32 *tnode = TMV + kTileMaxTypes * TNC;                         // [TN] node of each slot, or ~0
    u32 *pinfo = tnode + TN;                                        // [TN] first slot of the slot's graph | nodes << 16
    uint4 *gmask = reinterpret_cast<uint4 *>(pinfo + TN);           // [gmax] node slots of a graph inside its quad
    int *sums = reinterpret_cast<int *>(gmask + a.gmax);            // [gmax][KP]
    int *gq_first = sums + a.gmax * KP;                             // [Q+1] first graph of every quad
    int *cnt = gq_first + 12;                                       // [2][8] survivor counts per list and quad
    int *misc = cnt + 16;                                           // tile number, node range of a staging round
    unsigned long long *mbar_mem = reinterpret_cast<unsigned long long *>(misc + 4);
    unsigned char *gquad = reinterpret_cast<unsigned char *>(mbar_mem + 1);   // [gmax]
    unsigned char *pflag = gquad + ((a.gmax + 3) & ~3);             // [TN] slot's message row has bits
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = kTileThreads / 32;
    const unsigned bar = smem_u32(mbar_mem);
    const int cblocks = (m.C + 31) >> 5;                                                // blocks of 32 clauses
    uint4 *surv_r = a.surv_r + (size_t)blockIdx.x * 4 * ((Q + 1) >> 1) * m.C;         // [2][quad pairs][C][2 quads]
    const size_t x_words = (size_t)g.total_nodes * m.L0;

    if (tid == 0) mbar_init(bar, 1);
    __syncthreads();
    unsigned parity = 0;

    while (true) {
        if (tid == 0) misc[0] = a.tile_lo + (int)atomicAdd(a.tile_counter, 1u);
        __syncthreads();
        const int tile = misc[0];
        if (tile >= a.tile_hi) break;
        const int g0 = a.tile_graph ? a.tile_graph[tile] : (int)min((int64_t)tile * a.graphs_per_tile, a.n_graphs);
        const int g1 = a.tile_graph ? a.tile_graph[tile + 1] : (int)min((int64_t)(tile + 1) * a.graphs_per_tile, a.n_graphs);
        const int ng = g1 - g0;

        // ---- slot tables: which node sits where, which slots belong to which graph ----
        for (int i = tid; i < TN; i += kTileThreads) { tnode[i] = ~0u; pinfo[i] = 0u; }
        for (int i = tid; i < ng * KP; i += kTileThreads) sums[i] = 0;
        if (tid < 16) cnt[tid] = 0;
        __syncthreads();
        {
            const int gpq = a.uniform_n > 0 ? kQuadNodes / a.uniform_n : 1;
            for (int gl = tid; gl < ng; gl += kTileThreads) {
                const int n = (int)g.n_nodes[g0 + gl];
                const u32 nb = g.node_index[g0 + gl];
                const int pos = a.uniform_n > 0 ? (gl / gpq) * kQuadNodes + (gl % gpq) * n : (int)a.gpos[g0 + gl];
                for (int i = 0; i < n; ++i) { tnode[pos + i] = nb + i; pinfo[pos + i] = (u32)pos | ((u32)n << 16); }
                gmask[gl] = quad_mask(pos & (kQuadNodes - 1), n);
                gquad[gl] = (unsigned char)(pos >> 7);
            }
        }
        __syncthreads();
        for (int gl = tid; gl <= ng; gl += kTileThreads) {      // gq_first[q] = first graph whose quad is >= q
            const int qhi = gl < ng ? (int)gquad[gl] : Q, qlo = gl > 0 ? (int)gquad[gl - 1] + 1 : 0;
            for (int qq = qlo; qq <= qhi; ++qq) gq_first[qq] = gl;
        }

        // ---- literal rows of the tile: bulk copy into the staging buffer, transposed into bufA ----
        const int groups_per_round = a.stage_rows >> 5;
        for (int jr = 0; jr < TNC; jr += groups_per_round) {
            const int jend = min(TNC, jr + groups_per_round);
            if (tid == 0) { misc[1] = 0x7fffffff; misc[2] = -1; }
            __syncthreads();
            for (int p = 32 * jr + tid; p < 32 * jend; p += kTileThreads) {
                const u32 nd = tnode[p];
                if (nd != ~0u) { atomicMin(&misc[1], (int)nd); atomicMax(&misc[2], (int)nd); }
            }
            __syncthreads();
            const int na = misc[1], nb = misc[2] + 1;
            int lead = 0;
            if (nb > na) {
                // the rows of nodes [na, nb) are one contiguous piece of X; widened to 16-byte boundaries (the
                // array is allocated with that much slack)
                const size_t w0 = (size_t)na * m.L0, w1 = (size_t)nb * m.L0;
                const size_t a0 = w0 & ~(size_t)3, a1 = min((w1 + 3) & ~(size_t)3, (x_words + 3) & ~(size_t)3);
                lead = (int)(w0 - a0);
                if (tid == 0) bulk_copy_to_shared(smem_u32(bufB), g.X + a0, (unsigned)((a1 - a0) * sizeof(u32)), bar);
                if (!mbar_wait(bar, parity)) {
                    if (a.error) atomicExch(a.error, 2);
                    mbar_wait(bar, parity);           // the copy may still be in flight: give it one more bounded wait
                }
                parity ^= 1u;
            }
            const int nblk = (jend - jr) * m.L0;
            for (int blk = tid; blk < nblk; blk += kTileThreads) {
                const int jj = blk / m.L0, w = blk - jj * m.L0, j = jr + jj, rot = j & 31;
                u32 rows[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const u32 nd = tnode[32 * j + ((i + rot) & 31)];
                    rows[i] = nd != ~0u ? bufB[lead + (size_t)(nd - (u32)na) * m.L0 + w] : 0u;
                }
                transpose32(rows);
#pragma unroll
                for (int b = 0; b < 32; ++b) bufA[(size_t)(b * m.L0 + w) * TNC + j] = __funnelshift_l(rows[b], rows[b], rot);
            }
            __syncthreads();                          // the staging buffer is rewritten by the next round
        }
        for (int t = tid; t < kTilePadRows * TNC; t += kTileThreads) bufA[(size_t)(32 * m.L0) * TNC + t] = kFull;   // padding rows
        for (int j = warp; j < TNC; j += nwarps) {
            const u32 nd = tnode[32 * j + lane];
            const u32 ty = nd != ~0u ? g.node_type[nd] : ~0u;
            for (int t = 0; t < g.n_types; ++t) {
                const u32 col = __ballot_sync(kFull, ty == (u32)t);
                if (lane == 0) TMV[t * TNC + j] = col;
            }
        }
        if (m.D > 1)
            for (int i = tid; i < 32 * m.MW * TNC; i += kTileThreads) bufB[i] = 0u;
        __syncthreads();

        // ---- layers ----
        // bufA always holds the literal rows of the current layer (the transposed literals, then the transposed
        // messages); bufB takes, in turn, the message bits that the layer's true clauses mark on their nodes (bit-major,
        // the layout of the literal rows) and the node-major destination rows of the edge pass.
        const int U = (Q + 1) >> 1;                   // quad pairs: a thread evaluates a clause on two quads at a time
        const unsigned t32 = smem_u32(bufA);
        for (int d = 0; d < m.D; ++d) {
            const bool last = d == m.D - 1;
            const TileLayer L = a.layers[d];
            const int wr = d & 1, rd = wr ^ 1;        // survivor list written by this layer / read by it

            // OR of node bits r into row `dst` (four words of one quad) of the mark buffer; most bits are there already
            auto mark = [&](u32 *dst, const uint4 r) {
                const uint4 old = tile_lds128(smem_u32(dst));
                if (r.x & ~old.x) atomicOr(dst, r.x);
                if (r.y & ~old.y) atomicOr(dst + 1, r.y);
                if (r.z & ~old.z) atomicOr(dst + 2, r.z);
                if (r.w & ~old.w) atomicOr(dst + 3, r.w);
            };
            // votes of one quad: per graph, the weights of the lanes that fired, summed over the warp
            auto vote = [&](int q, const uint4 r, const int (&w)[KP]) {
                const u32 ax = __reduce_or_sync(kFull, r.x), ay = __reduce_or_sync(kFull, r.y),
                          az = __reduce_or_sync(kFull, r.z), aw = __reduce_or_sync(kFull, r.w);
                if ((ax | ay | az | aw) == 0) return;
                for (int gl = gq_first[q]; gl < gq_first[q + 1]; ++gl) {
                    const uint4 gm = gmask[gl];
                    if (((ax & gm.x) | (ay & gm.y) | (az & gm.z) | (aw & gm.w)) == 0) continue;    // nobody fired on this graph
                    const bool f = ((r.x & gm.x) | (r.y & gm.y) | (r.z & gm.z) | (r.w & gm.w)) != 0;
                    int mine = 0;
#pragma unroll
                    for (int k = 0; k < KP; ++k) {
                        const int sk = __reduce_add_sync(kFull, f ? w[k] : 0);
                        if (lane == k) mine = sk;
                    }
                    if (lane < m.K) atomicAdd(&sums[gl * KP + lane], mine);
                }
            };
            // one warp pass over the 32 clauses at positions 32*block .. 32*block+31 of the layer's order (c: the lane's
            // clause, -1: none) and the quads of pair u; ra / rb are the node bits as they were before the layer
            auto pass = [&](int block, int c, uint4 ra, uint4 rb, int u) {
                const int qa = 2 * u;
                const bool two = qa + 1 < Q;
                {
                    const bool flip = two && (lane & 4);                  // lanes 4..7 of every eight take the second quad first
                    const unsigned ta = t32 + qa * 16;
                    uint4 r0 = flip ? rb : ra, r1 = flip ? ra : rb;
                    const unsigned pad = (unsigned)tile_literal_rows(d, m.L0, m.MW);     // padding rows of classes lane, lane+1, ..
                    const uint2 pad4 = make_uint2((pad + (lane & 3)) | ((pad + ((lane + 1) & 3)) << 16),
                                                  (pad + ((lane + 2) & 3)) | ((pad + ((lane + 3) & 3)) << 16));
                    tile_eval(r0, r1, reinterpret_cast<const uint2 *>(L.list) + L.blk_off[block] + lane, c >= 0 ? L.cnt[c] : 0, pad4,
                              flip ? ta + 16 : ta, flip ? ta : ta + 16, rowshift, two);
                    ra = flip ? r1 : r0;
                    rb = flip ? r0 : r1;
                }
                const bool alive = (ra.x | ra.y | ra.z | ra.w | rb.x | rb.y | rb.z | rb.w) != 0;
                const u32 amask = __ballot_sync(kFull, alive);
                if (!last) {
                    // every clause's node bits (zeros included) for the next layer, which takes the clauses in its own order
                    if (c >= 0) {
                        const size_t at = (size_t)(wr * U + u) * m.C + c;
                        surv_r[2 * at] = ra;
                        surv_r[2 * at + 1] = rb;
                    }
                    if (amask != 0 && lane == 0) atomicAdd(&cnt[wr * 8 + u], __popc(amask));
                    if (alive) {
                        // the clause's hypervector bits on every node it is true on (the SOURCE side of kernels.py:571-588):
                        // in the bit-major buffer that is one 128-bit OR per hypervector bit and quad
                        for (int b = 0; b < m.MB; ++b) {
                            u32 *row = bufB + (size_t)tile_row((int)a.hvm[(size_t)c * m.MB + b], m.MW) * TNC + 4 * qa;
                            mark(row, ra);
                            if (two) mark(row + 4, rb);
                        }
                    }
                } else if (amask != 0) {
                    int w[KP];
#pragma unroll
                    for (int k = 0; k < KP; ++k) w[k] = 0;
                    if (alive) {
                        const int4 *wr4 = reinterpret_cast<const int4 *>(a.Wt + (size_t)c * a.KROW);
#pragma unroll
                        for (int k4 = 0; k4 < (KP + 3) / 4; ++k4) {
                            const int4 t = __ldg(wr4 + k4);
                            w[4 * k4] = t.x;
                            if (4 * k4 + 1 < KP) w[4 * k4 + 1] = t.y;
                            if (4 * k4 + 2 < KP) w[4 * k4 + 2] = t.z;
                            if (4 * k4 + 3 < KP) w[4 * k4 + 3] = t.w;
                        }
                    }
                    vote(qa, ra, w);
                    if (two) vote(qa + 1, rb, w);
                }
            };

            for (int task = warp; task < cblocks * U; task += nwarps) {
                const int u = task % U, block = task / U, p = block * 32 + lane;
                const int c = p < m.C ? L.order[p] : -1;
                uint4 ra = make_uint4(0u, 0u, 0u, 0u), rb = ra;
                if (c >= 0) {
                    if (d == 0) {
                        const u32 *tm_row = TMV + (c % g.n_types) * TNC + 8 * u;
                        ra = *reinterpret_cast<const uint4 *>(tm_row);
                        if (2 * u + 1 < Q) rb = *reinterpret_cast<const uint4 *>(tm_row + 4);
                    } else {
                        const size_t at = (size_t)(rd * U + u) * m.C + c;
                        ra = surv_r[2 * at];
                        rb = surv_r[2 * at + 1];
                    }
                }
                if (d > 0 && !__any_sync(kFull, (ra.x | ra.y | ra.z | ra.w | rb.x | rb.y | rb.z | rb.w) != 0)) {
                    // none of these clauses was true anywhere after the layer below: they stay false
                    if (!last && c >= 0) {
                        const size_t at = (size_t)(wr * U + u) * m.C + c;
                        surv_r[2 * at] = ra;
                        surv_r[2 * at + 1] = rb;
                    }
                    continue;
                }
                pass(block, c, ra, rb, u);
            }
            __syncthreads();
            if (last) break;

            // ---- messages of this layer -> literal rows of the next ----
            int survivors = 0;
            for (int u = 0; u < U; ++u) survivors += cnt[wr * 8 + u];
            if (survivors == 0) break;                // no clause is true anywhere: nothing can fire in later layers
            // (1) marked bits, bit-major in bufB -> node-major source rows in bufA (its literal rows are no longer needed)
            for (int blk = tid; blk < TNC * m.MW; blk += kTileThreads) {
                const int j = blk % TNC, w = blk / TNC, rot = (a.rot_step * j) & 31;
                u32 rows[32];
#pragma unroll
                for (int b = 0; b < 32; ++b) {
                    const u32 x = bufB[(size_t)(b * m.MW + w) * TNC + j];
                    rows[b] = __funnelshift_r(x, x, rot);
                }
                transpose32(rows);                    // rows[i] = word w of the node in slot 32j + ((i + rot) & 31)
#pragma unroll
                for (int i = 0; i < 32; ++i) bufA[(size_t)(32 * j + ((i + rot) & 31)) * PS + w] = rows[i];
            }
            if (tid < 8) cnt[rd * 8 + tid] = 0;      // the list the next layer writes
            __syncthreads();
            // (2) destination rows start empty; source rows without bits are skipped by the edge pass
            for (int i = tid; i < TN * PS; i += kTileThreads) bufB[i] = 0u;
            for (int u = tid; u < TN; u += kTileThreads) {
                u32 any = 0;
                if (tnode[u] != ~0u)
                    for (int w = 0; w < m.MW; ++w) any |= bufA[(size_t)u * PS + w];
                pflag[u] = any != 0;
            }
            __syncthreads();
            // (3) edge pass: a node's bits arrive at the destination rotated by the edge type (kernels.py:581)
            for (int i = tid; i < TN * m.MW; i += kTileThreads) {
                const int u = i / m.MW, w = i - u * m.MW;
                if (!pflag[u]) continue;
                const u32 nd = tnode[u], info = pinfo[u];
                const u32 base = info & 0xffffu, n = info >> 16;
                const u32 deg = g.degree[nd], e0 = g.edge_index[nd];
                const u32 *row = bufA + (size_t)u * PS;
                for (u32 k = 0; k < deg && e0 + k < g.total_edges; ++k) {
                    const u32 dst = g.edge[2 * (size_t)(e0 + k)], ty = g.edge[2 * (size_t)(e0 + k) + 1];
                    if (dst >= n) continue;           // malformed edge: ignore, never fault
                    const u32 val = rotated_word(row, w, ty >= (u32)m.MS ? ty % (u32)m.MS : ty, m.MS, m.MW);
                    if (val) atomicOr(&bufB[(size_t)(base + dst) * PS + w], val);
                }
            }
            __syncthreads();
            // (4) destination rows, node-major in bufB -> literal rows of the next layer, bit-major in bufA: the message
            //     bits and, 32*MW rows further, their complements (the negated message literals)
            for (int blk = tid; blk < TNC * m.MW; blk += kTileThreads) {
                const int j = blk % TNC, w = blk / TNC, rot = (a.rot_step * j) & 31;
                u32 rows[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) rows[i] = bufB[(size_t)(32 * j + ((i + rot) & 31)) * PS + w];
                transpose32(rows);
#pragma unroll
                for (int b = 0; b < 32; ++b) {
                    const u32 x = __funnelshift_l(rows[b], rows[b], rot);
                    bufA[(size_t)(b * m.MW + w) * TNC + j] = x;
                    bufA[(size_t)(32 * m.MW + b * m.MW + w) * TNC + j] = ~x;
                }
            }
            for (int t = tid; t < kTilePadRows * TNC; t += kTileThreads) bufA[(size_t)(64 * m.MW) * TNC + t] = kFull;
            __syncthreads();
            // (5) bufB is the mark buffer of the next layer, if that one sends messages too
            if (d + 1 < m.D - 1) {
                for (int i = tid; i < 32 * m.MW * TNC; i += kTileThreads) bufB[i] = 0u;
                __syncthreads();
            }
        }

        // ---- class sums of the tile's graphs (only those inside the requested range) ----
        for (int i = tid; i < ng * m.K; i += kTileThreads) {
            const int gl = i / m.K, k = i - gl * m.K;
            const int64_t gi = (int64_t)g0 + gl;
            if (gi >= a.first && gi < a.first + a.count) a.class_sums[(size_t)(gi - a.first) * m.K + k] = sums[gl * KP + k];
        }
        __syncthreads();                              // the shared tables are rewritten by the next tile
    }
}

// ------------------------------------------------------------------------------------------------ host side
static int tile_krow(int K) { return (K + 3) & ~3; }

template <int KP>
static const void *tile_kernel_ptr() { return (const void *)tile_score_kernel<KP>; }

static const void *tile_kernel_for(int K)
{
    if (K <= 2) return tile_kernel_ptr<2>();
    if (K <= 4) return tile_kernel_ptr<4>();
    if (K <= 8) return tile_kernel_ptr<8>();
    if (K <= 10) return tile_kernel_ptr<10>();
    if (K <= 12) return tile_kernel_ptr<12>();
    return tile_kernel_ptr<16>();
}

static int tile_kp(int K) { return K <= 2 ? 2 : K <= 4 ? 4 : K <= 8 ? 8 : K <= 10 ? 10 : K <= 12 ? 12 : 16; }

int tile_model_create(TileModel *tm, const DevModel &d)
{
    tm->applicable = false;
    tm->D = d.D;
    if (d.K > kTileMaxK) return GTM_OK;
    if ((size_t)std::max(32 * d.L0, d.D > 1 ? 64 * d.MW : 0) + kTilePadRows > 65535) return GTM_OK;   // row numbers are 16 bits
    tm->KROW = tile_krow(d.K);
    GTM_TRY(dev_alloc(&tm->Wt, (size_t)d.C * tm->KROW));
    GTM_TRY(dev_alloc(&tm->hvm, (size_t)d.C * d.MB));
    GTM_TRY(dev_alloc(&tm->layers, (size_t)d.D));
    for (int l = 0; l < d.D; ++l) {
        GTM_TRY(dev_alloc(&tm->cnt[l], (size_t)d.C));
        GTM_TRY(dev_alloc(&tm->order[l], (size_t)d.C));
        GTM_TRY(dev_alloc(&tm->blk_off[l], (size_t)((d.C + 31) / 32) + 1));
    }
    tm->applicable = true;
    return GTM_OK;
}

void tile_model_destroy(TileModel *tm)
{
    cudaFree(tm->Wt); cudaFree(tm->hvm); cudaFree(tm->layers);
    for (int l = 0; l < kMaxDepth; ++l) { cudaFree(tm->cnt[l]); cudaFree(tm->order[l]); cudaFree(tm->blk_off[l]); cudaFree(tm->list[l]); }
    *tm = TileModel();
}

// Rebuilds the included-literal lists of every layer (and the clause-major weights) from the current state: list
// lengths on the device, the order of the clauses (by decreasing length) and the block offsets on the host, the lists
// on the device.  One host round trip per layer; the list buffers grow to the length the state needs.
int tile_model_refresh(TileModel *tm, const DevModel &d, cudaStream_t s)
{
    if (!tm->applicable) return GTM_OK;
    const int blocks = (d.C + 255) / 256, cblocks = (d.C + 31) / 32;
    TileLayer host_layers[kMaxDepth];
    std::vector<int> cnt((size_t)d.C), order((size_t)d.C), blk_off((size_t)cblocks + 1);
    for (int l = 0; l < d.D; ++l) {
        tile_count_kernel<<<blocks, 256, 0, s>>>(d, l, tm->cnt[l]);
        GTM_CU(cudaGetLastError());
        GTM_CU(cudaMemcpyAsync(cnt.data(), tm->cnt[l], (size_t)d.C * sizeof(int), cudaMemcpyDeviceToHost, s));
        GTM_CU(cudaStreamSynchronize(s));
        for (int c = 0; c < d.C; ++c) order[(size_t)c] = c;
        std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return cnt[(size_t)x] > cnt[(size_t)y]; });
        size_t total = 0;
        for (int b = 0; b < cblocks; ++b) {           // the first clause of a block has its longest list
            blk_off[(size_t)b] = (int)total;
            total += (size_t)32 * cnt[(size_t)order[(size_t)b * 32]];
        }
        blk_off[(size_t)cblocks] = (int)total;
        if (total * 4 + 8 >= ((size_t)1 << 31)) return fail(GTM_ERR_ARG, "included-literal lists of layer %d are too long for the tile scoring kernel", l);
        const size_t need = 4 * total + 8;            // 16-bit row numbers, four per element
        if (need > tm->list_cap[l]) {
            cudaFree(tm->list[l]);
            tm->list[l] = nullptr;
            tm->list_cap[l] = 0;
            const size_t cap = need + need / 4;
            GTM_TRY(dev_alloc(&tm->list[l], cap));
            tm->list_cap[l] = cap;
        }
        GTM_CU(cudaMemcpyAsync(tm->order[l], order.data(), (size_t)d.C * sizeof(int), cudaMemcpyHostToDevice, s));
        GTM_CU(cudaMemcpyAsync(tm->blk_off[l], blk_off.data(), blk_off.size() * sizeof(int), cudaMemcpyHostToDevice, s));
        tile_fill_kernel<<<blocks, 256, 0, s>>>(d, l, tm->order[l], tm->cnt[l], tm->blk_off[l], tm->list[l], tm->Wt, tm->KROW, tm->hvm);
        GTM_CU(cudaGetLastError());
        GTM_CU(cudaStreamSynchronize(s));             // `order` and `blk_off` are reused for the next layer
        host_layers[l].order = tm->order[l];
        host_layers[l].cnt = tm->cnt[l];
        host_layers[l].blk_off = tm->blk_off[l];
        host_layers[l].list = tm->list[l];
    }
    GTM_CU(cudaMemcpyAsync(tm->layers, host_layers, (size_t)d.D * sizeof(TileLayer), cudaMemcpyHostToDevice, s));
    GTM_CU(cudaStreamSynchronize(s));                 // host_layers goes out of scope
    return GTM_OK;
}

// Shared-memory plan for tiles of TNC node words; 0 bytes when the shape cannot be served.
struct TilePlan { int words_a = 0, words_b = 0, stage_rows = 0, PS = 0; size_t bytes = 0; };

static TilePlan tile_plan(const DevModel &d, int TNC, int gmax)
{
    TilePlan p;
    const int TN = TNC * 32;
    p.PS = d.MW | 1;
    const size_t xt = (size_t)(32 * d.L0 + kTilePadRows) * TNC;
    // node-major message rows / bit-major message rows with their complements and the padding rows / mark buffer
    const size_t pm = d.D > 1 ? (size_t)TN * p.PS : 0, pt = d.D > 1 ? (size_t)(64 * d.MW + kTilePadRows) * TNC : 0;
    const size_t marks = d.D > 1 ? (size_t)32 * d.MW * TNC : 0;
    // staging: whole groups of 32 literal rows, up to 16 KB (or whatever the message rows need anyway), + 8 words of slack
    size_t stage = (size_t)32 * d.L0 * std::max<size_t>(1, std::min<size_t>(TNC, 4096 / ((size_t)32 * d.L0))) + 8;
    const size_t wa = (std::max(xt, std::max(pm, pt)) + 3) & ~(size_t)3;
    const size_t wb = (std::max(stage, std::max(pm, marks)) + 3) & ~(size_t)3;
    p.words_a = (int)wa;
    p.words_b = (int)wb;
    p.stage_rows = (int)std::min<size_t>(TN, ((wb - 8) / d.L0) / 32 * 32);
    const size_t words = wa + wb + (size_t)kTileMaxTypes * TNC + 2 * (size_t)TN + 4 * (size_t)gmax + (size_t)gmax * tile_kp(d.K) +
                         12 + 16 + 4 + 2;
    p.bytes = words * sizeof(u32) + (size_t)((gmax + 3) & ~3) + (size_t)TN;
    return p;
}

// n_min / n_max: node counts of the smallest and the largest graph when the caller knows them (0, 0 otherwise).
int tile_data_create(TileData *td, const TileModel &tm, const DevModel &d, const gtm_graphs_view *v, u32 n_min, u32 n_max,
                     int sm_count, cudaStream_t s)
{
    td->supported = 0;
    if (!tm.applicable || v->max_number_of_graph_nodes > kQuadNodes) return GTM_OK;    // a graph must fit one quad
    const int64_t N = v->number_of_graphs;
    if (n_max == 0) {
        n_min = ~0u;
        for (int64_t gi = 0; gi < N; ++gi) {
            const u32 n = v->number_of_graph_nodes[gi];
            n_min = std::min(n_min, n);
            n_max = std::max(n_max, n);
        }
    }
    if (n_min < 1 || n_max > (u32)kQuadNodes) return GTM_OK;
    const void *fn = tile_kernel_for(d.K);
    // node words per tile: the largest that lets two CTAs share an SM, else the largest that fits at all
    int TNC = 0;
    TilePlan plan;
    for (int pass = 0; pass < 2 && TNC == 0; ++pass)
        // models with many clauses spend their time in the evaluation, whose shared-memory loads are free of bank
        // conflicts with 32-byte rows (8 node words, see tile_count_kernel); small ones gain more from large tiles
        for (int cand = d.C >= 256 ? 8 : 32; cand >= 4; cand >>= 1) {
            const int gbound = (int)std::min<int64_t>(kTileMaxGraphs, std::min<int64_t>(N, cand * 32 / n_min));
            const TilePlan p = tile_plan(d, cand, gbound);
            if (p.bytes <= (pass == 0 ? (size_t)112 * 1024 : (size_t)224 * 1024)) { TNC = cand; plan = p; break; }
        }
    if (TNC == 0) return GTM_OK;
    const int TN = TNC * 32, Q = TNC / 4;
    td->TNC = TNC;
    td->uniform_n = n_min == n_max ? (int)n_min : 0;
    td->tile_graph_host.clear();
    td->tile_graph = nullptr;
    td->gpos = nullptr;
    td->stream = s;
    if (td->uniform_n > 0) {
        td->graphs_per_tile = std::min(kTileMaxGraphs, (kQuadNodes / td->uniform_n) * Q);
        td->n_tiles = (int)((N + td->graphs_per_tile - 1) / td->graphs_per_tile);
        td->gmax = (int)std::min<int64_t>(td->graphs_per_tile, N);
    } else {
        // greedy packing: consecutive graphs, a graph never straddles a quad, a tile never exceeds TN slots
        std::vector<unsigned short> gpos((size_t)N);
        std::vector<int> &tg = td->tile_graph_host;
        tg.push_back(0);
        int cur = 0, in_tile = 0, gmax = 0;
        for (int64_t gi = 0; gi < N; ++gi) {
            const int n = (int)v->number_of_graph_nodes[gi];
            int pos = cur;
            if ((pos & (kQuadNodes - 1)) + n > kQuadNodes) pos = (pos + kQuadNodes - 1) & ~(kQuadNodes - 1);
            if (pos + n > TN || in_tile >= kTileMaxGraphs) {
                tg.push_back((int)gi);
                gmax = std::max(gmax, in_tile);
                pos = 0;
                in_tile = 0;
            }
            gpos[(size_t)gi] = (unsigned short)pos;
            cur = pos + n;
            ++in_tile;
        }
        gmax = std::max(gmax, in_tile);
        tg.push_back((int)N);
        td->graphs_per_tile = 0;
        td->n_tiles = (int)tg.size() - 1;
        td->gmax = gmax;
        GTM_TRY(pool_alloc(&td->tile_graph, tg.size(), s));
        GTM_CU(cudaMemcpyAsync(td->tile_graph, tg.data(), tg.size() * sizeof(int), cudaMemcpyHostToDevice, s));
        GTM_TRY(pool_alloc(&td->gpos, (size_t)N, s));
        GTM_CU(cudaMemcpyAsync(td->gpos, gpos.data(), (size_t)N * sizeof(unsigned short), cudaMemcpyHostToDevice, s));
        GTM_CU(cudaStreamSynchronize(s));             // gpos goes out of scope
    }
    plan = tile_plan(d, TNC, td->gmax);
    td->PS = plan.PS;
    td->words_a = plan.words_a;
    td->words_b = plan.words_b;
    td->stage_rows = plan.stage_rows;
    td->smem = plan.bytes;
    GTM_CU(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)td->smem));
    int per_sm = 0;
    GTM_CU(cudaOccupancyMaxActiveBlocksPerMultiprocessorWithFlags(&per_sm, fn, kTileThreads, td->smem, 0));
    if (per_sm < 1) { tile_data_destroy(td); return GTM_OK; }
    td->grid = std::max(1, std::min(sm_count * per_sm, td->n_tiles));
    GTM_TRY(pool_alloc(&td->tile_counter, 1, s));
    td->n_graphs = N;
    td->supported = 1;
    return GTM_OK;
}

void tile_data_destroy(TileData *td)
{
    if (td->tile_graph) cudaFreeAsync(td->tile_graph, td->stream);
    if (td->gpos) cudaFreeAsync(td->gpos, td->stream);
    if (td->tile_counter) cudaFreeAsync(td->tile_counter, td->stream);
    if (td->surv_r) cudaFreeAsync(td->surv_r, td->stream);
    td->tile_graph = nullptr; td->gpos = nullptr; td->tile_counter = nullptr; td->surv_r = nullptr;
    td->supported = 0;
}

bool tile_supported(const TileData &td, int n_types) { return td.supported != 0 && n_types <= kTileMaxTypes; }

int tile_score(const TileModel &tm, TileData &td, const DevModel &d, const DevGraphs &dg, int n_types, int64_t first,
               int64_t count, int *sums_dev, int *error_dev, cudaStream_t s)
{
    const int U = (td.TNC / 4 + 1) / 2;
    if (!td.surv_r)            // node bits of every clause between layers, per resident CTA, layer parity and quad pair; allocated on first use
        GTM_TRY(pool_alloc(&td.surv_r, 2 * (size_t)td.grid * 2 * U * d.C, s));
    DevGraphs g = dg;
    g.n_types = n_types;
    TileArgs a;
    a.tile_graph = td.tile_graph;
    a.gpos = td.gpos;
    a.uniform_n = td.uniform_n;
    a.graphs_per_tile = td.graphs_per_tile;
    int lo, hi;
    if (td.graphs_per_tile > 0) {
        lo = (int)(first / td.graphs_per_tile);
        hi = (int)((first + count + td.graphs_per_tile - 1) / td.graphs_per_tile);
    } else {
        const std::vector<int> &tg = td.tile_graph_host;
        lo = (int)(std::upper_bound(tg.begin(), tg.end(), (int)first) - tg.begin()) - 1;
        hi = (int)(std::lower_bound(tg.begin(), tg.end(), (int)(first + count)) - tg.begin());
    }
    a.tile_lo = lo; a.tile_hi = hi;
    a.first = first; a.count = count; a.n_graphs = td.n_graphs;
    a.class_sums = sums_dev; a.tile_counter = td.tile_counter;
    a.TNC = td.TNC; a.PS = td.PS; a.words_a = td.words_a; a.words_b = td.words_b; a.stage_rows = td.stage_rows; a.gmax = td.gmax;
    int inv = 1;                                       // inverse of the (odd) message row stride modulo 32
    while ((td.PS * inv) % 32 != 1) inv += 2;
    a.rot_step = ((32 / td.TNC) * inv) & 31;
    a.layers = tm.layers; a.Wt = tm.Wt; a.KROW = tm.KROW; a.hvm = tm.hvm;
    a.surv_r = td.surv_r;
    a.error = error_dev;
    GTM_CU(cudaMemsetAsync(td.tile_counter, 0, sizeof(unsigned), s));
    const int grid = std::max(1, std::min(td.grid, hi - lo));
    DevModel dm = d;
    void *args[] = {&dm, &g, &a};
    GTM_CU(cudaLaunchKernel(tile_kernel_for(d.K), dim3(grid), dim3(kTileThreads), args, td.smem, s));
    return GTM_OK;
}

}  // namespace gtm
