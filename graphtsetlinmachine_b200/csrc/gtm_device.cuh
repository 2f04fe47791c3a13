// Device-side building blocks shared by the scoring and learning kernels: parameter blocks, the per-clause
// Philox4x32-10 draw streams, bit-sliced automaton arithmetic and the per-layer clause evaluation.
//
// Internal layouts (device memory):
//   ta0 / tam   uint32[C][SB][W] per layer: automaton planes of a clause are contiguous; plane SB-1 is the include mask;
//                                  W = ceil(literals/32) for layer 0, ceil(2*message_size/32) for layers >= 1.
//                                  (The reference keeps uint32[C][W][SB]: kernels.py:58,437.  Converted at the ABI.)
//   weights     int32[K][C]        as the reference (kernels.py:312).
//   hv          uint32[C][MB]      message hypervectors (kernels.py:567).
//   cno         uint32[slots][C][NC]  node-output bits per layer, bit v%32 of word v/32 (kernels.py:463-465);
//                                  only the bits of existing nodes are ever set.
//   P           uint32[D-1][max_nodes][MW]  POSITIVE half of the message literals of every node, MW =
//                                  ceil(message_size/32).  The reference materialises both halves
//                                  (kernels.py:544-545,582-583,613); here the negated half is derived on the
//                                  fly as the complement (msg_word).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace gtm {

typedef uint32_t u32;
typedef uint64_t u64;

constexpr int kMaxDepth = 16;
constexpr int kMaxStateBits = 32;
constexpr unsigned kFull = 0xffffffffu;

struct DevModel {
    int C, K, literals, SB, boost, T, max_included, MS, MB, D;
    int L0, M, MW;             // words: layer-0 literals, message literals (both halves), positive message half
    u32 lit_mask, msg_mask;    // valid bits of the last literal word (FILTER / MESSAGE_FILTER, kernels.py:37-47)
    float s[kMaxDepth];
    double q_keep;             // 1.0*Q/max(1, CLASSES-1)   (kernels.py:384)
    // The reference compares float uniforms with double thresholds (`u <= 1.0/s`, `u > 1.0*Q/...`).  For a float u
    // and a double d, u <= d  <=>  u <= rd(d) and u > d  <=>  u > rd(d), rd = round towards -inf to float, so the
    // hot loops compare floats and stay exact.
    float p_mask[kMaxDepth];   // rd(1.0 / s[layer])
    float q_keep_f;            // rd(q_keep)
    u32 *ta0;                  // layer 0 planes            [C][SB][L0]
    u32 *tam;                  // message-layer planes      [D-1][C][SB][M]
    int *weights;
    const u32 *hv;
    u64 *draw_pos;             // [C] draws consumed per clause stream
    const u32 *recorded;       // optional [C][recorded_len]
    u64 recorded_len;
    u32 seed_lo, seed_hi;
};

struct DevGraphs {
    const u32 *X, *node_type, *degree, *edge_index, *edge, *node_index, *n_nodes;
    const u32 *graph_edge0, *graph_edges;   // per graph: first edge row and number of edge rows (derived at upload)
    int n_types;
    // Bounds for the kernels' guards.  Host arrays are validated when a graph set is created; arrays that arrive as
    // device pointers cannot be, so a graph whose node range or node count is out of bounds is skipped (its class sums
    // are zero) and *error is raised, and edge rows past total_edges are ignored.
    u32 total_nodes, total_edges;
    int max_nodes;
    int *error;                             // may be null
};

// One graph as the evaluation sees it: either pointers into the uploaded arrays or into a shared-memory copy.
struct GraphView {
    const u32 *X;        // literal rows, row v at X + v*L0
    const u32 *type;     // [n] node types
    const u32 *degree;   // [n] out-degrees
    const u32 *eidx;     // [n] CSR row starts (absolute edge rows)
    const u32 *edge;     // edge rows (dst, type); row r of the graph set is at edge + 2*(r - e_off)
    u32 e_off;
    u32 e_cnt;           // rows addressable through `edge`: a row r is read only when r - e_off < e_cnt
    int n;
};

__device__ __forceinline__ GraphView global_graph(const DevGraphs &g, int64_t e, int L0)
{
    GraphView v;
    u32 base = g.node_index[e];
    u32 n = g.n_nodes[e];
    if (n > (u32)g.max_nodes || base > g.total_nodes || n > g.total_nodes - base) {   // malformed: skip, never index past the arrays or the scratch
        if (g.error) *g.error = 1;
        n = 0;
        base = 0;
    }
    v.n = (int)n;
    v.X = g.X + (size_t)base * L0;
    v.type = g.node_type + base;
    v.degree = g.degree + base;
    v.eidx = g.edge_index + base;
    v.edge = g.edge;
    v.e_off = 0;
    v.e_cnt = g.total_edges;
    return v;
}

// Per-"context" scratch: one for the learning kernel, one per CTA for the scoring kernel.
struct EvalScratch {
    u32 *cno;       // [cno_slots][C][NC]
    u32 *P;         // [D-1][max_nodes][MW]
    int *n_inc;     // [C]
    int NC;         // row stride of cno in words
    int cno_slots;  // D (every layer kept) or 2 (ping-pong)
    int max_nodes;
};

// ------------------------------------------------------------------------------------------------ Philox
__device__ __forceinline__ void philox4x32_10(u32 c0, u32 c1, u32 c2, u32 c3, u32 k0, u32 k1, u32 out[4])
{
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const u32 lo0 = 0xD2511F53u * c0, hi0 = __umulhi(0xD2511F53u, c0);
        const u32 lo1 = 0xCD9E8D57u * c2, hi1 = __umulhi(0xCD9E8D57u, c2);
        c0 = hi1 ^ c1 ^ k0; c1 = lo1;
        c2 = hi0 ^ c3 ^ k1; c3 = lo0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Four consecutive draws (stream positions 4*block .. 4*block+3) of the stream of clause c: Philox(counter = (block, c, 0)),
// or the recorded words at those positions.
__device__ __forceinline__ uint4 draw_block(const u32 *recorded, u64 recorded_len, u32 seed_lo, u32 seed_hi, u32 clause, u64 block)
{
    if (recorded) {
        const u32 *rec = recorded + (u64)clause * recorded_len;
        const u64 at = (4 * block) % recorded_len;
        uint4 r;
        r.x = rec[at];
        r.y = rec[(at + 1) % recorded_len];
        r.z = rec[(at + 2) % recorded_len];
        r.w = rec[(at + 3) % recorded_len];
        return r;
    }
    u32 o[4];
    philox4x32_10((u32)block, (u32)(block >> 32), clause, 0u, seed_lo, seed_hi, o);
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// Draw i of the stream of clause c: component (i & 3) of draw_block(i >> 2).
__device__ __forceinline__ u32 draw_at(const DevModel &m, int clause, u64 i)
{
    const uint4 o = draw_block(m.recorded, m.recorded_len, m.seed_lo, m.seed_hi, (u32)clause, i >> 2);
    const u32 sel = (u32)i & 3u;
    return sel == 0 ? o.x : sel == 1 ? o.y : sel == 2 ? o.z : o.w;
}

// (0, 1] mapping of curand_uniform: x * 2^-32 + 2^-33 in float (the product is exact, so one rounding either way).
__device__ __forceinline__ float to_uniform(u32 x)
{
    return __fadd_rn(__fmul_rn((float)x, 2.3283064365386963e-10f), 1.1641532182693481e-10f);
}

// ------------------------------------------------------------------------------------- message literal words
// Word w of a node's message literal vector in the reference's layout (2*MS literals: first the MS message bits,
// then their complements, zero padding; kernels.py:544-545,607-613), from the node's positive bits Prow[MW].
__device__ __forceinline__ u32 msg_word(const u32 *Prow, int w, int MS, int MW)
{
    if ((MS & 31) == 0) return w < MW ? Prow[w] : ~Prow[w - MW];
    const int lo = 32 * w;
    u32 r = 0;
    if (lo < MS) {
        u32 p = Prow[w];
        if (lo + 32 > MS) p &= (1u << (MS - lo)) - 1u;
        r = p;
    }
    if (lo + 32 > MS && lo < 2 * MS) {
        const int l0 = lo > MS ? lo : MS;              // first negated literal inside this word
        const int off = l0 - MS;                       // its bit index in Prow
        const int hi = lo + 32 < 2 * MS ? lo + 32 : 2 * MS;
        const int cnt = hi - l0;
        u32 a = Prow[off >> 5] >> (off & 31);
        if ((off & 31) && (off >> 5) + 1 < MW) a |= Prow[(off >> 5) + 1] << (32 - (off & 31));
        a = ~a;
        if (cnt < 32) a &= (1u << cnt) - 1u;
        r |= a << (l0 - lo);
    }
    return r;
}

// ------------------------------------------------------------------------------------------- clause evaluation
// Where one clause's state lives.  The general kernels point these at global memory, the state-resident learning
// kernel at shared memory; the arithmetic is the same code either way.
struct ClauseView {
    u32 *ta0;             // this clause's planes of layer 0: [SB][L0]; plane SB-1 = include mask
    u32 *tam;             // planes of message layer 1: [SB][M]; layer l >= 1 sits (l-1)*tam_stride words further
    size_t tam_stride;
    __device__ __forceinline__ u32 *ta(int l) const { return l == 0 ? ta0 : tam + (size_t)(l - 1) * tam_stride; }
    int *wgt;             // weight of class k at wgt[k * wstride]
    int wstride;
    u64 *pos;             // draws consumed by the clause's stream
    int *n_inc;           // include count summed over layers (kernels.py:440,502)
    const u32 *hv;        // [MB] message hypervector of the clause
};

// Message buffers that receive a scatter: the local one, or the same buffer on every GPU of a clause-sharded fit
// (peer pointers; plain atomics over NVLink).
constexpr int kMaxRanks = 8;
constexpr int kTransposedTypes = 8;   // node types a transposed graph keeps masks for
struct ScatterTargets {
    int world;
    int rank;              // own index in base[] (clause-sharded fit); bits are sent to the peers only when they are new here
    u32 *local;            // CTA-local accumulation in shared memory of SOURCE-node bits (see flush_messages), or null:
                           // node v's MW words start at local_row(v) * (MW | 1) - odd row stride, and for the transposed
                           // evaluation (lane = node word) the rows of the nodes of one word are `local_words` apart, so
                           // that neither evaluation's lanes meet in one bank
    int local_words;       // node words of the graph when the rows are in transposed order, 0 for node order
    u32 *all;              // [kTransposedTypes][MW | 1] bits of clauses that are true on EVERY node of their type (one mark
                           // instead of one per node; flush_messages folds them into the rows), or null
    u32 *base[kMaxRanks];
};

__device__ __forceinline__ u32 *local_row(const ScatterTargets &t, int v, int MW)
{
    const int r = t.local_words > 0 ? (v & 31) * t.local_words + (v >> 5) : v;
    return t.local + (size_t)r * (MW | 1);
}

// Bits [32w, 32w+32) of the message vector `row` (MS bits in MW words) rotated up by t: bit j = row bit (j - t) mod MS.
__device__ __forceinline__ u32 rotated_word(const u32 *row, int w, u32 t, int MS, int MW)
{
    if ((MS & 31) == 0) {
        const u32 start = (u32)(32 * w + MS - (int)t);                 // t < MS
        const u32 s0 = start >= (u32)MS ? start - (u32)MS : start;     // first source bit, a multiple-of-32 ring
        const int i = (int)(s0 >> 5), sh = (int)(s0 & 31);
        const u32 lo = row[i], hi = row[i + 1 < MW ? i + 1 : 0];
        return __funnelshift_r(lo, hi, sh);
    }
    u32 out = 0;
    for (int k = 0; k < 32; ++k) {
        const int j = 32 * w + k;
        if (j >= MS) break;
        int src = j - (int)t;
        if (src < 0) src += MS;
        out |= ((row[src >> 5] >> (src & 31)) & 1u) << k;
    }
    return out;
}

// The message a node sends is the OR of the hypervector bits of the clauses that are true on it; along an edge of
// type t it arrives rotated by t ((hv + t) mod MS, kernels.py:581).  So the clauses only mark their bits on the SOURCE
// node in a CTA-local buffer (MB atomics per true clause-node pair, no edge walk), and once per CTA and layer this
// routine walks the graph's edges and ORs the rotated source rows into the destination rows of every target buffer.
// All threads of the CTA, between two CTA barriers; the local buffer is cleared by the caller afterwards.
// `tid` / `nthreads`: the cooperating threads (a CTA by default, or one warp: lane, 32 - then t.all must be null).
__device__ __forceinline__ void flush_messages(const ScatterTargets &t, const GraphView &gv, int MS, int MW, int tid, int nthreads)
{
    // The merge is bound by the atomics that all CTAs send to the same rows: rows of an even number of words go out as
    // 64-bit atomics (half as many).  An item is (source node, word or word pair).
    if (t.all != nullptr) {
        for (int i = tid; i < gv.n * MW; i += nthreads) {
            const int u = i / MW, w = i - u * MW;
            const u32 ty = gv.type[u];
            const u32 v = ty < (u32)kTransposedTypes ? t.all[ty * (MW | 1) + w] : 0u;
            if (v) local_row(t, u, MW)[w] |= v;
        }
        __syncthreads();
        for (int i = tid; i < kTransposedTypes * (MW | 1); i += nthreads) t.all[i] = 0;
    }
    const bool pairs = (MW & 1) == 0;
    const int per_row = pairs ? MW >> 1 : MW;
    const int items = gv.n * per_row;
    constexpr int kInFlight = 4;      // items per thread whose CSR loads are issued together
    for (int i0 = tid; i0 < items; i0 += kInFlight * nthreads) {
        int u[kInFlight], w[kInFlight];
        u32 e0[kInFlight], deg[kInFlight], maxdeg = 0;
#pragma unroll
        for (int q = 0; q < kInFlight; ++q) {
            const int i = i0 + q * nthreads;
            u[q] = i < items ? i / per_row : 0;
            w[q] = (i - u[q] * per_row) << (pairs ? 1 : 0);
            e0[q] = gv.eidx[u[q]] - gv.e_off;
            deg[q] = i < items ? gv.degree[u[q]] : 0u;
        }
#pragma unroll
        for (int q = 0; q < kInFlight; ++q) {
            // a source row without bits sends nothing
            if (deg[q] != 0) {
                const u32 *row = local_row(t, u[q], MW);
                u32 any = 0;
                for (int x = 0; x < MW; ++x) any |= row[x];
                if (any == 0) deg[q] = 0;
            }
            maxdeg = max(maxdeg, deg[q]);
        }
        for (u32 k = 0; k < maxdeg; ++k) {
            u32 dst[kInFlight], ty[kInFlight];
#pragma unroll
            for (int q = 0; q < kInFlight; ++q) {
                const bool row_ok = k < deg[q] && e0[q] + k < gv.e_cnt;
                dst[q] = row_ok ? gv.edge[2 * (size_t)(e0[q] + k)] : ~0u;
                ty[q] = row_ok ? gv.edge[2 * (size_t)(e0[q] + k) + 1] : 0u;
            }
#pragma unroll
            for (int q = 0; q < kInFlight; ++q) {
                if (dst[q] >= (u32)gv.n) continue;                         // no edge in this slot, or a malformed edge: never fault
                const u32 tq = ty[q] >= (u32)MS ? ty[q] % (u32)MS : ty[q];
                const u32 *row = local_row(t, u[q], MW);
                const u32 lo = rotated_word(row, w[q], tq, MS, MW);
                if (pairs) {
                    const u32 hi = rotated_word(row, w[q] + 1, tq, MS, MW);
                    if ((lo | hi) == 0) continue;
                    unsigned long long v = ((unsigned long long)hi << 32) | lo;
                    const size_t at = (size_t)dst[q] * MW + w[q];
                    // own buffer first: what was set there already has been sent to the peers by whoever set it
#pragma unroll
                    for (int r = 0; r < kMaxRanks; ++r)
                        if (r == t.rank) v &= ~atomicOr(reinterpret_cast<unsigned long long *>(t.base[r] + at), v);
                    if (v == 0 || t.world == 1) continue;
#pragma unroll
                    for (int r = 0; r < kMaxRanks; ++r)
                        if (r < t.world && r != t.rank) atomicOr(reinterpret_cast<unsigned long long *>(t.base[r] + at), v);
                } else {
                    if (lo == 0) continue;
                    u32 v = lo;
                    const size_t at = (size_t)dst[q] * MW + w[q];
#pragma unroll
                    for (int r = 0; r < kMaxRanks; ++r)
                        if (r == t.rank) v &= ~atomicOr(t.base[r] + at, v);
                    if (v == 0 || t.world == 1) continue;
#pragma unroll
                    for (int r = 0; r < kMaxRanks; ++r)
                        if (r < t.world && r != t.rank) atomicOr(t.base[r] + at, v);
                }
            }
        }
    }
}

__device__ __forceinline__ void flush_messages(const ScatterTargets &t, const GraphView &gv, int MS, int MW)
{
    flush_messages(t, gv, MS, MW, (int)threadIdx.x, (int)blockDim.x);
}

// Small graphs (at most 32 nodes), learning kernels: instead of walking the edges in every CTA and sending every rotated
// row to the shared destination rows with atomics (flush_messages), a CTA sends only its SOURCE-node marks - one atomic
// per non-empty word (pair) of a node, no edge walk, no answer needed on a single GPU - into the layer's merged-marks
// buffer (the same global rows, node-major, on every rank; a clause-sharded fit sends a peer only the bits that were new
// in its own buffer).  After the grid barrier every CTA reads the merged marks once (n * MW words) and builds the
// destination rows itself, in shared memory (build_message_rows).  All threads of the CTA, between two CTA barriers.
__device__ __forceinline__ void flush_marks(const ScatterTargets &t, const GraphView &gv, int MW)
{
    const int n = gv.n;
    if (t.all != nullptr) {         // marks of clauses that are true on every node of their type: into the nodes' rows first
        for (int i = threadIdx.x; i < n * MW; i += blockDim.x) {
            const int u = i / MW, w = i - u * MW;
            const u32 ty = gv.type[u];
            const u32 v = ty < (u32)kTransposedTypes ? t.all[ty * (MW | 1) + w] : 0u;
            if (v) local_row(t, u, MW)[w] |= v;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < kTransposedTypes * (MW | 1); i += blockDim.x) t.all[i] = 0;
    }
    const bool pairs = (MW & 1) == 0;
    const int per_row = pairs ? MW >> 1 : MW;
    for (int i = threadIdx.x; i < n * per_row; i += blockDim.x) {
        const int u = i / per_row, w = (i - u * per_row) << (pairs ? 1 : 0);
        const u32 *row = local_row(t, u, MW);
        const u32 lo = row[w], hi = pairs ? row[w + 1] : 0u;
        if ((lo | hi) == 0) continue;
        const size_t at = (size_t)u * MW + w;
        if (pairs) {
            unsigned long long v = ((unsigned long long)hi << 32) | lo;
            if (t.world == 1) { atomicOr(reinterpret_cast<unsigned long long *>(t.base[0] + at), v); continue; }
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
                if (r == t.rank) v &= ~atomicOr(reinterpret_cast<unsigned long long *>(t.base[r] + at), v);
            if (v == 0) continue;
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
                if (r < t.world && r != t.rank) atomicOr(reinterpret_cast<unsigned long long *>(t.base[r] + at), v);
        } else {
            u32 v = lo;
            if (t.world == 1) { atomicOr(t.base[0] + at, v); continue; }
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
                if (r == t.rank) v &= ~atomicOr(t.base[r] + at, v);
            if (v == 0) continue;
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
                if (r < t.world && r != t.rank) atomicOr(t.base[r] + at, v);
        }
    }
}

// Destination rows of one layer from its merged source marks: rows[v] = OR over the edges (u -> v, type t) of marks[u]
// rotated up by t ((hv + t) mod MS, kernels.py:581).  `marks` = the layer's merged-marks rows in global memory (complete:
// call after the grid barrier), `tmp` = a CTA buffer of n rows with stride MW | 1 (the local marks buffer, which is left
// cleared for the next layer), `rows` = [32][MW] in shared memory.  All threads of the CTA; ends with a CTA barrier.
__device__ __forceinline__ void build_message_rows(const u32 *marks, u32 *tmp, u32 *rows, const GraphView &gv, int MS, int MW)
{
    const int n = gv.n, stride = MW | 1;
    for (int i = threadIdx.x; i < n * MW; i += blockDim.x) {
        const int u = i / MW, w = i - u * MW;
        tmp[u * stride + w] = __ldcg(marks + i);
        rows[i] = 0;
    }
    __syncthreads();
    const bool pairs = (MW & 1) == 0;
    const int per_row = pairs ? MW >> 1 : MW;
    for (int i = threadIdx.x; i < n * per_row; i += blockDim.x) {
        const int u = i / per_row, w = (i - u * per_row) << (pairs ? 1 : 0);
        const u32 *row = tmp + u * stride;
        const u32 e0 = gv.eidx[u] - gv.e_off, deg = gv.degree[u];
        for (u32 k = 0; k < deg && e0 + k < gv.e_cnt; ++k) {
            const u32 dst = gv.edge[2 * (size_t)(e0 + k)], ty = gv.edge[2 * (size_t)(e0 + k) + 1];
            if (dst >= (u32)n) continue;                               // malformed edge: ignore, never fault
            const u32 tq = ty >= (u32)MS ? ty % (u32)MS : ty;
            const u32 lo = rotated_word(row, w, tq, MS, MW);
            if (lo) atomicOr(rows + (size_t)dst * MW + w, lo);
            if (pairs) {
                const u32 hi = rotated_word(row, w + 1, tq, MS, MW);
                if (hi) atomicOr(rows + (size_t)dst * MW + w + 1, hi);
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n * MW; i += blockDim.x) tmp[(i / MW) * stride + (i % MW)] = 0;
    __syncthreads();
}

// Destination rows of a larger graph from the layer's merged marks, the work shared by the CTAs of the rank: CTA b
// takes the source nodes b, b + gridDim.x, ... and ORs their rotated marks into the destination rows `out` (global,
// node-major, stride MW, zero before the pass) with atomics that need no answer - n * degree * MW / 2 atomics per layer
// for the whole rank.  `marks` = the layer's merged-marks rows (complete: call after the grid barrier); a rank-local
// barrier has to follow before `out` is read.  All threads of the CTA.
__device__ __forceinline__ void scatter_message_rows_share(const u32 *marks, u32 *out, const GraphView &gv, int MS, int MW)
{
    const int n = gv.n;
    const bool pairs = (MW & 1) == 0;
    const int per_row = pairs ? MW >> 1 : MW;
    const int mine = ((int)blockIdx.x < n) ? (n - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;     // source nodes of this CTA
    for (int i = threadIdx.x; i < mine * per_row; i += blockDim.x) {
        const int u = (int)blockIdx.x + (i / per_row) * (int)gridDim.x, w = (i % per_row) << (pairs ? 1 : 0);
        const u32 *row = marks + (size_t)u * MW;
        const u32 e0 = gv.eidx[u] - gv.e_off, deg = gv.degree[u];
        for (u32 k = 0; k < deg && e0 + k < gv.e_cnt; ++k) {
            const u32 dst = gv.edge[2 * (size_t)(e0 + k)], ty = gv.edge[2 * (size_t)(e0 + k) + 1];
            if (dst >= (u32)n) continue;                               // malformed edge: ignore, never fault
            const u32 tq = ty >= (u32)MS ? ty % (u32)MS : ty;
            u32 lo, hi = 0;
            if ((MS & 31) == 0) {                                       // two or three words of the source row, read past L1
                const u32 start = (u32)(32 * w + MS - (int)tq);
                const u32 s0 = start >= (u32)MS ? start - (u32)MS : start;
                const int i0 = (int)(s0 >> 5), sh = (int)(s0 & 31);
                const int i1 = i0 + 1 < MW ? i0 + 1 : 0, i2 = i1 + 1 < MW ? i1 + 1 : 0;
                const u32 a0 = __ldcg(row + i0), a1 = __ldcg(row + i1);
                lo = __funnelshift_r(a0, a1, sh);
                if (pairs) hi = __funnelshift_r(a1, __ldcg(row + i2), sh);
            } else {
                lo = rotated_word(row, w, tq, MS, MW);
                if (pairs) hi = rotated_word(row, w + 1, tq, MS, MW);
            }
            if (pairs) {
                if (lo | hi) atomicOr(reinterpret_cast<unsigned long long *>(out + (size_t)dst * MW + w), ((unsigned long long)hi << 32) | lo);
            } else if (lo) {
                atomicOr(out + (size_t)dst * MW + w, lo);
            }
        }
    }
}

// In-register transpose of a 32x32 bit matrix: on return bit i of a[b] is what bit b of a[i] was.
__device__ __forceinline__ void transpose32(u32 (&a)[32])
{
    u32 mask = 0x0000ffffu;
#pragma unroll
    for (int j = 16; j != 0; j >>= 1, mask ^= mask << j) {
#pragma unroll
        for (int k = 0; k < 32; k = (k + j + 1) & ~j) {
            const u32 t = ((a[k] >> j) ^ a[k + j]) & mask;
            a[k] ^= t << j;
            a[k + j] ^= t;
        }
    }
}

// ------------------------------------------------------------------------------ transposed evaluation (large graphs)
// For graphs of 33..1024 nodes a CTA keeps the graph's literal rows TRANSPOSED in shared memory: row(l) holds, for
// literal l, one bit per node (word j = nodes 32j..32j+31).  A warp then evaluates a clause on ALL nodes at once, lane j
// owning node word j: r = type/valid mask; for every included literal l: r &= row(l) - one conflict-free shared load per
// included literal, instead of one pass over the include words per node word.  Layers >= 1 do the same on the
// transposed positive message bits (a negated message literal ANDs the complement).
// Storage: literal l = 32w + b lives at T[((b * W) + w) * S + j] with S odd (>= node words), so that the threads that
// build it (adjacent w) and the lanes that read it (adjacent j) are both conflict-free.
struct TransposedGraph {
    u32 *T;        // [32 * Wmax][S] literal rows of the current layer (layer 0: literals, layer d: positive message bits)
    u32 *TM;       // [n_types][S] nodes of each type (valid nodes only)
    int S;         // row stride in words (odd)
    int words;     // node words of the current graph (<= 32)
};

// All threads of the CTA: rows[v][0..W) of nodes v < n (row stride `stride` words) -> T.
__device__ __forceinline__ void build_transposed(const u32 *rows, int n, int W, int stride, const TransposedGraph &tg)
{
    const int blocks = tg.words * W;
    for (int blk = threadIdx.x; blk < blocks; blk += blockDim.x) {
        const int j = blk / W, w = blk - j * W;
        u32 r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int v = 32 * j + i;
            r[i] = v < n ? rows[(size_t)v * stride + w] : 0u;
        }
        transpose32(r);
#pragma unroll
        for (int b = 0; b < 32; ++b) tg.T[(size_t)(b * W + w) * tg.S + j] = r[b];
    }
}

// All threads of the CTA: node-type masks of the graph (types 0..n_types-1).
__device__ __forceinline__ void build_type_masks(const u32 *type, int n, int n_types, const TransposedGraph &tg)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int j = warp; j < tg.words; j += nwarps) {
        const int v = 32 * j + lane;
        const u32 ty = v < n ? type[v] : ~0u;
        for (int t = 0; t < n_types; ++t) {
            const u32 col = __ballot_sync(kFull, ty == (u32)t);
            if (lane == 0) tg.TM[(size_t)t * tg.S + j] = col;
        }
    }
}

template <int N>
__device__ __forceinline__ bool any_of(const bool (&f)[N])
{
    bool r = false;
#pragma unroll
    for (int i = 0; i < N; ++i) r = r || f[i];
    return r;
}

// Include words of a clause layer as eval_clause_layer holds them: word w0 + lane in lanes, layers of at most 64 words in
// two registers (cached), wider ones reloaded per 32 words.
struct IncludeWords {
    const u32 *inc;
    u32 a, b, last_mask;
    bool cached;
};

// kBatch consecutive node words (from j0) of one clause layer, with independent state so that the loads of the batch
// (node types, rows) are in flight together: a warp's evaluation is a chain of dependent memory latencies otherwise.
// Returns the OR of the node-output words written.
template <int kBatch>
__device__ __forceinline__ u32 eval_node_words(const DevModel &m, const GraphView &gv, const ClauseView &cv, int d, int W,
                                               const IncludeWords &iw_all, u32 my_type, int j0, int words, const u32 *prev,
                                               u32 *out, const u32 *Pread, const ScatterTargets *scatter, int lane)
{
    const int n = gv.n;
    const bool wide = d == 0 && (W & 3) == 0;     // literal rows are 16-byte aligned: 128-bit loads
    const bool cached = iw_all.cached;
    const u32 inc_a = iw_all.a, inc_b = iw_all.b, last_mask = iw_all.last_mask;
    const u32 *inc = iw_all.inc;
    u32 any = 0;
    {
        bool ok[kBatch];
        const u32 *row[kBatch];
#pragma unroll
        for (int q = 0; q < kBatch; ++q) {
            const int j = j0 + q, v = j * 32 + lane;
            ok[q] = j < words && v < n;
            if (d > 0 && j < words) ok[q] = ok[q] && ((prev[j] >> lane) & 1u);
        }
#pragma unroll
        for (int q = 0; q < kBatch; ++q) {
            const int v = (j0 + q) * 32 + lane;
            const u32 ty = ok[q] ? gv.type[v] : ~0u;
            ok[q] = ok[q] && ty == my_type;
            const int vv = ok[q] ? v : 0;
            row[q] = d == 0 ? gv.X + (size_t)vv * W : Pread + (size_t)vv * m.MW;
        }
        bool alive = __any_sync(kFull, any_of<kBatch>(ok));
        for (int w0 = 0; w0 < W && alive; w0 += 32) {
            u32 iw_l;
            if (cached) iw_l = w0 == 0 ? inc_a : inc_b;
            else iw_l = w0 + lane < W ? inc[w0 + lane] & (w0 + lane == W - 1 ? last_mask : kFull) : 0u;
            u32 nz = __ballot_sync(kFull, iw_l != 0);
            if (wide) {
                nz = (nz | (nz >> 1) | (nz >> 2) | (nz >> 3)) & 0x11111111u;      // groups of four words with an included literal
                while (nz) {
                    const int b = __ffs(nz) - 1;
                    nz &= nz - 1;
                    const u32 i0 = __shfl_sync(kFull, iw_l, b), i1 = __shfl_sync(kFull, iw_l, b + 1),
                              i2 = __shfl_sync(kFull, iw_l, b + 2), i3 = __shfl_sync(kFull, iw_l, b + 3);
                    uint4 x[kBatch];
#pragma unroll
                    for (int q = 0; q < kBatch; ++q)
                        x[q] = ok[q] ? reinterpret_cast<const uint4 *>(row[q])[(w0 + b) >> 2] : make_uint4(kFull, kFull, kFull, kFull);
#pragma unroll
                    for (int q = 0; q < kBatch; ++q)
                        ok[q] = ok[q] && (((i0 & ~x[q].x) | (i1 & ~x[q].y) | (i2 & ~x[q].z) | (i3 & ~x[q].w)) == 0);
                    if (!__any_sync(kFull, any_of<kBatch>(ok))) { alive = false; break; }   // warp-ballot early exit
                }
            } else {
                while (nz) {
                    const int b = __ffs(nz) - 1;
                    nz &= nz - 1;
                    const u32 iw = __shfl_sync(kFull, iw_l, b);
                    u32 x[kBatch];
#pragma unroll
                    for (int q = 0; q < kBatch; ++q)
                        x[q] = !ok[q] ? kFull : d == 0 ? row[q][w0 + b] : msg_word(row[q], w0 + b, m.MS, m.MW);
#pragma unroll
                    for (int q = 0; q < kBatch; ++q) ok[q] = ok[q] && ((iw & ~x[q]) == 0);
                    if (!__any_sync(kFull, any_of<kBatch>(ok))) { alive = false; break; }
                }
            }
        }
#pragma unroll
        for (int q = 0; q < kBatch; ++q) {
            const int j = j0 + q, v = j * 32 + lane;
            if (j >= words) break;
            const u32 word = __ballot_sync(kFull, ok[q]);
            if (lane == 0) out[j] = word;
            any |= word;
            if (scatter && ok[q]) {
                if (scatter->local) {
                    // mark the clause's hypervector bits on this (source) node; most are there already
                    for (int b = 0; b < m.MB; ++b) {
                        u32 bit = cv.hv[b];
                        if (bit >= (u32)m.MS) bit %= (u32)m.MS;
                        u32 *addr = local_row(*scatter, v, m.MW) + (bit >> 5);
                        const u32 mbit = 1u << (bit & 31);
                        if (!(*(volatile u32 *)addr & mbit)) atomicOr(addr, mbit);
                    }
                } else {
                    const u32 e0 = gv.eidx[v] - gv.e_off, deg = gv.degree[v];
                    for (u32 k = 0; k < deg && e0 + k < gv.e_cnt; ++k) {
                        const u32 dst = gv.edge[2 * (size_t)(e0 + k)], t = gv.edge[2 * (size_t)(e0 + k) + 1];
                        if (dst >= (u32)n) continue;                              // malformed edge: ignore, never fault
                        for (int b = 0; b < m.MB; ++b) {
                            u32 bit = cv.hv[b] + t;                               // (hv + edge type) mod MS without a 64-bit division
                            if (bit >= (u32)m.MS || bit < t) bit = (u32)(((u64)cv.hv[b] + t) % (u32)m.MS);
                            const u32 mbit = 1u << (bit & 31);
#pragma unroll
                            for (int r = 0; r < kMaxRanks; ++r)     // constant indices keep the pointers in registers
                                if (r < scatter->world) atomicOr(scatter->base[r] + (size_t)dst * m.MW + (bit >> 5), mbit);
                        }
                    }
                }
            }
        }
    }
    return any;
}

// eval_clause_layer for a graph of at most 32 nodes, with the lanes spread over the layer's include WORDS instead of
// over nodes: per candidate node (a node of the clause's type that was true in the layer below) every lane loads its
// words of the node's row - one coalesced load per 32 words - tests (include & ~row) and the warp votes.  A small
// graph has few candidates and every one costs W/32 loads, where the node-parallel form walks the include words one
// after the other in a chain of dependent loads.  Four candidates are in flight at a time.  Same results: node-output
// word in out[0], include count, messages through `scatter`.
__device__ __forceinline__ u32 eval_clause_layer_small(const DevModel &m, const GraphView &gv, int n_types, const ClauseView &cv,
                                                       int c, int d, const u32 *prev, u32 *out, const u32 *Pread,
                                                       const ScatterTargets *scatter, int lane)
{
    const int n = gv.n;
    const int W = d == 0 ? m.L0 : m.M;
    const u32 *inc = cv.ta(d) + (size_t)(m.SB - 1) * W;
    const u32 last_mask = d == 0 ? m.lit_mask : m.msg_mask;
    const u32 my_type = (u32)(c % n_types);
    const bool candidate = lane < n && gv.type[lane] == my_type && (d == 0 || ((prev[0] >> lane) & 1u));
    u32 cand = __ballot_sync(kFull, candidate);
    const bool fast_msg = (m.MS & 31) == 0;
    auto row_word = [&](int v, int w) -> u32 {          // word w of node v's literal vector of this layer
        if (d == 0) return gv.X[(size_t)v * W + w];
        const u32 *prow = Pread + (size_t)v * m.MW;
        if (fast_msg) return w < m.MW ? prow[w] : ~prow[w - m.MW];
        return msg_word(prow, w, m.MS, m.MW);
    };
    int cnt = 0;
    u32 result = 0;
    for (int w0 = 0; w0 < W; w0 += 128) {               // include words in registers, 128 words (4 per lane) at a time
        u32 iw[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int w = w0 + 32 * q + lane;
            iw[q] = w < W ? inc[w] & (w == W - 1 ? last_mask : kFull) : 0u;
            cnt += __popc(iw[q]);
        }
        u32 todo = cand, still = 0;                      // candidates that pass this stretch of words
        while (todo) {
            int v[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                v[t] = todo ? __ffs(todo) - 1 : -1;
                todo &= todo - 1;
            }
            bool fail[4] = {false, false, false, false};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int w = w0 + 32 * q + lane;
                if (w0 + 32 * q < W) {                   // warp-uniform
#pragma unroll
                    for (int t = 0; t < 4; ++t)
                        if (v[t] >= 0 && w < W) fail[t] = fail[t] || (iw[q] & ~row_word(v[t], w)) != 0;
                }
            }
#pragma unroll
            for (int t = 0; t < 4; ++t)
                if (v[t] >= 0 && !__any_sync(kFull, fail[t])) still |= 1u << v[t];
        }
        cand = still;
    }
    result = cand;
    cnt = __reduce_add_sync(kFull, cnt);
    if (lane == 0) {
        *cv.n_inc = (d == 0 ? 0 : *cv.n_inc) + cnt;
        out[0] = result;
    }
    if (scatter && ((result >> lane) & 1u)) {
        const int v = lane;
        if (scatter->local) {
            // mark the clause's hypervector bits on this (source) node; most are there already
            for (int b = 0; b < m.MB; ++b) {
                u32 bit = cv.hv[b];
                if (bit >= (u32)m.MS) bit %= (u32)m.MS;
                u32 *addr = local_row(*scatter, v, m.MW) + (bit >> 5);
                const u32 mbit = 1u << (bit & 31);
                if (!(*(volatile u32 *)addr & mbit)) atomicOr(addr, mbit);
            }
        } else {
            const u32 e0 = gv.eidx[v] - gv.e_off, deg = gv.degree[v];
            for (u32 k = 0; k < deg && e0 + k < gv.e_cnt; ++k) {
                const u32 dst = gv.edge[2 * (size_t)(e0 + k)], t = gv.edge[2 * (size_t)(e0 + k) + 1];
                if (dst >= (u32)n) continue;                              // malformed edge: ignore, never fault
                for (int b = 0; b < m.MB; ++b) {
                    u32 bit = cv.hv[b] + t;                               // (hv + edge type) mod MS without a 64-bit division
                    if (bit >= (u32)m.MS || bit < t) bit = (u32)(((u64)cv.hv[b] + t) % (u32)m.MS);
                    const u32 mbit = 1u << (bit & 31);
#pragma unroll
                    for (int r = 0; r < kMaxRanks; ++r)
                        if (r < scatter->world) atomicOr(scatter->base[r] + (size_t)dst * m.MW + (bit >> 5), mbit);
                }
            }
        }
    }
    return result;
}

// One warp evaluates a clause at layer `d` over all nodes of a graph (lanes = the 32 nodes of a node word) and
// writes the node-output words out[0..ceil(n/32)).  Layer 0 tests the node's literal row, layer d >= 1 the node's
// message row ANDed with the node's bit of layer d-1 in `prev` (kernels.py:407-530).  Returns the OR of the words
// written (warp-uniform).  When `scatter` is given, every true node sends the clause's hypervector bits along
// its out-edges into every target buffer (kernels.py:549-590): bit (hv[c][b] + edge type) mod MS of the destination node.
// kBatchNodes: node words are also taken four at a time (graph sets with more than 32 nodes per graph); without it the
// code for single node words is all there is, which keeps small-graph kernels lean.
template <bool kBatchNodes>
__device__ __forceinline__ u32 eval_clause_layer(const DevModel &m, const GraphView &gv, int n_types, const ClauseView &cv,
                                                 int c, int d, const u32 *prev, u32 *out, const u32 *Pread,
                                                 const ScatterTargets *scatter, int lane)
{
    const int n = gv.n;
    if (!kBatchNodes && n <= 32) return eval_clause_layer_small(m, gv, n_types, cv, c, d, prev, out, Pread, scatter, lane);
    const int W = d == 0 ? m.L0 : m.M;
    const u32 *inc = cv.ta(d) + (size_t)(m.SB - 1) * W;
    const u32 last_mask = d == 0 ? m.lit_mask : m.msg_mask;
    const u32 my_type = (u32)(c % n_types);

    // The layer's include words sit in lanes (word w0 + lane), fetched with one coalesced load per 32 words; layers of
    // at most 64 words keep them in registers for all node words.  Only words with included literals are visited.
    const bool cached = W <= 64;
    u32 inc_a = 0, inc_b = 0;
    if (cached) {
        if (lane < W) inc_a = inc[lane] & (lane == W - 1 ? last_mask : kFull);
        if (32 + lane < W) inc_b = inc[32 + lane] & (32 + lane == W - 1 ? last_mask : kFull);
    }

    // include count of this layer (kernels.py:251-277)
    int cnt = 0;
    if (cached) cnt = __popc(inc_a) + __popc(inc_b);
    else for (int w = lane; w < W; w += 32) cnt += __popc(inc[w] & (w == W - 1 ? last_mask : kFull));
    cnt = __reduce_add_sync(kFull, cnt);
    if (lane == 0) *cv.n_inc = (d == 0 ? 0 : *cv.n_inc) + cnt;

    const int words = (n + 31) >> 5;
    IncludeWords iw_all;
    iw_all.inc = inc; iw_all.a = inc_a; iw_all.b = inc_b; iw_all.last_mask = last_mask; iw_all.cached = cached;
    u32 any = 0;
    int j0 = 0;
    // batches of four node words while more than one is left (large graphs), single words otherwise
    if (kBatchNodes)
        for (; words - j0 > 1; j0 += 4)
            any |= eval_node_words<4>(m, gv, cv, d, W, iw_all, my_type, j0, words, prev, out, Pread, scatter, lane);
    for (; j0 < words; ++j0)
        any |= eval_node_words<1>(m, gv, cv, d, W, iw_all, my_type, j0, words, prev, out, Pread, scatter, lane);
    return any;
}

// eval_clause_layer on a transposed graph: lane j owns node word j (graphs of at most 1024 nodes).  Same results:
// node-output words in out[], include count, OR of the words returned, messages through `scatter`.
__device__ __forceinline__ u32 eval_clause_layer_transposed(const DevModel &m, const GraphView &gv, int n_types,
                                                            const ClauseView &cv, int c, int d, const u32 *prev, u32 *out,
                                                            const TransposedGraph &tg, const ScatterTargets *scatter, int lane)
{
    const int n = gv.n;
    const int W = d == 0 ? m.L0 : m.M;
    const int WT = d == 0 ? m.L0 : m.MW;                 // words per transposed source row
    const u32 *inc = cv.ta(d) + (size_t)(m.SB - 1) * W;
    const u32 last_mask = d == 0 ? m.lit_mask : m.msg_mask;

    // lanes past the graph's last node word keep r == 0; they read column 0 so that no load leaves the buffer
    const int col = lane < tg.words ? lane : 0;
    u32 r = lane < tg.words ? tg.TM[(size_t)(c % n_types) * tg.S + lane] : 0u;
    if (d > 0 && lane < tg.words) r &= prev[lane];
    int cnt = 0;
    bool alive = __any_sync(kFull, r != 0);
    for (int w0 = 0; w0 < W; w0 += 32) {
        const u32 iw_l = w0 + lane < W ? inc[w0 + lane] & (w0 + lane == W - 1 ? last_mask : kFull) : 0u;
        cnt += __popc(iw_l);
        if (!alive) continue;
        u32 nz = __ballot_sync(kFull, iw_l != 0);
        while (nz && alive) {
            const int bw = __ffs(nz) - 1;
            nz &= nz - 1;
            u32 iw = __shfl_sync(kFull, iw_l, bw);
            const int w = w0 + bw;
            // up to four included literals per step, their loads issued together
            if (d == 0 || (m.MS & 31) == 0) {
                // The 32 literals of an include word sit WT * S words apart in T, and a message word is all positive bits
                // (w < MW) or all complements: one multiply-add and one load per included literal, the rows of a
                // complement word are ORed and taken out of r at the end.
                const bool neg = d > 0 && w >= m.MW;
                const u32 *base = tg.T + (size_t)(neg ? w - m.MW : w) * tg.S + col;
                const int step = WT * tg.S;
                u32 acc = neg ? 0u : kFull;
                while (iw) {
                    u32 x0, x1, x2, x3;
                    x0 = base[(__ffs(iw) - 1) * step]; iw &= iw - 1;
                    x1 = x0; x2 = x0; x3 = x0;
                    if (iw) { x1 = base[(__ffs(iw) - 1) * step]; iw &= iw - 1; }
                    if (iw) { x2 = base[(__ffs(iw) - 1) * step]; iw &= iw - 1; }
                    if (iw) { x3 = base[(__ffs(iw) - 1) * step]; iw &= iw - 1; }
                    acc = neg ? acc | ((x0 | x1) | (x2 | x3)) : acc & ((x0 & x1) & (x2 & x3));
                }
                r &= neg ? ~acc : acc;
            } else {
                auto literal_row = [&](int b) -> u32 {
                    const int l = 32 * w + b;                                   // message literal: positive bits, then their complements
                    const int p = l < m.MS ? l : l - m.MS;
                    const u32 x = tg.T[(size_t)((p & 31) * WT + (p >> 5)) * tg.S + col];
                    return l < m.MS ? x : ~x;
                };
                while (iw) {
                    u32 x0, x1 = kFull, x2 = kFull, x3 = kFull;
                    x0 = literal_row(__ffs(iw) - 1); iw &= iw - 1;
                    if (iw) { x1 = literal_row(__ffs(iw) - 1); iw &= iw - 1; }
                    if (iw) { x2 = literal_row(__ffs(iw) - 1); iw &= iw - 1; }
                    if (iw) { x3 = literal_row(__ffs(iw) - 1); iw &= iw - 1; }
                    r &= (x0 & x1) & (x2 & x3);
                }
            }
            alive = __any_sync(kFull, r != 0);
        }
    }
    cnt = __reduce_add_sync(kFull, cnt);
    if (lane == 0) *cv.n_inc = (d == 0 ? 0 : *cv.n_inc) + cnt;
    if (lane >= tg.words) r = 0;                                             // lanes past the graph read nothing valid
    else if (d > 0) r &= tg.TM[(size_t)(c % n_types) * tg.S + lane];         // complements set bits of missing nodes
    if (lane < tg.words) out[lane] = r;
    const u32 any = __ballot_sync(kFull, r != 0);
    if (scatter && scatter->all != nullptr && any != 0 &&
        __all_sync(kFull, lane >= tg.words || r == tg.TM[(size_t)(c % n_types) * tg.S + col])) {
        // true on every node of its type: one mark per hypervector bit for the whole type
        if (lane < m.MB) {
            u32 bit = cv.hv[lane];
            if (bit >= (u32)m.MS) bit %= (u32)m.MS;
            atomicOr(scatter->all + (size_t)(c % n_types) * (m.MW | 1) + (bit >> 5), 1u << (bit & 31));
        }
        return any;
    }
    if (scatter && r) {
        u32 bits = r;
        while (bits) {
            const int i = __ffs(bits) - 1;
            bits &= bits - 1;
            const int v = 32 * lane + i;
            if (scatter->local) {
                for (int b = 0; b < m.MB; ++b) {
                    u32 bit = cv.hv[b];
                    if (bit >= (u32)m.MS) bit %= (u32)m.MS;
                    u32 *addr = local_row(*scatter, v, m.MW) + (bit >> 5);
                    const u32 mbit = 1u << (bit & 31);
                    if (!(*(volatile u32 *)addr & mbit)) atomicOr(addr, mbit);
                }
            } else {
                const u32 e0 = gv.eidx[v] - gv.e_off, deg = gv.degree[v];
                for (u32 k = 0; k < deg && e0 + k < gv.e_cnt; ++k) {
                    const u32 dst = gv.edge[2 * (size_t)(e0 + k)], t = gv.edge[2 * (size_t)(e0 + k) + 1];
                    if (dst >= (u32)n) continue;
                    for (int b = 0; b < m.MB; ++b) {
                        u32 bit = cv.hv[b] + t;
                        if (bit >= (u32)m.MS || bit < t) bit = (u32)(((u64)cv.hv[b] + t) % (u32)m.MS);
                        const u32 mbit = 1u << (bit & 31);
#pragma unroll
                        for (int rk = 0; rk < kMaxRanks; ++rk)
                            if (rk < scatter->world) atomicOr(scatter->base[rk] + (size_t)dst * m.MW + (bit >> 5), mbit);
                    }
                }
            }
        }
    }
    return any;
}

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

// ------------------------------------------------------------------------------------- bit-sliced automata
// +1 / -1 with saturation on the automata flagged in `active`; p[b] is plane b of one 32-automaton word
// (kernels.py:55-96).  MAXSB is a compile-time bound so that the planes stay in registers.
// Planes of up to 8 state bits stay in registers (loops fully unrolled, predicated on b < SB); wider automata
// take run-time loops over an indexed array (rare, slower, keeps the code small).
template <int MAXSB>
__device__ __forceinline__ int plane_bound(int SB) { return MAXSB <= 8 ? MAXSB : SB; }

template <int MAXSB>
__device__ __forceinline__ void automata_inc(u32 (&p)[MAXSB], int SB, u32 active)
{
    u32 carry = active;
#pragma unroll
    for (int b = 0; b < plane_bound<MAXSB>(SB); ++b)
        if (b < SB) { const u32 nx = p[b] & carry; p[b] ^= carry; carry = nx; }
#pragma unroll
    for (int b = 0; b < plane_bound<MAXSB>(SB); ++b)
        if (b < SB) p[b] |= carry;
}

template <int MAXSB>
__device__ __forceinline__ void automata_dec(u32 (&p)[MAXSB], int SB, u32 active)
{
    u32 borrow = active;
#pragma unroll
    for (int b = 0; b < plane_bound<MAXSB>(SB); ++b)
        if (b < SB) { const u32 nx = ~p[b] & borrow; p[b] ^= borrow; borrow = nx; }
#pragma unroll
    for (int b = 0; b < plane_bound<MAXSB>(SB); ++b)
        if (b < SB) p[b] &= ~borrow;
}

}  // namespace gtm
