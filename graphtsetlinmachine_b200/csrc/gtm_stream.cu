// Node-stream scoring: the fast path of batched inference for depth-1 models.
//
// Idea.  Layer-0 clause evaluation is a per-node test, so a graph set is one long stream of nodes.  A CTA
// takes a TILE of consecutive graphs (at most TN = 32*TNC nodes), turns the tile's literal rows into the
// transposed form XT[literal][node word] (bit i of word j = literal of node 32j+i) in shared memory, and then
// evaluates a clause on 32 nodes per AND: r = AND over the clause's INCLUDED literals of XT[literal][j].
// That is popcount(include) word operations per 32 nodes instead of 32*ceil(literals/32) for the row-wise
// test, and an empty clause costs nothing (and is true, as in kernels.py:443-460).  Included literals come
// from per-clause lists rebuilt from the include planes whenever the automata changed.
//
// A thread evaluates one clause on FOUR node words at a time (one 128-bit shared load per literal), and the
// literal lists hold byte offsets of the rows (literal * TNC * 4), so a literal costs a shift/mask, an add, a load
// and two 3-input ANDs for 128 nodes.
//
// Votes.  Clauses are processed in blocks of CB = 128.  Their node bits R[clause][node word] are transposed in
// registers (32x32 bit-matrix butterflies, one per thread) into RT[clause word][node] = the 32 clause outcomes of a
// node, and then one thread per graph ORs the words of its nodes and walks only the SET bits, adding the weight
// rows of the clauses that fired (kernels.py:279-317, batched).  Work is proportional to the clauses that fire
// instead of to all clauses.  Class sums stay in registers and leave the CTA once per graph, unclamped.
//
// Derived model data (StreamModel): literal lists (uint16 row offsets, padded to a multiple of 4 with the offset
// of an all-ones row) and weights transposed to [clause][KROW].
#include "../../include/gtm_b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <climits>
#include <vector>

#include "gtm_stream.h"

namespace gtm {

constexpr int kStreamThreads = 512;
constexpr int kStreamCB = 128;          // clauses per vote block
constexpr int kStreamMaxK = 16;

// ------------------------------------------------------------------------------------------- list building
__global__ void stream_count_kernel(DevModel m, int *cnt)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= m.C) return;
    const u32 *inc = m.ta0 + ((size_t)c * m.SB + (m.SB - 1)) * m.L0;
    int n = 0;
    for (int w = 0; w < m.L0; ++w) n += __popc(inc[w] & (w == m.L0 - 1 ? m.lit_mask : kFull));
    cnt[c] = (n + 3) & ~3;
}

__global__ void stream_scan_kernel(const int *cnt, int *off, int C)
{
    __shared__ int s_part[1024];
    const int per = (C + blockDim.x - 1) / blockDim.x;
    const int lo = min(C, (int)threadIdx.x * per), hi = min(C, lo + per);
    int sum = 0;
    for (int i = lo; i < hi; ++i) sum += cnt[i];
    s_part[threadIdx.x] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int t = 0; t < (int)blockDim.x; ++t) { const int v = s_part[t]; s_part[t] = run; run += v; }
        off[C] = run;
    }
    __syncthreads();
    int run = s_part[threadIdx.x];
    for (int i = lo; i < hi; ++i) { off[i] = run; run += cnt[i]; }
}

__global__ void stream_fill_kernel(DevModel m, const int *off, unsigned short *list, int *Wt, int KROW, int TNC)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= m.C) return;
    const u32 *inc = m.ta0 + ((size_t)c * m.SB + (m.SB - 1)) * m.L0;
    int at = off[c];
    for (int w = 0; w < m.L0; ++w) {
        u32 bits = inc[w] & (w == m.L0 - 1 ? m.lit_mask : kFull);
        while (bits) {
            const int b = __ffs(bits) - 1;
            bits &= bits - 1;
            list[at++] = (unsigned short)((w * 32 + b) * TNC * 4);
        }
    }
    while (at < off[c + 1]) list[at++] = (unsigned short)(m.literals * TNC * 4);   // sentinel: the all-ones row
    for (int k = 0; k < KROW; ++k) Wt[(size_t)c * KROW + k] = k < m.K ? m.weights[(size_t)k * m.C + c] : 0;
}

// -------------------------------------------------------------------------------------------------- scoring
struct StreamArgs {
    const int *tile_graph;              // first graph of every tile, or NULL: every tile holds graphs_per_tile graphs
    int graphs_per_tile;
    int tile_lo, tile_hi;               // tiles [tile_lo, tile_hi)
    int64_t first, count;               // graphs written: [first, first+count)
    int64_t n_graphs, total_nodes;
    int *class_sums;                    // [count][K]
    unsigned *tile_counter;             // dynamic tile scheduler (zeroed before launch)
    int TNC;
    const int *lit_off;
    const unsigned short *lit_list;
    const int *Wt;
    int KROW;
};

__device__ __forceinline__ uint4 lds128(unsigned addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

constexpr int kWarpVoteGraphs = 64;   // tiles of at most this many (multi-node) graphs vote warp-wise, see below
constexpr int kRTStride = 33;   // RT[cw][b * 33 + j] holds node 32j+b: conflict-free both for the writer (lanes = j) and the reader (lanes = b)

template <int KP>
__global__ void __launch_bounds__(kStreamThreads, 2) stream_score_kernel(DevModel m, DevGraphs g, StreamArgs a)
{
    extern __shared__ __align__(16) u32 s_dyn[];
    constexpr int CW = kStreamCB / 32;                 // clause words per block
    const int TNC = a.TNC, Q = TNC >> 2;               // node words per tile, 4-word groups
    u32 *XT = s_dyn;                                   // [literals+1][TNC]
    u32 *TMV = XT + (size_t)(m.literals + 1) * TNC;    // [n_types][TNC] valid & node type
    u32 *R = TMV + (size_t)g.n_types * TNC;            // [CB][TNC]        node bits per clause
    u32 *RT = R + (size_t)kStreamCB * TNC;             // [CW][32*33]      clause bits per node
    int *Wb = (int *)(RT + (size_t)CW * 32 * kRTStride);   // [CB][KROW]
    __shared__ int s_tile;
    __shared__ int s_vsum[kWarpVoteGraphs * KP];      // class sums of the tile's graphs when they are voted warp-wise
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = kStreamThreads / 32;
    const int KROW = a.KROW;
    const unsigned xt32 = (unsigned)__cvta_generic_to_shared(XT);

    while (true) {
        if (tid == 0) s_tile = a.tile_lo + (int)atomicAdd(a.tile_counter, 1u);
        __syncthreads();
        const int tile = s_tile;
        if (tile >= a.tile_hi) break;
        const int g0 = a.tile_graph ? a.tile_graph[tile] : (int)min((int64_t)tile * a.graphs_per_tile, a.n_graphs);
        const int g1 = a.tile_graph ? a.tile_graph[tile + 1] : (int)min((int64_t)(tile + 1) * a.graphs_per_tile, a.n_graphs);
        const int node0 = (int)g.node_index[g0];
        const int node1 = g1 < a.n_graphs ? (int)g.node_index[g1] : (int)a.total_nodes;
        const int nn = node1 - node0;

        // ---- transpose the tile's literal rows: XT[32w+b][j] = ballot over the 32 nodes of word j ----
        for (int jw = warp; jw < TNC * m.L0; jw += nwarps) {
            const int j = jw / m.L0, w = jw % m.L0;
            const int v = j * 32 + lane;
            u32 x = v < nn ? g.X[(size_t)(node0 + v) * m.L0 + w] : 0u;
            const int nbits = min(32, m.literals - 32 * w);
            for (int b = 0; b < nbits; ++b) {
                const u32 col = __ballot_sync(kFull, (x >> b) & 1u);
                if (lane == (b & 31)) XT[(size_t)(32 * w + b) * TNC + j] = col;
            }
        }
        for (int j = tid; j < TNC; j += kStreamThreads) XT[(size_t)m.literals * TNC + j] = kFull;
        for (int tj = warp; tj < g.n_types * TNC; tj += nwarps) {
            const int t = tj / TNC, j = tj % TNC;
            const int v = j * 32 + lane;
            const bool ok = v < nn && g.node_type[node0 + (v < nn ? v : 0)] == (u32)t;
            const u32 col = __ballot_sync(kFull, ok);
            if (lane == 0) TMV[tj] = col;
        }

        // Tiles of a few large graphs (e.g. 361-node images, two per tile) would leave the one-thread-per-graph votes to a
        // couple of threads: they vote warp-wise instead - lane = clause, OR of the clause's node words over the graph's
        // slots, the weights of the lanes that fired summed over the warp (redux.sync), one shared-memory add per warp.
        const int ng = g1 - g0;
        const bool warp_votes = ng <= kWarpVoteGraphs && nn >= 8 * ng;
        if (warp_votes)
            for (int i = tid; i < ng * KP; i += kStreamThreads) s_vsum[i] = 0;
        // ---- per-graph state: graphs tid and tid+512 of the tile ----
        int acc[2][KP];
        int seg_lo[2], seg_hi[2];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
#pragma unroll
            for (int k = 0; k < KP; ++k) acc[s][k] = 0;
            const int gi = g0 + tid + s * kStreamThreads;
            if (gi < g1) {
                seg_lo[s] = (int)g.node_index[gi] - node0;
                seg_hi[s] = seg_lo[s] + (int)g.n_nodes[gi];
            } else {
                seg_lo[s] = 0; seg_hi[s] = 0;
            }
        }
        __syncthreads();

        for (int cb0 = 0; cb0 < m.C; cb0 += kStreamCB) {
            const int cbn = min(kStreamCB, m.C - cb0);
            // ---- evaluation: (clause, 4 node words) per thread; AND the transposed rows of the included literals ----
            for (int idx = tid; idx < kStreamCB * Q; idx += kStreamThreads) {
                const int cb = idx / Q, quad = idx - cb * Q;
                uint4 r = make_uint4(0u, 0u, 0u, 0u);              // rows past the last clause stay empty
                if (cb < cbn) {
                    const int c = cb0 + cb;
                    const unsigned xq = xt32 + quad * 16;
                    r = *reinterpret_cast<const uint4 *>(TMV + (c % g.n_types) * TNC + quad * 4);
                    const int o0 = a.lit_off[c], o1 = a.lit_off[c + 1];
                    const uint2 *lp = reinterpret_cast<const uint2 *>(a.lit_list + o0);
                    const int groups = (o1 - o0) >> 2;
#pragma unroll 2
                    for (int q = 0; q < groups; ++q) {
                        const uint2 four = __ldg(lp + q);
                        const uint4 x0 = lds128(xq + (four.x & 0xffffu));
                        const uint4 x1 = lds128(xq + (four.x >> 16));
                        const uint4 x2 = lds128(xq + (four.y & 0xffffu));
                        const uint4 x3 = lds128(xq + (four.y >> 16));
                        r.x &= x0.x & x1.x; r.y &= x0.y & x1.y; r.z &= x0.z & x1.z; r.w &= x0.w & x1.w;
                        r.x &= x2.x & x3.x; r.y &= x2.y & x3.y; r.z &= x2.z & x3.z; r.w &= x2.w & x3.w;
                    }
                }
                *reinterpret_cast<uint4 *>(R + (size_t)cb * TNC + quad * 4) = r;
            }
            for (int i = tid; i < cbn * KROW; i += kStreamThreads) Wb[i] = a.Wt[(size_t)cb0 * KROW + i];
            __syncthreads();
            if (warp_votes) {
                for (int task = warp; task < CW * ng; task += nwarps) {
                    const int cw = task % CW, gl = task / CW;
                    const int cb = 32 * cw + lane;
                    const int lo = (int)g.node_index[g0 + gl] - node0, hi = lo + (int)g.n_nodes[g0 + gl];     // slots [lo, hi)
                    u32 any = 0;
                    if (cb < cbn)
                        for (int j = lo >> 5; j <= (hi - 1) >> 5; ++j) {
                            u32 mask = kFull;
                            if (j == lo >> 5) mask &= kFull << (lo & 31);
                            if (j == (hi - 1) >> 5) mask &= kFull >> (31 - ((hi - 1) & 31));
                            any |= R[(size_t)cb * TNC + j] & mask;
                        }
                    const bool fired = any != 0;
                    if (!__any_sync(kFull, fired)) continue;
                    int mine = 0;
#pragma unroll
                    for (int k = 0; k < KP; ++k) {
                        const int sk = __reduce_add_sync(kFull, fired && k < KROW ? Wb[(size_t)cb * KROW + k] : 0);
                        if (lane == k) mine = sk;
                    }
                    if (lane < m.K) atomicAdd(&s_vsum[gl * KP + lane], mine);
                }
                __syncthreads();
                continue;
            }
            // ---- 32 clauses x 32 nodes blocks of R, transposed in registers: warp = clause word, lane = node word ----
            for (int blk = tid; blk < CW * TNC; blk += kStreamThreads) {
                const int cw = blk / TNC, j = blk - cw * TNC;
                u32 rows[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) rows[i] = R[(size_t)(32 * cw + i) * TNC + j];
                transpose32(rows);
#pragma unroll
                for (int b = 0; b < 32; ++b) RT[(size_t)cw * 32 * kRTStride + b * kRTStride + j] = rows[b];
            }
            __syncthreads();
            // ---- votes: one thread per graph; OR of its nodes' clause words, then only the clauses that fired ----
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                if (seg_hi[s] <= seg_lo[s]) continue;
                for (int cw = 0; cw < CW; ++cw) {
                    const u32 *rt = RT + (size_t)cw * 32 * kRTStride;
                    u32 fired = 0;
                    for (int v = seg_lo[s]; v < seg_hi[s]; ++v) fired |= rt[(v & 31) * kRTStride + (v >> 5)];
                    while (fired) {
                        const int cb = 32 * cw + __ffs(fired) - 1;
                        fired &= fired - 1;
                        const int4 *wr = reinterpret_cast<const int4 *>(Wb + (size_t)cb * KROW);
#pragma unroll
                        for (int k4 = 0; k4 < (KP + 3) / 4; ++k4) {
                            const int4 t = wr[k4];
                            acc[s][4 * k4] += t.x;
                            if (4 * k4 + 1 < KP) acc[s][4 * k4 + 1] += t.y;
                            if (4 * k4 + 2 < KP) acc[s][4 * k4 + 2] += t.z;
                            if (4 * k4 + 3 < KP) acc[s][4 * k4 + 3] += t.w;
                        }
                    }
                }
            }
            __syncthreads();
        }

        // ---- class sums of the tile's graphs (only those inside the requested range) ----
        if (warp_votes)
            for (int i = tid; i < ng * m.K; i += kStreamThreads) {
                const int gl = i / m.K, k = i - gl * m.K;
                const int64_t gi = (int64_t)g0 + gl;
                if (gi >= a.first && gi < a.first + a.count) a.class_sums[(size_t)(gi - a.first) * m.K + k] = s_vsum[gl * KP + k];
            }
#pragma unroll
        for (int s = 0; s < 2 && !warp_votes; ++s) {
            const int64_t gi = (int64_t)g0 + tid + s * kStreamThreads;
            if (gi < g1 && gi >= a.first && gi < a.first + a.count) {
                int *out = a.class_sums + (size_t)(gi - a.first) * m.K;
#pragma unroll
                for (int k = 0; k < KP; ++k)
                    if (k < m.K) out[k] = acc[s][k];
            }
        }
        __syncthreads();   // s_tile and the shared buffers are reused by the next tile
    }
}

// ------------------------------------------------------------------------------------------------ host side
inline int stream_krow(int K) { return (K + 3) & ~3; }

// node words per tile: as many as keep the transposed literals within 64 KB (so that row offsets fit 16 bits),
// at most 2*threads/32 (two graphs per thread), at least 4 (a thread evaluates 4 words at a time)
inline int stream_tile_words(int literals)
{
    int TNC = 2 * kStreamThreads / 32;
    while (TNC > 4 && (size_t)(literals + 1) * TNC * sizeof(u32) > 64 * 1024) TNC >>= 1;
    return (size_t)(literals + 1) * TNC * sizeof(u32) <= 64 * 1024 ? TNC : 0;
}

int stream_model_create(StreamModel *sm, const DevModel &d)
{
    if (d.D != 1 || d.K > kStreamMaxK || stream_tile_words(d.literals) == 0) return GTM_OK;   // path not applicable
    sm->KROW = stream_krow(d.K);
    sm->TNC = stream_tile_words(d.literals);
    GTM_TRY(dev_alloc(&sm->lit_off, (size_t)d.C + 1));
    GTM_TRY(dev_alloc(&sm->lit_cnt, (size_t)d.C));
    GTM_TRY(dev_alloc(&sm->lit_list, (size_t)d.C * ((d.literals + 3) & ~3) + 4));
    GTM_TRY(dev_alloc(&sm->Wt, (size_t)d.C * sm->KROW));
    return GTM_OK;
}

void stream_model_destroy(StreamModel *sm)
{
    cudaFree(sm->lit_off); cudaFree(sm->lit_cnt); cudaFree(sm->lit_list); cudaFree(sm->Wt);
    *sm = StreamModel();
}

int stream_model_refresh(StreamModel *sm, const DevModel &d, cudaStream_t s)
{
    if (!sm->lit_off) return GTM_OK;
    const int blocks = (d.C + 255) / 256;
    stream_count_kernel<<<blocks, 256, 0, s>>>(d, sm->lit_cnt);
    stream_scan_kernel<<<1, 1024, 0, s>>>(sm->lit_cnt, sm->lit_off, d.C);
    stream_fill_kernel<<<blocks, 256, 0, s>>>(d, sm->lit_off, sm->lit_list, sm->Wt, sm->KROW, sm->TNC);
    GTM_CU(cudaGetLastError());
    return GTM_OK;
}

template <int KP>
inline const void *stream_kernel_ptr() { return (const void *)stream_score_kernel<KP>; }

inline const void *stream_kernel_for(int K)
{
    if (K <= 2) return stream_kernel_ptr<2>();
    if (K <= 4) return stream_kernel_ptr<4>();
    if (K <= 8) return stream_kernel_ptr<8>();
    if (K <= 10) return stream_kernel_ptr<10>();
    if (K <= 12) return stream_kernel_ptr<12>();
    return stream_kernel_ptr<16>();
}

inline size_t stream_smem_bytes(const DevModel &d, int TNC, int n_types, int KROW)
{
    return ((size_t)(d.literals + 1) * TNC + (size_t)n_types * TNC + (size_t)kStreamCB * TNC +
            (size_t)(kStreamCB / 32) * 32 * kRTStride) * sizeof(u32) + (size_t)kStreamCB * KROW * sizeof(int);
}

constexpr int kStreamMaxTypes = 8;

int stream_data_create(StreamData *sd, const StreamModel &sm, const DevModel &d, const DevGraphs &,
                              const gtm_graphs_view *v, int sm_count, cudaStream_t s)
{
    sd->supported = 0;
    if (!sm.lit_off) return GTM_OK;
    const int TNC = sm.TNC;
    if (v->max_number_of_graph_nodes > TNC * 32) return GTM_OK;        // a graph must fit one tile
    const size_t smem = stream_smem_bytes(d, TNC, kStreamMaxTypes, sm.KROW);
    if (smem > 200 * 1024) return GTM_OK;
    const void *fn = stream_kernel_for(d.K);
    GTM_CU(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int per_sm = 0;
    GTM_CU(cudaOccupancyMaxActiveBlocksPerMultiprocessorWithFlags(&per_sm, fn, kStreamThreads, smem, 0));
    if (per_sm < 1) return GTM_OK;

    // tiling: consecutive graphs while the node count stays within the tile (and at most two graphs per thread).
    // Sets of single-node graphs need no table: every tile holds the same number of graphs.
    const int TN = TNC * 32;
    std::vector<int> &tg = sd->tile_graph_host;
    tg.clear();
    sd->tile_graph = nullptr;
    if (v->max_number_of_graph_nodes == 1) {
        sd->graphs_per_tile = std::min(TN, 2 * kStreamThreads);
        sd->n_tiles = (int)((v->number_of_graphs + sd->graphs_per_tile - 1) / sd->graphs_per_tile);
    } else {
        sd->graphs_per_tile = 0;
        tg.reserve((size_t)(v->total_nodes / TN) * 2 + 16);
        tg.push_back(0);
        int64_t used = 0;
        for (int64_t gi = 0; gi < v->number_of_graphs; ++gi) {
            const int64_t n = v->number_of_graph_nodes[gi];
            if (used + n > TN || (gi - tg.back()) >= 2 * kStreamThreads) { tg.push_back((int)gi); used = 0; }
            used += n;
        }
        tg.push_back((int)v->number_of_graphs);
        sd->n_tiles = (int)tg.size() - 1;
        GTM_TRY(pool_alloc(&sd->tile_graph, tg.size(), s));
        GTM_CU(cudaMemcpyAsync(sd->tile_graph, tg.data(), tg.size() * sizeof(int), cudaMemcpyHostToDevice, s));
    }
    sd->stream = s;
    GTM_TRY(pool_alloc(&sd->tile_counter, 1, s));
    sd->TNC = TNC;
    sd->grid = sm_count * per_sm;
    sd->smem = smem;
    sd->total_nodes = v->total_nodes;
    sd->n_graphs = v->number_of_graphs;
    sd->supported = 1;
    return GTM_OK;
}

void stream_data_destroy(StreamData *sd)
{
    if (sd->tile_graph) cudaFreeAsync(sd->tile_graph, sd->stream);
    if (sd->tile_counter) cudaFreeAsync(sd->tile_counter, sd->stream);
    sd->tile_graph = nullptr; sd->tile_counter = nullptr; sd->supported = 0;
}

bool stream_supported(const StreamData &sd, int n_types) { return sd.supported != 0 && n_types <= kStreamMaxTypes; }

int stream_score(const StreamModel &sm, const StreamData &sd, const DevModel &d, const DevGraphs &dg, int n_types,
                        int64_t first, int64_t count, int *sums_dev, cudaStream_t s)
{
    DevGraphs g = dg;
    g.n_types = n_types;
    StreamArgs a;
    a.tile_graph = sd.tile_graph;
    // tiles that overlap [first, first+count)
    int lo, hi;
    if (sd.graphs_per_tile > 0) {
        lo = (int)(first / sd.graphs_per_tile);
        hi = (int)((first + count + sd.graphs_per_tile - 1) / sd.graphs_per_tile);
    } else {
        const std::vector<int> &tg = sd.tile_graph_host;
        lo = (int)(std::upper_bound(tg.begin(), tg.end(), (int)first) - tg.begin()) - 1;
        hi = (int)(std::lower_bound(tg.begin(), tg.end(), (int)(first + count)) - tg.begin());
    }
    a.graphs_per_tile = sd.graphs_per_tile;
    a.tile_lo = lo; a.tile_hi = hi;
    a.first = first; a.count = count; a.n_graphs = sd.n_graphs; a.total_nodes = sd.total_nodes;
    a.class_sums = sums_dev; a.tile_counter = sd.tile_counter; a.TNC = sd.TNC;
    a.lit_off = sm.lit_off; a.lit_list = sm.lit_list; a.Wt = sm.Wt; a.KROW = sm.KROW;
    GTM_CU(cudaMemsetAsync(sd.tile_counter, 0, sizeof(unsigned), s));
    const int grid = std::max(1, std::min(sd.grid, hi - lo));
    DevModel dm = d;
    void *args[] = {&dm, &g, &a};
    GTM_CU(cudaLaunchKernel(stream_kernel_for(d.K), dim3(grid), dim3(kStreamThreads), args,
                            stream_smem_bytes(d, sd.TNC, n_types, sm.KROW), s));
    return GTM_OK;
}

}  // namespace gtm
