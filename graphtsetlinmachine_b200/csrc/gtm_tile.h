// Tile scoring (gtm_tile.cu): batched inference for ANY depth on graph sets whose graphs have at most 128 nodes.
// Types and entry points used by the host runtime.
#pragma once
#include <vector>

#include "gtm_device.cuh"
#include "gtm_host.cuh"

namespace gtm {

// One layer's included-literal lists as the kernel reads them (device memory).  Clauses are taken in the layer's own
// order (by decreasing list length); the lists of the 32 clauses of a block of positions are interleaved: group g
// (four 16-bit row numbers, 8 bytes) of position p is element blk_off[p / 32] + 32 * g + p % 32.
struct TileLayer {
    const int *order;             // [C] clause at every position
    const int *cnt;               // [C] list length of every CLAUSE in groups of four rows
    const int *blk_off;           // [ceil(C/32)+1] first element of every block of 32 positions
    const unsigned short *list;   // row numbers in the transposed tile buffer, padded with rows of ones
};

struct TileModel {
    bool applicable = false;
    int D = 0, KROW = 0;
    int *cnt[kMaxDepth] = {};
    int *order[kMaxDepth] = {};
    int *blk_off[kMaxDepth] = {};
    unsigned short *list[kMaxDepth] = {};
    size_t list_cap[kMaxDepth] = {};
    int *Wt = nullptr;            // [C][KROW] weights, clause-major
    u32 *hvm = nullptr;           // [C][MB] hypervector bits reduced modulo the message size
    TileLayer *layers = nullptr;  // [D] device copy of the pointers above
};

struct TileData {
    int supported = 0;
    int TNC = 0;                        // node words per tile (4, 8, 16 or 32); a tile has TNC/4 quads of 128 node slots
    int PS = 0;                         // row stride (words, odd) of the node-major message buffers
    int words_a = 0, words_b = 0;       // sizes of the two big shared-memory buffers (words)
    int stage_rows = 0;                 // literal rows the staging buffer holds
    int gmax = 0;                       // most graphs in one tile
    int uniform_n = 0;                  // > 0: every graph has this many nodes: slots follow from the graph number
    int graphs_per_tile = 0;            // uniform sets: graphs per tile (no tile table)
    int n_tiles = 0;
    int *tile_graph = nullptr;          // [n_tiles+1] first graph of every tile (NULL for uniform sets)
    unsigned short *gpos = nullptr;     // [N] first node slot of every graph inside its tile (NULL for uniform sets)
    std::vector<int> tile_graph_host;
    unsigned *tile_counter = nullptr;
    uint4 *surv_r = nullptr;            // [grid][2][quad pairs][C][2] node bits of every clause on the pair's two quads after a layer
    cudaStream_t stream = nullptr;
    int grid = 0;
    size_t smem = 0;
    int64_t n_graphs = 0;
};

int tile_model_create(TileModel *tm, const DevModel &d);
void tile_model_destroy(TileModel *tm);
int tile_model_refresh(TileModel *tm, const DevModel &d, cudaStream_t s);
int tile_data_create(TileData *td, const TileModel &tm, const DevModel &d, const gtm_graphs_view *v, u32 n_min, u32 n_max,
                     int sm_count, cudaStream_t s);
void tile_data_destroy(TileData *td);
bool tile_supported(const TileData &td, int n_types);
int tile_score(const TileModel &tm, TileData &td, const DevModel &d, const DevGraphs &dg, int n_types, int64_t first,
               int64_t count, int *sums_dev, int *error_dev, cudaStream_t s);

}  // namespace gtm
