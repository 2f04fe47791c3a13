// Node-stream scoring (gtm_stream.cu): types and entry points used by the host runtime.
#pragma once
#include <vector>

#include "gtm_device.cuh"
#include "gtm_host.cuh"

namespace gtm {

struct StreamModel {
    int *lit_off = nullptr;             // [C+1] offsets into lit_list (multiples of 4)
    int *lit_cnt = nullptr;             // [C]   padded counts (scratch of the scan)
    unsigned short *lit_list = nullptr; // padded literal ids
    int *Wt = nullptr;                  // [C][KROW]
    int KROW = 0;
    int TNC = 0;                        // node words per tile (fixed by the number of literals)
};

struct StreamData {
    int supported = 0;
    int TNC = 0;                        // node words per tile
    int n_tiles = 0;
    int *tile_graph = nullptr;          // [n_tiles+1] first graph of every tile (NULL for sets of single-node graphs)
    int graphs_per_tile = 0;            // > 0: every tile holds this many graphs
    cudaStream_t stream = nullptr;      // stream the pooled buffers were allocated on
    std::vector<int> tile_graph_host;
    int grid = 0;
    size_t smem = 0;
    unsigned *tile_counter = nullptr;
    int64_t total_nodes = 0, n_graphs = 0;
};


int stream_model_create(StreamModel *sm, const DevModel &d);
void stream_model_destroy(StreamModel *sm);
int stream_model_refresh(StreamModel *sm, const DevModel &d, cudaStream_t s);
int stream_data_create(StreamData *sd, const StreamModel &sm, const DevModel &d, const DevGraphs &dg,
                       const gtm_graphs_view *v, int sm_count, cudaStream_t s);
void stream_data_destroy(StreamData *sd);
bool stream_supported(const StreamData &sd, int n_types);
int stream_score(const StreamModel &sm, const StreamData &sd, const DevModel &d, const DevGraphs &dg, int n_types,
                 int64_t first, int64_t count, int *sums_dev, cudaStream_t s);

}  // namespace gtm
