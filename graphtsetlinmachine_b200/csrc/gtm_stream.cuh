// Node-stream scoring path (fast path for batched inference).  Interface used by gtm_api.cu.
#pragma once
#include "gtm_device.cuh"
#include "gtm_host.cuh"

namespace gtm {

struct StreamModel { int unused; };
struct StreamData { int supported; };

inline int stream_model_create(StreamModel *, const DevModel &) { return GTM_OK; }
inline void stream_model_destroy(StreamModel *) {}
inline int stream_model_refresh(StreamModel *, const DevModel &, cudaStream_t) { return GTM_OK; }
inline int stream_data_create(StreamData *sd, const StreamModel &, const DevModel &, const DevGraphs &,
                              const gtm_graphs_view *, int, cudaStream_t) { sd->supported = 0; return GTM_OK; }
inline void stream_data_destroy(StreamData *) {}
inline bool stream_supported(const StreamData &sd) { return sd.supported != 0; }
inline int stream_score(const StreamModel &, const StreamData &, const DevModel &, const DevGraphs &, int, int64_t,
                        int64_t, int *, cudaStream_t) { return fail(GTM_ERR_STATE, "node-stream path not built"); }

}  // namespace gtm
