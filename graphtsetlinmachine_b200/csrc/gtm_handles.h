// Handle types behind the opaque pointers of the C ABI; shared by the translation units of the library.
#pragma once
#include <vector>

#include "gtm_device.cuh"
#include "gtm_host.cuh"
#include "gtm_stream.h"
#include "gtm_tile.h"

using namespace gtm;

// ---------------------------------------------------------------------------------------------- handles
struct gtm_model {
    gtm_config cfg;
    DevModel dm;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    bool has_state = false;
    u32 *recorded = nullptr;
    // learning-kernel buffers
    int fit_grid = 0, fit_block = 512;
    int *flag_host = nullptr;                 // page-locked landing place of score_error
    int *score_error = nullptr;               // raised by scoring kernels that skipped a malformed graph (device-pointer inputs)
    int *error = nullptr, *clause_node = nullptr, *update = nullptr, *class_sum_tap = nullptr;
    unsigned long long *exchange = nullptr;   // vote exchange area of a single-GPU fit (exchange_bytes(1, K))
    int opt_fit_block_clauses = 0;            // > 0: clauses per thread block of the state-resident kernel (0: automatic)
    int opt_fit_kernel = 0;                   // 0 auto, 1 state in global memory, 2 state resident in shared memory
    int opt_fit_wait_ms = 2000;               // budget of one device-side wait of the learning kernels
    int opt_fit_missing_cta = 0;              // test hook: waits expect one arrival that never comes (they must run out cleanly)
    int opt_fit_timers = 0;                   // 1: the learning kernels time their phases (gtm_debug_fit_phase_cycles)
    int opt_score_kernel = 0;                 // 0 auto, 1 general kernel, 2 node-stream kernel, 3 tile kernel
    unsigned *barrier = nullptr;
    unsigned long long *phase_cycles = nullptr;
    // node-stream scoring: derived include lists (rebuilt when the automata changed)
    StreamModel sm;
    bool lists_dirty = true;
    // tile scoring: included-literal lists of every layer, rebuilt when the state version moved on
    TileModel tm;
    unsigned long long state_version = 1, tile_lists_version = 0;
};

// Buffers through which the learning kernels of several GPUs talk to each other when clauses are sharded over ranks
// (one process per GPU): per rank one cudaMalloc'd block [arrival counter | vote slots | message buffers x 2], shared
// with the other ranks through CUDA IPC.
struct FitComm {
    void *block = nullptr;
    void *peer_block[kMaxRanks] = {};
    size_t bytes = 0, exchange_off = 0, P_off[2] = {0, 0};
    int world = 1, rank = 0, grid = 0;
    bool resident = false;
    int threads = 384, clauses_per_cta = 0, clause_words = 0, pre_words = 0, part_words = 0, stage = 1, t_stride = 0, rows_words = 0;
    size_t smem = 0;
    bool connected = false, broken = false;
    u32 tag_base = 0;
    unsigned barriers_done = 0;    // grid barriers of all launches so far (the counters in `block` only grow)
};

struct gtm_dataset {
    gtm_model *model;
    DevGraphs dg;
    int64_t n_graphs, total_nodes, total_edges;
    int max_nodes, NC;
    u32 n_min = 0, n_max = 0;      // smallest / largest graph (0: not known, e.g. a set that is copied chunk by chunk)
    std::vector<void *> owned;
    // learning scratch (every layer kept) and its message ping-pong
    EvalScratch fit_sc;
    u32 *P_pair[2] = {nullptr, nullptr};
    u32 *Q_pair[2] = {nullptr, nullptr};   // [D-1][max_nodes][MW] destination message rows by graph parity (learning, merged marks)
    unsigned *rank_barrier = nullptr;      // arrival counter of the barriers among one rank's CTAs
    // scoring scratch of the general path: one slice per CTA
    EvalScratch score_sc;
    size_t cno_stride = 0, P_stride = 0, ninc_stride = 0;
    int score_grid = 0;
    int score_units = 1;           // graphs in flight per CTA of the general scoring path: 1 (a CTA per graph) or 8 (a warp per graph)
    int score_block = 256;         // threads per CTA of the general scoring kernel
    int score_t_stride = 0;        // row stride of the general scoring kernel's transposed-graph buffer (0 = none)
    int score_part_words = 0;      // shared-memory message accumulation of the general scoring kernel (0 = none)
    size_t score_smem = 0;
    int *Y = nullptr;
    size_t Y_capacity = 0;
    // node-stream scoring
    StreamData sd;
    // tile scoring
    TileData td;
    // clause-sharded learning
    FitComm comm;
};


// learning kernels (gtm_fit.cu)
int fit_grid_for_global_state(const DevModel &d, int sm_count, int block, int *grid_out);
int launch_fit(gtm_model *m, gtm_dataset *ds, int n_types, const int *Y_dev, int64_t first, int64_t count, int epochs,
               int eval_only);
void fit_comm_release(gtm_dataset *ds);
size_t exchange_bytes(int world, int K);
