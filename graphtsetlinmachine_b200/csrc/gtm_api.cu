// Host runtime and C ABI (include/gtm_b200.h) of the B200-native Graph Tsetlin Machine engine.
#include "../../include/gtm_b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cmath>
#include <cstring>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "gtm_handles.h"
#include "gtm_kernels.cuh"

// The general scoring kernel with or without four-at-a-time node words (graph sets with more than 32 nodes per graph).
static const void *score_kernel_for(int max_nodes, int units = 1)
{
    if (units > 1) return (const void *)score_small_graphs_kernel;
    return max_nodes > 32 ? (const void *)score_graphs_kernel<true> : (const void *)score_graphs_kernel<false>;
}

static int bind(gtm_model *m)
{
    if (!m) return fail(GTM_ERR_ARG, "null model handle");
    GTM_CU(cudaSetDevice(m->cfg.device));
    return GTM_OK;
}

// largest float that is <= d
static float float_round_down(double d)
{
    float f = (float)d;
    if ((double)f > d) f = nextafterf(f, -INFINITY);
    return f;
}

static int words_for(int bits) { return (bits - 1) / 32 + 1; }
static u32 tail_mask(int bits) { return (bits % 32) ? ~(0xffffffffu << (bits % 32)) : 0xffffffffu; }
static int layer_words(const gtm_model *m, int layer) { return layer == 0 ? m->dm.L0 : m->dm.M; }
static u32 *layer_planes(const gtm_model *m, int layer)
{
    const DevModel &d = m->dm;
    return layer == 0 ? d.ta0 : d.tam + (size_t)(layer - 1) * d.C * d.SB * d.M;
}

// --------------------------------------------------------------------------------------------- library
extern "C" const char *gtm_version(void) { return "gtm_b200 0.1 (sm_100a)"; }
extern "C" const char *gtm_last_error(void) { return gtm_error_text().c_str(); }

extern "C" int gtm_device_count(int *count_out)
{
    if (!count_out) return fail(GTM_ERR_ARG, "count_out is null");
    GTM_CU(cudaGetDeviceCount(count_out));
    return GTM_OK;
}

// ---------------------------------------------------------------------------------------------- model
extern "C" int gtm_create(const gtm_config *cfg, gtm_model **out)
{
    if (!cfg || !out) return fail(GTM_ERR_ARG, "null argument");
    *out = nullptr;
    if (cfg->number_of_clauses < 1 || cfg->number_of_outputs < 1 || cfg->number_of_literals < 1)
        return fail(GTM_ERR_ARG, "clauses, outputs and literals must be positive");
    if (cfg->number_of_state_bits < 1 || cfg->number_of_state_bits > GTM_MAX_STATE_BITS)
        return fail(GTM_ERR_ARG, "number_of_state_bits must be in 1..%d", GTM_MAX_STATE_BITS);
    if (cfg->depth < 1 || cfg->depth > GTM_MAX_DEPTH) return fail(GTM_ERR_ARG, "depth must be in 1..%d", GTM_MAX_DEPTH);
    if (cfg->T < 1) return fail(GTM_ERR_ARG, "T must be positive");
    if (cfg->depth > 1 && (cfg->message_size < 1 || cfg->message_bits < 1))
        return fail(GTM_ERR_ARG, "message_size and message_bits must be positive when depth > 1");
    for (int d = 0; d < cfg->depth; ++d)
        if (!(cfg->s[d] > 0.0f)) return fail(GTM_ERR_ARG, "s[%d] must be positive", d);
    int ndev = 0;
    GTM_CU(cudaGetDeviceCount(&ndev));
    if (cfg->device < 0 || cfg->device >= ndev) return fail(GTM_ERR_ARG, "device %d out of range (%d visible)", cfg->device, ndev);
    GTM_CU(cudaSetDevice(cfg->device));

    gtm_model *m = new (std::nothrow) gtm_model();
    if (!m) return fail(GTM_ERR_OOM, "host allocation failed");
    m->cfg = *cfg;
    DevModel &d = m->dm;
    memset(&d, 0, sizeof d);
    d.C = cfg->number_of_clauses; d.K = cfg->number_of_outputs; d.literals = cfg->number_of_literals;
    d.SB = cfg->number_of_state_bits; d.boost = cfg->boost_true_positive_feedback; d.T = cfg->T;
    d.max_included = cfg->max_included_literals; d.MS = std::max(1, cfg->message_size);
    d.MB = std::max(1, cfg->message_bits); d.D = cfg->depth;
    d.L0 = words_for(d.literals); d.M = words_for(2 * d.MS); d.MW = words_for(d.MS);
    d.lit_mask = tail_mask(d.literals); d.msg_mask = tail_mask(2 * d.MS);
    for (int i = 0; i < kMaxDepth; ++i) d.s[i] = cfg->s[i];
    d.q_keep = 1.0 * cfg->q / (double)std::max(1, d.K - 1);
    d.q_keep_f = float_round_down(d.q_keep);
    for (int i = 0; i < kMaxDepth; ++i) d.p_mask[i] = cfg->s[i] > 0.0f ? float_round_down(1.0 / (double)cfg->s[i]) : 1.0f;
    d.seed_lo = (u32)cfg->seed; d.seed_hi = (u32)(cfg->seed >> 32);

    cudaDeviceProp prop;
    GTM_CU(cudaGetDeviceProperties(&prop, cfg->device));
    m->sm_count = prop.multiProcessorCount;
    { int st0 = pool_prepare(cfg->device); if (st0 != GTM_OK) { delete m; return st0; } }

    int st = GTM_OK;
    st = dev_alloc(&d.ta0, (size_t)d.C * d.SB * d.L0);
    if (st == GTM_OK) st = dev_alloc(&d.tam, (size_t)std::max(1, d.D - 1) * d.C * d.SB * d.M);
    u32 *hv = nullptr;
    if (st == GTM_OK) st = dev_alloc(&d.weights, (size_t)d.K * d.C);
    if (st == GTM_OK) st = dev_alloc(&hv, (size_t)d.C * d.MB);
    if (st == GTM_OK) st = dev_alloc(&d.draw_pos, (size_t)d.C);
    if (st == GTM_OK) st = dev_alloc(&m->clause_node, (size_t)d.C);
    if (st == GTM_OK) st = dev_alloc(&m->update, (size_t)d.K * d.C);
    if (st == GTM_OK) st = dev_alloc(&m->class_sum_tap, (size_t)d.K);
    if (st == GTM_OK) st = dev_alloc(&m->barrier, 1);
    if (st == GTM_OK) st = dev_alloc(&m->error, 1);
    if (st == GTM_OK) st = dev_alloc(&m->score_error, 1);
    if (st == GTM_OK && cudaMallocHost((void **)&m->flag_host, sizeof(int)) != cudaSuccess) st = fail(GTM_ERR_OOM, "page-locked host allocation failed");
    if (st == GTM_OK) st = dev_alloc(&m->phase_cycles, 8);
    if (st != GTM_OK) { gtm_destroy(m); return st; }
    d.hv = hv;
    cudaMemset(hv, 0, (size_t)d.C * d.MB * sizeof(u32));
    cudaMemset(d.draw_pos, 0, (size_t)d.C * sizeof(u64));
    cudaMemset(d.weights, 0, (size_t)d.K * d.C * sizeof(int));
    cudaMemset(m->score_error, 0, sizeof(int));

    // learning grid: all CTAs must be co-resident (cooperative launch); no more warps than clauses
    st = fit_grid_for_global_state(d, m->sm_count, m->fit_block, &m->fit_grid);
    if (st != GTM_OK) { gtm_destroy(m); return st; }
    st = dev_alloc(&m->exchange, exchange_bytes(1, d.K) / sizeof(unsigned long long) + 1);
    if (st == GTM_OK) st = stream_model_create(&m->sm, d);
    if (st == GTM_OK) st = tile_model_create(&m->tm, d);
    if (st != GTM_OK) { gtm_destroy(m); return fail(st, "device allocation failed"); }
    *out = m;
    return GTM_OK;
}

extern "C" int gtm_destroy(gtm_model *m)
{
    if (!m) return GTM_OK;
    cudaSetDevice(m->cfg.device);
    cudaFree(m->dm.ta0); cudaFree(m->dm.tam);
    cudaFree(m->dm.weights); cudaFree((void *)m->dm.hv); cudaFree(m->dm.draw_pos); cudaFree(m->recorded);
    cudaFree(m->exchange); cudaFree(m->error); cudaFree(m->score_error); cudaFree(m->clause_node); cudaFree(m->update);
    cudaFree(m->class_sum_tap); cudaFree(m->barrier); cudaFree(m->phase_cycles);
    stream_model_destroy(&m->sm);
    tile_model_destroy(&m->tm);
    if (m->flag_host) cudaFreeHost(m->flag_host);
    delete m;
    return GTM_OK;
}

extern "C" int gtm_set_stream(gtm_model *m, void *stream)
{
    GTM_TRY(bind(m));
    m->stream = (cudaStream_t)stream;
    return GTM_OK;
}

extern "C" int gtm_set_option(gtm_model *m, const char *name, int value)
{
    GTM_TRY(bind(m));
    if (!name) return fail(GTM_ERR_ARG, "option name is null");
    if (!strcmp(name, "fit_block_clauses") && value >= 0 && value <= 4096) { m->opt_fit_block_clauses = value; return GTM_OK; }
    if (!strcmp(name, "fit_kernel") && value >= 0 && value <= 2) { m->opt_fit_kernel = value; return GTM_OK; }
    if (!strcmp(name, "score_kernel") && value >= 0 && value <= 3) { m->opt_score_kernel = value; return GTM_OK; }
    if (!strcmp(name, "fit_timers") && value >= 0 && value <= 3) { m->opt_fit_timers = value; return GTM_OK; }
    if (!strcmp(name, "fit_wait_ms") && value >= 1 && value <= 600000) { m->opt_fit_wait_ms = value; return GTM_OK; }
    if (!strcmp(name, "fit_missing_cta") && value >= 0 && value <= 1) { m->opt_fit_missing_cta = value; return GTM_OK; }
    return fail(GTM_ERR_ARG, "unknown option '%s' or value %d out of range", name, value);
}

extern "C" int gtm_init_state(gtm_model *m, int reset_message_layers)
{
    GTM_TRY(bind(m));
    const DevModel &d = m->dm;
    init_weights_kernel<<<(d.C + 255) / 256, 256, 0, m->stream>>>(d);
    for (int l = 0; l < d.D; ++l) {
        if (l > 0 && !reset_message_layers) break;
        const size_t total = (size_t)d.C * d.SB * layer_words(m, l);
        init_planes_kernel<<<(unsigned)std::min<size_t>((total + 255) / 256, 4096), 256, 0, m->stream>>>(layer_planes(m, l), d.C, d.SB, layer_words(m, l));
    }
    GTM_CU(cudaGetLastError());
    GTM_CU(cudaStreamSynchronize(m->stream));
    m->has_state = true;
    m->lists_dirty = true; ++m->state_version;
    return GTM_OK;
}

static int check_layer(gtm_model *m, int layer)
{
    if (layer < 0 || layer >= m->dm.D) return fail(GTM_ERR_ARG, "layer %d out of range (depth %d)", layer, m->dm.D);
    return GTM_OK;
}

extern "C" int gtm_set_ta_state(gtm_model *m, int layer, const uint32_t *ta)
{
    GTM_TRY(bind(m));
    GTM_TRY(check_layer(m, layer));
    if (!ta) return fail(GTM_ERR_ARG, "ta_state is null");
    const DevModel &d = m->dm;
    const int W = layer_words(m, layer);
    const size_t total = (size_t)d.C * d.SB * W;
    u32 *tmp;
    GTM_TRY(pool_alloc(&tmp, total, m->stream));      // stream-ordered: no device-wide synchronisation
    cudaError_t e = cudaMemcpyAsync(tmp, ta, total * sizeof(u32), cudaMemcpyHostToDevice, m->stream);
    if (e == cudaSuccess)
        planes_from_reference_kernel<<<(unsigned)std::min<size_t>((total + 255) / 256, 4096), 256, 0, m->stream>>>(tmp, layer_planes(m, layer), d.C, d.SB, W);
    cudaFreeAsync(tmp, m->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    GTM_CU(e);
    m->has_state = true;
    m->lists_dirty = true; ++m->state_version;
    return GTM_OK;
}

extern "C" int gtm_get_ta_state(gtm_model *m, int layer, uint32_t *out)
{
    GTM_TRY(bind(m));
    GTM_TRY(check_layer(m, layer));
    if (!out) return fail(GTM_ERR_ARG, "ta_state_out is null");
    const DevModel &d = m->dm;
    const int W = layer_words(m, layer);
    const size_t total = (size_t)d.C * d.SB * W;
    u32 *tmp;
    GTM_TRY(pool_alloc(&tmp, total, m->stream));
    planes_to_reference_kernel<<<(unsigned)std::min<size_t>((total + 255) / 256, 4096), 256, 0, m->stream>>>(layer_planes(m, layer), tmp, d.C, d.SB, W);
    cudaError_t e = cudaMemcpyAsync(out, tmp, total * sizeof(u32), cudaMemcpyDeviceToHost, m->stream);
    cudaFreeAsync(tmp, m->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    GTM_CU(e);
    return GTM_OK;
}

extern "C" int gtm_set_weights(gtm_model *m, const int32_t *w)
{
    GTM_TRY(bind(m));
    if (!w) return fail(GTM_ERR_ARG, "clause_weights is null");
    GTM_CU(cudaMemcpyAsync(m->dm.weights, w, (size_t)m->dm.K * m->dm.C * sizeof(int), cudaMemcpyHostToDevice, m->stream));
    GTM_CU(cudaStreamSynchronize(m->stream));
    m->lists_dirty = true; ++m->state_version;
    return GTM_OK;
}

extern "C" int gtm_get_weights(gtm_model *m, int32_t *w)
{
    GTM_TRY(bind(m));
    if (!w) return fail(GTM_ERR_ARG, "clause_weights_out is null");
    GTM_CU(cudaMemcpyAsync(w, m->dm.weights, (size_t)m->dm.K * m->dm.C * sizeof(int), cudaMemcpyDeviceToHost, m->stream));
    GTM_CU(cudaStreamSynchronize(m->stream));
    return GTM_OK;
}

extern "C" int gtm_set_hypervectors(gtm_model *m, const uint32_t *hv)
{
    GTM_TRY(bind(m));
    if (!hv) return fail(GTM_ERR_ARG, "hypervectors is null");
    GTM_CU(cudaMemcpyAsync((void *)m->dm.hv, hv, (size_t)m->dm.C * m->dm.MB * sizeof(u32), cudaMemcpyHostToDevice, m->stream));
    GTM_CU(cudaStreamSynchronize(m->stream));
    m->lists_dirty = true; ++m->state_version;
    return GTM_OK;
}

extern "C" int gtm_set_draw_positions(gtm_model *m, const uint64_t *pos)
{
    GTM_TRY(bind(m));
    if (!pos) return fail(GTM_ERR_ARG, "positions is null");
    GTM_CU(cudaMemcpyAsync(m->dm.draw_pos, pos, (size_t)m->dm.C * sizeof(u64), cudaMemcpyHostToDevice, m->stream));
    GTM_CU(cudaStreamSynchronize(m->stream));
    return GTM_OK;
}

extern "C" int gtm_get_draw_positions(gtm_model *m, uint64_t *pos)
{
    GTM_TRY(bind(m));
    if (!pos) return fail(GTM_ERR_ARG, "positions_out is null");
    GTM_CU(cudaMemcpyAsync(pos, m->dm.draw_pos, (size_t)m->dm.C * sizeof(u64), cudaMemcpyDeviceToHost, m->stream));
    GTM_CU(cudaStreamSynchronize(m->stream));
    return GTM_OK;
}

extern "C" int gtm_set_recorded_draws(gtm_model *m, const uint32_t *draws, uint64_t per_clause)
{
    GTM_TRY(bind(m));
    GTM_CU(cudaStreamSynchronize(m->stream));
    cudaFree(m->recorded);
    m->recorded = nullptr; m->dm.recorded = nullptr; m->dm.recorded_len = 0;
    if (!draws) return GTM_OK;
    if (per_clause == 0) return fail(GTM_ERR_ARG, "draws_per_clause must be positive");
    const size_t total = (size_t)m->dm.C * per_clause;
    GTM_TRY(dev_alloc(&m->recorded, total));
    GTM_CU(cudaMemcpy(m->recorded, draws, total * sizeof(u32), cudaMemcpyHostToDevice));
    m->dm.recorded = m->recorded;
    m->dm.recorded_len = per_clause;
    return GTM_OK;
}

// --------------------------------------------------------------------------------------------- datasets
// `slack`: elements allocated beyond `count` (never copied, never interpreted)
template <class T>
static int upload(gtm_dataset *ds, const T **dev, const T *host, size_t count, cudaStream_t s, bool copy = true, size_t slack = 0)
{
    T *p;
    GTM_TRY(pool_alloc(&p, count + slack, s));
    ds->owned.push_back(p);
    if (copy && count && host) GTM_CU(cudaMemcpyAsync(p, host, count * sizeof(T), cudaMemcpyHostToDevice, s));
    *dev = p;
    return GTM_OK;
}

template <class T>
static int scratch(gtm_dataset *ds, T **dev, size_t count)
{
    GTM_TRY(pool_alloc(dev, count, ds->model->stream));
    ds->owned.push_back(*dev);
    return GTM_OK;
}

__global__ void graph_edge_ranges_kernel(const u32 *node_index, const u32 *n_nodes, const u32 *edge_index, const u32 *degree,
                                         int64_t n_graphs, u32 *e0, u32 *ne)
{
    for (int64_t gi = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; gi < n_graphs; gi += (int64_t)gridDim.x * blockDim.x) {
        const u32 first = node_index[gi], last = first + n_nodes[gi] - 1;
        const u32 start = edge_index[first];
        e0[gi] = start;
        ne[gi] = edge_index[last] + degree[last] - start;
    }
}

// Fills graph_edge0 / graph_edges from the uploaded arrays (queued on the model's stream).
static int derive_edge_ranges(gtm_dataset *ds, int64_t n_graphs)
{
    cudaStream_t s = ds->model->stream;
    u32 *e0 = const_cast<u32 *>(ds->dg.graph_edge0), *ne = const_cast<u32 *>(ds->dg.graph_edges);
    if (ds->total_edges == 0) {
        GTM_CU(cudaMemsetAsync(e0, 0, (size_t)n_graphs * sizeof(u32), s));
        GTM_CU(cudaMemsetAsync(ne, 0, (size_t)n_graphs * sizeof(u32), s));
        return GTM_OK;
    }
    graph_edge_ranges_kernel<<<(unsigned)std::min<int64_t>((n_graphs + 255) / 256, 4096), 256, 0, s>>>(
        ds->dg.node_index, ds->dg.n_nodes, ds->dg.edge_index, ds->dg.degree, n_graphs, e0, ne);
    GTM_CU(cudaGetLastError());
    return GTM_OK;
}

// Host arrays must have the layout that graphs.py produces: node_index and edge_index are exclusive prefix sums of the
// node counts and out-degrees (graphs.py:101-102,127-128), every graph has 1..max_number_of_graph_nodes nodes.  The
// kernels size their scratch rows from max_number_of_graph_nodes and index the arrays with these values, so anything
// else is refused here.  Checks graphs [g_lo, g_hi) and their nodes.
struct GraphChecks { u32 bad_count = 0, bad_index = 0, bad_edges = 0, n_min = ~0u, n_max = 0; };

static void check_graph_span(const gtm_graphs_view *v, int64_t g_lo, int64_t g_hi, GraphChecks *out)
{
    const int64_t N = v->number_of_graphs;
    const u32 max_nodes = (u32)v->max_number_of_graph_nodes;
    GraphChecks c;
    for (int64_t gi = g_lo; gi < g_hi; ++gi) {
        const u32 n = v->number_of_graph_nodes[gi];
        const uint64_t end = (uint64_t)v->node_index[gi] + n;
        const uint64_t want = gi + 1 < N ? (uint64_t)v->node_index[gi + 1] : (uint64_t)v->total_nodes;
        c.bad_count |= (u32)(n - 1u >= max_nodes);
        c.bad_index |= (u32)(end != want);
        c.n_min = std::min(c.n_min, n);
        c.n_max = std::max(c.n_max, n);
    }
    if (!c.bad_count && !c.bad_index) {          // node ranges are sound: the span's nodes
        const int64_t v_lo = v->node_index[g_lo], v_hi = g_hi < N ? (int64_t)v->node_index[g_hi] : v->total_nodes;
        for (int64_t vi = v_lo; vi < v_hi; ++vi) {
            const uint64_t end = (uint64_t)v->edge_index[vi] + v->number_of_graph_node_edges[vi];
            const uint64_t want = vi + 1 < v->total_nodes ? (uint64_t)v->edge_index[vi + 1] : (uint64_t)v->total_edges;
            c.bad_edges |= (u32)(end != want);
        }
    }
    *out = c;
}

static int validate_graphs(const gtm_graphs_view *v, int64_t g_lo, int64_t g_hi, u32 *n_min_out = nullptr, u32 *n_max_out = nullptr)
{
    if (g_lo == 0 && (v->node_index[0] != 0 || v->edge_index[0] != 0)) return fail(GTM_ERR_ARG, "node_index[0] and edge_index[0] must be 0");
    // large sets are checked by a few threads side by side (the arrays are only read)
    const int64_t span = g_hi - g_lo;
    const int workers = (int)std::max<int64_t>(1, std::min<int64_t>(8, span / (1 << 18)));
    std::vector<GraphChecks> parts((size_t)workers);
    if (workers == 1) {
        check_graph_span(v, g_lo, g_hi, &parts[0]);
    } else {
        std::vector<std::thread> threads;
        for (int w = 0; w < workers; ++w)
            threads.emplace_back(check_graph_span, v, g_lo + span * w / workers, g_lo + span * (w + 1) / workers, &parts[(size_t)w]);
        for (std::thread &t : threads) t.join();
    }
    GraphChecks all;
    for (const GraphChecks &c : parts) {
        all.bad_count |= c.bad_count; all.bad_index |= c.bad_index; all.bad_edges |= c.bad_edges;
        all.n_min = std::min(all.n_min, c.n_min); all.n_max = std::max(all.n_max, c.n_max);
    }
    if (all.bad_count) return fail(GTM_ERR_ARG, "a graph has no nodes or more than max_number_of_graph_nodes = %d", v->max_number_of_graph_nodes);
    if (all.bad_index) return fail(GTM_ERR_ARG, "node_index is not the running sum of number_of_graph_nodes (or exceeds total_nodes)");
    if (all.bad_edges) return fail(GTM_ERR_ARG, "edge_index is not the running sum of number_of_graph_node_edges (or exceeds total_edges)");
    if (n_min_out) *n_min_out = all.n_min;
    if (n_max_out) *n_max_out = all.n_max;
    return GTM_OK;
}

static int check_view(const gtm_graphs_view *v)
{
    if (!v) return fail(GTM_ERR_ARG, "null argument");
    if (v->number_of_graphs < 1 || v->total_nodes < 1) return fail(GTM_ERR_ARG, "empty graph set");
    if (!v->X || !v->node_type || !v->number_of_graph_node_edges || !v->edge_index || !v->node_index || !v->number_of_graph_nodes)
        return fail(GTM_ERR_ARG, "graph arrays must not be null");
    if (v->total_edges < 0 || (v->total_edges > 0 && !v->edge)) return fail(GTM_ERR_ARG, "edge array is null but total_edges > 0");
    if (v->max_number_of_graph_nodes < 1) return fail(GTM_ERR_ARG, "max_number_of_graph_nodes must be positive");
    if (v->total_nodes >= (int64_t)1 << 31 || v->total_edges >= (int64_t)1 << 31)
        return fail(GTM_ERR_ARG, "graph sets beyond 2^31 nodes or edges are not supported");
    if (v->number_of_graphs > v->total_nodes) return fail(GTM_ERR_ARG, "more graphs than nodes");
    return GTM_OK;
}

extern "C" int gtm_validate_graphs(const gtm_graphs_view *v)
{
    GTM_TRY(check_view(v));
    return validate_graphs(v, 0, v->number_of_graphs);
}

// copy_arrays == false: the per-node and per-graph arrays are only allocated; the caller copies them in pieces
// (gtm_dataset_create_scored).
static int dataset_build(gtm_model *m, const gtm_graphs_view *v, gtm_dataset *ds, bool copy_arrays = true)
{
    const DevModel &d = m->dm;
    cudaStream_t s = m->stream;
    // the tile kernel fetches literal rows with bulk copies widened to 16-byte boundaries: a little slack at the end
    GTM_TRY(upload(ds, &ds->dg.X, v->X, (size_t)v->total_nodes * d.L0, s, copy_arrays, 4));
    GTM_TRY(upload(ds, &ds->dg.node_type, v->node_type, (size_t)v->total_nodes, s, copy_arrays));
    GTM_TRY(upload(ds, &ds->dg.degree, v->number_of_graph_node_edges, (size_t)v->total_nodes, s, copy_arrays));
    GTM_TRY(upload(ds, &ds->dg.edge_index, v->edge_index, (size_t)v->total_nodes, s, copy_arrays));
    GTM_TRY(upload(ds, &ds->dg.edge, v->edge, 2 * (size_t)v->total_edges, s, copy_arrays));
    GTM_TRY(upload(ds, &ds->dg.node_index, v->node_index, (size_t)v->number_of_graphs, s, copy_arrays));
    GTM_TRY(upload(ds, &ds->dg.n_nodes, v->number_of_graph_nodes, (size_t)v->number_of_graphs, s, copy_arrays));
    {   // first edge row and number of edge rows of every graph (graphs own consecutive CSR rows): derived on the device
        u32 *e0, *ne;
        GTM_TRY(scratch(ds, &e0, (size_t)v->number_of_graphs));
        GTM_TRY(scratch(ds, &ne, (size_t)v->number_of_graphs));
        ds->dg.graph_edge0 = e0;
        ds->dg.graph_edges = ne;
        if (copy_arrays) GTM_TRY(derive_edge_ranges(ds, v->number_of_graphs));      // else: once the caller has copied the arrays
    }
    ds->dg.n_types = 1;
    ds->dg.total_nodes = (u32)v->total_nodes; ds->dg.total_edges = (u32)v->total_edges;
    ds->dg.max_nodes = ds->max_nodes; ds->dg.error = m->score_error;

    // learning scratch
    const size_t p_words = (size_t)std::max(1, d.D - 1) * ds->max_nodes * d.MW;
    ds->fit_sc.NC = ds->NC; ds->fit_sc.cno_slots = d.D; ds->fit_sc.max_nodes = ds->max_nodes;
    GTM_TRY(scratch(ds, &ds->fit_sc.cno, (size_t)d.D * d.C * ds->NC));
    GTM_TRY(scratch(ds, &ds->fit_sc.n_inc, (size_t)d.C));
    GTM_TRY(scratch(ds, &ds->P_pair[0], p_words));
    GTM_TRY(scratch(ds, &ds->P_pair[1], p_words));
    GTM_TRY(scratch(ds, &ds->Q_pair[0], p_words));
    GTM_TRY(scratch(ds, &ds->Q_pair[1], p_words));
    GTM_TRY(scratch(ds, &ds->rank_barrier, 64));
    ds->fit_sc.P = ds->P_pair[0];

    // general scoring scratch: one slice per resident CTA
    // General scoring kernel, shared memory per CTA: vote partial; for depth > 1 the source-node message bits of a graph
    // (flush_messages) when they are small enough not to cost resident CTAs; for graph sets of 33..1024 nodes per graph the
    // transposed copy of the graph - and then the message bits too (up to 64 KB), in CTAs of 512 threads, one or two per SM.
    ds->score_part_words = 0;
    ds->score_t_stride = 0;
    ds->score_block = 256;
    ds->score_smem = (size_t)((d.K + 3) & ~3) * sizeof(int);
    const size_t msg_bytes = (size_t)(((ds->max_nodes + 31) & ~31) + kTransposedTypes) * (d.MW | 1) * sizeof(u32);   // padded rows + per-type rows, see ScatterTargets
    {
        const int t_stride = ds->NC | 1;
        const size_t t_bytes = ((size_t)32 * std::max(d.L0, d.MW) + kTransposedTypes) * t_stride * sizeof(u32);
        if (ds->max_nodes > 32 && ds->NC <= 32 && t_bytes <= 96 * 1024) {
            ds->score_t_stride = t_stride;
            ds->score_smem += t_bytes;
            ds->score_block = 512;
        }
    }
    if (d.D > 1 && (msg_bytes <= 8 * 1024 || (ds->score_t_stride > 0 && msg_bytes <= 72 * 1024))) {
        ds->score_part_words = (int)(msg_bytes / sizeof(u32));
        ds->score_smem += msg_bytes;
    }
    // small models on small graphs: a warp per graph, eight graphs per CTA (score_small_graphs_kernel)
    ds->score_units = 1;
    if (ds->max_nodes <= 32 && d.C <= 128) {
        const size_t per_warp = ((size_t)((d.K + 3) & ~3) + ds->score_part_words) * sizeof(int);
        if (8 * per_warp <= 40 * 1024) {
            ds->score_units = 8;
            ds->score_smem = 8 * per_warp;
        }
    }
    if (ds->score_smem > 48 * 1024)
        GTM_CU(cudaFuncSetAttribute(score_kernel_for(ds->max_nodes), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ds->score_smem));
    int per_sm = 0;
    GTM_CU(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, score_kernel_for(ds->max_nodes, ds->score_units), ds->score_block, ds->score_smem));
    ds->score_grid = (int)std::max<int64_t>(1, std::min<int64_t>((int64_t)m->sm_count * std::max(1, per_sm), v->number_of_graphs));
    ds->cno_stride = (size_t)2 * d.C * ds->NC;
    ds->P_stride = p_words;
    ds->ninc_stride = (size_t)d.C;
    ds->score_sc.NC = ds->NC; ds->score_sc.cno_slots = 2; ds->score_sc.max_nodes = ds->max_nodes;
    ds->score_sc.cno = nullptr;   // allocated on first use of the general kernel (ensure_score_scratch)

    GTM_TRY(stream_data_create(&ds->sd, m->sm, d, ds->dg, v, m->sm_count, s));
    // tiles of whole graphs for the tile kernel: deeper models, or sets the node-stream kernel does not cover
    if (d.D > 1 || !ds->sd.supported || m->opt_score_kernel == 3) GTM_TRY(tile_data_create(&ds->td, m->tm, d, v, ds->n_min, ds->n_max, m->sm_count, s));
    GTM_CU(cudaStreamSynchronize(s));
    return GTM_OK;
}

static int dataset_create(gtm_model *m, const gtm_graphs_view *v, gtm_dataset **out, bool copy_arrays)
{
    GTM_TRY(bind(m));
    if (!v || !out) return fail(GTM_ERR_ARG, "null argument");
    *out = nullptr;
    GTM_TRY(check_view(v));
    gtm_dataset *ds = new (std::nothrow) gtm_dataset();
    if (!ds) return fail(GTM_ERR_OOM, "host allocation failed");
    ds->model = m;
    ds->n_graphs = v->number_of_graphs; ds->total_nodes = v->total_nodes; ds->total_edges = v->total_edges;
    ds->max_nodes = v->max_number_of_graph_nodes;
    ds->NC = words_for(ds->max_nodes);
    // the pipelined caller validates chunk by chunk, just before each chunk is copied
    int st = copy_arrays ? validate_graphs(v, 0, v->number_of_graphs, &ds->n_min, &ds->n_max) : GTM_OK;
    if (st == GTM_OK) st = dataset_build(m, v, ds, copy_arrays);
    if (st != GTM_OK) { gtm_dataset_destroy(ds); return st; }
    *out = ds;
    return GTM_OK;
}

extern "C" int gtm_dataset_create(gtm_model *m, const gtm_graphs_view *v, gtm_dataset **out)
{
    return dataset_create(m, v, out, true);
}

extern "C" int gtm_dataset_destroy(gtm_dataset *ds)
{
    if (!ds) return GTM_OK;
    cudaSetDevice(ds->model->cfg.device);
    cudaStreamSynchronize(ds->model->stream);
    for (void *p : ds->owned) cudaFreeAsync(p, ds->model->stream);
    cudaFree(ds->Y);
    stream_data_destroy(&ds->sd);
    tile_data_destroy(&ds->td);
    fit_comm_release(ds);
    delete ds;
    return GTM_OK;
}

// ---------------------------------------------------------------------------------------------- scoring
static int check_range(gtm_model *m, gtm_dataset *ds, int n_types, int64_t first, int64_t count)
{
    if (!ds || ds->model != m) return fail(GTM_ERR_ARG, "dataset does not belong to this model");
    if (!m->has_state) return fail(GTM_ERR_STATE, "model has no state: call gtm_init_state or gtm_set_ta_state first");
    if (n_types < 1) return fail(GTM_ERR_ARG, "number_of_node_types must be positive");
    if (first < 0 || count < 0 || first + count > ds->n_graphs)
        return fail(GTM_ERR_ARG, "graph range [%lld, %lld) outside the set of %lld graphs", (long long)first,
                    (long long)(first + count), (long long)ds->n_graphs);
    return GTM_OK;
}

// What the word that scoring kernels raise means to the caller (cleared once it was seen).
static int score_flag_status(gtm_model *m, int flag)
{
    if (flag == 0) return GTM_OK;
    cudaMemsetAsync(m->score_error, 0, sizeof(int), m->stream);
    if (flag == 2) return fail(GTM_ERR_TIMEOUT, "a scoring kernel gave up waiting for a bulk copy into shared memory; the class sums are not valid");
    return fail(GTM_ERR_ARG, "a scoring kernel skipped a malformed graph (node count or node range out of bounds)");
}

static int ensure_score_scratch(gtm_dataset *ds)
{
    if (ds->score_sc.cno) return GTM_OK;
    const size_t slices = (size_t)ds->score_grid * ds->score_units;     // one slice per graph in flight
    GTM_TRY(scratch(ds, &ds->score_sc.cno, ds->cno_stride * slices));
    GTM_TRY(scratch(ds, &ds->score_sc.P, ds->P_stride * slices));
    GTM_TRY(scratch(ds, &ds->score_sc.n_inc, ds->ninc_stride * slices));
    return GTM_OK;
}

static int launch_score_general(gtm_model *m, gtm_dataset *ds, int n_types, int64_t first, int64_t count,
                                int *sums_dev, int *clause_out_dev, int *node_out_dev = nullptr, int node_stride = 0)
{
    GTM_TRY(ensure_score_scratch(ds));
    DevGraphs g = ds->dg;
    g.n_types = n_types;
    ScoreArgs a;
    a.first = first; a.count = count; a.class_sums = sums_dev; a.clause_outputs = clause_out_dev;
    a.node_outputs = node_out_dev; a.node_stride = node_stride;
    a.cno_stride = ds->cno_stride; a.P_stride = ds->P_stride; a.ninc_stride = ds->ninc_stride;
    a.part_words = ds->score_part_words; a.t_stride = ds->score_t_stride;
    const int grid = (int)std::min<int64_t>(ds->score_grid, (count + ds->score_units - 1) / ds->score_units);
    {
        DevModel dm = m->dm;
        EvalScratch sc = ds->score_sc;
        void *args[] = {&dm, &g, &sc, &a};
        GTM_CU(cudaLaunchKernel(score_kernel_for(ds->max_nodes, ds->score_units), dim3(grid), dim3(ds->score_block), args, ds->score_smem, m->stream));
    }
    GTM_CU(cudaGetLastError());
    return GTM_OK;
}

static int refresh_lists(gtm_model *m)
{
    if (!m->lists_dirty) return GTM_OK;
    GTM_TRY(stream_model_refresh(&m->sm, m->dm, m->stream));
    m->lists_dirty = false;
    return GTM_OK;
}

static int refresh_tile_lists(gtm_model *m)
{
    if (m->tile_lists_version == m->state_version) return GTM_OK;
    GTM_TRY(tile_model_refresh(&m->tm, m->dm, m->stream));
    m->tile_lists_version = m->state_version;
    return GTM_OK;
}

extern "C" int gtm_score_device(gtm_model *m, gtm_dataset *ds, int n_types, int64_t first, int64_t count,
                                int32_t *sums_dev)
{
    GTM_TRY(bind(m));
    GTM_TRY(check_range(m, ds, n_types, first, count));
    if (count == 0) return GTM_OK;
    if (!sums_dev) return fail(GTM_ERR_ARG, "class_sums_device is null");
    if (m->opt_score_kernel == 2 && !stream_supported(ds->sd, n_types))
        return fail(GTM_ERR_ARG, "the node-stream scoring kernel does not cover this model / graph set");
    if (m->opt_score_kernel == 3 && !tile_supported(ds->td, n_types))
        return fail(GTM_ERR_ARG, "the tile scoring kernel does not cover this model / graph set");
    if ((m->opt_score_kernel == 0 || m->opt_score_kernel == 2) && stream_supported(ds->sd, n_types)) {
        GTM_TRY(refresh_lists(m));
        return stream_score(m->sm, ds->sd, m->dm, ds->dg, n_types, first, count, sums_dev, m->stream);
    }
    if ((m->opt_score_kernel == 0 || m->opt_score_kernel == 3) && tile_supported(ds->td, n_types)) {
        GTM_TRY(refresh_tile_lists(m));
        return tile_score(m->tm, ds->td, m->dm, ds->dg, n_types, first, count, sums_dev, m->score_error, m->stream);
    }
    return launch_score_general(m, ds, n_types, first, count, sums_dev, nullptr);
}

extern "C" int gtm_score(gtm_model *m, gtm_dataset *ds, int n_types, int64_t first, int64_t count, int32_t *out)
{
    GTM_TRY(bind(m));
    GTM_TRY(check_range(m, ds, n_types, first, count));
    if (count == 0) return GTM_OK;
    if (!out) return fail(GTM_ERR_ARG, "class_sums_out is null");
    int *dev;
    GTM_TRY(pool_alloc(&dev, (size_t)count * m->dm.K, m->stream));
    int st = gtm_score_device(m, ds, n_types, first, count, dev);
    cudaError_t e = cudaSuccess;
    if (st == GTM_OK) e = cudaMemcpyAsync(out, dev, (size_t)count * m->dm.K * sizeof(int), cudaMemcpyDeviceToHost, m->stream);
    cudaFreeAsync(dev, m->stream);
    if (st == GTM_OK && e == cudaSuccess) e = cudaMemcpyAsync(m->flag_host, m->score_error, sizeof(int), cudaMemcpyDeviceToHost, m->stream);
    if (st == GTM_OK && e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    if (st != GTM_OK) return st;
    GTM_CU(e);
    return score_flag_status(m, *m->flag_host);
}

// Upload and scoring of a whole host graph set in one call.  Sets that the node-stream kernel or the tile kernel covers
// are pipelined: the graph arrays go up in chunks of whole tiles (two full waves of thread blocks) on a copy stream - a
// chunk is the literal rows, per-node arrays and edge rows of a contiguous range of graphs - each chunk is scored as soon
// as it has landed, and its class sums go back on a second copy stream while the next chunk is scored.  Host arrays are
// validated chunk by chunk, just before they are copied.  Other sets take gtm_dataset_create followed by gtm_score.
// The dataset stays valid for later calls either way.
extern "C" int gtm_dataset_create_scored(gtm_model *m, const gtm_graphs_view *v, int n_types, int32_t *out,
                                         gtm_dataset **dataset_out)
{
    GTM_TRY(bind(m));
    if (!v || !out || !dataset_out) return fail(GTM_ERR_ARG, "null argument");
    *dataset_out = nullptr;
    if (!m->has_state) return fail(GTM_ERR_STATE, "model has no state: call gtm_init_state or gtm_set_ta_state first");
    if (n_types < 1) return fail(GTM_ERR_ARG, "number_of_node_types must be positive");
    GTM_TRY(check_view(v));
    // what a tiled kernel may cover; stream_supported / tile_supported decide once the tiles are made
    const bool pipelined = m->opt_score_kernel != 1 && n_types <= 8 && v->max_number_of_graph_nodes <= 1024 &&
                           (m->sm.lit_off != nullptr || m->tm.applicable);
    gtm_dataset *ds = nullptr;
    GTM_TRY(dataset_create(m, v, &ds, !pipelined));
    const int64_t n = ds->n_graphs;
    int st = GTM_OK;
    const bool by_stream = pipelined && (m->opt_score_kernel == 0 || m->opt_score_kernel == 2) && stream_supported(ds->sd, n_types);
    const bool by_tile = pipelined && !by_stream && (m->opt_score_kernel == 0 || m->opt_score_kernel == 3) && tile_supported(ds->td, n_types);
    if (!by_stream && !by_tile) {
        if (pipelined) {   // the arrays were not copied, but no tiled kernel turned out to cover the set
            gtm_dataset_destroy(ds);
            ds = nullptr;
            GTM_TRY(dataset_create(m, v, &ds, true));
        }
        st = gtm_score(m, ds, n_types, 0, n, out);
        if (st != GTM_OK) { gtm_dataset_destroy(ds); return st; }
        *dataset_out = ds;
        return GTM_OK;
    }

    const DevModel &d = m->dm;
    // tiles of the kernel that will run: first graph of tile t
    const int n_tiles = by_stream ? ds->sd.n_tiles : ds->td.n_tiles;
    const int uniform_gpt = by_stream ? ds->sd.graphs_per_tile : ds->td.graphs_per_tile;
    const std::vector<int> &table = by_stream ? ds->sd.tile_graph_host : ds->td.tile_graph_host;
    auto tile_first = [&](int t) -> int64_t {
        if (t >= n_tiles) return n;
        return uniform_gpt > 0 ? std::min<int64_t>((int64_t)t * uniform_gpt, n) : (int64_t)table[(size_t)t];
    };
    const int chunk_tiles = std::max(1, 2 * (by_stream ? ds->sd.grid : ds->td.grid));
    cudaStream_t in = nullptr, back = nullptr;
    std::vector<cudaEvent_t> events;
    int *dev = nullptr;
    auto body = [&]() -> int {
        GTM_CU(cudaStreamCreateWithFlags(&in, cudaStreamNonBlocking));
        GTM_CU(cudaStreamCreateWithFlags(&back, cudaStreamNonBlocking));
        if (by_stream) GTM_TRY(refresh_lists(m));
        else GTM_TRY(refresh_tile_lists(m));
        GTM_TRY(pool_alloc(&dev, (size_t)n * d.K, m->stream));
        auto event = [&](cudaStream_t s, cudaEvent_t *e) -> int {
            GTM_CU(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
            events.push_back(*e);
            GTM_CU(cudaEventRecord(*e, s));
            return GTM_OK;
        };
        auto up = [&](const u32 *dst, const u32 *src, size_t first, size_t count) -> int {
            if (count) GTM_CU(cudaMemcpyAsync(const_cast<u32 *>(dst) + first, src + first, count * sizeof(u32), cudaMemcpyHostToDevice, in));
            return GTM_OK;
        };
        cudaEvent_t ready;
        GTM_TRY(event(m->stream, &ready));                 // allocations, tile tables and literal lists are in stream order
        GTM_CU(cudaStreamWaitEvent(in, ready, 0));
        for (int t0 = 0; t0 < n_tiles; t0 += chunk_tiles) {
            const int64_t g0 = tile_first(t0), g1 = tile_first(t0 + chunk_tiles);
            if (g1 <= g0) continue;
            GTM_TRY(validate_graphs(v, g0, g1));            // overlaps the copies of the chunks before
            const size_t cnt = (size_t)(g1 - g0);
            const size_t v0 = v->node_index[g0], v1 = g1 < n ? (size_t)v->node_index[g1] : (size_t)v->total_nodes;
            const size_t e0 = v->edge_index[v0], e1 = v1 < (size_t)v->total_nodes ? (size_t)v->edge_index[v1] : (size_t)v->total_edges;
            GTM_TRY(up(ds->dg.X, v->X, v0 * d.L0, (v1 - v0) * d.L0));
            GTM_TRY(up(ds->dg.node_type, v->node_type, v0, v1 - v0));
            GTM_TRY(up(ds->dg.degree, v->number_of_graph_node_edges, v0, v1 - v0));
            GTM_TRY(up(ds->dg.edge_index, v->edge_index, v0, v1 - v0));
            if (e1 > e0) GTM_TRY(up(ds->dg.edge, v->edge, 2 * e0, 2 * (e1 - e0)));
            // one element more: a tile ends where the next graph's nodes begin
            GTM_TRY(up(ds->dg.node_index, v->node_index, (size_t)g0, cnt + (g1 < n ? 1 : 0)));
            GTM_TRY(up(ds->dg.n_nodes, v->number_of_graph_nodes, (size_t)g0, cnt));
            cudaEvent_t landed, scored;
            GTM_TRY(event(in, &landed));
            GTM_CU(cudaStreamWaitEvent(m->stream, landed, 0));
            if (by_stream) GTM_TRY(stream_score(m->sm, ds->sd, d, ds->dg, n_types, g0, (int64_t)cnt, dev + (size_t)g0 * d.K, m->stream));
            else GTM_TRY(tile_score(m->tm, ds->td, d, ds->dg, n_types, g0, (int64_t)cnt, dev + (size_t)g0 * d.K, m->score_error, m->stream));
            GTM_TRY(event(m->stream, &scored));
            GTM_CU(cudaStreamWaitEvent(back, scored, 0));
            GTM_CU(cudaMemcpyAsync(out + (size_t)g0 * d.K, dev + (size_t)g0 * d.K, cnt * d.K * sizeof(int), cudaMemcpyDeviceToHost, back));
        }
        GTM_TRY(derive_edge_ranges(ds, v->number_of_graphs));       // every array has been queued before this point of the stream
        GTM_CU(cudaMemcpyAsync(m->flag_host, m->score_error, sizeof(int), cudaMemcpyDeviceToHost, m->stream));
        GTM_CU(cudaStreamSynchronize(in));
        GTM_CU(cudaStreamSynchronize(back));
        GTM_CU(cudaStreamSynchronize(m->stream));
        return score_flag_status(m, *m->flag_host);
    };
    st = body();
    if (st != GTM_OK) {                                    // nothing may still be reading the host arrays when the call returns
        if (in) cudaStreamSynchronize(in);
        if (back) cudaStreamSynchronize(back);
        cudaStreamSynchronize(m->stream);
    }
    if (dev) cudaFreeAsync(dev, m->stream);
    for (cudaEvent_t e : events) cudaEventDestroy(e);
    if (in) cudaStreamDestroy(in);
    if (back) cudaStreamDestroy(back);
    if (st != GTM_OK) { gtm_dataset_destroy(ds); return st; }
    *dataset_out = ds;
    return GTM_OK;
}

// clause outputs per graph and / or per node through the general scoring kernel; results land in host arrays
static int transform_common(gtm_model *m, gtm_dataset *ds, int n_types, int64_t first, int64_t count, int32_t *clause_out,
                            int32_t *node_out, int node_stride, int32_t *sums_out)
{
    GTM_TRY(bind(m));
    GTM_TRY(check_range(m, ds, n_types, first, count));
    if (count == 0) return GTM_OK;
    int *sums_dev = nullptr, *co_dev = nullptr, *no_dev = nullptr;
    const size_t n_sums = (size_t)count * m->dm.K, n_co = (size_t)count * m->dm.C, n_no = n_co * (size_t)node_stride;
    int st = pool_alloc(&sums_dev, n_sums, m->stream);
    if (st == GTM_OK && clause_out) st = pool_alloc(&co_dev, n_co, m->stream);
    if (st == GTM_OK && node_out) st = pool_alloc(&no_dev, n_no, m->stream);
    if (st == GTM_OK) st = launch_score_general(m, ds, n_types, first, count, sums_dev, co_dev, no_dev, node_stride);
    cudaError_t e = cudaSuccess;
    if (st == GTM_OK && sums_out) e = cudaMemcpyAsync(sums_out, sums_dev, n_sums * sizeof(int), cudaMemcpyDeviceToHost, m->stream);
    if (st == GTM_OK && e == cudaSuccess && clause_out) e = cudaMemcpyAsync(clause_out, co_dev, n_co * sizeof(int), cudaMemcpyDeviceToHost, m->stream);
    if (st == GTM_OK && e == cudaSuccess && node_out) e = cudaMemcpyAsync(node_out, no_dev, n_no * sizeof(int), cudaMemcpyDeviceToHost, m->stream);
    if (sums_dev) cudaFreeAsync(sums_dev, m->stream);
    if (co_dev) cudaFreeAsync(co_dev, m->stream);
    if (no_dev) cudaFreeAsync(no_dev, m->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    if (st != GTM_OK) return st;
    GTM_CU(e);
    return GTM_OK;
}

extern "C" int gtm_transform(gtm_model *m, gtm_dataset *ds, int n_types, int64_t first, int64_t count,
                             int32_t *clause_out, int32_t *sums_out)
{
    return transform_common(m, ds, n_types, first, count, clause_out, nullptr, 0, sums_out);
}

extern "C" int gtm_transform_nodewise(gtm_model *m, gtm_dataset *ds, int n_types, int64_t first, int64_t count,
                                      int node_stride, int32_t *node_out, int32_t *sums_out)
{
    if (!node_out) return fail(GTM_ERR_ARG, "node_outputs_out is null");
    if (!ds || node_stride < ds->max_nodes) return fail(GTM_ERR_ARG, "node_stride must be at least the largest graph's node count");
    return transform_common(m, ds, n_types, first, count, nullptr, node_out, node_stride, sums_out);
}

// --------------------------------------------------------------------------------------------- learning
extern "C" int gtm_fit(gtm_model *m, gtm_dataset *ds, int n_types, const int32_t *Y, int64_t first, int64_t count, int epochs)
{
    GTM_TRY(bind(m));
    GTM_TRY(check_range(m, ds, n_types, first, count));
    if (!Y) return fail(GTM_ERR_ARG, "encoded_Y is null");
    if (epochs < 0) return fail(GTM_ERR_ARG, "epochs must not be negative");
    if (count == 0 || epochs == 0) return GTM_OK;
    const size_t need = (size_t)ds->n_graphs * m->dm.K;
    if (ds->Y_capacity < need) {
        cudaFree(ds->Y); ds->Y = nullptr; ds->Y_capacity = 0;
        GTM_TRY(dev_alloc(&ds->Y, need));
        ds->Y_capacity = need;
    }
    GTM_CU(cudaMemcpyAsync(ds->Y + (size_t)first * m->dm.K, Y + (size_t)first * m->dm.K,
                           (size_t)count * m->dm.K * sizeof(int), cudaMemcpyHostToDevice, m->stream));
    m->lists_dirty = true; ++m->state_version;
    return launch_fit(m, ds, n_types, ds->Y, first, count, epochs, 0);
}

// ------------------------------------------------------------------------------------------------- taps
extern "C" int gtm_debug_evaluate(gtm_model *m, gtm_dataset *ds, int n_types, int64_t graph, int path,
                                  uint32_t *cno_out, uint32_t *msg_out, int32_t *n_inc_out, int32_t *class_sum_out)
{
    GTM_TRY(bind(m));
    GTM_TRY(check_range(m, ds, n_types, graph, 1));
    const DevModel &d = m->dm;
    std::vector<u32> nn(1), ni(1);
    GTM_CU(cudaMemcpy(nn.data(), ds->dg.n_nodes + graph, sizeof(u32), cudaMemcpyDeviceToHost));
    const int n = (int)nn[0], words = (n + 31) / 32;
    if (path == 1) {
        GTM_TRY(launch_fit(m, ds, n_types, nullptr, graph, 1, 1, 1));
        if (cno_out)
            for (int l = 0; l < d.D; ++l)
                GTM_CU(cudaMemcpy2D(cno_out + (size_t)l * d.C * words, words * sizeof(u32),
                                    ds->fit_sc.cno + (size_t)l * d.C * ds->NC, ds->NC * sizeof(u32),
                                    words * sizeof(u32), d.C, cudaMemcpyDeviceToHost));
        if (msg_out && d.D > 1) {
            u32 *tmp;
            GTM_TRY(dev_alloc(&tmp, (size_t)n * d.M));
            for (int l = 0; l < d.D - 1; ++l) {
                expand_messages_kernel<<<64, 256, 0, m->stream>>>(ds->P_pair[0] + (size_t)l * ds->max_nodes * d.MW, tmp, n, d.MS, d.MW, d.M);
                cudaMemcpyAsync(msg_out + (size_t)l * n * d.M, tmp, (size_t)n * d.M * sizeof(u32), cudaMemcpyDeviceToHost, m->stream);
            }
            cudaError_t e = cudaStreamSynchronize(m->stream);
            cudaFree(tmp);
            GTM_CU(e);
        }
        if (n_inc_out) GTM_CU(cudaMemcpy(n_inc_out, ds->fit_sc.n_inc, (size_t)d.C * sizeof(int), cudaMemcpyDeviceToHost));
        if (class_sum_out) GTM_CU(cudaMemcpy(class_sum_out, m->class_sum_tap, (size_t)d.K * sizeof(int), cudaMemcpyDeviceToHost));
        return GTM_OK;
    }
    if (path == 0) {
        // general scoring kernel with a one-CTA grid and every layer kept (scratch of the learning kernel)
        DevGraphs g = ds->dg;
        g.n_types = n_types;
        int *sums;
        GTM_TRY(dev_alloc(&sums, (size_t)d.K));
        ScoreArgs a;
        a.first = graph; a.count = 1; a.class_sums = sums; a.clause_outputs = nullptr; a.node_outputs = nullptr; a.node_stride = 0;
        a.cno_stride = a.P_stride = a.ninc_stride = 0;
        a.part_words = 0; a.t_stride = 0;
        EvalScratch sc = ds->fit_sc;
        sc.P = ds->P_pair[0];
        score_graphs_kernel<true><<<1, 256, (size_t)d.K * sizeof(int), m->stream>>>(d, g, sc, a);
        cudaError_t e = cudaStreamSynchronize(m->stream);
        if (e == cudaSuccess && class_sum_out) e = cudaMemcpy(class_sum_out, sums, (size_t)d.K * sizeof(int), cudaMemcpyDeviceToHost);
        cudaFree(sums);
        GTM_CU(e);
        if (cno_out)
            for (int l = 0; l < d.D; ++l)
                GTM_CU(cudaMemcpy2D(cno_out + (size_t)l * d.C * words, words * sizeof(u32),
                                    ds->fit_sc.cno + (size_t)l * d.C * ds->NC, ds->NC * sizeof(u32),
                                    words * sizeof(u32), d.C, cudaMemcpyDeviceToHost));
        if (msg_out && d.D > 1) {
            u32 *tmp;
            GTM_TRY(dev_alloc(&tmp, (size_t)n * d.M));
            for (int l = 0; l < d.D - 1; ++l) {
                expand_messages_kernel<<<64, 256, 0, m->stream>>>(ds->P_pair[0] + (size_t)l * ds->max_nodes * d.MW, tmp, n, d.MS, d.MW, d.M);
                cudaMemcpyAsync(msg_out + (size_t)l * n * d.M, tmp, (size_t)n * d.M * sizeof(u32), cudaMemcpyDeviceToHost, m->stream);
            }
            e = cudaStreamSynchronize(m->stream);
            cudaFree(tmp);
            GTM_CU(e);
        }
        if (n_inc_out) GTM_CU(cudaMemcpy(n_inc_out, ds->fit_sc.n_inc, (size_t)d.C * sizeof(int), cudaMemcpyDeviceToHost));
        return GTM_OK;
    }
    return fail(GTM_ERR_ARG, "path must be 0 (scoring kernel) or 1 (learning kernel)");
}

// Eight independent chains of three-input logic operations per thread, all in registers.
__global__ void __launch_bounds__(256) logic_op_rate_kernel(int iterations, u32 seed, u32 *sink)
{
    u32 x[8], a = seed ^ (threadIdx.x * 2654435761u), b = seed + blockIdx.x * 40503u;
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = a * (2 * i + 3) + b;
    for (int it = 0; it < iterations; ++it) {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
#pragma unroll
            for (int i = 0; i < 8; ++i)                                       // one LOP3 each (bitwise select), chains independent of one another
                asm volatile("lop3.b32 %0, %0, %1, %2, 0xCA;" : "+r"(x[i]) : "r"(a), "r"(b));
        }
    }
    u32 v = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) v ^= x[i];
    if (v == 0x12345u) sink[0] = v;                                           // keeps the chains alive
}

extern "C" int gtm_debug_logic_op_rate(gtm_model *m, double *tera_ops_per_second_out)
{
    if (!m || !tera_ops_per_second_out) return fail(GTM_ERR_ARG, "null argument");
    GTM_TRY(bind(m));
    u32 *sink = nullptr;
    GTM_TRY(dev_alloc(&sink, 1));
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    const int iterations = 4096, grid = m->sm_count * 16;
    float ms = 0.0f;
    for (int rep = 0; rep < 3; ++rep) {          // the last repetition is the one reported
        cudaEventRecord(e0, m->stream);
        logic_op_rate_kernel<<<grid, 256, 0, m->stream>>>(iterations, 1u + rep, sink);
        cudaEventRecord(e1, m->stream);
        cudaEventSynchronize(e1);
        cudaEventElapsedTime(&ms, e0, e1);
    }
    cudaError_t e = cudaGetLastError();
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(sink);
    GTM_CU(e);
    *tera_ops_per_second_out = (double)grid * 256.0 * iterations * 64.0 / (ms * 1e-3) / 1e12;
    return GTM_OK;
}

extern "C" int gtm_debug_fit_phase_cycles(gtm_model *m, uint64_t *cycles_out)
{
    GTM_TRY(bind(m));
    if (!cycles_out) return fail(GTM_ERR_ARG, "cycles_out is null");
    GTM_CU(cudaStreamSynchronize(m->stream));
    GTM_CU(cudaMemcpy(cycles_out, m->phase_cycles, 8 * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    return GTM_OK;
}

extern "C" int gtm_debug_last_feedback(gtm_model *m, int32_t *clause_node_out, int32_t *update_out)
{
    GTM_TRY(bind(m));
    GTM_CU(cudaStreamSynchronize(m->stream));
    if (clause_node_out) GTM_CU(cudaMemcpy(clause_node_out, m->clause_node, (size_t)m->dm.C * sizeof(int), cudaMemcpyDeviceToHost));
    if (update_out) GTM_CU(cudaMemcpy(update_out, m->update, (size_t)m->dm.K * m->dm.C * sizeof(int), cudaMemcpyDeviceToHost));
    return GTM_OK;
}

// ------------------------------------------------------------------------- scoring with built-in scratch
// Scratch of gtm_score_static_scratch: lives in the library image, so every GPU that loads the library holds these
// GTM_STATIC_SCRATCH_BYTES until the process exits.  In host code the name below is only a stand-in for the
// symbol, not a device address; the address is looked up once per device (g_static_scratch_addr).
static __device__ __align__(256) unsigned int g_static_scratch[GTM_STATIC_SCRATCH_BYTES / sizeof(unsigned int)];
static unsigned int *g_static_scratch_addr[64];

extern "C" int gtm_score_static_scratch(gtm_model *m, const gtm_graphs_view *v, int n_types, int64_t first, int64_t count,
                                        int32_t *sums_dev)
{
    GTM_TRY(bind(m));
    if (!v) return fail(GTM_ERR_ARG, "device_graphs is null");
    if (!m->has_state) return fail(GTM_ERR_STATE, "model has no state: call gtm_init_state or gtm_set_ta_state first");
    if (n_types < 1) return fail(GTM_ERR_ARG, "number_of_node_types must be positive");
    if (first < 0 || count < 0 || first + count > v->number_of_graphs)
        return fail(GTM_ERR_ARG, "graph range [%lld, %lld) outside the set of %lld graphs", (long long)first,
                    (long long)(first + count), (long long)v->number_of_graphs);
    if (count == 0) return GTM_OK;
    if (!sums_dev || !v->X || !v->node_type || !v->number_of_graph_node_edges || !v->edge_index || !v->node_index ||
        !v->number_of_graph_nodes || (v->total_edges > 0 && !v->edge))
        return fail(GTM_ERR_ARG, "device arrays must not be null");
    if (v->max_number_of_graph_nodes < 1) return fail(GTM_ERR_ARG, "max_number_of_graph_nodes must be positive");
    if (v->total_nodes < 1 || v->total_nodes >= (int64_t)1 << 31 || v->total_edges < 0 || v->total_edges >= (int64_t)1 << 31)
        return fail(GTM_ERR_ARG, "total_nodes must be in 1..2^31-1 and total_edges in 0..2^31-1");
    // layer-0 rows of a multiple of four words are read with 128-bit loads; every array is read as 32-bit words
    if ((m->dm.L0 & 3) == 0 && ((uintptr_t)v->X & 15) != 0)
        return fail(GTM_ERR_ARG, "X must be 16-byte aligned when a literal row is a multiple of 16 bytes (it is %d bytes here)", m->dm.L0 * 4);
    {
        const void *arrays[] = {v->X, v->node_type, v->number_of_graph_node_edges, v->edge_index, v->edge, v->node_index,
                                v->number_of_graph_nodes, sums_dev};
        for (const void *p : arrays)
            if (((uintptr_t)p & 3) != 0) return fail(GTM_ERR_ARG, "device arrays must be 4-byte aligned");
    }
    const int dev = m->cfg.device;
    if (dev >= 64) return fail(GTM_ERR_ARG, "device ordinal %d beyond the 64 this entry point keeps an address for", dev);

    const DevModel &d = m->dm;
    const int NC = words_for(v->max_number_of_graph_nodes);
    const size_t cno_words = (size_t)2 * d.C * NC;
    const size_t p_words = (size_t)std::max(1, d.D - 1) * v->max_number_of_graph_nodes * d.MW;
    const size_t per_cta = cno_words + p_words + (size_t)d.C;                       // words of scratch one CTA needs
    const size_t capacity = GTM_STATIC_SCRATCH_BYTES / sizeof(unsigned int);
    if (per_cta > capacity)
        return fail(GTM_ERR_ARG,
                    "model and graph sizes need %zu bytes of scratch per thread block; the built-in scratch holds %u bytes "
                    "(use gtm_dataset_create + gtm_score_device for this size)", per_cta * sizeof(unsigned int),
                    (unsigned)GTM_STATIC_SCRATCH_BYTES);

    // first call on this device: resolve the device address of the built-in array (this device is current)
    if (!g_static_scratch_addr[dev]) {
        unsigned int *addr = nullptr;
        GTM_CU(cudaGetSymbolAddress((void **)&addr, g_static_scratch));
        g_static_scratch_addr[dev] = addr;
    }
    unsigned int *scratch_base = g_static_scratch_addr[dev];

    const int64_t fit_ctas = (int64_t)(capacity / per_cta);
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(count, fit_ctas), (int64_t)m->sm_count * 4));

    DevGraphs g;
    memset(&g, 0, sizeof g);
    g.X = v->X; g.node_type = v->node_type; g.degree = v->number_of_graph_node_edges; g.edge_index = v->edge_index;
    g.edge = v->edge; g.node_index = v->node_index; g.n_nodes = v->number_of_graph_nodes;
    g.n_types = n_types;
    // the arrays are in device memory and cannot be checked here: the kernel skips graphs that would leave them or the
    // scratch slice and raises the word that gtm_check_skipped_graphs reads
    g.total_nodes = (u32)v->total_nodes; g.total_edges = (u32)v->total_edges;
    g.max_nodes = v->max_number_of_graph_nodes; g.error = m->score_error;
    EvalScratch sc;
    sc.cno = scratch_base;
    sc.P = scratch_base + cno_words;
    sc.n_inc = reinterpret_cast<int *>(scratch_base + cno_words + p_words);
    sc.NC = NC; sc.cno_slots = 2; sc.max_nodes = v->max_number_of_graph_nodes;
    ScoreArgs a;
    a.first = first; a.count = count; a.class_sums = sums_dev; a.clause_outputs = nullptr; a.node_outputs = nullptr; a.node_stride = 0;
    a.cno_stride = a.P_stride = a.ninc_stride = per_cta;                             // one contiguous slice per CTA
    a.part_words = 0; a.t_stride = 0;
    score_graphs_kernel<true><<<grid, 256, (size_t)d.K * sizeof(int), m->stream>>>(d, g, sc, a);
    GTM_CU(cudaGetLastError());
    return GTM_OK;
}

extern "C" int gtm_check_skipped_graphs(gtm_model *m, int *skipped_out)
{
    GTM_TRY(bind(m));
    if (!skipped_out) return fail(GTM_ERR_ARG, "skipped_out is null");
    GTM_CU(cudaStreamSynchronize(m->stream));
    int flag = 0;
    GTM_CU(cudaMemcpy(&flag, m->score_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (flag) GTM_CU(cudaMemset(m->score_error, 0, sizeof(int)));
    *skipped_out = flag == 1;
    if (flag == 2) return score_flag_status(m, flag);
    return GTM_OK;
}
