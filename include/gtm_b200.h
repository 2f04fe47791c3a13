/* gtm_b200.h — C ABI of the B200-native Graph Tsetlin Machine engine (libgtm_b200.so).
 *
 * This is the seam at which the reference (cair/GraphTsetlinMachine) talks to PyCUDA
 * (GraphTsetlinMachine/tm.py: SourceModule/get_function/prepared_call, cuda.mem_alloc, memcpy_htod/dtoh,
 * Context.synchronize).  Every entry point names the reference interface it replaces.
 *
 * Conventions
 *  - Plain C types only; handles are opaque.  Host pointers are borrowed for the duration of the call.
 *  - Every function returns a gtm_status (0 = OK).  gtm_last_error() gives the message of the calling
 *    thread's last failure.  No exception or exit() crosses this boundary.
 *  - Calls are synchronous on return unless stated otherwise.  A model handle is not thread-safe.
 *  - Array layouts at the boundary are the reference's (see each function); the engine's internal layouts
 *    differ and are converted on the device.
 */
#ifndef GTM_B200_H
#define GTM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GTM_MAX_DEPTH 16
#define GTM_MAX_STATE_BITS 32

typedef enum gtm_status {
    GTM_OK = 0,
    GTM_ERR_ARG = 1,         /* bad argument / unsupported size */
    GTM_ERR_CUDA = 2,        /* a CUDA runtime call failed      */
    GTM_ERR_OOM = 3,         /* device or host allocation failed */
    GTM_ERR_TIMEOUT = 4,     /* a bounded device-side wait (grid barrier) gave up */
    GTM_ERR_STATE = 5        /* call order violated (e.g. score before any state was set) */
} gtm_status;

/* Hyper-parameters.  Mirrors the constants the reference bakes into its kernels at JIT time
 * (tm.py:438-464) plus the constructor arguments of CommonTsetlinMachine (tm.py:39-55). */
typedef struct gtm_config {
    int32_t number_of_clauses;            /* CLAUSES */
    int32_t number_of_outputs;            /* CLASSES */
    int32_t number_of_literals;           /* LITERALS = 2 * hypervector_size */
    int32_t number_of_state_bits;         /* STATE_BITS (1..32) */
    int32_t boost_true_positive_feedback; /* BOOST_TRUE_POSITIVE_FEEDBACK */
    int32_t T;                            /* THRESHOLD */
    int32_t max_included_literals;        /* MAX_INCLUDED_LITERALS */
    int32_t message_size;                 /* MESSAGE_SIZE */
    int32_t message_bits;                 /* MESSAGE_BITS */
    int32_t depth;                        /* number of layers; 1 = no message passing (tm.py:62) */
    int32_t device;                       /* CUDA device ordinal */
    int32_t reserved;
    double q;                             /* Q, already rounded the way the reference's "%f" format does */
    float s[GTM_MAX_DEPTH];               /* specificity per layer (tm.py:63-66) */
    uint64_t seed;                        /* key of the per-clause Philox4x32-10 draw streams */
} gtm_config;

/* A graph set in the array layout produced by GraphTsetlinMachine/graphs.py (Graphs): */
typedef struct gtm_graphs_view {
    const uint32_t *X;                          /* [total_nodes][ceil(literals/32)]  graphs.py:112      */
    const uint32_t *node_type;                  /* [total_nodes]                     graphs.py:107      */
    const uint32_t *number_of_graph_node_edges; /* [total_nodes] out-degrees         graphs.py:108      */
    const uint32_t *edge_index;                 /* [total_nodes] CSR row starts      graphs.py:110,128  */
    const uint32_t *edge;                       /* [total_edges][2] (dst local id, edge type) graphs.py:129 */
    const uint32_t *node_index;                 /* [number_of_graphs] first node     graphs.py:101      */
    const uint32_t *number_of_graph_nodes;      /* [number_of_graphs]                graphs.py:38       */
    int64_t number_of_graphs;
    int64_t total_nodes;
    int64_t total_edges;
    int32_t max_number_of_graph_nodes;
    int32_t reserved;
} gtm_graphs_view;

typedef struct gtm_model gtm_model;
typedef struct gtm_dataset gtm_dataset;

/* Library --------------------------------------------------------------------------------------------- */
const char *gtm_version(void);
const char *gtm_last_error(void);
int gtm_device_count(int *count_out);

/* Model life cycle.  Replaces tm.py:437-513 (_init_gpu_kernels: no JIT here, sizes are run-time values) and
 * tm.py:110-124 (allocate_gpu_memory). */
int gtm_create(const gtm_config *config, gtm_model **model_out);
int gtm_destroy(gtm_model *model);

/* All device work of a model is issued on this CUDA stream (a cudaStream_t passed as void*; NULL = the legacy
 * default stream, which is also the default). */
int gtm_set_stream(gtm_model *model, void *cuda_stream);

/* Kernel selection (the reference has one code path; its only launch knobs are grid/block, tm.py:53-54).
 *   "fit_kernel":   0 = automatic, 1 = learning kernel with state in global memory, 2 = state-resident kernel
 *   "score_kernel": 0 = automatic, 1 = general kernel, 2 = node-stream kernel (depth 1), 3 = tile kernel (any depth,
 *                   graphs of at most 128 nodes); set it before the graph set is created
 *   "fit_timers":   1 = the learning kernels time their phases for gtm_debug_fit_phase_cycles (default 0); 2 and 3 = the
 *                   state-resident kernel splits its evaluation phase instead of its feedback phase (see that function)
 *   "fit_block_clauses": clauses per thread block of the state-resident learning kernel, 0 = automatic (default)
 *   "fit_wait_ms":  wall-time budget of ONE device-side wait of the learning kernels (grid barrier, vote exchange between
 *                   thread blocks or GPUs), 1..600000 ms, default 2000.  A wait that runs out ends the launch; gtm_fit
 *                   returns GTM_ERR_TIMEOUT, the CUDA context stays usable.  The state-resident kernel leaves the model as
 *                   it was before the call; otherwise part of the call's updates may have been applied - restore a
 *                   checkpoint (gtm_set_ta_state / gtm_set_weights / gtm_set_draw_positions) before learning on.
 *   "fit_missing_cta": test hook, 1 = every wait of later gtm_fit calls expects one arrival more than there are thread
 *                   blocks, i.e. a participant that never shows up: the waits run out (default 0)
 * Forcing a kernel that cannot serve the model makes the next fit / score call fail with GTM_ERR_ARG. */
int gtm_set_option(gtm_model *model, const char *name, int value);

/* Replaces the `prepare` launch of tm.py:518,525 (kernels.py:638-664) and, when reset_message_layers != 0,
 * the `prepare_message_ta_state` launches of tm.py:520-521 (kernels.py:622-636): weights +-1 from one draw
 * per (clause, class), every automaton one step below the include boundary. */
int gtm_init_state(gtm_model *model, int reset_message_layers);

/* Tsetlin-automaton state of one layer in the reference's layout uint32[CLAUSES][chunks][STATE_BITS]
 * (layer 0: tm.py:111,283-284; layer d >= 1 = message_ta_state[d-1]: tm.py:113-115,319-323,406-408). */
int gtm_set_ta_state(gtm_model *model, int layer, const uint32_t *ta_state);
int gtm_get_ta_state(gtm_model *model, int layer, uint32_t *ta_state_out);

/* Clause weights int32[CLASSES][CLAUSES] (tm.py:117,285-286,409). */
int gtm_set_weights(gtm_model *model, const int32_t *clause_weights);
int gtm_get_weights(gtm_model *model, int32_t *clause_weights_out);

/* Message hypervectors uint32[CLAUSES][MESSAGE_BITS] (tm.py:123-124). */
int gtm_set_hypervectors(gtm_model *model, const uint32_t *hypervectors);

/* Random draws.  The engine has one counter-based stream per clause in place of the reference's one XORWOW
 * state per launched thread (tm.py:36; kernels.py:199,228,329,369,643).  Positions are the number of draws
 * each clause has consumed.  Recorded draws (uint32[CLAUSES][draws_per_clause], read modulo
 * draws_per_clause) replace the Philox output; pass NULL to go back to Philox.  The buffer is copied. */
int gtm_set_draw_positions(gtm_model *model, const uint64_t *positions);
int gtm_get_draw_positions(gtm_model *model, uint64_t *positions_out);
int gtm_set_recorded_draws(gtm_model *model, const uint32_t *draws, uint64_t draws_per_clause);

/* Graph sets on the device.  Replaces the uploads and scratch allocations of tm.py:528-555 (_init_fit) and
 * tm.py:759-784 (_score_init).  Signature caching stays with the caller.  The arrays must have the layout graphs.py
 * produces -- node_index / edge_index are the running sums of number_of_graph_nodes / number_of_graph_node_edges
 * (graphs.py:101-102,127-128) and every graph has 1..max_number_of_graph_nodes nodes -- otherwise GTM_ERR_ARG. */
int gtm_dataset_create(gtm_model *model, const gtm_graphs_view *graphs, gtm_dataset **dataset_out);
/* The same checks on HOST arrays without a model or a device (GTM_OK or GTM_ERR_ARG with the reason in
 * gtm_last_error).  No counterpart in the reference, whose kernels index whatever they are given. */
int gtm_validate_graphs(const gtm_graphs_view *graphs);
int gtm_dataset_destroy(gtm_dataset *dataset);

/* Replaces the per-graph loop of tm.py:786-812 (_score): raw, unclamped class sums int32[count][CLASSES] for
 * graphs [first, first+count).  number_of_node_types is graphs.number_of_node_types() at call time
 * (tm.py:587).  gtm_score copies the result to host memory; gtm_score_device leaves it in device memory at
 * class_sums_device and returns without synchronising (work is queued on the model's stream). */
int gtm_score(gtm_model *model, gtm_dataset *dataset, int number_of_node_types, int64_t first, int64_t count,
              int32_t *class_sums_out);

/* Upload + scoring of a whole graph set in one call (the reference does both inside `_score`: tm.py:759-784 uploads,
 * tm.py:786-812 scores): class_sums_out int32[number_of_graphs][CLASSES]; *dataset_out is the resident graph set, as
 * from gtm_dataset_create, for later calls.  Sets of single-node graphs are pipelined - chunks are scored while the next
 * chunk is still being copied and the previous chunk's sums are on their way back; page-locked host arrays make the
 * copies asynchronous.  Host pointers are borrowed for the call only. */
int gtm_dataset_create_scored(gtm_model *model, const gtm_graphs_view *graphs, int number_of_node_types,
                              int32_t *class_sums_out, gtm_dataset **dataset_out);
int gtm_score_device(gtm_model *model, gtm_dataset *dataset, int number_of_node_types, int64_t first,
                     int64_t count, int32_t *class_sums_device);

/* Scoring for callers that must not allocate device memory.  NO COUNTERPART IN THE REFERENCE (it allocates per graph
 * set with cuda.mem_alloc, tm.py:759-784).
 *
 * Who needs it: a host program that hands this library a GPU it manages itself -- all device memory reserved up
 * front in its own pool, or a serving loop whose latency budget rules out cudaMalloc/cudaFree (both serialise the
 * device) -- and therefore keeps graph sets and results in buffers it owns.  gtm_dataset_create and gtm_score
 * allocate (copies of the graph set, per-block scratch, a result buffer); this entry point allocates nothing:
 *  - device_graphs holds DEVICE pointers to the caller's copies of the graph arrays (same layouts as the host view);
 *  - class_sums_device is the caller's device buffer int32[count][CLASSES];
 *  - the scratch the scoring kernel needs (node-output words, message rows, include counts per thread block) is a
 *    GTM_STATIC_SCRATCH_BYTES array built into the library image; every GPU that loads the library holds it until
 *    the process exits.
 * It runs the general scoring kernel (any depth), queues the work on the model's stream and returns without
 * synchronising, like gtm_score_device, and gives the same class sums.
 * Requirements on the caller's buffers: every array 4-byte aligned; X 16-byte aligned when a literal row
 * (4*ceil(literals/32) bytes) is a multiple of 16 bytes, because such rows are read with 128-bit loads -- a buffer
 * carved out of a pool at an odd offset is refused with GTM_ERR_ARG before anything is launched.  The arrays are in
 * device memory, so their CONTENTS cannot be checked by the host: the kernel itself skips a graph whose node count
 * exceeds max_number_of_graph_nodes or whose node range leaves total_nodes (its class sums are zero), ignores edge
 * rows beyond total_edges and edges to nodes outside the graph, and records the fact; gtm_check_skipped_graphs
 * reports it.
 * Limits: the scratch of ONE thread block, 4*(2*CLAUSES*ceil(max_nodes/32) + max(1,depth-1)*max_nodes*
 * ceil(MESSAGE_SIZE/32) + CLAUSES) bytes, must fit in GTM_STATIC_SCRATCH_BYTES, otherwise GTM_ERR_ARG (nothing is
 * launched); fewer thread blocks run concurrently the larger that figure is.  Device ordinals 0..63.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress) -- make that first call
 * before any stream capture.  All calls share the one array and find the previous call's contents in it (the
 * kernel clears what it needs zeroed); two calls whose kernels overlap on the GPU, on any streams or models of the
 * same device, race on it -- serialise them. */
#define GTM_STATIC_SCRATCH_BYTES (8u * 1024u * 1024u)
int gtm_score_static_scratch(gtm_model *model, const gtm_graphs_view *device_graphs, int number_of_node_types,
                             int64_t first, int64_t count, int32_t *class_sums_device);

/* Waits for the model's stream and tells whether a scoring kernel launched since the last call skipped a malformed
 * graph (see gtm_score_static_scratch; *skipped_out = 0 or 1, then cleared).  NO COUNTERPART IN THE REFERENCE, which
 * checks nothing and indexes out of bounds on such input (tm.py:765 vs kernels.py:35). */
int gtm_check_skipped_graphs(gtm_model *model, int *skipped_out);

/* Replaces the learning loop of tm.py:668-747 (_fit): `epochs` passes over graphs [first, first+count) in
 * order; encoded_Y is int32[number_of_graphs][CLASSES] with +-T targets (tm.py:949-951), indexed by the
 * absolute graph id. */
int gtm_fit(gtm_model *model, gtm_dataset *dataset, int number_of_node_types, const int32_t *encoded_Y,
            int64_t first, int64_t count, int epochs);

/* Clause-sharded learning over the GPUs of one box, one process per GPU (NO COUNTERPART IN THE REFERENCE, which is
 * single-GPU).  Every rank holds the whole model and the whole graph set; during gtm_fit rank r learns clauses
 * gtm_shard_range(world, r) and the kernels of all ranks exchange, per graph, their vote partials (and, for depth > 1,
 * message bits and barrier arrivals) by direct stores / atomics into each other's buffers over NVLink.  Results do not
 * depend on the number of ranks (draw streams are per clause).  Protocol, per graph set:
 *   1. every rank: gtm_shard_prepare(model, dataset, world, rank, handle[64])   allocates the rank's buffers
 *   2. the ranks exchange the 64-byte handles (any transport), rank order
 *   3. every rank: gtm_shard_connect(model, dataset, handles[world][64])
 *   4. every rank: the same sequence of gtm_fit calls (same ranges and epochs), all ranks inside each call at the same
 *      time; AFTER every call the ranks must synchronise with each other (e.g. by gathering the updated shards:
 *      gtm_get_ta_state / gtm_get_weights rows of gtm_shard_range, then gtm_set_* of the assembled arrays) before
 *      the next call.  A rank that does not show up makes the others return GTM_ERR_TIMEOUT after a bounded wait. */
int gtm_shard_range(gtm_model *model, int world, int rank, int *first_clause_out, int *number_of_clauses_out);
int gtm_shard_prepare(gtm_model *model, gtm_dataset *dataset, int world, int rank, unsigned char *handle_out);
int gtm_shard_connect(gtm_model *model, gtm_dataset *dataset, const unsigned char *handles);

/* Replaces tm.py:814-851 (transform; kernels.py:671-691): clause outputs int32[count][CLAUSES] (0/1) and the
 * class sums int32[count][CLASSES] of graphs [first, first+count).  Either output may be NULL. */
int gtm_transform(gtm_model *model, gtm_dataset *dataset, int number_of_node_types, int64_t first, int64_t count,
                  int32_t *clause_outputs_out, int32_t *class_sums_out);

/* Replaces tm.py:853-900 (transform_nodewise; kernels.py:693-709): per-node clause outputs of the last layer,
 * int32[count][CLAUSES][node_stride] (0/1; entries beyond a graph's node count are 0), node_stride >= the largest
 * graph's node count, and the class sums (may be NULL).  One launch for the whole range. */
int gtm_transform_nodewise(gtm_model *model, gtm_dataset *dataset, int number_of_node_types, int64_t first, int64_t count,
                           int node_stride, int32_t *node_outputs_out, int32_t *class_sums_out);

/* Differential-test taps (no counterpart call in the reference; they expose the buffers its kernels leave in
 * device memory between launches of tm.py:563-747).
 *  gtm_debug_evaluate: inference on one graph through the scoring kernel (path 0) or through the learning
 *   kernel's inference phase (path 1).  cno_out: uint32[depth][CLAUSES][ceil(n/32)] node-output bits after
 *   each layer; messages_out: uint32[depth-1][n][ceil(2*MESSAGE_SIZE/32)] packed messages (clause_X);
 *   n_inc_out: int32[CLAUSES]; class_sum_out: int32[CLASSES].  Any output may be NULL.
 *  gtm_debug_last_feedback: after gtm_fit, the selected node per clause int32[CLAUSES] (clause_node) and the
 *   feedback type int32[CLASSES][CLAUSES] (class_clause_update) of the last graph processed. */
int gtm_debug_evaluate(gtm_model *model, gtm_dataset *dataset, int number_of_node_types, int64_t graph, int path,
                       uint32_t *cno_out, uint32_t *messages_out, int32_t *n_inc_out, int32_t *class_sum_out);
int gtm_debug_last_feedback(gtm_model *model, int32_t *clause_node_out, int32_t *class_clause_update_out);

/* Profiling tap (no counterpart in the reference): SM clock cycles that the first warp of CTA 0 of the last gtm_fit launch
 * spent in its phases, uint64[8] = {clause evaluation, waiting at grid barriers, vote exchange (with the work done in
 * its shadow), end of step, and then
 *   state-resident kernel, "fit_timers" 1: decisions, work-item table, remaining mask generation, automaton updates;
 *   state-resident kernel, "fit_timers" 2: next-graph copies issued, own clauses, waiting for the other warps, sending marks;
 *   state-resident kernel, "fit_timers" 3: next-graph copies issued, message rows built, transposition, own clauses
 *   (with 2 and 3 these four are not part of the first figure and the feedback is the fourth figure);
 *   global-state kernel: clause loops, sending marks, message rows / copies (not part of the first figure), 0}.
 * A phase that ends at a CTA barrier includes the wait for the CTA's slowest warp.  Filled only by launches made after
 * gtm_set_option(model, "fit_timers", 1..3): the clock reads sit on the per-graph critical path. */
int gtm_debug_fit_phase_cycles(gtm_model *model, uint64_t *cycles_out);

/* Measurement aid (no counterpart in the reference): the device's rate of register-resident, dependence-free 32-bit
 * three-input logic operations (LOP3), in 1e12 operations per second - the denominator of the integer roofline that
 * the word tests of clause evaluation are reported against.  Runs a short kernel on the model's device and stream. */
int gtm_debug_logic_op_rate(gtm_model *model, double *tera_ops_per_second_out);

#ifdef __cplusplus
}
#endif
#endif /* GTM_B200_H */
