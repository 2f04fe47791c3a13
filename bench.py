"""Benchmark of the Graph Tsetlin Machine hot path on B200: predict and fit throughput on the five benchmark
configurations, headline = the scaling-stress configuration (random multigraphs, 20,000 clauses, depth 3).

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the reference's own kernels compiled for the host, all host threads

One process per GPU.  Per configuration:

* `fit`      ordered passes over a training sample through the public API (clauses sharded over the ranks when
             N > 1, per-graph vote / message exchange over NVLink peer memory), wall clock;
* `value`    predict with the batch resident in device memory: ONE global graph set (N x the per-GPU batch) is cut
             into contiguous ranges of equal node counts by `sharding.GraphShardScorer`, every rank scores its own
             range, no collective on the data path; CUDA events on the launching stream, maximum over ranks;
* `e2e`      the same through the public API from page-locked host arrays: upload of the rank's graph arrays and
             read-back of its class sums inside the timed region, every step;
* roofline   algorithmic bytes (4nL0 + 8n + 8E + 4K per graph) against the measured copy bandwidth, and dense-equivalent
             word tests (C n L0 + (D-1) C n M per graph) against the LOP3 rate measured in the same run.

Rank 0 prints ONE JSON line: the headline configuration at the top level, all five under `configs`.
"""

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HEADLINE = 5

# name, workload text, model arguments, classes, hypervector (size, bits), graphs: training sample / distinct graphs of
# the scoring batch / copies of them per GPU and step, reference-kernel build parameters (oracle/ref_configs.py)
CONFIGS = {
    1: dict(name="noisy_xor",
            workload="Noisy XOR (BASELINE configs[0]): 2-node graphs, 10 clauses, T=100, s=1.0, depth 2, message 256/2, "
                     "hypervector 32/2, max_included_literals 4, 2 classes",
            model=dict(number_of_clauses=10, T=100, s=1.0, depth=2, message_size=256, message_bits=2, max_included_literals=4),
            classes=2, train=10000, unique=1 << 20, times=4, ref="noisy_xor"),
    2: dict(name="vanilla_images",
            workload="vanilla MNIST-shaped single-node graphs (BASELINE configs[1]): 2,500 clauses, T=3,125, s=10, depth 1, "
                     "hypervector 128/2, 10 classes",
            model=dict(number_of_clauses=2500, T=3125, s=10.0, depth=1),
            classes=10, train=60000, unique=1 << 18, times=16, ref="vanilla_images"),
    3: dict(name="convolution_images",
            workload="convolutional MNIST-shaped graphs (BASELINE configs[2]): 361 nodes (10x10 patches + position "
                     "thermometers), 2,500 clauses, T=3,125, s=10, depth 1, hypervector 128/2, 10 classes",
            model=dict(number_of_clauses=2500, T=3125, s=10.0, depth=1),
            classes=10, train=2000, unique=16384, times=1, ref="convolution_images"),
    4: dict(name="sequences",
            workload="sequence classification (BASELINE configs[3]): 1,000-node paths with Left/Right edges, 2,000 clauses, "
                     "T=2,000, s=5, depth 3, message 512/2, hypervector 256/2, 2 classes",
            model=dict(number_of_clauses=2000, T=2000, s=5.0, depth=3, message_size=512, message_bits=2),
            classes=2, train=300, unique=2048, times=1, ref="sequences"),
    5: dict(name="multigraphs",
            workload="scaling stress (BASELINE configs[4]): random directed multigraphs, 8..32 nodes, Poisson(3) out-degree, "
                     "4 edge types, 1..5 of 256 symbols per node, 20,000 clauses, T=10,000, s=10, depth 3, message 1,024/2, "
                     "hypervector 1,024/2, 10 classes",
            model=dict(number_of_clauses=20000, T=10000, s=10.0, depth=3, message_size=1024, message_bits=2),
            classes=10, train=2000, unique=32768, times=1, ref="multigraphs"),
}


def build_sets(idx, train_n, unique_n):
    """(training graphs, labels, distinct graphs of the scoring batch); seeded, identical on every rank."""
    from graphtsetlinmachine_b200 import datasets

    np.random.seed(1)                                   # symbol hypervectors
    if idx == 1:
        train, y = datasets.noisy_xor(train_n, 2)
        unique, _ = datasets.noisy_xor(unique_n, 1000, init_with=train)
    elif idx == 2:
        protos = datasets.image_prototypes(1)
        train, y = datasets.vanilla_images(train_n, 2, protos)
        unique, _ = datasets.vanilla_images(unique_n, 1000, protos, init_with=train)
    elif idx == 3:
        protos = datasets.image_prototypes(1)
        train, y = datasets.convolution_images(train_n, 2, protos)
        unique, _ = datasets.convolution_images(unique_n, 1000, protos, init_with=train)
    elif idx == 4:
        train, y = datasets.sequences(train_n, 2)
        unique, _ = datasets.sequences(unique_n, 1000, init_with=train)
    else:
        train, y = datasets.random_multigraphs(train_n, 2)
        unique, _ = datasets.random_multigraphs(unique_n, 1000, init_with=train)
    return train, y, unique


def shape_of(cfg, graphs):
    """Algorithmic bytes and dense-equivalent word tests per graph of a graph set under a configuration."""
    m = cfg["model"]
    L0 = int(graphs.X.shape[1])
    depth = m.get("depth", 1)
    M = (2 * m.get("message_size", 256) - 1) // 32 + 1
    n = graphs.X.shape[0] / graphs.number_of_graphs
    E = (graphs.edge.shape[0] if graphs.edge.size else 0) / graphs.number_of_graphs
    K, Cn = cfg["classes"], m["number_of_clauses"]
    bytes_per_graph = 4 * n * L0 + 8 * n + 8 * E + 4 * K
    lop3_per_graph = Cn * n * L0 + (depth - 1) * Cn * n * M
    ta_words = L0 + (depth - 1) * M
    return dict(nodes_per_graph=n, edges_per_graph=E, bytes_per_graph=bytes_per_graph, lop3_per_graph=lop3_per_graph,
                fit_bytes_per_graph=bytes_per_graph + 2 * 8 * 4 * ta_words * Cn)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured copy bandwidth (MEASURED_PEAKS.json)"
    return 6650.0, "fallback (earlier measurement on this pool)"


# DRAM bytes per graph of the dominant scoring kernel from ncu captures (profiles/): dram__bytes_read.sum +
# dram__bytes_write.sum of one launch divided by the graphs of that launch; None where no capture exists
NCU_DRAM_BYTES_PER_GRAPH = {1: (270.0e6 + 30.0e6) / 4194304,
                            2: (186.750208e6 + 124.236288e6) / 4194304,
                            4: (145.0e6 + 390.0e6) / 512,
                            5: (8.885644e9 + 3.636144e9) / 32768}

# what binds the scoring kernel of every configuration according to its ncu capture (profiles/)
NCU_BINDING = {
    1: "tile_score_kernel<2>: short barrier-separated phases per tile (barrier stall 17.7 warps per issue); shared-memory wavefronts 27 % of peak, DRAM 1.2 %",
    2: "stream_score_kernel<10>: shared memory (wavefronts 64 % of peak, short-scoreboard stall 5.7 warps per issue); DRAM 0.5 %",
    3: "stream_score_kernel<10>: shared memory (wavefronts 62 % of peak); DRAM 0.5 %",
    4: "score_graphs_kernel<1>: latency at 16 warps per SM with find-first-set loops on the quarter-rate pipe (XU 30 %, issue slots 43 %); DRAM 0.4 %",
    5: "tile_score_kernel<10>: shared memory (wavefronts 76 % of peak, 4.8 % of them from bank conflicts, issue slots 53 %); DRAM 7.9 %",
}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 <= t <= t1 + 0.2 and len(r) >= 7] or [r for _, r in self.rows if len(r) >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][1]), "reasons": reasons, "samples": len(rows)}


# ------------------------------------------------------------------------------------- reference on the host cores
def reference_params(cfg, graphs):
    from oracle.ref_configs import CONFIGS as REF

    return dict(REF[cfg["ref"]])


def checker_kwargs(cfg, hv_size, hypervectors, max_nodes):
    m = cfg["model"]
    return dict(clauses=m["number_of_clauses"], classes=cfg["classes"], literals=2 * hv_size, threshold=m["T"], s=m["s"],
                depth=m.get("depth", 1), message_size=m.get("message_size", 256), message_bits=m.get("message_bits", 2),
                max_included=m.get("max_included_literals"), max_nodes=max_nodes, hypervectors=hypervectors)


def cpu_reference_scorer(cfg, state, graphs, threads, max_nodes):
    """The reference's own scoring kernels compiled for the host (oracle/_ref), one instance per thread, or the C
    restatement when that build did not travel.  `state` = (layer-0 automata, message automata list, weights,
    hypervectors).  Returns (kind, run(first, count) -> (seconds, graphs scored, list of class-sum blocks))."""
    from oracle import build_ref
    from oracle.oracle import OracleTM

    kw = checker_kwargs(cfg, graphs.hypervector_size, state[3], max_nodes)
    params = dict(classes=kw["classes"], clauses=kw["clauses"], literals=kw["literals"], threshold=kw["threshold"],
                  max_included=kw["max_included"], max_nodes=max_nodes, message_size=kw["message_size"],
                  message_bits=kw["message_bits"])
    kind = "reference" if build_ref.build(params) is not None else "port"
    if kind == "reference":
        from oracle.ref_tm import RefTM as Impl
    else:
        Impl = OracleTM
    workers = []
    for _ in range(threads):
        tm = Impl(**kw)
        tm.ta_state[...] = state[0].reshape(tm.ta_state.shape)
        for mine, theirs in zip(tm.message_ta_state, state[1]):
            mine[...] = theirs.reshape(mine.shape)
        tm.clause_weights[...] = state[2].reshape(tm.clause_weights.shape)
        tm.set_graphs(graphs)
        workers.append(tm)

    def run(first, count):
        per = max(1, count // threads)
        used = min(threads, max(1, count // per))
        out = [None] * used

        def work(i):
            out[i] = workers[i].score(first + i * per, per)

        ts = [threading.Thread(target=work, args=(i,)) for i in range(used)]
        t0 = time.perf_counter()
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return time.perf_counter() - t0, per * used, out

    return kind, run


def timed_cpu_baseline(run, n_available, threads, budget_s):
    """Bounded sample: a probe sizes the run to about `budget_s` seconds of wall time on `threads` threads."""
    sec, cnt, _ = run(0, min(n_available, threads))
    per_s = cnt / max(sec, 1e-9)
    want = int(min(n_available, max(threads, per_s * budget_s))) // threads * threads
    sec, cnt, _ = run(0, max(threads, want))
    return cnt / sec, cnt


def synthetic_state(cfg, hv_size, seed=3):
    """A sparse model state for the reference arm (training 20,000 clauses on the host cores would take hours): every
    clause includes a handful of random negated literals per layer, weights +-1..9.  The reference's evaluation loops
    are dense (no early exit, kernels.py:443-460), so their speed does not depend on the state; the number of true
    clause-node pairs, which its message kernels walk, does, and is kept moderate by including negated literals."""
    m = cfg["model"]
    rng = np.random.default_rng(seed)
    Cn, K, depth = m["number_of_clauses"], cfg["classes"], m.get("depth", 1)
    MS = m.get("message_size", 256)

    def planes(literals, lo, hi, count):
        words = (literals - 1) // 32 + 1
        ta = np.zeros((Cn, words, 8), dtype=np.uint32)
        ta[:, :, :7] = 0xFFFFFFFF                      # every automaton one step below inclusion ...
        picks = rng.integers(lo, hi, size=(Cn, count))
        for j in range(count):                          # ... except the picked literals, which are included
            w, b = picks[:, j] // 32, picks[:, j] % 32
            ta[np.arange(Cn), w, 7] |= (np.uint32(1) << b.astype(np.uint32))
            ta[np.arange(Cn), w, :7] &= ~(np.uint32(1) << b.astype(np.uint32))[:, None]
        return ta

    ta0 = planes(2 * hv_size, hv_size, 2 * hv_size, 24)
    msg = [planes(2 * MS, MS, 2 * MS, 24) for _ in range(depth - 1)]
    weights = (rng.integers(1, 10, size=(K, Cn)) * rng.choice([-1, 1], size=(K, Cn))).astype(np.int32)
    hv = np.stack([rng.choice(MS, size=m.get("message_bits", 2), replace=False) for _ in range(Cn)]).astype(np.uint32)
    return ta0, msg, weights, hv


def run_reference(args, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    cfg = CONFIGS[HEADLINE]
    train, y_train, unique = build_sets(HEADLINE, 64, 4096)
    max_nodes = int(reference_params(cfg, unique)["max_nodes"])
    state = synthetic_state(cfg, unique.hypervector_size)
    kind, run = cpu_reference_scorer(cfg, state, unique, threads, max_nodes)
    sec, n, _ = run(0, threads)
    per_step = int(max(threads, min(unique.number_of_graphs, n / sec * 4.0))) // threads * threads
    for _ in range(args.warmup):
        run(0, per_step)
    total_s, total_n = 0.0, 0
    for _ in range(args.steps):
        sec, n, _ = run(0, per_step)
        total_s += sec
        total_n += n
    value = total_n / total_s
    line = {
        "impl": "reference", "metric": "predict graphs/sec (fit in `fit`)", "value": value, "unit": "graphs/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total_s / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
        "config": headline_config(cfg),
        "cpu_baseline": {"value": value, "unit": "graphs/s", "cores": threads, "kind": kind,
                         "sample": "%d graphs of the batch per step scored by the reference's kernels compiled for the host, "
                                   "%d threads; model state: synthetic sparse state (the reference's evaluation loops are dense, "
                                   "their speed does not depend on the state)" % (per_step, threads)},
        "e2e": {"value": value, "unit": "graphs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def headline_config(cfg):
    """The `config` object: identical in both arms."""
    return {"workload": cfg["workload"], "graphs_per_step_per_gpu": cfg["unique"] * cfg["times"],
            "l2": "inputs larger than L2", "partitioning": "predict: one global graph set cut into per-rank ranges of equal "
            "node counts, no collective; fit: clauses sharded over ranks"}


# ---------------------------------------------------------------------------------------------------- engine arm
def reference_kernels_on_gpu(cfg, tm, state, train, y_train, batch, sums_host, max_nodes, sample):
    """The reference's kernels compiled for this GPU and driven like its host code drives them (one launch and one
    synchronisation per kernel and graph): scoring checked against the engine's class sums, scoring and learning timed
    on a bounded sample by wall clock.  None when that build did not travel with the tree."""
    try:
        from oracle.ref_gpu_tm import RefGpuTM

        kw = checker_kwargs(cfg, batch.hypervector_size, state[3], max_nodes)
        ref = RefGpuTM(seed=7, **kw)
    except (FileNotFoundError, OSError):
        return None
    ref.ta_state[...] = state[0].reshape(ref.ta_state.shape)
    for mine, theirs in zip(ref.message_ta_state, state[1]):
        mine[...] = theirs.reshape(mine.shape)
    ref.clause_weights[...] = state[2].reshape(ref.clause_weights.shape)
    ref.upload()
    ref.set_graphs(batch)
    ref.score(0, min(8, sample))
    t0 = time.perf_counter()
    got = ref.score(0, sample)
    score_s = time.perf_counter() - t0
    assert np.array_equal(got, sums_host[:sample]), "class sums differ from the reference kernels run on this GPU"
    ref.set_graphs(train)
    T = cfg["model"]["T"]
    enc = np.where(y_train[:, None] == np.arange(cfg["classes"])[None, :], T, -T).astype(np.int32)
    n_fit = min(sample, train.number_of_graphs - 8)
    ref.fit(enc, 0, 8)
    t0 = time.perf_counter()
    ref.fit(enc, 8, n_fit)
    fit_s = time.perf_counter() - t0
    ref.close()
    return {"predict": sample / score_s, "fit": n_fit / fit_s, "unit": "graphs/s", "sample": "%d / %d graphs" % (sample, n_fit),
            "class_sums_equal_engine": True,
            "how": "reference kernel source compiled with nvcc for sm_100a, grid 832 x block 128, launched and synchronised "
                   "per kernel and per graph with the per-graph class-sum copies of the reference's host loop; wall clock"}


def host_side_baselines(sample_images=256, bulk_images=1 << 15):
    """The reference's host-side work on this box's cores: `Graphs` encoding of MNIST-shaped images through the per-item
    API (one core: it is Python-bound) and through the vectorised builders."""
    from graphtsetlinmachine_b200 import datasets
    from graphtsetlinmachine_b200.graphs import Graphs

    protos = datasets.image_prototypes(1)
    rng = np.random.default_rng(5)
    labels = rng.integers(0, 10, size=sample_images)
    pixels = rng.random((sample_images, protos.shape[1])) < protos[labels]
    np.random.seed(1)
    t0 = time.perf_counter()
    g = Graphs(sample_images, symbols=list(range(protos.shape[1])), hypervector_size=128, hypervector_bits=2)
    for i in range(sample_images):
        g.set_number_of_graph_nodes(i, 1)
    g.prepare_node_configuration()
    for i in range(sample_images):
        g.add_graph_node(i, "Image Node", 0)
    g.prepare_edge_configuration()
    for i in range(sample_images):
        for k in pixels[i].nonzero()[0]:
            g.add_graph_node_property(i, "Image Node", int(k))
    g.encode()
    api_s = time.perf_counter() - t0
    np.random.seed(1)
    t0 = time.perf_counter()
    datasets.vanilla_images(bulk_images, 6, protos, 128, 2)
    bulk_s = time.perf_counter() - t0
    return {"graphs_encoding_api": {"value": sample_images / api_s, "unit": "graphs/s", "cores": 1,
                                    "sample": "%d MNIST-shaped images through add_graph_node_property" % sample_images},
            "graphs_encoding_vectorised": {"value": bulk_images / bulk_s, "unit": "graphs/s", "cores": 1,
                                           "sample": "%d images through the bulk builders" % bulk_images}}


def numpy_clause_evaluation(state, batch, sums_host, threads, sample=2048):
    """NumPy evaluation of the same clause semantics for a depth-1 model (fail = any(include & ~X), votes by a matrix
    product) on `threads` threads, checked against the engine's class sums (single-node graphs)."""
    from concurrent.futures import ThreadPoolExecutor

    include = np.ascontiguousarray(state[0][:, :, 7])
    weights = state[2].astype(np.int32)
    X = np.ascontiguousarray(batch.X[:sample])

    def evaluate(span):
        lo, hi = span
        fails = ((include[None, :, :] & ~X[lo:hi, None, :]) != 0).any(axis=2)
        return (~fails).astype(np.int32) @ weights.T

    chunk = 64
    spans = [(lo, min(sample, lo + chunk)) for lo in range(0, sample, chunk)]
    with ThreadPoolExecutor(threads) as pool:
        list(pool.map(evaluate, spans[:threads]))
        t0 = time.perf_counter()
        parts = list(pool.map(evaluate, spans))
        sec = time.perf_counter() - t0
    assert np.array_equal(np.concatenate(parts), sums_host[:sample]), "NumPy evaluation differs from the engine"
    return {"value": sample / sec, "unit": "graphs/s", "cores": threads, "sample": "%d graphs, chunks of %d over a thread pool" % (sample, chunk)}


def measure_logic_op_rate(lib, device):
    """LOP3 rate of this GPU in 1e12 operations per second (register-resident independent chains): the denominator of
    the integer roofline.  Measured through a throw-away model handle."""
    from graphtsetlinmachine_b200 import _lib

    cfg = _lib.Config()
    cfg.number_of_clauses, cfg.number_of_outputs, cfg.number_of_literals = 4, 2, 64
    cfg.number_of_state_bits, cfg.boost_true_positive_feedback, cfg.T = 8, 1, 10
    cfg.max_included_literals, cfg.message_size, cfg.message_bits, cfg.depth, cfg.device = 64, 256, 2, 1, device
    cfg.q, cfg.seed = 1.0, 1
    cfg.s[0] = 2.0
    model = C.c_void_p()
    _lib.check(lib.gtm_create(C.byref(cfg), C.byref(model)))
    rate = C.c_double(0.0)
    _lib.check(lib.gtm_debug_logic_op_rate(model, C.byref(rate)))
    lib.gtm_destroy(model)
    return rate.value


def run_config(idx, ctx, steps, warmup, headline):
    """One configuration on this rank (all ranks run it together); returns the record (rank 0) or None."""
    import torch
    import torch.distributed as dist

    from graphtsetlinmachine_b200 import _lib, datasets
    from graphtsetlinmachine_b200.sharding import GraphShardScorer
    from graphtsetlinmachine_b200.tm import MultiClassGraphTsetlinMachine

    cfg = CONFIGS[idx]
    rank, world, local_rank, lib, args = ctx["rank"], ctx["world"], ctx["local_rank"], ctx["lib"], ctx["args"]
    barrier = ctx["barrier"]
    K, T = cfg["classes"], cfg["model"]["T"]
    depth = cfg["model"].get("depth", 1)
    t_cfg = time.perf_counter()
    if args.fit_graphs > 0 or args.batch_graphs > 0:         # reduced sizes for captures under a profiler
        cfg = dict(cfg, train=args.fit_graphs or cfg["train"], unique=args.batch_graphs or cfg["unique"])
    train, y_train, unique = build_sets(idx, cfg["train"], cfg["unique"])
    max_nodes = int(max(train.max_number_of_graph_nodes, unique.max_number_of_graph_nodes))

    def new_model():
        np.random.seed(1)                               # message hypervectors identical on every rank and in the re-fit
        return MultiClassGraphTsetlinMachine(seed=7, device=local_rank, **cfg["model"])

    tm = new_model()
    if world > 1:
        tm.shard_clauses()      # fit: clauses sharded over the ranks, per-graph exchange over NVLink peer stores

    # ---- fit: ordered passes over the training sample; the last one is timed ----
    tm.fit(train, y_train, epochs=1, incremental=True)
    barrier()
    t0 = time.perf_counter()
    tm.fit(train, y_train, epochs=1, incremental=True)
    barrier()
    fit_s = time.perf_counter() - t0
    train_acc = float((tm.predict(train) == y_train).mean())
    fit_identical = None
    if world > 1 and headline and rank == 0:
        # the same passes on this GPU alone must leave the same model: sharding must not change a single bit
        solo = new_model()
        solo.fit(train, y_train, epochs=1, incremental=True)
        solo.fit(train, y_train, epochs=1, incremental=True)
        a, b = tm.save(), solo.save()
        fit_identical = bool(np.array_equal(a["ta_state"], b["ta_state"]) and np.array_equal(a["clause_weights"], b["clause_weights"])
                             and all(np.array_equal(x, y) for x, y in zip(a["message_ta_state"], b["message_ta_state"])))
        assert fit_identical, "clause-sharded fit differs from single-GPU fit"
        solo._release()
    barrier()

    # ---- one global graph set, this rank's range of it ----
    global_set = datasets.RepeatedGraphs(unique, cfg["times"] * world)
    scorer = GraphShardScorer(tm)
    ranges, local = scorer.shard(global_set)
    first, n = ranges[rank]
    shape = shape_of(cfg, local)
    n_global = global_set.number_of_graphs

    # ---- predict, this rank's range resident in device memory ----
    stream = torch.cuda.current_stream()
    _lib.check(lib.gtm_set_stream(tm._model, C.c_void_p(stream.cuda_stream)))
    tm._score_init(local)                                    # upload once, outside the timed region
    sums_dev = torch.empty((n, K), dtype=torch.int32, device="cuda")
    nt = int(local.number_of_node_types())

    def step():
        _lib.check(lib.gtm_score_device(tm._model, tm._test_set.handle, nt, 0, n, C.c_void_p(sums_dev.data_ptr())))

    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank) if headline else None
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.time()
    start.record(stream)
    for _ in range(steps):
        step()
    stop.record(stream)
    barrier()
    w1 = time.time()
    clocks = sampler.stop(w0, w1) if sampler else None
    ms = torch.tensor([start.elapsed_time(stop) / steps], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item())
    value = n_global / (ms_per_step * 1e-3)
    sums_host = sums_dev.cpu().numpy()
    skipped = C.c_int(0)
    _lib.check(lib.gtm_check_skipped_graphs(tm._model, C.byref(skipped)))
    assert skipped.value == 0

    # ---- end to end through the public API: pinned host arrays in, class sums out, every step ----
    cudart = torch.cuda.cudart()
    pinned = [local.X, local.node_type, local.number_of_graph_node_edges, local.edge_index, local.node_index,
              local.number_of_graph_nodes] + ([local.edge] if local.edge.size else [])
    out_host = np.zeros((n, K), dtype=np.int32)
    for a in pinned + [out_host]:
        cudart.cudaHostRegister(a.ctypes.data, a.nbytes, 0)
    h2d = int(sum(a.nbytes for a in pinned))
    d2h = int(out_host.nbytes)
    e2e_steps = max(1, min(steps, 10))

    def e2e_step():
        tm.graphs_signature_test = np.array([])              # forget the cached upload: copy the inputs again
        scorer.score_local(global_set, out=out_host)

    e2e_step()
    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / e2e_steps], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_value = n_global / (float(e2e_ms.item()) * 1e-3)
    assert np.array_equal(out_host, sums_host), "API result differs from the device-resident run"
    for a in pinned + [out_host]:
        cudart.cudaHostUnregister(a.ctypes.data)
    tm.graphs_signature_test = np.array([])
    if tm._test_set is not None:
        tm._test_set.close()
        tm._test_set = None

    # ---- checks against the reference's kernels on the host + CPU baseline (rank 0; timing at N = 1 only) ----
    saved = tm.save()
    state = (saved["ta_state"].reshape(cfg["model"]["number_of_clauses"], -1, 8),
             [m.reshape(cfg["model"]["number_of_clauses"], -1, 8) for m in saved["message_ta_state"]],
             saved["clause_weights"].reshape(K, -1), np.asarray(saved["hypervectors"], dtype=np.uint32))
    cpu, ref_gpu, numpy_eval, checked = None, None, None, 0
    if rank == 0:
        threads = os.cpu_count() or 1
        kind, run = cpu_reference_scorer(cfg, state, local, threads, max_nodes)
        probe = min(n, threads if idx >= 4 else 8 * threads)
        sec, cnt, outs = run(0, probe)
        got = np.concatenate(outs)
        assert np.array_equal(got, sums_host[:cnt]), "class sums differ from the reference's kernels compiled for the host"
        checked = cnt
        if world == 1 and not args.skip_cpu_baseline:
            rate, cnt2 = timed_cpu_baseline(run, n, threads, 12.0 if headline else 3.0)
            cpu = {"value": rate, "unit": "graphs/s", "cores": threads, "kind": kind,
                   "sample": "%d graphs of the same batch, %d host threads, reference scoring kernels compiled for the host, "
                             "same trained state as the engine" % (cnt2, threads)}
            if headline or idx == 2:
                ref_gpu = reference_kernels_on_gpu(cfg, tm, state, train, y_train, local, sums_host, max_nodes,
                                                   sample=256 if idx == 5 else 2048)
            if idx == 2:
                numpy_eval = numpy_clause_evaluation(state, local, sums_host, threads)

    if rank != 0:
        tm._release()
        return None
    peak, peak_src = peaks()
    int_peak = ctx["int_peak"]
    achieved = shape["bytes_per_graph"] * n_global / world / (ms_per_step * 1e-3) / 1e9        # per GPU
    tlop3 = shape["lop3_per_graph"] * n_global / world / (ms_per_step * 1e-3) / 1e12
    fit_rate = cfg["train"] / fit_s
    traffic = NCU_DRAM_BYTES_PER_GRAPH.get(idx)
    record = {
        "config": idx, "name": cfg["name"], "workload": cfg["workload"],
        "graphs_per_step_per_gpu": cfg["unique"] * cfg["times"], "graphs_per_step": n_global,
        "nodes_per_graph": shape["nodes_per_graph"], "edges_per_graph": shape["edges_per_graph"],
        "predict": {"value": value, "unit": "graphs/s", "ms_per_step": ms_per_step, "steps": steps, "warmup": warmup},
        "e2e": {"value": e2e_value, "unit": "graphs/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps},
        "fit": {"value": fit_rate, "unit": "graphs/s", "graphs": cfg["train"], "epoch_s": fit_s, "n_gpus": world,
                "train_accuracy_after_2_passes": train_acc, "scaling": "strong",
                "partitioning": "clauses sharded over ranks, per-graph class-sum / message exchange by NVLink peer stores" if world > 1 else "single GPU",
                "sharded_fit_bit_identical_to_single_gpu": fit_identical,
                "roofline": {"bound": "automaton traffic: every automaton word of every clause read and written once per graph",
                             "bytes_per_graph": shape["fit_bytes_per_graph"],
                             "bound_graphs_per_s": peak * 1e9 / shape["fit_bytes_per_graph"],
                             "frac": fit_rate * shape["fit_bytes_per_graph"] / (peak * 1e9),
                             "note": "learning is sequential over graphs (online updates); the automata stay in shared memory "
                                     "when they fit, so DRAM is idle and the per-graph dependency chain binds"}},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None if traffic is None else traffic * n, "peak_source": peak_src,
                     "bytes_per_launch": shape["bytes_per_graph"] * n, "bytes_per_graph": shape["bytes_per_graph"],
                     "binding_resource_ncu": NCU_BINDING.get(idx),
                     "int_ops": {"dense_lop3_per_graph": shape["lop3_per_graph"], "achieved_tlop3_s": tlop3,
                                 "peak_tlop3_s": int_peak, "frac": tlop3 / max(int_peak, 1e-9),
                                 "peak_source": "register-resident independent LOP3 chains measured in this run (gtm_debug_logic_op_rate)",
                                 "note": "dense-equivalent word tests (C n L0 + (D-1) C n M per graph); the kernels test only "
                                         "included literals, so the executed count is smaller and the fraction can exceed 1"}},
        "checked_against_reference_host_kernels": checked,
        "cpu_baseline": cpu, "reference_kernels_on_gpu": ref_gpu, "numpy_clause_evaluation": numpy_eval,
        "clocks": clocks, "seconds": None,
    }
    tm._release()
    record["seconds"] = time.perf_counter() - t_cfg
    return record


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="engine", choices=["engine", "reference"])
    ap.add_argument("--configs", default="1,2,3,4,5", help="configurations to run besides the headline one")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--only", type=int, default=0, help="run this configuration alone and print its record (profiling runs)")
    ap.add_argument("--fit-graphs", type=int, default=0, help="training sample size of every configuration (profiling runs)")
    ap.add_argument("--batch-graphs", type=int, default=0, help="distinct graphs of every scoring batch (profiling runs)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    from graphtsetlinmachine_b200 import _lib

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    lib = _lib.load()
    int_peak = measure_logic_op_rate(lib, local_rank)

    ctx = dict(rank=rank, world=world, local_rank=local_rank, lib=lib, args=args, barrier=barrier, int_peak=int_peak)
    if args.only:
        rec = run_config(args.only, ctx, args.steps, args.warmup, False)
        if rank == 0:
            print(json.dumps(rec), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    wanted = sorted({int(c) for c in args.configs.split(",") if c.strip()} | {HEADLINE})
    records = {}
    for idx in wanted:
        headline = idx == HEADLINE
        rec = run_config(idx, ctx, args.steps if headline else max(1, min(args.steps, 5)), args.warmup if headline else 3, headline)
        if rank == 0:
            records[idx] = rec
        barrier()

    if rank == 0:
        head = records[HEADLINE]
        cfg = CONFIGS[HEADLINE]
        host_side = host_side_baselines() if world == 1 and not args.skip_cpu_baseline else None
        line = {
            "metric": "predict graphs/sec (fit in `fit`)", "value": head["predict"]["value"], "unit": "graphs/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["predict"]["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
            "config": headline_config(cfg),
            "e2e": head["e2e"],
            "gpu_launches": args.steps,
            "roofline": dict(head["roofline"], kernel="tile_score_kernel, one launch per step"),
            "cpu_baseline": head["cpu_baseline"],
            "reference_kernels_on_gpu": head["reference_kernels_on_gpu"],
            "fit": head["fit"],
            "clocks": head["clocks"],
            "host_side": host_side,
            "configs": [records[i] for i in sorted(records)],
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
