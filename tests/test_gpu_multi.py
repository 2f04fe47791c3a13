"""GPU suite, two GPUs: clause-sharded learning (one process per GPU, NCCL for the host-side plumbing, peer stores over
NVLink inside the kernels) gives bit-identical models to single-GPU learning.  Skipped on boxes with one GPU."""

import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, tmpdir):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [root, os.path.join(root, "tests")]
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist

    from graphtsetlinmachine_b200 import datasets
    from graphtsetlinmachine_b200.tm import MultiClassGraphTsetlinMachine
    from util import random_graphs

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    results = {}

    def run(name, make_model, graphs, Y, epochs):
        np.random.seed(21)
        sharded = make_model()
        sharded.shard_clauses()
        for _ in range(epochs):
            sharded.fit(graphs, Y, epochs=1, incremental=True)
        state = sharded.save()
        scores = sharded.score(graphs)
        if rank == 0:
            np.random.seed(21)
            single = make_model()
            for _ in range(epochs):
                single.fit(graphs, Y, epochs=1, incremental=True)
            ref = single.save()
            ok = np.array_equal(state["ta_state"], ref["ta_state"]) and np.array_equal(state["clause_weights"], ref["clause_weights"])
            for x, y in zip(state["message_ta_state"], ref["message_ta_state"]):
                ok = ok and np.array_equal(x, y)
            ok = ok and np.array_equal(scores, single.score(graphs))
            results[name] = bool(ok)

    # depth 1, 33 clauses (not divisible by the number of ranks), 3 classes
    rng = np.random.default_rng(4)
    np.random.seed(4)
    g1 = random_graphs(120, rng, hv_size=32, max_nodes=6, node_types=2)
    y1 = rng.integers(0, 3, size=120).astype(np.uint32)
    run("depth1", lambda: MultiClassGraphTsetlinMachine(33, 30, 2.5, depth=1, seed=3, device=rank), g1, y1, 3)
    # depth 3 with messages
    np.random.seed(4)
    g2 = random_graphs(80, rng, hv_size=24, max_nodes=40, node_types=1, edge_types=3)
    y2 = rng.integers(0, 2, size=80).astype(np.uint32)
    run("depth3", lambda: MultiClassGraphTsetlinMachine(50, 25, 2.0, depth=3, message_size=96, message_bits=2, seed=5, device=rank), g2, y2, 3)
    # the XOR demo configuration
    np.random.seed(4)
    g3, y3 = datasets.noisy_xor(1500, 1)
    run("xor", lambda: MultiClassGraphTsetlinMachine(10, 100, 1.0, depth=2, message_size=256, message_bits=2,
                                                     max_included_literals=4, seed=6, device=rank), g3, y3, 3)
    # automaton layers wider than a warp (work items per 32-word stretch), small graphs (merged marks, rows per block)
    np.random.seed(4)
    g4 = random_graphs(40, rng, hv_size=1100, max_nodes=5, edge_types=2)
    y4 = rng.integers(0, 2, size=40).astype(np.uint32)
    run("wide", lambda: MultiClassGraphTsetlinMachine(24, 20, 4.0, depth=2, message_size=64, message_bits=2, seed=8, device=rank), g4, y4, 2)
    # graphs of 200 nodes: merged marks with the rows built in the marks buffer
    np.random.seed(4)
    g5 = random_graphs(16, rng, hv_size=24, max_nodes=200, node_types=2, edge_types=3)
    y5 = rng.integers(0, 2, size=16).astype(np.uint32)
    run("large", lambda: MultiClassGraphTsetlinMachine(40, 30, 2.5, depth=3, message_size=96, message_bits=2, seed=9, device=rank), g5, y5, 2)
    # fewer clauses than ranks: the second rank learns nothing and still takes part in every exchange and barrier
    np.random.seed(4)
    run("one_clause", lambda: MultiClassGraphTsetlinMachine(1, 10, 2.0, depth=2, message_size=64, message_bits=2, seed=10, device=rank), g1, y1, 2)
    if rank == 0:
        np.save(os.path.join(tmpdir, "results.npy"),
                np.array([results[k] for k in ("depth1", "depth3", "xor", "wide", "large", "one_clause")]))
    dist.barrier()
    dist.destroy_process_group()


def test_clause_sharded_fit_equals_single_gpu_fit(engine_lib, tmp_path):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    ok = np.load(tmp_path / "results.npy")
    assert ok.tolist() == [True] * 6
