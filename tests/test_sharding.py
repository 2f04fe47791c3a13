"""CPU suite, part 4: the multi-process side of graph-sharded scoring, two gloo ranks on this machine.  The
scoring function plugged in here is the CPU checker; what is under test is range balancing, row gathering and
rank ordering."""

import os
import socket
import sys

import numpy as np
import pytest

from graphtsetlinmachine_b200.sharding import balanced_ranges, clause_shard


def test_balanced_ranges_cover_everything_in_order():
    rng = np.random.default_rng(0)
    for n, parts in [(1, 2), (7, 2), (100, 4), (1000, 8), (3, 8)]:
        nodes = rng.integers(1, 50, size=n)
        ranges = balanced_ranges(nodes, parts)
        assert len(ranges) == parts
        assert ranges[0][0] == 0 and sum(c for _, c in ranges) == n
        for (f0, c0), (f1, _) in zip(ranges, ranges[1:]):
            assert f0 + c0 == f1
        if n >= 10 * parts:
            loads = [nodes[f:f + c].sum() for f, c in ranges]
            assert max(loads) <= nodes.sum() / parts + nodes.max()


def test_clause_shards_partition_the_clauses():
    for clauses in (1, 7, 10, 33, 2500, 20000):
        for world in (1, 2, 3, 4, 8):
            shards = [clause_shard(clauses, world, r) for r in range(world)]
            assert shards[0][0] == 0 and sum(n for _, n in shards) == clauses
            for (f0, n0), (f1, _) in zip(shards, shards[1:]):
                assert f0 + n0 == f1 or (n0 == 0 and f1 == clauses)
            assert max(n for _, n in shards) == (clauses + world - 1) // world


def _worker(rank, world, port, tmpdir):
    sys.path[:0] = [os.path.dirname(os.path.dirname(os.path.abspath(__file__))), os.path.dirname(os.path.abspath(__file__))]
    import torch.distributed as dist

    from cases import make_case
    from graphtsetlinmachine_b200.sharding import GraphShardScorer
    from oracle.oracle import OracleTM

    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    kw, graphs, encY, _ = make_case("case_b")

    class CpuModel:                      # same surface as the model classes: score(graphs) -> int32[N][K]
        number_of_outputs = kw["classes"]

        def __init__(self):
            self.tm = OracleTM(**kw)
            self.tm.set_graphs(graphs)
            self.tm.prepare()
            self.tm.fit(encY)

        def score(self, subset):
            self.tm.set_graphs(subset)
            return self.tm.score()

    model = CpuModel()
    got = GraphShardScorer(model).score(graphs)
    want = model.score(graphs)
    np.save(os.path.join(tmpdir, "ok_%d.npy" % rank), np.array([np.array_equal(got, want)]))
    dist.destroy_process_group()


def test_two_rank_sharded_scoring_matches_single_process(tmp_path):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        assert np.load(tmp_path / ("ok_%d.npy" % rank))[0]
