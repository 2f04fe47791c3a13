"""Graph-sharded scoring over several GPUs of one box: one process per GPU, no collective on the data path.

Graphs are independent at inference, so rank ``r`` scores a contiguous range of graphs balanced by node count and
the per-rank class sums (disjoint rows of ``int32[N][K]``) are gathered at the end.  ``torch.distributed`` supplies
the process group (NCCL on GPUs, gloo in the CPU tests); the scoring itself is whatever ``score_range`` does —
``GraphShardScorer`` uses the engine, the tests plug in a CPU function.
"""

import numpy as np

__all__ = ["balanced_ranges", "clause_shard", "gather_rows", "GraphShardScorer"]


def balanced_ranges(number_of_graph_nodes, parts):
    """``parts`` contiguous (first, count) graph ranges whose node totals are as even as a prefix cut allows.
    Ranges may be empty when there are fewer graphs than parts."""
    nodes = np.asarray(number_of_graph_nodes, dtype=np.int64)
    n = len(nodes)
    prefix = np.concatenate([[0], np.cumsum(nodes)])
    cuts = [0]
    for p in range(1, parts):
        target = prefix[-1] * p / parts
        cut = int(np.searchsorted(prefix, target, side="left"))
        cuts.append(min(max(cut, cuts[-1]), n))
    cuts.append(n)
    return [(cuts[p], cuts[p + 1] - cuts[p]) for p in range(parts)]


def clause_shard(number_of_clauses, world, rank):
    """(first clause, number of clauses) that ``rank`` learns when fit is sharded over ``world`` ranks: equal shards of
    ``ceil(C / world)`` clauses, the last ones shorter or empty (the rule of ``gtm_shard_range`` in the C ABI)."""
    per = (number_of_clauses + world - 1) // world
    first = min(number_of_clauses, rank * per)
    return first, min(number_of_clauses, first + per) - first


def gather_rows(local_rows, counts, group=None):
    """All ranks contribute ``local_rows`` (``[counts[rank]][K]`` int32, numpy); every rank gets the rows of all ranks
    in rank order.  Uses a padded all_gather so that it works on every backend."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    K = local_rows.shape[1]
    longest = max(counts) if counts else 0
    device = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    mine = torch.zeros((longest, K), dtype=torch.int32, device=device)
    if counts[rank]:
        mine[:counts[rank]] = torch.from_numpy(np.ascontiguousarray(local_rows, dtype=np.int32)).to(device)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine, group=group)
    return np.concatenate([parts[r][:counts[r]].cpu().numpy() for r in range(world)], axis=0)


def _world_and_rank(group=None):
    """(world size, rank) of the group; (1, 0) in a process that has not joined any process group."""
    import torch.distributed as dist

    if not dist.is_available() or not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


class GraphShardScorer:
    """``score(graphs)`` over all ranks of a process group.  Every rank holds the same model and the same ``graphs``
    object (a ``Graphs``, or a ``datasets.RepeatedGraphs``); each builds, uploads and scores only its own contiguous
    range, chosen so that the ranks get equal numbers of nodes.  The rank's slice is kept until a graph set with another
    signature arrives, so repeated calls copy and score, but do not slice again."""

    def __init__(self, tm, group=None):
        self.tm = tm
        self.group = group
        self._signature = None
        self._ranges = None
        self._local = None

    def shard(self, graphs):
        """(ranges of all ranks, this rank's graphs or None when its range is empty)."""
        if self._signature is None or not np.array_equal(self._signature, graphs.signature):
            world, rank = _world_and_rank(self.group)
            self._ranges = balanced_ranges(graphs.number_of_graph_nodes, world)
            first, count = self._ranges[rank]
            self._local = graphs[first:first + count] if count else None
            self._signature = graphs.signature
        return self._ranges, self._local

    def score_local(self, graphs, out=None):
        """Class sums of this rank's range only: ((first, count), int32[count][K]); no communication at all.
        `out` (optional, e.g. page-locked) receives the rows in place."""
        ranges, local = self.shard(graphs)
        first, count = ranges[_world_and_rank(self.group)[1]]
        if not count:
            return (first, 0), np.zeros((0, self.tm.number_of_outputs), dtype=np.int32)
        rows = self.tm.score(local) if out is None else self.tm.score(local, out=out)
        return (first, count), rows

    def score(self, graphs):
        """Class sums of all graphs on every rank (the ranks' rows gathered in rank order)."""
        (_, _), local = self.score_local(graphs)
        if _world_and_rank(self.group)[0] == 1:
            return local
        return gather_rows(local, [c for _, c in self._ranges], self.group)

    def predict(self, graphs):
        return np.argmax(self.score(graphs), axis=1)
