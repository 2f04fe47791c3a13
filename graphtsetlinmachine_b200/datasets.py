"""Seeded synthetic graph sets with the shapes of the five benchmark configurations.

They stand in for the data sets the reference's demos download (MNIST etc.), which are not available offline:
same graph shapes, symbol vocabularies and encodings as the demos (``examples/NoisyXORDemo.py``,
``examples/MNISTVanillaDemo.py``, ``examples/MNISTConvolutionDemo.py`` / ``examples/CIFAR10Demo.py:60-113``,
``examples/SequenceClassificationDemo.py:40-72``), random content.  Everything is built with the bulk methods of
``Graphs`` and therefore yields the same arrays as the per-item API would.

Every generator returns ``(graphs, Y)``; pass ``init_with=train_graphs`` to build a test set that shares symbol
tables and hypervectors.  Symbol hypervectors come from the global ``numpy.random`` stream (as in the reference), so
call ``numpy.random.seed`` first for reproducible encodings; the content comes from ``numpy.random.default_rng(seed)``.
"""

import numpy as np

from .graphs import Graphs

__all__ = ["noisy_xor", "vanilla_images", "convolution_images", "sequences", "random_multigraphs",
           "image_prototypes", "sample_images", "replicate", "RepeatedGraphs"]


def _new(n, symbols, hv_size, hv_bits, init_with):
    if init_with is None:
        return Graphs(n, symbols=symbols, hypervector_size=hv_size, hypervector_bits=hv_bits)
    return Graphs(n, init_with=init_with)


def _or_symbols(graphs, active, symbol_ids, chunk=32768):
    """X rows |= OR of the hypervectors of the active symbols; ``active`` is bool[rows][len(symbol_ids)].

    Same result as one ``add_graph_node_property`` per active (row, symbol) pair: positive literal bits are set and
    the matching negated literal bits cleared (graphs.py:148-159), computed as a boolean matrix product."""
    hv = graphs.hypervectors[np.asarray(symbol_ids)]
    size = graphs.hypervector_size
    table = np.zeros((len(symbol_ids), size), dtype=np.float32)
    table[np.repeat(np.arange(len(symbol_ids)), hv.shape[1]), hv.ravel()] = 1.0
    words = graphs.number_of_hypervector_chunks
    for lo in range(0, active.shape[0], chunk):
        hit = (active[lo:lo + chunk].astype(np.float32) @ table) > 0          # [rows][size]
        lits = np.zeros((hit.shape[0], words * 32), dtype=np.uint8)
        lits[:, :size] = hit
        lits[:, size:2 * size] = ~hit
        packed = np.packbits(lits, axis=1, bitorder="little").view(np.uint32)
        rows = graphs.X[lo:lo + chunk]
        # keep bits set earlier on positive literals, and negated literals cleared earlier
        pos_mask = np.zeros(words * 32, dtype=np.uint8)
        pos_mask[:size] = 1
        pos_mask = np.packbits(pos_mask, bitorder="little").view(np.uint32)
        rows[:] = ((rows | packed) & pos_mask) | ((rows & packed) & ~pos_mask)


# ------------------------------------------------------------------------------------------ config 1
def noisy_xor(n_graphs, seed, noise=0.01, hv_size=32, hv_bits=2, init_with=None):
    """Two nodes with symbol 'A' or 'B' each, one 'Plain' edge in each direction, label = XOR with flips."""
    rng = np.random.default_rng(seed)
    g = _new(n_graphs, ["A", "B"], hv_size, hv_bits, init_with)
    g.set_number_of_graph_nodes_bulk(np.full(n_graphs, 2))
    g.prepare_node_configuration()
    g.set_nodes_bulk(np.ones(2 * n_graphs, dtype=np.uint32))
    g.prepare_edge_configuration()
    g.set_edges_bulk(np.tile([1, 0], n_graphs), np.zeros(2 * n_graphs, dtype=np.uint32), ["Plain"])
    sym = rng.integers(0, 2, size=(n_graphs, 2))
    ids = np.array([g.symbol_id["A"], g.symbol_id["B"]])
    g.add_graph_node_properties_bulk(np.arange(2 * n_graphs), ids[sym.ravel()])
    Y = (sym[:, 0] != sym[:, 1]).astype(np.uint32)
    flip = rng.random(n_graphs) <= noise
    Y[flip] = 1 - Y[flip]
    g.encode()
    return g, Y


# ------------------------------------------------------------------------------------------ configs 2, 3
def image_prototypes(seed, classes=10, side=28):
    """Per class, pixel on-probabilities drawn from U(0, 0.6)."""
    return np.random.default_rng(seed).uniform(0.0, 0.6, size=(classes, side * side))


def sample_images(prototypes, n, seed):
    rng = np.random.default_rng(seed)
    Y = rng.integers(0, prototypes.shape[0], size=n).astype(np.uint32)
    imgs = np.empty((n, prototypes.shape[1]), dtype=bool)
    for lo in range(0, n, 65536):
        y = Y[lo:lo + 65536]
        imgs[lo:lo + 65536] = rng.random((len(y), prototypes.shape[1])) < prototypes[y]
    return imgs, Y


def vanilla_images(n_graphs, seed, prototypes, hv_size=128, hv_bits=2, init_with=None):
    """One node per image; pixel i on => symbol i as a node property (MNISTVanillaDemo shape)."""
    n_pix = prototypes.shape[1]
    g = _new(n_graphs, list(range(n_pix)), hv_size, hv_bits, init_with)
    g.set_number_of_graph_nodes_bulk(np.ones(n_graphs))
    g.prepare_node_configuration()
    g.set_nodes_bulk(np.zeros(n_graphs, dtype=np.uint32))
    g.prepare_edge_configuration()
    g.set_edges_bulk([], [], [])
    imgs, Y = sample_images(prototypes, n_graphs, seed)
    _or_symbols(g, imgs, [g.symbol_id[i] for i in range(n_pix)])
    g.encode()
    return g, Y


def convolution_images(n_graphs, seed, prototypes, patch=10, hv_size=128, hv_bits=2, init_with=None):
    """One node per patch position (stride 1); node symbols = on-pixels of its patch (position inside the patch)
    plus thermometer-coded column and row symbols 'C:0..q', 'R:0..r' (CIFAR10Demo.py:109-113)."""
    side = int(round(np.sqrt(prototypes.shape[1])))
    dim = side - patch + 1
    symbols = []
    for i in range(dim):
        symbols += ["C:%d" % i, "R:%d" % i]
    symbols += list(range(patch * patch))
    g = _new(n_graphs, symbols, hv_size, hv_bits, init_with)
    g.set_number_of_graph_nodes_bulk(np.full(n_graphs, dim * dim))
    g.prepare_node_configuration()
    g.set_nodes_bulk(np.zeros(n_graphs * dim * dim, dtype=np.uint32))
    g.prepare_edge_configuration()
    g.set_edges_bulk([], [], [])
    imgs, Y = sample_images(prototypes, n_graphs, seed)
    imgs = imgs.reshape(n_graphs, side, side)
    ids = [g.symbol_id[i] for i in range(patch * patch)] + [g.symbol_id["C:%d" % i] for i in range(dim)] \
        + [g.symbol_id["R:%d" % i] for i in range(dim)]
    q = np.repeat(np.arange(dim), dim)
    r = np.tile(np.arange(dim), dim)
    thermo = np.concatenate([np.arange(dim)[None, :] <= q[:, None], np.arange(dim)[None, :] <= r[:, None]], axis=1)
    per_chunk = max(1, 16384 // (dim * dim))
    win = np.lib.stride_tricks.sliding_window_view(imgs, (patch, patch), axis=(1, 2))   # [n][dim][dim][p][p]
    for lo in range(0, n_graphs, per_chunk):
        w = win[lo:lo + per_chunk].reshape(-1, patch * patch)
        active = np.concatenate([w, np.tile(thermo, (w.shape[0] // (dim * dim), 1))], axis=1)
        sub = _RowWindow(g, lo * dim * dim, active.shape[0])
        _or_symbols(sub, active, ids, chunk=active.shape[0])
    g.encode()
    return g, Y


class _RowWindow:
    """View of a row range of a Graphs' X with the attributes `_or_symbols` reads."""

    def __init__(self, graphs, first, count):
        self.X = graphs.X[first:first + count]
        self.hypervectors = graphs.hypervectors
        self.hypervector_size = graphs.hypervector_size
        self.number_of_hypervector_chunks = graphs.number_of_hypervector_chunks


# ------------------------------------------------------------------------------------------ config 4
def sequences(n_graphs, seed, length=1000, hv_size=256, hv_bits=2, init_with=None):
    """Directed path graphs: one symbol of {A,B,C,D} per node, 'Left'/'Right' edges to the neighbours
    (SequenceClassificationDemo.py:54-72); label 1 iff some 'A' is followed within 3 positions by a 'B'."""
    rng = np.random.default_rng(seed)
    names = ["A", "B", "C", "D"]
    g = _new(n_graphs, names, hv_size, hv_bits, init_with)
    g.set_number_of_graph_nodes_bulk(np.full(n_graphs, length))
    g.prepare_node_configuration()
    deg = np.full((n_graphs, length), 2, dtype=np.uint32)
    deg[:, 0] = 1
    deg[:, -1] = 1
    if length == 1:
        deg[:] = 0
    g.set_nodes_bulk(deg.ravel())
    g.prepare_edge_configuration()
    pos = np.arange(length)
    dst = np.stack([pos - 1, pos + 1], axis=1).ravel()          # per node: Left first, then Right
    typ = np.tile([1, 0], length)                                # ids in order of first use: 'Right' = 0, 'Left' = 1
    keep = (dst >= 0) & (dst < length)
    g.set_edges_bulk(np.tile(dst[keep], n_graphs), np.tile(typ[keep], n_graphs), ["Right", "Left"])
    sym = rng.integers(0, 4, size=(n_graphs, length))
    ids = np.array([g.symbol_id[s] for s in names])
    g.add_graph_node_properties_bulk(np.arange(n_graphs * length), ids[sym.ravel()])
    is_a, is_b = sym == 0, sym == 1
    Y = np.zeros(n_graphs, dtype=bool)
    for k in (1, 2, 3):
        if length > k:
            Y |= np.any(is_a[:, :-k] & is_b[:, k:], axis=1)
    g.encode()
    return g, Y.astype(np.uint32)


# ------------------------------------------------------------------------------------------ config 5
def random_multigraphs(n_graphs, seed, min_nodes=8, max_nodes=32, mean_degree=3.0, edge_types=4, symbols=256,
                       max_props=5, classes=10, hv_size=1024, hv_bits=2, init_with=None):
    """Random directed multigraphs: node count uniform, out-degree Poisson, uniform targets and edge types,
    1..max_props symbols per node; label = argmax of a seeded random linear score over symbol counts."""
    rng = np.random.default_rng(seed)
    g = _new(n_graphs, list(range(symbols)), hv_size, hv_bits, init_with)
    n = rng.integers(min_nodes, max_nodes + 1, size=n_graphs)
    g.set_number_of_graph_nodes_bulk(n)
    g.prepare_node_configuration()
    total = int(n.sum())
    deg = rng.poisson(mean_degree, size=total).astype(np.uint32)
    g.set_nodes_bulk(deg)
    g.prepare_edge_configuration()
    node_graph = np.repeat(np.arange(n_graphs), n)
    src_graph = np.repeat(node_graph, deg)
    dst = (rng.random(len(src_graph)) * n[src_graph]).astype(np.uint32)
    typ = rng.integers(0, edge_types, size=len(src_graph))
    g.set_edges_bulk(dst, typ, ["E%d" % t for t in range(edge_types)])
    n_props = rng.integers(1, max_props + 1, size=total)
    rows = np.repeat(np.arange(total), n_props)
    syms = rng.integers(0, symbols, size=len(rows))
    ids = np.array([g.symbol_id[i] for i in range(symbols)])
    g.add_graph_node_properties_bulk(rows, ids[syms])
    score_w = np.random.default_rng(12345).normal(size=(symbols, classes))
    counts = np.zeros((n_graphs, symbols), dtype=np.float32)
    np.add.at(counts, (node_graph[rows], syms), 1.0)
    Y = np.argmax(counts @ score_w, axis=1).astype(np.uint32)
    g.encode()
    return g, Y


# ------------------------------------------------------------------------------------------ replication
def replicate(graphs, times):
    """A graph set made of `times` copies of `graphs` back to back (for throughput runs on tiny graphs)."""
    out = Graphs(graphs.number_of_graphs * times, init_with=graphs)
    out.set_number_of_graph_nodes_bulk(np.tile(graphs.number_of_graph_nodes, times))
    out.prepare_node_configuration()
    out.node_type[:] = np.tile(graphs.node_type, times)
    out.number_of_graph_node_edges[:] = np.tile(graphs.number_of_graph_node_edges, times)
    out.X[:] = np.tile(graphs.X, (times, 1))
    out.prepare_edge_configuration()
    out.edge[:] = np.tile(graphs.edge, (times, 1))
    out.graph_node_edge_counter[:] = out.number_of_graph_node_edges
    from .graphs import _LazyNodeIds

    out.graph_node_id = _LazyNodeIds(out.number_of_graph_nodes)
    out.encode()
    return out


class RepeatedGraphs:
    """`times` copies of `base` back to back, WITHOUT materialising them: a large global graph set for sharded
    scoring (``sharding.GraphShardScorer``), of which every rank only ever builds its own contiguous range.

    It has the attributes the scorer reads (``number_of_graphs``, ``number_of_graph_nodes``, ``signature``) and
    ``self[first:stop]``, which returns an ordinary ``Graphs`` holding copies of graphs ``first..stop-1`` of the
    repeated sequence (graph ``i`` is ``base[i % len(base)]``), equal to the same slice of ``replicate(base, times)``."""

    def __init__(self, base, times):
        import hashlib

        self.base = base
        self.times = int(times)
        self.number_of_graphs = int(base.number_of_graphs) * self.times
        self.number_of_graph_nodes = np.tile(base.number_of_graph_nodes, self.times)
        self.max_number_of_graph_nodes = base.max_number_of_graph_nodes
        self.signature = hashlib.sha256(bytes(base.signature) + b"x%d" % self.times).digest()

    def __len__(self):
        return self.number_of_graphs

    def number_of_node_types(self):
        return self.base.number_of_node_types()

    def __getitem__(self, index):
        if not isinstance(index, slice):
            raise TypeError("RepeatedGraphs supports contiguous slices only")
        first, stop, step = index.indices(self.number_of_graphs)
        if step != 1 or stop <= first:
            raise ValueError("RepeatedGraphs supports non-empty slices with step 1 only")
        n = int(self.base.number_of_graphs)
        if first % n == 0 and stop - first == n:
            return self.base                                    # exactly one copy: no need to build anything
        return self.base._create_subset(np.arange(first, stop) % n)
