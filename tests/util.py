"""Shared helpers of the test-suite: seeded random graph sets and a thin driver of the C ABI that exposes the
same surface as the two CPU checkers (``oracle.ref_tm.RefTM`` and ``oracle.oracle.OracleTM``)."""

import ctypes as C

import numpy as np

from graphtsetlinmachine_b200 import _lib
from graphtsetlinmachine_b200.graphs import Graphs


def random_graphs(n_graphs, rng, *, symbols=12, hv_size=32, hv_bits=2, max_nodes=5, node_types=1, edge_types=2,
                  max_degree=3, max_props=3, init_with=None, fixed_nodes=None):
    """Seeded random graph set built through the public per-item API (self-loops and multi-edges included)."""
    names = ["s%d" % i for i in range(symbols)]
    if init_with is None:
        g = Graphs(n_graphs, symbols=names, hypervector_size=hv_size, hypervector_bits=hv_bits)
    else:
        g = Graphs(n_graphs, init_with=init_with)
    ns = rng.integers(1, max_nodes + 1, size=n_graphs) if fixed_nodes is None else np.full(n_graphs, fixed_nodes)
    for i in range(n_graphs):
        g.set_number_of_graph_nodes(i, int(ns[i]))
    g.prepare_node_configuration()
    degrees = []
    for i in range(n_graphs):
        d = rng.integers(0, max_degree + 1, size=ns[i])
        degrees.append(d)
        for v in range(ns[i]):
            g.add_graph_node(i, v, int(d[v]), "T%d" % rng.integers(0, node_types))
    g.prepare_edge_configuration()
    for i in range(n_graphs):
        for v in range(ns[i]):
            for _ in range(degrees[i][v]):
                g.add_graph_node_edge(i, v, int(rng.integers(0, ns[i])), "E%d" % rng.integers(0, edge_types))
            for name in rng.choice(names, size=rng.integers(0, max_props + 1)):
                g.add_graph_node_property(i, v, str(name))
    g.encode()
    return g


def encode_labels(Y, K, T):
    return np.where(np.asarray(Y)[:, None] == np.arange(K)[None, :], T, -T).astype(np.int32)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class EngineTM:
    """The CUDA engine behind the C ABI, with the method names of the CPU checkers."""

    def __init__(self, *, clauses, classes, literals, threshold, s, depth=1, message_size=256, message_bits=2,
                 max_included=None, boost=1, state_bits=8, q=1.0, max_nodes=1, hypervectors=None, seed=1,
                 recorded=None, device=0, options=None):
        self.lib = lib = _lib.load()
        self.C, self.K, self.SB, self.depth = clauses, classes, state_bits, depth
        self.literals, self.message_size = literals, message_size
        self.la_chunks = (literals - 1) // 32 + 1
        self.message_chunks = (2 * message_size - 1) // 32 + 1
        cfg = _lib.Config()
        cfg.number_of_clauses, cfg.number_of_outputs, cfg.number_of_literals = clauses, classes, literals
        cfg.number_of_state_bits, cfg.boost_true_positive_feedback, cfg.T = state_bits, boost, threshold
        cfg.max_included_literals = literals if max_included is None else max_included
        cfg.message_size, cfg.message_bits, cfg.depth, cfg.device = message_size, message_bits, depth, device
        cfg.q = float("%f" % q)
        s = tuple(s) if isinstance(s, (tuple, list)) else (s,) * depth
        for d, v in enumerate(s):
            cfg.s[d] = v
        cfg.seed = seed
        self.model = C.c_void_p()
        _lib.check(lib.gtm_create(C.byref(cfg), C.byref(self.model)))
        if hypervectors is not None:
            _lib.check(lib.gtm_set_hypervectors(self.model, _ptr(np.ascontiguousarray(hypervectors, dtype=np.uint32))))
        if recorded is not None:
            rec = np.ascontiguousarray(recorded, dtype=np.uint32)
            _lib.check(lib.gtm_set_recorded_draws(self.model, _ptr(rec), rec.shape[1]))
        for name, value in (options or {}).items():
            _lib.check(lib.gtm_set_option(self.model, name.encode(), int(value)))
        self.ds = C.c_void_p()
        self.graphs = None

    def close(self):
        if self.ds:
            self.lib.gtm_dataset_destroy(self.ds)
            self.ds = C.c_void_p()
        if self.model:
            self.lib.gtm_destroy(self.model)
            self.model = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_graphs(self, graphs):
        if self.ds:
            self.lib.gtm_dataset_destroy(self.ds)
            self.ds = C.c_void_p()
        u32 = lambda a: np.ascontiguousarray(a, dtype=np.uint32)
        arrays = [u32(graphs.X), u32(graphs.node_type), u32(graphs.number_of_graph_node_edges), u32(graphs.edge_index),
                  u32(graphs.edge) if graphs.edge.size else None, u32(graphs.node_index), u32(graphs.number_of_graph_nodes)]
        v = _lib.GraphsView()
        (v.X, v.node_type, v.number_of_graph_node_edges, v.edge_index, v.edge, v.node_index,
         v.number_of_graph_nodes) = [_ptr(a) for a in arrays]
        v.number_of_graphs, v.total_nodes = int(graphs.number_of_graphs), int(arrays[0].shape[0])
        v.total_edges = int(graphs.edge.shape[0]) if graphs.edge.size else 0
        v.max_number_of_graph_nodes = int(graphs.max_number_of_graph_nodes)
        _lib.check(self.lib.gtm_dataset_create(self.model, C.byref(v), C.byref(self.ds)))
        self.graphs = graphs
        self.n_types = graphs.number_of_node_types()
        self.number_of_graphs = int(graphs.number_of_graphs)

    def prepare(self, reset_message_layers=True):
        _lib.check(self.lib.gtm_init_state(self.model, int(reset_message_layers)))

    def _chunks(self, layer):
        return self.la_chunks if layer == 0 else self.message_chunks

    def get_ta(self, layer):
        out = np.zeros((self.C, self._chunks(layer), self.SB), dtype=np.uint32)
        _lib.check(self.lib.gtm_get_ta_state(self.model, layer, _ptr(out)))
        return out

    def set_ta(self, layer, ta):
        _lib.check(self.lib.gtm_set_ta_state(self.model, layer, _ptr(np.ascontiguousarray(ta, dtype=np.uint32))))

    @property
    def ta_state(self):
        return self.get_ta(0)

    @property
    def message_ta_state(self):
        return [self.get_ta(d + 1) for d in range(self.depth - 1)]

    @property
    def clause_weights(self):
        out = np.zeros((self.K, self.C), dtype=np.int32)
        _lib.check(self.lib.gtm_get_weights(self.model, _ptr(out)))
        return out

    def set_weights(self, w):
        _lib.check(self.lib.gtm_set_weights(self.model, _ptr(np.ascontiguousarray(w, dtype=np.int32))))

    def load_from(self, other):
        """Copy automata, weights and draw positions from a CPU checker."""
        self.set_ta(0, other.ta_state)
        for d in range(self.depth - 1):
            self.set_ta(d + 1, other.message_ta_state[d])
        self.set_weights(other.clause_weights)
        pos = np.ascontiguousarray(other.draws_consumed(), dtype=np.uint64)
        _lib.check(self.lib.gtm_set_draw_positions(self.model, _ptr(pos)))

    def draws_consumed(self):
        out = np.zeros(self.C, dtype=np.uint64)
        _lib.check(self.lib.gtm_get_draw_positions(self.model, _ptr(out)))
        return out

    def evaluate_graph(self, e, path=0):
        n = int(self.graphs.number_of_graph_nodes[e])
        words = (n - 1) // 32 + 1
        cno = np.zeros((self.depth, self.C, words), dtype=np.uint32)
        msgs = np.zeros((max(self.depth - 1, 1), n, self.message_chunks), dtype=np.uint32)
        n_inc = np.zeros(self.C, dtype=np.int32)
        cs = np.zeros(self.K, dtype=np.int32)
        _lib.check(self.lib.gtm_debug_evaluate(self.model, self.ds, self.n_types, int(e), int(path), _ptr(cno), _ptr(msgs),
                                               _ptr(n_inc), _ptr(cs)))
        return dict(cno=cno, messages=[msgs[d] for d in range(self.depth - 1)], n_inc=n_inc, class_sum=cs)

    def score(self, first=0, count=None):
        count = self.number_of_graphs - first if count is None else count
        out = np.zeros((count, self.K), dtype=np.int32)
        _lib.check(self.lib.gtm_score(self.model, self.ds, self.n_types, int(first), int(count), _ptr(out)))
        return out

    def transform(self, first=0, count=None):
        count = self.number_of_graphs - first if count is None else count
        co = np.zeros((count, self.C), dtype=np.int32)
        cs = np.zeros((count, self.K), dtype=np.int32)
        _lib.check(self.lib.gtm_transform(self.model, self.ds, self.n_types, int(first), int(count), _ptr(co), _ptr(cs)))
        return co, cs

    def fit(self, encoded_Y, first=0, count=None, epochs=1):
        count = self.number_of_graphs - first if count is None else count
        y = np.ascontiguousarray(encoded_Y, dtype=np.int32)
        _lib.check(self.lib.gtm_fit(self.model, self.ds, self.n_types, _ptr(y), int(first), int(count), int(epochs)))

    def last_feedback(self):
        node = np.zeros(self.C, dtype=np.int32)
        upd = np.zeros((self.K, self.C), dtype=np.int32)
        _lib.check(self.lib.gtm_debug_last_feedback(self.model, _ptr(node), _ptr(upd)))
        return node, upd
