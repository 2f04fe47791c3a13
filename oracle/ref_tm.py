"""TEST INFRASTRUCTURE ONLY (checker, never the product path).

Drives the host-compiled reference kernels (``oracle/_ref/ref_<key>.so``, see ``oracle/build_ref.py``):
allocates the buffers with the sizes of ``GraphTsetlinMachine/tm.py:110-124`` and ``:528-555``, hands them to
the C restatement of the reference's launch order (``oracle/ref_driver.inc``) and exposes the intermediates
that differential tests compare: node outputs per layer, packed messages per layer, include counts, class
sums, selected nodes, feedback decisions, weights and Tsetlin-automaton planes.

One RNG stream per launched thread, one thread per clause (``nthreads == number_of_clauses``), so stream ``i``
belongs to clause ``i`` exactly as with the reference's default launch shape (106,496 threads >= clauses).
"""

import ctypes as C

import numpy as np

from . import build_ref


class _Ctx(C.Structure):
    _fields_ = [
        ("ta_state", C.c_void_p),
        ("message_ta_state", C.c_void_p * 15),
        ("clause_weights", C.c_void_p),
        ("hypervectors", C.c_void_p),
        ("state", C.c_void_p),
        ("s", C.c_float * 16),
        ("depth", C.c_int),
        ("nthreads", C.c_int),
        ("X", C.c_void_p),
        ("node_type", C.c_void_p),
        ("number_of_graph_node_edges", C.c_void_p),
        ("edge", C.c_void_p),
        ("node_index", C.c_void_p),
        ("number_of_graph_nodes", C.c_void_p),
        ("edge_index", C.c_void_p),
        ("number_of_node_types", C.c_int),
        ("cno_a", C.c_void_p),
        ("cno_b", C.c_void_p),
        ("clause_X_int", C.c_void_p),
        ("clause_X", C.c_void_p * 15),
        ("class_sum", C.c_void_p),
        ("clause_node", C.c_void_p),
        ("number_of_include_actions", C.c_void_p),
        ("class_clause_update", C.c_void_p),
        ("dump_cno", C.c_void_p),
    ]


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class RefTM:
    """Reference kernels on the host for one hyper-parameter set."""

    def __init__(self, *, clauses, classes, literals, threshold, s, depth=1, message_size=256, message_bits=2,
                 max_included=None, boost=1, state_bits=8, q=1.0, max_nodes=1, hypervectors=None, seed=1,
                 recorded=None):
        self.params = build_ref.normalise(dict(
            classes=classes, clauses=clauses, literals=literals, state_bits=state_bits, boost=boost,
            threshold=threshold, q=q, max_included=max_included, negative_clauses=1, max_nodes=max_nodes,
            message_size=message_size, message_bits=message_bits))
        path = build_ref.build(self.params)
        if path is None:
            raise FileNotFoundError("no host build of the reference kernels for %r" % (self.params,))
        self.lib = lib = C.CDLL(path)
        cfg = (C.c_int * 16)()
        lib.ref_get_config(cfg)
        self.la_chunks, self.message_chunks, self.node_chunks = cfg[11], cfg[12], cfg[13]
        assert cfg[15] == C.sizeof(_Ctx), "ref_ctx layout mismatch"
        self.C, self.K, self.SB, self.depth = clauses, classes, state_bits, depth
        self.max_nodes, self.message_size, self.message_bits = max_nodes, message_size, message_bits
        self.s = tuple(s) if isinstance(s, (tuple, list)) else (s,) * depth

        lib.ref_evaluate_graph.restype = C.c_void_p
        lib.ref_state_pos.restype = C.c_ulonglong
        lib.ref_seed_states.argtypes = [C.c_void_p, C.c_int, C.c_ulonglong, C.c_void_p, C.c_ulonglong]

        self.ta_state = np.zeros((clauses, self.la_chunks, state_bits), dtype=np.uint32)
        self.message_ta_state = [np.zeros((clauses, self.message_chunks, state_bits), dtype=np.uint32)
                                 for _ in range(depth - 1)]
        self.clause_weights = np.zeros((classes, clauses), dtype=np.int32)
        if hypervectors is None:
            hypervectors = np.zeros((clauses, message_bits), dtype=np.uint32)
        self.hypervectors = np.ascontiguousarray(hypervectors, dtype=np.int32)
        self.state = np.zeros(clauses * cfg[14], dtype=np.uint8)
        self.recorded = None if recorded is None else np.ascontiguousarray(recorded, dtype=np.uint32)
        lib.ref_seed_states(_ptr(self.state), clauses, seed, _ptr(self.recorded),
                            0 if self.recorded is None else self.recorded.shape[1])

        self.cno_a = np.zeros((clauses, self.node_chunks), dtype=np.int32)
        self.cno_b = np.zeros((clauses, self.node_chunks), dtype=np.int32)
        self.clause_X_int = np.zeros((max_nodes, 2 * message_size), dtype=np.uint32)
        self.clause_X = [np.zeros((max_nodes, self.message_chunks), dtype=np.uint32) for _ in range(depth - 1)]
        self.class_sum = np.zeros(classes, dtype=np.int32)
        self.clause_node = np.zeros(clauses, dtype=np.int32)
        self.number_of_include_actions = np.zeros(clauses, dtype=np.int32)
        self.class_clause_update = np.zeros((classes, clauses), dtype=np.int32)
        self.dump_cno = np.zeros((depth, clauses, self.node_chunks), dtype=np.int32)
        self.ctx = _Ctx()
        self._graphs = None
        self._fill()

    def _fill(self):
        c = self.ctx
        c.ta_state = _ptr(self.ta_state)
        for d in range(self.depth - 1):
            c.message_ta_state[d] = self.message_ta_state[d].ctypes.data
            c.clause_X[d] = self.clause_X[d].ctypes.data
        c.clause_weights = _ptr(self.clause_weights)
        c.hypervectors = _ptr(self.hypervectors)
        c.state = _ptr(self.state)
        for d, v in enumerate(self.s):
            c.s[d] = v
        c.depth, c.nthreads = self.depth, self.C
        c.cno_a, c.cno_b = _ptr(self.cno_a), _ptr(self.cno_b)
        c.clause_X_int = _ptr(self.clause_X_int)
        c.class_sum, c.clause_node = _ptr(self.class_sum), _ptr(self.clause_node)
        c.number_of_include_actions = _ptr(self.number_of_include_actions)
        c.class_clause_update = _ptr(self.class_clause_update)
        c.dump_cno = _ptr(self.dump_cno)

    def set_graphs(self, graphs):
        """Point the context at a graph set (any object with the array attributes of ``Graphs``)."""
        assert int(graphs.max_number_of_graph_nodes) <= self.max_nodes
        self._graphs = g = dict(
            X=np.ascontiguousarray(graphs.X, dtype=np.uint32),
            node_type=np.ascontiguousarray(graphs.node_type, dtype=np.uint32).view(np.int32),
            n_edges=np.ascontiguousarray(graphs.number_of_graph_node_edges, dtype=np.uint32).view(np.int32),
            edge=np.ascontiguousarray(graphs.edge, dtype=np.uint32).view(np.int32).reshape(-1, 2)
            if graphs.edge.size else np.zeros((1, 2), dtype=np.int32),
            node_index=np.ascontiguousarray(graphs.node_index, dtype=np.uint32),
            n_nodes=np.ascontiguousarray(graphs.number_of_graph_nodes, dtype=np.uint32),
            edge_index=np.ascontiguousarray(graphs.edge_index, dtype=np.uint32),
        )
        c = self.ctx
        c.X, c.node_type = _ptr(g["X"]), _ptr(g["node_type"])
        c.number_of_graph_node_edges, c.edge = _ptr(g["n_edges"]), _ptr(g["edge"])
        c.node_index, c.number_of_graph_nodes = _ptr(g["node_index"]), _ptr(g["n_nodes"])
        c.edge_index = _ptr(g["edge_index"])
        c.number_of_node_types = graphs.number_of_node_types()
        self.number_of_graphs = len(g["n_nodes"])

    # -- passes -------------------------------------------------------------------------------------------
    def prepare(self, reset_message_layers=True):
        self.lib.ref_prepare(C.byref(self.ctx), int(reset_message_layers))

    def evaluate_graph(self, e):
        """Inference on graph ``e``; returns dict of intermediates (copies)."""
        self.lib.ref_evaluate_graph(C.byref(self.ctx), int(e))
        n = int(self._graphs["n_nodes"][e])
        return dict(
            cno=self.dump_cno.view(np.uint32).copy(),
            messages=[m[:n].copy() for m in self.clause_X],
            n_inc=self.number_of_include_actions.copy(),
            class_sum=self.class_sum.copy(),
        )

    def score(self, first=0, count=None):
        count = self.number_of_graphs - first if count is None else count
        out = np.zeros((count, self.K), dtype=np.int32)
        self.lib.ref_score_graphs(C.byref(self.ctx), int(first), int(count), _ptr(out))
        return out

    def fit(self, encoded_Y, first=0, count=None):
        count = self.number_of_graphs - first if count is None else count
        self._y = np.ascontiguousarray(encoded_Y, dtype=np.int32)
        self.lib.ref_fit_graphs(C.byref(self.ctx), _ptr(self._y), int(first), int(count))

    def transform_graph(self, e, nodewise=False):
        n = int(self._graphs["n_nodes"][e])
        if nodewise:
            out = np.zeros((self.C, n), dtype=np.int32)
            self.lib.ref_transform_nodewise_graph(C.byref(self.ctx), int(e), _ptr(out))
        else:
            out = np.zeros(self.C, dtype=np.int32)
            self.lib.ref_transform_graph(C.byref(self.ctx), int(e), _ptr(out))
        return out

    def get_ta_states(self, layer):
        ta = self.ta_state if layer == 0 else self.message_ta_state[layer - 1]
        literals = self.params["literals"] if layer == 0 else 2 * self.message_size
        out = np.zeros((self.C, literals), dtype=np.uint32)
        self.lib.ref_get_ta_states(C.byref(self.ctx), _ptr(ta), C.c_uint(ta.shape[1]), C.c_uint(literals), _ptr(out))
        return out

    def get_hyperliterals(self, layer):
        ta = self.ta_state if layer == 0 else self.message_ta_state[layer - 1]
        literals = self.params["literals"] if layer == 0 else 2 * self.message_size
        out = np.zeros((self.C, literals), dtype=np.uint32)
        self.lib.ref_get_hyperliterals(C.byref(self.ctx), _ptr(ta), C.c_uint(ta.shape[1]), C.c_uint(literals), _ptr(out))
        return out

    def draws_consumed(self):
        return np.array([self.lib.ref_state_pos(_ptr(self.state), i) for i in range(self.C)], dtype=np.uint64)
