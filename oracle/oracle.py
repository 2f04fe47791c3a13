"""TEST INFRASTRUCTURE ONLY (checker, never the product path).

ctypes front end of ``oracle/gtm_oracle.c``, the run-time parameterised CPU restatement of the reference's
fit / score arithmetic.  ``OracleTM`` mirrors ``oracle.ref_tm.RefTM`` so differential tests can drive either.
"""

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libgtm_oracle.so")


def build(force=False):
    src = os.path.join(HERE, "gtm_oracle.c")
    if force or not os.path.isfile(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["gcc", "-O2", "-std=c11", "-shared", "-fPIC", "-o", LIB_PATH, src], check=True)
    return LIB_PATH


class _Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "clauses", "classes", "literals", "state_bits", "boost", "threshold", "max_included",
        "message_size", "message_bits", "depth", "la_chunks", "message_chunks")] + [
        ("q", C.c_double), ("s", C.c_float * 16)]


class _Model(C.Structure):
    _fields_ = [("ta_state", C.c_void_p), ("message_ta_state", C.c_void_p * 15), ("clause_weights", C.c_void_p),
                ("hypervectors", C.c_void_p), ("draw_pos", C.c_void_p), ("seed", C.c_uint64),
                ("recorded", C.c_void_p), ("recorded_len", C.c_uint64)]


class _Graphs(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "X", "node_type", "number_of_graph_node_edges", "edge_index", "edge", "node_index",
        "number_of_graph_nodes")] + [("number_of_graphs", C.c_int32), ("number_of_node_types", C.c_int32)]


class _Scratch(C.Structure):
    _fields_ = [("cno", C.c_void_p), ("cno_stride", C.c_int32), ("messages", C.c_void_p), ("max_nodes", C.c_int32),
                ("n_inc", C.c_void_p), ("class_sum", C.c_void_p), ("clause_node", C.c_void_p), ("update", C.c_void_p)]


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def philox4x32_10(ctr, key):
    lib = C.CDLL(build())
    c = (C.c_uint32 * 4)(*ctr)
    k = (C.c_uint32 * 2)(*key)
    o = (C.c_uint32 * 4)()
    lib.orc_philox4x32_10(c, k, o)
    return [int(v) for v in o]


def round_q(q):
    """The reference bakes q into its kernels through a ``%f`` format (tm.py:445,458): six decimals."""
    return float("%f" % q)


class OracleTM:
    def __init__(self, *, clauses, classes, literals, threshold, s, depth=1, message_size=256, message_bits=2,
                 max_included=None, boost=1, state_bits=8, q=1.0, max_nodes=1, hypervectors=None, seed=1,
                 recorded=None):
        self.lib = lib = C.CDLL(build())
        assert [lib.orc_sizeof(i) for i in range(4)] == [C.sizeof(t) for t in (_Config, _Model, _Graphs, _Scratch)]
        self.C, self.K, self.SB, self.depth = clauses, classes, state_bits, depth
        self.literals, self.message_size, self.message_bits = literals, message_size, message_bits
        self.la_chunks = (literals - 1) // 32 + 1
        self.message_chunks = (2 * message_size - 1) // 32 + 1
        self.max_nodes = max_nodes
        self.node_chunks = (max_nodes - 1) // 32 + 1
        self.s = tuple(s) if isinstance(s, (tuple, list)) else (s,) * depth
        cfg = self.cfg = _Config()
        cfg.clauses, cfg.classes, cfg.literals, cfg.state_bits = clauses, classes, literals, state_bits
        cfg.boost, cfg.threshold = boost, threshold
        cfg.max_included = literals if max_included is None else max_included
        cfg.message_size, cfg.message_bits, cfg.depth = message_size, message_bits, depth
        cfg.la_chunks, cfg.message_chunks = self.la_chunks, self.message_chunks
        cfg.q = round_q(q)
        for d, v in enumerate(self.s):
            cfg.s[d] = v

        self.ta_state = np.zeros((clauses, self.la_chunks, state_bits), dtype=np.uint32)
        self.message_ta_state = [np.zeros((clauses, self.message_chunks, state_bits), dtype=np.uint32)
                                 for _ in range(depth - 1)]
        self.clause_weights = np.zeros((classes, clauses), dtype=np.int32)
        if hypervectors is None:
            hypervectors = np.zeros((clauses, message_bits), dtype=np.uint32)
        self.hypervectors = np.ascontiguousarray(hypervectors, dtype=np.uint32)
        self.draw_pos = np.zeros(clauses, dtype=np.uint64)
        self.recorded = None if recorded is None else np.ascontiguousarray(recorded, dtype=np.uint32)
        m = self.model = _Model()
        m.ta_state = _ptr(self.ta_state)
        for d in range(depth - 1):
            m.message_ta_state[d] = self.message_ta_state[d].ctypes.data
        m.clause_weights, m.hypervectors = _ptr(self.clause_weights), _ptr(self.hypervectors)
        m.draw_pos, m.seed = _ptr(self.draw_pos), seed
        m.recorded = _ptr(self.recorded)
        m.recorded_len = 0 if self.recorded is None else self.recorded.shape[1]

        self.cno = np.zeros((depth, clauses, self.node_chunks), dtype=np.uint32)
        self.messages = np.zeros((max(depth - 1, 1), max_nodes, self.message_chunks), dtype=np.uint32)
        self.n_inc = np.zeros(clauses, dtype=np.int32)
        self.class_sum = np.zeros(classes, dtype=np.int32)
        self.clause_node = np.zeros(clauses, dtype=np.int32)
        self.update = np.zeros((classes, clauses), dtype=np.int32)
        sc = self.scratch = _Scratch()
        sc.cno, sc.cno_stride = _ptr(self.cno), self.node_chunks
        sc.messages, sc.max_nodes = _ptr(self.messages), max_nodes
        sc.n_inc, sc.class_sum = _ptr(self.n_inc), _ptr(self.class_sum)
        sc.clause_node, sc.update = _ptr(self.clause_node), _ptr(self.update)
        self.graphs = None

    def set_graphs(self, graphs):
        assert int(graphs.max_number_of_graph_nodes) <= self.max_nodes
        self._g = g = dict(
            X=np.ascontiguousarray(graphs.X, dtype=np.uint32),
            node_type=np.ascontiguousarray(graphs.node_type, dtype=np.uint32),
            n_edges=np.ascontiguousarray(graphs.number_of_graph_node_edges, dtype=np.uint32),
            edge_index=np.ascontiguousarray(graphs.edge_index, dtype=np.uint32),
            edge=np.ascontiguousarray(graphs.edge, dtype=np.uint32) if graphs.edge.size
            else np.zeros((1, 2), dtype=np.uint32),
            node_index=np.ascontiguousarray(graphs.node_index, dtype=np.uint32),
            n_nodes=np.ascontiguousarray(graphs.number_of_graph_nodes, dtype=np.uint32))
        gs = self.graphs = _Graphs()
        gs.X, gs.node_type = _ptr(g["X"]), _ptr(g["node_type"])
        gs.number_of_graph_node_edges, gs.edge_index = _ptr(g["n_edges"]), _ptr(g["edge_index"])
        gs.edge, gs.node_index = _ptr(g["edge"]), _ptr(g["node_index"])
        gs.number_of_graph_nodes = _ptr(g["n_nodes"])
        gs.number_of_graphs = self.number_of_graphs = len(g["n_nodes"])
        gs.number_of_node_types = graphs.number_of_node_types()

    def prepare(self, reset_message_layers=True):
        self.lib.orc_prepare(C.byref(self.cfg), C.byref(self.model), int(reset_message_layers))

    def evaluate_graph(self, e):
        self.lib.orc_evaluate_graph(C.byref(self.cfg), C.byref(self.model), C.byref(self.graphs), int(e),
                                    C.byref(self.scratch))
        n = int(self._g["n_nodes"][e])
        return dict(cno=self.cno.copy(), messages=[self.messages[d, :n].copy() for d in range(self.depth - 1)],
                    n_inc=self.n_inc.copy(), class_sum=self.class_sum.copy())

    def score(self, first=0, count=None):
        count = self.number_of_graphs - first if count is None else count
        out = np.zeros((count, self.K), dtype=np.int32)
        self.lib.orc_score(C.byref(self.cfg), C.byref(self.model), C.byref(self.graphs), int(first), int(count),
                           C.byref(self.scratch), _ptr(out))
        return out

    def fit(self, encoded_Y, first=0, count=None):
        count = self.number_of_graphs - first if count is None else count
        y = np.ascontiguousarray(encoded_Y, dtype=np.int32)
        self.lib.orc_fit(C.byref(self.cfg), C.byref(self.model), C.byref(self.graphs), _ptr(y), int(first),
                         int(count), C.byref(self.scratch))

    def draws_consumed(self):
        return self.draw_pos.copy()
