"""TEST / BASELINE INFRASTRUCTURE ONLY (checker, never the product path).

Drives the reference's own kernels compiled for the GPU (``oracle/_ref/refgpu_<key>.so``, see
``oracle/build_ref.py:build_gpu`` and ``oracle/ref_gpu_driver.inc``): same launch shape, launch order and
per-graph host round trips as ``GraphTsetlinMachine/tm.py:563-812``, with cuRAND XORWOW states as the reference
uses them.  Two uses: inference from an identical loaded state is compared bit for bit with the engine on the same
GPU, and its fit/score loops are timed as "the reference on this GPU".  Learning is not draw-for-draw comparable
(XORWOW per launched thread vs. one Philox stream per clause); it is compared statistically.
"""

import ctypes as C

import numpy as np

from . import build_ref


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class RefGpuTM:
    def __init__(self, *, clauses, classes, literals, threshold, s, depth=1, message_size=256, message_bits=2,
                 max_included=None, boost=1, state_bits=8, q=1.0, max_nodes=1, hypervectors=None, seed=1, **_unused):
        self.params = build_ref.normalise(dict(
            classes=classes, clauses=clauses, literals=literals, state_bits=state_bits, boost=boost,
            threshold=threshold, q=q, max_included=max_included, negative_clauses=1, max_nodes=max_nodes,
            message_size=message_size, message_bits=message_bits))
        path = build_ref.build_gpu(self.params)
        if path is None:
            raise FileNotFoundError("no GPU build of the reference kernels for %r" % (self.params,))
        self.lib = lib = C.CDLL(path)
        cfg = (C.c_int * 16)()
        lib.refgpu_get_config(cfg)
        assert (cfg[0], cfg[1], cfg[2], cfg[3]) == (classes, clauses, literals, state_bits)
        self.la_chunks, self.message_chunks, self.node_chunks = cfg[11], cfg[12], cfg[13]
        self.C, self.K, self.SB, self.depth = clauses, classes, state_bits, depth
        self.max_nodes, self.message_size = max_nodes, message_size
        s = tuple(s) if isinstance(s, (tuple, list)) else (s,) * depth
        lib.refgpu_create.restype = C.c_void_p
        lib.refgpu_create.argtypes = [C.c_int, C.c_void_p, C.c_ulonglong]
        for name in ("refgpu_destroy", "refgpu_prepare"):
            getattr(lib, name).argtypes = [C.c_void_p]
        lib.refgpu_set_model.argtypes = [C.c_void_p] * 5
        lib.refgpu_get_model.argtypes = [C.c_void_p] * 4
        lib.refgpu_set_graphs.argtypes = [C.c_void_p] * 8 + [C.c_int, C.c_longlong, C.c_longlong, C.c_int]
        lib.refgpu_score.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        lib.refgpu_evaluate_graph.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 4
        lib.refgpu_fit.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        self.handle = lib.refgpu_create(depth, _ptr(np.asarray(s, dtype=np.float32)), seed)
        if not self.handle:
            raise RuntimeError("the reference's GPU buffers could not be created")
        if hypervectors is None:
            hypervectors = np.zeros((clauses, message_bits), dtype=np.uint32)
        self.hypervectors = np.ascontiguousarray(hypervectors, dtype=np.uint32).view(np.int32)
        self.ta_state = np.zeros((clauses, self.la_chunks, state_bits), dtype=np.uint32)
        self.message_ta_state = [np.zeros((clauses, self.message_chunks, state_bits), dtype=np.uint32)
                                 for _ in range(depth - 1)]
        self.clause_weights = np.zeros((classes, clauses), dtype=np.int32)
        self._graphs = None

    def close(self):
        if self.handle:
            self.lib.refgpu_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _pointer_table(self):
        table = (C.c_void_p * 15)()
        for d, m in enumerate(self.message_ta_state):
            table[d] = m.ctypes.data
        return table

    def upload(self):
        """Host copies of automata / weights / hypervectors -> device."""
        self.lib.refgpu_set_model(self.handle, _ptr(self.ta_state), C.cast(self._pointer_table(), C.c_void_p),
                                  _ptr(self.clause_weights), _ptr(self.hypervectors))

    def download(self):
        self.lib.refgpu_get_model(self.handle, _ptr(self.ta_state), C.cast(self._pointer_table(), C.c_void_p),
                                  _ptr(self.clause_weights))

    def load_from(self, other):
        self.ta_state[...] = other.ta_state
        for mine, theirs in zip(self.message_ta_state, other.message_ta_state):
            mine[...] = theirs
        self.clause_weights[...] = other.clause_weights
        self.upload()

    def prepare(self):
        self.upload()                       # hypervectors; the automata are then reset on the device
        self.lib.refgpu_prepare(self.handle)

    def set_graphs(self, graphs):
        # graphs with more nodes than MAX_NODES would index past the reference's per-thread arrays
        assert int(graphs.max_number_of_graph_nodes) <= self.max_nodes
        u32 = lambda a: np.ascontiguousarray(a, dtype=np.uint32)
        g = self._graphs = dict(X=u32(graphs.X), node_type=u32(graphs.node_type),
                                n_edges=u32(graphs.number_of_graph_node_edges),
                                edge=u32(graphs.edge) if graphs.edge.size else None, node_index=u32(graphs.node_index),
                                n_nodes=u32(graphs.number_of_graph_nodes), edge_index=u32(graphs.edge_index))
        assert g["X"].shape[1] == self.la_chunks
        total_edges = int(graphs.edge.shape[0]) if graphs.edge.size else 0
        self.number_of_graphs = len(g["n_nodes"])
        self.lib.refgpu_set_graphs(self.handle, _ptr(g["X"]), _ptr(g["node_type"]), _ptr(g["n_edges"]), _ptr(g["edge"]),
                                   _ptr(g["node_index"]), _ptr(g["n_nodes"]), _ptr(g["edge_index"]),
                                   self.number_of_graphs, g["X"].shape[0], total_edges, graphs.number_of_node_types())

    def evaluate_graph(self, e):
        n = int(self._graphs["n_nodes"][e])
        cno = np.zeros((self.depth, self.C, self.node_chunks), dtype=np.uint32)
        msgs = np.zeros((max(self.depth - 1, 1), self.max_nodes, self.message_chunks), dtype=np.uint32)
        n_inc = np.zeros(self.C, dtype=np.int32)
        cs = np.zeros(self.K, dtype=np.int32)
        status = self.lib.refgpu_evaluate_graph(self.handle, int(e), _ptr(cno), _ptr(msgs), _ptr(n_inc), _ptr(cs))
        assert status == 0, "CUDA error %d" % status
        words = (n - 1) // 32 + 1
        return dict(cno=cno[:, :, :words].copy(), messages=[msgs[d, :n].copy() for d in range(self.depth - 1)],
                    n_inc=n_inc, class_sum=cs)

    def score(self, first=0, count=None):
        count = self.number_of_graphs - first if count is None else count
        out = np.zeros((count, self.K), dtype=np.int32)
        status = self.lib.refgpu_score(self.handle, int(first), int(count), _ptr(out))
        assert status == 0, "CUDA error %d" % status
        return out

    def fit(self, encoded_Y, first=0, count=None):
        count = self.number_of_graphs - first if count is None else count
        y = np.ascontiguousarray(encoded_Y, dtype=np.int32)
        assert y.shape == (self.number_of_graphs, self.K)
        status = self.lib.refgpu_fit(self.handle, _ptr(y), int(first), int(count))
        assert status == 0, "CUDA error %d" % status
