"""Graph Tsetlin Machine model classes over the B200 engine (``libgtm_b200.so``, C ABI in ``include/gtm_b200.h``).

Drop-in for the reference ``GraphTsetlinMachine/tm.py``: ``CommonTsetlinMachine`` (tm.py:38-900) and its three
subclasses ``MultiClassGraphTsetlinMachine`` (tm.py:903-959), ``MultiOutputGraphTsetlinMachine`` (tm.py:961-1017)
and ``GraphTsetlinMachine`` (tm.py:1019-1072), with the same constructor arguments, methods, attribute names and
array layouts.  Where the reference drives PyCUDA (JIT, ``prepared_call``, ``mem_alloc``, ``memcpy``), this module
calls the C ABI through ctypes; there is no other execution path.

Differences a user can observe:

* ``grid`` / ``block`` are accepted and ignored (the engine sizes its own launches).
* Randomness comes from one Philox4x32-10 stream per clause keyed by ``seed`` (new optional argument; by default
  taken from ``os.urandom``), not from PyCUDA's XORWOW generator, whose seeding is random per process anyway.
* A test set may have larger graphs than the training set (the reference indexes out of bounds, tm.py:765).
"""

import ctypes as C
import os
import pickle
import sys

import numpy as np

from . import _lib

__all__ = ["CommonTsetlinMachine", "MultiClassGraphTsetlinMachine", "MultiOutputGraphTsetlinMachine",
           "GraphTsetlinMachine"]


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


class _Dataset:
    """A graph set resident on the device (the uploads of tm.py:528-555 / :759-784)."""

    def __init__(self, lib, model, graphs, class_sums_out=None):
        """With `class_sums_out` (int32[N][outputs]) the set is scored while it is uploaded (one pipelined call)."""
        self._lib = lib
        self.handle = C.c_void_p()
        # keep the converted arrays alive for the duration of the call only; the engine copies them
        X = _u32(graphs.X)
        arrays = [X, _u32(graphs.node_type), _u32(graphs.number_of_graph_node_edges), _u32(graphs.edge_index),
                  _u32(graphs.edge) if graphs.edge.size else None, _u32(graphs.node_index),
                  _u32(graphs.number_of_graph_nodes)]
        view = _lib.GraphsView()
        (view.X, view.node_type, view.number_of_graph_node_edges, view.edge_index, view.edge, view.node_index,
         view.number_of_graph_nodes) = [_ptr(a) for a in arrays]
        view.number_of_graphs = int(graphs.number_of_graphs)
        view.total_nodes = int(X.shape[0])
        view.total_edges = int(graphs.edge.shape[0]) if graphs.edge.size else 0
        view.max_number_of_graph_nodes = int(graphs.max_number_of_graph_nodes)
        if class_sums_out is None:
            _lib.check(lib.gtm_dataset_create(model, C.byref(view), C.byref(self.handle)))
        else:
            _lib.check(lib.gtm_dataset_create_scored(model, C.byref(view), int(graphs.number_of_node_types()),
                                                     _ptr(class_sums_out), C.byref(self.handle)))

    def close(self):
        if self.handle:
            self._lib.gtm_dataset_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CommonTsetlinMachine:
    def __init__(
        self,
        number_of_clauses,
        T,
        s,
        q=1.0,
        max_included_literals=None,
        boost_true_positive_feedback=1,
        number_of_state_bits=8,
        depth=1,
        message_size=256,
        message_bits=2,
        double_hashing=False,
        one_hot_encoding=False,
        grid=(16 * 13 * 4, 1, 1),
        block=(128, 1, 1),
        seed=None,
        device=None,
    ):
        self._lib = _lib.load()   # fails loudly when the CUDA library is not built
        if os.environ.get("GTM_B200_VERBOSE"):
            print("Initialization of sparse structure.")

        self.number_of_clauses = number_of_clauses
        self.number_of_clause_chunks = (number_of_clauses - 1) // 32 + 1
        self.T = int(T)
        self.depth = depth
        self.s = s if type(s) == tuple else (s,) * depth
        self.q = q
        self.max_included_literals = max_included_literals
        self.boost_true_positive_feedback = boost_true_positive_feedback
        self.number_of_state_bits = number_of_state_bits
        self.message_size = message_size
        self.message_bits = message_bits
        self.double_hashing = double_hashing
        self.one_hot_encoding = one_hot_encoding
        self.grid = grid
        self.block = block
        self.negative_clauses = 1
        if seed is None:
            seed = int(os.environ.get("GTM_B200_SEED", int.from_bytes(os.urandom(8), "little")))
        self.seed = int(seed) & 0xFFFFFFFFFFFFFFFF
        if device is None:
            device = int(os.environ.get("LOCAL_RANK", os.environ.get("GTM_B200_DEVICE", 0)))
        self.device = device

        self.graphs_signature_train = np.array([])
        self.graphs_signature_test = np.array([])
        self.encoded_Y = np.array([])
        self.ta_state = np.array([])
        self.message_ta_state = [np.array([])] * (self.depth - 1)
        self.clause_weights = np.array([])

        # message hypervectors: same draws from the global numpy stream as tm.py:90-106
        if self.one_hot_encoding:
            self.message_bits = 1
            self.hypervectors = np.zeros((number_of_clauses, 1), dtype=np.uint32)   # filled in _init
        elif self.double_hashing:
            from sympy import prevprime

            self.message_bits = 2
            prime = prevprime(self.message_size)
            ids = np.arange(number_of_clauses, dtype=np.int64)
            self.hypervectors = np.stack([ids % self.message_size, prime - (ids % prime)], axis=1).astype(np.uint32)
        else:
            indexes = np.arange(self.message_size, dtype=np.uint32)
            self.hypervectors = np.zeros((number_of_clauses, self.message_bits), dtype=np.uint32)
            for i in range(number_of_clauses):
                self.hypervectors[i, :] = np.random.choice(indexes, size=(self.message_bits), replace=False)

        self.initialized = False
        self._model = C.c_void_p()
        self._train_set = None
        self._test_set = None
        self._shard_group = None      # torch.distributed group over which clauses are sharded during fit
        self._sharded = False

    # ------------------------------------------------------------------------------------------ life cycle
    def __del__(self):
        try:
            self._release()
        except Exception:
            pass

    def _release(self):
        for ds in (self._train_set, self._test_set):
            if ds is not None:
                ds.close()
        self._train_set = self._test_set = None
        if self._model:
            self._lib.gtm_destroy(self._model)
            self._model = C.c_void_p()

    # ------------------------------------------------------------------------------ clause-sharded learning
    def shard_clauses(self, group=None):
        """Learn with the clauses sharded over the ranks of a ``torch.distributed`` process group, one process per
        GPU of one box (not in the reference, which is single-GPU).  Every rank must build the model with the same
        arguments, seed and ``numpy.random`` state, and call ``fit`` with the same graphs and labels; after every
        ``fit`` all ranks hold the same, complete model again, so ``predict`` needs no communication.  The result is
        bit-identical to single-GPU learning."""
        import torch.distributed as dist

        self._shard_group = group
        self._sharded = dist.get_world_size(group) > 1

    def _connect_shards(self):
        """Exchange the IPC handles of the ranks' exchange buffers for the current training set."""
        import torch
        import torch.distributed as dist

        world, rank = dist.get_world_size(self._shard_group), dist.get_rank(self._shard_group)
        handle = (C.c_ubyte * 64)()
        _lib.check(self._lib.gtm_shard_prepare(self._model, self._train_set.handle, world, rank, handle))
        dev = "cuda" if dist.get_backend(self._shard_group) == "nccl" else "cpu"
        mine = torch.tensor(list(handle), dtype=torch.uint8, device=dev)
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine, group=self._shard_group)
        handles = np.concatenate([p.cpu().numpy() for p in parts]).astype(np.uint8)
        _lib.check(self._lib.gtm_shard_connect(self._model, self._train_set.handle, _ptr(handles)))
        self._train_set.shards_connected = True

    def _sync_shards(self):
        """After a sharded fit every rank owns the updated state of its clauses: gather the shards so that all ranks
        hold the complete model (also the synchronisation point the engine requires between two sharded fits)."""
        import torch
        import torch.distributed as dist

        group = self._shard_group
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        first, count = C.c_int(), C.c_int()
        _lib.check(self._lib.gtm_shard_range(self._model, world, rank, C.byref(first), C.byref(count)))
        first, count = first.value, count.value
        clauses = self.number_of_clauses
        per = (clauses + world - 1) // world
        dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"

        def gather_rows(rows):           # rows: int32/int64 [clauses][cols]; returns the array with every rank's rows
            mine = torch.zeros((per, rows.shape[1]), dtype=torch.from_numpy(rows[:1]).dtype, device=dev)
            if count:
                mine[:count] = torch.from_numpy(np.ascontiguousarray(rows[first:first + count])).to(dev)
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine, group=group)
            return np.concatenate([p.cpu().numpy() for p in parts], axis=0)[:clauses]

        for layer in range(self.depth):
            planes = self._download_ta(layer).view(np.int32).reshape(clauses, -1)
            full = np.ascontiguousarray(gather_rows(planes)).view(np.uint32)
            _lib.check(self._lib.gtm_set_ta_state(self._model, layer, _ptr(full)))
        weights = self._download_weights().reshape(self.number_of_outputs, clauses).T
        full_w = np.ascontiguousarray(gather_rows(np.ascontiguousarray(weights)).T, dtype=np.int32)
        _lib.check(self._lib.gtm_set_weights(self._model, _ptr(full_w)))
        pos = np.zeros(clauses, dtype=np.uint64)
        _lib.check(self._lib.gtm_get_draw_positions(self._model, _ptr(pos)))
        full_p = np.ascontiguousarray(gather_rows(pos.view(np.int64).reshape(clauses, 1))).view(np.uint64).reshape(clauses)
        _lib.check(self._lib.gtm_set_draw_positions(self._model, _ptr(np.ascontiguousarray(full_p))))

    def _create_engine(self):
        """tm.py:437-513 + :110-124: the engine takes sizes at run time, so there is nothing to compile."""
        self._release()
        cfg = _lib.Config()
        cfg.number_of_clauses = int(self.number_of_clauses)
        cfg.number_of_outputs = int(self.number_of_outputs)
        cfg.number_of_literals = int(self.number_of_literals)
        cfg.number_of_state_bits = int(self.number_of_state_bits)
        cfg.boost_true_positive_feedback = int(self.boost_true_positive_feedback)
        cfg.T = int(self.T)
        cfg.max_included_literals = int(self.max_included_literals)
        cfg.message_size = int(self.message_size)
        cfg.message_bits = int(self.message_bits)
        cfg.depth = int(self.depth)
        cfg.device = int(self.device)
        cfg.q = float("%f" % self.q)   # the reference passes q through a "%f" format (tm.py:445,458)
        for d, v in enumerate(self.s):
            cfg.s[d] = float(v)
        cfg.seed = self.seed
        _lib.check(self._lib.gtm_create(C.byref(cfg), C.byref(self._model)))
        _lib.check(self._lib.gtm_set_hypervectors(self._model, _ptr(_u32(self.hypervectors))))

    def _init(self, graphs):
        """Sizes derived from the first fitted graph set (tm.py:414-435)."""
        if self.one_hot_encoding:
            self.message_size = self.number_of_clauses * max(1, len(graphs.edge_type_id))
            for i in range(self.number_of_clauses):
                self.hypervectors[i, 0] = i * len(graphs.edge_type_id)
        self.number_of_features = graphs.hypervector_size
        self.number_of_literals = self.number_of_features * 2
        self.number_of_ta_chunks = int((self.number_of_literals - 1) // 32 + 1)
        self.number_of_message_features = self.message_size
        self.number_of_message_literals = self.number_of_message_features * 2
        self.number_of_message_chunks = int((self.number_of_message_literals - 1) // 32 + 1)
        if self.max_included_literals is None:
            self.max_included_literals = self.number_of_literals
        self.max_number_of_graph_nodes = graphs.max_number_of_graph_nodes
        self._create_engine()
        self.initialized = True

    def _layer_chunks(self, layer):
        return self.number_of_ta_chunks if layer == 0 else self.number_of_message_chunks

    def _download_ta(self, layer):
        out = np.empty(self.number_of_clauses * self._layer_chunks(layer) * self.number_of_state_bits, dtype=np.uint32)
        _lib.check(self._lib.gtm_get_ta_state(self._model, layer, _ptr(out)))
        return out

    def _download_weights(self):
        out = np.empty(self.number_of_outputs * self.number_of_clauses, dtype=np.int32)
        _lib.check(self._lib.gtm_get_weights(self._model, _ptr(out)))
        return out

    # ------------------------------------------------------------------------------------------- learning
    def _init_fit(self, graphs, encoded_Y, incremental):
        """tm.py:515-561."""
        if not self.initialized:
            self._init(graphs)
            _lib.check(self._lib.gtm_init_state(self._model, 1))
        elif not incremental:
            _lib.check(self._lib.gtm_init_state(self._model, 0))   # message layers keep their state (tm.py:524-526)
        if not np.array_equal(self.graphs_signature_train, graphs.signature):
            self.graphs_signature_train = graphs.signature
            if self._train_set is not None:
                self._train_set.close()
            self._train_set = _Dataset(self._lib, self._model, graphs)
        if not np.array_equal(self.encoded_Y, encoded_Y):
            self.encoded_Y = encoded_Y

    def _fit(self, graphs, encoded_Y, epochs=100, incremental=False):
        """tm.py:664-752: `epochs` ordered passes; the whole loop runs inside one persistent kernel."""
        if self.initialized and encoded_Y.shape[1] != self.number_of_outputs_at_init:
            raise ValueError("number of outputs changed from %d to %d after the model was sized"
                             % (self.number_of_outputs_at_init, encoded_Y.shape[1]))
        self._init_fit(graphs, encoded_Y, incremental)
        self.number_of_outputs_at_init = self.number_of_outputs
        y = np.ascontiguousarray(encoded_Y, dtype=np.int32)
        if self._sharded and not getattr(self._train_set, "shards_connected", False):
            self._connect_shards()
        _lib.check(self._lib.gtm_fit(self._model, self._train_set.handle,
                                     int(graphs.number_of_node_types()), _ptr(y), 0, int(graphs.number_of_graphs),
                                     int(epochs)))
        if self._sharded:
            self._sync_shards()
        self.ta_state = np.array([])
        self.clause_weights = np.array([])
        return

    # -------------------------------------------------------------------------------------------- scoring
    def _score_init(self, graphs):
        """tm.py:754-784."""
        if not self.initialized:
            print("Error: Model not trained.")
            sys.exit(-1)
        if not np.array_equal(self.graphs_signature_test, graphs.signature):
            self.graphs_signature_test = graphs.signature
            if self._test_set is not None:
                self._test_set.close()
            self._test_set = _Dataset(self._lib, self._model, graphs)

    def _score(self, graphs, out=None):
        """tm.py:786-812: raw class sums int32[N][outputs]; one batched launch instead of a per-graph loop.
        `out` (optional, C-contiguous int32[N][outputs], e.g. page-locked) receives the result in place."""
        if not self.initialized:
            print("Error: Model not trained.")
            sys.exit(-1)
        class_sum = np.zeros((graphs.number_of_graphs, self.number_of_outputs), dtype=np.int32) if out is None else out
        assert class_sum.dtype == np.int32 and class_sum.flags.c_contiguous
        assert class_sum.shape == (graphs.number_of_graphs, self.number_of_outputs)
        if not np.array_equal(self.graphs_signature_test, graphs.signature):
            # a new graph set: upload and scoring in one pipelined call; the set stays resident for later calls
            if self._test_set is not None:
                self._test_set.close()
                self._test_set = None
            self.graphs_signature_test = np.array([])
            self._test_set = _Dataset(self._lib, self._model, graphs, class_sums_out=class_sum)
            self.graphs_signature_test = graphs.signature
            return class_sum
        _lib.check(self._lib.gtm_score(self._model, self._test_set.handle, int(graphs.number_of_node_types()), 0,
                                       int(graphs.number_of_graphs), _ptr(class_sum)))
        return class_sum

    def transform(self, graphs):
        """tm.py:814-851: (clause outputs int32[N][clauses], class sums)."""
        self._score_init(graphs)
        class_sum = np.zeros((graphs.number_of_graphs, self.number_of_outputs), dtype=np.int32)
        transformed_X = np.zeros((graphs.number_of_graphs, self.number_of_clauses), dtype=np.int32)
        _lib.check(self._lib.gtm_transform(self._model, self._test_set.handle, int(graphs.number_of_node_types()), 0,
                                           int(graphs.number_of_graphs), _ptr(transformed_X), _ptr(class_sum)))
        return transformed_X, class_sum

    def transform_nodewise(self, graphs):
        """tm.py:853-900: (per-node clause outputs int32[N][clauses][max nodes], class sums)."""
        self._score_init(graphs)
        n_max = int(np.max(graphs.number_of_graph_nodes))
        class_sum = np.zeros((graphs.number_of_graphs, self.number_of_outputs), dtype=np.int32)
        transformed_X = np.zeros((graphs.number_of_graphs, self.number_of_clauses, n_max), dtype=np.int32)
        _lib.check(self._lib.gtm_transform_nodewise(self._model, self._test_set.handle, int(graphs.number_of_node_types()),
                                                    0, int(graphs.number_of_graphs), n_max, _ptr(transformed_X), _ptr(class_sum)))
        return transformed_X, class_sum

    # ---------------------------------------------------------------------------------------- introspection
    def ta_action(self, depth, clause, ta):
        """tm.py:126-142: include bit of automaton `ta` of `clause` at layer `depth`."""
        state = self._download_ta(depth)
        if depth == 0:
            self.ta_state = state
        else:
            self.message_ta_state[depth - 1] = state
        planes = state.reshape((self.number_of_clauses, self._layer_chunks(depth), self.number_of_state_bits))
        return (planes[clause, ta // 32, self.number_of_state_bits - 1] & (1 << (ta % 32))) > 0

    def _layer_literals(self, depth):
        return self.number_of_literals if depth == 0 else self.number_of_message_literals

    def get_ta_states(self, depth):
        """tm.py:174-205 (kernels.py:718-758): automaton states uint32[clauses][literals] of one layer."""
        planes = self._download_ta(depth).reshape(
            (self.number_of_clauses, self._layer_chunks(depth), self.number_of_state_bits))
        lits = self._layer_literals(depth)
        bits = np.unpackbits(planes.transpose(0, 2, 1).copy().view(np.uint8), axis=2, bitorder="little")
        weights = (np.uint32(1) << np.arange(self.number_of_state_bits, dtype=np.uint32))[None, :, None]
        return (bits[:, :, :lits].astype(np.uint32) * weights).sum(axis=1, dtype=np.uint32)

    def get_hyperliterals(self, depth):
        """tm.py:144-172 (kernels.py:761-796): include actions uint32[clauses][literals] (0/1) of one layer."""
        planes = self._download_ta(depth).reshape(
            (self.number_of_clauses, self._layer_chunks(depth), self.number_of_state_bits))
        inc = np.ascontiguousarray(planes[:, :, self.number_of_state_bits - 1])
        bits = np.unpackbits(inc.view(np.uint8), axis=1, bitorder="little")
        return bits[:, : self._layer_literals(depth)].astype(np.uint32)

    def get_weights(self):
        """tm.py:207-211."""
        if np.array_equal(self.clause_weights, np.array([])):
            self.clause_weights = self._download_weights()
        return self.clause_weights.reshape((self.number_of_outputs, self.number_of_clauses))

    def get_clause_literals(self, symbol_hv):
        """tm.py:213-240: per clause, how many hypervector bits of each symbol (and negated symbol) it includes."""
        hv_clauses = self.get_hyperliterals(0)
        half = self.number_of_literals // 2
        n_sym = symbol_hv.shape[0]
        expanded = np.zeros((half, n_sym), dtype=np.uint8)
        for sym in range(n_sym):
            expanded[symbol_hv[sym].ravel(), sym] = 1
        out = np.zeros((self.number_of_clauses, 2 * n_sym))
        out[:, :n_sym] = hv_clauses[:, :half] @ expanded
        out[:, n_sym:] = hv_clauses[:, half:] @ expanded
        return out

    def get_messages(self, depth, edge_types):
        """tm.py:242-279: per edge type and clause, how many hypervector bits of each sender clause it includes."""
        assert depth > 0, f"Expected depth > 0, got {depth}. Depth <= 0 means surface, use get_clause_literals()"
        hv_messages = self.get_hyperliterals(depth).astype(np.float32)
        half = self.number_of_message_literals // 2
        out = np.zeros((edge_types, self.number_of_clauses, 2 * self.number_of_clauses))
        for edge_type in range(edge_types):
            expanded = np.zeros((half, self.number_of_clauses))
            for c in range(self.number_of_clauses):
                expanded[(self.hypervectors[c].ravel() + edge_type) % self.message_size, c] = 1
            out[edge_type, :, : self.number_of_clauses] = hv_messages[:, :half] @ expanded
            out[edge_type, :, self.number_of_clauses:] = hv_messages[:, half:] @ expanded
        return out

    # ------------------------------------------------------------------------------------------ checkpoints
    def get_state(self):
        """tm.py:281-287: the 10-tuple (layer-0 automata, weights, sizes...)."""
        if np.array_equal(self.clause_weights, np.array([])):
            self.ta_state = self._download_ta(0)
            self.clause_weights = self._download_weights()
        return (self.ta_state, self.clause_weights, self.number_of_outputs, self.number_of_clauses,
                self.number_of_literals, self.depth, self.number_of_state_bits, self.number_of_ta_chunks,
                self.min_y, self.max_y)

    def set_state(self, state):
        """tm.py:289-310: layer-0 automata and weights from a `get_state` tuple."""
        self.number_of_outputs = state[2]
        self.number_of_clauses = state[3]
        self.number_of_literals = state[4]
        self.depth = state[5]
        self.number_of_state_bits = state[6]
        self.number_of_ta_chunks = state[7]
        self.min_y = state[8]
        self.max_y = state[9]
        if not self._model:
            self.number_of_message_literals = self.message_size * 2
            self.number_of_message_chunks = int((self.number_of_message_literals - 1) // 32 + 1)
            if self.max_included_literals is None:
                self.max_included_literals = self.number_of_literals
            self._create_engine()
            _lib.check(self._lib.gtm_init_state(self._model, 1))
            self.number_of_outputs_at_init = self.number_of_outputs
            self.initialized = True
        _lib.check(self._lib.gtm_set_ta_state(self._model, 0, _ptr(_u32(state[0]))))
        _lib.check(self._lib.gtm_set_weights(self._model, _ptr(np.ascontiguousarray(state[1], dtype=np.int32))))
        self.graphs_signature_train = np.array([])
        self.graphs_signature_test = np.array([])
        self.encoded_Y = np.array([])
        self.ta_state = np.array([])
        self.clause_weights = np.array([])

    def save(self, fname=""):
        """tm.py:312-362: dict with the reference's keys and array layouts (optionally pickled to `fname`)."""
        self.ta_state = self._download_ta(0)
        for d in range(self.depth - 1):
            self.message_ta_state[d] = self._download_ta(d + 1)
        self.clause_weights = self._download_weights()
        state_dict = {
            "ta_state": self.ta_state,
            "message_ta_state": self.message_ta_state,
            "clause_weights": self.clause_weights,
            "hypervectors": self.hypervectors,
            "number_of_outputs": self.number_of_outputs,
            "number_of_literals": self.number_of_literals,
            "number_of_message_literals": self.number_of_message_literals,
            "min_y": self.min_y,
            "max_y": self.max_y,
            "negative_clauses": self.negative_clauses,
            "max_number_of_graph_nodes": self.max_number_of_graph_nodes,
            "number_of_clauses": self.number_of_clauses,
            "T": self.T,
            "s": self.s,
            "q": self.q,
            "max_included_literals": self.max_included_literals,
            "boost_true_positive_feedback": self.boost_true_positive_feedback,
            "number_of_state_bits": self.number_of_state_bits,
            "depth": self.depth,
            "message_size": self.message_size,
            "message_bits": self.message_bits,
            "double_hashing": self.double_hashing,
            "one_hot_encoding": self.one_hot_encoding,
        }
        if len(fname) > 0:
            print(f"Saving model to {fname}.")
            with open(fname, "wb") as f:
                pickle.dump(state_dict, f)
        return state_dict

    def load(self, state_dict={}, fname=""):
        """tm.py:364-412."""
        if len(fname) == 0 and len(state_dict) == 0:
            print("Error: No file or state_dict provided. Pass either a file name or a state_dict.")
            return
        if len(fname) > 0:
            print(f"Loading model from {fname}.")
            with open(fname, "rb") as f:
                state_dict = pickle.load(f)
        self.ta_state = state_dict["ta_state"]
        self.message_ta_state = state_dict["message_ta_state"]
        self.clause_weights = state_dict["clause_weights"]
        self.hypervectors = state_dict["hypervectors"]
        self.number_of_outputs = state_dict["number_of_outputs"]
        self.number_of_literals = state_dict["number_of_literals"]
        self.number_of_message_literals = state_dict["number_of_message_literals"]
        self.min_y = state_dict["min_y"]
        self.max_y = state_dict["max_y"]
        self.negative_clauses = state_dict["negative_clauses"]
        self.max_number_of_graph_nodes = state_dict["max_number_of_graph_nodes"]
        self.message_size = state_dict["message_size"]
        self.number_of_features = self.number_of_literals // 2
        self.number_of_ta_chunks = int((self.number_of_literals - 1) // 32 + 1)
        self.number_of_message_features = self.number_of_message_literals // 2
        self.number_of_message_chunks = int((self.number_of_message_literals - 1) // 32 + 1)
        if self.max_included_literals is None:
            self.max_included_literals = self.number_of_literals
        self._create_engine()
        _lib.check(self._lib.gtm_init_state(self._model, 1))
        _lib.check(self._lib.gtm_set_ta_state(self._model, 0, _ptr(_u32(self.ta_state))))
        for d in range(self.depth - 1):
            _lib.check(self._lib.gtm_set_ta_state(self._model, d + 1, _ptr(_u32(self.message_ta_state[d]))))
        _lib.check(self._lib.gtm_set_weights(self._model, _ptr(np.ascontiguousarray(self.clause_weights, dtype=np.int32))))
        self.number_of_outputs_at_init = self.number_of_outputs
        self.graphs_signature_train = np.array([])
        self.graphs_signature_test = np.array([])
        self.initialized = True


class MultiClassGraphTsetlinMachine(CommonTsetlinMachine):
    """One-vs-all classifier (tm.py:903-959)."""

    def fit(self, graphs, Y, epochs=100, incremental=False):
        self.number_of_outputs = int(np.max(Y) + 1)
        self.max_y = None
        self.min_y = None
        encoded_Y = np.empty((Y.shape[0], self.number_of_outputs), dtype=np.int32)
        for i in range(self.number_of_outputs):
            encoded_Y[:, i] = np.where(Y == i, self.T, -self.T)
        self._fit(graphs, encoded_Y, epochs=epochs, incremental=incremental)

    def score(self, graphs, out=None):
        return self._score(graphs, out)

    def predict(self, graphs):
        return np.argmax(self.score(graphs), axis=1)


class MultiOutputGraphTsetlinMachine(CommonTsetlinMachine):
    """Independent binary outputs (tm.py:961-1017)."""

    def fit(self, graphs, Y, epochs=100, incremental=False):
        self.number_of_outputs = Y.shape[1]
        self.max_y = None
        self.min_y = None
        encoded_Y = np.where(Y == 1, self.T, -self.T).astype(np.int32)
        self._fit(graphs, encoded_Y, epochs=epochs, incremental=incremental)

    def score(self, graphs):
        return self._score(graphs)

    def predict(self, graphs):
        return (self.score(graphs) >= 0).astype(np.uint32)


class GraphTsetlinMachine(CommonTsetlinMachine):
    """Single binary output (tm.py:1019-1072)."""

    def fit(self, graphs, Y):
        self.number_of_outputs = 1
        self.max_y = None
        self.min_y = None
        encoded_Y = np.where(Y == 1, self.T, -self.T).astype(np.int32).reshape(-1, 1)
        self._fit(graphs, encoded_Y)
        return

    def score(self, graphs):
        return self._score(graphs)[:, 0]

    def predict(self, X):
        return self.score(X) >= 0
