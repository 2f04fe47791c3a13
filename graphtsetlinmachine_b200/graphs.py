"""Host-side graph encoder: symbols -> sparse hypervectors -> bit-packed node literals + CSR edges.

Drop-in for the reference ``GraphTsetlinMachine/graphs.py:26-305`` (class ``Graphs``): same constructor,
same builder call order (``set_number_of_graph_nodes`` -> ``prepare_node_configuration`` ->
``add_graph_node`` -> ``prepare_edge_configuration`` -> ``add_graph_node_edge`` ->
``add_graph_node_property`` -> ``encode``), same attribute names and array layouts, and the same sequence of
calls into the global ``numpy.random`` stream, so that equal seeds give equal symbol hypervectors
(``graphs.py:73-76``).

Array layouts produced (all little-endian, row-major):

* ``X``  ``uint32[total_nodes][chunks]`` with ``chunks = ceil(2*hypervector_size/32)``; literal ``k`` lives in
  bit ``k % 32`` of word ``k // 32``; literal ``k < hv`` is feature bit ``k``, literal ``hv + k`` its negation.
* ``node_index`` / ``number_of_graph_nodes``  ``uint32[N]``  first node / node count of every graph.
* ``node_type`` / ``number_of_graph_node_edges`` / ``edge_index``  ``uint32[total_nodes]``.
* ``edge``  ``uint32[total_edges][2]`` = (destination node id local to the graph, edge type id).

Besides the per-item builder calls of the reference, this class offers bulk (vectorised) variants
(``add_graph_node_properties_bulk``, ``set_edges_bulk`` ...) that write the very same arrays; the per-item
methods are thin wrappers over the same bit arithmetic.
"""

import hashlib
import sys

import numpy as np

__all__ = ["Graphs"]

_WORD = 32


def _ceil_words(bits):
    return (int(bits) - 1) // _WORD + 1


class Graphs:
    def __init__(
        self,
        number_of_graphs,
        hypervector_size=128,
        hypervector_bits=2,
        double_hashing=False,
        one_hot_encoding=False,
        symbols=None,
        init_with=None,
    ):
        self.number_of_graphs = number_of_graphs
        self.number_of_graph_nodes = np.zeros(number_of_graphs, dtype=np.uint32)
        self.double_hashing = double_hashing
        self.one_hot_encoding = one_hot_encoding
        # per graph: node name -> node id local to the graph (insertion order)
        self.graph_node_id = [dict() for _ in range(number_of_graphs)]
        self.init_with = init_with
        self.encoded = False

        if init_with is not None:
            # Share (by reference, like graphs.py:80-86) every table of the graph set we were initialised from.
            for attr in (
                "edge_type_id",
                "node_type_id",
                "symbol_id",
                "hypervector_size",
                "hypervector_bits",
                "hypervectors",
                "number_of_hypervector_chunks",
            ):
                setattr(self, attr, getattr(init_with, attr))
            return

        self.edge_type_id = {}
        self.node_type_id = {}
        self.symbol_id = {}
        for name in symbols:
            self.symbol_id[name] = len(self.symbol_id)
        n_symbols = len(self.symbol_id)
        self.hypervector_size = hypervector_size
        self.hypervector_bits = hypervector_bits

        if one_hot_encoding:
            # graphs.py:58-63: one private bit per symbol
            self.hypervector_size = n_symbols
            self.hypervector_bits = 1
            self.hypervectors = np.arange(n_symbols, dtype=np.uint32).reshape(n_symbols, 1)
        elif double_hashing:
            # graphs.py:64-71: two hash positions derived from the largest prime below the vector size
            from sympy import prevprime

            self.hypervector_bits = 2
            prime = prevprime(self.hypervector_size)
            ids = np.arange(n_symbols, dtype=np.int64)
            self.hypervectors = np.stack(
                [ids % self.hypervector_size, prime - (ids % prime)], axis=1
            ).astype(np.uint32)
        else:
            # graphs.py:73-76: one np.random.choice call per symbol, in symbol order (keeps seeds compatible)
            self.hypervectors = np.zeros((n_symbols, self.hypervector_bits), dtype=np.uint32)
            positions = np.arange(self.hypervector_size)
            for sym in range(n_symbols):
                self.hypervectors[sym, :] = np.random.choice(
                    positions, size=(self.hypervector_bits), replace=False
                )

        self.number_of_hypervector_chunks = _ceil_words(self.hypervector_size * 2)

    # ------------------------------------------------------------------ nodes
    def set_number_of_graph_nodes(self, graph_id, number_of_graph_nodes):
        self.number_of_graph_nodes[graph_id] = number_of_graph_nodes

    def set_number_of_graph_nodes_bulk(self, counts):
        """Vectorised ``set_number_of_graph_nodes`` for all graphs at once."""
        self.number_of_graph_nodes[:] = np.asarray(counts, dtype=np.uint32)

    def prepare_node_configuration(self):
        """Prefix sums over node counts and allocation of the node arrays (graphs.py:100-113)."""
        counts = self.number_of_graph_nodes
        self.node_index = np.zeros(counts.shape[0], dtype=np.uint32)
        self.node_index[1:] = np.add.accumulate(counts[:-1])
        self.max_number_of_graph_nodes = counts.max()
        self.max_number_of_graph_node_chunks = (self.max_number_of_graph_nodes - 1) // _WORD + 1
        self.number_of_nodes = counts.sum()
        total = int(self.number_of_nodes)
        self.node_type = np.empty(total, dtype=np.uint32)
        self.number_of_graph_node_edges = np.empty(total, dtype=np.uint32)
        self.graph_node_edge_counter = np.zeros(total, dtype=np.uint32)
        self.edge_index = np.zeros(total, dtype=np.uint32)
        # every negated literal starts at 1, every positive literal at 0; padding bits stay 0
        row = np.zeros(self.number_of_hypervector_chunks, dtype=np.uint32)
        lits = np.arange(self.hypervector_size, 2 * self.hypervector_size)
        np.bitwise_or.at(row, lits // _WORD, (np.uint32(1) << (lits % _WORD).astype(np.uint32)))
        self.X = np.tile(row, (total, 1))

    def add_graph_node(self, graph_id, node_name, number_of_graph_node_edges, node_type_name="Plain"):
        if node_type_name not in self.node_type_id:
            self.node_type_id[node_type_name] = len(self.node_type_id)
        ids = self.graph_node_id[graph_id]
        if node_name not in ids:
            ids[node_name] = len(ids)
        slot = int(self.node_index[graph_id]) + ids[node_name]
        self.node_type[slot] = self.node_type_id[node_type_name]
        self.number_of_graph_node_edges[slot] = number_of_graph_node_edges

    def set_nodes_bulk(self, out_degrees, node_types=None, node_type_names=("Plain",)):
        """Vectorised ``add_graph_node`` for every node of every graph.

        Nodes of a graph are named ``0 .. n-1`` (ints) and get local ids in that order.
        ``out_degrees``/``node_types`` are flat arrays over all nodes in graph order.
        """
        for name in node_type_names:
            if name not in self.node_type_id:
                self.node_type_id[name] = len(self.node_type_id)
        total = int(self.number_of_nodes)
        self.number_of_graph_node_edges[:] = np.asarray(out_degrees, dtype=np.uint32).reshape(total)
        if node_types is None:
            self.node_type[:] = self.node_type_id[node_type_names[0]]
        else:
            self.node_type[:] = np.asarray(node_types, dtype=np.uint32).reshape(total)
        self.graph_node_id = _LazyNodeIds(self.number_of_graph_nodes)

    def number_of_node_types(self):
        return len(self.node_type_id)

    # ------------------------------------------------------------------ edges
    def prepare_edge_configuration(self):
        """CSR row starts over the declared out-degrees (graphs.py:127-129)."""
        self.edge_index[1:] = np.add.accumulate(self.number_of_graph_node_edges[:-1])
        self.edge = np.empty((int(self.number_of_graph_node_edges.sum()), 2), dtype=np.uint32)

    def add_graph_node_edge(self, graph_id, source_node_name, destination_node_name, edge_type_name):
        ids = self.graph_node_id[graph_id]
        src_slot = int(self.node_index[graph_id]) + ids[source_node_name]
        used = int(self.graph_node_edge_counter[src_slot])
        if used >= int(self.number_of_graph_node_edges[src_slot]):
            print("Too many edges added to node '%s' of graph %d." % (source_node_name, graph_id))
            sys.exit(-1)
        if edge_type_name not in self.edge_type_id:
            self.edge_type_id[edge_type_name] = len(self.edge_type_id)
        row = int(self.edge_index[src_slot]) + used
        self.edge[row, 0] = ids[destination_node_name]
        self.edge[row, 1] = self.edge_type_id[edge_type_name]
        self.graph_node_edge_counter[src_slot] = used + 1

    def set_edges_bulk(self, destinations, edge_types, edge_type_names):
        """Vectorised ``add_graph_node_edge``: rows are given in CSR order (grouped by source node, in the
        order declared by the out-degrees); ``destinations`` are node ids local to the graph."""
        for name in edge_type_names:
            if name not in self.edge_type_id:
                self.edge_type_id[name] = len(self.edge_type_id)
        self.edge[:, 0] = np.asarray(destinations, dtype=np.uint32)
        self.edge[:, 1] = np.asarray(edge_types, dtype=np.uint32)
        self.graph_node_edge_counter[:] = self.number_of_graph_node_edges

    # ------------------------------------------------------------- properties
    def _set_symbol_bits(self, rows, symbols):
        """Set the positive literals and clear the negated literals of ``symbols`` on node rows ``rows``
        (the bit arithmetic of graphs.py:148-159, for many (node, symbol) pairs at once)."""
        hv = self.hypervectors[symbols].astype(np.int64)  # [pairs][bits]
        rows = np.broadcast_to(np.asarray(rows, dtype=np.int64)[:, None], hv.shape)
        pos = hv
        neg = hv + self.hypervector_size
        flat = self.X.reshape(-1)
        chunks = self.number_of_hypervector_chunks
        np.bitwise_or.at(flat, (rows * chunks + pos // _WORD).ravel(),
                         (np.uint32(1) << (pos % _WORD).astype(np.uint32)).ravel())
        np.bitwise_and.at(flat, (rows * chunks + neg // _WORD).ravel(),
                          (~(np.uint32(1) << (neg % _WORD).astype(np.uint32))).ravel())

    def add_graph_node_property(self, graph_id, node_name, symbol):
        row = int(self.node_index[graph_id]) + self.graph_node_id[graph_id][node_name]
        sym = self.symbol_id[symbol]
        size = self.hypervector_size
        X = self.X
        for k in self.hypervectors[sym, :]:
            k = int(k)
            X[row, k // _WORD] |= np.uint32(1 << (k % _WORD))
            kn = k + size
            X[row, kn // _WORD] &= np.uint32(~(1 << (kn % _WORD)) & 0xFFFFFFFF)

    def add_graph_node_properties_bulk(self, global_node_rows, symbol_ids):
        """Vectorised ``add_graph_node_property``: pair ``i`` adds symbol id ``symbol_ids[i]`` to the node
        whose row in ``X`` is ``global_node_rows[i]`` (= ``node_index[graph] + local node id``)."""
        self._set_symbol_bits(np.asarray(global_node_rows), np.asarray(symbol_ids, dtype=np.int64))

    # ---------------------------------------------------------------- printing
    def _node_symbols(self, graph_id, node_id):
        row = self.X[int(self.node_index[graph_id]) + node_id]
        present = []
        for name, sym in self.symbol_id.items():
            bits = self.hypervectors[sym, :].astype(np.int64)
            present.append(name if np.all((row[bits // _WORD] >> (bits % _WORD).astype(np.uint32)) & 1) else "*")
        return present

    def print_graph_nodes(self, graph_id):
        text = "Printing nodes of Graph#" + str(graph_id) + ":\n"
        for node_id in range(int(self.number_of_graph_nodes[graph_id])):
            text += "Node#" + str(node_id) + "( " + "".join(s + " " for s in self._node_symbols(graph_id, node_id)) + ") "
        print(text)
        print()

    def print_graph_edges(self, graph_id):
        text = "Printing edges of Graph#" + str(graph_id) + ":\n"
        base = int(self.node_index[graph_id])
        for node_id in range(int(self.number_of_graph_nodes[graph_id])):
            for k in range(int(self.graph_node_edge_counter[base + node_id])):
                row = int(self.edge_index[base + node_id]) + k
                text += "Edge#%d SrcNode#%d DestNode#%d EdgeType#%d\n" % (
                    row, node_id, self.edge[row][0], self.edge[row][1])
            text += "\n"
        print(text)
        print()

    def print_graph(self, graph_id):
        self.print_graph_nodes(graph_id)
        self.print_graph_edges(graph_id)

    # ------------------------------------------------------------------ encode
    def encode(self):
        """Check that every declared edge was added, then fingerprint the set (graphs.py:209-225)."""
        short = self.graph_node_edge_counter < self.number_of_graph_node_edges
        if np.any(short):
            for slot in np.nonzero(short)[0]:
                graph_id = int(np.searchsorted(self.node_index, slot, side="right") - 1)
                local = int(slot) - int(self.node_index[graph_id])
                name = next((k for k, v in self.graph_node_id[graph_id].items() if v == local), local)
                print("Node '%s' of graph %d misses edges." % (name, graph_id))
            sys.exit(-1)
        digest = hashlib.sha256()
        digest.update(np.ascontiguousarray(self.X).data)
        digest.update(np.ascontiguousarray(self.edge).data)
        self.signature = digest.digest()
        self.encoded = True

    # --------------------------------------------------------------- subsetting
    def __len__(self):
        return self.number_of_graphs

    def _get_indices(self, key):
        n = self.number_of_graphs
        if isinstance(key, (int, np.integer)):
            key = int(key)
            if key < 0:
                key += n
            if not 0 <= key < n:
                raise IndexError("Graph index out of range")
            return [key]
        if isinstance(key, slice):
            return list(range(*key.indices(n)))
        if isinstance(key, (list, np.ndarray)):
            out = []
            for k in key:
                k = int(k)
                if k < 0:
                    k += n
                if not 0 <= k < n:
                    raise IndexError("Graph index out of range")
                out.append(k)
            return out
        raise TypeError("Invalid graph index type")

    def _create_subset(self, indices):
        """New ``Graphs`` holding copies of the selected graphs (graphs.py:253-299), gathered with array ops."""
        sub = Graphs(len(indices), double_hashing=self.double_hashing,
                     one_hot_encoding=self.one_hot_encoding, init_with=self)
        idx = np.asarray(indices, dtype=np.int64)
        sub.number_of_graph_nodes[:] = self.number_of_graph_nodes[idx]
        lazy_ids = isinstance(self.graph_node_id, _LazyNodeIds)     # bulk-built sets: node i of a graph is named i
        if not lazy_ids:
            sub.graph_node_id = [self.graph_node_id[i] for i in indices]
        sub.prepare_node_configuration()
        if lazy_ids:
            sub.graph_node_id = _LazyNodeIds(sub.number_of_graph_nodes)
        counts = self.number_of_graph_nodes[idx].astype(np.int64)
        # source row of every node of the subset, in subset order
        starts = self.node_index[idx].astype(np.int64)
        offs = np.arange(int(counts.sum())) - np.repeat(np.cumsum(counts) - counts, counts)
        src_rows = np.repeat(starts, counts) + offs
        sub.node_type[:] = self.node_type[src_rows]
        sub.number_of_graph_node_edges[:] = self.number_of_graph_node_edges[src_rows]
        sub.graph_node_edge_counter[:] = self.graph_node_edge_counter[src_rows]
        sub.X[:] = self.X[src_rows]
        sub.prepare_edge_configuration()
        deg = self.graph_node_edge_counter[src_rows].astype(np.int64)
        if deg.sum() > 0:
            e_offs = np.arange(int(deg.sum())) - np.repeat(np.cumsum(deg) - deg, deg)
            src_e = np.repeat(self.edge_index[src_rows].astype(np.int64), deg) + e_offs
            dst_e = np.repeat(sub.edge_index.astype(np.int64), deg) + e_offs
            sub.edge[dst_e] = self.edge[src_e]
        sub.encode()
        return sub

    def __getitem__(self, index):
        indices = self._get_indices(index)
        if len(indices) == 0:
            raise ValueError("No graphs selected")
        return self._create_subset(indices)


class _LazyNodeIds:
    """Stand-in for the per-graph name->id dicts after a bulk build: node ``i`` of a graph is named ``i``."""

    def __init__(self, counts):
        self._counts = counts

    def __getitem__(self, graph_id):
        if isinstance(graph_id, (int, np.integer)):
            return {i: i for i in range(int(self._counts[graph_id]))}
        raise TypeError("graph id must be an integer")

    def __len__(self):
        return len(self._counts)
