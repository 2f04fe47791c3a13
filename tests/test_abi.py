"""CPU suite, part 3: the C-ABI library loads without a GPU and exports every symbol include/gtm_b200.h declares;
argument checks that need no device; the Python binding covers every declaration."""

import ctypes as C
import os
import re

import numpy as np

from graphtsetlinmachine_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "gtm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gtm_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    build.build()
    lib = C.CDLL(build.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), name


def test_binding_covers_header():
    bound = set(_lib.PROTOTYPES) | {"gtm_last_error", "gtm_version"}
    assert set(declared_functions()) == bound


def test_struct_layouts():
    assert C.sizeof(_lib.Config) == 12 * 4 + 8 + 16 * 4 + 8
    assert C.sizeof(_lib.GraphsView) == 7 * 8 + 3 * 8 + 2 * 4


def test_argument_errors_without_device():
    lib = _lib.load()
    assert lib.gtm_version().startswith(b"gtm_b200")
    assert lib.gtm_create(None, None) == 1
    assert b"null" in lib.gtm_last_error()
    out = C.c_void_p()
    cfg = _lib.Config()
    assert lib.gtm_create(C.byref(cfg), C.byref(out)) == 1      # zero clauses
    assert lib.gtm_init_state(None, 1) == 1
    assert lib.gtm_score(None, None, 1, 0, 0, None) == 1
    assert lib.gtm_destroy(None) == 0 and lib.gtm_dataset_destroy(None) == 0


def _view(arrays, n_graphs, max_nodes):
    X, node_type, degree, edge_index, edge, node_index, n_nodes = arrays
    v = _lib.GraphsView()
    ptr = lambda a: None if a is None else a.ctypes.data_as(C.c_void_p)
    (v.X, v.node_type, v.number_of_graph_node_edges, v.edge_index, v.edge, v.node_index,
     v.number_of_graph_nodes) = [ptr(a) for a in arrays]
    v.number_of_graphs, v.total_nodes = n_graphs, X.shape[0]
    v.total_edges = 0 if edge is None else edge.shape[0]
    v.max_number_of_graph_nodes = max_nodes
    return v


def test_graph_arrays_are_validated_on_the_host():
    """Inconsistent graph arrays are refused before anything reaches a kernel: a graph with more nodes than
    max_number_of_graph_nodes, an empty graph, node or edge ranges that leave the arrays."""
    lib = _lib.load()
    u32 = lambda *a: np.array(a, dtype=np.uint32)

    def arrays():
        # three graphs of 2, 1 and 3 nodes; out-degrees 1,0,2,0,1,1 -> five edge rows
        return [np.zeros((6, 2), dtype=np.uint32), u32(0, 0, 0, 0, 0, 0), u32(1, 0, 2, 0, 1, 1), u32(0, 1, 1, 3, 3, 4),
                np.zeros((5, 2), dtype=np.uint32), u32(0, 2, 3), u32(2, 1, 3)]

    good = arrays()
    assert lib.gtm_validate_graphs(C.byref(_view(good, 3, 3))) == 0
    assert lib.gtm_validate_graphs(C.byref(_view(good, 3, 2))) == 1                # a graph has 3 nodes, the set says at most 2
    assert b"max_number_of_graph_nodes" in lib.gtm_last_error()
    bad = arrays(); bad[6][1] = 0                                                  # a graph without nodes
    assert lib.gtm_validate_graphs(C.byref(_view(bad, 3, 3))) == 1
    bad = arrays(); bad[6][2] = 4                                                  # last graph runs past total_nodes
    assert lib.gtm_validate_graphs(C.byref(_view(bad, 3, 4))) == 1
    assert b"node_index" in lib.gtm_last_error()
    bad = arrays(); bad[5][1] = 1                                                  # node ranges overlap
    assert lib.gtm_validate_graphs(C.byref(_view(bad, 3, 3))) == 1
    bad = arrays(); bad[2][5] = 7                                                  # last CSR row runs past total_edges
    assert lib.gtm_validate_graphs(C.byref(_view(bad, 3, 3))) == 1
    assert b"edge_index" in lib.gtm_last_error()
    bad = arrays(); bad[3][3] = 2                                                  # CSR row starts are not the running sum
    assert lib.gtm_validate_graphs(C.byref(_view(bad, 3, 3))) == 1
    bad = arrays(); bad[4] = None                                                  # edges declared by the degrees but no edge array
    assert lib.gtm_validate_graphs(C.byref(_view(bad, 3, 3))) == 1
    assert lib.gtm_validate_graphs(None) == 1


def test_reference_graphs_pass_validation():
    import sys
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from util import random_graphs

    lib = _lib.load()
    rng = np.random.default_rng(2)
    np.random.seed(2)
    g = random_graphs(50, rng, max_nodes=9, node_types=2, edge_types=3)
    u32 = lambda a: np.ascontiguousarray(a, dtype=np.uint32)
    arrays = [u32(g.X), u32(g.node_type), u32(g.number_of_graph_node_edges), u32(g.edge_index), u32(g.edge),
              u32(g.node_index), u32(g.number_of_graph_nodes)]
    assert lib.gtm_validate_graphs(C.byref(_view(arrays, 50, int(g.max_number_of_graph_nodes)))) == 0
    sub = g[10:20]
    arrays = [u32(sub.X), u32(sub.node_type), u32(sub.number_of_graph_node_edges), u32(sub.edge_index), u32(sub.edge),
              u32(sub.node_index), u32(sub.number_of_graph_nodes)]
    assert lib.gtm_validate_graphs(C.byref(_view(arrays, 10, int(sub.max_number_of_graph_nodes)))) == 0
