"""Scoring through ``gtm_score_static_scratch``: the entry point for host programs that own all device memory
themselves (a pre-reserved pool, or a serving loop that cannot afford cudaMalloc / cudaFree) and so pass device
buffers in and get results in a device buffer, while the kernel's scratch comes from an array built into the
library.  The class sums must equal those of the allocating entry point (``gtm_score``), call after call: the
built-in scratch is shared and still holds the previous call's contents when the next one starts.

Collected last on purpose (file name), so a run that stops at the first failure has already run everything else.
"""

import ctypes as C

import numpy as np
import pytest

from cases import make_case
from graphtsetlinmachine_b200 import _lib
from oracle.oracle import OracleTM
from util import EngineTM, encode_labels, random_graphs

pytestmark = pytest.mark.gpu


def device_view(graphs, torch):
    """Caller-owned device copies of the graph arrays + the view that points at them."""
    u32 = lambda a: np.ascontiguousarray(a, dtype=np.uint32)
    host = [u32(graphs.X), u32(graphs.node_type), u32(graphs.number_of_graph_node_edges), u32(graphs.edge_index),
            u32(graphs.edge) if graphs.edge.size else np.zeros((1, 2), dtype=np.uint32), u32(graphs.node_index),
            u32(graphs.number_of_graph_nodes)]
    dev = [torch.from_numpy(a.view(np.int32)).cuda() for a in host]
    view = _lib.GraphsView()
    (view.X, view.node_type, view.number_of_graph_node_edges, view.edge_index, view.edge, view.node_index,
     view.number_of_graph_nodes) = [t.data_ptr() for t in dev]
    view.number_of_graphs = int(graphs.number_of_graphs)
    view.total_nodes = int(host[0].shape[0])
    view.total_edges = int(graphs.edge.shape[0]) if graphs.edge.size else 0
    view.max_number_of_graph_nodes = int(graphs.max_number_of_graph_nodes)
    return view, dev


@pytest.mark.parametrize("name", ["case_b", "case_d"])
def test_static_scratch_scoring_matches_allocating_entry_point(engine_lib, name):
    import torch

    kw, graphs, encY, _ = make_case(name)
    tm = EngineTM(**kw)
    tm.set_graphs(graphs)
    tm.prepare()
    tm.fit(encY)
    want = tm.score()                                   # existing entry point (allocates scratch and result)
    cpu = OracleTM(**kw)                                # and the CPU checker, from the same state
    cpu.set_graphs(graphs)
    cpu.ta_state[...] = tm.ta_state
    for mine, theirs in zip(cpu.message_ta_state, tm.message_ta_state):
        mine[...] = theirs
    cpu.clause_weights[...] = tm.clause_weights
    assert np.array_equal(cpu.score(), want)
    view, keep = device_view(graphs, torch)
    n, K = graphs.number_of_graphs, kw["classes"]
    out = torch.full((n, K), -12345, dtype=torch.int32, device="cuda")
    for call in range(2):                               # two calls in a row on the shared scratch
        out.fill_(-12345)
        _lib.check(engine_lib.gtm_score_static_scratch(tm.model, C.byref(view), tm.n_types, 0, n, C.c_void_p(out.data_ptr())))
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), want), "call %d" % call
    # another model and graph set in between, then the first one again: stale scratch contents must not matter
    kw2, graphs2, encY2, _ = make_case("case_c")
    tm2 = EngineTM(**kw2)
    tm2.set_graphs(graphs2)
    tm2.prepare()
    tm2.fit(encY2)
    view2, keep2 = device_view(graphs2, torch)
    out2 = torch.zeros((graphs2.number_of_graphs, kw2["classes"]), dtype=torch.int32, device="cuda")
    _lib.check(engine_lib.gtm_score_static_scratch(tm2.model, C.byref(view2), tm2.n_types, 0, graphs2.number_of_graphs,
                                                   C.c_void_p(out2.data_ptr())))
    torch.cuda.synchronize()
    assert np.array_equal(out2.cpu().numpy(), tm2.score())
    part = torch.zeros((7, K), dtype=torch.int32, device="cuda")
    _lib.check(engine_lib.gtm_score_static_scratch(tm.model, C.byref(view), tm.n_types, 5, 7, C.c_void_p(part.data_ptr())))
    torch.cuda.synchronize()
    assert np.array_equal(part.cpu().numpy(), want[5:12])
    tm.close()
    tm2.close()


def test_static_scratch_rejects_sizes_beyond_its_capacity(engine_lib):
    """A model / graph size whose per-block scratch exceeds the built-in array is refused before any launch."""
    import torch

    rng = np.random.default_rng(3)
    np.random.seed(3)
    graphs = random_graphs(2, rng, hv_size=16, fixed_nodes=2100, max_nodes=2100, max_degree=0, max_props=1)
    tm = EngineTM(clauses=20000, classes=2, literals=32, threshold=10, s=2.0, depth=1, max_nodes=2100)
    tm.prepare()
    view, keep = device_view(graphs, torch)
    out = torch.zeros((2, 2), dtype=torch.int32, device="cuda")
    status = engine_lib.gtm_score_static_scratch(tm.model, C.byref(view), 1, 0, 2, C.c_void_p(out.data_ptr()))
    assert status == 1 and b"built-in scratch" in engine_lib.gtm_last_error()
    tm.close()


def test_static_scratch_refuses_misaligned_literal_rows(engine_lib):
    """Literal rows that are a multiple of 16 bytes are read with 128-bit loads, so a caller that carves X out of its
    own pool at a 4-byte offset is told so (status 1, nothing launched) instead of faulting on the device."""
    import torch

    kw, graphs, encY, _ = make_case("case_d")           # 128 literals: 4 words = 16 bytes per row
    tm = EngineTM(**kw)
    tm.set_graphs(graphs)
    tm.prepare()
    view, keep = device_view(graphs, torch)
    n, K = graphs.number_of_graphs, kw["classes"]
    x_host = np.ascontiguousarray(graphs.X, dtype=np.uint32)
    shifted = torch.zeros(x_host.size + 8, dtype=torch.int32, device="cuda")
    shifted[1:1 + x_host.size] = torch.from_numpy(x_host.view(np.int32).ravel()).cuda()
    view.X = shifted.data_ptr() + 4
    out = torch.zeros((n, K), dtype=torch.int32, device="cuda")
    status = engine_lib.gtm_score_static_scratch(tm.model, C.byref(view), tm.n_types, 0, n, C.c_void_p(out.data_ptr()))
    assert status == 1 and b"16-byte aligned" in engine_lib.gtm_last_error()
    view.X = shifted.data_ptr() + 16                     # the same rows at an aligned address are fine
    shifted[4:4 + x_host.size] = torch.from_numpy(x_host.view(np.int32).ravel()).cuda()
    _lib.check(engine_lib.gtm_score_static_scratch(tm.model, C.byref(view), tm.n_types, 0, n, C.c_void_p(out.data_ptr())))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), tm.score())
    tm.close()


def test_static_scratch_skips_graphs_that_do_not_fit(engine_lib):
    """Graph arrays in device memory cannot be checked by the host.  A graph that claims more nodes than
    max_number_of_graph_nodes (its rows would leave the block's scratch slice) or a node range past total_nodes is
    skipped by the kernel - class sums zero, every other graph unaffected - and gtm_check_skipped_graphs reports it."""
    import torch

    kw, graphs, encY, _ = make_case("case_a")
    tm = EngineTM(**kw)
    tm.set_graphs(graphs)
    tm.prepare()
    tm.fit(encY)
    want = tm.score()
    view, dev = device_view(graphs, torch)
    n, K = graphs.number_of_graphs, kw["classes"]
    out = torch.zeros((n, K), dtype=torch.int32, device="cuda")
    flag = C.c_int(-1)
    _lib.check(engine_lib.gtm_score_static_scratch(tm.model, C.byref(view), tm.n_types, 0, n, C.c_void_p(out.data_ptr())))
    _lib.check(engine_lib.gtm_check_skipped_graphs(tm.model, C.byref(flag)))
    assert flag.value == 0 and np.array_equal(out.cpu().numpy(), want)
    n_nodes = dev[6]
    n_nodes[3] = 1000                                    # far more than max_number_of_graph_nodes
    n_nodes[n - 1] = int(graphs.max_number_of_graph_nodes)
    dev[5][n - 1] = view.total_nodes - 1                 # node range runs past total_nodes
    out.fill_(-7)
    _lib.check(engine_lib.gtm_score_static_scratch(tm.model, C.byref(view), tm.n_types, 0, n, C.c_void_p(out.data_ptr())))
    _lib.check(engine_lib.gtm_check_skipped_graphs(tm.model, C.byref(flag)))
    got = out.cpu().numpy()
    assert flag.value == 1
    keepers = np.ones(n, dtype=bool)
    keepers[[3, n - 1]] = False
    assert np.array_equal(got[keepers], want[keepers])
    assert not got[3].any()
    if int(graphs.max_number_of_graph_nodes) > 1:
        assert not got[n - 1].any()
    _lib.check(engine_lib.gtm_check_skipped_graphs(tm.model, C.byref(flag)))
    assert flag.value == 0                               # cleared by the call that reported it
    tm.close()
