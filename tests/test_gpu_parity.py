"""GPU suite: the CUDA engine, called through the C ABI, against the CPU checker, the golden vectors of the
reference's kernels and (when its prebuilt host version travelled along) the reference kernels themselves.
Everything is integer / bit work: the bar is equality."""

import ctypes
import os

import numpy as np
import pytest

from cases import CASES, make_case, state_of
from graphtsetlinmachine_b200 import _lib
from oracle import build_ref
from oracle.oracle import OracleTM
from test_oracle import check_against_golden
from util import EngineTM, encode_labels, random_graphs

pytestmark = pytest.mark.gpu


def assert_same_state(a, b, depth, what=""):
    sa, sb = state_of(a, depth), state_of(b, depth)
    assert np.array_equal(sa["ta_state"], sb["ta_state"]), what + " automata"
    for d, (x, y) in enumerate(zip(sa["message_ta_state"], sb["message_ta_state"])):
        assert np.array_equal(x, y), what + " message automata %d" % d
    assert np.array_equal(sa["clause_weights"], sb["clause_weights"]), what + " weights"
    assert np.array_equal(sa["draws"], sb["draws"]), what + " draws consumed"


def assert_same_eval(ra, rb, depth, what=""):
    words = rb["cno"].shape[2]
    assert np.array_equal(ra["cno"][:, :, :words], rb["cno"]), what + " node outputs"
    for d in range(depth - 1):
        assert np.array_equal(ra["messages"][d], rb["messages"][d]), what + " messages %d" % d
    assert np.array_equal(ra["n_inc"], rb["n_inc"]), what + " include counts"
    assert np.array_equal(ra["class_sum"], rb["class_sum"]), what + " class sums"


@pytest.mark.parametrize("name", sorted(CASES))
def test_engine_matches_golden(engine_lib, name):
    kw, graphs, encY, epochs = make_case(name)
    tm = EngineTM(**kw)
    check_against_golden(tm, name, graphs, encY, epochs, kw["depth"])
    tm.close()


@pytest.mark.parametrize("fit_kernel", [1, 2], ids=["state_in_global_memory", "state_resident"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_engine_matches_checker_step_by_step(engine_lib, name, fit_kernel):
    kw, graphs, encY, epochs = make_case(name, seed=200 + sorted(CASES).index(name))
    a, b = OracleTM(**kw), EngineTM(**kw, options={"fit_kernel": fit_kernel})
    for tm in (a, b):
        tm.set_graphs(graphs)
        tm.prepare()
    assert_same_state(a, b, kw["depth"], "init")
    n = graphs.number_of_graphs
    for ep in range(epochs):
        # uneven ranges: a few single graphs, then the rest
        for first, count in [(0, 1), (1, 1), (2, 5), (7, n - 7)]:
            a.fit(encY, first, count)
            b.fit(encY, first, count)
            node, upd = b.last_feedback()
            assert np.array_equal(a.clause_node, node) and np.array_equal(a.update, upd)
        assert_same_state(a, b, kw["depth"], "epoch %d" % ep)
        assert np.array_equal(a.score(), b.score())
    for e in range(0, n, 5):
        ra = a.evaluate_graph(e)
        assert_same_eval(ra, b.evaluate_graph(e, path=0), kw["depth"], "scoring kernel graph %d" % e)
        assert_same_eval(ra, b.evaluate_graph(e, path=1), kw["depth"], "learning kernel graph %d" % e)
    co, cs = b.transform()
    assert np.array_equal(cs, a.score())
    def fired(e):   # only the words of existing nodes are defined
        words = (int(graphs.number_of_graph_nodes[e]) - 1) // 32 + 1
        return a.evaluate_graph(e)["cno"][kw["depth"] - 1][:, :words].any(axis=1)

    last = np.stack([fired(e) for e in range(n)]).astype(np.int32)
    assert np.array_equal(co, last)
    b.close()


@pytest.mark.parametrize("name", ["case_a", "case_c"])
def test_engine_matches_reference_kernels(engine_lib, name):
    kw, graphs, encY, epochs = make_case(name)
    params = dict(classes=kw["classes"], clauses=kw["clauses"], literals=kw["literals"], threshold=kw["threshold"],
                  state_bits=kw.get("state_bits", 8), boost=kw.get("boost", 1), q=kw.get("q", 1.0),
                  max_included=kw.get("max_included"), max_nodes=kw["max_nodes"], message_size=kw["message_size"],
                  message_bits=kw["message_bits"])
    if build_ref.build(params) is None:
        pytest.skip("prebuilt host version of the reference kernels did not travel")
    from oracle.ref_tm import RefTM

    a, b = RefTM(**kw), EngineTM(**kw)
    for tm in (a, b):
        tm.set_graphs(graphs)
        tm.prepare()
    for ep in range(epochs):
        a.fit(encY)
        b.fit(encY)
        assert_same_state(a, b, kw["depth"], "epoch %d" % ep)
        assert np.array_equal(a.score(), b.score())
    b.close()


def test_recorded_draws(engine_lib):
    """Both sides consume the same recorded 32-bit draws (read modulo the buffer length)."""
    kw, graphs, encY, _ = make_case("case_b")
    rec = np.random.default_rng(5).integers(0, 2 ** 32, size=(kw["clauses"], 4099), dtype=np.uint64).astype(np.uint32)
    a, b = OracleTM(**dict(kw, recorded=rec)), EngineTM(**dict(kw, recorded=rec))
    for tm in (a, b):
        tm.set_graphs(graphs)
        tm.prepare()
        tm.fit(encY)
        tm.fit(encY)
    assert_same_state(a, b, kw["depth"])
    b.close()


def test_state_round_trip_and_load(engine_lib):
    """Automata / weights survive set -> get unchanged, and a state trained on the CPU checker scores the same."""
    kw, graphs, encY, _ = make_case("case_e")
    a = OracleTM(**kw)
    a.set_graphs(graphs)
    a.prepare()
    a.fit(encY)
    b = EngineTM(**kw)
    b.set_graphs(graphs)
    b.load_from(a)
    assert_same_state(a, b, kw["depth"])
    assert np.array_equal(a.score(), b.score())
    a.fit(encY)
    b.fit(encY)
    assert_same_state(a, b, kw["depth"], "continued")
    b.close()


@pytest.mark.parametrize("options", [{"fit_block_clauses": 1}, {"fit_block_clauses": 5, "fit_timers": 2},
                                     {"fit_timers": 3}, {"fit_timers": 1, "fit_kernel": 1}],
                         ids=["one_clause_per_block", "five_per_block_timed", "timed", "global_state_timed"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_launch_shape_and_phase_timers_do_not_change_results(engine_lib, name, options):
    """The learning result does not depend on how clauses are spread over thread blocks (every block boundary moves: more
    blocks vote, merge marks and meet at the barriers) nor on the phase timers being on; the timers report something."""
    kw, graphs, encY, epochs = make_case(name, seed=300 + sorted(CASES).index(name))
    a, b = OracleTM(**kw), EngineTM(**kw, options=options)
    for tm in (a, b):
        tm.set_graphs(graphs)
        tm.prepare()
        for _ in range(epochs):
            tm.fit(encY)
    assert_same_state(a, b, kw["depth"], str(options))
    assert np.array_equal(a.score(), b.score())
    if options.get("fit_timers"):
        cycles = (ctypes.c_uint64 * 8)()
        _lib.check(engine_lib.gtm_debug_fit_phase_cycles(b.model, cycles))
        assert sum(cycles) > 0
    b.close()


@pytest.mark.parametrize("fit_kernel", [1, 0], ids=["state_in_global_memory", "automatic"])
@pytest.mark.parametrize("shape", ["wide_literals", "many_clauses", "big_graphs", "many_classes"])
def test_larger_shapes(engine_lib, shape, fit_kernel):
    """Sizes that exercise loops the small cases do not: more than 32 automaton words per clause, more clauses
    than warps in the learning grid, graphs spanning many node words, more classes than lanes."""
    rng = np.random.default_rng(17)
    np.random.seed(17)
    if shape == "wide_literals":
        mk = dict(clauses=64, classes=2, literals=2200, threshold=50, s=8.0, depth=2, message_size=64, message_bits=2, state_bits=12)
        gk, n = dict(hv_size=1100, max_nodes=4, edge_types=2), 30
    elif shape == "many_clauses":
        mk = dict(clauses=6000, classes=3, literals=64, threshold=500, s=3.0, depth=2, message_size=1024, message_bits=2)
        gk, n = dict(hv_size=32, max_nodes=6, edge_types=2), 24
    elif shape == "big_graphs":
        mk = dict(clauses=40, classes=2, literals=48, threshold=30, s=2.5, depth=3, message_size=96, message_bits=2)
        gk, n = dict(hv_size=24, max_nodes=300, node_types=2, edge_types=3), 12
    else:
        mk = dict(clauses=48, classes=70, literals=40, threshold=25, s=2.0, depth=1)
        gk, n = dict(hv_size=20, max_nodes=3), 30
    graphs = random_graphs(n, rng, **gk)
    encY = encode_labels(rng.integers(0, mk["classes"], size=n), mk["classes"], mk["threshold"])
    ms, mb = mk.get("message_size", 256), mk.get("message_bits", 2)
    hv = np.stack([rng.choice(ms, size=mb, replace=False) for _ in range(mk["clauses"])]).astype(np.uint32)
    kw = dict(mk, hypervectors=hv, seed=3, max_nodes=gk["max_nodes"])
    a, b = OracleTM(**kw), EngineTM(**kw, options={"fit_kernel": fit_kernel})
    for tm in (a, b):
        tm.set_graphs(graphs)
        tm.prepare()
        tm.fit(encY)
        tm.fit(encY)
    assert_same_state(a, b, mk["depth"], shape)
    assert np.array_equal(a.score(), b.score())
    b.close()


def test_errors_through_the_abi(engine_lib):
    from graphtsetlinmachine_b200._lib import GtmError

    kw, graphs, encY, _ = make_case("case_a")
    tm = EngineTM(**kw)
    tm.set_graphs(graphs)
    with pytest.raises(GtmError) as e:
        tm.score()                      # no state yet
    assert e.value.status == 5
    tm.prepare()
    with pytest.raises(GtmError) as e:
        tm.score(50, 20)                # range beyond the set
    assert e.value.status == 1
    assert tm.score(3, 0).shape == (0, kw["classes"])     # empty range is fine
    tm.close()


@pytest.mark.parametrize("shape", ["single_node", "small_graphs_types", "big_graphs", "odd_literals_two_classes", "wide"])
def test_node_stream_scoring(engine_lib, shape):
    """Depth-1 scoring goes through the node-stream kernel (tiles of graphs, transposed literals, included-literal
    lists).  Class sums must equal the CPU checker's and the general kernel's (reached through transform), for whole
    sets spanning many tiles and for sub-ranges that start and end inside tiles."""
    rng = np.random.default_rng(23)
    np.random.seed(23)
    if shape == "single_node":
        mk, gk, n = dict(clauses=300, classes=10, literals=256, threshold=80, s=6.0), dict(hv_size=128, fixed_nodes=1, max_nodes=1, max_props=40, symbols=60), 2500
    elif shape == "small_graphs_types":
        mk, gk, n = dict(clauses=150, classes=3, literals=64, threshold=40, s=3.0), dict(hv_size=32, max_nodes=9, node_types=3), 700
    elif shape == "big_graphs":
        mk, gk, n = dict(clauses=90, classes=4, literals=96, threshold=40, s=3.0), dict(hv_size=48, max_nodes=400, node_types=2, max_degree=0), 40
    elif shape == "odd_literals_two_classes":
        mk, gk, n = dict(clauses=77, classes=2, literals=42, threshold=30, s=2.0, max_included=5), dict(hv_size=21, max_nodes=40), 300
    else:
        mk, gk, n = dict(clauses=64, classes=16, literals=4096, threshold=30, s=9.0), dict(hv_size=2048, max_nodes=20, symbols=200, max_props=30), 150
    graphs = random_graphs(n, rng, **gk)
    encY = encode_labels(rng.integers(0, mk["classes"], size=n), mk["classes"], mk["threshold"])
    kw = dict(mk, depth=1, seed=5, max_nodes=gk["max_nodes"])
    a, b = OracleTM(**kw), EngineTM(**kw)
    for tm in (a, b):
        tm.set_graphs(graphs)
        tm.prepare()
    assert np.array_equal(a.score(), b.score()), "fresh model"
    for _ in range(2):
        a.fit(encY)
        b.fit(encY)
        want = a.score()
        assert np.array_equal(want, b.score()), "node-stream kernel"
        assert np.array_equal(want, b.transform()[1]), "general kernel"
    for first, count in [(1, 1), (n // 3, n // 2), (n - 5, 5), (0, n - 1)]:
        assert np.array_equal(want[first:first + count], b.score(first, count)), "sub-range"
    b.close()


def test_wait_that_runs_out_ends_the_launch_cleanly(engine_lib):
    """Failure path of the learning kernels without a faulted GPU: with the test hook `fit_missing_cta` every device-side
    wait expects an arrival that never comes (a thread block, or on several GPUs a rank, that does not show up).  The
    waits are bounded by wall time, so the launch ends by itself, gtm_fit reports GTM_ERR_TIMEOUT, the CUDA context stays
    usable, and after restoring the state the same model learns on, bit for bit like the checker."""
    import ctypes as C
    import time

    from graphtsetlinmachine_b200 import _lib
    from oracle.oracle import OracleTM

    for name, fit_kernel in (("case_d", 0), ("case_b", 1), ("case_b", 2)):
        kw, graphs, encY, _ = make_case(name)
        kw = dict(kw, clauses=400)                       # several thread blocks, so that there is something to wait for
        rng = np.random.default_rng(3)
        kw["hypervectors"] = np.stack([rng.choice(kw["message_size"], size=kw["message_bits"], replace=False)
                                       for _ in range(400)]).astype(np.uint32)
        cpu, gpu = OracleTM(**kw), EngineTM(**kw, options={"fit_kernel": fit_kernel})
        for tm in (cpu, gpu):
            tm.set_graphs(graphs)
            tm.prepare()
            tm.fit(encY)
        assert_same_state(cpu, gpu, kw["depth"], "before the failed launch")
        _lib.check(engine_lib.gtm_set_option(gpu.model, b"fit_wait_ms", 30))
        _lib.check(engine_lib.gtm_set_option(gpu.model, b"fit_missing_cta", 1))
        t0 = time.perf_counter()
        with pytest.raises(_lib.GtmError) as err:
            gpu.fit(encY)
        assert err.value.status == 4 and time.perf_counter() - t0 < 5.0          # GTM_ERR_TIMEOUT, promptly
        _lib.check(engine_lib.gtm_set_option(gpu.model, b"fit_missing_cta", 0))
        _lib.check(engine_lib.gtm_set_option(gpu.model, b"fit_wait_ms", 2000))
        gpu.load_from(cpu)                                # restore the checkpoint (a global-state launch may have applied updates)
        for tm in (cpu, gpu):
            tm.fit(encY)
        assert_same_state(cpu, gpu, kw["depth"], "after the failed launch")
        assert np.array_equal(cpu.score(), gpu.score())
        gpu.close()
