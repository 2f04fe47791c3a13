"""CPU suite, part 1: the checker itself.

* Philox4x32-10 known answers (Random123 test vectors).
* The C restatement (oracle/gtm_oracle.c) reproduces the golden vectors that the reference's own kernels produced
  (tests/golden/case_*.npz, made by tests/golden/make_golden.py).
* Where a reference checkout or a prebuilt host version of the reference kernels is present, the restatement is
  run side by side with it.
* Derived known answers: a freshly initialised model votes with every clause; automata saturate.
"""

import os

import numpy as np
import pytest

from cases import CASES, make_case, state_of
from oracle import build_ref
from oracle.oracle import OracleTM, philox4x32_10

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_philox_known_answers():
    assert philox4x32_10([0, 0, 0, 0], [0, 0]) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert philox4x32_10([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert philox4x32_10([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0]) == [
        0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]


def check_against_golden(tm, name, graphs, encY, epochs, depth):
    gold = np.load(os.path.join(GOLDEN, name + ".npz"))
    tm.set_graphs(graphs)
    tm.prepare()
    assert np.array_equal(tm.clause_weights, gold["init_weights"])
    for ep in range(epochs):
        tm.fit(encY)
        st = state_of(tm, depth)
        assert np.array_equal(st["ta_state"], gold["ta_%d" % ep]), "automata, epoch %d" % ep
        for d in range(depth - 1):
            assert np.array_equal(st["message_ta_state"][d], gold["mta%d_%d" % (d, ep)]), "message automata"
        assert np.array_equal(st["clause_weights"], gold["weights_%d" % ep]), "weights"
        assert np.array_equal(st["draws"], gold["draws_%d" % ep]), "draws consumed"
        assert np.array_equal(tm.score(), gold["scores_%d" % ep]), "scores"
    for e in range(8):
        r = tm.evaluate_graph(e)
        words = gold["g%d_cno" % e].shape[2]
        assert np.array_equal(r["cno"][:, :, :words], gold["g%d_cno" % e])
        for d in range(depth - 1):
            assert np.array_equal(r["messages"][d], gold["g%d_msg%d" % (e, d)])
        assert np.array_equal(r["n_inc"], gold["g%d_ninc" % e])
        assert np.array_equal(r["class_sum"], gold["g%d_sum" % e])


@pytest.mark.parametrize("name", sorted(CASES))
def test_restatement_matches_golden(name):
    kw, graphs, encY, epochs = make_case(name)
    check_against_golden(OracleTM(**kw), name, graphs, encY, epochs, kw["depth"])


@pytest.mark.parametrize("name", sorted(CASES))
def test_restatement_matches_compiled_reference(name):
    kw, graphs, encY, epochs = make_case(name, seed=100 + sorted(CASES).index(name))
    params = dict(classes=kw["classes"], clauses=kw["clauses"], literals=kw["literals"], threshold=kw["threshold"],
                  state_bits=kw.get("state_bits", 8), boost=kw.get("boost", 1), q=kw.get("q", 1.0),
                  max_included=kw.get("max_included"), max_nodes=kw["max_nodes"], message_size=kw["message_size"],
                  message_bits=kw["message_bits"])
    if build_ref.build(params) is None:
        pytest.skip("no reference checkout and no prebuilt host version of the reference kernels")
    from oracle.ref_tm import RefTM

    a, b = RefTM(**kw), OracleTM(**kw)
    for tm in (a, b):
        tm.set_graphs(graphs)
        tm.prepare()
    for ep in range(epochs):
        a.fit(encY)
        b.fit(encY)
        sa, sb = state_of(a, kw["depth"]), state_of(b, kw["depth"])
        assert np.array_equal(sa["ta_state"], sb["ta_state"])
        for x, y in zip(sa["message_ta_state"], sb["message_ta_state"]):
            assert np.array_equal(x, y)
        assert np.array_equal(sa["clause_weights"], sb["clause_weights"])
        assert np.array_equal(sa["draws"], sb["draws"])
        assert np.array_equal(a.clause_node, b.clause_node)
        assert np.array_equal(a.class_clause_update, b.update)
        assert np.array_equal(a.score(), b.score())


def test_fresh_model_votes_with_every_clause():
    """Right after initialisation no literal is included, so every clause is true on every node of its node type
    and each class sum is the sum of the weights of the clauses whose type occurs in the graph."""
    kw, graphs, _, _ = make_case("case_b")
    tm = OracleTM(**kw)
    tm.set_graphs(graphs)
    tm.prepare()
    scores = tm.score()
    nt = graphs.number_of_node_types()
    for e in range(graphs.number_of_graphs):
        lo = int(graphs.node_index[e])
        present = set(graphs.node_type[lo:lo + int(graphs.number_of_graph_nodes[e])].tolist())
        active = np.array([c % nt in present for c in range(kw["clauses"])])
        assert np.array_equal(scores[e], tm.clause_weights[:, active].sum(axis=1))


def test_recorded_draws_drive_the_restatement():
    """With recorded all-zero draws every uniform is 2^-33: every feedback decision fires and every mask is all
    ones; with all-ones draws (uniform = 1.0) only decisions of probability 1 fire (the target class of a graph whose
    clamped sum sits at -T), and no negative-target class is ever kept."""
    kw, graphs, encY, _ = make_case("case_d")
    zeros = np.zeros((kw["clauses"], 64), dtype=np.uint32)
    tm = OracleTM(**dict(kw, recorded=zeros))
    tm.set_graphs(graphs)
    tm.prepare()
    assert np.all(tm.clause_weights == 1)            # 1 - 2*(0 % 2)
    tm.fit(encY, 0, 1)
    # sums clamp to +T: the target class has error 0 (never fires), every other class error 2T (always fires)
    assert np.all(tm.update[encY[0] < 0] == -1) and np.all(tm.update[encY[0] > 0] == 0)
    ones = np.full((kw["clauses"], 64), 0xFFFFFFFF, dtype=np.uint32)
    tm = OracleTM(**dict(kw, recorded=ones))
    tm.set_graphs(graphs)
    tm.prepare()
    assert np.all(tm.clause_weights == -1)
    tm.fit(encY, 0, 1)
    negative_target = encY[0] < 0
    assert np.all(tm.update[negative_target] == 0)
    assert np.all(tm.update[~negative_target] == -1)   # sum clamps to -T: error/(2T) = 1; target +1 times sign -1
