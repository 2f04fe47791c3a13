"""GPU suite, randomised: hypothesis draws small model / graph-set shapes (odd literal counts, message sizes that
are not multiples of 32, several node types, state bits, budgets, boosting on/off) and the engine must equal the CPU
checker after training: automata, weights, draws, scores."""

import numpy as np
import pytest
from hypothesis import HealthCheck, given, settings, strategies as st

from oracle.oracle import OracleTM
from util import EngineTM, encode_labels, random_graphs

pytestmark = pytest.mark.gpu


@settings(max_examples=30, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)
@given(seed=st.integers(0, 10 ** 6), clauses=st.integers(1, 70), classes=st.integers(1, 6), hv=st.integers(3, 75),
       depth=st.integers(1, 3), ms=st.integers(2, 140), mb=st.integers(1, 2), max_nodes=st.integers(1, 45),
       node_types=st.integers(1, 3), sb=st.sampled_from([2, 5, 8, 8, 8, 11]), boost=st.integers(0, 1),
       s=st.sampled_from([1.0, 1.3, 2.0, 4.5, 10.0]), q=st.sampled_from([0.2, 1.0, 2.5]),
       budget=st.sampled_from([None, 1, 4, 20]), fit_kernel=st.sampled_from([0, 1]))
def test_engine_equals_checker_on_random_shapes(engine_lib, seed, clauses, classes, hv, depth, ms, mb, max_nodes,
                                                node_types, sb, boost, s, q, budget, fit_kernel):
    rng = np.random.default_rng(seed)
    np.random.seed(seed % (2 ** 31))
    n = 14
    graphs = random_graphs(n, rng, hv_size=hv, hv_bits=min(2, hv), max_nodes=max_nodes, node_types=node_types,
                           edge_types=int(rng.integers(1, 4)))
    T = int(rng.integers(2, 40))
    encY = encode_labels(rng.integers(0, classes, size=n), classes, T)
    mb = min(mb, ms)
    hvs = np.stack([rng.choice(ms, size=mb, replace=False) for _ in range(clauses)]).astype(np.uint32)
    kw = dict(clauses=clauses, classes=classes, literals=2 * hv, threshold=T, s=s, depth=depth, message_size=ms,
              message_bits=mb, max_included=budget, boost=boost, state_bits=sb, q=q, max_nodes=max_nodes,
              hypervectors=hvs, seed=seed)
    a, b = OracleTM(**kw), EngineTM(**kw, options={"fit_kernel": fit_kernel})
    try:
        for tm in (a, b):
            tm.set_graphs(graphs)
            tm.prepare()
            tm.fit(encY)
            tm.fit(encY, 3, 8)
        assert np.array_equal(a.ta_state, b.ta_state)
        for x, y in zip(a.message_ta_state, b.message_ta_state):
            assert np.array_equal(x, y)
        assert np.array_equal(a.clause_weights, b.clause_weights)
        assert np.array_equal(a.draws_consumed(), b.draws_consumed())
        assert np.array_equal(a.score(), b.score())
        assert np.array_equal(a.score(), b.transform()[1])
    finally:
        b.close()


@pytest.mark.parametrize("hv,ms,max_nodes,depth", [(24, 96, 40, 3), (5, 37, 70, 2), (40, 64, 33, 3), (16, 512, 200, 2)])
def test_large_graphs_with_few_node_words(engine_lib, hv, ms, max_nodes, depth):
    """Graphs of more than 32 nodes go through the transposed evaluation, whose rows are only as long as the graph
    set's node words: shapes with two to seven node words, odd and even message word counts, against the checker."""
    rng = np.random.default_rng(hv + ms)
    np.random.seed(hv + ms)
    n, clauses, classes, T = 24, 50, 2, 25
    graphs = random_graphs(n, rng, hv_size=hv, hv_bits=2, max_nodes=max_nodes, node_types=2, edge_types=3)
    graphs_big = random_graphs(n, rng, hv_size=hv, hv_bits=2, fixed_nodes=max_nodes, node_types=2, edge_types=3, init_with=graphs)
    encY = encode_labels(rng.integers(0, classes, size=n), classes, T)
    hvs = np.stack([rng.choice(ms, size=2, replace=False) for _ in range(clauses)]).astype(np.uint32)
    kw = dict(clauses=clauses, classes=classes, literals=2 * hv, threshold=T, s=2.0, depth=depth, message_size=ms,
              message_bits=2, max_nodes=max_nodes, hypervectors=hvs, seed=9)
    for fit_kernel in (0, 1):
        a, b = OracleTM(**kw), EngineTM(**kw, options={"fit_kernel": fit_kernel})
        try:
            for g in (graphs, graphs_big):
                for tm in (a, b):
                    tm.set_graphs(g)
                    if g is graphs:
                        tm.prepare()
                    tm.fit(encY)
                assert np.array_equal(a.ta_state, b.ta_state)
                for x, y in zip(a.message_ta_state, b.message_ta_state):
                    assert np.array_equal(x, y)
                assert np.array_equal(a.clause_weights, b.clause_weights)
                assert np.array_equal(a.score(), b.score())
                assert np.array_equal(a.score(), b.transform()[1])
        finally:
            b.close()
