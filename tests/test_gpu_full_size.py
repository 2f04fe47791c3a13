"""GPU suite at the model sizes of the benchmark configurations (2,500 / 2,000 / 20,000 clauses, hypervectors up to
1,024 bits, depth up to 3), on seeded synthetic graph sets of the configurations' shapes.

* against the CPU checker on a handful of graphs (a full fit step and scores, equality);
* size-independent properties on large sets: the two scoring kernels (different algorithms) agree graph for graph,
  scoring is invariant under reordering and replication of the graphs, sub-ranges equal slices, and a freshly
  initialised model votes with every clause of a node type that occurs in the graph.
"""

import numpy as np
import pytest

from graphtsetlinmachine_b200 import datasets
from oracle.oracle import OracleTM
from util import EngineTM, encode_labels

pytestmark = pytest.mark.gpu


def config(name, n):
    np.random.seed(5)
    if name == "vanilla":
        g, y = datasets.vanilla_images(n, 3, datasets.image_prototypes(1))
        kw = dict(clauses=2500, classes=10, literals=256, threshold=3125, s=10.0, depth=1, max_nodes=1)
    elif name == "convolution":
        g, y = datasets.convolution_images(n, 3, datasets.image_prototypes(1))
        kw = dict(clauses=2500, classes=10, literals=256, threshold=3125, s=10.0, depth=1, max_nodes=361)
    elif name == "sequence":
        g, y = datasets.sequences(n, 3)
        kw = dict(clauses=2000, classes=2, literals=512, threshold=2000, s=5.0, depth=3, message_size=512, message_bits=2,
                  max_nodes=1000)
    else:
        g, y = datasets.random_multigraphs(n, 3)
        kw = dict(clauses=20000, classes=10, literals=2048, threshold=10000, s=10.0, depth=3, message_size=1024,
                  message_bits=2, max_nodes=int(g.max_number_of_graph_nodes))
    rng = np.random.default_rng(9)
    hv = np.stack([rng.choice(kw.get("message_size", 256), size=kw.get("message_bits", 2), replace=False)
                   for _ in range(kw["clauses"])]).astype(np.uint32)
    return dict(kw, hypervectors=hv, seed=11), g, encode_labels(y, kw["classes"], kw["threshold"])


@pytest.mark.parametrize("name,n", [("vanilla", 40), ("convolution", 6), ("sequence", 4), ("multigraph", 6)])
def test_full_size_models_match_checker(engine_lib, name, n):
    kw, graphs, encY = config(name, n)
    a, b = OracleTM(**kw), EngineTM(**kw)
    for tm in (a, b):
        tm.set_graphs(graphs)
        tm.prepare()
        tm.fit(encY)
    assert np.array_equal(a.ta_state, b.ta_state)
    for x, y in zip(a.message_ta_state, b.message_ta_state):
        assert np.array_equal(x, y)
    assert np.array_equal(a.clause_weights, b.clause_weights)
    assert np.array_equal(a.draws_consumed(), b.draws_consumed())
    assert np.array_equal(a.score(), b.score())
    b.close()


@pytest.mark.parametrize("name,n,train", [("vanilla", 60000, 3000), ("convolution", 400, 60)])
def test_scoring_kernels_agree_and_scoring_is_order_independent(engine_lib, name, n, train):
    kw, graphs, encY = config(name, n)
    tm = EngineTM(**kw)
    tm.set_graphs(graphs)
    tm.prepare()
    fresh = tm.score()
    weights = tm.clause_weights
    assert np.array_equal(fresh, np.tile(weights.sum(axis=1), (n, 1)))       # every clause empty: all vote everywhere
    tm.fit(encY, 0, train)
    stream = tm.score()                                                       # node-stream kernel
    general = tm.transform()[1]                                               # general kernel
    assert np.array_equal(stream, general)
    assert np.abs(stream).sum() > 0 and len(np.unique(stream, axis=0)) > 10
    for first, count in [(0, 1), (n // 3, n // 7), (n - 3, 3)]:
        assert np.array_equal(tm.score(first, count), stream[first:first + count])
    perm = np.random.default_rng(1).permutation(n)[: min(n, 5000)]
    sub = graphs[perm]
    tm2 = EngineTM(**kw)
    tm2.set_graphs(sub)
    tm2.set_ta(0, tm.get_ta(0))
    tm2.set_weights(tm.clause_weights)
    assert np.array_equal(tm2.score(), stream[perm])
    rep = datasets.replicate(sub, 3)
    tm2.set_graphs(rep)
    assert np.array_equal(tm2.score(), np.tile(stream[perm], (3, 1)))
    tm.close()
    tm2.close()
