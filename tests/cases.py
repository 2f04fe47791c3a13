"""Differential-test cases shared by the CPU and GPU suites: small seeded models and graph sets that cover odd
literal counts, message sizes that are not multiples of 32, several node and edge types, graphs larger than one
node word, boosting on/off, a literal budget, non-default state bits and q."""

import numpy as np

from util import encode_labels, random_graphs

# name -> (model keyword arguments, graph-set keyword arguments, number of graphs, epochs)
CASES = {
    "case_a": (dict(clauses=20, classes=2, literals=64, threshold=20, s=1.5, depth=2, message_size=64, message_bits=2),
               dict(hv_size=32, max_nodes=5, node_types=1, edge_types=2), 60, 3),
    "case_b": (dict(clauses=33, classes=3, literals=80, threshold=30, s=2.0, depth=3, message_size=50, message_bits=2,
                    boost=0, max_included=6),
               dict(hv_size=40, max_nodes=40, node_types=2, edge_types=3), 60, 3),
    "case_c": (dict(clauses=16, classes=4, literals=32, threshold=15, s=3.0, depth=2, message_size=37, message_bits=1,
                    state_bits=6, q=0.5),
               dict(hv_size=16, max_nodes=70, node_types=3, edge_types=1), 60, 3),
    "case_d": (dict(clauses=50, classes=5, literals=128, threshold=40, s=4.0, depth=1, message_size=128, message_bits=3),
               dict(hv_size=64, max_nodes=3, node_types=1, edge_types=1), 60, 3),
    "case_e": (dict(clauses=24, classes=2, literals=42, threshold=10, s=1.0, depth=4, message_size=33, message_bits=2,
                    max_included=3),
               dict(hv_size=21, max_nodes=9, node_types=2, edge_types=4), 60, 3),
}


def make_case(name, seed=None):
    """Returns (model kwargs incl. hypervectors/seed/max_nodes, graphs, encoded_Y, epochs)."""
    model_kw, graph_kw, n_graphs, epochs = CASES[name]
    seed = sorted(CASES).index(name) + 1 if seed is None else seed
    rng = np.random.default_rng(seed)
    np.random.seed(seed)
    graphs = random_graphs(n_graphs, rng, **graph_kw)
    Y = rng.integers(0, model_kw["classes"], size=n_graphs)
    hv = np.stack([rng.choice(model_kw["message_size"], size=model_kw["message_bits"], replace=False)
                   for _ in range(model_kw["clauses"])]).astype(np.uint32)
    kw = dict(model_kw, hypervectors=hv, seed=seed, max_nodes=graph_kw["max_nodes"])
    return kw, graphs, encode_labels(Y, model_kw["classes"], model_kw["threshold"]), epochs


def state_of(tm, depth):
    """Comparable snapshot of a checker or of the engine."""
    return dict(ta_state=np.array(tm.ta_state), message_ta_state=[np.array(m) for m in tm.message_ta_state][: depth - 1],
                clause_weights=np.array(tm.clause_weights), draws=np.array(tm.draws_consumed(), dtype=np.uint64))
