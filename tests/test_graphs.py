"""CPU suite, part 2: the host-side graph encoder against vectors produced by the reference's ``Graphs`` class
(tests/golden/graphs_*.npz) and its error behaviour."""

import os

import numpy as np
import pytest

from graphtsetlinmachine_b200 import datasets
from graphtsetlinmachine_b200.graphs import Graphs
from golden.make_golden import GRAPH_FIELDS, GRAPH_VARIANTS, scripted_build

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("variant", sorted(GRAPH_VARIANTS))
def test_encoder_matches_reference_vectors(variant):
    gold = np.load(os.path.join(GOLDEN, "graphs_%s.npz" % variant))
    train, test = scripted_build(Graphs, 11, **GRAPH_VARIANTS[variant])
    for f in GRAPH_FIELDS:
        assert np.array_equal(getattr(train, f), gold["train_" + f]), f
        assert getattr(train, f).dtype == gold["train_" + f].dtype, f
        assert np.array_equal(getattr(test, f), gold["test_" + f]), f
    assert train.signature == gold["train_signature"].tobytes()
    assert test.signature == gold["test_signature"].tobytes()
    sub = train[[5, 1, -1]]
    for f in GRAPH_FIELDS[:-1]:
        assert np.array_equal(getattr(sub, f), gold["subset_" + f]), f
    assert test.hypervectors is train.hypervectors and test.symbol_id is train.symbol_id


def test_index_errors():
    g, _ = datasets.noisy_xor(5, 1)
    with pytest.raises(IndexError):
        g[5]
    with pytest.raises(IndexError):
        g[[0, -6]]
    with pytest.raises(TypeError):
        g["a"]
    with pytest.raises(ValueError):
        g[3:3]
    assert len(g[1:4]) == 3 and len(g[-1]) == 1


def test_edge_count_checks_exit():
    g = Graphs(1, symbols=["A"], hypervector_size=8, hypervector_bits=1)
    g.set_number_of_graph_nodes(0, 2)
    g.prepare_node_configuration()
    g.add_graph_node(0, "a", 1)
    g.add_graph_node(0, "b", 0)
    g.prepare_edge_configuration()
    with pytest.raises(SystemExit):
        g.encode()                      # node 'a' misses an edge
    g.add_graph_node_edge(0, "a", "b", "t")
    with pytest.raises(SystemExit):
        g.add_graph_node_edge(0, "a", "b", "t")   # too many
    g.encode()


def test_bulk_builders_equal_per_item_api():
    np.random.seed(3)
    bulk, _ = datasets.sequences(3, 5, length=7, hv_size=24)
    np.random.seed(3)
    ref = Graphs(3, symbols=["A", "B", "C", "D"], hypervector_size=24, hypervector_bits=2)
    sym = np.random.default_rng(5).integers(0, 4, size=(3, 7))
    for i in range(3):
        ref.set_number_of_graph_nodes(i, 7)
    ref.prepare_node_configuration()
    for i in range(3):
        for v in range(7):
            ref.add_graph_node(i, v, 2 if 0 < v < 6 else 1)
    ref.prepare_edge_configuration()
    for i in range(3):
        for v in range(7):
            if v > 0:
                ref.add_graph_node_edge(i, v, v - 1, "Left")
            if v < 6:
                ref.add_graph_node_edge(i, v, v + 1, "Right")
            ref.add_graph_node_property(i, v, "ABCD"[sym[i, v]])
    ref.encode()
    for f in GRAPH_FIELDS:
        assert np.array_equal(getattr(bulk, f), getattr(ref, f)), f
    assert bulk.signature == ref.signature
