"""GPU suite, tile scoring kernel (``score_kernel`` = 3): batched inference for any depth on graphs of at most 128
nodes.  Class sums must equal the CPU checker's (``oracle/``) and the general scoring kernel's, bit for bit, on

* the differential-test cases (depth 1..4, message sizes that are not multiples of 32, several node and edge types),
* hypothesis-drawn shapes,
* the Noisy-XOR and multigraph configurations (uniform and ragged graph sizes, many tiles, sub-ranges),
* freshly initialised models (every clause empty, hence true on every node of its type: the densest message case).
"""

import numpy as np
import pytest
from hypothesis import HealthCheck, given, settings, strategies as st

from cases import CASES, make_case
from graphtsetlinmachine_b200 import datasets
from oracle.oracle import OracleTM
from util import EngineTM, encode_labels, random_graphs

pytestmark = pytest.mark.gpu

TILE = {"score_kernel": 3}


@pytest.mark.parametrize("name", sorted(CASES))
def test_cases_match_checker_and_general_kernel(engine_lib, name):
    kw, graphs, encY, epochs = make_case(name)
    cpu, gpu = OracleTM(**kw), EngineTM(**kw, options=TILE)
    for tm in (cpu, gpu):
        tm.set_graphs(graphs)
        tm.prepare()
    fresh = gpu.score()
    assert np.array_equal(fresh, cpu.score())                 # every clause empty
    for _ in range(epochs):
        cpu.fit(encY)
        gpu.fit(encY)
    want = cpu.score()
    assert np.array_equal(gpu.score(), want)
    assert np.array_equal(gpu.transform()[1], want)           # general kernel
    n = graphs.number_of_graphs
    for first, count in [(0, 1), (n // 3, n // 4), (n - 2, 2), (7, 0)]:
        assert np.array_equal(gpu.score(first, count), want[first:first + count])
    gpu.close()


@settings(max_examples=40, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)
@given(seed=st.integers(0, 10 ** 6), clauses=st.integers(1, 90), classes=st.integers(1, 12), hv=st.integers(3, 75),
       depth=st.integers(1, 4), ms=st.integers(2, 140), mb=st.integers(1, 3), max_nodes=st.integers(1, 128),
       node_types=st.integers(1, 4), edge_types=st.integers(1, 5), uniform=st.booleans(), n=st.integers(1, 70))
def test_random_shapes_match_checker(engine_lib, seed, clauses, classes, hv, depth, ms, mb, max_nodes, node_types,
                                     edge_types, uniform, n):
    rng = np.random.default_rng(seed)
    np.random.seed(seed % (2 ** 31))
    graphs = random_graphs(n, rng, hv_size=hv, hv_bits=min(2, hv), max_nodes=max_nodes, node_types=node_types,
                           edge_types=edge_types, fixed_nodes=max_nodes if uniform else None)
    T = int(rng.integers(2, 40))
    encY = encode_labels(rng.integers(0, classes, size=n), classes, T)
    mb = min(mb, ms)
    hvs = np.stack([rng.choice(ms, size=mb, replace=False) for _ in range(clauses)]).astype(np.uint32)
    kw = dict(clauses=clauses, classes=classes, literals=2 * hv, threshold=T, s=float(rng.choice([1.0, 2.0, 6.0])),
              depth=depth, message_size=ms, message_bits=mb, max_nodes=max_nodes, hypervectors=hvs, seed=seed)
    a, b = OracleTM(**kw), EngineTM(**kw, options=TILE)
    try:
        for tm in (a, b):
            tm.set_graphs(graphs)
            tm.prepare()
        assert np.array_equal(a.score(), b.score())
        for tm in (a, b):
            tm.fit(encY)
            tm.fit(encY)
        assert np.array_equal(a.clause_weights, b.clause_weights)
        want = a.score()
        assert np.array_equal(want, b.score())
        assert np.array_equal(want[n // 2:], b.score(n // 2, n - n // 2))
    finally:
        b.close()


def test_noisy_xor_many_tiles(engine_lib):
    """Two-node graphs, depth 2: tens of thousands of graphs over many tiles against the general kernel, a prefix against
    the checker; the tile kernel is also what the automatic choice takes for this shape."""
    np.random.seed(3)
    train, y = datasets.noisy_xor(3000, 1)
    test, _ = datasets.noisy_xor(40000, 2, init_with=train)
    rng = np.random.default_rng(4)
    hv = np.stack([rng.choice(256, size=2, replace=False) for _ in range(10)]).astype(np.uint32)
    kw = dict(clauses=10, classes=2, literals=64, threshold=100, s=2.0, depth=2, message_size=256, message_bits=2,
              max_included=4, max_nodes=2, hypervectors=hv, seed=9)
    cpu = OracleTM(**kw)
    tile, auto, general = EngineTM(**kw, options=TILE), EngineTM(**kw), EngineTM(**kw, options={"score_kernel": 1})
    encY = encode_labels(y, 2, 100)
    cpu.set_graphs(train)
    cpu.prepare()
    for _ in range(3):
        cpu.fit(encY)
    for tm in (tile, auto, general):
        tm.set_graphs(test)
        tm.load_from(cpu)
    want = general.score()
    assert np.array_equal(tile.score(), want)
    assert np.array_equal(auto.score(), want)
    cpu.set_graphs(test)
    assert np.array_equal(cpu.score(0, 500), want[:500])
    assert len(np.unique(want, axis=0)) > 2
    for first, count in [(1, 1), (511, 3), (512, 512), (39990, 10), (12345, 20000)]:
        assert np.array_equal(tile.score(first, count), want[first:first + count])
    for tm in (tile, auto, general):
        tm.close()


@pytest.mark.parametrize("clauses,n_graphs,n_check", [(600, 1500, 40), (20000, 400, 6)])
def test_multigraphs_depth_three(engine_lib, clauses, n_graphs, n_check):
    """The multigraph configuration (8..32 nodes, Poisson degrees, 4 edge types, hypervectors of 1,024 bits, depth 3,
    1,024 message bits): ragged tiles.  Tile kernel == general kernel on all graphs, == checker on a few."""
    np.random.seed(5)
    graphs, y = datasets.random_multigraphs(n_graphs, 3)
    rng = np.random.default_rng(9)
    hv = np.stack([rng.choice(1024, size=2, replace=False) for _ in range(clauses)]).astype(np.uint32)
    T = max(10, clauses // 2)
    kw = dict(clauses=clauses, classes=10, literals=2048, threshold=T, s=10.0, depth=3, message_size=1024, message_bits=2,
              max_nodes=int(graphs.max_number_of_graph_nodes), hypervectors=hv, seed=11)
    tile, general = EngineTM(**kw, options=TILE), EngineTM(**kw, options={"score_kernel": 1})
    encY = encode_labels(y, 10, T)
    tile.set_graphs(graphs)
    tile.prepare()
    tile.fit(encY, 0, min(n_graphs, 150), epochs=2)
    general.set_graphs(graphs)
    general.set_ta(0, tile.get_ta(0))
    for d in (1, 2):
        general.set_ta(d, tile.get_ta(d))
    general.set_weights(tile.clause_weights)
    want = general.score()
    got = tile.score()
    assert np.array_equal(got, want)
    assert np.abs(want).sum() > 0 and len(np.unique(want, axis=0)) > 10
    cpu = OracleTM(**kw)
    cpu.set_graphs(graphs)
    cpu.ta_state[...] = tile.get_ta(0)
    for d in (1, 2):
        cpu.message_ta_state[d - 1][...] = tile.get_ta(d)
    cpu.clause_weights[...] = tile.clause_weights
    assert np.array_equal(cpu.score(0, n_check), want[:n_check])
    perm = np.random.default_rng(1).permutation(n_graphs)[:200]
    sub = graphs[perm]
    tile.set_graphs(sub)
    assert np.array_equal(tile.score(), want[perm])            # other tiles, other slots: same sums
    tile.close()
    general.close()


def test_graphs_of_exactly_one_quad_and_many_types(engine_lib):
    """128-node graphs (a whole quad each), 8 node types, depth 2, odd message size."""
    rng = np.random.default_rng(21)
    np.random.seed(21)
    graphs = random_graphs(20, rng, hv_size=20, max_nodes=128, fixed_nodes=128, node_types=8, edge_types=3, max_degree=2)
    hv = np.stack([rng.choice(77, size=2, replace=False) for _ in range(40)]).astype(np.uint32)
    kw = dict(clauses=40, classes=3, literals=40, threshold=20, s=2.0, depth=2, message_size=77, message_bits=2,
              max_nodes=128, hypervectors=hv, seed=2)
    a, b = OracleTM(**kw), EngineTM(**kw, options=TILE)
    encY = encode_labels(rng.integers(0, 3, size=20), 3, 20)
    for tm in (a, b):
        tm.set_graphs(graphs)
        tm.prepare()
        tm.fit(encY)
    assert np.array_equal(a.score(), b.score())
    b.close()


def test_tile_kernel_refuses_what_it_cannot_serve(engine_lib):
    """Graphs of more than 128 nodes do not fit a quad: forcing the tile kernel is an argument error, the automatic
    choice falls back to the general kernel."""
    rng = np.random.default_rng(2)
    np.random.seed(2)
    graphs = random_graphs(3, rng, hv_size=16, max_nodes=150, fixed_nodes=150, max_degree=1)
    kw = dict(clauses=12, classes=2, literals=32, threshold=10, s=2.0, depth=2, message_size=64, message_bits=2, max_nodes=150)
    tm = EngineTM(**kw, options=TILE)
    tm.set_graphs(graphs)
    tm.prepare()
    with pytest.raises(Exception, match="tile scoring kernel"):
        tm.score()
    tm.close()
