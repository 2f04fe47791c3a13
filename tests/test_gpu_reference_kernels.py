"""The reference's own kernels, compiled for the GPU and launched the way the reference's host code launches them,
against the engine on the same GPU: bit-exact inference from an identical loaded state, and learning compared
statistically (the reference draws from per-thread XORWOW states, the engine from one Philox stream per clause)."""

import numpy as np
import pytest

from cases import make_case
from util import EngineTM, encode_labels

pytestmark = pytest.mark.gpu


def _reference(kw):
    from oracle.ref_gpu_tm import RefGpuTM

    try:
        return RefGpuTM(**kw)
    except FileNotFoundError:
        pytest.skip("no GPU build of the reference kernels for this hyper-parameter set")


@pytest.mark.parametrize("name", ["case_b", "case_e"])
def test_inference_matches_reference_kernels_on_the_gpu(name):
    kw, graphs, Y, epochs = make_case(name)
    engine = EngineTM(**kw)
    engine.set_graphs(graphs)
    engine.prepare()
    engine.fit(Y, epochs=epochs)
    ref = _reference(kw)
    ref.set_graphs(graphs)
    ref.load_from(engine)
    np.testing.assert_array_equal(ref.score(), engine.score())
    for e in range(0, graphs.number_of_graphs, 7):
        a, b = ref.evaluate_graph(e), engine.evaluate_graph(e)
        np.testing.assert_array_equal(a["cno"], b["cno"], err_msg="node outputs, graph %d" % e)
        for d in range(kw["depth"] - 1):
            np.testing.assert_array_equal(a["messages"][d], b["messages"][d], err_msg="messages, graph %d layer %d" % (e, d))
        np.testing.assert_array_equal(a["n_inc"], b["n_inc"])
        np.testing.assert_array_equal(a["class_sum"], b["class_sum"])


def test_vanilla_inference_matches_reference_kernels_on_the_gpu():
    from graphtsetlinmachine_b200 import datasets

    protos = datasets.image_prototypes(1)
    train, y = datasets.vanilla_images(600, 2, protos)
    test, _ = datasets.vanilla_images(300, 3, protos, init_with=train)
    kw = dict(clauses=2500, classes=10, literals=256, threshold=3125, s=10.0, depth=1, max_nodes=1, seed=5)
    engine = EngineTM(**kw)
    engine.set_graphs(train)
    engine.prepare()
    engine.fit(encode_labels(y, 10, 3125), epochs=1)
    ref = _reference(kw)
    ref.load_from(engine)
    ref.set_graphs(test)
    engine.set_graphs(test)
    np.testing.assert_array_equal(ref.score(), engine.score())


def _included(ta_state):
    """Number of included literals: set bits of the top state plane."""
    top = np.ascontiguousarray(ta_state[:, :, -1])
    return int(np.unpackbits(top.view(np.uint8)).sum())


def test_vanilla_learning_is_statistically_equivalent():
    """2500 clauses, two passes over 1500 single-node graphs, four seeds per learner: the seed-to-seed spread of the
    included-literal count is about 3 % for either learner, so the means over seeds are compared at 5 %."""
    from graphtsetlinmachine_b200 import datasets

    protos = datasets.image_prototypes(1)
    train, y = datasets.vanilla_images(1500, 2, protos)
    test, y_test = datasets.vanilla_images(1000, 3, protos, init_with=train)
    Y = encode_labels(y, 10, 3125)
    stats = {"engine": [], "reference": []}
    for seed in range(1, 5):
        kw = dict(clauses=2500, classes=10, literals=256, threshold=3125, s=10.0, depth=1, max_nodes=1, seed=seed)
        for name, tm in (("engine", EngineTM(**kw)), ("reference", _reference(kw))):
            tm.set_graphs(train)
            tm.prepare()
            for _ in range(2):
                tm.fit(Y)
            if name == "reference":
                tm.download()
            tm.set_graphs(test)
            stats[name].append((float((tm.score().argmax(axis=1) == y_test).mean()), _included(tm.ta_state),
                                float(np.abs(tm.clause_weights).mean())))
            tm.close()
    a, b = np.array(stats["engine"]).mean(axis=0), np.array(stats["reference"]).mean(axis=0)
    print("vanilla images after 2 passes (accuracy, included literals, mean |weight|): engine", a, "reference kernels", b)
    assert abs(a[0] - b[0]) <= 0.03
    assert abs(a[1] - b[1]) <= 0.05 * b[1]
    assert abs(a[2] - b[2]) <= 0.03 * b[2]


def test_noisy_xor_learning_is_statistically_equivalent():
    """Ten clauses either find XOR or stay stuck, seed by seed, for both learners alike: the mean accuracy over seeds
    agrees within the sampling noise of that bimodal outcome, and both find XOR for some seed."""
    from graphtsetlinmachine_b200 import datasets

    train, y_train = datasets.noisy_xor(2000, seed=11)
    test, y_test = datasets.noisy_xor(1000, seed=12, noise=0.0, init_with=train)
    rng = np.random.default_rng(4)
    hv = rng.integers(0, 256, size=(10, 2)).astype(np.uint32)
    kw = dict(clauses=10, classes=2, literals=64, threshold=100, s=1.0, depth=2, message_size=256, message_bits=2,
              max_included=4, max_nodes=2, hypervectors=hv)
    Y = encode_labels(y_train, 2, 100)
    accuracies = {"engine": [], "reference": []}
    for seed in range(1, 13):
        engine = EngineTM(seed=seed, **kw)
        ref = _reference(dict(kw, seed=seed))
        for name, tm in (("engine", engine), ("reference", ref)):
            tm.set_graphs(train)
            tm.prepare()
            for _ in range(10):
                tm.fit(Y)
            tm.set_graphs(test)
            accuracies[name].append(float((tm.score().argmax(axis=1) == y_test).mean()))
            tm.close()
    a, b = np.array(accuracies["engine"]), np.array(accuracies["reference"])
    print("noisy XOR accuracy: engine", a, "reference kernels", b)
    assert a.max() >= 0.99 and b.max() >= 0.99
    assert abs(a.mean() - b.mean()) <= 0.25


def _benchmark_shape(name):
    """(model kwargs, training graphs, labels, test graphs, passes) at the model sizes of the benchmark configurations."""
    from graphtsetlinmachine_b200 import datasets
    from util import random_graphs

    np.random.seed(5)
    if name == "convolution_images":
        protos = datasets.image_prototypes(1)
        train, y = datasets.convolution_images(60, 2, protos)
        test, _ = datasets.convolution_images(40, 3, protos, init_with=train)
        kw = dict(clauses=2500, classes=10, literals=256, threshold=3125, s=10.0, depth=1, max_nodes=361)
    elif name == "sequences":
        train, y = datasets.sequences(12, 2)
        test, _ = datasets.sequences(8, 3, init_with=train)
        kw = dict(clauses=2000, classes=2, literals=512, threshold=2000, s=5.0, depth=3, message_size=512, message_bits=2,
                  max_nodes=1000)
    elif name == "multigraphs":
        train, y = datasets.random_multigraphs(40, 2, min_nodes=8, max_nodes=32)
        test, _ = datasets.random_multigraphs(30, 3, init_with=train)
        kw = dict(clauses=20000, classes=10, literals=2048, threshold=10000, s=10.0, depth=3, message_size=1024,
                  message_bits=2, max_nodes=32)
    else:                                               # 33..1,024 nodes: the transposed evaluation of the general kernels
        rng = np.random.default_rng(17)
        train = random_graphs(30, rng, hv_size=64, max_nodes=200, node_types=2, edge_types=3, max_degree=3)
        test = random_graphs(24, rng, max_nodes=200, node_types=2, edge_types=3, max_degree=3, init_with=train)
        y = rng.integers(0, 3, size=30)
        kw = dict(clauses=300, classes=3, literals=128, threshold=150, s=3.0, depth=3, message_size=128, message_bits=2,
                  max_nodes=200)
    rng = np.random.default_rng(9)
    hv = np.stack([rng.choice(kw.get("message_size", 256), size=2, replace=False) for _ in range(kw["clauses"])]).astype(np.uint32)
    return dict(kw, hypervectors=hv, seed=13), train, y, test


@pytest.mark.parametrize("name", ["convolution_images", "sequences", "multigraphs", "mid_graphs"])
def test_benchmark_shapes_match_reference_kernels_on_the_gpu(name):
    """Benchmark configurations 3, 4 and 5 and a 33..1,024-node shape: after three learning passes the engine's class
    sums (every scoring kernel that serves the shape), node outputs per layer, messages and include counts equal what
    the reference's own kernels compute on the same GPU from the same state."""
    kw, train, y, test = _benchmark_shape(name)
    engine = EngineTM(**kw)
    engine.set_graphs(train)
    engine.prepare()
    engine.fit(encode_labels(y, kw["classes"], kw["threshold"]), epochs=3)
    ref = _reference(kw)
    ref.load_from(engine)
    ref.set_graphs(test)
    engine.set_graphs(test)
    want = ref.score()
    assert np.abs(want).sum() > 0
    np.testing.assert_array_equal(engine.score(), want, err_msg="automatic scoring kernel")
    np.testing.assert_array_equal(engine.transform()[1], want, err_msg="general scoring kernel")
    for e in range(0, test.number_of_graphs, max(1, test.number_of_graphs // 4)):
        a = ref.evaluate_graph(e)
        for path in (0, 1):
            b = engine.evaluate_graph(e, path=path)
            np.testing.assert_array_equal(a["cno"], b["cno"], err_msg="node outputs, graph %d path %d" % (e, path))
            for d in range(kw["depth"] - 1):
                np.testing.assert_array_equal(a["messages"][d], b["messages"][d], err_msg="messages, graph %d layer %d" % (e, d))
            np.testing.assert_array_equal(a["n_inc"], b["n_inc"])
            np.testing.assert_array_equal(a["class_sum"], b["class_sum"])
    if kw["max_nodes"] <= 128:
        tile = EngineTM(**kw, options={"score_kernel": 3})
        tile.set_graphs(test)
        for d in range(kw["depth"]):
            tile.set_ta(d, engine.get_ta(d))
        tile.set_weights(engine.clause_weights)
        np.testing.assert_array_equal(tile.score(), want, err_msg="tile scoring kernel")
        tile.close()
    engine.close()
    ref.close()


def _accuracy_runs(kw, train, Y, test, y_test, seeds, epochs):
    """Test accuracy after `epochs` passes for every seed, engine and reference kernels (same data, same hypervectors)."""
    acc = {"engine": [], "reference": []}
    for seed in seeds:
        for name, tm in (("engine", EngineTM(seed=seed, **kw)), ("reference", _reference(dict(kw, seed=seed)))):
            tm.set_graphs(train)
            tm.prepare()
            for _ in range(epochs):
                tm.fit(Y)
            tm.set_graphs(test)
            acc[name].append(float((tm.score().argmax(axis=1) == y_test).mean()))
            tm.close()
    return np.array(acc["engine"]), np.array(acc["reference"])


def _assert_same_accuracy(a, b, what):
    """|difference of the mean accuracies| <= 0.5 percentage points, or within two standard errors of the difference
    when the seed-to-seed spread is larger than that."""
    diff = abs(a.mean() - b.mean())
    se = float(np.sqrt(a.var(ddof=1) / len(a) + b.var(ddof=1) / len(b)))
    print("%s: engine %.4f +- %.4f, reference kernels %.4f +- %.4f (n = %d each), |diff| %.4f, s.e. %.4f"
          % (what, a.mean(), a.std(ddof=1), b.mean(), b.std(ddof=1), len(a), diff, se))
    assert diff <= max(0.005, 2.0 * se), what


def test_accuracy_after_training_matches_reference_kernels():
    """End-to-end accuracy, engine (Philox streams) against the reference's kernels on the same GPU (XORWOW states),
    the MNIST-shaped configuration after five passes over 10,000 graphs (sixteen seeds per learner), and Noisy XOR at
    s = 2.0 (where the task is learned reliably) after ten passes."""
    from graphtsetlinmachine_b200 import datasets

    protos = datasets.image_prototypes(1)
    np.random.seed(2)
    train, y = datasets.vanilla_images(10000, 2, protos)
    test, y_test = datasets.vanilla_images(4000, 3, protos, init_with=train)
    kw = dict(clauses=2500, classes=10, literals=256, threshold=3125, s=10.0, depth=1, max_nodes=1)
    a, b = _accuracy_runs(kw, train, encode_labels(y, 10, 3125), test, y_test, range(1, 17), 5)
    _assert_same_accuracy(a, b, "vanilla images")

    np.random.seed(3)
    train, y = datasets.noisy_xor(4000, 11)
    test, y_test = datasets.noisy_xor(2000, 12, noise=0.0, init_with=train)
    rng = np.random.default_rng(4)
    hv = np.stack([rng.choice(256, size=2, replace=False) for _ in range(10)]).astype(np.uint32)
    kw = dict(clauses=10, classes=2, literals=64, threshold=100, s=2.0, depth=2, message_size=256, message_bits=2,
              max_included=4, max_nodes=2, hypervectors=hv)
    a, b = _accuracy_runs(kw, train, encode_labels(y, 2, 100), test, y_test, range(1, 9), 10)
    _assert_same_accuracy(a, b, "noisy XOR, s = 2.0")
