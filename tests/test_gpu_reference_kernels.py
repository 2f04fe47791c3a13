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
