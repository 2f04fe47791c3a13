"""Generates the golden vectors of this folder.  Needs the reference checkout (``$GTM_REFERENCE``, or the
default location known to oracle/build_ref.py); run as ``python tests/golden/make_golden.py`` from the repository root.

Two kinds of vectors, both produced by the reference's own code:
 * ``graphs_*.npz``   arrays built by the reference's ``Graphs`` class (GraphTsetlinMachine/graphs.py, imported
                      from the checkout) for a seeded sequence of builder calls;
 * ``case_*.npz``     the state of the reference's kernels (compiled for the host by oracle/build_ref.py) after
                      every training epoch of the cases in tests/cases.py, plus scores and, for a few graphs, the
                      per-layer node outputs, packed messages, include counts and class sums.
The inputs are regenerated from seeds by tests/cases.py, so only outputs are stored.
"""

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]

from cases import CASES, make_case  # noqa: E402
from oracle.ref_tm import RefTM  # noqa: E402


def reference_graphs_class():
    import importlib.util

    from oracle import build_ref

    ref_root = os.environ.get("GTM_REFERENCE", build_ref.DEFAULT_REFERENCE)
    spec = importlib.util.spec_from_file_location("_ref_graphs", os.path.join(ref_root, "GraphTsetlinMachine", "graphs.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.Graphs


def scripted_build(Graphs, seed, **ctor):
    """A fixed, seeded sequence of builder calls (several node/edge types, multi-edges, repeated properties)."""
    import random

    rnd = random.Random(seed)
    np.random.seed(seed)
    symbols = ["sym%d" % i for i in range(9)]
    g = Graphs(7, symbols=symbols, **ctor)
    sizes = [rnd.randint(1, 6) for _ in range(7)]
    for i, n in enumerate(sizes):
        g.set_number_of_graph_nodes(i, n)
    g.prepare_node_configuration()
    degs = []
    for i, n in enumerate(sizes):
        d = [rnd.randint(0, 3) for _ in range(n)]
        degs.append(d)
        for v in range(n):
            g.add_graph_node(i, "n%d" % v, d[v], rnd.choice(["Plain", "Other", "Third"]))
    g.prepare_edge_configuration()
    for i, n in enumerate(sizes):
        for v in range(n):
            for _ in range(degs[i][v]):
                g.add_graph_node_edge(i, "n%d" % v, "n%d" % rnd.randrange(n), rnd.choice(["a", "b", "c"]))
            for _ in range(rnd.randint(0, 4)):
                g.add_graph_node_property(i, "n%d" % v, rnd.choice(symbols))
    g.encode()
    test = Graphs(2, init_with=g)
    test.set_number_of_graph_nodes(0, 2)
    test.set_number_of_graph_nodes(1, 1)
    test.prepare_node_configuration()
    test.add_graph_node(0, "x", 1)
    test.add_graph_node(0, "y", 0, "Other")
    test.add_graph_node(1, "z", 0)
    test.prepare_edge_configuration()
    test.add_graph_node_edge(0, "x", "y", "b")
    test.add_graph_node_property(0, "x", "sym3")
    test.add_graph_node_property(1, "z", "sym8")
    test.encode()
    return g, test


GRAPH_FIELDS = ["X", "node_type", "number_of_graph_node_edges", "edge_index", "edge", "node_index",
                "number_of_graph_nodes", "hypervectors"]
GRAPH_VARIANTS = {"plain": dict(hypervector_size=48, hypervector_bits=3), "odd": dict(hypervector_size=21, hypervector_bits=2),
                  "onehot": dict(one_hot_encoding=True), "dhash": dict(hypervector_size=64, double_hashing=True)}


def main():
    RefGraphs = reference_graphs_class()
    for name, ctor in GRAPH_VARIANTS.items():
        g, t = scripted_build(RefGraphs, 11, **ctor)
        out = {}
        for f in GRAPH_FIELDS:
            out["train_" + f] = getattr(g, f)
            out["test_" + f] = getattr(t, f)
        out["train_signature"] = np.frombuffer(g.signature, dtype=np.uint8)
        out["test_signature"] = np.frombuffer(t.signature, dtype=np.uint8)
        sub = g[[5, 1, -1]]
        for f in GRAPH_FIELDS[:-1]:
            out["subset_" + f] = getattr(sub, f)
        np.savez_compressed(os.path.join(HERE, "graphs_%s.npz" % name), **out)

    for name in CASES:
        kw, graphs, encY, epochs = make_case(name)
        ref = RefTM(**kw)
        ref.set_graphs(graphs)
        ref.prepare()
        out = {"init_weights": ref.clause_weights.copy()}
        for ep in range(epochs):
            ref.fit(encY)
            out["ta_%d" % ep] = ref.ta_state.copy()
            for d, m in enumerate(ref.message_ta_state):
                out["mta%d_%d" % (d, ep)] = m.copy()
            out["weights_%d" % ep] = ref.clause_weights.copy()
            out["draws_%d" % ep] = ref.draws_consumed()
            out["clause_node_%d" % ep] = ref.clause_node.copy()
            out["update_%d" % ep] = ref.class_clause_update.copy()
            out["scores_%d" % ep] = ref.score()
        for e in range(8):
            r = ref.evaluate_graph(e)
            words = (int(graphs.number_of_graph_nodes[e]) - 1) // 32 + 1
            out["g%d_cno" % e] = r["cno"][:, :, :words]
            for d, m in enumerate(r["messages"]):
                out["g%d_msg%d" % (e, d)] = m
            out["g%d_ninc" % e] = r["n_inc"]
            out["g%d_sum" % e] = r["class_sum"]
        np.savez_compressed(os.path.join(HERE, "%s.npz" % name), **out)
        print(name, "ok")


if __name__ == "__main__":
    main()
