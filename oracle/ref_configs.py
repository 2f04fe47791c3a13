"""TEST INFRASTRUCTURE ONLY.  Hyper-parameter sets for which ``oracle/build_ref.py`` builds the host version of the
reference kernels ahead of time (the reference specialises its kernels by preprocessor constants, so each set is
its own shared object).  The GPU box has no reference checkout; these prebuilt objects travel with the tree."""

# keys follow oracle/build_ref.py:PARAM_ORDER; anything omitted takes the reference's default
CONFIGS = {
    # the Noisy XOR demo (examples/NoisyXORDemo.py defaults)
    "noisy_xor": dict(classes=2, clauses=10, literals=64, threshold=100, max_included=4, max_nodes=2,
                      message_size=256, message_bits=2),
    # MNIST-shaped single-node graphs: the benchmark workload
    "vanilla_images": dict(classes=10, clauses=2500, literals=256, threshold=3125, max_nodes=1),
    # the other benchmark configurations: convolution-shaped images (361 nodes), sequences (1,000-node paths, depth 3),
    # random multigraphs (8..32 nodes, depth 3, 20,000 clauses)
    "convolution_images": dict(classes=10, clauses=2500, literals=256, threshold=3125, max_nodes=361),
    "sequences": dict(classes=2, clauses=2000, literals=512, threshold=2000, max_nodes=1000, message_size=512, message_bits=2),
    "multigraphs": dict(classes=10, clauses=20000, literals=2048, threshold=10000, max_nodes=32, message_size=1024,
                        message_bits=2),
    # a 33..1,024-node shape for the transposed evaluation (tests/test_gpu_reference_kernels.py)
    "mid_graphs": dict(classes=3, clauses=300, literals=128, threshold=150, max_nodes=200, message_size=128, message_bits=2),
    # a single-output model (GraphTsetlinMachine class, tests/test_gpu_api.py)
    "single_output": dict(classes=1, clauses=20, literals=64, threshold=20, max_nodes=5, message_size=64, message_bits=2),
    # small differential-test sets (tests/cases.py)
    "case_a": dict(classes=2, clauses=20, literals=64, threshold=20, max_nodes=5, message_size=64, message_bits=2),
    "case_b": dict(classes=3, clauses=33, literals=80, threshold=30, max_nodes=40, message_size=50, message_bits=2,
                   boost=0, max_included=6),
    "case_c": dict(classes=4, clauses=16, literals=32, threshold=15, max_nodes=70, message_size=37, message_bits=1,
                   state_bits=6, q=0.5),
    "case_d": dict(classes=5, clauses=50, literals=128, threshold=40, max_nodes=3, message_size=128, message_bits=3),
    "case_e": dict(classes=2, clauses=24, literals=42, threshold=10, max_nodes=9, message_size=33, message_bits=2,
                   max_included=3),
}

# sets that are also built for the GPU (the reference's kernels on the same B200, launched like the reference does)
GPU_CONFIGS = ("noisy_xor", "vanilla_images", "convolution_images", "sequences", "multigraphs", "mid_graphs", "case_b", "case_e")
