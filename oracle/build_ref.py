"""TEST INFRASTRUCTURE ONLY (checker, never the product path).

Builds ``oracle/_ref/ref_<key>.so``: the reference's own CUDA kernel source, compiled for the HOST.

The kernel strings are read from the reference checkout's ``GraphTsetlinMachine/kernels.py`` at build time
(never copied into this repository), prefixed with the ``#define`` block that the reference's host code
formats at JIT time (``GraphTsetlinMachine/tm.py:438-464``), and compiled with ``g++`` against
``oracle/ref_shim.h`` (CUDA execution-model stand-in + counter-based ``curandState``) and
``oracle/ref_driver.inc`` (launchers + the per-graph launch order of ``tm.py``).  The only edit made to the
reference text is the replacement of its ``#include <curand_kernel.h>`` line by the shim include.

Because the reference specialises its kernels by preprocessor constants, one shared object is built per
hyper-parameter set; ``config_key`` names it.  The intermediate translation unit is deleted after compiling.

The reference checkout is looked up in ``$GTM_REFERENCE``, ``baseline/_ref`` and a directory ``reference`` beside the
repository; when none
is present (e.g. on a GPU box) only shared objects built earlier can be used.
"""

import hashlib
import importlib.util
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")

PARAM_ORDER = (
    "classes", "clauses", "literals", "state_bits", "boost", "threshold", "q", "max_included",
    "negative_clauses", "max_nodes", "message_size", "message_bits",
)


# a checkout named `reference` beside the repository directory (where the build machine keeps its read-only copy)
SIBLING_REFERENCE = os.path.normpath(os.path.join(HERE, "..", "..", "reference"))


def find_reference():
    """Path of the reference's kernels.py, or None."""
    roots = [os.environ.get("GTM_REFERENCE"), os.path.join(HERE, "..", "baseline", "_ref"), SIBLING_REFERENCE]
    for root in roots:
        if not root:
            continue
        path = os.path.join(root, "GraphTsetlinMachine", "kernels.py")
        if os.path.isfile(path):
            return path
    return None


def normalise(params):
    p = dict(params)
    p.setdefault("state_bits", 8)
    p.setdefault("boost", 1)
    p.setdefault("q", 1.0)
    p.setdefault("negative_clauses", 1)
    p.setdefault("message_size", 256)
    p.setdefault("message_bits", 2)
    if p.get("max_included") is None:
        p["max_included"] = p["literals"]
    p["q"] = float(p["q"])
    for k in PARAM_ORDER:
        if k != "q":
            p[k] = int(p[k])
    return {k: p[k] for k in PARAM_ORDER}


def config_key(params):
    p = normalise(params)
    text = ";".join("%s=%s" % (k, ("%f" % p[k]) if k == "q" else p[k]) for k in PARAM_ORDER)
    return hashlib.sha1(text.encode()).hexdigest()[:16]


def so_path(params):
    return os.path.join(REF_DIR, "ref_%s.so" % config_key(params))


def _defines(p):
    # same names, order and formatting as the block formatted at tm.py:438-464
    return (
        "#define CLASSES %d\n#define CLAUSES %d\n#define LITERALS %d\n#define STATE_BITS %d\n"
        "#define BOOST_TRUE_POSITIVE_FEEDBACK %d\n#define THRESHOLD %d\n#define Q %f\n"
        "#define MAX_INCLUDED_LITERALS %d\n#define NEGATIVE_CLAUSES %d\n#define MAX_NODES %d\n"
        "#define MESSAGE_SIZE %d\n#define MESSAGE_BITS %d\n"
        % (p["classes"], p["clauses"], p["literals"], p["state_bits"], p["boost"], p["threshold"], p["q"],
           p["max_included"], p["negative_clauses"], p["max_nodes"], p["message_size"], p["message_bits"])
    )


def build(params, force=False, quiet=True):
    """Compile (if needed) and return the path of the shared object for ``params``; None if the reference
    checkout is absent and nothing was built earlier."""
    p = normalise(params)
    out = so_path(p)
    if os.path.isfile(out) and not force:
        return out
    kernels_py = find_reference()
    if kernels_py is None:
        return None
    spec = importlib.util.spec_from_file_location("_gtm_reference_kernels", kernels_py)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    header = mod.code_header.replace("#include <curand_kernel.h>", '#include "ref_shim.h"')
    if '#include "ref_shim.h"' not in header:
        raise RuntimeError("reference header no longer includes curand_kernel.h; shim include not placed")
    unit = (
        _defines(p) + header + mod.code_update + mod.code_evaluate + mod.code_prepare
        + mod.code_transform + mod.code_clauses + '\n#include "ref_driver.inc"\n'
    )
    os.makedirs(REF_DIR, exist_ok=True)
    with tempfile.NamedTemporaryFile("w", suffix=".cpp", dir=REF_DIR, delete=False) as f:
        f.write(unit)
        src = f.name
    try:
        cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-w", "-I", HERE, src, "-o", out + ".tmp"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("reference kernels failed to compile:\n" + res.stderr[-4000:])
        os.replace(out + ".tmp", out)
    finally:
        os.unlink(src)
    if not quiet:
        print("built", out)
    return out


def gpu_so_path(params):
    return os.path.join(REF_DIR, "refgpu_%s.so" % config_key(params))


def build_gpu(params, force=False, quiet=True):
    """The reference's kernel strings compiled with nvcc for sm_100a (its own `#include <curand_kernel.h>` stays) plus
    ``oracle/ref_gpu_driver.inc``; returns the path or None when the checkout is absent and nothing was built earlier."""
    p = normalise(params)
    out = gpu_so_path(p)
    if os.path.isfile(out) and not force:
        return out
    kernels_py = find_reference()
    if kernels_py is None:
        return None
    spec = importlib.util.spec_from_file_location("_gtm_reference_kernels", kernels_py)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    unit = (
        _defines(p) + mod.code_header + mod.code_update + mod.code_evaluate + mod.code_prepare
        + mod.code_transform + mod.code_clauses + '\n#include "ref_gpu_driver.inc"\n'
    )
    os.makedirs(REF_DIR, exist_ok=True)
    with tempfile.NamedTemporaryFile("w", suffix=".cu", dir=REF_DIR, delete=False) as f:
        f.write(unit)
        src = f.name
    try:
        cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-shared", "-Xcompiler", "-fPIC", "-w",
               "-I", HERE, src, "-o", out + ".tmp"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("reference kernels failed to compile for the GPU:\n" + res.stderr[-4000:])
        os.replace(out + ".tmp", out)
    finally:
        os.unlink(src)
    if not quiet:
        print("built", out)
    return out


if __name__ == "__main__":
    sys.path.insert(0, HERE)
    from ref_configs import CONFIGS, GPU_CONFIGS  # noqa: E402

    missing = 0
    for name, params in CONFIGS.items():
        path = build(params, force="--force" in sys.argv, quiet=False)
        if path is not None and name in GPU_CONFIGS:
            build_gpu(params, force="--force" in sys.argv, quiet=False)
        if path is None:
            print("reference checkout not found; cannot build", name)
            missing += 1
    sys.exit(1 if missing else 0)
