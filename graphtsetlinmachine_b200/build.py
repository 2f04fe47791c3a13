"""Builds ``libgtm_b200.so`` (CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

``python -m graphtsetlinmachine_b200.build`` or ``build()``; the shared object lands next to this file so that
it travels with the source tree.  nvcc cross-compiles without a GPU.
"""

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libgtm_b200.so")
SOURCES = [os.path.join(HERE, "csrc", f) for f in ("gtm_api.cu", "gtm_fit_global.cu", "gtm_fit_resident.cu", "gtm_stream.cu", "gtm_tile.cu")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]


def _stale():
    if not os.path.isfile(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(HERE, "csrc", f) for f in os.listdir(os.path.join(HERE, "csrc"))]
    deps.append(os.path.join(HERE, "..", "include", "gtm_b200.h"))
    return any(os.path.getmtime(d) > built for d in deps if os.path.isfile(d))


def build(force=False, verbose=False):
    if not force and not _stale():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    # one object per translation unit, compiled side by side, then one link
    jobs = []
    for src in SOURCES:
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        jobs.append((obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
    log = ""
    for obj, proc in jobs:
        out, err = proc.communicate()
        log += err
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + out[-2000:] + err[-6000:])
    res = subprocess.run([nvcc, "-shared", "-o", LIB_PATH + ".tmp"] + [obj for obj, _ in jobs], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout[-2000:] + res.stderr[-6000:])
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    if verbose:
        print(log)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
