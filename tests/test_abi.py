"""CPU suite, part 3: the C-ABI library loads without a GPU and exports every symbol include/gtm_b200.h declares;
argument checks that need no device; the Python binding covers every declaration."""

import ctypes as C
import os
import re

import numpy as np

from graphtsetlinmachine_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "gtm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gtm_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    build.build()
    lib = C.CDLL(build.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), name


def test_binding_covers_header():
    bound = set(_lib.PROTOTYPES) | {"gtm_last_error", "gtm_version"}
    assert set(declared_functions()) == bound


def test_struct_layouts():
    assert C.sizeof(_lib.Config) == 12 * 4 + 8 + 16 * 4 + 8
    assert C.sizeof(_lib.GraphsView) == 7 * 8 + 3 * 8 + 2 * 4


def test_argument_errors_without_device():
    lib = _lib.load()
    assert lib.gtm_version().startswith(b"gtm_b200")
    assert lib.gtm_create(None, None) == 1
    assert b"null" in lib.gtm_last_error()
    out = C.c_void_p()
    cfg = _lib.Config()
    assert lib.gtm_create(C.byref(cfg), C.byref(out)) == 1      # zero clauses
    assert lib.gtm_init_state(None, 1) == 1
    assert lib.gtm_score(None, None, 1, 0, 0, None) == 1
    assert lib.gtm_destroy(None) == 0 and lib.gtm_dataset_destroy(None) == 0
