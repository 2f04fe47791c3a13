"""ctypes binding of ``libgtm_b200.so`` (declarations of ``include/gtm_b200.h``).

There is no fallback: when the shared object is missing or cannot be loaded, importing the engine fails with
an error that says how to build it.
"""

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("GTM_B200_LIB", os.path.join(HERE, "libgtm_b200.so"))   # override: an alternative build of the library

GTM_MAX_DEPTH = 16
STATUS = {0: "GTM_OK", 1: "GTM_ERR_ARG", 2: "GTM_ERR_CUDA", 3: "GTM_ERR_OOM", 4: "GTM_ERR_TIMEOUT", 5: "GTM_ERR_STATE"}


class GtmError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("%s: %s" % (STATUS.get(status, status), message))
        self.status = status


class Config(C.Structure):
    _fields_ = [
        ("number_of_clauses", C.c_int32), ("number_of_outputs", C.c_int32), ("number_of_literals", C.c_int32),
        ("number_of_state_bits", C.c_int32), ("boost_true_positive_feedback", C.c_int32), ("T", C.c_int32),
        ("max_included_literals", C.c_int32), ("message_size", C.c_int32), ("message_bits", C.c_int32),
        ("depth", C.c_int32), ("device", C.c_int32), ("reserved", C.c_int32),
        ("q", C.c_double), ("s", C.c_float * GTM_MAX_DEPTH), ("seed", C.c_uint64),
    ]


class GraphsView(C.Structure):
    _fields_ = [
        ("X", C.c_void_p), ("node_type", C.c_void_p), ("number_of_graph_node_edges", C.c_void_p),
        ("edge_index", C.c_void_p), ("edge", C.c_void_p), ("node_index", C.c_void_p),
        ("number_of_graph_nodes", C.c_void_p),
        ("number_of_graphs", C.c_int64), ("total_nodes", C.c_int64), ("total_edges", C.c_int64),
        ("max_number_of_graph_nodes", C.c_int32), ("reserved", C.c_int32),
    ]


# name -> argument types (every function returns int status except the two string getters)
PROTOTYPES = {
    "gtm_device_count": [C.POINTER(C.c_int)],
    "gtm_create": [C.POINTER(Config), C.POINTER(C.c_void_p)],
    "gtm_destroy": [C.c_void_p],
    "gtm_set_stream": [C.c_void_p, C.c_void_p],
    "gtm_set_option": [C.c_void_p, C.c_char_p, C.c_int],
    "gtm_init_state": [C.c_void_p, C.c_int],
    "gtm_set_ta_state": [C.c_void_p, C.c_int, C.c_void_p],
    "gtm_get_ta_state": [C.c_void_p, C.c_int, C.c_void_p],
    "gtm_set_weights": [C.c_void_p, C.c_void_p],
    "gtm_get_weights": [C.c_void_p, C.c_void_p],
    "gtm_set_hypervectors": [C.c_void_p, C.c_void_p],
    "gtm_set_draw_positions": [C.c_void_p, C.c_void_p],
    "gtm_get_draw_positions": [C.c_void_p, C.c_void_p],
    "gtm_set_recorded_draws": [C.c_void_p, C.c_void_p, C.c_uint64],
    "gtm_dataset_create": [C.c_void_p, C.POINTER(GraphsView), C.POINTER(C.c_void_p)],
    "gtm_validate_graphs": [C.POINTER(GraphsView)],
    "gtm_dataset_destroy": [C.c_void_p],
    "gtm_score": [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p],
    "gtm_score_device": [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p],
    "gtm_score_static_scratch": [C.c_void_p, C.POINTER(GraphsView), C.c_int, C.c_int64, C.c_int64, C.c_void_p],
    "gtm_check_skipped_graphs": [C.c_void_p, C.POINTER(C.c_int)],
    "gtm_shard_range": [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)],
    "gtm_shard_prepare": [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p],
    "gtm_shard_connect": [C.c_void_p, C.c_void_p, C.c_void_p],
    "gtm_fit": [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_int],
    "gtm_transform": [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p],
    "gtm_transform_nodewise": [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p],
    "gtm_debug_evaluate": [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_void_p, C.c_void_p,
                           C.c_void_p, C.c_void_p],
    "gtm_debug_last_feedback": [C.c_void_p, C.c_void_p, C.c_void_p],
    "gtm_debug_fit_phase_cycles": [C.c_void_p, C.c_void_p],
    "gtm_debug_logic_op_rate": [C.c_void_p, C.POINTER(C.c_double)],
    "gtm_dataset_create_scored": [C.c_void_p, C.POINTER(GraphsView), C.c_int, C.c_void_p, C.POINTER(C.c_void_p)],
}

_lib = None


def load():
    """Load the shared object (once) and declare every prototype.  Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.isfile(LIB_PATH):
        raise ImportError(
            "libgtm_b200.so is not built (%s). Build it with `python -m graphtsetlinmachine_b200.build` "
            "(needs nvcc); this engine has no CPU or PyTorch fallback." % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, argtypes in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = C.c_int
    lib.gtm_last_error.restype = C.c_char_p
    lib.gtm_last_error.argtypes = []
    lib.gtm_version.restype = C.c_char_p
    lib.gtm_version.argtypes = []
    _lib = lib
    return lib


def check(status):
    if status != 0:
        raise GtmError(status, load().gtm_last_error().decode("utf-8", "replace"))
