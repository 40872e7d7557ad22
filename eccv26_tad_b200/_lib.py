"""ctypes binding of ``libsvtad.so`` (declared in ``include/svtad.h``).

The library is the only implementation behind this package: if it is missing, importing this
module raises - there is no eager / CPU fallback.
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libsvtad.so")

OK, ERR_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA = 0, 1, 2, 3, 4
F32, BF16, F16 = 0, 1, 2
OP_FWD, OP_DGRAD, OP_WGRAD, OP_BWD = 0, 1, 2, 3
TABLE_OUT_OF_RANGE, TABLE_ASYMMETRIC = 1, 2

c_int, c_i64, c_p, c_sz = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/svtad.h one to one
SIGNATURES = {
    "svtad_version": (c_int, []),
    "svtad_last_error_string": (ctypes.c_char_p, []),
    "svtad_table_init": (c_int, [c_int, c_int, c_int, c_int, c_int, c_p, c_p]),
    "svtad_table_build": (c_int, [c_p, c_int, c_int, c_int, c_int, c_int, c_int, c_p, c_p, c_p]),
    "svtad_topk_select": (c_int, [c_p, c_int, c_int, c_int, c_p, c_p]),
    "svtad_table_remap": (c_int, [c_p, c_p, c_int, c_int, c_int, c_int, c_p, c_p, c_p]),
    "svtad_table_select_remap": (c_int, [c_p, c_p, c_int, c_int, c_int, c_int, c_p, c_p, c_p, c_p]),
    "svtad_table_check": (c_int, [c_p, c_i64, c_int, c_int, c_p, c_p]),
    "svtad_workspace_bytes": (c_sz, [c_int, c_i64, c_int, c_int, c_int, c_int]),
    "svtad_conv_fwd": (c_int, [c_p, c_p, c_p, c_p, c_p, c_i64, c_int, c_int, c_int, c_int, c_int, c_p, c_sz, c_p]),
    "svtad_conv_dgrad": (c_int, [c_p, c_p, c_p, c_p, c_i64, c_int, c_int, c_int, c_int, c_int, c_p, c_p, c_sz, c_p]),
    "svtad_conv_wgrad": (c_int, [c_p, c_p, c_p, c_p, c_p, c_i64, c_int, c_int, c_int, c_int, c_int, c_p, c_sz, c_p]),
    "svtad_conv_bwd": (c_int, [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i64, c_int, c_int, c_int, c_int, c_int, c_p, c_p, c_sz, c_p]),
    "svtad_static_workspace_bytes": (c_sz, []),
    "svtad_conv_wgrad_static": (c_int, [c_p, c_p, c_p, c_p, c_p, c_i64, c_int, c_int, c_int, c_int, c_int, c_p]),
    "svtad_allreduce_stage_bytes": (c_sz, [c_i64]),
    "svtad_allreduce_epoch_bytes": (c_sz, []),
    "svtad_allreduce_sum": (c_int, [ctypes.POINTER(c_p), c_int, c_int, c_i64, c_int, c_sz, c_p, c_i64, c_p]),
    "svtad_allreduce_sum_emulated": (c_int, [ctypes.POINTER(c_p), c_int, c_i64, c_int, c_sz, c_p, c_i64, c_p]),
    "svtad_ffma_probe": (c_int, [c_int, c_int, c_p, c_p]),
    "svtad_device_error": (c_int, [ctypes.POINTER(ctypes.c_int32)]),
    "svtad_set_concurrency": (c_int, [c_int]),
    "svtad_get_concurrency": (c_int, []),
    "svtad_path_for": (c_int, [c_int, c_i64, c_int, c_int, c_int, c_int]),
}

_lib = None


def load():
    """Loads the shared library once.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m eccv26_tad_b200.build` "
                "(there is no fallback implementation)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error():
    return load().svtad_last_error_string().decode("utf-8", "replace")


def check(rc):
    """Turns a status code into the exception the reference wrapper's callers expect."""
    if rc == OK:
        return
    msg = last_error()
    if rc in (ERR_ARG, ERR_UNSUPPORTED):
        raise ValueError(msg)
    raise RuntimeError(f"libsvtad error {rc}: {msg}")
