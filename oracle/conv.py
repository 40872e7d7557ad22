"""ctypes front-end of the C conv oracle (``conv_oracle.c``).  TEST INFRASTRUCTURE ONLY.

All functions take and return numpy arrays.  ``acc="f64"`` is the ground truth (double
accumulate, double result); ``acc="f32"`` accumulates in float in the reference's
``(k, ci)`` order (opentad/models/bricks/2d_sparse_v3.cu:574-629) and is the flavour the
benchmark times as the CPU baseline.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libsvtad_oracle.so")
_lib = None


def build(force=False):
    src = os.path.join(_HERE, "conv_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE] + (["-B"] if force else []))
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        if _lib.svtad_oracle_version() < 3:      # an older build is lying around: rebuild and reload
            build(force=True)
            _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def set_threads(n):
    """Use n OpenMP threads in the timed (f32) functions; returns the count in effect."""
    lib().svtad_oracle_set_threads(int(n))
    return int(lib().svtad_oracle_get_threads())


def _f32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _acc(acc):
    return {"f32": np.float32, "f64": np.float64}[acc]


def fwd(x, nbr, w, bias=None, tokens_per_batch=0, acc="f64"):
    """``nbr`` may hold fewer rows than ``x`` (a sample of the table's rows, ``tokens_per_batch == 0`` only):
    the result then has one row per table row given."""
    x, w = _f32(x), _f32(w)
    nbr = np.ascontiguousarray(nbr, dtype=np.int32)
    n, cin = x.shape
    if nbr.shape[0] != n:
        assert tokens_per_batch == 0 and nbr.shape[0] < n, "a row sample needs global indices"
        n = nbr.shape[0]
    kk, _, cout = w.shape
    b = _f32(bias) if bias is not None else None
    y = np.empty((n, cout), dtype=_acc(acc))
    getattr(lib(), "svtad_oracle_fwd_" + acc)(
        _ptr(x), _ptr(nbr), _ptr(w), _ptr(b), _ptr(y),
        ctypes.c_int64(n), cin, cout, kk, int(tokens_per_batch))
    return y


def dgrad(gy, nbr, w, tokens_per_batch=0, acc="f64"):
    gy, w = _f32(gy), _f32(w)
    nbr = np.ascontiguousarray(nbr, dtype=np.int32)
    n, cout = gy.shape
    kk, cin, _ = w.shape
    gx = np.empty((n, cin), dtype=_acc(acc))
    getattr(lib(), "svtad_oracle_dgrad_" + acc)(
        _ptr(gy), _ptr(nbr), _ptr(w), _ptr(gx),
        ctypes.c_int64(n), cin, cout, kk, int(tokens_per_batch))
    return gx


def dgrad_rows(gy, nbr, w, rows, tokens_per_batch=0):
    """Rows ``rows`` of ``dgrad(gy, nbr, w)`` (float64), without computing the others."""
    gy, w = _f32(gy), _f32(w)
    nbr = np.ascontiguousarray(nbr, dtype=np.int32)
    sel = np.ascontiguousarray(rows, dtype=np.int64)
    n, cout = gy.shape
    kk, cin, _ = w.shape
    assert sel.size == 0 or (sel.min() >= 0 and sel.max() < n)
    assert len(np.unique(sel)) == sel.size
    gx = np.empty((sel.size, cin), dtype=np.float64)
    lib().svtad_oracle_dgrad_rows_f64(_ptr(gy), _ptr(nbr), _ptr(w), _ptr(gx), _ptr(sel), ctypes.c_int64(sel.size),
                                      ctypes.c_int64(n), cin, cout, kk, int(tokens_per_batch))
    return gx


def wgrad(gy, x, nbr, kk, tokens_per_batch=0, acc="f64", with_bias=True):
    gy, x = _f32(gy), _f32(x)
    nbr = np.ascontiguousarray(nbr, dtype=np.int32)
    n, cout = gy.shape
    cin = x.shape[1]
    gw = np.empty((kk, cin, cout), dtype=_acc(acc))
    gb = np.empty((cout,), dtype=_acc(acc)) if with_bias else None
    getattr(lib(), "svtad_oracle_wgrad_" + acc)(
        _ptr(gy), _ptr(x), _ptr(nbr), _ptr(gw), _ptr(gb),
        ctypes.c_int64(n), cin, cout, kk, int(tokens_per_batch))
    return gw, gb


def rel_err(a, ref):
    """The error metric of every parity test: max|a - ref| / max|ref| per tensor."""
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.abs(ref).max() if ref.size else 0.0
    num = np.abs(a - ref).max() if ref.size else 0.0
    return float(num / den) if den > 0 else float(num)
