"""Tensor-level entry points over the C ABI: raw device pointers in, status codes out.

These functions own what the C library does not: allocating outputs and workspaces through
torch's caching allocator (so they are ordered on the current stream), picking the current
stream and device, and translating status codes to exceptions.
"""
import torch
from torch.utils.weak import WeakIdKeyDictionary

from . import _lib

_DTYPES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


# Cheap equivalents of ``torch.cuda.current_stream().cuda_stream`` and ``torch.cuda.device(...)``: the
# public helpers cost tens of microseconds per call on the host, as much as the kernels they precede.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_get_device = getattr(torch._C, "_cuda_getDevice", None)
_exchange = getattr(torch.cuda, "_maybe_exchange_device", None)


def _stream():
    """Raw handle of the current stream of the current device."""
    if _raw_stream is not None and _get_device is not None:
        return _raw_stream(_get_device())
    return torch.cuda.current_stream().cuda_stream


class _on:
    """``with _on(tensor.device):`` makes that device current for the calls inside."""
    __slots__ = ("idx", "prev", "ctx")

    def __init__(self, device):
        self.idx = device.index
        self.ctx = None

    def __enter__(self):
        if _exchange is None or self.idx is None:
            self.ctx = torch.cuda.device(self.idx)
            self.ctx.__enter__()
        else:
            self.prev = _exchange(self.idx)

    def __exit__(self, *exc):
        if self.ctx is not None:
            return self.ctx.__exit__(*exc)
        _exchange(self.prev)
        return False


def _dtype_code(t):
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}; expected float32, bfloat16 or float16") from None


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("SparseConv2D tensors must live on a CUDA device (there is no CPU path)")


def _ptr(t):
    return t.data_ptr() if t is not None and t.numel() > 0 else None


def _c16(t):
    """Contiguous and 16-byte aligned (a contiguous slice of a larger tensor may start anywhere)."""
    t = t.contiguous()
    if t.numel() and t.data_ptr() % 16:
        t = t.clone()
    return t


def _i32_table(nbr):
    if nbr.dtype != torch.int32:
        nbr = nbr.to(torch.int32)
    return _c16(nbr)


def _check_shapes(who, n, kk, nbr, **feat):
    """The C library trusts its sizes; mismatched tensors are caught here."""
    if nbr.numel() != n * kk:
        raise ValueError(f"{who}: neighbor table has {nbr.numel()} entries, expected {n} rows x {kk} taps")
    for name, (t, cols) in feat.items():
        if t is not None and t.numel() != n * cols:
            raise ValueError(f"{who}: {name} has {t.numel()} elements, expected {n} x {cols}")


def _workspace(op, n, cin, cout, kk, code, device):
    nbytes = _lib.load().svtad_workspace_bytes(op, n, cin, cout, kk, code)
    if nbytes == 0:
        return None, 0
    return torch.empty(nbytes, dtype=torch.uint8, device=device), nbytes


# ----------------------------------------------------------------------------- table
# Tables this module built itself are symmetric by construction (entry (i, k) = j  <=>  entry (j, KK-1-k) = i):
# a full grid, a top-k subset of one, or a subset of a symmetric table.  They are remembered here (by tensor
# object and version, weakly) so that the backward can use the gather form of the input gradient without the
# device-side validation pass and without the scatter-form fallback launches.
_symmetric = WeakIdKeyDictionary()


def mark_symmetric(table):
    """Declare ``table`` symmetric (valid until the tensor is written to)."""
    _symmetric[table] = table._version
    return table


def is_known_symmetric(table):
    """True for tables built by this module (or marked by the caller) and views of them, unmodified since."""
    for t in (table, getattr(table, "_base", None)):
        if t is not None and _symmetric.get(t) == t._version:
            return True
    return False


def table_init(B, T, h, w, ksize=3, device="cuda"):
    out = torch.empty((B, T * h * w, ksize * ksize), dtype=torch.int32, device=device)
    with _on(out.device):
        _lib.check(_lib.load().svtad_table_init(B, T, h, w, ksize, _ptr(out), _stream()))
    return mark_symmetric(out)


def table_build(scores, k_keep, h, w, ksize=3):
    """scores float32 [n_seg, seg_len] -> (kept_idx int32 [n_seg, k], table int32 [n_seg*k, ksize^2])."""
    _require_cuda(scores)
    if scores.dtype != torch.float32:
        scores = scores.float()
    scores = scores.contiguous()
    n_seg, seg_len = scores.shape
    kept = torch.empty((n_seg, k_keep), dtype=torch.int32, device=scores.device)
    table = torch.empty((n_seg * k_keep, ksize * ksize), dtype=torch.int32, device=scores.device)
    with _on(scores.device):
        _lib.check(_lib.load().svtad_table_build(_ptr(scores), n_seg, seg_len, k_keep, h, w, ksize,
                                                 _ptr(kept), _ptr(table), _stream()))
    return kept, mark_symmetric(table)


def topk_select(scores, k_keep):
    """scores float32 [B, L] -> idx int64 [B, k], ascending (torch.topk + sort with a fixed tie rule)."""
    _require_cuda(scores)
    if scores.dtype != torch.float32:
        scores = scores.float()
    scores = scores.contiguous()
    B, L = scores.shape
    idx = torch.empty((B, k_keep), dtype=torch.int64, device=scores.device)
    with _on(scores.device):
        _lib.check(_lib.load().svtad_topk_select(_ptr(scores), B, L, k_keep, _ptr(idx), _stream()))
    return idx


def table_remap(table, idx, scratch=None):
    """table int32 [B, N_prev, KK], idx int64 [B, N_new] -> int32 [B, N_new, KK]."""
    _require_cuda(table, idx)
    sym = is_known_symmetric(table)
    table = _i32_table(table)
    idx = idx.to(torch.int64).contiguous()
    B, n_prev, kk = table.shape
    n_new = idx.shape[1]
    if scratch is None or scratch.numel() < B * n_prev:
        scratch = torch.empty(B * n_prev, dtype=torch.int32, device=table.device)
    out = torch.empty((B, n_new, kk), dtype=torch.int32, device=table.device)
    with _on(table.device):
        _lib.check(_lib.load().svtad_table_remap(_ptr(table), _ptr(idx), B, n_prev, n_new, kk,
                                                 _ptr(scratch), _ptr(out), _stream()))
    return mark_symmetric(out) if sym else out


def table_select_remap(scores, table, k_keep):
    """One later pruning round in one kernel: scores float32 [B, N_prev], table int32 [B, N_prev, KK] ->
    (idx int64 [B, k], table int32 [B, k, KK])."""
    _require_cuda(scores, table)
    if scores.dtype != torch.float32:
        scores = scores.float()
    scores = scores.contiguous()
    sym = is_known_symmetric(table)
    table = _i32_table(table)
    B, n_prev, kk = table.shape
    if tuple(scores.shape) != (B, n_prev):
        raise ValueError(f"table_select_remap: scores {tuple(scores.shape)} do not match the table's {(B, n_prev)}")
    kept = torch.empty((B, k_keep), dtype=torch.int32, device=table.device)
    idx = torch.empty((B, k_keep), dtype=torch.int64, device=table.device)
    out = torch.empty((B, k_keep, kk), dtype=torch.int32, device=table.device)
    with _on(table.device):
        _lib.check(_lib.load().svtad_table_select_remap(_ptr(scores), _ptr(table), B, n_prev, k_keep, kk, _ptr(kept),
                                                        _ptr(idx), _ptr(out), _stream()))
    return idx, (mark_symmetric(out) if sym else out)


def table_check(nbr, tokens_per_batch=0, status=None):
    """Returns a 1-element int32 device tensor: 0 = valid symmetric table (no host sync)."""
    _require_cuda(nbr)
    nbr = _i32_table(nbr)
    kk = nbr.shape[-1]
    n = nbr.numel() // kk
    if status is None:
        status = torch.empty(1, dtype=torch.int32, device=nbr.device)
    with _on(nbr.device):
        _lib.check(_lib.load().svtad_table_check(_ptr(nbr), n, kk, tokens_per_batch, _ptr(status), _stream()))
    return status


# ----------------------------------------------------------------------------- conv
def conv_fwd(x, nbr, weight, bias=None, tokens_per_batch=0):
    _require_cuda(x, nbr, weight, bias)
    code = _dtype_code(x)
    kk, cin, cout = weight.shape
    x = _c16(x)
    weight = _c16(weight)
    nbr = _i32_table(nbr)
    n = x.numel() // cin if cin else 0
    if weight.dtype != x.dtype or (bias is not None and bias.dtype != x.dtype):
        raise ValueError("x, weight and bias must share one dtype")
    _check_shapes("conv_fwd", n, kk, nbr)
    if bias is not None and bias.numel() != cout:
        raise ValueError(f"conv_fwd: bias has {bias.numel()} elements, expected {cout}")
    out = torch.empty((n, cout), dtype=x.dtype, device=x.device)
    with _on(x.device):
        _lib.check(_lib.load().svtad_conv_fwd(_ptr(x), _ptr(nbr), _ptr(weight),
                                              _ptr(_c16(bias)) if bias is not None else None,
                                              _ptr(out), n, cin, cout, kk, tokens_per_batch, code,
                                              None, 0, _stream()))
    return out


def conv_dgrad(gy, nbr, weight, tokens_per_batch=0, table_status=None, assume_symmetric=False):
    """table_status: tensor from table_check(); assume_symmetric=True skips the scatter-form launch."""
    _require_cuda(gy, nbr, weight)
    code = _dtype_code(gy)
    kk, cin, cout = weight.shape
    gy = _c16(gy)
    weight = _c16(weight)
    assume_symmetric = assume_symmetric or (table_status is None and is_known_symmetric(nbr))
    nbr = _i32_table(nbr)
    n = gy.numel() // cout
    if weight.dtype != gy.dtype:
        raise ValueError("grad_output and weight must share one dtype")
    _check_shapes("conv_dgrad", n, kk, nbr)
    gx = torch.empty((n, cin), dtype=gy.dtype, device=gy.device)
    with _on(gy.device):
        if assume_symmetric:
            status, ws, ws_bytes = None, None, 0
        else:
            status = table_status if table_status is not None else table_check(nbr, tokens_per_batch)
            ws, ws_bytes = _workspace(_lib.OP_DGRAD, n, cin, cout, kk, code, gy.device)
        _lib.check(_lib.load().svtad_conv_dgrad(_ptr(gy), _ptr(nbr), _ptr(weight), _ptr(gx), n, cin, cout,
                                                kk, tokens_per_batch, code, _ptr(status), _ptr(ws),
                                                ws_bytes, _stream()))
    return gx


def conv_wgrad(gy, x, nbr, kk, tokens_per_batch=0, with_bias=True):
    _require_cuda(gy, x, nbr)
    code = _dtype_code(x)
    cin = x.shape[-1]
    cout = gy.shape[-1]
    gy = _c16(gy)
    x = _c16(x)
    nbr = _i32_table(nbr)
    n = x.numel() // cin
    if gy.dtype != x.dtype:
        raise ValueError("grad_output and x must share one dtype")
    _check_shapes("conv_wgrad", n, kk, nbr, grad_output=(gy, cout))
    gw = torch.empty((kk, cin, cout), dtype=x.dtype, device=x.device)
    gb = torch.empty((cout,), dtype=x.dtype, device=x.device) if with_bias else None
    with _on(x.device):
        ws, ws_bytes = _workspace(_lib.OP_WGRAD, n, cin, cout, kk, code, x.device)
        _lib.check(_lib.load().svtad_conv_wgrad(_ptr(gy), _ptr(x), _ptr(nbr), _ptr(gw), _ptr(gb), n, cin,
                                                cout, kk, tokens_per_batch, code, _ptr(ws), ws_bytes,
                                                _stream()))
    return gw, gb


def conv_bwd(gy, x, nbr, weight, tokens_per_batch=0, table_status=None, need_x=True, need_w=True, need_b=True,
             assume_symmetric=False):
    """Both gradients of one layer in one library call (the weight gradient runs next to the input gradient
    on a stream of the library; for the caller everything is ordered on the current stream).
    ``assume_symmetric=True`` (or a table this module built itself) skips the device-side table validation and
    the scatter-form fallback of the input gradient.  Returns ``(gx, gw, gb)`` with None for what was not asked for."""
    _require_cuda(gy, x, nbr, weight)
    code = _dtype_code(gy)
    kk, cin, cout = weight.shape
    gy = _c16(gy)
    x = _c16(x)
    weight = _c16(weight)
    assume_symmetric = assume_symmetric or (table_status is None and is_known_symmetric(nbr))
    nbr = _i32_table(nbr)
    n = gy.numel() // cout
    if weight.dtype != gy.dtype or x.dtype != gy.dtype:
        raise ValueError("grad_output, x and weight must share one dtype")
    _check_shapes("conv_bwd", n, kk, nbr, x=(x, cin))
    need_w = need_w or need_b
    dev = gy.device
    gx = torch.empty((n, cin), dtype=gy.dtype, device=dev) if need_x else None
    gw = torch.empty((kk, cin, cout), dtype=gy.dtype, device=dev) if need_w else None
    gb = torch.empty((cout,), dtype=gy.dtype, device=dev) if need_b else None
    with _on(dev):
        if assume_symmetric:
            table_status = None
        elif need_x and table_status is None:
            table_status = table_check(nbr, tokens_per_batch)
        if assume_symmetric:     # no scatter-form part in the workspace
            op = _lib.OP_WGRAD if need_w else None
        else:
            op = _lib.OP_BWD if (need_x and need_w) else (_lib.OP_WGRAD if need_w else _lib.OP_DGRAD)
        ws, ws_bytes = _workspace(op, n, cin, cout, kk, code, dev) if op is not None else (None, 0)
        _lib.check(_lib.load().svtad_conv_bwd(_ptr(gy), _ptr(x), _ptr(nbr), _ptr(weight), _ptr(gx), _ptr(gw), _ptr(gb),
                                              n, cin, cout, kk, tokens_per_batch, code,
                                              _ptr(table_status) if (need_x and not assume_symmetric) else None,
                                              _ptr(ws), ws_bytes, _stream()))
    return gx, gw, gb


def conv_wgrad_static(gy, x, nbr, gw, gb, tokens_per_batch=0):
    """Weight / bias gradient into caller-provided ``gw`` / ``gb`` with the library's built-in workspace.

    For callers that must not allocate on the device once they are running (device memory owned by the
    host's own arena, allocation forbidden after start-up): nothing is allocated here, neither by the
    library nor by torch.  ``gb`` may be None.  Problems whose
    workspace exceeds the built-in array raise; calls that overlap on the GPU share the array and race.
    """
    _require_cuda(gy, x, nbr, gw, gb)
    code = _dtype_code(x)
    kk, cin, cout = gw.shape
    for t in (gy, x, nbr, gw) + ((gb,) if gb is not None else ()):
        if not t.is_contiguous():
            raise ValueError("conv_wgrad_static needs contiguous tensors (it cannot make copies)")
    if nbr.dtype != torch.int32 or gy.dtype != x.dtype or gw.dtype != x.dtype:
        raise ValueError("conv_wgrad_static: nbr must be int32 and gy, x, gw must share one dtype")
    n = x.numel() // cin
    _check_shapes("conv_wgrad_static", n, kk, nbr, x=(x, cin), grad_output=(gy, cout))
    if gb is not None and (gb.numel() != cout or gb.dtype != x.dtype):
        raise ValueError(f"conv_wgrad_static: gb must hold {cout} elements of x's dtype")
    for t in (gy, x, nbr, gw) + ((gb,) if gb is not None else ()):
        if t.numel() and t.data_ptr() % 16:
            raise ValueError("conv_wgrad_static needs 16-byte aligned tensors (it cannot make copies)")
    with _on(x.device):
        _lib.check(_lib.load().svtad_conv_wgrad_static(_ptr(gy), _ptr(x), _ptr(nbr), _ptr(gw), _ptr(gb), n, cin,
                                                       cout, kk, tokens_per_batch, code, _stream()))
    return gw, gb


def device_error():
    """Reads and clears the device error word (synchronises).  0 = no bounded wait gave up."""
    import ctypes
    v = ctypes.c_int32(0)
    _lib.check(_lib.load().svtad_device_error(ctypes.byref(v)))
    return v.value


def path_for(op, n, cin, cout, kk, dtype):
    return "tc" if _lib.load().svtad_path_for(op, n, cin, cout, kk, _DTYPES[dtype]) else "simt"


def set_concurrency(kernels):
    """How many of the library's kernels the caller expects to share the GPU at a time (independent layers on their
    own streams, forward next to backward).  1 (default) plans every kernel for the whole GPU - best for a kernel
    that runs alone; k > 1 plans for ``SMs / k``: fewer, longer CTAs that cost a lone kernel latency and save SM time
    under contention.  Process-wide; returns the previous value.  See ``svtad_set_concurrency`` in ``svtad.h``."""
    return int(_lib.load().svtad_set_concurrency(int(kernels)))


def get_concurrency():
    return int(_lib.load().svtad_get_concurrency())
