"""``SparseConv2d`` / ``SparseConv2dFunction`` with the reference's call surface.

Mirrors ``opentad/models/bricks/sparse_conv_layer.py`` of pcr-upm/eccv26_tad: same class names,
argument order, defaults, parameter names and shapes (``weight (K*K, C_in, C_out)``,
``bias (C_out)``), same autocast behaviour, same ``ValueError`` for ``C_in % 4 != 0``
(reference :39-42).  The implementation underneath is ``libsvtad.so`` only; a CPU tensor raises.

Differences, all additive:
* ``kernel_size`` (keyword-only, default 3) - the reference hard-codes 3x3 (:136, :182);
* ``chunk_size`` is accepted and ignored - the reference needs it to bound its ``[9, chunk, C]``
  temporaries (implicit_gemm_v2.cu:361-414); nothing is materialised here;
* the "indices are local to each batch row" heuristic (reference :170-177, a host sync on every
  call) is evaluated once per table object and cached, or skipped with ``local_indices=...``;
* parameters kept in another dtype than the activations (fp32 masters under bf16 autocast) are cast once per
  parameter version, not once per call (the reference casts on every forward, :196-203), and the backward is one
  library call with the weight gradient running next to the input gradient;
* checkpoints that hold the weight as ``(C_in, 9, C_out)`` are permuted on load (the reference does this in
  ``opentad/utils/checkpoint.py:44-57``; ``remap_legacy_sparse_conv_weights`` is provided too);
* the input gradient uses a gather form that needs a symmetric table (every table built by the
  backbone's code is).  Arbitrary tables are detected on the device by ``svtad_table_check`` and
  take the reference's scatter formulation, so results are defined for any table.
"""
import math

import torch
import torch.nn as nn
from torch.autograd import Function
from torch.utils.weak import WeakIdKeyDictionary

from . import ops

try:  # torch >= 2.4
    from torch.amp import custom_bwd as _custom_bwd, custom_fwd as _custom_fwd

    def custom_fwd(fn):
        return _custom_fwd(fn, device_type="cuda")

    def custom_bwd(fn):
        return _custom_bwd(fn, device_type="cuda")
except ImportError:  # pragma: no cover
    from torch.cuda.amp import custom_bwd, custom_fwd


class _PerTableCache:
    """Facts about a table tensor, valid while the tensor object lives and is not written to."""

    def __init__(self):
        self._d = WeakIdKeyDictionary()

    def get(self, t, key, make):
        ent = self._d.get(t)
        if ent is None or ent[0] != t._version:
            ent = (t._version, {})
            self._d[t] = ent
        if key not in ent[1]:
            ent[1][key] = make()
        return ent[1][key]


_table_cache = _PerTableCache()


_SYMMETRIC = "symmetric by construction"


def _status_for(nbr, tokens_per_batch):
    """What the backward needs to know about a table: ``_SYMMETRIC`` for tables built by this package (no
    validation pass, no scatter-form fallback), else the device status word of ``svtad_table_check``."""
    if tokens_per_batch == 0 and ops.is_known_symmetric(nbr):
        return _SYMMETRIC
    return _table_cache.get(nbr, ("status", tokens_per_batch), lambda: ops.table_check(nbr, tokens_per_batch))


def _bwd(grad_output, x, nbr, weight, tpb, status, need_x, need_w, need_b):
    if status is _SYMMETRIC:
        return ops.conv_bwd(grad_output, x, nbr, weight, tpb, need_x=need_x, need_w=need_w, need_b=need_b,
                            assume_symmetric=True)
    return ops.conv_bwd(grad_output, x, nbr, weight, tpb, table_status=status, need_x=need_x, need_w=need_w,
                        need_b=need_b)


class SparseConv2dFunction(Function):
    """apply(x, neighbor_indices, weight, bias=None, tokens_per_batch=0, chunk_size=0)
    (reference sparse_conv_layer.py:29-123)."""

    @staticmethod
    @custom_fwd
    def forward(ctx, x, neighbor_indices, weight, bias=None, tokens_per_batch=0, chunk_size=0):
        kk, C_in, C_out = weight.shape
        if C_in % 4 != 0:
            raise ValueError(f"C_in ({C_in}) must be divisible by 4 for optimized kernel.")
        ctx.save_for_backward(x, neighbor_indices, weight, bias)
        ctx.C_in = C_in
        ctx.tokens_per_batch = tokens_per_batch
        ctx.table_status = None
        if any(ctx.needs_input_grad[:1]):
            ctx.table_status = _status_for(neighbor_indices, tokens_per_batch)
        out = ops.conv_fwd(x.reshape(-1, C_in), neighbor_indices.reshape(-1, kk), weight, bias,
                           tokens_per_batch)
        return out

    @staticmethod
    @custom_bwd
    def backward(ctx, grad_output):
        x, neighbor_indices, weight, bias = ctx.saved_tensors
        kk = weight.shape[0]
        tpb = ctx.tokens_per_batch
        nbr = neighbor_indices.reshape(-1, kk)
        grad_input = grad_weight = grad_bias = None
        need_b = bias is not None and ctx.needs_input_grad[3]
        need_w = ctx.needs_input_grad[2]
        need_x = ctx.needs_input_grad[0]
        if not (need_x or need_w or need_b):
            return None, None, None, None, None, None
        status = None
        if need_x:
            status = ctx.table_status
            if status is None:
                status = _status_for(neighbor_indices, tpb)
        # one library call: the two halves of the backward are independent, so the weight gradient runs
        # next to the input gradient (the reference launches them one after the other, :100-117)
        grad_input, grad_weight, grad_bias = _bwd(grad_output, x.reshape(-1, ctx.C_in), nbr, weight, tpb, status,
                                                  need_x, need_w, need_b)
        if grad_input is not None and x.dim() == 3:
            grad_input = grad_input.view(x.shape)
        if not need_w:
            grad_weight = None
        return grad_input, None, grad_weight, grad_bias, None, None


class _SparseConv2dCastFunction(Function):
    """``SparseConv2dFunction`` for parameters kept in another dtype than the activations (autocast, or a bf16
    input to an fp32 layer): the low-precision copies are made by the module (and cached there), the gradients
    are handed back in the parameters' own dtype.  Same kernels, two autograd nodes fewer per call."""

    @staticmethod
    def forward(ctx, x, neighbor_indices, weight, bias, weight_c, bias_c, tokens_per_batch):
        kk, C_in, C_out = weight_c.shape
        if C_in % 4 != 0:
            raise ValueError(f"C_in ({C_in}) must be divisible by 4 for optimized kernel.")
        ctx.save_for_backward(x, neighbor_indices, weight_c)
        ctx.C_in = C_in
        ctx.tokens_per_batch = tokens_per_batch
        ctx.param_dtype = weight.dtype
        ctx.bias_dtype = bias.dtype if bias is not None else None
        ctx.table_status = _status_for(neighbor_indices, tokens_per_batch) if ctx.needs_input_grad[0] else None
        return ops.conv_fwd(x.reshape(-1, C_in), neighbor_indices.reshape(-1, kk), weight_c, bias_c, tokens_per_batch)

    @staticmethod
    def backward(ctx, grad_output):
        x, neighbor_indices, weight_c = ctx.saved_tensors
        kk = weight_c.shape[0]
        tpb = ctx.tokens_per_batch
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[2]
        need_b = ctx.bias_dtype is not None and ctx.needs_input_grad[3]
        if not (need_x or need_w or need_b):
            return None, None, None, None, None, None, None
        status = None
        if need_x:
            status = ctx.table_status if ctx.table_status is not None else _status_for(neighbor_indices, tpb)
        gx, gw, gb = _bwd(grad_output, x.reshape(-1, ctx.C_in), neighbor_indices.reshape(-1, kk), weight_c, tpb,
                          status, need_x, need_w, need_b)
        if gx is not None and x.dim() == 3:
            gx = gx.view(x.shape)
        gw = gw.to(ctx.param_dtype) if (need_w and gw is not None) else None
        gb = gb.to(ctx.bias_dtype) if (need_b and gb is not None) else None
        return gx, None, gw, gb, None, None, None


class SparseConv2d(nn.Module):
    """Drop-in for the reference module (sparse_conv_layer.py:126-211)."""

    def __init__(self, in_channels, out_channels, bias=True, chunk_size=4096, *, kernel_size=3):
        super().__init__()
        if kernel_size % 2 != 1:
            raise ValueError("kernel_size must be odd")
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.chunk_size = chunk_size      # accepted for compatibility; unused
        self.kernel_size = kernel_size
        kk = kernel_size * kernel_size
        self.weight = nn.Parameter(torch.empty(kk, in_channels, out_channels))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_channels))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self):
        # same scheme as the reference (:145-161): Kaiming-uniform(a=sqrt(5)) on (C_out, C_in, K, K),
        # stored as (K*K, C_in, C_out); bias U(-1/sqrt(fan_in), 1/sqrt(fan_in))
        k = self.kernel_size
        temp = torch.empty(self.out_channels, self.in_channels, k, k)
        nn.init.kaiming_uniform_(temp, a=math.sqrt(5))
        with torch.no_grad():
            self.weight.copy_(temp.view(self.out_channels, self.in_channels, k * k).permute(2, 1, 0))
        if self.bias is not None:
            fan_in = self.in_channels * k * k
            bound = 1 / math.sqrt(fan_in)
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, x, neighbor_indices, local_indices=None):
        kk = self.kernel_size * self.kernel_size
        is_batched = x.dim() == 3
        tokens_per_batch = 0
        if is_batched:
            B, N, C = x.shape
            if local_indices is None:
                # reference heuristic (:170-177): indices are local iff max < N; cached per table object
                if neighbor_indices.numel() > 0:
                    local_indices = _table_cache.get(
                        neighbor_indices, ("local", N), lambda: bool(neighbor_indices.max() < N))
                else:
                    local_indices = False
            if local_indices:
                tokens_per_batch = N
            x = x.reshape(-1, C)
        table = neighbor_indices
        if table.dtype != torch.int32:
            table = _table_cache.get(neighbor_indices, "int32", lambda: neighbor_indices.to(torch.int32))
            if ops.is_known_symmetric(neighbor_indices):
                ops.mark_symmetric(table)
        if table.dim() == 3:
            table = _table_cache.get(table, "flat", lambda: table.reshape(-1, kk)) if table.is_contiguous() \
                else table.reshape(-1, kk)

        weight = self.weight
        bias = self.bias
        target_dtype = x.dtype
        if torch.is_autocast_enabled():
            target_dtype = torch.get_autocast_dtype("cuda")
            if x.dtype != target_dtype:
                x = x.to(target_dtype)
        if weight.dtype == target_dtype and (bias is None or bias.dtype == target_dtype):
            output = SparseConv2dFunction.apply(x, table, weight, bias, tokens_per_batch, self.chunk_size)
        else:
            # parameters live in another dtype (the usual case under autocast): their low-precision copies are
            # kept until the parameters change, e.g. across the two forward passes of activation checkpointing
            weight_c, bias_c = self._cast_params(target_dtype)
            output = _SparseConv2dCastFunction.apply(x, table, weight, bias, weight_c, bias_c, tokens_per_batch)
        if is_batched:
            output = output.view(B, N, -1)
        return output

    def invalidate_cast_cache(self):
        """Drops the cached low-precision parameter copies.  They are keyed on the parameters' version counters,
        which in-place tensor ops bump; writes that bypass them (``param.data`` arithmetic of some fused
        optimizers, raw-pointer updates) do not, so such code must call this after every update - or set
        ``module.cache_casts = False`` to cast on every call as the reference does (:196-203)."""
        self._cast_cache = None

    def train(self, mode=True):
        self._cast_cache = None
        return super().train(mode)

    def _cast_params(self, dtype):
        w, b = self.weight, self.bias
        if not getattr(self, "cache_casts", True):
            with torch.no_grad():
                return w.detach().to(dtype), None if b is None else b.detach().to(dtype)
        key = (dtype, w.data_ptr(), w._version, None if b is None else (b.data_ptr(), b._version))
        cached = getattr(self, "_cast_cache", None)
        if cached is None or cached[0] != key:
            with torch.no_grad():
                cached = (key, w.detach().to(dtype), None if b is None else b.detach().to(dtype))
            self._cast_cache = cached
        return cached[1], cached[2]

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        # older checkpoints hold the weight as (C_in, K*K, C_out); same rule as the reference's
        # remap_legacy_sparse_conv_weights (opentad/utils/checkpoint.py:44-57)
        key = prefix + "weight"
        w = state_dict.get(key)
        if w is not None and w.dim() == 3 and w.shape != self.weight.shape and \
                w.permute(1, 0, 2).shape == self.weight.shape:
            state_dict[key] = w.permute(1, 0, 2).contiguous()
        self._cast_cache = None
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def extra_repr(self):
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, "
                f"bias={self.bias is not None}")


def remap_legacy_sparse_conv_weights(state_dict, model_state_dict):
    """Same contract as the reference helper (opentad/utils/checkpoint.py:44-57): every ``*sparse_conv.weight`` of
    ``state_dict`` whose shape differs from the model's but matches after swapping the first two axes
    (``(C_in, 9, C_out)`` -> ``(9, C_in, C_out)``) is permuted in place; the dict is returned."""
    for key, param in state_dict.items():
        if key.endswith("sparse_conv.weight") and key in model_state_dict:
            target = model_state_dict[key].shape
            if param.shape != target and param.dim() == 3 and param.permute(1, 0, 2).shape == target:
                state_dict[key] = param.permute(1, 0, 2).contiguous()
    return state_dict
