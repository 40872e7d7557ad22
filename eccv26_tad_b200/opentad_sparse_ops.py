"""The five callables of the reference's pybind module ``opentad_sparse_ops``
(``opentad/models/bricks/2d_sparse_v3_bind.cpp:8-14``), same positional signatures and return
shapes / dtypes, implemented on ``libsvtad.so``.

``install()`` registers this module under the name ``opentad_sparse_ops`` so that the reference's
own ``sparse_conv_layer.py`` (which does ``import opentad_sparse_ops as sparse_lib_opt``, :12-13)
runs unchanged on top of it.
"""
import sys

from . import ops


def fwd(x, neighbor_indices, w, C_out, tokens_per_batch):
    """launch_fwd (2d_sparse_v3.cu:751-822): no bias, output in x's dtype."""
    assert w.shape[2] == C_out
    return ops.conv_fwd(x.reshape(-1, x.shape[-1]), neighbor_indices, w, None, tokens_per_batch)


def bwd_in(grad_output, neighbor_indices, w, n_kept, C_in, tokens_per_batch):
    """launch_bwd_in (2d_sparse_v3.cu:824-835): [n_kept, C_in] in grad_output's dtype."""
    return ops.conv_dgrad(grad_output, neighbor_indices, w, tokens_per_batch)


def bwd_w(grad_output, x, neighbor_indices, C_in, tokens_per_batch):
    """launch_bwd_w (2d_sparse_v3.cu:837-850): [K*K, C_in, C_out] in x's dtype."""
    kk = neighbor_indices.shape[-1]
    gw, _ = ops.conv_wgrad(grad_output, x.reshape(-1, x.shape[-1]), neighbor_indices, kk,
                           tokens_per_batch, with_bias=False)
    return gw


def implicit_gemm_fwd_v2(x, neighbor_indices, weight, bias, tokens_per_batch):
    """implicit_gemm_v2.cu:197-300; an empty ``torch.Tensor()`` means "no bias"."""
    b = bias if (bias is not None and bias.numel() > 0) else None
    return ops.conv_fwd(x, neighbor_indices, weight, b, tokens_per_batch)


def implicit_gemm_fwd_v2_chunked(x, neighbor_indices, weight, bias, tokens_per_batch, chunk_size):
    """implicit_gemm_v2.cu:306-417; chunk_size is irrelevant here (nothing is materialised)."""
    return implicit_gemm_fwd_v2(x, neighbor_indices, weight, bias, tokens_per_batch)


def install(name="opentad_sparse_ops"):
    sys.modules[name] = sys.modules[__name__]
    return sys.modules[name]
