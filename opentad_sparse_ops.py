"""Top-level ``opentad_sparse_ops``: the name the reference wrapper imports
(``opentad/models/bricks/sparse_conv_layer.py:12-13``; the reference builds it as a CUDA extension,
``setup.py:21-34``), here the five callables of ``eccv26_tad_b200.opentad_sparse_ops`` on top of ``libsvtad.so``.
"""
from eccv26_tad_b200.opentad_sparse_ops import (  # noqa: F401
    bwd_in,
    bwd_w,
    fwd,
    implicit_gemm_fwd_v2,
    implicit_gemm_fwd_v2_chunked,
)
