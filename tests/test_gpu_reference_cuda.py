"""GPU tier: the new kernels against the reference's own CUDA extension on identical inputs.

The extension is built from the reference checkout by ``oracle/build_ref.py`` into
``oracle/_ref/`` (test infrastructure).  These tests skip when that file is absent.
Acceptance: both within tolerance of the float64 oracle, and the new kernel's error no larger
than twice the reference CUDA path's error (plus one rounding unit).
"""
import numpy as np
import pytest
import torch

from oracle import conv as oconv
from tests.helpers import BASE_SEED, f32np, make_conv_inputs, make_table

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import build_ref
    mod = build_ref.load_built()
    if mod is None:
        pytest.skip("reference CUDA extension not built (oracle/_ref missing)")
    return mod


def _both(ref, table, x, w, b, gy):
    from eccv26_tad_b200 import ops
    tc, xc, wc, bc, gc = (t.cuda() for t in (table, x, w, b, gy))
    n, cin = x.shape
    mine = (ops.conv_fwd(xc, tc, wc, bc), ops.conv_dgrad(gc, tc, wc), ops.conv_wgrad(gc, xc, tc, 9, with_bias=False)[0])
    if cin >= 128:   # the reference's own dispatch (sparse_conv_layer.py:55)
        ry = ref.implicit_gemm_fwd_v2_chunked(xc, tc, wc, bc, 0, 4096)
    else:
        ry = ref.fwd(xc, tc, wc, w.shape[2], 0) + bc.view(1, -1)
    theirs = (ry, ref.bwd_in(gc, tc, wc, n, cin, 0), ref.bwd_w(gc, xc, tc, cin, 0))
    torch.cuda.synchronize()
    return mine, theirs


@pytest.mark.parametrize("dtype,C,B,T,keep", [
    (torch.float32, 192, 1, 8, 0.5),          # config 1
    (torch.bfloat16, 192, 2, 20, 0.3),        # config 2 at a quarter of the slices
    (torch.bfloat16, 192, 2, 20, 0.1),
    (torch.bfloat16, 192, 2, 20, 0.55),
    (torch.bfloat16, 256, 1, 6, 0.3),         # config 3, reduced rows
    (torch.bfloat16, 64, 1, 8, 0.5),          # small-channel kernel of the reference (Cin < 128)
    (torch.float16, 128, 1, 8, 0.5),
])
def test_against_reference_cuda(ref, dtype, C, B, T, keep):
    torch.backends.cuda.matmul.allow_tf32 = False
    _, _, table = make_table(B, T, 14, 14, keep, 3, BASE_SEED + C)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, C, C, 3, dtype, BASE_SEED + C, bias="random")
    mine, theirs = _both(ref, table, x, w, b, gy)
    tn = table.numpy()
    xf, wf, bf, gf = (f32np(t) for t in (x, w, b, gy))
    truth = (oconv.fwd(xf, tn, wf, bf), oconv.dgrad(gf, tn, wf), oconv.wgrad(gf, xf, tn, 9, with_bias=False)[0])
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    unit = 2e-6 if dtype == torch.float32 else 4e-3
    for name, m, r, t in zip(("y", "gx", "gw"), mine, theirs, truth):
        em, er = oconv.rel_err(f32np(m), t), oconv.rel_err(f32np(r), t)
        assert em < tol, f"{name}: new kernel err {em:.3e}"
        assert oconv.rel_err(f32np(m), f32np(r)) < 2 * tol, f"{name}: differs from reference CUDA"
        assert em <= 2 * er + unit, f"{name}: new err {em:.3e} vs reference CUDA err {er:.3e}"
