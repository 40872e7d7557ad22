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


@pytest.mark.parametrize("keep", [0.10, 0.30, 0.55])
def test_config2_full_size_against_reference_cuda(ref, keep):
    """The benchmark's configuration at its full size (batch 2, T=80: 3 200 / 9 440 / 17 280 rows, C=192, bf16): the
    same acceptance as above, with the float64 oracle evaluated on a sample of rows / input channels."""
    _, _, table = make_table(2, 80, 14, 14, keep, 3, BASE_SEED + 2)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 192, 192, 3, torch.bfloat16, BASE_SEED + 2, bias="random")
    mine, theirs = _both(ref, table, x, w, b, gy)
    tn = table.numpy()
    xf, wf, bf, gf = (f32np(t) for t in (x, w, b, gy))
    sel = np.arange(16, n, 32)
    cs = np.linspace(0, 191, 8).astype(np.int64)
    truth = (oconv.fwd(xf, tn[sel], wf, bf), oconv.dgrad_rows(gf, tn, wf, sel),
             oconv.wgrad(gf, np.ascontiguousarray(xf[:, cs]), tn, 9, with_bias=False)[0])
    pick = (lambda a: f32np(a)[sel], lambda a: f32np(a)[sel], lambda a: f32np(a)[:, cs])
    for name, m, r, t, p in zip(("y", "gx", "gw"), mine, theirs, truth, pick):
        em, er = oconv.rel_err(p(m), t), oconv.rel_err(p(r), t)
        assert em < 2e-2, f"{name}: new kernel err {em:.3e}"
        assert oconv.rel_err(f32np(m), f32np(r)) < 4e-2, f"{name}: differs from reference CUDA"
        assert em <= 2 * er + 4e-3, f"{name}: new err {em:.3e} vs reference CUDA err {er:.3e}"


@pytest.mark.parametrize("dtype,C", [(torch.bfloat16, 192), (torch.float32, 64)])
def test_batch_local_indices_against_reference_cuda(ref, dtype, C):
    """``tokens_per_batch > 0``: per-clip tables with clip-local row numbers, offset by the kernels (the reference
    adds ``(i / tokens_per_batch) * tokens_per_batch``, 2d_sparse_v3.cu:432-436, implicit_gemm_v2.cu:63-77).
    tokens_per_batch is a multiple of 32 here, where the reference's per-32-row-block offset equals the per-row one."""
    from eccv26_tad_b200 import ops
    torch.backends.cuda.matmul.allow_tf32 = False
    _, _, tab1 = make_table(1, 16, 14, 14, 0.5, 3, BASE_SEED + 5)        # one clip: 16 slices x 98 rows = 1 568
    tpb = tab1.shape[0]
    assert tpb % 32 == 0
    B = 3
    local = tab1.repeat(B, 1)
    x, w, b, gy = make_conv_inputs(B * tpb, C, C, 3, dtype, BASE_SEED + 5, bias="random")
    tc, xc, wc, bc, gc = (t.cuda() for t in (local, x, w, b, gy))
    mine = (ops.conv_fwd(xc, tc, wc, bc, tpb), ops.conv_dgrad(gc, tc, wc, tpb), ops.conv_wgrad(gc, xc, tc, 9, tpb, with_bias=False)[0])
    if C >= 128:
        ry = ref.implicit_gemm_fwd_v2_chunked(xc, tc, wc, bc, tpb, 4096)
    else:
        ry = ref.fwd(xc, tc, wc, C, tpb) + bc.view(1, -1)
    theirs = (ry, ref.bwd_in(gc, tc, wc, B * tpb, C, tpb), ref.bwd_w(gc, xc, tc, C, tpb))
    torch.cuda.synchronize()
    tn = local.numpy()
    xf, wf, bf, gf = (f32np(t) for t in (x, w, b, gy))
    truth = (oconv.fwd(xf, tn, wf, bf, tpb), oconv.dgrad(gf, tn, wf, tpb), oconv.wgrad(gf, xf, tn, 9, tpb, with_bias=False)[0])
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    unit = 2e-6 if dtype == torch.float32 else 4e-3
    for name, m, r, t in zip(("y", "gx", "gw"), mine, theirs, truth):
        em, er = oconv.rel_err(f32np(m), t), oconv.rel_err(f32np(r), t)
        assert em < tol, f"{name}: new kernel err {em:.3e}"
        assert em <= 2 * er + unit, f"{name}: new err {em:.3e} vs reference CUDA err {er:.3e}"
