"""GPU tier: the reference-facing Python surface (module, autograd Function, pybind-module shim)."""
import numpy as np
import pytest
import torch

from oracle import conv as oconv
from tests.helpers import f32np, make_conv_inputs, make_table

pytestmark = pytest.mark.gpu


def _oracle_grads(table, x, w, b, gy, tpb=0):
    tn = table.numpy()
    xf, wf, bf, gf = (f32np(t) for t in (x, w, b, gy))
    y = oconv.fwd(xf, tn, wf, bf, tpb)
    gx = oconv.dgrad(gf, tn, wf, tpb)
    gw, gb = oconv.wgrad(gf, xf, tn, w.shape[0], tpb)
    return y, gx, gw, gb


def test_module_fp32_autograd_matches_oracle():
    from eccv26_tad_b200 import SparseConv2d
    _, _, table = make_table(1, 4, 14, 14, 0.5, 3, 31)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 64, 96, 3, torch.float32, 31, bias="random")
    m = SparseConv2d(64, 96).cuda()
    with torch.no_grad():
        m.weight.copy_(w); m.bias.copy_(b)
    xc = x.cuda().requires_grad_(True)
    y = m(xc, table.cuda())
    y.backward(gy.cuda())
    ey, egx, egw, egb = _oracle_grads(table, x, w, b, gy)
    assert oconv.rel_err(f32np(y), ey) < 1e-5
    assert oconv.rel_err(f32np(xc.grad), egx) < 1e-5
    assert oconv.rel_err(f32np(m.weight.grad), egw) < 1e-5
    assert oconv.rel_err(f32np(m.bias.grad), egb) < 1e-5


def test_module_autocast_bf16_batched_local_and_global_indices():
    """3-D input under bf16 autocast, fp32 master parameters (the reference's training setting)."""
    from eccv26_tad_b200 import SparseConv2d
    _, _, tab1 = make_table(1, 4, 14, 14, 0.3, 3, 32)
    N = tab1.shape[0]
    B = 3
    x, w, b, gy = make_conv_inputs(B * N, 192, 192, 3, torch.float32, 32, bias="random")
    m = SparseConv2d(192, 192).cuda()
    with torch.no_grad():
        m.weight.copy_(w); m.bias.copy_(b)
    local = tab1.unsqueeze(0).repeat(B, 1, 1).cuda()
    glob = torch.stack([torch.where(tab1 >= 0, tab1 + i * N, tab1) for i in range(B)]).cuda()
    # the oracle sees the bf16-rounded operands the autocast path produces
    xb, wb, bb, gb_ = (t.bfloat16() for t in (x, w, b, gy))
    ey, egx, egw, egb = _oracle_grads(glob.reshape(-1, 9).cpu(), xb, wb, bb, gb_)
    for table in (local, glob.long()):           # int64 tables are accepted like in the reference
        m.zero_grad()
        xc = x.view(B, N, 192).cuda().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = m(xc, table)
        assert y.shape == (B, N, 192) and y.dtype == torch.bfloat16
        y.backward(gy.view(B, N, 192).cuda().bfloat16())
        assert xc.grad.shape == xc.shape and xc.grad.dtype == torch.float32
        assert m.weight.grad.dtype == torch.float32
        assert oconv.rel_err(f32np(y).reshape(-1, 192), ey) < 2e-2
        assert oconv.rel_err(f32np(xc.grad).reshape(-1, 192), egx) < 2e-2
        assert oconv.rel_err(f32np(m.weight.grad), egw) < 2e-2
        assert oconv.rel_err(f32np(m.bias.grad), egb) < 2e-2


def test_autocast_parameter_copies_are_cached_until_the_parameters_change():
    """The bf16 copies of fp32 parameters are made once per parameter version (two forwards of activation
    checkpointing share them) and refreshed after an in-place update; gradients come back in fp32."""
    from eccv26_tad_b200 import SparseConv2d, SparseConv2dFunction
    _, _, table = make_table(1, 4, 14, 14, 0.3, 3, 41)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 64, 64, 3, torch.float32, 41, bias="random")
    m = SparseConv2d(64, 64).cuda()
    with torch.no_grad():
        m.weight.copy_(w); m.bias.copy_(b)
    tc, xc, gc = table.cuda(), x.cuda(), gy.cuda().bfloat16()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y1 = m(xc, tc)
        w1 = m._cast_cache[1]
        y2 = m(xc, tc)
        assert m._cast_cache[1] is w1 and w1.dtype == torch.bfloat16
        assert torch.equal(y1, y2)
        # gradients equal those of the explicit-cast route through the reference-shaped Function
        xa = xc.clone().requires_grad_(True)
        m.zero_grad()
        m(xa, tc).backward(gc)
        xb = xc.clone().requires_grad_(True)
        wr = m.weight.detach().clone().requires_grad_(True)
        br = m.bias.detach().clone().requires_grad_(True)
        SparseConv2dFunction.apply(xb.bfloat16(), tc, wr.bfloat16(), br.bfloat16(), 0, 0).backward(gc)
        assert m.weight.grad.dtype == torch.float32 and torch.equal(m.weight.grad, wr.grad)
        assert torch.equal(m.bias.grad, br.grad) and torch.equal(xa.grad, xb.grad)
        with torch.no_grad():
            m.weight.mul_(0.5)
        y3 = m(xc, tc)
        assert m._cast_cache[1] is not w1
        assert not torch.equal(y3, y1)


def test_function_apply_signature_and_partial_grads():
    from eccv26_tad_b200 import SparseConv2dFunction
    _, _, table = make_table(1, 2, 14, 14, 0.5, 3, 33)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 64, 64, 3, torch.bfloat16, 33, bias="random")
    xc = x.cuda()                                   # no grad for x
    wc = w.cuda().requires_grad_(True)
    y = SparseConv2dFunction.apply(xc, table.cuda(), wc, None, 0, 4096)
    y.backward(gy.cuda())
    assert wc.grad is not None and wc.grad.shape == wc.shape
    ey, _, egw, _ = _oracle_grads(table, x, w, torch.zeros(64), gy)
    assert oconv.rel_err(f32np(y), ey) < 2e-2
    assert oconv.rel_err(f32np(wc.grad), egw) < 2e-2
    with pytest.raises(ValueError, match="divisible by 4"):
        SparseConv2dFunction.apply(torch.randn(4, 6).cuda(), torch.zeros(4, 9, dtype=torch.int32).cuda(),
                                   torch.randn(9, 6, 8).cuda())


def test_pybind_module_shim_signatures():
    from eccv26_tad_b200 import opentad_sparse_ops as lib
    _, _, table = make_table(1, 3, 14, 14, 0.5, 3, 34)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 128, 128, 3, torch.bfloat16, 34, bias="random")
    tc, xc, wc, bc, gc = (t.cuda() for t in (table, x, w, b, gy))
    ey, egx, egw, _ = _oracle_grads(table, x, w, b, gy)
    y0, _, _, _ = _oracle_grads(table, x, w, torch.zeros(128), gy)
    assert oconv.rel_err(f32np(lib.fwd(xc, tc, wc, 128, 0)), y0) < 2e-2
    assert oconv.rel_err(f32np(lib.implicit_gemm_fwd_v2(xc, tc, wc, bc, 0)), ey) < 2e-2
    assert oconv.rel_err(f32np(lib.implicit_gemm_fwd_v2(xc, tc, wc, torch.Tensor(), 0)), y0) < 2e-2
    assert oconv.rel_err(f32np(lib.implicit_gemm_fwd_v2_chunked(xc, tc, wc, bc, 0, 4096)), ey) < 2e-2
    assert oconv.rel_err(f32np(lib.bwd_in(gc, tc, wc, n, 128, 0)), egx) < 2e-2
    assert oconv.rel_err(f32np(lib.bwd_w(gc, xc, tc, 128, 0)), egw) < 2e-2
    import sys
    lib.install()
    assert sys.modules["opentad_sparse_ops"].fwd is lib.fwd
    del sys.modules["opentad_sparse_ops"]


def test_kernel_size_5_module():
    from eccv26_tad_b200 import SparseConv2d
    _, _, table = make_table(1, 3, 14, 14, 0.4, 5, 35)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 64, 64, 5, torch.bfloat16, 35, bias="random")
    m = SparseConv2d(64, 64, kernel_size=5).cuda().bfloat16()
    with torch.no_grad():
        m.weight.copy_(w); m.bias.copy_(b)
    xc = x.cuda().requires_grad_(True)
    y = m(xc, table.cuda())
    y.backward(gy.cuda())
    ey, egx, egw, egb = _oracle_grads(table, x, w, b, gy)
    assert oconv.rel_err(f32np(y), ey) < 2e-2
    assert oconv.rel_err(f32np(xc.grad), egx) < 2e-2
    assert oconv.rel_err(f32np(m.weight.grad), egw) < 2e-2


def test_reference_wrapper_runs_unchanged_on_top_of_the_shim():
    """The reference's own ``sparse_conv_layer.py`` (byte-compiled by ``oracle/build_ref.py`` into ``oracle/_ref``;
    its ``import opentad_sparse_ops`` answered by this package's module) - ITS SparseConv2d / SparseConv2dFunction,
    forward and backward under bf16 autocast with fp32 master parameters, 2-D and batched 3-D input, and in plain
    fp32 - against the oracle."""
    from oracle import build_ref
    from eccv26_tad_b200 import opentad_sparse_ops as shim
    ref = build_ref.load_wrapper(shim)
    if ref is None:
        pytest.skip("oracle/_ref/ref_sparse_conv_layer.bytecode has not been built")
    assert ref.sparse_lib_opt is shim                     # no JIT fallback to the reference's CUDA sources
    _, _, tab1 = make_table(1, 6, 14, 14, 0.3, 3, 71)
    N = tab1.shape[0]
    B = 2
    glob = torch.cat([torch.where(tab1 >= 0, tab1 + i * N, tab1) for i in range(B)])
    x, w, b, gy = make_conv_inputs(B * N, 192, 192, 3, torch.float32, 71, bias="random")
    m = ref.SparseConv2d(192, 192).cuda()
    assert tuple(m.weight.shape) == (9, 192, 192)
    with torch.no_grad():
        m.weight.copy_(w); m.bias.copy_(b)
    xb, wb, bb, gb_ = (t.bfloat16() for t in (x, w, b, gy))
    ey, egx, egw, egb = _oracle_grads(glob, xb, wb, bb, gb_)
    cases = [(x.cuda(), glob.cuda(), gy.cuda().bfloat16()),                                     # [N, C], global indices
             (x.view(B, N, 192).cuda(), tab1.unsqueeze(0).repeat(B, 1, 1).cuda().long(),        # [B, N, C], local, int64
              gy.view(B, N, 192).cuda().bfloat16())]
    for xin, table, g in cases:
        m.zero_grad()
        xc = xin.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = m(xc, table)
        assert y.dtype == torch.bfloat16 and y.shape[:-1] == xin.shape[:-1]
        y.backward(g)
        assert oconv.rel_err(f32np(y).reshape(-1, 192), ey) < 2e-2
        assert oconv.rel_err(f32np(xc.grad).reshape(-1, 192), egx) < 2e-2
        assert oconv.rel_err(f32np(m.weight.grad), egw) < 2e-2
        assert oconv.rel_err(f32np(m.bias.grad), egb) < 2e-2
    # fp32, small-channel branch of the reference wrapper (fwd + bias added by the wrapper, :86-87)
    x, w, b, gy = make_conv_inputs(N, 64, 64, 3, torch.float32, 72, bias="random")
    m = ref.SparseConv2d(64, 64).cuda()
    with torch.no_grad():
        m.weight.copy_(w); m.bias.copy_(b)
    xc = x.cuda().requires_grad_(True)
    y = m(xc, tab1.cuda())
    y.backward(gy.cuda())
    ey, egx, egw, egb = _oracle_grads(tab1, x, w, b, gy)
    assert oconv.rel_err(f32np(y), ey) < 1e-5 and oconv.rel_err(f32np(xc.grad), egx) < 1e-5
    assert oconv.rel_err(f32np(m.weight.grad), egw) < 1e-5 and oconv.rel_err(f32np(m.bias.grad), egb) < 1e-5
    from eccv26_tad_b200 import ops
    assert ops.device_error() == 0
