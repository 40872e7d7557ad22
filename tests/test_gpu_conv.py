"""GPU tier: SparseConv2D forward / dgrad / wgrad through the C ABI against the CPU oracle.

Error metric everywhere: max|a - ref| / max|ref| per tensor (``oracle.conv.rel_err``).
Tolerances: fp32 1e-5, bf16 / fp16 outputs and gradients 2e-2.
"""
import os

import numpy as np
import pytest
import torch

from oracle import conv as oconv
from oracle import table as otab
from tests.helpers import BASE_SEED, f32np, make_conv_inputs, make_table

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def _ops():
    from eccv26_tad_b200 import ops
    return ops


@pytest.fixture(autouse=True)
def _no_forced_path(monkeypatch):
    monkeypatch.delenv("SVTAD_FORCE_PATH", raising=False)
    monkeypatch.delenv("SVTAD_TC_BN", raising=False)
    monkeypatch.delenv("SVTAD_TC_IMPL", raising=False)
    yield
    assert _ops().device_error() == 0, "a bounded wait inside a tensor-core kernel gave up"


def _run_all(table, x, w, b, gy, tpb=0, sym=None):
    ops = _ops()
    kk = w.shape[0]
    tc, xc, wc, bc, gc = (t.cuda() for t in (table, x, w, b, gy))
    y = ops.conv_fwd(xc, tc, wc, bc, tpb)
    gx = ops.conv_dgrad(gc, tc, wc, tpb, assume_symmetric=bool(sym)) if sym is not None else ops.conv_dgrad(gc, tc, wc, tpb)
    gw, gb = ops.conv_wgrad(gc, xc, tc, kk, tpb)
    torch.cuda.synchronize()
    return y, gx, gw, gb


def _check_all(table, x, w, b, gy, outs, tol, tpb=0):
    y, gx, gw, gb = outs
    tn = table.numpy()
    xf, wf, bf, gf = (f32np(t) for t in (x, w, b, gy))
    kk = w.shape[0]
    errs = {
        "y": oconv.rel_err(f32np(y), oconv.fwd(xf, tn, wf, bf, tpb)),
        "gx": oconv.rel_err(f32np(gx), oconv.dgrad(gf, tn, wf, tpb)),
    }
    egw, egb = oconv.wgrad(gf, xf, tn, kk, tpb)
    errs["gw"] = oconv.rel_err(f32np(gw), egw)
    errs["gb"] = oconv.rel_err(f32np(gb), egb)
    for k, v in errs.items():
        assert v < tol, f"{k}: rel err {v:.3e} >= {tol}"
    assert y.dtype == x.dtype and gx.dtype == gy.dtype and gw.dtype == x.dtype and gb.dtype == x.dtype
    return errs


def test_config1_fp32_forward_and_backward():
    """fp32, batch 1, T=8, 14x14, C=192, keep 50% by seeded random choice (98 tokens per slice)."""
    rng = np.random.default_rng(BASE_SEED + 1)
    scores = rng.standard_normal((8, 196)).astype(np.float32)      # top-k of iid scores == uniform subset
    kept, table = otab.build_table(scores, 98, 14, 14, 3)
    table = torch.from_numpy(table)
    assert table.shape == (784, 9)
    x, w, b, gy = make_conv_inputs(784, 192, 192, 3, torch.float32, BASE_SEED + 1)
    assert _ops().path_for(0, 784, 192, 192, 9, torch.float32) == "simt"
    outs = _run_all(table, x, w, b, gy)
    _check_all(table, x, w, b, gy, outs, 1e-5)


@pytest.mark.parametrize("keep", [0.10, 0.30, 0.55])
@pytest.mark.parametrize("path", ["tc", "simt"])
def test_config2_bf16_fwd_bwd_full_size(keep, path, monkeypatch):
    """bf16, batch 2, T=80 (160 slices), 14x14, C=192, keep sweep; both implementations."""
    monkeypatch.setenv("SVTAD_FORCE_PATH", path)
    _, _, table = make_table(2, 80, 14, 14, keep, 3, BASE_SEED + 2)
    n = table.shape[0]
    assert n == {0.10: 3200, 0.30: 9440, 0.55: 17280}[keep]
    x, w, b, gy = make_conv_inputs(n, 192, 192, 3, torch.bfloat16, BASE_SEED + 2, bias="random")
    outs = _run_all(table, x, w, b, gy)
    _check_all(table, x, w, b, gy, outs, 2e-2)


@pytest.mark.parametrize("hint", [2, 3, 6])
@pytest.mark.parametrize("keep", [0.10, 0.30, 0.55])
def test_concurrency_hint_changes_the_plans_not_the_results(hint, keep):
    """svtad_set_concurrency(k) plans the tensor-core kernels for a k-th of the GPU: wide column blocks, persistent
    CTAs that take several row tiles in turn, fewer token splits.  Forward and input gradient must come out bit for
    bit as under the default (their summation order does not depend on the plan); the weight gradient's partials
    are summed in another order, so it is held to the oracle and to the default's result within rounding."""
    ops = _ops()
    _, _, table = make_table(2, 80, 14, 14, keep, 3, BASE_SEED + 2)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 192, 192, 3, torch.bfloat16, BASE_SEED + 2, bias="random")
    assert ops.get_concurrency() == 1
    base = _run_all(table, x, w, b, gy)
    prev = ops.set_concurrency(hint)
    try:
        assert prev == 1 and ops.get_concurrency() == hint
        outs = _run_all(table, x, w, b, gy)
        tc_, xc, wc, gc = (t.cuda() for t in (table, x, w, gy))
        gx2, gw2, gb2 = ops.conv_bwd(gc, xc, tc_, wc, assume_symmetric=True)      # the one-call backward under the hint
        torch.cuda.synchronize()
    finally:
        ops.set_concurrency(1)
    assert torch.equal(outs[0], base[0]) and torch.equal(outs[1], base[1])
    assert torch.equal(gx2, base[1])
    _check_all(table, x, w, b, gy, outs, 2e-2)
    for a, r in ((outs[2], base[2]), (outs[3], base[3]), (gw2, base[2]), (gb2, base[3])):
        assert oconv.rel_err(f32np(a), f32np(r).astype(np.float64)) < 1e-2
    assert ops.device_error() == 0


@pytest.mark.parametrize("bn", ["64", "96", "192"])
def test_tc_column_block_variants(bn, monkeypatch):
    monkeypatch.setenv("SVTAD_FORCE_PATH", "tc")
    monkeypatch.setenv("SVTAD_TC_BN", bn)
    _, _, table = make_table(1, 10, 14, 14, 0.3, 3, 99)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 192, 192, 3, torch.bfloat16, 99, bias="random")
    outs = _run_all(table, x, w, b, gy)
    _check_all(table, x, w, b, gy, outs, 2e-2)


@pytest.mark.parametrize("C,ks,dtype,shape", [
    (192, 3, torch.bfloat16, (2, 20, 0.3)),      # 19 row tiles: odd, the last pair's second CTA has no rows
    (192, 3, torch.float16, (1, 3, 0.55)),
    (64, 3, torch.bfloat16, (1, 9, 0.3)),
    (128, 3, torch.bfloat16, (1, 7, 1.0)),
    (256, 5, torch.bfloat16, (1, 6, 0.3)),
    (1024, 3, torch.bfloat16, (1, 6, 0.3)),      # several column blocks per row-tile pair
    (192, 3, torch.bfloat16, (2, 80, 0.55)),     # 135 tiles on 74 CTA pairs: persistent loop, two accumulators
])
def test_cta_pair_kernels(C, ks, dtype, shape, monkeypatch):
    """Forward / dgrad on CTA pairs (tcgen05 cta_group::2, the default for large inputs) against the oracle."""
    monkeypatch.setenv("SVTAD_TC_IMPL", "pair")
    B, T, keep = shape
    _, _, table = make_table(B, T, 14, 14, keep, ks, 77)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, C, C, ks, dtype, 77, bias="random")
    outs = _run_all(table, x, w, b, gy)
    _check_all(table, x, w, b, gy, outs, 2e-2)
    monkeypatch.setenv("SVTAD_TC_IMPL", "hybrid")
    ref = _run_all(table, x, w, b, gy)
    for u, v in zip(outs[:2], ref[:2]):
        assert oconv.rel_err(f32np(u), f32np(v)) < 8e-3      # same products, fp32 accumulate, one rounding


def test_cta_pair_kernels_ragged_rows_and_batch_local_indices(monkeypatch):
    monkeypatch.setenv("SVTAD_TC_IMPL", "pair")
    for n in (1, 129, 1000):
        table = -np.ones((n, 9), dtype=np.int32)
        table[:, 4] = np.arange(n)
        table[1:, 3] = np.arange(n - 1)
        table[:-1, 5] = np.arange(1, n)
        table = torch.from_numpy(table)
        x, w, b, gy = make_conv_inputs(n, 192, 64, 3, torch.bfloat16, n, bias="random")
        outs = _run_all(table, x, w, b, gy)
        _check_all(table, x, w, b, gy, outs, 2e-2)
    # indices local to each batch row
    _, _, glob = make_table(3, 4, 14, 14, 0.3, 3, 9)
    n = glob.shape[0]
    tpb = n // 3
    local = glob.clone()
    local[local >= 0] %= tpb
    x, w, b, gy = make_conv_inputs(n, 128, 128, 3, torch.bfloat16, 9, bias="random")
    outs = _run_all(local, x, w, b, gy, tpb=tpb)
    _check_all(local, x, w, b, gy, outs, 2e-2, tpb=tpb)


def test_tc_and_simt_agree_tightly(monkeypatch):
    """Same bf16 inputs, fp32 accumulation on both paths: outputs differ by rounding only."""
    _, _, table = make_table(2, 8, 14, 14, 0.3, 3, 5)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 192, 192, 3, torch.bfloat16, 5, bias="random")
    monkeypatch.setenv("SVTAD_FORCE_PATH", "tc")
    a = _run_all(table, x, w, b, gy)
    monkeypatch.setenv("SVTAD_FORCE_PATH", "simt")
    c = _run_all(table, x, w, b, gy)
    for u, v in zip(a, c):
        assert oconv.rel_err(f32np(u), f32np(v)) < 8e-3      # one bf16 ulp is 2^-8 = 3.9e-3


@pytest.mark.parametrize("C,ks", [(256, 3), (256, 5), (768, 3), (1024, 3)])
def test_config3_large_channels_reduced_rows(C, ks):
    """Large-channel regime at reduced row count (batch 1, T=6) so the CPU oracle finishes in seconds."""
    _, _, table = make_table(1, 6, 14, 14, 0.3, ks, BASE_SEED + 3)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, C, C, ks, torch.bfloat16, BASE_SEED + 3, bias="random")
    assert _ops().path_for(0, n, C, C, ks * ks, torch.bfloat16) == "tc"
    outs = _run_all(table, x, w, b, gy)
    _check_all(table, x, w, b, gy, outs, 2e-2)


def _check_sampled(table, x, w, b, gy, outs, tol, row_step=64, n_ci=8):
    """Full-size problems against the float64 oracle on a sample: every ``row_step``-th row of the forward output
    and of the input gradient, ``n_ci`` input channels of the weight gradient (all taps, all output channels), the
    whole bias gradient.  Each error is max|a - ref| / max|ref| over the sampled entries."""
    y, gx, gw, gb = outs
    tn = table.numpy()
    n, kk = tn.shape
    sel = np.arange(row_step // 2, n, row_step)
    xf, wf, bf, gf = (f32np(t) for t in (x, w, b, gy))
    cs = np.linspace(0, x.shape[1] - 1, n_ci).astype(np.int64)
    egw, _ = oconv.wgrad(gf, np.ascontiguousarray(xf[:, cs]), tn, kk, with_bias=False)
    errs = {
        "y": oconv.rel_err(f32np(y)[sel], oconv.fwd(xf, tn[sel], wf, bf)),
        "gx": oconv.rel_err(f32np(gx)[sel], oconv.dgrad_rows(gf, tn, wf, sel)),
        "gw": oconv.rel_err(f32np(gw)[:, cs], egw),
        "gb": oconv.rel_err(f32np(gb), gf.astype(np.float64).sum(0)),
    }
    for k, v in errs.items():
        assert v < tol, f"{k}: rel err {v:.3e} >= {tol}"
    return errs


@pytest.mark.parametrize("C,ks", [(256, 3), (256, 5), (768, 3), (768, 5), (1024, 3), (1024, 5)])
def test_config3_full_size_against_sampled_oracle(C, ks):
    """The large-channel configuration at its configured size (batch 4, T=80, keep 30 % = 18 880 rows; C in
    {256, 768, 1024}; 3x3 and 5x5) through the default dispatch, checked against the float64 oracle on a sample
    of rows / channels so that the CPU side finishes in seconds."""
    _, _, table = make_table(4, 80, 14, 14, 0.3, ks, BASE_SEED + 3)
    n = table.shape[0]
    assert n == 18880
    x, w, b, gy = make_conv_inputs(n, C, C, ks, torch.bfloat16, BASE_SEED + 3, bias="random")
    assert _ops().path_for(0, n, C, C, ks * ks, torch.bfloat16) == "tc"
    outs = _run_all(table, x, w, b, gy)
    _check_sampled(table, x, w, b, gy, outs, 2e-2, row_step=32, n_ci=8)


def _chain_table(n):
    table = -np.ones((n, 9), dtype=np.int32)
    table[:, 4] = np.arange(n)
    table[1:, 3] = np.arange(n - 1)
    table[:-1, 5] = np.arange(1, n)
    return torch.from_numpy(table)


@pytest.mark.parametrize("n", [148 * 128, 148 * 128 + 1])
def test_default_dispatch_on_both_sides_of_the_pair_switch(n):
    """With no override the forward / dgrad run on single CTAs while the row tiles do not outnumber the SMs (148
    tiles of 128 rows on a B200) and on CTA pairs from one tile more; both sides against the oracle."""
    assert "SVTAD_TC_IMPL" not in os.environ
    table = _chain_table(n)
    x, w, b, gy = make_conv_inputs(n, 192, 192, 3, torch.bfloat16, n % 1000, bias="random")
    outs = _run_all(table, x, w, b, gy)
    _check_sampled(table, x, w, b, gy, outs, 2e-2, row_step=16, n_ci=16)
    # the last rows (a one-row tile on the far side of the switch) in full
    tail = np.arange(n - 130, n)
    tn = table.numpy()
    xf, wf, bf, gf = (f32np(t) for t in (x, w, b, gy))
    assert oconv.rel_err(f32np(outs[0])[tail], oconv.fwd(xf, tn[tail], wf, bf)) < 2e-2
    assert oconv.rel_err(f32np(outs[1])[tail], oconv.dgrad_rows(gf, tn, wf, tail)) < 2e-2


def test_geometric_tables_on_both_sides_of_the_pair_switch():
    """Same with tables from the builder: 18 880 rows (148 row tiles, single CTAs) and 19 520 rows (153 tiles, pairs)."""
    for keep, rows in ((0.30, 18880), (0.31, 19520)):
        _, _, table = make_table(4, 80, 14, 14, keep, 3, 41)
        n = table.shape[0]
        assert n == rows
        x, w, b, gy = make_conv_inputs(n, 192, 192, 3, torch.bfloat16, 41, bias="random")
        outs = _run_all(table, x, w, b, gy)
        _check_sampled(table, x, w, b, gy, outs, 2e-2, row_step=32, n_ci=8)


def test_config3_full_size_adjoint_identities():
    """Full size (batch 4, T=80, keep 30%, C=256): <fwd(x), gy> == <x, dgrad(gy)> == <W, wgrad>."""
    ops = _ops()
    _, _, table = make_table(4, 80, 14, 14, 0.3, 3, BASE_SEED + 3)
    n = table.shape[0]
    assert n == 18880
    x, w, b, gy = make_conv_inputs(n, 256, 256, 3, torch.bfloat16, BASE_SEED + 3)
    tc, xc, wc, gc = table.cuda(), x.cuda(), w.cuda(), gy.cuda()
    y = ops.conv_fwd(xc, tc, wc, None)
    gx = ops.conv_dgrad(gc, tc, wc)
    gw, gb = ops.conv_wgrad(gc, xc, tc, 9)
    lhs = (y.double() * gc.double()).sum().item()
    mid = (gx.double() * xc.double()).sum().item()
    rhs = (gw.double() * wc.double()).sum().item()
    scale = (y.double().abs() * gc.double().abs()).sum().item()
    assert abs(lhs - mid) < 2e-2 * scale and abs(lhs - rhs) < 2e-2 * scale
    assert oconv.rel_err(f32np(gb), f32np(gy).astype(np.float64).sum(0)) < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_golden_dense_identity(dtype, golden_dir):
    """scatter -> conv2d -> gather golden vectors (includes 5x5 and 100% keep)."""
    g = np.load(os.path.join(golden_dir, "conv_dense_identity.npz"))
    for name in ("k3", "k3_full", "k5", "k3_c16"):
        table = torch.from_numpy(g[name + "_table"])
        x, w, b, gy = (torch.from_numpy(g[f"{name}_{q}"]).to(dtype) for q in ("x", "w", "bias", "gy"))
        outs = _run_all(table, x, w, b, gy)
        if dtype == torch.float32:
            y, gx, gw, gb = outs
            assert oconv.rel_err(f32np(y), g[name + "_y"]) < 1e-5
            assert oconv.rel_err(f32np(gx), g[name + "_gx"]) < 1e-5
            assert oconv.rel_err(f32np(gw), g[name + "_gw"]) < 1e-5
            assert oconv.rel_err(f32np(gb), g[name + "_gb"]) < 1e-5
        else:
            _check_all(table, x, w, b, gy, outs, 2e-2)


@pytest.mark.parametrize("dtype,C", [(torch.float32, 64), (torch.bfloat16, 64), (torch.bfloat16, 192), (torch.float32, 40)])
def test_tokens_per_batch_local_indices(dtype, C):
    """Local tables + tokens_per_batch == global tables (tokens_per_batch a multiple of 32)."""
    ops = _ops()
    _, _, tab1 = make_table(1, 2, 8, 8, 0.5, 3, 11)          # 64 tokens, local to one batch row
    tpb = tab1.shape[0]
    assert tpb % 32 == 0
    B = 5
    local = tab1.repeat(B, 1)
    glob = torch.cat([torch.where(tab1 >= 0, tab1 + b * tpb, tab1) for b in range(B)])
    x, w, b, gy = make_conv_inputs(B * tpb, C, C, 3, dtype, 11, bias="random")
    a = _run_all(local, x, w, b, gy, tpb=tpb)
    c = _run_all(glob, x, w, b, gy, tpb=0)
    for u, v in zip(a, c):
        assert torch.equal(u, v)
    _check_all(local, x, w, b, gy, a, TOL[dtype], tpb=tpb)


@pytest.mark.parametrize("dtype,C", [(torch.float32, 32), (torch.bfloat16, 128)])
def test_asymmetric_table_takes_scatter_form(dtype, C):
    """Arbitrary (non-geometric) tables: dgrad must still be the adjoint of the forward."""
    rng = np.random.default_rng(21)
    n = 300
    table = torch.from_numpy(rng.integers(-1, n, size=(n, 9)).astype(np.int32))
    x, w, b, gy = make_conv_inputs(n, C, C, 3, dtype, 21, bias="random")
    outs = _run_all(table, x, w, b, gy)
    _check_all(table, x, w, b, gy, outs, TOL[dtype])


@pytest.mark.parametrize("n", [1, 31, 129, 1000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ragged_row_counts_and_odd_widths(n, dtype):
    rng = np.random.default_rng(n)
    # a geometric table on a ragged number of rows: 1-D chain (left / centre / right taps only)
    table = -np.ones((n, 9), dtype=np.int32)
    table[:, 4] = np.arange(n)
    table[1:, 3] = np.arange(n - 1)
    table[:-1, 5] = np.arange(1, n)
    table = torch.from_numpy(table)
    for cin, cout in [(64, 64), (8, 20), (192, 64)]:
        x, w, b, gy = make_conv_inputs(n, cin, cout, 3, dtype, n, bias="random")
        outs = _run_all(table, x, w, b, gy)
        _check_all(table, x, w, b, gy, outs, TOL[dtype])


def test_empty_input_and_all_pruned_rows():
    ops = _ops()
    w = torch.randn(9, 64, 64).cuda().bfloat16()
    y = ops.conv_fwd(torch.empty(0, 64).cuda().bfloat16(), torch.empty(0, 9, dtype=torch.int32).cuda(), w, None)
    assert y.shape == (0, 64)
    gw, gb = ops.conv_wgrad(torch.empty(0, 64).cuda().bfloat16(), torch.empty(0, 64).cuda().bfloat16(),
                            torch.empty(0, 9, dtype=torch.int32).cuda(), 9)
    assert float(gw.abs().sum()) == 0 and float(gb.abs().sum()) == 0
    # rows whose every neighbour (centre included) is -1 produce bias only
    n = 200
    table = -torch.ones(n, 9, dtype=torch.int32)
    x, w, b, gy = make_conv_inputs(n, 64, 64, 3, torch.bfloat16, 1, bias="random")
    y = ops.conv_fwd(x.cuda(), table.cuda(), w.cuda(), b.cuda())
    assert torch.equal(y.cpu(), b.expand(n, -1).contiguous())


@pytest.mark.parametrize("hint,keep", [(1, 0.3), (3, 0.3), (4, 0.55)])
def test_tensor_core_pipeline_is_race_free(hint, keep, monkeypatch):
    """The tensor-core kernels are deterministic, so any hazard between the copy engine's writes
    and the MMA's reads would show as a run-to-run difference.  40 repeats, bitwise equal - also with persistent
    CTAs that take several row tiles in turn (hint 3: 74 tiles on 49 CTAs; hint 4: 135 tiles on 37), where the
    table rows of the next tile, the two accumulators and the staged bias change hands between tiles."""
    monkeypatch.setenv("SVTAD_FORCE_PATH", "tc")
    ops = _ops()
    request_hint = ops.set_concurrency(hint)
    try:
        _race_free_body(ops, keep)
    finally:
        ops.set_concurrency(request_hint)


def _race_free_body(ops, keep):
    _, _, table = make_table(2, 80, 14, 14, keep, 3, 77)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 192, 192, 3, torch.bfloat16, 77, bias="random")
    tc, xc, wc, bc, gc = (t.cuda() for t in (table, x, w, b, gy))
    first = None
    for _ in range(40):
        cur = (ops.conv_fwd(xc, tc, wc, bc), ops.conv_dgrad(gc, tc, wc, assume_symmetric=True),
               ops.conv_wgrad(gc, xc, tc, 9)[0])
        if first is None:
            first = cur
        else:
            for u, v in zip(first, cur):
                assert torch.equal(u, v)
    # and the result is the right one
    assert oconv.rel_err(f32np(first[0]), oconv.fwd(f32np(x), table.numpy(), f32np(w), f32np(b))) < 2e-2


@pytest.mark.parametrize("C", [128, 192])
def test_persistent_ctas_with_a_ragged_last_tile(C):
    """Hint 16 leaves 9 CTAs for 21 row tiles, the last of them 37 rows: every CTA walks two or three tiles and one
    of them meets the ragged end.  Against the full oracle, bias on."""
    ops = _ops()
    n = 128 * 20 + 37
    table = _chain_table(n)
    x, w, b, gy = make_conv_inputs(n, C, C, 3, torch.bfloat16, 5, bias="random")
    ops.set_concurrency(16)
    try:
        outs = _run_all(table, x, w, b, gy, sym=True)
    finally:
        ops.set_concurrency(1)
    _check_all(table, x, w, b, gy, outs, 2e-2)
    assert ops.device_error() == 0


@pytest.mark.parametrize("dtype,C,kind", [(torch.bfloat16, 192, "geometric"), (torch.float32, 32, "geometric"),
                                          (torch.bfloat16, 128, "arbitrary")])
def test_one_call_backward_equals_the_two_halves(dtype, C, kind, monkeypatch):
    """svtad_conv_bwd (weight gradient on the library's side stream) gives bit-identical results to
    svtad_conv_dgrad + svtad_conv_wgrad, for every subset of requested gradients, repeatedly."""
    ops = _ops()
    if kind == "geometric":
        _, _, table = make_table(2, 12, 14, 14, 0.3, 3, 33)
    else:
        rng = np.random.default_rng(33)
        table = torch.from_numpy(rng.integers(-1, 700, size=(700, 9)).astype(np.int32))
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, C, C, 3, dtype, 33)
    tc, xc, wc, gc = (t.cuda() for t in (table, x, w, gy))
    gx0 = ops.conv_dgrad(gc, tc, wc)
    gw_alone, gb_alone = ops.conv_wgrad(gc, xc, tc, 9)
    # when both gradients are asked for, the call plans its two side-by-side kernels for half the GPU each: the same
    # plan (and so the same summation order of the weight gradient's partials) as the halves under a hint of 2
    ops.set_concurrency(2)
    try:
        gw0, gb0 = ops.conv_wgrad(gc, xc, tc, 9)
        assert torch.equal(ops.conv_dgrad(gc, tc, wc), gx0) or kind != "geometric"
    finally:
        ops.set_concurrency(1)
    assert oconv.rel_err(f32np(gw0), f32np(gw_alone).astype(np.float64)) < 1e-2

    def same_gx(a):
        if kind == "geometric":
            return torch.equal(a, gx0)
        # arbitrary tables take the scatter form: fp32 atomics, summation order differs from run to run
        return oconv.rel_err(f32np(a), f32np(gx0)) < 1e-2

    for _ in range(3):
        gx, gw, gb = ops.conv_bwd(gc, xc, tc, wc)
        assert same_gx(gx) and torch.equal(gw, gw0) and torch.equal(gb, gb0)
    gx, gw, gb = ops.conv_bwd(gc, xc, tc, wc, need_w=False, need_b=False)
    assert gw is None and gb is None and same_gx(gx)
    gx, gw, gb = ops.conv_bwd(gc, xc, tc, wc, need_x=False)       # one kernel: planned alone
    assert gx is None and torch.equal(gw, gw_alone) and torch.equal(gb, gb_alone)
    gx, gw, gb = ops.conv_bwd(gc, xc, tc, wc, need_b=False)
    assert gb is None and same_gx(gx) and torch.equal(gw, gw0)
    # the caller's stream alone orders the results: consume them at once on a non-default stream
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        gx, gw, gb = ops.conv_bwd(gc, xc, tc, wc)
        sums = torch.stack([gx.float().sum(), gw.float().sum(), gb.float().sum()])
    st.synchronize()
    ref = torch.stack([gx0.float().sum(), gw0.float().sum(), gb0.float().sum()])
    assert torch.equal(sums[1:], ref[1:])
    assert torch.equal(sums[:1], ref[:1]) if kind == "geometric" else abs(float(sums[0] - ref[0])) <= 1e-2 * float(gx0.float().abs().sum())


def test_one_call_backward_where_the_half_gpu_plan_needs_more_splits():
    """18 880 rows, C=192, 5x5: the weight gradient planned for half the GPU (as the one-call backward does) takes
    more token splits than planned for all of it; the workspace that svtad_workspace_bytes asks for must cover both."""
    ops = _ops()
    _, _, table = make_table(4, 80, 14, 14, 0.3, 5, BASE_SEED + 3)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 192, 192, 5, torch.bfloat16, BASE_SEED + 3, bias="random")
    tc, xc, wc, gc = (t.cuda() for t in (table, x, w, gy))
    gx, gw, gb = ops.conv_bwd(gc, xc, tc, wc, assume_symmetric=True)
    y = ops.conv_fwd(xc, tc, wc, b.cuda())
    torch.cuda.synchronize()
    _check_sampled(table, x, w, b, gy, (y, gx, gw, gb), 2e-2, row_step=64, n_ci=6)
    assert ops.device_error() == 0


def _fused_bwd(table, x, w, gy, tpb=0):
    ops = _ops()
    tc, xc, wc, gc = (t.cuda() for t in (table, x, w, gy))
    gx, gw, gb = ops.conv_bwd(gc, xc, tc, wc, tpb, assume_symmetric=True)
    torch.cuda.synchronize()
    return gx, gw, gb


@pytest.mark.parametrize("C,ks,dtype,shape", [
    (192, 3, torch.bfloat16, (2, 80, 0.10)),     # the benchmark's three layers
    (192, 3, torch.bfloat16, (2, 80, 0.30)),
    (192, 3, torch.bfloat16, (2, 80, 0.55)),
    (192, 3, torch.float16, (1, 3, 0.55)),
    (64, 3, torch.bfloat16, (1, 9, 0.3)),
    (128, 3, torch.bfloat16, (1, 7, 1.0)),
    (256, 5, torch.bfloat16, (1, 6, 0.3)),
    (768, 3, torch.bfloat16, (1, 6, 0.3)),       # three column blocks per row tile and per block pair
    (192, 3, torch.bfloat16, (1, 1, 0.02)),      # 4 rows: one tile, one split
])
def test_one_call_backward_symmetric_tables_against_oracle(C, ks, dtype, shape):
    """The one-call backward without a status word (the caller vouches for a symmetric table: no validation pass, no
    scatter-form launches): both gradients against the oracle, the input gradient bitwise equal to the stand-alone
    kernel's, and bitwise repeatable."""
    ops = _ops()
    B, T, keep = shape
    _, _, table = make_table(B, T, 14, 14, keep, ks, 55)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, C, C, ks, dtype, 55, bias="random")
    gx, gw, gb = _fused_bwd(table, x, w, gy)
    tn = table.numpy()
    xf, wf, gf = (f32np(t) for t in (x, w, gy))
    assert oconv.rel_err(f32np(gx), oconv.dgrad(gf, tn, wf)) < 2e-2
    egw, egb = oconv.wgrad(gf, xf, tn, ks * ks)
    assert oconv.rel_err(f32np(gw), egw) < 2e-2 and oconv.rel_err(f32np(gb), egb) < 2e-2
    gx0 = ops.conv_dgrad(gy.cuda(), table.cuda(), w.cuda(), assume_symmetric=True)
    assert torch.equal(gx, gx0)
    for _ in range(3):
        again = _fused_bwd(table, x, w, gy)
        for u, v in zip((gx, gw, gb), again):
            assert torch.equal(u, v)


def test_one_call_backward_symmetric_ragged_rows_and_batch_local_indices():
    for n in (1, 129, 1000):
        table = _chain_table(n)
        x, w, b, gy = make_conv_inputs(n, 192, 192, 3, torch.bfloat16, n, bias="random")
        gx, gw, gb = _fused_bwd(table, x, w, gy)
        tn = table.numpy()
        xf, wf, gf = (f32np(t) for t in (x, w, gy))
        assert oconv.rel_err(f32np(gx), oconv.dgrad(gf, tn, wf)) < 2e-2
        egw, egb = oconv.wgrad(gf, xf, tn, 9)
        assert oconv.rel_err(f32np(gw), egw) < 2e-2 and oconv.rel_err(f32np(gb), egb) < 2e-2
    _, _, glob = make_table(3, 4, 14, 14, 0.3, 3, 9)
    n = glob.shape[0]
    tpb = n // 3
    local = glob.clone()
    local[local >= 0] %= tpb
    x, w, b, gy = make_conv_inputs(n, 128, 128, 3, torch.bfloat16, 9, bias="random")
    gx, gw, gb = _fused_bwd(local, x, w, gy, tpb=tpb)
    xf, wf, gf = (f32np(t) for t in (x, w, gy))
    assert oconv.rel_err(f32np(gx), oconv.dgrad(gf, local.numpy(), wf, tpb)) < 2e-2
    egw, egb = oconv.wgrad(gf, xf, local.numpy(), 9, tpb)
    assert oconv.rel_err(f32np(gw), egw) < 2e-2 and oconv.rel_err(f32np(gb), egb) < 2e-2


def test_determinism_of_backward():
    _, _, table = make_table(2, 20, 14, 14, 0.3, 3, 8)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 192, 192, 3, torch.bfloat16, 8)
    a = _run_all(table, x, w, b, gy)
    c = _run_all(table, x, w, b, gy)
    for u, v in zip(a, c):
        assert torch.equal(u, v)


def test_errors_are_python_exceptions():
    ops = _ops()
    w = torch.randn(9, 6, 8).cuda()
    with pytest.raises(ValueError, match="divisible by 4"):
        ops.conv_fwd(torch.randn(4, 6).cuda(), torch.zeros(4, 9, dtype=torch.int32).cuda(), w, None)
    with pytest.raises(ValueError):
        ops.conv_fwd(torch.randn(4, 8).cuda().double(), torch.zeros(4, 9, dtype=torch.int32).cuda(),
                     torch.randn(9, 8, 8).cuda().double(), None)
