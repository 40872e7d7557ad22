"""CPU tier: the C conv oracle against the dense scatter->conv2d->gather golden vectors."""
import os

import numpy as np
import pytest

from oracle import conv as oconv
from oracle import table as otab

CASES = ["k3", "k3_full", "k5", "k3_c16"]


@pytest.fixture(scope="module")
def gold(golden_dir):
    return np.load(os.path.join(golden_dir, "conv_dense_identity.npz"))


@pytest.mark.parametrize("name", CASES)
def test_fwd_bwd_f64_matches_dense_identity(gold, name):
    B, T, h, w, cin, cout, ksize, k = (int(v) for v in gold[name + "_cfg"])
    tab = gold[name + "_table"]
    x, wt, bias, gy = (gold[f"{name}_{q}"] for q in ("x", "w", "bias", "gy"))
    y = oconv.fwd(x, tab, wt, bias, acc="f64")
    assert oconv.rel_err(y, gold[name + "_y"]) < 1e-12
    gx = oconv.dgrad(gy, tab, wt, acc="f64")
    assert oconv.rel_err(gx, gold[name + "_gx"]) < 1e-12
    gw, gb = oconv.wgrad(gy, x, tab, ksize * ksize, acc="f64")
    assert oconv.rel_err(gw, gold[name + "_gw"]) < 1e-12
    assert oconv.rel_err(gb, gold[name + "_gb"]) < 1e-12


@pytest.mark.parametrize("name", CASES)
def test_f32_flavour_close_to_f64(gold, name):
    tab = gold[name + "_table"]
    x, wt, bias, gy = (gold[f"{name}_{q}"] for q in ("x", "w", "bias", "gy"))
    kk = wt.shape[0]
    assert oconv.rel_err(oconv.fwd(x, tab, wt, bias, acc="f32"), gold[name + "_y"]) < 1e-5
    assert oconv.rel_err(oconv.dgrad(gy, tab, wt, acc="f32"), gold[name + "_gx"]) < 1e-5
    gw, gb = oconv.wgrad(gy, x, tab, kk, acc="f32")
    assert oconv.rel_err(gw, gold[name + "_gw"]) < 1e-5
    assert oconv.rel_err(gb, gold[name + "_gb"]) < 1e-5


def test_table_in_fixture_is_oracle_table(gold):
    for name in CASES:
        B, T, h, w, cin, cout, ksize, k = (int(v) for v in gold[name + "_cfg"])
        kept, tab = otab.build_table(gold[name + "_scores"], k, h, w, ksize)
        np.testing.assert_array_equal(tab, gold[name + "_table"])


def test_tokens_per_batch_offsets():
    rng = np.random.default_rng(3)
    h = w = 4
    n_local = h * w
    tab_local = otab.initial_table(h, w, 1, 1).reshape(-1, 9)
    tab_global = otab.initial_table(h, w, 1, 3).reshape(-1, 9)
    tab_rep = np.tile(tab_local, (3, 1))
    x = rng.standard_normal((3 * n_local, 8)).astype(np.float32)
    wt = rng.standard_normal((9, 8, 4)).astype(np.float32)
    gy = rng.standard_normal((3 * n_local, 4)).astype(np.float32)
    np.testing.assert_allclose(oconv.fwd(x, tab_rep, wt, None, n_local), oconv.fwd(x, tab_global, wt, None, 0))
    np.testing.assert_allclose(oconv.dgrad(gy, tab_rep, wt, n_local), oconv.dgrad(gy, tab_global, wt, 0))
    np.testing.assert_allclose(oconv.wgrad(gy, x, tab_rep, 9, n_local)[0], oconv.wgrad(gy, x, tab_global, 9, 0)[0])


def test_asymmetric_table_and_empty():
    rng = np.random.default_rng(4)
    n, cin, cout, kk = 10, 4, 4, 9
    tab = rng.integers(-1, n, size=(n, kk)).astype(np.int32)   # arbitrary, not geometric
    x = rng.standard_normal((n, cin)).astype(np.float32)
    wt = rng.standard_normal((kk, cin, cout)).astype(np.float32)
    gy = rng.standard_normal((n, cout)).astype(np.float32)
    # dgrad is the adjoint of fwd for ANY table: <fwd(x), gy> == <x, dgrad(gy)>
    lhs = (oconv.fwd(x, tab, wt) * gy).sum()
    rhs = (x * oconv.dgrad(gy, tab, wt)).sum()
    assert abs(lhs - rhs) < 1e-9 * max(1, abs(lhs))
    gw, _ = oconv.wgrad(gy, x, tab, kk)
    assert abs((gw * wt).sum() - lhs) < 1e-9 * max(1, abs(lhs))
    assert oconv.fwd(x[:0], tab[:0], wt).shape == (0, cout)


def test_row_and_channel_samples_equal_the_full_oracle():
    """The sampled forms used on full-size problems (forward rows, input-gradient rows, weight gradient of a
    few input channels) give exactly the corresponding entries of the full computation."""
    rng = np.random.default_rng(6)
    scores = rng.standard_normal((6, 196)).astype(np.float32)
    kept, tab = otab.build_table(scores, 59, 14, 14, 3)
    n = tab.shape[0]
    x = rng.standard_normal((n, 16)).astype(np.float32)
    wt = rng.standard_normal((9, 16, 8)).astype(np.float32)
    gy = rng.standard_normal((n, 8)).astype(np.float32)
    sel = np.arange(3, n, 7)
    np.testing.assert_array_equal(oconv.fwd(x, tab[sel], wt), oconv.fwd(x, tab, wt)[sel])
    np.testing.assert_array_equal(oconv.dgrad_rows(gy, tab, wt, sel), oconv.dgrad(gy, tab, wt)[sel])
    cs = [1, 5, 9]
    np.testing.assert_array_equal(oconv.wgrad(gy, np.ascontiguousarray(x[:, cs]), tab, 9)[0],
                                  oconv.wgrad(gy, x, tab, 9)[0][:, cs])
    # batch-local tables: the sampled input gradient follows the same per-row offsets
    tab_l = otab.initial_table(4, 4, 1, 1).reshape(-1, 9)
    rep = np.tile(tab_l, (3, 1))
    g2 = rng.standard_normal((48, 8)).astype(np.float32)
    np.testing.assert_array_equal(oconv.dgrad_rows(g2, rep, wt, [0, 17, 47], 16), oconv.dgrad(g2, rep, wt, 16)[[0, 17, 47]])
