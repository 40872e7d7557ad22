"""GPU tier: neighbor-table kernels, bit-exact against the numpy oracle and the golden vectors."""
import os

import numpy as np
import pytest
import torch

from oracle import table as otab
from tests.helpers import BASE_SEED, make_scores

pytestmark = pytest.mark.gpu


def _ops():
    from eccv26_tad_b200 import ops
    return ops


def test_table_init_matches_golden_and_oracle(golden_dir):
    ops = _ops()
    g = np.load(os.path.join(golden_dir, "table_init.npz"))
    for n in sorted(k[len("shape_"):] for k in g.files if k.startswith("shape_")):
        h, w, T, B = (int(v) for v in g["shape_" + n])
        got = ops.table_init(B, T, h, w, 3).cpu().numpy()
        np.testing.assert_array_equal(got, g["table_" + n])
    for (h, w, T, B, ks) in [(14, 14, 80, 2, 3), (7, 9, 3, 2, 5), (16, 16, 4, 1, 7), (1, 1, 1, 1, 3)]:
        got = ops.table_init(B, T, h, w, ks).cpu().numpy()
        np.testing.assert_array_equal(got, otab.initial_table(h, w, T, B, ks))
    assert ops.table_init(0, 8, 14, 14, 3).shape == (0, 8 * 196, 9)


@pytest.mark.parametrize("keep", [0.10, 0.25, 0.50])
def test_table_build_full_size_table_config(keep):
    """Table-only config at full size: batch 8, T=384 -> 3072 slices of 14x14 scores."""
    ops = _ops()
    scores = make_scores(8 * 384, 196, BASE_SEED + 4)
    k = otab.num_keep(keep, 196)
    assert k == {0.10: 20, 0.25: 49, 0.50: 98}[keep]
    kept, table = ops.table_build(scores.cuda(), k, 14, 14, 3)
    ekept, etable = otab.build_table(scores.numpy(), k, 14, 14, 3)
    np.testing.assert_array_equal(kept.cpu().numpy(), ekept)
    np.testing.assert_array_equal(table.cpu().numpy(), etable)
    # selection alone (int64, as torch.topk + sort would give)
    idx = ops.topk_select(scores.cuda(), k)
    assert idx.dtype == torch.int64
    np.testing.assert_array_equal(idx.cpu().numpy(), ekept.astype(np.int64))
    # size-independent properties at full size
    t = table.cpu().numpy()
    np.testing.assert_array_equal(t[:, 4], np.arange(t.shape[0]))
    assert otab.table_is_symmetric(t)
    status = ops.table_check(table)
    assert int(status.item()) == 0


@pytest.mark.parametrize("h,w,T,ks,keep", [(14, 14, 1, 3, 0.55), (14, 14, 1, 5, 0.3), (10, 10, 1, 3, 0.3),
                                           (16, 16, 1, 3, 0.5), (5, 7, 3, 3, 0.4), (5, 7, 3, 7, 0.9),
                                           (14, 14, 1, 3, 1.0), (3, 3, 1, 3, 0.01)])
def test_table_build_small_segments(h, w, T, ks, keep):
    ops = _ops()
    L = T * h * w
    scores = make_scores(37, L, BASE_SEED + h * 100 + w)
    k = max(1, otab.num_keep(keep, L))
    kept, table = ops.table_build(scores.cuda(), k, h, w, ks)
    ekept, etable = otab.build_table(scores.numpy(), k, h, w, ks)
    np.testing.assert_array_equal(kept.cpu().numpy(), ekept)
    np.testing.assert_array_equal(table.cpu().numpy(), etable)


@pytest.mark.parametrize("T,B,keep", [(8, 2, 0.6), (80, 2, 0.3), (2, 3, 0.1), (80, 1, 1.0)])
def test_table_build_per_clip_segments(T, B, keep):
    """Reference-style selection: top-k over all T*14*14 tokens of a clip (one CTA per clip)."""
    ops = _ops()
    L = T * 196
    scores = make_scores(B, L, BASE_SEED + T)
    k = otab.num_keep(keep, L)
    kept, table = ops.table_build(scores.cuda(), k, 14, 14, 3)
    ekept, etable = otab.build_table(scores.numpy(), k, 14, 14, 3)
    np.testing.assert_array_equal(kept.cpu().numpy(), ekept)
    np.testing.assert_array_equal(table.cpu().numpy(), etable)
    idx = ops.topk_select(scores.cuda(), k)
    np.testing.assert_array_equal(idx.cpu().numpy(), ekept.astype(np.int64))


def test_ties_nan_inf_and_zero_signs():
    ops = _ops()
    rng = np.random.default_rng(5)
    for L, h, w in [(196, 14, 14), (1568, 14, 14)]:
        s = rng.integers(-3, 4, size=(9, L)).astype(np.float32)        # heavy ties
        s[0, :] = 1.0                                                   # all equal
        s[1, ::7] = np.nan
        s[2, 5] = np.inf; s[2, 9] = -np.inf
        s[3, ::2] = 0.0; s[3, 1::2] = -0.0
        s[4, :] = np.nan
        s[5, 3] = np.nan; s[5, 100] = -np.nan
        for k in (1, 20, 97, L - 1, L):
            kept, table = ops.table_build(torch.from_numpy(s).cuda(), k, h, w, 3)
            ekept, etable = otab.build_table(s, k, h, w, 3)
            np.testing.assert_array_equal(kept.cpu().numpy(), ekept)
            np.testing.assert_array_equal(table.cpu().numpy(), etable)


def test_remap_chain_matches_golden(golden_dir):
    """Successive pruning rounds: selection + remap on the reference's schedule."""
    ops = _ops()
    g = np.load(os.path.join(golden_dir, "table_chain.npz"))
    for n in sorted(k[:-4] for k in g.files if k.endswith("_cfg")):
        h, w, T, B, rounds = (int(v) for v in g[n + "_cfg"])
        table = ops.table_init(B, T, h, w, 3)
        scratch = torch.empty(B * T * h * w, dtype=torch.int32, device="cuda")
        for r in range(rounds):
            scores = torch.from_numpy(g[f"{n}_scores{r}"]).cuda()
            k = g[f"{n}_idx{r}"].shape[1]
            idx = ops.topk_select(scores, k)
            np.testing.assert_array_equal(idx.cpu().numpy(), g[f"{n}_idx{r}"])
            table = ops.table_remap(table, idx, scratch)
            np.testing.assert_array_equal(table.cpu().numpy(), g[f"{n}_table{r}"])


def test_fused_select_remap_chain_matches_golden(golden_dir):
    """Same schedules as above with selection + remap of a round fused into one kernel."""
    ops = _ops()
    g = np.load(os.path.join(golden_dir, "table_chain.npz"))
    for n in sorted(k[:-4] for k in g.files if k.endswith("_cfg")):
        h, w, T, B, rounds = (int(v) for v in g[n + "_cfg"])
        table = ops.table_init(B, T, h, w, 3)
        for r in range(rounds):
            scores = torch.from_numpy(g[f"{n}_scores{r}"]).cuda()
            k = g[f"{n}_idx{r}"].shape[1]
            idx, table = ops.table_select_remap(scores, table, k)
            np.testing.assert_array_equal(idx.cpu().numpy(), g[f"{n}_idx{r}"])
            np.testing.assert_array_equal(table.cpu().numpy(), g[f"{n}_table{r}"])
    # ties / NaN through the fused path against the oracle
    rng = np.random.default_rng(9)
    s = rng.integers(-2, 3, size=(3, 392)).astype(np.float32)
    s[1, ::5] = np.nan
    t0 = otab.initial_table(14, 14, 2, 3)
    for k in (1, 100, 391, 392):
        idx, tab = ops.table_select_remap(torch.from_numpy(s).cuda(), torch.from_numpy(t0).cuda(), k)
        eidx = otab.select_topk(s, k)
        np.testing.assert_array_equal(idx.cpu().numpy(), eidx)
        np.testing.assert_array_equal(tab.cpu().numpy(), otab.remap_table(t0, eidx))


def test_remap_unsorted_and_bad_indices_do_not_fault():
    ops = _ops()
    table = ops.table_init(2, 1, 4, 4, 3)
    idx = torch.tensor([[5, 2, 9, 1], [0, 15, 7, 3]], dtype=torch.int64)
    got = ops.table_remap(table, idx.cuda()).cpu().numpy()
    np.testing.assert_array_equal(got, otab.remap_table(table.cpu().numpy(), idx.numpy()))
    bad = torch.tensor([[5, 99, -4, 1], [0, 15, 7, 3]], dtype=torch.int64)
    out = ops.table_remap(table, bad.cuda()).cpu().numpy()      # out-of-range rows come back as -1
    assert (out[0, 1] == -1).all() and (out[0, 2] == -1).all()


def test_table_check_flags():
    ops = _ops()
    from eccv26_tad_b200 import _lib
    t = ops.table_init(1, 2, 5, 5, 3).reshape(-1, 9)
    assert int(ops.table_check(t).item()) == 0
    t2 = t.clone(); t2[7, 0] = 11
    assert int(ops.table_check(t2).item()) & _lib.TABLE_ASYMMETRIC
    t3 = t.clone(); t3[3, 2] = 1000
    assert int(ops.table_check(t3).item()) & _lib.TABLE_OUT_OF_RANGE
    # local indices + tokens_per_batch
    loc = ops.table_init(1, 1, 5, 5, 3).reshape(-1, 9).repeat(3, 1)
    assert int(ops.table_check(loc, tokens_per_batch=25).item()) == 0
    assert int(ops.table_check(loc, tokens_per_batch=0).item()) != 0


def test_public_table_api_names():
    import eccv26_tad_b200 as pkg
    t = pkg.get_initial_neighbor_indices(14, 14, 2, "cuda", 2)
    assert t.shape == (2, 392, 9) and t.dtype == torch.int32
    scores = make_scores(2, 392, 3).cuda()
    k = pkg.num_keep_tokens(0.6, 392)
    idx = pkg.select_topk(scores, k)
    t2 = pkg.update_neighbor_indices(t, idx)
    kept, tab = pkg.build_neighbor_table(scores, 0.6, 14, 14)
    np.testing.assert_array_equal(t2.reshape(-1, 9).cpu().numpy(), tab.cpu().numpy())
