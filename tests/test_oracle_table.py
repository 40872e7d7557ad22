"""CPU tier: the numpy table oracle against the golden vectors produced by the reference's
own source text (tests/golden/make_golden.py) and against structural invariants."""
import math
import os

import numpy as np
import pytest

from oracle import table as otab


def test_initial_table_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "table_init.npz"))
    names = sorted(k[len("shape_"):] for k in g.files if k.startswith("shape_"))
    assert names
    for n in names:
        h, w, T, B = (int(v) for v in g["shape_" + n])
        got = otab.initial_table(h, w, T, B)
        assert got.dtype == np.int32
        np.testing.assert_array_equal(got, g["table_" + n])


def test_select_and_remap_chain_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "table_chain.npz"))
    names = sorted(k[:-4] for k in g.files if k.endswith("_cfg"))
    assert len(names) >= 4
    for n in names:
        h, w, T, B, rounds = (int(v) for v in g[n + "_cfg"])
        rate = float(g[n + "_rate"][0])
        table = otab.initial_table(h, w, T, B)
        cur = T * h * w
        for r in range(rounds):
            k = otab.num_keep(rate, cur)
            scores = g[f"{n}_scores{r}"]
            idx = otab.select_topk(scores, k)
            np.testing.assert_array_equal(idx, g[f"{n}_idx{r}"])
            table = otab.remap_table(table, idx)
            np.testing.assert_array_equal(table, g[f"{n}_table{r}"])
            cur = k


def test_fused_build_equals_first_round(golden_dir):
    g = np.load(os.path.join(golden_dir, "table_chain.npz"))
    for n in ("clip", "slice", "keep10"):
        h, w, T, B, _ = (int(v) for v in g[n + "_cfg"])
        scores = g[f"{n}_scores0"]
        k = g[f"{n}_idx0"].shape[1]
        kept, tab = otab.build_table(scores, k, h, w, 3)
        np.testing.assert_array_equal(kept, g[f"{n}_idx0"].astype(np.int32))
        np.testing.assert_array_equal(tab, g[f"{n}_table0"].reshape(-1, 9))


def test_num_keep_examples():
    # values quoted from the reference schedule: ceil(0.55*196)=108, ceil(0.6*1568)=941
    assert otab.num_keep(0.55, 196) == 108
    assert otab.num_keep(0.6, 1568) == 941
    assert otab.num_keep(0.6, 941) == 565
    assert otab.num_keep(0.6, 565) == 339
    assert otab.num_keep(0.1, 196) == 20
    assert otab.num_keep(0.3, 196) == 59
    assert otab.num_keep(1.0, 196) == 196
    assert otab.num_keep(0.0, 196) == 0


def test_tie_and_nan_rules():
    s = np.array([[0.5, np.nan, 2.0, -1.0, np.inf, 2.0, 2.0]], dtype=np.float32)
    np.testing.assert_array_equal(otab.select_topk(s, 3), [[1, 2, 4]])   # nan, inf, first 2.0
    np.testing.assert_array_equal(otab.select_topk(s, 4), [[1, 2, 4, 5]])
    z = np.array([[0.0, -0.0, 0.0, -0.0]], dtype=np.float32)
    np.testing.assert_array_equal(otab.select_topk(z, 2), [[0, 1]])      # -0.0 == +0.0
    n = np.array([[np.nan, 1.0, -np.nan, np.nan]], dtype=np.float32)
    np.testing.assert_array_equal(otab.select_topk(n, 2), [[0, 2]])      # all NaNs tie
    np.testing.assert_array_equal(otab.select_topk(s, 0).shape, (1, 0))
    np.testing.assert_array_equal(otab.select_topk(s, 99), [list(range(7))])


@pytest.mark.parametrize("h,w,T,B,ksize,rate", [(14, 14, 2, 2, 3, 0.3), (5, 7, 1, 3, 5, 0.5),
                                                (16, 16, 1, 1, 3, 0.1), (10, 10, 2, 1, 3, 1.0)])
def test_structural_invariants(h, w, T, B, ksize, rate):
    rng = np.random.default_rng(7)
    scores = rng.standard_normal((B, T * h * w)).astype(np.float32)
    k = otab.num_keep(rate, T * h * w)
    kept, tab = otab.build_table(scores, k, h, w, ksize)
    n, kk = tab.shape
    assert n == B * k and kk == ksize * ksize
    np.testing.assert_array_equal(tab[:, kk // 2], np.arange(n))
    assert tab.min() >= -1 and tab.max() < n
    assert otab.table_is_symmetric(tab)
    assert np.all(np.diff(kept, axis=1) > 0)
    # geometric meaning of every entry
    r = ksize // 2
    pos = kept.astype(np.int64)
    for b in range(B):
        rank = -np.ones(T * h * w, dtype=np.int64)
        rank[pos[b]] = np.arange(k)
        for i in range(0, k, max(1, k // 17)):
            p = pos[b, i]
            t, y, x = p // (h * w), (p % (h * w)) // w, p % w
            for dy in range(-r, r + 1):
                for dx in range(-r, r + 1):
                    kcol = (dy + r) * ksize + dx + r
                    yy, xx = y + dy, x + dx
                    exp = -1
                    if 0 <= yy < h and 0 <= xx < w and rank[t * h * w + yy * w + xx] >= 0:
                        exp = b * k + rank[t * h * w + yy * w + xx]
                    assert tab[b * k + i, kcol] == exp


def test_asymmetric_table_detected():
    tab = otab.initial_table(4, 4, 1, 1).reshape(-1, 9).copy()
    assert otab.table_is_symmetric(tab)
    tab[5, 0] = 7
    assert not otab.table_is_symmetric(tab)
