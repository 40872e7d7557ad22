"""CPU oracle for the neighbor-index table (TEST INFRASTRUCTURE, not product code).

A numpy restatement of the three pieces of torch code that build and maintain the
``[N_kept, K*K]`` int32 neighbor table in the reference backbone
(``opentad/models/backbones/vit_sparse_adapter_poguise.py``):

* ``initial_table``   follows ``get_initial_neighbor_indices`` (:1623-1670)
* ``select_topk``     follows the selection in ``KTPAttention.forward`` (:763, :784-787)
* ``remap_table``     follows the gather + remap in ``Block._inner_forward`` (:913-977)
* ``build_table``     is the composition "full grid -> select -> remap" for one round,
                      which is what the fused CUDA builder emits directly.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module.
The pin for this oracle is ``tests/golden/table_*.npz``: outputs of the reference's own
source text executed on CPU torch by ``tests/golden/make_golden.py``.

Tie rule.  ``torch.topk`` leaves the choice among equal scores unspecified; this oracle
(and the CUDA builder) fix "lower index wins".  NaN ranks above every number, as in
torch's ordering; all NaNs tie with each other; ``-0.0 == +0.0``.
"""
import math

import numpy as np


def num_keep(keep_rate, seg_len):
    """k = min(ceil(keep_rate * L), L) in Python double arithmetic (:763, :784)."""
    return max(0, min(int(math.ceil(keep_rate * seg_len)), seg_len))


def initial_table(h, w, T, B, ksize=3):
    """Full-grid table ``[B, T*h*w, ksize*ksize]`` int32, batch-global indices.

    Entry (b, t, y, x, k) with k = (dy+r)*ksize + (dx+r), dy outer / dx inner (:1633-1638),
    is the global index of (b, t, y+dy, x+dx) or -1 outside the h x w grid.  No neighbours
    across slices or clips (:1640-1668).
    """
    r = ksize // 2
    n_sp = h * w
    ys, xs = np.meshgrid(np.arange(h), np.arange(w), indexing="ij")
    cols = []
    for dy in range(-r, r + 1):
        for dx in range(-r, r + 1):
            yy, xx = ys + dy, xs + dx
            ok = (yy >= 0) & (yy < h) & (xx >= 0) & (xx < w)
            cols.append(np.where(ok, yy * w + xx, -1).reshape(-1))
    sp = np.stack(cols, axis=1).astype(np.int64)            # [h*w, KK]
    t_off = (np.arange(T, dtype=np.int64) * n_sp).reshape(T, 1, 1)
    tab = np.where(sp[None] != -1, sp[None] + t_off, -1).reshape(T * n_sp, -1)
    b_off = (np.arange(B, dtype=np.int64) * (T * n_sp)).reshape(B, 1, 1)
    tab = np.where(tab[None] != -1, tab[None] + b_off, -1)
    return tab.astype(np.int32)


def select_topk(scores, k):
    """Indices of the k largest scores of every row, ascending (:785-787).

    scores: float32 ``[B, L]``.  Returns int64 ``[B, k]``.  Stable tie rule: among equal
    scores the lower index is kept; NaN is larger than everything.
    """
    scores = np.asarray(scores, dtype=np.float32)
    B, L = scores.shape
    k = max(0, min(int(k), L))
    out = np.empty((B, k), dtype=np.int64)
    ar = np.arange(L)
    for b in range(B):
        s = scores[b]
        nan = np.isnan(s)
        val = np.where(nan, np.float32(0), s)
        # primary: NaN first; secondary: value descending; tertiary: index ascending
        order = np.lexsort((ar, -val.astype(np.float64), ~nan))
        out[b] = np.sort(order[:k])
    return out


def remap_table(table, idx):
    """One pruning round on an existing table (:913-977).

    table: int32 ``[B, N_prev, KK]`` with indices global over ``B*N_prev``;
    idx:   int64 ``[B, N_new]`` positions kept inside every batch row.
    Returns int32 ``[B, N_new, KK]`` global over ``B*N_new``.
    """
    table = np.asarray(table)
    idx = np.asarray(idx, dtype=np.int64)
    B, n_prev, kk = table.shape
    n_new = idx.shape[1]
    kept = np.take_along_axis(table, idx[:, :, None].repeat(kk, axis=2), axis=1)
    mapping = np.full(B * n_prev, -1, dtype=np.int32)
    old_global = idx + (np.arange(B, dtype=np.int64) * n_prev)[:, None]
    new_global = np.arange(n_new, dtype=np.int64)[None, :] + (np.arange(B, dtype=np.int64) * n_new)[:, None]
    mapping[old_global.reshape(-1)] = new_global.reshape(-1).astype(np.int32)
    flat = kept.reshape(-1)
    out = np.where(flat != -1, mapping[np.clip(flat, 0, None)], np.int32(-1))
    return out.reshape(B, n_new, kk).astype(np.int32)


def build_table(scores, k, h, w, ksize=3):
    """Fused "select + table" for one round starting from the full grid.

    scores: float32 ``[n_seg, seg_len]`` with ``seg_len = T*h*w``; each segment is one
    selection unit (a slice when T == 1, a clip otherwise).
    Returns ``(kept_idx int32 [n_seg, k], table int32 [n_seg*k, ksize*ksize])``.
    """
    scores = np.asarray(scores, dtype=np.float32)
    n_seg, seg_len = scores.shape
    assert seg_len % (h * w) == 0
    T = seg_len // (h * w)
    idx = select_topk(scores, k)
    full = initial_table(h, w, T, n_seg, ksize)
    tab = remap_table(full, idx)
    return idx.astype(np.int32), tab.reshape(n_seg * idx.shape[1], ksize * ksize)


def table_is_symmetric(table, tokens_per_batch=0):
    """True iff ``nbr[nbr[i,k]+off(i), KK-1-k] + off == i`` for every valid entry."""
    table = np.asarray(table).reshape(-1, np.asarray(table).shape[-1]).astype(np.int64)
    n, kk = table.shape
    rows = np.arange(n, dtype=np.int64)
    off = (rows // tokens_per_batch) * tokens_per_batch if tokens_per_batch > 0 else np.zeros(n, np.int64)
    for k in range(kk):
        j = table[:, k]
        valid = j != -1
        jj = np.where(valid, j + off, 0)
        if np.any(valid & ((jj < 0) | (jj >= n))):
            return False
        back = table[jj, kk - 1 - k]
        back_off = (jj // tokens_per_batch) * tokens_per_batch if tokens_per_batch > 0 else 0
        if np.any(valid & ((back == -1) | (back + back_off != rows))):
            return False
    return True
