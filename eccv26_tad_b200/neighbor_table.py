"""Neighbor-table construction with the reference backbone's meaning, one CUDA kernel per step.

Counterparts in ``opentad/models/backbones/vit_sparse_adapter_poguise.py``:
``get_initial_neighbor_indices`` (:1623-1670), the top-k + sort of ``KTPAttention.forward``
(:763, :784-787) and the gather + remap of ``Block._inner_forward`` (:913-977).
"""
import math

from . import ops


def get_initial_neighbor_indices(h, w, T, device, B, kernel_size=3):
    """int32 ``[B, T*h*w, K*K]`` full-grid table, batch-global indices, -1 outside the grid."""
    return ops.table_init(B, T, h, w, kernel_size, device)


def num_keep_tokens(keep_rate, n_tokens):
    """``min(ceil(keep_rate * N), N)`` in Python double arithmetic (reference :763, :784)."""
    return max(0, min(int(math.ceil(keep_rate * n_tokens)), n_tokens))


def select_topk(scores, num_keep):
    """Ascending int64 indices ``[B, k]`` of the k largest scores per row (reference :785-787).

    Ties keep the lower index; NaN ranks above every number.
    """
    return ops.topk_select(scores, num_keep)


def update_neighbor_indices(neighbor_indices, idx, global_mapping_buffer=None):
    """One pruning round: gather the kept rows and renumber them (reference :913-977).

    neighbor_indices int32 ``[B, N_prev, K*K]`` (global), idx int64 ``[B, N_new]``.
    """
    return ops.table_remap(neighbor_indices, idx, global_mapping_buffer)


def select_and_update(scores, neighbor_indices, num_keep):
    """``select_topk`` and ``update_neighbor_indices`` of one pruning round fused into one kernel.

    scores float32 ``[B, N_prev]``, neighbor_indices int32 ``[B, N_prev, K*K]`` -> ``(idx int64 [B, k], table)``.
    """
    return ops.table_select_remap(scores, neighbor_indices, num_keep)


def build_neighbor_table(scores, keep_rate=None, h=14, w=14, kernel_size=3, num_keep=None):
    """Fused first round: top-k per segment straight to ``(kept_idx, table)``.

    scores float32 ``[n_seg, seg_len]``; a segment is one slice (``seg_len == h*w``) or one clip
    (``seg_len == T*h*w``).  Returns kept_idx int32 ``[n_seg, k]`` and table int32 ``[n_seg*k, K*K]``.
    """
    if num_keep is None:
        num_keep = num_keep_tokens(keep_rate, scores.shape[1])
    return ops.table_build(scores, num_keep, h, w, kernel_size)
