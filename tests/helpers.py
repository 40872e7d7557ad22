"""Seeded synthetic workloads shared by the tests, the smoke check and the benchmark.

The generators follow the value distributions the benchmark configs name: features and
upstream gradients N(0,1), weights Kaiming-normal on (C_out, C_in, K, K) stored as
(K*K, C_in, C_out), scores N(0,1), kept tokens by per-segment top-k.  Everything is drawn
on the CPU from a seed so CPU oracle and GPU kernels see identical bits.
"""
import math

import numpy as np
import torch

from oracle import table as otab

BASE_SEED = 1234


def make_scores(n_seg, seg_len, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n_seg, seg_len, generator=g, dtype=torch.float32)


def make_table(B, T, h, w, keep_rate, ksize=3, seed=BASE_SEED, per_clip=False):
    """Returns (scores, kept_idx, table) with selection per slice (default) or per clip."""
    n_seg, seg_len = (B, T * h * w) if per_clip else (B * T, h * w)
    scores = make_scores(n_seg, seg_len, seed)
    k = otab.num_keep(keep_rate, seg_len)
    kept, table = otab.build_table(scores.numpy(), k, h, w, ksize)
    return scores, torch.from_numpy(kept), torch.from_numpy(table)


def make_conv_inputs(n, cin, cout, ksize=3, dtype=torch.float32, seed=BASE_SEED, bias="zero"):
    g = torch.Generator().manual_seed(seed + 7)
    x = torch.randn(n, cin, generator=g, dtype=torch.float32)
    std = math.sqrt(2.0 / (cin * ksize * ksize))
    w_conv = torch.randn(cout, cin, ksize, ksize, generator=g, dtype=torch.float32) * std
    w = w_conv.view(cout, cin, ksize * ksize).permute(2, 1, 0).contiguous()
    if bias == "zero":
        b = torch.zeros(cout)
    else:
        b = torch.randn(cout, generator=g, dtype=torch.float32) * 0.1
    gy = torch.randn(n, cout, generator=g, dtype=torch.float32)
    # round once to the working dtype so oracle and kernels start from the same values
    return tuple(t.to(dtype) for t in (x, w, b, gy))


def f32np(t):
    return t.detach().float().cpu().numpy()
