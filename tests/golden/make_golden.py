"""Generates the golden fixtures in this directory.  Run only where the reference checkout exists:

    python tests/golden/make_golden.py --reference <checkout of pcr-upm/eccv26_tad>

Table fixtures (``table_*.npz``) are outputs of the REFERENCE'S OWN SOURCE TEXT executed on
CPU torch.  The backbone module cannot be imported (it imports mmcv / mmengine / mmaction at
module level), so the three pieces on the table path are cut out of
``opentad/models/backbones/vit_sparse_adapter_poguise.py`` at run time and executed
unchanged:

* ``get_initial_neighbor_indices``  - the method's AST node, compiled as a free function;
* the selection                     - the ``torch.topk`` line and the ``sort`` line of
                                      ``KTPAttention.forward``;
* the gather + remap                - the body of the ``if neighbor_indices is not None``
                                      branch of ``Block._inner_forward`` (between the
                                      ``B, N_prev, _ = x_nonkey.shape`` line and the
                                      ``neighbor_indices = new_flat.view(B, N_new, 9)`` line).

Nothing of that text is written into this repository; only inputs and outputs are stored.

Conv fixtures (``conv_*.npz``) use the dense identity the reference itself relies on for its
``2d_conv`` adapter branch (scatter to the grid -> ``F.conv2d(padding=K//2)`` -> gather,
``vit_sparse_adapter_poguise.py:372-412, 488-490``) with
``w_conv = W.permute(2,1,0).reshape(Cout,Cin,K,K)`` (inverse of
``sparse_conv_layer.py:150-156``), evaluated by torch in float64 with autograd for the
gradients.  The reference op itself is CUDA-only and cannot run where there is no GPU.
"""
import argparse
import ast
import math
import os
import textwrap

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
BACKBONE = os.path.join("opentad", "models", "backbones", "vit_sparse_adapter_poguise.py")


# --------------------------------------------------------------------------- reference text
def _load_reference_pieces(root):
    path = os.path.join(root, BACKBONE)
    src = open(path).read()
    lines = src.splitlines()
    tree = ast.parse(src)

    # (1) get_initial_neighbor_indices as a free function
    init_fn = None
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == "get_initial_neighbor_indices":
            mod = ast.Module(body=[node], type_ignores=[])
            ns = {"torch": torch}
            exec(compile(mod, path, "exec"), ns)
            init_fn = ns["get_initial_neighbor_indices"]
            break
    assert init_fn is not None

    # (2) selection lines
    i_topk = next(i for i, l in enumerate(lines) if "idx_evad = torch.topk(attn_topk" in l)
    i_sort = next(i for i, l in enumerate(lines) if "idx = idx_evad.sort(dim=1)[0]" in l)
    assert 0 < i_sort - i_topk < 4
    select_src = textwrap.dedent("\n".join(lines[i_topk:i_sort + 1]))

    # (3) remap block (first occurrence: Block._inner_forward)
    i_a = next(i for i, l in enumerate(lines) if l.strip() == "B, N_prev, _ = x_nonkey.shape")
    i_b = next(i for i, l in enumerate(lines) if i > i_a and
               l.strip() == "neighbor_indices = new_flat.view(B, N_new, 9)")
    remap_src = textwrap.dedent("\n".join(lines[i_a:i_b + 1]))
    return init_fn, compile(select_src, path + ":select", "exec"), compile(remap_src, path + ":remap", "exec")


def ref_initial(init_fn, h, w, T, B):
    return init_fn(None, h, w, T, torch.device("cpu"), B)


def ref_select(select_code, scores, k):
    ns = {"torch": torch, "attn_topk": scores, "num_keep_tokens": k}
    exec(select_code, ns)
    return ns["idx"]


def ref_remap(remap_code, table, idx, mapping_buffer):
    B, n_prev, _ = table.shape
    n_new = idx.shape[1]
    ns = {
        "torch": torch,
        "x": torch.zeros(1),
        "x_nonkey": torch.zeros(B, n_prev, 1),
        "x_nonkey_keep": torch.zeros(B, n_new, 1),
        "idx_from_topk": idx,
        "neighbor_indices": table,
        "global_mapping_buffer": mapping_buffer,
    }
    exec(remap_code, ns)
    return ns["neighbor_indices"]


# --------------------------------------------------------------------------- fixtures
def make_table_fixtures(root):
    init_fn, select_code, remap_code = _load_reference_pieces(root)
    g = torch.Generator().manual_seed(20261)

    # initial tables
    init = {}
    for name, (h, w, T, B) in {"a": (14, 14, 8, 1), "b": (14, 14, 2, 2), "c": (3, 5, 2, 2),
                               "d": (16, 16, 1, 2), "e": (1, 4, 3, 1)}.items():
        init["shape_" + name] = np.array([h, w, T, B], dtype=np.int64)
        init["table_" + name] = ref_initial(init_fn, h, w, T, B).numpy()
    np.savez_compressed(os.path.join(HERE, "table_init.npz"), **init)

    # selection + successive remap rounds (reference schedule: same rate applied repeatedly)
    chain = {}
    for name, (h, w, T, B, rate, rounds) in {
        "clip": (14, 14, 8, 2, 0.6, 3),      # reference ViT schedule 1568 -> 941 -> 565 -> 339
        "slice": (14, 14, 1, 6, 0.5, 1),     # per-slice selection
        "odd": (5, 7, 3, 3, 0.3, 2),
        "keep10": (14, 14, 1, 4, 0.1, 1),
        "keep55": (14, 14, 2, 2, 0.55, 2),
    }.items():
        table = ref_initial(init_fn, h, w, T, B)
        buf = torch.empty(B * T * h * w, dtype=torch.int32)
        n = T * h * w
        chain[name + "_cfg"] = np.array([h, w, T, B, rounds], dtype=np.int64)
        chain[name + "_rate"] = np.array([rate], dtype=np.float64)
        for r in range(rounds):
            k = min(math.ceil(rate * n), n)
            scores = torch.randn(B, n, generator=g, dtype=torch.float32)
            idx = ref_select(select_code, scores, k)
            table = ref_remap(remap_code, table, idx, buf)
            chain[f"{name}_scores{r}"] = scores.numpy()
            chain[f"{name}_idx{r}"] = idx.numpy()
            chain[f"{name}_table{r}"] = table.numpy()
            n = k
    np.savez_compressed(os.path.join(HERE, "table_chain.npz"), **chain)


def dense_identity(x, kept_pos, w, bias, B, T, h, wd, ksize, gy=None):
    """scatter -> conv2d -> gather in float64.  kept_pos: flat positions in [0, B*T*h*wd)."""
    kk, cin, cout = w.shape
    x = x.clone().requires_grad_(True)
    w = w.clone().requires_grad_(True)
    bias = bias.clone().requires_grad_(True)
    grid = torch.zeros(B * T * h * wd, cin, dtype=torch.float64)
    grid = grid.index_put((kept_pos,), x)
    img = grid.view(B * T, h, wd, cin).permute(0, 3, 1, 2)
    w_conv = w.permute(2, 1, 0).reshape(cout, cin, ksize, ksize)
    out = F.conv2d(img, w_conv, bias, padding=ksize // 2)
    y = out.permute(0, 2, 3, 1).reshape(B * T * h * wd, cout)[kept_pos]
    res = {"y": y.detach().numpy()}
    if gy is not None:
        y.backward(gy)
        res.update(gx=x.grad.numpy(), gw=w.grad.numpy(), gb=bias.grad.numpy())
    return res


def make_conv_fixtures():
    from oracle import table as otab
    g = torch.Generator().manual_seed(20262)
    out = {}
    for name, (B, T, h, wd, cin, cout, ksize, rate) in {
        "k3": (1, 2, 6, 7, 8, 12, 3, 0.5),
        "k3_full": (1, 1, 5, 5, 4, 4, 3, 1.0),
        "k5": (2, 1, 7, 6, 8, 4, 5, 0.4),
        "k3_c16": (2, 2, 14, 14, 16, 16, 3, 0.3),
    }.items():
        n_seg, seg_len = B * T, h * wd
        k = min(math.ceil(rate * seg_len), seg_len)
        scores = torch.randn(n_seg, seg_len, generator=g, dtype=torch.float32)
        kept_idx, table = otab.build_table(scores.numpy(), k, h, wd, ksize)
        kept_pos = torch.from_numpy(
            (kept_idx.astype(np.int64) + np.arange(n_seg)[:, None] * seg_len).reshape(-1))
        n = n_seg * k
        # inputs are rounded to fp32 first so the stored inputs reproduce the stored outputs exactly
        x = torch.randn(n, cin, generator=g, dtype=torch.float64).float()
        w = (torch.randn(ksize * ksize, cin, cout, generator=g, dtype=torch.float64)
             * math.sqrt(2.0 / (cin * ksize * ksize))).float()
        bias = (torch.randn(cout, generator=g, dtype=torch.float64) * 0.1).float()
        gy = torch.randn(n, cout, generator=g, dtype=torch.float64).float()
        res = dense_identity(x.double(), kept_pos, w.double(), bias.double(), B, T, h, wd, ksize, gy.double())
        out[name + "_cfg"] = np.array([B, T, h, wd, cin, cout, ksize, k], dtype=np.int64)
        out[name + "_scores"] = scores.numpy()
        out[name + "_table"] = table
        for key, val in dict(x=x, w=w, bias=bias, gy=gy).items():
            out[f"{name}_{key}"] = val.numpy()
        for key, val in res.items():
            out[f"{name}_{key}"] = val
    np.savez_compressed(os.path.join(HERE, "conv_dense_identity.npz"), **out)


if __name__ == "__main__":
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("SVTAD_REFERENCE_ROOT"),
                    help="root of the reference checkout (default: $SVTAD_REFERENCE_ROOT)")
    a = ap.parse_args()
    if not a.reference:
        ap.error("give --reference or set SVTAD_REFERENCE_ROOT")
    make_table_fixtures(a.reference)
    make_conv_fixtures()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))
