"""The small backbone case behind ``backbone_reference.npz``: configuration, seeded inputs and weights, and the
translation between this package's parameter names and the reference model's.  Shared by the fixture generator
(``make_backbone_golden.py``) and by ``tests/test_backbone_reference.py``; test infrastructure only.

The weights are not stored: both sides draw them from one seeded CPU generator, name by name in sorted order, and
the fixture keeps a checksum so that a generator that ever changes shows up as a clear failure, not as a mismatch.
"""
import torch

# depth 12 is what switches on the reference's three-round schedule [1,1,1,r,1,1,r,1,1,r,1,1]
# (opentad/models/backbones/vit_sparse_adapter_poguise.py:1503-1504)
CFG = dict(img_size=32, patch_size=8, tubelet_size=2, num_frames=8, embed_dims=32, depth=12, num_heads=2,
           mlp_ratio=4.0, adapter_dims=8, keep_rate=0.6, batch=2)
SEED = 20263


def keep_rates():
    r = CFG["keep_rate"]
    return [1, 1, 1, r, 1, 1, r, 1, 1, r, 1, 1]


def video():
    g = torch.Generator().manual_seed(SEED + 1)
    return torch.randn(CFG["batch"], 3, CFG["num_frames"], CFG["img_size"], CFG["img_size"], generator=g)


def seeded_weights(shapes):
    """``{name: shape}`` -> ``{name: tensor}``.  Norm scales sit around one, everything else around zero with a
    spread large enough that every branch (attention scores, both projections of the adapter, gamma) matters."""
    g = torch.Generator().manual_seed(SEED)
    out = {}
    for name in sorted(shapes):
        t = torch.randn(tuple(shapes[name]), generator=g)
        if "norm" in name and name.endswith("weight"):
            out[name] = 1.0 + 0.1 * t
        elif name.endswith("gamma"):
            out[name] = 1.0 + 0.2 * t
        elif name.endswith("bias") or name == "cls_token":
            out[name] = 0.1 * t
        else:
            fan_in = t[0].numel() if t.dim() > 1 else t.numel()
            if "sparse_conv.weight" in name:
                fan_in = t.shape[0] * t.shape[1]
            out[name] = t * (1.5 / fan_in ** 0.5)
    return out


def checksum(weights):
    return float(sum(w.double().abs().sum() for _, w in sorted(weights.items())))


def to_reference_name(name):
    """This package's parameter name -> the reference model's (mmcv's PatchEmbed keeps its conv in ``projection``,
    mmcv's FFN keeps its two linears in ``layers.0.0`` and ``layers.1``)."""
    if name.startswith("patch_embed."):
        return name.replace("patch_embed.", "patch_embed.projection.")
    name = name.replace(".mlp.0.", ".mlp.layers.0.0.")
    name = name.replace(".mlp.2.", ".mlp.layers.1.")
    return name
