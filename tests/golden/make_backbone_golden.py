"""Generates ``backbone_reference.npz``: outputs of the REFERENCE'S OWN backbone module,
``VisionTransformerSparseAdapterPOGUISE`` (opentad/models/backbones/vit_sparse_adapter_poguise.py), run on CPU on
the small case of ``backbone_case.py``.  Run only where the reference checkout exists:

    python tests/golden/make_backbone_golden.py --reference <checkout of pcr-upm/eccv26_tad>

The reference file is loaded unchanged (importlib, from where it lies).  What it imports from third-party packages
that are absent here is stood in for by the few lines those pieces amount to at inference:

* mmengine ``BaseModule`` / ``ModuleList`` / the three ``*_init`` helpers / the registry decorator - plain
  ``nn.Module`` / ``nn.ModuleList`` / ``nn.init`` calls / identity;
* mmcv ``build_norm_layer`` (LayerNorm with the configured eps), ``DropPath`` (identity at rate 0), ``FFN``
  (Linear - GELU - Linear, no identity branch as the reference asks: ``add_identity=False``), ``PatchEmbed``
  (a Conv3d whose output is flattened slice-major);
* mmaction ``get_sinusoid_encoding`` - the fixed sine / cosine table (this package's ``sinusoid_table``).

The reference's ``SparseConv2d`` (opentad/models/bricks/sparse_conv_layer.py) is loaded unchanged as well; the CUDA
extension it calls, ``opentad_sparse_ops``, is answered on CPU by the conv oracle in float64 (``fwd`` is the only
entry the small-channel forward reaches).  Everything else - token scoring, top-k, gather, table remap, adapter,
schedule, pooling - is the reference's own code.  Nothing of its text is written into this repository; only the
outputs are stored (inputs and weights are seeded, see ``backbone_case.py``).
"""
import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)


def _module(name, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    return m


def install_stand_ins():
    from eccv26_tad_b200.backbone import sinusoid_table

    class BaseModule(nn.Module):
        def __init__(self, init_cfg=None):
            super().__init__()
            self.init_cfg = init_cfg

    class DropPath(nn.Module):
        def __init__(self, drop_prob=0.0):
            super().__init__()
            assert drop_prob == 0.0

        def forward(self, x):
            return x

    class FFN(nn.Module):
        def __init__(self, embed_dims, feedforward_channels, act_cfg=None, ffn_drop=0.0, add_identity=True, **kw):
            super().__init__()
            assert act_cfg["type"] == "GELU" and ffn_drop == 0.0 and not add_identity
            self.layers = nn.Sequential(
                nn.Sequential(nn.Linear(embed_dims, feedforward_channels), nn.GELU(), nn.Dropout(0.0)),
                nn.Linear(feedforward_channels, embed_dims), nn.Dropout(0.0))

        def forward(self, x):
            return self.layers(x)

    class PatchEmbed(nn.Module):
        def __init__(self, in_channels, embed_dims, conv_type, kernel_size, stride, padding, dilation):
            super().__init__()
            assert conv_type == "Conv3d"
            self.projection = nn.Conv3d(in_channels, embed_dims, kernel_size, stride, padding, dilation)

        def forward(self, x):
            x = self.projection(x)
            size = tuple(x.shape[2:])
            return x.flatten(2).transpose(1, 2), size

    def build_norm_layer(cfg, dims):
        assert cfg["type"] == "LN"
        return "ln", nn.LayerNorm(dims, eps=cfg.get("eps", 1e-5))

    def constant_init(module, val, bias=0):
        nn.init.constant_(module.weight, val)
        if getattr(module, "bias", None) is not None:
            nn.init.constant_(module.bias, bias)

    def trunc_normal_init(module, mean=0, std=1, a=-2, b=2, bias=0):
        nn.init.trunc_normal_(module.weight, mean, std, a, b)
        if getattr(module, "bias", None) is not None:
            nn.init.constant_(module.bias, bias)

    def kaiming_init(module, **kw):
        nn.init.kaiming_normal_(module.weight)

    class _Registry:
        def register_module(self, *a, **k):
            return lambda cls: cls

    _module("mmcv")
    _module("mmcv.cnn", build_norm_layer=build_norm_layer)
    _module("mmcv.cnn.bricks", DropPath=DropPath)
    _module("mmcv.cnn.bricks.transformer", FFN=FFN, PatchEmbed=PatchEmbed)
    _module("mmengine")
    _module("mmengine.model", BaseModule=BaseModule, ModuleList=nn.ModuleList)
    _module("mmengine.model.weight_init", constant_init=constant_init, kaiming_init=kaiming_init,
            trunc_normal_init=trunc_normal_init)
    _module("mmengine.registry", MODELS=_Registry())
    _module("mmaction")
    _module("mmaction.models")
    _module("mmaction.models.backbones")
    _module("mmaction.models.backbones.vit_mae",
            get_sinusoid_encoding=lambda n_position, embed_dims: sinusoid_table(n_position, embed_dims))
    _module("mmaction.utils", ConfigType=dict, OptConfigType=dict)

    # the CUDA extension, answered by the oracle (float64 accumulate, rounded once to the input's type)
    from oracle import conv as oconv

    def fwd(x, nbr, w, c_out, tokens_per_batch):
        y = oconv.fwd(x.detach().numpy(), nbr.numpy(), w.detach().numpy(), None, int(tokens_per_batch), acc="f64")
        assert y.shape[1] == c_out
        return torch.from_numpy(np.asarray(y)).to(x.dtype)

    def implicit_gemm_fwd_v2(x, nbr, w, bias, tokens_per_batch):
        b = bias.detach().numpy() if bias.numel() else None
        y = oconv.fwd(x.detach().numpy(), nbr.numpy(), w.detach().numpy(), b, int(tokens_per_batch), acc="f64")
        return torch.from_numpy(np.asarray(y)).to(x.dtype)

    _module("opentad_sparse_ops", fwd=fwd, implicit_gemm_fwd_v2=implicit_gemm_fwd_v2)


def load_reference(root):
    """The reference's wrapper and backbone files under a throw-away package name, so that the backbone's
    ``from ..bricks import SparseConv2d`` finds the reference's own class."""
    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(root, *rel))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod

    _module("refpkg").__path__ = []
    _module("refpkg.backbones").__path__ = []
    wrapper = load("refpkg.bricks_sparse_conv_layer", ("opentad", "models", "bricks", "sparse_conv_layer.py"))
    _module("refpkg.bricks", SparseConv2d=wrapper.SparseConv2d).__path__ = []
    return load("refpkg.backbones.vit_sparse_adapter_poguise",
                ("opentad", "models", "backbones", "vit_sparse_adapter_poguise.py"))


def main(reference_root):
    import backbone_case as case
    from eccv26_tad_b200.backbone import SparseAdapterViT

    install_stand_ins()
    ref_mod = load_reference(reference_root)
    c = case.CFG
    torch.manual_seed(0)
    ref = ref_mod.VisionTransformerSparseAdapterPOGUISE(
        img_size=c["img_size"], patch_size=c["patch_size"], embed_dims=c["embed_dims"], depth=c["depth"],
        num_heads=c["num_heads"], mlp_ratio=c["mlp_ratio"], num_frames=c["num_frames"],
        tubelet_size=c["tubelet_size"], keep_rate=c["keep_rate"], adapter_mlp_ratio=c["adapter_dims"] / c["embed_dims"],
        adapter_index=list(range(c["depth"])), adapter_conv_types=["sparse_conv"] * c["depth"]).eval()

    # weights: drawn under this package's names, loaded into the reference under its own
    mine = SparseAdapterViT(img_size=c["img_size"], patch_size=c["patch_size"], tubelet_size=c["tubelet_size"],
                            num_frames=c["num_frames"], embed_dims=c["embed_dims"], depth=c["depth"],
                            num_heads=c["num_heads"], mlp_ratio=c["mlp_ratio"], adapter_dims=c["adapter_dims"],
                            keep_rates=case.keep_rates(), conv_impl="dense", table_impl="torch")
    shapes = {k: tuple(v.shape) for k, v in mine.state_dict().items()}
    weights = case.seeded_weights(shapes)
    ref_state = {case.to_reference_name(k): v for k, v in weights.items()}
    ref_state["pos_embed"] = ref.state_dict()["pos_embed"]
    missing, unexpected = ref.load_state_dict(ref_state, strict=False)
    assert not missing and not unexpected, (missing, unexpected)

    # what every block hands on: kept grid positions and the running table
    trace = []
    for i, blk in enumerate(ref.blocks):
        def hook(_m, _inp, out, i=i):
            trace.append((i, out[1].clone(), None if out[2] is None else out[2].clone()))
        blk.register_forward_hook(hook)
    with torch.no_grad():
        y, heat = ref(case.video())
    assert heat is None
    out = {"y": y.numpy(), "weights_checksum": np.float64(case.checksum(weights))}
    for i, idx, table in trace:
        if case.keep_rates()[i] < 1:
            out[f"idx_after_block{i}"] = idx.numpy().astype(np.int64)
            out[f"table_after_block{i}"] = table.numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "backbone_reference.npz"), **out)
    print({k: getattr(v, "shape", v) for k, v in out.items()})


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("SVTAD_REFERENCE_ROOT"),
                    help="root of the reference checkout (default: $SVTAD_REFERENCE_ROOT)")
    a = ap.parse_args()
    if not a.reference:
        ap.error("give --reference or set SVTAD_REFERENCE_ROOT")
    main(a.reference)
