"""The backbone restatement against outputs of the REFERENCE'S OWN backbone module
(``VisionTransformerSparseAdapterPOGUISE``, opentad/models/backbones/vit_sparse_adapter_poguise.py), which
``tests/golden/make_backbone_golden.py`` loaded unchanged and ran on CPU: same seeded weights and video, the
reference's three-round schedule, kept positions and neighbor table after every selection round, final output.
"""
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import backbone_case as case                                   # noqa: E402
from eccv26_tad_b200.backbone import SparseAdapterViT          # noqa: E402

GOLD = np.load(os.path.join(HERE, "golden", "backbone_reference.npz"))


def _run(conv_impl, table_impl, device):
    c = case.CFG
    model = SparseAdapterViT(img_size=c["img_size"], patch_size=c["patch_size"], tubelet_size=c["tubelet_size"],
                             num_frames=c["num_frames"], embed_dims=c["embed_dims"], depth=c["depth"],
                             num_heads=c["num_heads"], mlp_ratio=c["mlp_ratio"], adapter_dims=c["adapter_dims"],
                             keep_rates=case.keep_rates(), conv_impl=conv_impl, table_impl=table_impl)
    weights = case.seeded_weights({k: tuple(v.shape) for k, v in model.state_dict().items()})
    assert abs(case.checksum(weights) - float(GOLD["weights_checksum"])) < 1e-6 * float(GOLD["weights_checksum"]), \
        "the seeded generator no longer reproduces the weights the fixture was made with"
    model.load_state_dict(weights, strict=True)
    model = model.to(device).eval()
    trace = {}
    for i, blk in enumerate(model.blocks):
        blk.register_forward_hook(lambda _m, _i, out, i=i: trace.__setitem__(i, (out[1], out[2])))
    with torch.no_grad():
        y = model(case.video().to(device))
    return y.cpu().numpy(), trace


def _check(y, trace, with_table):
    for i, r in enumerate(case.keep_rates()):
        if r < 1:
            idx, table = trace[i]
            np.testing.assert_array_equal(idx.cpu().numpy(), GOLD[f"idx_after_block{i}"])
            if with_table:
                np.testing.assert_array_equal(table.cpu().numpy().reshape(GOLD[f"table_after_block{i}"].shape),
                                              GOLD[f"table_after_block{i}"])
    ref = GOLD["y"]
    assert y.shape == ref.shape
    assert np.abs(y - ref).max() <= 2e-4 * np.abs(ref).max()


def test_dense_torch_path_matches_reference_module_on_cpu():
    y, trace = _run("dense", "torch", "cpu")
    _check(y, trace, with_table=False)


@pytest.mark.gpu
@pytest.mark.parametrize("table_impl", ["svtad", "torch"])
def test_sparse_path_matches_reference_module(table_impl):
    y, trace = _run("svtad", table_impl, "cuda")
    _check(y, trace, with_table=True)
