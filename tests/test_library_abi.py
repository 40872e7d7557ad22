"""CPU tier: the C-ABI library loads, exports every symbol the header declares, and rejects
bad arguments on the host (no kernel is launched by anything in this file)."""
import ctypes
import os
import re

import pytest

from eccv26_tad_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "svtad.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(svtad_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    names = _declared_symbols()
    assert len(names) >= 12
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/svtad.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_error_string():
    lib = _lib.load()
    assert lib.svtad_version() >= 100
    assert isinstance(_lib.last_error(), str)


def test_host_side_validation_returns_codes():
    lib = _lib.load()
    # C_in % 4 != 0 -> same complaint as the reference wrapper (sparse_conv_layer.py:39-42)
    rc = lib.svtad_conv_fwd(None, None, None, None, None, 10, 6, 8, 9, 0, _lib.F32, None, 0, None)
    assert rc == _lib.ERR_UNSUPPORTED and "divisible by 4" in _lib.last_error()
    rc = lib.svtad_conv_fwd(None, None, None, None, None, -1, 8, 8, 9, 0, _lib.F32, None, 0, None)
    assert rc == _lib.ERR_ARG
    rc = lib.svtad_conv_fwd(None, None, None, None, None, 4, 8, 8, 9, 0, 7, None, 0, None)
    assert rc == _lib.ERR_ARG and "dtype" in _lib.last_error()
    rc = lib.svtad_conv_fwd(None, None, None, None, None, 4, 8, 8, 9, 0, _lib.F32, None, 0, None)
    assert rc == _lib.ERR_ARG and "null" in _lib.last_error()
    rc = lib.svtad_conv_wgrad(None, None, None, None, None, 4, 8, 8, 9, 0, _lib.F32, None, 0, None)
    assert rc == _lib.ERR_ARG
    # a bias-gradient pointer at an odd offset is refused before any launch (the kernels store 8 bytes at a time)
    rc = lib.svtad_conv_wgrad(256, 256, 256, 256, 256 + 6, 4, 8, 8, 9, 0, _lib.BF16, 256, 1 << 20, None)
    assert rc == _lib.ERR_ARG and "gb" in _lib.last_error()
    rc = lib.svtad_table_build(None, 4, 196, 300, 14, 14, 3, None, None, None)
    assert rc == _lib.ERR_ARG and "k_keep" in _lib.last_error()
    rc = lib.svtad_table_build(None, 4, 200, 20, 14, 14, 3, None, None, None)
    assert rc == _lib.ERR_ARG
    rc = lib.svtad_table_init(1, 1, 14, 14, 4, None, None)
    assert rc == _lib.ERR_ARG and "odd" in _lib.last_error()
    with pytest.raises(ValueError):
        _lib.check(rc)
    # the one-call backward: something must be asked for, a bias gradient needs the weight gradient
    rc = lib.svtad_conv_bwd(None, None, None, None, None, None, None, 4, 8, 8, 9, 0, _lib.F32, None, None, 0, None)
    assert rc == _lib.ERR_ARG and "neither" in _lib.last_error()
    rc = lib.svtad_conv_bwd(None, None, None, None, 1, None, 1, 4, 8, 8, 9, 0, _lib.F32, None, None, 0, None)
    assert rc == _lib.ERR_ARG and "gb needs gw" in _lib.last_error()
    # fused selection + remap of a later round
    rc = lib.svtad_table_select_remap(None, None, 2, 100, 101, 9, None, None, None, None)
    assert rc == _lib.ERR_ARG and "k_keep" in _lib.last_error()
    rc = lib.svtad_table_select_remap(None, None, 2, 100, 50, 9, None, None, None, None)
    assert rc == _lib.ERR_ARG and "null" in _lib.last_error()
    rc = lib.svtad_table_select_remap(1, 1, 2, 60000, 50, 9, 1, None, 1, None)
    assert rc == _lib.ERR_UNSUPPORTED and "limit" in _lib.last_error()
    assert lib.svtad_table_select_remap(None, None, 0, 100, 50, 9, None, None, None, None) == 0
    assert lib.svtad_workspace_bytes(_lib.OP_BWD, 9440, 192, 192, 9, _lib.BF16) >= \
        lib.svtad_workspace_bytes(_lib.OP_WGRAD, 9440, 192, 192, 9, _lib.BF16) + 9440 * 192 * 4
    # empty problems are fine and touch nothing
    assert lib.svtad_conv_fwd(None, None, None, None, None, 0, 8, 8, 9, 0, _lib.F32, None, 0, None) == 0
    assert lib.svtad_table_init(0, 8, 14, 14, 3, None, None) == 0


def test_workspace_and_path_queries():
    lib = _lib.load()
    assert lib.svtad_workspace_bytes(_lib.OP_FWD, 9440, 192, 192, 9, _lib.BF16) == 0
    w = lib.svtad_workspace_bytes(_lib.OP_WGRAD, 9440, 192, 192, 9, _lib.BF16)
    assert w >= 9 * 192 * 192 * 4
    assert lib.svtad_workspace_bytes(_lib.OP_DGRAD, 100, 192, 192, 9, _lib.BF16) >= 100 * 192 * 4
    assert lib.svtad_path_for(_lib.OP_FWD, 9440, 192, 192, 9, _lib.BF16) == 1
    assert lib.svtad_path_for(_lib.OP_FWD, 784, 192, 192, 9, _lib.F32) == 0
    assert lib.svtad_path_for(_lib.OP_FWD, 784, 48, 48, 9, _lib.BF16) == 0


def test_module_surface_matches_reference():
    import inspect
    import torch
    from eccv26_tad_b200 import SparseConv2d, SparseConv2dFunction
    m = SparseConv2d(8, 12)
    assert tuple(m.weight.shape) == (9, 8, 12) and tuple(m.bias.shape) == (12,)
    assert m.chunk_size == 4096
    assert list(m.state_dict()) == ["weight", "bias"]
    assert SparseConv2d(8, 12, bias=False).bias is None
    assert tuple(SparseConv2d(8, 4, kernel_size=5).weight.shape) == (25, 8, 4)
    sig = inspect.signature(SparseConv2dFunction.forward)
    assert list(sig.parameters) == ["ctx", "x", "neighbor_indices", "weight", "bias", "tokens_per_batch", "chunk_size"]
    with pytest.raises(ValueError):   # no CPU path, loudly
        m(torch.zeros(4, 8), torch.zeros(4, 9, dtype=torch.int32))
    from eccv26_tad_b200 import opentad_sparse_ops as shim
    for name in ("fwd", "bwd_in", "bwd_w", "implicit_gemm_fwd_v2", "implicit_gemm_fwd_v2_chunked"):
        assert callable(getattr(shim, name))


def test_shape_mismatches_raise_before_any_launch():
    import torch
    from eccv26_tad_b200 import ops
    nbr = torch.zeros(5, 9, dtype=torch.int32)
    with pytest.raises(ValueError):
        ops._check_shapes("conv_fwd", 4, 9, nbr)
    with pytest.raises(ValueError):
        ops._check_shapes("conv_wgrad", 5, 9, nbr, grad_output=(torch.zeros(4, 8), 8))
    ops._check_shapes("conv_wgrad", 5, 9, nbr, grad_output=(torch.zeros(5, 8), 8))


def test_static_wgrad_wrapper_checks_shapes_before_the_library_sees_them():
    """conv_wgrad_static cannot copy or allocate, so every mismatch must be refused on the host."""
    import torch
    from eccv26_tad_b200 import ops

    class FakeCuda(torch.Tensor):          # CPU storage that claims to live on the device: nothing is launched
        is_cuda = True

    def t(*shape, dtype=torch.bfloat16):
        return torch.zeros(*shape, dtype=dtype).as_subclass(FakeCuda)

    n, c = 64, 8
    gw, gb = t(9, c, c), t(c)
    nbr = t(n, 9, dtype=torch.int32)
    with pytest.raises(ValueError, match="grad_output"):
        ops.conv_wgrad_static(t(n - 1, c), t(n, c), nbr, gw, gb)
    with pytest.raises(ValueError, match="neighbor table"):
        ops.conv_wgrad_static(t(n, c), t(n, c), t(n - 2, 9, dtype=torch.int32), gw, gb)
    with pytest.raises(ValueError, match="gb must hold"):
        ops.conv_wgrad_static(t(n, c), t(n, c), nbr, gw, t(c + 1))
    with pytest.raises(ValueError, match="gb must hold"):
        ops.conv_wgrad_static(t(n, c), t(n, c), nbr, gw, t(c, dtype=torch.float32))
    with pytest.raises(ValueError, match="16-byte aligned"):
        ops.conv_wgrad_static(t(n, c), t(n, c), nbr, gw, t(c + 3)[3:])


def test_tables_built_by_the_package_are_tagged_symmetric():
    import torch
    from eccv26_tad_b200 import ops
    a = torch.zeros(4, 9, dtype=torch.int32)
    assert not ops.is_known_symmetric(a)
    ops.mark_symmetric(a)
    assert ops.is_known_symmetric(a) and ops.is_known_symmetric(a.view(2, 2, 9))
    a[0, 0] = 1                                       # written to: the tag no longer holds
    assert not ops.is_known_symmetric(a)


def test_legacy_checkpoint_layout_is_remapped_on_load():
    """Weights stored as (C_in, 9, C_out) load into the (9, C_in, C_out) parameter, as with the reference's
    remap_legacy_sparse_conv_weights (opentad/utils/checkpoint.py:44-57)."""
    import torch
    from eccv26_tad_b200 import SparseConv2d, remap_legacy_sparse_conv_weights

    class Adapter(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.sparse_conv = SparseConv2d(8, 12)

    src = Adapter()
    legacy = {k: v.clone() for k, v in src.state_dict().items()}
    legacy["sparse_conv.weight"] = legacy["sparse_conv.weight"].permute(1, 0, 2).contiguous()   # (C_in, 9, C_out)
    assert legacy["sparse_conv.weight"].shape == (8, 9, 12)
    dst = Adapter()
    dst.load_state_dict({k: v.clone() for k, v in legacy.items()})
    assert torch.equal(dst.sparse_conv.weight, src.sparse_conv.weight)
    out = remap_legacy_sparse_conv_weights({k: v.clone() for k, v in legacy.items()}, Adapter().state_dict())
    assert torch.equal(out["sparse_conv.weight"], src.sparse_conv.weight)
    # current-layout checkpoints are left alone
    dst2 = Adapter()
    dst2.load_state_dict(src.state_dict())
    assert torch.equal(dst2.sparse_conv.weight, src.sparse_conv.weight)


def test_reference_wrapper_binds_to_the_shim_when_built():
    """Where ``oracle/_ref`` holds the byte-compiled reference wrapper, executing it with this package's
    ``opentad_sparse_ops`` in place picks the shim up (no JIT build of the reference's CUDA sources) and exposes
    the reference's class with the reference's constructor signature."""
    import inspect
    from oracle import build_ref
    from eccv26_tad_b200 import SparseConv2d, opentad_sparse_ops as shim
    ref = build_ref.load_wrapper(shim)
    if ref is None:
        pytest.skip("oracle/_ref/ref_sparse_conv_layer.bytecode has not been built")
    assert ref.sparse_lib_opt is shim
    theirs = list(inspect.signature(ref.SparseConv2d.__init__).parameters)
    ours = list(inspect.signature(SparseConv2d.__init__).parameters)
    assert ours[:len(theirs)] == theirs
    assert list(ref.SparseConv2d(8, 12).state_dict()) == list(SparseConv2d(8, 12).state_dict())


def test_top_level_opentad_sparse_ops_module():
    """``import opentad_sparse_ops`` (the module the reference wrapper looks for, built by the reference's setup.py as
    a CUDA extension) resolves to this package's callables without any install() call; setup.py ships it as a
    top-level module beside the package."""
    import importlib
    import sys
    sys.modules.pop("opentad_sparse_ops", None)
    mod = importlib.import_module("opentad_sparse_ops")
    from eccv26_tad_b200 import opentad_sparse_ops as shim
    for name in ("fwd", "bwd_in", "bwd_w", "implicit_gemm_fwd_v2", "implicit_gemm_fwd_v2_chunked"):
        assert getattr(mod, name) is getattr(shim, name)
    text = open(os.path.join(ROOT, "setup.py")).read()
    assert 'py_modules=["opentad_sparse_ops"]' in text and "libsvtad.so" in text


def test_concurrency_hint_round_trip_and_clamping():
    """The hint is host state of the library: settable and readable without a GPU, clamped to [1, 16]."""
    lib = _lib.load()
    start = lib.svtad_get_concurrency()
    try:
        assert lib.svtad_set_concurrency(3) == start and lib.svtad_get_concurrency() == 3
        assert lib.svtad_set_concurrency(0) == 3 and lib.svtad_get_concurrency() == 1
        assert lib.svtad_set_concurrency(99) == 1 and lib.svtad_get_concurrency() == 16
    finally:
        lib.svtad_set_concurrency(start)


def test_workspace_sizes_do_not_depend_on_the_concurrency_hint():
    """A workspace sized once must stay valid when the hint changes (svtad_conv_bwd plans its weight gradient for half
    the GPU whatever the caller's hint): svtad_workspace_bytes covers the plan under every hint."""
    lib = _lib.load()
    shapes = [(n, c, kk) for n in (4, 944, 3200, 9440, 17280, 18880, 40000, 226560) for c in (64, 192, 256, 768, 1024)
              for kk in (9, 25)]
    start = lib.svtad_get_concurrency()
    try:
        lib.svtad_set_concurrency(1)
        base = {s: [lib.svtad_workspace_bytes(op, s[0], s[1], s[1], s[2], _lib.BF16) for op in (_lib.OP_WGRAD, _lib.OP_BWD)]
                for s in shapes}
        for hint in (2, 3, 4, 7, 16):
            lib.svtad_set_concurrency(hint)
            for s in shapes:
                got = [lib.svtad_workspace_bytes(op, s[0], s[1], s[1], s[2], _lib.BF16) for op in (_lib.OP_WGRAD, _lib.OP_BWD)]
                assert got == base[s], (hint, s)
    finally:
        lib.svtad_set_concurrency(start)
