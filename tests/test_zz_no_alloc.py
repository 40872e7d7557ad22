"""GPU tier, collected last: the entry point for callers that cannot allocate device memory.

``svtad_conv_wgrad_static`` is ``svtad_conv_wgrad`` with the workspace taken from an array built
into the library, for hosts that must not call cudaMalloc once they are running (device memory owned
by the host's own arena, allocation forbidden after start-up).  The test calls it through the C ABI several times in a row - the array is shared and keeps the previous call's contents - and checks every result
against the regular entry point and against the CPU oracle.
"""
import numpy as np
import pytest
import torch

from oracle import conv as oconv
from tests.helpers import f32np, make_conv_inputs, make_table

pytestmark = pytest.mark.gpu


def test_static_workspace_wgrad_matches_regular_entry_point_twice():
    from eccv26_tad_b200 import _lib, ops
    lib = _lib.load()
    assert lib.svtad_static_workspace_bytes() == 32 << 20
    cases = [(2, 40, 0.30, 192, torch.bfloat16, 301), (2, 40, 0.55, 192, torch.bfloat16, 302),
             (1, 8, 0.50, 64, torch.float32, 303)]
    for B, T, keep, C, dtype, seed in cases:
        _, _, table = make_table(B, T, 14, 14, keep, 3, seed)
        n = table.shape[0]
        x, w, b, gy = make_conv_inputs(n, C, C, 3, dtype, seed)
        tc, xc, gc = table.cuda(), x.cuda(), gy.cuda()
        ref_gw, ref_gb = ops.conv_wgrad(gc, xc, tc, 9)
        gw = torch.full((9, C, C), float("nan"), dtype=dtype, device="cuda")
        gb = torch.full((C,), float("nan"), dtype=dtype, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = None
        for call in range(3):                    # calls in a row share the built-in array
            gw.fill_(float("nan")); gb.fill_(float("nan"))
            torch.cuda.synchronize()
            if call >= 1:
                # From the second call on (the first may make the driver load the kernels' code), the device's free
                # memory as the driver reports it must not move: that also sees a cudaMalloc made inside the
                # library, which torch's own counters cannot.
                free_before = torch.cuda.mem_get_info()[0]
            ops.conv_wgrad_static(gc, xc, tc, gw, gb)
            torch.cuda.synchronize()
            if free_before is not None:
                assert torch.cuda.mem_get_info()[0] == free_before, "device memory was allocated during the call"
            assert torch.cuda.memory_allocated() == before          # torch allocated nothing either
            assert torch.equal(gw, ref_gw) and torch.equal(gb, ref_gb)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        egw, egb = oconv.wgrad(f32np(gy), f32np(x), table.numpy(), 9)
        assert oconv.rel_err(f32np(gw), egw) < tol and oconv.rel_err(f32np(gb), egb) < tol
    assert ops.device_error() == 0


def test_static_workspace_rejects_oversized_problems():
    from eccv26_tad_b200 import _lib
    lib = _lib.load()
    n, C = 18880, 1024
    assert lib.svtad_workspace_bytes(_lib.OP_WGRAD, n, C, C, 9, _lib.BF16) > lib.svtad_static_workspace_bytes()
    dummy = torch.zeros(16, device="cuda")
    rc = lib.svtad_conv_wgrad_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), None,
                                     n, C, C, 9, 0, _lib.BF16, None)
    assert rc == _lib.ERR_WORKSPACE and "built-in" in _lib.last_error()
