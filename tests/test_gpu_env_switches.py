"""GPU tier: every environment switch of the library that selects a different plan or kernel is run against the
oracle, so that no code path sits untested behind a variable.  Switches that the library reads on every call are set
with monkeypatch; switches it reads once per process run in a child process."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import conv as oconv
from tests.helpers import BASE_SEED, f32np, make_conv_inputs, make_table

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ops():
    from eccv26_tad_b200 import ops
    return ops


def _wgrad_case():
    _, _, table = make_table(2, 20, 14, 14, 0.3, 3, BASE_SEED + 9)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 192, 192, 3, torch.bfloat16, BASE_SEED + 9, bias="random")
    return table, x, w, gy


@pytest.mark.parametrize("name,value", [("SVTAD_TC_WGRAD_SPLITS", "1"), ("SVTAD_TC_WGRAD_SPLITS", "3"),
                                        ("SVTAD_TC_WGRAD_SPLITS", "7"), ("SVTAD_TC_WGRAD_BN", "64"),
                                        ("SVTAD_TC_WGRAD_BN", "192")])
def test_weight_gradient_plan_overrides(name, value, monkeypatch):
    ops = _ops()
    table, x, w, gy = _wgrad_case()
    egw, egb = oconv.wgrad(f32np(gy), f32np(x), table.numpy(), 9)
    monkeypatch.setenv(name, value)
    gw, gb = ops.conv_wgrad(gy.cuda(), x.cuda(), table.cuda(), 9)
    torch.cuda.synchronize()
    assert oconv.rel_err(f32np(gw), egw) < 2e-2 and oconv.rel_err(f32np(gb), egb) < 2e-2
    assert ops.device_error() == 0


def test_generic_fp32_forward_kernel(monkeypatch):
    """SVTAD_SIMT_FWD_GENERIC=1 sends the fp32 forward to the shape-generic CUDA-core kernel instead of the
    pipelined one; both must meet the fp32 bound."""
    ops = _ops()
    _, _, table = make_table(1, 8, 14, 14, 0.5, 3, BASE_SEED + 1)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 192, 192, 3, torch.float32, BASE_SEED + 1, bias="random")
    ref = oconv.fwd(f32np(x), table.numpy(), f32np(w), f32np(b))
    y_fast = ops.conv_fwd(x.cuda(), table.cuda(), w.cuda(), b.cuda())
    monkeypatch.setenv("SVTAD_SIMT_FWD_GENERIC", "1")
    y_gen = ops.conv_fwd(x.cuda(), table.cuda(), w.cuda(), b.cuda())
    torch.cuda.synchronize()
    assert oconv.rel_err(f32np(y_fast), ref) < 1e-5 and oconv.rel_err(f32np(y_gen), ref) < 1e-5


_CHILD = r"""
import ctypes, sys, torch, numpy as np
sys.path.insert(0, %(root)r)
from eccv26_tad_b200 import _lib, ops
from eccv26_tad_b200.distributed import padded_numel
from oracle import conv as oconv
from tests.helpers import BASE_SEED, f32np, make_conv_inputs, make_table
lib = _lib.load()
mode = sys.argv[1]
if mode == "allreduce":
    world, numel = 4, 995904
    n_pad = padded_numel(numel, world)
    stage = lib.svtad_allreduce_stage_bytes(n_pad) // 2
    g = torch.Generator().manual_seed(3)
    vals = [torch.randn(numel, generator=g).bfloat16() for _ in range(world)]
    bufs = []
    for v in vals:
        b = torch.zeros(n_pad + stage, dtype=torch.bfloat16, device="cuda"); b[:numel].copy_(v); bufs.append(b)
    ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    epochs = torch.zeros(lib.svtad_allreduce_epoch_bytes() // 4, dtype=torch.int32, device="cuda")
    for call in range(2):
        _lib.check(lib.svtad_allreduce_sum_emulated(ptrs, world, n_pad, _lib.BF16, n_pad * 2, epochs.data_ptr(), 0,
                                                    torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        acc = torch.zeros(numel)
        for v in vals:
            acc += v.float()
        want = acc.bfloat16().cuda()
        assert all(torch.equal(b[:numel], want) for b in bufs)
        vals = [want.cpu()] * world                 # the buckets now hold the sums: the next call sums those
else:
    _, _, table = make_table(2, 12, 14, 14, 0.3, 3, 33)
    n = table.shape[0]
    x, w, b, gy = make_conv_inputs(n, 192, 192, 3, torch.bfloat16, 33)
    tc, xc, wc, gc = (t.cuda() for t in (table, x, w, gy))
    gx, gw, gb = ops.conv_bwd(gc, xc, tc, wc, assume_symmetric=True)
    gx0 = ops.conv_dgrad(gc, tc, wc, assume_symmetric=True)
    gw0, gb0 = ops.conv_wgrad(gc, xc, tc, 9)
    torch.cuda.synchronize()
    # one stream, one kernel at a time: the same plans as the separate calls, so bit-identical
    assert torch.equal(gx, gx0) and torch.equal(gw, gw0) and torch.equal(gb, gb0)
    egw, _ = oconv.wgrad(f32np(gy), f32np(x), table.numpy(), 9)
    assert oconv.rel_err(f32np(gw), egw) < 2e-2
assert ops.device_error() == 0
print("child ok")
"""


def _run_child(mode, env):
    e = dict(os.environ, **env)
    r = subprocess.run([sys.executable, "-c", _CHILD % {"root": ROOT}, mode], cwd=ROOT, env=e, capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0 and "child ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("env", [{"SVTAD_ALLREDUCE_CTAS": "16"}, {"SVTAD_ALLREDUCE_CTAS": "3", "SVTAD_ALLREDUCE_BACKOFF_NS": "200"}])
def test_exchange_kernel_switches(env):
    """CTA cap and poll back-off of the exchange kernel (read once per process): exact sums, twice in a row."""
    _run_child("allreduce", env)


def test_backward_without_the_side_stream():
    """SVTAD_OVERLAP_BACKWARD=0 (read once per process): the one-call backward runs its two kernels one after the
    other on the caller's stream and equals the separate calls bit for bit."""
    _run_child("bwd", {"SVTAD_OVERLAP_BACKWARD": "0"})
