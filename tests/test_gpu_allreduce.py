"""GPU tier: the two-shot gradient all-reduce (csrc/allreduce.cu) through the C ABI on ONE GPU.

With fewer GPUs than ranks the ranks cannot run as separate launches that wait for one another, so
``svtad_allreduce_sum_emulated`` runs every rank's part of the same protocol in one cooperative launch over local
buffers.  The wait limit is exercised with the real entry point and a peer that never shows up: the kernel must give
up after the limit, report through the device error word, and leave the context usable.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(world, numel, dtype, seed):
    from eccv26_tad_b200 import _lib
    from eccv26_tad_b200.distributed import padded_numel
    lib = _lib.load()
    n_pad = padded_numel(numel, world)
    flag_elems = lib.svtad_allreduce_stage_bytes(n_pad) // 2
    g = torch.Generator().manual_seed(seed)
    bufs, vals = [], []
    for r in range(world):
        b = torch.zeros(n_pad + flag_elems, dtype=dtype, device="cuda")
        v = torch.randn(numel, generator=g).to(dtype)
        b[:numel].copy_(v)
        bufs.append(b)
        vals.append(v)
    return lib, _lib, n_pad, bufs, vals


def _expected(vals, dtype):
    acc = torch.zeros_like(vals[0], dtype=torch.float32)
    for v in vals:                       # rank order, fp32, one rounding: exactly what the kernel does
        acc += v.float()
    return acc.to(dtype)


@pytest.mark.parametrize("world,numel,dtype", [(2, 995904, torch.bfloat16), (8, 995904, torch.bfloat16),
                                               (4, 1000, torch.float16), (3, 64 * 3, torch.bfloat16)])
def test_emulated_ranks_sum_bit_exactly_and_repeatedly(world, numel, dtype):
    lib, _lib, n_pad, bufs, vals = _setup(world, numel, dtype, 5 + world)
    epochs = torch.zeros(lib.svtad_allreduce_epoch_bytes() // 4, dtype=torch.int32, device="cuda")
    ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    code = _lib.BF16 if dtype == torch.bfloat16 else _lib.F16
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(3):                # the flags carry the call number: nothing is reset between calls
        if call:
            g = torch.Generator().manual_seed(100 * call + world)
            vals = [torch.randn(numel, generator=g).to(dtype) for _ in range(world)]
            for b, v in zip(bufs, vals):
                b[:numel].copy_(v)
        _lib.check(lib.svtad_allreduce_sum_emulated(ptrs, world, n_pad, code, n_pad * 2, epochs.data_ptr(), 0, stream))
        torch.cuda.synchronize()
        want = _expected(vals, dtype).cuda()
        for b in bufs:
            assert torch.equal(b[:numel], want)
            assert float(b[numel:n_pad].float().abs().sum()) == 0          # padding stays zero
    from eccv26_tad_b200 import ops
    assert ops.device_error() == 0


def test_wait_for_an_absent_peer_runs_out_and_reports():
    """Rank 0 of a two-rank exchange whose rank 1 never launches: the flag that nothing sets makes the first wait run
    out after the (short) limit; the kernel reports code 71, leaves the bucket as it was, and the GPU keeps working."""
    from eccv26_tad_b200 import ops
    lib, _lib, n_pad, bufs, vals = _setup(2, 4096, torch.bfloat16, 9)
    epoch = torch.zeros(lib.svtad_allreduce_epoch_bytes() // 4, dtype=torch.int32, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
    before = bufs[0][:4096].clone()
    limit = 2_000_000                    # about a millisecond of SM clock
    _lib.check(lib.svtad_allreduce_sum(ptrs, 0, 2, n_pad, _lib.BF16, n_pad * 2, epoch.data_ptr(), limit,
                                       torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert ops.device_error() == 71
    assert ops.device_error() == 0                       # reading clears it
    assert torch.equal(bufs[0][:4096], before)
    assert int(epoch.abs().sum()) == 0                   # the call did not count
    # the context is intact: an ordinary exchange (all ranks emulated) still works afterwards
    for b in bufs:
        b[n_pad:].zero_()
    epochs = torch.zeros(lib.svtad_allreduce_epoch_bytes() // 4, dtype=torch.int32, device="cuda")
    _lib.check(lib.svtad_allreduce_sum_emulated(ptrs, 2, n_pad, _lib.BF16, n_pad * 2, epochs.data_ptr(), 0,
                                                torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(bufs[0][:4096], _expected(vals, torch.bfloat16).cuda())
    assert ops.device_error() == 0


def test_bad_arguments_are_refused_on_the_host():
    from eccv26_tad_b200 import _lib
    lib = _lib.load()
    buf = torch.zeros(16384, dtype=torch.bfloat16, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(buf.data_ptr(), buf.data_ptr())
    ep = torch.zeros(lib.svtad_allreduce_epoch_bytes() // 4, dtype=torch.int32, device="cuda")
    assert lib.svtad_allreduce_sum(ptrs, 0, 2, 100, _lib.BF16, 4096, ep.data_ptr(), 0, None) == _lib.ERR_ARG      # not a multiple of 16
    assert lib.svtad_allreduce_sum(ptrs, 2, 2, 1024, _lib.BF16, 4096, ep.data_ptr(), 0, None) == _lib.ERR_ARG     # rank out of range
    assert lib.svtad_allreduce_sum(ptrs, 0, 2, 1024, _lib.F32, 4096, ep.data_ptr(), 0, None) == _lib.ERR_ARG      # 16-bit only
    assert lib.svtad_allreduce_sum(ptrs, 0, 2, 1024, _lib.BF16, 1024, ep.data_ptr(), 0, None) == _lib.ERR_ARG     # staging inside the bucket
    assert lib.svtad_allreduce_sum(ptrs, 0, 1, 1024, _lib.BF16, 4096, ep.data_ptr(), 0, None) == 0                # one rank: nothing to do
