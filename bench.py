#!/usr/bin/env python
"""SparseConv2D benchmark: retained tokens/s through forward + backward at keep 10/30/55 %.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the headline metric is quoted on): bf16 activations and weights with
fp32 accumulate, batch 2, T=80 slices of a 14x14 token grid, C_in = C_out = 192, 3x3 taps, kept
tokens chosen per slice as the top-k of N(0,1) scores at keep {10, 30, 55} % (3200 / 9440 / 17280
retained tokens), features and upstream gradients N(0,1), Kaiming-normal weights.  One "step" runs
forward, input gradient, weight + bias gradient for all three keep rates on one batch
(29 920 retained tokens per GPU).  Data are synthetic and seeded; there is no dataset behind
this op.  With N > 1 every rank owns its own batch (weak scaling, sharded by clip) and the
weight / bias gradients are all-reduced over NCCL every step, as data-parallel training does
(by this library's own two-shot exchange over NVLink peer memory; SVTAD_BENCH_ALLREDUCE=nccl: NCCL all-reduce).

Numbers on the JSON line
  value        tokens/s over all ranks with inputs already resident in HBM; every step reads a
               different one of R input sets whose total size exceeds the L2, steps replayed as
               CUDA graphs, timed with CUDA events, max over ranks
  e2e          same metric through the public Python surface (build_neighbor_table + SparseConv2d
               forward / backward under autograd) with HOST buffers: every step copies scores,
               features and upstream gradients from pinned host memory and copies the outputs and
               all gradients back; the three keep rates run as three layers on three streams, so
               copies in, kernels and copies out of different layers overlap; the calls of a step are
               captured into a CUDA graph per input set and replayed (eager if capture fails)
  roofline     the dominant kernel (largest share of device time among forward / dgrad / wgrad),
               dense-equivalent FLOPs 2*N*KK*Cin*Cout per launch over its CUDA-event duration,
               against the measured bf16 peak in MEASURED_PEAKS.json (fallback 1590 TFLOP/s)
  cpu_baseline the CPU oracle port (C, OpenMP, fp32 accumulate) timed on the host cores on a
               bounded sample of the same workload (rank 0, N = 1 only)

``--impl reference`` times that CPU port alone (the reference has no CPU implementation of this
op; its CUDA path is reported under ``reference_cuda`` on the main line when the prebuilt
extension under oracle/_ref/ is present).
"""
import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

KEEPS = (0.10, 0.30, 0.55)
B, T, H, W, C, KS = 2, 80, 14, 14, 192, 3
KK = KS * KS
N_SETS = 8
FALLBACK_TFLOPS = 1590.0
FALLBACK_HBM = 6650.0
METRIC = "SparseConv2D retained tokens/sec fwd+bwd at keep 10-55%"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu captures summarised under profiles/
# (the benchmark's largest layer: 17 280 rows, C=192), divided by the rows of that launch; traffic grows in
# proportion to the rows
NCU_DRAM_BYTES_PER_ROW = {"fwd": 7.97e6 / 17280, "dgrad": 7.97e6 / 17280, "wgrad": 13.93e6 / 17280}


def flops_pass(n):
    return 2.0 * n * KK * C * C


def num_keep(rate, L):
    return max(0, min(int(math.ceil(rate * L)), L))


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d.get("bf16_tflops", FALLBACK_TFLOPS)), float(d.get("hbm_gbs", FALLBACK_HBM)), "measured"
    return FALLBACK_TFLOPS, FALLBACK_HBM, "fallback"


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed regions run."""

    def __init__(self, device):
        super().__init__(daemon=True)
        self.samples = []
        self.active = False
        self.stop_flag = False
        self.ok = False
        self.max_mhz = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(device).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device.index or 0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            pass

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self.stop_flag:
            if self.active:
                try:
                    mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                    try:
                        reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                    except Exception:
                        reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                    self.samples.append((mhz, reasons))
                except Exception:
                    pass
                time.sleep(0.002)
            else:
                time.sleep(0.005)

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        nv = self.nv
        mhz = sorted(s[0] for s in self.samples)
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        seen = [k for k, bit in names.items() if any(s[1] & bit for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": seen,
                "samples": len(mhz)}


# ------------------------------------------------------------------------------------------ data
def make_host_sets(rank, n_sets, slices=B * T):
    """Seeded CPU tensors: per set and keep rate the scores, features and upstream gradients."""
    import torch
    g = torch.Generator().manual_seed(1234 + 2 + 1000 * rank)
    sets = []
    for s in range(n_sets):
        per_keep = []
        for r in KEEPS:
            k = num_keep(r, H * W)
            n = slices * k
            per_keep.append({
                "k": k, "n": n,
                "scores": torch.randn(slices, H * W, generator=g, dtype=torch.float32),
                "x": torch.randn(n, C, generator=g, dtype=torch.float32).bfloat16(),
                "gy": torch.randn(n, C, generator=g, dtype=torch.float32).bfloat16(),
            })
        sets.append(per_keep)
    std = math.sqrt(2.0 / (C * KK))
    w_conv = torch.randn(C, C, KS, KS, generator=torch.Generator().manual_seed(77), dtype=torch.float32) * std
    weight = w_conv.view(C, C, KK).permute(2, 1, 0).contiguous()
    return sets, weight, torch.zeros(C)


# ------------------------------------------------------------------------------------------ CPU arm
def cpu_port_run(steps, warmup, slices):
    """Times the C/OpenMP oracle port (fp32 accumulate) on `slices` slices per keep rate."""
    import torch
    from oracle import conv as oconv
    from oracle import table as otab
    sets, weight, bias = make_host_sets(0, 1, slices)
    wf = weight.bfloat16().float().numpy()
    bf = bias.numpy()
    work = []
    tokens = 0
    for item in sets[0]:
        kept, table = otab.build_table(item["scores"].numpy(), item["k"], H, W, KS)
        work.append((item["x"].float().numpy(), item["gy"].float().numpy(), table))
        tokens += item["n"]

    def step():
        for x, gy, table in work:
            oconv.fwd(x, table, wf, bf, acc="f32")
            oconv.dgrad(gy, table, wf, acc="f32")
            oconv.wgrad(gy, x, table, KK, acc="f32")

    cores = oconv.set_threads(len(os.sched_getaffinity(0)))   # all host cores, whatever OMP_NUM_THREADS says
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    return tokens * steps / dt, dt / steps * 1e3, cores, tokens


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    slices = 40   # a quarter of the workload's 160 slices per step
    value, ms, cores, tokens = cpu_port_run(args.steps, args.warmup, slices)
    sample = (f"{slices} of {B * T} slices per keep rate ({tokens} retained tokens per step), "
              f"C oracle port of the kernel math, OpenMP over {cores} threads; the reference has no CPU path")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "run": {"note": "CPU port, bounded sample"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(n_gpus):
    cfg = {
        "workload": "SparseConv2D fwd+bwd bf16 (fp32 accumulate): batch 2 x T=80 slices x 14x14 grid per GPU, "
                    "Cin=Cout=192, 3x3, keep sweep {10,30,55}% by per-slice top-k",
        "tokens_per_step_per_gpu": sum(B * T * num_keep(r, H * W) for r in KEEPS),
        "keep_rates": list(KEEPS),
        "parallelism": f"dp{n_gpus} (sharded by clip; one all-reduce of the weight/bias gradient bucket per step)" if n_gpus > 1 else "single GPU",
        "l2": f"inputs larger than L2: every step reads a different one of {N_SETS} resident input sets (~{N_SETS * 47} MB > 126 MB)",
    }
    return cfg


# ------------------------------------------------------------------------------------------ GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying CUDA graphs")
    ap.add_argument("--layer-streams", type=int, default=1, choices=[0, 1],
                    help="1 (default): the step's three layers (keep rates), which do not depend on one another, run on "
                         "three streams; 0: one after the other")
    ap.add_argument("--concurrency", default="3,2,2",
                    help="svtad_set_concurrency hints for the step, one per layer in the order of the keep rates (the "
                         "three layers run on streams of their own; the layers that carry more of the work are planned "
                         "for a larger share of the GPU), or one number for all; 1 plans every kernel for the whole GPU")
    ap.add_argument("--wgrad-concurrency", default=None,
                    help="hints for the weight-gradient kernels if they are to differ from --concurrency "
                         "(default: 4,3,3 in the N > 1 order, where they are issued first)")
    ap.add_argument("--ar-per-layer", type=int, default=0, choices=[0, 1],
                    help="N > 1: 1 = one gradient bucket per layer, exchanged while the other layers still compute")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-ref-cuda", action="store_true")
    ap.add_argument("--workload", default="sparseconv", choices=["sparseconv", "backbone", "configs"],
                    help="backbone: forward of the ViT-B sparse-adapter backbone on 160-frame clips (secondary line); "
                         "configs: the other benchmark configurations (--configs 1,3,4), one JSON line each")
    ap.add_argument("--configs", default="1,3,4")
    ap.add_argument("--backbone-schedule", default="primary", choices=["primary", "reference"],
                    help="primary: 30 %% keep after block 3 only; reference: the reference's ViT-B schedule, keep 0.6 after "
                         "blocks 3, 6 and 9 (vit_sparse_adapter_poguise.py:1503-1504)")
    ap.add_argument("--backbone-train", action="store_true",
                    help="with --workload backbone: one training step (forward, backward to the adapters, AdamW) per step")
    ap.add_argument("--kernel-case", default=None, choices=["fwd", "dgrad", "wgrad", "table"],
                    help="profiling aid: launch only this kernel a few times on --case-slices slices and exit")
    ap.add_argument("--case-slices", type=int, default=3840)
    ap.add_argument("--case-keep", type=float, default=0.30)
    ap.add_argument("--case-launches", type=int, default=4)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.kernel_case:
        return kernel_case(args)
    if args.workload == "backbone":
        return backbone_case(args)
    if args.workload == "configs":
        return configs_case(args)
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist
    from eccv26_tad_b200 import SparseConv2d, build_neighbor_table, ops
    from eccv26_tad_b200.distributed import allreduce_weight_grads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sampler = ClockSampler(dev)
    sampler.start()

    host_sets, weight_h, bias_h = make_host_sets(rank, N_SETS)
    weight = weight_h.bfloat16().to(dev)
    bias = bias_h.bfloat16().to(dev)
    tokens_step = sum(it["n"] for it in host_sets[0])

    # resident device sets: table built once per set by the CUDA builder, inputs and outputs preallocated
    dsets = []
    for per_keep in host_sets:
        dk = []
        for it in per_keep:
            scores = it["scores"].to(dev)
            kept, table = build_neighbor_table(scores, num_keep=it["k"], h=H, w=W, kernel_size=KS)
            dk.append({"n": it["n"], "table": table, "x": it["x"].to(dev), "gy": it["gy"].to(dev)})
        dsets.append(dk)
    lib = ops._lib.load()
    code = ops._lib.BF16
    ws_bytes = max(lib.svtad_workspace_bytes(ops._lib.OP_WGRAD, it["n"], C, C, KK, code) for it in host_sets[0])
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    n_max = max(it["n"] for it in host_sets[0])
    y_buf = torch.empty(n_max, C, dtype=torch.bfloat16, device=dev)
    gx_buf = torch.empty(n_max, C, dtype=torch.bfloat16, device=dev)
    LAUNCHES_PER_LAYER = 4   # fwd, dgrad, wgrad partials (bias row included), reduce
    # Gradient buckets (gw ++ gb per layer).  N > 1: they live in peer-mapped memory and are summed by
    # svtad_allreduce_sum (two-shot exchange by plain stores over NVLink that carry their own flags, bounded waits,
    # small CTAs that fit beside the compute kernels' CTAs); SVTAD_BENCH_ALLREDUCE=nccl keeps ordinary tensors +
    # NCCL.  The ranks decide together (one collective vote) before any set-up call; a "no" puts all of them on
    # NCCL.  --ar-per-layer 1: one bucket per layer, exchanged as soon as that layer's weight gradient is done, the
    # way DDP overlaps its bucket all-reduces with the rest of the backward (reference: src/eccv26_tad.py:288-300);
    # 0: one bucket for the step, exchanged at its end.  All exchanges go to ONE stream in layer order, so every
    # rank issues them in the same order.
    per_layer = KK * C * C + C
    from eccv26_tad_b200.distributed import GradBucket
    want_peer = os.environ.get("SVTAD_BENCH_ALLREDUCE", "peer") != "nccl"
    exch = "peer" if want_peer else "collective"
    if args.ar_per_layer:
        buckets = [GradBucket(per_layer, torch.bfloat16, dev, exchange=exch) for _ in KEEPS]
        gw_bufs = [b.buffer[:KK * C * C] for b in buckets]
        gb_bufs = [b.buffer[KK * C * C:per_layer] for b in buckets]
    else:
        buckets = [GradBucket(len(KEEPS) * per_layer, torch.bfloat16, dev, exchange=exch)]
        grads = buckets[0].buffer
        gw_bufs = [grads[i * per_layer:i * per_layer + KK * C * C] for i in range(len(KEEPS))]
        gb_bufs = [grads[i * per_layer + KK * C * C:(i + 1) * per_layer] for i in range(len(KEEPS))]
    allreduce_kind = buckets[0].kind
    if world > 1 and want_peer and buckets[0].kind == "nccl":
        sys.stderr.write(f"[bench] peer-memory all-reduce unavailable ({getattr(buckets[0], 'fallback_reason', '?')}); using NCCL\n")
    comm = torch.cuda.Stream(device=dev, priority=-1 if (world > 1 and os.environ.get("SVTAD_BENCH_STREAM_PRIORITY", "1") != "0") else 0)
    gw_buf, gb_buf = gw_bufs[0], gb_bufs[0]
    launches_per_step = 0

    # every layer (keep rate) has its own outputs and workspace, so the three layers of a step - which do not
    # depend on one another - may run on streams of their own (--layer-streams 1)
    y_bufs = [torch.empty(it["n"], C, dtype=torch.bfloat16, device=dev) for it in host_sets[0]]
    gx_bufs = [torch.empty(it["n"], C, dtype=torch.bfloat16, device=dev) for it in host_sets[0]]
    ws_l = [torch.empty(ws_bytes, dtype=torch.uint8, device=dev) for _ in KEEPS]
    # With N > 1 the weight gradients and the exchange that follows them are the step's critical path (everything
    # else only has to be done by the end of the step), so their streams get the higher priority: their CTAs are
    # placed first whenever an SM has room, and the exchange starts early enough to hide behind forward / dgrad.
    hi = -1 if (world > 1 and os.environ.get("SVTAD_BENCH_STREAM_PRIORITY", "1") != "0") else 0
    sides = [torch.cuda.Stream(device=dev, priority=hi) for _ in KEEPS]
    lanes = [torch.cuda.Stream(device=dev) for _ in KEEPS]

    def raw_step(dk, stream=None, count=False):
        """One step through the C ABI on resident buffers: 3 keep rates x (fwd, dgrad, wgrad+bias).  The passes of a
        layer are independent of one another here (the upstream gradient is an input), so the weight gradient runs
        on a side stream next to forward and input gradient.  With N > 1 the weight gradients are issued first and
        the all-reduce of their bucket follows them on a stream of its own, so that - as under DDP - the exchange
        runs while the rest of the step still computes."""
        nl = 0
        cur = torch.cuda.current_stream()
        early_wgrad = wgrad_first

        def wgrad(li, it, st):
            ops.set_concurrency(wgrad_hints[li])
            ops._lib.check(lib.svtad_conv_wgrad(it["gy"].data_ptr(), it["x"].data_ptr(), it["table"].data_ptr(),
                                                gw_bufs[li].data_ptr(), gb_bufs[li].data_ptr(), it["n"], C, C, KK, 0, code,
                                                ws_l[li].data_ptr(), ws_bytes, st.cuda_stream))

        order = list(range(len(dk)))
        if early_wgrad:
            order = order[::-1]          # the layer with the most rows first: its chain is the longest
        if early_wgrad:
            for li in order:
                it = dk[li]
                sides[li].wait_stream(cur)
                wgrad(li, it, sides[li])
                comm.wait_stream(sides[li])
            with torch.cuda.stream(comm):
                buckets[0].all_reduce()
            nl += 1 if world > 1 else 0
        for li in order:
            it = dk[li]
            n = it["n"]
            main = lanes[li] if args.layer_streams else cur
            side = sides[li]
            if args.layer_streams:
                main.wait_stream(cur)
            ops.set_concurrency(layer_hints[li])
            ops._lib.check(lib.svtad_conv_fwd(it["x"].data_ptr(), it["table"].data_ptr(), weight.data_ptr(),
                                              bias.data_ptr(), y_bufs[li].data_ptr(), n, C, C, KK, 0, code, None, 0,
                                              main.cuda_stream))
            if not early_wgrad:
                side.wait_stream(main)
                wgrad(li, it, side)
            ops._lib.check(lib.svtad_conv_dgrad(it["gy"].data_ptr(), it["table"].data_ptr(), weight.data_ptr(),
                                                gx_bufs[li].data_ptr(), n, C, C, KK, 0, code, None, None, 0,
                                                main.cuda_stream))
            if world > 1 and args.ar_per_layer:
                comm.wait_stream(side)
                with torch.cuda.stream(comm):
                    buckets[li].all_reduce()
                nl += 1
            if not early_wgrad:
                main.wait_stream(side)
            nl += LAUNCHES_PER_LAYER
        if args.layer_streams:
            for li in range(len(dk)):
                cur.wait_stream(lanes[li])
        if early_wgrad or (world > 1 and args.ar_per_layer):
            cur.wait_stream(comm)
        elif world > 1:
            buckets[0].all_reduce()
            nl += 1
        ops.set_concurrency(hint)
        return nl

    # The three layers of a step run side by side, so the kernels are planned for a share of the GPU each
    # (svtad_set_concurrency; workspace sizes do not depend on the hint).
    layer_hints = [max(1, int(v)) for v in str(args.concurrency).split(",")]
    if len(layer_hints) == 1:
        layer_hints = layer_hints * len(KEEPS)
    if len(layer_hints) != len(KEEPS) or not args.layer_streams:
        layer_hints = [1] * len(KEEPS)
    # With N > 1 the weight gradients are issued first (see raw_step) and run beside all three forwards: measured
    # best when they are planned a little leaner than forward / dgrad (0.0782 against 0.0807 ms per step on one GPU
    # in that order).  In the N = 1 order they share the layer's hint.
    wgrad_first = (world > 1 and not args.ar_per_layer and bool(args.layer_streams)
                   and os.environ.get("SVTAD_BENCH_EARLY_WGRAD", "1") != "0")
    wgrad_hints = layer_hints
    wg_arg = args.wgrad_concurrency or ("4,3,3" if wgrad_first and str(args.concurrency) == "3,2,2" else None)
    if wg_arg and args.layer_streams:
        wgrad_hints = [max(1, int(v)) for v in str(wg_arg).split(",")]
        if len(wgrad_hints) == 1:
            wgrad_hints = wgrad_hints * len(KEEPS)
        if len(wgrad_hints) != len(KEEPS):
            wgrad_hints = layer_hints
    hint = max(layer_hints)            # what stays set between the step's own calls
    ops.set_concurrency(hint)
    stream = torch.cuda.Stream(device=dev)
    graphs = None
    with torch.cuda.stream(stream):
        for s in range(min(3, N_SETS)):
            launches_per_step = raw_step(dsets[s])
        stream.synchronize()
        if not args.no_graph:
            try:
                graphs = []
                for s in range(N_SETS):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        raw_step(dsets[s])
                    graphs.append(g)
            except Exception as e:   # stay measurable without graphs
                sys.stderr.write(f"[bench] CUDA graph capture failed ({e}); launching eagerly\n")
                graphs = None
                torch.cuda.synchronize()

    def run_steps(k, first):
        for i in range(k):
            s = (first + i) % N_SETS
            if graphs is not None:
                graphs[s].replay()
            else:
                raw_step(dsets[s])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------------------------------------------------------- timed region (device resident)
    with torch.cuda.stream(stream):
        run_steps(args.warmup, 0)
        barrier()
        sampler.active = True
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        run_steps(args.steps, args.warmup)
        e1.record(stream)
        barrier()
        ms_total = e0.elapsed_time(e1)
        # keep the GPU under the same load a little longer so the clock sampler sees it
        t_end = time.perf_counter() + 0.25
        while time.perf_counter() < t_end:
            run_steps(20, 0)
            torch.cuda.synchronize()
        sampler.active = False
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    value = world * tokens_step * args.steps / (ms_total * 1e-3)

    # ---------------------------------------------------------------- per-kernel durations (instrumented repeat)
    def time_op(fn, reps):
        """Average device time of one launch: `reps` launches on rotating input sets captured into one CUDA
        graph (no host launch overhead between them), replayed between two events."""
        with torch.cuda.stream(stream):
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    for i in range(reps):
                        fn(i, torch.cuda.current_stream().cuda_stream)
                run = g.replay
            except Exception:
                torch.cuda.synchronize()
                run = lambda: [fn(i, stream.cuda_stream) for i in range(reps)]
            run()
            stream.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            run()
            b.record(stream)
            b.synchronize()
            return a.elapsed_time(b) / reps

    per_kernel = {}
    reps = 24
    ops.set_concurrency(1)        # a kernel timed alone is planned alone: for the whole GPU
    for ki, r in enumerate(KEEPS):
        def f_fwd(i, sc, ki=ki):
            it = dsets[i % N_SETS][ki]
            lib.svtad_conv_fwd(it["x"].data_ptr(), it["table"].data_ptr(), weight.data_ptr(), bias.data_ptr(),
                               y_buf.data_ptr(), it["n"], C, C, KK, 0, code, None, 0, sc)

        def f_dg(i, sc, ki=ki):
            it = dsets[i % N_SETS][ki]
            lib.svtad_conv_dgrad(it["gy"].data_ptr(), it["table"].data_ptr(), weight.data_ptr(), gx_buf.data_ptr(),
                                 it["n"], C, C, KK, 0, code, None, None, 0, sc)

        def f_wg(i, sc, ki=ki):
            it = dsets[i % N_SETS][ki]
            lib.svtad_conv_wgrad(it["gy"].data_ptr(), it["x"].data_ptr(), it["table"].data_ptr(), gw_buf.data_ptr(),
                                 gb_buf.data_ptr(), it["n"], C, C, KK, 0, code, ws.data_ptr(), ws_bytes, sc)

        for name, fn in (("fwd", f_fwd), ("dgrad", f_dg), ("wgrad", f_wg)):
            per_kernel[(name, ki)] = time_op(fn, reps)
    torch.cuda.synchronize()
    # the end-to-end part below is bound by the host link, its SMs are mostly idle: every kernel stays planned for the
    # whole GPU there (shortest latency per layer; measured no different from the step's hints: 0.73-0.75 ms either way)
    totals = {name: sum(per_kernel[(name, ki)] for ki in range(len(KEEPS))) for name in ("fwd", "dgrad", "wgrad")}
    dominant = max(totals, key=totals.get)
    peak_tf, peak_hbm, peak_kind = measured_peaks()
    dom_flops = sum(flops_pass(host_sets[0][ki]["n"]) for ki in range(len(KEEPS)))
    achieved = dom_flops / (totals[dominant] * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "kernel": {"fwd": "conv_hybrid_kernel<BN,false>", "dgrad": "conv_hybrid_kernel<BN,true>",
                                      "wgrad": "wgrad_hybrid_kernel<BN> + wgrad_reduce4_kernel"}[dominant],
        "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
        "peak_source": f"{peak_kind} bf16 burst", "traffic": NCU_DRAM_BYTES_PER_ROW[dominant] * tokens_step / len(KEEPS),
        "traffic_note": "not measured in this run: a constant, the ncu DRAM bytes per row of the captures summarised under "
                        "profiles/ times the mean rows per launch",
        "flops_per_launch": {f"keep{int(r * 100)}": flops_pass(host_sets[0][ki]["n"]) for ki, r in enumerate(KEEPS)},
        "ms_per_launch": {f"{name}_keep{int(KEEPS[ki] * 100)}": v for (name, ki), v in per_kernel.items()},
        "all_kernels_frac": {name: dom_flops / (totals[name] * 1e-3) / 1e12 / peak_tf for name in totals},
        "frac_per_launch": {f"{name}_keep{int(KEEPS[ki] * 100)}": flops_pass(host_sets[0][ki]["n"]) / (v * 1e-3) / 1e12 / peak_tf
                            for (name, ki), v in per_kernel.items()},
        "whole_step_frac": 3 * dom_flops / (ms_total / args.steps * 1e-3) / 1e12 / peak_tf,
        "planning": f"the per-launch figures time each kernel alone, planned for the whole GPU (svtad_set_concurrency(1)); "
                    f"inside the step the kernels of the three layers are planned with svtad_set_concurrency({layer_hints}) and overlap, "
                    f"whole_step_frac is their aggregate",
    }

    if os.environ.get("SVTAD_BENCH_VALUE_ONLY"):       # a short line for sweeps: the resident step only
        if rank == 0:
            print(json.dumps({"n_gpus": world, "ms_per_step": ms_total / args.steps, "sweep_line": True,
                              "run": {"allreduce": allreduce_kind, "concurrency_hints": layer_hints}}))
            sys.stdout.flush()
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier()
        os._exit(0)
    # ---------------------------------------------------------------- e2e through the public API, host buffers
    # One SparseConv2d per keep rate (three adapter layers with the same initial weights), each on its own
    # stream: copy in -> table -> forward -> backward -> copy out are ordered inside a layer's stream, and the
    # three layers' streams overlap one another, so the two copy engines and the SMs work at the same time.
    # Every input set has its own pinned result buffers.
    modules = [SparseConv2d(C, C).to(dev) for _ in KEEPS]
    with torch.no_grad():
        for m in modules:
            m.weight.copy_(weight_h)
            m.bias.copy_(bias_h)
    pin = []
    for per_keep in host_sets:
        pk = []
        for it in per_keep:
            pk.append({k: (v.pin_memory() if hasattr(v, "pin_memory") else v) for k, v in it.items()})
        pin.append(pk)
    out_h = [[{"y": torch.empty(it["n"], C, dtype=torch.bfloat16).pin_memory(),
               "gx": torch.empty(it["n"], C, dtype=torch.bfloat16).pin_memory(),
               "gw": torch.empty(KK, C, C, dtype=torch.float32).pin_memory(),
               "gb": torch.empty(C, dtype=torch.float32).pin_memory()} for it in host_sets[0]] for _ in range(N_SETS)]
    h2d = sum(it["scores"].numel() * 4 + it["x"].numel() * 2 + it["gy"].numel() * 2 for it in host_sets[0])
    d2h = sum(2 * it["n"] * C * 2 for it in host_sets[0]) + 3 * (KK * C * C * 4 + C * 4)
    layer_streams = [torch.cuda.Stream(device=dev) for _ in KEEPS]
    # N > 1: the three layers' fp32 gradients go into ONE bucket that is summed once per step on a stream of its own
    # (high priority, after the three layers' backward) and leaves for the host in one copy
    e2e_bucket = e2e_comm = grads_h = None
    if world > 1:
        e2e_bucket = GradBucket(len(KEEPS) * per_layer, torch.float32, dev)
        e2e_comm = torch.cuda.Stream(device=dev, priority=-1)
        grads_h = [torch.empty(len(KEEPS) * per_layer, dtype=torch.float32).pin_memory() for _ in range(N_SETS)]

    def e2e_body(si):
        """One step's public-API calls, layer ki on layer_streams[ki]; results land in out_h[si % N_SETS]."""
        slot = si % N_SETS
        for ki, it in enumerate(pin[slot]):
            module = modules[ki]
            with torch.cuda.stream(layer_streams[ki]):
                scores = it["scores"].to(dev, non_blocking=True)
                x = it["x"].to(dev, non_blocking=True).requires_grad_(True)
                gy = it["gy"].to(dev, non_blocking=True)
                kept, table = build_neighbor_table(scores, num_keep=it["k"], h=H, w=W, kernel_size=KS)
                module.zero_grad(set_to_none=True)
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    y = module(x, table, local_indices=False)   # tables of the builder hold global row numbers
                y.backward(gy)
                o = out_h[slot][ki]
                o["y"].copy_(y, non_blocking=True)
                o["gx"].copy_(x.grad, non_blocking=True)
                if world > 1:
                    e2e_bucket.view(ki * per_layer, (KK, C, C)).copy_(module.weight.grad)
                    e2e_bucket.view(ki * per_layer + KK * C * C, (C,)).copy_(module.bias.grad)
                else:
                    o["gw"].copy_(module.weight.grad, non_blocking=True)
                    o["gb"].copy_(module.bias.grad, non_blocking=True)
        if world > 1:
            for st in layer_streams:
                e2e_comm.wait_stream(st)
            with torch.cuda.stream(e2e_comm):
                e2e_bucket.all_reduce()
                grads_h[slot].copy_(e2e_bucket.buffer, non_blocking=True)

    def fork_join(si):
        """e2e_body between a fork from and a join back to the current stream."""
        cur = torch.cuda.current_stream()
        for st in layer_streams:
            st.wait_stream(cur)
        e2e_body(si)
        for st in layer_streams:
            cur.wait_stream(st)
        if e2e_comm is not None:
            cur.wait_stream(e2e_comm)

    # Steps alternate between two streams, so the copies in of one step overlap the copies out of the one before
    # (with N > 1 a single stream keeps the ranks' collectives in one order).
    n_step_streams = int(os.environ.get("SVTAD_BENCH_E2E_STREAMS", "2")) if world == 1 else 1
    step_streams = [torch.cuda.Stream(device=dev) for _ in range(n_step_streams)]
    for i in range(3):          # eager warm-up: allocator pools, cached parameter copies, the library's side stream
        with torch.cuda.stream(step_streams[0]):
            fork_join(i)
    torch.cuda.synchronize()
    # The step's calls are then captured once per input set (copies in, table, forward, backward, copies out) and
    # replayed: a user with fixed shapes does the same, and the host's share of a step drops from ~1.2 ms of
    # Python to one graph launch.  If capture is not possible the same calls are issued eagerly.
    e2e_graphs = None
    if not args.no_graph and os.environ.get("SVTAD_BENCH_E2E", "graph") != "eager":
        try:
            e2e_graphs = []
            for si in range(N_SETS):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=step_streams[0]):
                    fork_join(si)
                e2e_graphs.append(g)
        except Exception as e:
            sys.stderr.write(f"[bench] e2e: CUDA graph capture failed ({str(e)[:200]}); issuing the calls eagerly\n")
            e2e_graphs = None
            torch.cuda.synchronize()

    def e2e_step(si):
        with torch.cuda.stream(step_streams[si % len(step_streams)]):
            if e2e_graphs is not None:
                e2e_graphs[si % N_SETS].replay()
            else:
                fork_join(si)

    def e2e_drain():
        cur = torch.cuda.current_stream()
        for st in step_streams:
            cur.wait_stream(st)

    # Host-side copies on a shared machine are noisy (other tenants' PCIe and memory traffic): the timed steps
    # run as E2E_BLOCKS blocks of equal length, each bracketed by events after a full drain, and the median
    # block is reported (all block times are kept on the line).
    E2E_BLOCKS = 5
    e2e_steps = max(3, min(args.steps, 50) // E2E_BLOCKS)
    for i in range(3):
        e2e_step(i)
    e2e_drain()
    barrier()
    sampler.active = True
    block_ms = []
    step_no = 3
    for _ in range(E2E_BLOCKS):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for st in step_streams:
            st.wait_stream(torch.cuda.current_stream())
        for i in range(e2e_steps):
            e2e_step(step_no)
            step_no += 1
        e2e_drain()          # every copy of every timed step has landed before the closing event
        b.record()
        barrier()
        ms = a.elapsed_time(b)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        block_ms.append(ms)
    sampler.active = False
    # what landed in host memory is what the resident path computes from the same inputs (same kernels: bitwise)
    torch.cuda.synchronize()
    chk = (step_no - 1) % N_SETS
    for ki, it in enumerate(dsets[chk]):
        y_ref = ops.conv_fwd(it["x"], it["table"], weight, bias)
        gx_ref = ops.conv_dgrad(it["gy"], it["table"], weight, assume_symmetric=True)
        assert torch.equal(out_h[chk][ki]["y"].to(dev), y_ref), "e2e forward output differs from the resident path"
        assert torch.equal(out_h[chk][ki]["gx"].to(dev), gx_ref), "e2e input gradient differs from the resident path"
    e2e_ms = sorted(block_ms)[len(block_ms) // 2]
    e2e_value = world * tokens_step * e2e_steps / (e2e_ms * 1e-3)

    # what the host link gives in this run: pinned copies of the step's volume, each direction alone and both at once
    def copy_rate(do_h2d, do_d2h, reps=6):
        hb = torch.empty(h2d, dtype=torch.uint8).pin_memory()
        db = torch.empty(h2d, dtype=torch.uint8, device=dev)
        hb2 = torch.empty(d2h, dtype=torch.uint8).pin_memory()
        db2 = torch.empty(d2h, dtype=torch.uint8, device=dev)
        s1, s2 = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        s1.wait_stream(torch.cuda.current_stream()); s2.wait_stream(torch.cuda.current_stream())
        for _ in range(reps):
            if do_h2d:
                with torch.cuda.stream(s1):
                    db.copy_(hb, non_blocking=True)
            if do_d2h:
                with torch.cuda.stream(s2):
                    hb2.copy_(db2, non_blocking=True)
        torch.cuda.current_stream().wait_stream(s1); torch.cuda.current_stream().wait_stream(s2)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps
    ms_h, ms_d, ms_both = copy_rate(True, False), copy_rate(False, True), copy_rate(True, True)
    link = {"h2d_alone_GBs": h2d / (ms_h * 1e-3) / 1e9, "d2h_alone_GBs": d2h / (ms_d * 1e-3) / 1e9,
            "both_at_once_ms_per_step_volume": ms_both,
            "achieved_h2d_GBs": h2d / (e2e_ms / e2e_steps * 1e-3) / 1e9, "achieved_d2h_GBs": d2h / (e2e_ms / e2e_steps * 1e-3) / 1e9,
            "note": "pinned copies of one step's bytes measured in this run; 'both at once' is the floor of an e2e step"}
    if world > 1:
        link["note"] += "; with N > 1 all ranks share one host's memory and PCIe root, which bounds the e2e number"

    # the same public-API calls issued eagerly, no CUDA graph (what a training loop pays per step on the host)
    eager_ms = None
    if world == 1:
        with torch.cuda.stream(step_streams[0]):
            for i in range(2):
                fork_join(i)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(step_streams[0])
            for i in range(10):
                fork_join(i)
            b.record(step_streams[0])
            b.synchronize()
            eager_ms = a.elapsed_time(b) / 10
    sampler.stop_flag = True
    assert ops.device_error() == 0, "a bounded wait inside a tensor-core kernel gave up"

    # ---------------------------------------------------------------- reference CUDA path on the same GPU (rank 0)
    ref_cuda = None
    if rank == 0 and not args.skip_ref_cuda:
        try:
            ref_cuda = time_reference_cuda(dsets, weight, bias, stream, roofline["ms_per_launch"])
        except Exception as e:
            ref_cuda = {"unavailable": str(e)[:200]}

    # ---------------------------------------------------------------- CPU baseline (rank 0, N = 1)
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        slices = 40
        v, ms, cores, tokens = cpu_port_run(3, 1, slices)
        cpu = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": f"{slices} of {B * T} slices per keep rate ({tokens} tokens per step, 3 steps), C oracle port, OpenMP"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world),           # the same dictionary in both arms
            "run": dict(launch="cuda_graph" if graphs is not None else "eager", concurrency_hints=layer_hints,
                        wgrad_concurrency_hints=wgrad_hints, order="weight gradients first" if wgrad_first else "forward first",
                        layer_streams=bool(args.layer_streams), **({"allreduce": allreduce_kind} if world > 1 else {})),
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                    "stat": f"median of {E2E_BLOCKS} blocks of {e2e_steps} steps",
                    "launch": "cuda_graph of the public-API calls" if e2e_graphs is not None else "eager",
                    "block_ms_per_step": [round(m / e2e_steps, 4) for m in block_ms],
                    "host_link": link, "eager_ms_per_step": eager_ms},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": roofline, "cpu_baseline": cpu, "reference_cuda": ref_cuda,
            "clocks": sampler.summary(),
        }
        print(json.dumps(line))
    if world > 1:
        # leave together, and without tearing the communicator down under live CUDA graphs
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def backbone_case(args):
    """Secondary measurement: forward of the sparse-adapter ViT-B backbone, bf16, random-init weights, one 3x160x224x224
    clip per step and rank (clips are sharded over ranks; no collective in the forward), 30 % keep after block 3."""
    import torch
    import torch.distributed as dist
    from eccv26_tad_b200 import SparseAdapterViT
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(5 + rank)
    keep_rates = None
    if args.backbone_schedule == "reference":
        keep_rates = [1.0, 1.0, 1.0, 0.6, 1.0, 1.0, 0.6, 1.0, 1.0, 0.6, 1.0, 1.0]
    model = SparseAdapterViT(keep_rates=keep_rates).to(dev).eval()
    for blk in model.blocks:
        torch.nn.init.normal_(blk.adapter.up_proj.weight, std=0.02)
    clips = [torch.randn(1, 3, 160, 224, 224, device=dev) for _ in range(2)]
    steps, warm = max(1, min(args.steps, 20)), max(3, min(args.warmup, 5))
    train = bool(args.backbone_train)
    if train:
        # SV-TAD's setting: frozen backbone, trainable adapters; gradients flow back through the frozen blocks
        model.train()
        for p in model.parameters():
            p.requires_grad_(False)
        params = [p for blk in model.blocks for p in blk.adapter.parameters()]
        for p in params:
            p.requires_grad_(True)
        opt = torch.optim.AdamW(params, lr=1e-4)

        def step(clip):
            opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                out = model(clip)
            out.float().square().mean().backward()
            if world > 1:   # data parallel: one flat all-reduce of the adapters' gradients
                flat = torch.cat([p.grad.reshape(-1) for p in params])
                dist.all_reduce(flat)
                off = 0
                for p in params:
                    p.grad.copy_(flat[off:off + p.numel()].view_as(p.grad) / world)
                    off += p.numel()
            opt.step()
            return out
    else:
        def step(clip):
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                return model(clip)
    for i in range(warm):
        step(clips[i % 2])
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        out = step(clips[i % 2])
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    glue = None
    if rank == 0 and not train:
        # the adapter's glue around the op (GELU on down_proj's output, the copy that drops the special tokens, the
        # concatenation that puts them back), timed by itself at every adapter's token count
        counts = []
        hooks = [blk.adapter.register_forward_pre_hook(lambda _m, inp: counts.append(inp[0].shape[1]))
                 for blk in model.blocks]
        step(clips[0])
        for h_ in hooks:
            h_.remove()
        hidden = model.blocks[0].adapter.down_proj.out_features

        def timed(fn, reps=20):
            fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps * 1e3
        tot = {"gelu_us": 0.0, "slice_copy_us": 0.0, "cat_us": 0.0}
        for ntok in counts:
            z = torch.randn(1, ntok, hidden, device=dev, dtype=torch.bfloat16)
            conv = torch.randn(1, ntok - 1, hidden, device=dev, dtype=torch.bfloat16)
            tot["gelu_us"] += timed(lambda: torch.nn.functional.gelu(z))
            tot["slice_copy_us"] += timed(lambda: z[:, 1:].contiguous())
            tot["cat_us"] += timed(lambda: torch.cat([z[:, :1], conv], dim=1))
        per_clip = sum(tot.values())
        glue = dict({k: round(v, 1) for k, v in tot.items()}, per_clip_us=round(per_clip, 1),
                    share_of_forward=round(per_clip * 1e-3 / (ms / steps), 4), adapters=len(counts),
                    what="eager torch kernels around SparseConv2d in every adapter, summed over the clip's adapters")
    if rank == 0:
        what = "training step (forward, backward to the adapters, AdamW)" if train else "forward"
        print(json.dumps({"metric": f"sparse-adapter ViT-B backbone {what}, clips/s", "value": world * steps / (ms * 1e-3),
                          "unit": "clips/s", "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": ms / steps,
                          "higher_is_better": True, "scaling": "weak", "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": f"ViT-B/16 sparse-adapter backbone {what}, 3x160x224x224 clips, "
                                                 "15680 tokens + CLS, adapters 768->192->768 with SparseConv2D 3x3, " +
                                                 ("keep 30 % after block 3" if keep_rates is None else "keep 0.6 after blocks 3, 6, 9 (reference schedule)")},
                          "adapter_glue": glue, "out_shape": list(out.shape)}))
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


def kernel_case(args):
    """A few launches of one kernel on one large seeded case (for ncu captures; prints timings only)."""
    import torch
    from eccv26_tad_b200 import build_neighbor_table, ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(99)
    slices = args.case_slices
    k = num_keep(args.case_keep, H * W)
    scores = torch.randn(slices, H * W, generator=g).to(dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.case_launches + 1)]
    if args.kernel_case == "table":
        ev[0].record()
        for i in range(args.case_launches):
            kept, table = build_neighbor_table(scores, num_keep=k, h=H, w=W, kernel_size=KS)
            ev[i + 1].record()
        torch.cuda.synchronize()
        n = slices * k
        bytes_ = 4 * slices * H * W + 4 * n + 4 * n * KK
        ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.case_launches)]
        print(json.dumps({"kernel_case": "table", "slices": slices, "rows": n, "ms": ms,
                          "algorithmic_bytes": bytes_, "GB/s_best": bytes_ / (min(ms) * 1e-3) / 1e9}))
        return
    kept, table = build_neighbor_table(scores, num_keep=k, h=H, w=W, kernel_size=KS)
    n = table.shape[0]
    x = torch.randn(n, C, device=dev).bfloat16()
    gy = torch.randn(n, C, device=dev).bfloat16()
    w = (torch.randn(KK, C, C, device=dev) * math.sqrt(2.0 / (C * KK))).bfloat16()
    b = torch.zeros(C, device=dev).bfloat16()
    ev[0].record()
    for i in range(args.case_launches):
        if args.kernel_case == "fwd":
            ops.conv_fwd(x, table, w, b)
        elif args.kernel_case == "dgrad":
            ops.conv_dgrad(gy, table, w, assume_symmetric=True)
        else:
            ops.conv_wgrad(gy, x, table, KK)
        ev[i + 1].record()
    torch.cuda.synchronize()
    ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.case_launches)]
    print(json.dumps({"kernel_case": args.kernel_case, "slices": slices, "rows": n, "ms": ms,
                      "flops": flops_pass(n), "TFLOP/s_best": flops_pass(n) / (min(ms) * 1e-3) / 1e12}))


def _time_eager(fn, reps, warm=3):
    """Average milliseconds of `reps` eager calls of fn(i) on the legacy default stream (where the reference's
    extension launches), after `warm` untimed ones."""
    import torch
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(reps):
        fn(warm + i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def time_reference_cuda(dsets, weight, bias, stream, ours_ms_per_launch=None):
    """The reference's own CUDA extension (prebuilt under oracle/_ref/) on the same resident inputs, per keep rate:
    its own dispatch for C_in >= 128 (implicit_gemm_fwd_v2_chunked, then bwd_in, bwd_w and the bias sum), 50 eager
    repetitions per keep rate on rotating input sets."""
    import torch
    from oracle import build_ref
    mod = build_ref.load_built()
    if mod is None:
        return {"unavailable": "oracle/_ref extension not built"}
    reps = 50
    per_keep = {}
    total_ms = 0.0
    for ki, r in enumerate(KEEPS):
        def layer(i, ki=ki):
            it = dsets[i % N_SETS][ki]
            mod.implicit_gemm_fwd_v2_chunked(it["x"], it["table"], weight, bias, 0, 4096)
            mod.bwd_in(it["gy"], it["table"], weight, it["n"], C, 0)
            mod.bwd_w(it["gy"], it["x"], it["table"], C, 0)
            it["gy"].sum(0)
        ms = _time_eager(layer, reps)
        n = dsets[0][ki]["n"]
        row = {"ms": ms, "tokens_per_s": n / (ms * 1e-3), "TFLOP/s": 3 * flops_pass(n) / (ms * 1e-3) / 1e12}
        if ours_ms_per_launch is not None:
            ours = sum(ours_ms_per_launch[f"{name}_keep{int(r * 100)}"] for name in ("fwd", "dgrad", "wgrad"))
            row["ours_ms"] = ours
            row["speedup"] = ms / ours
        per_keep[f"keep{int(r * 100)}"] = row
        total_ms += ms
    tokens = sum(it["n"] for it in dsets[0])
    return {"value": tokens / (total_ms * 1e-3), "unit": "tokens/s", "ms_per_step": total_ms, "steps": reps,
            "per_keep": per_keep,
            "what": "reference extension (implicit_gemm_fwd_v2_chunked + bwd_in + bwd_w + sum) recompiled for sm_100a; "
                    "eager launches, 50 repetitions per keep rate; ours_ms = the three kernels of this library for the "
                    "same layer, timed back to back from a CUDA graph"}


# ------------------------------------------------------------------------------------------ other configurations
def _graph_time(fn, reps=24):
    """Average microseconds of one fn(i, stream) launch: `reps` launches captured into one CUDA graph and replayed."""
    import torch
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        fn(0, st.cuda_stream)
        st.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for i in range(reps):
                fn(i, torch.cuda.current_stream().cuda_stream)
        g.replay()
        st.synchronize()
        best = None
        for _ in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(st)
            g.replay()
            b.record(st)
            b.synchronize()
            t = a.elapsed_time(b) / reps
            best = t if best is None else min(best, t)
    return best * 1e3


def ffma_peak_tflops():
    """FFMA rate of this GPU (what the fp32 CUDA-core kernels are measured against): svtad_ffma_probe timed here."""
    import torch
    from eccv26_tad_b200 import _lib
    lib = _lib.load()
    scratch = torch.zeros(4, device="cuda")
    ctas, iters = 148 * 8, 4000
    us = _graph_time(lambda i, sc: _lib.check(lib.svtad_ffma_probe(ctas, iters, scratch.data_ptr(), sc)), 5)
    return 2.0 * 64 * iters * ctas * 256 / (us * 1e-6) / 1e12


def configs_case(args):
    """Secondary lines, one JSON line each: the benchmark configurations other than the headline one, every kernel
    with its fraction of the roofline that bounds it and the reference's CUDA path beside it where that can run.
      config1  fp32 forward, batch 1 x T=8, C=192, keep 50 % (784 rows)            -> fraction of the FFMA rate
      config3  bf16 fwd / dgrad / wgrad, batch 4 x T=80, keep 30 % (18 880 rows), C in {256, 768, 1024}, 3x3 and 5x5
      config4  neighbor-table construction alone, 3072 slices, keep {10, 25, 50} %  -> fraction of HBM bandwidth"""
    import torch
    from eccv26_tad_b200 import _lib, build_neighbor_table, ops
    from eccv26_tad_b200.backbone import _torch_remap
    from oracle import build_ref
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.backends.cuda.matmul.allow_tf32 = False
    lib = _lib.load()
    ref = build_ref.load_built()
    peak_tf, peak_hbm, peak_kind = measured_peaks()
    want = args.configs.split(",")

    def table_for(slices, keep, ks, seed):
        g = torch.Generator().manual_seed(seed)
        scores = torch.randn(slices, H * W, generator=g).to(dev)
        return scores, build_neighbor_table(scores, num_keep=num_keep(keep, H * W), h=H, w=W, kernel_size=ks)

    if "1" in want:
        ffma = ffma_peak_tflops()
        _, (kept, table) = table_for(8, 0.5, 3, 1235)
        n = table.shape[0]
        g = torch.Generator().manual_seed(1235)
        x = torch.randn(n, C, generator=g).to(dev)
        w = (torch.randn(C, C, 3, 3, generator=g) * math.sqrt(2.0 / (C * 9))).view(C, C, 9).permute(2, 1, 0).contiguous().to(dev)
        b = torch.zeros(C, device=dev)
        y = torch.empty(n, C, device=dev)
        us = _graph_time(lambda i, sc: _lib.check(lib.svtad_conv_fwd(x.data_ptr(), table.data_ptr(), w.data_ptr(), b.data_ptr(),
                                                                     y.data_ptr(), n, C, C, 9, 0, _lib.F32, None, 0, sc)))
        fl = 2.0 * n * 9 * C * C
        line = {"metric": "SparseConv2D forward fp32 (config 1), retained tokens/s", "value": n / (us * 1e-6), "unit": "tokens/s",
                "config": {"workload": "fp32 forward, batch 1 x T=8 x 14x14, Cin=Cout=192, 3x3, keep 50 % (784 rows)"},
                "us_per_launch": us, "dtype": "f32", "data": "synthetic",
                "roofline": {"bound": "ffma", "achieved": fl / (us * 1e-6) / 1e12, "peak": ffma, "unit": "TFLOP/s",
                             "frac": fl / (us * 1e-6) / 1e12 / ffma, "peak_source": "svtad_ffma_probe timed in this run",
                             "flops": "dense-equivalent 2*N*KK*Cin*Cout"}}
        if ref is not None:
            ms = _time_eager(lambda i: ref.implicit_gemm_fwd_v2(x, table, w, b, 0), 50)
            line["reference_cuda"] = {"us_per_launch": ms * 1e3, "speedup": ms * 1e3 / us,
                                      "what": "implicit_gemm_fwd_v2 in fp32 (gather + cuBLAS SGEMM, TF32 off + reduce), eager"}
        print(json.dumps(line), flush=True)

    if "3" in want:
        for Cc in (256, 768, 1024):
            for ks in (3, 5):
                kk = ks * ks
                _, (kept, table) = table_for(4 * 80, 0.3, ks, 1237)
                n = table.shape[0]
                x = torch.randn(n, Cc, device=dev).bfloat16()
                gy = torch.randn(n, Cc, device=dev).bfloat16()
                w = (torch.randn(kk, Cc, Cc, device=dev) * math.sqrt(2.0 / (Cc * kk))).bfloat16()
                b = torch.zeros(Cc, device=dev).bfloat16()
                y = torch.empty(n, Cc, dtype=torch.bfloat16, device=dev)
                gw = torch.empty(kk, Cc, Cc, dtype=torch.bfloat16, device=dev)
                gb = torch.empty(Cc, dtype=torch.bfloat16, device=dev)
                ws_bytes = lib.svtad_workspace_bytes(_lib.OP_WGRAD, n, Cc, Cc, kk, _lib.BF16)
                ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
                code = _lib.BF16
                t = {
                    "fwd": _graph_time(lambda i, sc: _lib.check(lib.svtad_conv_fwd(x.data_ptr(), table.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), n, Cc, Cc, kk, 0, code, None, 0, sc)), 6),
                    "dgrad": _graph_time(lambda i, sc: _lib.check(lib.svtad_conv_dgrad(gy.data_ptr(), table.data_ptr(), w.data_ptr(), y.data_ptr(), n, Cc, Cc, kk, 0, code, None, None, 0, sc)), 6),
                    "wgrad": _graph_time(lambda i, sc: _lib.check(lib.svtad_conv_wgrad(gy.data_ptr(), x.data_ptr(), table.data_ptr(), gw.data_ptr(), gb.data_ptr(), n, Cc, Cc, kk, 0, code, ws.data_ptr(), ws_bytes, sc)), 6),
                }
                fl = 2.0 * n * kk * Cc * Cc
                total_us = sum(t.values())
                line = {"metric": "SparseConv2D fwd+bwd bf16 (config 3), retained tokens/s", "value": n / (total_us * 1e-6),
                        "unit": "tokens/s", "dtype": "bf16", "data": "synthetic",
                        "config": {"workload": f"bf16 fwd+dgrad+wgrad, batch 4 x T=80 x 14x14, keep 30 % ({n} rows), Cin=Cout={Cc}, {ks}x{ks}"},
                        "us_per_launch": t,
                        "roofline": {"bound": "tensor", "peak": peak_tf, "unit": "TFLOP/s", "peak_source": f"{peak_kind} bf16 burst",
                                     "achieved": {k: fl / (v * 1e-6) / 1e12 for k, v in t.items()},
                                     "frac": {k: fl / (v * 1e-6) / 1e12 / peak_tf for k, v in t.items()},
                                     "frac_fwd_bwd": 3 * fl / (total_us * 1e-6) / 1e12 / peak_tf}}
                if ref is None:
                    pass
                elif ks != 3:
                    line["reference_cuda"] = "unsupported kernel size (the reference's kernels are 3x3 only)"
                else:
                    def layer(i):
                        ref.implicit_gemm_fwd_v2_chunked(x, table, w, b, 0, 4096)
                        ref.bwd_in(gy, table, w, n, Cc, 0)
                        ref.bwd_w(gy, x, table, Cc, 0)
                        gy.sum(0)
                    ms = _time_eager(layer, 5 if Cc > 256 else 20, warm=1)
                    line["reference_cuda"] = {"us_fwd_bwd": ms * 1e3, "speedup": ms * 1e3 / total_us, "what": "eager"}
                print(json.dumps(line), flush=True)
                del x, gy, w, y, gw, ws

    if "4" in want:
        slices = 8 * 384
        full = ops.table_init(slices, 1, H, W, 3, dev)            # one 14x14 slice per row of the batch dimension
        for keep in (0.10, 0.25, 0.50):
            k = num_keep(keep, H * W)
            g = torch.Generator().manual_seed(1238)
            scores = torch.randn(slices, H * W, generator=g).to(dev)
            kept = torch.empty(slices, k, dtype=torch.int32, device=dev)
            table = torch.empty(slices * k, 9, dtype=torch.int32, device=dev)
            us = _graph_time(lambda i, sc: _lib.check(lib.svtad_table_build(scores.data_ptr(), slices, H * W, k, H, W, 3,
                                                                            kept.data_ptr(), table.data_ptr(), sc)), 10)

            def torch_ops(i):
                idx = torch.topk(scores, k, dim=1, largest=True)[1].sort(dim=1)[0]
                return idx, _torch_remap(full, idx)
            ms = _time_eager(torch_ops, 20)
            idx, tref = torch_ops(0)
            same = bool(torch.equal(tref.reshape(-1, 9), table) and torch.equal(idx.to(torch.int32), kept))
            n = slices * k
            bytes_ = 4 * slices * H * W + 4 * n + 4 * n * 9
            line = {"metric": "neighbor-table construction (config 4), retained tokens/s", "value": n / (us * 1e-6),
                    "unit": "tokens/s", "dtype": "int32", "data": "synthetic",
                    "config": {"workload": f"top-k + 3x3 table, {slices} slices of 14x14 fp32 scores, keep {int(keep * 100)} % ({n} rows)"},
                    "us_per_launch": us,
                    "roofline": {"bound": "hbm", "achieved": bytes_ / (us * 1e-6) / 1e9, "peak": peak_hbm, "unit": "GB/s",
                                 "frac": bytes_ / (us * 1e-6) / 1e9 / peak_hbm, "peak_source": f"{peak_kind} copy bandwidth",
                                 "bytes": "4*S*L scores + 4*N kept + 36*N table"},
                    "torch_ops": {"us": ms * 1e3, "speedup": ms * 1e3 / us, "bit_identical": same,
                                  "what": "topk + sort + gather + remap of the reference restated in torch ops on the same GPU "
                                          "(vit_sparse_adapter_poguise.py:785-787, 913-977), full-grid table precomputed, eager"}}
            print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
