#!/usr/bin/env python
"""Benchmark of the quantized-inference hot path: u8/u8 ResNet-50 v2 images/s on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]
                  [--w-quant uint8|int8] [--layers] [--no-secondary]

One step = one forward pass of the whole quantized network over one batch of synthetic images
(seeded N(0,1) inputs standing in for ImageNet; random He-normal weights, BN folded). The
configuration the metric is quoted on is a GLOBAL batch of 512 images: on N GPUs (launch under
torchrun, one rank per GPU) every rank takes 512 / N of them, with no collective on the data path
(strong scaling). The weak-scaling figure (512 images on every GPU) is reported beside it as
`weak`.

Prints ONE JSON line (rank 0). `value` is device-resident throughput, `e2e` the same metric through
the public host-buffer call (pinned f32 input -> H2D -> kernels -> D2H logits, every step's copies
inside the timed region), `parity` the comparison of this very run's tensors with the CPU oracle,
`secondary` the other paths of the library measured in the same run (paged attention, a decode
step, the streaming kernels, single-image latency). `--impl reference` times the reference's own
CPU kernels running the same quantized network on the host cores.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIG_ID = 3  # ResNet-50 v2 in the list of benchmark configurations
SEED_W, SEED_X, SEED_CAL = 1000 + CONFIG_ID, 2000 + CONFIG_ID, 3000 + CONFIG_ID
METRIC = "u8/u8 ResNet-50 images/s"
UNIT = "images/s"

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum, one-pass ncu captures) of the convolution launches of
# one step, keyed by (images per GPU, weight type); see profiles/dram_traffic_tc_conv_resnet50v2.md. Traffic
# does NOT grow in proportion to the batch between these sizes (at 128 images most producer -> consumer tensors
# never leave the 126 MB L2), so no figure is scaled: other batches report null.
MEASURED_DRAM_BYTES_PER_STEP = {(512, "uint8"): 17.181e9, (128, "uint8"): 2.861e9}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_burst=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_burst=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=mx, reasons=sorted(reasons),
                    samples=len(sm))


def build_network(device, w_quant):
    from nncase_b200 import builder, networks
    graph = networks.resnet50v2(SEED_W)
    cal = [np.random.default_rng(SEED_CAL + i).normal(0, 1, (1, 3, 224, 224)).astype(np.float32) for i in range(16)]
    program = builder.build_program(graph, cal, w_quant, device=device)
    macs, per_layer, _ = networks.graph_macs(graph)
    return graph, program, macs, dict(per_layer)


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's own kernels running the quantized network on the host cores
# ---------------------------------------------------------------------------------------------
def cpu_reference_images(program, images, threads):
    """Runs `images` synthetic images, one after the other, through the WHOLE quantized network on the
    reference's own CPU kernels (oracle/_ref: every operator dequantize -> float kernel -> quantize, the
    way its cpu target executes a quantized graph), each convolution split over `threads` host threads by
    output channel. Falls back to the integer C port where the reference's library is not available.
    Returns (images per second, kind, seconds)."""
    from oracle import program as oprog
    from oracle import ref
    x = np.random.default_rng(SEED_X).normal(0, 1, (1, 3, 224, 224)).astype(np.float32)
    use_ref = ref.available()
    t0 = time.perf_counter()
    for _ in range(images):
        if use_ref:
            from oracle import ref_program
            ref_program.run_program(program, x, threads=threads)
        else:
            oprog.run_program(program, x, threads=threads)
    dt = time.perf_counter() - t0
    return images / dt, ("reference" if use_ref else "port"), dt


def cpu_baseline(program, seconds_target, threads=None):
    threads = threads or os.cpu_count() or 1
    rate, kind, dt = cpu_reference_images(program, 1, threads)      # also tells how long an image takes
    n = int(max(1, min(8, seconds_target / max(dt, 1e-3) - 1)))
    if n >= 1 and dt * (n + 1) <= 2.0 * seconds_target:
        rate, kind, dt = cpu_reference_images(program, n, threads)
    else:
        n = 1
    return dict(value=rate, unit=UNIT, cores=threads, kind=kind,
                sample=f"{n} image(s) through all {sum(1 for o in program['ops'] if o['op'] == 'conv')} convolutions and "
                       f"every other operator of the quantized network on the "
                       f"{'reference kernels (dequantize -> float kernel -> quantize per operator)' if kind == 'reference' else 'integer C port'}"
                       f", {dt:.1f} s wall, convolutions split over {threads} threads by output channel")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    _, program, _, _ = build_network("cpu", args.w_quant)
    threads = os.cpu_count() or 1
    steps = max(1, args.steps)
    vals, kind, secs = [], "port", 0.0
    for i in range(args.warmup + steps):        # one step = one image through the whole network
        r, kind, dt = cpu_reference_images(program, 1, threads)
        if i >= args.warmup:
            vals.append(r)
            secs += dt
    v = float(len(vals) / sum(1.0 / r for r in vals))
    cb = dict(value=v, unit=UNIT, cores=threads, kind=kind,
              sample=f"{steps} timed steps of one image each through the whole quantized network on the "
                     f"{'reference kernels' if kind == 'reference' else 'integer C port'}, {secs:.1f} s wall")
    line = dict(metric=METRIC, value=v, unit=UNIT, n_gpus=args.gpus, steps=steps, warmup=args.warmup,
                ms_per_step=1000.0 / v, higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype="f32", data="synthetic", impl="reference",
                config=dict(workload="resnet50v2_u8u8", global_batch=args.batch, images_per_step=1,
                            w_quant=args.w_quant, note="a step is a bounded sample of the workload: one image"),
                cpu_baseline=cb, e2e=dict(value=v, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
def _events(torch):
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def time_device(torch, fn, x, steps, barrier):
    """K steps with the input resident in HBM. The step's launch list is captured once (CudaFunction.capture) and
    replayed: the same kernels on the same buffers, without the host's per-launch cost between them (2 % of a
    512-image step, 8 % of a 64-image one)."""
    fn.capture(x)
    for _ in range(2):
        fn.replay()
    a, b = _events(torch)
    barrier()
    a.record()
    for _ in range(steps):
        fn.replay()
    b.record()
    barrier()
    return a.elapsed_time(b)


def time_e2e(torch, fn, xh, oh, steps, barrier):
    """K batches through the public host-buffer call (CudaFunction.submit_host / drain): pinned f32 input ->
    H2D -> kernels -> D2H logits, double-buffered inside the library, every copy inside the timed region."""
    dev = fn.ctx.device
    a, b = _events(torch)
    barrier()
    cur = torch.cuda.current_stream(dev)
    a.record(cur)
    p = fn._pipeline()
    p["copy"].wait_event(a)
    p["comp"].wait_event(a)
    for i in range(steps):
        fn.submit_host(xh[i & 1], oh[i & 1])
    cur.wait_stream(p["comp"])
    cur.wait_stream(p["copy"])
    b.record(cur)
    fn.drain()
    barrier()
    return a.elapsed_time(b)


def time_h2d_only(torch, dev, xh, steps, barrier):
    """The bare host-to-device copies of the same pinned input buffers, all ranks at once: the ceiling the
    end-to-end number cannot exceed."""
    xd = torch.empty(xh[0].shape, dtype=torch.float32, device=dev)
    a, b = _events(torch)
    barrier()
    a.record()
    for i in range(steps):
        xd.copy_(xh[i & 1], non_blocking=True)
    b.record()
    barrier()
    return a.elapsed_time(b)


def parity_check(torch, fn, program, x, idx):
    """This run's tensors against the CPU oracle on a few images of the benchmark batch (outside every timed
    region). Images are independent, so the oracle replays only the chosen ones; every tensor of the
    program is compared byte for byte (the f32 logits exactly, too)."""
    from oracle import program as oprog
    n = x.shape[0]
    idx = sorted(set(int(i) % n for i in idx))
    sel = torch.tensor(idx, device=x.device)
    fn.invoke(x)
    _, tens = oprog.run_program(program, x.index_select(0, sel).cpu().numpy(), threads=os.cpu_count() or 8)
    bad, elems = 0, 0
    for name, ref_t in tens.items():
        got = fn.tensor(name).index_select(0, sel).cpu().numpy()
        bad += int((got != ref_t).sum())
        elems += ref_t.size
    return dict(images=idx, tensors=len(tens), elements=elems, mismatches=bad,
                against="oracle/qoracle.c replay of the same program on the same inputs")


def conv_rows(torch, fn, layer_macs, B, reps=5):
    """Live CUDA-event time, operations and algorithmic bytes of every convolution launch of a step."""
    dev = fn.ctx.device
    rows = []
    for st in fn.steps:
        if st[0] != "conv":
            continue
        op, plan = st[1], st[2]
        res = fn.buffers[op["res"]] if op.get("res") else None
        y2 = fn.buffers[op["y2"]] if op.get("y2") else None
        plan(fn.buffers[op["in"]], res, fn.buffers[op["out"]], y2)
        torch.cuda.synchronize(dev)
        t = None
        for _ in range(2):  # two rounds, the quieter one counts (a host hiccup between launches shows up as GPU idle time)
            a, b = _events(torch)
            a.record()
            for _ in range(reps):
                plan(fn.buffers[op["in"]], res, fn.buffers[op["out"]], y2)
            b.record()
            torch.cuda.synchronize(dev)
            t = a.elapsed_time(b) / reps if t is None else min(t, a.elapsed_time(b) / reps)
        ops = 2.0 * layer_macs[op["name"]] * B
        # algorithmic bytes of the launch: activations in, every tensor written or added, weights once
        n_, oh_, ow_, oc_ = plan.out_shape
        out_el = n_ * oh_ * ow_ * oc_
        nbytes = (fn.buffers[op["in"]].numel() + out_el * (4 if op.get("f32_out") else 1) +
                  (out_el if res is not None else 0) + (out_el if y2 is not None else 0) + op["w"].size)
        rows.append((op["name"], plan.path, t, ops, nbytes))
    return rows


def int8_peak(ctx):
    """The kind::i8 tensor-pipe peak of this GPU, measured now (library self-test): burst = best of ten
    1 ms launches, sustained = mean of 300 launches back to back (power-capped)."""
    from nncase_b200 import lib as L
    best, mean = C.c_double(), C.c_double()
    L.check(ctx._lib.nncb_selftest_int8_peak(ctx._h, 8192, 10, 0, C.byref(best), C.byref(mean)))
    burst = best.value
    L.check(ctx._lib.nncb_selftest_int8_peak(ctx._h, 8192, 300, 0, C.byref(best), C.byref(mean)))
    return dict(burst=burst, sustained=mean.value)


def mma_issue_pace(ctx):
    """SM cycles per tcgen05.mma kind::i8 (M 128, K 32) when one or two warps issue them back to back on resident
    operands (library self-test): what bounds a K loop apart from the tensor pipe's own rate."""
    from nncase_b200 import lib as L
    out = {}
    for n in (64, 144, 256):
        for issuers in (1, 2):
            c = C.c_double()
            L.check(ctx._lib.nncb_selftest_mma_issue(ctx._h, n, issuers, 16384, C.byref(c)))
            out[f"n{n}_issuers{issuers}"] = round(c.value, 1)
    out["unit"] = "SM cycles per MMA (tensor pipe alone: n / 1.9 at 1965 MHz against the measured int8 peak)"
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the hot path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from nncase_b200 import lib as L
    from nncase_b200 import sharding
    from nncase_b200.kernels import Context
    from nncase_b200.runtime import CudaFunction

    dev = torch.device("cuda", local)
    graph, program, macs, layer_macs = build_network(dev, args.w_quant)
    ctx = Context(local)
    G = args.batch                                   # global batch of the configuration
    start, B = sharding.shard_range(G, world, rank)  # this rank's images (strong scaling)
    if B * world != G:
        raise SystemExit(f"bench.py: the global batch {G} must divide over {world} ranks")
    fn = CudaFunction(program, B, ctx)
    g = torch.Generator(device=dev).manual_seed(SEED_X + rank)
    x = torch.randn((B, 3, 224, 224), device=dev, generator=g)
    steps, warm = args.steps, max(3, args.warmup)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # -------- device-resident throughput --------
    for _ in range(warm):
        fn.invoke(x)
    ctx.check_status()
    launches_per_step = fn.launches_per_call
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = time_device(torch, fn, x, steps, barrier)
    gpu_launches = launches_per_step * steps   # kernels of this library run by the replays inside the timed region
    ctx.check_status()

    # -------- end to end through the library's host-buffer call --------
    xh = [torch.empty((B, 3, 224, 224), dtype=torch.float32).pin_memory() for _ in range(2)]
    for t in xh:
        t.copy_(x)
    oh = [torch.empty((B, 1, 1, 1000), dtype=torch.float32).pin_memory() for _ in range(2)]
    time_e2e(torch, fn, xh, oh, 3, barrier)
    e2e_ms = time_e2e(torch, fn, xh, oh, steps, barrier)
    clocks = sampler.stop() if rank == 0 else None
    h2d_ms = time_h2d_only(torch, dev, xh, steps, barrier)
    ctx.check_status()

    # -------- per-layer timing of the dominant kernel (tcgen05 conv) for the roofline --------
    rows = conv_rows(torch, fn, layer_macs, B)
    tc = [r for r in rows if r[1] == L.PATH_TC]
    tc_ms, tc_ops, tc_bytes = sum(r[2] for r in tc), sum(r[3] for r in tc), sum(r[4] for r in tc)
    ctx.check_status()

    # -------- weak-scaling figure: the full 512 images on every GPU --------
    weak = None
    if world > 1:
        fn_w = CudaFunction(program, G, ctx)
        xw = torch.randn((G, 3, 224, 224), device=dev, generator=g)
        for _ in range(3):
            fn_w.invoke(xw)
        ms_w = time_device(torch, fn_w, xw, steps, barrier)
        ms_w = sharding.max_over_ranks([ms_w], dev)[0]
        weak = dict(value=world * G * steps / (ms_w / 1000.0), unit=UNIT, images_per_gpu=G, ms_per_step=ms_w / steps,
                    scaling="weak")
        fn_w.close()
        del fn_w, xw
        torch.cuda.empty_cache()

    # max over ranks of the device-measured times, sum of the launch counters
    ms, e2e_ms, h2d_ms = sharding.max_over_ranks([ms, e2e_ms, h2d_ms], dev)
    gpu_launches = sharding.sum_over_ranks([gpu_launches], dev)[0]
    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    parity = parity_check(torch, fn, program, x, [0, B // 2 - 1, B - 1])
    pk = peaks()
    i8 = int8_peak(ctx)
    value = G * steps / (ms / 1000.0)
    e2e_value = G * steps / (e2e_ms / 1000.0)
    int8_burst = i8["burst"]
    achieved = tc_ops / (tc_ms / 1000.0) / 1e12 if tc_ms > 0 else 0.0
    # The convolution launches of one step move tc_bytes and do tc_ops: their ratio (operations per
    # byte) lies below the ridge point int8 peak / HBM peak, so HBM bandwidth is the roof that bounds
    # the kernel on this workload; the tensor-pipe figures are kept beside it.
    gbs = tc_bytes / (tc_ms / 1000.0) / 1e9 if tc_ms > 0 else 0.0
    intensity = tc_ops / tc_bytes if tc_bytes else 0.0
    ridge = int8_burst * 1e12 / (pk["hbm_gbs"] * 1e9)
    hbm_bound = intensity < ridge
    traffic = MEASURED_DRAM_BYTES_PER_STEP.get((B, args.w_quant))
    line = dict(
        metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=steps, warmup=warm,
        ms_per_step=ms / steps, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="u8",
        data="synthetic", impl="ours",
        config=dict(workload="resnet50v2_u8u8", global_batch=G, batch_per_gpu=B, w_quant=args.w_quant,
                    input="f32 NCHW [B,3,224,224] N(0,1)", l2="inputs and activations larger than L2 (no flush)",
                    launch="the step's launch list captured once and replayed as a CUDA graph (value and e2e)",
                    parallelism=f"batch-sharded x{world}, no collective"),
        e2e=dict(value=e2e_value, unit=UNIT, h2d_bytes_per_step=G * 3 * 224 * 224 * 4, d2h_bytes_per_step=G * 1000 * 4,
                 call="CudaFunction.submit_host / drain (pinned host buffers, two device staging buffers, two streams)",
                 h2d_ceiling_images_s=G * steps / (h2d_ms / 1000.0),
                 h2d_gbs_per_gpu=B * 3 * 224 * 224 * 4 * steps / (h2d_ms / 1000.0) / 1e9),
        gpu_launches=gpu_launches, launches_per_step=launches_per_step,
        clocks=clocks, parity=parity,
        roofline=dict(bound="hbm" if hbm_bound else "tensor", kernel="tc_conv_fast_kernel (all convolution launches of a step)",
                      achieved=gbs if hbm_bound else achieved, peak=pk["hbm_gbs"] if hbm_bound else int8_burst,
                      unit="GB/s" if hbm_bound else "TFLOP/s",
                      frac=(gbs / pk["hbm_gbs"]) if hbm_bound else achieved / int8_burst,
                      traffic=traffic,
                      traffic_source="ncu dram__bytes_read.sum + dram__bytes_write.sum summed over the convolution launches "
                                     "of one step at this batch (one-pass capture); null where no capture at this batch exists",
                      algorithmic_bytes_per_step=tc_bytes, ops_per_byte=intensity, ridge_ops_per_byte=ridge,
                      peak_source=f"{pk['source']} HBM copy bandwidth; int8 tensor peak measured in this run "
                                  f"(nncb_selftest_int8_peak)",
                      tensor=dict(achieved=achieved, peak=int8_burst, peak_sustained=i8["sustained"], unit="TFLOP/s",
                                  frac=achieved / int8_burst),
                      mma_issue_pace=mma_issue_pace(ctx),
                      tc_ms_per_step=tc_ms, tc_share_of_step=tc_ms / (ms / steps),
                      whole_step_tops=2.0 * macs * B / (ms / steps / 1000.0) / 1e12),
    )
    if weak is not None:
        line["weak"] = weak
    if world == 1 and not args.no_secondary:
        line["secondary"] = secondary(torch, ctx, args, pk)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(program, 15.0)
    if args.layers:
        for r in rows:
            print(f"# {r[0]:10s} path={r[1]} {r[2] * 1000:9.1f} us  {r[3] / (r[2] / 1000) / 1e12:8.1f} TOP/s "
                  f"{r[4] / (r[2] / 1000) / 1e9:8.1f} GB/s", file=sys.stderr)
    print(json.dumps(line))
    sys.stdout.flush()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# secondary measurements (same run, after the headline): the other paths of the library
# ---------------------------------------------------------------------------------------------
def stream_kernels(torch, ctx, pk, reps=10):
    """Quantize, dequantize, binary add and max-pool at the sizes they have in ResNet-50 at 512 images:
    achieved HBM GB/s over their algorithmic bytes (inputs + outputs at their stored types)."""
    from nncase_b200 import lib as L
    from nncase_b200.kernels import QuantParam
    dev, lib, h = ctx.device, ctx._lib, ctx._h
    n_in = 512 * 3 * 224 * 224           # the network input
    n_act = 512 * 56 * 56 * 256          # a stage-1 block output
    qp = QuantParam(120, 0.03)
    xf = torch.randn(n_in, device=dev)
    xq = torch.empty(n_in, dtype=torch.uint8, device=dev)
    a = torch.randint(0, 256, (n_act,), dtype=torch.uint8, device=dev)
    b = torch.randint(0, 256, (n_act,), dtype=torch.uint8, device=dev)
    y = torch.empty_like(a)
    yf = torch.empty(n_in, device=dev)
    pool_in = torch.randint(0, 256, (512, 112, 112, 64), dtype=torch.uint8, device=dev)
    pool_out = torch.empty((512, 56, 56, 64), dtype=torch.uint8, device=dev)
    s2d_in = torch.randn((512, 3, 224, 224), device=dev)
    s2d_out = torch.empty((512, 115, 115, 16), dtype=torch.uint8, device=dev)
    cases = {
        "quantize_f32_u8": (lambda: L.check(lib.nncb_quantize(h, xf.data_ptr(), xq.data_ptr(), n_in, qp.scale, qp.zero_point, L.U8)),
                            5 * n_in),
        "dequantize_u8_f32": (lambda: L.check(lib.nncb_dequantize(h, xq.data_ptr(), yf.data_ptr(), n_in, qp.scale, qp.zero_point, L.U8)),
                              5 * n_in),
        "qadd_u8": (lambda: L.check(lib.nncb_qadd_u8(h, a.data_ptr(), b.data_ptr(), y.data_ptr(), n_act, 0.05, 117, 0.04, 125,
                                                     0.06, 121)), 3 * n_act),
        "maxpool_3x3s2_u8": (lambda: L.check(lib.nncb_maxpool_u8(h, pool_in.data_ptr(), pool_out.data_ptr(), 512, 112, 112, 64,
                                                                 3, 3, 2, 2, 1, 1, 1, 1, 120)),
                             pool_in.numel() + pool_out.numel()),
        "quantize_input_stage_s2d": (lambda: L.check(lib.nncb_quantize_to_s2d_padded_u8(
            h, s2d_in.data_ptr(), 0, s2d_out.data_ptr(), 512, 3, 224, 224, 16, 2, 1, 2, 1, qp.scale, qp.zero_point)),
            s2d_in.numel() * 4 + s2d_out.numel()),
    }
    out = {}
    for name, (call, nbytes) in cases.items():
        for _ in range(3):
            call()
        e0, e1 = _events(torch)
        torch.cuda.synchronize(dev)
        e0.record()
        for _ in range(reps):
            call()
        e1.record()
        torch.cuda.synchronize(dev)
        us = e0.elapsed_time(e1) / reps * 1000.0
        gbs = nbytes / (us * 1e-6) / 1e9
        out[name] = dict(us=us, algorithmic_bytes=nbytes, gbs=gbs, frac_of_hbm_peak=gbs / pk["hbm_gbs"])
    ctx.check_status()
    return out


def latency_one_image(torch, ctx, which):
    """Single-image latency of a whole network replayed as one CUDA graph (capture / replay of CudaFunction)."""
    from nncase_b200 import builder, networks
    from nncase_b200.runtime import CudaFunction
    dev = ctx.device
    if which == "resnet50v2":
        graph, shape = networks.resnet50v2(SEED_W), (1, 3, 224, 224)
        cal = [np.random.default_rng(SEED_CAL + i).normal(0, 1, shape).astype(np.float32) for i in range(16)]
        x = torch.randn(shape, device=dev)
    else:
        graph, shape = networks.mobilenetv2(1002), (1, 224, 224, 3)
        cal = [(np.random.default_rng(3002 + i).uniform(0, 1, shape).astype(np.float32) - 0.5) / 0.5 for i in range(16)]
        x = (torch.rand(shape, device=dev) - 0.5) / 0.5
    program = builder.build_program(graph, cal, device=dev)
    fn = CudaFunction(program, 1, ctx)
    fn.capture(x)
    for _ in range(5):
        fn.replay()
    e0, e1 = _events(torch)
    torch.cuda.synchronize(dev)
    reps = 50
    e0.record()
    for _ in range(reps):
        fn.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    ctx.check_status()
    us = e0.elapsed_time(e1) / reps * 1000.0
    launches = fn.launches_per_call
    fn.close()
    return dict(us_per_image=us, images_per_s=1e6 / us, launches=launches, mode="CUDA graph replay, batch 1")


def measure_matmuls(torch, ctx, pk, reps=100):
    """The five w8a16 MatMuls of a Qwen2-0.5B-shaped decode step at 64 tokens, each replayed `reps` times in one CUDA
    graph (weights warm in L2 except the LM head, which is larger than L2): microseconds per call, weight GB/s, and the
    form that ran (tcgen05 for more than 32 tokens on matrices of 128 K weights or more, mma.sync otherwise)."""
    from nncase_b200 import lib as L
    dev = ctx.device
    lib, h = ctx._lib, ctx._h
    out = {}
    shapes = [("qkv", 1152, 896, False, reps), ("o", 896, 896, False, reps), ("down", 896, 4864, False, reps),
              ("gate_up_swiglu", 9728, 896, True, reps), ("lm_head", 151936, 896, False, max(4, reps // 5))]
    M = 64
    g = torch.Generator(device=dev).manual_seed(2007)
    for name, N, K, swiglu, n_rep in shapes:
        x = torch.randn((M, K), dtype=torch.float16, device=dev, generator=g)
        w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev, generator=g)
        sc = torch.rand((N,), dtype=torch.float16, device=dev, generator=g) * 0.01
        y = torch.empty((M, N // 2 if swiglu else N), dtype=torch.float16, device=dev)

        def call():
            if swiglu:
                L.check(lib.nncb_gemv_w8a16_swiglu(h, x.data_ptr(), w.data_ptr(), sc.data_ptr(), None, y.data_ptr(), M, N, K))
            else:
                L.check(lib.nncb_gemv_w8a16(h, x.data_ptr(), w.data_ptr(), sc.data_ptr(), None, None, y.data_ptr(), M, N, K))

        ctx.use_current_stream()
        for _ in range(3):
            call()
        torch.cuda.synchronize(dev)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                ctx.use_current_stream()
                for _ in range(n_rep):
                    call()
        ctx.use_current_stream()
        graph.replay()
        torch.cuda.synchronize(dev)
        a, b = _events(torch)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize(dev)
        us = a.elapsed_time(b) / n_rep * 1e3
        out[name] = dict(n=N, k=K, us=round(us, 2), weight_gbs=round(N * K / us / 1e3, 1),
                         form="tcgen05" if M > 32 and N * K >= (1 << 17) else "mma.sync")
        del graph
    ctx.check_status()
    out["tokens"] = M
    return out


def secondary(torch, ctx, args, pk):
    out = {}
    out["stream_kernels"] = stream_kernels(torch, ctx, pk)
    out["paged_attention"] = measure_attention(torch, ctx, pk, steps=20, warmup=3)
    out["decode"] = measure_decode(torch, ctx, pk, steps=20, warmup=3, world=1, rank=0)
    out["decode_matmuls"] = measure_matmuls(torch, ctx, pk)
    out["latency_batch1"] = dict(resnet50v2=latency_one_image(torch, ctx, "resnet50v2"),
                                 mobilenetv2=latency_one_image(torch, ctx, "mobilenetv2"))
    torch.cuda.empty_cache()
    return out


def run_layer(args):
    """Times one convolution layer of the network alone (for profiling): `--layer NAME`."""
    import torch
    from nncase_b200 import lib as L
    from nncase_b200.kernels import Context
    from nncase_b200.runtime import CudaFunction
    dev = torch.device("cuda", 0)
    graph, program, macs, layer_macs = build_network(dev, args.w_quant)
    want = args.layer
    keep = [op for op in program["ops"] if op["op"] == "conv" and op["name"] == want]
    if not keep:
        raise SystemExit(f"no conv layer named {want}; layers: {[o['name'] for o in program['ops'] if o['op'] == 'conv']}")
    op = keep[0]
    sub = dict(program, ops=[op])
    ctx = Context(0)
    fn = CudaFunction(sub, args.batch, ctx)
    g = torch.Generator(device=dev).manual_seed(1)
    for name in (op["in"], op.get("res")):
        if name:
            fn.buffers[name].copy_(torch.randint(0, 256, fn.buffers[name].shape, device=dev, generator=g, dtype=torch.uint8))
    plan = fn.plans[0]
    res = fn.buffers[op["res"]] if op.get("res") else None
    y2 = fn.buffers[op["y2"]] if op.get("y2") else None
    for _ in range(max(1, args.warmup)):
        plan(fn.buffers[op["in"]], res, fn.buffers[op["out"]], y2)
    torch.cuda.synchronize()
    a, b = _events(torch)
    a.record()
    for _ in range(args.steps):
        plan(fn.buffers[op["in"]], res, fn.buffers[op["out"]], y2)
    b.record()
    torch.cuda.synchronize()
    ctx.check_status()
    ms = a.elapsed_time(b) / args.steps
    n, oh, ow, oc = plan.out_shape
    in_bytes = fn.buffers[op["in"]].numel()
    out_bytes = n * oh * ow * oc * (1 + (1 if res is not None else 0) + (1 if y2 is not None else 0))
    print(json.dumps(dict(layer=want, batch=args.batch, path=plan.path, ms=ms,
                          tops=2.0 * layer_macs[want] * args.batch / (ms / 1000) / 1e12,
                          algorithmic_bytes=in_bytes + out_bytes + op["w"].size,
                          gbs=(in_bytes + out_bytes + op["w"].size) / (ms / 1000) / 1e9)))


def measure_attention(torch, ctx, pk, steps, warmup, batch=64):
    """Paged-attention decode at the Qwen2-0.5B decode shape (batch 64, context 2048, 14 query / 2 kv heads,
    head_dim 64, 16-token f16 pages, random block-table permutation). One step = the attention of all 24
    layers, each over its own KV pool (1.61 GB of K/V per step, larger than L2), replayed as one CUDA graph;
    achieved HBM GB/s over the K/V bytes referenced."""
    dev = ctx.device
    B, Hq, Hkv, D, page, n_ctx, layers = batch, 14, 2, 64, 16, 2048, 24
    pages = B * n_ctx // page
    g = torch.Generator(device=dev).manual_seed(2005)
    pools = [(torch.randn((pages, Hkv, page, D), device=dev, generator=g, dtype=torch.float16),
              torch.randn((pages, Hkv, page, D), device=dev, generator=g, dtype=torch.float16)) for _ in range(layers)]
    q = torch.randn((B, Hq, D), device=dev, generator=g, dtype=torch.float16)
    table = torch.randperm(pages, device=dev, generator=g).to(torch.int32).reshape(B, n_ctx // page).contiguous()
    lens = torch.full((B,), n_ctx, dtype=torch.int32, device=dev)
    ws = torch.empty(1 << 22, dtype=torch.uint8, device=dev)

    def step():
        for k, v in pools:
            ctx.paged_attention_decode(q, k, v, table, lens, workspace=ws)

    for _ in range(max(3, warmup)):
        step()
    torch.cuda.synchronize(dev)
    l0 = ctx.launches
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph):
            ctx.use_current_stream()
            step()
    ctx.use_current_stream()
    launches_per_step = ctx.launches - l0
    graph.replay()
    torch.cuda.synchronize(dev)
    a, b = _events(torch)
    a.record()
    for _ in range(steps):
        graph.replay()
    b.record()
    torch.cuda.synchronize(dev)
    ctx.check_status()
    ms = a.elapsed_time(b) / steps
    kv_bytes = layers * B * n_ctx * Hkv * D * 2 * 2
    gbs = kv_bytes / (ms / 1000) / 1e9
    del graph, pools
    torch.cuda.empty_cache()
    return dict(metric="paged-attention decode HBM GB/s", value=gbs, unit="GB/s", ms_per_step=ms, steps=steps,
                kv_bytes_per_step=kv_bytes, launches_per_step=launches_per_step,
                config=dict(workload="qwen2_0.5b_decode_attention", batch=B, context=n_ctx, q_heads=Hq, kv_heads=Hkv,
                            head_dim=D, page=page, layers=layers),
                roofline=dict(bound="hbm", achieved=gbs, peak=pk["hbm_gbs"], unit="GB/s", frac=gbs / pk["hbm_gbs"],
                              peak_source=pk["source"]))


def measure_decode(torch, ctx, pk, steps, warmup, world, rank, fused_rope=True, peer_reduce=True):
    """One decode step of the Qwen2-0.5B-shaped model (24 layers, hidden 896, 14/2 heads, SwiGLU 4864,
    vocabulary 151936, i8 weights, f16 activations, paged f16 KV cache) at batch 64 and context 2048, tensor
    parallel over `world` ranks, replayed as one CUDA graph. Tokens/s and the HBM bytes a step must read
    (KV pages referenced + weights) over the measured time."""
    import torch.distributed as dist
    from nncase_b200 import decoder as D
    from nncase_b200 import sharding
    dev = ctx.device
    cfg = D.DecoderConfig()
    B, n_ctx = 64, 2048
    weights = D.make_weights(cfg, 1005)
    max_pages = n_ctx // cfg.page + 1
    num_pages = B * max_pages
    dec = D.Decoder(cfg, weights, B, num_pages, ctx=ctx, world=world, rank=rank, fused_rope=fused_rope, peer_reduce=peer_reduce)
    g = torch.Generator(device=dev).manual_seed(2005)
    for lw in dec.layers:
        lw["k_pool"].normal_(generator=g)
        lw["v_pool"].normal_(generator=g)
    table = torch.randperm(num_pages, device=dev, generator=g).to(torch.int32).reshape(B, max_pages).contiguous()
    ids = torch.randint(0, cfg.vocab, (B,), device=dev, generator=g, dtype=torch.int32)
    pos = torch.full((B,), n_ctx - 1, dtype=torch.int32, device=dev)
    for _ in range(max(3, warmup)):
        dec.step(ids, pos, table)
    torch.cuda.synchronize(dev)
    l0 = ctx.launches
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph):
            ctx.use_current_stream()
            dec.step(ids, pos, table)
    ctx.use_current_stream()
    launches_per_step = ctx.launches - l0
    graph.replay()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    a, b = _events(torch)
    a.record()
    for _ in range(steps):
        graph.replay()
    b.record()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    ms = sharding.max_over_ranks([a.elapsed_time(b) / steps], dev)[0]
    ctx.check_status()
    kv = cfg.layers * B * n_ctx * cfg.kv_heads * cfg.head_dim * 2 * 2
    H, nq, nkv = cfg.hidden, cfg.q_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
    wbytes = cfg.layers * ((nq + 2 * nkv) * H + H * nq + 2 * cfg.inter * H + H * cfg.inter) + cfg.vocab * H
    gbs = (kv + wbytes) / world / (ms / 1000) / 1e9  # per GPU: each rank reads its share
    res = dict(metric="Qwen2-0.5B-shape decode tokens/s", value=B / (ms / 1000), unit="tokens/s", n_gpus=world,
               ms_per_step=ms, steps=steps, launches_per_step=launches_per_step,
               config=dict(workload="qwen2_0.5b_decode", batch=B, context=n_ctx, layers=cfg.layers,
                           parallelism=dec.parallelism, weights="i8 per-channel, f16 scales", kv="f16, 16-token pages"),
               bytes_per_step=dict(kv=kv, weights=wbytes),
               roofline=dict(bound="hbm", achieved=gbs, peak=pk["hbm_gbs"], unit="GB/s per GPU", frac=gbs / pk["hbm_gbs"],
                             peak_source=pk["source"]))
    del graph
    torch.cuda.synchronize(dev)
    return res


def run_streams(args):
    """Only the streaming kernels (profiling aid): one JSON line with their achieved GB/s."""
    import torch
    from nncase_b200.kernels import Context
    ctx = Context(0)
    print(json.dumps(stream_kernels(torch, ctx, peaks(), reps=max(1, args.steps))))


def run_attention(args):
    import torch
    from nncase_b200.kernels import Context
    ctx = Context(0)
    print(json.dumps(measure_attention(torch, ctx, peaks(), args.steps, args.warmup, args.attention_batch)))


def run_decode(args):
    import torch
    import torch.distributed as dist
    from nncase_b200.kernels import Context
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = Context(local)
    options = {}
    for item in args.option:
        name, _, value = item.partition("=")
        ctx.set_option(name, int(value))
        options[name] = int(value)
    res = measure_decode(torch, ctx, peaks(), args.steps, args.warmup, world, rank, fused_rope=not args.separate_rope, peer_reduce=not args.nccl_reduce)
    if options:
        res["config"]["options"] = options
    if rank == 0:
        print(json.dumps(res))
    # A CUDA graph that held captured NCCL kernels kept the communicator busy: the graph is dropped inside
    # measure_decode, the device drained; line the ranks up and leave without the NCCL teardown.
    sys.stdout.flush()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=512, help="global batch: images per step over all GPUs")
    ap.add_argument("--w-quant", default="uint8", choices=["uint8", "int8"])
    ap.add_argument("--layers", action="store_true", help="print per-layer timings to stderr")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary measurements (attention, decode, ...)")
    ap.add_argument("--layer", default=None, help="time only this conv layer (profiling aid)")
    ap.add_argument("--matmuls", action="store_true", help="only the w8a16 MatMuls of a decode step (64 tokens)")
    ap.add_argument("--attention", action="store_true", help="only the paged-attention decode measurement")
    ap.add_argument("--attention-batch", type=int, default=64, help="sequences of the --attention measurement (74 = one (sequence, kv head) pair per SM of a 148-SM part)")
    ap.add_argument("--decode", action="store_true", help="only the decoder step (tensor parallel under torchrun)")
    ap.add_argument("--separate-rope", action="store_true",
                    help="with --decode: rotary embedding and KV append as a launch of their own instead of inside the attention launch")
    ap.add_argument("--nccl-reduce", action="store_true",
                    help="with --decode under torchrun: NCCL all-reduce + norm kernel instead of the kernel over peer memory")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="with --decode: set a context option first (launch.overlap=0, matmul.tensor_core=0, ...); repeatable")
    ap.add_argument("--streams", action="store_true", help="only the streaming kernels (quantize, dequantize, add, max-pool, input stage)")
    args = ap.parse_args()
    if args.streams:
        run_streams(args)
    elif args.decode:
        run_decode(args)
    elif args.matmuls:
        import torch
        from nncase_b200.kernels import Context
        print(json.dumps(measure_matmuls(torch, Context(0), peaks(), reps=max(4, args.steps))))
    elif args.attention:
        run_attention(args)
    elif args.layer:
        run_layer(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
