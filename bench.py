#!/usr/bin/env python
"""Benchmark of the quantized-inference hot path: u8/u8 ResNet-50 v2 images/s on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]
                  [--w-quant uint8|int8] [--layers]

One step = one forward pass of the whole quantized network over one batch of synthetic images
per GPU (seeded N(0,1) inputs standing in for ImageNet; random He-normal weights, BN folded).
For N > 1 launch under torchrun, one rank per GPU; the batch is sharded by images with no
collective on the data path (weak scaling: every GPU runs `--batch` images).

Prints ONE JSON line (rank 0). `value` is device-resident throughput, `e2e` the same metric
through the public host-buffer call (pinned f32 input -> H2D -> kernels -> D2H logits, copies
double-buffered inside the timed region). `--impl reference` times the reference's own CPU
kernels (dequantize -> conv2d f32 -> quantize, ...) on the host cores on a bounded sample.
"""
import argparse
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


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_burst=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_burst=1590.0, bf16_sustained=1400.0, source="fallback")


# DRAM bytes (read + write) of all convolution launches of one step, from one ncu capture of this
# workload (dram__bytes_read.sum + dram__bytes_write.sum, summed over the tcgen05 convolution
# kernels of a step); None until a capture at that size exists. Keyed by (images per GPU, weights).
MEASURED_DRAM_BYTES_PER_STEP = {(512, "uint8"): 17.181e9}


def measured_traffic(batch, w_quant):
    return MEASURED_DRAM_BYTES_PER_STEP.get((batch, w_quant))


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


def build_network(batch_for_calib_device, w_quant):
    from nncase_b200 import builder, networks
    graph = networks.resnet50v2(SEED_W)
    cal = [np.random.default_rng(SEED_CAL + i).normal(0, 1, (1, 3, 224, 224)).astype(np.float32) for i in range(16)]
    program = builder.build_program(graph, cal, w_quant, device=batch_for_calib_device)
    macs, per_layer, _ = networks.graph_macs(graph)
    return graph, program, macs, dict(per_layer)


# ---------------------------------------------------------------------------------------------
# reference arm: the reference's own CPU kernels on the host cores
# ---------------------------------------------------------------------------------------------
def cpu_reference_sample(graph, program, macs_total, seconds_target=20.0, threads=None):
    """Times the reference's CPU implementation of the path on a bounded sample of the workload.

    Sample: one image; the stem, the max-pool, every `stride`-th convolution layer (with its
    residual add / ReLU requantisation) run through the reference's kernels exactly as its cpu
    target executes a quantized convolution: dequantize -> conv2d(f32, fused clamp) -> quantize.
    Layers are independent jobs spread over all host cores (the reference kernel itself is
    single-threaded). images/s is extrapolated by the sample's share of the network's MACs.
    """
    from oracle import program as oprog
    from oracle import qoracle, ref
    threads = threads or os.cpu_count() or 1
    x = np.random.default_rng(SEED_X).normal(0, 1, (1, 3, 224, 224)).astype(np.float32)
    _, tens = oprog.run_program(program, x, threads=threads)  # inputs of every layer, from the oracle
    convs = [op for op in program["ops"] if op["op"] == "conv" and not op.get("f32_out")]
    use_ref = ref.available()
    # reference f32 conv runs at ~0.3 GMAC/s per core: choose how many layers fit the time target
    est_rate = 0.3e9 if use_ref else 3e9
    layer_macs = []
    for op in convs:
        n, oh, ow, oc = tens[op["out"]].shape
        layer_macs.append(oh * ow * oc * op["w"].shape[1] * op["w"].shape[2] * op["w"].shape[3])
    budget = est_rate * seconds_target * threads
    order = np.argsort(layer_macs)[::-1]
    stride = max(1, int(np.ceil(sum(layer_macs) / budget)))
    chosen = sorted(order[::stride].tolist())
    T = program["tensors"]

    job_seconds = []

    def job(i):
        t_job = time.perf_counter()
        op = convs[i]
        xq, xqp, cq = tens[op["in"]], T[op["in"]]["qp"], op["conv_qp"]
        if use_ref:
            sw = op["mult"] / np.float32(xqp.scale)
            ref.qconv2d_composite_u8(xq, op["w"], op["w_zp"], sw, op["bias"], xqp.scale, xqp.zero_point, cq.scale,
                                     cq.zero_point, op["stride"], op["pad"], op["dil"], op["groups"], op["clamp"])
        else:
            qoracle.qconv2d_u8(xq, op["w"], op["w_zp"], op["mult"], op["bias"], xqp.zero_point, cq.scale,
                               cq.zero_point, op["stride"], op["pad"], op["dil"], op["groups"], op["clamp"])
        job_seconds.append(time.perf_counter() - t_job)

    if not use_ref:
        qoracle.lib().qo_set_threads(1)
    t0 = time.perf_counter()
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(job, chosen))
    dt = time.perf_counter() - t0
    sample_macs = sum(layer_macs[i] for i in chosen)
    macs_total = sum(layer_macs)  # same counting as the sample (the FC layer, 0.05 % of the MACs, is left out)
    # core-seconds the sample took (each layer ran on one core) -> core-seconds per image at
    # full-network MACs -> images/s with every core busy on its own image
    core_seconds = sum(job_seconds)
    img_per_s = threads / (core_seconds * macs_total / sample_macs)
    return dict(value=img_per_s, unit=UNIT, cores=threads, kind="reference" if use_ref else "port",
                sample=f"1 image, {len(chosen)} of {len(convs)} conv layers ({sample_macs / macs_total:.1%} of the "
                       f"network's MACs) through dequantize->conv2d(f32)->quantize, {dt:.1f} s wall, "
                       f"extrapolated by MACs"), dt


def run_reference(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    graph, program, macs, _ = build_network("cpu", args.w_quant)
    vals, last = [], None
    steps = max(1, args.steps)
    per_step = max(3.0, min(20.0, 150.0 / (steps + args.warmup)))
    for i in range(args.warmup + steps):
        cb, dt = cpu_reference_sample(graph, program, macs, per_step)
        if i >= args.warmup:
            vals.append(cb["value"])
            last = cb
    v = float(np.mean(vals))
    last["value"] = v
    line = dict(metric=METRIC, value=v, unit=UNIT, n_gpus=args.gpus, steps=steps, warmup=args.warmup,
                ms_per_step=1000.0 * args.batch / v, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="f32", data="synthetic", impl="reference",
                config=dict(workload="resnet50v2_u8u8", batch_per_gpu=args.batch, w_quant=args.w_quant),
                cpu_baseline=last, e2e=dict(value=v, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
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
    from nncase_b200.kernels import Context
    from nncase_b200.runtime import CudaFunction

    dev = torch.device("cuda", local)
    graph, program, macs, layer_macs = build_network(dev, args.w_quant)
    ctx = Context(local)
    fn = CudaFunction(program, args.batch, ctx)
    B = args.batch
    g = torch.Generator(device=dev).manual_seed(SEED_X + rank)
    x = torch.randn((B, 3, 224, 224), device=dev, generator=g)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # -------- device-resident throughput --------
    for _ in range(max(3, args.warmup)):
        fn.invoke(x)
    ctx.check_status()
    launches_per_step = fn.launches_per_call
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = ctx.launches
    ev0.record()
    for _ in range(args.steps):
        fn.invoke(x)
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    gpu_launches = ctx.launches - l0
    ctx.check_status()

    # -------- end to end through the host-buffer call --------
    xh = [torch.empty((B, 3, 224, 224), dtype=torch.float32).pin_memory() for _ in range(2)]
    for t in xh:
        t.copy_(x)
    oh = [torch.empty((B, 1, 1, 1000), dtype=torch.float32).pin_memory() for _ in range(2)]
    copy_stream, comp_stream = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    xd = [torch.empty_like(x) for _ in range(2)]
    e2e_steps = args.steps

    def e2e_loop(steps):
        # double buffered: the H2D copy of step i+1 overlaps the kernels of step i; every
        # step's input copy and result read-back are inside the timed region
        copied = [torch.cuda.Event() for _ in range(2)]
        done = [torch.cuda.Event() for _ in range(2)]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(copy_stream):
            start.record()
            xd[0].copy_(xh[0], non_blocking=True)
            copied[0].record()
        for i in range(steps):
            b = i & 1
            if i + 1 < steps:
                with torch.cuda.stream(copy_stream):
                    if i >= 1:
                        copy_stream.wait_event(done[b ^ 1])
                    xd[b ^ 1].copy_(xh[b ^ 1], non_blocking=True)
                    copied[b ^ 1].record()
            with torch.cuda.stream(comp_stream):
                comp_stream.wait_event(copied[b])
                out = fn.invoke(xd[b])
                oh[b].copy_(out, non_blocking=True)
                done[b].record()
        with torch.cuda.stream(comp_stream):
            comp_stream.wait_stream(copy_stream)
            end.record()
        comp_stream.synchronize()
        copy_stream.synchronize()
        return start.elapsed_time(end)

    e2e_loop(3)
    barrier()
    e2e_ms = e2e_loop(e2e_steps)
    barrier()
    ctx.use_current_stream()
    clocks = sampler.stop() if rank == 0 else None

    # -------- per-layer timing of the dominant kernel (tcgen05 conv) for the roofline --------
    tc_ops, tc_ms, tc_bytes, rows = 0.0, 0.0, 0.0, []
    reps = 5
    for st in fn.steps:
        if st[0] != "conv":
            continue
        op, plan = st[1], st[2]
        res = fn.buffers[op["res"]] if op.get("res") else None
        y2 = fn.buffers[op["y2"]] if op.get("y2") else None
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        plan(fn.buffers[op["in"]], res, fn.buffers[op["out"]], y2)
        torch.cuda.synchronize(dev)
        a.record()
        for _ in range(reps):
            plan(fn.buffers[op["in"]], res, fn.buffers[op["out"]], y2)
        b.record()
        torch.cuda.synchronize(dev)
        t = a.elapsed_time(b) / reps
        ops = 2.0 * layer_macs[op["name"]] * B
        # algorithmic bytes of the launch: activations in, every tensor written or added, weights once
        n_, oh_, ow_, oc_ = plan.out_shape
        out_el = n_ * oh_ * ow_ * oc_
        nbytes = (fn.buffers[op["in"]].numel() + out_el * (4 if op.get("f32_out") else 1) +
                  (out_el if res is not None else 0) + (out_el if y2 is not None else 0) + op["w"].size)
        rows.append((op["name"], plan.path, t, ops, nbytes))
        if plan.path == L.PATH_TC:
            tc_ops += ops
            tc_ms += t
            tc_bytes += nbytes
    ctx.check_status()

    # max over ranks of the device-measured times, sum of the launch counters
    from nncase_b200 import sharding
    ms, e2e_ms = sharding.max_over_ranks([ms, e2e_ms], dev)
    gpu_launches = sharding.sum_over_ranks([gpu_launches], dev)[0]
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    pk = peaks()
    value = world * B * args.steps / (ms / 1000.0)
    e2e_value = world * B * e2e_steps / (e2e_ms / 1000.0)
    int8_peak = 2.0 * pk["bf16_burst"]  # dense int8 = 2x the measured dense bf16 (int8 itself is not in the peaks file)
    achieved = tc_ops / (tc_ms / 1000.0) / 1e12 if tc_ms > 0 else 0.0
    # The convolution launches of one step move tc_bytes and do tc_ops: their ratio (operations per
    # byte) lies below the ridge point int8 peak / HBM peak, so HBM bandwidth is the roof that bounds
    # the kernel on this workload; the tensor-pipe figures are kept beside it.
    gbs = tc_bytes / (tc_ms / 1000.0) / 1e9 if tc_ms > 0 else 0.0
    intensity = tc_ops / tc_bytes if tc_bytes else 0.0
    ridge = int8_peak * 1e12 / (pk["hbm_gbs"] * 1e9)
    hbm_bound = intensity < ridge
    line = dict(
        metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=args.steps, warmup=max(3, args.warmup),
        ms_per_step=ms / args.steps, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="u8",
        data="synthetic", impl="ours",
        config=dict(workload="resnet50v2_u8u8", batch_per_gpu=B, global_batch=B * world, w_quant=args.w_quant,
                    input="f32 NCHW [B,3,224,224] N(0,1)", l2="inputs and activations larger than L2 (no flush)",
                    parallelism=f"batch-sharded x{world}, no collective"),
        e2e=dict(value=e2e_value, unit=UNIT, h2d_bytes_per_step=B * 3 * 224 * 224 * 4, d2h_bytes_per_step=B * 1000 * 4),
        gpu_launches=gpu_launches, launches_per_step=launches_per_step,
        clocks=clocks,
        roofline=dict(bound="hbm" if hbm_bound else "tensor", kernel="tc_conv_fast_kernel (all convolution launches of a step)",
                      achieved=gbs if hbm_bound else achieved, peak=pk["hbm_gbs"] if hbm_bound else int8_peak,
                      unit="GB/s" if hbm_bound else "TFLOP/s",
                      frac=(gbs / pk["hbm_gbs"]) if hbm_bound else achieved / int8_peak,
                      traffic=measured_traffic(B, args.w_quant),
                      algorithmic_bytes_per_step=tc_bytes, ops_per_byte=intensity, ridge_ops_per_byte=ridge,
                      peak_source=f"{pk['source']} peaks: HBM copy bandwidth; int8 dense taken as 2 x bf16 burst",
                      tensor=dict(achieved=achieved, peak=int8_peak, unit="TFLOP/s", frac=achieved / int8_peak),
                      tc_ms_per_step=tc_ms, tc_share_of_step=tc_ms / (ms / args.steps),
                      whole_step_tops=2.0 * macs * B / (ms / args.steps / 1000.0) / 1e12),
    )
    if world == 1 and not args.no_cpu_baseline:
        cb, _ = cpu_reference_sample(graph, program, macs, 15.0)
        line["cpu_baseline"] = cb
    if args.layers:
        for r in rows:
            print(f"# {r[0]:10s} path={r[1]} {r[2] * 1000:9.1f} us  {r[3] / (r[2] / 1000) / 1e12:8.1f} TOP/s "
                  f"{r[4] / (r[2] / 1000) / 1e9:8.1f} GB/s", file=sys.stderr)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


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
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
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


def run_attention(args):
    """Secondary measurement: paged-attention decode at the Qwen2-0.5B decode shape (batch 64, context
    2048, 14 query / 2 kv heads, head_dim 64, 16-token f16 pages, random block-table permutation).
    One step = the attention of all 24 layers, each over its own KV pool (1.61 GB of K/V per step,
    larger than L2), reported as achieved HBM GB/s over the K/V bytes referenced."""
    import torch
    from nncase_b200.kernels import Context
    dev = torch.device("cuda", 0)
    ctx = Context(0)
    B, Hq, Hkv, D, page, n_ctx, layers = 64, 14, 2, 64, 16, 2048, 24
    pages = B * n_ctx // page
    g = torch.Generator(device=dev).manual_seed(2005)
    pools = [(torch.randn((pages, Hkv, page, D), device=dev, generator=g, dtype=torch.float16),
              torch.randn((pages, Hkv, page, D), device=dev, generator=g, dtype=torch.float16)) for _ in range(layers)]
    q = torch.randn((B, Hq, D), device=dev, generator=g, dtype=torch.float16)
    table = torch.randperm(pages, device=dev, generator=g).to(torch.int32).reshape(B, n_ctx // page).contiguous()
    lens = torch.full((B,), n_ctx, dtype=torch.int32, device=dev)
    need = 1 << 22
    ws = torch.empty(need, dtype=torch.uint8, device=dev)

    def step():
        for k, v in pools:
            ctx.paged_attention_decode(q, k, v, table, lens, workspace=ws)

    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    # a decode step is launch-bound from Python (24 short kernels): replay it as one CUDA graph
    l0 = ctx.launches
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ctx.use_current_stream()
        step()
    ctx.use_current_stream()
    launches_per_step = ctx.launches - l0
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    ctx.check_status()
    ms = a.elapsed_time(b) / args.steps
    kv_bytes = layers * B * n_ctx * Hkv * D * 2 * 2
    pk = peaks()
    gbs = kv_bytes / (ms / 1000) / 1e9
    print(json.dumps(dict(metric="paged-attention decode HBM GB/s", value=gbs, unit="GB/s", ms_per_step=ms,
                          steps=args.steps, kv_bytes_per_step=kv_bytes, gpu_launches=launches_per_step * args.steps,
                          config=dict(workload="qwen2_0.5b_decode_attention", batch=B, context=n_ctx, q_heads=Hq,
                                      kv_heads=Hkv, head_dim=D, page=page, layers=layers),
                          roofline=dict(bound="hbm", achieved=gbs, peak=pk["hbm_gbs"], unit="GB/s",
                                        frac=gbs / pk["hbm_gbs"], peak_source=pk["source"]))))


def run_decode(args):
    """Secondary measurement: one decode step of the Qwen2-0.5B-shaped model (24 layers, hidden 896,
    14/2 heads, SwiGLU 4864, vocabulary 151936, i8 weights, f16 activations, paged f16 KV cache) at
    batch 64 and context 2048, tensor parallel over the launched ranks (NCCL all-reduce after the o
    and down projections). The step is replayed as one CUDA graph. Reports tokens/s and the HBM
    bytes a step must read (KV pages referenced + weights) over the measured time."""
    import torch
    import torch.distributed as dist
    from nncase_b200 import decoder as D
    from nncase_b200 import sharding
    from nncase_b200.kernels import Context
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = D.DecoderConfig()
    B, n_ctx = 64, 2048
    weights = D.make_weights(cfg, 1005)
    max_pages = n_ctx // cfg.page + 1
    num_pages = B * max_pages
    ctx = Context(local)
    dec = D.Decoder(cfg, weights, B, num_pages, ctx=ctx, world=world, rank=rank)
    g = torch.Generator(device=dev).manual_seed(2005)
    for lw in dec.layers:
        lw["k_pool"].normal_(generator=g)
        lw["v_pool"].normal_(generator=g)
    table = torch.randperm(num_pages, device=dev, generator=g).to(torch.int32).reshape(B, max_pages).contiguous()
    ids = torch.randint(0, cfg.vocab, (B,), device=dev, generator=g, dtype=torch.int32)
    pos = torch.full((B,), n_ctx - 1, dtype=torch.int32, device=dev)
    for _ in range(max(3, args.warmup)):
        dec.step(ids, pos, table)
    torch.cuda.synchronize()
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
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = sharding.max_over_ranks([a.elapsed_time(b) / args.steps], dev)[0]
    ctx.check_status()
    if rank == 0:
        kv = cfg.layers * B * n_ctx * cfg.kv_heads * cfg.head_dim * 2 * 2
        H, nq, nkv = cfg.hidden, cfg.q_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
        wbytes = cfg.layers * ((nq + 2 * nkv) * H + H * nq + 2 * cfg.inter * H + H * cfg.inter) + cfg.vocab * H
        pk = peaks()
        gbs = (kv + wbytes) / world / (ms / 1000) / 1e9  # per GPU: each rank reads its share
        print(json.dumps(dict(metric="Qwen2-0.5B-shape decode tokens/s", value=B / (ms / 1000), unit="tokens/s",
                              n_gpus=world, ms_per_step=ms, steps=args.steps, launches_per_step=launches_per_step,
                              config=dict(workload="qwen2_0.5b_decode", batch=B, context=n_ctx, layers=cfg.layers,
                                          parallelism=f"tp{world}", weights="i8 per-channel, f16 scales",
                                          kv="f16, 16-token pages"),
                              bytes_per_step=dict(kv=kv, weights=wbytes),
                              roofline=dict(bound="hbm", achieved=gbs, peak=pk["hbm_gbs"], unit="GB/s per GPU",
                                            frac=gbs / pk["hbm_gbs"], peak_source=pk["source"]))))
    # A CUDA graph that holds captured NCCL kernels keeps the communicator busy: tearing the process
    # group down while it is alive can block forever. Drop the graph, drain the device, line the ranks
    # up and leave without the NCCL teardown.
    sys.stdout.flush()
    del graph
    torch.cuda.synchronize()
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
    ap.add_argument("--batch", type=int, default=512, help="images per GPU per step")
    ap.add_argument("--w-quant", default="uint8", choices=["uint8", "int8"])
    ap.add_argument("--layers", action="store_true", help="print per-layer timings to stderr")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layer", default=None, help="time only this conv layer (profiling aid)")
    ap.add_argument("--attention", action="store_true", help="secondary metric: paged-attention decode GB/s")
    ap.add_argument("--decode", action="store_true", help="secondary metric: decoder step tokens/s (tensor parallel under torchrun)")
    args = ap.parse_args()
    if args.decode:
        run_decode(args)
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
