"""Whole-program parity on the GPU: every tensor of the quantized networks bit-exact against the
oracle's op-by-op replay, through the runtime function (C ABI underneath)."""
import numpy as np
import pytest
import torch

from nncase_b200 import builder, networks
from nncase_b200 import lib as L
from nncase_b200.runtime import CudaFunction
from oracle import program as oprog

pytestmark = pytest.mark.gpu


def test_config1_single_conv(ctx):
    """[1,64,56,56] f32 NCHW -> quantize -> 3x3 conv + ReLU6 -> u8, PTQ from 8 seeded samples."""
    graph = networks.single_conv(1001)
    cal = [np.random.default_rng(3001 + i).uniform(-1, 1, (1, 64, 56, 56)).astype(np.float32) for i in range(8)]
    program = builder.build_program(graph, cal)
    x = np.random.default_rng(2001).uniform(-1, 1, (1, 64, 56, 56)).astype(np.float32)
    fn = CudaFunction(program, 1, ctx)
    assert fn.conv_paths["conv"] == L.PATH_TC
    got = fn.invoke(torch.from_numpy(x).cuda()).cpu().numpy()
    ctx.check_status()
    want, _ = oprog.run_program(program, x)
    assert np.array_equal(got, want)
    fn.close()


@pytest.mark.parametrize("w_quant", ["uint8", "int8"])
def test_resnet50v2_every_tensor(ctx, w_quant):
    graph = networks.resnet50v2(1003)
    cal = [np.random.default_rng(3003 + i).normal(0, 1, (1, 3, 224, 224)).astype(np.float32) for i in range(2)]
    program = builder.build_program(graph, cal, w_quant)
    n = 3
    x = np.random.default_rng(2003).normal(0, 1, (n, 3, 224, 224)).astype(np.float32)
    fn = CudaFunction(program, n, ctx)
    paths = fn.conv_paths
    assert all(p == L.PATH_TC for p in paths.values()), paths
    out = fn.invoke(torch.from_numpy(x).cuda())
    ctx.check_status()
    want, tens = oprog.run_program(program, x)
    for name, ref_t in tens.items():
        got = fn.tensor(name).cpu().numpy()
        bad = int((got != ref_t).sum())
        assert bad == 0, f"tensor {name}: {bad} of {ref_t.size} elements differ"
    assert np.array_equal(out.cpu().numpy(), want)
    # CUDA-graph replay and the host-buffer entry give the same logits
    xd = torch.from_numpy(x).cuda()
    fn.capture(xd)
    assert torch.equal(fn.replay(xd), out)
    host = fn.invoke_host(x)
    assert np.array_equal(host.numpy(), want)
    fn.close()


def _check_every_tensor(fn, program, x, ctx):
    fn.invoke(torch.from_numpy(x).cuda())
    ctx.check_status()
    _, tens = oprog.run_program(program, x)
    for name, ref_t in tens.items():
        got = fn.tensor(name).cpu().numpy()
        bad = int((got != ref_t).sum())
        assert bad == 0, f"tensor {name}: {bad} of {ref_t.size} elements differ"
    return tens


def test_mobilenetv2_every_tensor(ctx):
    """NHWC f32 input, depthwise 3x3 (direct kernel) between 1x1 tensor-core layers, ReLU6, residual adds."""
    graph = networks.mobilenetv2(1005)
    cal = [np.random.default_rng(3005 + i).uniform(0, 1, (1, 224, 224, 3)).astype(np.float32) for i in range(2)]
    program = builder.build_program(graph, cal)
    n = 2
    x = np.random.default_rng(2005).uniform(0, 1, (n, 224, 224, 3)).astype(np.float32)
    fn = CudaFunction(program, n, ctx)
    ops = {o["name"]: o for o in program["ops"] if o["op"] == "conv"}
    for name, path in fn.conv_paths.items():
        assert path == (L.PATH_TC if ops[name]["groups"] == 1 else L.PATH_SIMT), (name, path)
    _check_every_tensor(fn, program, x, ctx)
    xd = torch.from_numpy(x).cuda()
    out = fn.invoke(xd).clone()
    fn.capture(xd)
    assert torch.equal(fn.replay(xd), out)
    fn.close()


def test_yolov8s_every_tensor(ctx):
    """SiLU tables in the convolution epilogue, Slice/Concat/Upsample, 5x5 max pooling, six u8 outputs."""
    graph = networks.yolov8s(1007, image=320)
    cal = [np.random.default_rng(3007 + i).uniform(0, 1, (1, 3, 320, 320)).astype(np.float32) for i in range(2)]
    program = builder.build_program(graph, cal)
    n = 2
    x = np.random.default_rng(2007).uniform(0, 1, (n, 3, 320, 320)).astype(np.float32)
    fn = CudaFunction(program, n, ctx)
    assert all(p == L.PATH_TC for p in fn.conv_paths.values()), fn.conv_paths
    tens = _check_every_tensor(fn, program, x, ctx)
    outs = fn.outputs()
    assert len(outs) == 6
    for name, t in zip(program["outputs"], outs):
        assert np.array_equal(t.cpu().numpy(), tens[name])
    fn.close()


# ---- the configurations the throughput numbers are quoted on ------------------------------------------
# Whole batches at the benchmark sizes; images are independent, so the oracle replays a few of them (first,
# middle, last: large batches take other tile counts, grid-stride trip counts and index ranges than small
# ones) and every tensor of those images must be bit-identical.
def _sampled_parity(ctx, program, x, idx):
    n = x.shape[0]
    fn = CudaFunction(program, n, ctx)
    out = fn.invoke(torch.from_numpy(x).to(ctx.device))
    ctx.check_status()
    idx = sorted(set(i % n for i in idx))
    want, tens = oprog.run_program(program, np.ascontiguousarray(x[idx]))
    sel = torch.tensor(idx, device=ctx.device)
    checked = 0
    for name, ref_t in tens.items():
        got = fn.tensor(name).index_select(0, sel).cpu().numpy()
        bad = int((got != ref_t).sum())
        assert bad == 0, f"batch {n}, tensor {name}: {bad} of {ref_t.size} elements differ"
        checked += 1
    assert np.array_equal(out.index_select(0, sel).cpu().numpy(), want)
    fn.close()
    del fn
    torch.cuda.empty_cache()
    return checked


@pytest.mark.parametrize("n", [1, 512])
def test_resnet50v2_benchmark_configuration(ctx, n):
    """ResNet-50 v2, 16 calibration samples, N = 1 and N = 512 (the benchmarked batch)."""
    graph = networks.resnet50v2(1003)
    cal = [np.random.default_rng(3003 + i).normal(0, 1, (1, 3, 224, 224)).astype(np.float32) for i in range(16)]
    program = builder.build_program(graph, cal, device=ctx.device)
    x = np.random.default_rng(2003).normal(0, 1, (n, 3, 224, 224)).astype(np.float32)
    assert _sampled_parity(ctx, program, x, [0, n // 2 - 1, n - 1]) == len(program["tensors"])


@pytest.mark.parametrize("n", [1, 256])
def test_mobilenetv2_benchmark_configuration(ctx, n):
    """MobileNetV2-1.0, NHWC input uniform[0,1] normalised to mean 0.5 / std 0.5, 16 calibration images."""
    graph = networks.mobilenetv2(1002)
    cal = [(np.random.default_rng(3002 + i).uniform(0, 1, (1, 224, 224, 3)).astype(np.float32) - 0.5) / 0.5
           for i in range(16)]
    program = builder.build_program(graph, cal, device=ctx.device)
    x = (np.random.default_rng(2002).uniform(0, 1, (n, 224, 224, 3)).astype(np.float32) - 0.5) / 0.5
    assert _sampled_parity(ctx, program, x, [0, n // 2 - 1, n - 1]) == len(program["tensors"])


def test_yolov8s_benchmark_configuration(ctx):
    """YOLOv8s at 640 x 640, N = 64, 8 calibration samples; two images through the oracle."""
    graph = networks.yolov8s(1004, image=640)
    cal = [np.random.default_rng(3004 + i).uniform(0, 1, (1, 3, 640, 640)).astype(np.float32) for i in range(8)]
    program = builder.build_program(graph, cal, device=ctx.device)
    x = np.random.default_rng(2004).uniform(0, 1, (64, 3, 640, 640)).astype(np.float32)
    assert _sampled_parity(ctx, program, x, [0, 63]) == len(program["tensors"])


def test_pipelined_host_calls_match_single_calls(ctx):
    """CudaFunction.submit_host / drain (the call the end-to-end benchmark number goes through): seven batches with
    different inputs, queued back to back from pinned host buffers through the two staging buffers and the captured
    graphs, give byte for byte what invoke() gives on each batch; results land in the caller's host buffers."""
    graph = networks.resnet50v2(1003)
    cal = [np.random.default_rng(3003 + i).normal(0, 1, (1, 3, 224, 224)).astype(np.float32) for i in range(2)]
    program = builder.build_program(graph, cal)
    n, batches = 4, 7
    fn = CudaFunction(program, n, ctx)
    rng = np.random.default_rng(2011)
    xs = [torch.from_numpy(rng.normal(0, 1, (n, 3, 224, 224)).astype(np.float32)).pin_memory() for _ in range(batches)]
    want = [fn.invoke(x.cuda()).cpu().clone() for x in xs]
    assert not torch.equal(want[0], want[1])
    outs = [torch.zeros(want[0].shape, dtype=want[0].dtype).pin_memory() for _ in range(batches)]
    with pytest.raises(L.NncbError):
        fn.submit_host(xs[0].clone(), outs[0])       # not pinned
    for x, o in zip(xs, outs):
        fn.submit_host(x, o)
    fn.drain()
    ctx.check_status()
    for i in range(batches):
        assert torch.equal(outs[i], want[i]), i
    # a single call afterwards still works on the caller's stream
    assert torch.equal(fn.invoke(xs[2].cuda()).cpu(), want[2])
    fn.close()
