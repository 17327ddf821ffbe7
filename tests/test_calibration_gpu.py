"""Calibration on the library's own float kernels (nncb_conv2d_f32, nncb_minmax_f32, ...) against the torch CPU
forward of the same graphs: float results within 1e-4 of each tensor's range (summation order differs), ranges
equal to that tolerance, and the quantized program built from GPU calibration bit-exact against the oracle."""
import numpy as np
import pytest
import torch

from nncase_b200 import builder, networks
from nncase_b200.runtime import CudaFunction
from oracle import program as oprog

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("net", ["resnet", "mobilenet", "yolo"])
def test_float_forward_matches_torch(ctx, net):
    if net == "resnet":
        g = networks.resnet50v2(1003, image=64)
        x = np.random.default_rng(1).normal(0, 1, (2, 3, 64, 64)).astype(np.float32)
    elif net == "mobilenet":
        g = networks.mobilenetv2(1002, image=64)
        x = np.random.default_rng(2).uniform(-1, 1, (2, 64, 64, 3)).astype(np.float32)
    else:
        g = networks.yolov8s(1004, image=64)
        x = np.random.default_rng(3).uniform(0, 1, (1, 3, 64, 64)).astype(np.float32)
    with torch.no_grad():
        _, want = builder.float_forward(g, torch.from_numpy(x))
    _, got = builder.float_forward_cuda(g, x, ctx)
    ctx.check_status()
    assert set(got) == set(want)
    for name, w in want.items():
        a, b = got[name].cpu().numpy(), w.numpy()
        assert a.shape == b.shape, name
        rng = max(float(b.max() - b.min()), 1e-6)
        assert float(np.abs(a - b).max()) <= 1e-4 * rng, (name, float(np.abs(a - b).max()), rng)


def test_minmax_ignores_non_finite(ctx):
    import ctypes as C

    from nncase_b200 import lib as L
    x = np.random.default_rng(4).normal(0, 3, 1_000_003).astype(np.float32)
    x[[5, 77, 100000]] = (np.inf, -np.inf, np.nan)
    xd = torch.from_numpy(x).cuda()
    mn, mx = C.c_float(), C.c_float()
    L.check(ctx._lib.nncb_minmax_f32(ctx._h, xd.data_ptr(), xd.numel(), C.byref(mn), C.byref(mx)))
    fin = x[np.isfinite(x)]
    assert mn.value == fin.min() and mx.value == fin.max()
    bad = torch.full((100,), float("nan"), device="cuda")
    L.check(ctx._lib.nncb_minmax_f32(ctx._h, bad.data_ptr(), bad.numel(), C.byref(mn), C.byref(mx)))
    assert mn.value > mx.value  # the "no finite value" result of the reference's GetMinMax


def test_calibrate_on_gpu_matches_cpu_and_builds_an_exact_program(ctx):
    g = networks.resnet50v2(1003, image=96)
    cal = [np.random.default_rng(3003 + i).normal(0, 1, (1, 3, 96, 96)).astype(np.float32) for i in range(4)]
    r_cpu = builder.calibrate(g, cal, "cpu")
    r_gpu = builder.calibrate(g, cal, ctx.device)
    assert set(r_cpu) == set(r_gpu)
    for name, (lo, hi) in r_cpu.items():
        glo, ghi = r_gpu[name]
        span = max(hi - lo, 1e-6)
        assert abs(glo - lo) <= 1e-4 * span and abs(ghi - hi) <= 1e-4 * span, name
    program = builder.build_program(g, cal, device=ctx.device)
    x = np.random.default_rng(2003).normal(0, 1, (2, 3, 96, 96)).astype(np.float32)
    fn = CudaFunction(program, 2, ctx)
    got = fn.invoke(torch.from_numpy(x).cuda()).cpu().numpy()
    want, _ = oprog.run_program(program, x)
    assert np.array_equal(got, want)
    fn.close()
