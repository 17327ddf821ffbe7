"""GPU parity of the quantized Conv2D / MatMul kernels against the C oracle: bit-exact u8,
through the C ABI, on both the CUDA-core and the tcgen05 path."""
import numpy as np
import pytest
import torch

from nncase_b200 import lib as L
from nncase_b200.kernels import QuantParam
from oracle import quant_params as QP

pytestmark = pytest.mark.gpu


def make_case(seed, n, h, w, c, oc, kh, kw, groups=1, w_signed=False, sym_w=False):
    """Seeded u8 activations / per-channel weights with realistic quant params."""
    rng = np.random.default_rng(seed)
    xq = rng.integers(0, 256, (n, h, w, c), dtype=np.uint8)
    zx = int(rng.integers(0, 256))
    sx = np.float32(0.02)
    gic = c // groups
    if w_signed:
        wq = rng.integers(-127, 128, (oc, kh, kw, gic), dtype=np.int8)
        zw = np.zeros(oc, np.int32) if sym_w else rng.integers(-20, 20, oc).astype(np.int32)
    else:
        wq = rng.integers(0, 256, (oc, kh, kw, gic), dtype=np.uint8)
        zw = rng.integers(100, 156, oc).astype(np.int32)
    sw = rng.uniform(0.001, 0.004, oc).astype(np.float32)
    mult = (sx * sw).astype(np.float32)
    k = kh * kw * gic
    bias = rng.normal(0, 0.3, oc).astype(np.float32)
    # output range ~ +-3 sigma of the accumulator
    sigma = float(np.sqrt(k) * 74 * 74 * mult.mean())
    zo, so = QP.get_quant_param(-2.5 * sigma, 2.5 * sigma)
    return xq, zx, wq, zw, mult, bias, QuantParam(zo, float(so))


def run_both(ctx, qo, case, path, stride=(1, 1), pad=(0, 0, 0, 0), dil=(1, 1), groups=1, clamp=(-np.inf, np.inf),
             **extra):
    xq, zx, wq, zw, mult, bias, oqp = case
    want = qo.qconv2d_u8(xq, wq, zw, mult, bias, zx, oqp.scale, oqp.zero_point, stride, pad, dil, groups, clamp)
    got = ctx.conv2d(torch.from_numpy(xq), wq, zw, mult, bias, zx, oqp, stride=stride, padding=pad, dilation=dil,
                     groups=groups, fused_clamp=clamp, force_path=path, **extra)
    ctx.check_status()
    return got.cpu().numpy(), want


SIMT_CASES = [
    # n, h, w, c, oc, kh, kw, stride, pad, dil, groups
    (1, 5, 5, 4, 8, 3, 3, 1, 1, 1, 1), (1, 16, 16, 4, 8, 3, 3, 2, 1, 2, 1), (2, 9, 7, 3, 5, 7, 7, 2, 3, 1, 1),
    (1, 12, 12, 32, 32, 3, 3, 1, 1, 1, 32), (1, 10, 10, 24, 48, 1, 1, 1, 0, 1, 1), (1, 8, 8, 16, 16, 3, 3, 1, 1, 1, 4),
]


@pytest.mark.parametrize("cfg", SIMT_CASES)
@pytest.mark.parametrize("w_signed", [False, True])
def test_simt_conv(ctx, qo, cfg, w_signed):
    n, h, w, c, oc, kh, kw, s, p, d, g = cfg
    case = make_case(21, n, h, w, c, oc, kh, kw, g, w_signed)
    got, want = run_both(ctx, qo, case, L.PATH_SIMT, (s, s), (p, p, p, p), (d, d), g, (0, 6))
    assert np.array_equal(got, want)


TC_CASES = [
    # n, h, w, c, oc, kh, kw, stride, pad, dil        GEMM mode (1x1, stride 1)
    (1, 1, 128, 128, 64, 1, 1, 1, 0, 1), (1, 1, 200, 64, 48, 1, 1, 1, 0, 1), (2, 14, 14, 256, 128, 1, 1, 1, 0, 1),
    (1, 7, 7, 32, 16, 1, 1, 1, 0, 1), (1, 1, 300, 384, 1000, 1, 1, 1, 0, 1),
    # channel counts that do not fill the last N tile of the width chosen for them (32, 32, 64, 64 columns)
    (2, 14, 14, 32, 144, 1, 1, 1, 0, 1), (1, 9, 9, 128, 80, 1, 1, 1, 0, 1), (1, 12, 12, 32, 176, 1, 1, 1, 0, 1), (1, 6, 6, 96, 576, 1, 1, 1, 0, 1),
    # im2col mode
    (1, 56, 56, 64, 64, 3, 3, 1, 1, 1), (2, 14, 14, 128, 256, 3, 3, 1, 1, 1), (1, 28, 28, 64, 128, 3, 3, 2, 1, 1),
    (3, 7, 7, 256, 64, 3, 3, 1, 1, 1), (1, 16, 16, 32, 32, 3, 3, 1, 2, 2), (2, 28, 28, 128, 64, 1, 1, 2, 0, 1),
    (1, 1, 37, 64, 32, 1, 3, 1, 1, 1), (1, 20, 20, 32, 16, 5, 5, 1, 2, 1),
    # pixel-patch tiles with one swizzle row per pixel (stride 1, c = 64 or 128, resident weights): padded and
    # not, patches that overhang the image, 64- and 128-byte rows
    (2, 20, 23, 64, 32, 3, 3, 1, 1, 1), (1, 9, 9, 64, 48, 2, 2, 1, 0, 1), (1, 12, 10, 128, 32, 2, 2, 1, 1, 1),
    (1, 30, 17, 64, 64, 3, 3, 1, 1, 1), (3, 8, 16, 64, 96, 3, 3, 1, 1, 1), (1, 33, 9, 64, 16, 4, 4, 1, 2, 1),
]


@pytest.mark.parametrize("cfg", TC_CASES)
@pytest.mark.parametrize("wmode", ["u8_asym", "i8_sym"])
def test_tc_conv(ctx, qo, cfg, wmode):
    n, h, w, c, oc, kh, kw, s, p, d = cfg
    ph, pw = (p if kh > 1 else 0), (p if kw > 1 else 0)
    case = make_case(31, n, h, w, c, oc, kh, kw, 1, wmode == "i8_sym", sym_w=True)
    got, want = run_both(ctx, qo, case, L.PATH_TC, (s, s), (ph, ph, pw, pw), (d, d), 1, (0, 6))
    bad = np.argwhere(got != want)
    assert bad.size == 0, f"{len(bad)} mismatches, first at {bad[:5].tolist()}"


@pytest.mark.parametrize("path", [L.PATH_SIMT, L.PATH_TC])
def test_conv_rounding_ties(ctx, qo, path):
    """Scales that are powers of two put half of all results exactly on a rounding boundary and
    the rest exactly on integers: the fast epilogue's guard band must hand every tie to the
    exact formula (round half to even), with and without the residual stage."""
    rng = np.random.default_rng(77)
    n, h, w, c, oc = 1, 16, 16, 64, 64
    xq = rng.integers(0, 256, (n, h, w, c), dtype=np.uint8)
    wq = rng.integers(0, 256, (oc, 3, 3, c), dtype=np.uint8)
    zw = rng.integers(120, 136, oc).astype(np.int32)
    mult = np.full(oc, 2.0 ** -13, np.float32)
    bias = (rng.integers(-8, 8, oc) * 0.25).astype(np.float32)
    oqp = QuantParam(128, 0.5)  # v / 0.5 is exact; acc * 2^-12 + k/2: ties wherever bit 11 of acc is set
    want = qo.qconv2d_u8(xq, wq, zw, mult, bias, 131, oqp.scale, oqp.zero_point, pad=(1, 1, 1, 1))
    got = ctx.conv2d(torch.from_numpy(xq), wq, zw, mult, bias, 131, oqp, padding=(1, 1, 1, 1), force_path=path)
    ctx.check_status()
    assert 5 < want.std() and np.array_equal(got.cpu().numpy(), want)
    res = rng.integers(0, 256, want.shape, dtype=np.uint8)
    rq, aq = QuantParam(100, 0.25), QuantParam(90, 0.5)  # (q-128)*0.5 + (r-100)*0.25 over 0.5: ties for odd r
    want2 = qo.qadd_u8(want, res, oqp.scale, oqp.zero_point, rq.scale, rq.zero_point, aq.scale, aq.zero_point)
    got2 = ctx.conv2d(torch.from_numpy(xq), wq, zw, mult, bias, 131, oqp, padding=(1, 1, 1, 1), force_path=path,
                      res=torch.from_numpy(res).cuda(), residual=(rq, aq))
    ctx.check_status()
    assert np.array_equal(got2.cpu().numpy(), want2)


@pytest.mark.parametrize("oc", [16, 48, 80, 96, 144, 160, 192, 272])
def test_tc_conv_channel_tiles(ctx, qo, oc):
    """Output-channel counts that give every staging-tile width (swizzled and not) and a partial
    last N tile."""
    case = make_case(90 + oc, 2, 9, 9, 64, oc, 3, 3)
    got, want = run_both(ctx, qo, case, L.PATH_TC, (1, 1), (1, 1, 1, 1), (1, 1), 1, (0, 6))
    assert np.array_equal(got, want)


@pytest.mark.parametrize("oc", [256, 96, 144, 64, 32])
def test_tc_conv_residual_and_second_output(ctx, qo, oc):
    """Fused add and second output on every staging-tile width (128, 96, 48, 64 and 32 columns)."""
    n, h, w, c = 2, 14, 14, 64
    case = make_case(41, n, h, w, c, oc, 1, 1)
    xq, zx, wq, zw, mult, bias, oqp = case
    rng = np.random.default_rng(42)
    res = rng.integers(0, 256, (n, h, w, oc), dtype=np.uint8)
    rq, aq, yq2 = QuantParam(117, 0.05), QuantParam(125, 0.06), QuantParam(0, 0.03)
    y1 = qo.qconv2d_u8(xq, wq, zw, mult, bias, zx, oqp.scale, oqp.zero_point)
    want = qo.qadd_u8(y1, res, oqp.scale, oqp.zero_point, rq.scale, rq.zero_point, aq.scale, aq.zero_point)
    want2 = qo.requant_u8(want, aq.scale, aq.zero_point, yq2.scale, yq2.zero_point, 0.0, np.inf)
    for path in (L.PATH_SIMT, L.PATH_TC):
        got, got2 = ctx.conv2d(torch.from_numpy(xq), wq, zw, mult, bias, zx, oqp, res=torch.from_numpy(res).cuda(),
                               residual=(rq, aq), y2=(yq2, 0.0, float("inf")), force_path=path)
        ctx.check_status()
        assert np.array_equal(got.cpu().numpy(), want)
        assert np.array_equal(got2.cpu().numpy(), want2)


@pytest.mark.parametrize("add_form", [0, 2])
@pytest.mark.parametrize("c,oc", [(64, 256), (512, 96), (256, 64), (512, 2048)])
def test_tc_conv_fused_add_table_and_arithmetic(ctx, qo, add_form, c, oc):
    """The fused residual add of the tensor-core convolution in its two forms -- a look-up in the table of all byte
    pairs (the default), and the unfused float chain itself on packed arithmetic (option conv.add_table = 2, which leaves
    the table's 65 KB to the pipeline stages): the same bits as the operator chain conv -> add (-> requantized second output), over every residual byte and a spread of convolution outputs."""
    n, h, w = 2, 14, 14
    case = make_case(300 + c + oc, n, h, w, c, oc, 1, 1)
    xq, zx, wq, zw, mult, bias, oqp = case
    rng = np.random.default_rng(43)
    res = rng.integers(0, 256, (n, h, w, oc), dtype=np.uint8)
    rq, aq, yq2 = QuantParam(117, 0.05), QuantParam(125, 0.06), QuantParam(0, 0.03)
    y1 = qo.qconv2d_u8(xq, wq, zw, mult, bias, zx, oqp.scale, oqp.zero_point)
    want = qo.qadd_u8(y1, res, oqp.scale, oqp.zero_point, rq.scale, rq.zero_point, aq.scale, aq.zero_point)
    want2 = qo.requant_u8(want, aq.scale, aq.zero_point, yq2.scale, yq2.zero_point, 0.0, np.inf)
    ctx.set_option("conv.add_table", add_form)
    try:
        got, got2 = ctx.conv2d(torch.from_numpy(xq), wq, zw, mult, bias, zx, oqp, res=torch.from_numpy(res).cuda(),
                               residual=(rq, aq), y2=(yq2, 0.0, float("inf")), force_path=L.PATH_TC)
        ctx.check_status()
        assert np.array_equal(got.cpu().numpy(), want)
        assert np.array_equal(got2.cpu().numpy(), want2)
        got = ctx.conv2d(torch.from_numpy(xq), wq, zw, mult, bias, zx, oqp, res=torch.from_numpy(res).cuda(),
                         residual=(rq, aq), force_path=L.PATH_TC)
        assert np.array_equal(got.cpu().numpy(), want)
    finally:
        ctx.set_option("conv.add_table", 0)


def test_tc_matmul_f32_logits(ctx, qo):
    """FC layer: [M,K] x [N,K] with real-valued f32 output (classifier logits)."""
    m, k, n = 70, 2048, 1000
    case = make_case(51, 1, 1, m, k, n, 1, 1)
    xq, zx, wq, zw, mult, bias, _ = case
    want = qo.qconv2d_u8(xq, wq, zw, mult, bias, zx, 1.0, 0, f32_out=True).reshape(m, n)
    for path in (L.PATH_SIMT, L.PATH_TC):
        got = ctx.mat_mul(torch.from_numpy(xq.reshape(m, k)), wq.reshape(n, k), zw, mult, bias, zx, None,
                          f32_out=True, force_path=path)
        ctx.check_status()
        assert np.array_equal(got.cpu().numpy(), want)


def test_lut_activation(ctx, qo):
    case = make_case(61, 1, 8, 8, 32, 32, 3, 3)
    xq, zx, wq, zw, mult, bias, oqp = case
    lut = np.random.default_rng(62).integers(0, 256, 256, dtype=np.uint8)
    want = qo.qconv2d_u8(xq, wq, zw, mult, bias, zx, oqp.scale, oqp.zero_point, pad=(1, 1, 1, 1), lut=lut)
    for path in (L.PATH_SIMT, L.PATH_TC):
        got = ctx.conv2d(torch.from_numpy(xq), wq, zw, mult, bias, zx, oqp, padding=(1, 1, 1, 1), lut=lut,
                         force_path=path)
        assert np.array_equal(got.cpu().numpy(), want)


def test_golden_conv_slice(ctx):
    """The committed fixture generated from the reference's kernels (config-1 slice)."""
    import os
    c = np.load(os.path.join(os.path.dirname(__file__), "golden", "conv_config1_slice.npz"))
    oqp = QuantParam(int(c["zo"]), float(c["so"]))
    for path in (L.PATH_SIMT, L.PATH_TC):
        got = ctx.conv2d(torch.from_numpy(c["xq"]), c["wq"], c["zw"], c["mult"], c["bias"], int(c["zx"]), oqp,
                         padding=(1, 1, 1, 1), fused_clamp=(0.0, 6.0), force_path=path).cpu().numpy()
        assert np.array_equal(got, c["y_integer"])
        d = np.abs(got.astype(int) - c["y_ref_composite"].astype(int))
        assert d.max() <= 1 and (d != 0).sum() <= int(c["allowed_mismatches"])


@pytest.mark.parametrize("scale", [0.5, 0.014035294, 0.029455967, 0.3709820, 12.381763, 1.0 / 3.0, 7.955359,
                                   1.1920929e-07 * 8388607, 3.4e-5, 1999.0])
def test_reciprocal_division_matches_ieee(ctx, scale):
    """The epilogue's division by a scale (reciprocal + two fused corrections) against the IEEE
    division on 2^26 operands per scale."""
    import ctypes
    m = ctypes.c_uint64(123)
    L.check(ctx._lib.nncb_selftest_reciprocal_division(ctx._h, scale, 1 << 26, 17, ctypes.byref(m)))
    assert m.value == 0


def test_bad_arguments_are_rejected(ctx):
    from nncase_b200.lib import NncbError
    w = np.zeros((8, 3, 3, 5), np.uint8)
    with pytest.raises(NncbError) as e:  # weights do not match channels
        ctx.conv2d_plan((1, 8, 8, 4), w, None, np.ones(8), np.zeros(8), 0, QuantParam(0, 1.0))
    assert e.value.code == -22
    w = np.zeros((8, 3, 3, 4), np.uint8)
    with pytest.raises(NncbError) as e:  # 4 channels cannot take the tensor-core path
        ctx.conv2d_plan((1, 8, 8, 4), w, None, np.ones(8), np.zeros(8), 0, QuantParam(0, 1.0), force_path=L.PATH_TC)
    assert e.value.code == -38
    with pytest.raises(NncbError) as e:  # empty output
        ctx.conv2d_plan((1, 2, 2, 4), w, None, np.ones(8), np.zeros(8), 0, QuantParam(0, 1.0))
    assert e.value.code == -22


ROWS_CASES = [
    # n, h, w, c, oc, kh, kw: unpadded stride-1 convolutions whose kernel row is 32, 64 or 128 contiguous bytes
    (2, 19, 19, 16, 64, 4, 4), (1, 115, 115, 16, 64, 4, 4), (2, 15, 16, 32, 32, 3, 2), (1, 9, 21, 16, 48, 2, 2),
    (3, 10, 37, 32, 128, 3, 4), (1, 6, 6, 16, 24, 4, 4), (1, 40, 11, 64, 16, 5, 2),
]


@pytest.mark.parametrize("cfg", ROWS_CASES)
@pytest.mark.parametrize("wmode", ["u8_asym", "i8_sym"])
def test_tc_conv_kernel_rows(ctx, qo, cfg, wmode):
    """The merged-kernel-row form (one K block per kernel row, pixel-patch tiles): patch shapes that
    divide the output and ones that overhang it, both epilogues (oc = 24 takes the general one)."""
    n, h, w, c, oc, kh, kw = cfg
    case = make_case(51, n, h, w, c, oc, kh, kw, 1, wmode == "i8_sym", sym_w=True)
    got, want = run_both(ctx, qo, case, L.PATH_TC, clamp=(0, 6))
    bad = np.argwhere(got != want)
    assert bad.size == 0, f"{len(bad)} mismatches, first at {bad[:5].tolist()}"


def test_tc_conv_kernel_rows_residual_second_output(ctx, qo):
    n, h, w, c, oc, kh, kw = 2, 22, 27, 16, 128, 3, 4
    case = make_case(52, n, h, w, c, oc, kh, kw)
    xq, zx, wq, zw, mult, bias, oqp = case
    rng = np.random.default_rng(53)
    oh, ow = h - kh + 1, w - kw + 1
    res = rng.integers(0, 256, (n, oh, ow, oc), dtype=np.uint8)
    rq, aq, yq2 = QuantParam(117, 0.05), QuantParam(125, 0.06), QuantParam(0, 0.03)
    conv = qo.qconv2d_u8(xq, wq, zw, mult, bias, zx, oqp.scale, oqp.zero_point)
    want = qo.qadd_u8(conv, res, oqp.scale, oqp.zero_point, rq.scale, rq.zero_point, aq.scale, aq.zero_point)
    want2 = qo.requant_u8(want, aq.scale, aq.zero_point, yq2.scale, yq2.zero_point, 0.0, np.inf)
    got, got2 = ctx.conv2d(torch.from_numpy(xq), wq, zw, mult, bias, zx, oqp, force_path=L.PATH_TC,
                           res=torch.from_numpy(res).cuda(), residual=(rq, aq), y2=(yq2, 0.0, float("inf")))
    ctx.check_status()
    assert np.array_equal(got.cpu().numpy(), want)
    assert np.array_equal(got2.cpu().numpy(), want2)


DEPTHWISE_CASES = [
    # n, h, w, c, kh, kw, stride, pad, dil: the streaming depthwise kernel (groups == channels, c % 4 == 0)
    (2, 28, 28, 96, 3, 3, 1, 1, 1), (1, 56, 56, 160, 3, 3, 2, 1, 1), (3, 9, 11, 32, 3, 3, 1, 1, 2), (1, 14, 14, 960, 3, 3, 1, 1, 1),
    (2, 7, 7, 4, 5, 5, 1, 2, 1), (1, 112, 112, 32, 3, 3, 2, 0, 1), (2, 7, 7, 8, 3, 3, 1, 1, 1), (1, 15, 13, 8, 3, 3, 2, 1, 1),
    (1, 5, 3, 4, 3, 3, 1, 0, 1), (1, 6, 9, 12, 3, 3, 2, 0, 1),
]


@pytest.mark.parametrize("cfg", DEPTHWISE_CASES)
@pytest.mark.parametrize("w_signed", [False, True])
def test_depthwise_conv(ctx, qo, cfg, w_signed):
    n, h, w, c, kh, kw, s, p, d = cfg
    case = make_case(61, n, h, w, c, c, kh, kw, c, w_signed)
    got, want = run_both(ctx, qo, case, L.PATH_AUTO, (s, s), (p, p, p, p), (d, d), c, (0, 6))
    assert np.array_equal(got, want)


def test_depthwise_conv_residual_and_second_output(ctx, qo):
    n, h, w, c = 2, 14, 14, 64
    case = make_case(62, n, h, w, c, c, 3, 3, c)
    xq, zx, wq, zw, mult, bias, oqp = case
    res = np.random.default_rng(63).integers(0, 256, (n, h, w, c), dtype=np.uint8)
    rq, aq, yq2 = QuantParam(117, 0.05), QuantParam(125, 0.06), QuantParam(0, 0.03)
    y1 = qo.qconv2d_u8(xq, wq, zw, mult, bias, zx, oqp.scale, oqp.zero_point, pad=(1, 1, 1, 1), groups=c)
    want = qo.qadd_u8(y1, res, oqp.scale, oqp.zero_point, rq.scale, rq.zero_point, aq.scale, aq.zero_point)
    want2 = qo.requant_u8(want, aq.scale, aq.zero_point, yq2.scale, yq2.zero_point, 0.0, np.inf)
    got, got2 = ctx.conv2d(torch.from_numpy(xq), wq, zw, mult, bias, zx, oqp, padding=(1, 1, 1, 1), groups=c,
                           res=torch.from_numpy(res).cuda(), residual=(rq, aq), y2=(yq2, 0.0, float("inf")))
    ctx.check_status()
    assert np.array_equal(got.cpu().numpy(), want) and np.array_equal(got2.cpu().numpy(), want2)


@pytest.mark.parametrize("issuers", [1, 2])
@pytest.mark.parametrize("loaders", [1, 2, 3])
@pytest.mark.parametrize("shape", ["im2col_3x3_c256", "gemm_k1024", "patch_3x3_c64", "im2col_odd_kblocks"])
def test_role_warp_counts_do_not_change_the_result(ctx, qo, shape, issuers, loaders):
    """Deep K loops run with two MMA-issuing warps (which take the stages of the ring in turn and accumulate into
    the same TMEM accumulator) and with a load warp each for activations and weights; the wide patch form deals
    its filter taps out to two issuers. Forced to one or two of each through the context options, the output is
    the oracle's, byte for byte."""
    # the 1x1 and the 96-channel case have more tiles than the GPU has SMs (every CTA crosses tile boundaries); the
    # 96-channel one has an odd number of stages per tile, so the owner of a tile's first stage alternates
    n, h, w, c, oc, k, pad = {"im2col_3x3_c256": (8, 14, 14, 256, 256, 3, 1), "gemm_k1024": (64, 14, 14, 1024, 256, 1, 0),
                              "patch_3x3_c64": (8, 56, 56, 64, 64, 3, 1), "im2col_odd_kblocks": (16, 40, 40, 96, 64, 3, 1)}[shape]
    xq, zx, wq, zw, mult, bias, oqp = make_case(91, n, h, w, c, oc, k, k)
    want = qo.qconv2d_u8(xq, wq, zw, mult, bias, zx, oqp.scale, oqp.zero_point, pad=(pad,) * 4)
    ctx.set_option("conv.mma_issuers", issuers)
    ctx.set_option("conv.load_warps", loaders)
    try:
        plan = ctx.conv2d_plan(tuple(xq.shape), wq, zw, mult, bias, zx, oqp, padding=(pad,) * 4, force_path=L.PATH_TC)
    finally:
        ctx.set_option("conv.mma_issuers", 0)
        ctx.set_option("conv.load_warps", 0)
    x = torch.from_numpy(xq).cuda()
    for _ in range(3):  # the persistent CTAs take several tiles each: repeat to vary the interleaving of the roles
        got = plan(x).cpu().numpy()
        assert np.array_equal(got, want)
    ctx.check_status()
    plan.close()


@pytest.mark.parametrize("overlap", [0, 1])
def test_chained_convolutions_with_and_without_launch_overlap(ctx, qo, overlap):
    """Convolutions are launched as programmatic dependents of the kernel before them: a kernel may become resident
    while its predecessor still runs and waits (griddepcontrol.wait) before it reads what the predecessor wrote. A
    chain of three layers, each reading the previous one's output (the third also as its residual), run twenty times
    back to back, gives the oracle's bytes with the overlap on and off."""
    n, h, w, c = 4, 28, 28, 128
    rng = np.random.default_rng(123)
    xq = rng.integers(0, 256, (n, h, w, c), dtype=np.uint8)
    cases = [make_case(200 + i, n, h, w, c, c, k, k) for i, k in enumerate((1, 3, 1))]
    rq, aq = QuantParam(117, 0.05), QuantParam(125, 0.06)
    ctx.set_option("launch.overlap", overlap)
    try:
        plans, want, cur, zx = [], [], xq, cases[0][1]
        for i, (_, _, wq, zw, mult, bias, oqp) in enumerate(cases):
            pad = 1 if wq.shape[1] == 3 else 0
            kw = dict(residual=(rq, aq)) if i == 2 else {}
            plans.append(ctx.conv2d_plan(cur.shape, wq, zw, mult, bias, zx, oqp, padding=(pad,) * 4, force_path=L.PATH_TC, **kw))
            y = qo.qconv2d_u8(cur, wq, zw, mult, bias, zx, oqp.scale, oqp.zero_point, pad=(pad,) * 4)
            if i == 2:
                y = qo.qadd_u8(y, want[0], oqp.scale, oqp.zero_point, rq.scale, rq.zero_point, aq.scale, aq.zero_point)
            want.append(y)
            cur, zx = y, oqp.zero_point
        x = torch.from_numpy(xq).cuda()
        for _ in range(20):
            y0 = plans[0](x)
            y1 = plans[1](y0)
            y2 = plans[2](y1, y0)
        assert np.array_equal(y0.cpu().numpy(), want[0]) and np.array_equal(y1.cpu().numpy(), want[1])
        assert np.array_equal(y2.cpu().numpy(), want[2])
        ctx.check_status()
        for p_ in plans:
            p_.close()
    finally:
        ctx.set_option("launch.overlap", 1)


@pytest.mark.parametrize("variant", ["plain", "residual", "deep"])
def test_bounded_wait_gives_up_and_the_context_stays_usable(ctx, qo, variant):
    """Every wait inside the tensor-core kernel has a time limit. With the limit shortened to 2 ms and the
    loader of one CTA told to expect bytes that no load delivers ("debug.withhold_load"), that CTA's waits run
    out: the kernel returns by itself, nncb_check_device_status reports -ETIMEDOUT with a role code once and
    clears the status word, and the same convolution on the same context is bit-exact afterwards."""
    n, h, w, c, oc = (2, 14, 14, 1024, 256) if variant == "deep" else (2, 28, 28, 64, 256)  # deep: two issuers, two load warps
    xq, zx, wq, zw, mult, bias, oqp = make_case(77, n, h, w, c, oc, 1, 1)
    x = torch.from_numpy(xq).cuda()
    kw, want = {}, qo.qconv2d_u8(xq, wq, zw, mult, bias, zx, oqp.scale, oqp.zero_point)
    if variant == "residual":
        rq, aq = QuantParam(117, 0.05), QuantParam(125, 0.06)
        res = np.random.default_rng(78).integers(0, 256, (n, h, w, oc), dtype=np.uint8)
        kw = dict(residual=(rq, aq))
        want = qo.qadd_u8(want, res, oqp.scale, oqp.zero_point, rq.scale, rq.zero_point, aq.scale, aq.zero_point)
        res_d = torch.from_numpy(res).cuda()
    plan = ctx.conv2d_plan(tuple(x.shape), wq, zw, mult, bias, zx, oqp, force_path=L.PATH_TC, **kw)
    run = (lambda: plan(x, res_d)) if variant == "residual" else (lambda: plan(x))
    assert np.array_equal(run().cpu().numpy(), want)
    ctx.check_status()
    ctx.set_option("wait_limit_us", 2000)
    ctx.set_option("debug.withhold_load", 1)
    try:
        run()
        with pytest.raises(L.NncbError) as e:
            ctx.check_status()
    finally:
        ctx.set_option("debug.withhold_load", 0)
        ctx.set_option("wait_limit_us", 1000000)
    assert e.value.code == -110, e.value            # -ETIMEDOUT
    assert any(f"role code {c_}" in str(e.value) for c_ in (101, 102, 103, 104, 105)), e.value
    ctx.check_status()                              # the status word was cleared by the read
    assert np.array_equal(run().cpu().numpy(), want)
    ctx.check_status()
    plan.close()


def test_options_reject_unknown_names_and_bad_values(ctx):
    with pytest.raises(L.NncbError) as e:
        ctx.set_option("no.such.option", 1)
    assert e.value.code == -22
    with pytest.raises(L.NncbError):
        ctx.set_option("wait_limit_us", 0)
    assert ctx.get_option("wait_limit_us") == 1000000 and ctx.get_option("conv.wide_patch") == 1


def test_two_devices_in_one_process():
    """Kernels that need more than 48 KB of dynamic shared memory raise their limit per device: contexts on
    two GPUs of one process both run paged attention and the w8a16 MatMul (no peer memory involved)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from nncase_b200.kernels import Context
    outs = []
    for dev in (0, 1):
        with torch.cuda.device(dev):
            c = Context(dev)
            g = torch.Generator(device=f"cuda:{dev}").manual_seed(5)
            k = torch.randn((40, 2, 16, 64), device=f"cuda:{dev}", generator=g, dtype=torch.float16)
            q = torch.randn((4, 14, 64), device=f"cuda:{dev}", generator=g, dtype=torch.float16)
            table = torch.arange(40, device=f"cuda:{dev}", dtype=torch.int32).reshape(4, 10)
            lens = torch.tensor([160, 33, 1, 100], device=f"cuda:{dev}", dtype=torch.int32)
            out = c.paged_attention_decode(q, k, k, table, lens)
            xh = torch.randn((8, 4864), device=f"cuda:{dev}", generator=g, dtype=torch.float16)
            wt = torch.randint(-127, 128, (896, 4864), device=f"cuda:{dev}", generator=g, dtype=torch.int8)
            sc = torch.full((896,), 0.01, device=f"cuda:{dev}", dtype=torch.float16)
            y = torch.empty((8, 896), device=f"cuda:{dev}", dtype=torch.float16)
            L.check(c._lib.nncb_gemv_w8a16(c._h, xh.data_ptr(), wt.data_ptr(), sc.data_ptr(), None, None, y.data_ptr(),
                                           8, 896, 4864))
            c.check_status()
            outs.append((out.cpu(), y.cpu()))
            c.close()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_int8_peak_selftest_runs(ctx):
    """The tensor-pipe peak loop returns by itself and reports a plausible rate (a B200 is far above 1 POP/s)."""
    import ctypes as C
    best, mean = C.c_double(), C.c_double()
    for signed in (0, 1):
        L.check(ctx._lib.nncb_selftest_int8_peak(ctx._h, 4096, 3, signed, C.byref(best), C.byref(mean)))
        ctx.check_status()
        assert best.value >= mean.value > 1000.0, (best.value, mean.value)


def test_mma_issue_selftest(ctx):
    """The issue-pace loop returns by itself; two issuing warps are not slower than one at a 64-column tile, and no
    configuration beats the pace of the tensor pipe itself (n / 2 cycles per MMA is below what any B200 clock allows)."""
    import ctypes as C
    with pytest.raises(L.NncbError):
        L.check(ctx._lib.nncb_selftest_mma_issue(ctx._h, 100, 1, 4096, C.byref(C.c_double())))
    got = {}
    for n in (64, 144, 256):
        for issuers in (1, 2):
            c = C.c_double()
            L.check(ctx._lib.nncb_selftest_mma_issue(ctx._h, n, issuers, 8192, C.byref(c)))
            ctx.check_status()
            got[n, issuers] = c.value
            assert c.value > n / 2.0, (n, issuers, c.value)
    assert got[64, 2] <= got[64, 1] * 1.05, got


def test_batched_matmul_with_broadcast_weights(ctx, qo):
    """[B1, B2, M, K] x [K, N]: leading dimensions are batches of rows over one constant right-hand side, the
    broadcast case of the reference's mat_mul (reference/matmul.cpp:57-89)."""
    rng = np.random.default_rng(51)
    a = rng.integers(0, 256, (2, 3, 40, 64), dtype=np.uint8)
    wq = rng.integers(0, 256, (48, 64), dtype=np.uint8)
    zw = rng.integers(100, 150, 48).astype(np.int32)
    mult = rng.uniform(2e-5, 6e-5, 48).astype(np.float32)
    bias = rng.normal(0, 0.2, 48).astype(np.float32)
    oqp = QuantParam(120, 0.02)
    got = ctx.mat_mul(torch.from_numpy(a), wq, zw, mult, bias, 117, oqp).cpu().numpy()
    want = qo.qconv2d_u8(a.reshape(1, 1, -1, 64), wq.reshape(48, 1, 1, 64), zw, mult, bias, 117, oqp.scale, oqp.zero_point)
    assert got.shape == (2, 3, 40, 48) and np.array_equal(got.reshape(-1, 48), want.reshape(-1, 48))
