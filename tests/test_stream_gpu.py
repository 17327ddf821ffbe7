"""GPU parity of the streaming kernels against the C oracle (bit-exact), through the C ABI."""
import numpy as np
import pytest
import torch

from nncase_b200.kernels import QuantParam

pytestmark = pytest.mark.gpu


def _edge_values(scale, zp):
    k = np.arange(-300, 300, dtype=np.float32)
    half = (k + np.float32(0.5) - np.float32(zp)) * np.float32(scale)
    return np.concatenate([half, np.nextafter(half, np.float32(np.inf)), np.nextafter(half, np.float32(-np.inf)),
                           np.array([0.0, -0.0, 1e-40, -1e-40, 1e6, -1e6], np.float32)])


@pytest.mark.parametrize("n", [0, 1, 15, 16, 17, 1000003])
@pytest.mark.parametrize("scale,zp", [(0.01, 127), (0.014035294, 88)])
def test_quantize_u8(ctx, qo, n, scale, zp):
    rng = np.random.default_rng(n + 1)
    x = rng.normal(0, 1, n).astype(np.float32)
    if n > 2000:
        e = _edge_values(scale, zp)
        x[: e.size] = e
    got = ctx.quantize(torch.from_numpy(x), QuantParam(zp, scale)).cpu().numpy()
    assert np.array_equal(got, qo.quantize_u8(x, scale, zp))


def test_quantize_unaligned_pointer(ctx, qo):
    x = np.random.default_rng(0).normal(0, 1, 4099).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    got = ctx.quantize(xd[3:], QuantParam(10, 0.02))  # .contiguous() keeps the offset view's storage offset
    assert np.array_equal(got.cpu().numpy(), qo.quantize_u8(x[3:], 0.02, 10))


@pytest.mark.parametrize("dtype,fn", [(torch.int8, "quantize_i8")])
def test_quantize_i8(ctx, qo, dtype, fn):
    x = np.random.default_rng(5).normal(0, 1, 70001).astype(np.float32)
    got = ctx.quantize(torch.from_numpy(x), QuantParam(-3, 0.02), dtype).cpu().numpy()
    assert np.array_equal(got, getattr(qo, fn)(x, 0.02, -3))


def test_quantize_i16(ctx):
    x = np.random.default_rng(6).normal(0, 100, 70001).astype(np.float32)
    got = ctx.quantize(torch.from_numpy(x), QuantParam(7, 0.01), torch.int16).cpu().numpy()
    want = np.clip(np.rint(x / np.float32(0.01) + np.float32(7)), -32768, 32767).astype(np.int16)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("n", [0, 1, 31, 4096, 999999])
def test_dequantize_u8(ctx, qo, n):
    q = np.random.default_rng(n).integers(0, 256, n, dtype=np.uint8)
    got = ctx.dequantize(torch.from_numpy(q), QuantParam(88, 0.014035294)).cpu().numpy()
    assert np.array_equal(got, qo.dequantize_u8(q, 0.014035294, 88))


def test_dequantize_i16(ctx):
    """(q - zp) * scale on int16 (reference/dequantize.cpp:29-59 instantiates it for int16 as well); both
    operations are exact-or-correctly-rounded f32, so numpy float32 arithmetic is the truth."""
    q = np.random.default_rng(8).integers(-32768, 32768, 70001).astype(np.int16)
    q[:4] = (-32768, 32767, 0, 7)
    got = ctx.dequantize(torch.from_numpy(q), QuantParam(7, 0.01)).cpu().numpy()
    want = (q.astype(np.float32) - np.float32(7)) * np.float32(0.01)
    assert got.dtype == np.float32 and np.array_equal(got, want)
    # round trip through quantize is the identity on in-range values
    back = ctx.quantize(torch.from_numpy(want), QuantParam(7, 0.01), torch.int16).cpu().numpy()
    assert np.array_equal(back, q)


def test_dequantize_i8(ctx, qo):
    q = np.random.default_rng(1).integers(-128, 128, 50001, dtype=np.int8)
    got = ctx.dequantize(torch.from_numpy(q), QuantParam(-3, 0.02)).cpu().numpy()
    assert np.array_equal(got, qo.dequantize_i8(q, 0.02, -3))


def test_host_buffer_round_trip(ctx, qo):
    x = np.random.default_rng(2).normal(0, 1, 12345).astype(np.float32)
    qp = QuantParam(100, 0.03)
    q = ctx.quantize_host(x, qp)
    assert np.array_equal(q, qo.quantize_u8(x, 0.03, 100))
    assert np.array_equal(ctx.dequantize_host(q, qp), qo.dequantize_u8(q, 0.03, 100))
    # quantize(dequantize(q)) is the identity on u8
    assert np.array_equal(ctx.quantize_host(ctx.dequantize_host(q, qp), qp), q)


@pytest.mark.parametrize("shape,c_pad", [((2, 3, 17, 19), 4), ((1, 64, 56, 56), 64), ((2, 5, 9, 7), 8),
                                         ((1, 3, 224, 224), 4)])
def test_quantize_nchw_to_nhwc(ctx, qo, shape, c_pad):
    x = np.random.default_rng(3).normal(0, 1, shape).astype(np.float32)
    got = ctx.quantize_nchw_to_nhwc(torch.from_numpy(x), QuantParam(120, 0.025), c_pad).cpu().numpy()
    assert np.array_equal(got, qo.quantize_nchw_to_nhwc_u8(x, 0.025, 120, c_pad))


@pytest.mark.parametrize("shape,c_pad", [((2, 3, 18, 22), 32), ((1, 3, 224, 224), 32), ((2, 4, 8, 8), 16)])
def test_quantize_nchw_to_s2d(ctx, qo, shape, c_pad):
    x = np.random.default_rng(13).normal(0, 1, shape).astype(np.float32)
    got = ctx.quantize_nchw_to_s2d(torch.from_numpy(x), QuantParam(117, 0.021), c_pad).cpu().numpy()
    assert np.array_equal(got, qo.quantize_nchw_to_s2d_u8(x, 0.021, 117, c_pad))


@pytest.mark.parametrize("shape", [(2, 7, 7, 40), (1, 1, 1, 1000), (3, 5, 6, 33)])
def test_dequantize_nhwc_to_nchw_and_layout(ctx, qo, shape):
    q = np.random.default_rng(4).integers(0, 256, shape, dtype=np.uint8)
    got = ctx.dequantize_nhwc_to_nchw(torch.from_numpy(q), QuantParam(9, 0.5)).cpu().numpy()
    assert np.array_equal(got, qo.dequantize_nhwc_to_nchw_f32(q, 0.5, 9))
    nchw = ctx.nhwc_to_nchw(torch.from_numpy(q))
    assert np.array_equal(nchw.cpu().numpy(), q.transpose(0, 3, 1, 2))
    assert np.array_equal(ctx.nchw_to_nhwc(nchw).cpu().numpy(), q)


@pytest.mark.parametrize("n", [1, 16, 100003])
def test_qadd(ctx, qo, n):
    rng = np.random.default_rng(n)
    a = rng.integers(0, 256, n, dtype=np.uint8)
    b = rng.integers(0, 256, n, dtype=np.uint8)
    qa, qb, qc = QuantParam(120, 0.021), QuantParam(131, 0.017), QuantParam(125, 0.03)
    got = ctx.binary_add(torch.from_numpy(a), qa, torch.from_numpy(b), qb, qc).cpu().numpy()
    assert np.array_equal(got, qo.qadd_u8(a, b, 0.021, 120, 0.017, 131, 0.03, 125))


def test_qadd_all_pairs(ctx, qo):
    a, b = np.meshgrid(np.arange(256, dtype=np.uint8), np.arange(256, dtype=np.uint8))
    a, b = a.ravel().copy(), b.ravel().copy()
    got = ctx.binary_add(torch.from_numpy(a), QuantParam(3, 0.11), torch.from_numpy(b), QuantParam(250, 0.07),
                         QuantParam(128, 0.09)).cpu().numpy()
    assert np.array_equal(got, qo.qadd_u8(a, b, 0.11, 3, 0.07, 250, 0.09, 128))


def test_requant_relu(ctx, qo):
    x = np.tile(np.arange(256, dtype=np.uint8), 300)
    got = ctx.clamp_requant(torch.from_numpy(x), QuantParam(121, 0.04), QuantParam(0, 0.02), 0.0, float("inf"))
    assert np.array_equal(got.cpu().numpy(), qo.requant_u8(x, 0.04, 121, 0.02, 0, 0.0, np.inf))
    got6 = ctx.clamp_requant(torch.from_numpy(x), QuantParam(121, 0.04), QuantParam(0, 0.0235), 0.0, 6.0)
    assert np.array_equal(got6.cpu().numpy(), qo.requant_u8(x, 0.04, 121, 0.0235, 0, 0.0, 6.0))


@pytest.mark.parametrize("shape,k,s,pad", [((2, 112, 112, 64), (3, 3), (2, 2), (1, 1, 1, 1)),
                                           ((1, 9, 11, 5), (3, 3), (2, 2), (1, 1, 1, 1)),
                                           ((1, 20, 20, 32), (5, 5), (1, 1), (2, 2, 2, 2)),
                                           ((1, 8, 8, 16), (2, 2), (2, 2), (0, 0, 0, 0)),
                                           ((1, 10, 10, 16), (3, 2), (1, 1), (1, 1, 0, 1))])
def test_maxpool(ctx, qo, shape, k, s, pad):
    q = np.random.default_rng(8).integers(0, 256, shape, dtype=np.uint8)
    q[0, :3, :3] = np.minimum(q[0, :3, :3], 100)  # corner below the zero point: padding must win
    got = ctx.reduce_window2d_max(torch.from_numpy(q), QuantParam(140, 0.05), k, s, pad).cpu().numpy()
    assert np.array_equal(got, qo.maxpool_u8(q, k, s, pad, 140))


@pytest.mark.parametrize("shape", [(4, 7, 7, 2048), (2, 3, 5, 7)])
def test_global_mean(ctx, qo, shape):
    q = np.random.default_rng(9).integers(0, 256, shape, dtype=np.uint8)
    got = ctx.global_mean(torch.from_numpy(q), QuantParam(10, 0.02), QuantParam(3, 0.011)).cpu().numpy()
    assert np.array_equal(got, qo.global_avgpool_u8(q, 0.02, 10, 0.011, 3))


def test_size_independent_properties_full_size(ctx):
    """At the ResNet-50 input size (512x3x224x224 = 77 M elements): idempotence of
    quantize(dequantize(.)) and monotonicity, which need no oracle."""
    n = 512 * 3 * 224 * 224
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(n, device="cuda", generator=g)
    qp = QuantParam(128, 0.03)
    q = ctx.quantize(x, qp)
    assert torch.equal(ctx.quantize(ctx.dequantize(q, qp), qp), q)
    xs, _ = torch.sort(x[: 1 << 22])
    qs = ctx.quantize(xs, qp)
    assert bool((qs[1:] >= qs[:-1]).all())
    ctx.check_status()


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
def test_activation(ctx, qo, kind):
    x = np.random.default_rng(20 + kind).integers(0, 256, 100003, dtype=np.uint8)
    qi, qo_ = QuantParam(131, 0.0471), QuantParam(9, 0.0312)
    got = ctx.activation(kind, torch.from_numpy(x), qi, qo_).cpu().numpy()
    assert np.array_equal(got, qo.lut_u8(x, qo.activation_table(kind, 0.0471, 131, 0.0312, 9)))


@pytest.mark.parametrize("shape", [(1, 1000), (512, 1000), (7, 33), (3, 1)])
def test_softmax(ctx, qo, shape):
    """f32 result within 1e-3 of the output range (the exp and the summation order differ)."""
    x = np.random.default_rng(30).normal(0, 4, shape).astype(np.float32)
    got = ctx.softmax(torch.from_numpy(x)).cpu().numpy()
    want = qo.softmax_f32(x)
    assert np.abs(got - want).max() <= 1e-3 * max(float(want.max() - want.min()), 1e-6)
    assert np.allclose(got.sum(-1), 1.0, atol=1e-5)


@pytest.mark.parametrize("shape,c_pad", [((2, 18, 22, 3), 32), ((1, 224, 224, 3), 32), ((2, 8, 8, 4), 16)])
def test_quantize_nhwc_to_s2d(ctx, qo, shape, c_pad):
    """The NHWC-input form gives the bytes of the NCHW form on the transposed input."""
    x = np.random.default_rng(14).normal(0, 1, shape).astype(np.float32)
    got = ctx.quantize_nhwc_to_s2d(torch.from_numpy(x), QuantParam(117, 0.021), c_pad).cpu().numpy()
    want = qo.quantize_nchw_to_s2d_u8(np.ascontiguousarray(x.transpose(0, 3, 1, 2)), 0.021, 117, c_pad)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("src_c,src_off,dst_c,dst_off,length", [(64, 0, 192, 64, 64), (64, 32, 32, 0, 32),
                                                               (40, 3, 51, 7, 29), (16, 0, 16, 0, 0)])
@pytest.mark.parametrize("with_table", [False, True])
def test_copy_channels(ctx, qo, src_c, src_off, dst_c, dst_off, length, with_table):
    rng = np.random.default_rng(15)
    src = rng.integers(0, 256, (2, 9, 11, src_c), dtype=np.uint8)
    dst0 = rng.integers(0, 256, (2, 9, 11, dst_c), dtype=np.uint8)
    table = qo.requant_table(0.031, 120, 0.047, 99) if with_table else None
    got = ctx.copy_channels(torch.from_numpy(src), src_off, torch.from_numpy(dst0.copy()), dst_off, length, table)
    want = dst0.copy()
    qo.copy_channels_u8(src, src_off, want, dst_off, length, table)
    assert np.array_equal(got.cpu().numpy(), want)


def test_copy_channels_rejects_out_of_range(ctx):
    from nncase_b200.kernels import NncbError
    a = torch.zeros((1, 2, 2, 16), dtype=torch.uint8)
    with pytest.raises(NncbError):
        ctx.copy_channels(a, 8, a.clone(), 0, 16)


@pytest.mark.parametrize("shape,f", [((2, 10, 10, 256), 2), ((1, 7, 5, 33), 3), ((3, 20, 20, 128), 2)])
def test_resize_nearest(ctx, qo, shape, f):
    x = np.random.default_rng(16).integers(0, 256, shape, dtype=np.uint8)
    got = ctx.resize_nearest(torch.from_numpy(x), f, f).cpu().numpy()
    assert np.array_equal(got, qo.resize_nearest_u8(x, f, f))
    assert np.array_equal(got, x.repeat(f, 1).repeat(f, 2))


@pytest.mark.parametrize("nhwc", [False, True])
@pytest.mark.parametrize("shape,c_pad,pad", [((2, 3, 18, 22), 16, (2, 1, 2, 1)), ((1, 3, 224, 224), 16, (2, 1, 2, 1)),
                                             ((2, 4, 8, 8), 32, (1, 0, 1, 0)), ((1, 3, 6, 4), 16, (0, 0, 0, 3))])
def test_quantize_to_s2d_padded(ctx, qo, shape, c_pad, pad, nhwc):
    """Space-to-depth cells inside a border of zero-point cells (the stem convolution's padding as data)."""
    x = np.random.default_rng(17).normal(0, 1, shape).astype(np.float32)
    xin = np.ascontiguousarray(x.transpose(0, 2, 3, 1)) if nhwc else x
    got = ctx.quantize_to_s2d_padded(torch.from_numpy(xin), QuantParam(117, 0.021), c_pad, pad, nhwc=nhwc).cpu().numpy()
    assert np.array_equal(got, qo.quantize_nchw_to_s2d_u8(x, 0.021, 117, c_pad, pad))


@pytest.mark.parametrize("op", ["mean", "min", "max", "sum"])
@pytest.mark.parametrize("geom", [((3, 3), (2, 2), (1, 1, 1, 1)), ((2, 2), (2, 2), (0, 0, 0, 0)), ((5, 3), (1, 2), (2, 2, 1, 0)),
                                  ((7, 7), (1, 1), (0, 0, 0, 0))])
def test_reduce_window2d_all_reducers(ctx, qo, op, geom):
    """Windowed mean / min / max / sum (reference/reduce_window.cpp:35-182) on ragged shapes, with and without
    counting padded taps in the mean."""
    k, s, pad = geom
    x = np.random.default_rng(31).integers(0, 256, (2, 13, 10, 24), dtype=np.uint8)
    qi = QuantParam(120, 0.05)
    qo_ = QuantParam(90, 0.05 * (k[0] * k[1] if op == "sum" else 1))
    for cip in (False, True):
        got = ctx.reduce_window2d(op, torch.from_numpy(x), qi, qo_, k, s, pad, cip).cpu().numpy()
        want = qo.reduce_window2d_u8(op, x, k, s, pad, qi.scale, qi.zero_point, qo_.scale, qo_.zero_point, cip)
        assert np.array_equal(got, want)
    # max with equal quant params is the specialised max-pool
    if op == "max":
        assert np.array_equal(ctx.reduce_window2d("max", torch.from_numpy(x), qi, qi, k, s, pad).cpu().numpy(),
                              qo.maxpool_u8(x, k, s, pad, qi.zero_point))


@pytest.mark.parametrize("op", ["add", "sub", "mul", "min", "max"])
def test_binary_operators(ctx, qo, op):
    rng = np.random.default_rng(32)
    a = rng.integers(0, 256, 100003, dtype=np.uint8)
    b = rng.integers(0, 256, 100003, dtype=np.uint8)
    qa, qb, qy = QuantParam(117, 0.05), QuantParam(125, 0.04), QuantParam(121, 0.2 if op == "mul" else 0.06)
    got = ctx.binary(op, torch.from_numpy(a), qa, torch.from_numpy(b), qb, qy).cpu().numpy()
    want = qo.qbinary_u8(op, a, b, qa.scale, qa.zero_point, qb.scale, qb.zero_point, qy.scale, qy.zero_point)
    assert np.array_equal(got, want)
