"""Pins the C oracle against the reference's own compiled CPU kernels (oracle/_ref) and against
the committed golden vectors (tests/golden, generated from those same kernels)."""
import os

import numpy as np
import pytest

from oracle import quant_params as QP

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _edge_values(scale, zp):
    # ties, clamp edges and denormals around every quantisation step
    k = np.arange(-300, 300, dtype=np.float32)
    half = (k + np.float32(0.5) - np.float32(zp)) * np.float32(scale)
    return np.concatenate([half, np.nextafter(half, np.float32(np.inf)), np.nextafter(half, np.float32(-np.inf)),
                           np.array([0.0, -0.0, 1e-40, -1e-40, 1e6, -1e6], np.float32)])


@pytest.mark.parametrize("scale,zp", [(0.01, 127), (0.014035294, 88), (0.0078125, 0), (3.7e-3, 255)])
def test_quantize_u8_matches_reference(qo, ref, scale, zp):
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.normal(0, 1, 100000).astype(np.float32), _edge_values(scale, zp)])
    a = qo.quantize_u8(x, scale, zp)
    assert np.array_equal(a, ref.quantize_u8(x, scale, zp, optimized=True))
    assert np.array_equal(a, ref.quantize_u8(x, scale, zp, optimized=False))


@pytest.mark.parametrize("scale,zp", [(0.01, 0), (0.02, -5)])
def test_quantize_i8_matches_reference(qo, ref, scale, zp):
    rng = np.random.default_rng(2)
    x = np.concatenate([rng.normal(0, 1, 50000).astype(np.float32), _edge_values(scale, zp)])
    assert np.array_equal(qo.quantize_i8(x, scale, zp), ref.quantize_i8(x, scale, zp))


def test_dequantize_matches_reference(qo, ref):
    q = np.arange(256, dtype=np.uint8)
    for scale, zp in [(0.01, 127), (0.014035294, 88), (1.5, 3)]:
        assert np.array_equal(qo.dequantize_u8(q, scale, zp), ref.dequantize_u8(q, scale, zp))
        assert np.array_equal(qo.dequantize_u8(q, scale, zp), ref.dequantize_u8(q, scale, zp, optimized=False))
    qi = np.arange(-128, 128, dtype=np.int8)
    assert np.array_equal(qo.dequantize_i8(qi, 0.02, -3), ref.dequantize_i8(qi, 0.02, -3))


def _conv_case(seed, n, h, w, c, oc, k, stride, pad, dil=1, w_signed=False):
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float32)
    wt = rng.normal(0, 0.05, (oc, k, k, c)).astype(np.float32)
    b = rng.normal(0, 0.01, oc).astype(np.float32)
    zx, sx = QP.get_quant_param(*QP.get_min_max(x))
    mode = QP.SIGNED_SYMMETRIC if w_signed else QP.UNSIGNED
    zw, sw = QP.weights_quant_params(wt, oc, 8, mode)
    return x, wt, b, zx, sx, zw, sw


@pytest.mark.parametrize("shape", [
    # n, h, w, c, oc, k, stride, pad, dil   (shapes of the reference's tests/kernels/test_conv2d.json plus config 1 scaled)
    (1, 5, 5, 4, 8, 3, 1, 1, 1), (1, 16, 16, 4, 8, 3, 2, 1, 1), (1, 16, 16, 4, 8, 3, 1, 1, 2),
    (1, 16, 16, 4, 8, 1, 1, 0, 1), (2, 14, 14, 64, 64, 3, 1, 1, 1), (1, 7, 9, 32, 16, 3, 2, 1, 1),
])
@pytest.mark.parametrize("w_signed", [False, True])
def test_integer_conv_vs_reference_composite(qo, ref, shape, w_signed):
    """The integer formulation against dequantize -> conv2d(f32, clamp) -> quantize run through the
    reference's kernels: equal up to rare 1-LSB differences from f32 accumulation order."""
    n, h, w, c, oc, k, stride, pad, dil = shape
    x, wt, b, zx, sx, zw, sw = _conv_case(11, n, h, w, c, oc, k, stride, pad, dil, w_signed)
    xq = qo.quantize_u8(x, sx, zx)
    if w_signed:
        wq = np.stack([qo.quantize_i8(wt[i], sw[i], zw[i]) for i in range(oc)])
    else:
        wq = np.stack([qo.quantize_u8(wt[i], sw[i], zw[i]) for i in range(oc)])
    pads = (pad, pad, pad, pad)
    yf = ref.conv2d_f32(x.transpose(0, 3, 1, 2), wt.transpose(0, 3, 1, 2), b, (stride, stride), pads, (dil, dil),
                        clamp=(0, 6))
    zo, so = QP.get_quant_param(*QP.get_min_max(yf))
    mult = (np.float32(sx) * sw).astype(np.float32)
    yq = qo.qconv2d_u8(xq, wq, zw, mult, b, zx, so, zo, (stride, stride), pads, (dil, dil), clamp=(0, 6))
    yr = ref.qconv2d_composite_u8(xq, wq, zw, sw, b, sx, zx, so, zo, (stride, stride), pads, (dil, dil), clamp=(0, 6))
    diff = np.abs(yq.astype(np.int32) - yr.astype(np.int32))
    assert diff.max() <= 1
    assert (diff != 0).mean() <= 1e-3


def test_maxpool_padding_takes_zero_point(qo, ref):
    """reduce_window2d max injects the real value 0 for padded taps (reference/reduce_window.cpp:86-90)."""
    rng = np.random.default_rng(3)
    scale, zp = 0.05, 140
    q = rng.integers(0, 130, (1, 9, 9, 4), dtype=np.uint8)  # all real values negative
    y = qo.maxpool_u8(q, (3, 3), (2, 2), (1, 1, 1, 1), zp)
    xf = ref.dequantize_u8(np.ascontiguousarray(q.transpose(0, 3, 1, 2)), scale, zp)
    yf = ref.reduce_window2d_f32("max", xf, (3, 3), (2, 2), (1, 1, 1, 1), init=float(np.finfo(np.float32).min))
    yr = ref.quantize_u8(yf, scale, zp).transpose(0, 2, 3, 1)
    assert np.array_equal(y, yr)
    assert (y[0, 0, 0] == zp).all()  # corner window overlaps padding and all taps are below zero


def test_qadd_vs_reference(qo, ref):
    rng = np.random.default_rng(4)
    a = rng.integers(0, 256, 10000, dtype=np.uint8)
    b = rng.integers(0, 256, 10000, dtype=np.uint8)
    sa, za, sb, zb, so, zo = 0.021, 120, 0.017, 131, 0.03, 125
    y = qo.qadd_u8(a, b, sa, za, sb, zb, so, zo)
    yr = ref.quantize_u8(ref.add_f32(ref.dequantize_u8(a, sa, za), ref.dequantize_u8(b, sb, zb)), so, zo)
    assert np.array_equal(y, yr)


def test_global_mean_vs_reference(qo, ref):
    rng = np.random.default_rng(5)
    q = rng.integers(0, 256, (2, 7, 7, 8), dtype=np.uint8)
    si, zi, so, zo = 0.02, 10, 0.011, 3
    y = qo.global_avgpool_u8(q, si, zi, so, zo)
    xf = ref.dequantize_u8(np.ascontiguousarray(q.transpose(0, 3, 1, 2)), si, zi)
    yf = ref.reduce_window2d_f32("mean", xf, (7, 7), (1, 1), (0, 0, 0, 0), init=0.0)
    yr = ref.quantize_u8(yf, so, zo).transpose(0, 2, 3, 1)
    d = np.abs(y.astype(int) - yr.astype(int))
    assert d.max() <= 1 and (d != 0).mean() < 0.02  # float summation order of the reference differs


def test_golden_vectors(qo):
    """Committed fixtures produced by tests/golden/make_golden.py from the reference's kernels."""
    g = np.load(os.path.join(GOLD, "quantize_dequantize.npz"))
    assert np.array_equal(qo.quantize_u8(g["x"], float(g["scale"]), int(g["zp"])), g["q_u8"])
    assert np.array_equal(qo.dequantize_u8(g["q_u8"], float(g["scale"]), int(g["zp"])), g["deq_f32"])
    c = np.load(os.path.join(GOLD, "conv_config1_slice.npz"))
    yq = qo.qconv2d_u8(c["xq"], c["wq"], c["zw"], c["mult"], c["bias"], int(c["zx"]), float(c["so"]), int(c["zo"]),
                       (1, 1), (1, 1, 1, 1), (1, 1), clamp=(0, 6))
    diff = np.abs(yq.astype(int) - c["y_ref_composite"].astype(int))
    assert diff.max() <= 1 and (diff != 0).sum() <= int(c["allowed_mismatches"])
    assert np.array_equal(yq, c["y_integer"])


def test_space_to_depth_stem_is_the_same_convolution(qo):
    """A 7x7 stride-2 pad-3 stem over 3 channels and its space-to-depth rewrite (4x4, stride 1 over
    32 channels) give identical integer results -- the rewrite only rearranges the products."""
    from nncase_b200.builder import space_to_depth_conv
    rng = np.random.default_rng(12)
    n, c, h, w, oc = 2, 3, 20, 16, 8
    x = rng.normal(0, 1, (n, c, h, w)).astype(np.float32)
    scale, zp = 0.03, 120
    wq = rng.integers(0, 256, (oc, 7, 7, c), dtype=np.uint8)
    zw = rng.integers(100, 150, oc).astype(np.int32)
    mult = rng.uniform(1e-4, 3e-4, oc).astype(np.float32)
    bias = rng.normal(0, 0.1, oc).astype(np.float32)
    x_nhwc = qo.quantize_nchw_to_nhwc_u8(x, scale, zp)
    want = qo.qconv2d_u8(x_nhwc, wq, zw, mult, bias, zp, 0.05, 10, (2, 2), (3, 3, 3, 3), clamp=(0, np.inf))
    x_s2d = qo.quantize_nchw_to_s2d_u8(x, scale, zp, 32)
    w2, pad2 = space_to_depth_conv(wq, zw, (3, 3, 3, 3), (h, w), 32)
    assert w2.shape == (oc, 4, 4, 32) and pad2 == (2, 1, 2, 1)
    got = qo.qconv2d_u8(x_s2d, w2, zw, mult, bias, zp, 0.05, 10, (1, 1), pad2, clamp=(0, np.inf))
    assert np.array_equal(got, want)
    # 3x3 stride 2 pad 1 (MobileNet / YOLO stems)
    wq3 = rng.integers(0, 256, (oc, 3, 3, c), dtype=np.uint8)
    want3 = qo.qconv2d_u8(x_nhwc, wq3, zw, mult, bias, zp, 0.05, 10, (2, 2), (1, 1, 1, 1))
    w3, pad3 = space_to_depth_conv(wq3, zw, (1, 1, 1, 1), (h, w), 32)
    got3 = qo.qconv2d_u8(x_s2d, w3, zw, mult, bias, zp, 0.05, 10, (1, 1), pad3)
    assert w3.shape == (oc, 2, 2, 32) and np.array_equal(got3, want3)


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
def test_activation_tables_vs_reference_kernels(qo, ref, kind):
    """relu / sigmoid / swish / hard_swish tables against the reference's own kernels run on the
    dequantized values and requantised with the reference's quantize."""
    si, zi, so, zo = 0.0471, 131, 0.0312, 9
    q = np.arange(256, dtype=np.uint8)
    want = ref.quantize_u8(ref.unary_f32(kind, ref.dequantize_u8(q, si, zi)), so, zo)
    assert np.array_equal(qo.activation_table(kind, si, zi, so, zo), want)


def test_library_activation_tables_match_oracle(qo):
    from nncase_b200 import kernels as K
    for kind in range(4):
        for (si, zi, so, zo) in [(0.0471, 131, 0.0312, 9), (0.1, 0, 0.004, 0), (0.02, 255, 0.02, 128)]:
            t = K.activation_table(kind, K.QuantParam(zi, si), K.QuantParam(zo, so))
            assert np.array_equal(t, qo.activation_table(kind, si, zi, so, zo))


def test_softmax_vs_reference(qo, ref):
    x = np.random.default_rng(6).normal(0, 3, (37, 1000)).astype(np.float32)
    assert np.array_equal(qo.softmax_f32(x), ref.softmax_f32(x))


@pytest.mark.parametrize("op,code", [("mean", 0), ("min", 1), ("max", 2), ("sum", 3)])
def test_reduce_window2d_vs_reference(qo, ref, op, code):
    """The quantized reduce_window2d against dequantize -> the reference's reduce_window2d -> quantize, padded and
    strided, with and without count_include_pad."""
    import ctypes as C
    q = np.random.default_rng(41).integers(0, 256, (2, 9, 11, 8), dtype=np.uint8)
    si, zi, zo = 0.05, 120, 110
    so = 0.04 * (9 if op == "sum" else 1)
    xf = ref.dequantize_u8(np.ascontiguousarray(q.transpose(0, 3, 1, 2)), si, zi)
    init = {"mean": 0.0, "sum": 0.0, "max": float(np.finfo(np.float32).min), "min": float(np.finfo(np.float32).max)}[op]
    n, c, h, w = xf.shape
    oh, ow = (h + 2 - 3) // 2 + 1, (w + 2 - 3) // 2 + 1
    for cip in (False, True):
        yf = np.empty((n, c, oh, ow), np.float32)
        S = C.c_size_t
        assert ref.lib().nncase_ref_reduce_window2d_f32(code, xf.ctypes.data_as(C.c_void_p), C.c_float(init),
                                                        yf.ctypes.data_as(C.c_void_p), S(n), S(c), S(h), S(w), 3, 3, 2, 2,
                                                        1, 1, 1, 1, int(cip)) == 0
        want = ref.quantize_u8(yf, so, zo).transpose(0, 2, 3, 1)
        got = qo.reduce_window2d_u8(op, q, (3, 3), (2, 2), (1, 1, 1, 1), si, zi, so, zo, cip)
        d = np.abs(got.astype(int) - want.astype(int))
        assert d.max() <= 1 and (d != 0).mean() < 0.02  # float summation order of the reference


@pytest.mark.parametrize("op,code", [("add", 0), ("sub", 1), ("mul", 2), ("min", 5), ("max", 6)])
def test_binary_operators_vs_reference(qo, ref, op, code):
    import ctypes as C
    rng = np.random.default_rng(42)
    a = rng.integers(0, 256, 20000, dtype=np.uint8)
    b = rng.integers(0, 256, 20000, dtype=np.uint8)
    so = 0.2 if op == "mul" else 0.06
    fa, fb = ref.dequantize_u8(a, 0.05, 117), ref.dequantize_u8(b, 0.04, 125)
    yf = np.empty(a.shape, np.float32)
    assert ref.lib().nncase_ref_binary_f32(code, fa.ctypes.data_as(C.c_void_p), fb.ctypes.data_as(C.c_void_p),
                                           yf.ctypes.data_as(C.c_void_p), C.c_size_t(a.size)) == 0
    assert np.array_equal(qo.qbinary_u8(op, a, b, 0.05, 117, 0.04, 125, so, 121), ref.quantize_u8(yf, so, 121))
