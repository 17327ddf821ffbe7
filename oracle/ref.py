"""ctypes bindings of the reference's own CPU kernels (oracle/_ref/libnncase_ref.so).

TEST INFRASTRUCTURE ONLY. The library is compiled by ``make -C oracle ref`` from the
reference checkout; where neither the checkout nor a prebuilt library exists,
``available()`` is False and callers skip.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "_ref", "libnncase_ref.so")
_LIB = None


def reference_root():
    """The nncase checkout to compile from: $NNCASE_REF, else a `reference` directory beside this
    repository; None when neither exists."""
    cand = os.environ.get("NNCASE_REF") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "src", "Native")) else None


def build(ref_root=None):
    ref_root = ref_root or reference_root()
    if ref_root:
        subprocess.check_call(["make", "-s", "-j8", "-C", _HERE, "ref", "REF=" + ref_root])


def available():
    return os.path.exists(_PATH)


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(_PATH)
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _chk(rc):
    if rc != 0:
        raise RuntimeError("reference kernel returned an error")


def quantize_u8(x, scale, zp, optimized=True):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(x.shape, np.uint8)
    _chk(lib().nncase_ref_quantize_u8(_p(x), _p(y), C.c_size_t(x.size), C.c_float(scale),
                                      C.c_int32(zp), int(optimized)))
    return y


def quantize_i8(x, scale, zp, optimized=True):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(x.shape, np.int8)
    _chk(lib().nncase_ref_quantize_i8(_p(x), _p(y), C.c_size_t(x.size), C.c_float(scale),
                                      C.c_int32(zp), int(optimized)))
    return y


def dequantize_u8(q, scale, zp, optimized=True):
    q = np.ascontiguousarray(q, np.uint8)
    y = np.empty(q.shape, np.float32)
    _chk(lib().nncase_ref_dequantize_u8(_p(q), _p(y), C.c_size_t(q.size), C.c_float(scale),
                                        C.c_int32(zp), int(optimized)))
    return y


def dequantize_i8(q, scale, zp, optimized=True):
    q = np.ascontiguousarray(q, np.int8)
    y = np.empty(q.shape, np.float32)
    _chk(lib().nncase_ref_dequantize_i8(_p(q), _p(y), C.c_size_t(q.size), C.c_float(scale),
                                        C.c_int32(zp), int(optimized)))
    return y


def conv2d_f32(x, w, b, stride=(1, 1), pad=(0, 0, 0, 0), dilation=(1, 1), groups=1,
               clamp=(-np.inf, np.inf)):
    """x NCHW, w OIHW, pad = (top, bottom, left, right)."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    n, c, h, wd = x.shape
    oc, _, kh, kw = w.shape
    oh = (h + pad[0] + pad[1] - ((kh - 1) * dilation[0] + 1)) // stride[0] + 1
    ow = (wd + pad[2] + pad[3] - ((kw - 1) * dilation[1] + 1)) // stride[1] + 1
    y = np.empty((n, oc, oh, ow), np.float32)
    S = C.c_size_t
    _chk(lib().nncase_ref_conv2d_f32(_p(x), _p(w), _p(b), _p(y), S(n), S(c), S(h), S(wd), S(oc),
                                     S(kh), S(kw), groups, stride[0], stride[1], pad[0], pad[1],
                                     pad[2], pad[3], dilation[0], dilation[1],
                                     C.c_float(clamp[0]), C.c_float(clamp[1])))
    return y


def matmul_f32(a, b):
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    out_shape = np.broadcast_shapes(a.shape[:-2], b.shape[:-2]) + (a.shape[-2], b.shape[-1])
    y = np.empty(out_shape, np.float32)
    sa = (C.c_size_t * a.ndim)(*a.shape)
    sb = (C.c_size_t * b.ndim)(*b.shape)
    _chk(lib().nncase_ref_matmul_f32(_p(a), _p(b), _p(y), sa, C.c_size_t(a.ndim), sb,
                                     C.c_size_t(b.ndim)))
    return y


def softmax_f32(x, axis=-1, beta=1.0):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(x.shape, np.float32)
    s = (C.c_size_t * x.ndim)(*x.shape)
    _chk(lib().nncase_ref_softmax_f32(_p(x), _p(y), s, C.c_size_t(x.ndim), C.c_int64(axis),
                                      C.c_float(beta)))
    return y


def add_f32(a, b):
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    y = np.empty(a.shape, np.float32)
    _chk(lib().nncase_ref_binary_f32(lib().nncase_ref_binary_op_add(), _p(a), _p(b), _p(y),
                                     C.c_size_t(a.size)))
    return y


def reduce_window2d_f32(op, x, k, s, pad, init, count_include_pad=False):
    """op: 'max' or 'mean'; x NCHW."""
    x = np.ascontiguousarray(x, np.float32)
    n, c, h, w = x.shape
    oh = (h + pad[0] + pad[1] - k[0]) // s[0] + 1
    ow = (w + pad[2] + pad[3] - k[1]) // s[1] + 1
    y = np.empty((n, c, oh, ow), np.float32)
    opc = lib().nncase_ref_reduce_op_max() if op == "max" else lib().nncase_ref_reduce_op_mean()
    S = C.c_size_t
    _chk(lib().nncase_ref_reduce_window2d_f32(opc, _p(x), C.c_float(init), _p(y), S(n), S(c),
                                              S(h), S(w), k[0], k[1], s[0], s[1], pad[0],
                                              pad[1], pad[2], pad[3], int(count_include_pad)))
    return y


def qconv2d_composite_u8(xq_nhwc, wq_ohwi, w_zp, w_scale, bias, x_scale, x_zp, out_scale,
                         out_zp, stride=(1, 1), pad=(0, 0, 0, 0), dilation=(1, 1), groups=1,
                         clamp=(-np.inf, np.inf)):
    """The u8 -> u8 convolution exactly as the reference cpu target executes it:
    dequantize(x) and dequantize(w) (per channel), f32 conv2d with fused clamp, quantize
    (how src/Nncase.Importer/Onnx/QLinearConv.cs:61-75 lowers QLinearConv). Takes and returns
    NHWC / OHWI so that it is directly comparable with the integer formulation."""
    n, h, w, c = xq_nhwc.shape
    oc = wq_ohwi.shape[0]
    xf = dequantize_u8(np.ascontiguousarray(xq_nhwc.transpose(0, 3, 1, 2)), x_scale, x_zp)
    w_oihw = np.ascontiguousarray(wq_ohwi.transpose(0, 3, 1, 2))
    wf = np.empty(w_oihw.shape, np.float32)
    for ch in range(oc):
        z = 0 if w_zp is None else int(w_zp[ch])
        if w_oihw.dtype == np.uint8:
            wf[ch] = dequantize_u8(w_oihw[ch], float(w_scale[ch]), z)
        else:
            wf[ch] = dequantize_i8(w_oihw[ch], float(w_scale[ch]), z)
    yf = conv2d_f32(xf, wf, bias, stride, pad, dilation, groups, clamp)
    yq = quantize_u8(yf, out_scale, out_zp)
    return np.ascontiguousarray(yq.transpose(0, 2, 3, 1))


def unary_f32(kind, x):
    """kind: 0 relu, 1 sigmoid, 2 swish, 3 hard_swish -- the reference's kernels::stackvm functions."""
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(x.shape, np.float32)
    _chk(lib().nncase_ref_unary_f32(kind, _p(x), _p(y), C.c_size_t(x.size)))
    return y
