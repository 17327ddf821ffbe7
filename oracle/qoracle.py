"""ctypes bindings of the C oracle (qoracle.c). TEST INFRASTRUCTURE ONLY."""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class ConvDesc(C.Structure):
    _fields_ = [(k, C.c_int32) for k in
                ("n", "h", "w", "c", "oc", "kh", "kw", "stride_h", "stride_w", "pad_t", "pad_b",
                 "pad_l", "pad_r", "dil_h", "dil_w", "groups", "w_signed", "x_zp")] + \
               [("out_scale", C.c_float), ("out_zp", C.c_int32), ("clamp_lo", C.c_float),
                ("clamp_hi", C.c_float)]


def build():
    subprocess.check_call(["make", "-s", "-C", _HERE, "port"])


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libqoracle.so")
        src = os.path.join(_HERE, "qoracle.c")
        if not os.path.exists(path) or (os.path.exists(src) and os.path.getmtime(src) > os.path.getmtime(path)):
            build()
        _LIB = C.CDLL(path)
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def out_size(i, k, s, d, pb, pa):
    return (i + pb + pa - ((k - 1) * d + 1)) // s + 1


def quantize_u8(x, scale, zp):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(x.shape, np.uint8)
    lib().qo_quantize_u8(_p(x), _p(y), C.c_size_t(x.size), C.c_float(scale), C.c_int32(zp))
    return y


def quantize_i8(x, scale, zp):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(x.shape, np.int8)
    lib().qo_quantize_i8(_p(x), _p(y), C.c_size_t(x.size), C.c_float(scale), C.c_int32(zp))
    return y


def dequantize_u8(q, scale, zp):
    q = np.ascontiguousarray(q, np.uint8)
    y = np.empty(q.shape, np.float32)
    lib().qo_dequantize_u8(_p(q), _p(y), C.c_size_t(q.size), C.c_float(scale), C.c_int32(zp))
    return y


def dequantize_i8(q, scale, zp):
    q = np.ascontiguousarray(q, np.int8)
    y = np.empty(q.shape, np.float32)
    lib().qo_dequantize_i8(_p(q), _p(y), C.c_size_t(q.size), C.c_float(scale), C.c_int32(zp))
    return y


def quantize_nchw_to_nhwc_u8(x, scale, zp, c_pad=None):
    x = np.ascontiguousarray(x, np.float32)
    n, c, h, w = x.shape
    c_pad = c_pad or c
    y = np.empty((n, h, w, c_pad), np.uint8)
    lib().qo_quantize_nchw_to_nhwc_u8(_p(x), _p(y), n, c, h, w, c_pad, C.c_float(scale),
                                      C.c_int32(zp))
    return y


def quantize_nchw_to_s2d_u8(x, scale, zp, c_pad=32, pad=(0, 0, 0, 0)):
    """pad = (top, bottom, left, right) cells of zero point around the space-to-depth cells."""
    x = np.ascontiguousarray(x, np.float32)
    n, c, h, w = x.shape
    y = np.empty((n, h // 2, w // 2, c_pad), np.uint8)
    lib().qo_quantize_nchw_to_s2d_u8(_p(x), _p(y), n, c, h, w, c_pad, C.c_float(scale), C.c_int32(zp))
    if any(pad):
        q0 = np.uint8(min(max(int(zp), 0), 255))
        y = np.pad(y, ((0, 0), (pad[0], pad[1]), (pad[2], pad[3]), (0, 0)), constant_values=q0)
    return np.ascontiguousarray(y)


def qconv2d_u8(x, w, w_zp, mult, bias, x_zp, out_scale, out_zp, stride=(1, 1),
               pad=(0, 0, 0, 0), dilation=(1, 1), groups=1, clamp=(-np.inf, np.inf), lut=None,
               return_acc=False, f32_out=False):
    """x: u8 NHWC; w: u8 or i8 OHWI ([oc, kh, kw, c/groups]); pad = (top, bottom, left, right)."""
    x = np.ascontiguousarray(x, np.uint8)
    assert w.dtype in (np.uint8, np.int8)
    w = np.ascontiguousarray(w)
    n, h, wd, c = x.shape
    oc, kh, kw, gic = w.shape
    assert gic * groups == c
    d = ConvDesc(n, h, wd, c, oc, kh, kw, stride[0], stride[1], pad[0], pad[1], pad[2], pad[3],
                 dilation[0], dilation[1], groups, int(w.dtype == np.int8), int(x_zp),
                 float(out_scale), int(out_zp), float(clamp[0]), float(clamp[1]))
    oh = out_size(h, kh, stride[0], dilation[0], pad[0], pad[1])
    ow = out_size(wd, kw, stride[1], dilation[1], pad[2], pad[3])
    mult = np.ascontiguousarray(mult, np.float32)
    bias = np.ascontiguousarray(bias, np.float32)
    wz = None if w_zp is None else np.ascontiguousarray(w_zp, np.int32)
    if f32_out:
        y = np.empty((n, oh, ow, oc), np.float32)
        lib().qo_qconv2d_f32out(C.byref(d), _p(x), _p(w), _p(wz), _p(mult), _p(bias), _p(y))
        return y
    y = np.empty((n, oh, ow, oc), np.uint8)
    acc = np.empty((n, oh, ow, oc), np.int32) if return_acc else None
    lt = None if lut is None else np.ascontiguousarray(lut, np.uint8)
    lib().qo_qconv2d_u8(C.byref(d), _p(x), _p(w), _p(wz), _p(mult), _p(bias), _p(lt), _p(y),
                        _p(acc))
    return (y, acc) if return_acc else y


def qadd_u8(a, b, sa, za, sb, zb, so, zo):
    a = np.ascontiguousarray(a, np.uint8)
    b = np.ascontiguousarray(b, np.uint8)
    y = np.empty(a.shape, np.uint8)
    lib().qo_qadd_u8(_p(a), _p(b), _p(y), C.c_size_t(a.size), C.c_float(sa), C.c_int32(za),
                     C.c_float(sb), C.c_int32(zb), C.c_float(so), C.c_int32(zo))
    return y


def requant_u8(x, si, zi, so, zo, lo=-np.inf, hi=np.inf):
    x = np.ascontiguousarray(x, np.uint8)
    y = np.empty(x.shape, np.uint8)
    lib().qo_requant_u8(_p(x), _p(y), C.c_size_t(x.size), C.c_float(si), C.c_int32(zi),
                        C.c_float(so), C.c_int32(zo), C.c_float(lo), C.c_float(hi))
    return y


def maxpool_u8(x, k, s, pad, zp):
    x = np.ascontiguousarray(x, np.uint8)
    n, h, w, c = x.shape
    oh = out_size(h, k[0], s[0], 1, pad[0], pad[1])
    ow = out_size(w, k[1], s[1], 1, pad[2], pad[3])
    y = np.empty((n, oh, ow, c), np.uint8)
    lib().qo_maxpool_u8(_p(x), _p(y), n, h, w, c, k[0], k[1], s[0], s[1], pad[0], pad[1],
                        pad[2], pad[3], C.c_int32(zp))
    return y


REDUCE_OPS = {"mean": 0, "min": 1, "max": 2, "sum": 3}   # reduce_op_t
BINARY_OPS = {"add": 0, "sub": 1, "mul": 2, "min": 5, "max": 6}  # binary_op_t


def reduce_window2d_u8(op, x, k, s, pad, si, zi, so, zo, count_include_pad=False):
    x = np.ascontiguousarray(x, np.uint8)
    n, h, w, c = x.shape
    oh = out_size(h, k[0], s[0], 1, pad[0], pad[1])
    ow = out_size(w, k[1], s[1], 1, pad[2], pad[3])
    y = np.empty((n, oh, ow, c), np.uint8)
    lib().qo_reduce_window2d_u8(REDUCE_OPS[op], _p(x), _p(y), n, h, w, c, k[0], k[1], s[0], s[1], pad[0], pad[1], pad[2],
                                pad[3], int(count_include_pad), C.c_float(si), C.c_int32(zi), C.c_float(so), C.c_int32(zo))
    return y


def qbinary_u8(op, a, b, sa, za, sb, zb, so, zo):
    a = np.ascontiguousarray(a, np.uint8)
    b = np.ascontiguousarray(b, np.uint8)
    y = np.empty(a.shape, np.uint8)
    assert lib().qo_qbinary_u8(BINARY_OPS[op], _p(a), _p(b), _p(y), C.c_size_t(a.size), C.c_float(sa), C.c_int32(za),
                               C.c_float(sb), C.c_int32(zb), C.c_float(so), C.c_int32(zo)) == 0
    return y


def global_avgpool_u8(x, si, zi, so, zo):
    x = np.ascontiguousarray(x, np.uint8)
    n, h, w, c = x.shape
    y = np.empty((n, 1, 1, c), np.uint8)
    lib().qo_global_avgpool_u8(_p(x), _p(y), n, h, w, c, C.c_float(si), C.c_int32(zi),
                               C.c_float(so), C.c_int32(zo))
    return y


def dequantize_nhwc_to_nchw_f32(q, scale, zp):
    q = np.ascontiguousarray(q, np.uint8)
    n, h, w, c = q.shape
    y = np.empty((n, c, h, w), np.float32)
    lib().qo_dequantize_nhwc_to_nchw_f32(_p(q), _p(y), n, h, w, c, C.c_float(scale),
                                         C.c_int32(zp))
    return y


def activation_table(kind, si, zi, so, zo):
    t = np.empty(256, np.uint8)
    assert lib().qo_activation_table(kind, C.c_float(si), C.c_int32(zi), C.c_float(so), C.c_int32(zo), _p(t)) == 0
    return t


def lut_u8(x, table):
    x = np.ascontiguousarray(x, np.uint8)
    y = np.empty(x.shape, np.uint8)
    t = np.ascontiguousarray(table, np.uint8)
    lib().qo_lut_u8(_p(x), _p(y), C.c_size_t(x.size), _p(t))
    return y


def softmax_f32(x, beta=1.0):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(x.shape, np.float32)
    cols = x.shape[-1]
    lib().qo_softmax_f32(_p(x), _p(y), C.c_size_t(x.size // cols), cols, C.c_float(beta))
    return y


def copy_channels_u8(src, src_off, dst, dst_off, length, table=None):
    """In place on dst (NHWC arrays): dst[..., dst_off:dst_off+length] = table[src[..., src_off:...]]."""
    assert src.flags.c_contiguous and dst.flags.c_contiguous
    pixels = src.size // src.shape[-1]
    t = None if table is None else np.ascontiguousarray(table, np.uint8)
    lib().qo_copy_channels_u8(_p(src), src.shape[-1], src_off, _p(dst), dst.shape[-1], dst_off, length,
                              C.c_size_t(pixels), _p(t))


def resize_nearest_u8(x, fy, fx):
    x = np.ascontiguousarray(x, np.uint8)
    n, h, w, c = x.shape
    y = np.empty((n, h * fy, w * fx, c), np.uint8)
    lib().qo_resize_nearest_u8(_p(x), _p(y), n, h, w, c, fy, fx)
    return y


def requant_table(si, zi, so, zo, lo=-np.inf, hi=np.inf):
    return requant_u8(np.arange(256, dtype=np.uint8), si, zi, so, zo, lo, hi)
