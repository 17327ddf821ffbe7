"""Host-side mirror of the reference's ``kernels::stackvm`` operators for the quantized path.

Every function takes and returns ``torch`` CUDA tensors (torch is used for device memory and
streams only) and forwards to the C ABI of ``libnncase_b200.so``. Names and argument meaning
follow ``src/Native/include/nncase/kernels/stackvm/tensor_ops.h`` of the reference:
``quantize(target_type, input, quant_param)``, ``dequantize``, ``conv2d`` (with ``fused_clamp``),
``mat_mul``, ``binary`` (add), ``reduce_window2d`` ... Errors of the library surface as
``NncbError`` carrying the negative errno code, the way the reference's C API reports them.
"""
import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import lib as L
from .lib import Conv2dDesc, NncbError, check

_DT = {torch.uint8: L.U8, torch.int8: L.I8, torch.int16: L.I16}


@dataclass(frozen=True)
class QuantParam:
    """quant_param_t {int32 zero_point; float scale} (include/nncase/runtime/simple_types.h:157-165)."""
    zero_point: int
    scale: float


def get_quant_param(rmin, rmax, bits=8, mode=L.UNSIGNED):
    """QuantUtility.GetQuantParam (src/Nncase.Core/Utilities/QuantUtility.cs:41-67)."""
    zp, sc = C.c_int32(), C.c_float()
    check(L.load().nncb_get_quant_param(float(rmin), float(rmax), bits, mode, C.byref(zp), C.byref(sc)))
    return QuantParam(zp.value, sc.value)


def activation_table(kind, qi, qo):
    """256-entry table of a unary activation between two quant params (host)."""
    t = np.empty(256, np.uint8)
    check(L.load().nncb_make_activation_table(kind, qi.scale, qi.zero_point, qo.scale, qo.zero_point,
                                              t.ctypes.data))
    return t


def fixup_range(rmin, rmax, symmetric=False):
    """QuantUtility.FixupRange (QuantUtility.cs:72-97)."""
    a, b = C.c_float(rmin), C.c_float(rmax)
    check(L.load().nncb_fixup_range(C.byref(a), C.byref(b), int(symmetric)))
    return a.value, b.value


class Context:
    """One device + stream; the stand-in for ``kernel_context``. Launches on torch's current
    stream of the device at construction (re-bind with ``use_current_stream``), so that torch
    events, copies and CUDA-graph capture order correctly with the kernels."""

    def __init__(self, device=0):
        self._lib = L.load()
        if not torch.cuda.is_available():
            raise NncbError(-5, "no CUDA device: nncase_b200 has no CPU fallback")
        self.device = torch.device("cuda", device)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        h = C.c_void_p()
        check(self._lib.nncb_context_create(device, C.c_void_p(stream), C.byref(h)))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            self._lib.nncb_context_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def use_current_stream(self):
        s = torch.cuda.current_stream(self.device).cuda_stream
        check(self._lib.nncb_context_set_stream(self._h, C.c_void_p(s)))

    def synchronize(self):
        check(self._lib.nncb_synchronize(self._h))

    def set_option(self, name, value):
        """Per-context option by name (see nncb_context_set_option): wait limit, tuning overrides."""
        check(self._lib.nncb_context_set_option(self._h, name.encode(), int(value)))

    def get_option(self, name):
        v = C.c_int64()
        check(self._lib.nncb_context_get_option(self._h, name.encode(), C.byref(v)))
        return v.value

    def check_status(self):
        check(self._lib.nncb_check_device_status(self._h))

    @property
    def launches(self):
        return int(self._lib.nncb_launch_count(self._h))

    # ---- Quantize / Dequantize -------------------------------------------------------------
    def quantize(self, x, qp, dtype=torch.uint8):
        x = self._cuda(x, torch.float32)
        y = torch.empty(x.shape, dtype=dtype, device=self.device)
        check(self._lib.nncb_quantize(self._h, x.data_ptr(), y.data_ptr(), x.numel(), qp.scale,
                                      qp.zero_point, _DT[dtype]))
        return y

    def dequantize(self, q, qp):
        q = self._cuda(q)
        y = torch.empty(q.shape, dtype=torch.float32, device=self.device)
        check(self._lib.nncb_dequantize(self._h, q.data_ptr(), y.data_ptr(), q.numel(), qp.scale,
                                        qp.zero_point, _DT[q.dtype]))
        return y

    def quantize_host(self, x, qp, dtype=np.uint8):
        """HOST numpy in, HOST numpy out (copies inside)."""
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty(x.shape, dtype)
        code = {np.dtype(np.uint8): L.U8, np.dtype(np.int8): L.I8, np.dtype(np.int16): L.I16}[np.dtype(dtype)]
        check(self._lib.nncb_quantize_host(self._h, x.ctypes.data, y.ctypes.data, x.size, qp.scale,
                                           qp.zero_point, code))
        return y

    def dequantize_host(self, q, qp):
        q = np.ascontiguousarray(q)
        y = np.empty(q.shape, np.float32)
        code = {np.dtype(np.uint8): L.U8, np.dtype(np.int8): L.I8, np.dtype(np.int16): L.I16}[q.dtype]
        check(self._lib.nncb_dequantize_host(self._h, q.ctypes.data, y.ctypes.data, q.size, qp.scale,
                                             qp.zero_point, code))
        return y

    def quantize_nchw_to_nhwc(self, x, qp, c_pad=None):
        x = self._cuda(x, torch.float32)
        n, c, h, w = x.shape
        c_pad = c_pad or c
        y = torch.empty((n, h, w, c_pad), dtype=torch.uint8, device=self.device)
        check(self._lib.nncb_quantize_nchw_to_nhwc_u8(self._h, x.data_ptr(), y.data_ptr(), n, c, h, w, c_pad,
                                                      qp.scale, qp.zero_point))
        return y

    def quantize_nchw_to_s2d(self, x, qp, c_pad=32):
        """f32 NCHW -> u8 [n, h/2, w/2, c_pad], channel (dy*2+dx)*c + ch (space-to-depth by 2)."""
        x = self._cuda(x, torch.float32)
        n, c, h, w = x.shape
        y = torch.empty((n, h // 2, w // 2, c_pad), dtype=torch.uint8, device=self.device)
        check(self._lib.nncb_quantize_nchw_to_s2d_u8(self._h, x.data_ptr(), y.data_ptr(), n, c, h, w, c_pad,
                                                     qp.scale, qp.zero_point))
        return y

    def quantize_to_s2d_padded(self, x, qp, c_pad, pad, nhwc=False):
        """f32 NCHW (or NHWC) -> u8 [n, h/2+pt+pb, w/2+pl+pr, c_pad]: space-to-depth cells inside a border of
        zero-point cells; pad = (top, bottom, left, right) in cells."""
        x = self._cuda(x, torch.float32)
        if nhwc:
            n, h, w, c = x.shape
        else:
            n, c, h, w = x.shape
        pt, pb, pl, pr = pad
        y = torch.empty((n, h // 2 + pt + pb, w // 2 + pl + pr, c_pad), dtype=torch.uint8, device=self.device)
        check(self._lib.nncb_quantize_to_s2d_padded_u8(self._h, x.data_ptr(), int(nhwc), y.data_ptr(), n, c, h, w, c_pad,
                                                       pt, pb, pl, pr, qp.scale, qp.zero_point))
        return y

    def quantize_nhwc_to_s2d(self, x, qp, c_pad=32):
        """f32 NHWC -> u8 [n, h/2, w/2, c_pad] with the same channel order as quantize_nchw_to_s2d."""
        x = self._cuda(x, torch.float32)
        n, h, w, c = x.shape
        y = torch.empty((n, h // 2, w // 2, c_pad), dtype=torch.uint8, device=self.device)
        check(self._lib.nncb_quantize_nhwc_to_s2d_u8(self._h, x.data_ptr(), y.data_ptr(), n, h, w, c, c_pad,
                                                     qp.scale, qp.zero_point))
        return y

    def copy_channels(self, src, src_off, dst, dst_off, length, table=None):
        """dst[..., dst_off:dst_off+length] = table[src[..., src_off:src_off+length]] on NHWC u8 tensors, in place
        on dst (Slice and one input of Concat; table None copies)."""
        src, dst = self._cuda(src, torch.uint8), self._cuda(dst, torch.uint8)
        pixels = src.numel() // src.shape[-1] if src.shape[-1] else 0
        t = None if table is None else np.ascontiguousarray(table, np.uint8)
        check(self._lib.nncb_copy_channels_u8(self._h, src.data_ptr(), src.shape[-1], src_off, dst.data_ptr(),
                                              dst.shape[-1], dst_off, length, pixels,
                                              t.ctypes.data if t is not None else None))
        return dst

    def resize_nearest(self, x, fy, fx):
        """NHWC u8 nearest-neighbour upsampling by integer factors."""
        x = self._cuda(x, torch.uint8)
        n, h, w, c = x.shape
        y = torch.empty((n, h * fy, w * fx, c), dtype=torch.uint8, device=self.device)
        check(self._lib.nncb_resize_nearest_u8(self._h, x.data_ptr(), y.data_ptr(), n, h, w, c, fy, fx))
        return y

    def dequantize_nhwc_to_nchw(self, q, qp):
        q = self._cuda(q, torch.uint8)
        n, h, w, c = q.shape
        y = torch.empty((n, c, h, w), dtype=torch.float32, device=self.device)
        check(self._lib.nncb_dequantize_nhwc_to_nchw_f32(self._h, q.data_ptr(), y.data_ptr(), n, h, w, c,
                                                         qp.scale, qp.zero_point))
        return y

    def nchw_to_nhwc(self, q):
        q = self._cuda(q, torch.uint8)
        n, c, h, w = q.shape
        y = torch.empty((n, h, w, c), dtype=torch.uint8, device=self.device)
        check(self._lib.nncb_nchw_to_nhwc_u8(self._h, q.data_ptr(), y.data_ptr(), n, c, h, w))
        return y

    def nhwc_to_nchw(self, q):
        q = self._cuda(q, torch.uint8)
        n, h, w, c = q.shape
        y = torch.empty((n, c, h, w), dtype=torch.uint8, device=self.device)
        check(self._lib.nncb_nhwc_to_nchw_u8(self._h, q.data_ptr(), y.data_ptr(), n, h, w, c))
        return y

    # ---- element-wise / pooling ------------------------------------------------------------
    def binary_add(self, a, qa, b, qb, qo):
        a, b = self._cuda(a, torch.uint8), self._cuda(b, torch.uint8)
        if a.shape != b.shape:
            raise NncbError(-22, "binary_add: shapes differ")
        y = torch.empty_like(a)
        check(self._lib.nncb_qadd_u8(self._h, a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(), qa.scale,
                                     qa.zero_point, qb.scale, qb.zero_point, qo.scale, qo.zero_point))
        return y

    def clamp_requant(self, x, qi, qo, lo=-float("inf"), hi=float("inf")):
        x = self._cuda(x, torch.uint8)
        y = torch.empty_like(x)
        check(self._lib.nncb_requant_u8(self._h, x.data_ptr(), y.data_ptr(), x.numel(), qi.scale, qi.zero_point,
                                        qo.scale, qo.zero_point, lo, hi))
        return y

    def activation(self, kind, x, qi, qo):
        """relu / sigmoid / swish / hard_swish (L.ACT_*) on a u8 tensor between quant params."""
        x = self._cuda(x, torch.uint8)
        y = torch.empty_like(x)
        check(self._lib.nncb_activation_u8(self._h, kind, x.data_ptr(), y.data_ptr(), x.numel(), qi.scale,
                                           qi.zero_point, qo.scale, qo.zero_point))
        return y

    def softmax(self, x, beta=1.0):
        """softmax over the last axis of an f32 tensor."""
        x = self._cuda(x, torch.float32)
        y = torch.empty_like(x)
        cols = x.shape[-1]
        check(self._lib.nncb_softmax_f32(self._h, x.data_ptr(), y.data_ptr(), x.numel() // cols, cols, beta))
        return y

    def lut(self, x, table):
        x = self._cuda(x, torch.uint8)
        t = np.ascontiguousarray(table, np.uint8)
        assert t.size == 256
        y = torch.empty_like(x)
        check(self._lib.nncb_lut_u8(self._h, x.data_ptr(), y.data_ptr(), x.numel(), t.ctypes.data))
        return y

    def reduce_window2d_max(self, x, qp, filter, stride, padding):
        """x u8 NHWC; padding = (top, bottom, left, right)."""
        x = self._cuda(x, torch.uint8)
        n, h, w, c = x.shape
        oh = (h + padding[0] + padding[1] - filter[0]) // stride[0] + 1
        ow = (w + padding[2] + padding[3] - filter[1]) // stride[1] + 1
        y = torch.empty((n, oh, ow, c), dtype=torch.uint8, device=self.device)
        check(self._lib.nncb_maxpool_u8(self._h, x.data_ptr(), y.data_ptr(), n, h, w, c, filter[0], filter[1],
                                        stride[0], stride[1], padding[0], padding[1], padding[2], padding[3],
                                        qp.zero_point))
        return y

    REDUCE_OPS = {"mean": 0, "min": 1, "max": 2, "sum": 3}    # reduce_op_t of the reference
    BINARY_OPS = {"add": 0, "sub": 1, "mul": 2, "min": 5, "max": 6}  # binary_op_t

    def reduce_window2d(self, op, x, qi, qo, filter, stride, padding, count_include_pad=False):
        """kernels::stackvm::reduce_window2d between quant params: op in mean / min / max / sum; x u8 NHWC;
        padding = (top, bottom, left, right)."""
        x = self._cuda(x, torch.uint8)
        n, h, w, c = x.shape
        oh = (h + padding[0] + padding[1] - filter[0]) // stride[0] + 1
        ow = (w + padding[2] + padding[3] - filter[1]) // stride[1] + 1
        y = torch.empty((n, oh, ow, c), dtype=torch.uint8, device=self.device)
        check(self._lib.nncb_reduce_window2d_u8(self._h, self.REDUCE_OPS[op], x.data_ptr(), y.data_ptr(), n, h, w, c,
                                                filter[0], filter[1], stride[0], stride[1], *padding, int(count_include_pad),
                                                qi.scale, qi.zero_point, qo.scale, qo.zero_point))
        return y

    def binary(self, op, a, qa, b, qb, qo):
        """kernels::stackvm::binary between quantized tensors of equal shape: op in add / sub / mul / min / max."""
        a, b = self._cuda(a, torch.uint8), self._cuda(b, torch.uint8)
        if a.shape != b.shape:
            raise NncbError(-22, "binary: shapes differ")
        y = torch.empty_like(a)
        check(self._lib.nncb_qbinary_u8(self._h, self.BINARY_OPS[op], a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(),
                                        qa.scale, qa.zero_point, qb.scale, qb.zero_point, qo.scale, qo.zero_point))
        return y

    def global_mean(self, x, qi, qo):
        x = self._cuda(x, torch.uint8)
        n, h, w, c = x.shape
        y = torch.empty((n, 1, 1, c), dtype=torch.uint8, device=self.device)
        check(self._lib.nncb_global_avgpool_u8(self._h, x.data_ptr(), y.data_ptr(), n, h, w, c, qi.scale,
                                               qi.zero_point, qo.scale, qo.zero_point))
        return y

    # ---- paged attention ----------------------------------------------------------------------
    def paged_attention_decode(self, q, k_pool, v_pool, block_table, context_lens, scale=None, workspace=None):
        """q [B,Hq,D] f16; k_pool/v_pool [pages,Hkv,page,D] f16; block_table [B,max_pages] i32;
        context_lens [B] i32 -> out [B,Hq,D] f16."""
        q = self._cuda(q, torch.float16)
        k_pool, v_pool = self._cuda(k_pool, torch.float16), self._cuda(v_pool, torch.float16)
        block_table = self._cuda(block_table, torch.int32)
        context_lens = self._cuda(context_lens, torch.int32)
        b, hq, d = q.shape
        _, hkv, page, _ = k_pool.shape
        max_pages = block_table.shape[1]
        scale = float(scale) if scale is not None else 1.0 / float(np.sqrt(d))
        need = C.c_size_t()
        check(self._lib.nncb_paged_attention_workspace_size(self._h, b, hq, hkv, d, page, max_pages, C.byref(need)))
        if workspace is None and need.value:
            workspace = torch.empty(need.value, dtype=torch.uint8, device=self.device)
        out = torch.empty_like(q)
        check(self._lib.nncb_paged_attention_decode(
            self._h, q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(),
            context_lens.data_ptr(), out.data_ptr(), b, hq, hkv, d, page, max_pages, k_pool.shape[0], scale,
            workspace.data_ptr() if workspace is not None else None,
            workspace.numel() if workspace is not None else 0))
        return out

    # ---- conv2d / mat_mul -------------------------------------------------------------------
    def conv2d_plan(self, in_shape, weights, w_zp, mult, bias, x_zp, out_qp, stride=(1, 1), padding=(0, 0, 0, 0),
                    dilation=(1, 1), groups=1, fused_clamp=(-float("inf"), float("inf")), lut=None,
                    residual=None, y2=None, f32_out=False, force_path=L.PATH_AUTO):
        """Create a reusable convolution plan.

        in_shape: (n, h, w, c); weights: numpy u8|i8 OHWI; w_zp: int32[oc] or None;
        mult: f32[oc] = sx*sw[oc]; bias f32[oc]; out_qp: QuantParam of the u8 result.
        residual: None or (res_qp, add_out_qp); y2: None or (y2_qp, lo, hi).
        """
        return Conv2dPlan(self, in_shape, weights, w_zp, mult, bias, x_zp, out_qp, stride, padding, dilation,
                          groups, fused_clamp, lut, residual, y2, f32_out, force_path)

    def conv2d(self, x, weights, w_zp, mult, bias, x_zp, out_qp, **kw):
        """One-shot quantized conv2d on a device tensor (plan is created and dropped)."""
        x = self._cuda(x, torch.uint8)
        res = kw.pop("res", None)
        plan = self.conv2d_plan(tuple(x.shape), weights, w_zp, mult, bias, x_zp, out_qp, **kw)
        try:
            return plan(x, res)
        finally:
            self.synchronize()
            plan.close()

    def mat_mul(self, a, weights_nk, w_zp, mult, bias, a_zp, out_qp, **kw):
        """[M,K] u8 x [N,K] weights -> [M,N]: the 1x1 convolution n=1,h=1,w=M,c=K."""
        a = self._cuda(a, torch.uint8)
        # leading dimensions are batches of rows over the same weights (the broadcast rhs of the reference's
        # batched mat_mul, reference/matmul.cpp:57-89): they fold into M
        lead, k = tuple(a.shape[:-1]), a.shape[-1]
        m = int(np.prod(lead))
        w = np.ascontiguousarray(weights_nk).reshape(weights_nk.shape[0], 1, 1, k)
        out = self.conv2d(a.reshape(1, 1, m, k), w, w_zp, mult, bias, a_zp, out_qp, **kw)
        if isinstance(out, tuple):
            return tuple(o.view(*lead, -1) for o in out)
        return out.view(*lead, -1)

    def _cuda(self, t, dtype=None):
        if isinstance(t, np.ndarray):
            t = torch.from_numpy(np.ascontiguousarray(t))
        if dtype is not None and t.dtype != dtype:
            raise NncbError(-22, f"expected {dtype}, got {t.dtype}")
        return t.to(self.device).contiguous()


class Conv2dPlan:
    def __init__(self, ctx, in_shape, weights, w_zp, mult, bias, x_zp, out_qp, stride, padding, dilation, groups,
                 fused_clamp, lut, residual, y2, f32_out, force_path):
        self.ctx = ctx
        n, h, w, c = in_shape
        weights = np.ascontiguousarray(weights)
        if weights.dtype not in (np.uint8, np.int8):
            raise NncbError(-22, "weights must be uint8 or int8")
        oc, kh, kw_, gic = weights.shape
        if gic * groups != c:
            raise NncbError(-22, "weights do not match input channels / groups")
        d = Conv2dDesc()
        d.n, d.h, d.w, d.c = n, h, w, c
        d.oc, d.kh, d.kw = oc, kh, kw_
        d.stride_h, d.stride_w = stride
        d.pad_t, d.pad_b, d.pad_l, d.pad_r = padding
        d.dil_h, d.dil_w = dilation
        d.groups = groups
        d.w_signed = int(weights.dtype == np.int8)
        d.x_zp = int(x_zp)
        d.out_scale, d.out_zp = (out_qp.scale, out_qp.zero_point) if out_qp is not None else (1.0, 0)
        d.clamp_lo, d.clamp_hi = fused_clamp
        if residual is not None:
            rq, aq = residual
            d.has_residual = 1
            d.res_scale, d.res_zp = rq.scale, rq.zero_point
            d.add_out_scale, d.add_out_zp = aq.scale, aq.zero_point
        if y2 is not None:
            yq, lo, hi = y2
            d.has_y2 = 1
            d.y2_scale, d.y2_zp, d.y2_lo, d.y2_hi = yq.scale, yq.zero_point, lo, hi
        d.f32_out = int(f32_out)
        d.force_path = force_path
        self.desc = d
        mult = np.ascontiguousarray(mult, np.float32)
        bias = np.ascontiguousarray(bias, np.float32)
        wz = None if w_zp is None else np.ascontiguousarray(w_zp, np.int32)
        lt = None if lut is None else np.ascontiguousarray(lut, np.uint8)
        h_ = C.c_void_p()
        check(ctx._lib.nncb_qconv2d_create(ctx._h, C.byref(d), weights.ctypes.data,
                                           None if wz is None else wz.ctypes.data, mult.ctypes.data,
                                           bias.ctypes.data, None if lt is None else lt.ctypes.data, C.byref(h_)))
        self._h = h_
        oh, ow = C.c_int(), C.c_int()
        check(ctx._lib.nncb_qconv2d_out_shape(self._h, C.byref(oh), C.byref(ow)))
        self.out_shape = (n, oh.value, ow.value, oc)
        self.path = ctx._lib.nncb_qconv2d_path(self._h)

    def __call__(self, x, res=None, out=None, out2=None):
        ctx, d = self.ctx, self.desc
        if tuple(x.shape) != (d.n, d.h, d.w, d.c) or x.dtype != torch.uint8 or not x.is_contiguous():
            raise NncbError(-22, "conv2d: input does not match the plan")
        y = out if out is not None else torch.empty(self.out_shape, device=ctx.device,
                                                    dtype=torch.float32 if d.f32_out else torch.uint8)
        y2 = None
        if d.has_y2:
            y2 = out2 if out2 is not None else torch.empty(self.out_shape, dtype=torch.uint8, device=ctx.device)
        if d.has_residual and (res is None or tuple(res.shape) != self.out_shape):
            raise NncbError(-22, "conv2d: residual missing or mis-shaped")
        check(ctx._lib.nncb_qconv2d_run(ctx._h, self._h, x.data_ptr(), res.data_ptr() if res is not None else None,
                                        y.data_ptr(), y2.data_ptr() if y2 is not None else None))
        return (y, y2) if d.has_y2 else y

    def close(self):
        if getattr(self, "_h", None):
            self.ctx._lib.nncb_qconv2d_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
