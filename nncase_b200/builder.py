"""Post-training quantization of a float layer graph into a program for the `cuda` module.

This is the host-side stand-in for what the reference does in C# between import and codegen:
  * calibration: run the float graph on the calibration samples and union per-tensor min/max
    over finite values (Quantizer.GetRangesAsync / GetMinMax,
    src/Nncase.Quantization/Quantization/Quantizer.cs:389-409, Quantizer.Algorithms.cs:14-30),
    NoClip (no KLD refinement), then the calibration range fix-up (Quantizer.cs:358-387);
  * QuantParams: activations asymmetric per-tensor u8, weights per output channel
    (QuantUtility.GetQuantParam, Quantizer.cs:620-661), computed by the library's own host code;
  * lowering of each marked Conv2D / MatMul into the integer kernel call with its fused
    epilogue (what a `cuda` ITarget's RegisterQuantizePass would emit).
The float forward used for calibration runs on the library's own float kernels when a CUDA device is given
(`float_forward_cuda`: nncb_conv2d_f32 and friends, ranges reduced by nncb_minmax_f32) and on torch's CPU
operators otherwise (model preparation on a machine without a GPU).
"""
import numpy as np
import torch
import torch.nn.functional as F

from . import kernels as K
from . import lib as L

INF = float("inf")
_ACT_CLAMP = {None: (-INF, INF), "relu": (0.0, INF), "relu6": (0.0, 6.0)}


# ---- float forward (calibration) -----------------------------------------------------------
def float_forward(graph, x, device="cpu", record=None):
    """Runs the float graph on x (torch f32 NCHW). `record(name, tensor)` sees every tensor."""
    t = {}
    rec = record or (lambda n, v: None)
    out = None
    for nd in graph:
        op = nd["op"]
        if op == "input":
            xin = x.to(device)
            if nd.get("layout") == "nhwc":
                xin = xin.permute(0, 3, 1, 2).contiguous()  # the float graph itself runs NCHW
            t[nd["out"]] = xin
            rec(nd["out"], t[nd["out"]])
        elif op == "conv":
            w = torch.from_numpy(nd["w"]).to(device)
            b = torch.from_numpy(nd["b"]).to(device)
            xin = t[nd["in"]]
            pt, pb, pl, pr = nd["pad"]
            if (pt, pl) != (pb, pr):
                xin = F.pad(xin, (pl, pr, pt, pb))
                padding = (0, 0)
            else:
                padding = (pt, pl)
            y = F.conv2d(xin, w, b, nd["stride"], padding, nd["dil"], nd["groups"])
            if nd["act"] == "silu":
                rec(nd["out"] + "@pre", y)
                y = y * torch.sigmoid(y)
            elif nd["act"] is not None:
                lo, hi = _ACT_CLAMP[nd["act"]]
                y = y.clamp(lo, hi)
            if nd.get("res"):
                rec(nd["out"] + "@conv", y)
                y = y + t[nd["res"]]
            t[nd["out"]] = y
            rec(nd["out"], y)
            if nd.get("relu_out"):
                t[nd["relu_out"]] = y.clamp_min(0)
                rec(nd["relu_out"], t[nd["relu_out"]])
        elif op == "maxpool":
            xin = t[nd["in"]]
            pt, pb, pl, pr = nd["pad"]
            # the reference pads max windows with the value 0 (reduce_window.cpp:86-90)
            xin = F.pad(xin, (pl, pr, pt, pb), value=0.0)
            t[nd["out"]] = F.max_pool2d(xin, nd["k"], nd["stride"])
            rec(nd["out"], t[nd["out"]])
        elif op == "relu":
            t[nd["out"]] = t[nd["in"]].clamp_min(0)
            rec(nd["out"], t[nd["out"]])
        elif op == "gap":
            t[nd["out"]] = t[nd["in"]].mean(dim=(2, 3), keepdim=True)
            rec(nd["out"], t[nd["out"]])
        elif op == "fc":
            w = torch.from_numpy(nd["w"]).to(device)
            b = torch.from_numpy(nd["b"]).to(device)
            t[nd["out"]] = t[nd["in"]].flatten(1) @ w.t() + b
            rec(nd["out"], t[nd["out"]])
        elif op == "slice":
            t[nd["out"]] = t[nd["in"]][:, nd["begin"]:nd["end"]]
            rec(nd["out"], t[nd["out"]])
        elif op == "concat":
            t[nd["out"]] = torch.cat([t[i] for i in nd["ins"]], 1)
            rec(nd["out"], t[nd["out"]])
        elif op == "upsample":
            t[nd["out"]] = t[nd["in"]].repeat_interleave(nd["factor"], 2).repeat_interleave(nd["factor"], 3)
            rec(nd["out"], t[nd["out"]])
        elif op == "output":
            return [t[i] for i in nd["ins"]], t
        else:
            raise ValueError(f"unknown node {op}")
        out = nd["out"]
    return t[out], t


class _FloatCuda:
    """The float graph on the library's calibration kernels. Tensors are torch CUDA tensors (device memory and
    views only); every arithmetic operator is a kernel of libnncase_b200.so."""

    def __init__(self, ctx):
        self.ctx, self.lib, self.h = ctx, ctx._lib, ctx._h
        self._weights = {}

    def const(self, arr):
        key = id(arr)
        if key not in self._weights:
            self._weights[key] = torch.from_numpy(np.ascontiguousarray(arr, np.float32)).to(self.ctx.device)
        return self._weights[key]

    def conv(self, x, w, b, stride, pad, dil, groups, lo, hi):
        n, c, h, wd = x.shape
        oc, _, kh, kw = w.shape
        oh = (h + pad[0] + pad[1] - ((kh - 1) * dil[0] + 1)) // stride[0] + 1
        ow = (wd + pad[2] + pad[3] - ((kw - 1) * dil[1] + 1)) // stride[1] + 1
        y = torch.empty((n, oc, oh, ow), dtype=torch.float32, device=x.device)
        L.check(self.lib.nncb_conv2d_f32(self.h, x.data_ptr(), w.data_ptr(), b.data_ptr() if b is not None else None,
                                         y.data_ptr(), n, c, h, wd, oc, kh, kw, stride[0], stride[1], pad[0], pad[1], pad[2],
                                         pad[3], dil[0], dil[1], groups, lo, hi))
        return y

    def clamp(self, x, lo, hi):
        y = torch.empty_like(x)
        L.check(self.lib.nncb_clamp_f32(self.h, x.data_ptr(), y.data_ptr(), x.numel(), lo, hi))
        return y

    def swish(self, x):
        y = torch.empty_like(x)
        L.check(self.lib.nncb_swish_f32(self.h, x.data_ptr(), y.data_ptr(), x.numel()))
        return y

    def add(self, a, b):
        y = torch.empty_like(a)
        L.check(self.lib.nncb_add_f32(self.h, a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel()))
        return y

    def maxpool(self, x, k, stride, pad):
        n, c, h, w = x.shape
        oh = (h + pad[0] + pad[1] - k[0]) // stride[0] + 1
        ow = (w + pad[2] + pad[3] - k[1]) // stride[1] + 1
        y = torch.empty((n, c, oh, ow), dtype=torch.float32, device=x.device)
        L.check(self.lib.nncb_maxpool_f32(self.h, x.data_ptr(), y.data_ptr(), n, c, h, w, k[0], k[1], stride[0], stride[1], *pad))
        return y

    def global_mean(self, x):
        n, c, h, w = x.shape
        y = torch.empty((n, c, 1, 1), dtype=torch.float32, device=x.device)
        L.check(self.lib.nncb_global_mean_f32(self.h, x.data_ptr(), y.data_ptr(), n * c, h * w))
        return y

    def minmax(self, x):
        import ctypes as C
        x = x.contiguous()
        mn, mx = C.c_float(), C.c_float()
        L.check(self.lib.nncb_minmax_f32(self.h, x.data_ptr(), x.numel(), C.byref(mn), C.byref(mx)))
        return mn.value, mx.value


def float_forward_cuda(graph, x, ctx, record=None):
    """float_forward on the library's own kernels (ctx: nncase_b200.kernels.Context). Slice / Concat / nearest
    upsampling are data movement and stay tensor views and copies."""
    k = _FloatCuda(ctx) if not isinstance(ctx, _FloatCuda) else ctx
    ctx = k.ctx
    ctx.use_current_stream()
    t = {}
    rec = record or (lambda n, v: None)
    out = None
    for nd in graph:
        op = nd["op"]
        if op == "input":
            xin = torch.as_tensor(x, dtype=torch.float32).to(ctx.device)
            if nd.get("layout") == "nhwc":
                xin = xin.permute(0, 3, 1, 2)
            t[nd["out"]] = xin.contiguous()
            rec(nd["out"], t[nd["out"]])
        elif op == "conv":
            lo, hi = (-INF, INF) if nd["act"] in (None, "silu") else _ACT_CLAMP[nd["act"]]
            y = k.conv(t[nd["in"]], k.const(nd["w"]), k.const(nd["b"]), nd["stride"], nd["pad"], nd["dil"], nd["groups"], lo, hi)
            if nd["act"] == "silu":
                rec(nd["out"] + "@pre", y)
                y = k.swish(y)
            if nd.get("res"):
                rec(nd["out"] + "@conv", y)
                y = k.add(y, t[nd["res"]])
            t[nd["out"]] = y
            rec(nd["out"], y)
            if nd.get("relu_out"):
                t[nd["relu_out"]] = k.clamp(y, 0.0, INF)
                rec(nd["relu_out"], t[nd["relu_out"]])
        elif op == "maxpool":
            t[nd["out"]] = k.maxpool(t[nd["in"]], nd["k"], nd["stride"], nd["pad"])
            rec(nd["out"], t[nd["out"]])
        elif op == "relu":
            t[nd["out"]] = k.clamp(t[nd["in"]], 0.0, INF)
            rec(nd["out"], t[nd["out"]])
        elif op == "gap":
            t[nd["out"]] = k.global_mean(t[nd["in"]])
            rec(nd["out"], t[nd["out"]])
        elif op == "fc":
            xin = t[nd["in"]].reshape(t[nd["in"]].shape[0], -1, 1, 1).contiguous()
            w = k.const(nd["w"]).reshape(nd["w"].shape[0], -1, 1, 1)
            t[nd["out"]] = k.conv(xin, w, k.const(nd["b"]), (1, 1), (0, 0, 0, 0), (1, 1), 1, -INF, INF).flatten(1)
            rec(nd["out"], t[nd["out"]])
        elif op == "slice":
            t[nd["out"]] = t[nd["in"]][:, nd["begin"]:nd["end"]].contiguous()
            rec(nd["out"], t[nd["out"]])
        elif op == "concat":
            t[nd["out"]] = torch.cat([t[i] for i in nd["ins"]], 1)
            rec(nd["out"], t[nd["out"]])
        elif op == "upsample":
            t[nd["out"]] = t[nd["in"]].repeat_interleave(nd["factor"], 2).repeat_interleave(nd["factor"], 3).contiguous()
            rec(nd["out"], t[nd["out"]])
        elif op == "output":
            return [t[i] for i in nd["ins"]], t
        else:
            raise ValueError(f"unknown node {op}")
        out = nd["out"]
    return t[out], t


def _is_cuda(device):
    return str(device).startswith("cuda")


def calibrate(graph, samples, device="cpu"):
    """Union of per-sample (min, max) over finite values for every tensor of the graph. On a CUDA device the
    forward pass and the range reduction run on the library's kernels."""
    ranges = {}
    if _is_cuda(device):
        dev = torch.device(device)
        k = _FloatCuda(K.Context(dev.index or 0))

        def rec_cuda(name, v):
            mn, mx = k.minmax(v)
            if mn > mx:
                return  # no finite value
            ranges[name] = (min(ranges[name][0], mn), max(ranges[name][1], mx)) if name in ranges else (mn, mx)

        with torch.cuda.device(dev):
            for s in samples:
                float_forward_cuda(graph, s, k, rec_cuda)
        k.ctx.synchronize()
        k.ctx.close()
        return ranges

    def rec(name, v):
        v = v[torch.isfinite(v)]
        if v.numel() == 0:
            return
        mn, mx = float(v.min()), float(v.max())
        if name in ranges:
            ranges[name] = (min(ranges[name][0], mn), max(ranges[name][1], mx))
        else:
            ranges[name] = (mn, mx)

    with torch.no_grad():
        for s in samples:
            float_forward(graph, torch.as_tensor(s, dtype=torch.float32), device, rec)
    return ranges


def calib_fixup_range(mn, mx):
    """Quantizer.FixUpRange, asymmetric branch (Quantizer.cs:358-387)."""
    mn, mx = np.float32(mn), np.float32(mx)
    if mx < 0:
        mx = np.float32(0)
    if mn > 0:
        mn = np.float32(0)
    r = np.float32(mx - mn)
    if r < np.float32(1e-6):
        r = np.float32(0.1)
    return mn, np.float32(mn + r)


def activation_qp(rng):
    mn, mx = calib_fixup_range(*rng)
    return K.get_quant_param(mn, mx, 8, L.UNSIGNED)


def quantize_weights(w_oihw, w_quant_type="uint8", c_pad=None):
    """Per-output-channel weight quantization -> (q OHWI, zero points int32[oc], scales f32[oc]).
    'uint8': asymmetric unsigned; 'int8': symmetric signed (zero points all 0)."""
    oc, ic = w_oihw.shape[:2]
    flat = w_oihw.reshape(oc, -1)
    zps = np.zeros(oc, np.int32)
    scales = np.zeros(oc, np.float32)
    mode = L.UNSIGNED if w_quant_type == "uint8" else L.SIGNED_SYMMETRIC
    for ch in range(oc):
        qp = K.get_quant_param(float(flat[ch].min()), float(flat[ch].max()), 8, mode)
        zps[ch], scales[ch] = qp.zero_point, qp.scale
    lo, hi = (0, 255) if w_quant_type == "uint8" else (-128, 127)
    # q = clamp(rint(w / scale + zp)) in f32: the reference's quantize formula
    q = np.rint(w_oihw / scales[:, None, None, None] + zps[:, None, None, None].astype(np.float32))
    q = np.clip(q, lo, hi).astype(np.uint8 if w_quant_type == "uint8" else np.int8)
    q = np.ascontiguousarray(q.transpose(0, 2, 3, 1))  # OHWI
    if c_pad and c_pad > ic:
        pad = np.empty(q.shape[:3] + (c_pad - ic,), q.dtype)
        pad[...] = zps[:, None, None, None].astype(q.dtype)  # (w - zw) = 0 on padded channels
        q = np.ascontiguousarray(np.concatenate([q, pad], axis=3))
    return q, zps, scales


def space_to_depth_conv(wq_ohwi, zw, pad, in_hw, c_pad=32):
    """Rewrites a stride-2 convolution over few channels as a stride-1 convolution over the
    space-to-depth(2) input [h/2, w/2, c_pad] (channel (dy*2+dx)*c + ch). Every product of the
    original convolution appears exactly once; added taps and channels get the weight zero point
    and contribute (w - zw) = 0. Returns (weights [oc][k2h][k2w][c_pad], pad (t, b, l, r))."""
    oc, kh, kw, c = wq_ohwi.shape
    h, w = in_hw
    assert h % 2 == 0 and w % 2 == 0 and 4 * c <= c_pad

    def dim(k, p_before, p_after, size):
        off = p_before % 2                    # a leading dummy row keeps cells aligned to even rows
        k2 = (k + off + 1) // 2
        out = (size + p_before + p_after - k) // 2 + 1
        pb = (p_before + off) // 2
        pa = out - 1 + k2 - size // 2 - pb
        assert pa >= 0
        return off, k2, pb, pa

    offy, k2h, pt, pb = dim(kh, pad[0], pad[1], h)
    offx, k2w, pl, pr = dim(kw, pad[2], pad[3], w)
    new = np.empty((oc, k2h, k2w, c_pad), wq_ohwi.dtype)
    new[...] = np.asarray(zw).reshape(oc, 1, 1, 1).astype(wq_ohwi.dtype)
    for ky in range(kh):
        ty, dy = divmod(ky + offy, 2)
        for kx in range(kw):
            tx, dx = divmod(kx + offx, 2)
            new[:, ty, tx, (dy * 2 + dx) * c:(dy * 2 + dx) * c + c] = wq_ohwi[:, ky, kx, :]
    return np.ascontiguousarray(new), (pt, pb, pl, pr)


def _pad_channels(c):
    """Channel counts the tensor-core kernel accepts need no padding; tiny ones pad to 4."""
    return 4 if c < 4 else c


def build_program(graph, calib_samples, w_quant_type="uint8", device="cpu"):
    """Calibrate and lower `graph` into a quantized program (a dict, see nncase_b200.runtime)."""
    ranges = calibrate(graph, calib_samples, device)
    qps = {name: activation_qp(r) for name, r in ranges.items()}
    tensors, ops = {}, []
    shapes = {}

    def add_tensor(name, c, h, w, qp, dtype="u8"):
        tensors[name] = dict(shape=(h, w, c), qp=qp, dtype=dtype)
        shapes[name] = (c, h, w)

    out_name, outputs = None, None
    # Tensors between layers are stored with their channel count rounded up to the tensor-core
    # kernel's K granule (32); added channels carry weight zero points / zero multipliers and
    # contribute nothing. Program outputs keep their own channel count.
    final = set(graph[-1]["ins"]) if graph[-1]["op"] == "output" else {graph[-1]["out"]}
    logical = {}
    for nd in graph:
        op = nd["op"]
        if op == "input":
            c, h, w = nd["shape"]
            users = [u for u in graph if u.get("in") == nd["out"] or u.get("res") == nd["out"] or
                     nd["out"] in u.get("ins", ())]
            nhwc = nd.get("layout") == "nhwc"
            s2d = (len(users) == 1 and users[0]["op"] == "conv" and tuple(users[0]["stride"]) == (2, 2) and
                   users[0]["groups"] == 1 and tuple(users[0]["dil"]) == (1, 1) and c <= 8 and h % 2 == 0 and
                   w % 2 == 0)
            if s2d:
                # image stem: quantize straight into the space-to-depth layout (see space_to_depth_conv).
                # With 16-byte cells and the padding written as zero-point cells, the stem is an unpadded
                # stride-1 convolution whose kernel rows are contiguous bytes (the kernel's row mode).
                cp = 16 if 4 * c <= 16 else 32
                _, pad2 = space_to_depth_conv(np.zeros((1,) + tuple(users[0]["w"].shape[2:]) + (c,), np.uint8), [0],
                                              users[0]["pad"], (h, w), cp)
                k2w = (users[0]["w"].shape[3] + users[0]["pad"][2] % 2 + 1) // 2
                pre_pad = pad2 if k2w * cp in (32, 64, 128) else (0, 0, 0, 0)
                add_tensor(nd["out"], cp, h // 2 + pre_pad[0] + pre_pad[1], w // 2 + pre_pad[2] + pre_pad[3],
                           qps[nd["out"]])
                ops.append(dict(op="quantize_input", out=nd["out"], c=c, c_pad=cp, s2d=True, nhwc=nhwc, pad=pre_pad))
                s2d_of = {nd["out"]: (c, h, w, pre_pad)}
            else:
                cp = _pad_channels(c)
                add_tensor(nd["out"], cp, h, w, qps[nd["out"]])
                ops.append(dict(op="quantize_input", out=nd["out"], c=c, c_pad=cp, nhwc=nhwc))
                s2d_of = {}
            in_name = nd["out"]
        elif op == "conv":
            c, h, w = shapes[nd["in"]]
            stride, pad = nd["stride"], nd["pad"]
            if nd["in"] in s2d_of:
                c0, h0, w0, pre_pad = s2d_of[nd["in"]]
                wq, zw, sw = quantize_weights(nd["w"], w_quant_type)
                wq, pad = space_to_depth_conv(wq, zw, pad, (h0, w0), c)
                if any(pre_pad):
                    assert tuple(pad) == tuple(pre_pad)
                    pad = (0, 0, 0, 0)  # already in the data
                stride = (1, 1)
            else:
                wq, zw, sw = quantize_weights(nd["w"], w_quant_type, c if nd["groups"] == 1 else None)
            bias = nd["b"].astype(np.float32)
            groups = nd["groups"]
            logical[nd["out"]] = wq.shape[0]
            oc_p = wq.shape[0]
            if groups != 1:
                if groups != wq.shape[0] or wq.shape[3] != 1:
                    raise ValueError("grouped convolutions other than depthwise are not lowered")
                oc_p = groups = c  # depthwise over the stored (padded) channels
            elif nd["out"] not in final and nd.get("relu_out") not in final:
                oc_p = -(-wq.shape[0] // 32) * 32
            extra = oc_p - wq.shape[0]
            if extra:
                wq = np.ascontiguousarray(np.concatenate([wq, np.zeros((extra,) + wq.shape[1:], wq.dtype)]))
                zw = np.concatenate([zw, np.zeros(extra, np.int32)])
                sw = np.concatenate([sw, np.zeros(extra, np.float32)])  # multiplier 0: the channel holds q(0)
                bias = np.concatenate([bias, np.zeros(extra, np.float32)])
            oc, kh, kw, _ = wq.shape
            oh = (h + pad[0] + pad[1] - ((kh - 1) * nd["dil"][0] + 1)) // stride[0] + 1
            ow = (w + pad[2] + pad[3] - ((kw - 1) * nd["dil"][1] + 1)) // stride[1] + 1
            xqp = tensors[nd["in"]]["qp"]
            mult = (np.float32(xqp.scale) * sw).astype(np.float32)
            has_res = bool(nd.get("res"))
            silu = nd["act"] == "silu"
            lut = None
            if silu:
                # conv output quantized with the pre-activation range, then SiLU as a table into the
                # activation's own quant param (quantize -> swish on the dequantized value -> quantize)
                conv_qp = qps[nd["out"] + "@pre"]
                act_qp = qps[nd["out"] + "@conv"] if has_res else qps[nd["out"]]
                lut = K.activation_table(L.ACT_SWISH, conv_qp, act_qp)
                clamp = (-INF, INF)
            else:
                conv_qp = qps[nd["out"] + "@conv"] if has_res else qps[nd["out"]]
                clamp = _ACT_CLAMP[nd["act"]]
            fuse_res = has_res and not silu  # a table and a fused add do not combine: emit a separate add
            conv_out = nd["out"] if (fuse_res or not has_res) else nd["out"] + "@conv"
            o = dict(op="conv", name=nd["name"], **{"in": nd["in"]}, out=conv_out, w=wq,
                     w_zp=zw if zw.any() else None, mult=mult, bias=bias, stride=tuple(stride),
                     pad=tuple(pad), dil=nd["dil"], groups=groups, clamp=clamp,
                     res=nd.get("res") if fuse_res else None, y2=nd.get("relu_out"), conv_qp=conv_qp, lut=lut,
                     w_scale=sw)
            ops.append(o)
            if has_res and not fuse_res:
                add_tensor(conv_out, oc, oh, ow, qps[nd["out"] + "@conv"])
                ops.append(dict(op="add", a=conv_out, b=nd["res"], out=nd["out"]))
            add_tensor(nd["out"], oc, oh, ow, qps[nd["out"]])
            if nd.get("relu_out"):
                add_tensor(nd["relu_out"], oc, oh, ow, qps[nd["relu_out"]])
        elif op == "maxpool":
            c, h, w = shapes[nd["in"]]
            oh = (h + nd["pad"][0] + nd["pad"][1] - nd["k"][0]) // nd["stride"][0] + 1
            ow = (w + nd["pad"][2] + nd["pad"][3] - nd["k"][1]) // nd["stride"][1] + 1
            add_tensor(nd["out"], c, oh, ow, tensors[nd["in"]]["qp"])  # max keeps the input's quant param
            ops.append(dict(op="maxpool", **{"in": nd["in"]}, out=nd["out"], k=nd["k"], stride=nd["stride"],
                            pad=nd["pad"]))
        elif op == "relu":
            c, h, w = shapes[nd["in"]]
            add_tensor(nd["out"], c, h, w, qps[nd["out"]])
            ops.append(dict(op="requant", **{"in": nd["in"]}, out=nd["out"], clamp=(0.0, INF)))
        elif op == "gap":
            c, h, w = shapes[nd["in"]]
            add_tensor(nd["out"], c, 1, 1, qps[nd["out"]])
            ops.append(dict(op="gap", **{"in": nd["in"]}, out=nd["out"]))
        elif op == "fc":
            c, h, w = shapes[nd["in"]]
            wq, zw, sw = quantize_weights(nd["w"].reshape(nd["w"].shape[0], -1, 1, 1), w_quant_type, c)
            xqp = tensors[nd["in"]]["qp"]
            mult = (np.float32(xqp.scale) * sw).astype(np.float32)
            add_tensor(nd["out"], wq.shape[0], 1, 1, None, "f32")
            ops.append(dict(op="conv", name=nd["name"], **{"in": nd["in"]}, out=nd["out"], w=wq,
                            w_zp=zw if zw.any() else None, mult=mult, bias=nd["b"].astype(np.float32), stride=(1, 1),
                            pad=(0, 0, 0, 0), dil=(1, 1), groups=1, clamp=(-INF, INF), res=None, y2=None,
                            conv_qp=None, f32_out=True, w_scale=sw))
        elif op == "slice":
            c, h, w = shapes[nd["in"]]
            if logical.get(nd["in"], c) != c:
                raise ValueError("slice of a channel-padded tensor is not lowered")
            add_tensor(nd["out"], nd["end"] - nd["begin"], h, w, tensors[nd["in"]]["qp"])  # same quant param
            ops.append(dict(op="slice", **{"in": nd["in"]}, out=nd["out"], begin=nd["begin"], end=nd["end"]))
        elif op == "concat":
            c0, h, w = shapes[nd["ins"][0]]
            if any(logical.get(i, shapes[i][0]) != shapes[i][0] for i in nd["ins"]):
                raise ValueError("concat of channel-padded tensors is not lowered")
            add_tensor(nd["out"], sum(shapes[i][0] for i in nd["ins"]), h, w, qps[nd["out"]])
            ops.append(dict(op="concat", ins=list(nd["ins"]), out=nd["out"]))
        elif op == "upsample":
            c, h, w = shapes[nd["in"]]
            add_tensor(nd["out"], c, h * nd["factor"], w * nd["factor"], tensors[nd["in"]]["qp"])
            ops.append(dict(op="upsample", **{"in": nd["in"]}, out=nd["out"], factor=nd["factor"]))
        elif op == "output":
            outputs = list(nd["ins"])
            continue
        else:
            raise ValueError(f"unknown node {op}")
        out_name = nd["out"]
    return dict(input=in_name, output=out_name, outputs=outputs or [out_name], tensors=tensors, ops=ops, ranges=ranges)
