"""Executes a quantized program with the REFERENCE's own CPU kernels (oracle/_ref). TEST INFRASTRUCTURE ONLY.

This is how the reference's cpu target runs a quantized graph: every quantized operator is
dequantize -> the float kernel -> quantize (src/Nncase.Importer/Onnx/QLinearConv.cs:61-75 for
convolutions, src/Nncase.Importer/Onnx/QLinearMatmul.cs:25-28 for MatMul; binary add, clamp, swish,
reduce_window2d run between a dequantize and a quantize in the same way). All arithmetic below goes
through kernels::stackvm::{dequantize, conv2d, quantize, binary, reduce_window2d, relu, swish}
compiled from the reference's sources; only data movement (layout changes, Slice, Concat's copy,
nearest-neighbour resize) is numpy.

Two uses:
  * `layer_gate`  -- every convolution of a program fed the integer oracle's own u8 input, compared
    with the integer formulation (differences come only from the reference's f32 accumulation order);
  * `run_program` -- the whole program free-running on the reference's kernels (each layer fed the
    reference's own output), the CPU baseline of the benchmark and the end-to-end mismatch figure.
"""
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from . import qoracle as Q
from . import ref as R

INF = float("inf")


def _nchw(q):
    return np.ascontiguousarray(q.transpose(0, 3, 1, 2))


def _nhwc(q):
    return np.ascontiguousarray(q.transpose(0, 2, 3, 1))


def conv_composite(op, xq, xqp, threads=1, pool=None):
    """One convolution op of a program through dequantize -> conv2d(f32, fused clamp) [-> quantize].
    Output channels are independent in the reference's loop nest, so the call is split over
    `threads` slices of them (identical results, the kernel itself is single-threaded)."""
    w, wz = op["w"], op["w_zp"]
    oc = w.shape[0]
    sw = op.get("w_scale")
    if sw is None:
        sw = (op["mult"] / np.float32(xqp.scale)).astype(np.float32)
    groups = op["groups"]
    f32_out = bool(op.get("f32_out"))
    cq = op.get("conv_qp")
    xf = R.dequantize_u8(_nchw(xq), xqp.scale, xqp.zero_point)

    def part(lo, hi):
        wq = np.ascontiguousarray(w[lo:hi].transpose(0, 3, 1, 2))
        wf = np.empty(wq.shape, np.float32)
        for ch in range(hi - lo):
            z = 0 if wz is None else int(wz[lo + ch])
            s = float(sw[lo + ch])
            if s == 0.0:           # a channel added by the builder for alignment: multiplier 0
                wf[ch] = 0.0
            elif wq.dtype == np.uint8:
                wf[ch] = R.dequantize_u8(wq[ch], s, z)
            else:
                wf[ch] = R.dequantize_i8(wq[ch], s, z)
        if groups == 1:
            xin, g = xf, 1
        else:                      # depthwise: channel ch reads input channel ch
            xin, g = np.ascontiguousarray(xf[:, lo:hi]), hi - lo
        yf = R.conv2d_f32(xin, wf, op["bias"][lo:hi], op["stride"], op["pad"], op["dil"], g, op["clamp"])
        return yf if f32_out else R.quantize_u8(yf, cq.scale, cq.zero_point)

    n_parts = max(1, min(threads, oc // 8 if oc >= 8 else 1))
    bounds = np.linspace(0, oc, n_parts + 1).astype(int)
    jobs = [(int(bounds[i]), int(bounds[i + 1])) for i in range(n_parts) if bounds[i + 1] > bounds[i]]
    if pool is not None and len(jobs) > 1:
        parts = list(pool.map(lambda j: part(*j), jobs))
    else:
        parts = [part(*j) for j in jobs]
    return _nhwc(np.concatenate(parts, axis=1))


def _requant(q, qi, qo, fn=None):
    f = R.dequantize_u8(q, qi.scale, qi.zero_point)
    if fn is not None:
        f = fn(f)
    return R.quantize_u8(f, qo.scale, qo.zero_point)


def run_program(program, x_f32, threads=8):
    """Free-running execution on the reference's kernels. Returns (output, tensors)."""
    T = program["tensors"]
    t = {}
    with ThreadPoolExecutor(threads) as pool:
        for op in program["ops"]:
            k = op["op"]
            if k == "quantize_input":
                # Quantize itself is bit-identical between the reference and the integer oracle (pinned by
                # tests/test_oracle_vs_reference.py); the oracle's helper also lays the result out.
                qp = T[op["out"]]["qp"]
                xin = np.ascontiguousarray(np.transpose(x_f32, (0, 3, 1, 2))) if op.get("nhwc") else x_f32
                if op.get("s2d"):
                    t[op["out"]] = Q.quantize_nchw_to_s2d_u8(xin, qp.scale, qp.zero_point, op["c_pad"],
                                                             op.get("pad", (0, 0, 0, 0)))
                else:
                    t[op["out"]] = Q.quantize_nchw_to_nhwc_u8(xin, qp.scale, qp.zero_point, op["c_pad"])
            elif k == "conv":
                xqp = T[op["in"]]["qp"]
                y = conv_composite(op, t[op["in"]], xqp, threads, pool)
                if op.get("f32_out"):
                    t[op["out"]] = y
                    continue
                cq = op["conv_qp"]
                if op.get("lut") is not None:  # swish between the convolution's and the activation's quant params
                    aq = T[op["out"]]["qp"]
                    y = _requant(y, cq, aq, lambda f: R.unary_f32(2, f))
                if op.get("res"):
                    rq, oq = T[op["res"]]["qp"], T[op["out"]]["qp"]
                    s = R.add_f32(R.dequantize_u8(y, cq.scale, cq.zero_point),
                                  R.dequantize_u8(t[op["res"]], rq.scale, rq.zero_point))
                    y = R.quantize_u8(s, oq.scale, oq.zero_point)
                t[op["out"]] = y
                if op.get("y2"):
                    t[op["y2"]] = _requant(y, T[op["out"]]["qp"], T[op["y2"]]["qp"], lambda f: R.unary_f32(0, f))
            elif k == "maxpool":
                qp = T[op["in"]]["qp"]
                f = R.dequantize_u8(_nchw(t[op["in"]]), qp.scale, qp.zero_point)
                f = R.reduce_window2d_f32("max", f, op["k"], op["stride"], op["pad"],
                                          init=float(np.finfo(np.float32).min))
                t[op["out"]] = _nhwc(R.quantize_u8(f, qp.scale, qp.zero_point))
            elif k == "requant":
                lo, hi = op["clamp"]
                t[op["out"]] = _requant(t[op["in"]], T[op["in"]]["qp"], T[op["out"]]["qp"],
                                        lambda f: np.clip(f, lo, hi))
            elif k == "add":
                qa, qb, qo = T[op["a"]]["qp"], T[op["b"]]["qp"], T[op["out"]]["qp"]
                s = R.add_f32(R.dequantize_u8(t[op["a"]], qa.scale, qa.zero_point),
                              R.dequantize_u8(t[op["b"]], qb.scale, qb.zero_point))
                t[op["out"]] = R.quantize_u8(s, qo.scale, qo.zero_point)
            elif k == "slice":
                t[op["out"]] = np.ascontiguousarray(t[op["in"]][..., op["begin"]:op["end"]])
            elif k == "concat":
                oq = T[op["out"]]["qp"]
                t[op["out"]] = np.ascontiguousarray(
                    np.concatenate([_requant(t[n_], T[n_]["qp"], oq) for n_ in op["ins"]], axis=-1))
            elif k == "upsample":
                t[op["out"]] = Q.resize_nearest_u8(t[op["in"]], op["factor"], op["factor"])
            elif k == "gap":
                qi, qo = T[op["in"]]["qp"], T[op["out"]]["qp"]
                f = R.dequantize_u8(_nchw(t[op["in"]]), qi.scale, qi.zero_point)
                hh, ww = f.shape[2:]
                f = R.reduce_window2d_f32("mean", f, (hh, ww), (1, 1), (0, 0, 0, 0), init=0.0)
                t[op["out"]] = _nhwc(R.quantize_u8(f, qo.scale, qo.zero_point))
            else:
                raise ValueError(k)
    return t[program["output"]], t


def layer_gate(program, oracle_tensors, threads=8):
    """Every convolution of `program`, fed the integer oracle's own input tensor, through the reference
    composite and through the integer formulation. Returns rows
    (layer, K, outputs, mismatches, max |delta|); the f32-output MatMul reports max |delta| relative to
    the output range instead of LSBs."""
    T = program["tensors"]
    rows = []
    with ThreadPoolExecutor(threads) as pool:
        for op in program["ops"]:
            if op["op"] != "conv":
                continue
            xq, xqp = oracle_tensors[op["in"]], T[op["in"]]["qp"]
            want = conv_composite(op, xq, xqp, threads, pool)
            kdim = int(np.prod(op["w"].shape[1:]))
            if op.get("f32_out"):
                got = Q.qconv2d_u8(xq, op["w"], op["w_zp"], op["mult"], op["bias"], xqp.zero_point, 1.0, 0,
                                   op["stride"], op["pad"], op["dil"], op["groups"], op["clamp"], f32_out=True)
                rng = float(want.max() - want.min()) or 1.0
                rows.append((op["name"], kdim, want.size, 0, float(np.abs(got - want).max() / rng)))
                continue
            cq = op["conv_qp"]
            got = Q.qconv2d_u8(xq, op["w"], op["w_zp"], op["mult"], op["bias"], xqp.zero_point, cq.scale,
                               cq.zero_point, op["stride"], op["pad"], op["dil"], op["groups"], op["clamp"])
            d = np.abs(got.astype(np.int32) - want.astype(np.int32))
            rows.append((op["name"], kdim, want.size, int((d != 0).sum()), int(d.max())))
    return rows
