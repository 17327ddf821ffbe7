"""Executes a quantized program op by op with the C oracle (CPU). TEST INFRASTRUCTURE ONLY.

Every fused kernel of the CUDA module is replayed here as its unfused sequence
(conv -> [table] -> [binary add] -> [relu requant]) so that fusion cannot change results.
Optionally feeds each op the CUDA path's own inputs (`feed`) to check layers in isolation.
"""
import numpy as np

from . import qoracle as Q

INF = float("inf")


def run_program(program, x_nchw_f32, threads=8, feed=None, keep=None):
    """Returns (output, tensors). feed: {tensor name: ndarray} replaces computed inputs."""
    Q.lib().qo_set_threads(threads)
    T = program["tensors"]
    t = {}

    def get(name):
        if feed is not None and name in feed:
            return feed[name]
        return t[name]

    for op in program["ops"]:
        k = op["op"]
        if k == "quantize_input":
            qp = T[op["out"]]["qp"]
            xin = x_nchw_f32
            if op.get("nhwc"):  # element-wise identical: bring the NHWC input to the NCHW form the helpers take
                xin = np.ascontiguousarray(np.transpose(x_nchw_f32, (0, 3, 1, 2)))
            if op.get("s2d"):
                t[op["out"]] = Q.quantize_nchw_to_s2d_u8(xin, qp.scale, qp.zero_point, op["c_pad"],
                                                         op.get("pad", (0, 0, 0, 0)))
            else:
                t[op["out"]] = Q.quantize_nchw_to_nhwc_u8(xin, qp.scale, qp.zero_point, op["c_pad"])
        elif k == "conv":
            xin = get(op["in"])
            xqp = T[op["in"]]["qp"]
            if op.get("f32_out"):
                t[op["out"]] = Q.qconv2d_u8(xin, op["w"], op["w_zp"], op["mult"], op["bias"], xqp.zero_point, 1.0, 0,
                                            op["stride"], op["pad"], op["dil"], op["groups"], op["clamp"],
                                            f32_out=True)
                continue
            cq = op["conv_qp"]
            y = Q.qconv2d_u8(xin, op["w"], op["w_zp"], op["mult"], op["bias"], xqp.zero_point, cq.scale,
                             cq.zero_point, op["stride"], op["pad"], op["dil"], op["groups"], op["clamp"],
                             lut=op.get("lut"))
            if op.get("res"):
                rq, oq = T[op["res"]]["qp"], T[op["out"]]["qp"]
                y = Q.qadd_u8(y, get(op["res"]), cq.scale, cq.zero_point, rq.scale, rq.zero_point, oq.scale,
                              oq.zero_point)
            t[op["out"]] = y
            if op.get("y2"):
                oq, yq = T[op["out"]]["qp"], T[op["y2"]]["qp"]
                t[op["y2"]] = Q.requant_u8(y, oq.scale, oq.zero_point, yq.scale, yq.zero_point, 0.0, INF)
        elif k == "maxpool":
            t[op["out"]] = Q.maxpool_u8(get(op["in"]), op["k"], op["stride"], op["pad"], T[op["in"]]["qp"].zero_point)
        elif k == "requant":
            qi, qo = T[op["in"]]["qp"], T[op["out"]]["qp"]
            t[op["out"]] = Q.requant_u8(get(op["in"]), qi.scale, qi.zero_point, qo.scale, qo.zero_point, *op["clamp"])
        elif k == "add":
            qa, qb, qo = T[op["a"]]["qp"], T[op["b"]]["qp"], T[op["out"]]["qp"]
            t[op["out"]] = Q.qadd_u8(get(op["a"]), get(op["b"]), qa.scale, qa.zero_point, qb.scale, qb.zero_point,
                                     qo.scale, qo.zero_point)
        elif k == "slice":
            t[op["out"]] = np.ascontiguousarray(get(op["in"])[..., op["begin"]:op["end"]])
        elif k == "concat":
            oq = T[op["out"]]["qp"]
            parts = []
            for name in op["ins"]:
                iq = T[name]["qp"]
                parts.append(Q.requant_u8(get(name), iq.scale, iq.zero_point, oq.scale, oq.zero_point))
            t[op["out"]] = np.ascontiguousarray(np.concatenate(parts, axis=-1))
        elif k == "upsample":
            t[op["out"]] = Q.resize_nearest_u8(get(op["in"]), op["factor"], op["factor"])
        elif k == "gap":
            qi, qo = T[op["in"]]["qp"], T[op["out"]]["qp"]
            t[op["out"]] = Q.global_avgpool_u8(get(op["in"]), qi.scale, qi.zero_point, qo.scale, qo.zero_point)
        else:
            raise ValueError(k)
    return t[program["output"]], t
