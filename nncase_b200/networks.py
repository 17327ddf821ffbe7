"""Float layer graphs of the benchmark networks with seeded random weights.

These stand in for the ONNX/TFLite models the reference imports (its importers and compiler
front end are out of scope); shapes follow the configurations the metric is quoted on. BatchNorm
is folded: every convolution carries a bias, and the pre-activation BatchNorm of ResNet v2 is
the identity for freshly initialised statistics, which leaves its ReLU.

A graph is a list of nodes (dicts). Tensors are named by strings. Node kinds:
  input    {out, shape=(c,h,w)}
  conv     {in, out, w (OIHW f32), b, stride, pad=(t,b,l,r), dil, groups, act: None|"relu"|"relu6",
            res: tensor added after the activation or None, relu_out: name of an extra output
            relu(out) or None}
  maxpool  {in, out, k, stride, pad}
  relu     {in, out}
  gap      {in, out}                      global mean over H x W
  fc       {in, out, w ([N,K] f32), b}    MatMul + bias, f32 logits
The composite conv node (activation, residual add and a second ReLU output in one node) is the
unit the `cuda` module executes as one kernel; unfused it is conv -> clamp -> binary add -> relu.
"""
import numpy as np


def _he_conv(rng, oc, ic, kh, kw):
    fan_in = ic * kh * kw
    return rng.normal(0.0, np.sqrt(2.0 / fan_in), (oc, ic, kh, kw)).astype(np.float32)


def _bias(rng, oc):
    return rng.normal(0.0, 0.01, oc).astype(np.float32)


def single_conv(seed=1001, c=64, oc=64, hw=56):
    """Config "single quantized Conv2D": [1,64,56,56] x [64,64,3,3], stride 1, pad 1, fused ReLU6;
    weights N(0, 0.05), bias N(0, 0.01)."""
    rng = np.random.default_rng(seed)
    w = rng.normal(0, 0.05, (oc, c, 3, 3)).astype(np.float32)
    b = rng.normal(0, 0.01, oc).astype(np.float32)
    return [
        dict(op="input", out="x", shape=(c, hw, hw)),
        dict(op="conv", name="conv", **{"in": "x"}, out="y", w=w, b=b, stride=(1, 1), pad=(1, 1, 1, 1), dil=(1, 1),
             groups=1, act="relu6", res=None, relu_out=None),
    ]


def resnet50v2(seed=1003, num_classes=1000, stages=(3, 4, 6, 3), widths=(64, 128, 256, 512), image=224,
               stem_channels=64):
    """ResNet-50 v2 (pre-activation bottlenecks [3,4,6,3], NCHW input [N,3,224,224], 1000-way FC).
    Stride sits on the 3x3 convolution; the first block of a stage projects its shortcut from
    the pre-activated input with a strided 1x1 convolution."""
    rng = np.random.default_rng(seed)
    g = [dict(op="input", out="input", shape=(3, image, image))]

    def conv(name, src, dst, oc, ic, k, stride, pad, act, res=None, relu_out=None):
        g.append(dict(op="conv", name=name, **{"in": src}, out=dst, w=_he_conv(rng, oc, ic, k, k), b=_bias(rng, oc),
                      stride=(stride, stride), pad=(pad, pad, pad, pad), dil=(1, 1), groups=1, act=act, res=res,
                      relu_out=relu_out))

    conv("stem", "input", "stem", stem_channels, 3, 7, 2, 3, "relu")
    g.append(dict(op="maxpool", **{"in": "stem"}, out="pool", k=(3, 3), stride=(2, 2), pad=(1, 1, 1, 1)))
    g.append(dict(op="relu", **{"in": "pool"}, out="pool_act"))
    x, xa, cin = "pool", "pool_act", stem_channels  # block input and its pre-activation
    for si, (blocks, width) in enumerate(zip(stages, widths)):
        for bi in range(blocks):
            p = f"s{si + 1}b{bi + 1}"
            stride = 2 if (bi == 0 and si > 0) else 1
            cout = width * 4
            if bi == 0:
                conv(p + "_sc", xa, p + "_sc", cout, cin, 1, stride, 0, None)
                shortcut = p + "_sc"
            else:
                shortcut = x
            conv(p + "_c1", xa, p + "_c1", width, cin, 1, 1, 0, "relu")
            conv(p + "_c2", p + "_c1", p + "_c2", width, width, 3, stride, 1, "relu")
            conv(p + "_c3", p + "_c2", p + "_out", cout, width, 1, 1, 0, None, res=shortcut, relu_out=p + "_act")
            x, xa, cin = p + "_out", p + "_act", cout
    g.append(dict(op="gap", **{"in": xa}, out="gap"))
    wfc = rng.normal(0.0, np.sqrt(2.0 / cin), (num_classes, cin)).astype(np.float32)
    g.append(dict(op="fc", name="fc", **{"in": "gap"}, out="logits", w=wfc, b=_bias(rng, num_classes)))
    return g


def graph_macs(graph):
    """Multiply-accumulates per image (padding taps counted, as a dense GEMM does)."""
    shapes, total, per_layer = {}, 0, []
    for nd in graph:
        if nd["op"] == "input":
            shapes[nd["out"]] = nd["shape"]
        elif nd["op"] == "conv":
            c, h, w = shapes[nd["in"]]
            oc, gic, kh, kw = nd["w"].shape
            oh = (h + nd["pad"][0] + nd["pad"][1] - ((kh - 1) * nd["dil"][0] + 1)) // nd["stride"][0] + 1
            ow = (w + nd["pad"][2] + nd["pad"][3] - ((kw - 1) * nd["dil"][1] + 1)) // nd["stride"][1] + 1
            shapes[nd["out"]] = (oc, oh, ow)
            if nd.get("relu_out"):
                shapes[nd["relu_out"]] = (oc, oh, ow)
            m = oc * oh * ow * gic * kh * kw
            per_layer.append((nd["name"], m))
            total += m
        elif nd["op"] == "maxpool":
            c, h, w = shapes[nd["in"]]
            oh = (h + nd["pad"][0] + nd["pad"][1] - nd["k"][0]) // nd["stride"][0] + 1
            ow = (w + nd["pad"][2] + nd["pad"][3] - nd["k"][1]) // nd["stride"][1] + 1
            shapes[nd["out"]] = (c, oh, ow)
        elif nd["op"] == "relu":
            shapes[nd["out"]] = shapes[nd["in"]]
        elif nd["op"] == "gap":
            shapes[nd["out"]] = (shapes[nd["in"]][0], 1, 1)
        elif nd["op"] == "fc":
            m = nd["w"].shape[0] * nd["w"].shape[1]
            per_layer.append((nd["name"], m))
            total += m
            shapes[nd["out"]] = (nd["w"].shape[0], 1, 1)
    return total, per_layer, shapes
