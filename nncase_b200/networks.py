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
  slice    {in, out, begin, end}          channel range;  concat {ins, out} on channels
  upsample {in, out, factor}              nearest neighbour;  output {ins} several graph outputs
  conv.act also takes "silu" (the reference's swish); input.layout "nhwc" for NHWC f32 inputs
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


def mobilenetv2(seed=1002, num_classes=1000, image=224, width=1.0):
    """MobileNetV2-1.0: NHWC f32 input [N,224,224,3]; inverted residuals (expand 1x1 + ReLU6, depthwise
    3x3 + ReLU6, linear 1x1 projection, residual add when stride 1 and channels match), 1280-wide last
    convolution, global mean, 1000-way FC."""
    rng = np.random.default_rng(seed)
    g = [dict(op="input", out="input", shape=(3, image, image), layout="nhwc")]

    def conv(name, src, dst, oc, ic, k, stride, act, groups=1, res=None):
        pad = k // 2
        g.append(dict(op="conv", name=name, **{"in": src}, out=dst, w=_he_conv(rng, oc, ic // groups, k, k),
                      b=_bias(rng, oc), stride=(stride, stride), pad=(pad, pad, pad, pad), dil=(1, 1), groups=groups,
                      act=act, res=res, relu_out=None))

    def c8(v):
        return max(8, int(v * width + 4) // 8 * 8)

    cin = c8(32)
    conv("stem", "input", "stem", cin, 3, 3, 2, "relu6")
    x = "stem"
    bi = 0
    for t, c, n, s in [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2),
                       (6, 320, 1, 1)]:
        cout = c8(c)
        for i in range(n):
            bi += 1
            p, stride, hid = f"b{bi}", (s if i == 0 else 1), cin * t
            y = x
            if t != 1:
                conv(p + "_exp", x, p + "_exp", hid, cin, 1, 1, "relu6")
                y = p + "_exp"
            conv(p + "_dw", y, p + "_dw", hid, hid, 3, stride, "relu6", groups=hid)
            conv(p + "_proj", p + "_dw", p + "_out", cout, hid, 1, 1, None,
                 res=x if (stride == 1 and cin == cout) else None)
            x, cin = p + "_out", cout
    conv("last", x, "last", 1280, cin, 1, 1, "relu6")
    g.append(dict(op="gap", **{"in": "last"}, out="gap"))
    wfc = rng.normal(0.0, np.sqrt(2.0 / 1280), (num_classes, 1280)).astype(np.float32)
    g.append(dict(op="fc", name="fc", **{"in": "gap"}, out="logits", w=wfc, b=_bias(rng, num_classes)))
    return g


def yolov8s(seed=1004, image=640, classes=80, width=(32, 64, 128, 256, 512)):
    """YOLOv8s detector: CSPDarknet backbone with C2f blocks, SPPF, PAN neck, decoupled head (box 4x16,
    class `classes`) on three scales; every Conv is convolution + folded BN + SiLU. NCHW f32 input
    [N,3,640,640]. Outputs: per scale the box and the class maps (raw, before any decoding)."""
    rng = np.random.default_rng(seed)
    g = [dict(op="input", out="input", shape=(3, image, image))]
    c1, c2, c3, c4, c5 = width

    def conv(name, src, oc, ic, k=1, stride=1, act="silu", res=None):
        pad = k // 2
        g.append(dict(op="conv", name=name, **{"in": src}, out=name, w=_he_conv(rng, oc, ic, k, k), b=_bias(rng, oc),
                      stride=(stride, stride), pad=(pad, pad, pad, pad), dil=(1, 1), groups=1, act=act, res=res,
                      relu_out=None))
        return name

    def c2f(name, src, cin, cout, n, shortcut):
        c = cout // 2
        y = conv(name + "_cv1", src, 2 * c, cin)
        g.append(dict(op="slice", **{"in": y}, out=name + "_y0", begin=0, end=c))
        g.append(dict(op="slice", **{"in": y}, out=name + "_y1", begin=c, end=2 * c))
        parts, cur = [name + "_y0", name + "_y1"], name + "_y1"
        for i in range(n):
            a = conv(f"{name}_m{i}a", cur, c, c, 3)
            cur = conv(f"{name}_m{i}b", a, c, c, 3, res=cur if shortcut else None)
            parts.append(cur)
        g.append(dict(op="concat", ins=parts, out=name + "_cat"))
        return conv(name + "_cv2", name + "_cat", cout, (2 + n) * c)

    x = conv("l0", "input", c1, 3, 3, 2)
    x = conv("l1", x, c2, c1, 3, 2)
    x = c2f("l2", x, c2, c2, 1, True)
    x = conv("l3", x, c3, c2, 3, 2)
    p3 = c2f("l4", x, c3, c3, 2, True)
    x = conv("l5", p3, c4, c3, 3, 2)
    p4 = c2f("l6", x, c4, c4, 2, True)
    x = conv("l7", p4, c5, c4, 3, 2)
    x = c2f("l8", x, c5, c5, 1, True)
    # SPPF
    y = conv("l9_cv1", x, c5 // 2, c5)
    pools = [y]
    for i in range(3):
        g.append(dict(op="maxpool", **{"in": pools[-1]}, out=f"l9_p{i}", k=(5, 5), stride=(1, 1), pad=(2, 2, 2, 2)))
        pools.append(f"l9_p{i}")
    g.append(dict(op="concat", ins=pools, out="l9_cat"))
    p5 = conv("l9_cv2", "l9_cat", c5, 2 * c5)
    # PAN neck
    g.append(dict(op="upsample", **{"in": p5}, out="l10", factor=2))
    g.append(dict(op="concat", ins=["l10", p4], out="l11"))
    n4 = c2f("l12", "l11", c5 + c4, c4, 1, False)
    g.append(dict(op="upsample", **{"in": n4}, out="l13", factor=2))
    g.append(dict(op="concat", ins=["l13", p3], out="l14"))
    o3 = c2f("l15", "l14", c4 + c3, c3, 1, False)
    x = conv("l16", o3, c3, c3, 3, 2)
    g.append(dict(op="concat", ins=[x, n4], out="l17"))
    o4 = c2f("l18", "l17", c3 + c4, c4, 1, False)
    x = conv("l19", o4, c4, c4, 3, 2)
    g.append(dict(op="concat", ins=[x, p5], out="l20"))
    o5 = c2f("l21", "l20", c4 + c5, c5, 1, False)
    outs = []
    cb, cc = max(16, c3 // 4, 64), max(c3, min(classes, 100))
    for i, (src, ch) in enumerate([(o3, c3), (o4, c4), (o5, c5)]):
        a = conv(f"box{i}_a", src, cb, ch, 3)
        a = conv(f"box{i}_b", a, cb, cb, 3)
        outs.append(conv(f"box{i}", a, 64, cb, 1, act=None))
        a = conv(f"cls{i}_a", src, cc, ch, 3)
        a = conv(f"cls{i}_b", a, cc, cc, 3)
        outs.append(conv(f"cls{i}", a, classes, cc, 1, act=None))
    g.append(dict(op="output", ins=outs))
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
        elif nd["op"] == "slice":
            c, h, w = shapes[nd["in"]]
            shapes[nd["out"]] = (nd["end"] - nd["begin"], h, w)
        elif nd["op"] == "concat":
            c0, h, w = shapes[nd["ins"][0]]
            shapes[nd["out"]] = (sum(shapes[i][0] for i in nd["ins"]), h, w)
        elif nd["op"] == "upsample":
            c, h, w = shapes[nd["in"]]
            shapes[nd["out"]] = (c, h * nd["factor"], w * nd["factor"])
        elif nd["op"] == "output":
            pass
        elif nd["op"] == "gap":
            shapes[nd["out"]] = (shapes[nd["in"]][0], 1, 1)
        elif nd["op"] == "fc":
            m = nd["w"].shape[0] * nd["w"].shape[1]
            per_layer.append((nd["name"], m))
            total += m
            shapes[nd["out"]] = (nd["w"].shape[0], 1, 1)
    return total, per_layer, shapes
