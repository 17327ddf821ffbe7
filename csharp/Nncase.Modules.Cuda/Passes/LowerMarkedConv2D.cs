// NOT COMPILED IN THIS REPOSITORY: the build image has no dotnet SDK. Written against nncase 2.x.
//
// Marker-driven lowering of Conv2D / MatMul into the cuda module's quantized calls. After calibration every
// Conv2D / MatMul operand and result is wrapped in Marker("RangeOf", target, range) with a constant range
// (AddRangeOfAndMarker.cs:99-189, Quantizer.AssignRanges Quantizer.cs:590-602). The only in-tree precedent of a
// target consuming those markers is the K210 module's LowerConv2D
// (modules/Nncase.Modules.K210/Transform/Rules/K210/LowerConv2D.cs:27-94); this rule has the same shape.
//
//   Marker(Conv2D(Marker(x, rx), Marker(W, rw), b, stride, pad, dil, groups, clamp), ry)
//     ->  Dequantize(cuda.qconv2d(Quantize(NHWC(x), qx), Wq, zw, sx * sw, b), qy)  transposed back to NCHW
// with qx, qy = GetQuantParam(range, 8, Unsigned) (QuantUtility.cs:41-67) and per-output-channel weight params
// from GetWeightsRangesByChannel (QuantUtility.cs:106-151). Arithmetic of the call: include/nncase_b200.h.
using System;
using System.Linq;
using Nncase.IR;
using Nncase.IR.Cuda;
using Nncase.IR.F;
using Nncase.PatternMatch;
using Nncase.Utilities;
using static Nncase.IR.TypePatternUtility;
using static Nncase.PatternMatch.F.Math;
using static Nncase.PatternMatch.F.NN;
using static Nncase.PatternMatch.Utility;

namespace Nncase.Passes.Rules.Cuda;

[RuleGenerator]
public sealed partial class LowerMarkedConv2D : IRewriteRule
{
    private readonly bool _symmetricWeights;

    public LowerMarkedConv2D(bool symmetricWeights)
    {
        _symmetricWeights = symmetricWeights;
    }

    public IPattern Pattern { get; } = IsRangeOfMarker(
        "outMarker",
        IsConv2D(
            null,
            "conv2d",
            PadMode.Constant,
            IsRangeOfMarker("inMarker", IsWildcard("input") with { TypePattern = HasFixedShape() }, IsTensorConst("inRange")),
            IsRangeOfMarker(IsTensorConst("weights"), IsWildcard()),
            IsTensorConst("bias"),
            IsTensorConst("strides"),
            IsTensorConst("paddings"),
            IsTensorConst("dilations"),
            IsTensorConst("groups"),
            IsTensorConst("fusedClamp")),
        IsTensorConst("outRange"));

    private Expr? GetReplace(Expr input, Tensor<float> weights, Tensor<float> bias, int[] strides, Tensor<int> paddings, int[] dilations, int groups, float[] fusedClamp, Tensor<float> inRange, Tensor<float> outRange)
    {
        var inChannels = input.CheckedShape[1].FixedValue;
        var outChannels = weights.Shape[0].FixedValue;
        if (groups != 1 && !(groups == inChannels && groups == outChannels))
        {
            return null; // grouped convolutions other than depthwise stay in float
        }

        var qx = QuantUtility.GetQuantParam(new ValueRange<float>(inRange[0], inRange[1]), 8, QuantMode.UnsignedMode);
        var qy = QuantUtility.GetQuantParam(new ValueRange<float>(outRange[0], outRange[1]), 8, QuantMode.UnsignedMode);
        var mode = _symmetricWeights ? QuantMode.SignedSymmetricMode : QuantMode.UnsignedMode;
        var (wq, zw, sw) = CudaQuantUtility.QuantizeWeightsByChannel(weights, mode); // OHWI bytes, i32[oc], f32[oc]
        var mult = sw.Select(s => qx.Scale * s).ToArray();

        var nhwc = Tensors.NCHWToNHWC(input);
        var xq = new Call(new CudaQuantize(DataTypes.UInt8), nhwc, Tensor.FromScalar(qx));
        var op = new CudaQConv2D(
            strides,
            new[] { paddings[0, 0], paddings[0, 1], paddings[1, 0], paddings[1, 1] },
            dilations,
            groups,
            _symmetricWeights,
            qx,
            qy,
            new ValueRange<float>(fusedClamp[0], fusedClamp[1]));
        var yq = new Call(op, xq, wq, Tensor.From(zw), Tensor.From(mult), bias);
        var y = new Call(new CudaDequantize(), yq, Tensor.FromScalar(qy));
        return Tensors.NHWCToNCHW(y);
    }
}

/// <summary>MatMul with a constant right-hand side = the 1x1 case of the convolution: [M,K] x [K,N] runs as
/// n = 1, h = 1, w = M, c = K, oc = N with weights [N][1][1][K] (MatMulToConv2D.cs:30-66 does the same in float).</summary>
[RuleGenerator]
public sealed partial class LowerMarkedMatMul : IRewriteRule
{
    private readonly bool _symmetricWeights;

    public LowerMarkedMatMul(bool symmetricWeights)
    {
        _symmetricWeights = symmetricWeights;
    }

    public IPattern Pattern { get; } = IsRangeOfMarker(
        "outMarker",
        IsMatMul(
            IsRangeOfMarker(IsWildcard("lhs") with { TypePattern = HasFixedShape() & HasRank(2) }, IsTensorConst("inRange")),
            IsRangeOfMarker(IsTensorConst("rhs") with { TypePattern = HasRank(2) }, IsWildcard())),
        IsTensorConst("outRange"));

    private Expr? GetReplace(Expr lhs, Tensor<float> rhs, Tensor<float> inRange, Tensor<float> outRange)
    {
        var m = lhs.CheckedShape[0].FixedValue;
        var k = lhs.CheckedShape[1].FixedValue;
        var n = rhs.Shape[1].FixedValue;
        var qx = QuantUtility.GetQuantParam(new ValueRange<float>(inRange[0], inRange[1]), 8, QuantMode.UnsignedMode);
        var qy = QuantUtility.GetQuantParam(new ValueRange<float>(outRange[0], outRange[1]), 8, QuantMode.UnsignedMode);
        var mode = _symmetricWeights ? QuantMode.SignedSymmetricMode : QuantMode.UnsignedMode;
        var weightsNK = rhs.Transpose(new[] { 1, 0 }).Reshape(new[] { n, 1, 1, k }); // [N][1][1][K] = OHWI
        var (wq, zw, sw) = CudaQuantUtility.QuantizeWeightsByChannel(weightsNK, mode, alreadyOHWI: true);
        var mult = sw.Select(s => qx.Scale * s).ToArray();
        var x = Tensors.Reshape(lhs, new[] { 1, 1, m, k });
        var xq = new Call(new CudaQuantize(DataTypes.UInt8), x, Tensor.FromScalar(qx));
        var op = new CudaQConv2D(new[] { 1, 1 }, new[] { 0, 0, 0, 0 }, new[] { 1, 1 }, 1, _symmetricWeights, qx, qy, ValueRange<float>.Full);
        var yq = new Call(op, xq, wq, Tensor.From(zw), Tensor.From(mult), Tensor.From(new float[n]));
        var y = new Call(new CudaDequantize(), yq, Tensor.FromScalar(qy));
        return Tensors.Reshape(y, new[] { m, n });
    }
}

/// <summary>Quantize(Dequantize(x, p), p) between two cuda calls is the identity on u8.</summary>
[RuleGenerator]
public sealed partial class FoldDequantizeQuantize : IRewriteRule
{
    public IPattern Pattern { get; } = IsCall(
        "q",
        IsOp<CudaQuantize>(),
        IsCall(IsOp<CudaDequantize>(), IsWildcard("x"), IsTensorConst("p0")),
        IsTensorConst("p1"));

    private Expr? GetReplace(Expr x, Tensor p0, Tensor p1)
    {
        return p0.BytesBuffer.SequenceEqual(p1.BytesBuffer) ? x : null;
    }
}

internal static class CudaQuantUtility
{
    /// <summary>Per-output-channel weight quantization: ranges from QuantUtility.GetWeightsRangesByChannel, params from
    /// GetQuantParam, q = clamp(rint(w / scale + zero_point)); returns the weights as OHWI bytes.</summary>
    public static (Tensor Weights, int[] ZeroPoints, float[] Scales) QuantizeWeightsByChannel(Tensor<float> oihw, QuantMode mode, bool alreadyOHWI = false)
    {
        var oc = oihw.Shape[0].FixedValue;
        var perChannel = oihw.Length / oc;
        var src = oihw.Buffer.Span;
        var zps = new int[oc];
        var scales = new float[oc];
        var dst = new byte[oihw.Length];
        var (qmin, qmax) = mode == QuantMode.UnsignedMode ? (0, 255) : (-128, 127);
        int ic = alreadyOHWI ? 1 : oihw.Shape[1].FixedValue;
        int taps = perChannel / ic;
        for (int o = 0; o < oc; o++)
        {
            var ch = src.Slice(o * perChannel, perChannel);
            float min = float.MaxValue, max = float.MinValue;
            foreach (var v in ch)
            {
                min = MathF.Min(min, v);
                max = MathF.Max(max, v);
            }

            var qp = QuantUtility.GetQuantParam(new ValueRange<float>(min, max), 8, mode);
            zps[o] = qp.ZeroPoint;
            scales[o] = qp.Scale;
            for (int i = 0; i < perChannel; i++)
            {
                // OIHW index i = c * taps + t  ->  OHWI index t * ic + c
                int di = alreadyOHWI ? i : ((i % taps) * ic) + (i / taps);
                var q = (int)MathF.Round((ch[i] / qp.Scale) + qp.ZeroPoint, MidpointRounding.ToEven);
                dst[(o * perChannel) + di] = unchecked((byte)Math.Clamp(q, qmin, qmax));
            }
        }

        var shape = alreadyOHWI ? oihw.Shape.ToValueArray() : new[] { oc, oihw.Shape[2].FixedValue, oihw.Shape[3].FixedValue, ic };
        var dtype = mode == QuantMode.UnsignedMode ? DataTypes.UInt8 : DataTypes.Int8;
        return (Tensor.FromBytes(dtype, dst, shape), zps, scales);
    }
}
