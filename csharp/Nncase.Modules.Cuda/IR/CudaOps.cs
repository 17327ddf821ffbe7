// NOT COMPILED IN THIS REPOSITORY: the build image has no dotnet SDK. Written against nncase 2.x.
//
// Operator-level entry points of the cuda module as CustomOps (src/Nncase.Core/IR/Op.cs:138-154). The StackVM
// code generator emits CUSCALL{RegisteredName, SerializeFields(), argument count} for a call whose target is a
// CustomOp (modules/Nncase.Modules.StackVM/CodeGen/StackVM/CodegenVisitor.cs:297-301) and lists ModuleType in
// the module's ".custom_calls" section (StackVMLinkableModule.cs:25-30); at run time the StackVM resolves the
// name in the table that libnncase.simulator.cuda.so exports through collect_custom_call.
//
// Field layouts are the ones the plugin reads (nncase_b200/plugin/cuda_runtime_module.cpp):
//   cuda.quantize / cuda.dequantize   int32 target typecode
//   cuda.qconv2d                      nncb_conv2d_desc (include/nncase_b200.h), 34 x 4 bytes, little endian
using System;
using System.IO;
using Nncase.CodeGen;
using Nncase.PatternMatch;

namespace Nncase.IR.Cuda;

public static class CudaModuleType
{
    public static readonly ModuleType Value = ModuleType.Create("cuda");
}

/// <summary>u8 x u8|i8 Conv2D with the fused requantising epilogue. Arguments: input (u8 NHWC), weights (OHWI),
/// weight zero points (i32[oc]), multipliers (f32[oc] = input scale x weight scale), bias (f32[oc]) and
/// optionally the residual (u8, output shape).</summary>
[PatternFunctionalGenerator]
public sealed partial class CudaQConv2D : CustomOp
{
    public static readonly ParameterInfo Input = new(typeof(CudaQConv2D), 0, "input");
    public static readonly ParameterInfo Weights = new(typeof(CudaQConv2D), 1, "weights");
    public static readonly ParameterInfo WeightZeroPoints = new(typeof(CudaQConv2D), 2, "wzp");
    public static readonly ParameterInfo Multipliers = new(typeof(CudaQConv2D), 3, "mult");
    public static readonly ParameterInfo Bias = new(typeof(CudaQConv2D), 4, "bias");

    public CudaQConv2D(int[] strides, int[] paddings, int[] dilations, int groups, bool signedWeights, QuantParam input, QuantParam output, ValueRange<float> fusedClamp)
    {
        Strides = strides;
        Paddings = paddings;
        Dilations = dilations;
        Groups = groups;
        SignedWeights = signedWeights;
        InputQuantParam = input;
        OutputQuantParam = output;
        FusedClamp = fusedClamp;
    }

    public int[] Strides { get; }

    /// <summary>Gets top, bottom, left, right.</summary>
    public int[] Paddings { get; }

    public int[] Dilations { get; }

    public int Groups { get; }

    public bool SignedWeights { get; }

    public QuantParam InputQuantParam { get; }

    public QuantParam OutputQuantParam { get; }

    public ValueRange<float> FusedClamp { get; }

    public override string RegisteredName => "cuda.qconv2d";

    public override ModuleType ModuleType => CudaModuleType.Value;

    public override byte[] SerializeFields()
    {
        using var ms = new MemoryStream();
        using var w = new BinaryWriter(ms);

        // n, h, w, c and oc, kh, kw: the plugin takes them from the tensors
        for (int i = 0; i < 7; i++)
        {
            w.Write(0);
        }

        w.Write(Strides[0]);
        w.Write(Strides[1]);
        foreach (var p in Paddings)
        {
            w.Write(p);
        }

        w.Write(Dilations[0]);
        w.Write(Dilations[1]);
        w.Write(Groups);
        w.Write(SignedWeights ? 1 : 0);
        w.Write(InputQuantParam.ZeroPoint);
        w.Write(OutputQuantParam.Scale);
        w.Write(OutputQuantParam.ZeroPoint);
        w.Write(FusedClamp.Min);
        w.Write(FusedClamp.Max);

        // has_residual .. add_out_zp (5), has_y2 .. y2_hi (5), f32_out, force_path: set by the plugin / unused here
        for (int i = 0; i < 12; i++)
        {
            w.Write(0);
        }

        w.Flush();
        return ms.ToArray();
    }
}

/// <summary>kernels::stackvm::quantize on the GPU: q = clamp(rint(x / scale + zero_point)).</summary>
[PatternFunctionalGenerator]
public sealed partial class CudaQuantize : CustomOp
{
    public static readonly ParameterInfo Input = new(typeof(CudaQuantize), 0, "input");
    public static readonly ParameterInfo QuantParam = new(typeof(CudaQuantize), 1, "quantParam");

    public CudaQuantize(DataType targetType)
    {
        TargetType = targetType;
    }

    public DataType TargetType { get; }

    public override string RegisteredName => "cuda.quantize";

    public override ModuleType ModuleType => CudaModuleType.Value;

    public override byte[] SerializeFields() => BitConverter.GetBytes((int)((PrimType)TargetType).TypeCode);
}

/// <summary>kernels::stackvm::dequantize on the GPU: y = (q - zero_point) * scale.</summary>
[PatternFunctionalGenerator]
public sealed partial class CudaDequantize : CustomOp
{
    public static readonly ParameterInfo Input = new(typeof(CudaDequantize), 0, "input");
    public static readonly ParameterInfo DequantParam = new(typeof(CudaDequantize), 1, "dequantParam");

    public override string RegisteredName => "cuda.dequantize";

    public override ModuleType ModuleType => CudaModuleType.Value;

    public override byte[] SerializeFields() => BitConverter.GetBytes((int)Runtime.TypeCode.Float32);
}
