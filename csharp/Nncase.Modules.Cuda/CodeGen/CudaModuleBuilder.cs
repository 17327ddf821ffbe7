// NOT COMPILED IN THIS REPOSITORY: the build image has no dotnet SDK. Written against nncase 2.x.
//
// IModuleBuilder for module kind "cuda" (src/Nncase.Core/CodeGen/IModuleBuilder.cs:141-154). ModelBuilder
// groups functions by BaseFunction.ModuleKind and hands each group to the builder its target returns
// (src/Nncase.CodeGen/CodeGen/ModelBuilder.cs:39-53); LinkedModel.Serialize then writes module_header,
// functions and sections (LinkedModel.cs:27-170). A cuda function is a chain of quantized calls produced by
// LowerMarkedConv2D and friends; its body is not bytecode but a launch list:
//
//   module section   ".rdata"  weights and per-channel tables, every blob 16-byte aligned
//   function section ".desc"   DescHeader | output tensor indices | DescTensor[] | DescOp[]
//
// DescHeader  12 x u32  magic "NCUD", version 1, batch, tensors, ops, input tensor, input is NHWC, in c/h/w,
//                       outputs, reserved
// DescTensor  6 words   h, w, c, dtype (0 u8, 1 f32), zero point (i32), scale (f32)
// DescOp      160 bytes kind (u32), name char[28], i32[24], f32[8]; the per-kind meaning of the fields is
//                       listed with the reader, nncase_b200/csrc/program.cu (nncb_program_create)
// The same bytes are produced by nncase_b200/kmodel.py, which is tested against the runtime.
using System;
using System.Collections.Generic;
using System.IO;
using System.Linq;
using System.Text;
using Nncase.IR;
using Nncase.IR.Cuda;

namespace Nncase.CodeGen.Cuda;

public sealed class CudaModuleBuilder : ModuleBuilder
{
    public const string Kind = "cuda";

    public const uint Version = 1;

    public override string ModuleKind => Kind;

    protected override ILinkableModule CreateLinkableModule(IReadOnlyList<ILinkableFunction> linkableFunctions)
    {
        return new CudaLinkableModule(linkableFunctions, SectionManager);
    }

    protected override FunctionBuilder CreateFunctionBuilder(uint id)
    {
        return new CudaFunctionBuilder(id, SectionManager);
    }
}

internal enum CudaOpKind : uint
{
    QuantizeInput = 0,
    Conv = 1,
    MaxPool = 2,
    Requant = 3,
    Add = 4,
    Slice = 5,
    ConcatPart = 6,
    Upsample = 7,
    GlobalMean = 8,
}

internal sealed record CudaTensorDesc(int H, int W, int C, bool IsFloat, int ZeroPoint, float Scale);

internal sealed class CudaOpRecord
{
    public CudaOpKind Kind { get; init; }

    public string Name { get; init; } = string.Empty;

    public int[] Ints { get; } = new int[24];

    public float[] Floats { get; } = new float[8];

    public void Write(BinaryWriter w)
    {
        w.Write((uint)Kind);
        var name = new byte[28];
        Encoding.UTF8.GetBytes(Name.AsSpan(0, Math.Min(Name.Length, 27)), name);
        w.Write(name);
        foreach (var v in Ints)
        {
            w.Write(v);
        }

        foreach (var v in Floats)
        {
            w.Write(v);
        }
    }
}

/// <summary>Walks the body of a cuda function (post-order over its calls) and turns every quantized call into an
/// operator record; constants go to the module's .rdata section.</summary>
internal sealed class CudaFunctionBuilder : FunctionBuilder
{
    private const uint Magic = 0x4455434E; // "NCUD"
    private readonly List<CudaTensorDesc> _tensors = new();
    private readonly List<CudaOpRecord> _ops = new();
    private readonly Dictionary<Expr, int> _tensorOf = new(ReferenceEqualityComparer.Instance);
    private readonly List<int> _outputs = new();
    private readonly MemoryStream _desc = new();
    private int _batch;
    private int[] _inputChw = new int[3];

    public CudaFunctionBuilder(uint id, SectionManager sectionManager)
        : base(id, sectionManager)
    {
    }

    protected override void Compile(BaseFunction callable)
    {
        var function = (Function)callable;
        var input = function.Parameters.ToArray().Single();
        var inShape = input.CheckedShape.ToValueArray(); // NCHW f32
        _batch = inShape[0];
        _inputChw = new[] { inShape[1], inShape[2], inShape[3] };
        foreach (var output in function.Body is IR.Tuple t ? t.Fields.ToArray() : new[] { function.Body })
        {
            _outputs.Add(Visit(output));
        }
    }

    protected override void WriteText()
    {
        using var w = new BinaryWriter(_desc, Encoding.UTF8, leaveOpen: true);
        foreach (var v in new uint[] { Magic, CudaModuleBuilder.Version, (uint)_batch, (uint)_tensors.Count, (uint)_ops.Count, 0, 0, (uint)_inputChw[0], (uint)_inputChw[1], (uint)_inputChw[2], (uint)_outputs.Count, 0 })
        {
            w.Write(v);
        }

        foreach (var o in _outputs)
        {
            w.Write((uint)o);
        }

        foreach (var t in _tensors)
        {
            w.Write((uint)t.H);
            w.Write((uint)t.W);
            w.Write((uint)t.C);
            w.Write(t.IsFloat ? 1u : 0u);
            w.Write(t.ZeroPoint);
            w.Write(t.Scale);
        }

        foreach (var op in _ops)
        {
            op.Write(w);
        }
    }

    protected override ILinkableFunction CreateLinkableFunction(uint id, BaseFunction callable, IReadOnlyList<FunctionRef> functionRefs, Stream text)
    {
        var desc = new LinkedSection(_desc, ".desc", 0, 8, (ulong)_desc.Length);
        return new CudaLinkableFunction(id, callable, functionRefs, text, new[] { desc });
    }

    private int NewTensor(int h, int w, int c, bool isFloat, QuantParam? qp)
    {
        _tensors.Add(new CudaTensorDesc(h, w, c, isFloat, qp?.ZeroPoint ?? 0, qp?.Scale ?? 1f));
        return _tensors.Count - 1;
    }

    private int AddRdata(ReadOnlySpan<byte> bytes)
    {
        var writer = SectionManager.GetWriter(WellknownSectionNames.Rdata);
        writer.AlignPosition(16);
        var offset = (int)writer.Position();
        writer.Write(bytes);
        return offset;
    }

    private int Visit(Expr expr)
    {
        if (_tensorOf.TryGetValue(expr, out var known))
        {
            return known;
        }

        int result;
        switch (expr)
        {
            case Call { Target: CudaQuantize } call:
                {
                    // the input stage: f32 NCHW parameter -> u8 NHWC
                    var qp = ((TensorConst)call[CudaQuantize.QuantParam]).Value.ToScalar<QuantParam>();
                    result = NewTensor(_inputChw[1], _inputChw[2], _inputChw[0], false, qp);
                    var op = new CudaOpRecord { Kind = CudaOpKind.QuantizeInput, Name = "input" };
                    op.Ints[0] = result;
                    op.Ints[1] = _inputChw[0];
                    op.Ints[2] = _inputChw[0];
                    _ops.Add(op);
                    break;
                }

            case Call { Target: CudaQConv2D conv } call:
                {
                    int src = Visit(call[CudaQConv2D.Input]);
                    var weights = ((TensorConst)call[CudaQConv2D.Weights]).Value;
                    var wshape = weights.Shape.ToValueArray(); // OHWI
                    var zw = ((TensorConst)call[CudaQConv2D.WeightZeroPoints]).Value;
                    var mult = ((TensorConst)call[CudaQConv2D.Multipliers]).Value;
                    var bias = ((TensorConst)call[CudaQConv2D.Bias]).Value;
                    var outShape = call.CheckedShape.ToValueArray(); // NHWC
                    result = NewTensor(outShape[1], outShape[2], outShape[3], false, conv.OutputQuantParam);
                    var op = new CudaOpRecord { Kind = CudaOpKind.Conv, Name = call.Metadata.OutputNames?.FirstOrDefault() ?? "conv2d" };
                    var i = op.Ints;
                    i[0] = src;
                    i[1] = result;
                    i[2] = -1; // residual: filled by the add-fusion step of the builder when present
                    i[3] = -1; // second (ReLU) output
                    i[4] = wshape[0];
                    i[5] = wshape[1];
                    i[6] = wshape[2];
                    i[7] = conv.Strides[0];
                    i[8] = conv.Strides[1];
                    Array.Copy(conv.Paddings, 0, i, 9, 4);
                    i[13] = conv.Dilations[0];
                    i[14] = conv.Dilations[1];
                    i[15] = conv.Groups;
                    i[16] = conv.SignedWeights ? 1 : 0;
                    i[17] = 0; // u8 output
                    i[18] = -1; // no activation table
                    i[19] = AddRdata(weights.BytesBuffer);
                    i[20] = AddRdata(zw.BytesBuffer);
                    i[21] = AddRdata(mult.BytesBuffer);
                    i[22] = AddRdata(bias.BytesBuffer);
                    i[23] = conv.OutputQuantParam.ZeroPoint;
                    op.Floats[0] = conv.FusedClamp.Min;
                    op.Floats[1] = conv.FusedClamp.Max;
                    op.Floats[2] = conv.OutputQuantParam.Scale;
                    _ops.Add(op);
                    break;
                }

            case Call { Target: CudaDequantize } call:
                // a function result: the u8 tensor itself is the function's output, the caller dequantizes
                result = Visit(call[CudaDequantize.Input]);
                break;

            default:
                throw new NotSupportedException($"{expr.GetType().Name} cannot be part of a cuda function; the partitioner should have left it to the StackVM.");
        }

        _tensorOf.Add(expr, result);
        return result;
    }
}

internal sealed class CudaLinkableFunction : ILinkableFunction
{
    public CudaLinkableFunction(uint id, BaseFunction sourceFunction, IEnumerable<FunctionRef> functionRefs, Stream text, IReadOnlyList<ILinkedSection> sections)
    {
        Id = id;
        SourceFunction = sourceFunction;
        FunctionRefs = functionRefs;
        Text = text;
        Sections = sections;
    }

    public uint Id { get; }

    public BaseFunction SourceFunction { get; }

    public IEnumerable<FunctionRef> FunctionRefs { get; }

    public Stream Text { get; }

    public IReadOnlyList<ILinkedSection> Sections { get; }
}

internal sealed class CudaLinkableModule : LinkableModule
{
    public CudaLinkableModule(IReadOnlyList<ILinkableFunction> functions, SectionManager sectionManager)
        : base(functions, sectionManager)
    {
    }

    protected override ILinkedModule CreateLinkedModule(IReadOnlyList<LinkedFunction> linkedFunctions, Stream text)
    {
        return new CudaLinkedModule(linkedFunctions, SectionManager.GetContent(WellknownSectionNames.Rdata));
    }
}

internal sealed class CudaLinkedModule : ILinkedModule
{
    public CudaLinkedModule(IReadOnlyList<LinkedFunction> functions, Stream? rdata)
    {
        Functions = functions;
        Sections = new[] { new LinkedSection(rdata, ".rdata", 0, 16, (ulong)(rdata?.Length ?? 0)) };
    }

    public string ModuleKind => CudaModuleBuilder.Kind;

    public uint Version => CudaModuleBuilder.Version;

    public IReadOnlyList<ILinkedFunction> Functions { get; }

    public IReadOnlyList<ILinkedSection> Sections { get; }
}
