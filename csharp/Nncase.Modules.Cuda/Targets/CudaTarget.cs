// NOT COMPILED IN THIS REPOSITORY: the build image has no dotnet SDK. Written against nncase 2.x.
//
// The `cuda` target. It differs from the cpu target (modules/Nncase.Modules.StackVM/Targets/CPUTarget.cs:23-95)
// at exactly the hooks that target leaves empty:
//   * RegisterQuantizePass: Conv2D / MatMul whose operands and result carry range markers (placed by
//     AddRangeOfAndMarker and filled by the Quantizer, Compiler.cs:339-350) are rewritten into u8 custom calls
//     of the cuda module with QuantParams computed from those ranges;
//   * CreateModuleBuilder: functions of module kind "cuda" go to CudaModuleBuilder, everything else stays on
//     the StackVM builder, so a model is a StackVM main plus cuda callees reached through EXTCALL / CUSCALL.
// Markers that no rule consumed are removed afterwards like on the cpu target, so unsupported operators run
// in float on the StackVM.
using System;
using System.Collections.Generic;
using System.CommandLine.Invocation;
using System.Threading.Tasks;
using Microsoft.Extensions.Configuration;
using Nncase.CodeGen;
using Nncase.CodeGen.Cuda;
using Nncase.CodeGen.StackVM;
using Nncase.IR;
using Nncase.Passes;
using Nncase.Quantization;

namespace Nncase.Targets;

public sealed class CudaTargetOptions : ITargetCompileOptions
{
    /// <summary>Gets or sets the CUDA device the runtime plugin uses (also: NNCASE_CUDA_DEVICE).</summary>
    public int Device { get; set; }

    /// <summary>Gets or sets a value indicating whether weights are quantized to symmetric int8 (no zero-point column in the MMA).</summary>
    public bool SymmetricWeights { get; set; }
}

public sealed class CudaTarget : ITarget
{
    public const string Kind = "cuda";

    private readonly CudaTargetOptions _options = new();

    string ITarget.Kind => Kind;

    public (System.CommandLine.Command Command, Func<InvocationContext, System.CommandLine.Command, ITargetCompileOptions> Parser) RegisterCommandAndParser()
    {
        var command = new System.CommandLine.Command(Kind);
        var device = new System.CommandLine.Option<int>("--cuda-device", () => 0, "CUDA device index used by the runtime");
        var symmetric = new System.CommandLine.Option<bool>("--cuda-symmetric-weights", () => false, "quantize weights to symmetric int8");
        command.AddOption(device);
        command.AddOption(symmetric);
        return (command, (context, _) =>
        {
            _options.Device = context.ParseResult.GetValueForOption(device);
            _options.SymmetricWeights = context.ParseResult.GetValueForOption(symmetric);
            return _options;
        });
    }

    public void ParseTargetDependentOptions(IConfigurationSection configure)
    {
        // [cuda] section of the per-target TOML (TargetProvider.cs:20-23)
        _options.Device = configure.GetValue("device", _options.Device);
        _options.SymmetricWeights = configure.GetValue("symmetric_weights", _options.SymmetricWeights);
    }

    public void RegisterTargetInDependentPass(IPassManager passManager, CompileOptions options)
    {
    }

    public void RegisterTargetDependentPass(IPassManager passManager, CompileOptions options)
    {
    }

    public Task<Dictionary<ENode, List<Tuple<List<DataType>, List<List<QuantParam>>, float>>>> BindQuantMethodCosine(ICalibrationDatasetProvider calibrationDataset, List<ENode> rangeOfs, List<ENode> childrenOfRangeOfs, QuantizeOptions quantizeOptions)
    {
        // one quantization scheme (u8 activations, per-channel 8-bit weights): nothing to search
        return Task.FromResult(new Dictionary<ENode, List<Tuple<List<DataType>, List<List<QuantParam>>, float>>>());
    }

    public Task AdaRoundWeights(ICalibrationDatasetProvider calibrationDataset, List<ENode> rangeOfs, List<ENode> childrenOfRangeOfs, QuantizeOptions quantizeOptions)
    {
        return Task.CompletedTask;
    }

    public void RegisterQuantizePass(IPassManager passManager, CompileOptions options)
    {
        if (options.QuantizeOptions.ModelQuantMode != ModelQuantMode.UsePTQ)
        {
            return;
        }

        passManager.AddWithName<DataflowPass>("LowerToCudaQuantized").Configure(p =>
        {
            p.Add<Passes.Rules.Cuda.LowerMarkedConv2D>(_options.SymmetricWeights);
            p.Add<Passes.Rules.Cuda.LowerMarkedMatMul>(_options.SymmetricWeights);
        });
    }

    public void RegisterTargetDependentAfterQuantPass(IPassManager passManager, CompileOptions options)
    {
        if (options.QuantizeOptions.ModelQuantMode == ModelQuantMode.UsePTQ)
        {
            passManager.AddWithName<DataflowPass>("RemoveMarker").Configure(p =>
            {
                p.Add<Passes.Rules.Lower.RemoveMarker>();
            });

            // Dequantize directly followed by Quantize with the same param between two cuda calls cancels.
            passManager.AddWithName<DataflowPass>("FoldCudaRequantize").Configure(p =>
            {
                p.Add<Passes.Rules.Cuda.FoldDequantizeQuantize>();
            });
        }
    }

    public void RegisterTargetDependentBeforeCodeGen(IPassManager passManager, CompileOptions options)
    {
    }

    public IModuleBuilder CreateModuleBuilder(string moduleKind, CompileOptions options)
    {
        return moduleKind switch
        {
            Callable.StackVMModuleKind => new StackVMModuleBuilder(),
            CudaModuleBuilder.Kind => new CudaModuleBuilder(),
            _ => throw new NotSupportedException($"{moduleKind} module is not supported by the cuda target."),
        };
    }
}
