// NOT COMPILED IN THIS REPOSITORY: the build image has no dotnet SDK. Written against nncase 2.x.
//
// Plugin entry point. The compiler's PluginLoader scans Nncase.Modules.*.dll for IApplicationPart
// implementations with a parameterless constructor (src/Nncase.Compiler/Hosting/PluginLoader.cs:136-149) and
// lets each register its services; the StackVM module registers the "cpu" target the same way
// (modules/Nncase.Modules.StackVM/StackVMModule.cs:16-19).
using DryIoc;
using Nncase.Hosting;
using Nncase.Targets;

namespace Nncase;

public sealed class CudaModule : IApplicationPart
{
    public void ConfigureServices(IRegistrator registrator)
    {
        registrator.Register<ITarget, CudaTarget>(reuse: Reuse.Singleton);
    }
}
