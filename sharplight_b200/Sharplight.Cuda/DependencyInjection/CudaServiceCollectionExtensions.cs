using Sharplight.Cuda;

namespace Microsoft.Extensions.DependencyInjection;

/// <summary>
/// Registration next to AddVulkanProvider (src/Sharplight.Vulkan/DependencyInjection/VulkanServiceCollectionExtensions.cs:18-28).
/// Register before the CPU provider so that ExecutionProviderCatalog.Discover lists "cuda" first
/// (src/Sharplight.Core/Runtime/ExecutionProviderCatalog.cs:7-9); a MatMul-only device needs the CPU as the placement fallback
/// (PlacementOptions.Fallback).
/// </summary>
public static class CudaServiceCollectionExtensions
{
    extension(IServiceCollection services)
    {
        public IServiceCollection AddCudaProvider()
        {
            ArgumentNullException.ThrowIfNull(services);
            return services.AddExecutionProvider<CudaExecutionProvider>();
        }
    }
}
