using System.Runtime.InteropServices;
using Sharplight.Cuda.Native;
using Sharplight.Runtime;

namespace Sharplight.Cuda;

/// <summary>
/// Execution provider "cuda": the quantized MatMul operator on NVIDIA B200 (compute capability 10.0) through
/// libsharplight_cuda. Cheap to construct; the driver is touched only by <see cref="CheckAvailability"/> and
/// <see cref="GetDevices"/> (src/Sharplight.Core/Runtime/IExecutionProvider.cs:4-5). Every other operator stays on the
/// placement fallback (the CPU provider): <see cref="CudaDevice.Supports"/> says no to it.
/// </summary>
public sealed class CudaExecutionProvider : IExecutionProvider
{
    public const string ProviderName = "cuda";

    public string Name => ProviderName;

    /// <summary>Never throws: a missing library or driver is an unavailable provider (ExecutionProviderCatalog.cs:28-47).</summary>
    public ProviderAvailability CheckAvailability()
    {
        try
        {
            if (NativeMethods.slc_abi_version() != NativeMethods.AbiVersion)
            {
                return ProviderAvailability.Unavailable("libsharplight_cuda ABI version differs from this binding");
            }

            if (NativeMethods.slc_device_count(out int count) < 0 || count == 0)
            {
                return ProviderAvailability.Unavailable("no CUDA device");
            }

            for (int i = 0; i < count; i++)
            {
                if (NativeMethods.slc_device_info_get(i, out var info) >= 0 && info.Supported != 0)
                {
                    return ProviderAvailability.Available("CUDA, compute capability 10.0");
                }
            }

            return ProviderAvailability.Unavailable("no compute-capability 10.0 device (the kernels are sm_100a only)");
        }
        catch (Exception e) when (e is DllNotFoundException or EntryPointNotFoundException or BadImageFormatException)
        {
            return ProviderAvailability.Unavailable(e.Message);
        }
    }

    public unsafe IReadOnlyList<DeviceInfo> GetDevices()
    {
        if (!CheckAvailability().IsAvailable)
        {
            return [];
        }

        Check.Ok(NativeMethods.slc_device_count(out int count));
        var devices = new List<DeviceInfo>();
        for (int i = 0; i < count; i++)
        {
            Check.Ok(NativeMethods.slc_device_info_get(i, out var info));
            if (info.Supported == 0)
            {
                continue;
            }

            devices.Add(new DeviceInfo
            {
                Provider = ProviderName,
                Index = i,
                Name = Marshal.PtrToStringUTF8((nint)info.Name) ?? "CUDA device",
                Kind = DeviceKind.DiscreteGpu,
                TotalMemory = info.TotalMemory,
                Vendor = "NVIDIA",
                Driver = Marshal.PtrToStringUTF8((nint)info.Driver) ?? "",
                // the GPU UUID, so the same GPU under Vulkan and CUDA is recognised as one device (DeviceInfo.cs:20-22)
                Uuid = Convert.ToHexString(new ReadOnlySpan<byte>(info.Uuid, 16)).ToLowerInvariant(),
                Features = new HashSet<string>(StringComparer.OrdinalIgnoreCase)
                {
                    DeviceFeatures.IntDot, DeviceFeatures.MatrixInt8, "subgroup_ops", "fp16", "bf16",
                },
                ConcurrentWorkgroups = info.ConcurrentWorkgroups,
                Capabilities = new Dictionary<string, string>
                {
                    ["sm_count"] = info.SmCount.ToString(),
                    ["compute_capability"] = $"{info.CcMajor}.{info.CcMinor}",
                    ["l2_bytes"] = info.L2Bytes.ToString(),
                    ["max_shared_per_block"] = info.MaxSharedPerBlock.ToString(),
                },
            });
        }

        return devices;
    }

    public IComputeDevice OpenDevice(DeviceInfo device, DeviceOptions? options = null)
    {
        ArgumentNullException.ThrowIfNull(device);
        if (device.Provider != Name)
        {
            throw new ArgumentException($"Device {device} does not belong to the cuda provider.");
        }

        return new CudaDevice(device, options);
    }

    /// <summary>The kernels are compiled ahead of time into the shared library: nothing portable to compile or cache.</summary>
    public string? PortableCodeFormat => null;

    public bool CanCompileFor(DeviceProfile profile) => false;

    public Task<PortableCodeSet> CompilePortableAsync(PortableCompilationRequest request, CancellationToken cancellationToken = default)
    {
        ArgumentNullException.ThrowIfNull(request);
        return Task.FromResult(PortableCodeSet.Empty(Name));
    }

    public Task<DeviceCodeSet> CompileDeviceSpecificAsync(IComputeDevice device, PortableCodeSet portable, CancellationToken cancellationToken = default)
    {
        ArgumentNullException.ThrowIfNull(device);
        ArgumentNullException.ThrowIfNull(portable);
        if (device.Info.Provider != Name)
        {
            throw new ArgumentException($"Device {device.Info} does not belong to the cuda provider.", nameof(device));
        }

        return Task.FromResult(DeviceCodeSet.Empty(Name, device.Info.Name));
    }

    public void Dispose()
    {
    }
}
