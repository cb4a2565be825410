using Sharplight.Cuda.Native;
using Sharplight.Graph;
using Sharplight.Runtime;
using Sharplight.Tensors;

namespace Sharplight.Cuda;

/// <summary>
/// One opened GPU (slc_device). Safe to share between threads: one opened device serves every model placed on that GPU,
/// each model running on its own scheduler thread (src/Sharplight.Core/Runtime/DevicePool.cs:3-8); the native device handle is
/// thread-safe, the per-segment handles are used by one Run at a time (CompiledModel.cs:223).
/// </summary>
internal sealed class CudaDevice : IComputeDevice
{
    private readonly DeviceOptions? _options;
    private nint _handle;

    internal CudaDevice(DeviceInfo info, DeviceOptions? options)
    {
        Info = info;
        _options = options;
        EnabledFeatures = DeviceFeatures.Effective(info.Features, options?.DisabledFeatures);
        Check.Ok(NativeMethods.slc_device_open(info.Index, out _handle));
    }

    public DeviceInfo Info { get; }

    public IReadOnlySet<string> EnabledFeatures { get; }

    internal nint Handle => _handle != 0 ? _handle : throw new ObjectDisposedException(nameof(CudaDevice));

    public long AvailableMemory
    {
        get
        {
            Check.Ok(NativeMethods.slc_device_memory(Handle, out long free, out _));
            return _options?.MemoryBudget is { } budget ? Math.Min(budget, free) : free;
        }
    }

    /// <summary>ggml type id of a weight type this provider has kernels for, or 0.</summary>
    internal static int FormatOf(DataType type)
        => type == DataType.Q4_0 ? Slc.FormatQ4_0 : type == DataType.Q8_0 ? Slc.FormatQ8_0
         : type == DataType.Q4_K ? Slc.FormatQ4_K : type == DataType.Q6_K ? Slc.FormatQ6_K
         : type == DataType.Q5_0 ? Slc.FormatQ5_0 : type == DataType.IQ4_NL ? Slc.FormatIQ4_NL   // Q8_0 records after upload
         : type == DataType.Q5_K ? Slc.FormatQ5_K : 0;                                               // two Q4_K weights after upload

    internal static int BlockSize(int format) => format is Slc.FormatQ4_K or Slc.FormatQ5_K or Slc.FormatQ6_K ? 256 : 32;

    /// <summary>
    /// Yes only for MatMul with a static Q8_0 / Q4_0 / Q4_K / Q6_K / Q5_0 / Q5_K / IQ4_NL weight whose K is a multiple of the block size, f32 or bf16
    /// activations, and activations that may be quantized to 8 bits -- the mirror of CpuOpSupport.CheckQuantizedMatMul
    /// (src/Sharplight.Cpu/CpuOpSupport.Linear.cs:21-53). Everything else goes to PlacementOptions.Fallback
    /// (PlacementPlanner.cs:238-248). View nodes (Reshape / Slice / Permute) are not asked: they stay on their group's device
    /// and the segment treats them as stride / offset metadata.
    /// </summary>
    public OpSupport Supports(Node node)
    {
        ArgumentNullException.ThrowIfNull(node);
        if (node.Op != StandardOps.MatMul)
        {
            return OpSupport.No($"{node.Op.Name} does not run on the cuda provider (quantized MatMul only)");
        }

        var x = node.Inputs[0];
        var weight = node.Inputs[1];
        if (x.Type != DataType.F32 && x.Type != DataType.BF16)
        {
            return OpSupport.No($"MatMul activations must be f32 or bf16, got {x.Type}");
        }

        int format = FormatOf(weight.Type);
        if (format == 0)
        {
            return OpSupport.No($"MatMul weight type {weight.Type} has no CUDA kernel");
        }

        if (weight.Kind != ValueKind.Weight)
        {
            return OpSupport.No("MatMul with an activation as the quantized weight");
        }

        long k = weight.Shape.Dims[1].Fixed;
        if (k % BlockSize(format) != 0)
        {
            return OpSupport.No($"K={k} is not a multiple of the {weight.Type} block size");
        }

        if (!EnabledFeatures.Contains(DeviceFeatures.IntDot))
        {
            return OpSupport.No("int_dot is disabled and this provider has no float path");
        }

        // StandardOps.F32ActivationsAttribute: the node keeps f32 activation math unless reduced precision is allowed. Such
        // a node is never silently quantized: it runs the dequant-fused f32 mat-vec (SLC_MATMUL_F32_ACTIVATIONS), which
        // keeps one f32 activation row in shared memory; a longer K goes to the placement fallback.
        if (node.Attributes.Get(StandardOps.F32ActivationsAttribute, false) && k > Slc.F32ActivationsMaxK)
        {
            return OpSupport.No($"f32 activations requested and K={k} exceeds the f32 mat-vec's {Slc.F32ActivationsMaxK}");
        }

        return OpSupport.Yes;
    }

    public ICompiledSegment Compile(GraphSegment segment, CompileOptions options)
    {
        ArgumentNullException.ThrowIfNull(segment);
        ArgumentNullException.ThrowIfNull(options);
        return new CudaSegment(this, segment, options);
    }

    public void Dispose()
    {
        nint h = Interlocked.Exchange(ref _handle, 0);
        if (h != 0)
        {
            NativeMethods.slc_device_close(h);
        }
    }
}
