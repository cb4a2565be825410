using Sharplight.Cuda.Native;
using Sharplight.Graph;
using Sharplight.Runtime;
using Sharplight.Tensors;

namespace Sharplight.Cuda;

/// <summary>
/// A compiled list of quantized MatMul nodes on one GPU (ICompiledSegment, src/Sharplight.Core/Runtime/ICompiledSegment.cs:6-25).
/// Weights are uploaded once at compile time. SetInput copies the host bytes into page-locked staging and starts the copy to the
/// device; Execute quantizes every distinct input once and runs all nodes that read it from that one 8-bit copy (as the
/// reference's lowering shares it, src/Sharplight.Shaders/Lowering/GraphLowerer.IntDot.cs:38-43), then starts the copy of the
/// outputs back; GetOutput waits for the device once and reads the staged bytes. Error behaviour follows the CPU segment
/// (src/Sharplight.Cpu/CpuCompiledSegment.cs:96-124,149,189). Used by one Run at a time (CompiledModel.cs:223).
/// </summary>
internal sealed unsafe class CudaSegment : ICompiledSegment, IDeviceForwardingSegment
{
    private sealed class Slot
    {
        public nint Device;          // device buffer of the value
        public nint Staging;         // page-locked host buffer (inputs and outputs only)
        public long Columns;
        public int ElementBytes;
        public int Dtype;            // Slc.F32 / Slc.Bf16
        public long Rows;            // rows of the last SetInput
        public bool Forwarded;       // the device buffer belongs to another segment
        public bool DeviceOnly;      // an output nobody reads on the host
    }

    private readonly CudaDevice _device;
    private readonly long _maxRows;
    private readonly Dictionary<Value, Slot> _slots = new();
    private readonly Dictionary<Value, nint> _activations = new();          // one 8-bit copy per distinct MatMul input
    private readonly List<(Node Node, nint Op, Value X, Value Y, bool F32)> _steps = new();
    private readonly List<nint> _weights = new();
    private long _weightBytes;
    private bool _executed;
    private bool _synced;
    private bool _disposed;

    internal CudaSegment(CudaDevice device, GraphSegment segment, CompileOptions options)
    {
        _device = device;
        Segment = segment;
        _maxRows = options.SymbolBounds.TryGetValue("T", out long t) ? t : 1;
        try
        {
            foreach (Node node in segment.Nodes)
            {
                if (node.Op.Category == OpCategory.View)
                {
                    // Reshape / Slice / Permute of a [T, K] activation that keeps rows contiguous is metadata only: the
                    // view's output aliases its input's buffer. (Anything that breaks row contiguity was refused by
                    // Supports of the MatMul that reads it.)
                    _slots[node.Outputs[0]] = SlotOf(node.Inputs[0]);
                    continue;
                }

                OpSupport support = device.Supports(node);
                if (!support.IsSupported)
                {
                    throw new NotSupportedException(support.Reason);
                }

                Value x = node.Inputs[0], w = node.Inputs[1], y = node.Outputs[0];
                int format = CudaDevice.FormatOf(w.Type);
                long n = w.Shape.Dims[0].Fixed, k = w.Shape.Dims[1].Fixed;
                ReadOnlySpan<byte> blocks = segment.Graph.GetWeightData(w);
                nint weight;
                fixed (byte* p = blocks)
                {
                    Check.Ok(NativeMethods.slc_weight_upload(device.Handle, format, n, k, p, blocks.Length, out weight));
                }

                _weights.Add(weight);
                Check.Ok(NativeMethods.slc_weight_shape(weight, out _, out _, out _, out long bytes));
                _weightBytes += bytes;

                // a node that keeps f32 activation math (StandardOps.F32ActivationsAttribute) is never quantized, unless the
                // compile options allow reduced precision (src/Sharplight.Cpu/CpuCompiledSegment.LowerLinear.cs:39)
                bool f32 = node.Attributes.Get(StandardOps.F32ActivationsAttribute, false) && !options.AllowReducedPrecision;
                uint flags = f32 ? Slc.MatMulF32Activations : options.Deterministic ? Slc.MatMulRowInvariant : 0u;
                Check.Ok(NativeMethods.slc_matmul_create(device.Handle, weight, _maxRows, flags, out nint op));
                Slot xs = SlotOf(x, k, x.Type == DataType.BF16 ? 2 : 4, x.Type == DataType.BF16 ? Slc.Bf16 : Slc.F32);
                SlotOf(y, n, 4, Slc.F32);
                if (!f32 && !_activations.ContainsKey(x))
                {
                    Check.Ok(NativeMethods.slc_activation_create(device.Handle, _maxRows, k, out nint act));
                    _activations[x] = act;
                }

                _ = xs;
                _steps.Add((node, op, x, y, f32));
            }

            foreach (Value v in segment.Inputs.Concat(segment.Outputs))
            {
                Slot s = _slots[v];
                if (s.Staging == 0)
                {
                    Check.Ok(NativeMethods.slc_host_alloc(_maxRows * s.Columns * s.ElementBytes, out s.Staging));
                }
            }
        }
        catch
        {
            Dispose();
            throw;
        }
    }

    public GraphSegment Segment { get; }

    public long DeviceMemoryBytes
        => _weightBytes + _slots.Values.Distinct().Where(s => !s.Forwarded).Sum(s => _maxRows * s.Columns * s.ElementBytes);

    private Slot SlotOf(Value v) => _slots.TryGetValue(v, out Slot? s) ? s : throw new ArgumentException($"'{v.Name}' has no producer in this segment");

    private Slot SlotOf(Value v, long columns, int elementBytes, int dtype)
    {
        if (_slots.TryGetValue(v, out Slot? s))
        {
            return s;
        }

        s = new Slot { Columns = columns, ElementBytes = elementBytes, Dtype = dtype };
        Check.Ok(NativeMethods.slc_buffer_alloc(_device.Handle, _maxRows * columns * elementBytes, out s.Device));
        _slots[v] = s;
        return s;
    }

    private void Live() => ObjectDisposedException.ThrowIf(_disposed, this);

    public void SetInput(Value value, ReadOnlySpan<byte> data)
    {
        Live();
        if (!Segment.Inputs.Contains(value))
        {
            throw new ArgumentException($"'{value.Name}' is not an input of this segment", nameof(value));
        }

        Slot s = _slots[value];
        if (s.Forwarded)
        {
            throw new InvalidOperationException($"input '{value.Name}' is forwarded from another segment's output");
        }

        long rowBytes = s.Columns * s.ElementBytes;
        if (data.Length % rowBytes != 0 || data.Length > _maxRows * rowBytes)
        {
            throw new ArgumentException($"input '{value.Name}' must be whole rows of {rowBytes} bytes, at most {_maxRows} of them", nameof(data));
        }

        data.CopyTo(new Span<byte>((void*)s.Staging, data.Length));
        Check.Ok(NativeMethods.slc_buffer_copy_async(_device.Handle, s.Device, s.Staging, data.Length, Slc.HostToDevice, 0));
        s.Rows = data.Length / rowBytes;
    }

    public void Execute(RunParameters parameters) => Execute(parameters, new HashSet<Value>());

    public void Execute(RunParameters parameters, IReadOnlySet<Value> skipDownloads)
    {
        Live();
        ArgumentNullException.ThrowIfNull(parameters);
        long rows = parameters.Symbols.TryGetValue("T", out long t) ? t : -1;
        if (rows > _maxRows)
        {
            throw new InvalidOperationException($"T={rows} exceeds the compiled bound {_maxRows}");
        }

        foreach (Value input in Segment.Inputs)
        {
            Slot s = _slots[input];
            if (!s.Forwarded && s.Rows == 0)
            {
                throw new InvalidOperationException($"input '{input.Name}' was not set");
            }

            rows = rows < 0 ? s.Rows : rows;
        }

        var quantized = new HashSet<Value>();
        foreach ((Node _, nint op, Value x, Value y, bool f32) in _steps)
        {
            Slot xs = _slots[x], ys = _slots[y];
            if (f32)
            {
                Check.Ok(NativeMethods.slc_matmul_run(op, (void*)xs.Device, xs.Dtype, rows, xs.Columns, 1, (float*)ys.Device, ys.Columns, 1, 0));
                ys.Rows = rows;
                continue;
            }

            nint act = _activations[x];
            if (quantized.Add(x))
            {
                Check.Ok(NativeMethods.slc_activation_quantize(act, xs.Device, xs.Dtype, rows, xs.Columns, 0));
            }

            Check.Ok(NativeMethods.slc_matmul_run_quantized(op, act, ys.Device, ys.Columns, 0));
            ys.Rows = rows;
        }

        foreach (Value output in Segment.Outputs)
        {
            Slot s = _slots[output];
            if (s.DeviceOnly || skipDownloads.Contains(output))
            {
                continue;
            }

            Check.Ok(NativeMethods.slc_buffer_copy_async(_device.Handle, s.Staging, s.Device, rows * s.Columns * 4, Slc.DeviceToHost, 0));
        }

        _executed = true;
        _synced = false;
    }

    public void GetOutput(Value value, Span<byte> destination)
    {
        Live();
        if (!Segment.Outputs.Contains(value))
        {
            throw new ArgumentException($"'{value.Name}' is not an output of this segment", nameof(value));
        }

        if (!_executed)
        {
            throw new InvalidOperationException("GetOutput before Execute");
        }

        Slot s = _slots[value];
        long bytes = s.Rows * s.Columns * 4;
        if (destination.Length < bytes)
        {
            throw new ArgumentException($"output '{value.Name}' needs {bytes} bytes", nameof(destination));
        }

        if (!_synced)
        {
            Check.Ok(NativeMethods.slc_device_sync(_device.Handle));
            Check.Ok(NativeMethods.slc_last_status(_device.Handle, out int status));
            if (status != 0)
            {
                throw new InvalidOperationException($"a kernel of this device reported status {status}");
            }

            _synced = true;
        }

        if (s.DeviceOnly)
        {
            fixed (byte* p = destination)
            {
                Check.Ok(NativeMethods.slc_buffer_download(_device.Handle, p, s.Device, bytes));
            }

            return;
        }

        new ReadOnlySpan<byte>((void*)s.Staging, (int)bytes).CopyTo(destination);
    }

    /// <summary>
    /// IDeviceForwardingSegment (src/Sharplight.Core/Runtime/IDeviceForwardingSegment.cs:10-21): from now on the input is read
    /// straight from the producer's output buffer in device memory. False when that buffer is not reachable from here.
    /// </summary>
    public bool TryForwardFrom(Value value, ICompiledSegment producer)
    {
        Live();
        if (producer is not CudaSegment other || other._disposed || !ReferenceEquals(other._device, _device))
        {
            return false;
        }

        if (!Segment.Inputs.Contains(value) || !other.Segment.Outputs.Contains(value) || other._maxRows > _maxRows)
        {
            return false;
        }

        Slot mine = _slots[value], theirs = other._slots[value];
        if (mine.Columns != theirs.Columns || mine.ElementBytes != theirs.ElementBytes)
        {
            return false;
        }

        if (!mine.Forwarded)
        {
            NativeMethods.slc_buffer_free(_device.Handle, mine.Device);
        }

        mine.Device = theirs.Device;
        mine.Forwarded = true;
        theirs.DeviceOnly = true;
        return true;
    }

    /// <summary>MatMul keeps no state between runs (no KV cache lives in this segment).</summary>
    public void ResetState() => Live();

    public void Dispose()
    {
        if (_disposed)
        {
            return;
        }

        _disposed = true;
        _ = NativeMethods.slc_device_sync(_device.Handle);
        foreach ((Node _, nint op, Value _, Value _, bool _) in _steps)
        {
            NativeMethods.slc_matmul_destroy(op);
        }

        foreach (nint act in _activations.Values)
        {
            NativeMethods.slc_activation_destroy(act);
        }

        foreach (Slot s in _slots.Values.Distinct())
        {
            if (s.Device != 0 && !s.Forwarded)
            {
                NativeMethods.slc_buffer_free(_device.Handle, s.Device);
            }

            if (s.Staging != 0)
            {
                NativeMethods.slc_host_free(s.Staging);
            }
        }

        foreach (nint w in _weights)
        {
            NativeMethods.slc_weight_free(w);
        }
    }
}
