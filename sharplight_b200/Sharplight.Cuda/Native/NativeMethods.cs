using System.Runtime.InteropServices;

namespace Sharplight.Cuda.Native;

/// <summary>
/// P/Invoke surface of libsharplight_cuda (include/sharplight_cuda.h), in the style of the repository's other native binding
/// (src/Sharplight.Audio/Native/NativeMethods.cs): source-generated marshalling, blittable arguments, raw handles that the
/// SafeHandle types of this folder wrap. Every function returns an slc_result (0 = success, negative = failure) unless noted.
/// </summary>
internal static unsafe partial class NativeMethods
{
    public const string Library = "sharplight_cuda";
    public const int AbiVersion = 1;

    [LibraryImport(Library)] public static partial int slc_abi_version();
    [LibraryImport(Library)] public static partial nint slc_version_string();
    [LibraryImport(Library)] public static partial nint slc_error_string(int code);
    [LibraryImport(Library)] public static partial nint slc_last_error_message();

    [LibraryImport(Library)] public static partial int slc_device_count(out int count);
    [LibraryImport(Library)] public static partial int slc_device_info_get(int index, out SlcDeviceInfo info);
    [LibraryImport(Library)] public static partial int slc_device_open(int index, out nint device);
    [LibraryImport(Library)] public static partial void slc_device_close(nint device);
    [LibraryImport(Library)] public static partial int slc_device_memory(nint device, out long free, out long total);
    [LibraryImport(Library)] public static partial int slc_device_sync(nint device);
    [LibraryImport(Library)] public static partial nint slc_device_stream(nint device);
    [LibraryImport(Library)] public static partial int slc_last_status(nint device, out int status);

    [LibraryImport(Library)] public static partial int slc_buffer_alloc(nint device, long bytes, out nint ptr);
    [LibraryImport(Library)] public static partial void slc_buffer_free(nint device, nint ptr);
    [LibraryImport(Library)] public static partial int slc_buffer_upload(nint device, nint dst, void* host, long bytes);
    [LibraryImport(Library)] public static partial int slc_buffer_download(nint device, void* host, nint src, long bytes);
    [LibraryImport(Library)] public static partial int slc_host_alloc(long bytes, out nint hostPtr);
    [LibraryImport(Library)] public static partial void slc_host_free(nint hostPtr);
    [LibraryImport(Library)] public static partial int slc_buffer_copy_async(nint device, nint dst, nint src, long bytes, int direction, nint stream);
    [LibraryImport(Library)] public static partial int slc_buffer_densify(nint device, nint dst, nint src, long batch, long rows, long cols, long batchStride, long rowStride, long colStride, int elemBytes, nint stream);

    [LibraryImport(Library)] public static partial int slc_stream_create(nint device, out nint stream);
    [LibraryImport(Library)] public static partial void slc_stream_destroy(nint device, nint stream);
    [LibraryImport(Library)] public static partial int slc_stream_wait(nint device, nint waiter, nint signal);
    [LibraryImport(Library)] public static partial int slc_graph_begin(nint device, nint stream);
    [LibraryImport(Library)] public static partial int slc_graph_end(nint device, nint stream, out nint graph);
    [LibraryImport(Library)] public static partial int slc_graph_launch(nint graph, nint stream);
    [LibraryImport(Library)] public static partial void slc_graph_destroy(nint graph);
    [LibraryImport(Library)] public static partial nint slc_graph_last_error();

    [LibraryImport(Library)] public static partial int slc_weight_upload(nint device, int format, long n, long k, void* blocks, long bytes, out nint weight);
    [LibraryImport(Library)] public static partial int slc_weight_upload_kslice(nint device, int format, long n, long k, void* blocks, long bytes, long k0, long k1, out nint weight);
    [LibraryImport(Library)] public static partial int slc_weight_download(nint weight, void* blocks, long bytes);
    [LibraryImport(Library)] public static partial int slc_weight_shape(nint weight, out int format, out long n, out long k, out long deviceBytes);
    [LibraryImport(Library, StringMarshalling = StringMarshalling.Utf8)] public static partial int slc_gguf_open(string path, out nint file);
    [LibraryImport(Library)] public static partial void slc_gguf_close(nint file);
    [LibraryImport(Library)] public static partial int slc_gguf_tensor_count(nint file, out long count);
    [LibraryImport(Library)] public static partial int slc_gguf_tensor_info(nint file, long index, byte* nameOut, int nameCapacity, out int format, out int rank, out long n, out long k, out long bytes);
    [LibraryImport(Library, StringMarshalling = StringMarshalling.Utf8)] public static partial int slc_gguf_find(nint file, string name, out long index);
    [LibraryImport(Library)] public static partial int slc_weight_upload_gguf(nint device, nint file, long index, out nint weight);
    [LibraryImport(Library)] public static partial nint slc_gguf_last_error();
    [LibraryImport(Library)] public static partial int slc_weight_layout_bytes(nint weight, out long bytes);
    [LibraryImport(Library)] public static partial int slc_weight_export_layout(nint weight, void* outHost, long bytes);
    [LibraryImport(Library)] public static partial int slc_weight_import_layout(nint device, void* artefactHost, long bytes, out nint weight);
    [LibraryImport(Library)] public static partial void slc_weight_free(nint weight);

    [LibraryImport(Library)] public static partial int slc_matmul_create(nint device, nint weight, long maxRows, uint flags, out nint op);
    [LibraryImport(Library)] public static partial int slc_matmul_create_dual(nint device, nint gate, nint up, long maxRows, uint flags, out nint op);
    [LibraryImport(Library)] public static partial void slc_matmul_destroy(nint op);
    [LibraryImport(Library)] public static partial int slc_matmul_run(nint op, void* x, int xDtype, long rows, long xStride, int xIsDevice, float* y, long yStride, int yIsDevice, nint stream);
    [LibraryImport(Library)] public static partial int slc_matmul_set_kernel(nint op, int kernel);
    [LibraryImport(Library)] public static partial int slc_matmul_last_kernel(nint op, out int kernel, out int launches);

    [LibraryImport(Library)] public static partial int slc_activation_create(nint device, long maxRows, long k, out nint act);
    [LibraryImport(Library)] public static partial void slc_activation_destroy(nint act);
    [LibraryImport(Library)] public static partial int slc_activation_quantize(nint act, nint xDevice, int xDtype, long rows, long xStride, nint stream);
    [LibraryImport(Library)] public static partial int slc_activation_set_rows(nint act, nint xDevice, int xDtype, long rows, long xStride, nint stream);
    [LibraryImport(Library)] public static partial int slc_activation_quantize_rmsnorm(nint act, nint xDevice, int xDtype, long rows, long xStride, nint weightDevice, float eps, nint yDevice, long yStride, nint stream);
    [LibraryImport(Library)] public static partial int slc_activation_quantize_silu_mul(nint act, nint gateDevice, long gateStride, nint upDevice, long upStride, long rows, nint yDevice, long yStride, nint stream);
    [LibraryImport(Library)] public static partial int slc_argmax_rows(nint device, nint yDevice, long rows, long n, long yStride, nint outIndexDevice, nint stream);
    [LibraryImport(Library)] public static partial int slc_matmul_id_run(nint weight, int experts, nint xDevice, int xDtype, long xStride, nint idsDevice, long tokens, long slots, int perSlot, nint yDevice, long yStride, nint stream);
    [LibraryImport(Library)] public static partial int slc_matmul_run_quantized(nint op, nint act, nint yDevice, long yStride, nint stream);
    [LibraryImport(Library)] public static partial int slc_matmul_run_quantized_epilogue(nint op, nint act, nint exchange, nint bias, nint residual, long residualStride, nint y, long yStride, nint stream);

    [LibraryImport(Library)] public static partial int slc_tp_exchange_create(nint device, int rank, int world, long maxRows, long n, out nint exchange, Span<byte> handle64);
    [LibraryImport(Library)] public static partial int slc_tp_exchange_connect(nint exchange, ReadOnlySpan<byte> handles);
    [LibraryImport(Library)] public static partial void slc_tp_exchange_destroy(nint exchange);
    [LibraryImport(Library)] public static partial int slc_tp_exchange_set_wait_ms(nint exchange, int milliseconds);
    [LibraryImport(Library)] public static partial int slc_tp_comm_unique_id(Span<byte> id128);
    [LibraryImport(Library)] public static partial int slc_tp_comm_create(nint device, int rank, int world, ReadOnlySpan<byte> id128, out nint comm);
    [LibraryImport(Library)] public static partial void slc_tp_comm_destroy(nint comm);
    [LibraryImport(Library)] public static partial int slc_tp_comm_set_chunking(nint comm, int minRows);
    [LibraryImport(Library)] public static partial int slc_tp_exchange_set_comm(nint exchange, nint comm, int inKernelRows);
    [LibraryImport(Library)] public static partial int slc_matmul_run_allreduce(nint op, nint exchange, nint x, int xDtype, long rows, long xStride, nint y, long yStride, nint stream);
    [LibraryImport(Library)] public static partial int slc_matmul_run_quantized_allreduce(nint op, nint act, nint exchange, nint y, long yStride, nint stream);

    [LibraryImport(Library)] public static partial int slc_matmul_run_static(nint weight, nint x, int xDtype, long rows, long xStride, nint y, long yStride, nint stream);
    [LibraryImport(Library)] public static partial nint slc_static_last_error();

    [LibraryImport(Library)] public static partial int slc_debug_quantize(nint device, void* x, int xDtype, long rows, long k, sbyte* q, float* d, float* gs);
    [LibraryImport(Library)] public static partial int slc_debug_block_dots(nint op, void* x, int xDtype, long rows, int* s32);
}

/// <summary>slc_device_info of the C header, field for field.</summary>
[StructLayout(LayoutKind.Sequential)]
internal unsafe struct SlcDeviceInfo
{
    public fixed byte Name[256];
    public fixed byte Driver[64];
    public fixed byte Uuid[16];
    public long TotalMemory;
    public long FreeMemory;
    public int SmCount;
    public int CcMajor;
    public int CcMinor;
    public int MaxSharedPerBlock;
    public int L2Bytes;
    public int ConcurrentWorkgroups;
    public int Supported;
    public int Reserved;
}

/// <summary>Constants of the C header.</summary>
internal static class Slc
{
    public const int FormatQ4_0 = 2, FormatQ8_0 = 8, FormatQ4_K = 12, FormatQ6_K = 14;
    public const int FormatQ5_0 = 6, FormatIQ4_NL = 20;   // rewritten at upload as Q8_0 device records
    public const int FormatQ5_K = 13;                     // split at upload into two Q4_K weights
    public const int F32 = 0, Bf16 = 1;
    public const uint MatMulRowInvariant = 1, MatMulF32Activations = 2;
    public const long F32ActivationsMaxK = 49152;
    public const int HostToDevice = 0, DeviceToHost = 1, DeviceToDevice = 2;
    public const int ErrTimeout = -7;
}

/// <summary>Native result -> the exception the managed contracts promise.</summary>
internal static class Check
{
    public static void Ok(int code)
    {
        if (code >= 0)
        {
            return;
        }

        string msg = Marshal.PtrToStringUTF8(NativeMethods.slc_last_error_message()) ?? "";
        if (msg.Length == 0)
        {
            msg = Marshal.PtrToStringUTF8(NativeMethods.slc_error_string(code)) ?? "";
        }

        throw code switch
        {
            -1 => new ArgumentException(msg),                 // SLC_ERR_INVALID_ARGUMENT
            -2 => new InsufficientMemoryException(msg),       // SLC_ERR_OUT_OF_MEMORY
            -3 or -4 => new NotSupportedException(msg),       // SLC_ERR_NO_DEVICE, SLC_ERR_UNSUPPORTED
            -6 => new InvalidOperationException(msg),         // SLC_ERR_INVALID_STATE
            -7 => new TimeoutException(msg),                  // a bounded device-side wait ran out
            _ => new InvalidOperationException($"libsharplight_cuda: {msg} (code {code})"),
        };
    }

    /// <summary>The stream / graph group reports through its own thread-local text.</summary>
    public static void Graph(int code)
    {
        if (code < 0)
        {
            throw new InvalidOperationException(Marshal.PtrToStringUTF8(NativeMethods.slc_graph_last_error()) ?? "stream / graph call failed");
        }
    }
}
