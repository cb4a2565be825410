/*
 * libsharplight_cuda: flat C ABI of the CUDA (sm_100a) execution provider for Sharplight's quantized MatMul operator.
 *
 * The managed provider (Sharplight.Cuda: CudaExecutionProvider / CudaDevice / CudaSegment) binds these entry points
 * with [LibraryImport]; each comment names the reference interface the entry point serves (paths relative to the
 * Sharplight source tree). The conventions follow the repository's own native ABI
 * (native/sharplight_audio/include/sharplight_audio.h:1-47):
 *  - every function returns an slc_result (0 = success, negative = failure) unless stated otherwise;
 *  - handles are opaque pointers owned by the caller until their *_close / *_free / *_destroy function is called;
 *  - strings are UTF-8, NUL terminated, in static or thread-local storage;
 *  - no callbacks into managed code;
 *  - a handle must not be destroyed while another thread is inside a call using it. An slc_device may be used from
 *    several threads at once (one opened device serves every model on that GPU, src/Sharplight.Core/Runtime/
 *    DevicePool.cs:3-8); an slc_matmul / slc_activation is used by one thread at a time (one Run at a time per
 *    compiled model, src/Sharplight.Core/Runtime/CompiledModel.cs:223).
 *
 * Weights are the raw ggml blocks the GGUF importer hands out (src/Sharplight.Import.Gguf/GgufWeightSource.cs:6-38),
 * row-major [N, K]; the library copies them and keeps a same-size device layout of its own.
 * There is no CPU fallback: without a CUDA device every compute entry point fails with SLC_ERR_NO_DEVICE.
 */
#ifndef SHARPLIGHT_CUDA_H
#define SHARPLIGHT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#if defined(_WIN32)
#define SLC_API __declspec(dllexport)
#elif defined(__GNUC__) || defined(__clang__)
#define SLC_API __attribute__((visibility("default")))
#else
#define SLC_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ABI version; incremented when an existing function or struct changes incompatibly. */
#define SLC_ABI_VERSION 1

typedef int32_t slc_result;

enum
{
    SLC_OK = 0,
    SLC_ERR_INVALID_ARGUMENT = -1,  /* -> ArgumentException */
    SLC_ERR_OUT_OF_MEMORY = -2,     /* -> InsufficientMemoryException */
    SLC_ERR_NO_DEVICE = -3,         /* no CUDA driver / no sm_100 device: the provider reports itself unavailable */
    SLC_ERR_UNSUPPORTED = -4,       /* -> NotSupportedException (format, shape) */
    SLC_ERR_CUDA = -5,              /* a CUDA runtime call failed; slc_last_error_message() has the text */
    SLC_ERR_INVALID_STATE = -6,     /* -> InvalidOperationException (e.g. rows beyond the compiled bound) */
    SLC_ERR_TIMEOUT = -7,           /* a bounded device-side wait ran out; the context stays usable */
    SLC_ERR_BUFFER_TOO_SMALL = -8
};

/* Weight formats, numbered like ggml (src/Sharplight.Import.Gguf/GgmlTypes.cs:51-92); block sizes and bytes as in
   src/Sharplight.Core/Tensors/DataType.cs:102,106,110,116,118,120,124. Q5_0 and IQ4_NL are rewritten at upload, exactly,
   as Q8_0 device records (their values are a signed byte times the block's f16 d, which is how the reference's
   integer-dot decoder treats them too, src/Sharplight.Cpu/IntDot.Decode.cs:101-123,225-238): they cost 34 bytes per 32
   values on the device and run through the Q8_0 kernels. Q5_K is split at upload, exactly, into two Q4_K weights -- the
   block without its fifth bits, and the fifth bits as nibbles with d' = 16 d, dmin' = 0 -- and every MatMul runs both
   (one two-weight launch on the mat-vec; elsewhere the second launch adds onto the first): 288 bytes per 256 values.
   An upload whose 16 d is not an f16 returns SLC_ERR_UNSUPPORTED. Converted weights have no slc_weight_download; Q5_K has no layout artefact and takes no
   part in a dual MatMul. */
typedef enum slc_format
{
    SLC_FMT_Q4_0 = 2,   /* 32 values, 18 bytes: f16 d; u8 qs[16] */
    SLC_FMT_Q5_0 = 6,   /* 32 values, 22 bytes: f16 d; u32 qh; u8 qs[16] (converted at upload) */
    SLC_FMT_Q8_0 = 8,   /* 32 values, 34 bytes: f16 d; i8 q[32] */
    SLC_FMT_Q4_K = 12,  /* 256 values, 144 bytes: f16 d; f16 dmin; u8 scales[12]; u8 qs[128] */
    SLC_FMT_Q5_K = 13,  /* 256 values, 176 bytes: f16 d; f16 dmin; u8 scales[12]; u8 qh[32]; u8 qs[128] (split at upload) */
    SLC_FMT_Q6_K = 14,  /* 256 values, 210 bytes: u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d */
    SLC_FMT_IQ4_NL = 20 /* 32 values, 18 bytes: f16 d; u8 qs[16], nibbles index a 16-entry codebook (converted at upload) */
} slc_format;

/* Activation element types. */
typedef enum slc_dtype
{
    SLC_F32 = 0,
    SLC_BF16 = 1   /* widened to f32 (exact) before quantization */
} slc_dtype;

/* slc_matmul_create flags. */
enum
{
    SLC_MATMUL_DEFAULT = 0,
    /* every activation row is computed exactly as a single row would be, so a 2-4 row verification step gives the
       logits of one-row decoding bit for bit (CompileOptions.RowInvariantRows, src/Sharplight.Core/Runtime/
       CompileOptions.cs:52-60; src/Sharplight.Cpu/MatMulOp.cs:36-41) */
    SLC_MATMUL_ROW_INVARIANT = 1,
    /* the node keeps f32 activation math (StandardOps' f32-activations attribute, src/Sharplight.Core/Graph/
       StandardOps.cs:130-135): the activations are never quantized; slc_matmul_run serves the op with the dequant-fused
       f32 mat-vec (GPU form in the reference: src/Sharplight.Shaders/Kernels/matmul.slang:148-226), up to 4 rows per
       pass over the weights. Meant for decode-sized row counts; K up to 49 152. Such an op refuses the entry points
       that take quantized activations. */
    SLC_MATMUL_F32_ACTIVATIONS = 2
};

/* Kernel families, for slc_matmul_set_kernel / slc_matmul_last_kernel. */
enum
{
    SLC_KERNEL_AUTO = 0,
    SLC_KERNEL_MMVQ = 1,     /* dp4a mat-vec, weights streamed once for up to 8 activation rows */
    SLC_KERNEL_SKINNY = 2,   /* int8 mma tiles with the weight as the streamed operand, 9..64 rows */
    SLC_KERNEL_MMQ = 3,      /* tcgen05 / TMEM int8 GEMM for prefill */
    SLC_KERNEL_TILE = 4,     /* tcgen05 kind::i8 / TMEM tiles with the weights as the M operand, stream-K over persistent
                                CTAs, 3 rows and more; selectable, not chosen automatically */
    SLC_KERNEL_F32 = 5       /* dequant-fused f32 mat-vec of SLC_MATMUL_F32_ACTIVATIONS ops (reported, not selectable) */
};

typedef struct slc_device slc_device;
typedef struct slc_weight slc_weight;
typedef struct slc_matmul slc_matmul;
typedef struct slc_activation slc_activation;

/* What DeviceInfo needs (src/Sharplight.Core/Runtime/DeviceInfo.cs:4-50). */
typedef struct slc_device_info
{
    char name[256];
    char driver[64];           /* "driver 12090 / runtime 12090" */
    uint8_t uuid[16];          /* the GPU UUID, so the same GPU under two providers is recognised */
    int64_t total_memory;
    int64_t free_memory;
    int32_t sm_count;
    int32_t cc_major;
    int32_t cc_minor;
    int32_t max_shared_per_block;
    int32_t l2_bytes;
    int32_t concurrent_workgroups;  /* SM count x resident CTAs of the mat-vec kernel */
    int32_t supported;              /* 1 when the device can run this library's kernels (compute capability 10.0) */
    int32_t reserved;
} slc_device_info;

/* ---- library: the ABI probe the managed loader performs (cf. src/Sharplight.Audio/Native/NativeAudioLibrary.cs:47-59) */
SLC_API int32_t slc_abi_version(void);
SLC_API const char *slc_version_string(void);
SLC_API const char *slc_error_string(slc_result code);
/* Detail text of the calling thread's most recent failure ("" when none). */
SLC_API const char *slc_last_error_message(void);

/* ---- devices: IExecutionProvider.CheckAvailability / GetDevices / OpenDevice
        (src/Sharplight.Core/Runtime/IExecutionProvider.cs:25-45) */
SLC_API slc_result slc_device_count(int32_t *out_count);
SLC_API slc_result slc_device_info_get(int32_t index, slc_device_info *out);
SLC_API slc_result slc_device_open(int32_t index, slc_device **out);
SLC_API void slc_device_close(slc_device *device);
/* IComputeDevice.AvailableMemory / GetMemoryInfo (src/Sharplight.Core/Runtime/IComputeDevice.cs:12-24). */
SLC_API slc_result slc_device_memory(slc_device *device, int64_t *out_free, int64_t *out_total);
/* Waits for everything queued on the device's own stream: the point where ICompiledSegment.GetOutput may read
   (src/Sharplight.Core/Runtime/ICompiledSegment.cs:11-19). */
SLC_API slc_result slc_device_sync(slc_device *device);
/* The device's own stream as a cudaStream_t, for callers that time or order work on it. */
SLC_API void *slc_device_stream(slc_device *device);
/* Device-side status word (0 = fine; SLC_ERR_TIMEOUT after a bounded wait ran out); reading clears it. */
SLC_API slc_result slc_last_status(slc_device *device, int32_t *out_status);

/* ---- device buffers: boundary values a segment keeps on the device (IDeviceForwardingSegment.TryForwardFrom,
        src/Sharplight.Core/Runtime/IDeviceForwardingSegment.cs:10-18) and staging for SetInput / GetOutput */
SLC_API slc_result slc_buffer_alloc(slc_device *device, int64_t bytes, void **out_device_ptr);
SLC_API void slc_buffer_free(slc_device *device, void *device_ptr);
SLC_API slc_result slc_buffer_upload(slc_device *device, void *device_ptr, const void *host, int64_t bytes);
SLC_API slc_result slc_buffer_download(slc_device *device, void *host, const void *device_ptr, int64_t bytes);
/* Page-locked host staging and asynchronous copies on a stream (NULL = the device's own): what lets a segment's
   Execute return before its outputs have arrived ("Implementations may run asynchronously until an output is read",
   src/Sharplight.Core/Runtime/ICompiledSegment.cs:11-12). direction: 0 host->device, 1 device->host, 2 device->device. */
SLC_API slc_result slc_host_alloc(int64_t bytes, void **out_host_ptr);
SLC_API void slc_host_free(void *host_ptr);
SLC_API slc_result slc_buffer_copy_async(slc_device *device, void *dst, const void *src, int64_t bytes, int32_t direction,
                                         void *stream);
/* A strided device view made dense: dst[z][r][c] = src[z * batch_stride + r * row_stride + c * col_stride] (strides in
   elements of elem_bytes = 2 or 4; dst is [batch][rows][cols], contiguous). slc_matmul_run and slc_activation_quantize take rows that are x_stride apart and start at any element, so a
   Slice or a row-splitting Reshape in front of a MatMul is only a pointer and a stride; a Permute's rows are not
   contiguous and come through here first (src/Sharplight.Shaders/Lowering/GraphLowerer.MatMul.cs:117-126). */
SLC_API slc_result slc_buffer_densify(slc_device *device, void *dst_device, const void *src_device, int64_t batch, int64_t rows,
                                      int64_t cols, int64_t batch_stride, int64_t row_stride, int64_t col_stride,
                                      int32_t elem_bytes, void *stream);

/* ---- side streams and captured step graphs: a segment's Execute captured once per row count and replayed with one
        call, its output copies on a second stream beside the kernels (the CUDA form of a command buffer that is
        recorded once and re-submitted; ICompiledSegment.cs:11-12 allows asynchronous execution until an output is
        read). slc_stream_wait makes `waiter` wait for everything queued so far on `signal` (NULL = the device's own
        stream); between slc_graph_begin and slc_graph_end on a stream, launches and copies issued to it -- and to
        streams made to wait on it, which must be joined back before the end -- are recorded instead of executed. Make
        every call that will be captured once outside a capture first (first launches configure kernels). Errors of
        this group: slc_graph_last_error. */
typedef struct slc_graph slc_graph;
SLC_API slc_result slc_stream_create(slc_device *device, void **out_stream);
SLC_API void slc_stream_destroy(slc_device *device, void *stream);
SLC_API slc_result slc_stream_wait(slc_device *device, void *waiter, void *signal);
SLC_API slc_result slc_graph_begin(slc_device *device, void *stream);
SLC_API slc_result slc_graph_end(slc_device *device, void *stream, slc_graph **out_graph);
SLC_API slc_result slc_graph_launch(slc_graph *graph, void *stream);
SLC_API void slc_graph_destroy(slc_graph *graph);
SLC_API const char *slc_graph_last_error(void);

/* ---- weights: WeightInfo.Source -> device (src/Sharplight.Core/Models/IWeightSource.cs:4-40).
        blocks: raw ggml blocks of an [n, k] weight, row-major, bytes == n * k / block_size * block_bytes.
        The data is copied (the caller may unmap afterwards) and re-laid-out on the device at the same byte count,
        as the reference does for Q8_0 at upload (src/Sharplight.Shaders/Lowering/WeightRepacker.cs:56-69). */
SLC_API slc_result slc_weight_upload(slc_device *device, int32_t format, int64_t n, int64_t k, const void *blocks,
                                     int64_t bytes, slc_weight **out);
/* Like slc_weight_upload but keeps only the K range [k0, k1) of every row (block-aligned): the row-split shard of a
   tensor-parallel o / down projection. */
SLC_API slc_result slc_weight_upload_kslice(slc_device *device, int32_t format, int64_t n, int64_t k,
                                            const void *blocks, int64_t bytes, int64_t k0, int64_t k1,
                                            slc_weight **out);
/* Writes the weight back as raw ggml blocks (inverse of the device layout; for verification). SLC_ERR_UNSUPPORTED for a
   weight that was converted at upload (Q5_0, IQ4_NL, Q5_K). */
SLC_API slc_result slc_weight_download(slc_weight *weight, void *blocks, int64_t bytes);
/* The device layout as an artefact (the reference's providers name artefact tiers a model package may carry for them,
   src/Sharplight.Core/Runtime/IComputeDevice.cs:47-52): export writes a 56-byte header (magic, version, format, shape)
   and the re-laid-out records; import uploads them as they are, without the re-layout pass and without the raw blocks.
   An artefact of another layout version is refused with SLC_ERR_UNSUPPORTED: fall back to slc_weight_upload. */
SLC_API slc_result slc_weight_layout_bytes(slc_weight *weight, int64_t *out_bytes);
SLC_API slc_result slc_weight_export_layout(slc_weight *weight, void *out_host, int64_t bytes);
SLC_API slc_result slc_weight_import_layout(slc_device *device, const void *artefact_host, int64_t bytes, slc_weight **out);
/* Weights straight out of a GGUF file (the reference reads them through IWeightSource.Read after
   src/Sharplight.Import.Gguf/GgufFile.cs has parsed the table): the file is memory-mapped, header / metadata / tensor
   table are parsed with bounds checks (GGUF versions 2 and 3, general.alignment honoured), and a 2-D tensor of one of
   the four served formats goes from the mapping to the device. tensor_info: name (UTF-8, NUL-terminated), ggml type,
   rank, n = dims[1] and k = dims[0] (GGUF stores the innermost dimension first), bytes = size of the raw blocks, or 0
   when slc_weight_upload_gguf would refuse the tensor. Errors: slc_gguf_last_error() (thread-local text). */
typedef struct slc_gguf slc_gguf;
SLC_API slc_result slc_gguf_open(const char *path, slc_gguf **out);
SLC_API void slc_gguf_close(slc_gguf *file);
SLC_API slc_result slc_gguf_tensor_count(slc_gguf *file, int64_t *count);
SLC_API slc_result slc_gguf_tensor_info(slc_gguf *file, int64_t index, char *name_out, int32_t name_capacity, int32_t *format,
                                        int32_t *rank, int64_t *n, int64_t *k, int64_t *bytes);
SLC_API slc_result slc_gguf_find(slc_gguf *file, const char *name, int64_t *index);
SLC_API slc_result slc_weight_upload_gguf(slc_device *device, slc_gguf *file, int64_t index, slc_weight **out);
SLC_API const char *slc_gguf_last_error(void);
SLC_API slc_result slc_weight_shape(slc_weight *weight, int32_t *format, int64_t *n, int64_t *k, int64_t *device_bytes);
SLC_API void slc_weight_free(slc_weight *weight);

/* ---- the operator: StandardOps.MatMul, y = x . W^T (src/Sharplight.Core/Graph/StandardOps.cs:144-163), lowered
        like the CPU provider's MatMulOp on its integer-dot path (src/Sharplight.Cpu/MatMulOp.cs:88-115,174-213) */
SLC_API slc_result slc_matmul_create(slc_device *device, slc_weight *weight, int64_t max_rows, uint32_t flags,
                                     slc_matmul **out);
/* Two weights of one shape that read the same activations and only feed silu(a) * b -- the gate and up projections of
   a gated FFN (the reference's dual MatMul, src/Sharplight.Shaders/Lowering/GraphLowerer.MatMul.cs:128-198). The op
   runs through the same entry points; y receives silu(x . gate^T) * (x . up^T), silu(v) = v / (1 + exp(-v)). For the
   mat-vec row counts it is one launch that streams both weights; above, the two MatMuls and an element-wise kernel. */
SLC_API slc_result slc_matmul_create_dual(slc_device *device, slc_weight *gate, slc_weight *up, int64_t max_rows,
                                          uint32_t flags, slc_matmul **out);
SLC_API void slc_matmul_destroy(slc_matmul *op);
/*
 * y[rows][n] (f32, row stride y_stride elements) = x[rows][k] . W^T. x rows are x_stride elements apart.
 * x_is_device / y_is_device: 0 = host memory (copied through the op's staging buffers on the stream, the call
 * returns after the result is in y), 1 = device memory (asynchronous on the stream).
 * stream: a cudaStream_t, or NULL for the device's own stream.
 * rows == 0 is a no-op; rows > max_rows fails with SLC_ERR_INVALID_STATE.
 */
SLC_API slc_result slc_matmul_run(slc_matmul *op, const void *x, int32_t x_dtype, int64_t rows, int64_t x_stride,
                                  int32_t x_is_device, float *y, int64_t y_stride, int32_t y_is_device,
                                  void *stream);
/* Forces a kernel family (SLC_KERNEL_*) for later runs; SLC_KERNEL_AUTO restores the row-count dispatch. */
SLC_API slc_result slc_matmul_set_kernel(slc_matmul *op, int32_t kernel);
/* The family the most recent run used, and the number of kernels it launched. */
SLC_API slc_result slc_matmul_last_kernel(slc_matmul *op, int32_t *out_kernel, int32_t *out_launches);

/* ---- shared quantized activations: one 8-bit copy of x serves every MatMul reading the same rows (Q/K/V, gate/up),
        as the reference's lowering shares it (src/Sharplight.Shaders/Lowering/GraphLowerer.IntDot.cs:38-43) */
SLC_API slc_result slc_activation_create(slc_device *device, int64_t max_rows, int64_t k, slc_activation **out);
SLC_API void slc_activation_destroy(slc_activation *act);
/* Quantizes device-resident x (rows x k, x_stride elements apart) per 32 values: d = max|x| / 127, round half away
   from zero (src/Sharplight.Cpu/IntDot.cs:92-126). Asynchronous on the stream. */
SLC_API slc_result slc_activation_quantize(slc_activation *act, const void *x_device, int32_t x_dtype, int64_t rows,
                                           int64_t x_stride, void *stream);
/* Deferred quantization: the rows are handed over as they are (device, f32 or bf16) and quantized when the first MatMul
   that reads them runs -- inside that MatMul's kernel when it is a mat-vec (up to 4 rows per launch) over a short K
   (K <= 2048: a tensor-parallel shard; one launch and one boundary on the dependent chain less), by the quantizer
   kernel on that MatMul's stream otherwise. x must stay unchanged until the MatMuls that read it have run. Results are
   bit-identical to slc_activation_quantize followed by the same MatMul. */
SLC_API slc_result slc_activation_set_rows(slc_activation *act, const void *x_device, int32_t x_dtype, int64_t rows,
                                           int64_t x_stride, void *stream);
/* Producers: the operation in front of a MatMul writes the 8-bit activations itself, in the same pass (the reference
   lets its norm kernels write the copy the next MatMul reads, src/Sharplight.Shaders/Lowering/GraphLowerer.IntDot.cs:146-184).
   Both fill `act` exactly as slc_activation_quantize would from the f32 values they compute; y (optional, device) also
   receives those f32 values (the residual stream needs the norm's input, not its output, so y is usually null).
   rmsnorm: v = (x * 1 / sqrt(sum x^2 / K + eps)) * weight (src/Sharplight.Cpu/RowOp.cs:63-76), weight f32 [K] or null.
   silu_mul: v = silu(gate) * up, silu(g) = g / (1 + exp(-g)) (src/Sharplight.Cpu/ScalarMath.cs:552-577): the gated-FFN
   tail in front of the down projection; gate and up may be the two halves of one stacked gate/up output (strides). */
SLC_API slc_result slc_activation_quantize_rmsnorm(slc_activation *act, const void *x_device, int32_t x_dtype, int64_t rows,
                                                   int64_t x_stride, const float *weight_device, float eps,
                                                   float *y_device, int64_t y_stride, void *stream);
SLC_API slc_result slc_activation_quantize_silu_mul(slc_activation *act, const float *gate_device, int64_t gate_stride,
                                                    const float *up_device, int64_t up_stride, int64_t rows,
                                                    float *y_device, int64_t y_stride, void *stream);
/* The sampling head behind the lm_head MatMul: out_index_device[t] = index of the first maximum of row t of y (NaN never
   beats a number; src/Sharplight.Cpu/RowOp.cs:174-189), so one int32 per sequence leaves the device instead of the row
   of logits. */
SLC_API slc_result slc_argmax_rows(slc_device *device, const float *y_device, int64_t rows, int64_t n, int64_t y_stride,
                                   int32_t *out_index_device, void *stream);

/* ---- MatMulId, the expert-indexed MatMul of mixture-of-experts layers (src/Sharplight.Core/Graph/StandardOps.Moe.cs:8-40):
        y[t, s] = W[ids[t, s]] . x[t]   (per_slot == 0, x: [tokens, K])   or   W[ids[t, s]] . x[t, s]   (per_slot != 0,
        x: [tokens * slots, K]). weight: the experts' [N, K] matrices uploaded as one [experts * N, K] weight, N a multiple
        of 16; ids: device int32 [tokens * slots]; y: device f32, tokens * slots rows of N values, y_stride apart. The
        arithmetic is the reference CPU operator's (src/Sharplight.Cpu/MatMulIdOp.cs): f32 activations against the
        dequantized weight, every item computed as a single row is. An id outside [0, experts) leaves its row untouched
        and raises the device status word (slc_last_status: -1), where the reference throws. Asynchronous on the stream. */
SLC_API slc_result slc_matmul_id_run(slc_weight *weight, int32_t experts, const void *x_device, int32_t x_dtype, int64_t x_stride,
                                     const int32_t *ids_device, int64_t tokens, int64_t slots, int32_t per_slot,
                                     float *y_device, int64_t y_stride, void *stream);

/* y (device, f32) = act . W^T with the rows last quantized into act. Asynchronous on the stream. Consecutive calls that
   read the same quantized rows may execute side by side on the device: their outputs must not overlap in memory. */
SLC_API slc_result slc_matmul_run_quantized(slc_matmul *op, slc_activation *act, float *y_device, int64_t y_stride,
                                            void *stream);

/* The MatMul with the elementwise tail the reference's lowering folds into the kernel
   (src/Sharplight.Shaders/Lowering/GraphLowerer.MatMul.cs:199-243, MatMulEpilogue): y[t][n] = (act . W^T + bias[n]) +
   residual[t][n], f32 adds in that order -- the sums the separate Add nodes would give, one launch and one dependency
   level less. bias (device, f32 [N]) and residual (device, f32, rows residual_stride apart, may be y itself) are each
   optional; exchange (optional) as in slc_matmul_run_quantized_allreduce below: the additions then follow the sum over
   the ranks. */
typedef struct slc_tp_exchange slc_tp_exchange;
SLC_API slc_result slc_matmul_run_quantized_epilogue(slc_matmul *op, slc_activation *act, slc_tp_exchange *exchange,
                                                     const float *bias_device, const float *residual_device,
                                                     int64_t residual_stride, float *y_device, int64_t y_stride,
                                                     void *stream);

/* ---- tensor parallelism: the reference has none (its multi-device story is layer placement,
        src/Sharplight.Core/Runtime/PlacementPlanner.cs:7-13), so these entry points have no counterpart there. One
        process per GPU. A row-split MatMul (o, down) leaves every rank with a partial output; with an exchange the
        MatMul kernel itself sums the partial outputs of all ranks, through receive areas that the ranks map into each
        other's address space (CUDA IPC, plain peer stores over NVLink, bounded waits), and y receives the total, the
        bit-identical value on every rank. For up to SLC_TP_MAX_ROWS rows per call; larger row counts go through
        the communicator below (slc_tp_exchange_set_comm), or slc_matmul_run_quantized and the caller's all-reduce.
        Set-up: every rank creates its exchange (same world, max_rows, n everywhere) and gets a 64-byte handle; the
        host exchanges the handles by any means and passes all of them, in rank order, to connect. All ranks must
        issue the same sequence of allreduce calls on an exchange. A peer that never arrives (it died, or its stream is
        stuck) ends the wait after about a second: the call's kernel raises the device status to SLC_ERR_TIMEOUT
        (slc_last_status) and y is not meaningful. The device and every other handle stay usable after that, the
        exchange itself does not: the ranks' call counts no longer agree (the rank that gave up counted its call, the
        one that never launched did not), so every later call on it would time out as well. Destroy it on all ranks
        and create and connect a new one. Destroy only when no rank has a launch in flight. */
#define SLC_TP_MAX_RANKS 8
#define SLC_TP_MAX_ROWS 64
#define SLC_TP_HANDLE_BYTES 64
SLC_API slc_result slc_tp_exchange_create(slc_device *device, int32_t rank, int32_t world, int64_t max_rows, int64_t n,
                                          slc_tp_exchange **out, uint8_t *out_handle /* [SLC_TP_HANDLE_BYTES] */);
SLC_API slc_result slc_tp_exchange_connect(slc_tp_exchange *exchange, const uint8_t *handles /* [world][64] */);
SLC_API void slc_tp_exchange_destroy(slc_tp_exchange *exchange);
/* How long a kernel waits for its peers before it gives up (default 1000 ms; 1..60000). */
SLC_API slc_result slc_tp_exchange_set_wait_ms(slc_tp_exchange *exchange, int32_t milliseconds);
/* The collective-library route for row counts the in-kernel sum does not serve. NCCL is loaded at run time
   (libnccl.so.2; the copy already in the process, if there is one): without it these calls fail with
   SLC_ERR_UNSUPPORTED and everything else works. Rank 0 obtains an id (slc_tp_comm_unique_id), the host hands it to all
   ranks, every rank creates its communicator (a collective call: all ranks at the same time). Attached to an exchange,
   it takes the sums of calls with more than in_kernel_rows rows (default 16: below that the in-kernel sum is faster)
   or more than the exchange's max_rows: plain MatMul, ncclAllReduce in place on y, then bias / residual if given.
   comm = null detaches. Destroy the communicator only when no rank has a launch in flight. */
#define SLC_TP_COMM_ID_BYTES 128
typedef struct slc_tp_comm slc_tp_comm;
SLC_API slc_result slc_tp_comm_unique_id(uint8_t *out_id /* [SLC_TP_COMM_ID_BYTES] */);
SLC_API slc_result slc_tp_comm_create(slc_device *device, int32_t rank, int32_t world,
                                      const uint8_t *id /* [SLC_TP_COMM_ID_BYTES] */, slc_tp_comm **out);
SLC_API void slc_tp_comm_destroy(slc_tp_comm *comm);
SLC_API slc_result slc_tp_exchange_set_comm(slc_tp_exchange *exchange, slc_tp_comm *comm, int32_t in_kernel_rows);
/* Option: prefill-sized sums (GEMM kernel family, at least min_rows rows) run in four chunks of rows, the all-reduce of
   one chunk beside the GEMM of the next (the communicator's own stream, joined back into the call's stream at the end).
   Off by default (min_rows = 0): on 2 and 4 B200 it measured 2-4 % slower than the sum after the GEMM. */
SLC_API slc_result slc_tp_comm_set_chunking(slc_tp_comm *comm, int32_t min_rows);
/* y (device, f32) = sum over ranks of (act . W^T), W being this rank's K range of the weight and act this rank's
   matching slice of the activations. Asynchronous on the stream. */
/* The same with x not yet quantized (device, rows x k): slc_matmul_run with the sum over the ranks. */
SLC_API slc_result slc_matmul_run_allreduce(slc_matmul *op, slc_tp_exchange *exchange, const void *x_device, int32_t x_dtype,
                                            int64_t rows, int64_t x_stride, float *y_device, int64_t y_stride, void *stream);
SLC_API slc_result slc_matmul_run_quantized_allreduce(slc_matmul *op, slc_activation *act, slc_tp_exchange *exchange,
                                                      float *y_device, int64_t y_stride, void *stream);

/* ---- no device allocation: this entry point has no counterpart in the reference. It serves hosts that may not call
        cudaMalloc while they run (a serving loop with a fixed memory budget, a framework that owns the allocator, a
        phase where an allocation would stall the device). Same result as slc_matmul_run with device pointers, for
        1..4 rows and K <= 32768, but the quantized activations go to a fixed SLC_STATIC_SCRATCH_BYTES array inside the
        library's device image (held by every GPU that loads the library until exit) instead of allocated planes.
        Limits are rejected with SLC_ERR_UNSUPPORTED (text: slc_static_last_error). All calls on a device share the
        array: calls that overlap on the GPU race, serialise them. The first call on a device resolves the array's
        address and should happen before any stream capture begins. x and y are device memory; asynchronous on the
        stream (NULL = the device's own). */
#define SLC_STATIC_SCRATCH_BYTES 491520
SLC_API slc_result slc_matmul_run_static(slc_weight *weight, const void *x_device, int32_t x_dtype, int64_t rows,
                                         int64_t x_stride, float *y_device, int64_t y_stride, void *stream);
SLC_API const char *slc_static_last_error(void);

/* ---- parity exports (host buffers; synchronous): the quantities the bit-exactness checks compare */
/* q[rows][k] int8, d[rows][k/32] f32 block scales, gs[rows][k/16] f32 group sums d * sum16(q), as IntDot.Quantize
   lays them out logically (src/Sharplight.Cpu/Q8Row.cs:9-20). x is host memory. */
SLC_API slc_result slc_debug_quantize(slc_device *device, const void *x, int32_t x_dtype, int64_t rows, int64_t k,
                                      int8_t *q, float *d, float *gs);
/* s32[rows][n][k/32]: per 32-value block, the int32 dot of the CPU decoder's unsigned weight codes
   (src/Sharplight.Cpu/IntDot.Decode.cs:70-99,125-148,189-223) with the activation codes, computed by the kernel
   family the op would run for this row count. x is host memory. */
SLC_API slc_result slc_debug_block_dots(slc_matmul *op, const void *x, int32_t x_dtype, int64_t rows, int32_t *s32);

#ifdef __cplusplus
}
#endif
#endif
