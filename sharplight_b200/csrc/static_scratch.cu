// slc_matmul_run_static: the decode MatMul for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: inside a latency-critical serving loop whose memory
// was budgeted up front, under a framework that owns the device allocator and forbids side allocations, or during
// phases in which any allocation would synchronise the device. The ordinary entry points create their quantized
// activation planes with cudaMalloc (once, at first use). This one never allocates: the planes live in a fixed array
// in the library's device image, so every GPU that loads the library pays SLC_STATIC_SCRATCH_BYTES (480 KB) until the
// process exits, whether the entry point is used or not.
//
// Limits, checked with a clear error: 1..4 activation rows, K up to 32768 (after padding to a multiple of 256). Where
// K is too long for the kernel to hold four rows of activations in shared memory (beyond 24576), the rows go in two
// launches on the same scratch, as the ordinary path does.
// The array is shared by every call on a device and keeps the previous call's contents; each call rewrites all of what
// its kernels read (the quantizer writes every padded row and block), so nothing needs clearing, but two calls that
// overlap on the GPU (different streams, or the same weight from two threads) race on it: serialise them.
// The first call on a device looks the array's device address up (cudaGetSymbolAddress, with that device current) and
// sets one kernel attribute; make that first call before starting any stream capture.
#include "../../include/sharplight_cuda.h"

#include "handles.cuh"

#include <atomic>
#include <string>

using namespace slc;

namespace {

constexpr int NA_MAX_ROWS = 4;          // the dp4a mat-vec kernel takes up to four rows per launch
constexpr int NA_ROWS_PAD = 8;
constexpr int NA_MAX_KPAD = 32768;
constexpr size_t NA_Q = (size_t)NA_ROWS_PAD * NA_MAX_KPAD;              // int8 codes
constexpr size_t NA_DS = (size_t)(NA_MAX_KPAD / 32) * NA_ROWS_PAD * 8;  // (d, d * sum q)
constexpr size_t NA_DX = NA_DS / 2, NA_SX = NA_DS / 2;
constexpr size_t NA_GS = (size_t)NA_ROWS_PAD * (NA_MAX_KPAD / 16) * 4;
constexpr size_t NA_IS = (size_t)NA_ROWS_PAD * (NA_MAX_KPAD / 32) * 4;
constexpr size_t NA_TOTAL = NA_Q + NA_DS + NA_DX + NA_SX + NA_GS + NA_IS;
static_assert(NA_TOTAL == SLC_STATIC_SCRATCH_BYTES, "header and implementation disagree on the scratch size");

// The scratch itself. In host code this name is only a stand-in for the symbol, not a device address: the address
// comes from cudaGetSymbolAddress below and only that pointer is ever handed to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[NA_TOTAL];

// per device, filled at first use; two host threads that race here both look the same address up and store the same value
std::atomic<unsigned char *> g_scratch_ptr[64];

thread_local std::string t_static_error;

slc_result na_fail(slc_result code, const std::string &msg)
{
    t_static_error = msg;
    return code;
}

}  // namespace

extern "C" {

const char *slc_static_last_error(void) { return t_static_error.c_str(); }

slc_result slc_matmul_run_static(slc_weight *weight, const void *x_device, int32_t x_dtype, int64_t rows, int64_t x_stride,
                                 float *y_device, int64_t y_stride, void *stream)
{
    if (!weight) return na_fail(SLC_ERR_INVALID_ARGUMENT, "weight is null");
    if (x_dtype != SLC_F32 && x_dtype != SLC_BF16) return na_fail(SLC_ERR_UNSUPPORTED, "activation dtype must be f32 or bf16");
    if (rows < 0) return na_fail(SLC_ERR_INVALID_ARGUMENT, "rows < 0");
    if (rows == 0 || weight->n == 0) return SLC_OK;
    if (rows > NA_MAX_ROWS) return na_fail(SLC_ERR_UNSUPPORTED, "slc_matmul_run_static takes at most 4 activation rows");
    const WeightView &wv = weight->view;
    if (wv.k_pad > NA_MAX_KPAD || !matvec_fits(1, wv.k_pad)) {
        return na_fail(SLC_ERR_UNSUPPORTED, "slc_matmul_run_static: K exceeds the static scratch (32768 values)");
    }
    if (!x_device || x_stride < weight->k) return na_fail(SLC_ERR_INVALID_ARGUMENT, "bad activation pointer or stride");
    if (!y_device || y_stride < weight->n) return na_fail(SLC_ERR_INVALID_ARGUMENT, "bad output pointer or stride");
    slc_device *dev = weight->dev;
    if (dev->index < 0 || dev->index >= 64) return na_fail(SLC_ERR_UNSUPPORTED, "device index out of range");
    cudaError_t e = cudaSetDevice(dev->index);
    if (e != cudaSuccess) return na_fail(SLC_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(e));

    // set-up, once per device, with that device current: the symbol's address on this device
    unsigned char *base = g_scratch_ptr[dev->index].load(std::memory_order_acquire);
    if (!base) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) {
            return na_fail(SLC_ERR_CUDA, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        }
        base = static_cast<unsigned char *>(p);
        g_scratch_ptr[dev->index].store(base, std::memory_order_release);
    }

    const int k_pad = wv.k_pad;
    ActPlanes planes;
    planes.q_tiled = nullptr;
    planes.q_sw = nullptr;
    planes.sx2 = nullptr;
    planes.q = reinterpret_cast<int8_t *>(base);
    planes.ds = reinterpret_cast<float2 *>(base + NA_Q);
    planes.dx = reinterpret_cast<float *>(base + NA_Q + NA_DS);
    planes.sx = reinterpret_cast<float *>(base + NA_Q + NA_DS + NA_DX);
    planes.gs = reinterpret_cast<float *>(base + NA_Q + NA_DS + NA_DX + NA_SX);
    planes.isum = reinterpret_cast<int *>(base + NA_Q + NA_DS + NA_DX + NA_SX + NA_GS);

    cudaStream_t s = stream ? (cudaStream_t)stream : dev->stream;
    e = launch_quantize(x_device, x_dtype, (int)rows, NA_ROWS_PAD, (int)weight->k, k_pad, x_stride, planes, s);
    if (e != cudaSuccess) return na_fail(SLC_ERR_CUDA, std::string("quantize: ") + cudaGetErrorString(e));
    ActView av;
    av.rows = (int)rows; av.rows_pad = NA_ROWS_PAD; av.k = (int)weight->k; av.k_pad = k_pad;
    av.q = planes.q; av.ds = planes.ds; av.dx = planes.dx; av.sx = planes.sx; av.gs = planes.gs; av.isum = planes.isum;
    // the largest chunk of rows whose activations fit the kernel's shared memory at this K (every row of a chunk is
    // computed exactly as a single row is, so the chunking does not change the result)
    // (a Q5_K weight is two Q4_K weights: both stream through one launch of the kernel's two-weight form, products added)
    const WeightView *second = weight->high ? &weight->high->view : nullptr;
    if (second && !matvec_fits(1, k_pad, true)) return na_fail(SLC_ERR_UNSUPPORTED, "slc_matmul_run_static: K of this Q5_K weight exceeds the two-weight mat-vec's shared memory");
    int chunk = (int)rows;
    while (chunk > 1 && !matvec_fits(chunk, k_pad, second != nullptr)) chunk--;
    for (int r0 = 0; r0 < (int)rows; r0 += chunk) {
        const int m = (int)rows - r0 < chunk ? (int)rows - r0 : chunk;
        e = launch_matvec(wv, av, r0, m, y_device, y_stride, nullptr, dev->status_dev, r0 > 0 ? 1 : 0, s, nullptr, nullptr, second);
        if (e != cudaSuccess) return na_fail(SLC_ERR_CUDA, std::string("mat-vec: ") + cudaGetErrorString(e));
    }
    return SLC_OK;
}

}  // extern "C"
