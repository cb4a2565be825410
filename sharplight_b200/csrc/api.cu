// The C ABI of libsharplight_cuda (include/sharplight_cuda.h): handles, argument checks, kernel dispatch.
// No CPU fallback lives here: every compute entry point needs a CUDA device and fails loudly without one.
#include "../../include/sharplight_cuda.h"

#include "internal.cuh"

#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

using namespace slc;

#include "handles.cuh"

// ---- errors ----------------------------------------------------------------------------------------------------------

static thread_local std::string t_last_error;

static slc_result fail(slc_result code, const std::string &msg)
{
    t_last_error = msg;
    return code;
}

static slc_result cuda_fail(cudaError_t e, const char *what)
{
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return fail(SLC_ERR_OUT_OF_MEMORY, std::string(what) + ": out of device memory");
    }
    if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) {
        cudaGetLastError();
        return fail(SLC_ERR_NO_DEVICE, std::string(what) + ": " + cudaGetErrorString(e));
    }
    return fail(SLC_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

#define SLC_CUDA(call)                                          \
    do {                                                        \
        cudaError_t e_ = (call);                                \
        if (e_ != cudaSuccess) return cuda_fail(e_, #call);     \
    } while (0)

// Rows are padded so that every token tile a kernel touches exists: 16, 32, 64, then multiples of 128.
static int pad_rows(long long rows)
{
    if (rows <= 16) return 16;
    if (rows <= 32) return 32;
    if (rows <= 64) return 64;
    return (int)((rows + 127) / 128 * 128);
}

extern "C" {

int32_t slc_abi_version(void) { return SLC_ABI_VERSION; }

const char *slc_version_string(void) { return "libsharplight_cuda 0.1 (sm_100a)"; }

const char *slc_error_string(slc_result code)
{
    switch (code) {
    case SLC_OK: return "ok";
    case SLC_ERR_INVALID_ARGUMENT: return "invalid argument";
    case SLC_ERR_OUT_OF_MEMORY: return "out of memory";
    case SLC_ERR_NO_DEVICE: return "no usable CUDA device";
    case SLC_ERR_UNSUPPORTED: return "unsupported format or shape";
    case SLC_ERR_CUDA: return "CUDA runtime error";
    case SLC_ERR_INVALID_STATE: return "invalid state";
    case SLC_ERR_TIMEOUT: return "device-side wait timed out";
    case SLC_ERR_BUFFER_TOO_SMALL: return "buffer too small";
    default: return "unknown error";
    }
}

const char *slc_last_error_message(void) { return t_last_error.c_str(); }

// ---- devices ---------------------------------------------------------------------------------------------------------

slc_result slc_device_count(int32_t *out_count)
{
    if (!out_count) return fail(SLC_ERR_INVALID_ARGUMENT, "out_count is null");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        *out_count = 0;
        return fail(SLC_ERR_NO_DEVICE, std::string("cudaGetDeviceCount: ") + cudaGetErrorString(e));
    }
    *out_count = n;
    return SLC_OK;
}

slc_result slc_device_info_get(int32_t index, slc_device_info *out)
{
    if (!out) return fail(SLC_ERR_INVALID_ARGUMENT, "out is null");
    int32_t n = 0;
    slc_result r = slc_device_count(&n);
    if (r != SLC_OK) return r;
    if (index < 0 || index >= n) return fail(SLC_ERR_INVALID_ARGUMENT, "device index out of range");
    cudaDeviceProp p;
    SLC_CUDA(cudaGetDeviceProperties(&p, index));
    memset(out, 0, sizeof(*out));
    snprintf(out->name, sizeof(out->name), "%s", p.name);
    int drv = 0, rt = 0;
    cudaDriverGetVersion(&drv);
    cudaRuntimeGetVersion(&rt);
    snprintf(out->driver, sizeof(out->driver), "driver %d / runtime %d", drv, rt);
    memcpy(out->uuid, p.uuid.bytes, 16);
    out->total_memory = (int64_t)p.totalGlobalMem;
    out->sm_count = p.multiProcessorCount;
    out->cc_major = p.major;
    out->cc_minor = p.minor;
    out->max_shared_per_block = (int32_t)p.sharedMemPerBlockOptin;
    out->l2_bytes = p.l2CacheSize;
    out->concurrent_workgroups = p.multiProcessorCount * 16;
    out->supported = (p.major == 10 && p.minor == 0) ? 1 : 0;
    size_t fr = 0, tot = 0;
    int prev = 0;
    cudaGetDevice(&prev);
    if (cudaSetDevice(index) == cudaSuccess && cudaMemGetInfo(&fr, &tot) == cudaSuccess) out->free_memory = (int64_t)fr;
    cudaSetDevice(prev);
    return SLC_OK;
}

slc_result slc_device_open(int32_t index, slc_device **out)
{
    if (!out) return fail(SLC_ERR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    int32_t n = 0;
    slc_result r = slc_device_count(&n);
    if (r != SLC_OK) return r;
    if (index < 0 || index >= n) return fail(SLC_ERR_INVALID_ARGUMENT, "device index out of range");
    slc_device *d = new (std::nothrow) slc_device();
    if (!d) return fail(SLC_ERR_OUT_OF_MEMORY, "host allocation failed");
    d->index = index;
    cudaError_t e = cudaGetDeviceProperties(&d->prop, index);
    if (e == cudaSuccess && !(d->prop.major == 10 && d->prop.minor == 0)) {
        delete d;
        return fail(SLC_ERR_NO_DEVICE, "device is not compute capability 10.0 (sm_100a kernels only)");
    }
    if (e == cudaSuccess) e = cudaSetDevice(index);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&d->status_dev, 256);
    if (e == cudaSuccess) e = cudaMemset(d->status_dev, 0, 256);
    if (e != cudaSuccess) {
        if (d->stream) cudaStreamDestroy(d->stream);
        if (d->status_dev) cudaFree(d->status_dev);
        delete d;
        return cuda_fail(e, "slc_device_open");
    }
    *out = d;
    return SLC_OK;
}

void slc_device_close(slc_device *d)
{
    if (!d) return;
    cudaSetDevice(d->index);
    cudaStreamSynchronize(d->stream);
    for (cudaEvent_t ev : d->events) cudaEventDestroy(ev);
    cudaStreamDestroy(d->stream);
    cudaFree(d->status_dev);
    delete d;
}

slc_result slc_device_memory(slc_device *d, int64_t *out_free, int64_t *out_total)
{
    if (!d) return fail(SLC_ERR_INVALID_ARGUMENT, "device is null");
    SLC_CUDA(cudaSetDevice(d->index));
    size_t fr = 0, tot = 0;
    SLC_CUDA(cudaMemGetInfo(&fr, &tot));
    if (out_free) *out_free = (int64_t)fr;
    if (out_total) *out_total = (int64_t)tot;
    return SLC_OK;
}

slc_result slc_device_sync(slc_device *d)
{
    if (!d) return fail(SLC_ERR_INVALID_ARGUMENT, "device is null");
    SLC_CUDA(cudaSetDevice(d->index));
    SLC_CUDA(cudaStreamSynchronize(d->stream));
    return SLC_OK;
}

void *slc_device_stream(slc_device *d) { return d ? (void *)d->stream : nullptr; }

slc_result slc_last_status(slc_device *d, int32_t *out_status)
{
    if (!d || !out_status) return fail(SLC_ERR_INVALID_ARGUMENT, "null argument");
    SLC_CUDA(cudaSetDevice(d->index));
    int v = 0;
    SLC_CUDA(cudaMemcpy(&v, d->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
    if (v != 0) SLC_CUDA(cudaMemset(d->status_dev, 0, sizeof(int)));
    *out_status = v;
    return SLC_OK;
}

// ---- buffers ---------------------------------------------------------------------------------------------------------

slc_result slc_buffer_alloc(slc_device *d, int64_t bytes, void **out)
{
    if (!d || !out || bytes < 0) return fail(SLC_ERR_INVALID_ARGUMENT, "bad buffer request");
    *out = nullptr;
    SLC_CUDA(cudaSetDevice(d->index));
    SLC_CUDA(cudaMalloc(out, bytes > 0 ? (size_t)bytes : 16));
    return SLC_OK;
}

void slc_buffer_free(slc_device *d, void *p)
{
    if (!d || !p) return;
    cudaSetDevice(d->index);
    cudaFree(p);
}

slc_result slc_buffer_upload(slc_device *d, void *dst, const void *host, int64_t bytes)
{
    if (!d || bytes < 0 || (bytes > 0 && (!dst || !host))) return fail(SLC_ERR_INVALID_ARGUMENT, "bad upload");
    if (bytes == 0) return SLC_OK;
    SLC_CUDA(cudaSetDevice(d->index));
    SLC_CUDA(cudaMemcpyAsync(dst, host, (size_t)bytes, cudaMemcpyHostToDevice, d->stream));
    SLC_CUDA(cudaStreamSynchronize(d->stream));
    return SLC_OK;
}

slc_result slc_buffer_download(slc_device *d, void *host, const void *src, int64_t bytes)
{
    if (!d || bytes < 0 || (bytes > 0 && (!src || !host))) return fail(SLC_ERR_INVALID_ARGUMENT, "bad download");
    if (bytes == 0) return SLC_OK;
    SLC_CUDA(cudaSetDevice(d->index));
    SLC_CUDA(cudaMemcpyAsync(host, src, (size_t)bytes, cudaMemcpyDeviceToHost, d->stream));
    SLC_CUDA(cudaStreamSynchronize(d->stream));
    return SLC_OK;
}

slc_result slc_host_alloc(int64_t bytes, void **out)
{
    if (!out || bytes < 0) return fail(SLC_ERR_INVALID_ARGUMENT, "bad host allocation request");
    *out = nullptr;
    SLC_CUDA(cudaHostAlloc(out, bytes > 0 ? (size_t)bytes : 16, cudaHostAllocDefault));
    return SLC_OK;
}

void slc_host_free(void *p)
{
    if (p) cudaFreeHost(p);
}

slc_result slc_buffer_copy_async(slc_device *d, void *dst, const void *src, int64_t bytes, int32_t direction, void *stream)
{
    if (!d || bytes < 0 || direction < 0 || direction > 2) return fail(SLC_ERR_INVALID_ARGUMENT, "bad copy request");
    if (bytes == 0) return SLC_OK;
    if (!dst || !src) return fail(SLC_ERR_INVALID_ARGUMENT, "null copy pointer");
    SLC_CUDA(cudaSetDevice(d->index));
    const cudaMemcpyKind kind = direction == 0 ? cudaMemcpyHostToDevice : direction == 1 ? cudaMemcpyDeviceToHost
                                                                                         : cudaMemcpyDeviceToDevice;
    SLC_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, kind, stream ? (cudaStream_t)stream : d->stream));
    return SLC_OK;
}

slc_result slc_buffer_densify(slc_device *d, void *dst, const void *src, int64_t batch, int64_t rows, int64_t cols,
                              int64_t batch_stride, int64_t row_stride, int64_t col_stride, int32_t elem_bytes, void *stream)
{
    if (!d || batch < 0 || batch > 65535 || rows < 0 || cols < 0 || rows > (1 << 24) || cols > (1 << 30)) {
        return fail(SLC_ERR_INVALID_ARGUMENT, "bad densify request (batch <= 65535)");
    }
    if (elem_bytes != 2 && elem_bytes != 4) return fail(SLC_ERR_UNSUPPORTED, "elements of 2 or 4 bytes");
    if (batch == 0 || rows == 0 || cols == 0) return SLC_OK;
    if (!dst || !src || batch_stride < 0 || row_stride < 0 || col_stride < 0) return fail(SLC_ERR_INVALID_ARGUMENT, "null pointer or negative stride");
    SLC_CUDA(cudaSetDevice(d->index));
    SLC_CUDA(launch_densify(dst, src, (int)batch, (int)rows, (int)cols, batch_stride, row_stride, col_stride, elem_bytes,
                            stream ? (cudaStream_t)stream : d->stream));
    return SLC_OK;
}

// ---- weights ---------------------------------------------------------------------------------------------------------

static slc_result check_weight_args(slc_device *d, int32_t fmt, int64_t n, int64_t k, const void *blocks, int64_t bytes)
{
    if (!d) return fail(SLC_ERR_INVALID_ARGUMENT, "device is null");
    const int bs = source_block_size(fmt);
    if (bs == 0) return fail(SLC_ERR_UNSUPPORTED, "weight format is not one of Q4_0, Q8_0, Q4_K, Q6_K, Q5_0, Q5_K, IQ4_NL");
    if (n < 0 || k <= 0) return fail(SLC_ERR_INVALID_ARGUMENT, "bad weight shape");
    if (k % bs != 0) {
        char msg[96];
        snprintf(msg, sizeof(msg), "K=%lld is not a multiple of the block size %d", (long long)k, bs);
        return fail(SLC_ERR_INVALID_ARGUMENT, msg);
    }
    if (n > (1 << 30) || k > (1 << 30)) return fail(SLC_ERR_UNSUPPORTED, "weight dimension too large");
    if (bytes != n * (k / bs) * source_block_bytes(fmt)) return fail(SLC_ERR_INVALID_ARGUMENT, "bytes != n * k / block_size * block_bytes");
    if (bytes > 0 && !blocks) return fail(SLC_ERR_INVALID_ARGUMENT, "blocks is null");
    return SLC_OK;
}

// A device weight of a format the kernels serve, from raw blocks of that format already on the device (no synchronize).
static cudaError_t weight_from_device_blocks(slc_device *d, int dev_fmt, int src_fmt, long long n, long long k, uint8_t *raw,
                                             slc_weight **out)
{
    *out = nullptr;
    slc_weight *w = new (std::nothrow) slc_weight();
    if (!w) return cudaErrorMemoryAllocation;
    w->dev = d; w->fmt = dev_fmt; w->src_fmt = src_fmt; w->n = n; w->k = k;
    const int n_pad = (int)round_up((size_t)n, 16), k_pad = (int)round_up((size_t)k, 256);
    w->bytes = round_up(weight_bytes(dev_fmt, n_pad, k_pad), 256) + 256;
    cudaError_t e = cudaMalloc(&w->base, w->bytes);
    if (e == cudaSuccess) e = launch_repack(dev_fmt, (int)n, (int)k, n_pad, k_pad, raw, w->base, false, d->stream);
    if (e != cudaSuccess) {
        if (w->base) cudaFree(w->base);
        delete w;
        return e;
    }
    w->view.fmt = dev_fmt; w->view.n = (int)n; w->view.k = (int)k; w->view.n_pad = n_pad; w->view.k_pad = k_pad;
    w->view.data = w->base;
    *out = w;
    return cudaSuccess;
}

slc_result slc_weight_upload(slc_device *d, int32_t fmt, int64_t n, int64_t k, const void *blocks, int64_t bytes,
                             slc_weight **out)
{
    if (!out) return fail(SLC_ERR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    slc_result r = check_weight_args(d, fmt, n, k, blocks, bytes);
    if (r != SLC_OK) return r;
    SLC_CUDA(cudaSetDevice(d->index));
    // Q5_0 and IQ4_NL are rewritten as Q8_0 blocks on the device first, Q5_K is split into two Q4_K weights (both exactly;
    // layout.cuh): the kernels only ever see the four formats they have decoders for
    const int dev_fmt = device_format(fmt);
    const long long src_blocks = n * (k / source_block_size(fmt));
    const size_t dev_raw_bytes = (size_t)src_blocks * block_bytes(dev_fmt);
    uint8_t *raw = nullptr, *conv = nullptr, *conv2 = nullptr;
    int *overflow = nullptr;
    slc_weight *w = nullptr, *high = nullptr;
    int overflowed = 0;
    cudaError_t e = cudaSuccess;
    if (bytes > 0) e = cudaMalloc(&raw, (size_t)bytes);
    if (e == cudaSuccess && bytes > 0) e = cudaMemcpyAsync(raw, blocks, (size_t)bytes, cudaMemcpyHostToDevice, d->stream);
    if (e == cudaSuccess && bytes > 0 && dev_fmt != fmt) {
        e = cudaMalloc(&conv, dev_raw_bytes);
        if (e == cudaSuccess && fmt == FMT_Q5_K) {
            e = cudaMalloc(&conv2, dev_raw_bytes);
            if (e == cudaSuccess) e = cudaMalloc(&overflow, sizeof(int));
            if (e == cudaSuccess) e = cudaMemsetAsync(overflow, 0, sizeof(int), d->stream);
            if (e == cudaSuccess) e = launch_split_q5_k(raw, conv, conv2, src_blocks, overflow, d->stream);
            if (e == cudaSuccess) e = cudaMemcpyAsync(&overflowed, overflow, sizeof(int), cudaMemcpyDeviceToHost, d->stream);
        } else if (e == cudaSuccess) {
            e = launch_convert_to_q8_0(fmt, raw, conv, src_blocks, d->stream);
        }
    }
    if (e == cudaSuccess) e = weight_from_device_blocks(d, dev_fmt, fmt, n, k, conv ? conv : raw, &w);
    if (e == cudaSuccess && fmt == FMT_Q5_K) e = weight_from_device_blocks(d, dev_fmt, fmt, n, k, conv2, &high);
    if (high) high->view.pair_sum = 1;   // in a two-weight mat-vec launch its product is added to the first weight's
    if (e == cudaSuccess) e = cudaStreamSynchronize(d->stream);
    if (raw) cudaFree(raw);
    if (conv) cudaFree(conv);
    if (conv2) cudaFree(conv2);
    if (overflow) cudaFree(overflow);
    if (e != cudaSuccess || overflowed) {
        if (w) { cudaFree(w->base); delete w; }
        if (high) { cudaFree(high->base); delete high; }
        if (e != cudaSuccess) return cuda_fail(e, "slc_weight_upload");
        return fail(SLC_ERR_UNSUPPORTED, "Q5_K block with a scale whose sixteenfold is not an f16: the split into two Q4_K weights would not be exact");
    }
    w->high = high;
    *out = w;
    return SLC_OK;
}

slc_result slc_weight_upload_kslice(slc_device *d, int32_t fmt, int64_t n, int64_t k, const void *blocks, int64_t bytes,
                                    int64_t k0, int64_t k1, slc_weight **out)
{
    if (!out) return fail(SLC_ERR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    slc_result r = check_weight_args(d, fmt, n, k, blocks, bytes);
    if (r != SLC_OK) return r;
    const int bs = source_block_size(fmt), bb = source_block_bytes(fmt);
    if (k0 < 0 || k1 <= k0 || k1 > k || k0 % bs != 0 || k1 % bs != 0) {
        return fail(SLC_ERR_INVALID_ARGUMENT, "K slice must be non-empty and aligned to the block size");
    }
    const size_t row_full = (size_t)(k / bs) * bb, row_slice = (size_t)((k1 - k0) / bs) * bb, off = (size_t)(k0 / bs) * bb;
    std::vector<uint8_t> packed;
    try { packed.resize((size_t)n * row_slice); } catch (...) { return fail(SLC_ERR_OUT_OF_MEMORY, "host allocation failed"); }
    for (int64_t row = 0; row < n; row++) {
        memcpy(packed.data() + (size_t)row * row_slice, (const uint8_t *)blocks + (size_t)row * row_full + off, row_slice);
    }
    return slc_weight_upload(d, fmt, n, k1 - k0, packed.data(), (int64_t)packed.size(), out);
}

slc_result slc_weight_download(slc_weight *w, void *blocks, int64_t bytes)
{
    if (!w) return fail(SLC_ERR_INVALID_ARGUMENT, "weight is null");
    if (w->src_fmt != w->fmt) return fail(SLC_ERR_UNSUPPORTED, "a weight converted at upload (Q5_0, IQ4_NL, Q5_K) keeps no raw blocks of its format");
    const long long want = w->n * (w->k / block_size(w->fmt)) * block_bytes(w->fmt);
    if (bytes != want) return fail(SLC_ERR_BUFFER_TOO_SMALL, "bytes != n * k / block_size * block_bytes");
    if (bytes == 0) return SLC_OK;
    if (!blocks) return fail(SLC_ERR_INVALID_ARGUMENT, "blocks is null");
    slc_device *d = w->dev;
    SLC_CUDA(cudaSetDevice(d->index));
    uint8_t *raw = nullptr;
    SLC_CUDA(cudaMalloc(&raw, (size_t)bytes));
    cudaError_t e = cudaMemsetAsync(raw, 0, (size_t)bytes, d->stream);
    if (e == cudaSuccess) {
        e = launch_repack(w->fmt, (int)w->n, (int)w->k, w->view.n_pad, w->view.k_pad, raw, w->base, true, d->stream);
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(blocks, raw, (size_t)bytes, cudaMemcpyDeviceToHost, d->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(d->stream);
    cudaFree(raw);
    if (e != cudaSuccess) return cuda_fail(e, "slc_weight_download");
    return SLC_OK;
}

// ---- the device layout as an artefact: written once, loaded without the re-layout pass ---------------------------------

static const uint32_t SLC_LAYOUT_MAGIC = 0x4C434C53u;   // "SLCL"
static const uint32_t SLC_LAYOUT_VERSION = 1;

struct LayoutHeader
{
    uint32_t magic, version;
    int32_t fmt, src_fmt;   // src_fmt: 0, or the uploaded format of a weight whose records are Q8_0 after conversion
    int64_t n, k, n_pad, k_pad, payload;
};

slc_result slc_weight_layout_bytes(slc_weight *w, int64_t *out_bytes)
{
    if (!w || !out_bytes) return fail(SLC_ERR_INVALID_ARGUMENT, "weight or out is null");
    if (w->high) return fail(SLC_ERR_UNSUPPORTED, "a Q5_K weight (two Q4_K weights on the device) has no single-layout artefact");
    *out_bytes = (int64_t)(sizeof(LayoutHeader) + weight_bytes(w->fmt, w->view.n_pad, w->view.k_pad));
    return SLC_OK;
}

slc_result slc_weight_export_layout(slc_weight *w, void *out, int64_t bytes)
{
    if (!w || !out) return fail(SLC_ERR_INVALID_ARGUMENT, "weight or out is null");
    if (w->high) return fail(SLC_ERR_UNSUPPORTED, "a Q5_K weight (two Q4_K weights on the device) has no single-layout artefact");
    const size_t payload = weight_bytes(w->fmt, w->view.n_pad, w->view.k_pad);
    if (bytes != (int64_t)(sizeof(LayoutHeader) + payload)) return fail(SLC_ERR_BUFFER_TOO_SMALL, "bytes != slc_weight_layout_bytes");
    // (the second format field: what was uploaded, when the records are of another format -- Q5_0, IQ4_NL; else 0)
    LayoutHeader h{ SLC_LAYOUT_MAGIC, SLC_LAYOUT_VERSION, w->fmt, w->src_fmt != w->fmt ? w->src_fmt : 0, w->n, w->k, w->view.n_pad, w->view.k_pad, (int64_t)payload };
    memcpy(out, &h, sizeof h);
    SLC_CUDA(cudaSetDevice(w->dev->index));
    SLC_CUDA(cudaMemcpy(static_cast<uint8_t *>(out) + sizeof h, w->base, payload, cudaMemcpyDeviceToHost));
    return SLC_OK;
}

slc_result slc_weight_import_layout(slc_device *d, const void *artefact, int64_t bytes, slc_weight **out)
{
    if (!out) return fail(SLC_ERR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (!d || !artefact || bytes < (int64_t)sizeof(LayoutHeader)) return fail(SLC_ERR_INVALID_ARGUMENT, "device or artefact is null, or too short");
    LayoutHeader h;
    memcpy(&h, artefact, sizeof h);
    if (h.magic != SLC_LAYOUT_MAGIC) return fail(SLC_ERR_INVALID_ARGUMENT, "not a weight-layout artefact");
    if (h.version != SLC_LAYOUT_VERSION) return fail(SLC_ERR_UNSUPPORTED, "weight-layout artefact of another version: upload the raw blocks again");
    const int bs = block_size(h.fmt);
    if (bs == 0 || h.n < 0 || h.k <= 0 || h.k % bs != 0 || h.n_pad != (int64_t)round_up((size_t)h.n, 16) ||
        h.k_pad != (int64_t)round_up((size_t)h.k, 256) || h.payload != (int64_t)weight_bytes(h.fmt, (int)h.n_pad, (int)h.k_pad) ||
        bytes != (int64_t)sizeof(LayoutHeader) + h.payload || (h.src_fmt != 0 && (device_format(h.src_fmt) != h.fmt || h.src_fmt == h.fmt || h.src_fmt == FMT_Q5_K))) {
        return fail(SLC_ERR_INVALID_ARGUMENT, "weight-layout artefact: inconsistent header");
    }
    SLC_CUDA(cudaSetDevice(d->index));
    slc_weight *w = new (std::nothrow) slc_weight();
    if (!w) return fail(SLC_ERR_OUT_OF_MEMORY, "host allocation failed");
    w->dev = d; w->fmt = h.fmt; w->src_fmt = h.src_fmt ? h.src_fmt : h.fmt; w->n = h.n; w->k = h.k;
    w->bytes = round_up((size_t)h.payload, 256) + 256;
    cudaError_t e = cudaMalloc(&w->base, w->bytes);
    if (e == cudaSuccess) e = cudaMemsetAsync(w->base, 0, w->bytes, d->stream);
    if (e == cudaSuccess && h.payload > 0) {
        e = cudaMemcpyAsync(w->base, static_cast<const uint8_t *>(artefact) + sizeof h, (size_t)h.payload, cudaMemcpyHostToDevice, d->stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(d->stream);
    if (e != cudaSuccess) {
        if (w->base) cudaFree(w->base);
        delete w;
        return cuda_fail(e, "slc_weight_import_layout");
    }
    w->view.fmt = h.fmt; w->view.n = (int)h.n; w->view.k = (int)h.k; w->view.n_pad = (int)h.n_pad; w->view.k_pad = (int)h.k_pad;
    w->view.data = w->base;
    *out = w;
    return SLC_OK;
}

slc_result slc_weight_shape(slc_weight *w, int32_t *format, int64_t *n, int64_t *k, int64_t *device_bytes)
{
    if (!w) return fail(SLC_ERR_INVALID_ARGUMENT, "weight is null");
    if (format) *format = w->src_fmt;   // the format that was uploaded
    if (n) *n = w->n;
    if (k) *k = w->k;
    if (device_bytes) *device_bytes = (int64_t)(w->bytes + (w->high ? w->high->bytes : 0));
    return SLC_OK;
}

void slc_weight_free(slc_weight *w)
{
    if (!w) return;
    cudaSetDevice(w->dev->index);
    if (w->high) { cudaFree(w->high->base); delete w->high; }
    cudaFree(w->base);
    delete w;
}

// ---- activations -----------------------------------------------------------------------------------------------------

slc_result slc_activation_create(slc_device *d, int64_t max_rows, int64_t k, slc_activation **out)
{
    if (!out) return fail(SLC_ERR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (!d || max_rows < 1 || k < 32 || k % 32 != 0 || k > (1 << 30) || max_rows > (1 << 24)) {
        return fail(SLC_ERR_INVALID_ARGUMENT, "activation shape: max_rows >= 1, K a positive multiple of 32");
    }
    SLC_CUDA(cudaSetDevice(d->index));
    slc_activation *a = new (std::nothrow) slc_activation();
    if (!a) return fail(SLC_ERR_OUT_OF_MEMORY, "host allocation failed");
    a->dev = d; a->max_rows = max_rows; a->k = k;
    a->k_pad = (int)round_up((size_t)k, 256);
    a->cap_rows = pad_rows(max_rows);
    const size_t cap = (size_t)a->cap_rows, kp = (size_t)a->k_pad;
    const size_t q_b = round_up(cap * kp, 256), ds_b = round_up(cap * (kp / 32) * 8, 256);
    const size_t gs_b = round_up(cap * (kp / 16) * 4, 256), is_b = round_up(cap * (kp / 32) * 4, 256);
    const size_t qt_b = a->cap_rows > 64 ? q_b : 0;   // core-matrix copy for the int8 tensor-core GEMM
    // the tile kernel's planes (3 rows and more): swizzled codes, split offset sums, partial-tile scratch and counters
    const bool tiles = max_rows >= 3;
    a->tile_ctas = d->prop.multiProcessorCount;
    const size_t ht_b = tiles ? round_up(cap * kp, 1024) : 0, s2_b = tiles ? round_up(cap * (kp / 256) * 64, 1024) : 0;
    const size_t sc_b = tiles ? round_up(umma_scratch_bytes(a->tile_ctas, a->cap_rows), 256) : 0;
    a->tile_scratch_floats = sc_b / sizeof(float);
    a->tile_counter_slots = a->tile_ctas > 4096 ? a->tile_ctas : 4096;
    const size_t ct_b = tiles ? round_up((size_t)a->tile_counter_slots * 4, 256) : 0;
    a->bytes = q_b + 2 * ds_b + gs_b + is_b + qt_b + ht_b + s2_b + sc_b + ct_b + (tiles ? 1024 : 0);
    cudaError_t e = cudaMalloc(&a->base, a->bytes);
    if (e == cudaSuccess) e = cudaMemset(a->base, 0, a->bytes);
    if (e != cudaSuccess) {
        if (a->base) cudaFree(a->base);
        delete a;
        return cuda_fail(e, "slc_activation_create");
    }
    a->planes.q = reinterpret_cast<int8_t *>(a->base);
    a->planes.ds = reinterpret_cast<float2 *>(a->base + q_b);
    a->planes.dx = reinterpret_cast<float *>(a->base + q_b + ds_b);
    a->planes.sx = reinterpret_cast<float *>(a->base + q_b + ds_b + ds_b / 2);
    a->planes.gs = reinterpret_cast<float *>(a->base + q_b + 2 * ds_b);
    a->planes.isum = reinterpret_cast<int *>(a->base + q_b + 2 * ds_b + gs_b);
    a->q_tiled = qt_b ? a->base + q_b + 2 * ds_b + gs_b + is_b : nullptr;
    if (tiles) {
        uint8_t *t0 = a->base + q_b + 2 * ds_b + gs_b + is_b + qt_b;   // 256-byte aligned so far; the planes want 1024
        t0 += (1024 - (reinterpret_cast<uintptr_t>(t0) & 1023)) & 1023;
        a->q_sw = t0;
        a->sx2 = t0 + ht_b;
        a->tile_scratch = reinterpret_cast<float *>(t0 + ht_b + s2_b);
        a->tile_counters = reinterpret_cast<int *>(t0 + ht_b + s2_b + sc_b);
    }
    *out = a;
    return SLC_OK;
}

void slc_activation_destroy(slc_activation *a)
{
    if (!a) return;
    cudaSetDevice(a->dev->index);
    cudaFree(a->base);
    delete a;
}

// What every way of filling an activation object does first: bounds, padded row count, which optional planes this row
// count needs, and the bookkeeping that decides whether later MatMul launches may run beside each other.
static slc_result begin_fill(slc_activation *a, int64_t rows, void *stream, cudaStream_t *s)
{
    if (rows < 0) return fail(SLC_ERR_INVALID_ARGUMENT, "rows < 0");
    if (rows > a->max_rows) return fail(SLC_ERR_INVALID_STATE, "rows exceed the bound the activation was created with");
    a->rows = (int)rows;
    a->rows_pad = rows > 0 ? pad_rows(rows) : 0;
    if (rows == 0) return SLC_OK;
    SLC_CUDA(cudaSetDevice(a->dev->index));
    *s = stream ? (cudaStream_t)stream : a->dev->stream;
    a->planes.q_tiled = rows > 64 ? a->q_tiled : nullptr;
    a->planes.q_sw = rows >= 3 ? a->q_sw : nullptr;
    a->planes.sx2 = rows >= 3 ? a->sx2 : nullptr;
    a->reads_since_quantize = 0;
    a->quantize_stream = *s;
    a->pending = false;
    return SLC_OK;
}

slc_result slc_activation_quantize(slc_activation *a, const void *x, int32_t x_dtype, int64_t rows, int64_t x_stride,
                                   void *stream)
{
    if (!a) return fail(SLC_ERR_INVALID_ARGUMENT, "activation is null");
    if (x_dtype != SLC_F32 && x_dtype != SLC_BF16) return fail(SLC_ERR_UNSUPPORTED, "activation dtype must be f32 or bf16");
    if (rows > 0 && !x) return fail(SLC_ERR_INVALID_ARGUMENT, "x is null");
    if (rows > 0 && x_stride < a->k) return fail(SLC_ERR_INVALID_ARGUMENT, "x_stride < K");
    cudaStream_t s = nullptr;
    slc_result r = begin_fill(a, rows, stream, &s);
    if (r != SLC_OK || rows == 0) return r;
    SLC_CUDA(launch_quantize(x, x_dtype, a->rows, a->rows_pad, (int)a->k, a->k_pad, x_stride, a->planes, s));
    return SLC_OK;
}

// Up to this K the mat-vec quantizes deferred rows itself; beyond it the quantizer kernel runs first. Every CTA redoes
// the row before its dots can start, so it pays only for short rows -- measured per dependent (quantize +) mat-vec on
// [8192, K] Q4_K at one row: K = 1024 4.17 -> 2.99 us, 2048 5.96 -> 5.29, 3584 7.69 -> 8.11, 4096 8.00 -> 8.66.
static const int FUSED_QUANTIZE_MAX_K = 2048;

slc_result slc_activation_set_rows(slc_activation *a, const void *x, int32_t x_dtype, int64_t rows, int64_t x_stride, void *stream)
{
    if (!a) return fail(SLC_ERR_INVALID_ARGUMENT, "activation is null");
    if (x_dtype != SLC_F32 && x_dtype != SLC_BF16) return fail(SLC_ERR_UNSUPPORTED, "activation dtype must be f32 or bf16");
    if (rows > 0 && !x) return fail(SLC_ERR_INVALID_ARGUMENT, "x is null");
    if (rows > 0 && x_stride < a->k) return fail(SLC_ERR_INVALID_ARGUMENT, "x_stride < K");
    cudaStream_t s = nullptr;
    slc_result r = begin_fill(a, rows, stream, &s);
    if (r != SLC_OK || rows == 0) return r;
    a->pending = true;
    a->pending_x = x; a->pending_dtype = x_dtype; a->pending_stride = x_stride;
    return SLC_OK;
}

slc_result slc_activation_quantize_rmsnorm(slc_activation *a, const void *x, int32_t x_dtype, int64_t rows, int64_t x_stride,
                                           const float *weight, float eps, float *y, int64_t y_stride, void *stream)
{
    if (!a) return fail(SLC_ERR_INVALID_ARGUMENT, "activation is null");
    if (x_dtype != SLC_F32 && x_dtype != SLC_BF16) return fail(SLC_ERR_UNSUPPORTED, "activation dtype must be f32 or bf16");
    if (rows > 0 && !x) return fail(SLC_ERR_INVALID_ARGUMENT, "x is null");
    if (rows > 0 && x_stride < a->k) return fail(SLC_ERR_INVALID_ARGUMENT, "x_stride < K");
    if (y && (y_stride < a->k || (y_stride & 3) || (reinterpret_cast<uintptr_t>(y) & 15))) {
        return fail(SLC_ERR_INVALID_ARGUMENT, "y: 16-byte aligned, y_stride >= K and a multiple of 4");
    }
    if (weight && (reinterpret_cast<uintptr_t>(weight) & 15)) return fail(SLC_ERR_INVALID_ARGUMENT, "weight must be 16-byte aligned");
    if (!(eps >= 0.0f)) return fail(SLC_ERR_INVALID_ARGUMENT, "eps must be >= 0");
    cudaStream_t s = nullptr;
    slc_result r = begin_fill(a, rows, stream, &s);
    if (r != SLC_OK || rows == 0) return r;
    SLC_CUDA(launch_rmsnorm_quantize(x, x_dtype, a->rows, a->rows_pad, (int)a->k, a->k_pad, x_stride, weight, eps, y, y_stride,
                                     a->planes, s));
    return SLC_OK;
}

slc_result slc_activation_quantize_silu_mul(slc_activation *a, const float *gate, int64_t gate_stride, const float *up,
                                            int64_t up_stride, int64_t rows, float *y, int64_t y_stride, void *stream)
{
    if (!a) return fail(SLC_ERR_INVALID_ARGUMENT, "activation is null");
    if (rows > 0 && (!gate || !up)) return fail(SLC_ERR_INVALID_ARGUMENT, "gate or up is null");
    if (rows > 0 && (gate_stride < a->k || up_stride < a->k)) return fail(SLC_ERR_INVALID_ARGUMENT, "gate_stride / up_stride < K");
    if (y && y_stride < a->k) return fail(SLC_ERR_INVALID_ARGUMENT, "y_stride < K");
    cudaStream_t s = nullptr;
    slc_result r = begin_fill(a, rows, stream, &s);
    if (r != SLC_OK || rows == 0) return r;
    SLC_CUDA(launch_silu_mul_quantize(gate, gate_stride, up, up_stride, a->rows, a->rows_pad, (int)a->k, a->k_pad, y, y_stride,
                                      a->planes, s));
    return SLC_OK;
}

slc_result slc_argmax_rows(slc_device *d, const float *y, int64_t rows, int64_t n, int64_t y_stride, int32_t *out_index, void *stream)
{
    if (!d) return fail(SLC_ERR_INVALID_ARGUMENT, "device is null");
    if (rows < 0 || n < 1 || n > (1ll << 30) || rows > (1 << 24)) return fail(SLC_ERR_INVALID_ARGUMENT, "rows >= 0, 1 <= n <= 2^30");
    if (rows == 0) return SLC_OK;
    if (!y || !out_index || y_stride < n) return fail(SLC_ERR_INVALID_ARGUMENT, "bad buffers or stride");
    SLC_CUDA(cudaSetDevice(d->index));
    SLC_CUDA(launch_argmax_rows(y, y_stride, (int)rows, (int)n, out_index, stream ? (cudaStream_t)stream : d->stream));
    return SLC_OK;
}

slc_result slc_matmul_id_run(slc_weight *w, int32_t experts, const void *x, int32_t x_dtype, int64_t x_stride, const int32_t *ids,
                             int64_t tokens, int64_t slots, int32_t per_slot, float *y, int64_t y_stride, void *stream)
{
    if (!w) return fail(SLC_ERR_INVALID_ARGUMENT, "weight is null");
    if (x_dtype != SLC_F32 && x_dtype != SLC_BF16) return fail(SLC_ERR_UNSUPPORTED, "activation dtype must be f32 or bf16");
    if (experts < 1 || w->n % experts != 0) return fail(SLC_ERR_INVALID_ARGUMENT, "the weight's rows are not a multiple of the expert count");
    const long long n = w->n / experts;
    if (n % 16 != 0) return fail(SLC_ERR_UNSUPPORTED, "MatMulId: rows per expert must be a multiple of 16 (an expert starts on a row group)");
    if (w->high) return fail(SLC_ERR_UNSUPPORTED, "MatMulId takes no Q5_K weight (two passes)");
    if (tokens < 0 || slots < 1 || slots > 65535 || tokens > (1 << 24)) return fail(SLC_ERR_INVALID_ARGUMENT, "tokens >= 0, 1 <= slots <= 65535");
    if (tokens == 0 || n == 0) return SLC_OK;
    if (!x || !ids || !y || x_stride < w->k || y_stride < n) return fail(SLC_ERR_INVALID_ARGUMENT, "bad buffers or strides");
    if (matvec_f32_rows(w->view.k_pad) == 0) return fail(SLC_ERR_UNSUPPORTED, "K is too long for the f32 mat-vec's shared memory");
    slc_device *d = w->dev;
    SLC_CUDA(cudaSetDevice(d->index));
    SLC_CUDA(launch_matvec_f32_id(w->view, experts, x, x_dtype, x_stride, ids, tokens, (int)slots, per_slot ? 1 : 0, y, y_stride,
                                  d->status_dev, stream ? (cudaStream_t)stream : d->stream));
    return SLC_OK;
}

static ActView view_of(const slc_activation *a)
{
    ActView v;
    v.rows = a->rows; v.rows_pad = a->rows_pad; v.k = (int)a->k; v.k_pad = a->k_pad;
    v.q = a->planes.q; v.ds = a->planes.ds; v.dx = a->planes.dx; v.sx = a->planes.sx; v.gs = a->planes.gs;
    v.isum = a->planes.isum;
    if (a->pending) { v.raw = a->pending_x; v.raw_dtype = a->pending_dtype; v.raw_stride = a->pending_stride; }
    return v;
}

// ---- the operator ----------------------------------------------------------------------------------------------------

slc_result slc_matmul_create(slc_device *d, slc_weight *w, int64_t max_rows, uint32_t flags, slc_matmul **out)
{
    if (!out) return fail(SLC_ERR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (!d || !w) return fail(SLC_ERR_INVALID_ARGUMENT, "null device or weight");
    if (w->dev != d) return fail(SLC_ERR_INVALID_ARGUMENT, "the weight lives on another device");
    if (max_rows < 1 || max_rows > (1 << 24)) return fail(SLC_ERR_INVALID_ARGUMENT, "max_rows out of range");
    if (flags & ~(uint32_t)(SLC_MATMUL_ROW_INVARIANT | SLC_MATMUL_F32_ACTIVATIONS)) return fail(SLC_ERR_INVALID_ARGUMENT, "unknown flags");
    if ((flags & SLC_MATMUL_F32_ACTIVATIONS) && matvec_f32_rows(w->view.k_pad) == 0) {
        return fail(SLC_ERR_UNSUPPORTED, "K is too long for the f32-activation mat-vec's shared memory");
    }
    slc_matmul *op = new (std::nothrow) slc_matmul();
    if (!op) return fail(SLC_ERR_OUT_OF_MEMORY, "host allocation failed");
    op->dev = d; op->w = w; op->max_rows = max_rows; op->flags = flags;
    *out = op;
    return SLC_OK;
}

slc_result slc_matmul_create_dual(slc_device *d, slc_weight *gate, slc_weight *up, int64_t max_rows, uint32_t flags,
                                  slc_matmul **out)
{
    if (!out) return fail(SLC_ERR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (!gate || !up) return fail(SLC_ERR_INVALID_ARGUMENT, "null weight");
    if (gate->dev != up->dev || gate->fmt != up->fmt || gate->n != up->n || gate->k != up->k) {
        return fail(SLC_ERR_INVALID_ARGUMENT, "gate and up must share device, format and shape");
    }
    if (gate->high || up->high) return fail(SLC_ERR_UNSUPPORTED, "a dual MatMul takes no Q5_K weights (two passes each): run gate and up as two MatMuls");
    slc_matmul *op = nullptr;
    slc_result r = slc_matmul_create(d, gate, max_rows, flags, &op);
    if (r != SLC_OK) return r;
    op->w2 = up;
    SLC_CUDA(cudaSetDevice(d->index));
    cudaError_t e = cudaMalloc(&op->dual_tmp, (size_t)max_rows * (gate->n > 0 ? gate->n : 1) * 4);
    if (e != cudaSuccess) {
        delete op;
        return cuda_fail(e, "slc_matmul_create_dual");
    }
    *out = op;
    return SLC_OK;
}

void slc_matmul_destroy(slc_matmul *op)
{
    if (!op) return;
    cudaSetDevice(op->dev->index);
    if (op->dual_tmp) cudaFree(op->dual_tmp);
    if (op->act) slc_activation_destroy(op->act);
    if (op->x_stage) cudaFree(op->x_stage);
    if (op->y_stage) cudaFree(op->y_stage);
    delete op;
}

slc_result slc_matmul_set_kernel(slc_matmul *op, int32_t kernel)
{
    if (!op) return fail(SLC_ERR_INVALID_ARGUMENT, "op is null");
    if (kernel < SLC_KERNEL_AUTO || kernel > SLC_KERNEL_TILE) return fail(SLC_ERR_INVALID_ARGUMENT, "unknown or not selectable kernel family");
    if (kernel == SLC_KERNEL_TILE && !umma_supports(op->w->fmt, 1 << 20)) {
        return fail(SLC_ERR_UNSUPPORTED, "the tile kernel does not take this weight format");
    }
    if (kernel == SLC_KERNEL_MMQ && !mmq_supports(op->w->fmt)) {
        return fail(SLC_ERR_UNSUPPORTED, "the tensor-core GEMM does not take this weight format");
    }
    op->forced_kernel = kernel;
    return SLC_OK;
}

slc_result slc_matmul_last_kernel(slc_matmul *op, int32_t *out_kernel, int32_t *out_launches)
{
    if (!op) return fail(SLC_ERR_INVALID_ARGUMENT, "op is null");
    if (out_kernel) *out_kernel = op->last_kernel;
    if (out_launches) *out_launches = op->last_launches_total > 0 ? op->last_launches_total : op->last_launches;
    return SLC_OK;
}

// Row-count dispatch. The reference's own GPU policy switches at 8 / 16 / 33 rows
// (src/Sharplight.Shaders/Lowering/GraphLowerer.IntDot.cs:18-19, GraphLowerer.Mmq.cs:16-52 of the Sharplight tree);
// these thresholds are the measured crossovers of this library's kernels on B200.
// From this row count the tile kernel is the default where it takes the format.
static const int UMMA_MIN_ROWS = 1 << 30;

static int choose_kernel(const slc_matmul *op, int rows, bool exchanging)
{
    if (op->forced_kernel != SLC_KERNEL_AUTO &&
        !(op->forced_kernel == SLC_KERNEL_TILE && (exchanging || rows < 3 || !umma_supports(op->w->fmt, rows)))) {
        return op->forced_kernel;
    }
    // the mat-vec keeps a row's quantized activations whole in shared memory; a K beyond that goes to the tiled kernel
    const bool mv = matvec_fits(1, op->w->view.k_pad, op->w2 != nullptr);
    if (mv && (op->flags & SLC_MATMUL_ROW_INVARIANT) && rows <= 8) return SLC_KERNEL_MMVQ;
    if (mv && rows <= 2) return SLC_KERNEL_MMVQ;
    // the tile kernel (stream-K, tcgen05) from UMMA_MIN_ROWS rows; the in-kernel sum over ranks lives in the older kernels
    if (rows >= UMMA_MIN_ROWS && umma_supports(op->w->fmt, rows) && !exchanging) return SLC_KERNEL_TILE;
    // more than 64 rows: the tensor-core GEMM for every format (Q6_K included: two half-masked MMAs per block; on
    // [4096, 4096] x 2048 rows 394 us against 554 of the tile kernel and 919 of 64-row chunks of the skinny kernel, on
    // [32064, 4096] 3058 against 4241 and 3287)
    if (rows <= 64 || !mmq_supports(op->w->fmt)) return SLC_KERNEL_SKINNY;
    return SLC_KERNEL_MMQ;
}

static slc_result run_family(slc_matmul *op, const WeightView &wv, const WeightView *w2, slc_activation *act, const ActView &av,
                             int kernel, float *y, long long y_stride, int *dump, cudaStream_t s, const Exchange *ex,
                             const Epilogue *ep, bool allow_early = true);

// ex (optional): the MatMul is the row-split part of a tensor-parallel group and its kernel sums over the ranks.
// ep (optional): bias and residual added before the store.
static slc_result run_kernels(slc_matmul *op, slc_activation *act, float *y, long long y_stride, int *dump,
                              cudaStream_t s, const Exchange *ex = nullptr, const Epilogue *ep = nullptr)
{
    if (op->flags & SLC_MATMUL_F32_ACTIVATIONS) return fail(SLC_ERR_INVALID_STATE, "this op keeps f32 activations: it takes no quantized ones");
    const int rows = act->rows;
    const int kernel = choose_kernel(op, rows, ex != nullptr);
    bool ran_quantizer = false;
    if (act->pending) {
        // deferred rows: the mat-vec quantizes them itself when K is short; otherwise the quantizer runs now, on this
        // stream, and the planes are there for this and every later MatMul
        const bool fuse = kernel == SLC_KERNEL_MMVQ && !dump && !op->w2 && !op->w->high && act->k_pad <= FUSED_QUANTIZE_MAX_K;   // (Q5_K: two passes read the rows)
        if (!fuse) {
            SLC_CUDA(launch_quantize(act->pending_x, act->pending_dtype, act->rows, act->rows_pad, (int)act->k, act->k_pad,
                                     act->pending_stride, act->planes, s));
            act->pending = false;
            act->quantize_stream = s;
            ran_quantizer = true;
        }
    }
    const ActView av = view_of(act);
    op->last_kernel = kernel;
    op->last_launches = ran_quantizer ? 1 : 0;   // (the deferred quantizer counts as a launch of this call)
    op->last_launches_total = 0;
    if (op->w2) {
        // gate / up pair: one dual mat-vec launch where that kernel serves the row count, else gate -> scratch,
        // up -> y, and the element-wise tail
        if (dump || ex || ep) return fail(SLC_ERR_UNSUPPORTED, "a dual MatMul takes no block-dot export, exchange or epilogue");
        if (kernel == SLC_KERNEL_MMVQ) return run_family(op, op->w->view, &op->w2->view, act, av, kernel, y, y_stride, nullptr, s, nullptr, nullptr);
        // the gate launch overwrites dual_tmp, which the element-wise tail of an earlier run of this op may still be
        // reading: it waits for its predecessor like any launch that writes shared state
        const long long n = op->w->n;
        slc_result r = run_family(op, op->w->view, nullptr, act, av, kernel, op->dual_tmp, n, nullptr, s, nullptr, nullptr, false);
        if (r == SLC_OK) r = run_family(op, op->w2->view, nullptr, act, av, kernel, y, y_stride, nullptr, s, nullptr, nullptr);
        if (r != SLC_OK) return r;
        SLC_CUDA(launch_gate_mul(op->dual_tmp, n, y, y_stride, rows, (int)n, s));
        op->last_launches++;
        return SLC_OK;
    }
    if (op->w->high && kernel == SLC_KERNEL_MMVQ && !dump && !ex && matvec_fits(1, op->w->view.k_pad, true)) {
        // Q5_K on the mat-vec: both Q4_K halves stream through one launch (the two-weight form of the kernel, products added)
        return run_family(op, op->w->view, &op->w->high->view, act, av, kernel, y, y_stride, nullptr, s, nullptr, ep);
    }
    slc_result r = run_family(op, op->w->view, nullptr, act, av, kernel, y, y_stride, dump, s, ex, ep);
    if (r == SLC_OK && op->w->high) {
        // Q5_K: the fifth bits are a second Q4_K weight whose product is added onto the first (in place: every output is
        // read and rewritten by the thread that owns it; a launch with an epilogue never runs beside its predecessor)
        if (dump) return fail(SLC_ERR_UNSUPPORTED, "block-dot export of a Q5_K weight goes through slc_debug_block_dots");
        const Epilogue add{ nullptr, y, y_stride };
        r = run_family(op, op->w->high->view, nullptr, act, av, kernel, y, y_stride, nullptr, s, ex, &add);
    }
    return r;
}

// The launches of one weight (two for the dual mat-vec) in the chosen kernel family.
static slc_result run_family(slc_matmul *op, const WeightView &wv, const WeightView *w2, slc_activation *act, const ActView &av,
                             int kernel, float *y, long long y_stride, int *dump, cudaStream_t s, const Exchange *ex,
                             const Epilogue *ep, bool allow_early)
{
    const int rows = act->rows;
    const long long dump_row = (long long)wv.n * (wv.k >> 5);
    // A launch may run beside its predecessor when an earlier launch on this stream has already read these
    // activations: they were complete before that launch started, and MatMul outputs do not alias each other. Not so
    // when the launch reads more than the activations -- a bias or a residual, which the predecessor may be writing
    // (y2 = W2 x + y1 right after y1 = W1 x) -- or when it runs on another stream than the quantization did.
    auto early = [&]() {
        return allow_early && !ex && !ep && !act->pending && act->reads_since_quantize > 0 && s == act->quantize_stream ? 1 : 0;
    };
    if (kernel == SLC_KERNEL_MMVQ) {
        // chunks of up to 4 rows; every row of a chunk is computed exactly as a single row is, so the row-invariant
        // guarantee holds for any chunking
        int chunk = 4;
        while (chunk > 1 && !matvec_fits(chunk, wv.k_pad, w2 != nullptr)) chunk--;
        if (!matvec_fits(chunk, wv.k_pad, w2 != nullptr)) return fail(SLC_ERR_UNSUPPORTED, "K is too large for the mat-vec kernel's shared memory");
        for (int r0 = 0; r0 < rows; r0 += chunk) {
            const int m = rows - r0 < chunk ? rows - r0 : chunk;
            SLC_CUDA(launch_matvec(wv, av, r0, m, y, y_stride, dump ? dump + r0 * dump_row : nullptr, op->dev->status_dev, early(), s, ex, ep, w2));
            act->reads_since_quantize++;
            op->last_launches++;
        }
    } else if (kernel == SLC_KERNEL_SKINNY) {
        // the activation object's scratch area (present from 3 rows of capacity) lets short-and-wide MatMuls split K
        const SkinnySplit split{ act->tile_scratch, act->tile_counters, act->tile_scratch_floats, act->tile_counter_slots, act->tile_ctas };
        for (int r0 = 0; r0 < rows; r0 += 64) {
            const int m = rows - r0 < 64 ? rows - r0 : 64;
            SLC_CUDA(launch_skinny(wv, av, r0, m, y, y_stride, dump ? dump + r0 * dump_row : nullptr, op->dev->status_dev, early(), s, ex, ep,
                                   act->tile_scratch ? &split : nullptr));
            act->reads_since_quantize++;
            op->last_launches++;
        }
    } else if (kernel == SLC_KERNEL_TILE) {
        if (ex) return fail(SLC_ERR_UNSUPPORTED, "the tile kernel does not sum over ranks");
        if (!act->planes.q_sw) return fail(SLC_ERR_INVALID_STATE, "the tile kernel needs an activation object created for 3 rows or more");
        // one persistent launch; it shares the activation object's scratch with other launches, so it never runs early
        SLC_CUDA(launch_umma(wv, av, act->planes.q_sw, act->planes.sx2, y, y_stride, dump, op->dev->status_dev,
                             act->tile_scratch, act->tile_counters, act->tile_ctas, s, ep));
        act->reads_since_quantize++;
        op->last_launches++;
    } else if (ex) {
        return fail(SLC_ERR_UNSUPPORTED, "the in-kernel all-reduce serves the mat-vec and skinny kernels (up to 64 rows)");
    } else {
        if (!act->planes.q_tiled) return fail(SLC_ERR_INVALID_STATE, "the tensor-core GEMM needs more than 64 rows");
        SLC_CUDA(launch_mmq(wv, av, act->planes.q_tiled, y, y_stride, dump, op->dev->status_dev, early(), s, ep));
        act->reads_since_quantize++;
        op->last_launches++;
    }
    return SLC_OK;
}

slc_result slc_matmul_run_quantized(slc_matmul *op, slc_activation *act, float *y, int64_t y_stride, void *stream)
{
    if (!op || !act) return fail(SLC_ERR_INVALID_ARGUMENT, "null op or activation");
    if (op->flags & SLC_MATMUL_F32_ACTIVATIONS) return fail(SLC_ERR_INVALID_STATE, "this op keeps f32 activations: it takes no quantized ones and does not sum over ranks");
    if (act->dev != op->dev) return fail(SLC_ERR_INVALID_ARGUMENT, "the activation lives on another device");
    if (act->k != op->w->k) return fail(SLC_ERR_INVALID_ARGUMENT, "activation K differs from the weight's K");
    if (act->rows > op->max_rows) return fail(SLC_ERR_INVALID_STATE, "rows exceed the op's compiled bound");
    if (act->rows == 0 || op->w->n == 0) return SLC_OK;
    if (!y || y_stride < op->w->n) return fail(SLC_ERR_INVALID_ARGUMENT, "bad output buffer or stride");
    SLC_CUDA(cudaSetDevice(op->dev->index));
    cudaStream_t s = stream ? (cudaStream_t)stream : op->dev->stream;
    return run_kernels(op, act, y, y_stride, nullptr, s);
}

// The prefill sum over ranks in chunks beside the GEMM is an option (slc_tp_comm_set_chunking), not the default: on the
// 70B-shaped stack at 2048 rows it measured 650 against 637 ms on two GPUs and 372 against 356 ms on four -- four smaller
// GEMM launches and NCCL's kernels sharing the SMs with the GEMM cost more than hiding the all-reduce gains.

// A row-split MatMul of a tensor-parallel group: the sum over the ranks happens inside the MatMul kernel (exchange) for
// few rows, and by the attached communicator's all-reduce above the exchange's in_kernel_rows (or its row bound).
static slc_result run_summed(slc_matmul *op, slc_activation *act, slc_tp_exchange *x, float *y, long long y_stride,
                             cudaStream_t s, const Epilogue *ep)
{
    const int rows = act->rows;
    if (!x->connected) return fail(SLC_ERR_INVALID_STATE, "the exchange is not connected");
    if (op->w->n > x->n) return fail(SLC_ERR_INVALID_ARGUMENT, "the weight has more rows than the exchange was created for");
    const bool by_comm = x->comm && x->world > 1 && (rows > x->in_kernel_rows || rows > x->max_rows);
    if (!by_comm) {
        if (rows > x->max_rows) return fail(SLC_ERR_UNSUPPORTED, "rows exceed the exchange's bound and no communicator is attached");
        return run_kernels(op, act, y, y_stride, nullptr, s, &x->view, ep);
    }
    const long long n = op->w->n;
    const int kernel = choose_kernel(op, rows, false);
    const bool chunked = x->comm->chunk_min_rows > 0 && rows >= x->comm->chunk_min_rows;
    if (kernel == SLC_KERNEL_MMQ && chunked && rows > 128 && !op->w2 && !op->w->high && act->planes.q_tiled) {
        // Prefill: the rows in four chunks of whole 128-token tiles; the all-reduce of chunk i runs on the communicator's
        // own stream while the GEMM of chunk i + 1 runs on the caller's, and the caller's stream joins at the end. (Forks
        // and joins by events, so the whole thing can sit inside a captured graph.)
        slc_tp_comm *c = x->comm;
        if (act->pending) {   // deferred rows: the GEMM reads the planes
            SLC_CUDA(launch_quantize(act->pending_x, act->pending_dtype, act->rows, act->rows_pad, (int)act->k, act->k_pad,
                                     act->pending_stride, act->planes, s));
            act->pending = false;
            act->quantize_stream = s;
        }
        const ActView av = view_of(act);
        const int tiles = (rows + 127) / 128, per = (tiles + 3) / 4;
        op->last_kernel = kernel;
        op->last_launches = 0;
        op->last_launches_total = 0;
        int ci = 0;
        for (int t0 = 0; t0 < tiles; t0 += per, ci++) {
            const int cnt = tiles - t0 < per ? tiles - t0 : per;
            const long long r0 = (long long)t0 * 128, r1 = r0 + (long long)cnt * 128 < rows ? r0 + (long long)cnt * 128 : rows;
            SLC_CUDA(launch_mmq(op->w->view, av, act->planes.q_tiled, y, y_stride, nullptr, op->dev->status_dev, 0, s, nullptr, t0, cnt));
            SLC_CUDA(cudaEventRecord(c->chunk_done[ci], s));
            SLC_CUDA(cudaStreamWaitEvent(c->side, c->chunk_done[ci], 0));
            const int e = tp_comm_allreduce(c->comm, y + r0 * y_stride, r1 - r0, n, y_stride, c->side);
            if (e != 0) return fail(SLC_ERR_CUDA, tp_comm_error(e));
            op->last_launches += 2;
        }
        SLC_CUDA(cudaEventRecord(c->joined, c->side));
        SLC_CUDA(cudaStreamWaitEvent(s, c->joined, 0));
        act->reads_since_quantize++;
    } else {
        slc_result r = run_kernels(op, act, y, y_stride, nullptr, s, nullptr, nullptr);
        if (r != SLC_OK) return r;
        const int e = tp_comm_allreduce(x->comm->comm, y, rows, n, y_stride, s);
        if (e != 0) return fail(SLC_ERR_CUDA, tp_comm_error(e));
        op->last_launches++;
    }
    if (ep) {
        SLC_CUDA(launch_add_epilogue(y, y_stride, rows, (int)op->w->n, *ep, s));
        op->last_launches++;
    }
    // the all-reduce (and the additions) wrote y after the MatMul: nothing that follows may run beside them as if the
    // activations' last reader were a MatMul of this stream
    act->reads_since_quantize = 0;
    return SLC_OK;
}

slc_result slc_matmul_run_quantized_epilogue(slc_matmul *op, slc_activation *act, slc_tp_exchange *x, const float *bias,
                                             const float *residual, int64_t residual_stride, float *y, int64_t y_stride,
                                             void *stream)
{
    if (!op || !act) return fail(SLC_ERR_INVALID_ARGUMENT, "null op or activation");
    if (op->flags & SLC_MATMUL_F32_ACTIVATIONS) return fail(SLC_ERR_INVALID_STATE, "this op keeps f32 activations: it takes no quantized ones and does not sum over ranks");
    if (act->dev != op->dev || (x && x->dev != op->dev)) return fail(SLC_ERR_INVALID_ARGUMENT, "op, activation and exchange live on different devices");
    if (act->k != op->w->k) return fail(SLC_ERR_INVALID_ARGUMENT, "activation K differs from the weight's K");
    if (act->rows > op->max_rows) return fail(SLC_ERR_INVALID_STATE, "rows exceed the op's compiled bound");
    if (act->rows == 0 || op->w->n == 0) return SLC_OK;
    if (!y || y_stride < op->w->n) return fail(SLC_ERR_INVALID_ARGUMENT, "bad output buffer or stride");
    if (residual && residual_stride < op->w->n) return fail(SLC_ERR_INVALID_ARGUMENT, "residual_stride < N");
    SLC_CUDA(cudaSetDevice(op->dev->index));
    cudaStream_t s = stream ? (cudaStream_t)stream : op->dev->stream;
    const Epilogue ep{ bias, residual, residual_stride };
    if (x) return run_summed(op, act, x, y, y_stride, s, (bias || residual) ? &ep : nullptr);
    return run_kernels(op, act, y, y_stride, nullptr, s, nullptr, (bias || residual) ? &ep : nullptr);
}

// ---- tensor-parallel exchange ---------------------------------------------------------------------------------------

slc_result slc_tp_exchange_create(slc_device *d, int32_t rank, int32_t world, int64_t max_rows, int64_t n,
                                  slc_tp_exchange **out, uint8_t *out_handle)
{
    if (!out || !out_handle) return fail(SLC_ERR_INVALID_ARGUMENT, "out or out_handle is null");
    *out = nullptr;
    if (!d || world < 1 || world > SLC_TP_MAX_RANKS || rank < 0 || rank >= world) {
        return fail(SLC_ERR_INVALID_ARGUMENT, "exchange: 1 <= world <= 8, 0 <= rank < world");
    }
    if (max_rows < 1 || max_rows > SLC_TP_MAX_ROWS || n < 1 || n > (1 << 24)) {
        return fail(SLC_ERR_INVALID_ARGUMENT, "exchange: 1 <= max_rows <= 64, 1 <= n <= 2^24");
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == SLC_TP_HANDLE_BYTES, "IPC handle size");
    SLC_CUDA(cudaSetDevice(d->index));
    slc_tp_exchange *x = new (std::nothrow) slc_tp_exchange();
    if (!x) return fail(SLC_ERR_OUT_OF_MEMORY, "host allocation failed");
    x->dev = d; x->rank = rank; x->world = world; x->max_rows = max_rows; x->n = n;
    const int n_stride = (int)round_up((size_t)n, 64), groups = n_stride / 16;
    const size_t recv_b = round_up((size_t)2 * world * max_rows * n_stride * 4, 256);
    const size_t flag_b = round_up((size_t)2 * world * groups * 4, 256);
    const size_t ll_b = round_up((size_t)2 * world * SLC_LL_ROWS * n_stride * 8, 256);
    x->flags_off = recv_b; x->ll_off = recv_b + flag_b; x->ctl_off = recv_b + flag_b + ll_b;
    x->bytes = x->ctl_off + 256;
    cudaError_t e = cudaMalloc(&x->base, x->bytes);
    if (e == cudaSuccess) e = cudaMemset(x->base, 0, x->bytes);
    cudaIpcMemHandle_t h;
    memset(&h, 0, sizeof h);
    if (e == cudaSuccess && world > 1) e = cudaIpcGetMemHandle(&h, x->base);
    if (e != cudaSuccess) {
        if (x->base) cudaFree(x->base);
        delete x;
        return cuda_fail(e, "slc_tp_exchange_create");
    }
    memcpy(out_handle, &h, sizeof h);
    Exchange &v = x->view;
    v.world = world; v.rank = rank; v.max_rows = (int)max_rows; v.n_stride = n_stride; v.groups = groups;
    v.wait_ms = 1000;
    v.epoch = reinterpret_cast<int *>(x->base + x->ctl_off);
    v.done = v.epoch + 1;
    x->peer[rank] = x->base;
    x->connected = world == 1;
    if (x->connected) {
        v.recv[0] = reinterpret_cast<float *>(x->base);
        v.flags[0] = reinterpret_cast<int *>(x->base + x->flags_off);
        v.ll[0] = reinterpret_cast<unsigned long long *>(x->base + x->ll_off);
    }
    *out = x;
    return SLC_OK;
}

slc_result slc_tp_exchange_connect(slc_tp_exchange *x, const uint8_t *handles)
{
    if (!x || !handles) return fail(SLC_ERR_INVALID_ARGUMENT, "exchange or handles is null");
    if (x->connected) return x->world == 1 ? SLC_OK : fail(SLC_ERR_INVALID_STATE, "the exchange is already connected");
    SLC_CUDA(cudaSetDevice(x->dev->index));
    for (int p = 0; p < x->world; p++) {
        if (p == x->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)p * SLC_TP_HANDLE_BYTES, sizeof h);
        cudaError_t e = cudaIpcOpenMemHandle(&x->peer[p], h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int q = 0; q < p; q++) {
                if (q != x->rank && x->peer[q]) { cudaIpcCloseMemHandle(x->peer[q]); x->peer[q] = nullptr; }
            }
            return cuda_fail(e, "cudaIpcOpenMemHandle (peer receive area)");
        }
    }
    for (int p = 0; p < x->world; p++) {
        x->view.recv[p] = reinterpret_cast<float *>(x->peer[p]);
        x->view.flags[p] = reinterpret_cast<int *>(reinterpret_cast<uint8_t *>(x->peer[p]) + x->flags_off);
        x->view.ll[p] = reinterpret_cast<unsigned long long *>(reinterpret_cast<uint8_t *>(x->peer[p]) + x->ll_off);
    }
    x->connected = true;
    return SLC_OK;
}

slc_result slc_tp_exchange_set_wait_ms(slc_tp_exchange *x, int32_t milliseconds)
{
    if (!x) return fail(SLC_ERR_INVALID_ARGUMENT, "exchange is null");
    if (milliseconds < 1 || milliseconds > 60000) return fail(SLC_ERR_INVALID_ARGUMENT, "wait limit: 1..60000 ms");
    x->view.wait_ms = (unsigned)milliseconds;
    return SLC_OK;
}

void slc_tp_exchange_destroy(slc_tp_exchange *x)
{
    if (!x) return;
    cudaSetDevice(x->dev->index);
    cudaDeviceSynchronize();
    for (int p = 0; p < x->world; p++) {
        if (p != x->rank && x->peer[p]) cudaIpcCloseMemHandle(x->peer[p]);
    }
    cudaFree(x->base);
    delete x;
}

// ---- tensor-parallel communicator (NCCL, loaded at run time) -------------------------------------------------------------

slc_result slc_tp_comm_unique_id(uint8_t *out_id)
{
    if (!out_id) return fail(SLC_ERR_INVALID_ARGUMENT, "out_id is null");
    if (const char *why = tp_comm_unavailable()) return fail(SLC_ERR_UNSUPPORTED, std::string("NCCL is not available: ") + why);
    const int e = tp_comm_unique_id(out_id);
    if (e != 0) return fail(SLC_ERR_CUDA, tp_comm_error(e));
    return SLC_OK;
}

slc_result slc_tp_comm_create(slc_device *d, int32_t rank, int32_t world, const uint8_t *id, slc_tp_comm **out)
{
    if (!out) return fail(SLC_ERR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (!d || !id || world < 1 || world > SLC_TP_MAX_RANKS || rank < 0 || rank >= world) {
        return fail(SLC_ERR_INVALID_ARGUMENT, "communicator: 1 <= world <= 8, 0 <= rank < world, id from slc_tp_comm_unique_id");
    }
    if (const char *why = tp_comm_unavailable()) return fail(SLC_ERR_UNSUPPORTED, std::string("NCCL is not available: ") + why);
    SLC_CUDA(cudaSetDevice(d->index));
    slc_tp_comm *c = new (std::nothrow) slc_tp_comm();
    if (!c) return fail(SLC_ERR_OUT_OF_MEMORY, "host allocation failed");
    c->dev = d; c->rank = rank; c->world = world;
    const int e = tp_comm_init(&c->comm, world, id, rank);
    if (e != 0) {
        delete c;
        return fail(SLC_ERR_CUDA, tp_comm_error(e));
    }
    cudaError_t ce = cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking);
    for (int i = 0; i < 8 && ce == cudaSuccess; i++) ce = cudaEventCreateWithFlags(&c->chunk_done[i], cudaEventDisableTiming);
    if (ce == cudaSuccess) ce = cudaEventCreateWithFlags(&c->joined, cudaEventDisableTiming);
    if (ce != cudaSuccess) {
        slc_tp_comm_destroy(c);
        return cuda_fail(ce, "slc_tp_comm_create");
    }
    *out = c;
    return SLC_OK;
}

void slc_tp_comm_destroy(slc_tp_comm *c)
{
    if (!c) return;
    cudaSetDevice(c->dev->index);
    cudaDeviceSynchronize();
    if (c->comm) tp_comm_destroy(c->comm);
    for (int i = 0; i < 8; i++) {
        if (c->chunk_done[i]) cudaEventDestroy(c->chunk_done[i]);
    }
    if (c->joined) cudaEventDestroy(c->joined);
    if (c->side) cudaStreamDestroy(c->side);
    delete c;
}

slc_result slc_tp_comm_set_chunking(slc_tp_comm *c, int32_t min_rows)
{
    if (!c) return fail(SLC_ERR_INVALID_ARGUMENT, "communicator is null");
    if (min_rows < 0) return fail(SLC_ERR_INVALID_ARGUMENT, "min_rows >= 0");
    c->chunk_min_rows = min_rows;
    return SLC_OK;
}

slc_result slc_tp_exchange_set_comm(slc_tp_exchange *x, slc_tp_comm *comm, int32_t in_kernel_rows)
{
    if (!x) return fail(SLC_ERR_INVALID_ARGUMENT, "exchange is null");
    if (comm && (comm->dev != x->dev || comm->world != x->world || comm->rank != x->rank)) {
        return fail(SLC_ERR_INVALID_ARGUMENT, "the communicator belongs to another device, rank or group size");
    }
    if (in_kernel_rows < 0 || in_kernel_rows > SLC_TP_MAX_ROWS) return fail(SLC_ERR_INVALID_ARGUMENT, "in_kernel_rows: 0..64");
    x->comm = comm;
    x->in_kernel_rows = in_kernel_rows;
    return SLC_OK;
}

slc_result slc_matmul_run_quantized_allreduce(slc_matmul *op, slc_activation *act, slc_tp_exchange *x, float *y,
                                              int64_t y_stride, void *stream)
{
    if (!op || !act || !x) return fail(SLC_ERR_INVALID_ARGUMENT, "null op, activation or exchange");
    if (op->flags & SLC_MATMUL_F32_ACTIVATIONS) return fail(SLC_ERR_INVALID_STATE, "this op keeps f32 activations: it takes no quantized ones and does not sum over ranks");
    if (act->dev != op->dev || x->dev != op->dev) return fail(SLC_ERR_INVALID_ARGUMENT, "op, activation and exchange live on different devices");
    if (act->k != op->w->k) return fail(SLC_ERR_INVALID_ARGUMENT, "activation K differs from the weight's K");
    if (act->rows > op->max_rows) return fail(SLC_ERR_INVALID_STATE, "rows exceed the op's compiled bound");
    if (act->rows == 0 || op->w->n == 0) return SLC_OK;
    if (!y || y_stride < op->w->n) return fail(SLC_ERR_INVALID_ARGUMENT, "bad output buffer or stride");
    SLC_CUDA(cudaSetDevice(op->dev->index));
    cudaStream_t s = stream ? (cudaStream_t)stream : op->dev->stream;
    return run_summed(op, act, x, y, y_stride, s, nullptr);
}

// x -> y through the op's own activation object (created at first use).
static slc_result quantize_and_run(slc_matmul *op, slc_tp_exchange *ex, const void *x_dev, int32_t x_dtype, int64_t rows,
                                   int64_t x_stride, float *y_dev, int64_t y_stride, cudaStream_t s)
{
    slc_result r;
    if (!op->act) {
        r = slc_activation_create(op->dev, op->max_rows, op->w->k, &op->act);
        if (r != SLC_OK) return r;
    }
    r = slc_activation_quantize(op->act, x_dev, x_dtype, rows, x_stride, s);
    if (r != SLC_OK) return r;
    r = ex ? run_summed(op, op->act, ex, y_dev, y_stride, s, nullptr) : run_kernels(op, op->act, y_dev, y_stride, nullptr, s);
    if (r != SLC_OK) return r;
    op->last_launches_total = op->last_launches + 1;
    return SLC_OK;
}

static slc_result ensure_op_buffers(slc_matmul *op, bool need_x_stage, bool need_y_stage)
{
    if (need_x_stage && !op->x_stage) SLC_CUDA(cudaMalloc(&op->x_stage, (size_t)op->max_rows * op->w->k * 4));
    if (need_y_stage && !op->y_stage) {
        SLC_CUDA(cudaMalloc(&op->y_stage, (size_t)op->max_rows * (op->w->n > 0 ? op->w->n : 1) * 4));
    }
    return SLC_OK;
}

slc_result slc_matmul_run(slc_matmul *op, const void *x, int32_t x_dtype, int64_t rows, int64_t x_stride,
                          int32_t x_is_device, float *y, int64_t y_stride, int32_t y_is_device, void *stream)
{
    if (!op) return fail(SLC_ERR_INVALID_ARGUMENT, "op is null");
    if (x_dtype != SLC_F32 && x_dtype != SLC_BF16) return fail(SLC_ERR_UNSUPPORTED, "activation dtype must be f32 or bf16");
    if (rows < 0) return fail(SLC_ERR_INVALID_ARGUMENT, "rows < 0");
    if (rows > op->max_rows) return fail(SLC_ERR_INVALID_STATE, "rows exceed the op's compiled bound");
    if (rows == 0) return SLC_OK;
    const long long n = op->w->n, k = op->w->k;
    if (!x || x_stride < k) return fail(SLC_ERR_INVALID_ARGUMENT, "bad activation buffer or stride");
    if (n > 0 && (!y || y_stride < n)) return fail(SLC_ERR_INVALID_ARGUMENT, "bad output buffer or stride");
    SLC_CUDA(cudaSetDevice(op->dev->index));
    cudaStream_t s = stream ? (cudaStream_t)stream : op->dev->stream;
    slc_result r = ensure_op_buffers(op, !x_is_device, !y_is_device);
    if (r != SLC_OK) return r;
    const size_t esz = x_dtype == SLC_F32 ? 4 : 2;
    const void *x_dev = x;
    long long xs = x_stride;
    if (!x_is_device) {
        SLC_CUDA(cudaMemcpy2DAsync(op->x_stage, (size_t)k * esz, x, (size_t)x_stride * esz, (size_t)k * esz, (size_t)rows,
                                   cudaMemcpyHostToDevice, s));
        x_dev = op->x_stage;
        xs = k;
    }
    if (n == 0) return SLC_OK;
    float *y_dev = y_is_device ? y : op->y_stage;
    const long long ys = y_is_device ? y_stride : n;
    if (op->flags & SLC_MATMUL_F32_ACTIVATIONS) {
        // the node keeps f32 activation math: no quantization, the dequant-fused f32 mat-vec in chunks of rows (every row
        // is computed the same way whatever the chunking)
        const int chunk = matvec_f32_rows(op->w->view.k_pad);
        op->last_kernel = SLC_KERNEL_F32;
        op->last_launches = 0;
        for (int64_t r0 = 0; r0 < rows; r0 += chunk) {
            const int m = (int)(rows - r0 < chunk ? rows - r0 : chunk);
            SLC_CUDA(launch_matvec_f32(op->w->view, x_dev, x_dtype, xs, (int)r0, m, y_dev, ys, s, nullptr));
            op->last_launches++;
            if (op->w->high) {   // Q5_K: the fifth bits, added onto the rows just written
                const Epilogue add{ nullptr, y_dev, ys };
                SLC_CUDA(launch_matvec_f32(op->w->high->view, x_dev, x_dtype, xs, (int)r0, m, y_dev, ys, s, &add));
                op->last_launches++;
            }
        }
        op->last_launches_total = op->last_launches;
    } else {
        r = quantize_and_run(op, nullptr, x_dev, x_dtype, rows, xs, y_dev, ys, s);
        if (r != SLC_OK) return r;
    }
    if (!y_is_device) {
        SLC_CUDA(cudaMemcpy2DAsync(y, (size_t)y_stride * 4, y_dev, (size_t)n * 4, (size_t)n * 4, (size_t)rows,
                                   cudaMemcpyDeviceToHost, s));
        SLC_CUDA(cudaStreamSynchronize(s));
    }
    return SLC_OK;
}

slc_result slc_matmul_run_allreduce(slc_matmul *op, slc_tp_exchange *x, const void *x_device, int32_t x_dtype, int64_t rows,
                                    int64_t x_stride, float *y, int64_t y_stride, void *stream)
{
    if (!op || !x) return fail(SLC_ERR_INVALID_ARGUMENT, "null op or exchange");
    if (op->flags & SLC_MATMUL_F32_ACTIVATIONS) return fail(SLC_ERR_INVALID_STATE, "this op keeps f32 activations: it takes no quantized ones and does not sum over ranks");
    if (x->dev != op->dev) return fail(SLC_ERR_INVALID_ARGUMENT, "op and exchange live on different devices");
    if (x_dtype != SLC_F32 && x_dtype != SLC_BF16) return fail(SLC_ERR_UNSUPPORTED, "activation dtype must be f32 or bf16");
    if (rows < 0) return fail(SLC_ERR_INVALID_ARGUMENT, "rows < 0");
    if (rows > op->max_rows) return fail(SLC_ERR_INVALID_STATE, "rows exceed the op's compiled bound");
    if (rows > x->max_rows && !x->comm) return fail(SLC_ERR_UNSUPPORTED, "rows exceed the exchange's bound and no communicator is attached");
    if (rows == 0 || op->w->n == 0) return SLC_OK;
    if (!x_device || x_stride < op->w->k) return fail(SLC_ERR_INVALID_ARGUMENT, "bad activation buffer or stride");
    if (!y || y_stride < op->w->n) return fail(SLC_ERR_INVALID_ARGUMENT, "bad output buffer or stride");
    SLC_CUDA(cudaSetDevice(op->dev->index));
    cudaStream_t s = stream ? (cudaStream_t)stream : op->dev->stream;
    slc_result r = ensure_op_buffers(op, false, false);
    if (r != SLC_OK) return r;
    return quantize_and_run(op, x, x_device, x_dtype, rows, x_stride, y, y_stride, s);
}

// ---- parity exports --------------------------------------------------------------------------------------------------

slc_result slc_debug_quantize(slc_device *d, const void *x, int32_t x_dtype, int64_t rows, int64_t k, int8_t *q, float *dd,
                              float *gs)
{
    if (!d || rows < 0) return fail(SLC_ERR_INVALID_ARGUMENT, "bad arguments");
    if (rows == 0) return SLC_OK;
    if (!x || !q || !dd || !gs) return fail(SLC_ERR_INVALID_ARGUMENT, "null buffer");
    slc_activation *a = nullptr;
    slc_result r = slc_activation_create(d, rows, k, &a);
    if (r != SLC_OK) return r;
    const size_t esz = x_dtype == SLC_F32 ? 4 : 2;
    void *xd = nullptr;
    cudaError_t e = cudaMalloc(&xd, (size_t)rows * k * esz);
    if (e == cudaSuccess) e = cudaMemcpyAsync(xd, x, (size_t)rows * k * esz, cudaMemcpyHostToDevice, d->stream);
    if (e != cudaSuccess) { slc_activation_destroy(a); if (xd) cudaFree(xd); return cuda_fail(e, "slc_debug_quantize"); }
    r = slc_activation_quantize(a, xd, x_dtype, rows, k, d->stream);
    if (r == SLC_OK) {
        const int kp = a->k_pad, rp = a->rows_pad;
        std::vector<float2> ds((size_t)(kp / 32) * rp);
        e = cudaMemcpy2DAsync(q, (size_t)k, a->planes.q, (size_t)kp, (size_t)k, (size_t)rows, cudaMemcpyDeviceToHost, d->stream);
        if (e == cudaSuccess) e = cudaMemcpy2DAsync(gs, (size_t)(k / 16) * 4, a->planes.gs, (size_t)(kp / 16) * 4,
                                                    (size_t)(k / 16) * 4, (size_t)rows, cudaMemcpyDeviceToHost, d->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(ds.data(), a->planes.ds, ds.size() * 8, cudaMemcpyDeviceToHost, d->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(d->stream);
        if (e != cudaSuccess) r = cuda_fail(e, "slc_debug_quantize");
        else {
            for (int64_t t = 0; t < rows; t++)
                for (int64_t b = 0; b < k / 32; b++) dd[t * (k / 32) + b] = ds[(size_t)b * rp + t].x;
        }
    }
    cudaFree(xd);
    slc_activation_destroy(a);
    return r;
}

slc_result slc_debug_block_dots(slc_matmul *op, const void *x, int32_t x_dtype, int64_t rows, int32_t *s32)
{
    if (!op || rows < 0) return fail(SLC_ERR_INVALID_ARGUMENT, "bad arguments");
    if (rows > op->max_rows) return fail(SLC_ERR_INVALID_STATE, "rows exceed the op's compiled bound");
    const long long n = op->w->n, k = op->w->k;
    if (rows == 0 || n == 0) return SLC_OK;
    if (!x || !s32) return fail(SLC_ERR_INVALID_ARGUMENT, "null buffer");
    slc_device *d = op->dev;
    SLC_CUDA(cudaSetDevice(d->index));
    slc_result r = ensure_op_buffers(op, true, true);
    if (r != SLC_OK) return r;
    const size_t esz = x_dtype == SLC_F32 ? 4 : 2;
    const size_t dump_bytes = (size_t)rows * n * (k / 32) * 4;
    int *dump = nullptr;
    SLC_CUDA(cudaMalloc(&dump, dump_bytes));
    cudaError_t e = cudaMemsetAsync(dump, 0xff, dump_bytes, d->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(op->x_stage, x, (size_t)rows * k * esz, cudaMemcpyHostToDevice, d->stream);
    if (e != cudaSuccess) { cudaFree(dump); return cuda_fail(e, "slc_debug_block_dots"); }
    if (!op->act) {
        r = slc_activation_create(op->dev, op->max_rows, op->w->k, &op->act);
        if (r != SLC_OK) { cudaFree(dump); return r; }
    }
    r = slc_activation_quantize(op->act, op->x_stage, x_dtype, rows, k, d->stream);
    // Q5_K (two Q4_K weights): the dots of the nibbles, then 16 times the dots of the fifth bits
    slc_weight *const whole = op->w, *const high = whole->high;
    whole->high = nullptr;
    if (r == SLC_OK) r = run_kernels(op, op->act, op->y_stage, n, dump, d->stream);
    if (r == SLC_OK) {
        e = cudaMemcpyAsync(s32, dump, dump_bytes, cudaMemcpyDeviceToHost, d->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(d->stream);
        if (e != cudaSuccess) r = cuda_fail(e, "slc_debug_block_dots");
    }
    if (r == SLC_OK && high) {
        std::vector<int32_t> bits;
        try { bits.resize(dump_bytes / 4); } catch (...) { r = fail(SLC_ERR_OUT_OF_MEMORY, "host allocation failed"); }
        if (r == SLC_OK) {
            op->w = high;
            r = run_kernels(op, op->act, op->y_stage, n, dump, d->stream);
            op->w = whole;
        }
        if (r == SLC_OK) {
            e = cudaMemcpyAsync(bits.data(), dump, dump_bytes, cudaMemcpyDeviceToHost, d->stream);
            if (e == cudaSuccess) e = cudaStreamSynchronize(d->stream);
            if (e != cudaSuccess) r = cuda_fail(e, "slc_debug_block_dots");
        }
        if (r == SLC_OK) {
            for (size_t i = 0; i < bits.size(); i++) s32[i] += 16 * bits[i];
        }
    }
    whole->high = high;
    cudaFree(dump);
    // A weight converted at upload: the kernels exported the dots with the device format's unsigned-code offset (Q8_0: 128);
    // the reference's decoder for the uploaded format uses another (Q5_0: 16). The difference times the block's
    // activation sum puts them right (host side: this is the parity export, not the data path).
    const int delta = unsigned_code_offset(op->w->src_fmt) - unsigned_code_offset(op->w->fmt);
    if (r == SLC_OK && delta != 0) {
        const long long kb = k / 32, kbp = op->act->k_pad / 32;
        std::vector<int> isum;
        try { isum.resize((size_t)rows * kbp); } catch (...) { return fail(SLC_ERR_OUT_OF_MEMORY, "host allocation failed"); }
        SLC_CUDA(cudaMemcpy(isum.data(), op->act->planes.isum, isum.size() * sizeof(int), cudaMemcpyDeviceToHost));
        for (long long t = 0; t < rows; t++) {
            for (long long row = 0; row < n; row++) {
                int32_t *o = s32 + (t * n + row) * kb;
                for (long long b = 0; b < kb; b++) o[b] += delta * isum[(size_t)(t * kbp + b)];
            }
        }
    }
    return r;
}

}  // extern "C"
