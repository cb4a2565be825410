// Kernels on either side of the quantized MatMul that produce its 8-bit activations, or consume its result, in one pass:
//
//   rmsnorm + quantize      y = (x * 1 / sqrt(sum x^2 / K + eps)) * w   (src/Sharplight.Cpu/RowOp.cs:63-76 and
//                           Simd.cs:464-483 of the Sharplight tree), quantized as it is produced: the norm in front of
//                           the q/k/v and the gate/up MatMuls writes the activation planes itself, the way the
//                           reference lets its norm kernels write the copy the next MatMul reads
//                           (src/Sharplight.Shaders/Lowering/GraphLowerer.IntDot.cs:146-184)
//   silu(gate) * up + quantize   the gated-FFN tail in front of the down projection (silu(v) = v / (1 + exp(-v)),
//                           src/Sharplight.Cpu/ScalarMath.cs:552-577)
//   arg-max over rows       the sampling head after the lm_head MatMul: only one index per sequence leaves the device
//                           instead of the row of logits (first maximum wins, NaN never beats a number:
//                           src/Sharplight.Cpu/RowOp.cs:174-189)
//
// The quantization itself is quantize.cuh's, bit for bit: quantizing the f32 output of these kernels with the plain
// quantizer gives the same planes.
#include "quantize.cuh"

#include <cuda_bf16.h>

namespace slc {

template <int DTYPE>
__device__ __forceinline__ void load4(const void *xv, long long base, bool live, float (&v)[4])
{
    v[0] = v[1] = v[2] = v[3] = 0.0f;
    if (!live) return;
    if (DTYPE == 0) {
        const float *x = (const float *)xv + base;
        if ((((uintptr_t)x) & 15) == 0) {
            const float4 f = *reinterpret_cast<const float4 *>(x);
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
            for (int i = 0; i < 4; i++) v[i] = x[i];
        }
    } else {
        const unsigned short *x = (const unsigned short *)xv + base;
        for (int i = 0; i < 4; i++) v[i] = __uint_as_float((unsigned)x[i] << 16);
    }
}

// One CTA of 1024 threads per (padded) row: sum of squares over K, then the row is read again (from L1 / L2), scaled and
// quantized.
template <int DTYPE>
__global__ void __launch_bounds__(1024) rmsnorm_quantize_kernel(const void *__restrict__ xv, int rows, int rows_pad, int k, int k_pad,
                                                               long long x_stride, const float *__restrict__ weight, float eps,
                                                               float *y, long long y_stride, ActPlanes out)
{
    __shared__ float warp_sums[32];
    __shared__ float scale_s;
    const int row = blockIdx.x;
    const bool row_live = row < rows;
    pdl_wait();
    pdl_launch_dependents();

    float sum = 0.0f;
    if (row_live) {
        for (int i = threadIdx.x * 4; i < k; i += 1024 * 4) {
            float v[4];
            load4<DTYPE>(xv, (long long)row * x_stride + i, true, v);
            sum = fmaf(v[0], v[0], sum); sum = fmaf(v[1], v[1], sum); sum = fmaf(v[2], v[2], sum); sum = fmaf(v[3], v[3], sum);
        }
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int i = 0; i < 32; i++) t += warp_sums[i];
        scale_s = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)k), eps)));
    }
    __syncthreads();
    const float scale = scale_s;

    // blocks of 32 values, eight lanes each; k_pad is a multiple of 256, so whole warps stay together
    const int sub = threadIdx.x & 7;
    for (int blk = threadIdx.x >> 3; blk < (k_pad >> 5); blk += 128) {
        const bool live = row_live && blk * 32 < k;
        float v[4];
        load4<DTYPE>(xv, (long long)row * x_stride + blk * 32 + sub * 4, live, v);
        if (live) {
            const float4 w = weight ? *reinterpret_cast<const float4 *>(weight + blk * 32 + sub * 4) : make_float4(1.f, 1.f, 1.f, 1.f);
            const float wv[4] = { w.x, w.y, w.z, w.w };
#pragma unroll
            for (int i = 0; i < 4; i++) v[i] = weight ? __fmul_rn(__fmul_rn(v[i], scale), wv[i]) : __fmul_rn(v[i], scale);
            if (y) *reinterpret_cast<float4 *>(y + (long long)row * y_stride + blk * 32 + sub * 4) = make_float4(v[0], v[1], v[2], v[3]);
        }
        quantize_block_lane(v, row, blk, sub, rows_pad, k_pad, out);
    }
}

__global__ void __launch_bounds__(256) silu_mul_quantize_kernel(const float *__restrict__ gate, long long gate_stride,
                                                                const float *__restrict__ up, long long up_stride, int rows,
                                                                int rows_pad, int k, int k_pad, float *y, long long y_stride,
                                                                ActPlanes out)
{
    const int nblk_pad = k_pad >> 5;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long blk_global = tid >> 3;
    const int sub = (int)(tid & 7);
    const int row = (int)(blk_global / nblk_pad), blk = (int)(blk_global % nblk_pad);
    const bool live = row < rows && blk * 32 < k;
    pdl_wait();
    pdl_launch_dependents();
    float g[4], u[4], v[4] = { 0.f, 0.f, 0.f, 0.f };
    load4<0>(gate, (long long)row * gate_stride + blk * 32 + sub * 4, live, g);
    load4<0>(up, (long long)row * up_stride + blk * 32 + sub * 4, live, u);
    if (live) {
#pragma unroll
        for (int i = 0; i < 4; i++) v[i] = __fmul_rn(__fdiv_rn(g[i], 1.0f + expf(-g[i])), u[i]);
        if (y) {
            float *dst = y + (long long)row * y_stride + blk * 32 + sub * 4;
            if ((((uintptr_t)dst) & 15) == 0) *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            else for (int i = 0; i < 4; i++) dst[i] = v[i];
        }
    }
    quantize_block_lane(v, row, blk, sub, rows_pad, k_pad, out);
}

// One CTA per row. A thread keeps the first maximum of its strided positions; pairs then meet by (larger value, lower
// index). NaN never wins against a number; a row whose first element is NaN answers 0, as the sequential scan does.
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float *__restrict__ y, long long y_stride, int n, int *out)
{
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    pdl_wait();
    pdl_launch_dependents();
    const float *x = y + (long long)blockIdx.x * y_stride;
    float bv = 0.0f;
    int bi = -1;   // -1: nothing seen yet
    for (int i = threadIdx.x; i < n; i += 1024) {
        const float v = x[i];
        if (v == v && (bi < 0 || v > bv)) { bv = v; bi = i; }
    }
    auto better = [](float v, int i, float bv, int bi) { return i >= 0 && (bi < 0 || v > bv || (v == bv && i < bi)); };
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { best_v[threadIdx.x >> 5] = bv; best_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        bv = best_v[threadIdx.x]; bi = best_i[threadIdx.x];
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (threadIdx.x == 0) out[blockIdx.x] = (bi < 0 || x[0] != x[0]) ? 0 : bi;
    }
}

cudaError_t launch_rmsnorm_quantize(const void *x, int x_dtype, int rows, int rows_pad, int k, int k_pad, long long x_stride,
                                    const float *weight, float eps, float *y, long long y_stride, ActPlanes out, cudaStream_t stream)
{
    if (rows_pad == 0) return cudaSuccess;
    if (x_dtype == 0) {
        return launch_pdl(rmsnorm_quantize_kernel<0>, dim3(rows_pad), dim3(1024), 0, stream, x, rows, rows_pad, k, k_pad, x_stride,
                          weight, eps, y, y_stride, out);
    }
    return launch_pdl(rmsnorm_quantize_kernel<1>, dim3(rows_pad), dim3(1024), 0, stream, x, rows, rows_pad, k, k_pad, x_stride,
                      weight, eps, y, y_stride, out);
}

cudaError_t launch_silu_mul_quantize(const float *gate, long long gate_stride, const float *up, long long up_stride, int rows,
                                     int rows_pad, int k, int k_pad, float *y, long long y_stride, ActPlanes out, cudaStream_t stream)
{
    const long long threads = (long long)rows_pad * (k_pad >> 5) * 8;
    if (threads == 0) return cudaSuccess;
    return launch_pdl(silu_mul_quantize_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, stream, gate, gate_stride, up,
                      up_stride, rows, rows_pad, k, k_pad, y, y_stride, out);
}

cudaError_t launch_argmax_rows(const float *y, long long y_stride, int rows, int n, int *out, cudaStream_t stream)
{
    if (rows == 0) return cudaSuccess;
    return launch_pdl(argmax_rows_kernel, dim3(rows), dim3(1024), 0, stream, y, y_stride, n, out);
}

}  // namespace slc
