// Activation quantization to 8 bits per 32-value block, bit-identical to the reference's CPU rule
// (src/Sharplight.Cpu/IntDot.cs:92-126 of the Sharplight tree): d = max|x| / 127, id = d != 0 ? 1 / d : 0,
// q = (int)(x * id + copysign(0.5, x * id)) -- round half away from zero through truncation, every step a separately
// rounded IEEE single operation (no fused multiply-add, no approximate division).
// Eight lanes share a block (four values each); amax and the sums travel by lane shuffles.
#include "quantize.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace slc {

template <int DTYPE>
__global__ void __launch_bounds__(256) quantize_kernel(const void *__restrict__ xv, int rows, int rows_pad, int k,
                                                       int k_pad, long long x_stride, ActPlanes out)
{
    const int nblk_pad = k_pad >> 5;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long blk_global = tid >> 3;
    // rows_pad and nblk_pad are multiples of 8, so the grid covers the blocks exactly and every lane of a warp
    // reaches the shuffles below
    const int sub = (int)(tid & 7);
    const int row = (int)(blk_global / nblk_pad), blk = (int)(blk_global % nblk_pad);
    const bool live = row < rows && blk * 32 < k;

    pdl_wait();                // x may come from the kernel before this one
    pdl_launch_dependents();   // the MatMul that follows may start fetching its weights

    float v[4] = { 0.f, 0.f, 0.f, 0.f };
    if (live) {
        const long long base = (long long)row * x_stride + blk * 32 + sub * 4;
        if (DTYPE == 0) {
            const float *x = (const float *)xv + base;
            if ((((uintptr_t)x) & 15) == 0) {
                const float4 f = *reinterpret_cast<const float4 *>(x);
                v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
            } else {
                for (int i = 0; i < 4; i++) v[i] = x[i];
            }
        } else {
            // bf16 -> f32 is exact: the 16 bits become the high half of the f32
            const unsigned short *x = (const unsigned short *)xv + base;
            if ((((uintptr_t)x) & 7) == 0) {
                const uint2 u = *reinterpret_cast<const uint2 *>(x);   // four values in one 8-byte load
                v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xffff0000u);
                v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xffff0000u);
            } else {
                for (int i = 0; i < 4; i++) v[i] = __uint_as_float((unsigned)x[i] << 16);
            }
        }
    }
    quantize_block_lane(v, row, blk, sub, rows_pad, k_pad, out);
}

cudaError_t launch_quantize(const void *x, int x_dtype, int rows, int rows_pad, int k, int k_pad, long long x_stride,
                            ActPlanes out, cudaStream_t stream)
{
    const long long threads = (long long)rows_pad * (k_pad >> 5) * 8;
    if (threads == 0) return cudaSuccess;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    if (x_dtype == 0) return launch_pdl(quantize_kernel<0>, dim3(grid), dim3(256), 0, stream, x, rows, rows_pad, k, k_pad, x_stride, out);
    return launch_pdl(quantize_kernel<1>, dim3(grid), dim3(256), 0, stream, x, rows, rows_pad, k, k_pad, x_stride, out);
}

}  // namespace slc
