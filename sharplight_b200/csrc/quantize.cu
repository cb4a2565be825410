// Activation quantization to 8 bits per 32-value block, bit-identical to the reference's CPU rule
// (src/Sharplight.Cpu/IntDot.cs:92-126 of the Sharplight tree): d = max|x| / 127, id = d != 0 ? 1 / d : 0,
// q = (int)(x * id + copysign(0.5, x * id)) -- round half away from zero through truncation, every step a separately
// rounded IEEE single operation (no fused multiply-add, no approximate division).
// Eight lanes share a block (four values each); amax and the sums travel by lane shuffles.
#include "internal.cuh"

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
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    int r[4];
    int s = 0;
    for (int i = 0; i < 4; i++) {
        const float w = __fmul_rn(v[i], id);
        r[i] = __float2int_rz(__fadd_rn(w, copysignf(0.5f, w)));
        s += r[i];
    }
    const unsigned packed = (unsigned)(r[0] & 0xff) | ((unsigned)(r[1] & 0xff) << 8) | ((unsigned)(r[2] & 0xff) << 16) |
                            ((unsigned)(r[3] & 0xff) << 24);
    *reinterpret_cast<unsigned *>(out.q + (long long)row * k_pad + blk * 32 + sub * 4) = packed;
    if (out.q_tiled) {
        // the same codes as 8-token x 16-byte core matrices, [super-tile][token / 8][16-byte K chunk][token % 8][16]:
        // a 128-token x 256-value tile is then 32 KB of contiguous bytes, ready for one bulk copy into the layout the
        // tensor core reads
        const int kk = blk * 32 + sub * 4;
        const long long off = ((long long)(kk >> 8) * (rows_pad >> 3) + (row >> 3)) * 2048 + ((kk & 255) >> 4) * 128 +
                              (row & 7) * 16 + (kk & 15);
        *reinterpret_cast<unsigned *>(out.q_tiled + off) = packed;
    }
    if (out.q_sw) {
        // the same codes once more, in the 128-byte swizzled operand rows the tile kernel's tensor-core instructions read:
        // [k / 128][token / 8][token % 8][eight 16-byte chunks, chunk c stored at c ^ (token % 8)]; the tile of NT tokens
        // x 128 K-values is then NT x 128 contiguous bytes, one bulk copy
        const int kk = blk * 32 + sub * 4;
        const long long off = ((long long)(kk >> 7) * (rows_pad >> 3) + (row >> 3)) * 1024 + (row & 7) * 128 +
                              ((((kk & 127) >> 4) ^ (row & 7)) << 4) + (kk & 15);
        *reinterpret_cast<unsigned *>(out.q_sw + off) = packed;
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);        // sum of this lane's 16-value group
    const int s_other = __shfl_xor_sync(0xffffffffu, s, 4);
    if ((sub & 3) == 0) {
        out.gs[(long long)row * (k_pad >> 4) + blk * 2 + (sub >> 2)] = __fmul_rn(d, (float)s);
    }
    if (sub == 0) {
        const int s32 = s + s_other;
        const float sxv = __fmul_rn(d, (float)s32);
        out.ds[(long long)blk * rows_pad + row] = make_float2(d, sxv);
        out.dx[(long long)blk * rows_pad + row] = d;
        out.sx[(long long)blk * rows_pad + row] = sxv;
        out.isum[(long long)row * nblk_pad + blk] = s32;
        if (out.sx2) {
            // d * sum32(q) as two tf32 values (high 11 significant bits, and the rest), in 64-byte swizzled operand
            // rows: [k / 256][token / 8][token % 8][four 16-byte chunks: hi of blocks 0-3, hi 4-7, lo 0-3, lo 4-7]
            const float hi = __uint_as_float(__float_as_uint(sxv) & 0xFFFFE000u), lo = __fsub_rn(sxv, hi);
            const int bq = blk & 7, sw = (row & 7) >> 1;
            uint8_t *base = out.sx2 + ((long long)(blk >> 3) * (rows_pad >> 3) + (row >> 3)) * 512 + (row & 7) * 64 + (bq & 3) * 4;
            *reinterpret_cast<float *>(base + (((bq >> 2) ^ sw) << 4)) = hi;
            *reinterpret_cast<float *>(base + (((2 + (bq >> 2)) ^ sw) << 4)) = lo;
        }
    }
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
