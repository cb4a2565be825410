// Upload-time conversion of the formats that are served through another format's device layout. Q5_0 / IQ4_NL -> Q8_0:
// one thread rewrites one 32-value
// block as { f16 d; i8 q[32] }. Exact: Q5_0's value is d * (q5 - 16) and IQ4_NL's is d * codebook[nibble], both a signed
// byte times the block's own f16 scale (src/Sharplight.Cpu/Quant.cs:409-423, 463-480 of the Sharplight tree); value j < 16
// of a block comes from the low nibble of qs[j], value j + 16 from the high nibble.
#include "internal.cuh"

#include <cuda_fp16.h>

namespace slc {

__constant__ signed char c_iq4nl_values[16] = { -127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113 };

__global__ void convert_to_q8_0_kernel(int src_fmt, const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, long long blocks)
{
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    const uint8_t *p = src + b * source_block_bytes(src_fmt);
    uint8_t *o = dst + b * 34;
    o[0] = p[0];
    o[1] = p[1];
    if (src_fmt == FMT_Q5_0) {
        const unsigned qh = (unsigned)p[2] | ((unsigned)p[3] << 8) | ((unsigned)p[4] << 16) | ((unsigned)p[5] << 24);
        for (int j = 0; j < 16; j++) {
            const int lo = (p[6 + j] & 15) | (int)(((qh >> j) & 1u) << 4), hi = (p[6 + j] >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4);
            o[2 + j] = (uint8_t)(signed char)(lo - 16);
            o[18 + j] = (uint8_t)(signed char)(hi - 16);
        }
    } else {   // FMT_IQ4_NL
        for (int j = 0; j < 16; j++) {
            o[2 + j] = (uint8_t)c_iq4nl_values[p[2 + j] & 15];
            o[18 + j] = (uint8_t)c_iq4nl_values[p[2 + j] >> 4];
        }
    }
}

// Q5_K -> two Q4_K blocks (layout.cuh). One thread per 256-value block. A block whose 16 * d leaves the f16 range raises
// *overflow (the upload is then refused: the split would not be exact).
__global__ void split_q5_k_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ low, uint8_t *__restrict__ high,
                                  long long blocks, int *overflow)
{
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    const uint8_t *p = src + b * 176;
    uint8_t *lo = low + b * 144, *hi = high + b * 144;
    for (int i = 0; i < 16; i++) lo[i] = p[i];                 // d, dmin, scales
    for (int i = 0; i < 128; i++) lo[16 + i] = p[48 + i];      // the nibbles
    const unsigned short dbits = (unsigned short)(p[0] | (p[1] << 8));
    const float d = __half2float(__ushort_as_half(dbits));
    const __half d16 = __float2half_rn(16.0f * d);
    if (!(__half2float(d16) == 16.0f * d)) atomicExch(overflow, 1);   // also catches NaN
    const unsigned short hbits = __half_as_ushort(d16);
    hi[0] = (uint8_t)(hbits & 0xff);
    hi[1] = (uint8_t)(hbits >> 8);
    hi[2] = 0;
    hi[3] = 0;                                                  // dmin' = 0: the mins are not counted twice
    for (int i = 0; i < 12; i++) hi[4 + i] = p[4 + i];
    const uint8_t *qh = p + 16;
    for (int j = 0; j < 4; j++) {
        for (int l = 0; l < 32; l++) hi[16 + 32 * j + l] = (uint8_t)(((qh[l] >> (2 * j)) & 1) | (((qh[l] >> (2 * j + 1)) & 1) << 4));
    }
}

cudaError_t launch_split_q5_k(const uint8_t *src, uint8_t *low, uint8_t *high, long long blocks, int *overflow, cudaStream_t stream)
{
    if (blocks <= 0) return cudaSuccess;
    const long long grid = (blocks + 127) / 128;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidValue;
    split_q5_k_kernel<<<(unsigned)grid, 128, 0, stream>>>(src, low, high, blocks, overflow);
    return cudaGetLastError();
}

cudaError_t launch_convert_to_q8_0(int src_fmt, const uint8_t *src, uint8_t *dst, long long blocks, cudaStream_t stream)
{
    if (src_fmt != FMT_Q5_0 && src_fmt != FMT_IQ4_NL) return cudaErrorInvalidValue;
    if (blocks <= 0) return cudaSuccess;
    const long long grid = (blocks + 255) / 256;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidValue;
    convert_to_q8_0_kernel<<<(unsigned)grid, 256, 0, stream>>>(src_fmt, src, dst, blocks);
    return cudaGetLastError();
}

}  // namespace slc
