// Upload-time conversion of the formats that are served through the Q8_0 device layout: one thread rewrites one 32-value
// block as { f16 d; i8 q[32] }. Exact: Q5_0's value is d * (q5 - 16) and IQ4_NL's is d * codebook[nibble], both a signed
// byte times the block's own f16 scale (src/Sharplight.Cpu/Quant.cs:409-423, 463-480 of the Sharplight tree); value j < 16
// of a block comes from the low nibble of qs[j], value j + 16 from the high nibble.
#include "internal.cuh"

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
