// The per-block core of the activation quantization, shared by the plain quantizer (quantize.cu) and the kernels that
// produce activations and quantize them in one pass (producers.cu). Bit-identical to the reference's CPU rule
// (src/Sharplight.Cpu/IntDot.cs:92-126 of the Sharplight tree): d = max|x| / 127, id = d != 0 ? 1 / d : 0,
// q = (int)(x * id + copysign(0.5, x * id)) -- round half away from zero through truncation, every step a separately
// rounded IEEE single operation (no fused multiply-add, no approximate division).
#pragma once

#include "internal.cuh"

namespace slc {

// Eight consecutive lanes share a 32-value block, four values each (v: this lane's, zero beyond the live range); all 32
// lanes of the warp must call. Writes every plane of `out` for (row, blk).
__device__ __forceinline__ void quantize_block_lane(const float (&v)[4], int row, int blk, int sub, int rows_pad, int k_pad,
                                                    const ActPlanes &out)
{
    const int nblk_pad = k_pad >> 5;
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

}  // namespace slc
