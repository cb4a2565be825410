// Decode mat-vec with the activation quantization fused in: one launch per MatMul for 1..4 activation rows.
//
// Arithmetic: the reference's integer-dot MatMul (src/Sharplight.Cpu/IntDot.cs:92-126 for the 8-bit activation rule,
// src/Sharplight.Cpu/IntDot.Kernels.cs:12-29 and src/Sharplight.Shaders/Kernels/mmvq.slang:92-173,319-424 of the
// Sharplight tree for the block sums): exact int32 dots per 32-value block, f32 scaling.
//
// Shape of the kernel: one CTA owns 16 weight rows; its warps split K in 256-value super-tiles. Each lane first puts
// two super-tiles of weight loads in flight (128-bit streaming loads from the fragment-major layout, layout.cuh), and
// while those travel the CTA quantizes the activation rows into shared memory (8 lanes per 32-value block, bit-identical
// to quantize.cu). The dot loop then runs dp4a on registers against shared memory, with the next super-tile's loads
// always in flight. Integer sub-block scales (Q4_K, Q6_K) are applied in int32 before the single int->float conversion.
#include "internal.cuh"

#include <cuda_bf16.h>

namespace slc {

constexpr int FV_WARPS = 4;
constexpr int FV_MAX_SMEM = 100 * 1024;

template <int FMT> struct FTile;
template <> struct FTile<FMT_Q8_0> { uint4 q[8]; uint4 s[2]; };
template <> struct FTile<FMT_Q4_0> { uint4 q[4]; uint4 s[2]; };
template <> struct FTile<FMT_Q4_K> { uint4 q[4]; uint4 s[2]; };
template <> struct FTile<FMT_Q6_K> { uint4 q[6]; uint4 s[2]; unsigned short d[2]; };

template <int FMT>
__device__ __forceinline__ void load_tile(FTile<FMT> &tl, const WeightView &w, int rg, int st, int lane)
{
    const int g = lane >> 2;
    const int nst = w.k_pad >> 8;
    constexpr int NQ = FMT == FMT_Q8_0 ? 8 : FMT == FMT_Q6_K ? 6 : 4;
    const uint4 *qp = w.qs + ((long long)rg * nst + st) * (NQ * 32) + lane;
#pragma unroll
    for (int i = 0; i < NQ; i++) tl.q[i] = ld_stream(qp + 32 * i);
    const long long r0 = (long long)(rg * 16 + g), r1 = r0 + 8;
    if (FMT == FMT_Q8_0 || FMT == FMT_Q4_0) {
        const __half *sp = reinterpret_cast<const __half *>(w.sc);
        const int nblk_pad = w.k_pad >> 5;
        tl.s[0] = __ldg(reinterpret_cast<const uint4 *>(sp + r0 * nblk_pad + st * 8));
        tl.s[1] = __ldg(reinterpret_cast<const uint4 *>(sp + r1 * nblk_pad + st * 8));
    } else {
        const uint4 *hp = reinterpret_cast<const uint4 *>(w.sc);
        tl.s[0] = __ldg(hp + r0 * nst + st);
        tl.s[1] = __ldg(hp + r1 * nst + st);
    }
    if constexpr (FMT == FMT_Q6_K) {
        tl.d[0] = __ldg(reinterpret_cast<const unsigned short *>(w.d6) + r0 * nst + st);
        tl.d[1] = __ldg(reinterpret_cast<const unsigned short *>(w.d6) + r1 * nst + st);
    }
}

__device__ __forceinline__ float h2f(unsigned bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

// Shared-memory activations: q[m][k_pad] int8, ds[m][nblk_pad] (d, d * sum32 q).
struct SmemAct
{
    const int8_t *q;
    const float2 *ds;
    const int *isum;   // sum32(q) per block, [m][nblk_pad]
    int k_pad, nblk_pad;
};

// Parity export: the full 32-value block dot with the CPU decoder's unsigned codes, [m][n][k/32].
struct DumpCtx
{
    int *out;
    int n, k, rg, g, t;
};

template <bool DUMP>
__device__ __forceinline__ void export_dot(const DumpCtx &dc, const SmemAct &a, int blk, int m, int r, int partial,
                                           int c_export)
{
    if (!DUMP) return;
    int full = partial + __shfl_xor_sync(0xffffffffu, partial, 1);
    full += __shfl_xor_sync(0xffffffffu, full, 2);
    const int row = dc.rg * 16 + dc.g + 8 * r;
    if (dc.t == 0 && row < dc.n && blk * 32 < dc.k) {
        dc.out[((long long)m * dc.n + row) * (dc.k >> 5) + blk] = full + c_export * a.isum[m * a.nblk_pad + blk];
    }
}

template <int FMT, int M, bool DUMP>
__device__ __forceinline__ void compute_tile(const FTile<FMT> &tl, const SmemAct &a, int st, int t, float acc[2][M],
                                             const DumpCtx &dc)
{
    const int8_t *xq = a.q + st * 256;
    const float2 *xs = a.ds + st * 8;
    if constexpr (FMT == FMT_Q8_0 || FMT == FMT_Q4_0) {
        const unsigned s0w[4] = { tl.s[0].x, tl.s[0].y, tl.s[0].z, tl.s[0].w };
        const unsigned s1w[4] = { tl.s[1].x, tl.s[1].y, tl.s[1].z, tl.s[1].w };
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float dw0 = h2f(s0w[i >> 1] >> (16 * (i & 1))), dw1 = h2f(s1w[i >> 1] >> (16 * (i & 1)));
            if constexpr (FMT == FMT_Q8_0) {
#pragma unroll
                for (int m = 0; m < M; m++) {
                    const int2 x = *reinterpret_cast<const int2 *>(xq + m * a.k_pad + i * 32 + 8 * t);
                    const float dx = xs[m * a.nblk_pad + i].x;
                    const int s0 = __dp4a((int)tl.q[i].x, x.x, __dp4a((int)tl.q[i].y, x.y, 0));
                    const int s1 = __dp4a((int)tl.q[i].z, x.x, __dp4a((int)tl.q[i].w, x.y, 0));
                    acc[0][m] = fmaf(dw0 * dx, (float)s0, acc[0][m]);
                    acc[1][m] = fmaf(dw1 * dx, (float)s1, acc[1][m]);
                    export_dot<DUMP>(dc, a, st * 8 + i, m, 0, s0, 128);
                    export_dot<DUMP>(dc, a, st * 8 + i, m, 1, s1, 128);
                }
            } else {
                const unsigned wg = (i & 1) ? tl.q[i >> 1].z : tl.q[i >> 1].x;
                const unsigned wg8 = (i & 1) ? tl.q[i >> 1].w : tl.q[i >> 1].y;
                const int lo0 = (int)(wg & 0x0F0F0F0Fu), hi0 = (int)((wg >> 4) & 0x0F0F0F0Fu);
                const int lo1 = (int)(wg8 & 0x0F0F0F0Fu), hi1 = (int)((wg8 >> 4) & 0x0F0F0F0Fu);
                // the -8 offset of the codes: d_w * 8 * (d_x * sum q), carried by the lane whose index matches the block
                const float off = (t == (i & 3)) ? 8.0f : 0.0f;
#pragma unroll
                for (int m = 0; m < M; m++) {
                    const int8_t *xp = xq + m * a.k_pad + i * 32 + 4 * t;
                    const int xlo = *reinterpret_cast<const int *>(xp), xhi = *reinterpret_cast<const int *>(xp + 16);
                    const float2 ds = xs[m * a.nblk_pad + i];
                    const int s0 = __dp4a(lo0, xlo, __dp4a(hi0, xhi, 0));
                    const int s1 = __dp4a(lo1, xlo, __dp4a(hi1, xhi, 0));
                    const float corr = off * ds.y;
                    acc[0][m] = fmaf(dw0, fmaf(ds.x, (float)s0, -corr), acc[0][m]);
                    acc[1][m] = fmaf(dw1, fmaf(ds.x, (float)s1, -corr), acc[1][m]);
                    export_dot<DUMP>(dc, a, st * 8 + i, m, 0, s0, 0);
                    export_dot<DUMP>(dc, a, st * 8 + i, m, 1, s1, 0);
                }
            }
        }
    } else if constexpr (FMT == FMT_Q4_K) {
        float d[2], dmin[2];
        unsigned sc[2][2], mn[2][2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const uint4 h = tl.s[r];
            d[r] = h2f(h.x & 0xffffu);
            dmin[r] = h2f(h.x >> 16);
            sc[r][0] = h.y & 0x3F3F3F3Fu;
            mn[r][0] = h.z & 0x3F3F3F3Fu;
            sc[r][1] = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
            mn[r][1] = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
        }
        float part[2][M];
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int m = 0; m < M; m++) part[r][m] = 0.0f;
#pragma unroll
        for (int sb = 0; sb < 8; sb++) {
            const int ch = sb >> 1, sh = 4 * (sb & 1);
            const int u0 = (int)((tl.q[ch].x >> sh) & 0x0F0F0F0Fu), u1 = (int)((tl.q[ch].y >> sh) & 0x0F0F0F0Fu);
            const int u2 = (int)((tl.q[ch].z >> sh) & 0x0F0F0F0Fu), u3 = (int)((tl.q[ch].w >> sh) & 0x0F0F0F0Fu);
            const int sc0 = (int)((sc[0][sb >> 2] >> (8 * (sb & 3))) & 0xffu);
            const int sc1 = (int)((sc[1][sb >> 2] >> (8 * (sb & 3))) & 0xffu);
#pragma unroll
            for (int m = 0; m < M; m++) {
                const int2 x = *reinterpret_cast<const int2 *>(xq + m * a.k_pad + sb * 32 + 8 * t);
                const float dx = xs[m * a.nblk_pad + sb].x;
                const int r0 = __dp4a(u0, x.x, __dp4a(u1, x.y, 0)), r1 = __dp4a(u2, x.x, __dp4a(u3, x.y, 0));
                const int s0 = r0 * sc0, s1 = r1 * sc1;   // |s| <= 60960 * 63 < 2^22: exact
                part[0][m] = fmaf((float)s0, dx, part[0][m]);
                part[1][m] = fmaf((float)s1, dx, part[1][m]);
                export_dot<DUMP>(dc, a, st * 8 + sb, m, 0, r0, 0);
                export_dot<DUMP>(dc, a, st * 8 + sb, m, 1, r1, 0);
            }
        }
        // the mins of sub-blocks t and t + 4 are this lane's share of the offset term
        float mpart[2][M];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const float m_lo = (float)((mn[r][0] >> (8 * t)) & 0xffu), m_hi = (float)((mn[r][1] >> (8 * t)) & 0xffu);
#pragma unroll
            for (int m = 0; m < M; m++) {
                mpart[r][m] = m_lo * xs[m * a.nblk_pad + t].y;
                mpart[r][m] = fmaf(m_hi, xs[m * a.nblk_pad + t + 4].y, mpart[r][m]);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int m = 0; m < M; m++) acc[r][m] += fmaf(d[r], part[r][m], -dmin[r] * mpart[r][m]);
    } else {  // Q6_K
        const float d[2] = { h2f(tl.d[0]), h2f(tl.d[1]) };
        const unsigned scw[2][4] = { { tl.s[0].x, tl.s[0].y, tl.s[0].z, tl.s[0].w },
                                     { tl.s[1].x, tl.s[1].y, tl.s[1].z, tl.s[1].w } };
        float part[2][M];
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int m = 0; m < M; m++) part[r][m] = 0.0f;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint4 A = tl.q[3 * h], B = tl.q[3 * h + 1], H = tl.q[3 * h + 2];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int blk = 4 * h + j;
                int code[2][2], sc8[2][2];  // [16-value group][row]
#pragma unroll
                for (int hl = 0; hl < 2; hl++) {
                    const unsigned lw[2] = { (j & 1) ? (hl ? A.w : A.y) : (hl ? A.z : A.x),
                                             (j & 1) ? (hl ? B.w : B.y) : (hl ? B.z : B.x) };
                    const unsigned hw[2] = { hl ? H.y : H.x, hl ? H.w : H.z };
                    const int gi = 8 * h + 2 * j + hl;
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        const unsigned lo4 = ((j & 2) ? (lw[r] >> 4) : lw[r]) & 0x0F0F0F0Fu;
                        const unsigned hi2 = ((hw[r] >> (2 * j)) & 0x03030303u) << 4;
                        code[hl][r] = (int)__vsub4(lo4 | hi2, 0x20202020u);
                        sc8[hl][r] = (int)(signed char)((scw[r][gi >> 2] >> (8 * (gi & 3))) & 0xffu);
                    }
                }
#pragma unroll
                for (int m = 0; m < M; m++) {
                    const int8_t *xp = xq + m * a.k_pad + blk * 32 + 4 * t;
                    const int x0 = *reinterpret_cast<const int *>(xp), x1 = *reinterpret_cast<const int *>(xp + 16);
                    const float dx = xs[m * a.nblk_pad + blk].x;
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        // two 16-value groups with their int8 scales: |sum| <= 2 * 16*32*127 * 128 < 2^24, exact
                        const int p0 = __dp4a(code[0][r], x0, 0), p1 = __dp4a(code[1][r], x1, 0);
                        const int s = p0 * sc8[0][r] + p1 * sc8[1][r];
                        part[r][m] = fmaf((float)s, dx, part[r][m]);
                        export_dot<DUMP>(dc, a, st * 8 + blk, m, r, p0 + p1, 32);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int m = 0; m < M; m++) acc[r][m] = fmaf(d[r], part[r][m], acc[r][m]);
    }
}

// Quantizes x[M][k] into shared memory; the same operations, in the same order, as quantize.cu.
template <int M>
__device__ __forceinline__ void quantize_to_smem(const void *xv, int x_dtype, long long x_stride, int k, int k_pad,
                                                 int8_t *sq, float2 *sds, int *sisum)
{
    const int nblk_pad = k_pad >> 5;
    const int sub = threadIdx.x & 7;
    for (int b = threadIdx.x >> 3; b < M * nblk_pad; b += (FV_WARPS * 32) >> 3) {
        const int m = b / nblk_pad, blk = b - m * nblk_pad;
        float v[4] = { 0.f, 0.f, 0.f, 0.f };
        if (blk * 32 < k) {
            const long long base = (long long)m * x_stride + blk * 32 + sub * 4;
            if (x_dtype == 0) {
                const float *x = (const float *)xv + base;
                if ((((uintptr_t)x) & 15) == 0) {
                    const float4 f = __ldg(reinterpret_cast<const float4 *>(x));
                    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                } else {
                    for (int i = 0; i < 4; i++) v[i] = __ldg(x + i);
                }
            } else {
                const __nv_bfloat16 *x = (const __nv_bfloat16 *)xv + base;
                for (int i = 0; i < 4; i++) v[i] = __bfloat162float(x[i]);
            }
        }
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
        int r[4], s = 0;
        for (int i = 0; i < 4; i++) {
            const float wv = __fmul_rn(v[i], id);
            r[i] = __float2int_rz(__fadd_rn(wv, copysignf(0.5f, wv)));
            s += r[i];
        }
        *reinterpret_cast<unsigned *>(sq + m * k_pad + blk * 32 + sub * 4) =
            (unsigned)(r[0] & 0xff) | ((unsigned)(r[1] & 0xff) << 8) | ((unsigned)(r[2] & 0xff) << 16) |
            ((unsigned)(r[3] & 0xff) << 24);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (sub == 0) {
            sds[m * nblk_pad + blk] = make_float2(d, __fmul_rn(d, (float)s));
            sisum[m * nblk_pad + blk] = s;
        }
    }
}

template <int FMT, int M, bool DUMP>
__global__ void __launch_bounds__(FV_WARPS * 32)
fused_matvec_kernel(const WeightView w, const void *__restrict__ x, int x_dtype, long long x_stride,
                    float *__restrict__ y, long long y_stride, int *dump)
{
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float red[FV_WARPS][16][M];
    const int nblk_pad = w.k_pad >> 5, nst = w.k_pad >> 8;
    int8_t *sq = reinterpret_cast<int8_t *>(smem);
    float2 *sds = reinterpret_cast<float2 *>(smem + (size_t)M * w.k_pad);
    int *sisum = reinterpret_cast<int *>(smem + (size_t)M * w.k_pad + (size_t)M * nblk_pad * 8);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, t = lane & 3, g = lane >> 2;
    const int rg = blockIdx.x;

    // weight loads first: they are in flight while the activations are quantized
    FTile<FMT> ta, tb;
    int st = warp;
    if (st < nst) load_tile<FMT>(ta, w, rg, st, lane);
    if (st + FV_WARPS < nst) load_tile<FMT>(tb, w, rg, st + FV_WARPS, lane);

    // M * nblk_pad is a multiple of 8 and the stride below keeps the 8 lanes of a block together
    quantize_to_smem<M>(x, x_dtype, x_stride, w.k, w.k_pad, sq, sds, sisum);
    __syncthreads();

    const SmemAct act{ sq, sds, sisum, w.k_pad, nblk_pad };
    const DumpCtx dc{ dump, w.n, w.k, rg, g, t };
    float acc[2][M];
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
        for (int m = 0; m < M; m++) acc[r][m] = 0.0f;

    for (; st < nst; st += 2 * FV_WARPS) {
        compute_tile<FMT, M, DUMP>(ta, act, st, t, acc, dc);
        if (st + 2 * FV_WARPS < nst) load_tile<FMT>(ta, w, rg, st + 2 * FV_WARPS, lane);
        if (st + FV_WARPS < nst) {
            compute_tile<FMT, M, DUMP>(tb, act, st + FV_WARPS, t, acc, dc);
            if (st + 3 * FV_WARPS < nst) load_tile<FMT>(tb, w, rg, st + 3 * FV_WARPS, lane);
        }
    }

#pragma unroll
    for (int r = 0; r < 2; r++) {
#pragma unroll
        for (int m = 0; m < M; m++) {
            float v = acc[r][m];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (t == 0) red[warp][g + 8 * r][m] = v;
        }
    }
    __syncthreads();
    if (threadIdx.x < 16 * M) {
        const int m = threadIdx.x / 16, rr = threadIdx.x % 16;
        float v = 0.0f;
#pragma unroll
        for (int wi = 0; wi < FV_WARPS; wi++) v += red[wi][rr][m];
        const int row = blockIdx.x * 16 + rr;
        if (row < w.n) y[(long long)m * y_stride + row] = v;
    }
}

size_t fused_matvec_smem(int rows, int k_pad) { return (size_t)rows * (k_pad + (k_pad >> 5) * 12); }

bool fused_matvec_fits(int rows, int k_pad) { return rows >= 1 && rows <= 4 && fused_matvec_smem(rows, k_pad) <= FV_MAX_SMEM; }

template <int FMT, int M, bool DUMP>
static cudaError_t launch_one(const WeightView &w, const void *x, int x_dtype, long long x_stride, float *y,
                              long long y_stride, int *dump, cudaStream_t stream)
{
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = fused_matvec_kernel<FMT, M, DUMP>;
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FV_MAX_SMEM);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const size_t smem = fused_matvec_smem(M, w.k_pad);
    kernel<<<w.n_pad / 16, FV_WARPS * 32, smem, stream>>>(w, x, x_dtype, x_stride, y, y_stride, dump);
    return cudaGetLastError();
}

template <int FMT>
static cudaError_t launch_fmt(const WeightView &w, const void *x, int x_dtype, long long x_stride, int rows, float *y,
                              long long y_stride, int *dump, cudaStream_t stream)
{
#define SLC_ROWS(MM)                                                                                     \
    case MM:                                                                                             \
        return dump ? launch_one<FMT, MM, true>(w, x, x_dtype, x_stride, y, y_stride, dump, stream)      \
                    : launch_one<FMT, MM, false>(w, x, x_dtype, x_stride, y, y_stride, nullptr, stream);
    switch (rows) {
        SLC_ROWS(1) SLC_ROWS(2) SLC_ROWS(3) SLC_ROWS(4)
    default: return cudaErrorInvalidValue;
    }
#undef SLC_ROWS
}

cudaError_t launch_fused_matvec(const WeightView &w, const void *x, int x_dtype, long long x_stride, int rows, float *y,
                                long long y_stride, int *dump, cudaStream_t stream)
{
    if (w.n_pad == 0 || rows == 0) return cudaSuccess;
    switch (w.fmt) {
    case FMT_Q8_0: return launch_fmt<FMT_Q8_0>(w, x, x_dtype, x_stride, rows, y, y_stride, dump, stream);
    case FMT_Q4_0: return launch_fmt<FMT_Q4_0>(w, x, x_dtype, x_stride, rows, y, y_stride, dump, stream);
    case FMT_Q4_K: return launch_fmt<FMT_Q4_K>(w, x, x_dtype, x_stride, rows, y, y_stride, dump, stream);
    case FMT_Q6_K: return launch_fmt<FMT_Q6_K>(w, x, x_dtype, x_stride, rows, y, y_stride, dump, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace slc
