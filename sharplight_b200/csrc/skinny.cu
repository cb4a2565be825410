// Skinny integer-dot GEMM for 3..64 activation rows (batched decode, speculative verification, short prefill).
//
// Same arithmetic as matvec.cu -- exact int32 block dots scaled in f32 (src/Sharplight.Cpu/IntDot.Kernels.cs:12-29,
// src/Sharplight.Shaders/Kernels/mmq.slang:224-233 of the Sharplight tree) -- but the int32 dots come from int8
// tensor-core tiles: the 16 weight rows of a CTA are the M operand of m16n8k32 (m16n8k16 for Q6_K, whose scales
// change every 16 values), eight activation rows are the N operand, one 32-value block is one K step. The weight
// fragments come straight from the fragment-major layout (one 128-bit streaming load per lane per tile, unpacked
// in registers): the kernel stays a weight-streaming, HBM-bound kernel; the reference's skinny kernel instead decodes
// to f16 (src/Sharplight.Shaders/Kernels/matmul_skinny.slang:1-31).
#include "internal.cuh"

namespace slc {

constexpr int SK_WARPS = 4;

__device__ __forceinline__ void mma_u8s8_k32(int c[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, int b0, int b1)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ void mma_s8s8_k32(int c[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, int b0, int b1)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ void mma_s8s8_k16(int c[4], unsigned a0, unsigned a1, int b0)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

template <int NT, bool DUMP>
struct SkCtx
{
    const WeightView &w;
    const ActView &a;
    int row0, rg, g, t;
    int *dump;
    float acc[NT][4];  // per token tile: (row g, tok 2t), (row g, tok 2t+1), (row g+8, tok 2t), (row g+8, tok 2t+1)

    // c: the int32 tile of one block (or 16-value group) for token tile nt.
    __device__ __forceinline__ void scale_tile(int blk, int nt, const int c[4], const float scale[2],
                                               const float minv[2], bool has_min, const float4 dsp)
    {
        acc[nt][0] = fmaf(scale[0] * dsp.x, (float)c[0], acc[nt][0]);
        acc[nt][1] = fmaf(scale[0] * dsp.z, (float)c[1], acc[nt][1]);
        acc[nt][2] = fmaf(scale[1] * dsp.x, (float)c[2], acc[nt][2]);
        acc[nt][3] = fmaf(scale[1] * dsp.z, (float)c[3], acc[nt][3]);
        if (has_min) {
            acc[nt][0] = fmaf(-minv[0], dsp.y, acc[nt][0]);
            acc[nt][1] = fmaf(-minv[0], dsp.w, acc[nt][1]);
            acc[nt][2] = fmaf(-minv[1], dsp.y, acc[nt][2]);
            acc[nt][3] = fmaf(-minv[1], dsp.w, acc[nt][3]);
        }
    }

    __device__ __forceinline__ float4 load_ds(int blk, int nt) const
    {
        return __ldg(reinterpret_cast<const float4 *>(&a.ds[(long long)blk * a.rows_pad + row0 + nt * 8 + 2 * t]));
    }

    __device__ __forceinline__ void export_tile(int blk, int nt, const int c[4], int c_export) const
    {
        if (!DUMP) return;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int row = rg * 16 + g + 8 * (e >> 1);
            const int m = nt * 8 + 2 * t + (e & 1);
            const int tok = row0 + m;
            if (row < w.n && tok < a.rows && blk * 32 < w.k) {
                const int add = c_export ? c_export * __ldg(&a.isum[(long long)tok * (a.k_pad >> 5) + blk]) : 0;
                dump[((long long)m * w.n + row) * (w.k >> 5) + blk] = c[e] + add;
            }
        }
    }
};

__device__ __forceinline__ float half_of(unsigned word, int which)
{
    return __half2float(__ushort_as_half((unsigned short)(word >> (16 * which))));
}

template <int NT, bool DUMP>
__device__ __forceinline__ void sk_q8_0(SkCtx<NT, DUMP> &c, int st, int lane)
{
    const uint8_t *rec = c.w.record(c.rg, st);
    const uint4 *qp = reinterpret_cast<const uint4 *>(rec) + lane;
    uint4 q[8];
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = ld_stream(qp + 32 * i);
    const uint4 *sp = reinterpret_cast<const uint4 *>(rec + code_bytes(FMT_Q8_0));
    const uint4 sc0 = ld_stream(sp + c.g), sc1 = ld_stream(sp + c.g + 8);
    const unsigned s0w[4] = { sc0.x, sc0.y, sc0.z, sc0.w }, s1w[4] = { sc1.x, sc1.y, sc1.z, sc1.w };
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int blk = st * 8 + i;
        const float scale[2] = { half_of(s0w[i >> 1], i & 1), half_of(s1w[i >> 1], i & 1) };
        const float minv[2] = { 0.f, 0.f };
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int2 x = __ldg(reinterpret_cast<const int2 *>(
                c.a.q + (long long)(c.row0 + nt * 8 + c.g) * c.a.k_pad + blk * 32 + 8 * c.t));
            int acc[4];
            mma_s8s8_k32(acc, q[i].x, q[i].z, q[i].y, q[i].w, x.x, x.y);
            c.scale_tile(blk, nt, acc, scale, minv, false, c.load_ds(blk, nt));
            c.export_tile(blk, nt, acc, 128);
        }
    }
}

template <int NT, bool DUMP>
__device__ __forceinline__ void sk_q4_0(SkCtx<NT, DUMP> &c, int st, int lane)
{
    const uint8_t *rec = c.w.record(c.rg, st);
    const uint4 *qp = reinterpret_cast<const uint4 *>(rec) + lane;
    uint4 q[4];
#pragma unroll
    for (int i = 0; i < 4; i++) q[i] = ld_stream(qp + 32 * i);
    const uint4 *sp = reinterpret_cast<const uint4 *>(rec + code_bytes(FMT_Q4_0));
    const uint4 sc0 = ld_stream(sp + c.g), sc1 = ld_stream(sp + c.g + 8);
    const unsigned s0w[4] = { sc0.x, sc0.y, sc0.z, sc0.w }, s1w[4] = { sc1.x, sc1.y, sc1.z, sc1.w };
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int blk = st * 8 + i;
        const unsigned wg = (i & 1) ? q[i >> 1].z : q[i >> 1].x;
        const unsigned wg8 = (i & 1) ? q[i >> 1].w : q[i >> 1].y;
        const float scale[2] = { half_of(s0w[i >> 1], i & 1), half_of(s1w[i >> 1], i & 1) };
        const float minv[2] = { 8.0f * scale[0], 8.0f * scale[1] };
        const unsigned a0 = wg & 0x0F0F0F0Fu, a1 = wg8 & 0x0F0F0F0Fu;
        const unsigned a2 = (wg >> 4) & 0x0F0F0F0Fu, a3 = (wg8 >> 4) & 0x0F0F0F0Fu;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int8_t *xp = c.a.q + (long long)(c.row0 + nt * 8 + c.g) * c.a.k_pad + blk * 32 + 4 * c.t;
            const int b0 = __ldg(reinterpret_cast<const int *>(xp)), b1 = __ldg(reinterpret_cast<const int *>(xp + 16));
            int acc[4];
            mma_u8s8_k32(acc, a0, a1, a2, a3, b0, b1);
            c.scale_tile(blk, nt, acc, scale, minv, true, c.load_ds(blk, nt));
            c.export_tile(blk, nt, acc, 0);
        }
    }
}

template <int NT, bool DUMP>
__device__ __forceinline__ void sk_q4_k(SkCtx<NT, DUMP> &c, int st, int lane)
{
    const uint8_t *rec = c.w.record(c.rg, st);
    const uint4 *qp = reinterpret_cast<const uint4 *>(rec) + lane;
    uint4 q[4];
#pragma unroll
    for (int i = 0; i < 4; i++) q[i] = ld_stream(qp + 32 * i);
    const uint4 *hp = reinterpret_cast<const uint4 *>(rec + code_bytes(FMT_Q4_K));
    const uint4 h[2] = { ld_stream(hp + c.g), ld_stream(hp + c.g + 8) };
    float d[2], dmin[2];
    unsigned sc[2][2], mn[2][2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        d[r] = half_of(h[r].x, 0);
        dmin[r] = half_of(h[r].x, 1);
        sc[r][0] = h[r].y & 0x3F3F3F3Fu;
        mn[r][0] = h[r].z & 0x3F3F3F3Fu;
        sc[r][1] = (h[r].w & 0x0F0F0F0Fu) | ((h[r].y >> 2) & 0x30303030u);
        mn[r][1] = ((h[r].w >> 4) & 0x0F0F0F0Fu) | ((h[r].z >> 2) & 0x30303030u);
    }
#pragma unroll
    for (int sb = 0; sb < 8; sb++) {
        const int blk = st * 8 + sb, ch = sb >> 1, sh = 4 * (sb & 1);
        float scale[2], minv[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            scale[r] = d[r] * (float)((sc[r][sb >> 2] >> (8 * (sb & 3))) & 0xffu);
            minv[r] = dmin[r] * (float)((mn[r][sb >> 2] >> (8 * (sb & 3))) & 0xffu);
        }
        const unsigned a0 = (q[ch].x >> sh) & 0x0F0F0F0Fu, a2 = (q[ch].y >> sh) & 0x0F0F0F0Fu;
        const unsigned a1 = (q[ch].z >> sh) & 0x0F0F0F0Fu, a3 = (q[ch].w >> sh) & 0x0F0F0F0Fu;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int2 x = __ldg(reinterpret_cast<const int2 *>(
                c.a.q + (long long)(c.row0 + nt * 8 + c.g) * c.a.k_pad + blk * 32 + 8 * c.t));
            int acc[4];
            mma_u8s8_k32(acc, a0, a1, a2, a3, x.x, x.y);
            c.scale_tile(blk, nt, acc, scale, minv, true, c.load_ds(blk, nt));
            c.export_tile(blk, nt, acc, 0);
        }
    }
}

template <int NT, bool DUMP>
__device__ __forceinline__ void sk_q6_k(SkCtx<NT, DUMP> &c, int st, int lane)
{
    const uint8_t *rec = c.w.record(c.rg, st);
    const uint4 *qp = reinterpret_cast<const uint4 *>(rec) + lane;
    const uint4 *scp = reinterpret_cast<const uint4 *>(rec + code_bytes(FMT_Q6_K));
    const __half *dp = reinterpret_cast<const __half *>(rec + code_bytes(FMT_Q6_K) + 256);
    const uint4 scv[2] = { ld_stream(scp + c.g), ld_stream(scp + c.g + 8) };
    const float d[2] = { __half2float(__ldg(dp + c.g)), __half2float(__ldg(dp + c.g + 8)) };
    const unsigned scw[2][4] = { { scv[0].x, scv[0].y, scv[0].z, scv[0].w }, { scv[1].x, scv[1].y, scv[1].z, scv[1].w } };
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint4 A = ld_stream(qp + 32 * (3 * h)), B = ld_stream(qp + 32 * (3 * h + 1)),
                    H = ld_stream(qp + 32 * (3 * h + 2));
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int blk = st * 8 + 4 * h + j;
            unsigned part[2][2];
            float scale[2][2];
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
                    part[hl][r] = __vsub4(lo4 | hi2, 0x20202020u);
                    const int s8 = (int)(signed char)((scw[r][gi >> 2] >> (8 * (gi & 3))) & 0xffu);
                    scale[hl][r] = d[r] * (float)s8;
                }
            }
            const float minv[2] = { 0.f, 0.f };
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int8_t *xp = c.a.q + (long long)(c.row0 + nt * 8 + c.g) * c.a.k_pad + blk * 32 + 4 * c.t;
                const int b0 = __ldg(reinterpret_cast<const int *>(xp)), b1 = __ldg(reinterpret_cast<const int *>(xp + 16));
                const float4 dsp = c.load_ds(blk, nt);
                int c0[4], c1[4];
                mma_s8s8_k16(c0, part[0][0], part[0][1], b0);
                mma_s8s8_k16(c1, part[1][0], part[1][1], b1);
                c.scale_tile(blk, nt, c0, scale[0], minv, false, dsp);
                c.scale_tile(blk, nt, c1, scale[1], minv, false, dsp);
                if (DUMP) {
                    const int sum[4] = { c0[0] + c1[0], c0[1] + c1[1], c0[2] + c1[2], c0[3] + c1[3] };
                    c.export_tile(blk, nt, sum, 32);
                }
            }
        }
    }
}

template <int FMT, int NT, bool DUMP>
__global__ void __launch_bounds__(SK_WARPS * 32)
skinny_kernel(const WeightView w, const ActView a, int row0, int rows, float *__restrict__ y, long long y_stride,
              int *dump, int early)
{
    __shared__ float red[SK_WARPS][16][NT * 8 + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    SkCtx<NT, DUMP> c{ w, a, row0, (int)blockIdx.x, lane >> 2, lane & 3, dump, {} };
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 4; e++) c.acc[nt][e] = 0.0f;

    pdl_enter(early);   // waits for the kernel that produced the activations unless they were complete before it

    const int nst = w.k_pad >> 8;
    for (int st = warp; st < nst; st += SK_WARPS) {
        if (FMT == FMT_Q8_0) sk_q8_0<NT, DUMP>(c, st, lane);
        else if (FMT == FMT_Q4_0) sk_q4_0<NT, DUMP>(c, st, lane);
        else if (FMT == FMT_Q4_K) sk_q4_k<NT, DUMP>(c, st, lane);
        else sk_q6_k<NT, DUMP>(c, st, lane);
    }

#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 4; e++) red[warp][c.g + 8 * (e >> 1)][nt * 8 + 2 * c.t + (e & 1)] = c.acc[nt][e];
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * NT * 8; i += SK_WARPS * 32) {
        const int rr = i & 15, m = i >> 4;
        float v = 0.0f;
#pragma unroll
        for (int wi = 0; wi < SK_WARPS; wi++) v += red[wi][rr][m];
        const int row = blockIdx.x * 16 + rr;
        if (row < w.n && m < rows) y[(long long)(row0 + m) * y_stride + row] = v;
    }
    pdl_exit(early);
}

template <int FMT, bool DUMP>
static cudaError_t launch_nt(const WeightView &w, const ActView &a, int row0, int rows, float *y, long long y_stride,
                             int *dump, int early, cudaStream_t stream)
{
    const dim3 grid(w.n_pad / 16), block(SK_WARPS * 32);
    if (rows <= 8) return launch_pdl(skinny_kernel<FMT, 1, DUMP>, grid, block, 0, stream, w, a, row0, rows, y, y_stride, dump, early);
    if (rows <= 16) return launch_pdl(skinny_kernel<FMT, 2, DUMP>, grid, block, 0, stream, w, a, row0, rows, y, y_stride, dump, early);
    if (rows <= 32) return launch_pdl(skinny_kernel<FMT, 4, DUMP>, grid, block, 0, stream, w, a, row0, rows, y, y_stride, dump, early);
    if (rows <= 64) return launch_pdl(skinny_kernel<FMT, 8, DUMP>, grid, block, 0, stream, w, a, row0, rows, y, y_stride, dump, early);
    return cudaErrorInvalidValue;
}

// row0 must be a multiple of 8 (activation scale pairs are fetched with aligned 128-bit loads).
cudaError_t launch_skinny(const WeightView &w, const ActView &a, int row0, int rows, float *y, long long y_stride,
                          int *dump, int early, cudaStream_t stream)
{
    if (w.n_pad == 0 || rows == 0) return cudaSuccess;
    if (row0 & 7) return cudaErrorInvalidValue;
#define SLC_FMT(F) \
    case F: return dump ? launch_nt<F, true>(w, a, row0, rows, y, y_stride, dump, early, stream) \
                        : launch_nt<F, false>(w, a, row0, rows, y, y_stride, nullptr, early, stream);
    switch (w.fmt) {
        SLC_FMT(FMT_Q8_0) SLC_FMT(FMT_Q4_0) SLC_FMT(FMT_Q4_K) SLC_FMT(FMT_Q6_K)
    default: return cudaErrorInvalidValue;
    }
#undef SLC_FMT
}

}  // namespace slc
