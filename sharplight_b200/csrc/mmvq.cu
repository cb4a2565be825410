// Dequant-fused integer-dot mat-vec (decode): y[m][n] = sum over 32-value blocks of scale_w * scale_x * int32 dot.
//
// The arithmetic is the reference's integer-dot MatMul (src/Sharplight.Cpu/IntDot.Kernels.cs:12-29 and the GPU form in
// src/Sharplight.Shaders/Kernels/mmvq.slang:92-173,319-424 of the Sharplight tree): per block an exact int32 sum of
// weight code x activation code, scaled in f32 by (weight scale x activation scale), minus (weight min x d_x * sum q)
// for the formats with an offset. The design is not the shader's: one CTA owns 16 weight rows, its warps split K in
// 256-value super-tiles, and each lane pulls its operand bytes with one 128-bit streaming load per tile from the
// fragment-major layout (layout.cuh), unpacks nibbles / high bits in registers, and runs dp4a against activation codes
// read through L1. Up to 8 activation rows share one pass over the weights.
#include "internal.cuh"

namespace slc {

constexpr int MMVQ_WARPS = 4;

__device__ __forceinline__ int ldg_i32(const int8_t *p) { return __ldg(reinterpret_cast<const int *>(p)); }
__device__ __forceinline__ int2 ldg_i64(const int8_t *p) { return __ldg(reinterpret_cast<const int2 *>(p)); }

// Sum over the four lanes of a group (the K slices of one row) -- only for the parity export.
__device__ __forceinline__ int group_sum(int v)
{
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}

template <int M, bool DUMP>
struct Ctx
{
    const WeightView &w;
    const ActView &a;
    int row0;        // first activation row of this launch
    int rg, g, t;    // row group, lane coordinates
    int *dump;
    float acc[2][M]; // rows g and g + 8

    // Adds one block's contribution. s[r]: this lane's partial int dot for row r; c_export: constant that turns the
    // full block sum into the unsigned-code dot (times sum32(q)).
    __device__ __forceinline__ void block(int blk, int m, const int s[2], const float scale[2], const float minv[2],
                                          bool has_min, int c_export)
    {
        const int tok = row0 + m;
        const float2 ds = __ldg(&a.ds[(long long)blk * a.rows_pad + tok]);
#pragma unroll
        for (int r = 0; r < 2; r++) {
            acc[r][m] = fmaf(scale[r] * ds.x, (float)s[r], acc[r][m]);
        }
        if (has_min) {
            const float sx = (t == (blk & 3)) ? ds.y : 0.0f;  // one lane of the group carries the offset term
#pragma unroll
            for (int r = 0; r < 2; r++) acc[r][m] = fmaf(-minv[r], sx, acc[r][m]);
        }
        if (DUMP) {
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const int full = group_sum(s[r]);
                const int row = rg * 16 + g + 8 * r;
                if (t == 0 && row < w.n && blk * 32 < w.k) {
                    const int add = c_export ? c_export * __ldg(&a.isum[(long long)tok * (a.k_pad >> 5) + blk]) : 0;
                    dump[((long long)m * w.n + row) * (w.k >> 5) + blk] = full + add;
                }
            }
        }
    }
};

// ---- per-format super-tile (256 values of 16 rows) ---------------------------------------------------------------

template <int M, bool DUMP>
__device__ __forceinline__ void supertile_q8_0(Ctx<M, DUMP> &c, int st, int lane)
{
    const int nst = c.w.k_pad >> 8, nblk_pad = c.w.k_pad >> 5;
    const uint4 *qp = c.w.qs + ((long long)c.rg * nst + st) * 256 + lane;
    uint4 q[8];
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = ld_stream(qp + 32 * i);
    const __half *sp = reinterpret_cast<const __half *>(c.w.sc);
    const uint4 sc0 = __ldg(reinterpret_cast<const uint4 *>(sp + (long long)(c.rg * 16 + c.g) * nblk_pad + st * 8));
    const uint4 sc1 = __ldg(reinterpret_cast<const uint4 *>(sp + (long long)(c.rg * 16 + c.g + 8) * nblk_pad + st * 8));
    const unsigned s0w[4] = { sc0.x, sc0.y, sc0.z, sc0.w }, s1w[4] = { sc1.x, sc1.y, sc1.z, sc1.w };
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int blk = st * 8 + i;
        const float scale[2] = {
            __half2float(__ushort_as_half((unsigned short)(s0w[i >> 1] >> (16 * (i & 1))))),
            __half2float(__ushort_as_half((unsigned short)(s1w[i >> 1] >> (16 * (i & 1))))) };
        const float minv[2] = { 0.f, 0.f };
#pragma unroll
        for (int m = 0; m < M; m++) {
            const int2 x = ldg_i64(c.a.q + (long long)(c.row0 + m) * c.a.k_pad + blk * 32 + 8 * c.t);
            const int s[2] = { __dp4a((int)q[i].x, x.x, __dp4a((int)q[i].y, x.y, 0)),
                               __dp4a((int)q[i].z, x.x, __dp4a((int)q[i].w, x.y, 0)) };
            c.block(blk, m, s, scale, minv, false, 128);
        }
    }
}

template <int M, bool DUMP>
__device__ __forceinline__ void supertile_q4_0(Ctx<M, DUMP> &c, int st, int lane)
{
    const int nst = c.w.k_pad >> 8, nblk_pad = c.w.k_pad >> 5;
    const uint4 *qp = c.w.qs + ((long long)c.rg * nst + st) * 128 + lane;
    uint4 q[4];
#pragma unroll
    for (int i = 0; i < 4; i++) q[i] = ld_stream(qp + 32 * i);
    const __half *sp = reinterpret_cast<const __half *>(c.w.sc);
    const uint4 sc0 = __ldg(reinterpret_cast<const uint4 *>(sp + (long long)(c.rg * 16 + c.g) * nblk_pad + st * 8));
    const uint4 sc1 = __ldg(reinterpret_cast<const uint4 *>(sp + (long long)(c.rg * 16 + c.g + 8) * nblk_pad + st * 8));
    const unsigned s0w[4] = { sc0.x, sc0.y, sc0.z, sc0.w }, s1w[4] = { sc1.x, sc1.y, sc1.z, sc1.w };
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int blk = st * 8 + i;
        const unsigned wg = (i & 1) ? q[i >> 1].z : q[i >> 1].x;
        const unsigned wg8 = (i & 1) ? q[i >> 1].w : q[i >> 1].y;
        const float scale[2] = {
            __half2float(__ushort_as_half((unsigned short)(s0w[i >> 1] >> (16 * (i & 1))))),
            __half2float(__ushort_as_half((unsigned short)(s1w[i >> 1] >> (16 * (i & 1))))) };
        const float minv[2] = { 8.0f * scale[0], 8.0f * scale[1] };
#pragma unroll
        for (int m = 0; m < M; m++) {
            const int8_t *xp = c.a.q + (long long)(c.row0 + m) * c.a.k_pad + blk * 32 + 4 * c.t;
            const int xlo = ldg_i32(xp), xhi = ldg_i32(xp + 16);
            const int s[2] = {
                __dp4a((int)(wg & 0x0F0F0F0Fu), xlo, __dp4a((int)((wg >> 4) & 0x0F0F0F0Fu), xhi, 0)),
                __dp4a((int)(wg8 & 0x0F0F0F0Fu), xlo, __dp4a((int)((wg8 >> 4) & 0x0F0F0F0Fu), xhi, 0)) };
            c.block(blk, m, s, scale, minv, true, 0);
        }
    }
}

// 6-bit scales and mins of a Q4_K header word triple (src/Sharplight.Cpu/Quant.cs:504-516 of the Sharplight tree),
// four at a time: bytes of lo = entries 0..3, bytes of hi = entries 4..7.
__device__ __forceinline__ void q4k_scales(const uint4 h, unsigned &sc_lo, unsigned &sc_hi, unsigned &m_lo, unsigned &m_hi)
{
    sc_lo = h.y & 0x3F3F3F3Fu;
    m_lo = h.z & 0x3F3F3F3Fu;
    sc_hi = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
    m_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
}

template <int M, bool DUMP>
__device__ __forceinline__ void supertile_q4_k(Ctx<M, DUMP> &c, int st, int lane)
{
    const int nst = c.w.k_pad >> 8;
    const uint4 *qp = c.w.qs + ((long long)c.rg * nst + st) * 128 + lane;
    uint4 q[4];
#pragma unroll
    for (int i = 0; i < 4; i++) q[i] = ld_stream(qp + 32 * i);
    const uint4 *hp = reinterpret_cast<const uint4 *>(c.w.sc);
    const uint4 h[2] = { __ldg(hp + (long long)(c.rg * 16 + c.g) * nst + st),
                         __ldg(hp + (long long)(c.rg * 16 + c.g + 8) * nst + st) };
    float d[2], dmin[2];
    unsigned sc[2][2], mn[2][2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        d[r] = __half2float(__ushort_as_half((unsigned short)(h[r].x & 0xffffu)));
        dmin[r] = __half2float(__ushort_as_half((unsigned short)(h[r].x >> 16)));
        q4k_scales(h[r], sc[r][0], sc[r][1], mn[r][0], mn[r][1]);
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
        const int u0 = (int)((q[ch].x >> sh) & 0x0F0F0F0Fu), u1 = (int)((q[ch].y >> sh) & 0x0F0F0F0Fu);
        const int u2 = (int)((q[ch].z >> sh) & 0x0F0F0F0Fu), u3 = (int)((q[ch].w >> sh) & 0x0F0F0F0Fu);
#pragma unroll
        for (int m = 0; m < M; m++) {
            const int2 x = ldg_i64(c.a.q + (long long)(c.row0 + m) * c.a.k_pad + blk * 32 + 8 * c.t);
            const int s[2] = { __dp4a(u0, x.x, __dp4a(u1, x.y, 0)), __dp4a(u2, x.x, __dp4a(u3, x.y, 0)) };
            c.block(blk, m, s, scale, minv, true, 0);
        }
    }
}

template <int M, bool DUMP>
__device__ __forceinline__ void supertile_q6_k(Ctx<M, DUMP> &c, int st, int lane)
{
    const int nst = c.w.k_pad >> 8;
    const uint4 *qp = c.w.qs + ((long long)c.rg * nst + st) * 192 + lane;
    const uint4 *scp = reinterpret_cast<const uint4 *>(c.w.sc);
    const long long e0 = (long long)(c.rg * 16 + c.g) * nst + st, e1 = (long long)(c.rg * 16 + c.g + 8) * nst + st;
    const uint4 scv[2] = { __ldg(scp + e0), __ldg(scp + e1) };
    const float d[2] = { __half2float(__ldg(c.w.d6 + e0)), __half2float(__ldg(c.w.d6 + e1)) };
    const unsigned scw[2][4] = { { scv[0].x, scv[0].y, scv[0].z, scv[0].w }, { scv[1].x, scv[1].y, scv[1].z, scv[1].w } };
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint4 A = ld_stream(qp + 32 * (3 * h)), B = ld_stream(qp + 32 * (3 * h + 1)),
                    H = ld_stream(qp + 32 * (3 * h + 2));
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int blk = st * 8 + 4 * h + j;
            int part[2][2];      // [16-value group][row]
            float scale[2][2];
#pragma unroll
            for (int hl = 0; hl < 2; hl++) {
                const unsigned lw[2] = { (j & 1) ? (hl ? A.w : A.y) : (hl ? A.z : A.x),
                                         (j & 1) ? (hl ? B.w : B.y) : (hl ? B.z : B.x) };
                const unsigned hw[2] = { hl ? H.y : H.x, hl ? H.w : H.z };
                const int gi = 8 * h + 2 * j + hl;  // scale index inside the super-block
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const unsigned lo4 = ((j & 2) ? (lw[r] >> 4) : lw[r]) & 0x0F0F0F0Fu;
                    const unsigned hi2 = ((hw[r] >> (2 * j)) & 0x03030303u) << 4;
                    part[hl][r] = (int)__vsub4(lo4 | hi2, 0x20202020u);  // codes - 32, as signed bytes
                    const int s8 = (int)(signed char)((scw[r][gi >> 2] >> (8 * (gi & 3))) & 0xffu);
                    scale[hl][r] = d[r] * (float)s8;
                }
            }
#pragma unroll
            for (int m = 0; m < M; m++) {
                const int8_t *xp = c.a.q + (long long)(c.row0 + m) * c.a.k_pad + blk * 32 + 4 * c.t;
                const int x0 = ldg_i32(xp), x1 = ldg_i32(xp + 16);
                const int tok = c.row0 + m;
                const float2 ds = __ldg(&c.a.ds[(long long)blk * c.a.rows_pad + tok]);
                int full[2];
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const int s0 = __dp4a(part[0][r], x0, 0), s1 = __dp4a(part[1][r], x1, 0);
                    c.acc[r][m] = fmaf(scale[0][r] * ds.x, (float)s0, c.acc[r][m]);
                    c.acc[r][m] = fmaf(scale[1][r] * ds.x, (float)s1, c.acc[r][m]);
                    full[r] = s0 + s1;
                }
                if (DUMP) {
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        const int sum = group_sum(full[r]);
                        const int row = c.rg * 16 + c.g + 8 * r;
                        if (c.t == 0 && row < c.w.n && blk * 32 < c.w.k) {
                            const int isum = __ldg(&c.a.isum[(long long)tok * (c.a.k_pad >> 5) + blk]);
                            c.dump[((long long)m * c.w.n + row) * (c.w.k >> 5) + blk] = sum + 32 * isum;
                        }
                    }
                }
            }
        }
    }
}

template <int FMT, int M, bool DUMP>
__global__ void __launch_bounds__(MMVQ_WARPS * 32)
mmvq_kernel(const WeightView w, const ActView a, int row0, float *__restrict__ y, long long y_stride, int *dump)
{
    __shared__ float red[MMVQ_WARPS][16][M];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    Ctx<M, DUMP> c{ w, a, row0, (int)blockIdx.x, lane >> 2, lane & 3, dump, {} };
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
        for (int m = 0; m < M; m++) c.acc[r][m] = 0.0f;

    const int nst = w.k_pad >> 8;
    for (int st = warp; st < nst; st += MMVQ_WARPS) {
        if (FMT == FMT_Q8_0) supertile_q8_0<M, DUMP>(c, st, lane);
        else if (FMT == FMT_Q4_0) supertile_q4_0<M, DUMP>(c, st, lane);
        else if (FMT == FMT_Q4_K) supertile_q4_k<M, DUMP>(c, st, lane);
        else supertile_q6_k<M, DUMP>(c, st, lane);
    }

#pragma unroll
    for (int r = 0; r < 2; r++) {
#pragma unroll
        for (int m = 0; m < M; m++) {
            float v = c.acc[r][m];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (c.t == 0) red[warp][c.g + 8 * r][m] = v;
        }
    }
    __syncthreads();
    if (threadIdx.x < 16 * M) {
        const int m = threadIdx.x / 16, rr = threadIdx.x % 16;
        float v = 0.0f;
#pragma unroll
        for (int wi = 0; wi < MMVQ_WARPS; wi++) v += red[wi][rr][m];
        const int row = blockIdx.x * 16 + rr;
        if (row < w.n) y[(long long)(row0 + m) * y_stride + row] = v;
    }
}

template <int FMT, bool DUMP>
static cudaError_t launch_m(const WeightView &w, const ActView &a, int row0, int rows, float *y, long long y_stride,
                            int *dump, cudaStream_t stream)
{
    const dim3 grid(w.n_pad / 16), block(MMVQ_WARPS * 32);
    switch (rows) {
#define SLC_CASE(MM) \
    case MM: mmvq_kernel<FMT, MM, DUMP><<<grid, block, 0, stream>>>(w, a, row0, y, y_stride, dump); break;
        SLC_CASE(1) SLC_CASE(2) SLC_CASE(3) SLC_CASE(4) SLC_CASE(5) SLC_CASE(6) SLC_CASE(7) SLC_CASE(8)
#undef SLC_CASE
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_mmvq(const WeightView &w, const ActView &a, int row0, int rows, float *y, long long y_stride,
                        int *dump, cudaStream_t stream)
{
    if (w.n_pad == 0 || rows == 0) return cudaSuccess;
#define SLC_FMT(F) \
    case F: return dump ? launch_m<F, true>(w, a, row0, rows, y, y_stride, dump, stream) \
                        : launch_m<F, false>(w, a, row0, rows, y, y_stride, nullptr, stream);
    switch (w.fmt) {
        SLC_FMT(FMT_Q8_0) SLC_FMT(FMT_Q4_0) SLC_FMT(FMT_Q4_K) SLC_FMT(FMT_Q6_K)
    default: return cudaErrorInvalidValue;
    }
#undef SLC_FMT
}

}  // namespace slc
