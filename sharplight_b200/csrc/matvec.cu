// Dequant-fused integer-dot mat-vec (decode), 1..4 activation rows per launch: the dp4a kernel family.
//
// Arithmetic: the reference's integer-dot MatMul (src/Sharplight.Cpu/IntDot.Kernels.cs:12-29 and the GPU form in
// src/Sharplight.Shaders/Kernels/mmvq.slang:92-173,319-424 of the Sharplight tree): per 32-value block an exact int32
// sum of weight code x activation code, scaled in f32 by (weight scale x activation scale), minus
// (weight min x d_x * sum q) for the formats with an offset.
//
// Shape of the kernel (not the shader's): one CTA owns 16 weight rows; its warps split K in 256-value super-tiles.
// Every warp streams its records (layout.cuh) into a private two-slot ring in shared memory with bulk async copies
// (cp.async.bulk + mbarrier, the TMA engine, no registers held by loads in flight). The first copies are issued before
// the kernel waits for its predecessor on the stream (programmatic dependent launch): weights never depend on earlier
// kernels, the quantized activations do, so the weight stream of this MatMul overlaps the tail of the previous kernel
// and the activation quantization. The activation codes and scales are copied to shared memory once per CTA; the dot
// loop reads a record from its slot (one 128-bit shared load per lane per tile), runs dp4a against the activations,
// and re-arms the slot with the warp's next record. Integer sub-block scales (Q4_K, Q6_K) are applied in int32 before
// the one int->float conversion per block. Every mbarrier wait is bounded: when it runs out the kernel raises the
// device status word and leaves.
#include "internal.cuh"
#include "exchange.cuh"

namespace slc {

constexpr int FV_MAX_WARPS = 8;
constexpr int FV_STAGES = 2;
constexpr int FV_MAX_SMEM = 200 * 1024;   // what a launch may ask for; typical launches take 25-60 KB

template <int FMT> struct FTile;
template <> struct FTile<FMT_Q8_0> { uint4 q[8]; uint4 s[2]; };
template <> struct FTile<FMT_Q4_0> { uint4 q[4]; uint4 s[2]; };
template <> struct FTile<FMT_Q4_K> { uint4 q[4]; uint4 s[2]; };
template <> struct FTile<FMT_Q6_K> { uint4 q[6]; uint4 s[2]; unsigned short d[2]; };

// One record of this lane: code units and the scale entries of rows g and g + 8, from a shared-memory slot.
template <int FMT>
__device__ __forceinline__ void load_tile(FTile<FMT> &tl, const uint8_t *slot, int lane)
{
    const int g = lane >> 2;
    constexpr int NQ = code_units(FMT) / 32;
    const uint4 *qp = reinterpret_cast<const uint4 *>(slot) + lane;
#pragma unroll
    for (int i = 0; i < NQ; i++) tl.q[i] = qp[32 * i];
    const uint4 *sp = reinterpret_cast<const uint4 *>(slot + code_bytes(FMT));
    tl.s[0] = sp[g];
    tl.s[1] = sp[g + 8];
    if constexpr (FMT == FMT_Q6_K) {
        const unsigned short *dp = reinterpret_cast<const unsigned short *>(slot + code_bytes(FMT) + 256);
        tl.d[0] = dp[g];
        tl.d[1] = dp[g + 8];
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

// ---- whole-block lane mapping (Q4_K, Q8_0, Q4_0) -----------------------------------------------------------------
// The record sits in shared memory, so a lane is free to read other lanes' code units: lane (g, t) takes, for rows g
// and g + 8, the whole 32-value blocks of quarter t of the super-tile (four 128-bit shared loads, visited in an order
// rotated by t so the four lanes of a group hit different banks). A lane then owns complete block dots: the per-block
// scaling is done once per (row, block) instead of once per quarter block in each of four lanes.

// unsigned bytes x signed bytes: high nibbles are used in place (value * 16), the sum is shifted down afterwards
__device__ __forceinline__ int dp4a_us(unsigned a, int b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <bool DUMP>
__device__ __forceinline__ void export_block(const DumpCtx &dc, const SmemAct &a, int blk, int m, int r, int dot, int c_export)
{
    if (!DUMP) return;
    const int row = dc.rg * 16 + dc.g + 8 * r;
    if (row < dc.n && blk * 32 < dc.k) {
        dc.out[((long long)m * dc.n + row) * (dc.k >> 5) + blk] = dot + c_export * a.isum[m * a.nblk_pad + blk];
    }
}

template <int FMT, int M, bool DUMP>
__device__ __forceinline__ void compute_slot(const uint8_t *slot, const SmemAct &a, int st, int lane, float acc[2][M],
                                             const DumpCtx &dc)
{
    const int g = lane >> 2, t = lane & 3;
    const int8_t *xq = a.q + st * 256;
    const float2 *xs = a.ds + st * 8;
    const uint4 *sp = reinterpret_cast<const uint4 *>(slot + code_bytes(FMT));
    const uint4 h0 = sp[g], h1 = sp[g + 8];

    if constexpr (FMT == FMT_Q4_K) {
        // chunk t = sub-blocks 2t (low nibbles) and 2t + 1 (high nibbles)
        const uint4 *tile = reinterpret_cast<const uint4 *>(slot + t * 512) + g * 4;
        int s[2][2][M];
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int b = 0; b < 2; b++)
#pragma unroll
                for (int m = 0; m < M; m++) s[r][b][m] = 0;
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
            const int j = (jj + t) & 3;
            const uint4 q = tile[j];
            const int l0 = (int)(q.x & 0x0F0F0F0Fu), l1 = (int)(q.y & 0x0F0F0F0Fu);
            const int l2 = (int)(q.z & 0x0F0F0F0Fu), l3 = (int)(q.w & 0x0F0F0F0Fu);
            const unsigned u0 = q.x & 0xF0F0F0F0u, u1 = q.y & 0xF0F0F0F0u, u2 = q.z & 0xF0F0F0F0u, u3 = q.w & 0xF0F0F0F0u;
#pragma unroll
            for (int m = 0; m < M; m++) {
                const int8_t *xp = xq + m * a.k_pad + 64 * t + 8 * j;
                const int2 xl = *reinterpret_cast<const int2 *>(xp), xh = *reinterpret_cast<const int2 *>(xp + 32);
                s[0][0][m] = __dp4a(l0, xl.x, __dp4a(l1, xl.y, s[0][0][m]));
                s[1][0][m] = __dp4a(l2, xl.x, __dp4a(l3, xl.y, s[1][0][m]));
                s[0][1][m] = dp4a_us(u0, xh.x, dp4a_us(u1, xh.y, s[0][1][m]));
                s[1][1][m] = dp4a_us(u2, xh.x, dp4a_us(u3, xh.y, s[1][1][m]));
            }
        }
        const int sh = 16 * (t & 1);
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const uint4 h = r ? h1 : h0;
            const float d = h2f(h.x & 0xffffu), dmin = h2f(h.x >> 16);
            // 6-bit scales / mins of sub-blocks 2t, 2t + 1 (src/Sharplight.Cpu/Quant.cs:504-516 of the Sharplight tree)
            const unsigned scw = t < 2 ? (h.y & 0x3F3F3F3Fu) : ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u));
            const unsigned mnw = t < 2 ? (h.z & 0x3F3F3F3Fu) : (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u));
            const int sc0 = (int)((scw >> sh) & 0xffu), sc1 = (int)((scw >> (sh + 8)) & 0xffu);
            const float mn0 = (float)((mnw >> sh) & 0xffu), mn1 = (float)((mnw >> (sh + 8)) & 0xffu);
#pragma unroll
            for (int m = 0; m < M; m++) {
                const float2 ds0 = xs[m * a.nblk_pad + 2 * t], ds1 = xs[m * a.nblk_pad + 2 * t + 1];
                const int d0 = s[r][0][m], d1 = s[r][1][m] >> 4;     // the high-nibble sum carries a factor 16
                // integer sub-block scale first: |dot * sc| <= 60960 * 63 < 2^22, exact in f32
                const float part = fmaf((float)(d0 * sc0), ds0.x, (float)(d1 * sc1) * ds1.x);
                const float mpart = fmaf(mn0, ds0.y, mn1 * ds1.y);
                acc[r][m] += fmaf(d, part, -dmin * mpart);
                export_block<DUMP>(dc, a, st * 8 + 2 * t, m, r, d0, 0);
                export_block<DUMP>(dc, a, st * 8 + 2 * t + 1, m, r, d1, 0);
            }
        }
    } else if constexpr (FMT == FMT_Q8_0) {
        // blocks 2t and 2t + 1, one 512-byte tile each
#pragma unroll
        for (int bl = 0; bl < 2; bl++) {
            const int blk = 2 * t + bl;
            const uint4 *tile = reinterpret_cast<const uint4 *>(slot + blk * 512) + g * 4;
            int s[2][M];
#pragma unroll
            for (int r = 0; r < 2; r++)
#pragma unroll
                for (int m = 0; m < M; m++) s[r][m] = 0;
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                const int j = (jj + t) & 3;
                const uint4 q = tile[j];
#pragma unroll
                for (int m = 0; m < M; m++) {
                    const int2 x = *reinterpret_cast<const int2 *>(xq + m * a.k_pad + blk * 32 + 8 * j);
                    s[0][m] = __dp4a((int)q.x, x.x, __dp4a((int)q.y, x.y, s[0][m]));
                    s[1][m] = __dp4a((int)q.z, x.x, __dp4a((int)q.w, x.y, s[1][m]));
                }
            }
            const unsigned w0 = t == 0 ? h0.x : t == 1 ? h0.y : t == 2 ? h0.z : h0.w;
            const unsigned w1 = t == 0 ? h1.x : t == 1 ? h1.y : t == 2 ? h1.z : h1.w;
            const float dw[2] = { h2f((w0 >> (16 * bl)) & 0xffffu), h2f((w1 >> (16 * bl)) & 0xffffu) };
#pragma unroll
            for (int m = 0; m < M; m++) {
                const float dx = xs[m * a.nblk_pad + blk].x;
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    acc[r][m] = fmaf(dw[r] * dx, (float)s[r][m], acc[r][m]);
                    export_block<DUMP>(dc, a, st * 8 + blk, m, r, s[r][m], 128);
                }
            }
        }
    } else {  // Q4_0: tile t holds blocks 2t and 2t + 1
        const uint4 *tile = reinterpret_cast<const uint4 *>(slot + t * 512) + g * 4;
        int lo[2][2][M], hi[2][2][M];   // [row][block][m]
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int b = 0; b < 2; b++)
#pragma unroll
                for (int m = 0; m < M; m++) { lo[r][b][m] = 0; hi[r][b][m] = 0; }
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
            const int j = (jj + t) & 3;
            const uint4 q = tile[j];
            const unsigned wv[4] = { q.x, q.y, q.z, q.w };   // row g blk 0, row g+8 blk 0, row g blk 1, row g+8 blk 1
#pragma unroll
            for (int m = 0; m < M; m++) {
#pragma unroll
                for (int b = 0; b < 2; b++) {
                    const int8_t *xp = xq + m * a.k_pad + (2 * t + b) * 32 + 4 * j;
                    const int xl = *reinterpret_cast<const int *>(xp), xh = *reinterpret_cast<const int *>(xp + 16);
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        const unsigned wq = wv[2 * b + r];
                        lo[r][b][m] = __dp4a((int)(wq & 0x0F0F0F0Fu), xl, lo[r][b][m]);
                        hi[r][b][m] = dp4a_us(wq & 0xF0F0F0F0u, xh, hi[r][b][m]);
                    }
                }
            }
        }
        const unsigned w0 = t == 0 ? h0.x : t == 1 ? h0.y : t == 2 ? h0.z : h0.w;
        const unsigned w1 = t == 0 ? h1.x : t == 1 ? h1.y : t == 2 ? h1.z : h1.w;
#pragma unroll
        for (int b = 0; b < 2; b++) {
            const float dw[2] = { h2f((w0 >> (16 * b)) & 0xffffu), h2f((w1 >> (16 * b)) & 0xffffu) };
#pragma unroll
            for (int m = 0; m < M; m++) {
                const float2 ds = xs[m * a.nblk_pad + 2 * t + b];
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const int dot = lo[r][b][m] + (hi[r][b][m] >> 4);
                    // codes are value + 8: d_w * (d_x * dot - 8 * d_x * sum q)
                    acc[r][m] = fmaf(dw[r], fmaf(ds.x, (float)dot, -8.0f * ds.y), acc[r][m]);
                    export_block<DUMP>(dc, a, st * 8 + 2 * t + b, m, r, dot, 0);
                }
            }
        }
    }
}

// DUAL: two weights of one shape share the activations (the gate and up projections of a gated FFN); every ring slot
// carries the record of each, both dots are accumulated, and the store writes silu(gate) * up -- the reference's dual
// MatMul with the SiLU-mul group as its epilogue (src/Sharplight.Shaders/Lowering/GraphLowerer.MatMul.cs:128-198),
// silu(v) = v / (1 + exp(-v)) as in src/Sharplight.Cpu/ScalarMath.cs:552-577.
template <int FMT, int M, bool DUMP, bool DUAL>
__global__ void __launch_bounds__(FV_MAX_WARPS * 32)
matvec_kernel(const WeightView w, const WeightView w2, const ActView a, int row0, float *__restrict__ y, long long y_stride,
              int *dump, int *status, int early, const Exchange ex, const Epilogue ep)
{
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t bars[FV_MAX_WARPS][FV_STAGES];
    __shared__ float red[DUAL ? 2 : 1][FV_MAX_WARPS][16][M];
    constexpr int REC1 = record_bytes(FMT), REC = DUAL ? 2 * REC1 : REC1;   // bytes of a ring slot
    const int warps = blockDim.x >> 5;
    const int nblk_pad = w.k_pad >> 5, nst = w.k_pad >> 8;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, t = lane & 3, g = lane >> 2;
    const int rg = blockIdx.x;
    uint8_t *ring = smem + (size_t)warp * FV_STAGES * REC;
    unsigned char *act_base = smem + (size_t)warps * FV_STAGES * REC;
    int8_t *sq = reinterpret_cast<int8_t *>(act_base);
    float2 *sds = reinterpret_cast<float2 *>(act_base + (size_t)M * w.k_pad);
    int *sisum = reinterpret_cast<int *>(act_base + (size_t)M * w.k_pad + (size_t)M * nblk_pad * 8);

    // this warp's records: super-tiles warp, warp + warps, ...; the first FV_STAGES copies start right away
    const int count = nst > warp ? (nst - warp + warps - 1) / warps : 0;
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < FV_STAGES; s++) mbar_init(&bars[warp][s], 1);
        fence_mbar_init();
#pragma unroll
        for (int s = 0; s < FV_STAGES; s++) {
            if (s < count) {
                if (DUAL) bulk_load2(ring + s * REC, w.record(rg, warp + s * warps), w2.record(rg, warp + s * warps), REC1, &bars[warp][s]);
                else bulk_load(ring + s * REC, w.record(rg, warp + s * warps), REC, &bars[warp][s]);
            }
        }
    }

    // early: the activations were complete before the preceding kernel began (it reads the same ones), so this kernel
    // may run beside it; otherwise wait for the preceding kernel, which produced them
    pdl_enter(early);

    // quantized activations -> shared memory
    if (a.raw) {
        // Deferred quantization: this CTA quantizes the rows itself, with the quantizer's arithmetic step for step
        // (quantize.cuh: d = max|x| / 127, id = 1 / d, round half away from zero by truncation, separately rounded IEEE
        // operations), eight lanes per 32-value block. Worth it when K is short (a tensor-parallel shard): the row is a few
        // kilobytes from L2, and the launch of a quantizer with its boundary on the dependent chain is saved.
        const int sub = threadIdx.x & 7;
        for (int m = 0; m < M; m++) {
            for (int blk = threadIdx.x >> 3; blk < nblk_pad; blk += blockDim.x >> 3) {
                float v[4] = { 0.f, 0.f, 0.f, 0.f };
                if (blk * 32 < a.k) {
                    const long long base = (long long)(row0 + m) * a.raw_stride + blk * 32 + sub * 4;
                    if (a.raw_dtype == 0) {
                        const float *x = reinterpret_cast<const float *>(a.raw) + base;
                        if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
                            const float4 f = *reinterpret_cast<const float4 *>(x);
                            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                        } else {
                            for (int i = 0; i < 4; i++) v[i] = x[i];
                        }
                    } else {
                        const unsigned short *x = reinterpret_cast<const unsigned short *>(a.raw) + base;
                        for (int i = 0; i < 4; i++) v[i] = __uint_as_float((unsigned)x[i] << 16);
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
                *reinterpret_cast<unsigned *>(sq + (size_t)m * w.k_pad + blk * 32 + sub * 4) =
                    (unsigned)(r[0] & 0xff) | ((unsigned)(r[1] & 0xff) << 8) | ((unsigned)(r[2] & 0xff) << 16) | ((unsigned)(r[3] & 0xff) << 24);
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                if (sub == 0) {
                    sds[m * nblk_pad + blk] = make_float2(d, __fmul_rn(d, (float)s));
                    if (DUMP) sisum[m * nblk_pad + blk] = s;
                }
            }
        }
    } else {
        const uint4 *src = reinterpret_cast<const uint4 *>(a.q + (long long)row0 * a.k_pad);
        uint4 *dst = reinterpret_cast<uint4 *>(sq);
        for (int i = threadIdx.x; i < M * (w.k_pad >> 4); i += blockDim.x) dst[i] = __ldg(src + i);
        for (int blk = threadIdx.x; blk < nblk_pad; blk += blockDim.x) {
#pragma unroll
            for (int m = 0; m < M; m++) {
                sds[m * nblk_pad + blk] = __ldg(&a.ds[(long long)blk * a.rows_pad + row0 + m]);
                if (DUMP) sisum[m * nblk_pad + blk] = __ldg(&a.isum[(long long)(row0 + m) * nblk_pad + blk]);
            }
        }
    }
    __syncthreads();

    const SmemAct act{ sq, sds, sisum, w.k_pad, nblk_pad };
    const DumpCtx dc{ dump, w.n, w.k, rg, g, t };
    float acc[2][M], acc2[2][M];
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
        for (int m = 0; m < M; m++) { acc[r][m] = 0.0f; acc2[r][m] = 0.0f; }
    auto refill = [&](int s, int i) {
        const int st = warp + (i + FV_STAGES) * warps;
        if (DUAL) bulk_load2(ring + s * REC, w.record(rg, st), w2.record(rg, st), REC1, &bars[warp][s]);
        else bulk_load(ring + s * REC, w.record(rg, st), REC, &bars[warp][s]);
    };

    bool alive = true;
    for (int i = 0; i < count; i++) {
        const int s = i % FV_STAGES;
        const uint8_t *slot = ring + s * REC;
        if (!mbar_wait(&bars[warp][s], (unsigned)(i / FV_STAGES) & 1u)) {
            // the copy never landed: report, stop computing, but still drain what else is in flight (bounded)
            if (lane == 0) atomicExch(status, -7);
            alive = false;
        }
        if (alive) {
            if constexpr (FMT == FMT_Q6_K) {
                FTile<FMT> tl, tl2;
                load_tile<FMT>(tl, slot, lane);
                if (DUAL) load_tile<FMT>(tl2, slot + REC1, lane);
                __syncwarp();   // every lane has its copy of the record: the slot may be refilled
                if (lane == 0 && i + FV_STAGES < count) refill(s, i);
                compute_tile<FMT, M, DUMP>(tl, act, warp + i * warps, t, acc, dc);
                if (DUAL) compute_tile<FMT, M, DUMP>(tl2, act, warp + i * warps, t, acc2, dc);
            } else {
                compute_slot<FMT, M, DUMP>(slot, act, warp + i * warps, lane, acc, dc);
                if (DUAL) compute_slot<FMT, M, DUMP>(slot + REC1, act, warp + i * warps, lane, acc2, dc);
                __syncwarp();   // every lane is done reading the slot: it may be refilled
                if (lane == 0 && i + FV_STAGES < count) refill(s, i);
            }
        }
    }

#pragma unroll
    for (int r = 0; r < 2; r++) {
#pragma unroll
        for (int m = 0; m < M; m++) {
            float v = acc[r][m];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (t == 0) red[0][warp][g + 8 * r][m] = v;
            if (DUAL) {
                float u = acc2[r][m];
                u += __shfl_xor_sync(0xffffffffu, u, 1);
                u += __shfl_xor_sync(0xffffffffu, u, 2);
                if (t == 0) red[DUAL ? 1 : 0][warp][g + 8 * r][m] = u;
            }
        }
    }
    __syncthreads();
    {
        // The CTA's 16 * M output values are dealt out to its threads; a CTA of a single warp (K of one super-tile)
        // has fewer threads than values for M > 2, so a thread may own two of them.
        constexpr int OWN = (16 * M + 31) / 32;
        float vals[OWN];
#pragma unroll
        for (int j = 0; j < OWN; j++) {
            const int o = threadIdx.x + j * blockDim.x;
            float v = 0.0f;
            if (o < 16 * M) {
                const int m = o / 16, rr = o % 16;
                for (int wi = 0; wi < warps; wi++) v += red[0][wi][rr][m];
                if (DUAL) {
                    float u = 0.0f;
                    for (int wi = 0; wi < warps; wi++) u += red[DUAL ? 1 : 0][wi][rr][m];
                    v = w2.pair_sum ? __fadd_rn(v, u)                        // the two halves of one weight (Q5_K)
                                    : __fdiv_rn(v, 1.0f + expf(-v)) * u;    // silu(gate) * up
                }
            }
            vals[j] = v;
        }
        if (ex.world == 0) {
#pragma unroll
            for (int j = 0; j < OWN; j++) {
                const int o = threadIdx.x + j * blockDim.x;
                const int m = o / 16, row = blockIdx.x * 16 + o % 16;
                if (o < 16 * M && row < w.n) y[(long long)(row0 + m) * y_stride + row] = ep.apply(vals[j], row0 + m, row);
            }
        } else {
            // row-split MatMul of a tensor-parallel group: the values are this rank's partial sums; every thread trades
            // its own with the peers as {value, tag} words (exchange.cuh), all sent before any is awaited
            const int epoch = ex_epoch(ex), slot = epoch & 1;
#pragma unroll
            for (int j = 0; j < OWN; j++) {
                const int o = threadIdx.x + j * blockDim.x;
                if (o < 16 * M) ex_ll_send(ex, slot, epoch, o / 16, blockIdx.x * 16 + o % 16, vals[j]);
            }
            bool ok = true;
            const unsigned long long wait_from = ex_now();
#pragma unroll
            for (int j = 0; j < OWN; j++) {
                const int o = threadIdx.x + j * blockDim.x;
                if (o < 16 * M) {
                    const int m = o / 16, row = blockIdx.x * 16 + o % 16;
                    const float total = ex_ll_collect(ex, slot, epoch, m, row, vals[j], ok, wait_from);
                    if (row < w.n) y[(long long)(row0 + m) * y_stride + row] = ep.apply(total, row0 + m, row);
                }
            }
            if (!ok) atomicExch(status, -7);
            ex_finish(ex, epoch);
        }
    }
    pdl_exit(early);
}

// Warps per CTA: four split K by default; eight when there are few row groups and K is long (the down projections),
// never more than there are super-tiles.
static int matvec_warps(const WeightView &w)
{
    const int nst = w.k_pad >> 8, rgs = w.n_pad / 16;
    int warps = (rgs < 444 && nst >= 8) ? 8 : 4;
    return warps < nst ? warps : nst;
}

static size_t matvec_smem(int fmt, int warps, int rows, int k_pad, bool dual = false)
{
    return (size_t)(dual ? 2 : 1) * warps * FV_STAGES * record_bytes(fmt) + (size_t)rows * (k_pad + (k_pad >> 5) * 12);
}

bool matvec_fits(int rows, int k_pad, bool dual)
{
    return rows >= 1 && rows <= 4 && matvec_smem(FMT_Q8_0, FV_MAX_WARPS, rows, k_pad, dual) <= FV_MAX_SMEM;
}

template <int FMT, int M, bool DUMP, bool DUAL>
static cudaError_t launch_one(const WeightView &w, const WeightView &w2, const ActView &a, int row0, float *y,
                              long long y_stride, int *dump, int *status, int early, cudaStream_t stream,
                              const Exchange &ex, const Epilogue &ep)
{
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = matvec_kernel<FMT, M, DUMP, DUAL>;
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FV_MAX_SMEM);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int warps = matvec_warps(w);
    if (ex.world > 1) {
        // a CTA that exchanges waits for the peers' CTAs of the same index: every CTA of the grid must be able to be
        // resident at once, or a wait could depend on a CTA that has not started (it would time out, not hang; refused)
        int per_sm = 0, sms = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, warps * 32, matvec_smem(FMT, warps, M, w.k_pad, DUAL));
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        if (w.n_pad / 16 > per_sm * sms) return cudaErrorLaunchOutOfResources;
    }
    return launch_pdl(kernel, dim3(w.n_pad / 16), dim3(warps * 32), matvec_smem(FMT, warps, M, w.k_pad, DUAL), stream, w, w2,
                      a, row0, y, y_stride, dump, status, early, ex, ep);
}

template <int FMT>
static cudaError_t launch_fmt(const WeightView &w, const WeightView *w2, const ActView &a, int row0, int rows, float *y,
                              long long y_stride, int *dump, int *status, int early, cudaStream_t stream,
                              const Exchange &ex, const Epilogue &ep)
{
#define SLC_ROWS(MM)                                                                        \
    case MM:                                                                                \
        if (w2) return launch_one<FMT, MM, false, true>(w, *w2, a, row0, y, y_stride, nullptr, status, early, stream, ex, ep); \
        return dump ? launch_one<FMT, MM, true, false>(w, w, a, row0, y, y_stride, dump, status, early, stream, ex, ep)      \
                    : launch_one<FMT, MM, false, false>(w, w, a, row0, y, y_stride, nullptr, status, early, stream, ex, ep);
    switch (rows) {
        SLC_ROWS(1) SLC_ROWS(2) SLC_ROWS(3) SLC_ROWS(4)
    default: return cudaErrorInvalidValue;
    }
#undef SLC_ROWS
}

// rows 1..4 starting at activation row row0; dump (optional) receives [rows][n][k/32] block dots.
cudaError_t launch_matvec(const WeightView &w, const ActView &a, int row0, int rows, float *y, long long y_stride,
                          int *dump, int *status, int early, cudaStream_t stream, const Exchange *exchange,
                          const Epilogue *epilogue, const WeightView *w2)
{
    if (w.n_pad == 0 || rows == 0) return cudaSuccess;
    const Epilogue ep = epilogue ? *epilogue : Epilogue{ nullptr, nullptr, 0 };
    if (w2 && (dump || exchange || w2->fmt != w.fmt || w2->n != w.n || w2->k != w.k)) return cudaErrorInvalidValue;
    Exchange ex{};
    if (exchange) {
        ex = *exchange;
        // a launch that exchanges waits for its predecessor before anything else, and needs room for its tile
        if (early || rows > SLC_LL_ROWS || w.n_pad > ex.n_stride) return cudaErrorInvalidValue;
    }
    switch (w.fmt) {
    case FMT_Q8_0: return launch_fmt<FMT_Q8_0>(w, w2, a, row0, rows, y, y_stride, dump, status, early, stream, ex, ep);
    case FMT_Q4_0: return launch_fmt<FMT_Q4_0>(w, w2, a, row0, rows, y, y_stride, dump, status, early, stream, ex, ep);
    case FMT_Q4_K: return launch_fmt<FMT_Q4_K>(w, w2, a, row0, rows, y, y_stride, dump, status, early, stream, ex, ep);
    case FMT_Q6_K: return launch_fmt<FMT_Q6_K>(w, w2, a, row0, rows, y, y_stride, dump, status, early, stream, ex, ep);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace slc
