// Skinny integer-dot GEMM for 3..64 activation rows (batched decode, speculative verification, short prefill).
//
// Same arithmetic as matvec.cu -- exact int32 block dots scaled in f32 (src/Sharplight.Cpu/IntDot.Kernels.cs:12-29,
// src/Sharplight.Shaders/Kernels/mmq.slang:224-233 of the Sharplight tree) -- with the int32 dots from int8 tensor-core
// tiles: 16 weight rows are the M operand of mma.sync m16n8k32 (m16n8k16 for Q6_K, whose scales change every 16
// values), eight activation rows the N operand, one 32-value block one K step. The reference's skinny kernel decodes to
// f16 instead (src/Sharplight.Shaders/Kernels/matmul_skinny.slang:1-31).
//
// A CTA owns 64 weight rows (4 row groups) and runs 8 warps: warp = (row group, K half). All warps walk their K half in
// lock step, one 256-value super-tile per step; the activation codes and scales of the two super-tiles of a step are
// staged once per CTA in shared memory (cp.async ring) and shared by the four row groups, while every warp streams its
// own weight records into a private shared-memory ring with bulk async copies (mbarrier, bounded waits). The accumulator
// operand of each MMA is the constant 0x4B400000, so the tile comes back as the bit pattern of the float
// 12582912 + dot: int->float costs no instruction (the conversion unit would be the bottleneck), and the integer
// sub-block scale is applied by one exact FMA, fma(f, sc, -12582912 * sc).
#include "internal.cuh"
#include "exchange.cuh"

namespace slc {

constexpr int SK_RGS = 4, SK_KS = 2, SK_WARPS = SK_RGS * SK_KS;
constexpr int SK_XROW = 288;            // bytes per token row of a staged 256-value tile: 256 + 32 keeps B-fragment loads
                                        // of eight consecutive tokens on different banks
constexpr int SK_BIAS = 0x4B400000;
constexpr float SK_BIAS_F = 12582912.0f;

__device__ __forceinline__ void mma_u8s8_k32(int c[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, int b0, int b1)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(SK_BIAS));
}

__device__ __forceinline__ void mma_s8s8_k32(int c[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, int b0, int b1)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(SK_BIAS));
}

__device__ __forceinline__ void mma_s8s8_k16(int c[4], unsigned a0, unsigned a1, int b0)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(SK_BIAS));
}

// C[16 x 8] += A[16 x 8] * B[8 x 8] in tf32 (f32 accumulate): the Q4_K offset term, whose factors (6-bit mins, and
// d_x * sum q split in a tf32 high part and the rest) lose nothing that matters in tf32.
__device__ __forceinline__ void mma_tf32_k8(float c[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float sk_h2f(unsigned bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

template <int FMT>
struct SkRec
{
    uint4 q[code_units(FMT) / 32];
    uint4 s0, s1;
    unsigned short d0, d1;   // Q6_K only
};

// A record from its shared-memory slot into this lane's registers.
template <int FMT>
__device__ __forceinline__ void sk_load(SkRec<FMT> &r, const uint8_t *rec, int lane)
{
    const int g = lane >> 2;
    const uint4 *qp = reinterpret_cast<const uint4 *>(rec) + lane;
#pragma unroll
    for (int i = 0; i < code_units(FMT) / 32; i++) r.q[i] = qp[32 * i];
    const uint4 *sp = reinterpret_cast<const uint4 *>(rec + code_bytes(FMT));
    r.s0 = sp[g];
    r.s1 = sp[g + 8];
    if constexpr (FMT == FMT_Q6_K) {
        const unsigned short *dp = reinterpret_cast<const unsigned short *>(rec + code_bytes(FMT) + 256);
        r.d0 = dp[g];
        r.d1 = dp[g + 8];
    }
}

// One staged activation tile: T tokens x 256 codes (rows SK_XROW bytes apart), then (d, d*sum q) as [8 blocks][T].
template <int NT>
struct SkTile
{
    static constexpr int T = NT * 8;
    static constexpr int BYTES = T * SK_XROW + 8 * T * 8;
    const unsigned char *base;
    __device__ __forceinline__ const int8_t *x(int tok, int koff) const { return reinterpret_cast<const int8_t *>(base + tok * SK_XROW + koff); }
    // d_x * sum q of (block, token) alone
    __device__ __forceinline__ float sx(int blk, int tok) const
    {
        return *reinterpret_cast<const float *>(base + T * SK_XROW + (blk * T + tok) * 8 + 4);
    }
    __device__ __forceinline__ float4 ds2(int blk, int tok) const
    {
        return *reinterpret_cast<const float4 *>(base + T * SK_XROW + (blk * T + tok) * 8);
    }
};

template <int FMT, int NT, bool DUMP>
struct SkCtx
{
    const WeightView &w;
    const ActView &a;
    int row0, rg, g, t;
    int *dump;

    // shift: the tile holds the dots times 2^shift (Q4_0 multiplies its codes by 16)
    __device__ __forceinline__ void export_tile(int blk, int nt, const int c[4], int c_export, int shift = 0) const
    {
        if (!DUMP) return;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int row = rg * 16 + g + 8 * (e >> 1);
            const int m = nt * 8 + 2 * t + (e & 1);
            const int tok = row0 + m;
            if (row < w.n && tok < a.rows && blk * 32 < w.k) {
                const int add = c_export ? c_export * __ldg(&a.isum[(long long)tok * (a.k_pad >> 5) + blk]) : 0;
                dump[((long long)m * w.n + row) * (w.k >> 5) + blk] = ((c[e] - SK_BIAS) >> shift) + add;
            }
        }
    }
};

// acc[nt][e]: e = (row g, tok 2t), (row g, tok 2t+1), (row g+8, tok 2t), (row g+8, tok 2t+1)
template <int FMT, int NT, bool DUMP>
__device__ __forceinline__ void sk_compute(const SkRec<FMT> &rec, const SkTile<NT> &tile, int st, const SkCtx<FMT, NT, DUMP> &c,
                                           float (&acc)[NT][4])
{
    const int g = c.g, t = c.t;
    if constexpr (FMT == FMT_Q4_K) {
        float d[2], dmin[2];
        unsigned sc[2][2], mn[2][2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const uint4 h = r ? rec.s1 : rec.s0;
            d[r] = sk_h2f(h.x & 0xffffu);
            dmin[r] = sk_h2f(h.x >> 16);
            sc[r][0] = h.y & 0x3F3F3F3Fu;
            mn[r][0] = h.z & 0x3F3F3F3Fu;
            sc[r][1] = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
            mn[r][1] = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
        }
        float part[NT][4], mpart[NT][4];   // sum over sub-blocks of sc * dot * d_x, and of m * d_x * sum q
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) { part[nt][e] = 0.f; mpart[nt][e] = 0.f; }
        // The offset term of the whole super-block is one small product, mins [16 rows x 8 sub-blocks] times
        // (d_x * sum q) [8 sub-blocks x 8 tokens]: two tf32 tensor-core instructions per token group (the second for what
        // the tf32 rounding of d_x * sum q leaves over) instead of four multiply-adds per sub-block and token group. The
        // accumulator comes back in the same (row, token) arrangement as the int8 tiles'.
        {
            const unsigned ma0 = __float_as_uint((float)((mn[0][0] >> (8 * t)) & 0xffu)), ma1 = __float_as_uint((float)((mn[1][0] >> (8 * t)) & 0xffu));
            const unsigned ma2 = __float_as_uint((float)((mn[0][1] >> (8 * t)) & 0xffu)), ma3 = __float_as_uint((float)((mn[1][1] >> (8 * t)) & 0xffu));
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const float s0 = tile.sx(t, nt * 8 + g), s1 = tile.sx(t + 4, nt * 8 + g);
                const unsigned h0 = __float_as_uint(s0) & 0xFFFFE000u, h1 = __float_as_uint(s1) & 0xFFFFE000u;
                mma_tf32_k8(mpart[nt], ma0, ma1, ma2, ma3, h0, h1);
                mma_tf32_k8(mpart[nt], ma0, ma1, ma2, ma3, __float_as_uint(s0 - __uint_as_float(h0)), __float_as_uint(s1 - __uint_as_float(h1)));
            }
        }
#pragma unroll
        for (int sb = 0; sb < 8; sb++) {
            const int ch = sb >> 1, sh = 4 * (sb & 1);
            const unsigned a0 = (rec.q[ch].x >> sh) & 0x0F0F0F0Fu, a2 = (rec.q[ch].y >> sh) & 0x0F0F0F0Fu;
            const unsigned a1 = (rec.q[ch].z >> sh) & 0x0F0F0F0Fu, a3 = (rec.q[ch].w >> sh) & 0x0F0F0F0Fu;
            float scf[2], scb[2];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                scf[r] = (float)((sc[r][sb >> 2] >> (8 * (sb & 3))) & 0xffu);
                scb[r] = -SK_BIAS_F * scf[r];   // exact: 1.5 * 2^23 * (6-bit integer)
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int2 x = *reinterpret_cast<const int2 *>(tile.x(nt * 8 + g, sb * 32 + 8 * t));
                int cc[4];
                mma_u8s8_k32(cc, a0, a1, a2, a3, x.x, x.y);
                const float4 ds = tile.ds2(sb, nt * 8 + 2 * t);
                // (biased - 12582912) * sc = dot * sc, exact in one FMA (|dot * sc| < 2^22)
                part[nt][0] = fmaf(fmaf(__int_as_float(cc[0]), scf[0], scb[0]), ds.x, part[nt][0]);
                part[nt][1] = fmaf(fmaf(__int_as_float(cc[1]), scf[0], scb[0]), ds.z, part[nt][1]);
                part[nt][2] = fmaf(fmaf(__int_as_float(cc[2]), scf[1], scb[1]), ds.x, part[nt][2]);
                part[nt][3] = fmaf(fmaf(__int_as_float(cc[3]), scf[1], scb[1]), ds.z, part[nt][3]);
                c.export_tile(st * 8 + sb, nt, cc, 0);
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[nt][e] += fmaf(d[e >> 1], part[nt][e], -dmin[e >> 1] * mpart[nt][e]);
    } else if constexpr (FMT == FMT_Q8_0 || FMT == FMT_Q4_0) {
        const unsigned s0w[4] = { rec.s0.x, rec.s0.y, rec.s0.z, rec.s0.w }, s1w[4] = { rec.s1.x, rec.s1.y, rec.s1.z, rec.s1.w };
#pragma unroll
        for (int i = 0; i < 8; i++) {
            constexpr float unit = FMT == FMT_Q4_0 ? 0.0625f : 1.0f;   // the Q4_0 codes enter the MMA times 16
            const float dw[2] = { sk_h2f((s0w[i >> 1] >> (16 * (i & 1))) & 0xffffu) * unit,
                                  sk_h2f((s1w[i >> 1] >> (16 * (i & 1))) & 0xffffu) * unit };
            const float cb[2] = { -SK_BIAS_F * dw[0], -SK_BIAS_F * dw[1] };   // exact: d_w has an 11-bit significand
            unsigned a0, a1, a2, a3;
            if constexpr (FMT == FMT_Q8_0) {
                a0 = rec.q[i].x; a1 = rec.q[i].z; a2 = rec.q[i].y; a3 = rec.q[i].w;
            } else {
                const unsigned wg = (i & 1) ? rec.q[i >> 1].z : rec.q[i >> 1].x;
                const unsigned wg8 = (i & 1) ? rec.q[i >> 1].w : rec.q[i >> 1].y;
                // 16 * (code - 8) as signed bytes, one logic operation per four codes (the nibble in the byte's high
                // half is 16 * code, flipping the top bit subtracts 128): no offset term, the 16 leaves through dw
                a0 = ((wg << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
                a1 = ((wg8 << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
                a2 = (wg & 0xF0F0F0F0u) ^ 0x80808080u;
                a3 = (wg8 & 0xF0F0F0F0u) ^ 0x80808080u;
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                int b0, b1;
                if constexpr (FMT == FMT_Q8_0) {
                    const int2 x = *reinterpret_cast<const int2 *>(tile.x(nt * 8 + g, i * 32 + 8 * t));
                    b0 = x.x; b1 = x.y;
                } else {
                    const int8_t *xp = tile.x(nt * 8 + g, i * 32 + 4 * t);
                    b0 = *reinterpret_cast<const int *>(xp);
                    b1 = *reinterpret_cast<const int *>(xp + 16);
                }
                int cc[4];
                mma_s8s8_k32(cc, a0, a1, a2, a3, b0, b1);
                const float4 ds = tile.ds2(i, nt * 8 + 2 * t);
                acc[nt][0] = fmaf(fmaf(__int_as_float(cc[0]), dw[0], cb[0]), ds.x, acc[nt][0]);
                acc[nt][1] = fmaf(fmaf(__int_as_float(cc[1]), dw[0], cb[0]), ds.z, acc[nt][1]);
                acc[nt][2] = fmaf(fmaf(__int_as_float(cc[2]), dw[1], cb[1]), ds.x, acc[nt][2]);
                acc[nt][3] = fmaf(fmaf(__int_as_float(cc[3]), dw[1], cb[1]), ds.z, acc[nt][3]);
                c.export_tile(st * 8 + i, nt, cc, FMT == FMT_Q8_0 ? 128 : 8, FMT == FMT_Q4_0 ? 4 : 0);
            }
        }
    } else {  // Q6_K
        const float d[2] = { sk_h2f(rec.d0), sk_h2f(rec.d1) };
        const unsigned scw[2][4] = { { rec.s0.x, rec.s0.y, rec.s0.z, rec.s0.w }, { rec.s1.x, rec.s1.y, rec.s1.z, rec.s1.w } };
        float part[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) part[nt][e] = 0.f;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint4 A = rec.q[3 * h], B = rec.q[3 * h + 1], H = rec.q[3 * h + 2];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int blk = 4 * h + j;
                unsigned code[2][2];
                float scf[2][2], scb[2][2];
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
                        code[hl][r] = __vsub4(lo4 | hi2, 0x20202020u);
                        scf[hl][r] = (float)(int)(signed char)((scw[r][gi >> 2] >> (8 * (gi & 3))) & 0xffu);
                        scb[hl][r] = -SK_BIAS_F * scf[hl][r];   // exact: 1.5 * 2^23 * (8-bit integer)
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int8_t *xp = tile.x(nt * 8 + g, blk * 32 + 4 * t);
                    const int b0 = *reinterpret_cast<const int *>(xp), b1 = *reinterpret_cast<const int *>(xp + 16);
                    int c0[4], c1[4];
                    mma_s8s8_k16(c0, code[0][0], code[0][1], b0);
                    mma_s8s8_k16(c1, code[1][0], code[1][1], b1);
                    const float4 ds = tile.ds2(blk, nt * 8 + 2 * t);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int r = e >> 1;
                        // sc * dot of both 16-value groups, each product exact, their sum < 2^24
                        const float v = fmaf(__int_as_float(c0[e]), scf[0][r], scb[0][r]) +
                                        fmaf(__int_as_float(c1[e]), scf[1][r], scb[1][r]);
                        part[nt][e] = fmaf(v, (e & 1) ? ds.z : ds.x, part[nt][e]);
                    }
                    if (DUMP) {
                        const int sum[4] = { c0[0] + c1[0] - SK_BIAS, c0[1] + c1[1] - SK_BIAS, c0[2] + c1[2] - SK_BIAS,
                                             c0[3] + c1[3] - SK_BIAS };
                        c.export_tile(st * 8 + blk, nt, sum, 32);
                    }
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[nt][e] = fmaf(d[e >> 1], part[nt][e], acc[nt][e]);
    }
}

// Depth of the activation ring. Deeper rings were measured slower on B200 (fewer CTAs per SM for the larger token
// tiles, no gain for the small ones, which are bound by instruction issue, not by latency).
__host__ __device__ constexpr int sk_depth(int nt) { return 2; }
// Slots of a warp's weight-record ring: one for the 64-token tile (its refill is issued as soon as the record is in
// registers and travels during the step's arithmetic), which keeps two CTAs per SM. Up to 16 tokens the depth depends on
// how the launch runs: beside its predecessor (early) the neighbours keep the memory system busy and two slots with more
// CTAs per SM are best (8.7 against 9.9 us per launch on [14336, 4096] at 4 rows); a launch that waits for its predecessor
// is alone on the machine, has too few bytes in flight with two slots, and takes four (13.9 against 18.9 us).
__host__ __device__ constexpr int sk_wdepth(int nt, bool deep) { return nt == 8 ? 1 : (nt <= 2 && deep) ? 4 : sk_depth(nt); }

template <int FMT, int NT, bool DUMP, bool DEEP>
__global__ void __launch_bounds__(SK_WARPS * 32)
skinny_kernel(const WeightView w, const ActView a, int row0, int rows, float *__restrict__ y, long long y_stride,
              int *dump, int *status, int early, const Exchange ex, const Epilogue ep, float *split_scratch, int *split_counters)
{
    extern __shared__ __align__(128) unsigned char sk_smem[];
    __shared__ __align__(8) uint64_t bars[SK_WARPS][4];
    constexpr int T = NT * 8, TILE = SkTile<NT>::BYTES, D = sk_depth(NT), WD = sk_wdepth(NT, DEEP), REC = record_bytes(FMT);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rgl = warp & (SK_RGS - 1), ks = warp / SK_RGS;
    const int rg_count = w.n_pad >> 4;
    const int rg = blockIdx.x * SK_RGS + rgl;
    const bool rg_live = rg < rg_count;
    // gridDim.y > 1: the K range is cut in gridDim.y chunks of super-tiles, one CTA each (few weight rows, long K: the row
    // tiles alone would leave most SMs idle); the chunks' partial tiles meet in global memory at the end
    const int nst_all = w.k_pad >> 8;
    const int chunk = (nst_all + (int)gridDim.y - 1) / (int)gridDim.y;
    const int sb = (int)blockIdx.y * chunk;                                   // first super-tile of this CTA
    const int nst = nst_all - sb < chunk ? (nst_all - sb > 0 ? nst_all - sb : 0) : chunk;   // and how many
    const int per = (nst + SK_KS - 1) / SK_KS;          // super-tiles per K half; both halves take `per` steps
    const int st0 = sb + ks * per;
    const int left = nst - ks * per;
    const int my_steps = !rg_live ? 0 : (left < per ? (left > 0 ? left : 0) : per);
    SkCtx<FMT, NT, DUMP> c{ w, a, row0, rg, lane >> 2, lane & 3, dump };
    unsigned char *act_ring = sk_smem;                                     // [D][SK_KS][TILE]
    uint8_t *w_ring = sk_smem + (size_t)D * SK_KS * TILE + (size_t)warp * WD * REC;   // this warp's [WD][REC]

    // this warp's weight records: the first D bulk copies start before anything else (weights depend on no kernel)
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < WD; s++) mbar_init(&bars[warp][s], 1);
        fence_mbar_init();
#pragma unroll
        for (int s = 0; s < WD; s++) {
            if (s < my_steps) bulk_load(w_ring + s * REC, w.record(rg, st0 + s), REC, &bars[warp][s]);
        }
    }

    pdl_enter(early);   // waits for the kernel that produced the activations unless they were complete before it

    // act_ring[b] <- activation tiles of step i for both K halves
    auto stage = [&](int b, int i) {
        if (i < per) {
            for (int h = 0; h < SK_KS; h++) {
                if (h * per + i >= nst) continue;
                const int st = sb + h * per + i;
                unsigned char *dst = act_ring + (b * SK_KS + h) * TILE;
                for (int idx = threadIdx.x; idx < T * 16; idx += SK_WARPS * 32) {
                    const int tok = idx >> 4, ch = idx & 15;
                    cp_async16(dst + tok * SK_XROW + ch * 16, a.q + (long long)(row0 + tok) * a.k_pad + st * 256 + ch * 16);
                }
                for (int idx = threadIdx.x; idx < 8 * (T / 2); idx += SK_WARPS * 32) {
                    const int blk = idx / (T / 2), pair = idx % (T / 2);
                    cp_async16(dst + T * SK_XROW + (blk * T + pair * 2) * 8,
                               a.ds + (long long)(st * 8 + blk) * a.rows_pad + row0 + pair * 2);
                }
            }
        }
        cp_async_commit();   // one group per step, empty past the end, so the wait below always counts the same
    };

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[nt][e] = 0.0f;

#pragma unroll
    for (int s = 0; s < D - 1; s++) stage(s, s);
    bool alive = true;
    for (int i = 0; i < per; i++) {
        stage((i + D - 1) % D, i + D - 1);
        cp_async_wait<D - 1>();   // the group of step i has landed
        __syncthreads();
        if (i < my_steps && alive) {
            const int s = i % WD;
            if (!mbar_wait(&bars[warp][s], (unsigned)(i / WD) & 1u)) {
                if (lane == 0) atomicExch(status, -7);
                alive = false;
            } else {
                SkRec<FMT> rec;
                sk_load<FMT>(rec, w_ring + s * REC, lane);
                __syncwarp();   // every lane holds its part of the record: the slot may be refilled
                if (lane == 0 && i + WD < my_steps) bulk_load(w_ring + s * REC, w.record(rg, st0 + i + WD), REC, &bars[warp][s]);
                const SkTile<NT> tile{ act_ring + ((i % D) * SK_KS + ks) * TILE };
                sk_compute<FMT, NT, DUMP>(rec, tile, st0 + i, c, acc);
            }
        }
        __syncthreads();   // buffer i % D is refilled by the next iteration: everyone is done reading it
    }
    cp_async_wait<0>();

    // the two K halves of a row group meet in shared memory
    float *red = reinterpret_cast<float *>(sk_smem);
    if (ks == 1) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) red[((rgl * NT + nt) * 4 + e) * 32 + lane] = acc[nt][e];
    }
    __syncthreads();
    if (gridDim.y > 1) {
        // K chunks: every CTA leaves its 64-column partial tile in global memory; the CTA that arrives last for these
        // columns adds the parts in chunk order (the same order whichever CTA it is) and stores
        __shared__ int is_last;
        float *part = split_scratch + ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * (T * 64);
        if (ks == 0) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float v = acc[nt][e] + red[((rgl * NT + nt) * 4 + e) * 32 + lane];   // zero for absent row groups
                    __stcg(&part[(nt * 8 + 2 * c.t + (e & 1)) * 64 + rgl * 16 + c.g + 8 * (e >> 1)], v);
                }
            }
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const int arrived = atomicAdd(&split_counters[blockIdx.x], 1);
            is_last = arrived == (int)gridDim.y - 1;
            if (is_last) split_counters[blockIdx.x] = 0;   // ready for the next launch
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            for (int idx = threadIdx.x; idx < rows * 64; idx += SK_WARPS * 32) {
                const int m = idx >> 6, col = idx & 63, row = blockIdx.x * 64 + col;
                float sum = 0.0f;
                for (int p = 0; p < (int)gridDim.y; p++) {
                    sum += __ldcg(split_scratch + ((size_t)p * gridDim.x + blockIdx.x) * (T * 64) + m * 64 + col);
                }
                if (row < w.n) y[(long long)(row0 + m) * y_stride + row] = ep.apply(sum, row0 + m, row);
            }
        }
    } else if (ex.world == 0) {
        if (ks == 0 && rg_live) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float v = acc[nt][e] + red[((rgl * NT + nt) * 4 + e) * 32 + lane];
                    const int row = rg * 16 + c.g + 8 * (e >> 1);
                    const int m = nt * 8 + 2 * c.t + (e & 1);
                    if (row < w.n && m < rows) y[(long long)(row0 + m) * y_stride + row] = ep.apply(v, row0 + m, row);
                }
            }
        }
    } else {
        // Row-split MatMul of a tensor-parallel group (exchange.cuh). The CTA's partial tile is first laid out in
        // shared memory as [token][64 columns], so that it leaves for the peers in 16-byte stores along the columns.
        float *tile = red + SK_RGS * NT * 4 * 32;
        if (ks == 0) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float v = acc[nt][e] + red[((rgl * NT + nt) * 4 + e) * 32 + lane];   // zero for absent row groups
                    tile[(nt * 8 + 2 * c.t + (e & 1)) * 64 + rgl * 16 + c.g + 8 * (e >> 1)] = v;
                }
            }
        }
        __syncthreads();
        const int epoch = ex_epoch(ex), slot = epoch & 1;
        const int col0 = blockIdx.x * 64;
        if (NT * 8 <= SLC_LL_ROWS) {
            // few rows: every value travels as one {value, tag} word and is awaited by the thread that owns it
            for (int idx = threadIdx.x; idx < rows * 64; idx += SK_WARPS * 32) {
                ex_ll_send(ex, slot, epoch, idx >> 6, col0 + (idx & 63), tile[idx]);
            }
            bool ok = true;
            const unsigned long long wait_from = ex_now();
            for (int idx = threadIdx.x; idx < rows * 64; idx += SK_WARPS * 32) {
                const int m = idx >> 6, col = col0 + (idx & 63);
                const float total = ex_ll_collect(ex, slot, epoch, m, col, tile[idx], ok, wait_from);
                if (col < w.n) y[(long long)(row0 + m) * y_stride + col] = ep.apply(total, row0 + m, col);
            }
            if (!ok) atomicExch(status, -7);
        } else {
            for (int idx = threadIdx.x; idx < rows * 16; idx += SK_WARPS * 32) {
                const int m = idx >> 4, c4 = (idx & 15) * 4;
                const float4 v = *reinterpret_cast<const float4 *>(tile + m * 64 + c4);
                for (int p = 0; p < ex.world; p++) {
                    *reinterpret_cast<float4 *>(ex.recv[p] + ex_index(ex, slot, ex.rank, m, col0 + c4)) = v;
                }
            }
            if (!ex_publish_and_wait(ex, slot, epoch, blockIdx.x) && threadIdx.x == 0) atomicExch(status, -7);
            for (int idx = threadIdx.x; idx < rows * 16; idx += SK_WARPS * 32) {
                const int m = idx >> 4, c4 = (idx & 15) * 4;
                const float4 sum = ex_sum4(ex, slot, m, col0 + c4);
                const float sv[4] = { sum.x, sum.y, sum.z, sum.w };
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (col0 + c4 + j < w.n) y[(long long)(row0 + m) * y_stride + col0 + c4 + j] = ep.apply(sv[j], row0 + m, col0 + c4 + j);
                }
            }
        }
        ex_finish(ex, epoch);
    }
    pdl_exit(early);
}

template <int FMT, int NT, bool DUMP, bool DEEP>
static cudaError_t launch_cfg_depth(const WeightView &w, const ActView &a, int row0, int rows, float *y, long long y_stride,
                                    int *dump, int *status, int early, cudaStream_t stream, const Exchange &ex, const Epilogue &ep,
                                    const SkinnySplit &sp)
{
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = skinny_kernel<FMT, NT, DUMP, DEEP>;
    // activation ring (depth x two K halves) + one weight-record ring per warp; the epilogue reuses the front of it
    // for the K-half reduction (NT x 2 KB) and, when exchanging, the outgoing tile (NT x 2 KB)
    size_t smem = (size_t)sk_depth(NT) * SK_KS * SkTile<NT>::BYTES + (size_t)SK_WARPS * sk_wdepth(NT, DEEP) * record_bytes(FMT);
    if (smem < (size_t)NT * 4096) smem = (size_t)NT * 4096;
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int rg_count = w.n_pad >> 4;
    const int ctas = (rg_count + SK_RGS - 1) / SK_RGS;
    if (ex.world > 1) {
        // as in the mat-vec: an exchanging grid must fit the machine at once
        int per_sm = 0, sms = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, SK_WARPS * 32, smem);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        if (ctas > per_sm * sms) return cudaErrorLaunchOutOfResources;
    }
    // K chunks when the row tiles alone leave CTA slots empty (4 CTAs of the small token tiles fit an SM, 2 of the large
    // ones): at least four super-tiles per chunk, at most 8 chunks, and only while the partial tiles fit the scratch area
    int split = 1;
    const int slots = (NT <= 2 ? 4 : 2) * sp.sm_count;
    if (sp.scratch && sp.counters && ex.world == 0 && ctas < sp.sm_count && ctas <= sp.counter_slots) {
        split = slots / ctas;
        const int nst = w.k_pad >> 8;
        if (split > nst / 4) split = nst / 4;
        if (split > 8) split = 8;
        while (split > 1 && (size_t)split * ctas * (NT * 8 * 64) > sp.scratch_floats) split--;
        if (split < 1) split = 1;
    }
    return launch_pdl(kernel, dim3(ctas, split), dim3(SK_WARPS * 32), smem, stream, w, a, row0, rows,
                      y, y_stride, dump, status, split > 1 ? 0 : early, ex, ep, sp.scratch, sp.counters);
}

// The deep weight ring for launches that run alone (not early); the parity export keeps the shallow one.
template <int FMT, int NT, bool DUMP>
static cudaError_t launch_cfg(const WeightView &w, const ActView &a, int row0, int rows, float *y, long long y_stride,
                              int *dump, int *status, int early, cudaStream_t stream, const Exchange &ex, const Epilogue &ep,
                              const SkinnySplit &sp)
{
    if constexpr (NT <= 2 && !DUMP) {
        if (!early) return launch_cfg_depth<FMT, NT, DUMP, true>(w, a, row0, rows, y, y_stride, dump, status, early, stream, ex, ep, sp);
    }
    return launch_cfg_depth<FMT, NT, DUMP, false>(w, a, row0, rows, y, y_stride, dump, status, early, stream, ex, ep, sp);
}

template <int FMT, bool DUMP>
static cudaError_t launch_nt(const WeightView &w, const ActView &a, int row0, int rows, float *y, long long y_stride,
                             int *dump, int *status, int early, cudaStream_t stream, const Exchange &ex, const Epilogue &ep,
                             const SkinnySplit &sp)
{
    if (rows <= 8) return launch_cfg<FMT, 1, DUMP>(w, a, row0, rows, y, y_stride, dump, status, early, stream, ex, ep, sp);
    if (rows <= 16) return launch_cfg<FMT, 2, DUMP>(w, a, row0, rows, y, y_stride, dump, status, early, stream, ex, ep, sp);
    if (rows <= 32) return launch_cfg<FMT, 4, DUMP>(w, a, row0, rows, y, y_stride, dump, status, early, stream, ex, ep, sp);
    if (rows <= 64) return launch_cfg<FMT, 8, DUMP>(w, a, row0, rows, y, y_stride, dump, status, early, stream, ex, ep, sp);
    return cudaErrorInvalidValue;
}

// row0 must be a multiple of 8 (activation scale pairs are fetched with aligned 128-bit accesses), and the quantized
// activations must be padded to the token tile (8, 16, 32 or 64 rows).
cudaError_t launch_skinny(const WeightView &w, const ActView &a, int row0, int rows, float *y, long long y_stride,
                          int *dump, int *status, int early, cudaStream_t stream, const Exchange *exchange,
                          const Epilogue *epilogue, const SkinnySplit *split)
{
    if (w.n_pad == 0 || rows == 0) return cudaSuccess;
    const SkinnySplit sp = split ? *split : SkinnySplit{ nullptr, nullptr, 0, 0, 0 };
    const Epilogue ep = epilogue ? *epilogue : Epilogue{ nullptr, nullptr, 0 };
    if (row0 & 7) return cudaErrorInvalidValue;
    Exchange ex{};
    if (exchange) {
        ex = *exchange;
        const int ctas = ((w.n_pad >> 4) + SK_RGS - 1) / SK_RGS;
        if (early || rows > ex.max_rows || ctas * 64 > ex.n_stride || ctas > ex.groups) return cudaErrorInvalidValue;
    }
#define SLC_FMT(F) \
    case F: return dump ? launch_nt<F, true>(w, a, row0, rows, y, y_stride, dump, status, early, stream, ex, ep, sp) \
                        : launch_nt<F, false>(w, a, row0, rows, y, y_stride, nullptr, status, early, stream, ex, ep, sp);
    switch (w.fmt) {
        SLC_FMT(FMT_Q8_0) SLC_FMT(FMT_Q4_0) SLC_FMT(FMT_Q4_K) SLC_FMT(FMT_Q6_K)
    default: return cudaErrorInvalidValue;
    }
#undef SLC_FMT
}

}  // namespace slc
