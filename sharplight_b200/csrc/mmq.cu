// Prefill GEMM on the 5th-generation tensor cores: y[t][n] = sum over 32-value blocks of d_w[n,b] * d_x[t,b] * S[n,t,b],
// S = the exact int32 dot of weight codes and 8-bit activation codes of block b -- the integer-dot arithmetic of
// src/Sharplight.Cpu/IntDot.Kernels.cs:12-29 applied to many rows, scaled per block as the reference's int8 GEMM does
// (src/Sharplight.Shaders/Kernels/mmq.slang:224-233 of the Sharplight tree: acc += float(C) * (d_x * d_w) - s_x * m_w).
//
// One CTA computes a 128 (weight rows) x 128 (tokens) tile. Roles, warp-specialised:
//   warps 0-15  epilogue, four per scheduler: read each block's tile from tensor memory (tcgen05.ld, 16 columns at a
//               time), scale, accumulate in f32 registers; warp w owns TMEM lanes 32*(w%4).. and columns 32*(w/4)..
//   warps 16-19 producers: stream the weight records (layout.cuh) with 128-bit loads, expand 4- and 6-bit codes to int8 in
//               registers and store them in the K-major core-matrix layout the tensor core reads; lane 0 of warp 16
//               also starts the bulk async copies (TMA engine) of the activation tile, which the quantizer already
//               wrote in that layout, and of the activation scales
//   warp 20     allocates tensor memory; its lane 0 issues tcgen05.mma kind::i8 (M=128, N=128, K=32: one quantization
//               block per instruction, each into its own accumulator buffer: per-block scales forbid accumulating
//               across blocks in int32; Q6_K, whose scale changes every 16 values: two instructions per block on two
//               half-masked copies of the weight rows) and commits to mbarriers
// Pipelines: 3 shared-memory stages of 256 K-values (8 blocks; 2 stages for Q4_K and Q6_K), 4 TMEM accumulator buffers of
// 128 columns; the producers keep the next stage's weight records in registers while the current one is expanded.
// Every mbarrier wait is bounded; when one runs out the kernel raises the device status word, and every role leaves
// through the common exit that frees tensor memory.
#include "internal.cuh"

namespace slc {

constexpr int MQ_TILE_N = 128;     // weight rows per CTA (UMMA M)
constexpr int MQ_TILE_T = 128;     // tokens per CTA (UMMA N)
// Q6_K changes its scale every 16 values: a 32-value block is two MMAs on two copies of the weight rows, one with the
// upper and one with the lower sixteen values zero (the same activation codes both times), into two accumulator buffers
// with a weight scale each (the reference's GEMM does the same, src/Sharplight.Shaders/Kernels/mmq.slang:235-239)
__host__ __device__ constexpr int mq_gpb(int fmt) { return fmt == FMT_Q6_K ? 2 : 1; }   // MMAs (scale groups) per block
// shared-memory stages: three, or two for the formats with a larger stage (Q4_K: offset tables; Q6_K: two weight copies)
__host__ __device__ constexpr int mq_stages(int fmt) { return fmt == FMT_Q4_K || fmt == FMT_Q6_K ? 2 : 3; }
constexpr int MQ_MAX_STAGES = 3;
constexpr int MQ_DBUF = 4;
constexpr int MQ_EPI_WARPS = 16, MQ_PROD_WARPS = 4;
constexpr int MQ_THREADS = 768;   // warps 0-15 epilogue, 16-19 producers, 20 MMA issuer, 21-23 idle (they fill the warpgroup)
// a wait suspends in hardware for up to ~20 us per attempt (the hint below) instead of spinning on issue slots the
// epilogue needs; 100000 attempts bound it at about two seconds
constexpr unsigned MQ_WAIT_LIMIT = 100000;

constexpr int MQ_A_BYTES = MQ_TILE_N * 256;          // int8 codes of one stage (one copy)
constexpr int MQ_B_BYTES = MQ_TILE_T * 256;
constexpr int MQ_DX_BYTES = 8 * MQ_TILE_T * 4;       // d per block and token (a second table of d * sum32(q) for Q4_K)
constexpr int MQ_DW_BYTES = MQ_TILE_N * 8 * 4;       // weight scale per row and block (a second table of mins for Q4_K)
__host__ __device__ constexpr int mq_stage_bytes(int fmt)
{
    return mq_gpb(fmt) * MQ_A_BYTES + MQ_B_BYTES + (fmt == FMT_Q4_K ? 2 : 1) * MQ_DX_BYTES + (fmt == FMT_Q4_K ? 2 : mq_gpb(fmt)) * MQ_DW_BYTES;
}
__host__ __device__ constexpr int mq_smem_bytes(int fmt) { return mq_stages(fmt) * mq_stage_bytes(fmt) + 1024; }

// ---- PTX wrappers ----------------------------------------------------------------------------------------------------

__device__ __forceinline__ unsigned mq_smem(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mq_bar_init(uint64_t *bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mq_smem(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mq_bar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mq_smem(bar)) : "memory");
}

__device__ __forceinline__ void mq_bar_expect_tx(uint64_t *bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mq_smem(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mq_bulk_load(void *dst, const void *src, unsigned bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(mq_smem(dst)), "l"(src), "r"(bytes), "r"(mq_smem(bar)) : "memory");
}

// Bounded wait on a phase parity. Returns false when the limit ran out.
__device__ __forceinline__ bool mq_bar_wait(uint64_t *bar, unsigned parity)
{
    const unsigned b = mq_smem(bar);
    for (unsigned i = 0; i < MQ_WAIT_LIMIT; i++) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(b), "r"(parity), "r"(20000u) : "memory");
        if (ok) return true;
    }
    return false;
}

__device__ __forceinline__ void mq_fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mq_tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mq_tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] += A[smem] * B[smem], int8 x int8 -> int32. The accumulator holds MQ_BIAS when the instruction starts (the
// epilogue re-arms it), so the result is MQ_BIAS + block dot: the bit pattern of the float 12582912 + dot.
__device__ __forceinline__ void mq_umma_i8(unsigned tmem_d, uint64_t adesc, uint64_t bdesc, unsigned idesc)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(1u), "r"(0u) : "memory");
}

__device__ __forceinline__ void mq_umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mq_smem(bar)) : "memory");
}

// The 32-bit results are declared as f32 registers: the values are used as floats (biased accumulators), and typing them
// so from the start leaves no integer-to-float register moves behind.
__device__ __forceinline__ void mq_tmem_ld16(unsigned taddr, float (&r)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]),
                   "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15])
                 : "r"(taddr) : "memory");
}

// int32 -> f32 without a conversion instruction (the conversion unit delivers 16 results per clock per SM, which alone
// would cost ~1000 cycles per 128x128 block): for |s| < 2^22 the bit pattern 0x4B400000 + s is the float 12582912 + s.
// The tensor core does the integer add: every accumulator buffer is pre-loaded with the pattern.
constexpr int MQ_BIAS = 0x4B400000;
constexpr float MQ_BIAS_F = 12582912.0f;

// Eight registers that hold the bias pattern for the whole kernel; tcgen05.st .x8 takes eight distinct registers. They
// are read from shared memory with volatile loads so that the compiler cannot re-create them from the constant before
// every store. Eight rather than sixteen (with .x16 stores): the epilogue's 88 registers then hold everything without
// spilling, which was worth 12 % of the kernel's time.
struct MqBias16
{
    int v[8];
    __device__ __forceinline__ void init(const int *word)   // word: shared memory holding MQ_BIAS
    {
        const unsigned addr = (unsigned)__cvta_generic_to_shared(word);
#pragma unroll
        for (int j = 0; j < 8; j++) asm volatile("ld.volatile.shared.b32 %0, [%1];" : "=r"(v[j]) : "r"(addr) : "memory");
    }
};

__device__ __forceinline__ void mq_tmem_st8(unsigned taddr, const MqBias16 &b)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(b.v[0]), "r"(b.v[1]), "r"(b.v[2]), "r"(b.v[3]), "r"(b.v[4]), "r"(b.v[5]), "r"(b.v[6]), "r"(b.v[7]) : "memory");
}
__device__ __forceinline__ void mq_tmem_st16(unsigned taddr, const MqBias16 &b)
{
    mq_tmem_st8(taddr, b);
    mq_tmem_st8(taddr + 8u, b);
}

__device__ __forceinline__ void mq_tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void mq_tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices of 128 contiguous bytes;
// the two core matrices of one K=32 step are lbo bytes apart, groups of 8 rows sbo bytes apart.
__device__ __forceinline__ uint64_t mq_desc(unsigned smem_addr, unsigned lbo, unsigned sbo)
{
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}

// Instruction descriptor of kind::i8: int32 accumulator, A signed or unsigned 8-bit, B signed, both K-major.
__host__ __device__ constexpr unsigned mq_idesc(bool a_signed, int m, int n)
{
    return (2u << 4) | ((a_signed ? 1u : 0u) << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

__device__ __forceinline__ float mq_h2f(unsigned bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

struct MqSmem
{
    uint64_t a_full[MQ_MAX_STAGES], b_full[MQ_MAX_STAGES], mma_done[MQ_MAX_STAGES], epi_done[MQ_MAX_STAGES];
    uint64_t d_full[MQ_DBUF], d_empty[MQ_DBUF];
    unsigned tmem_base;
    int abort;
    int bias_word;
};

// ---- producer: one row group (16 rows) of one stage -> int8 codes in the A tile, scales in the tables ------------------

template <int FMT>
struct MqRegs
{
    uint4 q[code_units(FMT) / 32];
    uint4 s0, s1;
    unsigned d01;   // Q6_K: the f16 super-block scales of rows g (low half) and g + 8
};

// The record of (rg, st) into registers (zeros for row groups beyond the weight).
template <int FMT>
__device__ __forceinline__ void mq_load(MqRegs<FMT> &rr, const WeightView &w, int rg, int st, int lane)
{
    const int g = lane >> 2;
    const bool live = rg * 16 < w.n_pad;
    const uint8_t *rec = w.record(live ? rg : 0, st);
    const uint4 *qp = reinterpret_cast<const uint4 *>(rec) + lane;
    const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int i = 0; i < code_units(FMT) / 32; i++) rr.q[i] = live ? ld_stream(qp + 32 * i) : zero;
    const uint4 *sp = reinterpret_cast<const uint4 *>(rec + code_bytes(FMT));
    rr.s0 = live ? ld_stream(sp + g) : zero;
    rr.s1 = live ? ld_stream(sp + g + 8) : zero;
    if constexpr (FMT == FMT_Q6_K) {
        const unsigned short *dp = reinterpret_cast<const unsigned short *>(rec + code_bytes(FMT) + 256);
        rr.d01 = live ? (unsigned)__ldg(dp + g) | ((unsigned)__ldg(dp + g + 8) << 16) : 0u;
    }
}

// Registers -> int8 codes in the A tile (rows rgl*16 .. +15), scales in the tables.
template <int FMT>
__device__ __forceinline__ void mq_store(const MqRegs<FMT> &rr, int rgl, int lane, uint8_t *a_tile, float *dws, float *dms)
{
    const int g = lane >> 2, t = lane & 3;
    uint8_t *row_lo = a_tile + (2 * rgl) * 2048 + g * 16, *row_hi = row_lo + 2048;   // rows g and g + 8
    const uint4 s0 = rr.s0, s1 = rr.s1;
    // scale tables are [block][row of the tile]: the epilogue's lanes (one row each) read them without bank conflicts
    float *dw_lo = dws + rgl * 16 + g, *dw_hi = dw_lo + 8;

    if constexpr (FMT == FMT_Q8_0) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint4 q = rr.q[i];
            const int off = (2 * i + (t >> 1)) * 128 + 8 * (t & 1);
            *reinterpret_cast<uint2 *>(row_lo + off) = make_uint2(q.x, q.y);
            *reinterpret_cast<uint2 *>(row_hi + off) = make_uint2(q.z, q.w);
        }
    } else if constexpr (FMT == FMT_Q4_0) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint4 q = rr.q[i];
            const unsigned wv[4] = { q.x, q.y, q.z, q.w };
#pragma unroll
            for (int j = 0; j < 4; j++) {
                // 16 * (code - 8) as signed bytes, one logic operation per four codes: the nibble moved to (or left in)
                // the byte's high half is 16 * code, and flipping the top bit subtracts 128. The block dot needs no
                // offset term; the factor 16 is taken out of the scale table below (exactly: a power of two).
                const unsigned lo = ((wv[j] << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
                const unsigned hi = (wv[j] & 0xF0F0F0F0u) ^ 0x80808080u;
                const int blk = 2 * i + (j >> 1);
                uint8_t *dst = ((j & 1) ? row_hi : row_lo) + (2 * blk) * 128 + 4 * t;
                *reinterpret_cast<unsigned *>(dst) = lo;
                *reinterpret_cast<unsigned *>(dst + 128) = hi;
            }
        }
    } else if constexpr (FMT == FMT_Q6_K) {
        // Half c of the super-block: planes 3c (row g) and 3c + 1 (row g + 8) hold L[l0..+3], L[32+l0..+3], L[l1..+3],
        // L[32+l1..+3] with l0 = 4t, l1 = 16 + 4t; plane 3c + 2 holds H[l0..+3], H[l1..+3] of row g, then of row g + 8.
        // Quarter v of the half is block 4c + v of the stage: its values l are (low or high nibble of L[l] or L[32 + l])
        // | (bits 2v, 2v+1 of H[l]) << 4, minus 32. Its lower sixteen values go to the first 16-byte chunk of the block
        // in the first copy, its upper sixteen to the second chunk in the second copy; the other chunks of both copies
        // stay zero (written once when the kernel starts).
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const uint4 L[2] = { rr.q[3 * c], rr.q[3 * c + 1] };
            const uint4 H = rr.q[3 * c + 2];
#pragma unroll
            for (int r = 0; r < 2; r++) {
#pragma unroll
                for (int li = 0; li < 2; li++) {
                    const unsigned lw = li ? L[r].z : L[r].x, lw32 = li ? L[r].w : L[r].y;
                    const unsigned hw = r ? (li ? H.w : H.z) : (li ? H.y : H.x);
                    uint8_t *dst = (r ? row_hi : row_lo) + li * MQ_A_BYTES + 4 * t;
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        const unsigned lsrc = (v & 1) ? lw32 : lw;
                        const unsigned lo4 = ((v & 2) ? (lsrc >> 4) : lsrc) & 0x0F0F0F0Fu;
                        const unsigned u = lo4 | (((hw >> (2 * v)) & 0x03030303u) << 4);       // 0..63
                        const unsigned x = u ^ 0x20202020u;                                     // six-bit two's complement of u - 32
                        const unsigned code = x | ((x & 0x20202020u) * 6u);                     // sign bit copied to bits 6, 7
                        *reinterpret_cast<unsigned *>(dst + (2 * (4 * c + v) + li) * 128) = code;
                    }
                }
            }
        }
    } else {  // Q4_K: unsigned nibbles, the mins go through the offset table
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const uint4 q = rr.q[c];
            const int off = (4 * c + (t >> 1)) * 128 + 8 * (t & 1);
            *reinterpret_cast<uint2 *>(row_lo + off) = make_uint2(q.x & 0x0F0F0F0Fu, q.y & 0x0F0F0F0Fu);
            *reinterpret_cast<uint2 *>(row_lo + off + 256) = make_uint2((q.x >> 4) & 0x0F0F0F0Fu, (q.y >> 4) & 0x0F0F0F0Fu);
            *reinterpret_cast<uint2 *>(row_hi + off) = make_uint2(q.z & 0x0F0F0F0Fu, q.w & 0x0F0F0F0Fu);
            *reinterpret_cast<uint2 *>(row_hi + off + 256) = make_uint2((q.z >> 4) & 0x0F0F0F0Fu, (q.w >> 4) & 0x0F0F0F0Fu);
        }
    }

    // scale tables: lane t converts blocks 2t and 2t + 1 of rows g and g + 8
    if constexpr (FMT == FMT_Q8_0 || FMT == FMT_Q4_0) {
        const unsigned w0 = t == 0 ? s0.x : t == 1 ? s0.y : t == 2 ? s0.z : s0.w;
        const unsigned w1 = t == 0 ? s1.x : t == 1 ? s1.y : t == 2 ? s1.z : s1.w;
        constexpr float unit = FMT == FMT_Q4_0 ? 0.0625f : 1.0f;   // the Q4_0 codes are stored times 16
        dw_lo[(2 * t) * MQ_TILE_N] = mq_h2f(w0 & 0xffffu) * unit;
        dw_lo[(2 * t + 1) * MQ_TILE_N] = mq_h2f(w0 >> 16) * unit;
        dw_hi[(2 * t) * MQ_TILE_N] = mq_h2f(w1 & 0xffffu) * unit;
        dw_hi[(2 * t + 1) * MQ_TILE_N] = mq_h2f(w1 >> 16) * unit;
    } else if constexpr (FMT == FMT_Q6_K) {
        // i8 scales of the 16-value groups 4t .. 4t + 3 (group 2b + li is copy li of block b), times the row's f16 d
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const uint4 h = r ? s1 : s0;
            const float d = mq_h2f(r ? rr.d01 >> 16 : rr.d01 & 0xffffu);
            const unsigned scw = t == 0 ? h.x : t == 1 ? h.y : t == 2 ? h.z : h.w;
#pragma unroll
            for (int i = 0; i < 4; i++) (r ? dw_hi : dw_lo)[(4 * t + i) * MQ_TILE_N] = d * (float)(int)(signed char)((scw >> (8 * i)) & 0xffu);
        }
    } else {
        float *dm_lo = dms + rgl * 16 + g, *dm_hi = dm_lo + 8;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const uint4 h = r ? s1 : s0;
            const float d = mq_h2f(h.x & 0xffffu), dmin = mq_h2f(h.x >> 16);
            const unsigned sc_lo = h.y & 0x3F3F3F3Fu, mn_lo = h.z & 0x3F3F3F3Fu;
            const unsigned sc_hi = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
            const unsigned mn_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
            const unsigned scw = t < 2 ? sc_lo : sc_hi, mnw = t < 2 ? mn_lo : mn_hi;
            const int sh = 16 * (t & 1);
            const float2 sc = make_float2(d * (float)((scw >> sh) & 0xffu), d * (float)((scw >> (sh + 8)) & 0xffu));
            const float2 mn = make_float2(dmin * (float)((mnw >> sh) & 0xffu), dmin * (float)((mnw >> (sh + 8)) & 0xffu));
            (r ? dw_hi : dw_lo)[(2 * t) * MQ_TILE_N] = sc.x;
            (r ? dw_hi : dw_lo)[(2 * t + 1) * MQ_TILE_N] = sc.y;
            (r ? dm_hi : dm_lo)[(2 * t) * MQ_TILE_N] = mn.x;
            (r ? dm_hi : dm_lo)[(2 * t + 1) * MQ_TILE_N] = mn.y;
        }
    }
}

// ---- the kernel ------------------------------------------------------------------------------------------------------

template <int FMT, bool DUMP>
__global__ void __launch_bounds__(MQ_THREADS, 1)
mmq_kernel(const WeightView w, const ActView a, const uint8_t *__restrict__ q_tiled, float *__restrict__ y,
           long long y_stride, int *dump, int *status, int early, const Epilogue ep, int tile_t0)
{
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ MqSmem sh;
    // 1024-byte alignment of the tiles
    unsigned char *smem = smem_raw + ((1024 - (mq_smem(smem_raw) & 1023)) & 1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * MQ_TILE_N, t0 = ((int)blockIdx.y + tile_t0) * MQ_TILE_T;   // tile_t0: first token tile of this launch
    const int nst = w.k_pad >> 8;
    constexpr bool HAS_MIN = FMT == FMT_Q4_K;
    constexpr int MQ_STAGES = mq_stages(FMT), MQ_STAGE_BYTES = mq_stage_bytes(FMT);

    // stage layout: A codes, B codes, d_x table, d_w table, then (Q4_K) the d_x * sum q table and the mins table
    auto stage_a = [&](int s) { return smem + s * MQ_STAGE_BYTES; };
    constexpr int GPB = mq_gpb(FMT), A_ALL = GPB * MQ_A_BYTES;   // Q6_K: two half-masked copies of the weight rows
    auto stage_b = [&](int s) { return smem + s * MQ_STAGE_BYTES + A_ALL; };
    auto stage_dx = [&](int s) { return reinterpret_cast<float *>(smem + s * MQ_STAGE_BYTES + A_ALL + MQ_B_BYTES); };
    auto stage_dw = [&](int s) { return stage_dx(s) + 8 * MQ_TILE_T; };
    auto stage_sx = [&](int s) { return stage_dw(s) + MQ_TILE_N * 8; };
    auto stage_dm = [&](int s) { return stage_sx(s) + 8 * MQ_TILE_T; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < MQ_STAGES; s++) {
            mq_bar_init(&sh.a_full[s], MQ_PROD_WARPS);
            mq_bar_init(&sh.b_full[s], 1);
            mq_bar_init(&sh.mma_done[s], 1);
            mq_bar_init(&sh.epi_done[s], MQ_EPI_WARPS);
        }
        for (int b = 0; b < MQ_DBUF; b++) {
            mq_bar_init(&sh.d_full[b], 1);
            mq_bar_init(&sh.d_empty[b], MQ_EPI_WARPS);
        }
        sh.abort = 0;
        sh.bias_word = MQ_BIAS;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if constexpr (GPB > 1) {
        // the halves of the two weight copies that no producer ever writes
        for (int st = 0; st < MQ_STAGES; st++) {
            uint4 *z = reinterpret_cast<uint4 *>(stage_a(st));
            for (int j = threadIdx.x; j < A_ALL / 16; j += MQ_THREADS) z[j] = make_uint4(0, 0, 0, 0);
        }
        mq_fence_proxy_async();
    }
    if (warp == MQ_EPI_WARPS + MQ_PROD_WARPS) {
        // all 512 columns: four 128-column accumulators (one CTA per SM: the shared-memory footprint guarantees it)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(mq_smem(&sh.tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    mq_tc_fence_before();
    __syncthreads();
    mq_tc_fence_after();
    const unsigned tmem = sh.tmem_base;

    pdl_enter(early);   // waits for the kernel that produced the activations unless they were complete before it

    // Register budget: 80 per thread at launch (768 threads). The MMA issuer's warpgroup gives back all but 24, the
    // producers (two records in registers, scale decoding) take 104, the epilogue 88: 4 x 88 + 104 + 24 = 6 x 80. No
    // instantiation spills.
    if (warp >= MQ_EPI_WARPS + MQ_PROD_WARPS) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");
    } else if (warp >= MQ_EPI_WARPS) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 88;");
    }

    if (warp < MQ_EPI_WARPS) {
        // ===== epilogue: 16 warps, four per scheduler; warp = (TMEM lane quarter, 32-column slice) =====
        // A warp requests its 32 columns of a block, waits, scales, and goes on to the next block; the other three
        // warps of its scheduler cover the tensor-memory and shared-memory latencies, so nothing is carried in
        // registers from one block to the next.
        const int q4 = warp & 3, cs = warp >> 2;
        const int r = q4 * 32 + lane;                 // weight row inside the tile = TMEM lane
        const int c0 = cs * 32;                       // first token column of this warp
        const unsigned tlane = tmem + ((unsigned)(q4 * 32) << 16) + (unsigned)c0;
        float acc[32];
#pragma unroll
        for (int j = 0; j < 32; j++) acc[j] = 0.0f;
        bool alive = true;
        MqBias16 bias;
        bias.init(&sh.bias_word);

        // arm this warp's part of every accumulator buffer with the bias, then open the buffers for the MMA issuer
#pragma unroll
        for (int buf = 0; buf < MQ_DBUF; buf++) {
            mq_tmem_st16(tlane + (unsigned)(buf * MQ_TILE_T), bias);
            mq_tmem_st16(tlane + (unsigned)(buf * MQ_TILE_T + 16), bias);
        }
        mq_tmem_wait_st();
        mq_tc_fence_before();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
            for (int buf = 0; buf < MQ_DBUF; buf++) mq_bar_arrive(&sh.d_empty[buf]);
        }

        // Stage loop outside, the stage's eight blocks inside: 8 is a multiple of the buffer count, so the buffer of block b
        // and the parity of its barrier depend on b alone, and the tables are walked with two pointers. (Unrolling the
        // inner loop, by 8 or by the buffer count, spills at this register budget and was measured 40-60 % slower.)
        static_assert(8 % MQ_DBUF == 0, "buffer index and parity must not depend on the stage");
        constexpr int NBLK = 8 * GPB;   // accumulator buffers' worth of work per stage
        int s = 0;
        unsigned spar = 0;
        for (int it = 0; it < nst && alive; it++) {
            // the stage's scale tables: weight scales come from the producers, activation scales from a bulk copy
            if (!mq_bar_wait(&sh.a_full[s], spar) || !mq_bar_wait(&sh.b_full[s], spar)) { alive = false; break; }
            // two walking pointers per stage: the per-token tables at this warp's columns, the per-row tables at this
            // lane's row; the d_x * sum q table and the mins table (Q4_K) lie a fixed distance behind them
            const float *tok_tab = stage_dx(s) + c0, *row_tab = stage_dw(s) + r;
            constexpr int SECOND = 8 * MQ_TILE_T + MQ_TILE_N * 8;   // floats from d_x to d_x * sum q, and from d_w to the mins
            {
#pragma unroll 1
            for (int b = 0; b < NBLK; b++) {
            const int buf = b % MQ_DBUF, hb = b / MQ_DBUF, i = it * 8 + b / GPB;   // i: the 32-value block
            const unsigned tcol = tlane + (unsigned)(buf * MQ_TILE_T);
            // the row's scales first: they come from the stage's tables, not from the accumulator, and their latency
            // then lies under the wait
            const float *dxs = tok_tab, *sxs = tok_tab + SECOND;
            const float dwv = row_tab[0];
            const float dmv = HAS_MIN ? -row_tab[SECOND] : 0.0f;
            if (GPB == 1 || (b & 1)) tok_tab += MQ_TILE_T;   // activation scales are per 32-value block
            row_tab += MQ_TILE_N;
            const float cw = -MQ_BIAS_F * dwv;
            {
                if (!mq_bar_wait(&sh.d_full[buf], (unsigned)hb & 1u)) { alive = false; break; }
            }
            mq_tc_fence_after();
            // the slice in two halves of 16 columns: 16 result registers live at a time
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float sv[16];
                mq_tmem_ld16(tcol + (unsigned)(h * 16), sv);
                {
                    mq_tmem_wait_ld();
                }
                // these columns have been read: re-arm them with the bias (asynchronously)
                mq_tmem_st16(tcol + (unsigned)(h * 16), bias);
#pragma unroll
                for (int j4 = 0; j4 < 4; j4++) {
                    const float4 dx = *reinterpret_cast<const float4 *>(dxs + h * 16 + j4 * 4);
                    const float dxv[4] = { dx.x, dx.y, dx.z, dx.w };
                    float sxv[4] = { 0.f, 0.f, 0.f, 0.f };
                    if (HAS_MIN) {
                        const float4 sx = *reinterpret_cast<const float4 *>(sxs + h * 16 + j4 * 4);
                        sxv[0] = sx.x; sxv[1] = sx.y; sxv[2] = sx.z; sxv[3] = sx.w;
                    }
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float f = sv[j4 * 4 + e];
                        float v = acc[h * 16 + j4 * 4 + e];
                        // (f - 12582912) * d_w in one FMA: -12582912 * d_w is exact for every format here -- d_w is an
                        // f16 (11 significant bits), or for Q4_K the product of an f16 and a 6-bit integer (17 bits,
                        // itself exact in f32), and the constant 1.5 * 2^23 adds one bit
                        v = fmaf(fmaf(f, dwv, cw), dxv[e], v);
                        if (HAS_MIN) v = fmaf(dmv, sxv[e], v);
                        acc[h * 16 + j4 * 4 + e] = v;
                    }
                }
                if (DUMP) {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int tok = t0 + c0 + h * 16 + j, row = n0 + r;
                        if (tok < a.rows && row < w.n && i * 32 < w.k) {
                            // the reference's block dot has unsigned weight codes: add the offset times the block's
                            // activation sum; Q6_K: the block's two groups come one after the other to this thread
                            const int cexp = FMT == FMT_Q8_0 ? 128 : FMT == FMT_Q4_0 ? 8 : FMT == FMT_Q6_K ? 32 : 0;
                            const int add = cexp ? cexp * __ldg(&a.isum[(long long)tok * (a.k_pad >> 5) + i]) : 0;
                            const int dot = __float_as_int(sv[j]) - MQ_BIAS;   // Q4_0: 16 times the dot, exactly
                            int *dst = &dump[((long long)tok * w.n + row) * (w.k >> 5) + i];
                            if (GPB == 1 || (b & 1) == 0) *dst = (FMT == FMT_Q4_0 ? dot >> 4 : dot) + add;
                            else *dst += dot;
                        }
                    }
                }
            }
            // the bias stores have landed by now: hand the buffer back to the MMA issuer
            {
                mq_tmem_wait_st();
                mq_tc_fence_before();
                __syncwarp();
                if (lane == 0) mq_bar_arrive(&sh.d_empty[buf]);
            }
            }
            }
            if (!alive) break;
            __syncwarp();
            if (lane == 0) mq_bar_arrive(&sh.epi_done[s]);   // the stage's scale tables are free
            if (++s == MQ_STAGES) { s = 0; spar ^= 1u; }
        }
        if (!alive) {
            if (lane == 0) atomicExch(status, -7);
        } else {
            const int row = n0 + r;
            if (row < w.n) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int tok = t0 + c0 + j;
                    if (tok < a.rows) y[(long long)tok * y_stride + row] = ep.apply(acc[j], tok, row);
                }
            }
        }
    } else if (warp < MQ_EPI_WARPS + MQ_PROD_WARPS) {
        // ===== producers =====
        const int pw = warp - MQ_EPI_WARPS;
        const int rg0 = (n0 >> 4) + 2 * pw;
        bool alive = true;
        MqRegs<FMT> ra, rb;
        if (nst > 0) {
            mq_load<FMT>(ra, w, rg0, 0, lane);
            mq_load<FMT>(rb, w, rg0 + 1, 0, lane);
        }
        for (int it = 0; it < nst && alive; it++) {
            const int s = it % MQ_STAGES;
            const unsigned par = ((unsigned)(it / MQ_STAGES) & 1u) ^ 1u;   // first use of a stage passes at once
            {
                if (!mq_bar_wait(&sh.mma_done[s], par)) { alive = false; break; }
            }
            {
                if (!mq_bar_wait(&sh.epi_done[s], par)) { alive = false; break; }
            }
            if (pw == 0 && lane == 0) {
                // activation codes (already in core-matrix order) and scales of this stage, by bulk async copy
                mq_bar_expect_tx(&sh.b_full[s], MQ_B_BYTES + (HAS_MIN ? 2 : 1) * MQ_DX_BYTES);
                const uint8_t *src = q_tiled + ((long long)it * (a.rows_pad >> 3) + (t0 >> 3)) * 2048;
                mq_bulk_load(stage_b(s), src, MQ_B_BYTES, &sh.b_full[s]);
                for (int b = 0; b < 8; b++) {
                    const long long off = (long long)(it * 8 + b) * a.rows_pad + t0;
                    mq_bulk_load(stage_dx(s) + b * MQ_TILE_T, a.dx + off, MQ_TILE_T * 4, &sh.b_full[s]);
                    if (HAS_MIN) mq_bulk_load(stage_sx(s) + b * MQ_TILE_T, a.sx + off, MQ_TILE_T * 4, &sh.b_full[s]);
                }
            }
            uint8_t *at = stage_a(s);
            mq_store<FMT>(ra, 2 * pw, lane, at, stage_dw(s), stage_dm(s));
            mq_store<FMT>(rb, 2 * pw + 1, lane, at, stage_dw(s), stage_dm(s));
            if (it + 1 < nst) {
                // the next stage's records travel while this stage is multiplied
                mq_load<FMT>(ra, w, rg0, it + 1, lane);
                mq_load<FMT>(rb, w, rg0 + 1, it + 1, lane);
            }
            mq_fence_proxy_async();   // generic-proxy stores -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mq_bar_arrive(&sh.a_full[s]);
        }
        if (!alive && lane == 0) atomicExch(status, -7);
    } else if (warp == MQ_EPI_WARPS + MQ_PROD_WARPS) {
        // ===== MMA issuer =====
        if (lane == 0) {
            constexpr unsigned idesc = mq_idesc(FMT != FMT_Q4_K, MQ_TILE_N, MQ_TILE_T);
            bool alive = true;
            for (int it = 0; it < nst && alive; it++) {
                const int s = it % MQ_STAGES;
                const unsigned par = (unsigned)(it / MQ_STAGES) & 1u;
                {
                    if (!mq_bar_wait(&sh.a_full[s], par)) { alive = false; break; }
                }
                {
                    if (!mq_bar_wait(&sh.b_full[s], par)) { alive = false; break; }
                }
                mq_tc_fence_after();
                const unsigned a_addr = mq_smem(stage_a(s)), b_addr = mq_smem(stage_b(s));
                for (int b = 0; b < 8 * GPB; b++) {
                    const int i = it * 8 * GPB + b, buf = i % MQ_DBUF;
                    {
                        if (!mq_bar_wait(&sh.d_empty[buf], (unsigned)(i / MQ_DBUF) & 1u)) { alive = false; break; }
                    }
                    mq_tc_fence_after();
                    // block b / GPB of the stage; Q6_K: copy b % 2 of the weight rows, the same activation codes
                    mq_umma_i8(tmem + (unsigned)(buf * MQ_TILE_T), mq_desc(a_addr + (b % GPB) * MQ_A_BYTES + (b / GPB) * 256, 128, 2048),
                               mq_desc(b_addr + (b / GPB) * 256, 128, 2048), idesc);
                    mq_umma_commit(&sh.d_full[buf]);
                }
                if (alive) mq_umma_commit(&sh.mma_done[s]);
            }
            if (!alive) atomicExch(status, -7);
        }
        __syncwarp();
    }

    pdl_exit(early);
    mq_tc_fence_before();
    __syncthreads();
    if (warp == MQ_EPI_WARPS + MQ_PROD_WARPS) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

bool mmq_supports(int fmt) { return fmt == FMT_Q4_0 || fmt == FMT_Q8_0 || fmt == FMT_Q4_K || fmt == FMT_Q6_K; }

template <int FMT, bool DUMP>
static cudaError_t mmq_launch_one(const WeightView &w, const ActView &a, const uint8_t *q_tiled, float *y,
                                  long long y_stride, int *dump, int *status, int early, cudaStream_t stream, const Epilogue &ep,
                                  int tile_t0, int tile_count)
{
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = mmq_kernel<FMT, DUMP>;
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mq_smem_bytes(FMT));
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int tiles_t = (a.rows + MQ_TILE_T - 1) / MQ_TILE_T;
    if (tile_t0 < 0 || tile_t0 >= tiles_t) return cudaErrorInvalidValue;
    if (tile_count <= 0 || tile_t0 + tile_count > tiles_t) tile_count = tiles_t - tile_t0;
    const dim3 grid((w.n_pad + MQ_TILE_N - 1) / MQ_TILE_N, tile_count);
    return launch_pdl(kernel, grid, dim3(MQ_THREADS), mq_smem_bytes(FMT), stream, w, a, q_tiled, y, y_stride, dump, status, early, ep, tile_t0);
}

// a.rows_pad must be a multiple of 128 and q_tiled the core-matrix copy of the activation codes (quantize.cu).
// tile_t0 / tile_count: only the 128-token tiles [tile_t0, tile_t0 + tile_count) (0 / 0: all), for callers that want the
// rows in chunks (a sum over ranks of one chunk while the next is computed).
cudaError_t launch_mmq(const WeightView &w, const ActView &a, const uint8_t *q_tiled, float *y, long long y_stride,
                       int *dump, int *status, int early, cudaStream_t stream, const Epilogue *epilogue, int tile_t0,
                       int tile_count)
{
    if (w.n_pad == 0 || a.rows == 0) return cudaSuccess;
    const Epilogue ep = epilogue ? *epilogue : Epilogue{ nullptr, nullptr, 0 };
    if ((a.rows_pad % MQ_TILE_T) != 0 || !q_tiled) return cudaErrorInvalidValue;
#define SLC_FMT(F)                                                                                 \
    case F:                                                                                        \
        return dump ? mmq_launch_one<F, true>(w, a, q_tiled, y, y_stride, dump, status, early, stream, ep, tile_t0, tile_count)    \
                    : mmq_launch_one<F, false>(w, a, q_tiled, y, y_stride, nullptr, status, early, stream, ep, tile_t0, tile_count);
    switch (w.fmt) {
        SLC_FMT(FMT_Q4_0) SLC_FMT(FMT_Q8_0) SLC_FMT(FMT_Q4_K) SLC_FMT(FMT_Q6_K)
    default: return cudaErrorInvalidValue;
    }
#undef SLC_FMT
}

}  // namespace slc
