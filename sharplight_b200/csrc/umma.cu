// Tile kernel on the 5th-generation tensor cores for 3 rows and more: batched decode, speculative verification, prefill.
//
// Arithmetic: the reference's integer-dot MatMul (src/Sharplight.Cpu/IntDot.Kernels.cs:12-29, GPU form
// src/Sharplight.Shaders/Kernels/mmq.slang:224-233 of the Sharplight tree): per 32-value block an exact integer dot of
// weight codes and 8-bit activation codes, scaled in f32. The integers are carried as f16 values: a 4-bit code times a
// 6-bit sub-block scale (<= 945), an int8 code, an activation code (|q| <= 127) are all exact in f16, their products are
// exact in the tensor core's f32 accumulator, and a block sum stays below 2^22, so tcgen05.mma kind::f16 returns the
// same integer the int8 path would -- already as a float, and for Q4_K already multiplied by the sub-block scale.
// What is left for the CUDA cores per (row, token, block) is one multiply-add with the activation scale (two for the
// formats whose weight scale changes every block), issued as packed fma.rn.f32x2. The Q4_K offset term
// sum_b m[n,b] * (d_x * sum q)[t,b] is a small product of its own and also runs on the tensor core (kind::tf32, the
// activation factor split in two tf32 halves).
//
// Shape: weights are the M operand (128 rows per tile, swap-AB), tokens the N operand (16 to 128 per tile), one MMA
// pair per 32-value block into a tensor-memory buffer of its own. Work is cut stream-K fashion: the (tile, 256-value
// super-tile) units of the whole MatMul are dealt evenly to one persistent CTA per SM, so a 112-tile decode MatMul
// still streams through all 148 SMs; a tile whose K range is shared by several CTAs is summed by the last of them to
// arrive, in CTA order (deterministic), through a scratch area that belongs to the activation object.
//
// Roles (24 warps): warps 0 and 2 issue the MMAs (every other stage each); warps 1 and 3 are bulk-copy (TMA engine)
// loaders for weight records and for activation scale tables and code tiles; warps 4-7 expand weight codes to f16 operand tiles (128-byte swizzled rows)
// and decode scales; warps 8-23 read tensor memory, scale and accumulate. Every wait is bounded and raises the
// device status word when it runs out.
#include "internal.cuh"

#include <cuda_fp16.h>

namespace slc {

typedef unsigned long long ull;

constexpr int UM_ROWS = 128;
constexpr int UM_THREADS = 768;
constexpr int UM_EPI0 = 8;                 // first epilogue warp
constexpr int UM_A_STAGE = UM_ROWS * 128;  // one 64-value stage of the weight operand: 128 rows x 128 bytes
constexpr int UM_SMEM_LIMIT = 227 * 1024;
constexpr int UM_REG_CTRL = 24, UM_REG_PROD = 72, UM_REG_EPI = 96;   // registers per thread after the roles have split

template <int FMT, int NT>
struct UmCfg
{
    static constexpr bool MINS = FMT == FMT_Q4_K;
    static constexpr int CS = NT >= 128 ? 4 : NT == 64 ? 2 : 1;   // column slices of the token tile
    static constexpr int BP = 4 / CS;                             // epilogue groups taking blocks in turn
    static constexpr int CW = NT / CS;                            // columns per epilogue warp
    static constexpr int DB = (NT == 128 && MINS) ? 2 : 4;        // tensor-memory buffers for block dots
    static constexpr int MB = NT == 128 ? 1 : 2;                  // offset-term buffers (Q4_K)
    static constexpr int TM_MINS = DB * NT;                       // first column of the offset-term buffers
    static constexpr int TM_ACC = TM_MINS + MB * NT;              // Q4_K: running sums of the tile, one region per block turn
    static constexpr int TM_NEED = DB * NT + (MINS ? (MB + BP) * NT : 0);
    static_assert(TM_NEED <= 512, "tensor memory budget");
    static constexpr int TM_COLS = TM_NEED <= 32 ? 32 : TM_NEED <= 64 ? 64 : TM_NEED <= 128 ? 128 : TM_NEED <= 256 ? 256 : 512;
    static constexpr int REC = record_bytes(FMT);
    static constexpr int RAW_SLOT = 8 * REC;
    static constexpr int S = 3;                                   // weight-operand stages (64 K-values each)
    // activation-operand stages: these tiles come from L2 by bulk copy, and enough of them must be in flight to cover
    // that latency at the rate the tensor core consumes them
    static constexpr int SB = NT == 128 ? 5 : NT == 64 ? 6 : 8;
    static constexpr int RS = FMT == FMT_Q8_0 ? 2 : NT >= 32 ? 3 : 4;   // weight-record ring (units)
    static constexpr int B_STAGE = NT * 128;
    static constexpr int DX_BYTES = 8 * NT * 4;
    static constexpr int SX2_BYTES = MINS ? NT * 64 : 0;
    static constexpr int ACT_SLOT = (DX_BYTES + SX2_BYTES + 511) / 512 * 512;
    static constexpr int WS_TAB = MINS ? UM_ROWS * 8 : 8 * UM_ROWS * 4;  // (d, -dmin) per row, or d_w per block and row
    static constexpr int WS_A2 = MINS ? UM_ROWS * 64 : 0;                // mins as a tf32 operand tile
    static constexpr int WS_SLOT = WS_TAB + WS_A2;
    static constexpr int COMB = (BP - 1) * UM_ROWS * NT * 4;
    // offsets inside the 1024-byte aligned dynamic shared memory
    static constexpr int OFF_A = 0;
    static constexpr int OFF_B = OFF_A + S * UM_A_STAGE;
    static constexpr int OFF_WS = OFF_B + SB * B_STAGE;           // multiples of 1024 so far
    static constexpr int OFF_ACT = OFF_WS + 2 * WS_SLOT;
    static constexpr int OFF_RAW = OFF_ACT + 2 * ACT_SLOT;
    static constexpr int OFF_COMB = OFF_RAW + RS * RAW_SLOT;
    static constexpr int BYTES = OFF_COMB + COMB + 1024;          // + alignment slack
    static_assert(BYTES <= UM_SMEM_LIMIT, "shared memory budget");
    static_assert(WS_SLOT % 512 == 0 && RAW_SLOT % 16 == 0, "alignment");
};

struct UmBars
{
    uint64_t rw_full[4], rw_empty[4];
    uint64_t ua_full[2], ua_empty[2];
    uint64_t ws_full[2], ws_empty[2];
    uint64_t a_full[3], a_empty[3], b_full[8], b_empty[8];
    uint64_t d_full[4], d_empty[4];
    uint64_t m_full[2], m_empty[2];
    uint64_t comb_full, comb_free;       // block turns of a tile meeting in shared memory
    uint64_t fx_written, fx_decided;     // fix-up: partial tile written by all its warps / arrival order known
    unsigned tmem_base;
    int abort;
    int last_flag;
};

struct UmParams
{
    WeightView w;
    ActView a;
    const uint8_t *h_tiled;   // activation codes as f16, 128-byte swizzled rows: [k/64][rows_pad/8][8][128 B]
    const uint8_t *sx2;       // d_x * sum q split in two tf32 halves, 64-byte swizzled rows: [k/256][rows_pad/8][8][64 B]
    float *y;
    long long y_stride;
    int *dump;
    int *status;
    float *scratch;           // [CTAs][2][NT][128] partial tiles
    int *counters;            // [CTAs] arrivals per split tile, indexed by the tile's first contributor; zero between launches
    int row_tiles, tok_tiles, nst;
    long long units;
    Epilogue ep;
};

// ---- PTX wrappers -----------------------------------------------------------------------------------------------------

__device__ __forceinline__ void um_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void um_expect_tx(uint64_t *bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void um_bulk(void *dst, const void *src, unsigned bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Bounded wait (about two seconds); gives up early when another role has already raised the abort flag. Between probes
// the warp naps for nap_ns, so that the roles that mostly wait (loaders, MMA issuer, producers) leave the issue slots
// to the warps that have work: a tight probing loop of eight waiting warps was measured to execute more instructions
// than the arithmetic of the kernel.
__device__ __forceinline__ bool um_wait(uint64_t *bar, unsigned parity, volatile int *abort_flag, unsigned nap_ns = 100)
{
    const unsigned b = smem_u32(bar);
#pragma unroll 1
    for (unsigned i = 0; i < 20000000u; i++) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(b), "r"(parity) : "memory");
        if (ok) return true;
        __nanosleep(nap_ns);
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void um_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void um_tc_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void um_tc_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory operand descriptor, K-major, swizzled rows (layout 2: 128-byte rows, 4: 64-byte rows); groups of eight
// rows are sbo bytes apart.
__device__ __forceinline__ uint64_t um_desc(unsigned addr, unsigned sbo, unsigned layout)
{
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46) |
           ((uint64_t)layout << 61);
}
// Instruction descriptors: f32 accumulator, M = 128, K-major operands; f16 x f16 or tf32 x tf32.
__host__ __device__ constexpr unsigned um_idesc_f16(int n) { return (1u << 4) | ((unsigned)(n >> 3) << 17) | (8u << 24); }
__host__ __device__ constexpr unsigned um_idesc_tf32(int n) { return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(n >> 3) << 17) | (8u << 24); }

__device__ __forceinline__ void um_mma_f16(unsigned d, uint64_t a, uint64_t b, unsigned idesc, unsigned accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void um_mma_tf32(unsigned d, uint64_t a, uint64_t b, unsigned idesc, unsigned accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void um_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void um_ld16(unsigned taddr, unsigned (&r)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
// The same with the results typed as floats from the start (the values are used as floats: no re-typing moves).
__device__ __forceinline__ void um_ld16f(unsigned taddr, float (&r)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]),
                   "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15])
                 : "r"(taddr));
}
// The same 16 columns as eight packed pairs (column 2j in the low half): the form the packed f32x2 arithmetic consumes.
__device__ __forceinline__ void um_ld16p(unsigned taddr, ull (&p)[8])
{
    asm volatile("{\n\t.reg .b32 t<16>;\n\t"
                 "tcgen05.ld.sync.aligned.32x32b.x16.b32 {t0, t1, t2, t3, t4, t5, t6, t7, t8, t9, t10, t11, t12, t13, t14, t15}, [%8];\n\t"
                 "mov.b64 %0, {t0, t1};\n\tmov.b64 %1, {t2, t3};\n\tmov.b64 %2, {t4, t5};\n\tmov.b64 %3, {t6, t7};\n\t"
                 "mov.b64 %4, {t8, t9};\n\tmov.b64 %5, {t10, t11};\n\tmov.b64 %6, {t12, t13};\n\tmov.b64 %7, {t14, t15};\n\t}"
                 : "=l"(p[0]), "=l"(p[1]), "=l"(p[2]), "=l"(p[3]), "=l"(p[4]), "=l"(p[5]), "=l"(p[6]), "=l"(p[7])
                 : "r"(taddr));
}
// (no memory clobber on these: they touch tensor memory only, and ordinary shared-memory loads may be scheduled across them)
__device__ __forceinline__ void um_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;"); }
__device__ __forceinline__ void um_st16(unsigned taddr, const ull (&a)[8])
{
    asm volatile("{\n\t.reg .b32 r<16>;\n\t"
                 "mov.b64 {r0, r1}, %1;\n\tmov.b64 {r2, r3}, %2;\n\tmov.b64 {r4, r5}, %3;\n\tmov.b64 {r6, r7}, %4;\n\t"
                 "mov.b64 {r8, r9}, %5;\n\tmov.b64 {r10, r11}, %6;\n\tmov.b64 {r12, r13}, %7;\n\tmov.b64 {r14, r15}, %8;\n\t"
                 "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {r0, r1, r2, r3, r4, r5, r6, r7, r8, r9, r10, r11, r12, r13, r14, r15};\n\t}"
                 ::"r"(taddr), "l"(a[0]), "l"(a[1]), "l"(a[2]), "l"(a[3]), "l"(a[4]), "l"(a[5]), "l"(a[6]), "l"(a[7]) : "memory");
}
__device__ __forceinline__ void um_st16f(unsigned taddr, const float (&a)[16])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "f"(a[0]), "f"(a[1]), "f"(a[2]), "f"(a[3]), "f"(a[4]), "f"(a[5]), "f"(a[6]), "f"(a[7]),
                   "f"(a[8]), "f"(a[9]), "f"(a[10]), "f"(a[11]), "f"(a[12]), "f"(a[13]), "f"(a[14]), "f"(a[15]) : "memory");
}
__device__ __forceinline__ void um_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// shared-memory loads by 32-bit shared address
__device__ __forceinline__ float um_lds_f32(unsigned addr) { float v; asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr)); return v; }
__device__ __forceinline__ void um_lds_2xf32(unsigned addr, float &a, float &b) { asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(a), "=f"(b) : "r"(addr)); }
__device__ __forceinline__ void um_lds_2x64(unsigned addr, ull &a, ull &b) { asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "r"(addr)); }

// packed f32 pairs
__device__ __forceinline__ ull um_pk(unsigned lo, unsigned hi) { ull r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi)); return r; }
__device__ __forceinline__ ull um_pkf(float lo, float hi) { ull r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void um_unpk(ull v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ ull um_fma2(ull a, ull b, ull c) { ull d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ ull um_mul2(ull a, ull b) { ull d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ ull um_add2(ull a, ull b) { ull d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }

__device__ __forceinline__ unsigned um_prmt(unsigned a, unsigned b, unsigned sel)
{
    unsigned d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ unsigned um_hfma2(unsigned a, unsigned b, unsigned c)
{
    unsigned d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ unsigned um_hadd2(unsigned a, unsigned b)
{
    unsigned d;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ unsigned um_hmul2(unsigned a, unsigned b)
{
    unsigned d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ float um_h2f(unsigned bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

// Byte offset of 16-byte chunk c (0..7) of row r inside a tile of 128-byte swizzled rows.
__device__ __forceinline__ int um_sw128(int r, int c) { return (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4); }
// The same for 64-byte rows (chunks 0..3).
__device__ __forceinline__ int um_sw64(int r, int c) { return (r >> 3) * 512 + (r & 7) * 64 + ((c ^ ((r & 7) >> 1)) << 4); }

// Four small unsigned bytes of `bytes` -> two f16x2 registers holding 1024 + value (0x6400 | v), values (0, 1) and (2, 3).
__device__ __forceinline__ void um_bytes_to_h1024(unsigned bytes, unsigned &h01, unsigned &h23)
{
    h01 = um_prmt(bytes, 0x64646464u, 0x5140u);
    h23 = um_prmt(bytes, 0x64646464u, 0x7362u);
}

// ---- work iteration ---------------------------------------------------------------------------------------------------

struct UmWork
{
    long long u, u_end;     // this CTA's units [u, u_end)
    int tile, st;           // tile and super-tile of unit u
    int nst;
    __device__ __forceinline__ void init(const UmParams &p)
    {
        const long long g = gridDim.x, c = blockIdx.x;
        u = c * p.units / g;
        u_end = (c + 1) * p.units / g;
        nst = p.nst;
        tile = (int)(u / nst);
        st = (int)(u - (long long)tile * nst);
    }
    __device__ __forceinline__ bool done() const { return u >= u_end; }
    __device__ __forceinline__ void next()
    {
        u++;
        if (++st == nst) { st = 0; tile++; }
    }
};

// ---- producers: one row group (16 rows) of one 64-value stage -> f16 operand rows ------------------------------------------

// Q4_K: the 6-bit scales of a row's eight sub-blocks as two words of four bytes (sub-blocks 0-3, 4-7), decoded once per
// unit (src/Sharplight.Cpu/Quant.cs:504-516 of the Sharplight tree); the export build multiplies by one instead.
template <bool DUMP>
__device__ __forceinline__ void um_q4k_scale_bytes(const uint4 &h, unsigned &lo, unsigned &hi)
{
    lo = DUMP ? 0x01010101u : (h.y & 0x3F3F3F3Fu);
    hi = DUMP ? 0x01010101u : ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u));
}

// The two f16x2 constants of stage c from the packed scale bytes: (sc, sc) and (-1024 sc, -1024 sc) for sub-blocks 2c, 2c+1.
__device__ __forceinline__ void um_q4k_stage_scales(unsigned lo, unsigned hi, int c, unsigned (&sc2)[2], unsigned (&off2)[2])
{
    const unsigned pair = ((c < 2 ? lo : hi) >> (16 * (c & 1)));                  // low two bytes: sc of 2c, sc of 2c+1
    const unsigned h1024 = um_prmt(pair, 0x64646464u, 0x5140u);                   // (1024 + sc_a, 1024 + sc_b)
    const unsigned sc = um_hadd2(h1024, 0xE400E400u);                             // (sc_a, sc_b), exact
    sc2[0] = um_prmt(sc, sc, 0x1010u);
    sc2[1] = um_prmt(sc, sc, 0x3232u);
    off2[0] = um_hmul2(sc2[0], 0xE400E400u);                                      // -1024 * sc <= 64512: exact in f16
    off2[1] = um_hmul2(sc2[1], 0xE400E400u);
}

// What a producer lane keeps of a row group for the four stages of a unit.
template <int FMT>
struct UmRowGroup
{
    unsigned sc_lo[2], sc_hi[2];   // Q4_K: packed sub-block scales of rows g and g + 8
};

// One 64-value stage of one row group. a_rg: the stage's operand rows of this row group (a_stage + rgl * 2048); soff: this
// lane's byte offset of row g, chunk t (or t / 2 for Q4_0) inside it, swizzle included. A chunk further along K differs
// only in bits 4-6 of the offset, so its address is soff ^ (chunk bits << 4); row g + 8 lies 1024 bytes on.
template <int FMT>
__device__ __forceinline__ void um_expand(const uint8_t *rec, int c, int lane, uint8_t *a_rg, unsigned soff, const UmRowGroup<FMT> &rg)
{
    if constexpr (FMT == FMT_Q4_K) {
        // tile c of the record: lane (g, t) holds qs[32c + 8t .. +7] of rows g (x, y) and g + 8 (z, w); low nibbles are
        // values 8t.. of sub-block 2c (chunk t of the stage), high nibbles the same of sub-block 2c + 1 (chunk 4 + t)
        const uint4 q = reinterpret_cast<const uint4 *>(rec + c * 512)[lane];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            unsigned sc2[2], off2[2];
            um_q4k_stage_scales(rg.sc_lo[r], rg.sc_hi[r], c, sc2, off2);
            const unsigned w0 = r ? q.z : q.x, w1 = r ? q.w : q.y;
#pragma unroll
            for (int nib = 0; nib < 2; nib++) {
                const unsigned b0 = (nib ? (w0 >> 4) : w0) & 0x0F0F0F0Fu, b1 = (nib ? (w1 >> 4) : w1) & 0x0F0F0F0Fu;
                uint4 o;
                unsigned h01, h23;
                um_bytes_to_h1024(b0, h01, h23);
                o.x = um_hfma2(h01, sc2[nib], off2[nib]);     // (1024 + v) * sc - 1024 * sc = v * sc, one rounding: exact
                o.y = um_hfma2(h23, sc2[nib], off2[nib]);
                um_bytes_to_h1024(b1, h01, h23);
                o.z = um_hfma2(h01, sc2[nib], off2[nib]);
                o.w = um_hfma2(h23, sc2[nib], off2[nib]);
                *reinterpret_cast<uint4 *>(a_rg + r * 1024 + (soff ^ (unsigned)(nib << 6))) = o;
            }
        }
    } else if constexpr (FMT == FMT_Q4_0) {
        // tile c: words w0 = row g block 2c, w1 = row g+8 block 2c, w2 = row g block 2c+1, w3 = row g+8 block 2c+1, each
        // qs[4t .. 4t+3]: low nibbles are values 4t.. of the block, high nibbles values 16 + 4t..; operand value = code - 8.
        // K offset inside the stage: 32 blk + 16 nib + 4t -> chunk 4 blk + 2 nib + t / 2, half t & 1 (in soff)
        const uint4 q = reinterpret_cast<const uint4 *>(rec + c * 512)[lane];
        const unsigned wv[4] = { q.x, q.y, q.z, q.w };
#pragma unroll
        for (int j = 0; j < 4; j++) {
#pragma unroll
            for (int nib = 0; nib < 2; nib++) {
                const unsigned b = (nib ? (wv[j] >> 4) : wv[j]) & 0x0F0F0F0Fu;
                unsigned h01, h23;
                um_bytes_to_h1024(b, h01, h23);
                uint2 o;
                o.x = um_hadd2(h01, 0xE408E408u);   // (1024 + v) - 1032 = v - 8
                o.y = um_hadd2(h23, 0xE408E408u);
                *reinterpret_cast<uint2 *>(a_rg + (j & 1) * 1024 + (soff ^ (unsigned)((4 * (j >> 1) + 2 * nib) << 4))) = o;
            }
        }
    } else {  // Q8_0: tiles 2c and 2c + 1 (one block each); lane: q[8t .. 8t+7] of rows g (x, y) and g + 8 (z, w)
#pragma unroll
        for (int blk = 0; blk < 2; blk++) {
            const uint4 q = reinterpret_cast<const uint4 *>(rec + (2 * c + blk) * 512)[lane];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const unsigned w0 = (r ? q.z : q.x) ^ 0x80808080u, w1 = (r ? q.w : q.y) ^ 0x80808080u;   // code + 128
                uint4 o;
                unsigned h01, h23;
                um_bytes_to_h1024(w0, h01, h23);
                o.x = um_hadd2(h01, 0xE480E480u);   // (1024 + code + 128) - 1152 = code
                o.y = um_hadd2(h23, 0xE480E480u);
                um_bytes_to_h1024(w1, h01, h23);
                o.z = um_hadd2(h01, 0xE480E480u);
                o.w = um_hadd2(h23, 0xE480E480u);
                *reinterpret_cast<uint4 *>(a_rg + r * 1024 + (soff ^ (unsigned)(blk << 6))) = o;
            }
        }
    }
}

// The per-unit tables of one row group: weight scales for the epilogue and (Q4_K) the mins as a tf32 operand tile.
template <int FMT>
__device__ __forceinline__ void um_tables(const uint8_t *rec, int rgl, int lane, uint8_t *ws_slot)
{
    const int g = lane >> 2, t = lane & 3;
    const uint4 *hdr = reinterpret_cast<const uint4 *>(rec + code_bytes(FMT));
    using Cfg = UmCfg<FMT, 128>;
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const uint4 h = hdr[g + 8 * r];
        const int row = rgl * 16 + g + 8 * r;
        if constexpr (FMT == FMT_Q4_K) {
            if (t == 0) reinterpret_cast<float2 *>(ws_slot)[row] = make_float2(um_h2f(h.x & 0xffffu), -um_h2f(h.x >> 16));
            // mins of sub-blocks 2t, 2t + 1 as floats (exact tf32 values) at K positions 2t, 2t+1 and again at 8 + 2t, 8 + 2t+1
            const unsigned mnw = t < 2 ? (h.z & 0x3F3F3F3Fu) : (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u));
            const int sh = 16 * (t & 1);
            const float2 mn = make_float2((float)((mnw >> sh) & 0xffu), (float)((mnw >> (sh + 8)) & 0xffu));
            uint8_t *a2 = ws_slot + Cfg::WS_TAB;
            *reinterpret_cast<float2 *>(a2 + um_sw64(row, t >> 1) + 8 * (t & 1)) = mn;
            *reinterpret_cast<float2 *>(a2 + um_sw64(row, 2 + (t >> 1)) + 8 * (t & 1)) = mn;
        } else {
            // f16 scale of blocks 2t and 2t + 1
            const unsigned wsc = t == 0 ? h.x : t == 1 ? h.y : t == 2 ? h.z : h.w;
            float *dw = reinterpret_cast<float *>(ws_slot);
            dw[(2 * t) * UM_ROWS + row] = um_h2f(wsc & 0xffffu);
            dw[(2 * t + 1) * UM_ROWS + row] = um_h2f(wsc >> 16);
        }
    }
}

// ---- the kernel ------------------------------------------------------------------------------------------------------

template <int FMT, int NT, bool DUMP>
__global__ void __launch_bounds__(UM_THREADS, 1) umma_kernel(const UmParams p)
{
    using Cfg = UmCfg<FMT, NT>;
    constexpr bool MINS = Cfg::MINS;
    constexpr int CS = Cfg::CS, BP = Cfg::BP, CW = Cfg::CW, DB = Cfg::DB, S = Cfg::S, SB = Cfg::SB, RS = Cfg::RS;
    extern __shared__ __align__(1024) unsigned char um_smem_raw[];
    __shared__ UmBars sh;
    unsigned char *smem = um_smem_raw + ((1024 - (smem_u32(um_smem_raw) & 1023)) & 1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *abort_flag = &sh.abort;

    if (threadIdx.x == 0) {
        for (int i = 0; i < RS; i++) { mbar_init(&sh.rw_full[i], 1); mbar_init(&sh.rw_empty[i], 4); }
        for (int i = 0; i < 2; i++) {
            mbar_init(&sh.ua_full[i], 1); mbar_init(&sh.ua_empty[i], 16);
            mbar_init(&sh.ws_full[i], 4); mbar_init(&sh.ws_empty[i], 16);
            mbar_init(&sh.m_full[i], 1); mbar_init(&sh.m_empty[i], 4 * CS);
        }
        // (with two block-dot buffers both MMA issuers read every stage and both release it)
        for (int i = 0; i < S; i++) { mbar_init(&sh.a_full[i], 4); mbar_init(&sh.a_empty[i], DB == 2 ? 2 : 1); }
        for (int i = 0; i < SB; i++) { mbar_init(&sh.b_full[i], 1); mbar_init(&sh.b_empty[i], DB == 2 ? 2 : 1); }
        for (int i = 0; i < DB; i++) { mbar_init(&sh.d_full[i], 1); mbar_init(&sh.d_empty[i], 4 * CS); }
        mbar_init(&sh.comb_full, BP > 1 ? 16 - 4 * CS : 1);
        mbar_init(&sh.comb_free, 4 * CS);
        mbar_init(&sh.fx_written, 4 * CS);
        mbar_init(&sh.fx_decided, 1);
        sh.abort = 0;
        sh.last_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)), "r"((unsigned)Cfg::TM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    um_tc_before();
    __syncthreads();
    um_tc_after();
    const unsigned tmem = sh.tmem_base;

    // Register budget. The CTA's pool is what it was launched with, 6 warpgroups x 80 registers per thread; setmaxnreg only
    // moves registers inside that pool, and an increase blocks until enough have been released -- for ever, if the
    // requests add up to more than the pool. Control 24 + producers 72 + 4 x epilogue 96 = 480 = 6 x 80.
    static_assert(UM_REG_CTRL + UM_REG_PROD + 4 * UM_REG_EPI <= 6 * 80, "setmaxnreg requests exceed the CTA's register pool");
    UmWork wk;
    const int rg_count = p.w.n_pad >> 4;
    const int tok_groups = p.a.rows_pad >> 3;

    if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(UM_REG_CTRL));
    if (warp == 1) {
        wk.init(p);
        // ===== weight-record loader: the raw records of a unit (8 row groups x 256 K-values), one bulk copy each. Weights
        // depend on no earlier kernel, so this role does not wait for the predecessor on the stream.
        pdl_launch_dependents();
        if (lane == 0) {
            int slot = 0;
            unsigned phase = 1;   // parity to wait on for "slot is free" (passes at once on a fresh barrier)
            for (; !wk.done(); wk.next()) {
                if (!um_wait(&sh.rw_empty[slot], phase, abort_flag, 1000)) break;
                const int row_tile = wk.tile / p.tok_tiles;
                const int rg0 = row_tile * 8;
                const int live = rg_count - rg0 < 8 ? rg_count - rg0 : 8;
                um_expect_tx(&sh.rw_full[slot], (unsigned)(live * Cfg::REC));
                unsigned char *dst = smem + Cfg::OFF_RAW + slot * Cfg::RAW_SLOT;
                for (int r = 0; r < live; r++) um_bulk(dst + r * Cfg::REC, p.w.record(rg0 + r, wk.st), Cfg::REC, &sh.rw_full[slot]);
                if (++slot == RS) { slot = 0; phase ^= 1u; }
            }
        }
    } else {
        pdl_enter(0);   // everything else touches activations or writes results: wait for the preceding kernel
        wk.init(p);
        if (warp == 0 || warp == 2) {
            // ===== MMA issuers: two threads (warps 0 and 2). Issuing a tcgen05 instruction, committing and probing a barrier
            // each cost the issuing thread some tens of cycles, a dozen such steps per stage; one thread alone was the
            // slowest stage of the pipeline. Every block-dot buffer must have ONE issuer: a parity wait tells "free again"
            // from "not yet used" only for a thread that is at most one use ahead of the barrier. With four buffers the
            // threads take every other 64-value stage (even stages use buffers 0-1, odd ones 2-3); with two buffers both
            // threads visit every stage and each issues the block of its own buffer. The issuers need only the number of
            // units, not which tiles they belong to.
            if (lane == 0) {
                constexpr unsigned idesc = um_idesc_f16(NT), idesc_m = um_idesc_tf32(NT);
                const unsigned a_lo0 = (smem_u32(smem + Cfg::OFF_A) >> 4) & 0x3FFFu, b_lo0 = (smem_u32(smem + Cfg::OFF_B) >> 4) & 0x3FFFu;
                const unsigned desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);          // bits 32..63: sbo 1024, version, 128-byte swizzle
                const unsigned desc_hi_m = (512u >> 4) | (1u << 14) | (4u << 29);         // sbo 512, version, 64-byte swizzle
                auto mk = [](unsigned lo14, unsigned hi) { return (uint64_t)(lo14 | (1u << 16)) | ((uint64_t)hi << 32); };
                const int n_stages = (int)(wk.u_end - wk.u) * 4;
                const int me = warp >> 1;                         // 0 or 1
                constexpr bool BY_BLOCK = DB == 2;
                constexpr int STEP = BY_BLOCK ? 1 : 2;
                // ring positions of this issuer's first stage, advanced by STEP stages per iteration
                int stage = BY_BLOCK ? 0 : me % S, stage_b = BY_BLOCK ? 0 : me % SB;
                unsigned a_phase = 0, b_phase = 0;
                bool ok = true;
#pragma unroll 1
                for (int k = BY_BLOCK ? 0 : me; k < n_stages && ok; k += STEP) {
                    const int unit = k >> 2, c = k & 3;
                    if (!um_wait(&sh.a_full[stage], a_phase, abort_flag, 100) || !um_wait(&sh.b_full[stage_b], b_phase, abort_flag, 100)) { ok = false; break; }
                    um_tc_after();
                    const unsigned a_lo = a_lo0 + (unsigned)(stage * (UM_A_STAGE >> 4)), b_lo = b_lo0 + (unsigned)(stage_b * (Cfg::B_STAGE >> 4));
#pragma unroll
                    for (int bb = 0; bb < 2; bb++) {
                        if (BY_BLOCK && bb != me) continue;
                        const int b = 2 * c + bb, buf = b % DB;
                        const unsigned dphase = ((unsigned)((unit * 8 + b) / DB) & 1u) ^ 1u;
                        if (!um_wait(&sh.d_empty[buf], dphase, abort_flag, 100)) { ok = false; break; }
                        um_tc_after();
                        const unsigned d = tmem + (unsigned)(buf * NT);
                        // K values 32 bb .. +15, then +16 .. +31: 32 bytes = 2 sixteen-byte units further along the swizzled row
                        um_mma_f16(d, mk(a_lo + 4 * bb, desc_hi), mk(b_lo + 4 * bb, desc_hi), idesc, 0);
                        um_mma_f16(d, mk(a_lo + 4 * bb + 2, desc_hi), mk(b_lo + 4 * bb + 2, desc_hi), idesc, 1);
                        um_commit(&sh.d_full[buf]);
                    }
                    if (!ok) break;
                    um_commit(&sh.a_empty[stage]);
                    um_commit(&sh.b_empty[stage_b]);
                    stage += STEP; if (stage >= S) { stage -= S; a_phase ^= 1u; }
                    stage_b += STEP; if (stage_b >= SB) { stage_b -= SB; b_phase ^= 1u; }
                    if (MINS && c == 3 && me == 1) {
                        // offset term of the unit (issued by the thread that has the unit's last stage):
                        // D2[n][t] = sum_b m[n,b] * (sx_hi + sx_lo)[t,b], two K = 8 steps
                        const int us = unit & 1, mb = unit % Cfg::MB;
                        const unsigned uphase = (unsigned)(unit >> 1) & 1u;
                        if (!um_wait(&sh.ws_full[us], uphase, abort_flag, 100) || !um_wait(&sh.ua_full[us], uphase, abort_flag, 100) ||
                            !um_wait(&sh.m_empty[mb], ((unsigned)(unit / Cfg::MB) & 1u) ^ 1u, abort_flag, 100)) { ok = false; break; }
                        um_tc_after();
                        const unsigned a2 = (smem_u32(smem + Cfg::OFF_WS + us * Cfg::WS_SLOT + Cfg::WS_TAB) >> 4) & 0x3FFFu;
                        const unsigned b2 = (smem_u32(smem + Cfg::OFF_ACT + us * Cfg::ACT_SLOT + Cfg::DX_BYTES) >> 4) & 0x3FFFu;
                        const unsigned d2 = tmem + (unsigned)(Cfg::TM_MINS + mb * NT);
                        um_mma_tf32(d2, mk(a2, desc_hi_m), mk(b2, desc_hi_m), idesc_m, 0);
                        um_mma_tf32(d2, mk(a2 + 2, desc_hi_m), mk(b2 + 2, desc_hi_m), idesc_m, 1);
                        um_commit(&sh.m_full[mb]);
                    }
                }
                if (!ok) atomicExch(p.status, -7);
            }
            __syncwarp();
        } else if (warp == 3) {
            // ===== activation-side loader: per unit the scale tables (d_x per block and token, and for Q4_K the split
            // d_x * sum q tile), then one bulk copy of the code tile per 64-value stage
            if (lane == 0) {
                int stage = 0, unit = 0;
                unsigned phase = 1;
                bool ok = true;
                for (; !wk.done() && ok; wk.next(), unit++) {
                    const int us = unit & 1;
                    const int t0 = (wk.tile % p.tok_tiles) * NT;
                    if (!um_wait(&sh.ua_empty[us], ((unsigned)(unit >> 1) & 1u) ^ 1u, abort_flag, 500)) break;
                    unsigned char *dst = smem + Cfg::OFF_ACT + us * Cfg::ACT_SLOT;
                    um_expect_tx(&sh.ua_full[us], (unsigned)(Cfg::DX_BYTES + Cfg::SX2_BYTES));
                    for (int b = 0; b < 8; b++) {
                        um_bulk(dst + b * NT * 4, p.a.dx + (long long)(wk.st * 8 + b) * p.a.rows_pad + t0, NT * 4, &sh.ua_full[us]);
                    }
                    if (MINS) um_bulk(dst + Cfg::DX_BYTES, p.sx2 + ((long long)wk.st * tok_groups + (t0 >> 3)) * 512, Cfg::SX2_BYTES, &sh.ua_full[us]);
                    for (int c = 0; c < 4; c++) {
                        if (!um_wait(&sh.b_empty[stage], phase, abort_flag, 500)) { ok = false; break; }
                        um_expect_tx(&sh.b_full[stage], (unsigned)Cfg::B_STAGE);
                        um_bulk(smem + Cfg::OFF_B + stage * Cfg::B_STAGE,
                                p.h_tiled + ((long long)(wk.st * 4 + c) * tok_groups + (t0 >> 3)) * 1024, Cfg::B_STAGE, &sh.b_full[stage]);
                        if (++stage == SB) { stage = 0; phase ^= 1u; }
                    }
                }
            }
        } else if (warp < UM_EPI0) {
            // ===== producers: weight codes -> f16 operand rows, scale tables
            asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(UM_REG_PROD));
            const int pw = warp - 4;
            const int pg = lane >> 2, pt = lane & 3;
            // this lane's byte offset of (row g, its first chunk) inside a row group's operand rows, swizzle included
            const unsigned soff = FMT == FMT_Q4_0 ? (unsigned)(pg * 128 + ((((pt >> 1) ^ pg) & 7) << 4) + 8 * (pt & 1))
                                                  : (unsigned)(pg * 128 + (((pt ^ pg) & 7) << 4));
            int slot = 0, stage = 0, unit = 0;
            unsigned rphase = 0, ab_phase = 1;
            bool ok = true;
            for (; !wk.done() && ok; wk.next(), unit++) {
                const int us = unit & 1;
                if (!um_wait(&sh.rw_full[slot], rphase, abort_flag, 300) ||
                    !um_wait(&sh.ws_empty[us], ((unsigned)(unit >> 1) & 1u) ^ 1u, abort_flag, 300)) { ok = false; break; }
                const uint8_t *raw = smem + Cfg::OFF_RAW + slot * Cfg::RAW_SLOT;
                const int rg0 = (wk.tile / p.tok_tiles) * 8;
                const bool live0 = rg0 + 2 * pw < rg_count, live1 = rg0 + 2 * pw + 1 < rg_count;
                const uint8_t *rec0 = raw + (2 * pw) * Cfg::REC, *rec1 = rec0 + Cfg::REC;
                uint8_t *ws_slot = smem + Cfg::OFF_WS + us * Cfg::WS_SLOT;
                if (live0) um_tables<FMT>(rec0, 2 * pw, lane, ws_slot);
                if (live1) um_tables<FMT>(rec1, 2 * pw + 1, lane, ws_slot);
                um_fence_async();
                __syncwarp();
                if (lane == 0) um_arrive(&sh.ws_full[us]);
                UmRowGroup<FMT> rga, rgb;
                if constexpr (FMT == FMT_Q4_K) {
                    const uint4 *h0 = reinterpret_cast<const uint4 *>(rec0 + code_bytes(FMT)), *h1 = reinterpret_cast<const uint4 *>(rec1 + code_bytes(FMT));
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        um_q4k_scale_bytes<DUMP>(h0[pg + 8 * r], rga.sc_lo[r], rga.sc_hi[r]);
                        um_q4k_scale_bytes<DUMP>(h1[pg + 8 * r], rgb.sc_lo[r], rgb.sc_hi[r]);
                    }
                }
#pragma unroll 1
                for (int c = 0; c < 4; c++) {
                    if (!um_wait(&sh.a_empty[stage], ab_phase, abort_flag, 300)) { ok = false; break; }
                    uint8_t *a_stage = smem + Cfg::OFF_A + stage * UM_A_STAGE + (2 * pw) * 2048;
                    if (live0) um_expand<FMT>(rec0, c, lane, a_stage, soff, rga);
                    if (live1) um_expand<FMT>(rec1, c, lane, a_stage + 2048, soff, rgb);
                    um_fence_async();   // generic-proxy stores -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) um_arrive(&sh.a_full[stage]);
                    if (++stage == S) { stage = 0; ab_phase ^= 1u; }
                }
                __syncwarp();
                if (lane == 0 && ok) um_arrive(&sh.rw_empty[slot]);
                if (++slot == RS) { slot = 0; rphase ^= 1u; }
            }
            if (!ok && lane == 0) atomicExch(p.status, -7);
        } else {
            // ===== epilogue: warp = (TMEM lane quarter q, column slice cs, block turn bp)
            asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(UM_REG_EPI));
            const int e = warp - UM_EPI0;
            const int q = e & 3, cs = (e >> 2) % CS, bp = (e >> 2) / CS;
            const int r = q * 32 + lane;                       // weight row inside the tile = TMEM lane
            const int c0 = cs * CW;
            const unsigned tlane = tmem + ((unsigned)(q * 32) << 16) + (unsigned)c0;
            const unsigned smem_s = smem_u32(smem);
            // Running sums of the tile. Q4_K keeps them in tensor memory (one region per block turn), touched once per
            // super-block, so that the registers hold only the super-block's partial sums; the formats with per-block
            // weight scales accumulate in registers.
            constexpr int NACC = MINS ? 1 : CW / 2;
            ull acc[NACC], accsb[MINS ? CW / 2 : 1];
#pragma unroll
            for (int j = 0; j < NACC; j++) acc[j] = 0ull;
            const unsigned tacc = tlane + (unsigned)(Cfg::TM_ACC + bp * NT);
            bool ok = true, seg_fresh = true;                  // seg_fresh: nothing accumulated yet for the running tile
            int unit = 0, n_comb = 0, n_fix = 0;               // tile ends / fix-ups so far (barrier phases)
            const long long u_first = wk.u;
            int seg_st0 = wk.st;                               // first super-tile of the running tile's segment
#pragma unroll 1
            for (; !wk.done() && ok; wk.next(), unit++) {
                const int us = unit & 1;
                const unsigned uphase = (unsigned)(unit >> 1) & 1u;
                if (!um_wait(&sh.ua_full[us], uphase, abort_flag) || !um_wait(&sh.ws_full[us], uphase, abort_flag)) { ok = false; break; }
                const unsigned ws_s = smem_s + (unsigned)(Cfg::OFF_WS + us * Cfg::WS_SLOT);
                // The unit's blocks of this warp as a stream of 16-column chunks, software-pipelined: the tensor-memory load
                // of the next chunk is in flight while the current one is scaled and accumulated, and a block's buffer goes
                // back to the MMA issuer as soon as its last chunk has arrived in registers. The loop over blocks is a real
                // loop (the code of all roles has to stay resident in the instruction cache).
                constexpr int HPB = CW / 16, NBLK = 8 / BP;
                const ulonglong2 *dx_tab = reinterpret_cast<const ulonglong2 *>(smem + Cfg::OFF_ACT + us * Cfg::ACT_SLOT) + c0 / 4;
                if constexpr (MINS) {
#pragma unroll
                    for (int j = 0; j < CW / 2; j++) accsb[j] = 0ull;
                }
#pragma unroll 1
                for (int bi = 0; bi < NBLK; bi++) {
                    const int b = bi * BP + bp, buf = b % DB;
                    if (!um_wait(&sh.d_full[buf], (unsigned)((unit * 8 + b) / DB) & 1u, abort_flag, 20)) { ok = false; break; }
                    um_tc_after();
                    const float dw = MINS ? 0.0f : um_lds_f32(ws_s + (unsigned)((b * UM_ROWS + r) * 4));
#pragma unroll
                    for (int h = 0; h < HPB; h++) {
                        unsigned v[16];
                        um_ld16(tlane + (unsigned)(buf * NT + h * 16), v);
                        um_wait_ld();
                        if (h == HPB - 1) {
                            // every chunk of the block is in registers: the buffer goes back to the MMA issuer
                            um_tc_before();
                            __syncwarp();
                            if (lane == 0) um_arrive(&sh.d_empty[buf]);
                        }
                        if (DUMP) {
                            const int n0 = (wk.tile / p.tok_tiles) * UM_ROWS, t0 = (wk.tile % p.tok_tiles) * NT;
#pragma unroll
                            for (int j = 0; j < 16; j++) {
                                const int tok = t0 + c0 + h * 16 + j, row = n0 + r, blk = wk.st * 8 + b;
                                if (tok < p.a.rows && row < p.w.n && blk * 32 < p.w.k) {
                                    const int cexp = FMT == FMT_Q8_0 ? 128 : FMT == FMT_Q4_0 ? 8 : 0;
                                    const int add = cexp ? cexp * __ldg(&p.a.isum[(long long)tok * (p.a.k_pad >> 5) + blk]) : 0;
                                    p.dump[((long long)tok * p.w.n + row) * (p.w.k >> 5) + blk] = (int)__uint_as_float(v[j]) + add;
                                }
                            }
                        }
#pragma unroll
                        for (int j4 = 0; j4 < 4; j4++) {
                            const ulonglong2 dx = dx_tab[(b * NT + h * 16) / 4 + j4];
                            const int o = h * 8 + j4 * 2;
                            if constexpr (MINS) {
                                // the MMA already applied the integer sub-block scale: one multiply-add with d_x
                                accsb[o] = um_fma2(um_pk(v[4 * j4], v[4 * j4 + 1]), dx.x, accsb[o]);
                                accsb[o + 1] = um_fma2(um_pk(v[4 * j4 + 2], v[4 * j4 + 3]), dx.y, accsb[o + 1]);
                            } else {
                                // d_w first, as two scalar multiplies whose results form a pair, then the packed multiply-add
                                const ull t01 = um_pkf(__uint_as_float(v[4 * j4]) * dw, __uint_as_float(v[4 * j4 + 1]) * dw);
                                const ull t23 = um_pkf(__uint_as_float(v[4 * j4 + 2]) * dw, __uint_as_float(v[4 * j4 + 3]) * dw);
                                acc[o] = um_fma2(t01, dx.x, acc[o]);
                                acc[o + 1] = um_fma2(t23, dx.y, acc[o + 1]);
                            }
                        }
                    }
                }
                if (!ok) break;
                if constexpr (MINS) {
                    // the unit's super-block: acc += d * sum_b(...) - dmin * D2, acc living in tensor memory
                    float d_w, nd_min;
                    um_lds_2xf32(ws_s + (unsigned)(r * 8), d_w, nd_min);
                    const ull d2 = um_pkf(d_w, d_w), nm2 = um_pkf(nd_min, nd_min);
                    // every epilogue warp waits for the offset-term MMAs: once they are done the unit's operand tiles
                    // (mins, split sums) are no longer read and the slots may be refilled
                    const int mb = unit % Cfg::MB;
                    if (!um_wait(&sh.m_full[mb], (unsigned)(unit / Cfg::MB) & 1u, abort_flag)) { ok = false; break; }
                    um_tc_after();
#pragma unroll
                    for (int h = 0; h < CW / 16; h++) {
                        ull a[8], v[8];
                        if (seg_fresh) {
#pragma unroll
                            for (int j = 0; j < 8; j++) a[j] = um_mul2(accsb[h * 8 + j], d2);
                        } else {
                            um_ld16p(tacc + (unsigned)(h * 16), v);
                            um_wait_ld();
#pragma unroll
                            for (int j = 0; j < 8; j++) a[j] = um_fma2(accsb[h * 8 + j], d2, v[j]);
                        }
                        if (bp == 0) {
                            um_ld16p(tlane + (unsigned)(Cfg::TM_MINS + mb * NT + h * 16), v);
                            um_wait_ld();
#pragma unroll
                            for (int j = 0; j < 8; j++) a[j] = um_fma2(v[j], nm2, a[j]);
                        }
                        um_st16(tacc + (unsigned)(h * 16), a);
                    }
                    um_wait_st();
                    seg_fresh = false;
                    if (bp == 0) {
                        um_tc_before();
                        __syncwarp();
                        if (lane == 0) um_arrive(&sh.m_empty[mb]);
                    }
                }
                __syncwarp();
                if (lane == 0) { um_arrive(&sh.ua_empty[us]); um_arrive(&sh.ws_empty[us]); }

                // ---- end of this CTA's segment of the tile: store, or hand the partial tile to the fix-up
                const bool tile_ends = wk.st == p.nst - 1, range_ends = wk.u + 1 == wk.u_end;
                if (!(tile_ends || range_ends)) continue;
                const int n0 = (wk.tile / p.tok_tiles) * UM_ROWS, t0 = (wk.tile % p.tok_tiles) * NT;
                const int row = n0 + r;
                const bool whole = seg_st0 == 0 && tile_ends;
                float *comb = reinterpret_cast<float *>(smem + Cfg::OFF_COMB);
                // 16 columns of this thread's running sums
                auto chunk = [&](int h, float (&a)[16]) {
                    if constexpr (MINS) {
                        um_ld16f(tacc + (unsigned)(h * 16), a);
                        um_wait_ld();
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; j++) { um_unpk(acc[h * 8 + j], a[2 * j], a[2 * j + 1]); acc[h * 8 + j] = 0ull; }
                    }
                };
                auto store_y = [&](int h, const float (&a)[16]) {
                    if (row < p.w.n) {
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const int tok = t0 + c0 + h * 16 + j;
                            if (tok < p.a.rows) p.y[(long long)tok * p.y_stride + row] = p.ep.apply(a[j], tok, row);
                        }
                    }
                };
                if (BP > 1 && bp > 0) {
                    // the block turns of a row meet in shared memory (bounded mbarrier waits, no named barrier)
                    if (!um_wait(&sh.comb_free, ((unsigned)n_comb & 1u) ^ 1u, abort_flag)) { ok = false; break; }
#pragma unroll
                    for (int h = 0; h < CW / 16; h++) {
                        float a[16];
                        chunk(h, a);
#pragma unroll
                        for (int j = 0; j < 16; j++) comb[((bp - 1) * NT + c0 + h * 16 + j) * UM_ROWS + r] = a[j];
                    }
                    __syncwarp();
                    if (lane == 0) um_arrive(&sh.comb_full);
                } else {
                    if (BP > 1 && !um_wait(&sh.comb_full, (unsigned)n_comb & 1u, abort_flag)) { ok = false; break; }
                    // This CTA may hold only part of the tile's K range. Its partial tile then goes to the scratch
                    // area; the CTA that arrives last adds the parts in CTA order and stores.
                    const long long g = gridDim.x;
                    const int my_slot = (u_first / p.nst == wk.tile) ? 0 : 1;   // slot 0: the tile this CTA's range starts in
                    float *mine = p.scratch + ((long long)blockIdx.x * 2 + my_slot) * NT * UM_ROWS;
#pragma unroll
                    for (int h = 0; h < CW / 16; h++) {
                        float a[16];
                        chunk(h, a);
                        if (BP > 1) {
#pragma unroll
                            for (int t = 1; t < BP; t++) {
#pragma unroll
                                for (int j = 0; j < 16; j++) a[j] += comb[((t - 1) * NT + c0 + h * 16 + j) * UM_ROWS + r];
                            }
                        }
                        if (whole) store_y(h, a);
                        else {
#pragma unroll
                            for (int j = 0; j < 16; j++) __stcg(&mine[(c0 + h * 16 + j) * UM_ROWS + r], a[j]);
                        }
                    }
                    if (BP > 1) {
                        __syncwarp();
                        if (lane == 0) um_arrive(&sh.comb_free);   // the buffer may be written again
                    }
                    if (!whole) {
                        const long long tile_u0 = (long long)wk.tile * p.nst, tile_u1 = tile_u0 + p.nst - 1;
                        const int c_first = (int)(((tile_u0 + 1) * g - 1) / p.units), c_last = (int)(((tile_u1 + 1) * g - 1) / p.units);
                        __threadfence();
                        __syncwarp();
                        if (lane == 0) um_arrive(&sh.fx_written);
                        if (e == 0) {
                            // every warp of the tile has written and fenced its part: count this CTA in
                            if (!um_wait(&sh.fx_written, (unsigned)n_fix & 1u, abort_flag)) { ok = false; break; }
                            if (lane == 0) {
                                const int arrived = atomicAdd(&p.counters[c_first], 1);
                                const int last = arrived == c_last - c_first;
                                if (last) p.counters[c_first] = 0;   // ready for the next launch
                                sh.last_flag = last;
                                um_arrive(&sh.fx_decided);
                            }
                        }
                        // (a warp reads the flag of this round before it can arrive for the next one, and the flag is
                        // rewritten only after all warps have arrived for that next round)
                        if (!um_wait(&sh.fx_decided, (unsigned)n_fix & 1u, abort_flag)) { ok = false; break; }
                        n_fix++;
                        if (*reinterpret_cast<volatile int *>(&sh.last_flag)) {
                            __threadfence();
#pragma unroll 1
                            for (int h = 0; h < CW / 16; h++) {
                                float sum[16];
#pragma unroll 1
                                for (int c = c_first; c <= c_last; c++) {
                                    const long long cu0 = (long long)c * p.units / g;
                                    const int slot_c = (cu0 / p.nst == wk.tile) ? 0 : 1;
                                    const float *part = p.scratch + ((long long)c * 2 + slot_c) * NT * UM_ROWS;
#pragma unroll
                                    for (int j = 0; j < 16; j++) {
                                        const float v = __ldcg(&part[(c0 + h * 16 + j) * UM_ROWS + r]);
                                        sum[j] = c == c_first ? v : sum[j] + v;
                                    }
                                }
                                store_y(h, sum);
                            }
                        }
                    }
                }
                n_comb++;
                seg_fresh = true;
                seg_st0 = 0;   // the next tile, if any, starts at its first super-tile
            }
            if (!ok && lane == 0) atomicExch(p.status, -7);
        }
    }

    um_tc_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((unsigned)Cfg::TM_COLS) : "memory");
    }
}

// ---- host side --------------------------------------------------------------------------------------------------------

bool umma_supports(int fmt) { return fmt == FMT_Q4_K || fmt == FMT_Q4_0 || fmt == FMT_Q8_0; }

int umma_token_tile(int rows) { return rows <= 16 ? 16 : rows <= 32 ? 32 : rows <= 64 ? 64 : 128; }

size_t umma_scratch_bytes(int max_ctas, int rows_pad)
{
    const int nt = rows_pad < 128 ? rows_pad : 128;
    return (size_t)max_ctas * 2 * nt * UM_ROWS * sizeof(float);
}

template <int FMT, int NT, bool DUMP>
static cudaError_t um_launch(const UmParams &p, int ctas, cudaStream_t stream)
{
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = umma_kernel<FMT, NT, DUMP>;
    constexpr int bytes = UmCfg<FMT, NT>::BYTES;
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    return launch_pdl(kernel, dim3(ctas), dim3(UM_THREADS), bytes, stream, p);
}

template <int FMT, bool DUMP>
static cudaError_t um_launch_nt(const UmParams &p, int nt, int ctas, cudaStream_t stream)
{
    switch (nt) {
    case 16: return um_launch<FMT, 16, DUMP>(p, ctas, stream);
    case 32: return um_launch<FMT, 32, DUMP>(p, ctas, stream);
    case 64: return um_launch<FMT, 64, DUMP>(p, ctas, stream);
    case 128: return um_launch<FMT, 128, DUMP>(p, ctas, stream);
    default: return cudaErrorInvalidValue;
    }
}

// a.rows_pad must be a multiple of the token tile (16, 32, 64, or 128 for more than 64 rows); h_tiled / sx2 are the
// tiled planes the quantizer wrote for these rows; scratch / counters belong to the activation object (umma_scratch_bytes
// for max_ctas CTAs; counters: max_ctas ints, zero).
cudaError_t launch_umma(const WeightView &w, const ActView &a, const uint8_t *h_tiled, const uint8_t *sx2, float *y,
                        long long y_stride, int *dump, int *status, float *scratch, int *counters, int max_ctas,
                        cudaStream_t stream, const Epilogue *epilogue)
{
    if (w.n_pad == 0 || a.rows == 0) return cudaSuccess;
    const int nt = umma_token_tile(a.rows);
    if (!h_tiled || !sx2 || !scratch || !counters || (a.rows_pad % nt) != 0 || max_ctas < 1) return cudaErrorInvalidValue;
    UmParams p;
    p.w = w; p.a = a; p.h_tiled = h_tiled; p.sx2 = sx2; p.y = y; p.y_stride = y_stride; p.dump = dump; p.status = status;
    p.scratch = scratch; p.counters = counters;
    p.row_tiles = (w.n_pad + UM_ROWS - 1) / UM_ROWS;
    p.tok_tiles = (a.rows + nt - 1) / nt;
    p.nst = w.k_pad >> 8;
    p.units = (long long)p.row_tiles * p.tok_tiles * p.nst;
    p.ep = epilogue ? *epilogue : Epilogue{ nullptr, nullptr, 0 };
    const int ctas = p.units < max_ctas ? (int)p.units : max_ctas;
#define SLC_FMT(F)                                                                   \
    case F: return dump ? um_launch_nt<F, true>(p, nt, ctas, stream) : um_launch_nt<F, false>(p, nt, ctas, stream);
    switch (w.fmt) {
        SLC_FMT(FMT_Q4_K) SLC_FMT(FMT_Q4_0) SLC_FMT(FMT_Q8_0)
    default: return cudaErrorInvalidValue;
    }
#undef SLC_FMT
}

}  // namespace slc
