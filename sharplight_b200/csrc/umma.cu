// Tile kernel on the 5th-generation tensor cores for 3 rows and more: batched decode, speculative verification, prefill.
//
// Arithmetic: the reference's integer-dot MatMul (src/Sharplight.Cpu/IntDot.Kernels.cs:12-29, GPU form
// src/Sharplight.Shaders/Kernels/mmq.slang:224-233 of the Sharplight tree): per 32-value block an exact int32 dot of
// weight codes and 8-bit activation codes (tcgen05.mma kind::i8, one K = 32 instruction per block, each block into a
// tensor-memory buffer of its own), scaled in f32 on the CUDA cores: acc += float(dot) * d_w[row, block] * d_x[token,
// block], issued as packed f32x2 operations. Weight codes reach the tensor core as int8: Q8_0 as stored, Q4_K nibbles as
// 0..15, Q4_0 as 16 * (nibble - 8) (the nibble moved to the high half of the byte and its top bit flipped -- one logic
// operation; the factor 16 is taken back by the scale table). The Q4_K offset term sum_b m[n,b] * (d_x * sum q)[t,b] is a
// small product of its own and also runs on the tensor core (kind::tf32, the activation factor split in two tf32
// halves).
//
// Shape: weights are the M operand (128 rows per tile, swap-AB), tokens the N operand (16 to 128 per tile). Work is cut
// stream-K fashion: the (tile, 256-value super-tile) units of the whole MatMul are dealt evenly to one persistent CTA
// per SM, so a 112-tile decode MatMul still streams through all 148 SMs; a tile whose K range is shared by several CTAs
// is summed by the last of them to arrive, in CTA order (deterministic), through a scratch area that belongs to the
// activation object.
//
// Roles (24 warps): warps 0 and 2 issue the MMAs (each owns every other block-dot buffer); warp 1 streams weight
// records from global memory and warp 3 the activation scale tables and code tiles (bulk async copies, mbarrier
// completion); 4 or 8 producer warps expand weight codes into 128-byte swizzled int8 operand rows and decode the scale
// tables; 16 or 8 epilogue warps read tensor memory, scale and accumulate (few tokens: more producers, the expansion is
// what has to keep up with memory; many tokens: more epilogue warps). Every wait is bounded and raises the device status
// word when it runs out.
#include "internal.cuh"

#include <cuda_fp16.h>

namespace slc {

typedef unsigned long long ull;

constexpr int UM_ROWS = 128;
constexpr int UM_THREADS = 768;
constexpr int UM_A_STAGE = UM_ROWS * 128;  // one 128-value stage of the weight operand: 128 rows x 128 int8
constexpr int UM_SMEM_LIMIT = 227 * 1024;
constexpr int UM_REG_CTRL = 40;            // registers per thread of the control warps
constexpr int UM_REG_IDLE = 24;            // and of warps without a role

template <int FMT, int NT>
struct UmCfg
{
    static constexpr bool MINS = FMT == FMT_Q4_K;
    // Q6_K changes its scale every 16 values: a 32-value block is two MMAs on two copies of the weight rows, one with the
    // upper and one with the lower sixteen values zero (the same activation codes both times), into two buffers with a
    // weight scale each (the reference's GEMM does the same, src/Sharplight.Shaders/Kernels/mmq.slang:235-239)
    static constexpr int GPB = FMT == FMT_Q6_K ? 2 : 1;           // MMAs (scale groups) per 32-value block
    static constexpr int NB = 8 * GPB;                            // block-dot buffers' worth of work per unit
    static_assert(FMT != FMT_Q6_K || NT == 128, "Q6_K is served at the 128-token tile only");
    static constexpr int PW = NT <= 32 ? 8 : 4;                   // producer warps (warps 4 .. 4 + PW)
    static constexpr int EG = NT <= 32 ? 2 : 4;                   // epilogue groups of four warps (one warp per 32 rows)
    static constexpr int EPI0 = 4 + PW;                           // first epilogue warp
    static constexpr int CS = NT >= 128 ? 4 : NT == 64 ? 2 : 1;   // column slices of the token tile
    static constexpr int BP = EG / CS;                            // epilogue groups taking blocks in turn
    static constexpr int CW = NT / CS;                            // columns per epilogue warp
    static constexpr int DB = NT == 128 ? (MINS ? 2 : 4) : NT == 64 ? 4 : 8;   // tensor-memory buffers for block dots (NB % DB == 0)
    static constexpr int MB = NT == 128 ? 1 : 2;                  // offset-term buffers (Q4_K)
    static constexpr int TM_MINS = DB * NT;                       // first column of the offset-term buffers
    static constexpr int TM_NEED = DB * NT + (MINS ? MB * NT : 0);
    static_assert(TM_NEED <= 512 && DB % 2 == 0 && NB % DB == 0, "tensor memory budget; one issuer per buffer");
    static constexpr int TM_COLS = TM_NEED <= 32 ? 32 : TM_NEED <= 64 ? 64 : TM_NEED <= 128 ? 128 : TM_NEED <= 256 ? 256 : 512;
    // registers per thread after the roles have split; the CTA's pool is 6 warpgroups x 80
    static constexpr int REG_PROD = PW == 8 ? 64 : 56, REG_EPI = EG == 2 ? 136 : 96;
    static_assert(UM_REG_CTRL + (PW / 4) * REG_PROD + EG * REG_EPI + (5 - PW / 4 - EG) * UM_REG_IDLE <= 6 * 80,
                  "setmaxnreg requests exceed the CTA's register pool");
    static constexpr int REC = record_bytes(FMT);
    static constexpr int RAW_SLOT = 8 * REC;
    static constexpr int S = NT == 128 ? 3 : 4;                   // operand stages (128 K-values each: weight rows + code tile)
    static constexpr int B_STAGE = NT * 128;
    static constexpr int A_BYTES = GPB * UM_A_STAGE;               // weight rows of a stage (Q6_K: the two half-masked copies)
    static constexpr int STAGE = A_BYTES + B_STAGE;
    static constexpr int DX_BYTES = 8 * NT * 4;
    static constexpr int SX2_BYTES = MINS ? NT * 64 : 0;
    static constexpr int ACT_SLOT = (DX_BYTES + SX2_BYTES + 511) / 512 * 512;
    static constexpr int WS_DW = NB * UM_ROWS * 4;                // d_w per block (Q6_K: per 16-value group) and row
    static constexpr int WS_ND = MINS ? UM_ROWS * 4 : 0;          // -dmin per row
    static constexpr int WS_A2 = MINS ? UM_ROWS * 64 : 0;         // mins as a tf32 operand tile
    static constexpr int WS_SLOT = WS_DW + WS_ND + WS_A2;
    static constexpr int COMB = (BP - 1) * UM_ROWS * NT * 4;
    // offsets inside the 1024-byte aligned dynamic shared memory
    static constexpr int OFF_STAGE = 0;
    static constexpr int OFF_WS = OFF_STAGE + S * STAGE;          // a multiple of 1024
    static constexpr int OFF_ACT = OFF_WS + 2 * WS_SLOT;
    static constexpr int OFF_COMB = OFF_ACT + 2 * ACT_SLOT;
    static constexpr int OFF_RAW = OFF_COMB + COMB;
    // the weight-record ring takes what is left: its depth is the number of bytes in flight from global memory
    static constexpr int RS_FIT = (UM_SMEM_LIMIT - 1024 - OFF_RAW) / RAW_SLOT;
    static constexpr int RS = RS_FIT > 6 ? 6 : RS_FIT;
    static constexpr int BYTES = OFF_RAW + RS * RAW_SLOT + 1024;  // + alignment slack
    static_assert(RS >= 2 && BYTES <= UM_SMEM_LIMIT, "shared memory budget");
    static_assert(WS_SLOT % 512 == 0 && (WS_DW + WS_ND) % 512 == 0 && STAGE % 1024 == 0 && RAW_SLOT % 16 == 0 && OFF_RAW % 16 == 0, "alignment");
};

struct UmBars
{
    uint64_t rw_full[6], rw_empty[6];    // weight-record ring
    uint64_t ua_full[2], ua_empty[2];    // per-unit activation tables
    uint64_t ws_full[2], ws_empty[2];    // per-unit weight scale tables
    uint64_t full[4], empty[4];          // operand stages
    uint64_t d_full[8], d_empty[8];      // block-dot buffers in tensor memory
    uint64_t m_full[2], m_empty[2];      // offset-term buffers
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
    const uint8_t *q_sw;      // activation codes, 128-byte swizzled rows: [k/128][rows_pad/8][8][128 B]
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
// Bounded wait (about two seconds with naps, well under a second without); gives up early when another role has already
// raised the abort flag. nap_ns > 0: the warp naps between probes, so that the roles that mostly wait leave the issue
// slots to the warps that have work while the tile is compute-bound; with few tokens every role waits on memory most of
// the time and a nap would only add its length to each hand-over.
__device__ __forceinline__ bool um_wait(uint64_t *bar, unsigned parity, volatile int *abort_flag, unsigned nap_ns = 0)
{
    const unsigned b = smem_u32(bar);
#pragma unroll 1
    for (unsigned i = 0; i < 20000000u; i++) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(b), "r"(parity) : "memory");
        if (ok) return true;
        if (nap_ns) __nanosleep(nap_ns);
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
// Instruction descriptors, M = 128, K-major operands: signed int8 x signed int8 -> int32, and tf32 x tf32 -> f32.
__host__ __device__ constexpr unsigned um_idesc_i8(int n) { return (2u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | (8u << 24); }
__host__ __device__ constexpr unsigned um_idesc_tf32(int n) { return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(n >> 3) << 17) | (8u << 24); }

__device__ __forceinline__ void um_mma_i8(unsigned d, uint64_t a, uint64_t b, unsigned idesc, unsigned accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
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
// two int32 -> a packed pair of floats
__device__ __forceinline__ ull um_i2f2(unsigned lo, unsigned hi)
{
    ull r;
    asm("{\n\t.reg .f32 a, b;\n\tcvt.rn.f32.s32 a, %1;\n\tcvt.rn.f32.s32 b, %2;\n\tmov.b64 %0, {a, b};\n\t}" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ ull um_fma2(ull a, ull b, ull c) { ull d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ ull um_mul2(ull a, ull b) { ull d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ ull um_add2(ull a, ull b) { ull d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }

__device__ __forceinline__ float um_h2f(unsigned bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

// Byte offset of 16-byte chunk c (0..7) of row r inside a tile of 128-byte swizzled rows.
__device__ __forceinline__ int um_sw128(int r, int c) { return (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4); }
// The same for 64-byte rows (chunks 0..3).
__device__ __forceinline__ int um_sw64(int r, int c) { return (r >> 3) * 512 + (r & 7) * 64 + ((c ^ ((r & 7) >> 1)) << 4); }
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

// ---- producers: one row group (16 rows) of one 128-value stage -> int8 operand rows ---------------------------------------
//
// a_rg: the stage's operand rows of this row group (two groups of eight 128-byte rows, 1024 bytes apart: rows g and g + 8
// of the record). Block j (0..3) of the stage occupies bytes 32 j .. 32 j + 31 of a row, i.e. 16-byte chunks 2j and
// 2j + 1, and chunk c of row g is stored at chunk position c ^ g (the 128-byte swizzle the operand descriptor names).
// A record hands lane (g, t) eight consecutive values of a block for rows g and g + 8 (Q4_K, Q8_0): an 8-byte store per
// row and block. Were all lanes to store the same block at a time, rows g and g ^ 1 would hit the same banks; so lane
// (g, t) takes the blocks in the order j = step ^ (g & 3), which puts the four rows of a half-warp on the four different
// chunk pairs of the 128-byte row: every store instruction covers all 32 banks exactly once.
template <int FMT>
__device__ __forceinline__ void um_expand(const uint8_t *rec, int c, int lane, uint8_t *a_rg)
{
    const int g = lane >> 2, t = lane & 3;
    const uint4 *tiles = reinterpret_cast<const uint4 *>(rec);
    if constexpr (FMT == FMT_Q4_K) {
        // record tile i (64 values): lane (g, t) holds qs[32 i + 8t .. +7] of rows g (x, y) and g + 8 (z, w); low nibbles
        // are values 8t.. of sub-block 2i, high nibbles the same of sub-block 2i + 1. Stage c = tiles 2c, 2c + 1.
        uint8_t *row_g = a_rg + g * 128 + 8 * (t & 1);
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
            const int ti = kk ^ ((g >> 1) & 1);
            const uint4 q = tiles[(2 * c + ti) * 32 + lane];
#pragma unroll
            for (int k2 = 0; k2 < 2; k2++) {
                const int nib = k2 ^ (g & 1);
                const int j = 2 * ti + nib;
                const unsigned sh = 4u * (unsigned)nib;
                const unsigned ch = (unsigned)(((2 * j + (t >> 1)) ^ g) << 4);
                *reinterpret_cast<uint2 *>(row_g + ch) = make_uint2((q.x >> sh) & 0x0F0F0F0Fu, (q.y >> sh) & 0x0F0F0F0Fu);
                *reinterpret_cast<uint2 *>(row_g + 1024 + ch) = make_uint2((q.z >> sh) & 0x0F0F0F0Fu, (q.w >> sh) & 0x0F0F0F0Fu);
            }
        }
    } else if constexpr (FMT == FMT_Q8_0) {
        // record tile i = block i: lane (g, t) holds q[8t .. 8t+7] of rows g (x, y) and g + 8 (z, w). Stage c = tiles 4c..4c+3.
        uint8_t *row_g = a_rg + g * 128 + 8 * (t & 1);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int j = k ^ (g & 3);
            const uint4 q = tiles[(4 * c + j) * 32 + lane];
            const unsigned ch = (unsigned)(((2 * j + (t >> 1)) ^ g) << 4);
            *reinterpret_cast<uint2 *>(row_g + ch) = make_uint2(q.x, q.y);
            *reinterpret_cast<uint2 *>(row_g + 1024 + ch) = make_uint2(q.z, q.w);
        }
    } else if constexpr (FMT == FMT_Q6_K) {
        // Stage c = half c of the super-block: planes 3c (row g) and 3c + 1 (row g + 8) hold L[l0..+3], L[32+l0..+3],
        // L[l1..+3], L[32+l1..+3] with l0 = 4t, l1 = 16 + 4t; plane 3c + 2 holds H[l0..+3], H[l1..+3] of row g, then of
        // row g + 8. Quarter v (0..3) of the half is block v of the stage: values l of it are
        // (low or high nibble of L[l] or L[32 + l]) | (bits 2v, 2v+1 of H[l]) << 4, minus 32. Its lower sixteen values
        // (l0 part) go to chunk 2v of the first copy, its upper sixteen (l1 part) to chunk 2v + 1 of the second copy;
        // the other halves of both copies stay zero. Four bytes per store, eight rows on eight chunk positions.
        const uint4 L[2] = { tiles[(3 * c) * 32 + lane], tiles[(3 * c + 1) * 32 + lane] };
        const uint4 H = tiles[(3 * c + 2) * 32 + lane];
        uint8_t *row_g = a_rg + g * 128 + 4 * t;
#pragma unroll
        for (int r = 0; r < 2; r++) {
#pragma unroll
            for (int li = 0; li < 2; li++) {
                const unsigned lw = li ? L[r].z : L[r].x, lw32 = li ? L[r].w : L[r].y;
                const unsigned hw = r ? (li ? H.w : H.z) : (li ? H.y : H.x);
#pragma unroll
                for (int v = 0; v < 4; v++) {
                    const unsigned lsrc = (v & 1) ? lw32 : lw;
                    const unsigned lo4 = ((v & 2) ? (lsrc >> 4) : lsrc) & 0x0F0F0F0Fu;
                    const unsigned u = lo4 | (((hw >> (2 * v)) & 0x03030303u) << 4);       // 0..63
                    const unsigned x = u ^ 0x20202020u;                                     // six-bit two's complement of u - 32
                    const unsigned code = x | ((x & 0x20202020u) * 6u);                     // sign bit copied to bits 6, 7
                    *reinterpret_cast<unsigned *>(row_g + li * UM_A_STAGE + r * 1024 + (((2 * v + li) ^ g) << 4)) = code;
                }
            }
        }
    } else {
        // Q4_0, record tile i (two blocks): words x = row g block 2i, y = row g+8 block 2i, z = row g block 2i+1,
        // w = row g+8 block 2i+1, each qs[4t .. 4t+3]: low nibbles are values 4t.. of the block, high nibbles values
        // 16 + 4t... Operand byte = 16 * (nibble - 8): the nibble in the high half, top bit flipped. Four bytes per
        // store; the eight rows of a store land on eight different chunk positions. Stage c = tiles 2c, 2c + 1.
        uint8_t *row_g = a_rg + g * 128 + 4 * t;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const uint4 q = tiles[(2 * c + i) * 32 + lane];
            const unsigned wv[4] = { q.x, q.y, q.z, q.w };
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const int j = 2 * i + (m >> 1);
                uint8_t *dst = row_g + (m & 1) * 1024;
                *reinterpret_cast<unsigned *>(dst + (((2 * j) ^ g) << 4)) = ((wv[m] << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
                *reinterpret_cast<unsigned *>(dst + (((2 * j + 1) ^ g) << 4)) = (wv[m] & 0xF0F0F0F0u) ^ 0x80808080u;
            }
        }
    }
}

// The per-unit tables of one row group: the f32 weight scale of every (block, row) for the epilogue -- Q4_K: d * 6-bit
// sub-block scale (decoded as in src/Sharplight.Cpu/Quant.cs:504-516 of the Sharplight tree), Q4_0: d / 16 (the operand
// carries 16 * code), Q8_0: d -- and for Q4_K -dmin per row and the sub-block mins as a tf32 operand tile.
template <int FMT>
__device__ __forceinline__ void um_tables(const uint8_t *rec, int rgl, int lane, uint8_t *ws_slot)
{
    const int g = lane >> 2, t = lane & 3;
    const uint4 *hdr = reinterpret_cast<const uint4 *>(rec + code_bytes(FMT));
    using Cfg = UmCfg<FMT, 128>;
    float *dw = reinterpret_cast<float *>(ws_slot);
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const uint4 h = hdr[g + 8 * r];
        const int row = rgl * 16 + g + 8 * r;
        if constexpr (FMT == FMT_Q4_K) {
            const float d = um_h2f(h.x & 0xffffu);
            if (t == 0) reinterpret_cast<float *>(ws_slot + Cfg::WS_DW)[row] = -um_h2f(h.x >> 16);
            // scales and mins of sub-blocks 2t, 2t + 1
            const unsigned scw = t < 2 ? (h.y & 0x3F3F3F3Fu) : ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u));
            const unsigned mnw = t < 2 ? (h.z & 0x3F3F3F3Fu) : (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u));
            const int sh = 16 * (t & 1);
            dw[(2 * t) * UM_ROWS + row] = d * (float)((scw >> sh) & 0xffu);
            dw[(2 * t + 1) * UM_ROWS + row] = d * (float)((scw >> (sh + 8)) & 0xffu);
            // mins as floats (exact tf32 values) at K positions 2t, 2t+1 and again at 8 + 2t, 8 + 2t+1
            const float2 mn = make_float2((float)((mnw >> sh) & 0xffu), (float)((mnw >> (sh + 8)) & 0xffu));
            uint8_t *a2 = ws_slot + Cfg::WS_DW + Cfg::WS_ND;
            *reinterpret_cast<float2 *>(a2 + um_sw64(row, t >> 1) + 8 * (t & 1)) = mn;
            *reinterpret_cast<float2 *>(a2 + um_sw64(row, 2 + (t >> 1)) + 8 * (t & 1)) = mn;
        } else if constexpr (FMT == FMT_Q6_K) {
            // i8 scales of the 16-value groups 4t .. 4t + 3, times the row's f16 d
            const unsigned short *dp = reinterpret_cast<const unsigned short *>(rec + code_bytes(FMT) + 256);
            const float d = um_h2f(dp[g + 8 * r]);
            const unsigned scw = t == 0 ? h.x : t == 1 ? h.y : t == 2 ? h.z : h.w;
#pragma unroll
            for (int i = 0; i < 4; i++) dw[(4 * t + i) * UM_ROWS + row] = d * (float)(int)(signed char)((scw >> (8 * i)) & 0xffu);
        } else {
            // f16 scale of blocks 2t and 2t + 1
            const unsigned wsc = t == 0 ? h.x : t == 1 ? h.y : t == 2 ? h.z : h.w;
            const float f = FMT == FMT_Q4_0 ? 0.0625f : 1.0f;
            dw[(2 * t) * UM_ROWS + row] = um_h2f(wsc & 0xffffu) * f;
            dw[(2 * t + 1) * UM_ROWS + row] = um_h2f(wsc >> 16) * f;
        }
    }
}

// ---- the kernel ------------------------------------------------------------------------------------------------------

template <int FMT, int NT, bool DUMP>
__global__ void __launch_bounds__(UM_THREADS, 1) umma_kernel(const UmParams p)
{
    using Cfg = UmCfg<FMT, NT>;
    constexpr bool MINS = Cfg::MINS;
    constexpr int CS = Cfg::CS, BP = Cfg::BP, CW = Cfg::CW, DB = Cfg::DB, S = Cfg::S, RS = Cfg::RS, PW = Cfg::PW, EG = Cfg::EG;
    constexpr int GPB = Cfg::GPB, NB = Cfg::NB;
    extern __shared__ __align__(1024) unsigned char um_smem_raw[];
    __shared__ UmBars sh;
    unsigned char *smem = um_smem_raw + ((1024 - (smem_u32(um_smem_raw) & 1023)) & 1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *abort_flag = &sh.abort;
    // Naps between barrier probes keep waiting warps out of the issue slots when the tile is compute-bound (128 tokens);
    // with few tokens every role waits on memory most of the time and a nap only adds its length to each hand-over.
    constexpr unsigned NAP = NT >= 128 ? 1u : 0u;

    if (threadIdx.x == 0) {
        for (int i = 0; i < RS; i++) { mbar_init(&sh.rw_full[i], 1); mbar_init(&sh.rw_empty[i], PW); }
        for (int i = 0; i < 2; i++) {
            mbar_init(&sh.ua_full[i], 1); mbar_init(&sh.ua_empty[i], 4 * EG);
            mbar_init(&sh.ws_full[i], PW); mbar_init(&sh.ws_empty[i], 4 * EG);
            mbar_init(&sh.m_full[i], 1); mbar_init(&sh.m_empty[i], 4 * CS);
        }
        // a stage is full when every producer warp has written its rows and the code tile's bytes have landed (the
        // loader's arrival carries the byte count); it is empty when both MMA issuers' instructions on it are done
        for (int i = 0; i < S; i++) { mbar_init(&sh.full[i], PW + 1); mbar_init(&sh.empty[i], 2); }
        for (int i = 0; i < DB; i++) { mbar_init(&sh.d_full[i], 1); mbar_init(&sh.d_empty[i], 4 * CS); }
        mbar_init(&sh.comb_full, BP > 1 ? 4 * EG - 4 * CS : 1);
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
    // requests add up to more than the pool (UmCfg checks the sum).
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
                if (!um_wait(&sh.rw_empty[slot], phase, abort_flag, NAP * 1000)) break;
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
            // ===== MMA issuers: two threads (warps 0 and 2). Both visit every stage; a stage holds four blocks (Q6_K: eight
            // 16-value groups), the i-th of them goes to buffer (first of the stage + i) % DB, and issuer `me` takes those
            // with i % 2 == me. Every block-dot buffer so has
            // ONE issuer: a parity wait tells "free again" from "not yet used" only for a thread that is at most one use
            // ahead of the barrier. The issuers need only the number of units, not which tiles they belong to.
            if (lane == 0) {
                constexpr unsigned idesc = um_idesc_i8(NT), idesc_m = um_idesc_tf32(NT);
                const unsigned st_lo0 = (smem_u32(smem + Cfg::OFF_STAGE) >> 4) & 0x3FFFu;
                const unsigned desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);          // bits 32..63: sbo 1024, version, 128-byte swizzle
                const unsigned desc_hi_m = (512u >> 4) | (1u << 14) | (4u << 29);         // sbo 512, version, 64-byte swizzle
                auto mk = [](unsigned lo14, unsigned hi) { return (uint64_t)(lo14 | (1u << 16)) | ((uint64_t)hi << 32); };
                const int n_stages = (int)(wk.u_end - wk.u) * 2;
                const int me = warp >> 1;                         // 0 or 1
                int stage = 0;
                unsigned phase = 0;
                bool ok = true;
#pragma unroll 1
                for (int k = 0; k < n_stages && ok; k++) {
                    const int unit = k >> 1, c = k & 1;
                    if (!um_wait(&sh.full[stage], phase, abort_flag, NAP * 100)) { ok = false; break; }
                    um_tc_after();
                    const unsigned a_lo = st_lo0 + (unsigned)(stage * (Cfg::STAGE >> 4)), b_lo = a_lo + (unsigned)(Cfg::A_BYTES >> 4);
#pragma unroll
                    for (int ii = 0; ii < 2 * GPB; ii++) {
                        const int i = me + 2 * ii;                       // this issuer's MMAs of the stage
                        const int j = i / GPB, half = i % GPB;           // block of the stage; Q6_K: which sixteen values
                        const int b = 4 * GPB * c + i, buf = b % DB;
                        const unsigned dphase = ((unsigned)((unit * NB + b) / DB) & 1u) ^ 1u;
                        if (!um_wait(&sh.d_empty[buf], dphase, abort_flag, NAP * 100)) { ok = false; break; }
                        um_tc_after();
                        // K values 32 j .. 32 j + 31: 32 bytes = 2 sixteen-byte units along the swizzled row
                        um_mma_i8(tmem + (unsigned)(buf * NT), mk(a_lo + (unsigned)(half * (UM_A_STAGE >> 4)) + 2 * j, desc_hi),
                                  mk(b_lo + 2 * j, desc_hi), idesc, 0);
                        um_commit(&sh.d_full[buf]);
                    }
                    if (!ok) break;
                    um_commit(&sh.empty[stage]);
                    if (++stage == S) { stage = 0; phase ^= 1u; }
                    if (MINS && c == 1 && me == 1) {
                        // offset term of the unit: D2[n][t] = sum_b m[n,b] * (sx_hi + sx_lo)[t,b], two K = 8 steps
                        const int us = unit & 1, mb = unit % Cfg::MB;
                        const unsigned uphase = (unsigned)(unit >> 1) & 1u;
                        if (!um_wait(&sh.ws_full[us], uphase, abort_flag, NAP * 100) || !um_wait(&sh.ua_full[us], uphase, abort_flag, NAP * 100) ||
                            !um_wait(&sh.m_empty[mb], ((unsigned)(unit / Cfg::MB) & 1u) ^ 1u, abort_flag, NAP * 100)) { ok = false; break; }
                        um_tc_after();
                        const unsigned a2 = (smem_u32(smem + Cfg::OFF_WS + us * Cfg::WS_SLOT + Cfg::WS_DW + Cfg::WS_ND) >> 4) & 0x3FFFu;
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
            // d_x * sum q tile), then one bulk copy of the code tile per 128-value stage
            if (lane == 0) {
                int stage = 0, unit = 0;
                unsigned phase = 1;
                bool ok = true;
                for (; !wk.done() && ok; wk.next(), unit++) {
                    const int us = unit & 1;
                    const int t0 = (wk.tile % p.tok_tiles) * NT;
                    if (!um_wait(&sh.ua_empty[us], ((unsigned)(unit >> 1) & 1u) ^ 1u, abort_flag, NAP * 500)) break;
                    unsigned char *dst = smem + Cfg::OFF_ACT + us * Cfg::ACT_SLOT;
                    um_expect_tx(&sh.ua_full[us], (unsigned)(Cfg::DX_BYTES + Cfg::SX2_BYTES));
                    for (int b = 0; b < 8; b++) {
                        um_bulk(dst + b * NT * 4, p.a.dx + (long long)(wk.st * 8 + b) * p.a.rows_pad + t0, NT * 4, &sh.ua_full[us]);
                    }
                    if (MINS) um_bulk(dst + Cfg::DX_BYTES, p.sx2 + ((long long)wk.st * tok_groups + (t0 >> 3)) * 512, Cfg::SX2_BYTES, &sh.ua_full[us]);
                    for (int c = 0; c < 2; c++) {
                        if (!um_wait(&sh.empty[stage], phase, abort_flag, NAP * 500)) { ok = false; break; }
                        um_expect_tx(&sh.full[stage], (unsigned)Cfg::B_STAGE);
                        um_bulk(smem + Cfg::OFF_STAGE + stage * Cfg::STAGE + Cfg::A_BYTES,
                                p.q_sw + ((long long)(wk.st * 2 + c) * tok_groups + (t0 >> 3)) * 1024, Cfg::B_STAGE, &sh.full[stage]);
                        if (++stage == S) { stage = 0; phase ^= 1u; }
                    }
                }
            }
        } else if (warp < Cfg::EPI0) {
            // ===== producers: weight codes -> int8 operand rows, scale tables. Warp pw owns 8 / PW row groups of every stage.
            asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::REG_PROD));
            constexpr int RPW = 8 / PW;
            const int pw = warp - 4;
            int slot = 0, stage = 0, unit = 0;
            unsigned rphase = 0, sphase = 1;
            bool ok = true;
            if constexpr (GPB == 2) {
                // the zero halves of the two masked copies never change: written once, for every stage
                for (int st = 0; st < S; st++) {
                    uint4 *z = reinterpret_cast<uint4 *>(smem + Cfg::OFF_STAGE + st * Cfg::STAGE);
                    for (int i = pw * 32 + lane; i < Cfg::A_BYTES / 16; i += PW * 32) z[i] = make_uint4(0u, 0u, 0u, 0u);
                }
                um_fence_async();
                asm volatile("bar.sync 1, %0;" ::"n"(PW * 32) : "memory");   // (the producer warps only; passed once, at the start)
            }
            for (; !wk.done() && ok; wk.next(), unit++) {
                const int us = unit & 1;
                if (!um_wait(&sh.rw_full[slot], rphase, abort_flag, NAP * 300) ||
                    !um_wait(&sh.ws_empty[us], ((unsigned)(unit >> 1) & 1u) ^ 1u, abort_flag, NAP * 300)) { ok = false; break; }
                const uint8_t *raw = smem + Cfg::OFF_RAW + slot * Cfg::RAW_SLOT;
                const int rg0 = (wk.tile / p.tok_tiles) * 8;
                uint8_t *ws_slot = smem + Cfg::OFF_WS + us * Cfg::WS_SLOT;
#pragma unroll
                for (int i = 0; i < RPW; i++) {
                    const int rgl = pw * RPW + i;
                    if (rg0 + rgl < rg_count) um_tables<FMT>(raw + rgl * Cfg::REC, rgl, lane, ws_slot);
                }
                um_fence_async();
                __syncwarp();
                if (lane == 0) um_arrive(&sh.ws_full[us]);
#pragma unroll 1
                for (int c = 0; c < 2; c++) {
                    if (!um_wait(&sh.empty[stage], sphase, abort_flag, NAP * 300)) { ok = false; break; }
                    uint8_t *a_stage = smem + Cfg::OFF_STAGE + stage * Cfg::STAGE;
#pragma unroll
                    for (int i = 0; i < RPW; i++) {
                        const int rgl = pw * RPW + i;
                        if (rg0 + rgl < rg_count) um_expand<FMT>(raw + rgl * Cfg::REC, c, lane, a_stage + rgl * 2048);
                    }
                    um_fence_async();   // generic-proxy stores -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) um_arrive(&sh.full[stage]);
                    if (++stage == S) { stage = 0; sphase ^= 1u; }
                }
                __syncwarp();
                if (lane == 0 && ok) um_arrive(&sh.rw_empty[slot]);
                if (++slot == RS) { slot = 0; rphase ^= 1u; }
            }
            if (!ok && lane == 0) atomicExch(p.status, -7);
        } else if (warp < Cfg::EPI0 + 4 * EG) {
            // ===== epilogue: warp = (TMEM lane quarter q, column slice cs, block turn bp)
            asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Cfg::REG_EPI));
            const int e = warp - Cfg::EPI0;
            const int q = e & 3, cs = (e >> 2) % CS, bp = (e >> 2) / CS;
            const int r = q * 32 + lane;                       // weight row inside the tile = TMEM lane
            const int c0 = cs * CW;
            const unsigned tlane = tmem + ((unsigned)(q * 32) << 16) + (unsigned)c0;
            const unsigned smem_s = smem_u32(smem);
            ull acc[CW / 2];                                   // running sums of the tile, packed pairs of columns
#pragma unroll
            for (int j = 0; j < CW / 2; j++) acc[j] = 0ull;
            bool ok = true;
            int unit = 0, n_comb = 0, n_fix = 0;               // tile ends / fix-ups so far (barrier phases)
            const long long u_first = wk.u;
            int seg_st0 = wk.st;                               // first super-tile of the running tile's segment
#pragma unroll 1
            for (; !wk.done() && ok; wk.next(), unit++) {
                const int us = unit & 1;
                const unsigned uphase = (unsigned)(unit >> 1) & 1u;
                if (!um_wait(&sh.ua_full[us], uphase, abort_flag, NAP * 100) || !um_wait(&sh.ws_full[us], uphase, abort_flag, NAP * 100)) { ok = false; break; }
                const unsigned ws_s = smem_s + (unsigned)(Cfg::OFF_WS + us * Cfg::WS_SLOT);
                // The unit's blocks of this warp as 16-column chunks; a block's buffer goes back to its MMA issuer as soon
                // as the last chunk has arrived in registers. The loop over blocks is a real loop (the code of all roles
                // has to stay resident in the instruction cache).
                constexpr int HPB = CW / 16, NBLK = NB / BP;
                const ulonglong2 *dx_tab = reinterpret_cast<const ulonglong2 *>(smem + Cfg::OFF_ACT + us * Cfg::ACT_SLOT) + c0 / 4;
#pragma unroll 1
                for (int bi = 0; bi < NBLK; bi++) {
                    const int b = bi * BP + bp, buf = b % DB;
                    if (!um_wait(&sh.d_full[buf], (unsigned)((unit * NB + b) / DB) & 1u, abort_flag, NAP * 20)) { ok = false; break; }
                    um_tc_after();
                    const float dw = um_lds_f32(ws_s + (unsigned)((b * UM_ROWS + r) * 4));
                    const ull dw2 = um_pkf(dw, dw);
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
                                const int tok = t0 + c0 + h * 16 + j, row = n0 + r, blk = wk.st * 8 + b / GPB;
                                if (tok < p.a.rows && row < p.w.n && blk * 32 < p.w.k) {
                                    // the reference's block dot has unsigned weight codes (code + 128, nibble, 6-bit value):
                                    // add the offset times the block's activation sum
                                    const int cexp = FMT == FMT_Q8_0 ? 128 : FMT == FMT_Q4_0 ? 8 : FMT == FMT_Q6_K ? 32 : 0;
                                    const int add = cexp ? cexp * __ldg(&p.a.isum[(long long)tok * (p.a.k_pad >> 5) + blk]) : 0;
                                    const int dot = FMT == FMT_Q4_0 ? ((int)v[j] >> 4) : (int)v[j];
                                    int *dst = &p.dump[((long long)tok * p.w.n + row) * (p.w.k >> 5) + blk];
                                    // Q6_K: the block's two groups come one after the other to this same thread
                                    if (GPB == 1 || (b & 1) == 0) *dst = dot + add;
                                    else *dst += dot;
                                }
                            }
                        }
#pragma unroll
                        for (int j4 = 0; j4 < 4; j4++) {
                            const ulonglong2 dx = dx_tab[((b / GPB) * NT + h * 16) / 4 + j4];
                            const int o = h * 8 + j4 * 2;
                            const ull t01 = um_mul2(um_i2f2(v[4 * j4], v[4 * j4 + 1]), dw2);
                            const ull t23 = um_mul2(um_i2f2(v[4 * j4 + 2], v[4 * j4 + 3]), dw2);
                            acc[o] = um_fma2(t01, dx.x, acc[o]);
                            acc[o + 1] = um_fma2(t23, dx.y, acc[o + 1]);
                        }
                    }
                }
                if (!ok) break;
                if (MINS && bp == 0) {
                    // the unit's offset term: acc -= dmin * D2. Waiting for its MMAs also means the unit's operand tiles
                    // (mins, split sums) are no longer read, so the slots may be refilled after this warp's arrival below.
                    const float nd_min = um_lds_f32(ws_s + (unsigned)(Cfg::WS_DW + r * 4));
                    const ull nm2 = um_pkf(nd_min, nd_min);
                    const int mb = unit % Cfg::MB;
                    if (!um_wait(&sh.m_full[mb], (unsigned)(unit / Cfg::MB) & 1u, abort_flag, NAP * 100)) { ok = false; break; }
                    um_tc_after();
#pragma unroll
                    for (int h = 0; h < CW / 16; h++) {
                        ull v[8];
                        um_ld16p(tlane + (unsigned)(Cfg::TM_MINS + mb * NT + h * 16), v);
                        um_wait_ld();
#pragma unroll
                        for (int j = 0; j < 8; j++) acc[h * 8 + j] = um_fma2(v[j], nm2, acc[h * 8 + j]);
                    }
                    um_tc_before();
                    __syncwarp();
                    if (lane == 0) um_arrive(&sh.m_empty[mb]);
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
                // 16 columns of this thread's running sums (cleared for the next tile)
                auto chunk = [&](int h, float (&a)[16]) {
#pragma unroll
                    for (int j = 0; j < 8; j++) { um_unpk(acc[h * 8 + j], a[2 * j], a[2 * j + 1]); acc[h * 8 + j] = 0ull; }
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
                    if (!um_wait(&sh.comb_free, ((unsigned)n_comb & 1u) ^ 1u, abort_flag, NAP * 100)) { ok = false; break; }
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
                    if (BP > 1 && !um_wait(&sh.comb_full, (unsigned)n_comb & 1u, abort_flag, NAP * 100)) { ok = false; break; }
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
                            if (!um_wait(&sh.fx_written, (unsigned)n_fix & 1u, abort_flag, NAP * 100)) { ok = false; break; }
                            if (lane == 0) {
                                const int arrived = atomicAdd(&p.counters[c_first], 1);
                                const int last = arrived == c_last - c_first;
                                if (last) p.counters[c_first] = 0;   // ready for the next launch
                                sh.last_flag = last;
                                um_arrive(&sh.fx_decided);
                            }
                        }
                        // (a warp reads the flag of this fix-up before it can arrive for the next one, and the flag is
                        // rewritten only after all warps have arrived for that next one)
                        if (!um_wait(&sh.fx_decided, (unsigned)n_fix & 1u, abort_flag, NAP * 100)) { ok = false; break; }
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
                seg_st0 = 0;   // the next tile, if any, starts at its first super-tile
            }
            if (!ok && lane == 0) atomicExch(p.status, -7);
        } else {
            // no role (few-token configurations): give the registers back
            asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(UM_REG_IDLE));
        }
    }

    um_tc_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((unsigned)Cfg::TM_COLS) : "memory");
    }
}

// ---- host side --------------------------------------------------------------------------------------------------------

// Q6_K at the 128-token tile only (more than 64 rows)
bool umma_supports(int fmt, int rows) { return fmt == FMT_Q4_K || fmt == FMT_Q4_0 || fmt == FMT_Q8_0 || (fmt == FMT_Q6_K && rows > 64); }

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
    if constexpr (FMT == FMT_Q6_K) {
        return nt == 128 ? um_launch<FMT, 128, DUMP>(p, ctas, stream) : cudaErrorInvalidValue;
    } else {
        switch (nt) {
        case 16: return um_launch<FMT, 16, DUMP>(p, ctas, stream);
        case 32: return um_launch<FMT, 32, DUMP>(p, ctas, stream);
        case 64: return um_launch<FMT, 64, DUMP>(p, ctas, stream);
        case 128: return um_launch<FMT, 128, DUMP>(p, ctas, stream);
        default: return cudaErrorInvalidValue;
        }
    }
}

// a.rows_pad must be a multiple of the token tile (16, 32, 64, or 128 for more than 64 rows); q_sw / sx2 are the
// tiled planes the quantizer wrote for these rows; scratch / counters belong to the activation object (umma_scratch_bytes
// for max_ctas CTAs; counters: max_ctas ints, zero).
cudaError_t launch_umma(const WeightView &w, const ActView &a, const uint8_t *q_sw, const uint8_t *sx2, float *y,
                        long long y_stride, int *dump, int *status, float *scratch, int *counters, int max_ctas,
                        cudaStream_t stream, const Epilogue *epilogue)
{
    if (w.n_pad == 0 || a.rows == 0) return cudaSuccess;
    const int nt = umma_token_tile(a.rows);
    if (!q_sw || !sx2 || !scratch || !counters || (a.rows_pad % nt) != 0 || max_ctas < 1) return cudaErrorInvalidValue;
    UmParams p;
    p.w = w; p.a = a; p.q_sw = q_sw; p.sx2 = sx2; p.y = y; p.y_stride = y_stride; p.dump = dump; p.status = status;
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
        SLC_FMT(FMT_Q4_K) SLC_FMT(FMT_Q4_0) SLC_FMT(FMT_Q8_0) SLC_FMT(FMT_Q6_K)
    default: return cudaErrorInvalidValue;
    }
#undef SLC_FMT
}

}  // namespace slc
