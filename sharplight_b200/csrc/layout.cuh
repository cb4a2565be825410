// Device-side data layout of weights and quantized activations, shared by every kernel of libsharplight_cuda.
//
// Weights arrive as raw ggml blocks (block layouts: src/Sharplight.Core/Tensors/DataType.cs:102,110,116,120 of the
// Sharplight tree) and are re-laid-out once at upload, at the same byte count apart from padding, the way the reference
// repacks Q8_0 at upload (src/Sharplight.Shaders/Lowering/WeightRepacker.cs:56-69). The layout is a sequence of
// "records": rows are grouped 16 at a time (row group rg = n / 16; N is padded to a multiple of 16 with zero rows),
// K is cut in 256-value super-tiles (K is padded to a multiple of 256 with zero blocks: zero scale, zero codes), and
// the record of (rg, st) holds everything the 16 rows need for those 256 values, contiguously:
//
//     record(rg, st) at byte ((rg * k_pad/256) + st) * record_bytes(fmt)
//     [ codes: "fragment-major" 16-byte units ][ scales: 16 rows x 16 bytes ][ Q6_K only: d, 16 rows x 2 bytes ]
//
// record_bytes = 16 rows x the raw bytes of 256 values: Q4_0 / Q4_K 2304, Q8_0 4352, Q6_K 3360 (all multiples of 16,
// so one record, or a run of records of one row group, is one bulk async copy into shared memory).
//
// Codes: the 4/6/8-bit codes of a 16-row x KT-value tile are 32 lanes x 16 bytes = 512 contiguous bytes, lane
// (g, t) = (lane / 4, lane % 4) holding exactly the bytes that lane needs of rows g and g + 8 -- the operand fragment
// of an int8 m16n8k32 tensor-core tile, which is also what a dp4a lane wants -- so every weight byte travels by a
// 128-bit access straight into the register that consumes it. Within a 32-value block the K order of a lane's bytes
// may differ from the natural order (a dot product does not care as long as the activation bytes are fetched in the
// same order); the per-format order:
//
//   Q8_0  8 tiles of 32 values (one block).  lane: [row g: q[8t..8t+7]] [row g+8: q[8t..8t+7]]
//         scales entry of a row: f16 d of its 8 blocks
//   Q4_0  4 tiles of 64 values (two blocks). lane words: w0 = row g   blk 2i   qs[4t..4t+3]
//                                                        w1 = row g+8 blk 2i   qs[4t..4t+3]
//                                                        w2 = row g   blk 2i+1 qs[4t..4t+3]
//                                                        w3 = row g+8 blk 2i+1 qs[4t..4t+3]
//         (low nibbles = values 4t..4t+3, high nibbles = values 16+4t..16+4t+3 of the block)
//         scales entry of a row: f16 d of its 8 blocks
//   Q4_K  4 tiles of 64 values (chunk c of the super-block: sub-block 2c in the low, 2c+1 in the high nibbles).
//                                            lane: [row g: qs[32c+8t..+7]] [row g+8: qs[32c+8t..+7]]
//         scales entry of a row: f16 d, f16 dmin, u8 scales[12] (the block header, verbatim)
//   Q6_K  2 tiles of 128 values (half h of the super-block), three 512-byte planes each; with L = ql + 64h,
//         H = qh + 32h, l0 = 4t, l1 = 16 + 4t:
//           plane 0 lane: row g:   L[l0..+3], L[32+l0..+3], L[l1..+3], L[32+l1..+3]
//           plane 1 lane: row g+8: the same
//           plane 2 lane: H[l0..+3] (row g), H[l1..+3] (row g), H[l0..+3] (row g+8), H[l1..+3] (row g+8)
//         scales entry of a row: i8 scales[16] (verbatim); then d: f16 per row
//
// Quantized activations (the reference's Q8Row, src/Sharplight.Cpu/Q8Row.cs:9-20, in a GPU-friendly arrangement):
//   q    int8   [rows_pad][k_pad]        codes, zero beyond K
//   ds   float2 [k_pad/32][rows_pad]     (d, d * sum32(q)) per block, token-minor so neighbouring tokens share a load
//   dx, sx float [k_pad/32][rows_pad]    the two halves of ds as planes of their own (GEMM scale tables)
//   gs   float  [rows_pad][k_pad/16]     d * sum16(q), the reference's group sums (parity export)
//   isum int32  [rows_pad][k_pad/32]     sum32(q) (parity export: converts signed block dots to unsigned-code dots)
// rows_pad = rows rounded up to 8, 16, 32 or a multiple of 64.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace slc {

enum : int { FMT_Q4_0 = 2, FMT_Q8_0 = 8, FMT_Q4_K = 12, FMT_Q6_K = 14 };

__host__ __device__ inline int block_size(int fmt)
{
    return (fmt == FMT_Q4_0 || fmt == FMT_Q8_0) ? 32 : (fmt == FMT_Q4_K || fmt == FMT_Q6_K) ? 256 : 0;
}

__host__ __device__ inline int block_bytes(int fmt)
{
    return fmt == FMT_Q4_0 ? 18 : fmt == FMT_Q8_0 ? 34 : fmt == FMT_Q4_K ? 144 : fmt == FMT_Q6_K ? 210 : 0;
}

// Formats that are accepted at upload and turned into the Q8_0 device layout, exactly: Q5_0 { f16 d; u32 qh; u8 qs[16] }
// (value d * (q - 16): the signed code q - 16 fits a byte) and IQ4_NL { f16 d; u8 qs[16] } (value d * codebook[nibble], the
// codebook entry being the signed byte). The reference's integer-dot path treats them the same way: unsigned code, the
// block's f16 d, an offset of -16 d or -128 d (src/Sharplight.Cpu/IntDot.Decode.cs:101-123, 225-238). They cost 34 bytes
// per 32 values on the device instead of 22 / 18.
//
// Q5_K { f16 d; f16 dmin; u8 scales[12]; u8 qh[32]; u8 qs[128] } is Q4_K with a fifth bit per value: d * sc * (q4 + 16 h)
// - dmin * m = [d * sc * q4 - dmin * m] + [(16 d) * sc * h]. It is split at upload, exactly, into two Q4_K weights -- the
// block without qh, and a block with d' = 16 d (a power of two: exact in f16), dmin' = 0, the same scales and the high
// bits as nibbles -- and a MatMul runs both, the second adding onto the first. 288 instead of 176 bytes per 256 values.
enum : int { FMT_Q5_0 = 6, FMT_Q5_K = 13, FMT_IQ4_NL = 20 };

// The format the kernels see for an uploaded format (0: not served).
__host__ __device__ inline int device_format(int fmt)
{
    return (fmt == FMT_Q5_0 || fmt == FMT_IQ4_NL) ? FMT_Q8_0 : fmt == FMT_Q5_K ? FMT_Q4_K : block_size(fmt) ? fmt : 0;
}
// Values and bytes per block of the format as the host hands it over.
__host__ __device__ inline int source_block_size(int fmt)
{
    return (fmt == FMT_Q5_0 || fmt == FMT_IQ4_NL) ? 32 : fmt == FMT_Q5_K ? 256 : block_size(fmt);
}
__host__ __device__ inline int source_block_bytes(int fmt)
{
    return fmt == FMT_Q5_0 ? 22 : fmt == FMT_IQ4_NL ? 18 : fmt == FMT_Q5_K ? 176 : block_bytes(fmt);
}
// What the reference's unsigned code adds to the signed code the kernels multiply (block-dot export): Q8_0 and IQ4_NL
// 128, Q4_0 8, Q6_K 32, Q4_K 0, Q5_0 16.
__host__ __device__ inline int unsigned_code_offset(int fmt)
{
    return fmt == FMT_Q8_0 || fmt == FMT_IQ4_NL ? 128 : fmt == FMT_Q4_0 ? 8 : fmt == FMT_Q6_K ? 32 : fmt == FMT_Q5_0 ? 16 : 0;
}

// 16-byte units of codes per record (all formats: a multiple of 32 lanes).
__host__ __device__ constexpr int code_units(int fmt)
{
    // Q8_0: 8 tiles, Q4_0 / Q4_K: 4 tiles, Q6_K: 2 tiles x 3 planes; 32 lanes each
    return (fmt == FMT_Q8_0 ? 8 : fmt == FMT_Q6_K ? 6 : 4) * 32;
}

__host__ __device__ constexpr int code_bytes(int fmt) { return code_units(fmt) * 16; }

// Bytes of one record: codes, 16 scale entries of 16 bytes, and for Q6_K the 16 f16 super-block scales.
__host__ __device__ constexpr int record_bytes(int fmt)
{
    return code_bytes(fmt) + 256 + (fmt == FMT_Q6_K ? 32 : 0);
}

struct WeightView
{
    int fmt;
    int n, k;          // logical shape
    int n_pad, k_pad;  // multiples of 16 / 256
    const uint8_t *data;  // records: [n_pad/16][k_pad/256][record_bytes(fmt)]
    int pair_sum = 0;     // as the second weight of a two-weight mat-vec launch: 1 = the two products are added (the two
                          // halves of a Q5_K weight), 0 = silu(first) * second (gate / up)

    __host__ __device__ const uint8_t *record(int rg, int st) const
    {
        return data + ((long long)rg * (k_pad >> 8) + st) * record_bytes(fmt);
    }
};

struct ActView
{
    int rows, rows_pad;  // rows_pad = multiple of 8
    int k, k_pad;
    const int8_t *q;     // [rows_pad][k_pad]
    const float2 *ds;    // [k_pad/32][rows_pad]
    const float *dx;     // [k_pad/32][rows_pad] d alone, and
    const float *sx;     // [k_pad/32][rows_pad] d * sum32(q) alone: the planes the tensor-core GEMM bulk-copies
    const float *gs;     // [rows_pad][k_pad/16]
    const int *isum;     // [rows_pad][k_pad/32]
    // Deferred quantization (mat-vec only): when raw is set, the planes above have not been written; the kernel reads the
    // rows themselves (f32 or bf16, raw_stride elements apart) and quantizes them into its shared memory.
    const void *raw = nullptr;
    int raw_dtype = 0;
    long long raw_stride = 0;
};

// What a MatMul adds to its result before the store, the elementwise tail the reference's lowering folds into the
// kernel (src/Sharplight.Shaders/Lowering/GraphLowerer.MatMul.cs:199-243: a bias row vector, then further adds such as
// the residual): y[t][n] = (dot + bias[n]) + residual[t][n], each an f32 add in that order, the same sums the
// stand-alone Add kernels would compute. Null pointers: nothing is added.
struct Epilogue
{
    const float *bias;          // [n]
    const float *residual;      // [rows][residual_stride], indexed like y
    long long residual_stride;
#ifdef __CUDACC__
    __device__ __forceinline__ float apply(float v, long long tok, int col) const
    {
        if (bias) v = __fadd_rn(v, bias[col]);
        if (residual) v = __fadd_rn(v, residual[tok * residual_stride + col]);
        return v;
    }
#endif
};

inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline size_t weight_bytes(int fmt, int n_pad, int k_pad)
{
    return (size_t)(n_pad / 16) * (k_pad / 256) * record_bytes(fmt);
}

// 128-bit read-only load that does not allocate in L1: weight bytes are used exactly once.
__device__ __forceinline__ uint4 ld_stream(const uint4 *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

}  // namespace slc
