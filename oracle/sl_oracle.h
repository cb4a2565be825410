/*
 * CPU oracle for Sharplight's quantized MatMul path. TEST INFRASTRUCTURE ONLY: it is the checker for the CUDA
 * kernels (tests, smoke check, the CPU-baseline leg of the benchmark) and is never linked into or called by
 * libsharplight_cuda.so or the host package.
 *
 * It restates, in plain C, the arithmetic of the reference's managed CPU provider (paths are relative to the
 * Sharplight source tree):
 *   - src/Sharplight.Cpu/Quant.cs            half decode, Q8_0 / Q4_0 / Q4_K / Q5_K / Q6_K / Q5_0 / IQ4_NL dequantization
 *   - src/Sharplight.Cpu/IntDot.cs           8-bit activation quantization (32-value blocks, 16-value group sums)
 *   - src/Sharplight.Cpu/IntDot.Decode.cs    weight rows -> unsigned codes u, multiplier a, offset b per 16 values
 *   - src/Sharplight.Cpu/IntDot.Kernels.cs   the scalar dot kernel (the specification of the float order)
 *   - src/Sharplight.Cpu/MatMulOp.cs         the integer-dot MatMul driver
 *
 * Parity pins: the dequantizers and decoders reproduce the ggml golden fixtures of the reference's own test suite
 * (tests/Sharplight.Cpu.Tests/Fixtures/ggml_quant_ext.bin and ggml_quant.bin, the records of ggml types 2, 6, 8, 12, 13, 14, 20);
 * the quantizer reproduces the analytic known-answer cases of IntDotTests.QuantizeMatchesReference. No reference test
 * stores int32 block dots or int-dot outputs, so those are pinned through this restatement.
 */
#ifndef SL_ORACLE_H
#define SL_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml type ids, as mapped by src/Sharplight.Import.Gguf/GgmlTypes.cs:51-92 */
enum { SLO_Q4_0 = 2, SLO_Q5_0 = 6, SLO_Q8_0 = 8, SLO_Q4_K = 12, SLO_Q5_K = 13, SLO_Q6_K = 14, SLO_IQ4_NL = 20 };

int slo_block_size(int fmt);   /* values per block, 0 if unknown */
int slo_block_bytes(int fmt);  /* bytes per block, 0 if unknown */

float slo_h2f(uint16_t h);

/* One row of k values -> f32. Returns 0, or -1 for a bad format / k. */
int slo_dequantize_row(int fmt, const uint8_t *src, int64_t k, float *dst);

/* One f32 row -> q[k] int8, d[k/32] block scales, gs[k/16] group sums d * sum16(q). */
void slo_quantize_row(const float *x, int64_t k, int8_t *q, float *d, float *gs);

/* One weight row -> u[k] codes, a[k/16], b[k/16] with value = a*u + b. Returns 0 or -1. */
int slo_decode_row(int fmt, const uint8_t *src, int64_t k, uint8_t *u, float *a, float *b);

/* The scalar dot kernel. */
float slo_dot_scalar(const uint8_t *u, const float *a, const float *b, const int8_t *q, const float *d,
                     const float *gs, int64_t k);

/* The same sum with every product and the accumulation in double (error-free reference for tolerances). */
double slo_dot_f64(const uint8_t *u, const float *a, const float *b, const int8_t *q, const float *d,
                   const float *gs, int64_t k);

/* s32[k/32]: exact integer dots of the unsigned codes with the activation codes, per 32-value block. */
void slo_block_dots(const uint8_t *u, const int8_t *q, int64_t k, int32_t *s32);

/*
 * y[m][n] = x[m][k] . W[n][k]^T on the integer-dot path, rows independent (any m). threads >= 1 worker threads
 * split the weight rows. tier: 0 = scalar kernel (the specification), 1 = fastest vector tier the host CPU
 * supports (same integers, different f32 summation order, as the reference's own tiers).
 * y64 (optional, may be NULL) receives the double-precision sums of the same integer-dot terms.
 * s32 (optional) receives the block dots as [m][n][k/32].
 * Returns 0 or -1.
 */
int slo_matmul_intdot(int fmt, const uint8_t *w, int64_t n, int64_t k, const float *x, int64_t m, float *y,
                      double *y64, int32_t *s32, int threads, int tier);

/* y64[m][n]: exact product of the dequantized weight with the unquantized f32 activations, in double. */
int slo_matmul_f64(int fmt, const uint8_t *w, int64_t n, int64_t k, const float *x, int64_t m, double *y64,
                   int threads);

/* The same MatMul driven the way the reference drives it: chunks = clamp(n / 16, 1, threads * 4) rows ranges handed to a
 * persistent spinning worker pool (src/Sharplight.Cpu/MatMulOp.cs:183, CpuParallel.cs:34-66, CpuThreadPool.cs:48-114). */
int slo_matmul_intdot_pooled(int fmt, const uint8_t *w, int64_t n, int64_t k, const float *x, int64_t m, float *y,
                             int threads, int tier);

/* The f32 GEMM path the reference's CPU provider takes from 32 activation rows (src/Sharplight.Cpu/MatMulOp.cs:218-369,
 * src/Sharplight.Cpu/Gemm.cs:16-60,210-330): weights dequantized per 256-value slice into packed panels, 8 x 32 AVX-512
 * micro-kernel (6 x 16 in plain C otherwise); every output is one chain of fused multiply-adds over k in order. */
int slo_matmul_gemm(int fmt, const uint8_t *w, int64_t n, int64_t k, const float *x, int64_t m, float *y, int threads);
const char *slo_gemm_tile_name(void);

/* MatMulOp.Run's row-count dispatch (src/Sharplight.Cpu/MatMulOp.cs:125-160): GEMM from 32 rows, integer dots below. */
int slo_matmul_run(int fmt, const uint8_t *w, int64_t n, int64_t k, const float *x, int64_t m, float *y, int threads);

/* Name of the vector tier slo_matmul_intdot(tier=1) uses on this host: "avx512vnni", "avx2" or "scalar". */
const char *slo_fast_tier_name(void);

#ifdef __cplusplus
}
#endif
#endif
