/*
 * CPU oracle for Sharplight's quantized MatMul path -- see sl_oracle.h. TEST INFRASTRUCTURE ONLY.
 * Build: oracle/Makefile (gcc -O2 -ffp-contract=off: every fused multiply-add below is an explicit fmaf, every
 * other float operation is a separately rounded IEEE single operation, as in the managed reference).
 */
#include "sl_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#if defined(__x86_64__)
#include <immintrin.h>
#endif

/* ---- formats: src/Sharplight.Core/Tensors/DataType.cs:102,110,116,120 ------------------------------------------- */

int slo_block_size(int fmt)
{
    switch (fmt) {
    case SLO_Q4_0: case SLO_Q8_0: case SLO_Q5_0: case SLO_IQ4_NL: return 32;
    case SLO_Q4_K: case SLO_Q5_K: case SLO_Q6_K: return 256;
    default: return 0;
    }
}

int slo_block_bytes(int fmt)
{
    switch (fmt) {
    case SLO_Q4_0: return 18;
    case SLO_Q5_0: return 22;
    case SLO_IQ4_NL: return 18;
    case SLO_Q8_0: return 34;
    case SLO_Q4_K: return 144;
    case SLO_Q5_K: return 176;
    case SLO_Q6_K: return 210;
    default: return 0;
    }
}

/* ---- half -> float: src/Sharplight.Cpu/Quant.cs:371-381 ------------------------------------------------------------ */

float slo_h2f(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = h & 0x7C00u;
    uint32_t m = h & 0x03FFu;
    uint32_t bits;
    if (e == 0) {
        if (m == 0) {
            bits = sign;
        } else { /* subnormal: value = m * 2^-24 */
            float f = (float)m * 5.9604644775390625e-8f;
            memcpy(&bits, &f, 4);
            bits |= sign;
        }
    } else if (e == 0x7C00u) {
        bits = sign | 0x7F800000u | (m << 13);
    } else {
        bits = sign | ((((uint32_t)h & 0x7FFFu) << 13) + 0x38000000u);
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

static float h_at(const uint8_t *p)
{
    return slo_h2f((uint16_t)(p[0] | (p[1] << 8)));
}

/* 6-bit scale / min of sub-block j of a Q4_K super-block: src/Sharplight.Cpu/Quant.cs:504-516 */
static void scale_min(int j, const uint8_t *s, int *sc, int *m)
{
    if (j < 4) {
        *sc = s[j] & 63;
        *m = s[j + 4] & 63;
    } else {
        *sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
        *m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

/* ---- dequantization, one FMA per value: src/Sharplight.Cpu/Quant.cs:384-405,519-545,585-618; Simd.cs:699-753 ------- */

/* the non-linear 4-bit codebook of IQ4_NL (ggml's kvalues_iq4nl; Quant.cs:409) */
static const int8_t iq4nl_values[16] = { -127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113 };

static void store16_u8(const uint8_t *v, float scale, float offset, float *dst)
{
    for (int i = 0; i < 16; i++) {
        dst[i] = fmaf((float)v[i], scale, offset);
    }
}

int slo_dequantize_row(int fmt, const uint8_t *p, int64_t k, float *dst)
{
    int bs = slo_block_size(fmt);
    if (bs == 0 || k < 0 || k % bs != 0) {
        return -1;
    }
    int64_t nb = k / bs;
    uint8_t v[16];
    switch (fmt) {
    case SLO_Q8_0:
        for (int64_t b = 0; b < nb; b++, p += 34, dst += 32) {
            float d = h_at(p);
            for (int i = 0; i < 32; i++) {
                dst[i] = fmaf((float)(int8_t)p[2 + i], d, 0.0f);
            }
        }
        return 0;
    case SLO_Q4_0:
        for (int64_t b = 0; b < nb; b++, p += 18, dst += 32) {
            float d = h_at(p);
            float off = -8.0f * d;
            for (int i = 0; i < 16; i++) v[i] = p[2 + i] & 15;
            store16_u8(v, d, off, dst);
            for (int i = 0; i < 16; i++) v[i] = p[2 + i] >> 4;
            store16_u8(v, d, off, dst + 16);
        }
        return 0;
    case SLO_Q5_0:
        /* Quant.cs:463-480: { f16 d; u32 qh; u8 qs[16] }, value j = (nibble | bit j of qh << 4) * d - 16 d (FMA form) */
        for (int64_t b = 0; b < nb; b++, p += 22, dst += 32) {
            float d = h_at(p);
            float off = -16.0f * d;
            uint32_t qh;
            memcpy(&qh, p + 2, 4);
            for (int i = 0; i < 16; i++) v[i] = (uint8_t)((p[6 + i] & 15) | (((qh >> i) & 1u) << 4));
            store16_u8(v, d, off, dst);
            for (int i = 0; i < 16; i++) v[i] = (uint8_t)((p[6 + i] >> 4) | (((qh >> (i + 16)) & 1u) << 4));
            store16_u8(v, d, off, dst + 16);
        }
        return 0;
    case SLO_IQ4_NL:
        /* Quant.cs:409-423: { f16 d; u8 qs[16] }, value = d * kvalues[nibble] (a plain product) */
        for (int64_t b = 0; b < nb; b++, p += 18, dst += 32) {
            float d = h_at(p);
            for (int i = 0; i < 16; i++) {
                dst[i] = d * (float)iq4nl_values[p[2 + i] & 15];
                dst[16 + i] = d * (float)iq4nl_values[p[2 + i] >> 4];
            }
        }
        return 0;
    case SLO_Q4_K:
        for (int64_t b = 0; b < nb; b++, p += 144, dst += 256) {
            float d = h_at(p), dmin = h_at(p + 2);
            const uint8_t *scales = p + 4, *qs = p + 16;
            for (int j = 0; j < 4; j++, qs += 32) {
                int sc1, m1, sc2, m2;
                scale_min(2 * j, scales, &sc1, &m1);
                scale_min(2 * j + 1, scales, &sc2, &m2);
                float d1 = d * (float)sc1, mm1 = dmin * (float)m1;
                float d2 = d * (float)sc2, mm2 = dmin * (float)m2;
                float *o = dst + 64 * j;
                for (int i = 0; i < 16; i++) v[i] = qs[i] & 15;
                store16_u8(v, d1, -mm1, o);
                for (int i = 0; i < 16; i++) v[i] = qs[16 + i] & 15;
                store16_u8(v, d1, -mm1, o + 16);
                for (int i = 0; i < 16; i++) v[i] = qs[i] >> 4;
                store16_u8(v, d2, -mm2, o + 32);
                for (int i = 0; i < 16; i++) v[i] = qs[16 + i] >> 4;
                store16_u8(v, d2, -mm2, o + 48);
            }
        }
        return 0;
    case SLO_Q5_K:
        /* Quant.cs:548-582: { f16 d; f16 dmin; u8 scales[12]; u8 qh[32]; u8 qs[128] }: Q4_K with a fifth bit per value,
           bit 2j (2j + 1) of qh[l] for value l of the low-nibble (high-nibble) sub-block of chunk j */
        for (int64_t b = 0; b < nb; b++, p += 176, dst += 256) {
            float d = h_at(p), dmin = h_at(p + 2);
            const uint8_t *scales = p + 4, *qh = p + 16, *qs = p + 48;
            for (int j = 0; j < 4; j++, qs += 32) {
                int sc1, m1, sc2, m2;
                scale_min(2 * j, scales, &sc1, &m1);
                scale_min(2 * j + 1, scales, &sc2, &m2);
                float d1 = d * (float)sc1, mm1 = dmin * (float)m1;
                float d2 = d * (float)sc2, mm2 = dmin * (float)m2;
                float *o = dst + 64 * j;
                for (int i = 0; i < 16; i++) v[i] = (uint8_t)((qs[i] & 15) | (((qh[i] >> (2 * j)) & 1) << 4));
                store16_u8(v, d1, -mm1, o);
                for (int i = 0; i < 16; i++) v[i] = (uint8_t)((qs[16 + i] & 15) | (((qh[16 + i] >> (2 * j)) & 1) << 4));
                store16_u8(v, d1, -mm1, o + 16);
                for (int i = 0; i < 16; i++) v[i] = (uint8_t)((qs[i] >> 4) | (((qh[i] >> (2 * j + 1)) & 1) << 4));
                store16_u8(v, d2, -mm2, o + 32);
                for (int i = 0; i < 16; i++) v[i] = (uint8_t)((qs[16 + i] >> 4) | (((qh[16 + i] >> (2 * j + 1)) & 1) << 4));
                store16_u8(v, d2, -mm2, o + 48);
            }
        }
        return 0;
    case SLO_Q6_K:
        for (int64_t b = 0; b < nb; b++, p += 210, dst += 256) {
            float d = h_at(p + 208);
            for (int n = 0; n < 2; n++) {
                const uint8_t *ql = p + 64 * n, *qh = p + 128 + 32 * n;
                const int8_t *sc = (const int8_t *)(p + 192) + 8 * n;
                float *o = dst + 128 * n;
                for (int h = 0; h < 2; h++) {
                    float s1 = d * (float)sc[h], s2 = d * (float)sc[h + 2];
                    float s3 = d * (float)sc[h + 4], s4 = d * (float)sc[h + 6];
                    const uint8_t *qa = ql + 16 * h, *qb = ql + 32 + 16 * h, *qq = qh + 16 * h;
                    for (int i = 0; i < 16; i++) v[i] = (uint8_t)((qa[i] & 15) | ((qq[i] & 3) << 4));
                    store16_u8(v, s1, -32.0f * s1, o + 16 * h);
                    for (int i = 0; i < 16; i++) v[i] = (uint8_t)((qb[i] & 15) | (((qq[i] >> 2) & 3) << 4));
                    store16_u8(v, s2, -32.0f * s2, o + 32 + 16 * h);
                    for (int i = 0; i < 16; i++) v[i] = (uint8_t)((qa[i] >> 4) | (((qq[i] >> 4) & 3) << 4));
                    store16_u8(v, s3, -32.0f * s3, o + 64 + 16 * h);
                    for (int i = 0; i < 16; i++) v[i] = (uint8_t)((qb[i] >> 4) | (((qq[i] >> 6) & 3) << 4));
                    store16_u8(v, s4, -32.0f * s4, o + 96 + 16 * h);
                }
            }
        }
        return 0;
    default:
        return -1;
    }
}

/* ---- activation quantization: src/Sharplight.Cpu/IntDot.cs:92-126 (QuantizeBlockScalar) ---------------------------- */

void slo_quantize_row(const float *x, int64_t k, int8_t *q, float *d_out, float *gs)
{
    for (int64_t b = 0; b < k; b += 32) {
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) {
            float ax = fabsf(x[b + i]);
            /* MathF.Max propagates NaN; inputs here are finite, fmaxf-free form keeps the comparison explicit */
            amax = ax > amax ? ax : amax;
        }
        float d = amax / 127.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        int s0 = 0, s1 = 0;
        for (int i = 0; i < 32; i++) {
            float v = x[b + i] * id;
            int r = (int)(v + copysignf(0.5f, v));
            q[b + i] = (int8_t)r;
            if (i < 16) s0 += r; else s1 += r;
        }
        d_out[b / 32] = d;
        gs[b / 16] = d * (float)s0;
        gs[b / 16 + 1] = d * (float)s1;
    }
}

/* ---- weight row decoders: src/Sharplight.Cpu/IntDot.Decode.cs:61-99,125-148,178-223 -------------------------------- */

static void set_block(float *a, float *b, float mul, float off)
{
    a[0] = mul; a[1] = mul; b[0] = off; b[1] = off;
}

int slo_decode_row(int fmt, const uint8_t *p, int64_t k, uint8_t *u, float *a, float *b)
{
    int bs = slo_block_size(fmt);
    if (bs == 0 || k < 0 || k % bs != 0) {
        return -1;
    }
    int64_t nb = k / bs;
    switch (fmt) {
    case SLO_Q8_0:
        for (int64_t blk = 0; blk < nb; blk++, p += 34, u += 32, a += 2, b += 2) {
            float d = h_at(p);
            for (int i = 0; i < 32; i++) u[i] = p[2 + i] ^ 0x80;
            set_block(a, b, d, -128.0f * d);
        }
        return 0;
    case SLO_Q4_0:
        for (int64_t blk = 0; blk < nb; blk++, p += 18, u += 32, a += 2, b += 2) {
            float d = h_at(p);
            for (int i = 0; i < 16; i++) {
                u[i] = p[2 + i] & 15;
                u[16 + i] = p[2 + i] >> 4;
            }
            set_block(a, b, d, -8.0f * d);
        }
        return 0;
    case SLO_Q5_0:
        /* IntDot.Decode.cs:101-123: u = the 5-bit code, a = d, b = -16 d */
        for (int64_t blk = 0; blk < nb; blk++, p += 22, u += 32, a += 2, b += 2) {
            float d = h_at(p);
            uint32_t qh;
            memcpy(&qh, p + 2, 4);
            for (int i = 0; i < 16; i++) {
                u[i] = (uint8_t)((p[6 + i] & 15) | (((qh >> i) & 1u) << 4));
                u[16 + i] = (uint8_t)((p[6 + i] >> 4) | (((qh >> (i + 16)) & 1u) << 4));
            }
            set_block(a, b, d, -16.0f * d);
        }
        return 0;
    case SLO_IQ4_NL:
        /* IntDot.Decode.cs:225-238: u = kvalues[nibble] + 128, a = d, b = -128 d */
        for (int64_t blk = 0; blk < nb; blk++, p += 18, u += 32, a += 2, b += 2) {
            float d = h_at(p);
            for (int i = 0; i < 16; i++) {
                u[i] = (uint8_t)(iq4nl_values[p[2 + i] & 15] + 128);
                u[16 + i] = (uint8_t)(iq4nl_values[p[2 + i] >> 4] + 128);
            }
            set_block(a, b, d, -128.0f * d);
        }
        return 0;
    case SLO_Q4_K:
        for (int64_t blk = 0; blk < nb; blk++, p += 144, u += 256, a += 16, b += 16) {
            float d = h_at(p), dmin = h_at(p + 2);
            const uint8_t *qs = p + 16;
            for (int j = 0; j < 4; j++) {
                uint8_t *uj = u + 64 * j;
                for (int i = 0; i < 32; i++) {
                    uj[i] = qs[32 * j + i] & 15;
                    uj[32 + i] = qs[32 * j + i] >> 4;
                }
            }
            for (int j = 0; j < 8; j++) {
                int sc, m;
                scale_min(j, p + 4, &sc, &m);
                set_block(a + 2 * j, b + 2 * j, d * (float)sc, -dmin * (float)m);
            }
        }
        return 0;
    case SLO_Q5_K:
        /* IntDot.Decode.cs:150-176: the 5-bit codes, a = d * sc, b = -dmin * m per 32-value sub-block */
        for (int64_t blk = 0; blk < nb; blk++, p += 176, u += 256, a += 16, b += 16) {
            float d = h_at(p), dmin = h_at(p + 2);
            const uint8_t *qh = p + 16, *qs = p + 48;
            for (int j = 0; j < 4; j++) {
                uint8_t *uj = u + 64 * j;
                for (int i = 0; i < 32; i++) {
                    uj[i] = (uint8_t)((qs[32 * j + i] & 15) | (((qh[i] >> (2 * j)) & 1) << 4));
                    uj[32 + i] = (uint8_t)((qs[32 * j + i] >> 4) | (((qh[i] >> (2 * j + 1)) & 1) << 4));
                }
            }
            for (int j = 0; j < 8; j++) {
                int sc, m;
                scale_min(j, p + 4, &sc, &m);
                set_block(a + 2 * j, b + 2 * j, d * (float)sc, -dmin * (float)m);
            }
        }
        return 0;
    case SLO_Q6_K:
        for (int64_t blk = 0; blk < nb; blk++, p += 210, u += 256, a += 16, b += 16) {
            float d = h_at(p + 208);
            for (int n = 0; n < 2; n++) {
                const uint8_t *ql = p + 64 * n, *qh = p + 128 + 32 * n;
                uint8_t *un = u + 128 * n;
                for (int l = 0; l < 32; l++) {
                    un[l] = (uint8_t)((ql[l] & 15) | ((qh[l] & 3) << 4));
                    un[32 + l] = (uint8_t)((ql[32 + l] & 15) | (((qh[l] >> 2) & 3) << 4));
                    un[64 + l] = (uint8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4));
                    un[96 + l] = (uint8_t)((ql[32 + l] >> 4) | (((qh[l] >> 6) & 3) << 4));
                }
            }
            const int8_t *sc = (const int8_t *)(p + 192);
            for (int g = 0; g < 16; g++) {
                float s = d * (float)sc[g];
                a[g] = s;
                b[g] = -32.0f * s;
            }
        }
        return 0;
    default:
        return -1;
    }
}

/* ---- dots: src/Sharplight.Cpu/IntDot.Kernels.cs:12-29 (DotScalar) --------------------------------------------------- */

float slo_dot_scalar(const uint8_t *u, const float *a, const float *b, const int8_t *q, const float *d,
                     const float *gs, int64_t k)
{
    float acc = 0.0f;
    for (int64_t g = 0; g < k / 16; g++) {
        int s = 0;
        for (int i = 0; i < 16; i++) {
            s += (int)u[g * 16 + i] * (int)q[g * 16 + i];
        }
        float t0 = a[g] * d[g / 2];
        t0 = t0 * (float)s;
        float t1 = b[g] * gs[g];
        acc = acc + (t0 + t1);
    }
    return acc;
}

double slo_dot_f64(const uint8_t *u, const float *a, const float *b, const int8_t *q, const float *d,
                   const float *gs, int64_t k)
{
    double acc = 0.0;
    for (int64_t g = 0; g < k / 16; g++) {
        int s = 0, sq = 0;
        for (int i = 0; i < 16; i++) {
            s += (int)u[g * 16 + i] * (int)q[g * 16 + i];
            sq += (int)q[g * 16 + i];
        }
        (void)gs;
        acc += (double)a[g] * (double)d[g / 2] * (double)s + (double)b[g] * ((double)d[g / 2] * (double)sq);
    }
    return acc;
}

void slo_block_dots(const uint8_t *u, const int8_t *q, int64_t k, int32_t *s32)
{
    for (int64_t blk = 0; blk < k / 32; blk++) {
        int s = 0;
        for (int i = 0; i < 32; i++) {
            s += (int)u[blk * 32 + i] * (int)q[blk * 32 + i];
        }
        s32[blk] = s;
    }
}

/* ---- vector tiers (same integers, different f32 order): src/Sharplight.Cpu/IntDot.Kernels.cs:101-121,200-269 -------- */

#if defined(__x86_64__)
/* lane scales: the block scale repeated once per four values (src/Sharplight.Cpu/Q8Row.cs:9-20) */
__attribute__((target("avx512f,avx512bw,avx512vl,avx512vnni,fma")))
static float dot_avx512vnni(const uint8_t *u, const float *a, const float *b, const int8_t *q,
                            const float *lane, const float *gs, int64_t k)
{
    __m512 acc0 = _mm512_setzero_ps(), acc1 = _mm512_setzero_ps();
    const __m512i spread = _mm512_setr_epi32(0, 0, 0, 0, 1, 1, 1, 1, 2, 2, 2, 2, 3, 3, 3, 3);
    int64_t i = 0;
    for (; i + 64 <= k; i += 64) {
        __m512i lanes = _mm512_dpbusd_epi32(_mm512_setzero_si512(), _mm512_loadu_si512(u + i),
                                            _mm512_loadu_si512(q + i));
        __m512 av = _mm512_permutexvar_ps(spread, _mm512_castps128_ps512(_mm_loadu_ps(a + i / 16)));
        __m512 scale = _mm512_mul_ps(av, _mm512_loadu_ps(lane + i / 4));
        if ((i & 64) == 0) acc0 = _mm512_fmadd_ps(_mm512_cvtepi32_ps(lanes), scale, acc0);
        else acc1 = _mm512_fmadd_ps(_mm512_cvtepi32_ps(lanes), scale, acc1);
    }
    float tail = 0.0f;
    if (i < k) { /* 32 values left */
        __m256i lanes = _mm256_dpbusd_epi32(_mm256_setzero_si256(), _mm256_loadu_si256((const __m256i *)(u + i)),
                                            _mm256_loadu_si256((const __m256i *)(q + i)));
        __m256 av = _mm256_set_m128(_mm_set1_ps(a[i / 16 + 1]), _mm_set1_ps(a[i / 16]));
        __m256 t = _mm256_mul_ps(_mm256_cvtepi32_ps(lanes), _mm256_mul_ps(av, _mm256_loadu_ps(lane + i / 4)));
        float tmp[8];
        _mm256_storeu_ps(tmp, t);
        for (int j = 0; j < 8; j++) tail += tmp[j];
    }
    float s = _mm512_reduce_add_ps(_mm512_add_ps(acc0, acc1)) + tail;
    __m512 off = _mm512_setzero_ps();
    int64_t groups = k / 16, g = 0;
    for (; g + 16 <= groups; g += 16) {
        off = _mm512_fmadd_ps(_mm512_loadu_ps(b + g), _mm512_loadu_ps(gs + g), off);
    }
    float o = _mm512_reduce_add_ps(off);
    for (; g < groups; g++) o += b[g] * gs[g];
    return s + o;
}

__attribute__((target("avx2,fma")))
static float dot_avx2(const uint8_t *u, const float *a, const float *b, const int8_t *q, const float *lane,
                      const float *gs, int64_t k)
{
    /* codes may use the full 0..255 range: |w| * sign(q, w) with w = u - 128 keeps vpmaddubsw exact, and moves
       128 * a into the offset term (src/Sharplight.Cpu/IntDot.Kernels.cs:76-121) */
    __m256 acc = _mm256_setzero_ps();
    const __m256i ones = _mm256_set1_epi16(1), flip = _mm256_set1_epi8((char)0x80);
    for (int64_t i = 0; i + 32 <= k; i += 32) {
        __m256i w = _mm256_xor_si256(_mm256_loadu_si256((const __m256i *)(u + i)), flip);
        __m256i qv = _mm256_loadu_si256((const __m256i *)(q + i));
        __m256i pairs = _mm256_maddubs_epi16(_mm256_abs_epi8(w), _mm256_sign_epi8(qv, w));
        __m256i lanes = _mm256_madd_epi16(pairs, ones);
        __m256 av = _mm256_set_m128(_mm_set1_ps(a[i / 16 + 1]), _mm_set1_ps(a[i / 16]));
        acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(lanes), _mm256_mul_ps(av, _mm256_loadu_ps(lane + i / 4)), acc);
    }
    float tmp[8], s = 0.0f;
    _mm256_storeu_ps(tmp, acc);
    for (int j = 0; j < 8; j++) s += tmp[j];
    float o = 0.0f;
    for (int64_t g = 0; g < k / 16; g++) o += (b[g] + 128.0f * a[g]) * gs[g];
    return s + o;
}
#endif

static int fast_tier(void)
{
#if defined(__x86_64__)
    static int tier = -1;
    if (tier < 0) {
        __builtin_cpu_init();
        if (__builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512bw") &&
            __builtin_cpu_supports("avx512vl")) tier = 2;
        else if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) tier = 1;
        else tier = 0;
    }
    return tier;
#else
    return 0;
#endif
}

const char *slo_fast_tier_name(void)
{
    switch (fast_tier()) {
    case 2: return "avx512vnni";
    case 1: return "avx2";
    default: return "scalar";
    }
}

/* ---- MatMul drivers: src/Sharplight.Cpu/MatMulOp.cs:174-213 (RunIntDot / IntDotBody) -------------------------------- */

static int64_t align64(int64_t v) { return (v + 63) & ~(int64_t)63; }

typedef struct {
    int fmt, tier;
    const uint8_t *w;
    int64_t n, k, m, n0, n1;
    const int8_t *q;    /* [m][k] */
    const float *d;     /* [m][k/32] */
    const float *lane;  /* [m][k/4] */
    const float *gs;    /* [m][k/16] */
    float *y;
    double *y64;
    int32_t *s32;
} intdot_job;

static void *intdot_worker(void *arg)
{
    intdot_job *j = (intdot_job *)arg;
    int64_t k = j->k, groups = k / 16;
    int64_t row_bytes = k / slo_block_size(j->fmt) * slo_block_bytes(j->fmt);
    uint8_t *u = (uint8_t *)aligned_alloc(64, (size_t)align64(k));
    float *a = (float *)aligned_alloc(64, (size_t)align64(groups * 4));
    float *b = (float *)aligned_alloc(64, (size_t)align64(groups * 4));
    for (int64_t n = j->n0; n < j->n1; n++) {
        slo_decode_row(j->fmt, j->w + n * row_bytes, k, u, a, b);
        for (int64_t t = 0; t < j->m; t++) {
            const int8_t *q = j->q + t * k;
            const float *d = j->d + t * (k / 32), *gs = j->gs + t * groups, *lane = j->lane + t * (k / 4);
            float r;
#if defined(__x86_64__)
            if (j->tier == 2) r = dot_avx512vnni(u, a, b, q, lane, gs, k);
            else if (j->tier == 1) r = dot_avx2(u, a, b, q, lane, gs, k);
            else
#endif
                r = slo_dot_scalar(u, a, b, q, d, gs, k);
            j->y[t * j->n + n] = r;
            if (j->y64) j->y64[t * j->n + n] = slo_dot_f64(u, a, b, q, d, gs, k);
            if (j->s32) slo_block_dots(u, q, k, j->s32 + (t * j->n + n) * (k / 32));
        }
    }
    free(u); free(a); free(b);
    return NULL;
}

int slo_matmul_intdot(int fmt, const uint8_t *w, int64_t n, int64_t k, const float *x, int64_t m, float *y,
                      double *y64, int32_t *s32, int threads, int tier)
{
    int bs = slo_block_size(fmt);
    if (bs == 0 || k <= 0 || k % bs != 0 || n < 0 || m < 0) {
        return -1;
    }
    if (n == 0 || m == 0) {
        return 0;
    }
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    int8_t *q = (int8_t *)aligned_alloc(64, (size_t)align64(m * k));
    float *d = (float *)aligned_alloc(64, (size_t)align64(m * (k / 32) * 4));
    float *gs = (float *)aligned_alloc(64, (size_t)align64(m * (k / 16) * 4));
    float *lane = (float *)aligned_alloc(64, (size_t)align64(m * (k / 4) * 4));
    for (int64_t t = 0; t < m; t++) {
        slo_quantize_row(x + t * k, k, q + t * k, d + t * (k / 32), gs + t * (k / 16));
        for (int64_t i = 0; i < k / 4; i++) lane[t * (k / 4) + i] = d[t * (k / 32) + i / 8];
    }
    intdot_job jobs[256];
    pthread_t tid[256];
    int64_t per = (n + threads - 1) / threads;
    int used = 0;
    for (int i = 0; i < threads; i++) {
        int64_t n0 = i * per, n1 = n0 + per < n ? n0 + per : n;
        if (n0 >= n1) break;
        intdot_job jb = { fmt, tier ? fast_tier() : 0, w, n, k, m, n0, n1, q, d, lane, gs, y, y64, s32 };
        jobs[used++] = jb;
    }
    for (int i = 1; i < used; i++) pthread_create(&tid[i], NULL, intdot_worker, &jobs[i]);
    intdot_worker(&jobs[0]);
    for (int i = 1; i < used; i++) pthread_join(tid[i], NULL);
    free(q); free(d); free(gs); free(lane);
    return 0;
}

typedef struct {
    int fmt;
    const uint8_t *w;
    int64_t n, k, m, n0, n1;
    const float *x;
    double *y64;
} f64_job;

static void *f64_worker(void *arg)
{
    f64_job *j = (f64_job *)arg;
    int64_t k = j->k;
    int64_t row_bytes = k / slo_block_size(j->fmt) * slo_block_bytes(j->fmt);
    float *wrow = (float *)malloc((size_t)k * 4);
    for (int64_t n = j->n0; n < j->n1; n++) {
        slo_dequantize_row(j->fmt, j->w + n * row_bytes, k, wrow);
        for (int64_t t = 0; t < j->m; t++) {
            double acc = 0.0;
            const float *x = j->x + t * k;
            for (int64_t i = 0; i < k; i++) acc += (double)wrow[i] * (double)x[i];
            j->y64[t * j->n + n] = acc;
        }
    }
    free(wrow);
    return NULL;
}

int slo_matmul_f64(int fmt, const uint8_t *w, int64_t n, int64_t k, const float *x, int64_t m, double *y64,
                   int threads)
{
    int bs = slo_block_size(fmt);
    if (bs == 0 || k <= 0 || k % bs != 0 || n < 0 || m < 0) {
        return -1;
    }
    if (n == 0 || m == 0) {
        return 0;
    }
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    f64_job jobs[256];
    pthread_t tid[256];
    int64_t per = (n + threads - 1) / threads;
    int used = 0;
    for (int i = 0; i < threads; i++) {
        int64_t n0 = i * per, n1 = n0 + per < n ? n0 + per : n;
        if (n0 >= n1) break;
        f64_job jb = { fmt, w, n, k, m, n0, n1, x, y64 };
        jobs[used++] = jb;
    }
    for (int i = 1; i < used; i++) pthread_create(&tid[i], NULL, f64_worker, &jobs[i]);
    f64_worker(&jobs[0]);
    for (int i = 1; i < used; i++) pthread_join(tid[i], NULL);
    return 0;
}

/* ---- parallel loops: the reference's CpuParallel.For over its spinning pool ------------------------------------------
 * src/Sharplight.Cpu/CpuParallel.cs:34-66 (For), CpuThreadPool.cs:48-114 (persistent workers that spin for a while after
 * the last job, then block), CpuThreadJob.cs:14-95 (one contiguous range of items per participant, the caller being
 * participant 0; own range first, then the others'; items claimed count / (participants * 8) at a time). */

#include <stdatomic.h>
#include <time.h>

typedef void (*slo_body)(int item, void *ctx);

#define POOL_MAX 256
#define POOL_STRIDE 16   /* longs between two counters: 128 bytes */

typedef struct {
    slo_body body;
    void *ctx;
    int count, participants, ranges, batch;
    _Atomic long counters[(POOL_MAX + 2) * POOL_STRIDE];   /* [(r + 1) * stride]: next item of range r; last: items done */
} pool_job;

static struct {
    pthread_mutex_t gate;
    pthread_cond_t wake;
    pthread_t tid[POOL_MAX];
    int workers;
    _Atomic long generation;
    pool_job *_Atomic job;
    pthread_mutex_t busy;
    int ready;
} g_pool = { PTHREAD_MUTEX_INITIALIZER, PTHREAD_COND_INITIALIZER, {0}, 0, 0, NULL, PTHREAD_MUTEX_INITIALIZER, 0 };

static long range_start(const pool_job *j, int r) { return (long)j->count * r / j->ranges; }

static void job_work(pool_job *j, int participant)
{
    int own = participant % j->ranges;
    for (int k = 0; k < j->ranges; k++) {
        int r = (own + k) % j->ranges;
        long end = range_start(j, r + 1);
        _Atomic long *next = &j->counters[(r + 1) * POOL_STRIDE];
        long start;
        while (atomic_load(next) < end && (start = atomic_fetch_add(next, j->batch)) < end) {
            long stop = start + j->batch < end ? start + j->batch : end;
            for (long i = start; i < stop; i++) j->body((int)i, j->ctx);
            atomic_fetch_add(&j->counters[(j->ranges + 1) * POOL_STRIDE], stop - start);
        }
    }
}

static double now_s(void)
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec + 1e-9 * ts.tv_nsec;
}

static void *pool_worker(void *arg)
{
    int id = (int)(intptr_t)arg;
    long seen = 0;
    for (;;) {
        /* spin for a while after the last job, then block until the generation changes */
        double start = now_s();
        int checks = 0;
        long gen;
        for (;;) {
            gen = atomic_load(&g_pool.generation);
            if (gen != seen) break;
            for (volatile int s = 0; s < 16; s++) { }
            if (++checks % 64 == 0 && now_s() - start > 2e-3) {
                pthread_mutex_lock(&g_pool.gate);
                while ((gen = atomic_load(&g_pool.generation)) == seen) pthread_cond_wait(&g_pool.wake, &g_pool.gate);
                pthread_mutex_unlock(&g_pool.gate);
                break;
            }
        }
        seen = gen;
        pool_job *j = atomic_load(&g_pool.job);
        if (j && id < j->participants) job_work(j, id + 1);
    }
    return NULL;
}

/* body(0 .. count-1) on the caller and up to threads - 1 pool workers. Not reentrant: callers serialize. */
static void pool_for(int count, int threads, slo_body body, void *ctx)
{
    if (count <= 0) return;
    if (threads > POOL_MAX) threads = POOL_MAX;
    if (count == 1 || threads <= 1) {
        for (int i = 0; i < count; i++) body(i, ctx);
        return;
    }
    pthread_mutex_lock(&g_pool.busy);
    while (g_pool.workers < threads - 1) {
        pthread_create(&g_pool.tid[g_pool.workers], NULL, pool_worker, (void *)(intptr_t)g_pool.workers);
        pthread_detach(g_pool.tid[g_pool.workers]);
        g_pool.workers++;
    }
    int helpers = (count < threads ? count : threads) - 1;
    static pool_job job;   /* one job at a time (busy lock) */
    job.body = body; job.ctx = ctx; job.count = count; job.participants = helpers;
    job.ranges = count < helpers + 1 ? count : helpers + 1;
    if (job.ranges < 1) job.ranges = 1;
    job.batch = count / ((helpers + 1) * 8);
    if (job.batch < 1) job.batch = 1;
    for (int r = 0; r < job.ranges; r++) atomic_store(&job.counters[(r + 1) * POOL_STRIDE], range_start(&job, r));
    atomic_store(&job.counters[(job.ranges + 1) * POOL_STRIDE], 0);
    pthread_mutex_lock(&g_pool.gate);
    atomic_store(&g_pool.job, &job);
    atomic_fetch_add(&g_pool.generation, 1);
    pthread_cond_broadcast(&g_pool.wake);
    pthread_mutex_unlock(&g_pool.gate);
    job_work(&job, 0);
    while (atomic_load(&job.counters[(job.ranges + 1) * POOL_STRIDE]) < count) { }
    /* a worker that woke late may still look at the job: it finds every range exhausted and touches nothing else */
    pthread_mutex_unlock(&g_pool.busy);
}

/* ---- the integer-dot driver with the reference's chunking (MatMulOp.RunIntDot, src/Sharplight.Cpu/MatMulOp.cs:174-213):
 * chunks = clamp(N / 16, 1, threads * 4), rows per chunk = ceil(N / chunks), one pool item per chunk. */

typedef struct {
    intdot_job base;
    int64_t per_chunk;
} intdot_chunks;

static void intdot_chunk_body(int c, void *ctx)
{
    intdot_chunks *jc = (intdot_chunks *)ctx;
    intdot_job jb = jc->base;
    jb.n0 = c * jc->per_chunk;
    jb.n1 = jb.n0 + jc->per_chunk < jb.n ? jb.n0 + jc->per_chunk : jb.n;
    if (jb.n0 < jb.n1) intdot_worker(&jb);
}

int slo_matmul_intdot_pooled(int fmt, const uint8_t *w, int64_t n, int64_t k, const float *x, int64_t m, float *y,
                             int threads, int tier)
{
    int bs = slo_block_size(fmt);
    if (bs == 0 || k <= 0 || k % bs != 0 || n < 0 || m < 0) return -1;
    if (n == 0 || m == 0) return 0;
    if (threads < 1) threads = 1;
    if (threads > POOL_MAX) threads = POOL_MAX;
    int8_t *q = (int8_t *)aligned_alloc(64, (size_t)align64(m * k));
    float *d = (float *)aligned_alloc(64, (size_t)align64(m * (k / 32) * 4));
    float *gs = (float *)aligned_alloc(64, (size_t)align64(m * (k / 16) * 4));
    float *lane = (float *)aligned_alloc(64, (size_t)align64(m * (k / 4) * 4));
    for (int64_t t = 0; t < m; t++) {
        slo_quantize_row(x + t * k, k, q + t * k, d + t * (k / 32), gs + t * (k / 16));
        for (int64_t i = 0; i < k / 4; i++) lane[t * (k / 4) + i] = d[t * (k / 32) + i / 8];
    }
    int64_t chunks = n / 16;
    if (chunks < 1) chunks = 1;
    if (chunks > (int64_t)threads * 4) chunks = (int64_t)threads * 4;
    intdot_chunks jc = { { fmt, tier ? fast_tier() : 0, w, n, k, m, 0, 0, q, d, lane, gs, y, NULL, NULL }, (n + chunks - 1) / chunks };
    pool_for((int)chunks, threads, intdot_chunk_body, &jc);
    free(q); free(d); free(gs); free(lane);
    return 0;
}

/* ---- the f32 GEMM path the reference takes from 32 rows (MatMulOp.RunGemm / PackBody / GemmBody,
 * src/Sharplight.Cpu/MatMulOp.cs:218-369; micro-kernel Gemm.K8x32, src/Sharplight.Cpu/Gemm.cs:16-33,210-330):
 * activations packed as [K][MR] tiles; per task (panel of NR weight rows x block of row tiles): for every KC = 256 slice,
 * dequantize the panel's rows into B[k][NR], then run the MR x NR micro-kernel over the block's tiles, accumulating in y.
 * Every output element is one chain of fused multiply-adds over k in order, whatever the tile shape. */

enum { GEMM_KC = 256 };

typedef struct {
    int fmt, mr, nr;
    const uint8_t *w;
    int64_t n, k, m;
    const float *x;
    float *y, *apack;
    int m_tiles, panels, m_blocks, tiles_per_block;
} gemm_job;

static void gemm_pack_body(int tile, void *ctx)
{
    gemm_job *j = (gemm_job *)ctx;
    int mr = j->mr;
    int64_t r0 = (int64_t)tile * mr;
    int rows = j->m - r0 < mr ? (int)(j->m - r0) : mr;
    float *dst = j->apack + (int64_t)tile * j->k * mr;
    for (int64_t k = 0; k < j->k; k++)
        for (int i = 0; i < mr; i++) dst[k * mr + i] = i < rows ? j->x[(r0 + i) * j->k + k] : 0.0f;
}

static void tile_generic(const float *a, const float *b, int ldb, float *c, int64_t ldc, int kc, int acc, int mr, int nr)
{
    float t[8 * 32];
    for (int i = 0; i < mr; i++)
        for (int jn = 0; jn < nr; jn++) t[i * nr + jn] = acc ? c[i * ldc + jn] : 0.0f;
    for (int k = 0; k < kc; k++)
        for (int i = 0; i < mr; i++)
            for (int jn = 0; jn < nr; jn++) t[i * nr + jn] = fmaf(a[k * mr + i], b[k * ldb + jn], t[i * nr + jn]);
    for (int i = 0; i < mr; i++)
        for (int jn = 0; jn < nr; jn++) c[i * ldc + jn] = t[i * nr + jn];
}

#if defined(__x86_64__)
#include <immintrin.h>
__attribute__((target("avx512f,fma")))
static void tile_8x32(const float *a, const float *b, int ldb, float *c, int64_t ldc, int kc, int acc)
{
    __m512 c0[8], c1[8];
    for (int i = 0; i < 8; i++) {
        c0[i] = acc ? _mm512_loadu_ps(c + i * ldc) : _mm512_setzero_ps();
        c1[i] = acc ? _mm512_loadu_ps(c + i * ldc + 16) : _mm512_setzero_ps();
    }
    for (int k = 0; k < kc; k++) {
        __m512 b0 = _mm512_loadu_ps(b), b1 = _mm512_loadu_ps(b + 16);
        for (int i = 0; i < 8; i++) {
            __m512 ai = _mm512_set1_ps(a[i]);
            c0[i] = _mm512_fmadd_ps(ai, b0, c0[i]);
            c1[i] = _mm512_fmadd_ps(ai, b1, c1[i]);
        }
        a += 8;
        b += ldb;
    }
    for (int i = 0; i < 8; i++) {
        _mm512_storeu_ps(c + i * ldc, c0[i]);
        _mm512_storeu_ps(c + i * ldc + 16, c1[i]);
    }
}
static int have_avx512(void) { return __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("fma"); }
#else
static int have_avx512(void) { return 0; }
#endif

static void gemm_tile(const gemm_job *j, const float *a, const float *b, float *c, int kc, int acc, int rows, int cols)
{
    int mr = j->mr, nr = j->nr;
    if (rows == mr && cols == nr) {
#if defined(__x86_64__)
        if (mr == 8 && nr == 32) { tile_8x32(a, b, nr, c, j->n, kc, acc); return; }
#endif
        tile_generic(a, b, nr, c, j->n, kc, acc, mr, nr);
        return;
    }
    /* partial tile: through a scratch tile, valid part copied (Gemm.TileEdge, Gemm.cs:87-111) */
    float tmp[8 * 32];
    for (int i = 0; i < mr; i++)
        for (int jn = 0; jn < nr; jn++) tmp[i * nr + jn] = (acc && i < rows && jn < cols) ? c[i * j->n + jn] : 0.0f;
#if defined(__x86_64__)
    if (mr == 8 && nr == 32) tile_8x32(a, b, nr, tmp, nr, kc, acc);
    else
#endif
        tile_generic(a, b, nr, tmp, nr, kc, acc, mr, nr);
    for (int i = 0; i < rows; i++)
        for (int jn = 0; jn < cols; jn++) c[i * j->n + jn] = tmp[i * nr + jn];
}

static void gemm_body(int task, void *ctx)
{
    gemm_job *j = (gemm_job *)ctx;
    int mr = j->mr, nr = j->nr;
    int panel = task % j->panels, block = task / j->panels;
    int t0 = block * j->tiles_per_block, t1 = t0 + j->tiles_per_block < j->m_tiles ? t0 + j->tiles_per_block : j->m_tiles;
    if (t0 >= t1) return;
    int64_t n0 = (int64_t)panel * nr;
    int cols = j->n - n0 < nr ? (int)(j->n - n0) : nr;
    float *bpack = (float *)aligned_alloc(64, (size_t)align64(((int64_t)GEMM_KC * nr + GEMM_KC) * 4));
    float *row = bpack + (int64_t)GEMM_KC * nr;
    int bs = slo_block_size(j->fmt), bb = slo_block_bytes(j->fmt);
    int64_t row_bytes = j->k / bs * bb;
    for (int64_t kb = 0; kb < j->k; kb += GEMM_KC) {
        int kc = j->k - kb < GEMM_KC ? (int)(j->k - kb) : GEMM_KC;
        for (int jn = 0; jn < nr; jn++) {
            if (jn < cols) {
                slo_dequantize_row(j->fmt, j->w + (n0 + jn) * row_bytes + kb / bs * bb, kc, row);
                for (int k = 0; k < kc; k++) bpack[k * nr + jn] = row[k];
            } else {
                for (int k = 0; k < kc; k++) bpack[k * nr + jn] = 0.0f;
            }
        }
        for (int t = t0; t < t1; t++) {
            const float *a = j->apack + ((int64_t)t * j->k + kb) * mr;
            float *c = j->y + (int64_t)t * mr * j->n + n0;
            int rows = j->m - (int64_t)t * mr < mr ? (int)(j->m - (int64_t)t * mr) : mr;
            gemm_tile(j, a, bpack, c, kc, kb > 0, rows, cols);
        }
    }
    free(bpack);
}

int slo_matmul_gemm(int fmt, const uint8_t *w, int64_t n, int64_t k, const float *x, int64_t m, float *y, int threads)
{
    int bs = slo_block_size(fmt);
    if (bs == 0 || k <= 0 || k % bs != 0 || n < 0 || m < 0) return -1;
    if (n == 0 || m == 0) return 0;
    if (threads < 1) threads = 1;
    if (threads > POOL_MAX) threads = POOL_MAX;
    gemm_job j;
    j.fmt = fmt; j.w = w; j.n = n; j.k = k; j.m = m; j.x = x; j.y = y;
    j.mr = have_avx512() ? 8 : 6;
    j.nr = have_avx512() ? 32 : 16;
    j.m_tiles = (int)((m + j.mr - 1) / j.mr);
    j.apack = (float *)aligned_alloc(64, (size_t)align64((int64_t)j.m_tiles * k * j.mr * 4));
    pool_for(j.m_tiles, threads, gemm_pack_body, &j);
    /* split the rows into blocks only as far as needed to give every thread work: each block dequantizes the weights again */
    j.panels = (int)((n + j.nr - 1) / j.nr);
    j.m_blocks = 1;
    while ((int64_t)j.panels * j.m_blocks < 2LL * threads && j.m_tiles / (j.m_blocks * 2) >= 4) j.m_blocks *= 2;
    j.tiles_per_block = (j.m_tiles + j.m_blocks - 1) / j.m_blocks;
    pool_for(j.panels * j.m_blocks, threads, gemm_body, &j);
    free(j.apack);
    return 0;
}

const char *slo_gemm_tile_name(void) { return have_avx512() ? "8x32 avx512" : "6x16 generic"; }

/* The reference's MatMulOp.Run dispatch for a quantized weight with integer dots enabled (MatMulOp.cs:125-160): the f32
 * GEMM from 32 rows, the integer-dot path below. */
int slo_matmul_run(int fmt, const uint8_t *w, int64_t n, int64_t k, const float *x, int64_t m, float *y, int threads)
{
    if (m >= 32) return slo_matmul_gemm(fmt, w, n, k, x, m, y, threads);
    return slo_matmul_intdot_pooled(fmt, w, n, k, x, m, y, threads, 1);
}
