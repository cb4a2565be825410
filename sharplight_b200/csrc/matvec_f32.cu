// Dequant-fused f32 mat-vec: the MatMul for nodes that keep f32 activation math (the reference's f32-activations
// attribute, src/Sharplight.Core/Graph/StandardOps.cs:130-135; GPU form src/Sharplight.Shaders/Kernels/matmul.slang:148-226
// of the Sharplight tree). Nothing is quantized on the activation side: y[t][n] = sum_k w[n][k] * x[t][k] in f32, with
// w = a * code + b per group of values, a and b pre-rounded f32 as the reference dequantizes
// (src/Sharplight.Cpu/Quant.cs:384-405,519-545,585-618): Q8_0 a = d, b = 0; Q4_0 a = d, b = -8 d; Q4_K a = d * sc_j,
// b = -(dmin * m_j); Q6_K a = d * sc_g, b = -32 a. A lane accumulates sum(code * x) and sum(x) per group and applies
// (a, b) once per group: one multiply-add per weight value and activation row.
//
// Shape: one CTA owns 16 weight rows (a row group of the record layout, layout.cuh); its 8 warps split K in 256-value
// super-tiles and read their records straight from global memory (each byte once, 128-bit loads that do not allocate in
// L1); the activation rows (1..4, f32) sit in shared memory. HBM-bound like the int8 mat-vec; the CUDA cores have about
// three operations per weight value to issue at one row.
#include "internal.cuh"

namespace slc {

constexpr int F32V_WARPS = 8;
constexpr int F32V_MAX_SMEM = 200 * 1024;

__device__ __forceinline__ float f32v_h2f(unsigned bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

// sum over j of byte j of `codes` (as given: signed or unsigned 8 bit) times xs[j], and the sum of the xs
template <bool SIGNED>
__device__ __forceinline__ void f32v_dot4(unsigned codes, const float *xs, float &su, float &sx)
{
    const float4 x = *reinterpret_cast<const float4 *>(xs);
    float c0, c1, c2, c3;
    if (SIGNED) {
        c0 = (float)(int)(signed char)(codes & 0xff); c1 = (float)(int)(signed char)((codes >> 8) & 0xff);
        c2 = (float)(int)(signed char)((codes >> 16) & 0xff); c3 = (float)(int)(signed char)(codes >> 24);
    } else {
        c0 = (float)(codes & 0xff); c1 = (float)((codes >> 8) & 0xff); c2 = (float)((codes >> 16) & 0xff); c3 = (float)(codes >> 24);
    }
    su = fmaf(c0, x.x, su); su = fmaf(c1, x.y, su); su = fmaf(c2, x.z, su); su = fmaf(c3, x.w, su);
    sx += (x.x + x.y) + (x.z + x.w);
}

// One record (16 rows x 256 values) of this lane: acc[m][r] += sum over the lane's values of w * x, r = rows g, g + 8.
template <int FMT, int M>
__device__ __forceinline__ void f32v_record(const uint8_t *rec, int lane, const float *xs, int x_row, float (&acc)[M][2])
{
    const int g = lane >> 2, t = lane & 3;
    const uint4 *tiles = reinterpret_cast<const uint4 *>(rec);
    const uint4 *hdr = reinterpret_cast<const uint4 *>(rec + code_bytes(FMT));
    if constexpr (FMT == FMT_Q8_0 || FMT == FMT_Q4_0) {
        // f16 d of the row's 8 blocks
        const uint4 h0 = hdr[g], h1 = hdr[g + 8];
        const unsigned d0w[4] = { h0.x, h0.y, h0.z, h0.w }, d1w[4] = { h1.x, h1.y, h1.z, h1.w };
#pragma unroll
        for (int blk = 0; blk < 8; blk++) {
            const float d[2] = { f32v_h2f((d0w[blk >> 1] >> (16 * (blk & 1))) & 0xffffu), f32v_h2f((d1w[blk >> 1] >> (16 * (blk & 1))) & 0xffffu) };
            unsigned c[2][2];   // [row][word]
            int koff[2];        // K offset of each word's four values inside the block
            if constexpr (FMT == FMT_Q8_0) {
                const uint4 q = ld_stream(tiles + blk * 32 + lane);          // q[8t..8t+7] of rows g (x, y) and g + 8 (z, w)
                c[0][0] = q.x; c[0][1] = q.y; c[1][0] = q.z; c[1][1] = q.w;
                koff[0] = 8 * t; koff[1] = 8 * t + 4;
            } else {
                // tile blk / 2: x = row g block 2i, y = row g+8 block 2i, z = row g block 2i+1, w = row g+8 block 2i+1;
                // low nibbles are values 4t.., high nibbles values 16 + 4t..
                const uint4 q = ld_stream(tiles + (blk >> 1) * 32 + lane);
                const unsigned w0 = (blk & 1) ? q.z : q.x, w1 = (blk & 1) ? q.w : q.y;
                c[0][0] = w0 & 0x0F0F0F0Fu; c[0][1] = (w0 >> 4) & 0x0F0F0F0Fu;
                c[1][0] = w1 & 0x0F0F0F0Fu; c[1][1] = (w1 >> 4) & 0x0F0F0F0Fu;
                koff[0] = 4 * t; koff[1] = 16 + 4 * t;
            }
#pragma unroll
            for (int m = 0; m < M; m++) {
                const float *xb = xs + m * x_row + blk * 32;
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    float su = 0.f, sx = 0.f;
                    f32v_dot4<FMT == FMT_Q8_0>(c[r][0], xb + koff[0], su, sx);
                    f32v_dot4<FMT == FMT_Q8_0>(c[r][1], xb + koff[1], su, sx);
                    acc[m][r] += FMT == FMT_Q8_0 ? d[r] * su : fmaf(d[r], su, (-8.0f * d[r]) * sx);
                }
            }
        }
    } else if constexpr (FMT == FMT_Q4_K) {
        const uint4 h[2] = { hdr[g], hdr[g + 8] };
        float d[2], dmin[2];
        unsigned sc_lo[2], sc_hi[2], mn_lo[2], mn_hi[2];   // 6-bit scales / mins of sub-blocks 0-3 and 4-7, one byte each
#pragma unroll
        for (int r = 0; r < 2; r++) {
            d[r] = f32v_h2f(h[r].x & 0xffffu);
            dmin[r] = f32v_h2f(h[r].x >> 16);
            sc_lo[r] = h[r].y & 0x3F3F3F3Fu;
            sc_hi[r] = (h[r].w & 0x0F0F0F0Fu) | ((h[r].y >> 2) & 0x30303030u);
            mn_lo[r] = h[r].z & 0x3F3F3F3Fu;
            mn_hi[r] = ((h[r].w >> 4) & 0x0F0F0F0Fu) | ((h[r].z >> 2) & 0x30303030u);
        }
#pragma unroll
        for (int c = 0; c < 4; c++) {
            // tile c: qs[32c + 8t .. +7] of rows g (x, y) and g + 8 (z, w); low nibbles sub-block 2c, high 2c + 1
            const uint4 q = ld_stream(tiles + c * 32 + lane);
            const unsigned w[2][2] = { { q.x, q.y }, { q.z, q.w } };
#pragma unroll
            for (int nib = 0; nib < 2; nib++) {
                const int j = 2 * c + nib;
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const unsigned scb = ((j < 4 ? sc_lo[r] : sc_hi[r]) >> (8 * (j & 3))) & 0xffu;
                    const unsigned mnb = ((j < 4 ? mn_lo[r] : mn_hi[r]) >> (8 * (j & 3))) & 0xffu;
                    const float a = d[r] * (float)scb, b = -(dmin[r] * (float)mnb);
                    const unsigned c0 = (w[r][0] >> (4 * nib)) & 0x0F0F0F0Fu, c1 = (w[r][1] >> (4 * nib)) & 0x0F0F0F0Fu;
#pragma unroll
                    for (int m = 0; m < M; m++) {
                        const float *xb = xs + m * x_row + j * 32 + 8 * t;
                        float su = 0.f, sx = 0.f;
                        f32v_dot4<false>(c0, xb, su, sx);
                        f32v_dot4<false>(c1, xb + 4, su, sx);
                        acc[m][r] += fmaf(a, su, b * sx);
                    }
                }
            }
        }
    } else {   // Q6_K
        const unsigned short *dp = reinterpret_cast<const unsigned short *>(rec + code_bytes(FMT) + 256);
        const float d[2] = { f32v_h2f(dp[g]), f32v_h2f(dp[g + 8]) };
        const uint4 sc[2] = { hdr[g], hdr[g + 8] };     // i8 scales[16] of rows g, g + 8
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            // planes 0 / 1: rows g / g + 8: L[l0..+3], L[32+l0..+3], L[l1..+3], L[32+l1..+3] with l0 = 4t, l1 = 16 + 4t
            // plane 2: H[l0..+3] (row g), H[l1..+3] (row g), H[l0..+3] (row g+8), H[l1..+3] (row g+8)
            const uint4 L[2] = { ld_stream(tiles + (3 * hf) * 32 + lane), ld_stream(tiles + (3 * hf + 1) * 32 + lane) };
            const uint4 H = ld_stream(tiles + (3 * hf + 2) * 32 + lane);
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const unsigned scw[4] = { sc[r].x, sc[r].y, sc[r].z, sc[r].w };
#pragma unroll
                for (int li = 0; li < 2; li++) {          // l0 group, l1 group
                    const unsigned lw = li ? L[r].z : L[r].x, lw32 = li ? L[r].w : L[r].y;
                    const unsigned hw = r ? (li ? H.w : H.z) : (li ? H.y : H.x);
                    const int l = li ? 16 + 4 * t : 4 * t;
#pragma unroll
                    for (int v = 0; v < 4; v++) {         // the four 32-value quarters of the half
                        const unsigned lo4 = ((v & 2) ? ((v & 1) ? lw32 : lw) >> 4 : ((v & 1) ? lw32 : lw)) & 0x0F0F0F0Fu;
                        const unsigned hi2 = ((hw >> (2 * v)) & 0x03030303u) << 4;
                        const unsigned codes = lo4 | hi2;                         // 0..63
                        const int kk = 128 * hf + 32 * v + l;                     // first of four consecutive values
                        const int gi = kk >> 4;                                   // scale group of 16
                        const float a = d[r] * (float)(int)(signed char)((scw[gi >> 2] >> (8 * (gi & 3))) & 0xffu);
#pragma unroll
                        for (int m = 0; m < M; m++) {
                            float su = 0.f, sx = 0.f;
                            f32v_dot4<false>(codes, xs + m * x_row + kk, su, sx);
                            acc[m][r] += fmaf(a, su, (-32.0f * a) * sx);
                        }
                    }
                }
            }
        }
    }
}

template <int FMT, int M>
__global__ void __launch_bounds__(F32V_WARPS * 32) matvec_f32_kernel(const WeightView w, const void *__restrict__ xv, int x_dtype,
                                                                     long long x_stride, int row0, float *__restrict__ y,
                                                                     long long y_stride, const Epilogue ep)
{
    extern __shared__ __align__(16) unsigned char f32v_smem[];
    float *xs = reinterpret_cast<float *>(f32v_smem);          // [M][k_pad]
    float *red = xs + (size_t)M * w.k_pad;                      // [warps][M][16]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rg = blockIdx.x;
    pdl_enter(0);
    for (int i = threadIdx.x; i < M * w.k_pad; i += F32V_WARPS * 32) {
        const int m = i / w.k_pad, kk = i - m * w.k_pad;
        float v = 0.0f;
        if (kk < w.k) {
            v = x_dtype == 0 ? reinterpret_cast<const float *>(xv)[(long long)(row0 + m) * x_stride + kk]
                             : __uint_as_float((unsigned)reinterpret_cast<const unsigned short *>(xv)[(long long)(row0 + m) * x_stride + kk] << 16);
        }
        xs[i] = v;
    }
    __syncthreads();
    float acc[M][2];
#pragma unroll
    for (int m = 0; m < M; m++) { acc[m][0] = 0.f; acc[m][1] = 0.f; }
    const int nst = w.k_pad >> 8;
    for (int st = warp; st < nst; st += F32V_WARPS) {
        f32v_record<FMT, M>(w.record(rg, st), lane, xs + st * 256, w.k_pad, acc);
    }
    // the four lanes of a row, then the warps
#pragma unroll
    for (int m = 0; m < M; m++) {
#pragma unroll
        for (int r = 0; r < 2; r++) {
            float v = acc[m][r];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if ((lane & 3) == 0) red[(warp * M + m) * 16 + (lane >> 2) + 8 * r] = v;
        }
    }
    __syncthreads();
    if (threadIdx.x < M * 16) {
        const int m = threadIdx.x >> 4, rr = threadIdx.x & 15;
        float v = 0.f;
        for (int wi = 0; wi < F32V_WARPS; wi++) v += red[(wi * M + m) * 16 + rr];
        const int row = rg * 16 + rr;
        if (row < w.n) y[(long long)(row0 + m) * y_stride + row] = ep.apply(v, row0 + m, row);
    }
}

// Expert-indexed form (the reference's MatMulId, src/Sharplight.Core/Graph/StandardOps.Moe.cs:8-40, CPU arithmetic as
// src/Sharplight.Cpu/MatMulIdOp.cs: f32 activations, each item computed as a single row is): the weight holds the E
// expert matrices one after the other ([E * N, K], N a multiple of 16 so that an expert starts on a row group);
// item = t * S + s multiplies the rows of expert ids[item] with activation row item (per_slot) or t, and writes output
// row item. Grid: (N / 16, items). The ids come from the kernel in front (top-k routing), so nothing is read before the
// dependency wait. An id outside [0, E) raises the device status word (-1) and leaves the item's row untouched.
template <int FMT>
__global__ void __launch_bounds__(F32V_WARPS * 32) matvec_f32_id_kernel(const WeightView w, int rg_per_expert, int n_expert, int experts,
                                                                        const void *__restrict__ xv, int x_dtype, long long x_stride,
                                                                        const int *__restrict__ ids, int slots, int per_slot,
                                                                        float *__restrict__ y, long long y_stride, int *status)
{
    extern __shared__ __align__(16) unsigned char f32v_smem[];
    float *xs = reinterpret_cast<float *>(f32v_smem);          // [k_pad]
    float *red = xs + w.k_pad;                                  // [warps][16]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int item = blockIdx.y;
    pdl_enter(0);
    const int e = ids[item];
    if (e < 0 || e >= experts) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicExch(status, -1);
        return;
    }
    const long long xrow = per_slot ? item : item / slots;
    for (int kk = threadIdx.x; kk < w.k_pad; kk += F32V_WARPS * 32) {
        float v = 0.0f;
        if (kk < w.k) {
            v = x_dtype == 0 ? reinterpret_cast<const float *>(xv)[xrow * x_stride + kk]
                             : __uint_as_float((unsigned)reinterpret_cast<const unsigned short *>(xv)[xrow * x_stride + kk] << 16);
        }
        xs[kk] = v;
    }
    __syncthreads();
    float acc[1][2] = { { 0.f, 0.f } };
    const int rg = e * rg_per_expert + (int)blockIdx.x, nst = w.k_pad >> 8;
    for (int st = warp; st < nst; st += F32V_WARPS) f32v_record<FMT, 1>(w.record(rg, st), lane, xs + st * 256, w.k_pad, acc);
#pragma unroll
    for (int r = 0; r < 2; r++) {
        float v = acc[0][r];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        if ((lane & 3) == 0) red[warp * 16 + (lane >> 2) + 8 * r] = v;
    }
    __syncthreads();
    if (threadIdx.x < 16) {
        float v = 0.f;
        for (int wi = 0; wi < F32V_WARPS; wi++) v += red[wi * 16 + threadIdx.x];
        const int row = (int)blockIdx.x * 16 + threadIdx.x;
        if (row < n_expert) y[(long long)item * y_stride + row] = v;
    }
}

static size_t f32v_smem_bytes(int m, int k_pad) { return (size_t)m * k_pad * 4 + (size_t)F32V_WARPS * m * 16 * 4; }

// rows per launch that fit the shared memory (0: K is too long even for one row)
int matvec_f32_rows(int k_pad)
{
    for (int m = 4; m >= 1; m--) {
        if (f32v_smem_bytes(m, k_pad) <= (size_t)F32V_MAX_SMEM) return m;
    }
    return 0;
}

template <int FMT, int M>
static cudaError_t f32v_launch(const WeightView &w, const void *x, int x_dtype, long long x_stride, int row0, float *y,
                               long long y_stride, const Epilogue &ep, cudaStream_t stream)
{
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = matvec_f32_kernel<FMT, M>;
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F32V_MAX_SMEM);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    return launch_pdl(kernel, dim3(w.n_pad >> 4), dim3(F32V_WARPS * 32), f32v_smem_bytes(M, w.k_pad), stream, w, x, x_dtype, x_stride,
                      row0, y, y_stride, ep);
}

// rows: 1 .. matvec_f32_rows(k_pad). x: device, f32 or bf16 (x_dtype 0 / 1), rows x_stride elements apart.
cudaError_t launch_matvec_f32(const WeightView &w, const void *x, int x_dtype, long long x_stride, int row0, int rows, float *y,
                              long long y_stride, cudaStream_t stream, const Epilogue *epilogue)
{
    if (w.n_pad == 0 || rows == 0) return cudaSuccess;
    const Epilogue ep = epilogue ? *epilogue : Epilogue{ nullptr, nullptr, 0 };
    if (rows < 1 || rows > 4 || f32v_smem_bytes(rows, w.k_pad) > (size_t)F32V_MAX_SMEM) return cudaErrorInvalidValue;
#define SLC_M(F, MM) case MM: return f32v_launch<F, MM>(w, x, x_dtype, x_stride, row0, y, y_stride, ep, stream);
#define SLC_FMT(F) case F: switch (rows) { SLC_M(F, 1) SLC_M(F, 2) SLC_M(F, 3) SLC_M(F, 4) } break;
    switch (w.fmt) {
        SLC_FMT(FMT_Q8_0) SLC_FMT(FMT_Q4_0) SLC_FMT(FMT_Q4_K) SLC_FMT(FMT_Q6_K)
    }
#undef SLC_FMT
#undef SLC_M
    return cudaErrorInvalidValue;
}

template <int FMT>
static cudaError_t f32v_id_launch(const WeightView &w, int experts, const void *x, int x_dtype, long long x_stride, const int *ids,
                                  long long items, int slots, int per_slot, float *y, long long y_stride, int *status,
                                  cudaStream_t stream)
{
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = matvec_f32_id_kernel<FMT>;
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F32V_MAX_SMEM);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int n_expert = w.n / experts, rg_per_expert = n_expert >> 4;
    cudaError_t e = cudaSuccess;
    // the grid's second dimension holds at most 65535 items: launches of whole tokens
    const long long per_launch = slots <= 65535 ? (65535 / slots) * (long long)slots : 0;
    if (per_launch == 0) return cudaErrorInvalidValue;
    const size_t esz = x_dtype == 0 ? 4 : 2;
    for (long long i0 = 0; i0 < items && e == cudaSuccess; i0 += per_launch) {
        const long long cnt = items - i0 < per_launch ? items - i0 : per_launch;
        const long long xrow0 = per_slot ? i0 : i0 / slots;   // the activation row of this launch's first item
        const void *xi = static_cast<const char *>(x) + (size_t)xrow0 * (size_t)x_stride * esz;
        e = launch_pdl(kernel, dim3(rg_per_expert, (unsigned)cnt), dim3(F32V_WARPS * 32), f32v_smem_bytes(1, w.k_pad), stream, w,
                       rg_per_expert, n_expert, experts, xi, x_dtype, x_stride, ids + i0, slots, per_slot, y + i0 * y_stride, y_stride, status);
    }
    return e;
}

// w: [experts * N, K] with N % 16 == 0; ids: device, items = tokens * slots entries; y: items rows, y_stride apart.
cudaError_t launch_matvec_f32_id(const WeightView &w, int experts, const void *x, int x_dtype, long long x_stride, const int *ids,
                                 long long tokens, int slots, int per_slot, float *y, long long y_stride, int *status,
                                 cudaStream_t stream)
{
    if (experts < 1 || w.n % experts != 0 || ((w.n / experts) & 15) != 0 || slots < 1) return cudaErrorInvalidValue;
    if (tokens <= 0 || w.n == 0) return cudaSuccess;
    if (f32v_smem_bytes(1, w.k_pad) > (size_t)F32V_MAX_SMEM) return cudaErrorInvalidValue;
    const long long items = tokens * slots;
    switch (w.fmt) {
    case FMT_Q8_0: return f32v_id_launch<FMT_Q8_0>(w, experts, x, x_dtype, x_stride, ids, items, slots, per_slot, y, y_stride, status, stream);
    case FMT_Q4_0: return f32v_id_launch<FMT_Q4_0>(w, experts, x, x_dtype, x_stride, ids, items, slots, per_slot, y, y_stride, status, stream);
    case FMT_Q4_K: return f32v_id_launch<FMT_Q4_K>(w, experts, x, x_dtype, x_stride, ids, items, slots, per_slot, y, y_stride, status, stream);
    case FMT_Q6_K: return f32v_id_launch<FMT_Q6_K>(w, experts, x, x_dtype, x_stride, ids, items, slots, per_slot, y, y_stride, status, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace slc
