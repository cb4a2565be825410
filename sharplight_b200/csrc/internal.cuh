// Launchers shared between the translation units of libsharplight_cuda.
#pragma once

#include "layout.cuh"

namespace slc {

// repack.cu
cudaError_t launch_repack(int fmt, int n, int k, int n_pad, int k_pad, uint8_t *raw, uint8_t *qs, uint8_t *sc,
                          uint8_t *d6, bool to_raw, cudaStream_t stream);

// quantize.cu: x (f32 or bf16, device) -> ActView planes. x_dtype: 0 = f32, 1 = bf16.
struct ActPlanes
{
    int8_t *q;
    float2 *ds;
    float *gs;
    int *isum;
};
cudaError_t launch_quantize(const void *x, int x_dtype, int rows, int rows_pad, int k, int k_pad, long long x_stride,
                            ActPlanes out, cudaStream_t stream);

// mmvq.cu: dp4a mat-vec for 1..8 activation rows. dump (optional) receives unsigned-code block dots
// [rows][n][k/32].
cudaError_t launch_mmvq(const WeightView &w, const ActView &a, int row0, int rows, float *y, long long y_stride,
                        int *dump, cudaStream_t stream);

// matvec_fused.cu: quantization fused into the dp4a mat-vec, 1..4 activation rows of device-resident x
// (f32 or bf16, rows x_stride elements apart); y rows y_stride apart. dump as for launch_mmvq.
bool fused_matvec_fits(int rows, int k_pad);
cudaError_t launch_fused_matvec(const WeightView &w, const void *x, int x_dtype, long long x_stride, int rows, float *y,
                                long long y_stride, int *dump, cudaStream_t stream);

// skinny.cu: int8 mma tiles, 1..64 activation rows per launch.
cudaError_t launch_skinny(const WeightView &w, const ActView &a, int row0, int rows, float *y, long long y_stride,
                          int *dump, cudaStream_t stream);

// mmq.cu: tcgen05 / TMEM int8 GEMM for many rows (Q4_0, Q8_0, Q4_K). status: device word set to a negative code when
// a bounded wait runs out.
bool mmq_supports(int fmt);
cudaError_t launch_mmq(const WeightView &w, const ActView &a, int rows, float *y, long long y_stride, int *dump,
                       int *status, cudaStream_t stream);

}  // namespace slc
