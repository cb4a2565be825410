// The gated-FFN tail for row counts the dual mat-vec does not serve: y = silu(g) * y, element by element, with
// silu(v) = v / (1 + exp(-v)) (src/Sharplight.Cpu/ScalarMath.cs:552-577 of the Sharplight tree).
#include "internal.cuh"

namespace slc {

__global__ void __launch_bounds__(256) gate_mul_kernel(const float *__restrict__ g, long long g_stride, float *y,
                                                       long long y_stride, int rows, int n)
{
    pdl_wait();                // g and y come from the two MatMuls before this kernel
    pdl_launch_dependents();
    const long long total = (long long)rows * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / n;
        const int c = (int)(i - t * n);
        const float v = g[t * g_stride + c];
        y[t * y_stride + c] = __fdiv_rn(v, 1.0f + expf(-v)) * y[t * y_stride + c];
    }
}

cudaError_t launch_gate_mul(const float *g, long long g_stride, float *y, long long y_stride, int rows, int n,
                            cudaStream_t stream)
{
    const long long total = (long long)rows * n;
    if (total == 0) return cudaSuccess;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    return launch_pdl(gate_mul_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, g, g_stride, y, y_stride, rows, n);
}

}  // namespace slc
