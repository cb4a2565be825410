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

// A strided view made dense: dst[z][r][c] = src[z * batch_stride + r * row_stride + c * col_stride] (strides in elements of
// elem_bytes = 2 or 4; dst is [batch][rows][cols], contiguous).
// The MatMul reads rows of contiguous elements; a Permute in front of it hands over a view whose rows are not, and this
// gather comes first, as the reference's lowering densifies such an input (src/Sharplight.Shaders/Lowering/
// GraphLowerer.MatMul.cs:117-126). Tiles go through shared memory so that reads and writes both run along memory.
template <typename T>
__global__ void __launch_bounds__(256) densify_kernel(T *__restrict__ dst, const T *__restrict__ src, int rows, int cols,
                                                      long long row_stride, long long col_stride, long long batch_stride)
{
    __shared__ T tile[32][33];
    pdl_wait();
    pdl_launch_dependents();
    dst += (long long)blockIdx.z * rows * cols;
    src += (long long)blockIdx.z * batch_stride;
    const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
    // read with the faster-varying source index along tx: rows if the view is a transpose, columns otherwise
    const bool by_rows = row_stride < col_stride;
    for (int i = ty; i < 32; i += 8) {
        const int r = by_rows ? r0 + tx : r0 + i, c = by_rows ? c0 + i : c0 + tx;
        if (r < rows && c < cols) tile[r - r0][c - c0] = src[(long long)r * row_stride + (long long)c * col_stride];
    }
    __syncthreads();
    for (int i = ty; i < 32; i += 8) {
        const int r = r0 + i, c = c0 + tx;
        if (r < rows && c < cols) dst[(long long)r * cols + c] = tile[i][tx];
    }
}

cudaError_t launch_densify(void *dst, const void *src, int batch, int rows, int cols, long long batch_stride, long long row_stride,
                           long long col_stride, int elem_bytes, cudaStream_t stream)
{
    if (batch == 0 || rows == 0 || cols == 0) return cudaSuccess;
    if (batch > 65535) return cudaErrorInvalidValue;
    const dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch);
    if (elem_bytes == 4) {
        return launch_pdl(densify_kernel<float>, grid, dim3(256), 0, stream, (float *)dst, (const float *)src, rows, cols, row_stride,
                          col_stride, batch_stride);
    }
    if (elem_bytes == 2) {
        return launch_pdl(densify_kernel<unsigned short>, grid, dim3(256), 0, stream, (unsigned short *)dst, (const unsigned short *)src,
                          rows, cols, row_stride, col_stride, batch_stride);
    }
    return cudaErrorInvalidValue;
}

}  // namespace slc
