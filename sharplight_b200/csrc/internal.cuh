// Launchers shared between the translation units of libsharplight_cuda.
#pragma once

#include <string>
#include <string.h>

#include "layout.cuh"

namespace slc {

// Programmatic dependent launch. Every kernel of this library is launched with the attribute below and calls
// pdl_wait() before its first read of data an earlier kernel may have produced and before its first global write, so
// consecutive kernels on a stream overlap only where that is safe: a kernel's independent prologue (weight loads)
// runs while its predecessor drains. `early` (launchers below): the launch reads quantized activations that an earlier
// launch on the same stream has already read, and writes nothing the preceding kernel touches.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// The two ways a kernel joins the chain. Ordinary: wait for the preceding kernel (which may have produced this one's
// input), and only then let the next kernel start -- so whatever starts after a kernel's trigger knows that everything
// before that kernel is complete. Early: the input was complete before the preceding kernel even started (the preceding
// kernel reads the same quantized activations), so run beside it; the wait moves to the exit, which keeps completion in
// stream order for whoever waits on this kernel.
__device__ __forceinline__ void pdl_enter(int early)
{
    if (!early) pdl_wait();
    pdl_launch_dependents();
}
__device__ __forceinline__ void pdl_exit(int early)
{
    if (early) pdl_wait();
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

constexpr unsigned SLC_WAIT_LIMIT = 100000;   // attempts of up to ~20 us each (suspend-time hint): about two seconds

// ---- mbarrier / bulk-copy primitives ------------------------------------------------------------------------------

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// Arms the barrier with the byte count and starts the bulk copy global -> shared that completes it.
__device__ __forceinline__ void bulk_load(void *dst, const void *src, unsigned bytes, uint64_t *bar)
{
    const unsigned b = smem_u32(bar);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(b) : "memory");
}

// The same for two sources of `bytes` each, landing back to back at dst, on one barrier phase.
__device__ __forceinline__ void bulk_load2(void *dst, const void *src_a, const void *src_b, unsigned bytes, uint64_t *bar)
{
    const unsigned b = smem_u32(bar);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(2 * bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src_a), "r"(bytes), "r"(b) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst) + bytes), "l"(src_b), "r"(bytes), "r"(b) : "memory");
}

// Bounded wait for the phase with the given parity. Returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity)
{
    const unsigned b = smem_u32(bar);
    for (unsigned i = 0; i < SLC_WAIT_LIMIT; i++) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(b), "r"(parity), "r"(20000u) : "memory");
        if (ok) return true;
    }
    return false;
}

// repack.cu
cudaError_t launch_repack(int fmt, int n, int k, int n_pad, int k_pad, uint8_t *raw, uint8_t *data, bool to_raw,
                          cudaStream_t stream);

// convert.cu: raw Q5_0 / IQ4_NL blocks -> raw Q8_0 blocks (34 bytes each), exactly.
cudaError_t launch_convert_to_q8_0(int src_fmt, const uint8_t *src, uint8_t *dst, long long blocks, cudaStream_t stream);
// raw Q5_K blocks -> two arrays of raw Q4_K blocks (144 bytes each): the block without its fifth bits, and the fifth bits
// as a Q4_K block with d' = 16 d, dmin' = 0. *overflow (device int, zero before) is set when a 16 d is not an f16.
cudaError_t launch_split_q5_k(const uint8_t *src, uint8_t *low, uint8_t *high, long long blocks, int *overflow, cudaStream_t stream);

// quantize.cu: x (f32 or bf16, device) -> ActView planes. x_dtype: 0 = f32, 1 = bf16.
struct ActPlanes
{
    uint8_t *q_sw;      // optional: a copy of the codes in 128-byte swizzled operand rows (umma.cu), or null
    uint8_t *sx2;       // optional, with q_sw: d * sum32(q) split in two tf32 halves, 64-byte swizzled operand rows
    uint8_t *q_tiled;   // optional second copy of the codes in tensor-core core-matrix order (mmq.cu), or null
    int8_t *q;
    float2 *ds;
    float *dx, *sx;
    float *gs;
    int *isum;
};
cudaError_t launch_quantize(const void *x, int x_dtype, int rows, int rows_pad, int k, int k_pad, long long x_stride,
                            ActPlanes out, cudaStream_t stream);

// matvec.cu: dp4a mat-vec for 1..4 activation rows (rows row0 .. row0+rows-1 of the quantized activations). dump
// (optional) receives unsigned-code block dots [rows][n][k/32]; status: device word raised when a bounded wait runs out.
bool matvec_fits(int rows, int k_pad, bool dual = false);
// exchange (optional, both kernels): the MatMul is the row-split part of a tensor-parallel group; the kernel sums the
// partial outputs of all ranks itself (exchange.cuh) and y receives the total. Such a launch is never early.
struct Exchange;
cudaError_t launch_matvec(const WeightView &w, const ActView &a, int row0, int rows, float *y, long long y_stride,
                          int *dump, int *status, int early, cudaStream_t stream, const Exchange *exchange = nullptr,
                          const Epilogue *epilogue = nullptr, const WeightView *w2 = nullptr);
// w2 (optional, mat-vec only): a second weight of the same shape and format; y receives silu(x . W^T) * (x . W2^T).

// gate.cu: y[t][n] = silu(g[t][n]) * y[t][n], the same tail for the row counts the other kernels serve.
cudaError_t launch_gate_mul(const float *g, long long g_stride, float *y, long long y_stride, int rows, int n,
                            cudaStream_t stream);

// gate.cu: dst[z][r][c] = src[z * batch_stride + r * row_stride + c * col_stride], dense, elements of 2 or 4 bytes.
cudaError_t launch_densify(void *dst, const void *src, int batch, int rows, int cols, long long batch_stride, long long row_stride,
                           long long col_stride, int elem_bytes, cudaStream_t stream);

// matvec_f32.cu: dequant-fused f32 mat-vec for ops that keep f32 activation math; rows: 1 .. matvec_f32_rows(k_pad).
int matvec_f32_rows(int k_pad);
cudaError_t launch_matvec_f32(const WeightView &w, const void *x, int x_dtype, long long x_stride, int row0, int rows, float *y,
                              long long y_stride, cudaStream_t stream, const Epilogue *epilogue = nullptr);
// The expert-indexed form (MatMulId): w holds `experts` matrices of N = w.n / experts rows (N % 16 == 0); item t * slots + s
// multiplies expert ids[item] with activation row item (per_slot) or t and writes output row item. status: device word,
// set to -1 by an id outside [0, experts).
cudaError_t launch_matvec_f32_id(const WeightView &w, int experts, const void *x, int x_dtype, long long x_stride, const int *ids,
                                 long long tokens, int slots, int per_slot, float *y, long long y_stride, int *status,
                                 cudaStream_t stream);

// producers.cu: kernels that produce the quantized activations in the same pass as the operation in front of the MatMul
// (y, optional: the f32 result as well), and the arg-max behind the lm_head.
cudaError_t launch_rmsnorm_quantize(const void *x, int x_dtype, int rows, int rows_pad, int k, int k_pad, long long x_stride,
                                    const float *weight, float eps, float *y, long long y_stride, ActPlanes out, cudaStream_t stream);
cudaError_t launch_silu_mul_quantize(const float *gate, long long gate_stride, const float *up, long long up_stride, int rows,
                                     int rows_pad, int k, int k_pad, float *y, long long y_stride, ActPlanes out, cudaStream_t stream);
cudaError_t launch_argmax_rows(const float *y, long long y_stride, int rows, int n, int *out, cudaStream_t stream);

// tp_comm.cu: NCCL, loaded at run time, for the sums over ranks the in-kernel exchange does not serve.
struct NcclId { char bytes[128]; };
const char *tp_comm_unavailable();   // null when NCCL is loaded, else the reason
std::string tp_comm_error(int code);
int tp_comm_unique_id(uint8_t *out);
int tp_comm_init(void **comm, int world, const uint8_t *id, int rank);
int tp_comm_destroy(void *comm);
int tp_comm_allreduce(void *comm, float *y, long long rows, long long n, long long y_stride, cudaStream_t stream);
cudaError_t launch_add_epilogue(float *y, long long y_stride, int rows, int n, const Epilogue &ep, cudaStream_t stream);

// skinny.cu: int8 mma tiles, 1..64 activation rows per launch. split (optional): a scratch area and zeroed counters that
// let a MatMul with few weight rows and a long K spread over the machine in chunks of K (partial tiles summed by the last
// CTA to arrive, in chunk order); launches that use it must not overlap each other -- they are never early.
struct SkinnySplit
{
    float *scratch;        // scratch_floats floats
    int *counters;         // counter_slots ints, zero between launches
    size_t scratch_floats;
    int counter_slots;
    int sm_count;
};
cudaError_t launch_skinny(const WeightView &w, const ActView &a, int row0, int rows, float *y, long long y_stride,
                          int *dump, int *status, int early, cudaStream_t stream, const Exchange *exchange = nullptr,
                          const Epilogue *epilogue = nullptr, const SkinnySplit *split = nullptr);

// mmq.cu: tcgen05 / TMEM int8 GEMM for many rows (Q4_0, Q8_0, Q4_K). status: device word set to a negative code when
// a bounded wait runs out.
bool mmq_supports(int fmt);
cudaError_t launch_mmq(const WeightView &w, const ActView &a, const uint8_t *q_tiled, float *y, long long y_stride,
                       int *dump, int *status, int early, cudaStream_t stream, const Epilogue *epilogue = nullptr,
                       int tile_t0 = 0, int tile_count = 0);

// umma.cu: tcgen05 kind::f16 tiles for 3 rows and more (Q4_K, Q4_0, Q8_0), stream-K over one persistent CTA per SM.
// q_sw / sx2: the tiled planes the quantizer wrote for these rows (rows_pad a multiple of umma_token_tile(rows));
// scratch (umma_scratch_bytes) and counters (max_ctas ints, zero between launches) serve the tiles whose K range is
// shared by several CTAs. Launches that use the same scratch must not overlap.
bool umma_supports(int fmt, int rows);   // Q6_K: more than 64 rows only
int umma_token_tile(int rows);
size_t umma_scratch_bytes(int max_ctas, int rows_pad);
cudaError_t launch_umma(const WeightView &w, const ActView &a, const uint8_t *q_sw, const uint8_t *sx2, float *y,
                        long long y_stride, int *dump, int *status, float *scratch, int *counters, int max_ctas,
                        cudaStream_t stream, const Epilogue *epilogue = nullptr);

}  // namespace slc
