// Prefill GEMM on the int8 tensor cores (tcgen05 / TMEM). Placeholder translation unit until the kernel lands.
#include "internal.cuh"

namespace slc {

bool mmq_supports(int) { return false; }

cudaError_t launch_mmq(const WeightView &, const ActView &, int, float *, long long, int *, int *, cudaStream_t)
{
    return cudaErrorNotSupported;
}

}  // namespace slc
