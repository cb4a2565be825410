// Collective-library side of tensor parallelism: the sum over ranks for row counts the in-kernel exchange does not
// serve (more rows than fit its receive areas, or more than pay for one {value, tag} word per element). NCCL is loaded
// at run time (dlopen of libnccl.so.2 -- the copy the process has already loaded, if any, so that a host that also uses
// torch.distributed runs one NCCL), never linked: the library builds and loads on machines without it, and only
// slc_tp_comm_* report its absence. Only the handful of entry points below are used; their types and constants are
// restated from NCCL's public header (ncclUniqueId is 128 bytes, ncclFloat32 = 7, ncclSum = 0).
#include "../../include/sharplight_cuda.h"
#include "handles.cuh"

#include <dlfcn.h>

#include <mutex>
#include <string>

namespace slc {

struct NcclApi
{
    void *lib = nullptr;
    int (*GetUniqueId)(void *id) = nullptr;
    int (*CommInitRank)(void **comm, int nranks, NcclId id, int rank) = nullptr;
    int (*CommDestroy)(void *comm) = nullptr;
    int (*AllReduce)(const void *send, void *recv, size_t count, int dtype, int op, void *comm, cudaStream_t stream) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    std::string why;   // why it is unavailable
};

static NcclApi &nccl()
{
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char *names[] = { "libnccl.so.2", "libnccl.so" };
        for (const char *name : names) {
            api.lib = dlopen(name, RTLD_NOW | RTLD_NOLOAD);   // the process's own copy first
            if (api.lib) break;
        }
        for (int i = 0; !api.lib && i < 2; i++) api.lib = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
        if (!api.lib) {
            api.why = "libnccl.so.2 not found";
            return;
        }
        auto sym = [&](const char *n) { return dlsym(api.lib, n); };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllReduce || !api.GroupStart || !api.GroupEnd) {
            api.why = "libnccl.so.2 lacks an entry point";
            api.lib = nullptr;
        }
    });
    return api;
}

const char *tp_comm_unavailable()
{
    NcclApi &a = nccl();
    return a.lib ? nullptr : a.why.c_str();
}

std::string tp_comm_error(int code)
{
    NcclApi &a = nccl();
    return std::string("NCCL: ") + (a.GetErrorString ? a.GetErrorString(code) : "error") + " (" + std::to_string(code) + ")";
}

int tp_comm_unique_id(uint8_t *out) { return nccl().GetUniqueId(out); }

int tp_comm_init(void **comm, int world, const uint8_t *id, int rank)
{
    NcclId v;
    memcpy(v.bytes, id, sizeof v.bytes);
    return nccl().CommInitRank(comm, world, v, rank);
}

int tp_comm_destroy(void *comm) { return nccl().CommDestroy(comm); }

// y[rows][n] (rows y_stride floats apart) <- the sum over ranks, in place: one call when the rows are contiguous, else
// one per row inside a group (NCCL fuses them into one launch).
int tp_comm_allreduce(void *comm, float *y, long long rows, long long n, long long y_stride, cudaStream_t stream)
{
    NcclApi &a = nccl();
    if (y_stride == n || rows == 1) return a.AllReduce(y, y, (size_t)(rows * n), 7, 0, comm, stream);
    int r = a.GroupStart();
    if (r != 0) return r;
    for (long long t = 0; t < rows && r == 0; t++) r = a.AllReduce(y + t * y_stride, y + t * y_stride, (size_t)n, 7, 0, comm, stream);
    const int e = a.GroupEnd();
    return r != 0 ? r : e;
}

// The elementwise tail after a sum that did not happen inside the MatMul kernel: y = (y + bias) + residual.
__global__ void __launch_bounds__(256) add_epilogue_kernel(float *y, long long y_stride, int rows, int n, Epilogue ep)
{
    const long long total = (long long)rows * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / n;
        const int c = (int)(i - t * n);
        y[t * y_stride + c] = ep.apply(y[t * y_stride + c], t, c);
    }
}

cudaError_t launch_add_epilogue(float *y, long long y_stride, int rows, int n, const Epilogue &ep, cudaStream_t stream)
{
    const long long total = (long long)rows * n;
    if (total == 0 || (!ep.bias && !ep.residual)) return cudaSuccess;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    add_epilogue_kernel<<<(unsigned)blocks, 256, 0, stream>>>(y, y_stride, rows, n, ep);
    return cudaGetLastError();
}

}  // namespace slc
