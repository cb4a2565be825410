// Sum of the partial outputs of a row-split MatMul over the GPUs of a tensor-parallel group, done inside the MatMul
// kernel itself (no collective-library call, no extra launch).
//
// Every rank owns a receive area that its peers map into their address space (CUDA IPC): two slots of
// [world][max_rows][n_stride] floats plus, per slot, one arrival word per (source rank, CTA). A CTA that has finished
// its 16 or 64 output columns
//   1. stores its partial values into the same place of every rank's area (plain stores over NVLink; its own area too),
//   2. fences, and one thread per destination publishes the CTA's arrival word there (release, system scope),
//   3. waits -- bounded -- until the same CTA of every other rank has arrived in its own area (acquire, system scope),
//   4. adds the `world` partial values in rank order (so every rank computes the bit-identical sum) and writes y.
// Every CTA stores before it waits, so a CTA never waits on anything but the scheduling of its counterparts.
//
// Slots alternate with the exchange counter, a device word that the last CTA of a launch advances. A launch begins
// only after the preceding kernel of its stream has completed (these launches never use the early mode), and a rank
// completes exchange e only after it has seen every peer's arrival for e, which the peer published after its own
// exchange e - 1 was over: when exchange e + 1 starts storing into a slot, nobody is still reading exchange e - 1 there.
//
// Launches of up to SLC_LL_ROWS rows (where latency is everything) use a lighter protocol in the same spirit, without fences or arrival words:
// every partial value travels as one 8-byte word {value, exchange number + 1}, written with a single store, which
// arrives whole or not at all; the receiving thread polls the word itself until it carries the current number. One
// NVLink crossing, no round trip. The same two-slot rule applies.
//
// Nothing here uses multicast objects or multimem: a rank that dies leaves its peers with a wait that runs out
// (status word, SLC_ERR_TIMEOUT), not with a fault.
#pragma once

#include <cstdint>

namespace slc {

constexpr int SLC_MAX_RANKS = 8;
constexpr int SLC_LL_ROWS = 16;  // launches of up to this many rows use the word protocol

struct Exchange
{
    float *recv[SLC_MAX_RANKS];   // rank p's receive area as this process sees it: [2][world][max_rows][n_stride]
    int *flags[SLC_MAX_RANKS];    // rank p's arrival words: [2][world][groups]
    unsigned long long *ll[SLC_MAX_RANKS];   // rank p's {value, tag} words: [2][world][SLC_LL_ROWS][n_stride]
    int *epoch;                   // this rank's exchange counter
    int *done;                    // CTAs of the running launch that are through
    int world, rank;              // world == 0: no exchange, the kernel writes y directly
    int max_rows, n_stride, groups;
    unsigned wait_ms;             // limit of step 3
};

#ifdef __CUDACC__

__device__ __forceinline__ long long ex_index(const Exchange &x, int slot, int src, int m, int col)
{
    return (((long long)slot * x.world + src) * x.max_rows + m) * x.n_stride + col;
}

__device__ __forceinline__ int ex_epoch(const Exchange &x) { return *reinterpret_cast<volatile int *>(x.epoch); }

__device__ __forceinline__ unsigned long long ex_now()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ long long ex_ll_index(const Exchange &x, int slot, int src, int m, int col)
{
    return (((long long)slot * x.world + src) * SLC_LL_ROWS + m) * x.n_stride + col;
}

// The word protocol for one value owned by the calling thread, in two halves so that a thread with several values
// sends them all before it waits for any: ex_ll_send stores {v, tag} into every peer's area; ex_ll_collect waits for
// the peers' words for the same value and returns the sum in rank order (ok turns false when a word never came).
__device__ __forceinline__ void ex_ll_send(const Exchange &x, int slot, int epoch, int m, int col, float v)
{
    const unsigned tag = (unsigned)epoch + 1u;
    const unsigned long long word = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    const long long at = ex_ll_index(x, slot, x.rank, m, col);
    for (int p = 0; p < x.world; p++) {
        if (p != x.rank) asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(x.ll[p] + at), "l"(word) : "memory");
    }
}

// t0: ex_now() taken once by the caller before its first collect, so that all values of a thread share one deadline.
__device__ __forceinline__ float ex_ll_collect(const Exchange &x, int slot, int epoch, int m, int col, float v, bool &ok,
                                               unsigned long long t0)
{
    const unsigned tag = (unsigned)epoch + 1u;
    const unsigned long long limit = (unsigned long long)x.wait_ms * 1000000ull;
    float s = 0.0f;
    for (int p = 0; p < x.world; p++) {
        float val = v;
        if (p != x.rank) {
            const unsigned long long *src = x.ll[x.rank] + ex_ll_index(x, slot, p, m, col);
            unsigned long long got;
            for (;;) {
                asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(got) : "l"(src) : "memory");
                if ((unsigned)(got >> 32) == tag) break;
                if (!ok || ex_now() - t0 > limit) { ok = false; break; }
            }
            val = __uint_as_float((unsigned)got);
        }
        s = p == 0 ? val : s + val;
    }
    return s;
}

// Steps 2 and 3. Every thread of the CTA calls it after its stores of step 1; returns false when a peer never arrived.
__device__ __forceinline__ bool ex_publish_and_wait(const Exchange &x, int slot, int epoch, int group)
{
    __threadfence_system();   // this thread's stores are ordered before the arrival word that follows the barrier
    __syncthreads();
    bool ok = true;
    if ((int)threadIdx.x < x.world) {
        const int p = threadIdx.x;
        int *theirs = x.flags[p] + ((long long)(slot * x.world + x.rank) * x.groups + group);
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(theirs), "r"(epoch + 1) : "memory");
        const int *mine = x.flags[x.rank] + ((long long)(slot * x.world + p) * x.groups + group);
        const unsigned long long t0 = ex_now(), limit = (unsigned long long)x.wait_ms * 1000000ull;
        for (;;) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (v == epoch + 1) break;
            if (ex_now() - t0 > limit) { ok = false; break; }
            __nanosleep(100);
        }
    }
    return __syncthreads_and(ok);
}

// Step 4 for one value (the L1 is bypassed: the data came from other GPUs).
__device__ __forceinline__ float ex_sum(const Exchange &x, int slot, int m, int col)
{
    const float *base = x.recv[x.rank];
    float s = __ldcg(base + ex_index(x, slot, 0, m, col));
    for (int p = 1; p < x.world; p++) s += __ldcg(base + ex_index(x, slot, p, m, col));
    return s;
}

__device__ __forceinline__ float4 ex_sum4(const Exchange &x, int slot, int m, int col)
{
    const float *base = x.recv[x.rank];
    float4 s = __ldcg(reinterpret_cast<const float4 *>(base + ex_index(x, slot, 0, m, col)));
    for (int p = 1; p < x.world; p++) {
        const float4 v = __ldcg(reinterpret_cast<const float4 *>(base + ex_index(x, slot, p, m, col)));
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    return s;
}

// The CTA is through with the exchange; the last CTA of the launch advances the counter. Every thread calls it.
__device__ __forceinline__ void ex_finish(const Exchange &x, int epoch)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned total = gridDim.x * gridDim.y;
        if (atomicAdd(reinterpret_cast<unsigned *>(x.done), 1u) == total - 1) {
            atomicExch(reinterpret_cast<unsigned *>(x.done), 0u);
            __threadfence();
            *reinterpret_cast<volatile int *>(x.epoch) = epoch + 1;
        }
    }
}

#endif  // __CUDACC__

}  // namespace slc
