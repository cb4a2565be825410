// The opaque handles of the C ABI (include/sharplight_cuda.h), shared by the translation units that implement it.
#pragma once

#include "internal.cuh"
#include "exchange.cuh"

#include <vector>

struct slc_device
{
    int index = 0;
    cudaStream_t stream = nullptr;
    int *status_dev = nullptr;   // device-side status word (bounded waits report here)
    cudaDeviceProp prop{};
    std::vector<cudaEvent_t> events;   // made by slc_stream_wait (some live on inside captured graphs); freed at close
};

struct slc_weight
{
    slc_device *dev = nullptr;
    int fmt = 0;       // the format of the device records (what the kernels see)
    int src_fmt = 0;   // the format that was uploaded (differs for the formats converted at upload: Q5_0, IQ4_NL -> Q8_0,
                       // Q5_K -> two Q4_K weights)
    slc_weight *high = nullptr;   // Q5_K: the second Q4_K weight (the fifth bits, d' = 16 d); a MatMul adds it onto the first
    long long n = 0, k = 0;
    uint8_t *base = nullptr;
    size_t bytes = 0;
    slc::WeightView view{};
};

struct slc_activation
{
    slc_device *dev = nullptr;
    long long max_rows = 0, k = 0;
    int k_pad = 0, cap_rows = 0;  // cap_rows: padded row capacity of the planes
    uint8_t *base = nullptr;
    size_t bytes = 0;
    slc::ActPlanes planes{};
    uint8_t *q_tiled = nullptr;   // present when the capacity allows GEMM-sized row counts
    uint8_t *q_sw = nullptr, *sx2 = nullptr;   // operand planes of the tile kernel (capacity of 3 rows and more)
    float *tile_scratch = nullptr;                // partial tiles of K ranges shared between CTAs (umma.cu, skinny.cu)
    size_t tile_scratch_floats = 0;
    int *tile_counters = nullptr;
    int tile_counter_slots = 0;
    int tile_ctas = 0;                            // CTAs the scratch was sized for (the device's SM count)
    int rows = 0, rows_pad = 0;   // what the last quantize call wrote
    int reads_since_quantize = 0;       // MatMul launches that have read the current contents ...
    cudaStream_t quantize_stream = nullptr;   // ... and the stream they were quantized on
    // deferred quantization (slc_activation_set_rows): the rows as given, not yet in the planes
    bool pending = false;
    const void *pending_x = nullptr;
    int pending_dtype = 0;
    long long pending_stride = 0;
};

struct slc_matmul
{
    slc_device *dev = nullptr;
    slc_weight *w = nullptr;
    slc_weight *w2 = nullptr;       // dual op: the up projection (w is the gate); y = silu(x . w^T) * (x . w2^T)
    float *dual_tmp = nullptr;      // dual op: the gate's result for the row counts that take two launches
    long long max_rows = 0;
    uint32_t flags = 0;
    int forced_kernel = SLC_KERNEL_AUTO;
    int last_kernel = 0, last_launches = 0;
    int last_launches_total = 0;    // including the activation quantization, when it was a launch of its own
    slc_activation *act = nullptr;  // the op's own quantized copy (slc_matmul_run)
    void *x_stage = nullptr;        // device staging for host activations (max_rows x k, 4 bytes each)
    float *y_stage = nullptr;       // device staging for host outputs (max_rows x n)
};


struct slc_tp_comm
{
    slc_device *dev = nullptr;
    int rank = 0, world = 0;
    void *comm = nullptr;   // ncclComm_t
    int chunk_min_rows = 0;  // > 0: prefill sums from this row count run in chunks beside the GEMM; 0 (default): after it
    // a stream of its own and events for prefill-sized sums: the all-reduce of one chunk of rows runs beside the GEMM of
    // the next
    cudaStream_t side = nullptr;
    cudaEvent_t chunk_done[8] = {}, joined = nullptr;
};

struct slc_tp_exchange
{
    slc_device *dev = nullptr;
    slc_tp_comm *comm = nullptr;          // optional: row counts above in_kernel_rows are summed by ncclAllReduce
    int in_kernel_rows = 16;
    int rank = 0, world = 0;
    long long max_rows = 0, n = 0;
    uint8_t *base = nullptr;              // this rank's receive area, arrival words and counters (one allocation)
    size_t bytes = 0, flags_off = 0, ll_off = 0, ctl_off = 0;
    void *peer[slc::SLC_MAX_RANKS] = {};  // the peers' allocations as mapped here (own entry = base)
    bool connected = false;
    slc::Exchange view{};
};
