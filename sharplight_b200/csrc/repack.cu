// Upload-time re-layout of raw ggml blocks into the fragment-major device layout (layout.cuh), and its inverse.
// One thread per 16-byte unit of the code plane, one thread per scale entry. Runs once per weight.
#include "internal.cuh"

namespace slc {

struct RawPos
{
    int row;
    int off;     // byte offset inside the raw row
    bool valid;
};

// Where byte i of code-plane unit (rg, st, r2) comes from in the raw tensor.
__device__ __forceinline__ RawPos code_source(int fmt, int n, int nblk, int rg, int st, int r2, int i)
{
    const int tile_plane = r2 >> 5, lane = r2 & 31, g = lane >> 2, t = lane & 3;
    RawPos p;
    int blk;  // raw block index along K
    if (fmt == FMT_Q8_0) {
        blk = st * 8 + tile_plane;
        p.row = rg * 16 + g + 8 * (i >> 3);
        p.off = blk * 34 + 2 + 8 * t + (i & 7);
    } else if (fmt == FMT_Q4_0) {
        const int word = i >> 2;
        blk = (st * 4 + tile_plane) * 2 + (word >> 1);
        p.row = rg * 16 + g + 8 * (word & 1);
        p.off = blk * 18 + 2 + 4 * t + (i & 3);
    } else if (fmt == FMT_Q4_K) {
        blk = st;
        p.row = rg * 16 + g + 8 * (i >> 3);
        p.off = blk * 144 + 16 + 32 * tile_plane + 8 * t + (i & 7);
    } else {  // Q6_K
        const int h = tile_plane / 3, plane = tile_plane % 3, word = i >> 2, bi = i & 3;
        blk = st;
        if (plane < 2) {
            p.row = rg * 16 + g + 8 * plane;
            const int l = ((word >> 1) ? 16 : 0) + 4 * t + bi;
            p.off = blk * 210 + 64 * h + ((word & 1) ? 32 : 0) + l;
        } else {
            p.row = rg * 16 + g + 8 * (word >> 1);
            const int l = ((word & 1) ? 16 : 0) + 4 * t + bi;
            p.off = blk * 210 + 128 + 32 * h + l;
        }
    }
    p.valid = p.row < n && blk < nblk;
    return p;
}

__global__ void repack_codes_kernel(int fmt, int n, int k, int n_pad, int k_pad, uint8_t *raw, uint8_t *qs, int to_raw)
{
    const int per_st = qs_units_per_supertile(fmt);
    const int nst = k_pad >> 8;
    const long long units = (long long)(n_pad / 16) * nst * per_st;
    const long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= units) return;
    const int r2 = (int)(u % per_st);
    const long long v = u / per_st;
    const int st = (int)(v % nst), rg = (int)(v / nst);
    const int nblk = k / block_size(fmt);
    const long long row_bytes = (long long)nblk * block_bytes(fmt);
    uint8_t *unit = qs + u * 16;
    for (int i = 0; i < 16; i++) {
        RawPos p = code_source(fmt, n, nblk, rg, st, r2, i);
        if (to_raw) {
            if (p.valid) raw[p.row * row_bytes + p.off] = unit[i];
        } else {
            unit[i] = p.valid ? raw[p.row * row_bytes + p.off] : (uint8_t)0;
        }
    }
}

__global__ void repack_scales_kernel(int fmt, int n, int k, int n_pad, int k_pad, uint8_t *raw, uint8_t *sc,
                                     uint8_t *d6, int to_raw)
{
    const int bs = block_size(fmt), bb = block_bytes(fmt);
    const int nblk = k / bs, nblk_pad = k_pad / bs;
    const long long total = (long long)n_pad * nblk_pad;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int blk = (int)(idx % nblk_pad), row = (int)(idx / nblk_pad);
    const bool valid = row < n && blk < nblk;
    uint8_t *src = raw + ((long long)row * nblk + blk) * bb;
    int entry_bytes, src_off;
    if (fmt == FMT_Q8_0 || fmt == FMT_Q4_0) { entry_bytes = 2; src_off = 0; }
    else if (fmt == FMT_Q4_K) { entry_bytes = 16; src_off = 0; }
    else { entry_bytes = 16; src_off = 192; }
    uint8_t *dst = sc + idx * entry_bytes;
    for (int i = 0; i < entry_bytes; i++) {
        if (to_raw) { if (valid) src[src_off + i] = dst[i]; }
        else dst[i] = valid ? src[src_off + i] : (uint8_t)0;
    }
    if (fmt == FMT_Q6_K) {
        for (int i = 0; i < 2; i++) {
            if (to_raw) { if (valid) src[208 + i] = d6[idx * 2 + i]; }
            else d6[idx * 2 + i] = valid ? src[208 + i] : (uint8_t)0;
        }
    }
}

cudaError_t launch_repack(int fmt, int n, int k, int n_pad, int k_pad, uint8_t *raw, uint8_t *qs, uint8_t *sc,
                          uint8_t *d6, bool to_raw, cudaStream_t stream)
{
    const long long units = (long long)(n_pad / 16) * (k_pad >> 8) * qs_units_per_supertile(fmt);
    const long long entries = (long long)n_pad * (k_pad / block_size(fmt));
    if (units > 0) {
        repack_codes_kernel<<<(unsigned)((units + 255) / 256), 256, 0, stream>>>(fmt, n, k, n_pad, k_pad, raw, qs,
                                                                                  to_raw ? 1 : 0);
    }
    if (entries > 0) {
        repack_scales_kernel<<<(unsigned)((entries + 255) / 256), 256, 0, stream>>>(fmt, n, k, n_pad, k_pad, raw, sc,
                                                                                    d6, to_raw ? 1 : 0);
    }
    return cudaGetLastError();
}

}  // namespace slc
