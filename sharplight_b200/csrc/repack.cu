// Upload-time re-layout of raw ggml blocks into the record layout (layout.cuh), and its inverse.
// One thread per 16-byte unit. Runs once per weight.
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

// One thread per 16-byte unit of a record: code units first, then the 16 scale entries, then (Q6_K) two units of d.
__global__ void repack_kernel(int fmt, int n, int k, int n_pad, int k_pad, uint8_t *raw, uint8_t *data, int to_raw)
{
    const int rec = record_bytes(fmt), units_per_rec = rec / 16, ncode = code_units(fmt);
    const int nst = k_pad >> 8;
    const long long units = (long long)(n_pad / 16) * nst * units_per_rec;
    const long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= units) return;
    const int r2 = (int)(u % units_per_rec);
    const long long v = u / units_per_rec;
    const int st = (int)(v % nst), rg = (int)(v / nst);
    const int bs = block_size(fmt), bb = block_bytes(fmt);
    const int nblk = k / bs;
    const long long row_bytes = (long long)nblk * bb;
    uint8_t *unit = data + u * 16;
    for (int i = 0; i < 16; i++) {
        RawPos p;
        if (r2 < ncode) {
            p = code_source(fmt, n, nblk, rg, st, r2, i);
        } else if (r2 < ncode + 16) {
            // scale entry of row r2 - ncode
            p.row = rg * 16 + (r2 - ncode);
            if (fmt == FMT_Q8_0 || fmt == FMT_Q4_0) {
                const int blk = st * 8 + (i >> 1);
                p.off = blk * bb + (i & 1);
                p.valid = p.row < n && blk < nblk;
            } else {
                p.off = st * bb + (fmt == FMT_Q4_K ? 0 : 192) + i;
                p.valid = p.row < n && st < nblk;
            }
        } else {
            // Q6_K super-block scales: two units, 8 rows x f16 each
            p.row = rg * 16 + (r2 - ncode - 16) * 8 + (i >> 1);
            p.off = st * bb + 208 + (i & 1);
            p.valid = p.row < n && st < nblk;
        }
        if (to_raw) {
            if (p.valid) raw[p.row * row_bytes + p.off] = unit[i];
        } else {
            unit[i] = p.valid ? raw[p.row * row_bytes + p.off] : (uint8_t)0;
        }
    }
}

cudaError_t launch_repack(int fmt, int n, int k, int n_pad, int k_pad, uint8_t *raw, uint8_t *data, bool to_raw,
                          cudaStream_t stream)
{
    const long long units = (long long)(n_pad / 16) * (k_pad >> 8) * (record_bytes(fmt) / 16);
    if (units > 0) {
        repack_kernel<<<(unsigned)((units + 255) / 256), 256, 0, stream>>>(fmt, n, k, n_pad, k_pad, raw, data,
                                                                           to_raw ? 1 : 0);
    }
    return cudaGetLastError();
}

}  // namespace slc
