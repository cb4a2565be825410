// Reading weights straight out of a GGUF file: the file is memory-mapped, its header, metadata and tensor table are
// parsed with bounds checks (layout as the reference's importer reads it, src/Sharplight.Import.Gguf/GgufFile.cs:62-137 of
// the Sharplight tree: magic "GGUF", version 2 or 3, tensor count, key/value count, the key/value pairs, the tensor infos
// -- name, rank, dimensions innermost first, ggml type, offset --, then the tensor data at the next multiple of
// general.alignment, default 32), and a 2-D tensor of one of the served formats is uploaded from the mapping without a
// copy through managed buffers (the reference goes through IWeightSource.Read). A linear weight is stored with K
// innermost, so its shape is [dims[1], dims[0]] = [N, K] (src/Sharplight.Import.Gguf/GgufTensorInfo.cs:22).
#include "../../include/sharplight_cuda.h"
#include "handles.cuh"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <new>
#include <string>
#include <vector>

using namespace slc;

struct GgufTensor
{
    std::string name;
    int rank = 0;
    uint64_t dims[4] = { 1, 1, 1, 1 };
    uint32_t type = 0;
    uint64_t offset = 0;   // from the start of the data section
};

struct slc_gguf
{
    int fd = -1;
    const uint8_t *base = nullptr;
    size_t length = 0;
    uint32_t version = 0;
    uint64_t alignment = 32, data_offset = 0;
    std::vector<GgufTensor> tensors;
};

namespace {

thread_local std::string t_gguf_error;

slc_result g_fail(slc_result code, const std::string &msg)
{
    t_gguf_error = msg;
    return code;
}

struct Cursor
{
    const uint8_t *p;
    size_t left;
    bool ok = true;
    template <typename T> T get()
    {
        T v{};
        if (left < sizeof(T)) { ok = false; left = 0; return v; }
        memcpy(&v, p, sizeof(T));
        p += sizeof(T); left -= sizeof(T);
        return v;
    }
    void skip(uint64_t n)
    {
        if (n > left) { ok = false; left = 0; return; }
        p += n; left -= (size_t)n;
    }
    std::string str()
    {
        const uint64_t n = get<uint64_t>();
        if (!ok || n > left) { ok = false; return std::string(); }
        std::string s(reinterpret_cast<const char *>(p), (size_t)n);
        skip(n);
        return s;
    }
};

// bytes of a scalar metadata value type (0 for string / array / unknown)
size_t scalar_bytes(uint32_t t)
{
    switch (t) {
    case 0: case 1: case 7: return 1;
    case 2: case 3: return 2;
    case 4: case 5: case 6: return 4;
    case 10: case 11: case 12: return 8;
    default: return 0;
    }
}

// Skips one metadata value; for an integer scalar also returns it (general.alignment).
bool skip_value(Cursor &c, uint32_t type, uint64_t *as_int, int depth = 0)
{
    if (as_int) *as_int = 0;
    if (const size_t n = scalar_bytes(type)) {
        if (as_int && type != 6 && type != 12 && n <= 8 && c.left >= n) memcpy(as_int, c.p, n);
        c.skip(n);
        return c.ok;
    }
    if (type == 8) { c.str(); return c.ok; }
    if (type == 9 && depth < 4) {
        const uint32_t et = c.get<uint32_t>();
        const uint64_t count = c.get<uint64_t>();
        if (!c.ok) return false;
        if (const size_t n = scalar_bytes(et)) {
            if (count > c.left / n) { c.ok = false; return false; }
            c.skip(count * n);
            return c.ok;
        }
        for (uint64_t i = 0; i < count && c.ok; i++) skip_value(c, et, nullptr, depth + 1);
        return c.ok;
    }
    c.ok = false;
    return false;
}

}  // namespace

extern "C" {

const char *slc_gguf_last_error(void) { return t_gguf_error.c_str(); }

void slc_gguf_close(slc_gguf *g)
{
    if (!g) return;
    if (g->base) munmap(const_cast<uint8_t *>(g->base), g->length);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

slc_result slc_gguf_open(const char *path, slc_gguf **out)
{
    if (!out) return g_fail(SLC_ERR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (!path) return g_fail(SLC_ERR_INVALID_ARGUMENT, "path is null");
    slc_gguf *g = new (std::nothrow) slc_gguf();
    if (!g) return g_fail(SLC_ERR_OUT_OF_MEMORY, "host allocation failed");
    g->fd = open(path, O_RDONLY);
    struct stat st;
    if (g->fd < 0 || fstat(g->fd, &st) != 0 || st.st_size < 24) {
        slc_gguf_close(g);
        return g_fail(SLC_ERR_INVALID_ARGUMENT, std::string("cannot open, or too small to be GGUF: ") + path);
    }
    g->length = (size_t)st.st_size;
    void *m = mmap(nullptr, g->length, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) {
        slc_gguf_close(g);
        return g_fail(SLC_ERR_OUT_OF_MEMORY, "mmap failed");
    }
    g->base = static_cast<const uint8_t *>(m);
    Cursor c{ g->base, g->length };
    const uint32_t magic = c.get<uint32_t>();
    g->version = c.get<uint32_t>();
    if (magic != 0x46554747u) { slc_gguf_close(g); return g_fail(SLC_ERR_INVALID_ARGUMENT, "not a GGUF file (bad magic)"); }
    if (g->version != 2 && g->version != 3) { slc_gguf_close(g); return g_fail(SLC_ERR_UNSUPPORTED, "unsupported GGUF version"); }
    const uint64_t tensor_count = c.get<uint64_t>(), kv_count = c.get<uint64_t>();
    if (!c.ok || tensor_count > g->length || kv_count > g->length) { slc_gguf_close(g); return g_fail(SLC_ERR_INVALID_ARGUMENT, "implausible tensor / key count"); }
    for (uint64_t i = 0; i < kv_count && c.ok; i++) {
        const std::string key = c.str();
        const uint32_t type = c.get<uint32_t>();
        uint64_t v = 0;
        skip_value(c, type, &v);
        if (c.ok && key == "general.alignment" && v > 0 && v <= (1u << 20)) g->alignment = v;
    }
    try { g->tensors.resize((size_t)tensor_count); } catch (...) { slc_gguf_close(g); return g_fail(SLC_ERR_OUT_OF_MEMORY, "host allocation failed"); }
    for (uint64_t i = 0; i < tensor_count && c.ok; i++) {
        GgufTensor &t = g->tensors[(size_t)i];
        t.name = c.str();
        const uint32_t rank = c.get<uint32_t>();
        if (rank > 4) { c.ok = false; break; }
        t.rank = (int)rank;
        for (uint32_t d = 0; d < rank; d++) t.dims[d] = c.get<uint64_t>();
        t.type = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
    }
    if (!c.ok) { slc_gguf_close(g); return g_fail(SLC_ERR_INVALID_ARGUMENT, "truncated or malformed GGUF header"); }
    const uint64_t pos = (uint64_t)(c.p - g->base);
    g->data_offset = (pos + g->alignment - 1) / g->alignment * g->alignment;
    *out = g;
    return SLC_OK;
}

slc_result slc_gguf_tensor_count(slc_gguf *g, int64_t *count)
{
    if (!g || !count) return g_fail(SLC_ERR_INVALID_ARGUMENT, "file or out is null");
    *count = (int64_t)g->tensors.size();
    return SLC_OK;
}

// bytes of the tensor when it is a 2-D tensor of a served format; 0 otherwise
static uint64_t served_bytes(const GgufTensor &t)
{
    const int bs = source_block_size((int)t.type), bb = source_block_bytes((int)t.type);
    if (bs == 0 || t.rank != 2 || t.dims[0] == 0 || t.dims[0] % bs != 0 || t.dims[1] > (1ull << 31) || t.dims[0] > (1ull << 31)) return 0;
    return t.dims[1] * (t.dims[0] / bs) * bb;
}

slc_result slc_gguf_tensor_info(slc_gguf *g, int64_t index, char *name_out, int32_t name_capacity, int32_t *format, int32_t *rank,
                                int64_t *n, int64_t *k, int64_t *bytes)
{
    if (!g || index < 0 || index >= (int64_t)g->tensors.size()) return g_fail(SLC_ERR_INVALID_ARGUMENT, "file is null or index out of range");
    const GgufTensor &t = g->tensors[(size_t)index];
    if (name_out && name_capacity > 0) {
        if ((size_t)name_capacity <= t.name.size()) return g_fail(SLC_ERR_BUFFER_TOO_SMALL, "name buffer too small");
        memcpy(name_out, t.name.c_str(), t.name.size() + 1);
    }
    if (format) *format = (int32_t)t.type;
    if (rank) *rank = t.rank;
    if (k) *k = (int64_t)t.dims[0];                         // innermost dimension
    if (n) *n = t.rank >= 2 ? (int64_t)t.dims[1] : 1;
    if (bytes) *bytes = (int64_t)served_bytes(t);           // 0: not a 2-D tensor of a served format
    return SLC_OK;
}

slc_result slc_gguf_find(slc_gguf *g, const char *name, int64_t *index)
{
    if (!g || !name || !index) return g_fail(SLC_ERR_INVALID_ARGUMENT, "null argument");
    for (size_t i = 0; i < g->tensors.size(); i++) {
        if (g->tensors[i].name == name) { *index = (int64_t)i; return SLC_OK; }
    }
    *index = -1;
    return g_fail(SLC_ERR_INVALID_ARGUMENT, std::string("no tensor named ") + name);
}

slc_result slc_weight_upload_gguf(slc_device *d, slc_gguf *g, int64_t index, slc_weight **out)
{
    if (!out) return g_fail(SLC_ERR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (!d || !g || index < 0 || index >= (int64_t)g->tensors.size()) return g_fail(SLC_ERR_INVALID_ARGUMENT, "null argument or index out of range");
    const GgufTensor &t = g->tensors[(size_t)index];
    const uint64_t bytes = served_bytes(t);
    if (bytes == 0) return g_fail(SLC_ERR_UNSUPPORTED, "'" + t.name + "' is not a 2-D tensor of Q4_0, Q8_0, Q4_K, Q6_K, Q5_0, Q5_K or IQ4_NL");
    const uint64_t start = g->data_offset + t.offset;
    if (t.offset % g->alignment != 0 || start > g->length || bytes > g->length - start) {
        return g_fail(SLC_ERR_INVALID_ARGUMENT, "'" + t.name + "': data outside the file or misaligned");
    }
    const slc_result r = slc_weight_upload(d, (int32_t)t.type, (int64_t)t.dims[1], (int64_t)t.dims[0], g->base + start, (int64_t)bytes, out);
    if (r != SLC_OK) t_gguf_error = slc_last_error_message();
    return r;
}

}  // extern "C"
