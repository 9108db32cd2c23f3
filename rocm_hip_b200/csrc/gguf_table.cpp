// gguf_table.cpp -- reads the tensor table of a GGUF file and uploads a tensor to the device: what stands between a
// model file and gpu_embed_rows. The reference maps the file and reads token_embd.weight in place from unified memory
// (src/gguf_mmap.h:15-17,92-100; QuantWeight, src/inference_internal.h:33-40); on B200 the table has to live in HBM,
// so the mapping is the source of one upload. This is a reader of the public GGUF container layout (version 2 / 3:
// header, typed key-value pairs, tensor infos, aligned data section), written for this one job; it is not the
// reference's parser (no split files, no tokenizer arrays, no staging).
//
// Every read is bounds-checked against the file size: a truncated or malformed file makes b200_gguf_open fail
// instead of faulting later.

#include "b200_layer_ops.h"

#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <new>
#include <string>
#include <vector>

namespace {

struct TensorInfo {
    std::string name;
    int type = -1, n_dims = 0;
    long long ne[4] = {1, 1, 1, 1};
    uint64_t offset = 0;   // from the start of the data section
    size_t row_bytes = 0, nbytes = 0;
};

struct KvEntry {
    std::string key;
    uint32_t type = 0;
    size_t value_off = 0;   // file offset of the value (for strings: of the length word)
};

// ggml type id -> (values per block, bytes per block) for the types this library handles
// (src/quant_types.h:19-47 ids; block sizes src/quant_types.cpp:583-598)
bool type_layout(int type, int* blck, int* bytes) {
    switch (type) {
        case 0: *blck = 1; *bytes = 4; return true;     // F32
        case 1: *blck = 1; *bytes = 2; return true;     // F16
        case 2: *blck = 32; *bytes = 18; return true;   // Q4_0
        case 3: *blck = 32; *bytes = 20; return true;   // Q4_1
        case 6: *blck = 32; *bytes = 22; return true;   // Q5_0
        case 7: *blck = 32; *bytes = 24; return true;   // Q5_1
        case 8: *blck = 32; *bytes = 34; return true;   // Q8_0
        case 12: *blck = 256; *bytes = 144; return true;  // Q4_K
        case 13: *blck = 256; *bytes = 176; return true;  // Q5_K
        case 14: *blck = 256; *bytes = 210; return true;  // Q6_K
        case 30: *blck = 1; *bytes = 2; return true;    // BF16
        default: return false;
    }
}

struct Reader {
    const uint8_t* p;
    size_t size, at = 0;
    bool ok = true;
    bool need(size_t n) {
        if (!ok || n > size - at) { ok = false; return false; }
        return true;
    }
    template <typename T>
    T get() {
        T v{};
        if (need(sizeof(T))) { memcpy(&v, p + at, sizeof(T)); at += sizeof(T); }
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        std::string s;
        if (n > (1u << 20) || !need((size_t)n)) { ok = false; return s; }
        s.assign((const char*)p + at, (size_t)n);
        at += (size_t)n;
        return s;
    }
    static size_t scalar_size(uint32_t t) {
        switch (t) {
            case 0: case 1: case 7: return 1;
            case 2: case 3: return 2;
            case 4: case 5: case 6: return 4;
            case 10: case 11: case 12: return 8;
            default: return 0;
        }
    }
    void skip_value(uint32_t t, int depth = 0) {
        if (t == 8) { (void)str(); return; }
        if (t == 9) {
            const uint32_t et = get<uint32_t>();
            const uint64_t n = get<uint64_t>();
            if (depth > 2) { ok = false; return; }
            const size_t es = scalar_size(et);
            if (es) {
                if (n > (size - at) / es) { ok = false; return; }
                at += (size_t)n * es;
            } else {
                for (uint64_t i = 0; i < n && ok; ++i) skip_value(et, depth + 1);
            }
            return;
        }
        const size_t es = scalar_size(t);
        if (!es || !need(es)) { ok = false; return; }
        at += es;
    }
};

}  // namespace

struct b200_gguf {
    int fd = -1;
    const uint8_t* map = nullptr;
    size_t size = 0;
    uint32_t version = 0;
    size_t alignment = 32, data_off = 0;
    std::vector<TensorInfo> tensors;
    std::vector<KvEntry> kv;
};

extern "C" {

void b200_gguf_close(b200_gguf* g) {
    if (!g) return;
    if (g->map) munmap(const_cast<uint8_t*>(g->map), g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

b200_gguf* b200_gguf_open(const char* path) {
    if (!path) return nullptr;
    b200_gguf* g = new (std::nothrow) b200_gguf;
    if (!g) return nullptr;
    struct stat st;
    g->fd = open(path, O_RDONLY);
    if (g->fd < 0 || fstat(g->fd, &st) != 0 || st.st_size < 24) { b200_gguf_close(g); return nullptr; }
    g->size = (size_t)st.st_size;
    void* m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) { b200_gguf_close(g); return nullptr; }
    g->map = (const uint8_t*)m;

    Reader r{g->map, g->size};
    const uint32_t magic = r.get<uint32_t>();
    g->version = r.get<uint32_t>();
    const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
    if (!r.ok || magic != 0x46554747u || g->version < 2 || g->version > 3 || n_tensors > (1u << 24) || n_kv > (1u << 24)) {
        b200_gguf_close(g);
        return nullptr;
    }
    for (uint64_t i = 0; i < n_kv && r.ok; ++i) {
        KvEntry e;
        e.key = r.str();
        e.type = r.get<uint32_t>();
        e.value_off = r.at;
        if (r.ok && e.key == "general.alignment" && e.type == 4 && r.need(4)) {   // (a file may end right after the type)
            uint32_t a;
            memcpy(&a, g->map + r.at, 4);
            if (a >= 1 && a <= (1u << 20) && (a & (a - 1)) == 0) g->alignment = a;
        }
        r.skip_value(e.type);
        if (r.ok) g->kv.push_back(std::move(e));
    }
    for (uint64_t i = 0; i < n_tensors && r.ok; ++i) {
        TensorInfo t;
        t.name = r.str();
        t.n_dims = (int)r.get<uint32_t>();
        if (t.n_dims < 1 || t.n_dims > 4) { r.ok = false; break; }
        for (int d = 0; d < t.n_dims; ++d) {
            t.ne[d] = (long long)r.get<uint64_t>();
            if (t.ne[d] <= 0) r.ok = false;
        }
        t.type = (int)r.get<uint32_t>();
        t.offset = r.get<uint64_t>();
        int blck = 0, bytes = 0;
        if (r.ok && type_layout(t.type, &blck, &bytes) && t.ne[0] % blck == 0) {
            // the extents come from the file: a product that wraps would pass the inside-the-file check below with a
            // small nbytes while ne[] still reports the huge extents, so every step is checked and a wrap fails the open
            size_t rb = 0, nb = 0;
            if (__builtin_mul_overflow((size_t)(t.ne[0] / blck), (size_t)bytes, &rb) ||
                __builtin_mul_overflow(rb, (size_t)t.ne[1], &nb) || __builtin_mul_overflow(nb, (size_t)t.ne[2], &nb) ||
                __builtin_mul_overflow(nb, (size_t)t.ne[3], &nb)) {
                r.ok = false;
                break;
            }
            t.row_bytes = rb;
            t.nbytes = nb;
        }
        if (r.ok) g->tensors.push_back(std::move(t));
    }
    if (!r.ok) { b200_gguf_close(g); return nullptr; }
    g->data_off = (r.at + g->alignment - 1) / g->alignment * g->alignment;
    for (const TensorInfo& t : g->tensors)   // a tensor of a known type must lie inside the file
        if (t.nbytes && (g->data_off > g->size || t.offset > g->size - g->data_off || t.nbytes > g->size - g->data_off - t.offset)) {
            b200_gguf_close(g);
            return nullptr;
        }
    return g;
}

long long b200_gguf_n_tensors(const b200_gguf* g) { return g ? (long long)g->tensors.size() : 0; }
unsigned b200_gguf_version(const b200_gguf* g) { return g ? g->version : 0; }
size_t b200_gguf_alignment(const b200_gguf* g) { return g ? g->alignment : 0; }
size_t b200_gguf_data_offset(const b200_gguf* g) { return g ? g->data_off : 0; }

int b200_gguf_find_tensor(const b200_gguf* g, const char* name) {
    if (!g || !name) return -1;
    for (size_t i = 0; i < g->tensors.size(); ++i)
        if (g->tensors[i].name == name) return (int)i;
    return -1;
}

int b200_gguf_tensor_info(const b200_gguf* g, int idx, const char** name, int* type, int* n_dims, long long ne[4],
                          size_t* row_bytes, size_t* nbytes, const void** host_data) {
    if (!g || idx < 0 || (size_t)idx >= g->tensors.size()) return -1;
    const TensorInfo& t = g->tensors[(size_t)idx];
    if (name) *name = t.name.c_str();
    if (type) *type = t.type;
    if (n_dims) *n_dims = t.n_dims;
    if (ne) for (int d = 0; d < 4; ++d) ne[d] = t.ne[d];
    if (row_bytes) *row_bytes = t.row_bytes;
    if (nbytes) *nbytes = t.nbytes;
    if (host_data) *host_data = t.nbytes ? g->map + g->data_off + t.offset : nullptr;
    return 0;
}

static const KvEntry* find_kv(const b200_gguf* g, const char* key, uint32_t type) {
    if (!g || !key) return nullptr;
    for (const KvEntry& e : g->kv)
        if (e.type == type && e.key == key) return &e;
    return nullptr;
}

int b200_gguf_kv_u32(const b200_gguf* g, const char* key, uint32_t* out) {
    const KvEntry* e = find_kv(g, key, 4);
    if (!e || !out) return -1;
    memcpy(out, g->map + e->value_off, 4);
    return 0;
}

int b200_gguf_kv_f32(const b200_gguf* g, const char* key, float* out) {
    const KvEntry* e = find_kv(g, key, 6);
    if (!e || !out) return -1;
    memcpy(out, g->map + e->value_off, 4);
    return 0;
}

// Copies the string value (without terminator) into buf (cap bytes, always terminated); returns its length or -1
long long b200_gguf_kv_str(const b200_gguf* g, const char* key, char* buf, size_t cap) {
    const KvEntry* e = find_kv(g, key, 8);
    if (!e) return -1;
    uint64_t n;
    memcpy(&n, g->map + e->value_off, 8);
    if (buf && cap) {
        const size_t c = n < cap - 1 ? (size_t)n : cap - 1;
        memcpy(buf, g->map + e->value_off + 8, c);
        buf[c] = 0;
    }
    return (long long)n;
}

cudaError_t b200_gguf_upload_tensor(const b200_gguf* g, int idx, void** dev_ptr, cudaStream_t stream) {
    if (!g || !dev_ptr || idx < 0 || (size_t)idx >= g->tensors.size() || g->tensors[(size_t)idx].nbytes == 0)
        return cudaErrorInvalidValue;
    const TensorInfo& t = g->tensors[(size_t)idx];
    void* d = nullptr;
    cudaError_t e = cudaMalloc(&d, t.nbytes);
    if (e != cudaSuccess) return e;
    e = cudaMemcpyAsync(d, g->map + g->data_off + t.offset, t.nbytes, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) { cudaFree(d); return e; }
    *dev_ptr = d;
    return cudaSuccess;
}

void b200_gguf_free_tensor(void* dev_ptr) { if (dev_ptr) cudaFree(dev_ptr); }

}  // extern "C"
