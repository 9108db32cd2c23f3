// gguf_table.cpp -- reads the tensor table of a GGUF file and uploads a tensor to the device: what stands between a
// model file and gpu_embed_rows. The reference maps the file and reads token_embd.weight in place from unified memory
// (src/gguf_mmap.h:15-17,92-100; QuantWeight, src/inference_internal.h:33-40); on B200 the table has to live in HBM,
// so the mapping is the source of one upload. This is a reader of the public GGUF container layout (version 2 / 3:
// header, typed key-value pairs, tensor infos, aligned data section), written for this one job; it is not the
// reference's parser (no tokenizer arrays, no staging). A split model (<prefix>-00001-of-0000N.gguf, opened by its
// first file, as src/gguf_mmap.cpp:384-437 does) is read as one tensor table over N mappings; metadata comes from the
// first file.
//
// Every read is bounds-checked against the file size: a truncated or malformed file makes b200_gguf_open fail
// instead of faulting later.

#include "b200_layer_ops.h"

#include <fcntl.h>
#include <stdio.h>
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
    uint64_t offset = 0;   // from the start of the data section of its file
    size_t row_bytes = 0, nbytes = 0;
    int part = 0;          // the file of a split model that holds it (0: the one opened)
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

struct FilePart {
    int fd = -1;
    const uint8_t* map = nullptr;
    size_t size = 0, data_off = 0;
};

struct b200_gguf {
    std::vector<FilePart> parts;   // one mapping per file of a split model
    uint32_t version = 0;
    size_t alignment = 32;
    std::vector<TensorInfo> tensors;
    std::vector<KvEntry> kv;       // of the first file
    const uint8_t* data(const TensorInfo& t) const { return parts[(size_t)t.part].map + parts[(size_t)t.part].data_off + t.offset; }
};

namespace {

constexpr int kMaxSplits = 64;   // the reference's limit (src/gguf_mmap.cpp:122)

void close_part(FilePart& f) {
    if (f.map) munmap(const_cast<uint8_t*>(f.map), f.size);
    if (f.fd >= 0) close(f.fd);
    f = FilePart();
}

// Maps one file and reads its header: the key-value entries into kv, the tensor infos (marked with part) appended to
// tensors. alignment: in / out (a file's own general.alignment places its data section). false: missing, truncated or
// malformed.
bool read_file(const char* path, int part, FilePart& f, uint32_t* version, size_t* alignment, std::vector<KvEntry>& kv,
               std::vector<TensorInfo>& tensors) {
    struct stat st;
    f.fd = open(path, O_RDONLY);
    if (f.fd < 0 || fstat(f.fd, &st) != 0 || st.st_size < 24) return false;
    f.size = (size_t)st.st_size;
    void* m = mmap(nullptr, f.size, PROT_READ, MAP_PRIVATE, f.fd, 0);
    if (m == MAP_FAILED) return false;
    f.map = (const uint8_t*)m;

    Reader r{f.map, f.size};
    const uint32_t magic = r.get<uint32_t>();
    *version = r.get<uint32_t>();
    const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
    if (!r.ok || magic != 0x46554747u || *version < 2 || *version > 3 || n_tensors > (1u << 24) || n_kv > (1u << 24))
        return false;
    size_t align = 32;
    for (uint64_t i = 0; i < n_kv && r.ok; ++i) {
        KvEntry e;
        e.key = r.str();
        e.type = r.get<uint32_t>();
        e.value_off = r.at;
        if (r.ok && e.key == "general.alignment" && e.type == 4 && r.need(4)) {   // (a file may end right after the type)
            uint32_t a;
            memcpy(&a, f.map + r.at, 4);
            if (a >= 1 && a <= (1u << 20) && (a & (a - 1)) == 0) align = a;
        }
        r.skip_value(e.type);
        if (r.ok) kv.push_back(std::move(e));
    }
    const size_t first = tensors.size();
    for (uint64_t i = 0; i < n_tensors && r.ok; ++i) {
        TensorInfo t;
        t.part = part;
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
        if (r.ok) tensors.push_back(std::move(t));
    }
    if (!r.ok) return false;
    f.data_off = (r.at + align - 1) / align * align;
    for (size_t i = first; i < tensors.size(); ++i) {   // a tensor of a known type must lie inside its file
        const TensorInfo& t = tensors[i];
        if (t.nbytes && (f.data_off > f.size || t.offset > f.size - f.data_off || t.nbytes > f.size - f.data_off - t.offset))
            return false;
    }
    *alignment = align;
    return true;
}

// An integer key-value entry of any integer type (split.count and split.no are 16-bit in files llama.cpp writes)
long long kv_int_or(const std::vector<KvEntry>& kv, const uint8_t* map, const char* key, long long def) {
    for (const KvEntry& e : kv) {
        if (e.key != key) continue;
        const uint8_t* p = map + e.value_off;
        switch (e.type) {
            case 0: return *p;
            case 1: return (int8_t)*p;
            case 2: { uint16_t v; memcpy(&v, p, 2); return v; }
            case 3: { int16_t v; memcpy(&v, p, 2); return v; }
            case 4: { uint32_t v; memcpy(&v, p, 4); return v; }
            case 5: { int32_t v; memcpy(&v, p, 4); return v; }
            case 10: { uint64_t v; memcpy(&v, p, 8); return (long long)v; }
            case 11: { int64_t v; memcpy(&v, p, 8); return v; }
            default: return def;
        }
    }
    return def;
}

}  // namespace

extern "C" {

void b200_gguf_close(b200_gguf* g) {
    if (!g) return;
    for (FilePart& f : g->parts) close_part(f);
    delete g;
}

b200_gguf* b200_gguf_open(const char* path) {
    if (!path) return nullptr;
    b200_gguf* g = new (std::nothrow) b200_gguf;
    if (!g) return nullptr;
    g->parts.emplace_back();
    if (!read_file(path, 0, g->parts[0], &g->version, &g->alignment, g->kv, g->tensors)) { b200_gguf_close(g); return nullptr; }
    // a split model: the other files are named after the first (src/gguf_mmap.cpp:389-410), each must say which one it is
    const long long count = kv_int_or(g->kv, g->parts[0].map, "split.count", 1);
    if (count > 1) {
        char suffix[40];
        snprintf(suffix, sizeof(suffix), "-00001-of-%05d.gguf", (int)count);
        const std::string first(path);
        const size_t sl = strlen(suffix);
        if (count > kMaxSplits || first.size() < sl || first.compare(first.size() - sl, sl, suffix) != 0) {
            b200_gguf_close(g);
            return nullptr;
        }
        g->parts.reserve((size_t)count);
        for (int i = 1; i < (int)count; ++i) {
            char tail[40];
            snprintf(tail, sizeof(tail), "-%05d-of-%05d.gguf", i + 1, (int)count);
            const std::string part = first.substr(0, first.size() - sl) + tail;
            g->parts.emplace_back();
            std::vector<KvEntry> kv;
            uint32_t version = 0;
            size_t alignment = 32;
            if (!read_file(part.c_str(), i, g->parts.back(), &version, &alignment, kv, g->tensors) ||
                kv_int_or(kv, g->parts.back().map, "split.no", -1) != i) {
                b200_gguf_close(g);
                return nullptr;
            }
        }
    }
    return g;
}

long long b200_gguf_n_tensors(const b200_gguf* g) { return g ? (long long)g->tensors.size() : 0; }
unsigned b200_gguf_version(const b200_gguf* g) { return g ? g->version : 0; }
size_t b200_gguf_alignment(const b200_gguf* g) { return g ? g->alignment : 0; }
size_t b200_gguf_data_offset(const b200_gguf* g) { return g ? g->parts[0].data_off : 0; }
int b200_gguf_n_files(const b200_gguf* g) { return g ? (int)g->parts.size() : 0; }
int b200_gguf_tensor_file(const b200_gguf* g, int idx) {
    return g && idx >= 0 && (size_t)idx < g->tensors.size() ? g->tensors[(size_t)idx].part : -1;
}

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
    if (host_data) *host_data = t.nbytes ? g->data(t) : nullptr;
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
    memcpy(out, g->parts[0].map + e->value_off, 4);
    return 0;
}

int b200_gguf_kv_f32(const b200_gguf* g, const char* key, float* out) {
    const KvEntry* e = find_kv(g, key, 6);
    if (!e || !out) return -1;
    memcpy(out, g->parts[0].map + e->value_off, 4);
    return 0;
}

// Copies the string value (without terminator) into buf (cap bytes, always terminated); returns its length or -1
long long b200_gguf_kv_str(const b200_gguf* g, const char* key, char* buf, size_t cap) {
    const KvEntry* e = find_kv(g, key, 8);
    if (!e) return -1;
    uint64_t n;
    memcpy(&n, g->parts[0].map + e->value_off, 8);
    if (buf && cap) {
        const size_t c = n < cap - 1 ? (size_t)n : cap - 1;
        memcpy(buf, g->parts[0].map + e->value_off + 8, c);
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
    e = cudaMemcpyAsync(d, g->data(t), t.nbytes, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) { cudaFree(d); return e; }
    *dev_ptr = d;
    return cudaSuccess;
}

void b200_gguf_free_tensor(void* dev_ptr) { if (dev_ptr) cudaFree(dev_ptr); }

}  // extern "C"
