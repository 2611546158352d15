// GGUF v3 directories and positional reads: the data side of the weight interface.
//
// Mirrors the reference's validated reader (src/gguf.rs:57-271 directory and shard rules,
// :346-460 positional reads, rows and matrices, :470-491 geometry) so that the files it opens, the
// errors it gives and the Tensor / Matrix descriptions it hands to the operators are the same:
//   * little-endian GGUF version 3 only; metadata values of the 13 GGUF types, arrays not nested,
//     no duplicate keys; general.alignment (default 32) a power of two;
//   * tensors of rank 1..4, no zero dimension, dims[0] a whole number of blocks of the type, offsets
//     aligned, no duplicate names, no range beyond the file, no two ranges overlapping;
//   * split models: the primary shard "-00001-of-NNNNN.gguf" names the others; split.no /
//     split.count / split.tensors.count must agree, non-split metadata must not contradict;
//   * a read that the file can no longer satisfy (truncated after it was opened) is INGOT_EOF, every
//     other violation INGOT_INVALID — io::ErrorKind::UnexpectedEof and InvalidData there.
// Host code only: nothing here touches the GPU except ingot_weight_load, which hands the tensor's
// bytes to ingot_weight_upload through a pinned staging buffer (the explicit copy that replaces the
// reference's no-copy mmap, src/metal.rs:546-582).
#include "../../include/ingot_cuda.h"

#include <errno.h>
#include <fcntl.h>
#include <stdio.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace {

thread_local std::string g_error;

ingot_status fail(ingot_status code, const std::string &msg) {
    g_error = msg;
    return code;
}

// (block elements, block bytes) of every GGML type the reference's directory accepts
// (src/gguf.rs:470-491): more than the kernels of this library decode, so that real files open.
bool directory_geometry(uint32_t kind, uint64_t &block, uint64_t &bytes) {
    switch (kind) {
    case 0: block = 1; bytes = 4; return true;
    case 1: case 30: block = 1; bytes = 2; return true;
    case 2: block = 32; bytes = 18; return true;
    case 8: block = 32; bytes = 34; return true;
    case 10: block = 256; bytes = 84; return true;
    case 12: block = 256; bytes = 144; return true;
    case 13: block = 256; bytes = 176; return true;
    case 14: block = 256; bytes = 210; return true;
    case 16: block = 256; bytes = 66; return true;
    case 17: block = 256; bytes = 74; return true;
    case 18: block = 256; bytes = 98; return true;
    case 20: block = 32; bytes = 18; return true;
    case 21: block = 256; bytes = 110; return true;
    case 22: block = 256; bytes = 82; return true;
    case 23: block = 256; bytes = 136; return true;
    case 29: block = 256; bytes = 56; return true;
    case 42: block = 64; bytes = 18; return true;
    default: return false;
    }
}

struct Value {
    enum Kind { INTEGER, FLOAT, TEXT, ARRAY } kind = INTEGER;
    uint64_t integer = 0;
    double real = 0.0;
    std::string text;
    std::vector<Value> items;
    bool operator==(const Value &o) const {
        return kind == o.kind && integer == o.integer && real == o.real && text == o.text && items == o.items;
    }
};

struct Directory {
    std::map<std::string, ingot_tensor_info> tensors;
    std::map<std::string, Value> metadata;
};

struct FileReader {
    int fd;
    uint64_t size, pos = 0;
    bool read(void *dst, uint64_t n, const char *what) {
        if (n > size - std::min(pos, size)) { g_error = std::string("truncated GGUF ") + what; return false; }
        uint8_t *p = static_cast<uint8_t *>(dst);
        uint64_t done = 0;
        while (done < n) {
            const ssize_t r = pread(fd, p + done, (size_t)std::min<uint64_t>(n - done, 1u << 30), (off_t)(pos + done));
            if (r < 0 && errno == EINTR) continue;
            if (r <= 0) { g_error = std::string("truncated GGUF ") + what; return false; }
            done += (uint64_t)r;
        }
        pos += n;
        return true;
    }
    bool u32(uint32_t &v) { return read(&v, 4, "value"); }
    bool u64(uint64_t &v) { return read(&v, 8, "value"); }
    bool string(std::string &s) {
        uint64_t n;
        if (!u64(n)) return false;
        if (n > size - std::min(pos, size)) { g_error = "truncated GGUF value"; return false; }
        s.resize((size_t)n);
        return n == 0 || read(&s[0], n, "value");
    }
    bool value(uint32_t kind, Value &out, bool nested) {
        switch (kind) {
        case 8: out.kind = Value::TEXT; return string(out.text);
        case 9: {
            if (nested) { g_error = "nested GGUF arrays"; return false; }
            uint32_t element;
            uint64_t n;
            if (!u32(element)) return false;
            if (element == 9) { g_error = "nested GGUF arrays"; return false; }
            if (!u64(n)) return false;
            if (n > size - std::min(pos, size)) { g_error = "truncated GGUF array"; return false; }
            out.kind = Value::ARRAY;
            out.items.resize((size_t)n);
            for (uint64_t i = 0; i < n; ++i)
                if (!value(element, out.items[(size_t)i], true)) return false;
            return true;
        }
        case 0: case 1: case 7: { uint8_t b; if (!read(&b, 1, "value")) return false; out.integer = b; return true; }
        case 2: case 3: { uint16_t h; if (!read(&h, 2, "value")) return false; out.integer = h; return true; }
        case 4: case 5: { uint32_t w; if (!u32(w)) return false; out.integer = w; return true; }
        case 10: case 11: return u64(out.integer);
        case 6: { uint32_t w; float f; if (!u32(w)) return false; memcpy(&f, &w, 4); out.kind = Value::FLOAT; out.real = f; return true; }
        case 12: { uint64_t w; if (!u64(w)) return false; out.kind = Value::FLOAT; memcpy(&out.real, &w, 8); return true; }
        default: g_error = "unknown GGUF metadata type " + std::to_string(kind); return false;
        }
    }
};

bool mul_overflow(uint64_t a, uint64_t b, uint64_t &out) { return __builtin_mul_overflow(a, b, &out); }

bool read_directory(int fd, uint64_t size, uint32_t shard, Directory &dir) {
    FileReader r{fd, size};
    uint32_t magic, version;
    if (!r.u32(magic) || !r.u32(version)) return false;
    if (magic != 0x46554747u || version != 3u) { g_error = "expected little-endian GGUF v3"; return false; }
    uint64_t nt, nm;
    if (!r.u64(nt) || !r.u64(nm)) return false;
    for (uint64_t i = 0; i < nm; ++i) {
        std::string key;
        uint32_t kind;
        Value v;
        if (!r.string(key) || !r.u32(kind) || !r.value(kind, v, false)) return false;
        if (!dir.metadata.emplace(key, std::move(v)).second) { g_error = "duplicate GGUF metadata"; return false; }
    }
    uint64_t alignment = 32;
    auto al = dir.metadata.find("general.alignment");
    if (al != dir.metadata.end()) {
        if (al->second.kind != Value::INTEGER) { g_error = "invalid alignment metadata"; return false; }
        alignment = al->second.integer;
    }
    if (alignment == 0 || (alignment & (alignment - 1))) { g_error = "invalid GGUF alignment"; return false; }
    for (uint64_t i = 0; i < nt; ++i) {
        std::string name;
        uint32_t rank;
        if (!r.string(name) || !r.u32(rank)) return false;
        if (rank < 1 || rank > 4) { g_error = "invalid tensor rank"; return false; }
        ingot_tensor_info t = {};
        t.rank = rank;
        t.shard = shard;
        bool zero = false;
        for (uint32_t d = 0; d < rank; ++d) {
            if (!r.u64(t.dims[d])) return false;
            zero = zero || t.dims[d] == 0;
        }
        if (!r.u32(t.kind) || !r.u64(t.offset)) return false;
        uint64_t block, bytes;
        if (!directory_geometry(t.kind, block, bytes)) { g_error = "GGML type " + std::to_string(t.kind) + " is unsupported"; return false; }
        if (zero || t.dims[0] % block || t.offset % alignment) { g_error = "invalid shape/alignment for " + name; return false; }
        if (mul_overflow(t.dims[0] / block, bytes, t.stride)) { g_error = "row overflow"; return false; }
        t.bytes = t.stride;
        for (uint32_t d = 1; d < rank; ++d)
            if (mul_overflow(t.bytes, t.dims[d], t.bytes)) { g_error = "tensor overflow"; return false; }
        if (!dir.tensors.emplace(name, t).second) { g_error = "duplicate tensor"; return false; }
    }
    if (r.pos > UINT64_MAX - (alignment - 1)) { g_error = "header overflow"; return false; }
    const uint64_t start = (r.pos + alignment - 1) & ~(alignment - 1);
    std::vector<std::pair<uint64_t, uint64_t>> ranges;
    for (auto &kv : dir.tensors) {
        ingot_tensor_info &t = kv.second;
        if (t.offset > UINT64_MAX - start) { g_error = "offset overflow"; return false; }
        t.offset += start;
        if (t.bytes > UINT64_MAX - t.offset || t.offset + t.bytes > size) { g_error = kv.first + ": extends beyond file"; return false; }
        ranges.emplace_back(t.offset, t.offset + t.bytes);
    }
    std::sort(ranges.begin(), ranges.end());
    for (size_t i = 1; i < ranges.size(); ++i)
        if (ranges[i - 1].second > ranges[i].first) { g_error = "overlapping tensor ranges"; return false; }
    return true;
}

}  // namespace

struct ingot_gguf {
    std::vector<int> files;
    std::map<std::string, ingot_tensor_info> tensors;
    std::vector<const std::string *> order;       // tensor names in map order, for ingot_gguf_tensor_at
    std::map<std::string, Value> metadata;
    std::string architecture;
    uint64_t bytes_read = 0;
    ~ingot_gguf() {
        for (int fd : files)
            if (fd >= 0) close(fd);
    }
};

namespace {

bool open_file(const std::string &path, int &fd, uint64_t &size) {
    fd = open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd < 0) { g_error = path + ": " + strerror(errno); return false; }
    struct stat st;
    if (fstat(fd, &st) != 0) { g_error = path + ": " + strerror(errno); close(fd); fd = -1; return false; }
    size = (uint64_t)st.st_size;
    return true;
}

const Value *find(const ingot_gguf *g, const char *key) {
    auto it = g->metadata.find(key);
    return it == g->metadata.end() ? nullptr : &it->second;
}

// Positional read of `len` bytes at `offset` inside tensor `t`; a short file is INGOT_EOF.
ingot_status read_at(ingot_gguf *g, const ingot_tensor_info &t, uint64_t offset, void *dst, uint64_t len) {
    if (offset > t.bytes || len > t.bytes - offset) return fail(INGOT_INVALID, "tensor read out of bounds");
    if (t.shard >= g->files.size()) return fail(INGOT_INVALID, "invalid tensor shard");
    if (t.offset > UINT64_MAX - offset) return fail(INGOT_INVALID, "tensor offset overflow");
    uint8_t *p = static_cast<uint8_t *>(dst);
    uint64_t done = 0;
    while (done < len) {
        const ssize_t r = pread(g->files[t.shard], p + done, (size_t)std::min<uint64_t>(len - done, 1u << 30), (off_t)(t.offset + offset + done));
        if (r < 0 && errno == EINTR) continue;
        if (r < 0) return fail(INGOT_DEVICE, std::string("read failed: ") + strerror(errno));
        if (r == 0) return fail(INGOT_EOF, "failed to fill whole buffer");
        done += (uint64_t)r;
    }
    g->bytes_read += len;
    return INGOT_OK;
}

}  // namespace

extern "C" {

const char *ingot_gguf_last_error(void) { return g_error.c_str(); }

ingot_status ingot_gguf_open(const char *path, ingot_gguf **out) {
    if (!path || !out) return fail(INGOT_INVALID, "null argument");
    *out = nullptr;
    std::unique_ptr<ingot_gguf> g(new ingot_gguf());
    int fd;
    uint64_t size;
    if (!open_file(path, fd, size)) return INGOT_INVALID;
    g->files.push_back(fd);
    Directory dir;
    if (!read_directory(fd, size, 0, dir)) return INGOT_INVALID;
    g->tensors = std::move(dir.tensors);
    g->metadata = std::move(dir.metadata);
    const Value *arch = find(g.get(), "general.architecture");
    if (!arch || arch->kind != Value::TEXT) return fail(INGOT_INVALID, "missing architecture");
    g->architecture = arch->text;
    const Value *count_v = find(g.get(), "split.count");
    const uint64_t count = count_v && count_v->kind == Value::INTEGER ? count_v->integer : 1;
    if (count > 1) {
        const Value *no = find(g.get(), "split.no");
        if (!no || no->kind != Value::INTEGER) return fail(INGOT_INVALID, "missing integer: split.no");
        if (no->integer != 0) return fail(INGOT_INVALID, "pass the primary GGUF shard");
        const std::string full(path);
        const size_t slash = full.find_last_of('/');
        const std::string folder = slash == std::string::npos ? "" : full.substr(0, slash + 1);
        const std::string name = slash == std::string::npos ? full : full.substr(slash + 1);
        char marker[64];
        snprintf(marker, sizeof marker, "-00001-of-%05llu.gguf", (unsigned long long)count);
        const size_t ml = strlen(marker);
        if (name.size() < ml || name.compare(name.size() - ml, ml, marker) != 0) return fail(INGOT_INVALID, "invalid split filename");
        const std::string prefix = name.substr(0, name.size() - ml);
        const Value *total = find(g.get(), "split.tensors.count");
        for (uint64_t shard = 1; shard < count; ++shard) {
            char tail[64];
            snprintf(tail, sizeof tail, "-%05llu-of-%05llu.gguf", (unsigned long long)(shard + 1), (unsigned long long)count);
            int sfd;
            uint64_t ssize;
            if (!open_file(folder + prefix + tail, sfd, ssize)) return INGOT_INVALID;
            g->files.push_back(sfd);
            Directory d;
            if (!read_directory(sfd, ssize, (uint32_t)shard, d)) return INGOT_INVALID;
            auto same_int = [&](const char *key, uint64_t want) {
                auto it = d.metadata.find(key);
                return it != d.metadata.end() && it->second.kind == Value::INTEGER && it->second.integer == want;
            };
            auto tc = d.metadata.find("split.tensors.count");
            const bool tc_same = (tc == d.metadata.end() && !total) || (tc != d.metadata.end() && total && tc->second == *total);
            if (!same_int("split.no", shard) || !same_int("split.count", count) || !tc_same) return fail(INGOT_INVALID, "inconsistent GGUF shards");
            for (const auto &kv : d.metadata) {
                if (kv.first.compare(0, 6, "split.") == 0) continue;
                const Value *old = find(g.get(), kv.first.c_str());
                if (old && !(*old == kv.second)) return fail(INGOT_INVALID, "inconsistent shard metadata: " + kv.first);
            }
            for (const auto &kv : d.tensors)
                if (!g->tensors.emplace(kv.first, kv.second).second) return fail(INGOT_INVALID, "duplicate tensor across shards");
        }
        if (!total || total->kind != Value::INTEGER) return fail(INGOT_INVALID, "missing integer: split.tensors.count");
        if (total->integer != g->tensors.size()) return fail(INGOT_INVALID, "split tensor count mismatch");
    }
    for (const auto &kv : g->tensors) g->order.push_back(&kv.first);
    *out = g.release();
    return INGOT_OK;
}

void ingot_gguf_close(ingot_gguf *g) { delete g; }

const char *ingot_gguf_architecture(const ingot_gguf *g) { return g ? g->architecture.c_str() : ""; }
uint64_t ingot_gguf_tensor_count(const ingot_gguf *g) { return g ? g->tensors.size() : 0; }
uint64_t ingot_gguf_bytes_read(const ingot_gguf *g) { return g ? g->bytes_read : 0; }

ingot_status ingot_gguf_tensor_at(const ingot_gguf *g, uint64_t index, const char **name, ingot_tensor_info *info) {
    if (!g || index >= g->order.size()) return fail(INGOT_INVALID, "tensor index out of range");
    if (name) *name = g->order[(size_t)index]->c_str();
    if (info) *info = g->tensors.find(*g->order[(size_t)index])->second;
    return INGOT_OK;
}

ingot_status ingot_gguf_tensor(const ingot_gguf *g, const char *name, ingot_tensor_info *info) {
    if (!g || !name) return fail(INGOT_INVALID, "null argument");
    auto it = g->tensors.find(name);
    if (it == g->tensors.end()) return fail(INGOT_INVALID, std::string("missing tensor: ") + name);
    if (info) *info = it->second;
    return INGOT_OK;
}

ingot_status ingot_gguf_integer(const ingot_gguf *g, const char *key, uint64_t *value) {
    const Value *v = g && key ? find(g, key) : nullptr;
    if (!v || v->kind != Value::INTEGER) return fail(INGOT_INVALID, std::string("missing integer: ") + (key ? key : ""));
    if (value) *value = v->integer;
    return INGOT_OK;
}

ingot_status ingot_gguf_float(const ingot_gguf *g, const char *key, float *value) {
    const Value *v = g && key ? find(g, key) : nullptr;
    const float f = v && v->kind == Value::FLOAT ? (float)v->real : 0.f;
    if (!v || v->kind != Value::FLOAT || !(f - f == 0.f)) return fail(INGOT_INVALID, std::string("missing float: ") + (key ? key : ""));
    if (value) *value = f;
    return INGOT_OK;
}

ingot_status ingot_gguf_string(const ingot_gguf *g, const char *key, const char **value) {
    const Value *v = g && key ? find(g, key) : nullptr;
    if (!v || v->kind != Value::TEXT) return fail(INGOT_INVALID, std::string("missing string: ") + (key ? key : ""));
    if (value) *value = v->text.c_str();
    return INGOT_OK;
}

ingot_status ingot_gguf_array_length(const ingot_gguf *g, const char *key, uint64_t *length) {
    const Value *v = g && key ? find(g, key) : nullptr;
    if (!v || v->kind != Value::ARRAY) return fail(INGOT_INVALID, std::string("missing array: ") + (key ? key : ""));
    if (length) *length = v->items.size();
    return INGOT_OK;
}

ingot_status ingot_gguf_array_integer(const ingot_gguf *g, const char *key, uint64_t index, uint64_t *value) {
    const Value *v = g && key ? find(g, key) : nullptr;
    if (!v || v->kind != Value::ARRAY) return fail(INGOT_INVALID, std::string("missing array: ") + (key ? key : ""));
    if (index >= v->items.size() || v->items[(size_t)index].kind != Value::INTEGER) return fail(INGOT_INVALID, key);
    if (value) *value = v->items[(size_t)index].integer;
    return INGOT_OK;
}

ingot_status ingot_gguf_array_string(const ingot_gguf *g, const char *key, uint64_t index, const char **value) {
    const Value *v = g && key ? find(g, key) : nullptr;
    if (!v || v->kind != Value::ARRAY) return fail(INGOT_INVALID, std::string("missing array: ") + (key ? key : ""));
    if (index >= v->items.size() || v->items[(size_t)index].kind != Value::TEXT) return fail(INGOT_INVALID, key);
    if (value) *value = v->items[(size_t)index].text.c_str();
    return INGOT_OK;
}

ingot_status ingot_gguf_read_range(ingot_gguf *g, const ingot_tensor_info *t, uint64_t offset, void *dst, uint64_t len) {
    if (!g || !t || (!dst && len)) return fail(INGOT_INVALID, "null argument");
    return read_at(g, *t, offset, dst, len);
}

ingot_status ingot_gguf_rows(ingot_gguf *g, const char *name, const uint64_t *rows, uint64_t n, void *dst) {
    ingot_tensor_info t;
    ingot_status st = ingot_gguf_tensor(g, name, &t);
    if (st) return st;
    const uint64_t total = t.bytes / t.stride;
    if (n == 0 || !rows || !dst) return fail(INGOT_INVALID, "row out of range");
    for (uint64_t i = 0; i < n; ++i)
        if (rows[i] >= total) return fail(INGOT_INVALID, "row out of range");
    uint64_t len;
    if (mul_overflow(t.stride, n, len)) return fail(INGOT_INVALID, "rows overflow");
    // every row is attempted (the reference drains all its read jobs) and the first failure is reported
    ingot_status first = INGOT_OK;
    std::string first_msg;
    for (uint64_t i = 0; i < n; ++i) {
        st = read_at(g, t, rows[i] * t.stride, static_cast<uint8_t *>(dst) + i * t.stride, t.stride);
        if (st && !first) { first = st; first_msg = g_error; }
    }
    if (first) return fail(first, first_msg);
    return INGOT_OK;
}

ingot_status ingot_gguf_matrix(ingot_gguf *g, const char *name, const uint64_t *shape, uint32_t rank, const uint64_t *experts,
                               uint64_t n_experts, void *dst) {
    ingot_tensor_info t;
    ingot_status st = ingot_gguf_tensor(g, name, &t);
    if (st) return st;
    bool same = shape && rank == t.rank;
    for (uint32_t d = 0; same && d < rank; ++d) same = shape[d] == t.dims[d];
    if (!same) return fail(INGOT_INVALID, std::string(name) + ": shape differs from the file's");
    const uint64_t rows = rank > 1 ? shape[1] : 1, count = rank > 2 ? shape[2] : 1;
    if (n_experts == 0 || !experts || !dst) return fail(INGOT_INVALID, "expert out of range");
    for (uint64_t i = 0; i < n_experts; ++i)
        if (experts[i] >= count) return fail(INGOT_INVALID, "expert out of range");
    const uint64_t size = t.stride * rows;
    for (uint64_t i = 0; i < n_experts; ++i)
        if ((st = read_at(g, t, experts[i] * size, static_cast<uint8_t *>(dst) + i * size, size))) return st;
    return INGOT_OK;
}

ingot_status ingot_weight_load(ingot_gpu *gpu, ingot_gguf *g, const char *name, const uint64_t *shape, uint32_t rank, void **device,
                               ingot_tensor_info *info) {
    if (!gpu || !device) return fail(INGOT_INVALID, "null argument");
    *device = nullptr;
    ingot_tensor_info t;
    ingot_status st = ingot_gguf_tensor(g, name, &t);
    if (st) return st;
    bool same = shape && rank == t.rank;
    for (uint32_t d = 0; same && d < rank; ++d) same = shape[d] == t.dims[d];
    if (!same) return fail(INGOT_INVALID, std::string(name) + ": shape differs from the file's");
    if (t.rank > 3) return fail(INGOT_INVALID, std::string(name) + ": weights have at most three dimensions (cols, rows, experts)");
    void *host = nullptr;
    if ((st = ingot_host_alloc(gpu, (size_t)t.bytes, &host))) return fail(st, ingot_last_error(gpu));
    st = read_at(g, t, 0, host, t.bytes);
    if (!st) {
        st = ingot_weight_upload(gpu, host, t.kind, t.dims[0], t.rank > 1 ? t.dims[1] : 1, t.rank > 2 ? t.dims[2] : 1, (size_t)t.bytes, device);
        if (!st) st = ingot_synchronize(gpu);          // the staging buffer goes away below
        if (st) g_error = ingot_last_error(gpu);
    }
    ingot_host_free(gpu, host);
    if (!st && info) *info = t;
    return st;
}

}  // extern "C"
