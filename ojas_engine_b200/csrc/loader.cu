// Loader-side pieces of the weight path (host code only): a GGUF tensor directory and a cache file of repacked
// weights.  Counterparts of the reference's reader (crates/ojas-formats/src/gguf.rs:158-205, 298-455: header, metadata,
// tensor infos, data offset) and of its requantized-weight cache keyed to the source file by size and modification
// time (crates/ojas-models/src/weights.rs:14-32, "OJASWC01").  The cache here holds this library's tile layout, so a
// second load of a model is a read of ready-to-upload bytes: every Q4_K / Q6_K / Q8_0 matrix of the GGUF, re-laid once.
//
// Cache file (little-endian):  header 64 B: magic "OJB2WC01", src_size u64, src_mtime u64, index_off u64, entries u64,
// zeros; entry payloads, each starting on a 256-byte boundary; index at index_off: per entry name_len u32, name,
// ggml_type u32, N u64, K u64, offset u64, bytes u64.
#include <errno.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "common.cuh"

namespace {
struct TensorInfo {
    std::string name;
    uint32_t type = 0, ndims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint64_t rel_offset = 0, offset = 0, bytes = 0;
};

// bytes per block and weights per block of the ggml tensor types (the public GGUF table); 0 = unknown
void ggml_block(uint32_t t, uint64_t &bytes, uint64_t &weights) {
    static const struct { uint32_t t; uint32_t b, w; } tab[] = {
        {0, 4, 1}, {1, 2, 1}, {2, 18, 32}, {3, 20, 32}, {6, 22, 32}, {7, 24, 32}, {8, 34, 32}, {9, 36, 32}, {10, 84, 256}, {11, 110, 256},
        {12, 144, 256}, {13, 176, 256}, {14, 210, 256}, {15, 292, 256}, {16, 66, 256}, {17, 74, 256}, {18, 98, 256}, {19, 50, 256},
        {20, 18, 32}, {21, 110, 256}, {22, 82, 256}, {23, 136, 256}, {24, 1, 1}, {25, 2, 1}, {26, 4, 1}, {27, 8, 1}, {28, 8, 1},
        {29, 56, 256}, {30, 2, 1}};
    bytes = weights = 0;
    for (const auto &e : tab)
        if (e.t == t) { bytes = e.b; weights = e.w; }
}

struct Reader {
    int fd = -1;
    uint64_t pos = 0, end = 0;
    bool ok = true;
    bool get(void *dst, size_t n) {
        if (!ok || n > end - pos) { ok = false; return false; }
        size_t done = 0;
        while (done < n) {
            const ssize_t r = pread(fd, (char *)dst + done, n - done, (off_t)(pos + done));
            if (r <= 0) { ok = false; return false; }
            done += (size_t)r;
        }
        pos += n;
        return true;
    }
    template <typename T> T num() { T v{}; get(&v, sizeof v); return v; }
    std::string str() {
        const uint64_t n = num<uint64_t>();
        if (!ok || n > (16u << 20) || n > end - pos) { ok = false; return std::string(); }
        std::string s((size_t)n, '\0');
        get(&s[0], (size_t)n);
        return s;
    }
    void skip(uint64_t n) { if (!ok || n > end - pos) ok = false; else pos += n; }
};

// Skips one metadata value of GGUF type t; *u32_out receives it when it is an unsigned 32-bit scalar.
void skip_value(Reader &r, uint32_t t, uint32_t *u32_out, int depth) {
    static const int size[] = {1, 1, 2, 2, 4, 4, 4, 1, -1, -2, 8, 8, 8};
    if (t > 12) { r.ok = false; return; }
    if (size[t] > 0) {
        if (t == 4 && u32_out) *u32_out = r.num<uint32_t>();
        else r.skip((uint64_t)size[t]);
    } else if (size[t] == -1) {
        r.str();
    } else {
        const uint32_t et = r.num<uint32_t>();
        const uint64_t n = r.num<uint64_t>();
        if (depth > 0 || et > 12 || et == 9) { r.ok = false; return; }
        if (et != 8 && size[et] > 0) r.skip(n * (uint64_t)size[et]);
        else for (uint64_t i = 0; i < n && r.ok; i++) skip_value(r, et, nullptr, depth + 1);
    }
}
}  // namespace

struct ojas_b200_gguf {
    int fd = -1;
    uint64_t file_size = 0, mtime = 0;
    uint32_t version = 0;
    std::vector<TensorInfo> tensors;
};

static int set_err(char *err, size_t n, const char *msg) {
    if (err && n) snprintf(err, n, "%s", msg);
    return OJAS_B200_E_ARG;
}

extern "C" int ojas_b200_gguf_open(const char *path, ojas_b200_gguf **out, char *err, size_t errlen) {
    if (!path || !out) return OJAS_B200_E_ARG;
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return set_err(err, errlen, "cannot open the file");
    struct stat st;
    if (fstat(fd, &st) != 0) { close(fd); return set_err(err, errlen, "cannot stat the file"); }
    Reader r;
    r.fd = fd; r.end = (uint64_t)st.st_size;
    char magic[4] = {0};
    r.get(magic, 4);
    if (!r.ok || memcmp(magic, "GGUF", 4) != 0) { close(fd); return set_err(err, errlen, "not a GGUF file"); }
    ojas_b200_gguf *g = new ojas_b200_gguf();
    g->fd = fd; g->file_size = (uint64_t)st.st_size; g->mtime = (uint64_t)st.st_mtime;
    g->version = r.num<uint32_t>();
    const uint64_t n_tensors = r.num<uint64_t>(), n_kv = r.num<uint64_t>();
    if (!r.ok || (g->version != 2 && g->version != 3) || n_tensors > (1u << 20) || n_kv > (1u << 20)) {
        close(fd); delete g;
        return set_err(err, errlen, "unsupported GGUF version or implausible header counts");
    }
    uint32_t align = 32;
    for (uint64_t i = 0; i < n_kv && r.ok; i++) {
        const std::string key = r.str();
        const uint32_t t = r.num<uint32_t>();
        uint32_t v = 0;
        skip_value(r, t, key == "general.alignment" ? &v : nullptr, 0);
        if (key == "general.alignment" && t == 4 && v) align = v;
    }
    if (!r.ok || (align & (align - 1)) != 0) { close(fd); delete g; return set_err(err, errlen, "malformed GGUF metadata"); }
    g->tensors.resize((size_t)n_tensors);
    for (auto &ti : g->tensors) {
        ti.name = r.str();
        ti.ndims = r.num<uint32_t>();
        if (!r.ok || ti.ndims < 1 || ti.ndims > 4) { r.ok = false; break; }
        for (uint32_t d = 0; d < ti.ndims; d++) ti.dims[d] = r.num<uint64_t>();
        ti.type = r.num<uint32_t>();
        ti.rel_offset = r.num<uint64_t>();
        uint64_t bb, bw;
        ggml_block(ti.type, bb, bw);
        uint64_t elems = 1;
        for (uint32_t d = 0; d < ti.ndims; d++) {
            if (ti.dims[d] == 0 || elems > (~0ull >> 8) / ti.dims[d]) { r.ok = false; break; }
            elems *= ti.dims[d];
        }
        ti.bytes = bw ? (elems / bw) * bb : 0;          // 0: a type this table does not know
        if (bw && ti.dims[0] % bw != 0) r.ok = false;
    }
    if (!r.ok) { close(fd); delete g; return set_err(err, errlen, "malformed GGUF tensor directory"); }
    const uint64_t data_offset = (r.pos + align - 1) & ~(uint64_t)(align - 1);
    for (auto &ti : g->tensors) {
        ti.offset = data_offset + ti.rel_offset;
        if (ti.offset > g->file_size || ti.bytes > g->file_size - ti.offset) {
            close(fd); delete g;
            return set_err(err, errlen, "a GGUF tensor extends beyond the file");
        }
    }
    *out = g;
    return 0;
}

extern "C" void ojas_b200_gguf_close(ojas_b200_gguf *g) {
    if (!g) return;
    if (g->fd >= 0) close(g->fd);
    delete g;
}

extern "C" size_t ojas_b200_gguf_tensor_count(const ojas_b200_gguf *g) { return g ? g->tensors.size() : 0; }

// dims as GGUF stores them: dims[0] = K (the contiguous, input dimension), dims[1] = N (rows = outputs).
extern "C" int ojas_b200_gguf_tensor_info(const ojas_b200_gguf *g, size_t index, const char **name, uint32_t *ggml_type, uint32_t *ndims,
                                          uint64_t dims[4], uint64_t *file_offset, uint64_t *bytes) {
    if (!g || index >= g->tensors.size()) return OJAS_B200_E_ARG;
    const TensorInfo &t = g->tensors[index];
    if (name) *name = t.name.c_str();
    if (ggml_type) *ggml_type = t.type;
    if (ndims) *ndims = t.ndims;
    if (dims) for (int d = 0; d < 4; d++) dims[d] = t.dims[d];
    if (file_offset) *file_offset = t.offset;
    if (bytes) *bytes = t.bytes;
    return 0;
}

extern "C" long long ojas_b200_gguf_find(const ojas_b200_gguf *g, const char *name) {
    if (!g || !name) return -1;
    for (size_t i = 0; i < g->tensors.size(); i++)
        if (g->tensors[i].name == name) return (long long)i;
    return -1;
}

// The tensor's payload as stored (GGUF blocks, rows contiguous): what ojas_b200_repack / _repack_host take.
extern "C" int ojas_b200_gguf_read_raw(const ojas_b200_gguf *g, size_t index, void *dst, size_t bytes) {
    if (!g || index >= g->tensors.size() || !dst) return OJAS_B200_E_ARG;
    const TensorInfo &t = g->tensors[index];
    if (t.bytes == 0 || bytes != t.bytes) return OJAS_B200_E_ARG;
    Reader r;
    r.fd = g->fd; r.pos = t.offset; r.end = g->file_size;
    return r.get(dst, bytes) ? 0 : OJAS_B200_E_ARG;
}

// ---------------------------------------------------------------------------- repacked-weight cache
struct CacheEntry { std::string name; uint32_t type; uint64_t N, K, offset, bytes; };
struct ojas_b200_weight_cache {
    int fd = -1;
    uint8_t *map = nullptr;
    uint64_t map_bytes = 0;
    std::vector<CacheEntry> entries;
};
static const char kCacheMagic[8] = {'O', 'J', 'B', '2', 'W', 'C', '0', '1'};

static bool write_all(int fd, const void *p, size_t n) {
    size_t done = 0;
    while (done < n) {
        const ssize_t w = write(fd, (const char *)p + done, n - done);
        if (w <= 0) return false;
        done += (size_t)w;
    }
    return true;
}

// Re-lays every Q4_K / Q6_K / Q8_0 matrix of the GGUF (rank 2, or rank 3 = experts stacked along the last dimension,
// whose row count must then be a multiple of 8) and writes the cache file.  Other tensors are left to the caller.
extern "C" int ojas_b200_weight_cache_build(const char *gguf_path, const char *cache_path, char *err, size_t errlen) {
    if (!gguf_path || !cache_path) return OJAS_B200_E_ARG;
    ojas_b200_gguf *g = nullptr;
    int rc = ojas_b200_gguf_open(gguf_path, &g, err, errlen);
    if (rc) return rc;
    const std::string tmp = std::string(cache_path) + ".part";
    const int fd = open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) { ojas_b200_gguf_close(g); return set_err(err, errlen, "cannot create the cache file"); }
    uint64_t header[8] = {0, g->file_size, g->mtime, 0, 0, 0, 0, 0};
    memcpy(&header[0], kCacheMagic, 8);
    bool ok = write_all(fd, header, sizeof header);
    uint64_t pos = sizeof header;
    std::vector<CacheEntry> entries;
    std::vector<uint8_t> raw, packed;
    static const uint8_t zeros[256] = {0};
    for (size_t i = 0; ok && i < g->tensors.size(); i++) {
        const TensorInfo &t = g->tensors[i];
        if (!type_supported(t.type) || t.ndims < 2 || t.ndims > 3 || t.dims[0] % 256 != 0) continue;
        const uint64_t K = t.dims[0], rows = t.dims[1], experts = t.ndims == 3 ? t.dims[2] : 1;
        if (experts > 1 && rows % OJAS_TILE_ROWS != 0) continue;       // stacked experts must start on tile boundaries
        const uint64_t N = rows * experts;
        raw.resize((size_t)t.bytes);
        packed.resize(ojas_b200_repacked_bytes(t.type, (size_t)N, (size_t)K));
        if (ojas_b200_gguf_read_raw(g, i, raw.data(), raw.size()) != 0 || ojas_b200_repack_host(t.type, raw.data(), (size_t)N, (size_t)K, packed.data()) != 0) {
            ok = false;
            break;
        }
        const uint64_t pad = (256 - pos % 256) % 256;
        ok = write_all(fd, zeros, (size_t)pad) && write_all(fd, packed.data(), packed.size());
        pos += pad;
        entries.push_back(CacheEntry{t.name, t.type, N, K, pos, (uint64_t)packed.size()});
        pos += packed.size();
    }
    const uint64_t index_off = pos;
    for (size_t i = 0; ok && i < entries.size(); i++) {
        const CacheEntry &e = entries[i];
        const uint32_t nl = (uint32_t)e.name.size();
        const uint64_t nums[4] = {e.N, e.K, e.offset, e.bytes};
        ok = write_all(fd, &nl, 4) && write_all(fd, e.name.data(), nl) && write_all(fd, &e.type, 4) && write_all(fd, nums, sizeof nums);
    }
    header[3] = index_off;
    header[4] = entries.size();
    ok = ok && pwrite(fd, header, sizeof header, 0) == (ssize_t)sizeof header && fsync(fd) == 0;
    close(fd);
    ojas_b200_gguf_close(g);
    if (!ok || rename(tmp.c_str(), cache_path) != 0) {
        unlink(tmp.c_str());
        return set_err(err, errlen, "writing the cache file failed");
    }
    return 0;
}

// Maps a cache file.  With gguf_path given, the cache must have been built from that very file (same size and
// modification time); otherwise OJAS_B200_E_UNSUPPORTED tells the caller to rebuild.
extern "C" int ojas_b200_weight_cache_open(const char *cache_path, const char *gguf_path, ojas_b200_weight_cache **out, char *err, size_t errlen) {
    if (!cache_path || !out) return OJAS_B200_E_ARG;
    *out = nullptr;
    const int fd = open(cache_path, O_RDONLY);
    if (fd < 0) return set_err(err, errlen, "cannot open the cache file");
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 64) { close(fd); return set_err(err, errlen, "the cache file is too short"); }
    void *m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (m == MAP_FAILED) { close(fd); return set_err(err, errlen, "cannot map the cache file"); }
    ojas_b200_weight_cache *c = new ojas_b200_weight_cache();
    c->fd = fd; c->map = (uint8_t *)m; c->map_bytes = (uint64_t)st.st_size;
    auto fail = [&](const char *msg, int code) {
        munmap(c->map, (size_t)c->map_bytes);
        close(fd);
        delete c;
        set_err(err, errlen, msg);
        return code;
    };
    uint64_t header[8];
    memcpy(header, c->map, sizeof header);
    if (memcmp(&header[0], kCacheMagic, 8) != 0) return fail("not a repacked-weight cache of this library", OJAS_B200_E_ARG);
    if (gguf_path) {
        struct stat gs;
        if (stat(gguf_path, &gs) != 0) return fail("cannot stat the source GGUF", OJAS_B200_E_ARG);
        if ((uint64_t)gs.st_size != header[1] || (uint64_t)gs.st_mtime != header[2])
            return fail("the cache was built from another version of the source file: rebuild it", OJAS_B200_E_UNSUPPORTED);
    }
    uint64_t pos = header[3];
    for (uint64_t i = 0; i < header[4]; i++) {
        uint32_t nl = 0;
        if (pos + 4 > c->map_bytes) return fail("the cache index is truncated", OJAS_B200_E_ARG);
        memcpy(&nl, c->map + pos, 4);
        pos += 4;
        if (nl > 4096 || pos + nl + 4 + 32 > c->map_bytes) return fail("the cache index is truncated", OJAS_B200_E_ARG);
        CacheEntry e;
        e.name.assign((const char *)c->map + pos, nl);
        pos += nl;
        memcpy(&e.type, c->map + pos, 4);
        pos += 4;
        uint64_t nums[4];
        memcpy(nums, c->map + pos, sizeof nums);
        pos += sizeof nums;
        e.N = nums[0]; e.K = nums[1]; e.offset = nums[2]; e.bytes = nums[3];
        if (e.offset % 256 != 0 || e.offset > c->map_bytes || e.bytes > c->map_bytes - e.offset) return fail("a cache entry lies outside the file", OJAS_B200_E_ARG);
        c->entries.push_back(e);
    }
    *out = c;
    return 0;
}

extern "C" void ojas_b200_weight_cache_close(ojas_b200_weight_cache *c) {
    if (!c) return;
    munmap(c->map, (size_t)c->map_bytes);
    close(c->fd);
    delete c;
}

extern "C" size_t ojas_b200_weight_cache_count(const ojas_b200_weight_cache *c) { return c ? c->entries.size() : 0; }

// Entry i: its name, type, shape [N, K] and the repacked bytes (a pointer into the mapping: ready for an upload).
extern "C" int ojas_b200_weight_cache_entry(const ojas_b200_weight_cache *c, size_t index, const char **name, uint32_t *ggml_type, uint64_t *N,
                                            uint64_t *K, const void **data, uint64_t *bytes) {
    if (!c || index >= c->entries.size()) return OJAS_B200_E_ARG;
    const CacheEntry &e = c->entries[index];
    if (name) *name = e.name.c_str();
    if (ggml_type) *ggml_type = e.type;
    if (N) *N = e.N;
    if (K) *K = e.K;
    if (data) *data = c->map + e.offset;
    if (bytes) *bytes = e.bytes;
    return 0;
}
