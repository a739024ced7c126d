// Weight loading for the W4A16 path: a safetensors reader for compressed-tensors `pack-quantized` checkpoints, the
// streamed upload that re-tiles a linear chunk by chunk, and the on-disk cache of the re-tiled (T64) layout.
//
// Mirrors, on the host side of the C ABI:
//   * crates/core/src/st.rs:115-360   -- archive of model*.safetensors shards: 8-byte header length, JSON header
//     {name: {dtype, shape, data_offsets}}, offsets checked against shape x dtype size;
//   * crates/core/src/w4a16.rs:108-191 -- every `<base>.weight_packed` (I32 [n, k/8]) must come with
//     `<base>.weight_scale` (F16 or BF16 [n, k/group]) and `<base>.weight_shape` (I64 [2]); group in {32, 64, 128};
//   * crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:1643 (upload_lin_g_stream: the caller fills pinned chunks
//     through a callback) and :99-179 (the repack that follows every load).
// Where the reference repacks on the host at every load, the re-tiled bytes can be written to a cache file once and
// read back with plain host-to-device copies: no staging copy, no repack kernel.
#include <dirent.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/w4a16_b200.h"
#include "dec.h"

namespace {

thread_local std::string g_st_error;

// ---- a JSON reader just large enough for safetensors headers ---------------------------------------------------
struct JsonCursor {
    const char* p;
    const char* end;
    bool fail = false;
    void ws() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) {
            ++p;
        }
    }
    bool eat(char c) {
        ws();
        if (p < end && *p == c) {
            ++p;
            return true;
        }
        return false;
    }
    bool string(std::string& out) {
        ws();
        if (p >= end || *p != '"') {
            return fail = true, false;
        }
        ++p;
        out.clear();
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                ++p;
                switch (*p) {
                case 'n': out.push_back('\n'); break;
                case 't': out.push_back('\t'); break;
                case 'u': out.push_back('?'); p += 4; break;   // names of tensors are ASCII; keep the length right
                default: out.push_back(*p); break;
                }
                ++p;
            } else {
                out.push_back(*p++);
            }
        }
        if (p >= end) {
            return fail = true, false;
        }
        ++p;
        return true;
    }
    bool number(double& v) {
        ws();
        char* e = nullptr;
        v = strtod(p, &e);
        if (e == p) {
            return fail = true, false;
        }
        p = e;
        return true;
    }
    // skips any value
    void skip() {
        ws();
        if (p >= end) {
            fail = true;
            return;
        }
        if (*p == '"') {
            std::string s;
            string(s);
        } else if (*p == '{' || *p == '[') {
            const char open = *p, close = open == '{' ? '}' : ']';
            ++p;
            ws();
            if (eat(close)) {
                return;
            }
            for (;;) {
                if (open == '{') {
                    std::string k;
                    if (!string(k) || !eat(':')) {
                        fail = true;
                        return;
                    }
                }
                skip();
                if (fail) {
                    return;
                }
                if (eat(',')) {
                    continue;
                }
                if (eat(close)) {
                    return;
                }
                fail = true;
                return;
            }
        } else {
            while (p < end && *p != ',' && *p != '}' && *p != ']') {
                ++p;
            }
        }
    }
    bool num_array(std::vector<uint64_t>& out) {
        out.clear();
        if (!eat('[')) {
            return fail = true, false;
        }
        if (eat(']')) {
            return true;
        }
        for (;;) {
            double v;
            if (!number(v) || v < 0) {
                return fail = true, false;
            }
            out.push_back((uint64_t)v);
            if (eat(',')) {
                continue;
            }
            if (eat(']')) {
                return true;
            }
            return fail = true, false;
        }
    }
};

enum StDtype { ST_I32, ST_I64, ST_F16, ST_BF16, ST_F32, ST_OTHER };

struct StEntry {
    StDtype dtype = ST_OTHER;
    int dtype_bytes = 0;
    std::vector<uint64_t> shape;
    uint64_t begin = 0, end = 0;
    int shard = 0;
};

struct StShard {
    std::string path;
    int fd = -1;
    const unsigned char* map = nullptr;
    size_t map_len = 0;
    uint64_t data_base = 0, data_len = 0;
};

struct LinInfo {
    std::string base;
    int n = 0, k = 0, group = 0, scale_bf16 = 0;
};

int dtype_of(const std::string& s, StDtype* d) {
    if (s == "I32") return *d = ST_I32, 4;
    if (s == "I64") return *d = ST_I64, 8;
    if (s == "F16") return *d = ST_F16, 2;
    if (s == "BF16") return *d = ST_BF16, 2;
    if (s == "F32") return *d = ST_F32, 4;
    *d = ST_OTHER;
    if (s == "F64" || s == "U64") return 8;
    if (s == "U32") return 4;
    if (s == "I16" || s == "U16") return 2;
    if (s == "I8" || s == "U8" || s == "BOOL" || s == "F8_E4M3" || s == "F8_E5M2") return 1;
    return 0;
}

}  // namespace

struct w4a16_st {
    std::vector<StShard> shards;
    std::map<std::string, StEntry> entries;
    std::vector<LinInfo> lins;
    ~w4a16_st() {
        for (auto& s : shards) {
            if (s.map) {
                munmap((void*)s.map, s.map_len);
            }
            if (s.fd >= 0) {
                close(s.fd);
            }
        }
    }
    const unsigned char* data(const StEntry& e) const { return shards[e.shard].map + shards[e.shard].data_base + e.begin; }
};

namespace {

int st_fail(const std::string& msg) {
    g_st_error = msg;
    return 1;
}

// One shard: st.rs:213-290.
int parse_shard(w4a16_st& ar, const std::string& path) {
    StShard sh;
    sh.path = path;
    sh.fd = open(path.c_str(), O_RDONLY);
    if (sh.fd < 0) {
        return st_fail(path + ": cannot open");
    }
    struct stat stt;
    if (fstat(sh.fd, &stt) != 0 || stt.st_size < 8) {
        close(sh.fd);
        return st_fail(path + ": too short for a safetensors file");
    }
    sh.map_len = (size_t)stt.st_size;
    void* m = mmap(nullptr, sh.map_len, PROT_READ, MAP_PRIVATE, sh.fd, 0);
    if (m == MAP_FAILED) {
        close(sh.fd);
        return st_fail(path + ": mmap failed");
    }
    sh.map = (const unsigned char*)m;
    uint64_t hlen = 0;
    memcpy(&hlen, sh.map, 8);   // little endian
    if (hlen == 0 || hlen > (1ull << 30) || 8 + hlen > sh.map_len) {
        munmap(m, sh.map_len);
        close(sh.fd);
        return st_fail(path + ": header len " + std::to_string(hlen));
    }
    sh.data_base = 8 + hlen;
    sh.data_len = sh.map_len - sh.data_base;
    const int shard_index = (int)ar.shards.size();
    ar.shards.push_back(sh);
    JsonCursor c{(const char*)sh.map + 8, (const char*)sh.map + 8 + hlen};
    if (!c.eat('{')) {
        return st_fail(path + ": header not an object");
    }
    if (c.eat('}')) {
        return 0;
    }
    for (;;) {
        std::string name;
        if (!c.string(name) || !c.eat(':')) {
            return st_fail(path + ": malformed header");
        }
        if (name == "__metadata__") {
            c.skip();
        } else {
            StEntry e;
            e.shard = shard_index;
            bool have_dtype = false, have_shape = false, have_offs = false;
            std::vector<uint64_t> offs;
            if (!c.eat('{')) {
                return st_fail(name + ": entry not an object");
            }
            if (!c.eat('}')) {
                for (;;) {
                    std::string key;
                    if (!c.string(key) || !c.eat(':')) {
                        return st_fail(name + ": malformed entry");
                    }
                    if (key == "dtype") {
                        std::string d;
                        if (!c.string(d)) {
                            return st_fail(name + ": dtype");
                        }
                        e.dtype_bytes = dtype_of(d, &e.dtype);
                        if (e.dtype_bytes == 0) {
                            return st_fail(name + ": unknown dtype " + d);
                        }
                        have_dtype = true;
                    } else if (key == "shape") {
                        if (!c.num_array(e.shape)) {
                            return st_fail(name + ": shape");
                        }
                        have_shape = true;
                    } else if (key == "data_offsets") {
                        if (!c.num_array(offs)) {
                            return st_fail(name + ": data_offsets");
                        }
                        have_offs = true;
                    } else {
                        c.skip();
                    }
                    if (c.fail) {
                        return st_fail(name + ": malformed entry");
                    }
                    if (c.eat(',')) {
                        continue;
                    }
                    if (c.eat('}')) {
                        break;
                    }
                    return st_fail(name + ": malformed entry");
                }
            }
            if (!have_dtype || !have_shape || !have_offs || offs.size() != 2) {
                return st_fail(name + ": dtype / shape / data_offsets missing");
            }
            uint64_t numel = 1;
            for (uint64_t d : e.shape) {
                if (d != 0 && numel > (~0ull) / d) {
                    return st_fail(name + ": numel overflow");
                }
                numel *= d;
            }
            if (offs[1] < offs[0]) {
                return st_fail(name + ": data_offsets reversed");
            }
            if (offs[1] - offs[0] != numel * (uint64_t)e.dtype_bytes) {
                return st_fail(name + ": bytes " + std::to_string(offs[1] - offs[0]) + " != numel " +
                               std::to_string(numel) + " x " + std::to_string(e.dtype_bytes));
            }
            if (offs[1] > sh.data_len) {
                return st_fail(name + ": data beyond the end of the file");
            }
            e.begin = offs[0];
            e.end = offs[1];
            if (!ar.entries.emplace(name, e).second) {
                return st_fail(name + ": duplicate tensor name");
            }
        }
        if (c.fail) {
            return st_fail(path + ": malformed header");
        }
        if (c.eat(',')) {
            continue;
        }
        if (c.eat('}')) {
            return 0;
        }
        return st_fail(path + ": malformed header");
    }
}

// Every <base>.weight_packed with its scale and shape tensors: w4a16.rs:124-175.
int collect_linears(w4a16_st& ar) {
    static const std::string suffix = ".weight_packed";
    for (const auto& kv : ar.entries) {
        const std::string& name = kv.first;
        if (name.size() <= suffix.size() || name.compare(name.size() - suffix.size(), suffix.size(), suffix) != 0) {
            continue;
        }
        const std::string base = name.substr(0, name.size() - suffix.size());
        const StEntry& pk = kv.second;
        auto isc = ar.entries.find(base + ".weight_scale"), ish = ar.entries.find(base + ".weight_shape");
        if (isc == ar.entries.end()) {
            return st_fail(base + ": weight_scale missing");
        }
        if (ish == ar.entries.end()) {
            return st_fail(base + ": weight_shape missing");
        }
        const StEntry &sc = isc->second, &shp = ish->second;
        if (pk.dtype != ST_I32) {
            return st_fail(base + ": weight_packed is not I32");
        }
        if (sc.dtype != ST_F16 && sc.dtype != ST_BF16) {
            return st_fail(base + ": weight_scale is neither F16 nor BF16");
        }
        if (shp.dtype != ST_I64) {
            return st_fail(base + ": weight_shape is not I64");
        }
        if (pk.shape.size() != 2 || sc.shape.size() != 2 || shp.shape.size() != 1 || shp.shape[0] != 2) {
            return st_fail(base + ": rank contract violated");
        }
        const uint64_t n = pk.shape[0], k = pk.shape[1] * 8;
        if (n == 0 || k == 0 || sc.shape[0] != n || sc.shape[1] == 0 || k % sc.shape[1] != 0 || n > 0x7fffffff ||
            k > 0x7fffffff) {
            return st_fail(base + ": scale shape does not match [n, k/group]");
        }
        const uint64_t group = k / sc.shape[1];
        if (group != 32 && group != 64 && group != 128) {
            return st_fail(base + ": group " + std::to_string(group) + " (only 32, 64, 128)");
        }
        int64_t dims[2];
        memcpy(dims, ar.data(shp), 16);
        if ((uint64_t)dims[0] != n || (uint64_t)dims[1] != k) {
            return st_fail(base + ": weight_shape disagrees with weight_packed");
        }
        LinInfo li;
        li.base = base;
        li.n = (int)n;
        li.k = (int)k;
        li.group = (int)group;
        li.scale_bf16 = sc.dtype == ST_BF16;
        ar.lins.push_back(li);
    }
    return 0;
}

const LinInfo* find_info(const w4a16_st* st, const char* base) {
    for (const auto& li : st->lins) {
        if (li.base == base) {
            return &li;
        }
    }
    return nullptr;
}

uint64_t fnv1a(const unsigned char* p, size_t len, uint64_t h) {
    for (size_t i = 0; i < len; ++i) {
        h = (h ^ p[i]) * 1099511628211ull;
    }
    return h;
}

// ---- T64 cache file ---------------------------------------------------------------------------------------------
struct CacheHeader {
    char magic[8];          // "W4T64LIN"
    uint32_t version;       // layout version of the tiles below (csrc/layout.cuh)
    uint32_t n, k, group_src, group, scale_bf16_src;
    float out_mul;
    uint64_t source_tag;    // what the tiles were made from (w4a16_st_lin_tag of the source tensors)
    uint64_t q_bytes, s_bytes;
};
constexpr uint32_t CACHE_VERSION = 1;
constexpr size_t IO_CHUNK = 8u << 20;   // 8 MiB, the reference's upload chunk (w4a16_dec/mem.rs)

}  // namespace

namespace w4 {

// Streamed upload: the source arrives through `fill` in row chunks of at most 8 MiB, each copied to the device and
// re-tiled into its place, so neither a whole host slice nor a second full device copy is ever needed.
int Dec::upload_stream(const char* name, int n, int k, int group, int scale_bf16, w4a16_fill_fn fill, void* user,
                       int glu_f) {
    Lin l;
    l.n = n;
    l.k = k;
    l.group_src = group;
    l.group = group == 64 ? 32 : group;
    l.glu_f = glu_f;
    const int src_div = group == 64 ? 2 : 1;
    const int ng_src = k / group;
    const size_t row_q = (size_t)k / 2, row_s = (size_t)ng_src * 2;
    const size_t qb = (size_t)n * row_q, sb = (size_t)n * (size_t)(k / l.group) * 2;
    // rows per chunk: whole 16-row blocks, at most 8 MiB of packed weights
    int rows_c = (int)(IO_CHUNK / row_q) / TILE_ROWS * TILE_ROWS;
    if (rows_c < TILE_ROWS) {
        rows_c = TILE_ROWS;
    }
    if (rows_c > n) {
        rows_c = n;
    }
    const size_t chunk_q = (size_t)rows_c * row_q, chunk_s = (size_t)rows_c * row_s;
    const size_t slot = ((chunk_q + chunk_s + 255) / 256) * 256;
    if (2 * slot > pin_cap) {
        cudaDeviceSynchronize();
        if (pin) cudaFreeHost(pin);
        if (stage_dev) cudaFree(stage_dev);
        pin = nullptr;
        stage_dev = nullptr;
        pin_cap = 0;
        cudaError_t e = cudaMallocHost(&pin, 2 * slot);
        if (e == cudaSuccess) {
            e = cudaMalloc(&stage_dev, 2 * slot);
        }
        if (e != cudaSuccess) {
            return cuda_fail("alloc upload staging", e);
        }
        pin_cap = 2 * slot;
    }
    cudaError_t e = cudaMalloc(&l.qt, qb);
    if (e != cudaSuccess) {
        return cuda_fail("alloc weights", e);
    }
    e = cudaMalloc(&l.st, sb);
    if (e != cudaSuccess) {
        cudaFree(l.qt);
        return cuda_fail("alloc scales", e);
    }
    auto drop = [&]() {
        cudaStreamSynchronize(stream);
        cudaFree(l.qt);
        cudaFree(l.st);
    };
    cudaEvent_t done[2];
    cudaEventCreateWithFlags(&done[0], cudaEventDisableTiming);
    cudaEventCreateWithFlags(&done[1], cudaEventDisableTiming);
    // bf16 scales: a first pass over the scales alone finds their exponent range (see upload_common)
    int shift = 0;
    if (scale_bf16) {
        const int preset[2] = {255, 0};
        cudaMemcpyAsync(err_flag + 1, preset, sizeof(preset), cudaMemcpyHostToDevice, stream);
        for (int r0 = 0, i = 0; r0 < n; r0 += rows_c, ++i) {
            const int rows = std::min(rows_c, n - r0);
            unsigned char* hp = (unsigned char*)pin + (i & 1) * slot;
            unsigned char* dp = (unsigned char*)stage_dev + (i & 1) * slot;
            if (i >= 2) {
                cudaEventSynchronize(done[i & 1]);
            }
            fill(user, 1, (size_t)r0 * row_s, hp, (size_t)rows * row_s);
            cudaMemcpyAsync(dp, hp, (size_t)rows * row_s, cudaMemcpyHostToDevice, stream);
            launch_scale_range((const uint16_t*)dp, (size_t)rows * ng_src, err_flag + 1, stream);
            cudaEventRecord(done[i & 1], stream);
        }
        int range[2] = {255, 0};
        e = cudaMemcpyAsync(range, err_flag + 1, sizeof(range), cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) {
            e = cudaStreamSynchronize(stream);
        }
        if (e != cudaSuccess) {
            drop();
            return cuda_fail("scale range", e);
        }
        if (range[0] <= range[1]) {
            const int lo = -17 - (range[0] - 127), hi = 12 - (range[1] - 127);
            if (lo > hi) {
                drop();
                return fail("w4a16 upload %s: bf16 scales span more than the 29 binades f16 weights can hold", name);
            }
            shift = lo > 0 ? lo : (hi < 0 ? hi : 0);
        }
    }
    l.out_mul = ldexpf(1.0f, -shift);
    cudaMemsetAsync(err_flag, 0, sizeof(int), stream);
    for (int r0 = 0, i = 0; r0 < n; r0 += rows_c, ++i) {
        const int rows = std::min(rows_c, n - r0);
        unsigned char* hp = (unsigned char*)pin + (i & 1) * slot;
        unsigned char* dp = (unsigned char*)stage_dev + (i & 1) * slot;
        if (i >= 2 || scale_bf16) {
            cudaEventSynchronize(done[i & 1]);   // the slot's previous copy has left the pinned buffer
        }
        fill(user, 0, (size_t)r0 * row_q, hp, (size_t)rows * row_q);
        fill(user, 1, (size_t)r0 * row_s, hp + chunk_q, (size_t)rows * row_s);
        cudaMemcpyAsync(dp, hp, chunk_q + (size_t)rows * row_s, cudaMemcpyHostToDevice, stream);
        launch_repack_q_rows((const uint32_t*)dp, l.qt, n, k, r0 / TILE_ROWS, rows / TILE_ROWS, glu_f, stream);
        launch_repack_s_rows((const uint16_t*)(dp + chunk_q), l.st, n, k, l.group, src_div, scale_bf16, shift, err_flag,
                             r0 / TILE_ROWS, rows / TILE_ROWS, glu_f, stream);
        cudaEventRecord(done[i & 1], stream);
    }
    int bad = 0;
    e = cudaMemcpyAsync(&bad, err_flag, sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) {
        e = cudaStreamSynchronize(stream);
    }
    cudaEventDestroy(done[0]);
    cudaEventDestroy(done[1]);
    if (e == cudaSuccess) {
        e = cudaGetLastError();
    }
    if (e != cudaSuccess || bad) {
        drop();
        if (e != cudaSuccess) {
            return cuda_fail("streamed upload", e);
        }
        return fail("w4a16 upload %s: a bf16 scale is not representable in f16 even after shifting", name);
    }
    l.bytes = qb + sb;
    auto it = lins.find(name);
    if (it != lins.end()) {
        cudaDeviceSynchronize();
        free_lin(it->second);
        lins.erase(it);
    }
    weights_bytes += l.bytes;
    lins[name] = l;
    return 0;
}

}  // namespace w4

using w4::Dec;
using w4::Lin;

extern "C" {

const char* w4a16_st_error(void) { return g_st_error.c_str(); }

int w4a16_st_open(const char* path, w4a16_st** out) {
    if (!out || !path) {
        return st_fail("w4a16_st_open: null argument");
    }
    *out = nullptr;
    struct stat stt;
    if (stat(path, &stt) != 0) {
        return st_fail(std::string(path) + ": no such file or directory");
    }
    w4a16_st* ar = new w4a16_st();
    std::vector<std::string> files;
    if (S_ISDIR(stt.st_mode)) {
        // st.rs:146-160: every model*.safetensors of the directory, in name order
        DIR* d = opendir(path);
        if (!d) {
            delete ar;
            return st_fail(std::string(path) + ": cannot list");
        }
        while (struct dirent* de = readdir(d)) {
            const std::string nm = de->d_name;
            const std::string ext = ".safetensors";
            if (nm.size() > ext.size() && nm.compare(0, 5, "model") == 0 &&
                nm.compare(nm.size() - ext.size(), ext.size(), ext) == 0) {
                files.push_back(std::string(path) + "/" + nm);
            }
        }
        closedir(d);
        std::sort(files.begin(), files.end());
        if (files.empty()) {
            delete ar;
            return st_fail(std::string("no model*.safetensors in ") + path);
        }
    } else {
        files.push_back(path);
    }
    for (const auto& f : files) {
        if (parse_shard(*ar, f)) {
            delete ar;
            return 1;
        }
    }
    if (collect_linears(*ar)) {
        delete ar;
        return 1;
    }
    *out = ar;
    return 0;
}

void w4a16_st_close(w4a16_st* st) { delete st; }

int w4a16_st_lin_count(const w4a16_st* st) { return st ? (int)st->lins.size() : 0; }

int w4a16_st_lin_at(const w4a16_st* st, int i, char* base_out, size_t cap, int* n, int* k, int* group, int* scale_bf16) {
    if (!st || i < 0 || i >= (int)st->lins.size()) {
        return st_fail("w4a16_st_lin_at: index out of range");
    }
    const LinInfo& li = st->lins[i];
    if (base_out && cap > 0) {
        snprintf(base_out, cap, "%s", li.base.c_str());
    }
    if (n) *n = li.n;
    if (k) *k = li.k;
    if (group) *group = li.group;
    if (scale_bf16) *scale_bf16 = li.scale_bf16;
    return 0;
}

int w4a16_st_lin_tag(const w4a16_st* st, const char* base, uint64_t* tag) {
    const LinInfo* li = st ? find_info(st, base) : nullptr;
    if (!li || !tag) {
        return st_fail(std::string("w4a16_st_lin_tag: unknown linear ") + (base ? base : "(null)"));
    }
    const StEntry& pk = st->entries.at(li->base + ".weight_packed");
    const StEntry& sc = st->entries.at(li->base + ".weight_scale");
    uint64_t h = 1469598103934665603ull;
    const uint32_t meta[4] = {(uint32_t)li->n, (uint32_t)li->k, (uint32_t)li->group, (uint32_t)li->scale_bf16};
    h = fnv1a((const unsigned char*)meta, sizeof(meta), h);
    h = fnv1a(st->data(pk), pk.end - pk.begin, h);
    h = fnv1a(st->data(sc), sc.end - sc.begin, h);
    *tag = h;
    return 0;
}

int w4a16_upload_lin_g_stream(w4a16_dec* dec, const char* name, int n, int k, int group, int scale_bf16,
                              w4a16_fill_fn fill, void* user) {
    Dec& d = dec->d;
    cudaSetDevice(d.device);
    if (!fill) {
        return d.fail("w4a16 upload_lin_g_stream: null fill callback");
    }
    if (!name || !*name) {
        return d.fail("w4a16 upload: empty name");
    }
    if (n <= 0 || k <= 0 || (group != 128 && group != 64 && group != 32) || k % group != 0) {
        return d.fail("w4a16 upload %s: unsupported n=%d k=%d group=%d", name, n, k, group);
    }
    if (!w4::shape_ok(n, k, group)) {
        return d.fail("w4a16 upload %s: tiled layout needs n%%16==0 and k%%64==0 (n=%d k=%d)", name, n, k);
    }
    return d.upload_stream(name, n, k, group, scale_bf16, fill, user);
}

namespace {
struct StFill {
    const unsigned char* q;
    const unsigned char* s;
};
void st_fill(void* user, int which, size_t off, void* dst, size_t len) {
    const StFill* f = (const StFill*)user;
    memcpy(dst, (which == 0 ? f->q : f->s) + off, len);
}
}  // namespace

int w4a16_upload_lin_st(w4a16_dec* dec, const char* name, const w4a16_st* st, const char* base) {
    Dec& d = dec->d;
    const LinInfo* li = st ? find_info(st, base) : nullptr;
    if (!li) {
        return d.fail("w4a16 upload_lin_st: no linear %s in the archive", base ? base : "(null)");
    }
    StFill f{st->data(st->entries.at(li->base + ".weight_packed")), st->data(st->entries.at(li->base + ".weight_scale"))};
    return w4a16_upload_lin_g_stream(dec, name, li->n, li->k, li->group, li->scale_bf16, st_fill, &f);
}

int w4a16_save_lin_cache(w4a16_dec* dec, const char* name, const char* path, uint64_t source_tag) {
    Dec& d = dec->d;
    auto it = d.lins.find(name ? name : "");
    if (it == d.lins.end()) {
        return d.fail("w4a16: unknown linear %s", name ? name : "(null)");
    }
    const Lin& l = it->second;
    cudaSetDevice(d.device);
    if (l.glu_f > 0) {
        return d.fail("w4a16 save_lin_cache: %s is an interleaved expert matrix, which the cache format does not describe", name);
    }
    CacheHeader h{};
    memcpy(h.magic, "W4T64LIN", 8);
    h.version = CACHE_VERSION;
    h.n = (uint32_t)l.n;
    h.k = (uint32_t)l.k;
    h.group_src = (uint32_t)l.group_src;
    h.group = (uint32_t)l.group;
    h.scale_bf16_src = 0;
    h.out_mul = l.out_mul;
    h.source_tag = source_tag;
    h.q_bytes = (uint64_t)l.n * (uint64_t)(l.k / 2);
    h.s_bytes = (uint64_t)l.n * (uint64_t)(l.k / l.group) * 2;
    const std::string tmp = std::string(path) + ".tmp";
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) {
        return d.fail("w4a16 save_lin_cache: cannot write %s", tmp.c_str());
    }
    bool ok = fwrite(&h, sizeof(h), 1, f) == 1;
    std::vector<unsigned char> buf(IO_CHUNK);
    const unsigned char* srcs[2] = {(const unsigned char*)l.qt, (const unsigned char*)l.st};
    const uint64_t lens[2] = {h.q_bytes, h.s_bytes};
    cudaStreamSynchronize(d.stream);
    for (int part = 0; part < 2 && ok; ++part) {
        for (uint64_t off = 0; off < lens[part] && ok; off += IO_CHUNK) {
            const size_t len = (size_t)std::min<uint64_t>(IO_CHUNK, lens[part] - off);
            ok = cudaMemcpy(buf.data(), srcs[part] + off, len, cudaMemcpyDeviceToHost) == cudaSuccess &&
                 fwrite(buf.data(), 1, len, f) == len;
        }
    }
    ok = fclose(f) == 0 && ok;
    if (!ok || rename(tmp.c_str(), path) != 0) {
        remove(tmp.c_str());
        return d.fail("w4a16 save_lin_cache: writing %s failed", path);
    }
    return 0;
}

int w4a16_load_lin_cache(w4a16_dec* dec, const char* name, const char* path, uint64_t source_tag) {
    Dec& d = dec->d;
    if (!name || !*name) {
        return d.fail("w4a16 load_lin_cache: empty name");
    }
    cudaSetDevice(d.device);
    FILE* f = fopen(path, "rb");
    if (!f) {
        return d.fail("w4a16 load_lin_cache: cannot open %s", path);
    }
    CacheHeader h{};
    if (fread(&h, sizeof(h), 1, f) != 1 || memcmp(h.magic, "W4T64LIN", 8) != 0) {
        fclose(f);
        return d.fail("w4a16 load_lin_cache: %s is not a tile cache file", path);
    }
    if (h.version != CACHE_VERSION) {
        fclose(f);
        return d.fail("w4a16 load_lin_cache: %s has layout version %u, this library reads %u", path, h.version, CACHE_VERSION);
    }
    if (h.source_tag != source_tag) {
        fclose(f);
        return d.fail("w4a16 load_lin_cache: %s was made from other source tensors (stale cache)", path);
    }
    const uint64_t qb = (uint64_t)h.n * (h.k / 2), sb = h.group ? (uint64_t)h.n * (h.k / h.group) * 2 : 0;
    if (!w4::shape_ok((int)h.n, (int)h.k, (int)h.group_src) || (h.group != 128 && h.group != 32) || h.q_bytes != qb ||
        h.s_bytes != sb) {
        fclose(f);
        return d.fail("w4a16 load_lin_cache: %s has an inconsistent header", path);
    }
    Lin l;
    l.n = (int)h.n;
    l.k = (int)h.k;
    l.group = (int)h.group;
    l.group_src = (int)h.group_src;
    l.out_mul = h.out_mul;
    cudaError_t e = cudaMalloc(&l.qt, qb);
    if (e == cudaSuccess) {
        e = cudaMalloc(&l.st, sb);
    }
    if (e != cudaSuccess) {
        if (l.qt) cudaFree(l.qt);
        fclose(f);
        return d.cuda_fail("alloc weights", e);
    }
    // straight copies into the resident buffers: no staging copy on the device, no repack kernel
    const size_t slot = IO_CHUNK;
    if (2 * slot > d.pin_cap) {
        cudaDeviceSynchronize();
        if (d.pin) cudaFreeHost(d.pin);
        if (d.stage_dev) cudaFree(d.stage_dev);
        d.pin = nullptr;
        d.stage_dev = nullptr;
        d.pin_cap = 0;
        e = cudaMallocHost(&d.pin, 2 * slot);
        if (e == cudaSuccess) {
            e = cudaMalloc(&d.stage_dev, 2 * slot);
        }
        if (e != cudaSuccess) {
            cudaFree(l.qt);
            cudaFree(l.st);
            fclose(f);
            return d.cuda_fail("alloc upload staging", e);
        }
        d.pin_cap = 2 * slot;
    }
    cudaEvent_t done[2];
    cudaEventCreateWithFlags(&done[0], cudaEventDisableTiming);
    cudaEventCreateWithFlags(&done[1], cudaEventDisableTiming);
    unsigned char* dsts[2] = {(unsigned char*)l.qt, (unsigned char*)l.st};
    const uint64_t lens[2] = {qb, sb};
    bool ok = true;
    int i = 0;
    for (int part = 0; part < 2 && ok; ++part) {
        for (uint64_t off = 0; off < lens[part] && ok; off += slot, ++i) {
            const size_t len = (size_t)std::min<uint64_t>(slot, lens[part] - off);
            unsigned char* hp = (unsigned char*)d.pin + (i & 1) * slot;
            if (i >= 2) {
                cudaEventSynchronize(done[i & 1]);
            }
            ok = fread(hp, 1, len, f) == len &&
                 cudaMemcpyAsync(dsts[part] + off, hp, len, cudaMemcpyHostToDevice, d.stream) == cudaSuccess;
            cudaEventRecord(done[i & 1], d.stream);
        }
    }
    fclose(f);
    e = cudaStreamSynchronize(d.stream);
    cudaEventDestroy(done[0]);
    cudaEventDestroy(done[1]);
    if (!ok || e != cudaSuccess) {
        cudaFree(l.qt);
        cudaFree(l.st);
        return d.fail("w4a16 load_lin_cache: reading %s failed", path);
    }
    l.bytes = qb + sb;
    auto it = d.lins.find(name);
    if (it != d.lins.end()) {
        cudaDeviceSynchronize();
        d.free_lin(it->second);
        d.lins.erase(it);
    }
    d.weights_bytes += l.bytes;
    d.lins[name] = l;
    return 0;
}

}  // extern "C"
