// Checkpoint-facing loaders (host only, load time): a safetensors reader and the mapping from the on-disk tensors of
// the model -- F8_E4M3 weights with UE8M0 32x32 scales, FP4 expert weights with UE8M0 1x32 scales -- to this library's
// tile-record images.  Replaces Checkpoint (crates/model/src/st.rs:17-106), Loader::fp8 (crates/engine/src/weights.rs:254-276)
// and the expert part of Loader::layer (weights.rs:421-446, expert_shard in crates/model/src/packing.rs:174-254).
// The reference shards experts over tensor-parallel ranks by slicing `inter`; this library shards whole experts
// (expert parallelism), so the expert loader takes an expert range and always the full matrices.
#include <dirent.h>
#include <fcntl.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "../../include/dsuf_qmm.h"

namespace {

struct Mapped {
    const uint8_t* base = nullptr;
    size_t len = 0;
};

struct TensorRec {
    std::string dtype;
    std::vector<int64_t> shape;
    int file = 0;
    size_t begin = 0, end = 0;   // byte range inside the file
};

}  // namespace

struct dsuf_ckpt {
    std::vector<Mapped> files;
    std::map<std::string, TensorRec> tensors;
    char err[512];
};

namespace {

int ck_fail(dsuf_ckpt* c, int code, const char* fmt, ...) {
    if (c) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(c->err, sizeof(c->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

// ---- the subset of JSON a safetensors header uses: objects, arrays, strings, non-negative integers, and (inside
// "__metadata__") string values; anything else is skipped structurally.
struct Json {
    const char* p;
    const char* end;
    bool ok = true;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool eat(char ch) {
        ws();
        if (p < end && *p == ch) { ++p; return true; }
        return false;
    }
    std::string str() {
        ws();
        std::string out;
        if (p >= end || *p != '"') { ok = false; return out; }
        ++p;
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                ++p;
                switch (*p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'u': out += '?'; p += (end - p > 4 ? 4 : 0); break;   // names here are ASCII
                    default: out += *p;
                }
                ++p;
            } else {
                out += *p++;
            }
        }
        if (p >= end) { ok = false; return out; }
        ++p;
        return out;
    }
    int64_t num() {
        ws();
        int64_t v = 0;
        bool any = false;
        while (p < end && *p >= '0' && *p <= '9') { v = v * 10 + (*p - '0'); ++p; any = true; }
        if (!any) ok = false;
        return v;
    }
    void skip() {   // any value
        ws();
        if (p >= end) { ok = false; return; }
        if (*p == '"') { str(); return; }
        if (*p == '{' || *p == '[') {
            const char open = *p, close = open == '{' ? '}' : ']';
            ++p;
            if (eat(close)) return;
            do {
                if (open == '{') { str(); if (!eat(':')) { ok = false; return; } }
                skip();
                if (!ok) return;
            } while (eat(','));
            if (!eat(close)) ok = false;
            return;
        }
        while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;   // number / literal
    }
};

bool parse_header(dsuf_ckpt* c, int file, const char* hdr, size_t n, size_t data0, size_t file_len) {
    Json j{hdr, hdr + n};
    if (!j.eat('{')) return false;
    if (j.eat('}')) return true;
    do {
        const std::string name = j.str();
        if (!j.ok || !j.eat(':')) return false;
        if (name == "__metadata__") { j.skip(); if (!j.ok) return false; continue; }
        TensorRec t;
        t.file = file;
        bool have_off = false;
        if (!j.eat('{')) return false;
        do {
            const std::string key = j.str();
            if (!j.ok || !j.eat(':')) return false;
            if (key == "dtype") {
                t.dtype = j.str();
            } else if (key == "shape") {
                if (!j.eat('[')) return false;
                if (!j.eat(']')) {
                    do t.shape.push_back(j.num()); while (j.eat(','));
                    if (!j.eat(']')) return false;
                }
            } else if (key == "data_offsets") {
                if (!j.eat('[')) return false;
                const int64_t b = j.num();
                if (!j.eat(',')) return false;
                const int64_t e = j.num();
                if (!j.eat(']')) return false;
                t.begin = data0 + (size_t)b;
                t.end = data0 + (size_t)e;
                have_off = true;
            } else {
                j.skip();
            }
            if (!j.ok) return false;
        } while (j.eat(','));
        if (!j.eat('}') || !have_off || t.begin > t.end || t.end > file_len) return false;
        c->tensors[name] = t;
    } while (j.eat(','));
    return j.eat('}') && j.ok;
}

int map_file(dsuf_ckpt* c, const std::string& path) {
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) return ck_fail(c, DSUF_E_BADARG, "cannot open %s", path.c_str());
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 8) { close(fd); return ck_fail(c, DSUF_E_BADARG, "%s: not a safetensors file", path.c_str()); }
    void* m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (m == MAP_FAILED) return ck_fail(c, DSUF_E_NOMEM, "%s: mmap failed", path.c_str());
    Mapped f{(const uint8_t*)m, (size_t)st.st_size};
    uint64_t n = 0;
    memcpy(&n, f.base, 8);
    if (n > f.len - 8) { munmap(m, f.len); return ck_fail(c, DSUF_E_BADARG, "%s: header length %llu exceeds the file", path.c_str(), (unsigned long long)n); }
    c->files.push_back(f);
    if (!parse_header(c, (int)c->files.size() - 1, (const char*)f.base + 8, (size_t)n, 8 + (size_t)n, f.len))
        return ck_fail(c, DSUF_E_BADARG, "%s: malformed safetensors header", path.c_str());
    return DSUF_OK;
}

const TensorRec* find(dsuf_ckpt* c, const std::string& name) {
    auto it = c->tensors.find(name);
    return it == c->tensors.end() ? nullptr : &it->second;
}

// `{name}` must exist with the dtype and 2-D shape given; returns its bytes.
int get2d(dsuf_ckpt* c, const std::string& name, const char* dtype_a, const char* dtype_b, int64_t d0, int64_t d1, size_t elem_num,
          size_t elem_den, const uint8_t** out) {
    const TensorRec* t = find(c, name);
    if (!t) return ck_fail(c, DSUF_E_BADARG, "tensor %s not in checkpoint", name.c_str());
    if (dtype_a && t->dtype != dtype_a && (!dtype_b || t->dtype != dtype_b))
        return ck_fail(c, DSUF_E_BADARG, "%s: dtype %s, expected %s", name.c_str(), t->dtype.c_str(), dtype_a);
    // dtype_a == nullptr: packed 4-bit codes, stored by different writers as bytes [d0][d1] or as 4-bit elements [d0][2 d1]
    if (t->shape.size() != 2 || t->shape[0] != d0 || (t->shape[1] != d1 && (dtype_a || t->shape[1] != 2 * d1)))
        return ck_fail(c, DSUF_E_BADARG, "%s: expected shape [%lld, %lld]", name.c_str(), (long long)d0, (long long)d1);
    if (t->end - t->begin != (size_t)d0 * (size_t)d1 * elem_num / elem_den)
        return ck_fail(c, DSUF_E_BADARG, "%s: %zu bytes of data do not match its shape", name.c_str(), t->end - t->begin);
    *out = c->files[t->file].base + t->begin;
    return DSUF_OK;
}

}  // namespace

extern "C" {

int32_t dsuf_ckpt_open(const char* path, dsuf_ckpt** out) {
    if (!path || !out) return DSUF_E_BADARG;
    *out = nullptr;
    dsuf_ckpt* c = new dsuf_ckpt();
    c->err[0] = 0;
    *out = c;   // returned even on failure so that the caller can read the message; close it either way
    struct stat st;
    if (stat(path, &st) != 0) return ck_fail(c, DSUF_E_BADARG, "%s: no such file or directory", path);
    std::vector<std::string> files;
    if (S_ISDIR(st.st_mode)) {
        DIR* d = opendir(path);
        if (!d) return ck_fail(c, DSUF_E_BADARG, "cannot list %s", path);
        while (struct dirent* e = readdir(d)) {
            const std::string n = e->d_name;
            if (n.size() > 12 && n.compare(n.size() - 12, 12, ".safetensors") == 0) files.push_back(std::string(path) + "/" + n);
        }
        closedir(d);
        std::sort(files.begin(), files.end());   // Checkpoint::open sorts the shards (st.rs:24-31)
        if (files.empty()) return ck_fail(c, DSUF_E_BADARG, "%s holds no *.safetensors file", path);
    } else {
        files.push_back(path);
    }
    for (const std::string& f : files) {
        const int rc = map_file(c, f);
        if (rc) return rc;
    }
    return DSUF_OK;
}

int32_t dsuf_ckpt_close(dsuf_ckpt* c) {
    if (!c) return DSUF_OK;
    for (const Mapped& f : c->files) munmap((void*)f.base, f.len);
    delete c;
    return DSUF_OK;
}

int32_t dsuf_ckpt_last_error(dsuf_ckpt* c, char* buf, size_t len) {
    if (!c || !buf || !len) return DSUF_E_BADARG;
    strncpy(buf, c->err, len - 1);
    buf[len - 1] = 0;
    return DSUF_OK;
}

int64_t dsuf_ckpt_count(dsuf_ckpt* c) { return c ? (int64_t)c->tensors.size() : 0; }

int32_t dsuf_ckpt_tensor(dsuf_ckpt* c, const char* name, dsuf_tensor_info* out) {
    if (!c || !name || !out) return DSUF_E_BADARG;
    const TensorRec* t = find(c, name);
    if (!t) return ck_fail(c, DSUF_E_BADARG, "tensor %s not in checkpoint", name);
    if (t->shape.size() > 8) return ck_fail(c, DSUF_E_UNSUPPORTED, "%s: rank %zu", name, t->shape.size());
    memset(out, 0, sizeof(*out));
    strncpy(out->dtype, t->dtype.c_str(), sizeof(out->dtype) - 1);
    out->rank = (int32_t)t->shape.size();
    for (size_t i = 0; i < t->shape.size(); ++i) out->shape[i] = t->shape[i];
    out->data = c->files[t->file].base + t->begin;
    out->nbytes = t->end - t->begin;
    return DSUF_OK;
}

int32_t dsuf_ckpt_load_fp8_dense(dsuf_ckpt* c, const char* name, int32_t n, int32_t k, int32_t r0, int32_t r1, uint8_t* tiles_out) {
    if (!c || !name || !tiles_out) return DSUF_E_BADARG;
    if (n <= 0 || k <= 0 || n % 32 || k % 128) return ck_fail(c, DSUF_E_BADARG, "%s: n (%d) must be a multiple of 32 and k (%d) of 128", name, n, k);
    if (r0 < 0 || r1 > n || r0 >= r1 || r0 % 32 || r1 % 32)
        return ck_fail(c, DSUF_E_BADARG, "%s: row range [%d, %d) must lie in [0, %d) on multiples of 32 (one scale row covers 32 weight rows)", name, r0, r1, n);
    const uint8_t *w = nullptr, *s = nullptr;
    int rc = get2d(c, std::string(name) + ".weight", "F8_E4M3", nullptr, n, k, 1, 1, &w);
    if (rc) return rc;
    rc = get2d(c, std::string(name) + ".scale", "F8_E8M0", "U8", n / 32, k / 32, 1, 1, &s);
    if (rc) return rc;
    rc = dsuf_pack_fp8_weight(DSUF_MODE_MX, w + (size_t)r0 * k, s + (size_t)(r0 / 32) * (k / 32), r1 - r0, k, tiles_out);
    if (rc) return ck_fail(c, rc, "%s: packing failed", name);
    return DSUF_OK;
}

int32_t dsuf_ckpt_load_fp4_experts(dsuf_ckpt* c, const char* prefix, int32_t e0, int32_t e1, int32_t dim, int32_t inter, uint8_t* w13_out,
                                   uint8_t* w2_out) {
    if (!c || !prefix || !w13_out || !w2_out) return DSUF_E_BADARG;
    if (e0 < 0 || e1 <= e0) return ck_fail(c, DSUF_E_BADARG, "expert range [%d, %d)", e0, e1);
    if (dim <= 0 || inter <= 0 || dim % 128 || inter % 128)
        return ck_fail(c, DSUF_E_BADARG, "dim (%d) and inter (%d) must be multiples of 128", dim, inter);
    const size_t per13 = dsuf_packed_bytes(DSUF_FMT_FP4, DSUF_MODE_MX, 2 * inter, dim), per2 = dsuf_packed_bytes(DSUF_FMT_FP4, DSUF_MODE_MX, dim, inter);
    std::vector<uint8_t> codes((size_t)2 * inter * dim / 2), scales((size_t)2 * inter * dim / 32);
    for (int e = e0; e < e1; ++e) {
        const std::string ep = std::string(prefix) + ".ffn.experts." + std::to_string(e) + ".";
        const uint8_t *w1, *s1, *w3, *s3, *w2, *s2;
        int rc;
        // FP4 weights are stored two codes per byte (low nibble = even k); the reference takes their bytes as they are
        // (weights.rs:436-438) and so does this loader, whatever container dtype the writer declared
        if ((rc = get2d(c, ep + "w1.weight", nullptr, nullptr, inter, dim / 2, 1, 1, &w1))) return rc;
        if ((rc = get2d(c, ep + "w1.scale", "F8_E8M0", "U8", inter, dim / 32, 1, 1, &s1))) return rc;
        if ((rc = get2d(c, ep + "w3.weight", nullptr, nullptr, inter, dim / 2, 1, 1, &w3))) return rc;
        if ((rc = get2d(c, ep + "w3.scale", "F8_E8M0", "U8", inter, dim / 32, 1, 1, &s3))) return rc;
        if ((rc = get2d(c, ep + "w2.weight", nullptr, nullptr, dim, inter / 2, 1, 1, &w2))) return rc;
        if ((rc = get2d(c, ep + "w2.scale", "F8_E8M0", "U8", dim, inter / 32, 1, 1, &s2))) return rc;
        // gate rows (w1) first, then up rows (w3): the packer interleaves them for the SwiGLU epilogue
        memcpy(codes.data(), w1, (size_t)inter * dim / 2);
        memcpy(codes.data() + (size_t)inter * dim / 2, w3, (size_t)inter * dim / 2);
        memcpy(scales.data(), s1, (size_t)inter * dim / 32);
        memcpy(scales.data() + (size_t)inter * dim / 32, s3, (size_t)inter * dim / 32);
        if ((rc = dsuf_pack_fp4_weight(codes.data(), scales.data(), 2 * inter, dim, 1, w13_out + (size_t)(e - e0) * per13)))
            return ck_fail(c, rc, "%sw1/w3: packing failed", ep.c_str());
        if ((rc = dsuf_pack_fp4_weight(w2, s2, dim, inter, 0, w2_out + (size_t)(e - e0) * per2)))
            return ck_fail(c, rc, "%sw2: packing failed", ep.c_str());
    }
    return DSUF_OK;
}

}  // extern "C"
