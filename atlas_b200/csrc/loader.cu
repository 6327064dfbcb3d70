// loader.cu — safetensors files straight onto the device.
//
// Replaces, for the GPU path, SafetensorsFile and the two loaders of the reference
// (crates/atlas-model/src/lib.rs: SafetensorsFile :2046-2240, load_model_from_safetensors
// :2283-2360, patch_config_from_hf_json :2367-2432, load_model_from_dir :2437-2570).  The reference
// reads every shard into RAM, converts every tensor to f32, truncates it back to bf16 and keeps the
// f32 copy.  Here a file is mapped, not read; a BF16 tensor goes to the device as the bytes it is
// stored as; each tensor-parallel rank touches only the rows or columns it keeps; int8/int4 models
// are quantised on the device while loading (atlas-quant recipe).  Host code only — no kernels.
#include <errno.h>
#include <fcntl.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/resource.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.cuh"

// ── a small JSON reader (objects keep their key order) ───────────────────────────────
namespace {

struct JVal {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0.0;
    bool integral = false; unsigned long long u = 0;     // set for non-negative integers written without fraction/exponent
    std::string str;
    std::vector<JVal> arr;
    std::vector<std::pair<std::string, JVal>> obj;
    const JVal* get(const char* key) const {
        if (kind != Obj) return nullptr;
        for (const auto& kv : obj) if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool as_usize(size_t* out) const { if (kind == Num && integral) { *out = (size_t)u; return true; } return false; }
    bool as_f64(double* out) const { if (kind == Num) { *out = num; return true; } return false; }
};

struct JParser {
    const char* p; const char* end; std::string err;
    void ws() { while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) p++; }
    bool fail(const char* m) { if (err.empty()) err = m; return false; }
    bool string(std::string& out) {
        if (p >= end || *p != '"') return fail("expected a string");
        p++;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail("bad escape");
                switch (*p) {
                    case 'n': out += '\n'; break; case 't': out += '\t'; break; case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break; case 'f': out += '\f'; break;
                    case 'u': {
                        if (end - p < 5) return fail("bad \\u escape");
                        unsigned cp = (unsigned)strtoul(std::string(p + 1, p + 5).c_str(), nullptr, 16);
                        p += 4;
                        if (cp < 0x80) out += (char)cp;
                        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
                        else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
                        break;
                    }
                    default: out += *p;
                }
                p++;
            } else out += *p++;
        }
        if (p >= end) return fail("unterminated string");
        p++;
        return true;
    }
    bool value(JVal& v, int depth) {
        if (depth > 64) return fail("nesting too deep");
        ws();
        if (p >= end) return fail("unexpected end");
        if (*p == '{') {
            v.kind = JVal::Obj; p++; ws();
            if (p < end && *p == '}') { p++; return true; }
            for (;;) {
                ws();
                std::string k; if (!string(k)) return false;
                ws(); if (p >= end || *p != ':') return fail("expected ':'");
                p++;
                JVal c; if (!value(c, depth + 1)) return false;
                v.obj.emplace_back(std::move(k), std::move(c));
                ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == '}') { p++; return true; }
                return fail("expected ',' or '}'");
            }
        }
        if (*p == '[') {
            v.kind = JVal::Arr; p++; ws();
            if (p < end && *p == ']') { p++; return true; }
            for (;;) {
                JVal c; if (!value(c, depth + 1)) return false;
                v.arr.push_back(std::move(c));
                ws();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == ']') { p++; return true; }
                return fail("expected ',' or ']'");
            }
        }
        if (*p == '"') { v.kind = JVal::Str; return string(v.str); }
        if (end - p >= 4 && !strncmp(p, "true", 4)) { v.kind = JVal::Bool; v.b = true; p += 4; return true; }
        if (end - p >= 5 && !strncmp(p, "false", 5)) { v.kind = JVal::Bool; v.b = false; p += 5; return true; }
        if (end - p >= 4 && !strncmp(p, "null", 4)) { v.kind = JVal::Null; p += 4; return true; }
        const char* s = p;
        bool plain = true;
        if (p < end && (*p == '-' || *p == '+')) { plain = false; p++; }
        while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '-' || *p == '+')) {
            if (*p < '0' || *p > '9') plain = false;
            p++;
        }
        if (p == s) return fail("unexpected character");
        const std::string t(s, p);
        v.kind = JVal::Num; v.num = strtod(t.c_str(), nullptr);
        if (plain) { v.integral = true; v.u = strtoull(t.c_str(), nullptr, 10); }
        return true;
    }
};

bool parse_json(const char* text, size_t n, JVal& root, std::string& err) {
    JParser P{ text, text + n, "" };
    if (!P.value(root, 0)) { err = P.err; return false; }
    return true;
}

bool read_text_file(const std::string& path, std::string& out) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return false;
    char buf[65536]; size_t n;
    while ((n = fread(buf, 1, sizeof(buf), f)) > 0) out.append(buf, n);
    fclose(f);
    return true;
}

// f16 → f32 as f16_to_f32 (:2243-2262) does it
float half_bits_to_f32(uint16_t h) {
    const uint32_t sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1Fu, mant = h & 0x3FFu;
    if (exp == 0) {
        if (mant == 0) return sign ? -0.0f : 0.0f;
        const float m = (float)mant / 1024.0f;
        return sign ? -m * 6.103515625e-05f : m * 6.103515625e-05f;      // 2^-14
    }
    if (exp == 31) return mant == 0 ? (sign ? -INFINITY : INFINITY) : NAN;
    const uint32_t bits = (sign << 31) | ((exp + 127u - 15u) << 23) | (mant << 13);
    float f; memcpy(&f, &bits, 4); return f;
}

struct TensorDesc {
    std::string name; std::string dtype_name;
    int dtype = -1;                      // ATLASX_F32, ATLASX_BF16, ATLASX_F16, or −1 (present but not readable)
    std::vector<size_t> shape;
    size_t off0 = 0, off1 = 0;
};

}  // namespace

struct atlasx_safetensors {
    std::string path;
    int fd = -1;
    const uint8_t* map = nullptr; size_t map_bytes = 0;
    size_t data_start = 0;
    std::vector<TensorDesc> tensors;
};

extern "C" int atlasx_safetensors_close(atlasx_safetensors* st) {
    if (!st) return ATLASX_OK;
    if (st->map) munmap((void*)st->map, st->map_bytes);
    if (st->fd >= 0) close(st->fd);
    delete st;
    return ATLASX_OK;
}

extern "C" int atlasx_safetensors_open(const char* path, atlasx_safetensors** out) {
    AX_ARG(path && out, "null argument");
    *out = nullptr;
    std::unique_ptr<atlasx_safetensors, int (*)(atlasx_safetensors*)> st(new atlasx_safetensors(), atlasx_safetensors_close);
    st->path = path;
    st->fd = open(path, O_RDONLY);
    if (st->fd < 0) return atlasx_fail(ATLASX_ERR_ARG, "safetensors: cannot open %s: %s", path, strerror(errno));
    struct stat sb;
    if (fstat(st->fd, &sb) != 0) return atlasx_fail(ATLASX_ERR_ARG, "safetensors: cannot stat %s", path);
    const size_t n = (size_t)sb.st_size;
    if (n < 8) return atlasx_fail(ATLASX_ERR_ARG, "safetensors: file too short");
    void* mp = mmap(nullptr, n, PROT_READ, MAP_PRIVATE, st->fd, 0);
    if (mp == MAP_FAILED) return atlasx_fail(ATLASX_ERR_ARG, "safetensors: cannot map %s: %s", path, strerror(errno));
    st->map = (const uint8_t*)mp; st->map_bytes = n;
    uint64_t hs = 0;
    for (int i = 7; i >= 0; i--) hs = (hs << 8) | st->map[i];            // little-endian u64
    if (hs > n - 8) return atlasx_fail(ATLASX_ERR_ARG, "safetensors: header truncated");
    JVal root; std::string err;
    if (!parse_json((const char*)st->map + 8, (size_t)hs, root, err))
        return atlasx_fail(ATLASX_ERR_ARG, "safetensors header JSON: %s", err.c_str());
    st->data_start = 8 + (size_t)hs;
    if (root.kind == JVal::Obj) {
        for (const auto& kv : root.obj) {
            if (kv.first == "__metadata__") continue;
            TensorDesc d;
            d.name = kv.first;
            const JVal* dt = kv.second.get("dtype");
            d.dtype_name = (dt && dt->kind == JVal::Str) ? dt->str : "F32";
            d.dtype = d.dtype_name == "F32" ? ATLASX_F32 : d.dtype_name == "BF16" ? ATLASX_BF16 : d.dtype_name == "F16" ? ATLASX_F16 : -1;
            if (const JVal* sh = kv.second.get("shape"))
                if (sh->kind == JVal::Arr) for (const JVal& x : sh->arr) { size_t v; if (x.as_usize(&v)) d.shape.push_back(v); }
            const JVal* off = kv.second.get("data_offsets");
            if (!off || off->kind != JVal::Arr || off->arr.size() < 2)
                return atlasx_fail(ATLASX_ERR_ARG, "safetensors: missing data_offsets for %s", d.name.c_str());
            if (!off->arr[0].as_usize(&d.off0) || !off->arr[1].as_usize(&d.off1))
                return atlasx_fail(ATLASX_ERR_ARG, "safetensors: data_offsets of %s are not non-negative integers", d.name.c_str());
            if (d.off1 < d.off0 || d.off1 > n - st->data_start)
                return atlasx_fail(ATLASX_ERR_ARG, "safetensors: data_offsets of %s lie outside the file", d.name.c_str());
            st->tensors.push_back(std::move(d));
        }
    }
    *out = st.release();
    return ATLASX_OK;
}

extern "C" int atlasx_safetensors_count(const atlasx_safetensors* st) { return st ? (int)st->tensors.size() : 0; }

extern "C" int atlasx_safetensors_find(const atlasx_safetensors* st, const char* name) {
    if (!st || !name) return -1;
    for (size_t i = 0; i < st->tensors.size(); i++) if (st->tensors[i].name == name) return (int)i;
    return -1;
}

extern "C" int atlasx_safetensors_tensor(const atlasx_safetensors* st, int index, const char** name, int* dtype,
                                         int* n_dims, size_t* dims4, size_t* nbytes) {
    AX_ARG(st && index >= 0 && index < (int)st->tensors.size(), "tensor index out of range");
    const TensorDesc& d = st->tensors[(size_t)index];
    if (name) *name = d.name.c_str();
    if (dtype) *dtype = d.dtype;
    if (n_dims) *n_dims = (int)d.shape.size();
    if (dims4) for (size_t i = 0; i < 4; i++) dims4[i] = i < d.shape.size() ? d.shape[i] : 1;
    if (nbytes) *nbytes = d.off1 - d.off0;
    return ATLASX_OK;
}

namespace {
// A tensor seen as [rows × cols]: the last dimension is the column count, everything before it rows.
bool tensor_2d(const TensorDesc& d, size_t* rows, size_t* cols) {
    const size_t esz = d.dtype == ATLASX_F32 ? 4 : 2;
    const size_t n = (d.off1 - d.off0) / esz;
    if (d.shape.empty()) { *rows = 1; *cols = n; return true; }
    size_t c = d.shape.back(), r = 1;
    for (size_t i = 0; i + 1 < d.shape.size(); i++) {
        if (d.shape[i] != 0 && r > n / d.shape[i] + 1) return false;      // a product that left the byte count behind (and could wrap)
        r *= d.shape[i];
    }
    if ((c != 0 && r > n / c + 1) || r * c != n) return false;
    *rows = r; *cols = c;
    return true;
}
}  // namespace

extern "C" int atlasx_safetensors_read(const atlasx_safetensors* st, int index, size_t r0, size_t r1, size_t c0, size_t c1,
                                       int out_dtype, void* dst_host) {
    AX_ARG(st && dst_host && index >= 0 && index < (int)st->tensors.size(), "bad argument");
    const TensorDesc& d = st->tensors[(size_t)index];
    if (d.dtype < 0) return atlasx_fail(ATLASX_ERR_ARG, "unsupported dtype: %s", d.dtype_name.c_str());
    AX_ARG(out_dtype == ATLASX_F32 || out_dtype == ATLASX_BF16, "tensors are read as f32 or as bf16 bits");
    if (out_dtype == ATLASX_BF16 && d.dtype != ATLASX_BF16)
        return atlasx_fail(ATLASX_ERR_ARG, "tensor '%s' dtype is '%s', not BF16", d.name.c_str(), d.dtype_name.c_str());
    size_t rows, cols;
    if (!tensor_2d(d, &rows, &cols)) return atlasx_fail(ATLASX_ERR_ARG, "tensor '%s': shape and byte count disagree", d.name.c_str());
    AX_ARG(r0 <= r1 && r1 <= rows && c0 <= c1 && c1 <= cols, "slice outside the tensor");
    const uint8_t* base = st->map + st->data_start + d.off0;
    const size_t nc = c1 - c0;
    for (size_t r = r0; r < r1; r++) {
        const size_t o = (r - r0) * nc;
        if (d.dtype == ATLASX_F32) {
            memcpy((float*)dst_host + o, base + (r * cols + c0) * 4, nc * 4);
        } else if (d.dtype == ATLASX_BF16) {
            const uint8_t* src = base + (r * cols + c0) * 2;
            if (out_dtype == ATLASX_BF16) memcpy((uint16_t*)dst_host + o, src, nc * 2);
            else for (size_t i = 0; i < nc; i++) {                 // the upper half of an f32 (:2219-2225)
                const uint32_t u = ((uint32_t)src[2 * i] | ((uint32_t)src[2 * i + 1] << 8)) << 16;
                memcpy((float*)dst_host + o + i, &u, 4);
            }
        } else {
            const uint8_t* src = base + (r * cols + c0) * 2;
            for (size_t i = 0; i < nc; i++)
                ((float*)dst_host)[o + i] = half_bits_to_f32((uint16_t)(src[2 * i] | (src[2 * i + 1] << 8)));
        }
    }
    return ATLASX_OK;
}

// The synthetic writer of the reference's tests (build_f32 :2154-2185), same header text — keys in the
// order given, no spaces — extended to BF16 tensors so that bf16 models can be written as stored.
extern "C" int atlasx_safetensors_write(const char* path, int n, const char* const* names, const int* dtypes,
                                        const int* n_dims, const size_t* dims4, const void* const* data_host) {
    AX_ARG(path && n >= 0 && (n == 0 || (names && dtypes && n_dims && dims4 && data_host)), "bad argument");
    std::string header = "{";
    std::vector<size_t> sizes((size_t)n);
    size_t off = 0;
    for (int i = 0; i < n; i++) {
        AX_ARG(dtypes[i] == ATLASX_F32 || dtypes[i] == ATLASX_BF16, "the writer stores F32 and BF16 tensors");
        AX_ARG(n_dims[i] >= 0 && n_dims[i] <= 4 && names[i] && data_host[i], "bad tensor description");
        size_t cnt = 1;
        std::string shape;
        for (int k = 0; k < n_dims[i]; k++) {
            cnt *= dims4[(size_t)i * 4 + k];
            if (k) shape += ",";
            shape += std::to_string(dims4[(size_t)i * 4 + k]);
        }
        sizes[(size_t)i] = cnt * (dtypes[i] == ATLASX_F32 ? 4 : 2);
        if (i) header += ",";
        header += "\"" + std::string(names[i]) + "\":{\"dtype\":\"" + (dtypes[i] == ATLASX_F32 ? "F32" : "BF16") + "\",\"shape\":[" + shape +
                  "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + sizes[(size_t)i]) + "]}";
        off += sizes[(size_t)i];
    }
    header += "}";
    FILE* f = fopen(path, "wb");
    if (!f) return atlasx_fail(ATLASX_ERR_ARG, "safetensors: cannot create %s: %s", path, strerror(errno));
    uint8_t len[8];
    const uint64_t hl = header.size();
    for (int i = 0; i < 8; i++) len[i] = (uint8_t)(hl >> (8 * i));
    bool ok = fwrite(len, 1, 8, f) == 8 && fwrite(header.data(), 1, header.size(), f) == header.size();
    for (int i = 0; i < n && ok; i++) ok = fwrite(data_host[i], 1, sizes[(size_t)i], f) == sizes[(size_t)i];
    ok = (fclose(f) == 0) && ok;
    return ok ? ATLASX_OK : atlasx_fail(ATLASX_ERR_ARG, "safetensors: short write to %s", path);
}

// ── model loading ─────────────────────────────────────────────────────────────────────
namespace {

struct Source { atlasx_safetensors* st; int index; };

// Peak resident set of THIS program image: VmHWM belongs to the address space, which starts afresh at exec,
// whereas getrusage's ru_maxrss also carries the peak of the process that forked us.
size_t peak_rss_bytes() {
    if (FILE* f = fopen("/proc/self/status", "r")) {
        char line[256];
        size_t kb = 0;
        while (fgets(line, sizeof line, f))
            if (sscanf(line, "VmHWM: %zu kB", &kb) == 1) break;
        fclose(f);
        if (kb) return kb * 1024;
    }
    struct rusage ru;
    if (getrusage(RUSAGE_SELF, &ru) != 0) return 0;
    return (size_t)ru.ru_maxrss * 1024;
}

bool ends_with(const std::string& s, const char* suf) {
    const size_t n = strlen(suf);
    return s.size() >= n && s.compare(s.size() - n, n, suf) == 0;
}

// name → (layer, tensor id); layer −1 for the three global tensors.  Names as matched at :2300-2346.
bool classify(const std::string& name, int n_layers, bool post_norm, int* layer, int* which) {
    *layer = -1;
    if (name == "model.embed_tokens.weight" || name == "tok_embeddings.weight") { *which = ATLASX_T_EMBED; return true; }
    if (name == "model.norm.weight" || name == "norm.weight") { *which = ATLASX_T_FINAL_NORM; return true; }
    if (name == "lm_head.weight") { *which = ATLASX_T_LM_HEAD; return true; }
    size_t p = 0;
    if (name.compare(0, 13, "model.layers.") == 0) p = 13;
    else if (name.compare(0, 7, "layers.") == 0) p = 7;
    else return false;
    size_t q = p;
    while (q < name.size() && name[q] >= '0' && name[q] <= '9') q++;
    if (q == p || q >= name.size() || name[q] != '.') return false;
    const long li = strtol(name.substr(p, q - p).c_str(), nullptr, 10);
    if (li < 0 || li >= n_layers) return false;
    const std::string local = name.substr(q + 1);
    *layer = (int)li;
    if (local == "self_attn.q_proj.weight") *which = ATLASX_T_WQ;
    else if (local == "self_attn.k_proj.weight") *which = ATLASX_T_WK;
    else if (local == "self_attn.v_proj.weight") *which = ATLASX_T_WV;
    else if (local == "self_attn.o_proj.weight") *which = ATLASX_T_WO;
    else if (local == "mlp.gate_proj.weight") *which = ATLASX_T_GATE;
    else if (local == "mlp.up_proj.weight") *which = ATLASX_T_UP;
    else if (local == "mlp.down_proj.weight") *which = ATLASX_T_DOWN;
    else if (local == "input_layernorm.weight") *which = ATLASX_T_ATTN_NORM;
    else if (local == "post_attention_layernorm.weight") *which = post_norm ? ATLASX_T_ATTN_NORM : ATLASX_T_FFN_NORM;
    else if (local == "post_feedforward_layernorm.weight") *which = ATLASX_T_FFN_NORM;
    else if (local == "self_attn.q_norm.weight") *which = ATLASX_T_Q_NORM;
    else if (local == "self_attn.k_norm.weight") *which = ATLASX_T_K_NORM;
    else return false;                                   // unknown weights are ignored (:2346)
    return true;
}

int load_from_files(atlasx_ctx* ctx, const std::vector<std::string>& paths, atlasx_model_config cfg, const int* layer_sliding,
                    atlasx_model** out, atlasx_load_stats* stats) {
    const auto t0 = std::chrono::steady_clock::now();
    *out = nullptr;
    std::vector<atlasx_safetensors*> files;
    atlasx_model* m = nullptr;
    // Whole-row tensors go file → pinned buffer → device without touching the mapping: two pinned chunks take turns
    // (pread into one while the copy engine drains the other), and a device staging buffer that only grows receives
    // the tensor before it is placed.  Host memory in use stays at the two chunks whatever the file size.
    constexpr size_t kChunk = (size_t)32 << 20;
    uint8_t* pin[2] = { nullptr, nullptr };
    cudaEvent_t pin_free[2] = { nullptr, nullptr };
    void* dev_stage = nullptr; size_t dev_stage_cap = 0;
    auto cleanup = [&](int rc) {
        for (atlasx_safetensors* f : files) atlasx_safetensors_close(f);
        if (rc && m) atlasx_model_free(m);
        cudaStreamSynchronize(ctx->stream);
        for (int i = 0; i < 2; i++) { if (pin[i]) cudaFreeHost(pin[i]); if (pin_free[i]) cudaEventDestroy(pin_free[i]); }
        cudaFree(dev_stage);
        return rc;
    };
    auto stream_rows = [&](const atlasx_safetensors* st, size_t file_off, size_t bytes) -> int {
        if (!pin[0]) {
            for (int i = 0; i < 2; i++) {
                AX_CUDA(cudaMallocHost((void**)&pin[i], kChunk));
                AX_CUDA(cudaEventCreateWithFlags(&pin_free[i], cudaEventDisableTiming));
            }
        }
        if (bytes > dev_stage_cap) {
            AX_CUDA(cudaStreamSynchronize(ctx->stream));
            cudaFree(dev_stage); dev_stage = nullptr; dev_stage_cap = 0;
            AX_CUDA(cudaMalloc(&dev_stage, bytes));
            dev_stage_cap = bytes;
        }
        int turn = 0;
        for (size_t o = 0; o < bytes; o += kChunk, turn ^= 1) {
            const size_t len = bytes - o < kChunk ? bytes - o : kChunk;
            AX_CUDA(cudaEventSynchronize(pin_free[turn]));                // the copy that last used this chunk is done
            size_t got = 0;
            while (got < len) {
                const ssize_t r = pread(st->fd, pin[turn] + got, len - got, (off_t)(file_off + o + got));
                if (r <= 0) return atlasx_fail(ATLASX_ERR_ARG, "%s: short read at offset %zu", st->path.c_str(), file_off + o + got);
                got += (size_t)r;
            }
            AX_CUDA(cudaMemcpyAsync((uint8_t*)dev_stage + o, pin[turn], len, cudaMemcpyHostToDevice, ctx->stream));
            AX_CUDA(cudaEventRecord(pin_free[turn], ctx->stream));
        }
        return ATLASX_OK;
    };
    // later files win over earlier ones for a repeated name, as inserting into the reference's map does (:2480)
    std::map<std::string, Source> all;
    for (const std::string& p : paths) {
        atlasx_safetensors* st = nullptr;
        int rc = atlasx_safetensors_open(p.c_str(), &st);
        if (rc) return cleanup(rc);
        files.push_back(st);
        for (int i = 0; i < (int)st->tensors.size(); i++) all[st->tensors[(size_t)i].name] = Source{ st, i };
    }
    // architecture features from the tensor names, before any tensor is placed (:2493-2515)
    bool post_norm = false, separate_head = false, any_linear = false, all_linear_bf16 = true;
    for (const auto& kv : all) {
        if (kv.first.find("post_feedforward_layernorm") != std::string::npos) post_norm = true;
        if (kv.first == "lm_head.weight") separate_head = true;
        if (ends_with(kv.first, "_proj.weight")) {
            any_linear = true;
            if (kv.second.st->tensors[(size_t)kv.second.index].dtype != ATLASX_BF16) all_linear_bf16 = false;
        }
    }
    cfg.post_norm = post_norm ? 1 : 0;
    if (cfg.weight_format == ATLASX_AUTO) cfg.weight_format = (any_linear && all_linear_bf16) ? ATLASX_BF16 : ATLASX_F32;
    int rc = atlasx_model_create(ctx, &cfg, layer_sliding, &m);
    if (rc) return cleanup(rc);

    size_t file_bytes = 0, up_bytes = 0;
    int used = 0;
    std::vector<uint8_t> stage;                           // host staging for gathered or converted slices
    for (const auto& kv : all) {
        int layer, which;
        if (!classify(kv.first, cfg.n_layers, post_norm, &layer, &which)) continue;
        const atlasx_safetensors* st = kv.second.st;
        const TensorDesc& d = st->tensors[(size_t)kv.second.index];
        if (d.dtype < 0) return cleanup(atlasx_fail(ATLASX_ERR_ARG, "unsupported dtype: %s (tensor %s)", d.dtype_name.c_str(), d.name.c_str()));
        size_t rows, cols;
        if (!tensor_2d(d, &rows, &cols)) return cleanup(atlasx_fail(ATLASX_ERR_ARG, "tensor '%s': shape and byte count disagree", d.name.c_str()));
        size_t fr, fc, r0, r1, c0, c1; int whole = 0;
        rc = atlasx_model_tensor_slice(m, which, &fr, &fc, &r0, &r1, &c0, &c1, &whole);
        if (rc) return cleanup(rc);
        if (rows * cols != fr * fc)
            return cleanup(atlasx_fail(ATLASX_ERR_ARG, "tensor '%s' holds %zu elements, the configuration expects %zu × %zu",
                                       d.name.c_str(), rows * cols, fr, fc));
        rows = fr; cols = fc;
        if (whole) { r0 = 0; r1 = rows; c0 = 0; c1 = cols; }
        const size_t nr = r1 - r0, nc = c1 - c0;
        if (nr == 0 || nc == 0) continue;                 // this rank keeps nothing of it (padded vocabulary)
        const int up_dtype = d.dtype == ATLASX_BF16 ? ATLASX_BF16 : ATLASX_F32;
        const size_t esz = up_dtype == ATLASX_BF16 ? 2 : 4;
        const uint8_t* src = st->map + st->data_start + d.off0;
        const void* host = nullptr;
        int on_device = 0;
        if (d.dtype != ATLASX_F16 && nc == cols) {
            // whole rows: the bytes as they lie in the file, streamed through the pinned chunks
            rc = stream_rows(st, st->data_start + d.off0 + r0 * cols * esz, nr * nc * esz);
            if (rc) return cleanup(rc);
            host = dev_stage; on_device = 1;
        } else {
            stage.resize(nr * nc * esz);
            rc = atlasx_safetensors_read(st, kv.second.index, r0, r1, c0, c1, up_dtype, stage.data());
            if (rc) return cleanup(rc);
            host = stage.data();
        }
        file_bytes += nr * nc * (d.dtype == ATLASX_F32 ? 4 : 2);
        up_bytes += nr * nc * esz;
        rc = whole ? atlasx_model_set_tensor(m, layer < 0 ? 0 : layer, which, host, up_dtype, on_device)
                   : atlasx_model_set_tensor_slice(m, layer < 0 ? 0 : layer, which, host, up_dtype, on_device);
        if (rc) return cleanup(rc);
        // pages of the mapping that a gathered or converted slice touched are not needed again
        if (!on_device) {
            const long pg = sysconf(_SC_PAGESIZE);
            const uintptr_t a0 = ((uintptr_t)src + r0 * cols * esz) & ~(uintptr_t)(pg - 1);
            const uintptr_t a1 = (uintptr_t)src + r1 * cols * esz;
            if (a1 > a0) madvise((void*)a0, a1 - a0, MADV_DONTNEED);
        }
        used++;
    }
    (void)separate_head;                                  // tying happens in finalize when no lm_head tensor was placed (:2309-2312)
    rc = atlasx_model_finalize(m);
    if (rc) return cleanup(rc);
    if (stats) {
        stats->seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        stats->file_bytes_read = file_bytes; stats->bytes_uploaded = up_bytes;
        stats->peak_host_rss_bytes = peak_rss_bytes();
        stats->n_tensors_used = used; stats->post_norm = post_norm ? 1 : 0; stats->tied_lm_head = separate_head ? 0 : 1;
        stats->weight_format = cfg.weight_format;
    }
    *out = m;
    return cleanup(ATLASX_OK);
}

}  // namespace

extern "C" int atlasx_model_load_safetensors(atlasx_ctx* ctx, const char* const* paths, int n_paths, const atlasx_model_config* cfg,
                                             const int* layer_sliding, atlasx_model** out, atlasx_load_stats* stats) {
    AX_ARG(ctx && paths && n_paths > 0 && cfg && out, "bad argument");
    std::vector<std::string> ps;
    for (int i = 0; i < n_paths; i++) { AX_ARG(paths[i], "null path"); ps.push_back(paths[i]); }
    return load_from_files(ctx, ps, *cfg, layer_sliding, out, stats);
}

// config.json overlay (patch_config_from_hf_json :2367-2432): only the fields present are changed;
// max_seq_len is never taken from the file.  sliding_out: n_layers ints when layer_types is present.
extern "C" int atlasx_config_patch_from_json(const char* config_json_path, atlasx_model_config* cfg, int* sliding_out, int* have_layer_types) {
    AX_ARG(config_json_path && cfg, "null argument");
    if (have_layer_types) *have_layer_types = 0;
    std::string text;
    if (!read_text_file(config_json_path, text)) return atlasx_fail(ATLASX_ERR_ARG, "config.json read: %s", strerror(errno));
    JVal j; std::string err;
    if (!parse_json(text.data(), text.size(), j, err)) return atlasx_fail(ATLASX_ERR_ARG, "config.json parse: %s", err.c_str());
    if (const JVal* lt = j.get("layer_types")) {
        if (lt->kind == JVal::Arr) {
            if (sliding_out)
                for (size_t i = 0; i < lt->arr.size() && (int)i < cfg->n_layers; i++)
                    sliding_out[i] = lt->arr[i].kind == JVal::Str && lt->arr[i].str == "sliding_attention";
            if (have_layer_types) *have_layer_types = (int)lt->arr.size();
        }
    }
    size_t u; double f;
    if (const JVal* v = j.get("sliding_window")) if (v->as_usize(&u)) cfg->sliding_window = (int)u;
    if (const JVal* rs = j.get("rope_scaling")) {
        const JVal* t = rs->get("rope_type");
        if (t && t->kind == JVal::Str && t->str == "yarn") {
            cfg->rope_scaling = 1;
            cfg->yarn_factor = 1.0f; cfg->yarn_orig_max_pos = cfg->max_seq_len; cfg->yarn_attn_factor = 1.0f;
            cfg->yarn_beta_fast = 32.0f; cfg->yarn_beta_slow = 1.0f;
            if (const JVal* v = rs->get("factor")) if (v->as_f64(&f)) cfg->yarn_factor = (float)f;
            if (const JVal* v = rs->get("original_max_position_embeddings")) if (v->as_usize(&u)) cfg->yarn_orig_max_pos = (int)u;
            if (const JVal* v = rs->get("attention_factor")) if (v->as_f64(&f)) cfg->yarn_attn_factor = (float)f;
            if (const JVal* v = rs->get("beta_fast")) if (v->as_f64(&f)) cfg->yarn_beta_fast = (float)f;
            if (const JVal* v = rs->get("beta_slow")) if (v->as_f64(&f)) cfg->yarn_beta_slow = (float)f;
        }
    }
    if (const JVal* v = j.get("rope_theta")) if (v->as_f64(&f)) cfg->rope_theta = (float)f;
    if (const JVal* v = j.get("rms_norm_eps")) if (v->as_f64(&f)) cfg->rms_norm_eps = (float)f;
    if (const JVal* v = j.get("eos_token_id")) if (v->as_usize(&u)) cfg->eos_token_id = (int)u;
    return ATLASX_OK;
}

extern "C" int atlasx_model_load_dir(atlasx_ctx* ctx, const char* dir, const atlasx_model_config* cfg_in, const int* layer_sliding,
                                     atlasx_model** out, atlasx_load_stats* stats) {
    AX_ARG(ctx && dir && cfg_in && out, "bad argument");
    atlasx_model_config cfg = *cfg_in;
    const std::string d(dir);
    std::vector<int> sliding((size_t)cfg.n_layers, 0);
    if (layer_sliding) for (int i = 0; i < cfg.n_layers; i++) sliding[(size_t)i] = layer_sliding[i];
    bool have_sliding = layer_sliding != nullptr;
    struct stat sb;
    const std::string cj = d + "/config.json";
    if (stat(cj.c_str(), &sb) == 0) {
        std::vector<int> from_file((size_t)cfg.n_layers, 0);
        int n_lt = 0;
        int rc = atlasx_config_patch_from_json(cj.c_str(), &cfg, from_file.data(), &n_lt);
        if (rc) return rc;
        if (n_lt > 0) { sliding = from_file; have_sliding = true; }
    }
    std::vector<std::string> shards;
    const std::string idx = d + "/model.safetensors.index.json";
    if (stat(idx.c_str(), &sb) == 0) {
        std::string text;
        if (!read_text_file(idx, text)) return atlasx_fail(ATLASX_ERR_ARG, "index.json: %s", strerror(errno));
        // every quoted string that ends in ".safetensors", sorted, once each (:2455-2462)
        size_t p = 0;
        while (p < text.size()) {
            const size_t q = text.find('"', p);
            const std::string piece = text.substr(p, q == std::string::npos ? std::string::npos : q - p);
            if (ends_with(piece, ".safetensors")) shards.push_back(d + "/" + piece);
            if (q == std::string::npos) break;
            p = q + 1;
        }
        std::sort(shards.begin(), shards.end());
        shards.erase(std::unique(shards.begin(), shards.end()), shards.end());
        if (shards.empty()) return atlasx_fail(ATLASX_ERR_ARG, "index.json names no shard");
    } else {
        shards.push_back(d + "/model.safetensors");
    }
    return load_from_files(ctx, shards, cfg, have_sliding ? sliding.data() : nullptr, out, stats);
}
