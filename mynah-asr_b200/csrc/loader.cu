// Direct-to-device model loading: a weight file (safetensors or GGUF) is mapped read-only, its tensor directory is
// read, and every tensor goes from the mapping through the pinned staging buffers into the device slabs, where
// block-quantised tensors are re-tiled and decoded once by kernels. Nothing is decoded on the host and no f32 copy
// of a quantised tensor ever exists in host memory.
//
// The reference opens the same two containers through its vendored reader and decodes every GGUF block tensor
// to f32 on the host at load (src/weights.c:60-117: ingot_wfile_open, then ingot_wfile_to_f32 per tensor), which
// doubles the host memory of a quantised model and takes seconds; its own int8 / int4 formats are mapped as they
// are ("<name>.q8" / "<name>.q4" + "<name>.scales", src/qmat.c:114-142). This file replaces that step for the
// device path. The container layouts are the published ones:
//   safetensors: u64 little-endian header length, a JSON object {name: {dtype, shape, data_offsets}}, raw data;
//   GGUF v2/v3:  "GGUF", u32 version, u64 tensor count, u64 key/value count, the key/value pairs, the tensor
//                infos (name, n_dims, dims with the fastest dimension FIRST, ggml type, offset), then the data
//                section aligned to general.alignment (default 32).
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <chrono>
#include <memory>

#include "model.h"

using namespace mb;

namespace {

struct Mapping {
    const uint8_t *p = nullptr;
    size_t n = 0;
    int open(const char *path) {
        const int fd = ::open(path, O_RDONLY);
        if (fd < 0) { set_error("cannot open '%s'", path); return -1; }
        struct stat st;
        if (fstat(fd, &st) != 0 || st.st_size <= 0) { ::close(fd); set_error("cannot stat '%s'", path); return -1; }
        void *m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
        ::close(fd);
        if (m == MAP_FAILED) { set_error("cannot map '%s'", path); return -1; }
        p = (const uint8_t *)m; n = (size_t)st.st_size;
        return 0;
    }
    ~Mapping() { if (p) munmap(const_cast<uint8_t *>(p), n); }
};

struct FileTensor {
    std::string name;
    std::string dtype;                 // safetensors dtype name, or "ggml" for a GGUF block type
    int ggml_type = -1;
    std::vector<int64_t> shape;        // row-major (PyTorch) order
    const uint8_t *data = nullptr;
    size_t bytes = 0;
};

// ------------------------------------------------------------------ safetensors header (a small JSON subset)
struct Json {
    const char *s, *e;
    bool fail = false;
    void ws() { while (s < e && (*s == ' ' || *s == '\n' || *s == '\t' || *s == '\r')) s++; }
    bool eat(char c) { ws(); if (s < e && *s == c) { s++; return true; } return false; }
    std::string str() {
        ws();
        std::string out;
        if (s >= e || *s != '"') { fail = true; return out; }
        for (s++; s < e && *s != '"'; s++) {
            if (*s == '\\' && s + 1 < e) { s++; out.push_back(*s == 'n' ? '\n' : *s == 't' ? '\t' : *s); }
            else out.push_back(*s);
        }
        if (s >= e) fail = true; else s++;
        return out;
    }
    long long num() {
        ws();
        char *end = nullptr;
        const long long v = strtoll(s, &end, 10);
        if (end == s) fail = true;
        s = end;
        return v;
    }
    void skip() {                      // any value
        ws();
        if (s >= e) { fail = true; return; }
        if (*s == '"') { str(); return; }
        if (*s == '{' || *s == '[') {
            const char close = *s == '{' ? '}' : ']';
            s++;
            if (eat(close)) return;
            do {
                if (close == '}') { str(); if (!eat(':')) { fail = true; return; } }
                skip();
                if (fail) return;
            } while (eat(','));
            if (!eat(close)) fail = true;
            return;
        }
        while (s < e && *s != ',' && *s != '}' && *s != ']') s++;      // number / true / false / null
    }
};

int parse_safetensors(const Mapping &mp, std::vector<FileTensor> &out) {
    if (mp.n < 10) { set_error("safetensors: file too short"); return -1; }
    uint64_t hl = 0;
    memcpy(&hl, mp.p, 8);
    if (hl > mp.n - 8) { set_error("safetensors: header length %llu exceeds the file", (unsigned long long)hl); return -1; }
    const uint8_t *data = mp.p + 8 + hl;
    const size_t data_bytes = mp.n - 8 - (size_t)hl;
    Json j{(const char *)mp.p + 8, (const char *)mp.p + 8 + hl};
    if (!j.eat('{')) { set_error("safetensors: header is not a JSON object"); return -1; }
    if (j.eat('}')) return 0;
    do {
        FileTensor t;
        t.name = j.str();
        if (j.fail || !j.eat(':')) { set_error("safetensors: malformed header"); return -1; }
        if (t.name == "__metadata__") { j.skip(); continue; }
        if (!j.eat('{')) { set_error("safetensors: entry '%s' is not an object", t.name.c_str()); return -1; }
        long long off0 = -1, off1 = -1;
        do {
            const std::string key = j.str();
            if (!j.eat(':')) { j.fail = true; break; }
            if (key == "dtype") t.dtype = j.str();
            else if (key == "shape") {
                if (!j.eat('[')) { j.fail = true; break; }
                if (!j.eat(']')) { do t.shape.push_back(j.num()); while (j.eat(',')); if (!j.eat(']')) j.fail = true; }
            } else if (key == "data_offsets") {
                if (!j.eat('[')) { j.fail = true; break; }
                off0 = j.num();
                if (!j.eat(',')) j.fail = true;
                off1 = j.num();
                if (!j.eat(']')) j.fail = true;
            } else j.skip();
        } while (!j.fail && j.eat(','));
        if (j.fail || !j.eat('}') || off0 < 0 || off1 < off0 || (size_t)off1 > data_bytes) {
            set_error("safetensors: malformed entry '%s'", t.name.c_str()); return -1;
        }
        t.data = data + off0;
        t.bytes = (size_t)(off1 - off0);
        out.push_back(std::move(t));
    } while (j.eat(','));
    if (j.fail) { set_error("safetensors: malformed header"); return -1; }
    return 0;
}

// ------------------------------------------------------------------ GGUF
struct Cursor {
    const uint8_t *p, *e;
    bool fail = false;
    template <typename T> T get() {
        T v{};
        if ((size_t)(e - p) < sizeof(T)) { fail = true; return v; }
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (fail || n > (size_t)(e - p)) { fail = true; return std::string(); }
        std::string s((const char *)p, (size_t)n);
        p += n;
        return s;
    }
    void skip(size_t n) { if (n > (size_t)(e - p)) fail = true; else p += n; }
};

// bytes of a scalar key/value type (GGUF value types 0..12; 8 = string, 9 = array)
size_t gguf_scalar(uint32_t t) {
    switch (t) {
    case 0: case 1: case 7: return 1;      // u8, i8, bool
    case 2: case 3: return 2;              // u16, i16
    case 4: case 5: case 6: return 4;      // u32, i32, f32
    case 10: case 11: case 12: return 8;   // u64, i64, f64
    default: return 0;
    }
}

int parse_gguf(const Mapping &mp, std::vector<FileTensor> &out) {
    Cursor c{mp.p, mp.p + mp.n};
    const uint32_t magic = c.get<uint32_t>(), version = c.get<uint32_t>();
    if (magic != 0x46554747u || version < 2 || version > 3) { set_error("GGUF: bad magic or unsupported version %u", version); return -1; }
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    uint64_t alignment = 32;
    for (uint64_t i = 0; i < n_kv && !c.fail; i++) {
        const std::string key = c.str();
        const uint32_t type = c.get<uint32_t>();
        if (type == 8) c.str();
        else if (type == 9) {
            const uint32_t et = c.get<uint32_t>();
            const uint64_t n = c.get<uint64_t>();
            if (et == 8) { for (uint64_t k = 0; k < n && !c.fail; k++) c.str(); }
            else if (gguf_scalar(et)) c.skip((size_t)n * gguf_scalar(et));
            else c.fail = true;
        } else if (gguf_scalar(type)) {
            if (key == "general.alignment" && type == 4) alignment = c.get<uint32_t>();
            else c.skip(gguf_scalar(type));
        } else c.fail = true;
    }
    if (c.fail || alignment == 0 || (alignment & (alignment - 1))) { set_error("GGUF: malformed key/value section"); return -1; }
    struct Info { FileTensor t; uint64_t off; };
    std::vector<Info> infos;
    for (uint64_t i = 0; i < n_tensors && !c.fail; i++) {
        Info in;
        in.t.name = c.str();
        const uint32_t nd = c.get<uint32_t>();
        if (nd > 8) { c.fail = true; break; }
        std::vector<int64_t> ne(nd);
        for (uint32_t d = 0; d < nd; d++) ne[d] = (int64_t)c.get<uint64_t>();
        in.t.shape.assign(ne.rbegin(), ne.rend());          // GGUF lists the fastest dimension first
        in.t.ggml_type = (int)c.get<uint32_t>();
        in.t.dtype = "ggml";
        in.off = c.get<uint64_t>();
        infos.push_back(std::move(in));
    }
    if (c.fail) { set_error("GGUF: malformed tensor directory"); return -1; }
    const size_t dir_end = (size_t)(c.p - mp.p);
    const size_t data0 = (dir_end + alignment - 1) & ~(size_t)(alignment - 1);
    for (Info &in : infos) {
        size_t nelem = 1;
        for (int64_t s : in.t.shape) nelem *= (size_t)s;
        size_t bytes = 0;
        switch (in.t.ggml_type) {
        case 0: bytes = nelem * 4; break;                    // F32
        case 1: bytes = nelem * 2; break;                    // F16
        case 2: bytes = nelem / 32 * 18; break;              // Q4_0
        case 8: bytes = nelem / 32 * 34; break;              // Q8_0
        case 12: bytes = nelem / 256 * 144; break;           // Q4_K
        case 14: bytes = nelem / 256 * 210; break;           // Q6_K
        default: set_error("GGUF: tensor '%s' has ggml type %d, which this backend does not take", in.t.name.c_str(), in.t.ggml_type); return -1;
        }
        if (in.off % alignment || data0 + in.off + bytes > mp.n) { set_error("GGUF: tensor '%s' lies outside the file", in.t.name.c_str()); return -1; }
        in.t.data = mp.p + data0 + in.off;
        in.t.bytes = bytes;
        out.push_back(std::move(in.t));
    }
    return 0;
}

float half_to_float(uint16_t h) {
    const uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 31, m = h & 1023;
    uint32_t u;
    if (e == 0) {
        if (m == 0) u = s;
        else { int sh = 0; uint32_t mm = m; while (!(mm & 1024)) { mm <<= 1; sh++; } u = s | ((uint32_t)(113 - sh) << 23) | ((mm & 1023) << 13); }
    } else if (e == 31) u = s | 0x7F800000u | (m << 13);
    else u = s | ((e + 112) << 23) | (m << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}

bool ends_with(const std::string &s, const char *suf) {
    const size_t n = strlen(suf);
    return s.size() >= n && s.compare(s.size() - n, n, suf) == 0;
}

}  // namespace

extern "C" mynah_b200_model *mynah_b200_model_load(const char *weights_path, const char *mel_path, const mynah_b200_config *cfg,
                                                   int quant) {
    if (!weights_path) { set_error("model_load: no path"); return nullptr; }
    const auto t0 = std::chrono::steady_clock::now();
    Mapping mw, mm;
    if (mw.open(weights_path)) return nullptr;
    std::vector<FileTensor> tensors, mel;
    const bool is_gguf = mw.n >= 4 && memcmp(mw.p, "GGUF", 4) == 0;
    if ((is_gguf ? parse_gguf(mw, tensors) : parse_safetensors(mw, tensors)) != 0) return nullptr;
    mynah_b200_model *h = mynah_b200_model_new(cfg);
    if (!h) return nullptr;
    std::vector<std::unique_ptr<std::vector<float>>> converted;       // f16 / bf16 tensors widened on the host (small ones)
    // the reference-native quantised forms a file may carry beside (or instead of) the f32 tensor
    auto has = [&](const std::string &n) { for (const FileTensor &t : tensors) if (t.name == n) return true; return false; };
    int rc = 0;
    for (const FileTensor &t : tensors) {
        if (rc) break;
        std::string name = t.name;
        int fmt = -1;
        const void *data = t.data;
        std::vector<int64_t> shape = t.shape;
        if (t.dtype == "ggml" && t.ggml_type != 1) fmt = t.ggml_type == 0 ? MYNAH_B200_F32 : 100 + t.ggml_type;
        if (t.dtype == "F32") fmt = MYNAH_B200_F32;
        const bool f16 = t.dtype == "F16" || (t.dtype == "ggml" && t.ggml_type == 1), bf16 = t.dtype == "BF16";
        if (f16 || bf16) {
            const size_t n = t.bytes / 2;
            converted.emplace_back(new std::vector<float>(n));
            const uint16_t *src = (const uint16_t *)t.data;
            float *dst = converted.back()->data();
            for (size_t i = 0; i < n; i++) {
                if (f16) dst[i] = half_to_float(src[i]);
                else { const uint32_t u = (uint32_t)src[i] << 16; memcpy(&dst[i], &u, 4); }
            }
            data = dst;
            fmt = MYNAH_B200_F32;
        }
        if (ends_with(name, ".q8") && t.dtype == "I8") {
            if (quant != 1) continue;                                  // the caller asked for another form of this weight
            name.resize(name.size() - 3);
            fmt = MYNAH_B200_MYNAH_Q8;
        } else if (ends_with(name, ".q4") && t.dtype == "U8") {
            if (quant != 2) continue;
            name.resize(name.size() - 3);
            fmt = MYNAH_B200_MYNAH_Q4;
            if (!shape.empty()) shape.back() *= 2;                     // two nibbles per byte
        } else if (fmt == MYNAH_B200_F32 && ((quant == 1 && has(name + ".q8")) || (quant == 2 && has(name + ".q4")))) {
            continue;                                                  // superseded by its pre-quantised form
        }
        if (fmt < 0) { set_error("model_load: tensor '%s' has dtype %s, which this backend does not take", t.name.c_str(), t.dtype.c_str()); rc = -1; break; }
        rc = mynah_b200_model_add_tensor(h, name.c_str(), fmt, shape.data(), (int)shape.size(), data);
    }
    if (rc == 0 && mel_path) {
        if (mm.open(mel_path) || parse_safetensors(mm, mel)) rc = -1;
        const FileTensor *fb = nullptr, *win = nullptr;
        for (const FileTensor &t : mel) { if (t.name == "mel_fb") fb = &t; if (t.name == "window") win = &t; }
        if (rc == 0 && (!fb || !win || fb->dtype != "F32" || win->dtype != "F32")) { set_error("model_load: '%s' lacks f32 mel_fb / window", mel_path); rc = -1; }
        if (rc == 0) rc = mynah_b200_model_set_mel(h, (const float *)fb->data, (const float *)win->data);
    }
    if (rc == 0) rc = mynah_b200_model_finalize(h);
    if (rc != 0) { mynah_b200_model_free(h); return nullptr; }
    set_load_seconds(h, std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
    return h;
}
