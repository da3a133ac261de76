// Reader for the safetensors container and the GPT-2 checkpoint loader on top of it (host code only).
//
// The reference reads checkpoints with the `safetensors` crate (crates/core/gpu-host/Cargo.toml) in
// crates/core/gpu-host/src/model.rs: list_tensors (201-221), load_gpt2_weights (308-386, Hugging
// Face key names, F32 only, Conv1D weights kept [in,out]) and load_all_tensors (388-397).  The file
// format is public: an 8-byte little-endian header length N, N bytes of JSON mapping each tensor
// name to {"dtype", "shape", "data_offsets": [begin, end)} (offsets relative to the end of the
// header; an optional "__metadata__" object of strings), then the raw little-endian tensor bytes.
// This file restates that format; nothing of the crate is used.
#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <map>

#include "model.h"

namespace {

struct StEntry {
    std::string name, dtype;
    std::vector<size_t> shape;
    size_t begin = 0, end = 0;
};

thread_local std::string g_st_error;

int st_fail(int code, const std::string &msg) {
    g_st_error = msg;
    return code;
}

// ---- a JSON reader sufficient for the header: objects, arrays, strings, non-negative integers ----
struct Json {
    const char *p, *e;
    bool ok = true;
    void ws() {
        while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
    }
    bool eat(char c) {
        ws();
        if (p < e && *p == c) { ++p; return true; }
        return false;
    }
    bool str(std::string &out) {
        ws();
        if (p >= e || *p != '"') return ok = false;
        ++p;
        out.clear();
        while (p < e && *p != '"') {
            if (*p == '\\') {
                if (++p >= e) return ok = false;
                switch (*p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': { // basic multilingual plane -> UTF-8
                        if (e - p < 5) return ok = false;
                        unsigned v = 0;
                        for (int i = 1; i <= 4; ++i) {
                            const char h = p[i];
                            v <<= 4;
                            if (h >= '0' && h <= '9') v |= h - '0';
                            else if (h >= 'a' && h <= 'f') v |= h - 'a' + 10;
                            else if (h >= 'A' && h <= 'F') v |= h - 'A' + 10;
                            else return ok = false;
                        }
                        p += 4;
                        if (v < 0x80) out += (char)v;
                        else if (v < 0x800) { out += (char)(0xC0 | (v >> 6)); out += (char)(0x80 | (v & 0x3F)); }
                        else { out += (char)(0xE0 | (v >> 12)); out += (char)(0x80 | ((v >> 6) & 0x3F)); out += (char)(0x80 | (v & 0x3F)); }
                        break;
                    }
                    default: out += *p; // \" \\ \/
                }
                ++p;
            } else {
                out += *p++;
            }
        }
        if (p >= e) return ok = false;
        ++p;
        return true;
    }
    bool uint(size_t &v) {
        ws();
        if (p >= e || *p < '0' || *p > '9') return ok = false;
        v = 0;
        while (p < e && *p >= '0' && *p <= '9') v = v * 10 + (size_t)(*p++ - '0');
        return true;
    }
    bool skip() { // any value
        ws();
        if (p >= e) return ok = false;
        if (*p == '"') { std::string s; return str(s); }
        if (*p == '{' || *p == '[') {
            const char close = *p == '{' ? '}' : ']';
            const bool obj = *p == '{';
            ++p;
            if (eat(close)) return true;
            do {
                if (obj) { std::string k; if (!str(k) || !eat(':')) return ok = false; }
                if (!skip()) return false;
            } while (eat(','));
            return eat(close) ? true : (ok = false);
        }
        while (p < e && *p != ',' && *p != '}' && *p != ']') ++p; // number / true / false / null
        return true;
    }
};

size_t dtype_size(const std::string &d) {
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
    if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
    return 0;
}

}  // namespace

struct b200nn_safetensors {
    std::string path;
    FILE *f = nullptr;
    size_t data_start = 0, file_size = 0;
    std::vector<StEntry> entries; // sorted by name, as list_tensors returns them
    ~b200nn_safetensors() {
        if (f) fclose(f);
    }
};

extern "C" const char *b200nn_safetensors_last_error(void) { return g_st_error.c_str(); }

extern "C" int32_t b200nn_safetensors_open(const char *path, b200nn_safetensors **out) {
    if (!path || !out) return st_fail(B200NN_ERR_ARG, "null argument");
    *out = nullptr;
    auto st = std::unique_ptr<b200nn_safetensors>(new b200nn_safetensors());
    st->path = path;
    st->f = fopen(path, "rb");
    if (!st->f) return st_fail(B200NN_ERR_IO, std::string("cannot open ") + path + ": " + strerror(errno));
    if (fseek(st->f, 0, SEEK_END) != 0) return st_fail(B200NN_ERR_IO, "seek failed");
    const long fsz = ftell(st->f);
    if (fsz < 8) return st_fail(B200NN_ERR_IO, "file shorter than the 8-byte header length");
    st->file_size = (size_t)fsz;
    fseek(st->f, 0, SEEK_SET);
    unsigned char lenb[8];
    if (fread(lenb, 1, 8, st->f) != 8) return st_fail(B200NN_ERR_IO, "cannot read the header length");
    uint64_t n = 0;
    for (int i = 7; i >= 0; --i) n = (n << 8) | lenb[i];
    if (n > st->file_size - 8 || n > ((uint64_t)100 << 20))
        return st_fail(B200NN_ERR_IO, "header length exceeds the file (or the 100 MB the format allows)");
    std::string hdr((size_t)n, '\0');
    if (n && fread(&hdr[0], 1, (size_t)n, st->f) != (size_t)n) return st_fail(B200NN_ERR_IO, "cannot read the header");
    st->data_start = 8 + (size_t)n;
    const size_t data_len = st->file_size - st->data_start;

    Json j{hdr.data(), hdr.data() + hdr.size()};
    if (!j.eat('{')) return st_fail(B200NN_ERR_IO, "header is not a JSON object");
    if (!j.eat('}')) {
        do {
            StEntry en;
            if (!j.str(en.name) || !j.eat(':')) return st_fail(B200NN_ERR_IO, "malformed header (tensor name)");
            if (en.name == "__metadata__") {
                if (!j.skip()) return st_fail(B200NN_ERR_IO, "malformed header (__metadata__)");
                continue;
            }
            if (!j.eat('{')) return st_fail(B200NN_ERR_IO, "malformed header (tensor entry)");
            bool have_d = false, have_s = false, have_o = false;
            do {
                std::string key;
                if (!j.str(key) || !j.eat(':')) return st_fail(B200NN_ERR_IO, "malformed header (entry key)");
                if (key == "dtype") {
                    have_d = j.str(en.dtype);
                } else if (key == "shape") {
                    if (!j.eat('[')) return st_fail(B200NN_ERR_IO, "malformed header (shape)");
                    if (!j.eat(']')) {
                        do {
                            size_t v;
                            if (!j.uint(v)) return st_fail(B200NN_ERR_IO, "malformed header (shape value)");
                            en.shape.push_back(v);
                        } while (j.eat(','));
                        if (!j.eat(']')) return st_fail(B200NN_ERR_IO, "malformed header (shape end)");
                    }
                    have_s = true;
                } else if (key == "data_offsets") {
                    if (!j.eat('[') || !j.uint(en.begin) || !j.eat(',') || !j.uint(en.end) || !j.eat(']'))
                        return st_fail(B200NN_ERR_IO, "malformed header (data_offsets)");
                    have_o = true;
                } else if (!j.skip()) {
                    return st_fail(B200NN_ERR_IO, "malformed header (entry value)");
                }
            } while (j.eat(','));
            if (!j.eat('}') || !have_d || !have_s || !have_o)
                return st_fail(B200NN_ERR_IO, "malformed header (entry of " + en.name + ")");
            // the checks the format's own reader makes: known dtype, range inside the file, size = numel * width
            const size_t width = dtype_size(en.dtype);
            if (!width) return st_fail(B200NN_ERR_IO, "unknown dtype " + en.dtype + " for " + en.name);
            // element count and byte size with overflow checks: a shape like [2^32, 2^32] must not wrap to 0
            size_t nbytes = width;
            for (size_t s : en.shape)
                if (__builtin_mul_overflow(nbytes, s, &nbytes))
                    return st_fail(B200NN_ERR_IO, "shape of " + en.name + " overflows the addressable size");
            if (en.end < en.begin || en.end > data_len) return st_fail(B200NN_ERR_IO, "data_offsets of " + en.name + " outside the file");
            if (en.end - en.begin != nbytes) return st_fail(B200NN_ERR_IO, "byte size of " + en.name + " does not match its shape");
            st->entries.push_back(std::move(en));
        } while (j.eat(','));
        if (!j.eat('}')) return st_fail(B200NN_ERR_IO, "malformed header (end of object)");
    }
    // as the format's own reader requires: in offset order the tensors follow one another without gap
    // or overlap, starting at 0 and ending at the end of the data section
    {
        std::vector<std::pair<size_t, size_t>> spans;
        for (const StEntry &en : st->entries) spans.emplace_back(en.begin, en.end);
        std::sort(spans.begin(), spans.end());
        size_t at = 0;
        for (const auto &sp : spans) {
            if (sp.first != at) return st_fail(B200NN_ERR_IO, "data_offsets overlap or leave a gap in the data section");
            at = sp.second;
        }
        if (at != data_len) return st_fail(B200NN_ERR_IO, "data_offsets do not cover the data section");
    }
    std::sort(st->entries.begin(), st->entries.end(), [](const StEntry &a, const StEntry &b) { return a.name < b.name; });
    for (size_t i = 1; i < st->entries.size(); ++i)
        if (st->entries[i].name == st->entries[i - 1].name) return st_fail(B200NN_ERR_IO, "duplicate tensor name " + st->entries[i].name);
    *out = st.release();
    return B200NN_OK;
}

extern "C" void b200nn_safetensors_close(b200nn_safetensors *st) { delete st; }
extern "C" int32_t b200nn_safetensors_count(const b200nn_safetensors *st) { return st ? (int32_t)st->entries.size() : 0; }

extern "C" int32_t b200nn_safetensors_info(const b200nn_safetensors *st, int32_t index, const char **name, const char **dtype,
                                           size_t *shape_out, int32_t shape_capacity, int32_t *ndim, size_t *nbytes) {
    if (!st || index < 0 || index >= (int32_t)st->entries.size()) return st_fail(B200NN_ERR_ARG, "tensor index out of range");
    const StEntry &en = st->entries[index];
    if (name) *name = en.name.c_str();
    if (dtype) *dtype = en.dtype.c_str();
    if (ndim) *ndim = (int32_t)en.shape.size();
    if (nbytes) *nbytes = en.end - en.begin;
    if (shape_out)
        for (int32_t i = 0; i < shape_capacity && i < (int32_t)en.shape.size(); ++i) shape_out[i] = en.shape[i];
    return B200NN_OK;
}

extern "C" int32_t b200nn_safetensors_find(const b200nn_safetensors *st, const char *name) {
    if (!st || !name) return -1;
    auto it = std::lower_bound(st->entries.begin(), st->entries.end(), std::string(name),
                               [](const StEntry &a, const std::string &n) { return a.name < n; });
    return (it != st->entries.end() && it->name == name) ? (int32_t)(it - st->entries.begin()) : -1;
}

extern "C" int32_t b200nn_safetensors_read(const b200nn_safetensors *st, int32_t index, void *out, size_t capacity_bytes) {
    if (!st || !out || index < 0 || index >= (int32_t)st->entries.size()) return st_fail(B200NN_ERR_ARG, "bad argument");
    const StEntry &en = st->entries[index];
    const size_t n = en.end - en.begin;
    if (capacity_bytes < n) return st_fail(B200NN_ERR_SHAPE, "destination too small for " + en.name);
    if (fseek(st->f, (long)(st->data_start + en.begin), SEEK_SET) != 0) return st_fail(B200NN_ERR_IO, "seek failed");
    if (n && fread(out, 1, n, st->f) != n) return st_fail(B200NN_ERR_IO, "short read of " + en.name);
    return B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// GPT-2 checkpoint -> model
// ---------------------------------------------------------------------------------------------
namespace {

// extract_f32_tensor (model.rs:243-275): the tensor must exist, be F32 and have exactly this shape.
int take_f32(b200nn_ctx *ctx, const b200nn_safetensors *st, const std::string &name, const std::vector<size_t> &shape,
             std::vector<float> *out) {
    const int idx = b200nn_safetensors_find(st, name.c_str());
    if (idx < 0) return set_error(ctx, B200NN_ERR_MISSING, "missing tensor " + name);
    const StEntry &en = st->entries[idx];
    if (en.dtype != "F32") return set_error(ctx, B200NN_ERR_UNSUPPORTED, "tensor " + name + ": expected dtype F32, got " + en.dtype);
    if (en.shape != shape) {
        std::string got, want;
        for (size_t s : en.shape) got += std::to_string(s) + " ";
        for (size_t s : shape) want += std::to_string(s) + " ";
        return set_error(ctx, B200NN_ERR_SHAPE, "tensor " + name + ": expected shape [ " + want + "], got [ " + got + "]");
    }
    out->resize((en.end - en.begin) / 4);
    if (b200nn_safetensors_read(st, idx, out->data(), out->size() * 4) != B200NN_OK)
        return set_error(ctx, B200NN_ERR_IO, g_st_error);
    return B200NN_OK;
}

}  // namespace

extern "C" int32_t b200nn_gpt2_load_safetensors(b200nn_ctx *ctx, const char *path, const b200nn_gpt2_config *cfg_in,
                                                size_t int4_group, uint32_t flags, b200nn_gpt2 **out) {
    if (!ctx || !path || !out) return B200NN_ERR_ARG;
    *out = nullptr;
    b200nn_safetensors *raw = nullptr;
    int rc = b200nn_safetensors_open(path, &raw);
    if (rc != B200NN_OK) return set_error(ctx, rc, g_st_error);
    std::unique_ptr<b200nn_safetensors> st(raw);

    // the configuration: given, or read off the tensor shapes (wte [vocab,d], wpe [positions,d], layers counted)
    b200nn_gpt2_config cfg;
    if (cfg_in) {
        cfg = *cfg_in;
    } else {
        const int iw = b200nn_safetensors_find(st.get(), "wte.weight"), ip = b200nn_safetensors_find(st.get(), "wpe.weight");
        if (iw < 0 || ip < 0) return set_error(ctx, B200NN_ERR_MISSING, "missing tensor wte.weight / wpe.weight");
        const StEntry &ew = st->entries[iw], &ep = st->entries[ip];
        if (ew.shape.size() != 2 || ep.shape.size() != 2 || ew.shape[1] != ep.shape[1] || ew.shape[1] % 64 != 0)
            return set_error(ctx, B200NN_ERR_SHAPE, "wte.weight / wpe.weight do not describe a GPT-2 (head_dim 64)");
        cfg.vocab_size = (int32_t)ew.shape[0];
        cfg.n_embd = (int32_t)ew.shape[1];
        cfg.n_positions = (int32_t)ep.shape[0];
        cfg.n_head = cfg.n_embd / 64;
        cfg.layer_norm_epsilon = 1e-5f;
        int L = 0;
        while (b200nn_safetensors_find(st.get(), ("h." + std::to_string(L) + ".ln_1.weight").c_str()) >= 0) ++L;
        cfg.n_layer = L;
    }
    if (cfg.n_layer <= 0 || cfg.n_embd <= 0) return set_error(ctx, B200NN_ERR_SHAPE, "empty model configuration");
    const size_t d = (size_t)cfg.n_embd, ffn = 4 * d, V = (size_t)cfg.vocab_size, P = (size_t)cfg.n_positions;

    // Hugging Face key names; Conv1D weights are stored [in,out], which is what the model takes
    std::vector<float> wte, wpe, lnf_w, lnf_b;
    TRY(take_f32(ctx, st.get(), "wte.weight", {V, d}, &wte));
    TRY(take_f32(ctx, st.get(), "wpe.weight", {P, d}, &wpe));
    TRY(take_f32(ctx, st.get(), "ln_f.weight", {d}, &lnf_w));
    TRY(take_f32(ctx, st.get(), "ln_f.bias", {d}, &lnf_b));
    struct Layer { std::vector<float> t[12]; };
    std::vector<Layer> store((size_t)cfg.n_layer);
    std::vector<b200nn_gpt2_layer_weights> lw((size_t)cfg.n_layer);
    for (int i = 0; i < cfg.n_layer; ++i) {
        const std::string h = "h." + std::to_string(i) + ".";
        Layer &s = store[i];
        TRY(take_f32(ctx, st.get(), h + "ln_1.weight", {d}, &s.t[0]));
        TRY(take_f32(ctx, st.get(), h + "ln_1.bias", {d}, &s.t[1]));
        TRY(take_f32(ctx, st.get(), h + "attn.c_attn.weight", {d, 3 * d}, &s.t[2]));
        TRY(take_f32(ctx, st.get(), h + "attn.c_attn.bias", {3 * d}, &s.t[3]));
        TRY(take_f32(ctx, st.get(), h + "attn.c_proj.weight", {d, d}, &s.t[4]));
        TRY(take_f32(ctx, st.get(), h + "attn.c_proj.bias", {d}, &s.t[5]));
        TRY(take_f32(ctx, st.get(), h + "ln_2.weight", {d}, &s.t[6]));
        TRY(take_f32(ctx, st.get(), h + "ln_2.bias", {d}, &s.t[7]));
        TRY(take_f32(ctx, st.get(), h + "mlp.c_fc.weight", {d, ffn}, &s.t[8]));
        TRY(take_f32(ctx, st.get(), h + "mlp.c_fc.bias", {ffn}, &s.t[9]));
        TRY(take_f32(ctx, st.get(), h + "mlp.c_proj.weight", {ffn, d}, &s.t[10]));
        TRY(take_f32(ctx, st.get(), h + "mlp.c_proj.bias", {d}, &s.t[11]));
        b200nn_gpt2_layer_weights &l = lw[i];
        l.ln_1_weight = s.t[0].data();   l.ln_1_bias = s.t[1].data();
        l.c_attn_weight = s.t[2].data(); l.c_attn_bias = s.t[3].data();
        l.c_proj_weight = s.t[4].data(); l.c_proj_bias = s.t[5].data();
        l.ln_2_weight = s.t[6].data();   l.ln_2_bias = s.t[7].data();
        l.mlp_fc_weight = s.t[8].data(); l.mlp_fc_bias = s.t[9].data();
        l.mlp_proj_weight = s.t[10].data(); l.mlp_proj_bias = s.t[11].data();
    }
    b200nn_gpt2_weights w;
    w.wte = wte.data();
    w.wpe = wpe.data();
    w.ln_f_weight = lnf_w.data();
    w.ln_f_bias = lnf_b.data();
    w.layers = lw.data();
    return int4_group ? b200nn_int4_gpt2_create(ctx, &cfg, &w, int4_group, flags, out) : b200nn_gpt2_create(ctx, &cfg, &w, flags, out);
}
