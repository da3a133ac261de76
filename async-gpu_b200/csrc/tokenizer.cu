// Byte-level BPE tokenizer of GPT-2 (host code only; no device work).
//
// The reference wraps the third-party tiktoken-rs crate with its r50k_base encoding
// (crates/core/gpu-host/src/tokenizer.rs:34-62: new, encode = encode_with_special_tokens, decode,
// vocab_size).  That crate and its 50 000-merge vocabulary are not part of the reference tree, so this
// is the published algorithm restated: a table of byte strings with ranks (the vocabulary, read at run
// time from a file in tiktoken's own format: one "base64(token bytes) rank" pair per line), text split
// into pieces by GPT-2's pattern
//     's|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+
// and each piece merged greedily: among the adjacent pairs of parts whose concatenation is in the
// table, the one of lowest rank is merged first, until none is left; the ranks of the parts are the
// token ids.  The one special token, <|endoftext|>, maps to the id given at creation (50256).
//
// Unicode classes in the C++ splitter are exact for ASCII and approximated by block for the rest
// (letters unless the code point lies in a punctuation / symbol / space / digit block listed below);
// the split only decides which merges may happen, so encode followed by decode returns the text
// byte for byte whatever the classification.  The Python mirror splits with exact general categories
// and calls b200nn_bpe_encode_piece per piece.
#include <algorithm>
#include <climits>
#include <cstring>
#include <fstream>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "b200nn.h"

struct b200nn_bpe {
    std::unordered_map<std::string, uint32_t> rank; // token bytes -> id
    std::vector<std::string> bytes_of;              // id -> token bytes ("" = unused id)
    std::string special = "<|endoftext|>";
    uint32_t special_id = 50256;
    size_t vocab_size = 0;
};

namespace {

thread_local std::string g_bpe_error;
int bpe_fail(int code, const std::string &msg) {
    g_bpe_error = msg;
    return code;
}

int b64_val(unsigned char c) {
    if (c >= 'A' && c <= 'Z') return c - 'A';
    if (c >= 'a' && c <= 'z') return c - 'a' + 26;
    if (c >= '0' && c <= '9') return c - '0' + 52;
    if (c == '+') return 62;
    if (c == '/') return 63;
    return -1;
}

bool b64_decode(const std::string &in, std::string *out) {
    out->clear();
    uint32_t acc = 0;
    int bits = 0;
    for (unsigned char c : in) {
        if (c == '=') break;
        const int v = b64_val(c);
        if (v < 0) return false;
        acc = (acc << 6) | (uint32_t)v;
        bits += 6;
        if (bits >= 8) {
            bits -= 8;
            out->push_back((char)((acc >> bits) & 0xFFu));
        }
    }
    return true;
}

// ---- code point classes ------------------------------------------------------------------------
struct Cp {
    uint32_t c;
    int len;
};
// Decodes one UTF-8 sequence; malformed bytes come back as themselves (class "other"), one at a time.
Cp next_cp(const unsigned char *s, size_t n) {
    const unsigned char b = s[0];
    if (b < 0x80) return {b, 1};
    int need = (b >= 0xF0 && b < 0xF8) ? 3 : (b >= 0xE0) ? 2 : (b >= 0xC0) ? 1 : -1;
    if (need < 0 || (size_t)need >= n) return {0xFFFFFFFFu, 1};
    uint32_t c = b & (0x3F >> need);
    for (int i = 1; i <= need; ++i) {
        if ((s[i] & 0xC0) != 0x80) return {0xFFFFFFFFu, 1};
        c = (c << 6) | (s[i] & 0x3Fu);
    }
    return {c, need + 1};
}
bool is_space(uint32_t c) { // Unicode White_Space
    return (c >= 9 && c <= 13) || c == 32 || c == 0x85 || c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) ||
           c == 0x2028 || c == 0x2029 || c == 0x202F || c == 0x205F || c == 0x3000;
}
bool is_number(uint32_t c) { // \p{N}: ASCII digits exactly; the common digit / numeral blocks beyond
    if (c < 0x80) return c >= '0' && c <= '9';
    return c == 0xB2 || c == 0xB3 || c == 0xB9 || (c >= 0xBC && c <= 0xBE) || (c >= 0x660 && c <= 0x669) ||
           (c >= 0x6F0 && c <= 0x6F9) || (c >= 0x966 && c <= 0x96F) || (c >= 0x2070 && c <= 0x2079) ||
           (c >= 0x2080 && c <= 0x2089) || (c >= 0x2150 && c <= 0x218B) || (c >= 0x2460 && c <= 0x249B) ||
           (c >= 0xFF10 && c <= 0xFF19);
}
bool is_letter(uint32_t c) { // \p{L}: ASCII letters exactly; beyond, everything outside the blocks below
    if (c < 0x80) return (c >= 'A' && c <= 'Z') || (c >= 'a' && c <= 'z');
    if (c == 0xFFFFFFFFu || is_space(c) || is_number(c)) return false;
    if (c == 0xAA || c == 0xB5 || c == 0xBA) return true;
    if (c < 0xC0 || c == 0xD7 || c == 0xF7) return false;                // Latin-1 punctuation and signs
    if (c >= 0x2000 && c <= 0x2BFF) return false;                         // punctuation, currency, arrows, math, boxes, symbols
    if (c >= 0x3000 && c <= 0x303F) return false;                         // CJK symbols and punctuation
    if (c >= 0xFE10 && c <= 0xFE6F) return false;                         // vertical / small forms
    if ((c >= 0xFF01 && c <= 0xFF0F) || (c >= 0xFF1A && c <= 0xFF20) || (c >= 0xFF3B && c <= 0xFF40) ||
        (c >= 0xFF5B && c <= 0xFF65))
        return false;                                                      // full-width punctuation
    if (c >= 0x1F000 && c <= 0x1FAFF) return false;                       // emoji and pictographs
    if (c >= 0x300 && c <= 0x36F) return false;                           // combining marks
    if (c >= 0xE000 && c <= 0xF8FF) return false;                         // private use
    return true;
}

// GPT-2's pattern, alternatives tried in order at each position; returns the piece's byte length.
size_t next_piece(const unsigned char *s, size_t n) {
    // 's 't 're 've 'm 'll 'd
    if (s[0] == '\'' && n >= 2) {
        static const char *suf[] = {"s", "t", "re", "ve", "m", "ll", "d"};
        for (const char *x : suf) {
            const size_t l = strlen(x);
            if (n >= 1 + l && !memcmp(s + 1, x, l)) return 1 + l;
        }
    }
    size_t i = 0;
    Cp c0 = next_cp(s, n);
    // optional single space before a run of letters / numbers / others
    size_t lead = 0;
    Cp c1 = c0;
    if (c0.c == ' ' && n > 1) {
        lead = 1;
        c1 = next_cp(s + 1, n - 1);
    }
    auto run = [&](bool (*pred)(uint32_t)) {
        size_t j = lead;
        while (j < n) {
            Cp c = next_cp(s + j, n - j);
            if (!pred(c.c)) break;
            j += c.len;
        }
        return j;
    };
    if (is_letter(c1.c)) return run(is_letter);
    if (is_number(c1.c)) return run(is_number);
    if (!is_space(c1.c)) return run([](uint32_t c) { return !is_space(c) && !is_letter(c) && !is_number(c); });
    // whitespace: \s+(?!\S) takes the run except its last character when a non-space follows; else \s+
    i = 0;
    size_t last = 0;
    while (i < n) {
        Cp c = next_cp(s + i, n - i);
        if (!is_space(c.c)) break;
        last = i;
        i += c.len;
    }
    if (i < n && last > 0) return last; // the last space stays with the next piece (" word")
    return i;
}

// tiktoken's byte_pair_merge on one piece.
void merge_piece(const b200nn_bpe *t, const unsigned char *p, size_t n, std::vector<uint32_t> *out) {
    if (n == 0) return;
    auto whole = t->rank.find(std::string((const char *)p, n));
    if (whole != t->rank.end()) {
        out->push_back(whole->second);
        return;
    }
    std::vector<size_t> start(n + 1);
    for (size_t i = 0; i <= n; ++i) start[i] = i; // part i = bytes [start[i], start[i+1])
    auto pair_rank = [&](size_t i) -> uint32_t {   // rank of parts i and i+1 joined, UINT_MAX if none
        if (i + 2 >= start.size()) return UINT_MAX;
        auto it = t->rank.find(std::string((const char *)p + start[i], start[i + 2] - start[i]));
        return it == t->rank.end() ? UINT_MAX : it->second;
    };
    while (start.size() > 2) {
        uint32_t best = UINT_MAX;
        size_t bi = 0;
        for (size_t i = 0; i + 2 < start.size(); ++i) {
            const uint32_t r = pair_rank(i);
            if (r < best) { // the first of equal ranks, as tiktoken's scan keeps it
                best = r;
                bi = i;
            }
        }
        if (best == UINT_MAX) break;
        start.erase(start.begin() + bi + 1);
    }
    for (size_t i = 0; i + 1 < start.size(); ++i) {
        auto it = t->rank.find(std::string((const char *)p + start[i], start[i + 1] - start[i]));
        out->push_back(it == t->rank.end() ? 0u : it->second); // single bytes are always in a valid table
    }
}

int finish_table(b200nn_bpe *t) {
    for (int b = 0; b < 256; ++b)
        if (!t->rank.count(std::string(1, (char)b))) return bpe_fail(B200NN_ERR_IO, "vocabulary lacks a single-byte token");
    size_t top = 0;
    for (auto &kv : t->rank) top = std::max<size_t>(top, kv.second + 1);
    top = std::max<size_t>(top, (size_t)t->special_id + 1);
    t->bytes_of.assign(top, std::string());
    for (auto &kv : t->rank) {
        if (kv.second == t->special_id) return bpe_fail(B200NN_ERR_IO, "a vocabulary entry uses the special token's id");
        t->bytes_of[kv.second] = kv.first;
    }
    t->vocab_size = top;
    return B200NN_OK;
}

}  // namespace

extern "C" const char *b200nn_bpe_last_error(void) { return g_bpe_error.c_str(); }

extern "C" int32_t b200nn_bpe_create(const uint8_t *token_bytes, const size_t *token_offsets, const uint32_t *ranks,
                                     size_t n_tokens, uint32_t endoftext_id, b200nn_bpe **out) {
    if (!token_bytes || !token_offsets || !ranks || !out) return bpe_fail(B200NN_ERR_ARG, "null argument");
    auto t = std::unique_ptr<b200nn_bpe>(new b200nn_bpe());
    t->special_id = endoftext_id;
    for (size_t i = 0; i < n_tokens; ++i) {
        if (token_offsets[i + 1] <= token_offsets[i]) return bpe_fail(B200NN_ERR_SHAPE, "empty or unordered token entry");
        std::string b((const char *)token_bytes + token_offsets[i], token_offsets[i + 1] - token_offsets[i]);
        if (!t->rank.emplace(std::move(b), ranks[i]).second) return bpe_fail(B200NN_ERR_IO, "duplicate token in the vocabulary");
    }
    int rc = finish_table(t.get());
    if (rc != B200NN_OK) return rc;
    *out = t.release();
    return B200NN_OK;
}

extern "C" int32_t b200nn_bpe_load(const char *path, uint32_t endoftext_id, b200nn_bpe **out) {
    if (!path || !out) return bpe_fail(B200NN_ERR_ARG, "null argument");
    std::ifstream f(path);
    if (!f) return bpe_fail(B200NN_ERR_IO, std::string("cannot open ") + path);
    auto t = std::unique_ptr<b200nn_bpe>(new b200nn_bpe());
    t->special_id = endoftext_id;
    std::string line, tok;
    size_t ln = 0;
    while (std::getline(f, line)) {
        ++ln;
        while (!line.empty() && (line.back() == '\r' || line.back() == ' ')) line.pop_back();
        if (line.empty()) continue;
        const size_t sp = line.find(' ');
        if (sp == std::string::npos || !b64_decode(line.substr(0, sp), &tok) || tok.empty())
            return bpe_fail(B200NN_ERR_IO, "malformed vocabulary line " + std::to_string(ln));
        char *end = nullptr;
        const unsigned long r = strtoul(line.c_str() + sp + 1, &end, 10);
        if (end == line.c_str() + sp + 1 || *end) return bpe_fail(B200NN_ERR_IO, "malformed rank on line " + std::to_string(ln));
        if (!t->rank.emplace(tok, (uint32_t)r).second) return bpe_fail(B200NN_ERR_IO, "duplicate token on line " + std::to_string(ln));
    }
    int rc = finish_table(t.get());
    if (rc != B200NN_OK) return rc;
    *out = t.release();
    return B200NN_OK;
}

extern "C" void b200nn_bpe_destroy(b200nn_bpe *t) { delete t; }
extern "C" size_t b200nn_bpe_vocab_size(const b200nn_bpe *t) { return t ? t->vocab_size : 0; }

static int copy_out(const std::vector<uint32_t> &ids, uint32_t *out, size_t capacity, size_t *n_out) {
    if (n_out) *n_out = ids.size();
    if (ids.size() > capacity) return bpe_fail(B200NN_ERR_SHAPE, "token buffer too small");
    if (out && !ids.empty()) memcpy(out, ids.data(), ids.size() * sizeof(uint32_t));
    return B200NN_OK;
}

extern "C" int32_t b200nn_bpe_encode_piece(const b200nn_bpe *t, const uint8_t *piece, size_t n, uint32_t *out,
                                           size_t capacity, size_t *n_out) {
    if (!t || (!piece && n)) return bpe_fail(B200NN_ERR_ARG, "null argument");
    std::vector<uint32_t> ids;
    merge_piece(t, piece, n, &ids);
    return copy_out(ids, out, capacity, n_out);
}

extern "C" int32_t b200nn_bpe_encode(const b200nn_bpe *t, const uint8_t *text, size_t n, uint32_t *out, size_t capacity,
                                     size_t *n_out) {
    if (!t || (!text && n)) return bpe_fail(B200NN_ERR_ARG, "null argument");
    std::vector<uint32_t> ids;
    size_t i = 0;
    const size_t sl = t->special.size();
    while (i < n) {
        // encode_with_special_tokens: the special token's text maps to its id wherever it occurs
        const void *hit = memmem(text + i, n - i, t->special.data(), sl);
        const size_t stop = hit ? (size_t)((const uint8_t *)hit - text) : n;
        while (i < stop) {
            size_t l = next_piece(text + i, stop - i);
            if (l == 0) l = 1;
            merge_piece(t, text + i, l, &ids);
            i += l;
        }
        if (hit) {
            ids.push_back(t->special_id);
            i += sl;
        }
    }
    return copy_out(ids, out, capacity, n_out);
}

extern "C" int32_t b200nn_bpe_decode(const b200nn_bpe *t, const uint32_t *ids, size_t n, uint8_t *out, size_t capacity,
                                     size_t *n_out) {
    if (!t || (!ids && n)) return bpe_fail(B200NN_ERR_ARG, "null argument");
    std::string s;
    for (size_t i = 0; i < n; ++i) {
        if (ids[i] == t->special_id) {
            s += t->special;
            continue;
        }
        if (ids[i] >= t->bytes_of.size() || t->bytes_of[ids[i]].empty())
            return bpe_fail(B200NN_ERR_DIM, "token id " + std::to_string(ids[i]) + " is not in the vocabulary");
        s += t->bytes_of[ids[i]];
    }
    if (n_out) *n_out = s.size();
    if (s.size() > capacity) return bpe_fail(B200NN_ERR_SHAPE, "text buffer too small");
    if (out && !s.empty()) memcpy(out, s.data(), s.size());
    return B200NN_OK;
}
