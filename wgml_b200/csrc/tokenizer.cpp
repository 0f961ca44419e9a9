// Tokenizers and the default chat template: the host-side text layer either side of the token loop.
//
//   LlamaTokenizer  crates/wgml/src/models/llama2/tokenizer.rs:8-180  SentencePiece-style: characters (or byte
//                   fallback), the special-token scans, then greedy merging of the best-scoring adjacent pair
//   Gpt2Tokenizer   crates/wgml/src/models/gpt2/tokenizer.rs:38-217   byte-level BPE over a pre-split by the GPT-2
//                   pattern, with `<...>` spans looked up as special tokens
//   chat template   crates/wgml-chat/src/chat_template.rs:10-40 + models/llama2/llama-2-chat.jinja
//
// All three work on what the GGUF metadata holds (tokenizer.ggml.tokens / scores / merges / *_token_id); no
// vocabulary is built in.  Pure host code: nothing here touches a device.
#include "common.cuh"

#include <wctype.h>
#include <locale.h>

#include <climits>
#include <cmath>
#include <map>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

using namespace wgb;

namespace {

// ---- UTF-8 helpers ---------------------------------------------------------------------------------------
// Next code point of s at i (advances i); malformed bytes come out as themselves, one at a time.
uint32_t next_cp(const std::string &s, size_t &i)
{
    const unsigned char c = (unsigned char)s[i];
    auto cont = [&](size_t k) { return i + k < s.size() && ((unsigned char)s[i + k] & 0xC0) == 0x80; };
    if (c < 0x80) { i += 1; return c; }
    if ((c >> 5) == 6 && cont(1)) { uint32_t v = ((c & 0x1Fu) << 6) | ((unsigned char)s[i + 1] & 0x3Fu); i += 2; return v; }
    if ((c >> 4) == 14 && cont(1) && cont(2)) {
        uint32_t v = ((c & 0x0Fu) << 12) | (((unsigned char)s[i + 1] & 0x3Fu) << 6) | ((unsigned char)s[i + 2] & 0x3Fu);
        i += 3;
        return v;
    }
    if ((c >> 3) == 30 && cont(1) && cont(2) && cont(3)) {
        uint32_t v = ((c & 0x07u) << 18) | (((unsigned char)s[i + 1] & 0x3Fu) << 12) | (((unsigned char)s[i + 2] & 0x3Fu) << 6) |
                     ((unsigned char)s[i + 3] & 0x3Fu);
        i += 4;
        return v;
    }
    i += 1;
    return c;
}

void put_cp(std::string &out, uint32_t cp)
{
    if (cp < 0x80) out.push_back((char)cp);
    else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) {
        out.push_back((char)(0xE0 | (cp >> 12)));
        out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
        out.push_back((char)(0x80 | (cp & 0x3F)));
    } else {
        out.push_back((char)(0xF0 | (cp >> 18)));
        out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
        out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
        out.push_back((char)(0x80 | (cp & 0x3F)));
    }
}

// Splits into the UTF-8 encodings of its characters.
std::vector<std::string> chars_of(const std::string &s)
{
    std::vector<std::string> out;
    for (size_t i = 0; i < s.size();) {
        const size_t b = i;
        next_cp(s, i);
        out.push_back(s.substr(b, i - b));
    }
    return out;
}

// Character classes of the GPT-2 pattern (\p{L}, \p{N}, \s).  ASCII is exact; beyond it the C library's UTF-8
// tables stand in for the Unicode general categories (letters: iswalpha; numbers: alphanumeric but not
// alphabetic, which covers the decimal digits of other scripts but not every \p{No} symbol).
locale_t utf8_locale()
{
    static locale_t loc = newlocale(LC_CTYPE_MASK, "C.UTF-8", (locale_t)0);
    return loc;
}
bool is_letter(uint32_t cp)
{
    if (cp < 0x80) return (cp >= 'a' && cp <= 'z') || (cp >= 'A' && cp <= 'Z');
    locale_t l = utf8_locale();
    return l ? iswalpha_l((wint_t)cp, l) != 0 : true;
}
bool is_number(uint32_t cp)
{
    if (cp < 0x80) return cp >= '0' && cp <= '9';
    locale_t l = utf8_locale();
    return l ? (iswalnum_l((wint_t)cp, l) != 0 && iswalpha_l((wint_t)cp, l) == 0) : false;
}
bool is_space(uint32_t cp)
{
    if (cp < 0x80) return cp == ' ' || (cp >= 9 && cp <= 13);
    return cp == 0x85 || cp == 0xA0 || cp == 0x1680 || (cp >= 0x2000 && cp <= 0x200A) || cp == 0x2028 || cp == 0x2029 ||
           cp == 0x202F || cp == 0x205F || cp == 0x3000;
}

int load_strings(const wgb_gguf *g, const char *key, std::vector<std::string> &out)
{
    const int64_t i = wgb_gguf_meta_find(g, key);
    if (i < 0) return fail(WGB_ERR_NOT_FOUND, "missing GGUF key '%s'", key);
    int type = 0, elem = 0;
    uint64_t len = 0;
    wgb_gguf_meta_type(g, (uint64_t)i, &type, &elem, &len);
    if (type != WGB_META_ARRAY || elem != WGB_META_STRING) return fail(WGB_ERR_INVALID, "GGUF key '%s' is not a string array", key);
    out.resize(len);
    for (uint64_t k = 0; k < len; k++) {
        const char *p = nullptr;
        uint64_t n = 0;
        const int rc = wgb_gguf_meta_arr_str(g, (uint64_t)i, k, &p, &n);
        if (rc) return rc;
        out[k].assign(p, n);
    }
    return WGB_OK;
}

int load_u32(const wgb_gguf *g, const char *key, uint32_t *out)
{
    const int64_t i = wgb_gguf_meta_find(g, key);
    if (i < 0) return fail(WGB_ERR_NOT_FOUND, "missing GGUF key '%s'", key);
    int type = 0;
    wgb_gguf_meta_type(g, (uint64_t)i, &type, nullptr, nullptr);
    if (type != WGB_META_U32) return fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type for '%s'.", key);
    uint64_t v = 0;
    wgb_gguf_meta_u64(g, (uint64_t)i, &v);
    *out = (uint32_t)v;
    return WGB_OK;
}

int copy_out(const std::string &s, char *buf, size_t cap, size_t *len)
{
    if (len) *len = s.size();
    if (!buf) return WGB_OK;   // size query
    if (cap < s.size() + 1) return fail(WGB_ERR_INVALID, "text of %zu bytes does not fit a buffer of %zu", s.size() + 1, cap);
    memcpy(buf, s.data(), s.size());
    buf[s.size()] = 0;
    return WGB_OK;
}

int copy_ids(const std::vector<uint32_t> &ids, uint32_t *out, size_t cap, size_t *n)
{
    if (n) *n = ids.size();
    if (!out) return WGB_OK;   // size query
    if (cap < ids.size()) return fail(WGB_ERR_INVALID, "%zu token ids do not fit a buffer of %zu", ids.size(), cap);
    if (!ids.empty()) memcpy(out, ids.data(), ids.size() * sizeof(uint32_t));
    return WGB_OK;
}

}  // namespace

// ---- LlamaTokenizer -----------------------------------------------------------------------------------
struct wgb_llama_tokenizer {
    uint32_t bos = 0, eos = 0, unk = 0;
    std::vector<std::string> vocab;
    std::vector<float> scores;
    std::unordered_map<std::string, uint32_t> index;
};

WGB_EXPORT int wgb_llama_tokenizer_from_gguf(const wgb_gguf *g, wgb_llama_tokenizer **out)
{
    WGB_REQUIRE(g && out, "null argument");
    wgb_llama_tokenizer *t = new (std::nothrow) wgb_llama_tokenizer();
    if (!t) return fail(WGB_ERR_INVALID, "out of host memory");
    int rc = load_strings(g, "tokenizer.ggml.tokens", t->vocab);
    if (!rc) {
        const int64_t i = wgb_gguf_meta_find(g, "tokenizer.ggml.scores");
        int type = 0, elem = 0;
        uint64_t len = 0;
        if (i < 0) rc = fail(WGB_ERR_NOT_FOUND, "missing GGUF key 'tokenizer.ggml.scores'");
        else {
            wgb_gguf_meta_type(g, (uint64_t)i, &type, &elem, &len);
            if (type != WGB_META_ARRAY || elem != WGB_META_F32) rc = fail(WGB_ERR_INVALID, "GGUF key 'tokenizer.ggml.scores' is not an f32 array");
            else if (len != t->vocab.size()) rc = fail(WGB_ERR_INVALID, "%llu scores for %zu tokens", (unsigned long long)len, t->vocab.size());
            else {
                t->scores.resize(len);
                for (uint64_t k = 0; k < len && !rc; k++) {
                    double d = 0;
                    rc = wgb_gguf_meta_arr_f64(g, (uint64_t)i, k, &d);
                    t->scores[k] = (float)d;
                }
            }
        }
    }
    if (!rc) rc = load_u32(g, "tokenizer.ggml.bos_token_id", &t->bos);
    if (!rc) rc = load_u32(g, "tokenizer.ggml.eos_token_id", &t->eos);
    if (!rc) rc = load_u32(g, "tokenizer.ggml.unknown_token_id", &t->unk);
    if (!rc && (t->bos >= t->vocab.size() || t->eos >= t->vocab.size() || t->unk >= t->vocab.size()))
        rc = fail(WGB_ERR_INVALID, "special token id outside a vocabulary of %zu", t->vocab.size());
    if (rc) { delete t; return rc; }
    // a later duplicate replaces an earlier one, as HashMap::insert does (tokenizer.rs:38-41)
    for (uint32_t n = 0; n < t->vocab.size(); n++) t->index[t->vocab[n]] = n;
    *out = t;
    return WGB_OK;
}

WGB_EXPORT int wgb_llama_tokenizer_destroy(wgb_llama_tokenizer *t) { delete t; return WGB_OK; }
WGB_EXPORT uint32_t wgb_llama_tokenizer_bos(const wgb_llama_tokenizer *t) { return t ? t->bos : 0; }
WGB_EXPORT uint32_t wgb_llama_tokenizer_eos(const wgb_llama_tokenizer *t) { return t ? t->eos : 0; }
WGB_EXPORT uint32_t wgb_llama_tokenizer_unk(const wgb_llama_tokenizer *t) { return t ? t->unk : 0; }
WGB_EXPORT size_t wgb_llama_tokenizer_vocab_size(const wgb_llama_tokenizer *t) { return t ? t->vocab.size() : 0; }

// LlamaTokenizer::encode, tokenizer.rs:75-164.
WGB_EXPORT int wgb_llama_tokenizer_encode(const wgb_llama_tokenizer *t, const char *text, size_t text_len, int bos, int eos,
                                          uint32_t *out_ids, size_t cap, size_t *n_out)
{
    WGB_REQUIRE(t && (text || text_len == 0), "null argument");
    std::string s;
    {   // text.replace(" ", "▁")
        const std::string in(text ? text : "", text_len);
        for (char c : in) {
            if (c == ' ') s += "\xE2\x96\x81";
            else s.push_back(c);
        }
    }
    std::vector<uint32_t> tok;
    if (bos) tok.push_back(t->bos);
    for (const std::string &ch : chars_of(s)) {
        auto it = t->index.find(ch);
        if (it != t->index.end()) tok.push_back(it->second);
        else
            for (unsigned char b : ch) tok.push_back((uint32_t)b + 3);   // byte fallback: bytes start after <unk>, <s>, </s>
    }
    for (uint32_t id : tok)
        if (id >= t->vocab.size()) return fail(WGB_ERR_INVALID, "byte-fallback id %u outside a vocabulary of %zu", id, t->vocab.size());
    auto piece = [&](size_t i) -> const std::string & { return t->vocab[tok[i]]; };
    // special tokens spelled out character by character: "<s>" (3 pieces) and "</s>" (4 pieces)
    for (size_t i = 0; i + 2 < tok.size(); i++) {
        if (piece(i) + piece(i + 1) + piece(i + 2) == "<s>") {
            tok[i] = t->bos;
            tok.erase(tok.begin() + (long)i + 1, tok.begin() + (long)i + 3);
        }
    }
    for (size_t i = 0; i + 3 < tok.size(); i++) {
        if (piece(i) + piece(i + 1) + piece(i + 2) + piece(i + 3) == "</s>") {
            tok[i] = t->eos;
            tok.erase(tok.begin() + (long)i + 1, tok.begin() + (long)i + 4);
        }
    }
    // merge the best-scoring adjacent pair until none is in the vocabulary (the first of equal scores wins)
    while (tok.size() >= 2) {
        float best_score = -INFINITY;
        uint32_t best_id = 0;
        long best_idx = -1;
        for (size_t i = 0; i + 1 < tok.size(); i++) {
            auto it = t->index.find(piece(i) + piece(i + 1));
            if (it != t->index.end() && t->scores[it->second] > best_score) {
                best_score = t->scores[it->second];
                best_id = it->second;
                best_idx = (long)i;
            }
        }
        if (best_idx < 0) break;
        tok[(size_t)best_idx] = best_id;
        tok.erase(tok.begin() + best_idx + 1);
    }
    if (eos) tok.push_back(t->eos);
    return copy_ids(tok, out_ids, cap, n_out);
}

// LlamaTokenizer::decode, tokenizer.rs:166-177: the text of one token given its predecessor.
WGB_EXPORT int wgb_llama_tokenizer_decode(const wgb_llama_tokenizer *t, uint32_t prev_token, uint32_t token, char *buf, size_t cap,
                                          size_t *len)
{
    WGB_REQUIRE(t, "null argument");
    WGB_REQUIRE(token < t->vocab.size(), "token %u outside a vocabulary of %zu", token, t->vocab.size());
    std::string piece = t->vocab[token];
    if (prev_token == 1) {   // trim_start: leading Unicode white space
        size_t i = 0;
        while (i < piece.size()) {
            size_t j = i;
            if (!is_space(next_cp(piece, j))) break;
            i = j;
        }
        piece = piece.substr(i);
    }
    if (piece.size() >= 5 && piece.compare(0, 3, "<0x") == 0) {
        auto hex = [](char c) { return c >= '0' && c <= '9' ? c - '0' : (c >= 'a' && c <= 'f' ? c - 'a' + 10 : (c >= 'A' && c <= 'F' ? c - 'A' + 10 : -1)); };
        const int hi = hex(piece[3]), lo = hex(piece[4]);
        if (hi >= 0 && lo >= 0) {
            std::string out;
            put_cp(out, (uint32_t)(hi * 16 + lo));   // `i as u8 as char`: the byte value as a code point
            return copy_out(out, buf, cap, len);
        }
    }
    std::string out;
    for (size_t i = 0; i < piece.size();) {
        if (piece.compare(i, 3, "\xE2\x96\x81") == 0) { out.push_back(' '); i += 3; }
        else out.push_back(piece[i++]);
    }
    return copy_out(out, buf, cap, len);
}

// ---- Gpt2Tokenizer ------------------------------------------------------------------------------------
struct wgb_gpt2_tokenizer {
    uint32_t bos = 0, eos = 0;
    std::vector<std::string> vocab;
    std::unordered_map<std::string, uint32_t> encoder;
    std::map<std::pair<std::string, std::string>, size_t> merges;
    uint32_t byte_to_cp[256];
    std::unordered_map<uint32_t, uint8_t> cp_to_byte;
};

namespace {

// bytes_to_unicode, gpt2/tokenizer.rs:22-36
void build_byte_map(wgb_gpt2_tokenizer *t)
{
    bool kept[256] = {};
    for (int b = 33; b <= 126; b++) kept[b] = true;
    for (int b = 161; b <= 172; b++) kept[b] = true;
    for (int b = 174; b <= 255; b++) kept[b] = true;
    uint32_t n = 0;
    for (int b = 0; b < 256; b++) {
        t->byte_to_cp[b] = kept[b] ? (uint32_t)b : 256 + n++;
        t->cp_to_byte[t->byte_to_cp[b]] = (uint8_t)b;
    }
}

// Gpt2Tokenizer::bpe, gpt2/tokenizer.rs:170-216.  Returns the merged symbols.
std::vector<std::string> bpe(const wgb_gpt2_tokenizer *t, const std::string &token)
{
    std::vector<std::string> word = chars_of(token);
    if (word.size() < 2) return word;
    for (;;) {
        // the adjacent pair with the lowest merge rank (pairs unknown to the table rank last)
        size_t best_rank = SIZE_MAX;
        std::pair<std::string, std::string> best;
        for (size_t i = 0; i + 1 < word.size(); i++) {
            auto it = t->merges.find({ word[i], word[i + 1] });
            if (it != t->merges.end() && it->second < best_rank) {
                best_rank = it->second;
                best = it->first;
            }
        }
        if (best_rank == SIZE_MAX) break;
        std::vector<std::string> merged;
        for (size_t i = 0; i < word.size();) {
            if (i + 1 < word.size() && word[i] == best.first && word[i + 1] == best.second) {
                merged.push_back(best.first + best.second);
                i += 2;
            } else {
                merged.push_back(word[i]);
                i += 1;
            }
        }
        word.swap(merged);
        if (word.size() == 1) break;
    }
    return word;
}

// One match of 's|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+ at byte offset i (leftmost
// alternative that matches, as the regex crate's leftmost-first semantics); returns the end offset, or i when
// nothing matches (cannot happen: the alternatives cover every character).
size_t match_piece(const std::string &s, size_t i)
{
    static const char *contr[] = { "'s", "'t", "'re", "'ve", "'m", "'ll", "'d" };
    for (const char *c : contr) {
        const size_t n = strlen(c);
        if (s.compare(i, n, c) == 0) return i + n;
    }
    auto run = [&](size_t from, bool (*cls)(uint32_t)) {
        size_t j = from;
        while (j < s.size()) {
            size_t k = j;
            if (!cls(next_cp(s, k))) break;
            j = k;
        }
        return j;
    };
    auto other = [](uint32_t cp) { return !is_space(cp) && !is_letter(cp) && !is_number(cp); };
    const size_t after_sp = (i < s.size() && s[i] == ' ') ? i + 1 : i;
    size_t e;
    if ((e = run(after_sp, is_letter)) > after_sp) return e;
    if ((e = run(after_sp, is_number)) > after_sp) return e;
    if ((e = run(after_sp, other)) > after_sp) return e;
    if ((e = run(i, is_space)) > i) return e;
    return i;
}

}  // namespace

WGB_EXPORT int wgb_gpt2_tokenizer_from_gguf(const wgb_gguf *g, wgb_gpt2_tokenizer **out)
{
    WGB_REQUIRE(g && out, "null argument");
    wgb_gpt2_tokenizer *t = new (std::nothrow) wgb_gpt2_tokenizer();
    if (!t) return fail(WGB_ERR_INVALID, "out of host memory");
    std::vector<std::string> lines;
    int rc = load_strings(g, "tokenizer.ggml.tokens", t->vocab);
    if (!rc) rc = load_strings(g, "tokenizer.ggml.merges", lines);
    if (!rc) rc = load_u32(g, "tokenizer.ggml.bos_token_id", &t->bos);
    if (!rc) rc = load_u32(g, "tokenizer.ggml.eos_token_id", &t->eos);
    for (size_t i = 0; i < lines.size() && !rc; i++) {
        // `line.split_whitespace()`: the first two fields
        std::vector<std::string> parts;
        std::string cur;
        for (size_t k = 0; k <= lines[i].size(); k++) {
            size_t k2 = k;
            const bool end = k == lines[i].size();
            const uint32_t cp = end ? ' ' : next_cp(lines[i], k2);
            if (end || is_space(cp)) {
                if (!cur.empty()) parts.push_back(cur);
                cur.clear();
            } else {
                cur.append(lines[i], k, k2 - k);
            }
            if (!end) k = k2 - 1;
        }
        if (parts.size() < 2) rc = fail(WGB_ERR_INVALID, "merge rule %zu has fewer than two fields", i);
        else t->merges[{ parts[0], parts[1] }] = i;   // a repeated pair keeps its last rank (HashMap::insert)
    }
    if (rc) { delete t; return rc; }
    for (uint32_t i = 0; i < t->vocab.size(); i++) t->encoder[t->vocab[i]] = i;
    build_byte_map(t);
    *out = t;
    return WGB_OK;
}

WGB_EXPORT int wgb_gpt2_tokenizer_destroy(wgb_gpt2_tokenizer *t) { delete t; return WGB_OK; }
WGB_EXPORT uint32_t wgb_gpt2_tokenizer_bos(const wgb_gpt2_tokenizer *t) { return t ? t->bos : 0; }
WGB_EXPORT uint32_t wgb_gpt2_tokenizer_eos(const wgb_gpt2_tokenizer *t) { return t ? t->eos : 0; }

// Gpt2Tokenizer::encode, gpt2/tokenizer.rs:108-146.
WGB_EXPORT int wgb_gpt2_tokenizer_encode(const wgb_gpt2_tokenizer *t, const char *text, size_t text_len, uint32_t *out_ids,
                                         size_t cap, size_t *n_out)
{
    WGB_REQUIRE(t && (text || text_len == 0), "null argument");
    const std::string s(text ? text : "", text_len);
    std::vector<uint32_t> ids;
    auto tokenize = [&](const std::string &sub) {
        for (size_t i = 0; i < sub.size();) {
            size_t e = match_piece(sub, i);
            if (e == i) { size_t k = i; next_cp(sub, k); e = k; }
            std::string mapped;
            for (size_t b = i; b < e; b++) put_cp(mapped, t->byte_to_cp[(unsigned char)sub[b]]);
            for (const std::string &sym : bpe(t, mapped)) {
                auto it = t->encoder.find(sym);
                if (it != t->encoder.end()) ids.push_back(it->second);   // symbols missing from the vocabulary are dropped
            }
            i = e;
        }
    };
    // spans "<...>" without nested angle brackets are special tokens, looked up as they are
    size_t cursor = 0;
    for (size_t i = 0; i < s.size(); i++) {
        if (s[i] != '<') continue;
        size_t j = i + 1;
        while (j < s.size() && s[j] != '<' && s[j] != '>') j++;
        if (j >= s.size() || s[j] != '>') continue;
        if (cursor != i) tokenize(s.substr(cursor, i - cursor));
        const std::string special = s.substr(i, j + 1 - i);
        auto it = t->encoder.find(special);
        if (it == t->encoder.end()) return fail(WGB_ERR_NOT_FOUND, "special token '%s' is not in the vocabulary", special.c_str());
        ids.push_back(it->second);
        cursor = j + 1;
        i = j;
    }
    if (cursor < s.size()) tokenize(s.substr(cursor));
    return copy_ids(ids, out_ids, cap, n_out);
}

// Gpt2Tokenizer::decode, gpt2/tokenizer.rs:156-168: unknown ids and unmapped characters are skipped; every
// mapped byte becomes the character of that value (`b as char`).
WGB_EXPORT int wgb_gpt2_tokenizer_decode(const wgb_gpt2_tokenizer *t, const uint32_t *tokens, size_t n, char *buf, size_t cap, size_t *len)
{
    WGB_REQUIRE(t && (tokens || n == 0), "null argument");
    std::string joined;
    for (size_t i = 0; i < n; i++)
        if (tokens[i] < t->vocab.size()) joined += t->vocab[tokens[i]];
    std::string out;
    for (size_t i = 0; i < joined.size();) {
        const uint32_t cp = next_cp(joined, i);
        auto it = t->cp_to_byte.find(cp);
        if (it != t->cp_to_byte.end()) put_cp(out, it->second);
    }
    return copy_out(out, buf, cap, len);
}

// ---- chat template ---------------------------------------------------------------------------------------
namespace {

std::string trim(const std::string &s)
{
    size_t b = 0, e = s.size();
    while (b < e) {
        size_t k = b;
        if (!is_space(next_cp(s, k))) break;
        b = k;
    }
    while (e > b) {
        // step back one code point
        size_t k = e - 1;
        while (k > b && ((unsigned char)s[k] & 0xC0) == 0x80) k--;
        size_t k2 = k;
        if (!is_space(next_cp(s, k2))) break;
        e = k;
    }
    return s.substr(b, e - b);
}

}  // namespace

// ChatTemplate::apply (crates/wgml-chat/src/chat_template.rs:27-39) for the default template,
// LlamaTokenizer::CHAT_TEMPLATE = llama-2-chat.jinja, rendered as the reference configures minijinja:
// trim_blocks on (the newline after a block tag is dropped), lstrip_blocks off (the indentation in front of a
// tag stays), add_generation_prompt unused by this template.  The white space between the tags is therefore
// part of the output and is reproduced here: a message renders as
//     "    \n" + 16 spaces + "\n" + 12 spaces + TEXT + "\n    "
// after a preamble of 8 spaces (a system message was folded into the first user message) or 4 spaces, and one
// "\n".  TEXT is bos + "[INST] " + trim(content) + " [/INST]" for a user message and
// " " + trim(content) + " " + eos for an assistant message.  Templates carried by a GGUF
// (`tokenizer.chat_template`) are arbitrary Jinja and are not interpreted: callers render those themselves.
WGB_EXPORT int wgb_chat_template_llama2(const char *const *roles, const char *const *contents, size_t n_messages, const char *bos,
                                        const char *eos, char *buf, size_t cap, size_t *len)
{
    WGB_REQUIRE(roles && contents && bos && eos && n_messages > 0, "null or empty conversation");
    for (size_t i = 0; i < n_messages; i++) WGB_REQUIRE(roles[i] && contents[i], "message %zu: null role or content", i);
    std::string out, system_message;
    size_t first = 0;
    if (std::string(roles[0]) == "system") {
        system_message = "<<SYS>>\n" + trim(contents[0]) + "\n<</SYS>>\n\n";
        first = 1;
        out += "        ";
    } else {
        out += "    ";
    }
    out += "\n";
    for (size_t i = first; i < n_messages; i++) {
        const size_t index0 = i - first;
        const std::string role = roles[i];
        if ((role == "user") != (index0 % 2 == 0))
            return fail(WGB_ERR_INVALID, "Conversation roles must alternate user/assistant/user/assistant/...");
        const std::string content = index0 == 0 ? system_message + contents[i] : std::string(contents[i]);
        out += "    \n";
        out += "                \n";
        out += "    ";
        if (role == "user") out += "        " + std::string(bos) + "[INST] " + trim(content) + " [/INST]" + "\n    ";
        else if (role == "assistant") out += "        " + std::string(" ") + trim(content) + " " + eos + "\n    ";
    }
    return copy_out(out, buf, cap, len);
}
