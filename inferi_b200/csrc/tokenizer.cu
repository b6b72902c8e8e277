// Tokenizers read from GGUF metadata: Llama (SentencePiece-style, score-driven merges) and GPT-2 byte-pair encoding.
// Host code.
//
// GPT-2: replaces `Gpt2Tokenizer::from_gguf`, `encode`, `decode`, `bpe` (crates/inferi/src/models/tokenizers/
// gpt2_tokenizer.rs:54-217).  The pre-tokenizer is the reference's regular expression written out as a matcher over Unicode
// classes (unicode_tables.inc); merges are applied lowest rank first to every occurrence; `decode` keeps the reference's
// byte -> U+00XX mapping.
//
// Llama:
// Replaces `LlamaTokenizer::from_gguf`, `encode` and `decode` (crates/inferi/src/models/tokenizers/llama2_tokenizer.rs:23-180),
// behaviour for behaviour, including its quirks: spaces become "▁" before anything else; a character missing from the
// vocabulary falls back to its UTF-8 bytes as ids byte + 3; "<s>" / "</s>" typed out in the text collapse to the bos / eos
// ids; the best-scoring adjacent pair is merged until none is left (first pair wins ties); `decode` maps "<0xXX>" pieces to
// the character U+00XX (not to the raw byte) and strips leading whitespace after the bos token (id 1).
// The reference panics on an empty token list (`tokens.len() - 1` underflows, :139); here that is an empty result.
#include "common.cuh"

#include <string.h>

#include <new>
#include <string>
#include <unordered_map>
#include <vector>

using namespace ib;

#include "unicode_tables.inc"

enum TokKind : int { TOK_LLAMA = 0, TOK_GPT2 = 1 };

struct ib_tokenizer {
    int kind = TOK_LLAMA;
    uint32_t bos = 0, eos = 0, unk = 0;
    std::vector<std::string> vocab;
    std::vector<float> scores;
    std::unordered_map<std::string, uint32_t> index;
    // GPT-2 byte-pair encoding: rank of a merge "first second", byte <-> printable code point
    std::unordered_map<std::string, uint32_t> merges;
    uint32_t byte_to_cp[256];
    std::unordered_map<uint32_t, uint8_t> cp_to_byte;
};

namespace {

// UTF-8 length of the character that starts with byte c (1 for a stray continuation byte: taken as a character of its own)
inline size_t utf8_len(unsigned char c) { return c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 1; }

void append_utf8(std::string &out, uint32_t cp) {
    if (cp < 0x80) out.push_back((char)cp);
    else { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }   // only U+0000..U+00FF are needed
}

bool in_ranges(const CpRange *r, size_t n, uint32_t cp) {
    size_t lo = 0, hi = n;
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        if (cp < r[mid].lo) hi = mid;
        else if (cp > r[mid].hi) lo = mid + 1;
        else return true;
    }
    return false;
}
inline bool is_letter(uint32_t cp) { return in_ranges(UNI_LETTER, sizeof(UNI_LETTER) / sizeof(CpRange), cp); }
inline bool is_number(uint32_t cp) { return in_ranges(UNI_NUMBER, sizeof(UNI_NUMBER) / sizeof(CpRange), cp); }
inline bool is_space(uint32_t cp) { return in_ranges(UNI_SPACE, sizeof(UNI_SPACE) / sizeof(CpRange), cp); }

// Decodes the UTF-8 character at s[i] (malformed bytes count as one character each); returns its length.
size_t utf8_decode(const std::string &s, size_t i, uint32_t &cp) {
    const unsigned char c = (unsigned char)s[i];
    size_t l = utf8_len(c);
    if (i + l > s.size()) l = 1;
    if (l == 1) { cp = c; return 1; }
    cp = c & (0xFF >> (l + 1));
    for (size_t k = 1; k < l; k++) cp = (cp << 6) | ((unsigned char)s[i + k] & 0x3F);
    return l;
}

void append_utf8_any(std::string &out, uint32_t cp) {
    if (cp < 0x80) out.push_back((char)cp);
    else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) { out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
    else { out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
}

// One match of the reference's pre-tokenizer expression at s[i..] (gpt2_tokenizer.rs:71-72; leftmost-first alternation):
//   's|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+
// Returns the length of the match in bytes (always > 0: every character belongs to one of the last four alternatives).
size_t pretoken_len(const std::string &s, size_t i) {
    static const char *const contractions[] = {"'s", "'t", "'re", "'ve", "'m", "'ll", "'d"};
    for (const char *c : contractions) {
        const size_t l = strlen(c);
        if (s.compare(i, l, c) == 0) return l;
    }
    auto run = [&](size_t from, int cls) {   // cls 0 letters, 1 numbers, 2 other (not space / letter / number), 3 spaces
        size_t j = from;
        while (j < s.size()) {
            uint32_t cp;
            const size_t l = utf8_decode(s, j, cp);
            const bool sp = is_space(cp), le = is_letter(cp), nu = is_number(cp);
            const bool ok = cls == 0 ? le : cls == 1 ? nu : cls == 2 ? (!sp && !le && !nu) : sp;
            if (!ok) break;
            j += l;
        }
        return j - from;
    };
    const size_t skip = s[i] == ' ' ? 1 : 0;   // the optional leading space of alternatives 2-4
    for (int cls = 0; cls < 3; cls++) {
        if (skip && i + 1 < s.size()) {
            const size_t n = run(i + 1, cls);
            if (n) return 1 + n;
        }
        const size_t n = run(i, cls);
        if (n) return n;
    }
    const size_t n = run(i, 3);
    return n ? n : 1;
}

// Byte-pair merges of one pre-token given as printable code points (gpt2_tokenizer.rs:168-217): repeatedly merge every
// occurrence of the adjacent pair with the lowest merge rank.
void bpe_merge(const ib_tokenizer *t, std::vector<std::string> &word) {
    while (word.size() > 1) {
        uint32_t best = 0xFFFFFFFFu;
        size_t best_i = 0;
        for (size_t i = 0; i + 1 < word.size(); i++) {
            auto it = t->merges.find(word[i] + " " + word[i + 1]);
            if (it != t->merges.end() && it->second < best) { best = it->second; best_i = i; }
        }
        if (best == 0xFFFFFFFFu) break;
        const std::string first = word[best_i], second = word[best_i + 1];
        std::vector<std::string> nw;
        for (size_t i = 0; i < word.size();) {
            if (word[i] == first && i + 1 < word.size() && word[i + 1] == second) { nw.push_back(first + second); i += 2; }
            else nw.push_back(word[i++]);
        }
        word.swap(nw);
    }
}

int32_t gpt2_tokenize_piece(const ib_tokenizer *t, const std::string &piece, std::vector<uint32_t> &out) {
    for (size_t i = 0; i < piece.size();) {
        const size_t l = pretoken_len(piece, i);
        std::vector<std::string> word;
        for (size_t b = 0; b < l; b++) {   // every byte as its printable stand-in (bytes_to_unicode, :21-35)
            std::string c;
            append_utf8_any(c, t->byte_to_cp[(unsigned char)piece[i + b]]);
            word.push_back(c);
        }
        bpe_merge(t, word);
        for (const std::string &w : word) {
            auto it = t->index.find(w);
            if (it != t->index.end()) out.push_back(it->second);   // pieces missing from the vocabulary are dropped (:116-118)
        }
        i += l;
    }
    return IB_OK;
}

}  // namespace

extern "C" {

int32_t ib_tokenizer_gpt2_from_gguf(ib_gguf *g, ib_tokenizer **out) {
    IB_REQUIRE(g && out, "ib_tokenizer_gpt2_from_gguf: null argument");
    *out = nullptr;
    int32_t et = 0, rc;
    uint64_t n = 0, nm = 0;
    if ((rc = ib_gguf_meta_array(g, "tokenizer.ggml.tokens", &et, &n, nullptr))) return rc;
    IB_REQUIRE(et == 8 && n > 0 && n < (1ull << 31), "tokenizer: tokenizer.ggml.tokens is not a non-empty array of strings");
    if ((rc = ib_gguf_meta_array(g, "tokenizer.ggml.merges", &et, &nm, nullptr))) return rc;
    IB_REQUIRE(et == 8, "tokenizer: tokenizer.ggml.merges is not an array of strings");
    uint64_t bos, eos;
    if ((rc = ib_gguf_meta_u64(g, "tokenizer.ggml.bos_token_id", &bos))) return rc;
    if ((rc = ib_gguf_meta_u64(g, "tokenizer.ggml.eos_token_id", &eos))) return rc;
    IB_REQUIRE(bos < n && eos < n, "tokenizer: special token ids outside the vocabulary");
    ib_tokenizer *t = new (std::nothrow) ib_tokenizer();
    if (!t) return set_error(IB_ERR_OOM, "host allocation failed");
    t->kind = TOK_GPT2;
    t->bos = (uint32_t)bos; t->eos = (uint32_t)eos; t->unk = 0;
    t->vocab.resize((size_t)n);
    std::vector<char> buf(1 << 16);
    uint64_t len = 0;
    for (uint64_t i = 0; i < n; i++) {
        if ((rc = ib_gguf_meta_array_str(g, "tokenizer.ggml.tokens", i, buf.data(), buf.size(), &len))) { delete t; return rc; }
        if (len >= buf.size()) { delete t; return set_error(IB_ERR_UNSUPPORTED, "tokenizer: token %llu is too long", (unsigned long long)i); }
        t->vocab[(size_t)i].assign(buf.data(), (size_t)len);
        t->index[t->vocab[(size_t)i]] = (uint32_t)i;
    }
    for (uint64_t i = 0; i < nm; i++) {   // "first second" -> rank (:60-68)
        if ((rc = ib_gguf_meta_array_str(g, "tokenizer.ggml.merges", i, buf.data(), buf.size(), &len))) { delete t; return rc; }
        std::string line(buf.data(), (size_t)(len < buf.size() ? len : buf.size() - 1));
        const size_t sp = line.find(' ');
        if (sp == std::string::npos || sp == 0 || sp + 1 >= line.size()) { delete t; return set_error(IB_ERR_INVALID, "tokenizer: merge %llu is not \"first second\"", (unsigned long long)i); }
        t->merges[line.substr(0, sp) + " " + line.substr(sp + 1)] = (uint32_t)i;
    }
    // bytes_to_unicode (:21-35): printable bytes stand for themselves, the others for 256, 257, ...
    uint32_t extra = 0;
    for (uint32_t b = 0; b < 256; b++) {
        const bool printable = (b >= 33 && b <= 126) || (b >= 161 && b <= 172) || (b >= 174 && b <= 255);
        t->byte_to_cp[b] = printable ? b : 256 + extra++;
        t->cp_to_byte[t->byte_to_cp[b]] = (uint8_t)b;
    }
    *out = t;
    return IB_OK;
}

int32_t ib_tokenizer_llama_from_gguf(ib_gguf *g, ib_tokenizer **out) {
    IB_REQUIRE(g && out, "ib_tokenizer_llama_from_gguf: null argument");
    *out = nullptr;
    int32_t et = 0;
    uint64_t n = 0, ns = 0;
    const void *data = nullptr;
    int32_t rc;
    if ((rc = ib_gguf_meta_array(g, "tokenizer.ggml.tokens", &et, &n, nullptr))) return rc;
    IB_REQUIRE(et == 8 && n > 0 && n < (1ull << 31), "tokenizer: tokenizer.ggml.tokens is not a non-empty array of strings");
    if ((rc = ib_gguf_meta_array(g, "tokenizer.ggml.scores", &et, &ns, &data))) return rc;
    IB_REQUIRE(et == 6 && ns == n, "tokenizer: tokenizer.ggml.scores must hold one f32 per token");
    uint64_t bos, eos, unk;
    if ((rc = ib_gguf_meta_u64(g, "tokenizer.ggml.bos_token_id", &bos))) return rc;
    if ((rc = ib_gguf_meta_u64(g, "tokenizer.ggml.eos_token_id", &eos))) return rc;
    if ((rc = ib_gguf_meta_u64(g, "tokenizer.ggml.unknown_token_id", &unk))) return rc;
    IB_REQUIRE(bos < n && eos < n && unk < n, "tokenizer: special token ids outside the vocabulary");
    ib_tokenizer *t = new (std::nothrow) ib_tokenizer();
    if (!t) return set_error(IB_ERR_OOM, "host allocation failed");
    t->bos = (uint32_t)bos; t->eos = (uint32_t)eos; t->unk = (uint32_t)unk;
    t->vocab.resize((size_t)n);
    t->scores.resize((size_t)n);
    memcpy(t->scores.data(), data, (size_t)n * sizeof(float));
    std::vector<char> buf(1 << 16);
    for (uint64_t i = 0; i < n; i++) {
        uint64_t len = 0;
        if ((rc = ib_gguf_meta_array_str(g, "tokenizer.ggml.tokens", i, buf.data(), buf.size(), &len))) { delete t; return rc; }
        if (len >= buf.size()) { delete t; return set_error(IB_ERR_UNSUPPORTED, "tokenizer: token %llu is longer than %zu bytes", (unsigned long long)i, buf.size() - 1); }
        t->vocab[(size_t)i].assign(buf.data(), (size_t)len);
        t->index[t->vocab[(size_t)i]] = (uint32_t)i;   // a later duplicate replaces an earlier one, as HashMap::insert does (:40-42)
    }
    *out = t;
    return IB_OK;
}

int32_t ib_tokenizer_destroy(ib_tokenizer *t) {
    delete t;
    return IB_OK;
}

int32_t ib_tokenizer_info(const ib_tokenizer *t, uint32_t *vocab_size, uint32_t *bos, uint32_t *eos, uint32_t *unk) {
    IB_REQUIRE(t, "ib_tokenizer_info: null tokenizer");
    if (vocab_size) *vocab_size = (uint32_t)t->vocab.size();
    if (bos) *bos = t->bos;
    if (eos) *eos = t->eos;
    if (unk) *unk = t->unk;
    return IB_OK;
}

int32_t ib_tokenizer_encode(const ib_tokenizer *t, const char *text, uint64_t text_len, int32_t add_bos, int32_t add_eos, uint32_t *out, uint64_t cap,
                            uint64_t *n_out) {
    IB_REQUIRE(t && text && n_out, "ib_tokenizer_encode: null argument");
    if (t->kind == TOK_GPT2) {
        // gpt2_tokenizer.rs:106-143: "<...>" stretches are special tokens looked up whole, the rest is pre-tokenized and merged.
        // (add_bos / add_eos: the reference's encode adds neither; honoured here as a convenience.)
        const std::string s(text, (size_t)text_len);
        std::vector<uint32_t> tok;
        if (add_bos) tok.push_back(t->bos);
        size_t cursor = 0, i = 0;
        while (i < s.size()) {
            if (s[i] == '<') {
                size_t j = i + 1;
                while (j < s.size() && s[j] != '<' && s[j] != '>') j++;
                if (j < s.size() && s[j] == '>') {
                    if (cursor != i) gpt2_tokenize_piece(t, s.substr(cursor, i - cursor), tok);
                    auto it = t->index.find(s.substr(i, j + 1 - i));
                    if (it == t->index.end())   // the reference panics here (:134)
                        return set_error(IB_ERR_INVALID, "tokenizer: special token %s is not in the vocabulary", s.substr(i, j + 1 - i).c_str());
                    tok.push_back(it->second);
                    i = cursor = j + 1;
                    continue;
                }
            }
            i++;
        }
        if (cursor < s.size()) gpt2_tokenize_piece(t, s.substr(cursor), tok);
        if (add_eos) tok.push_back(t->eos);
        *n_out = tok.size();
        if (out) {
            IB_REQUIRE(cap >= tok.size(), "ib_tokenizer_encode: %zu tokens do not fit the buffer of %llu", tok.size(), (unsigned long long)cap);
            memcpy(out, tok.data(), tok.size() * sizeof(uint32_t));
        }
        return IB_OK;
    }
    const size_t V = t->vocab.size();
    // " " -> "▁" (:77)
    std::string s;
    s.reserve((size_t)text_len * 2);
    for (uint64_t i = 0; i < text_len; i++) {
        if (text[i] == ' ') s += "\xE2\x96\x81";
        else s.push_back(text[i]);
    }
    std::vector<uint32_t> tok;
    if (add_bos) tok.push_back(t->bos);
    // one token per character, bytes + 3 for characters the vocabulary lacks (:84-97)
    for (size_t i = 0; i < s.size();) {
        size_t l = utf8_len((unsigned char)s[i]);
        if (i + l > s.size()) l = 1;
        auto it = t->index.find(s.substr(i, l));
        if (it != t->index.end()) tok.push_back(it->second);
        else
            for (size_t b = 0; b < l; b++) tok.push_back((uint32_t)(unsigned char)s[i + b] + 3);
        i += l;
    }
    for (uint32_t id : tok)
        if (id >= V) return set_error(IB_ERR_INVALID, "tokenizer: byte fallback id %u outside the vocabulary of %zu", id, V);
    // "<s>" and "</s>" typed out in the text (:100-134)
    for (size_t i = 0; i + 2 < tok.size(); i++)
        if (t->vocab[tok[i]] + t->vocab[tok[i + 1]] + t->vocab[tok[i + 2]] == "<s>") {
            tok[i] = t->bos;
            tok.erase(tok.begin() + i + 1, tok.begin() + i + 3);
        }
    for (size_t i = 0; i + 3 < tok.size(); i++)
        if (t->vocab[tok[i]] + t->vocab[tok[i + 1]] + t->vocab[tok[i + 2]] + t->vocab[tok[i + 3]] == "</s>") {
            tok[i] = t->eos;
            tok.erase(tok.begin() + i + 1, tok.begin() + i + 4);
        }
    // merge the best-scoring adjacent pair until no pair is in the vocabulary (:137-161)
    while (tok.size() >= 2) {
        float best_score = -INFINITY;
        uint32_t best_id = 0;
        size_t best_idx = (size_t)-1;
        for (size_t i = 0; i + 1 < tok.size(); i++) {
            auto it = t->index.find(t->vocab[tok[i]] + t->vocab[tok[i + 1]]);
            if (it != t->index.end() && t->scores[it->second] > best_score) {
                best_score = t->scores[it->second];
                best_id = it->second;
                best_idx = i;
            }
        }
        if (best_idx == (size_t)-1) break;
        tok[best_idx] = best_id;
        tok.erase(tok.begin() + best_idx + 1);
    }
    if (add_eos) tok.push_back(t->eos);
    *n_out = tok.size();
    if (out) {
        IB_REQUIRE(cap >= tok.size(), "ib_tokenizer_encode: %zu tokens do not fit the buffer of %llu", tok.size(), (unsigned long long)cap);
        memcpy(out, tok.data(), tok.size() * sizeof(uint32_t));
    }
    return IB_OK;
}

int32_t ib_tokenizer_decode(const ib_tokenizer *t, uint32_t prev_token, uint32_t token, char *out, uint64_t cap, uint64_t *len) {
    IB_REQUIRE(t && len, "ib_tokenizer_decode: null argument");
    IB_REQUIRE(token < t->vocab.size(), "ib_tokenizer_decode: token %u outside the vocabulary", token);
    if (t->kind == TOK_GPT2) {
        // gpt2_tokenizer.rs:152-166: printable stand-ins back to bytes; every byte then becomes the character U+00XX (the
        // reference does `b as char`, it does not reassemble multi-byte UTF-8), characters without a byte are dropped
        std::string res;
        const std::string &piece = t->vocab[token];
        for (size_t i = 0; i < piece.size();) {
            uint32_t cp;
            i += utf8_decode(piece, i, cp);
            auto it = t->cp_to_byte.find(cp);
            if (it != t->cp_to_byte.end()) append_utf8(res, it->second);
        }
        *len = res.size();
        if (out && cap) {
            const size_t n = res.size() < cap - 1 ? res.size() : (size_t)cap - 1;
            memcpy(out, res.data(), n);
            out[n] = 0;
        }
        return IB_OK;
    }
    std::string piece = t->vocab[token];
    if (prev_token == 1) {   // after the bos token: strip leading whitespace (:166-168; ASCII whitespace here)
        size_t k = 0;
        while (k < piece.size() && (piece[k] == ' ' || piece[k] == '\t' || piece[k] == '\n' || piece[k] == '\r' || piece[k] == '\v' || piece[k] == '\f')) k++;
        piece.erase(0, k);
    }
    std::string res;
    bool done = false;
    if (piece.rfind("<0x", 0) == 0 && piece.size() >= 5) {   // "<0xXX>": the character U+00XX (:169-173)
        auto hexv = [](char c) { return c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : -1; };
        const int h = hexv(piece[3]), l = hexv(piece[4]);
        if (h >= 0 && l >= 0) { append_utf8(res, (uint32_t)(h * 16 + l)); done = true; }
    }
    if (!done) {   // "▁" -> " " (:174)
        for (size_t i = 0; i < piece.size();) {
            if (piece.compare(i, 3, "\xE2\x96\x81") == 0) { res.push_back(' '); i += 3; }
            else res.push_back(piece[i++]);
        }
    }
    *len = res.size();
    if (out && cap) {
        const size_t n = res.size() < cap - 1 ? res.size() : (size_t)cap - 1;
        memcpy(out, res.data(), n);
        out[n] = 0;
    }
    return IB_OK;
}

}  // extern "C"
