// Llama (SentencePiece-style, score-driven merges) tokenizer read from GGUF metadata.  Host code.
//
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

struct ib_tokenizer {
    uint32_t bos = 0, eos = 0, unk = 0;
    std::vector<std::string> vocab;
    std::vector<float> scores;
    std::unordered_map<std::string, uint32_t> index;
};

namespace {

// UTF-8 length of the character that starts with byte c (1 for a stray continuation byte: taken as a character of its own)
inline size_t utf8_len(unsigned char c) { return c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 1; }

void append_utf8(std::string &out, uint32_t cp) {
    if (cp < 0x80) out.push_back((char)cp);
    else { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }   // only U+0000..U+00FF are needed
}

}  // namespace

extern "C" {

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
