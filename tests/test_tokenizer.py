"""Llama tokenizer from GGUF metadata against an independent Python restatement of the reference's algorithm
(crates/inferi/src/models/tokenizers/llama2_tokenizer.rs:76-180).  Host code only: no GPU."""
import numpy as np
import pytest

from inferi_b200 import gguf as G

SP = "▁"


def make_vocab():
    """A small SentencePiece-like vocabulary: <unk>, <s>, </s>, the 256 byte pieces, characters, and merged pieces with scores."""
    vocab = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)]
    scores = [0.0] * len(vocab)
    chars = list("abcdefghijklmnopqrstuvwxyz<>/s.,!é") + [SP]
    for c in dict.fromkeys(chars):
        vocab.append(c)
        scores.append(-100.0)
    rng = np.random.default_rng(3)
    words = ["he", "ll", "hell", "hello", "lo", SP + "w", "or", "ld", SP + "wor", SP + "world", "th", "the", SP + "the", "er", "re", "ér", SP + "a",
             "ab", "abc", "bc", SP + SP, "ss", "s>", "<s", "</", "</s"]
    for i, w in enumerate(words):
        vocab.append(w)
        scores.append(float(-1.0 - rng.random() * 5 - 0.01 * i))
    return vocab, scores


def py_encode(vocab, scores, text, bos, eos, bos_id=1, eos_id=2):
    index = {}
    for i, v in enumerate(vocab):
        index[v] = i
    text = text.replace(" ", SP)
    tok = [bos_id] if bos else []
    for ch in text:
        if ch in index:
            tok.append(index[ch])
        else:
            tok.extend(b + 3 for b in ch.encode("utf-8"))
    i = 0
    while i < max(0, len(tok) - 2):
        if vocab[tok[i]] + vocab[tok[i + 1]] + vocab[tok[i + 2]] == "<s>":
            tok[i:i + 3] = [bos_id]
        i += 1
    i = 0
    while i < max(0, len(tok) - 3):
        if vocab[tok[i]] + vocab[tok[i + 1]] + vocab[tok[i + 2]] + vocab[tok[i + 3]] == "</s>":
            tok[i:i + 4] = [eos_id]
        i += 1
    while len(tok) >= 2:
        best, best_id, best_idx = -np.inf, 0, None
        for i in range(len(tok) - 1):
            pid = index.get(vocab[tok[i]] + vocab[tok[i + 1]])
            if pid is not None and np.float32(scores[pid]) > best:
                best, best_id, best_idx = np.float32(scores[pid]), pid, i
        if best_idx is None:
            break
        tok[best_idx:best_idx + 2] = [best_id]
    if eos:
        tok.append(eos_id)
    return tok


def py_decode(vocab, prev, token):
    piece = vocab[token]
    if prev == 1:
        piece = piece.lstrip(" \t\n\r\v\f")
    if piece.startswith("<0x"):
        try:
            return chr(int(piece[3:5], 16))
        except ValueError:
            pass
    return piece.replace(SP, " ")


@pytest.fixture(scope="module")
def tok(tmp_path_factory):
    vocab, scores = make_vocab()
    path = str(tmp_path_factory.mktemp("tok") / "t.gguf")
    meta = [("tokenizer.ggml.tokens", G.ARRAY, (G.STRING, vocab)), ("tokenizer.ggml.scores", G.ARRAY, (G.F32, scores)),
            ("tokenizer.ggml.bos_token_id", G.U32, 1), ("tokenizer.ggml.eos_token_id", G.U32, 2), ("tokenizer.ggml.unknown_token_id", G.U32, 0)]
    G.write_gguf(path, meta, [])
    f = G.Gguf(path)
    t = G.LlamaTokenizer(f)
    yield t, vocab, scores
    t.close()
    f.close()


@pytest.mark.parametrize("text", ["hello world", "the hello abc", " hello", "hello  world", "héllo wörld", "abc<s>abc</s>x", "Zq", "日本", "a", "", "ss>s</s",
                                  "the the the the hello hello world.,!"])
@pytest.mark.parametrize("bos,eos", [(True, False), (False, True), (True, True), (False, False)])
def test_encode_matches_the_reference_algorithm(tok, text, bos, eos):
    t, vocab, scores = tok
    assert t.encode(text, bos, eos) == py_encode(vocab, scores, text, bos, eos)


def test_decode_and_round_trip(tok):
    t, vocab, scores = tok
    assert (t.vocab_size, t.bos, t.eos, t.unk) == (len(vocab), 1, 2, 0)
    for prev in (0, 1):
        for token in range(len(vocab)):
            assert t.decode(prev, token) == py_decode(vocab, prev, token)
    ids = t.encode("hello world the abc", bos=True)
    text = "".join(t.decode(p, c) for p, c in zip(ids[:-1], ids[1:]))
    assert text == "hello world the abc"                      # leading "▁" pieces come back as spaces
    assert t.decode(0, 3 + 0xE9) == "é"                        # byte piece -> the character U+00E9 (the reference's behaviour)


# ---- GPT-2 byte-pair encoding (crates/inferi/src/models/tokenizers/gpt2_tokenizer.rs:54-217) ----
regex = pytest.importorskip("regex")
PAT = regex.compile(r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+")


def bytes_to_unicode():
    bs = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, [chr(c) for c in cs]))


def make_bpe():
    enc = bytes_to_unicode()
    base = [enc[b] for b in range(256)]
    merges, vocab = [], list(base)
    corpus = "the quick brown fox jumps over the lazy dog hello world it's we're 123 4567 héllo wörld 日本語 " * 3
    words = [[enc[b] for b in w.encode()] for w in PAT.findall(corpus)]
    for _ in range(120):                                     # a small learned merge table
        counts = {}
        for w in words:
            for a, b in zip(w[:-1], w[1:]):
                counts[(a, b)] = counts.get((a, b), 0) + 1
        if not counts:
            break
        (a, b), _ = max(counts.items(), key=lambda kv: (kv[1], kv[0]))
        merges.append(f"{a} {b}")
        vocab.append(a + b)
        for w in words:
            i = 0
            while i < len(w) - 1:
                if w[i] == a and w[i + 1] == b:
                    w[i:i + 2] = [a + b]
                else:
                    i += 1
    vocab += ["<|begin_of_text|>", "<|end_of_text|>"]
    return vocab, merges


def py_bpe_encode(vocab, merges, text):
    enc = bytes_to_unicode()
    index = {v: i for i, v in enumerate(vocab)}
    rank = {tuple(m.split(" ")): i for i, m in enumerate(merges)}
    out = []

    def piece(sub):
        for tok in PAT.findall(sub):
            w = [enc[b] for b in tok.encode()]
            while len(w) > 1:
                pairs = {(a, b) for a, b in zip(w[:-1], w[1:])}
                best = min(pairs, key=lambda p: rank.get(p, 1 << 60))
                if best not in rank:
                    break
                a, b = best
                nw, i = [], 0
                while i < len(w):
                    if w[i] == a and i + 1 < len(w) and w[i + 1] == b:
                        nw.append(a + b)
                        i += 2
                    else:
                        nw.append(w[i])
                        i += 1
                w = nw
            out.extend(index[x] for x in w if x in index)

    cursor = 0
    for m in regex.finditer(r"<[^<>]*>", text):
        if cursor != m.start():
            piece(text[cursor:m.start()])
        out.append(index[m.group()])
        cursor = m.end()
    if cursor < len(text):
        piece(text[cursor:])
    return out


@pytest.fixture(scope="module")
def bpe(tmp_path_factory):
    vocab, merges = make_bpe()
    path = str(tmp_path_factory.mktemp("bpe") / "t.gguf")
    meta = [("tokenizer.ggml.tokens", G.ARRAY, (G.STRING, vocab)), ("tokenizer.ggml.merges", G.ARRAY, (G.STRING, merges)),
            ("tokenizer.ggml.bos_token_id", G.U32, len(vocab) - 2), ("tokenizer.ggml.eos_token_id", G.U32, len(vocab) - 1)]
    G.write_gguf(path, meta, [])
    f = G.Gguf(path)
    t = G.Gpt2Tokenizer(f)
    yield t, vocab, merges
    t.close()
    f.close()


@pytest.mark.parametrize("text", ["the quick brown fox", "hello world", " hello   world  ", "it's we're they'll I'd", "abc123 4567x", "héllo wörld!", "日本語 テスト",
                                  "a\n\nb\t c", "<|begin_of_text|>the dog<|end_of_text|>", "x < y z", "a > b < c", "tabs\tand nbsp em", "", "!!! ... ???", "'", "over9000's"])
def test_gpt2_encode_matches_the_reference_algorithm(bpe, text):
    t, vocab, merges = bpe
    assert t.encode(text) == py_bpe_encode(vocab, merges, text)


def test_gpt2_decode_and_specials(bpe):
    t, vocab, merges = bpe
    assert (t.bos, t.eos) == (len(vocab) - 2, len(vocab) - 1)
    ids = t.encode("the lazy dog jumps 123")
    assert t.decode_tokens(ids) == "the lazy dog jumps 123"
    assert t.decode_tokens(t.encode("é")) == "Ã©"            # the reference maps every byte to U+00XX: UTF-8 is not reassembled
    assert t.encode("x", bos=True, eos=True) == [t.bos] + t.encode("x") + [t.eos]
    from inferi_b200._lib import InferiError
    with pytest.raises(InferiError):
        t.encode("<nope>")                                     # a "<...>" stretch must be a vocabulary entry (the reference panics)
    with pytest.raises(InferiError):
        t.encode("x < y > z")
