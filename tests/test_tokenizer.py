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
