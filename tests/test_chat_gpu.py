"""The chat turn loop with its per-token events (`ib_llama_chat` ≙ `ChatLlama2::forward`, crates/inferi-chat/src/chat_llama2.rs:92-189)
against the plain token loop: same tokens, the event fields the reference computes, early stop by callback and by stop token."""
import numpy as np
import pytest

from inferi_b200 import quant
from inferi_b200.chat import ChatLlama2, ChatTemplate, Prompt, PromptTokens, TemplatedPrompt, Token
from inferi_b200.llama2 import Llama2, Llama2Config, Llama2Weights, Q4_K_M, synth_weights

pytestmark = pytest.mark.gpu

CFG = Llama2Config(512, 1024, 2, 8, 2, 512, 512, 500000.0, 1e-5)
RECIPE = dict(Q4_K_M, token_embd=quant.Q4_K, attn_v=quant.Q5_K, ffn_down=quant.Q8_0, output=quant.Q4_K)


class IdTokenizer:
    """Token ids as text, so that the test reads the event strings without a vocabulary."""
    bos, eos = 1, 2

    def __init__(self, eos=2):
        self.eos = eos

    def decode(self, prev, tok):
        return f"<{prev}>{tok}"


@pytest.fixture(scope="module")
def weights(backend):
    w = synth_weights(CFG, seed=77, recipe=RECIPE)
    dev_w = Llama2Weights(backend, CFG, w)
    yield dev_w
    dev_w.close()


@pytest.mark.parametrize("n_prompt,start_pos", [(1, 0), (3, 0), (40, 0), (5, 17)])
def test_events_follow_the_token_loop(backend, weights, n_prompt, start_pos):
    rng = np.random.default_rng(n_prompt)
    history = rng.integers(3, CFG.vocab_size, start_pos + n_prompt).tolist()
    plain = Llama2(backend, CFG, weights)
    want = plain.generate(history, 40).tolist()
    # an eos that never shows up, so that the turn runs to max_gen
    eos = next(t for t in range(CFG.vocab_size) if t not in want)
    chat_model = Llama2(backend, CFG, weights)
    if start_pos:
        chat_model.generate(history[:start_pos], 0)          # the earlier turns' cache rows
    chat = ChatLlama2(chat_model, IdTokenizer(eos))
    events = []
    n = chat.forward_tokens(history[start_pos:], start_pos, lambda e: events.append(e) and False, 40)
    assert n == 40 and len(events) == 40 and all(isinstance(e, Token) for e in events)
    toks, prev = [], history[-1]
    for i, e in enumerate(events):
        tok = int(e.string.split(">")[1])
        assert e.string == f"<{prev}>{tok}"
        pos = start_pos + n_prompt - 1 + i
        assert e.next_pos == pos and e.token_count == max(pos - start_pos - 1, 0)
        toks.append(tok)
        prev = tok
    assert toks == want
    times = [e.token_time for e in events]
    assert all(b >= a for a, b in zip(times, times[1:])) and times[-1] > 0.0
    if n_prompt == 1:
        assert events[0].token_count == 0 and events[0].token_time == 0.0     # chat_llama2.rs:168-177: no rate before the timer starts
    plain.close()
    chat_model.close()


def test_callback_and_stop_token_end_the_turn(backend, weights):
    prompt = [5, 9, 300, 41]
    plain = Llama2(backend, CFG, weights)
    want = plain.generate(prompt, 30).tolist()
    plain.close()
    # the callback asks to stop after 7 events
    m = Llama2(backend, CFG, weights)
    seen = []
    n = ChatLlama2(m, IdTokenizer(eos=next(t for t in range(CFG.vocab_size) if t not in want))).forward_tokens(
        prompt, 0, lambda e: seen.append(e) or len(seen) == 7, 30)
    assert n == 7 and [int(e.string.split(">")[1]) for e in seen] == want[:7]
    m.close()
    # the stop token is want[k] for the first k whose token has not occurred before: events are want[:k], none for the stop token
    k = next(i for i in range(3, 30) if want[i] not in want[:i])
    m = Llama2(backend, CFG, weights)
    seen = []
    n = ChatLlama2(m, IdTokenizer(eos=want[k])).forward_tokens(prompt, 0, lambda e: seen.append(e) and False, 30)
    assert n == k and [int(e.string.split(">")[1]) for e in seen] == want[:k]
    # an exception in the callback ends the turn and surfaces on the host side
    def boom(e):
        raise RuntimeError("stop")
    with pytest.raises(RuntimeError):
        ChatLlama2(m, IdTokenizer(eos=want[k])).forward_tokens(prompt, 0, boom, 30)
    m.close()


def test_turn_ends_when_the_context_is_full(backend, weights):
    m = Llama2(backend, CFG, weights)
    prompt = np.random.default_rng(5).integers(3, CFG.vocab_size, CFG.max_position_embeddings - 4).tolist()
    plain = Llama2(backend, CFG, weights)
    want = plain.generate(prompt, 5).tolist()
    plain.close()
    seen = []
    eos = next(t for t in range(CFG.vocab_size) if t not in want)
    n = ChatLlama2(m, IdTokenizer(eos=eos)).forward_tokens(prompt, 0, lambda e: seen.append(e) and False, 1000)
    assert [int(e.string.split(">")[1]) for e in seen] == want
    # positions 508 .. 511 are free: the forwards at 507 .. 511 yield five tokens, then the context is full
    assert n == 5 and seen[-1].next_pos == CFG.max_position_embeddings - 1
    m.close()


def test_full_turn_from_a_gguf_file(backend, tmp_path):
    """Template -> tokenizer -> token loop on a file with a vocabulary: the three event kinds in the reference's order."""
    from inferi_b200 import gguf as G
    cfg = CFG
    w = synth_weights(cfg, seed=9, recipe=RECIPE)
    vocab = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + ["▁", "[", "]", "INST", "/", "hi", "▁hi", "he", "l", "o", "▁[", "a", "b", "c"]
    vocab += [f"w{i}" for i in range(cfg.vocab_size - len(vocab))]
    path = str(tmp_path / "chat.gguf")
    G.write_llama_gguf(path, cfg, w, tokens=vocab, scores=[-float(i) for i in range(len(vocab))], special=(1, 2, 0))
    g = G.Gguf(path)
    chat = ChatLlama2.from_gguf(backend, g)
    template = ChatTemplate.from_gguf(g)
    p = Prompt()
    p.append_user("hi")
    events = []
    n = chat.forward(p, template, 0, lambda e: events.append(e) and False, max_gen=12)
    assert isinstance(events[0], TemplatedPrompt) and events[0].text == "<s>[INST] hi [/INST]"
    assert isinstance(events[1], PromptTokens) and [t for t, _ in events[1].tokens] == chat.tokenizer.encode(events[0].text, False, False)
    tokens = [e for e in events[2:]]
    assert n == len(tokens) and all(isinstance(e, Token) for e in tokens) and n <= 12
    want = chat.model.generate([t for t, _ in events[1].tokens], 12).tolist()
    got_ids = want[:n]
    prev = events[1].tokens[-1][0]
    for e, tok in zip(tokens, got_ids):
        assert e.string == chat.tokenizer.decode(prev, tok)
        prev = tok
    if n < 12:
        assert want[n] == chat.tokenizer.eos
    chat.model.close()
    chat.tokenizer.close()
    g.close()
