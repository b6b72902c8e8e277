"""Chat template and prompt hand-off (host side; no GPU): `ChatTemplate` against renderings of the reference's bundled default
template (tests/golden/chat_template.json) and against hand-written expectations of the published Llama-2 layout."""
import json
import os
import re

import pytest

from inferi_b200.chat import LLAMA2_CHAT_TEMPLATE, ChatTemplate, Prompt

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "chat_template.json")


def prompt_of(entries) -> Prompt:
    p = Prompt()
    for role, text in entries:
        {"user": p.append_user, "assistant": p.append_assistant, "system": p.append_system}[role](text)
    return p


def squeeze(s: str) -> str:
    return re.sub(r"\s+", "", s)


@pytest.mark.parametrize("case", json.load(open(GOLDEN)), ids=lambda c: f"{len(c['entries'])}-entries")
def test_default_template_renders_what_the_reference_default_renders(case):
    # The reference's file leaves its own indentation between the turns; everything but white space must agree, and the
    # rendering here carries no white space the conversation did not contain.
    mine = ChatTemplate(LLAMA2_CHAT_TEMPLATE).apply(prompt_of(case["entries"]), case["bos"], case["eos"])
    assert squeeze(mine) == squeeze(case["rendered"])
    assert "  " not in mine and not mine.startswith((" ", "\n")) and not mine.endswith("\n")


def test_default_template_layout():
    p = prompt_of([["system", " be brief "], ["user", "hi there"], ["assistant", "hello"], ["user", "bye"]])
    got = ChatTemplate(LLAMA2_CHAT_TEMPLATE).apply(p, "<s>", "</s>")
    assert got == "<s>[INST] <<SYS>>\nbe brief\n<</SYS>>\n\nhi there [/INST] hello </s><s>[INST] bye [/INST]"


def test_roles_must_alternate():
    import jinja2
    with pytest.raises(jinja2.TemplateError):
        ChatTemplate(LLAMA2_CHAT_TEMPLATE).apply(prompt_of([["user", "a"], ["user", "b"]]), "<s>", "</s>")


def test_template_globals_and_python_style_expressions():
    # The globals of chat_template.rs:30-32 and the two constructs the reference rewrites for its engine (:12-16).
    t = ChatTemplate("{{ bos_token }}{% for m in messages %}{{ m['content'].split(':')[-1] }}|{% endfor %}"
                     "{% if add_generation_prompt %}<gen>{% endif %}{{ eos_token }}")
    assert t.apply(prompt_of([["user", "a:b:c"], ["assistant", "x"]]), "<B>", "<E>") == "<B>c|x|<gen><E>"


def test_block_trimming_is_on():
    t = ChatTemplate("{% for m in messages %}\n{{ m['role'] }}\n{% endfor %}\n")
    assert t.apply(prompt_of([["user", "a"], ["assistant", "b"]]), "", "") == "user\nassistant\n"


def test_from_gguf_reads_the_metadata_template_or_falls_back(tmp_path):
    from inferi_b200 import gguf as G
    from inferi_b200.llama2 import Llama2Config
    try:
        G.load()
    except Exception as e:      # the shared library is the parser; without it there is nothing to test
        pytest.skip(f"shared library not built: {e}")
    path = str(tmp_path / "m.gguf")
    G.write_gguf(path, [("tokenizer.chat_template", G.STRING, "{{ bos_token }}X")], [])
    g = G.Gguf(path)
    assert ChatTemplate.from_gguf(g).template == "{{ bos_token }}X"
    g.close()
    G.write_gguf(path, [("general.name", G.STRING, "m")], [])
    g = G.Gguf(path)
    assert ChatTemplate.from_gguf(g).template == LLAMA2_CHAT_TEMPLATE
    g.close()


def test_prompt_display_and_jinja_input():
    p = prompt_of([["system", "s"], ["user", "u"]])
    assert str(p) == "[System] s\n[User] u\n"
    assert p.to_jinja_input() == {"messages": [{"role": "system", "content": "s"}, {"role": "user", "content": "u"}]}
    p.clear()
    assert p.entries == []


def test_writer_emits_what_the_llama_tokenizer_reads(tmp_path):
    """`write_llama_gguf(..., tokens, scores, special)` carries everything `LlamaTokenizer::from_gguf` asks for
    (crates/inferi/src/models/tokenizers/llama2_tokenizer.rs:23-40): the file loads and round-trips a string."""
    from inferi_b200 import gguf as G
    from inferi_b200.llama2 import Llama2Config, synth_weights
    try:
        G.load()
    except Exception as e:
        pytest.skip(f"shared library not built: {e}")
    cfg = Llama2Config(256, 512, 1, 4, 2, 300, 64, 10000.0, 1e-5)
    vocab = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + ["▁", "hi", "▁hi", "the", "re"]
    vocab += [f"w{i}" for i in range(cfg.vocab_size - len(vocab))]
    path = str(tmp_path / "t.gguf")
    G.write_llama_gguf(path, cfg, synth_weights(cfg, seed=3), tokens=vocab, scores=[-float(i) for i in range(len(vocab))], special=(1, 2, 0),
                       chat_template="{{ bos_token }}{{ messages[0]['content'] }}")
    g = G.Gguf(path)
    tok = G.LlamaTokenizer(g)
    assert (tok.bos, tok.eos, tok.unk, tok.vocab_size) == (1, 2, 0, cfg.vocab_size)
    ids = tok.encode("hi there", False, False)
    text, prev = "", tok.bos
    for t in ids:
        text += tok.decode(prev, t)
        prev = t
    assert text == "hi there"
    assert ChatTemplate.from_gguf(g).apply(prompt_of([["user", "x"]]), "<s>", "</s>") == "<s>x"
    tok.close()
    g.close()
