"""The chat turn around the token loop: host-side mirror of `ChatLlama2::forward` and its callback.

`Prompt` ≙ `Prompt` / `PromptEntry` (crates/inferi-chat/src/prompt.rs:16-110), `ChatTemplate` ≙ `ChatTemplate`
(crates/inferi-chat/src/chat_template.rs:6-38), the event classes ≙ `ChatEvent` (prompt.rs:4-13) and `ChatLlama2.forward`
≙ `ChatLlama2::forward` (crates/inferi-chat/src/chat_llama2.rs:92-189).  The template string comes out of the GGUF
metadata through the C ABI and is rendered here, on the host, with jinja2 (the reference renders it with minijinja); the
token loop and its per-token events run in the shared library (`ib_llama_chat`).  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np
import torch

from ._lib import TOKEN_EVENT_FN, check

# The published Llama-2 chat layout, for files without `tokenizer.chat_template` (the reference falls back to its own
# bundled copy of that layout, llama2_tokenizer.rs:21): an optional system message folded into the first user turn,
# each user turn as bos + "[INST] ... [/INST]", each assistant turn as " ... " + eos.
LLAMA2_CHAT_TEMPLATE = (
    "{% if messages[0]['role'] == 'system' %}{% set sys = '<<SYS>>\\n' + messages[0]['content'] | trim + '\\n<</SYS>>\\n\\n' %}"
    "{% set messages = messages[1:] %}{% else %}{% set sys = '' %}{% endif %}"
    "{% for m in messages %}"
    "{% if (m['role'] == 'user') != (loop.index0 % 2 == 0) %}{{ raise_exception('roles must alternate user/assistant') }}{% endif %}"
    "{% set content = (sys + m['content']) if loop.index0 == 0 else m['content'] %}"
    "{% if m['role'] == 'user' %}{{ bos_token + '[INST] ' + content | trim + ' [/INST]' }}"
    "{% elif m['role'] == 'assistant' %}{{ ' ' + content | trim + ' ' + eos_token }}{% endif %}"
    "{% endfor %}"
)


@dataclass
class Prompt:
    """The conversation so far, as (role, text) entries (prompt.rs:43-110)."""

    entries: list[tuple[str, str]] = field(default_factory=list)

    def append_user(self, text: str) -> None:
        self.entries.append(("user", text))

    def append_assistant(self, text: str) -> None:
        self.entries.append(("assistant", text))

    def append_system(self, text: str) -> None:
        self.entries.append(("system", text))

    def clear(self) -> None:
        self.entries.clear()

    def to_jinja_input(self) -> dict:
        return {"messages": [{"role": r, "content": t} for r, t in self.entries]}

    def __str__(self) -> str:
        return "".join(f"[{r.capitalize()}] {t}\n" for r, t in self.entries)


@dataclass
class TemplatedPrompt:
    """≙ `ChatEvent::TemplatedPrompt`: the rendered prompt string."""

    text: str


@dataclass
class PromptTokens:
    """≙ `ChatEvent::PromptTokens`: (token id, its string) for every prompt token."""

    tokens: list[tuple[int, str]]


@dataclass
class Token:
    """≙ `ChatEvent::Token` (prompt.rs:6-11)."""

    string: str
    next_pos: int
    token_count: int
    token_time: float


class ChatTemplate:
    """≙ `ChatTemplate` (chat_template.rs:6-38).  The reference rewrites `.split(` and `[-1]` into filters because its
    engine lacks them; jinja2 evaluates both natively, so the string is used as found."""

    def __init__(self, template: str):
        self.template = template

    @classmethod
    def from_gguf(cls, gguf) -> "ChatTemplate":
        keys = dict(gguf.keys())
        if "tokenizer.chat_template" in keys:
            return cls(gguf.get("tokenizer.chat_template", keys["tokenizer.chat_template"]))
        return cls(LLAMA2_CHAT_TEMPLATE)

    def apply(self, prompt: Prompt, bos: str, eos: str) -> str:
        """Render with the globals the reference sets (chat_template.rs:26-37): bos_token, eos_token,
        add_generation_prompt = true, block-trimming on."""
        import jinja2

        def raise_exception(msg):
            raise jinja2.TemplateError(msg)

        env = jinja2.Environment(trim_blocks=True)
        env.globals.update(bos_token=bos, eos_token=eos, add_generation_prompt=True, raise_exception=raise_exception)
        return env.from_string(self.template).render(**prompt.to_jinja_input())


class ChatLlama2:
    """≙ `ChatLlama2` (chat_llama2.rs:21-189): a model, its tokenizer and the turn loop."""

    def __init__(self, model, tokenizer, vocab: list[str] | None = None):
        self.model, self.tokenizer = model, tokenizer
        self._vocab = vocab

    @classmethod
    def from_gguf(cls, backend, gguf, **load_args) -> "ChatLlama2":
        from .gguf import Gpt2Tokenizer, LlamaTokenizer

        keys = dict(gguf.keys())
        kind = gguf.get("tokenizer.ggml.model", keys["tokenizer.ggml.model"]) if "tokenizer.ggml.model" in keys else "llama"
        tok = (Gpt2Tokenizer if kind == "gpt2" else LlamaTokenizer)(gguf)
        vocab = gguf.get("tokenizer.ggml.tokens", keys["tokenizer.ggml.tokens"])
        return cls(gguf.load_llama(backend, **load_args), tok, vocab)

    def bos_str(self) -> str:
        return self._vocab[self.tokenizer.bos] if self._vocab else ""

    def eos_str(self) -> str:
        return self._vocab[self.tokenizer.eos] if self._vocab else ""

    def forward(self, prompt: Prompt, template: ChatTemplate, start_pos: int, out, max_gen: int = 1 << 30,
                temperature: float = 0.0, topp: float = 1.0, seed: int = 0) -> int:
        """One turn: template -> TemplatedPrompt event -> encode (no bos/eos added, chat_llama2.rs:112) -> PromptTokens event
        -> the device token loop from `start_pos`, one Token event per generated token.  `out(event)` returning a true value
        (or raising) ends the turn, like an Err from the reference's callback.  Returns the number of Token events."""
        text = template.apply(prompt, self.bos_str(), self.eos_str())
        if out(TemplatedPrompt(text)):
            return 0
        toks = self.tokenizer.encode(text, False, False)
        if out(PromptTokens([(t, self.tokenizer.decode(0, t)) for t in toks])):
            return 0
        self.model.set_sampler(temperature, topp, seed)
        return self.forward_tokens(toks[start_pos:], start_pos, out, min(max_gen, 0xFFFFFFFF))

    def forward_tokens(self, tokens, start_pos: int, out, max_gen: int) -> int:
        """The loop alone, on token ids: `tokens` are the prompt tokens from `start_pos` on."""
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        failure: list[BaseException] = []

        def on_token(_user, prev, tok, next_pos, count, seconds):
            try:
                return 1 if out(Token(self.tokenizer.decode(prev, tok), next_pos, count, seconds)) else 0
            except BaseException as e:     # an exception must not unwind through the C frames
                failure.append(e)
                return 1

        cb = TOKEN_EVENT_FN(on_token)
        n = C.c_uint32()
        m = self.model
        check(m.lib.ib_llama_chat(m.handle, torch.cuda.current_stream().cuda_stream, toks.ctypes.data_as(C.c_void_p), toks.size, start_pos,
                                  max_gen, self.tokenizer.eos, cb, None, C.byref(n)))
        if failure:
            raise failure[0]
        return n.value
