"""Generates tests/golden/chat_template.json: conversations and what the reference's bundled default chat template
(crates/inferi/src/models/tokenizers/llama-2-chat.jinja, used by `ChatTemplate::from_gguf` when a file carries no
`tokenizer.chat_template`, crates/inferi-chat/src/chat_template.rs:19-24) renders for them with the settings of
`ChatTemplate::apply` (chat_template.rs:26-37: block trimming, bos_token / eos_token / add_generation_prompt globals).
The template is rendered with jinja2; the reference's engine, minijinja, implements the same language.  The rendering
keeps the template file's own indentation and line breaks between the turns; the test compares modulo white space.

Needs the reference checkout; run from the repository root:
    python tests/golden/make_chat_template_golden.py <path to the reference checkout>
"""
import json
import os
import sys

import jinja2

CASES = [
    [["user", "hi there"]],
    [["system", " be brief "], ["user", "hi there"]],
    [["system", "You are terse."], ["user", "What is 2+2?"], ["assistant", " 4 "], ["user", "and 3+3?"]],
    [["user", "one"], ["assistant", "two"], ["user", "three"], ["assistant", "four"], ["user", " five\n"]],
]


def main():
    ref = sys.argv[1]
    text = open(os.path.join(ref, "crates/inferi/src/models/tokenizers/llama-2-chat.jinja")).read()

    def raise_exception(msg):
        raise jinja2.TemplateError(msg)

    env = jinja2.Environment(trim_blocks=True)
    env.globals.update(bos_token="<s>", eos_token="</s>", add_generation_prompt=True, raise_exception=raise_exception)
    tmpl = env.from_string(text)
    out = []
    for case in CASES:
        msgs = [{"role": r, "content": c} for r, c in case]
        out.append({"entries": case, "bos": "<s>", "eos": "</s>", "rendered": tmpl.render(messages=msgs)})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "chat_template.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", path)


if __name__ == "__main__":
    main()
