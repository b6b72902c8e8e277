"""Prompt prefill on the tensor cores against the decode path it replaces.

The reference feeds a prompt token by token through the decode path (crates/inferi-chat/src/chat_llama2.rs:137-155); that loop
is the anchor: after `prefill` the logits of the last prompt position must agree with the loop's within 2e-2 and the greedy
tokens that follow must be identical."""
import numpy as np
import pytest
import torch

import oracle
from helpers import LOGITS_MAX_ABS
from inferi_b200 import quant
from inferi_b200.llama2 import LLAMA_3_2_1B, Llama2, Llama2Config, Llama2Weights, Q4_K_M, synth_weights, weights_to_host
from inferi_b200.ops import InferiError

pytestmark = pytest.mark.gpu


def loop_vs_prefill(backend, cfg, dev_w, prompt, n_gen):
    loop = Llama2(backend, cfg, dev_w, kv_f16=True)
    fast = Llama2(backend, cfg, dev_w, kv_f16=True)
    first = loop.generate(prompt, 1)                       # the prompt through the decode path
    want_logits = loop.last_logits()
    want = first.tolist() + loop.generate(first, n_gen - 1, start_pos=len(prompt)).tolist()
    nxt = fast.prefill(prompt)                             # the prompt through the GEMMs
    got_logits = fast.last_logits()
    err = float(np.abs(got_logits - want_logits).max())
    assert err <= LOGITS_MAX_ABS, f"logits of the last prompt position differ by {err}"
    got = [nxt] + fast.generate([nxt], n_gen - 1, start_pos=len(prompt)).tolist()
    assert got == want, f"greedy tokens after the prompt differ (logits agreed to {err:.2e})"
    loop.close()
    fast.close()
    return err, want


def test_llama_3_2_1b_architecture_prefill_then_64_tokens(backend):
    cfg = LLAMA_3_2_1B
    w = synth_weights(cfg, seed=3001, device="cuda")
    dev_w = Llama2Weights(backend, cfg, w)
    del w
    prompt = np.random.default_rng(3002).integers(0, cfg.vocab_size, 32).tolist()
    err, _ = loop_vs_prefill(backend, cfg, dev_w, prompt, 65)
    print(f"1B-architecture prefill: logits of the last prompt position agree with the decode loop to {err:.3e}")
    dev_w.close()


def test_long_prompt_goes_in_chunks_and_matches_the_oracle(backend):
    """300 prompt tokens = three GEMM passes; a later turn continues from start_pos > 0.  Small model, also against the oracle."""
    cfg = Llama2Config(512, 1024, 2, 8, 2, 512, 512, 500000.0, 1e-5)
    recipe = dict(Q4_K_M, token_embd=quant.Q4_K, attn_v=quant.Q5_K, ffn_down=quant.Q8_0, output=quant.Q4_K)   # 512 columns: no Q6_K rows here
    w = synth_weights(cfg, seed=21, recipe=recipe)
    dev_w = Llama2Weights(backend, cfg, w)
    prompt = np.random.default_rng(22).integers(0, cfg.vocab_size, 300).tolist()
    _, want = loop_vs_prefill(backend, cfg, dev_w, prompt, 12)
    ref = oracle.Llama(dict(hidden=512, ffn=1024, n_layers=2, n_heads=8, n_kv_heads=2, vocab=512, max_pos=512, rope_theta=500000.0, rms_eps=1e-5),
                       weights_to_host(w), kv_f16=True)
    toks, out = list(prompt), []
    for pos in range(len(prompt) + 11):
        lg = ref.forward(toks[pos], pos)
        if pos >= len(prompt) - 1:
            out.append(oracle.argmax(lg))
            toks.append(out[-1])
    ref.close()
    assert want == out
    # second turn: 40 more prompt tokens on top of the kept cache
    m = Llama2(backend, cfg, dev_w, kv_f16=True)
    a = m.prefill(prompt)
    more = np.random.default_rng(23).integers(0, cfg.vocab_size, 40).tolist()
    b = m.prefill(more, start_pos=len(prompt))
    loop = Llama2(backend, cfg, dev_w, kv_f16=True)
    assert int(loop.generate(prompt + more, 1)[0]) == b and a == want[0]
    m.close()
    loop.close()
    dev_w.close()


def test_prefill_refuses_what_the_tensor_core_path_does_not_take(backend):
    cfg = Llama2Config(256, 2048, 2, 4, 2, 512, 64, 500000.0, 1e-5)     # 2 query heads per kv head, 256-row matrices... kv_mul = 2
    w = synth_weights(cfg, seed=5, recipe=dict(Q4_K_M, token_embd=quant.Q4_K, attn_v=quant.Q4_K, ffn_down=quant.Q4_K, output=quant.Q4_K))
    dev_w = Llama2Weights(backend, cfg, w)
    m = Llama2(backend, cfg, dev_w, kv_f16=True)
    with pytest.raises(InferiError) as e:
        m.prefill([1, 2, 3])
    assert e.value.code == 4      # IB_ERR_UNSUPPORTED: the caller feeds the prompt through generate()
    assert m.generate([1, 2, 3], 4).shape == (4,)
    m.close()
    dev_w.close()
