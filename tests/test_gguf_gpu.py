"""GGUF -> device loader on the GPU: a model loaded from a file must behave exactly like the same checkpoint uploaded tensor
by tensor, and like the CPU oracle."""
import numpy as np
import pytest

import oracle
from inferi_b200 import gguf as G
from inferi_b200 import quant
from inferi_b200._lib import InferiError
from inferi_b200.llama2 import Llama2, Llama2Config, Llama2Weights, synth_weights, weights_to_host

pytestmark = pytest.mark.gpu

TINY = Llama2Config(256, 2048, 2, 4, 2, 512, 64, 500000.0, 1e-5)
RECIPE = dict(attn_q=quant.Q4_K, attn_k=quant.Q5_K, attn_v=quant.Q8_0, attn_output=quant.Q4_K, ffn_gate=quant.Q4_K, ffn_up=quant.Q4_K,
              ffn_down=quant.Q6_K, token_embd=quant.Q4_K, output=quant.Q8_0)


def oracle_tokens(cfg, w, prompt, n_gen, kv_f16=True):
    ref = oracle.Llama(dict(rope_variant=cfg.rope_variant, hidden=cfg.hidden_size, ffn=cfg.intermediate_size, n_layers=cfg.num_hidden_layers, n_heads=cfg.num_attention_heads,
                            n_kv_heads=cfg.num_key_value_heads, vocab=cfg.vocab_size, max_pos=cfg.max_position_embeddings,
                            rope_theta=float(np.float32(cfg.rope_theta)), rms_eps=float(np.float32(cfg.rms_norm_eps))), weights_to_host(w), kv_f16=kv_f16)
    want = []
    for pos in range(len(prompt) + n_gen - 1):
        tok = prompt[pos] if pos < len(prompt) else want[-1]
        lg = ref.forward(tok, pos)
        if pos >= len(prompt) - 1:
            want.append(oracle.argmax(lg))
    ref.close()
    return want


@pytest.mark.parametrize("tied", [False, True])
def test_model_from_file_equals_model_from_tensors(backend, tmp_path, tied):
    recipe = dict(RECIPE, token_embd=quant.Q8_0) if tied else RECIPE
    w = synth_weights(TINY, seed=21, recipe=recipe, tied=tied)
    path = str(tmp_path / "m.gguf")
    G.write_llama_gguf(path, TINY, w)
    f = G.Gguf(path)
    assert f.llama_config().vocab_size == TINY.vocab_size
    from_file = f.load_llama(backend, kv_f16=True)
    f.close()                                            # the model owns its weights: the mapping may go
    direct = Llama2(backend, TINY, Llama2Weights(backend, TINY, w), kv_f16=True)
    prompt, n_gen = [3, 500, 41], 20
    a = from_file.generate(prompt, n_gen).tolist()
    b = direct.generate(prompt, n_gen).tolist()
    assert a == b == oracle_tokens(TINY, w, prompt, n_gen)
    _, la = from_file.forward(a[-1], len(prompt) + n_gen - 1, want_logits=True)
    _, lb = direct.forward(b[-1], len(prompt) + n_gen - 1, want_logits=True)
    assert np.array_equal(la, lb)                        # same kernels on the same bytes
    from_file.close()
    direct.close()


def test_qwen2_file_with_biases(backend, tmp_path):
    """arch "qwen2" (crates/inferi/src/models/llama2/mod.rs:17-22): `qwen2.*` metadata keys, blk.N.attn_{q,k,v}.bias tensors
    (transformer.rs:307-335), NeoX rotation."""
    import dataclasses
    cfg = dataclasses.replace(TINY, rope_variant=1)
    w = synth_weights(cfg, seed=23, recipe=RECIPE, qkv_bias=True)
    path = str(tmp_path / "q.gguf")
    G.write_llama_gguf(path, cfg, w, arch="qwen2")
    f = G.Gguf(path)
    with pytest.raises(InferiError):
        f.llama_config()                                 # the default model type looks for llama.* keys (cpu.rs:74-76)
    got = f.llama_config("qwen2")
    assert got.rope_variant == 1 and (got.hidden_size, got.num_key_value_heads, got.vocab_size) == (cfg.hidden_size, cfg.num_key_value_heads, cfg.vocab_size)
    m = f.load_llama(backend, kv_f16=True, arch="qwen2")
    f.close()
    prompt, n_gen = [9, 17, 250], 20
    assert m.generate(prompt, n_gen).tolist() == oracle_tokens(cfg, w, prompt, n_gen)
    m.close()


def test_context_cap_and_unsupported_tensor_types(backend, tmp_path):
    w = synth_weights(TINY, seed=22, recipe=RECIPE)
    path = str(tmp_path / "m.gguf")
    G.write_llama_gguf(path, TINY, w)
    f = G.Gguf(path)
    m = f.load_llama(backend, max_context=16)
    with pytest.raises(InferiError):
        m.forward(1, 16)                                 # outside the capped context
    m.close()
    f.close()
    # an F16 matrix where the fused kernels need a quantized one
    cfg = TINY
    meta = [("llama.embedding_length", G.U32, cfg.hidden_size), ("llama.feed_forward_length", G.U32, cfg.intermediate_size), ("llama.block_count", G.U32, 1),
            ("llama.attention.head_count", G.U32, 4), ("llama.attention.head_count_kv", G.U32, 2), ("llama.context_length", G.U32, 32)]
    emb = quant.random_blocks(quant.Q8_0, 512, 256, seed=1)
    bad = str(tmp_path / "bad.gguf")
    G.write_gguf(bad, meta, [("token_embd.weight", quant.Q8_0, (512, 256), emb.tobytes()),
                             ("blk.0.attn_q.weight", 1, (256, 256), np.zeros((256, 256), np.float16).tobytes())])
    g = G.Gguf(bad)
    with pytest.raises(InferiError):
        g.load_llama(backend)
    g.close()
