"""GPU parity of the whole token loop against the CPU oracle: logits within 2e-2 max-abs, greedy tokens identical."""
import numpy as np
import pytest
import torch

import oracle
from helpers import LOGITS_MAX_ABS, TOKENS_EXACT
from inferi_b200 import quant
from inferi_b200.llama2 import LLAMA_3_2_1B, Llama2, Llama2Config, Llama2Weights, Q4_K_M, synth_weights, weights_to_host
from inferi_b200.ops import GpuQuantTensor, InferiError

pytestmark = pytest.mark.gpu


def oracle_cfg(c: Llama2Config) -> dict:
    return dict(hidden=c.hidden_size, ffn=c.intermediate_size, n_layers=c.num_hidden_layers, n_heads=c.num_attention_heads,
                n_kv_heads=c.num_key_value_heads, vocab=c.vocab_size, max_pos=c.max_position_embeddings, rope_theta=c.rope_theta,
                rms_eps=c.rms_norm_eps, rope_variant=c.rope_variant)


TINY = Llama2Config(256, 2048, 2, 4, 2, 512, 64, 500000.0, 1e-5)
TINY_RECIPE = dict(attn_q=quant.Q4_K, attn_k=quant.Q5_K, attn_v=quant.Q8_0, attn_output=quant.Q4_K, ffn_gate=quant.Q4_K, ffn_up=quant.Q4_K,
                   ffn_down=quant.Q6_K, token_embd=quant.Q4_K, output=quant.Q8_0)
SMALL = Llama2Config(2048, 8192, 2, 32, 8, 1024, 128, 500000.0, 1e-5)       # Llama-3.2-1B layer shapes, 2 layers
SMALL_TIED = dict(Q4_K_M, token_embd=quant.Q6_K)


def check_loop(backend, cfg, weights, kv_f16, prompt, n_gen, tied=False):
    host = weights_to_host(weights)
    ref = oracle.Llama(oracle_cfg(cfg), host, kv_f16=kv_f16)
    model = Llama2(backend, cfg, Llama2Weights(backend, cfg, weights), kv_f16=kv_f16)
    # 1. token by token with logits read back (the reference's forward_logits loop), prompt tokens forced
    tok, pos, worst = prompt[0], 0, 0.0
    fed, ref_tokens = [], []
    for step in range(len(prompt) + n_gen - 1):
        fed.append(tok)
        nxt, logits = model.forward(tok, pos, want_logits=True)
        want = ref.forward(tok, pos)
        worst = max(worst, float(np.abs(logits - want).max()))
        assert worst <= LOGITS_MAX_ABS, f"logits differ by {worst} at position {pos}"
        top2 = np.partition(want, -2)[-2:]
        want_next = oracle.argmax(want)
        assert nxt == oracle.argmax(logits), "device arg-max disagrees with the arg-max of its own logits"
        assert nxt == want_next, f"greedy token differs at position {pos}: {nxt} vs {want_next} (oracle margin {top2[1] - top2[0]:.3e})"
        pos += 1
        if step + 1 < len(prompt):
            tok = prompt[step + 1]
        else:
            ref_tokens.append(want_next)
            tok = want_next
    # 2. the on-device loop (one graph replay per token, no host round trip) must give the same ids
    out = model.generate(prompt, n_gen, start_pos=0)
    assert out.tolist() == ref_tokens
    # 3. continuing from a later start_pos with the cache kept (chat turns) reproduces the tail
    k = len(prompt) + n_gen // 2
    seq = list(prompt) + ref_tokens
    tail = model.generate(seq[k:k + 1], n_gen - (k - len(prompt)) - 1, start_pos=k)
    assert tail.tolist() == ref_tokens[k - len(prompt) + 1:]
    model.close()
    ref.close()
    return worst


@pytest.mark.parametrize("kv_f16", [False, True])
def test_tiny_model_all_quant_types(backend, kv_f16):
    w = synth_weights(TINY, seed=3001, recipe=TINY_RECIPE)
    check_loop(backend, TINY, w, kv_f16, prompt=[3, 500, 41, 7], n_gen=24)


def test_token_graph_launch_count_and_oracle_tokens(backend):
    """A token is a graph of 5 kernels per layer + 3 (begin, classifier, end); the launch counter must say so, and the
    greedy tokens must be the oracle's."""
    w = synth_weights(SMALL, seed=3005, device="cuda")
    prompt, n_gen = [5, 77, 1001], 10
    steps = len(prompt) + n_gen - 1
    model = Llama2(backend, SMALL, Llama2Weights(backend, SMALL, w), kv_f16=True)
    backend.reset_launch_count()
    got = model.generate(prompt, n_gen).tolist()
    assert backend.launch_count() == steps * (5 * SMALL.num_hidden_layers + 3)
    model.close()
    ref = oracle.Llama(oracle_cfg(SMALL), weights_to_host(w), kv_f16=True)
    want, tok = [], None
    for pos in range(steps):
        tok = prompt[pos] if pos < len(prompt) else want[-1]
        lg = ref.forward(tok, pos)
        if pos >= len(prompt) - 1:
            want.append(oracle.argmax(lg))
    ref.close()
    assert got == want


def test_small_model_tied_classifier(backend):
    w = synth_weights(SMALL, seed=3003, device="cuda", recipe=SMALL_TIED, tied=True)
    assert w["output"] is None
    check_loop(backend, SMALL, w, True, prompt=[1, 1000, 512], n_gen=12)


def test_llama_3_2_1b_architecture_64_tokens(backend):
    """16 layers, hidden 2048, 32 q / 8 kv heads of 64, FFN 8192, vocab 128256, Q4_K_M mix, f16 KV cache, context 4096:
    32 random prompt tokens through the decode path, then greedy decoding; the first 64 tokens must match the oracle."""
    cfg = LLAMA_3_2_1B
    w = synth_weights(cfg, seed=3001, device="cuda")
    prompt = np.random.default_rng(3002).integers(0, cfg.vocab_size, 32).tolist()
    worst = check_loop(backend, cfg, w, True, prompt=prompt, n_gen=TOKENS_EXACT - 32 + 1)
    print(f"1B-architecture: worst logits max-abs difference over 64 positions = {worst:.3e}")


@pytest.mark.parametrize("cfg,recipe", [(TINY, TINY_RECIPE), (SMALL, Q4_K_M)], ids=["head64", "head128"])
def test_qwen2_variant_neox_rotation_and_qkv_biases(backend, cfg, recipe):
    """`LlamaModelType::Qwen2` (crates/inferi/src/models/llama2/mod.rs:11-29): NeoX rotation, q / k / v biases added before it
    (transformer.rs:434-445).  The device model reorders the q / k rows at creation; the oracle rotates split halves."""
    import dataclasses
    qcfg = dataclasses.replace(cfg, rope_variant=1)
    w = synth_weights(qcfg, seed=77, recipe=recipe, qkv_bias=True)
    worst = check_loop(backend, qcfg, w, True, [2, 77, 300], 24)
    assert worst <= LOGITS_MAX_ABS
    # the biases and the rotation matter: the Llama reading of the same matrices gives other logits
    plain = Llama2(backend, cfg, Llama2Weights(backend, cfg, {**w, "layers": [{k: v for k, v in lw.items() if not k.endswith("_bias")} for lw in w["layers"]]}))
    qwen = Llama2(backend, qcfg, Llama2Weights(backend, qcfg, w))
    _, a = plain.forward(5, 3, want_logits=True)
    _, b = qwen.forward(5, 3, want_logits=True)
    assert np.abs(a - b).max() > 1e-2
    plain.close()
    qwen.close()


def test_generate_until_stops_at_the_stop_token(backend):
    w = synth_weights(TINY, seed=3001, recipe=TINY_RECIPE)
    model = Llama2(backend, TINY, Llama2Weights(backend, TINY, w), kv_f16=True)
    prompt = [3, 500, 41, 7]
    full = model.generate(prompt, 40).tolist()
    for k in (0, 5, 15, 16, 17, 33):                       # around the 16-token chunks of the device loop
        stop = full[k]
        first = full.index(stop)
        got = model.generate_until(prompt, 40, stop).tolist()
        assert got == full[:first + 1]
    absent = next(t for t in range(TINY.vocab_size) if t not in full)
    assert model.generate_until(prompt, 40, absent).tolist() == full
    # the next turn continues after the stop token with the cache kept
    k = 9
    head = model.generate_until(prompt, 40, full[k]).tolist()
    n = len(head)
    tail = model.generate([head[-1]], 40 - n, start_pos=len(prompt) + n - 1).tolist()
    assert head + tail == full
    model.close()


def test_model_contract_violations(backend):
    w = synth_weights(TINY, seed=1, recipe=TINY_RECIPE)
    weights = Llama2Weights(backend, TINY, w)
    bad = Llama2Config(256, 2048, 2, 4, 3, 512, 64)
    with pytest.raises(InferiError):
        Llama2(backend, bad, weights)                                 # head counts do not divide
    m = Llama2(backend, TINY, weights)
    with pytest.raises(InferiError):
        m.forward(512, 0)                                             # token outside the vocabulary
    with pytest.raises(InferiError):
        m.forward(0, 64)                                              # position outside the context
    with pytest.raises(InferiError):
        m.generate([1, 2, 3], 70)                                     # would run past the context
    with pytest.raises(InferiError):
        Llama2(backend, TINY, weights, tp_rank=2, tp_size=2)          # rank outside the group
    m.close()
    # a matrix that misses the alignment rules of the fused kernels is refused, not silently mis-read
    w2 = synth_weights(TINY, seed=1, recipe=dict(TINY_RECIPE, attn_v=quant.Q6_K))
    with pytest.raises(InferiError) as e:
        Llama2(backend, TINY, Llama2Weights(backend, TINY, w2))
    assert "alignment" in str(e.value)


def test_bounded_wait_expires_when_a_rank_never_arrives(backend):
    """A tensor-parallel rank whose peer never delivers: every wait inside the kernels is bounded, so the forward returns
    IB_ERR_TIMEOUT instead of hanging, the kernels have ended, and the context goes on serving other calls.
    The "peer" is a zeroed buffer in this GPU's own memory that nobody writes to (rank 1 does not exist), and the limit of
    the waits is set to a few milliseconds; nothing faults and no kernel is left waiting."""
    from inferi_b200 import tp
    from inferi_b200.ops import Backend, GemvQuant
    be = Backend(0)
    be.set_wait_limit(3_000_000)   # 3 ms per wait instead of the default 2 s
    cfg = Llama2Config(512, 2048, 2, 4, 2, 512, 32, 500000.0, 1e-5)
    recipe = {k: quant.Q4_K for k in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down", "token_embd", "output")}
    full = synth_weights(cfg, seed=11, recipe=recipe)
    mine = tp.shard_weights(cfg, full, 0, 2)
    shapes = tp.shard_shapes(cfg, 2, quant.Q4_K)
    # the exchange area of the rank that never comes: same size as ours, all zeros, never written by anyone else
    dev_w = Llama2Weights(be, cfg, mine, shapes=shapes)
    model = Llama2(be, cfg, dev_w, kv_f16=True, tp_rank=0, tp_size=2, connect=False)
    _, nbytes = model.tp_area()
    ghost = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    model.connect_areas([None, ghost.data_ptr()])
    with pytest.raises(InferiError) as e:
        model.forward(5, 0)
    assert e.value.code == 5 and "gave up waiting" in e.value.message     # IB_ERR_TIMEOUT
    torch.cuda.synchronize()                                              # the kernels have returned
    model.close()
    dev_w.close()
    # the context is still usable: a GEMV through it gives the oracle's result
    blocks = quant.random_blocks(quant.Q4_K, 64, 512, seed=3)
    v = np.random.default_rng(4).standard_normal(512).astype(np.float32)
    m = GpuQuantTensor(be, quant.Q4_K, 64, 512, blocks)
    out = torch.empty(64, device="cuda")
    GemvQuant(be).launch(out, m, torch.from_numpy(v).cuda())
    torch.cuda.synchronize()
    ref = oracle.gemv_ref(quant.Q4_K, 64, 512, blocks, v)
    assert np.abs(out.cpu().numpy() - ref).max() <= 1e-3 * np.abs(ref).max()
    m.close()
    be.close()   # every tensor and model of this context is gone by now


def test_logits_across_the_position_where_the_token_graph_changes(backend):
    """Below position 320 the model replays a token graph whose attention nodes merge their slices inside thread-block
    clusters, from there on the one that merges through global memory: the logits on both sides of the change must agree
    with the oracle fed the same tokens (teacher forcing, so that a near-tie cannot send the two down different branches)."""
    # 32 query / 8 kv heads of 64 (the 1B layer shapes): 8 kv heads make 55 slices, clusters of 5, and the change at 5 x 64 positions
    cfg = Llama2Config(2048, 8192, 2, 32, 8, 1024, 512, 500000.0, 1e-5)
    w = synth_weights(cfg, seed=4242)
    dev_w = Llama2Weights(backend, cfg, w)
    model = Llama2(backend, cfg, dev_w, kv_f16=True)
    seq = [7, 300, 41, 9] + model.generate([7, 300, 41, 9], 330).tolist()      # the device loop crosses the change by itself
    ref = oracle.Llama(oracle_cfg(cfg), weights_to_host(w), kv_f16=True)
    first, last = 312, 328
    probe = Llama2(backend, cfg, dev_w, kv_f16=True)
    probe.generate(seq[:first], 0)                                               # cache rows 0 .. first - 1
    worst = 0.0
    for pos in range(last + 1):
        want = ref.forward(seq[pos], pos)
        if pos < first:
            continue
        nxt, logits = probe.forward(seq[pos], pos, want_logits=True)
        worst = max(worst, float(np.abs(logits - want).max()))
        assert nxt == seq[pos + 1], f"the per-token path and the device loop disagree at position {pos}"
    assert worst <= LOGITS_MAX_ABS, f"logits differ by {worst} around the change of graphs"
    print(f"logits around position 320 agree with the oracle to {worst:.3e}")
    model.close()
    probe.close()
    dev_w.close()
