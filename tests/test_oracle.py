"""CPU tests of the oracle: pinned against the committed golden vectors (made with the third-party gguf package)
and against closed-form numpy restatements of each op."""
import os

import numpy as np
import pytest

import oracle
from inferi_b200 import quant

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "blocks.npz"))
QTYPES = [quant.Q8_0, quant.Q4_K, quant.Q5_K, quant.Q6_K]
LEGACY = [quant.Q4_0, quant.Q4_1, quant.Q5_0, quant.Q5_1]          # op-level formats with golden vectors from the gguf package


@pytest.mark.parametrize("qt", QTYPES + LEGACY)
def test_dequantize_matches_golden_bit_for_bit(qt):
    n = quant.NAMES[qt]
    blocks, deq = GOLDEN[f"{n}_blocks"], GOLDEN[f"{n}_deq"]
    mine = oracle.dequantize(qt, blocks, deq.size).reshape(deq.shape)
    assert np.array_equal(mine.view(np.uint32), deq.view(np.uint32))


@pytest.mark.parametrize("qt", QTYPES)
def test_gemv_ref_and_shader_match_golden(qt):
    n = quant.NAMES[qt]
    blocks, v, want = GOLDEN[f"{n}_blocks"], GOLDEN[f"{n}_v"], GOLDEN[f"{n}_gemv"]
    rows, cols = GOLDEN[f"{n}_deq"].shape
    ref = oracle.gemv_ref(qt, rows, cols, blocks, v)
    assert np.array_equal(ref, want.astype(np.float32))            # f64 accumulate, one rounding
    sh = oracle.gemv_shader(qt, rows, cols, blocks, v)
    scale = np.abs(want).max()
    assert np.abs(sh - want).max() <= 2e-6 * scale                 # f32 lane partials + tree


@pytest.mark.parametrize("qt", LEGACY)
def test_legacy_gemv_ref_matches_golden(qt):
    n = quant.NAMES[qt]
    blocks, v, want = GOLDEN[f"{n}_blocks"], GOLDEN[f"{n}_v"], GOLDEN[f"{n}_gemv"]
    rows, cols = GOLDEN[f"{n}_deq"].shape
    assert np.array_equal(oracle.gemv_ref(qt, rows, cols, blocks, v), want.astype(np.float32))


def test_q8_k_dequantize_closed_form():
    """Q8_K (crates/inferi/src/quantization.rs:205-211): f32 scale times int8 quants; the 16 block sums are not used."""
    blocks = quant.random_blocks(quant.Q8_K, 8, 512, seed=123)
    b = blocks.reshape(-1, 292)
    d = b[:, :4].copy().view(np.float32)
    want = (d * b[:, 4:260].view(np.int8).astype(np.float32)).reshape(-1)
    mine = oracle.dequantize(quant.Q8_K, blocks, want.size)
    assert np.array_equal(mine.view(np.uint32), want.view(np.uint32))
    v = np.random.default_rng(1).standard_normal(512).astype(np.float32)
    ref = oracle.gemv_ref(quant.Q8_K, 8, 512, blocks, v)
    assert np.array_equal(ref, (want.reshape(8, 512).astype(np.float64) @ v.astype(np.float64)).astype(np.float32))


@pytest.mark.parametrize("qt", QTYPES + LEGACY)
def test_dequantize_matches_gguf_package_on_fresh_blocks(qt):
    gguf = pytest.importorskip("gguf")
    from gguf.quants import dequantize
    gt = {quant.Q8_0: gguf.GGMLQuantizationType.Q8_0, quant.Q4_K: gguf.GGMLQuantizationType.Q4_K,
          quant.Q5_K: gguf.GGMLQuantizationType.Q5_K, quant.Q6_K: gguf.GGMLQuantizationType.Q6_K,
          quant.Q4_0: gguf.GGMLQuantizationType.Q4_0, quant.Q4_1: gguf.GGMLQuantizationType.Q4_1,
          quant.Q5_0: gguf.GGMLQuantizationType.Q5_0, quant.Q5_1: gguf.GGMLQuantizationType.Q5_1}[qt]
    blocks = quant.random_blocks(qt, 64, 512, seed=99 + qt, subnormal_frac=0.25)
    want = dequantize(blocks, gt).reshape(-1).astype(np.float32)
    mine = oracle.dequantize(qt, blocks, want.size)
    assert np.array_equal(mine.view(np.uint32), want.view(np.uint32))


def test_decode_f16_all_bit_patterns():
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([oracle.decode_f16(int(b)) for b in bits], dtype=np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


def test_encode_f16_round_to_nearest_even():
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(4000) * 10.0 ** rng.integers(-9, 5, 4000), [0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8, 3e-8]]).astype(np.float32)
    want = x.astype(np.float16).view(np.uint16)
    got = np.array([oracle.encode_f16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(got, want)


def test_gemv_shader_rejects_reference_contract_violations():
    b = quant.random_blocks(quant.Q4_K, 6, 256, seed=1)
    with pytest.raises(ValueError):
        oracle.gemv_shader(quant.Q4_K, 6, 256, b, np.zeros(256, np.float32))      # rows % 4
    b = quant.random_blocks(quant.Q6_K, 4, 256, seed=1)
    with pytest.raises(ValueError):
        oracle.gemv_shader(quant.Q6_K, 4, 256, b, np.zeros(256, np.float32))      # Q6_K pairs need cols % 512


def test_rms_norm_silu_add_argmax():
    rng = np.random.default_rng(11)
    n = 1757                                                     # the reference's test length (ops/rms_norm.rs:103)
    x, w = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    for eps in (1e-4, 1e-5):
        want = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean() + eps) * w
        assert np.allclose(oracle.rms_norm(x, w, eps), want, rtol=2e-6, atol=1e-7)
    h1, h2 = rng.standard_normal(n).astype(np.float32) * 4, rng.standard_normal(n).astype(np.float32)
    want = h2.astype(np.float64) * (h1.astype(np.float64) / (1 + np.exp(-h1.astype(np.float64))))
    assert np.allclose(oracle.silu_mul(h1, h2), want, rtol=2e-6, atol=1e-7)
    assert np.array_equal(oracle.add_assign(x, w), x + w)
    y = np.array([1.0, 5.0, -2.0, 5.0, 3.0], np.float32)
    assert oracle.argmax(y) == 1                                  # lowest index among equal maxima
    assert oracle.argmax(np.array([-3.0], np.float32)) == 0


@pytest.mark.parametrize("variant", [0, 1])
def test_rope_matches_closed_form(variant):
    # shapes of the reference's test: head 128, 13 query heads, 9 kv heads, pos 10, base 1e4 (ops/rope.rs:160-229)
    hs, nq, nk, pos, base = 128, 13, 9, 10, 1e4
    rng = np.random.default_rng(3)
    q, k = rng.standard_normal(hs * nq).astype(np.float32), rng.standard_normal(hs * nk).astype(np.float32)
    q2, k2 = oracle.rope(variant, q, k, hs, pos, base)

    def rot(v):
        v = v.astype(np.float64).reshape(-1, hs)
        out = v.copy()
        j = np.arange(hs // 2)
        ang = pos * base ** (-2.0 * j / hs)
        c, s = np.cos(ang), np.sin(ang)
        if variant == 0:
            a, b = v[:, 0::2], v[:, 1::2]
            out[:, 0::2], out[:, 1::2] = c * a - s * b, s * a + c * b
        else:
            a, b = v[:, : hs // 2], v[:, hs // 2:]
            out[:, : hs // 2], out[:, hs // 2:] = c * a - s * b, s * a + c * b
        return out.reshape(-1)

    assert np.allclose(q2, rot(q), atol=2e-5)
    assert np.allclose(k2, rot(k), atol=2e-5)
    # q beyond kv_dim is still rotated, k has no entries there
    assert not np.allclose(q2[hs * nk:], q[hs * nk:])


@pytest.mark.parametrize("kv_dtype", [np.float32, np.float16])
def test_attention_matches_closed_form(kv_dtype):
    rng = np.random.default_rng(8)
    hs, n_heads, kv_mul, pos, seq = 64, 8, 4, 37, 64
    kv_dim = n_heads // kv_mul * hs
    q = rng.standard_normal(n_heads * hs).astype(np.float32)
    kc = rng.standard_normal((seq, kv_dim)).astype(kv_dtype)
    vc = rng.standard_normal((seq, kv_dim)).astype(kv_dtype)
    got = oracle.attention(q, kc, vc, n_heads=n_heads, kv_mul=kv_mul, head_size=hs, pos=pos)
    want = np.empty_like(got, dtype=np.float64)
    for h in range(n_heads):
        g = h // kv_mul
        K = kc[: pos + 1, g * hs:(g + 1) * hs].astype(np.float64)
        V = vc[: pos + 1, g * hs:(g + 1) * hs].astype(np.float64)
        s = K @ q[h * hs:(h + 1) * hs].astype(np.float64) / np.sqrt(np.float32(hs))
        p = np.exp(s - s.max())
        want[h * hs:(h + 1) * hs] = (p / p.sum()) @ V
    assert np.allclose(got, want, rtol=1e-6, atol=1e-6)
    # rows after pos must not matter
    kc2, vc2 = kc.copy(), vc.copy()
    kc2[pos + 1:] = 1e4
    vc2[pos + 1:] = -1e4
    assert np.array_equal(got, oracle.attention(q, kc2, vc2, n_heads=n_heads, kv_mul=kv_mul, head_size=hs, pos=pos))


@pytest.mark.parametrize("qwen2", [False, True])
def test_llama_forward_matches_numpy_restatement(qwen2):
    """Whole-model oracle vs a dequantize-everything numpy forward in the op order of transformer.rs:418-478; the Qwen2 variant
    adds q / k / v biases before a NeoX rotation (transformer.rs:434-445, crates/inferi-shaders/src/rope.rs:97-141)."""
    import torch
    from inferi_b200.llama2 import Llama2Config, synth_weights, weights_to_host

    cfg = Llama2Config(256, 512, 2, 4, 2, 512, 16, 500000.0, 1e-5)
    recipe = {n: quant.Q4_K for n in ("attn_q", "attn_k", "attn_output", "ffn_gate", "ffn_up", "token_embd")}
    recipe.update(attn_v=quant.Q8_0, ffn_down=quant.Q5_K, output=quant.Q6_K)
    w = weights_to_host(synth_weights(cfg, seed=21, recipe=recipe, qkv_bias=qwen2))
    ocfg = dict(hidden=256, ffn=512, n_layers=2, n_heads=4, n_kv_heads=2, vocab=512, max_pos=16, rope_theta=500000.0, rms_eps=1e-5,
                rope_variant=int(qwen2))
    m = oracle.Llama(ocfg, w, kv_f16=False)
    sh = cfg.shapes()

    def deq(name, t):
        return oracle.dequantize(t[0], t[1], sh[name][0] * sh[name][1]).reshape(sh[name]).astype(np.float64)

    D = [{n: deq(n, lw[n]) for n in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")} for lw in w["layers"]]
    E, O = deq("token_embd", w["token_embd"]), deq("output", w["output"])
    hs, kvm = cfg.head_size, cfg.kv_mul
    kc = [np.zeros((16, cfg.kv_dim)) for _ in range(2)]
    vc = [np.zeros((16, cfg.kv_dim)) for _ in range(2)]

    def norm(x, g):
        return x / np.sqrt((x * x).mean() + 1e-5) * g

    def rope(v, pos):
        v = v.reshape(-1, hs).copy()
        ang = pos * 500000.0 ** (-2.0 * np.arange(hs // 2) / hs)
        c, s = np.cos(ang), np.sin(ang)
        if qwen2:
            a, b = v[:, :hs // 2].copy(), v[:, hs // 2:].copy()
            v[:, :hs // 2], v[:, hs // 2:] = c * a - s * b, s * a + c * b
        else:
            a, b = v[:, 0::2].copy(), v[:, 1::2].copy()
            v[:, 0::2], v[:, 1::2] = c * a - s * b, s * a + c * b
        return v.reshape(-1)

    def bias(l, n):
        return w["layers"][l][n].astype(np.float64) if qwen2 else 0.0

    tokens = [5, 77, 300, 12]
    for pos, tok in enumerate(tokens):
        x = E[tok].copy()
        for l in range(2):
            xb = norm(x, w["layers"][l]["attn_norm"])
            q, k = rope(D[l]["attn_q"] @ xb + bias(l, "attn_q_bias"), pos), rope(D[l]["attn_k"] @ xb + bias(l, "attn_k_bias"), pos)
            v = D[l]["attn_v"] @ xb + bias(l, "attn_v_bias")
            kc[l][pos], vc[l][pos] = k, v
            att = np.zeros(cfg.hidden_size)
            for h in range(4):
                g = h // kvm
                s = kc[l][: pos + 1, g * hs:(g + 1) * hs] @ q[h * hs:(h + 1) * hs] / np.sqrt(hs)
                p = np.exp(s - s.max())
                att[h * hs:(h + 1) * hs] = (p / p.sum()) @ vc[l][: pos + 1, g * hs:(g + 1) * hs]
            x = x + D[l]["attn_output"] @ att
            xb = norm(x, w["layers"][l]["ffn_norm"])
            g_, u_ = D[l]["ffn_gate"] @ xb, D[l]["ffn_up"] @ xb
            x = x + D[l]["ffn_down"] @ (u_ * (g_ / (1 + np.exp(-g_))))
        want = O @ norm(x, w["output_norm"])
        got = m.forward(tok, pos)
        assert np.abs(got - want).max() <= 2e-5 * max(1.0, np.abs(want).max()), pos
    m.close()


def test_neox_rotation_equals_adjacent_rotation_of_reordered_rows():
    """What the device model relies on for the Qwen2 variant: reordering the rows of Wq, Wk and their biases inside each head as
    [0, h/2, 1, h/2+1, ...] and rotating adjacent pairs gives the logits of the NeoX rotation on the original rows."""
    from inferi_b200.llama2 import Llama2Config, synth_weights, weights_to_host

    cfg = Llama2Config(256, 512, 2, 4, 2, 512, 16, 500000.0, 1e-5)
    recipe = {n: quant.Q4_K for n in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down", "token_embd", "output")}
    w = weights_to_host(synth_weights(cfg, seed=5, recipe=recipe, qkv_bias=True))
    ocfg = dict(hidden=256, ffn=512, n_layers=2, n_heads=4, n_kv_heads=2, vocab=512, max_pos=16, rope_theta=500000.0, rms_eps=1e-5)
    hs = cfg.head_size
    order = np.array([(i // 2) + (hs // 2 if i & 1 else 0) for i in range(hs)])

    def reorder(a):
        a = np.asarray(a)
        idx = (np.arange(a.shape[0]) // hs * hs) + order[np.arange(a.shape[0]) % hs]
        return a[idx]

    w2 = dict(w, layers=[dict(lw, attn_q=(lw["attn_q"][0], reorder(lw["attn_q"][1])), attn_k=(lw["attn_k"][0], reorder(lw["attn_k"][1])),
                              attn_q_bias=reorder(lw["attn_q_bias"]), attn_k_bias=reorder(lw["attn_k_bias"])) for lw in w["layers"]])
    neox = oracle.Llama(dict(ocfg, rope_variant=1), w, kv_f16=False)
    adj = oracle.Llama(dict(ocfg, rope_variant=0), w2, kv_f16=False)
    for pos, tok in enumerate([9, 100, 31, 7, 480]):
        a, b = neox.forward(tok, pos), adj.forward(tok, pos)
        assert np.abs(a - b).max() <= 1e-5 * max(1.0, np.abs(a).max())
    neox.close()
    adj.close()


def _np_sample(logits, temperature, topp, coin):
    """numpy restatement of crates/inferi/src/models/sampler.rs:32-130 (sequential float32 sums via cumsum)."""
    if temperature == 0.0:
        return int(np.argmax(logits))
    x = (logits / np.float32(temperature)).astype(np.float32)
    e = np.exp(x - x.max()).astype(np.float32)
    p = (e / np.cumsum(e, dtype=np.float32)[-1]).astype(np.float32)
    if topp <= 0.0 or topp >= 1.0:
        cdf = np.cumsum(p, dtype=np.float32)
        hit = np.nonzero(np.float32(coin) < cdf)[0]
        return int(hit[0]) if hit.size else p.size - 1
    cutoff = np.float32((np.float32(1.0) - np.float32(topp)) / (np.float32(p.size) - np.float32(1.0)))
    idx = np.nonzero(p >= cutoff)[0]
    order = idx[np.argsort(-p[idx], kind="stable")]
    cum = np.cumsum(p[order], dtype=np.float32)
    over = np.nonzero(cum > np.float32(topp))[0]
    last = int(over[0]) if over.size else order.size - 1
    r = np.float32(coin) * cum[last]
    hit = np.nonzero(r < cum[:last + 1])[0]
    return int(order[hit[0]]) if hit.size else int(order[last])


@pytest.mark.parametrize("temperature,topp", [(0.0, 0.9), (1.0, 0.0), (0.7, 1.0), (1.0, 0.9), (0.5, 0.3), (1.3, 0.99)])
def test_sampler_restatement(temperature, topp):
    rng = np.random.default_rng(int(temperature * 10) + int(topp * 100))
    for n in (2, 17, 1000, 20000):
        logits = (rng.standard_normal(n) * 2.5).astype(np.float32)
        for coin in np.concatenate([rng.random(8).astype(np.float32), np.float32([0.0, 0.9999999])]):
            tok, margin = oracle.sample(logits, temperature, topp, float(coin))
            want = _np_sample(logits, temperature, topp, float(coin))
            assert tok == want or margin < 1e-6      # libm expf vs numpy exp may differ in the last bit


def test_sample_coin_is_a_function_of_seed_and_position():
    c = [oracle.sample_coin(42, p) for p in range(2000)]
    assert all(0.0 <= v < 1.0 for v in c) and len(set(c)) > 1990
    assert c == [oracle.sample_coin(42, p) for p in range(2000)] and c[:5] != [oracle.sample_coin(43, p) for p in range(5)]
    assert abs(np.mean(c) - 0.5) < 0.03
