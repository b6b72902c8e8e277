"""On-device sampling (temperature, multinomial, top-p) against the oracle's restatement of the reference's CPU sampler."""
import numpy as np
import pytest
import torch

import oracle
from inferi_b200 import quant
from inferi_b200.llama2 import Llama2, Llama2Config, Llama2Weights, synth_weights, weights_to_host
from inferi_b200.ops import InferiError, Sampler

pytestmark = pytest.mark.gpu


def gpu_sample(backend, logits, temperature, topp, coin):
    s = Sampler(backend, logits.size, temperature, topp)
    out = s.sample(torch.from_numpy(logits).cuda(), coin)
    torch.cuda.synchronize()
    return int(out.item())


def check_many(backend, logits, temperature, topp, coins):
    close_calls = 0
    for coin in coins:
        want, margin = oracle.sample(logits, temperature, topp, float(coin))
        got = gpu_sample(backend, logits, temperature, topp, float(coin))
        if got != want:
            # a parallel sum differs from the sequential one in the last bits: only a coin on a boundary may decide otherwise
            assert margin < 2e-6, f"T={temperature} topp={topp} coin={coin}: {got} vs {want} (margin {margin})"
            close_calls += 1
    assert close_calls <= max(1, len(coins) // 20)


@pytest.mark.parametrize("n", [2, 50, 1000, 4097, 32000, 128256])
@pytest.mark.parametrize("temperature,topp", [(1.0, 0.0), (0.7, 1.0), (1.0, 0.9), (0.5, 0.5), (1.5, 0.95), (1.0, 0.05)])
def test_sampler_matches_the_reference_algorithm(backend, n, temperature, topp):
    rng = np.random.default_rng(n * 7 + int(temperature * 10) + int(topp * 100))
    logits = (rng.standard_normal(n) * 3.0).astype(np.float32)        # peaked: a nucleus of a few hundred tokens
    coins = np.concatenate([rng.random(10).astype(np.float32), np.float32([0.0, 0.999999])])
    check_many(backend, logits, temperature, topp, coins)


def test_flat_and_tied_distributions(backend):
    """Near-uniform logits put the whole vocabulary into the nucleus (the global-memory sort path); equal probabilities
    must be taken in index order (the reference's stable sort)."""
    rng = np.random.default_rng(5)
    n = 40000
    flat = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    check_many(backend, flat, 1.0, 0.9, rng.random(6).astype(np.float32))
    tied = np.zeros(512, dtype=np.float32)
    tied[[7, 300, 301]] = 5.0                                           # three equal winners
    for coin in (0.0, 0.2, 0.4, 0.6, 0.9):
        assert gpu_sample(backend, tied, 1.0, 0.9, coin) == oracle.sample(tied, 1.0, 0.9, coin)[0]


def test_temperature_zero_is_argmax_and_contract(backend):
    x = np.float32([0.1, 3.0, -1.0, 3.0, 2.0])
    assert gpu_sample(backend, x, 0.0, 0.9, 0.5) == 1                   # greedy, lowest index on ties
    with pytest.raises(InferiError):
        gpu_sample(backend, x, 1.0, 0.9, 1.0)                           # coin outside [0, 1)
    with pytest.raises(InferiError):
        gpu_sample(backend, x, -1.0, 0.9, 0.5)


def test_model_loop_with_sampling(backend):
    """The model's own loop with a sampler: every fed-back token must be what the reference's sampler picks from the
    oracle's logits with the same coin, and a run is reproducible from its seed."""
    cfg = Llama2Config(256, 2048, 2, 4, 2, 512, 64, 500000.0, 1e-5)
    recipe = dict(attn_q=quant.Q4_K, attn_k=quant.Q4_K, attn_v=quant.Q6_K, attn_output=quant.Q4_K, ffn_gate=quant.Q4_K, ffn_up=quant.Q4_K,
                  ffn_down=quant.Q6_K, token_embd=quant.Q4_K, output=quant.Q6_K)
    w = synth_weights(cfg, seed=77, recipe=recipe, std=0.1)             # larger weights: a distribution with some shape
    model = Llama2(backend, cfg, Llama2Weights(backend, cfg, w), kv_f16=True)
    temperature, topp, seed = 0.8, 0.9, 1234
    model.set_sampler(temperature, topp, seed)
    prompt, n_gen = [3, 99, 7], 24
    got = model.generate(prompt, n_gen).tolist()
    again = model.generate(prompt, n_gen).tolist()
    assert got == again                                                 # same seed, same positions, same tokens
    ref = oracle.Llama(dict(hidden=256, ffn=2048, n_layers=2, n_heads=4, n_kv_heads=2, vocab=512, max_pos=64, rope_theta=500000.0, rms_eps=1e-5),
                       weights_to_host(w), kv_f16=True)
    seq = list(prompt)
    for pos in range(len(prompt) + n_gen - 1):
        lg = ref.forward(seq[pos], pos)
        if pos >= len(prompt) - 1:
            tok, margin = oracle.sample(lg, temperature, topp, oracle.sample_coin(seed, pos))
            g = got[pos - len(prompt) + 1]
            if g != tok:
                assert margin < 1e-4, f"position {pos}: {g} vs {tok} (margin {margin})"   # logits differ by ~1e-5: a coin on a boundary
                tok = g                                                  # follow the device's branch
            seq.append(tok)
    ref.close()
    model.set_sampler(0.0)                                              # greedy again
    greedy = model.generate(prompt, 4).tolist()
    model.set_sampler(temperature, topp, seed + 1)
    assert model.generate(prompt, n_gen).tolist() != got                # another seed, another sequence
    model.set_sampler(0.0)
    assert model.generate(prompt, 4).tolist() == greedy
    model.close()
