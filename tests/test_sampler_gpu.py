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


def valid_within_rounding(logits, temperature, topp, coin, got, tol):
    """Is `got` what the reference algorithm picks when every running sum may be off by `tol`?  Recomputed in float64."""
    x = logits.astype(np.float64) / temperature
    p = np.exp(x - x.max())
    p /= p.sum()
    n = p.size
    if topp <= 0.0 or topp >= 1.0:
        cdf = np.cumsum(p)
        lo = cdf[got - 1] if got else 0.0
        return lo - tol <= coin < cdf[got] + tol or (got == n - 1 and coin >= cdf[-1] - tol)
    cutoff = (1.0 - topp) / (n - 1.0)
    cand = np.flatnonzero(p >= cutoff * (1 - 1e-6))
    if got not in cand:
        return False
    pc = np.sort(p[cand])[::-1]
    cum = np.cumsum(pc)
    # Tokens whose f32 probabilities are equal or a few ulps apart may be ordered either way (the sort sees f32 values, ties go by
    # index): `got` sits somewhere between the tokens clearly above it and the tokens clearly below it.
    eps = 1e-6
    k_min = int(np.count_nonzero(pc > p[got] * (1 + eps)))
    k_max = int(np.count_nonzero(pc >= p[got] * (1 - eps))) - 1
    lo_min = cum[k_min - 1] if k_min else 0.0
    hi_max = cum[k_max]
    # every place the nucleus may end when the comparison with topp is taken with a rounding error
    ends = [i for i in range(cum.size) if cum[i] > topp - tol and (i == 0 or cum[i - 1] <= topp + tol)] or [cum.size - 1]
    for last in ends:
        if k_min > last:
            continue
        r = coin * cum[last]
        if lo_min - tol <= r < hi_max + tol or (k_max >= last and r >= lo_min - tol):
            return True
    return False


def check_many(backend, logits, temperature, topp, coins):
    """Identical tokens, except where a running sum in another order may decide otherwise: the reference adds n probabilities
    one by one in f32, the device adds per-thread chunks and scans them; both are within ~sqrt(n) * 2^-24 of the exact sum, and
    a coin that close to the boundary between two tokens may fall on either side."""
    tol = 2e-6 + 8.0 * np.sqrt(logits.size) * 2.0 ** -24
    for coin in coins:
        want, margin = oracle.sample(logits, temperature, topp, float(coin))
        got = gpu_sample(backend, logits, temperature, topp, float(coin))
        if got != want:
            assert margin < tol, f"T={temperature} topp={topp} coin={coin}: {got} vs {want} (margin {margin}, allowed {tol})"
            assert valid_within_rounding(logits, temperature, topp, float(coin), got, tol), f"T={temperature} topp={topp} coin={coin}: {got} is not a neighbour of {want}"


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
    recipe = dict(attn_q=quant.Q4_K, attn_k=quant.Q4_K, attn_v=quant.Q8_0, attn_output=quant.Q4_K, ffn_gate=quant.Q4_K, ffn_up=quant.Q4_K,
                  ffn_down=quant.Q6_K, token_embd=quant.Q4_K, output=quant.Q8_0)
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
