"""GPU parity of RMSNorm, RoPE, SwiGLU, residual add, arg-max and decode attention against the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close
from inferi_b200 import ops, quant
from inferi_b200.ops import AttnParams, FusedAttention, InferiError, RmsNorm, RmsNormConfig, RoPE, RoPEConfig, Silu

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("n,eps", [(1757, 1e-4), (4096, 1e-5), (2048, 1e-5), (1, 1e-6), (14336, 1e-5)])
def test_rms_norm(backend, n, eps):
    rng = np.random.default_rng(n)
    x, w = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    out = torch.empty(n, device="cuda")
    RmsNorm.from_backend(backend).launch(RmsNormConfig(eps), out, dev(x), dev(w))
    assert_close(out.cpu().numpy(), oracle.rms_norm(x, w, eps), what="rms_norm")


@pytest.mark.parametrize("n", [1757, 8192, 14336, 3])
def test_silu_and_add(backend, n):
    rng = np.random.default_rng(n)
    h1, h2 = (rng.standard_normal(n) * 4).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    d1 = dev(h1)
    Silu.from_backend(backend).launch(d1, dev(h2))
    assert_close(d1.cpu().numpy(), oracle.silu_mul(h1, h2), what="silu")
    a = dev(h1)
    ops.add_assign(backend, a, dev(h2))
    assert np.array_equal(a.cpu().numpy(), oracle.add_assign(h1, h2))


@pytest.mark.parametrize("variant", [ops.ROPE_ORIGINAL, ops.ROPE_NEOX])
@pytest.mark.parametrize("hs,nq,nk,pos,base", [(128, 13, 9, 10, 1e4), (64, 32, 8, 4095, 5e5), (128, 32, 8, 32767, 5e5), (128, 4, 4, 0, 5e5)])
def test_rope(backend, variant, hs, nq, nk, pos, base):
    rng = np.random.default_rng(pos + hs)
    q, k = rng.standard_normal(hs * nq).astype(np.float32), rng.standard_normal(hs * nk).astype(np.float32)
    dq, dk = dev(q), dev(k)
    RoPE.from_backend(backend).launch(variant, RoPEConfig(hs, hs * nk, pos, base), dq, dk)
    q2, k2 = oracle.rope(variant, q, k, hs, pos, base)
    # angles reach 3e4 rad: one ulp of the f32 angle is 2e-3 rad there, so compare on the vector's scale
    assert np.abs(dq.cpu().numpy() - q2).max() <= 1e-3 * np.abs(q2).max()
    assert np.abs(dk.cpu().numpy() - k2).max() <= 1e-3 * np.abs(k2).max()
    if pos < 100:
        assert_close(dq.cpu().numpy(), q2, rtol=1e-5, what="rope q")


def test_rope_contract(backend):
    q, k = torch.zeros(127, device="cuda"), torch.zeros(64, device="cuda")
    with pytest.raises(InferiError):
        RoPE(backend).launch(ops.ROPE_ORIGINAL, RoPEConfig(64, 64, 0, 1e4), q, k)   # odd q_len
    with pytest.raises(InferiError):
        RoPE(backend).launch(ops.ROPE_ORIGINAL, RoPEConfig(64, 128, 0, 1e4), torch.zeros(64, device="cuda"), torch.zeros(128, device="cuda"))


@pytest.mark.parametrize("n", [1, 7, 128256, 1000003])
def test_argmax(backend, n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float32)
    if n > 100:
        x[[n // 3, n // 2, n - 1]] = x.max() + 1.0        # three equal maxima: the lowest index wins
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):                                     # twice: the arrival counter must reset itself
        ops.argmax(backend, dev(x), out)
        assert int(out.item()) == oracle.argmax(x)
    y = -np.abs(x) - 1.0                                   # all negative
    ops.argmax(backend, dev(y), out)
    assert int(out.item()) == oracle.argmax(y)


ATTN_CASES = [
    # hs, n_heads, kv_mul, pos, seq_len
    (64, 32, 4, 0, 64), (64, 32, 4, 33, 64), (64, 32, 4, 2047, 2048), (64, 32, 4, 2048, 4096),
    (128, 32, 4, 1, 16), (128, 32, 4, 640, 1024), (128, 32, 4, 4095, 4096),
    (128, 8, 1, 100, 128), (128, 16, 2, 300, 512), (64, 16, 8, 77, 128), (128, 4, 4, 513, 1024),
    (128, 32, 4, 31, 64), (128, 32, 4, 32, 64), (128, 32, 4, 190, 256), (64, 32, 4, 7, 16), (64, 32, 4, 255, 256),
    # head size 64 with few kv heads and long contexts: the slice count meets its cap (2 * head_size), the merge step's staging is full
    (64, 8, 4, 16500, 16640), (64, 16, 4, 9000, 9216), (64, 4, 1, 16384, 16400), (64, 4, 2, 8600, 8704), (128, 4, 4, 20000, 20480),
]


@pytest.mark.parametrize("kv_dtype", [np.float16, np.float32])
@pytest.mark.parametrize("hs,n_heads,kv_mul,pos,seq", ATTN_CASES)
def test_attention(backend, kv_dtype, hs, n_heads, kv_mul, pos, seq):
    rng = np.random.default_rng(pos * 7 + hs)
    kv_dim = n_heads // kv_mul * hs
    q = rng.standard_normal(n_heads * hs).astype(np.float32)
    kc = rng.standard_normal((seq, kv_dim)).astype(kv_dtype)
    vc = rng.standard_normal((seq, kv_dim)).astype(kv_dtype)
    kc[pos + 1:] = 1e4    # rows beyond pos must never be read into the result
    vc[pos + 1:] = -1e4
    out = torch.full((n_heads * hs,), float("nan"), device="cuda")
    p = AttnParams(seq, kv_dim, kv_mul, n_heads, hs, pos)
    att = FusedAttention.from_backend(backend)
    for _ in range(2):    # twice: split counters reset themselves
        att.launch(p, dev(q), dev(kc), dev(vc), out)
        ref = oracle.attention(q, kc, vc, n_heads=n_heads, kv_mul=kv_mul, head_size=hs, pos=pos)
        assert_close(out.cpu().numpy(), ref, what=f"attention hs={hs} pos={pos}")


@pytest.mark.parametrize("ctx_len", [8192, 16384, 32768])
def test_long_context_attention(backend, ctx_len):
    """Long-context stress: 32 query / 8 kv heads of 128, f16 cache from N(0,1), RoPE on q and on every k row."""
    hs, n_heads, kv_mul = 128, 32, 4
    kv_dim = n_heads // kv_mul * hs
    g = torch.Generator(device="cuda").manual_seed(5001)
    kc = torch.randn(ctx_len, kv_dim, generator=g, device="cuda")
    vc = torch.randn(ctx_len, kv_dim, generator=g, device="cuda").half()
    q = torch.randn(n_heads * hs, generator=g, device="cuda")
    # RoPE through the library itself, row by row position (vectorised with torch for speed: same formula)
    j = torch.arange(hs // 2, device="cuda", dtype=torch.float32)
    theta = torch.tensor([float(np.float32(5e5) ** np.float32(-2.0 * i / hs)) for i in range(hs // 2)], device="cuda")
    ang = torch.arange(ctx_len, device="cuda", dtype=torch.float32)[:, None] * theta[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    k4 = kc.view(ctx_len, -1, hs // 2, 2)
    a, b = k4[..., 0].clone(), k4[..., 1].clone()
    k4[..., 0], k4[..., 1] = c * a - s * b, s * a + c * b
    kc = kc.half()
    RoPE(backend).launch(ops.ROPE_ORIGINAL, RoPEConfig(hs, kv_dim, ctx_len - 1, 5e5), q, torch.zeros(kv_dim, device="cuda"))
    out = torch.empty(n_heads * hs, device="cuda")
    FusedAttention(backend).launch(AttnParams(ctx_len, kv_dim, kv_mul, n_heads, hs, ctx_len - 1), q, kc, vc, out)
    ref = oracle.attention(q.cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy(), n_heads=n_heads, kv_mul=kv_mul, head_size=hs, pos=ctx_len - 1)
    assert_close(out.cpu().numpy(), ref, what=f"attention ctx={ctx_len}")
    # size-independent property: appending a copy of the whole cache (same keys, same values) leaves the output unchanged
    if ctx_len <= 16384:
        out2 = torch.empty_like(out)
        FusedAttention(backend).launch(AttnParams(2 * ctx_len, kv_dim, kv_mul, n_heads, hs, 2 * ctx_len - 1), q, torch.cat([kc, kc]), torch.cat([vc, vc]), out2)
        assert np.abs(out2.cpu().numpy() - out.cpu().numpy()).max() <= 1e-5


def test_attention_contract(backend):
    z = torch.zeros(64, device="cuda")
    kc = torch.zeros(16, 64, device="cuda")
    with pytest.raises(InferiError):   # head size 32 unsupported
        FusedAttention(backend).launch(AttnParams(16, 64, 1, 2, 32, 3), z, kc, kc, torch.zeros(64, device="cuda"))
    with pytest.raises(InferiError):   # pos outside the cache
        FusedAttention(backend).launch(AttnParams(16, 64, 1, 1, 64, 16), z, kc, kc, torch.zeros(64, device="cuda"))
    with pytest.raises(InferiError):   # mixed cache types
        FusedAttention(backend).launch(AttnParams(16, 64, 1, 1, 64, 3), z, kc, kc.half(), torch.zeros(64, device="cuda"))


@pytest.mark.parametrize("qt,rows,cols,norm", [(quant.Q4_K, 1024, 2048, True), (quant.Q4_K, 14336, 4096, True), (quant.Q6_K, 512, 4096, False), (quant.Q8_0, 256, 1024, True)])
def test_ffn_gate_up_is_norm_two_gemvs_and_silu(backend, qt, rows, cols, norm):
    """`ib_ffn_gate_up` against the op sequence it replaces (transformer.rs:454-464): rms_norm, two quantized GEMVs, silu."""
    from inferi_b200.ops import FfnGateUp, GpuQuantTensor
    rng = np.random.default_rng(rows + cols)
    gate_b = quant.random_blocks(qt, rows, cols, seed=rows, scale=0.05)
    up_b = quant.random_blocks(qt, rows, cols, seed=rows + 1, scale=0.05)
    x = rng.standard_normal(cols).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    gate, up = GpuQuantTensor(backend, qt, rows, cols, gate_b), GpuQuantTensor(backend, qt, rows, cols, up_b)
    out = torch.full((rows,), float("nan"), device="cuda")
    FfnGateUp(backend).launch(out, gate, up, dev(x), dev(w) if norm else None, 1e-5)
    torch.cuda.synchronize()
    xn = oracle.rms_norm(x, w, 1e-5) if norm else x
    h1 = oracle.gemv_ref(qt, rows, cols, gate_b, xn)
    h2 = oracle.gemv_ref(qt, rows, cols, up_b, xn)
    assert_close(out.cpu().numpy(), oracle.silu_mul(h1, h2), what="ffn gate/up")
    gate.close()
    up.close()
