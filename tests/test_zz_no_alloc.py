"""The allocation-free attention entry point against the allocating one.

`ib_attention_static` exists for callers that may not allocate device memory when they call into the library (a
latency-critical thread, a plugin inside a host that owns the memory budget).  It must give what `ib_attention` gives,
on a first call and on a second one that finds the built-in scratch array as the first left it.  The file name sorts
last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close
from inferi_b200 import _lib
from inferi_b200.ops import AttnParams, FusedAttention

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("hs,n_heads,kv_mul,pos,seq,dtype", [(128, 32, 4, 700, 1024, torch.float16), (64, 32, 4, 2300, 4096, torch.float32)])
def test_static_scratch_attention_matches_allocating_entry_point(backend, hs, n_heads, kv_mul, pos, seq, dtype):
    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(pos)
    kv_dim = n_heads // kv_mul * hs
    kc = torch.randn(seq, kv_dim, generator=g, device="cuda").to(dtype)
    vc = torch.randn(seq, kv_dim, generator=g, device="cuda").to(dtype)
    p = AttnParams(seq, kv_dim, kv_mul, n_heads, hs, pos)
    kv = _lib.KV_F16 if dtype == torch.float16 else _lib.KV_F32
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                      # two calls in a row share the built-in array
        q = torch.randn(n_heads * hs, generator=g, device="cuda")
        want = torch.empty(n_heads * hs, device="cuda")
        FusedAttention(backend).launch(p, q, kc, vc, want)
        got = torch.full((n_heads * hs,), float("nan"), device="cuda")
        _lib.check(lib.ib_attention_static(stream, C.byref(p), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), kv, got.data_ptr()))
        torch.cuda.synchronize()
        assert_close(got.cpu().numpy(), want.cpu().numpy(), what=f"static-scratch attention, call {call}")
        # and against the CPU oracle directly: the two entry points split the positions differently
        ref = oracle.attention(q.cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy(), n_heads=n_heads, kv_mul=kv_mul, head_size=hs, pos=pos)
        assert_close(got.cpu().numpy(), ref, what=f"static-scratch attention vs oracle, call {call}")


def test_static_scratch_attention_rejects_what_does_not_fit(backend):
    lib = _lib.load()
    z = torch.zeros(8, device="cuda")
    p = AttnParams(16, 2048 * 128, 1, 2048, 128, 3)      # 2048 heads of 128: 266 240 floats per split > 262 144
    rc = lib.ib_attention_static(None, C.byref(p), z.data_ptr(), z.data_ptr(), z.data_ptr(), _lib.KV_F32, z.data_ptr())
    assert rc == 4 and b"exceed the built-in scratch" in lib.ib_last_error_string()
    assert lib.ib_attention_static(None, None, None, None, None, 0, None) == 1
