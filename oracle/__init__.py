"""ctypes front-end of the CPU oracle (`inferi_oracle.c`).

TEST INFRASTRUCTURE ONLY: imported by `tests/`, by `__graft_entry__.smoke()` and by the CPU-baseline legs of
`bench.py`, always as the checker or the timed CPU baseline — never by the `inferi_b200` package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")

F32, Q8_0, Q4_K, Q5_K, Q6_K = 0, 8, 12, 13, 14
W_Q, W_K, W_V, W_O, W_GATE, W_UP, W_DOWN = range(7)


def build(force: bool = False) -> str:
    """Compile liboracle.so with the Makefile beside this file (gcc, OpenMP)."""
    src = os.path.join(_HERE, "inferi_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return _SO


class AttnParams(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("seq_len", "kv_dim", "kv_mul", "n_heads", "head_size", "pos")]


class LlamaConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("hidden", "ffn", "n_layers", "n_heads", "n_kv_heads", "vocab", "max_pos")] + [
        ("rope_theta", C.c_float), ("rms_eps", C.c_float)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        L.orc_block_bytes.restype = C.c_size_t
        L.orc_block_elems.restype = C.c_size_t
        L.orc_decode_f16.restype = C.c_float
        L.orc_decode_f16.argtypes = [C.c_uint16]
        L.orc_encode_f16.restype = C.c_uint16
        L.orc_encode_f16.argtypes = [C.c_float]
        L.orc_dequantize.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
        for f in (L.orc_gemv_ref, L.orc_gemv_shader):
            f.argtypes = [C.c_int, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.orc_rms_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_float]
        L.orc_rope.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint32, C.c_float]
        L.orc_silu_mul.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.orc_add_assign.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.orc_argmax.restype = C.c_uint32
        L.orc_argmax.argtypes = [C.c_void_p, C.c_size_t]
        L.orc_attention.argtypes = [C.POINTER(AttnParams), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.orc_llama_create.restype = C.c_void_p
        L.orc_llama_create.argtypes = [C.POINTER(LlamaConfig), C.c_int, C.c_int]
        L.orc_llama_set_mat.argtypes = [C.c_void_p, C.c_uint32, C.c_int, C.c_int, C.c_void_p]
        L.orc_llama_set_norms.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
        L.orc_llama_set_globals.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        L.orc_llama_free.argtypes = [C.c_void_p]
        L.orc_llama_set_variant.argtypes = [C.c_void_p, C.c_int]
        L.orc_llama_set_bias.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_llama_set_gemv_mode.argtypes = [C.c_void_p, C.c_int]
        L.orc_llama_forward.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p]
        L.orc_llama_hidden.restype = C.POINTER(C.c_float)
        L.orc_llama_hidden.argtypes = [C.c_void_p]
        L.orc_max_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def max_threads() -> int:
    return int(lib().orc_max_threads())


def decode_f16(h: int) -> float:
    return float(lib().orc_decode_f16(h))


def encode_f16(f: float) -> int:
    return int(lib().orc_encode_f16(f))


def dequantize(qtype: int, blocks: np.ndarray, n_elems: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    be, bb = lib().orc_block_elems(qtype), lib().orc_block_bytes(qtype)
    assert n_elems % be == 0 and blocks.size == n_elems // be * bb
    out = np.empty(n_elems, dtype=np.float32)
    assert lib().orc_dequantize(qtype, _p(blocks), n_elems // be, _p(out)) == 0
    return out


def _gemv(fn, qtype, rows, cols, blocks, v, nthreads):
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    v = _f32(v)
    assert v.size == cols
    out = np.empty(rows, dtype=np.float32)
    rc = fn(qtype, rows, cols, _p(blocks), _p(v), _p(out), nthreads)
    if rc != 0:
        raise ValueError("oracle gemv rejected the shape")
    return out


def gemv_ref(qtype, rows, cols, blocks, v, nthreads=None):
    """dequantize + f64 dot: the definition every GEMV is checked against."""
    return _gemv(lib().orc_gemv_ref, qtype, rows, cols, blocks, v, nthreads or max_threads())


def gemv_shader(qtype, rows, cols, blocks, v, nthreads=None):
    """lane-structured restatement of the reference shaders (f32 partials + tree); the timed CPU baseline."""
    return _gemv(lib().orc_gemv_shader, qtype, rows, cols, blocks, v, nthreads or max_threads())


def rms_norm(x, w, eps):
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    lib().orc_rms_norm(_p(out), _p(x), _p(w), x.size, eps)
    return out


def rope(variant, q, k, head_size, pos, base_freq):
    """Returns rotated copies (q, k)."""
    q, k = _f32(q).copy(), _f32(k).copy()
    lib().orc_rope(variant, _p(q), q.size, _p(k), k.size, head_size, pos, base_freq)
    return q, k


def silu_mul(h1, h2):
    h1, h2 = _f32(h1).copy(), _f32(h2)
    lib().orc_silu_mul(_p(h1), _p(h2), h1.size)
    return h1


def add_assign(a, b):
    a, b = _f32(a).copy(), _f32(b)
    lib().orc_add_assign(_p(a), _p(b), a.size)
    return a


def argmax(x) -> int:
    x = _f32(x)
    return int(lib().orc_argmax(_p(x), x.size))


def sample_coin(seed: int, pos: int) -> float:
    f = lib().orc_sample_coin
    f.restype, f.argtypes = C.c_float, [C.c_uint64, C.c_uint32]
    return float(f(seed, pos))


def sample(logits, temperature: float, topp: float, coin: float):
    """(token, margin): the reference's Sampler::sample with the given coin; margin = distance of the decision to its threshold."""
    x = _f32(logits)
    f = lib().orc_sample
    f.restype, f.argtypes = C.c_uint32, [C.c_void_p, C.c_size_t, C.c_float, C.c_float, C.c_float, C.POINTER(C.c_float)]
    m = C.c_float()
    tok = f(_p(x), x.size, temperature, topp, coin, C.byref(m))
    return int(tok), float(m.value)


def attention(q, k_cache, v_cache, *, n_heads, kv_mul, head_size, pos, seq_len=None):
    """k_cache / v_cache: [>=pos+1, kv_dim] float32 or float16 arrays."""
    q = _f32(q)
    kv_f16 = k_cache.dtype == np.float16
    k_cache = np.ascontiguousarray(k_cache)
    v_cache = np.ascontiguousarray(v_cache)
    assert v_cache.dtype == k_cache.dtype and k_cache.dtype in (np.float16, np.float32)
    kv_dim = k_cache.shape[1]
    p = AttnParams(seq_len or k_cache.shape[0], kv_dim, kv_mul, n_heads, head_size, pos)
    out = np.empty(n_heads * head_size, dtype=np.float32)
    lib().orc_attention(C.byref(p), _p(q), _p(k_cache), _p(v_cache), int(kv_f16), _p(out))
    return out


class Llama:
    """Whole-model CPU forward in the op order of crates/inferi/src/models/llama2/transformer.rs:418-478."""

    def __init__(self, cfg: dict, weights: dict, kv_f16: bool, nthreads: int | None = None):
        """cfg keys = LlamaConfig fields, plus optionally 'rope_variant' (0 Original, 1 NeoX); weights: {'layers':
        [{'attn_q': (qtype, uint8 array), ..., 'attn_norm': f32, 'ffn_norm': f32, optionally 'attn_q_bias' / 'attn_k_bias' /
        'attn_v_bias': f32}], 'token_embd': (qtype, arr), 'output': (qtype, arr) | None, 'output_norm': f32}."""
        cfg = dict(cfg)
        rope_variant = int(cfg.pop("rope_variant", 0))
        self.cfg = LlamaConfig(**cfg)
        self._keep = []
        self.vocab = cfg["vocab"]
        self.hidden = cfg["hidden"]
        self.h = lib().orc_llama_create(C.byref(self.cfg), int(kv_f16), nthreads or max_threads())
        lib().orc_llama_set_variant(self.h, rope_variant)
        names = ["attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"]
        for l, lw in enumerate(weights["layers"]):
            biases = [(_f32(lw[n]) if lw.get(n) is not None else None) for n in ("attn_q_bias", "attn_k_bias", "attn_v_bias")]
            if any(b is not None for b in biases):
                self._keep += [b for b in biases if b is not None]
                lib().orc_llama_set_bias(self.h, l, *[(_p(b) if b is not None else None) for b in biases])
            for which, n in enumerate(names):
                qt, arr = lw[n]
                arr = np.ascontiguousarray(arr, dtype=np.uint8)
                self._keep.append(arr)
                lib().orc_llama_set_mat(self.h, l, which, qt, _p(arr))
            an, fn = _f32(lw["attn_norm"]), _f32(lw["ffn_norm"])
            self._keep += [an, fn]
            lib().orc_llama_set_norms(self.h, l, _p(an), _p(fn))
        eq, ea = weights["token_embd"]
        ea = np.ascontiguousarray(ea, dtype=np.uint8)
        on = _f32(weights["output_norm"])
        self._keep += [ea, on]
        if weights.get("output") is not None:
            oq, oa = weights["output"]
            oa = np.ascontiguousarray(oa, dtype=np.uint8)
            self._keep.append(oa)
            lib().orc_llama_set_globals(self.h, eq, _p(ea), oq, _p(oa), _p(on))
        else:
            lib().orc_llama_set_globals(self.h, eq, _p(ea), 0, None, _p(on))

    def forward(self, token: int, pos: int, want_logits: bool = True):
        if want_logits:
            logits = np.empty(self.vocab, dtype=np.float32)
            lib().orc_llama_forward(self.h, token, pos, _p(logits))
            return logits
        lib().orc_llama_forward(self.h, token, pos, None)
        return None

    def set_gemv_mode(self, shader_structured: bool) -> None:
        """True: every GEMV runs the lane-structured f32 shader restatement (CPU baseline); False: dequantize + f64 dot."""
        lib().orc_llama_set_gemv_mode(self.h, int(shader_structured))

    def hidden_state(self) -> np.ndarray:
        return np.ctypeslib.as_array(lib().orc_llama_hidden(self.h), shape=(self.hidden,)).copy()

    def close(self):
        if self.h:
            lib().orc_llama_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
