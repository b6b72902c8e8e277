"""ctypes binding of libinferi_b200.so — the same C ABI (include/inferi_b200.h) a Rust `extern "C"` block binds.

There is no CPU path: if the shared library is missing or cannot be loaded, importing the ops fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libinferi_b200.so")

IB_OK = 0
STATUS_NAMES = {0: "IB_OK", 1: "IB_ERR_INVALID", 2: "IB_ERR_CUDA", 3: "IB_ERR_OOM", 4: "IB_ERR_UNSUPPORTED", 5: "IB_ERR_TIMEOUT", 6: "IB_ERR_COMM"}
KV_F32, KV_F16 = 0, 1
ROPE_ORIGINAL, ROPE_NEOX = 0, 1
TP_HANDLE_BYTES = 64


class InferiError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {message}")
        self.code = code
        self.message = message


class AttnParams(C.Structure):
    """= AttentionParams (crates/inferi-shaders/src/batched_multiquery_attention.rs:18-31)."""
    _fields_ = [(n, C.c_uint32) for n in ("seq_len", "kv_dim", "kv_mul", "n_heads", "head_size", "pos")]


class LlamaConfig(C.Structure):
    """= Llama2Config (crates/inferi/src/models/llama2/cpu.rs:46-66)."""
    _fields_ = [(n, C.c_uint32) for n in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                          "num_key_value_heads", "vocab_size", "max_position_embeddings")] + [
        ("rope_theta", C.c_float), ("rms_norm_eps", C.c_float), ("rope_variant", C.c_uint32)]


class LlamaLayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down",
                                          "attn_norm_dev", "ffn_norm_dev", "attn_q_bias_dev", "attn_k_bias_dev", "attn_v_bias_dev")]


class LlamaWeights(C.Structure):
    _fields_ = [("layers", C.POINTER(LlamaLayerWeights)), ("token_embd", C.c_void_p), ("output", C.c_void_p), ("output_norm_dev", C.c_void_p)]


class GgufTensorInfo(C.Structure):
    """= ib_gguf_tensor_info: dims slowest first ([rows, cols] for a matrix), as the reference keeps them (gguf.rs:587-593)."""
    _fields_ = [("type", C.c_int32), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4), ("offset", C.c_uint64), ("nbytes", C.c_uint64),
                ("data", C.c_void_p)]


# name -> (restype, argtypes); every symbol include/inferi_b200.h declares
_vp, _u32, _u64, _i32, _f = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32, C.c_float
# ib_token_event_fn: (user, prev_token, token, next_pos, token_count, token_time) -> non-zero to stop
TOKEN_EVENT_FN = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_double)
SIGNATURES = {
    "ib_last_error_string": (C.c_char_p, []),
    "ib_ctx_create": (_i32, [_i32, C.POINTER(_vp)]),
    "ib_ctx_destroy": (_i32, [_vp]),
    "ib_ctx_launch_count": (_i32, [_vp, C.POINTER(_u64)]),
    "ib_ctx_reset_launch_count": (_i32, [_vp]),
    "ib_ctx_set_wait_limit": (_i32, [_vp, _u64]),
    "ib_malloc": (_i32, [_vp, _u64, C.POINTER(_vp)]),
    "ib_free": (_i32, [_vp, _vp]),
    "ib_memcpy_h2d": (_i32, [_vp, _vp, _vp, _vp, _u64]),
    "ib_memcpy_d2h": (_i32, [_vp, _vp, _vp, _vp, _u64]),
    "ib_stream_sync": (_i32, [_vp, _vp]),
    "ib_qtensor_upload": (_i32, [_vp, _i32, _u64, _u64, _vp, _u64, _i32, C.POINTER(_vp)]),
    "ib_qtensor_destroy": (_i32, [_vp]),
    "ib_qtensor_info": (_i32, [_vp, C.POINTER(_i32), C.POINTER(_u64), C.POINTER(_u64), C.POINTER(_u64)]),
    "ib_gemv_quant": (_i32, [_vp, _vp, _vp, _vp, _vp]),
    "ib_gemv_quant_host": (_i32, [_vp, _vp, _vp, _vp]),
    "ib_gemm_quant": (_i32, [_vp, _vp, _vp, _vp, _vp, _u32]),
    "ib_ffn_gate_up": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f]),
    "ib_rms_norm": (_i32, [_vp, _vp, _vp, _vp, _vp, _u32, _f]),
    "ib_rope": (_i32, [_vp, _vp, _i32, _vp, _u32, _vp, _u32, _u32, _u32, _f]),
    "ib_silu_mul": (_i32, [_vp, _vp, _vp, _vp, _u32]),
    "ib_add_assign": (_i32, [_vp, _vp, _vp, _vp, _u32]),
    "ib_attention": (_i32, [_vp, _vp, C.POINTER(AttnParams), _vp, _vp, _vp, _i32, _vp]),
    "ib_attention_static": (_i32, [_vp, C.POINTER(AttnParams), _vp, _vp, _vp, _i32, _vp]),
    "ib_argmax": (_i32, [_vp, _vp, _vp, _u32, _vp]),
    "ib_sample": (_i32, [_vp, _vp, _vp, _u32, _f, _f, _f, _vp]),
    "ib_llama_set_sampler": (_i32, [_vp, _f, _f, _u64]),
    "ib_llama_generate_until": (_i32, [_vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp, C.POINTER(_u32)]),
    "ib_llama_chat": (_i32, [_vp, _vp, _vp, _u32, _u32, _u32, _u32, TOKEN_EVENT_FN, _vp, C.POINTER(_u32)]),
    "ib_llama_create": (_i32, [_vp, C.POINTER(LlamaConfig), C.POINTER(LlamaWeights), _i32, _i32, _i32, C.POINTER(_vp)]),
    "ib_llama_destroy": (_i32, [_vp]),
    "ib_llama_forward": (_i32, [_vp, _vp, _u32, _u32, _vp, _vp]),
    "ib_llama_generate": (_i32, [_vp, _vp, _vp, _u32, _u32, _u32, _vp]),
    "ib_llama_state": (_i32, [_vp, C.POINTER(_vp), C.POINTER(_vp)]),
    "ib_llama_tp_export": (_i32, [_vp, _vp]),
    "ib_llama_prefill": (_i32, [_vp, _vp, _vp, _u32, _u32, C.POINTER(_u32)]),
    "ib_llama_tp_connect": (_i32, [_vp, _vp]),
    "ib_llama_tp_area": (_i32, [_vp, C.POINTER(_vp), C.POINTER(_u64)]),
    "ib_llama_tp_connect_ptrs": (_i32, [_vp, C.POINTER(_vp)]),
    "ib_gguf_open": (_i32, [C.c_char_p, C.POINTER(_vp)]),
    "ib_gguf_open_memory": (_i32, [_vp, _u64, C.POINTER(_vp)]),
    "ib_gguf_close": (_i32, [_vp]),
    "ib_gguf_counts": (_i32, [_vp, C.POINTER(_u32), C.POINTER(_u64), C.POINTER(_u64), C.POINTER(_u32)]),
    "ib_gguf_tensor_by_name": (_i32, [_vp, C.c_char_p, C.POINTER(GgufTensorInfo)]),
    "ib_gguf_tensor_by_index": (_i32, [_vp, _u64, C.c_char_p, _u64, C.POINTER(GgufTensorInfo)]),
    "ib_gguf_meta_key": (_i32, [_vp, _u64, C.c_char_p, _u64, C.POINTER(_i32)]),
    "ib_gguf_meta_u64": (_i32, [_vp, C.c_char_p, C.POINTER(_u64)]),
    "ib_gguf_meta_f64": (_i32, [_vp, C.c_char_p, C.POINTER(C.c_double)]),
    "ib_gguf_meta_str": (_i32, [_vp, C.c_char_p, C.c_char_p, _u64, C.POINTER(_u64)]),
    "ib_gguf_meta_array": (_i32, [_vp, C.c_char_p, C.POINTER(_i32), C.POINTER(_u64), C.POINTER(_vp)]),
    "ib_gguf_meta_array_str": (_i32, [_vp, C.c_char_p, _u64, C.c_char_p, _u64, C.POINTER(_u64)]),
    "ib_gguf_llama_config": (_i32, [_vp, C.c_char_p, C.POINTER(LlamaConfig)]),
    "ib_tokenizer_llama_from_gguf": (_i32, [_vp, C.POINTER(_vp)]),
    "ib_tokenizer_gpt2_from_gguf": (_i32, [_vp, C.POINTER(_vp)]),
    "ib_tokenizer_destroy": (_i32, [_vp]),
    "ib_tokenizer_info": (_i32, [_vp, C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32)]),
    "ib_tokenizer_encode": (_i32, [_vp, C.c_char_p, _u64, _i32, _i32, _vp, _u64, C.POINTER(_u64)]),
    "ib_tokenizer_decode": (_i32, [_vp, _u32, _u32, C.c_char_p, _u64, C.POINTER(_u64)]),
    "ib_gguf_load_llama": (_i32, [_vp, _vp, C.c_char_p, _i32, _u32, _i32, _i32, C.POINTER(_vp)]),
}

_lib = None


def load() -> C.CDLL:
    """Load libinferi_b200.so and bind every declared symbol.  Raises if the library is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m inferi_b200.build` (needs nvcc). "
                "inferi_b200 has no CPU or PyTorch fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(code: int) -> None:
    if code != IB_OK:
        msg = load().ib_last_error_string()
        raise InferiError(code, msg.decode("utf-8", "replace") if msg else "")
