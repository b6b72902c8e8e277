"""Host-side mirror of the reference's Llama model API over the C ABI.

`Llama2Config`, `Llama2Weights`, `Llama2` keep the names and field meaning of
crates/inferi/src/models/llama2/cpu.rs:46-141 and crates/inferi/src/models/llama2/transformer.rs:176-196, 294-481.
The token loop itself (embedding, 5 fused kernels per layer, classifier + greedy arg-max, CUDA graph) lives in
the shared library; this file only marshals handles.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np
import torch

from . import _lib, quant
from ._lib import KV_F16, KV_F32, InferiError, LlamaConfig, LlamaLayerWeights, LlamaWeights, check
from .ops import Backend, GpuQuantTensor

LAYER_MATS = ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")

# the "Q4_K_M" mix used by the synthetic checkpoints: Q4_K everywhere except Q6_K for v, down and the classifier
Q4_K_M = {"attn_q": quant.Q4_K, "attn_k": quant.Q4_K, "attn_v": quant.Q6_K, "attn_output": quant.Q4_K, "ffn_gate": quant.Q4_K,
          "ffn_up": quant.Q4_K, "ffn_down": quant.Q6_K, "token_embd": quant.Q4_K, "output": quant.Q6_K}


@dataclass
class Llama2Config:
    """≙ `Llama2Config` (crates/inferi/src/models/llama2/cpu.rs:46-66)."""
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float = 10000.0      # defaults of from_gguf (cpu.rs:95-106)
    rms_norm_eps: float = 1.0e-6
    rope_variant: int = 0            # 0 Original (Llama), 1 NeoX (Qwen2): crates/inferi/src/models/llama2/mod.rs:24-29

    @property
    def head_size(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def kv_dim(self) -> int:
        return self.hidden_size * self.num_key_value_heads // self.num_attention_heads

    @property
    def kv_mul(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def to_c(self) -> LlamaConfig:
        return LlamaConfig(self.hidden_size, self.intermediate_size, self.num_hidden_layers, self.num_attention_heads,
                           self.num_key_value_heads, self.vocab_size, self.max_position_embeddings, self.rope_theta, self.rms_norm_eps,
                           self.rope_variant)

    def shapes(self) -> dict:
        """[out_features, in_features] of every matrix (transformer.rs:304-315)."""
        h, f, kv, v = self.hidden_size, self.intermediate_size, self.kv_dim, self.vocab_size
        return {"attn_q": (h, h), "attn_k": (kv, h), "attn_v": (kv, h), "attn_output": (h, h), "ffn_gate": (f, h), "ffn_up": (f, h),
                "ffn_down": (h, f), "token_embd": (v, h), "output": (v, h)}

    def weight_bytes(self, recipe: dict = Q4_K_M, tied: bool = False) -> int:
        """Bytes of weights one token streams from HBM: every matrix once plus the f32 norm vectors."""
        sh = self.shapes()
        per_layer = sum(quant.matrix_bytes(recipe[n], *sh[n]) for n in LAYER_MATS)
        head = quant.matrix_bytes(recipe["token_embd" if tied else "output"], *sh["output"])
        norms = (2 * self.num_hidden_layers + 1) * self.hidden_size * 4
        return per_layer * self.num_hidden_layers + head + norms

    def matrix_params(self) -> int:
        """Weights of the layer matrices (what a prompt's GEMMs multiply with; classifier and embedding excluded)."""
        sh = self.shapes()
        return self.num_hidden_layers * sum(sh[n][0] * sh[n][1] for n in LAYER_MATS)

    def kv_bytes_per_position(self, kv_f16: bool = True) -> int:
        return 2 * self.num_hidden_layers * self.kv_dim * (2 if kv_f16 else 4)


LLAMA_3_2_1B = Llama2Config(2048, 8192, 16, 32, 8, 128256, 4096, 500000.0, 1e-5)
LLAMA_3_8B = Llama2Config(4096, 14336, 32, 32, 8, 128256, 8192, 500000.0, 1e-5)


BIAS_NAMES = ("attn_q_bias", "attn_k_bias", "attn_v_bias")


def synth_weights(cfg: Llama2Config, seed: int, device: str = "cpu", recipe: dict = Q4_K_M, tied: bool = False, std: float = 0.02,
                  qkv_bias: bool = False) -> dict:
    """Seeded random checkpoint in GGUF block bytes: f32 N(0, std) matrices quantized with the recipe's types, norm weights
    1 + N(0, std).  Returns {'layers': [{name: (qtype, uint8 tensor [rows, row_bytes]), 'attn_norm': f32, 'ffn_norm': f32}],
    'token_embd': (qtype, tensor), 'output': (qtype, tensor) | None, 'output_norm': f32} with tensors on `device`.
    `qkv_bias` adds f32 'attn_q_bias' / 'attn_k_bias' / 'attn_v_bias' ~ N(0, 0.1) to every layer (the Qwen2 variant:
    transformer.rs:181-183); they are drawn after everything else, so the matrices do not depend on the flag."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    sh = cfg.shapes()

    def mat(name):
        rows, cols = sh[name]
        out = []
        chunk = max(4, (1 << 24) // cols // 4 * 4)   # quantize in row chunks to bound temporary memory
        for r0 in range(0, rows, chunk):
            w = torch.randn(min(chunk, rows - r0), cols, generator=g, device=device, dtype=torch.float32) * std
            out.append(quant.quantize(recipe[name], w))
        return recipe[name], torch.cat(out, dim=0) if len(out) > 1 else out[0]

    def norm():
        return 1.0 + torch.randn(cfg.hidden_size, generator=g, device=device, dtype=torch.float32) * std

    layers = []
    for _ in range(cfg.num_hidden_layers):
        lw = {n: mat(n) for n in LAYER_MATS}
        lw["attn_norm"] = norm()
        lw["ffn_norm"] = norm()
        layers.append(lw)
    out = {"layers": layers, "token_embd": mat("token_embd"), "output": None if tied else mat("output"), "output_norm": norm()}
    if qkv_bias:
        for lw in layers:
            for n, width in zip(BIAS_NAMES, (cfg.hidden_size, cfg.kv_dim, cfg.kv_dim)):
                lw[n] = torch.randn(width, generator=g, device=device, dtype=torch.float32) * 0.1
    return out


def weights_to_host(weights: dict) -> dict:
    """The same checkpoint as numpy arrays (for a CPU checker)."""
    def m(t):
        return (t[0], t[1].cpu().numpy())
    return {"layers": [{**{n: m(lw[n]) for n in LAYER_MATS}, "attn_norm": lw["attn_norm"].cpu().numpy(), "ffn_norm": lw["ffn_norm"].cpu().numpy(),
                        **{n: lw[n].cpu().numpy() for n in BIAS_NAMES if lw.get(n) is not None}}
                       for lw in weights["layers"]],
            "token_embd": m(weights["token_embd"]), "output": None if weights["output"] is None else m(weights["output"]),
            "output_norm": weights["output_norm"].cpu().numpy()}


class Llama2Weights:
    """≙ `Llama2Weights` (crates/inferi/src/models/llama2/transformer.rs:176-196, 294-394): device tensors of one checkpoint."""

    def __init__(self, backend: Backend, cfg: Llama2Config, weights: dict, shapes: dict | None = None):
        """`shapes` overrides the [rows, cols] of the matrices (a tensor-parallel rank's shard, see tp.shard_shapes)."""
        self.backend, self.cfg = backend, cfg
        sh = shapes or cfg.shapes()
        dev = torch.device("cuda", backend.device)
        self.layers = []
        self._keep = []
        for lw in weights["layers"]:
            d = {n: GpuQuantTensor(backend, lw[n][0], sh[n][0], sh[n][1], lw[n][1]) for n in LAYER_MATS}
            for n in ("attn_norm", "ffn_norm") + BIAS_NAMES:
                if lw.get(n) is not None:
                    d[n] = torch.as_tensor(lw[n]).to(dev, torch.float32).contiguous()
            self.layers.append(d)
        qt, data = weights["token_embd"]
        self.token_embd = GpuQuantTensor(backend, qt, *sh["token_embd"], data)
        self.output = None
        if weights.get("output") is not None:
            qt, data = weights["output"]
            self.output = GpuQuantTensor(backend, qt, *sh["output"], data)
        self.output_norm = torch.as_tensor(weights["output_norm"]).to(dev, torch.float32).contiguous()

    def close(self) -> None:
        """Frees the device tensors (a model created from them must be closed first)."""
        for d in self.layers:
            for n in LAYER_MATS:
                d[n].close()
        self.layers = []
        for t in (self.token_embd, self.output):
            if t is not None:
                t.close()
        self.token_embd = self.output = None

    def to_c(self):
        arr = (LlamaLayerWeights * len(self.layers))()
        for i, d in enumerate(self.layers):
            for n in LAYER_MATS:
                setattr(arr[i], n, d[n].handle)
            arr[i].attn_norm_dev = d["attn_norm"].data_ptr()
            arr[i].ffn_norm_dev = d["ffn_norm"].data_ptr()
            for n in BIAS_NAMES:
                if n in d:
                    setattr(arr[i], n + "_dev", d[n].data_ptr())
        w = LlamaWeights(arr, self.token_embd.handle, self.output.handle if self.output else None, self.output_norm.data_ptr())
        return w, arr


class Llama2:
    """≙ `Llama2` + `Llama2State` (crates/inferi/src/models/llama2/transformer.rs:15-137, 396-481) and the greedy token loop of
    `ChatLlama2` (crates/inferi-chat/src/chat_llama2.rs:92-255)."""

    def __init__(self, backend: Backend, cfg: Llama2Config, weights: Llama2Weights, kv_f16: bool = True, tp_rank: int = 0, tp_size: int = 1,
                 group=None, connect: bool = True):
        """With tp_size > 1, `weights` holds this rank's shard (tp.shard_weights) and torch.distributed must be initialised:
        the ranks exchange the handles of their exchange areas here.  `forward` then returns this rank's slice of the logits.
        `connect=False` leaves the hand-shake to the caller: a host that runs all ranks in one process calls `tp_area` on
        every rank and then `connect_areas` with the device pointers."""
        self.backend, self.cfg, self.weights = backend, cfg, weights
        self.lib = backend.lib
        c_cfg = cfg.to_c()
        c_w, self._arr = weights.to_c()
        h = C.c_void_p()
        check(self.lib.ib_llama_create(backend.handle, C.byref(c_cfg), C.byref(c_w), KV_F16 if kv_f16 else KV_F32, tp_rank, tp_size, C.byref(h)))
        self.handle = h
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.vocab_local = cfg.vocab_size // tp_size
        if tp_size > 1 and connect:
            from . import tp
            tp.connect(self, group)      # every rank of the group must get here

    def connect_areas(self, areas) -> None:
        """Tensor-parallel set-up inside one process: `areas[r]` = device pointer of rank r's exchange area (`tp_area`), valid on
        this model's GPU; the model's own entry is ignored."""
        arr = (C.c_void_p * self.tp_size)(*[C.c_void_p(int(a) if a else 0) for a in areas])
        check(self.lib.ib_llama_tp_connect_ptrs(self.handle, arr))

    def tp_area(self):
        """(device pointer, bytes) of this rank's exchange area (tensor-parallel models)."""
        ptr, n = C.c_void_p(), C.c_uint64()
        check(self.lib.ib_llama_tp_area(self.handle, C.byref(ptr), C.byref(n)))
        return int(ptr.value), int(n.value)

    @classmethod
    def from_handle(cls, backend: Backend, cfg: Llama2Config, handle, tp_rank: int = 0, tp_size: int = 1, group=None) -> "Llama2":
        """Wraps a model the library created itself (the GGUF loader); the model owns its weights."""
        self = cls.__new__(cls)
        self.backend, self.cfg, self.weights, self.lib, self._arr = backend, cfg, None, backend.lib, None
        self.handle = handle
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.vocab_local = cfg.vocab_size // tp_size
        if tp_size > 1:
            from . import tp
            tp.connect(self, group)
        return self

    def set_sampler(self, temperature: float, topp: float = 0.0, seed: int = 0) -> None:
        """≙ `Sampler::new(vocab, temperature, topp)` for the model's own token loop: forward / generate then feed back sampled
        tokens (temperature 0 = greedy).  The coin of a position is a function of (seed, position)."""
        check(self.lib.ib_llama_set_sampler(self.handle, float(temperature), float(topp), int(seed)))

    def forward(self, token: int, pos: int, want_logits: bool = False):
        """One token at `pos`; returns (next_token, logits | None).  Host round trip per call, as in the reference."""
        nxt = C.c_uint32()
        logits = np.empty(self.vocab_local, dtype=np.float32) if want_logits else None
        check(self.lib.ib_llama_forward(self.handle, torch.cuda.current_stream().cuda_stream, token, pos,
                                        logits.ctypes.data_as(C.c_void_p) if want_logits else None, C.byref(nxt)))
        return int(nxt.value), logits

    def generate(self, tokens, n_gen: int, start_pos: int = 0) -> np.ndarray:
        """Feeds `tokens` from `start_pos`, then decodes `n_gen` tokens greedily on the device; one sync at the end."""
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        out = np.empty(max(n_gen, 1), dtype=np.uint32)
        check(self.lib.ib_llama_generate(self.handle, torch.cuda.current_stream().cuda_stream, toks.ctypes.data_as(C.c_void_p), toks.size,
                                         start_pos, n_gen, out.ctypes.data_as(C.c_void_p)))
        return out[:n_gen]

    def generate_until(self, tokens, max_gen: int, eos_token: int, start_pos: int = 0) -> np.ndarray:
        """`generate` that stops after `eos_token` (chat_llama2.rs:157-166); returns the valid tokens, stop token included."""
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        out = np.empty(max_gen, dtype=np.uint32)
        n = C.c_uint32()
        check(self.lib.ib_llama_generate_until(self.handle, torch.cuda.current_stream().cuda_stream, toks.ctypes.data_as(C.c_void_p), toks.size,
                                               start_pos, max_gen, eos_token, out.ctypes.data_as(C.c_void_p), C.byref(n)))
        return out[:n.value]

    def prefill(self, prompt, start_pos: int = 0) -> int:
        """The whole prompt at once on the tensor cores (no counterpart in the reference, whose `ChatLlama2::forward` feeds the
        prompt token by token, chat_llama2.rs:137-155): fills the cache for positions start_pos .. start_pos + len(prompt) - 1
        and returns the greedy token that follows.  Continue with generate([token], n, start_pos=start_pos + len(prompt))."""
        toks = np.ascontiguousarray(prompt, dtype=np.uint32)
        nxt = C.c_uint32()
        check(self.lib.ib_llama_prefill(self.handle, torch.cuda.current_stream().cuda_stream, toks.ctypes.data_as(C.c_void_p), toks.size, start_pos, C.byref(nxt)))
        return int(nxt.value)

    def last_logits(self) -> np.ndarray:
        """Logits of the last forward (this rank's slice of the vocabulary)."""
        lg = C.c_void_p()
        check(self.lib.ib_llama_state(self.handle, C.byref(lg), None))
        out = np.empty(self.vocab_local, dtype=np.float32)
        check(self.lib.ib_memcpy_d2h(self.backend.handle, None, out.ctypes.data_as(C.c_void_p), lg, out.nbytes))
        check(self.lib.ib_stream_sync(self.backend.handle, None))
        return out

    def hidden_state(self) -> np.ndarray:
        x = C.c_void_p()
        check(self.lib.ib_llama_state(self.handle, None, C.byref(x)))
        out = np.empty(self.cfg.hidden_size, dtype=np.float32)
        check(self.lib.ib_memcpy_d2h(self.backend.handle, None, out.ctypes.data_as(C.c_void_p), x, out.nbytes))
        check(self.lib.ib_stream_sync(self.backend.handle, None))
        return out

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.ib_llama_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
