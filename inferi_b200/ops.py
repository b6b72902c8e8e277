"""Host-side mirror of the reference's op objects for the token loop, over the C ABI.

Each class keeps the name, argument meaning and error behaviour of its counterpart in
crates/inferi/src/ops/ (`GemvQuant`, `RmsNorm`, `RoPE`, `Silu`, `FusedAttention`) and of the façade methods in
crates/inferi/src/context.rs:336-719; shape-contract violations raise `InferiError` where the reference panics.
Device buffers are torch CUDA tensors (torch is only the allocator and the stream provider here).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from ._lib import AttnParams, InferiError, KV_F16, KV_F32, ROPE_NEOX, ROPE_ORIGINAL, check  # noqa: F401
from .quant import BLOCK_BYTES, BLOCK_ELEMS, F32, NAMES, Q4_K, Q5_K, Q6_K, Q8_0, row_bytes  # noqa: F401


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _f32_dev(t: torch.Tensor, name: str) -> int:
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
        raise InferiError(1, f"{name}: expected a contiguous float32 CUDA tensor")
    return t.data_ptr()


class Backend:
    """≙ `GpuBackend` + `LlmOps::new` (crates/inferi/src/context.rs:58-85): one context per device."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        h = C.c_void_p()
        check(self.lib.ib_ctx_create(device, C.byref(h)))
        self.handle = h
        self.device = device

    def launch_count(self) -> int:
        n = C.c_uint64()
        check(self.lib.ib_ctx_launch_count(self.handle, C.byref(n)))
        return int(n.value)

    def reset_launch_count(self) -> None:
        check(self.lib.ib_ctx_reset_launch_count(self.handle))

    def set_wait_limit(self, nanoseconds: int) -> None:
        """How long a wait inside a kernel may last before the kernel gives up and the next synchronising call returns
        IB_ERR_TIMEOUT (default 2 s).  Applies to launches issued, and token graphs recorded, after the call."""
        check(self.lib.ib_ctx_set_wait_limit(self.handle, int(nanoseconds)))

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.ib_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GpuQuantTensor:
    """≙ `GpuQuantTensor` (crates/inferi/src/quantized_matrix.rs:11-54) built by `GgufTensor::to_gpu_quant`
    (crates/inferi/src/gguf.rs:141-197): a [rows, cols] matrix of GGUF blocks on the device."""

    def __init__(self, backend: Backend, qtype: int, rows: int, cols: int, blocks):
        self.backend = backend
        self.qtype, self.rows, self.cols = qtype, rows, cols
        h = C.c_void_p()
        if isinstance(blocks, torch.Tensor) and blocks.is_cuda:
            b = blocks.contiguous().view(torch.uint8)
            check(backend.lib.ib_qtensor_upload(backend.handle, qtype, rows, cols, b.data_ptr(), b.numel(), 1, C.byref(h)))
        else:
            if isinstance(blocks, torch.Tensor):
                blocks = blocks.contiguous().view(torch.uint8).numpy()
            b = np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
            check(backend.lib.ib_qtensor_upload(backend.handle, qtype, rows, cols, b.ctypes.data_as(C.c_void_p), b.size, 0, C.byref(h)))
        self.handle = h

    @property
    def nbytes(self) -> int:
        return self.rows * row_bytes(self.qtype, self.cols)

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.backend.lib.ib_qtensor_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GemvQuant:
    """≙ `GemvQuant` (crates/inferi/src/ops/gemv_quant.rs:105-341)."""

    def __init__(self, backend: Backend):
        self.backend = backend

    @classmethod
    def from_backend(cls, backend: Backend) -> "GemvQuant":
        return cls(backend)

    def launch(self, out: torch.Tensor, m: GpuQuantTensor, v: torch.Tensor) -> None:
        """out[rows] = m . v[cols] on the current stream (asynchronous, like recording into a pass)."""
        if v.numel() != m.cols or out.numel() != m.rows:
            raise InferiError(1, f"gemv: matrix is {m.rows}x{m.cols} but v has {v.numel()} and out {out.numel()} elements")
        check(self.backend.lib.ib_gemv_quant(self.backend.handle, _stream_ptr(), _f32_dev(out, "out"), m.handle, _f32_dev(v, "v")))

    def launch_host(self, m: GpuQuantTensor, v: np.ndarray) -> np.ndarray:
        """The same op for host buffers: copy in, run, copy out, synchronise."""
        v = np.ascontiguousarray(v, dtype=np.float32)
        if v.size != m.cols:
            raise InferiError(1, f"gemv: matrix has {m.cols} columns but v has {v.size} elements")
        out = np.empty(m.rows, dtype=np.float32)
        check(self.backend.lib.ib_gemv_quant_host(self.backend.handle, out.ctypes.data_as(C.c_void_p), m.handle, v.ctypes.data_as(C.c_void_p)))
        return out


class GemmQuant:
    """n quantized GEMVs as one GEMM on the tensor cores (prompt prefill); no counterpart in the reference, which repeats
    `GemvQuant::launch` per token."""

    def __init__(self, backend: Backend):
        self.backend = backend

    def launch(self, out: torch.Tensor, m: GpuQuantTensor, x: torch.Tensor) -> None:
        """out[n, rows] = x[n, cols] . m^T on the current stream."""
        n = x.shape[0]
        if x.dim() != 2 or x.shape[1] != m.cols or tuple(out.shape) != (n, m.rows) or not x.is_contiguous() or not out.is_contiguous():
            raise InferiError(1, f"gemm: matrix is {m.rows}x{m.cols}, x {tuple(x.shape)}, out {tuple(out.shape)}")
        check(self.backend.lib.ib_gemm_quant(self.backend.handle, _stream_ptr(), _f32_dev(out, "out"), m.handle, _f32_dev(x, "x"), n))


class FfnGateUp:
    """`rms_norm_assign` + `matmul_quant_assign` (gate) + `matmul_quant_assign` (up) + `silu` of
    crates/inferi/src/models/llama2/transformer.rs:454-464 as one launch."""

    def __init__(self, backend: Backend):
        self.backend = backend

    def launch(self, out: torch.Tensor, gate: GpuQuantTensor, up: GpuQuantTensor, x: torch.Tensor, norm_w: torch.Tensor | None = None, eps: float = 1e-5) -> None:
        if x.numel() != gate.cols or out.numel() != gate.rows:
            raise InferiError(1, f"ffn gate/up: matrices are {gate.rows}x{gate.cols} but x has {x.numel()} and out {out.numel()} elements")
        check(self.backend.lib.ib_ffn_gate_up(self.backend.handle, _stream_ptr(), _f32_dev(out, "out"), gate.handle, up.handle, _f32_dev(x, "x"),
                                              _f32_dev(norm_w, "norm_w") if norm_w is not None else None, float(eps)))


@dataclass
class RmsNormConfig:
    """≙ `RmsNormConfig` (crates/inferi-shaders/src/rms_norm.rs:24-26)."""
    nudge_factor: float


class RmsNorm:
    """≙ `RmsNorm` (crates/inferi/src/ops/rms_norm.rs:9-79)."""

    def __init__(self, backend: Backend):
        self.backend = backend

    from_backend = classmethod(lambda cls, backend: cls(backend))

    def launch(self, config: RmsNormConfig, result: torch.Tensor, value: torch.Tensor, weight: torch.Tensor) -> None:
        n = value.numel()
        if result.numel() != n or weight.numel() != n:
            raise InferiError(1, "rms_norm: result, value and weight must have the same length")
        check(self.backend.lib.ib_rms_norm(self.backend.handle, _stream_ptr(), _f32_dev(result, "result"), _f32_dev(value, "value"),
                                           _f32_dev(weight, "weight"), n, config.nudge_factor))


@dataclass
class RoPEConfig:
    """≙ `RoPEConfig` (crates/inferi-shaders/src/rope.rs:21-26)."""
    head_size: int
    kv_dim: int
    pos: int
    base_freq: float


class RoPE:
    """≙ `RoPE` (crates/inferi/src/ops/rope.rs:12-135)."""

    def __init__(self, backend: Backend):
        self.backend = backend

    from_backend = classmethod(lambda cls, backend: cls(backend))

    def launch(self, variant: int, config: RoPEConfig, in_out_q: torch.Tensor, in_out_k: torch.Tensor) -> None:
        if in_out_k.numel() < config.kv_dim:
            raise InferiError(1, "rope: k is shorter than kv_dim")
        check(self.backend.lib.ib_rope(self.backend.handle, _stream_ptr(), variant, _f32_dev(in_out_q, "q"), in_out_q.numel(),
                                       _f32_dev(in_out_k, "k"), config.kv_dim, config.head_size, config.pos, config.base_freq))


class Silu:
    """≙ `Silu` (crates/inferi/src/ops/silu.rs:9-63): h1 <- h2 * swish(h1)."""

    def __init__(self, backend: Backend):
        self.backend = backend

    from_backend = classmethod(lambda cls, backend: cls(backend))

    def launch(self, in_out_h1: torch.Tensor, in_h2: torch.Tensor) -> None:
        if in_out_h1.numel() != in_h2.numel():
            raise InferiError(1, "silu: h1 and h2 must have the same length")
        check(self.backend.lib.ib_silu_mul(self.backend.handle, _stream_ptr(), _f32_dev(in_out_h1, "h1"), _f32_dev(in_h2, "h2"), in_out_h1.numel()))


class FusedAttention:
    """≙ `FusedAttention` (crates/inferi/src/ops/batched_multiquery_attention.rs:14-77)."""

    def __init__(self, backend: Backend):
        self.backend = backend

    from_backend = classmethod(lambda cls, backend: cls(backend))

    def launch(self, params: AttnParams, q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, xb: torch.Tensor) -> None:
        """key_cache / value_cache: [seq_len, kv_dim] float32 or float16 CUDA tensors."""
        if key_cache.dtype != value_cache.dtype or key_cache.dtype not in (torch.float16, torch.float32):
            raise InferiError(1, "attention: the caches must both be float16 or both float32")
        for t, name in ((key_cache, "key_cache"), (value_cache, "value_cache")):
            if not (t.is_cuda and t.is_contiguous() and t.numel() >= params.seq_len * params.kv_dim):
                raise InferiError(1, f"attention: {name} must be a contiguous CUDA tensor of at least seq_len*kv_dim elements")
        if q.numel() != params.n_heads * params.head_size or xb.numel() != q.numel():
            raise InferiError(1, "attention: q and xb must hold n_heads*head_size elements")
        kv = KV_F16 if key_cache.dtype == torch.float16 else KV_F32
        check(self.backend.lib.ib_attention(self.backend.handle, _stream_ptr(), C.byref(params), _f32_dev(q, "q"), key_cache.data_ptr(),
                                            value_cache.data_ptr(), kv, _f32_dev(xb, "xb")))


def add_assign(backend: Backend, a: torch.Tensor, b: torch.Tensor) -> None:
    """≙ `LlmContext::add_assign` (crates/inferi/src/context.rs:516-530): a += b."""
    if a.numel() != b.numel():
        raise InferiError(1, "add_assign: length mismatch")
    check(backend.lib.ib_add_assign(backend.handle, _stream_ptr(), _f32_dev(a, "a"), _f32_dev(b, "b"), a.numel()))


def argmax(backend: Backend, logits: torch.Tensor, out: torch.Tensor) -> None:
    """≙ greedy `Sampler::sample` (crates/inferi/src/models/sampler.rs:32-36, 54-56); out: int32/uint32[1] on the device."""
    if not (out.is_cuda and out.element_size() == 4):
        raise InferiError(1, "argmax: out must be a 4-byte CUDA tensor")
    check(backend.lib.ib_argmax(backend.handle, _stream_ptr(), _f32_dev(logits, "logits"), logits.numel(), out.data_ptr()))


class Sampler:
    """≙ `Sampler` (crates/inferi/src/models/sampler.rs:14-52) with the logits left on the device.  `coin` in [0, 1) is the
    caller's random number; temperature 0 is the greedy arg-max."""

    def __init__(self, backend: Backend, vocab_size: int, temperature: float, topp: float):
        self.backend, self.vocab_size, self.temperature, self.topp = backend, vocab_size, float(temperature), float(topp)

    def sample(self, logits: torch.Tensor, coin: float, out: torch.Tensor | None = None) -> torch.Tensor:
        if logits.numel() != self.vocab_size:
            raise ValueError(f"expected {self.vocab_size} logits, got {logits.numel()}")
        out = out if out is not None else torch.empty(1, dtype=torch.int32, device=logits.device)
        check(self.backend.lib.ib_sample(self.backend.handle, _stream_ptr(), _f32_dev(logits, "logits"), self.vocab_size, self.temperature, self.topp,
                                         float(coin), out.data_ptr()))
        return out

