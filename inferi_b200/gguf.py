"""GGUF files: host-side mirror of the reference's `Gguf` over the C ABI, plus a writer for Llama checkpoints.

`Gguf` ≙ `Gguf::from_bytes` / `metadata` / `tensors` (crates/inferi/src/gguf.rs:516-692); `Gguf.llama_config` ≙
`Llama2Config::from_gguf` (crates/inferi/src/models/llama2/cpu.rs:74-107); `Gguf.load_llama` ≙ `Llama2Weights::from_gguf`
(crates/inferi/src/models/llama2/transformer.rs:294-394) + `Llama2State::new`.  Parsing, slicing and upload are done by the
shared library (csrc/gguf.cu); this file only marshals.

`write_llama_gguf` writes a checkpoint in the layout `llama2.synth_weights` produces as a GGUF v3 file with the tensor
names and metadata keys the reference (and llama.cpp) read, so the same file can be given to either.
"""
from __future__ import annotations

import ctypes as C
import struct

import numpy as np

from . import quant
from ._lib import KV_F16, KV_F32, GgufTensorInfo, LlamaConfig, check, load
from .llama2 import LAYER_MATS, Llama2, Llama2Config
from .ops import Backend

# metadata value type ids (gguf.rs:397-428)
U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
_SCALAR_NP = {U8: np.uint8, I8: np.int8, U16: np.uint16, I16: np.int16, U32: np.uint32, I32: np.int32, F32: np.float32, BOOL: np.uint8,
              U64: np.uint64, I64: np.int64, F64: np.float64}
_SIGNED = (I8, I16, I32, I64)


class Gguf:
    def __init__(self, path: str | None = None, data: bytes | None = None):
        self.lib = load()
        self._data = data                     # kept alive: ib_gguf_open_memory does not copy
        h = C.c_void_p()
        if path is not None:
            check(self.lib.ib_gguf_open(path.encode(), C.byref(h)))
        else:
            buf = C.create_string_buffer(data, len(data))
            self._data = buf
            check(self.lib.ib_gguf_open_memory(buf, len(data), C.byref(h)))
        self.handle = h
        v, nt, nm, al = C.c_uint32(), C.c_uint64(), C.c_uint64(), C.c_uint32()
        check(self.lib.ib_gguf_counts(h, C.byref(v), C.byref(nt), C.byref(nm), C.byref(al)))
        self.version, self.n_tensors, self.n_metadata, self.alignment = v.value, nt.value, nm.value, al.value

    # ---- tensors ----
    def tensor_names(self) -> list[str]:
        out, name, info = [], C.create_string_buffer(512), GgufTensorInfo()
        for i in range(self.n_tensors):
            check(self.lib.ib_gguf_tensor_by_index(self.handle, i, name, 512, C.byref(info)))
            out.append(name.value.decode())
        return out

    def tensor(self, name: str) -> dict:
        """{'type', 'shape' (slowest first), 'offset', 'nbytes', 'data' (uint8 view of the mapping)}."""
        info = GgufTensorInfo()
        check(self.lib.ib_gguf_tensor_by_name(self.handle, name.encode(), C.byref(info)))
        data = np.ctypeslib.as_array(C.cast(info.data, C.POINTER(C.c_uint8)), shape=(info.nbytes,)) if info.nbytes else np.empty(0, np.uint8)
        return {"type": info.type, "shape": tuple(info.dims[:info.n_dims]), "offset": info.offset, "nbytes": info.nbytes, "data": data}

    # ---- metadata ----
    def keys(self) -> list[tuple[str, int]]:
        out, key, ty = [], C.create_string_buffer(1024), C.c_int32()
        for i in range(self.n_metadata):
            check(self.lib.ib_gguf_meta_key(self.handle, i, key, 1024, C.byref(ty)))
            out.append((key.value.decode(), ty.value))
        return out

    def get(self, key: str, ty: int | None = None):
        if ty is None:
            ty = dict(self.keys())[key]
        k = key.encode()
        if ty == STRING:
            n = C.c_uint64()
            check(self.lib.ib_gguf_meta_str(self.handle, k, None, 0, C.byref(n)))
            buf = C.create_string_buffer(n.value + 1)
            check(self.lib.ib_gguf_meta_str(self.handle, k, buf, n.value + 1, None))
            return buf.raw[:n.value].decode("utf-8", "replace")
        if ty == ARRAY:
            et, cnt, ptr = C.c_int32(), C.c_uint64(), C.c_void_p()
            check(self.lib.ib_gguf_meta_array(self.handle, k, C.byref(et), C.byref(cnt), C.byref(ptr)))
            if et.value == STRING:
                out, n = [], C.c_uint64()
                buf = C.create_string_buffer(1 << 16)
                for i in range(cnt.value):
                    check(self.lib.ib_gguf_meta_array_str(self.handle, k, i, buf, 1 << 16, C.byref(n)))
                    out.append(buf.raw[:min(n.value, (1 << 16) - 1)].decode("utf-8", "replace"))
                return out
            if et.value in _SCALAR_NP:
                dt = np.dtype(_SCALAR_NP[et.value])
                raw = C.string_at(ptr.value, cnt.value * dt.itemsize) if cnt.value else b""
                return np.frombuffer(raw, dtype=dt).copy()
            raise ValueError(f"nested array in {key}")
        if ty in (F32, F64):
            v = C.c_double()
            check(self.lib.ib_gguf_meta_f64(self.handle, k, C.byref(v)))
            return v.value
        v = C.c_uint64()
        check(self.lib.ib_gguf_meta_u64(self.handle, k, C.byref(v)))
        if ty in _SIGNED:
            return v.value - (1 << 64) if v.value >> 63 else v.value
        return bool(v.value) if ty == BOOL else v.value

    # ---- Llama ----
    def llama_config(self, arch: str | None = None) -> Llama2Config:
        c = LlamaConfig()
        check(self.lib.ib_gguf_llama_config(self.handle, arch.encode() if arch else None, C.byref(c)))
        return Llama2Config(c.hidden_size, c.intermediate_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.vocab_size,
                            c.max_position_embeddings, c.rope_theta, c.rms_norm_eps, c.rope_variant)

    def load_llama(self, backend: Backend, kv_f16: bool = True, max_context: int = 0, tp_rank: int = 0, tp_size: int = 1, group=None,
                   arch: str | None = None) -> Llama2:
        cfg = self.llama_config(arch)
        if max_context and max_context < cfg.max_position_embeddings:
            cfg.max_position_embeddings = max_context
        h = C.c_void_p()
        check(self.lib.ib_gguf_load_llama(backend.handle, self.handle, arch.encode() if arch else None, KV_F16 if kv_f16 else KV_F32, max_context, tp_rank,
                                          tp_size, C.byref(h)))
        return Llama2.from_handle(backend, cfg, h, tp_rank, tp_size, group)

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.ib_gguf_close(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class LlamaTokenizer:
    """≙ `LlamaTokenizer` (crates/inferi/src/models/tokenizers/llama2_tokenizer.rs:8-180) over the C ABI."""

    FROM_GGUF = "ib_tokenizer_llama_from_gguf"

    def __init__(self, gguf: Gguf):
        self.lib = gguf.lib
        h = C.c_void_p()
        check(getattr(self.lib, self.FROM_GGUF)(gguf.handle, C.byref(h)))
        self.handle = h
        v, b, e, u = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint32()
        check(self.lib.ib_tokenizer_info(h, C.byref(v), C.byref(b), C.byref(e), C.byref(u)))
        self.vocab_size, self.bos, self.eos, self.unk = v.value, b.value, e.value, u.value

    def encode(self, text: str, bos: bool = True, eos: bool = False) -> list[int]:
        raw = text.encode("utf-8")
        n = C.c_uint64()
        check(self.lib.ib_tokenizer_encode(self.handle, raw, len(raw), int(bos), int(eos), None, 0, C.byref(n)))
        out = (C.c_uint32 * max(1, n.value))()
        check(self.lib.ib_tokenizer_encode(self.handle, raw, len(raw), int(bos), int(eos), out, n.value, C.byref(n)))
        return list(out[:n.value])

    def decode(self, prev_token: int, token: int) -> str:
        n = C.c_uint64()
        buf = C.create_string_buffer(1 << 12)
        check(self.lib.ib_tokenizer_decode(self.handle, prev_token, token, buf, 1 << 12, C.byref(n)))
        return buf.raw[:n.value].decode("utf-8", "replace")

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.ib_tokenizer_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Gpt2Tokenizer(LlamaTokenizer):
    """≙ `Gpt2Tokenizer` (crates/inferi/src/models/tokenizers/gpt2_tokenizer.rs:37-217) over the C ABI.  `encode` adds neither
    bos nor eos unless asked (the reference's never does)."""
    FROM_GGUF = "ib_tokenizer_gpt2_from_gguf"

    def encode(self, text: str, bos: bool = False, eos: bool = False) -> list[int]:
        return super().encode(text, bos, eos)

    def decode_tokens(self, tokens) -> str:
        return "".join(self.decode(0, int(t)) for t in tokens)


# ---- writer ----
def _s(b: bytes | str) -> bytes:
    b = b.encode() if isinstance(b, str) else b
    return struct.pack("<Q", len(b)) + b


def _value(ty: int, v) -> bytes:
    if ty == STRING:
        return _s(v)
    if ty == ARRAY:
        et, items = v
        body = b"".join(_value(et, x) for x in items) if et in (STRING, ARRAY) else np.asarray(items, dtype=_SCALAR_NP[et]).tobytes()
        return struct.pack("<IQ", et, len(items)) + body
    return np.asarray(v, dtype=_SCALAR_NP[ty]).tobytes()


def write_gguf(path: str, metadata: list[tuple[str, int, object]], tensors: list[tuple[str, int, tuple, bytes]], alignment: int = 32,
               version: int = 3) -> None:
    """Writes a GGUF file.  `metadata`: (key, type id, value); arrays as (elem type, items).  `tensors`: (name, ggml type id,
    shape slowest first, raw bytes): dimensions are stored fastest first as the format asks (gguf.rs:587-593)."""
    meta = list(metadata)
    if alignment != 32 and not any(k == "general.alignment" for k, _, _ in meta):
        meta.append(("general.alignment", U32, alignment))
    head = struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(meta))
    head += b"".join(_s(k) + struct.pack("<I", ty) + _value(ty, v) for k, ty, v in meta)
    table, off = b"", 0
    offsets = []
    for name, ty, shape, raw in tensors:
        offsets.append(off)
        table += _s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in reversed(shape)) + struct.pack("<IQ", ty, off)
        off = (off + len(raw) + alignment - 1) // alignment * alignment
    head += table
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * ((-len(head)) % alignment))
        for (name, ty, shape, raw), o in zip(tensors, offsets):
            f.write(raw)
            f.write(b"\0" * ((-len(raw)) % alignment))


def write_llama_gguf(path: str, cfg: Llama2Config, weights: dict, tokens: list[str] | None = None, arch: str = "llama",
                     scores=None, special: tuple[int, int, int] | None = None, chat_template: str | None = None) -> None:
    """A checkpoint in the layout of `llama2.synth_weights` as a GGUF v3 file (tensor names of transformer.rs:304-315,
    metadata keys of cpu.rs:81-88).  Without `tokens` the file carries no tokenizer and the vocabulary is read off token_embd;
    `scores` and `special` = (bos, eos, unk) ids complete what `LlamaTokenizer::from_gguf` reads (llama2_tokenizer.rs:23-40)."""
    meta = [("general.architecture", STRING, arch), (f"{arch}.embedding_length", U32, cfg.hidden_size),
            (f"{arch}.feed_forward_length", U32, cfg.intermediate_size), (f"{arch}.block_count", U32, cfg.num_hidden_layers),
            (f"{arch}.attention.head_count", U32, cfg.num_attention_heads), (f"{arch}.attention.head_count_kv", U32, cfg.num_key_value_heads),
            (f"{arch}.context_length", U32, cfg.max_position_embeddings), (f"{arch}.rope.freq_base", F32, cfg.rope_theta),
            (f"{arch}.attention.layer_norm_rms_epsilon", F32, cfg.rms_norm_eps)]
    if tokens is not None:
        meta.append(("tokenizer.ggml.tokens", ARRAY, (STRING, tokens)))
    if scores is not None:
        meta.append(("tokenizer.ggml.scores", ARRAY, (F32, list(scores))))
    if special is not None:
        meta += [(f"tokenizer.ggml.{n}_token_id", U32, v) for n, v in zip(("bos", "eos", "unknown"), special)]
    if chat_template is not None:
        meta.append(("tokenizer.chat_template", STRING, chat_template))
    sh = cfg.shapes()

    def raw(t) -> bytes:
        return (t.cpu().numpy() if hasattr(t, "cpu") else np.asarray(t)).tobytes()

    tensors = []
    qt, data = weights["token_embd"]
    tensors.append(("token_embd.weight", qt, sh["token_embd"], raw(data)))
    for i, lw in enumerate(weights["layers"]):
        for n in LAYER_MATS:
            tensors.append((f"blk.{i}.{n}.weight", lw[n][0], sh[n], raw(lw[n][1])))
        for n in ("attn_norm", "ffn_norm"):
            tensors.append((f"blk.{i}.{n}.weight", quant.F32, (cfg.hidden_size,), raw(lw[n])))
        for n, width in (("attn_q", cfg.hidden_size), ("attn_k", cfg.kv_dim), ("attn_v", cfg.kv_dim)):   # transformer.rs:307-309
            if lw.get(n + "_bias") is not None:
                tensors.append((f"blk.{i}.{n}.bias", quant.F32, (width,), raw(lw[n + "_bias"])))
    tensors.append(("output_norm.weight", quant.F32, (cfg.hidden_size,), raw(weights["output_norm"])))
    if weights.get("output") is not None:
        qt, data = weights["output"]
        tensors.append(("output.weight", qt, sh["output"], raw(data)))
    write_gguf(path, meta, tensors)
