"""Tensor-parallel sharding of a GGUF-block checkpoint and the rank hand-shake (one process per GPU).

The reference is single-GPU; this is the Megatron-style split the 8B-class configuration asks for inside one NVSwitch box:
q/k/v, gate/up and the classifier by output rows (heads, FFN units, vocabulary), attn_output and ffn_down by input columns
at block granularity, with one partial-sum exchange after attn_output and after ffn_down.  Slicing is done on the GGUF
bytes (no re-quantisation).  Q6_K rows can only be cut at multiples of 2048 columns (8 blocks) to stay 16-byte aligned, so
a rank's FFN slice is padded with all-zero blocks / rows up to that multiple; zero blocks dequantize to exactly 0.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import quant
from ._lib import TP_HANDLE_BYTES, check
from .llama2 import LAYER_MATS, Llama2Config


def _t(x) -> torch.Tensor:
    return x if isinstance(x, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(x))


def rows_slice(mat, r0: int, r1: int, pad_rows: int = 0):
    """Rows [r0, r1) of a (qtype, uint8 [rows, row_bytes]) matrix, plus `pad_rows` all-zero rows."""
    qt, data = mat
    out = _t(data)[r0:r1]
    if pad_rows:
        out = torch.cat([out, torch.zeros(pad_rows, out.shape[1], dtype=torch.uint8, device=out.device)], dim=0)
    return qt, out.contiguous()


def cols_slice(mat, c0: int, c1: int, pad_cols: int = 0):
    """Columns [c0, c1) of a quantized matrix (block-aligned), plus `pad_cols` columns of all-zero blocks."""
    qt, data = mat
    be, bb = quant.BLOCK_ELEMS[qt], quant.BLOCK_BYTES[qt]
    if c0 % be or c1 % be or pad_cols % be:
        raise ValueError(f"column range [{c0}, {c1}) + {pad_cols} is not aligned to the {quant.NAMES[qt]} block length {be}")
    d = _t(data)
    rows = d.shape[0]
    out = d.reshape(rows, -1, bb)[:, c0 // be:c1 // be, :]
    if pad_cols:
        out = torch.cat([out, torch.zeros(rows, pad_cols // be, bb, dtype=torch.uint8, device=d.device)], dim=1)
    return qt, out.reshape(rows, -1).contiguous()


def ffn_plan(cfg: Llama2Config, tp: int, down_qtype: int):
    """(real FFN units per rank, padded units per rank).  The padded width is what the rank's matrices carry."""
    f = cfg.intermediate_size
    if f % (tp * quant.QK_K):
        raise ValueError(f"intermediate_size={f} does not split into {tp} block-aligned slices")
    real = f // tp
    unit = 2048 if down_qtype == quant.Q6_K else 256
    padded = (real + unit - 1) // unit * unit
    return real, padded


def shard_weights(cfg: Llama2Config, weights: dict, rank: int, tp: int) -> dict:
    """This rank's shard of a checkpoint in the layout `llama2.synth_weights` returns."""
    if tp == 1:
        return weights
    if cfg.num_key_value_heads % tp or cfg.num_attention_heads % tp or cfg.vocab_size % (4 * tp):
        raise ValueError(f"{tp} ranks do not divide the heads / vocabulary of this model")
    hs = cfg.head_size
    q0, q1 = rank * cfg.hidden_size // tp, (rank + 1) * cfg.hidden_size // tp
    k0, k1 = rank * cfg.kv_dim // tp, (rank + 1) * cfg.kv_dim // tp
    assert (q1 - q0) % hs == 0 and (k1 - k0) % hs == 0
    layers = []
    for lw in weights["layers"]:
        real, padded = ffn_plan(cfg, tp, lw["ffn_down"][0])
        f0, f1, pad = rank * real, (rank + 1) * real, padded - real
        layers.append({
            "attn_q": rows_slice(lw["attn_q"], q0, q1), "attn_k": rows_slice(lw["attn_k"], k0, k1), "attn_v": rows_slice(lw["attn_v"], k0, k1),
            "attn_output": cols_slice(lw["attn_output"], q0, q1),
            "ffn_gate": rows_slice(lw["ffn_gate"], f0, f1, pad), "ffn_up": rows_slice(lw["ffn_up"], f0, f1, pad),
            "ffn_down": cols_slice(lw["ffn_down"], f0, f1, pad),
            "attn_norm": lw["attn_norm"], "ffn_norm": lw["ffn_norm"],
        })
        for n, (a, b) in (("attn_q_bias", (q0, q1)), ("attn_k_bias", (k0, k1)), ("attn_v_bias", (k0, k1))):
            if lw.get(n) is not None:
                layers[-1][n] = lw[n][a:b]
    v0, v1 = rank * cfg.vocab_size // tp, (rank + 1) * cfg.vocab_size // tp
    head = weights["output"] if weights.get("output") is not None else weights["token_embd"]
    return {"layers": layers, "token_embd": weights["token_embd"], "output": rows_slice(head, v0, v1), "output_norm": weights["output_norm"]}


def shard_shapes(cfg: Llama2Config, tp: int, down_qtype: int) -> dict:
    """[rows, cols] of every matrix of one rank."""
    h, kv, v = cfg.hidden_size, cfg.kv_dim, cfg.vocab_size
    _, f = ffn_plan(cfg, tp, down_qtype)
    return {"attn_q": (h // tp, h), "attn_k": (kv // tp, h), "attn_v": (kv // tp, h), "attn_output": (h, h // tp), "ffn_gate": (f, h),
            "ffn_up": (f, h), "ffn_down": (h, f), "token_embd": (v, h), "output": (v // tp, h)}


def connect(model, group=None) -> None:
    """Exchange the ranks' exchange-area handles over torch.distributed and map them (call on every rank)."""
    import torch.distributed as dist
    lib = model.lib
    mine = (C.c_ubyte * TP_HANDLE_BYTES)()
    check(lib.ib_llama_tp_export(model.handle, mine))
    world = dist.get_world_size(group)
    gathered = [None] * world
    dist.all_gather_object(gathered, bytes(mine), group=group)
    blob = b"".join(gathered)
    buf = (C.c_ubyte * len(blob)).from_buffer_copy(blob)
    check(lib.ib_llama_tp_connect(model.handle, buf))
    dist.barrier(group)
