"""GGUF block formats on the host: sizes, seeded synthetic blocks and a K-quant quantizer.

Block byte layouts follow crates/inferi/src/quantization.rs:42-45 (Q8_0, 34 B), :335-340 (Q4_K, 144 B),
:262-268 (Q5_K, 176 B) and :217-222 (Q6_K, 210 B, `d` last).  The reference can only *de*quantize; the
quantizers here exist to make "N(0, 0.02)-derived" synthetic model weights and are plain round-to-nearest
affine quantizers written with torch ops so that they run on CPU tensors (tests) and CUDA tensors (bench).
"""
from __future__ import annotations

import numpy as np
import torch

# GGUF tensor type ids (crates/inferi/src/gguf.rs:74-106)
F32, Q8_0, Q4_K, Q5_K, Q6_K = 0, 8, 12, 13, 14
Q4_0, Q4_1, Q5_0, Q5_1, Q8_K = 2, 3, 6, 7, 15   # op-level only (generic kernel); the token loop takes the five above
QK_K = 256

BLOCK_BYTES = {F32: 4, Q8_0: 34, Q4_K: 144, Q5_K: 176, Q6_K: 210, Q4_0: 18, Q4_1: 20, Q5_0: 22, Q5_1: 24, Q8_K: 292}
BLOCK_ELEMS = {F32: 1, Q8_0: 32, Q4_K: QK_K, Q5_K: QK_K, Q6_K: QK_K, Q4_0: 32, Q4_1: 32, Q5_0: 32, Q5_1: 32, Q8_K: QK_K}
NAMES = {F32: "F32", Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K", Q4_0: "Q4_0", Q4_1: "Q4_1", Q5_0: "Q5_0", Q5_1: "Q5_1", Q8_K: "Q8_K"}


def row_bytes(qtype: int, cols: int) -> int:
    be = BLOCK_ELEMS[qtype]
    if cols % be:
        raise ValueError(f"cols={cols} is not a multiple of the {NAMES[qtype]} block length {be}")
    return cols // be * BLOCK_BYTES[qtype]


def matrix_bytes(qtype: int, rows: int, cols: int) -> int:
    return rows * row_bytes(qtype, cols)


# ----------------------------------------------------------------------------------------------------
# seeded synthetic blocks: every bit pattern of quants / packed scales is legal; f16 super-scales are
# half(|N(0,1)| * scale) so that no inf/nan appears (the distribution the GEMV benchmarks are quoted on)
# ----------------------------------------------------------------------------------------------------

def random_blocks(qtype: int, rows: int, cols: int, seed: int, scale: float = 0.01, subnormal_frac: float = 0.0) -> np.ndarray:
    """uint8 array [rows, row_bytes] of random GGUF blocks.

    `subnormal_frac` pushes that share of the f16 scales into the binary16 subnormal range, as the
    reference's test helper does (crates/inferi/src/ops/gemv_quant.rs:356-365)."""
    rng = np.random.default_rng(seed)
    nb = rows * (cols // BLOCK_ELEMS[qtype])
    bb = BLOCK_BYTES[qtype]
    if qtype == F32:
        return rng.standard_normal((rows, cols), dtype=np.float32).view(np.uint8).reshape(rows, cols * 4)
    blocks = rng.integers(0, 256, size=(nb, bb), dtype=np.uint8)

    def f16_scales(n):
        s = np.abs(rng.standard_normal(n)).astype(np.float32) * scale
        if subnormal_frac > 0:
            sub = rng.random(n) < subnormal_frac
            s = np.where(sub, s * 1e-4, s).astype(np.float32)
        return s.astype(np.float16).view(np.uint16)

    def put_u16(col, vals):
        blocks[:, col] = (vals & 0xFF).astype(np.uint8)
        blocks[:, col + 1] = (vals >> 8).astype(np.uint8)

    if qtype == Q8_0:
        put_u16(0, f16_scales(nb))
        q = rng.integers(-127, 128, size=(nb, 32), dtype=np.int16).astype(np.int8)
        blocks[:, 2:] = q.view(np.uint8)
    elif qtype in (Q4_K, Q5_K):
        put_u16(0, f16_scales(nb))
        put_u16(2, f16_scales(nb))
    elif qtype == Q6_K:
        put_u16(208, f16_scales(nb))
    elif qtype in (Q4_0, Q5_0):
        put_u16(0, f16_scales(nb))
    elif qtype in (Q4_1, Q5_1):
        put_u16(0, f16_scales(nb))
        put_u16(2, f16_scales(nb))
    elif qtype == Q8_K:
        d = (np.abs(rng.standard_normal(nb)).astype(np.float32) * scale).view(np.uint8).reshape(nb, 4)   # f32 scale (random bytes could be NaN)
        blocks[:, 0:4] = d
    else:
        raise ValueError(f"unsupported qtype {qtype}")
    return blocks.reshape(rows, -1)


# ----------------------------------------------------------------------------------------------------
# quantizers (torch; device-agnostic).  Input f32 [rows, cols]; output uint8 [rows, row_bytes].
# ----------------------------------------------------------------------------------------------------

def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    """f32 [...] -> uint8 [..., 2] holding the little-endian binary16 encoding."""
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape, 2)


def _rt_f16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).to(torch.float32)


def quantize_q8_0(w: torch.Tensor) -> torch.Tensor:
    rows, cols = w.shape
    x = w.reshape(rows, cols // 32, 32).float()
    d = _rt_f16(x.abs().amax(dim=-1) / 127.0)
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = torch.clamp(torch.round(x * inv[..., None]), -127, 127).to(torch.int8)
    out = torch.cat([_f16_bytes(d), q.view(torch.uint8)], dim=-1)
    return out.reshape(rows, -1)


def _k_scales_pack(sc: torch.Tensor, m: torch.Tensor) -> torch.Tensor:
    """Pack eight 6-bit (scale, min) pairs into 12 bytes; inverse of get_scale_min_k4
    (crates/inferi/src/quantization.rs:394-402)."""
    sc = sc.to(torch.int32)
    m = m.to(torch.int32)
    lo_sc, hi_sc = sc[..., :4], sc[..., 4:]
    lo_m, hi_m = m[..., :4], m[..., 4:]
    b0 = lo_sc | ((hi_sc >> 4) << 6)
    b4 = lo_m | ((hi_m >> 4) << 6)
    b8 = (hi_sc & 0xF) | ((hi_m & 0xF) << 4)
    return torch.cat([b0, b4, b8], dim=-1).to(torch.uint8)


def _quantize_k45(w: torch.Tensor, levels: int):
    rows, cols = w.shape
    nb = cols // QK_K
    x = w.reshape(rows, nb, 8, 32).float()
    mn = torch.clamp(-x.amin(dim=-1), min=0.0)           # non-negative offsets
    sub_scale = (x.amax(dim=-1) + mn) / float(levels)
    d = _rt_f16(sub_scale.amax(dim=-1) / 63.0)
    dmin = _rt_f16(mn.amax(dim=-1) / 63.0)
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    inv_dmin = torch.where(dmin > 0, 1.0 / dmin, torch.zeros_like(dmin))
    sc = torch.clamp(torch.round(sub_scale * inv_d[..., None]), 0, 63)
    m = torch.clamp(torch.round(mn * inv_dmin[..., None]), 0, 63)
    eff = d[..., None] * sc
    inv_eff = torch.where(eff > 0, 1.0 / eff, torch.zeros_like(eff))
    q = torch.clamp(torch.round((x + (dmin[..., None] * m)[..., None]) * inv_eff[..., None]), 0, levels).to(torch.int32)
    header = torch.cat([_f16_bytes(d), _f16_bytes(dmin), _k_scales_pack(sc, m)], dim=-1)  # [rows, nb, 16]
    return q.reshape(rows, nb, 4, 2, 32), header


def quantize_q4_k(w: torch.Tensor) -> torch.Tensor:
    q, header = _quantize_k45(w, 15)
    qs = (q[:, :, :, 0, :] | (q[:, :, :, 1, :] << 4)).to(torch.uint8)      # [rows, nb, 4, 32]
    rows, nb = qs.shape[:2]
    return torch.cat([header, qs.reshape(rows, nb, 128)], dim=-1).reshape(rows, -1)


def quantize_q5_k(w: torch.Tensor) -> torch.Tensor:
    q, header = _quantize_k45(w, 31)
    rows, nb = q.shape[:2]
    lo = q & 0xF
    hi = q >> 4                                                            # [rows, nb, 4(chunk), 2(half), 32]
    qs = (lo[:, :, :, 0, :] | (lo[:, :, :, 1, :] << 4)).to(torch.uint8)
    shifts = torch.arange(8, device=w.device, dtype=torch.int32).reshape(1, 1, 4, 2, 1)   # bit 2*chunk + half
    qh = (hi << shifts).sum(dim=(2, 3)).to(torch.uint8)                    # [rows, nb, 32]
    return torch.cat([header, qh, qs.reshape(rows, nb, 128)], dim=-1).reshape(rows, -1)


def quantize_q6_k(w: torch.Tensor) -> torch.Tensor:
    rows, cols = w.shape
    nb = cols // QK_K
    x = w.reshape(rows, nb, 16, 16).float()
    amax_idx = x.abs().argmax(dim=-1, keepdim=True)
    signed_max = torch.gather(x, -1, amax_idx).squeeze(-1)                 # value with the largest magnitude
    sub_scale = signed_max / -32.0
    d = _rt_f16(sub_scale.abs().amax(dim=-1) / 127.0)
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    sc = torch.clamp(torch.round(sub_scale * inv_d[..., None]), -128, 127)
    eff = d[..., None] * sc
    inv_eff = torch.where(eff != 0, 1.0 / eff, torch.zeros_like(eff))
    q = (torch.clamp(torch.round(x * inv_eff[..., None]), -32, 31) + 32).to(torch.int32)   # 0..63
    # element e = 128 i + 32 g + l ; sub-block index 8 i + 2 g + l // 16
    q = q.reshape(rows, nb, 2, 4, 32)                                      # [.., i, g, l]
    lo, hi = q & 0xF, q >> 4
    ql = torch.stack([lo[:, :, :, 0] | (lo[:, :, :, 2] << 4), lo[:, :, :, 1] | (lo[:, :, :, 3] << 4)], dim=3)  # [.., i, 2, 32]
    qh = hi[:, :, :, 0] | (hi[:, :, :, 1] << 2) | (hi[:, :, :, 2] << 4) | (hi[:, :, :, 3] << 6)              # [.., i, 32]
    out = torch.cat([
        ql.to(torch.uint8).reshape(rows, nb, 128),
        qh.to(torch.uint8).reshape(rows, nb, 64),
        sc.to(torch.int8).view(torch.uint8).reshape(rows, nb, 16),
        _f16_bytes(d),
    ], dim=-1)
    return out.reshape(rows, -1)


def quantize(qtype: int, w: torch.Tensor) -> torch.Tensor:
    """f32 [rows, cols] -> uint8 [rows, row_bytes] in GGUF block layout."""
    if w.dim() != 2:
        raise ValueError("quantize expects a rank-2 tensor")
    row_bytes(qtype, w.shape[1])
    if qtype == F32:
        return w.float().contiguous().view(torch.uint8).reshape(w.shape[0], -1)
    fn = {Q8_0: quantize_q8_0, Q4_K: quantize_q4_k, Q5_K: quantize_q5_k, Q6_K: quantize_q6_k}.get(qtype)
    if fn is None:
        raise ValueError(f"unsupported qtype {qtype}")
    return fn(w).contiguous()
