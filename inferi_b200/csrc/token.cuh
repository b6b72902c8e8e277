// The token loop's device control block and the quantized-row descriptor of the embedding table.
#pragma once

#include "attention.cuh"
#include "common.cuh"

namespace ib {

struct TokenCtl {
    uint32_t step;      // index into seq of the token being processed
    uint32_t pos;       // its position in the context
    uint32_t n_prompt;  // tokens of seq that are given; beyond them the arg-max is fed back
    uint32_t next;      // greedy token of the last forward
};

struct QDesc {
    const uint8_t *w;
    uint64_t row_bytes;
    uint32_t qtype, layout, nb;
};

__device__ __forceinline__ float half_at(const uint8_t *p) {
    return __half2float(__ushort_as_half((unsigned short)((uint32_t)p[0] | ((uint32_t)p[1] << 8))));
}

// Value of element `col` of a quantized row under either device layout (block arithmetic of
// crates/inferi/src/quantization.rs:51-54, 227-256, 287-329, 364-402).
__device__ inline float dequant_at(const QDesc &q, const uint8_t *row, uint32_t col) {
    if (q.qtype == IB_F32) return reinterpret_cast<const float *>(row)[col];
    if (q.qtype == IB_Q8_0) {
        const uint32_t b = col >> 5, i = col & 31;
        if (q.layout == LAYOUT_SOA) {
            const uint8_t *grp = row + (size_t)(b >> 3) * 272;
            return (float)(int8_t)grp[32 * (b & 7) + i] * half_at(grp + 256 + 2 * (b & 7));
        }
        const uint8_t *blk = row + (size_t)b * 34;
        return (float)(int8_t)blk[2 + i] * half_at(blk);
    }
    const uint32_t b = col >> 8, e = col & 255;
    if (q.qtype == IB_Q4_K || q.qtype == IB_Q5_K) {
        const uint8_t *blk = row + (size_t)b * (q.qtype == IB_Q4_K ? 144 : 176);
        const uint8_t *sc = blk + 4, *qs = blk + (q.qtype == IB_Q4_K ? 16 : 48);
        const uint32_t c = e >> 6, hi = (e >> 5) & 1, l = e & 31, j = 2 * c + hi;
        uint32_t s, m;
        if (j < 4) { s = sc[j] & 63; m = sc[j + 4] & 63; }
        else { s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4); m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
        uint32_t qv = hi ? (qs[32 * c + l] >> 4) : (qs[32 * c + l] & 0xF);
        if (q.qtype == IB_Q5_K && (blk[16 + l] & ((hi ? 2u : 1u) << (2 * c)))) qv += 16;
        return half_at(blk) * (float)s * (float)qv - half_at(blk + 2) * (float)m;
    }
    // Q6_K
    const uint8_t *ql, *qh, *sc, *dp;
    if (q.layout == LAYOUT_SOA) {
        const uint8_t *grp = row + (size_t)(b >> 3) * 1680;
        const uint32_t bb = b & 7;
        ql = grp + 128 * bb; qh = grp + 1024 + 64 * bb; sc = grp + 1536 + 16 * bb; dp = grp + 1664 + 2 * bb;
    } else {
        const uint8_t *blk = row + (size_t)b * 210;
        ql = blk; qh = blk + 128; sc = blk + 192; dp = blk + 208;
    }
    const uint32_t i = e >> 7, g = (e >> 5) & 3, l = e & 31;
    const uint32_t lo = ql[64 * i + 32 * (g & 1) + l], h = qh[32 * i + l];
    const int qv = (int)(((g & 2) ? (lo >> 4) : (lo & 0xF)) | (((h >> (2 * g)) & 3) << 4)) - 32;
    return half_at(dp) * (float)(int8_t)sc[8 * i + 2 * g + l / 16] * (float)qv;
}

}  // namespace ib
