// The token loop's device control block, the quantized-row descriptor of the embedding table, and the program of the
// whole-token kernel (one cooperative launch per token: token_kernel.cu).
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


// ---- whole-token kernel ----
constexpr uint32_t TK_SLOTS = 4;            // tiles in flight per CTA (mbarrier pairs of the byte ring)
constexpr uint32_t TK_TILE_MAX = 75776;     // largest tile in bytes

enum TokenPhaseKind : uint32_t { PH_GEMV = 0, PH_ATTN = 1 };

// One matrix of a phase: what may differ from layer to layer (GGUF mixes give some layers wider formats).
struct __align__(16) LayerMat {
    const uint8_t *w;
    uint32_t row_bytes, qtype;
};

// One phase of the token, in global memory.  The producer warp and the consumer warps read it at the start of the
// phase; what the inner loops need all the time (outputs, cache geometry) is the same for every layer and travels as
// kernel parameters (constant bank) instead.
struct __align__(16) PhaseDesc {
    LayerMat m[3];            // PH_GEMV: 1-3 row segments streamed back to back (q|k|v, gate|up, or a single matrix)
    const float *x;           // input vector [cols]
    const float *norm_w;      // RMSNorm weights applied to x first, or null
    void *k_cache, *v_cache;  // this layer's cache (qkv epilogue, attention)
    uint32_t rows[3];
    uint32_t nseg, epi, cols;
    float eps;
    uint32_t kind;
};
static_assert(sizeof(PhaseDesc) % 16 == 0, "descriptors are read in 16-byte pieces");

struct TokenGeom {
    uint32_t ring_bytes, act_off, act_bytes, part_off, bar_off, tile_max;
};

struct TokenProgram {
    const PhaseDesc *phases;
    uint32_t n_phases;
    GemvParams qkv, res, gu, cls;       // epilogue parameters by kind: q/k/v, residual (o_proj and down), gate/up, classifier
    AttnArgs attn;                      // kc / vc come from the phase
    TokenCtl *ctl;
    uint32_t *seq;
    uint32_t seq_cap;
    QDesc embd;
    uint32_t hidden, vocab, half_head;
    float *x;
    const float *theta;
    float2 *rope_cs;
    uint32_t *grid_bar;                 // arrival counter of the grid barriers (only ever grows)
    uint32_t *epoch;                    // completed tokens
    uint32_t *tile_ctr;                 // [n_phases] tile hand-out counters, zero between tokens
    uint32_t barriers_per_token;
    uint32_t *err;
    uint32_t head_size, kv_mul, kv_dtype;
    TokenGeom geo;
};

struct TokenKernelPlan {
    TokenGeom geo;
    size_t smem_bytes;
    int grid;
    int variant;          // which instance of the kernel serves the model's attention shape
};

// Shared-memory layout for a model, or IB_ERR_UNSUPPORTED if some matrix does not fit the kernel.
int32_t plan_token_kernel(ib_ctx *ctx, const TokenProgram &prog, const PhaseDesc *phases_host, TokenKernelPlan &plan);
int32_t launch_token_kernel(ib_ctx *ctx, cudaStream_t stream, const TokenProgram &prog, const TokenKernelPlan &plan);

}  // namespace ib
