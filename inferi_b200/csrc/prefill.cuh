// Prompt prefill on the tensor cores: what the model code (llama.cu) uses of prefill.cu.
#pragma once

#include "token.cuh"

namespace ib {

constexpr uint32_t PREFILL_MAX_TOKENS = 128;   // tokens per GEMM (the N of the MMA); longer prompts go in chunks

// How a prefill GEMM's work is handed out: the (128-row tile, 256-column block) units, tile-major, are cut into `ctas`
// contiguous, equally long ranges - one per CTA of a grid that fills the GPU exactly once, whatever the matrix's shape
// (a grid of tiles x K slices was 1.5 waves for the FFN matrices).  A tile's K range can then fall to several CTAs; each
// writes its partial sums to the plane numbered by its position among the tile's CTAs, and the element-wise kernel behind
// the GEMM adds a tile's planes in that order.
struct StreamK {
    uint32_t ctas, nb, total;   // CTAs, 256-column blocks per row, units = tiles * nb
    __host__ __device__ uint32_t first_unit(uint32_t c) const { return (uint32_t)(((uint64_t)c * total) / ctas); }
    __host__ __device__ uint32_t cta_of(uint32_t u) const { return (uint32_t)((((uint64_t)u + 1) * ctas - 1) / total); }
    __host__ __device__ uint32_t pieces(uint32_t tile) const { return cta_of(tile * nb + nb - 1) - cta_of(tile * nb) + 1; }
};
StreamK prefill_streamk(const ib_ctx *ctx, uint32_t rows, uint32_t cols);
uint32_t prefill_max_pieces(const StreamK &sk, uint32_t rows);   // most planes any tile of the matrix needs

enum PrefillEpilogue : uint32_t { PE_Q = 0, PE_K = 1, PE_V = 2, PE_RESIDUAL = 3, PE_SWIGLU = 4, PE_STORE = 5 };
struct PrefillEpiParams {
    const float *planes, *planes2;   // [piece][n][rows] partial sums (planes2: the up matrix of PE_SWIGLU)
    StreamK sk;                      // the hand-out of the GEMM that wrote them: rows of tile t have sk.pieces(t) planes
    uint32_t n, rows, mode;
    const float *bias;               // PE_Q / PE_K / PE_V, or null
    const float *theta;              // [head_size / 2]
    uint32_t head_size, pos0, kv_dim, kv_dtype;
    float *out;                      // PE_Q: q [n][rows]; PE_RESIDUAL: X [n][rows] (added to); PE_STORE: [n][rows]
    void *cache;                     // PE_K / PE_V: this layer's cache [max_pos][kv_dim]
    __half *hi, *lo;                 // PE_SWIGLU: the product, split, [n_pad][rows]
};


bool prefill_gemm_eligible(const ib_qtensor *m);
// planes[piece][n][rows] = partial sums of W . x_t over the K ranges of the tile's CTAs; x_hi / x_lo: 128 x cols halves in the tiled layout that
// launch_prefill_norm_split and the PE_SWIGLU epilogue write (one 16 KiB tile per 64 columns), rows n .. (n rounded up to 16) - 1 zero
int32_t launch_prefill_gemm(ib_ctx *ctx, cudaStream_t s, const ib_qtensor *m, const __half *x_hi, const __half *x_lo, uint32_t n, float *planes, const StreamK &sk);
int32_t launch_prefill_embed(ib_ctx *ctx, cudaStream_t s, const ib_qtensor *embd, const uint32_t *tokens_dev, uint32_t n, uint32_t vocab, float *X);
int32_t launch_prefill_norm_split(ib_ctx *ctx, cudaStream_t s, const float *X, const float *w, float eps, uint32_t n, uint32_t cols, __half *hi, __half *lo);
int32_t launch_prefill_epilogue(ib_ctx *ctx, cudaStream_t s, const PrefillEpiParams &p);

}  // namespace ib
