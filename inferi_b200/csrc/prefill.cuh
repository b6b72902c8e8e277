// Prompt prefill on the tensor cores: what the model code (llama.cu) uses of prefill.cu.
#pragma once

#include "token.cuh"

namespace ib {

constexpr uint32_t PREFILL_MAX_TOKENS = 128;   // tokens per GEMM (the N of the MMA); longer prompts go in chunks

enum PrefillEpilogue : uint32_t { PE_Q = 0, PE_K = 1, PE_V = 2, PE_RESIDUAL = 3, PE_SWIGLU = 4, PE_STORE = 5 };
struct PrefillEpiParams {
    const float *planes, *planes2;   // [ksplit][n][rows] partial sums (planes2: the up matrix of PE_SWIGLU)
    uint32_t ksplit, n, rows, mode;
    const float *bias;               // PE_Q / PE_K / PE_V, or null
    const float *theta;              // [head_size / 2]
    uint32_t head_size, pos0, kv_dim, kv_dtype;
    float *out;                      // PE_Q: q [n][rows]; PE_RESIDUAL: X [n][rows] (added to); PE_STORE: [n][rows]
    void *cache;                     // PE_K / PE_V: this layer's cache [max_pos][kv_dim]
    __half *hi, *lo;                 // PE_SWIGLU: the product, split, [n_pad][rows]
};


uint32_t prefill_ksplit(const ib_ctx *ctx, uint32_t rows, uint32_t cols);
bool prefill_gemm_eligible(const ib_qtensor *m);
// planes[ksplit][n][rows] = partial sums of W . x_t over the K ranges; x_hi / x_lo: 128 x cols halves in the tiled layout that
// launch_prefill_norm_split and the PE_SWIGLU epilogue write (one 16 KiB tile per 64 columns), rows n .. (n rounded up to 16) - 1 zero
int32_t launch_prefill_gemm(ib_ctx *ctx, cudaStream_t s, const ib_qtensor *m, const __half *x_hi, const __half *x_lo, uint32_t n, float *planes, uint32_t ksplit);
int32_t launch_prefill_embed(ib_ctx *ctx, cudaStream_t s, const ib_qtensor *embd, const uint32_t *tokens_dev, uint32_t n, uint32_t vocab, float *X);
int32_t launch_prefill_norm_split(ib_ctx *ctx, cudaStream_t s, const float *X, const float *w, float eps, uint32_t n, uint32_t cols, __half *hi, __half *lo);
int32_t launch_prefill_epilogue(ib_ctx *ctx, cudaStream_t s, const PrefillEpiParams &p);

}  // namespace ib
