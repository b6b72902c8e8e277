// Shared declarations of the inferi_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <string>

#include "../../include/inferi_b200.h"

namespace ib {

// ---------------------------------------------------------------------------------------------
// errors: every entry point returns a status and leaves the text in a thread-local string
// ---------------------------------------------------------------------------------------------
int32_t set_error(int32_t code, const char *fmt, ...);

#define IB_CHECK_CUDA(expr)                                                                             \
    do {                                                                                                \
        cudaError_t _e = (expr);                                                                        \
        if (_e != cudaSuccess)                                                                          \
            return ib::set_error(_e == cudaErrorMemoryAllocation ? IB_ERR_OOM : IB_ERR_CUDA, "%s failed: %s (%s:%d)", \
                                 #expr, cudaGetErrorString(_e), __FILE__, __LINE__);                    \
    } while (0)

#define IB_REQUIRE(cond, ...)                                      \
    do {                                                           \
        if (!(cond)) return ib::set_error(IB_ERR_INVALID, __VA_ARGS__); \
    } while (0)

// ---------------------------------------------------------------------------------------------
// quantized tensors
// ---------------------------------------------------------------------------------------------
constexpr int QK_K = 256;

// Device layouts.  GGUF: the file's array-of-blocks byte stream, untouched.  SOA: every run of 8 blocks of a row
// re-tiled into sections of equal fields (same bytes, same row length) so that every 128-bit access is aligned and a
// row stays one contiguous stream that can be cut at any multiple of 8 blocks:
//   Q8_0: [8 x 32 B quants][8 x 2 B f16 scale]                              = 272 B per 256 columns
//   Q6_K: [8 x 128 B ql][8 x 64 B qh][8 x 16 B scales][8 x 2 B f16 d]       = 1680 B per 2048 columns
enum Layout : uint32_t { LAYOUT_GGUF = 0, LAYOUT_SOA = 1 };

__host__ __device__ inline uint32_t block_bytes(int qtype) {
    switch (qtype) {
    case IB_F32: return 4;
    case IB_Q8_0: return 34;
    case IB_Q4_K: return 144;
    case IB_Q5_K: return 176;
    case IB_Q6_K: return 210;
    case IB_Q4_0: return 18;
    case IB_Q4_1: return 20;
    case IB_Q5_0: return 22;
    case IB_Q5_1: return 24;
    case IB_Q8_K: return 292;
    default: return 0;
    }
}
__host__ __device__ inline uint32_t block_elems(int qtype) {
    switch (qtype) {
    case IB_F32: return 1;
    case IB_Q8_0: case IB_Q4_0: case IB_Q4_1: case IB_Q5_0: case IB_Q5_1: return 32;
    case IB_Q4_K: case IB_Q5_K: case IB_Q6_K: case IB_Q8_K: return QK_K;
    default: return 0;
    }
}

}  // namespace ib

struct ib_ctx {
    int device = 0;
    int sm_count = 0;
    uint64_t launches = 0;
    // attention split-K scratch (partials + per-kv-head arrival counters), grown on demand
    float *attn_scratch = nullptr;
    size_t attn_scratch_bytes = 0;
    unsigned int *attn_counters = nullptr;
    // argmax scratch
    unsigned long long *argmax_scratch = nullptr;
    unsigned int *argmax_counter = nullptr;
    // error word raised by kernels whose bounded waits give up: mapped pinned host memory, so the host reads it
    // after any synchronisation without a copy
    uint32_t *err_host = nullptr;
    uint32_t *err_dev = nullptr;
    // (claimed, finished) counter pairs through which the CTAs of a streaming GEMV launch share out its tiles; launch i
    // uses pair i mod IB_STREAM_COUNTER_PAIRS (only neighbouring launches overlap), its last CTA clears the pair
    uint32_t *stream_counters = nullptr;
    uint64_t stream_seq = 0;
    // scratch of the tensor-core GEMM entry point (input halves + partial planes), grown on demand
    void *tc_scratch = nullptr;
    size_t tc_scratch_bytes = 0;
    // limit of every wait inside a kernel (on a shared-memory barrier, on another rank's arrival); ib_ctx_set_wait_limit
    uint64_t wait_limit_ns = 2000000000ull;
};
constexpr uint32_t IB_STREAM_COUNTER_PAIRS = 16;

struct ib_qtensor {
    ib_ctx *ctx = nullptr;
    int32_t qtype = 0;
    uint32_t layout = ib::LAYOUT_GGUF;
    bool fast = false;          // eligible for the 128-bit-load kernels
    uint64_t rows = 0, cols = 0;
    uint64_t row_bytes = 0, nbytes = 0;
    uint32_t nb = 0;            // blocks per row
    uint8_t *dev = nullptr;
};

namespace ib {

// ---------------------------------------------------------------------------------------------
// GEMV launch description (gemv.cu)
// ---------------------------------------------------------------------------------------------
struct GemvSeg {
    const uint8_t *w;
    float *out;
    uint64_t row_bytes;
    uint32_t rows, qtype, layout, nb;
};

enum GemvEpilogue : uint32_t {
    EPI_STORE = 0,     // out[r] = dot
    EPI_RESIDUAL = 1,  // out[r] = resid[r] + dot
    EPI_SWIGLU = 2,    // seg0 = gate, seg1 = up: seg0.out[r] = up * gate / (1 + exp(-gate))
    EPI_QKV = 3,       // seg0 = q (rope, store f32), seg1 = k (rope, store to cache), seg2 = v (store to cache)
    EPI_ARGMAX = 4,    // store (if out != null) and track the arg-max over all rows
    EPI_PUSH = 5       // tensor parallel: store the pair into every rank's partial-sum slot of this rank (peer stores)
};

constexpr int IB_MAX_TP = 8;

struct GemvParams {
    GemvSeg seg[3];
    uint32_t nseg, cols, epi;
    const float *x;        // f32 input vector [cols]
    const float *norm_w;   // non-null: x is RMS-normalised with these weights first
    float eps;
    const float *resid;    // EPI_RESIDUAL
    // EPI_QKV
    const uint32_t *pos_ptr;    // device scalar: current position
    const float2 *rope_cs;      // [head_size/2] (cos, sin) of pos * theta_j for the current token
    uint32_t head_size, kv_dim, kv_dtype;
    void *k_cache, *v_cache;    // [max_pos, kv_dim] of this layer
    uint32_t *tile_claim;       // streaming kernel: [claimed, finished] counters of this launch (set by its launcher)
    const float *bias[3];       // optional f32 bias per segment, added before the rotation (Qwen2: transformer.rs:434-442)
    // EPI_ARGMAX
    unsigned long long *argmax_slots;  // one packed (value, ~index) per CTA
    unsigned int *argmax_counter;
    uint32_t *argmax_out;
    uint32_t row_offset;               // added to the row index (tensor-parallel vocabulary shard)
    uint32_t pdl;                      // 1: launched with programmatic dependent launch
    uint32_t pair_instance;            // 1: run Q4_K-only / Q6_K-only launches on the two-format instance too (shared code across a token graph)
    uint32_t *err;                     // device view of the context's error word (set by launch_gemv)
    unsigned long long wait_ns;        // how long a wait inside the kernel may last before it gives up (set by launch_gemv)
    // ---- tensor parallel (tp > 1): one-shot push all-reduce fused into epilogue and prologue ----
    // Every value travels as an 8-byte word {f32 value, u32 tag}: the tag names the exchange ((*epoch) * exchanges per token
    // + number of the exchange inside the token, never 0), 8-byte stores and loads are single transactions, so a reader that
    // sees the tag it expects has the value - no fence and no separate flag between the ranks.
    uint32_t tp;                                // number of ranks; 0 or 1 = single GPU
    const uint32_t *epoch_ptr;                  // device scalar: completed token-graph launches
    uint32_t xchg_per_epoch;                    // exchanges per token (2 per layer)
    // EPI_PUSH: rank p keeps this rank's partial sums at push_dst[p] ([hidden] words); push_use = number of the exchange
    uint2 *push_dst[IB_MAX_TP];
    uint32_t push_use;
    // prologue: x_out = x + sum over ranks of reduce_src[r][cols] (words tagged with exchange number reduce_use).  The sum is
    // formed once per rank: the CTAs share out the vector in groups of 32 columns, add their groups' count to reduce_done,
    // and every CTA reads x_out once reduce_done has reached ((*epoch) * xchg_per_epoch + reduce_use) * (cols / 32).
    const uint2 *reduce_src;
    uint32_t reduce_use;
    float *x_out;                               // the reduced residual stream (the other of two buffers)
    uint32_t *reduce_done;
    // EPI_ARGMAX with a sharded vocabulary: this rank's candidate goes to amax_dst[p] of every rank
    unsigned long long *amax_dst[IB_MAX_TP];
    uint32_t *amax_flag[IB_MAX_TP];
};

int32_t launch_gemv(ib_ctx *ctx, cudaStream_t stream, const GemvParams &p);
bool gemv_stream_eligible(const GemvParams &p);
int32_t launch_gemv_stream(ib_ctx *ctx, cudaStream_t stream, const GemvParams &p);
// IB_OK, or IB_ERR_TIMEOUT when a kernel raised the context's error word (call after a synchronisation)
int32_t check_device_error(ib_ctx *ctx);
int32_t launch_gemv_generic(ib_ctx *ctx, cudaStream_t stream, const ib_qtensor *m, const float *v, float *out);
int32_t retile_to_soa(ib_ctx *ctx, cudaStream_t stream, int qtype, const uint8_t *src, uint8_t *dst, uint64_t rows, uint32_t nb);
bool gemv_fast_eligible(int qtype, uint64_t rows, uint64_t cols);
void fill_seg(GemvSeg &s, const ib_qtensor *m, float *out);

// ops.cu
int32_t launch_rms_norm(ib_ctx *ctx, cudaStream_t s, float *out, const float *x, const float *w, uint32_t n, float eps);
int32_t launch_rope(ib_ctx *ctx, cudaStream_t s, int variant, float *q, uint32_t q_len, float *k, uint32_t kv_dim, uint32_t head_size,
                    uint32_t pos, float base_freq);
int32_t launch_silu_mul(ib_ctx *ctx, cudaStream_t s, float *h1, const float *h2, uint32_t n);
int32_t launch_add_assign(ib_ctx *ctx, cudaStream_t s, float *a, const float *b, uint32_t n);
int32_t launch_argmax(ib_ctx *ctx, cudaStream_t s, const float *x, uint32_t n, uint32_t *out);
int32_t ensure_argmax_scratch(ib_ctx *ctx);
// sampler.cu
int32_t launch_sample(ib_ctx *ctx, cudaStream_t s, const float *logits, uint32_t n, float temperature, float topp, uint64_t seed, const uint32_t *pos_ptr,
                      float coin, float *probs, unsigned long long *keys, uint32_t *out, uint32_t *out2, uint32_t pdl);
size_t sample_keys_capacity(uint32_t n);

// attention.cu
struct AttnLaunch {
    ib_attn_params p;          // p.pos is ignored when pos_ptr != null
    const uint32_t *pos_ptr;   // device scalar (graph replay) or null
    const float *q;
    const void *k_cache, *v_cache;
    int kv_dtype;
    float *out;
    float *scratch;            // [n_kv_heads][max_splits][kv_mul][head_size + 2]
    unsigned int *counters;    // [n_kv_heads], zero before the first launch; the kernel re-zeroes them
    uint32_t max_splits;
    uint32_t pdl;
    // With pos_ptr (a graph node that serves many positions): the caller promises that the position stays below
    // attn_cluster_positions(); the launch then groups a kv head's slices into a thread-block cluster and merges them there.
    // Such a launch is slower at long contexts (clusters constrain the placement of the grid's one wave of CTAs), so a graph
    // for longer contexts is recorded without it.  With a host-known position the launch decides by itself.
    uint32_t short_context;
    // batched launch (prompt prefill): n_queries > 1 queries at positions p.pos, p.pos + 1, ...; steps in elements between
    // consecutive queries' q / out / scratch / counters.  Only the kernel for the Llama-3 shape takes it.
    uint32_t n_queries, q_step, out_step, counter_step;
    size_t scratch_step;
};
bool attn_gqa4_eligible(const AttnLaunch &a);
size_t attn_scratch_bytes(const ib_attn_params &p, uint32_t max_splits);
uint32_t attn_max_splits(const ib_ctx *ctx, const ib_attn_params &p);
int32_t launch_attention(ib_ctx *ctx, cudaStream_t s, const AttnLaunch &a);
uint32_t attn_cluster_positions(const AttnLaunch &a);   // positions (pos + 1) up to which `short_context` may be set; 0: never

}  // namespace ib
