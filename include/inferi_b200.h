/*
 * inferi_b200 — C ABI of the B200-native (sm_100a) batch-1 Llama token loop over GGUF-quantized weights.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns an int32_t status
 * (IB_OK == 0) and never throws or aborts.  `ib_last_error_string()` gives the text of the last
 * failure on the calling thread.  "dev" pointers are CUDA device pointers on the context's device;
 * `stream` is a `cudaStream_t` passed as `void*` (NULL = the legacy default stream).  Handles are not
 * thread-safe; distinct handles may be used from distinct threads.
 *
 * Each declaration cites the interface of the reference project (dimforge/inferi, paths relative to
 * its root) that it replaces.
 */
#ifndef INFERI_B200_H
#define INFERI_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define IB_API __attribute__((visibility("default")))
#else
#define IB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ---- */
enum {
    IB_OK = 0,
    IB_ERR_INVALID = 1,      /* bad argument: null handle, shape contract violated, unsupported type */
    IB_ERR_CUDA = 2,         /* a CUDA runtime call failed */
    IB_ERR_OOM = 3,          /* device allocation failed */
    IB_ERR_UNSUPPORTED = 4,  /* valid request this build cannot serve */
    IB_ERR_TIMEOUT = 5,      /* a bounded device-side wait gave up */
    IB_ERR_COMM = 6          /* tensor-parallel set-up or exchange failed */
};

/* GGUF tensor type ids (crates/inferi/src/gguf.rs:74-106). */
/* Q8_0, Q4_K, Q5_K, Q6_K run on the streaming kernels (the token loop needs them); Q4_0, Q4_1, Q5_0, Q5_1, Q8_K complete the
 * reference's `GpuQuantTensor` variants at the op level (ib_gemv_quant) on the generic kernel. */
enum { IB_F32 = 0, IB_Q4_0 = 2, IB_Q4_1 = 3, IB_Q5_0 = 6, IB_Q5_1 = 7, IB_Q8_0 = 8, IB_Q4_K = 12, IB_Q5_K = 13, IB_Q6_K = 14, IB_Q8_K = 15 };

/* KV-cache element type.  F32 is the reference's layout (crates/inferi/src/models/llama2/transformer.rs:85-104);
 * F16 halves the cache traffic and is what the throughput figures are quoted on. */
enum { IB_KV_F32 = 0, IB_KV_F16 = 1 };

/* RoPE variants (crates/inferi/src/ops/rope.rs:12-23). */
enum { IB_ROPE_ORIGINAL = 0, IB_ROPE_NEOX = 1 };

typedef struct ib_ctx ib_ctx;
typedef struct ib_qtensor ib_qtensor;
typedef struct ib_llama ib_llama;

IB_API const char *ib_last_error_string(void);

/* Replaces `LlmOps::new` (crates/inferi/src/context.rs:58-85): binds a device and owns scratch memory. */
IB_API int32_t ib_ctx_create(int32_t device, ib_ctx **out);
IB_API int32_t ib_ctx_destroy(ib_ctx *ctx);
/* Number of kernels this context has launched since creation (or since the last reset). */
IB_API int32_t ib_ctx_launch_count(ib_ctx *ctx, uint64_t *out);
IB_API int32_t ib_ctx_reset_launch_count(ib_ctx *ctx);
/* Every wait inside a kernel (on a shared-memory barrier, on another rank's arrival) is bounded; a wait that gives up makes
 * the next synchronising call return IB_ERR_TIMEOUT while the context stays usable (the reference has no such waits: its
 * errors are `GpuBackendError`s and panics, crates/inferi/src/ops/gemv_quant.rs:113-122).  The limit, 2 s by default,
 * applies to launches issued or recorded into a model's token graph after this call. */
IB_API int32_t ib_ctx_set_wait_limit(ib_ctx *ctx, uint64_t nanoseconds);

/* Raw device memory for callers without a CUDA runtime of their own (the reference allocates through
 * `Tensor::vector` / `TensorBuilder`, crates/inferi/src/ops/gemv_quant.rs:459-490). */
IB_API int32_t ib_malloc(ib_ctx *ctx, uint64_t nbytes, void **out_dev);
IB_API int32_t ib_free(ib_ctx *ctx, void *dev);
IB_API int32_t ib_memcpy_h2d(ib_ctx *ctx, void *stream, void *dst_dev, const void *src_host, uint64_t nbytes);
IB_API int32_t ib_memcpy_d2h(ib_ctx *ctx, void *stream, void *dst_host, const void *src_dev, uint64_t nbytes);
IB_API int32_t ib_stream_sync(ib_ctx *ctx, void *stream);

/* Replaces `GgufTensor::to_gpu_quant` (crates/inferi/src/gguf.rs:141-197, 361) and `GpuQuantTensor`
 * (crates/inferi/src/quantized_matrix.rs:11-54): uploads a [rows, cols] matrix given as consecutive GGUF
 * blocks, row-major.  Contracts are checked instead of silently truncated: rows % 4 == 0
 * (crates/inferi/src/ops/gemv_quant.rs:271), cols a multiple of the block length, nbytes exact.
 * The bytes may be re-tiled on the device (same total size) for 128-bit loads.
 * `src_is_device` != 0 means `gguf_blocks` is already a device pointer. */
IB_API int32_t ib_qtensor_upload(ib_ctx *ctx, int32_t qtype, uint64_t rows, uint64_t cols, const void *gguf_blocks,
                          uint64_t nbytes, int32_t src_is_device, ib_qtensor **out);
IB_API int32_t ib_qtensor_destroy(ib_qtensor *qt);
IB_API int32_t ib_qtensor_info(const ib_qtensor *qt, int32_t *qtype, uint64_t *rows, uint64_t *cols, uint64_t *nbytes);

/* Replaces `GemvQuant::launch` (crates/inferi/src/ops/gemv_quant.rs:183-341): out[rows] = W . v[cols].  The streaming kernels
 * take v as 16-bit block fixed point (per 32 columns a scale and two int8 limbs): the result differs from an f32 evaluation by
 * 2e-5 to 1e-4 relative (the reference's shaders accumulate in f32; the tolerance of the parity tests is 1e-3). */
IB_API int32_t ib_gemv_quant(ib_ctx *ctx, void *stream, float *out_dev, const ib_qtensor *m, const float *v_dev);
/* The same call for host buffers: copies v in, runs the kernel, copies out back, synchronises. */
IB_API int32_t ib_gemv_quant_host(ib_ctx *ctx, float *out_host, const ib_qtensor *m, const float *v_host);
/* out[t][r] = sum_c W[r][c] * x[t][c] for n input vectors at once (row-major x [n][cols] and out [n][rows]) on the tensor
 * cores: the building block of prompt prefill.  The reference has no batched form: it repeats `GemvQuant::launch`
 * (crates/inferi/src/ops/gemv_quant.rs:183-341) per token.  Takes Q8_0/Q4_K/Q5_K/Q6_K matrices with rows % 128 == 0 and
 * cols % 256 == 0 (IB_ERR_UNSUPPORTED otherwise); results agree with n GEMVs (ib_gemv_quant
 * quantizes its input vector to 16-bit block fixed point, this call splits it into two f16) to ~1e-4 relative. */
IB_API int32_t ib_gemm_quant(ib_ctx *ctx, void *stream, float *out_dev, const ib_qtensor *m, const float *x_dev, uint32_t n);
/* The feed-forward input half of a layer as one launch: out[r] = (up . x')[r] * silu((gate . x')[r]) with x' = RMSNorm(x) * w
 * when `norm_w_dev` is given (x' = x when it is null).  Replaces the op sequence `rms_norm_assign`, `matmul_quant_assign`
 * (gate), `matmul_quant_assign` (up), `silu` of crates/inferi/src/models/llama2/transformer.rs:454-464.  gate and up must have
 * the same shape and type and meet the alignment rules of the streaming kernel. */
IB_API int32_t ib_ffn_gate_up(ib_ctx *ctx, void *stream, float *out_dev, const ib_qtensor *gate, const ib_qtensor *up, const float *x_dev,
                              const float *norm_w_dev, float eps);

/* Replaces `RmsNorm::launch` (crates/inferi/src/ops/rms_norm.rs:16-69; shader
 * crates/inferi-shaders/src/rms_norm.rs:78-121): out = (x * rsqrt(mean(x^2) + eps)) * w. */
IB_API int32_t ib_rms_norm(ib_ctx *ctx, void *stream, float *out_dev, const float *x_dev, const float *w_dev, uint32_t n, float eps);

/* Replaces `RoPE::launch` (crates/inferi/src/ops/rope.rs:25-95; shader crates/inferi-shaders/src/rope.rs:51-141):
 * rotates q[q_len] and the first kv_dim entries of k in place.  Requires q_len even, q_len >= kv_dim. */
IB_API int32_t ib_rope(ib_ctx *ctx, void *stream, int32_t variant, float *q_dev, uint32_t q_len, float *k_dev, uint32_t kv_dim,
                uint32_t head_size, uint32_t pos, float base_freq);

/* Replaces `Silu::launch` (crates/inferi/src/ops/silu.rs:14-53; shader crates/inferi-shaders/src/silu.rs:24-53):
 * h1 <- h2 * (h1 / (1 + exp(-h1))). */
IB_API int32_t ib_silu_mul(ib_ctx *ctx, void *stream, float *h1_dev, const float *h2_dev, uint32_t n);

/* Replaces `LlmContext::add_assign` (crates/inferi/src/context.rs:516-530): a += b. */
IB_API int32_t ib_add_assign(ib_ctx *ctx, void *stream, float *a_dev, const float *b_dev, uint32_t n);

/* = `AttentionParams` (crates/inferi-shaders/src/batched_multiquery_attention.rs:18-31), field for field. */
typedef struct ib_attn_params {
    uint32_t seq_len;   /* rows allocated in the cache */
    uint32_t kv_dim;    /* n_kv_heads * head_size */
    uint32_t kv_mul;    /* query heads per kv head */
    uint32_t n_heads;   /* query heads */
    uint32_t head_size; /* 64 or 128 */
    uint32_t pos;       /* current position; positions 0..=pos are attended */
} ib_attn_params;

/* Replaces `FusedAttention::launch` (crates/inferi/src/ops/batched_multiquery_attention.rs:27-77; shaders
 * crates/inferi-shaders/src/fused_attention.rs:63-241, 374-617): out[n_heads*head_size] =
 * softmax(q K^T / sqrt(head_size)) V over cache rows [pos+1, kv_dim].  One split-K flash-decoding kernel for
 * every context length (no 2048-token switch). */
IB_API int32_t ib_attention(ib_ctx *ctx, void *stream, const ib_attn_params *params, const float *q_dev, const void *k_cache_dev,
                     const void *v_cache_dev, int32_t kv_dtype, float *out_dev);

/* No counterpart in the reference.  The same attention as ib_attention for callers that must not allocate device
 * memory when they call it (a latency-critical thread that may not take the allocator's locks, a plugin whose host owns
 * the memory budget): it takes no context and calls no cudaMalloc/cudaFree.  The split-K scratch is a fixed array inside
 * the library, so every GPU that loads the library holds about 1 MiB for it until the process exits.
 * Limits: n_heads * (head_size + 2) <= 262144 and at most 256 kv heads, else IB_ERR_UNSUPPORTED with a message.
 * The device that is current when it is called is used, and `stream` must belong to it.  The first call on each device
 * looks the array's address up (cudaGetSymbolAddress) and, where the driver loads modules lazily, is also when the module
 * holding the array is loaded (the driver may allocate and synchronise then): make that first call during set-up, before
 * any stream capture.  The addresses are remembered per device ordinal for the life of the process (cudaDeviceReset
 * invalidates them).
 * All calls share the one array: two calls whose kernels may overlap on the GPU (different streams) race; calls on one
 * stream are safe, each call leaves the array's counters at zero for the next.  After a failed launch or a race the
 * counters are in an undefined state. */
IB_API int32_t ib_attention_static(void *stream, const ib_attn_params *params, const float *q_dev, const void *k_cache_dev,
                                   const void *v_cache_dev, int32_t kv_dtype, float *out_dev);

/* Replaces the greedy branch of `Sampler::sample` (crates/inferi/src/models/sampler.rs:32-36, 54-56), on the
 * device: index of the largest logit, lowest index on ties. */
IB_API int32_t ib_argmax(ib_ctx *ctx, void *stream, const float *logits_dev, uint32_t n, uint32_t *out_dev);

/* Replaces the non-greedy branches of `Sampler::sample` (crates/inferi/src/models/sampler.rs:32-52): logits / temperature,
 * softmax (crates/inferi/src/ops/softmax.rs:130-143), then `sample_mult` (:62-77) when topp <= 0 or >= 1, else
 * `sample_topp` (:84-129), all on the device; `coin` in [0, 1) is the caller's random number (the reference draws it
 * with rand::random()).  temperature == 0 is the arg-max.  The logits are not modified. */
IB_API int32_t ib_sample(ib_ctx *ctx, void *stream, const float *logits_dev, uint32_t n, float temperature, float topp, float coin,
                         uint32_t *out_dev);

/* = `Llama2Config` (crates/inferi/src/models/llama2/cpu.rs:46-66). */
typedef struct ib_llama_config {
    uint32_t hidden_size;
    uint32_t intermediate_size;
    uint32_t num_hidden_layers;
    uint32_t num_attention_heads;
    uint32_t num_key_value_heads;
    uint32_t vocab_size;
    uint32_t max_position_embeddings;
    float rope_theta;
    float rms_norm_eps;
    /* IB_ROPE_ORIGINAL (Llama: adjacent pairs) or IB_ROPE_NEOX (Qwen2: element i with i + head_size/2), as
     * `LlamaModelType::rope_variant` selects (crates/inferi/src/models/llama2/mod.rs:24-29). */
    uint32_t rope_variant;
} ib_llama_config;

/* = `Llama2LayerWeights` (crates/inferi/src/models/llama2/transformer.rs:176-196).  Norm weights are device
 * pointers to f32[hidden]; the matrices are this rank's shards when tp_size > 1. */
typedef struct ib_llama_layer_weights {
    const ib_qtensor *attn_q, *attn_k, *attn_v, *attn_output;
    const ib_qtensor *ffn_gate, *ffn_up, *ffn_down;
    const float *attn_norm_dev, *ffn_norm_dev;
    /* optional f32 biases of q / k / v (Qwen2; transformer.rs:434-442), device pointers or NULL; this rank's rows */
    const float *attn_q_bias_dev, *attn_k_bias_dev, *attn_v_bias_dev;
} ib_llama_layer_weights;

/* = `Llama2Weights` (crates/inferi/src/models/llama2/transformer.rs:176-196, 294-394).  `output == NULL`
 * ties the classifier to `token_embd` (:376-382).  `token_embd` stays quantized; one row is dequantized
 * per token (the reference dequantizes the whole table to f32, :367-374 — same values). */
typedef struct ib_llama_weights {
    const ib_llama_layer_weights *layers; /* [num_hidden_layers] */
    const ib_qtensor *token_embd;         /* [vocab, hidden], never sharded */
    const ib_qtensor *output;             /* [vocab / tp_size, hidden] or NULL */
    const float *output_norm_dev;
} ib_llama_weights;

/* Replaces `Llama2State::new` + `Llama2::new` (crates/inferi/src/models/llama2/transformer.rs:46-137, 400-407):
 * allocates activations and the per-layer KV cache [max_pos, kv_dim / tp_size] and records the token graph. */
IB_API int32_t ib_llama_create(ib_ctx *ctx, const ib_llama_config *config, const ib_llama_weights *weights, int32_t kv_dtype,
                        int32_t tp_rank, int32_t tp_size, ib_llama **out);
IB_API int32_t ib_llama_destroy(ib_llama *model);

/* Replaces `Llama2::launch` + `ChatLlama2::forward_logits` + greedy sampling
 * (crates/inferi/src/models/llama2/transformer.rs:409-481, crates/inferi-chat/src/chat_llama2.rs:191-255):
 * runs one token at `pos`, leaves the greedy next token on the device and, when the host pointers are
 * non-NULL, copies the logits (vocab floats) and/or the next token id back and synchronises. */
IB_API int32_t ib_llama_forward(ib_llama *model, void *stream, uint32_t token, uint32_t pos, float *logits_host, uint32_t *next_token_host);

/* Replaces the token loop of `ChatLlama2::forward` (crates/inferi-chat/src/chat_llama2.rs:137-171) for greedy
 * decoding: feeds `tokens[0..n_prompt)` at positions start_pos.. (each through the decode path, as the
 * reference does), then generates `n_gen` tokens, each fed back on the device.  Only token ids cross PCIe:
 * out_tokens_host[n_gen] receives the generated ids after one synchronisation at the end. */
IB_API int32_t ib_llama_generate(ib_llama *model, void *stream, const uint32_t *tokens_host, uint32_t n_prompt, uint32_t start_pos,
                          uint32_t n_gen, uint32_t *out_tokens_host);

/* Prompt prefill: the n prompt tokens at positions start_pos .. start_pos + n - 1 go through every matrix together, as GEMMs
 * on the tensor cores, instead of one by one.  Fills the KV cache for those positions, leaves the logits of the last
 * prompt position in the model state and returns the greedy token that follows the prompt (`next_token_host` may be
 * null); decoding continues with ib_llama_generate(model, stream, &next, 1, start_pos + n, ...).
 * The reference has no prefill - `ChatLlama2::forward` forces prompt tokens through the decode path one at a time
 * (crates/inferi-chat/src/chat_llama2.rs:137-155, crates/inferi-chat/src/sampler.rs:102-107) - and that loop is what this call
 * must agree with: same cache contents and logits within the logits tolerance (measured: 2.6e-3 max-abs on
 * the 1B architecture), same greedy tokens afterwards.
 * Takes single-GPU models with an f16 cache, 4 query heads per kv head and matrices of 128-row / 256-column multiples
 * (the Llama-3 family); IB_ERR_UNSUPPORTED otherwise, and the prompt then goes through ib_llama_generate. */
IB_API int32_t ib_llama_prefill(ib_llama *model, void *stream, const uint32_t *tokens_host, uint32_t n, uint32_t start_pos, uint32_t *next_token_host);

/* Tensor parallelism inside one NVLink/NVSwitch box (no counterpart in the reference, which is single-GPU): one process
 * per GPU, each creating its model with (tp_rank, tp_size > 1) and ITS SHARD of every matrix — q/k/v, gate/up and the
 * classifier split by rows (heads, FFN units, vocabulary), attn_output and ffn_down split by columns at block
 * granularity (Q6_K: multiples of 2048 columns), token_embd and the norm vectors replicated.  Partial sums of the two
 * row-split GEMVs are exchanged by a one-shot push all-reduce fused into the kernels (peer stores of 8-byte {value, tag}
 * words into each rank's exchange area - the tag names the token and the exchange, so the data is its own arrival signal
 * - every wait bounded).  Set-up: every rank calls ib_llama_tp_export, the hosts exchange
 * the IB_TP_HANDLE_BYTES-byte handles (any transport), every rank calls ib_llama_tp_connect with all handles ordered by
 * rank; only then can the model run.  All ranks must then issue the same forward/generate calls. */
#define IB_TP_HANDLE_BYTES 64
IB_API int32_t ib_llama_tp_export(ib_llama *model, void *handle_out);
IB_API int32_t ib_llama_tp_connect(ib_llama *model, const void *handles_by_rank);
/* The same set-up for a host that runs all ranks in ONE process (one thread or context per GPU, peer access enabled by the
 * host): ib_llama_tp_area gives the device pointer and size of this rank's exchange area, ib_llama_tp_connect_ptrs takes
 * every rank's area as a device pointer valid on this model's GPU, ordered by rank (the entry of the model's own rank is
 * ignored).  No counterpart in the reference. */
IB_API int32_t ib_llama_tp_area(ib_llama *model, void **area_dev, uint64_t *nbytes);
IB_API int32_t ib_llama_tp_connect_ptrs(ib_llama *model, void *const *areas_by_rank);

/* Device pointer of the last forward's logits (f32[vocab / tp_size]) and of the residual stream x (f32[hidden]);
 * for parity checks (the reference exposes `Llama2State::logits`, transformer.rs:15-43). */
/* ib_llama_generate that stops at `eos_token` (the stop test of the reference's chat loop, crates/inferi-chat/src/
 * chat_llama2.rs:157-166): generates at most max_gen tokens, *n_out receives how many are valid (the stop token included).
 * The device loop runs in chunks of 16 tokens between which the host looks for the stop token; the next turn continues at
 * start_pos + n_prompt + *n_out - 1 with the last token as its prompt (KV reuse). */
IB_API int32_t ib_llama_generate_until(ib_llama *model, void *stream, const uint32_t *tokens_host, uint32_t n_prompt, uint32_t start_pos,
                                       uint32_t max_gen, uint32_t eos_token, uint32_t *out_tokens_host, uint32_t *n_out);
/* The token loop of `ChatLlama2::forward` (crates/inferi-chat/src/chat_llama2.rs:92-189) with its event callback.  `out` is
 * called once per generated token with what `ChatEvent::Token` carries (chat_llama2.rs:173-178): the token and its
 * predecessor (the pair `tokenizer.decode(prev, token)` turns into the event's string), `next_pos` = the position whose
 * forward produced it, `token_count` = next_pos - start_pos - 1 and `token_time` = seconds since the forward at
 * start_pos + 1 began - the reference leaves the first forward out of its tok/s (`timing_delay = 1`, :131), so the first
 * event of a one-token prompt carries (0, 0.0).  A non-zero return from `out` ends the turn early (the reference stops when
 * its callback returns Err, :180-183); the stop token ends it without an event (:158-160).  Prompt positions are forced,
 * not sampled.  The device loop runs in chunks of 16 tokens, so the callback sees up to 16 events at once, their times
 * spread evenly over the chunk; prompts of 10 tokens and more go through ib_llama_prefill when the model qualifies.
 * *n_out (may be NULL) receives the number of events delivered; the next turn starts at start_pos + n_prompt + *n_out - 1
 * with the last delivered token as the head of its prompt. */
typedef int32_t (*ib_token_event_fn)(void *user, uint32_t prev_token, uint32_t token, uint32_t next_pos, uint32_t token_count, double token_time);
IB_API int32_t ib_llama_chat(ib_llama *model, void *stream, const uint32_t *tokens_host, uint32_t n_prompt, uint32_t start_pos, uint32_t max_gen,
                             uint32_t eos_token, ib_token_event_fn out, void *user, uint32_t *n_out);
/* ≙ `Sampler::new(vocab, temperature, topp)` (models/sampler.rs:22-30) for the model's own token loop: after this,
 * ib_llama_forward / ib_llama_generate feed back sampled tokens instead of the arg-max (temperature 0 = greedy again).
 * The coin of a position is splitmix64(seed, position) -> [0, 1), so a run can be reproduced.  Single GPU only. */
IB_API int32_t ib_llama_set_sampler(ib_llama *model, float temperature, float topp, uint64_t seed);
IB_API int32_t ib_llama_state(ib_llama *model, const float **logits_dev, const float **x_dev);

/* ---- GGUF container and GGUF -> device loader ----
 * Replaces `Gguf::from_bytes` (crates/inferi/src/gguf.rs:516-692: header, metadata, tensor table, data alignment),
 * `Llama2Config::from_gguf` (crates/inferi/src/models/llama2/cpu.rs:74-107) and `Llama2Weights::from_gguf`
 * (crates/inferi/src/models/llama2/transformer.rs:294-394).  The file is memory-mapped; tensors go to the device straight
 * from the mapping (no typed copies), `token_embd` stays quantized, a tensor-parallel rank uploads only its slice.
 * Malformed files give IB_ERR_INVALID (the reference panics on rank > 4, gguf.rs:583-586). */
typedef struct ib_gguf ib_gguf;

typedef struct ib_gguf_tensor_info {
    int32_t type;        /* ggml tensor type id (gguf.rs:74-106) */
    uint32_t n_dims;
    uint64_t dims[4];    /* slowest first: a matrix is [rows, cols] (the file stores them fastest first, gguf.rs:587-593) */
    uint64_t offset;     /* from the start of the file */
    uint64_t nbytes;     /* 0 for a type this reader does not size */
    const void *data;    /* inside the mapping; valid until ib_gguf_close */
} ib_gguf_tensor_info;

IB_API int32_t ib_gguf_open(const char *path, ib_gguf **out);
IB_API int32_t ib_gguf_open_memory(const void *bytes, uint64_t nbytes, ib_gguf **out);   /* the caller keeps the bytes alive */
IB_API int32_t ib_gguf_close(ib_gguf *g);
IB_API int32_t ib_gguf_counts(const ib_gguf *g, uint32_t *version, uint64_t *n_tensors, uint64_t *n_metadata, uint32_t *alignment);
IB_API int32_t ib_gguf_tensor_by_name(const ib_gguf *g, const char *name, ib_gguf_tensor_info *info);
IB_API int32_t ib_gguf_tensor_by_index(const ib_gguf *g, uint64_t index, char *name_out, uint64_t name_cap, ib_gguf_tensor_info *info);
/* Metadata (gguf.rs:397-513).  Value type ids: 0 U8, 1 I8, 2 U16, 3 I16, 4 U32, 5 I32, 6 F32, 7 Bool, 8 String, 9 Array,
 * 10 U64, 11 I64, 12 F64.  Numbers of any type read as u64 (two's complement for signed) or f64. */
IB_API int32_t ib_gguf_meta_key(const ib_gguf *g, uint64_t index, char *key_out, uint64_t key_cap, int32_t *type);
IB_API int32_t ib_gguf_meta_u64(const ib_gguf *g, const char *key, uint64_t *value);
IB_API int32_t ib_gguf_meta_f64(const ib_gguf *g, const char *key, double *value);
IB_API int32_t ib_gguf_meta_str(const ib_gguf *g, const char *key, char *out, uint64_t cap, uint64_t *len);
IB_API int32_t ib_gguf_meta_array(const ib_gguf *g, const char *key, int32_t *elem_type, uint64_t *count, const void **data);
IB_API int32_t ib_gguf_meta_array_str(ib_gguf *g, const char *key, uint64_t index, char *out, uint64_t cap, uint64_t *len);
/* `arch`: metadata prefix, null = "llama".  vocab_size = length of tokenizer.ggml.tokens (rows of token_embd.weight when
 * the file carries no tokenizer); rope_theta and rms_norm_eps default to 10000 and 1e-6 as in the reference. */
IB_API int32_t ib_gguf_llama_config(const ib_gguf *g, const char *arch, ib_llama_config *out);
/* Uploads this rank's share of every tensor and creates the model, which owns the uploaded weights (ib_llama_destroy frees
 * them; the file may be closed afterwards).  `max_context` > 0 caps the KV cache below the file's context length.
 * With tp_size > 1 continue with ib_llama_tp_export / ib_llama_tp_connect. */
IB_API int32_t ib_gguf_load_llama(ib_ctx *ctx, const ib_gguf *g, const char *arch, int32_t kv_dtype, uint32_t max_context, int32_t tp_rank,
                                  int32_t tp_size, ib_llama **out);

/* ---- Llama tokenizer from GGUF metadata ----
 * Replaces `LlamaTokenizer::from_gguf` / `encode` / `decode` (crates/inferi/src/models/tokenizers/llama2_tokenizer.rs:23-180):
 * vocabulary `tokenizer.ggml.tokens`, merge scores `tokenizer.ggml.scores`, ids `tokenizer.ggml.{bos,eos,unknown}_token_id`.
 * Same results as the reference, quirks included (see csrc/tokenizer.cu); an empty text without bos gives an empty list
 * where the reference panics. */
typedef struct ib_tokenizer ib_tokenizer;
IB_API int32_t ib_tokenizer_llama_from_gguf(ib_gguf *g, ib_tokenizer **out);
/* GPT-2 byte-pair encoding (Llama-3 files): replaces `Gpt2Tokenizer::from_gguf` / `encode` / `decode` (crates/inferi/src/
 * models/tokenizers/gpt2_tokenizer.rs:54-217) from `tokenizer.ggml.tokens`, `tokenizer.ggml.merges` and the bos / eos ids.
 * "<...>" stretches of the text are looked up whole as special tokens; one that is not in the vocabulary is
 * IB_ERR_INVALID (the reference panics).  ib_tokenizer_decode ignores prev_token for this kind. */
IB_API int32_t ib_tokenizer_gpt2_from_gguf(ib_gguf *g, ib_tokenizer **out);
IB_API int32_t ib_tokenizer_destroy(ib_tokenizer *t);
IB_API int32_t ib_tokenizer_info(const ib_tokenizer *t, uint32_t *vocab_size, uint32_t *bos, uint32_t *eos, uint32_t *unk);
/* `out` may be null to ask for the count only. */
IB_API int32_t ib_tokenizer_encode(const ib_tokenizer *t, const char *text_utf8, uint64_t text_len, int32_t add_bos, int32_t add_eos, uint32_t *out,
                                   uint64_t cap, uint64_t *n_out);
/* The text of `token` given the token before it (the reference strips leading whitespace after the bos token). */
IB_API int32_t ib_tokenizer_decode(const ib_tokenizer *t, uint32_t prev_token, uint32_t token, char *out, uint64_t cap, uint64_t *len);

#ifdef __cplusplus
}
#endif
#endif /* INFERI_B200_H */
