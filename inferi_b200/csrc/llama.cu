// The Llama-architecture token loop: state, per-token kernel sequence, CUDA graph and greedy generation.
//
// Replaces `Llama2State::new` / `Llama2::launch` (crates/inferi/src/models/llama2/transformer.rs:46-137, 409-481)
// and the token loop of `ChatLlama2::forward` / `forward_logits` (crates/inferi-chat/src/chat_llama2.rs:92-255).
//
// Per token the reference records 15 dispatches per layer + 2.  Here a token is 5 kernels per layer + 2:
//   begin      : embedding row dequantisation -> x, RoPE cos/sin table for this position
//   qkv        : RMSNorm(x) prologue, Wq|Wk|Wv GEMV, RoPE on q and k, k/v appended to the cache
//   attention  : split-K flash-decoding over the cache -> xb
//   o_proj     : x += Wo . xb
//   gate_up    : RMSNorm(x) prologue, Wgate and Wup GEMV, SwiGLU -> hb
//   down       : x += Wdown . hb
//   classifier : RMSNorm(x) prologue, Woutput GEMV -> logits, greedy arg-max, token/position bookkeeping
// All of it is captured once into a CUDA graph whose kernels read the token, the position and the step from a
// device control block, so that generation replays the same graph with no host round trip; kernels are chained
// with programmatic dependent launch.
#include "prefill.cuh"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <new>
#include <chrono>
#include <vector>

using namespace ib;

namespace ib {

// begin: x <- dequantized embedding row of the current token (transformer.rs:367-374, chat_llama2.rs:217-220);
// rope_cs[j] <- (cos, sin)(pos * theta_j) shared by every layer of this token (rope.rs:75-79).
__global__ void __launch_bounds__(256) begin_token_kernel(const TokenCtl *ctl, const uint32_t *seq, QDesc embd, uint32_t hidden, float *x,
                                                           const float *theta, uint32_t half_head, float2 *rope_cs, uint32_t vocab, uint32_t pdl) {
    if (pdl) {
        asm volatile("griddepcontrol.launch_dependents;");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    const uint32_t step = ctl->step, pos = ctl->pos;
    uint32_t token = __ldcg(seq + step);
    if (token >= vocab) token = vocab - 1;  // never index outside the table
    const uint8_t *row = embd.w + (size_t)token * embd.row_bytes;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden; i += gridDim.x * blockDim.x) x[i] = dequant_at(embd, row, i);
    if (blockIdx.x == 0 && threadIdx.x < half_head) {
        float sn, cs;
        sincosf((float)pos * theta[threadIdx.x], &sn, &cs);
        rope_cs[threadIdx.x] = make_float2(cs, sn);
    }
}

// end of token: feed the arg-max back when the prompt is exhausted, advance step and position
// (crates/inferi-chat/src/sampler.rs:102-110, chat_llama2.rs:137-171).  With a sharded vocabulary the ranks' candidates
// (packed value / ~index keys, pushed by the classifier kernels) are folded here, on every rank alike.
__global__ void end_token_kernel(TokenCtl *ctl, uint32_t *seq, uint32_t seq_cap, uint32_t *epoch, uint32_t tp, const unsigned long long *amax_slots,
                                 const uint32_t *amax_flag, uint32_t *err, unsigned long long wait_ns, uint32_t pdl) {
    if (pdl) {
        asm volatile("griddepcontrol.launch_dependents;");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        const uint32_t e = *epoch;
        if (tp > 1) {
            const uint32_t target = (e + 1) * tp;
            unsigned long long t0;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
            for (;;) {   // bounded wait for the other ranks' candidates
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(amax_flag) : "memory");
                if ((int32_t)(v - target) >= 0) break;
                unsigned long long t1;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                if (t1 - t0 > wait_ns) {
                    *(volatile uint32_t *)err = 4;
                    __threadfence_system();
                    break;
                }
            }
            unsigned long long best = 0ull;
            for (uint32_t r = 0; r < tp; r++) {
                const unsigned long long k = __ldcg(amax_slots + r);
                best = k > best ? k : best;
            }
            ctl->next = 0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull);
        }
        const uint32_t step = ctl->step;
        if (step + 1 >= ctl->n_prompt && step + 1 < seq_cap) seq[step + 1] = ctl->next;
        ctl->step = step + 1;
        ctl->pos = ctl->pos + 1;
        *epoch = e + 1;   // completed token-graph launches: the cross-GPU arrival counters are compared against it
    }
}

}  // namespace ib

struct ib_llama {
    ib_ctx *ctx = nullptr;
    ib_llama_config cfg{};
    int32_t kv_dtype = IB_KV_F16, tp_rank = 0, tp_size = 1;
    uint32_t head_size = 0, n_heads_l = 0, n_kv_l = 0, q_dim_l = 0, kv_dim_l = 0, ffn_l = 0, vocab_l = 0;
    std::vector<ib_llama_layer_weights> layers;
    const ib_qtensor *token_embd = nullptr, *output = nullptr;
    const float *output_norm = nullptr;
    // device state (transformer.rs:15-43)
    float *x = nullptr, *xb = nullptr, *q = nullptr, *hb = nullptr, *logits = nullptr, *theta = nullptr;
    float2 *rope_cs = nullptr;
    std::vector<void *> k_cache, v_cache;
    TokenCtl *ctl = nullptr;
    uint32_t *seq = nullptr;
    uint32_t seq_cap = 0;
    float *attn_scratch = nullptr;
    unsigned int *attn_counters = nullptr;
    uint32_t attn_splits = 0;
    unsigned long long *argmax_slots = nullptr;
    unsigned int *argmax_counter = nullptr;
    // tensor parallel: a second residual buffer (the reduced stream ping-pongs), this rank's exchange area and the
    // peers' views of theirs (cudaIpc), local CTA counters of the two pushing kernels, completed-launch count
    float *x2 = nullptr;
    uint8_t *comm = nullptr;
    uint8_t *comm_peer[IB_MAX_TP] = {nullptr};
    bool connected = false;
    bool peers_mapped_by_ipc = false;    // the peers' areas were opened with cudaIpcOpenMemHandle (and are closed with the model)
    float *x_final = nullptr;            // buffer that holds the residual stream after the last layer
    uint32_t *reduce_done = nullptr;     // groups of the reduced residual stream stored so far (only ever grows)
    uint32_t *epoch = nullptr;
    uint32_t *h_pinned = nullptr;  // [4 + seq_cap] staging for control block and token ids
    cudaEvent_t staged = nullptr;  // the last copy out of h_pinned has been issued and finished
    cudaGraphExec_t graph_exec = nullptr;
    // the same token for positions below `short_positions`: its attention nodes merge their slices inside thread-block clusters
    cudaGraphExec_t graph_exec_short = nullptr, graph_exec_sample_short = nullptr;
    uint32_t short_positions = 0;
    bool recording_short = false;
    cudaStream_t own_stream = nullptr;
    uint64_t launches_per_token = 0;
    // sampling beyond greedy (ib_llama_set_sampler): parameters, scratch, and the graph that carries the sampler node
    float temperature = 0.f, topp = 0.f;
    uint64_t sample_seed = 0;
    float *sample_probs = nullptr;
    unsigned long long *sample_keys = nullptr;
    cudaGraphExec_t graph_exec_sample = nullptr;
    uint64_t launches_per_token_sample = 0;
    // prompt prefill (ib_llama_prefill): buffers for up to PREFILL_MAX_TOKENS tokens at a time, allocated at the first call
    struct PrefillBuffers {
        float *X = nullptr, *q = nullptr, *att = nullptr, *planes = nullptr, *planes2 = nullptr, *attn_scratch = nullptr;
        __half *hi = nullptr, *lo = nullptr;
        uint32_t *tokens = nullptr;
        unsigned int *attn_counters = nullptr;
        uint32_t attn_splits = 0;
        size_t attn_scratch_step = 0;
        bool ready = false;
    } pf;
    // tensors and device vectors the model owns (a model loaded from a GGUF file frees its weights with itself)
    std::vector<ib_qtensor *> owned_tensors;
    std::vector<void *> owned_device;
};

namespace ib {

// Exchange area of one rank (tensor parallel).  Rank p stores into rank q's area over NVLink (plain peer stores):
//   part[set][rank][hidden]  partial sums of the row-split GEMVs: set 0 = o_proj, set 1 = down
//   amax[rank]               arg-max candidates of the sharded classifier
//   flag[0], flag[1], flag[2] arrival counters of set 0, set 1 and the arg-max exchange (they only ever grow)
struct CommLayout {
    size_t part_bytes, amax_off, flag_off, total;
    CommLayout(uint32_t hidden, int tp) {
        part_bytes = (size_t)tp * hidden * sizeof(uint2);   // {value, tag} words
        amax_off = 2 * part_bytes;
        flag_off = amax_off + (size_t)IB_MAX_TP * sizeof(unsigned long long);
        total = flag_off + 256;
    }
    uint2 *part(uint8_t *base, int set, int rank, uint32_t hidden) const { return reinterpret_cast<uint2 *>(base + set * part_bytes) + (size_t)rank * hidden; }
    unsigned long long *amax(uint8_t *base, int rank) const { return reinterpret_cast<unsigned long long *>(base + amax_off) + rank; }
    uint32_t *flag(uint8_t *base, int i) const { return reinterpret_cast<uint32_t *>(base + flag_off) + i; }
};

static void set_pdl(cudaLaunchConfig_t &cfg, cudaLaunchAttribute *attr, uint32_t pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
}

// Issues the kernels of one token into `s`.
static int32_t record_token(ib_llama *m, cudaStream_t s, uint32_t pdl) {
    ib_ctx *ctx = m->ctx;
    const ib_llama_config &c = m->cfg;
    const int tp = m->tp_size, rank = m->tp_rank;
    const uint32_t H = c.hidden_size, L = c.num_hidden_layers;
    const CommLayout cl(H, tp);
    int32_t rc;
    // every launch of the graph asks for the shared two-format instance where its formats allow (Q4_K_M models: all of them)
    auto emit_gemv = [&](GemvParams p) -> int32_t {
        p.pair_instance = 1;
        return launch_gemv(ctx, s, p);
    };
    auto emit_attn = [&](const AttnLaunch &a) -> int32_t { return launch_attention(ctx, s, a); };
    {
        QDesc e{m->token_embd->dev, m->token_embd->row_bytes, (uint32_t)m->token_embd->qtype, m->token_embd->layout, m->token_embd->nb};
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((H + 255) / 256);
        cfg.blockDim = dim3(256);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        set_pdl(cfg, attr, 0);  // first node of the token graph: nothing to overlap with
        IB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, begin_token_kernel, (const TokenCtl *)m->ctl, (const uint32_t *)m->seq, e, H, m->x,
                                         (const float *)m->theta, m->head_size / 2, m->rope_cs, c.vocab_size, pdl));
        ctx->launches++;
    }
    // Single GPU: the residual stream x is updated in place by the o_proj / down epilogues.
    // Tensor parallel: o_proj / down push partial sums to every rank; the next kernel's prologue adds them to x (fixed rank
    // order) and CTA 0 stores the sum into the other residual buffer, so the stream alternates between x and x2:
    //   qkv(l) reads cur (+ set 1 of layer l-1) ; gate/up(l) reads cur (+ set 0) ; classifier reads cur (+ set 1)
    float *cur = m->x, *other = m->x2;
    // Exchanges of a token are numbered 1 .. 2L in the order they happen: o_proj of layer l is number 2l + 1 (added up by the
    // gate/up kernel of the layer), down of layer l is number 2l + 2 (added up by the next layer's qkv kernel, or by the
    // classifier); the number is part of the tag every exchanged word carries.
    auto add_reduce = [&](GemvParams &p, int set, uint32_t number) {
        if (tp <= 1) return;
        p.tp = (uint32_t)tp; p.epoch_ptr = m->epoch; p.xchg_per_epoch = 2 * L;
        p.reduce_src = cl.part(m->comm, set, 0, H);
        p.reduce_use = number;
        p.reduce_done = m->reduce_done;
        p.x_out = other;
        float *t = cur; cur = other; other = t;
    };
    auto add_push = [&](GemvParams &p, int set, uint32_t number) {
        p.epi = EPI_PUSH; p.tp = (uint32_t)tp; p.epoch_ptr = m->epoch; p.xchg_per_epoch = 2 * L; p.resid = nullptr;
        for (int r = 0; r < tp; r++) p.push_dst[r] = cl.part(m->comm_peer[r], set, rank, H);
        p.push_use = number;
        p.seg[0].out = nullptr;
    };
    ib_attn_params ap{c.max_position_embeddings, m->kv_dim_l, c.num_attention_heads / c.num_key_value_heads, m->n_heads_l, m->head_size, 0};
    for (uint32_t l = 0; l < L; l++) {
        const ib_llama_layer_weights &w = m->layers[l];
        GemvParams p = {};
        // qkv (transformer.rs:420-445)
        fill_seg(p.seg[0], w.attn_q, m->q);
        fill_seg(p.seg[1], w.attn_k, nullptr);
        fill_seg(p.seg[2], w.attn_v, nullptr);
        p.nseg = 3; p.cols = H; p.epi = EPI_QKV; p.x = cur; p.norm_w = w.attn_norm_dev; p.eps = c.rms_norm_eps;
        p.pos_ptr = &m->ctl->pos; p.rope_cs = m->rope_cs; p.head_size = m->head_size; p.kv_dim = m->kv_dim_l; p.kv_dtype = (uint32_t)m->kv_dtype;
        p.k_cache = m->k_cache[l]; p.v_cache = m->v_cache[l]; p.pdl = pdl;
        p.bias[0] = w.attn_q_bias_dev; p.bias[1] = w.attn_k_bias_dev; p.bias[2] = w.attn_v_bias_dev;   // transformer.rs:434-442
        if (l > 0) add_reduce(p, 1, 2 * l);   // the down partials of layer l-1
        if ((rc = emit_gemv(p))) return rc;
        // attention (transformer.rs:448)
        AttnLaunch a = {};
        a.p = ap; a.pos_ptr = &m->ctl->pos; a.q = m->q; a.k_cache = m->k_cache[l]; a.v_cache = m->v_cache[l]; a.kv_dtype = m->kv_dtype;
        a.out = m->xb; a.scratch = m->attn_scratch; a.counters = m->attn_counters; a.max_splits = m->attn_splits; a.pdl = pdl;
        a.short_context = m->recording_short ? 1u : 0u;
        if (l == 0) m->short_positions = attn_cluster_positions(a);
        if ((rc = emit_attn(a))) return rc;
        // o_proj + residual (transformer.rs:450-453)
        p = GemvParams{};
        fill_seg(p.seg[0], w.attn_output, cur);
        p.nseg = 1; p.cols = m->q_dim_l; p.epi = EPI_RESIDUAL; p.x = m->xb; p.resid = cur; p.pdl = pdl;
        if (tp > 1) add_push(p, 0, 2 * l + 1);
        if ((rc = emit_gemv(p))) return rc;
        // gate/up + SwiGLU (transformer.rs:454-464)
        p = GemvParams{};
        fill_seg(p.seg[0], w.ffn_gate, m->hb);
        fill_seg(p.seg[1], w.ffn_up, nullptr);
        p.nseg = 2; p.cols = H; p.epi = EPI_SWIGLU; p.x = cur; p.norm_w = w.ffn_norm_dev; p.eps = c.rms_norm_eps; p.pdl = pdl;
        add_reduce(p, 0, 2 * l + 1);      // the o_proj partials of this layer
        if ((rc = emit_gemv(p))) return rc;
        // down + residual (transformer.rs:465-468)
        p = GemvParams{};
        fill_seg(p.seg[0], w.ffn_down, cur);
        p.nseg = 1; p.cols = m->ffn_l; p.epi = EPI_RESIDUAL; p.x = m->hb; p.resid = cur; p.pdl = pdl;
        if (tp > 1) add_push(p, 1, 2 * l + 2);
        if ((rc = emit_gemv(p))) return rc;
    }
    // classifier + greedy arg-max (transformer.rs:471-478, models/sampler.rs:54-56)
    GemvParams p = {};
    fill_seg(p.seg[0], m->output, m->logits);
    p.nseg = 1; p.cols = H; p.epi = EPI_ARGMAX; p.x = cur; p.norm_w = m->output_norm; p.eps = c.rms_norm_eps;
    p.argmax_slots = m->argmax_slots; p.argmax_counter = m->argmax_counter; p.argmax_out = &m->ctl->next; p.pdl = pdl;
    p.row_offset = (uint32_t)rank * m->vocab_l;
    add_reduce(p, 1, 2 * L);              // the down partials of the last layer
    if (tp > 1)
        for (int r = 0; r < tp; r++) {
            p.amax_dst[r] = cl.amax(m->comm_peer[r], rank);
            p.amax_flag[r] = cl.flag(m->comm_peer[r], 2);
        }
    if ((rc = emit_gemv(p))) return rc;
    m->x_final = cur;
    if (m->temperature > 0.f) {
        // temperature / top-p sampling replaces the greedy token (models/sampler.rs:32-52); the coin is a function of
        // (seed, position)
        if ((rc = launch_sample(ctx, s, m->logits, c.vocab_size, m->temperature, m->topp, m->sample_seed, &m->ctl->pos, 0.f, m->sample_probs, m->sample_keys,
                                &m->ctl->next, nullptr, pdl)))
            return rc;
    }
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1);
        cfg.blockDim = dim3(32);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        set_pdl(cfg, attr, pdl);
        IB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, end_token_kernel, m->ctl, m->seq, m->seq_cap, m->epoch, (uint32_t)tp,
                                         (const unsigned long long *)(tp > 1 ? cl.amax(m->comm, 0) : nullptr),
                                         (const uint32_t *)(tp > 1 ? cl.flag(m->comm, 2) : nullptr), ctx->err_dev, (unsigned long long)ctx->wait_limit_ns, pdl));
        ctx->launches++;
    }
    return IB_OK;
}

// NeoX rotation as a row order.  The NeoX variant rotates element j of a head with element j + head_size/2
// (crates/inferi-shaders/src/rope.rs:96-140); the fused q/k/v epilogue rotates adjacent rows.  Reordering the rows of
// Wq, Wk (and their biases) inside each head as [0, h/2, 1, h/2+1, ...] turns the first into the second, and the
// attention scores do not change when q and k are permuted alike.  dst row r <- src row neox_source_row(r).
__host__ __device__ inline uint32_t neox_source_row(uint32_t r, uint32_t head_size) {
    const uint32_t i = r % head_size;
    return r - i + ((i & 1u) ? head_size / 2 + i / 2 : i / 2);
}

template <typename V>
__global__ void gather_neox_rows_kernel(const V *src, V *dst, uint32_t rows, uint32_t row_units, uint32_t head_size) {
    for (uint32_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const V *s = src + (size_t)neox_source_row(r, head_size) * row_units;
        V *d = dst + (size_t)r * row_units;
        for (uint32_t i = threadIdx.x; i < row_units; i += blockDim.x) d[i] = s[i];
    }
}

static cudaError_t gather_neox_rows(const void *src, void *dst, uint32_t rows, uint64_t row_bytes, uint32_t head_size, cudaStream_t st) {
    const uint32_t grid = rows < 4096u ? rows : 4096u;
    if (row_bytes % 16 == 0 && ((uintptr_t)src % 16) == 0 && ((uintptr_t)dst % 16) == 0)
        gather_neox_rows_kernel<uint4><<<grid, 128, 0, st>>>((const uint4 *)src, (uint4 *)dst, rows, (uint32_t)(row_bytes / 16), head_size);
    else if (row_bytes % 4 == 0)
        gather_neox_rows_kernel<uint32_t><<<grid, 128, 0, st>>>((const uint32_t *)src, (uint32_t *)dst, rows, (uint32_t)(row_bytes / 4), head_size);
    else
        gather_neox_rows_kernel<uint16_t><<<grid, 128, 0, st>>>((const uint16_t *)src, (uint16_t *)dst, rows, (uint32_t)(row_bytes / 2), head_size);
    return cudaGetLastError();
}

// A model-owned copy of `t` with its rows in the order above (rows stay contiguous in both device layouts).
static int32_t neox_row_copy(ib_llama *m, const ib_qtensor *t, const ib_qtensor **out) {
    ib_qtensor *c = new (std::nothrow) ib_qtensor(*t);
    if (!c) return set_error(IB_ERR_OOM, "host allocation failed");
    c->dev = nullptr;
    cudaError_t e = cudaMalloc(&c->dev, t->nbytes + 16);
    if (e == cudaSuccess) e = gather_neox_rows(t->dev, c->dev, (uint32_t)t->rows, t->row_bytes, m->head_size, 0);
    if (e != cudaSuccess) {
        if (c->dev) cudaFree(c->dev);
        delete c;
        return set_error(e == cudaErrorMemoryAllocation ? IB_ERR_OOM : IB_ERR_CUDA, "ib_llama_create: NeoX row order of a %llux%llu matrix: %s",
                         (unsigned long long)t->rows, (unsigned long long)t->cols, cudaGetErrorString(e));
    }
    m->owned_tensors.push_back(c);
    *out = c;
    return IB_OK;
}

static int32_t neox_bias_copy(ib_llama *m, const float *b, uint32_t rows, const float **out) {
    float *d = nullptr;
    cudaError_t e = cudaMalloc(&d, sizeof(float) * rows);
    if (e == cudaSuccess) e = gather_neox_rows(b, d, rows, sizeof(float), m->head_size, 0);
    if (e != cudaSuccess) {
        if (d) cudaFree(d);
        return set_error(e == cudaErrorMemoryAllocation ? IB_ERR_OOM : IB_ERR_CUDA, "ib_llama_create: NeoX order of a bias: %s", cudaGetErrorString(e));
    }
    m->owned_device.push_back(d);
    *out = d;
    return IB_OK;
}

static int32_t check_matrix(const ib_qtensor *t, const char *name, uint64_t rows, uint64_t cols, bool need_fast) {
    IB_REQUIRE(t != nullptr, "ib_llama_create: missing tensor %s", name);
    IB_REQUIRE(t->rows == rows && t->cols == cols, "ib_llama_create: %s is %llux%llu, expected %llux%llu", name, (unsigned long long)t->rows,
               (unsigned long long)t->cols, (unsigned long long)rows, (unsigned long long)cols);
    if (need_fast && !t->fast)
        return set_error(IB_ERR_UNSUPPORTED,
                         "ib_llama_create: %s (%llux%llu, type %d) does not meet the alignment rules of the fused kernels "
                         "(quantized; Q4_K/Q5_K cols %% 256, Q8_0 cols %% 256, Q6_K cols %% 2048)",
                         name, (unsigned long long)rows, (unsigned long long)cols, t->qtype);
    return IB_OK;
}

}  // namespace ib

namespace ib {
void llama_adopt(ib_llama *m, std::vector<ib_qtensor *> &&tensors, std::vector<void *> &&device) {
    m->owned_tensors.insert(m->owned_tensors.end(), tensors.begin(), tensors.end());
    m->owned_device.insert(m->owned_device.end(), device.begin(), device.end());
    tensors.clear();
    device.clear();
}
}  // namespace ib

extern "C" {

static int32_t finish_graph(ib_llama *m);
static int32_t capture_graph(ib_llama *m, cudaGraphExec_t *exec, uint64_t *launches_per_token);

int32_t ib_llama_destroy(ib_llama *m) {
    if (!m) return IB_OK;
    cudaSetDevice(m->ctx->device);
    cudaDeviceSynchronize();
    if (m->graph_exec) cudaGraphExecDestroy(m->graph_exec);
    if (m->graph_exec_sample) cudaGraphExecDestroy(m->graph_exec_sample);
    if (m->graph_exec_short) cudaGraphExecDestroy(m->graph_exec_short);
    if (m->graph_exec_sample_short) cudaGraphExecDestroy(m->graph_exec_sample_short);
    if (m->sample_probs) cudaFree(m->sample_probs);
    if (m->sample_keys) cudaFree(m->sample_keys);
    if (m->own_stream) cudaStreamDestroy(m->own_stream);
    if (m->staged) cudaEventDestroy(m->staged);
    for (int r = 0; r < m->tp_size && r < IB_MAX_TP; r++)
        if (m->peers_mapped_by_ipc && m->comm_peer[r] && m->comm_peer[r] != m->comm) cudaIpcCloseMemHandle(m->comm_peer[r]);
    void *pbufs[] = {m->pf.X, m->pf.q, m->pf.att, m->pf.planes, m->pf.planes2, m->pf.attn_scratch, m->pf.hi, m->pf.lo, m->pf.tokens, m->pf.attn_counters};
    for (void *b : pbufs)
        if (b) cudaFree(b);
    void *bufs[] = {m->x, m->xb, m->q, m->hb, m->logits, m->theta, m->rope_cs, m->ctl, m->seq, m->attn_scratch, m->attn_counters, m->argmax_slots,
                    m->argmax_counter, m->x2, m->comm, m->epoch, m->reduce_done};
    for (void *b : bufs)
        if (b) cudaFree(b);
    for (void *b : m->k_cache)
        if (b) cudaFree(b);
    for (void *b : m->v_cache)
        if (b) cudaFree(b);
    if (m->h_pinned) cudaFreeHost(m->h_pinned);
    for (ib_qtensor *t : m->owned_tensors) ib_qtensor_destroy(t);
    for (void *b : m->owned_device) cudaFree(b);
    delete m;
    return IB_OK;
}

int32_t ib_llama_create(ib_ctx *ctx, const ib_llama_config *config, const ib_llama_weights *weights, int32_t kv_dtype, int32_t tp_rank,
                        int32_t tp_size, ib_llama **out) {
    IB_REQUIRE(ctx && config && weights && out, "ib_llama_create: null argument");
    *out = nullptr;
    IB_REQUIRE(cudaSetDevice(ctx->device) == cudaSuccess, "cudaSetDevice failed");
    const ib_llama_config &c = *config;
    IB_REQUIRE(kv_dtype == IB_KV_F32 || kv_dtype == IB_KV_F16, "ib_llama_create: unknown kv dtype %d", kv_dtype);
    IB_REQUIRE(tp_size >= 1 && tp_rank >= 0 && tp_rank < tp_size, "ib_llama_create: bad tensor-parallel rank %d of %d", tp_rank, tp_size);
    IB_REQUIRE(tp_size <= IB_MAX_TP, "ib_llama_create: at most %d tensor-parallel ranks", IB_MAX_TP);
    IB_REQUIRE(c.num_hidden_layers > 0 && c.hidden_size > 0 && c.num_attention_heads > 0 && c.num_key_value_heads > 0 && c.vocab_size > 0 &&
                   c.max_position_embeddings > 0 && c.intermediate_size > 0,
               "ib_llama_create: zero-sized configuration field");
    // derived sizes: crates/inferi/src/models/llama2/cpu.rs:110-141
    IB_REQUIRE(c.hidden_size % c.num_attention_heads == 0 && c.num_attention_heads % c.num_key_value_heads == 0,
               "ib_llama_create: head counts do not divide the hidden size");
    IB_REQUIRE(weights->layers != nullptr, "ib_llama_create: null layer array");
    IB_REQUIRE(c.rope_variant == IB_ROPE_ORIGINAL || c.rope_variant == IB_ROPE_NEOX, "ib_llama_create: unknown rope variant %u", c.rope_variant);
    ib_llama *m = new (std::nothrow) ib_llama();
    if (!m) return set_error(IB_ERR_OOM, "host allocation failed");
    m->ctx = ctx; m->cfg = c; m->kv_dtype = kv_dtype; m->tp_rank = tp_rank; m->tp_size = tp_size;
    m->head_size = c.hidden_size / c.num_attention_heads;
    // This rank's share.  Heads and vocabulary split evenly; the FFN width of a rank is read off its gate matrix, because
    // Q6_K rows can only be cut at multiples of 2048 columns and 14336 = 7 x 2048 does not split evenly.
    m->n_heads_l = c.num_attention_heads / tp_size;
    m->n_kv_l = c.num_key_value_heads / tp_size;
    m->q_dim_l = m->n_heads_l * m->head_size;
    m->kv_dim_l = m->n_kv_l * m->head_size;
    m->ffn_l = (tp_size > 1 && weights->layers[0].ffn_gate) ? (uint32_t)weights->layers[0].ffn_gate->rows : c.intermediate_size;
    m->vocab_l = c.vocab_size / tp_size;
    if (c.num_key_value_heads % tp_size || c.vocab_size % tp_size || m->vocab_l % 4 || m->ffn_l == 0 || m->ffn_l > c.intermediate_size) {
        delete m;
        return set_error(IB_ERR_INVALID, "ib_llama_create: %d ranks do not divide %u kv heads / vocabulary %u", tp_size, c.num_key_value_heads, c.vocab_size);
    }
    int32_t rc = IB_OK;
#define FAIL_IF(expr)                 \
    do {                              \
        if ((rc = (expr)) != IB_OK) { \
            ib_llama_destroy(m);      \
            return rc;                \
        }                             \
    } while (0)
#define CU(expr)                                                                                                       \
    do {                                                                                                               \
        cudaError_t _e = (expr);                                                                                       \
        if (_e != cudaSuccess) {                                                                                       \
            ib_llama_destroy(m);                                                                                       \
            return set_error(_e == cudaErrorMemoryAllocation ? IB_ERR_OOM : IB_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
        }                                                                                                              \
    } while (0)
    if (m->head_size != 64 && m->head_size != 128) {
        ib_llama_destroy(m);
        return set_error(IB_ERR_UNSUPPORTED, "ib_llama_create: head_size=%u (supported: 64, 128)", m->head_size);
    }
    m->layers.assign(weights->layers, weights->layers + c.num_hidden_layers);
    for (uint32_t l = 0; l < c.num_hidden_layers; l++) {
        const ib_llama_layer_weights &w = m->layers[l];
        FAIL_IF(check_matrix(w.attn_q, "attn_q", m->q_dim_l, c.hidden_size, true));
        FAIL_IF(check_matrix(w.attn_k, "attn_k", m->kv_dim_l, c.hidden_size, true));
        FAIL_IF(check_matrix(w.attn_v, "attn_v", m->kv_dim_l, c.hidden_size, true));
        FAIL_IF(check_matrix(w.attn_output, "attn_output", c.hidden_size, m->q_dim_l, true));
        FAIL_IF(check_matrix(w.ffn_gate, "ffn_gate", m->ffn_l, c.hidden_size, true));
        FAIL_IF(check_matrix(w.ffn_up, "ffn_up", m->ffn_l, c.hidden_size, true));
        FAIL_IF(check_matrix(w.ffn_down, "ffn_down", c.hidden_size, m->ffn_l, true));
        if (!w.attn_norm_dev || !w.ffn_norm_dev) {
            ib_llama_destroy(m);
            return set_error(IB_ERR_INVALID, "ib_llama_create: layer %u has a null norm weight", l);
        }
        if (w.ffn_gate->qtype != w.ffn_up->qtype) {
            ib_llama_destroy(m);
            return set_error(IB_ERR_UNSUPPORTED, "ib_llama_create: layer %u gate/up types differ", l);
        }
        if (c.rope_variant == IB_ROPE_NEOX) {
            ib_llama_layer_weights &mw = m->layers[l];
            FAIL_IF(neox_row_copy(m, w.attn_q, &mw.attn_q));
            FAIL_IF(neox_row_copy(m, w.attn_k, &mw.attn_k));
            if (w.attn_q_bias_dev) FAIL_IF(neox_bias_copy(m, w.attn_q_bias_dev, m->q_dim_l, &mw.attn_q_bias_dev));
            if (w.attn_k_bias_dev) FAIL_IF(neox_bias_copy(m, w.attn_k_bias_dev, m->kv_dim_l, &mw.attn_k_bias_dev));
        }
    }
    if (c.rope_variant == IB_ROPE_NEOX) CU(cudaDeviceSynchronize());
    FAIL_IF(check_matrix(weights->token_embd, "token_embd", c.vocab_size, c.hidden_size, false));
    {
        const int tq = weights->token_embd->qtype;
        if (tq != IB_F32 && tq != IB_Q8_0 && tq != IB_Q4_K && tq != IB_Q5_K && tq != IB_Q6_K) {
            ib_llama_destroy(m);
            return set_error(IB_ERR_UNSUPPORTED, "ib_llama_create: token_embd of type %d (the embedding look-up takes F32, Q8_0, Q4_K, Q5_K, Q6_K)", tq);
        }
    }
    m->token_embd = weights->token_embd;
    m->output = weights->output ? weights->output : weights->token_embd;  // tied classifier: transformer.rs:376-382
    FAIL_IF(check_matrix(m->output, "output", m->vocab_l, c.hidden_size, true));
    if (!weights->output_norm_dev) {
        ib_llama_destroy(m);
        return set_error(IB_ERR_INVALID, "ib_llama_create: null output_norm");
    }
    m->output_norm = weights->output_norm_dev;

    // state (transformer.rs:46-137)
    CU(cudaMalloc(&m->x, sizeof(float) * c.hidden_size));
    CU(cudaMalloc(&m->xb, sizeof(float) * m->q_dim_l));
    CU(cudaMalloc(&m->q, sizeof(float) * m->q_dim_l));
    CU(cudaMalloc(&m->hb, sizeof(float) * m->ffn_l));
    CU(cudaMalloc(&m->logits, sizeof(float) * m->vocab_l));
    CU(cudaMalloc(&m->theta, sizeof(float) * (m->head_size / 2)));
    CU(cudaMalloc(&m->rope_cs, sizeof(float2) * (m->head_size / 2)));
    {
        // theta_j = base^(-2j/head_size) with the C library's powf (crates/inferi-shaders/src/rope.rs:76-77)
        std::vector<float> th(m->head_size / 2);
        for (uint32_t j = 0; j < m->head_size / 2; j++) th[j] = powf(c.rope_theta, -(float)(2 * j) / (float)m->head_size);
        CU(cudaMemcpy(m->theta, th.data(), th.size() * sizeof(float), cudaMemcpyHostToDevice));
    }
    const size_t kv_elem = kv_dtype == IB_KV_F16 ? 2 : 4;
    const size_t kv_bytes = (size_t)c.max_position_embeddings * m->kv_dim_l * kv_elem;
    m->k_cache.assign(c.num_hidden_layers, nullptr);
    m->v_cache.assign(c.num_hidden_layers, nullptr);
    for (uint32_t l = 0; l < c.num_hidden_layers; l++) {
        CU(cudaMalloc(&m->k_cache[l], kv_bytes));
        CU(cudaMalloc(&m->v_cache[l], kv_bytes));
        CU(cudaMemset(m->k_cache[l], 0, kv_bytes));
        CU(cudaMemset(m->v_cache[l], 0, kv_bytes));
    }
    m->seq_cap = c.max_position_embeddings + 1;
    CU(cudaMalloc(&m->ctl, sizeof(TokenCtl)));
    CU(cudaMemset(m->ctl, 0, sizeof(TokenCtl)));
    CU(cudaMalloc(&m->seq, sizeof(uint32_t) * m->seq_cap));
    CU(cudaMemset(m->seq, 0, sizeof(uint32_t) * m->seq_cap));
    CU(cudaMallocHost(&m->h_pinned, sizeof(uint32_t) * (4 + (size_t)m->seq_cap)));
    CU(cudaEventCreateWithFlags(&m->staged, cudaEventDisableTiming));
    ib_attn_params ap{c.max_position_embeddings, m->kv_dim_l, c.num_attention_heads / c.num_key_value_heads, m->n_heads_l, m->head_size, 0};
    m->attn_splits = attn_max_splits(ctx, ap);
    CU(cudaMalloc(&m->attn_scratch, attn_scratch_bytes(ap, m->attn_splits)));
    CU(cudaMalloc(&m->attn_counters, sizeof(unsigned int) * m->n_kv_l));
    CU(cudaMemset(m->attn_counters, 0, sizeof(unsigned int) * m->n_kv_l));
    CU(cudaMalloc(&m->argmax_slots, sizeof(unsigned long long) * (size_t)ctx->sm_count * 2));
    CU(cudaMalloc(&m->argmax_counter, sizeof(unsigned int)));
    CU(cudaMemset(m->argmax_counter, 0, sizeof(unsigned int)));
    CU(cudaMalloc(&m->epoch, sizeof(uint32_t)));
    CU(cudaMemset(m->epoch, 0, sizeof(uint32_t)));
    CU(cudaStreamCreateWithFlags(&m->own_stream, cudaStreamNonBlocking));
    if (tp_size > 1) {
        // exchange area + second residual buffer; the graph is recorded once the peers' areas are mapped (ib_llama_tp_connect)
        const CommLayout cl(c.hidden_size, tp_size);
        CU(cudaMalloc(&m->comm, cl.total));
        CU(cudaMemset(m->comm, 0, cl.total));
        CU(cudaMalloc(&m->x2, sizeof(float) * c.hidden_size));
        CU(cudaMalloc(&m->reduce_done, sizeof(uint32_t)));
        CU(cudaMemset(m->reduce_done, 0, sizeof(uint32_t)));
        CU(cudaDeviceSynchronize());
        *out = m;
        return IB_OK;
    }
    rc = finish_graph(m);
    if (rc != IB_OK) {
        ib_llama_destroy(m);
        return rc;
    }
#undef FAIL_IF
#undef CU
    *out = m;
    return IB_OK;
}

// Records the token graph (once every pointer it needs is known) and instantiates it.
static int32_t finish_graph(ib_llama *m) {
    IB_CHECK_CUDA(cudaDeviceSynchronize());
    int32_t rc = capture_graph(m, &m->graph_exec, &m->launches_per_token);
    if (rc != IB_OK || m->short_positions == 0) return rc;
    // the variant for short contexts (record_token noted up to which position the attention kernel offers it)
    if (m->graph_exec_short) { cudaGraphExecDestroy(m->graph_exec_short); m->graph_exec_short = nullptr; }
    uint64_t same = 0;
    m->recording_short = true;
    rc = capture_graph(m, &m->graph_exec_short, &same);
    return rc;
}


// Records the token's kernels (with the sampler node when a temperature is set) into a graph and instantiates it.
static int32_t capture_graph(ib_llama *m, cudaGraphExec_t *exec, uint64_t *launches_per_token) {
    ib_ctx *ctx = m->ctx;
    const uint64_t before = ctx->launches;
    IB_CHECK_CUDA(cudaStreamBeginCapture(m->own_stream, cudaStreamCaptureModeThreadLocal));
    const int32_t rc = record_token(m, m->own_stream, 1);
    cudaGraph_t graph = nullptr;
    cudaError_t ce = cudaStreamEndCapture(m->own_stream, &graph);
    m->recording_short = false;
    *launches_per_token = ctx->launches - before;
    ctx->launches = before;  // recording is not launching
    if (rc != IB_OK) {
        if (graph) cudaGraphDestroy(graph);
        return rc;
    }
    if (ce != cudaSuccess) return set_error(IB_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(ce));
    ce = cudaGraphInstantiate(exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ce != cudaSuccess) {
        *exec = nullptr;
        return set_error(IB_ERR_CUDA, "graph instantiation failed: %s", cudaGetErrorString(ce));
    }
    return IB_OK;
}

int32_t ib_llama_set_sampler(ib_llama *m, float temperature, float topp, uint64_t seed) {
    IB_REQUIRE(m, "ib_llama_set_sampler: null model");
    IB_REQUIRE(cudaSetDevice(m->ctx->device) == cudaSuccess, "cudaSetDevice failed");
    IB_REQUIRE(temperature >= 0.f, "ib_llama_set_sampler: negative temperature");
    if (temperature > 0.f) {
        if (m->tp_size > 1) return set_error(IB_ERR_UNSUPPORTED, "ib_llama_set_sampler: sampling needs the whole vocabulary on one GPU (tensor-parallel models are greedy)");
    }
    IB_CHECK_CUDA(cudaDeviceSynchronize());
    if (m->graph_exec_sample) { cudaGraphExecDestroy(m->graph_exec_sample); m->graph_exec_sample = nullptr; }
    if (m->graph_exec_sample_short) { cudaGraphExecDestroy(m->graph_exec_sample_short); m->graph_exec_sample_short = nullptr; }
    m->temperature = temperature; m->topp = topp; m->sample_seed = seed;
    if (temperature == 0.f) return IB_OK;   // greedy: the graph recorded at creation
    if (!m->sample_probs) {
        IB_CHECK_CUDA(cudaMalloc(&m->sample_probs, sizeof(float) * m->cfg.vocab_size));
        IB_CHECK_CUDA(cudaMalloc(&m->sample_keys, sizeof(unsigned long long) * sample_keys_capacity(m->cfg.vocab_size)));
    }
    int32_t rc = capture_graph(m, &m->graph_exec_sample, &m->launches_per_token_sample);
    if (rc == IB_OK && m->short_positions) {
        if (m->graph_exec_sample_short) { cudaGraphExecDestroy(m->graph_exec_sample_short); m->graph_exec_sample_short = nullptr; }
        uint64_t same = 0;
        m->recording_short = true;
        rc = capture_graph(m, &m->graph_exec_sample_short, &same);
    }
    if (rc != IB_OK) { m->temperature = 0.f; return rc; }
    return IB_OK;
}

// ---- tensor parallel set-up: every rank publishes a handle of its exchange area and maps the others' ----
int32_t ib_llama_tp_export(ib_llama *m, void *handle_out) {
    IB_REQUIRE(m && handle_out, "ib_llama_tp_export: null argument");
    IB_REQUIRE(m->tp_size > 1 && m->comm, "ib_llama_tp_export: the model is not tensor parallel");
    IB_REQUIRE(cudaSetDevice(m->ctx->device) == cudaSuccess, "cudaSetDevice failed");
    static_assert(sizeof(cudaIpcMemHandle_t) == IB_TP_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, m->comm);
    if (e != cudaSuccess) return set_error(IB_ERR_COMM, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
    memcpy(handle_out, &h, sizeof h);
    return IB_OK;
}

int32_t ib_llama_tp_connect(ib_llama *m, const void *handles) {
    IB_REQUIRE(m && handles, "ib_llama_tp_connect: null argument");
    IB_REQUIRE(m->tp_size > 1 && m->comm, "ib_llama_tp_connect: the model is not tensor parallel");
    IB_REQUIRE(!m->connected, "ib_llama_tp_connect: already connected");
    IB_REQUIRE(cudaSetDevice(m->ctx->device) == cudaSuccess, "cudaSetDevice failed");
    for (int r = 0; r < m->tp_size; r++) {
        if (r == m->tp_rank) { m->comm_peer[r] = m->comm; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t *)handles + (size_t)r * IB_TP_HANDLE_BYTES, sizeof h);
        void *ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return set_error(IB_ERR_COMM, "cudaIpcOpenMemHandle for rank %d failed: %s (are the GPUs NVLink/P2P peers?)", r, cudaGetErrorString(e));
        m->comm_peer[r] = (uint8_t *)ptr;
        m->peers_mapped_by_ipc = true;
    }
    m->connected = true;
    return finish_graph(m);
}

int32_t ib_llama_tp_area(ib_llama *m, void **area_dev, uint64_t *nbytes) {
    IB_REQUIRE(m && area_dev && nbytes, "ib_llama_tp_area: null argument");
    IB_REQUIRE(m->tp_size > 1 && m->comm, "ib_llama_tp_area: the model is not tensor parallel");
    *area_dev = m->comm;
    *nbytes = CommLayout(m->cfg.hidden_size, m->tp_size).total;
    return IB_OK;
}

int32_t ib_llama_tp_connect_ptrs(ib_llama *m, void *const *areas) {
    IB_REQUIRE(m && areas, "ib_llama_tp_connect_ptrs: null argument");
    IB_REQUIRE(m->tp_size > 1 && m->comm, "ib_llama_tp_connect_ptrs: the model is not tensor parallel");
    IB_REQUIRE(!m->connected, "ib_llama_tp_connect_ptrs: already connected");
    IB_REQUIRE(cudaSetDevice(m->ctx->device) == cudaSuccess, "cudaSetDevice failed");
    for (int r = 0; r < m->tp_size; r++) {
        if (r != m->tp_rank) IB_REQUIRE(areas[r] != nullptr, "ib_llama_tp_connect_ptrs: null area for rank %d", r);
        m->comm_peer[r] = r == m->tp_rank ? m->comm : (uint8_t *)areas[r];
    }
    m->connected = true;
    m->peers_mapped_by_ipc = false;
    return finish_graph(m);
}

static int32_t run_tokens(ib_llama *m, cudaStream_t s, const uint32_t *tokens, uint32_t n_prompt, uint32_t start_pos, uint32_t n_steps) {
    if (!m->graph_exec) return set_error(IB_ERR_COMM, "the tensor-parallel model is not connected yet: call ib_llama_tp_connect on every rank first");
    // control block + given tokens in one pinned staging buffer -> two small async copies
    uint32_t *h = m->h_pinned;
    IB_CHECK_CUDA(cudaEventSynchronize(m->staged));  // an earlier call's copies out of the staging buffer are done
    h[0] = 0; h[1] = start_pos; h[2] = n_prompt; h[3] = 0;
    for (uint32_t i = 0; i < n_prompt; i++) h[4 + i] = tokens[i];
    IB_CHECK_CUDA(cudaMemcpyAsync(m->ctl, h, sizeof(TokenCtl), cudaMemcpyHostToDevice, s));
    IB_CHECK_CUDA(cudaMemcpyAsync(m->seq, h + 4, sizeof(uint32_t) * n_prompt, cudaMemcpyHostToDevice, s));
    IB_CHECK_CUDA(cudaEventRecord(m->staged, s));
    const bool sampled = m->temperature > 0.f && m->graph_exec_sample;
    for (uint32_t i = 0; i < n_steps; i++) {
        // positions below short_positions replay the graph whose attention nodes merge inside thread-block clusters
        const bool shrt = (uint64_t)start_pos + i + 1 <= m->short_positions;
        cudaGraphExec_t exec = sampled ? (shrt && m->graph_exec_sample_short ? m->graph_exec_sample_short : m->graph_exec_sample)
                                       : (shrt && m->graph_exec_short ? m->graph_exec_short : m->graph_exec);
        IB_CHECK_CUDA(cudaGraphLaunch(exec, s));
        m->ctx->launches += sampled ? m->launches_per_token_sample : m->launches_per_token;
    }
    return IB_OK;
}

int32_t ib_llama_forward(ib_llama *m, void *stream, uint32_t token, uint32_t pos, float *logits_host, uint32_t *next_token_host) {
    IB_REQUIRE(m, "ib_llama_forward: null model");
    IB_REQUIRE(cudaSetDevice(m->ctx->device) == cudaSuccess, "cudaSetDevice failed");
    IB_REQUIRE(token < m->cfg.vocab_size, "ib_llama_forward: token %u outside the vocabulary of %u", token, m->cfg.vocab_size);
    IB_REQUIRE(pos < m->cfg.max_position_embeddings, "ib_llama_forward: pos %u outside the context of %u", pos, m->cfg.max_position_embeddings);
    cudaStream_t s = (cudaStream_t)stream;
    int32_t rc = run_tokens(m, s, &token, 1, pos, 1);
    if (rc) return rc;
    if (logits_host) IB_CHECK_CUDA(cudaMemcpyAsync(logits_host, m->logits, sizeof(float) * m->vocab_l, cudaMemcpyDeviceToHost, s));
    if (next_token_host) IB_CHECK_CUDA(cudaMemcpyAsync(next_token_host, &m->ctl->next, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    if (logits_host || next_token_host) {
        IB_CHECK_CUDA(cudaStreamSynchronize(s));
        return check_device_error(m->ctx);
    }
    return IB_OK;
}

// ---- prompt prefill on the tensor cores ----
static int32_t prefill_prepare(ib_llama *m) {
    if (m->pf.ready) return IB_OK;
    const ib_llama_config &c = m->cfg;
    const uint32_t H = c.hidden_size, F = m->ffn_l, Q = m->q_dim_l, KV = m->kv_dim_l, N = PREFILL_MAX_TOKENS;
    const uint32_t widest = F > H ? (F > Q ? F : Q) : (H > Q ? H : Q);
    size_t plane_elems = 0;   // largest planes * rows over the matrices (per token)
    const ib_llama_layer_weights &w = m->layers[0];
    const ib_qtensor *mats[] = {w.attn_q, w.attn_k, w.attn_v, w.attn_output, w.ffn_gate, w.ffn_up, w.ffn_down};
    for (const ib_qtensor *t : mats) {
        const size_t e = (size_t)prefill_max_pieces(prefill_streamk(m->ctx, (uint32_t)t->rows, (uint32_t)t->cols), (uint32_t)t->rows) * t->rows;
        if (e > plane_elems) plane_elems = e;
    }
    ib_attn_params ap{c.max_position_embeddings, KV, c.num_attention_heads / c.num_key_value_heads, m->n_heads_l, m->head_size, 0};
    m->pf.attn_splits = 16;   // per query; the queries of a prompt fill the GPU between them
    m->pf.attn_scratch_step = attn_scratch_bytes(ap, m->pf.attn_splits) / sizeof(float);
    IB_CHECK_CUDA(cudaMalloc(&m->pf.X, sizeof(float) * N * H));
    IB_CHECK_CUDA(cudaMalloc(&m->pf.q, sizeof(float) * N * Q));
    IB_CHECK_CUDA(cudaMalloc(&m->pf.att, sizeof(float) * N * Q));
    IB_CHECK_CUDA(cudaMalloc(&m->pf.hi, sizeof(__half) * (N + 8) * widest));   // the inputs' tiles + the tiles of their sub-block sums
    IB_CHECK_CUDA(cudaMalloc(&m->pf.lo, sizeof(__half) * (N + 8) * widest));
    IB_CHECK_CUDA(cudaMalloc(&m->pf.planes, sizeof(float) * N * plane_elems));
    IB_CHECK_CUDA(cudaMalloc(&m->pf.planes2, sizeof(float) * N * plane_elems));
    IB_CHECK_CUDA(cudaMalloc(&m->pf.tokens, sizeof(uint32_t) * N));
    IB_CHECK_CUDA(cudaMalloc(&m->pf.attn_scratch, sizeof(float) * N * m->pf.attn_scratch_step));
    IB_CHECK_CUDA(cudaMalloc(&m->pf.attn_counters, sizeof(unsigned int) * N * m->n_kv_l));
    IB_CHECK_CUDA(cudaMemset(m->pf.attn_counters, 0, sizeof(unsigned int) * N * m->n_kv_l));
    m->pf.ready = true;
    return IB_OK;
}

int32_t ib_llama_prefill(ib_llama *m, void *stream, const uint32_t *tokens_host, uint32_t n, uint32_t start_pos, uint32_t *next_token_host) {
    IB_REQUIRE(m && tokens_host, "ib_llama_prefill: null argument");
    IB_REQUIRE(cudaSetDevice(m->ctx->device) == cudaSuccess, "cudaSetDevice failed");
    IB_REQUIRE(n >= 1, "ib_llama_prefill: empty prompt");
    const ib_llama_config &c = m->cfg;
    IB_REQUIRE((uint64_t)start_pos + n <= c.max_position_embeddings, "ib_llama_prefill: %u positions from %u exceed the context of %u", n, start_pos, c.max_position_embeddings);
    for (uint32_t i = 0; i < n; i++) IB_REQUIRE(tokens_host[i] < c.vocab_size, "ib_llama_prefill: token %u outside the vocabulary", tokens_host[i]);
    ib_ctx *ctx = m->ctx;
    // what the tensor-core path takes; everything else goes through ib_llama_generate (the prompt through the decode path)
    if (m->tp_size > 1) return set_error(IB_ERR_UNSUPPORTED, "ib_llama_prefill: tensor-parallel models feed their prompt through the decode path (ib_llama_generate)");
    const uint32_t kv_mul = c.num_attention_heads / c.num_key_value_heads;
    if (m->kv_dtype != IB_KV_F16 || kv_mul != 4)
        return set_error(IB_ERR_UNSUPPORTED, "ib_llama_prefill: needs the f16 cache and 4 query heads per kv head (have kv_mul=%u); use ib_llama_generate", kv_mul);
    for (const ib_llama_layer_weights &w : m->layers) {
        const ib_qtensor *mats[] = {w.attn_q, w.attn_k, w.attn_v, w.attn_output, w.ffn_gate, w.ffn_up, w.ffn_down};
        for (const ib_qtensor *t : mats)
            if (!prefill_gemm_eligible(t))
                return set_error(IB_ERR_UNSUPPORTED, "ib_llama_prefill: a %llux%llu matrix of type %d is outside the tensor-core path; use ib_llama_generate",
                                 (unsigned long long)t->rows, (unsigned long long)t->cols, t->qtype);
    }
    int32_t rc = prefill_prepare(m);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t H = c.hidden_size, F = m->ffn_l, Q = m->q_dim_l, KV = m->kv_dim_l;
    auto &B = m->pf;
    auto gemm = [&](const ib_qtensor *w, uint32_t nc, float *planes, StreamK &ks) -> int32_t {
        ks = prefill_streamk(ctx, (uint32_t)w->rows, (uint32_t)w->cols);
        return launch_prefill_gemm(ctx, s, w, B.hi, B.lo, nc, planes, ks);
    };
#define PF(expr) do { if ((rc = (expr)) != IB_OK) return rc; } while (0)
    for (uint32_t t0 = 0; t0 < n; t0 += PREFILL_MAX_TOKENS) {
        const uint32_t nc = n - t0 < PREFILL_MAX_TOKENS ? n - t0 : PREFILL_MAX_TOKENS, pos0 = start_pos + t0;
        IB_CHECK_CUDA(cudaMemcpyAsync(B.tokens, tokens_host + t0, sizeof(uint32_t) * nc, cudaMemcpyHostToDevice, s));
        PF(launch_prefill_embed(ctx, s, m->token_embd, B.tokens, nc, c.vocab_size, B.X));
        for (uint32_t l = 0; l < c.num_hidden_layers; l++) {
            const ib_llama_layer_weights &w = m->layers[l];
            StreamK ks = {};
            PrefillEpiParams e = {};
            e.n = nc; e.theta = m->theta; e.head_size = m->head_size; e.pos0 = pos0; e.kv_dim = KV; e.kv_dtype = (uint32_t)m->kv_dtype;
            // q, k, v: RMSNorm, GEMM, bias, RoPE, cache append (transformer.rs:420-445)
            PF(launch_prefill_norm_split(ctx, s, B.X, w.attn_norm_dev, c.rms_norm_eps, nc, H, B.hi, B.lo));
            PF(gemm(w.attn_q, nc, B.planes, ks));
            e.planes = B.planes; e.sk = ks; e.rows = Q; e.mode = PE_Q; e.bias = w.attn_q_bias_dev; e.out = B.q;
            PF(launch_prefill_epilogue(ctx, s, e));
            PF(gemm(w.attn_k, nc, B.planes, ks));
            e.sk = ks; e.rows = KV; e.mode = PE_K; e.bias = w.attn_k_bias_dev; e.cache = m->k_cache[l];
            PF(launch_prefill_epilogue(ctx, s, e));
            PF(gemm(w.attn_v, nc, B.planes, ks));
            e.sk = ks; e.mode = PE_V; e.bias = w.attn_v_bias_dev; e.cache = m->v_cache[l];
            PF(launch_prefill_epilogue(ctx, s, e));
            // causal attention: query t over positions 0 .. pos0 + t (transformer.rs:448), all queries in one launch
            AttnLaunch a = {};
            a.p = ib_attn_params{c.max_position_embeddings, KV, kv_mul, m->n_heads_l, m->head_size, pos0};
            a.q = B.q; a.k_cache = m->k_cache[l]; a.v_cache = m->v_cache[l]; a.kv_dtype = m->kv_dtype; a.out = B.att;
            a.scratch = B.attn_scratch; a.counters = B.attn_counters; a.max_splits = B.attn_splits;
            a.n_queries = nc; a.q_step = Q; a.out_step = Q; a.counter_step = m->n_kv_l; a.scratch_step = B.attn_scratch_step;
            if (nc > 1 && !attn_gqa4_eligible(a)) return set_error(IB_ERR_UNSUPPORTED, "ib_llama_prefill: head size %u is outside the batched attention kernel; use ib_llama_generate", m->head_size);
            PF(launch_attention(ctx, s, a));
            // o_proj + residual (transformer.rs:450-453)
            PF(launch_prefill_norm_split(ctx, s, B.att, nullptr, 0.f, nc, Q, B.hi, B.lo));
            PF(gemm(w.attn_output, nc, B.planes, ks));
            e.sk = ks; e.rows = H; e.mode = PE_RESIDUAL; e.bias = nullptr; e.out = B.X;
            PF(launch_prefill_epilogue(ctx, s, e));
            // gate, up, SwiGLU (transformer.rs:454-464)
            PF(launch_prefill_norm_split(ctx, s, B.X, w.ffn_norm_dev, c.rms_norm_eps, nc, H, B.hi, B.lo));
            PF(gemm(w.ffn_gate, nc, B.planes, ks));
            PF(gemm(w.ffn_up, nc, B.planes2, ks));
            e.planes2 = B.planes2; e.sk = ks; e.rows = F; e.mode = PE_SWIGLU; e.hi = B.hi; e.lo = B.lo;
            PF(launch_prefill_epilogue(ctx, s, e));
            // down + residual (transformer.rs:465-468)
            PF(gemm(w.ffn_down, nc, B.planes, ks));
            e.sk = ks; e.rows = H; e.mode = PE_RESIDUAL; e.out = B.X;
            PF(launch_prefill_epilogue(ctx, s, e));
        }
        if (t0 + nc == n) IB_CHECK_CUDA(cudaMemcpyAsync(m->x, B.X + (size_t)(nc - 1) * H, sizeof(float) * H, cudaMemcpyDeviceToDevice, s));
    }
#undef PF
    // classifier + greedy arg-max of the last prompt token (transformer.rs:471-478, models/sampler.rs:54-56): the decode kernel
    GemvParams p = {};
    fill_seg(p.seg[0], m->output, m->logits);
    p.nseg = 1; p.cols = H; p.epi = EPI_ARGMAX; p.x = m->x; p.norm_w = m->output_norm; p.eps = c.rms_norm_eps;
    p.argmax_slots = m->argmax_slots; p.argmax_counter = m->argmax_counter; p.argmax_out = &m->ctl->next; p.pair_instance = 1;
    if ((rc = launch_gemv(ctx, s, p))) return rc;
    m->x_final = m->x;
    if (next_token_host) IB_CHECK_CUDA(cudaMemcpyAsync(next_token_host, &m->ctl->next, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    IB_CHECK_CUDA(cudaStreamSynchronize(s));
    return check_device_error(ctx);
}

int32_t ib_llama_generate(ib_llama *m, void *stream, const uint32_t *tokens_host, uint32_t n_prompt, uint32_t start_pos, uint32_t n_gen,
                          uint32_t *out_tokens_host) {
    IB_REQUIRE(m && tokens_host, "ib_llama_generate: null argument");
    IB_REQUIRE(cudaSetDevice(m->ctx->device) == cudaSuccess, "cudaSetDevice failed");
    IB_REQUIRE(n_prompt >= 1, "ib_llama_generate: empty prompt");
    IB_REQUIRE(n_gen == 0 || out_tokens_host, "ib_llama_generate: null output buffer");
    const uint64_t steps = (uint64_t)n_prompt + (n_gen ? n_gen - 1 : 0);  // the last generated token is not fed back
    IB_REQUIRE((uint64_t)start_pos + steps <= m->cfg.max_position_embeddings, "ib_llama_generate: %llu positions from %u exceed the context of %u",
               (unsigned long long)steps, start_pos, m->cfg.max_position_embeddings);
    for (uint32_t i = 0; i < n_prompt; i++)
        IB_REQUIRE(tokens_host[i] < m->cfg.vocab_size, "ib_llama_generate: token %u outside the vocabulary", tokens_host[i]);
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t n_steps = n_gen ? (uint32_t)steps : n_prompt;
    int32_t rc = run_tokens(m, s, tokens_host, n_prompt, start_pos, n_steps);
    if (rc) return rc;
    if (n_gen) IB_CHECK_CUDA(cudaMemcpyAsync(out_tokens_host, m->seq + n_prompt, sizeof(uint32_t) * n_gen, cudaMemcpyDeviceToHost, s));
    IB_CHECK_CUDA(cudaStreamSynchronize(s));
    return check_device_error(m->ctx);
}

int32_t ib_llama_generate_until(ib_llama *m, void *stream, const uint32_t *tokens_host, uint32_t n_prompt, uint32_t start_pos, uint32_t max_gen,
                                uint32_t eos_token, uint32_t *out_tokens_host, uint32_t *n_out) {
    IB_REQUIRE(m && tokens_host && out_tokens_host && n_out, "ib_llama_generate_until: null argument");
    IB_REQUIRE(n_prompt >= 1 && max_gen >= 1, "ib_llama_generate_until: empty prompt or nothing to generate");
    *n_out = 0;
    // The device loop runs in chunks; between chunks the host looks for the stop token.  At most CHUNK - 1 tokens are computed
    // past it (their cache rows are simply overwritten by the next turn, which starts at the position after the stop token).
    constexpr uint32_t CHUNK = 16;
    const uint32_t *cur = tokens_host;
    uint32_t cur_n = n_prompt, pos = start_pos, done = 0;
    while (done < max_gen) {
        const uint32_t g = max_gen - done < CHUNK ? max_gen - done : CHUNK;
        const int32_t rc = ib_llama_generate(m, stream, cur, cur_n, pos, g, out_tokens_host + done);
        if (rc) return rc;
        for (uint32_t i = 0; i < g; i++)
            if (out_tokens_host[done + i] == eos_token) {
                *n_out = done + i + 1;   // the stop token is reported (chat_llama2.rs:157-166 breaks after seeing it)
                return IB_OK;
            }
        pos += cur_n + g - 1;            // positions consumed: the chunk's last token has not been fed back yet
        done += g;
        cur = out_tokens_host + done - 1;
        cur_n = 1;
    }
    *n_out = done;
    return IB_OK;
}

int32_t ib_llama_chat(ib_llama *m, void *stream, const uint32_t *tokens_host, uint32_t n_prompt, uint32_t start_pos, uint32_t max_gen,
                      uint32_t eos_token, ib_token_event_fn out, void *user, uint32_t *n_out) {
    IB_REQUIRE(m && tokens_host && out, "ib_llama_chat: null argument");
    IB_REQUIRE(n_prompt >= 1 && max_gen >= 1, "ib_llama_chat: empty prompt or nothing to generate");
    if (n_out) *n_out = 0;
    const uint64_t ctx_len = m->cfg.max_position_embeddings;
    IB_REQUIRE((uint64_t)start_pos + n_prompt <= ctx_len, "ib_llama_chat: %u prompt positions from %u exceed the context of %llu", n_prompt, start_pos,
               (unsigned long long)ctx_len);
    // The turn also ends when the context is full: the forward at the last position still yields a token.
    if ((uint64_t)max_gen > ctx_len - start_pos - n_prompt + 1) max_gen = (uint32_t)(ctx_len - start_pos - n_prompt + 1);
    using clock = std::chrono::steady_clock;
    auto seconds_since = [](clock::time_point t0) { return std::chrono::duration<double>(clock::now() - t0).count(); };
    // chat_llama2.rs:131-140: the forward at start_pos is outside the timed span (`timing_delay = 1`), so it runs alone.
    uint32_t first_next = 0;
    int32_t rc = ib_llama_forward(m, stream, tokens_host[0], start_pos, nullptr, &first_next);
    if (rc) return rc;
    const clock::time_point t_start = clock::now();
    uint32_t pos = start_pos + 1;            // next position to feed
    uint32_t emitted = 0;
    uint32_t prev = tokens_host[n_prompt - 1];
    uint32_t last = first_next;              // the token the model produced for position pos - 1
    if (n_prompt == 1) {
        // The only prompt token was the untimed one: its successor is the first event, with no rate yet (chat_llama2.rs:168-177).
        if (last == eos_token) return IB_OK;
        if (out(user, prev, last, start_pos, 0, 0.0)) return IB_OK;
        emitted = 1;
        if (n_out) *n_out = emitted;
        prev = last;
    } else {
        // The rest of the prompt: positions start_pos + 1 .. start_pos + n_prompt - 2 only fill the cache (the tensor-core
        // prefill when the model qualifies, the decode loop otherwise); the last prompt token then goes through the token loop.
        const uint32_t mid = n_prompt - 2;
        if (mid >= 8) {
            rc = ib_llama_prefill(m, stream, tokens_host + 1, mid, pos, nullptr);
            if (rc == IB_OK) pos += mid;
            else if (rc != IB_ERR_UNSUPPORTED) return rc;
        }
    }
    constexpr uint32_t CHUNK = 16;
    std::vector<uint32_t> buf(CHUNK);
    // What is still to feed: the prompt tokens from index pos - start_pos on, or (after the prompt) the last produced token.
    while (emitted < max_gen) {
        const uint32_t fed = pos - start_pos;
        const uint32_t *cur = fed < n_prompt ? tokens_host + fed : &last;
        const uint32_t cur_n = fed < n_prompt ? n_prompt - fed : 1;
        const uint32_t g = max_gen - emitted < CHUNK ? max_gen - emitted : CHUNK;
        const double t_before = seconds_since(t_start);
        rc = ib_llama_generate(m, stream, cur, cur_n, pos, g, buf.data());
        if (rc) return rc;
        const double t_after = seconds_since(t_start);
        const uint32_t first_gen_pos = pos + cur_n - 1;   // the forward at this position produced buf[0]
        for (uint32_t i = 0; i < g; i++) {
            const uint32_t tok = buf[i];
            if (tok == eos_token) return IB_OK;           // chat_llama2.rs:158-160: the stop token ends the turn unreported
            // The host sees a chunk's tokens together; their times are spread evenly over the chunk's forwards.
            const double t = t_before + (t_after - t_before) * double(cur_n + i) / double(cur_n + g - 1);
            const uint32_t at = first_gen_pos + i;
            if (out(user, prev, tok, at, at - start_pos - 1, t)) { if (n_out) *n_out = emitted + 1; return IB_OK; }
            emitted++;
            if (n_out) *n_out = emitted;
            prev = tok;
        }
        last = buf[g - 1];
        pos = first_gen_pos + g;
    }
    return IB_OK;
}

int32_t ib_llama_state(ib_llama *m, const float **logits_dev, const float **x_dev) {
    IB_REQUIRE(m, "ib_llama_state: null model");
    if (logits_dev) *logits_dev = m->logits;
    if (x_dev) *x_dev = m->x_final ? m->x_final : m->x;
    return IB_OK;
}

}  // extern "C"
