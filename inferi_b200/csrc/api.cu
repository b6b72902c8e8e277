// C ABI: contexts, quantized tensors and the op-level entry points (see include/inferi_b200.h).
#include "common.cuh"

#include <stdarg.h>
#include <new>

namespace ib {

static thread_local std::string g_last_error;

int32_t set_error(int32_t code, const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = (cudaSetDevice(dev) == cudaSuccess);
    }
    ~DeviceGuard() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

int32_t check_device_error(ib_ctx *ctx) {
    const uint32_t e = *(volatile uint32_t *)ctx->err_host;
    if (e == 0) return IB_OK;
    *(volatile uint32_t *)ctx->err_host = 0;
    static const char *const what[] = {"", "a tile of weights never arrived in shared memory", "a ring stage was never handed back to the producer",
                                       "another rank's partial sums never arrived", "another rank's arg-max candidate never arrived",
                                       "the consumer warps never finished a tile", "the input's sum of squares never completed",
                                       "this rank's reduction of the partial sums never completed", "a GEMM stage was never released by the tensor core",
                                       "a GEMM stage was never filled", "the GEMM accumulator never completed"};
    return set_error(IB_ERR_TIMEOUT, "a kernel gave up waiting (%s); results of that launch are invalid", e < sizeof(what) / sizeof(what[0]) ? what[e] : "unknown wait");
}

}  // namespace ib

using namespace ib;

#define IB_ENTER(ctx)                                                   \
    IB_REQUIRE((ctx) != nullptr, "null context");                       \
    ib::DeviceGuard _guard((ctx)->device);                              \
    if (!_guard.ok) return ib::set_error(IB_ERR_CUDA, "cudaSetDevice(%d) failed", (ctx)->device)

extern "C" {

const char *ib_last_error_string(void) { return g_last_error.c_str(); }

int32_t ib_ctx_create(int32_t device, ib_ctx **out) {
    IB_REQUIRE(out != nullptr, "ib_ctx_create: null output pointer");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return set_error(IB_ERR_CUDA, "no CUDA device available (%s); this library has no CPU path", cudaGetErrorString(e));
    IB_REQUIRE(device >= 0 && device < count, "ib_ctx_create: device %d out of range (0..%d)", device, count - 1);
    DeviceGuard guard(device);
    if (!guard.ok) return set_error(IB_ERR_CUDA, "cudaSetDevice(%d) failed", device);
    cudaDeviceProp prop;
    IB_CHECK_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return set_error(IB_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a (B200) only", device, prop.major, prop.minor);
    ib_ctx *ctx = new (std::nothrow) ib_ctx();
    if (!ctx) return set_error(IB_ERR_OOM, "host allocation failed");
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    cudaError_t he = cudaHostAlloc((void **)&ctx->err_host, sizeof(uint32_t), cudaHostAllocMapped);
    if (he == cudaSuccess) {
        *ctx->err_host = 0;
        he = cudaHostGetDevicePointer((void **)&ctx->err_dev, ctx->err_host, 0);
    }
    if (he != cudaSuccess) {
        if (ctx->err_host) cudaFreeHost(ctx->err_host);
        delete ctx;
        return set_error(IB_ERR_CUDA, "allocating the error word failed: %s", cudaGetErrorString(he));
    }
    cudaError_t ce = cudaMalloc((void **)&ctx->stream_counters, sizeof(uint32_t) * 2 * IB_STREAM_COUNTER_PAIRS);
    if (ce == cudaSuccess) ce = cudaMemset(ctx->stream_counters, 0, sizeof(uint32_t) * 2 * IB_STREAM_COUNTER_PAIRS);
    if (ce != cudaSuccess) {
        if (ctx->stream_counters) cudaFree(ctx->stream_counters);
        cudaFreeHost(ctx->err_host);
        delete ctx;
        return set_error(IB_ERR_CUDA, "allocating the tile counters failed: %s", cudaGetErrorString(ce));
    }
    *out = ctx;
    return IB_OK;
}

int32_t ib_ctx_destroy(ib_ctx *ctx) {
    if (!ctx) return IB_OK;
    DeviceGuard guard(ctx->device);
    if (ctx->attn_scratch) cudaFree(ctx->attn_scratch);
    if (ctx->attn_counters) cudaFree(ctx->attn_counters);
    if (ctx->argmax_scratch) cudaFree(ctx->argmax_scratch);
    if (ctx->argmax_counter) cudaFree(ctx->argmax_counter);
    if (ctx->err_host) cudaFreeHost(ctx->err_host);
    if (ctx->stream_counters) cudaFree(ctx->stream_counters);
    if (ctx->tc_scratch) cudaFree(ctx->tc_scratch);
    delete ctx;
    return IB_OK;
}

int32_t ib_ctx_launch_count(ib_ctx *ctx, uint64_t *out) {
    IB_REQUIRE(ctx && out, "ib_ctx_launch_count: null argument");
    *out = ctx->launches;
    return IB_OK;
}
int32_t ib_ctx_reset_launch_count(ib_ctx *ctx) {
    IB_REQUIRE(ctx, "null context");
    ctx->launches = 0;
    return IB_OK;
}

int32_t ib_ctx_set_wait_limit(ib_ctx *ctx, uint64_t nanoseconds) {
    IB_REQUIRE(ctx, "null context");
    IB_REQUIRE(nanoseconds >= 1000 && nanoseconds <= 600000000000ull, "ib_ctx_set_wait_limit: %llu ns is outside 1 us .. 600 s", (unsigned long long)nanoseconds);
    ctx->wait_limit_ns = nanoseconds;
    return IB_OK;
}

int32_t ib_malloc(ib_ctx *ctx, uint64_t nbytes, void **out_dev) {
    IB_ENTER(ctx);
    IB_REQUIRE(out_dev, "ib_malloc: null output pointer");
    IB_CHECK_CUDA(cudaMalloc(out_dev, nbytes ? nbytes : 1));
    return IB_OK;
}
int32_t ib_free(ib_ctx *ctx, void *dev) {
    IB_ENTER(ctx);
    if (dev) IB_CHECK_CUDA(cudaFree(dev));
    return IB_OK;
}
int32_t ib_memcpy_h2d(ib_ctx *ctx, void *stream, void *dst_dev, const void *src_host, uint64_t nbytes) {
    IB_ENTER(ctx);
    IB_REQUIRE(dst_dev && src_host, "ib_memcpy_h2d: null pointer");
    IB_CHECK_CUDA(cudaMemcpyAsync(dst_dev, src_host, nbytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return IB_OK;
}
int32_t ib_memcpy_d2h(ib_ctx *ctx, void *stream, void *dst_host, const void *src_dev, uint64_t nbytes) {
    IB_ENTER(ctx);
    IB_REQUIRE(dst_host && src_dev, "ib_memcpy_d2h: null pointer");
    IB_CHECK_CUDA(cudaMemcpyAsync(dst_host, src_dev, nbytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return IB_OK;
}
int32_t ib_stream_sync(ib_ctx *ctx, void *stream) {
    IB_ENTER(ctx);
    IB_CHECK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return check_device_error(ctx);
}

// ---- quantized tensors ----
int32_t ib_qtensor_upload(ib_ctx *ctx, int32_t qtype, uint64_t rows, uint64_t cols, const void *gguf_blocks, uint64_t nbytes,
                          int32_t src_is_device, ib_qtensor **out) {
    IB_ENTER(ctx);
    IB_REQUIRE(out != nullptr, "ib_qtensor_upload: null output pointer");
    *out = nullptr;
    IB_REQUIRE(gguf_blocks != nullptr, "ib_qtensor_upload: null data pointer");
    const uint32_t be = block_elems(qtype), bb = block_bytes(qtype);
    IB_REQUIRE(be != 0, "ib_qtensor_upload: unsupported tensor type id %d (supported: F32=0, Q4_0=2, Q4_1=3, Q5_0=6, Q5_1=7, Q8_0=8, Q4_K=12, Q5_K=13, Q6_K=14, Q8_K=15)", qtype);
    IB_REQUIRE(rows > 0 && cols > 0, "ib_qtensor_upload: empty matrix %llux%llu", (unsigned long long)rows, (unsigned long long)cols);
    // the reference truncates rows/4 silently (crates/inferi/src/ops/gemv_quant.rs:271); here it is an error
    IB_REQUIRE(rows % 4 == 0, "ib_qtensor_upload: rows=%llu must be a multiple of 4", (unsigned long long)rows);
    IB_REQUIRE(cols % be == 0, "ib_qtensor_upload: cols=%llu must be a multiple of the block length %u", (unsigned long long)cols, be);
    IB_REQUIRE(rows < (1ull << 31) && cols < (1ull << 31), "ib_qtensor_upload: dimension too large");
    const uint64_t row_bytes = cols / be * bb;
    IB_REQUIRE(nbytes == rows * row_bytes, "ib_qtensor_upload: nbytes=%llu but %llux%llu of this type needs %llu", (unsigned long long)nbytes,
               (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)(rows * row_bytes));

    ib_qtensor *qt = new (std::nothrow) ib_qtensor();
    if (!qt) return set_error(IB_ERR_OOM, "host allocation failed");
    qt->ctx = ctx; qt->qtype = qtype; qt->rows = rows; qt->cols = cols; qt->row_bytes = row_bytes; qt->nbytes = nbytes;
    qt->nb = (uint32_t)(cols / be);
    qt->fast = gemv_fast_eligible(qtype, rows, cols);
    const bool soa = qt->fast && (qtype == IB_Q8_0 || qtype == IB_Q6_K);
    qt->layout = soa ? LAYOUT_SOA : LAYOUT_GGUF;
    // 16 spare bytes so that a 128-bit load of the last partial field never leaves the allocation
    cudaError_t e = cudaMalloc(&qt->dev, nbytes + 16);
    if (e != cudaSuccess) {
        delete qt;
        return set_error(IB_ERR_OOM, "cudaMalloc of %llu bytes failed: %s", (unsigned long long)nbytes, cudaGetErrorString(e));
    }
    int32_t rc = IB_OK;
    const cudaMemcpyKind kind = src_is_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    if (!soa) {
        e = cudaMemcpy(qt->dev, gguf_blocks, nbytes, kind);
        if (e != cudaSuccess) rc = set_error(IB_ERR_CUDA, "upload copy failed: %s", cudaGetErrorString(e));
    } else {
        uint8_t *staging = nullptr;
        const uint8_t *src = (const uint8_t *)gguf_blocks;
        if (!src_is_device) {
            e = cudaMalloc(&staging, nbytes);
            if (e == cudaSuccess) e = cudaMemcpy(staging, gguf_blocks, nbytes, cudaMemcpyHostToDevice);
            if (e != cudaSuccess) rc = set_error(e == cudaErrorMemoryAllocation ? IB_ERR_OOM : IB_ERR_CUDA, "upload staging failed: %s", cudaGetErrorString(e));
            src = staging;
        }
        if (rc == IB_OK) rc = retile_to_soa(ctx, 0, qtype, src, qt->dev, rows, qt->nb);
        if (rc == IB_OK) {
            e = cudaDeviceSynchronize();
            if (e != cudaSuccess) rc = set_error(IB_ERR_CUDA, "re-tiling failed: %s", cudaGetErrorString(e));
        }
        if (staging) cudaFree(staging);
    }
    if (rc != IB_OK) {
        cudaFree(qt->dev);
        delete qt;
        return rc;
    }
    *out = qt;
    return IB_OK;
}

int32_t ib_qtensor_destroy(ib_qtensor *qt) {
    if (!qt) return IB_OK;
    DeviceGuard guard(qt->ctx->device);
    if (qt->dev) cudaFree(qt->dev);
    delete qt;
    return IB_OK;
}

int32_t ib_qtensor_info(const ib_qtensor *qt, int32_t *qtype, uint64_t *rows, uint64_t *cols, uint64_t *nbytes) {
    IB_REQUIRE(qt, "ib_qtensor_info: null tensor");
    if (qtype) *qtype = qt->qtype;
    if (rows) *rows = qt->rows;
    if (cols) *cols = qt->cols;
    if (nbytes) *nbytes = qt->nbytes;
    return IB_OK;
}

// ---- ops ----
int32_t ib_gemv_quant(ib_ctx *ctx, void *stream, float *out_dev, const ib_qtensor *m, const float *v_dev) {
    IB_ENTER(ctx);
    IB_REQUIRE(m && out_dev && v_dev, "ib_gemv_quant: null argument");
    IB_REQUIRE(m->ctx->device == ctx->device, "ib_gemv_quant: tensor lives on device %d, context on %d", m->ctx->device, ctx->device);
    if (!m->fast) return launch_gemv_generic(ctx, (cudaStream_t)stream, m, v_dev, out_dev);
    GemvParams p = {};
    fill_seg(p.seg[0], m, out_dev);
    p.nseg = 1; p.cols = (uint32_t)m->cols; p.epi = EPI_STORE; p.x = v_dev;
    return launch_gemv(ctx, (cudaStream_t)stream, p);
}

int32_t ib_ffn_gate_up(ib_ctx *ctx, void *stream, float *out_dev, const ib_qtensor *gate, const ib_qtensor *up, const float *x_dev, const float *norm_w_dev,
                       float eps) {
    IB_ENTER(ctx);
    IB_REQUIRE(gate && up && out_dev && x_dev, "ib_ffn_gate_up: null argument");
    IB_REQUIRE(gate->ctx->device == ctx->device && up->ctx->device == ctx->device, "ib_ffn_gate_up: tensors live on another device");
    IB_REQUIRE(gate->rows == up->rows && gate->cols == up->cols && gate->qtype == up->qtype, "ib_ffn_gate_up: gate and up differ in shape or type");
    IB_REQUIRE(gate->fast && up->fast, "ib_ffn_gate_up: the matrices do not meet the alignment rules of the fused kernel");
    GemvParams p = {};
    fill_seg(p.seg[0], gate, out_dev);
    fill_seg(p.seg[1], up, nullptr);
    p.nseg = 2; p.cols = (uint32_t)gate->cols; p.epi = EPI_SWIGLU; p.x = x_dev; p.norm_w = norm_w_dev; p.eps = eps;
    return launch_gemv(ctx, (cudaStream_t)stream, p);
}

int32_t ib_gemv_quant_host(ib_ctx *ctx, float *out_host, const ib_qtensor *m, const float *v_host) {
    IB_ENTER(ctx);
    IB_REQUIRE(m && out_host && v_host, "ib_gemv_quant_host: null argument");
    float *buf = nullptr;
    IB_CHECK_CUDA(cudaMalloc(&buf, (m->rows + m->cols) * sizeof(float)));
    float *v = buf, *o = buf + m->cols;
    int32_t rc = IB_OK;
    cudaError_t e = cudaMemcpyAsync(v, v_host, m->cols * sizeof(float), cudaMemcpyHostToDevice, 0);
    if (e != cudaSuccess) rc = set_error(IB_ERR_CUDA, "h2d copy failed: %s", cudaGetErrorString(e));
    if (rc == IB_OK) rc = ib_gemv_quant(ctx, nullptr, o, m, v);
    if (rc == IB_OK) {
        e = cudaMemcpyAsync(out_host, o, m->rows * sizeof(float), cudaMemcpyDeviceToHost, 0);
        if (e == cudaSuccess) e = cudaStreamSynchronize(0);
        if (e != cudaSuccess) rc = set_error(IB_ERR_CUDA, "d2h copy failed: %s", cudaGetErrorString(e));
        if (rc == IB_OK) rc = check_device_error(ctx);
    }
    cudaFree(buf);
    return rc;
}

int32_t ib_rms_norm(ib_ctx *ctx, void *stream, float *out_dev, const float *x_dev, const float *w_dev, uint32_t n, float eps) {
    IB_ENTER(ctx);
    IB_REQUIRE(out_dev && x_dev && w_dev, "ib_rms_norm: null pointer");
    IB_REQUIRE(n > 0, "ib_rms_norm: empty vector");
    return launch_rms_norm(ctx, (cudaStream_t)stream, out_dev, x_dev, w_dev, n, eps);
}

int32_t ib_rope(ib_ctx *ctx, void *stream, int32_t variant, float *q_dev, uint32_t q_len, float *k_dev, uint32_t kv_dim, uint32_t head_size,
                uint32_t pos, float base_freq) {
    IB_ENTER(ctx);
    IB_REQUIRE(q_dev && k_dev, "ib_rope: null pointer");
    IB_REQUIRE(variant == IB_ROPE_ORIGINAL || variant == IB_ROPE_NEOX, "ib_rope: unknown variant %d", variant);
    // crates/inferi/src/ops/rope.rs:39-44
    IB_REQUIRE(q_len % 2 == 0 && q_len >= kv_dim, "ib_rope: q_len=%u must be even and >= kv_dim=%u", q_len, kv_dim);
    IB_REQUIRE(head_size >= 2 && head_size % 2 == 0 && head_size <= 256 && q_len % head_size == 0 && kv_dim % head_size == 0,
               "ib_rope: head_size=%u must be even, <= 256 and divide q_len and kv_dim", head_size);
    return launch_rope(ctx, (cudaStream_t)stream, variant, q_dev, q_len, k_dev, kv_dim, head_size, pos, base_freq);
}

int32_t ib_silu_mul(ib_ctx *ctx, void *stream, float *h1_dev, const float *h2_dev, uint32_t n) {
    IB_ENTER(ctx);
    IB_REQUIRE(h1_dev && h2_dev, "ib_silu_mul: null pointer");
    if (n == 0) return IB_OK;
    return launch_silu_mul(ctx, (cudaStream_t)stream, h1_dev, h2_dev, n);
}

int32_t ib_add_assign(ib_ctx *ctx, void *stream, float *a_dev, const float *b_dev, uint32_t n) {
    IB_ENTER(ctx);
    IB_REQUIRE(a_dev && b_dev, "ib_add_assign: null pointer");
    if (n == 0) return IB_OK;
    return launch_add_assign(ctx, (cudaStream_t)stream, a_dev, b_dev, n);
}

int32_t ib_attention(ib_ctx *ctx, void *stream, const ib_attn_params *params, const float *q_dev, const void *k_cache_dev, const void *v_cache_dev,
                     int32_t kv_dtype, float *out_dev) {
    IB_ENTER(ctx);
    IB_REQUIRE(params && q_dev && k_cache_dev && v_cache_dev && out_dev, "ib_attention: null argument");
    IB_REQUIRE(kv_dtype == IB_KV_F32 || kv_dtype == IB_KV_F16, "ib_attention: unknown kv dtype %d", kv_dtype);
    IB_REQUIRE(params->kv_mul >= 1 && params->n_heads >= params->kv_mul, "ib_attention: bad head counts");
    AttnLaunch a = {};
    a.p = *params;
    a.max_splits = attn_max_splits(ctx, *params);
    const size_t need = attn_scratch_bytes(*params, a.max_splits);
    if (need > ctx->attn_scratch_bytes) {
        // growing the scratch: wait for work that may still use the old one
        IB_CHECK_CUDA(cudaDeviceSynchronize());
        if (ctx->attn_scratch) cudaFree(ctx->attn_scratch);
        ctx->attn_scratch = nullptr;
        ctx->attn_scratch_bytes = 0;
        IB_CHECK_CUDA(cudaMalloc(&ctx->attn_scratch, need));
        ctx->attn_scratch_bytes = need;
    }
    if (!ctx->attn_counters) {
        IB_CHECK_CUDA(cudaMalloc(&ctx->attn_counters, 1024 * sizeof(unsigned int)));
        IB_CHECK_CUDA(cudaMemset(ctx->attn_counters, 0, 1024 * sizeof(unsigned int)));
    }
    IB_REQUIRE(params->n_heads / params->kv_mul <= 1024, "ib_attention: too many kv heads");
    a.q = q_dev; a.k_cache = k_cache_dev; a.v_cache = v_cache_dev; a.kv_dtype = kv_dtype; a.out = out_dev;
    a.scratch = ctx->attn_scratch; a.counters = ctx->attn_counters;
    return launch_attention(ctx, (cudaStream_t)stream, a);
}

int32_t ib_argmax(ib_ctx *ctx, void *stream, const float *logits_dev, uint32_t n, uint32_t *out_dev) {
    IB_ENTER(ctx);
    IB_REQUIRE(logits_dev && out_dev, "ib_argmax: null pointer");
    IB_REQUIRE(n > 0, "ib_argmax: empty vector");
    return launch_argmax(ctx, (cudaStream_t)stream, logits_dev, n, out_dev);
}

}  // extern "C"
