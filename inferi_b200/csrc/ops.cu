// Stand-alone element-wise ops of the token loop (RMSNorm, RoPE, SwiGLU, residual add, arg-max).
// Inside the model these are fused into GEMV prologues/epilogues; the stand-alone kernels serve the
// op-level API that mirrors crates/inferi/src/ops/{rms_norm,rope,silu}.rs and context.rs:516-530.
#include "common.cuh"

#include <math.h>

namespace ib {

// ---- RMSNorm: crates/inferi-shaders/src/rms_norm.rs:78-121 ----
__global__ void __launch_bounds__(1024) rms_norm_kernel(float *__restrict__ out, const float *__restrict__ x, const float *__restrict__ w, uint32_t n,
                                                        float eps) {
    __shared__ float red[33];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    float ss = 0.f;
    for (uint32_t i = tid; i < n; i += blockDim.x) {
        const float v = x[i];
        ss += v * v;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (int i = 0; i < nwarps; i++) t += red[i];
        red[32] = 1.0f / sqrtf(t / (float)n + eps);
    }
    __syncthreads();
    const float rms = red[32];
    for (uint32_t i = tid; i < n; i += blockDim.x) out[i] = (x[i] * rms) * w[i];
}

int32_t launch_rms_norm(ib_ctx *ctx, cudaStream_t s, float *out, const float *x, const float *w, uint32_t n, float eps) {
    const int threads = n >= 4096 ? 1024 : (n >= 1024 ? 512 : 128);
    rms_norm_kernel<<<1, threads, 0, s>>>(out, x, w, n, eps);
    ctx->launches++;
    IB_CHECK_CUDA(cudaGetLastError());
    return IB_OK;
}

// ---- RoPE: crates/inferi-shaders/src/rope.rs:51-92 (Original), :97-141 (NeoX) ----
// The per-dimension frequencies theta_j = base^(-2j/head_size) are computed on the host with the C library's
// powf and passed by value, so that device and host agree on them bit for bit.
struct RopeTheta { float t[128]; };

__global__ void rope_kernel(int variant, float *__restrict__ q, uint32_t q_len, float *__restrict__ k, uint32_t kv_dim, uint32_t head_size, uint32_t pos,
                            const RopeTheta th) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= q_len / 2) return;
    const uint32_t half = head_size / 2;
    uint32_t i0, i1, j;
    if (variant == IB_ROPE_ORIGINAL) { i0 = 2 * i; i1 = i0 + 1; j = ((2 * i) % head_size) / 2; }
    else { const uint32_t head = i / half; j = i % half; i0 = head * head_size + j; i1 = i0 + half; }
    float sn, cs;
    sincosf((float)pos * th.t[j], &sn, &cs);
    float x = q[i0], y = q[i1];
    q[i0] = cs * x - sn * y;
    q[i1] = sn * x + cs * y;
    if (i0 < kv_dim) {
        x = k[i0]; y = k[i1];
        k[i0] = cs * x - sn * y;
        k[i1] = sn * x + cs * y;
    }
}

int32_t launch_rope(ib_ctx *ctx, cudaStream_t s, int variant, float *q, uint32_t q_len, float *k, uint32_t kv_dim, uint32_t head_size, uint32_t pos,
                    float base_freq) {
    RopeTheta th;
    for (uint32_t j = 0; j < head_size / 2; j++) th.t[j] = powf(base_freq, -(float)(2 * j) / (float)head_size);
    const uint32_t n = q_len / 2;
    rope_kernel<<<(n + 127) / 128, 128, 0, s>>>(variant, q, q_len, k, kv_dim, head_size, pos, th);
    ctx->launches++;
    IB_CHECK_CUDA(cudaGetLastError());
    return IB_OK;
}

// ---- SwiGLU: crates/inferi-shaders/src/silu.rs:24-53 ----
__global__ void silu_mul_kernel(float *__restrict__ h1, const float *__restrict__ h2, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float a = h1[i];
        h1[i] = h2[i] * (a / (1.0f + expf(-a)));
    }
}
int32_t launch_silu_mul(ib_ctx *ctx, cudaStream_t s, float *h1, const float *h2, uint32_t n) {
    silu_mul_kernel<<<(n + 255) / 256, 256, 0, s>>>(h1, h2, n);
    ctx->launches++;
    IB_CHECK_CUDA(cudaGetLastError());
    return IB_OK;
}

// ---- residual add: crates/inferi/src/context.rs:516-530 ----
__global__ void add_assign_kernel(float *__restrict__ a, const float *__restrict__ b, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] += b[i];
}
int32_t launch_add_assign(ib_ctx *ctx, cudaStream_t s, float *a, const float *b, uint32_t n) {
    add_assign_kernel<<<(n + 255) / 256, 256, 0, s>>>(a, b, n);
    ctx->launches++;
    IB_CHECK_CUDA(cudaGetLastError());
    return IB_OK;
}

// ---- greedy arg-max: crates/inferi/src/models/sampler.rs:54-56; lowest index on ties ----
__device__ __forceinline__ unsigned long long amax_key(float v, uint32_t idx) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - idx);
}

constexpr int ARGMAX_MAX_CTAS = 1024;

__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ x, uint32_t n, unsigned long long *slots, unsigned int *counter, uint32_t *out) {
    __shared__ unsigned long long sm[8];
    __shared__ bool is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned long long best = 0ull;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) best = max(best, amax_key(x[i], i));
#pragma unroll
    for (int o = 16; o; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (lane == 0) sm[warp] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 0; w < 8; w++) best = max(best, sm[w]);
        slots[blockIdx.x] = best;
        __threadfence();
        is_last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (is_last) {
        __threadfence();
        best = 0ull;
        for (uint32_t i = threadIdx.x; i < gridDim.x; i += blockDim.x) best = max(best, __ldcg(slots + i));
#pragma unroll
        for (int o = 16; o; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
        __syncthreads();
        if (lane == 0) sm[warp] = best;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 0; w < 8; w++) best = max(best, sm[w]);
            *out = 0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull);
            *counter = 0u;
        }
    }
}

int32_t ensure_argmax_scratch(ib_ctx *ctx) {
    if (!ctx->argmax_scratch) {
        IB_CHECK_CUDA(cudaMalloc(&ctx->argmax_scratch, sizeof(unsigned long long) * ARGMAX_MAX_CTAS));
        IB_CHECK_CUDA(cudaMalloc(&ctx->argmax_counter, sizeof(unsigned int)));
        IB_CHECK_CUDA(cudaMemset(ctx->argmax_counter, 0, sizeof(unsigned int)));
    }
    return IB_OK;
}

int32_t launch_argmax(ib_ctx *ctx, cudaStream_t s, const float *x, uint32_t n, uint32_t *out) {
    int32_t rc = ensure_argmax_scratch(ctx);
    if (rc) return rc;
    int grid = (int)((n + 1023) / 1024);
    if (grid > ctx->sm_count * 2) grid = ctx->sm_count * 2;
    if (grid < 1) grid = 1;
    argmax_kernel<<<grid, 256, 0, s>>>(x, n, ctx->argmax_scratch, ctx->argmax_counter, out);
    ctx->launches++;
    IB_CHECK_CUDA(cudaGetLastError());
    return IB_OK;
}

}  // namespace ib
