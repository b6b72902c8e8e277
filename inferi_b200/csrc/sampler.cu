// On-device token sampling: temperature, softmax, multinomial and top-p (nucleus) sampling.
//
// Replaces `Sampler::sample`, `sample_mult` and `sample_topp` (crates/inferi/src/models/sampler.rs:32-130) and the CPU
// softmax they call (crates/inferi/src/ops/softmax.rs:130-143).  The reference reads all logits back and samples on the
// host with an unseeded `rand::random()`; here the logits stay on the device and the coin of a position is a pure
// function of (seed, position), so a sequence can be reproduced.
//
// One CTA of 1024 threads (the work is a few passes over <= a few hundred thousand floats in L2):
//   x_i = logit_i / temperature;  p_i = exp(x_i - max x) / sum          (softmax.rs:134-142)
//   multinomial: first i with coin < p_0 + ... + p_i, else n - 1         (sampler.rs:62-77)
//   top-p: candidates p_i >= (1 - topp) / (n - 1), sorted by descending p (stable: ascending index on ties), cut after
//          the first prefix whose sum exceeds topp, then first i with coin * prefix_sum < running sum (sampler.rs:84-129)
// Sums run in a fixed order (per-thread chunks, then a block scan): results are deterministic; they can differ from a
// sequential f32 sum by rounding (of the order of sqrt(n) * 2^-24 in the running sum), which changes the sampled token only when
// the coin falls that close to a boundary between two tokens.
#include "common.cuh"

#include <math.h>

namespace ib {

constexpr int SAMPLE_THREADS = 1024;
constexpr uint32_t SAMPLE_SMEM_KEYS = 4096;   // candidates that are sorted in shared memory; more go through global memory

// coin of a position: splitmix64 of (seed, position), top 24 bits -> [0, 1)
__host__ __device__ inline float sample_coin(uint64_t seed, uint32_t pos) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * ((uint64_t)pos + 1ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(uint32_t)(z >> 40) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ float block_reduce_max(float v, float *sm) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (lane == 0) sm[warp] = v;
    __syncthreads();
    float r = sm[0];
    for (int w = 1; w < SAMPLE_THREADS / 32; w++) r = fmaxf(r, sm[w]);
    __syncthreads();
    return r;
}

// Exclusive scan of one value per thread in thread order; returns the prefix of this thread, *total gets the sum.
__device__ __forceinline__ float block_scan(float v, float *sm, float *total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) sm[warp] = inc;
    __syncthreads();
    float base = 0.f, tot = 0.f;
    for (int w = 0; w < SAMPLE_THREADS / 32; w++) {
        if (w == warp) base = tot;
        tot += sm[w];
    }
    __syncthreads();
    *total = tot;
    return base + inc - v;
}
__device__ __forceinline__ uint32_t block_scan_u32(uint32_t v, uint32_t *sm, uint32_t *total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) sm[warp] = inc;
    __syncthreads();
    uint32_t base = 0, tot = 0;
    for (int w = 0; w < SAMPLE_THREADS / 32; w++) {
        if (w == warp) base = tot;
        tot += sm[w];
    }
    __syncthreads();
    *total = tot;
    return base + inc - v;
}

// First index i in [0, count) with limit < value(0) + ... + value(i) (running sum in index order), or `none`.
// `running_at` receives the running sum at that index (or the total).  Values come from `get(i)`.
template <typename Get>
__device__ __forceinline__ uint32_t first_crossing(uint32_t count, float limit, Get get, float *smf, uint32_t *smu, uint32_t none, float *running_at) {
    const uint32_t chunk = (count + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const uint32_t i0 = min(count, threadIdx.x * chunk), i1 = min(count, i0 + chunk);
    float s = 0.f;
    for (uint32_t i = i0; i < i1; i++) s += get(i);
    float total;
    const float base = block_scan(s, smf, &total);
    uint32_t found = 0xFFFFFFFFu;
    float at = 0.f, run = base;
    for (uint32_t i = i0; i < i1; i++) {
        run += get(i);
        if (limit < run) { found = i; at = run; break; }
    }
    // the lowest index over the block, with its running sum
    __shared__ unsigned long long best;
    if (threadIdx.x == 0) best = ~0ull;
    __syncthreads();
    if (found != 0xFFFFFFFFu) atomicMin(&best, ((unsigned long long)found << 32) | __float_as_uint(at));
    __syncthreads();
    const unsigned long long b = best;
    __syncthreads();
    (void)smu;
    if (b == ~0ull) { *running_at = total; return none; }
    *running_at = __uint_as_float((uint32_t)b);
    return (uint32_t)(b >> 32);
}

__device__ __forceinline__ void cmp_swap(unsigned long long &a, unsigned long long &b, bool up) {
    if ((a > b) == up) { const unsigned long long t = a; a = b; b = t; }
}

// `probs` [n] and `keys` [next power of two >= n] are scratch.  `pos_ptr` / `seed`: the coin (sample_coin); with
// pos_ptr == null `coin_in` is used.  Writes the token to *out (and to *out2 if non-null).
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float *__restrict__ logits, uint32_t n, float temperature, float topp, uint64_t seed,
                                                                const uint32_t *pos_ptr, float coin_in, float *probs, unsigned long long *keys,
                                                                uint32_t *out, uint32_t *out2, uint32_t pdl) {
    extern __shared__ unsigned long long sm_keys[];   // SAMPLE_SMEM_KEYS
    __shared__ float smf[SAMPLE_THREADS / 32];
    __shared__ uint32_t smu[SAMPLE_THREADS / 32];
    if (pdl) {
        asm volatile("griddepcontrol.launch_dependents;");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    const float coin = pos_ptr ? sample_coin(seed, *pos_ptr) : coin_in;
    const uint32_t tid = threadIdx.x;

    // x = logits / temperature, softmax (softmax.rs:134-142)
    float mx = -INFINITY;
    for (uint32_t i = tid; i < n; i += SAMPLE_THREADS) {
        const float x = __fdiv_rn(__ldcg(logits + i), temperature);
        probs[i] = x;
        mx = fmaxf(mx, x);
    }
    mx = block_reduce_max(mx, smf);
    const uint32_t chunk = (n + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const uint32_t i0 = min(n, tid * chunk), i1 = min(n, i0 + chunk);
    __syncthreads();   // probs written with a strided pattern, read back in chunks
    float s = 0.f;
    for (uint32_t i = i0; i < i1; i++) {
        const float e = expf(probs[i] - mx);
        probs[i] = e;
        s += e;
    }
    float sum;
    block_scan(s, smf, &sum);
    for (uint32_t i = i0; i < i1; i++) probs[i] = __fdiv_rn(probs[i], sum);
    __syncthreads();

    uint32_t token;
    float run;
    if (topp <= 0.f || topp >= 1.f) {
        // sampler.rs:62-77
        token = first_crossing(n, coin, [&](uint32_t i) { return probs[i]; }, smf, smu, n - 1, &run);
    } else {
        // sampler.rs:84-129.  Candidates in index order (stable), key = descending probability then ascending index.
        const float cutoff = __fdiv_rn(1.0f - topp, (float)n - 1.0f);
        uint32_t cnt = 0;
        for (uint32_t i = i0; i < i1; i++) cnt += probs[i] >= cutoff;
        uint32_t n0;
        uint32_t at = block_scan_u32(cnt, smu, &n0);
        if (n0 == 0) {
            // No probability reaches the cut-off ((1 - topp) / (n - 1) can exceed the largest one, e.g. n = 2 with a small
            // topp).  The reference subtracts 1 from an unsigned zero there (sampler.rs:108); defined here as the arg-max,
            // lowest index on ties.
            __shared__ unsigned long long amax;
            if (tid == 0) amax = 0ull;
            __syncthreads();
            unsigned long long b = 0ull;
            for (uint32_t i = i0; i < i1; i++) {
                const unsigned long long k = ((unsigned long long)__float_as_uint(probs[i]) << 32) | (0xFFFFFFFFu - i);   // p >= 0: bits order like values
                b = k > b ? k : b;
            }
            if (i0 < i1) atomicMax(&amax, b);
            __syncthreads();
            if (tid == 0) {
                const uint32_t t = 0xFFFFFFFFu - (uint32_t)(amax & 0xFFFFFFFFull);
                *out = t;
                if (out2) *out2 = t;
            }
            return;
        }
        uint32_t cap = 1;
        while (cap < n0) cap <<= 1;
        unsigned long long *K = cap <= SAMPLE_SMEM_KEYS ? sm_keys : keys;
        for (uint32_t i = i0; i < i1; i++)
            if (probs[i] >= cutoff) K[at++] = ((unsigned long long)(~__float_as_uint(probs[i])) << 32) | i;
        for (uint32_t i = n0 + tid; i < cap; i += SAMPLE_THREADS) K[i] = ~0ull;
        __syncthreads();
        // bitonic sort, ascending keys
        for (uint32_t k = 2; k <= cap; k <<= 1)
            for (uint32_t j = k >> 1; j > 0; j >>= 1) {
                for (uint32_t t = tid; t < cap / 2; t += SAMPLE_THREADS) {
                    const uint32_t lo = ((t & ~(j - 1)) << 1) | (t & (j - 1)), hi = lo | j;
                    unsigned long long a = K[lo], b = K[hi];
                    cmp_swap(a, b, (lo & k) == 0);
                    K[lo] = a; K[hi] = b;
                }
                __syncthreads();
            }
        auto prob_at = [&](uint32_t i) { return __uint_as_float(~(uint32_t)(K[i] >> 32)); };
        float cumulative;
        uint32_t last = first_crossing(n0, topp, prob_at, smf, smu, n0 - 1, &cumulative);   // first prefix whose sum exceeds topp
        const float r = coin * cumulative;
        const uint32_t pick = first_crossing(last + 1, r, prob_at, smf, smu, last, &run);
        token = (uint32_t)(K[pick] & 0xFFFFFFFFull);
    }
    if (tid == 0) {
        *out = token;
        if (out2) *out2 = token;
    }
}

int32_t launch_sample(ib_ctx *ctx, cudaStream_t s, const float *logits, uint32_t n, float temperature, float topp, uint64_t seed, const uint32_t *pos_ptr,
                      float coin, float *probs, unsigned long long *keys, uint32_t *out, uint32_t *out2, uint32_t pdl) {
    static bool attr_set[16] = {false};
    const size_t smem = SAMPLE_SMEM_KEYS * sizeof(unsigned long long);
    if (!attr_set[ctx->device & 15]) {
        IB_CHECK_CUDA(cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[ctx->device & 15] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(SAMPLE_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    IB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, sample_kernel, logits, n, temperature, topp, seed, pos_ptr, coin, probs, keys, out, out2, pdl));
    ctx->launches++;
    return IB_OK;
}

size_t sample_keys_capacity(uint32_t n) {
    size_t cap = 1;
    while (cap < n) cap <<= 1;
    return cap;
}

}  // namespace ib

extern "C" int32_t ib_sample(ib_ctx *ctx, void *stream, const float *logits_dev, uint32_t n, float temperature, float topp, float coin, uint32_t *out_dev) {
    using namespace ib;
    IB_REQUIRE(ctx && logits_dev && out_dev, "ib_sample: null argument");
    IB_REQUIRE(cudaSetDevice(ctx->device) == cudaSuccess, "cudaSetDevice failed");
    IB_REQUIRE(n >= 2 && n <= (1u << 22), "ib_sample: n=%u outside [2, 4194304]", n);
    IB_REQUIRE(coin >= 0.f && coin < 1.f, "ib_sample: coin=%f outside [0, 1)", (double)coin);
    IB_REQUIRE(temperature >= 0.f, "ib_sample: negative temperature");
    if (temperature == 0.f) return launch_argmax(ctx, (cudaStream_t)stream, logits_dev, n, out_dev);   // sampler.rs:33-35
    // one stream-ordered allocation for both scratch arrays (probabilities, then the sort keys, 8-byte aligned)
    const size_t probs_bytes = (sizeof(float) * n + 7) & ~(size_t)7;
    uint8_t *scratch = nullptr;
    IB_CHECK_CUDA(cudaMallocAsync((void **)&scratch, probs_bytes + sizeof(unsigned long long) * sample_keys_capacity(n), (cudaStream_t)stream));
    const int32_t rc = launch_sample(ctx, (cudaStream_t)stream, logits_dev, n, temperature, topp, 0, nullptr, coin, reinterpret_cast<float *>(scratch),
                                     reinterpret_cast<unsigned long long *>(scratch + probs_bytes), out_dev, nullptr, 0);
    cudaFreeAsync(scratch, (cudaStream_t)stream);
    return rc;
}
