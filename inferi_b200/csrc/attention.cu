// Grouped-query decode attention over the KV cache: split-K flash-decoding with a log-sum-exp merge.
//
// Replaces crates/inferi-shaders/src/fused_attention.rs:63-241 (fused_attention, <= 2048 positions) and
// :374-617 (flash_attention) and their launcher crates/inferi/src/ops/batched_multiquery_attention.rs:27-77.
// Semantics follow `run_cpu` (:191-245): score = q.k / sqrt(head_size), softmax over positions 0..=pos, weighted
// sum of V.  Cache rows are [position, kv_dim] (fused_attention.rs:107-108), f32 as in the reference or f16.
//
// One CTA per (kv head, position slice): the slice's K and V rows are read once and used for all kv_mul query
// heads of the group (the reference reads them kv_mul times, one workgroup per query head).  Every CTA leaves an
// un-normalised partial (max, sum, accumulator); the last CTA of a kv head to arrive merges the partials — no CTA
// ever waits for another.  The split count is derived from the position on the device, so the same launch (and
// the same CUDA graph node) serves every context length.
#include "common.cuh"

#include <math.h>

namespace ib {

constexpr int ATTN_WARPS = 4;
constexpr int ATTN_THREADS = ATTN_WARPS * 32;
constexpr int ATTN_STEPS = 8;              // row steps per tile kept in registers
constexpr uint32_t ATTN_MIN_PER_SPLIT = 64;  // positions below which a further split does not pay

struct AttnArgs {
    ib_attn_params p;
    const uint32_t *pos_ptr;
    const float *q;
    const void *kc, *vc;
    float *out, *scratch;
    unsigned int *counters;
    uint32_t max_splits;
    uint32_t pdl;
};

template <typename T> struct KvVec;
template <> struct KvVec<__half> {
    static constexpr int EPL = 8;
    __device__ static __forceinline__ void unpack(const uint4 &r, float (&f)[8]) {
        const __half2 *h = reinterpret_cast<const __half2 *>(&r);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 t = __half22float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
};
template <> struct KvVec<float> {
    static constexpr int EPL = 4;
    __device__ static __forceinline__ void unpack(const uint4 &r, float (&f)[4]) {
        f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
    }
};

__device__ __forceinline__ float merge_weight(float m, float mx) { return (m == -INFINITY) ? 0.f : expf(m - mx); }

template <int HS, int KVM, typename T>
__global__ void __launch_bounds__(ATTN_THREADS) attn_kernel(const AttnArgs a) {
    constexpr int EPL = KvVec<T>::EPL;   // elements per 16-byte lane load
    constexpr int LPR = HS / EPL;        // lanes covering one cache row of this kv head
    constexpr int RPW = 32 / LPR;        // rows per warp step
    constexpr int TILE = ATTN_STEPS * RPW;
    static_assert(LPR >= 1 && LPR <= 32 && (32 % LPR) == 0, "head size / element type combination unsupported");

    __shared__ float sm_acc[ATTN_WARPS][KVM][HS];
    __shared__ float sm_m[ATTN_WARPS][KVM], sm_l[ATTN_WARPS][KVM];
    __shared__ bool is_last;

    if (a.pdl) {
        asm volatile("griddepcontrol.launch_dependents;");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    const uint32_t kvh = blockIdx.x, split = blockIdx.y;
    const uint32_t pos = a.pos_ptr ? *a.pos_ptr : a.p.pos;
    const uint32_t total = pos + 1;
    uint32_t nsplit = (total + ATTN_MIN_PER_SPLIT - 1) / ATTN_MIN_PER_SPLIT;
    if (nsplit > a.max_splits) nsplit = a.max_splits;
    const uint32_t per = (total + nsplit - 1) / nsplit;
    nsplit = (total + per - 1) / per;  // every remaining split is non-empty
    if (split >= nsplit) return;
    const uint32_t t0 = split * per, t1 = min(total, t0 + per);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane / LPR, li = lane % LPR;
    const uint32_t kv_dim = a.p.kv_dim;
    const T *kc = reinterpret_cast<const T *>(a.kc) + (size_t)kvh * HS + li * EPL;
    const T *vc = reinterpret_cast<const T *>(a.vc) + (size_t)kvh * HS + li * EPL;
    const float scale = 1.0f / sqrtf((float)HS);

    float qr[KVM][EPL];
#pragma unroll
    for (int m = 0; m < KVM; m++)
#pragma unroll
        for (int e = 0; e < EPL; e++) qr[m][e] = __ldcg(a.q + (size_t)(kvh * KVM + m) * HS + li * EPL + e);

    float M[KVM], l[KVM], acc[KVM][EPL];
#pragma unroll
    for (int m = 0; m < KVM; m++) {
        M[m] = -INFINITY;
        l[m] = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; e++) acc[m][e] = 0.f;
    }

    for (uint32_t base = t0 + warp * TILE; base < t1; base += ATTN_WARPS * TILE) {
        uint4 kraw[ATTN_STEPS], vraw[ATTN_STEPS];
#pragma unroll
        for (int s = 0; s < ATTN_STEPS; s++) {
            const uint32_t t = base + s * RPW + g;
            const uint32_t tc = t < t1 ? t : t1 - 1;
            kraw[s] = __ldcg(reinterpret_cast<const uint4 *>(kc + (size_t)tc * kv_dim));
            vraw[s] = __ldcg(reinterpret_cast<const uint4 *>(vc + (size_t)tc * kv_dim));
        }
        float sc[ATTN_STEPS][KVM];
#pragma unroll
        for (int s = 0; s < ATTN_STEPS; s++) {
            float kf[EPL];
            KvVec<T>::unpack(kraw[s], kf);
            const bool valid = (base + s * RPW + g) < t1;
#pragma unroll
            for (int m = 0; m < KVM; m++) {
                float d = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; e++) d = fmaf(qr[m][e], kf[e], d);
#pragma unroll
                for (int o = LPR / 2; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                sc[s][m] = valid ? d * scale : -INFINITY;
            }
        }
#pragma unroll
        for (int m = 0; m < KVM; m++) {
            float mx = sc[0][m];
#pragma unroll
            for (int s = 1; s < ATTN_STEPS; s++) mx = fmaxf(mx, sc[s][m]);
#pragma unroll
            for (int o = LPR; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float mn = fmaxf(M[m], mx);  // finite: the tile holds at least one valid position
            const float alpha = expf(M[m] - mn);
            M[m] = mn;
            l[m] *= alpha;
#pragma unroll
            for (int e = 0; e < EPL; e++) acc[m][e] *= alpha;
#pragma unroll
            for (int s = 0; s < ATTN_STEPS; s++) {
                const float pe = expf(sc[s][m] - mn);
                sc[s][m] = pe;
                l[m] += pe;
            }
        }
#pragma unroll
        for (int s = 0; s < ATTN_STEPS; s++) {
            float vf[EPL];
            KvVec<T>::unpack(vraw[s], vf);
#pragma unroll
            for (int m = 0; m < KVM; m++)
#pragma unroll
                for (int e = 0; e < EPL; e++) acc[m][e] = fmaf(sc[s][m], vf[e], acc[m][e]);
        }
    }

    // fold the row groups of the warp, then the warps of the CTA
#pragma unroll
    for (int m = 0; m < KVM; m++) {
#pragma unroll
        for (int o = LPR; o < 32; o <<= 1) {
            l[m] += __shfl_xor_sync(0xffffffffu, l[m], o);
#pragma unroll
            for (int e = 0; e < EPL; e++) acc[m][e] += __shfl_xor_sync(0xffffffffu, acc[m][e], o);
        }
        if (g == 0) {
#pragma unroll
            for (int e = 0; e < EPL; e++) sm_acc[warp][m][li * EPL + e] = acc[m][e];
            if (li == 0) { sm_m[warp][m] = M[m]; sm_l[warp][m] = l[m]; }
        }
    }
    __syncthreads();

    const uint32_t slot = HS + 2;
    float *part = a.scratch + ((size_t)kvh * a.max_splits + split) * KVM * slot;
    for (int idx = threadIdx.x; idx < KVM * HS; idx += ATTN_THREADS) {
        const int m = idx / HS, d = idx % HS;
        float mx = sm_m[0][m];
#pragma unroll
        for (int w = 1; w < ATTN_WARPS; w++) mx = fmaxf(mx, sm_m[w][m]);
        float o = 0.f, ls = 0.f;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; w++) {
            const float wt = merge_weight(sm_m[w][m], mx);
            o += wt * sm_acc[w][m][d];
            ls += wt * sm_l[w][m];
        }
        if (nsplit == 1) {
            a.out[(size_t)(kvh * KVM + m) * HS + d] = o / ls;
        } else {
            part[m * slot + d] = o;
            if (d == 0) { part[m * slot + HS] = mx; part[m * slot + HS + 1] = ls; }
        }
    }
    if (nsplit == 1) return;

    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = (atomicAdd(a.counters + kvh, 1u) == nsplit - 1);
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float *parts = a.scratch + (size_t)kvh * a.max_splits * KVM * slot;
    for (int idx = threadIdx.x; idx < KVM * HS; idx += ATTN_THREADS) {
        const int m = idx / HS, d = idx % HS;
        float mx = -INFINITY;
        for (uint32_t s = 0; s < nsplit; s++) mx = fmaxf(mx, __ldcg(parts + ((size_t)s * KVM + m) * slot + HS));
        float o = 0.f, ls = 0.f;
        for (uint32_t s = 0; s < nsplit; s++) {
            const float *ps = parts + ((size_t)s * KVM + m) * slot;
            const float wt = merge_weight(__ldcg(ps + HS), mx);
            o += wt * __ldcg(ps + d);
            ls += wt * __ldcg(ps + HS + 1);
        }
        a.out[(size_t)(kvh * KVM + m) * HS + d] = o / ls;
    }
    if (threadIdx.x == 0) a.counters[kvh] = 0u;
}

size_t attn_scratch_bytes(const ib_attn_params &p, uint32_t max_splits) {
    const size_t n_kv = p.n_heads / p.kv_mul;
    return n_kv * max_splits * p.kv_mul * (p.head_size + 2) * sizeof(float);
}

uint32_t attn_max_splits(const ib_ctx *ctx, const ib_attn_params &p) {
    const uint32_t n_kv = p.n_heads / p.kv_mul;
    uint32_t s = (uint32_t)(ctx->sm_count * 4) / (n_kv ? n_kv : 1);
    if (s < 1) s = 1;
    if (s > 256) s = 256;
    return s;
}

template <int HS, int KVM, typename T>
static int32_t launch_t(ib_ctx *ctx, cudaStream_t s, const AttnArgs &args, dim3 grid) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(ATTN_THREADS);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = args.pdl ? 1 : 0;
    IB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, attn_kernel<HS, KVM, T>, args));
    ctx->launches++;
    return IB_OK;
}

template <int HS, typename T>
static int32_t launch_kvm(ib_ctx *ctx, cudaStream_t s, const AttnArgs &args, dim3 grid) {
    switch (args.p.kv_mul) {
    case 1: return launch_t<HS, 1, T>(ctx, s, args, grid);
    case 2: return launch_t<HS, 2, T>(ctx, s, args, grid);
    case 4: return launch_t<HS, 4, T>(ctx, s, args, grid);
    case 8: return launch_t<HS, 8, T>(ctx, s, args, grid);
    default: return set_error(IB_ERR_UNSUPPORTED, "attention: kv_mul=%u (supported: 1, 2, 4, 8)", args.p.kv_mul);
    }
}

int32_t launch_attention(ib_ctx *ctx, cudaStream_t s, const AttnLaunch &a) {
    const ib_attn_params &p = a.p;
    IB_REQUIRE(p.kv_mul >= 1 && p.n_heads % p.kv_mul == 0, "attention: n_heads=%u is not a multiple of kv_mul=%u", p.n_heads, p.kv_mul);
    const uint32_t n_kv = p.n_heads / p.kv_mul;
    IB_REQUIRE(p.kv_dim == n_kv * p.head_size, "attention: kv_dim=%u != n_kv_heads*head_size=%u", p.kv_dim, n_kv * p.head_size);
    IB_REQUIRE(a.pos_ptr || p.pos < p.seq_len, "attention: pos=%u outside the cache of %u rows", p.pos, p.seq_len);
    AttnArgs args{p, a.pos_ptr, a.q, a.k_cache, a.v_cache, a.out, a.scratch, a.counters, a.max_splits, a.pdl};
    // with a host-known position only the splits that will do work are launched
    uint32_t splits = a.max_splits;
    if (!a.pos_ptr) {
        uint32_t need = (p.pos + 1 + ATTN_MIN_PER_SPLIT - 1) / ATTN_MIN_PER_SPLIT;
        if (need < splits) splits = need;
    }
    const dim3 grid(n_kv, splits);
    const bool f16 = a.kv_dtype == IB_KV_F16;
    if (p.head_size == 128) return f16 ? launch_kvm<128, __half>(ctx, s, args, grid) : launch_kvm<128, float>(ctx, s, args, grid);
    if (p.head_size == 64) return f16 ? launch_kvm<64, __half>(ctx, s, args, grid) : launch_kvm<64, float>(ctx, s, args, grid);
    return set_error(IB_ERR_UNSUPPORTED, "attention: head_size=%u (supported: 64, 128)", p.head_size);
}

}  // namespace ib

// -------------------------------------------------------------------------------------------------------------------
// ib_attention_static: decode attention for callers that must not allocate.
//
// Some hosts of this library run where device allocation is off limits once set-up is over: a real-time audio/serving
// thread that may not take the allocator's locks, a plugin whose host application owns the memory budget, code running
// inside a region where cudaMalloc would synchronise the device.  ib_attention() grows a scratch buffer with cudaMalloc
// on demand and needs a context (whose creation allocates); this variant needs neither.  Its split-K scratch is the
// fixed array below, part of the library image: every GPU that loads the library carries these ~1 MiB until the process
// exits, whether or not the entry point is ever called.
// -------------------------------------------------------------------------------------------------------------------
namespace ib {
constexpr uint32_t STATIC_ATTN_FLOATS = 262144;    // 1 MiB of partials: bounds n_heads * (head_size + 2) * splits
constexpr uint32_t STATIC_ATTN_KV_HEADS = 256;     // arrival counters, one per kv head
constexpr uint32_t STATIC_ATTN_MAX_SPLITS = 32;
constexpr int STATIC_ATTN_MAX_DEVICES = 64;
}  // namespace ib

static __device__ __align__(256) float g_static_attn_scratch[ib::STATIC_ATTN_FLOATS];
static __device__ __align__(256) unsigned int g_static_attn_counters[ib::STATIC_ATTN_KV_HEADS];

// Device addresses of the two arrays, looked up once per device.  In host code the array names above are only
// host-side stand-ins for the symbols; the addresses a kernel can use come from cudaGetSymbolAddress, called with the
// device in question current.
static float *g_static_scratch_addr[ib::STATIC_ATTN_MAX_DEVICES];
static unsigned int *g_static_counters_addr[ib::STATIC_ATTN_MAX_DEVICES];

extern "C" int32_t ib_attention_static(void *stream, const ib_attn_params *params, const float *q_dev, const void *k_cache_dev,
                                       const void *v_cache_dev, int32_t kv_dtype, float *out_dev) {
    using namespace ib;
    IB_REQUIRE(params && q_dev && k_cache_dev && v_cache_dev && out_dev, "ib_attention_static: null argument");
    IB_REQUIRE(kv_dtype == IB_KV_F32 || kv_dtype == IB_KV_F16, "ib_attention_static: unknown kv dtype %d", kv_dtype);
    const ib_attn_params &p = *params;
    IB_REQUIRE(p.kv_mul >= 1 && p.n_heads >= p.kv_mul && p.n_heads % p.kv_mul == 0 && p.head_size > 0, "ib_attention_static: bad head counts");
    const uint32_t n_kv = p.n_heads / p.kv_mul;
    const uint64_t per_split = (uint64_t)p.n_heads * (p.head_size + 2);   // floats one split of all heads leaves behind
    if (n_kv > STATIC_ATTN_KV_HEADS || per_split > STATIC_ATTN_FLOATS)
        return set_error(IB_ERR_UNSUPPORTED,
                         "ib_attention_static: %u heads of %u exceed the built-in scratch (n_heads * (head_size + 2) <= %u, kv heads <= %u); "
                         "use ib_attention, which allocates",
                         p.n_heads, p.head_size, STATIC_ATTN_FLOATS, STATIC_ATTN_KV_HEADS);
    uint32_t splits = (uint32_t)(STATIC_ATTN_FLOATS / per_split);
    if (splits > STATIC_ATTN_MAX_SPLITS) splits = STATIC_ATTN_MAX_SPLITS;

    int dev = -1;
    IB_CHECK_CUDA(cudaGetDevice(&dev));
    IB_REQUIRE(dev >= 0 && dev < STATIC_ATTN_MAX_DEVICES, "ib_attention_static: device ordinal %d not supported", dev);
    if (!g_static_scratch_addr[dev]) {
        // first call on this device: resolve the symbols (no allocation takes place; the arrays already exist)
        float *s = nullptr;
        unsigned int *c = nullptr;
        IB_CHECK_CUDA(cudaGetSymbolAddress((void **)&s, g_static_attn_scratch));
        IB_CHECK_CUDA(cudaGetSymbolAddress((void **)&c, g_static_attn_counters));
        g_static_counters_addr[dev] = c;
        g_static_scratch_addr[dev] = s;
    }
    ib_ctx local;                 // plain bookkeeping struct on the stack: launch_attention only counts launches in it
    local.device = dev;
    AttnLaunch a = {};
    a.p = p;
    a.q = q_dev; a.k_cache = k_cache_dev; a.v_cache = v_cache_dev; a.kv_dtype = kv_dtype; a.out = out_dev;
    a.scratch = g_static_scratch_addr[dev];
    a.counters = g_static_counters_addr[dev];   // zero when the library is loaded; the kernel puts every counter back to zero
    a.max_splits = splits;
    return launch_attention(&local, (cudaStream_t)stream, a);
}
