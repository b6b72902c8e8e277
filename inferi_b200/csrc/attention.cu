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
#include "attention.cuh"
#include "attention_gqa4.cuh"

namespace ib {

constexpr int ATTN_STEPS = 8;              // row steps per tile kept in registers

template <int HS, int KVM, typename T>
__global__ void __launch_bounds__(ATTN_THREADS) attn_kernel(const AttnArgs a) {
    __shared__ float sm[attn_block_smem_floats(HS, KVM)];
    if (a.pdl) asm volatile("griddepcontrol.launch_dependents;");
    // The position was written by the end of the previous token, many kernels ago, and not by the predecessor (which
    // only waits for its own predecessor after it has let this kernel start): it can be read before the wait.
    const uint32_t kvh = blockIdx.x, split = blockIdx.y;
    const uint32_t pos = a.pos_ptr ? *a.pos_ptr : a.p.pos;
    uint32_t nsplit, per;
    attn_split_plan(pos + 1, a.max_splits, nsplit, per);
    if (split >= nsplit) return;
    attn_block<HS, KVM, T, ATTN_STEPS>(a, a.kc, a.vc, kvh, split, nsplit, per, pos + 1, (int)threadIdx.x, 1, sm, a.pdl != 0);
}

size_t attn_scratch_bytes(const ib_attn_params &p, uint32_t max_splits) {
    const size_t n_kv = p.n_heads / p.kv_mul;
    return n_kv * max_splits * p.kv_mul * (p.head_size + 2) * sizeof(float);
}

uint32_t attn_max_splits(const ib_ctx *ctx, const ib_attn_params &p) {
    const uint32_t n_kv = p.n_heads / p.kv_mul;
    uint32_t s = (uint32_t)(ctx->sm_count * 3) / (n_kv ? n_kv : 1);   // three CTAs of either kernel fit one SM: one wave
    if (s < 1) s = 1;
    if (s > 256) s = 256;
    // the merging block stages every slice's (max, sum) in its accumulator area: 2 * splits * kv_mul floats must fit the
    // 4 * kv_mul * head_size it owns
    if (s > 2 * p.head_size) s = 2 * p.head_size;
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

// the Llama-3 shape (f16 cache, 4 query heads per kv head, head size 64 or 128, 16-byte aligned buffers) has a kernel of its own
bool attn_gqa4_eligible(const AttnLaunch &a) {
    return a.kv_dtype == IB_KV_F16 && a.p.kv_mul == 4 && (a.p.head_size == 64 || a.p.head_size == 128) && ((uintptr_t)a.q % 16) == 0 &&
           ((uintptr_t)a.k_cache % 16) == 0 && ((uintptr_t)a.v_cache % 16) == 0 && ((uintptr_t)a.out % 16) == 0 && ((uintptr_t)a.scratch % 16) == 0;
}

uint32_t attn_cluster_positions(const AttnLaunch &a) {
    return attn_gqa4_eligible(a) ? gqa4_cluster_size(a.max_splits) * GQA4_CLUSTER_PER : 0u;
}

int32_t launch_attention(ib_ctx *ctx, cudaStream_t s, const AttnLaunch &a) {
    const ib_attn_params &p = a.p;
    IB_REQUIRE(p.kv_mul >= 1 && p.n_heads % p.kv_mul == 0, "attention: n_heads=%u is not a multiple of kv_mul=%u", p.n_heads, p.kv_mul);
    const uint32_t n_kv = p.n_heads / p.kv_mul;
    IB_REQUIRE(p.kv_dim == n_kv * p.head_size, "attention: kv_dim=%u != n_kv_heads*head_size=%u", p.kv_dim, n_kv * p.head_size);
    IB_REQUIRE(a.pos_ptr || p.pos < p.seq_len, "attention: pos=%u outside the cache of %u rows", p.pos, p.seq_len);
    IB_REQUIRE(a.max_splits >= 1 && a.max_splits <= 2 * p.head_size && a.max_splits <= 256, "attention: %u position slices exceed what the merge step holds (%u)",
               a.max_splits, 2 * p.head_size < 256 ? 2 * p.head_size : 256);
    AttnArgs args{p, a.pos_ptr, a.q, a.k_cache, a.v_cache, a.out, a.scratch, a.counters, a.max_splits, a.pdl, 0u, a.q_step, a.out_step, a.counter_step, a.scratch_step};
    const bool f16 = a.kv_dtype == IB_KV_F16;
    const bool gqa4 = attn_gqa4_eligible(a);
    const uint32_t nq = a.n_queries > 1 ? a.n_queries : 1;
    IB_REQUIRE(nq == 1 || (gqa4 && !a.pos_ptr && p.pos + nq <= p.seq_len), "attention: a batched launch needs the f16 / 4-heads-per-kv-head kernel and host-known positions inside the cache");
    // with a host-known position only the splits that will do work are launched
    uint32_t splits = a.max_splits;
    if (!a.pos_ptr) {
        uint32_t need, per;
        if (gqa4) attn_split_plan(p.pos + nq, a.max_splits, need, per, GQA4_MIN_PER_SPLIT, GQA4_KNEE, GQA4_KNEE_PER);
        else attn_split_plan(p.pos + nq, a.max_splits, need, per);
        if (need < splits) splits = need;
    }
    if (gqa4) {
        // short contexts merge inside a thread-block cluster (the first one of the kv head)
        if (a.pos_ptr) {
            args.cluster = a.short_context ? gqa4_cluster_size(splits) : 0u;
        } else if (p.pos + nq <= GQA4_CLUSTER_MAX * GQA4_CLUSTER_PER) {
            const uint32_t want = (p.pos + nq + GQA4_MIN_PER_SPLIT - 1) / GQA4_MIN_PER_SPLIT;
            const uint32_t cs = want < GQA4_CLUSTER_MAX ? want : GQA4_CLUSTER_MAX;
            if (cs >= 2 && cs <= a.max_splits) { splits = cs; args.cluster = cs; }
        }
    }
    const dim3 grid(n_kv, splits, nq);
    if (gqa4) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(ATTN_THREADS);
        cfg.stream = s;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = args.cluster ? args.cluster : 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = args.pdl ? 2 : 1;
        if (p.head_size == 128) IB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, attn_gqa4_kernel<128>, args));
        else IB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, attn_gqa4_kernel<64>, args));
        ctx->launches++;
        return IB_OK;
    }
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
        // first call on this device: resolve the symbols.  With lazy module loading this is also the moment the driver loads
        // the module that holds the arrays (which may allocate and synchronise): make this call during set-up.
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
