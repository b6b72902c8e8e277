// Device side of the grouped-query decode attention: one 4-warp block of threads handles one (kv head, position slice)
// pair.  Used by the stand-alone attention kernel (one CTA per pair) and by the whole-token kernel (four such blocks
// per CTA, synchronised with named barriers).
//
// Semantics follow `run_cpu` of crates/inferi-shaders/src/fused_attention.rs:191-245: score = q.k / sqrt(head_size),
// softmax over positions 0..=pos, weighted sum of V.  Cache rows are [position, kv_dim] (fused_attention.rs:107-108).
#pragma once

#include "common.cuh"

#include <math.h>

namespace ib {

constexpr int ATTN_WARPS = 4;
constexpr int ATTN_THREADS = ATTN_WARPS * 32;
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
    uint32_t cluster;   // CTAs per thread-block cluster along the slices of a kv head (attn_gqa4_kernel only); 0: no clusters
    // Several queries in one launch (prompt prefill; gridDim.z = number of queries, only in the kernel for the Llama-3
    // shape): query z sits at position p.pos + z, its vectors, scratch and counters `*_step` elements after query 0's.
    uint32_t q_step, out_step, counter_step;
    size_t scratch_step;
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

__device__ __forceinline__ void attn_bar(int id) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(ATTN_THREADS) : "memory"); }

// Shared memory one block needs, in floats: accumulators [ATTN_WARPS][KVM][HS], running max and sum [ATTN_WARPS][KVM] each,
// one flag word.
__host__ __device__ constexpr uint32_t attn_block_smem_floats(uint32_t hs, uint32_t kvm) { return ATTN_WARPS * kvm * hs + 2 * ATTN_WARPS * kvm + 4; }

// The split of `total` positions: number of non-empty slices and positions per slice.
// With `knee` > 0 the slices stop multiplying at `knee` until each holds `knee_per` positions: the merge reads every
// slice's partial (eight per L2 round trip), so beyond a dozen slices more of them only pay once they shorten the row loop
// by more than they lengthen the merge.
__host__ __device__ __forceinline__ void attn_split_plan(uint32_t total, uint32_t max_splits, uint32_t &nsplit, uint32_t &per,
                                                         uint32_t min_per_split = ATTN_MIN_PER_SPLIT, uint32_t knee = 0, uint32_t knee_per = 0) {
    nsplit = (total + min_per_split - 1) / min_per_split;
    if (knee && nsplit > knee) {
        const uint32_t by_len = (total + knee_per - 1) / knee_per;
        nsplit = by_len > knee ? by_len : knee;
    }
    if (nsplit > max_splits) nsplit = max_splits;
    per = (total + nsplit - 1) / nsplit;
    nsplit = (total + per - 1) / per;  // every remaining split is non-empty
}

// QS = the group's query vectors are staged in shared memory (KVM * HS more floats after the block's other arrays) and
// read per use instead of being held in registers: for callers that are short of registers.
// One block (ATTN_THREADS threads, `tid` = 0..127, synchronised on named barrier `bar`) computes slice `split` of kv head
// `kvh` for all KVM query heads of the group; K and V rows are read once for the group.  With more than one slice every
// block leaves an un-normalised partial (max, sum, accumulator) and the last block of the kv head to arrive merges them:
// no block ever waits for another.  STEPS = cache-row steps per tile kept in registers.
template <int HS, int KVM, typename T, int STEPS, bool QS = false>
__device__ __forceinline__ void attn_block(const AttnArgs &a, const void *k_cache, const void *v_cache, uint32_t kvh, uint32_t split, uint32_t nsplit,
                                           uint32_t per, uint32_t total, int tid, int bar, float *sm, bool wait_inside = false) {
    constexpr int EPL = KvVec<T>::EPL;   // elements per 16-byte lane load
    constexpr int LPR = HS / EPL;        // lanes covering one cache row of this kv head
    constexpr int RPW = 32 / LPR;        // rows per warp step
    constexpr int TILE = STEPS * RPW;
    static_assert(LPR >= 1 && LPR <= 32 && (32 % LPR) == 0, "head size / element type combination unsupported");

    float *sm_acc = sm;                                  // [ATTN_WARPS][KVM][HS]
    float *sm_m = sm + ATTN_WARPS * KVM * HS;            // [ATTN_WARPS][KVM]
    float *sm_l = sm_m + ATTN_WARPS * KVM;               // [ATTN_WARPS][KVM]
    uint32_t *sm_last = reinterpret_cast<uint32_t *>(sm_l + ATTN_WARPS * KVM);

    const uint32_t t0 = split * per, t1 = min(total, t0 + per);
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane / LPR, li = lane % LPR;
    const uint32_t kv_dim = a.p.kv_dim;
    const T *kc = reinterpret_cast<const T *>(k_cache) + (size_t)kvh * HS + li * EPL;
    const T *vc = reinterpret_cast<const T *>(v_cache) + (size_t)kvh * HS + li * EPL;
    const float scale = 1.0f / sqrtf((float)HS);

    // `wait_inside`: the kernel was launched ahead of its predecessor's completion (programmatic dependent launch) and has
    // not waited for it yet.  The predecessor writes this token's q and the newest cache row (position total - 1); every
    // older cache row was written by earlier tokens.  So the first tile's older rows are requested now, the wait comes
    // next, and q and the newest row are read after it: the cache round trip overlaps the predecessor's tail.
    uint4 kraw[STEPS], vraw[STEPS];
    const uint32_t base0 = t0 + warp * TILE;
    if (wait_inside) {
        if (base0 < t1) {
#pragma unroll
            for (int s = 0; s < STEPS; s++) {
                const uint32_t t = base0 + s * RPW + g;
                const uint32_t tc = t < t1 ? t : t1 - 1;
                if (tc + 1 != total) {
                    kraw[s] = __ldcg(reinterpret_cast<const uint4 *>(kc + (size_t)tc * kv_dim));
                    vraw[s] = __ldcg(reinterpret_cast<const uint4 *>(vc + (size_t)tc * kv_dim));
                }
            }
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (base0 < t1) {
#pragma unroll
            for (int s = 0; s < STEPS; s++) {
                const uint32_t t = base0 + s * RPW + g;
                const uint32_t tc = t < t1 ? t : t1 - 1;
                if (tc + 1 == total) {
                    kraw[s] = __ldcg(reinterpret_cast<const uint4 *>(kc + (size_t)tc * kv_dim));
                    vraw[s] = __ldcg(reinterpret_cast<const uint4 *>(vc + (size_t)tc * kv_dim));
                }
            }
        }
    }

    float qr[QS ? 1 : KVM][QS ? 1 : EPL];
    float *sm_q = reinterpret_cast<float *>(sm_last + 4);   // [KVM][HS], only with QS
    if (QS) {
        for (int i = tid; i < KVM * HS; i += ATTN_THREADS) sm_q[i] = __ldcg(a.q + (size_t)kvh * KVM * HS + i);
        attn_bar(bar);
    } else {
#pragma unroll
        for (int m = 0; m < KVM; m++)
#pragma unroll
            for (int e = 0; e < EPL; e++) qr[QS ? 0 : m][QS ? 0 : e] = __ldcg(a.q + (size_t)(kvh * KVM + m) * HS + li * EPL + e);
    }

    float M[KVM], l[KVM], acc[KVM][EPL];
#pragma unroll
    for (int m = 0; m < KVM; m++) {
        M[m] = -INFINITY;
        l[m] = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; e++) acc[m][e] = 0.f;
    }

    for (uint32_t base = base0; base < t1; base += ATTN_WARPS * TILE) {
        if (!(wait_inside && base == base0)) {
#pragma unroll
            for (int s = 0; s < STEPS; s++) {
                const uint32_t t = base + s * RPW + g;
                const uint32_t tc = t < t1 ? t : t1 - 1;
                kraw[s] = __ldcg(reinterpret_cast<const uint4 *>(kc + (size_t)tc * kv_dim));
                vraw[s] = __ldcg(reinterpret_cast<const uint4 *>(vc + (size_t)tc * kv_dim));
            }
        }
        float sc[STEPS][KVM];
#pragma unroll
        for (int s = 0; s < STEPS; s++) {
            float kf[EPL];
            KvVec<T>::unpack(kraw[s], kf);
            const bool valid = (base + s * RPW + g) < t1;
#pragma unroll
            for (int m = 0; m < KVM; m++) {
                float d = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; e++) d = fmaf(QS ? sm_q[m * HS + li * EPL + e] : qr[QS ? 0 : m][QS ? 0 : e], kf[e], d);
#pragma unroll
                for (int o = LPR / 2; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                sc[s][m] = valid ? d * scale : -INFINITY;
            }
        }
#pragma unroll
        for (int m = 0; m < KVM; m++) {
            float mx = sc[0][m];
#pragma unroll
            for (int s = 1; s < STEPS; s++) mx = fmaxf(mx, sc[s][m]);
#pragma unroll
            for (int o = LPR; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float mn = fmaxf(M[m], mx);  // finite: the tile holds at least one valid position
            const float alpha = expf(M[m] - mn);
            M[m] = mn;
            l[m] *= alpha;
#pragma unroll
            for (int e = 0; e < EPL; e++) acc[m][e] *= alpha;
#pragma unroll
            for (int s = 0; s < STEPS; s++) {
                const float pe = expf(sc[s][m] - mn);
                sc[s][m] = pe;
                l[m] += pe;
            }
        }
#pragma unroll
        for (int s = 0; s < STEPS; s++) {
            float vf[EPL];
            KvVec<T>::unpack(vraw[s], vf);
#pragma unroll
            for (int m = 0; m < KVM; m++)
#pragma unroll
                for (int e = 0; e < EPL; e++) acc[m][e] = fmaf(sc[s][m], vf[e], acc[m][e]);
        }
    }

    // fold the row groups of the warp, then the warps of the block
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
            for (int e = 0; e < EPL; e++) sm_acc[(warp * KVM + m) * HS + li * EPL + e] = acc[m][e];
            if (li == 0) { sm_m[warp * KVM + m] = M[m]; sm_l[warp * KVM + m] = l[m]; }
        }
    }
    attn_bar(bar);

    const uint32_t slot = HS + 2;
    float *part = a.scratch + ((size_t)kvh * a.max_splits + split) * KVM * slot;
    for (int idx = tid; idx < KVM * HS; idx += ATTN_THREADS) {
        const int m = idx / HS, d = idx % HS;
        float mx = sm_m[m];
#pragma unroll
        for (int w = 1; w < ATTN_WARPS; w++) mx = fmaxf(mx, sm_m[w * KVM + m]);
        float o = 0.f, ls = 0.f;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; w++) {
            const float wt = merge_weight(sm_m[w * KVM + m], mx);
            o += wt * sm_acc[(w * KVM + m) * HS + d];
            ls += wt * sm_l[w * KVM + m];
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
    attn_bar(bar);
    if (tid == 0) *sm_last = (atomicAdd(a.counters + kvh, 1u) == nsplit - 1) ? 1u : 0u;
    attn_bar(bar);
    if (*sm_last == 0u) return;
    __threadfence();
    // merge of the kv head's partials.  Maxima and sums of all slices first go to shared memory (the block's accumulator
    // area is free by now), so that the weighted sum over slices is a loop of independent loads.
    const float *parts = a.scratch + (size_t)kvh * a.max_splits * KVM * slot;
    float *pm = sm_acc, *pl = sm_acc + nsplit * KVM;   // [nsplit][KVM] each; fits because the launcher keeps nsplit <= 2 * HS (sm_acc holds 4 * KVM * HS floats)
    for (uint32_t i = tid; i < nsplit * KVM; i += ATTN_THREADS) {
        const float *ps = parts + (size_t)i * slot;    // slice i / KVM, head i % KVM
        pm[i] = __ldcg(ps + HS);
        pl[i] = __ldcg(ps + HS + 1);
    }
    attn_bar(bar);
    // every thread owns KVM * HS / ATTN_THREADS outputs of one head (HS is a multiple of ATTN_THREADS or divides it); the
    // loads of eight slices are issued together
    constexpr int PER = (KVM * HS + ATTN_THREADS - 1) / ATTN_THREADS;
    float o[PER], ls[PER], mx[PER];
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int m = min((tid + j * ATTN_THREADS) / HS, KVM - 1);
        float v = -INFINITY;
        for (uint32_t s = 0; s < nsplit; s++) v = fmaxf(v, pm[s * KVM + m]);
        mx[j] = v; o[j] = 0.f; ls[j] = 0.f;
    }
#pragma unroll 8
    for (uint32_t s = 0; s < nsplit; s++) {
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const int idx = min(tid + j * ATTN_THREADS, KVM * HS - 1), m = idx / HS, d = idx % HS;
            const float wt = merge_weight(pm[s * KVM + m], mx[j]);
            o[j] += wt * __ldcg(parts + ((size_t)s * KVM + m) * slot + d);
            ls[j] += wt * pl[s * KVM + m];
        }
    }
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int idx = tid + j * ATTN_THREADS, m = idx / HS, d = idx % HS;
        if (idx < KVM * HS) a.out[(size_t)(kvh * KVM + m) * HS + d] = o[j] / ls[j];
    }
    if (tid == 0) a.counters[kvh] = 0u;
}

}  // namespace ib
