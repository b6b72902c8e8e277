// Decode attention for the shape the Llama-3 family uses: f16 cache, 4 query heads per kv head, head size 64 or 128.
//
// Same semantics and the same split-K scheme as attention.cuh (one CTA per (kv head, position slice), un-normalised
// partials, the last CTA of a kv head to arrive merges them; crates/inferi-shaders/src/fused_attention.rs:63-241 and
// :374-617 are what it replaces), but built for a short critical path at small contexts and for few instructions per
// cache row at long ones:
//  * a warp step covers 8 cache rows (HS 128: 4 steps of 2 rows, 16 lanes per row; HS 64: 2 steps of 4 rows, 8 lanes per
//    row); a lane holds 8 elements of a row and the matching 8 elements of the 4 query vectors;
//  * the 16 (or 8) per-lane partial scores of the step go through a halving exchange (each shuffle moves one value and
//    leaves half as many to reduce) instead of a butterfly per score: afterwards every lane owns exactly one
//    (row, head) score, so exp() is evaluated once per score, not once per lane;
//  * the probabilities travel back to the lanes through 128 bytes of shared memory per warp;
//  * multiply-adds are issued as packed pairs (fma.rn.f32x2);
//  * the loop body is small (no 8-step unrolling): at short contexts the kernel runs its code once, and the time goes
//    to instruction fetch if the code is long.
#pragma once

#include "attention.cuh"

#include <cooperative_groups.h>

namespace ib {

constexpr uint32_t GQA4_ROWS_PER_WARP_STEP = 8;
// Slices: one warp step of every warp (32 positions) each while there are at most 16 of them, then 16 slices that grow to
// 128 positions, then slices of 128 positions up to the launch's maximum, then longer ones.  Measured on a B200 (us per
// launch at 128 / 512 / 2048 / 8192 positions): 32 per slice throughout 4.6 / 6.1 / 12.6 / 17.1; 128 per slice 5.4 / 7.6 /
// 9.1 / 17.1; 256 per slice 5.4 / 10.6 / 11.3 / 16.1.
constexpr uint32_t GQA4_MIN_PER_SPLIT = ATTN_WARPS * GQA4_ROWS_PER_WARP_STEP, GQA4_KNEE = 16, GQA4_KNEE_PER = 128;
// Short contexts: the slices of a kv head (at most 8) are the CTAs of one thread-block cluster.  They leave their partials in
// the shared memory of the cluster's first CTA (distributed shared memory) and meet at the cluster barrier; the first CTA
// merges from its own shared memory.  Publishing the partials through global memory, counting arrivals with an atomic and
// reading them back are three L2 round trips (~2.6 us of a ~6 us kernel at these lengths); the cluster barrier is one
// hardware barrier.  Longer contexts use more slices than a cluster has CTAs and keep the global-memory merge.
// The cluster size is a divisor of the launch's slice count (so that no CTA is launched for the clusters' sake: with 55
// slices x 8 kv heads = 440 CTAs the grid is exactly one wave of 148 SMs x 3, and rounding 55 up to 56 made a second wave
// that cost 40 % at long contexts); `cluster` = 0: no clusters.
constexpr uint32_t GQA4_CLUSTER_MAX = 8, GQA4_CLUSTER_PER = 64;   // beyond two row-loop iterations per slice the sixteen slices of the global merge are faster
__host__ __device__ __forceinline__ uint32_t gqa4_cluster_size(uint32_t splits) {
    for (uint32_t c = GQA4_CLUSTER_MAX; c >= 2; c--)
        if (splits % c == 0) return c;
    return 0;
}
__host__ __device__ __forceinline__ void gqa4_plan(uint32_t total, uint32_t max_splits, uint32_t cluster, uint32_t &nsplit, uint32_t &per, bool &in_cluster) {
    in_cluster = cluster != 0 && total <= cluster * GQA4_CLUSTER_PER;
    if (in_cluster) {
        nsplit = (total + GQA4_MIN_PER_SPLIT - 1) / GQA4_MIN_PER_SPLIT;
        if (nsplit > cluster) nsplit = cluster;
        per = (total + nsplit - 1) / nsplit;
        nsplit = (total + per - 1) / per;
    } else {
        attn_split_plan(total, max_splits, nsplit, per, GQA4_MIN_PER_SPLIT, GQA4_KNEE, GQA4_KNEE_PER);
    }
}

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    unsigned long long ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

// Halving exchange over the L lanes of a row: on entry every lane holds N partial sums (one per (step, head)); after the
// round with lane distance o the lanes whose bit o is set keep the upper half of the values, the others the lower half,
// each added to the partner's copy.  After log2(L) rounds (N == L) lane li of the row holds the complete sum number li.
template <int N>
__device__ __forceinline__ void halve_exchange(float (&v)[N], int lane, int o) {
    const bool up = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < N / 2; i++) {
        const float keep = up ? v[i + N / 2] : v[i];
        const float send = up ? v[i] : v[i + N / 2];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
    }
}

template <int HS>
__global__ void __launch_bounds__(ATTN_THREADS, 3) attn_gqa4_kernel(const AttnArgs a_in) {
    // query blockIdx.z of a batched launch (prompt prefill); z = 0 and steps of 0 otherwise
    AttnArgs a = a_in;
    a.q += (size_t)blockIdx.z * a_in.q_step;
    a.out += (size_t)blockIdx.z * a_in.out_step;
    a.scratch += (size_t)blockIdx.z * a_in.scratch_step;
    a.counters += (size_t)blockIdx.z * a_in.counter_step;
    a.p.pos += blockIdx.z;
    constexpr int KVM = 4, EPL = 8;
    constexpr int L = HS / EPL;          // lanes per cache row
    constexpr int RPW = 32 / L;          // rows per warp step
    constexpr int STEPS = L / KVM;       // steps per warp iteration: STEPS * KVM partial scores per lane = L
    constexpr int ROWS = STEPS * RPW;    // = 8
    static_assert(ROWS == (int)GQA4_ROWS_PER_WARP_STEP && STEPS * KVM == L, "lane layout");
    __shared__ __align__(16) float sm_acc[ATTN_WARPS * KVM * HS];
    __shared__ float sm_m[ATTN_WARPS * KVM], sm_l[ATTN_WARPS * KVM];
    __shared__ __align__(16) float sm_p[ATTN_WARPS][32];
    __shared__ __align__(16) float sm_alpha[ATTN_WARPS][4];
    __shared__ uint32_t sm_last;
    __shared__ __align__(16) float sm_cl[GQA4_CLUSTER_MAX * KVM * (HS + 2)];   // cluster mode: the slices' partials, in the first CTA

    if (a.pdl) asm volatile("griddepcontrol.launch_dependents;");
    // The position was written at the end of the previous token, not by the predecessor: it can be read before the wait.
    const uint32_t kvh = blockIdx.x, split = blockIdx.y;
    const uint32_t total = (a.pos_ptr ? *a.pos_ptr : a.p.pos) + 1;
    uint32_t nsplit, per;
    bool in_cluster;
    gqa4_plan(total, a.max_splits, a.cluster, nsplit, per, in_cluster);
    // cluster mode: the first cluster of a kv head (slices 0 .. a.cluster - 1) does the work, all of its CTAs meet at the barrier below
    // (the ones without a slice bring nothing); the other clusters leave as a whole
    if (in_cluster ? split >= a.cluster : split >= nsplit) return;
    if (in_cluster && split >= nsplit) {
        if (nsplit > 1) cooperative_groups::this_cluster().sync();   // the barrier of the working CTAs below
        return;
    }
    const uint32_t t0 = split * per, t1 = min(total, t0 + per);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane / L, li = lane % L;
    const uint32_t kv_dim = a.p.kv_dim;
    const __half *kc = reinterpret_cast<const __half *>(a.kc) + (size_t)kvh * HS + li * EPL;
    const __half *vc = reinterpret_cast<const __half *>(a.vc) + (size_t)kvh * HS + li * EPL;
    const float scale = 1.0f / sqrtf((float)HS);

    // First iteration: the predecessor (the q/k/v kernel) writes this token's q and the newest cache row (position
    // total - 1); every older row is from earlier tokens.  So the older rows are requested before the wait for the
    // predecessor, q and the newest row after it: the cache round trip overlaps the predecessor's tail.
    uint4 kraw[STEPS], vraw[STEPS];
    const uint32_t base0 = t0 + warp * ROWS;
    if (base0 < t1) {
#pragma unroll
        for (int s = 0; s < STEPS; s++) {
            const uint32_t t = base0 + s * RPW + g, tc = t < t1 ? t : t1 - 1;
            if (tc + 1 != total || !a.pdl) {
                kraw[s] = __ldcg(reinterpret_cast<const uint4 *>(kc + (size_t)tc * kv_dim));
                vraw[s] = __ldcg(reinterpret_cast<const uint4 *>(vc + (size_t)tc * kv_dim));
            }
        }
    }
    if (a.pdl) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (base0 < t1) {
#pragma unroll
            for (int s = 0; s < STEPS; s++) {
                const uint32_t t = base0 + s * RPW + g, tc = t < t1 ? t : t1 - 1;
                if (tc + 1 == total) {
                    kraw[s] = __ldcg(reinterpret_cast<const uint4 *>(kc + (size_t)tc * kv_dim));
                    vraw[s] = __ldcg(reinterpret_cast<const uint4 *>(vc + (size_t)tc * kv_dim));
                }
            }
        }
    }
    float2 q2[KVM][EPL / 2];
#pragma unroll
    for (int m = 0; m < KVM; m++) {
        const float4 *qp = reinterpret_cast<const float4 *>(a.q + (size_t)(kvh * KVM + m) * HS + li * EPL);
        const float4 x = __ldcg(qp), y = __ldcg(qp + 1);
        q2[m][0] = make_float2(x.x, x.y); q2[m][1] = make_float2(x.z, x.w);
        q2[m][2] = make_float2(y.x, y.y); q2[m][3] = make_float2(y.z, y.w);
    }

    // running maximum and sum of the head this lane scores (m_own); accumulators of all four heads for the lane's 8 elements
    const int s_own = li / KVM;   // (and head li % KVM)
    float M = -INFINITY, l = 0.f;
    float2 acc[KVM][EPL / 2];
#pragma unroll
    for (int m = 0; m < KVM; m++)
#pragma unroll
        for (int j = 0; j < EPL / 2; j++) acc[m][j] = make_float2(0.f, 0.f);

    // The rows of the next iteration are requested before the current ones are used: a slice is then one cache round
    // trip plus arithmetic, however many iterations it has, and twice the bytes are in flight per warp.
    uint4 knext[STEPS], vnext[STEPS];
#pragma unroll 1
    for (uint32_t base = base0; base < t1; base += ATTN_WARPS * ROWS) {
        const uint32_t nbase = base + ATTN_WARPS * ROWS;
        if (nbase < t1) {
#pragma unroll
            for (int s = 0; s < STEPS; s++) {
                const uint32_t t = nbase + s * RPW + g, tc = t < t1 ? t : t1 - 1;
                knext[s] = __ldcg(reinterpret_cast<const uint4 *>(kc + (size_t)tc * kv_dim));
                vnext[s] = __ldcg(reinterpret_cast<const uint4 *>(vc + (size_t)tc * kv_dim));
            }
        }
        // partial scores of the lane's 8 elements: v[s * KVM + m]
        float v[L];
#pragma unroll
        for (int s = 0; s < STEPS; s++) {
            const __half2 *h = reinterpret_cast<const __half2 *>(&kraw[s]);
            float2 k2[EPL / 2];
#pragma unroll
            for (int j = 0; j < EPL / 2; j++) k2[j] = __half22float2(h[j]);
#pragma unroll
            for (int m = 0; m < KVM; m++) {
                float2 d = make_float2(0.f, 0.f);
#pragma unroll
                for (int j = 0; j < EPL / 2; j++) d = ffma2(q2[m][j], k2[j], d);
                v[s * KVM + m] = d.x + d.y;
            }
        }
        // complete sums: lane li of the row ends up with score number li = s_own * KVM + m_own
        if constexpr (L == 16) {
            halve_exchange<16>(v, lane, 8);
        }
        halve_exchange<8>(reinterpret_cast<float (&)[8]>(v), lane, 4);
        halve_exchange<4>(reinterpret_cast<float (&)[4]>(v), lane, 2);
        halve_exchange<2>(reinterpret_cast<float (&)[2]>(v), lane, 1);
        const bool valid = (base + s_own * RPW + g) < t1;
        const float sc = valid ? v[0] * scale : -INFINITY;
        // block maximum of the head over the warp's 8 rows: the lanes that share m_own differ in bits 2..4
        float bm = sc;
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 4));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 8));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 16));
        const float Mn = fmaxf(M, bm);   // finite: row `base` (step 0, group 0) is valid
        const float alpha = expf(M - Mn), pe = expf(sc - Mn);
        M = Mn;
        l = l * alpha + pe;
        __syncwarp();   // the previous iteration's reads of sm_p are done
        sm_p[warp][lane] = pe;   // index g * L + s * KVM + m
        if (lane < KVM) sm_alpha[warp][lane] = alpha;   // lanes 0..3: group 0, step 0, m_own = lane
        __syncwarp();
        const float4 al = *reinterpret_cast<const float4 *>(sm_alpha[warp]);
        const float alv[KVM] = {al.x, al.y, al.z, al.w};
#pragma unroll
        for (int m = 0; m < KVM; m++)
#pragma unroll
            for (int j = 0; j < EPL / 2; j++) { acc[m][j].x *= alv[m]; acc[m][j].y *= alv[m]; }
#pragma unroll
        for (int s = 0; s < STEPS; s++) {
            const __half2 *h = reinterpret_cast<const __half2 *>(&vraw[s]);
            const float4 p4 = *reinterpret_cast<const float4 *>(&sm_p[warp][g * L + s * KVM]);
            const float pv[KVM] = {p4.x, p4.y, p4.z, p4.w};
            float2 v2[EPL / 2];
#pragma unroll
            for (int j = 0; j < EPL / 2; j++) v2[j] = __half22float2(h[j]);
#pragma unroll
            for (int m = 0; m < KVM; m++)
#pragma unroll
                for (int j = 0; j < EPL / 2; j++) acc[m][j] = ffma2(make_float2(pv[m], pv[m]), v2[j], acc[m][j]);
        }
        if (nbase < t1) {
#pragma unroll
            for (int s = 0; s < STEPS; s++) { kraw[s] = knext[s]; vraw[s] = vnext[s]; }
        }
    }

    // fold the row groups of the warp (lanes with the same li), then the warps of the block
#pragma unroll
    for (int o = L; o < 32; o <<= 1) {
#pragma unroll
        for (int m = 0; m < KVM; m++)
#pragma unroll
            for (int j = 0; j < EPL / 2; j++) {
                acc[m][j].x += __shfl_xor_sync(0xffffffffu, acc[m][j].x, o);
                acc[m][j].y += __shfl_xor_sync(0xffffffffu, acc[m][j].y, o);
            }
    }
    l += __shfl_xor_sync(0xffffffffu, l, 4);    // the lanes that score the same head: bits 2..4
    l += __shfl_xor_sync(0xffffffffu, l, 8);
    l += __shfl_xor_sync(0xffffffffu, l, 16);
    if (g == 0) {
#pragma unroll
        for (int m = 0; m < KVM; m++)
#pragma unroll
            for (int j = 0; j < EPL / 2; j++)
                *reinterpret_cast<float2 *>(&sm_acc[(warp * KVM + m) * HS + li * EPL + 2 * j]) = acc[m][j];
    }
    if (lane < KVM) { sm_m[warp * KVM + lane] = M; sm_l[warp * KVM + lane] = l; }
    __syncthreads();

    // every thread owns PER consecutive outputs of one head; all of them are in flight together
    constexpr uint32_t slot = HS + 2;
    constexpr int PER = KVM * HS / ATTN_THREADS;   // 4 (head size 128) or 2 (64)
    static_assert(PER == 2 || PER == 4, "outputs per thread");
    const int m_out = (tid * PER) / HS, d_out = (tid * PER) % HS;
    float *part = a.scratch + ((size_t)kvh * a.max_splits + split) * KVM * slot;
    {
        float mx = sm_m[m_out];
#pragma unroll
        for (int w = 1; w < ATTN_WARPS; w++) mx = fmaxf(mx, sm_m[w * KVM + m_out]);
        float o[PER], ls = 0.f;
#pragma unroll
        for (int e = 0; e < PER; e++) o[e] = 0.f;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; w++) {
            const float wt = merge_weight(sm_m[w * KVM + m_out], mx);
            ls += wt * sm_l[w * KVM + m_out];
#pragma unroll
            for (int e = 0; e < PER; e += 2) {
                const float2 t = *reinterpret_cast<const float2 *>(&sm_acc[(w * KVM + m_out) * HS + d_out + e]);
                o[e] += wt * t.x;
                o[e + 1] += wt * t.y;
            }
        }
        if (nsplit == 1) {
            const float inv = 1.0f / ls;
#pragma unroll
            for (int e = 0; e < PER; e += 2)
                *reinterpret_cast<float2 *>(a.out + (size_t)(kvh * KVM + m_out) * HS + d_out + e) = make_float2(o[e] * inv, o[e + 1] * inv);
            return;
        }
        if (in_cluster) {
            // the partial goes into the first CTA's shared memory; after the cluster barrier that CTA merges the slices
            namespace cg = cooperative_groups;
            cg::cluster_group cluster = cg::this_cluster();
            float *dst = cluster.map_shared_rank(sm_cl, 0) + ((size_t)split * KVM + m_out) * slot;
#pragma unroll
            for (int e = 0; e < PER; e += 2) *reinterpret_cast<float2 *>(dst + d_out + e) = make_float2(o[e], o[e + 1]);
            if (d_out == 0) *reinterpret_cast<float2 *>(dst + HS) = make_float2(mx, ls);
            cluster.sync();
            if (split != 0) return;
            float cm = -INFINITY;
            for (uint32_t s = 0; s < nsplit; s++) cm = fmaxf(cm, sm_cl[(s * KVM + m_out) * slot + HS]);
            float lsum = 0.f, acc[PER];
#pragma unroll
            for (int e = 0; e < PER; e++) acc[e] = 0.f;
            for (uint32_t s = 0; s < nsplit; s++) {
                const float *ps = sm_cl + (s * KVM + m_out) * slot;
                const float wt = merge_weight(ps[HS], cm);
                lsum += wt * ps[HS + 1];
#pragma unroll
                for (int e = 0; e < PER; e++) acc[e] += wt * ps[d_out + e];
            }
            const float inv = 1.0f / lsum;
#pragma unroll
            for (int e = 0; e < PER; e += 2)
                *reinterpret_cast<float2 *>(a.out + (size_t)(kvh * KVM + m_out) * HS + d_out + e) = make_float2(acc[e] * inv, acc[e + 1] * inv);
            return;
        }
#pragma unroll
        for (int e = 0; e < PER; e += 2) *reinterpret_cast<float2 *>(part + m_out * slot + d_out + e) = make_float2(o[e], o[e + 1]);
        if (d_out == 0) *reinterpret_cast<float2 *>(part + m_out * slot + HS) = make_float2(mx, ls);
    }

    // The block's partial is published by one release/acquire arrival of thread 0: the barrier before it orders the other
    // threads' stores ahead of the release, the barrier after it orders their reads of the other blocks' partials (from
    // L2) behind the acquire.
    __syncthreads();
    if (tid == 0) {
        uint32_t old;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(a.counters + kvh) : "memory");
        sm_last = (old == nsplit - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (sm_last == 0u) return;
    // merge of the kv head's partials: every thread adds up its outputs over the slices, eight slices at a time - their
    // (max, sum) pairs and their accumulator values are requested together (one round trip to L2 per eight slices), then
    // folded into a running (max, sum, accumulator) the way the main loop folds cache rows.
    const float *mine = a.scratch + (size_t)kvh * a.max_splits * KVM * slot + (size_t)m_out * slot;
    float Mr = -INFINITY, ls = 0.f, o[PER];
#pragma unroll
    for (int e = 0; e < PER; e++) o[e] = 0.f;
#pragma unroll 1
    for (uint32_t s0 = 0; s0 < nsplit; s0 += 8) {
        float2 ml[8], dat[8][PER / 2];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t sj = min(s0 + j, nsplit - 1);
            const float *ps = mine + (size_t)sj * KVM * slot;
            ml[j] = __ldcg(reinterpret_cast<const float2 *>(ps + HS));
#pragma unroll
            for (int e = 0; e < PER / 2; e++) dat[j][e] = __ldcg(reinterpret_cast<const float2 *>(ps + d_out + 2 * e));
            if (s0 + j >= nsplit) ml[j] = make_float2(-INFINITY, 0.f);
        }
        float cm = ml[0].x;
#pragma unroll
        for (int j = 1; j < 8; j++) cm = fmaxf(cm, ml[j].x);
        const float Mn = fmaxf(Mr, cm), alpha = merge_weight(Mr, Mn);
        Mr = Mn;
        ls *= alpha;
#pragma unroll
        for (int e = 0; e < PER; e++) o[e] *= alpha;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float wt = merge_weight(ml[j].x, Mn);
            ls += wt * ml[j].y;
#pragma unroll
            for (int e = 0; e < PER / 2; e++) {
                o[2 * e] += wt * dat[j][e].x;
                o[2 * e + 1] += wt * dat[j][e].y;
            }
        }
    }
    const float inv = 1.0f / ls;
#pragma unroll
    for (int e = 0; e < PER; e += 2)
        *reinterpret_cast<float2 *>(a.out + (size_t)(kvh * KVM + m_out) * HS + d_out + e) = make_float2(o[e] * inv, o[e + 1] * inv);
    if (tid == 0) a.counters[kvh] = 0u;
}

}  // namespace ib
