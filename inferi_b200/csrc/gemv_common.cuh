// Device helpers shared by the quantized GEMV kernels: the block-fixed-point activation form, dp4a wrappers and
// the per-format 64-weight "unit" dot products.
#pragma once

#include "common.cuh"

namespace ib {

constexpr int PACK_THREADS = 512;        // threads that take part in the activation prologue of the streaming kernel
constexpr uint32_t GEMV_MAX_COLS = 32768;

// Activation form in shared memory, for `cols` columns (a multiple of 32):
//   ACT_LIMBS int8 limbs a0, a1 [cols] each;  f32 scale s/127 per 32 columns;  f32 sum of the quantized x per 16 columns
//   x ~= (s/127) * (a0 + a1/254)      (resolution 1.6e-5 * max|x| of the 32-group: 16-bit block fixed point)
//   (+ 192 bytes: in the group-major chunk order each limb array carries one 16-byte skew per group, see act_chunk_pos)
// The 16-column sums (used for the k-quants' minimums and the Q6_K -32 terms) are sums of the QUANTIZED values, so that
// sum_k w_k a_k is evaluated exactly for the a_k the dot products see; the only error of a GEMV is sum_k w_k (a_k - x_k),
// 2e-5 .. 1e-4 relative.  (A third limb - 24-bit fixed point - costs a third more dp4a and 16 more registers per lane: 583
// against 619 tok/s on the 8B architecture; the logits of the 1B architecture then differ from the f32 oracle's by 7e-4
// instead of 2.7e-3 max-abs, at a tolerance of 2e-2.)
constexpr int ACT_LIMBS = 2;
__host__ __device__ inline size_t act_smem_bytes(uint32_t cols) { return (size_t)cols * ACT_LIMBS + cols / 32 * 4 + cols / 16 * 4 + 192; }

struct Act {
    const uint8_t *base;
    uint32_t cols;
    uint32_t nq = 0;   // 0: 16-column chunks in column order; else cols / 64: group-major order, see act_chunk_pos
    __device__ __forceinline__ uint32_t pos(uint32_t e16) const { return nq ? (e16 & 3u) * (nq + 1) + (e16 >> 2) : e16; }
    __device__ __forceinline__ uint32_t lstride() const { return cols + (nq ? 64u : 0u); }
    __device__ __forceinline__ const uint4 *limb(int k) const { return reinterpret_cast<const uint4 *>(base + (size_t)k * lstride()); }
    __device__ __forceinline__ const float *sc() const { return reinterpret_cast<const float *>(base + (size_t)ACT_LIMBS * lstride()); }
    __device__ __forceinline__ const float *sx16() const { return sc() + cols / 32; }
};

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// the integer dot products of the limbs -> the dot product in units of the group's scale; d[0 .. ACT_LIMBS-1]
__device__ __forceinline__ float limb_combine(const int *d) {
    float v = (float)d[0] + (float)d[1] * (1.0f / 254.0f);
    if (ACT_LIMBS > 2) v += (float)d[ACT_LIMBS - 1] * (1.0f / 64516.0f);
    return v;
}
__device__ __forceinline__ float h2f(uint32_t bits16) { return __half2float(__ushort_as_half((unsigned short)bits16)); }

__device__ __forceinline__ void named_barrier(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }

__device__ __forceinline__ unsigned long long argmax_key(float v, uint32_t idx) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - idx);  // ties -> lowest index
}

// -------------------------------------------------------------------------------------------------
// prologue: (optional RMSNorm) + conversion of x into the limb form in shared memory.
// Called by the first PACK_THREADS threads of the CTA; synchronises them on named barrier 1.
// A thread owns runs of 16 consecutive columns (run number tid + 256 i): the 16-column sum needs no shuffle, the
// 32-column maximum one shuffle with the neighbour lane, and the 16 conversions are independent of each other.
// -------------------------------------------------------------------------------------------------
constexpr int PACK_RUNS = 2;   // runs of 16 columns kept in registers per thread (covers 16384 columns with 512 threads)

struct PackRegs {
    float4 x[PACK_RUNS][4];
};

// Issues the loads of this thread's norm weights.  They are weights, so a kernel may call this before it waits for
// its predecessor.
__device__ __forceinline__ void pack_prefetch_norm(const float *__restrict__ norm_w, uint32_t cols, float4 (&g)[4]) {
    const uint32_t run = threadIdx.x;   // only the first run's weights are kept (cols <= 4096); wider rows re-fetch
    if (norm_w && run < cols / 16) {
        const float4 *w4 = reinterpret_cast<const float4 *>(norm_w) + 4 * run;
#pragma unroll
        for (int j = 0; j < 4; j++) g[j] = __ldg(w4 + j);
    } else {
#pragma unroll
        for (int j = 0; j < 4; j++) g[j] = make_float4(1.f, 1.f, 1.f, 1.f);
    }
}

// Position of the 16-column chunk `run` inside a limb array.  With nq = cols / 64 the chunks are stored "group-major":
// chunk 4u + g sits at g * (nq + 1) + u.  The lanes of a warp, each reading chunk 4u + g of its unit u, then touch
// consecutive 16-byte words (in column order they would be 64 bytes apart: a 4-way bank conflict on every 128-bit load),
// and the one-chunk skew between groups keeps the four chunks that neighbouring threads store apart as well.
__device__ __forceinline__ uint32_t act_chunk_pos(uint32_t run, uint32_t nq) { return nq ? (run & 3u) * (nq + 1) + (run >> 2) : run; }

__device__ __forceinline__ void pack_run(const float4 (&v)[4], uint32_t run, uint32_t cols, uint8_t *smem, bool store, uint32_t nq = 0) {
    const int lane = threadIdx.x & 31;
    float amax = 0.f, sum = 0.f;   // sum: of the quantized values, in units of the group's scale
#pragma unroll
    for (int j = 0; j < 4; j++) amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));   // the other half of the 32-column group
    const float inv = amax > 0.f ? __fdividef(127.0f, amax) : 0.f;   // 2 ulp: the limbs absorb it (|t| stays within 127 + 1e-5)
    // round-to-nearest-even by adding 1.5 * 2^23: the sum's low mantissa byte is the rounded value in two's complement
    // (|t| <= 127), and subtracting the constant again gives it back as a float - no conversion instructions
    constexpr float MAGIC = 12582912.0f;
    uint32_t w0[4], w1[4], w2[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float e[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
        uint32_t b0[4], b1[4], b2[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float t = e[k] * inv;
            const float r0 = t + MAGIC, q0 = r0 - MAGIC;            // the limbs as floats: q0, q1, q2
            const float t1 = (t - q0) * 254.0f;
            const float r1 = t1 + MAGIC, q1 = r1 - MAGIC;
            const float t2 = (t1 - q1) * 254.0f;
            const float r2 = t2 + MAGIC;
            b0[k] = __float_as_uint(r0); b1[k] = __float_as_uint(r1); b2[k] = __float_as_uint(r2);
            sum += q0 + q1 * (1.0f / 254.0f) + (ACT_LIMBS > 2 ? (r2 - MAGIC) * (1.0f / 64516.0f) : 0.f);
        }
        // low bytes of four words -> one word
        w0[j] = __byte_perm(__byte_perm(b0[0], b0[1], 0x0040), __byte_perm(b0[2], b0[3], 0x0040), 0x5410);
        w1[j] = __byte_perm(__byte_perm(b1[0], b1[1], 0x0040), __byte_perm(b1[2], b1[3], 0x0040), 0x5410);
        w2[j] = __byte_perm(__byte_perm(b2[0], b2[1], 0x0040), __byte_perm(b2[2], b2[3], 0x0040), 0x5410);
    }
    if (store) {
        const size_t ls = cols + (nq ? 64u : 0u);   // = Act::lstride()
        uint4 *l0 = reinterpret_cast<uint4 *>(smem), *l1 = reinterpret_cast<uint4 *>(smem + ls), *l2 = reinterpret_cast<uint4 *>(smem + 2 * ls);
        float *sc = reinterpret_cast<float *>(smem + ACT_LIMBS * ls), *sx16 = sc + cols / 32;
        const uint32_t at = act_chunk_pos(run, nq);
        l0[at] = make_uint4(w0[0], w0[1], w0[2], w0[3]);
        l1[at] = make_uint4(w1[0], w1[1], w1[2], w1[3]);
        if (ACT_LIMBS > 2) l2[at] = make_uint4(w2[0], w2[1], w2[2], w2[3]);
        if ((lane & 1) == 0) sc[run >> 1] = amax * (1.0f / 127.0f);
        sx16[run] = sum * (amax * (1.0f / 127.0f));
    }
}

// Tensor-parallel input: x + the partial sums every rank left in this rank's slots (fixed rank order, so every rank gets
// the same bits); CTA 0 also stores the result as the new residual stream.  Only for rows that fit the registers.
struct PackReduce {
    const float *src;   // [tp][cols], null = plain x
    uint32_t tp;
    float *x_out;       // may be null
};

// `g` holds the norm weights of the thread's first run (from pack_prefetch_norm).
template <int NT = PACK_THREADS>
__device__ __forceinline__ void pack_activation(uint8_t *smem, uint32_t cols, const float *__restrict__ x, const float *__restrict__ norm_w, float eps,
                                                float *red /* [NT/32 + 1] */, const float4 (&g)[4], const PackReduce rd = PackReduce{nullptr, 0, nullptr},
                                                uint32_t nq = 0) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t nruns = cols / 16;    // cols is a multiple of 32, so runs pair up inside a warp
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    const float4 *w4 = reinterpret_cast<const float4 *>(norm_w);
    PackRegs r;
#pragma unroll
    for (int i = 0; i < PACK_RUNS; i++) {
        const uint32_t run = tid + NT * i;
#pragma unroll
        for (int j = 0; j < 4; j++) r.x[i][j] = run < nruns ? __ldcg(x4 + 4 * run + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (rd.src) {
#pragma unroll
        for (int i = 0; i < PACK_RUNS; i++) {
            const uint32_t run = tid + NT * i;
            if (run < nruns) {
                for (uint32_t rk = 0; rk < rd.tp; rk++) {
                    const float4 *s4 = reinterpret_cast<const float4 *>(rd.src + (size_t)rk * cols) + 4 * run;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float4 a = __ldcg(s4 + j);
                        r.x[i][j].x += a.x; r.x[i][j].y += a.y; r.x[i][j].z += a.z; r.x[i][j].w += a.w;
                    }
                }
                if (rd.x_out && blockIdx.x == 0) {
#pragma unroll
                    for (int j = 0; j < 4; j++) reinterpret_cast<float4 *>(rd.x_out)[4 * run + j] = r.x[i][j];
                }
            }
        }
    }
    float rms = 1.0f;
    if (norm_w) {
        // crates/inferi-shaders/src/rms_norm.rs:112-120
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < PACK_RUNS; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) ss += (r.x[i][j].x * r.x[i][j].x + r.x[i][j].y * r.x[i][j].y) + (r.x[i][j].z * r.x[i][j].z + r.x[i][j].w * r.x[i][j].w);
        for (uint32_t run = tid + NT * PACK_RUNS; run < nruns; run += NT)   // rows wider than the registers hold
            for (int j = 0; j < 4; j++) {
                const float4 v = __ldcg(x4 + 4 * run + j);
                ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
            }
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[warp] = ss;
        named_barrier(1, NT);
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < NT / 32; w++) t += red[w];
        rms = 1.0f / sqrtf(t / (float)cols + eps);
    }
#pragma unroll
    for (int i = 0; i < PACK_RUNS; i++) {
        const uint32_t run = tid + NT * i;
        if ((uint32_t)(warp * 32 + NT * i) < nruns) {   // warp-uniform: both lanes of a 32-column group are present
            const bool ok = run < nruns;
            if (norm_w && ok) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float4 w = (i == 0) ? g[j] : __ldg(w4 + 4 * run + j);
                    float4 &v = r.x[i][j];
                    v.x = (v.x * rms) * w.x; v.y = (v.y * rms) * w.y; v.z = (v.z * rms) * w.z; v.w = (v.w * rms) * w.w;
                }
            }
            pack_run(r.x[i], run, cols, smem, ok, nq);
        }
    }
    for (uint32_t base = warp * 32 + NT * PACK_RUNS; base < nruns; base += NT) {   // rows wider than the registers hold
        const uint32_t run = base + lane;
        const bool ok = run < nruns;
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            v[j] = ok ? __ldcg(x4 + 4 * run + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (norm_w && ok) {
                const float4 w = __ldg(w4 + 4 * run + j);
                v[j].x = (v[j].x * rms) * w.x; v[j].y = (v[j].y * rms) * w.y; v[j].z = (v[j].z * rms) * w.z; v[j].w = (v[j].w * rms) * w.w;
            }
        }
        pack_run(v, run, cols, smem, ok, nq);
    }
    named_barrier(1, NT);
}

}  // namespace ib
