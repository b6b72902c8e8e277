// Device helpers shared by the quantized GEMV kernels: the block-fixed-point activation form, dp4a wrappers and
// the per-format 64-weight "unit" dot products.
#pragma once

#include "common.cuh"

namespace ib {

constexpr int PACK_THREADS = 256;        // threads that take part in the activation prologue
constexpr uint32_t GEMV_MAX_COLS = 32768;

// Activation form in shared memory, for `cols` columns (a multiple of 32):
//   3 int8 limbs a0,a1,a2 [cols] each;  f32 scale s/127 per 32 columns;  f32 sum of x per 16 columns
//   x ~= (s/127) * (a0 + a1/254 + a2/254^2)      (resolution 6e-8 * max|x| of the 32-group)
__host__ __device__ inline size_t act_smem_bytes(uint32_t cols) { return (size_t)cols * 3 + cols / 32 * 4 + cols / 16 * 4; }

struct Act {
    const uint8_t *base;
    uint32_t cols;
    __device__ __forceinline__ const uint4 *limb(int k) const { return reinterpret_cast<const uint4 *>(base + (size_t)k * cols); }
    __device__ __forceinline__ const float *sc() const { return reinterpret_cast<const float *>(base + (size_t)3 * cols); }
    __device__ __forceinline__ const float *sx16() const { return sc() + cols / 32; }
};

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ float limb_combine(int d0, int d1, int d2) {
    return (float)d0 + (float)d1 * (1.0f / 254.0f) + (float)d2 * (1.0f / 64516.0f);
}
__device__ __forceinline__ float h2f(uint32_t bits16) { return __half2float(__ushort_as_half((unsigned short)bits16)); }

__device__ __forceinline__ void named_barrier(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }

__device__ __forceinline__ unsigned long long argmax_key(float v, uint32_t idx) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - idx);  // ties -> lowest index
}

// 6-bit (scale, min) pairs of sub-blocks 2c and 2c+1 of a Q4_K / Q5_K block header (crates/inferi/src/quantization.rs:394-402):
// returns sc_lo | sc_hi << 8 and m_lo | m_hi << 8.
__device__ __forceinline__ void kquant_scales(const uint4 &hdr, uint32_t c, uint32_t &sc2, uint32_t &m2) {
    const uint32_t sh = 16 * (c & 1);
    const uint32_t y2 = (hdr.y >> sh) & 0xFFFFu, z2 = (hdr.z >> sh) & 0xFFFFu, w2 = (hdr.w >> sh) & 0xFFFFu;
    if (c < 2) { sc2 = y2 & 0x3F3Fu; m2 = z2 & 0x3F3Fu; }
    else { sc2 = (w2 & 0x0F0Fu) | ((y2 >> 2) & 0x3030u); m2 = ((w2 >> 4) & 0x0F0Fu) | ((z2 >> 2) & 0x3030u); }
}

// -------------------------------------------------------------------------------------------------
// prologue: (optional RMSNorm) + conversion of x into the limb form in shared memory.
// Called by the first PACK_THREADS threads of the CTA; synchronises them on named barrier 1.
// Each thread owns float4 number tid + 256 i, so a 32-column group is 8 consecutive lanes.
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ void pack_float4(float4 v, uint32_t idx, uint32_t cols, uint8_t *smem, bool store) {
    const int lane = threadIdx.x & 31;
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    float sum = (v.x + v.y) + (v.z + v.w);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const float inv = amax > 0.f ? 127.0f / amax : 0.f;
    const float e[4] = {v.x, v.y, v.z, v.w};
    // round-to-nearest-even by adding 1.5 * 2^23: the sum's low mantissa byte is the rounded value in two's complement
    // (|t| <= 127), and subtracting the constant again gives it back as a float - no conversion instructions
    constexpr float MAGIC = 12582912.0f;
    uint32_t b0[4], b1[4], b2[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float t = e[k] * inv;
        const float r0 = t + MAGIC;
        const float t1 = (t - (r0 - MAGIC)) * 254.0f;
        const float r1 = t1 + MAGIC;
        const float r2 = (t1 - (r1 - MAGIC)) * 254.0f + MAGIC;
        b0[k] = __float_as_uint(r0); b1[k] = __float_as_uint(r1); b2[k] = __float_as_uint(r2);
    }
    // low bytes of four words -> one word
    const uint32_t w0 = __byte_perm(__byte_perm(b0[0], b0[1], 0x0040), __byte_perm(b0[2], b0[3], 0x0040), 0x5410);
    const uint32_t w1 = __byte_perm(__byte_perm(b1[0], b1[1], 0x0040), __byte_perm(b1[2], b1[3], 0x0040), 0x5410);
    const uint32_t w2 = __byte_perm(__byte_perm(b2[0], b2[1], 0x0040), __byte_perm(b2[2], b2[3], 0x0040), 0x5410);
    if (store) {
        uint32_t *l0 = reinterpret_cast<uint32_t *>(smem), *l1 = l0 + cols / 4, *l2 = l1 + cols / 4;
        float *sc = reinterpret_cast<float *>(smem + (size_t)3 * cols), *sx16 = sc + cols / 32;
        l0[idx] = w0; l1[idx] = w1; l2[idx] = w2;
        if ((lane & 7) == 0) sc[idx >> 3] = amax * (1.0f / 127.0f);
        if ((lane & 3) == 0) sx16[idx >> 2] = sum;
    }
}

__device__ __forceinline__ void pack_activation(uint8_t *smem, uint32_t cols, const float *__restrict__ x, const float *__restrict__ norm_w, float eps,
                                                float *red /* [PACK_THREADS/32 + 1] */) {
    constexpr int MAXV = 14;  // float4 registers per thread: covers 14336 columns without re-reading x
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t nv = cols / 4;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    const float4 *w4 = reinterpret_cast<const float4 *>(norm_w);
    const bool in_regs = nv <= (uint32_t)MAXV * PACK_THREADS;
    constexpr int MAXG = 4;   // norm weights fetched together with x (covers 4096 columns; wider rows fetch them later)
    float4 xv[MAXV], gv[MAXG];
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
            const uint32_t idx = tid + PACK_THREADS * i;
            xv[i] = idx < nv ? __ldcg(x4 + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < MAXG; i++) {
            const uint32_t idx = tid + PACK_THREADS * i;
            gv[i] = (norm_w && idx < nv) ? __ldg(w4 + idx) : make_float4(1.f, 1.f, 1.f, 1.f);
        }
    }
    float rms = 1.0f;
    if (norm_w) {
        // crates/inferi-shaders/src/rms_norm.rs:112-120
        float ss = 0.f;
        if (in_regs) {
#pragma unroll
            for (int i = 0; i < MAXV; i++) ss += (xv[i].x * xv[i].x + xv[i].y * xv[i].y) + (xv[i].z * xv[i].z + xv[i].w * xv[i].w);
        } else {
            for (uint32_t idx = tid; idx < nv; idx += PACK_THREADS) {
                const float4 v = __ldcg(x4 + idx);
                ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
            }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[warp] = ss;
        named_barrier(1, PACK_THREADS);
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < PACK_THREADS / 32; w++) t += red[w];
        rms = 1.0f / sqrtf(t / (float)cols + eps);
    }
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
            const uint32_t idx = tid + PACK_THREADS * i;
            if ((uint32_t)(warp * 32 + PACK_THREADS * i) < nv) {  // warp-uniform: the whole warp shuffles together
                float4 v = xv[i];
                const bool ok = idx < nv;
                if (norm_w && ok) {
                    const float4 g = i < MAXG ? gv[i < MAXG ? i : 0] : __ldg(w4 + idx);
                    v.x = (v.x * rms) * g.x; v.y = (v.y * rms) * g.y; v.z = (v.z * rms) * g.z; v.w = (v.w * rms) * g.w;
                }
                pack_float4(v, idx, cols, smem, ok);
            }
        }
    } else {
        for (uint32_t base = warp * 32; base < nv; base += PACK_THREADS) {
            const uint32_t idx = base + lane;
            const bool ok = idx < nv;
            float4 v = ok ? __ldcg(x4 + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (norm_w && ok) {
                const float4 g = __ldg(w4 + idx);
                v.x = (v.x * rms) * g.x; v.y = (v.y * rms) * g.y; v.z = (v.z * rms) * g.z; v.w = (v.w * rms) * g.w;
            }
            pack_float4(v, idx, cols, smem, ok);
        }
    }
    named_barrier(1, PACK_THREADS);
}

}  // namespace ib
