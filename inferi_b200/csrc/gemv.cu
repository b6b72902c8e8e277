// Quantized GEMV, second-line kernels and host dispatch.
//
// The token loop runs on the streaming kernel (gemv_stream.cu).  This file holds
//  * gemv_wide_kernel: direct 128-bit global loads, one warp per row pair, activations in shared memory; used for
//    matrices too wide for the streaming kernel's register-resident activations (16384 < cols <= 32768);
//  * gemv_generic_kernel: any shape the contracts allow, straight from the GGUF byte stream with scalar loads; used
//    where the alignment rules of the 128-bit kernels fail (for instance Q6_K with cols % 2048 != 0);
//  * the upload-time re-tiling of Q8_0 / Q6_K rows into groups of 8 blocks, and the launch dispatch.
// All of them replace crates/inferi-shaders/src/gemv_quant_*.rs behind crates/inferi/src/ops/gemv_quant.rs:183-341.
#include "gemv_common.cuh"

namespace ib {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;

// streaming 128-bit weight load: read-only path, no L1 allocation (every weight byte is used exactly once)
__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_u16(const void *p) {
    uint16_t v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// -------------------------------------------------------------------------------------------------
// per-format dot products of NR rows with the packed activation; each lane returns partial sums
// -------------------------------------------------------------------------------------------------
template <int NR>
__device__ __forceinline__ void dot_q4k(const uint8_t *const (&row)[NR], uint32_t nb, const Act &A, int lane, float (&acc)[NR]) {
    const float *SC = A.sc(), *SX = A.sx16();
    for (uint32_t u = lane; u < 4 * nb; u += 32) {
        const uint32_t b = u >> 2, c = u & 3;
        uint4 hdr[NR], q0[NR], q1[NR];
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const uint8_t *blk = row[r] + (size_t)b * 144;
            hdr[r] = ldg_stream(blk);
            q0[r] = ldg_stream(blk + 16 + 32 * c);
            q1[r] = ldg_stream(blk + 32 + 32 * c);
        }
        const uint32_t e16 = 16 * b + 4 * c;  // index of the unit's first 16-element group
        int D[NR][2][3];
#pragma unroll
        for (int k = 0; k < ACT_LIMBS; k++) {
            const uint4 *L = A.limb(k) + e16;
            const uint4 aL0 = L[0], aL1 = L[1], aH0 = L[2], aH1 = L[3];
#pragma unroll
            for (int r = 0; r < NR; r++) {
                int lo = 0, hi = 0;
                lo = dp4a_ss(q0[r].x & 0x0F0F0F0Fu, aL0.x, lo); hi = dp4a_us(q0[r].x & 0xF0F0F0F0u, aH0.x, hi);
                lo = dp4a_ss(q0[r].y & 0x0F0F0F0Fu, aL0.y, lo); hi = dp4a_us(q0[r].y & 0xF0F0F0F0u, aH0.y, hi);
                lo = dp4a_ss(q0[r].z & 0x0F0F0F0Fu, aL0.z, lo); hi = dp4a_us(q0[r].z & 0xF0F0F0F0u, aH0.z, hi);
                lo = dp4a_ss(q0[r].w & 0x0F0F0F0Fu, aL0.w, lo); hi = dp4a_us(q0[r].w & 0xF0F0F0F0u, aH0.w, hi);
                lo = dp4a_ss(q1[r].x & 0x0F0F0F0Fu, aL1.x, lo); hi = dp4a_us(q1[r].x & 0xF0F0F0F0u, aH1.x, hi);
                lo = dp4a_ss(q1[r].y & 0x0F0F0F0Fu, aL1.y, lo); hi = dp4a_us(q1[r].y & 0xF0F0F0F0u, aH1.y, hi);
                lo = dp4a_ss(q1[r].z & 0x0F0F0F0Fu, aL1.z, lo); hi = dp4a_us(q1[r].z & 0xF0F0F0F0u, aH1.z, hi);
                lo = dp4a_ss(q1[r].w & 0x0F0F0F0Fu, aL1.w, lo); hi = dp4a_us(q1[r].w & 0xF0F0F0F0u, aH1.w, hi);
                D[r][0][k] = lo;
                D[r][1][k] = hi;
            }
        }
        const uint32_t j = 8 * b + 2 * c;  // first 32-element sub-block of the unit
        const float s_lo = SC[j], s_hi = SC[j + 1] * (1.0f / 16.0f);
        const float x_lo = SX[2 * j] + SX[2 * j + 1], x_hi = SX[2 * j + 2] + SX[2 * j + 3];
        const uint32_t sh = 16 * (c & 1);
#pragma unroll
        for (int r = 0; r < NR; r++) {
            // 6-bit (scale, min) pairs of sub-blocks 2c and 2c+1: crates/inferi/src/quantization.rs:394-402
            const uint32_t y2 = (hdr[r].y >> sh) & 0xFFFFu, z2 = (hdr[r].z >> sh) & 0xFFFFu, w2 = (hdr[r].w >> sh) & 0xFFFFu;
            uint32_t sc2, m2;
            if (c < 2) { sc2 = y2 & 0x3F3Fu; m2 = z2 & 0x3F3Fu; }
            else { sc2 = (w2 & 0x0F0Fu) | ((y2 >> 2) & 0x3030u); m2 = ((w2 >> 4) & 0x0F0Fu) | ((z2 >> 2) & 0x3030u); }
            const float d = h2f(hdr[r].x & 0xFFFFu), dmin = h2f(hdr[r].x >> 16);
            const float d_lo = d * (float)(sc2 & 0xFFu), d_hi = d * (float)(sc2 >> 8);
            const float m_lo = dmin * (float)(m2 & 0xFFu), m_hi = dmin * (float)(m2 >> 8);
            float v = d_lo * (s_lo * limb_combine(D[r][0])) - m_lo * x_lo;
            v += d_hi * (s_hi * limb_combine(D[r][1])) - m_hi * x_hi;
            acc[r] += v;
        }
    }
}

template <int NR>
__device__ __forceinline__ void dot_q5k(const uint8_t *const (&row)[NR], uint32_t nb, const Act &A, int lane, float (&acc)[NR]) {
    const float *SC = A.sc(), *SX = A.sx16();
    for (uint32_t u = lane; u < 4 * nb; u += 32) {
        const uint32_t b = u >> 2, c = u & 3;
        const uint32_t e16 = 16 * b + 4 * c;
        const uint32_t j = 8 * b + 2 * c;
        const float s_lo = SC[j], s_hi = SC[j + 1];
        const float x_lo = SX[2 * j] + SX[2 * j + 1], x_hi = SX[2 * j + 2] + SX[2 * j + 3];
        const uint32_t sh = 16 * (c & 1);
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const uint8_t *blk = row[r] + (size_t)b * 176;
            const uint4 hdr = ldg_stream(blk);
            const uint4 hA = ldg_stream(blk + 16), hB = ldg_stream(blk + 32);
            const uint4 q0 = ldg_stream(blk + 48 + 32 * c), q1 = ldg_stream(blk + 64 + 32 * c);
            const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            const uint32_t hw[8] = {hA.x, hA.y, hA.z, hA.w, hB.x, hB.y, hB.z, hB.w};
            uint32_t lo[8], hi[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t t = hw[i] >> (2 * c);  // bit 0 of each byte: low-half flag, bit 1: high-half flag
                lo[i] = (qw[i] & 0x0F0F0F0Fu) | ((t << 4) & 0x10101010u);
                hi[i] = ((qw[i] >> 4) & 0x0F0F0F0Fu) | ((t << 3) & 0x10101010u);
            }
            int D[2][3];
#pragma unroll
            for (int k = 0; k < ACT_LIMBS; k++) {
                const uint4 *L = A.limb(k) + e16;
                const uint4 aL0 = L[0], aL1 = L[1], aH0 = L[2], aH1 = L[3];
                const uint32_t al[8] = {aL0.x, aL0.y, aL0.z, aL0.w, aL1.x, aL1.y, aL1.z, aL1.w};
                const uint32_t ah[8] = {aH0.x, aH0.y, aH0.z, aH0.w, aH1.x, aH1.y, aH1.z, aH1.w};
                int dl = 0, dh = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) { dl = dp4a_ss(lo[i], al[i], dl); dh = dp4a_ss(hi[i], ah[i], dh); }
                D[0][k] = dl;
                D[1][k] = dh;
            }
            const uint32_t y2 = (hdr.y >> sh) & 0xFFFFu, z2 = (hdr.z >> sh) & 0xFFFFu, w2 = (hdr.w >> sh) & 0xFFFFu;
            uint32_t sc2, m2;
            if (c < 2) { sc2 = y2 & 0x3F3Fu; m2 = z2 & 0x3F3Fu; }
            else { sc2 = (w2 & 0x0F0Fu) | ((y2 >> 2) & 0x3030u); m2 = ((w2 >> 4) & 0x0F0Fu) | ((z2 >> 2) & 0x3030u); }
            const float d = h2f(hdr.x & 0xFFFFu), dmin = h2f(hdr.x >> 16);
            const float d_lo = d * (float)(sc2 & 0xFFu), d_hi = d * (float)(sc2 >> 8);
            const float m_lo = dmin * (float)(m2 & 0xFFu), m_hi = dmin * (float)(m2 >> 8);
            float v = d_lo * (s_lo * limb_combine(D[0])) - m_lo * x_lo;
            v += d_hi * (s_hi * limb_combine(D[1])) - m_hi * x_hi;
            acc[r] += v;
        }
    }
}

// Q6_K rows are stored as groups of 8 blocks: [8 x 128 ql][8 x 64 qh][8 x 16 scales][8 x 2 d] = 1680 bytes per 2048 columns.
// A unit is (block b, 128-half i, 16-byte half h): 64 weights = 4 groups g of 16 elements at 256b + 128i + 32g + 16h, each
// with its own int8 scale [8i + 2g + h].
template <int NR>
__device__ __forceinline__ void dot_q6k(const uint8_t *const (&row)[NR], uint32_t nb, const Act &A, int lane, float (&acc)[NR]) {
    const float *SC = A.sc(), *SX = A.sx16();
    for (uint32_t u = lane; u < 4 * nb; u += 32) {
        const uint32_t b = u >> 2, i = (u >> 1) & 1, h = u & 1, bb = b & 7;
        uint4 qa[NR], qb[NR], qh[NR], scw[NR];
        uint32_t dbits[NR];
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const uint8_t *p = row[r] + (size_t)(b >> 3) * 1680;
            qa[r] = ldg_stream(p + 128 * bb + 64 * i + 16 * h);
            qb[r] = ldg_stream(p + 128 * bb + 64 * i + 32 + 16 * h);
            qh[r] = ldg_stream(p + 1024 + 64 * bb + 32 * i + 16 * h);
            scw[r] = ldg_stream(p + 1536 + 16 * bb);
            dbits[r] = ldg_u16(p + 1664 + 2 * bb);
        }
        const uint32_t e16 = 16 * b + 8 * i + h;  // 16-element group index of g = 0; group g is at e16 + 2g
        const uint32_t j0 = 8 * b + 4 * i;        // 32-element sub-block of g = 0
        int D[NR][4][3];
#pragma unroll
        for (int k = 0; k < ACT_LIMBS; k++) {
            const uint4 *L = A.limb(k) + e16;
            const uint4 a0 = L[0], a1 = L[2], a2 = L[4], a3 = L[6];
#pragma unroll
            for (int r = 0; r < NR; r++) {
                const uint32_t la[4] = {qa[r].x, qa[r].y, qa[r].z, qa[r].w};
                const uint32_t lb[4] = {qb[r].x, qb[r].y, qb[r].z, qb[r].w};
                const uint32_t hh[4] = {qh[r].x, qh[r].y, qh[r].z, qh[r].w};
                const uint32_t x0[4] = {a0.x, a0.y, a0.z, a0.w}, x1[4] = {a1.x, a1.y, a1.z, a1.w};
                const uint32_t x2[4] = {a2.x, a2.y, a2.z, a2.w}, x3[4] = {a3.x, a3.y, a3.z, a3.w};
                int d0 = 0, d1 = 0, d2 = 0, d3 = 0;
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    // crates/inferi/src/quantization.rs:237-246: 4 low bits from ql, 2 high bits from qh
                    const uint32_t g0 = (la[w] & 0x0F0F0F0Fu) | ((hh[w] << 4) & 0x30303030u);
                    const uint32_t g1 = (lb[w] & 0x0F0F0F0Fu) | ((hh[w] << 2) & 0x30303030u);
                    const uint32_t g2 = ((la[w] >> 4) & 0x0F0F0F0Fu) | (hh[w] & 0x30303030u);
                    const uint32_t g3 = ((lb[w] >> 4) & 0x0F0F0F0Fu) | ((hh[w] >> 2) & 0x30303030u);
                    d0 = dp4a_ss(g0, x0[w], d0);
                    d1 = dp4a_ss(g1, x1[w], d1);
                    d2 = dp4a_ss(g2, x2[w], d2);
                    d3 = dp4a_ss(g3, x3[w], d3);
                }
                D[r][0][k] = d0; D[r][1][k] = d1; D[r][2][k] = d2; D[r][3][k] = d3;
            }
        }
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const float d = h2f(dbits[r]);
            const uint32_t w01 = i ? scw[r].z : scw[r].x;  // scales[8i + 0..3]
            const uint32_t w23 = i ? scw[r].w : scw[r].y;  // scales[8i + 4..7]
            float v = 0.f;
#pragma unroll
            for (int g = 0; g < 4; g++) {
                const uint32_t word = (g < 2) ? w01 : w23;
                const int sc = (int)(int8_t)(word >> (8 * (2 * (g & 1) + h)));
                const float dot = SC[j0 + g] * limb_combine(D[r][g]) - 32.0f * SX[e16 + 2 * g];
                v += (d * (float)sc) * dot;
            }
            acc[r] += v;
        }
    }
}

// Q8_0 rows are stored as groups of 8 blocks: [8 x 32 quants][8 x 2 scale] = 272 bytes per 256 columns; a unit is one block.
template <int NR>
__device__ __forceinline__ void dot_q80(const uint8_t *const (&row)[NR], uint32_t nb, const Act &A, int lane, float (&acc)[NR]) {
    const float *SC = A.sc();
    for (uint32_t b = lane; b < nb; b += 32) {
        uint4 q0[NR], q1[NR];
        uint32_t dbits[NR];
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const uint8_t *p = row[r] + (size_t)(b >> 3) * 272;
            q0[r] = ldg_stream(p + 32 * (b & 7));
            q1[r] = ldg_stream(p + 32 * (b & 7) + 16);
            dbits[r] = ldg_u16(p + 256 + 2 * (b & 7));
        }
        int D[NR][3];
#pragma unroll
        for (int k = 0; k < ACT_LIMBS; k++) {
            const uint4 *L = A.limb(k) + 2 * b;
            const uint4 a0 = L[0], a1 = L[1];
#pragma unroll
            for (int r = 0; r < NR; r++) {
                int d = 0;
                d = dp4a_ss(q0[r].x, a0.x, d); d = dp4a_ss(q0[r].y, a0.y, d); d = dp4a_ss(q0[r].z, a0.z, d); d = dp4a_ss(q0[r].w, a0.w, d);
                d = dp4a_ss(q1[r].x, a1.x, d); d = dp4a_ss(q1[r].y, a1.y, d); d = dp4a_ss(q1[r].z, a1.z, d); d = dp4a_ss(q1[r].w, a1.w, d);
                D[r][k] = d;
            }
        }
        const float s = SC[b];
#pragma unroll
        for (int r = 0; r < NR; r++) acc[r] += h2f(dbits[r]) * (s * limb_combine(D[r]));
    }
}

template <int NR>
__device__ __forceinline__ void dot_rows(uint32_t qtype, const uint8_t *const (&row)[NR], uint32_t nb, const Act &A, int lane, float (&acc)[NR]) {
    switch (qtype) {
    case IB_Q4_K: dot_q4k<NR>(row, nb, A, lane, acc); break;
    case IB_Q6_K: dot_q6k<NR>(row, nb, A, lane, acc); break;
    case IB_Q5_K: dot_q5k<NR>(row, nb, A, lane, acc); break;
    case IB_Q8_0: dot_q80<NR>(row, nb, A, lane, acc); break;
    default: break;
    }
}

// -------------------------------------------------------------------------------------------------
// the wide kernel: one warp per pair of rows, CTA-strided, activations in shared memory
// -------------------------------------------------------------------------------------------------
template <uint32_t EPI>
__global__ void __launch_bounds__(GEMV_THREADS, 2) gemv_wide_kernel(const GemvParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ float red[GEMV_WARPS + 1];
    __shared__ unsigned long long best_sm[GEMV_WARPS];
    __shared__ bool is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    if (p.pdl) {
        asm volatile("griddepcontrol.launch_dependents;");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    float4 norm_g[4];
    pack_prefetch_norm(p.norm_w, p.cols, norm_g);
    pack_activation<GEMV_THREADS>(smem, p.cols, p.x, p.norm_w, p.eps, red, norm_g);
    const Act A{smem, p.cols};

    uint32_t pairs[3], total = 0;
#pragma unroll
    for (int s = 0; s < 3; s++) {
        pairs[s] = (s < (int)p.nseg) ? ((EPI == EPI_SWIGLU) ? (s == 0 ? p.seg[0].rows : 0u) : p.seg[s].rows / 2) : 0u;
        total += pairs[s];
    }
    unsigned long long best = 0ull;

    for (uint32_t pr = blockIdx.x * GEMV_WARPS + warp; pr < total; pr += gridDim.x * GEMV_WARPS) {
        uint32_t s = 0, local = pr;
        if (EPI != EPI_SWIGLU) {
            if (local >= pairs[0]) { local -= pairs[0]; s = 1; if (local >= pairs[1]) { local -= pairs[1]; s = 2; } }
        }
        const uint8_t *row[2];
        uint32_t r0, qtype, nb;
        if (EPI == EPI_SWIGLU) {
            r0 = local;
            row[0] = p.seg[0].w + (size_t)r0 * p.seg[0].row_bytes;
            row[1] = p.seg[1].w + (size_t)r0 * p.seg[1].row_bytes;
            qtype = p.seg[0].qtype; nb = p.seg[0].nb;
        } else {
            r0 = 2 * local;
            row[0] = p.seg[s].w + (size_t)r0 * p.seg[s].row_bytes;
            row[1] = row[0] + p.seg[s].row_bytes;
            qtype = p.seg[s].qtype; nb = p.seg[s].nb;
        }
        float acc[2] = {0.f, 0.f};
        dot_rows<2>(qtype, row, nb, A, lane, acc);
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], o);
            acc[1] += __shfl_xor_sync(0xffffffffu, acc[1], o);
        }
        if (lane == 0) {
            if (EPI == EPI_STORE) {
                p.seg[s].out[r0] = acc[0];
                p.seg[s].out[r0 + 1] = acc[1];
            } else if (EPI == EPI_RESIDUAL) {
                p.seg[s].out[r0] = __ldcg(p.resid + r0) + acc[0];
                p.seg[s].out[r0 + 1] = __ldcg(p.resid + r0 + 1) + acc[1];
            } else if (EPI == EPI_SWIGLU) {
                // crates/inferi-shaders/src/silu.rs:16-19,46-52
                const float g = acc[0], up = acc[1];
                p.seg[0].out[r0] = up * (g / (1.0f + expf(-g)));
            } else if (EPI == EPI_QKV) {
                const uint32_t pos = *p.pos_ptr;
                float a = acc[0], bb = acc[1];
                if (p.bias[s]) {   // transformer.rs:434-442
                    a += p.bias[s][r0];
                    bb += p.bias[s][r0 + 1];
                }
                if (s < 2) {
                    // crates/inferi-shaders/src/rope.rs:75-91 (adjacent pairs)
                    const float2 cs = p.rope_cs[(r0 % p.head_size) >> 1];
                    const float x = a, y = bb;
                    a = cs.x * x - cs.y * y;
                    bb = cs.y * x + cs.x * y;
                }
                if (s == 0) {
                    p.seg[0].out[r0] = a;
                    p.seg[0].out[r0 + 1] = bb;
                } else {
                    void *cache = (s == 1) ? p.k_cache : p.v_cache;
                    const size_t off = (size_t)pos * p.kv_dim + r0;
                    if (p.kv_dtype == IB_KV_F16) {
                        reinterpret_cast<__half2 *>(cache)[off >> 1] = __floats2half2_rn(a, bb);
                    } else {
                        reinterpret_cast<float2 *>(cache)[off >> 1] = make_float2(a, bb);
                    }
                }
            } else if (EPI == EPI_ARGMAX) {
                if (p.seg[0].out) {
                    p.seg[0].out[r0] = acc[0];
                    p.seg[0].out[r0 + 1] = acc[1];
                }
                const unsigned long long k0 = argmax_key(acc[0], p.row_offset + r0), k1 = argmax_key(acc[1], p.row_offset + r0 + 1);
                best = max(best, max(k0, k1));
            }
        }
    }

    if (EPI == EPI_ARGMAX) {
        if (lane == 0) best_sm[warp] = best;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long b = 0ull;
            for (int w = 0; w < GEMV_WARPS; w++) b = max(b, best_sm[w]);
            p.argmax_slots[blockIdx.x] = b;
            __threadfence();
            const unsigned int prev = atomicAdd(p.argmax_counter, 1u);
            is_last = (prev == gridDim.x - 1);
        }
        __syncthreads();
        if (is_last) {
            // the last CTA to arrive folds every CTA's candidate; no CTA ever waits on another
            __threadfence();
            unsigned long long b = 0ull;
            for (uint32_t i = threadIdx.x; i < gridDim.x; i += GEMV_THREADS) b = max(b, __ldcg(p.argmax_slots + i));
#pragma unroll
            for (int o = 16; o; o >>= 1) b = max(b, __shfl_xor_sync(0xffffffffu, b, o));
            if (lane == 0) best_sm[warp] = b;
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int w = 0; w < GEMV_WARPS; w++) b = max(b, best_sm[w]);
                *p.argmax_out = 0xFFFFFFFFu - (uint32_t)(b & 0xFFFFFFFFull);
                *p.argmax_counter = 0u;
            }
        }
    }
}

// -------------------------------------------------------------------------------------------------
// generic fallback: any shape the contracts allow, straight from the GGUF byte stream with scalar loads.
// One warp per row, one block per lane step.  Used only where the 128-bit kernels' alignment rules fail.
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ float ld_h(const uint8_t *p) { return h2f((uint32_t)p[0] | ((uint32_t)p[1] << 8)); }

__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *q, uint32_t &d, uint32_t &m) {
    if (j < 4) { d = q[j] & 63; m = q[j + 4] & 63; }
    else { d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

__device__ float generic_block_dot(int qtype, const uint8_t *b, const float *__restrict__ v) {
    float acc = 0.f;
    if (qtype == IB_Q8_0) {
        const float s = ld_h(b);
        for (int i = 0; i < 32; i++) acc += ((float)(int8_t)b[2 + i] * s) * v[i];
    } else if (qtype == IB_Q4_K || qtype == IB_Q5_K) {
        const float d = ld_h(b), mn = ld_h(b + 2);
        const uint8_t *scales = b + 4, *qh = b + 16, *qs = b + (qtype == IB_Q4_K ? 16 : 48);
        for (int c = 0; c < 4; c++) {
            uint32_t sc, m;
            scale_min_k4(2 * c, scales, sc, m);
            const float d1 = d * (float)sc, m1 = mn * (float)m;
            scale_min_k4(2 * c + 1, scales, sc, m);
            const float d2 = d * (float)sc, m2 = mn * (float)m;
            for (int l = 0; l < 32; l++) {
                uint32_t lo = qs[32 * c + l] & 0xF, hi = qs[32 * c + l] >> 4;
                if (qtype == IB_Q5_K) {
                    lo += (qh[l] & (1u << (2 * c))) ? 16 : 0;
                    hi += (qh[l] & (2u << (2 * c))) ? 16 : 0;
                }
                acc += (d1 * (float)lo - m1) * v[64 * c + l];
                acc += (d2 * (float)hi - m2) * v[64 * c + 32 + l];
            }
        }
    } else if (qtype == IB_Q4_0 || qtype == IB_Q4_1 || qtype == IB_Q5_0 || qtype == IB_Q5_1) {
        // crates/inferi/src/quantization.rs:68-82, 96-111, 125-142, 157-175: 32 elements, low nibbles first, optional
        // minimum (the _1 types) and fifth bit (the Q5 types)
        const bool has_m = qtype == IB_Q4_1 || qtype == IB_Q5_1, five = qtype == IB_Q5_0 || qtype == IB_Q5_1;
        const float d = ld_h(b), m = has_m ? ld_h(b + 2) : 0.f;
        const uint8_t *qhp = b + (has_m ? 4 : 2), *qs = qhp + (five ? 4 : 0);
        const uint32_t qh = five ? ((uint32_t)qhp[0] | ((uint32_t)qhp[1] << 8) | ((uint32_t)qhp[2] << 16) | ((uint32_t)qhp[3] << 24)) : 0u;
        const int off = has_m ? 0 : (five ? 16 : 8);
        for (int j = 0; j < 16; j++) {
            const uint32_t x0 = (qs[j] & 0x0Fu) | (((qh >> j) << 4) & 0x10u), x1 = (uint32_t)(qs[j] >> 4) | ((qh >> (j + 12)) & 0x10u);
            acc += ((float)((int)x0 - off) * d + m) * v[j];
            acc += ((float)((int)x1 - off) * d + m) * v[j + 16];
        }
    } else if (qtype == IB_Q8_K) {
        // crates/inferi/src/quantization.rs:205-211: f32 scale, 256 int8 quants (the block sums are not used by the GEMV)
        float d;
        memcpy(&d, b, 4);
        for (int j = 0; j < 256; j++) acc += (d * (float)(int8_t)b[4 + j]) * v[j];
    } else if (qtype == IB_Q6_K) {
        const uint8_t *ql = b, *qh = b + 128;
        const int8_t *sc = reinterpret_cast<const int8_t *>(b + 192);
        const float d = ld_h(b + 208);
        for (int i = 0; i < 2; i++)
            for (int l = 0; l < 32; l++) {
                const int is = l / 16;
                const uint32_t ql0 = ql[64 * i + l], ql32 = ql[64 * i + 32 + l], h = qh[32 * i + l];
                const int q1 = (int)((ql0 & 0xF) | ((h & 3) << 4)) - 32;
                const int q2 = (int)((ql32 & 0xF) | (((h >> 2) & 3) << 4)) - 32;
                const int q3 = (int)((ql0 >> 4) | (((h >> 4) & 3) << 4)) - 32;
                const int q4 = (int)((ql32 >> 4) | (((h >> 6) & 3) << 4)) - 32;
                acc += (d * (float)sc[8 * i + is + 0] * (float)q1) * v[128 * i + l];
                acc += (d * (float)sc[8 * i + is + 2] * (float)q2) * v[128 * i + l + 32];
                acc += (d * (float)sc[8 * i + is + 4] * (float)q3) * v[128 * i + l + 64];
                acc += (d * (float)sc[8 * i + is + 6] * (float)q4) * v[128 * i + l + 96];
            }
    }
    return acc;
}

__global__ void __launch_bounds__(256) gemv_generic_kernel(const uint8_t *__restrict__ w, int qtype, uint32_t rows, uint32_t cols, uint64_t row_bytes,
                                                           const float *__restrict__ v, float *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const uint32_t r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const uint8_t *row = w + (size_t)r * row_bytes;
    float acc = 0.f;
    if (qtype == IB_F32) {
        const float *fr = reinterpret_cast<const float *>(row);
        for (uint32_t c = lane; c < cols; c += 32) acc += fr[c] * v[c];
    } else {
        const uint32_t be = block_elems(qtype), bb = block_bytes(qtype);
        for (uint32_t b = lane; b < cols / be; b += 32) acc += generic_block_dot(qtype, row + (size_t)b * bb, v + (size_t)b * be);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[r] = acc;
}

// -------------------------------------------------------------------------------------------------
// upload-time re-tiling into the SOA row layout (same bytes per row)
// -------------------------------------------------------------------------------------------------
__global__ void retile_kernel(int qtype, const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, uint64_t rows, uint32_t nb) {
    const uint64_t total = rows * nb;
    for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = t / nb;
        const uint32_t b = (uint32_t)(t % nb), bb = b & 7;
        if (qtype == IB_Q8_0) {
            const uint8_t *s = src + (r * nb + b) * 34;
            uint8_t *d = dst + r * nb * 34 + (size_t)(b >> 3) * 272;
            for (int i = 0; i < 32; i++) d[32 * bb + i] = s[2 + i];
            d[256 + 2 * bb] = s[0];
            d[256 + 2 * bb + 1] = s[1];
        } else {  // Q6_K
            const uint8_t *s = src + (r * nb + b) * 210;
            uint8_t *d = dst + r * nb * 210 + (size_t)(b >> 3) * 1680;
            for (int i = 0; i < 128; i++) d[128 * bb + i] = s[i];
            for (int i = 0; i < 64; i++) d[1024 + 64 * bb + i] = s[128 + i];
            for (int i = 0; i < 16; i++) d[1536 + 16 * bb + i] = s[192 + i];
            d[1664 + 2 * bb] = s[208];
            d[1664 + 2 * bb + 1] = s[209];
        }
    }
}

int32_t retile_to_soa(ib_ctx *ctx, cudaStream_t stream, int qtype, const uint8_t *src, uint8_t *dst, uint64_t rows, uint32_t nb) {
    const uint64_t total = rows * nb;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 65535 ? (total + threads - 1) / threads : 65535);
    retile_kernel<<<blocks, threads, 0, stream>>>(qtype, src, dst, rows, nb);
    ctx->launches++;
    IB_CHECK_CUDA(cudaGetLastError());
    return IB_OK;
}

bool gemv_fast_eligible(int qtype, uint64_t rows, uint64_t cols) {
    if (rows % 2 || cols > GEMV_MAX_COLS) return false;
    switch (qtype) {
    case IB_Q4_K: case IB_Q5_K: return cols % 256 == 0;
    case IB_Q6_K: return cols % (256 * 8) == 0;  // row bytes 210*nb must be a 16-byte multiple
    case IB_Q8_0: return cols % (32 * 8) == 0;   // row bytes 34*nb must be a 16-byte multiple
    default: return false;
    }
}

void fill_seg(GemvSeg &s, const ib_qtensor *m, float *out) {
    s.w = m->dev; s.out = out; s.row_bytes = m->row_bytes; s.rows = (uint32_t)m->rows;
    s.qtype = (uint32_t)m->qtype; s.layout = m->layout; s.nb = m->nb;
}

template <uint32_t EPI>
static int32_t launch_epi(ib_ctx *ctx, cudaStream_t stream, const GemvParams &p, int grid, size_t smem) {
    static bool attr_set[8] = {false};
    if (!attr_set[ctx->device & 7]) {
        IB_CHECK_CUDA(cudaFuncSetAttribute(gemv_wide_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)act_smem_bytes(GEMV_MAX_COLS)));
        attr_set[ctx->device & 7] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl ? 1 : 0;
    IB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, gemv_wide_kernel<EPI>, p));
    ctx->launches++;
    return IB_OK;
}

int32_t launch_gemv(ib_ctx *ctx, cudaStream_t stream, const GemvParams &p_in) {
    GemvParams p = p_in;
    p.err = ctx->err_dev;
    p.wait_ns = ctx->wait_limit_ns;
    IB_REQUIRE(p.nseg >= 1 && p.nseg <= 3, "gemv: bad segment count %u", p.nseg);
    if (gemv_stream_eligible(p)) return launch_gemv_stream(ctx, stream, p);
    if (p.tp > 1 || p.epi == EPI_PUSH)   // the cross-GPU exchange exists only in the streaming kernel
        return set_error(IB_ERR_UNSUPPORTED, "gemv: a tensor-parallel shard (cols=%u) does not meet the streaming kernel's shape rules", p.cols);
    IB_REQUIRE(p.cols % 32 == 0 && p.cols <= GEMV_MAX_COLS, "gemv: cols=%u unsupported by the fast kernels", p.cols);
    uint32_t pairs = 0;
    for (uint32_t s = 0; s < p.nseg; s++) {
        IB_REQUIRE(p.seg[s].rows % 2 == 0, "gemv: odd row count");
        pairs += p.seg[s].rows / 2;
    }
    if (p.epi == EPI_SWIGLU) {
        IB_REQUIRE(p.nseg == 2 && p.seg[0].rows == p.seg[1].rows && p.seg[0].qtype == p.seg[1].qtype && p.seg[0].nb == p.seg[1].nb,
                   "gemv: gate/up must have the same shape and type");
        pairs = p.seg[0].rows;
    }
    const int max_ctas = ctx->sm_count * 2;
    int grid = (int)((pairs + GEMV_WARPS - 1) / GEMV_WARPS);
    if (grid > max_ctas) grid = max_ctas;
    if (grid < 1) grid = 1;
    const size_t smem = act_smem_bytes(p.cols);
    switch (p.epi) {
    case EPI_STORE: return launch_epi<EPI_STORE>(ctx, stream, p, grid, smem);
    case EPI_RESIDUAL: return launch_epi<EPI_RESIDUAL>(ctx, stream, p, grid, smem);
    case EPI_SWIGLU: return launch_epi<EPI_SWIGLU>(ctx, stream, p, grid, smem);
    case EPI_QKV: return launch_epi<EPI_QKV>(ctx, stream, p, grid, smem);
    case EPI_ARGMAX: return launch_epi<EPI_ARGMAX>(ctx, stream, p, grid, smem);
    default: return set_error(IB_ERR_INVALID, "gemv: unknown epilogue %u", p.epi);
    }
}

int32_t launch_gemv_generic(ib_ctx *ctx, cudaStream_t stream, const ib_qtensor *m, const float *v, float *out) {
    const int warps = 8;
    const int grid = (int)((m->rows + warps - 1) / warps);
    gemv_generic_kernel<<<grid, warps * 32, 0, stream>>>(m->dev, m->qtype, (uint32_t)m->rows, (uint32_t)m->cols, m->row_bytes, v, out);
    ctx->launches++;
    IB_CHECK_CUDA(cudaGetLastError());
    return IB_OK;
}

}  // namespace ib
