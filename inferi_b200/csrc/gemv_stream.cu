// Streaming quantized GEMV for sm_100a: the kernel of the token loop.
//
// Replaces the reference shaders crates/inferi-shaders/src/gemv_quant_{q8_0x2,q4_k,q5_k,q6_kx2}.rs (one 32-thread
// workgroup per 4 rows, 4-byte scattered loads) and their launcher crates/inferi/src/ops/gemv_quant.rs:183-341.
//
// One persistent CTA per SM owns a contiguous, byte-balanced range of row pairs.
//  * A producer warp streams the CTA's rows from HBM into a shared-memory ring with bulk asynchronous copies
//    (cp.async.bulk, one copy per tile of up to 8 contiguous row pairs, completion on an mbarrier).  It starts
//    before the kernel waits for its predecessor (programmatic dependent launch): weights never depend on the
//    previous kernel, so the ring fills while that kernel is still finishing.
//  * Eight consumer warps split a row's columns: every lane owns one 64-weight unit of the row and keeps that
//    unit's activations — three int8 limbs per column, see gemv_common.cuh — in registers for the whole kernel, so
//    the inner loop touches shared memory only for weights.  Per weight the work is a byte mask and dp4a.
//  * Per row the lane partials are shuffled down, per-warp partials meet in shared memory, and the last warp of a
//    row group to arrive adds them in a fixed order and runs the epilogue (store / residual add / SwiGLU /
//    RoPE + KV append / arg-max).  No warp ever waits for another one except through the ring.
// Every wait on an mbarrier is bounded; a wait that gives up raises the context's error word and carries on.
#include "gemv_common.cuh"

namespace ib {

constexpr int CW = 8;                           // consumer warps
constexpr int STREAM_THREADS = (CW + 1) * 32;   // + 1 producer warp
constexpr int PT_MAX = 8;                       // row pairs per tile
constexpr unsigned long long WAIT_LIMIT_NS = 4000000000ull;   // a wait on an mbarrier gives up after 4 s

struct StreamGeom {
    uint32_t stages, stage_bytes, act_off, part_off, bar_off;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and raises *err) if the phase never completes.
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t *err, uint32_t code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 256; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - t0 > WAIT_LIMIT_NS) break;
    }
    if (err) {
        *(volatile uint32_t *)err = code;   // mapped host memory: a plain store, made visible system-wide
        __threadfence_system();
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// ---- this CTA's share of the work: per segment a contiguous range of row pairs, balanced by bytes ----
struct Share {
    uint32_t a[3], b[3];     // pair range per segment
    uint32_t cost[3];        // bytes per pair
    uint32_t pt[3];          // pairs per tile
    uint32_t nseg;
};

template <uint32_t EPI>
__device__ __forceinline__ void make_share(const GemvParams &p, uint32_t stage_bytes, Share &sh) {
    uint32_t pairs[3];
    unsigned long long start[4];
    sh.nseg = (EPI == EPI_SWIGLU) ? 1u : p.nseg;
    start[0] = 0;
#pragma unroll
    for (int s = 0; s < 3; s++) {
        if (s < (int)sh.nseg) {
            if (EPI == EPI_SWIGLU) { pairs[s] = p.seg[0].rows; sh.cost[s] = (uint32_t)(p.seg[0].row_bytes + p.seg[1].row_bytes); }
            else { pairs[s] = p.seg[s].rows / 2; sh.cost[s] = (uint32_t)(2 * p.seg[s].row_bytes); }
        } else { pairs[s] = 0; sh.cost[s] = 1; }
        start[s + 1] = start[s] + (unsigned long long)pairs[s] * sh.cost[s];
        uint32_t pt = stage_bytes / sh.cost[s];
        sh.pt[s] = pt < 1 ? 1 : (pt > PT_MAX ? PT_MAX : pt);
    }
    const unsigned long long total = start[3];
    const unsigned long long lo = total * blockIdx.x / gridDim.x, hi = total * (blockIdx.x + 1) / gridDim.x;
#pragma unroll
    for (int s = 0; s < 3; s++) {
        const unsigned long long c = sh.cost[s];
        unsigned long long a = lo > start[s] ? (lo - start[s] + c - 1) / c : 0;
        unsigned long long b = hi > start[s] ? (hi - start[s] + c - 1) / c : 0;
        sh.a[s] = (uint32_t)(a > pairs[s] ? pairs[s] : a);
        sh.b[s] = (uint32_t)(b > pairs[s] ? pairs[s] : b);
    }
}

struct TileCursor {
    uint32_t seg, next;   // segment and first pair of the next tile
    __device__ __forceinline__ void init(const Share &sh) {
        seg = 0;
        next = sh.a[0];
        skip(sh);
    }
    __device__ __forceinline__ void skip(const Share &sh) {
        while (seg < sh.nseg && next >= sh.b[seg]) {
            seg++;
            if (seg < sh.nseg) next = sh.a[seg];
        }
    }
    __device__ __forceinline__ bool valid(const Share &sh) const { return seg < sh.nseg; }
    // current tile: pairs [next, next + n) of segment seg
    __device__ __forceinline__ uint32_t count(const Share &sh) const {
        const uint32_t left = sh.b[seg] - next;
        return left < sh.pt[seg] ? left : sh.pt[seg];
    }
    __device__ __forceinline__ void advance(const Share &sh) {
        next += count(sh);
        skip(sh);
    }
};

// ---- per-lane activation registers of one 64-weight unit ----
struct UnitAct {
    uint4 l[3][4];   // 3 limbs x 4 groups of 16 columns
    float s[4];      // per-group scale (already divided where the format needs it)
    float x[4];      // per-group sum of x
};

// Unit u of a row, by format:
//   Q4_K / Q5_K: block u>>2, 64-column chunk c = u&3: columns 256b + 64c .. +63; groups 0,1 = low nibbles, 2,3 = high nibbles
//   Q6_K       : block u>>2, half i = (u>>1)&1, 16-byte half h = u&1: groups g = 0..3 at 256b + 128i + 32g + 16h
//   Q8_0       : blocks 2u, 2u+1: columns 64u .. +63
__device__ __forceinline__ void load_unit_act(uint32_t qtype, uint32_t u, const Act &A, UnitAct &ua) {
    const float *SC = A.sc(), *SX = A.sx16();
    uint32_t e16[4];
    if (qtype == IB_Q6_K) {
        const uint32_t b = u >> 2, i = (u >> 1) & 1, h = u & 1, base = 16 * b + 8 * i + h;
#pragma unroll
        for (int g = 0; g < 4; g++) e16[g] = base + 2 * g;
    } else {
#pragma unroll
        for (int g = 0; g < 4; g++) e16[g] = 4 * u + g;
    }
#pragma unroll
    for (int g = 0; g < 4; g++) {
#pragma unroll
        for (int k = 0; k < 3; k++) ua.l[k][g] = A.limb(k)[e16[g]];
        ua.s[g] = SC[e16[g] >> 1];
        ua.x[g] = SX[e16[g]];
    }
    if (qtype == IB_Q4_K) { ua.s[2] *= (1.0f / 16.0f); ua.s[3] *= (1.0f / 16.0f); }  // high nibbles are used in place (16 q)
}

__device__ __forceinline__ int dot4_ss(const uint4 &q, const uint4 &a, int d) {
    d = dp4a_ss(q.x, a.x, d); d = dp4a_ss(q.y, a.y, d); d = dp4a_ss(q.z, a.z, d); return dp4a_ss(q.w, a.w, d);
}
__device__ __forceinline__ int dot4_us(const uint4 &q, const uint4 &a, int d) {
    d = dp4a_us(q.x, a.x, d); d = dp4a_us(q.y, a.y, d); d = dp4a_us(q.z, a.z, d); return dp4a_us(q.w, a.w, d);
}
__device__ __forceinline__ uint4 and4(const uint4 &q, uint32_t m) { return make_uint4(q.x & m, q.y & m, q.z & m, q.w & m); }

// One row (in shared memory) x one unit.  Returns the lane's partial dot product.
__device__ __forceinline__ float unit_dot_q4k(const uint8_t *row, uint32_t u, const UnitAct &ua) {
    const uint32_t b = u >> 2, c = u & 3;
    const uint8_t *blk = row + b * 144;
    const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
    const uint4 q0 = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * c);
    const uint4 q1 = *reinterpret_cast<const uint4 *>(blk + 32 + 32 * c);
    const uint4 l0 = and4(q0, 0x0F0F0F0Fu), l1 = and4(q1, 0x0F0F0F0Fu), h0 = and4(q0, 0xF0F0F0F0u), h1 = and4(q1, 0xF0F0F0F0u);
    int D[4][3];
#pragma unroll
    for (int k = 0; k < 3; k++) {
        D[0][k] = dot4_ss(l0, ua.l[k][0], 0);
        D[1][k] = dot4_ss(l1, ua.l[k][1], 0);
        D[2][k] = dot4_us(h0, ua.l[k][2], 0);
        D[3][k] = dot4_us(h1, ua.l[k][3], 0);
    }
    uint32_t sc2, m2;
    kquant_scales(hdr, c, sc2, m2);
    const float d = h2f(hdr.x & 0xFFFFu), dmin = h2f(hdr.x >> 16);
    const float lo = ua.s[0] * limb_combine(D[0][0], D[0][1], D[0][2]) + ua.s[1] * limb_combine(D[1][0], D[1][1], D[1][2]);
    const float hi = ua.s[2] * limb_combine(D[2][0], D[2][1], D[2][2]) + ua.s[3] * limb_combine(D[3][0], D[3][1], D[3][2]);
    return (d * (float)(sc2 & 0xFFu)) * lo - (dmin * (float)(m2 & 0xFFu)) * (ua.x[0] + ua.x[1]) + (d * (float)(sc2 >> 8)) * hi -
           (dmin * (float)(m2 >> 8)) * (ua.x[2] + ua.x[3]);
}

__device__ __forceinline__ float unit_dot_q5k(const uint8_t *row, uint32_t u, const UnitAct &ua) {
    const uint32_t b = u >> 2, c = u & 3;
    const uint8_t *blk = row + b * 176;
    const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
    const uint4 hA = *reinterpret_cast<const uint4 *>(blk + 16), hB = *reinterpret_cast<const uint4 *>(blk + 32);
    const uint4 q0 = *reinterpret_cast<const uint4 *>(blk + 48 + 32 * c), q1 = *reinterpret_cast<const uint4 *>(blk + 64 + 32 * c);
    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    const uint32_t hw[8] = {hA.x, hA.y, hA.z, hA.w, hB.x, hB.y, hB.z, hB.w};
    uint32_t lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t t = hw[i] >> (2 * c);  // bit 0 of each byte: flag of the low-nibble element, bit 1: of the high-nibble element
        lo[i] = (qw[i] & 0x0F0F0F0Fu) | ((t << 4) & 0x10101010u);
        hi[i] = ((qw[i] >> 4) & 0x0F0F0F0Fu) | ((t << 3) & 0x10101010u);
    }
    int D[4][3];
#pragma unroll
    for (int k = 0; k < 3; k++) {
        D[0][k] = dot4_ss(make_uint4(lo[0], lo[1], lo[2], lo[3]), ua.l[k][0], 0);
        D[1][k] = dot4_ss(make_uint4(lo[4], lo[5], lo[6], lo[7]), ua.l[k][1], 0);
        D[2][k] = dot4_ss(make_uint4(hi[0], hi[1], hi[2], hi[3]), ua.l[k][2], 0);
        D[3][k] = dot4_ss(make_uint4(hi[4], hi[5], hi[6], hi[7]), ua.l[k][3], 0);
    }
    uint32_t sc2, m2;
    kquant_scales(hdr, c, sc2, m2);
    const float d = h2f(hdr.x & 0xFFFFu), dmin = h2f(hdr.x >> 16);
    const float lo_f = ua.s[0] * limb_combine(D[0][0], D[0][1], D[0][2]) + ua.s[1] * limb_combine(D[1][0], D[1][1], D[1][2]);
    const float hi_f = ua.s[2] * limb_combine(D[2][0], D[2][1], D[2][2]) + ua.s[3] * limb_combine(D[3][0], D[3][1], D[3][2]);
    return (d * (float)(sc2 & 0xFFu)) * lo_f - (dmin * (float)(m2 & 0xFFu)) * (ua.x[0] + ua.x[1]) + (d * (float)(sc2 >> 8)) * hi_f -
           (dmin * (float)(m2 >> 8)) * (ua.x[2] + ua.x[3]);
}

// Q6_K rows are stored as groups of 8 blocks: [8 x 128 ql][8 x 64 qh][8 x 16 scales][8 x 2 d] = 1680 bytes per 2048 columns.
__device__ __forceinline__ float unit_dot_q6k(const uint8_t *row, uint32_t u, const UnitAct &ua) {
    const uint32_t b = u >> 2, i = (u >> 1) & 1, h = u & 1;
    const uint8_t *grp = row + (b >> 3) * 1680;
    const uint32_t bb = b & 7;
    const uint4 qa = *reinterpret_cast<const uint4 *>(grp + 128 * bb + 64 * i + 16 * h);
    const uint4 qb = *reinterpret_cast<const uint4 *>(grp + 128 * bb + 64 * i + 32 + 16 * h);
    const uint4 qh = *reinterpret_cast<const uint4 *>(grp + 1024 + 64 * bb + 32 * i + 16 * h);
    const uint2 scw = *reinterpret_cast<const uint2 *>(grp + 1536 + 16 * bb + 8 * i);  // scales[8i .. 8i+7]
    const float d = h2f(*reinterpret_cast<const unsigned short *>(grp + 1664 + 2 * bb));
    const uint32_t la[4] = {qa.x, qa.y, qa.z, qa.w}, lb[4] = {qb.x, qb.y, qb.z, qb.w}, hh[4] = {qh.x, qh.y, qh.z, qh.w};
    uint32_t g0[4], g1[4], g2[4], g3[4];
#pragma unroll
    for (int w = 0; w < 4; w++) {
        // crates/inferi/src/quantization.rs:237-246: 4 low bits from ql, 2 high bits from qh
        g0[w] = (la[w] & 0x0F0F0F0Fu) | ((hh[w] << 4) & 0x30303030u);
        g1[w] = (lb[w] & 0x0F0F0F0Fu) | ((hh[w] << 2) & 0x30303030u);
        g2[w] = ((la[w] >> 4) & 0x0F0F0F0Fu) | (hh[w] & 0x30303030u);
        g3[w] = ((lb[w] >> 4) & 0x0F0F0F0Fu) | ((hh[w] >> 2) & 0x30303030u);
    }
    int D[4][3];
#pragma unroll
    for (int k = 0; k < 3; k++) {
        D[0][k] = dot4_ss(make_uint4(g0[0], g0[1], g0[2], g0[3]), ua.l[k][0], 0);
        D[1][k] = dot4_ss(make_uint4(g1[0], g1[1], g1[2], g1[3]), ua.l[k][1], 0);
        D[2][k] = dot4_ss(make_uint4(g2[0], g2[1], g2[2], g2[3]), ua.l[k][2], 0);
        D[3][k] = dot4_ss(make_uint4(g3[0], g3[1], g3[2], g3[3]), ua.l[k][3], 0);
    }
    float v = 0.f;
#pragma unroll
    for (int g = 0; g < 4; g++) {
        const uint32_t word = (g < 2) ? scw.x : scw.y;   // scale index 8i + 2g + h
        const int sc = (int)(int8_t)(word >> (8 * (2 * (g & 1) + h)));
        v += (d * (float)sc) * (ua.s[g] * limb_combine(D[g][0], D[g][1], D[g][2]) - 32.0f * ua.x[g]);
    }
    return v;
}

// Q8_0 rows are stored as groups of 8 blocks: [8 x 32 quants][8 x 2 scale] = 272 bytes per 256 columns.
__device__ __forceinline__ float unit_dot_q80(const uint8_t *row, uint32_t u, const UnitAct &ua) {
    const uint32_t b0 = 2 * u;
    const uint8_t *grp = row + (b0 >> 3) * 272;
    const uint32_t bb = b0 & 7;
    const uint4 q0 = *reinterpret_cast<const uint4 *>(grp + 32 * bb), q1 = *reinterpret_cast<const uint4 *>(grp + 32 * bb + 16);
    const uint4 q2 = *reinterpret_cast<const uint4 *>(grp + 32 * bb + 32), q3 = *reinterpret_cast<const uint4 *>(grp + 32 * bb + 48);
    const uint32_t dd = *reinterpret_cast<const uint32_t *>(grp + 256 + 2 * bb);   // two f16 scales
    int D[4][3];
#pragma unroll
    for (int k = 0; k < 3; k++) {
        D[0][k] = dot4_ss(q0, ua.l[k][0], 0);
        D[1][k] = dot4_ss(q1, ua.l[k][1], 0);
        D[2][k] = dot4_ss(q2, ua.l[k][2], 0);
        D[3][k] = dot4_ss(q3, ua.l[k][3], 0);
    }
    const float a = ua.s[0] * limb_combine(D[0][0], D[0][1], D[0][2]) + ua.s[1] * limb_combine(D[1][0], D[1][1], D[1][2]);
    const float c = ua.s[2] * limb_combine(D[2][0], D[2][1], D[2][2]) + ua.s[3] * limb_combine(D[3][0], D[3][1], D[3][2]);
    return h2f(dd & 0xFFFFu) * a + h2f(dd >> 16) * c;
}

__device__ __forceinline__ float unit_dot(uint32_t qtype, const uint8_t *row, uint32_t u, const UnitAct &ua) {
    switch (qtype) {
    case IB_Q4_K: return unit_dot_q4k(row, u, ua);
    case IB_Q6_K: return unit_dot_q6k(row, u, ua);
    case IB_Q5_K: return unit_dot_q5k(row, u, ua);
    default: return unit_dot_q80(row, u, ua);
    }
}

// ---- epilogue of one row pair ----
template <uint32_t EPI>
__device__ __forceinline__ void epilogue(const GemvParams &p, uint32_t s, uint32_t pair, float a, float b, unsigned long long &best) {
    if (EPI == EPI_SWIGLU) {
        // crates/inferi-shaders/src/silu.rs:16-19,46-52: a = gate row, b = up row
        p.seg[0].out[pair] = b * (a / (1.0f + expf(-a)));
        return;
    }
    const uint32_t r0 = 2 * pair;
    if (EPI == EPI_STORE) {
        *reinterpret_cast<float2 *>(p.seg[s].out + r0) = make_float2(a, b);
    } else if (EPI == EPI_RESIDUAL) {
        const float2 r = __ldcg(reinterpret_cast<const float2 *>(p.resid + r0));
        *reinterpret_cast<float2 *>(p.seg[s].out + r0) = make_float2(r.x + a, r.y + b);
    } else if (EPI == EPI_QKV) {
        if (s < 2) {
            // crates/inferi-shaders/src/rope.rs:75-91 (adjacent pairs)
            const float2 cs = __ldcg(p.rope_cs + ((r0 % p.head_size) >> 1));
            const float x = a, y = b;
            a = cs.x * x - cs.y * y;
            b = cs.y * x + cs.x * y;
        }
        if (s == 0) {
            *reinterpret_cast<float2 *>(p.seg[0].out + r0) = make_float2(a, b);
        } else {
            void *cache = (s == 1) ? p.k_cache : p.v_cache;
            const size_t off = (size_t)(*p.pos_ptr) * p.kv_dim + r0;
            if (p.kv_dtype == IB_KV_F16) reinterpret_cast<__half2 *>(cache)[off >> 1] = __floats2half2_rn(a, b);
            else reinterpret_cast<float2 *>(cache)[off >> 1] = make_float2(a, b);
        }
    } else if (EPI == EPI_ARGMAX) {
        if (p.seg[0].out) *reinterpret_cast<float2 *>(p.seg[0].out + r0) = make_float2(a, b);
        best = max(best, max(argmax_key(a, p.row_offset + r0), argmax_key(b, p.row_offset + r0 + 1)));
    }
}

// ---- the kernel ----
template <uint32_t EPI>
__global__ void __launch_bounds__(STREAM_THREADS, 2) gemv_stream_kernel(const GemvParams p, const StreamGeom geo) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float red[PACK_THREADS / 32 + 1];
    __shared__ unsigned long long best_sm[CW];
    __shared__ bool is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    uint8_t *ring = smem;
    uint8_t *act_sm = smem + geo.act_off;
    float *part = reinterpret_cast<float *>(smem + geo.part_off);              // [stages][PT_MAX][2][CW]
    uint32_t *cnt = reinterpret_cast<uint32_t *>(part + geo.stages * PT_MAX * 2 * CW);   // [stages][CW]
    const uint32_t bar0 = smem_u32(smem + geo.bar_off);                         // full[stages], empty[stages]
    const uint32_t S = geo.stages;

    const uint32_t units = p.cols / 64;
    const uint32_t CG = (units + 31) / 32;       // warps that split one row's columns
    const uint32_t RG = CW / CG;                 // row groups working side by side
    const uint32_t active = CG * RG;             // consumer warps with work

    Share sh;
    make_share<EPI>(p, geo.stage_bytes, sh);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; s++) {
            mbar_init(bar0 + 8 * s, 1);                 // full: the producer's expect_tx arrival
            mbar_init(bar0 + 8 * (S + s), active);      // empty: one arrival per working consumer warp
        }
        for (uint32_t i = 0; i < S * CW; i++) cnt[i] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (p.pdl) asm volatile("griddepcontrol.launch_dependents;");

    if (warp == CW) {
        // ================= producer warp: one lane streams this CTA's tiles =================
        if (lane == 0) {
            TileCursor tc;
            tc.init(sh);
            for (uint32_t k = 0; tc.valid(sh); k++, tc.advance(sh)) {
                const uint32_t st = k % S;
                if (k >= S && !mbar_wait(bar0 + 8 * (S + st), ((k / S) - 1) & 1, p.err, 2)) break;
                const uint32_t n = tc.count(sh), s = tc.seg;
                const uint32_t dst = smem_u32(ring + (size_t)st * geo.stage_bytes), full = bar0 + 8 * st;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                if (EPI == EPI_SWIGLU) {
                    const uint32_t ba = n * (uint32_t)p.seg[0].row_bytes, bb = n * (uint32_t)p.seg[1].row_bytes;
                    mbar_expect_tx(full, ba + bb);
                    bulk_g2s(dst, p.seg[0].w + (size_t)tc.next * p.seg[0].row_bytes, ba, full);
                    bulk_g2s(dst + ba, p.seg[1].w + (size_t)tc.next * p.seg[1].row_bytes, bb, full);
                } else {
                    const uint32_t bytes = n * sh.cost[s];
                    mbar_expect_tx(full, bytes);
                    bulk_g2s(dst, p.seg[s].w + (size_t)tc.next * sh.cost[s], bytes, full);
                }
            }
        }
        return;
    }

    // ================= consumer warps =================
    if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    pack_activation(act_sm, p.cols, p.x, p.norm_w, p.eps, red);
    const Act A{act_sm, p.cols};

    const uint32_t cg = warp % CG, rg = warp / CG;
    const uint32_t u = cg * 32 + lane;
    const bool has_unit = (uint32_t)warp < active && u < units;
    unsigned long long best = 0ull;

    if ((uint32_t)warp < active) {
        UnitAct ua;
        uint32_t ua_type = 0xFFFFFFFFu;
        TileCursor tc;
        tc.init(sh);
        for (uint32_t k = 0; tc.valid(sh); k++, tc.advance(sh)) {
            const uint32_t st = k % S, s = tc.seg, n = tc.count(sh);
            const uint32_t qtype = p.seg[s].qtype;
            if (qtype != ua_type) {   // (re)load this lane's activations in the layout of the segment's format
                if (has_unit) load_unit_act(qtype, u, A, ua);
                ua_type = qtype;
            }
            if (!mbar_wait(bar0 + 8 * st, (k / S) & 1, p.err, 1)) break;   // the error word is raised; give up on this CTA's rows
            const uint8_t *tile = ring + (size_t)st * geo.stage_bytes;
            const uint32_t rbA = (uint32_t)p.seg[s].row_bytes;
            const uint32_t rbB = (EPI == EPI_SWIGLU) ? (uint32_t)p.seg[1].row_bytes : rbA;
            float *pt = part + (size_t)st * PT_MAX * 2 * CW;
            for (uint32_t pr = rg; pr < n; pr += RG) {
                const uint8_t *rowA = (EPI == EPI_SWIGLU) ? tile + (size_t)pr * rbA : tile + (size_t)(2 * pr) * rbA;
                const uint8_t *rowB = (EPI == EPI_SWIGLU) ? tile + (size_t)n * rbA + (size_t)pr * rbB : rowA + rbA;
                float va = 0.f, vb = 0.f;
                if (has_unit) {
                    va = unit_dot(qtype, rowA, u, ua);
                    vb = unit_dot(qtype, rowB, u, ua);
                }
#pragma unroll
                for (int o = 16; o; o >>= 1) {
                    va += __shfl_xor_sync(0xffffffffu, va, o);
                    vb += __shfl_xor_sync(0xffffffffu, vb, o);
                }
                if (CG == 1) {
                    if (lane == 0) epilogue<EPI>(p, s, tc.next + pr, va, vb, best);
                } else if (lane == 0) {
                    pt[(pr * 2 + 0) * CW + cg] = va;
                    pt[(pr * 2 + 1) * CW + cg] = vb;
                }
            }
            if (CG > 1) {
                // the last warp of the row group to finish the tile folds the column partials in a fixed order
                uint32_t last = 0;
                if (lane == 0) {
                    __threadfence_block();
                    last = (atomicAdd(cnt + st * CW + rg, 1u) == CG - 1) ? 1u : 0u;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence_block();
                    const uint32_t pr = rg + RG * lane;
                    if (pr < n) {
                        float va = 0.f, vb = 0.f;
                        for (uint32_t c = 0; c < CG; c++) {
                            va += pt[(pr * 2 + 0) * CW + c];
                            vb += pt[(pr * 2 + 1) * CW + c];
                        }
                        epilogue<EPI>(p, s, tc.next + pr, va, vb, best);
                    }
                    __syncwarp();
                    if (lane == 0) cnt[st * CW + rg] = 0;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar0 + 8 * (S + st));   // this warp is done with the stage
        }
    }

    if (EPI == EPI_ARGMAX) {
#pragma unroll
        for (int o = 16; o; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
        if (lane == 0) best_sm[warp] = best;
        named_barrier(1, PACK_THREADS);
        if (threadIdx.x == 0) {
            unsigned long long b = 0ull;
            for (int w = 0; w < CW; w++) b = max(b, best_sm[w]);
            p.argmax_slots[blockIdx.x] = b;
            __threadfence();
            is_last = (atomicAdd(p.argmax_counter, 1u) == gridDim.x - 1);
        }
        named_barrier(1, PACK_THREADS);
        if (is_last) {
            // the last CTA to arrive folds every CTA's candidate; no CTA waits for another
            __threadfence();
            unsigned long long b = 0ull;
            for (uint32_t i = threadIdx.x; i < gridDim.x; i += PACK_THREADS) b = max(b, __ldcg(p.argmax_slots + i));
#pragma unroll
            for (int o = 16; o; o >>= 1) b = max(b, __shfl_xor_sync(0xffffffffu, b, o));
            named_barrier(1, PACK_THREADS);
            if (lane == 0) best_sm[warp] = b;
            named_barrier(1, PACK_THREADS);
            if (threadIdx.x == 0) {
                for (int w = 0; w < CW; w++) b = max(b, best_sm[w]);
                *p.argmax_out = 0xFFFFFFFFu - (uint32_t)(b & 0xFFFFFFFFull);
                *p.argmax_counter = 0u;
            }
        }
    }
}

// -------------------------------------------------------------------------------------------------
// host side
// -------------------------------------------------------------------------------------------------
constexpr size_t STREAM_SMEM_BUDGET = 108 * 1024;   // two CTAs (this kernel and the next one, prefetching) share an SM

bool gemv_stream_eligible(const GemvParams &p) {
    if (p.cols % 64 || p.cols > 16384) return false;
    for (uint32_t s = 0; s < p.nseg; s++) {
        const uint32_t q = p.seg[s].qtype;
        if (q != IB_Q4_K && q != IB_Q5_K && q != IB_Q6_K && q != IB_Q8_0) return false;
        if (p.seg[s].row_bytes % 16) return false;
    }
    return true;
}

template <uint32_t EPI>
static int32_t launch_stream_epi(ib_ctx *ctx, cudaStream_t stream, const GemvParams &p, int grid, const StreamGeom &geo, size_t smem) {
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        IB_CHECK_CUDA(cudaFuncSetAttribute(gemv_stream_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)STREAM_SMEM_BUDGET));
        attr_set[ctx->device & 15] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(STREAM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl ? 1 : 0;
    IB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, gemv_stream_kernel<EPI>, p, geo));
    ctx->launches++;
    return IB_OK;
}

int32_t launch_gemv_stream(ib_ctx *ctx, cudaStream_t stream, const GemvParams &p) {
    uint32_t max_cost = 0, pairs = 0;
    if (p.epi == EPI_SWIGLU) {
        max_cost = (uint32_t)(p.seg[0].row_bytes + p.seg[1].row_bytes);
        pairs = p.seg[0].rows;
    } else {
        for (uint32_t s = 0; s < p.nseg; s++) {
            const uint32_t c = (uint32_t)(2 * p.seg[s].row_bytes);
            if (c > max_cost) max_cost = c;
            pairs += p.seg[s].rows / 2;
        }
    }
    // stage: as many pairs as fit in ~20 KB (at least one), the same byte budget for every segment
    uint32_t stage = 0;
    if (p.epi == EPI_SWIGLU) {
        uint32_t pt = 20480 / max_cost;
        pt = pt < 1 ? 1 : (pt > PT_MAX ? PT_MAX : pt);
        stage = pt * max_cost;
    } else {
        for (uint32_t s = 0; s < p.nseg; s++) {
            const uint32_t c = (uint32_t)(2 * p.seg[s].row_bytes);
            uint32_t pt = 20480 / c;
            pt = pt < 1 ? 1 : (pt > PT_MAX ? PT_MAX : pt);
            if (pt * c > stage) stage = pt * c;
        }
    }
    stage = (stage + 127) & ~127u;
    const size_t act = (act_smem_bytes(p.cols) + 127) & ~(size_t)127;
    StreamGeom geo;
    uint32_t S = 4;
    size_t total = 0;
    for (;; S--) {
        const size_t part = (size_t)S * PT_MAX * 2 * CW * 4 + (size_t)S * CW * 4;
        total = (size_t)S * stage + act + ((part + 127) & ~(size_t)127) + 2 * S * 8;
        if (total <= STREAM_SMEM_BUDGET || S == 2) break;
    }
    if (total > STREAM_SMEM_BUDGET)
        return set_error(IB_ERR_UNSUPPORTED, "gemv: a row pair of %u bytes with %u columns does not fit the streaming kernel's ring", max_cost, p.cols);
    geo.stages = S;
    geo.stage_bytes = stage;
    geo.act_off = S * stage;
    geo.part_off = (uint32_t)(geo.act_off + act);
    geo.bar_off = (uint32_t)(geo.part_off + (((size_t)S * PT_MAX * 2 * CW * 4 + (size_t)S * CW * 4 + 127) & ~(size_t)127));
    int grid = ctx->sm_count;
    if ((uint32_t)grid > pairs) grid = (int)pairs;
    if (grid < 1) grid = 1;
    switch (p.epi) {
    case EPI_STORE: return launch_stream_epi<EPI_STORE>(ctx, stream, p, grid, geo, total);
    case EPI_RESIDUAL: return launch_stream_epi<EPI_RESIDUAL>(ctx, stream, p, grid, geo, total);
    case EPI_SWIGLU: return launch_stream_epi<EPI_SWIGLU>(ctx, stream, p, grid, geo, total);
    case EPI_QKV: return launch_stream_epi<EPI_QKV>(ctx, stream, p, grid, geo, total);
    case EPI_ARGMAX: return launch_stream_epi<EPI_ARGMAX>(ctx, stream, p, grid, geo, total);
    default: return set_error(IB_ERR_INVALID, "gemv: unknown epilogue %u", p.epi);
    }
}

}  // namespace ib
