// Device-side building blocks of the streaming quantized GEMV (shared by the stand-alone GEMV kernel and the
// whole-token kernel): mbarrier / bulk-copy wrappers with bounded waits, the byte-balanced row split, the per-format
// 64-weight unit dot products and the row-pair epilogues.
#pragma once

#include "gemv_common.cuh"

namespace ib {


constexpr int CW = 16;                          // consumer warps
constexpr int W_PRODUCER = CW, W_EPILOGUE = CW + 1;
constexpr int STREAM_THREADS = (CW + 2) * 32;   // + 1 producer warp + 1 epilogue warp
constexpr int PT_MAX = 16;                      // row pairs per tile

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
constexpr uint32_t TRY_WAIT_HINT_NS = 2000u;   // suspend-time hint of mbarrier.try_wait
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(TRY_WAIT_HINT_NS)   // suspend-time hint in ns: a waiting warp sleeps instead of spinning through issue slots
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and raises *err) if the phase does not complete within `limit_ns` (a context setting).
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t *err, uint32_t code, unsigned long long limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 256; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - t0 > limit_ns) break;
    }
    if (err) {
        *(volatile uint32_t *)err = code;   // mapped host memory: a plain store, made visible system-wide
        __threadfence_system();
    }
    return false;
}
// ---- waits on words that another GPU (or another CTA) writes.  Counters only grow; a reader waits until the counter has
// reached the value that the current use implies.  Bounded like every other wait here. ----
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ bool wait_counter(const uint32_t *flag, uint32_t target, uint32_t *err, uint32_t code, unsigned long long limit_ns) {
    if ((int32_t)(ld_acquire_sys(flag) - target) >= 0) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if ((int32_t)(ld_acquire_sys(flag) - target) >= 0) return true;
        if (global_ns() - t0 > limit_ns) break;
    }
    if (err) {
        *(volatile uint32_t *)err = code;
        __threadfence_system();
    }
    return false;
}

// A tagged word of the tensor-parallel exchange: waits (bounded) until the word carries `tag`, returns its value.
__device__ __forceinline__ float wait_tagged(const uint2 *w, uint32_t tag, uint32_t *err, unsigned long long limit_ns) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(w) : "memory");
    if (v.y != tag) {
        const unsigned long long t0 = global_ns();
        for (;;) {
            for (int i = 0; i < 64 && v.y != tag; i++) asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(w) : "memory");
            if (v.y == tag) break;
            if (global_ns() - t0 > limit_ns) {
                if (err) {
                    *(volatile uint32_t *)err = 3;
                    __threadfence_system();
                }
                break;
            }
        }
    }
    return __uint_as_float(v.x);
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// the same bounded wait on a counter that only this GPU's CTAs advance
__device__ __forceinline__ bool wait_counter_gpu(const uint32_t *flag, uint32_t target, uint32_t *err, uint32_t code, unsigned long long limit_ns) {
    if ((int32_t)(ld_acquire_gpu(flag) - target) >= 0) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if ((int32_t)(ld_acquire_gpu(flag) - target) >= 0) return true;
        if (global_ns() - t0 > limit_ns) break;
    }
    if (err) {
        *(volatile uint32_t *)err = code;
        __threadfence_system();
    }
    return false;
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Shared-memory loads by 32-bit shared address (no generic-address arithmetic in the inner loop).  volatile: they stay
// between the mbarrier wait before them and the arrival after them.
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}

// ---- this CTA's share of the work: per segment a contiguous range of row pairs, balanced by bytes ----
// (three scalar sets instead of arrays: indexing them with a run-time segment number would put them in local memory)
struct Share {
    uint32_t a0, a1, a2, b0, b1, b2;   // pair range per segment
    uint32_t c0, c1, c2;               // bytes per pair
    uint32_t t0, t1, t2;               // pairs per tile
    uint32_t nseg;
    __device__ __forceinline__ uint32_t a(uint32_t s) const { return s == 0 ? a0 : (s == 1 ? a1 : a2); }
    __device__ __forceinline__ uint32_t b(uint32_t s) const { return s == 0 ? b0 : (s == 1 ? b1 : b2); }
    __device__ __forceinline__ uint32_t cost(uint32_t s) const { return s == 0 ? c0 : (s == 1 ? c1 : c2); }
    __device__ __forceinline__ uint32_t pt(uint32_t s) const { return s == 0 ? t0 : (s == 1 ? t1 : t2); }
};

// all byte counts in units of 16 bytes so that the arithmetic stays in 32 bits (64-bit divisions cost ~0.2 us each)
__device__ __forceinline__ void share_range(uint32_t lo, uint32_t hi, uint32_t start, uint32_t cost16, uint32_t pairs, uint32_t &a, uint32_t &b) {
    const uint32_t x = lo > start ? (lo - start + cost16 - 1) / cost16 : 0;
    const uint32_t y = hi > start ? (hi - start + cost16 - 1) / cost16 : 0;
    a = x > pairs ? pairs : x;
    b = y > pairs ? pairs : y;
}

__device__ __forceinline__ uint32_t tile_pairs(uint32_t stage_bytes, uint32_t cost, uint32_t RG) {
    uint32_t pt = stage_bytes / cost;
    pt = pt < 1 ? 1 : (pt > PT_MAX ? PT_MAX : pt);
    if (pt > RG) pt = pt / RG * RG;   // whole rounds of the row groups
    return pt;
}

// `swiglu`: gate and up rows travel together (one "pair" = gate row r + up row r).  `sources`/`me`: the CTAs sharing the
// work and this CTA's index among them.
__device__ __forceinline__ void make_share_rt(bool swiglu, uint32_t nseg, uint32_t rows0, uint32_t rows1, uint32_t rows2, uint32_t rb0, uint32_t rb1,
                                              uint32_t rb2, uint32_t stage_bytes, uint32_t RG, uint32_t G, uint32_t me, Share &sh) {
    uint32_t n0, n1 = 0, n2 = 0;
    sh.nseg = swiglu ? 1u : nseg;
    sh.c1 = sh.c2 = 16;
    if (swiglu) { n0 = rows0; sh.c0 = rb0 + rb1; }
    else {
        n0 = rows0 / 2; sh.c0 = 2 * rb0;
        if (sh.nseg > 1) { n1 = rows1 / 2; sh.c1 = 2 * rb1; }
        if (sh.nseg > 2) { n2 = rows2 / 2; sh.c2 = 2 * rb2; }
    }
    const uint32_t k0 = sh.c0 / 16, k1 = sh.c1 / 16, k2 = sh.c2 / 16;
    const uint32_t s1 = n0 * k0, s2 = s1 + n1 * k1, total = s2 + n2 * k2;
    const uint32_t q = total / G, r = total % G;
    const uint32_t lo = q * me + r * me / G, hi = q * (me + 1) + r * (me + 1) / G;
    share_range(lo, hi, 0, k0, n0, sh.a0, sh.b0);
    share_range(lo, hi, s1, k1, n1, sh.a1, sh.b1);
    share_range(lo, hi, s2, k2, n2, sh.a2, sh.b2);
    sh.t0 = tile_pairs(stage_bytes, sh.c0, RG);
    sh.t1 = tile_pairs(stage_bytes, sh.c1, RG);
    sh.t2 = tile_pairs(stage_bytes, sh.c2, RG);
}

__device__ __forceinline__ void make_share(const GemvParams &p, uint32_t stage_bytes, uint32_t RG, Share &sh) {
    make_share_rt(p.epi == EPI_SWIGLU, p.nseg, p.seg[0].rows, p.seg[1].rows, p.seg[2].rows, (uint32_t)p.seg[0].row_bytes, (uint32_t)p.seg[1].row_bytes,
                  (uint32_t)p.seg[2].row_bytes, stage_bytes, RG, gridDim.x, blockIdx.x, sh);
}

struct TileCursor {
    uint32_t seg, next, end, pt;   // segment, first pair of the next tile, end of the segment's range, pairs per tile
    __device__ __forceinline__ void enter(const Share &sh) {
        while (seg < sh.nseg) {
            next = sh.a(seg); end = sh.b(seg); pt = sh.pt(seg);
            if (next < end) break;
            seg++;
        }
    }
    __device__ __forceinline__ void init(const Share &sh) { seg = 0; next = end = pt = 0; enter(sh); }
    __device__ __forceinline__ bool valid(const Share &sh) const { return seg < sh.nseg; }
    __device__ __forceinline__ uint32_t count(const Share &) const { return (end - next) < pt ? (end - next) : pt; }
    __device__ __forceinline__ void advance(const Share &sh) {
        next += count(sh);
        if (next >= end) { seg++; enter(sh); }
    }
};

// ---- per-lane activation registers of one 64-weight unit ----
struct UnitAct {
    uint4 l[ACT_LIMBS][4];   // limbs x 4 groups of 16 columns
    float s[4];      // per-group scale (already divided where the format needs it)
    float x[4];      // per-group sum of x
};

// Unit u of a row, by format:
//   Q4_K / Q5_K: block u>>2, 64-column chunk c = u&3: columns 256b + 64c .. +63; groups 0,1 = low nibbles, 2,3 = high nibbles
//   Q6_K       : block u>>2, half i = (u>>1)&1, 16-byte half h = u&1: groups g = 0..3 at 256b + 128i + 32g + 16h
//   Q8_0       : blocks 2u, 2u+1: columns 64u .. +63
__device__ __forceinline__ void load_unit_act(uint32_t qtype, uint32_t u, const Act &A, UnitAct &ua) {
    uint32_t e16[4];
    if (qtype == IB_Q6_K) {
        const uint32_t b = u >> 2, i = (u >> 1) & 1, h = u & 1, base = 16 * b + 8 * i + h;
#pragma unroll
        for (int g = 0; g < 4; g++) e16[g] = base + 2 * g;
    } else {
#pragma unroll
        for (int g = 0; g < 4; g++) e16[g] = 4 * u + g;
    }
    // 32-bit shared addresses, computed once; volatile loads: they must stay where they are (as ordinary loads they are
    // loop-invariant and would be hoisted to one place where every format's copies stay live at once)
    const uint32_t base = smem_u32(A.base), ls = A.lstride();
    const uint32_t sc0 = base + ACT_LIMBS * ls, sx0 = sc0 + A.cols / 8;   // f32 scale per 32 columns, then f32 sum per 16 columns
#pragma unroll
    for (int g = 0; g < 4; g++) {
        const uint32_t at = base + 16 * A.pos(e16[g]);
#pragma unroll
        for (int k = 0; k < ACT_LIMBS; k++) ua.l[k][g] = lds128(at + k * ls);
        ua.s[g] = __uint_as_float(lds32(sc0 + 4 * (e16[g] >> 1)));
        ua.x[g] = __uint_as_float(lds32(sx0 + 4 * e16[g]));
    }
    if (qtype == IB_Q4_K) { ua.s[2] *= (1.0f / 16.0f); ua.s[3] *= (1.0f / 16.0f); }  // high nibbles are used in place (16 q)
    if (qtype == IB_Q4_K || qtype == IB_Q5_K) {   // groups 0,1 (and 2,3) form one 32-column sub-block: one sum each
        ua.x[0] += ua.x[1];
        ua.x[2] += ua.x[3];
    }
}

// One row (in shared memory, 32-bit shared address) x one unit -> the lane's partial dot product.  Everything that
// depends only on the lane (byte offsets inside a row, shift amounts, masks) is computed once in init().
struct LaneConst { uint32_t o0, o1, o2, o3, k, ma, mb, mc; };
// component w of a 128-bit register group; w is a compile-time constant wherever this is used (unrolled loops)
__device__ __forceinline__ uint32_t comp(const uint4 &v, int w) { return w == 0 ? v.x : (w == 1 ? v.y : (w == 2 ? v.z : v.w)); }
template <uint32_t QT> struct Unit;

// 6-bit (scale, min) pairs of sub-blocks 2c and 2c+1 of a Q4_K / Q5_K header without a branch on c (the lanes of a warp
// differ in c): lanes with c < 2 carry masks (0x3F3F, 0, 0), the others (0, 0x3030, 0x0F0F), and both read the same three
// half-words (crates/inferi/src/quantization.rs:394-402).
__device__ __forceinline__ void kquant_scales_lane(const uint4 &hdr, const LaneConst &lc, uint32_t &sc2, uint32_t &m2) {
    const uint32_t y2 = hdr.y >> lc.o2, z2 = hdr.z >> lc.o2, w2 = hdr.w >> lc.o2;   // o2 = 16 * (c & 1); the masks drop the upper half
    sc2 = (y2 & lc.ma) | ((y2 >> 2) & lc.mb) | (w2 & lc.mc);
    m2 = (z2 & lc.ma) | ((z2 >> 2) & lc.mb) | ((w2 >> 4) & lc.mc);
}
__device__ __forceinline__ void kquant_lane_init(uint32_t c, LaneConst &lc) {
    lc.k = c;
    lc.o2 = 16 * (c & 1);
    lc.ma = c < 2 ? 0x3F3Fu : 0u;
    lc.mb = c < 2 ? 0u : 0x3030u;
    lc.mc = c < 2 ? 0u : 0x0F0Fu;
}
// d * (sc_lo * lo + sc_hi * hi) - dmin * (m_lo * x_lo + m_hi * x_hi) for one 64-column chunk of a Q4_K / Q5_K block
__device__ __forceinline__ float kquant_finish(const uint4 &hdr, uint32_t sc2, uint32_t m2, float lo, float hi, float x_lo, float x_hi) {
    const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
    const float a = (float)(sc2 & 0xFFu) * lo + (float)(sc2 >> 8) * hi;
    const float b = (float)(m2 & 0xFFu) * x_lo + (float)(m2 >> 8) * x_hi;
    return dm.x * a - dm.y * b;
}

template <> struct Unit<IB_Q4_K> {
    static __device__ __forceinline__ void init(uint32_t u, LaneConst &lc) {
        kquant_lane_init(u & 3, lc);
        lc.o0 = (u >> 2) * 144;
        lc.o1 = lc.o0 + 16 + 32 * lc.k;
    }
    static __device__ __forceinline__ float dot(uint32_t row, const LaneConst &lc, const UnitAct &ua) {
        const uint4 hdr = lds128(row + lc.o0), q0 = lds128(row + lc.o1), q1 = lds128(row + lc.o1 + 16);
        const uint32_t qa[4] = {q0.x, q0.y, q0.z, q0.w}, qb[4] = {q1.x, q1.y, q1.z, q1.w};
        int L[3] = {0, 0, 0}, H[3] = {0, 0, 0};   // low nibbles = sub-block 2c (groups 0,1), high nibbles = sub-block 2c+1 (groups 2,3)
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const uint32_t lo = qa[w] & 0x0F0F0F0Fu, hi = qa[w] & 0xF0F0F0F0u;
#pragma unroll
            for (int k = 0; k < ACT_LIMBS; k++) {
                L[k] = dp4a_ss(lo, comp(ua.l[k][0], w), L[k]);
                H[k] = dp4a_us(hi, comp(ua.l[k][2], w), H[k]);
            }
        }
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const uint32_t lo = qb[w] & 0x0F0F0F0Fu, hi = qb[w] & 0xF0F0F0F0u;
#pragma unroll
            for (int k = 0; k < ACT_LIMBS; k++) {
                L[k] = dp4a_ss(lo, comp(ua.l[k][1], w), L[k]);
                H[k] = dp4a_us(hi, comp(ua.l[k][3], w), H[k]);
            }
        }
        uint32_t sc2, m2;
        kquant_scales_lane(hdr, lc, sc2, m2);
        return kquant_finish(hdr, sc2, m2, ua.s[0] * limb_combine(L), ua.s[2] * limb_combine(H), ua.x[0], ua.x[2]);
    }
};

template <> struct Unit<IB_Q5_K> {
    static __device__ __forceinline__ void init(uint32_t u, LaneConst &lc) {
        kquant_lane_init(u & 3, lc);
        lc.o0 = (u >> 2) * 176;
        lc.o1 = lc.o0 + 48 + 32 * lc.k;
        lc.o3 = 2 * lc.k;
    }
    static __device__ __forceinline__ float dot(uint32_t row, const LaneConst &lc, const UnitAct &ua) {
        const uint4 hdr = lds128(row + lc.o0), hA = lds128(row + lc.o0 + 16), hB = lds128(row + lc.o0 + 32);
        const uint4 q0 = lds128(row + lc.o1), q1 = lds128(row + lc.o1 + 16);
        const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const uint32_t hw[8] = {hA.x, hA.y, hA.z, hA.w, hB.x, hB.y, hB.z, hB.w};
        int L[3] = {0, 0, 0}, H[3] = {0, 0, 0};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t t = hw[i] >> lc.o3;  // bit 0 of each byte: fifth bit of the low-nibble element, bit 1: of the high-nibble element
            const uint32_t lo = (qw[i] & 0x0F0F0F0Fu) | ((t << 4) & 0x10101010u);
            const uint32_t hi = ((qw[i] >> 4) & 0x0F0F0F0Fu) | ((t << 3) & 0x10101010u);
#pragma unroll
            for (int k = 0; k < ACT_LIMBS; k++) {
                L[k] = dp4a_ss(lo, comp(ua.l[k][i >> 2], i & 3), L[k]);
                H[k] = dp4a_ss(hi, comp(ua.l[k][2 + (i >> 2)], i & 3), H[k]);
            }
        }
        uint32_t sc2, m2;
        kquant_scales_lane(hdr, lc, sc2, m2);
        return kquant_finish(hdr, sc2, m2, ua.s[0] * limb_combine(L), ua.s[2] * limb_combine(H), ua.x[0], ua.x[2]);
    }
};

// Q6_K rows are stored as groups of 8 blocks: [8 x 128 ql][8 x 64 qh][8 x 16 scales][8 x 2 d] = 1680 bytes per 2048 columns.
template <> struct Unit<IB_Q6_K> {
    static __device__ __forceinline__ void init(uint32_t u, LaneConst &lc) {
        const uint32_t b = u >> 2, i = (u >> 1) & 1, h = u & 1, grp = (b >> 3) * 1680, bb = b & 7;
        lc.o0 = grp + 128 * bb + 64 * i + 16 * h;
        lc.o1 = grp + 1024 + 64 * bb + 32 * i + 16 * h;
        lc.o2 = grp + 1536 + 16 * bb + 8 * i;
        lc.o3 = grp + 1664 + 2 * bb;
        lc.k = 8 * h;
        lc.ma = lc.mb = lc.mc = 0;
    }
    static __device__ __forceinline__ float dot(uint32_t row, const LaneConst &lc, const UnitAct &ua) {
        const uint4 qa = lds128(row + lc.o0), qb = lds128(row + lc.o0 + 32), qh = lds128(row + lc.o1);
        const uint2 scw = lds64(row + lc.o2);   // scales[8i .. 8i+7]
        const float d = h2f(lds16(row + lc.o3));
        const uint32_t la[4] = {qa.x, qa.y, qa.z, qa.w}, lb[4] = {qb.x, qb.y, qb.z, qb.w}, hh[4] = {qh.x, qh.y, qh.z, qh.w};
        int D[4][3] = {{0, 0, 0}, {0, 0, 0}, {0, 0, 0}, {0, 0, 0}};
#pragma unroll
        for (int w = 0; w < 4; w++) {
            // crates/inferi/src/quantization.rs:237-246: 4 low bits from ql, 2 high bits from qh
            const uint32_t g0 = (la[w] & 0x0F0F0F0Fu) | ((hh[w] << 4) & 0x30303030u);
            const uint32_t g1 = (lb[w] & 0x0F0F0F0Fu) | ((hh[w] << 2) & 0x30303030u);
            const uint32_t g2 = ((la[w] >> 4) & 0x0F0F0F0Fu) | (hh[w] & 0x30303030u);
            const uint32_t g3 = ((lb[w] >> 4) & 0x0F0F0F0Fu) | ((hh[w] >> 2) & 0x30303030u);
#pragma unroll
            for (int k = 0; k < ACT_LIMBS; k++) {
                D[0][k] = dp4a_ss(g0, comp(ua.l[k][0], w), D[0][k]);
                D[1][k] = dp4a_ss(g1, comp(ua.l[k][1], w), D[1][k]);
                D[2][k] = dp4a_ss(g2, comp(ua.l[k][2], w), D[2][k]);
                D[3][k] = dp4a_ss(g3, comp(ua.l[k][3], w), D[3][k]);
            }
        }
        // scale of group g is byte 2g + h of the 8 loaded: bytes {h, 2+h} of word x, {h, 2+h} of word y
        const uint32_t sx = scw.x >> lc.k, sy = scw.y >> lc.k;
        const float s0 = (float)(int)(int8_t)(sx & 0xFF), s1 = (float)(int)(int8_t)((sx >> 16) & 0xFF);
        const float s2 = (float)(int)(int8_t)(sy & 0xFF), s3 = (float)(int)(int8_t)((sy >> 16) & 0xFF);
        float v = s0 * (ua.s[0] * limb_combine(D[0]) - 32.0f * ua.x[0]);
        v += s1 * (ua.s[1] * limb_combine(D[1]) - 32.0f * ua.x[1]);
        v += s2 * (ua.s[2] * limb_combine(D[2]) - 32.0f * ua.x[2]);
        v += s3 * (ua.s[3] * limb_combine(D[3]) - 32.0f * ua.x[3]);
        return d * v;
    }
};

// Q8_0 rows are stored as groups of 8 blocks: [8 x 32 quants][8 x 2 scale] = 272 bytes per 256 columns.
template <> struct Unit<IB_Q8_0> {
    static __device__ __forceinline__ void init(uint32_t u, LaneConst &lc) {
        const uint32_t b0 = 2 * u, grp = (b0 >> 3) * 272, bb = b0 & 7;
        lc.o0 = grp + 32 * bb;
        lc.o1 = grp + 256 + 2 * bb;
        lc.o2 = lc.o3 = lc.k = lc.ma = lc.mb = lc.mc = 0;
    }
    static __device__ __forceinline__ float dot(uint32_t row, const LaneConst &lc, const UnitAct &ua) {
        const uint4 q[4] = {lds128(row + lc.o0), lds128(row + lc.o0 + 16), lds128(row + lc.o0 + 32), lds128(row + lc.o0 + 48)};
        const uint32_t dbits = lds32(row + lc.o1);   // f16 scales of the two blocks
        const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&dbits));
        int A[3] = {0, 0, 0}, B[3] = {0, 0, 0};   // block 2u (groups 0,1), block 2u+1 (groups 2,3)
#pragma unroll
        for (int g = 0; g < 4; g++)
#pragma unroll
            for (int w = 0; w < 4; w++)
#pragma unroll
                for (int k = 0; k < ACT_LIMBS; k++) {
                    if (g < 2) A[k] = dp4a_ss(comp(q[g], w), comp(ua.l[k][g], w), A[k]);
                    else B[k] = dp4a_ss(comp(q[g], w), comp(ua.l[k][g], w), B[k]);
                }
        return dd.x * (ua.s[0] * limb_combine(A)) + dd.y * (ua.s[2] * limb_combine(B));
    }
};

constexpr uint32_t QT_MIXED = 0xFFu;   // kernel instance for launches whose segments differ in format
constexpr uint32_t QT_Q4_Q6 = 0xFEu;   // ... and hold only Q4_K and Q6_K (q, k, v of the Q4_K_M recipe): two formats to switch between, not four

template <uint32_t QT>
__device__ __forceinline__ void unit_init(uint32_t qtype, uint32_t u, LaneConst &lc) {
    lc.o0 = lc.o1 = lc.o2 = lc.o3 = lc.k = lc.ma = lc.mb = lc.mc = 0;
    if (QT == QT_Q4_Q6) {
        if (qtype == IB_Q4_K) Unit<IB_Q4_K>::init(u, lc);
        else Unit<IB_Q6_K>::init(u, lc);
        return;
    }
    if (QT != QT_MIXED) { Unit<(QT == QT_MIXED || QT == QT_Q4_Q6) ? IB_Q4_K : QT>::init(u, lc); return; }
    switch (qtype) {
    case IB_Q4_K: Unit<IB_Q4_K>::init(u, lc); break;
    case IB_Q6_K: Unit<IB_Q6_K>::init(u, lc); break;
    case IB_Q5_K: Unit<IB_Q5_K>::init(u, lc); break;
    default: Unit<IB_Q8_0>::init(u, lc); break;
    }
}
template <uint32_t QT>
__device__ __forceinline__ float unit_dot(uint32_t qtype, uint32_t row, const LaneConst &lc, const UnitAct &ua) {
    if (QT == QT_Q4_Q6) return qtype == IB_Q4_K ? Unit<IB_Q4_K>::dot(row, lc, ua) : Unit<IB_Q6_K>::dot(row, lc, ua);
    if (QT != QT_MIXED) return Unit<(QT == QT_MIXED || QT == QT_Q4_Q6) ? IB_Q4_K : QT>::dot(row, lc, ua);
    switch (qtype) {
    case IB_Q4_K: return Unit<IB_Q4_K>::dot(row, lc, ua);
    case IB_Q6_K: return Unit<IB_Q6_K>::dot(row, lc, ua);
    case IB_Q5_K: return Unit<IB_Q5_K>::dot(row, lc, ua);
    default: return Unit<IB_Q8_0>::dot(row, lc, ua);
    }
}

// -------------------------------------------------------------------------------------------------
// Prologue of the streaming kernel, run by the 16 consumer warps: y = x * w -> limb form in
// shared memory.  The RMS factor is NOT applied here: it is one scalar for the whole vector, the GEMV is linear, so the
// epilogue warp multiplies the finished row sums by it.  That takes the sum-of-squares reduction off the consumers'
// critical path: every warp leaves its part of the sum in red[warp], arrives on `ss_bar` and carries on; only the
// epilogue warp waits there.
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ void pack_stream(uint8_t *smem, uint32_t cols, const float *__restrict__ x, const float *__restrict__ norm_w, float *red,
                                            uint32_t ss_bar, const float4 (&g)[4], uint32_t nq) {
    constexpr int NT = PACK_THREADS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t nruns = cols / 16;    // cols is a multiple of 64: runs pair up inside a warp; at most 2 * NT of them (cols <= 16384)
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    const float4 *w4 = reinterpret_cast<const float4 *>(norm_w);
    PackRegs r;
#pragma unroll
    for (int i = 0; i < PACK_RUNS; i++) {
        const uint32_t run = tid + NT * i;
#pragma unroll
        for (int j = 0; j < 4; j++) r.x[i][j] = run < nruns ? __ldcg(x4 + 4 * run + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (norm_w) {
        // crates/inferi-shaders/src/rms_norm.rs:112-120: the sum of squares; the factor itself is applied by the epilogue warp
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < PACK_RUNS; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) ss += (r.x[i][j].x * r.x[i][j].x + r.x[i][j].y * r.x[i][j].y) + (r.x[i][j].z * r.x[i][j].z + r.x[i][j].w * r.x[i][j].w);
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) {
            red[warp] = ss;
            mbar_arrive(ss_bar);   // a release: the epilogue warp's wait sees red[warp]
        }
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
                    v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w;
                }
            }
            pack_run(r.x[i], run, cols, smem, ok, nq);
        }
    }
    named_barrier(1, NT);
}

__device__ __forceinline__ float2 residual_prefetch(const float *resid, uint32_t pair) { return __ldcg(reinterpret_cast<const float2 *>(resid + 2 * pair)); }

// ---- epilogue of one row pair (run by the epilogue warp only, so the kind of epilogue is a run-time switch: one kernel
// instance per weight format serves every role in the token graph and stays in the instruction cache) ----
// `resid_pre`: the pair's residual values (EPI_RESIDUAL), fetched by the caller ahead of the wait for the dot products.
__device__ __forceinline__ void epilogue(const GemvParams &p, uint32_t s, uint32_t pair, float a, float b, unsigned long long &best, float2 resid_pre) {
    const uint32_t epi = p.epi;
    if (epi == EPI_SWIGLU) {
        // crates/inferi-shaders/src/silu.rs:16-19,46-52: a = gate row, b = up row
        p.seg[0].out[pair] = b * (a / (1.0f + expf(-a)));
        return;
    }
    const uint32_t r0 = 2 * pair;
    if (epi == EPI_STORE) {
        *reinterpret_cast<float2 *>(p.seg[s].out + r0) = make_float2(a, b);
    } else if (epi == EPI_RESIDUAL) {
        *reinterpret_cast<float2 *>(p.seg[s].out + r0) = make_float2(resid_pre.x + a, resid_pre.y + b);
    } else if (epi == EPI_QKV) {
        if (p.bias[s]) {
            const float2 bv = __ldg(reinterpret_cast<const float2 *>(p.bias[s] + r0));
            a += bv.x;
            b += bv.y;
        }
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
    } else if (epi == EPI_PUSH) {
        // row-split matrix of a tensor-parallel model: this rank's partial goes straight into every rank's memory
        // ({value, tag} words: see GemvParams)
        const uint32_t tag = (*p.epoch_ptr) * p.xchg_per_epoch + p.push_use;
        const uint4 w = make_uint4(__float_as_uint(a), tag, __float_as_uint(b), tag);
        for (uint32_t rk = 0; rk < p.tp; rk++) *reinterpret_cast<uint4 *>(p.push_dst[rk] + r0) = w;
    } else if (epi == EPI_ARGMAX) {
        if (p.seg[0].out) *reinterpret_cast<float2 *>(p.seg[0].out + r0) = make_float2(a, b);
        best = max(best, max(argmax_key(a, p.row_offset + r0), argmax_key(b, p.row_offset + r0 + 1)));
    }
}

}  // namespace ib
