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
//  * Sixteen consumer warps split a row's columns: every lane owns one 64-weight unit of the row and keeps that
//    unit's activations — three int8 limbs per column, see gemv_common.cuh — in registers for the whole kernel, so
//    the inner loop touches shared memory only for weights.  Per weight the work is a byte mask and dp4a.
//  * Per row the lane partials are shuffled down, per-warp partials meet in shared memory, and the last warp of a
//    row group to arrive adds them in a fixed order and runs the epilogue (store / residual add / SwiGLU /
//    RoPE + KV append / arg-max).  No warp ever waits for another one except through the ring.
// Every wait on an mbarrier is bounded; a wait that gives up raises the context's error word and carries on.
#include "gemv_common.cuh"

namespace ib {

constexpr int CW = 16;                          // consumer warps
constexpr int STREAM_THREADS = (CW + 1) * 32;   // + 1 producer warp
constexpr int PT_MAX = 16;                      // row pairs per tile
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // a wait on an mbarrier or on a peer gives up after 2 s

#ifdef IB_STREAM_TRACE
// Timeline probes for latency studies: globaltimer stamps of CTA 0 (and of the last CTA's end), one row of 16 slots
// per epilogue kind, read back with ib_debug_stream_trace().  Never compiled into the shipped library.
__device__ unsigned long long g_trace[16 * 16];
#define TRACE(slot)                                                                                   \
    do {                                                                                              \
        if (lane == 0 && blockIdx.x == 0 && (warp == 0 || warp == CW)) {                              \
            unsigned long long _t;                                                                    \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t));                                    \
            g_trace[(warp == CW ? 128 : 0) + EPI * 16 + (slot)] = _t;                                 \
        }                                                                                             \
        if (lane == 0 && blockIdx.x == gridDim.x - 1 && warp == 0 && (slot) == 15) {                  \
            unsigned long long _t;                                                                    \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t));                                    \
            g_trace[EPI * 16 + 14] = _t;                                                              \
        }                                                                                             \
    } while (0)
#else
#define TRACE(slot) do { } while (0)
#endif

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
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(2000u)   // suspend-time hint in ns: a waiting warp sleeps instead of spinning through issue slots
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
// ---- cross-GPU arrival counters (tensor parallel).  Counters only grow; a rank waits until its own counter has
// reached the value that the current use implies.  The wait is bounded like every other wait here. ----
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ bool wait_counter(const uint32_t *flag, uint32_t target, uint32_t *err, uint32_t code) {
    if ((int32_t)(ld_acquire_sys(flag) - target) >= 0) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if ((int32_t)(ld_acquire_sys(flag) - target) >= 0) return true;
        if (global_ns() - t0 > WAIT_LIMIT_NS) break;
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

template <uint32_t EPI>
__device__ __forceinline__ void make_share(const GemvParams &p, uint32_t stage_bytes, uint32_t RG, Share &sh) {
    uint32_t n0, n1 = 0, n2 = 0;
    sh.nseg = (EPI == EPI_SWIGLU) ? 1u : p.nseg;
    sh.c1 = sh.c2 = 16;
    if (EPI == EPI_SWIGLU) { n0 = p.seg[0].rows; sh.c0 = (uint32_t)(p.seg[0].row_bytes + p.seg[1].row_bytes); }
    else {
        n0 = p.seg[0].rows / 2; sh.c0 = (uint32_t)(2 * p.seg[0].row_bytes);
        if (sh.nseg > 1) { n1 = p.seg[1].rows / 2; sh.c1 = (uint32_t)(2 * p.seg[1].row_bytes); }
        if (sh.nseg > 2) { n2 = p.seg[2].rows / 2; sh.c2 = (uint32_t)(2 * p.seg[2].row_bytes); }
    }
    const uint32_t k0 = sh.c0 / 16, k1 = sh.c1 / 16, k2 = sh.c2 / 16;
    const uint32_t s1 = n0 * k0, s2 = s1 + n1 * k1, total = s2 + n2 * k2;
    const uint32_t G = gridDim.x, q = total / G, r = total % G;
    const uint32_t lo = q * blockIdx.x + r * blockIdx.x / G, hi = q * (blockIdx.x + 1) + r * (blockIdx.x + 1) / G;
    share_range(lo, hi, 0, k0, n0, sh.a0, sh.b0);
    share_range(lo, hi, s1, k1, n1, sh.a1, sh.b1);
    share_range(lo, hi, s2, k2, n2, sh.a2, sh.b2);
    sh.t0 = tile_pairs(stage_bytes, sh.c0, RG);
    sh.t1 = tile_pairs(stage_bytes, sh.c1, RG);
    sh.t2 = tile_pairs(stage_bytes, sh.c2, RG);
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
    // asm volatile loads: they must stay where they are.  As ordinary loads they are loop-invariant and the compiler
    // hoists the copies of every format's consumer loop to one place, where they all stay live at once.
#pragma unroll
    for (int g = 0; g < 4; g++) {
#pragma unroll
        for (int k = 0; k < 3; k++) {
            const uint32_t addr = smem_u32(A.limb(k) + e16[g]);
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(ua.l[k][g].x), "=r"(ua.l[k][g].y), "=r"(ua.l[k][g].z), "=r"(ua.l[k][g].w)
                         : "r"(addr)
                         : "memory");
        }
        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(ua.s[g]) : "r"(smem_u32(SC + (e16[g] >> 1))) : "memory");
        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(ua.x[g]) : "r"(smem_u32(SX + e16[g])) : "memory");
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

// One row (in shared memory) x one unit -> the lane's partial dot product.  Everything that depends only on the
// lane (byte offsets inside a row, shift amounts) is computed once in init().
struct LaneConst { uint32_t o0, o1, o2, o3, k; };
template <uint32_t QT> struct Unit;

template <> struct Unit<IB_Q4_K> {
    static __device__ __forceinline__ void init(uint32_t u, LaneConst &lc) { lc.k = u & 3; lc.o0 = (u >> 2) * 144; lc.o1 = lc.o0 + 16 + 32 * lc.k; }
    static __device__ __forceinline__ float dot(const uint8_t *row, const LaneConst &lc, const UnitAct &ua) {
        const uint32_t off_hdr = lc.o0, off_q = lc.o1, c = lc.k;
        const uint4 hdr = *reinterpret_cast<const uint4 *>(row + off_hdr);
        const uint4 q0 = *reinterpret_cast<const uint4 *>(row + off_q);
        const uint4 q1 = *reinterpret_cast<const uint4 *>(row + off_q + 16);
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
        const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
        // groups 0,1 (and 2,3) share the activation scale and the sub-block scale: add them as integers
        const float lo = ua.s[0] * limb_combine(D[0][0] + D[1][0], D[0][1] + D[1][1], D[0][2] + D[1][2]);
        const float hi = ua.s[2] * limb_combine(D[2][0] + D[3][0], D[2][1] + D[3][1], D[2][2] + D[3][2]);
        return (dm.x * (float)(sc2 & 0xFFu)) * lo - (dm.y * (float)(m2 & 0xFFu)) * (ua.x[0] + ua.x[1]) + (dm.x * (float)(sc2 >> 8)) * hi -
               (dm.y * (float)(m2 >> 8)) * (ua.x[2] + ua.x[3]);
    }
};

template <> struct Unit<IB_Q5_K> {
    static __device__ __forceinline__ void init(uint32_t u, LaneConst &lc) { lc.k = u & 3; lc.o0 = (u >> 2) * 176; lc.o1 = lc.o0 + 48 + 32 * lc.k; }
    static __device__ __forceinline__ float dot(const uint8_t *row, const LaneConst &lc, const UnitAct &ua) {
        const uint32_t off_hdr = lc.o0, off_q = lc.o1, c = lc.k;
        const uint4 hdr = *reinterpret_cast<const uint4 *>(row + off_hdr);
        const uint4 hA = *reinterpret_cast<const uint4 *>(row + off_hdr + 16), hB = *reinterpret_cast<const uint4 *>(row + off_hdr + 32);
        const uint4 q0 = *reinterpret_cast<const uint4 *>(row + off_q), q1 = *reinterpret_cast<const uint4 *>(row + off_q + 16);
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
        const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
        const float lo_f = ua.s[0] * limb_combine(D[0][0] + D[1][0], D[0][1] + D[1][1], D[0][2] + D[1][2]);
        const float hi_f = ua.s[2] * limb_combine(D[2][0] + D[3][0], D[2][1] + D[3][1], D[2][2] + D[3][2]);
        return (dm.x * (float)(sc2 & 0xFFu)) * lo_f - (dm.y * (float)(m2 & 0xFFu)) * (ua.x[0] + ua.x[1]) + (dm.x * (float)(sc2 >> 8)) * hi_f -
               (dm.y * (float)(m2 >> 8)) * (ua.x[2] + ua.x[3]);
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
    }
    static __device__ __forceinline__ float dot(const uint8_t *row, const LaneConst &lc, const UnitAct &ua) {
        const uint32_t off_qa = lc.o0, off_qh = lc.o1, off_sc = lc.o2, off_d = lc.o3, sh = lc.k;
        const uint4 qa = *reinterpret_cast<const uint4 *>(row + off_qa);
        const uint4 qb = *reinterpret_cast<const uint4 *>(row + off_qa + 32);
        const uint4 qh = *reinterpret_cast<const uint4 *>(row + off_qh);
        const uint2 scw = *reinterpret_cast<const uint2 *>(row + off_sc);   // scales[8i .. 8i+7]
        const float d = h2f(*reinterpret_cast<const unsigned short *>(row + off_d));
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
        // scale of group g is byte 2g + h of the 8 loaded: bytes {h, 2+h} of word x, {h, 2+h} of word y
        const uint32_t sx = scw.x >> sh, sy = scw.y >> sh;
        const float s0 = (float)(int)(int8_t)(sx & 0xFF), s1 = (float)(int)(int8_t)((sx >> 16) & 0xFF);
        const float s2 = (float)(int)(int8_t)(sy & 0xFF), s3 = (float)(int)(int8_t)((sy >> 16) & 0xFF);
        float v = s0 * (ua.s[0] * limb_combine(D[0][0], D[0][1], D[0][2]) - 32.0f * ua.x[0]);
        v += s1 * (ua.s[1] * limb_combine(D[1][0], D[1][1], D[1][2]) - 32.0f * ua.x[1]);
        v += s2 * (ua.s[2] * limb_combine(D[2][0], D[2][1], D[2][2]) - 32.0f * ua.x[2]);
        v += s3 * (ua.s[3] * limb_combine(D[3][0], D[3][1], D[3][2]) - 32.0f * ua.x[3]);
        return d * v;
    }
};

// Q8_0 rows are stored as groups of 8 blocks: [8 x 32 quants][8 x 2 scale] = 272 bytes per 256 columns.
template <> struct Unit<IB_Q8_0> {
    static __device__ __forceinline__ void init(uint32_t u, LaneConst &lc) {
        const uint32_t b0 = 2 * u, grp = (b0 >> 3) * 272, bb = b0 & 7;
        lc.o0 = grp + 32 * bb;
        lc.o1 = grp + 256 + 2 * bb;
    }
    static __device__ __forceinline__ float dot(const uint8_t *row, const LaneConst &lc, const UnitAct &ua) {
        const uint32_t off_q = lc.o0, off_d = lc.o1;
        const uint4 q0 = *reinterpret_cast<const uint4 *>(row + off_q), q1 = *reinterpret_cast<const uint4 *>(row + off_q + 16);
        const uint4 q2 = *reinterpret_cast<const uint4 *>(row + off_q + 32), q3 = *reinterpret_cast<const uint4 *>(row + off_q + 48);
        const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(row + off_d));   // scales of the two blocks
        int D[4][3];
#pragma unroll
        for (int k = 0; k < 3; k++) {
            D[0][k] = dot4_ss(q0, ua.l[k][0], 0);
            D[1][k] = dot4_ss(q1, ua.l[k][1], 0);
            D[2][k] = dot4_ss(q2, ua.l[k][2], 0);
            D[3][k] = dot4_ss(q3, ua.l[k][3], 0);
        }
        const float a = ua.s[0] * limb_combine(D[0][0] + D[1][0], D[0][1] + D[1][1], D[0][2] + D[1][2]);
        const float c = ua.s[2] * limb_combine(D[2][0] + D[3][0], D[2][1] + D[3][1], D[2][2] + D[3][2]);
        return dd.x * a + dd.y * c;
    }
};

constexpr uint32_t QT_MIXED = 0xFFu;   // kernel instance for launches whose segments differ in format

template <uint32_t QT>
__device__ __forceinline__ void unit_init(uint32_t qtype, uint32_t u, LaneConst &lc) {
    lc.o0 = lc.o1 = lc.o2 = lc.o3 = lc.k = 0;
    if (QT != QT_MIXED) { Unit<QT == QT_MIXED ? IB_Q4_K : QT>::init(u, lc); return; }
    switch (qtype) {
    case IB_Q4_K: Unit<IB_Q4_K>::init(u, lc); break;
    case IB_Q6_K: Unit<IB_Q6_K>::init(u, lc); break;
    case IB_Q5_K: Unit<IB_Q5_K>::init(u, lc); break;
    default: Unit<IB_Q8_0>::init(u, lc); break;
    }
}
template <uint32_t QT>
__device__ __forceinline__ float unit_dot(uint32_t qtype, const uint8_t *row, const LaneConst &lc, const UnitAct &ua) {
    if (QT != QT_MIXED) return Unit<QT == QT_MIXED ? IB_Q4_K : QT>::dot(row, lc, ua);
    switch (qtype) {
    case IB_Q4_K: return Unit<IB_Q4_K>::dot(row, lc, ua);
    case IB_Q6_K: return Unit<IB_Q6_K>::dot(row, lc, ua);
    case IB_Q5_K: return Unit<IB_Q5_K>::dot(row, lc, ua);
    default: return Unit<IB_Q8_0>::dot(row, lc, ua);
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
    } else if (EPI == EPI_PUSH) {
        // row-split matrix of a tensor-parallel model: this rank's partial goes straight into every rank's memory
        for (uint32_t rk = 0; rk < p.tp; rk++) *reinterpret_cast<float2 *>(p.push_dst[rk] + r0) = make_float2(a, b);
    } else if (EPI == EPI_ARGMAX) {
        if (p.seg[0].out) *reinterpret_cast<float2 *>(p.seg[0].out + r0) = make_float2(a, b);
        best = max(best, max(argmax_key(a, p.row_offset + r0), argmax_key(b, p.row_offset + r0 + 1)));
    }
}

// ---- consumer side ----
struct Consumer {
    const uint8_t *ring;
    float *part;          // [stages][PT_MAX][2][CW] per-warp column partials
    uint32_t *cnt;        // [stages][CW] arrivals of a row group's warps
    uint32_t bar0, S, stage_bytes;
    uint32_t CG, RG, cg, rg, u;
    bool has_unit;
    int lane;
};

// Consumes this warp's share of every tile.  One loop for all formats (the format switch sits at the dot product):
// separate inlined loops per format made the register allocator spill.
template <uint32_t EPI, uint32_t QT>
__device__ __forceinline__ void consume_tiles(const GemvParams &p, const Share &sh, const Consumer &c, const Act &A, unsigned long long &best) {
    const int lane = c.lane;
    UnitAct ua;
    LaneConst lc;
    uint32_t cur_type = 0xFFFFFFFFu;
    const uint32_t S = c.S, CG = c.CG, RG = c.RG;
    TileCursor tc;
    tc.init(sh);
#pragma unroll 1
    for (uint32_t k = 0; tc.valid(sh); k++, tc.advance(sh)) {
        const uint32_t st = k % S, s = tc.seg, n = tc.count(sh);
        const uint32_t qtype = (QT != QT_MIXED) ? QT : p.seg[s].qtype;
        if (qtype != cur_type) {   // (re)load this lane's activations in the layout of the segment's format
            unit_init<QT>(qtype, c.u, lc);
            if (c.has_unit) load_unit_act(qtype, c.u, A, ua);
            cur_type = qtype;
        }
        if (!mbar_wait(c.bar0 + 8 * st, (k / S) & 1, p.err, 1)) return;   // the error word is raised; give up on this CTA's rows
        const uint8_t *tile = c.ring + (size_t)st * c.stage_bytes;
        const uint32_t rbA = (uint32_t)p.seg[s].row_bytes;
        const uint32_t rbB = (EPI == EPI_SWIGLU) ? (uint32_t)p.seg[1].row_bytes : rbA;
        const uint32_t strideA = (EPI == EPI_SWIGLU) ? rbA : 2 * rbA, offB = (EPI == EPI_SWIGLU) ? n * rbA : rbA;
        float *pt = c.part + (size_t)st * PT_MAX * 2 * CW;
        for (uint32_t pr = c.rg; pr < n; pr += RG) {
            const uint8_t *rowA = tile + pr * strideA;
            const uint8_t *rowB = (EPI == EPI_SWIGLU) ? tile + offB + pr * rbB : rowA + rbA;
            float va = 0.f, vb = 0.f;
            if (c.has_unit) {
                va = unit_dot<QT>(qtype, rowA, lc, ua);
                vb = unit_dot<QT>(qtype, rowB, lc, ua);
            }
#pragma unroll
            for (int o = 16; o; o >>= 1) {
                va += __shfl_xor_sync(0xffffffffu, va, o);
                vb += __shfl_xor_sync(0xffffffffu, vb, o);
            }
            if (CG == 1) {
                if (lane == 0) epilogue<EPI>(p, s, tc.next + pr, va, vb, best);
            } else if (lane == 0) {
                pt[(pr * 2 + 0) * CW + c.cg] = va;
                pt[(pr * 2 + 1) * CW + c.cg] = vb;
            }
        }
        if (CG > 1) {
            // the last warp of the row group to finish the tile folds the column partials in a fixed order
            uint32_t last = 0;
            if (lane == 0) {
                __threadfence_block();
                last = (atomicAdd(c.cnt + st * CW + c.rg, 1u) == CG - 1) ? 1u : 0u;
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                __threadfence_block();
                const uint32_t pr = c.rg + RG * lane;
                if (pr < n) {
                    float va = 0.f, vb = 0.f;
                    for (uint32_t g = 0; g < CG; g++) {
                        va += pt[(pr * 2 + 0) * CW + g];
                        vb += pt[(pr * 2 + 1) * CW + g];
                    }
                    epilogue<EPI>(p, s, tc.next + pr, va, vb, best);
                }
                __syncwarp();
                if (lane == 0) c.cnt[st * CW + c.rg] = 0;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(c.bar0 + 8 * (S + st));   // this warp is done with the stage
    }
}

// ---- the kernel ----
template <uint32_t EPI, uint32_t QT>
__global__ void __launch_bounds__(STREAM_THREADS, 1) gemv_stream_kernel(const GemvParams p, const StreamGeom geo) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float red[PACK_THREADS / 32 + 1];
    __shared__ unsigned long long best_sm[CW];
    __shared__ bool is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    TRACE(0);

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
    make_share<EPI>(p, geo.stage_bytes, RG, sh);


    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; s++) {
            mbar_init(bar0 + 8 * s, 1);                 // full: the producer's expect_tx arrival
            mbar_init(bar0 + 8 * (S + s), active);      // empty: one arrival per working consumer warp
        }
        for (uint32_t i = 0; i < S * CW; i++) cnt[i] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    TRACE(1);
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
                    const uint32_t bytes = n * sh.cost(s);
                    mbar_expect_tx(full, bytes);
                    bulk_g2s(dst, p.seg[s].w + (size_t)tc.next * sh.cost(s), bytes, full);
                }
                TRACE(2 + (k < 6 ? k : 6));
            }
        }
        return;
    }

    // ================= consumer warps =================
    float4 norm_g[4];
    pack_prefetch_norm(p.norm_w, p.cols, norm_g);   // weights: fetched while the previous kernel is still running
    if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    TRACE(2);
    PackReduce rd{nullptr, 0, nullptr};
    if (p.reduce_src) {
        // every rank's partial sums of the previous row-split GEMV must have landed in this rank's slots
        if (threadIdx.x == 0) wait_counter(p.reduce_flag, ((*p.epoch_ptr) * p.reduce_per_epoch + p.reduce_use) * p.tp, p.err, 3);
        named_barrier(1, PACK_THREADS);
        rd = PackReduce{p.reduce_src, p.tp, p.x_out};
    }
    pack_activation(act_sm, p.cols, p.x, p.norm_w, p.eps, red, norm_g, rd);
    const Act A{act_sm, p.cols};
    TRACE(3);

    unsigned long long best = 0ull;
    if ((uint32_t)warp < active) {
        Consumer c;
        c.ring = ring; c.part = part; c.cnt = cnt; c.bar0 = bar0; c.S = S; c.stage_bytes = geo.stage_bytes;
        c.CG = CG; c.RG = RG; c.cg = warp % CG; c.rg = warp / CG; c.u = c.cg * 32 + lane; c.has_unit = c.u < units; c.lane = lane;
        consume_tiles<EPI, QT>(p, sh, c, A, best);
    }
    TRACE(15);

    if (EPI == EPI_PUSH) {
        // all of this CTA's peer stores are out; the last CTA of the grid tells every rank that this rank has delivered
        __threadfence_system();
        named_barrier(1, PACK_THREADS);
        if (threadIdx.x == 0) {
            if (atomicAdd(p.push_done, 1u) == gridDim.x - 1) {
                *p.push_done = 0u;
                __threadfence_system();
                for (uint32_t rk = 0; rk < p.tp; rk++) atomicAdd_system(p.push_flag[rk], 1u);
            }
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
                if (p.tp > 1) {
                    // sharded vocabulary: every rank gets this rank's candidate; the end-of-token kernel folds them
                    for (uint32_t rk = 0; rk < p.tp; rk++) *p.amax_dst[rk] = b;
                    __threadfence_system();
                    for (uint32_t rk = 0; rk < p.tp; rk++) atomicAdd_system(p.amax_flag[rk], 1u);
                }
            }
        }
    }
}

// -------------------------------------------------------------------------------------------------
// host side
// -------------------------------------------------------------------------------------------------
constexpr size_t STREAM_SMEM_BUDGET = 200 * 1024;   // one CTA per SM

bool gemv_stream_eligible(const GemvParams &p) {
    if (p.cols % 64 || p.cols > 16384) return false;
    for (uint32_t s = 0; s < p.nseg; s++) {
        const uint32_t q = p.seg[s].qtype;
        if (q != IB_Q4_K && q != IB_Q5_K && q != IB_Q6_K && q != IB_Q8_0) return false;
        if (p.seg[s].row_bytes % 16) return false;
    }
    return true;
}

template <uint32_t EPI, uint32_t QT>
static int32_t launch_stream_inst(ib_ctx *ctx, cudaStream_t stream, const GemvParams &p, int grid, const StreamGeom &geo, size_t smem) {
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        IB_CHECK_CUDA(cudaFuncSetAttribute(gemv_stream_kernel<EPI, QT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)STREAM_SMEM_BUDGET));
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
    IB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, gemv_stream_kernel<EPI, QT>, p, geo));
    ctx->launches++;
    return IB_OK;
}

template <uint32_t EPI>
static int32_t launch_stream_epi(ib_ctx *ctx, cudaStream_t stream, const GemvParams &p, int grid, const StreamGeom &geo, size_t smem) {
    uint32_t qt = p.seg[0].qtype;
    for (uint32_t s = 1; s < p.nseg; s++)
        if (p.seg[s].qtype != qt) qt = QT_MIXED;
    switch (qt) {
    case IB_Q4_K: return launch_stream_inst<EPI, IB_Q4_K>(ctx, stream, p, grid, geo, smem);
    case IB_Q6_K: return launch_stream_inst<EPI, IB_Q6_K>(ctx, stream, p, grid, geo, smem);
    case IB_Q5_K: return launch_stream_inst<EPI, IB_Q5_K>(ctx, stream, p, grid, geo, smem);
    case IB_Q8_0: return launch_stream_inst<EPI, IB_Q8_0>(ctx, stream, p, grid, geo, smem);
    default: return launch_stream_inst<EPI, QT_MIXED>(ctx, stream, p, grid, geo, smem);
    }
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
    // tile = whole "rounds" of the row groups (RG pairs each): two rounds when they fit in ~37 KB, so that the
    // per-tile hand-offs are paid once per two pairs of a warp; at least two stages must fit beside the activations
    const uint32_t units = p.cols / 64, CG = (units + 31) / 32, RG = CW / CG;
    const size_t act = (act_smem_bytes(p.cols) + 127) & ~(size_t)127;
    auto layout = [&](uint32_t max_tile_bytes, uint32_t &stage, uint32_t &S, size_t &total) {
        auto pairs_per_tile = [&](uint32_t cost) {
            uint32_t pt = RG;
            while (pt * 2 <= PT_MAX && pt * 2 * cost <= max_tile_bytes) pt *= 2;
            while (pt > 1 && pt * cost > max_tile_bytes) pt--;
            return pt;
        };
        stage = 0;
        if (p.epi == EPI_SWIGLU) stage = pairs_per_tile(max_cost) * max_cost;
        else
            for (uint32_t s = 0; s < p.nseg; s++) {
                const uint32_t c = (uint32_t)(2 * p.seg[s].row_bytes);
                const uint32_t b = pairs_per_tile(c) * c;
                if (b > stage) stage = b;
            }
        stage = (stage + 127) & ~127u;
        for (S = 4;; S--) {
            const size_t part = (size_t)S * PT_MAX * 2 * CW * 4 + (size_t)S * CW * 4;
            total = (size_t)S * stage + act + ((part + 127) & ~(size_t)127) + 2 * S * 8;
            if (total <= STREAM_SMEM_BUDGET || S == 2) break;
        }
        return total <= STREAM_SMEM_BUDGET;
    };
    uint32_t stage = 0, S = 0;
    size_t total = 0;
    if (!layout(75776, stage, S, total) && !layout(49152, stage, S, total) && !layout(32768, stage, S, total) && !layout(max_cost, stage, S, total))
        return set_error(IB_ERR_UNSUPPORTED, "gemv: a row pair of %u bytes with %u columns does not fit the streaming kernel's ring", max_cost, p.cols);
    StreamGeom geo;
    geo.stages = S;
    geo.stage_bytes = stage;
    geo.act_off = S * stage;
    geo.part_off = (uint32_t)(geo.act_off + act);
    geo.bar_off = (uint32_t)(geo.part_off + (((size_t)S * PT_MAX * 2 * CW * 4 + (size_t)S * CW * 4 + 127) & ~(size_t)127));
    int grid = ctx->sm_count;       // one persistent CTA per SM: 16 consumer warps hide the latency of the dependent dp4a / shuffle chains
    if ((uint32_t)grid > pairs) grid = (int)pairs;
    if (grid < 1) grid = 1;
    switch (p.epi) {
    case EPI_STORE: return launch_stream_epi<EPI_STORE>(ctx, stream, p, grid, geo, total);
    case EPI_RESIDUAL: return launch_stream_epi<EPI_RESIDUAL>(ctx, stream, p, grid, geo, total);
    case EPI_SWIGLU: return launch_stream_epi<EPI_SWIGLU>(ctx, stream, p, grid, geo, total);
    case EPI_QKV: return launch_stream_epi<EPI_QKV>(ctx, stream, p, grid, geo, total);
    case EPI_ARGMAX: return launch_stream_epi<EPI_ARGMAX>(ctx, stream, p, grid, geo, total);
    case EPI_PUSH: return launch_stream_epi<EPI_PUSH>(ctx, stream, p, grid, geo, total);
    default: return set_error(IB_ERR_INVALID, "gemv: unknown epilogue %u", p.epi);
    }
}

#ifdef IB_STREAM_TRACE
extern "C" __attribute__((visibility("default"))) int32_t ib_debug_stream_trace(unsigned long long *out64) {
    return cudaMemcpyFromSymbol(out64, g_trace, sizeof(unsigned long long) * 256) == cudaSuccess ? 0 : 2;
}
#endif

}  // namespace ib
