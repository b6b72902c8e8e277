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
#include "gemv_stream.cuh"

#include <stdlib.h>

namespace ib {

#ifdef IB_STREAM_TRACE
// Timeline probes for latency studies: globaltimer stamps of CTA 0 (and of the last CTA's end), one row of 16 slots
// per epilogue kind, read back with ib_debug_stream_trace().  Never compiled into the shipped library.
__device__ unsigned long long g_trace[16 * 16];
__device__ unsigned long long g_cta_end[8][160], g_cta_packed[8][160];   // per CTA: end of the kernel / activations packed
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
#define TRACE_CTA(arr)                                                                                \
    do {                                                                                              \
        if (lane == 0 && warp == 0 && blockIdx.x < 160) arr[EPI][blockIdx.x] = global_ns();           \
    } while (0)
// Where a consumer warp of CTA 0 spends its cycles, per epilogue kind: [wait for the tile, dot products, shuffle tree,
// partials / direct epilogue, cross-warp fold, slot release, tiles, total, loop bookkeeping before the wait]
__device__ long long g_phase[8][32][10];
#define PH_DECL long long _pc[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0}; long long _t0 = clock64(); const long long _tb = _t0
#define PH_MARK(i, dep)                                                                       \
    do {                                                                                      \
        long long _t;                                                                         \
        asm volatile("mov.u64 %0, %%clock64;" : "=l"(_t) : "f"(dep) : "memory");             \
        _pc[i] += _t - _t0;                                                                   \
        _t0 = _t;                                                                             \
    } while (0)
#define PH_DUMP(warp_id)                                                                      \
    do {                                                                                      \
        if (lane == 0 && blockIdx.x == 0) {                                                   \
            _pc[7] = clock64() - _tb;                                                         \
            for (int _i = 0; _i < 10; _i++) g_phase[EPI][warp_id][_i] = _pc[_i];               \
        }                                                                                     \
    } while (0)
#else
#define TRACE(slot) do { } while (0)
#define TRACE_CTA(arr) do { } while (0)
#define PH_DECL do { } while (0)
#define PH_MARK(i, dep) do { } while (0)
#define PH_DUMP(warp_id) do { } while (0)
#endif

#ifndef IB_COPY_PIECE_BYTES
#define IB_COPY_PIECE_BYTES (1u << 24)   // larger than any tile: one bulk copy per tile part
#endif
constexpr uint32_t COPY_PIECE = IB_COPY_PIECE_BYTES;   // a multiple of 16; 32 x COPY_PIECE must fit 32 bits
static_assert(COPY_PIECE % 16 == 0 && COPY_PIECE <= (1u << 26), "piece size");

struct StreamGeom {
    uint32_t stages, stage_bytes, act_off, part_off, bar_off;
    // the launch's tiles in hand-out order: per segment the pairs, the pairs per tile and the tiles; bytes per pair
    uint32_t seg_pairs[3], seg_pt[3], seg_tiles[3], seg_cost[3], total_tiles, meta_off;
    uint32_t dynamic;   // 1: tiles are claimed from a counter; 0: every CTA streams its own byte-balanced range of pairs
    uint32_t head_per_cta, head_tiles, tail_pt;   // counter hand-out: see tile_of
};

// Counter hand-out (one segment only): tile number -> (segment 0, first pair, pairs); pairs == 0 past the last tile.
// The first `head_tiles` tiles hold `seg_pt[0]` pairs each and belong to the CTAs by position (CTA b: tiles b * head_per_cta
// ...); the rest of the pairs follow as smaller tiles of `tail_pt` pairs, claimed from the counter.
__device__ __forceinline__ uint4 tile_of(const StreamGeom &g, uint32_t t) {
    const uint32_t np = g.seg_pairs[0];
    uint32_t first, pt;
    if (t < g.head_tiles) { pt = g.seg_pt[0]; first = t * pt; }
    else { pt = g.tail_pt; first = g.head_tiles * g.seg_pt[0] + (t - g.head_tiles) * pt; }
    if (first >= np) return make_uint4(0, 0, 0, 0);
    return make_uint4(0, first, (np - first) < pt ? (np - first) : pt, 0);
}

// ---- consumer side ----
struct Consumer {
    const uint8_t *ring;
    float *part;          // [stages][PT_MAX][2][CW] per-warp column partials
    uint32_t fold0;       // mbarriers [stages][CW]: the other warps of a row group have left their partials of the tile
    const uint4 *meta;    // [stages] (segment, first pair, pairs, -) of the tile in the slot, written by the producer
    uint32_t bar0, S, stage_bytes;
    uint32_t CG, RG, cg, rg, u;
    bool has_unit;
    int lane;
};

// Consumes this warp's share of every tile.  One loop for all formats (the format switch sits at the dot product):
// separate inlined loops per format made the register allocator spill.
template <uint32_t EPI, uint32_t QT>
__device__ __forceinline__ void consume_tiles(const GemvParams &p, const Consumer &c, const Act &A, unsigned long long &best) {
    const int lane = c.lane;
    UnitAct ua;
    LaneConst lc;
    uint32_t cur_type = 0xFFFFFFFFu;
    const uint32_t S = c.S, CG = c.CG, RG = c.RG;
    PH_DECL;
    // stage and phase parity of the tile, and the warp of the row group that folds it (they take turns), kept as counters:
    // a division by a run-time value per tile is a chain of ~200 cycles that nothing overlaps
    uint32_t st = 0, par = 0, folder = c.rg % CG;
#pragma unroll 1
    for (;; st = (st + 1 == S) ? 0 : st + 1, par ^= (st == 0) ? 1u : 0u, folder = (folder + 1 == CG) ? 0 : folder + 1) {
        PH_MARK(8, 0.f);   // loop bookkeeping since the slot release
        if (!mbar_wait(c.bar0 + 8 * st, par, p.err, 1)) return;   // the error word is raised; give up on this CTA's rows
        PH_MARK(0, 0.f);
        // which tile the producer put into the slot (tiles are handed out through a counter: a CTA that starts late or
        // runs slowly takes fewer of them); no pairs = no tiles left
        const uint4 tm = c.meta[st];
        const uint32_t s = tm.x, first_pair = tm.y, n = tm.z;
        if (n == 0) break;
        const uint32_t qtype = (QT != QT_MIXED && QT != QT_Q4_Q6) ? QT : p.seg[s].qtype;
        if (qtype != cur_type) {   // (re)load this lane's activations in the layout of the segment's format
            unit_init<QT>(qtype, c.u, lc);
            if (c.has_unit) load_unit_act(qtype, c.u, A, ua);
            cur_type = qtype;
        }
        const uint8_t *tile = c.ring + (size_t)st * c.stage_bytes;
        const uint32_t rbA = (uint32_t)p.seg[s].row_bytes;
        const uint32_t rbB = (EPI == EPI_SWIGLU) ? (uint32_t)p.seg[1].row_bytes : rbA;
        const uint32_t strideA = (EPI == EPI_SWIGLU) ? rbA : 2 * rbA, offB = (EPI == EPI_SWIGLU) ? n * rbA : rbA;
        float *pt = c.part + (size_t)st * PT_MAX * 2 * CW;
        // residual values of the pair this lane has to finish (CG > 1: in the warp that folds this tile; CG == 1: lane 0 of
        // each pair's warp, fetched per pair below): requested now, needed after the dot products
        float2 rpre = make_float2(0.f, 0.f);
        if (EPI == EPI_RESIDUAL && CG > 1 && c.cg == folder && c.rg + RG * lane < n) rpre = residual_prefetch(p.resid, first_pair + c.rg + RG * lane);
        for (uint32_t pr = c.rg; pr < n; pr += RG) {
            const uint8_t *rowA = tile + pr * strideA;
            const uint8_t *rowB = (EPI == EPI_SWIGLU) ? tile + offB + pr * rbB : rowA + rbA;
            if (EPI == EPI_RESIDUAL && CG == 1 && lane == 0) rpre = residual_prefetch(p.resid, first_pair + pr);
            float va = 0.f, vb = 0.f;
            if (c.has_unit) {
                va = unit_dot<QT>(qtype, rowA, lc, ua);
                vb = unit_dot<QT>(qtype, rowB, lc, ua);
            }
            PH_MARK(1, va + vb);
            {
                // one shuffle tree for both rows: after the first exchange the upper half-warp carries row B
                // (the same pairs are added in the same order as two separate trees would: the bits do not change)
                const bool up = lane & 16;
                float v = (up ? vb : va) + __shfl_xor_sync(0xffffffffu, up ? va : vb, 16);
#pragma unroll
                for (int o = 8; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (CG == 1) {
                    va = __shfl_sync(0xffffffffu, v, 0);
                    vb = __shfl_sync(0xffffffffu, v, 16);
                } else if ((lane & 15) == 0) {
                    pt[(pr * 2 + (lane >> 4)) * CW + c.cg] = v;   // lane 0 holds row A's sum, lane 16 row B's
                }
            }
            PH_MARK(2, va + vb);
            if (CG == 1 && lane == 0) epilogue<EPI>(p, s, first_pair + pr, va, vb, best, ParamCaches{p}, rpre);
            PH_MARK(3, 0.f);
        }
        if (CG > 1) {
            // The row group's warps take turns folding a tile.  The others leave their partials and arrive on the tile's
            // fold barrier (a release) without waiting; the folding warp waits for their CG - 1 arrivals (an acquire), adds
            // the column partials in a fixed order and runs the epilogue.
            const uint32_t fb = c.fold0 + 8 * (st * CW + c.rg);
            if (c.cg != folder) {
                __syncwarp();   // lane 16's partials are ordered before lane 0's arrival (a release)
                if (lane == 0) mbar_arrive(fb);
            } else {
                __syncwarp();   // lane 0's own partials, read by the other lanes below
                if (!mbar_wait(fb, par, p.err, 5)) return;
                const uint32_t pr = c.rg + RG * lane;
                if (pr < n) {
                    float va = 0.f, vb = 0.f;
                    for (uint32_t g = 0; g < CG; g++) {
                        va += pt[(pr * 2 + 0) * CW + g];
                        vb += pt[(pr * 2 + 1) * CW + g];
                    }
                    epilogue<EPI>(p, s, first_pair + pr, va, vb, best, ParamCaches{p}, rpre);
                }
            }
        }
        __syncwarp();
        PH_MARK(4, 0.f);
        if (lane == 0) mbar_arrive(c.bar0 + 8 * (S + st));   // this warp is done with the stage
        PH_MARK(5, 0.f);
#ifdef IB_STREAM_TRACE
        _pc[6] += 1;
#endif
    }
    PH_DUMP(c.cg + c.rg * c.CG);
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
    const uint32_t fold0 = smem_u32(part + geo.stages * PT_MAX * 2 * CW);                // mbarriers [stages][CW]
    const uint32_t bar0 = smem_u32(smem + geo.bar_off);                         // full[stages], empty[stages]
    const uint32_t S = geo.stages;

    const uint32_t units = p.cols / 64;
    const uint32_t CG = (units + 31) / 32;       // warps that split one row's columns
    const uint32_t RG = CW / CG;                 // row groups working side by side
    const uint32_t active = CG * RG;             // consumer warps with work


    // set-up spread over threads: it sits on the critical path of a CTA that starts late (its SM was the last to be freed)
    if (threadIdx.x < 2 * S) {
        // full[s]: the producer's expect_tx arrival; empty[s]: one arrival per working consumer warp
        mbar_init(bar0 + 8 * threadIdx.x, threadIdx.x < S ? 1u : active);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    } else if (threadIdx.x >= 32 && threadIdx.x < 32 + S * CW) {
        // fold barrier of (stage, row group): the arrivals of the row group's warps other than the folding one
        mbar_init(fold0 + 8 * (threadIdx.x - 32), CG > 1 ? CG - 1 : 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    TRACE(1);
    if (p.pdl) asm volatile("griddepcontrol.launch_dependents;");

    if (warp == CW) {
        // ================= producer warp: picks tiles and streams them =================
        // With many tiles per CTA they are handed out through a counter in global memory, so that a CTA which starts late
        // (its SM was the last to be freed by the previous kernel) or runs slowly takes fewer of them.  With few tiles per
        // CTA a tile is too coarse a unit for that: every CTA then streams its own byte-balanced range of row pairs, cut
        // into tiles.  Either way the slot's descriptor tells the consumers what the tile is.  Lane 0 picks, waits for the
        // slot and announces the tile; the copy is issued as pieces of at most COPY_PIECE bytes, one lane each.
        uint4 *meta = reinterpret_cast<uint4 *>(smem + geo.meta_off);
        const bool dyn = geo.dynamic != 0;
        Share sh;
        TileCursor tc;
        if (!dyn) {
            make_share<EPI>(p, geo.stage_bytes, RG, sh);
            tc.init(sh);
        }
        uint32_t st = 0, par = 1;   // parity of the slot's previous use ("1" before the first one: nothing to wait for)
        bool first_round = true;
        // counter hand-out: the CTA's first tiles are its own by position (no round trip before the first copy), every
        // later one is claimed
        uint32_t t = blockIdx.x * geo.head_per_cta, held = geo.head_per_cta;
        for (uint32_t k = 0;; k++, st = (st + 1 == S) ? 0 : st + 1) {
            if (st == 0 && k > 0) { par ^= 1u; first_round = false; }
            // the tile after this one is claimed now: the counter's round trip overlaps the wait for the slot
            const uint4 tm = dyn ? tile_of(geo, t) : (tc.valid(sh) ? make_uint4(tc.seg, tc.next, tc.count(sh), 0) : make_uint4(0, 0, 0, 0));
            uint32_t tn = 0;
            if (dyn && held == 1 && tm.z != 0 && lane == 0) tn = geo.head_tiles + atomicAdd(p.tile_claim, 1u);
            uint32_t ok = 1;
            if (!first_round && lane == 0) ok = mbar_wait(bar0 + 8 * (S + st), par, p.err, 2) ? 1u : 0u;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            const uint32_t s = tm.x, first_pair = tm.y, n = tm.z;
            const uint32_t full = bar0 + 8 * st;
            if (lane == 0) meta[st] = tm;
            if (n == 0) {
                // no tiles left: tell the consumers, and let the last CTA to get here clear the counters for their next use
                if (lane == 0) {
                    mbar_arrive(full);
                    if (dyn && atomicAdd(p.tile_claim + 1, 1u) == gridDim.x - 1) {
                        p.tile_claim[0] = 0u;
                        p.tile_claim[1] = 0u;
                    }
                }
                break;
            }
            const uint32_t cost = s == 0 ? geo.seg_cost[0] : (s == 1 ? geo.seg_cost[1] : geo.seg_cost[2]);
            const uint32_t dst = smem_u32(ring + (size_t)st * geo.stage_bytes);
            const uint32_t ba = (EPI == EPI_SWIGLU) ? n * (uint32_t)p.seg[0].row_bytes : n * cost;
            const uint32_t bb = (EPI == EPI_SWIGLU) ? n * (uint32_t)p.seg[1].row_bytes : 0u;
            const uint8_t *srcA = (EPI == EPI_SWIGLU) ? p.seg[0].w + (size_t)first_pair * p.seg[0].row_bytes : p.seg[s].w + (size_t)first_pair * cost;
            const uint8_t *srcB = (EPI == EPI_SWIGLU) ? p.seg[1].w + (size_t)first_pair * p.seg[1].row_bytes : nullptr;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // every issuing lane: the consumers' reads of the slot come first
            if (lane == 0) mbar_expect_tx(full, ba + bb);
            __syncwarp();
            for (uint32_t off = lane * COPY_PIECE; off < ba; off += 32 * COPY_PIECE) bulk_g2s(dst + off, srcA + off, min(COPY_PIECE, ba - off), full);
            if constexpr (EPI == EPI_SWIGLU)
                for (uint32_t off = lane * COPY_PIECE; off < bb; off += 32 * COPY_PIECE) bulk_g2s(dst + ba + off, srcB + off, min(COPY_PIECE, bb - off), full);
            TRACE(2 + (k < 6 ? k : 6));
            if (!dyn) tc.advance(sh);
            else if (held > 1) { t++; held--; }
            else t = __shfl_sync(0xffffffffu, tn, 0);
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
        if (threadIdx.x == 0) wait_counter(p.reduce_flag, ((*p.epoch_ptr) * p.reduce_per_epoch + p.reduce_use) * p.reduce_arrivals, p.err, 3);
        named_barrier(1, PACK_THREADS);
        rd = PackReduce{p.reduce_src, p.tp, p.x_out};
    }
    pack_activation(act_sm, p.cols, p.x, p.norm_w, p.eps, red, norm_g, rd, p.cols / 64);
    const Act A{act_sm, p.cols, p.cols / 64};
    TRACE(3);
    TRACE_CTA(g_cta_packed);

    unsigned long long best = 0ull;
    if ((uint32_t)warp < active) {
        Consumer c;
        c.ring = ring; c.part = part; c.fold0 = fold0; c.meta = reinterpret_cast<const uint4 *>(smem + geo.meta_off); c.bar0 = bar0; c.S = S; c.stage_bytes = geo.stage_bytes;
        c.CG = CG; c.RG = RG; c.cg = warp % CG; c.rg = warp / CG; c.u = c.cg * 32 + lane; c.has_unit = c.u < units; c.lane = lane;
        consume_tiles<EPI, QT>(p, c, A, best);
    }
    TRACE(15);
    TRACE_CTA(g_cta_end);

    if (EPI == EPI_PUSH) {
        // All of this CTA's peer stores are issued.  One thread per CTA arrives on a local counter with a system-scope
        // release (the CTA barrier makes it cumulative over the other threads' stores); the last CTA to arrive tells every
        // rank that this rank has delivered.  (One remote arrival per CTA instead was faster on 2 GPUs and slower on 4:
        // hundreds of remote atomics on one word.)
        named_barrier(1, PACK_THREADS);
        if (threadIdx.x == 0) {
            uint32_t before;
            asm volatile("atom.acq_rel.sys.global.add.u32 %0, [%1], %2;" : "=r"(before) : "l"(p.push_done), "r"(1u) : "memory");
            if (before == gridDim.x - 1) {
                *p.push_done = 0u;   // next used by a later kernel
                for (uint32_t rk = 0; rk < p.tp; rk++) asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.push_flag[rk]), "r"(1u) : "memory");
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
constexpr size_t STREAM_SMEM_BUDGET = 194 * 1024;   // one CTA per SM; stays under the 196 KB shared-memory configuration, which leaves 60 KB of L1 (register spills live there)

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
    bool only_q4_q6 = true;
    for (uint32_t s = 0; s < p.nseg; s++) {
        if (p.seg[s].qtype != qt) qt = QT_MIXED;
        only_q4_q6 = only_q4_q6 && (p.seg[s].qtype == IB_Q4_K || p.seg[s].qtype == IB_Q6_K);
    }
    if constexpr (EPI == EPI_QKV)
        if (qt == QT_MIXED && only_q4_q6) return launch_stream_inst<EPI, QT_Q4_Q6>(ctx, stream, p, grid, geo, smem);
    switch (qt) {
    case IB_Q4_K: return launch_stream_inst<EPI, IB_Q4_K>(ctx, stream, p, grid, geo, smem);
    case IB_Q6_K: return launch_stream_inst<EPI, IB_Q6_K>(ctx, stream, p, grid, geo, smem);
    case IB_Q5_K: return launch_stream_inst<EPI, IB_Q5_K>(ctx, stream, p, grid, geo, smem);
    case IB_Q8_0: return launch_stream_inst<EPI, IB_Q8_0>(ctx, stream, p, grid, geo, smem);
    default: return launch_stream_inst<EPI, QT_MIXED>(ctx, stream, p, grid, geo, smem);
    }
}

static int32_t launch_stream_switch(ib_ctx *ctx, cudaStream_t stream, const GemvParams &p, int grid, const StreamGeom &geo, size_t total);

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
            const size_t part = (size_t)S * PT_MAX * 2 * CW * 4 + (size_t)S * CW * 8;
            total = (size_t)S * stage + act + ((part + 127) & ~(size_t)127) + 2 * S * 8 + S * 16;   // + barriers + tile descriptors
            if (total <= STREAM_SMEM_BUDGET || S == 2) break;
        }
        return total <= STREAM_SMEM_BUDGET;
    };
    uint32_t stage = 0, S = 0;
    size_t total = 0;
    static const uint32_t first_try = [] {
        const char *e = getenv("INFERI_B200_TILE_BYTES");   // experiments: the largest tile to try first
        const long v = e ? atol(e) : 0;
        return (uint32_t)(v >= 4096 && v <= 98304 ? v : 75776);
    }();
    if (!layout(first_try, stage, S, total) && !layout(49152, stage, S, total) && !layout(32768, stage, S, total) && !layout(max_cost, stage, S, total))
        return set_error(IB_ERR_UNSUPPORTED, "gemv: a row pair of %u bytes with %u columns does not fit the streaming kernel's ring", max_cost, p.cols);
    StreamGeom geo;
    geo.stages = S;
    geo.stage_bytes = stage;
    geo.act_off = S * stage;
    geo.part_off = (uint32_t)(geo.act_off + act);
    geo.bar_off = (uint32_t)(geo.part_off + (((size_t)S * PT_MAX * 2 * CW * 4 + (size_t)S * CW * 8 + 127) & ~(size_t)127));
    geo.meta_off = geo.bar_off + 2 * S * 8;
    // the tiles in hand-out order: per segment whole rounds of the row groups, as many as fit a stage
    geo.total_tiles = 0;
    for (uint32_t s = 0; s < 3; s++) {
        geo.seg_pairs[s] = geo.seg_tiles[s] = 0;
        geo.seg_pt[s] = 1;
        geo.seg_cost[s] = 16;
        const bool swiglu = p.epi == EPI_SWIGLU;
        if (s >= (swiglu ? 1u : p.nseg)) continue;
        const uint32_t cost = swiglu ? max_cost : (uint32_t)(2 * p.seg[s].row_bytes);
        uint32_t pt = stage / cost;
        pt = pt < 1 ? 1 : (pt > (uint32_t)PT_MAX ? (uint32_t)PT_MAX : pt);
        if (pt > RG) pt = pt / RG * RG;
        geo.seg_cost[s] = cost;
        geo.seg_pt[s] = pt;
        geo.seg_pairs[s] = swiglu ? p.seg[0].rows : p.seg[s].rows / 2;
        geo.seg_tiles[s] = (geo.seg_pairs[s] + pt - 1) / pt;
        geo.total_tiles += geo.seg_tiles[s];
    }
    int grid = ctx->sm_count;       // one persistent CTA per SM: 16 consumer warps hide the latency of the dependent dp4a / shuffle chains
    if ((uint32_t)grid > pairs) grid = (int)pairs;
    if (grid < 1) grid = 1;
    // Hand-out: launches of one segment with enough tiles per CTA give every CTA its first tiles by position and let the
    // CTAs claim the rest from a counter - whole tiles when there are many (>= 6 per CTA), one-round tiles for the last
    // third or so when there are few (>= 2.5 per CTA, e.g. gate/up with 3.0), where a whole tile would be too coarse a
    // unit to even out the CTAs' end times.  Everything else: static byte-balanced ranges.
    geo.dynamic = 0;
    geo.head_per_cta = geo.head_tiles = 0;
    geo.tail_pt = geo.seg_pt[0];
    const bool single = p.epi == EPI_SWIGLU || p.nseg == 1;
    const uint32_t tiles_x2_per_cta = 2u * geo.total_tiles / (uint32_t)grid;
    if (single && tiles_x2_per_cta >= 12u) {
        geo.dynamic = 1;
        geo.head_per_cta = S;
    } else if (single && tiles_x2_per_cta >= 5u && geo.seg_pt[0] >= 2 * RG) {
        geo.dynamic = 1;
        const uint32_t whole = geo.total_tiles / (uint32_t)grid;
        geo.head_per_cta = whole - 1 < S ? whole - 1 : S;
        geo.tail_pt = RG;
    }
    geo.head_tiles = (uint32_t)grid * geo.head_per_cta;
    // the counters through which this launch's CTAs share out the tiles: consecutive launches overlap (programmatic
    // dependent launch), so they take different pairs of a small ring; the last CTA of a launch clears its pair
    GemvParams q = p;
    q.tile_claim = ctx->stream_counters + 2 * (ctx->stream_seq++ % IB_STREAM_COUNTER_PAIRS);
    return launch_stream_switch(ctx, stream, q, grid, geo, total);
}

static int32_t launch_stream_switch(ib_ctx *ctx, cudaStream_t stream, const GemvParams &p, int grid, const StreamGeom &geo, size_t total) {
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
extern "C" __attribute__((visibility("default"))) int32_t ib_debug_cta_times(unsigned long long *ends, unsigned long long *packed) {
    if (cudaMemcpyFromSymbol(ends, g_cta_end, sizeof(unsigned long long) * 8 * 160) != cudaSuccess) return 2;
    return cudaMemcpyFromSymbol(packed, g_cta_packed, sizeof(unsigned long long) * 8 * 160) == cudaSuccess ? 0 : 2;
}
extern "C" __attribute__((visibility("default"))) int32_t ib_debug_consumer_phases(long long *out) {
    return cudaMemcpyFromSymbol(out, g_phase, sizeof(long long) * 8 * 32 * 10) == cudaSuccess ? 0 : 2;
}
#endif

}  // namespace ib
