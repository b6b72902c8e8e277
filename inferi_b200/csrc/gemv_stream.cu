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
//    unit's activations — two int8 limbs per column, see gemv_common.cuh — in registers for the whole kernel, so
//    the inner loop touches shared memory only for weights.  Per weight the work is a byte mask and dp4a.
//  * Per row the lane partials are shuffled down, per-warp partials meet in shared memory, and the last warp of a
//    row group to arrive adds them in a fixed order and runs the epilogue (store / residual add / SwiGLU /
//    RoPE + KV append / arg-max).  No warp ever waits for another one except through the ring.
// Every wait on an mbarrier is bounded; a wait that gives up raises the context's error word and carries on.
#include "gemv_stream.cuh"

#include <stdlib.h>

namespace ib {


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
    uint32_t ring;        // shared address of the ring
    uint32_t part;        // shared address of the per-stage partial sums [stages][2][CW][PT_MAX]
    uint32_t meta;        // shared address of [stages] (segment, first pair, pairs, -) descriptors written by the producer
    uint32_t bar0, S, stage_bytes;
    uint32_t CG, RG, cg, rg, u;
    bool has_unit;
    int lane;
};

// Offset (in floats) of the partial of (row of the pair, column-group warp, pair of the tile) inside a stage's block:
// pairs are the fastest index, so that the lanes of the epilogue warp (one pair each) read consecutive words.
__device__ __forceinline__ uint32_t part_index(uint32_t row, uint32_t cg, uint32_t pr) { return (row * CW + cg) * PT_MAX + pr; }
constexpr uint32_t PART_STAGE_FLOATS = 2 * CW * PT_MAX;

// A consumer warp: its lanes' 64-column units of every row pair of every tile.  Per tile it waits for the weights, leaves
// two partial sums per pair (its columns of the two rows) in the stage's partial block and arrives on the stage's "done"
// barrier.  It never waits for another consumer warp: adding up the column groups and everything that follows is the
// epilogue warp's work.
template <uint32_t QT>
__device__ __forceinline__ void consume_tiles(const GemvParams &p, const Consumer &c, const Act &A) {
    const int lane = c.lane;
    UnitAct ua;
    LaneConst lc;
    uint32_t cur_type = 0xFFFFFFFFu;
    const uint32_t S = c.S, RG = c.RG;
    uint32_t st = 0, par = 0;
    constexpr bool ONE_TYPE = (QT != QT_MIXED && QT != QT_Q4_Q6);
    const uint32_t rb0 = (uint32_t)p.seg[0].row_bytes, rb1 = (uint32_t)p.seg[1].row_bytes, rb2 = (uint32_t)p.seg[2].row_bytes;
    const bool swiglu = p.epi == EPI_SWIGLU;   // gate rows, then up rows, in one tile: a "pair" is gate row r + up row r
    {
        // The lane's activations go into registers in the layout of the first segment's format before the first tile is
        // waited for: the copy of that tile and this load overlap.
        const uint32_t q0 = ONE_TYPE ? QT : p.seg[0].qtype;
        unit_init<QT>(q0, c.u, lc);
        if (c.has_unit) load_unit_act(q0, c.u, A, ua);
        cur_type = q0;
    }
#pragma unroll 1
    for (;; st = (st + 1 == S) ? 0 : st + 1, par ^= (st == 0) ? 1u : 0u) {
        if (!mbar_wait(c.bar0 + 8 * st, par, p.err, 1, p.wait_ns)) return;   // the error word is raised; give up on this CTA's rows
        const uint4 tm = lds128(c.meta + 16 * st);
        const uint32_t s = tm.x, n = tm.z;
        if (n == 0) break;   // no tiles left
        const uint32_t qtype = ONE_TYPE ? QT : (s == 0 ? p.seg[0].qtype : (s == 1 ? p.seg[1].qtype : p.seg[2].qtype));
        if (qtype != cur_type) {   // (re)load this lane's activations in the layout of the segment's format
            unit_init<QT>(qtype, c.u, lc);
            if (c.has_unit) load_unit_act(qtype, c.u, A, ua);
            cur_type = qtype;
        }
        const uint32_t tile = c.ring + st * c.stage_bytes;
        const uint32_t rbA = (swiglu || s == 0) ? rb0 : (s == 1 ? rb1 : rb2);
        const uint32_t strideA = swiglu ? rbA : 2 * rbA;
        const uint32_t offB = swiglu ? n * rbA : rbA, strideB = swiglu ? rb1 : strideA;
        const uint32_t pt = c.part + 4 * (st * PART_STAGE_FLOATS);
        for (uint32_t pr = c.rg; pr < n; pr += RG) {
            float va = 0.f, vb = 0.f;
            if (c.has_unit) {
                va = unit_dot<QT>(qtype, tile + pr * strideA, lc, ua);
                vb = unit_dot<QT>(qtype, tile + offB + pr * strideB, lc, ua);
            }
            // one shuffle tree for both rows: after the first exchange the upper half-warp carries row B
            const bool up = lane & 16;
            float v = (up ? vb : va) + __shfl_xor_sync(0xffffffffu, up ? va : vb, 16);
#pragma unroll
            for (int o = 8; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if ((lane & 15) == 0)   // lane 0 holds row A's sum, lane 16 row B's
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(pt + 4 * part_index(lane >> 4, c.cg, pr)), "f"(v) : "memory");
        }
        __syncwarp();   // lane 16's partials are ordered before lane 0's arrival (a release)
        if (lane == 0) mbar_arrive(c.bar0 + 8 * (2 * S + st));   // this warp is done with the stage: weights read, partials left
    }
}

// The epilogue warp: per tile it waits until every consumer warp has left its partials, adds up the column groups in a
// fixed order (bitwise deterministic results), hands the stage back to the producer and runs the epilogue of the tile's
// row pairs, one pair per lane.
__device__ __forceinline__ void finish_tiles(const GemvParams &p, uint32_t part, uint32_t meta, uint32_t bar0, uint32_t S, uint32_t CG, int lane,
                                             const float *red, unsigned long long &best) {
    uint32_t st = 0, par = 0;
    float rms = 1.0f;
    bool rms_known = p.norm_w == nullptr;
    const bool residual = p.epi == EPI_RESIDUAL;
#pragma unroll 1
    for (;; st = (st + 1 == S) ? 0 : st + 1, par ^= (st == 0) ? 1u : 0u) {
        if (!mbar_wait(bar0 + 8 * st, par, p.err, 1, p.wait_ns)) return;
        const uint4 tm = lds128(meta + 16 * st);
        const uint32_t s = tm.x, first_pair = tm.y, n = tm.z;
        if (n == 0) break;
        const bool mine = (uint32_t)lane < n;
        // the pair's residual values are requested before the wait for the dot products: the L2 round trip overlaps it
        float2 rpre = make_float2(0.f, 0.f);
        if (residual && mine) rpre = residual_prefetch(p.resid, first_pair + lane);
        if (!rms_known) {
            // RMSNorm factor of the input vector (crates/inferi-shaders/src/rms_norm.rs:112-120): the consumer warps left
            // their parts of the sum of squares in `red`; added in a fixed order
            if (!mbar_wait(bar0 + 8 * (3 * S), 0, p.err, 6, p.wait_ns)) return;
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < PACK_THREADS / 32; w++) t += red[w];
            rms = 1.0f / sqrtf(t / (float)p.cols + p.eps);
            rms_known = true;
        }
        if (!mbar_wait(bar0 + 8 * (2 * S + st), par, p.err, 5, p.wait_ns)) return;
        float va = 0.f, vb = 0.f;
        if (mine) {
            const uint32_t pt = part + 4 * (st * PART_STAGE_FLOATS);
            for (uint32_t g = 0; g < CG; g++) {
                va += __uint_as_float(lds32(pt + 4 * part_index(0, g, lane)));
                vb += __uint_as_float(lds32(pt + 4 * part_index(1, g, lane)));
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar0 + 8 * (S + st));   // partials read: the producer may refill the stage
        if (mine) epilogue(p, s, first_pair + lane, va * rms, vb * rms, best, rpre);
    }
}

// ---- the kernel ----
// Shared-memory barriers: full[S] (the producer's expect_tx arrival + the copy's bytes), empty[S] (one arrival: the
// epilogue warp has read the stage's partials, which implies that every consumer warp is done with its weights),
// done[S] (one arrival per working consumer warp), ss (one arrival per consumer warp: its part of the input's sum of squares).
// One instance per weight format (or format pair); what the launch does with the row sums is a run-time switch in the
// epilogue warp, so that the launches of a token graph share their code.
template <uint32_t QT>
__global__ void __launch_bounds__(STREAM_THREADS, 1) gemv_stream_kernel(const GemvParams p, const StreamGeom geo) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float red[PACK_THREADS / 32 + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    uint8_t *ring = smem;
    uint8_t *act_sm = smem + geo.act_off;
    const uint32_t part = smem_u32(smem + geo.part_off);                        // [stages][2][CW][PT_MAX] floats
    const uint32_t bar0 = smem_u32(smem + geo.bar_off);                         // full[stages], empty[stages], done[stages]
    const uint32_t S = geo.stages;

    const uint32_t units = p.cols / 64;
    const uint32_t CG = (units + 31) / 32;       // warps that split one row's columns
    const uint32_t RG = CW / CG;                 // row groups working side by side
    const uint32_t active = CG * RG;             // consumer warps with work

    if (threadIdx.x <= 3 * S) {
        const uint32_t which = threadIdx.x / S;
        mbar_init(bar0 + 8 * threadIdx.x, which == 2 ? active : (which == 3 ? (uint32_t)CW : 1u));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (p.pdl) asm volatile("griddepcontrol.launch_dependents;");

    if (warp == W_PRODUCER) {
        // ================= producer warp: picks tiles and streams them =================
        // With many tiles per CTA they are handed out through a counter in global memory, so that a CTA which starts late
        // (its SM was the last to be freed by the previous kernel) or runs slowly takes fewer of them.  With few tiles per
        // CTA a tile is too coarse a unit for that: every CTA then streams its own byte-balanced range of row pairs, cut
        // into tiles.  Either way the slot's descriptor tells the other warps what the tile is.  Lane 0 picks, waits for
        // the slot, announces the tile and issues its bulk copies.
        uint4 *meta = reinterpret_cast<uint4 *>(smem + geo.meta_off);
        const bool dyn = geo.dynamic != 0;
        Share sh;
        TileCursor tc;
        const bool swiglu = p.epi == EPI_SWIGLU;
        if (!dyn) {
            make_share(p, geo.stage_bytes, RG, sh);
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
            if (!first_round && lane == 0) ok = mbar_wait(bar0 + 8 * (S + st), par, p.err, 2, p.wait_ns) ? 1u : 0u;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            const uint32_t s = tm.x, first_pair = tm.y, n = tm.z;
            const uint32_t full = bar0 + 8 * st;
            if (lane == 0) meta[st] = tm;
            if (n == 0) {
                // no tiles left: tell the others, and let the last CTA to get here clear the counters for their next use
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
            const uint32_t ba = swiglu ? n * (uint32_t)p.seg[0].row_bytes : n * cost;
            const uint32_t bb = swiglu ? n * (uint32_t)p.seg[1].row_bytes : 0u;
            const uint8_t *srcA = swiglu ? p.seg[0].w + (size_t)first_pair * p.seg[0].row_bytes : p.seg[s].w + (size_t)first_pair * cost;
            const uint8_t *srcB = swiglu ? p.seg[1].w + (size_t)first_pair * p.seg[1].row_bytes : nullptr;
            if (lane == 0) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the consumers' reads of the slot come first
                mbar_expect_tx(full, ba + bb);
                bulk_g2s(dst, srcA, ba, full);
                if (swiglu) bulk_g2s(dst + ba, srcB, bb, full);
            }
            if (!dyn) tc.advance(sh);
            else if (held > 1) { t++; held--; }
            else t = __shfl_sync(0xffffffffu, tn, 0);
            // The CTA's first tile travels alone: with a ring-full of copies in flight at once the copy engine interleaves
            // them and all of them - the first one too - arrive when the last byte does, which is later than the consumers
            // are ready for the first tile.  The others follow as soon as the first has landed.
            if (k == 0) {
                uint32_t ok0 = 1;
                if (lane == 0) ok0 = mbar_wait(bar0, 0, p.err, 1, p.wait_ns) ? 1u : 0u;
                if (!__shfl_sync(0xffffffffu, ok0, 0)) break;
            }
        }
        return;
    }

    if (warp == W_EPILOGUE) {
        // ================= epilogue warp =================
        // outputs (and the residual it reads) are touched by the previous kernels of the stream: wait for them like the consumers do
        if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
        if (p.reduce_src) {
            // Tensor parallel: the previous row-split GEMV of every rank leaves its partial sums in this rank's slots.  The sum
            // (x + the partials in rank order, so every rank gets the same bits) is formed once per rank: this warp adds up
            // the groups of 32 columns that fall to its CTA and stores them as the new residual stream; the consumer warps of
            // all CTAs wait until every group is there.  (Each CTA adding up the whole vector for itself was N x 16 KiB of L2
            // reads per CTA: at 8 ranks more than its share of the weights.)
            const uint32_t tag = (*p.epoch_ptr) * p.xchg_per_epoch + p.reduce_use;
            uint32_t cnt = 0;
            for (uint32_t grp = blockIdx.x; grp < p.cols / 32; grp += gridDim.x) {
                const uint32_t col = grp * 32 + lane;
                float v = __ldcg(p.x + col);
                // on a time-out the error word is raised and the launch runs to its end on whatever is there
                for (uint32_t rk = 0; rk < p.tp; rk++) v += wait_tagged(p.reduce_src + (size_t)rk * p.cols + col, tag, p.err, p.wait_ns);
                p.x_out[col] = v;
                cnt++;
            }
            __threadfence();
            __syncwarp();
            if (lane == 0 && cnt) asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p.reduce_done), "r"(cnt) : "memory");
        }
        unsigned long long best = 0ull;
        finish_tiles(p, part, smem_u32(smem + geo.meta_off), bar0, S, CG, lane, red, best);
        if (p.epi == EPI_ARGMAX) {
#pragma unroll
            for (int o = 16; o; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
            uint32_t last = 0;
            if (lane == 0) {
                p.argmax_slots[blockIdx.x] = best;
                __threadfence();
                last = (atomicAdd(p.argmax_counter, 1u) == gridDim.x - 1) ? 1u : 0u;
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                // the last CTA to arrive folds every CTA's candidate; no CTA waits for another
                __threadfence();
                unsigned long long b = 0ull;
                for (uint32_t i = lane; i < gridDim.x; i += 32) b = max(b, __ldcg(p.argmax_slots + i));
#pragma unroll
                for (int o = 16; o; o >>= 1) b = max(b, __shfl_xor_sync(0xffffffffu, b, o));
                if (lane == 0) {
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
        return;
    }

    // ================= consumer warps =================
    Consumer c;
    c.ring = smem_u32(ring); c.part = part; c.meta = smem_u32(smem + geo.meta_off); c.bar0 = bar0; c.S = S; c.stage_bytes = geo.stage_bytes;
    c.CG = CG; c.RG = RG; c.cg = warp % CG; c.rg = warp / CG; c.u = c.cg * 32 + lane; c.has_unit = c.u < units; c.lane = lane;
    const Act A{act_sm, p.cols, p.cols / 64};
    float4 norm_g[4];
    pack_prefetch_norm(p.norm_w, p.cols, norm_g);   // weights: fetched while the previous kernel is still running
    {
        // The launch parameters the tile loop reads, touched while the previous kernel is still running: their first read
        // misses the constant cache, and that round trip would otherwise sit between the activations and the first tile.
        const uint32_t touch = (uint32_t)p.seg[0].row_bytes ^ (uint32_t)p.seg[1].row_bytes ^ (uint32_t)p.seg[2].row_bytes ^ p.seg[0].qtype ^
                               p.seg[1].qtype ^ p.seg[2].qtype ^ p.epi ^ (uint32_t)p.wait_ns ^ (uint32_t)(uintptr_t)p.err;
        asm volatile("" ::"r"(touch));
    }
    if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (p.reduce_src) {
        // tensor parallel: the reduced residual stream is complete once the epilogue warps of all CTAs have stored their groups
        if (threadIdx.x == 0) wait_counter_gpu(p.reduce_done, ((*p.epoch_ptr) * p.xchg_per_epoch + p.reduce_use) * (p.cols / 32), p.err, 7, p.wait_ns);
        named_barrier(1, PACK_THREADS);
    }
    pack_stream(act_sm, p.cols, p.reduce_src ? p.x_out : p.x, p.norm_w, red, bar0 + 8 * (3 * S), norm_g, p.cols / 64);
    if ((uint32_t)warp < active) consume_tiles<QT>(p, c, A);
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

template <uint32_t QT>
static int32_t launch_stream_inst(ib_ctx *ctx, cudaStream_t stream, const GemvParams &p, int grid, const StreamGeom &geo, size_t smem) {
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        IB_CHECK_CUDA(cudaFuncSetAttribute(gemv_stream_kernel<QT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)STREAM_SMEM_BUDGET));
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
    IB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, gemv_stream_kernel<QT>, p, geo));
    ctx->launches++;
    return IB_OK;
}

// Which instance serves a launch: the one of its format; launches that mix Q4_K and Q6_K segments - or that ask for it
// (`pair_instance`: the launches of a Q4_K_M token graph, so that all of them run the same code) - the two-format one.
static int32_t launch_stream_format(ib_ctx *ctx, cudaStream_t stream, const GemvParams &p, int grid, const StreamGeom &geo, size_t smem) {
    uint32_t qt = p.seg[0].qtype;
    bool only_q4_q6 = true;
    for (uint32_t s = 0; s < p.nseg; s++) {
        if (p.seg[s].qtype != qt) qt = QT_MIXED;
        only_q4_q6 = only_q4_q6 && (p.seg[s].qtype == IB_Q4_K || p.seg[s].qtype == IB_Q6_K);
    }
    if (only_q4_q6 && (qt == QT_MIXED || p.pair_instance)) return launch_stream_inst<QT_Q4_Q6>(ctx, stream, p, grid, geo, smem);
    switch (qt) {
    case IB_Q4_K: return launch_stream_inst<IB_Q4_K>(ctx, stream, p, grid, geo, smem);
    case IB_Q6_K: return launch_stream_inst<IB_Q6_K>(ctx, stream, p, grid, geo, smem);
    case IB_Q5_K: return launch_stream_inst<IB_Q5_K>(ctx, stream, p, grid, geo, smem);
    case IB_Q8_0: return launch_stream_inst<IB_Q8_0>(ctx, stream, p, grid, geo, smem);
    default: return launch_stream_inst<QT_MIXED>(ctx, stream, p, grid, geo, smem);
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
    // tile = whole "rounds" of the row groups (RG pairs each, one pair per consumer warp) of up to ~56 KB, in as many stages
    // as fit beside the activations (at most 4): several copies in flight per SM keep HBM busy while one tile is consumed
    const uint32_t units = p.cols / 64, CG = (units + 31) / 32, RG = CW / CG;
    const size_t act = (act_smem_bytes(p.cols) + 127) & ~(size_t)127;
    auto part_bytes = [](uint32_t S) { return (size_t)S * PART_STAGE_FLOATS * 4; };
    auto bar_bytes = [](uint32_t S) { return ((size_t)(3 * S + 1) * 8 + 15) & ~(size_t)15; };
    // returns 0 if the layout does not fit, 1 if it fits, 2 if it fits and every segment's tile is whole rounds
    auto layout = [&](uint32_t max_tile_bytes, uint32_t &stage, uint32_t &S, size_t &total) {
        bool whole = true;
        auto pairs_per_tile = [&](uint32_t cost) {
            uint32_t pt = RG;
            while (pt * 2 <= PT_MAX && pt * 2 * cost <= max_tile_bytes) pt *= 2;
            while (pt > 1 && pt * cost > max_tile_bytes) pt--;
            if (pt % RG) whole = false;
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
            total = (size_t)S * stage + act + part_bytes(S) + bar_bytes(S) + S * 16;   // + partials + barriers + tile descriptors
            if (total <= STREAM_SMEM_BUDGET || S == 2) break;
        }
        return total <= STREAM_SMEM_BUDGET ? (whole ? 2 : 1) : 0;
    };
    uint32_t stage = 0, S = 0;
    size_t total = 0;
    const uint32_t tries[5] = {57344, 75776, 49152, 32768, max_cost};
    int chosen = -1;
    for (int pass = 2; pass >= 1 && chosen < 0; pass--)
        for (int i = 0; i < 5 && chosen < 0; i++)
            if (layout(tries[i], stage, S, total) >= pass) chosen = i;
    if (chosen < 0)
        return set_error(IB_ERR_UNSUPPORTED, "gemv: a row pair of %u bytes with %u columns does not fit the streaming kernel's ring", max_cost, p.cols);
    StreamGeom geo;
    geo.stages = S;
    geo.stage_bytes = stage;
    geo.act_off = S * stage;
    geo.part_off = (uint32_t)(geo.act_off + act);
    geo.bar_off = (uint32_t)(geo.part_off + part_bytes(S));
    geo.meta_off = (uint32_t)(geo.bar_off + bar_bytes(S));
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
    int grid = ctx->sm_count;       // one persistent CTA per SM
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
    IB_REQUIRE(q.epi <= EPI_PUSH, "gemv: unknown epilogue %u", q.epi);
    return launch_stream_format(ctx, stream, q, grid, geo, total);
}

}  // namespace ib
