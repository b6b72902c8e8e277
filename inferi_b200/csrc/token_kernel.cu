// The whole-token kernel: one cooperative launch runs every phase of a token (embedding, then per layer qkv ->
// attention -> o_proj -> gate/up -> down, then classifier + greedy arg-max) on one persistent CTA per SM.
//
// Replaces the per-token dispatch sequence of `Llama2::launch` (crates/inferi/src/models/llama2/transformer.rs:409-481)
// and the bookkeeping of the token loop (crates/inferi-chat/src/chat_llama2.rs:137-171, sampler.rs:102-110).
//
// Why one kernel: a batch-1 token is ~160 dependent matrix-vector products of 10-70 MB each.  As separate launches each
// pays its own start-up (barrier set-up, pipeline fill, tail) and HBM idles in between.  Here
//  * a producer warp per CTA walks the token's whole weight list and keeps a shared-memory byte ring full with bulk
//    asynchronous copies; weights do not depend on activations, so it runs ahead across phase boundaries and HBM stays
//    busy while the consumers synchronise and convert the next activation vector;
//  * sixteen consumer warps per CTA do the arithmetic of the streaming GEMV (gemv_stream.cuh) and, in the attention
//    phases, split-K decode attention (attention.cuh) as four 4-warp blocks per CTA;
//  * phases are separated by a grid barrier on a counter that only grows (arrive with a release, poll with an acquire).
// Every wait (mbarrier, grid barrier) is bounded; when one gives up the kernel raises the context's error word, stops
// issuing copies, waits for the copies in flight and returns.
#include "gemv_stream.cuh"
#include "token.cuh"

namespace ib {

constexpr uint32_t NS = TK_SLOTS;
// 16 warps per CTA, four per SM sub-partition, so that every thread can have 128 registers (the whole register file):
// 15 consumer warps + 1 producer warp.  With the 17 warps of the stand-alone GEMV kernel the limit would be 96, and a
// spilled register costs an L2 round trip here: the kernel's shared memory leaves next to no L1.
constexpr int TCW = 15;                       // consumer warps
constexpr int TK_CONSUMERS = TCW * 32;        // threads that take part in the prologues and the grid barriers
constexpr int TK_THREADS = (TCW + 1) * 32;
constexpr int TK_REGS = 128;
static_assert((NS & (NS - 1)) == 0, "slot count must be a power of two");

#ifdef IB_TOKEN_TRACE
// Timeline probes for latency studies (never compiled into the shipped library): globaltimer stamps of warp 0 of four
// CTAs (first, two in the middle, last) at the marks of each of the first 64 phases, plus the producer lane of CTA 0.
// Read back with ib_debug_token_trace().
__device__ unsigned long long g_tk_trace[5][64][8];
__device__ unsigned long long g_tk_done[64][160];   // when warp 0 of every CTA finished each phase
#define TK_TRACE(ph, mark)                                                                                          \
    do {                                                                                                            \
        if ((threadIdx.x & 31) == 0 && (threadIdx.x >> 5) == 0 && (ph) < 64) {                                      \
            const int _c = blockIdx.x == 0 ? 0 : blockIdx.x == gridDim.x / 3 ? 1 : blockIdx.x == 2 * gridDim.x / 3 ? 2 : blockIdx.x == gridDim.x - 1 ? 3 : -1; \
            if (_c >= 0) g_tk_trace[_c][ph][mark] = global_ns();                                                    \
        }                                                                                                           \
    } while (0)
#define TK_TRACE_DONE(ph)                                                                                           \
    do {                                                                                                            \
        if ((threadIdx.x & 31) == 0 && (threadIdx.x >> 5) == 0 && (ph) < 64 && blockIdx.x < 160) g_tk_done[ph][blockIdx.x] = global_ns(); \
    } while (0)
#define TK_TRACE_PROD(ph, mark)                                                                                     \
    do {                                                                                                            \
        if (blockIdx.x == 0 && (ph) < 64) g_tk_trace[4][ph][mark] = global_ns();                                    \
    } while (0)
#else
#define TK_TRACE(ph, mark) do { } while (0)
#define TK_TRACE_DONE(ph) do { } while (0)
#define TK_TRACE_PROD(ph, mark) do { } while (0)
#endif

// The current phase as the consumer threads see it: fetched from the descriptor and worked out (this CTA's share of the
// rows) by one thread while the CTA waits at the grid barrier, so that none of it costs the others registers or time.
struct PhaseShared {
    uint32_t kind, epi, cols, nseg;
    uint32_t rb0, rb1, rb2, qt0, qt1, qt2;
    float eps;
    const float *x, *norm_w;
    void *kc, *vc;
};

struct __align__(16) TkShared {
    PhaseShared cur;
    float red[TK_CONSUMERS / 32 + 1];
    unsigned long long best_sm[TCW];
    volatile uint32_t abort_flag;       // a wait gave up somewhere in this CTA
    volatile uint32_t go;               // decision after a grid barrier, identical for every consumer thread
    volatile uint32_t issued;           // tiles the producer has issued (valid once it has stopped)
    uint32_t tile_bytes[NS];            // ring bytes held by the tile in each slot (producer's book-keeping)
    uint4 meta[NS];                     // what the slot holds: ring offset, first row pair, pairs | segment << 8 | end-of-phase << 16
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <typename Ptr>
__device__ __forceinline__ Ptr load_ptr(const Ptr *p) {   // read-only pointer field of a phase descriptor
    return reinterpret_cast<Ptr>(__ldg(reinterpret_cast<const unsigned long long *>(p)));
}

__device__ __forceinline__ LayerMat load_mat(const LayerMat *m) {
    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(m));
    LayerMat r;
    r.w = reinterpret_cast<const uint8_t *>(((unsigned long long)v.y << 32) | v.x);
    r.row_bytes = v.z;
    r.qtype = v.w;
    return r;
}

// The scalar part of a descriptor (rows[3], nseg, epi, cols, eps, kind) as two 16-byte loads.
struct PhaseScalars {
    uint32_t rows0, rows1, rows2, nseg, epi, cols, kind;
    float eps;
};
__device__ __forceinline__ PhaseScalars load_scalars(const PhaseDesc *d) {
    const uint4 a = __ldg(reinterpret_cast<const uint4 *>(&d->rows[0])), b = __ldg(reinterpret_cast<const uint4 *>(&d->rows[0]) + 1);
    PhaseScalars s;
    s.rows0 = a.x; s.rows1 = a.y; s.rows2 = a.z; s.nseg = a.w;
    s.epi = b.x; s.cols = b.y; s.eps = __uint_as_float(b.z); s.kind = b.w;
    return s;
}

// Grid barrier for the consumer threads of every CTA, entered at the start of each phase (and once more at the end of the
// token, with d == null).  Thread 0 arrives on the global counter with a release and polls it with an acquire; meanwhile
// thread 32 turns the phase's descriptor into ts->cur.  Returns false (for every thread alike) when this CTA has to give
// up: its own wait ran out, or some warp of the CTA raised the abort flag earlier.
__device__ __forceinline__ bool phase_sync(const TokenProgram &P, const PhaseDesc *d, uint32_t target, TkShared *ts) {
    const bool scribe = threadIdx.x == 32 && d != nullptr;
    PhaseScalars sc;
    LayerMat m0, m1, m2;
    const float *x = nullptr, *norm_w = nullptr;
    void *kc = nullptr, *vc = nullptr;
    if (scribe) {   // issued before the CTA's own barrier: the latency overlaps the wait for the CTA's warps
        sc = load_scalars(d);
        m0 = load_mat(&d->m[0]); m1 = load_mat(&d->m[1]); m2 = load_mat(&d->m[2]);
        x = load_ptr(&d->x); norm_w = load_ptr(&d->norm_w);
        kc = load_ptr(&d->k_cache); vc = load_ptr(&d->v_cache);
    }
    named_barrier(1, TK_CONSUMERS);
    if (threadIdx.x == 0) {
        bool ok = ts->abort_flag == 0;
        if (ok) {
            // release: everything this CTA wrote in the phase (ordered before by the CTA barrier) is visible to whoever
            // observes the arrival
            asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(P.grid_bar), "r"(1u) : "memory");
            ok = (int32_t)(ld_acquire_gpu(P.grid_bar) - target) >= 0;
            if (!ok) {
                const unsigned long long t0 = global_ns();
                for (;;) {
                    for (int i = 0; i < 32 && !ok; i++) ok = (int32_t)(ld_acquire_gpu(P.grid_bar) - target) >= 0;
                    if (ok || global_ns() - t0 > WAIT_LIMIT_NS) break;
                }
            }
            if (!ok) {
                *(volatile uint32_t *)P.err = 5;
                __threadfence_system();
                ts->abort_flag = 1;
            }
        }
        ts->go = ok ? 1u : 0u;
    } else if (scribe) {
        PhaseShared &c = ts->cur;
        c.kind = sc.kind; c.epi = sc.epi; c.cols = sc.cols; c.nseg = sc.nseg; c.eps = sc.eps;
        c.rb0 = m0.row_bytes; c.rb1 = m1.row_bytes; c.rb2 = m2.row_bytes; c.qt0 = m0.qtype; c.qt1 = m1.qtype; c.qt2 = m2.qtype;
        c.x = x; c.norm_w = norm_w; c.kc = kc; c.vc = vc;
    }
    named_barrier(1, TK_CONSUMERS);
    return ts->go != 0;
}

// ---- producer: one lane streams this CTA's share of every matrix of the token into the byte ring ----
struct StreamSrc {
    const uint8_t *w0, *w1, *w2;
    uint32_t rb0, rb1, rb2;
    const float *norm;
    PhaseScalars sc;
};

__device__ __forceinline__ StreamSrc load_src(const PhaseDesc *d) {
    StreamSrc s;
    s.sc = load_scalars(d);
    const LayerMat a = load_mat(&d->m[0]), b = load_mat(&d->m[1]), c = load_mat(&d->m[2]);
    s.w0 = a.w; s.rb0 = a.row_bytes; s.w1 = b.w; s.rb1 = b.row_bytes; s.w2 = c.w; s.rb2 = c.row_bytes;
    s.norm = load_ptr(&d->norm_w);
    return s;
}

// Pairs per tile: one round of the row groups, doubled while the tile stays under 16 KB (short rows) and within limits.
__device__ __forceinline__ uint32_t dyn_tile_pairs(uint32_t tile_max, uint32_t cost, uint32_t RG) {
    uint32_t pt = RG;
    while (pt * 2 <= (uint32_t)PT_MAX && pt * cost < 16384u && pt * 2 * cost <= tile_max) pt *= 2;
    while (pt > 1 && pt * cost > tile_max) pt--;
    return pt;
}

__device__ __forceinline__ void produce_token(const TokenProgram &P, TkShared *ts, uint32_t epoch) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *ring = smem;
    const uint32_t bar0 = smem_u32(smem + P.geo.bar_off);
    const uint32_t RING = P.geo.ring_bytes;
    uint32_t kt = 0, off = 0, used = 0, tail = 0;
    bool stop = false;
    StreamSrc cur = load_src(P.phases);
    for (uint32_t ph = 0; ph < P.n_phases && !stop; ph++) {
        StreamSrc nxt = cur;
        if (ph + 1 < P.n_phases) nxt = load_src(P.phases + ph + 1);   // in flight while this phase streams
        TK_TRACE_PROD(ph, 0);
        if (cur.sc.kind == PH_GEMV) {
            if (cur.norm && blockIdx.x == ph % gridDim.x)   // the phase's norm weights: into L2 ahead of the consumers
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(cur.norm), "r"(cur.sc.cols * 4u) : "memory");
            // The phase's tiles are handed out through a global counter: a CTA that falls behind simply claims fewer.  Tile
            // t covers pt row pairs of one segment.  The counters are zeroed at the end of every token.
            const uint32_t units = cur.sc.cols / 64, CG = (units + 31) / 32, RG = TCW / CG;
            const bool swiglu = cur.sc.epi == EPI_SWIGLU;
            const uint32_t n0 = swiglu ? cur.sc.rows0 : cur.sc.rows0 / 2, c0 = swiglu ? cur.rb0 + cur.rb1 : 2 * cur.rb0;
            const uint32_t n1 = (!swiglu && cur.sc.nseg > 1) ? cur.sc.rows1 / 2 : 0, c1 = 2 * cur.rb1;
            const uint32_t n2 = (!swiglu && cur.sc.nseg > 2) ? cur.sc.rows2 / 2 : 0, c2 = 2 * cur.rb2;
            const uint32_t pt0 = dyn_tile_pairs(P.geo.tile_max, c0, RG), pt1 = dyn_tile_pairs(P.geo.tile_max, c1, RG), pt2 = dyn_tile_pairs(P.geo.tile_max, c2, RG);
            const uint32_t nt0 = (n0 + pt0 - 1) / pt0, nt1 = (n1 + pt1 - 1) / pt1, nt2 = (n2 + pt2 - 1) / pt2, NT = nt0 + nt1 + nt2;
            // A CTA may run at most one tile ahead of its fair share (else the CTAs whose producers are furthest ahead would
            // hoard the tiles of a short phase), and near the end of the phase it claims the next tile only once its
            // consumers have caught up (else the tiles already sitting in its ring decide when the phase ends).
            const uint32_t cap = (NT + gridDim.x - 1) / gridDim.x + 1;
            uint32_t claimed = 1;
            uint32_t t = atomicAdd(P.tile_ctr + ph, 1u);
            while (t < NT) {
                const bool tail_zone = t + 2 * gridDim.x >= NT;
                uint32_t t_next = NT;   // = no further tile
                if (!tail_zone && claimed < cap) { t_next = atomicAdd(P.tile_ctr + ph, 1u); claimed++; }   // in flight while this tile waits for ring space
                uint32_t sgm, first, n, cost;
                if (t < nt0) { sgm = 0; first = t * pt0; n = min(pt0, n0 - first); cost = c0; }
                else if (t < nt0 + nt1) { sgm = 1; first = (t - nt0) * pt1; n = min(pt1, n1 - first); cost = c1; }
                else { sgm = 2; first = (t - nt0 - nt1) * pt2; n = min(pt2, n2 - first); cost = c2; }
                const uint32_t bytes = n * cost, bytes_al = (bytes + 127u) & ~127u;
                uint32_t gap = 0;
                if (off + bytes_al > RING) { gap = RING - off; off = 0; }
                const uint32_t need = bytes_al + gap;
                while (kt - tail >= NS || used + need > RING) {   // oldest tiles first: wait until the consumers have released them
                    if (ts->abort_flag || !mbar_wait(bar0 + 8 * (NS + (tail & (NS - 1))), (tail / NS) & 1, P.err, 2)) { stop = true; break; }
                    used -= ts->tile_bytes[tail & (NS - 1)];
                    tail++;
                }
                if (stop || ts->abort_flag) { stop = true; break; }
                const uint32_t slot = kt & (NS - 1);
                ts->tile_bytes[slot] = need;
                ts->meta[slot] = make_uint4(off, first, n | (sgm << 8), 0u);
                used += need;
                const uint32_t dst = smem_u32(ring + off), full = bar0 + 8 * slot;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(full, bytes);
                if (swiglu) {
                    const uint32_t ba = n * cur.rb0, bb = n * cur.rb1;
                    bulk_g2s(dst, cur.w0 + (size_t)first * cur.rb0, ba, full);
                    bulk_g2s(dst + ba, cur.w1 + (size_t)first * cur.rb1, bb, full);
                } else {
                    const uint8_t *w = sgm == 0 ? cur.w0 : (sgm == 1 ? cur.w1 : cur.w2);
                    bulk_g2s(dst, w + (size_t)first * cost, bytes, full);
                }
                off += bytes_al;
                kt++;
                if (tail_zone && claimed < cap) {
                    while (kt - tail > 1) {   // all but the tile just issued have been consumed
                        if (ts->abort_flag || !mbar_wait(bar0 + 8 * (NS + (tail & (NS - 1))), (tail / NS) & 1, P.err, 2)) { stop = true; break; }
                        used -= ts->tile_bytes[tail & (NS - 1)];
                        tail++;
                    }
                    if (stop) break;
                    t_next = atomicAdd(P.tile_ctr + ph, 1u);
                    claimed++;
                }
                t = t_next;
            }
            if (stop) break;
            // end-of-phase marker: a slot without data
            while (kt - tail >= NS) {
                if (ts->abort_flag || !mbar_wait(bar0 + 8 * (NS + (tail & (NS - 1))), (tail / NS) & 1, P.err, 2)) { stop = true; break; }
                used -= ts->tile_bytes[tail & (NS - 1)];
                tail++;
            }
            if (stop) break;
            ts->tile_bytes[kt & (NS - 1)] = 0;
            ts->meta[kt & (NS - 1)] = make_uint4(0u, 0u, 1u << 16, 0u);
            mbar_arrive(bar0 + 8 * (kt & (NS - 1)));
            kt++;
        }
        TK_TRACE_PROD(ph, 1);
        cur = nxt;
    }
    ts->issued = kt;
}

// Where the qkv epilogue appends the k / v rows: read from the phase descriptor at the moment of use (a few rows per
// CTA: no registers are held for them).
struct DescCaches {
    const PhaseShared *c;
    __device__ __forceinline__ void *k() const { return c->kc; }
    __device__ __forceinline__ void *v() const { return c->vc; }
};

// Epilogue of one row pair, by the phase's kind.  The parameters of each kind are the same for every layer.
__device__ __forceinline__ void phase_epilogue(const TokenProgram &P, const PhaseShared *d, uint32_t epi, uint32_t s, uint32_t pair, float a, float b,
                                               unsigned long long &best, float2 rpre) {
    switch (epi) {
    case EPI_QKV: epilogue<EPI_QKV>(P.qkv, s, pair, a, b, best, DescCaches{d}, rpre); break;
    case EPI_RESIDUAL: epilogue<EPI_RESIDUAL>(P.res, s, pair, a, b, best, DescCaches{d}, rpre); break;
    case EPI_SWIGLU: epilogue<EPI_SWIGLU>(P.gu, s, pair, a, b, best, DescCaches{d}, rpre); break;
    default: epilogue<EPI_ARGMAX>(P.cls, s, pair, a, b, best, DescCaches{d}, rpre); break;
    }
}

// ---- consumer side of one matrix phase: activation prologue, this warp's share of every tile, epilogues ----
// One body serves every phase (format and epilogue are looked up per tile / per row pair): the kernel stays small,
// and nothing of one phase is kept alive in registers during another.
__device__ __forceinline__ void gemv_phase(const TokenProgram &P, TkShared *ts, uint32_t &kt, uint32_t &off, unsigned long long &best, uint32_t ph) {
    const PhaseShared *d = &ts->cur;
    const uint32_t cols = d->cols;
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint8_t *ring = smem;
    uint8_t *act_sm = smem + P.geo.act_off;
    float *part = reinterpret_cast<float *>(smem + P.geo.part_off);             // [NS][PT_MAX][2][CW]
    uint32_t *cnt = reinterpret_cast<uint32_t *>(part + NS * PT_MAX * 2 * CW);  // [NS][CW]
    const uint32_t bar0 = smem_u32(smem + P.geo.bar_off);
    pack_activation_lean<TK_CONSUMERS>(act_sm, cols, d->x, d->norm_w, d->eps, ts->red, cols / 64);
    const Act A{act_sm, cols, cols / 64};
    TK_TRACE(ph, 2);

    const uint32_t epi = d->epi;
    const bool swiglu = epi == EPI_SWIGLU;
    const uint32_t rb0 = d->rb0, rb1 = d->rb1;
    const uint32_t units = cols / 64, CG = (units + 31) / 32, RG = TCW / CG;
    const bool working = (uint32_t)warp < CG * RG;
    const uint32_t cg = warp % CG, rg = warp / CG, u = cg * 32 + lane;
    const bool has_unit = working && u < units;
    TK_TRACE(ph, 5);

    UnitAct ua;
    LaneConst lc;
    uint32_t cur_type = d->qt0;   // the first segment's format: this lane's activations go to registers before any tile is waited for
    unit_init<QT_MIXED>(cur_type, u, lc);
    if (has_unit) load_unit_act(cur_type, u, A, ua);
    TK_TRACE(ph, 6);
    bool first_tile = true;
#pragma unroll 1
    for (;;) {
        const uint32_t st = kt & (NS - 1);
        if (ts->abort_flag || !mbar_wait(bar0 + 8 * st, (kt / NS) & 1, P.err, 1)) {
            ts->abort_flag = 1;   // give up on the rest of this phase; the next grid barrier ends the kernel for the whole CTA
            break;
        }
        const uint4 meta = ts->meta[st];
        if (meta.z >> 16) {   // end of the phase for this CTA
            __syncwarp();
            if (lane == 0) mbar_arrive(bar0 + 8 * (NS + st));
            kt++;
            break;
        }
        if (first_tile) { TK_TRACE(ph, 3); first_tile = false; }
        const uint32_t n = meta.z & 0xFFu, s = (meta.z >> 8) & 0xFFu, first = meta.y;
        const uint32_t qtype = s == 0 ? d->qt0 : (s == 1 ? d->qt1 : d->qt2);
        if (qtype != cur_type) {   // (re)load this lane's activations in the layout of the segment's format
            unit_init<QT_MIXED>(qtype, u, lc);
            if (has_unit) load_unit_act(qtype, u, A, ua);
            cur_type = qtype;
        }
        const uint32_t cost = swiglu ? rb0 + rb1 : 2 * (s == 0 ? rb0 : (s == 1 ? rb1 : d->rb2));
        const uint8_t *tile = ring + meta.x;
        // pair = rows 2r, 2r+1 of one segment (adjacent in the tile), or gate row r + up row r (two blocks of the tile)
        const uint32_t rbA = swiglu ? rb0 : cost / 2, rbB = swiglu ? rb1 : rbA;
        const uint32_t strideA = swiglu ? rbA : cost, offB = swiglu ? n * rbA : rbA, strideB = swiglu ? rbB : cost;
        float *pt = part + (size_t)st * PT_MAX * 2 * CW;
        if (working) {
            // residual values of the pair this lane may have to finish: requested now, needed after the dot products
            float2 rpre = make_float2(0.f, 0.f);
            if (epi == EPI_RESIDUAL && CG > 1 && rg + RG * lane < n) rpre = residual_prefetch(P.res.resid, first + rg + RG * lane);
            for (uint32_t pr = rg; pr < n; pr += RG) {
                const uint8_t *rowA = tile + pr * strideA;
                const uint8_t *rowB = tile + offB + pr * strideB;
                if (epi == EPI_RESIDUAL && CG == 1 && lane == 0) rpre = residual_prefetch(P.res.resid, first + pr);
                float va = 0.f, vb = 0.f;
                if (has_unit) {
                    va = unit_dot<QT_MIXED>(qtype, rowA, lc, ua);
                    vb = unit_dot<QT_MIXED>(qtype, rowB, lc, ua);
                }
#pragma unroll
                for (int o = 16; o; o >>= 1) {
                    va += __shfl_xor_sync(0xffffffffu, va, o);
                    vb += __shfl_xor_sync(0xffffffffu, vb, o);
                }
                if (CG == 1) {
                    if (lane == 0) phase_epilogue(P, d, epi, s, first + pr, va, vb, best, rpre);
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
                        for (uint32_t g = 0; g < CG; g++) {
                            va += pt[(pr * 2 + 0) * CW + g];
                            vb += pt[(pr * 2 + 1) * CW + g];
                        }
                        phase_epilogue(P, d, epi, s, first + pr, va, vb, best, rpre);
                    }
                    __syncwarp();
                    if (lane == 0) cnt[st * CW + rg] = 0;
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar0 + 8 * (NS + st));   // this warp is done with the tile
        kt++;
    }
}

// ---- attention phase: twelve of the CTA's consumer warps act as three independent 4-warp blocks ----
constexpr int TK_ATTN_BLOCKS = TCW / ATTN_WARPS;
template <int HS, int KVM, typename T>
__device__ __forceinline__ void attn_phase(const TokenProgram &P, uint32_t total, const void *kc, const void *vc) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int STEPS = KVM >= 8 ? 1 : (KVM >= 4 ? 2 : 4);   // cache-row steps held in registers: fewer with more query heads per group
    const AttnArgs &a = P.attn;
    const int warp = threadIdx.x >> 5, vl = warp >> 2, tid = threadIdx.x & (ATTN_THREADS - 1);
    if (vl >= TK_ATTN_BLOCKS) return;
    uint32_t nsplit, per;
    attn_split_plan(total, a.max_splits, nsplit, per, 16);   // short slices: one load round per warp, the merge is cheap
    const uint32_t n_kv = a.p.n_heads / KVM;
    constexpr bool QS = KVM * (16 / (int)sizeof(T)) >= 32;   // the query registers of the group would be 32 or more: stage q in shared memory
    constexpr uint32_t BLOCK_FLOATS = attn_block_smem_floats(HS, KVM) + KVM * HS;
    float *sm = reinterpret_cast<float *>(smem + P.geo.act_off) + (size_t)vl * BLOCK_FLOATS;
    // consecutive work items go to different SMs
    for (uint32_t item = vl * gridDim.x + blockIdx.x; item < n_kv * nsplit; item += TK_ATTN_BLOCKS * gridDim.x) {
        attn_block<HS, KVM, T, STEPS, QS>(a, kc, vc, item % n_kv, item / n_kv, nsplit, per, total, tid, 2 + vl, sm);
        attn_bar(2 + vl);
    }
}

// The consumer warps' walk through the token.  Returns the number of tiles this thread has seen complete.
template <int HS, int KVM, typename T>
__device__ __forceinline__ uint32_t consume_token(const TokenProgram &P, TkShared *ts, uint32_t epoch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t G = gridDim.x;
    // begin: x <- dequantized embedding row of the current token (transformer.rs:367-374, chat_llama2.rs:217-220);
    // rope_cs[j] <- (cos, sin)(pos * theta_j) shared by every layer of this token (rope.rs:75-79)
    {
        const uint32_t step = P.ctl->step, pos = P.ctl->pos;
        uint32_t token = __ldcg(P.seq + step);
        if (token >= P.vocab) token = P.vocab - 1;   // never index outside the table
        const uint8_t *row = P.embd.w + (size_t)token * P.embd.row_bytes;
        for (uint32_t i = blockIdx.x * TK_CONSUMERS + threadIdx.x; i < P.hidden; i += G * TK_CONSUMERS) P.x[i] = dequant_at(P.embd, row, i);
        if (blockIdx.x == 0 && threadIdx.x < P.half_head) {
            float sn, cs;
            sincosf((float)pos * P.theta[threadIdx.x], &sn, &cs);
            P.rope_cs[threadIdx.x] = make_float2(cs, sn);
        }
    }
    uint32_t kt = 0, off = 0;
    uint32_t target = epoch * P.barriers_per_token * G;   // arrivals before this launch
    unsigned long long best = 0ull;
#pragma unroll 1
    for (uint32_t ph = 0; ph < P.n_phases; ph++) {
        TK_TRACE(ph, 0);
        if (!phase_sync(P, P.phases + ph, target += G, ts)) return kt;
        TK_TRACE(ph, 1);
        if (ts->cur.kind == PH_ATTN) attn_phase<HS, KVM, T>(P, P.ctl->pos + 1, ts->cur.kc, ts->cur.vc);
        else gemv_phase(P, ts, kt, off, best, ph);
        TK_TRACE(ph, 4);
        TK_TRACE_DONE(ph);
    }
    // this CTA's arg-max candidate (the classifier is the only phase that tracks one)
#pragma unroll
    for (int o = 16; o; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (lane == 0) ts->best_sm[warp] = best;
    named_barrier(1, TK_CONSUMERS);
    if (threadIdx.x == 0) {
        unsigned long long b = 0ull;
        for (int w = 0; w < TCW; w++) b = max(b, ts->best_sm[w]);
        P.cls.argmax_slots[blockIdx.x] = b;
    }
    if (!phase_sync(P, nullptr, target += G, ts)) return kt;

    // end of token: greedy arg-max over the CTAs' candidates (models/sampler.rs:54-56), fed back when the prompt is
    // exhausted; advance step and position (sampler.rs:102-110, chat_llama2.rs:137-171)
    if (blockIdx.x == 0 && warp == 0) {
        unsigned long long b = 0ull;
        for (uint32_t i = lane; i < G; i += 32) b = max(b, __ldcg(P.cls.argmax_slots + i));
#pragma unroll
        for (int o = 16; o; o >>= 1) b = max(b, __shfl_xor_sync(0xffffffffu, b, o));
        if (lane == 0) {
            const uint32_t step = P.ctl->step, pos = P.ctl->pos;
            const uint32_t next = 0xFFFFFFFFu - (uint32_t)(b & 0xFFFFFFFFull);
            P.ctl->next = next;
            if (step + 1 >= P.ctl->n_prompt && step + 1 < P.seq_cap) P.seq[step + 1] = next;
            P.ctl->step = step + 1;
            P.ctl->pos = pos + 1;
            *P.epoch = epoch + 1;
        }
        for (uint32_t i = lane; i < P.n_phases; i += 32) P.tile_ctr[i] = 0u;   // every CTA is past every phase
    }
    return kt;
}

// One instance per attention shape (head size, query heads per kv head, cache element type); the matrix phases are
// generic.
template <int HS, int KVM, typename T>
__global__ void __maxnreg__(TK_REGS) token_kernel(const TokenProgram P) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ TkShared ts;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t bar0 = smem_u32(smem + P.geo.bar_off);
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < NS; s++) {
            mbar_init(bar0 + 8 * s, 1);            // full: the producer's expect_tx arrival
            mbar_init(bar0 + 8 * (NS + s), TCW);    // empty: one arrival per consumer warp
        }
        uint32_t *cnt = reinterpret_cast<uint32_t *>(reinterpret_cast<float *>(smem + P.geo.part_off) + NS * PT_MAX * 2 * CW);
        for (uint32_t i = 0; i < NS * CW; i++) cnt[i] = 0;
        ts.abort_flag = 0;
        ts.go = 1;
        ts.issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const uint32_t epoch = *P.epoch;
    __syncthreads();

    uint32_t seen = 0;
    if (warp == TCW) {
        if (lane == 0) produce_token(P, &ts, epoch);
    } else {
        seen = consume_token<HS, KVM, T>(P, &ts, epoch);
    }
    __syncthreads();
    // After a wait that gave up: copies the producer issued and nobody consumed may still be in flight; wait for them
    // (bounded) before the CTA's shared memory is released.
    if (threadIdx.x == 0 && ts.abort_flag) {
        const uint32_t issued = ts.issued;
        for (uint32_t k = seen; (int32_t)(issued - k) > 0; k++) mbar_wait(bar0 + 8 * (k & (NS - 1)), (k / NS) & 1, nullptr, 0);
    }
}

// -------------------------------------------------------------------------------------------------
// host side
// -------------------------------------------------------------------------------------------------
constexpr size_t TK_SMEM_LIMIT = 232448;   // 227 KB per CTA on sm_100

typedef void (*TokenKernelFn)(const TokenProgram);

template <int HS, typename T>
static TokenKernelFn token_kernel_kvm(uint32_t kv_mul) {
    switch (kv_mul) {
    case 1: return token_kernel<HS, 1, T>;
    case 2: return token_kernel<HS, 2, T>;
    case 4: return token_kernel<HS, 4, T>;
    case 8: return token_kernel<HS, 8, T>;
    default: return nullptr;
    }
}

// variant = head_size | kv_mul << 8 | f16 << 16
static TokenKernelFn token_kernel_variant(int variant) {
    const uint32_t hs = variant & 0xFF, kvm = (variant >> 8) & 0xFF;
    const bool f16 = (variant >> 16) & 1;
    if (hs == 128) return f16 ? token_kernel_kvm<128, __half>(kvm) : token_kernel_kvm<128, float>(kvm);
    if (hs == 64) return f16 ? token_kernel_kvm<64, __half>(kvm) : token_kernel_kvm<64, float>(kvm);
    return nullptr;
}

// Bytes of one row of `cols` columns in the device layout of a format (K-quants as in GGUF; Q6_K and Q8_0 re-tiled in
// groups of eight blocks), or 0 when the streaming kernel cannot take the format / width.
static uint32_t stream_row_bytes(uint32_t qt, uint32_t cols) {
    switch (qt) {
    case IB_Q4_K: return cols % 256 ? 0 : cols / 256 * 144;
    case IB_Q5_K: return cols % 256 ? 0 : cols / 256 * 176;
    case IB_Q6_K: return cols % 2048 ? 0 : cols / 2048 * 1680;
    case IB_Q8_0: return cols % 256 ? 0 : cols / 256 * 272;
    default: return 0;
    }
}

int32_t plan_token_kernel(ib_ctx *ctx, const TokenProgram &prog, const PhaseDesc *phases, TokenKernelPlan &plan) {
    plan.variant = (int)(prog.head_size | (prog.kv_mul << 8) | ((prog.kv_dtype == IB_KV_F16 ? 1u : 0u) << 16));
    TokenKernelFn fn = token_kernel_variant(plan.variant);
    if (!fn) return set_error(IB_ERR_UNSUPPORTED, "token kernel: head_size=%u, kv_mul=%u (supported: 64/128 and 1/2/4/8)", prog.head_size, prog.kv_mul);
    size_t act = 0, max_round = 0;
    for (uint32_t i = 0; i < prog.n_phases; i++) {
        const PhaseDesc &d = phases[i];
        if (d.kind != PH_GEMV) continue;
        if (d.cols % 64 || d.cols > 16384) return set_error(IB_ERR_UNSUPPORTED, "token kernel: %u columns do not meet the streaming rules", d.cols);
        if (d.epi != EPI_RESIDUAL && d.epi != EPI_SWIGLU && d.epi != EPI_QKV && d.epi != EPI_ARGMAX)
            return set_error(IB_ERR_UNSUPPORTED, "token kernel: epilogue %u is not part of the single-GPU token", d.epi);
        const uint32_t units = d.cols / 64, CG = (units + 31) / 32, RG = TCW / CG;
        const size_t a = (act_smem_bytes(d.cols) + 127) & ~(size_t)127;
        if (a > act) act = a;
        for (uint32_t s = 0; s < d.nseg; s++) {
            if (d.m[s].row_bytes == 0 || d.m[s].row_bytes != stream_row_bytes(d.m[s].qtype, d.cols) || d.rows[s] % 2)
                return set_error(IB_ERR_UNSUPPORTED, "token kernel: phase %u matrix %u (type %u, %u bytes per row, %u rows) does not meet the streaming rules", i, s,
                                 d.m[s].qtype, d.m[s].row_bytes, d.rows[s]);
            const size_t cost = d.epi == EPI_SWIGLU ? (size_t)d.m[0].row_bytes + d.m[1].row_bytes : (size_t)2 * d.m[s].row_bytes;
            if (cost * RG > max_round) max_round = cost * RG;
        }
    }
    const size_t attn = (((size_t)TK_ATTN_BLOCKS * (attn_block_smem_floats(prog.head_size, prog.kv_mul) + prog.kv_mul * prog.head_size) * sizeof(float)) + 127) & ~(size_t)127;
    if (attn > act) act = attn;
    cudaFuncAttributes fa;
    IB_CHECK_CUDA(cudaFuncGetAttributes(&fa, fn));
    const size_t part = (((size_t)NS * PT_MAX * 2 * CW * 4 + (size_t)NS * CW * 4) + 127) & ~(size_t)127;
    const size_t bars = 128;
    const size_t fixed = act + part + bars + ((fa.sharedSizeBytes + 127) & ~(size_t)127) + 1024;
    if (fixed + 2 * max_round > TK_SMEM_LIMIT)
        return set_error(IB_ERR_UNSUPPORTED, "token kernel: %zu bytes of activations and rounds of %zu bytes do not fit shared memory", act, max_round);
    const size_t ring = (TK_SMEM_LIMIT - fixed) & ~(size_t)127;
    uint32_t tile_max = TK_TILE_MAX;
    if (tile_max > ring / 2) tile_max = (uint32_t)(ring / 2);
    if (max_round > tile_max) return set_error(IB_ERR_UNSUPPORTED, "token kernel: a round of %zu bytes exceeds the tile limit of %u", max_round, tile_max);
    plan.geo.ring_bytes = (uint32_t)ring;
    plan.geo.act_off = (uint32_t)ring;
    plan.geo.act_bytes = (uint32_t)act;
    plan.geo.part_off = (uint32_t)(ring + act);
    plan.geo.bar_off = (uint32_t)(ring + act + part);
    plan.geo.tile_max = tile_max;
    plan.smem_bytes = ring + act + part + bars;
    plan.grid = ctx->sm_count;
    IB_CHECK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem_bytes));
    int per_sm = 0;
    IB_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, TK_THREADS, plan.smem_bytes));
    if (per_sm < 1) return set_error(IB_ERR_UNSUPPORTED, "token kernel: one CTA of %zu bytes of shared memory does not fit an SM", plan.smem_bytes);
    return IB_OK;
}

int32_t launch_token_kernel(ib_ctx *ctx, cudaStream_t stream, const TokenProgram &prog, const TokenKernelPlan &plan) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.grid);
    cfg.blockDim = dim3(TK_THREADS);
    cfg.dynamicSmemBytes = plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;   // every CTA is resident at once: the grid barriers rely on it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    IB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, token_kernel_variant(plan.variant), prog));
    ctx->launches++;
    return IB_OK;
}

#ifdef IB_TOKEN_TRACE
extern "C" __attribute__((visibility("default"))) int32_t ib_debug_token_trace(unsigned long long *out) {
    return cudaMemcpyFromSymbol(out, g_tk_trace, sizeof(unsigned long long) * 5 * 64 * 8) == cudaSuccess ? 0 : 2;
}
extern "C" __attribute__((visibility("default"))) int32_t ib_debug_token_done(unsigned long long *out) {
    return cudaMemcpyFromSymbol(out, g_tk_done, sizeof(unsigned long long) * 64 * 160) == cudaSuccess ? 0 : 2;
}
#endif

}  // namespace ib
