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
static_assert((NS & (NS - 1)) == 0, "slot count must be a power of two");

struct __align__(16) TkShared {
    TokenPhase desc[2];                 // descriptor of the current phase and the next one (double buffer)
    float red[PACK_THREADS / 32 + 1];
    unsigned long long best_sm[CW];
    volatile uint32_t abort_flag;       // a wait gave up somewhere in this CTA
    volatile uint32_t go;               // decision after a grid barrier, identical for every consumer thread
    volatile uint32_t issued;           // tiles the producer has issued (valid once it has stopped)
    uint32_t tile_bytes[NS];            // ring bytes held by the tile in each slot (producer's book-keeping)
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Grid barrier for the 512 consumer threads of every CTA.  Returns false (for every thread alike) when this CTA has to
// give up: its own wait ran out, or some warp of the CTA raised the abort flag earlier.
__device__ __forceinline__ bool grid_sync(uint32_t *ctr, uint32_t target, TkShared *ts, uint32_t *err) {
    named_barrier(1, PACK_THREADS);
    if (threadIdx.x == 0) {
        bool ok = ts->abort_flag == 0;
        if (ok) {
            __threadfence();
            atomicAdd(ctr, 1u);
            ok = (int32_t)(ld_acquire_gpu(ctr) - target) >= 0;
            if (!ok) {
                const unsigned long long t0 = global_ns();
                for (;;) {
                    for (int i = 0; i < 32 && !ok; i++) ok = (int32_t)(ld_acquire_gpu(ctr) - target) >= 0;
                    if (ok || global_ns() - t0 > WAIT_LIMIT_NS) break;
                }
            }
            if (!ok) {
                *(volatile uint32_t *)err = 5;
                __threadfence_system();
                ts->abort_flag = 1;
            }
            __threadfence();
        }
        ts->go = ok ? 1u : 0u;
    }
    named_barrier(1, PACK_THREADS);
    return ts->go != 0;
}

// ---- producer: one lane streams this CTA's share of every GEMV phase of the token into the byte ring ----
__device__ __forceinline__ const uint8_t *sel3(uint32_t s, const uint8_t *a, const uint8_t *b, const uint8_t *c) { return s == 0 ? a : (s == 1 ? b : c); }

__device__ __forceinline__ void produce_token(const TokenProgram &P, TkShared *ts) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *ring = smem;
    const uint32_t bar0 = smem_u32(smem + P.geo.bar_off);
    const uint32_t RING = P.geo.ring_bytes;
    uint32_t kt = 0, off = 0, used = 0, tail = 0;
    bool stop = false;
    PhaseStream cur = P.phases[0].ps;
    for (uint32_t ph = 0; ph < P.n_phases && !stop; ph++) {
        PhaseStream nxt = cur;
        if (ph + 1 < P.n_phases) nxt = P.phases[ph + 1].ps;   // in flight while this phase streams
        if (cur.kind == PH_GEMV) {
            if (cur.norm_w && blockIdx.x == ph % gridDim.x)     // the phase's norm weights: into L2 ahead of the consumers
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(cur.norm_w), "r"(cur.cols * 4u) : "memory");
            const uint32_t units = cur.cols / 64, CG = (units + 31) / 32, RG = CW / CG;
            const bool swiglu = cur.epi == EPI_SWIGLU;
            Share sh;
            make_share_rt(swiglu, cur.nseg, cur.rows[0], cur.rows[1], cur.rows[2], cur.row_bytes[0], cur.row_bytes[1], cur.row_bytes[2],
                          P.geo.tile_max, RG, gridDim.x, blockIdx.x, sh);
            TileCursor tc;
            tc.init(sh);
            for (; tc.valid(sh); tc.advance(sh)) {
                const uint32_t n = tc.count(sh), s = tc.seg;
                const uint32_t bytes = n * sh.cost(s), bytes_al = (bytes + 127u) & ~127u;
                uint32_t gap = 0;
                if (off + bytes_al > RING) { gap = RING - off; off = 0; }
                const uint32_t need = bytes_al + gap;
                while (kt - tail >= NS || used + need > RING) {   // oldest tiles first: wait until the consumers have released them
                    if (ts->abort_flag || !mbar_wait(bar0 + 8 * (NS + (tail & (NS - 1))), (tail / NS) & 1, P.err, 2)) { stop = true; break; }
                    used -= ts->tile_bytes[tail & (NS - 1)];
                    tail++;
                }
                if (stop || ts->abort_flag) { stop = true; break; }
                ts->tile_bytes[kt & (NS - 1)] = need;
                used += need;
                const uint32_t dst = smem_u32(ring + off), full = bar0 + 8 * (kt & (NS - 1));
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(full, bytes);
                if (swiglu) {
                    const uint32_t ba = n * cur.row_bytes[0], bb = n * cur.row_bytes[1];
                    bulk_g2s(dst, cur.w[0] + (size_t)tc.next * cur.row_bytes[0], ba, full);
                    bulk_g2s(dst + ba, cur.w[1] + (size_t)tc.next * cur.row_bytes[1], bb, full);
                } else {
                    bulk_g2s(dst, sel3(s, cur.w[0], cur.w[1], cur.w[2]) + (size_t)tc.next * sh.cost(s), bytes, full);
                }
                off += bytes_al;
                kt++;
            }
        }
        cur = nxt;
    }
    ts->issued = kt;
}

// ---- consumer side of one GEMV phase: activation prologue, this warp's share of every tile, epilogues ----
template <uint32_t EPI, uint32_t QT>
__device__ __noinline__ unsigned long long gemv_phase(const GemvParams *pp, const TokenGeom geo, TkShared *ts, uint32_t kt, uint32_t off) {
    extern __shared__ __align__(128) uint8_t smem[];
    const GemvParams &p = *pp;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint8_t *ring = smem;
    uint8_t *act_sm = smem + geo.act_off;
    float *part = reinterpret_cast<float *>(smem + geo.part_off);               // [NS][PT_MAX][2][CW]
    uint32_t *cnt = reinterpret_cast<uint32_t *>(part + NS * PT_MAX * 2 * CW);  // [NS][CW]
    const uint32_t bar0 = smem_u32(smem + geo.bar_off);

    float4 norm_g[4];
    pack_prefetch_norm(p.norm_w, p.cols, norm_g);
    pack_activation(act_sm, p.cols, p.x, p.norm_w, p.eps, ts->red, norm_g);
    const Act A{act_sm, p.cols};

    const uint32_t units = p.cols / 64, CG = (units + 31) / 32, RG = CW / CG;
    const bool working = (uint32_t)warp < CG * RG;
    const uint32_t cg = warp % CG, rg = warp / CG, u = cg * 32 + lane;
    const bool has_unit = working && u < units;
    Share sh;
    make_share<EPI>(p, geo.tile_max, RG, sh);

    UnitAct ua;
    LaneConst lc;
    uint32_t cur_type = 0xFFFFFFFFu;
    unsigned long long best = 0ull;
    TileCursor tc;
    tc.init(sh);
#pragma unroll 1
    for (; tc.valid(sh); tc.advance(sh)) {
        const uint32_t st = kt & (NS - 1), s = tc.seg, n = tc.count(sh);
        const uint32_t qtype = (QT != QT_MIXED) ? QT : p.seg[s].qtype;
        if (qtype != cur_type) {   // (re)load this lane's activations in the layout of the segment's format
            unit_init<QT>(qtype, u, lc);
            if (has_unit) load_unit_act(qtype, u, A, ua);
            cur_type = qtype;
        }
        const uint32_t bytes_al = (n * sh.cost(s) + 127u) & ~127u;
        if (off + bytes_al > geo.ring_bytes) off = 0;
        if (ts->abort_flag || !mbar_wait(bar0 + 8 * st, (kt / NS) & 1, p.err, 1)) {
            ts->abort_flag = 1;   // give up on the rest of this phase; the next grid barrier ends the kernel for the whole CTA
            break;
        }
        const uint8_t *tile = ring + off;
        const uint32_t rbA = (uint32_t)p.seg[s].row_bytes;
        const uint32_t rbB = (EPI == EPI_SWIGLU) ? (uint32_t)p.seg[1].row_bytes : rbA;
        const uint32_t strideA = (EPI == EPI_SWIGLU) ? rbA : 2 * rbA, offB = (EPI == EPI_SWIGLU) ? n * rbA : rbA;
        float *pt = part + (size_t)st * PT_MAX * 2 * CW;
        if (working) {
            for (uint32_t pr = rg; pr < n; pr += RG) {
                const uint8_t *rowA = tile + pr * strideA;
                const uint8_t *rowB = (EPI == EPI_SWIGLU) ? tile + offB + pr * rbB : rowA + rbA;
                float va = 0.f, vb = 0.f;
                if (has_unit) {
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
                        epilogue<EPI>(p, s, tc.next + pr, va, vb, best);
                    }
                    __syncwarp();
                    if (lane == 0) cnt[st * CW + rg] = 0;
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar0 + 8 * (NS + st));   // this warp is done with the tile
        off += bytes_al;
        kt++;
    }

    if (EPI == EPI_ARGMAX) {
        // this CTA's candidate; the end of the token folds the CTAs' candidates after the last grid barrier
#pragma unroll
        for (int o = 16; o; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
        if (lane == 0) ts->best_sm[warp] = best;
        named_barrier(1, PACK_THREADS);
        if (threadIdx.x == 0) {
            unsigned long long b = 0ull;
            for (int w = 0; w < CW; w++) b = max(b, ts->best_sm[w]);
            p.argmax_slots[blockIdx.x] = b;
        }
    }
    return ((unsigned long long)kt << 32) | off;
}

// ---- attention phase: the CTA's 16 consumer warps act as four independent 4-warp blocks ----
template <int HS, int KVM, typename T>
__device__ __noinline__ void attn_phase(const AttnArgs *ap, uint32_t act_off) {
    extern __shared__ __align__(128) uint8_t smem[];
    const AttnArgs &a = *ap;
    const int warp = threadIdx.x >> 5, vl = warp >> 2, tid = threadIdx.x & (ATTN_THREADS - 1);
    const uint32_t total = *a.pos_ptr + 1;
    uint32_t nsplit, per;
    attn_split_plan(total, a.max_splits, nsplit, per);
    const uint32_t n_kv = a.p.n_heads / a.p.kv_mul;
    float *sm = reinterpret_cast<float *>(smem + act_off) + (size_t)vl * attn_block_smem_floats(HS, KVM);
    // consecutive work items go to different SMs
    for (uint32_t item = vl * gridDim.x + blockIdx.x; item < n_kv * nsplit; item += 4 * gridDim.x) {
        attn_block<HS, KVM, T, 4>(a, item % n_kv, item / n_kv, nsplit, per, total, tid, 2 + vl, sm);
        attn_bar(2 + vl);
    }
}

template <int HS, typename T>
__device__ __forceinline__ void attn_phase_kvm(const AttnArgs *ap, uint32_t act_off, uint32_t kv_mul) {
    switch (kv_mul) {
    case 1: attn_phase<HS, 1, T>(ap, act_off); break;
    case 2: attn_phase<HS, 2, T>(ap, act_off); break;
    case 4: attn_phase<HS, 4, T>(ap, act_off); break;
    default: attn_phase<HS, 8, T>(ap, act_off); break;
    }
}

#define IB_PHASE_CASE(E, Q) \
    case (((E) << 8) | (Q)): r = gemv_phase<E, Q>(&d->g, P.geo, ts, kt, off); break;
#define IB_PHASE_CASES(E) \
    IB_PHASE_CASE(E, IB_Q4_K) IB_PHASE_CASE(E, IB_Q5_K) IB_PHASE_CASE(E, IB_Q6_K) IB_PHASE_CASE(E, IB_Q8_0) IB_PHASE_CASE(E, QT_MIXED)

// The consumer warps' walk through the token.  Returns the number of tiles this thread has seen complete.
__device__ __forceinline__ uint32_t consume_token(const TokenProgram &P, TkShared *ts, uint32_t epoch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t G = gridDim.x;
    // begin: x <- dequantized embedding row of the current token (transformer.rs:367-374, chat_llama2.rs:217-220);
    // rope_cs[j] <- (cos, sin)(pos * theta_j) shared by every layer of this token (rope.rs:75-79)
    const uint32_t step = P.ctl->step, pos = P.ctl->pos;
    {
        uint32_t token = __ldcg(P.seq + step);
        if (token >= P.vocab) token = P.vocab - 1;   // never index outside the table
        const uint8_t *row = P.embd.w + (size_t)token * P.embd.row_bytes;
        for (uint32_t i = blockIdx.x * PACK_THREADS + threadIdx.x; i < P.hidden; i += G * PACK_THREADS) P.x[i] = dequant_at(P.embd, row, i);
        if (blockIdx.x == 0 && threadIdx.x < P.half_head) {
            float sn, cs;
            sincosf((float)pos * P.theta[threadIdx.x], &sn, &cs);
            P.rope_cs[threadIdx.x] = make_float2(cs, sn);
        }
    }
    uint32_t kt = 0, off = 0, nb = 0;
    const uint32_t base = epoch * P.barriers_per_token;
    constexpr uint32_t DESC_VECS = sizeof(TokenPhase) / 16;
    for (uint32_t ph = 0; ph < P.n_phases; ph++) {
        TokenPhase *d = &ts->desc[ph & 1];
        if (warp == 1) asm volatile("cp.async.wait_all;" ::: "memory");   // this phase's descriptor has landed
        if (!grid_sync(P.grid_bar, (base + ++nb) * G, ts, P.err)) return kt;
        if (warp == 1 && ph + 1 < P.n_phases) {
            // next phase's descriptor: asynchronous copy into the other buffer (its readers are all past the barrier)
            const uint4 *src = reinterpret_cast<const uint4 *>(P.phases + ph + 1);
            const uint32_t dst = smem_u32(&ts->desc[(ph + 1) & 1]);
            for (uint32_t i = lane; i < DESC_VECS; i += 32)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst + 16 * i), "l"(src + i) : "memory");
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        if (d->ps.kind == PH_ATTN) {
            const bool f16 = P.kv_dtype == IB_KV_F16;
            if (P.head_size == 128) {
                if (f16) attn_phase_kvm<128, __half>(&d->a, P.geo.act_off, P.kv_mul);
                else attn_phase_kvm<128, float>(&d->a, P.geo.act_off, P.kv_mul);
            } else {
                if (f16) attn_phase_kvm<64, __half>(&d->a, P.geo.act_off, P.kv_mul);
                else attn_phase_kvm<64, float>(&d->a, P.geo.act_off, P.kv_mul);
            }
        } else {
            unsigned long long r = ((unsigned long long)kt << 32) | off;
            switch ((d->g.epi << 8) | d->qt) {
                IB_PHASE_CASES(EPI_RESIDUAL)
                IB_PHASE_CASES(EPI_SWIGLU)
                IB_PHASE_CASES(EPI_QKV)
                IB_PHASE_CASES(EPI_ARGMAX)
            default: break;
            }
            kt = (uint32_t)(r >> 32);
            off = (uint32_t)r;
        }
    }
    if (!grid_sync(P.grid_bar, (base + ++nb) * G, ts, P.err)) return kt;

    // end of token: greedy arg-max over the CTAs' candidates (models/sampler.rs:54-56), feed it back when the prompt
    // is exhausted, advance step and position (sampler.rs:102-110, chat_llama2.rs:137-171)
    if (blockIdx.x == 0 && warp == 0) {
        unsigned long long b = 0ull;
        for (uint32_t i = lane; i < G; i += 32) b = max(b, __ldcg(P.argmax_slots + i));
#pragma unroll
        for (int o = 16; o; o >>= 1) b = max(b, __shfl_xor_sync(0xffffffffu, b, o));
        if (lane == 0) {
            const uint32_t next = 0xFFFFFFFFu - (uint32_t)(b & 0xFFFFFFFFull);
            P.ctl->next = next;
            if (step + 1 >= P.ctl->n_prompt && step + 1 < P.seq_cap) P.seq[step + 1] = next;
            P.ctl->step = step + 1;
            P.ctl->pos = pos + 1;
            *P.epoch = epoch + 1;
        }
    }
    return kt;
}

__global__ void __maxnreg__(96) token_kernel(const TokenProgram P) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ TkShared ts;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t bar0 = smem_u32(smem + P.geo.bar_off);
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < NS; s++) {
            mbar_init(bar0 + 8 * s, 1);            // full: the producer's expect_tx arrival
            mbar_init(bar0 + 8 * (NS + s), CW);    // empty: one arrival per consumer warp
        }
        uint32_t *cnt = reinterpret_cast<uint32_t *>(reinterpret_cast<float *>(smem + P.geo.part_off) + NS * PT_MAX * 2 * CW);
        for (uint32_t i = 0; i < NS * CW; i++) cnt[i] = 0;
        ts.abort_flag = 0;
        ts.go = 1;
        ts.issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (uint32_t i = threadIdx.x; i < sizeof(TokenPhase) / 16; i += blockDim.x)
        reinterpret_cast<uint4 *>(&ts.desc[0])[i] = reinterpret_cast<const uint4 *>(P.phases)[i];
    const uint32_t epoch = *P.epoch;
    __syncthreads();

    uint32_t seen = 0;
    if (warp == CW) {
        if (lane == 0) produce_token(P, &ts);
    } else {
        seen = consume_token(P, &ts, epoch);
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

int32_t plan_token_kernel(ib_ctx *ctx, const TokenPhase *phases, uint32_t n, uint32_t head_size, uint32_t kv_mul, TokenKernelPlan &plan) {
    cudaFuncAttributes fa;
    IB_CHECK_CUDA(cudaFuncGetAttributes(&fa, token_kernel));
    size_t act = 0, max_round = 0;
    for (uint32_t i = 0; i < n; i++) {
        if (phases[i].ps.kind != PH_GEMV) continue;
        const GemvParams &g = phases[i].g;
        if (!gemv_stream_eligible(g)) return set_error(IB_ERR_UNSUPPORTED, "token kernel: a matrix of %u columns does not meet the streaming rules", g.cols);
        if (g.epi != EPI_RESIDUAL && g.epi != EPI_SWIGLU && g.epi != EPI_QKV && g.epi != EPI_ARGMAX)
            return set_error(IB_ERR_UNSUPPORTED, "token kernel: epilogue %u is not part of the single-GPU token", g.epi);
        const size_t a = (act_smem_bytes(g.cols) + 127) & ~(size_t)127;
        if (a > act) act = a;
        const uint32_t units = g.cols / 64, CG = (units + 31) / 32, RG = CW / CG;
        for (uint32_t s = 0; s < g.nseg; s++) {
            const size_t cost = g.epi == EPI_SWIGLU ? (size_t)(g.seg[0].row_bytes + g.seg[1].row_bytes) : (size_t)(2 * g.seg[s].row_bytes);
            if (cost * RG > max_round) max_round = cost * RG;
        }
    }
    if ((head_size != 64 && head_size != 128) || (kv_mul != 1 && kv_mul != 2 && kv_mul != 4 && kv_mul != 8))
        return set_error(IB_ERR_UNSUPPORTED, "token kernel: head_size=%u, kv_mul=%u (supported: 64/128 and 1/2/4/8)", head_size, kv_mul);
    const size_t attn = (((size_t)4 * attn_block_smem_floats(head_size, kv_mul) * sizeof(float)) + 127) & ~(size_t)127;
    if (attn > act) act = attn;
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
    IB_CHECK_CUDA(cudaFuncSetAttribute(token_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem_bytes));
    int per_sm = 0;
    IB_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, token_kernel, STREAM_THREADS, plan.smem_bytes));
    if (per_sm < 1) return set_error(IB_ERR_UNSUPPORTED, "token kernel: one CTA of %zu bytes of shared memory does not fit an SM", plan.smem_bytes);
    return IB_OK;
}

int32_t launch_token_kernel(ib_ctx *ctx, cudaStream_t stream, const TokenProgram &prog, const TokenKernelPlan &plan) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.grid);
    cfg.blockDim = dim3(STREAM_THREADS);
    cfg.dynamicSmemBytes = plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;   // every CTA is resident at once: the grid barriers rely on it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    IB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, token_kernel, prog));
    ctx->launches++;
    return IB_OK;
}

}  // namespace ib
