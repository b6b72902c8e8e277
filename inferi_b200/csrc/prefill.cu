// Prompt prefill: the prompt's tokens go through every matrix together, as GEMMs on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory), instead of one by one through the decode path.
//
// The reference has no prefill: `ChatLlama2::forward` forces the prompt through the decode path token by token
// (crates/inferi-chat/src/chat_llama2.rs:137-155, crates/inferi-chat/src/sampler.rs:102-107), which reads every weight
// once per prompt token.  Here the weights are read once per prompt.
//
// Two GEMM kernels, both out^T tile = W tile (128 rows of the quantized matrix) x X^T (the tokens' input vectors):
// gemm_kquant_tc_kernel for Q4_K / Q5_K (exact integer weights on the tensor cores; its own comment below) and
// gemm_quant_tc_kernel for Q6_K and everything else:
//  * the quantized blocks of the tile's 128 rows travel to shared memory by tiled TMA copies (one 256-column block of every
//    row per step, a ring of steps ahead of their use) - no thread-per-row global loads, which were 32 cache lines per load
//    instruction and kept the L1 busy 91 % of the time;
//  * sixteen producer warps, four threads per weight row: read the row's block from shared memory, dequantize 64 columns of
//    the row per stage to f32, split the value into two f16 (w = hi + lo, exact to ~2^-22) and store both into shared
//    memory in the K-major core-matrix layout the tensor core reads (8 rows x 16 bytes per core matrix, no swizzle);
//  * the tokens' inputs (already split into f16 hi / lo by the kernel that produced them, and laid out in global memory
//    as tiles of that same layout) arrive by one bulk copy per tile, requested by a loader thread into a ring of their own;
//  * one thread issues, per 16 columns, three tcgen05.mma (hi x hi, hi x lo, lo x hi; lo x lo is below f32 resolution)
//    that accumulate in f32 in tensor memory: the result matches an f32 GEMV to ~1e-6 relative;
//  * shared-memory stages cycle through mbarriers (filled by the producers, released by tcgen05.commit);
//  * when a tile's K range is done the producer warps read the accumulator (tcgen05.ld: TMEM lane = weight row, column =
//    token) and store it transposed, [token][row], coalesced over the rows.
// The (tile, 256-column block) units of a matrix are dealt out as equal contiguous ranges over one wave of CTAs (StreamK in
// prefill.cuh); a tile whose K range falls to several CTAs gets one partial plane per CTA, and the element-wise kernel that
// follows (RoPE + cache append, residual add, SwiGLU) adds a tile's planes in CTA order.
// Every wait is bounded; a wait that gives up raises the context's error word and the kernel returns after freeing its
// tensor memory.
#include "prefill.cuh"

#include <cuda.h>   // CUtensorMap and the enumerations of cuTensorMapEncodeTiled (the entry point is looked up at run time)

namespace ib {

constexpr int TC_ROWS = 128;              // weight rows per CTA = M of the MMA
constexpr int TC_KSTAGE = 64;             // columns per stage
constexpr int TC_STAGES = 2;                // stages of the weights' split f16 tiles (W hi, W lo: 32 KiB each)
constexpr int TC_XSTAGES = 3;               // stages of the inputs' tiles (X hi, X lo: 32 KiB each), requested further ahead: they come from L2
constexpr uint32_t TC_RAW_MAX = 4;         // most stages of raw blocks (as many as fit are used)
constexpr int TC_PRODUCER_WARPS = 16;      // four threads per weight row, 16 columns each per stage (4 warps per scheduler hide the conversion's latencies)
constexpr int TC_THREADS = (TC_PRODUCER_WARPS + 2) * 32;   // + the MMA warp + the warp that requests the inputs' tiles
constexpr uint32_t TC_TILE_BYTES = TC_ROWS * TC_KSTAGE * 2;                  // one f16 tile of 128 x 64
constexpr uint32_t TC_STAGE_BYTES = 2 * TC_TILE_BYTES;                        // hi and lo
constexpr uint32_t TC_SMEM_FIXED = (TC_STAGES + TC_XSTAGES) * TC_STAGE_BYTES + 1024 + 1024;  // + barriers and TMEM address, + slack to align the tiles to 1 KiB
constexpr uint32_t TC_SMEM_LIMIT = 227 * 1024;

__device__ __forceinline__ uint32_t tc_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long tc_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, unsigned long long limit_ns, uint32_t *err, uint32_t code) {
    uint32_t ok = 0;
    // the common case - the phase is already complete - costs one instruction; the clock (a long-latency read) is only
    // looked at once a try has failed
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    const unsigned long long t0 = tc_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++) {
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
            if (ok) return true;
        }
        if (tc_ns() - t0 > limit_ns) break;
    }
    if (err) {
        *(volatile uint32_t *)err = code;
        __threadfence_system();
    }
    return false;
}

// Shared-memory matrix descriptor of a K-major tile without swizzle: core matrices of 8 rows x 16 bytes, `lbo` bytes
// between core matrices that are neighbours along K, `sbo` bytes between 8-row groups.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);          // bits 0-13: start address / 16
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;           // bits 16-29: leading-dimension byte offset / 16
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;           // bits 32-45: stride-dimension byte offset / 16
    d |= (uint64_t)1 << 46;                                 // bits 46-47: descriptor version of this architecture
    return d;                                               // base offset 0, layout type 0 = no swizzle
}
// Instruction descriptor of kind::f16: f16 A and B (both K-major), f32 accumulator, M x N.
__device__ __forceinline__ uint32_t tc_idesc_f16(uint32_t M, uint32_t N) {
    return (1u << 4) | ((N >> 3) << 17) | ((M >> 4) << 24);   // c_format = f32; a/b format 0 = f16; no negation, no transposition
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    const uint32_t zero = 0;   // no output lane is masked off
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem), "l"(a_desc),
        "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(zero)
        : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Element (row, k) of a 64-column K-major tile in the core-matrix layout: byte offset.  LBO = 128, SBO = 1024.
constexpr uint32_t TC_LBO = 128, TC_SBO = (TC_KSTAGE / 8) * 128;
__device__ __forceinline__ uint32_t tc_chunk_off(uint32_t row, uint32_t k8) { return (row >> 3) * TC_SBO + k8 * TC_LBO + (row & 7) * 16; }

// ---- 16 consecutive weights of a row (k0 a multiple of 16) as f32 ----
__device__ __forceinline__ float tc_h2f(uint32_t bits16) { return __half2float(__ushort_as_half((unsigned short)bits16)); }

// How a matrix reaches the producers.  0: Q4_K, 1: Q5_K (gemm_kquant_tc_kernel), 2: Q6_K in the 8-block row layout - their
// blocks are copied into shared memory by tiled TMA copies, one 256-column block of every row of the tile per step;
// 3: everything else (read from global memory element by element).
constexpr int TC_PATH_Q4K = 0, TC_PATH_Q5K = 1, TC_PATH_Q6K = 2, TC_PATH_OTHER = 3;
__host__ __device__ inline int tc_path(uint32_t qtype, uint32_t layout) {
    return qtype == IB_Q4_K ? TC_PATH_Q4K : (qtype == IB_Q5_K ? TC_PATH_Q5K : ((qtype == IB_Q6_K && layout == LAYOUT_SOA) ? TC_PATH_Q6K : TC_PATH_OTHER));
}
// A raw stage holds one block of each of the tile's 128 rows.  Row strides are odd multiples of 16 bytes, so that the 16-byte
// reads of 8 consecutive rows fall into different bank groups.  Q6_K: four arrays (low bits, high bits, scales, d).
constexpr uint32_t TC_Q6_QL = 0, TC_Q6_QH = TC_ROWS * 144, TC_Q6_SC = TC_Q6_QH + TC_ROWS * 80, TC_Q6_D = TC_Q6_SC + TC_ROWS * 16;
__host__ __device__ constexpr uint32_t tc_raw_stage_bytes(int path) {
    return path == TC_PATH_Q4K ? TC_ROWS * 144u : (path == TC_PATH_Q5K ? TC_ROWS * 176u : (path == TC_PATH_Q6K ? TC_Q6_D + TC_ROWS * 16u : 0u));
}

__device__ __forceinline__ uint4 tc_lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t tc_lds8(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t tc_lds16(uint32_t a) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}

// The thread's bytes of 16 weights - sixteenth `kq` (0..3) of the 64-column quarter `c` of the block: shared memory -> registers.
struct TcRaw {
    uint4 q, h;       // Q6_K: 16 bytes of low bits, 16 bytes of high bits
    uint32_t s, d;    // the scale of the 16 weights, the block's f16 scale
};
template <int PATH>
__device__ __forceinline__ void tc_read_raw(uint32_t raw, uint32_t row, uint32_t kb, uint32_t c, uint32_t kq, TcRaw &r) {
    const uint32_t hq = kq & 1;   // which 16 of the sub-block's 32 weights
    if (PATH == TC_PATH_Q6K) {
        const uint32_t i = c >> 1, g = (2 * c + (kq >> 1)) & 3;
        r.q = tc_lds128(raw + TC_Q6_QL + row * 144 + 64 * i + 32 * (g & 1) + 16 * hq);
        r.h = tc_lds128(raw + TC_Q6_QH + row * 80 + 32 * i + 16 * hq);
        r.s = tc_lds8(raw + TC_Q6_SC + row * 16 + 8 * i + 2 * g + hq);
        r.d = tc_lds16(raw + TC_Q6_D + row * 16 + 2 * (kb & 7));
    }
}

// crates/inferi/src/quantization.rs:227-256, rows stored as groups of 8 blocks [8 x 128 ql][8 x 64 qh][8 x 16 scales][8 x 2 d]
__device__ __forceinline__ void tc_convert16_q6k_soa(const TcRaw &r, uint32_t k0, float (&w)[16]) {
    const uint32_t g = ((k0 & 255) >> 5) & 3;
    const float sc = tc_h2f(r.d) * (float)(int)(int8_t)(r.s & 0xFF);
    const uint32_t lw[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
    const uint32_t hw[4] = {r.h.x, r.h.y, r.h.z, r.h.w};
#pragma unroll
    for (int wi = 0; wi < 4; wi++) {
        const uint32_t nib = (g & 2) ? (lw[wi] >> 4) & 0x0F0F0F0Fu : lw[wi] & 0x0F0F0F0Fu;
        const uint32_t q = nib | (((hw[wi] >> (2 * g)) & 0x03030303u) << 4);
#pragma unroll
        for (int bt = 0; bt < 4; bt++) w[4 * wi + bt] = sc * (float)((int)((q >> (8 * bt)) & 0xFFu) - 32);
    }
}

template <int PATH>
__device__ __forceinline__ void tc_convert16(const QDesc &q, const uint8_t *row, const TcRaw &r, uint32_t k0, float (&w)[16]) {
    if (PATH == TC_PATH_Q6K) tc_convert16_q6k_soa(r, k0, w);
    else {
#pragma unroll
        for (int e = 0; e < 16; e++) w[e] = dequant_at(q, row, k0 + e);   // unrolled: w stays in registers
    }
}

// The tokens' inputs in global memory are laid out the way the tensor core reads them from shared memory: per 64 columns
// one tile of 128 token rows in the K-major core-matrix layout (16 KiB), so that a stage's tile is one bulk copy.
__host__ __device__ inline size_t tc_x_index(uint32_t t, uint32_t c) {
    return (size_t)(c >> 6) * (TC_ROWS * TC_KSTAGE) + ((t >> 3) * TC_SBO + ((c & 63) >> 3) * TC_LBO + (t & 7) * 16) / 2 + (c & 7);
}

// Behind the input tiles of a vector of `cols` columns sit the tiles of its sub-block sums: per 256 columns one tile of 128
// token rows x 16 halves in the same core-matrix layout (K = 16: the sums of the unit's eight 32-column sub-blocks, then
// eight zeros), hi and lo halves like the inputs.  The k-quant GEMM multiplies them with the sub-blocks' minimums.
__host__ __device__ inline size_t tc_s_index(uint32_t t, uint32_t sb, uint32_t cols) {
    return (size_t)TC_ROWS * cols + (size_t)(sb >> 3) * (TC_ROWS * 16) + ((t >> 3) * 256 + (t & 7) * 16) / 2 + (sb & 7);
}
__host__ __device__ inline size_t tc_x_halves(uint32_t cols) { return (size_t)(TC_ROWS + 8) * cols; }   // halves per split buffer (hi or lo)

struct GemmTcParams {
    QDesc w;                    // the quantized matrix, device layout
    uint32_t rows, cols;        // rows % 128 == 0, cols % 256 == 0
    const __half *x_hi, *x_lo;  // the tokens' inputs split into two f16, tiled (tc_x_index); rows n_tokens .. n_pad-1 are zero
    uint32_t n_tokens, n_pad;   // n_pad = n_tokens rounded up to 16, <= 128
    float *out;                 // [piece][n_tokens][rows] partial planes
    StreamK sk;                 // the hand-out of (tile, 256-column block) units; gridDim.x == sk.ctas
    uint32_t raw_stages;        // depth of the ring of raw blocks
    uint32_t *err;
    unsigned long long wait_ns;
};

// The accumulator of one (tile, K range) segment: TMEM lane = weight row, column = token; stored as [token][row].  A warp
// reaches the 32 lanes 32 * (warp % 4); the four warps that share a lane group take every fourth group of 16 token columns.
__device__ __forceinline__ void tc_drain(const GemmTcParams &p, uint32_t tmem_base, int warp, uint32_t row, float *out) {
    const uint32_t groups = p.n_pad / 16;
    const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    for (uint32_t c0 = 16 * (warp >> 2); c0 < 16 * groups; c0 += 16 * (TC_PRODUCER_WARPS / 4)) {
        uint32_t r[16];
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
                       "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                     : "r"(taddr + c0)
                     : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; j++)
            if (c0 + j < p.n_tokens) out[(size_t)(c0 + j) * p.rows + row] = __uint_as_float(r[j]);
    }
}

template <int PATH>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_quant_tc_kernel(const GemmTcParams p, const __grid_constant__ CUtensorMap map_ql,
                                                                      const __grid_constant__ CUtensorMap map_qh, const __grid_constant__ CUtensorMap map_16) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t RAW_BYTES = tc_raw_stage_bytes(PATH);
    const uint32_t R = p.raw_stages;
    uint8_t *xst = smem + TC_STAGES * TC_STAGE_BYTES;                                   // the inputs' stages
    const uint32_t raw0 = tc_smem_u32(smem + (TC_STAGES + TC_XSTAGES) * TC_STAGE_BYTES);
    // barriers: full[S], empty[S], accumulator, raw_full[RAW_MAX], raw_empty[RAW_MAX], x_full[XS], x_empty[XS]
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (TC_STAGES + TC_XSTAGES) * TC_STAGE_BYTES + R * RAW_BYTES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * TC_STAGES + 1 + 2 * TC_RAW_MAX + 2 * TC_XSTAGES);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bar0 = tc_smem_u32(bars);
    const uint32_t bar_acc = bar0 + 8 * (2 * TC_STAGES), bar_rawfull = bar_acc + 8, bar_rawempty = bar_rawfull + 8 * TC_RAW_MAX;
    const uint32_t bar_xfull = bar_rawempty + 8 * TC_RAW_MAX, bar_xempty = bar_xfull + 8 * TC_XSTAGES;
    // this CTA's units: u0 .. u1-1 of the tile-major list of (tile, 256-column block); four 64-column stages per unit
    const StreamK sk = p.sk;
    const uint32_t u0 = sk.first_unit(blockIdx.x), u1 = sk.first_unit(blockIdx.x + 1), nunits = u1 - u0, nstage = 4 * nunits;

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + 8 * s), "r"(TC_PRODUCER_WARPS));   // full: one arrival per producer warp
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + 8 * (TC_STAGES + s)), "r"(1));  // empty: one tcgen05.commit
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_acc), "r"(1));       // a segment's accumulator is complete
        for (uint32_t s = 0; s < TC_RAW_MAX; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_rawfull + 8 * s), "r"(1));                          // the copying thread's arrival + the bytes
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_rawempty + 8 * s), "r"(TC_PRODUCER_WARPS));         // every producer warp has read it
        }
        for (int s = 0; s < TC_XSTAGES; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_xfull + 8 * s), "r"(1));    // the requesting thread's arrival + the bytes
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_xempty + 8 * s), "r"(1));   // one tcgen05.commit
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_PRODUCER_WARPS) {
        // tensor memory for the 128 x n_pad f32 accumulator: 128 columns (a power of two >= 32), allocated by one warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)), "r"(128u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    bool ok = true;

    if (warp < TC_PRODUCER_WARPS) {
        // ===== producers: thread = (weight row `tid & 127` of the unit's tile, quarter `tid >> 7` of the stage's 64 columns) =====
        const uint32_t row = tid & (TC_ROWS - 1), kq = tid >> 7;
        constexpr bool RAW = PATH != TC_PATH_OTHER;
        // Every index of the loop is carried forward by additions: a division by a run-time value (ring depth, blocks per
        // row) per stage and thread costs more instructions than the 16 weights' conversion.
        uint32_t tile = u0 / sk.nb, kb = u0 - tile * sk.nb;          // the current unit
        uint32_t ptile = tile, pkb = kb;                              // the next unit to request into the ring
        auto row_at = [&](uint32_t t) { return p.w.w + (size_t)(t * TC_ROWS + row) * p.w.row_bytes; };
        // The ring of raw blocks is filled ahead, one block of each of the unit's 128 rows per step.  The re-tiled Q6_K row keeps a
        // block's low bits, high bits, scales and d in four places: four tiled TMA copies (boxes of 128 rows; the boxes of the low
        // and high bits are 16 bytes wider than the field, which gives the shared-memory rows their conflict-free strides of
        // 144 and 80 bytes - the extra bytes are the row's own next bytes and are never read).
        auto issue_raw = [&](uint32_t t, uint32_t b, uint32_t dst, uint32_t bar) {
            const uint32_t x0 = (b >> 3) * 1680, bb = b & 7, y = t * (uint32_t)TC_ROWS;
            auto copy = [&](const CUtensorMap &map, uint32_t d, uint32_t x) {
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(d),
                             "l"(reinterpret_cast<uint64_t>(&map)), "r"(x), "r"(y), "r"(bar)
                             : "memory");
            };
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)TC_ROWS * (144u + 80u + 16u + 16u)) : "memory");
            copy(map_ql, dst + TC_Q6_QL, x0 + 128 * bb);
            copy(map_qh, dst + TC_Q6_QH, x0 + 1024 + 64 * bb);
            copy(map_16, dst + TC_Q6_SC, x0 + 1536 + 16 * bb);
            copy(map_16, dst + TC_Q6_D, x0 + 1664);
        };
        uint32_t issued = 0;
        for (; issued < R && issued < nunits; issued++) {
            if (RAW && tid == 0) issue_raw(ptile, pkb, raw0 + issued * RAW_BYTES, bar_rawfull + 8 * issued);
            if (++pkb == sk.nb) { pkb = 0; ptile++; }
        }
        uint32_t slot = 0, slot_par = 0;        // ring slot of the current unit and the parity of its use
        uint32_t pslot = 0, pslot_par = 0;      // the same for the previous unit (the slot that is refilled next)
        const uint8_t *wrow = row_at(tile);
        uint32_t seg = 0;   // segments (tile, K range) finished so far: the parity of the accumulator barrier
        for (uint32_t it = 0; it < nstage && ok; it++) {
            const uint32_t s = it % TC_STAGES, round = it / TC_STAGES;
            const uint32_t j = it >> 2, c = it & 3, u = u0 + j;
            if (c == 0 && j >= 1) {
                pslot = slot; pslot_par = slot_par;
                if (++slot == R) { slot = 0; slot_par ^= 1u; }
                if (++kb == sk.nb) { kb = 0; tile++; }
                wrow = row_at(tile);
            }
            if (RAW && c == 0) {
                if (j >= 1 && issued < nunits) {
                    // the slot of the previous step is refilled once every producer thread has read it
                    if (warp == 0) {
                        ok = __all_sync(0xffffffffu, tc_wait(bar_rawempty + 8 * pslot, pslot_par, p.wait_ns, p.err, 8));   // warp-uniform: the lanes stay together
                        if (!ok) break;
                        if (lane == 0) issue_raw(ptile, pkb, raw0 + pslot * RAW_BYTES, bar_rawfull + 8 * pslot);
                    }
                    issued++;
                    if (++pkb == sk.nb) { pkb = 0; ptile++; }
                }
                ok = __all_sync(0xffffffffu, tc_wait(bar_rawfull + 8 * slot, slot_par, p.wait_ns, p.err, 8));
                if (!ok) break;
            }
            const uint32_t k0 = kb * 256 + c * TC_KSTAGE + 16 * kq;
            TcRaw raw;
            if (RAW) tc_read_raw<PATH>(raw0 + slot * RAW_BYTES, row, kb, c, kq, raw);
            float w[16];
            tc_convert16<PATH>(p.w, wrow, raw, k0, w);
            if (RAW && c == 3) {
                __syncwarp();   // every lane has read its part of the raw stage
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_rawempty + 8 * slot) : "memory");
            }
            if (round > 0) ok = __all_sync(0xffffffffu, tc_wait(bar0 + 8 * (TC_STAGES + s), (round - 1) & 1, p.wait_ns, p.err, 8));
            if (!ok) break;
            uint8_t *st = smem + s * TC_STAGE_BYTES;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint4 hi, lo;
                uint32_t *hp = &hi.x, *lp = &lo.x;
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float a = w[8 * h + 2 * e], b2 = w[8 * h + 2 * e + 1];
                    const __half2 hh = __floats2half2_rn(a, b2);
                    const float2 back = __half22float2(hh);
                    const __half2 l = __floats2half2_rn(a - back.x, b2 - back.y);
                    hp[e] = *reinterpret_cast<const uint32_t *>(&hh);
                    lp[e] = *reinterpret_cast<const uint32_t *>(&l);
                }
                const uint32_t off = tc_chunk_off(row, 2 * kq + h);
                *reinterpret_cast<uint4 *>(st + off) = hi;
                *reinterpret_cast<uint4 *>(st + TC_TILE_BYTES + off) = lo;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads shared memory through the async proxy
            __syncwarp();   // one arrival per warp, behind every lane's stores and fence
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar0 + 8 * s) : "memory");
            if (c == 3 && (kb + 1 == sk.nb || u + 1 == u1)) {
                // the tile's K range in this CTA ends here: when its MMAs are done, the accumulator goes to the plane that
                // this CTA holds among the tile's CTAs.  The next segment's first stage only becomes full after every
                // producer warp has arrived on it, i.e. after every warp is through with this read of tensor memory.
                ok = __all_sync(0xffffffffu, tc_wait(bar_acc, seg & 1, p.wait_ns, p.err, 10));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t piece = blockIdx.x - sk.cta_of(tile * sk.nb);
                tc_drain(p, tmem_base, warp, tile * TC_ROWS + row, p.out + (size_t)piece * p.n_tokens * p.rows);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                seg++;
            }
        }
        if (!ok) {
            // a wait gave up: bulk copies of this CTA may still be in flight; give them time to land before the CTA ends
            const unsigned long long t0 = tc_ns();
            while (tc_ns() - t0 < 100000ull) {}
        }
    } else if (warp == TC_PRODUCER_WARPS && lane == 0) {
        // ===== MMA issue: one thread =====
        const uint32_t idesc = tc_idesc_f16(TC_ROWS, p.n_pad);
        // per MMA the issuing thread does as little as possible (it is one warp's serial instruction stream): the
        // descriptors of stage 0 are built once, the block index is carried by additions
        const uint64_t wdesc0 = tc_smem_desc(tc_smem_u32(smem), TC_LBO, TC_SBO), xdesc0 = tc_smem_desc(tc_smem_u32(xst), TC_LBO, TC_SBO);
        uint32_t kb = u0 % sk.nb;
        for (uint32_t it = 0; it < nstage && ok; it++) {
            const uint32_t s = it % TC_STAGES, round = it / TC_STAGES;
            const uint32_t xs = it % TC_XSTAGES;
            const uint32_t j = it >> 2, c = it & 3, u = u0 + j;
            if (c == 0 && j >= 1 && ++kb == sk.nb) kb = 0;
            const bool seg_first = c == 0 && (j == 0 || kb == 0), seg_last = c == 3 && (kb + 1 == sk.nb || u + 1 == u1);
            ok = tc_wait(bar_xfull + 8 * xs, (it / TC_XSTAGES) & 1, p.wait_ns, p.err, 9) && tc_wait(bar0 + 8 * s, round & 1, p.wait_ns, p.err, 9);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // descriptors differ from the stage-0 ones only in the start-address field (units of 16 bytes): one addition each
            const uint64_t wh = wdesc0 + s * (TC_STAGE_BYTES >> 4), wl = wh + (TC_TILE_BYTES >> 4);
            const uint64_t xh = xdesc0 + xs * (TC_STAGE_BYTES >> 4), xl = xh + (TC_TILE_BYTES >> 4);
#pragma unroll
            for (uint32_t kk = 0; kk < TC_KSTAGE / 16; kk++) {
                const uint32_t ko = kk * (2 * TC_LBO >> 4);   // 16 columns = two core matrices along K
                tc_mma_f16(tmem_base, wh + ko, xh + ko, idesc, !(seg_first && kk == 0));   // a segment starts a new sum
                tc_mma_f16(tmem_base, wh + ko, xl + ko, idesc, 1);
                tc_mma_f16(tmem_base, wl + ko, xh + ko, idesc, 1);
            }
            tc_commit(bar0 + 8 * (TC_STAGES + s));   // the stage is free again once these MMAs have read it
            tc_commit(bar_xempty + 8 * xs);
            if (seg_last) tc_commit(bar_acc);         // ... and the segment's accumulator is complete when all of them are done
        }
    }

    if (warp == TC_PRODUCER_WARPS + 1 && lane == 0) {
        // ===== the inputs' tiles: two bulk copies per stage (hi, lo), straight into the layout the tensor core reads, as far
        // ahead as there are stages =====
        bool okx = true;
        for (uint32_t it = 0; it < nstage && okx; it++) {
            const uint32_t xs = it % TC_XSTAGES;
            if (it >= (uint32_t)TC_XSTAGES) okx = tc_wait(bar_xempty + 8 * xs, (it / TC_XSTAGES - 1) & 1, p.wait_ns, p.err, 8);
            if (!okx) break;
            const uint32_t full = bar_xfull + 8 * xs, dst = tc_smem_u32(xst + xs * TC_STAGE_BYTES);
            const uint32_t kb = (u0 + (it >> 2)) % sk.nb;
            const size_t at = (size_t)(4 * kb + (it & 3)) * (TC_ROWS * TC_KSTAGE);
            // the tile's first n_pad token rows are its first n_pad / 8 groups of 1 KiB: only those are read by the MMA
            const uint32_t xbytes = p.n_pad * (TC_KSTAGE * 2);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"(2 * xbytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(p.x_hi + at), "r"(xbytes),
                         "r"(full)
                         : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst + TC_TILE_BYTES), "l"(p.x_lo + at),
                         "r"(xbytes), "r"(full)
                         : "memory");
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == TC_PRODUCER_WARPS) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128u) : "memory");
}


// ---------------------------------------------------------------------------------------------------------------------
// gemm_kquant_tc_kernel: the GEMM for Q4_K and Q5_K, with exact integer weights on the tensor cores.
//
// A k-quant weight is w = d * (sc * q) - dmin * m with d, dmin one f16 pair per 256 columns and row, sc / m 6-bit integers
// per 32 columns, q a 4- or 5-bit integer (crates/inferi/src/quantization.rs:287-402).  sc * q <= 63 * 31 < 2048 is an
// integer that f16 holds exactly, so per 256-column block
//     sum_k w_k x_k = d * P - Z,   P = sum_k (sc * q)_k x_k,   Z = sum_sb (dmin * m_sb) * S_sb,   S_sb = sum_{k in sb} x_k
// and P needs no hi / lo split of the weights: two MMAs per 16 columns (x hi, x lo) instead of three, one f16 tile to
// write instead of two, and a conversion that is a byte permute and one packed f16 multiply-add per two weights
// ((1024 + q) * sc - 1024 * sc, exact) instead of ~12 instructions per weight - the producers' instruction stream is what
// bounds the general kernel.  The price: P must be scaled by d per (row, block), so every block's P is accumulated in
// its own tensor-memory buffer (two, alternating) and folded into register accumulators by the producer warps
// (tcgen05.ld, one f32 multiply-add per value) while the next block's MMAs run; Z (minimums x sub-block sums of the
// inputs, both split hi / lo) accumulates over the whole K range in a third buffer: three small MMAs per block.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int KQ_WSTAGES = 3;                 // stages of the weights' tile (one f16 tile of 128 x 64: 16 KiB)
constexpr int KQ_XSTAGES = 3;                 // stages of the inputs' tiles (hi, lo: 32 KiB)
constexpr uint32_t KQ_ZSLOTS = 1;             // slots for a block's minimums / sub-block sums
constexpr uint32_t KQ_ZTILE = TC_ROWS * 16 * 2;   // a 128 x 16 f16 tile of minimums or of sub-block sums: 4 KiB
constexpr uint32_t KQ_ZSLOT = 4 * KQ_ZTILE;       // minimums hi, lo; sums hi, lo
constexpr uint32_t KQ_SMEM_FIXED = KQ_WSTAGES * TC_TILE_BYTES + KQ_XSTAGES * 2 * TC_TILE_BYTES + KQ_ZSLOTS * KQ_ZSLOT + 1024 + 1024;
constexpr uint32_t KQ_ZLBO = 128, KQ_ZSBO = 256;  // core matrices of the 16-column tiles

template <bool Q5>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_kquant_tc_kernel(const GemmTcParams p, const __grid_constant__ CUtensorMap wmap) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int PATH = Q5 ? TC_PATH_Q5K : TC_PATH_Q4K;
    constexpr uint32_t RAW_BYTES = tc_raw_stage_bytes(PATH), RB = Q5 ? 176u : 144u;
    const uint32_t R = p.raw_stages;
    uint8_t *wst = smem;                                                   // weights' stages
    uint8_t *xst = wst + KQ_WSTAGES * TC_TILE_BYTES;                       // inputs' stages
    uint8_t *zst = xst + KQ_XSTAGES * 2 * TC_TILE_BYTES;                   // minimum / sum slots
    const uint32_t raw0 = tc_smem_u32(zst + KQ_ZSLOTS * KQ_ZSLOT);
    uint64_t *bars = reinterpret_cast<uint64_t *>(zst + KQ_ZSLOTS * KQ_ZSLOT + R * RAW_BYTES);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // barriers, in this order
    const uint32_t b_wfull = tc_smem_u32(bars), b_wempty = b_wfull + 8 * KQ_WSTAGES, b_xfull = b_wempty + 8 * KQ_WSTAGES, b_xempty = b_xfull + 8 * KQ_XSTAGES;
    const uint32_t b_zfull = b_xempty + 8 * KQ_XSTAGES, b_zempty = b_zfull + 16, b_rawfull = b_zempty + 16, b_rawempty = b_rawfull + 8 * TC_RAW_MAX;
    const uint32_t b_pdone = b_rawempty + 8 * TC_RAW_MAX, b_pfree = b_pdone + 16, b_zdone = b_pfree + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * KQ_WSTAGES + 2 * KQ_XSTAGES + 4 + 2 * TC_RAW_MAX + 5);
    const StreamK sk = p.sk;
    const uint32_t u0 = sk.first_unit(blockIdx.x), u1 = sk.first_unit(blockIdx.x + 1), nunits = u1 - u0, nstage = 4 * nunits;

    if (tid == 0) {
        auto init = [](uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); };
        for (int s = 0; s < KQ_WSTAGES; s++) { init(b_wfull + 8 * s, TC_PRODUCER_WARPS); init(b_wempty + 8 * s, 1); }
        for (int s = 0; s < KQ_XSTAGES; s++) { init(b_xfull + 8 * s, 1); init(b_xempty + 8 * s, 1); }
        for (int s = 0; s < 2; s++) {
            init(b_zfull + 8 * s, TC_PRODUCER_WARPS + 1);   // the producer warps' minimums + the loader's arrival with the sums' bytes
            init(b_zempty + 8 * s, 1);
            init(b_pdone + 8 * s, 1);                       // tcgen05.commit: the block's P is complete
            init(b_pfree + 8 * s, TC_PRODUCER_WARPS);       // every producer warp has folded it into its registers
        }
        for (uint32_t s = 0; s < TC_RAW_MAX; s++) { init(b_rawfull + 8 * s, 1); init(b_rawempty + 8 * s, TC_PRODUCER_WARPS); }
        init(b_zdone, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < TC_ROWS) {
        // columns 8..15 of the minimums' tiles stay zero for the whole kernel
        for (uint32_t s = 0; s < KQ_ZSLOTS; s++)
            for (int t = 0; t < 2; t++)
                *reinterpret_cast<uint4 *>(zst + s * KQ_ZSLOT + t * KQ_ZTILE + (tid >> 3) * KQ_ZSBO + KQ_ZLBO + (tid & 7) * 16) = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == TC_PRODUCER_WARPS) {
        // tensor memory: two P buffers and Z, 128 columns each (512 allocated: a power of two)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    const uint32_t groups = p.n_pad / 16;
    bool ok = true;

    if (warp < TC_PRODUCER_WARPS) {
        // ===== producers: thread = (weight row `tid & 127` of the unit's tile, quarter `tid >> 7` of a stage's 64 columns);
        // the same thread owns row `tid & 127` x 32 token columns of the output (tensor-memory lane = row) =====
        const uint32_t row = tid & (TC_ROWS - 1), kq = tid >> 7;
        uint32_t tile = u0 / sk.nb, kb = u0 - tile * sk.nb, ptile = tile, pkb = kb;
        // One block of each of the tile's 128 rows = one box of the matrix seen as a 2-D byte array [rows][row_bytes]: a
        // single tiled TMA copy per step.  (With 128 one-row bulk copies per step the producers waited 1.6 us per step
        // for the block: the copies completed ~6 us after they were issued.)
        auto issue_raw = [&](uint32_t t, uint32_t b, uint32_t dst, uint32_t bar) {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)TC_ROWS * RB) : "memory");
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                         "l"(reinterpret_cast<uint64_t>(&wmap)), "r"(b * RB), "r"(t * (uint32_t)TC_ROWS), "r"(bar)
                         : "memory");
        };
        uint32_t issued = 0;
        for (; issued < R && issued < nunits; issued++) {
            if (tid == 0) issue_raw(ptile, pkb, raw0 + issued * RAW_BYTES, b_rawfull + 8 * issued);
            if (++pkb == sk.nb) { pkb = 0; ptile++; }
        }
        uint32_t slot = 0, slot_par = 0, pslot = 0, pslot_par = 0;
        uint32_t ws = 0, wround = 0;                 // weights' stage and how often the ring has wrapped
        float Y[32];
#pragma unroll
        for (int i = 0; i < 32; i++) Y[i] = 0.f;
        float d_cur = 0.f, d_prev = 0.f;
        uint32_t seg = 0;   // segments (tile, K range) finished so far: the parity of the Z barrier
        uint32_t sc_y = 0, sc_z = 0, sc_w = 0;       // the block's twelve scale bytes
        const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        // fold P buffer `pb` (scaled by `dd`) into Y: the warp's 32 lanes x its token columns
        auto fold = [&](uint32_t pb, float dd) {
            // one 16-column read at a time: both in flight at once need 16 more registers than 18 warps leave (96 per thread)
#pragma unroll
            for (int g = 0; g < 2; g++) {
                const uint32_t c0 = 16 * (warp >> 2) + 64 * g;
                if (c0 < 16 * groups) {
                    uint32_t r[16];
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
                                   "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                                 : "r"(taddr + pb * 128 + c0)
                                 : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; i++) Y[16 * g + i] = fmaf(dd, __uint_as_float(r[i]), Y[16 * g + i]);
                }
            }
        };
        for (uint32_t it = 0; it < nstage && ok; it++) {
            const uint32_t j = it >> 2, c = it & 3, u = u0 + j, pb = j & 1, zs = j % KQ_ZSLOTS, zuse = j / KQ_ZSLOTS;
            if (c == 0) {
                if (j >= 1) {
                    pslot = slot; pslot_par = slot_par;
                    if (++slot == R) { slot = 0; slot_par ^= 1u; }
                    if (++kb == sk.nb) { kb = 0; tile++; }
                    if (issued < nunits) {
                        // the slot of the previous step is refilled once every producer thread has read it
                        if (warp == 0) {
                            ok = __all_sync(0xffffffffu, tc_wait(b_rawempty + 8 * pslot, pslot_par, p.wait_ns, p.err, 8));
                            if (!ok) break;
                            if (lane == 0) issue_raw(ptile, pkb, raw0 + pslot * RAW_BYTES, b_rawfull + 8 * pslot);
                        }
                        issued++;
                        if (++pkb == sk.nb) { pkb = 0; ptile++; }
                    }
                }
                ok = __all_sync(0xffffffffu, tc_wait(b_rawfull + 8 * slot, slot_par, p.wait_ns, p.err, 8));
                if (!ok) break;
                // the block's header: d, dmin and the twelve scale bytes stay in registers for its four stages
                const uint4 hdr = tc_lds128(raw0 + slot * RAW_BYTES + row * RB);
                d_prev = d_cur;
                d_cur = tc_h2f(hdr.x & 0xFFFFu);
                sc_y = hdr.y; sc_z = hdr.z; sc_w = hdr.w;
                // the minimums of sub-blocks 2 kq and 2 kq + 1, times dmin, split hi / lo: columns 2 kq, 2 kq + 1 of the
                // block's 128 x 16 tile (get_scale_min_k4, quantization.rs:394-402)
                if (j >= KQ_ZSLOTS) {
                    ok = __all_sync(0xffffffffu, tc_wait(b_zempty + 8 * zs, (zuse - 1) & 1, p.wait_ns, p.err, 8));
                    if (!ok) break;
                }
                {
                    const float dmin = tc_h2f(hdr.x >> 16);
                    const uint32_t sb[3] = {sc_y, sc_z, sc_w};
                    auto byte_at = [&](uint32_t i) { return (sb[i >> 2] >> (8 * (i & 3))) & 0xFFu; };
                    float mm[2];
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const uint32_t jj = 2 * kq + e;
                        const uint32_t mn = jj < 4 ? (byte_at(jj + 4) & 63u) : ((byte_at(jj + 4) >> 4) | ((byte_at(jj) >> 6) << 4));
                        mm[e] = dmin * (float)mn;
                    }
                    const __half2 h = __floats2half2_rn(mm[0], mm[1]);
                    const float2 back = __half22float2(h);
                    const __half2 l = __floats2half2_rn(mm[0] - back.x, mm[1] - back.y);
                    uint8_t *zt = zst + zs * KQ_ZSLOT + (row >> 3) * KQ_ZSBO + (row & 7) * 16 + 4 * kq;
                    *reinterpret_cast<__half2 *>(zt) = h;
                    *reinterpret_cast<__half2 *>(zt + KQ_ZTILE) = l;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(b_zfull + 8 * zs) : "memory");
                }
            }
            // ---- the stage's 16 weights of this thread: sub-block jj = 2 c + (kq >> 1), bytes 16 (kq & 1) .. + 15 of its 32 ----
            const uint32_t jj = 2 * c + (kq >> 1), high = jj & 1, hq = kq & 1;
            const uint32_t blk = raw0 + slot * RAW_BYTES + row * RB;
            const uint4 qv = tc_lds128(blk + (Q5 ? 48 : 16) + 32 * c + 16 * hq);
            uint4 hv = make_uint4(0, 0, 0, 0);
            if (Q5) hv = tc_lds128(blk + 16 + 16 * hq);
            uint32_t sc;
            {
                const uint32_t sb[3] = {sc_y, sc_z, sc_w};
                auto byte_at = [&](uint32_t i) { return (sb[i >> 2] >> (8 * (i & 3))) & 0xFFu; };
                sc = jj < 4 ? (byte_at(jj) & 63u) : ((byte_at(jj + 4) & 0xFu) | ((byte_at(jj - 4) >> 6) << 4));
            }
            // (1024 + q) * sc - 1024 * sc = q * sc, exact in f16 (q * sc < 2048; 1024 * sc <= 64512 is representable)
            const __half2 sc2 = __float2half2_rn((float)sc), off2 = __float2half2_rn(-1024.0f * (float)sc);
            const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w}, hw[4] = {hv.x, hv.y, hv.z, hv.w};
            uint32_t out[8];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t nib = high ? (qw[i] >> 4) & 0x0F0F0F0Fu : qw[i] & 0x0F0F0F0Fu;
                if (Q5) nib |= ((hw[i] >> (2 * c + high)) & 0x01010101u) << 4;
                const uint32_t p01 = __byte_perm(nib, 0x64646464u, 0x4140), p23 = __byte_perm(nib, 0x64646464u, 0x4342);   // f16 pairs (1024 + q)
                const __half2 r01 = __hfma2(*reinterpret_cast<const __half2 *>(&p01), sc2, off2);
                const __half2 r23 = __hfma2(*reinterpret_cast<const __half2 *>(&p23), sc2, off2);
                out[2 * i] = *reinterpret_cast<const uint32_t *>(&r01);
                out[2 * i + 1] = *reinterpret_cast<const uint32_t *>(&r23);
            }
            if (c == 3) {
                __syncwarp();   // every lane has read its part of the raw stage
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(b_rawempty + 8 * slot) : "memory");
            }
            if (wround > 0) ok = __all_sync(0xffffffffu, tc_wait(b_wempty + 8 * ws, (wround - 1) & 1, p.wait_ns, p.err, 8));
            if (!ok) break;
            uint8_t *st = wst + ws * TC_TILE_BYTES;
            *reinterpret_cast<uint4 *>(st + tc_chunk_off(row, 2 * kq)) = make_uint4(out[0], out[1], out[2], out[3]);
            *reinterpret_cast<uint4 *>(st + tc_chunk_off(row, 2 * kq + 1)) = make_uint4(out[4], out[5], out[6], out[7]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(b_wfull + 8 * ws) : "memory");
            if (++ws == KQ_WSTAGES) { ws = 0; wround++; }
            if (c == 3) {
                const bool seg_end = kb + 1 == sk.nb || u + 1 == u1, seg_start = j == 0 || kb == 0;
                // the previous block's P (complete long ago: its MMAs ran while this block was converted)
                if (!seg_start) {
                    ok = __all_sync(0xffffffffu, tc_wait(b_pdone + 8 * (pb ^ 1), ((j - 1) >> 1) & 1, p.wait_ns, p.err, 10));
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    fold(pb ^ 1, d_prev);
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(b_pfree + 8 * (pb ^ 1)) : "memory");
                }
                if (seg_end) {
                    // the tile's K range in this CTA ends: this block's P too, then Z, then the plane
                    ok = __all_sync(0xffffffffu, tc_wait(b_pdone + 8 * pb, (j >> 1) & 1, p.wait_ns, p.err, 10));
                    if (ok) ok = __all_sync(0xffffffffu, tc_wait(b_zdone, seg & 1, p.wait_ns, p.err, 10));
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    fold(pb, d_cur);
                    fold(2, -1.0f);
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(b_pfree + 8 * pb) : "memory");
                    const uint32_t piece = blockIdx.x - sk.cta_of(tile * sk.nb);
                    float *outp = p.out + (size_t)piece * p.n_tokens * p.rows + tile * TC_ROWS + row;
#pragma unroll
                    for (int g = 0; g < 2; g++)
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            const uint32_t t = 16 * (warp >> 2) + 64 * g + i;
                            if (t < p.n_tokens) outp[(size_t)t * p.rows] = Y[16 * g + i];
                            Y[16 * g + i] = 0.f;
                        }
                    seg++;
                }
            }
        }
        if (!ok) {
            const unsigned long long t0 = tc_ns();
            while (tc_ns() - t0 < 100000ull) {}
        }
    } else if (warp == TC_PRODUCER_WARPS && lane == 0) {
        // ===== MMA issue: one thread =====
        const uint32_t idesc = tc_idesc_f16(TC_ROWS, p.n_pad);
        uint32_t ws = 0, wpar = 0, xs = 0, xpar = 0;
        // The issuing thread is one warp's instruction stream: whatever it computes per MMA is serial latency between two
        // MMAs, so the descriptors of stage 0 are built once and the others are one addition away.
        const uint64_t wdesc0 = tc_smem_desc(tc_smem_u32(wst), TC_LBO, TC_SBO), xdesc0 = tc_smem_desc(tc_smem_u32(xst), TC_LBO, TC_SBO);
        const uint64_t zdesc0 = tc_smem_desc(tc_smem_u32(zst), KQ_ZLBO, KQ_ZSBO);
        uint32_t kb = u0 % sk.nb;
        for (uint32_t it = 0; it < nstage && ok; it++) {
            const uint32_t j = it >> 2, c = it & 3, u = u0 + j, pb = j & 1;
            if (c == 0 && j >= 1 && ++kb == sk.nb) kb = 0;
            const bool seg_start = j == 0 || kb == 0, seg_end = kb + 1 == sk.nb || u + 1 == u1;
            if (c == 0) {
                // the P buffer of this block must have been folded (two blocks ago); then Z: the block's minimums x sums
                if (j >= 2) ok = tc_wait(b_pfree + 8 * pb, ((j >> 1) - 1) & 1, p.wait_ns, p.err, 9);
                const uint32_t zs = j % KQ_ZSLOTS, zuse = j / KQ_ZSLOTS;
                if (ok) ok = tc_wait(b_zfull + 8 * zs, zuse & 1, p.wait_ns, p.err, 9);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t m_hi = zdesc0 + zs * (KQ_ZSLOT >> 4), m_lo = m_hi + (KQ_ZTILE >> 4), s_hi = m_hi + 2 * (KQ_ZTILE >> 4), s_lo = m_hi + 3 * (KQ_ZTILE >> 4);
                tc_mma_f16(tmem_base + 256, m_hi, s_hi, idesc, !seg_start);
                tc_mma_f16(tmem_base + 256, m_hi, s_lo, idesc, 1);
                tc_mma_f16(tmem_base + 256, m_lo, s_hi, idesc, 1);
                tc_commit(b_zempty + 8 * zs);
            }
            ok = tc_wait(b_xfull + 8 * xs, xpar, p.wait_ns, p.err, 9) && tc_wait(b_wfull + 8 * ws, wpar, p.wait_ns, p.err, 9);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // descriptors differ from the stage-0 ones only in the start-address field (units of 16 bytes): one addition each
            const uint64_t wd = wdesc0 + ws * (TC_TILE_BYTES >> 4), xh = xdesc0 + xs * (2 * TC_TILE_BYTES >> 4), xl = xh + (TC_TILE_BYTES >> 4);
#pragma unroll
            for (uint32_t kk = 0; kk < TC_KSTAGE / 16; kk++) {
                const uint32_t ko = kk * (2 * TC_LBO >> 4);   // 16 columns = two core matrices along K
                tc_mma_f16(tmem_base + pb * 128, wd + ko, xh + ko, idesc, !(c == 0 && kk == 0));   // every block starts a new P
                tc_mma_f16(tmem_base + pb * 128, wd + ko, xl + ko, idesc, 1);
            }
            tc_commit(b_wempty + 8 * ws);
            tc_commit(b_xempty + 8 * xs);
            if (c == 3) {
                tc_commit(b_pdone + 8 * pb);
                if (seg_end) tc_commit(b_zdone);
            }
            if (++ws == KQ_WSTAGES) { ws = 0; wpar ^= 1u; }
            if (++xs == KQ_XSTAGES) { xs = 0; xpar ^= 1u; }
        }
    }

    if (warp == TC_PRODUCER_WARPS + 1 && lane == 0) {
        // ===== the inputs' tiles (two bulk copies per stage) and, per block, the tiles of their sub-block sums =====
        bool okx = true;
        const uint32_t xbytes = p.n_pad * (TC_KSTAGE * 2), sbytes = p.n_pad * 32;
        const __half *s_hi = p.x_hi + (size_t)TC_ROWS * p.cols, *s_lo = p.x_lo + (size_t)TC_ROWS * p.cols;
        uint32_t xs = 0, xround = 0;
        for (uint32_t it = 0; it < nstage && okx; it++) {
            const uint32_t j = it >> 2, c = it & 3, kb = (u0 + j) % sk.nb;
            if (c == 0) {
                const uint32_t zs = j % KQ_ZSLOTS, zuse = j / KQ_ZSLOTS;
                if (j >= KQ_ZSLOTS) okx = tc_wait(b_zempty + 8 * zs, (zuse - 1) & 1, p.wait_ns, p.err, 8);
                if (!okx) break;
                const uint32_t full = b_zfull + 8 * zs, dst = tc_smem_u32(zst + zs * KQ_ZSLOT + 2 * KQ_ZTILE);
                const size_t at = (size_t)kb * (TC_ROWS * 16);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"(2 * sbytes) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(s_hi + at), "r"(sbytes), "r"(full)
                             : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst + KQ_ZTILE), "l"(s_lo + at), "r"(sbytes),
                             "r"(full)
                             : "memory");
            }
            if (xround > 0) okx = tc_wait(b_xempty + 8 * xs, (xround - 1) & 1, p.wait_ns, p.err, 8);
            if (!okx) break;
            const uint32_t full = b_xfull + 8 * xs, dst = tc_smem_u32(xst + xs * 2 * TC_TILE_BYTES);
            const size_t at = (size_t)(4 * kb + c) * (TC_ROWS * TC_KSTAGE);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"(2 * xbytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(p.x_hi + at), "r"(xbytes), "r"(full)
                         : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst + TC_TILE_BYTES), "l"(p.x_lo + at), "r"(xbytes),
                         "r"(full)
                         : "memory");
            if (++xs == KQ_XSTAGES) { xs = 0; xround++; }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == TC_PRODUCER_WARPS) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
}


// ---------------------------------------------------------------------------------------------------------------------
// element-wise kernels around the GEMMs (one thread per element or pair; rows = tokens)
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void split_store(__half *hi, __half *lo, size_t i, float v) {
    const __half h = __float2half_rn(v);
    hi[i] = h;
    lo[i] = __float2half_rn(v - __half2float(h));
}

// X[t][c] = dequantized embedding row of token t (crates/inferi/src/models/llama2/transformer.rs:367-374, chat_llama2.rs:217-220)
__global__ void prefill_embed_kernel(QDesc embd, const uint32_t *tokens, uint32_t n, uint32_t hidden, uint32_t vocab, float *X) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)n * hidden; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(i / hidden), c = (uint32_t)(i % hidden);
        uint32_t tok = tokens[t];
        if (tok >= vocab) tok = vocab - 1;
        X[i] = dequant_at(embd, embd.w + (size_t)tok * embd.row_bytes, c);
    }
}

// One CTA per token row: y = (x * rsqrt(mean(x^2) + eps)) * w (crates/inferi-shaders/src/rms_norm.rs:112-120; `w` null: y = x),
// stored as the two f16 halves the GEMM reads, in its tiled layout (tc_x_index).  Rows n .. n_pad-1 are zero-filled.
__global__ void __launch_bounds__(256) prefill_norm_split_kernel(const float *X, const float *w, float eps, uint32_t n, uint32_t cols, __half *hi, __half *lo) {
    // grid: (token row, chunk of 1024 columns).  Every CTA of a row forms the row's sum of squares itself (16 KiB from L2)
    // rather than wait for a second kernel: with one CTA per row the kernel was a 16-pass latency chain of 14-19 us.
    __shared__ float red[8];
    const uint32_t t = blockIdx.x, c_beg = blockIdx.y * 1024, c_end = c_beg + 1024 < cols ? c_beg + 1024 : cols;
    if (t >= n) {
        for (uint32_t c = c_beg + threadIdx.x; c < c_end; c += blockDim.x) { hi[tc_x_index(t, c)] = __float2half_rn(0.f); lo[tc_x_index(t, c)] = __float2half_rn(0.f); }
        for (uint32_t k = c_beg / 16 + threadIdx.x; k < c_end / 16; k += blockDim.x) {   // 16 halves per 256 columns
            const size_t at = tc_s_index(t, (k >> 4) * 8, cols) + ((k & 8) ? 64 : 0) + (k & 7);
            hi[at] = __float2half_rn(0.f);
            lo[at] = __float2half_rn(0.f);
        }
        return;
    }
    const float *x = X + (size_t)t * cols;
    float rms = 1.0f;
    if (w) {
        float ss = 0.f;
        for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) ss += x[c] * x[c];
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int i = 0; i < 8; i++) tot += red[i];
        rms = 1.0f / sqrtf(tot / (float)cols + eps);
    }
    // cols is a multiple of 256 = blockDim.x: a warp's lanes hold one 32-column sub-block per pass
    for (uint32_t c = c_beg + threadIdx.x; c < c_end; c += blockDim.x) {
        const float y = w ? (x[c] * rms) * w[c] : x[c];
        split_store(hi, lo, tc_x_index(t, c), y);
        float sum = y;
#pragma unroll
        for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if ((threadIdx.x & 31) == 0) split_store(hi, lo, tc_s_index(t, c >> 5, cols), sum);
        if ((threadIdx.x & 31) == 1 && ((c >> 5) & 7) == 0) {   // the eight zero halves of the unit's tile row
            *reinterpret_cast<uint4 *>(hi + tc_s_index(t, c >> 5, cols) + 64) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4 *>(lo + tc_s_index(t, c >> 5, cols) + 64) = make_uint4(0, 0, 0, 0);
        }
    }
}

// Elements i, i + 1 (i even) summed over a tile's planes, in plane order (deterministic); the loads of the planes are
// independent 8-byte loads, all in flight together.
__device__ __forceinline__ float2 plane_sum2(const float *planes, uint32_t pieces, size_t plane_elems, size_t i) {
    float2 v = make_float2(0.f, 0.f);
    for (uint32_t s0 = 0; s0 < pieces; s0 += 4) {
        float2 t[4];
#pragma unroll
        for (int k = 0; k < 4; k++)
            t[k] = s0 + k < pieces ? __ldcs(reinterpret_cast<const float2 *>(planes + (s0 + k) * plane_elems + i)) : make_float2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < 4; k++) { v.x += t[k].x; v.y += t[k].y; }
    }
    return v;
}

// One thread per pair of neighbouring rows (the rotation acts on pairs).
__global__ void prefill_epilogue_kernel(const PrefillEpiParams p) {
    // PE_SWIGLU also zero-fills the padding rows n .. n_pad-1 of the split product (the GEMM that follows reads them)
    const uint32_t n_rows = p.mode == PE_SWIGLU ? ((p.n + 15) & ~15u) : p.n;
    const size_t plane = (size_t)p.n * p.rows, pairs = (size_t)n_rows * p.rows / 2;
    for (size_t pi = (size_t)blockIdx.x * blockDim.x + threadIdx.x; pi < pairs; pi += (size_t)gridDim.x * blockDim.x) {
        const size_t i = 2 * pi;
        const uint32_t t = (uint32_t)(i / p.rows), r = (uint32_t)(i % p.rows);
        if (t >= p.n) {
            split_store(p.hi, p.lo, tc_x_index(t, r), 0.f);
            split_store(p.hi, p.lo, tc_x_index(t, r + 1), 0.f);
            if ((r & 31) == 0) split_store(p.hi, p.lo, tc_s_index(t, r >> 5, p.rows), 0.f);
            if ((r & 255) == 2) {
                *reinterpret_cast<uint4 *>(p.hi + tc_s_index(t, (r >> 8) * 8, p.rows) + 64) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4 *>(p.lo + tc_s_index(t, (r >> 8) * 8, p.rows) + 64) = make_uint4(0, 0, 0, 0);
            }
            continue;
        }
        const uint32_t np = p.sk.pieces(r / 128);   // the planes that the row's tile was spread over
        const float2 ab = plane_sum2(p.planes, np, plane, i);
        float a = ab.x, b = ab.y;
        if (p.mode == PE_SWIGLU) {
            // crates/inferi-shaders/src/silu.rs:16-19,46-52
            const float2 uab = plane_sum2(p.planes2, np, plane, i);
            const float ua = uab.x, ub = uab.y;
            const float ya = ua * (a / (1.0f + expf(-a))), yb = ub * (b / (1.0f + expf(-b)));
            split_store(p.hi, p.lo, tc_x_index(t, r), ya);
            split_store(p.hi, p.lo, tc_x_index(t, r + 1), yb);
            // the sums of the 32-column sub-blocks for the GEMM that follows: 16 neighbouring threads hold one sub-block
            // (whole warps run this loop together: the number of pairs is a multiple of 64)
            float sum = ya + yb;
#pragma unroll
            for (int o = 8; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if ((r & 31) == 0) split_store(p.hi, p.lo, tc_s_index(t, r >> 5, p.rows), sum);
            if ((r & 255) == 2) {
                *reinterpret_cast<uint4 *>(p.hi + tc_s_index(t, (r >> 8) * 8, p.rows) + 64) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4 *>(p.lo + tc_s_index(t, (r >> 8) * 8, p.rows) + 64) = make_uint4(0, 0, 0, 0);
            }
            continue;
        }
        if (p.mode == PE_RESIDUAL) { p.out[i] += a; p.out[i + 1] += b; continue; }
        if (p.mode == PE_STORE) { p.out[i] = a; p.out[i + 1] = b; continue; }
        if (p.bias) { a += p.bias[r]; b += p.bias[r + 1]; }   // crates/inferi/src/models/llama2/transformer.rs:434-442
        if (p.mode != PE_V) {
            // crates/inferi-shaders/src/rope.rs:75-91 (adjacent pairs), the angle as the decode path forms it
            float sn, cs;
            sincosf((float)(p.pos0 + t) * p.theta[(r % p.head_size) >> 1], &sn, &cs);
            const float x = a, y = b;
            a = cs * x - sn * y;
            b = sn * x + cs * y;
        }
        if (p.mode == PE_Q) { p.out[i] = a; p.out[i + 1] = b; continue; }
        const size_t off = (size_t)(p.pos0 + t) * p.kv_dim + r;
        if (p.kv_dtype == IB_KV_F16) reinterpret_cast<__half2 *>(p.cache)[off >> 1] = __floats2half2_rn(a, b);
        else reinterpret_cast<float2 *>(p.cache)[off >> 1] = make_float2(a, b);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------------
StreamK prefill_streamk(const ib_ctx *ctx, uint32_t rows, uint32_t cols) {
    StreamK sk;
    sk.nb = cols / 256;
    sk.total = (rows / TC_ROWS) * sk.nb;
    sk.ctas = sk.total < (uint32_t)ctx->sm_count ? sk.total : (uint32_t)ctx->sm_count;
    return sk;
}
uint32_t prefill_max_pieces(const StreamK &sk, uint32_t rows) {
    uint32_t most = 1;
    for (uint32_t t = 0; t < rows / TC_ROWS; t++) most = sk.pieces(t) > most ? sk.pieces(t) : most;
    return most;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) ptr = nullptr;
        return (EncodeTiledFn)ptr;
    }();
    return fn;
}

bool prefill_gemm_eligible(const ib_qtensor *m) {
    return m->rows % TC_ROWS == 0 && m->cols % 256 == 0 && (m->qtype == IB_Q4_K || m->qtype == IB_Q5_K || m->qtype == IB_Q6_K || m->qtype == IB_Q8_0);
}

int32_t launch_prefill_gemm(ib_ctx *ctx, cudaStream_t s, const ib_qtensor *m, const __half *x_hi, const __half *x_lo, uint32_t n, float *planes, const StreamK &sk) {
    const int path = tc_path((uint32_t)m->qtype, m->layout);
    const bool exact = path == TC_PATH_Q4K || path == TC_PATH_Q5K;   // integer weights on the tensor cores (gemm_kquant_tc_kernel)
    const uint32_t raw_bytes = tc_raw_stage_bytes(path), fixed = exact ? KQ_SMEM_FIXED : TC_SMEM_FIXED;
    uint32_t raw_stages = raw_bytes ? (TC_SMEM_LIMIT - fixed) / raw_bytes : 1;
    if (raw_stages > TC_RAW_MAX) raw_stages = TC_RAW_MAX;
    const uint32_t smem_bytes = fixed + raw_stages * raw_bytes;
    static bool attr_set[16][4] = {};
    if (!attr_set[ctx->device & 15][path]) {
        if (exact) {
            IB_CHECK_CUDA(cudaFuncSetAttribute(gemm_kquant_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(TC_SMEM_LIMIT)));
            IB_CHECK_CUDA(cudaFuncSetAttribute(gemm_kquant_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(TC_SMEM_LIMIT)));
        } else {
            IB_CHECK_CUDA(cudaFuncSetAttribute(gemm_quant_tc_kernel<TC_PATH_Q6K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(TC_SMEM_LIMIT)));
            IB_CHECK_CUDA(cudaFuncSetAttribute(gemm_quant_tc_kernel<TC_PATH_OTHER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(TC_SMEM_LIMIT)));
        }
        attr_set[ctx->device & 15][path] = true;
    }
    IB_REQUIRE(((uintptr_t)m->dev % 16) == 0 && (m->row_bytes % 16) == 0 && ((uintptr_t)x_hi % 16) == 0 && ((uintptr_t)x_lo % 16) == 0,
               "prefill GEMM: the matrix rows and the input tiles must be 16-byte aligned for the bulk copies");
    GemmTcParams p;
    p.raw_stages = raw_stages;
    p.w = QDesc{m->dev, m->row_bytes, (uint32_t)m->qtype, m->layout, m->nb};
    p.rows = (uint32_t)m->rows; p.cols = (uint32_t)m->cols;
    p.x_hi = x_hi; p.x_lo = x_lo; p.n_tokens = n; p.n_pad = (n + 15) & ~15u;
    p.out = planes; p.sk = sk; p.err = ctx->err_dev; p.wait_ns = ctx->wait_limit_ns;
    if (exact) {
        // the matrix as a 2-D byte array [rows][row_bytes]; a box = one block (144 / 176 bytes) of 128 consecutive rows
        CUtensorMap wmap;
        const cuuint64_t dims[2] = {(cuuint64_t)m->row_bytes, (cuuint64_t)m->rows}, strides[1] = {(cuuint64_t)m->row_bytes};
        const cuuint32_t box[2] = {path == TC_PATH_Q5K ? 176u : 144u, (cuuint32_t)TC_ROWS}, estr[2] = {1, 1};
        EncodeTiledFn encode = encode_tiled();
        IB_REQUIRE(encode, "prefill GEMM: the driver does not export cuTensorMapEncodeTiled");
        const CUresult cr = encode(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)m->dev, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        IB_REQUIRE(cr == CUDA_SUCCESS, "prefill GEMM: cuTensorMapEncodeTiled failed with %d", (int)cr);
        if (path == TC_PATH_Q5K) gemm_kquant_tc_kernel<true><<<sk.ctas, TC_THREADS, smem_bytes, s>>>(p, wmap);
        else gemm_kquant_tc_kernel<false><<<sk.ctas, TC_THREADS, smem_bytes, s>>>(p, wmap);
    } else {
        // Q6_K in the 8-block row layout: boxes of 128 rows x 144 / 80 / 16 bytes (see the kernel); other formats: unused
        CUtensorMap maps[3] = {};
        if (path == TC_PATH_Q6K) {
            const cuuint64_t dims[2] = {(cuuint64_t)m->row_bytes, (cuuint64_t)m->rows}, strides[1] = {(cuuint64_t)m->row_bytes};
            const cuuint32_t widths[3] = {144, 80, 16}, estr[2] = {1, 1};
            EncodeTiledFn encode = encode_tiled();
            IB_REQUIRE(encode, "prefill GEMM: the driver does not export cuTensorMapEncodeTiled");
            for (int i = 0; i < 3; i++) {
                const cuuint32_t box[2] = {widths[i], (cuuint32_t)TC_ROWS};
                const CUresult cr = encode(&maps[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)m->dev, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                IB_REQUIRE(cr == CUDA_SUCCESS, "prefill GEMM: cuTensorMapEncodeTiled failed with %d", (int)cr);
            }
        }
        if (path == TC_PATH_Q6K) gemm_quant_tc_kernel<TC_PATH_Q6K><<<sk.ctas, TC_THREADS, smem_bytes, s>>>(p, maps[0], maps[1], maps[2]);
        else gemm_quant_tc_kernel<TC_PATH_OTHER><<<sk.ctas, TC_THREADS, smem_bytes, s>>>(p, maps[0], maps[1], maps[2]);
    }
    ctx->launches++;
    IB_CHECK_CUDA(cudaGetLastError());
    return IB_OK;
}

int32_t launch_prefill_embed(ib_ctx *ctx, cudaStream_t s, const ib_qtensor *embd, const uint32_t *tokens_dev, uint32_t n, uint32_t vocab, float *X) {
    QDesc e{embd->dev, embd->row_bytes, (uint32_t)embd->qtype, embd->layout, embd->nb};
    const uint32_t hidden = (uint32_t)embd->cols;
    prefill_embed_kernel<<<(unsigned)(((size_t)n * hidden + 255) / 256), 256, 0, s>>>(e, tokens_dev, n, hidden, vocab, X);
    ctx->launches++;
    IB_CHECK_CUDA(cudaGetLastError());
    return IB_OK;
}

int32_t launch_prefill_norm_split(ib_ctx *ctx, cudaStream_t s, const float *X, const float *w, float eps, uint32_t n, uint32_t cols, __half *hi, __half *lo) {
    prefill_norm_split_kernel<<<dim3((n + 15) & ~15u, (cols + 1023) / 1024), 256, 0, s>>>(X, w, eps, n, cols, hi, lo);
    ctx->launches++;
    IB_CHECK_CUDA(cudaGetLastError());
    return IB_OK;
}

int32_t launch_prefill_epilogue(ib_ctx *ctx, cudaStream_t s, const PrefillEpiParams &p) {
    const size_t pairs = (size_t)((p.n + 15) & ~15u) * p.rows / 2;
    unsigned grid = (unsigned)((pairs + 255) / 256);
    if (grid > 4096) grid = 4096;
    prefill_epilogue_kernel<<<grid, 256, 0, s>>>(p);
    ctx->launches++;
    IB_CHECK_CUDA(cudaGetLastError());
    return IB_OK;
}

}  // namespace ib

using namespace ib;

extern "C" int32_t ib_gemm_quant(ib_ctx *ctx, void *stream, float *out_dev, const ib_qtensor *m, const float *x_dev, uint32_t n) {
    IB_REQUIRE(ctx && m && out_dev && x_dev, "ib_gemm_quant: null argument");
    IB_REQUIRE(m->ctx->device == ctx->device, "ib_gemm_quant: tensor lives on device %d, context on %d", m->ctx->device, ctx->device);
    IB_REQUIRE(n >= 1, "ib_gemm_quant: no rows");
    if (!prefill_gemm_eligible(m))
        return set_error(IB_ERR_UNSUPPORTED, "ib_gemm_quant: %llux%llu of type %d (the tensor-core path takes Q8_0/Q4_K/Q5_K/Q6_K with rows %% 128 == 0 and cols %% 256 == 0)",
                         (unsigned long long)m->rows, (unsigned long long)m->cols, m->qtype);
    int prev = -1;
    cudaGetDevice(&prev);
    IB_REQUIRE(cudaSetDevice(ctx->device) == cudaSuccess, "cudaSetDevice failed");
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t rows = (uint32_t)m->rows, cols = (uint32_t)m->cols;
    const StreamK sk = prefill_streamk(ctx, rows, cols);
    const uint32_t ks = prefill_max_pieces(sk, rows);
    const size_t half_bytes = tc_x_halves(cols) * sizeof(__half), plane_bytes = (size_t)ks * TC_ROWS * rows * sizeof(float);
    const size_t need = 2 * half_bytes + plane_bytes;
    int32_t rc = IB_OK;
    if (need > ctx->tc_scratch_bytes) {
        // growing the scratch: wait for work that may still use the old one
        cudaError_t e = cudaDeviceSynchronize();
        if (e == cudaSuccess && ctx->tc_scratch) e = cudaFree(ctx->tc_scratch);
        ctx->tc_scratch = nullptr;
        ctx->tc_scratch_bytes = 0;
        if (e == cudaSuccess) e = cudaMalloc(&ctx->tc_scratch, need);
        if (e != cudaSuccess) rc = set_error(e == cudaErrorMemoryAllocation ? IB_ERR_OOM : IB_ERR_CUDA, "ib_gemm_quant: scratch of %llu bytes: %s", (unsigned long long)need, cudaGetErrorString(e));
        else ctx->tc_scratch_bytes = need;
    }
    __half *hi = reinterpret_cast<__half *>(ctx->tc_scratch), *lo = reinterpret_cast<__half *>((uint8_t *)ctx->tc_scratch + half_bytes);
    float *planes = reinterpret_cast<float *>((uint8_t *)ctx->tc_scratch + 2 * half_bytes);
    for (uint32_t t0 = 0; rc == IB_OK && t0 < n; t0 += TC_ROWS) {
        const uint32_t nc = n - t0 < (uint32_t)TC_ROWS ? n - t0 : (uint32_t)TC_ROWS;
        rc = launch_prefill_norm_split(ctx, s, x_dev + (size_t)t0 * cols, nullptr, 0.f, nc, cols, hi, lo);
        if (rc == IB_OK) rc = launch_prefill_gemm(ctx, s, m, hi, lo, nc, planes, sk);
        if (rc == IB_OK) {
            PrefillEpiParams e = {};
            e.planes = planes; e.sk = sk; e.n = nc; e.rows = rows; e.mode = PE_STORE; e.out = out_dev + (size_t)t0 * rows;
            rc = launch_prefill_epilogue(ctx, s, e);
        }
    }
    if (prev >= 0 && prev != ctx->device) cudaSetDevice(prev);
    return rc;
}
