// Prompt prefill: the prompt's tokens go through every matrix together, as GEMMs on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory), instead of one by one through the decode path.
//
// The reference has no prefill: `ChatLlama2::forward` forces the prompt through the decode path token by token
// (crates/inferi-chat/src/chat_llama2.rs:137-155, crates/inferi-chat/src/sampler.rs:102-107), which reads every weight
// once per prompt token.  Here the weights are read once per prompt.
//
// gemm_quant_tc_kernel: out^T tile = W tile (128 rows of the quantized matrix) x X^T (the tokens' input vectors).
//  * the quantized blocks of the tile's 128 rows travel to shared memory by bulk copies (cp.async.bulk, one 256-column
//    block per row and step, a ring of steps ahead of their use) - no thread-per-row global loads, which were 32 cache
//    lines per load instruction and kept the L1 busy 91 % of the time;
//  * eight producer warps, two threads per weight row: read the row's block from shared memory, dequantize 64 columns of
//    the row per stage to f32, split the value into two f16 (w = hi + lo, exact to ~2^-22) and store both into shared
//    memory in the K-major core-matrix layout the tensor core reads (8 rows x 16 bytes per core matrix, no swizzle);
//  * the tokens' inputs (already split into f16 hi / lo by the kernel that produced them, and laid out in global memory
//    as tiles of that same layout) arrive by one bulk copy per tile;
//  * one thread issues, per 16 columns, three tcgen05.mma (hi x hi, hi x lo, lo x hi; lo x lo is below f32 resolution)
//    that accumulate in f32 in tensor memory: the result matches the f32 arithmetic of the decode path to ~1e-6;
//  * shared-memory stages cycle through mbarriers (filled by the producers, released by tcgen05.commit);
//  * when the K range is done the producer warps read the accumulator (tcgen05.ld: TMEM lane = weight row, column =
//    token) and store it transposed, [token][row], coalesced over the rows.
// Matrices with few row tiles split K over several CTAs; each writes its own partial plane and the element-wise kernel
// that follows (RoPE + cache append, residual add, SwiGLU) adds the planes in a fixed order.
// Every wait is bounded; a wait that gives up raises the context's error word and the kernel returns after freeing its
// tensor memory.
#include "prefill.cuh"

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

// How a matrix reaches the producers.  0: Q4_K, 1: Q5_K, 2: Q6_K in the 8-block row layout - their blocks are copied into
// shared memory by bulk copies, one 256-column block of every row of the tile per step; 3: everything else (read from
// global memory element by element).
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

// One row's block of the step -> shared memory; called by whole warps (lane 0's arrival announces the warp's bytes: an arrival
// per thread would be hundreds of serialized updates of one barrier word per step).  `kb` = block number in the row.
template <int PATH>
__device__ __forceinline__ void tc_issue_raw(const uint8_t *wrow, uint32_t kb, uint32_t raw, uint32_t row, uint32_t bar) {
    auto copy = [&](uint32_t dst, const uint8_t *src, uint32_t bytes) {
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
    };
    if (PATH == TC_PATH_Q4K || PATH == TC_PATH_Q5K) {
        constexpr uint32_t B = PATH == TC_PATH_Q4K ? 144u : 176u;
        if ((threadIdx.x & 31) == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(32u * B) : "memory");
        __syncwarp();
        copy(raw + row * B, wrow + (size_t)kb * B, B);
    } else if (PATH == TC_PATH_Q6K) {
        const uint8_t *grp = wrow + (size_t)(kb >> 3) * 1680;
        const uint32_t bb = kb & 7;
        if ((threadIdx.x & 31) == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(32u * (128u + 64u + 16u + 16u)) : "memory");
        __syncwarp();
        copy(raw + TC_Q6_QL + row * 144, grp + 128 * bb, 128);
        copy(raw + TC_Q6_QH + row * 80, grp + 1024 + 64 * bb, 64);
        copy(raw + TC_Q6_SC + row * 16, grp + 1536 + 16 * bb, 16);
        copy(raw + TC_Q6_D + row * 16, grp + 1664, 16);
    }
}

// The thread's bytes of 16 weights - sixteenth `kq` (0..3) of the 64-column quarter `c` of the block: shared memory -> registers.
struct TcRaw {
    uint4 hdr, q, h;  // Q4_K / Q5_K: header, 16 quant bytes, (Q5_K) the 16 high-bit bytes; Q6_K: q = low bits, h = high bits
    uint32_t s, d;    // Q6_K: the scale of the 16 weights, the block's f16 scale
};
template <int PATH>
__device__ __forceinline__ void tc_read_raw(uint32_t raw, uint32_t row, uint32_t kb, uint32_t c, uint32_t kq, TcRaw &r) {
    const uint32_t hq = kq & 1;   // which 16 of the sub-block's 32 weights
    if (PATH == TC_PATH_Q4K) {
        const uint32_t blk = raw + row * 144;
        r.hdr = tc_lds128(blk);
        r.q = tc_lds128(blk + 16 + 32 * c + 16 * hq);
    } else if (PATH == TC_PATH_Q5K) {
        const uint32_t blk = raw + row * 176;
        r.hdr = tc_lds128(blk);
        r.q = tc_lds128(blk + 48 + 32 * c + 16 * hq);
        r.h = tc_lds128(blk + 16 + 16 * hq);
    } else if (PATH == TC_PATH_Q6K) {
        const uint32_t i = c >> 1, g = (2 * c + (kq >> 1)) & 3;
        r.q = tc_lds128(raw + TC_Q6_QL + row * 144 + 64 * i + 32 * (g & 1) + 16 * hq);
        r.h = tc_lds128(raw + TC_Q6_QH + row * 80 + 32 * i + 16 * hq);
        r.s = tc_lds8(raw + TC_Q6_SC + row * 16 + 8 * i + 2 * g + hq);
        r.d = tc_lds16(raw + TC_Q6_D + row * 16 + 2 * (kb & 7));
    }
}

// crates/inferi/src/quantization.rs:364-402 (Q4_K) and :287-329 (Q5_K): sub-block j of the block, low or high nibbles of a
// 32-byte chunk, w = d * sc * q - dmin * m
template <bool Q5>
__device__ __forceinline__ void tc_convert16_q45k(const TcRaw &r, uint32_t k0, float (&w)[16]) {
    const uint32_t j = (k0 & 255) >> 5, c = j >> 1, high = j & 1;
    const uint4 hdr = r.hdr;
    // get_scale_min_k4 (quantization.rs:394-402) on the 12 scale bytes held in hdr.y, hdr.z, hdr.w
    const uint32_t sb[3] = {hdr.y, hdr.z, hdr.w};
    auto byte_at = [&](uint32_t i) { return (sb[i >> 2] >> (8 * (i & 3))) & 0xFFu; };
    uint32_t sc, mn;
    if (j < 4) { sc = byte_at(j) & 63; mn = byte_at(j + 4) & 63; }
    else { sc = (byte_at(j + 4) & 0xF) | ((byte_at(j - 4) >> 6) << 4); mn = (byte_at(j + 4) >> 4) | ((byte_at(j) >> 6) << 4); }
    const float dsc = tc_h2f(hdr.x & 0xFFFFu) * (float)sc, dm = tc_h2f(hdr.x >> 16) * (float)mn;
    const uint32_t qw[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
    const uint32_t hw[4] = {r.h.x, r.h.y, r.h.z, r.h.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t nib = high ? (qw[i] >> 4) & 0x0F0F0F0Fu : qw[i] & 0x0F0F0F0Fu;
        if (Q5) nib |= ((hw[i] >> (2 * c + high)) & 0x01010101u) << 4;
#pragma unroll
        for (int b = 0; b < 4; b++) w[4 * i + b] = (float)((nib >> (8 * b)) & 0xFFu) * dsc - dm;
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
    if (PATH == TC_PATH_Q4K) tc_convert16_q45k<false>(r, k0, w);
    else if (PATH == TC_PATH_Q5K) tc_convert16_q45k<true>(r, k0, w);
    else if (PATH == TC_PATH_Q6K) tc_convert16_q6k_soa(r, k0, w);
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
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_quant_tc_kernel(const GemmTcParams p) {
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
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_rawfull + 8 * s), "r"(TC_ROWS / 32));               // one arrival per copying warp
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
        // the ring of raw blocks is filled ahead: one block of every row of the unit's tile per step, each row by its own bulk copy
        uint32_t issued = 0;
        for (; issued < R && issued < nunits; issued++) {
            if (RAW && tid < TC_ROWS) tc_issue_raw<PATH>(row_at(ptile), pkb, raw0 + issued * RAW_BYTES, row, bar_rawfull + 8 * issued);
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
                    if (tid < TC_ROWS) {
                        ok = __all_sync(0xffffffffu, tc_wait(bar_rawempty + 8 * pslot, pslot_par, p.wait_ns, p.err, 8));   // warp-uniform: the lanes stay together
                        if (!ok) break;
                        tc_issue_raw<PATH>(row_at(ptile), pkb, raw0 + pslot * RAW_BYTES, row, bar_rawfull + 8 * pslot);
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
        for (uint32_t it = 0; it < nstage && ok; it++) {
            const uint32_t s = it % TC_STAGES, round = it / TC_STAGES;
            const uint32_t xs = it % TC_XSTAGES;
            const uint32_t j = it >> 2, c = it & 3, u = u0 + j, kb = u % sk.nb;
            const bool seg_first = c == 0 && (j == 0 || kb == 0), seg_last = c == 3 && (kb + 1 == sk.nb || u + 1 == u1);
            ok = tc_wait(bar_xfull + 8 * xs, (it / TC_XSTAGES) & 1, p.wait_ns, p.err, 9) && tc_wait(bar0 + 8 * s, round & 1, p.wait_ns, p.err, 9);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t st = tc_smem_u32(smem + s * TC_STAGE_BYTES), xt = tc_smem_u32(xst + xs * TC_STAGE_BYTES);
#pragma unroll
            for (uint32_t kk = 0; kk < TC_KSTAGE / 16; kk++) {
                const uint32_t koff = kk * 2 * TC_LBO;   // 16 columns = two core matrices along K
                const uint64_t w_hi = tc_smem_desc(st + koff, TC_LBO, TC_SBO), w_lo = tc_smem_desc(st + TC_TILE_BYTES + koff, TC_LBO, TC_SBO);
                const uint64_t x_hi = tc_smem_desc(xt + koff, TC_LBO, TC_SBO), x_lo = tc_smem_desc(xt + TC_TILE_BYTES + koff, TC_LBO, TC_SBO);
                tc_mma_f16(tmem_base, w_hi, x_hi, idesc, !(seg_first && kk == 0));   // a segment starts a new sum
                tc_mma_f16(tmem_base, w_hi, x_lo, idesc, 1);
                tc_mma_f16(tmem_base, w_lo, x_hi, idesc, 1);
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
    __shared__ float red[8];
    const uint32_t t = blockIdx.x;
    if (t >= n) {
        for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) { hi[tc_x_index(t, c)] = __float2half_rn(0.f); lo[tc_x_index(t, c)] = __float2half_rn(0.f); }
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
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) split_store(hi, lo, tc_x_index(t, c), w ? (x[c] * rms) * w[c] : x[c]);
}

__device__ __forceinline__ float plane_sum(const float *planes, uint32_t pieces, size_t plane_elems, size_t i) {
    float v = 0.f;
    for (uint32_t s = 0; s < pieces; s++) v += planes[s * plane_elems + i];   // fixed order: deterministic
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
            continue;
        }
        const uint32_t np = p.sk.pieces(r / 128);   // the planes that the row's tile was spread over
        float a = plane_sum(p.planes, np, plane, i), b = plane_sum(p.planes, np, plane, i + 1);
        if (p.mode == PE_SWIGLU) {
            // crates/inferi-shaders/src/silu.rs:16-19,46-52
            const float ua = plane_sum(p.planes2, np, plane, i), ub = plane_sum(p.planes2, np, plane, i + 1);
            split_store(p.hi, p.lo, tc_x_index(t, r), ua * (a / (1.0f + expf(-a))));
            split_store(p.hi, p.lo, tc_x_index(t, r + 1), ub * (b / (1.0f + expf(-b))));
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

bool prefill_gemm_eligible(const ib_qtensor *m) {
    return m->rows % TC_ROWS == 0 && m->cols % 256 == 0 && (m->qtype == IB_Q4_K || m->qtype == IB_Q5_K || m->qtype == IB_Q6_K || m->qtype == IB_Q8_0);
}

int32_t launch_prefill_gemm(ib_ctx *ctx, cudaStream_t s, const ib_qtensor *m, const __half *x_hi, const __half *x_lo, uint32_t n, float *planes, const StreamK &sk) {
    const int path = tc_path((uint32_t)m->qtype, m->layout);
    const uint32_t raw_bytes = tc_raw_stage_bytes(path);
    uint32_t raw_stages = raw_bytes ? (TC_SMEM_LIMIT - TC_SMEM_FIXED) / raw_bytes : 1;
    if (raw_stages > TC_RAW_MAX) raw_stages = TC_RAW_MAX;
    const uint32_t smem_bytes = TC_SMEM_FIXED + raw_stages * raw_bytes;
    void (*kernel)(GemmTcParams) = path == TC_PATH_Q4K ? gemm_quant_tc_kernel<TC_PATH_Q4K>
                                   : (path == TC_PATH_Q5K ? gemm_quant_tc_kernel<TC_PATH_Q5K>
                                                          : (path == TC_PATH_Q6K ? gemm_quant_tc_kernel<TC_PATH_Q6K> : gemm_quant_tc_kernel<TC_PATH_OTHER>));
    static bool attr_set[16][4] = {};
    if (!attr_set[ctx->device & 15][path]) {
        IB_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(TC_SMEM_LIMIT)));
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
    kernel<<<sk.ctas, TC_THREADS, smem_bytes, s>>>(p);
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
    prefill_norm_split_kernel<<<(n + 15) & ~15u, 256, 0, s>>>(X, w, eps, n, cols, hi, lo);
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
    const size_t half_bytes = (size_t)TC_ROWS * cols * sizeof(__half), plane_bytes = (size_t)ks * TC_ROWS * rows * sizeof(float);
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
