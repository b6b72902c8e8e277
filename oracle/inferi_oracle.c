/*
 * CPU oracle for the batch-1 Llama token loop over GGUF-quantized weights.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference's arithmetic for that path; it exists so that the CUDA kernels can
 * be checked against it and so that a CPU baseline can be timed beside them.
 * Nothing in the shipped library links, loads or calls it.
 *
 * Parity status: the reference (dimforge/inferi) is Rust and cannot be built
 * where this oracle was written, and its tests hold no fixed-value vectors for
 * this path (they draw unseeded random inputs and compare shader output to
 * `Block*::dequantize` + dot).  The block dequantizers below are pinned
 * against the independent `gguf` Python package (same ggml block semantics the
 * reference cites); the shader restatements are pinned against the
 * dequantize+dot definition, which is the relationship the reference's own
 * tests assert.  Attention, the whole-model forward and greedy argmax have no
 * live reference test: "parity unpinned" for those.
 *
 * Every function cites the reference file:line it follows (paths are relative
 * to the reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QK_K 256

enum { ORC_F32 = 0, ORC_Q4_0 = 2, ORC_Q4_1 = 3, ORC_Q5_0 = 6, ORC_Q5_1 = 7, ORC_Q8_0 = 8, ORC_Q4_K = 12, ORC_Q5_K = 13, ORC_Q6_K = 14, ORC_Q8_K = 15 };

/* ---- block formats: crates/inferi/src/quantization.rs:42-45, 217-222, 262-268, 335-340 ---- */
#pragma pack(push, 1)
typedef struct { uint16_t scale; int8_t data[32]; } blk_q8_0;                                   /* 34 B  */
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qs[128]; } blk_q4_k;             /* 144 B */
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qh[32]; uint8_t qs[128]; } blk_q5_k; /* 176 B */
typedef struct { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; } blk_q6_k;    /* 210 B */
typedef struct { uint16_t d; uint8_t qs[16]; } blk_q4_0;                                        /* 18 B  */
typedef struct { uint16_t d, m; uint8_t qs[16]; } blk_q4_1;                                     /* 20 B  */
typedef struct { uint16_t d; uint8_t qh[4]; uint8_t qs[16]; } blk_q5_0;                         /* 22 B  */
typedef struct { uint16_t d, m; uint8_t qh[4]; uint8_t qs[16]; } blk_q5_1;                      /* 24 B  */
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } blk_q8_k;                        /* 292 B */
#pragma pack(pop)

size_t orc_block_bytes(int qtype) {
    switch (qtype) {
    case ORC_F32: return 4;
    case ORC_Q8_0: return sizeof(blk_q8_0);
    case ORC_Q4_K: return sizeof(blk_q4_k);
    case ORC_Q5_K: return sizeof(blk_q5_k);
    case ORC_Q6_K: return sizeof(blk_q6_k);
    case ORC_Q4_0: return sizeof(blk_q4_0);
    case ORC_Q4_1: return sizeof(blk_q4_1);
    case ORC_Q5_0: return sizeof(blk_q5_0);
    case ORC_Q5_1: return sizeof(blk_q5_1);
    case ORC_Q8_K: return sizeof(blk_q8_k);
    default: return 0;
    }
}

size_t orc_block_elems(int qtype) {
    switch (qtype) {
    case ORC_F32: return 1;
    case ORC_Q8_0: case ORC_Q4_0: case ORC_Q4_1: case ORC_Q5_0: case ORC_Q5_1: return 32;
    case ORC_Q4_K: case ORC_Q5_K: case ORC_Q6_K: case ORC_Q8_K: return QK_K;
    default: return 0;
    }
}

/* crates/inferi/src/quantization.rs:405-422 (decode_f16): exact IEEE binary16 -> binary32. */
float orc_decode_f16(uint16_t half) {
    uint16_t exp = (half >> 10) & 0x1f;
    uint16_t mant = half & 0x3ff;
    float val;
    if (exp == 0) val = (float)mant * ldexpf(1.0f, -24);
    else if (exp != 31) val = ((float)mant + 1024.0f) * ldexpf(1.0f, (int)exp - 25);
    else if (mant == 0) val = INFINITY;
    else val = NAN;
    return (half & 0x8000) ? -val : val;
}

/* binary32 -> binary16, round to nearest even (the rounding the GPU's f16 KV store uses).
 * No reference counterpart: the reference keeps its KV cache in f32
 * (crates/inferi/src/models/llama2/transformer.rs:85-104). */
uint16_t orc_encode_f16(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mant = x & 0x007fffffu;
    int32_t exp = (int32_t)((x >> 23) & 0xff);
    if (exp == 255) return (uint16_t)(sign | 0x7c00u | (mant ? 0x200u : 0));
    int32_t e = exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        mant |= 0x00800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t h = mant >> shift;
        uint32_t rem = mant & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (h & 1u))) h++;
        return (uint16_t)(sign | h);
    }
    uint32_t h = ((uint32_t)e << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
    return (uint16_t)(sign | h);
}

/* crates/inferi/src/quantization.rs:394-402 (get_scale_min_k4). */
static inline void get_scale_min_k4(int j, const uint8_t *q, uint8_t *d, uint8_t *m) {
    if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
    else { *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

/* crates/inferi/src/quantization.rs:51-54 (BlockQ8_0::dequantize). */
static void deq_q8_0(const blk_q8_0 *b, float *out) {
    float s = orc_decode_f16(b->scale);
    for (int i = 0; i < 32; i++) out[i] = (float)b->data[i] * s;
}

/* crates/inferi/src/quantization.rs:364-391 (BlockQ4K::dequantize). */
static void deq_q4_k(const blk_q4_k *b, float *out) {
    float d = orc_decode_f16(b->d), mn = orc_decode_f16(b->dmin);
    int is = 0, iq = 0; uint8_t sc, m;
    for (int j = 0; j < QK_K; j += 64) {
        get_scale_min_k4(is, b->scales, &sc, &m);
        float d1 = d * (float)sc, m1 = mn * (float)m;
        get_scale_min_k4(is + 1, b->scales, &sc, &m);
        float d2 = d * (float)sc, m2 = mn * (float)m;
        for (int l = 0; l < 32; l++) out[j + l] = d1 * (float)(b->qs[iq + l] & 0xF) - m1;
        for (int l = 0; l < 32; l++) out[j + l + 32] = d2 * (float)(b->qs[iq + l] >> 4) - m2;
        iq += 32; is += 2;
    }
}

/* crates/inferi/src/quantization.rs:287-329 (BlockQ5K::dequantize). */
static void deq_q5_k(const blk_q5_k *b, float *out) {
    float d = orc_decode_f16(b->d), mn = orc_decode_f16(b->dmin);
    int is = 0, iq = 0; uint8_t sc, m; uint8_t u1 = 1, u2 = 2;
    for (int j = 0; j < QK_K; j += 64) {
        get_scale_min_k4(is, b->scales, &sc, &m);
        float d1 = d * (float)sc, m1 = mn * (float)m;
        get_scale_min_k4(is + 1, b->scales, &sc, &m);
        float d2 = d * (float)sc, m2 = mn * (float)m;
        for (int l = 0; l < 32; l++)
            out[j + l] = d1 * (float)((b->qs[iq + l] & 0xF) + ((b->qh[l] & u1) ? 16 : 0)) - m1;
        for (int l = 0; l < 32; l++)
            out[j + l + 32] = d2 * (float)((b->qs[iq + l] >> 4) + ((b->qh[l] & u2) ? 16 : 0)) - m2;
        iq += 32; is += 2; u1 <<= 2; u2 <<= 2;
    }
}

/* crates/inferi/src/quantization.rs:227-256 (BlockQ6K::dequantize). */
static void deq_q6_k(const blk_q6_k *b, float *out) {
    float d = orc_decode_f16(b->d);
    for (int i = 0; i < 2; i++) {
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            uint8_t ql0 = b->ql[i * 64 + l], ql32 = b->ql[i * 64 + l + 32], qh = b->qh[i * 32 + l];
            int8_t q1 = (int8_t)((ql0 & 0xF) | (((qh >> 0) & 3) << 4)) - 32;
            int8_t q2 = (int8_t)((ql32 & 0xF) | (((qh >> 2) & 3) << 4)) - 32;
            int8_t q3 = (int8_t)((ql0 >> 4) | (((qh >> 4) & 3) << 4)) - 32;
            int8_t q4 = (int8_t)((ql32 >> 4) | (((qh >> 6) & 3) << 4)) - 32;
            out[i * 128 + l + 0] = d * (float)b->scales[i * 8 + is + 0] * (float)q1;
            out[i * 128 + l + 32] = d * (float)b->scales[i * 8 + is + 2] * (float)q2;
            out[i * 128 + l + 64] = d * (float)b->scales[i * 8 + is + 4] * (float)q3;
            out[i * 128 + l + 96] = d * (float)b->scales[i * 8 + is + 6] * (float)q4;
        }
    }
}

/* crates/inferi/src/quantization.rs:68-82 (BlockQ4_0::dequantize). */
static void deq_q4_0(const blk_q4_0 *b, float *out) {
    float d = orc_decode_f16(b->d);
    for (int j = 0; j < 16; j++) {
        out[j] = (float)((int)(b->qs[j] & 0x0F) - 8) * d;
        out[j + 16] = (float)((int)(b->qs[j] >> 4) - 8) * d;
    }
}

/* crates/inferi/src/quantization.rs:96-111 (BlockQ4_1::dequantize). */
static void deq_q4_1(const blk_q4_1 *b, float *out) {
    float d = orc_decode_f16(b->d), m = orc_decode_f16(b->m);
    for (int j = 0; j < 16; j++) {
        out[j] = (float)(b->qs[j] & 0x0F) * d + m;
        out[j + 16] = (float)(b->qs[j] >> 4) * d + m;
    }
}

/* crates/inferi/src/quantization.rs:125-142 (BlockQ5_0::dequantize). */
static void deq_q5_0(const blk_q5_0 *b, float *out) {
    float d = orc_decode_f16(b->d);
    uint32_t qh; memcpy(&qh, b->qh, 4);
    for (int j = 0; j < 16; j++) {
        uint32_t xh0 = ((qh >> j) << 4) & 0x10, xh1 = (qh >> (j + 12)) & 0x10;
        out[j] = (float)((int)((b->qs[j] & 0x0Fu) | xh0) - 16) * d;
        out[j + 16] = (float)((int)((uint32_t)(b->qs[j] >> 4) | xh1) - 16) * d;
    }
}

/* crates/inferi/src/quantization.rs:157-175 (BlockQ5_1::dequantize). */
static void deq_q5_1(const blk_q5_1 *b, float *out) {
    float d = orc_decode_f16(b->d), m = orc_decode_f16(b->m);
    uint32_t qh; memcpy(&qh, b->qh, 4);
    for (int j = 0; j < 16; j++) {
        uint32_t xh0 = ((qh >> j) << 4) & 0x10, xh1 = (qh >> (j + 12)) & 0x10;
        out[j] = (float)((b->qs[j] & 0x0Fu) | xh0) * d + m;
        out[j + 16] = (float)((uint32_t)(b->qs[j] >> 4) | xh1) * d + m;
    }
}

/* crates/inferi/src/quantization.rs:205-211 (BlockQ8K::dequantize). */
static void deq_q8_k(const blk_q8_k *b, float *out) {
    for (int j = 0; j < QK_K; j++) out[j] = b->d * (float)b->qs[j];
}

static void deq_block(int qtype, const uint8_t *blk, float *out) {
    switch (qtype) {
    case ORC_Q4_0: deq_q4_0((const blk_q4_0 *)blk, out); break;
    case ORC_Q4_1: deq_q4_1((const blk_q4_1 *)blk, out); break;
    case ORC_Q5_0: deq_q5_0((const blk_q5_0 *)blk, out); break;
    case ORC_Q5_1: deq_q5_1((const blk_q5_1 *)blk, out); break;
    case ORC_Q8_K: deq_q8_k((const blk_q8_k *)blk, out); break;
    case ORC_Q8_0: deq_q8_0((const blk_q8_0 *)blk, out); break;
    case ORC_Q4_K: deq_q4_k((const blk_q4_k *)blk, out); break;
    case ORC_Q5_K: deq_q5_k((const blk_q5_k *)blk, out); break;
    case ORC_Q6_K: deq_q6_k((const blk_q6_k *)blk, out); break;
    default: break;
    }
}

/* Dequantize `nblocks` consecutive blocks of `qtype` into f32. */
int orc_dequantize(int qtype, const void *blocks, size_t nblocks, float *out) {
    size_t bb = orc_block_bytes(qtype), be = orc_block_elems(qtype);
    if (!bb) return -1;
    if (qtype == ORC_F32) { memcpy(out, blocks, nblocks * 4); return 0; }
    const uint8_t *p = (const uint8_t *)blocks;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)nblocks; i++) deq_block(qtype, p + (size_t)i * bb, out + (size_t)i * be);
    return 0;
}

/* One row of a quantized (or f32) matrix dotted with v, accumulated in f64.
 * crates/inferi/src/ops/gemv_quant.rs:444-456 (cpu_gemv: dequantize, f64 accumulate, cast). */
static double row_dot(int qtype, const uint8_t *row, size_t cols, const float *v) {
    double acc = 0.0;
    if (qtype == ORC_F32) {
        const float *w = (const float *)row;
        for (size_t c = 0; c < cols; c++) acc += (double)w[c] * (double)v[c];
        return acc;
    }
    size_t bb = orc_block_bytes(qtype), be = orc_block_elems(qtype);
    float tmp[QK_K];
    for (size_t b = 0; b < cols / be; b++) {
        deq_block(qtype, row + b * bb, tmp);
        const float *vv = v + b * be;
        for (size_t e = 0; e < be; e++) acc += (double)tmp[e] * (double)vv[e];
    }
    return acc;
}

static size_t row_bytes(int qtype, size_t cols) { return cols / orc_block_elems(qtype) * orc_block_bytes(qtype); }

/* out = W v with W [rows, cols] row-major in GGUF blocks; the definition every GEMV is checked against. */
int orc_gemv_ref(int qtype, size_t rows, size_t cols, const void *blocks, const float *v, float *out, int nthreads) {
    size_t be = orc_block_elems(qtype);
    if (!be || cols % be) return -1;
    size_t rb = row_bytes(qtype, cols);
    const uint8_t *p = (const uint8_t *)blocks;
    if (nthreads <= 0) nthreads = 1;
#pragma omp parallel for schedule(static) num_threads(nthreads)
    for (long long r = 0; r < (long long)rows; r++) out[r] = (float)row_dot(qtype, p + (size_t)r * rb, cols, v);
    return 0;
}

/* ---------------------------------------------------------------------------------------------
 * Lane-structured restatements of the reference GEMV shaders: one "workgroup" of 32 lanes per 4
 * output rows, every lane keeping an f32 partial per row over the elements the shader assigns to it,
 * then the shader's shared-memory tree (16,8,4,2,1).  This is the stand-in for the reference's shader
 * code run on host cores (its `cpu` backend) and the timed CPU baseline.
 * ------------------------------------------------------------------------------------------- */

static inline float dot4(const float *a, const float *b) { return ((a[0] * b[0] + a[1] * b[1]) + a[2] * b[2]) + a[3] * b[3]; }

static void tree_reduce(float sum[32][4], float *out4) {
    for (int stride = 16; stride >= 1; stride >>= 1)
        for (int i = 0; i < stride; i++)
            for (int r = 0; r < 4; r++) sum[i][r] += sum[i + stride][r];
    for (int r = 0; r < 4; r++) out4[r] = sum[0][r];
}

/* crates/inferi-shaders/src/gemv_quant_q8_0x2.rs:50-134: per iteration 128 columns; lane `lid` owns
 * columns 128j + 4*lid .. +3 of Q8_0 block 4j + lid/8. */
static void wg_q8_0(const uint8_t *rows4[4], size_t cols, const float *v, float *out4) {
    float sum[32][4]; memset(sum, 0, sizeof sum);
    size_t iters = cols / 128;
    for (size_t j = 0; j < iters; j++)
        for (int lid = 0; lid < 32; lid++) {
            const float *vj = v + 128 * j + 4 * lid;
            for (int r = 0; r < 4; r++) {
                const blk_q8_0 *b = (const blk_q8_0 *)rows4[r] + 4 * j + lid / 8;
                float s = orc_decode_f16(b->scale), row[4];
                for (int e = 0; e < 4; e++) row[e] = (float)b->data[4 * (lid % 8) + e] * s;
                sum[lid][r] += dot4(row, vj);
            }
        }
    tree_reduce(sum, out4);
}

/* crates/inferi-shaders/src/gemv_quant_q4_k.rs:47-93,120-151 and gemv_quant_q5_k.rs:48-107: one
 * super-block per iteration; lane k owns qs word k: low nibbles -> columns 64(k/8)+4(k%8)+0..3 with
 * sub-block 2(k/8), high nibbles -> +32 with sub-block 2(k/8)+1. */
static void wg_q45_k(int qtype, const uint8_t *rows4[4], size_t cols, const float *v, float *out4) {
    float sum[32][4]; memset(sum, 0, sizeof sum);
    size_t nb = cols / QK_K;
    size_t bb = orc_block_bytes(qtype);
    for (size_t j = 0; j < nb; j++)
        for (int k = 0; k < 32; k++) {
            int ch = k / 8, l = k % 8;
            const float *va = v + 256 * j + 64 * ch + 4 * l, *vb = va + 32;
            for (int r = 0; r < 4; r++) {
                const uint8_t *blk = rows4[r] + j * bb;
                const blk_q4_k *b4 = (const blk_q4_k *)blk;
                const blk_q5_k *b5 = (const blk_q5_k *)blk;
                float d = orc_decode_f16(b4->d), mn = orc_decode_f16(b4->dmin);
                uint8_t sc, m;
                get_scale_min_k4(2 * ch, b4->scales, &sc, &m);
                float d1 = d * (float)sc, m1 = mn * (float)m;
                get_scale_min_k4(2 * ch + 1, b4->scales, &sc, &m);
                float d2 = d * (float)sc, m2 = mn * (float)m;
                float a[4], bq[4];
                for (int e = 0; e < 4; e++) {
                    if (qtype == ORC_Q4_K) {
                        uint8_t q = b4->qs[32 * ch + 4 * l + e];
                        a[e] = (float)(q & 0xF) * d1 - m1;
                        bq[e] = (float)(q >> 4) * d2 - m2;
                    } else {
                        uint8_t q = b5->qs[32 * ch + 4 * l + e], h = b5->qh[4 * l + e];
                        a[e] = (float)((q & 0xF) + ((h & (1u << (2 * ch))) ? 16 : 0)) * d1 - m1;
                        bq[e] = (float)((q >> 4) + ((h & (2u << (2 * ch))) ? 16 : 0)) * d2 - m2;
                    }
                }
                sum[k][r] += dot4(a, va);
                sum[k][r] += dot4(bq, vb);
            }
        }
    tree_reduce(sum, out4);
}

/* crates/inferi-shaders/src/gemv_quant_q6_kx2.rs:45-140,167-193: one pair of super-blocks (512 columns)
 * per iteration; lane k owns block k/16 of the pair, 128-half i=(k/8)%2, byte group l=k%8: columns
 * 128i+4l+0..3 and +32,+64,+96. */
static void wg_q6_k(const uint8_t *rows4[4], size_t cols, const float *v, float *out4) {
    float sum[32][4]; memset(sum, 0, sizeof sum);
    size_t iters = cols / 512;
    for (size_t j = 0; j < iters; j++)
        for (int k = 0; k < 32; k++) {
            int blk = k / 16, i = (k / 8) % 2, l = k % 8, is = l / 4;
            const float *vj = v + 512 * j + 256 * blk + 128 * i + 4 * l;
            for (int r = 0; r < 4; r++) {
                const blk_q6_k *b = (const blk_q6_k *)rows4[r] + 2 * j + blk;
                float d = orc_decode_f16(b->d);
                float p[4][4];
                for (int e = 0; e < 4; e++) {
                    uint8_t ql0 = b->ql[64 * i + 4 * l + e], ql32 = b->ql[64 * i + 32 + 4 * l + e], qh = b->qh[32 * i + 4 * l + e];
                    int q1 = (int)((ql0 & 0xF) | ((qh & 3) << 4)) - 32;
                    int q2 = (int)((ql32 & 0xF) | (((qh >> 2) & 3) << 4)) - 32;
                    int q3 = (int)((ql0 >> 4) | (((qh >> 4) & 3) << 4)) - 32;
                    int q4 = (int)((ql32 >> 4) | (((qh >> 6) & 3) << 4)) - 32;
                    p[0][e] = (d * (float)b->scales[8 * i + is + 0]) * (float)q1;
                    p[1][e] = (d * (float)b->scales[8 * i + is + 2]) * (float)q2;
                    p[2][e] = (d * (float)b->scales[8 * i + is + 4]) * (float)q3;
                    p[3][e] = (d * (float)b->scales[8 * i + is + 6]) * (float)q4;
                }
                sum[k][r] += ((dot4(p[0], vj) + dot4(p[1], vj + 32)) + dot4(p[2], vj + 64)) + dot4(p[3], vj + 96);
            }
        }
    tree_reduce(sum, out4);
}

/* Shader-structured GEMV over all workgroups (crates/inferi/src/ops/gemv_quant.rs:265-275: grid = rows/4). */
int orc_gemv_shader(int qtype, size_t rows, size_t cols, const void *blocks, const float *v, float *out, int nthreads) {
    if (rows % 4) return -1;
    if (qtype == ORC_Q8_0 && cols % 128) return -1;
    if ((qtype == ORC_Q4_K || qtype == ORC_Q5_K) && cols % 256) return -1;
    if (qtype == ORC_Q6_K && cols % 512) return -1;
    if (qtype != ORC_Q8_0 && qtype != ORC_Q4_K && qtype != ORC_Q5_K && qtype != ORC_Q6_K) return -1;
    size_t rb = row_bytes(qtype, cols);
    const uint8_t *p = (const uint8_t *)blocks;
    if (nthreads <= 0) nthreads = 1;
#pragma omp parallel for schedule(static) num_threads(nthreads)
    for (long long wg = 0; wg < (long long)(rows / 4); wg++) {
        const uint8_t *rows4[4];
        for (int r = 0; r < 4; r++) rows4[r] = p + ((size_t)wg * 4 + r) * rb;
        if (qtype == ORC_Q8_0) wg_q8_0(rows4, cols, v, out + 4 * wg);
        else if (qtype == ORC_Q6_K) wg_q6_k(rows4, cols, v, out + 4 * wg);
        else wg_q45_k(qtype, rows4, cols, v, out + 4 * wg);
    }
    return 0;
}

/* ---- element-wise ops ---- */

/* crates/inferi-shaders/src/rms_norm.rs:112-120: rms = 1/sqrt(sum(x^2)/n + eps); out = (x*rms)*w.
 * The sum of squares is taken in f64 so the oracle bounds every f32 summation order. */
void orc_rms_norm(float *out, const float *x, const float *w, size_t n, float eps) {
    double ss = 0.0;
    for (size_t i = 0; i < n; i++) ss += (double)x[i] * (double)x[i];
    float rms = 1.0f / sqrtf((float)(ss / (double)n) + eps);
    for (size_t i = 0; i < n; i++) out[i] = (x[i] * rms) * w[i];
}

/* crates/inferi-shaders/src/rope.rs:75-91 (Original: adjacent pairs) and :97-141 (NeoX: split halves).
 * variant 0 = Original, 1 = NeoX.  base_freq comes from the model config, not the constant in
 * crates/inferi/src/models/llama2/cpu.rs:473. */
void orc_rope(int variant, float *q, size_t q_len, float *k, size_t kv_dim, uint32_t head_size, uint32_t pos, float base_freq) {
    for (size_t i = 0; i < q_len / 2; i++) {
        if (variant == 0) {
            float head_dim = (float)((i * 2) % head_size);
            float theta = powf(base_freq, -head_dim / (float)head_size);
            float a = (float)pos * theta, c = cosf(a), s = sinf(a);
            float x = q[2 * i], y = q[2 * i + 1];
            q[2 * i] = c * x - s * y; q[2 * i + 1] = s * x + c * y;
            if (2 * i < kv_dim) {
                x = k[2 * i]; y = k[2 * i + 1];
                k[2 * i] = c * x - s * y; k[2 * i + 1] = s * x + c * y;
            }
        } else {
            size_t half = head_size / 2, head = i / half, j = i % half;
            float theta = powf(base_freq, -(float)(2 * j) / (float)head_size);
            float a = (float)pos * theta, c = cosf(a), s = sinf(a);
            size_t i0 = head * head_size + j, i1 = i0 + half;
            float x = q[i0], y = q[i1];
            q[i0] = c * x - s * y; q[i1] = s * x + c * y;
            if (i0 < kv_dim) {
                x = k[i0]; y = k[i1];
                k[i0] = c * x - s * y; k[i1] = s * x + c * y;
            }
        }
    }
}

/* crates/inferi-shaders/src/silu.rs:16-19,46-52: h1 <- h2 * (h1 / (1 + exp(-h1))). */
void orc_silu_mul(float *h1, const float *h2, size_t n) {
    for (size_t i = 0; i < n; i++) h1[i] = h2[i] * (h1[i] / (1.0f + expf(-h1[i])));
}

/* crates/inferi/src/context.rs:516-530: a += b. */
void orc_add_assign(float *a, const float *b, size_t n) { for (size_t i = 0; i < n; i++) a[i] += b[i]; }

/* crates/inferi/src/models/sampler.rs:54-56 (greedy).  Ties go to the lowest index (the reference's
 * nalgebra `imax` tie rule is not pinned by any test). */
uint32_t orc_argmax(const float *x, size_t n) {
    size_t best = 0;
    for (size_t i = 1; i < n; i++) if (x[i] > x[best]) best = i;
    return (uint32_t)best;
}

/* Coin of a position: splitmix64 of (seed, position), top 24 bits -> [0, 1).  The reference draws its coin with an
 * unseeded rand::random() (sampler.rs:41); a reproducible stand-in shared with the device sampler. */
float orc_sample_coin(uint64_t seed, uint32_t pos) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * ((uint64_t)pos + 1ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(uint32_t)(z >> 40) * (1.0f / 16777216.0f);
}

typedef struct { float prob; uint32_t index; } orc_prob_index;
static int cmp_prob_desc(const void *a, const void *b) {
    const orc_prob_index *x = (const orc_prob_index *)a, *y = (const orc_prob_index *)b;
    if (x->prob != y->prob) return x->prob > y->prob ? -1 : 1;   /* decreasing probability */
    return x->index < y->index ? -1 : (x->index > y->index);      /* stable: the reference's sort_by_key keeps index order */
}

/* crates/inferi/src/models/sampler.rs:32-130 (Sampler::sample with sample_mult / sample_topp) and the CPU softmax it calls
 * (crates/inferi/src/ops/softmax.rs:130-143), sequential f32 sums as there.  `logits` is not modified.  *margin receives the
 * smallest distance between a threshold (the coin, topp, coin * cumulative) and the running sums next to the decision: a
 * parallel sum may decide differently only when it is tiny. */
uint32_t orc_sample(const float *logits, size_t n, float temperature, float topp, float coin, float *margin) {
    float mg = 1.0f;
    if (margin) *margin = mg;
    if (temperature == 0.0f) return orc_argmax(logits, n);
    float *p = (float *)malloc(n * sizeof(float));
    float mx = -INFINITY, sum = 0.0f;
    for (size_t i = 0; i < n; i++) { p[i] = logits[i] / temperature; if (p[i] > mx) mx = p[i]; }
    for (size_t i = 0; i < n; i++) { p[i] = expf(p[i] - mx); sum += p[i]; }
    for (size_t i = 0; i < n; i++) p[i] /= sum;
    uint32_t tok;
    if (topp <= 0.0f || topp >= 1.0f) {
        float cdf = 0.0f;
        tok = (uint32_t)(n - 1);
        for (size_t i = 0; i < n; i++) {
            const float prev = cdf;
            cdf += p[i];
            if (coin < cdf) { tok = (uint32_t)i; mg = fminf(cdf - coin, i ? coin - prev : 1.0f); break; }
        }
    } else {
        orc_prob_index *pi = (orc_prob_index *)malloc(n * sizeof(orc_prob_index));
        size_t n0 = 0;
        const float cutoff = (1.0f - topp) / ((float)n - 1.0f);
        for (size_t i = 0; i < n; i++)
            if (p[i] >= cutoff) { pi[n0].index = (uint32_t)i; pi[n0].prob = p[i]; n0++; }
        if (n0 == 0) {
            /* No probability reaches the cut-off (possible when (1 - topp) / (n - 1) > max p, e.g. n = 2 with a small topp).
             * The reference computes n0 - 1 on an unsigned zero there (sampler.rs:108: a panic in a checked build);
             * the defined behaviour here and on the device is the arg-max. */
            free(pi); free(p);
            return orc_argmax(logits, n);
        }
        qsort(pi, n0, sizeof(orc_prob_index), cmp_prob_desc);
        float cumulative = 0.0f;
        size_t last = n0 - 1;
        for (size_t i = 0; i < n0; i++) {
            const float prev = cumulative;
            cumulative += pi[i].prob;
            if (cumulative > topp) { last = i; mg = fminf(mg, fminf(cumulative - topp, i ? topp - prev : 1.0f)); break; }
        }
        const float r = coin * cumulative;
        float cdf = 0.0f;
        tok = pi[last].index;
        for (size_t i = 0; i <= last; i++) {
            const float prev = cdf;
            cdf += pi[i].prob;
            if (r < cdf) { tok = pi[i].index; mg = fminf(mg, fminf(cdf - r, i ? r - prev : 1.0f)); break; }
        }
        free(pi);
    }
    free(p);
    if (margin) *margin = mg;
    return tok;
}

/* crates/inferi/src/ops/batched_multiquery_attention.rs:191-245 (run_cpu) with the softmax of
 * crates/inferi/src/models/llama2/cpu.rs:359-372.  KV rows are [pos, kv_dim] row-major
 * (crates/inferi-shaders/src/fused_attention.rs:107-108); kv_f16 selects a cache of binary16 values.
 * Scores and the weighted sum are taken in f64. */
typedef struct { uint32_t seq_len, kv_dim, kv_mul, n_heads, head_size, pos; } orc_attn_params;

void orc_attention(const orc_attn_params *p, const float *q, const void *kc, const void *vc, int kv_f16, float *out) {
    size_t hs = p->head_size, T = (size_t)p->pos + 1;
    float inv_div = sqrtf((float)hs);
#pragma omp parallel
    {
        double *att = (double *)malloc(T * sizeof(double));
        double *acc = (double *)malloc(hs * sizeof(double));
#pragma omp for schedule(static)
        for (long long h = 0; h < (long long)p->n_heads; h++) {
            const float *qh = q + (size_t)h * hs;
            size_t koff = ((size_t)h / p->kv_mul) * hs;
            double mx = -INFINITY;
            for (size_t t = 0; t < T; t++) {
                double s = 0.0;
                if (kv_f16) {
                    const uint16_t *kr = (const uint16_t *)kc + t * p->kv_dim + koff;
                    for (size_t d = 0; d < hs; d++) s += (double)qh[d] * (double)orc_decode_f16(kr[d]);
                } else {
                    const float *kr = (const float *)kc + t * p->kv_dim + koff;
                    for (size_t d = 0; d < hs; d++) s += (double)qh[d] * (double)kr[d];
                }
                s /= (double)inv_div;
                att[t] = s;
                if (s > mx) mx = s;
            }
            double sum = 0.0;
            for (size_t t = 0; t < T; t++) { att[t] = exp(att[t] - mx); sum += att[t]; }
            for (size_t d = 0; d < hs; d++) acc[d] = 0.0;
            for (size_t t = 0; t < T; t++) {
                double w = att[t] / sum;
                if (kv_f16) {
                    const uint16_t *vr = (const uint16_t *)vc + t * p->kv_dim + koff;
                    for (size_t d = 0; d < hs; d++) acc[d] += w * (double)orc_decode_f16(vr[d]);
                } else {
                    const float *vr = (const float *)vc + t * p->kv_dim + koff;
                    for (size_t d = 0; d < hs; d++) acc[d] += w * (double)vr[d];
                }
            }
            for (size_t d = 0; d < hs; d++) out[(size_t)h * hs + d] = (float)acc[d];
        }
        free(att); free(acc);
    }
}

/* ---- whole-model forward: op order of crates/inferi/src/models/llama2/transformer.rs:418-478 ---- */

typedef struct {
    uint32_t hidden, ffn, n_layers, n_heads, n_kv_heads, vocab, max_pos;
    float rope_theta, rms_eps;
} orc_llama_config;

typedef struct { int qtype; const void *data; } orc_qmat;

enum { ORC_W_Q = 0, ORC_W_K, ORC_W_V, ORC_W_O, ORC_W_GATE, ORC_W_UP, ORC_W_DOWN, ORC_W_PER_LAYER };

typedef struct orc_llama {
    orc_llama_config c;
    orc_qmat *mats;            /* [n_layers * 7] */
    const float **attn_norm;   /* [n_layers] */
    const float **ffn_norm;    /* [n_layers] */
    orc_qmat token_embd, output;
    const float *output_norm;
    int kv_f16, nthreads, gemv_mode; /* gemv_mode 0: dequantize + f64 dot; 1: shader-structured f32 (CPU baseline) */
    uint32_t kv_dim, head_size, kv_mul;
    float *x, *xb, *xb2, *hb, *hb2, *q, *krow, *vrow;
    void **kc, **vc;           /* per layer [max_pos, kv_dim] f32 or f16 */
    int rope_variant;          /* 0 Original (Llama), 1 NeoX (Qwen2): crates/inferi/src/models/llama2/mod.rs:24-29 */
    const float **bias;        /* [n_layers * 3] optional q / k / v biases (transformer.rs:181-183) */
} orc_llama;

/* crates/inferi/src/models/llama2/cpu.rs:110-141 (derived sizes) and transformer.rs:46-137 (state). */
orc_llama *orc_llama_create(const orc_llama_config *c, int kv_f16, int nthreads) {
    orc_llama *m = (orc_llama *)calloc(1, sizeof *m);
    m->c = *c; m->kv_f16 = kv_f16; m->nthreads = nthreads > 0 ? nthreads : 1;
    m->kv_dim = c->hidden * c->n_kv_heads / c->n_heads;
    m->head_size = c->hidden / c->n_heads;
    m->kv_mul = c->n_heads / c->n_kv_heads;
    m->mats = (orc_qmat *)calloc((size_t)c->n_layers * ORC_W_PER_LAYER, sizeof(orc_qmat));
    m->attn_norm = (const float **)calloc(c->n_layers, sizeof(float *));
    m->ffn_norm = (const float **)calloc(c->n_layers, sizeof(float *));
    m->x = (float *)calloc(c->hidden, 4); m->xb = (float *)calloc(c->hidden, 4); m->xb2 = (float *)calloc(c->hidden, 4);
    m->hb = (float *)calloc(c->ffn, 4); m->hb2 = (float *)calloc(c->ffn, 4); m->q = (float *)calloc(c->hidden, 4);
    m->krow = (float *)calloc(m->kv_dim, 4); m->vrow = (float *)calloc(m->kv_dim, 4);
    m->bias = (const float **)calloc((size_t)c->n_layers * 3, sizeof(float *));
    m->kc = (void **)calloc(c->n_layers, sizeof(void *)); m->vc = (void **)calloc(c->n_layers, sizeof(void *));
    size_t esz = kv_f16 ? 2 : 4;
    for (uint32_t l = 0; l < c->n_layers; l++) {
        m->kc[l] = calloc((size_t)c->max_pos * m->kv_dim, esz);
        m->vc[l] = calloc((size_t)c->max_pos * m->kv_dim, esz);
    }
    return m;
}

void orc_llama_set_mat(orc_llama *m, uint32_t layer, int which, int qtype, const void *data) {
    m->mats[(size_t)layer * ORC_W_PER_LAYER + which].qtype = qtype;
    m->mats[(size_t)layer * ORC_W_PER_LAYER + which].data = data;
}
void orc_llama_set_norms(orc_llama *m, uint32_t layer, const float *attn_norm, const float *ffn_norm) {
    m->attn_norm[layer] = attn_norm; m->ffn_norm[layer] = ffn_norm;
}
/* Qwen2 variant: NeoX rotation and q / k / v biases (any of them may be NULL). */
void orc_llama_set_variant(orc_llama *m, int rope_variant) { m->rope_variant = rope_variant; }
void orc_llama_set_bias(orc_llama *m, uint32_t layer, const float *q_bias, const float *k_bias, const float *v_bias) {
    m->bias[(size_t)layer * 3 + 0] = q_bias; m->bias[(size_t)layer * 3 + 1] = k_bias; m->bias[(size_t)layer * 3 + 2] = v_bias;
}
/* output.data == NULL ties the classifier to token_embd (transformer.rs:376-382). */
void orc_llama_set_globals(orc_llama *m, int embd_qtype, const void *embd, int out_qtype, const void *output, const float *output_norm) {
    m->token_embd.qtype = embd_qtype; m->token_embd.data = embd;
    if (output) { m->output.qtype = out_qtype; m->output.data = output; } else m->output = m->token_embd;
    m->output_norm = output_norm;
}

void orc_llama_free(orc_llama *m) {
    if (!m) return;
    for (uint32_t l = 0; l < m->c.n_layers; l++) { free(m->kc[l]); free(m->vc[l]); }
    free(m->kc); free(m->vc); free(m->mats); free(m->attn_norm); free(m->ffn_norm); free(m->bias);
    free(m->x); free(m->xb); free(m->xb2); free(m->hb); free(m->hb2); free(m->q); free(m->krow); free(m->vrow);
    free(m);
}

static void model_gemv(const orc_llama *m, const orc_qmat *w, size_t rows, size_t cols, const float *v, float *out) {
    if (m->gemv_mode == 1 && orc_gemv_shader(w->qtype, rows, cols, w->data, v, out, m->nthreads) == 0) return;
    orc_gemv_ref(w->qtype, rows, cols, w->data, v, out, m->nthreads);
}

/* mode 1 runs every GEMV through the lane-structured shader restatement (the timed CPU baseline). */
void orc_llama_set_gemv_mode(orc_llama *m, int mode) { m->gemv_mode = mode; }

/* One token through the decoder; logits may be NULL.  The current hidden state stays in m->x. */
void orc_llama_forward(orc_llama *m, uint32_t token, uint32_t pos, float *logits) {
    const orc_llama_config *c = &m->c;
    size_t H = c->hidden, F = c->ffn, KV = m->kv_dim;
    /* embedding = dequantized row of token_embd (transformer.rs:367-374) */
    {
        const orc_qmat *e = &m->token_embd;
        size_t rb = row_bytes(e->qtype, H);
        orc_dequantize(e->qtype, (const uint8_t *)e->data + (size_t)token * rb, H / orc_block_elems(e->qtype), m->x);
    }
    orc_attn_params ap = { c->max_pos, (uint32_t)KV, m->kv_mul, c->n_heads, m->head_size, pos };
    for (uint32_t l = 0; l < c->n_layers; l++) {
        const orc_qmat *w = m->mats + (size_t)l * ORC_W_PER_LAYER;
        orc_rms_norm(m->xb, m->x, m->attn_norm[l], H, c->rms_eps);
        model_gemv(m, &w[ORC_W_Q], H, H, m->xb, m->q);
        model_gemv(m, &w[ORC_W_K], KV, H, m->xb, m->krow);
        model_gemv(m, &w[ORC_W_V], KV, H, m->xb, m->vrow);
        /* biases before the rotation: transformer.rs:434-442 */
        if (m->bias[(size_t)l * 3 + 0]) orc_add_assign(m->q, m->bias[(size_t)l * 3 + 0], H);
        if (m->bias[(size_t)l * 3 + 1]) orc_add_assign(m->krow, m->bias[(size_t)l * 3 + 1], KV);
        if (m->bias[(size_t)l * 3 + 2]) orc_add_assign(m->vrow, m->bias[(size_t)l * 3 + 2], KV);
        orc_rope(m->rope_variant, m->q, H, m->krow, KV, m->head_size, pos, c->rope_theta);
        if (m->kv_f16) {
            uint16_t *kr = (uint16_t *)m->kc[l] + (size_t)pos * KV, *vr = (uint16_t *)m->vc[l] + (size_t)pos * KV;
            for (size_t i = 0; i < KV; i++) { kr[i] = orc_encode_f16(m->krow[i]); vr[i] = orc_encode_f16(m->vrow[i]); }
        } else {
            memcpy((float *)m->kc[l] + (size_t)pos * KV, m->krow, KV * 4);
            memcpy((float *)m->vc[l] + (size_t)pos * KV, m->vrow, KV * 4);
        }
        orc_attention(&ap, m->q, m->kc[l], m->vc[l], m->kv_f16, m->xb);
        model_gemv(m, &w[ORC_W_O], H, H, m->xb, m->xb2);
        orc_add_assign(m->x, m->xb2, H);
        orc_rms_norm(m->xb, m->x, m->ffn_norm[l], H, c->rms_eps);
        model_gemv(m, &w[ORC_W_GATE], F, H, m->xb, m->hb);
        model_gemv(m, &w[ORC_W_UP], F, H, m->xb, m->hb2);
        orc_silu_mul(m->hb, m->hb2, F);
        model_gemv(m, &w[ORC_W_DOWN], H, F, m->hb, m->xb2);
        orc_add_assign(m->x, m->xb2, H);
    }
    if (logits) {
        orc_rms_norm(m->xb, m->x, m->output_norm, H, c->rms_eps);
        model_gemv(m, &m->output, c->vocab, H, m->xb, logits);
    }
}

const float *orc_llama_hidden(const orc_llama *m) { return m->x; }

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
