/*
 * pmoe_oracle.c -- CPU restatement of paramecia's quantised MoE FFN block.
 *
 * TEST INFRASTRUCTURE ONLY (see pmoe_oracle.h).  PARITY UNPINNED against the
 * Rust reference: it cannot be built here and holds no golden vectors for this
 * path; the codecs are pinned against gguf-py instead.
 *
 * Every function names the reference code it follows, by the file's path inside
 * nicksenger/paramecia, or the candle routine (candle-core 0.9.2-alpha.2,
 * quantized/k_quants.rs) whose published algorithm it restates.
 *
 * Build with -ffp-contract=off: the restatement relies on products and sums
 * being rounded separately unless fmaf() is written out.
 */
#include "pmoe_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <stddef.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QK_K 256
#define QK8_0 32

/* ------------------------------------------------------------------ f16 */

static inline float f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* round-to-nearest-even, like half::f16::from_f32 */
static inline uint16_t f32_to_f16(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x200u : 0));
    }
    if (ax >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (ax < 0x38800000u) { /* subnormal or zero in f16 */
        if (ax < 0x33000000u) return (uint16_t)sign; /* < 2^-25 -> 0 */
        int e = (int)(ax >> 23);
        uint32_t man = (ax & 0x7fffffu) | 0x800000u;
        int shift = 126 - e; /* 14..24 */
        uint32_t r = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (r & 1))) r++;
        return (uint16_t)(sign | r);
    }
    uint32_t e = (ax >> 23) - 112;
    uint32_t man = ax & 0x7fffffu;
    uint32_t r = (e << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) r++;
    return (uint16_t)(sign | r);
}

/* ------------------------------------------------------------------ blocks */

#pragma pack(push, 1)
typedef struct { uint16_t d; int8_t qs[QK8_0]; } block_q8_0;                      /* 34 B  */
typedef struct { uint8_t scales[QK_K / 16]; uint8_t qs[QK_K / 4]; uint16_t d, dmin; } block_q2_K;       /* 84 B  */
typedef struct { uint8_t hmask[QK_K / 8]; uint8_t qs[QK_K / 4]; uint8_t scales[12]; uint16_t d; } block_q3_K; /* 110 B */
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qs[QK_K / 2]; } block_q4_K; /* 144 B */
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qh[QK_K / 8]; uint8_t qs[QK_K / 2]; } block_q5_K; /* 176 B */
typedef struct { uint8_t ql[QK_K / 2]; uint8_t qh[QK_K / 4]; int8_t scales[QK_K / 16]; uint16_t d; } block_q6_K; /* 210 B */
#pragma pack(pop)
typedef struct { float d; int8_t qs[QK_K]; int16_t bsums[QK_K / 16]; } block_q8_K; /* activation block */

size_t pmo_block_size(int dtype)
{
    switch (dtype) {
    case PMO_F32: case PMO_F16: return 1;
    case PMO_Q8_0: return QK8_0;
    case PMO_Q2_K: case PMO_Q3_K: case PMO_Q4_K: case PMO_Q5_K: case PMO_Q6_K: return QK_K;
    default: return 0;
    }
}

size_t pmo_type_size(int dtype)
{
    switch (dtype) {
    case PMO_F32: return 4;
    case PMO_F16: return 2;
    case PMO_Q8_0: return sizeof(block_q8_0);
    case PMO_Q2_K: return sizeof(block_q2_K);
    case PMO_Q3_K: return sizeof(block_q3_K);
    case PMO_Q4_K: return sizeof(block_q4_K);
    case PMO_Q5_K: return sizeof(block_q5_K);
    case PMO_Q6_K: return sizeof(block_q6_K);
    default: return 0;
    }
}

size_t pmo_row_bytes(int dtype, size_t cols)
{
    size_t bs = pmo_block_size(dtype);
    if (!bs || cols % bs) return 0;
    return cols / bs * pmo_type_size(dtype);
}

/* 6-bit scale/min pair j of a Q4_K block (ggml get_scale_min_k4) */
static inline void q4k_scale_min(int j, const uint8_t *q, uint8_t *sc, uint8_t *m)
{
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* ------------------------------------------------------------------ dequantise
 * GGUF block formats as candle's GgmlType::to_float for BlockQ4K / BlockQ6K /
 * BlockQ8_0 decodes them; d*sc and dmin*m are rounded to f32 before use. */

static void dequant_q8_0(const block_q8_0 *b, size_t nb, float *y)
{
    for (size_t i = 0; i < nb; i++) {
        float d = f16_to_f32(b[i].d);
        for (int j = 0; j < QK8_0; j++) y[i * QK8_0 + j] = (float)b[i].qs[j] * d;
    }
}

/* BlockQ2K::to_float (ggml dequantize_row_q2_K): 16 sub-blocks of 16, 4-bit scale and 4-bit min each */
static void dequant_q2_K(const block_q2_K *b, size_t nb, float *y)
{
    for (size_t i = 0; i < nb; i++) {
        float d = f16_to_f32(b[i].d);
        float min = f16_to_f32(b[i].dmin);
        const uint8_t *q = b[i].qs;
        int is = 0;
        for (int n = 0; n < QK_K; n += 128) {
            int shift = 0;
            for (int j = 0; j < 4; j++) {
                uint8_t sc = b[i].scales[is++];
                float dl = d * (float)(sc & 0xF), ml = min * (float)(sc >> 4);
                for (int l = 0; l < 16; l++) *y++ = dl * (float)((int8_t)((q[l] >> shift) & 3)) - ml;
                sc = b[i].scales[is++];
                dl = d * (float)(sc & 0xF);
                ml = min * (float)(sc >> 4);
                for (int l = 0; l < 16; l++) *y++ = dl * (float)((int8_t)((q[l + 16] >> shift) & 3)) - ml;
                shift += 2;
            }
            q += 32;
        }
    }
}

/* the 16 six-bit scales of a Q3_K block (ggml's kmask unpacking), still offset by 32 */
static void q3k_scales(const uint8_t *packed, int8_t *out)
{
    const uint32_t kmask1 = 0x03030303u, kmask2 = 0x0f0f0f0fu;
    uint32_t aux[4];
    memcpy(aux, packed, 12);
    uint32_t tmp = aux[2];
    aux[2] = ((aux[0] >> 4) & kmask2) | (((tmp >> 4) & kmask1) << 4);
    aux[3] = ((aux[1] >> 4) & kmask2) | (((tmp >> 6) & kmask1) << 4);
    aux[0] = (aux[0] & kmask2) | (((tmp >> 0) & kmask1) << 4);
    aux[1] = (aux[1] & kmask2) | (((tmp >> 2) & kmask1) << 4);
    memcpy(out, aux, 16);
}

/* BlockQ3K::to_float (ggml dequantize_row_q3_K): 2 low bits in qs, the third in hmask (clear = -4) */
static void dequant_q3_K(const block_q3_K *b, size_t nb, float *y)
{
    for (size_t i = 0; i < nb; i++) {
        float d_all = f16_to_f32(b[i].d);
        const uint8_t *q = b[i].qs;
        const uint8_t *hm = b[i].hmask;
        uint8_t m = 1;
        int8_t scales[16];
        q3k_scales(b[i].scales, scales);
        int is = 0;
        for (int n = 0; n < QK_K; n += 128) {
            int shift = 0;
            for (int j = 0; j < 4; j++) {
                float dl = d_all * (float)(scales[is++] - 32);
                for (int l = 0; l < 16; l++)
                    *y++ = dl * (float)((int8_t)((q[l] >> shift) & 3) - ((hm[l] & m) ? 0 : 4));
                dl = d_all * (float)(scales[is++] - 32);
                for (int l = 0; l < 16; l++)
                    *y++ = dl * (float)((int8_t)((q[l + 16] >> shift) & 3) - ((hm[l + 16] & m) ? 0 : 4));
                shift += 2;
                m = (uint8_t)(m << 1);
            }
            q += 32;
        }
    }
}

static void dequant_q4_K(const block_q4_K *b, size_t nb, float *y)
{
    for (size_t i = 0; i < nb; i++) {
        const uint8_t *q = b[i].qs;
        float d = f16_to_f32(b[i].d);
        float min = f16_to_f32(b[i].dmin);
        int is = 0;
        for (int j = 0; j < QK_K; j += 64) {
            uint8_t sc, m;
            q4k_scale_min(is, b[i].scales, &sc, &m);
            float d1 = d * sc, m1 = min * m;
            q4k_scale_min(is + 1, b[i].scales, &sc, &m);
            float d2 = d * sc, m2 = min * m;
            for (int l = 0; l < 32; l++) *y++ = d1 * (float)(q[l] & 0xF) - m1;
            for (int l = 0; l < 32; l++) *y++ = d2 * (float)(q[l] >> 4) - m2;
            q += 32;
            is += 2;
        }
    }
}

/* BlockQ5K::to_float (ggml dequantize_row_q5_K): the fifth bit of the two sub-blocks of 64-group
 * j sits in bits 2j and 2j+1 of qh[l] */
static void dequant_q5_K(const block_q5_K *b, size_t nb, float *y)
{
    for (size_t i = 0; i < nb; i++) {
        const uint8_t *ql = b[i].qs;
        const uint8_t *qh = b[i].qh;
        float d = f16_to_f32(b[i].d);
        float min = f16_to_f32(b[i].dmin);
        int is = 0;
        uint8_t u1 = 1, u2 = 2;
        for (int j = 0; j < QK_K; j += 64) {
            uint8_t sc, m;
            q4k_scale_min(is, b[i].scales, &sc, &m);
            float d1 = d * sc, m1 = min * m;
            q4k_scale_min(is + 1, b[i].scales, &sc, &m);
            float d2 = d * sc, m2 = min * m;
            for (int l = 0; l < 32; l++) *y++ = d1 * (float)((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - m1;
            for (int l = 0; l < 32; l++) *y++ = d2 * (float)((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
            ql += 32;
            is += 2;
            u1 = (uint8_t)(u1 << 2);
            u2 = (uint8_t)(u2 << 2);
        }
    }
}

static void dequant_q6_K(const block_q6_K *b, size_t nb, float *y)
{
    for (size_t i = 0; i < nb; i++) {
        float d = f16_to_f32(b[i].d);
        const uint8_t *ql = b[i].ql;
        const uint8_t *qh = b[i].qh;
        const int8_t *sc = b[i].scales;
        for (int n = 0; n < QK_K; n += 128) {
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                y[l + 0] = d * (float)sc[is + 0] * (float)q1;
                y[l + 32] = d * (float)sc[is + 2] * (float)q2;
                y[l + 64] = d * (float)sc[is + 4] * (float)q3;
                y[l + 96] = d * (float)sc[is + 6] * (float)q4;
            }
            y += 128;
            ql += 64;
            qh += 32;
            sc += 8;
        }
    }
}

int pmo_dequantize(int dtype, const void *blocks, size_t n, float *out)
{
    size_t bs = pmo_block_size(dtype);
    if (!bs || n % bs) return -1;
    switch (dtype) {
    case PMO_F32: memcpy(out, blocks, n * 4); return 0;
    case PMO_F16: for (size_t i = 0; i < n; i++) out[i] = f16_to_f32(((const uint16_t *)blocks)[i]); return 0;
    case PMO_Q8_0: dequant_q8_0((const block_q8_0 *)blocks, n / bs, out); return 0;
    case PMO_Q2_K: dequant_q2_K((const block_q2_K *)blocks, n / bs, out); return 0;
    case PMO_Q3_K: dequant_q3_K((const block_q3_K *)blocks, n / bs, out); return 0;
    case PMO_Q4_K: dequant_q4_K((const block_q4_K *)blocks, n / bs, out); return 0;
    case PMO_Q5_K: dequant_q5_K((const block_q5_K *)blocks, n / bs, out); return 0;
    case PMO_Q6_K: dequant_q6_K((const block_q6_K *)blocks, n / bs, out); return 0;
    }
    return -1;
}

/* ------------------------------------------------------------------ weight quantisers
 * Used only to make synthetic GGUF blocks from seeded normal weights.  Q8_0 is
 * the ggml/candle reference quantiser.  The K-quant quantisers (Q2_K ... Q6_K) are plain
 * min/max quantisers of this build (not ggml's error-minimising search): any
 * valid quantiser serves, since oracle and library consume the same bytes. */

static void quant_q8_0(const float *x, size_t nb, block_q8_0 *y)
{
    for (size_t i = 0; i < nb; i++) {
        float amax = 0.f;
        for (int j = 0; j < QK8_0; j++) amax = fmaxf(amax, fabsf(x[i * QK8_0 + j]));
        float d = amax / 127.f;
        float id = d != 0.f ? 1.f / d : 0.f;
        y[i].d = f32_to_f16(d);
        for (int j = 0; j < QK8_0; j++) y[i].qs[j] = (int8_t)roundf(x[i * QK8_0 + j] * id);
    }
}

/* element e of a Q2_K / Q3_K block lives in byte 32*(e/128) + e%32 of qs at bit 2*((e%128)/32) */
static inline void q23_set(uint8_t *qs, int e, int q2)
{
    qs[32 * (e / 128) + (e % 32)] |= (uint8_t)((q2 & 3) << (2 * ((e % 128) / 32)));
}

/* min/max quantiser: 16 sub-blocks of 16, scale = range/3 and min on 4 bits each */
static void quant_q2_K(const float *x, size_t nb, block_q2_K *y)
{
    for (size_t i = 0; i < nb; i++) {
        const float *xb = x + i * QK_K;
        float scales[16], mins[16], max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 16; j++) {
            float mn = 0.f, mx = 0.f;
            for (int l = 0; l < 16; l++) {
                mn = fminf(mn, xb[16 * j + l]);
                mx = fmaxf(mx, xb[16 * j + l]);
            }
            scales[j] = (mx - mn) / 3.f;
            mins[j] = -mn;
            max_scale = fmaxf(max_scale, scales[j]);
            max_min = fmaxf(max_min, mins[j]);
        }
        float inv_scale = max_scale > 0.f ? 15.f / max_scale : 0.f;
        float inv_min = max_min > 0.f ? 15.f / max_min : 0.f;
        y[i].d = f32_to_f16(max_scale / 15.f);
        y[i].dmin = f32_to_f16(max_min / 15.f);
        float d = f16_to_f32(y[i].d), dmin = f16_to_f32(y[i].dmin);
        memset(y[i].qs, 0, sizeof y[i].qs);
        for (int j = 0; j < 16; j++) {
            int ls = (int)roundf(inv_scale * scales[j]), lm = (int)roundf(inv_min * mins[j]);
            ls = ls > 15 ? 15 : ls;
            lm = lm > 15 ? 15 : lm;
            y[i].scales[j] = (uint8_t)(ls | (lm << 4));
            float dq = d * (float)ls, mq = dmin * (float)lm;
            for (int l = 0; l < 16; l++) {
                int q = 0;
                if (dq > 0.f) {
                    q = (int)roundf((xb[16 * j + l] + mq) / dq);
                    q = q < 0 ? 0 : (q > 3 ? 3 : q);
                }
                q23_set(y[i].qs, 16 * j + l, q);
            }
        }
    }
}

/* symmetric quantiser: 16 sub-blocks of 16, signed 6-bit scale, quants in [-4, 3] */
static void quant_q3_K(const float *x, size_t nb, block_q3_K *y)
{
    for (size_t i = 0; i < nb; i++) {
        const float *xb = x + i * QK_K;
        float scales[16], max_scale = 0.f;
        for (int j = 0; j < 16; j++) {
            float amax = 0.f;
            for (int l = 0; l < 16; l++) amax = fmaxf(amax, fabsf(xb[16 * j + l]));
            scales[j] = amax / 4.f;
            max_scale = fmaxf(max_scale, scales[j]);
        }
        float inv = max_scale > 0.f ? 31.f / max_scale : 0.f;
        y[i].d = f32_to_f16(max_scale / 31.f);
        float d = f16_to_f32(y[i].d);
        memset(y[i].qs, 0, sizeof y[i].qs);
        memset(y[i].hmask, 0, sizeof y[i].hmask);
        memset(y[i].scales, 0, sizeof y[i].scales);
        for (int j = 0; j < 16; j++) {
            int s = (int)roundf(inv * scales[j]);
            s = s > 31 ? 31 : s;
            int l6 = s + 32; /* stored with an offset of 32 */
            /* low 4 bits: nibble j%8 half j/8 of scales[0..7]; high 2 bits: scales[8 + j%4] at bit 2*(j/4) */
            if (j < 8) y[i].scales[j] |= (uint8_t)(l6 & 0xF);
            else y[i].scales[j - 8] |= (uint8_t)((l6 & 0xF) << 4);
            y[i].scales[8 + j % 4] |= (uint8_t)((l6 >> 4) << (2 * (j / 4)));
            float dq = d * (float)s;
            for (int l = 0; l < 16; l++) {
                int e = 16 * j + l;
                int q = 0;
                if (dq > 0.f) {
                    q = (int)roundf(xb[e] / dq);
                    q = q < -4 ? -4 : (q > 3 ? 3 : q);
                }
                int u = q + 4; /* 0..7: two low bits in qs, the third in hmask */
                q23_set(y[i].qs, e, u & 3);
                if (u & 4) y[i].hmask[e % 32] |= (uint8_t)(1 << (4 * (e / 128) + (e % 128) / 32));
            }
        }
    }
}

static void quant_q4_K(const float *x, size_t nb, block_q4_K *y)
{
    for (size_t i = 0; i < nb; i++) {
        const float *xb = x + i * QK_K;
        float scales[8], mins[8];
        float max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 8; j++) {
            float mn = 0.f, mx = 0.f;
            for (int l = 0; l < 32; l++) {
                mn = fminf(mn, xb[32 * j + l]);
                mx = fmaxf(mx, xb[32 * j + l]);
            }
            scales[j] = (mx - mn) / 15.f;
            mins[j] = -mn;
            max_scale = fmaxf(max_scale, scales[j]);
            max_min = fmaxf(max_min, mins[j]);
        }
        float inv_scale = max_scale > 0.f ? 63.f / max_scale : 0.f;
        float inv_min = max_min > 0.f ? 63.f / max_min : 0.f;
        uint8_t ls[8], lm[8];
        for (int j = 0; j < 8; j++) {
            int a = (int)roundf(inv_scale * scales[j]);
            int b = (int)roundf(inv_min * mins[j]);
            ls[j] = (uint8_t)(a > 63 ? 63 : a);
            lm[j] = (uint8_t)(b > 63 ? 63 : b);
        }
        y[i].d = f32_to_f16(max_scale / 63.f);
        y[i].dmin = f32_to_f16(max_min / 63.f);
        for (int j = 0; j < 4; j++) {
            y[i].scales[j] = (uint8_t)(ls[j] | ((ls[j + 4] >> 4) << 6));
            y[i].scales[j + 4] = (uint8_t)(lm[j] | ((lm[j + 4] >> 4) << 6));
            y[i].scales[j + 8] = (uint8_t)((ls[j + 4] & 0xF) | ((lm[j + 4] & 0xF) << 4));
        }
        float d = f16_to_f32(y[i].d), dmin = f16_to_f32(y[i].dmin);
        uint8_t L[QK_K];
        for (int j = 0; j < 8; j++) {
            float dq = d * (float)ls[j];
            float mq = dmin * (float)lm[j];
            for (int l = 0; l < 32; l++) {
                int q = 0;
                if (dq > 0.f) {
                    q = (int)roundf((xb[32 * j + l] + mq) / dq);
                    q = q < 0 ? 0 : (q > 15 ? 15 : q);
                }
                L[32 * j + l] = (uint8_t)q;
            }
        }
        for (int g = 0; g < 4; g++)
            for (int l = 0; l < 32; l++)
                y[i].qs[32 * g + l] = (uint8_t)(L[64 * g + l] | (L[64 * g + 32 + l] << 4));
    }
}

/* the Q4_K min/max quantiser with 32 levels */
static void quant_q5_K(const float *x, size_t nb, block_q5_K *y)
{
    for (size_t i = 0; i < nb; i++) {
        const float *xb = x + i * QK_K;
        float scales[8], mins[8];
        float max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 8; j++) {
            float mn = 0.f, mx = 0.f;
            for (int l = 0; l < 32; l++) {
                mn = fminf(mn, xb[32 * j + l]);
                mx = fmaxf(mx, xb[32 * j + l]);
            }
            scales[j] = (mx - mn) / 31.f;
            mins[j] = -mn;
            max_scale = fmaxf(max_scale, scales[j]);
            max_min = fmaxf(max_min, mins[j]);
        }
        float inv_scale = max_scale > 0.f ? 63.f / max_scale : 0.f;
        float inv_min = max_min > 0.f ? 63.f / max_min : 0.f;
        uint8_t ls[8], lm[8];
        for (int j = 0; j < 8; j++) {
            int a = (int)roundf(inv_scale * scales[j]);
            int b = (int)roundf(inv_min * mins[j]);
            ls[j] = (uint8_t)(a > 63 ? 63 : a);
            lm[j] = (uint8_t)(b > 63 ? 63 : b);
        }
        y[i].d = f32_to_f16(max_scale / 63.f);
        y[i].dmin = f32_to_f16(max_min / 63.f);
        for (int j = 0; j < 4; j++) {
            y[i].scales[j] = (uint8_t)(ls[j] | ((ls[j + 4] >> 4) << 6));
            y[i].scales[j + 4] = (uint8_t)(lm[j] | ((lm[j + 4] >> 4) << 6));
            y[i].scales[j + 8] = (uint8_t)((ls[j + 4] & 0xF) | ((lm[j + 4] & 0xF) << 4));
        }
        float d = f16_to_f32(y[i].d), dmin = f16_to_f32(y[i].dmin);
        uint8_t L[QK_K];
        for (int j = 0; j < 8; j++) {
            float dq = d * (float)ls[j];
            float mq = dmin * (float)lm[j];
            for (int l = 0; l < 32; l++) {
                int q = 0;
                if (dq > 0.f) {
                    q = (int)roundf((xb[32 * j + l] + mq) / dq);
                    q = q < 0 ? 0 : (q > 31 ? 31 : q);
                }
                L[32 * j + l] = (uint8_t)q;
            }
        }
        memset(y[i].qh, 0, sizeof(y[i].qh));
        for (int g = 0; g < 4; g++)
            for (int l = 0; l < 32; l++) {
                uint8_t a = L[64 * g + l], b = L[64 * g + 32 + l];
                y[i].qs[32 * g + l] = (uint8_t)((a & 0xF) | ((b & 0xF) << 4));
                y[i].qh[l] = (uint8_t)(y[i].qh[l] | ((a >> 4) << (2 * g)) | ((b >> 4) << (2 * g + 1)));
            }
    }
}

static void quant_q6_K(const float *x, size_t nb, block_q6_K *y)
{
    for (size_t i = 0; i < nb; i++) {
        const float *xb = x + i * QK_K;
        float scales[16];
        float max_scale = 0.f;
        for (int j = 0; j < 16; j++) {
            float amax = 0.f;
            for (int l = 0; l < 16; l++) amax = fmaxf(amax, fabsf(xb[16 * j + l]));
            scales[j] = amax / 31.f;
            max_scale = fmaxf(max_scale, scales[j]);
        }
        float inv = max_scale > 0.f ? 127.f / max_scale : 0.f;
        y[i].d = f32_to_f16(max_scale / 127.f);
        float d = f16_to_f32(y[i].d);
        uint8_t L[QK_K];
        for (int j = 0; j < 16; j++) {
            int s = (int)roundf(inv * scales[j]);
            s = s > 127 ? 127 : s;
            y[i].scales[j] = (int8_t)s;
            float dq = d * (float)s;
            for (int l = 0; l < 16; l++) {
                int q = 0;
                if (dq > 0.f) {
                    q = (int)roundf(xb[16 * j + l] / dq);
                    q = q < -32 ? -32 : (q > 31 ? 31 : q);
                }
                L[16 * j + l] = (uint8_t)(q + 32);
            }
        }
        for (int n = 0; n < 2; n++) {
            for (int l = 0; l < 32; l++) {
                uint8_t q1 = L[128 * n + l], q2 = L[128 * n + l + 32];
                uint8_t q3 = L[128 * n + l + 64], q4 = L[128 * n + l + 96];
                y[i].ql[64 * n + l] = (uint8_t)((q1 & 0xF) | ((q3 & 0xF) << 4));
                y[i].ql[64 * n + l + 32] = (uint8_t)((q2 & 0xF) | ((q4 & 0xF) << 4));
                y[i].qh[32 * n + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
            }
        }
    }
}

/* ------------------------------------------------------------------ block-scale multipliers
 * QTensor::modify_block_scales as the reference's training mode calls it
 * (paramecia-model/src/qwen3_next.rs:1604-1606 for the routed experts, one f32 multiplier per
 * block of the [E, rows, cols] tensor, expert e taking blocks [e*B, (e+1)*B) -- extract_expert_scales,
 * 1688-1703; models/with_tracing.rs:217-248 for a single QMatMul).  The routine itself lives in the
 * candle fork, which is not part of the reference tree [UNVERIFIED]: restated here as "the block's
 * dequantised values are multiplied by m", i.e. every f16 super-scale of the block (d, and dmin
 * where the type has one) becomes f16(f32(scale) * m), rounded to nearest even like half::f16::from_f32;
 * quants and the packed 6-bit / 4-bit sub-scales are copied unchanged. */
int pmo_modify_block_scales(int dtype, const void *blocks, size_t n_blocks, const float *mults, void *out)
{
    const size_t ts = pmo_type_size(dtype);
    if (dtype != PMO_Q8_0 && !(dtype >= PMO_Q2_K && dtype <= PMO_Q6_K)) return -1;
    if (out != blocks) memcpy(out, blocks, n_blocks * ts);
    for (size_t i = 0; i < n_blocks; i++) {
        uint8_t *b = (uint8_t *)out + i * ts;
        const float m = mults[i];
        size_t d_off = 0, dmin_off = (size_t)-1;
        switch (dtype) {
        case PMO_Q8_0: d_off = offsetof(block_q8_0, d); break;
        case PMO_Q2_K: d_off = offsetof(block_q2_K, d); dmin_off = offsetof(block_q2_K, dmin); break;
        case PMO_Q3_K: d_off = offsetof(block_q3_K, d); break;
        case PMO_Q4_K: d_off = offsetof(block_q4_K, d); dmin_off = offsetof(block_q4_K, dmin); break;
        case PMO_Q5_K: d_off = offsetof(block_q5_K, d); dmin_off = offsetof(block_q5_K, dmin); break;
        case PMO_Q6_K: d_off = offsetof(block_q6_K, d); break;
        }
        uint16_t h;
        memcpy(&h, b + d_off, 2);
        h = f32_to_f16(f16_to_f32(h) * m);
        memcpy(b + d_off, &h, 2);
        if (dmin_off != (size_t)-1) {
            memcpy(&h, b + dmin_off, 2);
            h = f32_to_f16(f16_to_f32(h) * m);
            memcpy(b + dmin_off, &h, 2);
        }
    }
    return 0;
}

int pmo_quantize(int dtype, const float *x, size_t n, void *blocks)
{
    size_t bs = pmo_block_size(dtype);
    if (!bs || n % bs) return -1;
    size_t nb = n / bs;
    size_t chunk = 4096;
    if (dtype == PMO_F32) { memcpy(blocks, x, n * 4); return 0; }
    if (dtype == PMO_F16) { for (size_t i = 0; i < n; i++) ((uint16_t *)blocks)[i] = f32_to_f16(x[i]); return 0; }
    if (dtype != PMO_Q8_0 && dtype != PMO_Q2_K && dtype != PMO_Q3_K && dtype != PMO_Q4_K && dtype != PMO_Q5_K &&
        dtype != PMO_Q6_K)
        return -1;
#pragma omp parallel for schedule(static)
    for (size_t b0 = 0; b0 < nb; b0 += chunk) {
        size_t cnt = nb - b0 < chunk ? nb - b0 : chunk;
        if (dtype == PMO_Q8_0) quant_q8_0(x + b0 * bs, cnt, (block_q8_0 *)blocks + b0);
        else if (dtype == PMO_Q2_K) quant_q2_K(x + b0 * bs, cnt, (block_q2_K *)blocks + b0);
        else if (dtype == PMO_Q3_K) quant_q3_K(x + b0 * bs, cnt, (block_q3_K *)blocks + b0);
        else if (dtype == PMO_Q4_K) quant_q4_K(x + b0 * bs, cnt, (block_q4_K *)blocks + b0);
        else if (dtype == PMO_Q5_K) quant_q5_K(x + b0 * bs, cnt, (block_q5_K *)blocks + b0);
        else quant_q6_K(x + b0 * bs, cnt, (block_q6_K *)blocks + b0);
    }
    return 0;
}

/* ------------------------------------------------------------------ activation quantisers */

/* candle BlockQ8K::from_float: the element of largest magnitude keeps its sign,
 * iscale = -128/max, q = min(127, round_half_away(iscale*x)), d = 1/iscale,
 * bsums = sums of 16 consecutive quants; an all-zero block gives d = 0. */
static void quantize_row_q8_K(const float *x, size_t n, block_q8_K *y)
{
    for (size_t i = 0; i < n / QK_K; i++) {
        const float *xs = x + i * QK_K;
        float max = 0.f, amax = 0.f;
        for (int j = 0; j < QK_K; j++) {
            if (amax < fabsf(xs[j])) { amax = fabsf(xs[j]); max = xs[j]; }
        }
        if (amax == 0.f) {
            y[i].d = 0.f;
            memset(y[i].qs, 0, sizeof y[i].qs);
            memset(y[i].bsums, 0, sizeof y[i].bsums);
            continue;
        }
        float iscale = -128.f / max;
        for (int j = 0; j < QK_K; j++) {
            float v = roundf(iscale * xs[j]);
            y[i].qs[j] = (int8_t)(v < 127.f ? v : 127.f);
        }
        for (int j = 0; j < QK_K / 16; j++) {
            int sum = 0;
            for (int ii = 0; ii < 16; ii++) sum += y[i].qs[j * 16 + ii];
            y[i].bsums[j] = (int16_t)sum;
        }
        y[i].d = 1.0f / iscale;
    }
}

/* candle BlockQ8_0::from_float: d = amax/127 stored as f16, q = round_half_away(x * (1/d)) */
static void quantize_row_q8_0(const float *x, size_t n, block_q8_0 *y) { quant_q8_0(x, n / QK8_0, y); }

void pmo_quantize_q8k(const float *x, size_t n, float *d, int8_t *qs, int16_t *bsums)
{
    block_q8_K *t = (block_q8_K *)malloc(sizeof(block_q8_K) * (n / QK_K));
    quantize_row_q8_K(x, n, t);
    for (size_t i = 0; i < n / QK_K; i++) {
        d[i] = t[i].d;
        memcpy(qs + i * QK_K, t[i].qs, QK_K);
        memcpy(bsums + i * 16, t[i].bsums, 32);
    }
    free(t);
}

void pmo_quantize_q8_0_act(const float *x, size_t n, uint16_t *d_f16, int8_t *qs)
{
    block_q8_0 *t = (block_q8_0 *)malloc(sizeof(block_q8_0) * (n / QK8_0));
    quantize_row_q8_0(x, n, t);
    for (size_t i = 0; i < n / QK8_0; i++) {
        d_f16[i] = t[i].d;
        memcpy(qs + i * QK8_0, t[i].qs, QK8_0);
    }
    free(t);
}

/* ------------------------------------------------------------------ block dot products
 * candle's portable vec_dot (GgmlType::vec_dot_unopt).  The integer sums are
 * exact; the f32 steps keep the reference's association: eight running f32
 * lanes per row, summed at the end. */

/* BlockQ2K::vec_dot against Q8_K (portable path, ggml_vec_dot_q2_K_q8_K generic) */
static float vec_dot_q2_K_q8_K(size_t n, const block_q2_K *x, const block_q8_K *y)
{
    float sumf = 0.f;
    for (size_t i = 0; i < n / QK_K; i++) {
        const uint8_t *q2 = x[i].qs;
        const int8_t *q8 = y[i].qs;
        const uint8_t *sc = x[i].scales;
        int summs = 0;
        for (int j = 0; j < 16; j++) summs += y[i].bsums[j] * (sc[j] >> 4);
        float dall = y[i].d * f16_to_f32(x[i].d);
        float dmin = y[i].d * f16_to_f32(x[i].dmin);
        int isum = 0, is = 0;
        for (int k = 0; k < QK_K / 128; k++) {
            int shift = 0;
            for (int j = 0; j < 4; j++) {
                int d = sc[is++] & 0xF;
                int isuml = 0;
                for (int l = 0; l < 16; l++) isuml += q8[l] * ((q2[l] >> shift) & 3);
                isum += d * isuml;
                d = sc[is++] & 0xF;
                isuml = 0;
                for (int l = 16; l < 32; l++) isuml += q8[l] * ((q2[l] >> shift) & 3);
                isum += d * isuml;
                shift += 2;
                q8 += 32;
            }
            q2 += 32;
        }
        sumf += dall * (float)isum - dmin * (float)summs;
    }
    return sumf;
}

/* BlockQ3K::vec_dot against Q8_K (portable path): the quants as signed values -4..3, eight f32 lanes */
static float vec_dot_q3_K_q8_K(size_t n, const block_q3_K *x, const block_q8_K *y)
{
    float sums[8] = {0};
    int8_t aux8[QK_K];
    for (size_t i = 0; i < n / QK_K; i++) {
        const uint8_t *q3 = x[i].qs;
        const uint8_t *hm = x[i].hmask;
        int8_t *a = aux8;
        uint8_t m = 1;
        for (int j = 0; j < QK_K; j += 128) {
            for (int sh = 0; sh < 8; sh += 2) {
                for (int l = 0; l < 32; l++) a[l] = (int8_t)((q3[l] >> sh) & 3);
                for (int l = 0; l < 32; l++) a[l] = (int8_t)(a[l] - ((hm[l] & m) ? 0 : 4));
                a += 32;
                m = (uint8_t)(m << 1);
            }
            q3 += 32;
        }
        int8_t scales[16];
        q3k_scales(x[i].scales, scales);
        int32_t aux32[8] = {0};
        const int8_t *q8 = y[i].qs;
        a = aux8;
        for (int j = 0; j < QK_K / 16; j++) {
            int32_t scale = scales[j] - 32;
            for (int r = 0; r < 2; r++) {
                for (int l = 0; l < 8; l++) aux32[l] += scale * ((int32_t)q8[l] * (int32_t)a[l]);
                q8 += 8;
                a += 8;
            }
        }
        float d = f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; l++) sums[l] += d * (float)aux32[l];
    }
    float s = 0.f;
    for (int l = 0; l < 8; l++) s += sums[l];
    return s;
}

static float vec_dot_q4_K_q8_K(size_t n, const block_q4_K *x, const block_q8_K *y)
{
    float sums[8] = {0};
    float sumf = 0.f;
    int8_t aux8[QK_K];
    for (size_t i = 0; i < n / QK_K; i++) {
        const uint8_t *q4 = x[i].qs;
        int8_t *a = aux8;
        for (int j = 0; j < QK_K / 64; j++) {
            for (int l = 0; l < 32; l++) a[l] = (int8_t)(q4[l] & 0xF);
            a += 32;
            for (int l = 0; l < 32; l++) a[l] = (int8_t)(q4[l] >> 4);
            a += 32;
            q4 += 32;
        }
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; j++) q4k_scale_min(j, x[i].scales, &sc[j], &mn[j]);
        int32_t sumi = 0;
        for (int j = 0; j < QK_K / 16; j++) sumi += (int32_t)y[i].bsums[j] * (int32_t)mn[j / 2];
        int32_t aux32[8] = {0};
        const int8_t *q8 = y[i].qs;
        a = aux8;
        for (int j = 0; j < 8; j++) {
            int32_t scale = sc[j];
            for (int r = 0; r < 4; r++) {
                for (int l = 0; l < 8; l++) aux32[l] += scale * ((int32_t)q8[l] * (int32_t)a[l]);
                q8 += 8;
                a += 8;
            }
        }
        float d = f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; l++) sums[l] += d * (float)aux32[l];
        float dmin = f16_to_f32(x[i].dmin) * y[i].d;
        sumf -= dmin * (float)sumi;
    }
    float s = 0.f;
    for (int l = 0; l < 8; l++) s += sums[l];
    return sumf + s;
}

/* BlockQ5K::vec_dot against Q8_K (portable path): as Q4_K with the fifth bit added to each quant */
static float vec_dot_q5_K_q8_K(size_t n, const block_q5_K *x, const block_q8_K *y)
{
    float sums[8] = {0};
    float sumf = 0.f;
    int8_t aux8[QK_K];
    for (size_t i = 0; i < n / QK_K; i++) {
        const uint8_t *q4 = x[i].qs;
        const uint8_t *hm = x[i].qh;
        int8_t *a = aux8;
        uint8_t m = 1;
        for (int j = 0; j < QK_K / 64; j++) {
            for (int l = 0; l < 32; l++) a[l] = (int8_t)((q4[l] & 0xF) + ((hm[l] & m) ? 16 : 0));
            a += 32;
            m = (uint8_t)(m << 1);
            for (int l = 0; l < 32; l++) a[l] = (int8_t)((q4[l] >> 4) + ((hm[l] & m) ? 16 : 0));
            a += 32;
            m = (uint8_t)(m << 1);
            q4 += 32;
        }
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; j++) q4k_scale_min(j, x[i].scales, &sc[j], &mn[j]);
        int32_t sumi = 0;
        for (int j = 0; j < QK_K / 16; j++) sumi += (int32_t)y[i].bsums[j] * (int32_t)mn[j / 2];
        int32_t aux32[8] = {0};
        const int8_t *q8 = y[i].qs;
        a = aux8;
        for (int j = 0; j < 8; j++) {
            int32_t scale = sc[j];
            for (int r = 0; r < 4; r++) {
                for (int l = 0; l < 8; l++) aux32[l] += scale * ((int32_t)q8[l] * (int32_t)a[l]);
                q8 += 8;
                a += 8;
            }
        }
        float d = f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; l++) sums[l] += d * (float)aux32[l];
        float dmin = f16_to_f32(x[i].dmin) * y[i].d;
        sumf -= dmin * (float)sumi;
    }
    float s = 0.f;
    for (int l = 0; l < 8; l++) s += sums[l];
    return sumf + s;
}

static float vec_dot_q6_K_q8_K(size_t n, const block_q6_K *x, const block_q8_K *y)
{
    float sums[8] = {0};
    int8_t aux8[QK_K];
    for (size_t i = 0; i < n / QK_K; i++) {
        const uint8_t *q4 = x[i].ql;
        const uint8_t *qh = x[i].qh;
        int8_t *a = aux8;
        for (int j = 0; j < QK_K; j += 128) {
            for (int l = 0; l < 32; l++) {
                a[l + 0] = (int8_t)((int)((q4[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32);
                a[l + 32] = (int8_t)((int)((q4[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32);
                a[l + 64] = (int8_t)((int)((q4[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
                a[l + 96] = (int8_t)((int)((q4[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
            }
            a += 128;
            q4 += 64;
            qh += 32;
        }
        /* candle keeps these eight lanes in f32; every partial value is an integer
         * below 2^24, so int32 lanes give the same numbers. */
        int32_t aux32[8] = {0};
        const int8_t *q8 = y[i].qs;
        a = aux8;
        for (int j = 0; j < QK_K / 16; j++) {
            int32_t scale = x[i].scales[j];
            for (int l = 0; l < 8; l++) aux32[l] += scale * ((int32_t)q8[l] * (int32_t)a[l]);
            q8 += 8;
            a += 8;
            for (int l = 0; l < 8; l++) aux32[l] += scale * ((int32_t)q8[l] * (int32_t)a[l]);
            q8 += 8;
            a += 8;
        }
        float d = f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; l++) sums[l] += (float)aux32[l] * d;
    }
    float s = 0.f;
    for (int l = 0; l < 8; l++) s += sums[l];
    return s;
}

static float vec_dot_q8_0_q8_0(size_t n, const block_q8_0 *x, const block_q8_0 *y)
{
    float sumf = 0.f;
    for (size_t i = 0; i < n / QK8_0; i++) {
        int32_t sumi = 0;
        for (int j = 0; j < QK8_0; j++) sumi += (int32_t)x[i].qs[j] * (int32_t)y[i].qs[j];
        sumf += (float)sumi * f16_to_f32(x[i].d) * f16_to_f32(y[i].d);
    }
    return sumf;
}

/* ------------------------------------------------------------------ the same block dots with AVX2
 * What candle does on x86 hosts: SIMD integer dots.  These restate the three hot ones (Q4_K, Q6_K and Q8_0
 * weights) so that the CPU baseline is not a scalar loop, with THE SAME eight f32 lanes as the portable
 * routines above: lane l collects the elements l, l + 8, l + 16, ... of a block, which is what the byte
 * shuffle below arranges before the pairwise multiply-add.  Integer sums are exact in any order, the f32 steps
 * are the portable ones in the same order: results are bit-identical (tests/test_oracle.py checks it). */
#if defined(__AVX2__)
#include <immintrin.h>
static int g_use_simd = 1;

/* bytes (b0..b15) of each 128-bit half -> (b0,b8,b1,b9,...,b7,b15): neighbours become the pair (l, l + 8) */
static inline __m256i pair_mod8(__m256i v)
{
    const __m256i m = _mm256_setr_epi8(0, 8, 1, 9, 2, 10, 3, 11, 4, 12, 5, 13, 6, 14, 7, 15,
                                       0, 8, 1, 9, 2, 10, 3, 11, 4, 12, 5, 13, 6, 14, 7, 15);
    return _mm256_shuffle_epi8(v, m);
}

/* 32 unsigned bytes a (0..63) times 32 signed bytes y, both already paired: eight int32 lanes, lane l = sum of
 * a[i] * y[i] over i = l mod 8 */
static inline __m256i dot32_mod8(__m256i a, __m256i y)
{
    const __m256i p = _mm256_maddubs_epi16(a, y);                            /* 16 x int16: half h, lane l = groups 2h, 2h+1 */
    const __m128i s = _mm_add_epi16(_mm256_castsi256_si128(p), _mm256_extracti128_si256(p, 1));
    return _mm256_cvtepi16_epi32(s);
}

static float vec_dot_q4_K_q8_K_avx2(size_t n, const block_q4_K *x, const block_q8_K *y)
{
    float sums[8] = {0};
    float sumf = 0.f;
    for (size_t i = 0; i < n / QK_K; i++) {
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; j++) q4k_scale_min(j, x[i].scales, &sc[j], &mn[j]);
        int32_t sumi = 0;
        for (int j = 0; j < QK_K / 16; j++) sumi += (int32_t)y[i].bsums[j] * (int32_t)mn[j / 2];
        __m256i acc = _mm256_setzero_si256();
        const __m256i lowmask = _mm256_set1_epi8(0xF);
        for (int j = 0; j < QK_K / 64; j++) {
            const __m256i q = pair_mod8(_mm256_loadu_si256((const __m256i *)(x[i].qs + 32 * j)));
            const __m256i y0 = pair_mod8(_mm256_loadu_si256((const __m256i *)(y[i].qs + 64 * j)));
            const __m256i y1 = pair_mod8(_mm256_loadu_si256((const __m256i *)(y[i].qs + 64 * j + 32)));
            const __m256i lo = _mm256_and_si256(q, lowmask), hi = _mm256_and_si256(_mm256_srli_epi16(q, 4), lowmask);
            acc = _mm256_add_epi32(acc, _mm256_mullo_epi32(dot32_mod8(lo, y0), _mm256_set1_epi32(sc[2 * j])));
            acc = _mm256_add_epi32(acc, _mm256_mullo_epi32(dot32_mod8(hi, y1), _mm256_set1_epi32(sc[2 * j + 1])));
        }
        int32_t aux32[8];
        _mm256_storeu_si256((__m256i *)aux32, acc);
        float d = f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; l++) sums[l] += d * (float)aux32[l];
        float dmin = f16_to_f32(x[i].dmin) * y[i].d;
        sumf -= dmin * (float)sumi;
    }
    float s = 0.f;
    for (int l = 0; l < 8; l++) s += sums[l];
    return sumf + s;
}

static float vec_dot_q6_K_q8_K_avx2(size_t n, const block_q6_K *x, const block_q8_K *y)
{
    float sums[8] = {0};
    for (size_t i = 0; i < n / QK_K; i++) {
        __m256i acc = _mm256_setzero_si256();
        const __m256i m4 = _mm256_set1_epi8(0xF), m2 = _mm256_set1_epi8(3), off = _mm256_set1_epi8(32);
        for (int h = 0; h < 2; h++) {   /* 128 weights: four streams of 32 over ql[64], qh[32] */
            const __m256i la = _mm256_loadu_si256((const __m256i *)(x[i].ql + 64 * h));
            const __m256i lb = _mm256_loadu_si256((const __m256i *)(x[i].ql + 64 * h + 32));
            const __m256i qh = _mm256_loadu_si256((const __m256i *)(x[i].qh + 32 * h));
            __m256i q[4];
            q[0] = _mm256_or_si256(_mm256_and_si256(la, m4), _mm256_slli_epi16(_mm256_and_si256(qh, m2), 4));
            q[1] = _mm256_or_si256(_mm256_and_si256(lb, m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 2), m2), 4));
            q[2] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(la, 4), m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 4), m2), 4));
            q[3] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(lb, 4), m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 6), m2), 4));
            for (int st = 0; st < 4; st++) {
                /* 32 weights = two sub-blocks of 16 (one 128-bit half each).  (q - 32) * y as q * y - 32 * y: the
                 * quants stay unsigned bytes (a Q8_K block always holds a -128, which no sign trick may negate) */
                const __m256i a = pair_mod8(q[st]);
                const __m256i yy = pair_mod8(_mm256_loadu_si256((const __m256i *)(y[i].qs + 128 * h + 32 * st)));
                const __m256i p = _mm256_sub_epi16(_mm256_maddubs_epi16(a, yy), _mm256_maddubs_epi16(off, yy));
                const int s0 = x[i].scales[8 * h + 2 * st], s1 = x[i].scales[8 * h + 2 * st + 1];
                const __m256i p0 = _mm256_cvtepi16_epi32(_mm256_castsi256_si128(p));
                const __m256i p1 = _mm256_cvtepi16_epi32(_mm256_extracti128_si256(p, 1));
                acc = _mm256_add_epi32(acc, _mm256_mullo_epi32(p0, _mm256_set1_epi32(s0)));
                acc = _mm256_add_epi32(acc, _mm256_mullo_epi32(p1, _mm256_set1_epi32(s1)));
            }
        }
        int32_t aux32[8];
        _mm256_storeu_si256((__m256i *)aux32, acc);
        float d = f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; l++) sums[l] += (float)aux32[l] * d;
    }
    float s = 0.f;
    for (int l = 0; l < 8; l++) s += sums[l];
    return s;
}

static float vec_dot_q8_0_q8_0_avx2(size_t n, const block_q8_0 *x, const block_q8_0 *y)
{
    float sumf = 0.f;
    const __m256i ones = _mm256_set1_epi16(1);
    for (size_t i = 0; i < n / QK8_0; i++) {
        const __m256i a = _mm256_loadu_si256((const __m256i *)x[i].qs), b = _mm256_loadu_si256((const __m256i *)y[i].qs);
        const __m256i p = _mm256_madd_epi16(_mm256_maddubs_epi16(_mm256_abs_epi8(a), _mm256_sign_epi8(b, a)), ones);
        __m128i s = _mm_add_epi32(_mm256_castsi256_si128(p), _mm256_extracti128_si256(p, 1));
        s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4E));
        s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xB1));
        const int32_t sumi = _mm_cvtsi128_si32(s);
        sumf += (float)sumi * f16_to_f32(x[i].d) * f16_to_f32(y[i].d);
    }
    return sumf;
}
#else
static int g_use_simd = 0;
#endif

/* ------------------------------------------------------------------ quantised mat-mul */

/* candle k_quants::matmul: each activation row is quantised to the weight type's
 * vec-dot type (Q4K,Q6K -> Q8K; Q8_0 -> Q8_0), then every output element is one
 * block dot product.  `rows0..rows1` lets callers split the output columns the
 * way candle's rayon loop does; the numbers do not depend on the split. */
typedef struct {
    int dtype;
    size_t cols, m;
    void *blocks; /* block_q8_K[m*cols/256] or block_q8_0[m*cols/32] */
} qact;

static int qact_make(qact *a, int wdtype, const float *x, size_t m, size_t cols)
{
    a->dtype = wdtype;
    a->cols = cols;
    a->m = m;
    if (wdtype == PMO_Q2_K || wdtype == PMO_Q3_K || wdtype == PMO_Q4_K || wdtype == PMO_Q5_K || wdtype == PMO_Q6_K) {
        if (cols % QK_K) return -1;
        block_q8_K *b = (block_q8_K *)malloc(sizeof(block_q8_K) * m * (cols / QK_K));
        for (size_t r = 0; r < m; r++) quantize_row_q8_K(x + r * cols, cols, b + r * (cols / QK_K));
        a->blocks = b;
        return 0;
    }
    if (wdtype == PMO_Q8_0) {
        if (cols % QK8_0) return -1;
        block_q8_0 *b = (block_q8_0 *)malloc(sizeof(block_q8_0) * m * (cols / QK8_0));
        for (size_t r = 0; r < m; r++) quantize_row_q8_0(x + r * cols, cols, b + r * (cols / QK8_0));
        a->blocks = b;
        return 0;
    }
    return -1;
}

static void qact_free(qact *a) { free(a->blocks); a->blocks = NULL; }

static inline float qdot(int dtype, const void *w, size_t row, size_t cols, const qact *a, size_t r)
{
#if defined(__AVX2__)
    if (g_use_simd) {
        if (dtype == PMO_Q4_K)
            return vec_dot_q4_K_q8_K_avx2(cols, (const block_q4_K *)w + row * (cols / QK_K),
                                          (const block_q8_K *)a->blocks + r * (cols / QK_K));
        if (dtype == PMO_Q6_K)
            return vec_dot_q6_K_q8_K_avx2(cols, (const block_q6_K *)w + row * (cols / QK_K),
                                          (const block_q8_K *)a->blocks + r * (cols / QK_K));
        if (dtype == PMO_Q8_0)
            return vec_dot_q8_0_q8_0_avx2(cols, (const block_q8_0 *)w + row * (cols / QK8_0),
                                          (const block_q8_0 *)a->blocks + r * (cols / QK8_0));
    }
#endif
    switch (dtype) {
    case PMO_Q4_K:
        return vec_dot_q4_K_q8_K(cols, (const block_q4_K *)w + row * (cols / QK_K),
                                 (const block_q8_K *)a->blocks + r * (cols / QK_K));
    case PMO_Q2_K:
        return vec_dot_q2_K_q8_K(cols, (const block_q2_K *)w + row * (cols / QK_K),
                                 (const block_q8_K *)a->blocks + r * (cols / QK_K));
    case PMO_Q3_K:
        return vec_dot_q3_K_q8_K(cols, (const block_q3_K *)w + row * (cols / QK_K),
                                 (const block_q8_K *)a->blocks + r * (cols / QK_K));
    case PMO_Q5_K:
        return vec_dot_q5_K_q8_K(cols, (const block_q5_K *)w + row * (cols / QK_K),
                                 (const block_q8_K *)a->blocks + r * (cols / QK_K));
    case PMO_Q6_K:
        return vec_dot_q6_K_q8_K(cols, (const block_q6_K *)w + row * (cols / QK_K),
                                 (const block_q8_K *)a->blocks + r * (cols / QK_K));
    default:
        return vec_dot_q8_0_q8_0(cols, (const block_q8_0 *)w + row * (cols / QK8_0),
                                 (const block_q8_0 *)a->blocks + r * (cols / QK8_0));
    }
}

static void qmatmul_rows(int dtype, const void *w, size_t rows, size_t cols, const qact *a, float *y,
                         size_t row0, size_t row1)
{
    for (size_t r = 0; r < a->m; r++)
        for (size_t c = row0; c < row1; c++) y[r * rows + c] = qdot(dtype, w, c, cols, a, r);
}

int pmo_qmatmul(int dtype, const void *w, size_t rows, size_t cols, const float *x, size_t m, float *y)
{
    qact a;
    if (qact_make(&a, dtype, x, m, cols)) return -1;
    size_t chunk = 32;
#pragma omp parallel for schedule(dynamic)
    for (size_t c0 = 0; c0 < rows; c0 += chunk)
        qmatmul_rows(dtype, w, rows, cols, &a, y, c0, c0 + chunk < rows ? c0 + chunk : rows);
    qact_free(&a);
    return 0;
}

/* ------------------------------------------------------------------ router */

/* logits = x * W_r^T (qwen3_next.rs:1916-1918; an F32 tensor makes QMatMul a dense
 * f32 product).  The f32 summation order of the reference's GEMM is unspecified,
 * so this build fixes one and the CUDA router follows it bit for bit:
 *   32 partial sums; partial p takes elements 128*i + 4*p + j (i ascending, then
 *   j = 0..3), each step one fused multiply-add; the partials are then folded by
 *   a butterfly v[p] += v[p ^ s] for s = 16, 8, 4, 2, 1.
 * H must be a multiple of 128. */
void pmo_router_logits(const float *W, const float *bias, int E, int H, const float *x, int n, float *logits)
{
#pragma omp parallel for schedule(static) collapse(2)
    for (int t = 0; t < n; t++) {
        for (int e = 0; e < E; e++) {
            const float *w = W + (size_t)e * H;
            const float *xt = x + (size_t)t * H;
            float v[32];
            for (int p = 0; p < 32; p++) {
                float acc = 0.f;
                for (int i = 0; i < H / 128; i++)
                    for (int j = 0; j < 4; j++) acc = fmaf(xt[128 * i + 4 * p + j], w[128 * i + 4 * p + j], acc);
                v[p] = acc;
            }
            for (int s = 16; s >= 1; s >>= 1) {
                float t2[32];
                for (int p = 0; p < 32; p++) t2[p] = v[p] + v[p ^ s];
                memcpy(v, t2, sizeof v);
            }
            logits[(size_t)t * E + e] = bias ? v[0] + bias[e] : v[0];
        }
    }
}

/* clamp (qwen3_next.rs:1923), softmax over the last dim (1924), then
 * topk_moe_routing_optimized (ops.rs:38-59): descending sort, first k, weights
 * divided by their sum.  A stable sort is assumed: equal probabilities keep
 * ascending expert order, which repeated strict-greater selection reproduces. */
void pmo_route_topk(const float *logits, int n, int E, int k, uint32_t *idx, float *w, float *probs_opt)
{
#pragma omp parallel for schedule(static)
    for (int t = 0; t < n; t++) {
        float *p = (float *)malloc(sizeof(float) * E);
        unsigned char *taken = (unsigned char *)calloc(E, 1);
        float mx = -INFINITY;
        for (int e = 0; e < E; e++) {
            float v = logits[(size_t)t * E + e];
            v = v < -100.f ? -100.f : (v > 100.f ? 100.f : v);
            p[e] = v;
            if (v > mx) mx = v;
        }
        float sum = 0.f;
        for (int e = 0; e < E; e++) { p[e] = expf(p[e] - mx); sum += p[e]; }
        for (int e = 0; e < E; e++) p[e] = p[e] / sum;
        if (probs_opt) memcpy(probs_opt + (size_t)t * E, p, sizeof(float) * E);
        float wsum = 0.f;
        for (int j = 0; j < k; j++) {
            int best = -1;
            for (int e = 0; e < E; e++)
                if (!taken[e] && (best < 0 || p[e] > p[best])) best = e;
            taken[best] = 1;
            idx[(size_t)t * k + j] = (uint32_t)best;
            w[(size_t)t * k + j] = p[best];
            wsum += p[best];
        }
        for (int j = 0; j < k; j++) w[(size_t)t * k + j] = w[(size_t)t * k + j] / wsum;
        free(p);
        free(taken);
    }
}

/* ------------------------------------------------------------------ experts */

static inline float silu_f(float v) { return v / (1.f + expf(-v)); }   /* candle unary silu */
static inline float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); } /* candle_nn::ops::sigmoid */

/* apply_experts_sequential grouping (qwen3_next.rs:2037-2050) followed by
 * process_experts_tokio (tokio_experts.rs:81-153) and
 * process_single_expert_optimized (157-204): active experts in ascending id,
 * rows gathered per expert, gate/up quantised mat-muls, silu(gate)*up, down
 * mat-mul, rows scaled by the routing weight, then added into a zeroed buffer
 * expert by expert.  Indices >= E are skipped (qwen3_next.rs:2045). */
int pmo_experts_forward(const pmo_layer *L, const float *x, int n, const uint32_t *idx, const float *w,
                        int k, float *out)
{
    const int H = L->H, F = L->F, E = L->E;
    size_t gsz = pmo_row_bytes(L->gate_dtype, H) * F;
    size_t usz = pmo_row_bytes(L->up_dtype, H) * F;
    size_t dsz = pmo_row_bytes(L->down_dtype, F) * H;
    if (!gsz || !usz || !dsz) return -1;

    int *count = (int *)calloc((size_t)E + 1, sizeof(int));
    for (int i = 0; i < n * k; i++) if (idx[i] < (uint32_t)E) count[idx[i] + 1]++;
    for (int e = 0; e < E; e++) count[e + 1] += count[e];
    int total = count[E];
    int *tok = (int *)malloc(sizeof(int) * (total ? total : 1));
    float *tw = (float *)malloc(sizeof(float) * (total ? total : 1));
    int *fill = (int *)calloc(E, sizeof(int));
    for (int t = 0; t < n; t++)
        for (int j = 0; j < k; j++) {
            uint32_t e = idx[t * k + j];
            if (e >= (uint32_t)E) continue;
            int pos = count[e] + fill[e]++;
            tok[pos] = t;
            tw[pos] = w[t * k + j];
        }
    free(fill);

    float *xg = (float *)malloc(sizeof(float) * (size_t)(total ? total : 1) * H);
    float *act = (float *)malloc(sizeof(float) * (size_t)(total ? total : 1) * F);
    float *dn = (float *)malloc(sizeof(float) * (size_t)(total ? total : 1) * H);
    for (int i = 0; i < total; i++) memcpy(xg + (size_t)i * H, x + (size_t)tok[i] * H, sizeof(float) * H);

    int n_active = 0;
    int *active = (int *)malloc(sizeof(int) * E);
    for (int e = 0; e < E; e++) if (count[e + 1] > count[e]) active[n_active++] = e;

    /* activation blocks once per expert (rows are quantised per mat-mul call in candle,
       with identical results for gate and up when their dtypes share a vec-dot type) */
    qact *qa_g = (qact *)calloc(n_active ? n_active : 1, sizeof(qact));
    qact *qa_u = (qact *)calloc(n_active ? n_active : 1, sizeof(qact));
    int err = 0;
#pragma omp parallel for schedule(dynamic)
    for (int a = 0; a < n_active; a++) {
        int e = active[a];
        size_t m = count[e + 1] - count[e];
        if (qact_make(&qa_g[a], L->gate_dtype, xg + (size_t)count[e] * H, m, H)) err = 1;
        if (qact_make(&qa_u[a], L->up_dtype, xg + (size_t)count[e] * H, m, H)) err = 1;
    }
    if (err) return -1;

    const int RC = 32; /* output-column chunk per task */
    int fchunks = (F + RC - 1) / RC;
#pragma omp parallel for schedule(dynamic) collapse(2)
    for (int a = 0; a < n_active; a++) {
        for (int c = 0; c < fchunks; c++) {
            int e = active[a];
            size_t m = count[e + 1] - count[e];
            int r0 = c * RC, r1 = r0 + RC < F ? r0 + RC : F;
            const char *wg = (const char *)L->gate_exps + (size_t)e * gsz;
            const char *wu = (const char *)L->up_exps + (size_t)e * usz;
            float *ae = act + (size_t)count[e] * F;
            for (size_t r = 0; r < m; r++)
                for (int f = r0; f < r1; f++) {
                    float g = qdot(L->gate_dtype, wg, f, H, &qa_g[a], r);
                    float u = qdot(L->up_dtype, wu, f, H, &qa_u[a], r);
                    ae[r * F + f] = silu_f(g) * u;
                }
        }
    }
    for (int a = 0; a < n_active; a++) { qact_free(&qa_g[a]); qact_free(&qa_u[a]); }

    qact *qa_d = qa_g;
#pragma omp parallel for schedule(dynamic)
    for (int a = 0; a < n_active; a++) {
        int e = active[a];
        size_t m = count[e + 1] - count[e];
        if (qact_make(&qa_d[a], L->down_dtype, act + (size_t)count[e] * F, m, F)) err = 1;
    }
    if (err) return -1;
    int hchunks = (H + RC - 1) / RC;
#pragma omp parallel for schedule(dynamic) collapse(2)
    for (int a = 0; a < n_active; a++) {
        for (int c = 0; c < hchunks; c++) {
            int e = active[a];
            size_t m = count[e + 1] - count[e];
            int r0 = c * RC, r1 = r0 + RC < H ? r0 + RC : H;
            const char *wd = (const char *)L->down_exps + (size_t)e * dsz;
            float *de = dn + (size_t)count[e] * H;
            for (size_t r = 0; r < m; r++)
                for (int h = r0; h < r1; h++)
                    de[r * H + h] = qdot(L->down_dtype, wd, h, F, &qa_d[a], r) * tw[count[e] + r];
        }
    }
    for (int a = 0; a < n_active; a++) qact_free(&qa_d[a]);

    /* serial aggregation in expert order into zeros (tokio_experts.rs:133-145) */
    memset(out, 0, sizeof(float) * (size_t)n * H);
#pragma omp parallel for schedule(static)
    for (int h0 = 0; h0 < H; h0 += 64)
        for (int i = 0; i < total; i++) {
            float *o = out + (size_t)tok[i] * H;
            const float *s = dn + (size_t)i * H;
            for (int h = h0; h < h0 + 64 && h < H; h++) o[h] += s[h];
        }

    free(qa_g); free(qa_u); free(active); free(xg); free(act); free(dn); free(tok); free(tw); free(count);
    return 0;
}

/* SharedExpert::forward (qwen3_next.rs:1776-1823) */
int pmo_shared_forward(const pmo_layer *L, const float *x, int n, float *out)
{
    const int H = L->H, F = L->F;
    if (!L->has_shared) { memset(out, 0, sizeof(float) * (size_t)n * H); return 0; }
    float *g = (float *)malloc(sizeof(float) * (size_t)n * F);
    float *u = (float *)malloc(sizeof(float) * (size_t)n * F);
    int rc = 0;
    rc |= pmo_qmatmul(L->sh_gate_dtype, L->sh_gate, F, H, x, n, g);
    rc |= pmo_qmatmul(L->sh_up_dtype, L->sh_up, F, H, x, n, u);
    for (size_t i = 0; i < (size_t)n * F; i++) g[i] = silu_f(g[i]) * u[i];
    rc |= pmo_qmatmul(L->sh_down_dtype, L->sh_down, H, F, g, n, out);
    for (int t = 0; t < n; t++) {
        float s = 0.f;
        for (int h = 0; h < H; h++) s += x[(size_t)t * H + h] * L->sh_gate_inp[h];
        float sg = sigmoid_f(s);
        for (int h = 0; h < H; h++) out[(size_t)t * H + h] *= sg;
    }
    free(g); free(u);
    return rc;
}

/* gate.forward (qwen3_next.rs:1916-1918).  ffn_gate_inp is a QMatMul (models/with_tracing.rs:324-335): held as f32 it
   is the canonical-order GEMV; held quantised it takes the same CPU route as the expert matrices -- rows quantised to
   Q8_K / Q8_0, integer block dots (candle k_quants::matmul). */
int pmo_layer_router_logits(const pmo_layer *L, const float *x, int n, float *logits)
{
    if (L->router_dtype == PMO_F32 || !L->router_q) {
        pmo_router_logits(L->router_w, L->router_bias, L->E, L->H, x, n, logits);
        return 0;
    }
    int rc = pmo_qmatmul(L->router_dtype, L->router_q, (size_t)L->E, (size_t)L->H, x, (size_t)n, logits);
    if (!rc && L->router_bias)
        for (size_t i = 0; i < (size_t)n * L->E; i++) logits[i] += L->router_bias[i % L->E];
    return rc;
}

/* MoeBlock::forward_with_stats (qwen3_next.rs:1903-1940): returns the unclamped logits */
int pmo_moe_forward(const pmo_layer *L, const float *x, int n, float *out,
                    float *logits_out, uint32_t *idx_out, float *w_out)
{
    const int H = L->H, E = L->E, k = L->k;
    float *logits = logits_out ? logits_out : (float *)malloc(sizeof(float) * (size_t)n * E);
    uint32_t *idx = idx_out ? idx_out : (uint32_t *)malloc(sizeof(uint32_t) * (size_t)n * k);
    float *w = w_out ? w_out : (float *)malloc(sizeof(float) * (size_t)n * k);
    int rc = pmo_layer_router_logits(L, x, n, logits);
    pmo_route_topk(logits, n, E, k, idx, w, NULL);
    if (!rc) rc = pmo_experts_forward(L, x, n, idx, w, k, out);
    if (!rc && L->has_shared) {
        float *sh = (float *)malloc(sizeof(float) * (size_t)n * H);
        rc = pmo_shared_forward(L, x, n, sh);
        for (size_t i = 0; i < (size_t)n * H; i++) out[i] = out[i] + sh[i];
        free(sh);
    }
    if (!logits_out) free(logits);
    if (!idx_out) free(idx);
    if (!w_out) free(w);
    return rc;
}

/* ------------------------------------------------------------------ exact-math variant */

static void exact_matvec(int dtype, const void *w, size_t rows, size_t cols, const double *x, double *y)
{
    size_t rb = pmo_row_bytes(dtype, cols);
#pragma omp parallel
    {
        float *tmp = (float *)malloc(sizeof(float) * cols);
#pragma omp for schedule(static)
        for (size_t r = 0; r < rows; r++) {
            pmo_dequantize(dtype, (const char *)w + r * rb, cols, tmp);
            double s = 0;
            for (size_t c = 0; c < cols; c++) s += (double)tmp[c] * x[c];
            y[r] = s;
        }
        free(tmp);
    }
}

int pmo_moe_forward_exact(const pmo_layer *L, const float *x, int n, const uint32_t *idx, const float *w,
                          float *out)
{
    const int H = L->H, F = L->F, E = L->E, k = L->k;
    size_t gsz = pmo_row_bytes(L->gate_dtype, H) * F;
    size_t usz = pmo_row_bytes(L->up_dtype, H) * F;
    size_t dsz = pmo_row_bytes(L->down_dtype, F) * H;
    double *xd = (double *)malloc(sizeof(double) * H);
    double *g = (double *)malloc(sizeof(double) * F), *u = (double *)malloc(sizeof(double) * F);
    double *d = (double *)malloc(sizeof(double) * H), *acc = (double *)malloc(sizeof(double) * H);
    for (int t = 0; t < n; t++) {
        for (int h = 0; h < H; h++) { xd[h] = x[(size_t)t * H + h]; acc[h] = 0; }
        for (int j = 0; j <= k; j++) {
            const void *wg, *wu, *wd; int gd, ud, dd; double wt;
            if (j < k) {
                uint32_t e = idx[t * k + j];
                if (e >= (uint32_t)E) continue;
                wg = (const char *)L->gate_exps + e * gsz; wu = (const char *)L->up_exps + e * usz;
                wd = (const char *)L->down_exps + e * dsz;
                gd = L->gate_dtype; ud = L->up_dtype; dd = L->down_dtype; wt = w[t * k + j];
            } else {
                if (!L->has_shared) continue;
                wg = L->sh_gate; wu = L->sh_up; wd = L->sh_down;
                gd = L->sh_gate_dtype; ud = L->sh_up_dtype; dd = L->sh_down_dtype;
                double s = 0;
                for (int h = 0; h < H; h++) s += xd[h] * (double)L->sh_gate_inp[h];
                wt = 1.0 / (1.0 + exp(-s));
            }
            exact_matvec(gd, wg, F, H, xd, g);
            exact_matvec(ud, wu, F, H, xd, u);
            for (int f = 0; f < F; f++) g[f] = g[f] / (1.0 + exp(-g[f])) * u[f];
            exact_matvec(dd, wd, H, F, g, d);
            for (int h = 0; h < H; h++) acc[h] += wt * d[h];
        }
        for (int h = 0; h < H; h++) out[(size_t)t * H + h] = (float)acc[h];
    }
    free(xd); free(g); free(u); free(d); free(acc);
    return 0;
}

/* RmsNorm::forward (paramecia-model/src/quantized_nn.rs:172-190 -> candle_nn::ops::rms_norm):
 * f32 sum of squares, m = sqrt(sum/H + eps), y = x / m * weight */
void pmo_rms_norm(const float *x, const float *weight, int n, int H, float eps, float *y)
{
#pragma omp parallel for schedule(static)
    for (int t = 0; t < n; t++) {
        const float *xt = x + (size_t)t * H;
        float s = 0.f;
        for (int h = 0; h < H; h++) s += xt[h] * xt[h];
        float m = sqrtf(s / (float)H + eps);
        for (int h = 0; h < H; h++) y[(size_t)t * H + h] = xt[h] / m * (weight ? weight[h] : 1.f);
    }
}

int pmo_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void pmo_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* 1: AVX2 block dots for Q4_K / Q6_K / Q8_0 weights (the default where the build has AVX2), 0: the portable ones */
void pmo_set_simd(int on)
{
#if defined(__AVX2__)
    g_use_simd = on ? 1 : 0;
#else
    (void)on;
#endif
}

const char *pmo_simd_kind(void)
{
    return g_use_simd ? "AVX2 integer block dots for Q4_K / Q6_K / Q8_0 (portable for the other types)"
                      : "portable vec_dot (compiler-vectorised)";
}
