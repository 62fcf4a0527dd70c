// Device-side building blocks of the expert kernels, shared by pmoe_gemv.cu (streaming dp4a kernels) and
// pmoe_gemv_mma.cu (tensor-core kernels): per-dtype lane units, the shared-memory ring and its producer,
// the work partition, and the item loops of the streaming kind.
#pragma once
#include <atomic>
#include <cstdlib>
#include "pmoe_common.cuh"
#include "pmoe_quant.cuh"

namespace pmoe {

constexpr int GEMV_WARPS = 8;
constexpr int GEMV_THREADS = (GEMV_WARPS + 1) * 32;  // compute warps + one producer warp
constexpr int NSTAGE = 3;
constexpr int STAGE_BYTES = 36864;  // one ring slot
constexpr int BULK_PIECE = 12288;   // bytes per bulk copy
constexpr int TG = GEMV_TG;         // tokens per pass of the gate/up kernels and of Q4_K down
constexpr int TG_MAX = GEMV_TG_WIDE; // tokens per pass of the Q6_K / Q8_0 down kernels

// ---------------------------------------------------------------- per-dtype lane units
// A "unit" is the piece of a row one lane handles at a time.
struct ActQ4K {   // 64 activations of one quarter of a Q8_K block
    uint32_t a[16];
    float dx;
    int bs_lo, bs_hi;  // sums of the quants under the low-nibble / high-nibble sub-block
};
struct ActQ16 {   // 4 groups of 4 activations
    uint32_t a[4];
    float dx;
};
struct ActQ32 {   // 4 runs of 8 activations
    uint32_t a[8];
    float dx;
};
struct ActQ6K {   // 64 activations of a Q8_K block: four runs of 16, one per 6-bit scale of the unit
    uint32_t a[16];
    float dx;
    int bs[4];    // sum of each run (the block's partial sums)
};

// Internal variant of Q6_K for the down kernels of calls with several tokens per expert: 32-weight
// lane units, whose eight activation words per token let a pass take four tokens.  Same bytes,
// same arithmetic; only the split of a row over lanes and passes differs.
constexpr int Q6_K_T4 = 1000 + PMOE_Q6_K;

template <int DT> struct Tr;
template <> struct Tr<PMOE_Q4_K> {
    static constexpr int UNIT = 64;
    static constexpr bool KQ = true;
    using Act = ActQ4K;
};
// Q2_K and Q3_K interleave their 2-bit quants like Q6_K (element 128*half + 32*stream + l sits in byte
// 32*half + l at bits 2*stream), so a lane takes the same 64 weights: 16 positions of four streams.
template <> struct Tr<PMOE_Q2_K> {
    static constexpr int UNIT = 64;
    static constexpr bool KQ = true;
    using Act = ActQ6K;
};
template <> struct Tr<PMOE_Q3_K> {
    static constexpr int UNIT = 64;
    static constexpr bool KQ = true;
    using Act = ActQ6K;
};
template <> struct Tr<PMOE_Q5_K> {   // same split of a block over lanes as Q4_K
    static constexpr int UNIT = 64;
    static constexpr bool KQ = true;
    using Act = ActQ4K;
};
template <> struct Tr<PMOE_Q6_K> {
    static constexpr int UNIT = 64;
    static constexpr bool KQ = true;
    using Act = ActQ6K;
};
template <> struct Tr<Q6_K_T4> {
    static constexpr int UNIT = 32;
    static constexpr bool KQ = true;
    using Act = ActQ32;
};
template <> struct Tr<PMOE_Q8_0> {
    static constexpr int UNIT = 16;
    static constexpr bool KQ = false;
    using Act = ActQ16;
};

template <int DT> __device__ inline void zero_act(typename Tr<DT>::Act &o);
template <> __device__ inline void zero_act<PMOE_Q4_K>(ActQ4K &o)
{
#pragma unroll
    for (int i = 0; i < 16; i++) o.a[i] = 0;
    o.dx = 0.f; o.bs_lo = 0; o.bs_hi = 0;
}
template <> __device__ inline void zero_act<PMOE_Q5_K>(ActQ4K &o) { zero_act<PMOE_Q4_K>(o); }
template <> __device__ inline void zero_act<PMOE_Q6_K>(ActQ6K &o)
{
#pragma unroll
    for (int i = 0; i < 16; i++) o.a[i] = 0;
    o.dx = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) o.bs[i] = 0;
}
template <> __device__ inline void zero_act<PMOE_Q2_K>(ActQ6K &o) { zero_act<PMOE_Q6_K>(o); }
template <> __device__ inline void zero_act<PMOE_Q3_K>(ActQ6K &o) { zero_act<PMOE_Q6_K>(o); }
template <> __device__ inline void zero_act<PMOE_Q8_0>(ActQ16 &o)
{
#pragma unroll
    for (int i = 0; i < 4; i++) o.a[i] = 0;
    o.dx = 0.f;
}
template <> __device__ inline void zero_act<Q6_K_T4>(ActQ32 &o)
{
#pragma unroll
    for (int i = 0; i < 8; i++) o.a[i] = 0;
    o.dx = 0.f;
}

template <int DT> __device__ inline void load_act(const QAct &q, size_t row, int K, int u, typename Tr<DT>::Act &o);

template <> __device__ inline void load_act<PMOE_Q4_K>(const QAct &q, size_t row, int K, int u, ActQ4K &o)
{
    const int b = u >> 2, qd = u & 3;
    const uint4 *p = reinterpret_cast<const uint4 *>(q.qs + row * K + 256 * b + 64 * qd);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint4 v = p[i];
        o.a[4 * i + 0] = v.x; o.a[4 * i + 1] = v.y; o.a[4 * i + 2] = v.z; o.a[4 * i + 3] = v.w;
    }
    o.dx = q.d[row * (K / QK_K) + b];
    const short4 bs = *reinterpret_cast<const short4 *>(q.bsums + row * (K / 16) + 16 * b + 4 * qd);
    o.bs_lo = (int)bs.x + (int)bs.y;
    o.bs_hi = (int)bs.z + (int)bs.w;
}

template <> __device__ inline void load_act<PMOE_Q5_K>(const QAct &q, size_t row, int K, int u, ActQ4K &o)
{
    load_act<PMOE_Q4_K>(q, row, K, u, o);
}

// Unit u of a Q6_K row: block u/4, 128-element half (u/2)%2, and inside the half the 16 positions
// l = 16*jj .. 16*jj+15 (jj = u%2) of each of the four interleaved quant streams, i.e. elements
// 128*half + 32*g + 16*jj + (0..15) for g = 0..3.  Each run lies under one 6-bit scale.
template <> __device__ inline void load_act<PMOE_Q6_K>(const QAct &q, size_t row, int K, int u, ActQ6K &o)
{
    const int b = u >> 2, half = (u >> 1) & 1, jj = u & 1;
    const int8_t *p = q.qs + row * K + 256 * b + 128 * half + 16 * jj;
#pragma unroll
    for (int g = 0; g < 4; g++) {
        const uint4 v = *reinterpret_cast<const uint4 *>(p + 32 * g);
        o.a[4 * g + 0] = v.x; o.a[4 * g + 1] = v.y; o.a[4 * g + 2] = v.z; o.a[4 * g + 3] = v.w;
    }
    o.dx = q.d[row * (K / QK_K) + b];
    const int16_t *bs = q.bsums + row * (K / 16) + 16 * b + 8 * half + jj;
#pragma unroll
    for (int g = 0; g < 4; g++) o.bs[g] = bs[2 * g];
}

template <> __device__ inline void load_act<PMOE_Q2_K>(const QAct &q, size_t row, int K, int u, ActQ6K &o)
{
    load_act<PMOE_Q6_K>(q, row, K, u, o);
}
template <> __device__ inline void load_act<PMOE_Q3_K>(const QAct &q, size_t row, int K, int u, ActQ6K &o)
{
    load_act<PMOE_Q6_K>(q, row, K, u, o);
}

// 32-weight unit u: block u/8, half (u/4)%2, positions l = 8jj .. 8jj+7 (jj = u%4) of the four streams
template <> __device__ inline void load_act<Q6_K_T4>(const QAct &q, size_t row, int K, int u, ActQ32 &o)
{
    const int b = u >> 3, half = (u >> 2) & 1, jj = u & 3;
    const int8_t *p = q.qs + row * K + 256 * b + 128 * half + 8 * jj;
#pragma unroll
    for (int g = 0; g < 4; g++) {
        const uint2 v = *reinterpret_cast<const uint2 *>(p + 32 * g);
        o.a[2 * g] = v.x; o.a[2 * g + 1] = v.y;
    }
    o.dx = q.d[row * (K / QK_K) + b];
}

template <> __device__ inline void load_act<PMOE_Q8_0>(const QAct &q, size_t row, int K, int u, ActQ16 &o)
{
    const int b = u >> 1, hf = u & 1;
    const uint4 v = *reinterpret_cast<const uint4 *>(q.qs + row * K + 32 * b + 16 * hf);
    o.a[0] = v.x; o.a[1] = v.y; o.a[2] = v.z; o.a[3] = v.w;
    o.dx = q.d[row * (K / QK8_0) + b];
}

// dp4a with unsigned bytes in a and signed bytes in b
__device__ inline int dp4a_us(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Dot<DT>: the per-lane inner product of one unit of one weight row (in shared memory) with the
// activations of CNT tokens.  Pre holds what depends only on the lane's unit (byte offsets
// inside the row, shift amounts) and is computed once per kernel.
template <int DT> struct Dot;

template <> struct Dot<PMOE_Q4_K> {
    struct Pre {
        int hdr_off, q_off, sh, hi;
    };
    __device__ static inline Pre pre(int u)
    {
        const int qd = u & 3;
        return Pre{(u >> 2) * Q4_K_BYTES, (u >> 2) * Q4_K_BYTES + 16 + 32 * qd, 16 * (qd & 1), qd >> 1};
    }
    template <int CNT, bool A4 = true>  // A4: the row starts on a 4-byte boundary
    __device__ static inline void run(const uint8_t *row, const Pre &p, const ActQ4K *act, float *acc)
    {
        const uint4 hdr = *reinterpret_cast<const uint4 *>(row + p.hdr_off);
        const uint4 qa = *reinterpret_cast<const uint4 *>(row + p.q_off);
        const uint4 qb = *reinterpret_cast<const uint4 *>(row + p.q_off + 16);
        // high nibbles stay in place (x16): 1/16 goes into d
        const float d16 = half_bits_to_float((uint16_t)(hdr.x & 0xffffu)) * 0.0625f;
        const float dmin = half_bits_to_float((uint16_t)(hdr.x >> 16));
        // 6-bit scales / mins of sub-blocks 2*qd and 2*qd+1 as byte pairs, without a branch
        const uint32_t a0 = hdr.y >> p.sh, a1 = hdr.z >> p.sh, a2 = hdr.w >> p.sh;
        const uint32_t sc_lo = a0 & 0x3F3Fu, m_lo = a1 & 0x3F3Fu;
        const uint32_t sc_hi = (a2 & 0x0F0Fu) | ((a0 >> 2) & 0x3030u);
        const uint32_t m_hi = ((a2 >> 4) & 0x0F0Fu) | ((a1 >> 2) & 0x3030u);
        const uint32_t scp = p.hi ? sc_hi : sc_lo, mp = p.hi ? m_hi : m_lo;
        const int sc0_16 = (int)(scp & 0xFFu) << 4, sc1 = (int)(scp >> 8) & 0xFF;
        const int m0 = (int)(mp & 0xFFu), m1 = (int)(mp >> 8) & 0xFF;
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
        for (int t = 0; t < CNT; t++) {
            int s_lo = 0, s_lo2 = 0, s_hi16 = 0, s_hi16b = 0;  // two chains each for ILP
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                s_lo = dp4a_us(w[i] & 0x0F0F0F0Fu, act[t].a[i], s_lo);
                s_hi16 = dp4a_us(w[i] & 0xF0F0F0F0u, act[t].a[8 + i], s_hi16);
                s_lo2 = dp4a_us(w[i + 1] & 0x0F0F0F0Fu, act[t].a[i + 1], s_lo2);
                s_hi16b = dp4a_us(w[i + 1] & 0xF0F0F0F0u, act[t].a[9 + i], s_hi16b);
            }
            const int isum16 = sc0_16 * (s_lo + s_lo2) + sc1 * (s_hi16 + s_hi16b);
            const int imin = m0 * act[t].bs_lo + m1 * act[t].bs_hi;
            acc[t] += act[t].dx * (d16 * (float)isum16 - dmin * (float)imin);
        }
    }
};

// Q5_K: the Q4_K unit with the fifth bit of each quant taken from qh (bit 2*qd for the low-nibble
// sub-block, 2*qd+1 for the high-nibble one).  With five bits the high quants no longer fit a byte
// in place, so they are shifted down.
template <> struct Dot<PMOE_Q5_K> {
    struct Pre {
        int hdr_off, q_off, sh, hi, hsh;
    };
    __device__ static inline Pre pre(int u)
    {
        const int qd = u & 3, blk = (u >> 2) * Q5_K_BYTES;
        return Pre{blk, blk + 48 + 32 * qd, 16 * (qd & 1), qd >> 1, 2 * qd};
    }
    template <int CNT, bool A4 = true>
    __device__ static inline void run(const uint8_t *row, const Pre &p, const ActQ4K *act, float *acc)
    {
        const uint4 hdr = *reinterpret_cast<const uint4 *>(row + p.hdr_off);
        const uint4 ha = *reinterpret_cast<const uint4 *>(row + p.hdr_off + 16);
        const uint4 hb = *reinterpret_cast<const uint4 *>(row + p.hdr_off + 32);
        const uint4 qa = *reinterpret_cast<const uint4 *>(row + p.q_off);
        const uint4 qb = *reinterpret_cast<const uint4 *>(row + p.q_off + 16);
        const float d = half_bits_to_float((uint16_t)(hdr.x & 0xffffu));
        const float dmin = half_bits_to_float((uint16_t)(hdr.x >> 16));
        const uint32_t a0 = hdr.y >> p.sh, a1 = hdr.z >> p.sh, a2 = hdr.w >> p.sh;
        const uint32_t sc_lo = a0 & 0x3F3Fu, m_lo = a1 & 0x3F3Fu;
        const uint32_t sc_hi = (a2 & 0x0F0Fu) | ((a0 >> 2) & 0x3030u);
        const uint32_t m_hi = ((a2 >> 4) & 0x0F0Fu) | ((a1 >> 2) & 0x3030u);
        const uint32_t scp = p.hi ? sc_hi : sc_lo, mp = p.hi ? m_hi : m_lo;
        const int sc0 = (int)(scp & 0xFFu), sc1 = (int)(scp >> 8) & 0xFF;
        const int m0 = (int)(mp & 0xFFu), m1 = (int)(mp >> 8) & 0xFF;
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        const uint32_t h[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t t = h[i] >> p.hsh;   // bit 0 of each byte: low sub-block, bit 1: high sub-block
            lo[i] = (w[i] & 0x0F0F0F0Fu) | ((t << 4) & 0x10101010u);
            hi[i] = ((w[i] >> 4) & 0x0F0F0F0Fu) | ((t << 3) & 0x10101010u);
        }
#pragma unroll
        for (int t = 0; t < CNT; t++) {
            int s_lo = 0, s_lo2 = 0, s_hi = 0, s_hi2 = 0;
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                s_lo = dp4a_us(lo[i], act[t].a[i], s_lo);
                s_hi = dp4a_us(hi[i], act[t].a[8 + i], s_hi);
                s_lo2 = dp4a_us(lo[i + 1], act[t].a[i + 1], s_lo2);
                s_hi2 = dp4a_us(hi[i + 1], act[t].a[9 + i], s_hi2);
            }
            const int isum = sc0 * (s_lo + s_lo2) + sc1 * (s_hi + s_hi2);
            const int imin = m0 * act[t].bs_lo + m1 * act[t].bs_hi;
            acc[t] += act[t].dx * (d * (float)isum - dmin * (float)imin);
        }
    }
};

// 16 bytes at row + off, 2-byte aligned: five aligned words and a funnel shift by the address's own
// misalignment (0 or 16 bits).  `mis` = (address of row) & 2.  The address is formed from `row` by
// plain offsets so that loads from a shared-memory row stay shared-memory loads.  Reads up to 4
// bytes past the 16 (inside the block for every caller).
__device__ inline void load16_a2(const uint8_t *row, int mis, int off, uint32_t (&o)[4])
{
    const int a = off + mis;
    const uint32_t *q = reinterpret_cast<const uint32_t *>(row - mis + (a & ~3));
    const uint32_t sh = (uint32_t)(a & 2) * 8;
    uint32_t u[5];
#pragma unroll
    for (int i = 0; i < 5; i++) u[i] = q[i];
#pragma unroll
    for (int i = 0; i < 4; i++) o[i] = __funnelshift_r(u[i], u[i + 1], sh);
}

__device__ inline int misalign2(const uint8_t *p) { return (int)(reinterpret_cast<uintptr_t>(p) & 2); }

// 12 bytes at row + off, 2-byte aligned: four aligned words and a funnel shift; reads nothing past
// the 14th byte from the aligned base
__device__ inline void load12_a2(const uint8_t *row, int mis, int off, uint32_t (&o)[3])
{
    const int a = off + mis;
    const uint32_t *q = reinterpret_cast<const uint32_t *>(row - mis + (a & ~3));
    const uint32_t sh = (uint32_t)(a & 2) * 8;
    const uint32_t u0 = q[0], u1 = q[1], u2 = q[2];
    const uint32_t u3 = sh ? q[3] : 0u;
    o[0] = __funnelshift_r(u0, u1, sh);
    o[1] = __funnelshift_r(u1, u2, sh);
    o[2] = __funnelshift_r(u2, u3, sh);
}

// Q2_K: unit u = block u/4, half (u/2)%2, positions 16*s .. 16*s+15 (s = u%2) of the four 2-bit streams.
// Blocks are 84 bytes, so every field is 4-byte aligned.
template <> struct Dot<PMOE_Q2_K> {
    struct Pre {
        int q_off, sc_off, d_off;
    };
    __device__ static inline Pre pre(int u)
    {
        const int blk = (u >> 2) * Q2_K_BYTES, half = (u >> 1) & 1, s = u & 1;
        return Pre{blk + 16 + 32 * half + 16 * s, blk + 8 * half + s, blk + 80};
    }
    template <int CNT, bool A4 = true>
    __device__ static inline void run(const uint8_t *row, const Pre &p, const ActQ6K *act, float *acc)
    {
        const uint32_t *qp = reinterpret_cast<const uint32_t *>(row + p.q_off);
        const uint32_t w[4] = {qp[0], qp[1], qp[2], qp[3]};
        const uint8_t *sc = row + p.sc_off;
        const uint32_t c[4] = {sc[0], sc[2], sc[4], sc[6]};   // 4-bit scale | 4-bit min << 4
        const uint32_t dd = *reinterpret_cast<const uint32_t *>(row + p.d_off);
        const float d = half_bits_to_float((uint16_t)(dd & 0xffffu));
        const float dmin = half_bits_to_float((uint16_t)(dd >> 16));
        int isum[CNT];
#pragma unroll
        for (int t = 0; t < CNT; t++) isum[t] = 0;
#pragma unroll
        for (int g = 0; g < 4; g++) {
            uint32_t v[4];
#pragma unroll
            for (int i = 0; i < 4; i++) v[i] = (w[i] >> (2 * g)) & 0x03030303u;
#pragma unroll
            for (int t = 0; t < CNT; t++) {
                int s = 0, s2 = 0;
                s = dp4a_us(v[0], act[t].a[4 * g + 0], s);
                s2 = dp4a_us(v[1], act[t].a[4 * g + 1], s2);
                s = dp4a_us(v[2], act[t].a[4 * g + 2], s);
                s2 = dp4a_us(v[3], act[t].a[4 * g + 3], s2);
                isum[t] += (int)(c[g] & 0xFu) * (s + s2);
            }
        }
#pragma unroll
        for (int t = 0; t < CNT; t++) {
            const int imin = (int)(c[0] >> 4) * act[t].bs[0] + (int)(c[1] >> 4) * act[t].bs[1] +
                             (int)(c[2] >> 4) * act[t].bs[2] + (int)(c[3] >> 4) * act[t].bs[3];
            acc[t] += act[t].dx * (d * (float)isum[t] - dmin * (float)imin);
        }
    }
};

// Q3_K: the same unit; the third bit of stream g's quants is bit 4*half + g of hmask[16*s + l], and a clear
// bit means -4: with u = q2 | bit << 2 (0..7) the signed quant is u - 4, and the -4 comes back through the
// activations' partial sums.  Blocks are 110 bytes: fields of odd blocks start 2 bytes off a word.
template <> struct Dot<PMOE_Q3_K> {
    struct Pre {
        int q_off, hm_off, sc_off, d_off, hbit, is0;
    };
    __device__ static inline Pre pre(int u)
    {
        const int blk = (u >> 2) * Q3_K_BYTES, half = (u >> 1) & 1, s = u & 1;
        return Pre{blk + 32 + 32 * half + 16 * s, blk + 16 * s, blk + 96, blk + 108, 4 * half, 8 * half + s};
    }
    template <int CNT, bool A4 = true>
    __device__ static inline void run(const uint8_t *row, const Pre &p, const ActQ6K *act, float *acc)
    {
        const int mis = A4 ? 0 : misalign2(row);
        uint32_t w[4], hm[4], sw[3];
        load16_a2(row, mis, p.q_off, w);
        load16_a2(row, mis, p.hm_off, hm);
        load12_a2(row, mis, p.sc_off, sw);   // scales[0..3], scales[4..7], scales[8..11]
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(row + p.d_off));
        int c[4];
#pragma unroll
        for (int g = 0; g < 4; g++) {
            // six-bit scale `is`: low nibble in byte is%8 (upper nibbles for is >= 8), high two bits in
            // byte 8 + is%4 at bit 2*(is/4); stored with an offset of 32
            const int is = p.is0 + 2 * g;
            const uint32_t src = ((is >> 2) & 1) ? sw[1] : sw[0];
            const uint32_t nib = (is >= 8 ? src >> 4 : src) >> (8 * (is & 3));
            const uint32_t hi2 = sw[2] >> (8 * (is & 3) + 2 * (is >> 2));
            c[g] = (int)((nib & 0xFu) | ((hi2 & 3u) << 4)) - 32;
        }
        int isum[CNT];
#pragma unroll
        for (int t = 0; t < CNT; t++)
            isum[t] = -4 * (c[0] * act[t].bs[0] + c[1] * act[t].bs[1] + c[2] * act[t].bs[2] + c[3] * act[t].bs[3]);
#pragma unroll
        for (int g = 0; g < 4; g++) {
            uint32_t v[4];
#pragma unroll
            for (int i = 0; i < 4; i++)
                v[i] = ((w[i] >> (2 * g)) & 0x03030303u) | (((hm[i] >> (p.hbit + g)) & 0x01010101u) << 2);
#pragma unroll
            for (int t = 0; t < CNT; t++) {
                int s = 0, s2 = 0;
                s = dp4a_us(v[0], act[t].a[4 * g + 0], s);
                s2 = dp4a_us(v[1], act[t].a[4 * g + 1], s2);
                s = dp4a_us(v[2], act[t].a[4 * g + 2], s);
                s2 = dp4a_us(v[3], act[t].a[4 * g + 3], s2);
                isum[t] += c[g] * (s + s2);
            }
        }
#pragma unroll
        for (int t = 0; t < CNT; t++) acc[t] += (d * act[t].dx) * (float)isum[t];
    }
};

template <> struct Dot<PMOE_Q6_K> {
    struct Pre {
        int la_off, h_off, sc_off, d_off;
    };
    __device__ static inline Pre pre(int u)
    {
        const int blk = (u >> 2) * Q6_K_BYTES, half = (u >> 1) & 1, jj = u & 1;
        return Pre{blk + 64 * half + 16 * jj, blk + 128 + 32 * half + 16 * jj, blk + 192 + 8 * half + jj, blk + 208};
    }
    template <int CNT, bool A4 = true>  // A4: the row starts on a 4-byte boundary
    __device__ static inline void run(const uint8_t *row, const Pre &p, const ActQ6K *act, float *acc)
    {
        uint32_t la[4], lb[4], h[4];
        const int mis = A4 ? 0 : misalign2(row);
        load16_a2(row, mis, p.la_off, la);
        load16_a2(row, mis, p.la_off + 32, lb);
        load16_a2(row, mis, p.h_off, h);
        const int8_t *sc = reinterpret_cast<const int8_t *>(row + p.sc_off);
        const int c[4] = {sc[0], sc[2], sc[4], sc[6]};
        // quants are used as the unsigned bytes 4*q (0..252); the offset -32 comes back through the
        // activations' partial sums (4*(q-32) = 4*q - 128) and the factor 4 is taken out of d
        const float d4 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(row + p.d_off)) * 0.25f;
        int isum[CNT];
#pragma unroll
        for (int t = 0; t < CNT; t++)
            isum[t] = -128 * (c[0] * act[t].bs[0] + c[1] * act[t].bs[1] + c[2] * act[t].bs[2] + c[3] * act[t].bs[3]);
#pragma unroll
        for (int g = 0; g < 4; g++) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t lo = g == 0 ? la[i] << 2 : g == 1 ? lb[i] << 2 : g == 2 ? la[i] >> 2 : lb[i] >> 2;
                const uint32_t hi = g == 3 ? h[i] : h[i] << (6 - 2 * g);
                w[i] = (lo & 0x3C3C3C3Cu) | (hi & 0xC0C0C0C0u);
            }
#pragma unroll
            for (int t = 0; t < CNT; t++) {
                int s = 0, s2 = 0;
                s = dp4a_us(w[0], act[t].a[4 * g + 0], s);
                s2 = dp4a_us(w[1], act[t].a[4 * g + 1], s2);
                s = dp4a_us(w[2], act[t].a[4 * g + 2], s);
                s2 = dp4a_us(w[3], act[t].a[4 * g + 3], s2);
                isum[t] += c[g] * (s + s2);
            }
        }
#pragma unroll
        for (int t = 0; t < CNT; t++) acc[t] += (d4 * act[t].dx) * (float)isum[t];
    }
};

// 8 bytes at row + off, 2-byte aligned: three aligned words and a funnel shift (see load16_a2)
__device__ inline void load8_a2(const uint8_t *row, int mis, int off, uint32_t &o0, uint32_t &o1)
{
    const int a = off + mis;
    const uint32_t *q = reinterpret_cast<const uint32_t *>(row - mis + (a & ~3));
    const uint32_t sh = (uint32_t)(a & 2) * 8;
    const uint32_t u0 = q[0], u1 = q[1], u2 = q[2];
    o0 = __funnelshift_r(u0, u1, sh);
    o1 = __funnelshift_r(u1, u2, sh);
}

template <> struct Dot<Q6_K_T4> {
    struct Pre {
        int la_off, h_off, sc_off, d_off;
    };
    __device__ static inline Pre pre(int u)
    {
        const int blk = (u >> 3) * Q6_K_BYTES, half = (u >> 2) & 1, jj = u & 3;
        return Pre{blk + 64 * half + 8 * jj, blk + 128 + 32 * half + 8 * jj, blk + 192 + 8 * half + (jj >> 1), blk + 208};
    }
    template <int CNT, bool A4 = true>  // A4: the row starts on a 4-byte boundary
    __device__ static inline void run(const uint8_t *row, const Pre &p, const ActQ32 *act, float *acc)
    {
        uint32_t la[2], lb[2], h[2];
        const int mis = A4 ? 0 : misalign2(row);
        load8_a2(row, mis, p.la_off, la[0], la[1]);
        load8_a2(row, mis, p.la_off + 32, lb[0], lb[1]);
        load8_a2(row, mis, p.h_off, h[0], h[1]);
        const int8_t *sc = reinterpret_cast<const int8_t *>(row + p.sc_off);
        const int c[4] = {sc[0], sc[2], sc[4], sc[6]};
        // the 6-bit quant goes to the top of each byte with its top bit flipped: as a signed
        // byte that is 4*(q-32); the factor 4 is taken out of d
        const float d4 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(row + p.d_off)) * 0.25f;
        uint32_t w[4][2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            w[0][i] = (((la[i] << 2) & 0x3C3C3C3Cu) | ((h[i] << 6) & 0xC0C0C0C0u)) ^ 0x80808080u;
            w[1][i] = (((lb[i] << 2) & 0x3C3C3C3Cu) | ((h[i] << 4) & 0xC0C0C0C0u)) ^ 0x80808080u;
            w[2][i] = (((la[i] >> 2) & 0x3C3C3C3Cu) | ((h[i] << 2) & 0xC0C0C0C0u)) ^ 0x80808080u;
            w[3][i] = (((lb[i] >> 2) & 0x3C3C3C3Cu) | (h[i] & 0xC0C0C0C0u)) ^ 0x80808080u;
        }
#pragma unroll
        for (int t = 0; t < CNT; t++) {
            int isum = 0;
#pragma unroll
            for (int g = 0; g < 4; g++)
                isum += c[g] * __dp4a((int)w[g][1], (int)act[t].a[2 * g + 1], __dp4a((int)w[g][0], (int)act[t].a[2 * g], 0));
            acc[t] += (d4 * act[t].dx) * (float)isum;
        }
    }
};

template <> struct Dot<PMOE_Q8_0> {
    struct Pre {
        int d_off, q_off;
    };
    __device__ static inline Pre pre(int u) { return Pre{(u >> 1) * Q8_0_BYTES, (u >> 1) * Q8_0_BYTES + 2 + 16 * (u & 1)}; }
    template <int CNT, bool A4 = true>  // A4: the row starts on a 4-byte boundary
    __device__ static inline void run(const uint8_t *row, const Pre &p, const ActQ16 *act, float *acc)
    {
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(row + p.d_off));
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) w[i] = lds_u32_a2(row + p.q_off + 4 * i);
#pragma unroll
        for (int t = 0; t < CNT; t++) {
            int isum = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) isum = __dp4a((int)w[i], (int)act[t].a[i], isum);
            acc[t] += (d * act[t].dx) * (float)isum;
        }
    }
};

// ---------------------------------------------------------------- compile-time shape of one kernel kind
constexpr int cmin(int a, int b) { return a < b ? a : b; }
constexpr int cmax(int a, int b) { return a > b ? a : b; }
constexpr int floor_pow2(int v) { int p = 1; while (2 * p <= v) p *= 2; return p; }

template <int DT, int NMAT> struct Cfg {
    static constexpr int K = NMAT == 2 ? 2048 : 512;  // reduction length: H for gate/up, F for down
    static constexpr int UNIT = Tr<DT>::UNIT;
    static constexpr int UNITS = K / UNIT;
    static constexpr int LPR = cmin(32, UNITS);       // lanes that share one row
    static constexpr int UPL = UNITS / LPR;           // units per lane
    static constexpr int GROUPS = 32 / LPR;           // rows a warp works on at once
    static constexpr int ROW_BYTES = K / (DT == PMOE_Q8_0 ? QK8_0 : QK_K) *
                                     (DT == PMOE_Q8_0 ? Q8_0_BYTES : DT == PMOE_Q2_K ? Q2_K_BYTES : DT == PMOE_Q3_K ? Q3_K_BYTES
                                      : DT == PMOE_Q4_K ? Q4_K_BYTES : DT == PMOE_Q5_K ? Q5_K_BYTES : Q6_K_BYTES);
    static constexpr int ROWS = floor_pow2(STAGE_BYTES / (ROW_BYTES * NMAT));  // rows of each matrix per item
    static constexpr int ITEM_BYTES = ROWS * ROW_BYTES;                        // per matrix
    // tokens per pass: bounded by the activation registers a lane keeps (16 words per token for Q4_K and Q6_K, 4 for Q8_0)
    static constexpr int TGK = (NMAT == 1 && (DT == PMOE_Q8_0 || DT == Q6_K_T4)) ? 4 : 2;
    static constexpr int RPW = ROWS / GEMV_WARPS;     // rows per warp per item
    static constexpr int PASSES = RPW / GROUPS;
    static constexpr int RB = cmin(cmin(PASSES, 4), cmax(1, LPR / (NMAT * TGK)));  // rows reduced together
    static constexpr int V = NMAT * RB * TGK;         // values per transposed reduction (<= LPR)
    static_assert(RPW >= GROUPS && PASSES % RB == 0 && V <= LPR && ITEM_BYTES % 16 == 0, "bad tiling");
};

// ---------------------------------------------------------------- kernel arguments
struct GemvArgs {
    const uint8_t *w0, *w1;    // routed matrices (gate, up) or (down, unused); expert e at + e*expert_bytes
    size_t expert_bytes;
    const uint8_t *sw0, *sw1;  // shared expert matrices
    int rows_total;            // output length (F for gate/up, H for down)
    int e_local;               // routed experts this layer holds
    int routed;                // serve the routed experts listed in g
    int has_shared;            // serve the shared expert
    int n, top_k;
    int sh_begin, sh_count;    // tokens the shared expert serves: [sh_begin, sh_begin + sh_count)
    Groups g;
    QAct in_r, in_s;           // quantised activations matching the routed / shared weight type
    float *out;                // act [., F] or partial [., H]
    const float *scale_r;      // routing weights [n*top_k]      (down only)
    const float *scale_s;      // shared gate sigmoid [n]        (down only)
    DevStatus *status;
    int debug;                 // 1: skip the arithmetic, 2: skip the copies (timing experiments)
    int stage_bytes;           // bytes between the slots of the shared-memory ring
    uint32_t max_polls;        // tensor-core kernels: limit of every bounded wait (try_wait calls, each up to ~20 us)
    int shw_min;               // tensor-core kernels: a Q8_0 shared expert over this many tokens or more gets its own warp
    // gate/up only: the CTA that completes an expert's last item re-quantises the expert's activated rows
    int *slot_done;            // [E_local + 1] items finished per slot (shared expert last); returns to zero
    int quant_dt_r, quant_dt_s; // block types the down matrices will consume (0 = no fused re-quantisation)
    QAct q8k_out, q80_out;
};


// Token rows of one pass.
struct Pass {
    int cnt;
    int out_row[TG_MAX];
    float scale[TG_MAX];
};

template <int DT, int NMAT>
__device__ inline void load_pass(const GemvArgs &A, bool is_shared, const int *list, int m, int t0, const QAct &in,
                                 int ul, Pass &P, typename Tr<DT>::Act (&act)[Cfg<DT, NMAT>::UPL][Cfg<DT, NMAT>::TGK])
{
    using C = Cfg<DT, NMAT>;
    P.cnt = m - t0 < C::TGK ? m - t0 : C::TGK;
#pragma unroll
    for (int t = 0; t < C::TGK; t++) {
        P.out_row[t] = -1;
        P.scale[t] = 0.f;
        if (t < P.cnt) {
            int in_row;
            if (is_shared) {
                const int tok = A.sh_begin + t0 + t;
                P.out_row[t] = A.n * A.top_k + tok;
                in_row = NMAT == 2 ? tok : P.out_row[t];
                if (NMAT == 1) P.scale[t] = A.scale_s[tok];
            } else {
                const int p = list[t0 + t];
                P.out_row[t] = p;
                in_row = NMAT == 2 ? p / A.top_k : p;
                if (NMAT == 1) P.scale[t] = A.scale_r[p];
            }
#pragma unroll
            for (int i = 0; i < C::UPL; i++) load_act<DT>(in, (size_t)in_row, C::K, i * C::LPR + ul, act[i][t]);
        } else {
#pragma unroll
            for (int i = 0; i < C::UPL; i++) zero_act<DT>(act[i][t]);
        }
    }
}

// All rows of one item (in shared memory) against one pass of CNT tokens.
template <int DT, int NMAT, int CNT>
__device__ inline void compute_item(const GemvArgs &A, const uint8_t *stage, int chunk, const Pass &P,
                                    const typename Tr<DT>::Act (&act)[Cfg<DT, NMAT>::UPL][Cfg<DT, NMAT>::TGK],
                                    const typename Dot<DT>::Pre (&pre)[Cfg<DT, NMAT>::UPL], int warp, int lane)
{
    using C = Cfg<DT, NMAT>;
    const int grp = lane / C::LPR, ul = lane % C::LPR;
#pragma unroll 1
    for (int b0 = 0; b0 < C::PASSES; b0 += C::RB) {
        float acc[C::V];
#pragma unroll
        for (int i = 0; i < C::V; i++) acc[i] = 0.f;
#pragma unroll
        for (int rb = 0; rb < C::RB; rb++) {
            const int row = warp * C::RPW + (b0 + rb) * C::GROUPS + grp;
#pragma unroll
            for (int mat = 0; mat < NMAT; mat++) {
                const uint8_t *rp = stage + mat * C::ITEM_BYTES + row * C::ROW_BYTES;
#pragma unroll
                for (int i = 0; i < C::UPL; i++) {
                    Dot<DT>::template run<CNT>(rp, pre[i], act[i], acc + (mat * C::RB + rb) * C::TGK);
                    // keeps the compiler from hoisting every unit's loads at once (register pressure)
                    if (C::UPL > 1) asm volatile("" ::: "memory");
                }
            }
        }
        float v = transposed_reduce<C::V, C::LPR>(acc, lane);
        constexpr int DUP = C::LPR / C::V;  // lanes holding the same total
        const int vi = ul / DUP;
        const int t = vi % C::TGK, rb = (vi / C::TGK) % C::RB, mat = vi / (C::TGK * C::RB);
        if (NMAT == 2) {
            const float other = __shfl_xor_sync(0xffffffffu, v, C::LPR / 2);  // up total sits LPR/2 lanes away
            v = v / (1.f + expf(-v)) * other;                                 // silu(gate) * up
        }
        const int row = chunk * C::ROWS + warp * C::RPW + (b0 + rb) * C::GROUPS + grp;
        int orow = P.out_row[0];  // t depends on the lane: pick with selects, not an indexed load
        float sc = P.scale[0];
#pragma unroll
        for (int q = 1; q < C::TGK; q++)
            if (t == q) { orow = P.out_row[q]; sc = P.scale[q]; }
        if (ul % DUP == 0 && mat == 0 && orow >= 0)
            A.out[(size_t)orow * A.rows_total + row] = NMAT == 2 ? v : v * sc;
    }
}

// Shared-memory row pitch of a gate/up item of a Q8_0 shared expert that runs as tensor-core tiles
// (run_items_shared_mma): the rows of a Q8_0 [*, 2048] matrix are
// 2176 bytes apart, a multiple of 128, so the eight rows of a fragment would meet in the same
// banks; the producer copies such an item row by row with 32 bytes of padding (a lane reads 8 bytes,
// so eight rows 32 bytes apart fill the 32 banks twice, the minimum).
template <int NMAT> struct SharedMma {
    using C = Cfg<PMOE_Q8_0, NMAT>;
    static constexpr int KB = C::K / QK8_0;                    // Q8_0 blocks per row
    static constexpr int MT = NMAT == 2 ? 1 : C::ROWS / 16;    // 16-row tiles per item
    static constexpr int PITCH = NMAT == 2 ? C::ROW_BYTES + 32 : C::ROW_BYTES;
    static constexpr bool PER_ROW_COPIES = PITCH != C::ROW_BYTES;
    static_assert(NMAT == 1 || C::ROWS == 8, "a gate/up item must be 8 + 8 rows");
    static_assert(NMAT * C::ROWS * PITCH <= STAGE_BYTES, "padded item must fit its ring slot");
    static_assert(KB % 8 == 0 && PITCH % 16 == 0, "bad shape");
};

// ---------------------------------------------------------------- work partition
// Items are ordered (slot 0 chunk 0, slot 0 chunk 1, ..., slot 1 chunk 0, ...); slot n_active is
// the shared expert.  An item of a slot with m tokens costs ceil(m / TG) passes, and the CTAs
// split the total cost evenly: a CTA takes the items whose starting cost position falls into
// its share.  The per-slot cost prefix comes from the grouping kernel.
struct Cursor {
    int slot, chunk;
};

struct Plan {
    int n_active, has_shared, cpe_r, cpe_s, cost_shared;
    bool shared_mma;     // the shared expert's items run as tensor-core tiles (own shared-memory layout)
    const int *prefix;  // [n_active + 1] in shared memory

    __device__ inline int cpe(int slot) const { return slot < n_active ? cpe_r : cpe_s; }
    __device__ inline long routed_cost() const { return (long)cpe_r * prefix[n_active]; }
    __device__ inline long total_cost() const { return routed_cost() + (has_shared ? (long)cpe_s * cost_shared : 0); }
    __device__ inline Cursor end() const { return Cursor{n_active + (has_shared ? 1 : 0), 0}; }
    __device__ inline void advance(Cursor &c) const
    {
        if (++c.chunk == cpe(c.slot)) { c.slot++; c.chunk = 0; }
    }
    __device__ inline int index(Cursor c) const  // items before c
    {
        return c.slot <= n_active ? c.slot * cpe_r + c.chunk : n_active * cpe_r + cpe_s;
    }
    // first item whose starting cost position is >= p
    __device__ inline Cursor find(long p) const
    {
        if (p >= total_cost()) return end();
        const long rc = routed_cost();
        if (p >= rc) {
            const int chunk = (int)((p - rc + cost_shared - 1) / cost_shared);
            return chunk >= cpe_s ? end() : Cursor{n_active, chunk};
        }
        int lo = 0, hi = n_active - 1;  // largest slot with cpe_r * prefix[slot] <= p
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if ((long)cpe_r * prefix[mid] <= p) lo = mid; else hi = mid - 1;
        }
        const int c = prefix[lo + 1] - prefix[lo];
        const int chunk = (int)((p - (long)cpe_r * prefix[lo] + c - 1) / c);
        if (chunk < cpe_r) return Cursor{lo, chunk};
        return lo + 1 < n_active || has_shared ? Cursor{lo + 1, 0} : end();
    }
};

__device__ inline uint8_t *ring_stage(uint8_t *base, int s, int stride) { return base + 128 + s * stride; }
__device__ inline uint64_t *ring_full(uint8_t *base, int s) { return reinterpret_cast<uint64_t *>(base) + s; }
__device__ inline uint64_t *ring_empty(uint8_t *base, int s) { return reinterpret_cast<uint64_t *>(base) + NSTAGE + s; }

// After its last copy a producer waits (bounded) until the copies still in flight have landed, so
// that no asynchronous write can reach shared memory after the CTA has left.
__device__ inline void drain_ring(uint8_t *ring, int issued, uint32_t max_polls = (1u << 20))
{
    for (int it = issued > NSTAGE ? issued - NSTAGE : 0; it < issued; it++)
        mbar_wait(ring_full(ring, it % NSTAGE), (uint32_t)(it / NSTAGE) & 1, max_polls);
}

// The producer's side of the ring: issues the bulk copies of its next item once the compute
// warps have released the slot's previous contents.
template <int DT_R, int DT_S1, int NMAT> struct Producer {
    using CR = Cfg<DT_R, NMAT>;
    using CS = Cfg<DT_S1, NMAT>;
    const GemvArgs &A;
    const Plan &plan;
    uint8_t *ring;
    Cursor cur;
    int issued, n_items;

    __device__ inline bool issue_next()
    {
        if (issued >= n_items) return true;
        const int it = issued++;
        const int s = it % NSTAGE;
        const uint32_t use = (uint32_t)(it / NSTAGE);
        // the slot must have been released, and its previous copy must have landed: warps that gave up waiting
        // release slots early, and a barrier must not be armed twice in one phase
        if (use > 0 && !(mbar_wait(ring_empty(ring, s), (use - 1) & 1) && mbar_wait(ring_full(ring, s), (use - 1) & 1))) {
            set_status(A.status, PMOE_ERR_TIMEOUT, 20 + NMAT, it);
            return false;
        }
        const uint8_t *src0, *src1;
        uint32_t bytes;
        if (cur.slot < plan.n_active) {
            const size_t off = (size_t)A.g.active[cur.slot] * A.expert_bytes + (size_t)cur.chunk * CR::ITEM_BYTES;
            src0 = A.w0 + off;
            src1 = A.w1 + off;
            bytes = CR::ITEM_BYTES;
        } else {
            const size_t off = (size_t)cur.chunk * CS::ITEM_BYTES;
            src0 = A.sw0 + off;
            src1 = A.sw1 + off;
            bytes = CS::ITEM_BYTES;
        }
        const bool padded = cur.slot >= plan.n_active && plan.shared_mma && SharedMma<NMAT>::PER_ROW_COPIES;
        plan.advance(cur);
        uint64_t *full = ring_full(ring, s);
        mbar_expect_tx(full, bytes * NMAT);
        if (padded) {  // rows land SharedMma::PITCH apart: gate rows first, then the up rows
            constexpr int RB = Cfg<PMOE_Q8_0, NMAT>::ROW_BYTES, ROWS = Cfg<PMOE_Q8_0, NMAT>::ROWS;
#pragma unroll
            for (int mat = 0; mat < NMAT; mat++)
                for (int r = 0; r < ROWS; r++)
                    bulk_g2s(ring_stage(ring, s, A.stage_bytes) + (mat * ROWS + r) * SharedMma<NMAT>::PITCH,
                             (mat == 0 ? src0 : src1) + r * RB, RB, full);
            return true;
        }
#pragma unroll
        for (int mat = 0; mat < NMAT; mat++) {
            const uint8_t *src = mat == 0 ? src0 : src1;
            uint8_t *dst = ring_stage(ring, s, A.stage_bytes) + mat * bytes;
            for (uint32_t off = 0; off < bytes; off += BULK_PIECE)
                bulk_g2s(dst + off, src + off, bytes - off < (uint32_t)BULK_PIECE ? bytes - off : (uint32_t)BULK_PIECE,
                         full);
        }
        return true;
    }
};

// One pass with the arithmetic compiled for the number of tokens actually present (1, 2 or up to TGK).
template <int DT, int NMAT>
__device__ inline void run_pass(const GemvArgs &A, const uint8_t *stage, int chunk, const Pass &P,
                                const typename Tr<DT>::Act (&act)[Cfg<DT, NMAT>::UPL][Cfg<DT, NMAT>::TGK],
                                const typename Dot<DT>::Pre (&pre)[Cfg<DT, NMAT>::UPL], int warp, int lane)
{
    using C = Cfg<DT, NMAT>;
    if (P.cnt == 1) compute_item<DT, NMAT, 1>(A, stage, chunk, P, act, pre, warp, lane);
    else if (P.cnt == 2 || C::TGK == 2) compute_item<DT, NMAT, 2>(A, stage, chunk, P, act, pre, warp, lane);
    else compute_item<DT, NMAT, C::TGK>(A, stage, chunk, P, act, pre, warp, lane);  // 3 tokens: the 4th slot is zero
}

// Called by the eight compute warps when they leave a slot: adds the items this CTA finished to the slot's
// counter; the CTA that brings it to `cpe` (all rows of the expert's activation are in memory) quantises those
// rows for the down projection.  Writers fence before the counter update, the reader after it.
// The shared expert's rows may be finished tile by tile: `first` is the first of the m tokens then.
__device__ inline void finish_slot(const GemvArgs &A, int counter_idx, int items, int cpe, bool is_shared,
                                   const int *list, int m, int warp, int lane, int first = 0)
{
    __shared__ int s_last;
    if (A.debug == 4) return;
    asm volatile("bar.sync 2, 256;" ::: "memory");
    if (warp == 0 && lane == 0) {
        __threadfence();
        const int old = atomicAdd(&A.slot_done[counter_idx], items);
        s_last = old + items == cpe;
        if (s_last) A.slot_done[counter_idx] = 0;
    }
    asm volatile("bar.sync 2, 256;" ::: "memory");
    if (!s_last || A.debug == 3) return;
    __threadfence();
    const int dt = is_shared ? A.quant_dt_s : A.quant_dt_r;
    const bool kq = is_kquant(dt);
    for (int i = warp; i < m; i += GEMV_WARPS) {
        const size_t r = is_shared ? (size_t)A.n * A.top_k + A.sh_begin + first + i : (size_t)list[i];
        if (A.rows_total == 512) warp_quant_row512(A.out + r * 512, kq, A.q8k_out, A.q80_out, r, lane);
        else block_quant_row(A.out + r * A.rows_total, A.rows_total, kq, !kq, A.q8k_out, A.q80_out, r, 0, 1, lane);
    }
}

// The CTA's items of one kind (routed or shared), consumed in order from `cur` while the slot
// stays below `slot_end`.  `it` numbers the CTA's items; the ring position follows from it.
template <int DT, int NMAT>
__device__ inline bool run_items(const GemvArgs &A, uint8_t *ring, const Plan &plan, bool is_shared, Cursor &cur,
                                 int slot_end, int &it, int n_items, const QAct &in, int warp, int lane)
{
    using C = Cfg<DT, NMAT>;
    using Act = typename Tr<DT>::Act;
    const int ul = lane % C::LPR;
    const int cpe_of = is_shared ? plan.cpe_s : plan.cpe_r;
    int cur_slot = -1, m = 0;
    const int *list = nullptr;
    Pass P;
    Act act[C::UPL][C::TGK];
    typename Dot<DT>::Pre pre[C::UPL];
#pragma unroll
    for (int i = 0; i < C::UPL; i++) pre[i] = Dot<DT>::pre(i * C::LPR + ul);
    const bool fuse_quant = NMAT == 2 && (is_shared ? A.quant_dt_s : A.quant_dt_r) != 0;
    int items_in_slot = 0;
    bool failed = false;
    while (it < n_items && cur.slot < slot_end) {
        const int s = it % NSTAGE;
        const uint32_t use = (uint32_t)(it / NSTAGE);
        if (cur.slot != cur_slot) {
            if (fuse_quant && cur_slot >= 0)
                finish_slot(A, is_shared ? plan.n_active : cur_slot, items_in_slot, cpe_of, is_shared, list, m, warp, lane);
            items_in_slot = 0;
            cur_slot = cur.slot;
            if (is_shared) {
                m = A.sh_count;
            } else {
                const int e = A.g.active[cur.slot];
                m = A.g.count[e];
                list = A.g.pairs + A.g.offset[e];
            }
            if (m <= C::TGK) load_pass<DT, NMAT>(A, is_shared, list, m, 0, in, ul, P, act);
        }
        // a wait that runs out is recorded and the warp keeps walking its items without computing,
        // so that the barriers it shares with the other warps still see it
        if (!failed && A.debug != 2 && !mbar_wait(ring_full(ring, s), use & 1)) {
            set_status(A.status, PMOE_ERR_TIMEOUT, 10 + NMAT, it);
            failed = true;
        }
        const uint8_t *stage = ring_stage(ring, s, A.stage_bytes);
        if (A.debug == 1 || failed) {
        } else if (m <= C::TGK) {
            run_pass<DT, NMAT>(A, stage, cur.chunk, P, act, pre, warp, lane);
        } else {
            for (int t0 = 0; t0 < m; t0 += C::TGK) {
                load_pass<DT, NMAT>(A, is_shared, list, m, t0, in, ul, P, act);
                run_pass<DT, NMAT>(A, stage, cur.chunk, P, act, pre, warp, lane);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(ring_empty(ring, s));
        plan.advance(cur);
        it++;
        items_in_slot++;
    }
    if (fuse_quant && cur_slot >= 0)
        finish_slot(A, is_shared ? plan.n_active : cur_slot, items_in_slot, cpe_of, is_shared, list, m, warp, lane);
    return !failed;
}

// ---------------------------------------------------------------- shared expert over many tokens
// A Q8_0 shared expert that serves SHARED_MMA_MIN tokens or more runs its items as int8 tensor-core
// tiles instead of per-token dp4a passes: an item's rows are the M side (gate rows 0..7 and up rows
// 8..15 of one 16-row tile, or ROWS/16 tiles of down rows), eight tokens are the N side and one
// Q8_0 block (32 weights) is the K of one mma.  The integer block sum is exact, so every block
// contributes (d_w * d_x) * isum in f32 exactly as in the dp4a path; blocks are added in K order.
constexpr int SHARED_MMA_MIN = 24;

__device__ inline void mma_s8_16x8x32(int (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(0));
}

// Cost of one shared item in units of one dp4a pass over an item, for the work partition.
template <int NMAT> __host__ __device__ inline int shared_mma_cost(int tokens)
{
    using C = Cfg<PMOE_Q8_0, NMAT>;
    constexpr int MT = NMAT == 2 ? 1 : C::ROWS / 16;
    const int jobs = MT * ((tokens + 7) / 8);
    const int per_warp = (jobs + GEMV_WARPS - 1) / GEMV_WARPS;
    // measured at 64 tokens: the 64 blocks a warp walks per item take about as long as eight dp4a
    // passes (the activation fragments come from L2 under the weight stream's load)
    const int c = per_warp * (C::K / QK8_0) / 8;
    return c < 1 ? 1 : c;
}

// Activations of four consecutive blocks for one lane: its 8 bytes of each block of token column g
// and the block scales of token columns 2t and 2t+1.
struct MmaActs {
    uint2 q[4];
    float4 x0, x1;
};

__device__ inline void mma_load_acts(MmaActs &o, const int8_t *xq, const float *dx0, const float *dx1, int kb)
{
#pragma unroll
    for (int i = 0; i < 4; i++) o.q[i] = *reinterpret_cast<const uint2 *>(xq + (kb + i) * QK8_0);
    o.x0 = *reinterpret_cast<const float4 *>(dx0 + kb);
    o.x1 = *reinterpret_cast<const float4 *>(dx1 + kb);
}

// Bytes [8t, 8t+8) of the quants of block kb of one row, as two words.  The quants start 2 bytes
// into a 34-byte block, so the address is 4-byte aligned for odd kb only; even blocks take three
// aligned words and two funnel shifts.  ODD is a compile-time fact of the unrolled caller.
template <bool ODD> __device__ inline void mma_load_row(const uint8_t *q, uint32_t &w0, uint32_t &w1)
{
    if (ODD) {
        w0 = *reinterpret_cast<const uint32_t *>(q);
        w1 = *reinterpret_cast<const uint32_t *>(q + 4);
    } else {
        const uint32_t u0 = *reinterpret_cast<const uint32_t *>(q - 2);
        const uint32_t u1 = *reinterpret_cast<const uint32_t *>(q + 2);
        const uint32_t u2 = *reinterpret_cast<const uint32_t *>(q + 6);
        w0 = __funnelshift_r(u0, u1, 16);
        w1 = __funnelshift_r(u1, u2, 16);
    }
}

template <bool ODD>
__device__ inline void mma_step(const uint8_t *p0, const uint8_t *p1, int t, const uint2 &bq, float x0, float x1,
                                float (&acc)[4])
{
    uint32_t a[4];
    // the lane's share of K is bytes 8t..8t+7 of the block, for the weights and the activations alike
    mma_load_row<ODD>(p0 + 2 + 8 * t, a[0], a[2]);
    mma_load_row<ODD>(p1 + 2 + 8 * t, a[1], a[3]);
    const uint32_t b[2] = {bq.x, bq.y};
    int c[4];
    mma_s8_16x8x32(c, a, b);
    const float dw0 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(p0));
    const float dw1 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(p1));
    acc[0] += (dw0 * x0) * (float)c[0];
    acc[1] += (dw0 * x1) * (float)c[1];
    acc[2] += (dw1 * x0) * (float)c[2];
    acc[3] += (dw1 * x1) * (float)c[3];
}

__device__ inline void mma_step4(const uint8_t *r0, const uint8_t *r1, int kb, int t, const MmaActs &v, float (&acc)[4])
{
    // kb is a multiple of 4: blocks kb, kb+2 start 4-byte aligned (quants do not), kb+1, kb+3 the other way round
    mma_step<false>(r0 + (kb + 0) * Q8_0_BYTES, r1 + (kb + 0) * Q8_0_BYTES, t, v.q[0], v.x0.x, v.x1.x, acc);
    mma_step<true>(r0 + (kb + 1) * Q8_0_BYTES, r1 + (kb + 1) * Q8_0_BYTES, t, v.q[1], v.x0.y, v.x1.y, acc);
    mma_step<false>(r0 + (kb + 2) * Q8_0_BYTES, r1 + (kb + 2) * Q8_0_BYTES, t, v.q[2], v.x0.z, v.x1.z, acc);
    mma_step<true>(r0 + (kb + 3) * Q8_0_BYTES, r1 + (kb + 3) * Q8_0_BYTES, t, v.q[3], v.x0.w, v.x1.w, acc);
}

// job_lo / job_hi (hi < 0: none): the CTA's share of the jobs (16-row tile x 8-token tile) when the shared expert is
// split over the CTAs by jobs instead of whole items, numbered chunk * jobs_per_chunk + job over all chunks; an
// item may then be served by several CTAs, each taking its range of the item's jobs.
template <int NMAT>
__device__ inline bool run_items_shared_mma(const GemvArgs &A, uint8_t *ring, const Plan &plan, Cursor &cur, int &it,
                                            int n_items, const QAct &in, int warp, int lane, long job_lo = 0,
                                            long job_hi = -1)
{
    using C = Cfg<PMOE_Q8_0, NMAT>;
    using SM = SharedMma<NMAT>;
    constexpr int KB = SM::KB, MT = SM::MT, PITCH = SM::PITCH;
    const int g = lane >> 2, t = lane & 3;
    const int m = A.sh_count;
    const int ntiles = (m + 7) / 8;
    const size_t row0 = NMAT == 2 ? (size_t)A.sh_begin : (size_t)A.n * A.top_k + A.sh_begin;  // activation row of token 0
    const size_t out0 = (size_t)A.n * A.top_k + A.sh_begin;                                   // output row of token 0
    const bool fuse_quant = NMAT == 2 && A.quant_dt_s != 0;
    int items_in_slot = 0;
    bool failed = false;
    while (it < n_items && cur.slot <= plan.n_active) {
        const int s = it % NSTAGE;
        const uint32_t use = (uint32_t)(it / NSTAGE);
        if (!failed && A.debug != 2 && !mbar_wait(ring_full(ring, s), use & 1)) {
            set_status(A.status, PMOE_ERR_TIMEOUT, 14 + NMAT, it);
            failed = true;
        }
        const uint8_t *stage = ring_stage(ring, s, A.stage_bytes);
        if (A.debug != 1 && !failed) {
            int jb = 0, je = MT * ntiles;
            if (job_hi >= 0) {
                const long base = (long)cur.chunk * (MT * ntiles);
                jb = job_lo > base ? (int)(job_lo - base) : 0;
                je = job_hi - base < je ? (int)(job_hi - base) : je;
            }
            for (int job = jb + warp; job < je; job += GEMV_WARPS) {
                const int mt = job / ntiles, nt = job - mt * ntiles;
                // fragment rows g and g + 8 of the tile: gate row g and up row g, or two down rows
                const uint8_t *r0 = stage + (NMAT == 2 ? g : mt * 16 + g) * PITCH;
                const uint8_t *r1 = r0 + 8 * PITCH;
                // B column g = token nt*8 + g; C columns 2t, 2t+1 = tokens nt*8 + 2t (+1).  Columns past
                // the last token read token 0's rows; their sums are never stored.
                const int tok_b = nt * 8 + g, tok_c = nt * 8 + 2 * t;
                const bool c0_ok = tok_c < m, c1_ok = tok_c + 1 < m;
                const int8_t *xq = in.qs + (row0 + (tok_b < m ? tok_b : 0)) * C::K + 8 * t;
                const float *dx0 = in.d + (row0 + (c0_ok ? tok_c : 0)) * KB;
                const float *dx1 = in.d + (row0 + (c1_ok ? tok_c + 1 : 0)) * KB;
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                MmaActs va, vb;
                mma_load_acts(va, xq, dx0, dx1, 0);
#pragma unroll 1
                for (int kb = 0; kb < KB; kb += 8) {   // the loads of the next four blocks fly under the current four
                    mma_load_acts(vb, xq, dx0, dx1, kb + 4);
                    mma_step4(r0, r1, kb, t, va, acc);
                    if (kb + 8 < KB) mma_load_acts(va, xq, dx0, dx1, kb + 8);
                    mma_step4(r0, r1, kb + 4, t, vb, acc);
                }
                if (NMAT == 2) {
                    const int row = cur.chunk * C::ROWS + g;
                    const float v0 = acc[0] / (1.f + expf(-acc[0])) * acc[2];  // silu(gate) * up
                    const float v1 = acc[1] / (1.f + expf(-acc[1])) * acc[3];
                    if (c0_ok) A.out[(out0 + tok_c) * A.rows_total + row] = v0;
                    if (c1_ok) A.out[(out0 + tok_c + 1) * A.rows_total + row] = v1;
                } else {
                    const int row = cur.chunk * C::ROWS + mt * 16 + g;
                    if (c0_ok) {
                        const float sc = A.scale_s[A.sh_begin + tok_c];
                        float *o = A.out + (out0 + tok_c) * A.rows_total + row;
                        o[0] = acc[0] * sc;
                        o[8] = acc[2] * sc;
                    }
                    if (c1_ok) {
                        const float sc = A.scale_s[A.sh_begin + tok_c + 1];
                        float *o = A.out + (out0 + tok_c + 1) * A.rows_total + row;
                        o[0] = acc[1] * sc;
                        o[8] = acc[3] * sc;
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(ring_empty(ring, s));
        plan.advance(cur);
        it++;
        items_in_slot++;
    }
    if (fuse_quant && job_hi >= 0) {
        // split by jobs: every 8-token tile has its own counter (behind the per-expert ones), and the CTA that
        // completes a tile's last chunk re-quantises those eight rows -- no CTA is left with all the rows at the end
        for (int nt = 0; nt < ntiles; nt++) {
            const long cmin = job_lo > nt ? (job_lo - nt + ntiles - 1) / ntiles : 0;
            const long cmax = job_hi - 1 >= nt ? (job_hi - 1 - nt) / ntiles : -1;
            if (cmax < cmin) continue;
            const int rows = m - 8 * nt < 8 ? m - 8 * nt : 8;
            finish_slot(A, A.e_local + 1 + nt, (int)(cmax - cmin + 1), plan.cpe_s, true, nullptr, rows, warp, lane, 8 * nt);
        }
    } else if (fuse_quant && items_in_slot > 0) {
        finish_slot(A, plan.n_active, items_in_slot, plan.cpe_s, true, nullptr, m, warp, lane);
    }
    return !failed;
}


// pmoe_gemv_mma.cu
cudaError_t launch_gate_up_q4k_mma(GemvArgs &A, int dt_s, cudaStream_t s);
cudaError_t launch_down_q6k_mma(GemvArgs &A, int dt_s, cudaStream_t s);
bool mma_enabled(int kernel);   // 1: Q4_K gate/up, 2: Q6_K down
int sm_count();

}  // namespace pmoe
