// Decode path of the MoE block: expert-grouped, dequant-fused GEMV kernels over raw GGUF
// Q4_K / Q6_K / Q8_0 blocks.
//
//   k_expert_gemv<.., NMAT=2>  gate and up projections of every selected expert (and of the
//                              shared expert) with silu(gate)*up fused in
//   k_act_quant                re-quantises the activated rows for the down projection
//   k_expert_gemv<.., NMAT=1>  down projection scaled by the routing weight / shared gate
//   k_combine                  sums each token's rows in slot order, adds the shared expert
//
// Reference semantics: MoeExperts::forward_batched (paramecia-model/src/qwen3_next.rs:1347-1394),
// process_single_expert_optimized (paramecia-model/src/tokio_experts.rs:157-204),
// SharedExpert::forward (qwen3_next.rs:1776-1823) and the final add (1932-1937).  The numbers
// follow the reference CPU path: activations quantised to Q8_K / Q8_0, integer block dot
// products, f32 scales and accumulation.
//
// The expert kernels are persistent: two CTAs per SM, each taking a contiguous range of
// work items (an item = a few rows of one selected expert's matrix, ~36 KB).  One elected
// thread streams the items through a three-stage shared-memory ring with bulk (TMA) copies,
// so every weight byte crosses HBM once in contiguous 16-byte-aligned runs and two stages
// are always in flight while the warps work on the third.  A lane owns a fixed slice of
// the reduction dimension: the quantised activations of the expert's tokens stay in its
// registers across all rows of the expert, and the partial sums of several rows and tokens
// meet in one transposed shuffle reduction.
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
__device__ inline void drain_ring(uint8_t *ring, int issued)
{
    for (int it = issued > NSTAGE ? issued - NSTAGE : 0; it < issued; it++)
        mbar_wait(ring_full(ring, it % NSTAGE), (uint32_t)(it / NSTAGE) & 1);
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
        if (use > 0 && !mbar_wait(ring_empty(ring, s), (use - 1) & 1)) {
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
__device__ inline void finish_slot(const GemvArgs &A, int counter_idx, int items, int cpe, bool is_shared,
                                   const int *list, int m, int warp, int lane)
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
        const size_t r = is_shared ? (size_t)A.n * A.top_k + A.sh_begin + i : (size_t)list[i];
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

template <int NMAT>
__device__ inline bool run_items_shared_mma(const GemvArgs &A, uint8_t *ring, const Plan &plan, Cursor &cur, int &it,
                                            int n_items, const QAct &in, int warp, int lane)
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
            for (int job = warp; job < MT * ntiles; job += GEMV_WARPS) {
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
    if (fuse_quant && items_in_slot > 0)
        finish_slot(A, plan.n_active, items_in_slot, plan.cpe_s, true, nullptr, m, warp, lane);
    return !failed;
}

// DT_S == 0 compiles the kernel without a shared-expert branch.
template <int DT_R, int DT_S, int NMAT>
__global__ void __launch_bounds__(GEMV_THREADS, 2) k_expert_gemv(const GemvArgs A)
{
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ int s_prefix[1025];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Gate/up follows the grouping kernel and needs its lists at once.  The down kernel follows
    // gate/up (or the re-quantisation), which called pdl_launch_dependents() after its own wait:
    // the lists are complete by then, so the down kernel plans and its producer starts to stream
    // weights while the predecessor still runs; only the compute warps wait, for the activations.
    if (NMAT == 2) pdl_wait();
    pdl_launch_dependents();

    constexpr int DT_S1 = DT_S ? DT_S : DT_R;
    using CR = Cfg<DT_R, NMAT>;
    using CS = Cfg<DT_S1, NMAT>;
    Plan plan;
    plan.n_active = A.routed ? *A.g.n_active : 0;
    plan.has_shared = (DT_S != 0 && A.has_shared) ? 1 : 0;
    plan.cpe_r = A.rows_total / CR::ROWS;
    plan.cpe_s = A.rows_total / CS::ROWS;
    const bool shared_mma = DT_S == PMOE_Q8_0 && A.sh_count >= SHARED_MMA_MIN;
    plan.shared_mma = shared_mma;
    plan.cost_shared = shared_mma ? shared_mma_cost<NMAT>(A.sh_count) : (A.sh_count + CS::TGK - 1) / CS::TGK;
    plan.prefix = s_prefix;
    for (int i = threadIdx.x; i <= plan.n_active; i += GEMV_THREADS) s_prefix[i] = plan.n_active ? (CR::TGK == GEMV_TG ? A.g.cost_prefix[i] : A.g.cost_prefix_wide[i]) : 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(ring_full(ring, s), 1);
            mbar_init(ring_empty(ring, s), GEMV_WARPS);
        }
        fence_mbar_init();
    }
    __syncthreads();

    const long total = plan.total_cost();
    Cursor cur = plan.find(total * blockIdx.x / gridDim.x);
    const Cursor last = plan.find(total * (blockIdx.x + 1) / gridDim.x);
    const int n_items = plan.index(last) - plan.index(cur);
    if (n_items <= 0) return;

    if (warp == GEMV_WARPS) {  // the producer warp: one lane keeps the ring full
        if (lane == 0 && A.debug != 2) {
            Producer<DT_R, DT_S1, NMAT> prod{A, plan, ring, cur, 0, n_items};
            for (int i = 0; i < n_items; i++)
                if (!prod.issue_next()) { prod.issued--; break; }   // the item whose slot never came free was not issued
            drain_ring(ring, prod.issued);
        }
        return;
    }
    if (NMAT == 1) pdl_wait();
    int it = 0;
    bool ok = run_items<DT_R, NMAT>(A, ring, plan, false, cur, plan.n_active, it, n_items, A.in_r, warp, lane);
    if constexpr (DT_S != 0) {
        if (!ok) return;
        if (DT_S == PMOE_Q8_0 && shared_mma) run_items_shared_mma<NMAT>(A, ring, plan, cur, it, n_items, A.in_s, warp, lane);
        else run_items<DT_S, NMAT>(A, ring, plan, true, cur, plan.n_active + 1, it, n_items, A.in_s, warp, lane);
    }
}

// ---------------------------------------------------------------- Q4_K gate/up on the tensor cores
// The same gate/up step for Q4_K routed experts with the dot products on the tensor cores
// (mma.sync.m16n8k32, u8 weights x s8 activations -> s32): sixteen weight rows are the M side, up to
// eight tokens of the expert the N side, and one 32-weight sub-block -- the span of one 6-bit
// scale -- the K of one instruction, so the integer sub-block sums are exact and meet their scales
// as integers exactly like the dp4a path.  One instruction replaces 16 x tokens dp4a, and no
// shuffle reduction over the reduction dimension is left.
//
// An item is still 16 gate + 16 up rows of one expert, but a slot with more than eight tokens is
// walked once per group of eight (the ring delivers its items again, from L2).  Warp w of the eight
// compute warps owns block column w of all 32 rows (K = 2048 = 8 blocks), so the eight tokens'
// quantised activations of that column stay in 16 registers per lane for the whole expert.  The
// mins term sum_j m_j * bsum_j goes through two more instructions over the partial sums split into
// signed byte digits (bsum = 64 h + l).  The eight warps' partial sums meet in shared memory, in
// the part of the ring slot the warp itself has finished reading, and are added in warp order.
//
// Rows land in shared memory 1168 bytes apart (1152 + 16): with rows 0,2,4,6 / 1,3,5,7 on the
// eight row positions of a fragment the 8-byte loads of a half-warp fall into 32 different banks.
constexpr int Q4K_ROW = 8 * Q4_K_BYTES;                 // 1152: one row of K = 2048
constexpr int Q4K_MMA_PITCH = Q4K_ROW + 16;
constexpr int MMA_STAGE_BYTES = 32 * Q4K_MMA_PITCH;     // 37 376
static_assert(MMA_STAGE_BYTES % 128 == 0 && MMA_STAGE_BYTES >= STAGE_BYTES, "ring slot of the tensor-core GEMV");

__device__ inline void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                    uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Items of the tensor-core kernel, in order: (slot, token group, chunk), chunk fastest.  Every item
// costs the same, so a CTA takes an equal share of the item count.
struct MmaCursor {
    int slot, group, chunk, groups;   // groups = token groups of `slot`
};

struct MmaWork {
    int n_active, cpe, groups_sh;   // groups_sh = 0 when the shared expert is not served by these items
    const int *prefix;              // [n_active + 1] exclusive prefix of ceil(count / 8) over the active slots (global)

    __device__ inline int routed_groups() const { return n_active ? prefix[n_active] : 0; }
    __device__ inline long total() const { return (long)cpe * (routed_groups() + groups_sh); }
    __device__ inline MmaCursor at(long q) const
    {
        const int G = (int)(q / cpe), chunk = (int)(q % cpe);
        const int rg = routed_groups();
        if (G >= rg) return MmaCursor{n_active, G - rg, chunk, groups_sh};
        int lo = 0, hi = n_active - 1;   // largest slot with prefix[slot] <= G
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (prefix[mid] <= G) lo = mid; else hi = mid - 1;
        }
        return MmaCursor{lo, G - prefix[lo], chunk, prefix[lo + 1] - prefix[lo]};
    }
    __device__ inline void advance(MmaCursor &c) const
    {
        if (++c.chunk < cpe) return;
        c.chunk = 0;
        if (++c.group < c.groups) return;
        c.group = 0;
        c.slot++;
        c.groups = c.slot < n_active ? prefix[c.slot + 1] - prefix[c.slot] : groups_sh;
    }
};

struct Q4Hdr {
    float d16, dmin;              // d / 16 (high nibbles stay in place) and dmin
    uint32_t sca, scb, mna, mnb;  // 6-bit scales 0..3 / 4..7 and mins 0..3 / 4..7 as bytes
};

__device__ inline Q4Hdr q4k_hdr(const uint4 h)
{
    Q4Hdr o;
    o.d16 = half_bits_to_float((uint16_t)(h.x & 0xffffu)) * 0.0625f;
    o.dmin = half_bits_to_float((uint16_t)(h.x >> 16));
    o.sca = h.y & 0x3F3F3F3Fu;
    o.mna = h.z & 0x3F3F3F3Fu;
    o.scb = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
    o.mnb = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    return o;
}

// byte `i` (compile-time) of w, zero-extended
template <int I> __device__ inline int byte_of(uint32_t w) { return (int)__byte_perm(w, 0u, 0x4440u + I); }

// The compute warps' side: items [it, n_items) of this CTA starting at `cur`.
__device__ inline bool run_items_q4k_mma(const GemvArgs &A, uint8_t *ring, const MmaWork &work, MmaCursor cur, int n_items,
                                         int &it, int warp, int lane)
{
    const int g = lane >> 2, t = lane & 3;
    const int r0 = ((g & 3) << 1) | (g >> 2);   // tile row under fragment row g (fragment row g + 8: tile row r0 + 8)
    // this thread's share of the cross-warp sum: value (matrix rmt, fragment lane rsrc, register ri)
    const int rq = warp * 16 + (lane & 15), rmt = lane >> 4;
    const int rsrc = rq >> 2, ri = rq & 3;
    const int rg = rsrc >> 2, rt = rsrc & 3;
    const int r_row = (((rg & 3) << 1) | (rg >> 2)) + ((ri & 2) ? 8 : 0);
    const int r_tok = 2 * rt + (ri & 1);
    const uint32_t part_wr = (uint32_t)((lane >> 3) * Q4K_MMA_PITCH + Q4_K_BYTES * warp + (lane & 7) * 16);
    const uint32_t part_rd = (uint32_t)((rmt * 4 + (rsrc >> 3)) * Q4K_MMA_PITCH + (rsrc & 7) * 16 + 4 * ri);

    uint32_t bq[8][2];   // token g: its 8 bytes of each sub-block of block column `warp`
    uint32_t bh = 0, bl = 0;
    float dx0 = 0.f, dx1 = 0.f;
    int r_orow = -1;
#pragma unroll
    for (int j = 0; j < 8; j++) bq[j][0] = bq[j][1] = 0;

    int cur_slot = -1, cur_group = -1, m = 0, items_in_slot = 0, slot_groups = 0;
    const int *list = nullptr;
    bool is_sh = false, failed = false;
    for (; it < n_items; it++) {
        const int s = it % NSTAGE;
        const uint32_t use = (uint32_t)(it / NSTAGE);
        if (cur.slot != cur_slot) {
            if (cur_slot >= 0 && (is_sh ? A.quant_dt_s : A.quant_dt_r) != 0)
                finish_slot(A, is_sh ? work.n_active : cur_slot, items_in_slot, work.cpe * slot_groups, is_sh, list, m, warp,
                            lane);
            items_in_slot = 0;
            cur_slot = cur.slot;
            cur_group = -1;
            slot_groups = cur.groups;
            is_sh = cur.slot >= work.n_active;
            if (is_sh) {
                m = A.sh_count;
                list = nullptr;
            } else {
                const int e = A.g.active[cur.slot];
                m = A.g.count[e];
                list = A.g.pairs + A.g.offset[e];
            }
        }
        if (cur.group != cur_group) {   // the group's tokens: fragments of their quantised rows
            cur_group = cur.group;
            const int t0 = 8 * cur.group;
            const int cnt = m - t0 < 8 ? m - t0 : 8;
            const QAct &in = is_sh ? A.in_s : A.in_r;
            bh = bl = 0;
            if (g < cnt) {
                const size_t row = is_sh ? (size_t)(A.sh_begin + t0 + g) : (size_t)(list[t0 + g] / A.top_k);
                const int8_t *xp = in.qs + row * 2048 + 256 * warp + 8 * t;
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const uint2 lo = *reinterpret_cast<const uint2 *>(xp + 64 * c);
                    const uint2 hi = *reinterpret_cast<const uint2 *>(xp + 64 * c + 32);
                    bq[2 * c][0] = lo.x; bq[2 * c][1] = lo.y;
                    bq[2 * c + 1][0] = hi.x; bq[2 * c + 1][1] = hi.y;
                }
                if (t < 2) {   // sums of the quants under sub-blocks 4t .. 4t+3, as two signed byte digits
                    const uint4 bs = *reinterpret_cast<const uint4 *>(in.bsums + row * 128 + 16 * warp + 8 * t);
                    const uint32_t w4[4] = {bs.x, bs.y, bs.z, bs.w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int v = (int)(int16_t)(w4[i] & 0xffffu) + (int)(int16_t)(w4[i] >> 16);
                        bh |= (uint32_t)((v >> 6) & 0xFF) << (8 * i);
                        bl |= (uint32_t)(v & 63) << (8 * i);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) bq[j][0] = bq[j][1] = 0;
            }
            dx0 = dx1 = 0.f;
            if (2 * t < cnt) {
                const size_t row = is_sh ? (size_t)(A.sh_begin + t0 + 2 * t) : (size_t)(list[t0 + 2 * t] / A.top_k);
                dx0 = in.d[row * 8 + warp];
            }
            if (2 * t + 1 < cnt) {
                const size_t row = is_sh ? (size_t)(A.sh_begin + t0 + 2 * t + 1) : (size_t)(list[t0 + 2 * t + 1] / A.top_k);
                dx1 = in.d[row * 8 + warp];
            }
            r_orow = -1;
            if (r_tok < cnt) r_orow = is_sh ? A.n * A.top_k + A.sh_begin + t0 + r_tok : list[t0 + r_tok];
        }
        // a wait that runs out is recorded; the warp keeps walking its items (and meeting the barriers
        // it shares with the other warps) without computing
        if (!failed && A.debug != 2 && !mbar_wait(ring_full(ring, s), use & 1)) {
            set_status(A.status, PMOE_ERR_TIMEOUT, 18, it);
            failed = true;
        }
        uint8_t *stage = ring_stage(ring, s, A.stage_bytes);
        const bool compute = !failed && A.debug != 1;
        float acc[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
#pragma unroll
            for (int i = 0; i < 4; i++) acc[mt][i] = 0.f;
            if (!compute) continue;
            const uint8_t *p0 = stage + (mt * 16 + r0) * Q4K_MMA_PITCH + Q4_K_BYTES * warp;
            const uint8_t *p1 = p0 + 8 * Q4K_MMA_PITCH;
            const Q4Hdr h0 = q4k_hdr(*reinterpret_cast<const uint4 *>(p0));
            const Q4Hdr h1 = q4k_hdr(*reinterpret_cast<const uint4 *>(p1));
            int ie[4] = {0, 0, 0, 0}, io[4] = {0, 0, 0, 0};   // even (low-nibble) and odd (high-nibble, x16) sub-blocks
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint2 q0 = *reinterpret_cast<const uint2 *>(p0 + 16 + 32 * c + 8 * t);
                const uint2 q1 = *reinterpret_cast<const uint2 *>(p1 + 16 + 32 * c + 8 * t);
                const uint32_t sw0 = c < 2 ? h0.sca : h0.scb, sw1 = c < 2 ? h1.sca : h1.scb;
                int cc[4];
                mma_u8s8_k32(cc, q0.x & 0x0F0F0F0Fu, q1.x & 0x0F0F0F0Fu, q0.y & 0x0F0F0F0Fu, q1.y & 0x0F0F0F0Fu, bq[2 * c][0],
                             bq[2 * c][1]);
                {
                    const int s0 = (c & 1) ? byte_of<2>(sw0) : byte_of<0>(sw0);
                    const int s1 = (c & 1) ? byte_of<2>(sw1) : byte_of<0>(sw1);
                    ie[0] += cc[0] * s0; ie[1] += cc[1] * s0; ie[2] += cc[2] * s1; ie[3] += cc[3] * s1;
                }
                mma_u8s8_k32(cc, q0.x & 0xF0F0F0F0u, q1.x & 0xF0F0F0F0u, q0.y & 0xF0F0F0F0u, q1.y & 0xF0F0F0F0u,
                             bq[2 * c + 1][0], bq[2 * c + 1][1]);
                {
                    const int s0 = (c & 1) ? byte_of<3>(sw0) : byte_of<1>(sw0);
                    const int s1 = (c & 1) ? byte_of<3>(sw1) : byte_of<1>(sw1);
                    io[0] += cc[0] * s0; io[1] += cc[1] * s0; io[2] += cc[2] * s1; io[3] += cc[3] * s1;
                }
            }
            // mins: K positions 0..7 carry m_0..m_7 (lanes t = 0, 1), the rest is zero
            const uint32_t am0 = t == 0 ? h0.mna : (t == 1 ? h0.mnb : 0u);
            const uint32_t am1 = t == 0 ? h1.mna : (t == 1 ? h1.mnb : 0u);
            int ch[4], cl[4];
            mma_u8s8_k32(ch, am0, am1, 0u, 0u, bh, 0u);
            mma_u8s8_k32(cl, am0, am1, 0u, 0u, bl, 0u);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const Q4Hdr &h = i < 2 ? h0 : h1;
                const float dx = (i & 1) ? dx1 : dx0;
                acc[mt][i] = dx * (h.d16 * (float)(16 * ie[i] + io[i]) - h.dmin * (float)(64 * ch[i] + cl[i]));
            }
        }
        // partial sums of this warp's block column into its own part of rows 0..7 of the slot
        __syncwarp();
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
            *reinterpret_cast<float4 *>(stage + part_wr + mt * 4 * Q4K_MMA_PITCH) =
                make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
        asm volatile("bar.sync 1, 256;" ::: "memory");
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < GEMV_WARPS; w++) v += *reinterpret_cast<const float *>(stage + part_rd + Q4_K_BYTES * w);
        const float up = __shfl_xor_sync(0xffffffffu, v, 16);
        if (lane < 16 && r_orow >= 0 && compute)
            A.out[(size_t)r_orow * A.rows_total + cur.chunk * 16 + r_row] = v / (1.f + expf(-v)) * up;   // silu(gate) * up
        __syncwarp();
        if (lane == 0) mbar_arrive(ring_empty(ring, s));
        work.advance(cur);
        items_in_slot++;
    }
    if (cur_slot >= 0 && (is_sh ? A.quant_dt_s : A.quant_dt_r) != 0)
        finish_slot(A, is_sh ? work.n_active : cur_slot, items_in_slot, work.cpe * slot_groups, is_sh, list, m, warp, lane);
    return !failed;
}

// DT_S: type of the shared expert's gate/up matrices served by this launch (0 = none).  A Q4_K shared
// expert is one more slot of the tensor-core items; other types follow as items of the streaming kind.
template <int DT_S>
__global__ void __launch_bounds__(GEMV_THREADS, 2) k_gate_up_q4k_mma(const GemvArgs A)
{
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ int s_prefix1[2];
    __shared__ MmaCursor s_first;
    __shared__ int s_items;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    pdl_launch_dependents();

    MmaWork work;
    work.n_active = A.routed ? *A.g.n_active : 0;
    work.cpe = A.rows_total / 16;
    work.groups_sh = (DT_S == PMOE_Q4_K && A.has_shared) ? (A.sh_count + GEMV_TG_MMA - 1) / GEMV_TG_MMA : 0;
    work.prefix = A.g.cost_prefix_mma;
    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(ring_full(ring, s), 1);
            mbar_init(ring_empty(ring, s), GEMV_WARPS);
        }
        fence_mbar_init();
        const long total = work.total();
        const long q0 = total * blockIdx.x / gridDim.x, q1 = total * (blockIdx.x + 1) / gridDim.x;
        s_items = (int)(q1 - q0);
        s_first = q1 > q0 ? work.at(q0) : MmaCursor{0, 0, 0, 0};
        s_prefix1[0] = s_prefix1[1] = 0;
    }
    __syncthreads();
    const int n_mma = s_items;
    const MmaCursor first = s_first;

    // items of the streaming kind for a shared expert of another type: an equal share of their cost
    constexpr bool STREAM_SH = DT_S != 0 && DT_S != PMOE_Q4_K;
    constexpr int DT_S1 = STREAM_SH ? DT_S : PMOE_Q8_0;
    using CS = Cfg<DT_S1, 2>;
    Plan plan;
    Cursor scur{0, 0};
    int n_sh = 0;
    if (STREAM_SH && A.has_shared) {
        plan.n_active = 0;
        plan.has_shared = 1;
        plan.cpe_r = plan.cpe_s = A.rows_total / CS::ROWS;
        plan.shared_mma = DT_S == PMOE_Q8_0 && A.sh_count >= SHARED_MMA_MIN;
        plan.cost_shared = plan.shared_mma ? shared_mma_cost<2>(A.sh_count) : (A.sh_count + CS::TGK - 1) / CS::TGK;
        plan.prefix = s_prefix1;
        const long total = plan.total_cost();
        scur = plan.find(total * blockIdx.x / gridDim.x);
        const Cursor last = plan.find(total * (blockIdx.x + 1) / gridDim.x);
        n_sh = plan.index(last) - plan.index(scur);
    }
    if (n_mma + n_sh <= 0) return;

    if (warp == GEMV_WARPS) {   // the producer warp: every lane copies one row of an item
        if (A.debug == 2) return;
        MmaCursor pc = first;
        int issued = 0;
        bool ok = true;
        for (; issued < n_mma; issued++) {
            const int s = issued % NSTAGE;
            const uint32_t use = (uint32_t)(issued / NSTAGE);
            if (use > 0) {
                int w = 1;
                if (lane == 0) w = mbar_wait(ring_empty(ring, s), (use - 1) & 1) ? 1 : 0;
                w = __shfl_sync(0xffffffffu, w, 0);
                if (!w) {
                    if (lane == 0) set_status(A.status, PMOE_ERR_TIMEOUT, 23, issued);
                    ok = false;
                    break;
                }
            }
            const uint8_t *base;
            if (pc.slot < work.n_active) base = (lane < 16 ? A.w0 : A.w1) + (size_t)A.g.active[pc.slot] * A.expert_bytes;
            else base = lane < 16 ? A.sw0 : A.sw1;
            uint64_t *full = ring_full(ring, s);
            if (lane == 0) mbar_expect_tx(full, 32 * Q4K_ROW);
            __syncwarp();
            bulk_g2s(ring_stage(ring, s, A.stage_bytes) + lane * Q4K_MMA_PITCH,
                     base + (size_t)(pc.chunk * 16 + (lane & 15)) * Q4K_ROW, Q4K_ROW, full);
            work.advance(pc);
        }
        if (lane == 0) {
            if (STREAM_SH && ok && n_sh > 0) {
                Producer<DT_S1, DT_S1, 2> prod{A, plan, ring, scur, issued, n_mma + n_sh};
                for (int i = 0; i < n_sh; i++)
                    if (!prod.issue_next()) { prod.issued--; break; }
                issued = prod.issued;
            }
            drain_ring(ring, issued);
        }
        return;
    }
    int it = 0;
    bool ok = run_items_q4k_mma(A, ring, work, first, n_mma, it, warp, lane);
    if constexpr (STREAM_SH) {
        if (ok && n_sh > 0) {
            if (DT_S == PMOE_Q8_0 && plan.shared_mma)
                run_items_shared_mma<2>(A, ring, plan, scur, it, n_mma + n_sh, A.in_s, warp, lane);
            else
                run_items<DT_S1, 2>(A, ring, plan, true, scur, 1, it, n_mma + n_sh, A.in_s, warp, lane);
        }
    }
}

// ---------------------------------------------------------------- host-side dispatch
bool gemv_supported(int dtype, int K, int rows, const char **why)
{
    if (!(dtype >= PMOE_Q2_K && dtype <= PMOE_Q6_K) && dtype != PMOE_Q8_0) {
        *why = "expert weights must be Q2_K ... Q6_K or Q8_0";
        return false;
    }
    if (!((K == 2048 && rows == 512) || (K == 512 && rows == 2048))) {
        *why = "this build serves hidden 2048 with expert intermediate 512";
        return false;
    }
    return true;
}

static int g_sm_count = 0;

static int sm_count()
{
    if (!g_sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    return g_sm_count;
}

template <int DT_R, int DT_S, int NMAT>
static cudaError_t launch_gemv_t(const GemvArgs &A, cudaStream_t s)
{
    constexpr size_t smem = 128 + (size_t)NSTAGE * STAGE_BYTES;
    auto kern = k_expert_gemv<DT_R, DT_S, NMAT>;
    static bool configured = false;  // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    cudaError_t e = launch_pdl(kern, dim3(2 * sm_count()), dim3(GEMV_THREADS), smem, s, A);
    count_launch();
    return e;
}

template <int DT_R, int NMAT>
static cudaError_t launch_gemv_s(const GemvArgs &A, int dt_s, cudaStream_t s)
{
    switch (dt_s) {
    case 0: return launch_gemv_t<DT_R, 0, NMAT>(A, s);
    case PMOE_Q4_K: return launch_gemv_t<DT_R, PMOE_Q4_K, NMAT>(A, s);
    case PMOE_Q5_K: return launch_gemv_t<DT_R, PMOE_Q5_K, NMAT>(A, s);
    case PMOE_Q6_K:
        // a down matrix shared by three or more tokens: the four-tokens-per-pass variant
        if constexpr (NMAT == 1) {
            if (A.sh_count >= 3) return launch_gemv_t<DT_R, Q6_K_T4, NMAT>(A, s);
        }
        return launch_gemv_t<DT_R, PMOE_Q6_K, NMAT>(A, s);
    case PMOE_Q8_0: return launch_gemv_t<DT_R, PMOE_Q8_0, NMAT>(A, s);
    }
    return cudaErrorInvalidValue;
}

// Q2_K / Q3_K routed experts: the shared expert may be absent, of the same type, or Q4_K / Q6_K / Q8_0
// (pmoe_layer_create refuses the other pairings; this keeps the number of kernel variants bounded)
template <int DT_R, int NMAT>
static cudaError_t launch_gemv_s_low(const GemvArgs &A, int dt_s, cudaStream_t s)
{
    if (dt_s == DT_R) return launch_gemv_t<DT_R, DT_R, NMAT>(A, s);
    switch (dt_s) {
    case 0: return launch_gemv_t<DT_R, 0, NMAT>(A, s);
    case PMOE_Q4_K: return launch_gemv_t<DT_R, PMOE_Q4_K, NMAT>(A, s);
    case PMOE_Q6_K:
        if constexpr (NMAT == 1) {
            if (A.sh_count >= 3) return launch_gemv_t<DT_R, Q6_K_T4, NMAT>(A, s);
        }
        return launch_gemv_t<DT_R, PMOE_Q6_K, NMAT>(A, s);
    case PMOE_Q8_0: return launch_gemv_t<DT_R, PMOE_Q8_0, NMAT>(A, s);
    }
    return cudaErrorInvalidValue;
}

template <int NMAT>
static cudaError_t launch_gemv(const GemvArgs &A, int dt_r, int dt_s, cudaStream_t s)
{
    switch (dt_r) {
    case PMOE_Q2_K: return launch_gemv_s_low<PMOE_Q2_K, NMAT>(A, dt_s, s);
    case PMOE_Q3_K: return launch_gemv_s_low<PMOE_Q3_K, NMAT>(A, dt_s, s);
    case PMOE_Q4_K: return launch_gemv_s<PMOE_Q4_K, NMAT>(A, dt_s, s);
    case PMOE_Q5_K: return launch_gemv_s<PMOE_Q5_K, NMAT>(A, dt_s, s);
    case PMOE_Q6_K:
        // down projection of a call with more than about one token per expert: experts with
        // three or four tokens are common, and the variant that takes four per pass wins
        if constexpr (NMAT == 1) {
            if (A.routed && (long)A.n * A.top_k >= A.e_local) return launch_gemv_s<Q6_K_T4, NMAT>(A, dt_s, s);
        }
        return launch_gemv_s<PMOE_Q6_K, NMAT>(A, dt_s, s);
    case PMOE_Q8_0: return launch_gemv_s<PMOE_Q8_0, NMAT>(A, dt_s, s);
    }
    return cudaErrorInvalidValue;
}

template <int DT_S> static cudaError_t launch_q4k_mma_t(const GemvArgs &A, cudaStream_t s)
{
    constexpr size_t smem = 128 + (size_t)NSTAGE * MMA_STAGE_BYTES;
    auto kern = k_gate_up_q4k_mma<DT_S>;
    static bool configured = false;  // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    cudaError_t e = launch_pdl(kern, dim3(2 * sm_count()), dim3(GEMV_THREADS), smem, s, A);
    count_launch();
    return e;
}

// PMOE_MMA=0 in the environment keeps the dp4a kernels for Q4_K gate/up (comparison runs)
static bool mma_enabled()
{
    static const bool on = !(getenv("PMOE_MMA") && atoi(getenv("PMOE_MMA")) == 0);
    return on;
}

cudaError_t launch_gate_up(const LayerDev &L, const Workspace &ws, int n, int top_k, bool routed, bool shared,
                           cudaStream_t s)
{
    if (n <= 0 || (!routed && !shared)) return cudaSuccess;
    GemvArgs A{};
    A.w0 = L.gate_exps; A.w1 = L.up_exps;
    A.expert_bytes = row_bytes(L.gate_dtype, L.H) * L.F;
    A.sw0 = L.sh_gate; A.sw1 = L.sh_up;
    A.rows_total = L.F;
    A.e_local = L.E_local;
    A.routed = routed; A.has_shared = shared;
    A.n = n; A.top_k = top_k;
    A.sh_begin = ws.sh_begin; A.sh_count = ws.sh_count;
    A.g = ws.groups;
    A.in_r = is_kquant(L.gate_dtype) ? ws.x_q8k : ws.x_q80;
    A.in_s = is_kquant(L.sh_gate_dtype) ? ws.x_q8k : ws.x_q80;
    A.out = ws.act;
    A.status = ws.status;
    A.debug = getenv("PMOE_DEBUG") ? atoi(getenv("PMOE_DEBUG")) : 0;
    A.stage_bytes = STAGE_BYTES;
    A.slot_done = ws.slot_done;
    A.quant_dt_r = routed ? L.down_dtype : 0;
    A.quant_dt_s = shared ? L.sh_down_dtype : 0;
    A.q8k_out = ws.act_q8k;
    A.q80_out = ws.act_q80;
    if (routed && L.gate_dtype == PMOE_Q4_K && L.H == 2048 && L.F == 512 && mma_enabled()) {
        A.stage_bytes = MMA_STAGE_BYTES;
        switch (shared ? L.sh_gate_dtype : 0) {
        case 0: return launch_q4k_mma_t<0>(A, s);
        case PMOE_Q4_K: return launch_q4k_mma_t<PMOE_Q4_K>(A, s);
        case PMOE_Q5_K: return launch_q4k_mma_t<PMOE_Q5_K>(A, s);
        case PMOE_Q6_K: return launch_q4k_mma_t<PMOE_Q6_K>(A, s);
        case PMOE_Q8_0: return launch_q4k_mma_t<PMOE_Q8_0>(A, s);
        }
        A.stage_bytes = STAGE_BYTES;
    }
    // a kernel without routed items still needs a routed type to instantiate; reuse the shared one
    return launch_gemv<2>(A, routed ? L.gate_dtype : L.sh_gate_dtype, shared ? L.sh_gate_dtype : 0, s);
}

cudaError_t launch_down(const LayerDev &L, const Workspace &ws, const float *w, int n, int top_k, bool routed,
                        bool shared, cudaStream_t s)
{
    if (n <= 0 || (!routed && !shared)) return cudaSuccess;
    GemvArgs A{};
    A.w0 = L.down_exps; A.w1 = nullptr;
    A.expert_bytes = row_bytes(L.down_dtype, L.F) * L.H;
    A.sw0 = L.sh_down; A.sw1 = nullptr;
    A.rows_total = L.H;
    A.e_local = L.E_local;
    A.routed = routed; A.has_shared = shared;
    A.n = n; A.top_k = top_k;
    A.sh_begin = ws.sh_begin; A.sh_count = ws.sh_count;
    A.g = ws.groups;
    A.in_r = is_kquant(L.down_dtype) ? ws.act_q8k : ws.act_q80;
    A.in_s = is_kquant(L.sh_down_dtype) ? ws.act_q8k : ws.act_q80;
    A.out = ws.partial;
    A.scale_r = w;
    A.scale_s = ws.sh_sigmoid;
    A.status = ws.status;
    A.debug = getenv("PMOE_DEBUG") ? atoi(getenv("PMOE_DEBUG")) : 0;
    A.stage_bytes = STAGE_BYTES;
    return launch_gemv<1>(A, routed ? L.down_dtype : L.sh_down_dtype, shared ? L.sh_down_dtype : 0, s);
}

// ---------------------------------------------------------------- stand-alone quantised mat-mul
// QMatMul::forward for one quantised matrix: y[m, rows] = x[m, cols] * W[rows, cols]^T with the
// activations quantised to the weight type's dot type.  One warp per output row, weights read
// straight from global memory; meant for parity checks and small operands, not for the block.
__global__ void __launch_bounds__(64) k_quant_rows(const float *__restrict__ x, int K, bool kq, QAct a8k, QAct a80)
{
    block_quant_row(x + (size_t)blockIdx.x * K, K, kq, !kq, a8k, a80, (size_t)blockIdx.x, threadIdx.x >> 5, 2,
                    threadIdx.x & 31);
}

template <int DT>
__global__ void __launch_bounds__(128) k_qmatmul(const uint8_t *__restrict__ w, int rows, int K, QAct in, int m,
                                                 float *__restrict__ y)
{
    using Act = typename Tr<DT>::Act;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp;
    const int t0 = blockIdx.y * TG;
    if (row >= rows) return;
    const uint8_t *rp = w + (size_t)row * row_bytes(DT, K);
    float acc[TG];
#pragma unroll
    for (int t = 0; t < TG; t++) acc[t] = 0.f;
    for (int u = lane; u < K / Tr<DT>::UNIT; u += 32) {
        Act act[TG];
#pragma unroll
        for (int t = 0; t < TG; t++) {
            if (t0 + t < m) load_act<DT>(in, (size_t)(t0 + t), K, u, act[t]);
            else zero_act<DT>(act[t]);
        }
        const typename Dot<DT>::Pre pre = Dot<DT>::pre(u);
        Dot<DT>::template run<TG, false>(rp, pre, act, acc);
    }
#pragma unroll
    for (int t = 0; t < TG; t++) {
        float v = acc[t];
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
        if (lane == 0 && t0 + t < m) y[(size_t)(t0 + t) * rows + row] = v;
    }
}

cudaError_t launch_qmatmul(int dtype, const void *w, int rows, int K, const float *x, int m, float *y, void *scratch,
                           cudaStream_t s)
{
    // scratch layout: qs int8 [m,K] | d f32 [m, K/32] | bsums i16 [m, K/16]
    QAct a{};
    uint8_t *p = (uint8_t *)scratch;
    a.qs = (int8_t *)p;
    p += ((size_t)m * K + 255) / 256 * 256;
    a.d = (float *)p;
    p += ((size_t)m * (K / 32) * 4 + 255) / 256 * 256;
    a.bsums = (int16_t *)p;
    const bool kq = is_kquant(dtype);
    k_quant_rows<<<m, 64, 0, s>>>(x, K, kq, a, a);
    dim3 grid((rows + 3) / 4, (m + TG - 1) / TG);
    const uint8_t *wb = (const uint8_t *)w;
    if (dtype == PMOE_Q4_K) k_qmatmul<PMOE_Q4_K><<<grid, 128, 0, s>>>(wb, rows, K, a, m, y);
    else if (dtype == PMOE_Q2_K) k_qmatmul<PMOE_Q2_K><<<grid, 128, 0, s>>>(wb, rows, K, a, m, y);
    else if (dtype == PMOE_Q3_K) k_qmatmul<PMOE_Q3_K><<<grid, 128, 0, s>>>(wb, rows, K, a, m, y);
    else if (dtype == PMOE_Q5_K) k_qmatmul<PMOE_Q5_K><<<grid, 128, 0, s>>>(wb, rows, K, a, m, y);
    else if (dtype == PMOE_Q6_K) k_qmatmul<PMOE_Q6_K><<<grid, 128, 0, s>>>(wb, rows, K, a, m, y);
    else k_qmatmul<PMOE_Q8_0><<<grid, 128, 0, s>>>(wb, rows, K, a, m, y);
    count_launch(2);
    return cudaGetLastError();
}

size_t qmatmul_scratch_bytes(int m, int K)
{
    return ((size_t)m * K + 255) / 256 * 256 + ((size_t)m * (K / 32) * 4 + 255) / 256 * 256 + (size_t)m * (K / 16) * 2 + 256;
}

// ---------------------------------------------------------------- fixed scratch for callers that must not allocate
// The quantised activations of pmoe_qmatmul_noalloc live here instead of in stream-ordered
// allocations.  Every GPU that loads the library carries these 96 KB until the process exits.
// In host code `g_qmm_scratch` is only a handle for the runtime, never a device address:
// the address a kernel may use comes from cudaGetSymbolAddress, asked once per device with
// that device current.
constexpr size_t QMM_STATIC_BYTES = 96 * 1024;
static __device__ __align__(256) unsigned char g_qmm_scratch[QMM_STATIC_BYTES];

constexpr int QMM_MAX_DEVICES = 64;
static std::atomic<void *> g_qmm_scratch_addr[QMM_MAX_DEVICES];  // device address of g_qmm_scratch, per ordinal

cudaError_t qmatmul_static_scratch(int device, void **ptr, size_t *bytes)
{
    *ptr = nullptr;
    *bytes = QMM_STATIC_BYTES;
    if (device < 0 || device >= QMM_MAX_DEVICES) return cudaErrorInvalidDevice;
    void *p = g_qmm_scratch_addr[device].load(std::memory_order_acquire);
    if (!p) {  // set-up: the calling thread has made `device` current; two threads racing here store the same address
        cudaError_t e = cudaGetSymbolAddress(&p, g_qmm_scratch);
        if (e != cudaSuccess) return e;
        g_qmm_scratch_addr[device].store(p, std::memory_order_release);
    }
    *ptr = p;
    return cudaSuccess;
}

// ---------------------------------------------------------------- re-quantise the activated rows
// One CTA per row of act[., F]: routed pair rows that belong to a local expert, then the
// shared expert's rows.  The block type follows the down matrix that will consume the row.
__global__ void __launch_bounds__(64) k_act_quant(const float *__restrict__ act, int F, int n_routed_rows,
                                                  const int *__restrict__ pos, bool routed, int dt_r, int dt_s,
                                                  QAct a8k, QAct a80)
{
    const int r = blockIdx.x;
    int dt;
    pdl_wait();
    pdl_launch_dependents();
    if (r < n_routed_rows) {
        if (!routed || pos[r] < 0) return;
        dt = dt_r;
    } else {
        dt = dt_s;
    }
    const bool kq = is_kquant(dt);
    block_quant_row(act + (size_t)r * F, F, kq, !kq, a8k, a80, (size_t)r, threadIdx.x >> 5, 2, threadIdx.x & 31);
}

cudaError_t launch_act_quant(const LayerDev &L, const Workspace &ws, const uint32_t *idx, int n, int top_k,
                             bool routed, bool shared, cudaStream_t s)
{
    (void)idx;
    if (n <= 0) return cudaSuccess;
    int rows = n * top_k + (shared ? n : 0);
    cudaError_t e = launch_pdl(k_act_quant, dim3(rows), dim3(64), 0, s, (const float *)ws.act, L.F, n * top_k,
                               (const int *)ws.groups.pos, routed, L.down_dtype, L.sh_down_dtype, ws.act_q8k, ws.act_q80);
    count_launch();
    return e;
}

// ---------------------------------------------------------------- combine
// out[t] = sum over the token's local slots (slot order) of its weighted down rows, plus the
// gated shared-expert row (forward_batched's weighted sum, qwen3_next.rs:1391-1393, and the
// final add, 1932-1937).
template <typename OT>
__global__ void __launch_bounds__(256) k_combine(const float *__restrict__ partial, const int *__restrict__ pos,
                                                 int n, int top_k, int H, bool routed, bool shared, int sh_begin,
                                                 int sh_count, OT *__restrict__ out)
{
    const int t = blockIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    // which of the token's slots belong to a local expert: read once, so that the row loads below do
    // not each wait for their own flag
    uint32_t valid = 0;
    if (routed)
        for (int j = 0; j < top_k; j++) valid |= (pos[t * top_k + j] >= 0 ? 1u : 0u) << j;
    const bool with_shared = shared && t >= sh_begin && t < sh_begin + sh_count;
    // grid.y splits the row; the sum still runs in slot order
    for (int h = (blockIdx.y * blockDim.x + threadIdx.x) * 4; h < H; h += gridDim.y * blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j0 = 0; j0 < top_k; j0 += 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {   // four independent loads in flight
                const int j = j0 + u;
                v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (j < top_k && ((valid >> j) & 1u))
                    v[u] = *reinterpret_cast<const float4 *>(partial + (size_t)(t * top_k + j) * H + h);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int j = j0 + u;
                if (j < top_k && ((valid >> j) & 1u)) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
            }
        }
        if (with_shared) {
            const float4 v = *reinterpret_cast<const float4 *>(partial + (size_t)(n * top_k + t) * H + h);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        store_from_float(out, (size_t)t * H + h + 0, acc.x);
        store_from_float(out, (size_t)t * H + h + 1, acc.y);
        store_from_float(out, (size_t)t * H + h + 2, acc.z);
        store_from_float(out, (size_t)t * H + h + 3, acc.w);
    }
}

cudaError_t launch_combine(const LayerDev &L, const Workspace &ws, const uint32_t *idx, int n, int top_k, bool routed,
                           bool shared, void *out, int out_dtype, cudaStream_t s)
{
    (void)idx;
    if (n <= 0) return cudaSuccess;
    cudaError_t e;
    // few tokens: split each row over several CTAs so that the machine has enough loads in flight
    const int parts = n >= 512 ? 1 : (L.H + 1023) / 1024;
    const dim3 grid(n, parts);
    if (out_dtype == PMOE_F32)
        e = launch_pdl(k_combine<float>, grid, dim3(256), 0, s, (const float *)ws.partial, (const int *)ws.groups.pos, n,
                       top_k, L.H, routed, shared, ws.sh_begin, ws.sh_count, (float *)out);
    else
        e = launch_pdl(k_combine<__nv_bfloat16>, grid, dim3(256), 0, s, (const float *)ws.partial,
                       (const int *)ws.groups.pos, n, top_k, L.H, routed, shared, ws.sh_begin, ws.sh_count,
                       (__nv_bfloat16 *)out);
    count_launch();
    return e;
}

}  // namespace pmoe
