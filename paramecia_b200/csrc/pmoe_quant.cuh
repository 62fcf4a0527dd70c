// Activation quantisers shared by the routing and expert kernels.  They restate, per warp,
// candle's CPU BlockQ8K::from_float and BlockQ8_0::from_float so that the quantised
// activations are bit-identical to the reference CPU path's.
#pragma once
#include "pmoe_common.cuh"

namespace pmoe {

// ---------------------------------------------------------------- activation quantisers
// One warp quantises one block of 256 values the way candle's BlockQ8K::from_float does:
// the first element of largest magnitude keeps its sign, iscale = -128/max,
// q = min(127, round_half_away(iscale*x)), d = 1/iscale, bsums = sums of 16 quants.
__device__ inline void warp_quant_q8k(const float *src, int8_t *qs, float *d_out, int16_t *bsums, int lane)
{
    float v[8];
    {
        const float4 *s4 = reinterpret_cast<const float4 *>(src) + 2 * lane;
        float4 a = s4[0], b = s4[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    float amax = 0.f, mx = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++)
        if (amax < fabsf(v[j])) { amax = fabsf(v[j]); mx = v[j]; }
    int who = lane;
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        float oa = __shfl_xor_sync(0xffffffffu, amax, s);
        float om = __shfl_xor_sync(0xffffffffu, mx, s);
        int ow = __shfl_xor_sync(0xffffffffu, who, s);
        if (oa > amax || (oa == amax && ow < who)) { amax = oa; mx = om; who = ow; }
    }
    uint2 packed = make_uint2(0u, 0u);
    int sum = 0;
    float iscale = 0.f;
    if (amax != 0.f) {
        iscale = __fdiv_rn(-128.f, mx);
        uint32_t w[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float r = fminf(roundf(__fmul_rn(iscale, v[j])), 127.f);
            int q = (int)r;
            sum += q;
            w[j >> 2] |= (uint32_t)(q & 0xff) << (8 * (j & 3));
        }
        packed = make_uint2(w[0], w[1]);
    }
    *reinterpret_cast<uint2 *>(qs + 8 * lane) = packed;
    int sum16 = sum + __shfl_xor_sync(0xffffffffu, sum, 1);
    if (!(lane & 1)) bsums[lane >> 1] = (int16_t)sum16;
    if (lane == 0) *d_out = amax != 0.f ? __fdiv_rn(1.f, iscale) : 0.f;
}

// One warp quantises one block of 32 values as candle's BlockQ8_0::from_float:
// d = amax/127 (kept as f16), q = round_half_away(x * (1/d)).
__device__ inline void warp_quant_q80(const float *src, int8_t *qs, float *d_out, int lane)
{
    float x = src[lane];
    float amax = fabsf(x);
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
    float d = __fdiv_rn(amax, 127.f);
    float id = d != 0.f ? __fdiv_rn(1.f, d) : 0.f;
    qs[lane] = (int8_t)(int)roundf(__fmul_rn(x, id));
    if (lane == 0) *d_out = __half2float(__float2half_rn(d));
}

// Quantise `rows` rows of K floats held in shared memory or global memory.
__device__ inline void block_quant_row(const float *row, int K, bool q8k, bool q80, const QAct &a8k,
                                       const QAct &a80, size_t r, int warp, int nwarps, int lane)
{
    if (q8k)
        for (int b = warp; b < K / QK_K; b += nwarps)
            warp_quant_q8k(row + b * QK_K, a8k.qs + r * K + b * QK_K, a8k.d + r * (K / QK_K) + b,
                           a8k.bsums + r * (K / 16) + b * 16, lane);
    if (q80)
        for (int b = warp; b < K / QK8_0; b += nwarps)
            warp_quant_q80(row + b * QK8_0, a80.qs + r * K + b * QK8_0, a80.d + r * (K / QK8_0) + b, lane);
}


// A whole row of 512 floats quantised by one warp with a single round of loads: lane l owns the 16
// consecutive values 16l .. 16l+15.  Q8_K: a block is 16 lanes and a lane's values are exactly one
// 16-wide partial sum; Q8_0: a block is a lane pair.  Same arithmetic and tie rules as above.
__device__ inline void warp_quant_row512(const float *src, bool q8k, const QAct &a8k, const QAct &a80, size_t r, int lane)
{
    float v[16];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float4 t = reinterpret_cast<const float4 *>(src)[4 * lane + i];
        v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
    uint32_t w[4] = {0u, 0u, 0u, 0u};
    if (q8k) {
        float amax = 0.f, mx = 0.f;
#pragma unroll
        for (int j = 0; j < 16; j++)
            if (amax < fabsf(v[j])) { amax = fabsf(v[j]); mx = v[j]; }
        int who = lane;
#pragma unroll
        for (int s = 8; s >= 1; s >>= 1) {  // the 16 lanes of one block
            const float oa = __shfl_xor_sync(0xffffffffu, amax, s), om = __shfl_xor_sync(0xffffffffu, mx, s);
            const int ow = __shfl_xor_sync(0xffffffffu, who, s);
            if (oa > amax || (oa == amax && ow < who)) { amax = oa; mx = om; who = ow; }
        }
        int sum = 0;
        float iscale = 0.f;
        if (amax != 0.f) {
            iscale = __fdiv_rn(-128.f, mx);
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const int qv = (int)fminf(roundf(__fmul_rn(iscale, v[j])), 127.f);
                sum += qv;
                w[j >> 2] |= (uint32_t)(qv & 0xff) << (8 * (j & 3));
            }
        }
        *reinterpret_cast<uint4 *>(a8k.qs + r * 512 + 16 * lane) = make_uint4(w[0], w[1], w[2], w[3]);
        a8k.bsums[r * 32 + lane] = (int16_t)sum;
        if ((lane & 15) == 0) a8k.d[r * 2 + (lane >> 4)] = amax != 0.f ? __fdiv_rn(1.f, iscale) : 0.f;
    } else {
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(v[j]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        const float d = __fdiv_rn(amax, 127.f);
        const float id = d != 0.f ? __fdiv_rn(1.f, d) : 0.f;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const int qv = (int)roundf(__fmul_rn(v[j], id));
            w[j >> 2] |= (uint32_t)(qv & 0xff) << (8 * (j & 3));
        }
        *reinterpret_cast<uint4 *>(a80.qs + r * 512 + 16 * lane) = make_uint4(w[0], w[1], w[2], w[3]);
        if (!(lane & 1)) a80.d[r * 16 + (lane >> 1)] = __half2float(__float2half_rn(d));
    }
}

}  // namespace pmoe
