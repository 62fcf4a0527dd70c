// Block codecs and the small f32 kernels around the MoE block.
//
// k_dequantize restates candle's GgmlType::to_float for BlockQ8_0 and BlockQ2K ... BlockQ6K (the
// QTensor::dequantize the reference calls, e.g. paramecia-model/src/qwen3_next.rs:1758-1762);
// products are rounded one by one so the f32 bits equal the host codec's.
// k_add_rms_norm is RmsNorm::forward (paramecia-model/src/quantized_nn.rs:172-190) fused with
// the residual add of LayerWeights::forward_with_stats (qwen3_next.rs:4273-4286).
#include "pmoe_common.cuh"

namespace pmoe {

__device__ inline void q4k_scale_min(int j, const uint8_t *q, int &sc, int &m)
{
    if (j < 4) {
        sc = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

// one thread per output element; consecutive threads read one block's bytes and write
// consecutive floats
__global__ void __launch_bounds__(256) k_dequantize(int dtype, const uint8_t *__restrict__ blocks, size_t n,
                                                    float *__restrict__ out)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (dtype == PMOE_Q8_0) {
        const uint8_t *b = blocks + (i / QK8_0) * Q8_0_BYTES;
        float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
        out[i] = __fmul_rn((float)(int8_t)b[2 + i % QK8_0], d);
    } else if (dtype == PMOE_Q2_K) {
        const uint8_t *b = blocks + (i / QK_K) * Q2_K_BYTES;
        int w = (int)(i % QK_K);
        int half = w / 128, j = (w % 128) / 32, l = w % 32;
        float d = half_bits_to_float((uint16_t)(b[80] | (b[81] << 8)));
        float dmin = half_bits_to_float((uint16_t)(b[82] | (b[83] << 8)));
        uint8_t sc = b[8 * half + 2 * j + l / 16];
        int q = (b[16 + 32 * half + l] >> (2 * j)) & 3;
        out[i] = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)(sc & 0xF)), (float)q), __fmul_rn(dmin, (float)(sc >> 4)));
    } else if (dtype == PMOE_Q3_K) {
        const uint8_t *b = blocks + (i / QK_K) * Q3_K_BYTES;
        int w = (int)(i % QK_K);
        int half = w / 128, j = (w % 128) / 32, l = w % 32;
        float d = half_bits_to_float((uint16_t)(b[108] | (b[109] << 8)));
        int is = 8 * half + 2 * j + l / 16;   // 6-bit scale: low nibble in scales[is % 8], high 2 bits in scales[8 + is % 4]
        int low = is < 8 ? (b[96 + is] & 0xF) : (b[96 + is - 8] >> 4);
        int sc = (low | (((b[104 + (is & 3)] >> (2 * (is >> 2))) & 3) << 4)) - 32;
        int q = ((b[32 + 32 * half + l] >> (2 * j)) & 3) - (((b[l] >> (4 * half + j)) & 1) ? 0 : 4);
        out[i] = __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
    } else if (dtype == PMOE_Q4_K) {
        const uint8_t *b = blocks + (i / QK_K) * Q4_K_BYTES;
        int w = (int)(i % QK_K);
        int sub = w / 32, l = w % 32, grp = w / 64;
        float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
        float dmin = half_bits_to_float((uint16_t)(b[2] | (b[3] << 8)));
        int sc, m;
        q4k_scale_min(sub, b + 4, sc, m);
        uint8_t q = b[16 + 32 * grp + l];
        int v = (sub & 1) ? (q >> 4) : (q & 0xF);
        out[i] = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)v), __fmul_rn(dmin, (float)m));
    } else if (dtype == PMOE_Q5_K) {
        const uint8_t *b = blocks + (i / QK_K) * Q5_K_BYTES;
        int w = (int)(i % QK_K);
        int sub = w / 32, l = w % 32, grp = w / 64;
        float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
        float dmin = half_bits_to_float((uint16_t)(b[2] | (b[3] << 8)));
        int sc, m;
        q4k_scale_min(sub, b + 4, sc, m);
        uint8_t q = b[48 + 32 * grp + l];
        int v = ((sub & 1) ? (q >> 4) : (q & 0xF)) + (((b[16 + l] >> sub) & 1) << 4);
        out[i] = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)v), __fmul_rn(dmin, (float)m));
    } else if (dtype == PMOE_Q6_K) {
        const uint8_t *b = blocks + (i / QK_K) * Q6_K_BYTES;
        int w = (int)(i % QK_K);
        int half = w / 128, r = w % 128, quad = r / 32, l = r % 32;
        const uint8_t *ql = b + 64 * half, *qh = b + 128 + 32 * half;
        const int8_t *sc = reinterpret_cast<const int8_t *>(b + 192 + 8 * half);
        float d = half_bits_to_float((uint16_t)(b[208] | (b[209] << 8)));
        uint8_t lo = ql[l + 32 * (quad & 1)];
        int nib = quad >= 2 ? (lo >> 4) : (lo & 0xF);
        int q = (nib | (((qh[l] >> (2 * quad)) & 3) << 4)) - 32;
        out[i] = __fmul_rn(__fmul_rn(d, (float)sc[l / 16 + 2 * quad]), (float)q);
    } else if (dtype == PMOE_F16) {
        out[i] = half_bits_to_float(reinterpret_cast<const uint16_t *>(blocks)[i]);
    } else if (dtype == PMOE_BF16) {
        out[i] = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t *>(blocks)[i] << 16);
    } else {
        out[i] = reinterpret_cast<const float *>(blocks)[i];
    }
}

cudaError_t launch_dequantize(int dtype, const void *blocks, size_t n_elems, float *out, cudaStream_t s)
{
    if (!n_elems) return cudaSuccess;
    size_t grid = (n_elems + 255) / 256;
    k_dequantize<<<(unsigned)grid, 256, 0, s>>>(dtype, (const uint8_t *)blocks, n_elems, out);
    count_launch();
    return cudaGetLastError();
}

// QTensor::modify_block_scales as the reference's training mode uses it (qwen3_next.rs:1604-1606,
// models/with_tracing.rs:230): out = blocks with block i's f16 super-scale d (and dmin where the type
// has one) replaced by f16(f32(scale) * mults[i]), round to nearest even; quants and packed sub-scales
// are copied.  Blocks are 2-byte aligned only (34, 110, 210 bytes), so the copy runs in 16-bit units:
// one warp per block, lanes stride over its halfwords.
__global__ void __launch_bounds__(256) k_modify_block_scales(int type_bytes, int d_off, int dmin_off,
                                                             const uint16_t *__restrict__ blocks, size_t n_blocks,
                                                             const float *__restrict__ mults, uint16_t *__restrict__ out)
{
    const size_t b = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= n_blocks) return;
    const int lane = threadIdx.x & 31;
    const int hw = type_bytes / 2;
    const uint16_t *src = blocks + b * hw;
    uint16_t *dst = out + b * hw;
    const float m = mults[b];
    for (int i = lane; i < hw; i += 32) {
        uint16_t v = src[i];
        if (2 * i == d_off || 2 * i == dmin_off) v = __half_as_ushort(__float2half_rn(__fmul_rn(half_bits_to_float(v), m)));
        dst[i] = v;
    }
}

cudaError_t launch_modify_block_scales(int dtype, const void *blocks, size_t n_blocks, const float *mults, void *out,
                                       cudaStream_t s)
{
    if (!n_blocks) return cudaSuccess;
    int d_off = 0, dmin_off = -1;
    switch (dtype) {
    case PMOE_Q8_0: d_off = 0; break;
    case PMOE_Q2_K: d_off = 80; dmin_off = 82; break;
    case PMOE_Q3_K: d_off = 108; break;
    case PMOE_Q4_K: case PMOE_Q5_K: d_off = 0; dmin_off = 2; break;
    case PMOE_Q6_K: d_off = 208; break;
    default: return cudaErrorInvalidValue;
    }
    const size_t grid = (n_blocks + 7) / 8;
    k_modify_block_scales<<<(unsigned)grid, 256, 0, s>>>(block_bytes(dtype), d_off, dmin_off, (const uint16_t *)blocks,
                                                         n_blocks, mults, (uint16_t *)out);
    count_launch();
    return cudaGetLastError();
}

// resid_out = resid_in + delta; y = resid_out / sqrt(mean(resid_out^2) + eps) * weight
// (resid_out may be resid_in: a thread reads and later writes the same elements)
__global__ void __launch_bounds__(256) k_add_rms_norm(const float *resid_in, const float *__restrict__ delta,
                                                      const float *__restrict__ weight, int H, float eps,
                                                      float *resid_out, float *__restrict__ y)
{
    extern __shared__ float row[];
    __shared__ float red[8];
    __shared__ float inv_m;
    const int t = blockIdx.x;
    float ss = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float v = resid_in[(size_t)t * H + h];
        if (delta) v = __fadd_rn(v, delta[(size_t)t * H + h]);
        row[h] = v;
        ss += v * v;
    }
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) tot += red[w];
        inv_m = sqrtf(tot / (float)H + eps);
    }
    __syncthreads();
    const float m = inv_m;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float v = row[h];
        if (resid_out) resid_out[(size_t)t * H + h] = v;
        float o = __fdiv_rn(v, m);
        y[(size_t)t * H + h] = weight ? __fmul_rn(o, weight[h]) : o;
    }
}

// out[t] = sum_r parts[r][t] (+ extra[t]): the home rank's side of the expert-parallel combine.
// Rank order is fixed, so the result does not depend on message arrival order.
template <typename ET, typename OT>
__global__ void __launch_bounds__(256) k_reduce_rows(const float *__restrict__ parts, int R, size_t stride,
                                                     const ET *__restrict__ extra, size_t total,
                                                     OT *__restrict__ out)
{
    size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= total) return;
    float4 acc = *reinterpret_cast<const float4 *>(parts + i);
    for (int r = 1; r < R; r++) {
        const float4 v = *reinterpret_cast<const float4 *>(parts + (size_t)r * stride + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (extra) {
        acc.x += load_as_float(extra, i); acc.y += load_as_float(extra, i + 1);
        acc.z += load_as_float(extra, i + 2); acc.w += load_as_float(extra, i + 3);
    }
    store_from_float(out, i, acc.x); store_from_float(out, i + 1, acc.y);
    store_from_float(out, i + 2, acc.z); store_from_float(out, i + 3, acc.w);
}

cudaError_t launch_reduce_rows(const float *parts, int R, const void *extra, int extra_dtype, int n, int H, void *out,
                               int out_dtype, cudaStream_t s)
{
    if (n <= 0) return cudaSuccess;
    const size_t total = (size_t)n * H;
    const unsigned grid = (unsigned)((total / 4 + 255) / 256);
    const bool ef = extra_dtype == PMOE_F32, of = out_dtype == PMOE_F32;
    if (ef && of)
        k_reduce_rows<float, float><<<grid, 256, 0, s>>>(parts, R, total, (const float *)extra, total, (float *)out);
    else if (ef)
        k_reduce_rows<float, __nv_bfloat16><<<grid, 256, 0, s>>>(parts, R, total, (const float *)extra, total,
                                                                 (__nv_bfloat16 *)out);
    else if (of)
        k_reduce_rows<__nv_bfloat16, float><<<grid, 256, 0, s>>>(parts, R, total, (const __nv_bfloat16 *)extra, total,
                                                                 (float *)out);
    else
        k_reduce_rows<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, s>>>(parts, R, total, (const __nv_bfloat16 *)extra,
                                                                         total, (__nv_bfloat16 *)out);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_add_rms_norm(const float *resid_in, const float *delta, const float *weight, int n, int H,
                                float eps, float *resid_out, float *y, cudaStream_t s)
{
    if (n <= 0) return cudaSuccess;
    k_add_rms_norm<<<n, 256, (size_t)H * sizeof(float), s>>>(resid_in, delta, weight, H, eps, resid_out, y);
    count_launch();
    return cudaGetLastError();
}

}  // namespace pmoe
