// Routing side of the MoE block: activation quantisation of the input rows, the router
// GEMV in a fixed summation order, clamp + softmax + top-k + renormalisation, and the
// device-side grouping of (token, slot) pairs by expert.
//
// Reference semantics: MoeBlock::forward_with_stats (paramecia-model/src/qwen3_next.rs:1903-1940),
// ops::topk_moe_routing (paramecia-model/src/ops.rs:28-59), the host-side grouping of
// apply_experts_sequential (qwen3_next.rs:2037-2050) and ops::group_tokens_by_expert (ops.rs:74-157).
#include <cstdlib>
#include "pmoe_common.cuh"
#include "pmoe_quant.cuh"

namespace pmoe {

// ---------------------------------------------------------------- prep: per-token work
// One CTA per token: widen the row to f32 in shared memory, quantise it for the expert
// mat-muls and evaluate the shared expert's gate sigmoid(sum_j x_j * w_j)
// (SharedExpert::forward, qwen3_next.rs:1811-1812).
// per-token work; any block size up to 8 warps; xrow = H floats of shared memory
struct PrepArgs {
    int n;             // tokens to prepare (0 = none)
    bool q8k, q80;
    QAct a8k, a80;
    const float *gate_inp;
    float *sh_sigmoid;
};

template <typename XT>
__device__ inline void prep_token(const XT *__restrict__ x, int H, int t, const PrepArgs &P, float *xrow, float *red)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float part = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float v = load_as_float(x, (size_t)t * H + h);
        xrow[h] = v;
        if (P.gate_inp) part += v * P.gate_inp[h];
    }
    __syncthreads();
    block_quant_row(xrow, H, P.q8k, P.q80, P.a8k, P.a80, t, warp, blockDim.x >> 5, lane);
    if (P.gate_inp) {
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) part += __shfl_xor_sync(0xffffffffu, part, s);
        if (lane == 0) red[warp] = part;
        __syncthreads();
        if (threadIdx.x == 0) {
            float s = 0.f;
            for (int w = 0; w < (int)(blockDim.x >> 5); w++) s += red[w];
            P.sh_sigmoid[t] = 1.f / (1.f + expf(-s));
        }
    }
}

template <typename XT>
__global__ void __launch_bounds__(256) k_prep(const XT *__restrict__ x, int H, PrepArgs P)
{
    extern __shared__ __align__(16) float xrow[];
    __shared__ float red[8];
    pdl_wait();
    pdl_launch_dependents();
    prep_token(x, H, blockIdx.x, P, xrow, red);
}

static PrepArgs make_prep_args(const LayerDev &L, const Workspace &ws, int n, bool need_q8k, bool need_q80, bool need_gate)
{
    PrepArgs P{};
    P.n = n;
    P.q8k = need_q8k; P.q80 = need_q80;
    P.a8k = ws.x_q8k; P.a80 = ws.x_q80;
    P.gate_inp = need_gate ? L.sh_gate_inp : nullptr;
    P.sh_sigmoid = ws.sh_sigmoid;
    return P;
}

cudaError_t launch_prep(const LayerDev &L, const Workspace &ws, const void *x, int x_dtype, int n, bool need_q8k,
                        bool need_q80, bool need_gate, cudaStream_t s)
{
    if (n <= 0) return cudaSuccess;
    size_t smem = (size_t)L.H * sizeof(float);
    const PrepArgs P = make_prep_args(L, ws, n, need_q8k, need_q80, need_gate);
    cudaError_t e;
    if (x_dtype == PMOE_F32) e = launch_pdl(k_prep<float>, dim3(n), dim3(256), smem, s, (const float *)x, L.H, P);
    else e = launch_pdl(k_prep<__nv_bfloat16>, dim3(n), dim3(256), smem, s, (const __nv_bfloat16 *)x, L.H, P);
    count_launch();
    return e;
}

// ---------------------------------------------------------------- router logits
// logits[t, e] = sum_h x[t, h] * W[e, h] (+ bias[e]) in f32.  The summation order is part of
// the contract (the top-k indices must equal the CPU oracle's): lane p of a warp owns
// elements 128*i + 4*p + j, takes them i ascending then j = 0..3 with one fused
// multiply-add each, and the 32 partial sums fold through v += shfl_xor(v, s), s = 16..1.
__device__ inline float4 load_x4(const float *x, size_t off) { return *reinterpret_cast<const float4 *>(x + off); }
__device__ inline float4 load_x4(const __nv_bfloat16 *x, size_t off)
{
    uint2 r = *reinterpret_cast<const uint2 *>(x + off);
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162 *>(&r.x);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162 *>(&r.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

constexpr int ROUTER_WPB = 2;

// The router matrix is static: a kernel pulls its own rows towards L2 before it waits for the
// previous kernel (whose output, x, it may not touch yet), so the cold read of W overlaps that
// kernel's tail instead of following it.
__device__ inline void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ inline void prefetch_row_l2(const float *row, int H, int lane)
{
    for (int j = lane * 32; j < H; j += 32 * 32) prefetch_l2(row + j);   // one 128-byte line per lane and step
}

template <typename XT, int TT>
__global__ void __launch_bounds__(ROUTER_WPB * 32) k_router(const float *__restrict__ W,
                                                            const float *__restrict__ bias,
                                                            const XT *__restrict__ x, int n, int E, int H,
                                                            float *__restrict__ logits, int router_ctas, PrepArgs P)
{
    extern __shared__ __align__(16) float xrow[];
    __shared__ float red[8];
    {
        const int e_pf = blockIdx.x * ROUTER_WPB + (threadIdx.x >> 5);
        if ((int)blockIdx.x < router_ctas && e_pf < E) prefetch_row_l2(W + (size_t)e_pf * H, H, threadIdx.x & 31);
    }
    pdl_wait();
    pdl_launch_dependents();
    if ((int)blockIdx.x >= router_ctas) {  // CTAs past the router rows prepare one token each
        prep_token(x, H, (int)blockIdx.x - router_ctas, P, xrow, red);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * ROUTER_WPB + warp;
    if (e >= E) return;
    const float4 *w4 = reinterpret_cast<const float4 *>(W + (size_t)e * H);
    const int steps = H / 128;
    for (int t0 = 0; t0 < n; t0 += TT) {
        float acc[TT];
#pragma unroll
        for (int tt = 0; tt < TT; tt++) acc[tt] = 0.f;
#pragma unroll 4
        for (int i = 0; i < steps; i++) {
            float4 wv = w4[32 * i + lane];
#pragma unroll
            for (int tt = 0; tt < TT; tt++) {
                if (t0 + tt < n) {
                    float4 xv = load_x4(x, (size_t)(t0 + tt) * H + 128 * i + 4 * lane);
                    acc[tt] = fmaf(xv.x, wv.x, acc[tt]);
                    acc[tt] = fmaf(xv.y, wv.y, acc[tt]);
                    acc[tt] = fmaf(xv.z, wv.z, acc[tt]);
                    acc[tt] = fmaf(xv.w, wv.w, acc[tt]);
                }
            }
        }
#pragma unroll
        for (int tt = 0; tt < TT; tt++) {
            float v = acc[tt];
#pragma unroll
            for (int s = 16; s >= 1; s >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, s));
            if (lane == 0 && t0 + tt < n) logits[(size_t)(t0 + tt) * E + e] = bias ? __fadd_rn(v, bias[e]) : v;
        }
    }
}

// The same product for more than a handful of tokens, register-tiled.  A CTA stages a tile of T
// rows of x in shared memory as f32; a warp works on R router rows at once against all T tokens,
// so one shared-memory read of x feeds 4*R multiply-adds and one read of W feeds 4*T.  Each
// (row, token) partial sum is still built by lane p over elements 128*i + 4*p + j in ascending
// order and folded 16, 8, 4, 2, 1 lanes apart like the butterfly (the transposed reduction only
// changes which lane ends up with which total), so the bits do not depend on which kernel ran.
// H <= 2048, a multiple of 128.  PASSES row groups per warp amortise the tile load.
constexpr int RT_WARPS = 8;

template <typename XT, int R, int T>
__global__ void __launch_bounds__(RT_WARPS * 32) k_router_tiled(const float *__restrict__ W,
                                                                const float *__restrict__ bias,
                                                                const XT *__restrict__ x, int n, int E, int H,
                                                                int passes, float *__restrict__ logits,
                                                                int token_tiles, PrepArgs P)
{
    extern __shared__ __align__(16) float xs[];  // [T][H]
    __shared__ float red[8];
    if ((int)blockIdx.y == 0) {   // the CTAs of the first token tile cover every row once
        for (int pass = 0; pass < passes; pass++) {
            const int e0 = ((blockIdx.x * passes + pass) * RT_WARPS + (threadIdx.x >> 5)) * R;
#pragma unroll
            for (int r_ = 0; r_ < R; r_++)
                if (e0 + r_ < E) prefetch_row_l2(W + (size_t)(e0 + r_) * H, H, threadIdx.x & 31);
        }
    }
    pdl_wait();
    pdl_launch_dependents();
    if ((int)blockIdx.y >= token_tiles) {  // grid rows past the token tiles prepare one token per CTA
        const int t = ((int)blockIdx.y - token_tiles) * gridDim.x + blockIdx.x;
        if (t < P.n) prep_token(x, H, t, P, xs, red);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.y * T;
    const int nt = n - t0 < T ? n - t0 : T;
    for (int i = threadIdx.x * 4; i < T * H; i += RT_WARPS * 32 * 4) {
        const int tt = i / H;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tt < nt) v = load_x4(x, (size_t)(t0 + tt) * H + (i - tt * H));
        *reinterpret_cast<float4 *>(xs + i) = v;
    }
    __syncthreads();
    const int steps = H / 128;  // <= 16
    const int h4 = H / 4;
    const float4 *xs4 = reinterpret_cast<const float4 *>(xs);
    for (int pass = 0; pass < passes; pass++) {
        const int e0 = ((blockIdx.x * passes + pass) * RT_WARPS + warp) * R;
        if (e0 >= E) break;
        const float4 *w4[R];
#pragma unroll
        for (int r = 0; r < R; r++) w4[r] = reinterpret_cast<const float4 *>(W + (size_t)(e0 + r < E ? e0 + r : E - 1) * H) + lane;
        float acc[R * T];
#pragma unroll
        for (int i = 0; i < R * T; i++) acc[i] = 0.f;
#pragma unroll 4
        for (int i = 0; i < steps; i++) {
            float4 wv[R];
#pragma unroll
            for (int r = 0; r < R; r++) wv[r] = w4[r][32 * i];
#pragma unroll
            for (int tt = 0; tt < T; tt++) {
                const float4 xv = xs4[tt * h4 + 32 * i + lane];
#pragma unroll
                for (int r = 0; r < R; r++) {
                    float a = acc[r * T + tt];
                    a = fmaf(xv.x, wv[r].x, a);
                    a = fmaf(xv.y, wv[r].y, a);
                    a = fmaf(xv.z, wv[r].z, a);
                    a = fmaf(xv.w, wv[r].w, a);
                    acc[r * T + tt] = a;
                }
            }
        }
        // fold 32 (or fewer) totals at a time: value index = r * T + tt, lane / DUP holds it
        constexpr int V = R * T < 32 ? R * T : 32;
        constexpr int DUP = 32 / V;
#pragma unroll
        for (int c = 0; c < R * T / V; c++) {
            const float v = transposed_reduce<V, 32>(*reinterpret_cast<float(*)[V]>(acc + c * V), lane);
            const int vi = c * V + lane / DUP;
            const int r = vi / T, tt = vi % T;
            if (lane % DUP == 0 && tt < nt && e0 + r < E)
                logits[(size_t)(t0 + tt) * E + e0 + r] = bias ? __fadd_rn(v, bias[e0 + r]) : v;
        }
    }
}

template <typename XT, int R, int T>
static cudaError_t launch_router_tiled(const LayerDev &L, const void *x, int n, int passes, float *logits, const PrepArgs &P,
                                       cudaStream_t s)
{
    auto kern = k_router_tiled<XT, R, T>;
    const size_t smem = (size_t)T * L.H * sizeof(float);
    static bool configured = false;  // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T * 2048 * (int)sizeof(float));
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const int rows_per_cta = RT_WARPS * R * passes;
    const int gx = (L.E + rows_per_cta - 1) / rows_per_cta, tiles = (n + T - 1) / T;
    dim3 grid(gx, tiles + (P.n + gx - 1) / gx);
    cudaError_t e = launch_pdl(kern, grid, dim3(RT_WARPS * 32), smem, s, L.router_w, L.router_bias, (const XT *)x, n, L.E,
                               L.H, passes, logits, tiles, P);
    count_launch();
    return e;
}

// The prefill-sized form of the same product on the packed f32x2 multiply-add of this architecture: one instruction
// advances the sums of two tokens (each half is an IEEE fma of its own, so every (row, token) sum is still built in
// the order above and the bits are the same).  The token tile lies in shared memory with the tokens of a pair
// interleaved, in the order a lane reads it: for pair p, step i and half hf, lane l finds
// (x0[j], x1[j], x0[j + 1], x1[j + 1]), j = 2 hf, of its elements 128 i + 4 l + j, at
// ((p * steps + i) * 2 + hf) * 32 + l: 16 consecutive bytes per lane, no bank conflicts.
__device__ inline uint64_t pack2(float lo, float hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ inline void unpack2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ inline uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

template <typename XT, int R, int T, int NW>
__global__ void __launch_bounds__(NW * 32) k_router_pairs(const float *__restrict__ W, const float *__restrict__ bias,
                                                                const XT *__restrict__ x, int n, int E, int H, int passes,
                                                                float *__restrict__ logits)
{
    extern __shared__ __align__(16) float xs[];  // [T / 2][steps][2][32] float4
    static_assert(T % 2 == 0, "tokens go in pairs");
    if ((int)blockIdx.y == 0) {   // the CTAs of the first token tile cover every row once
        for (int pass = 0; pass < passes; pass++) {
            const int e0 = ((blockIdx.x * passes + pass) * NW + (threadIdx.x >> 5)) * R;
#pragma unroll
            for (int r_ = 0; r_ < R; r_++)
                if (e0 + r_ < E) prefetch_row_l2(W + (size_t)(e0 + r_) * H, H, threadIdx.x & 31);
        }
    }
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.y * T;
    const int nt = n - t0 < T ? n - t0 : T;
    const int steps = H / 128;  // <= 16
    // fill: one (pair, step, lane) item = the lane's four elements of both tokens
    for (int it = threadIdx.x; it < (T / 2) * steps * 32; it += NW * 32) {
        const int l = it & 31, i = (it >> 5) % steps, pr = (it >> 5) / steps;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (2 * pr < nt) a = load_x4(x, (size_t)(t0 + 2 * pr) * H + 128 * i + 4 * l);
        if (2 * pr + 1 < nt) b = load_x4(x, (size_t)(t0 + 2 * pr + 1) * H + 128 * i + 4 * l);
        float4 *dst = reinterpret_cast<float4 *>(xs) + ((size_t)(pr * steps + i) * 2) * 32 + l;
        dst[0] = make_float4(a.x, b.x, a.y, b.y);
        dst[32] = make_float4(a.z, b.z, a.w, b.w);
    }
    __syncthreads();
    const ulonglong2 *xp = reinterpret_cast<const ulonglong2 *>(xs);
    for (int pass = 0; pass < passes; pass++) {
        const int e0 = ((blockIdx.x * passes + pass) * NW + warp) * R;
        if (e0 >= E) break;
        const float4 *w4[R];
#pragma unroll
        for (int r = 0; r < R; r++) w4[r] = reinterpret_cast<const float4 *>(W + (size_t)(e0 + r < E ? e0 + r : E - 1) * H) + lane;
        uint64_t acc2[R * (T / 2)];   // (row r, pair p): the sums of tokens 2p (low half) and 2p + 1
#pragma unroll
        for (int i = 0; i < R * (T / 2); i++) acc2[i] = 0ull;
#pragma unroll 1
        for (int i = 0; i < steps; i++) {
            uint64_t wd[R][4];   // the lane's four elements of each row, each in both halves
#pragma unroll
            for (int r = 0; r < R; r++) {
                const float4 wv = w4[r][32 * i];
                wd[r][0] = pack2(wv.x, wv.x);
                wd[r][1] = pack2(wv.y, wv.y);
                wd[r][2] = pack2(wv.z, wv.z);
                wd[r][3] = pack2(wv.w, wv.w);
            }
#pragma unroll
            for (int pr = 0; pr < T / 2; pr++) {
                const ulonglong2 xa = xp[((size_t)(pr * steps + i) * 2) * 32 + lane];
                const ulonglong2 xb = xp[((size_t)(pr * steps + i) * 2 + 1) * 32 + lane];
#pragma unroll
                for (int r = 0; r < R; r++) {
                    uint64_t a = acc2[r * (T / 2) + pr];
                    a = ffma2(xa.x, wd[r][0], a);
                    a = ffma2(xa.y, wd[r][1], a);
                    a = ffma2(xb.x, wd[r][2], a);
                    a = ffma2(xb.y, wd[r][3], a);
                    acc2[r * (T / 2) + pr] = a;
                }
            }
        }
        float acc[R * T];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int pr = 0; pr < T / 2; pr++) unpack2(acc2[r * (T / 2) + pr], acc[r * T + 2 * pr], acc[r * T + 2 * pr + 1]);
        // fold 32 totals at a time: value index = r * T + tt, lane holds it
        constexpr int V = 32;
        static_assert(R * T % V == 0, "whole folds");
#pragma unroll
        for (int c = 0; c < R * T / V; c++) {
            const float v = transposed_reduce<V, 32>(*reinterpret_cast<float(*)[V]>(acc + c * V), lane);
            const int vi = c * V + lane;
            const int r = vi / T, tt = vi % T;
            if (tt < nt && e0 + r < E) logits[(size_t)(t0 + tt) * E + e0 + r] = bias ? __fadd_rn(v, bias[e0 + r]) : v;
        }
    }
}

template <typename XT, int R, int T, int NW>
static cudaError_t launch_router_pairs(const LayerDev &L, const void *x, int n, int passes, float *logits, cudaStream_t s)
{
    auto kern = k_router_pairs<XT, R, T, NW>;
    const size_t smem = (size_t)T * L.H * sizeof(float);
    static bool configured = false;  // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T * 2048 * (int)sizeof(float));
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const int rows_per_cta = NW * R * passes;
    dim3 grid((L.E + rows_per_cta - 1) / rows_per_cta, (n + T - 1) / T);
    cudaError_t e = launch_pdl(kern, grid, dim3(NW * 32), smem, s, L.router_w, L.router_bias, (const XT *)x, n, L.E, L.H,
                               passes, logits);
    count_launch();
    return e;
}

__global__ void k_add_bias(float *__restrict__ logits, const float *__restrict__ bias, int n, int E)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n * E) logits[i] += bias[i % E];
}

// Router launch.  With `prep` set the same launch also prepares the tokens (quantised rows, shared
// gate) in extra CTAs, which saves the separate k_prep launch of a decode-sized call.
cudaError_t launch_router(const LayerDev &L, const Workspace &ws, const void *x, int x_dtype, int n, float *logits,
                          cudaStream_t s, bool prep, bool need_q8k, bool need_q80, bool need_gate)
{
    if (n <= 0) return cudaSuccess;
    if (L.router_q) {
        // A quantised ffn_gate_inp is a QMatMul like the experts' (models/with_tracing.rs:324-335): the rows are
        // quantised to the type its block dots take and the logits are integer block sums with f32 scales.  The
        // preparation runs first, whether or not the caller wants it for the experts.
        const bool kq = is_kquant(L.router_dtype);
        cudaError_t e = launch_prep(L, ws, x, x_dtype, n, need_q8k || kq, need_q80 || !kq, prep && need_gate, s);
        if (e != cudaSuccess) return e;
        e = launch_qmatmul_quantised(L.router_dtype, L.router_q, L.E, L.H, kq ? ws.x_q8k : ws.x_q80, n, logits, s);
        if (e != cudaSuccess || !L.router_bias) return e;
        k_add_bias<<<(n * L.E + 255) / 256, 256, 0, s>>>(logits, L.router_bias, n, L.E);
        count_launch();
        return cudaGetLastError();
    }
    const bool f32 = x_dtype == PMOE_F32;
    using BT = __nv_bfloat16;
    const PrepArgs P = make_prep_args(L, ws, prep ? n : 0, need_q8k, need_q80, need_gate);
    // (also for one token: with W cold in HBM, as it is when a model's layers take turns, the tiled kernel's
    // eight loads in flight per lane beat the row-per-warp kernel below: 27 -> 16 us)
    if (L.H <= 2048 && L.H % 128 == 0) {
        if (n > 512) {  // prefill sizes: 16-token tiles (128 KB of shared memory: one CTA per SM), 128 rows per CTA, packed
            // multiply-adds; sixteen warps of 4 rows x 16 tokens each measured a little faster than eight of 8 x 16
            // (token preparation in its own launch: riding along it would hold 128 KB per token)
            if (prep) {
                cudaError_t e = launch_prep(L, ws, x, x_dtype, n, need_q8k, need_q80, need_gate, s);
                if (e != cudaSuccess) return e;
            }
            return f32 ? launch_router_pairs<float, 4, 16, 16>(L, x, n, 2, logits, s)
                       : launch_router_pairs<BT, 4, 16, 16>(L, x, n, 2, logits, s);
        }
        if (n >= 128) {   // (at 64 tokens two rows per warp = twice the CTAs measured faster: 21 -> 17.5 us)
            const int tiles = (n + 7) / 8, passes = tiles >= 32 ? tiles / 16 : 1;  // about 256 CTAs
            return f32 ? launch_router_tiled<float, 4, 8>(L, x, n, passes, logits, P, s)
                       : launch_router_tiled<BT, 4, 8>(L, x, n, passes, logits, P, s);
        }
        if (n <= 8)   // one token tile: one row per warp spreads the rows of W over twice the SMs
            return f32 ? launch_router_tiled<float, 1, 8>(L, x, n, 1, logits, P, s)
                       : launch_router_tiled<BT, 1, 8>(L, x, n, 1, logits, P, s);
        return f32 ? launch_router_tiled<float, 2, 8>(L, x, n, 1, logits, P, s)
                   : launch_router_tiled<BT, 2, 8>(L, x, n, 1, logits, P, s);
    }
    if (L.H > 2048 && prep) {  // the shared-memory row of the fused form is sized for H <= 2048
        cudaError_t e = launch_prep(L, ws, x, x_dtype, n, need_q8k, need_q80, need_gate, s);
        if (e != cudaSuccess) return e;
    }
    const int rc = (L.E + ROUTER_WPB - 1) / ROUTER_WPB;
    const int pn = L.H > 2048 ? 0 : P.n;
    dim3 grid(rc + pn), block(ROUTER_WPB * 32);
    const size_t smem = pn ? (size_t)L.H * sizeof(float) : 0;
    cudaError_t e;
    if (f32) {
        if (n == 1)
            e = launch_pdl(k_router<float, 1>, grid, block, smem, s, L.router_w, L.router_bias, (const float *)x, n, L.E, L.H, logits, rc, P);
        else
            e = launch_pdl(k_router<float, 8>, grid, block, smem, s, L.router_w, L.router_bias, (const float *)x, n, L.E, L.H, logits, rc, P);
    } else {
        if (n == 1)
            e = launch_pdl(k_router<BT, 1>, grid, block, smem, s, L.router_w, L.router_bias, (const BT *)x, n, L.E, L.H, logits, rc, P);
        else
            e = launch_pdl(k_router<BT, 8>, grid, block, smem, s, L.router_w, L.router_bias, (const BT *)x, n, L.E, L.H, logits, rc, P);
    }
    count_launch();
    return e;
}

// ---------------------------------------------------------------- softmax + top-k
// One warp per token.  clamp(+-100) (qwen3_next.rs:1923), softmax over E (1924), then the
// first k entries of a stable descending sort with the weights divided by their sum
// (ops.rs:44-52): k rounds of arg-max where a tie goes to the lower expert id.
constexpr int TOPK_WPB = 4;

__global__ void __launch_bounds__(TOPK_WPB * 32) k_topk(const float *__restrict__ logits, int n, int E, int k,
                                                        uint32_t *__restrict__ idx_out, float *__restrict__ w_out)
{
    extern __shared__ float sprob[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * TOPK_WPB + warp;
    pdl_wait();
    pdl_launch_dependents();
    if (t >= n) return;
    float *p = sprob + (size_t)warp * E;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) {
        float v = logits[(size_t)t * E + e];
        v = fminf(fmaxf(v, -100.f), 100.f);
        p[e] = v;
        mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        float v = expf(p[e] - mx);
        p[e] = v;
        sum += v;
    }
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
    for (int e = lane; e < E; e += 32) p[e] = __fdiv_rn(p[e], sum);
    __syncwarp();
    float my_w = 0.f;      // lane j keeps the j-th selection
    uint32_t my_i = 0;
    for (int j = 0; j < k; j++) {
        float bv = -1.f;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            float v = p[e];
            if (v > bv) { bv = v; bi = e; }
        }
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, s);
            int oi = __shfl_xor_sync(0xffffffffu, bi, s);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == j) { my_w = bv; my_i = (uint32_t)bi; }
        if (lane == 0) p[bi] = -2.f;
        __syncwarp();
    }
    float wsum = 0.f;
    for (int j = 0; j < k; j++) wsum += __shfl_sync(0xffffffffu, my_w, j);
    if (lane < k) {
        if (idx_out) idx_out[(size_t)t * k + lane] = my_i;
        if (w_out) w_out[(size_t)t * k + lane] = __fdiv_rn(my_w, wsum);
    }
}

// The same selection with a token's probabilities in registers (E = 32 * NV): lane l owns experts
// l, l + 32, ...  Same operations on the same values as k_topk, so the same bits come out; it only
// drops the shared-memory round trips of the k arg-max rounds.
template <int NV>
__global__ void __launch_bounds__(TOPK_WPB * 32) k_topk_reg(const float *__restrict__ logits, int n, int k,
                                                            uint32_t *__restrict__ idx_out, float *__restrict__ w_out)
{
    constexpr int E = 32 * NV;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * TOPK_WPB + warp;
    pdl_wait();
    pdl_launch_dependents();
    if (t >= n) return;
    float p[NV];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        float v = logits[(size_t)t * E + lane + 32 * i];
        v = fminf(fmaxf(v, -100.f), 100.f);
        p[i] = v;
        mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        p[i] = expf(p[i] - mx);
        sum += p[i];
    }
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
#pragma unroll
    for (int i = 0; i < NV; i++) p[i] = __fdiv_rn(p[i], sum);
    float my_w = 0.f;      // lane j keeps the j-th selection
    uint32_t my_i = 0;
    for (int j = 0; j < k; j++) {
        float bv = -1.f;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < NV; i++)
            if (p[i] > bv) { bv = p[i]; bi = lane + 32 * i; }
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, s);
            int oi = __shfl_xor_sync(0xffffffffu, bi, s);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == j) { my_w = bv; my_i = (uint32_t)bi; }
#pragma unroll
        for (int i = 0; i < NV; i++)
            if (bi == lane + 32 * i) p[i] = -2.f;   // taken
    }
    float wsum = 0.f;
    for (int j = 0; j < k; j++) wsum += __shfl_sync(0xffffffffu, my_w, j);
    if (lane < k) {
        if (idx_out) idx_out[(size_t)t * k + lane] = my_i;
        if (w_out) w_out[(size_t)t * k + lane] = __fdiv_rn(my_w, wsum);
    }
}

cudaError_t launch_topk(const LayerDev &L, const Workspace &ws, const float *logits, int n, uint32_t *idx, float *w,
                        cudaStream_t s)
{
    (void)ws;
    if (n <= 0) return cudaSuccess;
    if (L.E == 512) {
        cudaError_t e = launch_pdl(k_topk_reg<16>, dim3((n + TOPK_WPB - 1) / TOPK_WPB), dim3(TOPK_WPB * 32), 0, s,
                                   (const float *)logits, n, L.k, idx, w);
        count_launch();
        return e;
    }
    size_t smem = (size_t)TOPK_WPB * L.E * sizeof(float);
    cudaError_t e = launch_pdl(k_topk, dim3((n + TOPK_WPB - 1) / TOPK_WPB), dim3(TOPK_WPB * 32), smem, s,
                               (const float *)logits, n, L.E, L.k, idx, w);
    count_launch();
    return e;
}

// ---------------------------------------------------------------- grouping by expert
// Counting sort of the n*k (token, slot) pairs by local expert id: counts through shared-memory
// atomics, a scan, then the scatter.  The order of pairs inside one expert's list depends on
// atomic arrival order; no result depends on it (every pair's rows are computed on their own and
// combined in slot order).  Decode-sized calls do all of it in one CTA (k_group alone); from
// GROUP_MULTI_MIN pairs on, the counting and the scatter, which walk the pairs, are spread over
// one CTA per GROUP_CHUNK pairs (k_group_count, k_group_scatter) around the same one-CTA scan.
constexpr int GROUP_THREADS = 1024;
constexpr int GROUP_MULTI_MIN = 8192;
static_assert(GROUP_CHUNK == GROUP_THREADS, "one pair per thread of a counting CTA");

// inclusive scan of six integers per thread across the CTA: shuffles inside a warp, one pass
// over the 32 warp totals, three barriers in all
constexpr int NSCAN = 6;
struct Scan5 {
    int v[NSCAN];
};

__device__ inline Scan5 block_scan5(Scan5 x, int (*warp_tot)[NSCAN], int tid)
{
    const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
#pragma unroll
        for (int i = 0; i < NSCAN; i++) {
            const int y = __shfl_up_sync(0xffffffffu, x.v[i], off);
            if (lane >= off) x.v[i] += y;
        }
    }
    if (lane == 31) {
#pragma unroll
        for (int i = 0; i < NSCAN; i++) warp_tot[warp][i] = x.v[i];
    }
    __syncthreads();
    if (warp == 0) {
        Scan5 t;
#pragma unroll
        for (int i = 0; i < NSCAN; i++) t.v[i] = warp_tot[lane][i];
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
#pragma unroll
            for (int i = 0; i < NSCAN; i++) {
                const int y = __shfl_up_sync(0xffffffffu, t.v[i], off);
                if (lane >= off) t.v[i] += y;
            }
        }
#pragma unroll
        for (int i = 0; i < NSCAN; i++) warp_tot[lane][i] = t.v[i];   // inclusive totals up to and including warp `lane`
    }
    __syncthreads();
    if (warp > 0) {
#pragma unroll
        for (int i = 0; i < NSCAN; i++) x.v[i] += warp_tot[warp - 1][i];
    }
    return x;
}

// per chunk of pairs: every pair's position among its chunk's pairs of the same expert, and the chunk's counts
__global__ void __launch_bounds__(GROUP_THREADS) k_group_count(const uint32_t *__restrict__ idx, int npairs, int base,
                                                               int E_local, int stride, int rem, Groups g)
{
    __shared__ int cnt[1024];
    const int tid = threadIdx.x;
    cnt[tid] = 0;
    pdl_wait();
    pdl_launch_dependents();
    __syncthreads();
    const int p = blockIdx.x * GROUP_CHUNK + tid;
    if (p < npairs) {
        const int e = local_expert(idx[p], base, E_local, stride, rem);
        g.pos[p] = e >= 0 ? atomicAdd(&cnt[e], 1) : -1;
    }
    __syncthreads();
    if (tid < E_local) g.chunk_cnt[(size_t)blockIdx.x * E_local + tid] = cnt[tid];
}

// n_chunks == 0: the whole sort in this CTA.  Otherwise k_group_count has run: the counts are the sums over the
// chunks (whose entries become the expert's pairs in earlier chunks), and k_group_scatter follows.
__global__ void __launch_bounds__(GROUP_THREADS) k_group(const uint32_t *__restrict__ idx, int npairs, int base,
                                                         int E_local, int stride, int rem, Groups g, int n_chunks)
{
    __shared__ int cnt[1024];
    __shared__ int warp_tot[32][NSCAN];
    const int tid = threadIdx.x;
    cnt[tid] = 0;
    pdl_wait();
    pdl_launch_dependents();
    __syncthreads();
    int c = 0;
    if (n_chunks == 0) {
        for (int p = tid; p < npairs; p += GROUP_THREADS) {
            const int e = local_expert(idx[p], base, E_local, stride, rem);
            int pos = -1;
            if (e >= 0) pos = atomicAdd(&cnt[e], 1);
            g.pos[p] = pos;
        }
        __syncthreads();
        c = tid < E_local ? cnt[tid] : 0;
    } else if (tid < E_local) {
        for (int b = 0; b < n_chunks; b++) {
            const int v = g.chunk_cnt[(size_t)b * E_local + tid];
            g.chunk_cnt[(size_t)b * E_local + tid] = c;
            c += v;
        }
    }
    const int flag = c > 0 ? 1 : 0;
    const int cost = (c + GEMV_TG - 1) / GEMV_TG;
    const int tiles = (c + PREFILL_NT - 1) / PREFILL_NT;
    const int wcost = (c + GEMV_TG_WIDE - 1) / GEMV_TG_WIDE;
    const int mcost = (c + GEMV_TG_MMA - 1) / GEMV_TG_MMA;
    Scan5 in;
    in.v[0] = c; in.v[1] = flag; in.v[2] = cost; in.v[3] = tiles; in.v[4] = wcost; in.v[5] = mcost;
    const Scan5 sc = block_scan5(in, warp_tot, tid);   // inclusive
    const int excl = sc.v[0] - c;
    if (tid < E_local) {
        g.count[tid] = c;
        g.offset[tid] = excl;
        if (flag) {
            const int slot = sc.v[1] - 1;
            g.active[slot] = tid;
            g.cost_prefix[slot] = sc.v[2] - cost;
            g.cost_prefix_wide[slot] = sc.v[4] - wcost;
            g.cost_prefix_mma[slot] = sc.v[5] - mcost;
            g.tile_prefix[slot] = sc.v[3] - tiles;
            for (int i = 0; i < tiles; i++) g.tile_table[sc.v[3] - tiles + i] = make_int2(tid, i);
        }
    }
    if (tid == GROUP_THREADS - 1) {
        g.offset[E_local] = sc.v[0];
        *g.n_active = sc.v[1];
        g.cost_prefix[sc.v[1]] = sc.v[2];
        g.cost_prefix_wide[sc.v[1]] = sc.v[4];
        g.cost_prefix_mma[sc.v[1]] = sc.v[5];
        g.tile_prefix[sc.v[1]] = sc.v[3];
    }
    if (n_chunks) return;
    __syncthreads();   // every thread has read its count
    cnt[tid] = excl;   // reuse as the per-expert base
    __syncthreads();
    for (int p = tid; p < npairs; p += GROUP_THREADS) {
        int pos = g.pos[p];
        if (pos >= 0) {
            const int e = local_expert(idx[p], base, E_local, stride, rem);
            g.pairs[cnt[e] + pos] = p;
        }
    }
}

// per chunk of pairs: positions inside the chunk become positions inside the expert's list, and the pairs go to their places
__global__ void __launch_bounds__(GROUP_THREADS) k_group_scatter(const uint32_t *__restrict__ idx, int npairs, int base,
                                                                 int E_local, int stride, int rem, Groups g)
{
    pdl_wait();
    pdl_launch_dependents();
    const int p = blockIdx.x * GROUP_CHUNK + threadIdx.x;
    if (p >= npairs) return;
    const int pos = g.pos[p];
    if (pos < 0) return;
    const int e = local_expert(idx[p], base, E_local, stride, rem);
    const int fp = g.chunk_cnt[(size_t)blockIdx.x * E_local + e] + pos;
    g.pos[p] = fp;
    g.pairs[g.offset[e] + fp] = p;
}

cudaError_t launch_group(const LayerDev &L, const Workspace &ws, const uint32_t *idx, int n, int top_k,
                         cudaStream_t s)
{
    const int npairs = n * top_k;
    const int n_chunks = npairs >= GROUP_MULTI_MIN ? (npairs + GROUP_CHUNK - 1) / GROUP_CHUNK : 0;
    cudaError_t e = cudaSuccess;
    if (n_chunks) {
        e = launch_pdl(k_group_count, dim3(n_chunks), dim3(GROUP_THREADS), 0, s, idx, npairs, L.expert_base, L.E_local, L.ep_stride,
                       L.ep_rem, ws.groups);
        count_launch();
        if (e != cudaSuccess) return e;
    }
    e = launch_pdl(k_group, dim3(1), dim3(GROUP_THREADS), 0, s, idx, npairs, L.expert_base, L.E_local, L.ep_stride, L.ep_rem,
                   ws.groups, n_chunks);
    count_launch();
    if (e != cudaSuccess || !n_chunks) return e;
    e = launch_pdl(k_group_scatter, dim3(n_chunks), dim3(GROUP_THREADS), 0, s, idx, npairs, L.expert_base, L.E_local, L.ep_stride,
                   L.ep_rem, ws.groups);
    count_launch();
    return e;
}

// ---------------------------------------------------------------- router statistics
// What the reference's auxiliary losses take from (router_logits, selected_experts) of one block
// (compute_z_loss / compute_load_balance_loss, qwen3_next.rs:5549-5648):
//   counts[e] = number of selections of expert e (ids >= E are skipped),
//   z    = mean_t logsumexp(logits_t)^2,
//   lb   = E * sum_e (counts[e] / (n*k)) * mean_t softmax(logits_t)[e].
// Every sum runs in a fixed order (no float atomics), so repeated calls give the same bits.
constexpr int STATS_CHUNK = 256;  // tokens per partial column sum

// one warp per token: max, 1 / sum exp, logsumexp
__global__ void __launch_bounds__(128) k_stats_tokens(const float *__restrict__ logits, int n, int E,
                                                      float *__restrict__ mx, float *__restrict__ inv,
                                                      float *__restrict__ lse)
{
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= n) return;
    const float *p = logits + (size_t)t * E;
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, p[e]);
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, s));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(p[e] - m);
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
    if (lane == 0) {
        mx[t] = m;
        inv[t] = 1.f / sum;
        lse[t] = m + logf(sum);
    }
}

// thread per expert column, one chunk of tokens per grid row: partial[chunk][e] = sum_t softmax(logits_t)[e]
__global__ void __launch_bounds__(128) k_stats_columns(const float *__restrict__ logits, int n, int E,
                                                       const float *__restrict__ mx, const float *__restrict__ inv,
                                                       float *__restrict__ partial)
{
    const int e = blockIdx.x * 128 + threadIdx.x;
    if (e >= E) return;
    const int t0 = blockIdx.y * STATS_CHUNK, t1 = min(n, t0 + STATS_CHUNK);
    float acc = 0.f;
    for (int t = t0; t < t1; t++) acc += expf(logits[(size_t)t * E + e] - mx[t]) * inv[t];
    partial[(size_t)blockIdx.y * E + e] = acc;
}

// one CTA: selection counts (integer atomics in shared memory), then the two losses
__global__ void __launch_bounds__(1024) k_stats_final(const uint32_t *__restrict__ idx, int n, int top_k, int E, int chunks,
                                                      const float *__restrict__ partial, const float *__restrict__ lse,
                                                      float *__restrict__ counts_out, float *__restrict__ losses_out)
{
    extern __shared__ int cnt[];  // [E]
    __shared__ float red[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int e = tid; e < E; e += 1024) cnt[e] = 0;
    __syncthreads();
    for (int p = tid; p < n * top_k; p += 1024) {
        const uint32_t e = idx[p];
        if (e < (uint32_t)E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    float lb = 0.f, z = 0.f;
    const float total = (float)n * (float)top_k;
    for (int e = tid; e < E; e += 1024) {
        float p = 0.f;
        for (int c = 0; c < chunks; c++) p += partial[(size_t)c * E + e];
        const float f = (float)cnt[e] / total;
        lb += f * (p / (float)n);
        if (counts_out) counts_out[e] = (float)cnt[e];
    }
    for (int t = tid; t < n; t += 1024) z += lse[t] * lse[t];
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        lb += __shfl_xor_sync(0xffffffffu, lb, s);
        z += __shfl_xor_sync(0xffffffffu, z, s);
    }
    if (lane == 0) red[warp] = lb;
    __syncthreads();
    float lb_all = 0.f;
    if (tid == 0)
        for (int w = 0; w < 32; w++) lb_all += red[w];
    __syncthreads();
    if (lane == 0) red[warp] = z;
    __syncthreads();
    if (tid == 0 && losses_out) {
        float z_all = 0.f;
        for (int w = 0; w < 32; w++) z_all += red[w];
        losses_out[0] = z_all / (float)n;
        losses_out[1] = lb_all * (float)E;
    }
}

size_t router_stats_scratch_floats(int n, int E) { return 3 * (size_t)n + (size_t)((n + STATS_CHUNK - 1) / STATS_CHUNK) * E; }

cudaError_t launch_router_stats(const float *logits, const uint32_t *idx, int n, int top_k, int E, float *scratch,
                                float *counts_out, float *losses_out, cudaStream_t s)
{
    if (n <= 0) return cudaSuccess;
    float *mx = scratch, *inv = scratch + n, *lse = scratch + 2 * (size_t)n, *partial = scratch + 3 * (size_t)n;
    const int chunks = (n + STATS_CHUNK - 1) / STATS_CHUNK;
    k_stats_tokens<<<(n + 3) / 4, 128, 0, s>>>(logits, n, E, mx, inv, lse);
    k_stats_columns<<<dim3((E + 127) / 128, chunks), 128, 0, s>>>(logits, n, E, mx, inv, partial);
    k_stats_final<<<1, 1024, (size_t)E * sizeof(int), s>>>(idx, n, top_k, E, chunks, partial, lse, counts_out, losses_out);
    count_launch(3);
    return cudaGetLastError();
}

}  // namespace pmoe
