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
// Each CTA owns a slice of rows of one expert's matrix.  One elected thread streams the
// slice into shared memory with bulk (TMA) copies -- every weight byte crosses HBM once,
// in contiguous 16-byte-aligned runs -- while the warps fetch the quantised activations
// of the expert's tokens into registers.  A lane owns a fixed slice of the reduction
// dimension, so its activation registers serve every row of the slice; a row's partial
// sums meet in a shuffle reduction.
#include "pmoe_common.cuh"
#include "pmoe_quant.cuh"

namespace pmoe {

constexpr int GEMV_WARPS = 4;
constexpr int GATE_UP_ROWS = 16;  // rows of gate AND of up per CTA
constexpr int DOWN_ROWS = 64;
constexpr int BULK_PIECE = 16384; // bytes per bulk copy

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

template <int DT> struct Tr;
template <> struct Tr<PMOE_Q4_K> {
    static constexpr int UNIT = 64;
    static constexpr bool KQ = true;
    using Act = ActQ4K;
};
template <> struct Tr<PMOE_Q6_K> {
    static constexpr int UNIT = 16;
    static constexpr bool KQ = true;
    using Act = ActQ16;
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
template <> __device__ inline void zero_act<PMOE_Q6_K>(ActQ16 &o)
{
#pragma unroll
    for (int i = 0; i < 4; i++) o.a[i] = 0;
    o.dx = 0.f;
}
template <> __device__ inline void zero_act<PMOE_Q8_0>(ActQ16 &o) { zero_act<PMOE_Q6_K>(o); }

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

template <> __device__ inline void load_act<PMOE_Q6_K>(const QAct &q, size_t row, int K, int u, ActQ16 &o)
{
    const int b = u >> 4, half = (u >> 3) & 1, j = u & 7;
    const uint32_t *p = reinterpret_cast<const uint32_t *>(q.qs + row * K + 256 * b + 128 * half + 4 * j);
    o.a[0] = p[0]; o.a[1] = p[8]; o.a[2] = p[16]; o.a[3] = p[24];
    o.dx = q.d[row * (K / QK_K) + b];
}

template <> __device__ inline void load_act<PMOE_Q8_0>(const QAct &q, size_t row, int K, int u, ActQ16 &o)
{
    const int b = u >> 1, hf = u & 1;
    const uint4 v = *reinterpret_cast<const uint4 *>(q.qs + row * K + 32 * b + 16 * hf);
    o.a[0] = v.x; o.a[1] = v.y; o.a[2] = v.z; o.a[3] = v.w;
    o.dx = q.d[row * (K / QK8_0) + b];
}

// Decodes unit u of the row at `row` (shared memory) once and adds its dot product with
// each token's activations to acc[].
template <int DT, int TG>
__device__ inline void unit_dot(const uint8_t *row, int u, const typename Tr<DT>::Act (&act)[TG], float (&acc)[TG]);

template <int TG> __device__ inline void unit_dot_q4k(const uint8_t *row, int u, const ActQ4K (&act)[TG], float (&acc)[TG])
{
    const uint8_t *blk = row + (u >> 2) * Q4_K_BYTES;
    const int qd = u & 3;
    const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
    const uint4 qa = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * qd);
    const uint4 qb = *reinterpret_cast<const uint4 *>(blk + 32 + 32 * qd);
    const float d = half_bits_to_float((uint16_t)(hdr.x & 0xffffu));
    const float dmin = half_bits_to_float((uint16_t)(hdr.x >> 16));
    const uint32_t s0 = hdr.y, s1 = hdr.z, s2 = hdr.w;
    int sc0, sc1, m0, m1;  // 6-bit scale / min of sub-blocks 2*qd and 2*qd+1
    if (qd < 2) {
        const int sh = 16 * qd;
        sc0 = (s0 >> sh) & 63; sc1 = (s0 >> (sh + 8)) & 63;
        m0 = (s1 >> sh) & 63;  m1 = (s1 >> (sh + 8)) & 63;
    } else {
        const int sh = 16 * (qd - 2);
        sc0 = ((s2 >> sh) & 0xF) | (((s0 >> (sh + 6)) & 3) << 4);
        sc1 = ((s2 >> (sh + 8)) & 0xF) | (((s0 >> (sh + 14)) & 3) << 4);
        m0 = ((s2 >> (sh + 4)) & 0xF) | (((s1 >> (sh + 6)) & 3) << 4);
        m1 = ((s2 >> (sh + 12)) & 0xF) | (((s1 >> (sh + 14)) & 3) << 4);
    }
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    uint32_t lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        lo[i] = w[i] & 0x0F0F0F0Fu;
        hi[i] = (w[i] >> 4) & 0x0F0F0F0Fu;
    }
#pragma unroll
    for (int t = 0; t < TG; t++) {
        int s_lo = 0, s_hi = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            s_lo = __dp4a((int)lo[i], (int)act[t].a[i], s_lo);
            s_hi = __dp4a((int)hi[i], (int)act[t].a[8 + i], s_hi);
        }
        const int isum = sc0 * s_lo + sc1 * s_hi;
        const int imin = m0 * act[t].bs_lo + m1 * act[t].bs_hi;
        acc[t] += act[t].dx * (d * (float)isum - dmin * (float)imin);
    }
}

template <int TG> __device__ inline void unit_dot_q6k(const uint8_t *row, int u, const ActQ16 (&act)[TG], float (&acc)[TG])
{
    const uint8_t *blk = row + (u >> 4) * Q6_K_BYTES;  // 2-byte aligned
    const int half = (u >> 3) & 1, j = u & 7;
    const uint32_t la = lds_u32_a2(blk + 64 * half + 4 * j);
    const uint32_t lb = lds_u32_a2(blk + 64 * half + 32 + 4 * j);
    const uint32_t h = lds_u32_a2(blk + 128 + 32 * half + 4 * j);
    const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192 + 8 * half + (j >> 2));
    const int c0 = sc[0], c1 = sc[2], c2 = sc[4], c3 = sc[6];
    const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk + 208));
    const uint32_t w1 = __vsub4((la & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u), 0x20202020u);
    const uint32_t w2 = __vsub4((lb & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u), 0x20202020u);
    const uint32_t w3 = __vsub4(((la >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u), 0x20202020u);
    const uint32_t w4 = __vsub4(((lb >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u), 0x20202020u);
#pragma unroll
    for (int t = 0; t < TG; t++) {
        const int isum = c0 * __dp4a((int)w1, (int)act[t].a[0], 0) + c1 * __dp4a((int)w2, (int)act[t].a[1], 0) +
                         c2 * __dp4a((int)w3, (int)act[t].a[2], 0) + c3 * __dp4a((int)w4, (int)act[t].a[3], 0);
        acc[t] += (d * act[t].dx) * (float)isum;
    }
}

template <int TG> __device__ inline void unit_dot_q80(const uint8_t *row, int u, const ActQ16 (&act)[TG], float (&acc)[TG])
{
    const uint8_t *blk = row + (u >> 1) * Q8_0_BYTES;  // 2-byte aligned
    const int hf = u & 1;
    const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk));
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) w[i] = lds_u32_a2(blk + 2 + 16 * hf + 4 * i);
#pragma unroll
    for (int t = 0; t < TG; t++) {
        int isum = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) isum = __dp4a((int)w[i], (int)act[t].a[i], isum);
        acc[t] += (d * act[t].dx) * (float)isum;
    }
}

template <> __device__ inline void unit_dot<PMOE_Q4_K, 4>(const uint8_t *r, int u, const ActQ4K (&a)[4], float (&c)[4]) { unit_dot_q4k<4>(r, u, a, c); }
template <> __device__ inline void unit_dot<PMOE_Q4_K, 8>(const uint8_t *r, int u, const ActQ4K (&a)[8], float (&c)[8]) { unit_dot_q4k<8>(r, u, a, c); }
template <> __device__ inline void unit_dot<PMOE_Q6_K, 4>(const uint8_t *r, int u, const ActQ16 (&a)[4], float (&c)[4]) { unit_dot_q6k<4>(r, u, a, c); }
template <> __device__ inline void unit_dot<PMOE_Q6_K, 8>(const uint8_t *r, int u, const ActQ16 (&a)[8], float (&c)[8]) { unit_dot_q6k<8>(r, u, a, c); }
template <> __device__ inline void unit_dot<PMOE_Q8_0, 4>(const uint8_t *r, int u, const ActQ16 (&a)[4], float (&c)[4]) { unit_dot_q80<4>(r, u, a, c); }
template <> __device__ inline void unit_dot<PMOE_Q8_0, 8>(const uint8_t *r, int u, const ActQ16 (&a)[8], float (&c)[8]) { unit_dot_q80<8>(r, u, a, c); }

// ---------------------------------------------------------------- kernel arguments
struct GemvArgs {
    const uint8_t *w0, *w1;    // routed matrices (gate, up) or (down, unused); expert e at + e*expert_bytes
    size_t expert_bytes;
    const uint8_t *sw0, *sw1;  // shared expert matrices
    int K;                     // reduction length (H for gate/up, F for down)
    int rows_total;            // output length (F for gate/up, H for down)
    int routed_slots;          // grid.y entries that serve routed experts
    int has_shared;            // one more grid.y entry serves the shared expert
    int n, top_k;
    Groups g;
    QAct in_r, in_s;           // quantised activations matching the routed / shared weight type
    float *out;                // act [., F] or partial [., H]
    const float *scale_r;      // routing weights [n*top_k]      (down only)
    const float *scale_s;      // shared gate sigmoid [n]        (down only)
    DevStatus *status;
};

// UPL = units per lane (compile-time bound; K <= UPL*32*UNIT), TG = tokens per pass.
template <int DT, int NMAT, int UPL, int TG, int ROWS>
__device__ inline void gemv_cta(const GemvArgs &A, uint8_t *smem, uint64_t *bar, bool is_shared, const uint8_t *wsrc0,
                                const uint8_t *wsrc1, int m, const int *list, const QAct &in)
{
    using Act = typename Tr<DT>::Act;
    constexpr int UNIT = Tr<DT>::UNIT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = A.K;
    const uint32_t rb = (uint32_t)row_bytes(DT, K);
    const uint32_t slice = rb * ROWS;  // bytes of one matrix slice
    const int chunk = blockIdx.x;

    // ---- stream the weight slice(s) into shared memory
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_expect_tx(bar, slice * NMAT);
#pragma unroll
        for (int mat = 0; mat < NMAT; mat++) {
            const uint8_t *src = (mat == 0 ? wsrc0 : wsrc1) + (size_t)chunk * slice;
            uint8_t *dst = smem + mat * slice;
            for (uint32_t off = 0; off < slice; off += BULK_PIECE) {
                uint32_t sz = slice - off < (uint32_t)BULK_PIECE ? slice - off : (uint32_t)BULK_PIECE;
                bulk_g2s(dst + off, src + off, sz, bar);
            }
        }
    }

    const int units = K / UNIT;
    const int lpr = units < 32 ? units : 32;      // lanes per row (power of two)
    const int rpp = 32 / lpr;                     // rows per warp pass
    const int sub = lane / lpr, ul = lane % lpr;
    constexpr int ROWS_PER_WARP = ROWS / GEMV_WARPS;
    bool waited = false;

    for (int t0 = 0; t0 < m; t0 += TG) {
        // ---- this pass's token rows
        Act act[UPL][TG];
        int out_row[TG];
        float scale[TG];
#pragma unroll
        for (int t = 0; t < TG; t++) {
            const bool valid = t0 + t < m;
            int in_row = 0;
            out_row[t] = -1;
            scale[t] = 0.f;
            if (valid) {
                if (is_shared) {
                    const int tok = t0 + t;
                    out_row[t] = A.n * A.top_k + tok;
                    in_row = NMAT == 2 ? tok : out_row[t];
                    if (NMAT == 1) scale[t] = A.scale_s[tok];
                } else {
                    const int p = list[t0 + t];
                    out_row[t] = p;
                    in_row = NMAT == 2 ? p / A.top_k : p;
                    if (NMAT == 1) scale[t] = A.scale_r[p];
                }
            }
#pragma unroll
            for (int i = 0; i < UPL; i++) {
                const int u = i * lpr + ul;
                if (valid && u < units) load_act<DT>(in, (size_t)in_row, K, u, act[i][t]);
                else zero_act<DT>(act[i][t]);
            }
        }
        if (!waited) {
            if (!mbar_wait(bar, 0)) {
                set_status(A.status, PMOE_ERR_TIMEOUT, NMAT, chunk);
                return;
            }
            waited = true;
        }
        // ---- rows of this warp
        for (int r0 = 0; r0 < ROWS_PER_WARP; r0 += rpp) {
            const int rloc = r0 + sub;
            const bool row_ok = rloc < ROWS_PER_WARP;
            const int row = warp * ROWS_PER_WARP + (row_ok ? rloc : 0);
            float acc[NMAT][TG];
#pragma unroll
            for (int mat = 0; mat < NMAT; mat++) {
#pragma unroll
                for (int t = 0; t < TG; t++) acc[mat][t] = 0.f;
                const uint8_t *rp = smem + mat * slice + (size_t)row * rb;
#pragma unroll
                for (int i = 0; i < UPL; i++) {
                    const int u = i * lpr + ul;
                    if (u < units) unit_dot<DT, TG>(rp, u, act[i], acc[mat]);
                }
#pragma unroll
                for (int t = 0; t < TG; t++) {
                    float v = acc[mat][t];
                    for (int s = lpr >> 1; s >= 1; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
                    acc[mat][t] = v;
                }
            }
            if (ul == 0 && row_ok) {
                const int orow = chunk * ROWS + row;
#pragma unroll
                for (int t = 0; t < TG; t++) {
                    if (out_row[t] < 0) continue;
                    float v;
                    if (NMAT == 2) {
                        const float g = acc[0][t];
                        v = g / (1.f + expf(-g)) * acc[NMAT - 1][t];
                    } else {
                        v = acc[0][t] * scale[t];
                    }
                    A.out[(size_t)out_row[t] * A.rows_total + orow] = v;
                }
            }
        }
    }
    // every issued copy has landed before the CTA may exit
    if (!waited && !mbar_wait(bar, 0)) set_status(A.status, PMOE_ERR_TIMEOUT, NMAT, chunk);
}

template <int DT> struct Upl {  // units per lane at the largest supported K for the kernel kind
    static constexpr int gate_up = (2048 / Tr<DT>::UNIT) / 32;                        // K <= 2048
    static constexpr int down = (512 / Tr<DT>::UNIT) / 32 > 0 ? (512 / Tr<DT>::UNIT) / 32 : 1;  // K <= 512
};

// DT_S == 0 compiles the kernel without a shared-expert branch.
template <int DT_R, int DT_S, int NMAT>
__global__ void __launch_bounds__(GEMV_WARPS * 32) k_expert_gemv(const GemvArgs A)
{
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem_raw);
    uint8_t *smem = smem_raw + 128;
    constexpr int ROWS = NMAT == 2 ? GATE_UP_ROWS : DOWN_ROWS;
    // tokens per pass: bounded by the activation registers a lane keeps (64 per token group)
    constexpr int TG_R = (NMAT == 2 || DT_R == PMOE_Q4_K) ? 4 : 8;
    constexpr int TG_S = (NMAT == 2 || DT_S == PMOE_Q4_K) ? 4 : 8;
    const int slot = blockIdx.y;
    if (slot >= A.routed_slots) {
        if constexpr (DT_S != 0) {
            constexpr int UPL = NMAT == 2 ? Upl<DT_S>::gate_up : Upl<DT_S>::down;
            gemv_cta<DT_S, NMAT, UPL, TG_S, ROWS>(A, smem, bar, true, A.sw0, A.sw1, A.n, nullptr, A.in_s);
        }
        return;
    }
    if (slot >= *A.g.n_active) return;
    const int e = A.g.active[slot];
    const int m = A.g.count[e];
    const int *list = A.g.pairs + A.g.offset[e];
    constexpr int UPL = NMAT == 2 ? Upl<DT_R>::gate_up : Upl<DT_R>::down;
    gemv_cta<DT_R, NMAT, UPL, TG_R, ROWS>(A, smem, bar, false, A.w0 + (size_t)e * A.expert_bytes,
                                        A.w1 + (size_t)e * A.expert_bytes, m, list, A.in_r);
}

// ---------------------------------------------------------------- host-side dispatch
bool gemv_supported(int dtype, int K, int rows, const char **why)
{
    if (dtype != PMOE_Q4_K && dtype != PMOE_Q6_K && dtype != PMOE_Q8_0) {
        *why = "expert weights must be Q4_K, Q6_K or Q8_0";
        return false;
    }
    if (K < 256 || K > 2048 || (K & (K - 1))) {
        *why = "reduction length must be a power of two in [256, 2048]";
        return false;
    }
    if (rows % DOWN_ROWS) {
        *why = "output length must be a multiple of 64";
        return false;
    }
    return true;
}

static size_t gemv_smem(int dt, int K, int nmat)
{
    if (!dt) return 0;
    return row_bytes(dt, K) * (nmat == 2 ? GATE_UP_ROWS * 2 : DOWN_ROWS);
}

template <int DT_R, int DT_S, int NMAT>
static cudaError_t launch_gemv_t(const GemvArgs &A, int dt_s_rt, dim3 grid, cudaStream_t s)
{
    size_t smem = 128 + (gemv_smem(DT_R, A.K, NMAT) > gemv_smem(dt_s_rt, A.K, NMAT) ? gemv_smem(DT_R, A.K, NMAT)
                                                                                     : gemv_smem(dt_s_rt, A.K, NMAT));
    auto kern = k_expert_gemv<DT_R, DT_S, NMAT>;
    static size_t configured = 0;  // per instantiation
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = smem;
    }
    kern<<<grid, GEMV_WARPS * 32, smem, s>>>(A);
    count_launch();
    return cudaGetLastError();
}

template <int DT_R, int NMAT>
static cudaError_t launch_gemv_s(const GemvArgs &A, int dt_s, dim3 grid, cudaStream_t s)
{
    switch (dt_s) {
    case 0: return launch_gemv_t<DT_R, 0, NMAT>(A, 0, grid, s);
    case PMOE_Q4_K: return launch_gemv_t<DT_R, PMOE_Q4_K, NMAT>(A, dt_s, grid, s);
    case PMOE_Q6_K: return launch_gemv_t<DT_R, PMOE_Q6_K, NMAT>(A, dt_s, grid, s);
    case PMOE_Q8_0: return launch_gemv_t<DT_R, PMOE_Q8_0, NMAT>(A, dt_s, grid, s);
    }
    return cudaErrorInvalidValue;
}

template <int NMAT>
static cudaError_t launch_gemv(const GemvArgs &A, int dt_r, int dt_s, dim3 grid, cudaStream_t s)
{
    switch (dt_r) {
    case PMOE_Q4_K: return launch_gemv_s<PMOE_Q4_K, NMAT>(A, dt_s, grid, s);
    case PMOE_Q6_K: return launch_gemv_s<PMOE_Q6_K, NMAT>(A, dt_s, grid, s);
    case PMOE_Q8_0: return launch_gemv_s<PMOE_Q8_0, NMAT>(A, dt_s, grid, s);
    }
    return cudaErrorInvalidValue;
}

static int routed_slots_for(const LayerDev &L, int n, int top_k)
{
    long pairs = (long)n * top_k;
    return (int)(pairs < L.E_local ? pairs : L.E_local);
}

cudaError_t launch_gate_up(const LayerDev &L, const Workspace &ws, int n, int top_k, bool routed, bool shared,
                           cudaStream_t s)
{
    if (n <= 0 || (!routed && !shared)) return cudaSuccess;
    GemvArgs A{};
    A.w0 = L.gate_exps; A.w1 = L.up_exps;
    A.expert_bytes = row_bytes(L.gate_dtype, L.H) * L.F;
    A.sw0 = L.sh_gate; A.sw1 = L.sh_up;
    A.K = L.H; A.rows_total = L.F;
    A.routed_slots = routed ? routed_slots_for(L, n, top_k) : 0;
    A.has_shared = shared;
    A.n = n; A.top_k = top_k;
    A.g = ws.groups;
    A.in_r = is_kquant(L.gate_dtype) ? ws.x_q8k : ws.x_q80;
    A.in_s = is_kquant(L.sh_gate_dtype) ? ws.x_q8k : ws.x_q80;
    A.out = ws.act;
    A.status = ws.status;
    dim3 grid(L.F / GATE_UP_ROWS, A.routed_slots + (shared ? 1 : 0));
    // a kernel without routed slots still needs a routed type to instantiate; reuse the shared one
    int dt_r = routed ? L.gate_dtype : L.sh_gate_dtype;
    return launch_gemv<2>(A, dt_r, shared ? L.sh_gate_dtype : 0, grid, s);
}

cudaError_t launch_down(const LayerDev &L, const Workspace &ws, const float *w, int n, int top_k, bool routed,
                        bool shared, cudaStream_t s)
{
    if (n <= 0 || (!routed && !shared)) return cudaSuccess;
    GemvArgs A{};
    A.w0 = L.down_exps; A.w1 = nullptr;
    A.expert_bytes = row_bytes(L.down_dtype, L.F) * L.H;
    A.sw0 = L.sh_down; A.sw1 = nullptr;
    A.K = L.F; A.rows_total = L.H;
    A.routed_slots = routed ? routed_slots_for(L, n, top_k) : 0;
    A.has_shared = shared;
    A.n = n; A.top_k = top_k;
    A.g = ws.groups;
    A.in_r = is_kquant(L.down_dtype) ? ws.act_q8k : ws.act_q80;
    A.in_s = is_kquant(L.sh_down_dtype) ? ws.act_q8k : ws.act_q80;
    A.out = ws.partial;
    A.scale_r = w;
    A.scale_s = ws.sh_sigmoid;
    A.status = ws.status;
    dim3 grid(L.H / DOWN_ROWS, A.routed_slots + (shared ? 1 : 0));
    int dt_r = routed ? L.down_dtype : L.sh_down_dtype;
    return launch_gemv<1>(A, dt_r, shared ? L.sh_down_dtype : 0, grid, s);
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
    k_act_quant<<<rows, 64, 0, s>>>(ws.act, L.F, n * top_k, ws.groups.pos, routed, L.down_dtype, L.sh_down_dtype,
                                    ws.act_q8k, ws.act_q80);
    count_launch();
    return cudaGetLastError();
}

// ---------------------------------------------------------------- combine
// out[t] = sum over the token's local slots (slot order) of its weighted down rows, plus the
// gated shared-expert row (forward_batched's weighted sum, qwen3_next.rs:1391-1393, and the
// final add, 1932-1937).
template <typename OT>
__global__ void __launch_bounds__(256) k_combine(const float *__restrict__ partial, const int *__restrict__ pos,
                                                 int n, int top_k, int H, bool routed, bool shared,
                                                 OT *__restrict__ out)
{
    const int t = blockIdx.x;
    for (int h = threadIdx.x * 4; h < H; h += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (routed) {
            for (int j = 0; j < top_k; j++) {
                const int p = t * top_k + j;
                if (pos[p] < 0) continue;
                const float4 v = *reinterpret_cast<const float4 *>(partial + (size_t)p * H + h);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
        }
        if (shared) {
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
    if (out_dtype == PMOE_F32)
        k_combine<float><<<n, 256, 0, s>>>(ws.partial, ws.groups.pos, n, top_k, L.H, routed, shared, (float *)out);
    else
        k_combine<__nv_bfloat16><<<n, 256, 0, s>>>(ws.partial, ws.groups.pos, n, top_k, L.H, routed, shared,
                                                   (__nv_bfloat16 *)out);
    count_launch();
    return cudaGetLastError();
}

}  // namespace pmoe
