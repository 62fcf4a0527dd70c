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

#include "pmoe_gemv.cuh"

namespace pmoe {

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

int sm_count()
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
    if (routed && L.gate_dtype == PMOE_Q4_K && L.H == 2048 && L.F == 512 && mma_enabled(1))
        return launch_gate_up_q4k_mma(A, shared ? L.sh_gate_dtype : 0, s);
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
    // Q2_K / Q3_K shared matrices only come beside routed matrices of their own type, never beside Q6_K
    if (routed && L.down_dtype == PMOE_Q6_K && L.H == 2048 && L.F == 512 && mma_enabled(2))
        return launch_down_q6k_mma(A, shared ? L.sh_down_dtype : 0, s);
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
    count_launch();
    return launch_qmatmul_quantised(dtype, w, rows, K, a, m, y, s);
}

cudaError_t launch_qmatmul_quantised(int dtype, const void *w, int rows, int K, const QAct &a, int m, float *y, cudaStream_t s)
{
    dim3 grid((rows + 3) / 4, (m + TG - 1) / TG);
    const uint8_t *wb = (const uint8_t *)w;
    if (dtype == PMOE_Q4_K) k_qmatmul<PMOE_Q4_K><<<grid, 128, 0, s>>>(wb, rows, K, a, m, y);
    else if (dtype == PMOE_Q2_K) k_qmatmul<PMOE_Q2_K><<<grid, 128, 0, s>>>(wb, rows, K, a, m, y);
    else if (dtype == PMOE_Q3_K) k_qmatmul<PMOE_Q3_K><<<grid, 128, 0, s>>>(wb, rows, K, a, m, y);
    else if (dtype == PMOE_Q5_K) k_qmatmul<PMOE_Q5_K><<<grid, 128, 0, s>>>(wb, rows, K, a, m, y);
    else if (dtype == PMOE_Q6_K) k_qmatmul<PMOE_Q6_K><<<grid, 128, 0, s>>>(wb, rows, K, a, m, y);
    else k_qmatmul<PMOE_Q8_0><<<grid, 128, 0, s>>>(wb, rows, K, a, m, y);
    count_launch();
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
