// Shared device/host definitions of libpmoe: GGUF block layouts, small PTX wrappers,
// the workspace layout and the internal launch interface between the .cu files.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pmoe.h"

#define QK_K 256
#define QK8_0 32

namespace pmoe {

// ---------------------------------------------------------------- GGUF block layouts
// Q8_0:  34 B = f16 d, int8 qs[32]
// Q2_K:  84 B = u8 scales[16] (4-bit scale | 4-bit min << 4 per 16 weights), u8 qs[64] (2 bits), f16 d, f16 dmin
// Q3_K: 110 B = u8 hmask[32] (third bits), u8 qs[64] (2 bits), u8 scales[12] (16 x 6 bits, offset 32), f16 d
// Q4_K: 144 B = f16 d, f16 dmin, u8 scales[12] (8x 6-bit scale + 8x 6-bit min), u8 qs[128]
// Q5_K: 176 B = the Q4_K header, u8 qh[32] (fifth bits: bit j of qh[l] belongs to sub-block j), u8 qs[128]
// Q6_K: 210 B = u8 ql[128], u8 qh[64], i8 scales[16], f16 d
constexpr int Q8_0_BYTES = 34;
constexpr int Q2_K_BYTES = 84;
constexpr int Q3_K_BYTES = 110;
constexpr int Q4_K_BYTES = 144;
constexpr int Q5_K_BYTES = 176;
constexpr int Q6_K_BYTES = 210;

__host__ __device__ inline int block_elems(int dtype)
{
    switch (dtype) {
    case PMOE_F32: case PMOE_F16: case PMOE_BF16: return 1;
    case PMOE_Q8_0: return QK8_0;
    case PMOE_Q2_K: case PMOE_Q3_K: case PMOE_Q4_K: case PMOE_Q5_K: case PMOE_Q6_K: return QK_K;
    default: return 0;
    }
}

__host__ __device__ inline int block_bytes(int dtype)
{
    switch (dtype) {
    case PMOE_F32: return 4;
    case PMOE_F16: case PMOE_BF16: return 2;
    case PMOE_Q8_0: return Q8_0_BYTES;
    case PMOE_Q2_K: return Q2_K_BYTES;
    case PMOE_Q3_K: return Q3_K_BYTES;
    case PMOE_Q4_K: return Q4_K_BYTES;
    case PMOE_Q5_K: return Q5_K_BYTES;
    case PMOE_Q6_K: return Q6_K_BYTES;
    default: return 0;
    }
}

__host__ __device__ inline size_t row_bytes(int dtype, size_t cols)
{
    int be = block_elems(dtype);
    return be ? cols / be * (size_t)block_bytes(dtype) : 0;
}

// Activation blocks follow the weight type's dot type on the reference CPU path:
// Q2_K ... Q6_K -> Q8_K (256 values, f32 scale, 16 sums of 16); Q8_0 -> Q8_0 (32 values, f16 scale).
__host__ __device__ inline bool is_kquant(int dtype) { return dtype >= PMOE_Q2_K && dtype <= PMOE_Q6_K; }

// ---------------------------------------------------------------- status word
// Kernels never trap: a failed range check or an expired wait records a code here.
struct DevStatus {
    int code;   // 0, PMOE_ERR_TIMEOUT or PMOE_ERR_BAD_INDEX
    int where;  // kernel tag
    int detail;
};

__device__ inline void set_status(DevStatus *st, int code, int where, int detail)
{
    if (st && atomicCAS(&st->code, 0, code) == 0) {
        st->where = where;
        st->detail = detail;
    }
}

// ---------------------------------------------------------------- PTX helpers
__device__ inline uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ inline void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ inline void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ inline void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ inline void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ inline void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// One bounded wait on an mbarrier phase.  Returns false when the limit ran out.
__device__ inline bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t max_polls = (1u << 20))
{
    uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < max_polls; i++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity), "r"(20000u)  // may sleep up to ~20 us per try instead of spinning
            : "memory");
        if (done) return true;
    }
    return false;
}

// The same wait without a suspend hint: plain polling, for waits that are expected to be short.
__device__ inline bool mbar_wait_spin(uint64_t *bar, uint32_t parity, uint32_t max_polls = (1u << 24))
{
    uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < max_polls; i++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// 1-D bulk copy global -> this CTA's shared memory through the TMA unit (no multicast).
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ inline void bulk_g2s(void *smem_dst, const void *gmem_src, uint32_t bytes, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(smem_dst)),
        "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Programmatic dependent launch.  A kernel started through launch_pdl may begin while its
// predecessor in the stream still runs: it must call pdl_wait() before it reads anything an
// earlier kernel wrote or writes anything an earlier kernel may still read (the wait returns
// once every earlier grid has completed and its writes are visible).  pdl_launch_dependents()
// lets the next kernel's CTAs become resident early; where a kernel calls it after its own
// wait, its successor may rely on everything before this kernel being complete.  Both are
// no-ops in a kernel that was launched the ordinary way.
__device__ inline void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ inline void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 32-bit load from a 2-byte aligned shared-memory address
__device__ inline uint32_t lds_u32_a2(const uint8_t *p)
{
    const uint16_t *h = reinterpret_cast<const uint16_t *>(p);
    return (uint32_t)h[0] | ((uint32_t)h[1] << 16);
}

__device__ inline float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

__device__ inline float load_as_float(const float *p, size_t i) { return p[i]; }
__device__ inline float load_as_float(const __nv_bfloat16 *p, size_t i) { return __bfloat162float(p[i]); }
__device__ inline void store_from_float(float *p, size_t i, float v) { p[i] = v; }
__device__ inline void store_from_float(__nv_bfloat16 *p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// Sums V per-lane values across the LPR lanes of a row group with LPR-1 shuffles in total:
// every step halves the number of values a lane still carries.  The lane at in-group position
// pl ends with the total of value index pl / (LPR / V).  The pairing order (LPR/2, ..., 1) is
// that of a plain xor butterfly.
template <int V, int LPR> __device__ inline float transposed_reduce(float (&v)[V], int lane)
{
    int cnt = V;
#pragma unroll
    for (int step = LPR / 2; step >= 1; step >>= 1) {
        if (cnt > 1) {
            const int half = cnt / 2;
            const bool up = (lane & step) != 0;
#pragma unroll
            for (int i = 0; i < V / 2; i++) {
                if (i < half) {
                    const float send = up ? v[i] : v[i + half];
                    const float keep = up ? v[i + half] : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, step);
                }
            }
            cnt = half;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], step);
        }
    }
    return v[0];
}

// ---------------------------------------------------------------- activation blocks in the workspace
// Q8_K rows: qs int8 [rows, K], d f32 [rows, K/256], bsums i16 [rows, K/16]
// Q8_0 rows: qs int8 [rows, K], d f32 [rows, K/32] (the f16-rounded scale, widened)
struct QAct {
    int8_t *qs;
    float *d;
    int16_t *bsums;  // Q8_K only
};

// ---------------------------------------------------------------- expert lists (device)
// Built by the grouping kernels from the [n, k] routing table.
struct Groups {
    int *count;       // [E_local]
    int *offset;      // [E_local + 1] exclusive scan of count
    int *pos;         // [n*k] position of pair p inside its expert's list, -1 if not local
    int *pairs;       // [n*k] pair ids (t*k + j) sorted by expert
    int *active;      // [E_local] local expert ids with count > 0, ascending
    int *n_active;    // [1]
    int *cost_prefix; // [E_local + 1] exclusive prefix over active slots of ceil(count / GEMV_TG)
    int *cost_prefix_wide; // same with ceil(count / GEMV_TG_WIDE)
    int *cost_prefix_mma;  // same with ceil(count / GEMV_TG_MMA): 8-token groups of the tensor-core GEMV
    int *tile_prefix; // [E_local + 1] exclusive prefix over active slots of ceil(count / PREFILL_NT)
    int2 *tile_table; // [tile_prefix[n_active]] (local expert id, tile index inside the expert) per prefill tile
    int *chunk_cnt;   // [ceil(n*k / GROUP_CHUNK), E_local] scratch of the multi-CTA grouping: per chunk of pairs and
                      // expert, the count, then the number of the expert's pairs in earlier chunks
};
constexpr int GROUP_CHUNK = 1024;   // pairs per CTA of the multi-CTA grouping

// Local index of global expert id `g` on this handle, or -1 when another rank holds it (or the id is out of range).
__host__ __device__ inline int local_expert(uint32_t g, int base, int E_local, int stride, int rem)
{
    if (stride > 1) {
        const uint32_t q = g / (uint32_t)stride;
        return (g % (uint32_t)stride == (uint32_t)rem && q < (uint32_t)E_local) ? (int)q : -1;
    }
    const uint32_t e = g - (uint32_t)base;   // wraps to a large value when below base
    return e < (uint32_t)E_local ? (int)e : -1;
}

constexpr int GEMV_TG = 2;      // tokens one GEMV pass handles; the unit of the work partition
constexpr int GEMV_TG_WIDE = 4; // ... for the kernels whose activation registers are small (Q6_K / Q8_0 down)
constexpr int GEMV_TG_MMA = 8;  // tokens one pass of the tensor-core GEMV takes (the N of mma.m16n8k32)
constexpr int PREFILL_NT = 64;  // tokens per tile of the prefill GEMMs

// Everything a forward call needs, resolved to raw pointers.
struct LayerDev {
    int H, F, E, k;
    int expert_base, E_local;
    int ep_stride, ep_rem;   // round-robin placement: this handle holds the experts e with e % ep_stride == ep_rem (0: contiguous)
    int gate_dtype, up_dtype, down_dtype;
    const uint8_t *gate_exps, *up_exps, *down_exps;
    int has_shared, sh_gate_dtype, sh_up_dtype, sh_down_dtype;
    const uint8_t *sh_gate, *sh_up, *sh_down;
    const float *sh_gate_inp;
    const float *router_w, *router_bias;   // router_w: f32 [E, H], or null when the router is quantised
    const uint8_t *router_q;               // quantised router: GGUF blocks [E, H / block] of type router_dtype
    int router_dtype;                      // PMOE_F32 (16-bit weights are widened at create) or a block type
};

struct Workspace {
    int max_tokens;
    int sh_begin, sh_count;  // tokens of the current call the shared expert serves (set per call)
    DevStatus *status;
    float *logits;       // [n, E]
    uint32_t *topk_idx;  // [n, k]
    float *topk_w;       // [n, k]
    QAct x_q8k, x_q80;   // quantised input rows [n, H]
    float *sh_sigmoid;   // [n]
    Groups groups;
    float *act;          // [n*(k+1), F]  silu(gate)*up ; routed pair p at row p, shared token t at row n_cap*k + t
    QAct act_q8k, act_q80;
    __half *act_h;       // [n*(k+1), F]  fake-quantised activation for the fp16 down GEMM: the routed pairs' rows in
                         // expert-sorted order (row offset[e] + pos), then the shared expert's rows at n*k + token
    alignas(64) unsigned char act_h_map[128];   // TMA descriptor (CUtensorMap) of act_h: boxes of 64 rows x 64 halves, 128-byte swizzle
    bool act_h_map_ok;
    alignas(64) unsigned char xq_map[128];      // TMA descriptor of x_q8k.qs: boxes of one row x 128 bytes, 128-byte swizzle
    const void *xq_map_base;                    // the array it was made for
    bool xq_map_ok;
    alignas(64) unsigned char xq80_map[128];    // the same of x_q80.qs ...
    alignas(64) unsigned char xd80_map[128];    // ... and of x_q80.d as [n, H / 32] floats: boxes of one row x four floats
    const void *xq80_map_base, *xd80_map_base;
    bool xq80_map_ok;
    float *act_h_scale;  // [n*(k+1)]     power of two a row of act_h was divided by (1 unless it would leave the fp16 range)
    float *partial;      // [n*(k+1), H]  weighted down-projection rows
    int *slot_done;      // [E_local + 1 + max_tokens/8] completion counters of the gate/up kernel: per expert, the shared
                         // expert, and the shared expert's 8-token tiles (zero between calls)
};

// ---------------------------------------------------------------- launch interface
// pmoe_route.cu
cudaError_t launch_prep(const LayerDev &L, const Workspace &ws, const void *x, int x_dtype, int n,
                        bool need_q8k, bool need_q80, bool need_gate, cudaStream_t s);
// y[m, rows] = quantised rows x W^T over activations that are already quantised (the type W's dots take)
cudaError_t launch_qmatmul_quantised(int dtype, const void *w, int rows, int K, const QAct &a, int m, float *y, cudaStream_t s);
cudaError_t launch_router(const LayerDev &L, const Workspace &ws, const void *x, int x_dtype, int n,
                          float *logits, cudaStream_t s, bool prep = false, bool need_q8k = false,
                          bool need_q80 = false, bool need_gate = false);
cudaError_t launch_topk(const LayerDev &L, const Workspace &ws, const float *logits, int n,
                        uint32_t *idx, float *w, cudaStream_t s);
cudaError_t launch_group(const LayerDev &L, const Workspace &ws, const uint32_t *idx, int n, int top_k,
                         cudaStream_t s);
size_t router_stats_scratch_floats(int n, int E);
cudaError_t launch_router_stats(const float *logits, const uint32_t *idx, int n, int top_k, int E, float *scratch,
                                float *counts_out, float *losses_out, cudaStream_t s);
// pmoe_gemv.cu
cudaError_t launch_gate_up(const LayerDev &L, const Workspace &ws, int n, int top_k, bool routed,
                           bool shared, cudaStream_t s);
cudaError_t launch_act_quant(const LayerDev &L, const Workspace &ws, const uint32_t *idx, int n, int top_k,
                             bool routed, bool shared, cudaStream_t s);
cudaError_t launch_down(const LayerDev &L, const Workspace &ws, const float *w, int n, int top_k,
                        bool routed, bool shared, cudaStream_t s);
cudaError_t launch_combine(const LayerDev &L, const Workspace &ws, const uint32_t *idx, int n, int top_k,
                           bool routed, bool shared, void *out, int out_dtype, cudaStream_t s);
bool gemv_supported(int dtype, int K, int rows, const char **why);
cudaError_t launch_qmatmul(int dtype, const void *w, int rows, int K, const float *x, int m, float *y, void *scratch,
                           cudaStream_t s);
size_t qmatmul_scratch_bytes(int m, int K);
cudaError_t qmatmul_static_scratch(int device, void **ptr, size_t *bytes);
// pmoe_prefill.cu
bool prefill_supported(const LayerDev &L, const Workspace &ws, bool routed, bool shared);
cudaError_t launch_gate_up_prefill(const LayerDev &L, const Workspace &ws, int n, int top_k, bool routed, bool shared,
                                   cudaStream_t s);
bool prefill_down_supported(const LayerDev &L, const Workspace &ws, bool routed, bool shared);
// fills ws.act_h_map for ws.act_h of `rows` rows of F halves; false when the driver refuses
bool make_act_h_map(Workspace &ws, size_t rows, int F);
// the same for ws.x_q8k.qs of `rows` rows of H bytes
bool make_xq_map(Workspace &ws, size_t rows, int H);
cudaError_t launch_down_prefill(const LayerDev &L, const Workspace &ws, const float *w, int n, int top_k, bool routed,
                                bool shared, cudaStream_t s);
// pmoe_codec.cu
cudaError_t launch_dequantize(int dtype, const void *blocks, size_t n_elems, float *out, cudaStream_t s);
cudaError_t launch_modify_block_scales(int dtype, const void *blocks, size_t n_blocks, const float *mults, void *out,
                                       cudaStream_t s);
cudaError_t launch_reduce_rows(const float *parts, int R, const void *extra, int extra_dtype, int n, int H, void *out,
                               int out_dtype, cudaStream_t s);
cudaError_t launch_add_rms_norm(const float *resid_in, const float *delta, const float *weight, int n, int H,
                                float eps, float *resid_out, float *y, cudaStream_t s);

void count_launch(int n = 1);
bool pdl_enabled();  // PMOE_PDL=0 in the environment turns the overlap off (plain stream order)

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args &&...args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace pmoe
