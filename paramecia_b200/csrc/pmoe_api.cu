// C ABI of libpmoe (include/pmoe.h): layer handles, argument checks, workspace layout and the
// kernel sequence of one MoE block.  Host code only; every kernel lives in the other .cu files.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "pmoe_internal.h"

namespace pmoe {

static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }
bool pdl_enabled()
{
    static const bool on = !(getenv("PMOE_PDL") && atoi(getenv("PMOE_PDL")) == 0);
    return on;
}

static thread_local std::string g_last_error;

int fail(int code, const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

int fail_cuda(cudaError_t e, const char *what)
{
    return fail(PMOE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

static bool dtype_known(int dt)
{
    return dt == PMOE_F32 || dt == PMOE_F16 || dt == PMOE_BF16 || dt == PMOE_Q8_0 || (dt >= PMOE_Q2_K && dt <= PMOE_Q6_K);
}

}  // namespace pmoe

using namespace pmoe;

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Bump allocator over one device block.  First pass (base == nullptr) only measures.
struct Carver {
    uint8_t *base;
    size_t off = 0;
    template <typename T> T *take(size_t count)
    {
        off = align_up(off, 256);
        T *p = base ? reinterpret_cast<T *>(base + off) : nullptr;
        off += count * sizeof(T);
        return p;
    }
};

void carve_workspace(pmoe_layer *L, Carver &c)
{
    const pmoe_layer_desc &d = L->desc;
    const size_t n = (size_t)d.max_tokens, H = d.H, F = d.F, E = d.E, k = d.k;
    const size_t El = L->dev.E_local;
    const size_t rows = n * (k + 1);
    Workspace &w = L->ws;
    w.max_tokens = d.max_tokens;
    w.sh_begin = 0;
    w.sh_count = -1;
    w.status = c.take<DevStatus>(1);
    w.logits = c.take<float>(n * E);
    w.topk_idx = c.take<uint32_t>(n * k);
    w.topk_w = c.take<float>(n * k);
    w.x_q8k.qs = c.take<int8_t>(n * H);
    w.x_q8k.d = c.take<float>(n * (H / QK_K));
    w.x_q8k.bsums = c.take<int16_t>(n * (H / 16));
    w.x_q80.qs = c.take<int8_t>(n * H);
    w.x_q80.d = c.take<float>(n * (H / QK8_0));
    w.x_q80.bsums = nullptr;
    w.sh_sigmoid = c.take<float>(n);
    w.groups.count = c.take<int>(El);
    w.groups.offset = c.take<int>(El + 1);
    w.groups.pos = c.take<int>(n * k);
    w.groups.pairs = c.take<int>(n * k);
    w.groups.active = c.take<int>(El);
    w.groups.n_active = c.take<int>(1);
    w.groups.cost_prefix = c.take<int>(El + 1);
    w.groups.cost_prefix_wide = c.take<int>(El + 1);
    w.groups.cost_prefix_mma = c.take<int>(El + 1);
    w.groups.tile_prefix = c.take<int>(El + 1);
    w.groups.tile_table = c.take<int2>(n * k / PREFILL_NT + El + 1);
    w.groups.chunk_cnt = c.take<int>((n * k + GROUP_CHUNK - 1) / GROUP_CHUNK * El);
    w.act = c.take<float>(rows * F);
    w.act_q8k.qs = c.take<int8_t>(rows * F);
    w.act_q8k.d = c.take<float>(rows * (F / QK_K));
    w.act_q8k.bsums = c.take<int16_t>(rows * (F / 16));
    w.act_q80.qs = c.take<int8_t>(rows * F);
    w.act_q80.d = c.take<float>(rows * (F / QK8_0));
    w.act_q80.bsums = nullptr;
    w.act_h = c.take<__half>(rows * F);
    w.act_h_scale = c.take<float>(rows);
    w.partial = c.take<float>(rows * H);
    w.slot_done = c.take<int>(El + 1 + (n + 7) / 8);   // per expert, the shared expert, and its 8-token tiles
    L->st_x = c.take<float>(n * H);
    L->st_out = c.take<float>(n * H);
    L->st_logits = c.take<float>(n * E);
    L->st_idx = c.take<uint32_t>(n * k);
    L->st_w = c.take<float>(n * k);
}

int place_tensor(pmoe_layer *L, const void *src, size_t bytes, int location, const uint8_t **dst, const char *name)
{
    if (!src) return fail(PMOE_ERR_INVALID_ARG, "%s is NULL", name);
    if (location == 2) {
        if ((uintptr_t)src & 15) return fail(PMOE_ERR_INVALID_ARG, "%s: adopted pointers must be 16-byte aligned", name);
        *dst = (const uint8_t *)src;
        return PMOE_OK;
    }
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
    if (e != cudaSuccess) return fail_cuda(e, name);
    L->owned.push_back(p);
    e = cudaMemcpy(p, src, bytes, location == 0 ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice);
    if (e != cudaSuccess) return fail_cuda(e, name);
    *dst = (const uint8_t *)p;
    return PMOE_OK;
}

}  // namespace

int pmoe::check_call(pmoe_layer *L, const void *x, int x_dtype, int n, const void *out, int out_dtype)
{
    if (!L) return fail(PMOE_ERR_INVALID_ARG, "layer is NULL");
    if (L->desc.training_mode)
        return fail(PMOE_ERR_TRAINING_MODE, "block-scale multipliers are installed; use the reference path");
    if (n < 0) return fail(PMOE_ERR_INVALID_ARG, "n must be >= 0");
    if (n > L->desc.max_tokens)
        return fail(PMOE_ERR_TOO_MANY_TOKENS, "n = %d exceeds max_tokens = %d", n, L->desc.max_tokens);
    if (n > 0 && (!x || !out)) return fail(PMOE_ERR_INVALID_ARG, "x / out is NULL");
    if (x_dtype != PMOE_F32 && x_dtype != PMOE_BF16)
        return fail(PMOE_ERR_UNSUPPORTED_DTYPE, "activations must be F32 or BF16 (got %d)", x_dtype);
    if (out_dtype != PMOE_F32 && out_dtype != PMOE_BF16)
        return fail(PMOE_ERR_UNSUPPORTED_DTYPE, "outputs must be F32 or BF16 (got %d)", out_dtype);
    return PMOE_OK;
}

namespace {

struct Needs {
    bool q8k, q80;
};

// Brackets one launch with the layer's events when tracing is on.
struct PhaseTimer {
    pmoe_layer *L;
    int phase;
    cudaStream_t s;
    PhaseTimer(pmoe_layer *l, int p, cudaStream_t st) : L(l), phase(p), s(st)
    {
        if (L->trace) cudaEventRecord(L->ev0[phase], s);
    }
    ~PhaseTimer()
    {
        if (L->trace) {
            cudaEventRecord(L->ev1[phase], s);
            L->ev_used[phase] = true;
        }
    }
};
#define PHASE(L, p, s, call)        \
    do {                            \
        PhaseTimer _pt(L, p, s);    \
        CU(call);                   \
    } while (0)

Needs input_needs(const LayerDev &d, bool routed, bool shared)
{
    Needs nd{false, false};
    if (routed) (is_kquant(d.gate_dtype) ? nd.q8k : nd.q80) = true;
    if (shared) (is_kquant(d.sh_gate_dtype) ? nd.q8k : nd.q80) = true;
    return nd;
}

}  // namespace

// experts (+ shared) given routing already in device memory
int pmoe::run_experts(pmoe_layer *L, Workspace &ws, const void *x, int x_dtype, const uint32_t *idx, const float *w, int n,
                      int top_k, bool routed, bool shared, bool prep_done, void *out, int out_dtype, cudaStream_t s)
{
    const LayerDev &d = L->dev;
    ws.sh_begin = L->req_sh_count < 0 ? 0 : L->req_sh_begin;
    ws.sh_count = L->req_sh_count < 0 ? n : L->req_sh_count;
    L->req_sh_count = -1;  // a request holds for one call
    if (!prep_done) {
        Needs nd = input_needs(d, routed, shared);
        PHASE(L, 0, s, launch_prep(d, ws, x, x_dtype, n, nd.q8k, nd.q80, shared, s));
    }
    if (routed) PHASE(L, 3, s, launch_group(d, ws, idx, n, top_k, s));
    // prefill: many tokens per expert -> grouped tensor-core GEMM; decode: streaming GEMV.  The
    // expected number of tokens per routed expert is n * top_k / E whatever slice this layer holds.
    const char *force = getenv("PMOE_PREFILL");
    // Measured with uniform routing (every expert meets about n k / E tokens, so there are at least as many token tiles
    // as experts): the streaming kernels take 150 us + 0.7 us per token, the tensor-core kernels 970 us flat up to
    // 1 024 tokens and little more beyond; they cross at 23 tokens per expert.  One rank of eight (512 rows, 64 local
    // experts, 10 tokens each): 94 us against 219.  A router that sends most tokens to few experts fills its tiles
    // earlier, but the host does not see the counts.
    const bool want_prefill = force ? atoi(force) != 0 : (long)n * top_k >= 24L * d.E && n >= 512;
    bool prefill = want_prefill && prefill_supported(d, ws, routed, shared);
    // A shared expert the tensor-core kernels do not take (e.g. Q8_0) does not hold the routed experts
    // back: they go through the tensor-core kernels and the shared expert through the streaming ones.
    const bool split = want_prefill && !prefill && routed && shared && prefill_supported(d, ws, true, false);
    if (split) {
        PHASE(L, 4, s, launch_gate_up_prefill(d, ws, n, top_k, true, false, s));
        if (prefill_down_supported(d, ws, true, false)) {
            CU(launch_down_prefill(d, ws, w, n, top_k, true, false, s));
        } else {
            CU(launch_act_quant(d, ws, idx, n, top_k, true, false, s));
            CU(launch_down(d, ws, w, n, top_k, true, false, s));
        }
        CU(launch_gate_up(d, ws, n, top_k, false, true, s));
        PHASE(L, 6, s, launch_down(d, ws, w, n, top_k, false, true, s));
        PHASE(L, 7, s, launch_combine(d, ws, idx, n, top_k, routed, shared, out, out_dtype, s));
        return PMOE_OK;
    }
    if (prefill)
        PHASE(L, 4, s, launch_gate_up_prefill(d, ws, n, top_k, routed, shared, s));
    else
        PHASE(L, 4, s, launch_gate_up(d, ws, n, top_k, routed, shared, s));
    if (prefill && prefill_down_supported(d, ws, routed, shared)) {
        PHASE(L, 6, s, launch_down_prefill(d, ws, w, n, top_k, routed, shared, s));
    } else {
        // the decode gate/up kernel has already re-quantised every expert's activated rows (last-CTA
        // ticket); after the tensor-core gate/up kernel a separate pass does it
        if (prefill) PHASE(L, 5, s, launch_act_quant(d, ws, idx, n, top_k, routed, shared, s));
        PHASE(L, 6, s, launch_down(d, ws, w, n, top_k, routed, shared, s));
    }
    PHASE(L, 7, s, launch_combine(d, ws, idx, n, top_k, routed, shared, out, out_dtype, s));
    return PMOE_OK;
}

extern "C" {

int pmoe_version(void) { return PMOE_VERSION; }
const char *pmoe_last_error(void) { return g_last_error.c_str(); }
uint64_t pmoe_launch_count(void) { return g_launches.load(); }
size_t pmoe_block_size(int dtype) { return (size_t)block_elems(dtype); }
size_t pmoe_type_size(int dtype) { return (size_t)block_bytes(dtype); }

int pmoe_layer_create(const pmoe_layer_desc *desc, pmoe_layer **out)
{
    if (!desc || !out) return fail(PMOE_ERR_INVALID_ARG, "desc / out is NULL");
    *out = nullptr;
    if (desc->struct_size != sizeof(pmoe_layer_desc))
        return fail(PMOE_ERR_INVALID_ARG, "struct_size %u does not match this library (%zu)", desc->struct_size,
                    sizeof(pmoe_layer_desc));
    const pmoe_layer_desc &d = *desc;
    if (d.H <= 0 || d.F <= 0 || d.E <= 0 || d.k <= 0 || d.max_tokens <= 0)
        return fail(PMOE_ERR_INVALID_ARG, "H, F, E, k and max_tokens must be positive");
    if (d.k > 32 || d.k > d.E) return fail(PMOE_ERR_UNSUPPORTED_SHAPE, "k must be <= min(32, E)");
    if (d.E > 1024) return fail(PMOE_ERR_UNSUPPORTED_SHAPE, "E must be <= 1024");
    if (d.H % 128) return fail(PMOE_ERR_UNSUPPORTED_SHAPE, "H must be a multiple of 128");
    int E_local = d.E_local > 0 ? d.E_local : d.E;
    if (d.ep_placement != 0 && d.ep_placement != 1) return fail(PMOE_ERR_INVALID_ARG, "ep_placement must be 0 or 1");
    if (d.ep_size < 0 || d.ep_rank < 0 || (d.ep_size > 0 && d.ep_rank >= d.ep_size))
        return fail(PMOE_ERR_INVALID_ARG, "ep_rank %d / ep_size %d", d.ep_rank, d.ep_size);
    if (d.ep_placement == 1) {
        if (d.ep_size < 1 || d.E % d.ep_size || E_local != d.E / d.ep_size)
            return fail(PMOE_ERR_INVALID_ARG, "round-robin placement: E = %d must divide by ep_size = %d and E_local be E / ep_size",
                        d.E, d.ep_size);
    } else if (d.expert_base < 0 || d.expert_base + E_local > d.E)
        return fail(PMOE_ERR_INVALID_ARG, "expert slice [%d, %d) is outside [0, %d)", d.expert_base,
                    d.expert_base + E_local, d.E);
    if (d.weights_location < 0 || d.weights_location > 2)
        return fail(PMOE_ERR_INVALID_ARG, "weights_location must be 0, 1 or 2");
    const int dts[3] = {d.gate_dtype, d.up_dtype, d.down_dtype};
    for (int dt : dts)
        if (!dtype_known(dt)) return fail(PMOE_ERR_UNSUPPORTED_DTYPE, "unknown GGML dtype id %d", dt);
    if (d.gate_dtype != d.up_dtype)
        return fail(PMOE_ERR_UNSUPPORTED_DTYPE, "gate and up experts must share one dtype (got %d and %d)", d.gate_dtype,
                    d.up_dtype);
    const bool router_quantised = dtype_known(d.router_dtype) && block_elems(d.router_dtype) > 1;
    if (d.router_dtype != PMOE_F32 && d.router_dtype != PMOE_F16 && d.router_dtype != PMOE_BF16 && !router_quantised)
        return fail(PMOE_ERR_UNSUPPORTED_DTYPE, "router weights must be F32, F16, BF16 or a GGUF block type (got %d)", d.router_dtype);
    if (router_quantised && d.H % block_elems(d.router_dtype))
        return fail(PMOE_ERR_UNSUPPORTED_SHAPE, "H must be a multiple of the router's block size");
    const char *why = "";
    if (!gemv_supported(d.gate_dtype, d.H, d.F, &why) || !gemv_supported(d.down_dtype, d.F, d.H, &why))
        return fail(dtype_known(d.gate_dtype) && (block_elems(d.gate_dtype) > 1) && (block_elems(d.down_dtype) > 1)
                        ? PMOE_ERR_UNSUPPORTED_SHAPE
                        : PMOE_ERR_UNSUPPORTED_DTYPE,
                    "experts: %s", why);
    if (d.F > 512) return fail(PMOE_ERR_UNSUPPORTED_SHAPE, "F must be <= 512");
    if (d.has_shared) {
        if (d.sh_gate_dtype != d.sh_up_dtype)
            return fail(PMOE_ERR_UNSUPPORTED_DTYPE, "shared gate and up must share one dtype");
        if (!gemv_supported(d.sh_gate_dtype, d.H, d.F, &why) || !gemv_supported(d.sh_down_dtype, d.F, d.H, &why))
            return fail(PMOE_ERR_UNSUPPORTED_DTYPE, "shared expert: %s", why);
        // Q2_K / Q3_K / Q5_K shared matrices only beside routed matrices of the same type (kernel variants
        // exist for those pairings and for Q4_K / Q6_K / Q8_0 shared experts)
        auto low = [](int t) { return t == PMOE_Q2_K || t == PMOE_Q3_K; };
        auto pair_ok = [&](int routed_t, int shared_t) {
            if (low(shared_t)) return shared_t == routed_t;
            if (low(routed_t) && shared_t == PMOE_Q5_K) return false;
            return true;
        };
        if (!pair_ok(d.gate_dtype, d.sh_gate_dtype) || !pair_ok(d.down_dtype, d.sh_down_dtype))
            return fail(PMOE_ERR_UNSUPPORTED_DTYPE,
                        "shared expert types (%d, %d) beside routed types (%d, %d): Q2_K / Q3_K shared matrices need routed "
                        "matrices of the same type, and Q2_K / Q3_K routed matrices a shared expert of their own type, "
                        "Q4_K, Q6_K or Q8_0", d.sh_gate_dtype, d.sh_down_dtype, d.gate_dtype, d.down_dtype);
    }
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        cudaGetLastError();
        return fail(PMOE_ERR_NO_DEVICE, "no CUDA device is available; libpmoe has no CPU path");
    }
    if (d.device < 0 || d.device >= ndev) return fail(PMOE_ERR_INVALID_ARG, "device %d of %d", d.device, ndev);
    DeviceGuard guard(d.device);
    if (!guard.ok) return fail(PMOE_ERR_CUDA, "cannot select device %d", d.device);

    pmoe_layer *L = new pmoe_layer();
    L->desc = d;
    L->desc.E_local = E_local;
    L->device = d.device;
    LayerDev &v = L->dev;
    v.H = d.H; v.F = d.F; v.E = d.E; v.k = d.k;
    v.expert_base = d.expert_base; v.E_local = E_local;
    v.ep_stride = d.ep_placement == 1 ? d.ep_size : 0;
    v.ep_rem = d.ep_placement == 1 ? d.ep_rank : 0;
    v.gate_dtype = d.gate_dtype; v.up_dtype = d.up_dtype; v.down_dtype = d.down_dtype;
    v.has_shared = d.has_shared ? 1 : 0;
    v.sh_gate_dtype = d.sh_gate_dtype; v.sh_up_dtype = d.sh_up_dtype; v.sh_down_dtype = d.sh_down_dtype;
    int rc = PMOE_OK;
    const int loc = d.weights_location;
    const size_t El = (size_t)E_local;
    const uint8_t *tmp = nullptr;
    if (!rc) rc = place_tensor(L, d.gate_exps, El * d.F * row_bytes(d.gate_dtype, d.H), loc, &v.gate_exps, "gate_exps");
    if (!rc) rc = place_tensor(L, d.up_exps, El * d.F * row_bytes(d.up_dtype, d.H), loc, &v.up_exps, "up_exps");
    if (!rc) rc = place_tensor(L, d.down_exps, El * d.H * row_bytes(d.down_dtype, d.F), loc, &v.down_exps, "down_exps");
    if (!rc && d.has_shared) {
        rc = place_tensor(L, d.sh_gate, (size_t)d.F * row_bytes(d.sh_gate_dtype, d.H), loc, &v.sh_gate, "sh_gate");
        if (!rc) rc = place_tensor(L, d.sh_up, (size_t)d.F * row_bytes(d.sh_up_dtype, d.H), loc, &v.sh_up, "sh_up");
        if (!rc) rc = place_tensor(L, d.sh_down, (size_t)d.H * row_bytes(d.sh_down_dtype, d.F), loc, &v.sh_down, "sh_down");
        if (!rc) rc = place_tensor(L, d.sh_gate_inp, (size_t)d.H * 4, loc, &tmp, "sh_gate_inp");
        v.sh_gate_inp = (const float *)tmp;
    }
    v.router_q = nullptr;
    v.router_dtype = PMOE_F32;
    if (!rc && d.router_dtype == PMOE_F32) {
        rc = place_tensor(L, d.router_w, (size_t)d.E * d.H * 4, loc, &tmp, "router_w");
        v.router_w = (const float *)tmp;
    } else if (!rc && router_quantised) {
        rc = place_tensor(L, d.router_w, (size_t)d.E * row_bytes(d.router_dtype, d.H), loc, &v.router_q, "router_w");
        v.router_w = nullptr;
        v.router_dtype = d.router_dtype;
    } else if (!rc) {
        // 16-bit router weights are widened to f32 once, like the dequantised tensor the reference's
        // QMatMul holds for an F16/BF16 ffn_gate_inp (models/with_tracing.rs:120-124)
        rc = place_tensor(L, d.router_w, (size_t)d.E * d.H * 2, loc, &tmp, "router_w");
        float *wide = nullptr;
        if (!rc) {
            cudaError_t e = cudaMalloc(&wide, (size_t)d.E * d.H * 4);
            if (e != cudaSuccess) rc = fail_cuda(e, "router_w (f32 copy)");
            else L->owned.push_back(wide);
        }
        if (!rc) {
            cudaError_t e = launch_dequantize(d.router_dtype, tmp, (size_t)d.E * d.H, wide, 0);
            if (e == cudaSuccess) e = cudaStreamSynchronize(0);
            if (e != cudaSuccess) rc = fail_cuda(e, "router_w (f32 copy)");
        }
        v.router_w = wide;
    }
    v.router_bias = nullptr;
    if (!rc && d.router_bias) {
        rc = place_tensor(L, d.router_bias, (size_t)d.E * 4, loc, &tmp, "router_bias");
        v.router_bias = (const float *)tmp;
    }
    if (!rc) {
        Carver measure{nullptr};
        carve_workspace(L, measure);
        void *block = nullptr;
        cudaError_t e = cudaMalloc(&block, measure.off + 256);
        if (e != cudaSuccess) {
            rc = fail_cuda(e, "workspace");
        } else {
            L->owned.push_back(block);
            Carver real{(uint8_t *)block};
            carve_workspace(L, real);
            e = cudaMemset(L->ws.status, 0, sizeof(DevStatus));
            if (e == cudaSuccess) e = cudaMemset(L->ws.slot_done, 0, sizeof(int) * (El + 1 + ((size_t)d.max_tokens + 7) / 8));
            // (the down GEMM's copies take whole 64-row boxes: rows no call has written yet must hold numbers)
            const size_t act_rows = (size_t)d.max_tokens * (d.k + 1);
            if (e == cudaSuccess) e = cudaMemset(L->ws.act_h, 0, act_rows * d.F * sizeof(__half));
            if (e != cudaSuccess) rc = fail_cuda(e, "workspace");
            L->ws.act_h_map_ok = !rc && make_act_h_map(L->ws, act_rows, d.F);
            L->ws.xq_map_ok = !rc && make_xq_map(L->ws, (size_t)d.max_tokens, d.H);
        }
    }
    if (rc) {
        for (void *p : L->owned) cudaFree(p);
        delete L;
        return rc;
    }
    L->orig[0] = v.gate_exps; L->orig[1] = v.up_exps; L->orig[2] = v.down_exps;
    L->orig[3] = v.sh_gate; L->orig[4] = v.sh_up; L->orig[5] = v.sh_down;
    *out = L;
    return PMOE_OK;
}

int pmoe_layer_destroy(pmoe_layer *L)
{
    if (!L) return PMOE_OK;
    DeviceGuard guard(L->device);
    cudaDeviceSynchronize();
    for (void *p : L->owned) cudaFree(p);
    for (void *p : L->scaled)
        if (p) cudaFree(p);
    if (L->ep) ep_state_destroy(L->ep);
    if (L->hg_exec) cudaGraphExecDestroy(L->hg_exec);
    if (L->cap_stream) cudaStreamDestroy(L->cap_stream);
    for (int i = 0; i < PMOE_TRACE_PHASES; i++) {
        if (L->ev0[i]) cudaEventDestroy(L->ev0[i]);
        if (L->ev1[i]) cudaEventDestroy(L->ev1[i]);
    }
    delete L;
    return PMOE_OK;
}

int pmoe_layer_trace(pmoe_layer *L, int enable)
{
    if (!L) return fail(PMOE_ERR_INVALID_ARG, "layer is NULL");
    DeviceGuard guard(L->device);
    if (enable && !L->ev0[0]) {
        for (int i = 0; i < PMOE_TRACE_PHASES; i++) {
            CU(cudaEventCreate(&L->ev0[i]));
            CU(cudaEventCreate(&L->ev1[i]));
        }
    }
    L->trace = enable != 0;
    for (bool &u : L->ev_used) u = false;
    return PMOE_OK;
}

int pmoe_layer_trace_read(pmoe_layer *L, float *ms)
{
    if (!L || !ms) return fail(PMOE_ERR_INVALID_ARG, "layer / ms is NULL");
    DeviceGuard guard(L->device);
    for (int i = 0; i < PMOE_TRACE_PHASES; i++) {
        ms[i] = 0.f;
        if (!L->ev_used[i]) continue;
        CU(cudaEventSynchronize(L->ev1[i]));
        CU(cudaEventElapsedTime(&ms[i], L->ev0[i], L->ev1[i]));
    }
    return PMOE_OK;
}

const char *pmoe_trace_phase_name(int phase)
{
    static const char *names[PMOE_TRACE_PHASES] = {"prep", "router", "topk", "group",
                                                   "gate_up", "act_quant", "down", "combine"};
    return phase >= 0 && phase < PMOE_TRACE_PHASES ? names[phase] : "";
}

int pmoe_route(pmoe_layer *L, const void *x, int x_dtype, int n, float *logits_out, uint32_t *idx_out, float *w_out,
               void *stream)
{
    float dummy = 0.f;
    int rc = check_call(L, x, x_dtype, n, &dummy, PMOE_F32);
    if (rc) return rc;
    if (n == 0) return PMOE_OK;
    DeviceGuard guard(L->device);
    cudaStream_t s = (cudaStream_t)stream;
    float *logits = logits_out ? logits_out : L->ws.logits;
    CU(launch_router(L->dev, L->ws, x, x_dtype, n, logits, s));
    if (idx_out || w_out) CU(launch_topk(L->dev, L->ws, logits, n, idx_out, w_out, s));
    return PMOE_OK;
}

int pmoe_forward(pmoe_layer *L, const void *x, int x_dtype, int n, void *out, int out_dtype, float *logits_out,
                 uint32_t *idx_out, float *w_out, void *stream)
{
    int rc = check_call(L, x, x_dtype, n, out, out_dtype);
    if (rc) return rc;
    if (n == 0) return PMOE_OK;
    DeviceGuard guard(L->device);
    cudaStream_t s = (cudaStream_t)stream;
    const LayerDev &d = L->dev;
    float *logits = logits_out ? logits_out : L->ws.logits;
    uint32_t *idx = idx_out ? idx_out : L->ws.topk_idx;
    float *w = w_out ? w_out : L->ws.topk_w;
    Needs nd = input_needs(d, true, d.has_shared);
    for (bool &u : L->ev_used) u = false;
    // one launch: router rows plus, in extra CTAs, the per-token preparation
    PHASE(L, 1, s, launch_router(d, L->ws, x, x_dtype, n, logits, s, true, nd.q8k, nd.q80, d.has_shared));
    PHASE(L, 2, s, launch_topk(d, L->ws, logits, n, idx, w, s));
    return run_experts(L, L->ws, x, x_dtype, idx, w, n, d.k, true, d.has_shared, true, out, out_dtype, s);
}

int pmoe_router_stats(pmoe_layer *L, const float *logits, const uint32_t *idx, int n, int top_k, float *counts_out,
                      float *losses_out, void *stream)
{
    if (!L) return fail(PMOE_ERR_INVALID_ARG, "layer is NULL");
    if (n < 0 || n > L->desc.max_tokens) return fail(PMOE_ERR_TOO_MANY_TOKENS, "n = %d, max_tokens = %d", n, L->desc.max_tokens);
    if (n == 0) return PMOE_OK;
    if (!logits || !idx) return fail(PMOE_ERR_INVALID_ARG, "logits / idx is NULL");
    if (top_k <= 0 || top_k > L->desc.k) return fail(PMOE_ERR_INVALID_ARG, "top_k = %d must be in [1, %d]", top_k, L->desc.k);
    DeviceGuard guard(L->device);
    // scratch: the workspace's partial-row buffer (rows * H floats), idle outside a forward call
    const size_t have = (size_t)L->desc.max_tokens * (L->desc.k + 1) * L->desc.H;
    if (router_stats_scratch_floats(n, L->desc.E) > have) return fail(PMOE_ERR_UNSUPPORTED_SHAPE, "statistics scratch too small");
    CU(launch_router_stats(logits, idx, n, top_k, L->desc.E, L->ws.partial, counts_out, losses_out, (cudaStream_t)stream));
    return PMOE_OK;
}

int pmoe_experts_forward(pmoe_layer *L, const void *x, int x_dtype, const uint32_t *idx, const float *w, int n,
                         int top_k, void *out, int out_dtype, void *stream)
{
    int rc = check_call(L, x, x_dtype, n, out, out_dtype);
    if (rc) return rc;
    if (n == 0) return PMOE_OK;
    if (!idx || !w) return fail(PMOE_ERR_INVALID_ARG, "idx / w is NULL");
    if (top_k <= 0 || top_k > L->desc.k)
        return fail(PMOE_ERR_INVALID_ARG, "top_k = %d must be in [1, %d]", top_k, L->desc.k);
    DeviceGuard guard(L->device);
    return run_experts(L, L->ws, x, x_dtype, idx, w, n, top_k, true, false, false, out, out_dtype, (cudaStream_t)stream);
}

int pmoe_experts_forward_ep(pmoe_layer *L, const void *x, int x_dtype, const uint32_t *idx, const float *w, int n,
                            int top_k, int shared_begin, int shared_count, void *out, int out_dtype, void *stream)
{
    int rc = check_call(L, x, x_dtype, n, out, out_dtype);
    if (rc) return rc;
    if (n == 0) return PMOE_OK;
    if (!idx || !w) return fail(PMOE_ERR_INVALID_ARG, "idx / w is NULL");
    if (top_k <= 0 || top_k > L->desc.k)
        return fail(PMOE_ERR_INVALID_ARG, "top_k = %d must be in [1, %d]", top_k, L->desc.k);
    if (shared_begin < 0 || shared_count < 0 || shared_begin + shared_count > n)
        return fail(PMOE_ERR_INVALID_ARG, "shared rows [%d, %d) are outside [0, %d)", shared_begin,
                    shared_begin + shared_count, n);
    const bool shared = shared_count > 0 && L->dev.has_shared;
    DeviceGuard guard(L->device);
    L->req_sh_begin = shared_begin;
    L->req_sh_count = shared ? shared_count : -1;
    return run_experts(L, L->ws, x, x_dtype, idx, w, n, top_k, true, shared, false, out, out_dtype, (cudaStream_t)stream);
}

int pmoe_shared_forward(pmoe_layer *L, const void *x, int x_dtype, int n, void *out, int out_dtype, void *stream)
{
    int rc = check_call(L, x, x_dtype, n, out, out_dtype);
    if (rc) return rc;
    if (n == 0) return PMOE_OK;
    if (!L->dev.has_shared) return fail(PMOE_ERR_INVALID_ARG, "the layer has no shared expert");
    DeviceGuard guard(L->device);
    return run_experts(L, L->ws, x, x_dtype, nullptr, nullptr, n, L->desc.k, false, true, false, out, out_dtype,
                       (cudaStream_t)stream);
}

int pmoe_forward_host(pmoe_layer *L, const void *x_host, int x_dtype, int n, void *out_host, int out_dtype,
                      float *logits_host, uint32_t *idx_host, float *w_host, void *stream)
{
    int rc = check_call(L, x_host, x_dtype, n, out_host, out_dtype);
    if (rc) return rc;
    if (n == 0) return PMOE_OK;
    DeviceGuard guard(L->device);
    cudaStream_t s = (cudaStream_t)stream;
    const pmoe_layer_desc &d = L->desc;
    const size_t xin = (size_t)n * d.H * (x_dtype == PMOE_F32 ? 4 : 2);
    const size_t xout = (size_t)n * d.H * (out_dtype == PMOE_F32 ? 4 : 2);
    CU(cudaMemcpyAsync(L->st_x, x_host, xin, cudaMemcpyHostToDevice, s));
    float *lg = logits_host ? L->st_logits : nullptr;
    uint32_t *ix = idx_host ? L->st_idx : nullptr;
    float *wt = w_host ? L->st_w : nullptr;
    // Pinned (mapped) output memory is written by the combine kernel itself, without a copy afterwards.
    // (looked up on every call: an address can change hands between pinned and pageable memory)
    void *out_dev = L->st_out;
    {
        cudaPointerAttributes pa{};
        if (cudaPointerGetAttributes(&pa, out_host) == cudaSuccess && pa.type == cudaMemoryTypeHost && pa.devicePointer &&
            !((uintptr_t)pa.devicePointer & 15))
            out_dev = pa.devicePointer;
        cudaGetLastError();
    }
    // The chain between the two copies: first call of a shape runs directly, the second records it
    // into a graph, later ones replay the graph (PMOE_HOST_GRAPH=0 keeps direct launches).
    const int flags = (lg ? 1 : 0) | (ix ? 2 : 0) | (wt ? 4 : 0);
    static const bool graphs_on = !(getenv("PMOE_HOST_GRAPH") && atoi(getenv("PMOE_HOST_GRAPH")) == 0);
    bool done = false;
    if (graphs_on && !L->hg_off && !L->trace) {
        const bool cached = L->hg_exec && L->hg_n == n && L->hg_x_dtype == x_dtype && L->hg_out_dtype == out_dtype &&
                            L->hg_flags == flags && L->hg_out == out_dev;
        const bool seen = L->hg_seen_n == n && L->hg_seen_x == x_dtype && L->hg_seen_out == out_dtype &&
                          L->hg_seen_flags == flags && L->hg_seen_out_ptr == out_dev;
        if (!cached && seen) {
            if (!L->cap_stream && cudaStreamCreateWithFlags(&L->cap_stream, cudaStreamNonBlocking) != cudaSuccess) {
                cudaGetLastError();
                L->hg_off = true;
            }
            if (!L->hg_off) {
                cudaGraph_t graph = nullptr;
                cudaGraphExec_t exec = nullptr;
                const unsigned long long before = pmoe_launch_count();
                bool ok = cudaStreamBeginCapture(L->cap_stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
                if (ok) {
                    const int frc = pmoe_forward(L, L->st_x, x_dtype, n, out_dev, out_dtype, lg, ix, wt, L->cap_stream);
                    const cudaError_t ee = cudaStreamEndCapture(L->cap_stream, &graph);
                    ok = frc == PMOE_OK && ee == cudaSuccess && graph != nullptr;
                }
                if (ok) ok = cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
                if (graph) cudaGraphDestroy(graph);
                if (ok) {
                    if (L->hg_exec) cudaGraphExecDestroy(L->hg_exec);
                    L->hg_exec = exec;
                    L->hg_n = n; L->hg_x_dtype = x_dtype; L->hg_out_dtype = out_dtype; L->hg_flags = flags;
                    L->hg_out = out_dev;
                    L->hg_launches = (int)(pmoe_launch_count() - before);
                    count_launch(-L->hg_launches);   // recorded, not run
                } else {
                    cudaGetLastError();
                    L->hg_off = true;   // this handle keeps direct launches
                }
            }
        }
        if (!L->hg_off && L->hg_exec && L->hg_n == n && L->hg_x_dtype == x_dtype && L->hg_out_dtype == out_dtype &&
            L->hg_flags == flags && L->hg_out == out_dev) {
            CU(cudaGraphLaunch(L->hg_exec, s));
            count_launch(L->hg_launches);
            done = true;
        }
        L->hg_seen_n = n; L->hg_seen_x = x_dtype; L->hg_seen_out = out_dtype; L->hg_seen_flags = flags;
        L->hg_seen_out_ptr = out_dev;
    }
    if (!done) {
        rc = pmoe_forward(L, L->st_x, x_dtype, n, out_dev, out_dtype, lg, ix, wt, stream);
        if (rc) return rc;
    }
    if (out_dev == L->st_out) CU(cudaMemcpyAsync(out_host, L->st_out, xout, cudaMemcpyDeviceToHost, s));
    if (logits_host) CU(cudaMemcpyAsync(logits_host, L->st_logits, (size_t)n * d.E * 4, cudaMemcpyDeviceToHost, s));
    if (idx_host) CU(cudaMemcpyAsync(idx_host, L->st_idx, (size_t)n * d.k * 4, cudaMemcpyDeviceToHost, s));
    if (w_host) CU(cudaMemcpyAsync(w_host, L->st_w, (size_t)n * d.k * 4, cudaMemcpyDeviceToHost, s));
    CU(cudaStreamSynchronize(s));
    return PMOE_OK;
}

int pmoe_layer_status(pmoe_layer *L, void *stream)
{
    if (!L) return fail(PMOE_ERR_INVALID_ARG, "layer is NULL");
    DeviceGuard guard(L->device);
    cudaStream_t s = (cudaStream_t)stream;
    DevStatus st{};
    CU(cudaMemcpyAsync(&st, L->ws.status, sizeof st, cudaMemcpyDeviceToHost, s));
    CU(cudaStreamSynchronize(s));
    if (st.code) {
        CU(cudaMemsetAsync(L->ws.status, 0, sizeof st, s));
        CU(cudaStreamSynchronize(s));
        return fail(st.code, "device status %d raised by kernel tag %d (detail %d)", st.code, st.where, st.detail);
    }
    return PMOE_OK;
}

int pmoe_dequantize(int device, int dtype, const void *blocks, size_t n_elems, float *out, void *stream)
{
    if (!dtype_known(dtype)) return fail(PMOE_ERR_UNSUPPORTED_DTYPE, "unknown GGML dtype id %d", dtype);
    if (n_elems % (size_t)block_elems(dtype))
        return fail(PMOE_ERR_INVALID_ARG, "n_elems must be a multiple of the block size %d", block_elems(dtype));
    if (n_elems && (!blocks || !out)) return fail(PMOE_ERR_INVALID_ARG, "blocks / out is NULL");
    if (n_elems > ((size_t)1 << 39)) return fail(PMOE_ERR_INVALID_ARG, "n_elems too large");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(PMOE_ERR_NO_DEVICE, "cannot select device %d", device);
    CU(launch_dequantize(dtype, blocks, n_elems, out, (cudaStream_t)stream));
    return PMOE_OK;
}

int pmoe_add_rms_norm(int device, const float *resid_in, const float *delta, const float *weight, int n, int H,
                      float eps, float *resid_out, float *y, void *stream)
{
    if (n < 0 || H <= 0 || H > 12288) return fail(PMOE_ERR_INVALID_ARG, "bad n / H");
    if (n && (!resid_in || !y)) return fail(PMOE_ERR_INVALID_ARG, "resid_in / y is NULL");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(PMOE_ERR_NO_DEVICE, "cannot select device %d", device);
    CU(launch_add_rms_norm(resid_in, delta, weight, n, H, eps, resid_out, y, (cudaStream_t)stream));
    return PMOE_OK;
}

int pmoe_reduce_rows(int device, const float *parts, int n_parts, const void *extra, int extra_dtype, int n, int H,
                     void *out, int out_dtype, void *stream)
{
    if (n < 0 || H <= 0 || H % 4 || n_parts <= 0) return fail(PMOE_ERR_INVALID_ARG, "bad n / H / n_parts");
    if (n && (!parts || !out)) return fail(PMOE_ERR_INVALID_ARG, "parts / out is NULL");
    if ((extra && extra_dtype != PMOE_F32 && extra_dtype != PMOE_BF16) || (out_dtype != PMOE_F32 && out_dtype != PMOE_BF16))
        return fail(PMOE_ERR_UNSUPPORTED_DTYPE, "extra / out must be F32 or BF16");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(PMOE_ERR_NO_DEVICE, "cannot select device %d", device);
    CU(launch_reduce_rows(parts, n_parts, extra, extra ? extra_dtype : PMOE_F32, n, H, out, out_dtype,
                          (cudaStream_t)stream));
    return PMOE_OK;
}

int pmoe_qmatmul(int device, int dtype, const void *w, size_t rows, size_t cols, const float *x, size_t m, float *y,
                 void *stream)
{
    if (!(dtype >= PMOE_Q2_K && dtype <= PMOE_Q6_K) && dtype != PMOE_Q8_0)
        return fail(PMOE_ERR_UNSUPPORTED_DTYPE, "pmoe_qmatmul serves Q2_K ... Q6_K and Q8_0 (got %d)", dtype);
    if (!rows || !cols || cols % 256 || cols > 16384 || rows > (1u << 24) || m > 4096)
        return fail(PMOE_ERR_UNSUPPORTED_SHAPE, "cols must be a multiple of 256 (<= 16384), m <= 4096");
    if (!m) return PMOE_OK;
    if (!w || !x || !y) return fail(PMOE_ERR_INVALID_ARG, "w / x / y is NULL");
    if (((uintptr_t)w & 15) || ((uintptr_t)x & 15)) return fail(PMOE_ERR_INVALID_ARG, "w and x must be 16-byte aligned");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(PMOE_ERR_NO_DEVICE, "cannot select device %d", device);
    cudaStream_t s = (cudaStream_t)stream;
    void *scratch = nullptr;
    CU(cudaMallocAsync(&scratch, qmatmul_scratch_bytes((int)m, (int)cols), s));
    cudaError_t e = launch_qmatmul(dtype, w, (int)rows, (int)cols, x, (int)m, y, scratch, s);
    cudaFreeAsync(scratch, s);
    if (e != cudaSuccess) return fail_cuda(e, "pmoe_qmatmul");
    return PMOE_OK;
}

int pmoe_qmatmul_noalloc(int device, int dtype, const void *w, size_t rows, size_t cols, const float *x, size_t m,
                         float *y, void *stream)
{
    if (!(dtype >= PMOE_Q2_K && dtype <= PMOE_Q6_K) && dtype != PMOE_Q8_0)
        return fail(PMOE_ERR_UNSUPPORTED_DTYPE, "pmoe_qmatmul_noalloc serves Q2_K ... Q6_K and Q8_0 (got %d)", dtype);
    if (!rows || !cols || cols % 256 || cols > 16384 || rows > (1u << 24))
        return fail(PMOE_ERR_UNSUPPORTED_SHAPE, "cols must be a multiple of 256 (<= 16384)");
    if (!m) return PMOE_OK;
    if (!w || !x || !y) return fail(PMOE_ERR_INVALID_ARG, "w / x / y is NULL");
    if (((uintptr_t)w & 15) || ((uintptr_t)x & 15)) return fail(PMOE_ERR_INVALID_ARG, "w and x must be 16-byte aligned");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(PMOE_ERR_NO_DEVICE, "cannot select device %d", device);
    void *scratch = nullptr;
    size_t cap = 0;
    cudaError_t e = qmatmul_static_scratch(device, &scratch, &cap);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(static scratch)");
    if (m > 4096 || qmatmul_scratch_bytes((int)m, (int)cols) > cap)
        return fail(PMOE_ERR_TOO_MANY_TOKENS,
                    "m = %zu rows of %zu columns need %zu bytes of scratch; the built-in buffer holds %zu "
                    "(1.25 * m * cols + 768 <= 98304, i.e. m * cols <= 78028: 32 rows of 2048 fit, 39 do not); use "
                    "pmoe_qmatmul for larger operands",
                    m, cols, qmatmul_scratch_bytes((int)(m > 4096 ? 4096 : m), (int)cols), cap);
    e = launch_qmatmul(dtype, w, (int)rows, (int)cols, x, (int)m, y, scratch, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail_cuda(e, "pmoe_qmatmul_noalloc");
    return PMOE_OK;
}

}  // extern "C"

// ---------------------------------------------------------------- block-scale multipliers
namespace {

struct TensorSlot {
    int dtype;
    size_t blocks;
    const uint8_t **live;   // the pointer the kernels read
};

TensorSlot tensor_slot(pmoe_layer *L, int which)
{
    LayerDev &v = L->dev;
    const size_t El = (size_t)v.E_local, H = v.H, F = v.F;
    switch (which) {
    case 0: return {v.gate_dtype, El * F * (H / block_elems(v.gate_dtype)), &v.gate_exps};
    case 1: return {v.up_dtype, El * F * (H / block_elems(v.up_dtype)), &v.up_exps};
    case 2: return {v.down_dtype, El * H * (F / block_elems(v.down_dtype)), &v.down_exps};
    case 3: return {v.sh_gate_dtype, F * (H / block_elems(v.sh_gate_dtype)), &v.sh_gate};
    case 4: return {v.sh_up_dtype, F * (H / block_elems(v.sh_up_dtype)), &v.sh_up};
    default: return {v.sh_down_dtype, H * (F / block_elems(v.sh_down_dtype)), &v.sh_down};
    }
}

// Installs (mults != NULL) or removes (NULL) the multipliers of one tensor of the handle.
int set_tensor_multipliers(pmoe_layer *L, int which, const float *mults, cudaStream_t s)
{
    TensorSlot t = tensor_slot(L, which);
    if (!mults) {
        if (L->scaled[which]) {
            CU(cudaStreamSynchronize(s));   // a forward still reading the copy must finish first
            CU(cudaFree(L->scaled[which]));
            L->scaled[which] = nullptr;
        }
        *t.live = L->orig[which];
        return PMOE_OK;
    }
    const size_t bytes = t.blocks * (size_t)block_bytes(t.dtype);
    if (!L->scaled[which]) CU(cudaMalloc(&L->scaled[which], bytes));
    CU(launch_modify_block_scales(t.dtype, L->orig[which], t.blocks, mults, L->scaled[which], s));
    *t.live = (const uint8_t *)L->scaled[which];
    return PMOE_OK;
}

// the host-buffer entry point replays a recorded kernel chain that holds the old weight pointers
void drop_host_graph(pmoe_layer *L)
{
    if (L->hg_exec) cudaGraphExecDestroy(L->hg_exec);
    L->hg_exec = nullptr;
    L->hg_n = L->hg_seen_n = -1;
}

}  // namespace

extern "C" {

int pmoe_layer_set_block_multipliers(pmoe_layer *L, const float *gate_mults, const float *up_mults,
                                     const float *down_mults, void *stream)
{
    if (!L) return fail(PMOE_ERR_INVALID_ARG, "layer is NULL");
    const int given = (gate_mults ? 1 : 0) + (up_mults ? 1 : 0) + (down_mults ? 1 : 0);
    if (given != 0 && given != 3)
        return fail(PMOE_ERR_INVALID_ARG, "gate, up and down multipliers are installed together (or all NULL to clear)");
    DeviceGuard guard(L->device);
    drop_host_graph(L);
    const float *m[3] = {gate_mults, up_mults, down_mults};
    for (int i = 0; i < 3; i++) {
        int rc = set_tensor_multipliers(L, i, m[i], (cudaStream_t)stream);
        if (rc) return rc;
    }
    return PMOE_OK;
}

int pmoe_layer_set_shared_scales(pmoe_layer *L, const float *gate_scales, const float *up_scales,
                                 const float *down_scales, void *stream)
{
    if (!L) return fail(PMOE_ERR_INVALID_ARG, "layer is NULL");
    if (!L->dev.has_shared) {
        if (gate_scales || up_scales || down_scales) return fail(PMOE_ERR_INVALID_ARG, "the layer has no shared expert");
        return PMOE_OK;
    }
    DeviceGuard guard(L->device);
    drop_host_graph(L);
    const float *m[3] = {gate_scales, up_scales, down_scales};
    for (int i = 0; i < 3; i++) {
        int rc = set_tensor_multipliers(L, 3 + i, m[i], (cudaStream_t)stream);
        if (rc) return rc;
    }
    return PMOE_OK;
}

int pmoe_modify_block_scales(int device, int dtype, const void *blocks, size_t n_blocks, const float *mults, void *out,
                             void *stream)
{
    if (!(dtype >= PMOE_Q2_K && dtype <= PMOE_Q6_K) && dtype != PMOE_Q8_0)
        return fail(PMOE_ERR_UNSUPPORTED_DTYPE, "pmoe_modify_block_scales serves Q2_K ... Q6_K and Q8_0 (got %d)", dtype);
    if (n_blocks && (!blocks || !mults || !out)) return fail(PMOE_ERR_INVALID_ARG, "blocks / mults / out is NULL");
    if (((uintptr_t)blocks & 1) || ((uintptr_t)out & 1)) return fail(PMOE_ERR_INVALID_ARG, "blocks and out must be 2-byte aligned");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(PMOE_ERR_NO_DEVICE, "cannot select device %d", device);
    CU(launch_modify_block_scales(dtype, blocks, n_blocks, mults, out, (cudaStream_t)stream));
    return PMOE_OK;
}

}  // extern "C"
