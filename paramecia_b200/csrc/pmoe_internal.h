// Host-side internals shared by the files that implement the C ABI: error reporting, the device guard and the
// layer handle.
#pragma once
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "pmoe_common.cuh"

namespace pmoe {

int fail(int code, const char *fmt, ...);
int fail_cuda(cudaError_t e, const char *what);

#define CU(call)                                                  \
    do {                                                          \
        cudaError_t _e = (call);                                  \
        if (_e != cudaSuccess) return fail_cuda(_e, #call);       \
    } while (0)

// Makes `device` current for the calling thread and restores the previous one on exit.
struct DeviceGuard {
    int prev = -1;
    bool ok = false;
    explicit DeviceGuard(int device)
    {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        ok = cudaSetDevice(device) == cudaSuccess;
    }
    ~DeviceGuard()
    {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

}  // namespace pmoe

struct pmoe_ep_state;   // buffers of the expert-parallel forward (pmoe_ep.cu)

struct pmoe_layer {
    pmoe_layer_desc desc;
    pmoe::LayerDev dev;
    pmoe::Workspace ws;
    int device;
    std::vector<void *> owned;  // device allocations freed at destroy
    // device staging for the host-buffer entry point
    void *st_x = nullptr, *st_out = nullptr;
    float *st_logits = nullptr;
    uint32_t *st_idx = nullptr;
    float *st_w = nullptr;
    // per-phase CUDA events of the last traced call (pmoe_layer_trace)
    // pmoe_forward_host replays the kernel chain of its last shape as a CUDA graph (the chain works on
    // the handle's own staging buffers, so its arguments do not change from call to call)
    cudaStream_t cap_stream = nullptr;
    cudaGraphExec_t hg_exec = nullptr;
    int hg_n = -1, hg_x_dtype = 0, hg_out_dtype = 0, hg_flags = 0, hg_launches = 0;
    int hg_seen_n = -1, hg_seen_x = 0, hg_seen_out = 0, hg_seen_flags = 0;
    void *hg_out = nullptr, *hg_seen_out_ptr = nullptr;   // where the chain writes the block output
    bool hg_off = false;
    // rows the shared expert serves in the next run_experts call; count < 0 = every row
    int req_sh_begin = 0, req_sh_count = -1;
    // block-scale multipliers (training mode): the tensors as created, and the scaled copies the kernels read
    // while multipliers are installed (index: 0 gate_exps, 1 up_exps, 2 down_exps, 3 sh_gate, 4 sh_up, 5 sh_down)
    const uint8_t *orig[6] = {};
    void *scaled[6] = {};
    pmoe_ep_state *ep = nullptr;   // created by the first pmoe_ep_forward
    bool trace = false;
    cudaEvent_t ev0[PMOE_TRACE_PHASES] = {}, ev1[PMOE_TRACE_PHASES] = {};
    bool ev_used[PMOE_TRACE_PHASES] = {};
};

namespace pmoe {

// experts (+ shared expert) given routing already in device memory; `ws` is the layer's workspace or a copy of it
// with some arrays redirected
int run_experts(pmoe_layer *L, Workspace &ws, const void *x, int x_dtype, const uint32_t *idx, const float *w, int n, int top_k,
                bool routed, bool shared, bool prep_done, void *out, int out_dtype, cudaStream_t s);
int check_call(pmoe_layer *L, const void *x, int x_dtype, int n, const void *out, int out_dtype);
void ep_state_destroy(pmoe_ep_state *st);

}  // namespace pmoe
