// Expert-parallel forward of the MoE block behind the C ABI: token dispatch and combine over NCCL.
//
// The reference runs one process on one device; its "expert parallelism" is a rayon loop over the experts
// (paramecia-model/src/tokio_experts.rs:116-130).  Here every rank of a communicator holds E / N routed experts
// (pmoe_layer_desc: contiguous slice or round-robin), the router and the shared expert, and is home to n tokens:
//
//   1. route the home tokens; the same launch quantises their rows (Q8_K / Q8_0, what the expert kernels eat);
//   2. plan: for every destination rank the home tokens that have one of their top-k experts there, in token
//      order (the home rank itself takes all its tokens: the shared expert runs on them);
//   3. pack one record per (token, destination): the QUANTISED row, the token's ids with the ones the destination
//      does not hold replaced by an invalid id, and its routing weights -- 2.4 KB instead of a 4 KB bf16 row, and
//      the receiver needs no preparation pass;
//   4. exchange: one grouped ncclSend / ncclRecv per peer (an all-to-all-v).  With exact counts the ranks first
//      all-gather their count vectors and the host reads them (one synchronisation); with padded counts every
//      pair exchanges n records (ids of absent tokens invalid), nothing is synchronised and the call can be
//      captured in a CUDA graph;
//   5. unpack into the layer's activation arrays and run the expert kernels over the received rows (the shared
//      expert on the rank's own rows, in the same kernels), one pre-reduced f32 row per received record;
//   6. send those rows back the way they came and add, per home token, the rows of the ranks it visited in rank
//      order (fixed order: the result does not depend on arrival order).
//
// No kernel reads another GPU's memory: NCCL delivers into local HBM first.  NCCL is opened with dlopen at the
// first use, so the library has no link-time dependency on it; a process that already loaded a libnccl.so.2 (a
// Python host with torch, say) shares that copy.
#include <dlfcn.h>
#include <nccl.h>

#include "pmoe_internal.h"

namespace pmoe {

// ---------------------------------------------------------------- NCCL entry points
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId *);
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    const char *(*GetErrorString)(ncclResult_t);
};

static const NcclApi *nccl_api(std::string *why)
{
    static NcclApi api;
    static bool tried = false, ok = false;
    static std::string err;
    if (!tried) {
        tried = true;
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);   // a copy the process already has
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) {
            err = std::string("cannot load libnccl.so.2: ") + dlerror();
        } else {
            bool all = true;
            auto sym = [&](const char *name) -> void * {
                void *p = dlsym(h, name);
                if (!p) { all = false; err = std::string("libnccl lacks ") + name; }
                return p;
            };
            api.GetUniqueId = (decltype(api.GetUniqueId))sym("ncclGetUniqueId");
            api.CommInitRank = (decltype(api.CommInitRank))sym("ncclCommInitRank");
            api.CommDestroy = (decltype(api.CommDestroy))sym("ncclCommDestroy");
            api.GroupStart = (decltype(api.GroupStart))sym("ncclGroupStart");
            api.GroupEnd = (decltype(api.GroupEnd))sym("ncclGroupEnd");
            api.Send = (decltype(api.Send))sym("ncclSend");
            api.Recv = (decltype(api.Recv))sym("ncclRecv");
            api.AllGather = (decltype(api.AllGather))sym("ncclAllGather");
            api.GetErrorString = (decltype(api.GetErrorString))sym("ncclGetErrorString");
            ok = all;
        }
    }
    if (!ok && why) *why = err;
    return ok ? &api : nullptr;
}

#define NC(api, call)                                                                          \
    do {                                                                                       \
        ncclResult_t _r = (call);                                                              \
        if (_r != ncclSuccess) return fail(PMOE_ERR_CUDA, "%s: %s", #call, (api)->GetErrorString(_r)); \
    } while (0)

constexpr int EP_MAX_RANKS = 64;

}  // namespace pmoe

using namespace pmoe;

struct pmoe_ep_comm {
    ncclComm_t comm = nullptr;
    int rank = 0, size = 1, device = 0;
    bool owned = false;
    const NcclApi *api = nullptr;
};

// Buffers of the expert-parallel forward, sized for the layer's max_tokens records.
struct pmoe_ep_state {
    int rows = 0;              // capacity in records (= max_tokens)
    int rec_bytes = 0;
    QAct home_q8k{}, home_q80{};   // the home tokens' quantised rows (router launch writes them)
    float *home_sig = nullptr;
    float *recv_sig = nullptr;     // shared gate per received row (own rows only)
    uint8_t *send = nullptr, *recv = nullptr;   // records
    uint32_t *idx = nullptr;       // [rows, k] ids of the received rows
    float *w = nullptr;            // [rows, k]
    float *part = nullptr;         // [rows, H] this rank's pre-reduced rows
    float *back = nullptr;         // [rows, H] rows returned by the ranks the home tokens visited
    int *pos = nullptr;            // [n_home, N] position of token t among the records for rank r, -1: not sent
    int *cnt = nullptr;            // [N] records per destination
    int *cnt_all = nullptr;        // [N, N] everybody's counts (exact mode)
    int *cnt_host = nullptr;       // pinned copy of cnt_all
    std::vector<void *> owned;
    cudaEvent_t ev[4] = {};        // dispatch start / end, combine start / end of the last profiled call
    float last_dispatch_ms = 0.f, last_combine_ms = 0.f;
    bool profile = false;
};

namespace pmoe {

void ep_state_destroy(pmoe_ep_state *st)
{
    if (!st) return;
    for (void *p : st->owned) cudaFree(p);
    if (st->cnt_host) cudaFreeHost(st->cnt_host);
    for (cudaEvent_t e : st->ev)
        if (e) cudaEventDestroy(e);
    delete st;
}

namespace {

struct EpOffsets {
    int send_off[EP_MAX_RANKS + 1];   // records for destination r start here in the send buffer (and in `back`)
    int recv_off[EP_MAX_RANKS + 1];   // records from source s start here in the receive buffer
};

// Record of one (token, destination): quantised row | ids | weights.  kq: Q8_K form (qs, d f32[H/256],
// bsums i16[H/16]); else Q8_0 form (qs, d f32[H/32]).
__host__ __device__ inline int rec_act_bytes(int H, bool kq) { return kq ? H + (H / 256) * 4 + (H / 16) * 2 : H + (H / 32) * 4; }
__host__ __device__ inline int rec_bytes_of(int H, int k, bool kq) { return (rec_act_bytes(H, kq) + 8 * k + 15) / 16 * 16; }

__device__ inline int ep_owner(uint32_t g, int E, int N, int placement)
{
    if (g >= (uint32_t)E) return -1;
    return placement == 1 ? (int)(g % (uint32_t)N) : (int)(g / (uint32_t)(E / N));
}

// Block r: the home tokens that travel to rank r, in token order.  pos[t*N + r] = position or -1, cnt[r] = how many.
// padded: every token travels everywhere (position t).
__global__ void __launch_bounds__(1024) k_ep_plan(const uint32_t *__restrict__ idx, int n, int k, int E, int N, int placement,
                                                  int self, int self_takes_all, int padded, int *__restrict__ pos,
                                                  int *__restrict__ cnt)
{
    __shared__ int s_warp[32];
    __shared__ int s_base;
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) s_base = 0;
    __syncthreads();
    for (int t0 = 0; t0 < n; t0 += blockDim.x) {
        const int t = t0 + threadIdx.x;
        int flag = 0;
        if (t < n) {
            if (padded || (r == self && self_takes_all)) flag = 1;
            else
                for (int j = 0; j < k; j++) flag |= ep_owner(idx[(size_t)t * k + j], E, N, placement) == r;
        }
        // exclusive scan of the flags over the block
        const unsigned bal = __ballot_sync(0xffffffffu, flag);
        const int in_warp = __popc(bal & ((1u << lane) - 1));
        if (lane == 0) s_warp[warp] = __popc(bal);
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; w++) before += s_warp[w];
        const int base = s_base;
        if (t < n) pos[(size_t)t * N + r] = flag ? base + before + in_warp : -1;
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
            for (int w = 0; w < (int)(blockDim.x >> 5); w++) tot += s_warp[w];
            s_base = base + tot;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) cnt[r] = s_base;
}

// CTA t: the records of home token t, one per destination it travels to.
__global__ void __launch_bounds__(128) k_ep_pack(QAct home, bool kq, const uint32_t *__restrict__ idx,
                                                 const float *__restrict__ w, int H, int k, int E, int N, int placement,
                                                 int n, int padded, const int *__restrict__ pos, const int *__restrict__ cnt,
                                                 uint8_t *__restrict__ send, int rec)
{
    const int t = blockIdx.x;
    int off = 0;
    for (int r = 0; r < N; r++) {
        const int p = pos[(size_t)t * N + r];
        const int base = off;
        off += padded ? n : cnt[r];
        if (p < 0) continue;
        uint8_t *dst = send + (size_t)(base + p) * rec;
        // quantised row: qs | d | bsums (16-byte pieces; every part is a multiple of 16 bytes long for H = 2048)
        const uint4 *qs = reinterpret_cast<const uint4 *>(home.qs + (size_t)t * H);
        for (int i = threadIdx.x; i < H / 16; i += blockDim.x) reinterpret_cast<uint4 *>(dst)[i] = qs[i];
        uint8_t *o = dst + H;
        if (kq) {
            const float *d = home.d + (size_t)t * (H / 256);
            for (int i = threadIdx.x; i < H / 256; i += blockDim.x) reinterpret_cast<float *>(o)[i] = d[i];
            o += (H / 256) * 4;
            const int16_t *bs = home.bsums + (size_t)t * (H / 16);
            for (int i = threadIdx.x; i < H / 16; i += blockDim.x) reinterpret_cast<int16_t *>(o)[i] = bs[i];
            o += (H / 16) * 2;
        } else {
            const float *d = home.d + (size_t)t * (H / 32);
            for (int i = threadIdx.x; i < H / 32; i += blockDim.x) reinterpret_cast<float *>(o)[i] = d[i];
            o += (H / 32) * 4;
        }
        for (int j = threadIdx.x; j < k; j += blockDim.x) {
            const uint32_t g = idx[(size_t)t * k + j];
            reinterpret_cast<uint32_t *>(o)[j] = ep_owner(g, E, N, placement) == r ? g : 0xFFFFFFFFu;
            reinterpret_cast<float *>(o + 4 * k)[j] = w[(size_t)t * k + j];
        }
    }
}

// CTA row: one received record into the layer's activation arrays and the routing arrays of the expert call.  The
// rank's own rows also get the other quantised form (when the shared expert's type needs it) and the shared gate.
__global__ void __launch_bounds__(128) k_ep_unpack(const uint8_t *__restrict__ recv, int rec, bool kq, QAct dst, int H, int k,
                                                   uint32_t *__restrict__ idx, float *__restrict__ w, int own_begin, int own_count,
                                                   QAct home_other, QAct dst_other, bool other_kq, bool copy_other,
                                                   const float *__restrict__ home_sig, float *__restrict__ recv_sig)
{
    const int row = blockIdx.x;
    const uint8_t *src = recv + (size_t)row * rec;
    uint4 *qs = reinterpret_cast<uint4 *>(dst.qs + (size_t)row * H);
    for (int i = threadIdx.x; i < H / 16; i += blockDim.x) qs[i] = reinterpret_cast<const uint4 *>(src)[i];
    const uint8_t *o = src + H;
    if (kq) {
        for (int i = threadIdx.x; i < H / 256; i += blockDim.x) dst.d[(size_t)row * (H / 256) + i] = reinterpret_cast<const float *>(o)[i];
        o += (H / 256) * 4;
        for (int i = threadIdx.x; i < H / 16; i += blockDim.x) dst.bsums[(size_t)row * (H / 16) + i] = reinterpret_cast<const int16_t *>(o)[i];
        o += (H / 16) * 2;
    } else {
        for (int i = threadIdx.x; i < H / 32; i += blockDim.x) dst.d[(size_t)row * (H / 32) + i] = reinterpret_cast<const float *>(o)[i];
        o += (H / 32) * 4;
    }
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
        idx[(size_t)row * k + j] = reinterpret_cast<const uint32_t *>(o)[j];
        w[(size_t)row * k + j] = reinterpret_cast<const float *>(o + 4 * k)[j];
    }
    const int t = row - own_begin;
    if (t >= 0 && t < own_count) {   // the rank's own token t (it sent itself all its tokens, in order)
        if (home_sig && threadIdx.x == 0) recv_sig[row] = home_sig[t];
        if (copy_other) {
            const uint4 *s = reinterpret_cast<const uint4 *>(home_other.qs + (size_t)t * H);
            uint4 *d = reinterpret_cast<uint4 *>(dst_other.qs + (size_t)row * H);
            for (int i = threadIdx.x; i < H / 16; i += blockDim.x) d[i] = s[i];
            const int nd = other_kq ? H / 256 : H / 32;
            for (int i = threadIdx.x; i < nd; i += blockDim.x) dst_other.d[(size_t)row * nd + i] = home_other.d[(size_t)t * nd + i];
            if (other_kq)
                for (int i = threadIdx.x; i < H / 16; i += blockDim.x)
                    dst_other.bsums[(size_t)row * (H / 16) + i] = home_other.bsums[(size_t)t * (H / 16) + i];
        }
    }
}

// CTA t: out[t] = sum over the ranks token t visited, in rank order, of the row that rank returned.
template <typename OT>
__global__ void __launch_bounds__(256) k_ep_combine(const float *__restrict__ back, const int *__restrict__ pos,
                                                    const int *__restrict__ cnt, int n, int N, int H, int padded,
                                                    OT *__restrict__ out)
{
    __shared__ int s_row[EP_MAX_RANKS];
    const int t = blockIdx.x;
    if (threadIdx.x == 0) {
        int off = 0;
        for (int r = 0; r < N; r++) {
            const int p = pos[(size_t)t * N + r];
            s_row[r] = p < 0 ? -1 : off + p;
            off += padded ? n : cnt[r];
        }
    }
    __syncthreads();
    for (int h = threadIdx.x * 4; h < H; h += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < N; r++) {
            const int row = s_row[r];
            if (row < 0) continue;
            const float4 v = *reinterpret_cast<const float4 *>(back + (size_t)row * H + h);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        store_from_float(out, (size_t)t * H + h + 0, acc.x);
        store_from_float(out, (size_t)t * H + h + 1, acc.y);
        store_from_float(out, (size_t)t * H + h + 2, acc.z);
        store_from_float(out, (size_t)t * H + h + 3, acc.w);
    }
}

template <typename T> int ep_alloc(pmoe_ep_state *st, T **p, size_t count)
{
    void *q = nullptr;
    cudaError_t e = cudaMalloc(&q, count * sizeof(T) + 16);
    if (e != cudaSuccess) return fail_cuda(e, "expert-parallel buffers");
    st->owned.push_back(q);
    *p = reinterpret_cast<T *>(q);
    return PMOE_OK;
}

int ep_state_create(pmoe_layer *L, int N)
{
    pmoe_ep_state *st = new pmoe_ep_state();
    const size_t rows = (size_t)L->desc.max_tokens, H = L->desc.H, k = L->desc.k;
    st->rows = (int)rows;
    const int rk = rec_bytes_of((int)H, (int)k, true), r0 = rec_bytes_of((int)H, (int)k, false);
    st->rec_bytes = rk > r0 ? rk : r0;
    int rc = PMOE_OK;
    if (!rc) rc = ep_alloc(st, &st->home_q8k.qs, rows * H);
    if (!rc) rc = ep_alloc(st, &st->home_q8k.d, rows * (H / QK_K));
    if (!rc) rc = ep_alloc(st, &st->home_q8k.bsums, rows * (H / 16));
    if (!rc) rc = ep_alloc(st, &st->home_q80.qs, rows * H);
    if (!rc) rc = ep_alloc(st, &st->home_q80.d, rows * (H / QK8_0));
    if (!rc) rc = ep_alloc(st, &st->home_sig, rows);
    if (!rc) rc = ep_alloc(st, &st->recv_sig, rows);
    if (!rc) rc = ep_alloc(st, &st->send, rows * (size_t)st->rec_bytes);
    if (!rc) rc = ep_alloc(st, &st->recv, rows * (size_t)st->rec_bytes);
    if (!rc) rc = ep_alloc(st, &st->idx, rows * k);
    if (!rc) rc = ep_alloc(st, &st->w, rows * k);
    if (!rc) rc = ep_alloc(st, &st->part, rows * H);
    if (!rc) rc = ep_alloc(st, &st->back, rows * H);
    if (!rc) rc = ep_alloc(st, &st->pos, rows * (size_t)N);
    if (!rc) rc = ep_alloc(st, &st->cnt, (size_t)N);
    if (!rc) rc = ep_alloc(st, &st->cnt_all, (size_t)N * N);
    if (!rc && cudaMallocHost((void **)&st->cnt_host, sizeof(int) * N * N) != cudaSuccess) rc = fail(PMOE_ERR_CUDA, "pinned count buffer");
    for (int i = 0; i < 4 && !rc; i++)
        if (cudaEventCreate(&st->ev[i]) != cudaSuccess) rc = fail(PMOE_ERR_CUDA, "cudaEventCreate");
    if (rc) {
        ep_state_destroy(st);
        return rc;
    }
    L->ep = st;
    return PMOE_OK;
}

}  // namespace
}  // namespace pmoe

extern "C" {

int pmoe_ep_unique_id(void *id_out, size_t id_bytes)
{
    if (!id_out || id_bytes < sizeof(ncclUniqueId)) return fail(PMOE_ERR_INVALID_ARG, "id buffer must hold %zu bytes", sizeof(ncclUniqueId));
    std::string why;
    const NcclApi *api = nccl_api(&why);
    if (!api) return fail(PMOE_ERR_CUDA, "%s", why.c_str());
    ncclUniqueId id;
    NC(api, api->GetUniqueId(&id));
    memcpy(id_out, &id, sizeof id);
    return PMOE_OK;
}

int pmoe_ep_comm_create(const void *id, size_t id_bytes, int rank, int size, int device, pmoe_ep_comm **out)
{
    if (!id || !out || id_bytes < sizeof(ncclUniqueId)) return fail(PMOE_ERR_INVALID_ARG, "id / out is NULL or the id is too short");
    *out = nullptr;
    if (size < 1 || size > EP_MAX_RANKS || rank < 0 || rank >= size) return fail(PMOE_ERR_INVALID_ARG, "rank %d of %d (at most %d ranks)", rank, size, EP_MAX_RANKS);
    std::string why;
    const NcclApi *api = nccl_api(&why);
    if (!api) return fail(PMOE_ERR_CUDA, "%s", why.c_str());
    DeviceGuard guard(device);
    if (!guard.ok) return fail(PMOE_ERR_NO_DEVICE, "cannot select device %d", device);
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof uid);
    ncclComm_t comm = nullptr;
    NC(api, api->CommInitRank(&comm, size, uid, rank));
    pmoe_ep_comm *c = new pmoe_ep_comm();
    c->comm = comm; c->rank = rank; c->size = size; c->device = device; c->owned = true; c->api = api;
    *out = c;
    return PMOE_OK;
}

int pmoe_ep_comm_adopt(void *nccl_comm, int rank, int size, int device, pmoe_ep_comm **out)
{
    if (!nccl_comm || !out) return fail(PMOE_ERR_INVALID_ARG, "nccl_comm / out is NULL");
    *out = nullptr;
    if (size < 1 || size > EP_MAX_RANKS || rank < 0 || rank >= size) return fail(PMOE_ERR_INVALID_ARG, "rank %d of %d (at most %d ranks)", rank, size, EP_MAX_RANKS);
    std::string why;
    const NcclApi *api = nccl_api(&why);
    if (!api) return fail(PMOE_ERR_CUDA, "%s", why.c_str());
    pmoe_ep_comm *c = new pmoe_ep_comm();
    c->comm = (ncclComm_t)nccl_comm; c->rank = rank; c->size = size; c->device = device; c->owned = false; c->api = api;
    *out = c;
    return PMOE_OK;
}

int pmoe_ep_comm_destroy(pmoe_ep_comm *c)
{
    if (!c) return PMOE_OK;
    if (c->owned && c->comm) {
        DeviceGuard guard(c->device);
        c->api->CommDestroy(c->comm);
    }
    delete c;
    return PMOE_OK;
}

int pmoe_ep_forward(pmoe_layer *L, pmoe_ep_comm *C, const void *x, int x_dtype, int n, void *out, int out_dtype,
                    float *logits_out, uint32_t *idx_out, float *w_out, int mode, void *stream)
{
    int rc = check_call(L, x, x_dtype, n, out, out_dtype);
    if (rc) return rc;
    if (!C) return fail(PMOE_ERR_INVALID_ARG, "communicator is NULL");
    if (n <= 0) return fail(PMOE_ERR_INVALID_ARG, "every rank must bring at least one token (n = %d)", n);
    if (mode < 0 || mode > 2) return fail(PMOE_ERR_INVALID_ARG, "mode must be 0 (auto), 1 (padded counts) or 2 (exact counts)");
    const pmoe_layer_desc &d = L->desc;
    const LayerDev &dev = L->dev;
    const int N = C->size, me = C->rank;
    if (d.ep_size != N || d.ep_rank != me || dev.E_local != d.E / N || d.E % N)
        return fail(PMOE_ERR_INVALID_ARG, "the layer was created for rank %d of %d with %d local experts; the communicator is rank %d of %d",
                    d.ep_rank, d.ep_size, dev.E_local, me, N);
    if (d.ep_placement == 0 && d.expert_base != me * (d.E / N))
        return fail(PMOE_ERR_INVALID_ARG, "contiguous placement: expert_base must be rank * E / N");
    if ((long)n * N > d.max_tokens)
        return fail(PMOE_ERR_TOO_MANY_TOKENS, "n = %d tokens on each of %d ranks exceed max_tokens = %d", n, N, d.max_tokens);
    if (C->device != L->device) return fail(PMOE_ERR_INVALID_ARG, "communicator and layer live on different devices");
    DeviceGuard guard(L->device);
    if (!L->ep && (rc = ep_state_create(L, N)) != PMOE_OK) return rc;
    pmoe_ep_state *st = L->ep;
    const NcclApi *api = C->api;
    cudaStream_t s = (cudaStream_t)stream;
    const bool padded = mode == 1 || (mode == 0 && (long)n * N < 2048);
    const int H = d.H, k = d.k;
    const bool kq = is_kquant(dev.gate_dtype);                         // form of the travelling rows
    const bool sh = dev.has_shared != 0;
    const bool sh_kq = sh && is_kquant(dev.sh_gate_dtype);
    const bool need_other = sh && sh_kq != kq;                          // the shared expert eats the other form
    const int rec = rec_bytes_of(H, k, kq);

    // ---- 1. route the home tokens; the same launch quantises them into the home arrays
    float *logits = logits_out ? logits_out : L->ws.logits;
    uint32_t *idx = idx_out ? idx_out : L->ws.topk_idx;
    float *w = w_out ? w_out : L->ws.topk_w;
    Workspace wh = L->ws;
    wh.x_q8k = st->home_q8k;
    wh.x_q80 = st->home_q80;
    wh.sh_sigmoid = st->home_sig;
    CU(launch_router(dev, wh, x, x_dtype, n, logits, s, true, kq || (sh && sh_kq), !kq || (sh && !sh_kq), sh));
    CU(launch_topk(dev, wh, logits, n, idx, w, s));

    // ---- 2, 3. plan and pack
    if (st->profile) cudaEventRecord(st->ev[0], s);
    k_ep_plan<<<N, 1024, 0, s>>>(idx, n, k, d.E, N, d.ep_placement, me, 1, padded ? 1 : 0, st->pos, st->cnt);
    k_ep_pack<<<n, 128, 0, s>>>(kq ? st->home_q8k : st->home_q80, kq, idx, w, H, k, d.E, N, d.ep_placement, n, padded ? 1 : 0,
                                st->pos, st->cnt, st->send, rec);
    count_launch(2);
    CU(cudaGetLastError());

    // ---- 4. counts and exchange
    EpOffsets off{};
    int send_cnt[EP_MAX_RANKS], recv_cnt[EP_MAX_RANKS];
    if (padded) {
        for (int r = 0; r < N; r++) send_cnt[r] = recv_cnt[r] = n;
    } else {
        NC(api, api->AllGather(st->cnt, st->cnt_all, (size_t)N, ncclInt32, C->comm, s));
        CU(cudaMemcpyAsync(st->cnt_host, st->cnt_all, sizeof(int) * N * N, cudaMemcpyDeviceToHost, s));
        CU(cudaStreamSynchronize(s));
        for (int r = 0; r < N; r++) {
            send_cnt[r] = st->cnt_host[me * N + r];
            recv_cnt[r] = st->cnt_host[r * N + me];
        }
    }
    for (int r = 0; r < N; r++) {
        off.send_off[r + 1] = off.send_off[r] + send_cnt[r];
        off.recv_off[r + 1] = off.recv_off[r] + recv_cnt[r];
    }
    const int rows = off.recv_off[N];
    if (rows > d.max_tokens) return fail(PMOE_ERR_TOO_MANY_TOKENS, "%d records arrive, max_tokens = %d", rows, d.max_tokens);
    NC(api, api->GroupStart());
    for (int r = 0; r < N; r++) {
        if (send_cnt[r])
            NC(api, api->Send(st->send + (size_t)off.send_off[r] * rec, (size_t)send_cnt[r] * rec, ncclUint8, r, C->comm, s));
        if (recv_cnt[r])
            NC(api, api->Recv(st->recv + (size_t)off.recv_off[r] * rec, (size_t)recv_cnt[r] * rec, ncclUint8, r, C->comm, s));
    }
    NC(api, api->GroupEnd());
    if (st->profile) cudaEventRecord(st->ev[1], s);

    // ---- 5. unpack and run this rank's experts over the received rows; the shared expert on the rank's own rows
    const int own_begin = off.recv_off[me], own_count = recv_cnt[me];   // = n: a rank sends itself all its tokens
    Workspace wr = L->ws;
    wr.sh_sigmoid = st->recv_sig;
    k_ep_unpack<<<rows, 128, 0, s>>>(st->recv, rec, kq, kq ? wr.x_q8k : wr.x_q80, H, k, st->idx, st->w, own_begin, own_count,
                                     kq ? st->home_q80 : st->home_q8k, kq ? wr.x_q80 : wr.x_q8k, !kq, need_other,
                                     sh ? st->home_sig : nullptr, st->recv_sig);
    count_launch();
    CU(cudaGetLastError());
    L->req_sh_begin = own_begin;
    L->req_sh_count = sh ? own_count : -1;
    for (bool &u : L->ev_used) u = false;
    rc = run_experts(L, wr, nullptr, PMOE_F32, st->idx, st->w, rows, k, true, sh, true, st->part, PMOE_F32, s);
    if (rc) return rc;

    // ---- 6. the rows go back the way they came; per home token the returned rows are added in rank order
    if (st->profile) cudaEventRecord(st->ev[2], s);
    NC(api, api->GroupStart());
    for (int r = 0; r < N; r++) {
        if (recv_cnt[r])
            NC(api, api->Send(st->part + (size_t)off.recv_off[r] * H, (size_t)recv_cnt[r] * H, ncclFloat32, r, C->comm, s));
        if (send_cnt[r])
            NC(api, api->Recv(st->back + (size_t)off.send_off[r] * H, (size_t)send_cnt[r] * H, ncclFloat32, r, C->comm, s));
    }
    NC(api, api->GroupEnd());
    if (out_dtype == PMOE_F32)
        k_ep_combine<float><<<n, 256, 0, s>>>(st->back, st->pos, st->cnt, n, N, H, padded ? 1 : 0, (float *)out);
    else
        k_ep_combine<__nv_bfloat16><<<n, 256, 0, s>>>(st->back, st->pos, st->cnt, n, N, H, padded ? 1 : 0, (__nv_bfloat16 *)out);
    count_launch();
    CU(cudaGetLastError());
    if (st->profile) cudaEventRecord(st->ev[3], s);
    return PMOE_OK;
}

int pmoe_ep_profile(pmoe_layer *L, int enable, float *dispatch_ms, float *combine_ms)
{
    if (!L) return fail(PMOE_ERR_INVALID_ARG, "layer is NULL");
    if (!L->ep) {
        if (enable >= 0) return fail(PMOE_ERR_INVALID_ARG, "no expert-parallel forward has run on this layer yet");
        return PMOE_OK;
    }
    DeviceGuard guard(L->device);
    pmoe_ep_state *st = L->ep;
    if (dispatch_ms || combine_ms) {
        if (!st->profile) return fail(PMOE_ERR_INVALID_ARG, "profiling is off");
        CU(cudaEventSynchronize(st->ev[3]));
        float a = 0.f, b = 0.f;
        CU(cudaEventElapsedTime(&a, st->ev[0], st->ev[1]));
        CU(cudaEventElapsedTime(&b, st->ev[2], st->ev[3]));
        if (dispatch_ms) *dispatch_ms = a;
        if (combine_ms) *combine_ms = b;
    }
    if (enable >= 0) st->profile = enable != 0;
    return PMOE_OK;
}

}  // extern "C"
