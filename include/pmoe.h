/*
 * pmoe.h -- C ABI of libpmoe: the Qwen3-Next quantised mixture-of-experts FFN block
 * for NVIDIA B200 (sm_100a).
 *
 * The entry points are what paramecia-model's FFI for this path binds.  Each one names
 * the reference interface it stands in for (path inside nicksenger/paramecia : lines).
 * Plain pointers and sizes only.  Unless stated otherwise every data pointer is a
 * DEVICE pointer on the layer's device and `stream` is a cudaStream_t passed as void*
 * (NULL = the default stream).  Calls are asynchronous on that stream.
 *
 * Every function returns 0 on success or a negative pmoe_status; the message of the
 * last failure on the calling thread is available from pmoe_last_error().  Nothing
 * here aborts, traps or falls back to the CPU.
 *
 * A layer handle serves one call at a time (the reference serialises forwards behind
 * Arc<tokio::Mutex<ModelWeights>>, paramecia-llm/src/backend/local.rs:60,741) but may
 * be used from any host thread.
 */
#ifndef PMOE_H
#define PMOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PMOE_VERSION 4

/* GGML tensor-type ids, the numbering of candle's GgmlDType / GGUF files. */
typedef enum {
    PMOE_F32 = 0,
    PMOE_F16 = 1,
    PMOE_Q8_0 = 8,
    PMOE_Q2_K = 10,
    PMOE_Q3_K = 11,
    PMOE_Q4_K = 12,
    PMOE_Q5_K = 13,
    PMOE_Q6_K = 14,
    PMOE_BF16 = 30
} pmoe_dtype;

typedef enum {
    PMOE_OK = 0,
    PMOE_ERR_INVALID_ARG = -1,
    PMOE_ERR_UNSUPPORTED_DTYPE = -2,
    PMOE_ERR_UNSUPPORTED_SHAPE = -3,
    PMOE_ERR_CUDA = -4,
    PMOE_ERR_TOO_MANY_TOKENS = -5,
    /* block-scale multipliers are installed (EGGROLL/QZO training): the fast paths are
       bypassed in the reference too (qwen3_next.rs:1977,1989); the caller falls back */
    PMOE_ERR_TRAINING_MODE = -6,
    PMOE_ERR_TIMEOUT = -7,   /* a bounded device-side wait ran out */
    PMOE_ERR_BAD_INDEX = -8, /* a device-side range check failed */
    PMOE_ERR_NO_DEVICE = -9
} pmoe_status;

typedef struct pmoe_layer pmoe_layer; /* opaque */

/*
 * One MoE block.  Mirrors what MoeBlock::new / MoeExperts::new / SharedExpert::new read
 * from a GGUF file (qwen3_next.rs:1864-1895, 1256-1258, 1749-1774):
 *   blk.N.ffn_gate_inp.weight             router_w       [E, H]
 *   blk.N.ffn_{gate,up}_exps.weight       gate/up_exps   [E_local, F, H]
 *   blk.N.ffn_down_exps.weight            down_exps      [E_local, H, F]
 *   blk.N.ffn_{gate,up,down}_shexp.weight sh_gate/up/down
 *   blk.N.ffn_gate_inp_shexp[.weight]     sh_gate_inp    [H] (dequantised to f32 at load)
 * Expert tensors are raw GGUF blocks, row-major, expert e one contiguous slice
 * (QTensor::data(), slice_first_dim; qwen3_next.rs:1052,1548).
 */
typedef struct {
    uint32_t struct_size;  /* sizeof(pmoe_layer_desc) */
    int32_t device;        /* CUDA device ordinal */
    int32_t H, F, E, k;    /* hidden, expert intermediate, experts (global), experts per token */
    int32_t max_tokens;    /* workspace is sized for this many tokens per call */

    /* Routed experts held by this handle.  ep_placement 0 (contiguous): global ids
       [expert_base, expert_base+E_local), local expert i = global expert_base + i;
       E_local == 0 means all E.  ep_placement 1 (round-robin over ep_size ranks): the
       E_local = E / ep_size experts ep_rank, ep_rank + ep_size, ... in that order
       (expert_base is ignored); under a skewed router neighbouring hot experts then land
       on different ranks.  Indices the handle does not hold are skipped, the way the
       reference skips indices >= num_experts (qwen3_next.rs:2045); expert parallelism
       gives every rank one share.  The reference runs one process and has no such table. */
    int32_t expert_base, E_local;

    int32_t gate_dtype, up_dtype, down_dtype;
    const void *gate_exps, *up_exps, *down_exps;

    int32_t has_shared;
    int32_t sh_gate_dtype, sh_up_dtype, sh_down_dtype;
    const void *sh_gate, *sh_up, *sh_down;
    const float *sh_gate_inp;

    int32_t router_dtype;     /* PMOE_F32, PMOE_F16 / PMOE_BF16 (widened to f32 at create), or a GGUF block type
                                 (Q8_0, Q2_K ... Q6_K; [E, H / block] blocks): the router is then a quantised
                                 mat-mul like the experts' (models/with_tracing.rs:324-335), rows quantised to
                                 Q8_K / Q8_0, integer block dots, f32 scales */
    const void *router_w;
    const float *router_bias; /* [E] added to the logits, or NULL (not in the reference;
                                 used to skew synthetic routing) */

    /* 0: the pointers above are host memory, copied to the device at create.
       1: device memory, copied into storage the handle owns.
       2: device memory, adopted in place (no copy); it must outlive the handle and be
          16-byte aligned.  This is how a candle QTensor already on the GPU is used. */
    int32_t weights_location;

    /* non-zero when the host holds custom block multipliers (MoeExperts::set_block_multipliers,
       qwen3_next.rs:1705-1720) that it has NOT handed to pmoe_layer_set_block_multipliers: every
       forward then returns PMOE_ERR_TRAINING_MODE, the way the reference bypasses its own fast
       paths (qwen3_next.rs:1977,1989).  A host that installs the multipliers in the handle
       leaves this 0 and keeps the fast path. */
    int32_t training_mode;

    /* expert -> rank table of an expert-parallel group (see expert_base above) */
    int32_t ep_placement; /* 0 contiguous, 1 round-robin */
    int32_t ep_rank, ep_size; /* used by ep_placement 1 and by pmoe_ep_forward; 0, 0 = a single GPU */
} pmoe_layer_desc;

/* MoeBlock::new (qwen3_next.rs:1864-1895) */
int pmoe_layer_create(const pmoe_layer_desc *desc, pmoe_layer **out);
/* Drop for MoeBlock */
int pmoe_layer_destroy(pmoe_layer *layer);

/*
 * MoeBlock::forward_with_stats (qwen3_next.rs:1903-1940).
 *   x       [n, H]  x_dtype in {PMOE_F32, PMOE_BF16}
 *   out     [n, H]  out_dtype in {PMOE_F32, PMOE_BF16}
 *   logits_out [n, E] f32, the UNCLAMPED router logits (qwen3_next.rs:1939), or NULL
 *   idx_out    [n, k] u32 top-k expert ids, descending probability, or NULL
 *   w_out      [n, k] f32 renormalised routing weights, or NULL
 */
int pmoe_forward(pmoe_layer *layer, const void *x, int x_dtype, int n, void *out, int out_dtype,
                 float *logits_out, uint32_t *idx_out, float *w_out, void *stream);

/*
 * The same call with HOST buffers: copies x to the device, runs the block, copies the
 * results back and synchronises the stream.  This is the shape of the reference's own
 * offload paths (Tensor::to_device around the expert computation, ops.rs:188-198,291-293).
 * From the third call with the same n and dtypes on, the kernels between the two copies are
 * replayed from a CUDA graph the handle recorded (PMOE_HOST_GRAPH=0 in the environment keeps
 * direct launches).
 */
int pmoe_forward_host(pmoe_layer *layer, const void *x_host, int x_dtype, int n, void *out_host,
                      int out_dtype, float *logits_host, uint32_t *idx_host, float *w_host,
                      void *stream);

/*
 * Router only: gate.forward, clamp, softmax, ops::topk_moe_routing
 * (qwen3_next.rs:1916-1925, ops.rs:28-59).  Any output may be NULL.
 */
int pmoe_route(pmoe_layer *layer, const void *x, int x_dtype, int n, float *logits_out,
               uint32_t *idx_out, float *w_out, void *stream);

/*
 * Router statistics of one block, as the reference's auxiliary training losses use them
 * (compute_z_loss and compute_load_balance_loss, qwen3_next.rs:5549-5648) -- here per block,
 * on the device, from the (router_logits, top_indices) pair pmoe_forward / pmoe_route return:
 *   counts_out [E] f32   number of selections of each expert (ids >= E are skipped),
 *   losses_out [0]       z    = mean_t logsumexp(logits_t)^2,
 *   losses_out [1]       lb   = E * sum_e (counts[e] / (n*top_k)) * mean_t softmax(logits_t)[e].
 * The reference averages both over the blocks and multiplies by its loss weights; that is left
 * to the caller.  Either output may be NULL.  Uses the handle's workspace: not concurrent with
 * another call on the same handle.
 */
int pmoe_router_stats(pmoe_layer *layer, const float *logits, const uint32_t *idx, int n, int top_k,
                      float *counts_out, float *losses_out, void *stream);

/*
 * MoeExperts::forward_batched (qwen3_next.rs:1347-1394): routed experts only, with the
 * caller's routing.  idx [n, top_k] u32 (global expert ids), w [n, top_k] f32.
 */
int pmoe_experts_forward(pmoe_layer *layer, const void *x, int x_dtype, const uint32_t *idx,
                         const float *w, int n, int top_k, void *out, int out_dtype, void *stream);

/*
 * Expert-parallel form of the two calls around this one: the routed experts over all n rows
 * (MoeExperts::forward_batched, qwen3_next.rs:1347-1394) plus the shared expert
 * (SharedExpert::forward, qwen3_next.rs:1776-1823) added on rows [shared_begin,
 * shared_begin + shared_count) only, in the same kernels.  A rank that received n rows from
 * every rank calls it with the range of its own rows, so that each token's shared expert is
 * computed exactly once across the ranks.  shared_count = 0, or a layer without a shared
 * expert, gives pmoe_experts_forward.  The reference has no such call: it runs one process.
 */
int pmoe_experts_forward_ep(pmoe_layer *layer, const void *x, int x_dtype, const uint32_t *idx,
                            const float *w, int n, int top_k, int shared_begin, int shared_count,
                            void *out, int out_dtype, void *stream);

/*
 * MoeExperts::set_block_multipliers / clear_block_multipliers (qwen3_next.rs:1705-1732): the
 * per-block scale multipliers of the EGGROLL / QZO training mode.  Each array is DEVICE f32 with
 * one value per quantisation block of this handle's tensor in storage order -- [E_local, F, H/blk],
 * [E_local, F, H/blk], [E_local, H, F/blk]; expert e owns blocks [e*B, (e+1)*B) as in
 * extract_expert_scales (1688-1703).  The three come together; all NULL removes them.
 *
 * The reference builds, per expert and per use, QTensor::modify_block_scales copies of the three
 * matrices (build_scaled_mats, 1554-1621) and multiplies through those.  Here the handle keeps one
 * scaled copy of each tensor (device memory of the tensor's own size, allocated by this call) and
 * every entry point reads the copies, tensor-core paths included, until the multipliers are
 * removed.  The scaling runs on `stream`; use the stream the forwards use.  Not concurrent with
 * another call on the handle.
 */
int pmoe_layer_set_block_multipliers(pmoe_layer *layer, const float *gate_mults, const float *up_mults,
                                     const float *down_mults, void *stream);

/* SharedExpert's custom_gate_scales / custom_up_scales / custom_down_scales (qwen3_next.rs:1743-1745,
 * used through QMatMul::forward_with_scales at 1780-1799): independent of one another, NULL = none.
 * Same layout rule and lifetime as above for the [F, H/blk], [F, H/blk], [H, F/blk] tensors. */
int pmoe_layer_set_shared_scales(pmoe_layer *layer, const float *gate_scales, const float *up_scales,
                                 const float *down_scales, void *stream);

/* QTensor::modify_block_scales as QMatMul::forward_with_scales calls it (models/with_tracing.rs:217-248):
 * out = blocks with block i's f16 scale d -- and dmin for Q2_K / Q4_K / Q5_K -- multiplied by mults[i]
 * and rounded back to f16; quants and packed sub-scales unchanged.  out may be blocks.  All device
 * pointers.  (The routine itself is in the candle fork the reference depends on, which is not part of
 * its tree: this restates "every value of the block times m".) */
int pmoe_modify_block_scales(int device, int dtype, const void *blocks, size_t n_blocks, const float *mults,
                             void *out, void *stream);

/*
 * Expert-parallel form of pmoe_forward: MoeBlock::forward_with_stats (qwen3_next.rs:1903-1940) for a block whose
 * routed experts are spread over the ranks of a communicator, one process per GPU.  The reference has no
 * counterpart: it runs one process on one device (its expert loop is a rayon loop, tokio_experts.rs:116-130).
 *
 * Every rank creates its layer with ep_rank / ep_size, E_local = E / ep_size experts (ep_placement says which) and
 * max_tokens >= ep_size * n, and calls pmoe_ep_forward with its own n tokens (the same n on every rank).  A
 * token's quantised row travels once to every rank that holds one of its top-k experts (grouped ncclSend /
 * ncclRecv, an all-to-all-v), that rank returns one pre-reduced f32 row, and the home rank adds the returned rows
 * in rank order; the shared expert runs on the home rank.  x, out, logits_out, idx_out, w_out as in pmoe_forward,
 * for the rank's own tokens.
 *
 * mode 1 (padded counts): every pair of ranks exchanges n records; no host synchronisation.  mode 2 (exact
 * counts): the ranks all-gather their counts first and the host reads them (one stream synchronisation per call);
 * only the rows that are needed travel.  mode 0: padded below 2048 rows in flight, exact from there on.
 *
 * The communicator: rank 0 calls pmoe_ep_unique_id and hands the bytes to the others over any channel the host
 * has, then every rank calls pmoe_ep_comm_create (ncclCommInitRank; collective).  A host that already owns an
 * ncclComm_t for exactly these ranks passes it to pmoe_ep_comm_adopt instead.  NCCL (libnccl.so.2) is loaded on
 * first use.  At most 64 ranks.
 */
typedef struct pmoe_ep_comm pmoe_ep_comm; /* opaque */
#define PMOE_EP_ID_BYTES 128
int pmoe_ep_unique_id(void *id_out, size_t id_bytes);
int pmoe_ep_comm_create(const void *id, size_t id_bytes, int rank, int size, int device, pmoe_ep_comm **out);
int pmoe_ep_comm_adopt(void *nccl_comm, int rank, int size, int device, pmoe_ep_comm **out);
int pmoe_ep_comm_destroy(pmoe_ep_comm *comm);
int pmoe_ep_forward(pmoe_layer *layer, pmoe_ep_comm *comm, const void *x, int x_dtype, int n, void *out,
                    int out_dtype, float *logits_out, uint32_t *idx_out, float *w_out, int mode, void *stream);
/* Device time the two exchanges of the last pmoe_ep_forward took on its stream (dispatch: plan, pack, counts,
 * exchange; combine: return exchange and the sum), in milliseconds; either pointer may be NULL.  enable 1 / 0
 * switches the event records on / off for the following calls, -1 leaves the setting.  Valid after the layer's
 * first pmoe_ep_forward. */
int pmoe_ep_profile(pmoe_layer *layer, int enable, float *dispatch_ms, float *combine_ms);

/* SharedExpert::forward (qwen3_next.rs:1776-1823), sigmoid gate included. */
int pmoe_shared_forward(pmoe_layer *layer, const void *x, int x_dtype, int n, void *out,
                        int out_dtype, void *stream);

/*
 * QMatMul::forward on a quantised tensor (models/with_tracing.rs:324-335):
 * y[m, rows] = x[m, cols] * W[rows, cols]^T, activations quantised to the weight type's
 * dot type as the reference CPU path does.  x, y f32; w and x 16-byte aligned; cols a multiple
 * of 256.  Stream-ordered scratch comes from cudaMallocAsync.  Meant for parity checks and
 * small operands (one warp per output row), not for the block's hot path.
 */
int pmoe_qmatmul(int device, int dtype, const void *w, size_t rows, size_t cols, const float *x,
                 size_t m, float *y, void *stream);

/*
 * pmoe_qmatmul for hosts that must not allocate.  No counterpart in the reference: paramecia
 * lets candle allocate freely.  It is for embedders that have already handed every byte of
 * device memory to their own pool (a serving process that sized its KV cache to fill the
 * card, say) or that forbid allocator calls on the request path because an allocation can
 * stall every stream of the process.  This entry point calls neither cudaMalloc, cudaFree,
 * their stream-ordered forms nor any allocating library routine: the quantised activations
 * go into a 96 KB buffer compiled into the library (held by every GPU that loads it, until
 * the process exits).
 *
 * Limits: the quantised rows must fit that buffer: 1.25 * m * cols + 768 <= 98 304 bytes, so
 * every m * cols <= 78 028 fits -- 38 rows of 2048 columns, 152 rows of 512 -- otherwise
 * PMOE_ERR_TOO_MANY_TOKENS with the sizes in pmoe_last_error(); nothing is truncated.  Same
 * arguments (cols a multiple of 256, at most 16 384), results and other errors as pmoe_qmatmul.
 *
 * The first call on a device looks up the buffer's device address (one runtime query, no
 * allocation); make that first call during start-up, before any stream capture begins.
 * All calls on a device share the one buffer: it keeps the previous call's contents, every
 * byte a call reads is written by that call first (nothing relies on zeros), and two calls
 * that overlap on the GPU -- different streams, or different threads without ordering --
 * race on it.  Order them on one stream or with events.
 */
int pmoe_qmatmul_noalloc(int device, int dtype, const void *w, size_t rows, size_t cols,
                         const float *x, size_t m, float *y, void *stream);

/* QTensor::dequantize: blocks -> f32 (the "dequantised weights bit-exact" check). */
int pmoe_dequantize(int device, int dtype, const void *blocks, size_t n_elems, float *out,
                    void *stream);

/* RmsNorm::forward (quantized_nn.rs:172-190) fused with the residual add of
 * LayerWeights::forward_with_stats (qwen3_next.rs:4273-4286):
 *   resid_out = resid_in + delta (delta may be NULL), y = rms_norm(resid_out) * weight.
 * f32 throughout; weight NULL = all ones. */
int pmoe_add_rms_norm(int device, const float *resid_in, const float *delta, const float *weight,
                      int n, int H, float eps, float *resid_out, float *y, void *stream);

/*
 * Home-rank side of the expert-parallel combine: out[t] = sum_r parts[r][t] (+ extra[t]).
 * parts [n_parts, n, H] f32 are the per-rank partial sums a token's expert owners returned,
 * extra [n, H] (F32 or BF16, may be NULL) is the gated shared-expert row.  It continues the
 * reference's accumulation of expert outputs into one buffer (tokio_experts.rs:133-145) and
 * the final add (qwen3_next.rs:1932-1937) across GPUs; the reference itself is single-device.
 */
int pmoe_reduce_rows(int device, const float *parts, int n_parts, const void *extra, int extra_dtype,
                     int n, int H, void *out, int out_dtype, void *stream);

/* Synchronises the stream and reports the device-side status word of the layer
 * (PMOE_OK, PMOE_ERR_TIMEOUT, PMOE_ERR_BAD_INDEX), clearing it. */
int pmoe_layer_status(pmoe_layer *layer, void *stream);

/*
 * Per-phase device timing, the counterpart of the reference's tracing spans ("moe-block",
 * "moe-experts", "qmatmul"; qwen3_next.rs:1884,1260, models/with_tracing.rs:116).  While
 * enabled, pmoe_forward brackets each kernel with CUDA events on the caller's stream;
 * pmoe_layer_trace_read waits for the last call and returns its milliseconds per phase
 * (ms[PMOE_TRACE_PHASES]; phases a call did not run read 0).
 */
#define PMOE_TRACE_PHASES 8
int pmoe_layer_trace(pmoe_layer *layer, int enable);
int pmoe_layer_trace_read(pmoe_layer *layer, float *ms);
const char *pmoe_trace_phase_name(int phase);

/* number of kernels of this library launched by this process so far */
uint64_t pmoe_launch_count(void);

size_t pmoe_block_size(int dtype); /* weights per block */
size_t pmoe_type_size(int dtype);  /* bytes per block */
const char *pmoe_last_error(void);
int pmoe_version(void);

#ifdef __cplusplus
}
#endif
#endif
