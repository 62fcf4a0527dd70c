/*
 * pmoe_oracle.h -- CPU restatement of paramecia's quantised MoE FFN block.
 *
 * TEST INFRASTRUCTURE ONLY.  This is the checker that the CUDA library is
 * compared against and the CPU baseline that the benchmark times.  Nothing in
 * the shipped library links, loads or calls it.
 *
 * PARITY UNPINNED: the arithmetic of the reference path lives in a third-party
 * crate that is not part of the reference tree (candle-core 0.9.2-alpha.2,
 * git nicksenger/candle, branch paramecia, commit 2278f29b, pinned at
 * Cargo.lock:388-390) and the reference holds no golden vectors for this path
 * (its only routing test, paramecia-model/src/ops.rs:644-663, checks shapes and
 * that the renormalised weights sum to 1).  The block codecs here are pinned
 * bit-exactly against the independent gguf-py dequantiser (tests/golden); the
 * activation quantisers and integer block dot products restate candle's
 * published CPU algorithm (k_quants: BlockQ8K::from_float, BlockQ8_0::from_float,
 * vec_dot for Q4K/Q6K/Q8_0 and the row-by-row `matmul`).
 */
#ifndef PMOE_ORACLE_H
#define PMOE_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML dtype numbering (the ids candle's GgmlDType uses). */
enum { PMO_F32 = 0, PMO_F16 = 1, PMO_Q8_0 = 8, PMO_Q2_K = 10, PMO_Q3_K = 11, PMO_Q4_K = 12, PMO_Q5_K = 13, PMO_Q6_K = 14 };

typedef struct {
    int32_t H, F, E, k;           /* hidden, expert intermediate, experts, experts per token */
    int32_t gate_dtype, up_dtype, down_dtype;
    const void *gate_exps;        /* [E,F,H] blocks, row-major, expert e = contiguous slice */
    const void *up_exps;          /* [E,F,H] */
    const void *down_exps;        /* [E,H,F] */
    int32_t has_shared;
    int32_t sh_gate_dtype, sh_up_dtype, sh_down_dtype;
    const void *sh_gate;          /* [F,H] */
    const void *sh_up;            /* [F,H] */
    const void *sh_down;          /* [H,F] */
    const float *sh_gate_inp;     /* [H] f32 */
    const float *router_w;        /* [E,H] f32 */
    const float *router_bias;     /* [E] f32 or NULL; synthetic-workload knob, added to the logits */
    int32_t router_dtype;         /* PMO_F32 (router_w), or a block type: the router is a quantised mat-mul over router_q */
    const void *router_q;         /* [E, H / block] blocks when router_dtype is a block type */
} pmo_layer;

size_t pmo_block_size(int dtype);      /* weights per block */
size_t pmo_type_size(int dtype);       /* bytes per block   */
size_t pmo_row_bytes(int dtype, size_t cols);

/* block codecs */
int pmo_dequantize(int dtype, const void *blocks, size_t n_elems, float *out);
int pmo_quantize(int dtype, const float *x, size_t n_elems, void *blocks);   /* weight quantisers */

/* QTensor::modify_block_scales (training mode, qwen3_next.rs:1604-1606): block i's f16 scale(s) times mults[i];
   out may equal blocks.  [UNVERIFIED: the routine lives in the candle fork] */
int pmo_modify_block_scales(int dtype, const void *blocks, size_t n_blocks, const float *mults, void *out);

/* activation quantisers (candle BlockQ8K / BlockQ8_0 from_float) */
void pmo_quantize_q8k(const float *x, size_t n, float *d, int8_t *qs, int16_t *bsums);
void pmo_quantize_q8_0_act(const float *x, size_t n, uint16_t *d_f16, int8_t *qs);

/* y[m,rows] = x[m,cols] * W[rows,cols]^T with W quantised (candle k_quants::matmul) */
int pmo_qmatmul(int dtype, const void *w, size_t rows, size_t cols, const float *x, size_t m, float *y);

/* the layer's router, f32 or quantised (a QMatMul like the experts': models/with_tracing.rs:324-335): unclamped logits */
int pmo_layer_router_logits(const pmo_layer *L, const float *x, int n, float *logits);
/* router: canonical-order f32 GEMV + optional bias; unclamped logits out */
void pmo_router_logits(const float *router_w, const float *bias, int E, int H, const float *x, int n, float *logits);
/* clamp(+-100) -> softmax -> first k of a stable descending sort -> renormalise */
void pmo_route_topk(const float *logits, int n, int E, int k, uint32_t *idx, float *w, float *probs_opt);

/* routed experts only (MoeExperts::forward_batched semantics computed the CPU way) */
int pmo_experts_forward(const pmo_layer *L, const float *x, int n, const uint32_t *idx, const float *w,
                        int k, float *out);
/* shared expert incl. sigmoid gate */
int pmo_shared_forward(const pmo_layer *L, const float *x, int n, float *out);
/* whole block: MoeBlock::forward_with_stats */
int pmo_moe_forward(const pmo_layer *L, const float *x, int n, float *out,
                    float *logits_out, uint32_t *idx_out, float *w_out);
/* same block in exact arithmetic: fp64 dots of the dequantised weights, no activation quantisation.
   Uses the routing given (idx,w) so that only the expert arithmetic differs. */
int pmo_moe_forward_exact(const pmo_layer *L, const float *x, int n, const uint32_t *idx, const float *w,
                          float *out);

/* RmsNorm::forward (quantized_nn.rs:172-190): y = x / sqrt(mean(x^2)+eps) * weight */
void pmo_rms_norm(const float *x, const float *weight, int n, int H, float eps, float *y);

int pmo_max_threads(void);
void pmo_set_threads(int n);
void pmo_set_simd(int on);   /* 0: the portable block dots everywhere (same bits, slower) */
const char *pmo_simd_kind(void);

#ifdef __cplusplus
}
#endif
#endif
