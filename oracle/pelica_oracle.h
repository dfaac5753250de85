/* pelica_oracle.h - CPU restatement of Pelica's mixture-of-experts arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product path may call this: it is
 * the checker the CUDA path is compared with, and the timed CPU baseline.
 *
 * Each function restates the reference code cited beside it (paths inside the
 * Pelica source tree). The reference is Rust + WGSL and cannot be built where
 * this oracle is built, and its tests hold no stored expected numbers for this
 * path; what pins this oracle is (a) the reference's own relational tests
 * re-run on it (scalar vs SIMD rows, multi-token vs single-token rows,
 * f16 round trip incl. its two exact ties-to-even cases, bf16 dot == f32 dot)
 * and (b) hand-computed known-answer vectors for each block format.
 * Routing, plan, combine, Q6_K rows, MXFP4 rows, group-limited selection and
 * whole-layer outputs have no known-answer test in the reference:
 * PARITY UNPINNED for those (the oracle is a statement-by-statement reading).
 *
 * Build: make -C oracle   (gcc, -ffp-contract=off so only spelled-out fmaf fuse)
 */
#ifndef PELICA_ORACLE_H
#define PELICA_ORACLE_H

#include <stddef.h>
#include <stdint.h>
#include "../include/pelica_moe.h" /* enums and pm_layer_desc only (plain data) */

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scalars ----------------------------------------------------------- */
float po_f16_to_f32(uint16_t h);   /* src/ds4.rs:168-180 */
uint16_t po_f32_to_f16(float x);   /* src/q4x.rs:102-134 (round to nearest even) */
float po_bf16_to_f32(uint16_t h);  /* src/moe.rs:355 */
uint16_t po_f32_to_bf16(float x);  /* round to nearest even (generator side only) */
/* e^x from adds, multiplies and explicit fmas only: `pexp`
 * (src/moe_kernels.rs:437-468, src/cpu_attn.rs:30-44) with its argument range
 * widened to [-87, 88] (below -> 0, above -> +inf) so SwiGLU and sigmoid can use
 * the same bit-reproducible exp on CPU and GPU. */
float po_exp(float x);
/* ln(1+x) for x >= 0 from the same kind of arithmetic (fmas, one division);
 * used by sqrt-softplus gating only */
float po_log1p(float x);
/* `dot_f32` (src/quant.rs:215-236): 32 lanes, lane = column mod 32, fma chains,
 * lanes summed (0+1)+(2+3) accumulators then 4,2,1 */
float po_dot_f32(const float *a, const float *b, size_t n);
float po_dot_bf16(const uint16_t *a, const float *b, size_t n); /* src/quant.rs:282-304 */

/* ---- block formats ----------------------------------------------------- */
size_t po_type_block_bytes(int ggml_type);
size_t po_type_block_values(int ggml_type);
/* values of whole blocks -> f32 (`deq4`, src/moe_kernels.rs:63-84 on raw GGUF
 * blocks; Q8_0 also src/q4x_cpu.rs:443-452). returns 0 or PM_ERR_UNSUPPORTED */
int po_dequant(int ggml_type, const uint8_t *blocks, size_t n_values, float *out);

/* ---- activation quantisers -------------------------------------------- */
/* `Q8x::new` (src/ds4_cpu.rs:13-35): n % 256 == 0; q[n], d[n/256], bsum[n/32] */
void po_q8x(const float *x, size_t n, int8_t *q, float *d, int32_t *bsum);
/* `Q8::new` (src/q4x_cpu.rs:23-37): n % 32 == 0; q[n], d[n/32] */
void po_q8_32(const float *x, size_t n, int8_t *q, float *d);
/* the same with every block scale rounded through f16 (PM_AQ_Q8_32_F16; no reference code) */
void po_q8_32_f16(const float *x, size_t n, int8_t *q, float *d);

/* ---- rows -------------------------------------------------------------- */
/* `row_scalar` (src/ds4_cpu.rs:59-83) */
float po_row_q4k(const uint8_t *w, size_t ncols, const int8_t *q, const float *d,
                 const int32_t *bsum);
/* the same sums with AVX-512 VNNI integer dots but `row_scalar`'s float tail:
 * bit-identical to po_row_q4k (falls back to it without AVX-512 VNNI) */
float po_row_q4k_fast(const uint8_t *w, size_t ncols, const int8_t *q, const float *d,
                      const int32_t *bsum);
/* `row_vnni` (src/ds4_cpu.rs:87-118): lane-wise float accumulation; equals the
 * scalar row within 1e-3 (the reference's own tolerance, src/ds4_cpu.rs:468).
 * returns NaN without AVX-512 VNNI */
float po_row_q4k_vnni(const uint8_t *w, size_t ncols, const int8_t *q, const float *d,
                      const int32_t *bsum);
/* `q4k_rows_multi` (src/ds4_cpu.rs:248-271) over `row_vnni_multi` (:205-244):
 * out[r*nt + t]; xs given as arrays of pointers */
void po_q4k_rows_multi(const uint8_t *w, size_t nrows, size_t ncols, int nt,
                       const int8_t *const *q, const float *const *d,
                       const int32_t *const *bsum, float *out, int canonical);
/* Q6_K row against Q8x activations. No reference code pairs these; restated by
 * analogy with row_scalar: per block isum = sum_k sc[k] * sum_{16} (q6-32)*xq,
 * total += x.d[b] * (d * isum). PARITY UNPINNED. */
float po_row_q6k(const uint8_t *w, size_t ncols, const int8_t *q, const float *d);
/* bit-identical to po_row_q6k (AVX-512 VNNI integer sums, same float tail) */
float po_row_q6k_fast(const uint8_t *w, size_t ncols, const int8_t *q, const float *d);
/* Q8_0 row against 32-block activations (src/q4x_cpu.rs:85-90) */
float po_row_q8_0(const uint8_t *w, size_t ncols, const int8_t *q, const float *d32);
/* Q4_K row against 32-block Q8 activations (no reference code pairs them: row_scalar,
 * src/ds4_cpu.rs:59-83, restated with one activation scale per 32-value sub-block) */
float po_row_q4k_q8_32(const uint8_t *w, size_t ncols, const int8_t *q, const float *d32);
/* IQ4_NL row against 32-block activations (src/q4x_cpu.rs:92-101) */
float po_row_iq4nl(const uint8_t *w, size_t ncols, const int8_t *q, const float *d32);
/* IQ4_XS row against 32-block activations (src/q4x_cpu.rs:102-117) */
float po_row_iq4xs(const uint8_t *w, size_t ncols, const int8_t *q, const float *d32);
/* a row of the int4 container (groups of 64, f32 scales) against f32 activations
 * (`dot_q4_scalar`, src/quant.rs:464-476) */
float po_row_glm_q4(const uint8_t *q, const uint8_t *scales, size_t ncols, const float *x);
/* IQ3_S row against 32-block activations (src/q4x_cpu.rs:118-127) */
float po_row_iq3s(const uint8_t *w, size_t ncols, const int8_t *q, const float *d32);
/* any decodable type against f32 activations (src/oss_batch.rs:774-789 for
 * MXFP4): per block s = sum_i w_i * x_i in value order, total += s (block order);
 * for MXFP4 the block scale multiplies the block's sum as the shader does. */
float po_row_f32(int ggml_type, const uint8_t *w, size_t ncols, const float *x);

/* ---- routing ----------------------------------------------------------- */
/* logits[t*E+e] = dot_f32(Wr[e], x[t]) (+ logit_bias[e]) */
void po_router_logits(const float *wr, const float *logit_bias, const float *x, int T, int E,
                      int d, float *logits);
/* ids[T*k] in descending score order (ties -> lower index), w[T*k].
 * select_bias may be NULL. Returns 0, or PM_ERR_INVALID. */
int po_route(const pm_layer_desc *desc, const float *logits, const float *select_bias, int T,
             uint32_t *ids, float *w);

/* ---- plan -------------------------------------------------------------- */
/* arrays sized as in pm_plan_out; returns n_active */
int po_plan(const uint32_t *ids, int T, int K, int E, uint32_t *active, uint32_t *offset,
            uint32_t *count, uint32_t *pair_token, uint32_t *pair_pos);

/* ---- expert / layer ---------------------------------------------------- */
typedef struct po_expert_w {
  const uint8_t *gate, *up, *down;          /* raw GGUF blocks */
  const float *bias_gate, *bias_up, *bias_down; /* or NULL */
} po_expert_w;

typedef struct po_layer {
  pm_layer_desc desc;
  const float *router;        /* [E][d] f32 */
  const float *logit_bias;    /* [E] or NULL */
  const float *select_bias;   /* [E] or NULL */
  const po_expert_w *experts; /* [E] (entries of non-local experts unused) */
  po_expert_w shared;         /* used when desc.shared != NONE */
  const float *shared_gate_inp; /* [d] or NULL */
} po_layer;

/* one expert over nt tokens: xs[t] points at token t's f32 activation [d];
 * wts[t] its routing weight; out[nt][d]. Follows `ds4_cpu::expert`
 * (src/ds4_cpu.rs:297-328) for PM_AQ_Q8X_256 and the f32 shader arithmetic
 * (src/moe_kernels.rs:1183, src/oss_batch.rs:785,89) for PM_AQ_F32.
 * With PM_FOLD_IN_COMBINE the weight is NOT applied here. */
int po_expert(const pm_layer_desc *desc, const po_expert_w *w, int ff, const float *const *xs,
              const float *wts, int nt, float *out);
/* pair_out[P][d] in plan order */
int po_experts(const po_layer *L, const float *x, int T, const uint32_t *ids, const float *w,
               float *pair_out);
/* `combine` (src/moe_kernels.rs:1798-1808): fixed k order, then shared */
void po_combine(const pm_layer_desc *desc, const float *pair_out, const uint32_t *pair_pos,
                const float *w, const float *shared_out, const float *shared_gate_logit,
                int T, float *y, int accumulate);
/* the whole layer; y[T][d]. threads > 1 runs experts side by side (OpenMP). */
int po_moe_forward(const po_layer *L, const float *x, int T, float *y, int accumulate,
                   int threads);
/* x <- x + moe_l(rmsnorm(x)) over n layers (unit norm weight) */
int po_stack_forward(const po_layer *layers, int n_layers, float eps, const float *x, int T,
                     float *x_out, int threads);
void po_rmsnorm(const float *x, int d, float eps, float *out);

/* ---- the reference's fast CPU path, for timing (the CPU baseline) ------- */
/* `cpu_experts` + `ds4_cpu::expert` (src/ds4.rs:1766-1822, src/ds4_cpu.rs:297-328)
 * as the reference threads it: 64-row chunks over all threads, row_vnni_multi
 * 16 tokens per pass; experts side by side when there are several. Q4_K gate/up;
 * Q4_K or Q6_K down. Numerics: lane-wise float sums (reference SIMD order). */
int po_moe_forward_fast(const po_layer *L, const float *x, int T, float *y, int threads);
int po_have_vnni(void);
int po_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
