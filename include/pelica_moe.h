/* pelica_moe.h - C ABI of the B200 (sm_100a) mixture-of-experts FFN path.
 *
 * This is the boundary a Pelica engine binds instead of its own expert code.
 * Pelica (Rust + WGSL) has no FFI for this path; the functions below replace
 * its four in-process seams, cited per entry point as "replaces: file:line"
 * (paths inside the Pelica source tree).
 *
 * Conventions
 *  - Every function returns int32_t: 0 = PM_OK, negative = PM_ERR_*. Nothing
 *    throws or aborts across the boundary. pm_last_error() gives a
 *    thread-local, human-readable string for the last failure.
 *  - Host pointers belong to the caller and are only read/written during the
 *    call. Weight bytes are copied (and re-laid out) at upload, so the caller
 *    may free or unmap them afterwards, as Pelica drops its `Pin` after upload
 *    (src/ds4.rs:1749).
 *  - `x`, `y`, ids, weights ... may be host or device pointers; the library
 *    asks the CUDA runtime which. Host buffers are staged through the
 *    context's pinned staging area.
 *  - One pm_ctx per GPU, used by one host thread at a time. All work is
 *    ordered on the context's stream; calls that return results into host
 *    memory synchronise, calls on device pointers do not (use pm_sync).
 *  - There is no CPU fallback: without a CUDA device pm_ctx_create fails.
 */
#ifndef PELICA_MOE_H
#define PELICA_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PM_API __attribute__((visibility("default")))

/* ---- error codes ------------------------------------------------------ */
enum {
  PM_OK = 0,
  PM_ERR_INVALID = -1,     /* bad argument / shape the path does not take   */
  PM_ERR_UNSUPPORTED = -2, /* a type or mode that is not built              */
  PM_ERR_CUDA = -3,        /* a CUDA runtime call failed (see last error)   */
  PM_ERR_OOM = -4,         /* device or pinned allocation failed            */
  PM_ERR_STATE = -5,       /* weights missing, layer not finalised ...      */
  PM_ERR_TIMEOUT = -6,     /* a bounded device-side wait gave up            */
  PM_ERR_LIMIT = -7,       /* a size beyond a documented fixed maximum      */
  PM_ERR_COMM = -8         /* the collective library is missing or reported an error */
};

/* ---- ggml tensor type ids (src/gguf.rs:85-121) ------------------------- */
enum {
  PM_TYPE_F32 = 0,
  PM_TYPE_F16 = 1,
  PM_TYPE_Q8_0 = 8,   /* 32 values / 34 B  */
  PM_TYPE_Q4_K = 12,  /* 256 values / 144 B */
  PM_TYPE_Q5_K = 13,  /* 256 values / 176 B: Q4_K's header, 32 B of fifth bits, 128 B of nibbles
                         (src/moe_kernels.rs:74); f32 activations only, as in the reference */
  PM_TYPE_Q6_K = 14,  /* 256 values / 210 B */
  PM_TYPE_IQ4_NL = 20, /* 32 values / 18 B: f16 d + 16 B of 4-bit indices into a fixed
                          non-linear codebook (src/iq_tables.rs:72, src/q4x_cpu.rs:92-101) */
  PM_TYPE_IQ3_S = 21,  /* 256 values / 110 B: f16 d, 8-bit + 1-bit indices into a 512-entry codebook of
                          four magnitudes, sign bits, 4-bit sub-scales 1 + 2 s (src/iq_tables.rs:4,
                          src/q4x_cpu.rs:64-82,118-127) */
  PM_TYPE_IQ4_XS = 23, /* 256 values / 136 B: f16 d, 8 six-bit sub-scales (bias 32), indices into
                          the IQ4_NL codebook (src/q4x_cpu.rs:102-117,462-476) */
  PM_TYPE_BF16 = 30,
  PM_TYPE_MXFP4 = 39, /* 32 values / 17 B  */
  /* not a ggml id: the reference's own int4 container (src/quant.rs:9-11, src/gpu.rs:70-117). A
     [rows][cols] matrix is rows * cols / 2 bytes of nibbles (value c in byte c / 2, low nibble
     first, stored as level + 8) followed by rows * cols / 64 f32 scales, one per group of 64
     columns; value = (nibble - 8) * scale. f32 activations. (The container's table-indexed
     scales, `Q4T`, hold the same values: expand them to f32 before the upload.) */
  PM_TYPE_GLM_Q4 = 1064
};

/* ---- router gating (src/moe_kernels.rs:1019-1081, src/oss_kernels.rs:15-35,
 *      src/ds4.rs:1371-1426, src/q4x.rs:2213-2231, src/forward.rs:488-504) - */
enum {
  PM_GATE_SOFTMAX_ALL = 0,      /* softmax over all experts, select on p(+bias) */
  PM_GATE_SIGMOID = 1,          /* sigmoid scores, select on s(+bias)           */
  PM_GATE_SQRT_SOFTPLUS = 2,    /* sqrt(softplus(v)), select on s(+bias)        */
  PM_GATE_SOFTMAX_SELECTED = 3  /* top-k by logit, softmax over the selected    */
};

/* ---- expert activation (src/moe_kernels.rs:1183, src/ds4_cpu.rs:311,
 *      src/oss_batch.rs:785) ----------------------------------------------- */
enum {
  PM_ACT_SILU = 0,       /* h = g/(1+exp(-g)) * u                                  */
  PM_ACT_SILU_CLAMP = 1, /* g=min(g,lim); u=clamp(u,-lim,lim) first (lim>0)        */
  PM_ACT_OSS_GLU = 2     /* x=min(g+bg,lim); y=clamp(u+bu,-lim,lim);
                            h = x/(1+exp(-alpha*x))*(y+1)                           */
};

/* ---- activation arithmetic ------------------------------------------------ */
enum {
  PM_AQ_F32 = 0,      /* f32 activations x dequantised weights (src/oss_batch.rs:767-877) */
  PM_AQ_Q8X_256 = 1,  /* int8 per 256 values, f32 scale, 8 partial sums
                         (`Q8x`, src/ds4_cpu.rs:7-36); the hidden vector is
                         re-quantised before down (src/ds4_cpu.rs:306-317)        */
  PM_AQ_Q8_32 = 2,    /* int8 per 32 values, f32 scale (`Q8`, src/q4x_cpu.rs:13-51)
                         against Q8_0 / IQ4_NL / IQ4_XS / IQ3_S weights: per block f16(d_w) * x.d * idot
                         (src/q4x_cpu.rs:85-101); hidden vector re-quantised the
                         same way before down (src/q4x_cpu.rs:399-440)            */
  PM_AQ_Q8_32_F16 = 3 /* the same quantiser with the block scale rounded through f16 (a ggml Q8_0
                         block's scale), for the 32-block types and, as a second mode that no
                         reference code has, for Q4_K weights: per 32-value sub-block j of a
                         super-block x.d[j] * ((d * sc_j) * isum_j - (dmin * m_j) * bsum_j),
                         sub-blocks in ascending order. The reference pairs Q4_K with
                         PM_AQ_Q8X_256 only (src/ds4_cpu.rs:59-83).                */
};

/* ---- where the routing weight is applied ------------------------------- */
enum {
  PM_FOLD_BEFORE_DOWN = 0, /* h *= w_t before down (src/ds4_cpu.rs:312)             */
  PM_FOLD_IN_COMBINE = 1   /* y += w * down(h) (src/moe_kernels.rs:1798-1802);
                              with expert biases: w*(down+bias) (src/oss_batch.rs:89) */
};

enum { PM_SHARED_NONE = 0, PM_SHARED_PLAIN = 1, PM_SHARED_SIGMOID_GATED = 2 };

/* fixed maxima of the path (the reference: NEMAX 512, KMAX 8,
 * src/moe_kernels.rs:16-20; q4x routes up to 16) */
#define PM_MAX_EXPERTS 512
#define PM_MAX_TOPK 16
#define PM_MAX_TOKENS 16384
#define PM_MAX_D 49152       /* model width: a token's f32 row must fit one SM's shared memory */

/* One MoE FFN layer. Plain data; copy freely. */
typedef struct pm_layer_desc {
  int32_t d;            /* hidden size                                      */
  int32_t ff;           /* expert intermediate size                         */
  int32_t n_exp;        /* routed experts in the model                      */
  int32_t top_k;
  int32_t gating;       /* PM_GATE_*                                        */
  int32_t norm_w;       /* 1: w /= max(sum_k w, 2^-14) (src/moe_kernels.rs:1073) */
  float w_scale;        /* 0 = none; else w *= w_scale                      */
  int32_t n_group;      /* 0 = off; group-limited selection                 */
  int32_t topk_group;
  int32_t act;          /* PM_ACT_*                                         */
  float act_limit;      /* lim (0 = no clamp)                               */
  float act_alpha;      /* OSS_GLU alpha (1.702)                            */
  int32_t type_gate, type_up, type_down; /* PM_TYPE_*                       */
  int32_t act_quant;    /* PM_AQ_*                                          */
  int32_t weight_fold;  /* PM_FOLD_*                                        */
  int32_t has_expert_bias; /* f32 bias per gate/up/down row (gpt-oss)       */
  int32_t shared;       /* PM_SHARED_*                                      */
  int32_t shared_ff;    /* intermediate size of the shared expert           */
  int32_t first_local_expert; /* expert parallelism: this context holds     */
  int32_t n_exp_local;        /* experts [first, first+n_local); 0 = all    */
} pm_layer_desc;

/* Dispatch plan of one call (src/moe_kernels.rs:24-34,1086-1129 layout;
 * token lists in ascending token order as src/ds4.rs:1461-1472).
 * All arrays are caller-allocated (host or device):
 *   active[n_exp], offset[n_exp], count[n_exp], pair_token[T*k], pair_pos[T*k] */
typedef struct pm_plan_out {
  int32_t *n_active;     /* [1]  experts with >= 1 pair                     */
  uint32_t *active;      /* expert ids, ascending                           */
  uint32_t *offset;      /* exclusive prefix sum of count                   */
  uint32_t *count;
  uint32_t *pair_token;  /* token of pair p; per expert ascending token     */
  uint32_t *pair_pos;    /* pair of (t,k) = pair_pos[t*k_top + k]           */
} pm_plan_out;

typedef struct pm_ctx pm_ctx;
typedef struct pm_layer pm_layer;
typedef struct pm_stack pm_stack;
typedef struct pm_ep pm_ep;

/* ---- library ----------------------------------------------------------- */
PM_API const char *pm_last_error(void);
PM_API const char *pm_version(void);
/* bytes per block / values per block of a ggml type (src/gguf.rs:85-121);
 * returns 0 for a type this path does not decode */
PM_API size_t pm_type_block_bytes(int32_t ggml_type);
PM_API size_t pm_type_block_values(int32_t ggml_type);

/* ---- context ----------------------------------------------------------- */
/* replaces: wgpu device + queue per engine (src/moe.rs:786, src/ds4_gpu.rs:568) */
PM_API int32_t pm_ctx_create(int32_t device, pm_ctx **out);
/* the same, ordered on a stream the caller owns (cudaStream_t; NULL = the legacy
 * default stream), e.g. the stream its NCCL collectives are queued on */
PM_API int32_t pm_ctx_create_on_stream(int32_t device, void *stream, pm_ctx **out);
PM_API int32_t pm_ctx_destroy(pm_ctx *ctx);
/* replaces: Pending::wait (src/ds4_gpu.rs:733) */
PM_API int32_t pm_sync(pm_ctx *ctx);
/* expert products run on the tensor cores (tcgen05 int8, exact integer sums) when a
 * call has at least this many tokens (default 32, the reference's TC_MIN,
 * src/moe.rs:35; 0 = never). Both paths give the same bits. */
PM_API int32_t pm_ctx_set_tensor_core_min_tokens(pm_ctx *ctx, int32_t min_tokens);
/* the CUDA stream all work of this context is ordered on (cudaStream_t) */
PM_API void *pm_ctx_stream(pm_ctx *ctx);
/* pinned host memory for activations that cross the bus every call */
PM_API int32_t pm_host_alloc(pm_ctx *ctx, size_t bytes, void **out);
PM_API int32_t pm_host_free(pm_ctx *ctx, void *p);
/* device memory helpers for callers that keep activations resident */
PM_API int32_t pm_dev_alloc(pm_ctx *ctx, size_t bytes, void **out);
PM_API int32_t pm_dev_free(pm_ctx *ctx, void *p);
PM_API int32_t pm_copy(pm_ctx *ctx, void *dst, const void *src, size_t bytes);

/* ---- layer ------------------------------------------------------------- */
/* replaces: the per-layer FFN block of the recorded op list (src/moe.rs:1377-1437)
 * and the layer tensors of src/ds4.rs / src/oss.rs:521-527 */
PM_API int32_t pm_layer_create(pm_ctx *ctx, const pm_layer_desc *desc, pm_layer **out);
PM_API int32_t pm_layer_destroy(pm_layer *layer);
/* router weight [n_exp][d] (f32, or bf16 when dtype == PM_TYPE_BF16);
 * logit_bias [n_exp] is added before top-k (gpt-oss, src/oss_batch.rs:478);
 * select_bias [n_exp] only ranks (exp_probs_b, src/moe_kernels.rs:1047);
 * either may be NULL */
PM_API int32_t pm_layer_set_router(pm_layer *layer, const void *w, int32_t dtype,
                                   const float *logit_bias, const float *select_bias);
/* raw GGUF block bytes, row-major: gate/up [ff][d], down [d][ff]
 * (`Pin::piece(0..2)`, src/ds4_io.rs:220-234); biases f32 or NULL.
 * `e` is the global expert id; must be local to this context. */
PM_API int32_t pm_layer_set_expert(pm_layer *layer, int32_t e, const uint8_t *gate,
                                   const uint8_t *up, const uint8_t *down, const float *bias_gate,
                                   const float *bias_up, const float *bias_down);
/* shared expert (src/moe.rs:1422-1434): same types as the routed experts;
 * gate_inp [d] f32 is the scalar sigmoid gate (src/moe_kernels.rs:1805) or NULL */
PM_API int32_t pm_layer_set_shared(pm_layer *layer, const uint8_t *gate, const uint8_t *up,
                                   const uint8_t *down, const float *gate_inp);
/* usage[e] += pairs routed to e on every forward (src/moe_kernels.rs:1114);
 * out[n_exp] host */
PM_API int32_t pm_layer_read_usage(pm_layer *layer, uint32_t *out);

/* ---- the operator ------------------------------------------------------ */
/* y[T][d] = sum_k w[t,k] * expert_{id[t,k]}(x[t]) (+ shared(x[t])).
 * x is the normed activation the engines hand to their FFN (src/moe.rs:1367).
 * flags: PM_FWD_ACCUMULATE adds into y (the residual, src/moe_kernels.rs:1808).
 * replaces: src/moe.rs:1377-1437, ds4 `ffn` src/ds4.rs:1428-1763,
 *           `Model::moe` src/forward.rs:481-753 */
#define PM_FWD_ACCUMULATE 1u
PM_API int32_t pm_moe_forward(pm_layer *layer, const float *x, int32_t T, float *y,
                              uint32_t flags);

/* split entry points (parity tests; callers that own part of the pipeline) */
/* logits[T][n_exp] = W_r x (+ logit bias); replaces `matvec` src/moe_kernels.rs:140,
 * `cpu::dot` loop src/ds4.rs:1376-1383 */
PM_API int32_t pm_router_logits(pm_layer *layer, const float *x, int32_t T, float *logits);
/* ids[T][k] (descending score), w[T][k]; replaces `plan` head
 * src/moe_kernels.rs:1019-1081, `TOPK` src/oss_kernels.rs:15-35 */
PM_API int32_t pm_route(pm_layer *layer, const float *x, int32_t T, uint32_t *ids, float *w);
PM_API int32_t pm_route_logits(pm_layer *layer, const float *logits, int32_t T, uint32_t *ids,
                               float *w);
/* pm_route for callers that must not allocate. No counterpart in the reference.
 * Some hosts cannot let a library call cudaMalloc in the middle of their run:
 * an engine that has handed all device memory to its own pool, a serving loop
 * where the implicit device synchronisation of an allocation is a latency
 * spike, a process under a hard memory budget. pm_route may grow the context's
 * workspace on such a call; this variant never does. Its only scratch (the
 * router logits) is a fixed array inside the library, sized for at most
 * PM_ROUTE_NOALLOC_MAX_TOKENS tokens x PM_MAX_EXPERTS experts (512 KB on every
 * GPU that loads the library, held until exit); larger T is refused with
 * PM_ERR_LIMIT. x [T][d], ids [T][k], w [T][k] must already be DEVICE pointers.
 * Work is queued on the context's stream and not waited for. The first call on
 * a GPU looks up the array's device address; make that first call before any
 * stream capture. All calls share the one array: two calls whose kernels can
 * overlap on the GPU (different contexts of one device) race on it - order them.
 * Nothing in it needs clearing: every logit read is written earlier in the same
 * call. Results are the bits pm_route gives. */
#define PM_ROUTE_NOALLOC_MAX_TOKENS 256
PM_API int32_t pm_route_noalloc(pm_layer *layer, const float *x, int32_t T, uint32_t *ids,
                                float *w);
/* replaces: `plan` tail src/moe_kernels.rs:1083-1129, rows[e] src/ds4.rs:1461-1472 */
PM_API int32_t pm_plan(pm_layer *layer, const uint32_t *ids, int32_t T, pm_plan_out *out);
/* pair_out[P][d]: expert outputs per pair in plan order (weights folded when
 * the layer says BEFORE_DOWN); replaces `ds4_cpu::expert` src/ds4_cpu.rs:297-328,
 * `expert`/`expert_dec` src/moe_kernels.rs:1170,1423 */
PM_API int32_t pm_experts(pm_layer *layer, const float *x, int32_t T, const uint32_t *ids,
                          const float *w, float *pair_out);
/* expert parallelism, the serving side: row r of x [R][d] goes through expert
 * eids[r] (which must be local to this context) with routing weight w[r];
 * out[R][d] in row order, the same values pm_experts gives for that pair.
 * replaces: the device side of the bridge RUN op, src/bridge.rs:412-466 */
PM_API int32_t pm_experts_rows(pm_layer *layer, const float *x, int32_t R, const uint32_t *eids,
                               const float *w, float *out);
/* the shared expert alone (times its sigmoid gate, if any), out[T][d];
 * replaces: the dense MLP ops src/moe.rs:1422-1434 */
PM_API int32_t pm_shared(pm_layer *layer, const float *x, int32_t T, float *out);
/* y from pair outputs; replaces `combine` src/moe_kernels.rs:1787-1813 */
PM_API int32_t pm_combine(pm_layer *layer, const float *pair_out, const uint32_t *ids,
                          const float *w, const float *shared_out, int32_t T, float *y,
                          uint32_t flags);

/* ---- expert parallelism: experts sharded over the GPUs of a node ----------------------
 * replaces: the bridge, Pelica's only expert-offload mechanism: `RUN` sends activations and
 * per-expert (token, weight) rows to the machine that holds the experts and gets the summed
 * outputs back (src/bridge.rs:412-466, host side `Remote::start/finish/fail`
 * src/bridge.rs:730-786, callers src/ds4.rs:1527-1552,1695-1713). Here the transport is NCCL
 * (grouped ncclSend/ncclRecv on the context's stream, NVLink/NVSwitch), one rank per GPU:
 * expert e lives on rank e / (n_exp / world); router, selection bias and shared expert are
 * replicated; tokens are data-parallel. NCCL is bound at run time (dlopen of libnccl.so.2).
 * Failure behaviour: a missing library or a failed NCCL call is PM_ERR_COMM (also the
 * asynchronous errors NCCL reports, polled by every call); a rank that never enters the call
 * shows as PM_ERR_TIMEOUT on the others after pm_ep_set_timeout_ms (default 60 s), as the
 * bridge's callers fall back when a link fails (src/ds4.rs:1706-1710). */
/* 128 bytes identifying a new communicator: rank 0 calls this and hands the bytes to the other
 * ranks by its own means (a file, a socket, its launcher) */
PM_API int32_t pm_ep_unique_id(uint8_t *out128);
/* collective: every rank calls it with the same id; the context's GPU joins the communicator */
PM_API int32_t pm_ep_init(pm_ctx *ctx, const uint8_t *unique_id128, int32_t rank, int32_t world, pm_ep **out);
PM_API int32_t pm_ep_destroy(pm_ep *ep);
PM_API int32_t pm_ep_set_timeout_ms(pm_ep *ep, int64_t ms);
/* collective: y[T][d] = the layer's output for this rank's T tokens (x, y device pointers; T may
 * differ per rank and may be 0). The layer must have been created with first_local_expert =
 * rank * n_exp / world and n_exp_local = n_exp / world. Same values as pm_moe_forward on a
 * layer that holds every expert. Work is queued on the context's stream; the call waits on the
 * host once, for the ranks' pair counts. flags: PM_FWD_ACCUMULATE. */
PM_API int32_t pm_moe_forward_ep(pm_ep *ep, pm_layer *layer, const float *x, int32_t T, float *y, uint32_t flags);
/* the last call's traffic: out[4] = rows sent, rows received, bytes sent, bytes received
 * (to and from other ranks; rows that stay on the rank are not counted) */
PM_API int32_t pm_ep_last_stats(pm_ep *ep, uint64_t *out);

/* ---- usage-driven placement of experts over the ranks ------------------
 * replaces: `Adapt` / `adapt` / `swap_round` (src/moe.rs:246-278,1965-2069): a decayed use score per
 * (layer, expert) from the plan's counters; the experts used more than the least used resident ones
 * change places with them, biggest gains first, up to a byte budget a round, with a margin against
 * going back and forth; a slot table says where each expert sits. The reference's places are VRAM and
 * host memory; here they are the ranks of an expert-parallel group: slot s is held by rank
 * s / (n_exp / world), and a round evens out the scores the ranks serve. */
typedef struct pm_placement pm_placement;
/* host-side planner (no GPU work) */
PM_API int32_t pm_placement_create(int32_t n_layers, int32_t n_exp, int32_t world, pm_placement **out);
PM_API int32_t pm_placement_destroy(pm_placement *p);
/* usage[n_exp]: the layer's cumulative counters (pm_layer_usage); score = score * 0.944 + the increase
 * since the last observation (src/moe.rs:273,1977-1980) */
PM_API int32_t pm_placement_observe(pm_placement *p, int32_t layer, const uint32_t *usage);
/* One round: swaps[3 * i] = (layer, hot expert, cold expert), at most max_swaps and at most
 * budget_bytes moved (2 * expert_bytes a swap); a swap must clear the reference's margin
 * (hot >= cold * 1.25 + 1.5, src/moe.rs:2013) and lower the load of the heavier rank. The planner's
 * table is updated as if the swaps were done: carry them out in the order returned. */
PM_API int32_t pm_placement_plan(pm_placement *p, uint64_t expert_bytes, uint64_t budget_bytes, int32_t *swaps,
                                 int32_t max_swaps, int32_t *n_swaps);
PM_API int32_t pm_placement_slots(const pm_placement *p, int32_t layer, int32_t *slot_of_expert);
/* score[n_exp] and / or rank_load[world] (sum of the scores of the experts a rank holds); either may be null */
PM_API int32_t pm_placement_scores(const pm_placement *p, int32_t layer, float *score, float *rank_load);
/* The layer's slot table on an expert-parallel group (`loc`, src/moe.rs:262-263,2065): after routing,
 * expert ids are mapped through it, and everything downstream - plan, destination rank, the serving
 * rank's planes - names slots. The weights must already sit in the slots the table says
 * (pm_layer_set_expert takes the slot index then). Null: expert e in slot e again. The usage counters
 * keep counting by expert id. */
PM_API int32_t pm_ep_set_slots(pm_ep *ep, pm_layer *layer, const int32_t *slot_of_expert);
PM_API int32_t pm_ep_get_slots(pm_ep *ep, pm_layer *layer, int32_t *slot_of_expert);
/* Collective: experts a and b change places - the ranks that hold them exchange the experts' bytes
 * (grouped ncclSend / ncclRecv through a staging area; device copies when one rank holds both) and
 * every rank rewrites its table. Every rank calls it with the same arguments in the same order, between
 * forward calls. */
PM_API int32_t pm_ep_swap_experts(pm_ep *ep, pm_layer *layer, int32_t expert_a, int32_t expert_b);

/* ---- format checks (bit-exact against the reference arithmetic) -------- */
/* replaces: `deq4` src/moe_kernels.rs:63-84, `deq_row` src/q4x_cpu.rs:443-496 */
PM_API int32_t pm_dequant(pm_ctx *ctx, int32_t ggml_type, const uint8_t *blocks,
                          size_t n_values, float *out);
/* replaces: `Q8x::new` src/ds4_cpu.rs:13-35 (mode PM_AQ_Q8X_256; n % 256 == 0;
 * q[n], scale[n/256], bsum[n/32]) and `Q8::new` src/q4x_cpu.rs:23-37 (mode
 * PM_AQ_Q8_32; n % 32 == 0; q[n], scale[n/32]; bsum unused, may be null) */
PM_API int32_t pm_quant_act(pm_ctx *ctx, int32_t mode, const float *x, size_t n, int8_t *q,
                            float *scale, int32_t *bsum);

/* ---- layer stacks (the benchmark's unit: x <- x + moe(rmsnorm(x)) per layer) */
/* the engines' layer loop around the FFN (src/moe.rs:1279-1440 `after` ops:
 * rmsnorm, FFN, residual add) reduced to its MoE part */
/* out[T][d] = x / rms(x) (unit norm weight), the norm pm_stack_forward applies */
PM_API int32_t pm_rmsnorm(pm_ctx *ctx, const float *x, int32_t T, int32_t d, float eps, float *out);
PM_API int32_t pm_stack_create(pm_ctx *ctx, pm_layer **layers, int32_t n_layers, float eps,
                               pm_stack **out);
PM_API int32_t pm_stack_destroy(pm_stack *stack);
/* x[T][d] in, x_out[T][d] out (may alias); every layer: xn = x/rms(x) (unit
 * norm weight), x += moe(xn) */
PM_API int32_t pm_stack_forward(pm_stack *stack, const float *x, int32_t T, float *x_out);
/* mode 0 (default): one-token calls run in the persistent decode kernel when
 * the stack's shape allows it; mode 1: the general kernels always. Both give
 * the same bits. With device pointers a failed bounded wait of the decode
 * kernel is reported by pm_stack_status. A layer whose weights are (re)loaded after the stack
 * was created is picked up by the next pm_stack_forward. */
PM_API int32_t pm_stack_set_mode(pm_stack *stack, int32_t mode);
PM_API int32_t pm_stack_decode_kernel_available(pm_stack *stack);
/* PM_OK, or PM_ERR_TIMEOUT when a device-side wait of an earlier call gave up
 * (synchronises the context's stream) */
PM_API int32_t pm_stack_status(pm_stack *stack);
/* ---- synthetic weights generated on the device (benchmark set-up) ------ */
/* fills every expert (and the router, biases, shared expert) of `layer` with
 * N(0, sigma) weights quantised to the layer's types by on-device encoders;
 * deterministic in (seed, expert, tensor, element). A router logit bias /
 * selection bias is generated when its sigma is > 0. */
PM_API int32_t pm_layer_fill_synthetic(pm_layer *layer, uint64_t seed, float sigma,
                                       float logit_bias_sigma, float select_bias_sigma);
/* raw GGUF-format bytes of one expert tensor as stored by the library,
 * converted back from its device layout (which = 0 gate, 1 up, 2 down);
 * `out` host, sized rows*cols/block_values*block_bytes */
PM_API int32_t pm_layer_get_expert(pm_layer *layer, int32_t e, int32_t which, uint8_t *out);
PM_API int32_t pm_layer_get_router(pm_layer *layer, float *w, float *logit_bias,
                                   float *select_bias);
/* f32 biases of expert e (NULL entries are skipped); layers with has_expert_bias */
PM_API int32_t pm_layer_get_expert_bias(pm_layer *layer, int32_t e, float *bias_gate,
                                        float *bias_up, float *bias_down);

#ifdef __cplusplus
}
#endif
#endif /* PELICA_MOE_H */
