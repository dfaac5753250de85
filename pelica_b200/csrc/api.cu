// api.cu - the C ABI (include/pelica_moe.h): contexts, layers, the operator
// and its split entry points, layer stacks, synthetic fill.
//
// Host orchestration only; every computation is a kernel of this library.
// There is no CPU fallback: without a CUDA device pm_ctx_create fails.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <map>
#include <vector>

#include "decode_mega.cuh"
#include "../../include/pelica_moe_diag.h"

void launch_synth_blocks(const Launch &L, int type, uint8_t *raw, size_t nb, uint64_t seed,
                         float sigma);
void launch_synth_f32(const Launch &L, float *out, size_t n, uint64_t seed, float sigma,
                      int bf16_round);

// ---------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------
static thread_local char g_err[512] = "";

static int32_t fail(int32_t code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
  return code;
}

#define CU(call)                                                                       \
  do {                                                                                 \
    cudaError_t e_ = (call);                                                           \
    if (e_ != cudaSuccess)                                                             \
      return fail(e_ == cudaErrorMemoryAllocation ? PM_ERR_OOM : PM_ERR_CUDA,          \
                  "%s: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
  } while (0)
#define TRY(call)            \
  do {                       \
    int32_t r_ = (call);     \
    if (r_ != PM_OK) return r_; \
  } while (0)

extern "C" const char *pm_last_error(void) { return g_err; }
extern "C" const char *pm_version(void) { return "pelica-moe-b200 0.1 (sm_100a)"; }

extern "C" size_t pm_type_block_bytes(int32_t t) {
  switch (t) {
    case PM_TYPE_Q8_0: return 34;
    case PM_TYPE_IQ4_NL: return 18;
    case PM_TYPE_IQ4_XS: return 136;
    case PM_TYPE_Q4_K: return 144;
    case PM_TYPE_Q5_K: return 176;
    case PM_TYPE_Q6_K: return 210;
    case PM_TYPE_IQ3_S: return 110;
    case PM_TYPE_MXFP4: return 17;
    case PM_TYPE_GLM_Q4: return 36;  // 32 bytes of nibbles + the group's f32 scale (kept in a region of their own)
  }
  return 0;
}
extern "C" size_t pm_type_block_values(int32_t t) {
  switch (t) {
    case PM_TYPE_Q8_0:
    case PM_TYPE_IQ4_NL:
    case PM_TYPE_MXFP4: return 32;
    case PM_TYPE_GLM_Q4: return 64;
    case PM_TYPE_Q4_K:
    case PM_TYPE_Q5_K:
    case PM_TYPE_IQ4_XS:
    case PM_TYPE_IQ3_S:
    case PM_TYPE_Q6_K: return 256;
  }
  return 0;
}
static size_t raw_bytes(int type, size_t rows, size_t cols) {
  return rows * (cols / pm_type_block_values(type)) * pm_type_block_bytes(type);
}

// ---------------------------------------------------------------------------
// context
// ---------------------------------------------------------------------------
struct pm_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = true;
  int *dev_err = nullptr;   // error word of kernels with bounded waits
  unsigned int *route_ticket = nullptr;  // [1] zero between launches: the few-token routing kernel's last-CTA ticket
  int tc_min_tokens = 32;   // tensor-core expert products from this many tokens (the reference's TC_MIN, src/moe.rs:35); 0 = never
  int64_t launches = 0;
  int64_t path_count[PM_PATH_N] = {0, 0, 0, 0};  // launches per expert-product path (pelica_moe_diag.h)
  unsigned long long wait_ns = 2000000000ull;    // limit of every bounded device-side wait
  int tc_fault_block = -1;                       // test hook: the tensor-core kernel never completes this block
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  // workspace: one region, carved per call
  uint8_t *ws = nullptr;
  size_t ws_cap = 0, ws_off = 0;
  // staging for weight uploads
  uint8_t *stage = nullptr;
  size_t stage_cap = 0;
  void *flush = nullptr;
  size_t flush_bytes = 0;
  // optional per-phase timing (CUDA events on the stream)
  bool prof_on = false;
  std::vector<cudaEvent_t> prof_ev;
  size_t prof_used = 0;
  std::vector<int> prof_phase;  // phase of event pair i
  int n_sm = 148;  // SMs of the device
  Launch launch() { return Launch{stream, &launches, n_sm}; }
};

enum { PH_ROUTER = 0, PH_ROUTE, PH_PLAN, PH_QUANT_X, PH_GATEUP, PH_QUANT_H, PH_DOWN, PH_SHARED,
       PH_COMBINE, PH_NORM, PH_FUSED, PH_N };
static const char *PH_NAMES[PH_N] = {"router", "route", "plan", "quant_x", "gateup", "quant_h",
                                     "down", "shared", "combine", "rmsnorm", "fused"};

struct ProfSpan {
  pm_ctx *c;
  bool on;
  ProfSpan(pm_ctx *ctx, int phase) : c(ctx), on(ctx->prof_on) {
    if (!on) return;
    if (c->prof_used + 2 > c->prof_ev.size()) {
      for (int i = 0; i < 64; i++) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) { on = false; return; }
        c->prof_ev.push_back(e);
      }
    }
    c->prof_phase.push_back(phase);
    cudaEventRecord(c->prof_ev[c->prof_used], c->stream);
  }
  ~ProfSpan() {
    if (!on) return;
    cudaEventRecord(c->prof_ev[c->prof_used + 1], c->stream);
    c->prof_used += 2;
  }
};
#define PROF(c, ph) ProfSpan prof_span_##ph(c, ph)

static bool is_device_ptr(const void *p) {
  if (!p) return false;
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

static int32_t ws_reserve(pm_ctx *c, size_t bytes) {
  c->ws_off = 0;
  if (bytes <= c->ws_cap) return PM_OK;
  CU(cudaStreamSynchronize(c->stream));
  if (c->ws) CU(cudaFree(c->ws));
  c->ws = nullptr;
  c->ws_cap = 0;
  size_t cap = bytes + bytes / 8 + (1 << 20);
  CU(cudaMalloc(&c->ws, cap));
  c->ws_cap = cap;
  return PM_OK;
}
template <typename T>
static T *ws_take(pm_ctx *c, size_t n) {
  size_t off = (c->ws_off + 255) & ~(size_t)255;
  c->ws_off = off + n * sizeof(T);
  return (T *)(c->ws + off);
}
static size_t al(size_t b) { return (b + 255) & ~(size_t)255; }

static int32_t stage_reserve(pm_ctx *c, size_t bytes) {
  if (bytes <= c->stage_cap) return PM_OK;
  CU(cudaStreamSynchronize(c->stream));
  if (c->stage) CU(cudaFree(c->stage));
  c->stage = nullptr;
  c->stage_cap = 0;
  CU(cudaMalloc(&c->stage, bytes));
  c->stage_cap = bytes;
  return PM_OK;
}

extern "C" int32_t pm_ctx_create(int32_t device, pm_ctx **out) {
  if (!out) return fail(PM_ERR_INVALID, "pm_ctx_create: out is null");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return fail(PM_ERR_CUDA, "pm_ctx_create: no CUDA device (%s); this library has no CPU path",
                cudaGetErrorString(e));
  if (device < 0 || device >= n) return fail(PM_ERR_INVALID, "pm_ctx_create: device %d of %d", device, n);
  CU(cudaSetDevice(device));
  pm_ctx *c = new (std::nothrow) pm_ctx();
  if (!c) return fail(PM_ERR_OOM, "pm_ctx_create: host allocation");
  c->device = device;
  CU(cudaDeviceGetAttribute(&c->n_sm, cudaDevAttrMultiProcessorCount, device));
  CU(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
  CU(cudaMalloc(&c->dev_err, 4));
  CU(cudaMemset(c->dev_err, 0, 4));
  CU(cudaMalloc(&c->route_ticket, 4));
  CU(cudaMemset(c->route_ticket, 0, 4));
  CU(cudaEventCreate(&c->ev0));
  CU(cudaEventCreate(&c->ev1));
  *out = c;
  return PM_OK;
}

// a context whose work is ordered on a stream the caller owns (e.g. the stream
// its collectives run on), so no cross-stream synchronisation is needed
extern "C" int32_t pm_ctx_create_on_stream(int32_t device, void *stream, pm_ctx **out) {
  if (!out) return fail(PM_ERR_INVALID, "pm_ctx_create_on_stream: out is null");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return fail(PM_ERR_CUDA, "pm_ctx_create_on_stream: no CUDA device (%s); this library has no CPU path",
                cudaGetErrorString(e));
  if (device < 0 || device >= n) return fail(PM_ERR_INVALID, "device %d of %d", device, n);
  CU(cudaSetDevice(device));
  pm_ctx *c = new (std::nothrow) pm_ctx();
  if (!c) return fail(PM_ERR_OOM, "host allocation");
  c->device = device;
  CU(cudaDeviceGetAttribute(&c->n_sm, cudaDevAttrMultiProcessorCount, device));
  c->stream = (cudaStream_t)stream;
  c->own_stream = false;
  CU(cudaMalloc(&c->dev_err, 4));
  CU(cudaMemset(c->dev_err, 0, 4));
  CU(cudaMalloc(&c->route_ticket, 4));
  CU(cudaMemset(c->route_ticket, 0, 4));
  CU(cudaEventCreate(&c->ev0));
  CU(cudaEventCreate(&c->ev1));
  *out = c;
  return PM_OK;
}

extern "C" int32_t pm_ctx_destroy(pm_ctx *c) {
  if (!c) return PM_OK;
  cudaSetDevice(c->device);
  cudaStreamSynchronize(c->stream);
  if (c->ws) cudaFree(c->ws);
  if (c->stage) cudaFree(c->stage);
  if (c->flush) cudaFree(c->flush);
  if (c->dev_err) cudaFree(c->dev_err);
  if (c->route_ticket) cudaFree(c->route_ticket);
  for (cudaEvent_t e : c->prof_ev) cudaEventDestroy(e);
  cudaEventDestroy(c->ev0);
  cudaEventDestroy(c->ev1);
  if (c->own_stream) cudaStreamDestroy(c->stream);
  delete c;
  return PM_OK;
}

// the error word of kernels with bounded waits (call after a synchronisation)
static int32_t check_dev_err(pm_ctx *c) {
  int e = 0;
  CU(cudaMemcpy(&e, c->dev_err, 4, cudaMemcpyDeviceToHost));
  if (e) {
    CU(cudaMemset(c->dev_err, 0, 4));
    if (e == PM_DEVERR_BAD_EXPERT_ID)
      return fail(PM_ERR_INVALID, "an expert id in a device buffer is outside the layer's experts "
                                  "(its pairs were left out; nothing was read or written out of bounds)");
    return fail(PM_ERR_TIMEOUT, "a bounded device-side wait gave up (code %d)", e);
  }
  return PM_OK;
}
extern "C" int32_t pm_sync(pm_ctx *c) {
  if (!c) return fail(PM_ERR_INVALID, "pm_sync: null context");
  CU(cudaStreamSynchronize(c->stream));
  CU(cudaGetLastError());
  return check_dev_err(c);
}
extern "C" int32_t pm_ctx_set_tensor_core_min_tokens(pm_ctx *c, int32_t min_tokens) {
  if (!c || min_tokens < 0) return fail(PM_ERR_INVALID, "pm_ctx_set_tensor_core_min_tokens");
  c->tc_min_tokens = min_tokens;
  return PM_OK;
}
extern "C" int32_t pm_stack_destroy(pm_stack *s);
extern "C" void *pm_ctx_stream(pm_ctx *c) { return c ? (void *)c->stream : nullptr; }
extern "C" int64_t pm_ctx_launch_count(pm_ctx *c) { return c ? c->launches : 0; }
extern "C" int32_t pm_ctx_path_counts(pm_ctx *c, int64_t *out) {
  if (!c || !out) return fail(PM_ERR_INVALID, "pm_ctx_path_counts: null argument");
  for (int i = 0; i < PM_PATH_N; i++) out[i] = c->path_count[i];
  return PM_OK;
}
extern "C" int32_t pm_debug_set_wait_limit_ns(pm_ctx *c, uint64_t ns) {
  if (!c || ns == 0) return fail(PM_ERR_INVALID, "pm_debug_set_wait_limit_ns");
  c->wait_ns = ns;
  return PM_OK;
}
extern "C" int32_t pm_debug_device_free_bytes(pm_ctx *c, uint64_t *out) {
  if (!c || !out) return fail(PM_ERR_INVALID, "pm_debug_device_free_bytes");
  CU(cudaSetDevice(c->device));
  size_t fr = 0, tot = 0;
  CU(cudaMemGetInfo(&fr, &tot));
  *out = (uint64_t)fr;
  return PM_OK;
}
extern "C" int32_t pm_debug_tc_fault_block(pm_ctx *c, int32_t block) {
  if (!c) return fail(PM_ERR_INVALID, "pm_debug_tc_fault_block");
  c->tc_fault_block = block;
  return PM_OK;
}

extern "C" int32_t pm_timer_start(pm_ctx *c) {
  CU(cudaEventRecord(c->ev0, c->stream));
  return PM_OK;
}
extern "C" int32_t pm_timer_stop(pm_ctx *c, float *ms) {
  CU(cudaEventRecord(c->ev1, c->stream));
  CU(cudaEventSynchronize(c->ev1));
  CU(cudaEventElapsedTime(ms, c->ev0, c->ev1));
  return PM_OK;
}
extern "C" int32_t pm_flush_l2(pm_ctx *c) {
  const size_t bytes = (size_t)256 << 20;  // 2x the 126 MB L2
  if (!c->flush) {
    CU(cudaMalloc(&c->flush, bytes));
    c->flush_bytes = bytes;
  }
  CU(cudaMemsetAsync(c->flush, 0x5a, c->flush_bytes, c->stream));
  return PM_OK;
}
extern "C" int32_t pm_profile_enable(pm_ctx *c, int32_t on) {
  if (!c) return fail(PM_ERR_INVALID, "pm_profile_enable: null context");
  CU(cudaStreamSynchronize(c->stream));
  c->prof_on = on != 0;
  c->prof_used = 0;
  c->prof_phase.clear();
  return PM_OK;
}
extern "C" int32_t pm_profile_phases(void) { return PH_N; }
extern "C" const char *pm_profile_phase_name(int32_t i) {
  return (i >= 0 && i < PH_N) ? PH_NAMES[i] : "";
}
extern "C" int32_t pm_profile_read(pm_ctx *c, float *ms, int64_t *spans) {
  if (!c || !ms || !spans) return fail(PM_ERR_INVALID, "pm_profile_read: null argument");
  CU(cudaStreamSynchronize(c->stream));
  for (int i = 0; i < PH_N; i++) { ms[i] = 0.0f; spans[i] = 0; }
  for (size_t i = 0; i < c->prof_phase.size(); i++) {
    float t = 0.0f;
    CU(cudaEventElapsedTime(&t, c->prof_ev[2 * i], c->prof_ev[2 * i + 1]));
    ms[c->prof_phase[i]] += t;
    spans[c->prof_phase[i]]++;
  }
  c->prof_used = 0;
  c->prof_phase.clear();
  return PM_OK;
}
extern "C" int32_t pm_host_alloc(pm_ctx *c, size_t bytes, void **out) {
  if (!c || !out) return fail(PM_ERR_INVALID, "pm_host_alloc: null argument");
  CU(cudaSetDevice(c->device));
  CU(cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault));
  return PM_OK;
}
extern "C" int32_t pm_host_free(pm_ctx *c, void *p) {
  CU(cudaFreeHost(p));
  return PM_OK;
}
extern "C" int32_t pm_dev_alloc(pm_ctx *c, size_t bytes, void **out) {
  CU(cudaSetDevice(c->device));
  CU(cudaMalloc(out, bytes ? bytes : 1));
  return PM_OK;
}
extern "C" int32_t pm_dev_free(pm_ctx *c, void *p) {
  CU(cudaStreamSynchronize(c->stream));
  CU(cudaFree(p));
  return PM_OK;
}
extern "C" int32_t pm_copy(pm_ctx *c, void *dst, const void *src, size_t bytes) {
  CU(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, c->stream));
  if (!is_device_ptr(dst) || !is_device_ptr(src)) CU(cudaStreamSynchronize(c->stream));
  return PM_OK;
}

// ---------------------------------------------------------------------------
// layer
// ---------------------------------------------------------------------------
struct pm_layer {
  pm_ctx *ctx = nullptr;
  LayerDev dev{};
  std::vector<void *> owned;
  std::vector<uint8_t> expert_set;
  bool router_set = false, shared_set = false;
  uint64_t gen = 0;  // bumped by every call that may change a device pointer or a weight (stacks re-snapshot)
  float *router_w = nullptr, *logit_bias = nullptr, *select_bias = nullptr;
  float *bias_gate = nullptr, *bias_up = nullptr, *bias_down = nullptr, *gate_inp = nullptr;
};

static bool type_ok(int t) {
  return t == PM_TYPE_Q4_K || t == PM_TYPE_Q6_K || t == PM_TYPE_MXFP4 || t == PM_TYPE_Q8_0 || t == PM_TYPE_IQ4_NL ||
         t == PM_TYPE_IQ4_XS || t == PM_TYPE_IQ3_S || t == PM_TYPE_Q5_K || t == PM_TYPE_GLM_Q4;
}

static int32_t wmat_alloc(pm_layer *ly, WMat &W, int type, int n_exp, int rows, int cols) {
  W.type = type;
  W.rows = rows;
  W.cols = cols;
  for (int p = 0; p < 4; p++) {
    W.plane[p] = nullptr;
    W.stride[p] = wmat_plane_bytes(type, rows, cols, p);
    if (W.stride[p]) {
      // 256 spare bytes: vector loads of a partial last chunk never leave the allocation
      CU(cudaMalloc(&W.plane[p], W.stride[p] * (size_t)n_exp + 256));
      ly->owned.push_back(W.plane[p]);
    }
  }
  return PM_OK;
}

static int32_t validate_desc(const pm_layer_desc *D) {
  if (D->d < 32 || D->ff < 32 || D->d % 32 || D->ff % 32)
    return fail(PM_ERR_INVALID, "d and ff must be multiples of 32 (d=%d ff=%d)", D->d, D->ff);
  if (D->d > PM_MAX_D) return fail(PM_ERR_LIMIT, "d %d above %d", D->d, PM_MAX_D);
  if (D->n_exp < 1 || D->n_exp > PM_MAX_EXPERTS)
    return fail(PM_ERR_LIMIT, "n_exp %d outside 1..%d", D->n_exp, PM_MAX_EXPERTS);
  if (D->top_k < 1 || D->top_k > PM_MAX_TOPK || D->top_k > D->n_exp)
    return fail(PM_ERR_LIMIT, "top_k %d outside 1..%d", D->top_k, PM_MAX_TOPK);
  if (D->gating < 0 || D->gating > PM_GATE_SOFTMAX_SELECTED)
    return fail(PM_ERR_INVALID, "gating %d", D->gating);
  if (D->n_group > 0) {
    if (D->n_exp % D->n_group || D->topk_group < 1 || D->topk_group > D->n_group ||
        D->n_exp / D->n_group < 2 || D->topk_group * (D->n_exp / D->n_group) < D->top_k ||
        D->n_group > PM_MAX_EXPERTS / 2)
      return fail(PM_ERR_INVALID, "group-limited selection: n_group=%d topk_group=%d n_exp=%d",
                  D->n_group, D->topk_group, D->n_exp);
  }
  if (D->act < 0 || D->act > PM_ACT_OSS_GLU) return fail(PM_ERR_INVALID, "act %d", D->act);
  if (!type_ok(D->type_gate) || !type_ok(D->type_up) || !type_ok(D->type_down))
    return fail(PM_ERR_UNSUPPORTED, "expert tensor types %d/%d/%d", D->type_gate, D->type_up,
                D->type_down);
  if (D->act_quant == PM_AQ_Q8X_256) {
    if (D->d % 256 || D->ff % 256)
      return fail(PM_ERR_INVALID, "Q8x activations need d and ff multiples of 256 (src/ds4_cpu.rs:15)");
    const int ts[3] = {D->type_gate, D->type_up, D->type_down};
    for (int t : ts)
      if (t != PM_TYPE_Q4_K && t != PM_TYPE_Q6_K)
        return fail(PM_ERR_UNSUPPORTED, "Q8x activations pair with Q4_K / Q6_K weights only");
    if (D->shared && D->shared_ff % 256) return fail(PM_ERR_INVALID, "shared_ff %% 256");
  } else if (D->act_quant == PM_AQ_Q8_32 || D->act_quant == PM_AQ_Q8_32_F16) {
    if (D->d % 32 || D->ff % 32 || (D->shared && D->shared_ff % 32))
      return fail(PM_ERR_INVALID, "32-block Q8 activations need d and ff multiples of 32 (src/q4x_cpu.rs:24)");
    const int t32[3] = {D->type_gate, D->type_up, D->type_down};
    for (int t : t32)
      if (t != PM_TYPE_Q8_0 && t != PM_TYPE_IQ4_NL && t != PM_TYPE_IQ4_XS && t != PM_TYPE_IQ3_S &&
          !(t == PM_TYPE_Q4_K && D->act_quant == PM_AQ_Q8_32_F16))
        return fail(PM_ERR_UNSUPPORTED, "32-block Q8 activations pair with Q8_0 / IQ4_NL / IQ4_XS / IQ3_S weights (and, with "
                                        "the f16 scale, Q4_K) only");
  } else if (D->act_quant != PM_AQ_F32) {
    return fail(PM_ERR_UNSUPPORTED, "act_quant %d", D->act_quant);
  }
  const int ts[3] = {D->type_gate, D->type_up, D->type_down};
  const int cs[3] = {D->d, D->d, D->ff};
  for (int i = 0; i < 3; i++)
    if (cs[i] % (int)pm_type_block_values(ts[i]))
      return fail(PM_ERR_INVALID, "row length %d is not whole blocks of type %d", cs[i], ts[i]);
  if (D->weight_fold != PM_FOLD_BEFORE_DOWN && D->weight_fold != PM_FOLD_IN_COMBINE)
    return fail(PM_ERR_INVALID, "weight_fold %d", D->weight_fold);
  if (D->shared < 0 || D->shared > PM_SHARED_SIGMOID_GATED) return fail(PM_ERR_INVALID, "shared");
  if (D->shared && (D->shared_ff < 32 || D->shared_ff % 32))
    return fail(PM_ERR_INVALID, "shared_ff %d", D->shared_ff);
  if (D->n_exp_local < 0 || D->first_local_expert < 0 ||
      D->first_local_expert + D->n_exp_local > D->n_exp)
    return fail(PM_ERR_INVALID, "local expert range");
  return PM_OK;
}

extern "C" int32_t pm_layer_destroy(pm_layer *ly) {
  if (!ly) return PM_OK;
  cudaSetDevice(ly->ctx->device);
  cudaStreamSynchronize(ly->ctx->stream);
  for (void *p : ly->owned) cudaFree(p);
  delete ly;
  return PM_OK;
}

template <typename T>
static int32_t dev_new(pm_layer *ly, T **out, size_t n, bool zero) {
  CU(cudaMalloc(out, (n ? n : 1) * sizeof(T)));
  ly->owned.push_back(*out);
  if (zero) CU(cudaMemsetAsync(*out, 0, (n ? n : 1) * sizeof(T), ly->ctx->stream));
  return PM_OK;
}

extern "C" int32_t pm_layer_create(pm_ctx *ctx, const pm_layer_desc *desc, pm_layer **out) {
  if (!ctx || !desc || !out) return fail(PM_ERR_INVALID, "pm_layer_create: null argument");
  TRY(validate_desc(desc));
  CU(cudaSetDevice(ctx->device));
  pm_layer *ly = new (std::nothrow) pm_layer();
  if (!ly) return fail(PM_ERR_OOM, "host allocation");
  ly->ctx = ctx;
  LayerDev &dv = ly->dev;
  dv.desc = *desc;
  dv.n_local = desc->n_exp_local > 0 ? desc->n_exp_local : desc->n_exp;
  dv.first_local = desc->n_exp_local > 0 ? desc->first_local_expert : 0;
  ly->expert_set.assign((size_t)dv.n_local, 0);
  int32_t rc = PM_OK;
  auto chk = [&](int32_t r) { if (rc == PM_OK) rc = r; };
  const int E = desc->n_exp, d = desc->d, ff = desc->ff, nl = dv.n_local;
  chk(dev_new(ly, &ly->router_w, (size_t)E * d, true));
  chk(dev_new(ly, &dv.usage, (size_t)E, true));
  if (rc == PM_OK) chk(wmat_alloc(ly, dv.gate, desc->type_gate, nl, ff, d));
  if (rc == PM_OK) chk(wmat_alloc(ly, dv.up, desc->type_up, nl, ff, d));
  if (rc == PM_OK) chk(wmat_alloc(ly, dv.down, desc->type_down, nl, d, ff));
  if (rc == PM_OK && desc->has_expert_bias) {
    chk(dev_new(ly, &ly->bias_gate, (size_t)nl * ff, true));
    chk(dev_new(ly, &ly->bias_up, (size_t)nl * ff, true));
    chk(dev_new(ly, &ly->bias_down, (size_t)nl * d, true));
  }
  if (rc == PM_OK && desc->shared) {
    chk(wmat_alloc(ly, dv.sgate, desc->type_gate, 1, desc->shared_ff, d));
    chk(wmat_alloc(ly, dv.sup, desc->type_up, 1, desc->shared_ff, d));
    chk(wmat_alloc(ly, dv.sdown, desc->type_down, 1, d, desc->shared_ff));
  }
  if (rc != PM_OK) {
    pm_layer_destroy(ly);
    return rc;
  }
  dv.router = ly->router_w;
  dv.bias_gate = ly->bias_gate;
  dv.bias_up = ly->bias_up;
  dv.bias_down = ly->bias_down;
  *out = ly;
  return PM_OK;
}

extern "C" int32_t pm_layer_set_router(pm_layer *ly, const void *w, int32_t dtype,
                                       const float *logit_bias, const float *select_bias) {
  if (!ly || !w) return fail(PM_ERR_INVALID, "pm_layer_set_router: null argument");
  pm_ctx *c = ly->ctx;
  CU(cudaSetDevice(c->device));
  const pm_layer_desc &D = ly->dev.desc;
  size_t n = (size_t)D.n_exp * D.d;
  if (dtype == PM_TYPE_F32) {
    CU(cudaMemcpyAsync(ly->router_w, w, n * 4, cudaMemcpyDefault, c->stream));
  } else if (dtype == PM_TYPE_BF16) {
    // bf16 -> f32 is exact (src/quant.rs:282: dot_bf16 == dot_f32 bit for bit)
    if (is_device_ptr(w)) return fail(PM_ERR_UNSUPPORTED, "bf16 router must be a host pointer");
    std::vector<uint32_t> tmp(n);
    const uint16_t *s = (const uint16_t *)w;
    for (size_t i = 0; i < n; i++) tmp[i] = (uint32_t)s[i] << 16;
    CU(cudaMemcpyAsync(ly->router_w, tmp.data(), n * 4, cudaMemcpyHostToDevice, c->stream));
    CU(cudaStreamSynchronize(c->stream));
  } else {
    return fail(PM_ERR_UNSUPPORTED, "router dtype %d (f32 or bf16)", dtype);
  }
  if (logit_bias) {
    if (!ly->logit_bias) TRY(dev_new(ly, &ly->logit_bias, (size_t)D.n_exp, false));
    CU(cudaMemcpyAsync(ly->logit_bias, logit_bias, (size_t)D.n_exp * 4, cudaMemcpyDefault, c->stream));
    ly->dev.logit_bias = ly->logit_bias;
  }
  if (select_bias) {
    if (!ly->select_bias) TRY(dev_new(ly, &ly->select_bias, (size_t)D.n_exp, false));
    CU(cudaMemcpyAsync(ly->select_bias, select_bias, (size_t)D.n_exp * 4, cudaMemcpyDefault, c->stream));
    ly->dev.select_bias = ly->select_bias;
  }
  CU(cudaStreamSynchronize(c->stream));
  ly->router_set = true;
  ly->gen++;
  return PM_OK;
}

// raw GGUF bytes (host or device) -> planes of expert slot `el`
static int32_t upload_mat(pm_layer *ly, WMat &W, int el, const uint8_t *raw) {
  pm_ctx *c = ly->ctx;
  size_t bytes = raw_bytes(W.type, (size_t)W.rows, (size_t)W.cols);
  size_t nb = (size_t)W.rows * (W.cols / pm_type_block_values(W.type));
  const uint8_t *src = raw;
  if (!is_device_ptr(raw)) {
    TRY(stage_reserve(c, bytes));
    CU(cudaMemcpyAsync(c->stage, raw, bytes, cudaMemcpyHostToDevice, c->stream));
    src = c->stage;
  }
  uint8_t *p[4];
  for (int i = 0; i < 4; i++) p[i] = W.plane[i] ? W.plane[i] + (size_t)el * W.stride[i] : nullptr;
  launch_repack(c->launch(), W.type, src, nb, p[0], p[1], p[2], p[3]);
  CU(cudaGetLastError());
  CU(cudaStreamSynchronize(c->stream));  // the staging buffer is reused by the next upload
  return PM_OK;
}

extern "C" int32_t pm_layer_set_expert(pm_layer *ly, int32_t e, const uint8_t *gate,
                                       const uint8_t *up, const uint8_t *down,
                                       const float *bias_gate, const float *bias_up,
                                       const float *bias_down) {
  if (!ly || !gate || !up || !down) return fail(PM_ERR_INVALID, "pm_layer_set_expert: null argument");
  LayerDev &dv = ly->dev;
  int el = e - dv.first_local;
  if (el < 0 || el >= dv.n_local)
    return fail(PM_ERR_INVALID, "expert %d is not local to this context [%d, %d)", e, dv.first_local,
                dv.first_local + dv.n_local);
  CU(cudaSetDevice(ly->ctx->device));
  TRY(upload_mat(ly, dv.gate, el, gate));
  TRY(upload_mat(ly, dv.up, el, up));
  TRY(upload_mat(ly, dv.down, el, down));
  if (dv.desc.has_expert_bias) {
    if (!bias_gate || !bias_up || !bias_down)
      return fail(PM_ERR_INVALID, "layer has expert biases; all three are required");
    cudaStream_t s = ly->ctx->stream;
    int ff = dv.desc.ff, d = dv.desc.d;
    CU(cudaMemcpyAsync(ly->bias_gate + (size_t)el * ff, bias_gate, (size_t)ff * 4, cudaMemcpyDefault, s));
    CU(cudaMemcpyAsync(ly->bias_up + (size_t)el * ff, bias_up, (size_t)ff * 4, cudaMemcpyDefault, s));
    CU(cudaMemcpyAsync(ly->bias_down + (size_t)el * d, bias_down, (size_t)d * 4, cudaMemcpyDefault, s));
    CU(cudaStreamSynchronize(s));
  }
  ly->expert_set[(size_t)el] = 1;
  ly->gen++;
  return PM_OK;
}

extern "C" int32_t pm_layer_set_shared(pm_layer *ly, const uint8_t *gate, const uint8_t *up,
                                       const uint8_t *down, const float *gate_inp) {
  if (!ly || !gate || !up || !down) return fail(PM_ERR_INVALID, "pm_layer_set_shared: null argument");
  LayerDev &dv = ly->dev;
  if (!dv.desc.shared) return fail(PM_ERR_STATE, "layer was created without a shared expert");
  CU(cudaSetDevice(ly->ctx->device));
  TRY(upload_mat(ly, dv.sgate, 0, gate));
  TRY(upload_mat(ly, dv.sup, 0, up));
  TRY(upload_mat(ly, dv.sdown, 0, down));
  if (dv.desc.shared == PM_SHARED_SIGMOID_GATED) {
    if (!gate_inp) return fail(PM_ERR_INVALID, "sigmoid-gated shared expert needs gate_inp");
    if (!ly->gate_inp) TRY(dev_new(ly, &ly->gate_inp, (size_t)dv.desc.d, false));
    CU(cudaMemcpyAsync(ly->gate_inp, gate_inp, (size_t)dv.desc.d * 4, cudaMemcpyDefault, ly->ctx->stream));
    CU(cudaStreamSynchronize(ly->ctx->stream));
    dv.shared_gate_inp = ly->gate_inp;
  }
  ly->shared_set = true;
  ly->gen++;
  return PM_OK;
}

extern "C" int32_t pm_layer_read_usage(pm_layer *ly, uint32_t *out) {
  if (!ly || !out) return fail(PM_ERR_INVALID, "pm_layer_read_usage: null argument");
  CU(cudaMemcpyAsync(out, ly->dev.usage, (size_t)ly->dev.desc.n_exp * 4, cudaMemcpyDeviceToHost,
                     ly->ctx->stream));
  CU(cudaStreamSynchronize(ly->ctx->stream));
  return PM_OK;
}

static int32_t layer_ready(const pm_layer *ly, bool need_experts) {
  if (!ly) return fail(PM_ERR_INVALID, "null layer");
  if (!ly->router_set) return fail(PM_ERR_STATE, "router weights not set");
  if (need_experts) {
    for (size_t i = 0; i < ly->expert_set.size(); i++)
      if (!ly->expert_set[i])
        return fail(PM_ERR_STATE, "expert %d has no weights", (int)i + ly->dev.first_local);
    if (ly->dev.desc.shared && !ly->shared_set) return fail(PM_ERR_STATE, "shared expert not set");
  }
  return PM_OK;
}

extern "C" int32_t pm_layer_get_expert(pm_layer *ly, int32_t e, int32_t which, uint8_t *out) {
  if (!ly || !out || which < 0 || which > 2) return fail(PM_ERR_INVALID, "pm_layer_get_expert");
  LayerDev &dv = ly->dev;
  pm_ctx *c = ly->ctx;
  bool shared = e < 0;
  int el = shared ? 0 : e - dv.first_local;
  if (!shared && (el < 0 || el >= dv.n_local)) return fail(PM_ERR_INVALID, "expert %d not local", e);
  if (shared && !dv.desc.shared) return fail(PM_ERR_STATE, "no shared expert");
  WMat &W = shared ? (which == 0 ? dv.sgate : which == 1 ? dv.sup : dv.sdown)
                   : (which == 0 ? dv.gate : which == 1 ? dv.up : dv.down);
  size_t bytes = raw_bytes(W.type, (size_t)W.rows, (size_t)W.cols);
  size_t nb = (size_t)W.rows * (W.cols / pm_type_block_values(W.type));
  CU(cudaSetDevice(c->device));
  TRY(stage_reserve(c, bytes));
  const uint8_t *p[4];
  for (int i = 0; i < 4; i++) p[i] = W.plane[i] ? W.plane[i] + (size_t)el * W.stride[i] : nullptr;
  launch_unpack(c->launch(), W.type, c->stage, nb, p[0], p[1], p[2], p[3]);
  CU(cudaGetLastError());
  CU(cudaMemcpyAsync(out, c->stage, bytes, cudaMemcpyDeviceToHost, c->stream));
  CU(cudaStreamSynchronize(c->stream));
  return PM_OK;
}

extern "C" int32_t pm_layer_get_router(pm_layer *ly, float *w, float *logit_bias,
                                       float *select_bias) {
  if (!ly) return fail(PM_ERR_INVALID, "pm_layer_get_router");
  const pm_layer_desc &D = ly->dev.desc;
  cudaStream_t s = ly->ctx->stream;
  if (w) CU(cudaMemcpyAsync(w, ly->router_w, (size_t)D.n_exp * D.d * 4, cudaMemcpyDeviceToHost, s));
  if (logit_bias && ly->logit_bias)
    CU(cudaMemcpyAsync(logit_bias, ly->logit_bias, (size_t)D.n_exp * 4, cudaMemcpyDeviceToHost, s));
  if (select_bias && ly->select_bias)
    CU(cudaMemcpyAsync(select_bias, ly->select_bias, (size_t)D.n_exp * 4, cudaMemcpyDeviceToHost, s));
  CU(cudaStreamSynchronize(s));
  return PM_OK;
}

// synthetic weights, generated and quantised on the device
static int32_t synth_mat(pm_layer *ly, WMat &W, int n_exp, uint64_t seed, float sigma) {
  pm_ctx *c = ly->ctx;
  size_t per = raw_bytes(W.type, (size_t)W.rows, (size_t)W.cols);
  size_t nb_per = (size_t)W.rows * (W.cols / pm_type_block_values(W.type));
  if (W.type != PM_TYPE_Q4_K && W.type != PM_TYPE_Q6_K && W.type != PM_TYPE_MXFP4) return fail(PM_ERR_UNSUPPORTED, "synthetic weights of type %d", W.type);
  // groups of experts so the raw staging stays below ~1 GB
  int group = (int)((((size_t)1 << 30) / per) ? (((size_t)1 << 30) / per) : 1);
  if (group > n_exp) group = n_exp;
  TRY(stage_reserve(c, per * (size_t)group));
  for (int e0 = 0; e0 < n_exp; e0 += group) {
    int n = n_exp - e0 < group ? n_exp - e0 : group;
    launch_synth_blocks(c->launch(), W.type, c->stage, nb_per * n,
                        seed + 0x1000193ull * (uint64_t)e0, sigma);
    uint8_t *p[4];
    for (int i = 0; i < 4; i++) p[i] = W.plane[i] ? W.plane[i] + (size_t)e0 * W.stride[i] : nullptr;
    launch_repack(c->launch(), W.type, c->stage, nb_per * n, p[0], p[1], p[2], p[3]);
    CU(cudaGetLastError());
  }
  return PM_OK;
}

extern "C" int32_t pm_layer_get_expert_bias(pm_layer *ly, int32_t e, float *bg, float *bu,
                                            float *bd) {
  if (!ly) return fail(PM_ERR_INVALID, "pm_layer_get_expert_bias");
  const LayerDev &dv = ly->dev;
  int el = e - dv.first_local;
  if (!dv.desc.has_expert_bias) return fail(PM_ERR_STATE, "layer has no expert biases");
  if (el < 0 || el >= dv.n_local) return fail(PM_ERR_INVALID, "expert %d not local", e);
  cudaStream_t s = ly->ctx->stream;
  int ff = dv.desc.ff, d = dv.desc.d;
  if (bg) CU(cudaMemcpyAsync(bg, ly->bias_gate + (size_t)el * ff, (size_t)ff * 4, cudaMemcpyDeviceToHost, s));
  if (bu) CU(cudaMemcpyAsync(bu, ly->bias_up + (size_t)el * ff, (size_t)ff * 4, cudaMemcpyDeviceToHost, s));
  if (bd) CU(cudaMemcpyAsync(bd, ly->bias_down + (size_t)el * d, (size_t)d * 4, cudaMemcpyDeviceToHost, s));
  CU(cudaStreamSynchronize(s));
  return PM_OK;
}

extern "C" int32_t pm_layer_fill_synthetic(pm_layer *ly, uint64_t seed, float sigma,
                                           float logit_bias_sigma, float select_bias_sigma) {
  if (!ly) return fail(PM_ERR_INVALID, "pm_layer_fill_synthetic: null layer");
  pm_ctx *c = ly->ctx;
  LayerDev &dv = ly->dev;
  const pm_layer_desc &D = dv.desc;
  CU(cudaSetDevice(c->device));
  Launch L = c->launch();
  launch_synth_f32(L, ly->router_w, (size_t)D.n_exp * D.d, seed ^ 0x11, sigma, 0);
  if (logit_bias_sigma > 0.0f) {
    if (!ly->logit_bias) TRY(dev_new(ly, &ly->logit_bias, (size_t)D.n_exp, false));
    launch_synth_f32(L, ly->logit_bias, (size_t)D.n_exp, seed ^ 0xcc, logit_bias_sigma, 1);
    dv.logit_bias = ly->logit_bias;
  }
  if (select_bias_sigma > 0.0f) {
    if (!ly->select_bias) TRY(dev_new(ly, &ly->select_bias, (size_t)D.n_exp, false));
    launch_synth_f32(L, ly->select_bias, (size_t)D.n_exp, seed ^ 0xdd, select_bias_sigma, 0);
    dv.select_bias = ly->select_bias;
  }
  TRY(synth_mat(ly, dv.gate, dv.n_local, seed ^ 0x22 ^ ((uint64_t)dv.first_local << 32), sigma));
  TRY(synth_mat(ly, dv.up, dv.n_local, seed ^ 0x33 ^ ((uint64_t)dv.first_local << 32), sigma));
  TRY(synth_mat(ly, dv.down, dv.n_local, seed ^ 0x44 ^ ((uint64_t)dv.first_local << 32), sigma));
  if (D.has_expert_bias) {
    launch_synth_f32(L, ly->bias_gate, (size_t)dv.n_local * D.ff, seed ^ 0x55, sigma, 1);
    launch_synth_f32(L, ly->bias_up, (size_t)dv.n_local * D.ff, seed ^ 0x66, sigma, 1);
    launch_synth_f32(L, ly->bias_down, (size_t)dv.n_local * D.d, seed ^ 0x77, sigma, 1);
  }
  if (D.shared) {
    TRY(synth_mat(ly, dv.sgate, 1, seed ^ 0x88, sigma));
    TRY(synth_mat(ly, dv.sup, 1, seed ^ 0x99, sigma));
    TRY(synth_mat(ly, dv.sdown, 1, seed ^ 0xaa, sigma));
    if (D.shared == PM_SHARED_SIGMOID_GATED) {
      if (!ly->gate_inp) TRY(dev_new(ly, &ly->gate_inp, (size_t)D.d, false));
      launch_synth_f32(L, ly->gate_inp, (size_t)D.d, seed ^ 0xbb, sigma, 0);
      dv.shared_gate_inp = ly->gate_inp;
    }
    ly->shared_set = true;
  }
  CU(cudaGetLastError());
  CU(cudaStreamSynchronize(c->stream));
  ly->router_set = true;
  std::fill(ly->expert_set.begin(), ly->expert_set.end(), 1);
  ly->gen++;
  return PM_OK;
}

// ---------------------------------------------------------------------------
// the pipeline on device pointers
// ---------------------------------------------------------------------------
struct Scratch {
  float *logits;
  uint32_t *ids;
  float *w;
  PlanDev plan;
  int8_t *xq; float *xd; int32_t *xbsum; uint16_t *xbm; int32_t *xs;
  float *h; int8_t *hq; float *hd; int32_t *hbsum; uint16_t *hbm; int32_t *hs;
  float *eo;
  uint16_t *xhl, *hhl;  // MXFP4 tensor-core path: bf16 (hi, lo) split of x [2][T*d] and of h [2][P*ff]
  uint32_t *tiles;  // tile list of the tensor-core kernels
  uint8_t *rec;     // activation rows regrouped into the int8 tensor-core kernel's records
  // shared expert
  int *one; uint32_t *zero_u, *tcount, *iota;
  float *sh; int8_t *shq; float *shd; int32_t *shbsum; uint16_t *shbm; int32_t *shs;
  float *shared_out, *shared_logit;
};

// the largest record buffer any tensor-core launch of a T-token call needs (Q8x activations only)
static size_t scratch_rec_bytes(const pm_layer_desc &D, int T) {
  if (D.act_quant != PM_AQ_Q8X_256) return 0;
  const int P = T * D.top_k, E = D.n_exp;
  size_t r = std::max(tc_rec_bytes(P, E, D.d), tc_rec_bytes(P, E, D.ff));
  if (D.shared) r = std::max(r, std::max(tc_rec_bytes(T, 1, D.d), tc_rec_bytes(T, 1, D.shared_ff)));
  return r;
}

static size_t scratch_bytes(const pm_layer_desc &D, int T) {
  size_t P = (size_t)T * D.top_k, E = (size_t)D.n_exp, d = (size_t)D.d, ff = (size_t)D.ff;
  size_t b = 0;
  b += al(T * E * 4) + al(P * 4) * 2;                  // logits, ids, w
  b += al(4) + al(E * 4) * 5 + al(P * 4) * 3;          // plan
  b += al(T * d) + al(T * (d / 32 + 1) * 4) + al(T * (d / 256 + 1) * 4) + al(T * (d / 32) * 4) * 2;
  b += al(P * ff * 4) + al(P * ff) + al(P * (ff / 32 + 1) * 4) + al(P * (ff / 256 + 1) * 4) + al(P * (ff / 32) * 4) * 2;
  b += al(P * d * 4);
  if (D.act_quant == PM_AQ_F32 && D.type_gate == PM_TYPE_MXFP4) b += al(T * d * 4) + al(P * ff * 4);
  b += al(tc_tile_words((int)(P > (size_t)T ? P : (size_t)T), (int)E + 1) * 4);
  b += al(scratch_rec_bytes(D, T));
  if (D.shared) {
    size_t sf = (size_t)D.shared_ff;
    b += al(4) + al(4) * 2 + al((size_t)T * 4);
    b += al(T * sf * 4) + al(T * sf) + al(T * (sf / 32 + 1) * 4) + al(T * (sf / 256 + 1) * 4) + al(T * (sf / 32) * 4) * 2;
    b += al(T * d * 4) + al((size_t)T * 4);
  }
  return b + 4096;
}

static void scratch_carve(pm_ctx *c, const pm_layer_desc &D, int T, Scratch &S) {
  size_t P = (size_t)T * D.top_k, E = (size_t)D.n_exp, d = (size_t)D.d, ff = (size_t)D.ff;
  S.logits = ws_take<float>(c, T * E);
  S.ids = ws_take<uint32_t>(c, P);
  S.w = ws_take<float>(c, P);
  S.plan.n_active = ws_take<int>(c, 1);
  S.plan.active = ws_take<uint32_t>(c, E);
  S.plan.offset = ws_take<uint32_t>(c, E);
  S.plan.count = ws_take<uint32_t>(c, E);
  S.plan.base = ws_take<uint32_t>(c, E);
  S.plan.cnt = ws_take<uint32_t>(c, E);
  S.plan.pair_token = ws_take<uint32_t>(c, P);
  S.plan.pair_pos = ws_take<uint32_t>(c, P);
  S.plan.pair_src = ws_take<uint32_t>(c, P);
  S.xq = ws_take<int8_t>(c, T * d);
  S.xd = ws_take<float>(c, T * (d / 32 + 1));  // per 256 values (Q8x) or per 32 (Q8)
  S.xbsum = ws_take<int32_t>(c, T * (d / 32));
  S.xbm = ws_take<uint16_t>(c, T * (d / 16));
  S.xs = ws_take<int32_t>(c, T * (d / 256 + 1));
  S.h = ws_take<float>(c, P * ff);
  S.hq = ws_take<int8_t>(c, P * ff);
  S.hd = ws_take<float>(c, P * (ff / 32 + 1));
  S.hbsum = ws_take<int32_t>(c, P * (ff / 32));
  S.hbm = ws_take<uint16_t>(c, P * (ff / 16));
  S.hs = ws_take<int32_t>(c, P * (ff / 256 + 1));
  S.eo = ws_take<float>(c, P * d);
  S.xhl = S.hhl = nullptr;
  if (D.act_quant == PM_AQ_F32 && D.type_gate == PM_TYPE_MXFP4) {
    S.xhl = ws_take<uint16_t>(c, 2 * T * d);
    S.hhl = ws_take<uint16_t>(c, 2 * P * ff);
  }
  S.tiles = ws_take<uint32_t>(c, tc_tile_words((int)(P > (size_t)T ? P : (size_t)T), (int)E + 1));
  S.rec = ws_take<uint8_t>(c, scratch_rec_bytes(D, T));
  if (D.shared) {
    size_t sf = (size_t)D.shared_ff;
    S.one = ws_take<int>(c, 1);
    S.zero_u = ws_take<uint32_t>(c, 1);
    S.tcount = ws_take<uint32_t>(c, 1);
    S.iota = ws_take<uint32_t>(c, (size_t)T);
    S.sh = ws_take<float>(c, T * sf);
    S.shq = ws_take<int8_t>(c, T * sf);
    S.shd = ws_take<float>(c, T * (sf / 32 + 1));
    S.shbsum = ws_take<int32_t>(c, T * (sf / 32));
    S.shbm = ws_take<uint16_t>(c, T * (sf / 16));
    S.shs = ws_take<int32_t>(c, T * (sf / 256 + 1));
    S.shared_out = ws_take<float>(c, T * d);
    S.shared_logit = ws_take<float>(c, (size_t)T);
  } else {
    S.shared_out = nullptr;
    S.shared_logit = nullptr;
  }
}

static Groups plan_groups(const PlanDev &pl, int E) {
  Groups g;
  g.n_groups = pl.n_active;
  g.expert = pl.active;
  g.offset = pl.offset;
  g.count = pl.count;
  g.pair_token = pl.pair_token;
  g.pair_src = pl.pair_src;
  g.max_groups = E;
  return g;
}

// routed experts: x (and its Q8x form) -> eo[P][d]
// prequant: S.xq / S.xd / S.xbsum (and their derived forms) already hold the rows' quantised
// form (rows received from another rank arrive quantised)
static int32_t dev_experts(pm_layer *ly, const float *x, int T, Scratch &S, const float *w, bool prequant = false) {
  pm_ctx *c = ly->ctx;
  const LayerDev &dv = ly->dev;
  const pm_layer_desc &D = dv.desc;
  Launch L = c->launch();
  int P = T * D.top_k;
  Groups g = plan_groups(S.plan, D.n_exp);
  const bool q8 = D.act_quant == PM_AQ_Q8X_256, f16s = D.act_quant == PM_AQ_Q8_32_F16;
  const bool q32 = D.act_quant == PM_AQ_Q8_32 || f16s;
  if (q8 && !prequant) { PROF(c, PH_QUANT_X); launch_quant_q8x(L, x, (size_t)T, D.d, S.xq, S.xd, S.xbsum, S.xbm, S.xs); }
  if (q32 && !prequant) { PROF(c, PH_QUANT_X); launch_quant_q8_32(L, x, (size_t)T, D.d, S.xq, S.xd, f16s); }
  const bool tc = q8 && c->tc_min_tokens > 0 && T >= c->tc_min_tokens;
  // MXFP4 weights with f32 activations: the bf16 tensor-core kernels (tolerance parity, not bits)
  const bool tcmx = D.act_quant == PM_AQ_F32 && D.type_gate == PM_TYPE_MXFP4 && D.type_up == PM_TYPE_MXFP4 &&
                    D.type_down == PM_TYPE_MXFP4 && c->tc_min_tokens > 0 && T >= c->tc_min_tokens && S.xhl;
  if (tcmx) {
    const size_t nx = (size_t)T * D.d, nh = (size_t)P * D.ff;
    {
      PROF(c, PH_QUANT_X);
      launch_split_bf16(L, x, nx, S.xhl, S.xhl + nx);
    }
    {
      PROF(c, PH_GATEUP);
      CU(launch_tc_mx(L, dv, false, g, P, S.tiles, S.xhl, S.xhl + nx, w, S.h, c->dev_err, c->wait_ns));
    }
    {
      PROF(c, PH_QUANT_H);
      launch_split_bf16(L, S.h, nh, S.hhl, S.hhl + nh);
    }
    {
      PROF(c, PH_DOWN);
      CU(launch_tc_mx(L, dv, true, g, P, S.tiles, S.hhl, S.hhl + nh, nullptr, S.eo, c->dev_err, c->wait_ns));
    }
    c->path_count[PM_PATH_TENSOR] += 2;
    CU(cudaGetLastError());
    return PM_OK;
  }
  {
    PROF(c, PH_GATEUP);
    if (tc && D.type_gate == D.type_up) {
      CU(launch_tc_q4k(L, dv, false, false, g, P, S.tiles, S.rec, g.pair_token, S.xq, S.xd, S.xbm, S.xs, w, S.h, c->dev_err, c->wait_ns, c->tc_fault_block));
      c->path_count[PM_PATH_TENSOR]++;
    } else {
      launch_gateup(L, dv, false, g, P, x, S.xq, S.xd, S.xbsum, w, S.h);
      c->path_count[PM_PATH_GENERAL]++;
    }
  }
  if (q8) { PROF(c, PH_QUANT_H); launch_quant_q8x(L, S.h, (size_t)P, D.ff, S.hq, S.hd, S.hbsum, S.hbm, S.hs); }
  if (q32) { PROF(c, PH_QUANT_H); launch_quant_q8_32(L, S.h, (size_t)P, D.ff, S.hq, S.hd, f16s); }
  {
    PROF(c, PH_DOWN);
    if (tc) {
      CU(launch_tc_q4k(L, dv, false, true, g, P, S.tiles, S.rec, nullptr, S.hq, S.hd, S.hbm, S.hs, nullptr, S.eo, c->dev_err, c->wait_ns, c->tc_fault_block));
      c->path_count[PM_PATH_TENSOR]++;
    } else {
      launch_down(L, dv, false, g, P, S.h, S.hq, S.hd, S.hbsum, S.eo);
      c->path_count[PM_PATH_GENERAL]++;
    }
  }
  CU(cudaGetLastError());
  return PM_OK;
}

// shared expert over every token -> S.shared_out (and the gate logit)
static int32_t dev_shared(pm_layer *ly, const float *x, int T, Scratch &S) {
  pm_ctx *c = ly->ctx;
  const LayerDev &dv = ly->dev;
  const pm_layer_desc &D = dv.desc;
  if (!D.shared) return PM_OK;
  PROF(c, PH_SHARED);
  Launch L = c->launch();
  const int one = 1;
  const uint32_t zero = 0, tc = (uint32_t)T;
  CU(cudaMemcpyAsync(S.one, &one, 4, cudaMemcpyHostToDevice, c->stream));
  CU(cudaMemcpyAsync(S.zero_u, &zero, 4, cudaMemcpyHostToDevice, c->stream));
  CU(cudaMemcpyAsync(S.tcount, &tc, 4, cudaMemcpyHostToDevice, c->stream));
  launch_iota(L, S.iota, (uint32_t)T);
  Groups g;
  g.n_groups = S.one;
  g.expert = S.zero_u;
  g.offset = S.zero_u;
  g.count = S.tcount;
  g.pair_token = S.iota;
  g.pair_src = nullptr;
  g.max_groups = 1;
  const bool q8 = D.act_quant == PM_AQ_Q8X_256, f16s = D.act_quant == PM_AQ_Q8_32_F16;
  const bool q32 = D.act_quant == PM_AQ_Q8_32 || f16s;
  // (S.xq holds the tokens' Q8x form already when the routed experts ran first)
  if (q8) launch_quant_q8x(L, x, (size_t)T, D.d, S.xq, S.xd, S.xbsum, S.xbm, S.xs);
  if (q32) launch_quant_q8_32(L, x, (size_t)T, D.d, S.xq, S.xd, f16s);
  const bool use_tc = q8 && c->tc_min_tokens > 0 && T >= c->tc_min_tokens;
  if (use_tc && D.type_gate == D.type_up)
    CU(launch_tc_q4k(L, dv, true, false, g, T, S.tiles, S.rec, g.pair_token, S.xq, S.xd, S.xbm, S.xs, nullptr, S.sh, c->dev_err, c->wait_ns, c->tc_fault_block));
  else
    launch_gateup(L, dv, true, g, T, x, S.xq, S.xd, S.xbsum, nullptr, S.sh);
  if (q8) launch_quant_q8x(L, S.sh, (size_t)T, D.shared_ff, S.shq, S.shd, S.shbsum, S.shbm, S.shs);
  if (q32) launch_quant_q8_32(L, S.sh, (size_t)T, D.shared_ff, S.shq, S.shd, f16s);
  if (use_tc)
    CU(launch_tc_q4k(L, dv, true, true, g, T, S.tiles, S.rec, nullptr, S.shq, S.shd, S.shbm, S.shs, nullptr, S.shared_out, c->dev_err, c->wait_ns, c->tc_fault_block));
  else
    launch_down(L, dv, true, g, T, S.sh, S.shq, S.shd, S.shbsum, S.shared_out);
  if (D.shared == PM_SHARED_SIGMOID_GATED) launch_shared_gate_logit(L, dv, x, T, S.shared_logit);
  else S.shared_logit = nullptr;
  CU(cudaGetLastError());
  return PM_OK;
}

// the whole layer on device pointers (workspace already reserved and carved)
static int32_t dev_forward(pm_layer *ly, const float *x, int T, float *y, bool accumulate,
                           Scratch &S) {
  pm_ctx *c = ly->ctx;
  const LayerDev &dv = ly->dev;
  Launch L = c->launch();
  if (T < PM_SMALL_ROUTE_TOKENS) {  // a few tokens: logits, top-k and plan in one launch
    PROF(c, PH_ROUTER);
    launch_route_plan_small(L, dv, x, T, S.logits, S.ids, S.w, S.plan, nullptr, c->route_ticket);
  } else {
    { PROF(c, PH_ROUTER); launch_router(L, dv, x, T, S.logits); }
    { PROF(c, PH_ROUTE); launch_route(L, dv, S.logits, T, S.ids, S.w); }
    { PROF(c, PH_PLAN); launch_plan(L, dv, S.ids, T, S.plan, c->dev_err); }
  }
  TRY(dev_experts(ly, x, T, S, S.w));
  TRY(dev_shared(ly, x, T, S));
  {
    PROF(c, PH_COMBINE);
    launch_combine(L, dv, S.eo, S.plan.pair_pos, S.w, S.shared_out, S.shared_logit, T, y, accumulate);
  }
  CU(cudaGetLastError());
  return PM_OK;
}

static int32_t check_T(int32_t T) {
  if (T < 0 || T > PM_MAX_TOKENS) return fail(PM_ERR_LIMIT, "T=%d outside 0..%d", T, PM_MAX_TOKENS);
  return PM_OK;
}

// host-or-device input -> device pointer (staged in the workspace when host)
template <typename T>
static int32_t in_dev(pm_ctx *c, const T *p, size_t n, const T **out) {
  if (is_device_ptr(p)) {
    *out = p;
    return PM_OK;
  }
  T *t = ws_take<T>(c, n);
  CU(cudaMemcpyAsync(t, p, n * sizeof(T), cudaMemcpyHostToDevice, c->stream));
  *out = t;
  return PM_OK;
}
struct OutBuf {
  void *host = nullptr;
  void *dev = nullptr;
  size_t bytes = 0;
};
template <typename T>
static T *out_dev(pm_ctx *c, T *p, size_t n, OutBuf &ob) {
  if (is_device_ptr(p)) return p;
  T *t = ws_take<T>(c, n);
  ob.host = p;
  ob.dev = t;
  ob.bytes = n * sizeof(T);
  return t;
}
static int32_t out_flush(pm_ctx *c, OutBuf *obs, int n) {
  bool any = false;
  for (int i = 0; i < n; i++)
    if (obs[i].host && obs[i].bytes) {
      CU(cudaMemcpyAsync(obs[i].host, obs[i].dev, obs[i].bytes, cudaMemcpyDeviceToHost, c->stream));
      any = true;
    }
  if (any) {
    CU(cudaStreamSynchronize(c->stream));
    return check_dev_err(c);
  }
  return PM_OK;
}

extern "C" int32_t pm_moe_forward(pm_layer *ly, const float *x, int32_t T, float *y,
                                  uint32_t flags) {
  TRY(layer_ready(ly, true));
  TRY(check_T(T));
  if (T == 0) return PM_OK;
  if (!x || !y) return fail(PM_ERR_INVALID, "pm_moe_forward: null x or y");
  pm_ctx *c = ly->ctx;
  const pm_layer_desc &D = ly->dev.desc;
  CU(cudaSetDevice(c->device));
  size_t n = (size_t)T * D.d;
  TRY(ws_reserve(c, scratch_bytes(D, T) + 2 * al(n * 4)));
  const float *xd;
  TRY(in_dev(c, x, n, &xd));
  OutBuf ob;
  float *yd = out_dev(c, y, n, ob);
  bool acc = flags & PM_FWD_ACCUMULATE;
  if (acc && ob.host) CU(cudaMemcpyAsync(yd, y, n * 4, cudaMemcpyHostToDevice, c->stream));
  Scratch S;
  scratch_carve(c, D, T, S);
  TRY(dev_forward(ly, xd, T, yd, acc, S));
  return out_flush(c, &ob, 1);
}

extern "C" int32_t pm_router_logits(pm_layer *ly, const float *x, int32_t T, float *logits) {
  TRY(layer_ready(ly, false));
  TRY(check_T(T));
  if (T == 0) return PM_OK;
  pm_ctx *c = ly->ctx;
  const pm_layer_desc &D = ly->dev.desc;
  CU(cudaSetDevice(c->device));
  size_t n = (size_t)T * D.d, nl = (size_t)T * D.n_exp;
  TRY(ws_reserve(c, al(n * 4) + al(nl * 4) + 4096));
  const float *xd;
  TRY(in_dev(c, x, n, &xd));
  OutBuf ob;
  float *ld = out_dev(c, logits, nl, ob);
  launch_router(c->launch(), ly->dev, xd, T, ld);
  CU(cudaGetLastError());
  return out_flush(c, &ob, 1);
}

extern "C" int32_t pm_route_logits(pm_layer *ly, const float *logits, int32_t T, uint32_t *ids,
                                   float *w) {
  TRY(layer_ready(ly, false));
  TRY(check_T(T));
  if (T == 0) return PM_OK;
  pm_ctx *c = ly->ctx;
  const pm_layer_desc &D = ly->dev.desc;
  CU(cudaSetDevice(c->device));
  size_t nl = (size_t)T * D.n_exp, P = (size_t)T * D.top_k;
  TRY(ws_reserve(c, al(nl * 4) + 2 * al(P * 4) + 4096));
  const float *ld;
  TRY(in_dev(c, logits, nl, &ld));
  OutBuf ob[2];
  uint32_t *idd = out_dev(c, ids, P, ob[0]);
  float *wd = out_dev(c, w, P, ob[1]);
  launch_route(c->launch(), ly->dev, ld, T, idd, wd);
  CU(cudaGetLastError());
  return out_flush(c, ob, 2);
}

extern "C" int32_t pm_route(pm_layer *ly, const float *x, int32_t T, uint32_t *ids, float *w) {
  TRY(layer_ready(ly, false));
  TRY(check_T(T));
  if (T == 0) return PM_OK;
  pm_ctx *c = ly->ctx;
  const pm_layer_desc &D = ly->dev.desc;
  CU(cudaSetDevice(c->device));
  size_t n = (size_t)T * D.d, nl = (size_t)T * D.n_exp, P = (size_t)T * D.top_k;
  TRY(ws_reserve(c, al(n * 4) + al(nl * 4) + 2 * al(P * 4) + 4096));
  const float *xd;
  TRY(in_dev(c, x, n, &xd));
  float *ld = ws_take<float>(c, nl);
  OutBuf ob[2];
  uint32_t *idd = out_dev(c, ids, P, ob[0]);
  float *wd = out_dev(c, w, P, ob[1]);
  { PROF(c, PH_ROUTER); launch_router(c->launch(), ly->dev, xd, T, ld); }
  { PROF(c, PH_ROUTE); launch_route(c->launch(), ly->dev, ld, T, idd, wd); }
  CU(cudaGetLastError());
  return out_flush(c, ob, 2);
}

// ---------------------------------------------------------------------------
// routing without any allocation
// ---------------------------------------------------------------------------
// Scratch for pm_route_noalloc: the router logits of up to
// PM_ROUTE_NOALLOC_MAX_TOKENS tokens. It lives in the library image, so every
// GPU that loads the library carries these 512 KB until the process exits.
static __device__ __align__(256) float g_noalloc_logits[PM_ROUTE_NOALLOC_MAX_TOKENS * PM_MAX_EXPERTS];
// The array's name is only a host-side handle; kernels need its device address,
// which differs per GPU. Looked up once per device, with that device current.
static float *g_noalloc_logits_dev[64] = {nullptr};

extern "C" int32_t pm_route_noalloc(pm_layer *ly, const float *x, int32_t T, uint32_t *ids,
                                    float *w) {
  TRY(layer_ready(ly, false));
  if (T < 0 || T > PM_ROUTE_NOALLOC_MAX_TOKENS)
    return fail(PM_ERR_LIMIT, "pm_route_noalloc: T=%d, but its fixed scratch holds at most %d tokens "
                              "(use pm_route for more)", T, PM_ROUTE_NOALLOC_MAX_TOKENS);
  if (T == 0) return PM_OK;
  if (!x || !ids || !w) return fail(PM_ERR_INVALID, "pm_route_noalloc: null argument");
  if (!is_device_ptr(x) || !is_device_ptr(ids) || !is_device_ptr(w))
    return fail(PM_ERR_INVALID, "pm_route_noalloc: x, ids and w must be device pointers "
                                "(staging host buffers would need an allocation)");
  pm_ctx *c = ly->ctx;
  if (c->device < 0 || c->device >= 64) return fail(PM_ERR_LIMIT, "pm_route_noalloc: device index %d", c->device);
  CU(cudaSetDevice(c->device));
  if (!g_noalloc_logits_dev[c->device]) {  // first call on this GPU: resolve the symbol
    float *p = nullptr;
    CU(cudaGetSymbolAddress((void **)&p, g_noalloc_logits));
    g_noalloc_logits_dev[c->device] = p;
  }
  float *logits = g_noalloc_logits_dev[c->device];
  launch_router(c->launch(), ly->dev, x, T, logits);
  launch_route(c->launch(), ly->dev, logits, T, ids, w);
  CU(cudaGetLastError());
  return PM_OK;
}

static void plan_carve(pm_ctx *c, int E, size_t P, PlanDev &pl) {
  pl.n_active = ws_take<int>(c, 1);
  pl.active = ws_take<uint32_t>(c, (size_t)E);
  pl.offset = ws_take<uint32_t>(c, (size_t)E);
  pl.count = ws_take<uint32_t>(c, (size_t)E);
  pl.base = ws_take<uint32_t>(c, (size_t)E);
  pl.cnt = ws_take<uint32_t>(c, (size_t)E);
  pl.pair_token = ws_take<uint32_t>(c, P);
  pl.pair_pos = ws_take<uint32_t>(c, P);
  pl.pair_src = ws_take<uint32_t>(c, P);
}

static int32_t check_ids_host(const pm_layer_desc &D, const uint32_t *ids, size_t P) {
  for (size_t i = 0; i < P; i++)
    if (ids[i] >= (uint32_t)D.n_exp)
      return fail(PM_ERR_INVALID, "expert id %u at %zu is outside 0..%d", ids[i], i, D.n_exp - 1);
  return PM_OK;
}

extern "C" int32_t pm_plan(pm_layer *ly, const uint32_t *ids, int32_t T, pm_plan_out *out) {
  if (!ly || !out) return fail(PM_ERR_INVALID, "pm_plan: null argument");
  TRY(check_T(T));
  pm_ctx *c = ly->ctx;
  const pm_layer_desc &D = ly->dev.desc;
  CU(cudaSetDevice(c->device));
  size_t P = (size_t)T * D.top_k, E = (size_t)D.n_exp;
  if (P && !is_device_ptr(ids)) TRY(check_ids_host(D, ids, P));
  TRY(ws_reserve(c, al(P * 4) * 4 + al(E * 4) * 5 + 8192));
  const uint32_t *idd = nullptr;
  if (P) TRY(in_dev(c, ids, P, &idd));
  PlanDev pl;
  plan_carve(c, D.n_exp, P, pl);
  // the plan of a split call does not count towards usage[]
  LayerDev tmp = ly->dev;
  tmp.usage = nullptr;
  launch_plan(c->launch(), tmp, idd, T, pl, c->dev_err);
  CU(cudaGetLastError());
  cudaStream_t s = c->stream;
  CU(cudaMemcpyAsync(out->n_active, pl.n_active, 4, cudaMemcpyDefault, s));
  CU(cudaMemcpyAsync(out->active, pl.active, E * 4, cudaMemcpyDefault, s));
  CU(cudaMemcpyAsync(out->offset, pl.offset, E * 4, cudaMemcpyDefault, s));
  CU(cudaMemcpyAsync(out->count, pl.count, E * 4, cudaMemcpyDefault, s));
  if (P) {
    CU(cudaMemcpyAsync(out->pair_token, pl.pair_token, P * 4, cudaMemcpyDefault, s));
    CU(cudaMemcpyAsync(out->pair_pos, pl.pair_pos, P * 4, cudaMemcpyDefault, s));
  }
  CU(cudaStreamSynchronize(s));
  return check_dev_err(c);
}

extern "C" int32_t pm_experts(pm_layer *ly, const float *x, int32_t T, const uint32_t *ids,
                              const float *w, float *pair_out) {
  TRY(layer_ready(ly, true));
  TRY(check_T(T));
  if (T == 0) return PM_OK;
  if (!x || !ids || !w || !pair_out) return fail(PM_ERR_INVALID, "pm_experts: null argument");
  pm_ctx *c = ly->ctx;
  const pm_layer_desc &D = ly->dev.desc;
  CU(cudaSetDevice(c->device));
  size_t n = (size_t)T * D.d, P = (size_t)T * D.top_k;
  if (!is_device_ptr(ids)) TRY(check_ids_host(D, ids, P));
  TRY(ws_reserve(c, scratch_bytes(D, T) + al(n * 4) + 2 * al(P * 4) + al(P * D.d * 4)));
  const float *xd, *wd;
  const uint32_t *idd;
  TRY(in_dev(c, x, n, &xd));
  TRY(in_dev(c, ids, P, &idd));
  TRY(in_dev(c, w, P, &wd));
  Scratch S;
  scratch_carve(c, D, T, S);
  LayerDev tmp = ly->dev;
  tmp.usage = nullptr;
  launch_plan(c->launch(), tmp, idd, T, S.plan, c->dev_err);
  TRY(dev_experts(ly, xd, T, S, wd));
  CU(cudaMemcpyAsync(pair_out, S.eo, P * D.d * 4, cudaMemcpyDefault, c->stream));
  CU(cudaStreamSynchronize(c->stream));
  return check_dev_err(c);
}

// one expert per row (expert parallelism: the rows another rank dispatched here)
extern "C" int32_t pm_experts_rows(pm_layer *ly, const float *x, int32_t R, const uint32_t *eids,
                                   const float *w, float *out) {
  TRY(layer_ready(ly, true));
  if (R < 0 || R > PM_MAX_TOKENS * PM_MAX_TOPK)
    return fail(PM_ERR_LIMIT, "pm_experts_rows: R=%d outside 0..%d", R, PM_MAX_TOKENS * PM_MAX_TOPK);
  if (R == 0) return PM_OK;
  if (!x || !eids || !w || !out) return fail(PM_ERR_INVALID, "pm_experts_rows: null argument");
  pm_ctx *c = ly->ctx;
  pm_layer_desc D = ly->dev.desc;
  D.top_k = 1;
  CU(cudaSetDevice(c->device));
  size_t n = (size_t)R * D.d;
  if (!is_device_ptr(eids)) TRY(check_ids_host(D, eids, (size_t)R));
  TRY(ws_reserve(c, scratch_bytes(D, R) + 3 * al(n * 4) + 2 * al((size_t)R * 4)));
  const float *xd, *wd;
  const uint32_t *idd;
  TRY(in_dev(c, x, n, &xd));
  TRY(in_dev(c, eids, (size_t)R, &idd));
  TRY(in_dev(c, w, (size_t)R, &wd));
  OutBuf ob;
  float *od = out_dev(c, out, n, ob);
  Scratch S;
  scratch_carve(c, D, R, S);
  // the same layer seen with one expert per token; outputs are raw pair outputs
  // (routing weight folded only where the layer folds it before down)
  pm_layer view = *ly;
  view.dev.desc = D;
  view.dev.usage = nullptr;
  { PROF(c, PH_PLAN); launch_plan(c->launch(), view.dev, idd, R, S.plan, c->dev_err); }
  TRY(dev_experts(&view, xd, R, S, wd));
  LayerDev cp = view.dev;
  cp.desc.weight_fold = PM_FOLD_BEFORE_DOWN;  // plain gather back to row order
  launch_combine(c->launch(), cp, S.eo, S.plan.pair_pos, wd, nullptr, nullptr, R, od, false);
  CU(cudaGetLastError());
  return out_flush(c, &ob, 1);
}

// the shared expert alone: out[T][d] = shared(x) (times its sigmoid gate, if any)
extern "C" int32_t pm_shared(pm_layer *ly, const float *x, int32_t T, float *out) {
  TRY(layer_ready(ly, true));
  TRY(check_T(T));
  if (!ly->dev.desc.shared) return fail(PM_ERR_STATE, "pm_shared: the layer has no shared expert");
  if (T == 0) return PM_OK;
  if (!x || !out) return fail(PM_ERR_INVALID, "pm_shared: null argument");
  pm_ctx *c = ly->ctx;
  pm_layer_desc D = ly->dev.desc;
  D.top_k = 1;
  CU(cudaSetDevice(c->device));
  size_t n = (size_t)T * D.d;
  TRY(ws_reserve(c, scratch_bytes(D, T) + 2 * al(n * 4) + al((size_t)T * 4) * 2));
  const float *xd;
  TRY(in_dev(c, x, n, &xd));
  OutBuf ob;
  float *od = out_dev(c, out, n, ob);
  Scratch S;
  scratch_carve(c, D, T, S);
  TRY(dev_shared(ly, xd, T, S));
  // y = 0 + shared * gate, through the combine kernel with no routed pairs (K = 0)
  LayerDev cp = ly->dev;
  cp.desc.top_k = 0;
  launch_combine(c->launch(), cp, S.eo, S.plan.pair_pos, nullptr, S.shared_out, S.shared_logit, T, od, false);
  CU(cudaGetLastError());
  return out_flush(c, &ob, 1);
}

extern "C" int32_t pm_combine(pm_layer *ly, const float *pair_out, const uint32_t *ids,
                              const float *w, const float *shared_out, int32_t T, float *y,
                              uint32_t flags) {
  if (!ly) return fail(PM_ERR_INVALID, "pm_combine: null layer");
  TRY(check_T(T));
  if (T == 0) return PM_OK;
  if (!pair_out || !ids || !w || !y) return fail(PM_ERR_INVALID, "pm_combine: null argument");
  pm_ctx *c = ly->ctx;
  const pm_layer_desc &D = ly->dev.desc;
  CU(cudaSetDevice(c->device));
  size_t n = (size_t)T * D.d, P = (size_t)T * D.top_k, E = (size_t)D.n_exp;
  if (!is_device_ptr(ids)) TRY(check_ids_host(D, ids, P));
  TRY(ws_reserve(c, al(P * D.d * 4) + al(P * 4) * 5 + al(E * 4) * 5 + 3 * al(n * 4) + 8192));
  const float *pod, *wd, *sod = nullptr;
  const uint32_t *idd;
  TRY(in_dev(c, pair_out, P * D.d, &pod));
  TRY(in_dev(c, ids, P, &idd));
  TRY(in_dev(c, w, P, &wd));
  if (shared_out) TRY(in_dev(c, shared_out, n, &sod));
  OutBuf ob;
  float *yd = out_dev(c, y, n, ob);
  bool acc = flags & PM_FWD_ACCUMULATE;
  if (acc && ob.host) CU(cudaMemcpyAsync(yd, y, n * 4, cudaMemcpyHostToDevice, c->stream));
  PlanDev pl;
  plan_carve(c, D.n_exp, P, pl);
  LayerDev tmp = ly->dev;
  tmp.usage = nullptr;
  launch_plan(c->launch(), tmp, idd, T, pl, c->dev_err);
  launch_combine(c->launch(), ly->dev, pod, pl.pair_pos, wd, sod, nullptr, T, yd, acc);
  CU(cudaGetLastError());
  return out_flush(c, &ob, 1);
}

// ---------------------------------------------------------------------------
// format checks
// ---------------------------------------------------------------------------
extern "C" int32_t pm_dequant(pm_ctx *c, int32_t type, const uint8_t *blocks, size_t n_values,
                              float *out) {
  if (!c || !blocks || !out) return fail(PM_ERR_INVALID, "pm_dequant: null argument");
  if (!type_ok(type)) return fail(PM_ERR_UNSUPPORTED, "pm_dequant: type %d", type);
  size_t bv = pm_type_block_values(type), bb = pm_type_block_bytes(type);
  if (n_values % bv) return fail(PM_ERR_INVALID, "pm_dequant: %zu values is not whole blocks", n_values);
  if (n_values == 0) return PM_OK;
  CU(cudaSetDevice(c->device));
  size_t nb = n_values / bv, rawb = nb * bb;
  size_t pb[4];
  for (int p = 0; p < 4; p++) pb[p] = wmat_plane_bytes(type, 1, (int)bv, p) * nb;
  TRY(ws_reserve(c, al(rawb) + al(pb[0]) + al(pb[1]) + al(pb[2]) + al(pb[3]) + al(n_values * 4) + 4096));
  const uint8_t *rd;
  TRY(in_dev(c, blocks, rawb, &rd));
  uint8_t *p[4];
  for (int i = 0; i < 4; i++) p[i] = pb[i] ? ws_take<uint8_t>(c, pb[i]) : nullptr;
  OutBuf ob;
  float *od = out_dev(c, out, n_values, ob);
  launch_repack(c->launch(), type, rd, nb, p[0], p[1], p[2], p[3]);
  launch_dequant(c->launch(), type, n_values, p[0], p[1], p[2], p[3], od);
  CU(cudaGetLastError());
  return out_flush(c, &ob, 1);
}

extern "C" int32_t pm_quant_act(pm_ctx *c, int32_t mode, const float *x, size_t n, int8_t *q,
                                float *scale, int32_t *bsum) {
  if (!c || !x || !q || !scale) return fail(PM_ERR_INVALID, "pm_quant_act: null argument");
  if (mode != PM_AQ_Q8X_256 && mode != PM_AQ_Q8_32 && mode != PM_AQ_Q8_32_F16)
    return fail(PM_ERR_UNSUPPORTED, "pm_quant_act: mode %d", mode);
  const bool q32 = mode != PM_AQ_Q8X_256;
  if (!q32 && !bsum) return fail(PM_ERR_INVALID, "pm_quant_act: null bsum");
  if (!q32 && n % 256) return fail(PM_ERR_INVALID, "pm_quant_act: n %% 256 != 0 (src/ds4_cpu.rs:15)");
  if (q32 && n % 32) return fail(PM_ERR_INVALID, "pm_quant_act: n %% 32 != 0 (src/q4x_cpu.rs:24)");
  if (n == 0) return PM_OK;
  CU(cudaSetDevice(c->device));
  TRY(ws_reserve(c, al(n * 4) + al(n) + al(n / 32 * 4) * 2 + 4096));
  const float *xd;
  TRY(in_dev(c, x, n, &xd));
  OutBuf ob[3];
  int8_t *qd = out_dev(c, q, n, ob[0]);
  if (q32) {
    float *sd = out_dev(c, scale, n / 32, ob[1]);
    launch_quant_q8_32(c->launch(), xd, 1, (int)n, qd, sd, mode == PM_AQ_Q8_32_F16);
    CU(cudaGetLastError());
    return out_flush(c, ob, 2);
  }
  float *sd = out_dev(c, scale, n / 256, ob[1]);
  int32_t *bd = out_dev(c, bsum, n / 32, ob[2]);
  launch_quant_q8x(c->launch(), xd, 1, (int)n, qd, sd, bd);
  CU(cudaGetLastError());
  return out_flush(c, ob, 3);
}

// x / rms(x) with unit weight, the norm the stack applies before each layer
extern "C" int32_t pm_rmsnorm(pm_ctx *c, const float *x, int32_t T, int32_t d, float eps, float *out) {
  if (!c || !x || !out) return fail(PM_ERR_INVALID, "pm_rmsnorm: null argument");
  TRY(check_T(T));
  if (T == 0) return PM_OK;
  if (d < 32 || d % 32) return fail(PM_ERR_INVALID, "pm_rmsnorm: d=%d", d);
  CU(cudaSetDevice(c->device));
  size_t n = (size_t)T * d;
  TRY(ws_reserve(c, 2 * al(n * 4) + 4096));
  const float *xd;
  TRY(in_dev(c, x, n, &xd));
  OutBuf ob;
  float *od = out_dev(c, out, n, ob);
  launch_rmsnorm(c->launch(), xd, T, d, eps, od);
  CU(cudaGetLastError());
  return out_flush(c, &ob, 1);
}

// ---------------------------------------------------------------------------
// layer stacks
// ---------------------------------------------------------------------------
struct pm_stack {
  pm_ctx *ctx = nullptr;
  std::vector<pm_layer *> layers;
  float eps = 1e-6f;
  int mode = 0;  // 0 = pick per call, 1 = general kernels only
  // the one-token decode kernel (decode_mega.cu)
  MegaPlan mega;
  bool mega_ok = false;
  MegaLayer *mega_layers = nullptr;
  uint8_t *mega_buf = nullptr;  // exchange buffers + counters + error word
  float *mega_io = nullptr;     // staged input / output token
  size_t mega_buf_bytes = 0, mega_xw_bytes = 0;
  unsigned long long *mega_trace = nullptr;
  unsigned long long calls = 0;
  // general path for a few tokens: the layer loop recorded once as a CUDA graph per token
  // count and replayed (a decode step is a few hundred short launches: host-paced otherwise)
  struct Graph {
    int T;
    uint8_t *ws;          // workspace the recorded kernels point into
    float *gx;            // residual stream of the recorded loop
    cudaGraphExec_t exec;
    int64_t launches;
  };
  std::vector<Graph> graphs;
  std::vector<int> seen_T;  // token counts the general path ran once already
  bool graph_off = false;
  bool fault_next = false;         // pm_debug_stack_fault_next_call
  std::vector<uint64_t> seen_gen;  // the layers' generation counters when their pointers were last snapshot
};

// (re)writes the decode kernel's per-layer pointer table from the layers' current state
static int32_t stack_fill_mega_layers(pm_stack *s) {
  size_t L = s->layers.size();
  std::vector<MegaLayer> ml(L);
  for (size_t i = 0; i < L; i++) {
    const LayerDev &dv = s->layers[i]->dev;
    ml[i].router = dv.router;
    ml[i].logit_bias = dv.logit_bias;
    ml[i].select_bias = dv.select_bias;
    ml[i].gate = dv.gate.plane[0];
    ml[i].gate_stride = dv.gate.stride[0];
    ml[i].up = dv.up.plane[0];
    ml[i].up_stride = dv.up.stride[0];
    for (int p = 0; p < 4; p++) {
      ml[i].down[p] = dv.down.plane[p];
      ml[i].down_stride[p] = dv.down.stride[p];
    }
    ml[i].usage = dv.usage;
  }
  CU(cudaMemcpy(s->mega_layers, ml.data(), L * sizeof(MegaLayer), cudaMemcpyHostToDevice));
  return PM_OK;
}

static void stack_drop_graphs(pm_stack *s) {
  for (auto &g : s->graphs) {
    if (g.exec) cudaGraphExecDestroy(g.exec);
    if (g.gx) cudaFree(g.gx);
  }
  s->graphs.clear();
  s->seen_T.clear();
}

// A layer whose weights, biases or router were (re)loaded after the stack last looked at it:
// the decode kernel's pointer table and the recorded graphs hold the old device pointers
// (a bias buffer, for one, is only allocated by the call that first sets it).
static int32_t stack_refresh(pm_stack *s) {
  bool same = s->seen_gen.size() == s->layers.size();
  for (size_t i = 0; same && i < s->layers.size(); i++) same = s->seen_gen[i] == s->layers[i]->gen;
  if (same) return PM_OK;
  CU(cudaStreamSynchronize(s->ctx->stream));
  if (s->mega_layers) TRY(stack_fill_mega_layers(s));
  stack_drop_graphs(s);
  s->seen_gen.resize(s->layers.size());
  for (size_t i = 0; i < s->layers.size(); i++) s->seen_gen[i] = s->layers[i]->gen;
  return PM_OK;
}

static int32_t stack_setup_mega(pm_stack *s) {
  pm_ctx *c = s->ctx;
  const pm_layer_desc &D = s->layers[0]->dev.desc;
  for (pm_layer *ly : s->layers)
    if (memcmp(&ly->dev.desc, &D, sizeof D) != 0) return PM_OK;  // mixed shapes: general path
  cudaDeviceProp prop;
  CU(cudaGetDeviceProperties(&prop, c->device));
  int coop = 0;
  CU(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, c->device));
  if (!coop || prop.major < 9) return PM_OK;
  if (!mega_plan(D, prop.multiProcessorCount, prop.sharedMemPerBlockOptin, s->mega)) return PM_OK;
  CU(mega_prepare(D, s->mega.smem));
  if (mega_max_ctas_per_sm(D, s->mega.smem) < 1) return PM_OK;
  size_t L = s->layers.size();
  CU(cudaMalloc(&s->mega_layers, L * sizeof(MegaLayer)));
  TRY(stack_fill_mega_layers(s));
  // the three exchanges, two buffers each, of 64-bit (epoch, value) words; epoch 0 = never written
  size_t xb = al((size_t)D.d * 16), lb = al((size_t)D.n_exp * 16), hb = al((size_t)D.top_k * D.ff * 16);
  size_t fb = al(128 + (size_t)(D.top_k * D.ff / 256) * 128);  // the counters, a 128-byte line each
  size_t total = xb + lb + hb + fb + 512;
  CU(cudaMalloc(&s->mega_buf, total));
  CU(cudaMemset(s->mega_buf, 0, total));
  CU(cudaMalloc(&s->mega_io, (size_t)D.d * 4 * 2));
  MegaParams &P = s->mega.P;
  P.n_layers = (int)L;
  P.layers = s->mega_layers;
  P.eps = s->eps;
  P.xw = (unsigned long long *)s->mega_buf;
  P.lw = (unsigned long long *)(s->mega_buf + xb);
  P.hw = (unsigned long long *)(s->mega_buf + xb + lb);
  P.xcount = (unsigned long long *)(s->mega_buf + xb + lb + hb);
  P.hcount = (unsigned long long *)(s->mega_buf + xb + lb + hb + 128);
  P.err = (int *)(s->mega_buf + xb + lb + hb + fb + 256);
  s->mega_buf_bytes = total;
  s->mega_xw_bytes = xb + lb + hb;
  s->mega_ok = true;
  return PM_OK;
}

extern "C" int32_t pm_stack_create(pm_ctx *ctx, pm_layer **layers, int32_t n, float eps,
                                   pm_stack **out) {
  if (!ctx || !layers || n < 1 || !out) return fail(PM_ERR_INVALID, "pm_stack_create");
  for (int i = 0; i < n; i++) {
    if (!layers[i] || layers[i]->ctx != ctx) return fail(PM_ERR_INVALID, "layer %d: wrong context", i);
    if (layers[i]->dev.desc.d != layers[0]->dev.desc.d)
      return fail(PM_ERR_INVALID, "layer %d: hidden size differs", i);
  }
  CU(cudaSetDevice(ctx->device));
  pm_stack *s = new (std::nothrow) pm_stack();
  if (!s) return fail(PM_ERR_OOM, "host allocation");
  s->ctx = ctx;
  s->layers.assign(layers, layers + n);
  s->eps = eps;
  int32_t rc = stack_setup_mega(s);
  if (rc != PM_OK) {
    pm_stack_destroy(s);
    return rc;
  }
  for (pm_layer *ly : s->layers) s->seen_gen.push_back(ly->gen);
  *out = s;
  return PM_OK;
}
extern "C" int32_t pm_stack_destroy(pm_stack *s) {
  if (!s) return PM_OK;
  cudaSetDevice(s->ctx->device);
  cudaStreamSynchronize(s->ctx->stream);
  stack_drop_graphs(s);
  if (s->mega_layers) cudaFree(s->mega_layers);
  if (s->mega_buf) cudaFree(s->mega_buf);
  if (s->mega_io) cudaFree(s->mega_io);
  if (s->mega_trace) cudaFree(s->mega_trace);
  delete s;
  return PM_OK;
}
extern "C" int32_t pm_stack_set_mode(pm_stack *s, int32_t mode) {
  if (!s || mode < 0 || mode > 1) return fail(PM_ERR_INVALID, "pm_stack_set_mode");
  s->mode = mode;
  return PM_OK;
}
extern "C" int32_t pm_stack_decode_kernel_available(pm_stack *s) { return s && s->mega_ok ? 1 : 0; }

extern "C" int32_t pm_stack_trace(pm_stack *s, int64_t *out, int32_t capacity) {
  if (!s || !s->mega_ok) return fail(PM_ERR_STATE, "pm_stack_trace: no decode kernel for this stack");
  int n = s->mega.grid * (int)s->layers.size() * MG_TRACE_PH;
  if (!out) {  // switch tracing on
    if (!s->mega_trace) {
      CU(cudaMalloc(&s->mega_trace, (size_t)n * 8));
      CU(cudaMemset(s->mega_trace, 0, (size_t)n * 8));
    }
    s->mega.P.trace = s->mega_trace;
    return n;
  }
  if (!s->mega_trace || capacity < n) return fail(PM_ERR_INVALID, "pm_stack_trace: capacity %d < %d", capacity, n);
  CU(cudaStreamSynchronize(s->ctx->stream));
  CU(cudaMemcpy(out, s->mega_trace, (size_t)n * 8, cudaMemcpyDeviceToHost));
  return n;
}

extern "C" int32_t pm_debug_stack_fault_next_call(pm_stack *s) {
  if (!s || !s->mega_ok) return fail(PM_ERR_STATE, "pm_debug_stack_fault_next_call: no decode kernel for this stack");
  s->fault_next = true;
  return PM_OK;
}

extern "C" int32_t pm_stack_status(pm_stack *s) {
  if (!s) return fail(PM_ERR_INVALID, "pm_stack_status");
  CU(cudaStreamSynchronize(s->ctx->stream));
  if (!s->mega_buf) return PM_OK;
  int err = 0;
  CU(cudaMemcpy(&err, s->mega.P.err, 4, cudaMemcpyDeviceToHost));
  if (err) {
    s->mega_ok = false;
    return fail(PM_ERR_TIMEOUT, "decode kernel: a bounded device-side wait gave up (code %d)", err);
  }
  return PM_OK;
}

// one token through every layer in one persistent kernel
static int32_t stack_forward_mega(pm_stack *s, const float *x, float *x_out) {
  pm_ctx *c = s->ctx;
  const int d = s->layers[0]->dev.desc.d;
  MegaParams &P = s->mega.P;
  const float *xin = x;
  float *xo = x_out;
  if (!is_device_ptr(x)) {
    CU(cudaMemcpyAsync(s->mega_io, x, (size_t)d * 4, cudaMemcpyHostToDevice, c->stream));
    xin = s->mega_io;
  }
  bool out_host = !is_device_ptr(x_out);
  if (out_host) xo = s->mega_io + d;
  size_t L = s->layers.size();
  s->calls++;
  P.x_in = xin;
  P.x_out = xo;
  // epochs of this call: base + 1 .. base + L (32 bits; the words are cleared before they could repeat)
  if ((s->calls * (unsigned long long)L) >> 32 != ((s->calls - 1) * (unsigned long long)L) >> 32) {
    CU(cudaMemsetAsync(s->mega_buf, 0, s->mega_xw_bytes, c->stream));  // (the words only: the counters never repeat)
  }
  P.epoch_base = (uint32_t)((s->calls - 1) * (unsigned long long)L);
  P.count_base = (s->calls - 1) * (unsigned long long)L;
  P.xcount_base = (s->calls - 1) * (unsigned long long)(L - 1);
  P.wait_ns = c->wait_ns;
  P.fault = 0;
  if (s->fault_next) {  // test hook: the readers of h expect an epoch nobody writes
    P.fault = 1u;
    s->fault_next = false;
  }
  {
    PROF(c, PH_FUSED);
    CU(mega_launch(s->mega, c->stream));
    c->launches++;
    c->path_count[PM_PATH_DECODE]++;
  }
  if (out_host) {
    CU(cudaMemcpyAsync(x_out, xo, (size_t)d * 4, cudaMemcpyDeviceToHost, c->stream));
    int err = 0;
    CU(cudaMemcpyAsync(&err, P.err, 4, cudaMemcpyDeviceToHost, c->stream));
    CU(cudaStreamSynchronize(c->stream));
    if (err) {
      s->mega_ok = false;  // counters are no longer consistent: general kernels from now on
      return fail(PM_ERR_TIMEOUT, "decode kernel: a bounded device-side wait gave up (code %d)", err);
    }
  }
  return PM_OK;
}

extern "C" int32_t pm_stack_forward(pm_stack *s, const float *x, int32_t T, float *x_out) {
  if (!s || !x || !x_out) return fail(PM_ERR_INVALID, "pm_stack_forward: null argument");
  TRY(check_T(T));
  if (T == 0) return PM_OK;
  pm_ctx *c = s->ctx;
  CU(cudaSetDevice(c->device));
  for (pm_layer *ly : s->layers) TRY(layer_ready(ly, true));
  TRY(stack_refresh(s));
  if (T == 1 && s->mega_ok && s->mode == 0) return stack_forward_mega(s, x, x_out);
  const int d = s->layers[0]->dev.desc.d;
  size_t n = (size_t)T * d;
  size_t need = 0;
  for (pm_layer *ly : s->layers) {
    size_t b = scratch_bytes(ly->dev.desc, T);
    if (b > need) need = b;
  }
  TRY(ws_reserve(c, need + 3 * al(n * 4)));
  // ---- a few tokens: replay the recorded loop ----
  bool graphable = T <= 16 && !c->prof_on && !s->graph_off;
  for (pm_layer *ly : s->layers) graphable = graphable && ly->dev.desc.shared == PM_SHARED_NONE;
  if (graphable) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(c->stream, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) {
      cudaGetLastError();
      graphable = false;
    }
  }
  if (graphable) {
    pm_stack::Graph *g = nullptr;
    for (auto &q : s->graphs)
      if (q.T == T && q.ws == c->ws) g = &q;
    bool seen = false;
    for (int t : s->seen_T) seen = seen || t == T;
    if (!g && seen) {  // second call with this token count: record
      pm_stack::Graph q{T, c->ws, nullptr, nullptr, 0};
      CU(cudaMalloc(&q.gx, n * 4));
      float *xn = ws_take<float>(c, n);
      size_t mark = c->ws_off;
      int64_t l0 = c->launches;
      cudaGraph_t graph = nullptr;
      bool ok = cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
      int32_t rc = PM_OK;
      if (ok) {
        for (pm_layer *ly : s->layers) {
          c->ws_off = mark;
          Scratch S;
          scratch_carve(c, ly->dev.desc, T, S);
          launch_rmsnorm(c->launch(), q.gx, T, d, s->eps, xn);
          rc = dev_forward(ly, xn, T, q.gx, true, S);
          if (rc != PM_OK) break;
        }
        ok = cudaStreamEndCapture(c->stream, &graph) == cudaSuccess && rc == PM_OK && graph;
      }
      q.launches = c->launches - l0;
      c->launches = l0;
      if (ok) ok = cudaGraphInstantiate(&q.exec, graph, 0) == cudaSuccess;
      if (graph) cudaGraphDestroy(graph);
      if (ok) {
        s->graphs.push_back(q);
        g = &s->graphs.back();
      } else {  // not recordable here: the plain loop from now on
        cudaGetLastError();
        cudaFree(q.gx);
        s->graph_off = true;
        c->ws_off = 0;
      }
    }
    if (g) {
      CU(cudaMemcpyAsync(g->gx, x, n * 4, cudaMemcpyDefault, c->stream));
      CU(cudaGraphLaunch(g->exec, c->stream));
      c->launches += g->launches;
      CU(cudaMemcpyAsync(x_out, g->gx, n * 4, cudaMemcpyDefault, c->stream));
      if (!is_device_ptr(x_out)) CU(cudaStreamSynchronize(c->stream));
      return PM_OK;
    }
    if (!seen) s->seen_T.push_back(T);
    c->ws_off = 0;
  }
  // residual stream: in place in x_out when it is a device pointer
  float *xc = is_device_ptr(x_out) ? x_out : ws_take<float>(c, n);
  float *xn = ws_take<float>(c, n);
  if (xc != x) CU(cudaMemcpyAsync(xc, x, n * 4, cudaMemcpyDefault, c->stream));
  size_t mark = c->ws_off;
  for (pm_layer *ly : s->layers) {
    c->ws_off = mark;
    Scratch S;
    scratch_carve(c, ly->dev.desc, T, S);
    { PROF(c, PH_NORM); launch_rmsnorm(c->launch(), xc, T, d, s->eps, xn); }
    TRY(dev_forward(ly, xn, T, xc, true, S));
  }
  if (xc != x_out) {
    CU(cudaMemcpyAsync(x_out, xc, n * 4, cudaMemcpyDeviceToHost, c->stream));
    CU(cudaStreamSynchronize(c->stream));
  }
  return PM_OK;
}


// ---------------------------------------------------------------------------
// expert parallelism over NCCL (one rank per GPU; experts sharded by rank)
// ---------------------------------------------------------------------------
// NCCL is bound at run time (dlopen), so the library loads on hosts without it and a process
// that already carries an NCCL (a framework's) shares that copy. Only the calls below are used.
#include <dlfcn.h>

#include <chrono>

typedef struct ncclComm *pm_ncclComm_t;
typedef struct { char internal[128]; } pm_ncclUniqueId;
enum { PM_NCCL_INT8 = 0, PM_NCCL_UINT8 = 1, PM_NCCL_INT32 = 2, PM_NCCL_UINT32 = 3, PM_NCCL_FLOAT32 = 7 };
struct NcclApi {
  void *handle = nullptr;
  int (*GetUniqueId)(pm_ncclUniqueId *) = nullptr;
  int (*CommInitRank)(pm_ncclComm_t *, int, pm_ncclUniqueId, int) = nullptr;
  int (*CommDestroy)(pm_ncclComm_t) = nullptr;
  int (*CommAbort)(pm_ncclComm_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*Send)(const void *, size_t, int, int, pm_ncclComm_t, cudaStream_t) = nullptr;
  int (*Recv)(void *, size_t, int, int, pm_ncclComm_t, cudaStream_t) = nullptr;
  int (*AllGather)(const void *, void *, size_t, int, pm_ncclComm_t, cudaStream_t) = nullptr;
  int (*CommGetAsyncError)(pm_ncclComm_t, int *) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
};
static NcclApi g_nccl;

static int32_t nccl_load() {
  if (g_nccl.handle) return PM_OK;
  void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return fail(PM_ERR_COMM, "NCCL is not available: %s", dlerror());
  NcclApi a;
  a.handle = h;
#define PM_NCCL_SYM(field, name)                                                     \
  do {                                                                               \
    *(void **)(&a.field) = dlsym(h, name);                                           \
    if (!a.field) return fail(PM_ERR_COMM, "NCCL symbol %s is missing", name);       \
  } while (0)
  PM_NCCL_SYM(GetUniqueId, "ncclGetUniqueId");
  PM_NCCL_SYM(CommInitRank, "ncclCommInitRank");
  PM_NCCL_SYM(CommDestroy, "ncclCommDestroy");
  PM_NCCL_SYM(CommAbort, "ncclCommAbort");
  PM_NCCL_SYM(GroupStart, "ncclGroupStart");
  PM_NCCL_SYM(GroupEnd, "ncclGroupEnd");
  PM_NCCL_SYM(Send, "ncclSend");
  PM_NCCL_SYM(Recv, "ncclRecv");
  PM_NCCL_SYM(AllGather, "ncclAllGather");
  PM_NCCL_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
  PM_NCCL_SYM(GetErrorString, "ncclGetErrorString");
#undef PM_NCCL_SYM
  g_nccl = a;
  return PM_OK;
}
#define NC(call)                                                                                  \
  do {                                                                                            \
    int r_ = (call);                                                                              \
    if (r_ != 0) return fail(PM_ERR_COMM, "%s: %s (%s:%d)", #call, g_nccl.GetErrorString(r_), __FILE__, __LINE__); \
  } while (0)

struct pm_ep {
  pm_ctx *ctx = nullptr;   // the rank's context: routing, the rank's own tokens, the exchanges' stream
  uint8_t *ws2 = nullptr;  // a second workspace (swapped in for the rows received from the other ranks,
  size_t ws2_cap = 0;      // whose number is only known in mid-call, when the first one is in use)
  pm_ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  int32_t *d_cnt = nullptr;  // [W] pairs this rank sends to each rank, then [W*W] everybody's
  int32_t *h_cnt = nullptr;  // pinned copy of the [W*W] table
  cudaEvent_t ev = nullptr;
  int64_t timeout_ms = 60000;  // host watchdog on the counts (a peer that never enters the call)
  uint64_t stats[4] = {0, 0, 0, 0};  // last call: rows sent, rows received, bytes sent, bytes received
  // placement tables: slot of every expert of a layer (absent: expert e sits in slot e)
  struct Slots {
    std::vector<int32_t> host;
    int32_t *dev = nullptr;
  };
  std::map<pm_layer *, Slots> slots;
};

extern "C" int32_t pm_ep_unique_id(uint8_t *out) {
  if (!out) return fail(PM_ERR_INVALID, "pm_ep_unique_id: null argument");
  TRY(nccl_load());
  pm_ncclUniqueId id;
  NC(g_nccl.GetUniqueId(&id));
  memcpy(out, id.internal, 128);
  return PM_OK;
}

extern "C" int32_t pm_ep_destroy(pm_ep *ep) {
  if (!ep) return PM_OK;
  cudaSetDevice(ep->ctx->device);
  cudaError_t q = cudaStreamQuery(ep->ctx->stream);
  if (ep->comm) {
    // work still queued behind a peer that never came: abort instead of waiting for it
    if (q == cudaErrorNotReady) g_nccl.CommAbort(ep->comm);
    else g_nccl.CommDestroy(ep->comm);
  }
  cudaGetLastError();
  for (auto &kv : ep->slots)
    if (kv.second.dev) cudaFree(kv.second.dev);
  if (ep->ws2) cudaFree(ep->ws2);
  if (ep->d_cnt) cudaFree(ep->d_cnt);
  if (ep->h_cnt) cudaFreeHost(ep->h_cnt);
  if (ep->ev) cudaEventDestroy(ep->ev);
  delete ep;
  return PM_OK;
}

extern "C" int32_t pm_ep_init(pm_ctx *ctx, const uint8_t *unique_id, int32_t rank, int32_t world, pm_ep **out) {
  if (!ctx || !unique_id || !out || world < 1 || world > 64 || rank < 0 || rank >= world)
    return fail(PM_ERR_INVALID, "pm_ep_init: bad argument (rank %d of %d)", rank, world);
  TRY(nccl_load());
  CU(cudaSetDevice(ctx->device));
  pm_ep *ep = new (std::nothrow) pm_ep();
  if (!ep) return fail(PM_ERR_OOM, "host allocation");
  ep->ctx = ctx;
  ep->rank = rank;
  ep->world = world;
  cudaError_t e = cudaMalloc(&ep->d_cnt, (size_t)(world + world * world) * 4);
  if (e == cudaSuccess) e = cudaHostAlloc((void **)&ep->h_cnt, (size_t)world * world * 4, cudaHostAllocDefault);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ep->ev, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    pm_ep_destroy(ep);
    return fail(PM_ERR_CUDA, "pm_ep_init: %s", cudaGetErrorString(e));
  }
  pm_ncclUniqueId id;
  memcpy(id.internal, unique_id, 128);
  int r = g_nccl.CommInitRank(&ep->comm, world, id, rank);
  if (r != 0) {
    ep->comm = nullptr;
    pm_ep_destroy(ep);
    return fail(PM_ERR_COMM, "ncclCommInitRank: %s", g_nccl.GetErrorString(r));
  }
  *out = ep;
  return PM_OK;
}

extern "C" int32_t pm_ep_set_timeout_ms(pm_ep *ep, int64_t ms) {
  if (!ep || ms < 1) return fail(PM_ERR_INVALID, "pm_ep_set_timeout_ms");
  ep->timeout_ms = ms;
  return PM_OK;
}
static int32_t ep_comm_ok(pm_ep *ep);

// ---- usage-driven placement (the reference moves experts between VRAM and host memory by a decayed
// use score and rewrites its slot table, src/moe.rs:246-278,1965-2069; here the places are the ranks)
extern "C" int32_t pm_ep_set_slots(pm_ep *ep, pm_layer *ly, const int32_t *slot_of_expert) {
  if (!ep || !ly) return fail(PM_ERR_INVALID, "pm_ep_set_slots: null argument");
  pm_ctx *c = ep->ctx;
  if (ly->ctx != c) return fail(PM_ERR_INVALID, "pm_ep_set_slots: the layer belongs to another context");
  CU(cudaSetDevice(c->device));
  const int E = ly->dev.desc.n_exp;
  auto it = ep->slots.find(ly);
  if (!slot_of_expert) {  // back to expert e in slot e
    if (it != ep->slots.end()) {
      CU(cudaStreamSynchronize(c->stream));
      if (it->second.dev) cudaFree(it->second.dev);
      ep->slots.erase(it);
    }
    return PM_OK;
  }
  std::vector<char> seen((size_t)E, 0);
  for (int e = 0; e < E; e++) {
    const int32_t sl = slot_of_expert[e];
    if (sl < 0 || sl >= E || seen[(size_t)sl]) return fail(PM_ERR_INVALID, "pm_ep_set_slots: not a permutation of the %d slots", E);
    seen[(size_t)sl] = 1;
  }
  pm_ep::Slots &S = ep->slots[ly];
  if (!S.dev) CU(cudaMalloc(&S.dev, (size_t)E * 4));
  S.host.assign(slot_of_expert, slot_of_expert + E);
  CU(cudaStreamSynchronize(c->stream));  // earlier calls read the old table
  CU(cudaMemcpyAsync(S.dev, S.host.data(), (size_t)E * 4, cudaMemcpyHostToDevice, c->stream));
  CU(cudaStreamSynchronize(c->stream));
  return PM_OK;
}

extern "C" int32_t pm_ep_get_slots(pm_ep *ep, pm_layer *ly, int32_t *slot_of_expert) {
  if (!ep || !ly || !slot_of_expert) return fail(PM_ERR_INVALID, "pm_ep_get_slots: null argument");
  const int E = ly->dev.desc.n_exp;
  auto it = ep->slots.find(ly);
  for (int e = 0; e < E; e++) slot_of_expert[e] = it == ep->slots.end() ? e : it->second.host[(size_t)e];
  return PM_OK;
}

// the device regions of one slot of a sharded layer: every plane of the three matrices, and the biases
static void slot_regions(pm_layer *ly, int el, std::vector<std::pair<uint8_t *, size_t>> &out) {
  LayerDev &dv = ly->dev;
  WMat *ms[3] = {&dv.gate, &dv.up, &dv.down};
  for (WMat *m : ms)
    for (int p = 0; p < 4; p++)
      if (m->plane[p] && m->stride[p]) out.push_back({m->plane[p] + (size_t)el * m->stride[p], m->stride[p]});
  const int ff = dv.desc.ff, d = dv.desc.d;
  if (ly->bias_gate) out.push_back({(uint8_t *)(ly->bias_gate + (size_t)el * ff), (size_t)ff * 4});
  if (ly->bias_up) out.push_back({(uint8_t *)(ly->bias_up + (size_t)el * ff), (size_t)ff * 4});
  if (ly->bias_down) out.push_back({(uint8_t *)(ly->bias_down + (size_t)el * d), (size_t)d * 4});
}

// Collective: experts a and b of the layer change places. The ranks that hold them exchange the
// experts' bytes (every plane of gate, up and down, and the biases) through a staging area, every rank
// rewrites its table. All ranks call it with the same arguments in the same order.
extern "C" int32_t pm_ep_swap_experts(pm_ep *ep, pm_layer *ly, int32_t expert_a, int32_t expert_b) {
  if (!ep || !ly) return fail(PM_ERR_INVALID, "pm_ep_swap_experts: null argument");
  pm_ctx *c = ep->ctx;
  if (ly->ctx != c) return fail(PM_ERR_INVALID, "pm_ep_swap_experts: the layer belongs to another context");
  const LayerDev &dv = ly->dev;
  const int E = dv.desc.n_exp, W = ep->world, rank = ep->rank;
  if (E % W) return fail(PM_ERR_INVALID, "%d experts do not split over %d ranks", E, W);
  const int per = E / W;
  if (dv.first_local != rank * per || dv.n_local != per)
    return fail(PM_ERR_INVALID, "pm_ep_swap_experts: the layer does not hold this rank's slots");
  if (expert_a < 0 || expert_a >= E || expert_b < 0 || expert_b >= E) return fail(PM_ERR_INVALID, "pm_ep_swap_experts: expert id");
  if (expert_a == expert_b) return PM_OK;
  CU(cudaSetDevice(c->device));
  pm_ep::Slots &S = ep->slots[ly];
  if (S.host.empty()) {
    S.host.resize((size_t)E);
    for (int e = 0; e < E; e++) S.host[(size_t)e] = e;
  }
  if (!S.dev) CU(cudaMalloc(&S.dev, (size_t)E * 4));
  const int sa = S.host[(size_t)expert_a], sb = S.host[(size_t)expert_b];
  const int ra = sa / per, rb = sb / per;
  std::vector<std::pair<uint8_t *, size_t>> mine, other;
  size_t bytes = 0;
  if (ra == rank) slot_regions(ly, sa - rank * per, mine);
  if (rb == rank) slot_regions(ly, sb - rank * per, ra == rank ? other : mine);
  for (auto &r : mine) bytes += al(r.second);
  if (ra == rank || rb == rank) {
    TRY(stage_reserve(c, bytes));
    uint8_t *tmp = c->stage;
    if (ra == rank && rb == rank) {  // both here: through the staging area
      size_t o = 0;
      for (size_t i = 0; i < mine.size(); i++) {
        CU(cudaMemcpyAsync(tmp + o, mine[i].first, mine[i].second, cudaMemcpyDeviceToDevice, c->stream));
        CU(cudaMemcpyAsync(mine[i].first, other[i].first, mine[i].second, cudaMemcpyDeviceToDevice, c->stream));
        CU(cudaMemcpyAsync(other[i].first, tmp + o, mine[i].second, cudaMemcpyDeviceToDevice, c->stream));
        o += al(mine[i].second);
      }
    } else {  // send this rank's expert, receive the peer's into the staging area, then put it in the slot
      const int peer = ra == rank ? rb : ra;
      TRY(ep_comm_ok(ep));
      NC(g_nccl.GroupStart());
      size_t o = 0;
      for (auto &r : mine) {
        NC(g_nccl.Send(r.first, r.second, PM_NCCL_UINT8, peer, ep->comm, c->stream));
        NC(g_nccl.Recv(tmp + o, r.second, PM_NCCL_UINT8, peer, ep->comm, c->stream));
        o += al(r.second);
      }
      NC(g_nccl.GroupEnd());
      o = 0;
      for (auto &r : mine) {
        CU(cudaMemcpyAsync(r.first, tmp + o, r.second, cudaMemcpyDeviceToDevice, c->stream));
        o += al(r.second);
      }
    }
  }
  std::swap(S.host[(size_t)expert_a], S.host[(size_t)expert_b]);
  CU(cudaMemcpyAsync(S.dev, S.host.data(), (size_t)E * 4, cudaMemcpyHostToDevice, c->stream));
  CU(cudaStreamSynchronize(c->stream));
  ly->gen++;
  return ep_comm_ok(ep);
}

extern "C" int32_t pm_ep_last_stats(pm_ep *ep, uint64_t *out) {
  if (!ep || !out) return fail(PM_ERR_INVALID, "pm_ep_last_stats");
  for (int i = 0; i < 4; i++) out[i] = ep->stats[i];
  return PM_OK;
}

static int32_t ep_comm_ok(pm_ep *ep) {
  int ae = 0;
  NC(g_nccl.CommGetAsyncError(ep->comm, &ae));
  if (ae != 0) return fail(PM_ERR_COMM, "NCCL reported an asynchronous error: %s", g_nccl.GetErrorString(ae));
  return PM_OK;
}

// y[T][d] for this rank's T tokens; the layer holds experts [rank * E / W, (rank + 1) * E / W).
// Per call: route and plan the rank's tokens; every rank learns every rank's per-destination pair
// counts (one small all-gather, read by the host while the shared expert runs); the pairs' rows go
// to the ranks that hold their experts in their quantised wire form (Q8x: int8 + scales + group
// sums, 3.5 times fewer bytes than f32; sender-side quantisation is the same pure function the
// receiver would apply) together with (expert, weight); the rows received run through the local
// experts; the outputs travel back and are combined in k order with the shared expert's.
extern "C" int32_t pm_moe_forward_ep(pm_ep *ep, pm_layer *ly, const float *x, int32_t T, float *y, uint32_t flags) {
  if (!ep || !ly) return fail(PM_ERR_INVALID, "pm_moe_forward_ep: null argument");
  TRY(layer_ready(ly, true));
  TRY(check_T(T));
  pm_ctx *c = ep->ctx;
  if (ly->ctx != c) return fail(PM_ERR_INVALID, "pm_moe_forward_ep: the layer belongs to another context");
  const LayerDev &dv = ly->dev;
  const pm_layer_desc &D = dv.desc;
  const int W = ep->world, rank = ep->rank, E = D.n_exp, K = D.top_k, d = D.d;
  if (E % W) return fail(PM_ERR_INVALID, "%d experts do not split over %d ranks", E, W);
  const int per = E / W;
  if (dv.first_local != rank * per || dv.n_local != per)
    return fail(PM_ERR_INVALID, "rank %d of %d must hold experts [%d, %d); the layer holds [%d, %d)", rank, W, rank * per,
                (rank + 1) * per, dv.first_local, dv.first_local + dv.n_local);
  if (T > 0 && (!x || !y || !is_device_ptr(x) || !is_device_ptr(y)))
    return fail(PM_ERR_INVALID, "pm_moe_forward_ep: x and y must be device pointers");
  CU(cudaSetDevice(c->device));
  const bool q8 = D.act_quant == PM_AQ_Q8X_256;
  const size_t P = (size_t)T * K;
  const int nd = q8 ? d / 256 : 0, nbs = q8 ? d / 32 : 0;
  const size_t row_bytes = q8 ? (size_t)d : (size_t)d * 4;  // wire form of a row: int8 (Q8x) or f32
  Launch L = c->launch();

  // ---- this rank's tokens: route, plan, counts ----
  TRY(ws_reserve(c, scratch_bytes(D, T > 0 ? T : 1) + al(P * row_bytes) + al(P * (nd + 1) * 4) + al(P * (nbs + 1) * 4) +
                        al(P * 8) + 4096));
  Scratch S;
  scratch_carve(c, D, T > 0 ? T : 1, S);
  uint8_t *srows = ws_take<uint8_t>(c, P * row_bytes);
  float *sd = ws_take<float>(c, P * (size_t)(nd + 1));
  int32_t *sbs = ws_take<int32_t>(c, P * (size_t)(nbs + 1));
  uint32_t *smeta = ws_take<uint32_t>(c, P * 2);
  if (T > 0 && T < PM_SMALL_ROUTE_TOKENS) {  // a few tokens: logits, top-k, (slots) and plan in one launch
    auto st = ep->slots.find(ly);
    PROF(c, PH_ROUTER);
    launch_route_plan_small(L, dv, x, T, S.logits, S.ids, S.w, S.plan, st != ep->slots.end() ? st->second.dev : nullptr,
                            c->route_ticket);
  } else {
    if (T > 0) {
      { PROF(c, PH_ROUTER); launch_router(L, dv, x, T, S.logits); }
      { PROF(c, PH_ROUTE); launch_route(L, dv, S.logits, T, S.ids, S.w); }
    }
    // with a placement table everything from here on names slots: the plan groups by slot, a pair goes
    // to the rank of its slot, the serving rank indexes its planes by slot
    auto st = ep->slots.find(ly);
    LayerDev dvp = dv;
    if (st != ep->slots.end()) {
      launch_ep_slots(L, S.ids, (int)P, E, st->second.dev, dv.usage);
      dvp.usage = nullptr;  // counted by expert above
    }
    PROF(c, PH_PLAN);
    launch_plan(L, dvp, S.ids, T, S.plan, c->dev_err);
  }
  launch_ep_rank_counts(L, S.plan.cnt, E, W, ep->d_cnt);
  NC(g_nccl.AllGather(ep->d_cnt, ep->d_cnt + W, (size_t)W, PM_NCCL_INT32, ep->comm, c->stream));
  CU(cudaMemcpyAsync(ep->h_cnt, ep->d_cnt + W, (size_t)W * W * 4, cudaMemcpyDeviceToHost, c->stream));
  CU(cudaEventRecord(ep->ev, c->stream));
  // ---- meanwhile on the GPU: the rows' wire form and the shared expert ----
  if (T > 0) {
    if (q8) { PROF(c, PH_QUANT_X); launch_quant_q8x(L, x, (size_t)T, d, S.xq, S.xd, S.xbsum, S.xbm, S.xs); }
    launch_ep_pack(L, (int)P, (int)row_bytes, nd, nbs, q8 ? (const void *)S.xq : (const void *)x, S.xd, S.xbsum,
                   S.plan.pair_token, S.plan.pair_src, S.ids, S.w, srows, sd, sbs, smeta);
    TRY(dev_shared(ly, x, T, S));
  }
  // ---- the host learns the counts (bounded: a peer that never enters the call shows here) ----
  {
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
      cudaError_t q = cudaEventQuery(ep->ev);
      if (q == cudaSuccess) break;
      if (q != cudaErrorNotReady) return fail(PM_ERR_CUDA, "pm_moe_forward_ep: %s", cudaGetErrorString(q));
      TRY(ep_comm_ok(ep));
      if (std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() > ep->timeout_ms)
        return fail(PM_ERR_TIMEOUT, "pm_moe_forward_ep: the ranks' pair counts did not arrive within %lld ms "
                                    "(a rank that did not enter the call?)", (long long)ep->timeout_ms);
    }
  }
  std::vector<size_t> scnt(W), soff(W), rcnt(W), roff(W);
  size_t R = 0, so = 0;
  for (int j = 0; j < W; j++) {
    scnt[j] = (size_t)ep->h_cnt[rank * W + j];
    rcnt[j] = (size_t)ep->h_cnt[j * W + rank];
    soff[j] = so;
    roff[j] = R;
    so += scnt[j];
    R += rcnt[j];
  }
  if (so != P) return fail(PM_ERR_STATE, "pm_moe_forward_ep: %zu pairs planned, %zu counted", P, so);
  if (R > (size_t)PM_MAX_TOKENS * PM_MAX_TOPK) return fail(PM_ERR_LIMIT, "pm_moe_forward_ep: %zu rows received", R);

  // ---- the rows this rank serves: the second workspace is swapped in (its size is only known
  // now, and what was carved from the first one is still in use) ----
  struct WsSwap {
    pm_ctx *c;
    pm_ep *ep;
    size_t off;
    WsSwap(pm_ctx *c_, pm_ep *e_) : c(c_), ep(e_), off(c_->ws_off) { std::swap(c->ws, ep->ws2); std::swap(c->ws_cap, ep->ws2_cap); }
    ~WsSwap() { std::swap(c->ws, ep->ws2); std::swap(c->ws_cap, ep->ws2_cap); c->ws_off = off; }
  } ws_swap(c, ep);
  pm_layer_desc D1 = D;
  D1.top_k = 1;
  const size_t Rr = R > 0 ? R : 1;
  TRY(ws_reserve(c, scratch_bytes(D1, (int)Rr) + al(Rr * row_bytes) + al(Rr * 8) + 2 * al(Rr * 4) + al(Rr * (size_t)d * 4) + 4096));
  Scratch RS;
  scratch_carve(c, D1, (int)Rr, RS);
  uint8_t *rrows = q8 ? (uint8_t *)RS.xq : ws_take<uint8_t>(c, Rr * row_bytes);
  uint32_t *rmeta = ws_take<uint32_t>(c, Rr * 2);
  uint32_t *reid = ws_take<uint32_t>(c, Rr);
  float *rw = ws_take<float>(c, Rr);
  float *orows = ws_take<float>(c, Rr * (size_t)d);

  // ---- dispatch ----
  {
    PROF(c, PH_FUSED);
    NC(g_nccl.GroupStart());
    for (int j = 0; j < W; j++) {
      if (j == rank) continue;
      if (scnt[j]) {
        NC(g_nccl.Send(srows + soff[j] * row_bytes, scnt[j] * row_bytes, PM_NCCL_UINT8, j, ep->comm, c->stream));
        NC(g_nccl.Send(smeta + soff[j] * 2, scnt[j] * 2, PM_NCCL_UINT32, j, ep->comm, c->stream));
        if (q8) {
          NC(g_nccl.Send(sd + soff[j] * nd, scnt[j] * nd, PM_NCCL_FLOAT32, j, ep->comm, c->stream));
          NC(g_nccl.Send(sbs + soff[j] * nbs, scnt[j] * nbs, PM_NCCL_INT32, j, ep->comm, c->stream));
        }
      }
      if (rcnt[j]) {
        NC(g_nccl.Recv(rrows + roff[j] * row_bytes, rcnt[j] * row_bytes, PM_NCCL_UINT8, j, ep->comm, c->stream));
        NC(g_nccl.Recv(rmeta + roff[j] * 2, rcnt[j] * 2, PM_NCCL_UINT32, j, ep->comm, c->stream));
        if (q8) {
          NC(g_nccl.Recv(RS.xd + roff[j] * nd, rcnt[j] * nd, PM_NCCL_FLOAT32, j, ep->comm, c->stream));
          NC(g_nccl.Recv(RS.xbsum + roff[j] * nbs, rcnt[j] * nbs, PM_NCCL_INT32, j, ep->comm, c->stream));
        }
      }
    }
    NC(g_nccl.GroupEnd());
    if (scnt[rank]) {  // the pairs that stay on this rank
      const size_t o = soff[rank], r0 = roff[rank], n = scnt[rank];
      CU(cudaMemcpyAsync(rrows + r0 * row_bytes, srows + o * row_bytes, n * row_bytes, cudaMemcpyDeviceToDevice, c->stream));
      CU(cudaMemcpyAsync(rmeta + r0 * 2, smeta + o * 2, n * 8, cudaMemcpyDeviceToDevice, c->stream));
      if (q8) {
        CU(cudaMemcpyAsync(RS.xd + r0 * nd, sd + o * nd, n * nd * 4, cudaMemcpyDeviceToDevice, c->stream));
        CU(cudaMemcpyAsync(RS.xbsum + r0 * nbs, sbs + o * nbs, n * nbs * 4, cudaMemcpyDeviceToDevice, c->stream));
      }
    }
  }
  // ---- the local experts over the received rows ----
  if (R > 0) {
    launch_ep_unmeta(L, (int)R, rmeta, dv.first_local, dv.n_local, reid, rw, c->dev_err);
    if (q8) launch_q8x_aux(L, R * (size_t)nd, RS.xbsum, RS.xbm, RS.xs);
    pm_layer view = *ly;
    view.dev.desc = D1;
    view.dev.usage = nullptr;
    { PROF(c, PH_PLAN); launch_plan(L, view.dev, reid, (int)R, RS.plan, c->dev_err); }
    TRY(dev_experts(&view, q8 ? nullptr : (const float *)rrows, (int)R, RS, rw, q8));
    LayerDev cp = view.dev;
    cp.desc.weight_fold = PM_FOLD_BEFORE_DOWN;  // plain gather back to row order
    launch_combine(L, cp, RS.eo, RS.plan.pair_pos, rw, nullptr, nullptr, (int)R, orows, false);
  }
  // ---- the outputs go home (they arrive in the sender's plan order: S.eo is what combine takes) ----
  {
    PROF(c, PH_FUSED);
    NC(g_nccl.GroupStart());
    for (int j = 0; j < W; j++) {
      if (j == rank) continue;
      if (rcnt[j]) NC(g_nccl.Send(orows + roff[j] * d, rcnt[j] * (size_t)d, PM_NCCL_FLOAT32, j, ep->comm, c->stream));
      if (scnt[j]) NC(g_nccl.Recv(S.eo + soff[j] * d, scnt[j] * (size_t)d, PM_NCCL_FLOAT32, j, ep->comm, c->stream));
    }
    NC(g_nccl.GroupEnd());
    if (scnt[rank])
      CU(cudaMemcpyAsync(S.eo + soff[rank] * d, orows + roff[rank] * d, scnt[rank] * (size_t)d * 4, cudaMemcpyDeviceToDevice,
                         c->stream));
  }
  if (T > 0) {
    PROF(c, PH_COMBINE);
    launch_combine(L, dv, S.eo, S.plan.pair_pos, S.w, S.shared_out, S.shared_logit, T, y, (flags & PM_FWD_ACCUMULATE) != 0);
  }
  CU(cudaGetLastError());
  ep->stats[0] = P - scnt[rank];
  ep->stats[1] = R - rcnt[rank];
  const size_t per_row = row_bytes + 8 + (size_t)nd * 4 + (size_t)nbs * 4;
  ep->stats[2] = (P - scnt[rank]) * per_row + (R - rcnt[rank]) * (size_t)d * 4;
  ep->stats[3] = (R - rcnt[rank]) * per_row + (P - scnt[rank]) * (size_t)d * 4;
  return ep_comm_ok(ep);
}
