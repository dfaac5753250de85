// decode_mega.cuh - parameters of the persistent one-token decode kernel.
#pragma once

#include "moe_internal.cuh"

#define MG_NT 512
#define MG_WARPS (MG_NT / 32)
#define MG_GU_CHUNKS 4
#define MG_TRACE_PH 20  // trace points per layer

struct MegaLayer {
  const float *router, *logit_bias, *select_bias;
  const uint8_t *gate, *up;
  size_t gate_stride, up_stride;
  const uint8_t *down[4];
  size_t down_stride[4];
  uint32_t *usage;
};

struct MegaParams {
  pm_layer_desc D;
  int n_layers;
  const MegaLayer *layers;
  const float *x_in;
  float *x_out;
  float eps;
  float *xbuf;               // [d]      the residual stream between layers
  unsigned long long *lbuf;  // [E]      the layer's router logits: (epoch << 32) | float bits
  float *hbuf;               // [K*ff]
  // arrival counters (never reset: each call waits for base + its own arrivals):
  unsigned long long *hcount;  // CTAs that finished their h rows
  unsigned long long *xcount;  // CTAs that published their slice of the next layer's residual stream
  unsigned long long hcount_base, xcount_base;
  uint32_t lepoch_base;  // epochs before this call: (calls - 1) * layers
  int *err;
  unsigned long long wait_ns;  // limit of every bounded wait
  long long *trace;  // optional [2][n_layers][MG_TRACE_PH] SM clocks (CTA 0 and the last CTA)
  // shared-memory layout (bytes from the dynamic base)
  int rows_max, cols_max;
  uint32_t off_gs, off_us, off_dn, off_dsm, off_xs, off_xq, off_xd, off_xbs, off_hq, off_hd,
      off_hbs, off_rw, off_eo, off_lg, off_misc, off_ml, dn_k_bytes, dsm_k_bytes;
};

struct MegaPlan {
  bool ok = false;
  int grid = 0;
  size_t smem = 0;
  MegaParams P{};
};


bool mega_plan(const pm_layer_desc &D, int n_sm, size_t smem_optin, MegaPlan &mp);
cudaError_t mega_prepare(const pm_layer_desc &D, size_t smem);
int mega_max_ctas_per_sm(const pm_layer_desc &D, size_t smem);
cudaError_t mega_launch(const MegaPlan &mp, cudaStream_t stream);
