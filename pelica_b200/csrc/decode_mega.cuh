// decode_mega.cuh - parameters of the persistent one-token decode kernel.
#pragma once

#include "moe_internal.cuh"

#define MG_NT 512
#define MG_WARPS (MG_NT / 32)
#define MG_CW (MG_WARPS - 1)  // warps that run gate/up passes; the last warp routes and issues the down copies
#define MG_GU_CHUNKS 4
// the down slices of the first / second half of the expert slots are requested once this gate/up
// chunk has landed (the gate/up bytes are needed first; the down bytes are not needed before h
// has gone round, but HBM should not idle for long either)
#ifndef MG_DN_TRIG0
#define MG_DN_TRIG0 2
#endif
#ifndef MG_DN_TRIG1
#define MG_DN_TRIG1 3
#endif
#define MG_TRACE_PH 16        // stamps per layer

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
  // The three all-CTA exchanges of a layer. Every word is (epoch << 32) | float bits, written
  // with one relaxed 64-bit store and polled by its readers until it carries the layer's epoch:
  // no counter, no release fence. Two buffers each, alternating by layer.
  unsigned long long *xw;  // [2][d]    the residual stream entering a layer
  unsigned long long *lw;  // [2][E]    the layer's router logits
  unsigned long long *hw;  // [2][K*ff] the layer's hidden values (activation applied, weight folded)
  // arrival counters, never reset (a call waits for count_base + its own arrivals), bumped without
  // a release: what a reader polls before it reads the words, which carry the epoch themselves
  unsigned long long *xcount;  // [1]       CTAs that published their columns of the next layer's x
  unsigned long long *hcount;  // [K*ff/256] per 256-value block of h: CTAs that produced their rows of it
  unsigned long long count_base;   // layers run by earlier calls: (calls - 1) * layers
  unsigned long long xcount_base;  // residual hand-offs of earlier calls: (calls - 1) * (layers - 1)
  uint32_t epoch_base;     // epochs used by earlier calls: (calls - 1) * layers
  uint32_t fault;          // test hook: the readers of h wait for this many extra arrivals in layer 0
  int *err;
  unsigned long long wait_ns;  // limit of every bounded wait
  unsigned long long *trace;   // optional [grid][n_layers][MG_TRACE_PH] global-timer stamps (ns)
  // shared-memory layout (bytes from the dynamic base)
  int rows_max, cols_max;
  uint32_t off_gs, off_us, off_dn, off_dsm, off_xs, off_xq, off_xd, off_xbs, off_hq, off_hd,
      off_hbs, off_rw, off_tmp, off_lg, off_misc, off_ml, dn_k_bytes, dsm_k_bytes;
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
