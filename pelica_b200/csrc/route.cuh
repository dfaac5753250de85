// route.cuh - one token's top-k experts and routing weights by one warp
// (src/moe_kernels.rs:1019-1081, src/oss_kernels.rs:15-35, src/ds4.rs:1371-1426,
// src/q4x.rs:2213-2231). Shared by the general kernel and the decode kernel so
// both give the same bits.
#pragma once

#include "common.cuh"

#define NPER (PM_MAX_EXPERTS / 32)

// lane L holds experts L, L+32, ...; `lg` points at the token's E logits (any
// address space); ssv[E], gsc[E/2], keep[E/2] are per-warp scratch in shared
// memory (used for group-limited selection only). Lane 0 writes ids_out[K],
// w_out[K].
__device__ __forceinline__ void pm_route_warp(const pm_layer_desc &D, const float *lg,
                                              const float *__restrict__ sel_bias, int lane,
                                              float *ssv, float *gsc, unsigned char *keep,
                                              uint32_t *ids_out, float *w_out) {
  const int E = D.n_exp, K = D.top_k;
  float pr[NPER], sv[NPER];
  float mx = PM_NEG;
#pragma unroll
  for (int i = 0; i < NPER; i++) {
    int e = lane + 32 * i;
    float v = e < E ? lg[e] : PM_NEG;
    pr[i] = v;
    mx = fmaxf(mx, v);
  }
  if (D.gating == PM_GATE_SOFTMAX_ALL) {
    mx = pm_warp_max(mx);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < NPER; i++) {
      int e = lane + 32 * i;
      if (e < E) {
        pr[i] = pm_exp(__fsub_rn(pr[i], mx));
        sum = __fadd_rn(sum, pr[i]);
      }
    }
    sum = pm_warp_sum_16_1(sum);
#pragma unroll
    for (int i = 0; i < NPER; i++) pr[i] = __fdiv_rn(pr[i], sum);
  } else if (D.gating == PM_GATE_SIGMOID) {
#pragma unroll
    for (int i = 0; i < NPER; i++)
      if (lane + 32 * i < E) pr[i] = __fdiv_rn(1.0f, __fadd_rn(1.0f, pm_exp(-pr[i])));
  } else if (D.gating == PM_GATE_SQRT_SOFTPLUS) {
#pragma unroll
    for (int i = 0; i < NPER; i++)
      if (lane + 32 * i < E) {
        float v = pr[i];
        float sp = v > 20.0f ? v : pm_log1p(pm_exp(v));
        pr[i] = __fsqrt_rn(sp);
      }
  }
#pragma unroll
  for (int i = 0; i < NPER; i++) {
    int e = lane + 32 * i;
    sv[i] = e < E ? (sel_bias ? __fadd_rn(pr[i], sel_bias[e]) : pr[i]) : PM_NEG;
  }
  // group-limited selection (this repository's definition: group score = sum of
  // the group's two largest biased scores; best topk_group groups stay, ties ->
  // lower group index)
  if (D.n_group > 0) {
#pragma unroll
    for (int i = 0; i < NPER; i++)
      if (lane + 32 * i < E) ssv[lane + 32 * i] = sv[i];
    __syncwarp();
    const int G = D.n_group, gs = E / G;
    for (int g = lane; g < G; g += 32) {  // lane g scores groups g, g+32, ...
      int i1 = 0;
      float v1 = ssv[g * gs];
      for (int i = 1; i < gs; i++)
        if (ssv[g * gs + i] > v1) { v1 = ssv[g * gs + i]; i1 = i; }
      float v2 = PM_NEG;
      for (int i = 0; i < gs; i++)
        if (i != i1 && ssv[g * gs + i] > v2) v2 = ssv[g * gs + i];
      gsc[g] = __fadd_rn(v1, v2);
      keep[g] = 0;
    }
    __syncwarp();
    if (lane == 0) {
      for (int r = 0; r < D.topk_group; r++) {
        int bg = -1;
        float bv = 0.0f;
        for (int g = 0; g < G; g++) {
          if (keep[g]) continue;
          float v = gsc[g];
          if (bg < 0 || v > bv) { bv = v; bg = g; }
        }
        keep[bg] = 1;
      }
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < NPER; i++) {
      int e = lane + 32 * i;
      if (e < E && !keep[e / gs]) sv[i] = PM_NEG;
    }
  }
  // K rounds of (max, lowest index)
  float tw[PM_MAX_TOPK];
  uint32_t te[PM_MAX_TOPK];
  float wsum = 0.0f;
#pragma unroll 1
  for (int k = 0; k < K; k++) {
    float bv = PM_NEG;
    uint32_t bi = 0xffffffffu;
#pragma unroll
    for (int i = 0; i < NPER; i++) {
      int e = lane + 32 * i;
      if (e < E && (bi == 0xffffffffu || sv[i] > bv)) { bv = sv[i]; bi = (uint32_t)e; }
    }
    float m = pm_warp_max(bi == 0xffffffffu ? PM_NEG : bv);
    uint32_t e = pm_warp_min_u32((bi != 0xffffffffu && bv == m) ? bi : 0xffffffffu);
    float mine = 0.0f;
#pragma unroll
    for (int i = 0; i < NPER; i++)
      if ((uint32_t)(lane + 32 * i) == e) { mine = pr[i]; sv[i] = PM_NEG; }
    // only the owning lane has a non-zero `mine`; a shuffle fetches it exactly
    float w = __shfl_sync(PM_FULL, mine, e & 31);
    te[k] = e;
    tw[k] = w;
    wsum = __fadd_rn(wsum, w);
  }
  if (lane == 0) {
    if (D.gating == PM_GATE_SOFTMAX_SELECTED) {  // src/oss_kernels.rs:31-32
      float ev[PM_MAX_TOPK];
      float sum = 0.0f;
      for (int k = 0; k < K; k++) {
        ev[k] = pm_exp(__fsub_rn(tw[k], tw[0]));
        sum = __fadd_rn(sum, ev[k]);
      }
      for (int k = 0; k < K; k++) {
        float x = __fdiv_rn(ev[k], sum);
        if (D.w_scale != 0.0f) x = __fmul_rn(x, D.w_scale);
        tw[k] = x;
      }
    } else if (D.gating == PM_GATE_SQRT_SOFTPLUS) {  // src/ds4.rs:1416-1424
      for (int k = 0; k < K; k++) {
        float x = __fdiv_rn(tw[k], wsum);
        if (D.w_scale != 0.0f) x = __fmul_rn(x, D.w_scale);
        tw[k] = x;
      }
    } else {  // src/moe_kernels.rs:1072-1074
      for (int k = 0; k < K; k++) {
        float x = tw[k];
        if (D.norm_w) x = __fdiv_rn(x, fmaxf(wsum, 6.103515625e-5f));
        if (D.w_scale != 0.0f) x = __fmul_rn(x, D.w_scale);
        tw[k] = x;
      }
    }
    for (int k = 0; k < K; k++) {
      ids_out[k] = te[k];
      w_out[k] = tw[k];
    }
  }
}
