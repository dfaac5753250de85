// route.cuh - one token's top-k experts and routing weights by one warp
// (src/moe_kernels.rs:1019-1081, src/oss_kernels.rs:15-35, src/ds4.rs:1371-1426,
// src/q4x.rs:2213-2231). Shared by the general kernel and the decode kernel so
// both give the same bits.
#pragma once

#include "common.cuh"

// float -> unsigned key with the same order (finite values; -0 is folded onto
// +0 first so that equal floats get equal keys). Maxima over keys are maxima
// over the floats, bit for bit.
__device__ __forceinline__ uint32_t pm_fkey(float v) {
  uint32_t u = __float_as_uint(__fadd_rn(v, 0.0f));
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float pm_funkey(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// lane L holds experts L, L+32, ... (NP per lane, NP*32 >= E); `lg` points at the
// token's E logits (any address space); ssv[E], gsc[E/2], keep[E/2] are per-warp
// scratch in shared memory (used for group-limited selection only). Lane k < K
// writes ids_out[k], w_out[k].
// Scores of one token by one warp. lane L holds experts L, L+32, ... (NP per lane,
// NP*32 >= E); `lg` points at the token's E logits (any address space); ssv[E],
// gsc[E/2], keep[E/2] are per-warp scratch in shared memory (group-limited
// selection only). Out: pr[] = the score the weight is taken from, key[] = the
// ordered key of what the selection ranks (score + bias, masked groups lowest).
template <int NP>
__device__ __forceinline__ void pm_route_scores(const pm_layer_desc &D, const float *lg,
                                                const float *__restrict__ sel_bias, int lane,
                                                float *ssv, float *gsc, unsigned char *keep,
                                                float pr[NP], uint32_t key[NP]) {
  const int E = D.n_exp;
  float sv[NP];
#pragma unroll
  for (int i = 0; i < NP; i++) {
    int e = lane + 32 * i;
    pr[i] = e < E ? lg[e] : PM_NEG;
  }
  if (D.gating == PM_GATE_SOFTMAX_ALL) {  // src/moe_kernels.rs:1023-1042
    float mx = PM_NEG;
#pragma unroll
    for (int i = 0; i < NP; i++) mx = fmaxf(mx, pr[i]);
    mx = pm_funkey(__reduce_max_sync(PM_FULL, pm_fkey(mx)));
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < NP; i++) {
      if (lane + 32 * i < E) {
        pr[i] = pm_exp(__fsub_rn(pr[i], mx));
        sum = __fadd_rn(sum, pr[i]);
      }
    }
    sum = pm_warp_sum_16_1(sum);
#pragma unroll
    for (int i = 0; i < NP; i++) pr[i] = __fdiv_rn(pr[i], sum);
  } else if (D.gating == PM_GATE_SIGMOID) {  // src/moe_kernels.rs:1034
#pragma unroll
    for (int i = 0; i < NP; i++)
      if (lane + 32 * i < E) pr[i] = __fdiv_rn(1.0f, __fadd_rn(1.0f, pm_exp(-pr[i])));
  } else if (D.gating == PM_GATE_SQRT_SOFTPLUS) {  // src/ds4.rs:1377-1379
#pragma unroll
    for (int i = 0; i < NP; i++)
      if (lane + 32 * i < E) {
        float v = pr[i];
        float sp = v > 20.0f ? v : pm_log1p(pm_exp(v));
        pr[i] = __fsqrt_rn(sp);
      }
  }
  // what the selection ranks: score (+ bias) (src/moe_kernels.rs:1044-1049)
#pragma unroll
  for (int i = 0; i < NP; i++) {
    int e = lane + 32 * i;
    sv[i] = e < E ? (sel_bias ? __fadd_rn(pr[i], sel_bias[e]) : pr[i]) : PM_NEG;
  }
  // group-limited selection (this repository's definition: group score = sum of
  // the group's two largest biased scores; best topk_group groups stay, ties ->
  // lower group index)
  if (D.n_group > 0) {
#pragma unroll
    for (int i = 0; i < NP; i++)
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
    for (int i = 0; i < NP; i++) {
      int e = lane + 32 * i;
      if (e < E && !keep[e / gs]) sv[i] = PM_NEG;
    }
  }
#pragma unroll
  for (int i = 0; i < NP; i++) key[i] = pm_fkey(sv[i]);
}

// The routing weight of pick k = lane (< K) from the picked scores in selection
// order sel_p[0..K) (src/moe_kernels.rs:1072-1074, src/oss_kernels.rs:31-32,
// src/ds4.rs:1416-1424). Sums run in k order, every lane repeats them.
__device__ __forceinline__ float pm_route_weight(const pm_layer_desc &D, const float *sel_p,
                                                 int k) {
  const int K = D.top_k;
  float x;
  if (D.gating == PM_GATE_SOFTMAX_SELECTED) {
    float evsum = 0.0f, mine = 0.0f;
    for (int j = 0; j < K; j++) {
      float ev = pm_exp(__fsub_rn(sel_p[j], sel_p[0]));
      evsum = __fadd_rn(evsum, ev);
      if (j == k) mine = ev;
    }
    x = __fdiv_rn(mine, evsum);
  } else {
    float wsum = 0.0f;
    for (int j = 0; j < K; j++) wsum = __fadd_rn(wsum, sel_p[j]);
    x = sel_p[k];
    if (D.gating == PM_GATE_SQRT_SOFTPLUS) x = __fdiv_rn(x, wsum);
    else if (D.norm_w) x = __fdiv_rn(x, fmaxf(wsum, 6.103515625e-5f));
  }
  if (D.w_scale != 0.0f) x = __fmul_rn(x, D.w_scale);
  return x;
}

// The whole routing of one token by one warp; lane k < K writes ids_out[k], w_out[k].
// sel_p: K floats of per-warp shared scratch.
template <int NP>
__device__ __forceinline__ void pm_route_warp_n(const pm_layer_desc &D, const float *lg,
                                                const float *__restrict__ sel_bias, int lane,
                                                float *ssv, float *gsc, unsigned char *keep,
                                                uint32_t *ids_out, float *w_out) {
  const int K = D.top_k;
  float pr[NP];
  uint32_t key[NP];
  pm_route_scores<NP>(D, lg, sel_bias, lane, ssv, gsc, keep, pr, key);
  float *sel_p = ssv;  // the group scratch is free again
  __syncwarp();
  // K rounds of (max, lowest index) (src/moe_kernels.rs:1053-1067), on ordered
  // integer keys: one warp-wide max, then the first slot/lane that holds it
  const uint32_t KNEG = pm_fkey(PM_NEG);
  uint32_t my_e = 0;
#pragma unroll 1
  for (int k = 0; k < K; k++) {
    uint32_t lk = key[0];
#pragma unroll
    for (int i = 1; i < NP; i++) lk = max(lk, key[i]);
    uint32_t m = __reduce_max_sync(PM_FULL, lk);
    uint32_t e = 0;
    float w = 0.0f;
    bool found = false;
#pragma unroll
    for (int i = 0; i < NP; i++) {
      uint32_t b = __ballot_sync(PM_FULL, key[i] == m);
      if (!found && b != 0) {  // uniform across the warp
        found = true;
        int lw = __ffs((int)b) - 1;
        e = (uint32_t)(32 * i + lw);
        w = __shfl_sync(PM_FULL, pr[i], lw);
        if (lane == lw) key[i] = KNEG;
      }
    }
    if (lane == k) my_e = e;
    if (lane == 0) sel_p[k] = w;
  }
  __syncwarp();
  if (lane < K) {
    ids_out[lane] = my_e;
    w_out[lane] = pm_route_weight(D, sel_p, lane);
  }
}

__device__ __forceinline__ void pm_route_warp(const pm_layer_desc &D, const float *lg,
                                              const float *__restrict__ sel_bias, int lane,
                                              float *ssv, float *gsc, unsigned char *keep,
                                              uint32_t *ids_out, float *w_out) {
  if (D.n_exp <= 128) pm_route_warp_n<4>(D, lg, sel_bias, lane, ssv, gsc, keep, ids_out, w_out);
  else if (D.n_exp <= 256) pm_route_warp_n<8>(D, lg, sel_bias, lane, ssv, gsc, keep, ids_out, w_out);
  else pm_route_warp_n<16>(D, lg, sel_bias, lane, ssv, gsc, keep, ids_out, w_out);
}
