// common.cuh - shared device helpers of the sm_100a MoE kernels.
//
// Everything here is arithmetic that must give the same bits as the CPU code of
// the reference (paths cited are inside the Pelica source tree). The library
// is compiled with -fmad=false: a fused multiply-add happens only where
// __fmaf_rn is written.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pelica_moe.h"

#define PM_NEG (-3.0e38f)  // the shaders' "minus infinity" (src/moe_kernels.rs:1026)
#define PM_FULL 0xffffffffu

// f16 bits -> f32 (src/ds4.rs:168-180): exact, subnormals included
__device__ __forceinline__ float pm_f16(uint32_t h) {
  return __half2float(__ushort_as_half((unsigned short)(h & 0xffffu)));
}

// e^x, the reference's `pexp` (src/moe_kernels.rs:437-468, src/cpu_attn.rs:30-44)
// with the argument range widened to [-87, 88]: adds, multiplies and explicit
// fmas only, so CPU and GPU agree bit for bit.
__device__ __forceinline__ float pm_exp(float x) {
  if (x < -87.0f) return 0.0f;
  if (x > 88.0f) return __int_as_float(0x7f800000);
  float n = floorf(__fmaf_rn(x, 1.44269504f, 0.5f));
  float r = __fmaf_rn(n, -0.693359375f, x);
  r = __fmaf_rn(n, 2.12194440e-4f, r);
  float p = 1.98756915e-4f;
  p = __fmaf_rn(p, r, 1.39819995e-3f);
  p = __fmaf_rn(p, r, 8.3334519e-3f);
  p = __fmaf_rn(p, r, 4.1665796e-2f);
  p = __fmaf_rn(p, r, 0.16666665f);
  p = __fmaf_rn(p, r, 0.50000001f);
  float y = __fmaf_rn(p, __fmul_rn(r, r), r);
  y = __fadd_rn(y, 1.0f);
  return __fmul_rn(y, __int_as_float(((int)n + 127) << 23));
}

// ln(1+x), x >= 0: the fixed spelling both sides of this repository use for
// sqrt-softplus gating (the reference calls the platform ln_1p, src/ds4.rs:1378)
__device__ __forceinline__ float pm_log1p(float x) {
  float u = __fadd_rn(1.0f, x);
  float c = __fdiv_rn(__fsub_rn(x, __fsub_rn(u, 1.0f)), u);
  uint32_t ub = __float_as_uint(u);
  int e = (int)((ub >> 23) & 0xff) - 126;
  float m = __uint_as_float((ub & 0x007fffffu) | 0x3f000000u);
  if (m < 0.707106781186547524f) {
    e -= 1;
    m = __fsub_rn(__fadd_rn(m, m), 1.0f);
  } else {
    m = __fsub_rn(m, 1.0f);
  }
  float z = __fmul_rn(m, m);
  float p = 7.0376836292e-2f;
  p = __fmaf_rn(p, m, -1.1514610310e-1f);
  p = __fmaf_rn(p, m, 1.1676998740e-1f);
  p = __fmaf_rn(p, m, -1.2420140846e-1f);
  p = __fmaf_rn(p, m, 1.4249322787e-1f);
  p = __fmaf_rn(p, m, -1.6668057665e-1f);
  p = __fmaf_rn(p, m, 2.0000714765e-1f);
  p = __fmaf_rn(p, m, -2.4999993993e-1f);
  p = __fmaf_rn(p, m, 3.3333331174e-1f);
  float y = __fmul_rn(__fmul_rn(m, z), p);
  float fe = (float)e;
  y = __fmaf_rn(fe, -2.12194440e-4f, y);
  y = __fmaf_rn(-0.5f, z, y);
  float r = __fadd_rn(m, y);
  r = __fmaf_rn(fe, 0.693359375f, r);
  return __fadd_rn(r, c);
}

// the expert activation (src/ds4_cpu.rs:311-312, src/moe_kernels.rs:52,
// src/oss_batch.rs:785); biases are added by the caller. `fold`: multiply by w.
__device__ __forceinline__ float pm_act(int act, float limit, float alpha, float g, float u,
                                        float w, bool fold) {
  float h;
  if (act == PM_ACT_OSS_GLU) {
    float x = fminf(g, limit);
    float y = fminf(fmaxf(u, -limit), limit);
    float den = __fadd_rn(1.0f, pm_exp(__fmul_rn(-alpha, x)));
    h = __fmul_rn(__fdiv_rn(x, den), __fadd_rn(y, 1.0f));
  } else {
    if (act == PM_ACT_SILU_CLAMP && limit > 0.0f) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
    }
    float den = __fadd_rn(1.0f, pm_exp(-g));
    h = __fmul_rn(__fdiv_rn(g, den), u);
  }
  return fold ? __fmul_rn(h, w) : h;
}

// Q4_K sub-block scale/min j of a 12-byte field given as three words
// (`scales`, src/ds4_cpu.rs:45-57; `scmin_k4`, src/moe_kernels.rs:98-107)
__device__ __forceinline__ void pm_q4k_scmin(uint32_t w0, uint32_t w1, uint32_t w2, int j, int &sc,
                                             int &m) {
  // bytes s[0..3]=w0, s[4..7]=w1, s[8..11]=w2
  if (j < 4) {
    sc = (w0 >> (8 * j)) & 63;
    m = (w1 >> (8 * j)) & 63;
  } else {
    int jj = j - 4;
    uint32_t a = (w2 >> (8 * jj)) & 0xff;
    sc = (a & 15) | ((((w0 >> (8 * jj)) & 0xff) >> 6) << 4);
    m = (a >> 4) | ((((w1 >> (8 * jj)) & 0xff) >> 6) << 4);
  }
}

// all eight (scale, min) pairs of a Q4_K block at once, as bytes of four words: sub-blocks
// 0..3 in sc03 / m03, 4..7 in sc47 / m47 (same field as pm_q4k_scmin)
__device__ __forceinline__ void pm_q4k_scmin_packed(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t &sc03,
                                                    uint32_t &sc47, uint32_t &m03, uint32_t &m47) {
  sc03 = w0 & 0x3f3f3f3fu;
  m03 = w1 & 0x3f3f3f3fu;
  sc47 = (w2 & 0x0f0f0f0fu) | ((w0 >> 2) & 0x30303030u);
  m47 = ((w2 >> 4) & 0x0f0f0f0fu) | ((w1 >> 2) & 0x30303030u);
}
// bytes (b_lo, b_hi) selected by `sel` (a __byte_perm selector placing them in the low bytes
// of the two 16-bit lanes) as two f16 values: 0x6400 | b is 1024 + b, minus 1024 is exact
__device__ __forceinline__ uint32_t pm_bytes_to_half2(uint32_t w, uint32_t sel) {
  const uint32_t h = __byte_perm(w, 0u, sel) | 0x64006400u;
  const __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&h), __half2half2(__ushort_as_half((unsigned short)0x6400)));
  return *reinterpret_cast<const uint32_t *>(&r);
}

// four 6-bit values (bytes 0..63) minus 32 each, as signed bytes: with bit 7 set no byte
// borrows from its neighbour, and flipping it back leaves q + 96 - 128 (mod 256) = q - 32
__device__ __forceinline__ uint32_t pm_sub32x4(uint32_t q) {
  return ((q | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
}

// the IQ4_NL codebook (src/iq_tables.rs:72), entry i in byte i of four words
__device__ __forceinline__ int pm_iq4nl(uint32_t i) {
  const uint32_t t[4] = {0xbfad9881u, 0xf6eaddcfu, 0x26190d01u, 0x71594535u};
  return (int)(int8_t)(t[(i >> 2) & 3] >> (8 * (i & 3)));
}
// four codebook entries at once: the low nibble of each byte of `idx` selects
__device__ __forceinline__ uint32_t pm_iq4nl_x4(uint32_t idx) {
  const uint32_t s = idx & 0x07070707u;
  const uint32_t sel = (s & 0xfu) | ((s >> 4) & 0xf0u) | ((s >> 8) & 0xf00u) | ((s >> 12) & 0xf000u);
  const uint32_t lo = __byte_perm(0xbfad9881u, 0xf6eaddcfu, sel);  // entries 0..7
  const uint32_t hi = __byte_perm(0x26190d01u, 0x71594535u, sel);  // entries 8..15
  const uint32_t m = ((idx >> 3) & 0x01010101u) * 0xffu;
  return (lo & ~m) | (hi & m);
}

// `e8` (src/oss_kernels.rs:42-45): 2^(e-128)
__device__ __forceinline__ float pm_e8(uint32_t e) {
  return e < 2 ? __uint_as_float(0x00200000u << e) : __uint_as_float((e - 1) << 23);
}

// doubled E2M1 code -> value (`KV_MX`, src/moe_kernels.rs:109) without a table:
// magnitudes {0,1,2,3,4,6,8,12}
__device__ __forceinline__ float pm_e2m1(uint32_t c) {
  uint32_t m = c & 7;
  // 0,1 -> m ; 2..7 -> (2 + (m&1)) << ((m>>1) - 1)
  float v = m < 2 ? (float)m : (float)((2 + (m & 1)) << ((m >> 1) - 1));
  return ((c & 8) && m) ? -v : v;  // code 8 is +0, as the table has it
}

__device__ __forceinline__ float pm_warp_max(float v) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(PM_FULL, v, o));
  return v;
}
__device__ __forceinline__ uint32_t pm_warp_min_u32(uint32_t v) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v = min(v, __shfl_xor_sync(PM_FULL, v, o));
  return v;
}
// lanes summed by xor shuffles 16, 8, 4, 2, 1 (the order the reference spells
// out for its subgroup sums, src/moe_kernels.rs:489-492)
__device__ __forceinline__ float pm_warp_sum_16_1(float v) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(PM_FULL, v, o));
  return v;
}
// `dot_f32`'s lane reduction (src/quant.rs:205-236): accumulators (0+1)+(2+3)
// then 4, 2, 1 -> xor 8, 16, 4, 2, 1 on a warp whose lane = column mod 32
__device__ __forceinline__ float pm_warp_sum_dot(float v) {
  v = __fadd_rn(v, __shfl_xor_sync(PM_FULL, v, 8));
  v = __fadd_rn(v, __shfl_xor_sync(PM_FULL, v, 16));
  v = __fadd_rn(v, __shfl_xor_sync(PM_FULL, v, 4));
  v = __fadd_rn(v, __shfl_xor_sync(PM_FULL, v, 2));
  v = __fadd_rn(v, __shfl_xor_sync(PM_FULL, v, 1));
  return v;
}
// 1/rms(x), unit weight (the layer loop's glue, src/forward.rs:63-69). Sum of
// squares in a fixed order: thread j of the first 256 takes x[j], x[j+256], ...
// by fma, warps are summed by xor shuffles 16..1, the 8 warp sums one after
// another. Called by every thread of a CTA of >= 256 threads; red8 = 8 floats
// of shared memory.
__device__ __forceinline__ float pm_rms_inv(const float *xr, int d, float eps, float *red8) {
  int tid = threadIdx.x;
  if (tid < 256) {
    float acc = 0.0f;
    for (int c = tid; c < d; c += 256) acc = __fmaf_rn(xr[c], xr[c], acc);
    acc = pm_warp_sum_16_1(acc);
    if ((tid & 31) == 0) red8[tid >> 5] = acc;
  }
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int g = 0; g < 8; g++) total = __fadd_rn(total, red8[g]);
  float ms = __fdiv_rn(total, (float)d);
  return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, eps)));
}

__device__ __forceinline__ int pm_warp_sum_i32(int v) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(PM_FULL, v, o);
  return v;
}
