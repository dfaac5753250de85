// synth.cu - seeded N(0, sigma) weights quantised on the device into GGUF block
// formats (benchmark set-up; 18.8 GB of Q4_K/Q6_K experts are generated in
// seconds instead of minutes on the host).
//
// Pelica has no quantiser for these formats (it only reads them from files,
// src/gguf.rs:85-121); these encoders are this repository's own. They write
// raw GGUF-layout blocks, which then go through the same re-layout as uploaded
// weights.
#include "moe_internal.cuh"

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// N(0,1) from a counter: Box-Muller on two 24-bit uniforms
__device__ __forceinline__ float synth_normal(uint64_t seed, uint64_t idx) {
  uint64_t r = splitmix64(seed ^ splitmix64(idx));
  float u1 = ((float)((r >> 40) & 0xffffff) + 1.0f) * (1.0f / 16777217.0f);
  float u2 = (float)((r >> 8) & 0xffffff) * (1.0f / 16777216.0f);
  return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}

__device__ __forceinline__ float rhaf(float x) { return roundf(x); }

// one CTA (256 threads) per Q4_K super-block
__global__ void __launch_bounds__(256) k_synth_q4k(uint8_t *raw, size_t nb, uint64_t seed,
                                                  float sigma) {
  __shared__ float s_scale[8], s_min[8];
  __shared__ uint8_t s_q[256];
  size_t b = blockIdx.x;
  if (b >= nb) return;
  int tid = threadIdx.x, lane = tid & 31, j = tid >> 5;
  float v = sigma * synth_normal(seed, b * 256 + tid);
  float mn = v, mx = v;
  for (int o = 16; o >= 1; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(PM_FULL, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(PM_FULL, mx, o));
  }
  mn = fminf(mn, 0.0f);
  if (lane == 0) {
    s_scale[j] = fmaxf(mx - mn, 0.0f) / 15.0f;
    s_min[j] = -mn;
  }
  __syncthreads();
  float smax = 0.0f, mmax = 0.0f;
  for (int i = 0; i < 8; i++) {
    smax = fmaxf(smax, s_scale[i]);
    mmax = fmaxf(mmax, s_min[i]);
  }
  __half dh = __float2half_rn(smax / 63.0f), dmh = __float2half_rn(mmax / 63.0f);
  float d = __half2float(dh), dmin = __half2float(dmh);
  int sc = d > 0.0f ? (int)fminf(fmaxf(rhaf(s_scale[j] / d), 0.0f), 63.0f) : 0;
  int m = dmin > 0.0f ? (int)fminf(fmaxf(rhaf(s_min[j] / dmin), 0.0f), 63.0f) : 0;
  float step = d * (float)sc;
  int q = step > 0.0f ? (int)fminf(fmaxf(rhaf((v + dmin * (float)m) / step), 0.0f), 15.0f) : 0;
  s_q[tid] = (uint8_t)q;
  __shared__ uint8_t s_sc[8], s_m[8];
  if (lane == 0) {
    s_sc[j] = (uint8_t)sc;
    s_m[j] = (uint8_t)m;
  }
  __syncthreads();
  uint8_t *blk = raw + b * 144;
  if (tid == 0) {
    *(__half *)(blk) = dh;
    *(__half *)(blk + 2) = dmh;
  }
  if (tid < 4) {
    blk[4 + tid] = s_sc[tid] | ((s_sc[tid + 4] >> 4) << 6);
    blk[8 + tid] = s_m[tid] | ((s_m[tid + 4] >> 4) << 6);
    blk[12 + tid] = (s_sc[tid + 4] & 15) | ((s_m[tid + 4] & 15) << 4);
  }
  if (tid < 128) {
    int c = tid >> 5, i = tid & 31;
    blk[16 + tid] = s_q[64 * c + i] | (s_q[64 * c + 32 + i] << 4);
  }
}

// one CTA (256 threads) per Q6_K super-block
__global__ void __launch_bounds__(256) k_synth_q6k(uint8_t *raw, size_t nb, uint64_t seed,
                                                  float sigma) {
  __shared__ float s_gs[16];
  __shared__ uint8_t s_q[256];
  __shared__ int8_t s_sc[16];
  size_t b = blockIdx.x;
  if (b >= nb) return;
  int tid = threadIdx.x, g = tid >> 4;
  float v = sigma * synth_normal(seed, b * 256 + tid);
  float a = fabsf(v);
  for (int o = 8; o >= 1; o >>= 1) a = fmaxf(a, __shfl_xor_sync(PM_FULL, a, o));
  if ((tid & 15) == 0) s_gs[g] = a / 31.0f;
  __syncthreads();
  float gmax = 0.0f;
  for (int i = 0; i < 16; i++) gmax = fmaxf(gmax, s_gs[i]);
  __half dh = __float2half_rn(gmax / 127.0f);
  float d = __half2float(dh);
  int sc = d > 0.0f ? (int)fminf(fmaxf(rhaf(s_gs[g] / d), 0.0f), 127.0f) : 0;
  float step = d * (float)sc;
  int q = step > 0.0f ? (int)fminf(fmaxf(rhaf(v / step), -32.0f), 31.0f) : 0;
  s_q[tid] = (uint8_t)(q + 32);
  if ((tid & 15) == 0) s_sc[g] = (int8_t)sc;
  __syncthreads();
  uint8_t *blk = raw + b * 210;
  if (tid < 128) {  // ql byte 64n + 32*(qt&1) + l : low nibble qt, high nibble qt+2
    int n = tid >> 6, o = tid & 63, h = o >> 5, l = o & 31;
    uint8_t lo = s_q[128 * n + 32 * h + l] & 15, hi = s_q[128 * n + 32 * (h + 2) + l] & 15;
    blk[tid] = lo | (hi << 4);
  } else if (tid < 192) {  // qh byte 32n + l : 2 bits per qt
    int i = tid - 128, n = i >> 5, l = i & 31;
    uint8_t x = 0;
    for (int qt = 0; qt < 4; qt++) x |= (s_q[128 * n + 32 * qt + l] >> 4) << (2 * qt);
    blk[tid] = x;
  } else if (tid < 208) {
    blk[tid] = (uint8_t)s_sc[tid - 192];
  } else if (tid == 208) {
    *(__half *)(blk + 208) = dh;
  }
}

// one warp per MXFP4 block (8 blocks per 256-thread CTA)
__global__ void __launch_bounds__(256) k_synth_mxfp4(uint8_t *raw, size_t nb, uint64_t seed,
                                                    float sigma) {
  size_t b = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (b >= nb) return;
  int lane = threadIdx.x & 31;
  float v = sigma * synth_normal(seed, b * 32 + lane);
  float a = fabsf(v);
  for (int o = 16; o >= 1; o >>= 1) a = fmaxf(a, __shfl_xor_sync(PM_FULL, a, o));
  int e = 2;
  if (a > 0.0f) {
    int ex = (int)((__float_as_uint(a) >> 23) & 0xff) - 127;  // floor(log2 a) for normals
    e = min(max(ex - 3 + 128, 2), 254);
  }
  float s = pm_e8((uint32_t)e);
  float mag = fabsf(v) / s;
  const float tab[8] = {0.f, 1.f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f};
  int best = 0;
  float bd = mag;
  for (int i = 1; i < 8; i++) {
    float dd = fabsf(mag - tab[i]);
    if (dd < bd) { bd = dd; best = i; }
  }
  uint32_t code = (uint32_t)best | ((v < 0.0f && best > 0) ? 8u : 0u);
  uint32_t hi = __shfl_down_sync(PM_FULL, code, 16);
  uint8_t *blk = raw + b * 17;
  if (lane == 0) blk[0] = (uint8_t)e;
  if (lane < 16) blk[1 + lane] = (uint8_t)(code | (hi << 4));
}

__global__ void k_synth_f32(float *out, size_t n, uint64_t seed, float sigma, int bf16_round) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = sigma * synth_normal(seed, i);
  if (bf16_round) {
    uint32_t u = __float_as_uint(v);
    u = (u + 0x7fffu + ((u >> 16) & 1)) & 0xffff0000u;
    v = __uint_as_float(u);
  }
  out[i] = v;
}

void launch_synth_blocks(const Launch &L, int type, uint8_t *raw, size_t nb, uint64_t seed,
                         float sigma) {
  if (nb == 0) return;
  switch (type) {
    case PM_TYPE_Q4_K:
      k_synth_q4k<<<(unsigned)nb, 256, 0, L.stream>>>(raw, nb, seed, sigma);
      break;
    case PM_TYPE_Q6_K:
      k_synth_q6k<<<(unsigned)nb, 256, 0, L.stream>>>(raw, nb, seed, sigma);
      break;
    case PM_TYPE_MXFP4:
      k_synth_mxfp4<<<(unsigned)((nb + 7) / 8), 256, 0, L.stream>>>(raw, nb, seed, sigma);
      break;
  }
  if (L.count) ++*L.count;
}
void launch_synth_f32(const Launch &L, float *out, size_t n, uint64_t seed, float sigma,
                      int bf16_round) {
  if (n == 0) return;
  k_synth_f32<<<(unsigned)((n + 255) / 256), 256, 0, L.stream>>>(out, n, seed, sigma, bf16_round);
  if (L.count) ++*L.count;
}
