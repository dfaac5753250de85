// kernels_basic.cu - the general (any token count) kernels of the MoE path:
// block-format re-layout and decode, activation quantiser, router, top-k,
// dispatch plan, grouped gate/up + activation, grouped down, combine.
//
// Integer work (block decode, quantised dots, routing, plan) is bit-exact
// against the reference CPU code; float tails follow `row_scalar`'s order
// (src/ds4_cpu.rs:59-83). Citations are paths inside the Pelica source tree.
#include "moe_internal.cuh"
#include "route.cuh"

#define KLAUNCH(L, kern, grid, block, smem, ...)            \
  do {                                                      \
    kern<<<grid, block, smem, (L).stream>>>(__VA_ARGS__);   \
    if ((L).count) ++*(L).count;                            \
  } while (0)

// ===========================================================================
// block formats: GGUF bytes <-> device planes
// ===========================================================================

__global__ void k_repack_q6k(const uint8_t *__restrict__ raw, size_t nb, uint8_t *ql, uint8_t *qh,
                             uint8_t *sc, uint8_t *d) {
  // one thread per 2 bytes of a 210-byte block: 105 threads per block
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t b = i / 105;
  int j = (int)(i % 105) * 2;
  if (b >= nb) return;
  uint16_t v = *(const uint16_t *)(raw + b * 210 + j);
  uint8_t *dst;
  if (j < 128) dst = ql + b * 128 + j;
  else if (j < 192) dst = qh + b * 64 + (j - 128);
  else if (j < 208) dst = sc + b * 16 + (j - 192);
  else dst = d + b * 2;
  *(uint16_t *)dst = v;
}
__global__ void k_unpack_q6k(uint8_t *raw, size_t nb, const uint8_t *ql, const uint8_t *qh,
                             const uint8_t *sc, const uint8_t *d) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t b = i / 105;
  int j = (int)(i % 105) * 2;
  if (b >= nb) return;
  const uint8_t *src;
  if (j < 128) src = ql + b * 128 + j;
  else if (j < 192) src = qh + b * 64 + (j - 128);
  else if (j < 208) src = sc + b * 16 + (j - 192);
  else src = d + b * 2;
  *(uint16_t *)(raw + b * 210 + j) = *(const uint16_t *)src;
}
// byte-granular split: `head` bytes to plane h, the rest to plane r (or swapped)
__global__ void k_repack_split(const uint8_t *__restrict__ raw, size_t nb, int bb, int head,
                               uint8_t *ph, uint8_t *pr, int back) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t b = i / bb;
  int j = (int)(i % bb);
  if (b >= nb) return;
  uint8_t *rawm = const_cast<uint8_t *>(raw);
  uint8_t *p = j < head ? ph + b * head + j : pr + b * (bb - head) + (j - head);
  if (back) rawm[b * bb + j] = *p;
  else *p = raw[b * bb + j];
}

void launch_repack(const Launch &L, int type, const uint8_t *raw, size_t nb, uint8_t *p0,
                   uint8_t *p1, uint8_t *p2, uint8_t *p3) {
  if (nb == 0) return;
  switch (type) {
    case PM_TYPE_Q4_K:
      cudaMemcpyAsync(p0, raw, nb * 144, cudaMemcpyDeviceToDevice, L.stream);
      break;
    case PM_TYPE_Q5_K:
      cudaMemcpyAsync(p0, raw, nb * 176, cudaMemcpyDeviceToDevice, L.stream);
      break;
    case PM_TYPE_GLM_Q4:  // the nibble region, then the scale region
      cudaMemcpyAsync(p0, raw, nb * 32, cudaMemcpyDeviceToDevice, L.stream);
      cudaMemcpyAsync(p1, raw + nb * 32, nb * 4, cudaMemcpyDeviceToDevice, L.stream);
      break;
    case PM_TYPE_IQ3_S: {  // the f16 d first in the raw block, the four byte fields after
      size_t n = nb * 110;
      KLAUNCH(L, k_repack_split, (unsigned)((n + 255) / 256), 256, 0, raw, nb, 110, 2, p1, p0, 0);
      break;
    }
    case PM_TYPE_Q6_K: {
      size_t n = nb * 105;
      KLAUNCH(L, k_repack_q6k, (unsigned)((n + 255) / 256), 256, 0, raw, nb, p0, p1, p2, p3);
      break;
    }
    case PM_TYPE_MXFP4: {  // scale byte first in the raw block, nibbles after
      size_t n = nb * 17;
      KLAUNCH(L, k_repack_split, (unsigned)((n + 255) / 256), 256, 0, raw, nb, 17, 1, p1, p0, 0);
      break;
    }
    case PM_TYPE_Q8_0: {
      size_t n = nb * 34;
      KLAUNCH(L, k_repack_split, (unsigned)((n + 255) / 256), 256, 0, raw, nb, 34, 2, p1, p0, 0);
      break;
    }
    case PM_TYPE_IQ4_NL: {
      size_t n = nb * 18;
      KLAUNCH(L, k_repack_split, (unsigned)((n + 255) / 256), 256, 0, raw, nb, 18, 2, p1, p0, 0);
      break;
    }
    case PM_TYPE_IQ4_XS: {
      size_t n = nb * 136;
      KLAUNCH(L, k_repack_split, (unsigned)((n + 255) / 256), 256, 0, raw, nb, 136, 8, p1, p0, 0);
      break;
    }
  }
}
void launch_unpack(const Launch &L, int type, uint8_t *raw, size_t nb, const uint8_t *p0,
                   const uint8_t *p1, const uint8_t *p2, const uint8_t *p3) {
  if (nb == 0) return;
  switch (type) {
    case PM_TYPE_Q4_K:
      cudaMemcpyAsync(raw, p0, nb * 144, cudaMemcpyDeviceToDevice, L.stream);
      break;
    case PM_TYPE_Q5_K:
      cudaMemcpyAsync(raw, p0, nb * 176, cudaMemcpyDeviceToDevice, L.stream);
      break;
    case PM_TYPE_GLM_Q4:
      cudaMemcpyAsync(raw, p0, nb * 32, cudaMemcpyDeviceToDevice, L.stream);
      cudaMemcpyAsync(raw + nb * 32, p1, nb * 4, cudaMemcpyDeviceToDevice, L.stream);
      break;
    case PM_TYPE_IQ3_S: {
      size_t n = nb * 110;
      KLAUNCH(L, k_repack_split, (unsigned)((n + 255) / 256), 256, 0, raw, nb, 110, 2,
              const_cast<uint8_t *>(p1), const_cast<uint8_t *>(p0), 1);
      break;
    }
    case PM_TYPE_Q6_K: {
      size_t n = nb * 105;
      KLAUNCH(L, k_unpack_q6k, (unsigned)((n + 255) / 256), 256, 0, raw, nb, p0, p1, p2, p3);
      break;
    }
    case PM_TYPE_MXFP4: {
      size_t n = nb * 17;
      KLAUNCH(L, k_repack_split, (unsigned)((n + 255) / 256), 256, 0, raw, nb, 17, 1,
              const_cast<uint8_t *>(p1), const_cast<uint8_t *>(p0), 1);
      break;
    }
    case PM_TYPE_Q8_0: {
      size_t n = nb * 34;
      KLAUNCH(L, k_repack_split, (unsigned)((n + 255) / 256), 256, 0, raw, nb, 34, 2,
              const_cast<uint8_t *>(p1), const_cast<uint8_t *>(p0), 1);
      break;
    }
    case PM_TYPE_IQ4_NL: {
      size_t n = nb * 18;
      KLAUNCH(L, k_repack_split, (unsigned)((n + 255) / 256), 256, 0, raw, nb, 18, 2,
              const_cast<uint8_t *>(p1), const_cast<uint8_t *>(p0), 1);
      break;
    }
    case PM_TYPE_IQ4_XS: {
      size_t n = nb * 136;
      KLAUNCH(L, k_repack_split, (unsigned)((n + 255) / 256), 256, 0, raw, nb, 136, 8,
              const_cast<uint8_t *>(p1), const_cast<uint8_t *>(p0), 1);
      break;
    }
  }
}

// the IQ3_S codebook, a constant of the format (src/iq_tables.rs:4): 512 entries of four odd
// magnitudes, three bits each
__device__ const uint16_t g_iq3s_codes[512] = {
#include "../../include/pelica_iq3s_grid.inc"
};
// entry idx as four bytes (magnitude j in byte j), as the reference's table holds them
__device__ __forceinline__ uint32_t pm_iq3s_grid(uint32_t idx) {
  const uint32_t c = __ldg(&g_iq3s_codes[idx]);
  const uint32_t h = (c & 7u) | ((c & 0x38u) << 5) | ((c & 0x1c0u) << 10) | ((c & 0xe00u) << 15);
  return 2u * h + 0x01010101u;
}
// sub-block ib of an IQ3_S block (plane 0: qs @0, qh @64, signs @72, scales @104 of 108 bytes):
// its 32 signed magnitudes as eight words of four int8, and the scale 1 + 2 * sc
// (`iq3s_sub`, src/q4x_cpu.rs:64-82)
__device__ __forceinline__ int pm_iq3s_sub(const uint8_t *__restrict__ blk, int ib, uint32_t out[8]) {
  const uint32_t qh = blk[64 + ib];
  const uint32_t sg = *(const uint32_t *)(blk + 72 + 4 * ib);  // bit v = sign of value v
  const uint32_t q0 = *(const uint32_t *)(blk + 8 * ib), q1 = *(const uint32_t *)(blk + 8 * ib + 4);
#pragma unroll
  for (int k = 0; k < 8; k++) {
    const uint32_t qs = ((k < 4 ? q0 : q1) >> (8 * (k & 3))) & 0xffu;
    const uint32_t mag = pm_iq3s_grid(qs | (((qh >> k) & 1u) << 8));
    // negate the bytes whose sign bit is set: (m ^ mask) - mask per byte with mask 0xff
    const uint32_t nb = (sg >> (4 * k)) & 0xfu;
    const uint32_t mask = ((nb & 1u) | ((nb & 2u) << 7) | ((nb & 4u) << 14) | ((nb & 8u) << 21)) * 0xffu;
    out[k] = __vsub4(mag ^ mask, mask);
  }
  return 1 + 2 * (int)((blk[104 + ib / 2] >> (4 * (ib % 2))) & 15);
}

// value v of block b, from the device planes (`deq4`, src/moe_kernels.rs:63-84)
template <int TYPE>
__device__ __forceinline__ float deq_value(const uint8_t *p0, const uint8_t *p1, const uint8_t *p2,
                                           const uint8_t *p3, size_t b, int v) {
  if (TYPE == PM_TYPE_Q4_K) {  // (d*sc)*q - dmin*m (src/moe_kernels.rs:73)
    const uint8_t *blk = p0 + b * 144;
    const uint32_t *hw = (const uint32_t *)blk;
    uint32_t h0 = hw[0];
    int sc, m;
    pm_q4k_scmin(hw[1], hw[2], hw[3], v / 32, sc, m);
    int c = v / 64, i = v % 32;
    uint8_t byte = blk[16 + 32 * c + i];
    int q = (v % 64) >= 32 ? (byte >> 4) : (byte & 15);
    float d = pm_f16(h0), dmin = pm_f16(h0 >> 16);
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
  } else if (TYPE == PM_TYPE_Q5_K) {  // (d*sc)*(q | hb << 4) - dmin*m (src/moe_kernels.rs:74)
    const uint8_t *blk = p0 + b * 176;
    const uint32_t *hw = (const uint32_t *)blk;
    uint32_t h0 = hw[0];
    int sc, m;
    pm_q4k_scmin(hw[1], hw[2], hw[3], v / 32, sc, m);
    int c = v / 64, i = v % 32, hi = (v % 64) >= 32;
    uint8_t byte = blk[48 + 32 * c + i];
    int q = (hi ? (byte >> 4) : (byte & 15)) | (((blk[16 + i] >> (2 * c + hi)) & 1) << 4);
    float d = pm_f16(h0), dmin = pm_f16(h0 >> 16);
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
  } else if (TYPE == PM_TYPE_IQ3_S) {  // (d * scale) * signed magnitude (src/q4x_cpu.rs:477-487)
    const uint8_t *blk = p0 + b * 108;
    const int ib = v >> 5, i = v & 31, k = i >> 2, j = i & 3;
    const uint32_t idx = (uint32_t)blk[8 * ib + k] | ((((uint32_t)blk[64 + ib] >> k) & 1u) << 8);
    const int mag = (int)((pm_iq3s_grid(idx) >> (8 * j)) & 0xffu);
    const int neg = (blk[72 + 4 * ib + i / 8] >> (i % 8)) & 1;
    const int sc = 1 + 2 * (int)((blk[104 + ib / 2] >> (4 * (ib % 2))) & 15);
    const float d = pm_f16(*(const uint16_t *)(p1 + b * 2));
    return __fmul_rn(__fmul_rn(d, (float)sc), (float)(neg ? -mag : mag));
  } else if (TYPE == PM_TYPE_GLM_Q4) {  // (nibble - 8) * scale of the group (src/gpu.rs:96-99)
    const uint8_t byte = p0[b * 32 + (v >> 1)];
    const int q = (v & 1) ? (byte >> 4) : (byte & 15);
    return __fmul_rn((float)(q - 8), *(const float *)(p1 + b * 4));
  } else if (TYPE == PM_TYPE_Q6_K) {  // (d*sc)*(q-32) (src/moe_kernels.rs:75)
    int n = v / 128, r = v % 128, qt = r / 32, l = r % 32;
    uint8_t qlb = p0[b * 128 + 64 * n + l + 32 * (qt & 1)];
    int lo = qt >= 2 ? (qlb >> 4) : (qlb & 15);
    int hb = (p1[b * 64 + 32 * n + l] >> (2 * qt)) & 3;
    int k = 8 * n + l / 16 + 2 * qt;
    float sc = (float)(int8_t)p2[b * 16 + k];
    float d = pm_f16(*(const uint16_t *)(p3 + b * 2));
    return __fmul_rn(__fmul_rn(d, sc), __fsub_rn((float)(lo | (hb << 4)), 32.0f));
  } else if (TYPE == PM_TYPE_MXFP4) {  // e8(e)*KV_MX[q] (src/moe_kernels.rs:80)
    uint8_t byte = p0[b * 16 + (v & 15)];
    uint32_t c = v >= 16 ? (byte >> 4) : (byte & 15);
    return __fmul_rn(pm_e8(p1[b]), pm_e2m1(c));
  } else if (TYPE == PM_TYPE_IQ4_XS) {  // (d * (ls - 32)) * codebook[index] (src/q4x_cpu.rs:462-476)
    const uint8_t *hd = p1 + b * 8;
    const int ib = v >> 5, i = v & 31;
    const uint32_t sh = (uint32_t)hd[2] | ((uint32_t)hd[3] << 8);
    const int ls = (int)((hd[4 + ib / 2] >> (4 * (ib % 2))) & 15) | (int)(((sh >> (2 * ib)) & 3) << 4);
    const float dl = __fmul_rn(pm_f16(*(const uint16_t *)hd), (float)(ls - 32));
    const uint8_t byte = p0[b * 128 + 16 * ib + (i & 15)];
    return __fmul_rn(dl, (float)pm_iq4nl(i >= 16 ? (byte >> 4) : (byte & 15)));
  } else if (TYPE == PM_TYPE_IQ4_NL) {  // d * codebook[index] (src/q4x_cpu.rs:453-461)
    uint8_t byte = p0[b * 16 + (v & 15)];
    float d = pm_f16(*(const uint16_t *)(p1 + b * 2));
    return __fmul_rn(d, (float)pm_iq4nl(v >= 16 ? (byte >> 4) : (byte & 15)));
  } else {  // Q8_0: d*q (src/moe_kernels.rs:68)
    float d = pm_f16(*(const uint16_t *)(p1 + b * 2));
    return __fmul_rn(d, (float)(int8_t)p0[b * 32 + v]);
  }
}

template <int TYPE, int BV>
__global__ void k_dequant(size_t n, const uint8_t *p0, const uint8_t *p1, const uint8_t *p2,
                          const uint8_t *p3, float *out) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  out[i] = deq_value<TYPE>(p0, p1, p2, p3, i / BV, (int)(i % BV));
}

void launch_dequant(const Launch &L, int type, size_t n, const uint8_t *p0, const uint8_t *p1,
                    const uint8_t *p2, const uint8_t *p3, float *out) {
  if (n == 0) return;
  unsigned g = (unsigned)((n + 255) / 256);
  switch (type) {
    case PM_TYPE_Q4_K: KLAUNCH(L, (k_dequant<PM_TYPE_Q4_K, 256>), g, 256, 0, n, p0, p1, p2, p3, out); break;
    case PM_TYPE_Q6_K: KLAUNCH(L, (k_dequant<PM_TYPE_Q6_K, 256>), g, 256, 0, n, p0, p1, p2, p3, out); break;
    case PM_TYPE_MXFP4: KLAUNCH(L, (k_dequant<PM_TYPE_MXFP4, 32>), g, 256, 0, n, p0, p1, p2, p3, out); break;
    case PM_TYPE_Q8_0: KLAUNCH(L, (k_dequant<PM_TYPE_Q8_0, 32>), g, 256, 0, n, p0, p1, p2, p3, out); break;
    case PM_TYPE_IQ4_NL: KLAUNCH(L, (k_dequant<PM_TYPE_IQ4_NL, 32>), g, 256, 0, n, p0, p1, p2, p3, out); break;
    case PM_TYPE_IQ4_XS: KLAUNCH(L, (k_dequant<PM_TYPE_IQ4_XS, 256>), g, 256, 0, n, p0, p1, p2, p3, out); break;
    case PM_TYPE_Q5_K: KLAUNCH(L, (k_dequant<PM_TYPE_Q5_K, 256>), g, 256, 0, n, p0, p1, p2, p3, out); break;
    case PM_TYPE_IQ3_S: KLAUNCH(L, (k_dequant<PM_TYPE_IQ3_S, 256>), g, 256, 0, n, p0, p1, p2, p3, out); break;
    case PM_TYPE_GLM_Q4: KLAUNCH(L, (k_dequant<PM_TYPE_GLM_Q4, 64>), g, 256, 0, n, p0, p1, p2, p3, out); break;
  }
}

// ===========================================================================
// activation quantiser: `Q8x::new` (src/ds4_cpu.rs:13-35)
// ===========================================================================
// one warp per 256-value block, 8 blocks per CTA; lane L holds values L, L+32, ...
// so that value group j (32 consecutive values) is exactly register j across the warp
__global__ void __launch_bounds__(256) k_quant_q8x(const float *__restrict__ x, size_t n_blocks,
                                                  int8_t *q, float *d, int32_t *bsum, uint16_t *bm,
                                                  int32_t *xs) {
  size_t b = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (b >= n_blocks) return;
  int lane = threadIdx.x & 31;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; j++) v[j] = x[b * 256 + 32 * j + lane];
  float a = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; j++) a = fmaxf(a, fabsf(v[j]));
  a = pm_warp_max(a);
  float id = a != 0.0f ? __fdiv_rn(127.0f, a) : 0.0f;
  int tot = 0;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    int r = 0;
    if (a != 0.0f) {
      float f = roundf(__fmul_rn(v[j], id));  // half away from zero, as f32::round
      r = (int)fminf(fmaxf(f, -127.0f), 127.0f);
    }
    q[b * 256 + 32 * j + lane] = (int8_t)r;
    int s = __reduce_add_sync(PM_FULL, r);
    tot += s;
    if (lane == 0) {
      bsum[b * 8 + j] = s;
      if (bm) {  // s = 64 * (s >> 6) + (s & 63), both parts exact in f16
        bm[b * 16 + j] = __half_as_ushort(__int2half_rn((s >> 6) * 64));
        bm[b * 16 + 8 + j] = __half_as_ushort(__int2half_rn(s & 63));
      }
    }
  }
  if (lane == 0) {
    d[b] = a != 0.0f ? __fdiv_rn(a, 127.0f) : 0.0f;
    if (xs) xs[b] = tot;
  }
}

void launch_quant_q8x(const Launch &L, const float *x, size_t rows, int n, int8_t *q, float *d,
                      int32_t *bsum, uint16_t *bm, int32_t *xs) {
  size_t nb = rows * (size_t)(n / 256);
  if (nb == 0) return;
  KLAUNCH(L, k_quant_q8x, (unsigned)((nb + 7) / 8), 256, 0, x, nb, q, d, bsum, bm, xs);
}

// `Q8::new` (src/q4x_cpu.rs:23-37): per 32 values amax, d = amax / 127, values rounded
// half away from zero and clamped; an all-zero block keeps d = 0. One warp per block.
// f16_scale (PM_AQ_Q8_32_F16): the stored scale is rounded through f16, the values are not touched.
__global__ void __launch_bounds__(256) k_quant_q8_32(const float *__restrict__ x, size_t n_blocks,
                                                    int8_t *q, float *d, int f16_scale) {
  size_t b = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (b >= n_blocks) return;
  int lane = threadIdx.x & 31;
  float v = x[b * 32 + lane];
  float a = pm_warp_max(fabsf(v));
  int r = 0;
  if (a != 0.0f) {
    float id = __fdiv_rn(127.0f, a);
    float f = roundf(__fmul_rn(v, id));
    r = (int)fminf(fmaxf(f, -127.0f), 127.0f);
  }
  q[b * 32 + lane] = (int8_t)r;
  if (lane == 0) {
    float s = a != 0.0f ? __fdiv_rn(a, 127.0f) : 0.0f;
    if (f16_scale) s = __half2float(__float2half_rn(s));
    d[b] = s;
  }
}

void launch_quant_q8_32(const Launch &L, const float *x, size_t rows, int n, int8_t *q, float *d, bool f16_scale) {
  size_t nb = rows * (size_t)(n / 32);
  if (nb == 0) return;
  KLAUNCH(L, k_quant_q8_32, (unsigned)((nb + 7) / 8), 256, 0, x, nb, q, d, f16_scale ? 1 : 0);
}

// ===========================================================================
// router logits: `dot_f32` order (src/quant.rs:215-236; src/ds4.rs:1376-1383)
// ===========================================================================
// CTA = 8 warps; blockIdx.y = token, each warp one expert; x[t] staged in
// shared memory. lane L runs the fma chain over columns L, L+32, ...
__global__ void __launch_bounds__(256) k_router(const float *__restrict__ wr,
                                                const float *__restrict__ bias,
                                                const float *__restrict__ x, int E, int d,
                                                float *logits) {
  extern __shared__ float xs[];
  int t = blockIdx.y;
  for (int i = threadIdx.x; i < d; i += 256) xs[i] = x[(size_t)t * d + i];
  __syncthreads();
  int lane = threadIdx.x & 31;
  int e = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (e >= E) return;
  const float *w = wr + (size_t)e * d;
  float acc = 0.0f;
  for (int c = lane; c < d; c += 32) acc = __fmaf_rn(w[c], xs[c], acc);
  float s = pm_warp_sum_dot(acc);
  if (lane == 0) {
    if (bias) s = __fadd_rn(s, bias[e]);
    logits[(size_t)t * E + e] = s;
  }
}

// The same sums for many tokens: a warp owns EXP experts x TOK tokens (TOK * EXP accumulators a
// lane), a CTA 8 * EXP experts x TOK tokens; the tokens' columns are staged in shared memory
// 512 at a time. Lane L still runs, for every (token, expert), the fma chain over columns
// L, L+32, ... in ascending order, so the result has the bits of k_router; the router
// row is read once per TOK tokens instead of once per token.
// 8 x 8 tiles have the fewest loads per fma (a 4096-token call on 256 experts is 2048 CTAs). While
// such a grid does not even fill the SMs (512 tokens on 128 experts: 128 CTAs of 8 warps, every
// column an L2 round trip that nothing hides) 4 x 4 tiles give four times the CTAs at a quarter of
// the registers, several CTAs an SM, with UNROLL columns' router loads in flight together
// (512 tokens on 128 experts: 45 -> 29 us a call).
#define RT_CH 512
template <int TOK, int EXP, int UNROLL>
__global__ void __launch_bounds__(256) k_router_tile(const float *__restrict__ wr,
                                                     const float *__restrict__ bias,
                                                     const float *__restrict__ x, int T, int E, int d,
                                                     float *logits) {
  __shared__ float xs[TOK][RT_CH];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t0 = blockIdx.y * TOK, e0 = blockIdx.x * (8 * EXP) + warp * EXP;
  float acc[TOK][EXP];
#pragma unroll
  for (int t = 0; t < TOK; t++)
#pragma unroll
    for (int e = 0; e < EXP; e++) acc[t][e] = 0.0f;
  for (int c0 = 0; c0 < d; c0 += RT_CH) {
    const int n = min(RT_CH, d - c0);  // a multiple of 32 (d is)
    __syncthreads();
    for (int i = threadIdx.x; i < TOK * RT_CH; i += 256) {
      const int t = i / RT_CH, c = i - t * RT_CH;
      xs[t][c] = (t0 + t < T && c < n) ? x[(size_t)(t0 + t) * d + c0 + c] : 0.0f;
    }
    __syncthreads();
    if (e0 < E) {
#pragma unroll UNROLL
      for (int c = lane; c < n; c += 32) {
        float w[EXP], xv[TOK];
#pragma unroll
        for (int e = 0; e < EXP; e++) w[e] = e0 + e < E ? __ldg(wr + (size_t)(e0 + e) * d + c0 + c) : 0.0f;
#pragma unroll
        for (int t = 0; t < TOK; t++) xv[t] = xs[t][c];
#pragma unroll
        for (int t = 0; t < TOK; t++)
#pragma unroll
          for (int e = 0; e < EXP; e++) acc[t][e] = __fmaf_rn(w[e], xv[t], acc[t][e]);
      }
    }
  }
  if (e0 >= E) return;
#pragma unroll
  for (int t = 0; t < TOK; t++)
#pragma unroll
    for (int e = 0; e < EXP; e++) {
      float s = pm_warp_sum_dot(acc[t][e]);
      if (lane == 0 && t0 + t < T && e0 + e < E) {
        if (bias) s = __fadd_rn(s, bias[e0 + e]);
        logits[(size_t)(t0 + t) * E + e0 + e] = s;
      }
    }
}

void launch_router(const Launch &L, const LayerDev &ly, const float *x, int T, float *logits) {
  if (T == 0) return;
  int E = ly.desc.n_exp, d = ly.desc.d;
  if (T >= 8) {
    dim3 grid((E + 63) / 64, (T + 7) / 8);
    if ((int)(grid.x * grid.y) <= L.n_sm) {
      dim3 g4((E + 31) / 32, (T + 3) / 4);
      KLAUNCH(L, (k_router_tile<4, 4, 4>), g4, 256, 0, ly.router, ly.logit_bias, x, T, E, d, logits);
    } else if ((int)(grid.x * grid.y) <= 2 * L.n_sm) {  // (2048 tokens on 32 experts: 1.62 -> 1.30 ms of a 24-layer step)
      KLAUNCH(L, (k_router_tile<8, 8, 2>), grid, 256, 0, ly.router, ly.logit_bias, x, T, E, d, logits);
    } else {  // (4096 tokens on 256 experts: two columns in flight measured 4 % slower)
      KLAUNCH(L, (k_router_tile<8, 8, 1>), grid, 256, 0, ly.router, ly.logit_bias, x, T, E, d, logits);
    }
    return;
  }
  dim3 grid((E + 7) / 8, T);
  // (x is staged in d * 4 bytes of dynamic shared memory: beyond 48 KB that needs the opt-in; the
  // layer descriptor is refused above PM_MAX_D, which fits)
  if ((size_t)d * 4 > 48 * 1024) cudaFuncSetAttribute(k_router, cudaFuncAttributeMaxDynamicSharedMemorySize, d * 4);
  KLAUNCH(L, k_router, grid, 256, (size_t)d * 4, ly.router, ly.logit_bias, x, E, d, logits);
}

__global__ void __launch_bounds__(256) k_gate_logit(const float *__restrict__ wv,
                                                    const float *__restrict__ x, int T, int d,
                                                    float *out) {
  int lane = threadIdx.x & 31;
  int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  float acc = 0.0f;
  for (int c = lane; c < d; c += 32) acc = __fmaf_rn(wv[c], x[(size_t)t * d + c], acc);
  float s = pm_warp_sum_dot(acc);
  if (lane == 0) out[t] = s;
}
void launch_shared_gate_logit(const Launch &L, const LayerDev &ly, const float *x, int T,
                              float *out) {
  if (T == 0) return;
  KLAUNCH(L, k_gate_logit, (T + 7) / 8, 256, 0, ly.shared_gate_inp, x, T, ly.desc.d, out);
}

// ===========================================================================
// top-k and weights (src/moe_kernels.rs:1019-1081, src/oss_kernels.rs:15-35,
// src/ds4.rs:1371-1426, src/q4x.rs:2213-2231)
// ===========================================================================
// one warp per token
__global__ void __launch_bounds__(128) k_route(pm_layer_desc D, const float *__restrict__ logits,
                                               const float *__restrict__ sel_bias, int T,
                                               uint32_t *ids, float *wout) {
  __shared__ float sm_sv[4][PM_MAX_EXPERTS];
  __shared__ float sm_gs[4][PM_MAX_EXPERTS / 2];
  __shared__ unsigned char sm_keep[4][PM_MAX_EXPERTS / 2];
  int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
  int t = blockIdx.x * 4 + wi;
  if (t >= T) return;
  pm_route_warp(D, logits + (size_t)t * D.n_exp, sel_bias, lane, sm_sv[wi], sm_gs[wi], sm_keep[wi],
                ids + (size_t)t * D.top_k, wout + (size_t)t * D.top_k);
}

void launch_route(const Launch &L, const LayerDev &ly, const float *logits, int T, uint32_t *ids,
                  float *w) {
  if (T == 0) return;
  KLAUNCH(L, k_route, (T + 3) / 4, 128, 0, ly.desc, logits, ly.select_bias, T, ids, w);
}

// ===========================================================================
// dispatch plan (src/moe_kernels.rs:1083-1129 layout; ascending (token, k)
// within an expert as src/ds4.rs:1461-1472)
// ===========================================================================
__global__ void k_plan_zero(uint32_t *cnt, int E) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < E) cnt[i] = 0;
}
// An expert id outside [0, E) (a caller's device buffer, or a peer's message under expert
// parallelism) is never used as an index: its pair is left out of every expert's list, its
// pair_pos becomes PM_PAIR_NONE (read as a zero row by combine) and the context's error word
// is set so that the call reports PM_ERR_INVALID at its next synchronisation.
__global__ void k_plan_count(const uint32_t *__restrict__ ids, int P, int E, uint32_t *cnt,
                             uint32_t *pair_pos, int *err) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  uint32_t e = ids[i];
  if (e < (uint32_t)E) {
    atomicAdd(&cnt[e], 1u);
  } else {
    pair_pos[i] = PM_PAIR_NONE;
    if (err) atomicCAS(err, 0, PM_DEVERR_BAD_EXPERT_ID);
  }
}
// single CTA of 512 threads: exclusive scans over the experts
__global__ void __launch_bounds__(512) k_plan_scan(PlanDev pl, int E, uint32_t *usage) {
  __shared__ uint32_t s_c[PM_MAX_EXPERTS], s_a[PM_MAX_EXPERTS];
  int e = threadIdx.x;
  uint32_t c = e < E ? pl.cnt[e] : 0;
  s_c[e] = c;
  s_a[e] = c > 0;
  __syncthreads();
  // Hillis-Steele inclusive scans (512 wide)
  for (int off = 1; off < PM_MAX_EXPERTS; off <<= 1) {
    uint32_t vc = e >= off ? s_c[e - off] : 0, va = e >= off ? s_a[e - off] : 0;
    __syncthreads();
    s_c[e] += vc;
    s_a[e] += va;
    __syncthreads();
  }
  uint32_t o = s_c[e] - c, na = s_a[e] - (c > 0);
  if (e < E) {
    pl.base[e] = o;
    if (c > 0) {
      pl.active[na] = (uint32_t)e;
      pl.offset[na] = o;
      pl.count[na] = c;
      if (usage) usage[e] += c;
    }
  }
  __syncthreads();
  uint32_t total_a = s_a[PM_MAX_EXPERTS - 1];
  if (e < E && (uint32_t)e >= total_a) {
    pl.active[e] = 0;
    pl.offset[e] = 0;
    pl.count[e] = 0;
  }
  if (e == 0) *pl.n_active = (int)total_a;
}
// one CTA per expert walks all pairs in order: stable placement
__global__ void __launch_bounds__(256) k_plan_place(const uint32_t *__restrict__ ids, int P, int K,
                                                    PlanDev pl) {
  __shared__ uint32_t wsum[8];
  uint32_t e = blockIdx.x;
  uint32_t total = pl.cnt[e];
  if (total == 0) return;
  uint32_t base = pl.base[e];
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t run = 0;
  for (int i0 = 0; i0 < P && run < total; i0 += 256) {
    int i = i0 + threadIdx.x;
    bool hit = i < P && ids[i] == e;
    uint32_t bal = __ballot_sync(PM_FULL, hit);
    if (lane == 0) wsum[warp] = __popc(bal);
    __syncthreads();
    uint32_t before = 0, all = 0;
#pragma unroll
    for (int w = 0; w < 8; w++) {
      uint32_t v = wsum[w];
      if (w < warp) before += v;
      all += v;
    }
    if (hit) {
      uint32_t p = base + run + before + __popc(bal & ((1u << lane) - 1));
      pl.pair_pos[i] = p;
      pl.pair_token[p] = (uint32_t)(i / K);
      pl.pair_src[p] = (uint32_t)i;
    }
    run += all;
    __syncthreads();
  }
}

void launch_plan(const Launch &L, const LayerDev &ly, const uint32_t *ids, int T, PlanDev pl, int *err) {
  int E = ly.desc.n_exp, K = ly.desc.top_k, P = T * K;
  KLAUNCH(L, k_plan_zero, (E + 255) / 256, 256, 0, pl.cnt, E);
  if (P > 0) KLAUNCH(L, k_plan_count, (P + 255) / 256, 256, 0, ids, P, E, pl.cnt, pl.pair_pos, err);
  KLAUNCH(L, k_plan_scan, 1, 512, 0, pl, E, ly.usage);
  if (P > 0) KLAUNCH(L, k_plan_place, E, 256, 0, ids, P, K, pl);
}

// Router logits, top-k and the dispatch plan of a few tokens (T < 8) in ONE launch: the grid of
// k_router computes the logits; the CTA that finishes last (a ticket counter; nobody waits for
// anybody) routes every token, one warp each, and builds the plan in shared memory. Six launches of a
// decode step become one; the values are those of k_router, k_route and k_plan_*.
#define RS_TOK 8   /* tokens (= warps of the last CTA) */
__global__ void __launch_bounds__(256) k_route_plan_small(pm_layer_desc D, const float *__restrict__ wr,
                                                          const float *__restrict__ bias,
                                                          const float *__restrict__ sel_bias,
                                                          const float *__restrict__ x, int T, float *logits,
                                                          uint32_t *ids, float *wout, PlanDev pl, uint32_t *usage,
                                                          const int32_t *__restrict__ slot_table, unsigned int *ticket) {
  extern __shared__ float xs[];  // d floats (the token's row), reused by the last CTA
  const int E = D.n_exp, d = D.d, K = D.top_k;
  const int t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < d; i += 256) xs[i] = x[(size_t)t * d + i];
  __syncthreads();
  {
    const int e = blockIdx.x * 8 + warp;
    if (e < E) {
      const float *w = wr + (size_t)e * d;
      float acc = 0.0f;
      for (int c = lane; c < d; c += 32) acc = __fmaf_rn(w[c], xs[c], acc);
      float s = pm_warp_sum_dot(acc);
      if (lane == 0) {
        if (bias) s = __fadd_rn(s, bias[e]);
        logits[(size_t)t * E + e] = s;
      }
    }
  }
  __shared__ unsigned int s_last;
  __threadfence();  // this CTA's logits before its ticket
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(ticket, 1u) == gridDim.x * gridDim.y - 1 ? 1u : 0u;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (tid == 0) *ticket = 0;  // ready for the next launch (graph replays included)

  // ---- the last CTA: top-k per token (warp = token) ----
  __shared__ float sm_lg[RS_TOK][PM_MAX_EXPERTS];
  __shared__ float sm_sv[RS_TOK][PM_MAX_EXPERTS];
  __shared__ float sm_gs[RS_TOK][PM_MAX_EXPERTS / 2];
  __shared__ unsigned char sm_keep[RS_TOK][PM_MAX_EXPERTS / 2];
  __shared__ uint32_t s_ids[RS_TOK * PM_MAX_TOPK];
  __shared__ uint32_t s_cnt[PM_MAX_EXPERTS], s_base[PM_MAX_EXPERTS], s_act[PM_MAX_EXPERTS];
  if (warp < T) {
    for (int e = lane; e < E; e += 32) sm_lg[warp][e] = __ldcg(logits + (size_t)warp * E + e);
    __syncwarp();
    pm_route_warp(D, sm_lg[warp], sel_bias, lane, sm_sv[warp], sm_gs[warp], sm_keep[warp], ids + (size_t)warp * K,
                  wout + (size_t)warp * K);
    __syncwarp();
  }
  for (int e = tid; e < PM_MAX_EXPERTS; e += 256) s_cnt[e] = 0;
  __syncthreads();
  // ---- the plan of the P = T * K pairs (src/moe_kernels.rs:1083-1129 layout) ----
  const int P = T * K;
  if (tid < P) {
    uint32_t e = ids[tid];  // written by this CTA's warps above
    if (slot_table) {  // a placement table: everything from here on names slots; use is counted by expert
      if (usage) atomicAdd(&usage[e], 1u);
      e = (uint32_t)slot_table[e];
      ids[tid] = e;
    }
    s_ids[tid] = e;
    atomicAdd(&s_cnt[e], 1u);
  }
  __syncthreads();
  if (tid == 0) {  // E <= 512 counts: one thread's pass is shorter than a scan's barriers
    uint32_t o = 0, na = 0;
    for (int e = 0; e < E; e++) {
      const uint32_t c = s_cnt[e];
      s_base[e] = o;
      pl.base[e] = o;
      pl.cnt[e] = c;
      if (c) {
        pl.active[na] = (uint32_t)e;
        pl.offset[na] = o;
        pl.count[na] = c;
        if (usage && !slot_table) usage[e] += c;
        na++;
      }
      o += c;
    }
    s_act[0] = na;
    *pl.n_active = (int)na;
  }
  __syncthreads();
  for (int e = (int)s_act[0] + tid; e < E; e += 256) {
    pl.active[e] = 0;
    pl.offset[e] = 0;
    pl.count[e] = 0;
  }
  if (tid < P) {  // stable: a pair goes behind the earlier pairs of its expert
    const uint32_t e = s_ids[tid];
    uint32_t before = 0;
    for (int j = 0; j < tid; j++) before += s_ids[j] == e;
    const uint32_t p = s_base[e] + before;
    pl.pair_pos[tid] = p;
    pl.pair_token[p] = (uint32_t)(tid / K);
    pl.pair_src[p] = (uint32_t)tid;
  }
}

// T < 8 tokens; ticket: a zeroed word of the context
void launch_route_plan_small(const Launch &L, const LayerDev &ly, const float *x, int T, float *logits, uint32_t *ids,
                             float *w, PlanDev pl, const int32_t *slot_table, unsigned int *ticket) {
  const int E = ly.desc.n_exp, d = ly.desc.d;
  dim3 grid((E + 7) / 8, T);
  // (its static arrays take most of the 48 KB a kernel gets without asking; the attribute is raised on
  // a layer's first call, which is never inside a stream capture)
  static int smem_set = 0;
  if (d * 4 > smem_set) {
    cudaFuncSetAttribute(k_route_plan_small, cudaFuncAttributeMaxDynamicSharedMemorySize, d * 4);
    smem_set = d * 4;
  }
  KLAUNCH(L, k_route_plan_small, grid, 256, (size_t)d * 4, ly.desc, ly.router, ly.logit_bias, ly.select_bias, x, T, logits,
          ids, w, pl, ly.usage, slot_table, ticket);
}

__global__ void k_iota(uint32_t *p, uint32_t n) {
  uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = i;
}
void launch_iota(const Launch &L, uint32_t *p, uint32_t n) {
  if (n) KLAUNCH(L, k_iota, (n + 255) / 256, 256, 0, p, n);
}

// ===========================================================================
// rows
// ===========================================================================

// Q4_K row . Q8x activations, one warp; every lane returns the row's sum.
// Integer sums per block as `row_scalar` (src/ds4_cpu.rs:59-83), the float
// term of block b = x.d[b]*(d*isum - dmin*msum), added in block order.
__device__ __forceinline__ float row_q4k_q8x(const uint8_t *__restrict__ rowp, int nb,
                                             const int8_t *__restrict__ xq,
                                             const float *__restrict__ xd,
                                             const int32_t *__restrict__ xbsum, int lane) {
  float total = 0.0f;
  const int nchunks = nb * 4;  // 32-byte chunks of quants: block b = ci/4, c = ci%4
  for (int c0 = 0; c0 < nchunks; c0 += 32) {
    int ci = c0 + lane;
    bool valid = ci < nchunks;
    int b = ci >> 2, c = ci & 3;
    int pi = 0, pm = 0;
    float dd = 0.0f, dmin = 0.0f;
    if (valid) {
      const uint8_t *blk = rowp + (size_t)b * 144;
      uint4 hdr = __ldg((const uint4 *)blk);
      const uint4 *qp = (const uint4 *)(blk + 16 + 32 * c);
      uint4 q0 = __ldg(qp), q1 = __ldg(qp + 1);
      const int4 *xp = (const int4 *)(xq + (size_t)b * 256 + 64 * c);
      int4 xl0 = xp[0], xl1 = xp[1], xh0 = xp[2], xh1 = xp[3];
      int lo = 0, hi = 0;
      const uint32_t M = 0x0f0f0f0fu;
      lo = __dp4a((int)(q0.x & M), xl0.x, lo); hi = __dp4a((int)((q0.x >> 4) & M), xh0.x, hi);
      lo = __dp4a((int)(q0.y & M), xl0.y, lo); hi = __dp4a((int)((q0.y >> 4) & M), xh0.y, hi);
      lo = __dp4a((int)(q0.z & M), xl0.z, lo); hi = __dp4a((int)((q0.z >> 4) & M), xh0.z, hi);
      lo = __dp4a((int)(q0.w & M), xl0.w, lo); hi = __dp4a((int)((q0.w >> 4) & M), xh0.w, hi);
      lo = __dp4a((int)(q1.x & M), xl1.x, lo); hi = __dp4a((int)((q1.x >> 4) & M), xh1.x, hi);
      lo = __dp4a((int)(q1.y & M), xl1.y, lo); hi = __dp4a((int)((q1.y >> 4) & M), xh1.y, hi);
      lo = __dp4a((int)(q1.z & M), xl1.z, lo); hi = __dp4a((int)((q1.z >> 4) & M), xh1.z, hi);
      lo = __dp4a((int)(q1.w & M), xl1.w, lo); hi = __dp4a((int)((q1.w >> 4) & M), xh1.w, hi);
      int sc0, m0, sc1, m1;
      pm_q4k_scmin(hdr.y, hdr.z, hdr.w, 2 * c, sc0, m0);
      pm_q4k_scmin(hdr.y, hdr.z, hdr.w, 2 * c + 1, sc1, m1);
      pi = sc0 * lo + sc1 * hi;
      pm = m0 * xbsum[b * 8 + 2 * c] + m1 * xbsum[b * 8 + 2 * c + 1];
      dd = pm_f16(hdr.x);
      dmin = pm_f16(hdr.x >> 16);
    }
    pi += __shfl_xor_sync(PM_FULL, pi, 1);
    pm += __shfl_xor_sync(PM_FULL, pm, 1);
    pi += __shfl_xor_sync(PM_FULL, pi, 2);
    pm += __shfl_xor_sync(PM_FULL, pm, 2);
    float term = 0.0f;
    if (valid)
      term = __fmul_rn(xd[b], __fsub_rn(__fmul_rn(dd, (float)pi), __fmul_rn(dmin, (float)pm)));
    int nblk = min(8, nb - (c0 >> 2));
    for (int j = 0; j < nblk; j++) total = __fadd_rn(total, __shfl_sync(PM_FULL, term, 4 * j));
  }
  return total;
}

// Two Q4_K rows against the same Q8x activations (a gate row and its up row, or two down rows): the
// loads of both rows leave together and the activations are read once, so a warp keeps twice the
// weight bytes in flight; per row the same operations in the same order as row_q4k_q8x.
__device__ __forceinline__ void rows2_q4k_q8x(const uint8_t *__restrict__ rowA, const uint8_t *__restrict__ rowB,
                                              int nb, const int8_t *__restrict__ xq, const float *__restrict__ xd,
                                              const int32_t *__restrict__ xbsum, int lane, float &outA, float &outB) {
  float totA = 0.0f, totB = 0.0f;
  const int nchunks = nb * 4;
  const uint32_t M = 0x0f0f0f0fu;
  for (int c0 = 0; c0 < nchunks; c0 += 32) {
    const int ci = c0 + lane;
    const bool valid = ci < nchunks;
    const int b = ci >> 2, c = ci & 3;
    int piA = 0, pmA = 0, piB = 0, pmB = 0;
    float ddA = 0.0f, dmA = 0.0f, ddB = 0.0f, dmB = 0.0f;
    if (valid) {
      const uint8_t *ba = rowA + (size_t)b * 144, *bb = rowB + (size_t)b * 144;
      const uint4 ha = __ldg((const uint4 *)ba), hb = __ldg((const uint4 *)bb);
      const uint4 *qa = (const uint4 *)(ba + 16 + 32 * c), *qb = (const uint4 *)(bb + 16 + 32 * c);
      const uint4 a0 = __ldg(qa), a1 = __ldg(qa + 1), b0 = __ldg(qb), b1 = __ldg(qb + 1);
      const int4 *xp = (const int4 *)(xq + (size_t)b * 256 + 64 * c);
      const int4 xl0 = xp[0], xl1 = xp[1], xh0 = xp[2], xh1 = xp[3];
      const int s0 = xbsum[b * 8 + 2 * c], s1 = xbsum[b * 8 + 2 * c + 1];
      const uint32_t wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const uint32_t wb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      const int xl[8] = {xl0.x, xl0.y, xl0.z, xl0.w, xl1.x, xl1.y, xl1.z, xl1.w};
      const int xh[8] = {xh0.x, xh0.y, xh0.z, xh0.w, xh1.x, xh1.y, xh1.z, xh1.w};
      int loA = 0, hiA = 0, loB = 0, hiB = 0;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        loA = __dp4a((int)(wa[i] & M), xl[i], loA);
        hiA = __dp4a((int)((wa[i] >> 4) & M), xh[i], hiA);
        loB = __dp4a((int)(wb[i] & M), xl[i], loB);
        hiB = __dp4a((int)((wb[i] >> 4) & M), xh[i], hiB);
      }
      int sc0, m0, sc1, m1;
      pm_q4k_scmin(ha.y, ha.z, ha.w, 2 * c, sc0, m0);
      pm_q4k_scmin(ha.y, ha.z, ha.w, 2 * c + 1, sc1, m1);
      piA = sc0 * loA + sc1 * hiA;
      pmA = m0 * s0 + m1 * s1;
      pm_q4k_scmin(hb.y, hb.z, hb.w, 2 * c, sc0, m0);
      pm_q4k_scmin(hb.y, hb.z, hb.w, 2 * c + 1, sc1, m1);
      piB = sc0 * loB + sc1 * hiB;
      pmB = m0 * s0 + m1 * s1;
      ddA = pm_f16(ha.x);
      dmA = pm_f16(ha.x >> 16);
      ddB = pm_f16(hb.x);
      dmB = pm_f16(hb.x >> 16);
    }
    piA += __shfl_xor_sync(PM_FULL, piA, 1);
    pmA += __shfl_xor_sync(PM_FULL, pmA, 1);
    piB += __shfl_xor_sync(PM_FULL, piB, 1);
    pmB += __shfl_xor_sync(PM_FULL, pmB, 1);
    piA += __shfl_xor_sync(PM_FULL, piA, 2);
    pmA += __shfl_xor_sync(PM_FULL, pmA, 2);
    piB += __shfl_xor_sync(PM_FULL, piB, 2);
    pmB += __shfl_xor_sync(PM_FULL, pmB, 2);
    float tA = 0.0f, tB = 0.0f;
    if (valid) {
      const float x = xd[b];
      tA = __fmul_rn(x, __fsub_rn(__fmul_rn(ddA, (float)piA), __fmul_rn(dmA, (float)pmA)));
      tB = __fmul_rn(x, __fsub_rn(__fmul_rn(ddB, (float)piB), __fmul_rn(dmB, (float)pmB)));
    }
    const int nblk = min(8, nb - (c0 >> 2));
    for (int j = 0; j < nblk; j++) {
      totA = __fadd_rn(totA, __shfl_sync(PM_FULL, tA, 4 * j));
      totB = __fadd_rn(totB, __shfl_sync(PM_FULL, tB, 4 * j));
    }
  }
  outA = totA;
  outB = totB;
}

// Q6_K row . Q8x activations (planes of this row given). Per block
// isum = sum_k sc[k] * sum_16 (q-32)*xq, term = x.d[b]*(d*isum), block order.
__device__ __forceinline__ float row_q6k_q8x(const uint8_t *__restrict__ ql,
                                             const uint8_t *__restrict__ qh,
                                             const uint8_t *__restrict__ sc,
                                             const uint8_t *__restrict__ dp, int nb,
                                             const int8_t *__restrict__ xq,
                                             const float *__restrict__ xd, int lane) {
  float total = 0.0f;
  const int n = lane >> 4, qtb = (lane >> 3) & 1, l4 = lane & 7;
  const int vA = 128 * n + 32 * qtb + 4 * l4;  // first value of the low-nibble quad
  for (int b = 0; b < nb; b++) {
    uint32_t qlw = __ldg((const uint32_t *)(ql + (size_t)b * 128) + lane);
    uint32_t qhw = __ldg((const uint32_t *)(qh + (size_t)b * 64) + n * 8 + l4);
    uint32_t qa = (qlw & 0x0f0f0f0fu) | (((qhw >> (2 * qtb)) & 0x03030303u) << 4);
    uint32_t qb = ((qlw >> 4) & 0x0f0f0f0fu) | (((qhw >> (2 * qtb + 4)) & 0x03030303u) << 4);
    qa = pm_sub32x4(qa);
    qb = pm_sub32x4(qb);
    const int *xp = (const int *)(xq + (size_t)b * 256);
    int xa = xp[vA >> 2], xb = xp[(vA + 64) >> 2];
    const int8_t *scb = (const int8_t *)(sc + (size_t)b * 16);
    int kA = vA >> 4;
    int isum = (int)scb[kA] * __dp4a((int)qa, xa, 0) + (int)scb[kA + 4] * __dp4a((int)qb, xb, 0);
    isum = pm_warp_sum_i32(isum);
    float d = pm_f16(__ldg((const uint16_t *)(dp + (size_t)b * 2)));
    total = __fadd_rn(total, __fmul_rn(xd[b], __fmul_rn(d, (float)isum)));
  }
  return total;
}

// row r of expert slot `el` of W against Q8x activations
__device__ __forceinline__ float row_q8x(const WMat &W, int el, int r, const int8_t *xq,
                                         const float *xd, const int32_t *xbsum, int lane) {
  int nb = W.cols / 256;
  if (W.type == PM_TYPE_Q4_K) {
    const uint8_t *rowp = W.plane[0] + (size_t)el * W.stride[0] + (size_t)r * nb * 144;
    return row_q4k_q8x(rowp, nb, xq, xd, xbsum, lane);
  }
  size_t rb = (size_t)r * nb;
  return row_q6k_q8x(W.plane[0] + (size_t)el * W.stride[0] + rb * 128,
                     W.plane[1] + (size_t)el * W.stride[1] + rb * 64,
                     W.plane[2] + (size_t)el * W.stride[2] + rb * 16,
                     W.plane[3] + (size_t)el * W.stride[3] + rb * 2, nb, xq, xd, lane);
}

// Q4_K row . 32-block Q8 activations (PM_AQ_Q8_32_F16). No reference code pairs them: row_scalar
// (src/ds4_cpu.rs:59-83) with the activation scale per 32-value sub-block j of a super-block,
// total += x.d[j] * ((d * sc_j) * isum_j - (dmin * m_j) * bsum_j), sub-blocks in ascending order.
// A lane takes a sub-block: 32 bytes of the block's quants hold sub-blocks 2c (low nibbles) and
// 2c + 1 (high nibbles). Not inlined: the callers' register budget is set by their hot branches.
__device__ __noinline__ float row_q4k_q8_32(const uint8_t *__restrict__ blks, int nb, const int8_t *__restrict__ xq,
                                            const float *__restrict__ xd, int lane) {
  float total = 0.0f;
  for (int b0 = 0; b0 < nb; b0 += 32) {
    const int b = b0 + lane;
    float term = 0.0f;
    if (b < nb) {
      const uint8_t *blk = blks + (size_t)(b >> 3) * 144;
      const int j = b & 7;
      const uint4 hdr = __ldg((const uint4 *)blk);
      const uint4 *qp = (const uint4 *)(blk + 16 + 32 * (j >> 1));
      const uint4 q0 = __ldg(qp), q1 = __ldg(qp + 1);
      const int sh = 4 * (j & 1);
      const uint32_t M = 0x0f0f0f0fu;
      const int4 *xp = (const int4 *)(xq + (size_t)b * 32);
      const int4 x0 = xp[0], x1 = xp[1];
      int is = 0, bs = 0;
      is = __dp4a((int)((q0.x >> sh) & M), x0.x, is); is = __dp4a((int)((q0.y >> sh) & M), x0.y, is);
      is = __dp4a((int)((q0.z >> sh) & M), x0.z, is); is = __dp4a((int)((q0.w >> sh) & M), x0.w, is);
      is = __dp4a((int)((q1.x >> sh) & M), x1.x, is); is = __dp4a((int)((q1.y >> sh) & M), x1.y, is);
      is = __dp4a((int)((q1.z >> sh) & M), x1.z, is); is = __dp4a((int)((q1.w >> sh) & M), x1.w, is);
      const int one = 0x01010101;
      bs = __dp4a(one, x0.x, bs); bs = __dp4a(one, x0.y, bs); bs = __dp4a(one, x0.z, bs); bs = __dp4a(one, x0.w, bs);
      bs = __dp4a(one, x1.x, bs); bs = __dp4a(one, x1.y, bs); bs = __dp4a(one, x1.z, bs); bs = __dp4a(one, x1.w, bs);
      int sc, mn;
      pm_q4k_scmin(hdr.y, hdr.z, hdr.w, j, sc, mn);
      const float dd = pm_f16(hdr.x), dmin = pm_f16(hdr.x >> 16);
      const float a = __fmul_rn(__fmul_rn(dd, (float)sc), (float)is);
      const float c = __fmul_rn(__fmul_rn(dmin, (float)mn), (float)bs);
      term = __fmul_rn(xd[b], __fsub_rn(a, c));
    }
    const int n = min(32, nb - b0);
    for (int jj = 0; jj < n; jj++) total = __fadd_rn(total, __shfl_sync(PM_FULL, term, jj));
  }
  return total;
}

// Q8_0 / IQ4_NL row . 32-block Q8 activations (src/q4x_cpu.rs:85-101): per block
// total += f16(d_w) * x.d[b] * (float)idot, left to right, in block order. Lanes take
// one block each; the 32 terms are then added in order.
__device__ __forceinline__ float row_q8_0_q8(const WMat &W, int el, int r, const int8_t *__restrict__ xq,
                                             const float *__restrict__ xd, int lane) {
  const int nb = W.cols / 32;  // 32-value units: a block of Q8_0 / IQ4_NL, a sub-block of IQ4_XS
  const bool xs = W.type == PM_TYPE_IQ4_XS;
  const bool nl = W.type == PM_TYPE_IQ4_NL || xs;
  float total = 0.0f;
  if (W.type == PM_TYPE_Q4_K) return row_q4k_q8_32(W.plane[0] + (size_t)el * W.stride[0] + (size_t)r * (nb / 8) * 144, nb, xq, xd, lane);
  if (W.type == PM_TYPE_IQ3_S) {  // src/q4x_cpu.rs:118-127: per sub-block ((d * scale) * x.d) * idot
    const uint8_t *blks = W.plane[0] + (size_t)el * W.stride[0] + (size_t)r * (nb / 8) * 108;
    const uint8_t *ds = W.plane[1] + (size_t)el * W.stride[1] + (size_t)r * (nb / 8) * 2;
    for (int b0 = 0; b0 < nb; b0 += 32) {
      const int b = b0 + lane;
      float term = 0.0f;
      if (b < nb) {
        uint32_t w[8];
        const int sc = pm_iq3s_sub(blks + (size_t)(b >> 3) * 108, b & 7, w);
        const int4 *xp = (const int4 *)(xq + (size_t)b * 32);
        const int4 x0 = xp[0], x1 = xp[1];
        int s = 0;
        s = __dp4a((int)w[0], x0.x, s); s = __dp4a((int)w[1], x0.y, s); s = __dp4a((int)w[2], x0.z, s); s = __dp4a((int)w[3], x0.w, s);
        s = __dp4a((int)w[4], x1.x, s); s = __dp4a((int)w[5], x1.y, s); s = __dp4a((int)w[6], x1.z, s); s = __dp4a((int)w[7], x1.w, s);
        const float d = pm_f16(__ldg((const uint16_t *)(ds + (size_t)(b >> 3) * 2)));
        term = __fmul_rn(__fmul_rn(__fmul_rn(d, (float)sc), xd[b]), (float)s);
      }
      const int n = min(32, nb - b0);
      for (int j = 0; j < n; j++) total = __fadd_rn(total, __shfl_sync(PM_FULL, term, j));
    }
    return total;
  }
  const uint8_t *vals = W.plane[0] + (size_t)el * W.stride[0] + (size_t)r * nb * (nl ? 16 : 32);
  const uint8_t *scl = W.plane[1] + (size_t)el * W.stride[1] + (size_t)r * (xs ? (nb / 8) * 8 : nb * 2);
  for (int b0 = 0; b0 < nb; b0 += 32) {
    const int b = b0 + lane;
    float term = 0.0f;
    if (b < nb) {
      const int4 *xp = (const int4 *)(xq + (size_t)b * 32);
      const int4 x0 = xp[0], x1 = xp[1];
      int s = 0;
      if (nl) {  // byte j: index of value j (low nibble) and of value j + 16 (high nibble)
        const uint4 w = __ldg((const uint4 *)(vals + (size_t)b * 16));
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        const int xl[4] = {x0.x, x0.y, x0.z, x0.w}, xh[4] = {x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
          s = __dp4a((int)pm_iq4nl_x4(ww[i] & 0x0f0f0f0fu), xl[i], s);
          s = __dp4a((int)pm_iq4nl_x4((ww[i] >> 4) & 0x0f0f0f0fu), xh[i], s);
        }
      } else {
        const int4 *wp = (const int4 *)(vals + (size_t)b * 32);
        const int4 w0 = __ldg(wp), w1 = __ldg(wp + 1);
        s = __dp4a(w0.x, x0.x, s); s = __dp4a(w0.y, x0.y, s); s = __dp4a(w0.z, x0.z, s); s = __dp4a(w0.w, x0.w, s);
        s = __dp4a(w1.x, x1.x, s); s = __dp4a(w1.y, x1.y, s); s = __dp4a(w1.z, x1.z, s); s = __dp4a(w1.w, x1.w, s);
      }
      float dw;
      if (xs) {  // d * (ls - 32) of sub-block b & 7 (src/q4x_cpu.rs:102-117)
        const uint2 hd = __ldg((const uint2 *)(scl + (size_t)(b >> 3) * 8));
        const int ib = b & 7;
        const int ls = (int)((hd.y >> (4 * ib)) & 15) | (int)((((hd.x >> 16) >> (2 * ib)) & 3) << 4);
        dw = __fmul_rn(pm_f16(hd.x), (float)(ls - 32));
      } else {
        dw = pm_f16(__ldg((const uint16_t *)(scl + (size_t)b * 2)));
      }
      term = __fmul_rn(__fmul_rn(dw, xd[b]), (float)s);
    }
    const int n = min(32, nb - b0);
    for (int j = 0; j < n; j++) total = __fadd_rn(total, __shfl_sync(PM_FULL, term, j));
  }
  return total;
}

// any type against f32 activations; lanes take quads of a 32-value block each
// (MXFP4: src/oss_batch.rs:774-789), f32 accumulation
__device__ __forceinline__ float row_f32(const WMat &W, int el, int r, const float *__restrict__ x,
                                         int lane) {
  float acc = 0.0f;
  if (W.type == PM_TYPE_MXFP4) {
    int nb = W.cols / 32;
    const uint8_t *nib = W.plane[0] + (size_t)el * W.stride[0] + (size_t)r * nb * 16;
    const uint8_t *scl = W.plane[1] + (size_t)el * W.stride[1] + (size_t)r * nb;
    // a lane takes whole blocks (16 bytes of codes, 32 activations): few, wide loads per row
    for (int b = lane; b < nb; b += 32) {
      const uint4 qv = __ldg((const uint4 *)(nib + (size_t)b * 16));
      const float s = pm_e8(__ldg(scl + b));
      const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
      const float4 *xp = (const float4 *)(x + b * 32);
      // An E2M1 code (sign, 2 exponent bits, 1 mantissa bit) placed at bits 15, 10..9 of an f16 is
      // that value times 2^-14 exactly (exponent 0 lands on the f16 subnormals 0 and 2^-15); the
      // doubled table of the reference (src/moe_kernels.rs:109) is 2^15 times the f16. Two codes
      // a word operation; the sums are exact products either way, only their order differs.
      float t = 0.0f;
#pragma unroll
      for (int w = 0; w < 4; w++) {  // byte j of the block: value j (low nibble), value j + 16 (high)
        const float4 x0 = xp[w], x1 = xp[4 + w];
        const uint32_t q = qw[w];
        const uint32_t ha = ((q << 9) & 0x0e000e00u) | ((q << 12) & 0x80008000u);   // bytes 0, 2 low
        const uint32_t hb = ((q << 1) & 0x0e000e00u) | ((q << 4) & 0x80008000u);    // bytes 1, 3 low
        const uint32_t hc = ((q << 5) & 0x0e000e00u) | ((q << 8) & 0x80008000u);    // bytes 0, 2 high
        const uint32_t hd = ((q >> 3) & 0x0e000e00u) | (q & 0x80008000u);           // bytes 1, 3 high
        const float2 fa = __half22float2(*reinterpret_cast<const __half2 *>(&ha));
        const float2 fb = __half22float2(*reinterpret_cast<const __half2 *>(&hb));
        const float2 fc = __half22float2(*reinterpret_cast<const __half2 *>(&hc));
        const float2 fd = __half22float2(*reinterpret_cast<const __half2 *>(&hd));
        t = __fmaf_rn(fa.x, x0.x, t);
        t = __fmaf_rn(fb.x, x0.y, t);
        t = __fmaf_rn(fa.y, x0.z, t);
        t = __fmaf_rn(fb.y, x0.w, t);
        t = __fmaf_rn(fc.x, x1.x, t);
        t = __fmaf_rn(fd.x, x1.y, t);
        t = __fmaf_rn(fc.y, x1.z, t);
        t = __fmaf_rn(fd.y, x1.w, t);
      }
      t = __fmul_rn(t, 32768.0f);
      acc = __fmaf_rn(s, t, acc);
    }
  } else if (W.type == PM_TYPE_GLM_Q4) {
    // `dot_q4_scalar` (src/quant.rs:464-476): per group of 64 the sum of level * x, then times the
    // group's scale; a lane takes whole groups (two 16-byte loads of nibbles, 64 activations)
    const int ng = W.cols / 64;
    const uint8_t *nib = W.plane[0] + (size_t)el * W.stride[0] + (size_t)r * ng * 32;
    const float *scl = (const float *)(W.plane[1] + (size_t)el * W.stride[1]) + (size_t)r * ng;
    for (int g = lane; g < ng; g += 32) {
      const uint4 q0 = __ldg((const uint4 *)(nib + (size_t)g * 32)), q1 = __ldg((const uint4 *)(nib + (size_t)g * 32 + 16));
      const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
      const float4 *xp = (const float4 *)(x + g * 64);
      float t = 0.0f;
#pragma unroll
      for (int w = 0; w < 8; w++) {  // a word = 8 consecutive values, low nibble first
        const float4 x0 = xp[2 * w], x1 = xp[2 * w + 1];
        const uint32_t q = qw[w];
        t = __fmaf_rn((float)((int)(q & 15) - 8), x0.x, t);
        t = __fmaf_rn((float)((int)((q >> 4) & 15) - 8), x0.y, t);
        t = __fmaf_rn((float)((int)((q >> 8) & 15) - 8), x0.z, t);
        t = __fmaf_rn((float)((int)((q >> 12) & 15) - 8), x0.w, t);
        t = __fmaf_rn((float)((int)((q >> 16) & 15) - 8), x1.x, t);
        t = __fmaf_rn((float)((int)((q >> 20) & 15) - 8), x1.y, t);
        t = __fmaf_rn((float)((int)((q >> 24) & 15) - 8), x1.z, t);
        t = __fmaf_rn((float)((int)(q >> 28) - 8), x1.w, t);
      }
      acc = __fmaf_rn(t, __ldg(scl + g), acc);
    }
  } else {
    const uint8_t *p0 = W.plane[0] + (size_t)el * W.stride[0];
    const uint8_t *p1 = W.plane[1] ? W.plane[1] + (size_t)el * W.stride[1] : nullptr;
    const uint8_t *p2 = W.plane[2] ? W.plane[2] + (size_t)el * W.stride[2] : nullptr;
    const uint8_t *p3 = W.plane[3] ? W.plane[3] + (size_t)el * W.stride[3] : nullptr;
    int bv = (W.type == PM_TYPE_Q8_0 || W.type == PM_TYPE_IQ4_NL) ? 32 : 256;
    size_t b0 = (size_t)r * (W.cols / bv);
    for (int v = lane; v < W.cols; v += 32) {
      float wv;
      size_t b = b0 + v / bv;
      int iv = v % bv;
      if (W.type == PM_TYPE_Q4_K) wv = deq_value<PM_TYPE_Q4_K>(p0, p1, p2, p3, b, iv);
      else if (W.type == PM_TYPE_Q6_K) wv = deq_value<PM_TYPE_Q6_K>(p0, p1, p2, p3, b, iv);
      else if (W.type == PM_TYPE_IQ4_NL) wv = deq_value<PM_TYPE_IQ4_NL>(p0, p1, p2, p3, b, iv);
      else if (W.type == PM_TYPE_IQ4_XS) wv = deq_value<PM_TYPE_IQ4_XS>(p0, p1, p2, p3, b, iv);
      else if (W.type == PM_TYPE_Q5_K) wv = deq_value<PM_TYPE_Q5_K>(p0, p1, p2, p3, b, iv);
      else if (W.type == PM_TYPE_IQ3_S) wv = deq_value<PM_TYPE_IQ3_S>(p0, p1, p2, p3, b, iv);
      else wv = deq_value<PM_TYPE_Q8_0>(p0, p1, p2, p3, b, iv);
      acc = __fmaf_rn(wv, x[v], acc);
    }
  }
  return pm_warp_sum_16_1(acc);
}

// NR MXFP4 rows against one f32 activation vector, the activations read once for all of them (a
// single row reads 8 times as many activation bytes as weight bytes, and the L1 path was what
// bound it). Per row the same operations in the same order as row_f32.
template <int NR>
__device__ __forceinline__ void rows_mx_f32(const uint8_t *const (&nib)[NR], const uint8_t *const (&scl)[NR], int nb,
                                            const float *__restrict__ x, int lane, float (&out)[NR]) {
  float acc[NR];
#pragma unroll
  for (int i = 0; i < NR; i++) acc[i] = 0.0f;
  for (int b = lane; b < nb; b += 32) {
    const float4 *xp = (const float4 *)(x + b * 32);
    float4 xv[8];
#pragma unroll
    for (int w = 0; w < 8; w++) xv[w] = xp[w];
#pragma unroll
    for (int i = 0; i < NR; i++) {
      const uint4 qv = __ldg((const uint4 *)(nib[i] + (size_t)b * 16));
      const float s = pm_e8(__ldg(scl[i] + b));
      const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
      float t = 0.0f;
#pragma unroll
      for (int w = 0; w < 4; w++) {
        const float4 x0 = xv[w], x1 = xv[4 + w];
        const uint32_t q = qw[w];
        const uint32_t ha = ((q << 9) & 0x0e000e00u) | ((q << 12) & 0x80008000u);
        const uint32_t hb = ((q << 1) & 0x0e000e00u) | ((q << 4) & 0x80008000u);
        const uint32_t hc = ((q << 5) & 0x0e000e00u) | ((q << 8) & 0x80008000u);
        const uint32_t hd = ((q >> 3) & 0x0e000e00u) | (q & 0x80008000u);
        const float2 fa = __half22float2(*reinterpret_cast<const __half2 *>(&ha));
        const float2 fb = __half22float2(*reinterpret_cast<const __half2 *>(&hb));
        const float2 fc = __half22float2(*reinterpret_cast<const __half2 *>(&hc));
        const float2 fd = __half22float2(*reinterpret_cast<const __half2 *>(&hd));
        t = __fmaf_rn(fa.x, x0.x, t);
        t = __fmaf_rn(fb.x, x0.y, t);
        t = __fmaf_rn(fa.y, x0.z, t);
        t = __fmaf_rn(fb.y, x0.w, t);
        t = __fmaf_rn(fc.x, x1.x, t);
        t = __fmaf_rn(fd.x, x1.y, t);
        t = __fmaf_rn(fc.y, x1.z, t);
        t = __fmaf_rn(fd.y, x1.w, t);
      }
      t = __fmul_rn(t, 32768.0f);
      acc[i] = __fmaf_rn(s, t, acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < NR; i++) out[i] = pm_warp_sum_16_1(acc[i]);
}

// gate/up for MXFP4 experts and f32 activations: a warp takes the gate and the up row of two
// consecutive h values (four rows an activation read); grid (ceil(ff / 16), groups)
__global__ void __launch_bounds__(256) k_gateup_mx(LayerDev ly, Groups g, const float *__restrict__ x,
                                                   const float *__restrict__ wts, float *h) {
  int a = blockIdx.y;
  if (a >= *g.n_groups) return;
  const WMat &G = ly.gate, &U = ly.up;
  const int ff = G.rows, d = G.cols, nb = d / 32;
  const int lane = threadIdx.x & 31;
  const int r = (blockIdx.x * 8 + (threadIdx.x >> 5)) * 2;
  if (r >= ff) return;
  const int r1 = min(r + 1, ff - 1);  // an odd ff: the last warp computes its row twice
  const int el = (int)g.expert[a] - ly.first_local;
  if (el < 0 || el >= ly.n_local) return;  // not held here
  const uint32_t off = g.offset[a], cnt = g.count[a];
  const pm_layer_desc &D = ly.desc;
  const bool fold = D.weight_fold == PM_FOLD_BEFORE_DOWN;
  const bool bias = ly.bias_gate != nullptr;
  const uint8_t *gn = G.plane[0] + (size_t)el * G.stride[0], *gs = G.plane[1] + (size_t)el * G.stride[1];
  const uint8_t *un = U.plane[0] + (size_t)el * U.stride[0], *us = U.plane[1] + (size_t)el * U.stride[1];
  const uint8_t *const nib[4] = {gn + (size_t)r * nb * 16, un + (size_t)r * nb * 16, gn + (size_t)r1 * nb * 16,
                                 un + (size_t)r1 * nb * 16};
  const uint8_t *const scl[4] = {gs + (size_t)r * nb, us + (size_t)r * nb, gs + (size_t)r1 * nb, us + (size_t)r1 * nb};
  for (uint32_t i = 0; i < cnt; i++) {
    const uint32_t p = off + i;
    float v[4];
    rows_mx_f32<4>(nib, scl, nb, x + (size_t)g.pair_token[p] * d, lane, v);
    if (lane < 2 && r + lane < ff) {
      const int rr = r + lane;
      float gv = lane ? v[2] : v[0], uv = lane ? v[3] : v[1];
      if (bias) {
        gv = __fadd_rn(gv, ly.bias_gate[(size_t)el * ff + rr]);
        uv = __fadd_rn(uv, ly.bias_up[(size_t)el * ff + rr]);
      }
      const float w = (fold && wts) ? wts[g.pair_src[p]] : 1.0f;
      h[(size_t)p * ff + rr] = pm_act(D.act, D.act_limit, D.act_alpha, gv, uv, w, fold && wts);
    }
  }
}

// down for MXFP4 experts and f32 hidden vectors: a warp takes four consecutive output rows;
// grid (ceil(d / 32), groups)
__global__ void __launch_bounds__(256) k_down_mx(LayerDev ly, Groups g, const float *__restrict__ h, float *eo) {
  int a = blockIdx.y;
  if (a >= *g.n_groups) return;
  const WMat &Dn = ly.down;
  const int d = Dn.rows, ff = Dn.cols, nb = ff / 32;
  const int lane = threadIdx.x & 31;
  const int r = (blockIdx.x * 8 + (threadIdx.x >> 5)) * 4;
  if (r >= d) return;
  const int el = (int)g.expert[a] - ly.first_local;
  const uint32_t off = g.offset[a], cnt = g.count[a];
  if (el < 0 || el >= ly.n_local) {  // not held here: zeros
    if (lane < 4 && r + lane < d)
      for (uint32_t i = 0; i < cnt; i++) eo[(size_t)(off + i) * d + r + lane] = 0.0f;
    return;
  }
  const uint8_t *dn = Dn.plane[0] + (size_t)el * Dn.stride[0], *ds = Dn.plane[1] + (size_t)el * Dn.stride[1];
  const int rr[4] = {r, min(r + 1, d - 1), min(r + 2, d - 1), min(r + 3, d - 1)};
  const uint8_t *const nib[4] = {dn + (size_t)rr[0] * nb * 16, dn + (size_t)rr[1] * nb * 16, dn + (size_t)rr[2] * nb * 16,
                                 dn + (size_t)rr[3] * nb * 16};
  const uint8_t *const scl[4] = {ds + (size_t)rr[0] * nb, ds + (size_t)rr[1] * nb, ds + (size_t)rr[2] * nb,
                                 ds + (size_t)rr[3] * nb};
  for (uint32_t i = 0; i < cnt; i++) {
    const uint32_t p = off + i;
    float v[4];
    rows_mx_f32<4>(nib, scl, nb, h + (size_t)p * ff, lane, v);
    if (lane < 4 && r + lane < d) {
      float o = lane == 0 ? v[0] : (lane == 1 ? v[1] : (lane == 2 ? v[2] : v[3]));
      if (ly.bias_down) o = __fadd_rn(o, ly.bias_down[(size_t)el * d + r + lane]);  // src/oss_batch.rs:89
      eo[(size_t)p * d + r + lane] = o;
    }
  }
}

// ===========================================================================
// grouped gate/up + activation, grouped down
// ===========================================================================
// grid (rows/8, groups); one warp per output row, looping over the group's pairs
__global__ void __launch_bounds__(256, 3) k_gateup(LayerDev ly, int shared, Groups g,
                                                const float *__restrict__ x,
                                                const int8_t *__restrict__ xq,
                                                const float *__restrict__ xd,
                                                const int32_t *__restrict__ xbsum,
                                                const float *__restrict__ wts, float *h) {
  int a = blockIdx.y;
  if (a >= *g.n_groups) return;
  const WMat &G = shared ? ly.sgate : ly.gate;
  const WMat &U = shared ? ly.sup : ly.up;
  const int ff = G.rows, d = G.cols;
  int lane = threadIdx.x & 31;
  int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= ff) return;
  int e = (int)g.expert[a];
  int el = shared ? 0 : e - ly.first_local;
  if (el < 0 || el >= (shared ? 1 : ly.n_local)) return;  // not held here
  uint32_t off = g.offset[a], cnt = g.count[a];
  const pm_layer_desc &D = ly.desc;
  const bool fold = !shared && D.weight_fold == PM_FOLD_BEFORE_DOWN;
  float bg = 0.0f, bu = 0.0f;
  const bool bias = !shared && ly.bias_gate;
  if (bias) {
    bg = ly.bias_gate[(size_t)el * ff + r];
    bu = ly.bias_up[(size_t)el * ff + r];
  }
  const int nbx = d / 256;
  for (uint32_t i = 0; i < cnt; i++) {
    uint32_t p = off + i;
    uint32_t t = g.pair_token[p];
    float gv, uv;
    if (D.act_quant == PM_AQ_Q8X_256) {
      const int8_t *q = xq + (size_t)t * d;
      const float *qd = xd + (size_t)t * nbx;
      const int32_t *qb = xbsum + (size_t)t * nbx * 8;
      if (G.type == PM_TYPE_Q4_K && U.type == PM_TYPE_Q4_K) {
        rows2_q4k_q8x(G.plane[0] + (size_t)el * G.stride[0] + (size_t)r * nbx * 144,
                      U.plane[0] + (size_t)el * U.stride[0] + (size_t)r * nbx * 144, nbx, q, qd, qb, lane, gv, uv);
      } else {
        gv = row_q8x(G, el, r, q, qd, qb, lane);
        uv = row_q8x(U, el, r, q, qd, qb, lane);
      }
    } else if (D.act_quant == PM_AQ_Q8_32 || D.act_quant == PM_AQ_Q8_32_F16) {
      const int8_t *q = xq + (size_t)t * d;
      const float *qd = xd + (size_t)t * (d / 32);
      gv = row_q8_0_q8(G, el, r, q, qd, lane);
      uv = row_q8_0_q8(U, el, r, q, qd, lane);
    } else {
      gv = row_f32(G, el, r, x + (size_t)t * d, lane);
      uv = row_f32(U, el, r, x + (size_t)t * d, lane);
    }
    if (lane == 0) {
      if (bias) {
        gv = __fadd_rn(gv, bg);
        uv = __fadd_rn(uv, bu);
      }
      float w = (fold && wts) ? wts[g.pair_src[p]] : 1.0f;
      h[(size_t)p * ff + r] = pm_act(D.act, D.act_limit, D.act_alpha, gv, uv, w, fold && wts);
    }
  }
}

__global__ void __launch_bounds__(256) k_down(LayerDev ly, int shared, Groups g,
                                              const float *__restrict__ h,
                                              const int8_t *__restrict__ hq,
                                              const float *__restrict__ hd,
                                              const int32_t *__restrict__ hbsum, float *eo) {
  int a = blockIdx.y;
  if (a >= *g.n_groups) return;
  const WMat &Dn = shared ? ly.sdown : ly.down;
  const int d = Dn.rows, ff = Dn.cols;
  int lane = threadIdx.x & 31;
  int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= d) return;
  int e = (int)g.expert[a];
  int el = shared ? 0 : e - ly.first_local;
  uint32_t off = g.offset[a], cnt = g.count[a];
  if (el < 0 || el >= (shared ? 1 : ly.n_local)) {  // not held here: zeros
    if (lane == 0)
      for (uint32_t i = 0; i < cnt; i++) eo[(size_t)(off + i) * d + r] = 0.0f;
    return;
  }
  const pm_layer_desc &D = ly.desc;
  float bd = (!shared && ly.bias_down) ? ly.bias_down[(size_t)el * d + r] : 0.0f;
  const int nbh = ff / 256;
  for (uint32_t i = 0; i < cnt; i++) {
    uint32_t p = off + i;
    float o;
    if (D.act_quant == PM_AQ_Q8X_256)
      o = row_q8x(Dn, el, r, hq + (size_t)p * ff, hd + (size_t)p * nbh,
                  hbsum + (size_t)p * nbh * 8, lane);
    else if (D.act_quant == PM_AQ_Q8_32 || D.act_quant == PM_AQ_Q8_32_F16)
      o = row_q8_0_q8(Dn, el, r, hq + (size_t)p * ff, hd + (size_t)p * (ff / 32), lane);
    else
      o = row_f32(Dn, el, r, h + (size_t)p * ff, lane);
    if (lane == 0) {
      if (!shared && ly.bias_down) o = __fadd_rn(o, bd);  // src/oss_batch.rs:89
      eo[(size_t)p * d + r] = o;
    }
  }
}

// down for Q4_K experts and Q8x hidden vectors: a warp takes two consecutive output rows
// (rows2_q4k_q8x); grid (ceil(d / 16), groups)
__global__ void __launch_bounds__(256, 3) k_down_q4k2(LayerDev ly, int shared, Groups g, const int8_t *__restrict__ hq,
                                                      const float *__restrict__ hd, const int32_t *__restrict__ hbsum,
                                                      float *eo) {
  int a = blockIdx.y;
  if (a >= *g.n_groups) return;
  const WMat &Dn = shared ? ly.sdown : ly.down;
  const int d = Dn.rows, ff = Dn.cols, nbh = ff / 256;
  const int lane = threadIdx.x & 31;
  const int r = (blockIdx.x * 8 + (threadIdx.x >> 5)) * 2;
  if (r >= d) return;
  const int r1 = min(r + 1, d - 1);
  const int el = shared ? 0 : (int)g.expert[a] - ly.first_local;
  const uint32_t off = g.offset[a], cnt = g.count[a];
  if (el < 0 || el >= (shared ? 1 : ly.n_local)) {  // not held here: zeros
    if (lane < 2 && r + lane < d)
      for (uint32_t i = 0; i < cnt; i++) eo[(size_t)(off + i) * d + r + lane] = 0.0f;
    return;
  }
  const uint8_t *base = Dn.plane[0] + (size_t)el * Dn.stride[0];
  const uint8_t *rowA = base + (size_t)r * nbh * 144, *rowB = base + (size_t)r1 * nbh * 144;
  const bool bias = !shared && ly.bias_down;
  for (uint32_t i = 0; i < cnt; i++) {
    const size_t p = off + i;
    float oA, oB;
    rows2_q4k_q8x(rowA, rowB, nbh, hq + p * ff, hd + p * nbh, hbsum + p * nbh * 8, lane, oA, oB);
    if (lane < 2 && r + lane < d) {
      float o = lane ? oB : oA;
      if (bias) o = __fadd_rn(o, ly.bias_down[(size_t)el * d + r + lane]);  // src/oss_batch.rs:89
      eo[p * d + r + lane] = o;
    }
  }
}

void launch_gateup(const Launch &L, const LayerDev &ly, bool shared, Groups g, int n_pairs,
                   const float *x, const int8_t *xq, const float *xd, const int32_t *xbsum,
                   const float *w, float *h) {
  if (n_pairs == 0) return;
  int ff = shared ? ly.sgate.rows : ly.gate.rows;
  if (!shared && ly.desc.act_quant == PM_AQ_F32 && ly.gate.type == PM_TYPE_MXFP4 && ly.up.type == PM_TYPE_MXFP4) {
    dim3 grid((ff + 15) / 16, min(g.max_groups, n_pairs));
    KLAUNCH(L, k_gateup_mx, grid, 256, 0, ly, g, x, w, h);
    return;
  }
  dim3 grid((ff + 7) / 8, min(g.max_groups, n_pairs));
  KLAUNCH(L, k_gateup, grid, 256, 0, ly, (int)shared, g, x, xq, xd, xbsum, w, h);
}
void launch_down(const Launch &L, const LayerDev &ly, bool shared, Groups g, int n_pairs,
                 const float *h, const int8_t *hq, const float *hd, const int32_t *hbsum,
                 float *eo) {
  if (n_pairs == 0) return;
  int d = ly.desc.d;
  if (!shared && ly.desc.act_quant == PM_AQ_F32 && ly.down.type == PM_TYPE_MXFP4) {
    dim3 grid((d + 31) / 32, min(g.max_groups, n_pairs));
    KLAUNCH(L, k_down_mx, grid, 256, 0, ly, g, h, eo);
    return;
  }
  if (ly.desc.act_quant == PM_AQ_Q8X_256 && (shared ? ly.sdown : ly.down).type == PM_TYPE_Q4_K) {
    dim3 grid((d + 15) / 16, min(g.max_groups, n_pairs));
    KLAUNCH(L, k_down_q4k2, grid, 256, 0, ly, (int)shared, g, hq, hd, hbsum, eo);
    return;
  }
  dim3 grid((d + 7) / 8, min(g.max_groups, n_pairs));
  KLAUNCH(L, k_down, grid, 256, 0, ly, (int)shared, g, h, hq, hd, hbsum, eo);
}

// ===========================================================================
// combine (src/moe_kernels.rs:1798-1808): fixed k order, then the shared expert
// ===========================================================================
__global__ void __launch_bounds__(256) k_combine(int d, int K, int in_combine,
                                                 const float *__restrict__ eo,
                                                 const uint32_t *__restrict__ pair_pos,
                                                 const float *__restrict__ w,
                                                 const float *__restrict__ shared_out,
                                                 const float *__restrict__ shared_logit, float *y,
                                                 int accumulate) {
  int t = blockIdx.y;
  int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= d) return;
  float s = 0.0f;
  for (int k = 0; k < K; k++) {
    const uint32_t p = pair_pos[t * K + k];
    float v = p == PM_PAIR_NONE ? 0.0f : eo[(size_t)p * d + c];  // a pair whose expert id was refused
    if (in_combine) v = __fmul_rn(w[t * K + k], v);
    s = __fadd_rn(s, v);
  }
  if (shared_out) {
    float sv = shared_out[(size_t)t * d + c];
    if (shared_logit)
      sv = __fmul_rn(sv, __fdiv_rn(1.0f, __fadd_rn(1.0f, pm_exp(-shared_logit[t]))));
    s = __fadd_rn(s, sv);
  }
  size_t o = (size_t)t * d + c;
  y[o] = accumulate ? __fadd_rn(y[o], s) : s;
}

void launch_combine(const Launch &L, const LayerDev &ly, const float *eo, const uint32_t *pair_pos,
                    const float *w, const float *shared_out, const float *shared_logit, int T,
                    float *y, bool accumulate) {
  if (T == 0) return;
  int d = ly.desc.d;
  dim3 grid((d + 255) / 256, T);
  KLAUNCH(L, k_combine, grid, 256, 0, d, ly.desc.top_k,
          (int)(ly.desc.weight_fold == PM_FOLD_IN_COMBINE), eo, pair_pos, w, shared_out,
          shared_logit, y, (int)accumulate);
}

// x / rms(x), unit weight; the sum order is pm_rms_inv's (common.cuh)
__global__ void __launch_bounds__(256) k_rmsnorm(const float *__restrict__ x, int T, int d,
                                                 float eps, float *out) {
  __shared__ float red8[8];
  int t = blockIdx.x;
  const float *xr = x + (size_t)t * d;
  float inv = pm_rms_inv(xr, d, eps, red8);
  for (int c = threadIdx.x; c < d; c += 256) out[(size_t)t * d + c] = __fmul_rn(xr[c], inv);
}
void launch_rmsnorm(const Launch &L, const float *x, int T, int d, float eps, float *out) {
  if (T == 0) return;
  KLAUNCH(L, k_rmsnorm, T, 256, 0, x, T, d, eps, out);
}

// ===========================================================================
// expert parallelism: the wire records of a dispatch (replaces the body of the
// bridge RUN message, src/bridge.rs:412-466: activations and (expert, weight) rows)
// ===========================================================================
// pairs routed to each rank's experts: cnt[e] summed over the rank's E / W experts
__global__ void k_ep_rank_counts(const uint32_t *__restrict__ cnt, int E, int W, int32_t *out) {
  int r = threadIdx.x;
  if (r >= W) return;
  int per = E / W, s = 0;
  for (int e = r * per; e < (r + 1) * per; e++) s += (int)cnt[e];
  out[r] = s;
}
void launch_ep_rank_counts(const Launch &L, const uint32_t *cnt, int E, int W, int32_t *out) {
  KLAUNCH(L, k_ep_rank_counts, 1, 64, 0, cnt, E, W, out);
}

// one CTA per pair p (dispatch-plan order: ascending expert, so every destination rank's
// pairs are contiguous): the token's row in its wire form and the pair's (expert, weight)
__global__ void __launch_bounds__(256) k_ep_pack(int P, int row_bytes, int nd, int nbs, const uint8_t *__restrict__ rows,
                                                 const float *__restrict__ xd, const int32_t *__restrict__ xbs,
                                                 const uint32_t *__restrict__ pair_token,
                                                 const uint32_t *__restrict__ pair_src, const uint32_t *__restrict__ ids,
                                                 const float *__restrict__ w, uint8_t *srows, float *sd, int32_t *sbs,
                                                 uint32_t *smeta) {
  const int p = blockIdx.x;
  if (p >= P) return;
  const uint32_t t = pair_token[p];
  const uint4 *src = (const uint4 *)(rows + (size_t)t * row_bytes);
  uint4 *dst = (uint4 *)(srows + (size_t)p * row_bytes);
  for (int i = threadIdx.x; i < row_bytes / 16; i += 256) dst[i] = src[i];
  for (int i = threadIdx.x; i < nd; i += 256) sd[(size_t)p * nd + i] = xd[(size_t)t * nd + i];
  for (int i = threadIdx.x; i < nbs; i += 256) sbs[(size_t)p * nbs + i] = xbs[(size_t)t * nbs + i];
  if (threadIdx.x == 0) {
    const uint32_t s = pair_src[p];
    smeta[2 * p] = ids[s];
    smeta[2 * p + 1] = __float_as_uint(w[s]);
  }
}
void launch_ep_pack(const Launch &L, int P, int row_bytes, int nd, int nbs, const void *rows, const float *xd,
                    const int32_t *xbs, const uint32_t *pair_token, const uint32_t *pair_src, const uint32_t *ids,
                    const float *w, void *srows, float *sd, int32_t *sbs, uint32_t *smeta) {
  if (P == 0) return;
  KLAUNCH(L, k_ep_pack, P, 256, 0, P, row_bytes, nd, nbs, (const uint8_t *)rows, xd, xbs, pair_token, pair_src, ids, w,
          (uint8_t *)srows, sd, sbs, smeta);
}

// received (expert, weight) records -> expert ids and weights; an expert this rank does not
// hold is reported through the error word (and mapped to the rank's first expert so that
// nothing indexes out of its planes)
__global__ void k_ep_unmeta(int R, const uint32_t *__restrict__ meta, int first, int n_local, uint32_t *eids, float *w,
                            int *err) {
  int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  uint32_t e = meta[2 * r];
  if (e < (uint32_t)first || e >= (uint32_t)(first + n_local)) {
    atomicCAS(err, 0, PM_DEVERR_BAD_EXPERT_ID);
    e = (uint32_t)first;
  }
  eids[r] = e;
  w[r] = __uint_as_float(meta[2 * r + 1]);
}
void launch_ep_unmeta(const Launch &L, int R, const uint32_t *meta, int first, int n_local, uint32_t *eids, float *w,
                      int *err) {
  if (R == 0) return;
  KLAUNCH(L, k_ep_unmeta, (R + 255) / 256, 256, 0, R, meta, first, n_local, eids, w, err);
}

// expert ids -> the slots that hold them (a placement table), counting the use of every expert
// on the way (the plan that follows sees slots, so it cannot)
__global__ void k_ep_slots(uint32_t *ids, int P, int E, const int32_t *__restrict__ table, uint32_t *usage) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  const uint32_t e = ids[i];
  if (e >= (uint32_t)E) return;  // the plan refuses it
  if (usage) atomicAdd(&usage[e], 1u);
  ids[i] = (uint32_t)table[e];
}
void launch_ep_slots(const Launch &L, uint32_t *ids, int P, int E, const int32_t *table, uint32_t *usage) {
  if (P == 0) return;
  KLAUNCH(L, k_ep_slots, (P + 255) / 256, 256, 0, ids, P, E, table, usage);
}

// the two derived forms of the 8 group sums of a Q8x block that the tensor-core kernels read
// (k_quant_q8x writes them when it quantises; received rows carry the sums only)
__global__ void k_q8x_aux(size_t n_blocks, const int32_t *__restrict__ bsum, uint16_t *bm, int32_t *xs) {
  size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_blocks) return;
  int tot = 0;
  for (int j = 0; j < 8; j++) {
    const int s = bsum[b * 8 + j];
    tot += s;
    bm[b * 16 + j] = __half_as_ushort(__int2half_rn((s >> 6) * 64));
    bm[b * 16 + 8 + j] = __half_as_ushort(__int2half_rn(s & 63));
  }
  xs[b] = tot;
}
void launch_q8x_aux(const Launch &L, size_t n_blocks, const int32_t *bsum, uint16_t *bm, int32_t *xs) {
  if (n_blocks == 0) return;
  KLAUNCH(L, k_q8x_aux, (unsigned)((n_blocks + 255) / 256), 256, 0, n_blocks, bsum, bm, xs);
}
