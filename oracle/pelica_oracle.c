/* pelica_oracle.c - CPU restatement of Pelica's mixture-of-experts arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY (the checker and the timed CPU baseline); see
 * pelica_oracle.h for what pins it and what is "parity unpinned".
 * Compile with -ffp-contract=off: only the fmaf() calls written below fuse.
 * Citations are paths inside the Pelica source tree.
 */
#include "pelica_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

static inline float bits_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint32_t f32_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

/* ------------------------------------------------------------------------ */
/* scalars                                                                   */
/* ------------------------------------------------------------------------ */

/* src/ds4.rs:168-180 */
float po_f16_to_f32(uint16_t h) {
  uint32_t s = ((uint32_t)(h >> 15)) << 31;
  uint32_t e = (h >> 10) & 31;
  uint32_t m = h & 1023;
  if (e == 0) {
    float v = (float)m * (1.0f / (float)(1u << 24));
    return s ? -v : v;
  }
  if (e == 31) return bits_f32(s | 0x7f800000u | (m << 13));
  return bits_f32(s | ((e + 112) << 23) | (m << 13));
}

/* src/q4x.rs:102-134 */
uint16_t po_f32_to_f16(float x) {
  uint32_t b = f32_bits(x);
  uint16_t sign = (uint16_t)((b >> 16) & 0x8000);
  int32_t e = (int32_t)((b >> 23) & 0xff);
  uint32_t m = b & 0x7fffff;
  if (e == 255) return (uint16_t)(sign | 0x7c00 | (m ? 0x200 : 0));
  int32_t e2 = e - 112;
  if (e2 >= 31) return (uint16_t)(sign | 0x7c00);
  if (e2 <= 0) {
    if (e2 < -10) return sign;
    uint32_t mf = m | 0x800000;
    uint32_t shift = (uint32_t)(14 - e2);
    uint32_t half = 1u << (shift - 1);
    uint32_t r = mf >> shift;
    uint32_t rem = mf & ((1u << shift) - 1);
    if (rem > half || (rem == half && (r & 1))) r += 1;
    return (uint16_t)(sign | r);
  }
  uint32_t r = ((uint32_t)e2 << 10) | (m >> 13);
  uint32_t rem = m & 0x1fff;
  if (rem > 0x1000 || (rem == 0x1000 && (r & 1))) r += 1;
  return (uint16_t)(sign | r);
}

float po_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

uint16_t po_f32_to_bf16(float x) {
  uint32_t b = f32_bits(x);
  if ((b & 0x7f800000u) == 0x7f800000u) return (uint16_t)(b >> 16);
  b += 0x7fffu + ((b >> 16) & 1);
  return (uint16_t)(b >> 16);
}

/* `pexp` constants: src/moe_kernels.rs:439-444 */
#define PO_EXP_LOG2E 1.44269504f
#define PO_EXP_C1 0.693359375f
#define PO_EXP_C2 (-2.12194440e-4f)
static const float PO_EXP_P[6] = {1.98756915e-4f, 1.39819995e-3f, 8.3334519e-3f,
                                  4.1665796e-2f,  0.16666665f,    0.50000001f};

/* src/cpu_attn.rs:30-44, range widened (see header) */
float po_exp(float x) {
  if (x < -87.0f) return 0.0f;
  if (x > 88.0f) return INFINITY;
  float n = floorf(fmaf(x, PO_EXP_LOG2E, 0.5f));
  float r = fmaf(n, -PO_EXP_C1, x);
  r = fmaf(n, -PO_EXP_C2, r);
  float p = PO_EXP_P[0];
  for (int i = 1; i < 6; i++) p = fmaf(p, r, PO_EXP_P[i]);
  float y = fmaf(p, r * r, r);
  y = y + 1.0f;
  return y * bits_f32((uint32_t)((int32_t)n + 127) << 23);
}

/* ln(1+x), x >= 0: u = 1+x, ln(u) by the Cephes logf polynomial written with
 * explicit fmas, plus the (u-1-x)/u correction. The reference calls the
 * platform's ln_1p (src/ds4.rs:1378), which no other device reproduces bit for
 * bit; this fixed spelling is what both sides of this repository use. */
float po_log1p(float x) {
  float u = 1.0f + x;
  float c = (x - (u - 1.0f)) / u; /* correction for the rounding of 1+x */
  uint32_t ub = f32_bits(u);
  int32_t e = (int32_t)((ub >> 23) & 0xff) - 126; /* u = m * 2^e, m in [0.5,1) */
  float m = bits_f32((ub & 0x007fffffu) | 0x3f000000u);
  if (m < 0.707106781186547524f) {
    e -= 1;
    m = m + m - 1.0f;
  } else {
    m = m - 1.0f;
  }
  float z = m * m;
  float p = 7.0376836292e-2f;
  p = fmaf(p, m, -1.1514610310e-1f);
  p = fmaf(p, m, 1.1676998740e-1f);
  p = fmaf(p, m, -1.2420140846e-1f);
  p = fmaf(p, m, 1.4249322787e-1f);
  p = fmaf(p, m, -1.6668057665e-1f);
  p = fmaf(p, m, 2.0000714765e-1f);
  p = fmaf(p, m, -2.4999993993e-1f);
  p = fmaf(p, m, 3.3333331174e-1f);
  float y = m * z * p;
  float fe = (float)e;
  y = fmaf(fe, -2.12194440e-4f, y);
  y = fmaf(-0.5f, z, y);
  float r = m + y;
  r = fmaf(fe, 0.693359375f, r);
  return r + c;
}

/* src/quant.rs:215-236: accumulators k=0..3 of 8 lanes; column i+8k+j goes to
 * lane (k,j); then (acc0+acc1)+(acc2+acc3), hsum = (lo+hi), (+movehl), (+lane1) */
static float hsum32(float lane[32]) {
  float v[8], s[4];
  for (int j = 0; j < 8; j++) v[j] = (lane[j] + lane[8 + j]) + (lane[16 + j] + lane[24 + j]);
  for (int j = 0; j < 4; j++) s[j] = v[j] + v[j + 4];
  s[0] = s[0] + s[2];
  s[1] = s[1] + s[3];
  return s[0] + s[1];
}

float po_dot_f32(const float *a, const float *b, size_t n) {
  float lane[32];
  for (int j = 0; j < 32; j++) lane[j] = 0.0f;
  size_t i = 0;
  for (; i + 32 <= n; i += 32)
    for (int j = 0; j < 32; j++) lane[j] = fmaf(a[i + j], b[i + j], lane[j]);
  for (; i + 8 <= n; i += 8)
    for (int j = 0; j < 8; j++) lane[j] = fmaf(a[i + j], b[i + j], lane[j]);
  float s = hsum32(lane);
  for (; i < n; i++) s += a[i] * b[i];
  return s;
}

/* src/quant.rs:282-304 */
float po_dot_bf16(const uint16_t *a, const float *b, size_t n) {
  float lane[32];
  for (int j = 0; j < 32; j++) lane[j] = 0.0f;
  size_t i = 0;
  for (; i + 32 <= n; i += 32)
    for (int j = 0; j < 32; j++) lane[j] = fmaf(po_bf16_to_f32(a[i + j]), b[i + j], lane[j]);
  for (; i + 8 <= n; i += 8)
    for (int j = 0; j < 8; j++) lane[j] = fmaf(po_bf16_to_f32(a[i + j]), b[i + j], lane[j]);
  float s = hsum32(lane);
  for (; i < n; i++) s += po_bf16_to_f32(a[i]) * b[i];
  return s;
}

/* ------------------------------------------------------------------------ */
/* block formats                                                             */
/* ------------------------------------------------------------------------ */

/* src/gguf.rs:85-121 */
size_t po_type_block_bytes(int t) {
  switch (t) {
    case PM_TYPE_F32: return 4;
    case PM_TYPE_F16: return 2;
    case PM_TYPE_BF16: return 2;
    case PM_TYPE_Q8_0: return 34;
    case PM_TYPE_IQ4_NL: return 18;
    case PM_TYPE_IQ4_XS: return 136;
    case PM_TYPE_Q4_K: return 144;
    case PM_TYPE_Q5_K: return 176;
    case PM_TYPE_Q6_K: return 210;
    case PM_TYPE_IQ3_S: return 110;
    case PM_TYPE_MXFP4: return 17;
    case PM_TYPE_GLM_Q4: return 36;
  }
  return 0;
}
size_t po_type_block_values(int t) {
  switch (t) {
    case PM_TYPE_F32:
    case PM_TYPE_F16:
    case PM_TYPE_BF16: return 1;
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

/* the IQ4_NL codebook: a constant of the format (src/iq_tables.rs:72) */
static const int8_t KV_IQ4NL[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

/* the IQ3_S codebook, a constant of the format (src/iq_tables.rs:4), three bits a magnitude */
static const uint16_t IQ3S_CODES[512] = {
#include "../include/pelica_iq3s_grid.inc"
};

static inline float f16le(const uint8_t *b) {
  return po_f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
}

/* `scales` (src/ds4_cpu.rs:45-57); same bits as `scmin_k4` (src/moe_kernels.rs:98-107) */
static void q4k_scales(const uint8_t *s, int32_t sc[8], int32_t m[8]) {
  for (int j = 0; j < 8; j++) {
    if (j < 4) {
      sc[j] = s[j] & 63;
      m[j] = s[j + 4] & 63;
    } else {
      sc[j] = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
      m[j] = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
  }
}

/* `iq3s_sub` (src/q4x_cpu.rs:64-82): sub-block ib (32 values) of a 110-byte IQ3_S block (d @0,
 * qs @2, qh @66, signs @74, scales @106) as signed magnitudes; returns the scale 1 + 2 * sc */
static int iq3s_sub(const uint8_t *blk, int ib, int8_t out[32]) {
  const uint8_t *qs = blk + 2, *signs = blk + 74;
  uint8_t qh = blk[66 + ib];
  int sc = (blk[106 + ib / 2] >> (4 * (ib % 2))) & 15;
  for (int k = 0; k < 8; k++) {
    unsigned idx = (unsigned)qs[8 * ib + k] | (((unsigned)(qh >> k) & 1u) << 8);
    unsigned code = IQ3S_CODES[idx];
    for (int j = 0; j < 4; j++) {
      int v = 4 * k + j;
      int mag = 2 * (int)((code >> (3 * j)) & 7) + 1;
      int neg = (signs[4 * ib + v / 8] >> (v % 8)) & 1;
      out[v] = (int8_t)(neg ? -mag : mag);
    }
  }
  return 1 + 2 * sc;
}

/* `e8` (src/oss_kernels.rs:42-45) */
static inline float mx_e8(uint32_t e) {
  if (e < 2) return bits_f32(0x00200000u << e);
  return bits_f32((e - 1) << 23);
}
/* `KV_MX` (src/moe_kernels.rs:109) */
static const float KV_MX[16] = {0.0f,  1.0f,  2.0f,  3.0f,  4.0f,  6.0f,  8.0f,  12.0f,
                                0.0f, -1.0f, -2.0f, -3.0f, -4.0f, -6.0f, -8.0f, -12.0f};

/* one Q6_K value's 6-bit code and scale index (src/moe_kernels.rs:75 on raw
 * blocks: ql @0, qh @128, scales @192, d @208) */
static inline int q6k_code(const uint8_t *blk, int v, int *k) {
  int n = v / 128, r = v % 128, qt = r / 32, l = r % 32;
  uint8_t qlb = blk[64 * n + l + 32 * (qt & 1)];
  int lo = (qt >= 2) ? (qlb >> 4) : (qlb & 15);
  int hb = (blk[128 + 32 * n + l] >> (2 * qt)) & 3;
  *k = 8 * n + l / 16 + 2 * qt;
  return lo | (hb << 4);
}

int po_dequant(int t, const uint8_t *blocks, size_t n, float *out) {
  size_t bv = po_type_block_values(t), bb = po_type_block_bytes(t);
  if (!bv || n % bv) return PM_ERR_UNSUPPORTED;
  size_t nb = n / bv;
  switch (t) {
    case PM_TYPE_F32:
      memcpy(out, blocks, n * 4);
      return 0;
    case PM_TYPE_F16:
      for (size_t i = 0; i < n; i++) out[i] = f16le(blocks + 2 * i);
      return 0;
    case PM_TYPE_BF16:
      for (size_t i = 0; i < n; i++)
        out[i] = po_bf16_to_f32((uint16_t)(blocks[2 * i] | (blocks[2 * i + 1] << 8)));
      return 0;
    case PM_TYPE_Q8_0: /* src/moe_kernels.rs:68 */
      for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * bb;
        float d = f16le(blk);
        for (int i = 0; i < 32; i++) out[b * 32 + i] = d * (float)(int8_t)blk[2 + i];
      }
      return 0;
    case PM_TYPE_IQ4_NL: /* src/q4x_cpu.rs:453-461 */
      for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * bb;
        float d = f16le(blk);
        for (int i = 0; i < 16; i++) {
          out[b * 32 + i] = d * (float)KV_IQ4NL[blk[2 + i] & 15];
          out[b * 32 + 16 + i] = d * (float)KV_IQ4NL[blk[2 + i] >> 4];
        }
      }
      return 0;
    case PM_TYPE_IQ4_XS: /* src/q4x_cpu.rs:462-476 */
      for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * bb;
        float d = f16le(blk);
        unsigned sh = (unsigned)blk[2] | ((unsigned)blk[3] << 8);
        for (int ib = 0; ib < 8; ib++) {
          int ls = ((blk[4 + ib / 2] >> (4 * (ib % 2))) & 15) | (int)(((sh >> (2 * ib)) & 3) << 4);
          float dl = d * (float)(ls - 32);
          for (int i = 0; i < 16; i++) {
            uint8_t q = blk[8 + 16 * ib + i];
            out[b * 256 + 32 * ib + i] = dl * (float)KV_IQ4NL[q & 15];
            out[b * 256 + 32 * ib + 16 + i] = dl * (float)KV_IQ4NL[q >> 4];
          }
        }
      }
      return 0;
    case PM_TYPE_IQ3_S: /* src/q4x_cpu.rs:477-487: d * scale * magnitude, signed */
      for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * bb;
        float d = f16le(blk);
        int8_t q[32];
        for (int ib = 0; ib < 8; ib++) {
          int sc = iq3s_sub(blk, ib, q);
          for (int i = 0; i < 32; i++) out[b * 256 + 32 * ib + i] = d * (float)sc * (float)q[i];
        }
      }
      return 0;
    case PM_TYPE_Q5_K: /* src/moe_kernels.rs:74: d @0, dmin @2, scales @4, qh @16, qs @48;
                          dm.x * sm.x * (q | hb << 4) - dm.y * sm.y */
      for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * bb;
        float d = f16le(blk), dmin = f16le(blk + 2);
        int32_t sc[8], m[8];
        q4k_scales(blk + 4, sc, m);
        const uint8_t *qh = blk + 16, *qs = blk + 48;
        for (int c = 0; c < 4; c++)
          for (int i = 0; i < 32; i++) {
            uint8_t v = qs[32 * c + i];
            int lo = (v & 15) | (((qh[i] >> (2 * c)) & 1) << 4);
            int hi = (v >> 4) | (((qh[i] >> (2 * c + 1)) & 1) << 4);
            out[b * 256 + 64 * c + i] = d * (float)sc[2 * c] * (float)lo - dmin * (float)m[2 * c];
            out[b * 256 + 64 * c + 32 + i] = d * (float)sc[2 * c + 1] * (float)hi - dmin * (float)m[2 * c + 1];
          }
      }
      return 0;
    case PM_TYPE_Q4_K: /* src/moe_kernels.rs:73: dm.x * sm.x * q - dm.y * sm.y */
      for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * bb;
        float d = f16le(blk), dmin = f16le(blk + 2);
        int32_t sc[8], m[8];
        q4k_scales(blk + 4, sc, m);
        const uint8_t *qs = blk + 16;
        for (int c = 0; c < 4; c++)
          for (int i = 0; i < 32; i++) {
            uint8_t v = qs[32 * c + i];
            out[b * 256 + 64 * c + i] =
                d * (float)sc[2 * c] * (float)(v & 15) - dmin * (float)m[2 * c];
            out[b * 256 + 64 * c + 32 + i] =
                d * (float)sc[2 * c + 1] * (float)(v >> 4) - dmin * (float)m[2 * c + 1];
          }
      }
      return 0;
    case PM_TYPE_Q6_K: /* src/moe_kernels.rs:75: d * sc * (q - 32) */
      for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * bb;
        float d = f16le(blk + 208);
        for (int v = 0; v < 256; v++) {
          int k;
          int q = q6k_code(blk, v, &k);
          float sc = (float)(int8_t)blk[192 + k];
          out[b * 256 + v] = d * sc * ((float)q - 32.0f);
        }
      }
      return 0;
    case PM_TYPE_GLM_Q4: { /* src/quant.rs:9-11: nibbles (level + 8, low nibble first), then the f32
                              group scales; value = (nibble - 8) * scale (src/gpu.rs:96-99) */
      const uint8_t *sc = blocks + nb * 32;
      for (size_t g = 0; g < nb; g++) {
        float scale;
        memcpy(&scale, sc + 4 * g, 4);
        for (int j = 0; j < 32; j++) {
          uint8_t v = blocks[g * 32 + j];
          out[g * 64 + 2 * j] = (float)((int)(v & 15) - 8) * scale;
          out[g * 64 + 2 * j + 1] = (float)((int)(v >> 4) - 8) * scale;
        }
      }
      return 0;
    }
    case PM_TYPE_MXFP4: /* src/moe_kernels.rs:80 */
      for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * bb;
        float s = mx_e8(blk[0]);
        for (int j = 0; j < 16; j++) {
          out[b * 32 + j] = s * KV_MX[blk[1 + j] & 15];
          out[b * 32 + 16 + j] = s * KV_MX[blk[1 + j] >> 4];
        }
      }
      return 0;
  }
  return PM_ERR_UNSUPPORTED;
}

/* ------------------------------------------------------------------------ */
/* activation quantisers                                                     */
/* ------------------------------------------------------------------------ */

/* Rust f32::round: half away from zero */
static inline float round_away(float v) { return roundf(v); }

/* src/ds4_cpu.rs:13-35 */
void po_q8x(const float *x, size_t n, int8_t *q, float *d, int32_t *bsum) {
  size_t nb = n / 256;
  memset(q, 0, n);
  for (size_t b = 0; b < nb; b++) d[b] = 0.0f;
  for (size_t j = 0; j < nb * 8; j++) bsum[j] = 0;
  for (size_t b = 0; b < nb; b++) {
    const float *xs = x + b * 256;
    float amax = 0.0f;
    for (int i = 0; i < 256; i++) amax = fmaxf(amax, fabsf(xs[i]));
    if (amax == 0.0f) continue;
    float id = 127.0f / amax;
    d[b] = amax / 127.0f;
    for (int i = 0; i < 256; i++) {
      float r = round_away(xs[i] * id);
      if (r < -127.0f) r = -127.0f;
      if (r > 127.0f) r = 127.0f;
      q[b * 256 + i] = (int8_t)r;
      bsum[b * 8 + i / 32] += (int32_t)r;
    }
  }
}

/* src/q4x_cpu.rs:23-37 */
void po_q8_32(const float *x, size_t n, int8_t *q, float *d) {
  size_t nb = n / 32;
  memset(q, 0, n);
  for (size_t b = 0; b < nb; b++) {
    const float *xs = x + b * 32;
    d[b] = 0.0f;
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(xs[i]));
    if (amax == 0.0f) continue;
    d[b] = amax / 127.0f;
    float id = 127.0f / amax;
    for (int i = 0; i < 32; i++) {
      float r = round_away(xs[i] * id);
      if (r < -127.0f) r = -127.0f;
      if (r > 127.0f) r = 127.0f;
      q[b * 32 + i] = (int8_t)r;
    }
  }
}

/* PM_AQ_Q8_32_F16: `Q8::new` with the block scale a ggml Q8_0 block would store (f16). The int8
 * values are those of po_q8_32 (rounded against the unrounded scale). No reference code. */
void po_q8_32_f16(const float *x, size_t n, int8_t *q, float *d) {
  po_q8_32(x, n, q, d);
  for (size_t b = 0; b < n / 32; b++) d[b] = po_f16_to_f32(po_f32_to_f16(d[b]));
}

/* ------------------------------------------------------------------------ */
/* rows                                                                      */
/* ------------------------------------------------------------------------ */

/* src/ds4_cpu.rs:59-83 */
float po_row_q4k(const uint8_t *w, size_t ncols, const int8_t *q, const float *xd,
                 const int32_t *bsum) {
  float total = 0.0f;
  size_t nb = ncols / 256;
  for (size_t b = 0; b < nb; b++) {
    const uint8_t *blk = w + b * 144;
    float d = f16le(blk), dmin = f16le(blk + 2);
    int32_t sc[8], m[8];
    q4k_scales(blk + 4, sc, m);
    const uint8_t *qs = blk + 16;
    const int8_t *xq = q + b * 256;
    int32_t isum = 0, msum = 0;
    for (int c = 0; c < 4; c++) {
      int32_t lo = 0, hi = 0;
      for (int i = 0; i < 32; i++) {
        uint8_t v = qs[32 * c + i];
        lo += (int32_t)(v & 15) * (int32_t)xq[64 * c + i];
        hi += (int32_t)(v >> 4) * (int32_t)xq[64 * c + 32 + i];
      }
      isum += sc[2 * c] * lo + sc[2 * c + 1] * hi;
    }
    for (int j = 0; j < 8; j++) msum += m[j] * bsum[b * 8 + j];
    total += xd[b] * (d * (float)isum - dmin * (float)msum);
  }
  return total;
}

/* PARITY UNPINNED: see header */
float po_row_q6k(const uint8_t *w, size_t ncols, const int8_t *q, const float *xd) {
  float total = 0.0f;
  size_t nb = ncols / 256;
  for (size_t b = 0; b < nb; b++) {
    const uint8_t *blk = w + b * 210;
    float d = f16le(blk + 208);
    const int8_t *xq = q + b * 256;
    int32_t isum = 0;
    for (int g = 0; g < 16; g++) {
      int32_t s = 0;
      for (int i = 0; i < 16; i++) {
        int k;
        int code = q6k_code(blk, 16 * g + i, &k);
        s += (code - 32) * (int32_t)xq[16 * g + i];
      }
      isum += (int32_t)(int8_t)blk[192 + g] * s;
    }
    total += xd[b] * (d * (float)isum);
  }
  return total;
}

/* src/q4x_cpu.rs:85-90 */
float po_row_q8_0(const uint8_t *w, size_t ncols, const int8_t *q, const float *d32) {
  float total = 0.0f;
  size_t nb = ncols / 32;
  for (size_t b = 0; b < nb; b++) {
    const uint8_t *blk = w + b * 34;
    int32_t s = 0;
    for (int i = 0; i < 32; i++) s += (int32_t)(int8_t)blk[2 + i] * (int32_t)q[32 * b + i];
    total += f16le(blk) * d32[b] * (float)s;
  }
  return total;
}

/* src/q4x_cpu.rs:92-101 */
float po_row_iq4nl(const uint8_t *w, size_t ncols, const int8_t *q, const float *d32) {
  float total = 0.0f;
  size_t nb = ncols / 32;
  for (size_t b = 0; b < nb; b++) {
    const uint8_t *blk = w + b * 18;
    int32_t s = 0;
    for (int i = 0; i < 16; i++) {
      s += (int32_t)KV_IQ4NL[blk[2 + i] & 15] * (int32_t)q[32 * b + i];
      s += (int32_t)KV_IQ4NL[blk[2 + i] >> 4] * (int32_t)q[32 * b + 16 + i];
    }
    total += f16le(blk) * d32[b] * (float)s;
  }
  return total;
}

/* src/q4x_cpu.rs:102-117 */
float po_row_iq4xs(const uint8_t *w, size_t ncols, const int8_t *q, const float *d32) {
  float total = 0.0f;
  size_t nb = ncols / 256;
  for (size_t b = 0; b < nb; b++) {
    const uint8_t *blk = w + b * 136;
    float d = f16le(blk);
    unsigned sh = (unsigned)blk[2] | ((unsigned)blk[3] << 8);
    for (int ib = 0; ib < 8; ib++) {
      int ls = ((blk[4 + ib / 2] >> (4 * (ib % 2))) & 15) | (int)(((sh >> (2 * ib)) & 3) << 4);
      const uint8_t *qs = blk + 8 + 16 * ib;
      size_t s = 8 * b + (size_t)ib;
      int32_t acc = 0;
      for (int i = 0; i < 16; i++) {
        acc += (int32_t)KV_IQ4NL[qs[i] & 15] * (int32_t)q[32 * s + i];
        acc += (int32_t)KV_IQ4NL[qs[i] >> 4] * (int32_t)q[32 * s + 16 + i];
      }
      total += d * (float)(ls - 32) * d32[s] * (float)acc;
    }
  }
  return total;
}

/* src/q4x_cpu.rs:118-127 */
float po_row_iq3s(const uint8_t *w, size_t ncols, const int8_t *q, const float *d32) {
  float total = 0.0f;
  size_t nb = ncols / 256;
  for (size_t b = 0; b < nb; b++) {
    const uint8_t *blk = w + b * 110;
    float d = f16le(blk);
    int8_t v[32];
    for (int ib = 0; ib < 8; ib++) {
      int sc = iq3s_sub(blk, ib, v);
      size_t s = 8 * b + (size_t)ib;
      int32_t acc = 0;
      for (int i = 0; i < 32; i++) acc += (int32_t)v[i] * (int32_t)q[32 * s + i];
      total += d * (float)sc * d32[s] * (float)acc;
    }
  }
  return total;
}

/* a row of a type of the q4x path against 32-block Q8 activations (`row`, src/q4x_cpu.rs:367) */
/* Q4_K row . 32-block Q8 activations. The reference has no such pair; this is `row_scalar`
 * (src/ds4_cpu.rs:59-83) with the activation scale per 32-value sub-block instead of per
 * super-block: total += x.d[j] * ((d * sc_j) * isum_j - (dmin * m_j) * bsum_j), ascending j. */
float po_row_q4k_q8_32(const uint8_t *w, size_t ncols, const int8_t *q, const float *d32) {
  float total = 0.0f;
  size_t nb = ncols / 256;
  for (size_t b = 0; b < nb; b++) {
    const uint8_t *blk = w + b * 144;
    float d = f16le(blk), dmin = f16le(blk + 2);
    int32_t sc[8], m[8];
    q4k_scales(blk + 4, sc, m);
    const uint8_t *qs = blk + 16;
    for (int j = 0; j < 8; j++) { /* chunk j / 2: low nibbles = sub-block 2c, high = 2c + 1 */
      const uint8_t *qc = qs + 32 * (j / 2);
      const int8_t *xq = q + b * 256 + 32 * (size_t)j;
      int32_t isum = 0, bsum = 0;
      for (int i = 0; i < 32; i++) {
        int32_t nib = (j & 1) ? (qc[i] >> 4) : (qc[i] & 15);
        isum += nib * (int32_t)xq[i];
        bsum += (int32_t)xq[i];
      }
      float a = (d * (float)sc[j]) * (float)isum;
      float c = (dmin * (float)m[j]) * (float)bsum;
      total += d32[b * 8 + (size_t)j] * (a - c);
    }
  }
  return total;
}

static float row_q8_32(int t, const uint8_t *w, size_t ncols, const int8_t *q, const float *d32) {
  if (t == PM_TYPE_Q4_K) return po_row_q4k_q8_32(w, ncols, q, d32);
  if (t == PM_TYPE_IQ4_NL) return po_row_iq4nl(w, ncols, q, d32);
  if (t == PM_TYPE_IQ4_XS) return po_row_iq4xs(w, ncols, q, d32);
  if (t == PM_TYPE_IQ3_S) return po_row_iq3s(w, ncols, q, d32);
  return po_row_q8_0(w, ncols, q, d32);
}

/* `dot_q4_scalar` (src/quant.rs:464-476): per group of 64 the sum of level * x, then times the scale */
float po_row_glm_q4(const uint8_t *q, const uint8_t *scales, size_t ncols, const float *x) {
  float total = 0.0f;
  for (size_t g = 0; g < ncols / 64; g++) {
    float scale, acc = 0.0f;
    memcpy(&scale, scales + 4 * g, 4);
    for (int j = 0; j < 32; j++) {
      uint8_t b = q[g * 32 + j];
      size_t c = g * 64 + 2 * (size_t)j;
      acc += (float)((int)(b & 15) - 8) * x[c] + (float)((int)(b >> 4) - 8) * x[c + 1];
    }
    total += acc * scale;
  }
  return total;
}

static size_t row_bytes(int type, size_t ncols);

/* row r of a [rows][ncols] matrix of type t, as the layer holds it: GGUF types are rows of whole
 * blocks; the int4 container keeps all the nibble rows first and the scale rows after them */
static float mat_row_f32(int t, const uint8_t *m, size_t rows, size_t ncols, size_t r, const float *x) {
  if (t == PM_TYPE_GLM_Q4)
    return po_row_glm_q4(m + r * (ncols / 2), m + rows * (ncols / 2) + r * (ncols / 64) * 4, ncols, x);
  return po_row_f32(t, m + r * row_bytes(t, ncols), ncols, x);
}

float po_row_f32(int t, const uint8_t *w, size_t ncols, const float *x) {
  float total = 0.0f;
  if (t == PM_TYPE_GLM_Q4) return po_row_glm_q4(w, w + ncols / 2, ncols, x); /* a one-row matrix */
  if (t == PM_TYPE_MXFP4) { /* src/oss_batch.rs:774-789: scale * (dots of the block) */
    size_t nb = ncols / 32;
    for (size_t b = 0; b < nb; b++) {
      const uint8_t *blk = w + b * 17;
      float s = 0.0f;
      for (int j = 0; j < 16; j++) s += KV_MX[blk[1 + j] & 15] * x[b * 32 + j];
      for (int j = 0; j < 16; j++) s += KV_MX[blk[1 + j] >> 4] * x[b * 32 + 16 + j];
      total += mx_e8(blk[0]) * s;
    }
    return total;
  }
  size_t bv = po_type_block_values(t), bb = po_type_block_bytes(t);
  if (bv == 1) bv = 32; /* float types: walk 32 values at a time */
  float tmp[256];
  size_t step = bv;
  size_t bytes_per_step = (po_type_block_values(t) == 1) ? 32 * bb : bb;
  for (size_t c = 0; c + step <= ncols; c += step) {
    po_dequant(t, w + (c / step) * bytes_per_step, step, tmp);
    float s = 0.0f;
    for (size_t i = 0; i < step; i++) s += tmp[i] * x[c + i];
    total += s;
  }
  return total;
}

/* ------------------------------------------------------------------------ */
/* routing                                                                   */
/* ------------------------------------------------------------------------ */

void po_router_logits(const float *wr, const float *logit_bias, const float *x, int T, int E,
                      int d, float *logits) {
#pragma omp parallel for schedule(static) if (T * E > 256)
  for (int i = 0; i < T * E; i++) {
    int t = i / E, e = i % E;
    float v = po_dot_f32(wr + (size_t)e * d, x + (size_t)t * d, (size_t)d);
    if (logit_bias) v = v + logit_bias[e];
    logits[i] = v;
  }
}

/* sum of n values the way one 32-lane subgroup does it: lane L adds elements
 * L, L+32, ... in order, lanes are then summed by xor shuffles 16, 8, 4, 2, 1
 * (the order the reference spells out for its attention sums,
 * src/moe_kernels.rs:489-492; `plan` itself leaves subgroupAdd's order open) */
static float lane_sum(const float *v, int n) {
  float lane[32];
  for (int l = 0; l < 32; l++) {
    float s = 0.0f;
    for (int i = l; i < n; i += 32) s = s + v[i];
    lane[l] = s;
  }
  for (int off = 16; off >= 1; off >>= 1)
    for (int l = 0; l < off; l++) lane[l] = lane[l] + lane[l + off];
  return lane[0];
}

#define PO_NEG (-3.0e38f) /* the shaders' "minus infinity" (src/moe_kernels.rs:1026) */

/* index of the largest value, ties -> lowest index (src/moe_kernels.rs:1053-1060,
 * src/oss_kernels.rs:22-27, src/ds4.rs:1406) */
static int argmax_low(const float *v, int n) {
  int bi = -1;
  float bv = 0.0f;
  for (int i = 0; i < n; i++)
    if (bi < 0 || v[i] > bv) {
      bv = v[i];
      bi = i;
    }
  return bi;
}

int po_route(const pm_layer_desc *D, const float *logits, const float *sel_bias, int T,
             uint32_t *ids, float *w) {
  int E = D->n_exp, K = D->top_k;
  if (E < 1 || E > PM_MAX_EXPERTS || K < 1 || K > PM_MAX_TOPK || K > E) return PM_ERR_INVALID;
  if (D->n_group > 0 &&
      (E % D->n_group || D->topk_group < 1 || D->topk_group > D->n_group ||
       E / D->n_group < 2 || D->topk_group * (E / D->n_group) < K))
    return PM_ERR_INVALID;
  for (int t = 0; t < T; t++) {
    const float *lg = logits + (size_t)t * E;
    float pr[PM_MAX_EXPERTS], sv[PM_MAX_EXPERTS];
    uint32_t *tid = ids + (size_t)t * K;
    float *tw = w + (size_t)t * K;
    /* scores */
    switch (D->gating) {
      case PM_GATE_SOFTMAX_ALL: { /* src/moe_kernels.rs:1023-1042 */
        float mx = PO_NEG;
        for (int e = 0; e < E; e++) mx = fmaxf(mx, lg[e]);
        for (int e = 0; e < E; e++) pr[e] = po_exp(lg[e] - mx);
        float sum = lane_sum(pr, E);
        for (int e = 0; e < E; e++) pr[e] = pr[e] / sum;
        break;
      }
      case PM_GATE_SIGMOID: /* src/moe_kernels.rs:1034 */
        for (int e = 0; e < E; e++) pr[e] = 1.0f / (1.0f + po_exp(-lg[e]));
        break;
      case PM_GATE_SQRT_SOFTPLUS: /* src/ds4.rs:1377-1379 */
        for (int e = 0; e < E; e++) {
          float v = lg[e];
          float sp = v > 20.0f ? v : po_log1p(po_exp(v));
          pr[e] = sqrtf(sp);
        }
        break;
      case PM_GATE_SOFTMAX_SELECTED: /* src/oss_kernels.rs:17-27: rank the logits */
        for (int e = 0; e < E; e++) pr[e] = lg[e];
        break;
      default: return PM_ERR_INVALID;
    }
    /* what the selection ranks: score (+ bias) (src/moe_kernels.rs:1044-1049) */
    for (int e = 0; e < E; e++) sv[e] = sel_bias ? pr[e] + sel_bias[e] : pr[e];
    /* group-limited selection. NOT in the reference; this repository's
     * definition: a group's score is the sum of its two largest biased scores
     * (largest + second largest), the topk_group best groups stay (ties ->
     * lower group), every other expert is masked. PARITY UNPINNED. */
    if (D->n_group > 0) {
      int G = D->n_group, gs = E / G;
      float gscore[PM_MAX_EXPERTS];
      for (int g = 0; g < G; g++) {
        int i1 = argmax_low(sv + g * gs, gs);
        float v1 = sv[g * gs + i1];
        float v2 = PO_NEG;
        for (int i = 0; i < gs; i++)
          if (i != i1 && sv[g * gs + i] > v2) v2 = sv[g * gs + i];
        gscore[g] = v1 + v2;
      }
      uint8_t keep[PM_MAX_EXPERTS];
      memset(keep, 0, sizeof keep);
      for (int r = 0; r < D->topk_group; r++) {
        int g = argmax_low(gscore, G);
        keep[g] = 1;
        gscore[g] = PO_NEG;
      }
      for (int e = 0; e < E; e++)
        if (!keep[e / gs]) sv[e] = PO_NEG;
    }
    /* K rounds of (max, lowest index) (src/moe_kernels.rs:1053-1067) */
    float vals[PM_MAX_TOPK];
    float wsum = 0.0f;
    for (int k = 0; k < K; k++) {
      int e = argmax_low(sv, E);
      vals[k] = sv[e];
      tid[k] = (uint32_t)e;
      tw[k] = pr[e];
      wsum += pr[e];
      sv[e] = PO_NEG;
    }
    /* weights */
    if (D->gating == PM_GATE_SOFTMAX_SELECTED) { /* src/oss_kernels.rs:31-32 */
      float ev[PM_MAX_TOPK];
      float sum = 0.0f;
      for (int k = 0; k < K; k++) {
        ev[k] = po_exp(lg[tid[k]] - lg[tid[0]]);
        sum += ev[k];
      }
      for (int k = 0; k < K; k++) {
        float x = ev[k] / sum;
        if (D->w_scale != 0.0f) x = x * D->w_scale;
        tw[k] = x;
      }
      (void)vals;
    } else if (D->gating == PM_GATE_SQRT_SOFTPLUS) { /* src/ds4.rs:1416-1424 */
      for (int k = 0; k < K; k++) {
        float x = tw[k] / wsum;
        if (D->w_scale != 0.0f) x = x * D->w_scale;
        tw[k] = x;
      }
    } else { /* src/moe_kernels.rs:1072-1074 */
      for (int k = 0; k < K; k++) {
        float x = tw[k];
        if (D->norm_w) x = x / fmaxf(wsum, 6.103515625e-5f);
        if (D->w_scale != 0.0f) x = x * D->w_scale;
        tw[k] = x;
      }
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------ */
/* plan                                                                      */
/* ------------------------------------------------------------------------ */

/* output layout of src/moe_kernels.rs:1086-1129; pair order within an expert is
 * ascending (token, k) as the CPU engines build their rows (src/ds4.rs:1461-1472) */
int po_plan(const uint32_t *ids, int T, int K, int E, uint32_t *active, uint32_t *offset,
            uint32_t *count, uint32_t *pair_token, uint32_t *pair_pos) {
  uint32_t *cnt = (uint32_t *)calloc((size_t)E, 4), *base = (uint32_t *)calloc((size_t)E, 4);
  for (int i = 0; i < T * K; i++) cnt[ids[i]]++;
  int na = 0;
  uint32_t o = 0;
  for (int e = 0; e < E; e++) {
    if (cnt[e]) {
      active[na] = (uint32_t)e;
      offset[na] = o;
      count[na] = cnt[e];
      na++;
    }
    base[e] = o;
    o += cnt[e];
    cnt[e] = 0;
  }
  for (int e = na; e < E; e++) active[e] = offset[e] = count[e] = 0;
  for (int i = 0; i < T * K; i++) {
    uint32_t e = ids[i];
    uint32_t p = base[e] + cnt[e]++;
    pair_pos[i] = p;
    pair_token[p] = (uint32_t)(i / K);
  }
  free(cnt);
  free(base);
  return na;
}

/* ------------------------------------------------------------------------ */
/* expert / layer                                                            */
/* ------------------------------------------------------------------------ */

static size_t row_bytes(int type, size_t ncols) {
  return ncols / po_type_block_values(type) * po_type_block_bytes(type);
}

typedef struct {
  int8_t *q;
  float *d;
  int32_t *bsum;
} q8x_t;

static q8x_t q8x_new(const float *x, size_t n) {
  q8x_t r;
  r.q = (int8_t *)malloc(n);
  r.d = (float *)malloc((n / 256) * 4);
  r.bsum = (int32_t *)malloc((n / 32) * 4);
  po_q8x(x, n, r.q, r.d, r.bsum);
  return r;
}
static void q8x_free(q8x_t *r) {
  free(r->q);
  free(r->d);
  free(r->bsum);
}

static float row_q8x(int type, const uint8_t *w, size_t ncols, const q8x_t *x) {
  if (type == PM_TYPE_Q4_K) return po_row_q4k_fast(w, ncols, x->q, x->d, x->bsum);
  return po_row_q6k_fast(w, ncols, x->q, x->d);
}

/* the activation of one (gate, up) pair; `w` is the routing weight or 1 */
static inline float act_fn(const pm_layer_desc *D, float g, float u, float w, int fold) {
  if (D->act == PM_ACT_OSS_GLU) { /* src/oss_batch.rs:785 (biases added by the caller) */
    float x = fminf(g, D->act_limit);
    float y = fminf(fmaxf(u, -D->act_limit), D->act_limit);
    float h = x / (1.0f + po_exp(-D->act_alpha * x)) * (y + 1.0f);
    return fold ? h * w : h;
  }
  if (D->act == PM_ACT_SILU_CLAMP && D->act_limit > 0.0f) { /* src/ds4_cpu.rs:311 */
    g = fminf(g, D->act_limit);
    u = fminf(fmaxf(u, -D->act_limit), D->act_limit);
  }
  float h = g / (1.0f + po_exp(-g)) * u; /* src/ds4_cpu.rs:312, src/moe_kernels.rs:52 */
  return fold ? h * w : h;
}

int po_expert(const pm_layer_desc *D, const po_expert_w *W, int ff, const float *const *xs,
              const float *wts, int nt, float *out) {
  int d = D->d;
  int fold = D->weight_fold == PM_FOLD_BEFORE_DOWN;
  size_t bg = row_bytes(D->type_gate, (size_t)d), bu = row_bytes(D->type_up, (size_t)d);
  size_t bd = row_bytes(D->type_down, (size_t)ff);
  float *h = (float *)malloc((size_t)ff * 4);
  if (D->act_quant == PM_AQ_Q8X_256) {
    if (d % 256 || ff % 256) return PM_ERR_INVALID;
    if (D->type_gate != PM_TYPE_Q4_K && D->type_gate != PM_TYPE_Q6_K) return PM_ERR_UNSUPPORTED;
    for (int t = 0; t < nt; t++) {
      q8x_t xq = q8x_new(xs[t], (size_t)d); /* src/ds4.rs:1772 */
      for (int j = 0; j < ff; j++) {
        float g = row_q8x(D->type_gate, W->gate + (size_t)j * bg, (size_t)d, &xq);
        float u = row_q8x(D->type_up, W->up + (size_t)j * bu, (size_t)d, &xq);
        if (W->bias_gate) g = g + W->bias_gate[j];
        if (W->bias_up) u = u + W->bias_up[j];
        h[j] = act_fn(D, g, u, wts ? wts[t] : 1.0f, fold);
      }
      q8x_t hq = q8x_new(h, (size_t)ff); /* src/ds4_cpu.rs:315 */
      for (int r = 0; r < d; r++) {
        float o = row_q8x(D->type_down, W->down + (size_t)r * bd, (size_t)ff, &hq);
        if (W->bias_down) o = o + W->bias_down[r];
        out[(size_t)t * d + r] = o;
      }
      q8x_free(&xq);
      q8x_free(&hq);
    }
  } else if (D->act_quant == PM_AQ_Q8_32 || D->act_quant == PM_AQ_Q8_32_F16) { /* src/q4x_cpu.rs:399-440 */
    const int f16s = D->act_quant == PM_AQ_Q8_32_F16;
    void (*quant)(const float *, size_t, int8_t *, float *) = f16s ? po_q8_32_f16 : po_q8_32;
    if (d % 32 || ff % 32) { free(h); return PM_ERR_INVALID; }
    {
      const int ts[3] = {D->type_gate, D->type_up, D->type_down};
      for (int i = 0; i < 3; i++)
        if (ts[i] != PM_TYPE_Q8_0 && ts[i] != PM_TYPE_IQ4_NL && ts[i] != PM_TYPE_IQ4_XS && ts[i] != PM_TYPE_IQ3_S &&
            !(f16s && ts[i] == PM_TYPE_Q4_K)) {
          free(h);
          return PM_ERR_UNSUPPORTED;
        }
    }
    int8_t *xq = (int8_t *)malloc((size_t)d), *hq = (int8_t *)malloc((size_t)ff);
    float *xd = (float *)malloc((size_t)d / 32 * 4), *hd = (float *)malloc((size_t)ff / 32 * 4);
    for (int t = 0; t < nt; t++) {
      quant(xs[t], (size_t)d, xq, xd);
      for (int j = 0; j < ff; j++) {
        float g = row_q8_32(D->type_gate, W->gate + (size_t)j * bg, (size_t)d, xq, xd);
        float u = row_q8_32(D->type_up, W->up + (size_t)j * bu, (size_t)d, xq, xd);
        if (W->bias_gate) g = g + W->bias_gate[j];
        if (W->bias_up) u = u + W->bias_up[j];
        h[j] = act_fn(D, g, u, wts ? wts[t] : 1.0f, fold);
      }
      quant(h, (size_t)ff, hq, hd);
      for (int r = 0; r < d; r++) {
        float o = row_q8_32(D->type_down, W->down + (size_t)r * bd, (size_t)ff, hq, hd);
        if (W->bias_down) o = o + W->bias_down[r];
        out[(size_t)t * d + r] = o;
      }
    }
    free(xq); free(hq); free(xd); free(hd);
  } else if (D->act_quant == PM_AQ_F32) {
    for (int t = 0; t < nt; t++) {
      for (int j = 0; j < ff; j++) {
        float g = mat_row_f32(D->type_gate, W->gate, (size_t)ff, (size_t)d, (size_t)j, xs[t]);
        float u = mat_row_f32(D->type_up, W->up, (size_t)ff, (size_t)d, (size_t)j, xs[t]);
        if (W->bias_gate) g = g + W->bias_gate[j];
        if (W->bias_up) u = u + W->bias_up[j];
        h[j] = act_fn(D, g, u, wts ? wts[t] : 1.0f, fold);
      }
      for (int r = 0; r < d; r++) {
        float o = mat_row_f32(D->type_down, W->down, (size_t)d, (size_t)ff, (size_t)r, h);
        if (W->bias_down) o = o + W->bias_down[r]; /* src/oss_batch.rs:89 */
        out[(size_t)t * d + r] = o;
      }
    }
  } else {
    free(h);
    return PM_ERR_UNSUPPORTED;
  }
  free(h);
  return 0;
}

static int expert_is_local(const pm_layer_desc *D, int e) {
  if (D->n_exp_local <= 0) return 1;
  return e >= D->first_local_expert && e < D->first_local_expert + D->n_exp_local;
}

static int experts_from_plan(const po_layer *L, const float *x, int na, const uint32_t *active,
                             const uint32_t *offset, const uint32_t *count,
                             const uint32_t *pair_token, const uint32_t *pair_pos,
                             const uint32_t *ids, const float *w, int T, float *pair_out,
                             int threads) {
  const pm_layer_desc *D = &L->desc;
  int d = D->d, K = D->top_k;
  /* routing weight per pair */
  float *pw = (float *)malloc((size_t)T * K * 4);
  for (int i = 0; i < T * K; i++) pw[pair_pos[i]] = w[i];
  (void)ids;
  int rc = 0;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1)
  for (int a = 0; a < na; a++) {
    int e = (int)active[a];
    uint32_t n = count[a], o = offset[a];
    if (!expert_is_local(D, e)) {
      memset(pair_out + (size_t)o * d, 0, (size_t)n * d * 4);
      continue;
    }
    const float **xs = (const float **)malloc(n * sizeof(float *));
    for (uint32_t i = 0; i < n; i++) xs[i] = x + (size_t)pair_token[o + i] * d;
    int r = po_expert(D, &L->experts[e], D->ff, xs, pw + o, (int)n, pair_out + (size_t)o * d);
    if (r) rc = r;
    free(xs);
  }
  free(pw);
  return rc;
}

int po_experts(const po_layer *L, const float *x, int T, const uint32_t *ids, const float *w,
               float *pair_out) {
  const pm_layer_desc *D = &L->desc;
  int E = D->n_exp, K = D->top_k;
  uint32_t *buf = (uint32_t *)malloc(((size_t)3 * E + (size_t)2 * T * K) * 4);
  uint32_t *active = buf, *offset = buf + E, *count = buf + 2 * E;
  uint32_t *ptok = buf + 3 * E, *ppos = ptok + (size_t)T * K;
  int na = po_plan(ids, T, K, E, active, offset, count, ptok, ppos);
  int rc = experts_from_plan(L, x, na, active, offset, count, ptok, ppos, ids, w, T, pair_out, 1);
  free(buf);
  return rc;
}

/* src/moe_kernels.rs:1798-1808 */
void po_combine(const pm_layer_desc *D, const float *pair_out, const uint32_t *pair_pos,
                const float *w, const float *shared_out, const float *shared_gate_logit,
                int T, float *y, int accumulate) {
  int d = D->d, K = D->top_k;
  int in_combine = D->weight_fold == PM_FOLD_IN_COMBINE;
  for (int t = 0; t < T; t++) {
    float sg = 1.0f;
    if (shared_out && shared_gate_logit) sg = 1.0f / (1.0f + po_exp(-shared_gate_logit[t]));
    for (int c = 0; c < d; c++) {
      float s = 0.0f;
      for (int k = 0; k < K; k++) {
        float eo = pair_out[(size_t)pair_pos[t * K + k] * d + c];
        if (in_combine)
          s += w[t * K + k] * eo;
        else
          s += eo;
      }
      if (shared_out) {
        float sv = shared_out[(size_t)t * d + c];
        if (shared_gate_logit) sv *= sg;
        s += sv;
      }
      if (accumulate)
        y[(size_t)t * d + c] += s;
      else
        y[(size_t)t * d + c] = s;
    }
  }
}

int po_moe_forward(const po_layer *L, const float *x, int T, float *y, int accumulate,
                   int threads) {
  const pm_layer_desc *D = &L->desc;
  int E = D->n_exp, K = D->top_k, d = D->d;
  if (T == 0) return 0;
  float *logits = (float *)malloc((size_t)T * E * 4);
  uint32_t *ids = (uint32_t *)malloc((size_t)T * K * 4);
  float *w = (float *)malloc((size_t)T * K * 4);
  po_router_logits(L->router, L->logit_bias, x, T, E, d, logits);
  int rc = po_route(D, logits, L->select_bias, T, ids, w);
  if (rc) return rc;
  uint32_t *buf = (uint32_t *)malloc(((size_t)3 * E + (size_t)2 * T * K) * 4);
  uint32_t *active = buf, *offset = buf + E, *count = buf + 2 * E;
  uint32_t *ptok = buf + 3 * E, *ppos = ptok + (size_t)T * K;
  int na = po_plan(ids, T, K, E, active, offset, count, ptok, ppos);
  float *pair_out = (float *)malloc((size_t)T * K * d * 4);
  rc = experts_from_plan(L, x, na, active, offset, count, ptok, ppos, ids, w, T, pair_out,
                         threads);
  float *shared_out = NULL, *glog = NULL;
  if (!rc && D->shared != PM_SHARED_NONE) {
    pm_layer_desc SD = *D;
    SD.weight_fold = PM_FOLD_IN_COMBINE; /* no routing weight on the shared expert */
    shared_out = (float *)malloc((size_t)T * d * 4);
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1)
    for (int t = 0; t < T; t++) {
      const float *xs = x + (size_t)t * d;
      po_expert(&SD, &L->shared, D->shared_ff, &xs, NULL, 1, shared_out + (size_t)t * d);
    }
    if (D->shared == PM_SHARED_SIGMOID_GATED && L->shared_gate_inp) {
      glog = (float *)malloc((size_t)T * 4);
      for (int t = 0; t < T; t++)
        glog[t] = po_dot_f32(L->shared_gate_inp, x + (size_t)t * d, (size_t)d);
    }
  }
  if (!rc) po_combine(D, pair_out, ppos, w, shared_out, glog, T, y, accumulate);
  free(logits);
  free(ids);
  free(w);
  free(buf);
  free(pair_out);
  free(shared_out);
  free(glog);
  return rc;
}

/* x / rms(x) with unit weight: `rms` (src/forward.rs:63-69). The reference sums
 * the squares one after another; no parallel device reproduces that order, so
 * this glue (it is not one of the reference's hot-path functions) fixes an order
 * a 256-thread block has: lane j of 256 takes x[j], x[j+256], ... by fma, each 32
 * lanes are summed by xor shuffles 16,8,4,2,1, the 8 group sums one after another. */
void po_rmsnorm(const float *x, int d, float eps, float *out) {
  float lane[256];
  for (int j = 0; j < 256; j++) {
    float a = 0.0f;
    for (int i = j; i < d; i += 256) a = fmaf(x[i], x[i], a);
    lane[j] = a;
  }
  float total = 0.0f;
  for (int g = 0; g < 8; g++) {
    float *l = lane + 32 * g;
    for (int off = 16; off >= 1; off >>= 1)
      for (int i = 0; i < off; i++) l[i] = l[i] + l[i + off];
    total = total + l[0];
  }
  float ms = total / (float)d;
  float inv = 1.0f / sqrtf(ms + eps);
  for (int i = 0; i < d; i++) out[i] = x[i] * inv;
}

int po_stack_forward(const po_layer *layers, int n_layers, float eps, const float *x, int T,
                     float *x_out, int threads) {
  if (n_layers < 1) return PM_ERR_INVALID;
  int d = layers[0].desc.d;
  float *xn = (float *)malloc((size_t)T * d * 4);
  if (x_out != x) memcpy(x_out, x, (size_t)T * d * 4);
  for (int l = 0; l < n_layers; l++) {
    for (int t = 0; t < T; t++) po_rmsnorm(x_out + (size_t)t * d, d, eps, xn + (size_t)t * d);
    int rc = po_moe_forward(&layers[l], xn, T, x_out, 1, threads);
    if (rc) {
      free(xn);
      return rc;
    }
  }
  free(xn);
  return 0;
}
