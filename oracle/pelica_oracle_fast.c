/* pelica_oracle_fast.c - the reference's SIMD CPU kernels, restated.
 *
 * TEST INFRASTRUCTURE ONLY: (a) bit-identical fast forms of the scalar rows
 * (integer sums by AVX-512 VNNI, float tail in `row_scalar`'s order) so parity
 * cases of realistic size finish in seconds; (b) the reference's own fast path
 * (`row_vnni`, `row_vnni_multi`, `q4k_rows_multi`, `expert`, `cpu_experts`:
 * src/ds4_cpu.rs:87-118,205-271,297-328; src/ds4.rs:1766-1822), threaded the
 * way the reference threads it, which is what the CPU baseline times.
 * Citations are paths inside the Pelica source tree.
 */
#include "pelica_oracle.h"

#include <immintrin.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define VNNI_TARGET __attribute__((target("avx512f,avx512bw,avx512vnni,avx512vl,avx2,fma")))

int po_have_vnni(void) {
  static int ok = -1;
  if (ok < 0) {
    __builtin_cpu_init();
    ok = __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") &&
         __builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512vl");
  }
  return ok;
}

int po_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

static inline float f16le(const uint8_t *b) {
  return po_f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
}

/* `scales` (src/ds4_cpu.rs:45-57) */
static inline void q4k_scales(const uint8_t *s, int32_t sc[8], int32_t m[8]) {
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

/* one Q4_K block's nibbles as 4 x 64 unsigned bytes (32 low then 32 high, the
 * order the activations are stored in) and its sub-scales per lane
 * (src/ds4_cpu.rs:219-227) */
VNNI_TARGET static inline void q4k_unpack(const uint8_t *qs, const int32_t sc[8], __m512i qv[4],
                                          __m512i sv[4]) {
  const __m256i mask = _mm256_set1_epi8(15);
  for (int c = 0; c < 4; c++) {
    __m256i q = _mm256_loadu_si256((const __m256i *)(qs + 32 * c));
    __m256i lo = _mm256_and_si256(q, mask);
    __m256i hi = _mm256_and_si256(_mm256_srli_epi16(q, 4), mask);
    qv[c] = _mm512_inserti64x4(_mm512_castsi256_si512(lo), hi, 1);
    sv[c] = _mm512_mask_blend_epi32(0xFF00, _mm512_set1_epi32(sc[2 * c]),
                                    _mm512_set1_epi32(sc[2 * c + 1]));
  }
}

/* ---- bit-identical fast form of row_scalar ------------------------------ */
VNNI_TARGET static float row_q4k_canon_vnni(const uint8_t *w, size_t ncols, const int8_t *q,
                                            const float *xd, const int32_t *bsum) {
  float total = 0.0f;
  size_t nb = ncols / 256;
  for (size_t b = 0; b < nb; b++) {
    const uint8_t *blk = w + b * 144;
    float d = f16le(blk), dmin = f16le(blk + 2);
    int32_t sc[8], m[8];
    q4k_scales(blk + 4, sc, m);
    __m512i qv[4], sv[4];
    q4k_unpack(blk + 16, sc, qv, sv);
    const int8_t *xq = q + b * 256;
    __m512i acc = _mm512_setzero_si512();
    for (int c = 0; c < 4; c++) {
      __m512i xv = _mm512_loadu_si512((const void *)(xq + 64 * c));
      __m512i dp = _mm512_dpbusd_epi32(_mm512_setzero_si512(), qv[c], xv);
      acc = _mm512_add_epi32(acc, _mm512_mullo_epi32(dp, sv[c]));
    }
    int32_t isum = _mm512_reduce_add_epi32(acc);
    int32_t msum = 0;
    for (int j = 0; j < 8; j++) msum += m[j] * bsum[b * 8 + j];
    total += xd[b] * (d * (float)isum - dmin * (float)msum); /* src/ds4_cpu.rs:80 */
  }
  return total;
}

float po_row_q4k_fast(const uint8_t *w, size_t ncols, const int8_t *q, const float *d,
                      const int32_t *bsum) {
  if (po_have_vnni()) return row_q4k_canon_vnni(w, ncols, q, d, bsum);
  return po_row_q4k(w, ncols, q, d, bsum);
}

/* ---- `row_vnni` (src/ds4_cpu.rs:87-118) --------------------------------- */
VNNI_TARGET static float row_q4k_vnni_impl(const uint8_t *w, size_t ncols, const int8_t *q,
                                           const float *xd, const int32_t *bsum) {
  __m512 lanes = _mm512_setzero_ps();
  float mins = 0.0f;
  size_t nb = ncols / 256;
  for (size_t b = 0; b < nb; b++) {
    const uint8_t *blk = w + b * 144;
    float d = f16le(blk), dmin = f16le(blk + 2);
    int32_t sc[8], m[8];
    q4k_scales(blk + 4, sc, m);
    __m512i qv[4], sv[4];
    q4k_unpack(blk + 16, sc, qv, sv);
    const int8_t *xq = q + b * 256;
    __m512i acc = _mm512_setzero_si512();
    for (int c = 0; c < 4; c++) {
      __m512i xv = _mm512_loadu_si512((const void *)(xq + 64 * c));
      __m512i dp = _mm512_dpbusd_epi32(_mm512_setzero_si512(), qv[c], xv);
      acc = _mm512_add_epi32(acc, _mm512_mullo_epi32(dp, sv[c]));
    }
    lanes = _mm512_fmadd_ps(_mm512_cvtepi32_ps(acc), _mm512_set1_ps(xd[b] * d), lanes);
    int32_t msum = 0;
    for (int j = 0; j < 8; j++) msum += m[j] * bsum[b * 8 + j];
    mins += xd[b] * dmin * (float)msum;
  }
  return _mm512_reduce_add_ps(lanes) - mins;
}

float po_row_q4k_vnni(const uint8_t *w, size_t ncols, const int8_t *q, const float *d,
                      const int32_t *bsum) {
  if (!po_have_vnni()) return NAN;
  return row_q4k_vnni_impl(w, ncols, q, d, bsum);
}

/* ---- `row_vnni_multi` (src/ds4_cpu.rs:205-244) --------------------------- */
#define MULTI 16
VNNI_TARGET static void row_q4k_multi(const uint8_t *w, size_t ncols, int nt,
                                      const int8_t *const *q, const float *const *xd,
                                      const int32_t *const *bsum, float *out, int canonical) {
  __m512 lanes[MULTI];
  float mins[MULTI], total[MULTI];
  for (int t = 0; t < MULTI; t++) {
    lanes[t] = _mm512_setzero_ps();
    mins[t] = 0.0f;
    total[t] = 0.0f;
  }
  size_t nb = ncols / 256;
  for (size_t b = 0; b < nb; b++) {
    const uint8_t *blk = w + b * 144;
    float d = f16le(blk), dmin = f16le(blk + 2);
    int32_t sc[8], m[8];
    q4k_scales(blk + 4, sc, m);
    __m512i qv[4], sv[4];
    q4k_unpack(blk + 16, sc, qv, sv);
    for (int t = 0; t < nt; t++) {
      const int8_t *xq = q[t] + b * 256;
      __m512i acc = _mm512_setzero_si512();
      for (int c = 0; c < 4; c++) {
        __m512i xv = _mm512_loadu_si512((const void *)(xq + 64 * c));
        __m512i dp = _mm512_dpbusd_epi32(_mm512_setzero_si512(), qv[c], xv);
        acc = _mm512_add_epi32(acc, _mm512_mullo_epi32(dp, sv[c]));
      }
      int32_t msum = 0;
      for (int j = 0; j < 8; j++) msum += m[j] * bsum[t][b * 8 + j];
      if (canonical) {
        int32_t isum = _mm512_reduce_add_epi32(acc);
        total[t] += xd[t][b] * (d * (float)isum - dmin * (float)msum);
      } else {
        lanes[t] = _mm512_fmadd_ps(_mm512_cvtepi32_ps(acc), _mm512_set1_ps(xd[t][b] * d),
                                   lanes[t]);
        mins[t] += xd[t][b] * dmin * (float)msum;
      }
    }
  }
  for (int t = 0; t < nt; t++)
    out[t] = canonical ? total[t] : _mm512_reduce_add_ps(lanes[t]) - mins[t];
}

/* Q6_K block as 4 x 64 unsigned 6-bit codes in value order, and the i8
 * sub-scales per lane (scale k covers values 16k..16k+15 = 4 lanes) */
VNNI_TARGET static inline void q6k_unpack(const uint8_t *blk, __m512i qv[4], __m512i sv[4]) {
  const __m256i m4 = _mm256_set1_epi8(15), m2 = _mm256_set1_epi8(3);
  for (int n = 0; n < 2; n++) {
    __m256i ql0 = _mm256_loadu_si256((const __m256i *)(blk + 64 * n));
    __m256i ql1 = _mm256_loadu_si256((const __m256i *)(blk + 64 * n + 32));
    __m256i qh = _mm256_loadu_si256((const __m256i *)(blk + 128 + 32 * n));
    __m256i v0 = _mm256_or_si256(_mm256_and_si256(ql0, m4),
                                 _mm256_slli_epi16(_mm256_and_si256(qh, m2), 4));
    __m256i v1 = _mm256_or_si256(
        _mm256_and_si256(ql1, m4),
        _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 2), m2), 4));
    __m256i v2 = _mm256_or_si256(
        _mm256_and_si256(_mm256_srli_epi16(ql0, 4), m4),
        _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 4), m2), 4));
    __m256i v3 = _mm256_or_si256(
        _mm256_and_si256(_mm256_srli_epi16(ql1, 4), m4),
        _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 6), m2), 4));
    qv[2 * n] = _mm512_inserti64x4(_mm512_castsi256_si512(v0), v1, 1);
    qv[2 * n + 1] = _mm512_inserti64x4(_mm512_castsi256_si512(v2), v3, 1);
  }
  const int8_t *sc = (const int8_t *)(blk + 192);
  for (int z = 0; z < 4; z++) {
    int32_t s[16];
    for (int i = 0; i < 16; i++) s[i] = sc[4 * z + i / 4];
    sv[z] = _mm512_loadu_si512((const void *)s);
  }
}

VNNI_TARGET static void row_q6k_multi(const uint8_t *w, size_t ncols, int nt,
                                      const int8_t *const *q, const float *const *xd,
                                      float *out, int canonical) {
  __m512 lanes[MULTI];
  float total[MULTI];
  for (int t = 0; t < MULTI; t++) {
    lanes[t] = _mm512_setzero_ps();
    total[t] = 0.0f;
  }
  const __m512i ones = _mm512_set1_epi8(1);
  size_t nb = ncols / 256;
  for (size_t b = 0; b < nb; b++) {
    const uint8_t *blk = w + b * 210;
    float d = f16le(blk + 208);
    __m512i qv[4], sv[4];
    q6k_unpack(blk, qv, sv);
    for (int t = 0; t < nt; t++) {
      const int8_t *xq = q[t] + b * 256;
      __m512i acc = _mm512_setzero_si512();
      for (int z = 0; z < 4; z++) {
        __m512i xv = _mm512_loadu_si512((const void *)(xq + 64 * z));
        __m512i dp = _mm512_dpbusd_epi32(_mm512_setzero_si512(), qv[z], xv);
        __m512i dx = _mm512_dpbusd_epi32(_mm512_setzero_si512(), ones, xv);
        dp = _mm512_sub_epi32(dp, _mm512_slli_epi32(dx, 5)); /* sum (q-32)*x */
        acc = _mm512_add_epi32(acc, _mm512_mullo_epi32(dp, sv[z]));
      }
      if (canonical) {
        int32_t isum = _mm512_reduce_add_epi32(acc);
        total[t] += xd[t][b] * (d * (float)isum);
      } else {
        lanes[t] = _mm512_fmadd_ps(_mm512_cvtepi32_ps(acc), _mm512_set1_ps(xd[t][b] * d),
                                   lanes[t]);
      }
    }
  }
  for (int t = 0; t < nt; t++) out[t] = canonical ? total[t] : _mm512_reduce_add_ps(lanes[t]);
}

/* `q4k_rows_multi` (src/ds4_cpu.rs:248-271): out[r*nt + t] */
void po_q4k_rows_multi(const uint8_t *w, size_t nrows, size_t ncols, int nt,
                       const int8_t *const *q, const float *const *d,
                       const int32_t *const *bsum, float *out, int canonical) {
  if (nt == 0) return;
  size_t bpr = ncols / 256 * 144;
  int fast = po_have_vnni();
  for (size_t r = 0; r < nrows; r++) {
    const uint8_t *row = w + r * bpr;
    float *o = out + r * (size_t)nt;
    for (int g = 0; g < nt; g += MULTI) {
      int n = nt - g < MULTI ? nt - g : MULTI;
      if (fast) {
        row_q4k_multi(row, ncols, n, q + g, d + g, bsum + g, o + g, canonical);
      } else {
        for (int t = 0; t < n; t++) o[g + t] = po_row_q4k(row, ncols, q[g + t], d[g + t], bsum[g + t]);
      }
    }
  }
}

static void q6k_rows_multi(const uint8_t *w, size_t nrows, size_t ncols, int nt,
                           const int8_t *const *q, const float *const *d, float *out,
                           int canonical) {
  if (nt == 0) return;
  size_t bpr = ncols / 256 * 210;
  int fast = po_have_vnni();
  for (size_t r = 0; r < nrows; r++) {
    const uint8_t *row = w + r * bpr;
    float *o = out + r * (size_t)nt;
    for (int g = 0; g < nt; g += MULTI) {
      int n = nt - g < MULTI ? nt - g : MULTI;
      if (fast) {
        row_q6k_multi(row, ncols, n, q + g, d + g, o + g, canonical);
      } else {
        for (int t = 0; t < n; t++) o[g + t] = po_row_q6k(row, ncols, q[g + t], d[g + t]);
      }
    }
  }
}

float po_row_q6k_fast(const uint8_t *w, size_t ncols, const int8_t *q, const float *d) {
  if (!po_have_vnni()) return po_row_q6k(w, ncols, q, d);
  float o;
  row_q6k_multi(w, ncols, 1, &q, &d, &o, 1);
  return o;
}

static void rows_multi(int type, const uint8_t *w, size_t nrows, size_t ncols, int nt,
                       const int8_t *const *q, const float *const *d,
                       const int32_t *const *bsum, float *out) {
  if (type == PM_TYPE_Q4_K)
    po_q4k_rows_multi(w, nrows, ncols, nt, q, d, bsum, out, 0);
  else
    q6k_rows_multi(w, nrows, ncols, nt, q, d, out, 0);
}

/* ---- the threaded layer, as the reference runs it ------------------------ */
typedef struct {
  const po_expert_w *w;
  int ff;
  int nt;          /* tokens of this expert */
  const int8_t **q; /* per token */
  const float **d;
  const int32_t **bsum;
  const float *wts; /* routing weights per token (or NULL = 1) */
  float *gu;       /* [2ff][nt] */
  int8_t *hq;      /* [nt][ff] */
  float *hd;       /* [nt][ff/256] */
  int32_t *hb;     /* [nt][ff/32] */
  const int8_t **hqp;
  const float **hdp;
  const int32_t **hbp;
  float *o;        /* [d][nt] */
} job_t;

int po_moe_forward_fast(const po_layer *L, const float *x, int T, float *y, int threads) {
  const pm_layer_desc *D = &L->desc;
  int E = D->n_exp, K = D->top_k, d = D->d;
  if (D->act_quant != PM_AQ_Q8X_256 || D->type_gate != PM_TYPE_Q4_K ||
      D->type_up != PM_TYPE_Q4_K ||
      (D->type_down != PM_TYPE_Q4_K && D->type_down != PM_TYPE_Q6_K) || D->has_expert_bias)
    return PM_ERR_UNSUPPORTED;
  if (T == 0) return 0;
  if (threads < 1) threads = 1;
  /* route (src/ds4.rs:1449: tokens across threads) */
  float *logits = (float *)malloc((size_t)T * E * 4);
  uint32_t *ids = (uint32_t *)malloc((size_t)T * K * 4);
  float *w = (float *)malloc((size_t)T * K * 4);
  po_router_logits(L->router, L->logit_bias, x, T, E, d, logits);
  int rc = po_route(D, logits, L->select_bias, T, ids, w);
  if (rc) return rc;
  uint32_t *pb = (uint32_t *)malloc(((size_t)3 * E + (size_t)2 * T * K) * 4);
  uint32_t *active = pb, *offset = pb + E, *count = pb + 2 * E;
  uint32_t *ptok = pb + 3 * E, *ppos = ptok + (size_t)T * K;
  int na = po_plan(ids, T, K, E, active, offset, count, ptok, ppos);
  float *pw = (float *)malloc((size_t)T * K * 4);
  for (int i = 0; i < T * K; i++) pw[ppos[i]] = w[i];
  /* every token quantised once (src/ds4.rs:1770-1774) */
  int8_t *xq = (int8_t *)malloc((size_t)T * d);
  float *xd = (float *)malloc((size_t)T * (d / 256) * 4);
  int32_t *xb = (int32_t *)malloc((size_t)T * (d / 32) * 4);
#pragma omp parallel for schedule(static) num_threads(threads)
  for (int t = 0; t < T; t++)
    po_q8x(x + (size_t)t * d, (size_t)d, xq + (size_t)t * d, xd + (size_t)t * (d / 256),
           xb + (size_t)t * (d / 32));
  /* jobs: the active experts (+ the shared expert over every token) */
  int nj = na + (D->shared != PM_SHARED_NONE ? 1 : 0);
  job_t *J = (job_t *)calloc((size_t)nj, sizeof(job_t));
  for (int a = 0; a < nj; a++) {
    job_t *j = &J[a];
    int shared = a >= na;
    j->w = shared ? &L->shared : &L->experts[active[a]];
    j->ff = shared ? D->shared_ff : D->ff;
    j->nt = shared ? T : (int)count[a];
    j->wts = shared ? NULL : pw + offset[a];
    int nt = j->nt;
    j->q = (const int8_t **)malloc(nt * sizeof(void *));
    j->d = (const float **)malloc(nt * sizeof(void *));
    j->bsum = (const int32_t **)malloc(nt * sizeof(void *));
    for (int i = 0; i < nt; i++) {
      int t = shared ? i : (int)ptok[offset[a] + i];
      j->q[i] = xq + (size_t)t * d;
      j->d[i] = xd + (size_t)t * (d / 256);
      j->bsum[i] = xb + (size_t)t * (d / 32);
    }
    j->gu = (float *)malloc((size_t)2 * j->ff * nt * 4);
    j->hq = (int8_t *)malloc((size_t)nt * j->ff);
    j->hd = (float *)malloc((size_t)nt * (j->ff / 256) * 4);
    j->hb = (int32_t *)malloc((size_t)nt * (j->ff / 32) * 4);
    j->hqp = (const int8_t **)malloc(nt * sizeof(void *));
    j->hdp = (const float **)malloc(nt * sizeof(void *));
    j->hbp = (const int32_t **)malloc(nt * sizeof(void *));
    for (int i = 0; i < nt; i++) {
      j->hqp[i] = j->hq + (size_t)i * j->ff;
      j->hdp[i] = j->hd + (size_t)i * (j->ff / 256);
      j->hbp[i] = j->hb + (size_t)i * (j->ff / 32);
    }
    j->o = (float *)malloc((size_t)d * nt * 4);
  }
  /* gate rows then up rows in 64-row chunks across threads, experts side by
   * side (src/ds4_cpu.rs:301-305, src/ds4.rs:1776-1813) */
  size_t bpr_g = (size_t)d / 256 * 144;
  int *cbase = (int *)malloc(((size_t)nj + 1) * sizeof(int));
  cbase[0] = 0;
  for (int a = 0; a < nj; a++) cbase[a + 1] = cbase[a] + 2 * J[a].ff / 64;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
  for (int c = 0; c < cbase[nj]; c++) {
    int a = 0;
    while (c >= cbase[a + 1]) a++;
    job_t *j = &J[a];
    int ci = c - cbase[a], gch = j->ff / 64;
    const uint8_t *src = ci < gch ? j->w->gate + (size_t)ci * 64 * bpr_g
                                  : j->w->up + (size_t)(ci - gch) * 64 * bpr_g;
    po_q4k_rows_multi(src, 64, (size_t)d, j->nt, j->q, j->d, j->bsum,
                      j->gu + (size_t)ci * 64 * j->nt, 0);
  }
  /* h = silu(min(g,lim)) * clamp(u) * w, re-quantised (src/ds4_cpu.rs:306-317) */
  int *tbase = (int *)malloc(((size_t)nj + 1) * sizeof(int));
  tbase[0] = 0;
  for (int a = 0; a < nj; a++) tbase[a + 1] = tbase[a] + J[a].nt;
  int fold = D->weight_fold == PM_FOLD_BEFORE_DOWN;
#pragma omp parallel for schedule(dynamic, 4) num_threads(threads)
  for (int i = 0; i < tbase[nj]; i++) {
    int a = 0;
    while (i >= tbase[a + 1]) a++;
    job_t *j = &J[a];
    int t = i - tbase[a], nt = j->nt, ff = j->ff;
    float *h = (float *)malloc((size_t)ff * 4);
    float lim = (D->act == PM_ACT_SILU_CLAMP) ? D->act_limit : 0.0f;
    float wt = (fold && j->wts) ? j->wts[t] : 1.0f;
    for (int r = 0; r < ff; r++) {
      float gv = j->gu[(size_t)r * nt + t], uv = j->gu[(size_t)(ff + r) * nt + t];
      if (lim > 0.0f) {
        gv = fminf(gv, lim);
        uv = fminf(fmaxf(uv, -lim), lim);
      }
      float hv = gv / (1.0f + po_exp(-gv)) * uv;
      h[r] = (fold && j->wts) ? hv * wt : hv;
    }
    po_q8x(h, (size_t)ff, j->hq + (size_t)t * ff, j->hd + (size_t)t * (ff / 256),
           j->hb + (size_t)t * (ff / 32));
    free(h);
  }
  /* down rows in 64-row chunks (src/ds4_cpu.rs:319-320) */
  int dch = d / 64;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
  for (int c = 0; c < nj * dch; c++) {
    int a = c / dch, ci = c % dch;
    job_t *j = &J[a];
    size_t bpr_d = (size_t)j->ff / 256 * po_type_block_bytes(D->type_down);
    rows_multi(D->type_down, j->w->down + (size_t)ci * 64 * bpr_d, 64, (size_t)j->ff, j->nt,
               j->hqp, j->hdp, j->hbp, j->o + (size_t)ci * 64 * j->nt);
  }
  /* outputs added per token in k order, then the shared expert */
  int *pa = (int *)malloc((size_t)T * K * sizeof(int)); /* pair -> active index */
  for (int a = 0; a < na; a++)
    for (uint32_t i = 0; i < count[a]; i++) pa[offset[a] + i] = a;
#pragma omp parallel for schedule(static) num_threads(threads)
  for (int t = 0; t < T; t++) {
    for (int c = 0; c < d; c++) {
      float s = 0.0f;
      for (int k = 0; k < K; k++) {
        uint32_t p = ppos[t * K + k];
        int a = pa[p];
        float eo = J[a].o[(size_t)c * J[a].nt + (p - offset[a])];
        s += fold ? eo : w[t * K + k] * eo;
      }
      if (nj > na) s += J[na].o[(size_t)c * T + t];
      y[(size_t)t * d + c] = s;
    }
  }
  free(pa);
  for (int a = 0; a < nj; a++) {
    job_t *j = &J[a];
    free((void *)j->q); free((void *)j->d); free((void *)j->bsum);
    free(j->gu); free(j->hq); free(j->hd); free(j->hb);
    free((void *)j->hqp); free((void *)j->hdp); free((void *)j->hbp);
    free(j->o);
  }
  free(J); free(cbase); free(tbase);
  free(logits); free(ids); free(w); free(pb); free(pw);
  free(xq); free(xd); free(xb);
  return 0;
}
