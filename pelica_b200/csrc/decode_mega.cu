// decode_mega.cu - one-token decode of a whole MoE layer stack in ONE persistent
// cooperative kernel (one CTA per SM).
//
// Why: at batch 1 a Qwen3-30B-A3B-shaped layer reads 24.5 MB of expert blocks,
// 3.8 us at HBM speed; a kernel launch per phase costs more than that. Here
// every CTA walks all layers; per layer it
//   1. collects the residual stream x (published by all CTAs, epoch-tagged),
//   2. norms it and quantises it to Q8x (`Q8x::new`, src/ds4_cpu.rs:13-35),
//   3. computes "its" router logit in `dot_f32` order (src/quant.rs:215-236) and
//      publishes it; collects all logits; picks the top-k (route.cuh),
//   4. issues bulk async copies (cp.async.bulk + mbarrier) of ITS slice of the
//      chosen experts' gate/up rows and down rows into shared memory: the whole
//      layer's 24.5 MB is spread over the SMs' shared memories, so HBM streams
//      without waiting for any compute,
//   5. gate/up rows . xq -> SwiGLU -> h, published to all,
//   6. collects h, re-quantises it (src/ds4_cpu.rs:306-317),
//   7. down rows for ITS columns of all k experts, summed in k order
//      (src/moe_kernels.rs:1798-1808), x += y, published for the next layer.
// The arithmetic is the general kernels' (same bits as the CPU reference path).
//
// Cross-CTA waits are bounded: a wait that runs out sets an error word, every
// CTA then drains its own copies (bounded) and returns; the host reports
// PM_ERR_TIMEOUT. The launch is cooperative, so all CTAs are co-resident.
#include "decode_mega.cuh"
#include "route.cuh"

// every cross-CTA or copy wait gives up after this long (wall time on the device)
#define MG_WAIT_NS 2000000000ull

// ---- PTX helpers -----------------------------------------------------------
__device__ __forceinline__ uint32_t s32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(s32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// global -> this CTA's shared memory, completion counted on `bar` (no multicast)
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes,
                                         uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(s32(dst)),
      "l"(src), "r"(bytes), "r"(s32(bar))
      : "memory");
}
__device__ __forceinline__ void st_pair(unsigned long long *p, float v, uint32_t epoch) {
  unsigned long long u = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(u) : "memory");
}
__device__ __forceinline__ unsigned long long ld_pair(const unsigned long long *p) {
  unsigned long long u;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(u) : "l"(p) : "memory");
  return u;
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
  unsigned long long u;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(u) : "l"(p) : "memory");
  return u;
}
__device__ __forceinline__ void red_release_add_u64(unsigned long long *p, unsigned long long v) {
  asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ int ld_volatile_i32(const int *p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// bounded wait on an mbarrier phase (non-blocking test in a timed loop);
// false = gave up (error word set)
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *err) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = now_ns();
  for (uint32_t it = 1;; it++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255) == 0) {
      if (ld_volatile_i32(err) != 0) return false;
      if (now_ns() - t0 > MG_WAIT_NS) break;
    }
  }
  atomicCAS(err, 0, 2);
  return false;
}
// bounded wait for an epoch-tagged value; false = gave up
__device__ __forceinline__ bool wait_pair(const unsigned long long *p, uint32_t epoch, float &v,
                                          int *err) {
  unsigned long long t0 = 0;
  for (uint32_t it = 0;; it++) {
    unsigned long long u = ld_pair(p);
    if ((uint32_t)(u >> 32) == epoch) {
      v = __uint_as_float((uint32_t)u);
      return true;
    }
    if ((it & 63) == 63) {
      if (ld_volatile_i32(err) != 0) return false;
      unsigned long long t = now_ns();
      if (t0 == 0) t0 = t;
      else if (t - t0 > MG_WAIT_NS) break;
    }
  }
  atomicCAS(err, 0, 1);
  return false;
}

// ---- Q8x of 256 values held 8 per lane (value j of the lane = element 32j+lane)
// (`Q8x::new`, src/ds4_cpu.rs:13-35); writes q, d, bsum of the block
__device__ __forceinline__ void q8x_block_warp(const float v[8], int lane, int8_t *q, float *d,
                                               int32_t *bsum) {
  float a = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; j++) a = fmaxf(a, fabsf(v[j]));
  a = pm_warp_max(a);
  float id = a != 0.0f ? __fdiv_rn(127.0f, a) : 0.0f;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    int r = 0;
    if (a != 0.0f) {
      float f = roundf(__fmul_rn(v[j], id));
      r = (int)fminf(fmaxf(f, -127.0f), 127.0f);
    }
    q[32 * j + lane] = (int8_t)r;
    int s = __reduce_add_sync(PM_FULL, r);
    if (lane == 0) bsum[j] = s;
  }
  if (lane == 0) *d = a != 0.0f ? __fdiv_rn(a, 127.0f) : 0.0f;
}

// ---- rows from shared memory (same sums and order as kernels_basic.cu) -------
__device__ __forceinline__ float row_q4k_smem(const uint8_t *rowp, int nb, const int8_t *xq,
                                              const float *xd, const int32_t *xbsum, int lane) {
  float total = 0.0f;
  const int nchunks = nb * 4;
  for (int c0 = 0; c0 < nchunks; c0 += 32) {
    int ci = c0 + lane;
    bool valid = ci < nchunks;
    int b = ci >> 2, c = ci & 3;
    int pi = 0, pm = 0;
    float dd = 0.0f, dmin = 0.0f;
    if (valid) {
      const uint8_t *blk = rowp + b * 144;
      uint4 hdr = *(const uint4 *)blk;
      const uint4 *qp = (const uint4 *)(blk + 16 + 32 * c);
      uint4 q0 = qp[0], q1 = qp[1];
      const int4 *xp = (const int4 *)(xq + b * 256 + 64 * c);
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

__device__ __forceinline__ float row_q6k_smem(const uint8_t *ql, const uint8_t *qh,
                                              const uint8_t *sc, const __half *dp, int nb,
                                              const int8_t *xq, const float *xd, int lane) {
  float total = 0.0f;
  const int n = lane >> 4, qtb = (lane >> 3) & 1, l4 = lane & 7;
  const int vA = 128 * n + 32 * qtb + 4 * l4;
  for (int b = 0; b < nb; b++) {
    uint32_t qlw = ((const uint32_t *)(ql + b * 128))[lane];
    uint32_t qhw = ((const uint32_t *)(qh + b * 64))[n * 8 + l4];
    uint32_t qa = (qlw & 0x0f0f0f0fu) | (((qhw >> (2 * qtb)) & 0x03030303u) << 4);
    uint32_t qb = ((qlw >> 4) & 0x0f0f0f0fu) | (((qhw >> (2 * qtb + 4)) & 0x03030303u) << 4);
    qa = __vsub4(qa, 0x20202020u);
    qb = __vsub4(qb, 0x20202020u);
    const int *xp = (const int *)(xq + b * 256);
    int xa = xp[vA >> 2], xb = xp[(vA + 64) >> 2];
    const int8_t *scb = (const int8_t *)(sc + b * 16);
    int kA = vA >> 4;
    int isum = (int)scb[kA] * __dp4a((int)qa, xa, 0) + (int)scb[kA + 4] * __dp4a((int)qb, xb, 0);
    isum = __reduce_add_sync(PM_FULL, isum);
    float d = __half2float(dp[b]);
    total = __fadd_rn(total, __fmul_rn(xd[b], __fmul_rn(d, (float)isum)));
  }
  return total;
}

// ---- the kernel ------------------------------------------------------------
__global__ void __launch_bounds__(MG_NT, 1) k_decode_mega(const MegaParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  const pm_layer_desc &D = P.D;
  const int d = D.d, ff = D.ff, E = D.n_exp, K = D.top_k;
  const int G = gridDim.x, cta = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nbx = d / 256, nbh = ff / 256;
  const int RBG = nbx * 144;  // bytes of a gate/up row
  const bool dq6 = D.type_down == PM_TYPE_Q6_K;

  uint8_t *gs = smem + P.off_gs, *us = smem + P.off_us, *dn = smem + P.off_dn;
  __half *dsm = (__half *)(smem + P.off_dsm);
  float *xs = (float *)(smem + P.off_xs);
  int8_t *xq = (int8_t *)(smem + P.off_xq);
  float *xd = (float *)(smem + P.off_xd);
  int32_t *xbs = (int32_t *)(smem + P.off_xbs);
  int8_t *hq = (int8_t *)(smem + P.off_hq);
  float *hd = (float *)(smem + P.off_hd);
  int32_t *hbs = (int32_t *)(smem + P.off_hbs);
  float *rw = (float *)(smem + P.off_rw);
  float *eo = (float *)(smem + P.off_eo);
  float *lg = (float *)(smem + P.off_lg);
  // misc: mbarriers, reduction scratch, ids/weights, route scratch
  uint64_t *bar_gu = (uint64_t *)(smem + P.off_misc);  // [MG_GU_CHUNKS]
  uint64_t *bar_dn = bar_gu + MG_GU_CHUNKS;            // [PM_MAX_TOPK]
  uint64_t *bar_rw = bar_dn + PM_MAX_TOPK;             // [1]
  float *red8 = (float *)(bar_rw + 1);                 // [8]
  uint32_t *ids = (uint32_t *)(red8 + 8);              // [PM_MAX_TOPK]
  float *wts = (float *)(ids + PM_MAX_TOPK);           // [PM_MAX_TOPK]
  int *s_dead = (int *)(wts + PM_MAX_TOPK);            // [1]
  float *r_sv = (float *)(s_dead + 4);                 // [E] route scratch
  float *r_gs = r_sv + PM_MAX_EXPERTS;                 // [E/2]
  unsigned char *r_keep = (unsigned char *)(r_gs + PM_MAX_EXPERTS / 2);

  // this CTA's slices
  const long long HR = (long long)K * ff;  // h rows of the layer: R = k*ff + j
  const int R0 = (int)(HR * cta / G), R1 = (int)(HR * (cta + 1) / G);
  const int C0 = (int)((long long)d * cta / G), C1 = (int)((long long)d * (cta + 1) / G);
  const int ncols = C1 - C0;
  const bool has_logit = cta < E;  // E <= G (checked by the host)

  if (tid == 0) {
    for (int i = 0; i < MG_GU_CHUNKS; i++) mbar_init(&bar_gu[i], 1);
    for (int i = 0; i < K; i++) mbar_init(&bar_dn[i], 1);
    mbar_init(bar_rw, 1);
    *s_dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // router row of layer 0
  if (has_logit && tid == 0) {
    mbar_expect_tx(bar_rw, (uint32_t)d * 4);
    bulk_g2s(rw, P.layers[0].router + (size_t)cta * d, (uint32_t)d * 4, bar_rw);
  }

  bool dead = false;
  bool copies_pending = false;
  int l = 0;
  for (; l < P.n_layers; l++) {
    const MegaLayer &ML = P.layers[l];
    const uint32_t par = l & 1;
    const uint32_t ep = P.epoch_base + (uint32_t)l;  // tag of this layer's x and logits

    // ---- 1. the residual stream ----
    for (int i = tid; i < d; i += MG_NT) {
      float v = 0.0f;
      if (l == 0) v = P.x_in[i];
      else if (!wait_pair(P.xbuf + i, ep, v, P.err)) dead = true;
      xs[i] = v;
    }
    if (__syncthreads_or(dead)) { dead = true; break; }

    // ---- 2. norm, Q8x of the normed token ----
    float inv = pm_rms_inv(xs, d, P.eps, red8);
    if (warp < nbx) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; j++) v[j] = __fmul_rn(xs[warp * 256 + 32 * j + lane], inv);
      q8x_block_warp(v, lane, xq + warp * 256, xd + warp, xbs + warp * 8);
    } else if (warp == MG_WARPS - 1) {
      // ---- 3. this CTA's router logit, then all logits, then the top-k ----
      if (has_logit) {
        if (!mbar_wait(bar_rw, par, P.err)) dead = true;
        float acc = 0.0f;
        for (int c = lane; c < d; c += 32) acc = __fmaf_rn(rw[c], __fmul_rn(xs[c], inv), acc);
        float s = pm_warp_sum_dot(acc);
        if (lane == 0) {
          if (ML.logit_bias) s = __fadd_rn(s, ML.logit_bias[cta]);
          st_pair(P.lbuf + cta, s, ep);
        }
        __syncwarp();
        if (lane == 0 && l + 1 < P.n_layers) {  // next layer's row into the same buffer
          mbar_expect_tx(bar_rw, (uint32_t)d * 4);
          bulk_g2s(rw, P.layers[l + 1].router + (size_t)cta * d, (uint32_t)d * 4, bar_rw);
        }
      }
      for (int e = lane; e < E; e += 32) {
        float v = 0.0f;
        if (!wait_pair(P.lbuf + e, ep, v, P.err)) dead = true;
        lg[e] = v;
      }
      __syncwarp();
      pm_route_warp(D, lg, ML.select_bias, lane, r_sv, r_gs, r_keep, ids, wts);
      __syncwarp();  // ids[] written by lane 0
      if (cta == 0 && lane < K && ML.usage) atomicAdd(&ML.usage[ids[lane]], 1u);
    }
    if (__syncthreads_or(dead)) { dead = true; break; }

    // ---- 4. bulk copies of this CTA's slices ----
    // gate/up: chunk ch covers rows [ra, rb); a chunk spans at most two experts
    if (tid < MG_GU_CHUNKS * 4) {
      int ch = tid >> 2, seg = (tid >> 1) & 1, isup = tid & 1;
      int ra = R0 + (int)((long long)(R1 - R0) * ch / MG_GU_CHUNKS);
      int rb = R0 + (int)((long long)(R1 - R0) * (ch + 1) / MG_GU_CHUNKS);
      int ka = ra / ff;
      int split = min(rb, (ka + 1) * ff);  // rows [ra, split) expert slot ka, [split, rb) slot ka+1
      int s0 = seg == 0 ? ra : split, s1 = seg == 0 ? split : rb;
      if (seg == 0 && isup == 0) mbar_expect_tx(&bar_gu[ch], (uint32_t)(rb - ra) * 2u * (uint32_t)RBG);
      if (s1 > s0) {
        int k = s0 / ff, j0 = s0 - k * ff;
        int el = (int)ids[k];
        const uint8_t *src = (isup ? ML.up + (size_t)el * ML.up_stride : ML.gate + (size_t)el * ML.gate_stride) +
                             (size_t)j0 * RBG;
        uint8_t *dst = (isup ? us : gs) + (size_t)(s0 - R0) * RBG;
        bulk_g2s(dst, src, (uint32_t)(s1 - s0) * (uint32_t)RBG, &bar_gu[ch]);
      }
    } else if (tid >= 32 && tid < 32 + K * 4) {
      // down: expert slot k, plane p; columns [C0, C1)
      int k = (tid - 32) >> 2, p = (tid - 32) & 3;
      int el = (int)ids[k];
      const uint32_t fb6[4] = {128, 64, 16, 0}, fb4[4] = {144, 0, 0, 0};
      uint32_t fb = dq6 ? fb6[p] : fb4[p];
      uint32_t tot = dq6 ? 208u : 144u;
      if (p == 0) mbar_expect_tx(&bar_dn[k], (uint32_t)ncols * (uint32_t)nbh * tot);
      if (fb && ncols > 0) {
        uint32_t poff = dq6 ? (p == 0 ? 0u : p == 1 ? 128u : 192u) : 0u;  // plane offset per block unit
        const uint8_t *src = ML.down[p] + (size_t)el * ML.down_stride[p] + (size_t)C0 * nbh * fb;
        uint8_t *dst = dn + (size_t)k * P.dn_k_bytes + (size_t)P.cols_max * nbh * poff;
        bulk_g2s(dst, src, (uint32_t)ncols * (uint32_t)nbh * fb, &bar_dn[k]);
      }
    }
    copies_pending = true;
    if (dq6) {  // the f16 block scales (2 B each) by plain loads
      int n = K * ncols * nbh;
      for (int i = tid; i < n; i += MG_NT) {
        int k = i / (ncols * nbh), r = i - k * (ncols * nbh);
        int el = (int)ids[k];
        dsm[k * P.cols_max * nbh + r] =
            *(const __half *)(ML.down[3] + (size_t)el * ML.down_stride[3] + ((size_t)C0 * nbh + r) * 2);
      }
    }

    // ---- 5. gate/up rows -> h ----
    const bool fold = D.weight_fold == PM_FOLD_BEFORE_DOWN;
    for (int r = R0 + warp; r < R1; r += MG_WARPS) {
      int rel = r - R0;
      // chunk of this row: the largest ch with start <= r
      int ch = (int)(((long long)(rel + 1) * MG_GU_CHUNKS - 1) / (R1 - R0));
      while (ch > 0 && R0 + (int)((long long)(R1 - R0) * ch / MG_GU_CHUNKS) > r) ch--;
      while (ch + 1 < MG_GU_CHUNKS && R0 + (int)((long long)(R1 - R0) * (ch + 1) / MG_GU_CHUNKS) <= r) ch++;
      if (!__all_sync(PM_FULL, mbar_wait(&bar_gu[ch], par, P.err))) { dead = true; break; }
      int k = r / ff;
      float gv = row_q4k_smem(gs + (size_t)rel * RBG, nbx, xq, xd, xbs, lane);
      float uv = row_q4k_smem(us + (size_t)rel * RBG, nbx, xq, xd, xbs, lane);
      if (lane == 0) {
        float hv = pm_act(D.act, D.act_limit, D.act_alpha, gv, uv, wts[k], fold);
        __stcg(P.hbuf + r, hv);
      }
    }
    if (__syncthreads_or(dead)) { dead = true; break; }
    if (tid == 0) red_release_add_u64(P.hcount, 1ull);

    // ---- 6. all of h, re-quantised ----
    if (tid == 0) {
      unsigned long long want = P.hcount_base + (unsigned long long)(l + 1) * (unsigned long long)G;
      bool ok = false;
      unsigned long long t0 = now_ns();
      for (uint32_t it = 0;; it++) {
        if (ld_acquire_u64(P.hcount) >= want) { ok = true; break; }
        if ((it & 63) == 63 && (ld_volatile_i32(P.err) != 0 || now_ns() - t0 > MG_WAIT_NS)) break;
      }
      if (!ok) { atomicCAS(P.err, 0, 3); dead = true; }
    }
    if (__syncthreads_or(dead)) { dead = true; break; }
    for (int b = warp; b < K * nbh; b += MG_WARPS) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; j++) v[j] = __ldcg(P.hbuf + b * 256 + 32 * j + lane);
      q8x_block_warp(v, lane, hq + b * 256, hd + b, hbs + b * 8);
    }
    __syncthreads();

    // ---- 7. down rows of this CTA's columns, all k; sum in k order; publish ----
    for (int i = warp; i < K * ncols; i += MG_WARPS) {
      int k = i / ncols, ci = i - k * ncols;
      if (!__all_sync(PM_FULL, mbar_wait(&bar_dn[k], par, P.err))) { dead = true; break; }
      const uint8_t *base = dn + (size_t)k * P.dn_k_bytes;
      float o;
      if (dq6) {
        size_t cm = (size_t)P.cols_max * nbh;
        o = row_q6k_smem(base + (size_t)ci * nbh * 128, base + cm * 128 + (size_t)ci * nbh * 64,
                         base + cm * 192 + (size_t)ci * nbh * 16, dsm + k * P.cols_max * nbh + ci * nbh,
                         nbh, hq + k * ff, hd + k * nbh, lane);
      } else {
        o = row_q4k_smem(base + (size_t)ci * nbh * 144, nbh, hq + k * ff, hd + k * nbh, hbs + k * nbh * 8,
                         lane);
      }
      if (lane == 0) eo[k * P.cols_max + ci] = o;
    }
    copies_pending = false;  // every gate/up chunk and every down barrier was waited on
    if (__syncthreads_or(dead)) { dead = true; copies_pending = true; break; }
    if (tid < ncols) {
      float s = 0.0f;
      for (int k = 0; k < K; k++) {
        float v = eo[k * P.cols_max + tid];
        if (!fold) v = __fmul_rn(wts[k], v);
        s = __fadd_rn(s, v);
      }
      float xn = __fadd_rn(xs[C0 + tid], s);
      if (l + 1 < P.n_layers) st_pair(P.xbuf + C0 + tid, xn, ep + 1);
      else P.x_out[C0 + tid] = xn;
    }
    __syncthreads();  // eo, xs, ids are rewritten by the next layer
  }

  if (dead) {
    // give this CTA's own copies a bounded time to land before its shared memory goes away
    __syncthreads();
    if (tid == 0 && copies_pending) {
      uint32_t par = l & 1;
      for (int i = 0; i < MG_GU_CHUNKS; i++)
        for (uint32_t it = 0; it < (1u << 16) && !mbar_try_wait(&bar_gu[i], par); it++) {}
      for (int i = 0; i < K; i++)
        for (uint32_t it = 0; it < (1u << 16) && !mbar_try_wait(&bar_dn[i], par); it++) {}
    }
    if (tid == 0 && has_logit)
      for (uint32_t it = 0; it < (1u << 16) && !mbar_try_wait(bar_rw, l & 1); it++) {}
    __syncthreads();
  }
}

// ---- host side ---------------------------------------------------------------
static uint32_t up16(uint32_t v) { return (v + 127u) & ~127u; }

// Can this stack shape run in the decode kernel on this device? Fills the layout.
bool mega_plan(const pm_layer_desc &D, int n_sm, size_t smem_optin, MegaPlan &mp) {
  mp.ok = false;
  if (D.act_quant != PM_AQ_Q8X_256) return false;
  if (D.type_gate != PM_TYPE_Q4_K || D.type_up != PM_TYPE_Q4_K) return false;
  if (D.type_down != PM_TYPE_Q4_K && D.type_down != PM_TYPE_Q6_K) return false;
  if (D.shared || D.has_expert_bias || D.n_exp_local > 0) return false;
  if (D.n_exp > n_sm || D.top_k > PM_MAX_TOPK) return false;
  if (D.d / 256 > MG_WARPS - 1) return false;
  int G = n_sm;
  const int d = D.d, ff = D.ff, K = D.top_k;
  const int nbx = d / 256, nbh = ff / 256;
  long long HR = (long long)K * ff;
  int rows_max = (int)((HR + G - 1) / G) + 1, cols_max = (d + G - 1) / G + 1;
  if (HR < G || d < G) return false;
  if (cols_max > MG_NT) return false;
  MegaParams &P = mp.P;
  P.D = D;
  P.rows_max = rows_max;
  P.cols_max = cols_max;
  uint32_t off = 0;
  auto take = [&](uint32_t bytes) { uint32_t o = off; off = up16(off + bytes); return o; };
  P.off_gs = take((uint32_t)rows_max * nbx * 144);
  P.off_us = take((uint32_t)rows_max * nbx * 144);
  uint32_t per_blk = D.type_down == PM_TYPE_Q6_K ? 208u : 144u;
  P.dn_k_bytes = up16((uint32_t)cols_max * nbh * per_blk);
  P.off_dn = take(P.dn_k_bytes * K);
  P.off_dsm = take((uint32_t)K * cols_max * nbh * 2);
  P.off_xs = take((uint32_t)d * 4);
  P.off_xq = take((uint32_t)d);
  P.off_xd = take((uint32_t)nbx * 4);
  P.off_xbs = take((uint32_t)nbx * 8 * 4);
  P.off_hq = take((uint32_t)K * ff);
  P.off_hd = take((uint32_t)K * nbh * 4);
  P.off_hbs = take((uint32_t)K * nbh * 8 * 4);
  P.off_rw = take((uint32_t)d * 4);
  P.off_eo = take((uint32_t)K * cols_max * 4);
  P.off_lg = take((uint32_t)D.n_exp * 4);
  P.off_misc = take(8 * (MG_GU_CHUNKS + PM_MAX_TOPK + 1) + 8 * 4 + PM_MAX_TOPK * 8 + 16 +
                    PM_MAX_EXPERTS * 4 + PM_MAX_EXPERTS * 2 + PM_MAX_EXPERTS / 2 + 64);
  mp.smem = off;
  if (mp.smem > smem_optin) return false;
  mp.grid = G;
  mp.ok = true;
  return true;
}

cudaError_t mega_prepare(size_t smem) {
  return cudaFuncSetAttribute(k_decode_mega, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

int mega_max_ctas_per_sm(size_t smem) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k_decode_mega, MG_NT, smem) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

cudaError_t mega_launch(const MegaPlan &mp, cudaStream_t stream) {
  MegaParams P = mp.P;
  void *args[] = {(void *)&P};
  return cudaLaunchCooperativeKernel((const void *)k_decode_mega, dim3(mp.grid), dim3(MG_NT), args, mp.smem,
                                     stream);
}
