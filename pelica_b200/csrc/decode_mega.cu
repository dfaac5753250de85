// decode_mega.cu - one-token decode of a whole MoE layer stack in ONE persistent
// cooperative kernel (one CTA per SM).
//
// Why: at batch 1 a Qwen3-30B-A3B-shaped layer reads 24.5 MB of expert blocks,
// 3.8 us at HBM speed; a kernel launch per phase costs more than that. Here
// every CTA walks all layers; per layer it
//   1. collects the residual stream x (published by all CTAs; one thread waits for the
//      layer's arrival counter, then everybody reads: a poller per CTA instead of
//      per word keeps the few L2 lines of the exchange from becoming a hot spot),
//   2. norms it and quantises it to Q8x (`Q8x::new`, src/ds4_cpu.rs:13-35),
//   3. computes "its" router logit in `dot_f32` order (src/quant.rs:215-236) and
//      publishes it as one 64-bit word (layer epoch, float bits) with a relaxed store;
//      the routing warp polls all E words until they carry the epoch; picks the top-k
//      (route.cuh),
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

// every cross-CTA or copy wait gives up after MegaParams::wait_ns (wall time on the device)

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
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
  unsigned long long u;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(u) : "l"(p) : "memory");
  return u;
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long *p) {
  unsigned long long u;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(u) : "l"(p) : "memory");
  return u;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long *p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_release_add_u64(unsigned long long *p, unsigned long long v) {
  asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ int ld_volatile_i32(const int *p);
__device__ __forceinline__ unsigned long long now_ns();
// one thread waits until an arrival counter reaches `want` (bounded); false = gave up.
// One poller per CTA: 148 loads a round trip on the counter's line, instead of every
// thread polling its own words (tens of thousands of loads on a few lines of one L2 slice).
__device__ __noinline__ bool wait_count(const unsigned long long *p, unsigned long long want, int *err, int code, unsigned long long wait_ns) {
  unsigned long long t0 = 0;
  for (uint32_t it = 0;; it++) {
    if (ld_acquire_u64(p) >= want) return true;
    if ((it & 63) == 63) {
      if (ld_volatile_i32(err) != 0) return false;
      unsigned long long t = now_ns();
      if (t0 == 0) t0 = t;
      else if (t - t0 > wait_ns) break;
    }
  }
  atomicCAS(err, 0, code);
  return false;
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
// blocking form with an explicit suspend-time hint: the warp sleeps in hardware
// (no issue slots burnt) for at most `ns` before the instruction returns
__device__ __forceinline__ bool mbar_try_wait_ns(uint64_t *bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      " selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(s32(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// bounded wait on an mbarrier phase: short hardware-suspended waits in a timed
// loop; false = gave up (error word set)
__device__ __noinline__ bool mbar_wait_slow(uint64_t *bar, uint32_t parity, int *err, unsigned long long wait_ns) {
  unsigned long long t0 = now_ns();
  for (uint32_t it = 1;; it++) {
    if (mbar_try_wait_ns(bar, parity, 4000u)) return true;
    if ((it & 15) == 0) {
      if (ld_volatile_i32(err) != 0) return false;
      if (now_ns() - t0 > wait_ns) break;
    }
  }
  atomicCAS(err, 0, 2);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *err, unsigned long long wait_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, err, wait_ns);
}
// ---- Q8x of 256 values held 8 per lane (value j of the lane = element 32j+lane)
// (`Q8x::new`, src/ds4_cpu.rs:13-35); writes q, d, bsum of the block
// `swz`: 16-byte chunk c of the block is stored at chunk c ^ swz (so that lanes
// reading the same chunk of 8 different blocks hit different banks)
// `fold8`: chunks 8-15 additionally swap their halves (c ^ 4), for the Q6_K down units, whose
// lanes read chunks {0-3, 8-11} (then {4-7, 12-15}) at once: banks 0-15 twice without it
__device__ __noinline__ void q8x_block_warp(const float v[8], int lane, int8_t *q, float *d,
                                               int32_t *bsum, int swz = 0, bool fold8 = false) {
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
    const int c = 2 * j + (lane >> 4);
    q[(((c ^ swz) ^ (fold8 ? (c & 8) >> 1 : 0)) << 4) + (lane & 15)] = (int8_t)r;
    int s = __reduce_add_sync(PM_FULL, r);
    if (lane == 0) bsum[j] = s;
  }
  if (lane == 0) *d = a != 0.0f ? __fdiv_rn(a, 127.0f) : 0.0f;
}

// ---- rows from shared memory (same sums and order as kernels_basic.cu) -------
// Several rows at once: every row's chain is independent, so the loads, the
// integer dots, the shuffles and the ordered float tails of NR rows overlap.

// Q4_K sub-block scale/min pair (2c, 2c+1) of a block header, branch-free
__device__ __forceinline__ void q4k_scmin_pair(const uint4 &hdr, int c, int &sc0, int &m0, int &sc1,
                                               int &m1) {
  // j = 2c, 2c+1.  c < 2: plain 6-bit fields of words y (scales) and z (mins);
  // c >= 2: low nibbles from word w, high 2 bits from the top of y / z bytes.
  int jj = (2 * c) & 3;  // byte index inside the word (0 or 2)
  uint32_t by0 = (hdr.y >> (8 * jj)) & 0xff, by1 = (hdr.y >> (8 * jj + 8)) & 0xff;
  uint32_t bz0 = (hdr.z >> (8 * jj)) & 0xff, bz1 = (hdr.z >> (8 * jj + 8)) & 0xff;
  uint32_t bw0 = (hdr.w >> (8 * jj)) & 0xff, bw1 = (hdr.w >> (8 * jj + 8)) & 0xff;
  bool hi = c >= 2;
  sc0 = hi ? (int)((bw0 & 15) | ((by0 >> 6) << 4)) : (int)(by0 & 63);
  m0 = hi ? (int)((bw0 >> 4) | ((bz0 >> 6) << 4)) : (int)(bz0 & 63);
  sc1 = hi ? (int)((bw1 & 15) | ((by1 >> 6) << 4)) : (int)(by1 & 63);
  m1 = hi ? (int)((bw1 >> 4) | ((bz1 >> 6) << 4)) : (int)(bz1 & 63);
}

template <int NR>
__device__ __forceinline__ void rows_q4k_smem(const uint8_t *const rowp[NR], int nb,
                                              const int8_t *const xq[NR], const float *const xd[NR],
                                              const int32_t *const xbs[NR], int lane,
                                              float total[NR]) {
#pragma unroll
  for (int r = 0; r < NR; r++) total[r] = 0.0f;
  const int nchunks = nb * 4;
  const uint32_t M = 0x0f0f0f0fu;
  for (int c0 = 0; c0 < nchunks; c0 += 32) {
    int ci = c0 + lane;
    bool valid = ci < nchunks;
    int b = valid ? (ci >> 2) : 0, c = ci & 3;
    uint4 hdr[NR], q0[NR], q1[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) {
      const uint8_t *blk = rowp[r] + b * 144;
      hdr[r] = *(const uint4 *)blk;
      const uint4 *qp = (const uint4 *)(blk + 16 + 32 * c);
      q0[r] = qp[0];
      q1[r] = qp[1];
    }
    float term[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) {
      const int4 *xp = (const int4 *)(xq[r] + b * 256 + 64 * c);
      int4 xl0 = xp[0], xl1 = xp[1], xh0 = xp[2], xh1 = xp[3];
      int lo = 0, hi = 0;
      lo = __dp4a((int)(q0[r].x & M), xl0.x, lo); hi = __dp4a((int)((q0[r].x >> 4) & M), xh0.x, hi);
      lo = __dp4a((int)(q0[r].y & M), xl0.y, lo); hi = __dp4a((int)((q0[r].y >> 4) & M), xh0.y, hi);
      lo = __dp4a((int)(q0[r].z & M), xl0.z, lo); hi = __dp4a((int)((q0[r].z >> 4) & M), xh0.z, hi);
      lo = __dp4a((int)(q0[r].w & M), xl0.w, lo); hi = __dp4a((int)((q0[r].w >> 4) & M), xh0.w, hi);
      lo = __dp4a((int)(q1[r].x & M), xl1.x, lo); hi = __dp4a((int)((q1[r].x >> 4) & M), xh1.x, hi);
      lo = __dp4a((int)(q1[r].y & M), xl1.y, lo); hi = __dp4a((int)((q1[r].y >> 4) & M), xh1.y, hi);
      lo = __dp4a((int)(q1[r].z & M), xl1.z, lo); hi = __dp4a((int)((q1[r].z >> 4) & M), xh1.z, hi);
      lo = __dp4a((int)(q1[r].w & M), xl1.w, lo); hi = __dp4a((int)((q1[r].w >> 4) & M), xh1.w, hi);
      int sc0, m0, sc1, m1;
      q4k_scmin_pair(hdr[r], c, sc0, m0, sc1, m1);
      int pi = sc0 * lo + sc1 * hi;
      int pm = m0 * xbs[r][b * 8 + 2 * c] + m1 * xbs[r][b * 8 + 2 * c + 1];
      if (!valid) { pi = 0; pm = 0; }
      pi += __shfl_xor_sync(PM_FULL, pi, 1);
      pm += __shfl_xor_sync(PM_FULL, pm, 1);
      pi += __shfl_xor_sync(PM_FULL, pi, 2);
      pm += __shfl_xor_sync(PM_FULL, pm, 2);
      float dd = pm_f16(hdr[r].x), dmin = pm_f16(hdr[r].x >> 16);
      term[r] = __fmul_rn(xd[r][b], __fsub_rn(__fmul_rn(dd, (float)pi), __fmul_rn(dmin, (float)pm)));
    }
    int nblk = min(8, nb - (c0 >> 2));
    for (int j = 0; j < nblk; j++) {
#pragma unroll
      for (int r = 0; r < NR; r++) total[r] = __fadd_rn(total[r], __shfl_sync(PM_FULL, term[r], 4 * j));
    }
  }
}

__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Four Q4_K rows of exactly 8 blocks (2048 values) against one activation
// vector, one WHOLE block per lane: lane = 8*row + block. The lane's block of
// the quantised token (64 words), its 8 partial sums and its scale stay in
// registers for the whole layer; no cross-lane reduction of the integer sums.
// All lanes of row group g return that row's sum (block terms added in order).
struct XBlk {
  int x[64];
  int bs[8];
  float d;
};
__device__ __forceinline__ float row4_q4k_blk(const uint8_t *rowp, const XBlk &X, int lane) {
  const int b = lane & 7;
  const uint8_t *blk = rowp + b * 144;
  const uint4 hdr = *(const uint4 *)blk;
  const uint4 *qp = (const uint4 *)(blk + 16);
  const uint32_t ML = 0x0f0f0f0fu, MH = 0xf0f0f0f0u;
  int lo[4], hi[4];
#pragma unroll
  for (int c = 0; c < 4; c++) {
    uint4 q0 = qp[2 * c], q1 = qp[2 * c + 1];
    int l = 0, h = 0;
    l = __dp4a((int)(q0.x & ML), X.x[16 * c + 0], l); h = dp4a_us(q0.x & MH, X.x[16 * c + 8], h);
    l = __dp4a((int)(q0.y & ML), X.x[16 * c + 1], l); h = dp4a_us(q0.y & MH, X.x[16 * c + 9], h);
    l = __dp4a((int)(q0.z & ML), X.x[16 * c + 2], l); h = dp4a_us(q0.z & MH, X.x[16 * c + 10], h);
    l = __dp4a((int)(q0.w & ML), X.x[16 * c + 3], l); h = dp4a_us(q0.w & MH, X.x[16 * c + 11], h);
    l = __dp4a((int)(q1.x & ML), X.x[16 * c + 4], l); h = dp4a_us(q1.x & MH, X.x[16 * c + 12], h);
    l = __dp4a((int)(q1.y & ML), X.x[16 * c + 5], l); h = dp4a_us(q1.y & MH, X.x[16 * c + 13], h);
    l = __dp4a((int)(q1.z & ML), X.x[16 * c + 6], l); h = dp4a_us(q1.z & MH, X.x[16 * c + 14], h);
    l = __dp4a((int)(q1.w & ML), X.x[16 * c + 7], l); h = dp4a_us(q1.w & MH, X.x[16 * c + 15], h);
    lo[c] = l;
    hi[c] = h >> 4;  // the high-nibble dot was accumulated 16-fold (exact)
  }
  // 6-bit sub-block scales and mins (`scales`, src/ds4_cpu.rs:45-57)
  int isum = 0, msum = 0;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    int sc, m;
    if (j < 4) {
      sc = (hdr.y >> (8 * j)) & 63;
      m = (hdr.z >> (8 * j)) & 63;
    } else {
      uint32_t a = (hdr.w >> (8 * (j - 4))) & 0xff;
      sc = (int)((a & 15) | ((((hdr.y >> (8 * (j - 4))) & 0xff) >> 6) << 4));
      m = (int)((a >> 4) | ((((hdr.z >> (8 * (j - 4))) & 0xff) >> 6) << 4));
    }
    isum += sc * ((j & 1) ? hi[j >> 1] : lo[j >> 1]);
    msum += m * X.bs[j];
  }
  float dd = pm_f16(hdr.x), dmin = pm_f16(hdr.x >> 16);
  float term = __fmul_rn(X.d, __fsub_rn(__fmul_rn(dd, (float)isum), __fmul_rn(dmin, (float)msum)));
  float total = 0.0f;
  const int g0 = lane & ~7;
#pragma unroll
  for (int j = 0; j < 8; j++) total = __fadd_rn(total, __shfl_sync(PM_FULL, term, g0 + j));
  return total;
}

template <int NR>
__device__ __forceinline__ void rows_q6k_smem(const uint8_t *const ql[NR], const uint8_t *const qh[NR],
                                              const uint8_t *const sc[NR], const __half *const dp[NR],
                                              int nb, const int8_t *const xq[NR],
                                              const float *const xd[NR], int lane, float total[NR]) {
  const int n = lane >> 4, qtb = (lane >> 3) & 1, l4 = lane & 7;
  const int vA = 128 * n + 32 * qtb + 4 * l4;
  const int kA = vA >> 4;
#pragma unroll
  for (int r = 0; r < NR; r++) total[r] = 0.0f;
  for (int b = 0; b < nb; b++) {
    uint32_t qlw[NR], qhw[NR];
    int xa[NR], xb[NR], sa[NR], sb[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) {
      qlw[r] = ((const uint32_t *)(ql[r] + b * 128))[lane];
      qhw[r] = ((const uint32_t *)(qh[r] + b * 64))[n * 8 + l4];
      const int *xp = (const int *)(xq[r] + b * 256);
      xa[r] = xp[vA >> 2];
      xb[r] = xp[(vA + 64) >> 2];
      const int8_t *scb = (const int8_t *)(sc[r] + b * 16);
      sa[r] = scb[kA];
      sb[r] = scb[kA + 4];
    }
    int isum[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) {
      uint32_t qa = (qlw[r] & 0x0f0f0f0fu) | (((qhw[r] >> (2 * qtb)) & 0x03030303u) << 4);
      uint32_t qb = ((qlw[r] >> 4) & 0x0f0f0f0fu) | (((qhw[r] >> (2 * qtb + 4)) & 0x03030303u) << 4);
      qa = pm_sub32x4(qa);
      qb = pm_sub32x4(qb);
      isum[r] = sa[r] * __dp4a((int)qa, xa[r], 0) + sb[r] * __dp4a((int)qb, xb[r], 0);
    }
#pragma unroll
    for (int r = 0; r < NR; r++) isum[r] = __reduce_add_sync(PM_FULL, isum[r]);
#pragma unroll
    for (int r = 0; r < NR; r++) {
      float d = __half2float(dp[r][b]);
      total[r] = __fadd_rn(total[r], __fmul_rn(xd[r][b], __fmul_rn(d, (float)isum[r])));
    }
  }
}

// ---- the kernel ------------------------------------------------------------
#define MG_GH 2  // h rows (gate+up pairs) a warp works on at once
#define MG_DR 4  // down rows a warp works on at once

// DQ6: down weights are Q6_K (else Q4_K); NB8: d == 2048 (8 blocks per gate/up row);
// NP: router slots per lane (4: up to 128 experts, 8: up to 256). Compile-time so that
// only the taken paths are in the instruction stream (the loop body must stay cache-resident).
template <bool DQ6, bool NB8, int NP>
__global__ void __launch_bounds__(MG_NT, 1) k_decode_mega(const MegaParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  const pm_layer_desc &D = P.D;
  const int d = D.d, ff = D.ff, E = D.n_exp, K = D.top_k;
  const int G = gridDim.x, cta = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nbx = d / 256, nbh = ff / 256;
  const int RBG = nbx * 144;  // bytes of a gate/up row
  constexpr bool dq6 = DQ6;

  uint8_t *gs = smem + P.off_gs, *us = smem + P.off_us, *dn = smem + P.off_dn;
  uint8_t *dsm = smem + P.off_dsm;
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
  uint64_t *bar_gu = (uint64_t *)(smem + P.off_misc);  // [MG_GU_CHUNKS]
  uint64_t *bar_dn = bar_gu + MG_GU_CHUNKS;            // [PM_MAX_TOPK]
  uint64_t *bar_rw = bar_dn + PM_MAX_TOPK;             // [1]
  float *red8 = (float *)(bar_rw + 1);                 // [8]
  uint32_t *ids = (uint32_t *)(red8 + 8);              // [PM_MAX_TOPK]
  float *wts = (float *)(ids + PM_MAX_TOPK);           // [PM_MAX_TOPK]
  int *s_dead = (int *)(wts + PM_MAX_TOPK);            // [4]
  float *r_sv = (float *)(((uintptr_t)(s_dead + 4) + 15) & ~(uintptr_t)15);  // route scratch, 16-byte aligned
  float *r_gs = r_sv + PM_MAX_EXPERTS;
  unsigned char *r_keep = (unsigned char *)(r_gs + PM_MAX_EXPERTS / 2);

  // this CTA's slices: h rows [R0, R1) of the layer's K*ff (R = k*ff + j), and
  // output columns [C0, C1)
  const int HR = K * ff;
  const int R0 = (int)((long long)HR * cta / G), R1 = (int)((long long)HR * (cta + 1) / G);
  const int C0 = (int)((long long)d * cta / G), C1 = (int)((long long)d * (cta + 1) / G);
  const int nrows = R1 - R0, ncols = C1 - C0;
  const int per_w = (nrows + MG_WARPS - 1) / MG_WARPS;        // h rows per warp
  const int wpc = MG_WARPS / MG_GU_CHUNKS;                     // warps per gate/up chunk
  const int ndown = K * ncols;
  const int per_d = (ndown + MG_WARPS - 1) / MG_WARPS;         // down rows per warp
  const bool has_logit = cta < E;  // E <= G (checked by the host)

  // the copy job of this thread (fixed for the whole call; only the expert changes)
  //   tid  0..15 : gate/up chunk ch, segment seg (a chunk spans at most 2 experts), gate|up
  //   tid 32..   : down, expert slot k, plane p (Q6_K: ql, qh, scales, f16 d window)
  int job_k = -1, job_off = 0, job_dst = 0, job_bytes = 0, job_bar = 0, job_plane = 0, job_tx = 0;
  if (tid < MG_GU_CHUNKS * 4) {
    int ch = tid >> 2, seg = (tid >> 1) & 1, isup = tid & 1;
    // rows of chunk ch: with 8-block rows, chunks hold whole pairs of h rows
    const int npairs_j = (nrows + 1) >> 1, ppc_j = (npairs_j + MG_GU_CHUNKS - 1) / MG_GU_CHUNKS;
    int ra = NB8 ? min(R1, R0 + 2 * ch * ppc_j) : min(R1, R0 + ch * wpc * per_w);
    int rb = NB8 ? min(R1, R0 + 2 * (ch + 1) * ppc_j) : min(R1, R0 + (ch + 1) * wpc * per_w);
    int ka = ra / ff;
    int split = min(rb, (ka + 1) * ff);
    int s0 = seg == 0 ? ra : split, s1 = seg == 0 ? split : rb;
    job_bar = ch;
    job_plane = isup;
    if (seg == 0 && isup == 0) job_tx = (rb - ra) * 2 * RBG + 1;  // +1: "this thread arms the barrier"
    if (s1 > s0) {
      job_k = s0 / ff;
      job_off = (s0 - job_k * ff) * RBG;
      job_dst = (s0 - R0) * RBG;
      job_bytes = (s1 - s0) * RBG;
    }
  } else if (tid >= 32 && tid < 32 + K * 4) {
    int k = (tid - 32) >> 2, p = (tid - 32) & 3;
    job_bar = MG_GU_CHUNKS + k;
    job_plane = 2 + p;
    int dwin0 = (C0 * nbh * 2) & ~15, dwin1 = ((C0 + ncols) * nbh * 2 + 15) & ~15;
    if (dq6) {
      const int fb[4] = {128, 64, 16, 0}, po[4] = {0, 128, 192, 0};
      if (p == 0) job_tx = ncols * nbh * 208 + (dwin1 - dwin0) + 1;
      if (p < 3) {
        job_k = k;
        job_off = C0 * nbh * fb[p];
        job_dst = k * (int)P.dn_k_bytes + P.cols_max * nbh * po[p];
        job_bytes = ncols * nbh * fb[p];
      } else {
        job_k = k;
        job_off = dwin0;
        job_dst = k * (int)P.dsm_k_bytes;
        job_bytes = dwin1 - dwin0;
      }
    } else if (p == 0) {
      job_tx = ncols * nbh * 144 + 1;
      job_k = k;
      job_off = C0 * nbh * 144;
      job_dst = k * (int)P.dn_k_bytes;
      job_bytes = ncols * nbh * 144;
    }
  }
  const int dsm_skew = ((C0 * nbh * 2) & 15) / 2;  // halfs to skip inside the 16-byte aligned window

  if (tid == 0) {
    for (int i = 0; i < MG_GU_CHUNKS; i++) mbar_init(&bar_gu[i], 1);
    for (int i = 0; i < K; i++) mbar_init(&bar_dn[i], 1);
    mbar_init(bar_rw, 1);
    *s_dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (has_logit && tid == 0) {  // router row of layer 0
    mbar_expect_tx(bar_rw, (uint32_t)d * 4);
    bulk_g2s(rw, P.layers[0].router + (size_t)cta * d, (uint32_t)d * 4, bar_rw);
  }

  // layer descriptors are staged in shared memory one layer ahead (their fields
  // would otherwise be L2-latency loads on the critical path)
  MegaLayer *mls = (MegaLayer *)(smem + P.off_ml);
  if (tid < (int)(sizeof(MegaLayer) / 8)) ((unsigned long long *)&mls[0])[tid] = ((const unsigned long long *)&P.layers[0])[tid];

  long long *trace = nullptr;
  if (P.trace && tid == 0 && (cta == 0 || cta == G - 1))
    trace = P.trace + (cta == 0 ? 0 : (size_t)P.n_layers * MG_TRACE_PH);
#define MG_TRACE(ph) do { if (trace) trace[(size_t)l * MG_TRACE_PH + (ph)] = clock64(); } while (0)
  long long *trace_r = nullptr;  // the routing warp's own stamps
  if (P.trace && tid == MG_NT - 32 && (cta == 0 || cta == G - 1))
    trace_r = P.trace + (cta == 0 ? 0 : (size_t)P.n_layers * MG_TRACE_PH);
#define MG_TRACE_R(ph) do { if (trace_r) trace_r[(size_t)l * MG_TRACE_PH + (ph)] = clock64(); } while (0)

  bool dead = false;
  bool copies_pending = false;
  const bool fold = D.weight_fold == PM_FOLD_BEFORE_DOWN;
  const bool h_fold8 = dq6 && ndown * nbh <= PM_MAX_EXPERTS;  // the Q6_K down phase works in (row, block) units
  int l = 0;
  for (; l < P.n_layers; l++) {
    const MegaLayer &ML = mls[l & 1];
    const uint32_t par = l & 1;
    const uint32_t lepoch = P.lepoch_base + (uint32_t)l + 1u;  // never repeats within 2^32 layers
    MG_TRACE(0);
    if (l + 1 < P.n_layers && tid >= 64 && tid < 64 + (int)(sizeof(MegaLayer) / 8))
      ((unsigned long long *)&mls[(l + 1) & 1])[tid - 64] = ((const unsigned long long *)&P.layers[l + 1])[tid - 64];

    // ---- 1. the residual stream (written by all CTAs at the end of the previous layer) ----
    if (l > 0) {
      if (tid == 0 && !wait_count(P.xcount, P.xcount_base + (unsigned long long)l * (unsigned long long)G, P.err, 1, P.wait_ns)) dead = true;
      if (__syncthreads_or(dead)) { dead = true; break; }
    }
    for (int i0 = tid; i0 < d; i0 += MG_NT) xs[i0] = l == 0 ? P.x_in[i0] : __ldcg(P.xbuf + i0);
    if (__syncthreads_or(dead)) { dead = true; break; }
    MG_TRACE(1);

    // ---- 2. norm, Q8x of the normed token ----
    float inv = pm_rms_inv(xs, d, P.eps, red8);
    // block qb of x is quantised by a warp that does not share an issue scheduler (warp & 3)
    // with the routing warp, which runs the layer's longest serial chain meanwhile
    const int qb = (warp & 3) == 3 ? -1 : (warp >> 2) * 3 + (warp & 3);
    if (qb >= 0 && qb < nbx) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; j++) v[j] = __fmul_rn(xs[qb * 256 + 32 * j + lane], inv);
      q8x_block_warp(v, lane, xq + qb * 256, xd + qb, xbs + qb * 8, NB8 ? qb : 0);
    } else if (warp == MG_WARPS - 1) {
      // ---- 3. this CTA's router logit, then all logits, then the scores (one warp) ----
      float *r_pr = r_sv;                          // [E] score the weight comes from
      uint32_t *r_key = (uint32_t *)(r_sv + 160);  // [E] ordered key of what is ranked
      float *sel_p = r_sv + 320;                   // [K] picked scores, selection order
      uint32_t *sel_e = (uint32_t *)(r_sv + 336);  // [K] picked experts
      {
        MG_TRACE_R(12);
        if (has_logit) {
          if (!mbar_wait(bar_rw, par, P.err, P.wait_ns)) dead = true;
          float acc = 0.0f;
#pragma unroll 16
          for (int c = lane; c < d; c += 32) acc = __fmaf_rn(rw[c], __fmul_rn(xs[c], inv), acc);
          float sdot = pm_warp_sum_dot(acc);
          if (lane == 0) {
            if (ML.logit_bias) sdot = __fadd_rn(sdot, ML.logit_bias[cta]);
            // the logit and the layer's epoch travel in one 64-bit word: a single store,
            // no release (and its half microsecond) before it, nothing else to order
            st_relaxed_u64(P.lbuf + cta, ((unsigned long long)lepoch << 32) | (unsigned long long)__float_as_uint(sdot));
          }
          __syncwarp();
          if (lane == 0 && l + 1 < P.n_layers) {  // next layer's row into the same buffer
            mbar_expect_tx(bar_rw, (uint32_t)d * 4);
            bulk_g2s(rw, P.layers[l + 1].router + (size_t)cta * d, (uint32_t)d * 4, bar_rw);
          }
        }
        MG_TRACE_R(13);
        {
          // every lane polls its own words until all of them carry this layer's epoch:
          // one round trip after the last arrival (a counter first and the values after
          // it were two); 32 x NP loads a CTA a round
          bool ok = false;
          unsigned long long t0 = 0;
          for (uint32_t it = 0;; it++) {
            bool all = true;
#pragma unroll
            for (int i = 0; i < NP; i++) {
              int e0 = lane + 32 * i;
              if (e0 < E) {
                unsigned long long w = ld_relaxed_u64(P.lbuf + e0);
                if ((uint32_t)(w >> 32) == lepoch) lg[e0] = __uint_as_float((uint32_t)w);
                else all = false;
              }
            }
            if (__all_sync(PM_FULL, all)) { ok = true; break; }
            if ((it & 63) == 63) {
              unsigned long long t = now_ns();
              if (t0 == 0) t0 = t;
              bool stop = ld_volatile_i32(P.err) != 0 || t - t0 > P.wait_ns;
              if (__any_sync(PM_FULL, stop)) break;
            }
          }
          if (!ok) {
            if (lane == 0) atomicCAS(P.err, 0, 2);
            dead = true;
          }
        }
        __syncwarp();
        MG_TRACE_R(14);
        {
          float pr[NP];
          uint32_t key[NP];
          pm_route_scores<NP>(D, lg, ML.select_bias, lane, r_sv + 352, r_gs, r_keep, pr, key);
#pragma unroll
          for (int i = 0; i < NP; i++)
            if (lane + 32 * i < E) { r_pr[lane + 32 * i] = pr[i]; r_key[lane + 32 * i] = key[i]; }
        }
      }
      MG_TRACE_R(16);
    }
    if (__syncthreads_or(dead)) { dead = true; break; }
    {
      // rank of expert e = how many experts come before it in (key descending, index
      // ascending) order: exactly the order K rounds of (max, lowest index) pick in.
      // Four threads per expert, each over a quarter of the keys.
      const float *r_pr = r_sv;
      const uint32_t *r_key = (const uint32_t *)(r_sv + 160);
      float *sel_p = r_sv + 320;
      uint32_t *sel_e = (uint32_t *)(r_sv + 336);
      const int q = tid & 3;
      const int fq = (E + 3) >> 2;
      for (int e0 = 0; e0 < E; e0 += MG_NT / 4) {
        int e = e0 + (tid >> 2);
        int rank = 0, rank2 = 0;
        if (e < E && (fq & 7) == 0 && E == 4 * fq && r_key[e] != 0u) {
          // "before e" is k_f >= ke for f < e and k_f > ke for f > e: one compare against
          // ke - 1 or ke (ke != 0), the keys read eight at a time
          const uint32_t ke = r_key[e], kem1 = ke - 1u;
          const int fa = q * fq, nlo = e - fa;  // keys j < nlo of this quarter lie below e
          // the four quarters of an expert start eight keys apart: their 32-byte reads would
          // otherwise fall on the same banks (quarters are fq words apart) four ways
          const int jrot = (8 * q) % fq;
          for (int j0 = 0; j0 < fq; j0 += 8) {
            const int j = j0 + jrot < fq ? j0 + jrot : j0 + jrot - fq;
            const uint4 a = *(const uint4 *)(r_key + fa + j), b = *(const uint4 *)(r_key + fa + j + 4);
            rank += a.x > (j + 0 < nlo ? kem1 : ke);
            rank2 += a.y > (j + 1 < nlo ? kem1 : ke);
            rank += a.z > (j + 2 < nlo ? kem1 : ke);
            rank2 += a.w > (j + 3 < nlo ? kem1 : ke);
            rank += b.x > (j + 4 < nlo ? kem1 : ke);
            rank2 += b.y > (j + 5 < nlo ? kem1 : ke);
            rank += b.z > (j + 6 < nlo ? kem1 : ke);
            rank2 += b.w > (j + 7 < nlo ? kem1 : ke);
          }
        } else if (e < E) {
          uint32_t ke = r_key[e];
          int fa = q * fq, fb = min(E, fa + fq);
          for (int f = fa; f + 1 < fb; f += 2) {
            uint32_t k0 = r_key[f], k1 = r_key[f + 1];
            rank += (k0 > ke) || (k0 == ke && f < e);
            rank2 += (k1 > ke) || (k1 == ke && f + 1 < e);
          }
          if ((fb - fa) & 1) {
            uint32_t k0 = r_key[fb - 1];
            rank += (k0 > ke) || (k0 == ke && fb - 1 < e);
          }
        }
        rank += rank2;
        rank += __shfl_xor_sync(PM_FULL, rank, 1);
        rank += __shfl_xor_sync(PM_FULL, rank, 2);
        if (q == 0 && e < E && rank < K) { sel_e[rank] = (uint32_t)e; sel_p[rank] = r_pr[e]; }
      }
    }
    // ---- 4. bulk copies of this CTA's slices: gate/up now, down once gate/up has landed
    // (the gate/up bytes are needed first and should not share HBM with bytes needed later) ----
    auto issue_job = [&]() {
      if (job_tx) mbar_expect_tx(&bar_gu[job_bar], (uint32_t)(job_tx - 1));  // bar_dn follows bar_gu in memory
      if (job_bytes > 0) {
        // gate/up jobs go out before `ids` is written: they read the ranking's own list
        int el = (int)(job_plane < 2 ? ((const uint32_t *)(r_sv + 336))[job_k] : ids[job_k]);
        const uint8_t *src;
        uint8_t *dst;
        if (job_plane == 0) { src = ML.gate + (size_t)el * ML.gate_stride; dst = gs; }
        else if (job_plane == 1) { src = ML.up + (size_t)el * ML.up_stride; dst = us; }
        else {
          int p = job_plane - 2;
          src = ML.down[p] + (size_t)el * ML.down_stride[p];
          dst = p == 3 ? dsm : dn;
        }
        bulk_g2s(dst + job_dst, src + job_off, (uint32_t)job_bytes, &bar_gu[job_bar]);
      }
    };
    __syncthreads();
    // the experts are known: the gate/up copies leave now, the weights follow meanwhile
    if (tid < MG_GU_CHUNKS * 4) issue_job();
    copies_pending = true;
    if (warp == MG_WARPS - 1) {
      const float *sel_p = r_sv + 320;
      const uint32_t *sel_e = (const uint32_t *)(r_sv + 336);
      MG_TRACE_R(18);
      if (lane < K) {
        ids[lane] = sel_e[lane];
        wts[lane] = pm_route_weight(D, sel_p, lane);
      }
      __syncwarp();
      MG_TRACE_R(15);
      if (cta == 0 && lane < K && ML.usage) atomicAdd(&ML.usage[ids[lane]], 1u);
    }
    if (__syncthreads_or(dead)) { dead = true; break; }
    MG_TRACE(2);

    MG_TRACE(3);

    // ---- 5. gate/up rows -> h ----
    if (NB8) {
      // pairs of h rows: lanes 0-7 gate(h0), 8-15 up(h0), 16-23 gate(h1), 24-31 up(h1)
      XBlk X;
      {
        const int4 *xp = (const int4 *)(xq + 256 * (lane & 7));
#pragma unroll
        for (int j = 0; j < 16; j++) {
          int4 t = xp[j ^ (lane & 7)];  // chunks are stored swizzled by the block index
          X.x[4 * j] = t.x; X.x[4 * j + 1] = t.y; X.x[4 * j + 2] = t.z; X.x[4 * j + 3] = t.w;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) X.bs[j] = xbs[8 * (lane & 7) + j];
        X.d = xd[lane & 7];
      }
      const int npairs = (nrows + 1) >> 1;
      const int ppc = (npairs + MG_GU_CHUNKS - 1) / MG_GU_CHUNKS;  // pairs per copy chunk
      for (int p = warp; p < npairs; p += MG_WARPS) {
        if (!__all_sync(PM_FULL, mbar_wait(&bar_gu[p / ppc], par, P.err, P.wait_ns))) { dead = true; break; }
        if (p == warp) MG_TRACE(8);
        int rel = 2 * p + ((lane >> 4) & 1);
        rel = min(rel, nrows - 1);
        const uint8_t *rowp = ((lane >> 3) & 1 ? us : gs) + (size_t)rel * RBG;
        float tot = row4_q4k_blk(rowp, X, lane);
        float gv = __shfl_sync(PM_FULL, tot, (lane & 1) * 16);
        float uv = __shfl_sync(PM_FULL, tot, (lane & 1) * 16 + 8);
        int r = R0 + 2 * p + lane;
        if (lane < 2 && r < R1) {
          float hv = pm_act(D.act, D.act_limit, D.act_alpha, gv, uv, wts[r / ff], fold);
          __stcg(P.hbuf + r, hv);
        }
      }
    } else {
      int ra = R0 + warp * per_w, rb = min(R1, ra + per_w);
      if (ra < rb) {
        if (!__all_sync(PM_FULL, mbar_wait(&bar_gu[warp / wpc], par, P.err, P.wait_ns))) dead = true;
      }
      MG_TRACE(8);
      for (int r0 = ra; r0 < rb && !dead; r0 += MG_GH) {
        const uint8_t *rowp[2 * MG_GH];
        const int8_t *xqp[2 * MG_GH];
        const float *xdp[2 * MG_GH];
        const int32_t *xbp[2 * MG_GH];
#pragma unroll
        for (int i = 0; i < MG_GH; i++) {
          int rel = min(r0 + i, rb - 1) - R0;
          rowp[2 * i] = gs + (size_t)rel * RBG;
          rowp[2 * i + 1] = us + (size_t)rel * RBG;
        }
#pragma unroll
        for (int i = 0; i < 2 * MG_GH; i++) { xqp[i] = xq; xdp[i] = xd; xbp[i] = xbs; }
        float tot[2 * MG_GH];
        rows_q4k_smem<2 * MG_GH>(rowp, nbx, xqp, xdp, xbp, lane, tot);
#pragma unroll
        for (int i = 0; i < MG_GH; i++) {
          int r = r0 + i;
          if (lane == i && r < rb) {
            float hv = pm_act(D.act, D.act_limit, D.act_alpha, tot[2 * i], tot[2 * i + 1], wts[r / ff], fold);
            __stcg(P.hbuf + r, hv);
          }
        }
      }
    }
    MG_TRACE(11);
    if (__syncthreads_or(dead)) { dead = true; break; }
    // h is published first, the down slices (job threads 32 .. 32 + 4K: warps 1 and 2) are
    // issued after it: with 70 KB of bulk copies in flight the release took three times as long
    if (warp == 0) {
      if (tid == 0) red_release_add_u64(P.hcount, 1ull);
      __syncwarp();
      asm volatile("bar.arrive 3, 96;" ::: "memory");
    } else if (warp <= 2) {
      asm volatile("bar.sync 3, 96;" ::: "memory");
      issue_job();
    }
    MG_TRACE(4);

    // ---- 6. all of h, re-quantised ----
    if (tid == 0) {
      unsigned long long want = P.hcount_base + (unsigned long long)(l + 1) * (unsigned long long)G;
      bool ok = false;
      unsigned long long t0 = now_ns();
      for (uint32_t it = 0;; it++) {
        if (ld_acquire_u64(P.hcount) >= want) { ok = true; break; }
        if ((it & 63) == 63 && (ld_volatile_i32(P.err) != 0 || now_ns() - t0 > P.wait_ns)) break;
      }
      if (!ok) { atomicCAS(P.err, 0, 3); dead = true; }
    }
    if (__syncthreads_or(dead)) { dead = true; break; }
    MG_TRACE(5);
    for (int b0 = warp; b0 < K * nbh; b0 += 2 * MG_WARPS) {
      int b1 = b0 + MG_WARPS;
      float v0[8], v1[8];
#pragma unroll
      for (int j = 0; j < 8; j++) v0[j] = __ldcg(P.hbuf + b0 * 256 + 32 * j + lane);
      if (b1 < K * nbh) {
#pragma unroll
        for (int j = 0; j < 8; j++) v1[j] = __ldcg(P.hbuf + b1 * 256 + 32 * j + lane);
      }
      q8x_block_warp(v0, lane, hq + b0 * 256, hd + b0, hbs + b0 * 8, 0, h_fold8);
      if (b1 < K * nbh) q8x_block_warp(v1, lane, hq + b1 * 256, hd + b1, hbs + b1 * 8, 0, h_fold8);
    }
    __syncthreads();
    MG_TRACE(6);

    // ---- 7. down rows of this CTA's columns, all k; sum in k order; publish ----
    if (h_fold8) {
      // One (row, block) unit per lane: 256 six-bit values against the block of h, no
      // cross-lane traffic. isum = sum_c sc[c] * (q_c . h_c - 32 * sum(h_c)) over the 16
      // chunks c of 16 values (the integer sum of `row_q6k_q8x`, regrouped). Lanes walk the
      // 16-byte pieces in a rotated order so that units 128 bytes apart hit different banks.
      float *tmp = r_sv;  // [ndown * nbh] terms; the routing scratch is idle here
      const size_t cm = (size_t)P.cols_max * nbh;
      for (int u = tid; u < ndown * nbh; u += MG_NT) {
        const int i = u / nbh, b = u - i * nbh, k = i / ncols, cc = i - k * ncols;
        if (!mbar_wait(&bar_dn[k], par, P.err, P.wait_ns)) dead = true;
        const uint8_t *base = dn + (size_t)k * P.dn_k_bytes;
        const size_t rb = (size_t)cc * nbh + b;
        const uint8_t *qlp = base + rb * 128, *qhp = base + cm * 128 + rb * 64;
        const int8_t *scp = (const int8_t *)(base + cm * 192 + rb * 16);
        const int8_t *xb = hq + k * ff + b * 256;
        int isum = 0;
#pragma unroll
        for (int p = 0; p < 8; p++) {
          // piece order per lane: a rotation of a permutation (bits 0 and 1 of the lane
          // swapped) under which lanes 128 bytes apart in the 64-byte-a-unit qh plane, i.e.
          // lanes of equal parity, take four different qh pieces
          const int pl = (lane & 4) | ((lane & 1) << 1) | ((lane >> 1) & 1);
          const int pp = (p + pl) & 7, n = pp >> 2, jj = (pp >> 1) & 1, g = pp & 1;
          const uint4 qlv = *(const uint4 *)(qlp + pp * 16);
          const uint4 qhv = *(const uint4 *)(qhp + (2 * n + g) * 16);
          const int clo = 8 * n + 2 * jj + g, chi = clo + 4;  // chunks of the low / high nibbles
          // h's chunks 8-15 are stored with their halves swapped (`fold8`)
          const int4 xlo = *(const int4 *)(xb + (clo + 4 * n) * 16), xhi = *(const int4 *)(xb + (chi - 4 * n) * 16);
          const int sh = 2 * jj;
          const uint32_t qlw[4] = {qlv.x, qlv.y, qlv.z, qlv.w}, qhw[4] = {qhv.x, qhv.y, qhv.z, qhv.w};
          const int xl[4] = {xlo.x, xlo.y, xlo.z, xlo.w}, xh[4] = {xhi.x, xhi.y, xhi.z, xhi.w};
          int dlo = 0, dhi = 0, slo = 0, shi = 0;  // q . h and sum(h) of the two chunks
#pragma unroll
          for (int w = 0; w < 4; w++) {
            const uint32_t qa = (qlw[w] & 0x0f0f0f0fu) | (((qhw[w] >> sh) & 0x03030303u) << 4);
            const uint32_t qb = ((qlw[w] >> 4) & 0x0f0f0f0fu) | (((qhw[w] >> (sh + 4)) & 0x03030303u) << 4);
            dlo = __dp4a((int)qa, xl[w], dlo);
            dhi = __dp4a((int)qb, xh[w], dhi);
            slo = __dp4a(0x01010101, xl[w], slo);
            shi = __dp4a(0x01010101, xh[w], shi);
          }
          isum += (int)scp[clo] * (dlo - 32 * slo) + (int)scp[chi] * (dhi - 32 * shi);
        }
        const float dd = __half2float(((const __half *)(dsm + (size_t)k * P.dsm_k_bytes))[dsm_skew + cc * nbh + b]);
        tmp[u] = __fmul_rn(hd[k * nbh + b], __fmul_rn(dd, (float)isum));
      }
      MG_TRACE(9);
      if (__syncthreads_or(dead)) { dead = true; copies_pending = true; break; }
      for (int i = tid; i < ndown; i += MG_NT) {  // the row's terms in block order
        float total = 0.0f;
        for (int b = 0; b < nbh; b++) total = __fadd_rn(total, tmp[i * nbh + b]);
        const int k = i / ncols, cc = i - k * ncols;
        eo[k * P.cols_max + cc] = total;
      }
    } else {
      int ia = warp * per_d, ib = min(ndown, ia + per_d);
      for (int i0 = ia; i0 < ib && !dead; i0 += MG_DR) {
        int kk[MG_DR], cc[MG_DR];
#pragma unroll
        for (int r = 0; r < MG_DR; r++) {
          int i = min(i0 + r, ib - 1);
          kk[r] = i / ncols;
          cc[r] = i - kk[r] * ncols;
          if (!__all_sync(PM_FULL, mbar_wait(&bar_dn[kk[r]], par, P.err, P.wait_ns))) dead = true;
        }
        if (dead) break;
        if (i0 == ia) MG_TRACE(9);
        const int8_t *xqp[MG_DR];
        const float *xdp[MG_DR];
        float tot[MG_DR];
        if (dq6) {
          const uint8_t *ql[MG_DR], *qh[MG_DR], *sc[MG_DR];
          const __half *dp[MG_DR];
          size_t cm = (size_t)P.cols_max * nbh;
#pragma unroll
          for (int r = 0; r < MG_DR; r++) {
            const uint8_t *base = dn + (size_t)kk[r] * P.dn_k_bytes;
            ql[r] = base + (size_t)cc[r] * nbh * 128;
            qh[r] = base + cm * 128 + (size_t)cc[r] * nbh * 64;
            sc[r] = base + cm * 192 + (size_t)cc[r] * nbh * 16;
            dp[r] = (const __half *)(dsm + (size_t)kk[r] * P.dsm_k_bytes) + dsm_skew + cc[r] * nbh;
            xqp[r] = hq + kk[r] * ff;
            xdp[r] = hd + kk[r] * nbh;
          }
          rows_q6k_smem<MG_DR>(ql, qh, sc, dp, nbh, xqp, xdp, lane, tot);
        } else {
          const uint8_t *rowp[MG_DR];
          const int32_t *xbp[MG_DR];
#pragma unroll
          for (int r = 0; r < MG_DR; r++) {
            rowp[r] = dn + (size_t)kk[r] * P.dn_k_bytes + (size_t)cc[r] * nbh * 144;
            xqp[r] = hq + kk[r] * ff;
            xdp[r] = hd + kk[r] * nbh;
            xbp[r] = hbs + kk[r] * nbh * 8;
          }
          rows_q4k_smem<MG_DR>(rowp, nbh, xqp, xdp, xbp, lane, tot);
        }
#pragma unroll
        for (int r = 0; r < MG_DR; r++)
          if (lane == r && i0 + r < ib) eo[kk[r] * P.cols_max + cc[r]] = tot[r];
      }
    }
    MG_TRACE(10);
    copies_pending = false;  // every chunk barrier of this layer was waited on by some warp
    if (__syncthreads_or(dead)) { dead = true; copies_pending = true; break; }
    if (tid < ncols) {
      float s = 0.0f;
      for (int k = 0; k < K; k++) {
        float v = eo[k * P.cols_max + tid];
        if (!fold) v = __fmul_rn(wts[k], v);
        s = __fadd_rn(s, v);
      }
      float xn = __fadd_rn(xs[C0 + tid], s);
      if (l + 1 < P.n_layers) __stcg(P.xbuf + C0 + tid, xn);
      else P.x_out[C0 + tid] = xn;
    }
    MG_TRACE(7);
    __syncthreads();  // eo, xs, ids are rewritten by the next layer
    if (tid == 0 && l + 1 < P.n_layers) red_release_add_u64(P.xcount, 1ull);
  }

  if (dead) {
    // give this CTA's own copies a bounded time to land before its shared memory goes away
    __syncthreads();
    if (tid == 0) {
      uint32_t par = l & 1;
      // (one time bound for the whole drain, the same as every other wait's: a barrier that was
      // never armed for this layer has nothing in flight and is simply given up on)
      const unsigned long long t0 = now_ns();
      if (copies_pending) {
        for (int i = 0; i < MG_GU_CHUNKS + K; i++)
          while (!mbar_try_wait_ns(&bar_gu[i], par, 2000u) && now_ns() - t0 < P.wait_ns) {}
      }
      if (has_logit)
        while (!mbar_try_wait_ns(bar_rw, par, 2000u) && now_ns() - t0 < P.wait_ns) {}
    }
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
  if (D.d / 256 > MG_WARPS - 4) return false;  // the last 4 warps route while the first d/256 quantise
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
  P.dsm_k_bytes = up16((uint32_t)cols_max * nbh * 2 + 32);
  P.off_dsm = take(P.dsm_k_bytes * K);
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
  P.off_ml = take(2 * (uint32_t)sizeof(MegaLayer));
  P.off_misc = take(8 * (MG_GU_CHUNKS + PM_MAX_TOPK + 1) + 8 * 4 + PM_MAX_TOPK * 8 + 16 +
                    PM_MAX_EXPERTS * 4 + PM_MAX_EXPERTS * 2 + PM_MAX_EXPERTS / 2 + 64);
  mp.smem = off;
  if (mp.smem > smem_optin) return false;
  mp.grid = G;
  mp.ok = true;
  return true;
}

typedef void (*MegaKernel)(const MegaParams);
static MegaKernel mega_kernel(const pm_layer_desc &D) {
  bool dq6 = D.type_down == PM_TYPE_Q6_K, nb8 = D.d == 2048, big = D.n_exp > 128;
  if (dq6) {
    if (nb8) return big ? k_decode_mega<true, true, 8> : k_decode_mega<true, true, 4>;
    return big ? k_decode_mega<true, false, 8> : k_decode_mega<true, false, 4>;
  }
  if (nb8) return big ? k_decode_mega<false, true, 8> : k_decode_mega<false, true, 4>;
  return big ? k_decode_mega<false, false, 8> : k_decode_mega<false, false, 4>;
}

cudaError_t mega_prepare(const pm_layer_desc &D, size_t smem) {
  return cudaFuncSetAttribute((const void *)mega_kernel(D), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

int mega_max_ctas_per_sm(const pm_layer_desc &D, size_t smem) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, (const void *)mega_kernel(D), MG_NT, smem) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

cudaError_t mega_launch(const MegaPlan &mp, cudaStream_t stream) {
  MegaParams P = mp.P;
  void *args[] = {(void *)&P};
  return cudaLaunchCooperativeKernel((const void *)mega_kernel(P.D), dim3(mp.grid), dim3(MG_NT), args, mp.smem, stream);
}
