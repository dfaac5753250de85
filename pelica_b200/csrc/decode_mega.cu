// decode_mega.cu - one-token decode of a whole MoE layer stack in ONE persistent
// cooperative kernel (one CTA per SM).
//
// Why: at batch 1 a Qwen3-30B-A3B-shaped layer reads 24.5 MB of expert blocks,
// 3.8 us at HBM speed; a kernel launch per phase costs more than that, and so does
// every grid-wide hand-off that is built from a release fence and an arrival counter.
// Here every CTA walks all layers, and the three hand-offs a layer needs (the residual
// stream, the router logits, the hidden vector) are arrays of 64-bit words
// (layer epoch << 32 | float bits): a writer stores a word once, relaxed, with no fence;
// a reader polls the words it needs until they carry the layer's epoch. Per layer a CTA
//   1. collects the residual stream x (every thread polls four words),
//   2. norms it and quantises it to Q8x (`Q8x::new`, src/ds4_cpu.rs:13-35),
//   3. computes "its" router logit in `dot_f32` order (src/quant.rs:215-236), publishes
//      it; its last warp polls all E logits, turns them into scores (route.cuh); all
//      threads rank the keys (rank < k = picked, in the order k rounds of (max, lowest
//      index) would pick),
//   4. issues bulk async copies (cp.async.bulk + mbarrier) of ITS slice of the chosen
//      experts' gate/up rows into shared memory, and of its slice of their down rows
//      once the first gate/up chunks have landed (the bytes needed first go first): the
//      layer's 24.5 MB is spread over the SMs' shared memories and HBM streams without
//      waiting for any compute,
//   5. gate/up rows . xq -> SwiGLU -> h, published word by word,
//   6. collects all of h (each warp polls the blocks it quantises) and re-quantises it
//      (src/ds4_cpu.rs:306-317),
//   7. down rows of ITS columns for all k experts, one (row, 256-value block) per lane,
//      summed in block order, then in k order (src/moe_kernels.rs:1798-1808); x += y is
//      published for the next layer.
// The arithmetic is the general kernels' (same bits as the CPU reference path).
//
// Every wait (words of another CTA, copy barriers) is bounded by MegaParams::wait_ns: a
// wait that runs out sets an error word, every CTA then leaves its layer loop at the next
// CTA barrier, waits (bounded) for its own copies in flight and returns; the host reports
// PM_ERR_TIMEOUT. The launch is cooperative, so all CTAs are co-resident.
//
// The loop body is kept small on purpose (no per-shape template variants inside, few
// unrolled loops): most of it runs once per layer in a single warp, where every
// instruction-cache miss is exposed latency.
#include "decode_mega.cuh"
#include "route.cuh"

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
// blocking form with a suspend-time hint: the warp sleeps in hardware for at most `ns`
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
// global -> this CTA's shared memory, completion counted on `bar` (no multicast). The bytes
// are read once per token: they are marked evict-first in L2, so that a layer's 24.5 MB do not
// push out the few lines the CTAs talk through (a hand-off word that has left L2 costs its
// writer and every reader a DRAM round trip).
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes,
                                         uint64_t *bar) {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
          "r"(s32(dst)),
      "l"(src), "r"(bytes), "r"(s32(bar)), "l"(pol)
      : "memory");
}
__device__ __forceinline__ void ld_relaxed_2u64(const unsigned long long *p, unsigned long long &a,
                                                unsigned long long &b) {
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long *p) {
  unsigned long long u;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(u) : "l"(p) : "memory");
  return u;
}
__device__ __forceinline__ void red_relaxed_add_u64(unsigned long long *p, unsigned long long v) {
  asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long *p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
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
__device__ __forceinline__ unsigned long long tagged(uint32_t epoch, float v) {
  return ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
}
// has this wait run out (or has any CTA recorded an error)? Called every few dozen polls.
__device__ __noinline__ bool wait_expired(unsigned long long &t0, const int *err, unsigned long long wait_ns) {
  if (ld_volatile_i32(err) != 0) return true;
  const unsigned long long t = now_ns();
  if (t0 == 0) t0 = t;
  return t - t0 > wait_ns;
}
// bounded wait on an mbarrier phase; false = gave up (error word set)
__device__ __noinline__ bool mbar_wait_slow(uint64_t *bar, uint32_t parity, int *err, unsigned long long wait_ns) {
  unsigned long long t0 = 0;
  for (uint32_t it = 1;; it++) {
    if (mbar_try_wait_ns(bar, parity, 2000u)) return true;
    if ((it & 7) == 0 && wait_expired(t0, err, wait_ns)) break;
  }
  atomicCAS(err, 0, 2);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *err, unsigned long long wait_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, err, wait_ns);
}

// round half away from zero, as f32::round (|x| < 2^23): the truncation and the remainder
// are exact, so this is roundf's result without its general-range code
__device__ __forceinline__ float round_half_away(float x) {
  const float t = truncf(x);
  return fabsf(__fsub_rn(x, t)) >= 0.5f ? __fadd_rn(t, copysignf(1.0f, x)) : t;
}

// ---- Q8x of 256 values held 8 per lane (value j of the lane = element 32j + lane)
// (`Q8x::new`, src/ds4_cpu.rs:13-35) by one warp; writes q, d and the block's partial sums.
// `swz`: 16-byte chunk c of the block is stored at chunk c ^ swz (so that lanes reading the
// same chunk of 8 different blocks hit different banks).
// `fold8`: chunks 8-15 additionally swap their halves (c ^ 4), for the Q6_K down units, whose
// lanes read chunks {0-3, 8-11} (then {4-7, 12-15}) at once: banks 0-15 twice without it.
// `sum16`: sums[0..15] = sums of the 16 chunks of 16 values (the Q6_K units' offset term);
// otherwise sums[0..7] = sums of the 8 groups of 32 values (`bsum`, the Q4_K mins' term).
// Built for latency (one warp runs it alone): the eight values are independent chains, the
// block maximum is one warp reduction on the bit patterns (non-negative floats order like
// unsigned integers), the partial sums are byte sums (dp4a) over the stored chunks.
__device__ __forceinline__ void q8x_block_regs(const float v[8], int lane, int8_t *q, float *d, int32_t *sums,
                                               int swz, bool fold8, bool sum16) {
  float a = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; j++) a = fmaxf(a, fabsf(v[j]));
  a = __uint_as_float(__reduce_max_sync(PM_FULL, __float_as_uint(a)));
  const float id = a != 0.0f ? __fdiv_rn(127.0f, a) : 0.0f;  // (a == 0: every value is 0, and stays 0)
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const float f = round_half_away(__fmul_rn(v[j], id));
    const int r = (int)fminf(fmaxf(f, -127.0f), 127.0f);
    int c = (2 * j + (lane >> 4)) ^ swz;
    if (fold8) c ^= (c & 8) >> 1;
    q[(c << 4) + (lane & 15)] = (int8_t)r;
  }
  __syncwarp();
  if (lane < 16) {
    // lane = logical chunk (sum16) / group g = lane >> 1 with its two chunks (else)
    int c = lane ^ swz;
    if (fold8) c ^= (c & 8) >> 1;
    const int4 w = *(const int4 *)(q + (c << 4));
    int sacc = __dp4a(0x01010101, w.x, 0);
    sacc = __dp4a(0x01010101, w.y, sacc);
    sacc = __dp4a(0x01010101, w.z, sacc);
    sacc = __dp4a(0x01010101, w.w, sacc);
    if (sum16) {
      sums[lane] = sacc;
    } else {
      sacc += __shfl_xor_sync(0x0000ffffu, sacc, 1);
      if ((lane & 1) == 0) sums[lane >> 1] = sacc;
    }
  }
  if (lane == 0) *d = a != 0.0f ? __fdiv_rn(a, 127.0f) : 0.0f;
}

__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Q4_K sub-block scale/min pair (2c, 2c+1) of a block header, branch-free
// (`scales`, src/ds4_cpu.rs:45-57)
__device__ __forceinline__ void q4k_scmin_pair(const uint4 &hdr, int c, int &sc0, int &m0, int &sc1, int &m1) {
  // j = 2c, 2c+1.  c < 2: plain 6-bit fields of words y (scales) and z (mins);
  // c >= 2: low nibbles from word w, high 2 bits from the top of y / z bytes.
  const int sh = 8 * ((2 * c) & 3);
  const uint32_t by0 = (hdr.y >> sh) & 0xff, by1 = (hdr.y >> (sh + 8)) & 0xff;
  const uint32_t bz0 = (hdr.z >> sh) & 0xff, bz1 = (hdr.z >> (sh + 8)) & 0xff;
  const uint32_t bw0 = (hdr.w >> sh) & 0xff, bw1 = (hdr.w >> (sh + 8)) & 0xff;
  const bool hi = c >= 2;
  sc0 = hi ? (int)((bw0 & 15) | ((by0 >> 6) << 4)) : (int)(by0 & 63);
  m0 = hi ? (int)((bw0 >> 4) | ((bz0 >> 6) << 4)) : (int)(bz0 & 63);
  sc1 = hi ? (int)((bw1 & 15) | ((by1 >> 6) << 4)) : (int)(by1 & 63);
  m1 = hi ? (int)((bw1 >> 4) | ((bz1 >> 6) << 4)) : (int)(bz1 & 63);
}

// A lane's block of a quantised vector: 64 words of int8, the 8 group sums, the scale.
struct XBlk {
  int x[64];
  int bs[8];
  float d;
};

// One Q4_K block (144 bytes at `blk`) against X: the block's float term
// x.d * (d * isum - dmin * msum) with the integer sums of `row_scalar` (src/ds4_cpu.rs:59-83).
// Unrolled on purpose: the four rounds are independent chains (a lane runs this once or
// twice a layer, on the layer's critical path).
__device__ __forceinline__ float q4k_block_term(const uint8_t *blk, const XBlk &X) {
  const uint4 hdr = *(const uint4 *)blk;
  const uint4 *qp = (const uint4 *)(blk + 16);
  const uint32_t ML = 0x0f0f0f0fu, MH = 0xf0f0f0f0u;
  int isum = 0, msum = 0;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    const uint4 q0 = qp[2 * c], q1 = qp[2 * c + 1];
    int l = 0, h = 0;
    l = __dp4a((int)(q0.x & ML), X.x[16 * c + 0], l); h = dp4a_us(q0.x & MH, X.x[16 * c + 8], h);
    l = __dp4a((int)(q0.y & ML), X.x[16 * c + 1], l); h = dp4a_us(q0.y & MH, X.x[16 * c + 9], h);
    l = __dp4a((int)(q0.z & ML), X.x[16 * c + 2], l); h = dp4a_us(q0.z & MH, X.x[16 * c + 10], h);
    l = __dp4a((int)(q0.w & ML), X.x[16 * c + 3], l); h = dp4a_us(q0.w & MH, X.x[16 * c + 11], h);
    l = __dp4a((int)(q1.x & ML), X.x[16 * c + 4], l); h = dp4a_us(q1.x & MH, X.x[16 * c + 12], h);
    l = __dp4a((int)(q1.y & ML), X.x[16 * c + 5], l); h = dp4a_us(q1.y & MH, X.x[16 * c + 13], h);
    l = __dp4a((int)(q1.z & ML), X.x[16 * c + 6], l); h = dp4a_us(q1.z & MH, X.x[16 * c + 14], h);
    l = __dp4a((int)(q1.w & ML), X.x[16 * c + 7], l); h = dp4a_us(q1.w & MH, X.x[16 * c + 15], h);
    int sc0, m0, sc1, m1;
    q4k_scmin_pair(hdr, c, sc0, m0, sc1, m1);
    isum += sc0 * l + sc1 * (h >> 4);  // the high-nibble dot was accumulated 16-fold (exact)
    msum += m0 * X.bs[2 * c] + m1 * X.bs[2 * c + 1];
  }
  const float dd = pm_f16(hdr.x), dmin = pm_f16(hdr.x >> 16);
  return __fmul_rn(X.d, __fsub_rn(__fmul_rn(dd, (float)isum), __fmul_rn(dmin, (float)msum)));
}

// block `b` of a quantised vector in shared memory (chunk c stored at c ^ swz; the block's
// 8 group sums at bs[bs_stride * b ..]) -> registers
__device__ __forceinline__ void load_xblk(XBlk &X, const int8_t *q, const float *dv, const int32_t *bs,
                                          int bs_stride, int b, int swz) {
  const int4 *xp = (const int4 *)(q + 256 * b);
#pragma unroll
  for (int j = 0; j < 16; j++) {
    const int4 t = xp[j ^ swz];
    X.x[4 * j] = t.x; X.x[4 * j + 1] = t.y; X.x[4 * j + 2] = t.z; X.x[4 * j + 3] = t.w;
  }
#pragma unroll
  for (int j = 0; j < 8; j++) X.bs[j] = bs[bs_stride * b + j];
  X.d = dv[b];
}

// Softmax over all E <= 128 logits by one warp (src/moe_kernels.rs:1023-1049): the same
// operations in the same order as pm_route_scores (lane L holds experts L, L+32, ...: their
// exponentials are summed per lane in ascending order, the lanes by xor shuffles 16..1),
// without the other gating variants around it. pr[e] = the probability, key[e] = the
// ordered key of probability (+ selection bias).
__device__ __forceinline__ void scores_softmax4(const float *lg, const float *__restrict__ sel_bias, int E, int lane,
                                                float *pr, uint32_t *key) {
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; i++) v[i] = lane + 32 * i < E ? lg[lane + 32 * i] : PM_NEG;
  float mx = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
  mx = pm_funkey(__reduce_max_sync(PM_FULL, pm_fkey(mx)));
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; i++)
    if (lane + 32 * i < E) {
      v[i] = pm_exp(__fsub_rn(v[i], mx));
      sum = __fadd_rn(sum, v[i]);
    }
  sum = pm_warp_sum_16_1(sum);
#pragma unroll
  for (int i = 0; i < 4; i++)
    if (lane + 32 * i < E) {
      const int e = lane + 32 * i;
      const float p = __fdiv_rn(v[i], sum);
      pr[e] = p;
      key[e] = pm_fkey(sel_bias ? __fadd_rn(p, sel_bias[e]) : p);
    }
}

// ---- the kernel ------------------------------------------------------------
// DQ6: the down weights are Q6_K (else Q4_K). TR: phase stamps are compiled in (the plain
// kernel carries none: even predicated-off stamps cost a few per cent here).
template <bool DQ6, bool TR>
__global__ void __launch_bounds__(MG_NT, 1) k_decode_mega(const MegaParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  const pm_layer_desc &D = P.D;
  const int d = D.d, ff = D.ff, E = D.n_exp, K = D.top_k;
  const int G = gridDim.x, cta = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nbx = d >> 8, nbh = ff >> 8;  // nbx is 1, 2, 4 or 8 (checked by the host)
  const int RBG = nbx * 144;              // bytes of a gate/up row

  uint8_t *gs = smem + P.off_gs, *us = smem + P.off_us, *dn = smem + P.off_dn;
  uint8_t *dsm = smem + P.off_dsm;
  float *xs = (float *)(smem + P.off_xs);
  int8_t *xq = (int8_t *)(smem + P.off_xq);
  float *xd = (float *)(smem + P.off_xd);
  int32_t *xbs = (int32_t *)(smem + P.off_xbs);
  int8_t *hq = (int8_t *)(smem + P.off_hq);
  float *hd = (float *)(smem + P.off_hd);
  int32_t *hbs = (int32_t *)(smem + P.off_hbs);  // per block of h: 16 chunk sums (Q6_K) / 8 group sums (Q4_K)
  float *rw = (float *)(smem + P.off_rw);
  float *tmp = (float *)(smem + P.off_tmp);
  float *lg = (float *)(smem + P.off_lg);
  uint64_t *bar_gu = (uint64_t *)(smem + P.off_misc);  // [MG_GU_CHUNKS]
  uint64_t *bar_dn = bar_gu + MG_GU_CHUNKS;            // [PM_MAX_TOPK]
  uint64_t *bar_rw = bar_dn + PM_MAX_TOPK;             // [1]
  float *red8 = (float *)(bar_rw + 1);                 // [8]
  float *wts = red8 + 8;                               // [PM_MAX_TOPK]
  float *sel_p = wts + PM_MAX_TOPK;                    // [PM_MAX_TOPK] picked scores, selection order
  uint32_t *sel_e = (uint32_t *)(sel_p + PM_MAX_TOPK); // [PM_MAX_TOPK] picked experts
  // per copy barrier: 0 = never armed, else 1 + the parity of the phase its last copies complete
  int *armed = (int *)(sel_e + PM_MAX_TOPK);           // [MG_GU_CHUNKS + PM_MAX_TOPK + 1]
  int *s_cnt = armed + MG_GU_CHUNKS + PM_MAX_TOPK + 1; // [2] warps done with their h rows / their columns
  const int A_RW = MG_GU_CHUNKS + PM_MAX_TOPK;
  float *r_pr = (float *)(armed + MG_GU_CHUNKS + PM_MAX_TOPK + 4);  // [128] score the weight comes from
  uint32_t *r_key = (uint32_t *)(r_pr + 128);                       // [128] ordered key of what is ranked
  float *r_sv = (float *)(r_key + 128);                             // [128] group-limited selection scratch
  float *r_gs = r_sv + 128;                                         // [64]
  unsigned char *r_keep = (unsigned char *)(r_gs + 64);             // [64]

  // this CTA's slices: h rows [R0, R1) of the layer's K*ff (R = k*ff + j), and
  // output columns [C0, C1)
  const int HR = K * ff;
  const int R0 = (int)((long long)HR * cta / G), R1 = (int)((long long)HR * (cta + 1) / G);
  const int C0 = (int)((long long)d * cta / G), C1 = (int)((long long)d * (cta + 1) / G);
  const int nrows = R1 - R0, ncols = C1 - C0;
  // gate/up passes: a warp pass is 32 / nbx weight rows = rp h rows (gate row and up row each),
  // a lane one whole block of one row. Passes go round the first MG_CW warps; the rows of
  // ppc consecutive passes form one copy chunk.
  const int rp = 16 / nbx;
  const int npass = (nrows + rp - 1) / rp;
  const int ppc = (npass + MG_GU_CHUNKS - 1) / MG_GU_CHUNKS;
  const int nch = (npass + ppc - 1) / ppc;  // chunks in use
  const int ndown = K * ncols;
  const int lbx = 31 - __clz(nbx);  // log2(nbx)
  const int npub = (ncols + 1) / 2;  // warps that publish columns of the residual stream
  // blocks of h this CTA's rows lie in (at most two: rows_max <= 256 is checked by the host)
  const int hb_lo = R0 >> 8, hb_hi = (R1 - 1) >> 8;
  const int ka0 = R0 / ff;          // expert slot of this CTA's first h row
  const bool has_logit = cta < E;  // E <= G (checked by the host)

  // the gate/up copy job of threads 0..15 (fixed for the whole call; only the expert changes):
  // chunk ch, segment seg (a chunk spans at most 2 experts), gate | up
  int job_k = 0, job_off = 0, job_dst = 0, job_bytes = 0, job_tx = 0;
  if (tid < MG_GU_CHUNKS * 4) {
    const int ch = tid >> 2, seg = (tid >> 1) & 1;
    const int ra = min(R1, R0 + ch * ppc * rp), rb = min(R1, R0 + (ch + 1) * ppc * rp);
    const int ka = ra / ff;
    const int split = min(rb, (ka + 1) * ff);
    const int s0 = seg == 0 ? ra : split, s1 = seg == 0 ? split : rb;
    if ((tid & 3) == 0) job_tx = (rb - ra) * 2 * RBG;
    if (s1 > s0) {
      job_k = s0 / ff;
      job_off = (s0 - job_k * ff) * RBG;
      job_dst = (s0 - R0) * RBG;
      job_bytes = (s1 - s0) * RBG;
    }
  }
  // the down unit of this thread's first round: row i = (slot k, column cc), block b
  const int u0_i = tid / nbh, u0_b = tid - u0_i * nbh, u0_k = u0_i / ncols, u0_cc = u0_i - u0_k * ncols;
  const int dwin0 = (C0 * nbh * 2) & ~15, dwin1 = ((C0 + ncols) * nbh * 2 + 15) & ~15;
  const int dsm_skew = ((C0 * nbh * 2) & 15) / 2;  // halfs to skip inside the 16-byte aligned window

  if (tid == 0) {
    for (int i = 0; i < MG_GU_CHUNKS; i++) mbar_init(&bar_gu[i], 1);
    for (int i = 0; i < PM_MAX_TOPK; i++) mbar_init(&bar_dn[i], 1);
    mbar_init(bar_rw, 1);
    for (int i = 0; i < MG_GU_CHUNKS + PM_MAX_TOPK + 3; i++) armed[i] = 0;  // (and the two counters behind)
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (has_logit && tid == MG_NT - 32) {  // router row of layer 0
    armed[A_RW] = 1;
    mbar_expect_tx(bar_rw, (uint32_t)d * 4);
    bulk_g2s(rw, P.layers[0].router + (size_t)cta * d, (uint32_t)d * 4, bar_rw);
  }

  // layer descriptors are staged in shared memory one layer ahead (their fields
  // would otherwise be L2-latency loads on the critical path)
  MegaLayer *mls = (MegaLayer *)(smem + P.off_ml);
  if (tid < (int)(sizeof(MegaLayer) / 8)) ((unsigned long long *)&mls[0])[tid] = ((const unsigned long long *)&P.layers[0])[tid];

  unsigned long long *trace = nullptr;
  if (TR && P.trace && lane == 0) trace = P.trace + (size_t)cta * P.n_layers * MG_TRACE_PH;
#define MG_TRACE(ph) do { if (TR && trace) trace[(size_t)l * MG_TRACE_PH + (ph)] = now_ns(); } while (0)

  bool dead = false;
  const bool fold = D.weight_fold == PM_FOLD_BEFORE_DOWN;
  float x_own = 0.0f;  // threads 16 cc .. 16 cc + 15: column C0 + cc of the residual stream
  int l = 0;
#pragma unroll 1
  for (; l < P.n_layers; l++) {
    const MegaLayer &ML = mls[l & 1];
    const uint32_t par = l & 1;
    const uint32_t epoch = P.epoch_base + (uint32_t)l + 1u;  // never repeats within 2^32 layers
    if (tid == 0) MG_TRACE(0);
    if (l + 1 < P.n_layers && tid >= 64 && tid < 64 + (int)(sizeof(MegaLayer) / 8))
      ((unsigned long long *)&mls[(l + 1) & 1])[tid - 64] = ((const unsigned long long *)&P.layers[l + 1])[tid - 64];

    // ---- 1. the residual stream ----
    if (l == 0) {
      for (int i = tid; i < d; i += MG_NT) xs[i] = P.x_in[i];
    } else {
      // One thread waits for the layer's arrival counter (148 pollers on one line; when every
      // thread polls its own words, the writes of the later CTAs queue behind the polls of the
      // earlier ones), then every thread reads its four words, both 16-byte loads in flight at
      // once. The counter is bumped without a release; the words carry the epoch themselves.
      if (tid == 0) {
        const unsigned long long want = (P.xcount_base + (unsigned long long)l) * (unsigned long long)G;
        unsigned long long t0 = 0;
        for (uint32_t it = 1;; it++) {
          if (ld_relaxed_u64(P.xcount) >= want) break;
          if ((it & 63) == 0 && wait_expired(t0, P.err, P.wait_ns)) { atomicCAS(P.err, 0, 1); dead = true; break; }
        }
      }
      if (__syncthreads_or(dead)) { dead = true; break; }
      const unsigned long long *src = P.xw + (size_t)par * d;
      for (int i = 4 * tid; i < d; i += 4 * MG_NT) {
        unsigned long long a, b, c, e, t0 = 0;
        for (uint32_t it = 1;; it++) {
          ld_relaxed_2u64(src + i, a, b);
          ld_relaxed_2u64(src + i + 2, c, e);
          if ((uint32_t)(a >> 32) == epoch && (uint32_t)(b >> 32) == epoch && (uint32_t)(c >> 32) == epoch &&
              (uint32_t)(e >> 32) == epoch)
            break;
          if ((it & 63) == 0 && wait_expired(t0, P.err, P.wait_ns)) { atomicCAS(P.err, 0, 1); dead = true; break; }
        }
        *(float4 *)(xs + i) = make_float4(__uint_as_float((uint32_t)a), __uint_as_float((uint32_t)b),
                                          __uint_as_float((uint32_t)c), __uint_as_float((uint32_t)e));
      }
    }
    if (__syncthreads_or(dead)) { dead = true; break; }
    if (tid == 0) MG_TRACE(1);
    if ((tid >> 4) < ncols) x_own = xs[C0 + (tid >> 4)];

    // ---- 2. norm, Q8x of the normed token; 3. logit, all logits, scores ----
    const float inv = pm_rms_inv(xs, d, P.eps, red8);  // (one CTA barrier inside)
    if (warp < nbx) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; j++) v[j] = __fmul_rn(xs[warp * 256 + 32 * j + lane], inv);
      q8x_block_regs(v, lane, xq + warp * 256, xd + warp, xbs + warp * 8, warp & 7, false, false);
    } else if (warp == MG_WARPS - 1) {
      if (has_logit) {
        if (!mbar_wait(bar_rw, par, P.err, P.wait_ns)) dead = true;
        float acc = 0.0f;
#pragma unroll 8
        for (int c = lane; c < d; c += 32) acc = __fmaf_rn(rw[c], __fmul_rn(xs[c], inv), acc);
        float sdot = pm_warp_sum_dot(acc);
        if (lane == 0) {
          if (ML.logit_bias) sdot = __fadd_rn(sdot, ML.logit_bias[cta]);
          st_relaxed_u64(P.lw + (size_t)par * E + cta, tagged(epoch, sdot));
          MG_TRACE(2);
          if (l + 1 < P.n_layers) {  // next layer's row into the same buffer
            armed[A_RW] = 1 + (int)(par ^ 1u);
            mbar_expect_tx(bar_rw, (uint32_t)d * 4);
            bulk_g2s(rw, P.layers[l + 1].router + (size_t)cta * d, (uint32_t)d * 4, bar_rw);
          }
        }
        __syncwarp();
      }
      {
        // every lane polls its own words until all of them carry this layer's epoch
        const unsigned long long *src = P.lw + (size_t)par * E;
        unsigned long long t0 = 0;
        for (uint32_t it = 1;; it++) {
          bool all = true;
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const int e0 = lane + 32 * i;
            if (e0 < E) {
              const unsigned long long w = ld_relaxed_u64(src + e0);
              if ((uint32_t)(w >> 32) == epoch) lg[e0] = __uint_as_float((uint32_t)w);
              else all = false;
            }
          }
          if (__all_sync(PM_FULL, all)) break;
          if ((it & 63) == 0 && __any_sync(PM_FULL, wait_expired(t0, P.err, P.wait_ns))) {
            if (lane == 0) atomicCAS(P.err, 0, 3);
            dead = true;
            break;
          }
        }
      }
      __syncwarp();
      if (lane == 0) MG_TRACE(3);
      if (D.gating == PM_GATE_SOFTMAX_ALL && D.n_group == 0) {
        scores_softmax4(lg, ML.select_bias, E, lane, r_pr, r_key);
      } else {
        float pr[4];
        uint32_t key[4];
        pm_route_scores<4>(D, lg, ML.select_bias, lane, r_sv, r_gs, r_keep, pr, key);
#pragma unroll
        for (int i = 0; i < 4; i++)
          if (lane + 32 * i < E) { r_pr[lane + 32 * i] = pr[i]; r_key[lane + 32 * i] = key[i]; }
      }
      if (lane == 0) MG_TRACE(4);
    }
    if (__syncthreads_or(dead)) { dead = true; break; }
    {
      // rank of expert e = how many experts come before it in (key descending, index
      // ascending) order: exactly the order K rounds of (max, lowest index) pick in. With
      // the index folded into a 64-bit key (key << 32 | ~index) "before" is one compare. A
      // warp ranks 8 experts: every lane holds 4 of the E keys and counts those before e, one
      // warp reduction adds the lanes' counts.
      unsigned long long kk[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int f = lane + 32 * i;
        kk[i] = f < E ? ((unsigned long long)r_key[f] << 32) | (uint32_t)~f : 0ull;
      }
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int e = warp * 8 + j;
        if (e < E) {
          const unsigned long long ke = ((unsigned long long)r_key[e] << 32) | (uint32_t)~e;
          int rank = 0;
#pragma unroll
          for (int i = 0; i < 4; i++) rank += kk[i] > ke;
          rank = __reduce_add_sync(PM_FULL, rank);
          if (lane == 0 && rank < K) { sel_e[rank] = (uint32_t)e; sel_p[rank] = r_pr[e]; }
        }
      }
    }
    if (__syncthreads_or(dead)) { dead = true; break; }
    if (tid == 0) MG_TRACE(5);

    // ---- 4. bulk copies of this CTA's gate/up slice; the weights; the down slices later ----
    if (tid < MG_GU_CHUNKS * 4) {
      if (job_tx) {
        armed[tid >> 2] = 1 + (int)par;
        mbar_expect_tx(&bar_gu[tid >> 2], (uint32_t)job_tx);
      }
      if (job_bytes > 0) {
        const int el = (int)sel_e[job_k];
        const bool isup = tid & 1;
        const uint8_t *src = isup ? ML.up + (size_t)el * ML.up_stride : ML.gate + (size_t)el * ML.gate_stride;
        bulk_g2s((isup ? us : gs) + job_dst, src + job_off, (uint32_t)job_bytes, &bar_gu[tid >> 2]);
      }
    }
    if (warp == MG_WARPS - 1) {
      if (lane < K) wts[lane] = pm_route_weight(D, sel_p, lane);
      __syncwarp();
      asm volatile("bar.arrive 1, %0;" ::"n"(MG_NT) : "memory");  // the weights are there
      if (cta == 0 && lane < K && ML.usage) atomicAdd(&ML.usage[sel_e[lane]], 1u);
      // the down slices: slot k's planes on bar_dn[k]; the first half of the slots once the
      // second gate/up chunk has landed, the rest once the third has (the gate/up bytes are
      // needed first and should not share HBM with bytes needed later, but HBM must not idle)
#pragma unroll 1
      for (int half = 0; half < 2; half++) {
        const int trig = min(MG_DN_TRIG0 + half * (MG_DN_TRIG1 - MG_DN_TRIG0), nch - 1);
        if (!mbar_wait(&bar_gu[trig], par, P.err, P.wait_ns)) dead = true;
        const int k0 = half == 0 ? 0 : (K + 1) / 2, k1 = half == 0 ? (K + 1) / 2 : K;
        const int np = DQ6 ? 4 : 1;
        const int j = lane;  // (at most 8 slots x 4 planes a half)
        if (j < (k1 - k0) * np && !dead) {
          const int k = k0 + j / np, p = j - (j / np) * np;
          const int el = (int)sel_e[k];
          if (DQ6) {
            const int fb = p == 0 ? 128 : p == 1 ? 64 : 16, po = p == 0 ? 0 : p == 1 ? 128 : 192;
            if (p == 0) {
              armed[MG_GU_CHUNKS + k] = 1 + (int)par;
              mbar_expect_tx(&bar_dn[k], (uint32_t)(ncols * nbh * 208 + (dwin1 - dwin0)));
            }
            if (p < 3)
              bulk_g2s(dn + (size_t)k * P.dn_k_bytes + (size_t)P.cols_max * nbh * po,
                       ML.down[p] + (size_t)el * ML.down_stride[p] + (size_t)C0 * nbh * fb, (uint32_t)(ncols * nbh * fb),
                       &bar_dn[k]);
            else
              bulk_g2s(dsm + (size_t)k * P.dsm_k_bytes, ML.down[3] + (size_t)el * ML.down_stride[3] + dwin0,
                       (uint32_t)(dwin1 - dwin0), &bar_dn[k]);
          } else {
            armed[MG_GU_CHUNKS + k] = 1 + (int)par;
            mbar_expect_tx(&bar_dn[k], (uint32_t)(ncols * nbh * 144));
            bulk_g2s(dn + (size_t)k * P.dn_k_bytes, ML.down[0] + (size_t)el * ML.down_stride[0] + (size_t)C0 * nbh * 144,
                     (uint32_t)(ncols * nbh * 144), &bar_dn[k]);
          }
        }
        __syncwarp();
        if (lane == 0 && half == 1) MG_TRACE(15);
      }
    } else {
      // ---- 5. gate/up rows -> h ----
      // lane = (weight row wi of the pass, block b): wi even = gate row, odd = up row of h row wi / 2
      const int b = lane & (nbx - 1), wi = lane >> lbx;
      XBlk X;
      load_xblk(X, xq, xd, xbs, 8, b, b & 7);
      asm volatile("bar.sync 1, %0;" ::"n"(MG_NT) : "memory");  // the weights are there
#pragma unroll 1
      for (int p = warp; p < npass; p += MG_CW) {
        if (!__all_sync(PM_FULL, mbar_wait(&bar_gu[p / ppc], par, P.err, P.wait_ns))) { dead = true; break; }
        if (p == 0 && tid == 0) MG_TRACE(6);
        const int rel = min(p * rp + (wi >> 1), nrows - 1);
        const float term = q4k_block_term(((wi & 1) ? us : gs) + (size_t)rel * RBG + b * 144, X);
        // the row's block terms in block order; all eight shuffles in flight, then the adds
        float tot = 0.0f;
        const int g0 = lane & ~(nbx - 1);
        float tj[8];
#pragma unroll
        for (int j = 0; j < 8; j++) tj[j] = __shfl_sync(PM_FULL, term, g0 + (j & (nbx - 1)));
#pragma unroll
        for (int j = 0; j < 8; j++)
          if (j < nbx) tot = __fadd_rn(tot, tj[j]);
        const int sl = min(lane, rp - 1);
        const float gv = __shfl_sync(PM_FULL, tot, (2 * sl) << lbx);
        const float uv = __shfl_sync(PM_FULL, tot, (2 * sl + 1) << lbx);
        const int r = R0 + p * rp + lane;
        if (lane < rp && r < R1) {
          // (this CTA's rows lie in at most two experts' slots)
          const float hv = pm_act(D.act, D.act_limit, D.act_alpha, gv, uv, wts[ka0 + (r >= (ka0 + 1) * ff)], fold);
          st_relaxed_u64(P.hw + (size_t)par * HR + r, tagged(epoch, hv));
        }
      }
      __syncwarp();
      // the last gate/up warp raises this CTA's flag: its h rows are on their way
      if (lane == 0 && atomicAdd(&s_cnt[0], 1) == MG_CW - 1) {
        s_cnt[0] = 0;
        red_relaxed_add_u64(P.hcount + 16 * hb_lo, 1ull);  // (a counter a 128-byte line)
        if (hb_hi != hb_lo) red_relaxed_add_u64(P.hcount + 16 * hb_hi, 1ull);
        MG_TRACE(12);
      }
      if (tid == 0) MG_TRACE(7);
    }

    // ---- 6. all of h, re-quantised: a warp collects the (one or two) blocks it quantises ----
    {
      const unsigned long long *src = P.hw + (size_t)par * HR;
      const uint32_t want = epoch;
      const int nblk = K * nbh;
#pragma unroll 1
      for (int b0 = warp; b0 < nblk && !dead; b0 += 2 * MG_WARPS) {
        const int b1 = b0 + MG_WARPS < nblk ? b0 + MG_WARPS : b0;  // (b1 == b0: a single block)
        unsigned long long t0 = 0;
        // the blocks' arrival counters first (one word a block, bumped once per layer by each CTA
        // that produces rows of it; lanes 0 and 1 poll): polling the data words themselves, from
        // every warp of every CTA while the weights still stream, takes the L2 bandwidth the
        // stream needs
        {
          const int blk = lane == 0 ? b0 : b1;
          // CTA i owns rows [HR i / G, HR (i + 1) / G) (integer divisions): the owners of the block's
          // first and last row, and every CTA between them, bump its counter
          auto owner = [&](int r) {
            int i = (int)(((long long)r * G) / HR);
            if ((int)(((long long)HR * (i + 1)) / G) <= r) i++;
            return i;
          };
          const int i_lo = owner(256 * blk), i_hi = owner(256 * blk + 255);
          const unsigned long long wantc = (P.count_base + (unsigned long long)l + 1ull + (l == 0 ? (unsigned long long)P.fault : 0ull)) *
                                           (unsigned long long)(i_hi - i_lo + 1);
          for (uint32_t it = 1;; it++) {
            const bool ok = lane >= 2 || ld_relaxed_u64(P.hcount + 16 * blk) >= wantc;
            if (__all_sync(PM_FULL, ok)) break;
            if ((it & 63) == 0 && __any_sync(PM_FULL, wait_expired(t0, P.err, P.wait_ns))) {
              if (lane == 0) atomicCAS(P.err, 0, 4);
              dead = true;
              break;
            }
          }
        }
        if (dead) break;
        if (b0 == 0 && lane == 0) MG_TRACE(13);
        // the words themselves, all sixteen loads in flight; they carry the epoch too, so a
        // flag seen ahead of its data only costs another round
        float v0[8], v1[8];
        for (uint32_t it = 1;; it++) {
          bool all = true;
          unsigned long long w0[8], w1[8];
#pragma unroll
          for (int j = 0; j < 8; j++) w0[j] = ld_relaxed_u64(src + b0 * 256 + 32 * j + lane);
#pragma unroll
          for (int j = 0; j < 8; j++) w1[j] = ld_relaxed_u64(src + b1 * 256 + 32 * j + lane);
#pragma unroll
          for (int j = 0; j < 8; j++) {
            if ((uint32_t)(w0[j] >> 32) != want || (uint32_t)(w1[j] >> 32) != want) all = false;
            v0[j] = __uint_as_float((uint32_t)w0[j]);
            v1[j] = __uint_as_float((uint32_t)w1[j]);
          }
          if (__all_sync(PM_FULL, all)) break;
          if ((it & 31) == 0 && __any_sync(PM_FULL, wait_expired(t0, P.err, P.wait_ns))) {
            if (lane == 0) atomicCAS(P.err, 0, 4);
            dead = true;
            break;
          }
        }
        if (b0 == 0 && lane == 0) MG_TRACE(14);
        q8x_block_regs(v0, lane, hq + b0 * 256, hd + b0, hbs + b0 * 16, 0, DQ6, DQ6);
        if (b1 != b0) q8x_block_regs(v1, lane, hq + b1 * 256, hd + b1, hbs + b1 * 16, 0, DQ6, DQ6);
      }
    }
    if (tid == 0) MG_TRACE(8);
    if (__syncthreads_or(dead)) { dead = true; break; }
    if (tid == 0) MG_TRACE(9);

    // ---- 7. down rows of this CTA's columns, all k: one (row, block) unit per lane ----
#pragma unroll 1
    for (int u = tid; u < ndown * nbh; u += MG_NT) {
      int b = u0_b, k = u0_k, cc = u0_cc;
      if (u != tid) {  // (further rounds: shapes with more than MG_NT units)
        const int i = u / nbh;
        b = u - i * nbh;
        k = i / ncols;
        cc = i - k * ncols;
      }
      if (!mbar_wait(&bar_dn[k], par, P.err, P.wait_ns)) { dead = true; break; }
      if (DQ6) {
        // 256 six-bit values against the block of h, no cross-lane traffic.
        // isum = sum_c sc[c] * (q_c . h_c - 32 * sum(h_c)) over the 16 chunks c of 16 values
        // (the integer sum of `row_q6k_q8x`, regrouped). Lanes walk the 16-byte pieces in a
        // rotated order so that units 128 bytes apart hit different banks.
        const int8_t *xb = hq + k * ff + b * 256;
        const size_t cm = (size_t)P.cols_max * nbh;
        const uint8_t *base = dn + (size_t)k * P.dn_k_bytes;
        const size_t rb = (size_t)cc * nbh + b;
        const uint8_t *qlp = base + rb * 128, *qhp = base + cm * 128 + rb * 64;
        const int8_t *scp = (const int8_t *)(base + cm * 192 + rb * 16);
        const int32_t *hs = hbs + (k * nbh + b) * 16;
        int isum = 0;
        // piece order per lane: a rotation of a permutation (bits 0 and 1 of the lane
        // swapped) under which lanes 128 bytes apart in the 64-byte-a-unit qh plane, i.e.
        // lanes of equal parity, take four different qh pieces
        const int pl = (lane & 4) | ((lane & 1) << 1) | ((lane >> 1) & 1);
#pragma unroll
        for (int p = 0; p < 8; p++) {
          const int pp = (p + pl) & 7, n = pp >> 2, jj = (pp >> 1) & 1, g = pp & 1;
          const uint4 qlv = *(const uint4 *)(qlp + pp * 16);
          const uint4 qhv = *(const uint4 *)(qhp + (2 * n + g) * 16);
          const int clo = 8 * n + 2 * jj + g, chi = clo + 4;  // chunks of the low / high nibbles
          // h's chunks 8-15 are stored with their halves swapped (`fold8`)
          const int4 xlo = *(const int4 *)(xb + (clo + 4 * n) * 16), xhi = *(const int4 *)(xb + (chi - 4 * n) * 16);
          const int sh = 2 * jj;
          const uint32_t qlw[4] = {qlv.x, qlv.y, qlv.z, qlv.w}, qhw[4] = {qhv.x, qhv.y, qhv.z, qhv.w};
          const int xl[4] = {xlo.x, xlo.y, xlo.z, xlo.w}, xh[4] = {xhi.x, xhi.y, xhi.z, xhi.w};
          int dlo = 0, dhi = 0;  // q . h of the two chunks
#pragma unroll
          for (int w = 0; w < 4; w++) {
            const uint32_t qa = (qlw[w] & 0x0f0f0f0fu) | (((qhw[w] >> sh) & 0x03030303u) << 4);
            const uint32_t qb = ((qlw[w] >> 4) & 0x0f0f0f0fu) | (((qhw[w] >> (sh + 4)) & 0x03030303u) << 4);
            dlo = __dp4a((int)qa, xl[w], dlo);
            dhi = __dp4a((int)qb, xh[w], dhi);
          }
          isum += (int)scp[clo] * (dlo - 32 * hs[clo]) + (int)scp[chi] * (dhi - 32 * hs[chi]);
        }
        const float dd = __half2float(((const __half *)(dsm + (size_t)k * P.dsm_k_bytes))[dsm_skew + cc * nbh + b]);
        tmp[u] = __fmul_rn(hd[k * nbh + b], __fmul_rn(dd, (float)isum));
      } else {
        XBlk X;
        load_xblk(X, hq + k * ff, hd + k * nbh, hbs + k * nbh * 16, 16, b, 0);
        tmp[u] = q4k_block_term(dn + (size_t)k * P.dn_k_bytes + ((size_t)cc * nbh + b) * 144, X);
      }
    }
    if (__syncthreads_or(dead)) { dead = true; break; }
    if (tid == 0) MG_TRACE(10);
    // a row's terms in block order, the rows in k order, then the residual
    // (16 lanes a column: lane k sums row (k, column)'s terms, lane 0 of the 16 adds them in k order)
    if (2 * warp < ncols) {  // (whole warps: the shuffles below name every lane)
      const int cc = tid >> 4, k = tid & 15;
      float total = 0.0f;
      if (k < K && cc < ncols) {
        for (int b = 0; b < nbh; b++) total = __fadd_rn(total, tmp[(k * ncols + cc) * nbh + b]);
        if (!fold) total = __fmul_rn(wts[k], total);
      }
      float s = 0.0f;
      float tj[PM_MAX_TOPK];  // (all shuffles in flight before the ordered adds)
#pragma unroll
      for (int j = 0; j < PM_MAX_TOPK; j++) tj[j] = __shfl_sync(PM_FULL, total, (lane & 16) + j);
#pragma unroll
      for (int j = 0; j < PM_MAX_TOPK; j++)
        if (j < K) s = __fadd_rn(s, tj[j]);
      if (k == 0 && cc < ncols) {
        const float xn = __fadd_rn(x_own, s);
        if (l + 1 < P.n_layers) st_relaxed_u64(P.xw + (size_t)(par ^ 1u) * d + C0 + cc, tagged(epoch + 1u, xn));
        else P.x_out[C0 + cc] = xn;
      }
      __syncwarp();
      // the last publishing warp of this CTA bumps the next layer's arrival counter
      if (lane == 0 && l + 1 < P.n_layers && atomicAdd(&s_cnt[1], 1) == npub - 1) {
        s_cnt[1] = 0;
        red_relaxed_add_u64(P.xcount, 1ull);
      }
    }
    if (tid == 0) MG_TRACE(11);
    // (no barrier here: the next layer's first steps write xs and red8 only, which nothing
    // above reads any more; tmp, wts and sel_* are rewritten behind two more CTA barriers)
  }

  if (dead) {
    // give this CTA's own copies a bounded time to land before its shared memory goes away
    __syncthreads();
    if (tid == 0) {
      const unsigned long long t0 = now_ns();
      for (int i = 0; i < MG_GU_CHUNKS + PM_MAX_TOPK + 1; i++)
        if (armed[i])
          while (!mbar_try_wait_ns(&bar_gu[i], (uint32_t)(armed[i] - 1), 2000u) && now_ns() - t0 < P.wait_ns) {}
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
  // one logit a CTA, four ranking threads an expert
  if (D.n_exp > n_sm || D.n_exp > 128 || D.top_k > PM_MAX_TOPK) return false;
  const int d = D.d, ff = D.ff, K = D.top_k;
  const int nbx = d / 256, nbh = ff / 256;
  if (nbx != 1 && nbx != 2 && nbx != 4 && nbx != 8) return false;  // a lane = one block of a row, 32 / nbx rows a warp pass
  int G = n_sm;
  long long HR = (long long)K * ff;
  int rows_max = (int)((HR + G - 1) / G) + 1, cols_max = (d + G - 1) / G + 1;
  if (HR < G || d < G) return false;
  if (cols_max * 16 > MG_NT) return false;  // 16 lanes a column in the final sum
  if (rows_max > ff || rows_max > 256) return false;  // a CTA's rows span at most two experts and two blocks of h
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
  P.off_hbs = take((uint32_t)K * nbh * 16 * 4);
  P.off_rw = take((uint32_t)d * 4);
  P.off_tmp = take((uint32_t)K * cols_max * nbh * 4);
  P.off_lg = take((uint32_t)D.n_exp * 4);
  P.off_ml = take(2 * (uint32_t)sizeof(MegaLayer));
  P.off_misc = take(8 * (MG_GU_CHUNKS + PM_MAX_TOPK + 1) + 8 * 4 + PM_MAX_TOPK * 12 +
                    4 * (MG_GU_CHUNKS + PM_MAX_TOPK + 4) + 128 * 12 + 64 * 4 + 64 + 64);
  mp.smem = off;
  if (mp.smem > smem_optin) return false;
  mp.grid = G;
  mp.ok = true;
  return true;
}

typedef void (*MegaKernel)(const MegaParams);
static MegaKernel mega_kernel(const pm_layer_desc &D, bool trace) {
  if (trace) return D.type_down == PM_TYPE_Q6_K ? k_decode_mega<true, true> : k_decode_mega<false, true>;
  return D.type_down == PM_TYPE_Q6_K ? k_decode_mega<true, false> : k_decode_mega<false, false>;
}

cudaError_t mega_prepare(const pm_layer_desc &D, size_t smem) {
  cudaError_t e = cudaFuncSetAttribute((const void *)mega_kernel(D, false), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute((const void *)mega_kernel(D, true), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

int mega_max_ctas_per_sm(const pm_layer_desc &D, size_t smem) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, (const void *)mega_kernel(D, false), MG_NT, smem) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

cudaError_t mega_launch(const MegaPlan &mp, cudaStream_t stream) {
  MegaParams P = mp.P;
  void *args[] = {(void *)&P};
  return cudaLaunchCooperativeKernel((const void *)mega_kernel(P.D, P.trace != nullptr), dim3(mp.grid), dim3(MG_NT), args, mp.smem, stream);
}
