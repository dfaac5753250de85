// prefill_tc.cu - grouped expert products for many tokens per expert on the 5th-gen
// tensor cores (tcgen05.mma kind::i8, accumulators in TMEM), exact in the integer
// domain of the reference's CPU path (src/ds4_cpu.rs:59-83).
//
// One CTA = (128 weight rows of one active expert) x (up to 128 of its tokens).
// Per 256-value block b of the rows:
//   1. CUDA cores unpack the Q4_K block into THREE int8 operand planes in shared
//      memory (K-major, no swizzle, 8x16-byte core matrices):
//        A_hi = nibble * (sc >> 3), A_lo = nibble * (sc & 7), A_m = m (per sub-block)
//      so that with the token's int8 activations xq as the other operand
//        isum = 8 * (A_hi . xq) + (A_lo . xq) = sum_j sc_j * sum_i nib_ji * xq_ji
//        msum = A_m . xq                     = sum_j m_j * bsum_j
//      are the reference's exact integer sums (6-bit scales do not fit one int8
//      product with a nibble; two 3-bit halves do).
//   2. one thread issues 24 tcgen05.mma (8 K-steps of 32 x 3 planes) into three TMEM
//      accumulators and commits to an mbarrier;
//   3. every warp reads its TMEM lanes (tcgen05.ld) and adds the block's float term
//      total += x.d[b] * (d * isum - dmin * msum) in block order, as `row_scalar`.
// Gate and up rows share a CTA (64 + 64 rows) so SwiGLU is fused in the epilogue;
// down rows write the pair outputs. Waits are time-bounded; TMEM is freed on
// every exit path.
#include "moe_internal.cuh"

#define TC_NT 256
#define TC_M 128
#define TC_NMAX 128
#define TC_WAIT_NS 2000000000ull

__device__ __forceinline__ uint32_t tc_s32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ unsigned long long tc_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// shared-memory matrix descriptor, K-major, no swizzle: 8x16 B core matrices,
// lbo = bytes between the two 16-byte K chunks of one MMA, sbo = bytes between
// 8-row groups
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)((lbo >> 4) & 0x3fff) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3fff) << 32) | (1ull << 46);
}
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_c, uint64_t da, uint64_t db, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n" ::"r"(tmem_c),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   tc_s32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t r[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ bool tc_bar_test(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      " selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(tc_s32(bar)), "r"(parity), "r"(20000u)
      : "memory");
  return ok != 0;
}
__device__ __noinline__ bool tc_bar_wait(uint64_t *bar, uint32_t parity, int *err) {
  unsigned long long t0 = tc_now();
  for (uint32_t it = 0;; it++) {
    if (tc_bar_test(bar, parity)) return true;
    if ((it & 15) == 15 && tc_now() - t0 > TC_WAIT_NS) break;
  }
  atomicCAS(err, 0, 7);
  return false;
}

int tc_max_tiles(int n_pairs, int max_groups);

struct TcArgs {
  LayerDev ly;
  int shared;      // 1: the shared expert's matrices (one group over all tokens)
  int down;        // 0: gate+up with activation -> h; 1: down -> pair outputs
  Groups g;
  const int8_t *xq;      // gate/up: [T][d] by token; down: [P][ff] by pair
  const float *xd;       // per row of xq: [cols/256]
  const float *wts;      // routing weights [T*K] (gate/up with fold) or null
  float *out;            // gate/up: h [P][ff]; down: eo [P][d]
  int *err;
  const int *n_tiles;          // [1]
  const uint32_t *tile_group;  // [tiles] index into the groups
  const uint32_t *tile_n0;     // [tiles] first token of the tile inside its group
};

// The (group, token tile) list of a grouping: group a contributes ceil(count/128)
// tiles. One CTA; groups <= 512 (experts of a layer, or the one shared-expert group
// whose count may be the whole batch).
__global__ void __launch_bounds__(512) k_tc_tiles(Groups g, int *n_tiles, uint32_t *tile_group,
                                                  uint32_t *tile_n0, int max_tiles) {
  __shared__ uint32_t s[512];
  const int a = threadIdx.x;
  const int ng = min(*g.n_groups, 512);
  uint32_t tc = a < ng ? (g.count[a] + TC_NMAX - 1) / TC_NMAX : 0;
  s[a] = tc;
  __syncthreads();
  for (int off = 1; off < 512; off <<= 1) {
    uint32_t v = a >= off ? s[a - off] : 0;
    __syncthreads();
    s[a] += v;
    __syncthreads();
  }
  uint32_t first = s[a] - tc;
  for (uint32_t i = 0; i < tc && (int)(first + i) < max_tiles; i++) {
    tile_group[first + i] = (uint32_t)a;
    tile_n0[first + i] = i * TC_NMAX;
  }
  if (a == 511) *n_tiles = min((int)s[511], max_tiles);
}

// WT: the weight type of the product's matrices (PM_TYPE_Q4_K: planes hi, lo, m;
// PM_TYPE_Q6_K: four base-4 digit planes of the int8 sub-scale, see below)
template <int WT>
__global__ void __launch_bounds__(TC_NT, 1) k_tc(const TcArgs A) {
  constexpr int NP = WT == PM_TYPE_Q6_K ? 4 : 3;  // operand planes = TMEM accumulators
  extern __shared__ __align__(128) uint8_t smem[];
  // blockIdx.y walks the list of (group, 128-token tile) pairs made by k_tc_tiles
  if ((int)blockIdx.y >= *A.n_tiles) return;
  const int a = (int)A.tile_group[blockIdx.y];
  const LayerDev &ly = A.ly;
  const WMat &W0 = A.down ? (A.shared ? ly.sdown : ly.down) : (A.shared ? ly.sgate : ly.gate);
  const WMat &W1 = A.shared ? ly.sup : ly.up;  // used by gate/up only
  const int cols = W0.cols, nb = cols / 256, rows = W0.rows;
  const int e = (int)A.g.expert[a];
  const int el = A.shared ? 0 : e - ly.first_local;
  const uint32_t off = A.g.offset[a], cnt = A.g.count[a];
  const int n0 = (int)A.tile_n0[blockIdx.y];
  const int nvalid = min((int)cnt - n0, TC_NMAX);
  const int npad = (nvalid + 15) & ~15;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool local = el >= 0 && el < (A.shared ? 1 : ly.n_local);
  const int rows_per_cta = A.down ? TC_M : TC_M / 2;  // gate/up: 64 gate + 64 up rows
  const int r0 = blockIdx.x * rows_per_cta;
  if (!local) {  // an expert another rank holds: zeros (down) / nothing to do (gate/up)
    if (A.down)
      for (int i = tid; i < nvalid * TC_M; i += TC_NT) {
        int n = i / TC_M, m = i % TC_M;
        if (r0 + m < rows) A.out[(size_t)(off + n0 + n) * rows + r0 + m] = 0.0f;
      }
    return;
  }

  // shared memory: three A planes (hi, lo, m), B, per-row scales, per-token scales
  uint8_t *sA = smem;                                   // 3 x [16 chunks][128 rows][16 B]
  uint8_t *sB = smem + NP * 32768;                      // [16 chunks][npad rows][16 B]
  float2 *sDm = (float2 *)(sB + 16 * TC_NMAX * 16);     // [128] (d, dmin) of the block
  float *sXd = (float *)(sDm + TC_M);                   // [128] x.d of the block per token
  uint64_t *bar = (uint64_t *)(sXd + TC_NMAX);
  uint32_t *tmem_slot = (uint32_t *)(bar + 1);
  int *s_tok = (int *)(tmem_slot + 2);                  // [128] row of xq per token of the tile

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     tc_s32(tmem_slot)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tc_s32(bar)), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int n = tid; n < TC_NMAX; n += TC_NT) {
    int row = -1;
    if (n < nvalid) row = A.down ? (int)(off + n0 + n) : (int)A.g.pair_token[off + n0 + n];
    s_tok[n] = row;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  // instruction descriptor: D s32, A unsigned 8-bit, B signed 8-bit, both K-major
  const uint32_t idesc = (2u << 4) | ((WT == PM_TYPE_Q6_K ? 1u : 0u) << 7) | (1u << 10) | ((uint32_t)(npad >> 3) << 17) |
                         ((uint32_t)(TC_M >> 4) << 24);
  // this thread: one weight row, one half of the block
  const int m = tid & 127, hf = tid >> 7;  // a warp = 32 consecutive rows, one half: conflict-free 16-byte stores
  const uint8_t *rowp = nullptr, *rp_qh = nullptr, *rp_sc = nullptr, *rp_d = nullptr;
  {
    int r;
    const WMat *W;
    if (A.down) { r = r0 + m; W = &W0; }
    else if (m < 64) { r = r0 + m; W = &W0; }
    else { r = r0 + m - 64; W = &W1; }
    if (r < rows) {
      if (WT == PM_TYPE_Q6_K) {
        size_t rb = (size_t)r * nb;
        rowp = W->plane[0] + (size_t)el * W->stride[0] + rb * 128;
        rp_qh = W->plane[1] + (size_t)el * W->stride[1] + rb * 64;
        rp_sc = W->plane[2] + (size_t)el * W->stride[2] + rb * 16;
        rp_d = W->plane[3] + (size_t)el * W->stride[3] + rb * 2;
      } else {
        rowp = W->plane[0] + (size_t)el * W->stride[0] + (size_t)r * nb * 144;
      }
    }
  }
  // epilogue role: TMEM lanes of this warp's quarter, half of the token columns
  const int q = warp & 3, ch = warp >> 2;
  const int erow = 32 * q + lane;                 // row of the tile this thread accumulates
  const int ecol0 = ch * (TC_NMAX / 2);           // its 64 token columns
  float total[TC_NMAX / 2];
#pragma unroll
  for (int i = 0; i < TC_NMAX / 2; i++) total[i] = 0.0f;

  // raw bytes of one block, one step ahead, in registers:
  //   Q4_K: pf[0] header, pf[1..4] this thread's 64 quant bytes
  //   Q6_K: pf[0..3] ql (64 B), pf[4..5] qh (32 B), pf[6] = (8 scales, f16 d)
  //   pfb[0..7]: this thread's 16-byte pieces of the tokens' activations, pfx: a token's x.d
  uint4 pf[7], pfb[8];
  float pfx = 0.0f;
  auto load_raw = [&](int bb) {
    if (bb >= nb) return;
    if (rowp) {
      if (WT == PM_TYPE_Q6_K) {
        const uint8_t *ql = rowp + (size_t)bb * 128 + 64 * hf;
        const uint8_t *qh = rp_qh + (size_t)bb * 64 + 32 * hf;
#pragma unroll
        for (int j = 0; j < 4; j++) pf[j] = __ldg((const uint4 *)(ql + 16 * j));
        pf[4] = __ldg((const uint4 *)qh);
        pf[5] = __ldg((const uint4 *)(qh + 16));
        uint2 scw = __ldg((const uint2 *)(rp_sc + (size_t)bb * 16 + 8 * hf));
        pf[6] = make_uint4(scw.x, scw.y, (uint32_t)__ldg((const uint16_t *)(rp_d + (size_t)bb * 2)), 0);
      } else {
        const uint8_t *blk = rowp + (size_t)bb * 144;
        pf[0] = __ldg((const uint4 *)blk);
#pragma unroll
        for (int j = 0; j < 4; j++) pf[1 + j] = __ldg((const uint4 *)(blk + 16 + 64 * hf + 16 * j));
      }
    }
    {
      const int row = (tid & 127) < npad ? s_tok[tid & 127] : -1;
      const int8_t *src = A.xq + (size_t)(row < 0 ? 0 : row) * cols + (size_t)bb * 256 + (tid >> 7) * 16;
#pragma unroll
      for (int j = 0; j < 8; j++) pfb[j] = row >= 0 ? *(const uint4 *)(src + 32 * j) : make_uint4(0, 0, 0, 0);
    }
    if (tid < TC_NMAX) {
      int row = s_tok[tid];
      pfx = row >= 0 ? A.xd[(size_t)row * nb + bb] : 0.0f;
    }
  };
  load_raw(0);

  bool dead = false;
  for (int b = 0; b < nb; b++) {
    // ---- 1. operands of block b into shared memory ----
    if (rowp && WT == PM_TYPE_Q6_K) {
      // Q6_K: value = sc * (q - 32), sc int8 per 16 values (one K chunk), q 6 bits.
      // sc = 64*a3 + 16*a2 + 4*a1 + a0 with a0..a2 in 0..3 and a3 in -2..1, so each
      // plane (q-32)*a_i fits int8 and isum = I0 + 4*I1 + 16*I2 + 64*I3 exactly.
      const uint4 qlv[4] = {pf[0], pf[1], pf[2], pf[3]};
      const uint4 qhv[2] = {pf[4], pf[5]};
      const uint2 scw = make_uint2(pf[6].x, pf[6].y);
      if (hf == 0) sDm[m] = make_float2(pm_f16(pf[6].z), 0.0f);
#pragma unroll
      for (int qt = 0; qt < 4; qt++) {
#pragma unroll
        for (int lh = 0; lh < 2; lh++) {
          const uint4 qlw = qlv[2 * (qt & 1) + lh];
          const uint4 qhw = qhv[lh];
          const int si = 2 * qt + lh;
          const int sv = (int)(int8_t)((si < 4 ? scw.x >> (8 * si) : scw.y >> (8 * (si - 4))) & 0xff);
          const uint32_t dg[4] = {(uint32_t)sv & 3u, ((uint32_t)sv >> 2) & 3u, ((uint32_t)sv >> 4) & 3u,
                                  (uint32_t)(sv >> 6 < 0 ? -(sv >> 6) : (sv >> 6))};
          const bool neg3 = (sv >> 6) < 0;
          const uint32_t ws[4] = {qlw.x, qlw.y, qlw.z, qlw.w}, hs[4] = {qhw.x, qhw.y, qhw.z, qhw.w};
          uint32_t o[4][4];
#pragma unroll
          for (int i = 0; i < 4; i++) {
            uint32_t qv = ((ws[i] >> (qt >= 2 ? 4 : 0)) & 0x0f0f0f0fu) | (((hs[i] >> (2 * qt)) & 0x03030303u) << 4);
#pragma unroll
            for (int pp = 0; pp < 4; pp++) {
              uint32_t v = __vsub4(qv * dg[pp], 0x20202020u * dg[pp]);  // (q - 32) * digit per byte
              if (pp == 3 && neg3) v = __vneg4(v);
              o[pp][i] = v;
            }
          }
          size_t off_c = (size_t)(8 * hf + 2 * qt + lh) * (TC_M * 16) + (size_t)m * 16;
#pragma unroll
          for (int pp = 0; pp < 4; pp++)
            *(uint4 *)(sA + (size_t)pp * 32768 + off_c) = make_uint4(o[pp][0], o[pp][1], o[pp][2], o[pp][3]);
        }
      }
    } else if (rowp) {
      const uint4 hdr = pf[0];
      if (hf == 0) sDm[m] = make_float2(pm_f16(hdr.x), pm_f16(hdr.x >> 16));
#pragma unroll
      for (int cc = 0; cc < 2; cc++) {
        int c = 2 * hf + cc;
        const uint4 w0 = pf[1 + 2 * cc], w1 = pf[2 + 2 * cc];
        int sc0, m0, sc1, m1;
        pm_q4k_scmin(hdr.y, hdr.z, hdr.w, 2 * c, sc0, m0);
        pm_q4k_scmin(hdr.y, hdr.z, hdr.w, 2 * c + 1, sc1, m1);
        const uint32_t M4 = 0x0f0f0f0fu;
        // sub-block 2c = low nibbles -> K chunks 4c, 4c+1 ; sub-block 2c+1 = high -> 4c+2, 4c+3
        uint32_t lo[8] = {w0.x & M4, w0.y & M4, w0.z & M4, w0.w & M4, w1.x & M4, w1.y & M4, w1.z & M4, w1.w & M4};
        uint32_t hi[8] = {(w0.x >> 4) & M4, (w0.y >> 4) & M4, (w0.z >> 4) & M4, (w0.w >> 4) & M4,
                          (w1.x >> 4) & M4, (w1.y >> 4) & M4, (w1.z >> 4) & M4, (w1.w >> 4) & M4};
        uint32_t sh0 = (uint32_t)sc0 >> 3, sl0 = (uint32_t)sc0 & 7, sh1 = (uint32_t)sc1 >> 3, sl1 = (uint32_t)sc1 & 7;
        uint32_t mm0 = (uint32_t)m0 * 0x01010101u, mm1 = (uint32_t)m1 * 0x01010101u;
#pragma unroll
        for (int h2 = 0; h2 < 2; h2++) {
          size_t o_lo = (size_t)(4 * c + h2) * (TC_M * 16) + (size_t)m * 16;      // chunk of sub-block 2c
          size_t o_hi = (size_t)(4 * c + 2 + h2) * (TC_M * 16) + (size_t)m * 16;  // chunk of sub-block 2c+1
          const uint32_t *l4 = lo + 4 * h2, *h4 = hi + 4 * h2;
          *(uint4 *)(sA + o_lo) = make_uint4(l4[0] * sh0, l4[1] * sh0, l4[2] * sh0, l4[3] * sh0);
          *(uint4 *)(sA + 32768 + o_lo) = make_uint4(l4[0] * sl0, l4[1] * sl0, l4[2] * sl0, l4[3] * sl0);
          *(uint4 *)(sA + 65536 + o_lo) = make_uint4(mm0, mm0, mm0, mm0);
          *(uint4 *)(sA + o_hi) = make_uint4(h4[0] * sh1, h4[1] * sh1, h4[2] * sh1, h4[3] * sh1);
          *(uint4 *)(sA + 32768 + o_hi) = make_uint4(h4[0] * sl1, h4[1] * sl1, h4[2] * sl1, h4[3] * sl1);
          *(uint4 *)(sA + 65536 + o_hi) = make_uint4(mm1, mm1, mm1, mm1);
        }
      }
    } else {  // rows past the matrix: zero operands
      if (hf == 0) sDm[m] = make_float2(0.0f, 0.0f);
      for (int kc = 8 * hf; kc < 8 * hf + 8; kc++) {
        size_t o = (size_t)kc * (TC_M * 16) + (size_t)m * 16;
#pragma unroll
        for (int pp = 0; pp < NP; pp++) *(uint4 *)(sA + (size_t)pp * 32768 + o) = make_uint4(0, 0, 0, 0);
      }
    }
    if ((tid & 127) < npad) {  // thread = (token row tid & 127, chunks tid >> 7, +2, ...)
#pragma unroll
      for (int j = 0; j < 8; j++)
        *(uint4 *)(sB + (size_t)((tid >> 7) + 2 * j) * (npad * 16) + (size_t)(tid & 127) * 16) = pfb[j];
    }
    if (tid < TC_NMAX) sXd[tid] = pfx;
    // the next block's bytes start their trip from HBM now, and land while this
    // block is multiplied and folded
    load_raw(b + 1);
    // generic-proxy writes -> visible to the tensor core's (async proxy) reads
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // ---- 2. 8 K-steps x 3 planes ----
    if (tid == 0) {
      const uint32_t a0 = tc_s32(sA), b0 = tc_s32(sB);
#pragma unroll 1
      for (int ks = 0; ks < 8; ks++) {
        uint64_t db = tc_desc(b0 + (uint32_t)ks * 2u * (uint32_t)npad * 16u, (uint32_t)npad * 16u, 128u);
#pragma unroll
        for (int p = 0; p < NP; p++) {
          uint64_t da = tc_desc(a0 + (uint32_t)p * 32768u + (uint32_t)ks * 2u * (TC_M * 16u), TC_M * 16u, 128u);
          tc_mma_i8(tmem + (uint32_t)p * TC_NMAX, da, db, idesc, ks > 0 ? 1u : 0u);
        }
      }
      tc_commit(bar);
    }
    // ---- 3. the block's float term, in block order ----
    if (!tc_bar_test(bar, (uint32_t)(b & 1)) && !tc_bar_wait(bar, (uint32_t)(b & 1), A.err)) dead = true;
    if (__syncthreads_or(dead)) { dead = true; break; }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    {
      const float2 dm = sDm[erow];
      const uint32_t tl = tmem + ((uint32_t)(32 * q) << 16);
#pragma unroll
      for (int c32 = 0; c32 < TC_NMAX / 2; c32 += 32) {
        if (ecol0 + c32 < npad) {
          uint32_t vh[32], vl[32], vm[32];
          tc_ld32(tl + (uint32_t)(0 * TC_NMAX + ecol0 + c32), vh);
          tc_ld32(tl + (uint32_t)(1 * TC_NMAX + ecol0 + c32), vl);
          tc_ld32(tl + (uint32_t)(2 * TC_NMAX + ecol0 + c32), vm);
          if (WT == PM_TYPE_Q6_K) {
            uint32_t v3[32];
            tc_ld32(tl + (uint32_t)(3 * TC_NMAX + ecol0 + c32), v3);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 32; i++) {
              int isum = (int)vh[i] + 4 * (int)vl[i] + 16 * (int)vm[i] + 64 * (int)v3[i];
              float term = __fmul_rn(sXd[ecol0 + c32 + i], __fmul_rn(dm.x, (float)isum));
              total[c32 + i] = __fadd_rn(total[c32 + i], term);
            }
          } else {
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 32; i++) {
              int isum = 8 * (int)vh[i] + (int)vl[i];
              int msum = (int)vm[i];
              float term = __fmul_rn(sXd[ecol0 + c32 + i],
                                     __fsub_rn(__fmul_rn(dm.x, (float)isum), __fmul_rn(dm.y, (float)msum)));
              total[c32 + i] = __fadd_rn(total[c32 + i], term);
            }
          }
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();  // operands and accumulators are rewritten by the next block
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }

  if (!dead) {
    if (A.down) {
      const float bd = (!A.shared && ly.bias_down && r0 + erow < rows) ? ly.bias_down[(size_t)el * rows + r0 + erow] : 0.0f;
#pragma unroll
      for (int i = 0; i < TC_NMAX / 2; i++) {
        int n = ecol0 + i;
        if (n < nvalid && r0 + erow < rows) {
          float o = total[i];
          if (!A.shared && ly.bias_down) o = __fadd_rn(o, bd);
          A.out[(size_t)(off + n0 + n) * rows + r0 + erow] = o;
        }
      }
    } else {
      // gate rows in tile rows 0..63, up rows in 64..127: exchange through shared memory
      float *S = (float *)sA;  // [128][129]
#pragma unroll
      for (int i = 0; i < TC_NMAX / 2; i++) S[erow * (TC_NMAX + 1) + ecol0 + i] = total[i];
      __syncthreads();
      const pm_layer_desc &D = ly.desc;
      const bool fold = !A.shared && D.weight_fold == PM_FOLD_BEFORE_DOWN && A.wts;
      const bool bias = !A.shared && ly.bias_gate;
      for (int i = tid; i < nvalid * 64; i += TC_NT) {
        int j = i & 63, n = i >> 6;
        if (r0 + j >= rows) continue;
        float gv = S[j * (TC_NMAX + 1) + n], uv = S[(64 + j) * (TC_NMAX + 1) + n];
        if (bias) {
          gv = __fadd_rn(gv, ly.bias_gate[(size_t)el * rows + r0 + j]);
          uv = __fadd_rn(uv, ly.bias_up[(size_t)el * rows + r0 + j]);
        }
        uint32_t p = off + n0 + n;
        float w = fold ? A.wts[A.g.pair_src[p]] : 1.0f;
        A.out[(size_t)p * rows + r0 + j] = pm_act(D.act, D.act_limit, D.act_alpha, gv, uv, w, fold);
      }
    }
  }
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

int tc_max_tiles(int n_pairs, int max_groups) {
  int groups = max_groups < n_pairs ? max_groups : n_pairs;
  return n_pairs / TC_NMAX + groups;
}
static size_t tc_smem(int planes) {
  return (size_t)planes * 32768 + 16 * TC_NMAX * 16 + TC_M * 8 + TC_NMAX * 4 + 64 + TC_NMAX * 4 + 256;
}

// Tensor-core form of launch_gateup / launch_down for Q4_K or Q6_K weights and Q8x
// activations. `max_count` bounds the tokens of one group (for the grid's z extent).
cudaError_t launch_tc_q4k(const Launch &L, const LayerDev &ly, bool shared, bool down, Groups g,
                          int n_pairs, uint32_t *tile_buf, const int8_t *xq, const float *xd,
                          const float *wts, float *out, int *err) {
  if (n_pairs == 0) return cudaSuccess;
  // tile list: at most one partial tile per group plus the full ones
  const int max_tiles = tc_max_tiles(n_pairs, g.max_groups);
  int *n_tiles = (int *)tile_buf;
  uint32_t *tile_group = tile_buf + 4, *tile_n0 = tile_buf + 4 + max_tiles;
  k_tc_tiles<<<1, 512, 0, L.stream>>>(g, n_tiles, tile_group, tile_n0, max_tiles);
  if (L.count) ++*L.count;
  const WMat &W = down ? (shared ? ly.sdown : ly.down) : (shared ? ly.sgate : ly.gate);
  const bool q6 = W.type == PM_TYPE_Q6_K;
  const size_t smem = tc_smem(q6 ? 4 : 3);
  const void *kern = q6 ? (const void *)k_tc<PM_TYPE_Q6_K> : (const void *)k_tc<PM_TYPE_Q4_K>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  TcArgs A;
  A.ly = ly;
  A.shared = shared;
  A.down = down;
  A.g = g;
  A.xq = xq;
  A.xd = xd;
  A.wts = wts;
  A.out = out;
  A.err = err;
  A.n_tiles = n_tiles;
  A.tile_group = tile_group;
  A.tile_n0 = tile_n0;
  int row_tiles = down ? (W.rows + TC_M - 1) / TC_M : (W.rows + 63) / 64;
  dim3 grid(row_tiles, max_tiles);
  if (q6) k_tc<PM_TYPE_Q6_K><<<grid, TC_NT, smem, L.stream>>>(A);
  else k_tc<PM_TYPE_Q4_K><<<grid, TC_NT, smem, L.stream>>>(A);
  if (L.count) ++*L.count;
  return cudaGetLastError();
}
