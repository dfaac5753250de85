// prefill_tc.cu - grouped expert products for many tokens per expert on the 5th-gen
// tensor cores (tcgen05.mma kind::i8, operand A and the accumulators in TMEM), exact in
// the integer domain of the reference's CPU path (src/ds4_cpu.rs:59-83).
//
// A work item = (128 weight rows of one active expert) x (up to 128 of its tokens); a CTA (16 worker
// warps, one warp that issues the tensor-core instructions and one producer warp) runs one item, or -
// persistent form - one item after another with its rings running on. Per 256-value block b of
// the rows:
//   1. the producer stages the block's bytes in row-contiguous pieces; each worker unpacks
//      64 values of one row into two u8 operand planes IN REGISTERS and stores them to
//      tensor memory (tcgen05.st), where the products read operand A from: shared memory
//      carries only the tokens' activations. Q4_K: A_hi = nibble * (sc >> 3),
//      A_lo = nibble * (sc & 7), so that with the token's int8 activations xq
//        isum = 8 * (A_hi . xq) + (A_lo . xq) = sum_j sc_j * sum_i nib_ji * xq_ji
//      (6-bit scales do not fit one u8 product with a nibble; two 3-bit halves do), and
//      msum = sum_j m_j * bsum_j comes from one K=16 f16 product (see k_tc).
//   2. the issuing warp runs the block's tcgen05.mma (8 K-steps of 32 per plane) into
//      TMEM accumulators and commits to an mbarrier; meanwhile the workers unpack the
//      next block into registers;
//   3. every worker reads its TMEM lane (tcgen05.ld) and adds the block's float term
//      total += x.d[b] * (d * isum - dmin * msum) in block order, as `row_scalar`. Tiles of at
//      most 64 tokens have two accumulator sets, and step 3 of block b - 1 runs under step 2 of
//      block b.
// Gate and up rows share an item (64 + 64 rows) so SwiGLU is fused in the epilogue;
// down rows write the pair outputs. Waits are time-bounded; TMEM is freed on
// every exit path.
#include <cuda_fp16.h>

#include "moe_internal.cuh"

#define TC_NW 512                 /* worker threads */
#define TC_NT (TC_NW + 64)        /* workers, the warp that issues the products, the producer warp */
// The tokens' operand is read from records laid out for the products (k_tc_rows writes them):
// record (row group rg of 8 rows, block b) = [16 K chunks][8 rows][16 B] int8 activations,
// [2 K chunks][8 rows][8 f16] sub-block sums for the Q4_K mins product, [8] f32 x.d, [8] i32
// block sums (Q6_K), padded to a multiple of 128 bytes so that every 8 x 16 B core matrix sits in
// one 128-byte line of shared memory - one contiguous bulk copy per row group and block, at
// ((rg * n_blocks) + b) * TC_REC
#define TC_REC 2432
#define TC_REC_BM 2048
#define TC_REC_XD 2304
#define TC_REC_XS 2336
#define TC_M 128
#define TC_NMAX 128
#define TC_TMEM_COLS 512
/* TMEM columns 0..383: the accumulators hi, lo, mins - one set of three 128-column accumulators, or
   (tiles of at most TC_DUAL_N tokens) two sets of three 64-column ones that the blocks use in turn */
#define TC_DUAL_N 64
#define TC_A_HI 384u              /* ... and operand A: 64 columns (256 K values) a plane */
#define TC_A_LO 448u
#define TC_RAW_Q4 (TC_M * 144)                       /* bytes of the raw staging area */
#define TC_RAW_Q6 (TC_M * (128 + 64 + 16 + 4))
#define TC_RAW_STAGES_Q4 4                          /* weight blocks in flight */
#define TC_RAW_STAGES_Q6 3

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
// D[tmem_c] (+)= A[tmem_a] * B[db]: A from tensor memory (row = lane, 32-bit column c =
// K values 4c..4c+3), B from shared memory
__device__ __forceinline__ void tc_mma_i8_ta(uint32_t tmem_c, uint32_t tmem_a, uint64_t db, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}\n" ::"r"(tmem_c),
      "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_c, uint64_t da, uint64_t db, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n" ::"r"(tmem_c),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   tc_s32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, uint32_t r[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}
__device__ __forceinline__ void tc_ld4(uint32_t taddr, uint32_t r[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr));
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t r[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// global -> shared without registers, 16 / 4 bytes
__device__ __forceinline__ void tc_cp16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void tc_cp4(uint32_t dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
// named barriers: 1 = operands of a block ready (workers arrive, the issuing warp waits),
// 2 = among the workers
__device__ __forceinline__ void tc_workers_sync() { asm volatile("bar.sync 2, %0;" ::"n"(TC_NW) : "memory"); }
__device__ __forceinline__ void tc_ready_arrive() { asm volatile("bar.arrive 1, %0;" ::"n"(TC_NW + 32) : "memory"); }
__device__ __forceinline__ void tc_ready_wait() { asm volatile("bar.sync 1, %0;" ::"n"(TC_NW + 32) : "memory"); }
__device__ __forceinline__ void tc_mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tc_s32(bar)), "r"(count));
}
__device__ __forceinline__ void tc_mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_s32(bar)) : "memory");
}
__device__ __forceinline__ bool tc_bar_test(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(tc_s32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// false after the wait limit (or at once when an error is already recorded): the caller
// carries on with whatever the accumulators hold and the call reports the error
__device__ __noinline__ bool tc_bar_wait(uint64_t *bar, uint32_t parity, int *err, unsigned long long wait_ns) {
  unsigned long long t0 = tc_now();
  for (uint32_t it = 0;; it++) {
    if (tc_bar_test(bar, parity)) return true;
    if ((it & 15) == 15 && (*(volatile int *)err != 0 || tc_now() - t0 > wait_ns)) break;
  }
  atomicCAS(err, 0, 7);
  return false;
}

// a bounded wait on a phase of an mbarrier (see tc_bar_wait)
__device__ __forceinline__ bool tc_wait(uint64_t *bar, uint32_t parity, int *err, unsigned long long wait_ns) {
  return tc_bar_test(bar, parity) || tc_bar_wait(bar, parity, err, wait_ns);
}

int tc_max_tiles(int n_pairs, int max_groups);

// Compile with -DPM_TC_TRACE=1 (gate/up launches) or =2 (down launches) to stamp the phases of
// CTA 0's first item (persistent form: its second) with the SM clock: [thread 0 | thread 511][block][stamp],
// block slot 30 = the item's start, first block unpacked, blocks done, end; read back with pm_debug_tc_trace.
#ifdef PM_TC_TRACE
__device__ unsigned long long g_tc_trace[3 * 32 * 8];
#define TC_STAMP(b, i)                                                                         \
  if (blockIdx.x == 0 && tc_trace_item && (tid == 0 || tid == 511) && (b) < 32 && A.down + 1 == PM_TC_TRACE) \
    g_tc_trace[((tid ? 1 : 0) * 32 + (b)) * 8 + (i)] = clock64();
extern "C" __attribute__((visibility("default"))) int pm_debug_tc_trace(unsigned long long *out) {
  return (int)cudaMemcpyFromSymbol(out, g_tc_trace, sizeof(g_tc_trace));
}
// the issuing warp's lane 0: section 2
#define TC_STAMP_M(b, i)                                                                       \
  if (blockIdx.x == 0 && tc_trace_item && (tid & 31) == 0 && (b) < 32 && A.down + 1 == PM_TC_TRACE) \
    g_tc_trace[(2 * 32 + (b)) * 8 + (i)] = clock64();
#else
#define TC_STAMP(b, i)
#define TC_STAMP_M(b, i)
#endif

struct TcArgs {
  LayerDev ly;
  int shared;      // 1: the shared expert's matrices (one group over all tokens)
  int down;        // 0: gate+up with activation -> h; 1: down -> pair outputs
  Groups g;
  const uint8_t *rec;    // the tokens' operand as records (see TC_REC), rows grouped and padded as tile_r0 says
  const float *wts;      // routing weights [T*K] (gate/up with fold) or null
  float *out;            // gate/up: h [P][ff]; down: eo [P][d]
  int *err;
  unsigned long long wait_ns;  // limit of every wait on an mbarrier
  int fault_block;             // test hook: no products are issued or signalled from this block on (-1 = off)
  const int *n_tiles;          // [1]
  const uint32_t *tile_group;  // [tiles] index into the groups
  const uint32_t *tile_n0;     // [tiles] first token of the tile inside its group
  const uint32_t *tile_r0;     // [tiles] row of that token among the records' rows (a multiple of 16)
  int row_tiles;               // tiles of rows of the matrix (128 rows, or 64 gate + 64 up)
};

// The (group, token tile) list of a grouping: group a contributes ceil(count/128)
// tiles. The records' rows keep a group's pairs together and start every group on a
// multiple of 16 rows (group_r0), so that a tile's rows are whole row groups. One CTA;
// groups <= 512 (experts of a layer, or the one shared-expert group whose count may be the
// whole batch). tile_r0 / group_r0 may be null (callers that only want the tile list).
__global__ void __launch_bounds__(512) k_tc_tiles(Groups g, int *n_tiles, uint32_t *tile_group,
                                                  uint32_t *tile_n0, uint32_t *tile_r0, uint32_t *group_r0,
                                                  int max_tiles) {
  __shared__ uint32_t s[512], sr[512];
  const int a = threadIdx.x;
  const int ng = min(*g.n_groups, 512);
  const uint32_t cnt = a < ng ? g.count[a] : 0;
  uint32_t tc = (cnt + TC_NMAX - 1) / TC_NMAX;
  const uint32_t rp = (cnt + 15u) & ~15u;
  s[a] = tc;
  sr[a] = rp;
  __syncthreads();
  for (int off = 1; off < 512; off <<= 1) {
    uint32_t v = a >= off ? s[a - off] : 0, w = a >= off ? sr[a - off] : 0;
    __syncthreads();
    s[a] += v;
    sr[a] += w;
    __syncthreads();
  }
  uint32_t first = s[a] - tc, r0 = sr[a] - rp;
  if (group_r0 && a < ng) group_r0[a] = r0;
  for (uint32_t i = 0; i < tc && (int)(first + i) < max_tiles; i++) {
    tile_group[first + i] = (uint32_t)a;
    tile_n0[first + i] = i * TC_NMAX;
    if (tile_r0) tile_r0[first + i] = r0 + i * TC_NMAX;
  }
  if (a == 511) *n_tiles = min((int)s[511], max_tiles);
}

// Quantised activation rows -> the records the products read (TC_REC): one warp per (row
// group of 8 rows, block). Row i of group a is record row group_r0[a] + i and comes from
// row src_row[offset[a] + i] of the quantiser's outputs (null: row offset[a] + i itself);
// rows past a group's count are zeros.
__global__ void __launch_bounds__(256) k_tc_rows(Groups g, const uint32_t *__restrict__ group_r0,
                                                 const uint32_t *__restrict__ src_row, int cols,
                                                 const int8_t *__restrict__ xq, const float *__restrict__ xd,
                                                 const uint16_t *__restrict__ xbm, const int32_t *__restrict__ xs,
                                                 uint8_t *__restrict__ rec) {
  const int a = blockIdx.y;
  if (a >= *g.n_groups) return;
  const int nb = cols / 256;
  const uint32_t off = g.offset[a], cnt = g.count[a], r0 = group_r0[a];
  const int lane = threadIdx.x & 31;
  const int units = (int)((cnt + 15u) / 16u) * 2 * nb;  // (row group, block) pairs of this group
  for (int u = blockIdx.x * 8 + (threadIdx.x >> 5); u < units; u += gridDim.x * 8) {
    const int rgl = u / nb, b = u - rgl * nb;
    uint8_t *R = rec + ((size_t)(r0 / 8 + rgl) * nb + b) * TC_REC;
    {  // int8 values: lane = (row of the group, quarter of the block's 16 chunks)
      const int r8 = lane >> 2, q = lane & 3;
      const uint32_t i = (uint32_t)rgl * 8 + r8;
      uint4 v[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
      if (i < cnt) {
        const size_t row = src_row ? src_row[off + i] : off + i;
        const uint4 *src = (const uint4 *)(xq + row * cols + (size_t)b * 256 + 64 * q);
#pragma unroll
        for (int c = 0; c < 4; c++) v[c] = __ldg(src + c);
      }
#pragma unroll
      for (int c = 0; c < 4; c++) *(uint4 *)(R + ((4 * q + c) * 8 + r8) * 16) = v[c];
    }
    if (lane < 16) {  // the f16 form of the sub-block sums: lane = (row, K chunk of the mins product)
      const int r8 = lane >> 1, k = lane & 1;
      const uint32_t i = (uint32_t)rgl * 8 + r8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (i < cnt && xbm) {
        const size_t row = src_row ? src_row[off + i] : off + i;
        v = __ldg((const uint4 *)(xbm + (row * nb + b) * 16 + 8 * k));
      }
      *(uint4 *)(R + TC_REC_BM + (k * 8 + r8) * 16) = v;
    } else if (lane < 24) {
      const int r8 = lane - 16;
      const uint32_t i = (uint32_t)rgl * 8 + r8;
      float v = 0.0f;
      if (i < cnt) v = xd[(src_row ? (size_t)src_row[off + i] : (size_t)(off + i)) * nb + b];
      *(float *)(R + TC_REC_XD + r8 * 4) = v;
    } else {
      const int r8 = lane - 24;
      const uint32_t i = (uint32_t)rgl * 8 + r8;
      int32_t v = 0;
      if (i < cnt && xs) v = xs[(src_row ? (size_t)src_row[off + i] : (size_t)(off + i)) * nb + b];
      *(int32_t *)(R + TC_REC_XS + r8 * 4) = v;
    }
  }
}

// WT: the weight type of the product's matrices.
//  PM_TYPE_Q4_K: u8 planes hi = nibble * (sc >> 3), lo = nibble * (sc & 7) and one
//    kind::f16 product for the mins: A_m = (m_0..m_7, m_0..m_7) against the token's
//    (64 * (bsum_j >> 6), bsum_j & 63) - every product and the sum (< 2^22) are exact in
//    f32, so the accumulator holds msum = sum_j m_j * bsum_j as an integer-valued float.
//  PM_TYPE_Q6_K: the product v = sc * (q - 32) in [-4064, 4096] is split after the
//    multiplication: v + 4128 = 64 * th + tl with th in [1, 128], tl in [0, 63] - two u8
//    planes, and isum = 64 * (th . xq) + (tl . xq) - 4128 * sum(xq) exactly. The planes are
//    th and 4 * tl (the two bytes of 4 * (v + 4128)), so the products give 4 * isum and the
//    fold multiplies by d / 4: both scalings are by a power of two, the rounding is that of
//    d * float(isum).
//  PERSIST, DOWN, SMALL: the launch's form (see launch_tc_q4k).
// Memory: one producer warp feeds two rings, each with a full and an empty mbarrier per stage.
// The weight bytes of a block go to one of TC_RAW_STAGES raw areas as stored, by 16-byte
// cp.async pieces (consecutive lanes on consecutive pieces of a row; the completion of a
// lane's pieces arrives on the stage's barrier), freed once every worker warp has unpacked
// it. The tokens' operand of a block - up to 16 records written by k_tc_rows in the
// products' own layout - comes by one bulk copy a record into one of three areas, freed once
// its products have completed (tcgen05.commit) and every worker warp has read the block's
// x.d for the fold. (The workers used to issue the copies themselves, the activations as
// 16-byte cp.async pieces: those retire at about one warp instruction per 24 cycles on this
// part, and waiting for them was the longest phase of a block.)
template <int WT, bool PERSIST, bool DOWN, bool SMALL>
__global__ void __launch_bounds__(TC_NT, 1) k_tc(const TcArgs A) {
  constexpr bool Q6 = WT == PM_TYPE_Q6_K;
  constexpr int NS = Q6 ? TC_RAW_STAGES_Q6 : TC_RAW_STAGES_Q4;
  constexpr int RAWB = Q6 ? TC_RAW_Q6 : TC_RAW_Q4;
  constexpr int BSTAGE = (TC_NMAX / 8) * TC_REC;  // the tokens' block: a record per 8 tokens
  extern __shared__ __align__(128) uint8_t smem[];
  const LayerDev &ly = A.ly;
  const WMat &W0 = DOWN ? (A.shared ? ly.sdown : ly.down) : (A.shared ? ly.sgate : ly.gate);
  const WMat &W1 = A.shared ? ly.sup : ly.up;  // used by gate/up only
  const int cols = W0.cols, nb = cols / 256, rows = W0.rows;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int rows_per_cta = DOWN ? TC_M : TC_M / 2;  // gate/up: 64 gate + 64 up rows
  // Work items are (token tile, row tile) pairs, row tiles fastest so that the CTAs running together
  // share a tile's records in L2. One-item form: a CTA per item, grid (row tiles, token tiles).
  // Persistent form: gridDim.x CTAs, CTA i takes items i, i + gridDim.x, ...; the rings and the
  // block counter run on across items, and the producer is already fetching the next item's
  // operands while the workers write an item's outputs.
  const int n_items = *A.n_tiles * A.row_tiles;
  int a = 0, el = 0, n0 = 0, nvalid = 0, npad = 16, r0 = 0, tile = 0;
  uint32_t off = 0, cnt = 0;
  bool local = false;
  auto set_item = [&](int w) {
    if (!PERSIST) {
      tile = blockIdx.y;
      r0 = blockIdx.x * rows_per_cta;
    } else {
      tile = w / A.row_tiles;
      r0 = (w - tile * A.row_tiles) * rows_per_cta;
    }
    a = (int)A.tile_group[tile];
    el = A.shared ? 0 : (int)A.g.expert[a] - ly.first_local;
    off = A.g.offset[a];
    cnt = A.g.count[a];
    n0 = (int)A.tile_n0[tile];
    nvalid = min((int)cnt - n0, TC_NMAX);
    npad = (nvalid + 15) & ~15;
    local = el >= 0 && el < (A.shared ? 1 : ly.n_local);  // else: an expert another rank holds
  };
  // every role walks the CTA's items with its own copy of w
  int w = PERSIST ? blockIdx.x : blockIdx.y * A.row_tiles + blockIdx.x;
  if (w >= n_items) return;
  set_item(w);
  auto next_item = [&]() -> bool {
    if (!PERSIST) return false;
    w += gridDim.x;
    if (w >= n_items) return false;
    set_item(w);
    return true;
  };

  uint8_t *sRaw = smem;                                        // [NS] blocks of the 128 rows as stored
  float *sS = (float *)smem;                                   // (after the last block) gate/up exchange [128][129]
  uint8_t *sB = smem + (NS * RAWB > TC_M * (TC_NMAX + 1) * 4 ? NS * RAWB : TC_M * (TC_NMAX + 1) * 4);
                                                               // [3] x [npad / 8 records]
  uint8_t *sAm = sB + 3 * BSTAGE;                              // Q4_K: [2][2 chunks][128 rows][8 f16]
  uint64_t *bar = (uint64_t *)(sAm + 2 * 2 * TC_M * 16);       // the products of a block have completed
  uint64_t *full_raw = bar + 1, *empty_raw = full_raw + 4;     // rings of the raw areas ...
  uint64_t *full_b = empty_raw + 4, *empty_b = full_b + 3;     // ... and of the tokens' areas
  uint64_t *epi_done = empty_b + 3;                            // gate/up over the raw areas: the exchange has been read
  uint32_t *tmem_slot = (uint32_t *)(epi_done + 1);

  if (warp == TC_NW / 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     tc_s32(tmem_slot)),
                 "r"((uint32_t)TC_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    tc_mbar_init(bar, 1);
    for (int i = 0; i < 4; i++) {
      tc_mbar_init(full_raw + i, 32);  // every producer lane's copies
      tc_mbar_init(empty_raw + i, TC_NW / 32);
    }
    for (int i = 0; i < 3; i++) {
      tc_mbar_init(full_b + i, 1);  // the producer's expect_tx; the bulk copies complete the bytes
      tc_mbar_init(empty_b + i, 1 + TC_NW / 32);  // the products' commit and every worker warp after its fold
    }
    tc_mbar_init(epi_done, TC_NW / 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  const uint32_t sB_a = tc_s32(sB), sAm_a = tc_s32(sAm);

  // Global row of tile row i (gate rows, then up rows, in a gate/up tile), or -1 past the
  // matrix; `second`: the row belongs to the up matrix
  auto grow = [&](int i, bool &second) -> int {
    second = !DOWN && i >= 64;
    int r = r0 + (second ? i - 64 : i);
    return r < rows ? r : -1;
  };

  if (warp == TC_NW / 32) {
    // ================= the issuing warp =================
    // instruction descriptors: D s32, A u8, B s8, K-major; and the f16 one (D f32)
    int gb = 0;  // blocks this CTA has run so far
    for (;;) {
    if (!local) {
      if (next_item()) continue;
      break;
    }
    const bool tc_trace_item = w == (PERSIST ? (int)gridDim.x : 0);  // persistent form: CTA 0's second item
    (void)tc_trace_item;
    const uint32_t idesc = (2u << 4) | (1u << 10) | ((uint32_t)(npad >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24);
    const uint32_t idesc_h = (1u << 4) | ((uint32_t)(npad >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24);
    for (int b = 0; b < nb; b++, gb++) {
      const int sb = gb % 3;
      const uint32_t bs = sB_a + (uint32_t)sb * BSTAGE;
      const uint64_t dB0 = tc_desc(bs, 128u, (uint32_t)TC_REC);  // K chunks 128 B apart, 8-token groups a record apart
      TC_STAMP_M(b, 0)
      tc_wait(full_b + sb, (uint32_t)((gb / 3) & 1), A.err, A.wait_ns);  // the tokens' block is in shared memory
      TC_STAMP_M(b, 1)
      tc_ready_wait();  // operand A in TMEM, the accumulators read
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      TC_STAMP_M(b, 2)
      // tiles of at most 64 tokens: two accumulator sets, blocks alternate (see the workers)
      const bool dual = SMALL && npad <= TC_DUAL_N;
      const uint32_t acc_w = dual ? (uint32_t)TC_DUAL_N : (uint32_t)TC_NMAX;
      const uint32_t acc = tmem + (dual ? (uint32_t)(gb & 1) * (3u * TC_DUAL_N) : 0u);
      if ((tid & 31) == 0 && !(A.fault_block >= 0 && b >= A.fault_block)) {
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
          const uint64_t db = dB0 + (uint64_t)(ks * 16);  // two K chunks a step
          tc_mma_i8_ta(acc, tmem + TC_A_HI + 8u * ks, db, idesc, ks > 0 ? 1u : 0u);
          tc_mma_i8_ta(acc + acc_w, tmem + TC_A_LO + 8u * ks, db, idesc, ks > 0 ? 1u : 0u);
        }
        if (!Q6)
          tc_mma_f16(acc + 2u * acc_w, tc_desc(sAm_a + (uint32_t)(gb & 1) * (2 * TC_M * 16), TC_M * 16u, 128u),
                     tc_desc(bs + TC_REC_BM, 128u, (uint32_t)TC_REC), idesc_h, 0u);
        tc_commit(bar);
        tc_commit(empty_b + sb);
      }
      TC_STAMP_M(b, 3)
      __syncwarp();
    }
    if (!next_item()) break;
    }
  } else if (warp > TC_NW / 32) {
    // ================= the producer =================
    const int lane = tid & 31;
    const uint32_t sRaw_a = tc_s32(sRaw);
    int gb = 0, k_local = 0;  // blocks and items this CTA has run so far
    bool prev_small = false;  // the previous item's gate/up exchange took two raw areas only
    for (;;) {
    if (!local) {
      if (next_item()) continue;
      break;
    }
    const uint8_t *wb0[4], *wb1[4];  // the expert's planes of the tile's matrices
#pragma unroll
    for (int pl = 0; pl < 4; pl++) {
      wb0[pl] = W0.plane[pl] ? W0.plane[pl] + (size_t)el * W0.stride[pl] : nullptr;
      wb1[pl] = (!DOWN && W1.plane[pl]) ? W1.plane[pl] + (size_t)el * W1.stride[pl] : nullptr;
    }
    const uint8_t *rec0 = A.rec + (size_t)(A.tile_r0[tile] / 8) * nb * TC_REC;  // the tile's first record
    const int nrec = npad >> 3;
    // Q4_K: 9 pieces a row, [row][144 B]; piece p = lane + 32 j of the tile. Pieces 0..575 are
    // tile rows 0..63 and pieces 576.. the same (row, piece) pattern 64 rows on: of the other matrix
    // (gate/up tiles) or of the same one (down tiles). So 18 byte offsets (of the piece in block 0
    // of its row) and two validity masks stay in registers, and a block costs one address and one
    // copy instruction a piece.
    uint32_t roff[Q6 ? 1 : 18];
    uint32_t okA = 0, okB = 0;
    const uint8_t *pA = wb0[0], *pB = DOWN ? wb0[0] + (size_t)64 * nb * 144 : wb1[0];
    if (!Q6) {
#pragma unroll
      for (int j = 0; j < 18; j++) {
        const int p = lane + 32 * j, i = p / 9, c = p - 9 * i;
        roff[j] = (uint32_t)(r0 + i) * (uint32_t)nb * 144u + 16u * c;
        if (r0 + i < rows) okA |= 1u << j;
        if (r0 + i + (DOWN ? 64 : 0) < rows) okB |= 1u << j;
      }
    }
    // Q6_K: ql 8 pieces a row, [row][128 B], piece c at c ^ (row & 7); qh 4 pieces a row,
    // [row][64 B], piece c at c ^ ((row >> 1) & 3) (both conflict-free for the row-per-lane reads
    // of the unpack); sc [row][16 B]; d: the aligned word holding the row's f16. A lane keeps its
    // piece column and walks rows: tile row i = i0 + step * j.
    // gate/up, persistent form: the previous item's exchange of gate and up sums lives in the raw
    // areas and its readers must be done before this item's weights land there. A tile of at most 64
    // tokens exchanges through the two areas that this item's blocks 2 and 3 will use, so blocks 0
    // and 1 (and their tokens' records) are fetched during the previous item's epilogue.
    const int wait_at = (!DOWN && PERSIST && k_local > 0) ? (prev_small ? (nb < 2 ? nb : 2) : 0) : -1;
    const uint32_t epi_par = (uint32_t)((k_local - 1) & 1);
    prev_small = NS == 4 && npad <= TC_DUAL_N;
    k_local++;
    for (int bb = 0; bb < nb; bb++, gb++) {
      if (bb == wait_at) tc_wait(epi_done, epi_par, A.err, A.wait_ns);
      // ---- the weights of block bb -> the next raw area ----
      {
        const int st = gb % NS;
        const uint32_t ra = sRaw_a + (uint32_t)st * RAWB;
        if (gb >= NS) tc_wait(empty_raw + st, (uint32_t)((gb / NS - 1) & 1), A.err, A.wait_ns);
        if (!Q6) {
#pragma unroll
          for (int j = 0; j < 18; j++) {
            if (okA & (1u << j)) tc_cp16(ra + (uint32_t)(lane + 32 * j) * 16u, pA + roff[j] + (size_t)bb * 144);
            if (okB & (1u << j)) tc_cp16(ra + (uint32_t)(lane + 32 * (j + 18)) * 16u, pB + roff[j] + (size_t)bb * 144);
          }
        } else {
          const int halves = DOWN ? 1 : 2, hrows = DOWN ? TC_M : TC_M / 2;
          for (int hf = 0; hf < halves; hf++) {
            const uint8_t *const *wb = hf ? wb1 : wb0;
            const int lim = min(hrows, rows - r0);  // rows of this half inside the matrix
            {
              const int c = lane & 7;
              const uint8_t *src = wb[0] + ((size_t)(r0 + (lane >> 3)) * nb + bb) * 128 + 16 * c;
              for (int il = lane >> 3; il < lim; il += 4, src += (size_t)4 * nb * 128) {
                const int i = hf * hrows + il;
                tc_cp16(ra + (uint32_t)(i * 128 + ((c ^ (i & 7)) << 4)), src);
              }
            }
            {
              const int c = lane & 3;
              const uint8_t *src = wb[1] + ((size_t)(r0 + (lane >> 2)) * nb + bb) * 64 + 16 * c;
              for (int il = lane >> 2; il < lim; il += 8, src += (size_t)8 * nb * 64) {
                const int i = hf * hrows + il;
                tc_cp16(ra + 16384u + (uint32_t)(i * 64 + ((c ^ ((i >> 1) & 3)) << 4)), src);
              }
            }
            for (int il = lane; il < lim; il += 32) {
              const int i = hf * hrows + il;
              tc_cp16(ra + 24576u + (uint32_t)i * 16u, wb[2] + ((size_t)(r0 + il) * nb + bb) * 16);
              tc_cp4(ra + 26624u + (uint32_t)i * 4u,
                     (const uint8_t *)((uintptr_t)(wb[3] + ((size_t)(r0 + il) * nb + bb) * 2) & ~(uintptr_t)3));
            }
          }
        }
        // this lane's pieces, once they have landed, count as its arrival on the stage's barrier
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(tc_s32(full_raw + st)) : "memory");
      }
      // ---- the tokens' records of block bb -> their area ----
      {
        const int sb = gb % 3;
        if (gb >= 3) tc_wait(empty_b + sb, (uint32_t)((gb / 3 - 1) & 1), A.err, A.wait_ns);
        if (lane == 0)
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tc_s32(full_b + sb)),
                       "r"((uint32_t)(nrec * TC_REC))
                       : "memory");
        __syncwarp();
        if (lane < nrec)
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                           sB_a + (uint32_t)(sb * BSTAGE + lane * TC_REC)),
                       "l"(rec0 + ((size_t)lane * nb + bb) * TC_REC), "r"((uint32_t)TC_REC), "r"(tc_s32(full_b + sb))
                       : "memory");
      }
    }
    if (wait_at == nb) tc_wait(epi_done, epi_par, A.err, A.wait_ns);  // (an item shorter than three blocks)
    if (!next_item()) break;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    // the last bulk copies have landed before the CTA gives up its shared memory (the workers waited
    // for them already unless a wait ran out; in the one-item form, where the check measured 3 %
    // slower, that is relied on)
    if (PERSIST)
    for (int g = gb > 3 ? gb - 3 : 0; g < gb; g++) {
      const unsigned long long t0 = tc_now();
      while (!tc_bar_test(full_b + g % 3, (uint32_t)((g / 3) & 1)) && tc_now() - t0 < A.wait_ns) {
      }
    }
  } else {
    // ================= the workers =================
    // unpack: thread = (row m of the tile, quarter `part` of the block: K values
    // 64 part .. 64 part + 63 = TMEM columns 16 part .. 16 part + 15 of each plane). The same
    // thread folds row m's accumulators (TMEM lane m), a quarter of the token columns, so
    // the row's (d, dmin) stay in registers.
    const int m = tid & 127, part = tid >> 7;
    const uint32_t tlane = tmem + ((uint32_t)(32 * (warp & 3)) << 16);
    int gb0 = 0;  // blocks this CTA ran before the current item
    for (;;) {
    if (!local) {  // zeros (down) / nothing to do (gate/up)
      if (DOWN)
        for (int i = tid; i < nvalid * TC_M; i += TC_NW) {
          int n = i / TC_M, mm = i % TC_M;
          if (r0 + mm < rows) A.out[(size_t)(off + n0 + n) * rows + r0 + mm] = 0.0f;
        }
      if (next_item()) continue;
      break;
    }
    const bool tc_trace_item = w == (PERSIST ? (int)gridDim.x : 0);  // persistent form: CTA 0's second item
    (void)tc_trace_item;
    TC_STAMP(30, 0)
    bool msec;
    const int mrow = grow(m, msec);
    // the f16 d of a Q6_K row sits in the low or high half of the staged word
    const uint32_t dsel = Q6 && mrow >= 0
                              ? (uint32_t)(((uintptr_t)((msec ? W1 : W0).plane[3] + (size_t)el * (msec ? W1 : W0).stride[3]) >> 1) & 1)
                              : 0u;
    uint32_t ah[16], al[16];  // this thread's 64 values of the two planes
    float nrd = 0.0f, nrdmin = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i++) ah[i] = al[i] = 0u;
    if (mrow < 0 && !Q6) {  // rows past the matrix: zero mins, once, both buffers
      if (part < 2) *(uint4 *)(sAm + (size_t)(part * TC_M + m) * 16) = make_uint4(0, 0, 0, 0);
      else *(uint4 *)(sAm + 2 * TC_M * 16 + (size_t)((part - 2) * TC_M + m) * 16) = make_uint4(0, 0, 0, 0);
    }
    // block bb of the item (the CTA's block g) of its raw area -> ah/al, nrd/nrdmin (and the mins of
    // the row into sAm[g & 1])
    auto unpack = [&](int bb, int g) {
      if (mrow < 0) return;
      const uint8_t *raw = sRaw + (size_t)(g % NS) * RAWB;
      if (Q6) {
        const int hf = part >> 1, p2 = part & 1;
        const uint8_t *rq = raw + m * 128, *rh = raw + 16384 + m * 64;
        uint4 qlv[4], qhv[2];
#pragma unroll
        for (int j = 0; j < 4; j++) qlv[j] = *(const uint4 *)(rq + (((4 * hf + j) ^ (m & 7)) << 4));
#pragma unroll
        for (int j = 0; j < 2; j++) qhv[j] = *(const uint4 *)(rh + (((2 * hf + j) ^ ((m >> 1) & 3)) << 4));
        const uint32_t scw = *(const uint32_t *)(raw + 24576 + m * 16 + 8 * hf + 4 * p2);
        const uint32_t dw = *(const uint32_t *)(raw + 26624 + m * 4);
        nrd = pm_f16(((((size_t)mrow * nb + bb) & 1) ^ dsel) ? (dw >> 16) : (dw & 0xffffu));
#pragma unroll
        for (int qq = 0; qq < 2; qq++) {
#pragma unroll
          for (int lh = 0; lh < 2; lh++) {
            // 16 values: sub-block 8 hf + 2 qt + lh of the block, qt = 2 p2 + qq
            const uint4 qlw = qlv[2 * qq + lh];
            const uint4 qhw = qhv[lh];
            const int sv = (int)(int8_t)((scw >> (8 * (2 * qq + lh))) & 0xff);
            // z4 = 4 * (sv * (q - 32) + 4128) in [256, 32896]: its high byte is th, its low byte 4 * tl
            // (v + 4128 = 64 th + tl). The low plane holds 4 * tl, the fold takes a quarter of d.
            const uint32_t sv4 = (uint32_t)(4 * sv);
            const uint32_t kk = (uint32_t)(4 * (4128 - 32 * sv)) * 0x00010001u;
            const uint32_t ws[4] = {qlw.x, qlw.y, qlw.z, qlw.w}, hs[4] = {qhw.x, qhw.y, qhw.z, qhw.w};
            const int rot = (4 * p2 + 2 * qq - 4) & 31;  // brings the pair of high bits to bits 4, 5 of its byte
#pragma unroll
            for (int i = 0; i < 4; i++) {
              const uint32_t qv = ((ws[i] >> (4 * p2)) & 0x0f0f0f0fu) | (__funnelshift_r(hs[i], hs[i], rot) & 0x30303030u);
              // two values per 32-bit product (16-bit lanes, each lane's result positive): values 0, 2 and 1, 3
              const uint32_t ze = __byte_perm(qv, 0u, 0x4240) * sv4 + kk;
              const uint32_t zo = __byte_perm(qv, 0u, 0x4341) * sv4 + kk;
              al[4 * (2 * qq + lh) + i] = __byte_perm(ze, zo, 0x6240);
              ah[4 * (2 * qq + lh) + i] = __byte_perm(ze, zo, 0x7351);
            }
          }
        }
      } else {
        const uint8_t *rp = raw + m * 144;
        const uint4 hdr = *(const uint4 *)rp;
        nrd = pm_f16(hdr.x);
        nrdmin = pm_f16(hdr.x >> 16);
        uint32_t sc03, sc47, m03, m47;
        pm_q4k_scmin_packed(hdr.y, hdr.z, hdr.w, sc03, sc47, m03, m47);
        if (part < 2)  // the eight mins as f16, K chunk `part` of the f16 product (both hold m_0..m_7)
          *(uint4 *)(sAm + (size_t)(g & 1) * (2 * TC_M * 16) + (size_t)(part * TC_M + m) * 16) =
              make_uint4(pm_bytes_to_half2(m03, 0x4140), pm_bytes_to_half2(m03, 0x4342),
                         pm_bytes_to_half2(m47, 0x4140), pm_bytes_to_half2(m47, 0x4342));
        const int c = part;
        const uint4 w0 = *(const uint4 *)(rp + 16 + 32 * c), w1 = *(const uint4 *)(rp + 32 + 32 * c);
        const uint32_t scw = ((c & 2) ? sc47 : sc03) >> (16 * (c & 1));
        const uint32_t sc0 = scw & 0xffu, sc1 = (scw >> 8) & 0xffu;  // scales of sub-blocks 2c, 2c+1
        const uint32_t M4 = 0x0f0f0f0fu;
        // sub-block 2c = low nibbles -> K 64c .. 64c+31 ; sub-block 2c+1 = high -> K 64c+32 .. 64c+63
        const uint32_t lo[8] = {w0.x & M4, w0.y & M4, w0.z & M4, w0.w & M4, w1.x & M4, w1.y & M4, w1.z & M4, w1.w & M4};
        const uint32_t hi[8] = {(w0.x >> 4) & M4, (w0.y >> 4) & M4, (w0.z >> 4) & M4, (w0.w >> 4) & M4,
                                (w1.x >> 4) & M4, (w1.y >> 4) & M4, (w1.z >> 4) & M4, (w1.w >> 4) & M4};
        const uint32_t sh0 = sc0 >> 3, sl0 = sc0 & 7, sh1 = sc1 >> 3, sl1 = sc1 & 7;
#pragma unroll
        for (int i = 0; i < 8; i++) {
          ah[i] = lo[i] * sh0;
          al[i] = lo[i] * sl0;
          ah[8 + i] = hi[i] * sh1;
          al[8 + i] = hi[i] * sl1;
        }
      }
    };
    // wait for raw block bb, unpack it, and free its area once the whole warp has read it
    auto take = [&](int bb) {
      const int g = gb0 + bb, st = g % NS;
      tc_wait(full_raw + st, (uint32_t)((g / NS) & 1), A.err, A.wait_ns);
      unpack(bb, g);
      __syncwarp();
      if ((tid & 31) == 0) tc_mbar_arrive(empty_raw + st);
    };

    // (3) fold: TMEM lane m, a quarter of the tile's token columns (npad / 4: a multiple of 4)
    const int ew = npad >> 2, ecol0 = part * ew;
    float total[32];
#pragma unroll
    for (int i = 0; i < 32; i++) total[i] = 0.0f;

    // Tiles of at most 64 tokens keep two accumulator sets in tensor memory: the float term of block
    // b - 1 is then added while the products of block b run, and the period of a block is the
    // products' time instead of products + float term. (Operand A has one buffer, so the products of
    // consecutive blocks never overlap; wider tiles fill tensor memory with one set.)
    const bool dual = SMALL && npad <= TC_DUAL_N;
    const uint32_t acc_w = dual ? (uint32_t)TC_DUAL_N : (uint32_t)TC_NMAX;
    float rd_p = 0.0f, rdmin_p = 0.0f;  // dual: the scales of the block whose float term is pending
    take(0);
    TC_STAMP(30, 1)
    for (int b = 0; b <= nb; b++) {
      const int g = gb0 + b;
      float rd_b = 0.0f, rdmin_b = 0.0f;
      if (dual && b > 0) {  // the previous block's products: operand A is free, its accumulators are ready
        tc_wait(bar, (uint32_t)((g - 1) & 1), A.err, A.wait_ns);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      if (b < nb) {
        TC_STAMP(b, 0)
        rd_b = Q6 ? __fmul_rn(nrd, 0.25f) : nrd;  // Q6_K: the products come out times 4
        rdmin_b = nrdmin;
        // ---- 1. operand A of block b -> tensor memory (the previous block's products have
        // completed: every worker waited on their barrier) ----
        tc_st16(tlane + TC_A_HI + 16u * part, ah);
        tc_st16(tlane + TC_A_LO + 16u * part, al);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the mins written by unpack(b)
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        tc_ready_arrive();
        TC_STAMP(b, 1)
        // ---- 2. while the products run: the next block -> registers ----
        if (b + 1 < nb) take(b + 1);
        TC_STAMP(b, 2)
        if (!dual) {
          tc_wait(bar, (uint32_t)(g & 1), A.err, A.wait_ns);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        TC_STAMP(b, 3)
      }
      // ---- 3. the float term of block fb (this block, or in dual mode the previous one), in block order ----
      const int fb = dual ? b - 1 : b;
      const float rd = dual ? rd_p : rd_b, rdmin = dual ? rdmin_p : rdmin_b;
      rd_p = rd_b;
      rdmin_p = rdmin_b;
      if (fb < 0 || fb >= nb) continue;
      const int gf = gb0 + fb, sb = gf % 3;
      tc_wait(full_b + sb, (uint32_t)((gf / 3) & 1), A.err, A.wait_ns);  // (long complete) the block's x.d is visible
      const uint32_t acc_hi = tlane + (dual ? (uint32_t)(gf & 1) * (3u * TC_DUAL_N) : 0u) + (uint32_t)ecol0;
      const uint32_t acc_lo = acc_hi + acc_w, acc_m = acc_lo + acc_w;
      TC_STAMP(fb, 4)
      {
        const uint8_t *bst = sB + (size_t)sb * BSTAGE;  // column n: record n / 8, slot n % 8
        // (four columns a wait: eight a wait, and requesting a step ahead, both measured slower -
        // the extra live registers cost more than the read latency they hide)
        if (ew <= 8) {  // tiles of at most 32 tokens: the thread's columns behind one wait
          uint32_t v0[8], v1[8], v2[8];
          tc_ld8(acc_hi, v0);
          tc_ld8(acc_lo, v1);
          if (!Q6) tc_ld8(acc_m, v2);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int h4 = 0; h4 < 8; h4 += 4) {
            if (h4 < ew) {
              const int n = ecol0 + h4;
              const uint8_t *rcd = bst + (size_t)(n >> 3) * TC_REC + (n & 7) * 4;
              const float4 x4 = *(const float4 *)(rcd + TC_REC_XD);
              const float xs[4] = {x4.x, x4.y, x4.z, x4.w};
              int ss[4] = {0, 0, 0, 0};
              if (Q6) {
                const int4 s4 = *(const int4 *)(rcd + TC_REC_XS);
                ss[0] = s4.x; ss[1] = s4.y; ss[2] = s4.z; ss[3] = s4.w;
              }
#pragma unroll
              for (int u = 0; u < 4; u++) {
                float term;
                if (Q6) {
                  int isum = 256 * (int)v0[h4 + u] + (int)v1[h4 + u] - 16512 * ss[u];
                  term = __fmul_rn(xs[u], __fmul_rn(rd, (float)isum));
                } else {
                  int isum = 8 * (int)v0[h4 + u] + (int)v1[h4 + u];
                  term = __fmul_rn(xs[u], __fsub_rn(__fmul_rn(rd, (float)isum), __fmul_rn(rdmin, __uint_as_float(v2[h4 + u]))));
                }
                total[h4 + u] = __fadd_rn(total[h4 + u], term);
              }
            }
          }
        } else
#pragma unroll
        for (int c4 = 0; c4 < 32; c4 += 4) {
          if (c4 < ew) {
            uint32_t v0[4], v1[4], v2[4];
            tc_ld4(acc_hi + (uint32_t)c4, v0);
            tc_ld4(acc_lo + (uint32_t)c4, v1);
            if (!Q6) tc_ld4(acc_m + (uint32_t)c4, v2);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const int n = ecol0 + c4;
            const uint8_t *rcd = bst + (size_t)(n >> 3) * TC_REC + (n & 7) * 4;
            const float4 x4 = *(const float4 *)(rcd + TC_REC_XD);
            const float xs[4] = {x4.x, x4.y, x4.z, x4.w};
            int ss[4] = {0, 0, 0, 0};
            if (Q6) {
              const int4 s4 = *(const int4 *)(rcd + TC_REC_XS);
              ss[0] = s4.x; ss[1] = s4.y; ss[2] = s4.z; ss[3] = s4.w;
            }
            // (scalar on purpose: packed f32x2 forms - mul.rn.f32x2 then add.rn.f32x2, and the same
            // written as fma.rn.f32x2 with a -0 addend / a unit factor - came out with other bits
            // than the reference's separately rounded steps, and ran no faster)
#pragma unroll
            for (int u = 0; u < 4; u++) {
              float term;
              if (Q6) {
                // 4 * isum (exact in int32; (d / 4) * float(4 isum) rounds as d * float(isum) does)
                int isum = 256 * (int)v0[u] + (int)v1[u] - 16512 * ss[u];
                term = __fmul_rn(xs[u], __fmul_rn(rd, (float)isum));
              } else {
                int isum = 8 * (int)v0[u] + (int)v1[u];
                term = __fmul_rn(xs[u], __fsub_rn(__fmul_rn(rd, (float)isum), __fmul_rn(rdmin, __uint_as_float(v2[u]))));
              }
              total[c4 + u] = __fadd_rn(total[c4 + u], term);
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if ((tid & 31) == 0) tc_mbar_arrive(empty_b + sb);  // this warp has read the block's x.d
      TC_STAMP(fb, 5)
    }
    gb0 += nb;
    TC_STAMP(30, 2)
    if (!DOWN) tc_workers_sync();  // every worker has unpacked the item's last block: the raw areas carry the gate/up exchange

    const bool dead = *(volatile int *)A.err != 0;
    if (DOWN) {
      if (!dead) {
        const float bd = (!A.shared && ly.bias_down && r0 + m < rows) ? ly.bias_down[(size_t)el * rows + r0 + m] : 0.0f;
#pragma unroll
        for (int i = 0; i < 32; i++) {
          int n = ecol0 + i;
          if (i < ew && n < nvalid && r0 + m < rows) {
            float o = total[i];
            if (!A.shared && ly.bias_down) o = __fadd_rn(o, bd);
            A.out[(size_t)(off + n0 + n) * rows + r0 + m] = o;
          }
        }
      }
    } else {
      // gate rows in tile rows 0..63, up rows in 64..127: exchange through shared memory. A tile of at
      // most 64 tokens takes the two raw areas that held the item's last blocks - the next item's
      // blocks 2 and 3 - and leaves the other two to the producer (Q4_K: four areas); a wider tile
      // takes all of them.
      const bool xsmall = NS == 4 && npad <= TC_DUAL_N;
      const int xstride = xsmall ? TC_DUAL_N + 1 : TC_NMAX + 1;
      float *sG = xsmall ? (float *)(sRaw + (size_t)((gb0 + 2) % NS) * RAWB) : sS;
      float *sU = xsmall ? (float *)(sRaw + (size_t)((gb0 + 3) % NS) * RAWB) : sS + 64 * (TC_NMAX + 1);
#pragma unroll
      for (int i = 0; i < 32; i++)
        if (i < ew) (m < 64 ? sG + m * xstride : sU + (m - 64) * xstride)[ecol0 + i] = total[i];
      tc_workers_sync();
      const pm_layer_desc &D = ly.desc;
      const bool fold = !A.shared && D.weight_fold == PM_FOLD_BEFORE_DOWN && A.wts;
      const bool bias = !A.shared && ly.bias_gate;
      if (!dead)
        for (int i = tid; i < nvalid * 64; i += TC_NW) {
          int j = i & 63, n = i >> 6;
          if (r0 + j >= rows) continue;
          float gv = sG[j * xstride + n], uv = sU[j * xstride + n];
          if (bias) {
            gv = __fadd_rn(gv, ly.bias_gate[(size_t)el * rows + r0 + j]);
            uv = __fadd_rn(uv, ly.bias_up[(size_t)el * rows + r0 + j]);
          }
          uint32_t p = off + n0 + n;
          float w = fold ? A.wts[A.g.pair_src[p]] : 1.0f;
          A.out[(size_t)p * rows + r0 + j] = pm_act(D.act, D.act_limit, D.act_alpha, gv, uv, w, fold);
        }
      __syncwarp();
      if (PERSIST && (tid & 31) == 0) tc_mbar_arrive(epi_done);  // this warp has read the exchange area
    }
    TC_STAMP(30, 3)
    if (!next_item()) break;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == TC_NW / 32)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TC_TMEM_COLS) : "memory");
}

void launch_tc_tiles(const Launch &L, Groups g, int *n_tiles, uint32_t *tile_group, uint32_t *tile_n0, int max_tiles) {
  k_tc_tiles<<<1, 512, 0, L.stream>>>(g, n_tiles, tile_group, tile_n0, nullptr, nullptr, max_tiles);
  if (L.count) ++*L.count;
}

int tc_max_tiles(int n_pairs, int max_groups) {
  int groups = max_groups < n_pairs ? max_groups : n_pairs;
  return n_pairs / TC_NMAX + groups;
}
size_t tc_tile_words(int n_pairs, int max_groups) {
  return 4 + 3 * (size_t)tc_max_tiles(n_pairs, max_groups) + 512;
}
// bytes of the records of n_pairs rows of `cols` values in at most max_groups groups (every group
// starts on a multiple of 16 rows)
size_t tc_rec_bytes(int n_pairs, int max_groups, int cols) {
  size_t groups = (size_t)(max_groups < n_pairs ? max_groups : n_pairs);
  size_t rows = (size_t)n_pairs + 15 * groups + 16;
  return (rows / 8 + 1) * (size_t)(cols / 256) * TC_REC;
}
static size_t tc_smem(bool q6) {
  size_t raw = q6 ? (size_t)TC_RAW_STAGES_Q6 * TC_RAW_Q6 : (size_t)TC_RAW_STAGES_Q4 * TC_RAW_Q4;
  size_t ex = (size_t)TC_M * (TC_NMAX + 1) * 4;  // the gate/up exchange shares the raw areas' memory
  return (raw > ex ? raw : ex) + 3 * (size_t)(TC_NMAX / 8) * TC_REC + 2 * 2 * TC_M * 16 + 16 * 8 + 16 + 16;
}

// Tensor-core form of launch_gateup / launch_down for Q4_K or Q6_K weights and Q8x
// activations (xbm: the f16 form of the sub-block sums the quantiser writes): the tile list,
// the activation rows regrouped into records (rec_buf: tc_rec_bytes), the products.
// src_row: row of xq / xd / xbm / xs that holds pair p (null: row p itself).
cudaError_t launch_tc_q4k(const Launch &L, const LayerDev &ly, bool shared, bool down, Groups g,
                          int n_pairs, uint32_t *tile_buf, uint8_t *rec_buf, const uint32_t *src_row,
                          const int8_t *xq, const float *xd, const uint16_t *xbm, const int32_t *xs,
                          const float *wts, float *out, int *err, unsigned long long wait_ns, int fault_block) {
  if (n_pairs == 0) return cudaSuccess;
  // tile list: at most one partial tile per group plus the full ones
  const int max_tiles = tc_max_tiles(n_pairs, g.max_groups);
  int *n_tiles = (int *)tile_buf;
  uint32_t *tile_group = tile_buf + 4, *tile_n0 = tile_group + max_tiles, *tile_r0 = tile_n0 + max_tiles;
  uint32_t *group_r0 = tile_r0 + max_tiles;
  k_tc_tiles<<<1, 512, 0, L.stream>>>(g, n_tiles, tile_group, tile_n0, tile_r0, group_r0, max_tiles);
  if (L.count) ++*L.count;
  const WMat &W = down ? (shared ? ly.sdown : ly.down) : (shared ? ly.sgate : ly.gate);
  const bool q6 = W.type == PM_TYPE_Q6_K;
  {
    const int groups = g.max_groups < n_pairs ? g.max_groups : n_pairs;
    const long units = ((long)n_pairs / 8 + 2 * groups) * (W.cols / 256);  // (row group, block) records in all
    long gx = units / groups / 32;  // a warp writes a few records
    gx = gx < 1 ? 1 : (gx > 128 ? 128 : gx);
    k_tc_rows<<<dim3((unsigned)gx, (unsigned)groups), 256, 0, L.stream>>>(g, group_r0, src_row, W.cols, xq, xd, xbm, xs, rec_buf);
    if (L.count) ++*L.count;
  }
  const size_t smem = tc_smem(q6);
  const int row_tiles = down ? (W.rows + TC_M - 1) / TC_M : (W.rows + 63) / 64;
  // Down tiles: one persistent CTA an SM. An item is short (ff / 256 blocks) and the next item's
  // operands arrive during an item's last fold and its output writes: 20 % faster at ff 768
  // (128 experts, 512 tokens), 6 % at ff 2048.
  // Gate/up tiles of more than 64 tokens on average: a CTA an item. Their exchange of gate and up sums
  // fills the raw areas, so the next item's weights cannot be fetched early; run persistently they
  // measured no faster (d 2048) or 9 % slower (d 7168) - also with the items drawn from a counter in
  // global memory instead of a fixed share per CTA, and with the up sums exchanged through an area
  // of their own. Smaller gate/up tiles exchange through two of the four raw areas and run
  // persistently too (the producer is two blocks into the next item during an item's epilogue): 9 %
  // faster at 32 tokens an expert.
  const long items = (long)row_tiles * max_tiles;
  // tiles of at most 64 tokens on average: the instantiation with two accumulator sets (its larger
  // register footprint costs wider tiles 4 %), and gate/up persistent as well
  // (the experts that can have pairs: under expert parallelism the plan holds this rank's only)
  const int n_groups = shared ? 1 : (g.max_groups < ly.n_local ? g.max_groups : ly.n_local);
  const bool small = (long)n_pairs <= 64L * (n_groups < n_pairs ? n_groups : n_pairs);
  const bool persist = items > L.n_sm && (down || small);
  const void *kern;
  if (q6) {
    kern = !down ? (small ? (persist ? (const void *)k_tc<PM_TYPE_Q6_K, true, false, true> : (const void *)k_tc<PM_TYPE_Q6_K, false, false, true>)
                          : (const void *)k_tc<PM_TYPE_Q6_K, false, false, false>)
           : small ? (persist ? (const void *)k_tc<PM_TYPE_Q6_K, true, true, true> : (const void *)k_tc<PM_TYPE_Q6_K, false, true, true>)
                   : (persist ? (const void *)k_tc<PM_TYPE_Q6_K, true, true, false> : (const void *)k_tc<PM_TYPE_Q6_K, false, true, false>);
  } else {
    kern = !down ? (small ? (persist ? (const void *)k_tc<PM_TYPE_Q4_K, true, false, true> : (const void *)k_tc<PM_TYPE_Q4_K, false, false, true>)
                          : (const void *)k_tc<PM_TYPE_Q4_K, false, false, false>)
           : small ? (persist ? (const void *)k_tc<PM_TYPE_Q4_K, true, true, true> : (const void *)k_tc<PM_TYPE_Q4_K, false, true, true>)
                   : (persist ? (const void *)k_tc<PM_TYPE_Q4_K, true, true, false> : (const void *)k_tc<PM_TYPE_Q4_K, false, true, false>);
  }
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  TcArgs A;
  A.ly = ly;
  A.shared = shared;
  A.down = down;
  A.g = g;
  A.rec = rec_buf;
  A.wts = wts;
  A.out = out;
  A.err = err;
  A.wait_ns = wait_ns;
  A.fault_block = fault_block;
  A.n_tiles = n_tiles;
  A.tile_group = tile_group;
  A.tile_n0 = tile_n0;
  A.tile_r0 = tile_r0;
  A.row_tiles = row_tiles;
  void *args[] = {&A};
  e = cudaLaunchKernel(kern, persist ? dim3(L.n_sm) : dim3(row_tiles, max_tiles), dim3(TC_NT), args, smem, L.stream);
  if (e != cudaSuccess) return e;
  if (L.count) ++*L.count;
  return cudaGetLastError();
}
