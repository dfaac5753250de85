// prefill_mx.cu - grouped expert products for many tokens per expert on MXFP4 weights and
// f32 activations (the gpt-oss path, src/oss_prefill.rs:237,548) on the 5th-gen tensor cores:
// tcgen05.mma kind::f16 with bf16 operands, f32 accumulators in tensor memory.
//
// MXFP4 weights are exact in bf16 (a one-bit mantissa times a power of two: the E2M1 code
// doubled, times the halved E8M0 scale, src/oss_kernels.rs:41-55), the f32 activations are
// not: each is split x = hi + lo into two bf16 values (lo = bf16(x - hi)) by a small kernel
// before the products, and every K step runs twice, W * hi and W * lo, into the same
// accumulator. Products of two bf16 values are exact in f32, so what differs from the f32
// reference path (src/oss_batch.rs:774-789) is the 2^-17 relative residue of the split and
// the summation order: parity is the layer tolerance (1e-3 relative + 1e-4 of the RMS), not bits.
//
// One CTA = (128 weight rows of one active expert: 64 gate + 64 up, or 128 down rows) x
// (up to 128 of its tokens): 16 worker warps and one warp that issues the products. K runs
// in chunks of 64 values (two MXFP4 blocks) through a ring of MX_ST stages:
//   workers: the chunk's activations (bf16, gathered through the token list) arrive by
//            cp.async two chunks ahead; the chunk's weight nibbles and scale bytes arrive in
//            registers one chunk ahead, are decoded to bf16 and stored as operand A in the
//            canonical K-major layout ([8 K-chunks][128 rows][16 B]);
//   issuer:  waits for the stage (named barrier), runs 4 K steps x (hi, lo) products and
//            commits them to the stage's mbarrier, which the workers wait on before they
//            refill that stage.
// One accumulator for the whole K (the block scale lives in the bf16 weight), so there is no
// per-block float step as in the exact integer kernels. Epilogue: bias + GLU (gate/up,
// src/oss_prefill.rs:339) or bias (down; the routing weight is applied at combine,
// src/oss_prefill.rs:342). Waits are time-bounded; tensor memory is freed on every path.
#include <cuda_bf16.h>

#include "moe_internal.cuh"

#define MX_NW 512
#define MX_NT (MX_NW + 32)
#define MX_M 128
#define MX_NMAX 128
#define MX_KC 64            /* K values per stage */
#define MX_ST 4             /* stages */
#define MX_TMEM_COLS 128
#define MX_A_BYTES (8 * MX_M * 16)                 /* operand A of a stage */
#define MX_B_BYTES (8 * (MX_NMAX + 1) * 16)        /* one of the two B operands of a stage (odd pitch) */
#define MX_STAGE (MX_A_BYTES + 2 * MX_B_BYTES)

__device__ __forceinline__ uint32_t mx_s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long mx_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// shared-memory matrix descriptor, K-major, no swizzle: 8x16 B core matrices,
// lbo = bytes between the two 16-byte K chunks of one product, sbo = bytes between 8-row groups
__device__ __forceinline__ uint64_t mx_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)((lbo >> 4) & 0x3fff) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3fff) << 32) | (1ull << 46);
}
__device__ __forceinline__ void mx_mma(uint32_t tmem_c, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n" ::"r"(tmem_c),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void mx_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mx_s32(bar))
               : "memory");
}
__device__ __forceinline__ void mx_ld8(uint32_t taddr, uint32_t r[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}
__device__ __forceinline__ void mx_cp16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ bool mx_bar_test(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(mx_s32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// false after the wait limit (or at once when an error is already recorded)
__device__ __noinline__ bool mx_bar_wait(uint64_t *bar, uint32_t parity, int *err, unsigned long long wait_ns) {
  unsigned long long t0 = mx_now();
  for (uint32_t it = 0;; it++) {
    if (mx_bar_test(bar, parity)) return true;
    if ((it & 15) == 15 && (*(volatile int *)err != 0 || mx_now() - t0 > wait_ns)) break;
  }
  atomicCAS(err, 0, 8);
  return false;
}

// x -> (hi, lo) bf16 with hi + lo = x up to 2^-17 relative
__global__ void __launch_bounds__(256) k_split_bf16(const float *__restrict__ x, size_t n, __nv_bfloat16 *hi,
                                                    __nv_bfloat16 *lo) {
  size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const float v = x[i];
  const __nv_bfloat16 h = __float2bfloat16_rn(v);
  hi[i] = h;
  lo[i] = __float2bfloat16_rn(__fsub_rn(v, __bfloat162float(h)));
}
void launch_split_bf16(const Launch &L, const float *x, size_t n, void *hi, void *lo) {
  if (n == 0) return;
  k_split_bf16<<<(unsigned)((n + 255) / 256), 256, 0, L.stream>>>(x, n, (__nv_bfloat16 *)hi, (__nv_bfloat16 *)lo);
  if (L.count) ++*L.count;
}

// Four E2M1 codes (one in the low nibble of each byte of c4) -> the four bf16 patterns of
// code * 2^(e-128), as two words (codes 0,1 and 2,3), by byte-table look-ups (prmt): the low
// and the high byte of the offset {0, 0, 128, 192, 256, 320, 384, 448}[m] that magnitude m adds to
// the scale's own pattern `base2` ((e - 1) << 7 in both halves), the sign into bit 15, and a
// mask that zeroes the lanes with m = 0.
__device__ __forceinline__ void mx_decode4(uint32_t c4, uint32_t base2, uint32_t &w01, uint32_t &w23) {
  const uint32_t m = c4 & 0x07070707u;
  const uint32_t sel = (m & 0x7u) | ((m >> 4) & 0x70u) | ((m >> 8) & 0x700u) | ((m >> 12) & 0x7000u);
  const uint32_t lo = __byte_perm(0xc0800000u, 0xc0804000u, sel);
  const uint32_t hi = __byte_perm(0x00000000u, 0x01010101u, sel);
  const uint32_t nz = __byte_perm(0xffffff00u, 0xffffffffu, sel);
  const uint32_t hs = hi | ((c4 & 0x08080808u) << 4);
  const uint32_t d01 = __byte_perm(lo, hs, 0x5140), d23 = __byte_perm(lo, hs, 0x7362);
  w01 = (d01 + base2) & __byte_perm(nz, nz, 0x1100);
  w23 = (d23 + base2) & __byte_perm(nz, nz, 0x3322);
}

// Compile with -DPM_MX_TRACE to stamp the phases of CTA (0, 0) with the SM clock:
// [worker thread 0 | issuing thread][chunk][stamp]; read back with pm_debug_mx_trace.
#ifdef PM_MX_TRACE
__device__ unsigned long long g_mx_trace[2 * 64 * 8];
#define MX_STAMP(who, kc, i)                                                                   \
  if (blockIdx.x == 0 && blockIdx.y == 0 && (kc) < 64) g_mx_trace[(((who) * 64) + (kc)) * 8 + (i)] = clock64();
extern "C" __attribute__((visibility("default"))) int pm_debug_mx_trace(unsigned long long *out) {
  return (int)cudaMemcpyFromSymbol(out, g_mx_trace, sizeof(g_mx_trace));
}
#else
#define MX_STAMP(who, kc, i)
#endif

struct MxArgs {
  LayerDev ly;
  int down;               // 0: gate+up with activation -> h; 1: down -> pair outputs
  Groups g;
  const __nv_bfloat16 *xhi, *xlo;  // gate/up: [T][cols] by token; down: [P][cols] by pair
  const float *wts;       // routing weights [T*K] (gate/up with fold) or null
  float *out;             // gate/up: h [P][ff]; down: eo [P][d]
  int *err;
  unsigned long long wait_ns;
  const int *n_tiles;
  const uint32_t *tile_group, *tile_n0;
};

__global__ void __launch_bounds__(MX_NT, 1) k_tc_mx(const MxArgs A) {
  extern __shared__ __align__(128) uint8_t smem[];
  if ((int)blockIdx.y >= *A.n_tiles) return;
  const int a = (int)A.tile_group[blockIdx.y];
  const LayerDev &ly = A.ly;
  const WMat &W0 = A.down ? ly.down : ly.gate;
  const WMat &W1 = ly.up;
  const int cols = W0.cols, nb = cols / 32, rows = W0.rows;
  const int nkc = (cols + MX_KC - 1) / MX_KC;  // K chunks (the last one may hold a single block)
  const int e = (int)A.g.expert[a];
  const int el = e - ly.first_local;
  const uint32_t off = A.g.offset[a], cnt = A.g.count[a];
  const int n0 = (int)A.tile_n0[blockIdx.y];
  const int nvalid = min((int)cnt - n0, MX_NMAX);
  const int npad = (nvalid + 15) & ~15;
  const int tid = threadIdx.x, warp = tid >> 5;
  const bool local = el >= 0 && el < ly.n_local;
  const int rows_per_cta = A.down ? MX_M : MX_M / 2;
  const int r0 = blockIdx.x * rows_per_cta;
  if (!local) {  // an expert another rank holds: zeros (down) / nothing to do (gate/up)
    if (A.down)
      for (int i = tid; i < nvalid * MX_M; i += MX_NT) {
        int n = i / MX_M, m = i % MX_M;
        if (r0 + m < rows) A.out[(size_t)(off + n0 + n) * rows + r0 + m] = 0.0f;
      }
    return;
  }
  uint8_t *sStage = smem;                               // [MX_ST] x (A, B hi, B lo)
  float *sS = (float *)smem;                            // (after the last chunk) gate/up exchange [128][129]
  uint64_t *bar_empty = (uint64_t *)(smem + MX_ST * MX_STAGE);  // [MX_ST] products of a stage done
  uint64_t *bar_done = bar_empty + MX_ST;
  uint32_t *tmem_slot = (uint32_t *)(bar_done + 1);

  if (warp == MX_NW / 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(mx_s32(tmem_slot)),
                 "r"((uint32_t)MX_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    for (int i = 0; i <= MX_ST; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mx_s32(bar_empty + i)), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  const uint32_t sStage_a = mx_s32(sStage);
  const uint32_t bpitch = (uint32_t)(npad + 1) * 16u;

  if (warp == MX_NW / 32) {
    // ================= the issuing warp =================
    // instruction descriptor: D f32, A and B bf16, both K-major, N = npad, M = 128
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(npad >> 3) << 17) | ((uint32_t)(MX_M >> 4) << 24);
    const uint64_t da0 = mx_desc(sStage_a, MX_M * 16u, 128u);
    const uint64_t dbh0 = mx_desc(sStage_a + MX_A_BYTES, bpitch, 128u);
    for (int kc = 0; kc < nkc; kc++) {
      const int s = kc % MX_ST;
      // full[s]: named barrier 1 + s (workers arrive, this warp waits)
      asm volatile("bar.sync %0, %1;" ::"r"(1 + s), "n"(MX_NT) : "memory");
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if ((tid & 31) == 0) {
        MX_STAMP(1, kc, 0)
        // (descriptors of stage s, step ks = those of stage 0, step 0 plus the byte offset >> 4 in
        // the address field: shared memory addresses stay below 2^18)
        const uint32_t so = (uint32_t)s * MX_STAGE;
        const int ksteps = min(4, (cols - kc * MX_KC) / 16);  // (a trailing single block: 2 steps)
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
          if (ks < ksteps) {
            const uint64_t da = da0 + ((so + (uint32_t)(2 * ks) * (MX_M * 16u)) >> 4);
            const uint64_t dbh = dbh0 + ((so + (uint32_t)(2 * ks) * bpitch) >> 4);
            const uint64_t dbl = dbh + (MX_B_BYTES >> 4);
            mx_mma(tmem, da, dbh, idesc, (kc > 0 || ks > 0) ? 1u : 0u);
            mx_mma(tmem, da, dbl, idesc, 1u);
          }
        }
        mx_commit(&bar_empty[s]);
        if (kc == nkc - 1) mx_commit(bar_done);
        MX_STAMP(1, kc, 1)
      }
      __syncwarp();
    }
  } else {
    // ================= the workers =================
    // B: thread = (token t of the tile, K chunk c of 8 values): 2 x 16 B a stage (hi, lo);
    // 128 tokens x 8 chunks = 1024 pieces, two a thread
    int brow[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int t = (tid >> 3) + 64 * i;
      brow[i] = t < nvalid ? (A.down ? (int)(off + n0 + t) : (int)A.g.pair_token[off + n0 + t]) : -1;
    }
    const int bc = tid & 7;
    // (through registers: 16-byte cp.async moves about 21 bytes a cycle per SM, a chunk's 32 KB of
    // activations would take three times as long as its products)
    uint4 breg[4];
    auto load_b = [&](int kc) {  // the tokens' chunk kc -> registers
      const int k0 = kc * MX_KC + 8 * bc;
      const bool on = kc < nkc && k0 < cols;
#pragma unroll
      for (int i = 0; i < 2; i++) {
        if (on && brow[i] >= 0) {
          breg[2 * i] = __ldg((const uint4 *)(A.xhi + (size_t)brow[i] * cols + k0));
          breg[2 * i + 1] = __ldg((const uint4 *)(A.xlo + (size_t)brow[i] * cols + k0));
        }
      }
    };
    auto store_b = [&](int kc) {  // registers -> chunk kc's stage
      if (kc >= nkc) return;
      uint8_t *sb = sStage + (size_t)(kc % MX_ST) * MX_STAGE + MX_A_BYTES;
      if (kc * MX_KC + 8 * bc >= cols) return;
#pragma unroll
      for (int i = 0; i < 2; i++) {
        if (brow[i] < 0) continue;
        const int t = (tid >> 3) + 64 * i;
        uint8_t *dst = sb + (size_t)bc * bpitch + (size_t)t * 16;
        *(uint4 *)dst = breg[2 * i];
        *(uint4 *)(dst + MX_B_BYTES) = breg[2 * i + 1];
      }
    };
    // padding tokens (and, in a trailing half chunk, the missing K): zero operands, once
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int t = (tid >> 3) + 64 * i;
      if (t >= nvalid && t < npad)
        for (int st = 0; st < MX_ST; st++) {
          uint8_t *sb = sStage + (size_t)st * MX_STAGE + MX_A_BYTES;
          *(uint4 *)(sb + (size_t)bc * bpitch + (size_t)t * 16) = make_uint4(0, 0, 0, 0);
          *(uint4 *)(sb + MX_B_BYTES + (size_t)bc * bpitch + (size_t)t * 16) = make_uint4(0, 0, 0, 0);
        }
    }
    // A: thread = (row m of the tile, quarter q of the chunk): block b2 = q >> 1 of the chunk's
    // two, bytes 8 h .. 8 h + 7 of its 16 (h = q & 1): values 8 h + i (low nibbles) -> K chunk
    // 4 b2 + h, values 16 + 8 h + i (high nibbles) -> K chunk 4 b2 + 2 + h
    const int m = tid & 127, q = tid >> 7, b2 = q >> 1, hh = q & 1;
    const bool second = !A.down && m >= 64;  // the row belongs to the up matrix
    const int grow = r0 + (second ? m - 64 : m);
    const bool rvalid = grow < rows;
    const WMat &W = second ? W1 : W0;
    const uint8_t *nibp = W.plane[0] + (size_t)el * W.stride[0] + (size_t)(rvalid ? grow : 0) * nb * 16 + 8 * hh;
    const uint8_t *sclp = W.plane[1] + (size_t)el * W.stride[1] + (size_t)(rvalid ? grow : 0) * nb;
    uint2 raw = make_uint2(0, 0);
    uint32_t rsc = 0;
    auto load_a = [&](int kc) {  // chunk kc's bytes of this thread -> registers
      const int blk = 2 * kc + b2;
      if (kc < nkc && rvalid && blk < nb) {
        raw = __ldg((const uint2 *)(nibp + (size_t)blk * 16));
        rsc = __ldg(sclp + blk);
      } else {
        raw = make_uint2(0, 0);
        rsc = 0;
      }
    };
    auto store_a = [&](int kc, const uint2 raw, const uint32_t rsc) {  // (the bytes loaded one chunk earlier)
      uint8_t *sa = sStage + (size_t)(kc % MX_ST) * MX_STAGE;
      // (e < 2, the scale's own subnormal branch, src/oss_kernels.rs:42-45, and scales near the top of the range: decoded through f32)
      uint32_t lo4[4], hi4[4];
      if ((rsc >= 2u && rsc < 250u) || (raw.x | raw.y) == 0u) {
        const uint32_t base2 = ((rsc - 1u) << 7) * 0x00010001u;
        mx_decode4(raw.x, base2, lo4[0], lo4[1]);
        mx_decode4(raw.y, base2, lo4[2], lo4[3]);
        mx_decode4(raw.x >> 4, base2, hi4[0], hi4[1]);
        mx_decode4(raw.y >> 4, base2, hi4[2], hi4[3]);
      } else {
        const float s = pm_e8(rsc);
        const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
        for (int j = 0; j < 2; j++)
#pragma unroll
          for (int p = 0; p < 2; p++) {
            const uint32_t b0 = (w[j] >> (16 * p)) & 0xffu, b1 = (w[j] >> (16 * p + 8)) & 0xffu;
            auto cv = [&](uint32_t c) { return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(__fmul_rn(s, pm_e2m1(c)))); };
            lo4[2 * j + p] = cv(b0 & 15u) | (cv(b1 & 15u) << 16);
            hi4[2 * j + p] = cv(b0 >> 4) | (cv(b1 >> 4) << 16);
          }
      }
      *(uint4 *)(sa + (size_t)(4 * b2 + hh) * (MX_M * 16) + (size_t)m * 16) = make_uint4(lo4[0], lo4[1], lo4[2], lo4[3]);
      *(uint4 *)(sa + (size_t)(4 * b2 + 2 + hh) * (MX_M * 16) + (size_t)m * 16) = make_uint4(hi4[0], hi4[1], hi4[2], hi4[3]);
    };

    // chunk 0's activations directly, chunk 1's and the weight bytes of chunk 0 in registers
    // (one chunk ahead: two chunks ahead, with twice the registers, measured slower)
    load_b(0);
    store_b(0);
    load_b(1);
    load_a(0);
    bool dead = false;
    for (int kc = 0; kc < nkc; kc++) {
      const int s = kc % MX_ST;
      if (tid == 0) { MX_STAMP(0, kc, 0) }
      // chunk kc + 1's activations (in registers since the last round) go to the stage that held
      // chunk kc + 1 - MX_ST: its products must be done
      if (kc + 1 >= MX_ST && kc + 1 < nkc) {
        const int kp = kc + 1 - MX_ST;  // (completion number kp / MX_ST of that stage's barrier)
        if (!dead && !mx_bar_wait(&bar_empty[kp % MX_ST], (uint32_t)((kp / MX_ST) & 1), A.err, A.wait_ns)) dead = true;
      }
      if (tid == 0) { MX_STAMP(0, kc, 1) }
      store_b(kc + 1);
      load_b(kc + 2);
      if (tid == 0) { MX_STAMP(0, kc, 2) }
      // this chunk's own stage held chunk kc - MX_ST: waited for in the last round (as kc + 1 then).
      // The next chunk's weight bytes are requested before this chunk's are decoded.
      const uint2 raw_now = raw;
      const uint32_t rsc_now = rsc;
      load_a(kc + 1);
      store_a(kc, raw_now, rsc_now);
      if (tid == 0) { MX_STAMP(0, kc, 3) }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("bar.arrive %0, %1;" ::"r"(1 + s), "n"(MX_NT) : "memory");
      if (tid == 0) { MX_STAMP(0, kc, 5) }
    }
    // ---- epilogue: all products done -> TMEM lane m, a quarter of the token columns ----
    if (!mx_bar_test(bar_done, 0)) mx_bar_wait(bar_done, 0, A.err, A.wait_ns);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tlane = tmem + ((uint32_t)(32 * (warp & 3)) << 16);
    const int part = tid >> 7;
    const int ew = npad >> 2, ecol0 = part * ew;  // npad / 4 columns: a multiple of 4
    float total[32];
#pragma unroll
    for (int c8 = 0; c8 < 32; c8 += 8) {
      if (c8 < ew) {
        uint32_t v[8];
        // (ew is a multiple of 4: the second half of an 8-wide read may lie past this quarter; it is ignored below)
        mx_ld8(tlane + (uint32_t)(ecol0 + c8), v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int u = 0; u < 8; u++) total[c8 + u] = __uint_as_float(v[u]);
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    asm volatile("bar.sync 6, %0;" ::"n"(MX_NW) : "memory");  // the stages are dead: their memory carries the exchange
    const bool bad = *(volatile int *)A.err != 0;
    if (A.down) {
      if (!bad) {
        const float bd = (ly.bias_down && rvalid) ? ly.bias_down[(size_t)el * rows + grow] : 0.0f;
#pragma unroll
        for (int i = 0; i < 32; i++) {
          const int n = ecol0 + i;
          if (i < ew && n < nvalid && rvalid) {
            float o = total[i];
            if (ly.bias_down) o = __fadd_rn(o, bd);
            A.out[(size_t)(off + n0 + n) * rows + grow] = o;
          }
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; i++)
        if (i < ew) sS[m * (MX_NMAX + 1) + ecol0 + i] = total[i];
      asm volatile("bar.sync 6, %0;" ::"n"(MX_NW) : "memory");
      const pm_layer_desc &D = ly.desc;
      const bool fold = D.weight_fold == PM_FOLD_BEFORE_DOWN && A.wts;
      const bool bias = ly.bias_gate != nullptr;
      if (!bad)
        for (int i = tid; i < nvalid * 64; i += MX_NW) {
          const int j = i & 63, n = i >> 6;
          if (r0 + j >= rows) continue;
          float gv = sS[j * (MX_NMAX + 1) + n], uv = sS[(64 + j) * (MX_NMAX + 1) + n];
          if (bias) {
            gv = __fadd_rn(gv, ly.bias_gate[(size_t)el * rows + r0 + j]);
            uv = __fadd_rn(uv, ly.bias_up[(size_t)el * rows + r0 + j]);
          }
          const uint32_t p = off + n0 + n;
          const float w = fold ? A.wts[A.g.pair_src[p]] : 1.0f;
          A.out[(size_t)p * rows + r0 + j] = pm_act(D.act, D.act_limit, D.act_alpha, gv, uv, w, fold);
        }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == MX_NW / 32)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)MX_TMEM_COLS) : "memory");
}

int tc_max_tiles(int n_pairs, int max_groups);
void launch_tc_tiles(const Launch &L, Groups g, int *n_tiles, uint32_t *tile_group, uint32_t *tile_n0, int max_tiles);

// Tensor-core form of launch_gateup / launch_down for MXFP4 weights and f32 activations given
// as their bf16 (hi, lo) split.
cudaError_t launch_tc_mx(const Launch &L, const LayerDev &ly, bool down, Groups g, int n_pairs, uint32_t *tile_buf,
                         const void *xhi, const void *xlo, const float *wts, float *out, int *err,
                         unsigned long long wait_ns) {
  if (n_pairs == 0) return cudaSuccess;
  const int max_tiles = tc_max_tiles(n_pairs, g.max_groups);
  int *n_tiles = (int *)tile_buf;
  uint32_t *tile_group = tile_buf + 4, *tile_n0 = tile_buf + 4 + max_tiles;
  launch_tc_tiles(L, g, n_tiles, tile_group, tile_n0, max_tiles);
  const WMat &W = down ? ly.down : ly.gate;
  const size_t ex = (size_t)MX_M * (MX_NMAX + 1) * 4;
  const size_t smem = ((size_t)MX_ST * MX_STAGE > ex ? (size_t)MX_ST * MX_STAGE : ex) + 8 * (MX_ST + 1) + 16;
  cudaError_t e = cudaFuncSetAttribute((const void *)k_tc_mx, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  MxArgs A;
  A.ly = ly;
  A.down = down;
  A.g = g;
  A.xhi = (const __nv_bfloat16 *)xhi;
  A.xlo = (const __nv_bfloat16 *)xlo;
  A.wts = wts;
  A.out = out;
  A.err = err;
  A.wait_ns = wait_ns;
  A.n_tiles = n_tiles;
  A.tile_group = tile_group;
  A.tile_n0 = tile_n0;
  const int row_tiles = down ? (W.rows + MX_M - 1) / MX_M : (W.rows + 63) / 64;
  dim3 grid(row_tiles, max_tiles);
  k_tc_mx<<<grid, MX_NT, smem, L.stream>>>(A);
  if (L.count) ++*L.count;
  return cudaGetLastError();
}
