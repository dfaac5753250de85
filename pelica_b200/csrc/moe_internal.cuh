// moe_internal.cuh - device-side descriptions shared by the kernels and the C ABI.
#pragma once

#include "common.cuh"

// One expert tensor family ([n_local experts][rows][cols]) in its device layout.
//  Q4_K : plane 0 = the GGUF blocks unchanged (144 B, 16-byte aligned rows)
//  Q6_K : plane 0 = ql (128 B/block), 1 = qh (64 B), 2 = scales (16 B),
//         3 = d (2 B): the block's four fields split into planes so every
//         field is aligned; 210 B/block in total, as stored (no padding)
//  MXFP4: plane 0 = E2M1 nibbles (16 B/block), 1 = E8M0 scale bytes (1 B/block)
//         (the reference splits gpt-oss tensors the same way, src/oss.rs:241-253)
//  Q8_0 : plane 0 = int8 values (32 B/block), 1 = f16 scales (2 B/block)
//  IQ4_NL: plane 0 = codebook indices (16 B/block), 1 = f16 scales (2 B/block)
//  IQ4_XS: plane 0 = codebook indices (128 B/block), 1 = the 8-byte header (f16 d, u16 high
//          scale bits, 4 bytes of low scale nibbles)
//  Q5_K : plane 0 = the GGUF blocks unchanged (176 B)
//  IQ3_S: plane 0 = qs, qh, signs, scales as stored (108 B/block), 1 = f16 d (2 B/block)
//  GLM_Q4: plane 0 = nibbles (32 B per group of 64), 1 = f32 group scales: the container's two regions
struct WMat {
  int type;
  int rows, cols;
  uint8_t *plane[4];
  size_t stride[4];  // bytes per expert in each plane
};

struct LayerDev {
  pm_layer_desc desc;
  int n_local, first_local;
  const float *router;       // [E][d]
  const float *logit_bias;   // [E] or null
  const float *select_bias;  // [E] or null
  WMat gate, up, down;
  const float *bias_gate, *bias_up, *bias_down;  // [n_local][ff|d] or null
  WMat sgate, sup, sdown;                        // shared expert (1 "expert")
  const float *shared_gate_inp;                  // [d] or null
  uint32_t *usage;                               // [E]
};

// pair_pos of a pair whose expert id was refused by the plan (combine reads a zero row)
#define PM_PAIR_NONE 0xffffffffu
// values of a context's device error word (0 = none; 1..99 = a bounded wait gave up)
#define PM_DEVERR_BAD_EXPERT_ID 100

// A grouping of pairs by expert (the dispatch plan, or the trivial one-group
// plan of the shared expert).
struct Groups {
  const int *n_groups;         // [1]
  const uint32_t *expert;      // [g] global expert id
  const uint32_t *offset;      // [g]
  const uint32_t *count;       // [g]
  const uint32_t *pair_token;  // [P]
  const uint32_t *pair_src;    // [P] index t*K+k of the pair (or null)
  int max_groups;
};

struct PlanDev {
  int *n_active;
  uint32_t *active, *offset, *count;  // [E]
  uint32_t *base;                     // [E] first pair of expert e
  uint32_t *cnt;                      // [E] scratch counters
  uint32_t *pair_token, *pair_pos, *pair_src;  // [P]
};

// bytes of one expert's tensor in plane p
static inline size_t wmat_plane_bytes(int type, int rows, int cols, int p) {
  size_t nb;
  switch (type) {
    case PM_TYPE_Q4_K:
      nb = (size_t)rows * (cols / 256);
      return p == 0 ? nb * 144 : 0;
    case PM_TYPE_Q6_K: {
      nb = (size_t)rows * (cols / 256);
      const size_t f[4] = {128, 64, 16, 2};
      return nb * f[p];
    }
    case PM_TYPE_MXFP4:
      nb = (size_t)rows * (cols / 32);
      return p == 0 ? nb * 16 : (p == 1 ? nb : 0);
    case PM_TYPE_Q8_0:
      nb = (size_t)rows * (cols / 32);
      return p == 0 ? nb * 32 : (p == 1 ? nb * 2 : 0);
    case PM_TYPE_IQ4_NL:
      nb = (size_t)rows * (cols / 32);
      return p == 0 ? nb * 16 : (p == 1 ? nb * 2 : 0);
    case PM_TYPE_IQ4_XS:
      nb = (size_t)rows * (cols / 256);
      return p == 0 ? nb * 128 : (p == 1 ? nb * 8 : 0);
    case PM_TYPE_Q5_K:
      nb = (size_t)rows * (cols / 256);
      return p == 0 ? nb * 176 : 0;
    case PM_TYPE_IQ3_S:
      nb = (size_t)rows * (cols / 256);
      return p == 0 ? nb * 108 : (p == 1 ? nb * 2 : 0);
    case PM_TYPE_GLM_Q4:
      nb = (size_t)rows * (cols / 64);
      return p == 0 ? nb * 32 : (p == 1 ? nb * 4 : 0);
  }
  return 0;
}

// ---- launchers (kernels_basic.cu) -----------------------------------------
struct Launch {
  cudaStream_t stream;
  int64_t *count;  // kernels launched
  int n_sm = 148;  // SMs of the device
};

void launch_repack(const Launch &L, int type, const uint8_t *raw, size_t n_blocks, uint8_t *p0,
                   uint8_t *p1, uint8_t *p2, uint8_t *p3);
void launch_unpack(const Launch &L, int type, uint8_t *raw, size_t n_blocks, const uint8_t *p0,
                   const uint8_t *p1, const uint8_t *p2, const uint8_t *p3);
void launch_dequant(const Launch &L, int type, size_t n_values, const uint8_t *p0,
                    const uint8_t *p1, const uint8_t *p2, const uint8_t *p3, float *out);
// bm (optional): per block 16 f16 values, 64 * (bsum_j >> 6) for the 8 sub-blocks, then
// bsum_j & 63: the operand the tensor-core kernel multiplies the Q4_K mins with;
// xs (optional): per block the sum of its 256 values (the Q6_K offset term)
void launch_quant_q8x(const Launch &L, const float *x, size_t rows, int n, int8_t *q, float *d,
                      int32_t *bsum, uint16_t *bm = nullptr, int32_t *xs = nullptr);
void launch_quant_q8_32(const Launch &L, const float *x, size_t rows, int n, int8_t *q, float *d, bool f16_scale);
void launch_router(const Launch &L, const LayerDev &ly, const float *x, int T, float *logits);
void launch_route(const Launch &L, const LayerDev &ly, const float *logits, int T, uint32_t *ids,
                  float *w);
// err: the context's error word (an expert id outside the layer is reported there, never used)
void launch_plan(const Launch &L, const LayerDev &ly, const uint32_t *ids, int T, PlanDev plan, int *err);
// router + top-k + plan of T < PM_SMALL_ROUTE_TOKENS tokens in one launch (ticket: a zeroed word the
// kernel leaves zeroed; slot_table: expert -> slot of an expert-parallel placement, or null)
#define PM_SMALL_ROUTE_TOKENS 8
void launch_route_plan_small(const Launch &L, const LayerDev &ly, const float *x, int T, float *logits, uint32_t *ids,
                             float *w, PlanDev pl, const int32_t *slot_table, unsigned int *ticket);
void launch_iota(const Launch &L, uint32_t *p, uint32_t n);
void launch_gateup(const Launch &L, const LayerDev &ly, bool shared, Groups g, int n_pairs,
                   const float *x, const int8_t *xq, const float *xd, const int32_t *xbsum,
                   const float *w, float *h);
void launch_down(const Launch &L, const LayerDev &ly, bool shared, Groups g, int n_pairs,
                 const float *h, const int8_t *hq, const float *hd, const int32_t *hbsum,
                 float *eo);
// tensor-core (tcgen05 int8) form of launch_gateup / launch_down for Q4_K x Q8x (prefill_tc.cu)
// tile_buf: tc_tile_words(n_pairs, g.max_groups) words of scratch for the tile list; rec_buf:
// tc_rec_bytes(n_pairs, g.max_groups, cols) bytes for the activation rows regrouped by expert in the
// products' layout; src_row: row of xq / xd / xbm / xs that holds pair p (null: row p itself)
int tc_max_tiles(int n_pairs, int max_groups);
size_t tc_tile_words(int n_pairs, int max_groups);
size_t tc_rec_bytes(int n_pairs, int max_groups, int cols);
cudaError_t launch_tc_q4k(const Launch &L, const LayerDev &ly, bool shared, bool down, Groups g,
                          int n_pairs, uint32_t *tile_buf, uint8_t *rec_buf, const uint32_t *src_row,
                          const int8_t *xq, const float *xd, const uint16_t *xbm, const int32_t *xs,
                          const float *wts, float *out, int *err, unsigned long long wait_ns, int fault_block);
// tensor-core (tcgen05 bf16) form for MXFP4 weights and f32 activations given as their bf16
// (hi, lo) split (prefill_mx.cu); launch_split_bf16 makes the split: hi[n], lo[n] bf16
void launch_split_bf16(const Launch &L, const float *x, size_t n, void *hi, void *lo);
cudaError_t launch_tc_mx(const Launch &L, const LayerDev &ly, bool down, Groups g, int n_pairs, uint32_t *tile_buf,
                         const void *xhi, const void *xlo, const float *wts, float *out, int *err,
                         unsigned long long wait_ns);
// expert parallelism (kernels_basic.cu): per-rank pair counts, the wire records of a dispatch,
// the received (expert, weight) records, the derived forms of received Q8x group sums
void launch_ep_slots(const Launch &L, uint32_t *ids, int P, int E, const int32_t *table, uint32_t *usage);
void launch_ep_rank_counts(const Launch &L, const uint32_t *cnt, int E, int W, int32_t *out);
void launch_ep_pack(const Launch &L, int P, int row_bytes, int nd, int nbs, const void *rows, const float *xd,
                    const int32_t *xbs, const uint32_t *pair_token, const uint32_t *pair_src, const uint32_t *ids,
                    const float *w, void *srows, float *sd, int32_t *sbs, uint32_t *smeta);
void launch_ep_unmeta(const Launch &L, int R, const uint32_t *meta, int first, int n_local, uint32_t *eids, float *w,
                      int *err);
void launch_q8x_aux(const Launch &L, size_t n_blocks, const int32_t *bsum, uint16_t *bm, int32_t *xs);
void launch_combine(const Launch &L, const LayerDev &ly, const float *eo, const uint32_t *pair_pos,
                    const float *w, const float *shared_out, const float *shared_logit, int T,
                    float *y, bool accumulate);
void launch_rmsnorm(const Launch &L, const float *x, int T, int d, float eps, float *out);
void launch_shared_gate_logit(const Launch &L, const LayerDev &ly, const float *x, int T,
                              float *out);
