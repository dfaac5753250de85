// placement.cu - usage-driven placement of experts over the ranks of an expert-parallel group.
//
// The reference keeps a decayed use score per (layer, expert), read from the counters its plan
// kernel bumps, and lets the experts used more than the least used resident ones change places with
// them, biggest gains first, up to a byte budget per round, with a margin so that experts do not go
// back and forth (src/moe.rs:246-278 `Adapt`, :1965-1995 `adapt`, :1997-2069 `swap_round`). Its two
// places are VRAM and host memory. Here every expert is resident on some GPU and the places are the
// ranks: what a round evens out is the sum of scores a rank serves, by swapping a much-used expert
// of the most loaded rank with a little-used one of the least loaded rank. Host code only: the
// scores come from pm_layer_usage, the swaps are carried out by pm_ep_swap_experts.
#include <algorithm>
#include <cstdint>
#include <vector>

#include "../../include/pelica_moe.h"

struct pm_placement {
  int n_layers, n_exp, world;
  std::vector<float> score;     // [layer][expert]
  std::vector<uint32_t> prev;   // the counters as last read
  std::vector<int32_t> slot;    // [layer][expert]: slot s lives on rank s / (n_exp / world)
  uint64_t moved = 0;           // experts moved so far
};

// how fast old use fades per observation, and the margin a swap must clear (src/moe.rs:272-273,2013)
static const float kDecay = 0.944f;
static inline bool clears_margin(float hot, float cold) { return !(hot < cold * 1.25f + 1.5f); }

extern "C" int32_t pm_placement_create(int32_t n_layers, int32_t n_exp, int32_t world, pm_placement **out) {
  if (!out || n_layers < 1 || n_exp < 1 || world < 1 || n_exp % world) return PM_ERR_INVALID;
  pm_placement *p = new pm_placement;
  p->n_layers = n_layers;
  p->n_exp = n_exp;
  p->world = world;
  p->score.assign((size_t)n_layers * n_exp, 0.0f);
  p->prev.assign((size_t)n_layers * n_exp, 0u);
  p->slot.resize((size_t)n_layers * n_exp);
  for (int l = 0; l < n_layers; l++)
    for (int e = 0; e < n_exp; e++) p->slot[(size_t)l * n_exp + e] = e;
  *out = p;
  return PM_OK;
}

extern "C" int32_t pm_placement_destroy(pm_placement *p) {
  delete p;
  return PM_OK;
}

// score = score * decay + (counter - counter as last read), per expert (src/moe.rs:1977-1980)
extern "C" int32_t pm_placement_observe(pm_placement *p, int32_t layer, const uint32_t *usage) {
  if (!p || !usage || layer < 0 || layer >= p->n_layers) return PM_ERR_INVALID;
  for (int e = 0; e < p->n_exp; e++) {
    const size_t i = (size_t)layer * p->n_exp + e;
    p->score[i] = p->score[i] * kDecay + (float)(uint32_t)(usage[e] - p->prev[i]);
    p->prev[i] = usage[e];
  }
  return PM_OK;
}

extern "C" int32_t pm_placement_slots(const pm_placement *p, int32_t layer, int32_t *slot_of_expert) {
  if (!p || !slot_of_expert || layer < 0 || layer >= p->n_layers) return PM_ERR_INVALID;
  std::copy(p->slot.begin() + (size_t)layer * p->n_exp, p->slot.begin() + (size_t)(layer + 1) * p->n_exp, slot_of_expert);
  return PM_OK;
}

extern "C" int32_t pm_placement_scores(const pm_placement *p, int32_t layer, float *score, float *rank_load) {
  if (!p || layer < 0 || layer >= p->n_layers) return PM_ERR_INVALID;
  const int per = p->n_exp / p->world;
  if (rank_load) std::fill(rank_load, rank_load + p->world, 0.0f);
  for (int e = 0; e < p->n_exp; e++) {
    const size_t i = (size_t)layer * p->n_exp + e;
    if (score) score[e] = p->score[i];
    if (rank_load) rank_load[p->slot[i] / per] += p->score[i];
  }
  return PM_OK;
}

namespace {
struct Cand {
  float gain;  // by how much the swap lowers the load of the heavier of the two ranks
  int layer, hot, cold;
};
}  // namespace

// One round. Per layer, repeatedly: the most and the least loaded rank; of the first one's experts
// that clear the margin against an expert of the second, the pair whose exchange leaves the smaller
// maximum of the two loads. The candidates of all layers are then taken biggest gain first while
// 2 * expert_bytes each fit the budget (src/moe.rs:2021-2035). The table is updated as if the chosen
// swaps had been carried out: the caller runs them (pm_ep_swap_experts) in the order returned.
extern "C" int32_t pm_placement_plan(pm_placement *p, uint64_t expert_bytes, uint64_t budget_bytes, int32_t *swaps,
                                 int32_t max_swaps, int32_t *n_swaps) {
  if (!p || !n_swaps || (max_swaps > 0 && !swaps)) return PM_ERR_INVALID;
  *n_swaps = 0;
  const int E = p->n_exp, W = p->world, per = E / W;
  if (W < 2) return PM_OK;
  std::vector<Cand> cands;
  for (int l = 0; l < p->n_layers; l++) {
    std::vector<int32_t> slot(p->slot.begin() + (size_t)l * E, p->slot.begin() + (size_t)(l + 1) * E);
    const float *sc = &p->score[(size_t)l * E];
    std::vector<float> load((size_t)W, 0.0f);
    for (int e = 0; e < E; e++) load[(size_t)(slot[(size_t)e] / per)] += sc[e];
    std::vector<char> used((size_t)E, 0);  // an expert moves at most once a round
    for (int iter = 0; iter < E; iter++) {
      int hi = 0, lo = 0;
      for (int r = 1; r < W; r++) {
        if (load[(size_t)r] > load[(size_t)hi]) hi = r;
        if (load[(size_t)r] < load[(size_t)lo]) lo = r;
      }
      if (hi == lo) break;
      const float gap = load[(size_t)hi] - load[(size_t)lo];
      int best_h = -1, best_c = -1;
      float best_max = load[(size_t)hi];
      for (int h = 0; h < E; h++) {
        if (used[(size_t)h] || slot[(size_t)h] / per != hi) continue;
        for (int cidx = 0; cidx < E; cidx++) {
          if (used[(size_t)cidx] || slot[(size_t)cidx] / per != lo) continue;
          if (!clears_margin(sc[h], sc[cidx])) continue;
          const float g = sc[h] - sc[cidx];
          if (g <= 0.0f || g >= gap) continue;  // would only trade places
          const float m = std::max(load[(size_t)hi] - g, load[(size_t)lo] + g);
          if (m < best_max) {
            best_max = m;
            best_h = h;
            best_c = cidx;
          }
        }
      }
      if (best_h < 0) break;
      const float g = sc[best_h] - sc[best_c];
      cands.push_back({load[(size_t)hi] - best_max, l, best_h, best_c});
      load[(size_t)hi] -= g;
      load[(size_t)lo] += g;
      std::swap(slot[(size_t)best_h], slot[(size_t)best_c]);
      used[(size_t)best_h] = used[(size_t)best_c] = 1;
    }
  }
  // the swaps of a layer were found in sequence (each assumes the ones before it): keep that order
  // inside a layer and let the layers compete by their first, largest gain
  std::stable_sort(cands.begin(), cands.end(), [](const Cand &a, const Cand &b) { return a.gain > b.gain; });
  std::vector<char> layer_closed((size_t)p->n_layers, 0);
  uint64_t moved = 0;
  int n = 0;
  // (within a layer gains fall monotonically as the loads even out, so the global order by gain keeps
  // every layer's sequence; a layer stops at its first swap that does not fit)
  for (const Cand &c : cands) {
    if (layer_closed[(size_t)c.layer]) continue;
    if (n >= max_swaps || moved + 2 * expert_bytes > budget_bytes) {
      layer_closed[(size_t)c.layer] = 1;
      continue;
    }
    moved += 2 * expert_bytes;
    swaps[3 * n] = c.layer;
    swaps[3 * n + 1] = c.hot;
    swaps[3 * n + 2] = c.cold;
    n++;
    std::swap(p->slot[(size_t)c.layer * E + c.hot], p->slot[(size_t)c.layer * E + c.cold]);
  }
  p->moved += (uint64_t)n;
  *n_swaps = n;
  return PM_OK;
}
