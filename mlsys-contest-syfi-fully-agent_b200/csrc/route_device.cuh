// Device functions shared by the routing kernels and the decode-fused GEMM kernel:
// DeepSeek-V3 no-aux routing of one token by one warp (definition
// full-agent-pipeline/references/moe.py:123-158; replaces route_kernel,
// moe/solution/cuda/moe.cu:60-186) and the split-K choice.
#pragma once
#include "kernels.h"

namespace moe {

__device__ __forceinline__ uint32_t order_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Routes token t with the calling warp.  On return lanes 0..7 hold the selected
// global expert (descending biased score) and its combination weight.
__device__ __forceinline__ void route_token(const float* __restrict__ logits_row, const float* bias_smem,
                                            float routed_scaling_factor, int lane, int& sel_idx, float& sel_w) {
  float s[kNGroup];
  uint32_t key[kNGroup];
#pragma unroll
  for (int g = 0; g < kNGroup; ++g) {
    const float x = logits_row[g * 32 + lane];
    s[g] = 1.0f / (1.0f + expf(-x));
    key[g] = order_key(s[g] + bias_smem[g * 32 + lane]);
  }
  // group score = sum of the two largest biased scores of the group
  float gscore[kNGroup];
#pragma unroll
  for (int g = 0; g < kNGroup; ++g) {
    const uint32_t k1 = __reduce_max_sync(0xFFFFFFFFu, key[g]);
    const uint32_t who = __ballot_sync(0xFFFFFFFFu, key[g] == k1);
    const int first = __ffs(who) - 1;
    const uint32_t k2 = __reduce_max_sync(0xFFFFFFFFu, lane == first ? 0u : key[g]);
    // undo the order-preserving map
    const uint32_t u1 = (k1 & 0x80000000u) ? (k1 & 0x7FFFFFFFu) : ~k1;
    const uint32_t u2 = (k2 & 0x80000000u) ? (k2 & 0x7FFFFFFFu) : ~k2;
    gscore[g] = __uint_as_float(u1) + __uint_as_float(u2);
  }
  // keep the 4 best groups (ties: lower group index first)
  uint32_t keep = 0;
#pragma unroll
  for (int g = 0; g < kNGroup; ++g) {
    int rank = 0;
#pragma unroll
    for (int h = 0; h < kNGroup; ++h) rank += (gscore[h] > gscore[g]) || (gscore[h] == gscore[g] && h < g);
    keep |= (rank < kTopKGroup ? 1u : 0u) << g;
  }
  // 8 rounds of warp-wide arg-max over the kept candidates (ties: lower expert index first)
  uint32_t avail = keep;
  sel_idx = -1;
  float sel_s = 0.0f;
#pragma unroll
  for (int r = 0; r < kTopK; ++r) {
    uint32_t bk = 0;
    int bg = 0;
#pragma unroll
    for (int g = kNGroup - 1; g >= 0; --g) {
      const bool ok = (avail >> g) & 1u;
      if (ok && key[g] >= bk) { bk = key[g]; bg = g; }   // descending g with >= keeps the lowest g on ties
    }
    const bool has = avail != 0;
    const uint32_t kmax = __reduce_max_sync(0xFFFFFFFFu, has ? bk : 0u);
    const uint32_t cand = (has && bk == kmax) ? static_cast<uint32_t>(bg * 32 + lane) : 0xFFFFFFFFu;
    const uint32_t win = __reduce_min_sync(0xFFFFFFFFu, cand);
    const int wl = win & 31, wg = win >> 5;
    float sv = 0.0f;
#pragma unroll
    for (int g = 0; g < kNGroup; ++g) sv = (g == wg) ? s[g] : sv;
    sv = __shfl_sync(0xFFFFFFFFu, sv, wl);
    if (lane == wl) avail &= ~(1u << wg);
    if (lane == r) { sel_idx = static_cast<int>(win); sel_s = sv; }
  }
  // weights: s / (sum of the 8 selected s + 1e-20) * factor  (references/moe.py:154-158)
  float sum = 0.0f;
#pragma unroll
  for (int k = 0; k < kTopK; ++k) sum += __shfl_sync(0xFFFFFFFFu, sel_s, k);
  sum += 1e-20f;
  sel_w = (sel_s / sum) * routed_scaling_factor;
}

// Split-K factor of a grouped GEMM, one candidate per lane.  `tiles` equal (expert, weight tile,
// token tile) units, each with `kb_total` K-blocks that can only be cut at multiples of `kps`
// (one pipeline stage), run on `ctas` persistent CTAs that take items round-robin.  The estimated
// makespan of S splits is  waves(S) x (longest item in K-blocks + a fixed per-item cost of about two
// K-blocks: decode, scale table, result store);  the smallest S with the least makespan wins,
// subject to the slab capacity S * n_sel_pad <= slab_rows.
__device__ __forceinline__ int choose_split_warp(int tiles, int max_split, int ctas, int n_sel_pad, int slab_rows,
                                                 int lane, int kb_total, int kps) {
  if (tiles <= 0) return 1;
  const int S = lane + 1;
  const int units = kb_total / kps;
  int cost = 0x7FFFFFFF;
  if (S <= max_split && S <= units && static_cast<long long>(S) * n_sel_pad <= slab_rows) {
    const int items = tiles * S;
    const int waves = (items + ctas - 1) / ctas;
    const int longest = ((units + S - 1) / S) * kps;
    cost = waves * (longest + 2);
  }
  int best = 1, best_cost = 0x7FFFFFFF;
  for (int k = 0; k < max_split; ++k) {
    const int c = __shfl_sync(0xFFFFFFFFu, cost, k);
    if (c < best_cost) { best_cost = c; best = k + 1; }
  }
  return best;
}

}  // namespace moe
