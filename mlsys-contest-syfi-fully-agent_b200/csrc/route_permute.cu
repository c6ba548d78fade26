// Routing, histogram, prefix sum and stable permutation.
//
// route: DeepSeek-V3 no-aux routing of one token per warp
//   (full-agent-pipeline/references/moe.py:123-158; replaces route_kernel,
//   moe/solution/cuda/moe.cu:60-186).  Lane l holds experts 32*g + l, so register
//   index g is routing group g and every group reduction is one warp-wide redux.
//   IEEE expf and division (this file is compiled without fast-math): selection
//   must agree with the definition bit for bit.
// permute: deterministic counting sort of (token, local expert) pairs: rows are in
//   ascending token order inside ascending local expert, the order torch.nonzero
//   gives the definition (references/moe.py:168-179).  Replaces scan_offsets_*_kernel
//   and the atomics-ordered perm_fill_kernel (moe.cu:217-309), and also builds the
//   split-K schedule on the device so that no regime needs a host round trip.
#include "kernels.h"

namespace moe {

namespace {

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

__device__ __forceinline__ void route_tokens_strided(const RouteArgs& a, const float* bias_smem, int first_token,
                                                     int token_stride, int lane) {
  for (int t = first_token; t < a.T; t += token_stride) {
    int idx;
    float w;
    route_token(a.logits + static_cast<size_t>(t) * kEGlobal, bias_smem, a.routed_scaling_factor, lane, idx, w);
    uint32_t bit = 0;
    if (lane < kTopK) {
      a.topk_idx[t * kTopK + lane] = idx;
      a.topk_w[t * kTopK + lane] = w;
      const int le = idx - a.local_expert_offset;
      if (le >= 0 && le < kELocal) bit = 1u << le;
    }
    bit = __reduce_or_sync(0xFFFFFFFFu, bit);
    if (lane == 0) a.local_mask[t] = bit;
  }
}

__device__ __forceinline__ void load_bias(const uint16_t* bias_bf16, float* bias_smem) {
  for (int i = threadIdx.x; i < kEGlobal; i += blockDim.x)
    bias_smem[i] = __uint_as_float(static_cast<uint32_t>(bias_bf16[i]) << 16);
}

// Best split-K factor for `tiles` equal work items on `ctas` persistent CTAs:
// the smallest S whose last wave is fullest (within 4 %), subject to the slab capacity.
__device__ int choose_split(int tiles, int max_split, int ctas, int n_sel_pad, int slab_rows) {
  if (tiles <= 0) return 1;
  int best = 1;
  float best_eff = 0.0f;
  for (int S = 1; S <= max_split; ++S) {
    if (static_cast<long long>(S) * n_sel_pad > slab_rows) break;
    const int items = tiles * S;
    const int waves = (items + ctas - 1) / ctas;
    const float eff = static_cast<float>(items) / static_cast<float>(waves * ctas);
    if (eff > best_eff * 1.04f) { best_eff = eff; best = S; }
  }
  return best;
}

// Best split-K factors, evaluated one candidate per lane.
__device__ int choose_split_warp(int tiles, int max_split, int ctas, int n_sel_pad, int slab_rows, int lane) {
  if (tiles <= 0) return 1;
  const int S = lane + 1;
  float eff = 0.0f;
  if (S <= max_split && static_cast<long long>(S) * n_sel_pad <= slab_rows) {
    const int items = tiles * S;
    const int waves = (items + ctas - 1) / ctas;
    eff = static_cast<float>(items) / static_cast<float>(waves * ctas);
  }
  // same rule as choose_split: walk S upwards, move on only for a > 4 % fuller last wave
  int best = 1;
  float best_eff = 0.0f;
  for (int k = 0; k < max_split; ++k) {
    const float e = __shfl_sync(0xFFFFFFFFu, eff, k);
    if (e > best_eff * 1.04f) { best_eff = e; best = k + 1; }
  }
  return best;
}

// Block-wide (1024 threads) histogram, scan, stable permutation and schedule.  Warp w owns
// the contiguous token range [w * span, (w + 1) * span); inside a 32-token chunk lane = token.
// Phase 1 counts, per warp and expert, the tokens that selected the expert; an exclusive
// scan over (expert, warp) then gives every warp its first row for every expert, and phase
// 2 fills rows in token order, so rows are ascending in token inside ascending expert.
// Requires the routing outputs of all T tokens to be visible.
__device__ void permute_block(const PermuteArgs& a) {
  __shared__ int s_wcount[32][kELocal + 1];     // [warp][expert]: count, then first row (+1: no bank conflicts)
  __shared__ int s_offs[kELocal + 1];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const uint32_t lt_mask = (1u << lane) - 1u;
  const int chunks = (a.T + 31) / 32;
  const int span = (chunks + 31) / 32;          // chunks per warp
  const int c0 = warp * span, c1 = min(chunks, c0 + span);

  // phase 1: lane le accumulates this warp's count for expert le
  int cnt = 0;
  for (int c = c0; c < c1; ++c) {
    const int t = c * 32 + lane;
    const uint32_t m = t < a.T ? a.local_mask[t] : 0u;
#pragma unroll
    for (int le = 0; le < kELocal; ++le) {
      const int n = __popc(__ballot_sync(0xFFFFFFFFu, (m >> le) & 1u));
      if (lane == le) cnt += n;
    }
  }
  s_wcount[warp][lane] = cnt;
  __syncthreads();
  if (warp == 0) {
    // lane = expert: totals over warps, exclusive scan over experts, per-warp first rows
    int c = 0;
    for (int w = 0; w < 32; ++w) c += s_wcount[w][lane];
    const int tiles = (c + a.n_tile - 1) / a.n_tile;
    int inc = c, tinc = tiles;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xFFFFFFFFu, inc, d);
      const int tv = __shfl_up_sync(0xFFFFFFFFu, tinc, d);
      if (lane >= d) { inc += v; tinc += tv; }
    }
    int run = inc - c;                          // first row of expert `lane`
    for (int w = 0; w < 32; ++w) {
      const int n = s_wcount[w][lane];
      s_wcount[w][lane] = run;
      run += n;
    }
    MoeSched* sc = a.sched;
    s_offs[lane + 1] = inc;
    sc->counts[lane] = c;
    sc->offs[lane + 1] = inc;
    sc->tile_prefix[lane + 1] = tinc;
    const uint32_t act = __ballot_sync(0xFFFFFFFFu, c > 0);
    const int n_sel = __shfl_sync(0xFFFFFFFFu, inc, 31), tiles_total = __shfl_sync(0xFFFFFFFFu, tinc, 31);
    const int n_sel_pad = (n_sel + 15) & ~15;
    const int s1 = choose_split_warp(tiles_total * kMT1, kMaxSplit1, a.ctas, n_sel_pad, a.slab_rows, lane);
    const int s2 = choose_split_warp(tiles_total * kMT2, kMaxSplit2, a.ctas, n_sel_pad, a.slab_rows, lane);
    if (lane == 31) {
      s_offs[0] = 0;
      sc->offs[0] = 0;
      sc->tile_prefix[0] = 0;
      sc->status = (n_sel > a.rows_cap) ? kErrSchedOverflow : 0;
      sc->n_sel = n_sel;
      sc->n_sel_pad = n_sel_pad;
      sc->n_active = __popc(act);
      sc->n_tile = a.n_tile;
      sc->tiles_total = tiles_total;
      sc->split1 = s1;
      sc->split2 = s2;
      sc->items1 = tiles_total * kMT1 * s1;
      sc->items2 = tiles_total * kMT2 * s2;
    }
  }
  __syncthreads();
  // phase 2: fill.  `base` (lane = expert) is this warp's next free row of each expert.
  int base = s_wcount[warp][lane];
  for (int c = c0; c < c1; ++c) {
    const int t = c * 32 + lane;
    const uint32_t m = t < a.T ? a.local_mask[t] : 0u;
    int idx[kTopK];
    float wgt[kTopK];
    if (m) {
#pragma unroll
      for (int k = 0; k < kTopK; ++k) {
        idx[k] = a.topk_idx[t * kTopK + k] - a.local_expert_offset;
        wgt[k] = a.topk_w[t * kTopK + k];
      }
    }
    int j = 0;                                  // rank of the expert among this token's local experts
#pragma unroll
    for (int le = 0; le < kELocal; ++le) {
      const bool mine = (m >> le) & 1u;
      const uint32_t b = __ballot_sync(0xFFFFFFFFu, mine);
      const int first = __shfl_sync(0xFFFFFFFFu, base, le);
      if (mine) {
        const int row = first + __popc(b & lt_mask);
        float w = 0.0f;
#pragma unroll
        for (int k = 0; k < kTopK; ++k) w = (idx[k] == le) ? wgt[k] : w;
        a.perm_token[row] = t;
        a.perm_weight[row] = w;
        a.tok_rows[t * kTopK + j] = row;
        ++j;
      }
      if (lane == le) base += __popc(b);
    }
  }
}

}  // namespace

// One warp per token, 8 warps per CTA.
__global__ void __launch_bounds__(256) route_kernel(RouteArgs a) {
  __shared__ float bias_smem[kEGlobal];
  griddep_launch_dependents();
  griddep_wait();
  load_bias(a.bias_bf16, bias_smem);
  __syncthreads();
  const int warps = blockDim.x >> 5;
  route_tokens_strided(a, bias_smem, blockIdx.x * warps + (threadIdx.x >> 5), gridDim.x * warps, threadIdx.x & 31);
}

__global__ void __launch_bounds__(1024) permute_kernel(PermuteArgs a) {
  griddep_launch_dependents();
  griddep_wait();
  permute_block(a);
}

// Small batches: routing and permutation in one single-CTA launch.
__global__ void __launch_bounds__(1024) route_permute_kernel(RouteArgs r, PermuteArgs p) {
  __shared__ float bias_smem[kEGlobal];
  griddep_launch_dependents();
  griddep_wait();
  load_bias(r.bias_bf16, bias_smem);
  __syncthreads();
  route_tokens_strided(r, bias_smem, threadIdx.x >> 5, 32, threadIdx.x & 31);
  __threadfence_block();
  __syncthreads();
  permute_block(p);
}

// Packed copy of the fp8 activation rows in permuted order: a_packed[r, :] = hidden[perm_token[r], :]
// (the B operand of GEMM1 is then one TMA box per token tile), 16 bytes per thread, plus the
// row's 56 block scales gathered from the transposed [56, T] layout into a row-major table.
__global__ void __launch_bounds__(256) gather_rows_kernel(GatherArgs a) {
  griddep_launch_dependents();
  griddep_wait();
  const int n_sel = a.sched->n_sel;
  constexpr int kData = kH / 16;            // 448 x 16 B of fp8 per row
  constexpr int kChunks = kData + kKB1 / 4; // + 14 x 4 scales
  const long long total = static_cast<long long>(n_sel) * kChunks;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / kChunks), c = static_cast<int>(i % kChunks);
    const int t = a.perm_token[r];
    if (c < kData) {
      reinterpret_cast<uint4*>(a.a_packed + static_cast<size_t>(r) * kH)[c] =
          __ldg(reinterpret_cast<const uint4*>(a.hidden + static_cast<size_t>(t) * kH) + c);
    } else {
      const int kb = (c - kData) * 4;
      float4 v;
      v.x = __ldg(a.hidden_scale + static_cast<size_t>(kb + 0) * a.T + t);
      v.y = __ldg(a.hidden_scale + static_cast<size_t>(kb + 1) * a.T + t);
      v.z = __ldg(a.hidden_scale + static_cast<size_t>(kb + 2) * a.T + t);
      v.w = __ldg(a.hidden_scale + static_cast<size_t>(kb + 3) * a.T + t);
      reinterpret_cast<float4*>(a.a_scale_rows + static_cast<size_t>(r) * kKB1)[c - kData] = v;
    }
  }
}

void launch_route_permute(const RouteArgs& r, const PermuteArgs& p, cudaStream_t stream) {
  if (r.T <= 256) {
    launch_pdl(route_permute_kernel, dim3(1), dim3(1024), 0, stream, r, p);
  } else {
    const int grid = (r.T + 7) / 8 < 4 * kNumSMs ? (r.T + 7) / 8 : 4 * kNumSMs;
    launch_pdl(route_kernel, dim3(grid), dim3(256), 0, stream, r);
    launch_pdl(permute_kernel, dim3(1), dim3(1024), 0, stream, p);
  }
}

void launch_route_only(const RouteArgs& r, cudaStream_t stream) {
  const int grid = (r.T + 7) / 8 < 4 * kNumSMs ? (r.T + 7) / 8 : 4 * kNumSMs;
  launch_pdl(route_kernel, dim3(grid), dim3(256), 0, stream, r);
}

void launch_gather_rows(const GatherArgs& a, int T, cudaStream_t stream) {
  long long chunks = static_cast<long long>(T) * kTopK * (kH / 16 + kKB1 / 4);
  long long blocks = (chunks + 255) / 256;
  if (blocks > 8 * kNumSMs) blocks = 8 * kNumSMs;
  if (blocks < 1) blocks = 1;
  launch_pdl(gather_rows_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, a);
}

}  // namespace moe
