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
#include "route_device.cuh"

namespace moe {

namespace {

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

constexpr int kPermuteFillInline = 1024;   // up to here the single permutation CTA also fills the rows

// Rows of one 32-token chunk (lane = token).  `base`: lane = expert, the chunk's first row per expert;
// returns the base of the next chunk.
__device__ __forceinline__ int fill_chunk(const PermuteArgs& a, int c, int base, int lane) {
  const uint32_t lt_mask = (1u << lane) - 1u;
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
  return base;
}

// Block-wide (1024 threads) histogram, scan, stable permutation and schedule.  Warp w owns
// the contiguous token range [w * span, (w + 1) * span); inside a 32-token chunk lane = token.
// Phase 1 counts, per warp and expert, the tokens that selected the expert; an exclusive
// scan over (expert, warp) then gives every warp its first row for every expert, and phase
// 2 fills rows in token order, so rows are ascending in token inside ascending expert.
// Requires the routing outputs of all T tokens to be visible.
// Tokens of chunk c (lane = token) per local expert: lane le returns the count of expert le.
__device__ __forceinline__ int chunk_counts(const PermuteArgs& a, int c, int lane) {
  const int t = c * 32 + lane;
  const uint32_t m = t < a.T ? a.local_mask[t] : 0u;
  int cnt = 0;
#pragma unroll
  for (int le = 0; le < kELocal; ++le) {
    const int n = __popc(__ballot_sync(0xFFFFFFFFu, (m >> le) & 1u));
    if (lane == le) cnt = n;
  }
  return cnt;
}

// `counted`: chunk_base already holds every chunk's per-expert counts (written by chunk_count_kernel, many
// CTAs); otherwise this CTA counts the masks itself.
__device__ void permute_block(const PermuteArgs& a, bool counted) {
  __shared__ int s_wcount[32][kELocal + 1];     // [warp][expert]: count, then first row (+1: no bank conflicts)
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int chunks = (a.T + 31) / 32;
  const int span = (chunks + 31) / 32;          // chunks per warp
  const int c0 = warp * span, c1 = min(chunks, c0 + span);

  // phase 1: lane le accumulates this warp's count for expert le
  int cnt = 0;
  for (int c = c0; c < c1; ++c) cnt += counted ? a.chunk_base[c * kELocal + lane] : chunk_counts(a, c, lane);
  s_wcount[warp][lane] = cnt;
  __syncthreads();
  if (warp == 0) {
    // lane = expert: totals over warps, exclusive scan over experts, per-warp first rows
    int c = 0;
    for (int w = 0; w < 32; ++w) c += s_wcount[w][lane];
    const int tiles = (c + a.n_tile - 1) / a.n_tile, tiles2 = (c + a.n_tile2 - 1) / a.n_tile2;
    int inc = c, tinc = tiles, tinc2 = tiles2;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xFFFFFFFFu, inc, d);
      const int tv = __shfl_up_sync(0xFFFFFFFFu, tinc, d);
      const int tv2 = __shfl_up_sync(0xFFFFFFFFu, tinc2, d);
      if (lane >= d) { inc += v; tinc += tv; tinc2 += tv2; }
    }
    int run = inc - c;                          // first row of expert `lane`
    for (int w = 0; w < 32; ++w) {
      const int n = s_wcount[w][lane];
      s_wcount[w][lane] = run;
      run += n;
    }
    MoeSched* sc = a.sched;
    sc->counts[lane] = c;
    sc->offs[lane + 1] = inc;
    sc->tile_prefix[lane + 1] = tinc;
    sc->tile_prefix2[lane + 1] = tinc2;
    const uint32_t act = __ballot_sync(0xFFFFFFFFu, c > 0);
    const int n_sel = __shfl_sync(0xFFFFFFFFu, inc, 31), tiles_total = __shfl_sync(0xFFFFFFFFu, tinc, 31);
    const int tiles_total2 = __shfl_sync(0xFFFFFFFFu, tinc2, 31);
    const int n_sel_pad = (n_sel + 15) & ~15;
    int s1 = choose_split_warp(tiles_total * kMT1, kMaxSplit1, a.ctas, n_sel_pad, a.slab_rows, lane, kKB1, a.kps1);
    int s2 = choose_split_warp(tiles_total2 * kMT2, kMaxSplit2, a.ctas, n_sel_pad, a.slab_rows, lane, kKB2, a.kps2);
    if (a.large) s1 = 1;          // the SwiGLU epilogue needs whole K sums
    if (a.large > 1) s2 = 1;      // ... and so does the fused combine
    if (lane == 31) {
      sc->offs[0] = 0;
      sc->tile_prefix[0] = 0;
      sc->tile_prefix2[0] = 0;
      sc->n_tile2 = a.n_tile2;
      sc->ctas = 0;
      sc->status = (n_sel > a.rows_cap) ? kErrSchedOverflow : 0;
      sc->n_sel = n_sel;
      sc->n_sel_pad = n_sel_pad;
      sc->n_active = __popc(act);
      sc->n_tile = a.n_tile;
      sc->tiles_total = tiles_total;
      sc->split1 = s1;
      sc->split2 = s2;
      sc->items1 = a.large ? tiles_total * kKB2 : tiles_total * kMT1 * s1;   // large: one item per 128-column block of C
      sc->items2 = a.large > 1 ? tiles_total2 * (kMT2 / 2) : tiles_total2 * kMT2 * s2;   // large: 256-row weight units
    }
  }
  __syncthreads();
  // phase 2.  `base` (lane = expert) is this warp's next free row of each expert.  Small batches are
  // filled here; for large ones the per-chunk bases are published and a multi-CTA kernel fills.
  int base = s_wcount[warp][lane];
  const bool fill_here = a.T <= kPermuteFillInline;
  for (int c = c0; c < c1; ++c) {
    if (fill_here) {
      base = fill_chunk(a, c, base, lane);
    } else {
      const int n = counted ? a.chunk_base[c * kELocal + lane] : chunk_counts(a, c, lane);
      a.chunk_base[c * kELocal + lane] = base;      // the count is replaced by the chunk's first row
      base += n;
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

// One 256-thread CTA per token (thread = expert, warp = routing group): sigmoid + bias, the group's
// two best by two warp reductions, then every kept expert counts the kept experts that beat it; the
// eight with rank < 8 are the selection in descending order.  Same arithmetic and tie rules as
// route_token, a third of its latency; used while there are at most a couple of tokens per CTA.
__global__ void __launch_bounds__(256) route_block_kernel(RouteArgs a) {
  __shared__ __align__(16) uint32_t keys[kEGlobal];
  __shared__ float gscore[kNGroup];
  __shared__ int selidx[kTopK];
  __shared__ float sels[kTopK];
  griddep_launch_dependents();
  griddep_wait();
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  const float bias_e = __uint_as_float(static_cast<uint32_t>(a.bias_bf16[e]) << 16);
  for (int t = blockIdx.x; t < a.T; t += gridDim.x) {
    const float s_e = 1.0f / (1.0f + expf(-a.logits[static_cast<size_t>(t) * kEGlobal + e]));
    const uint32_t key_e = order_key(s_e + bias_e);
    keys[e] = key_e;
    const uint32_t k1 = __reduce_max_sync(0xFFFFFFFFu, key_e);
    const int first = __ffs(__ballot_sync(0xFFFFFFFFu, key_e == k1)) - 1;
    const uint32_t k2 = __reduce_max_sync(0xFFFFFFFFu, lane == first ? 0u : key_e);
    const uint32_t u1 = (k1 & 0x80000000u) ? (k1 & 0x7FFFFFFFu) : ~k1;
    const uint32_t u2 = (k2 & 0x80000000u) ? (k2 & 0x7FFFFFFFu) : ~k2;
    if (lane == 0) gscore[warp] = __uint_as_float(u1) + __uint_as_float(u2);
    __syncthreads();
    uint32_t keep = 0;
#pragma unroll
    for (int g = 0; g < kNGroup; ++g) {
      int rank = 0;
#pragma unroll
      for (int h = 0; h < kNGroup; ++h) rank += (gscore[h] > gscore[g]) || (gscore[h] == gscore[g] && h < g);
      keep |= (rank < kTopKGroup ? 1u : 0u) << g;
    }
    if ((keep >> warp) & 1u) {
      int rank = 0;
      for (int g = 0; g < kNGroup; ++g) {
        if (!((keep >> g) & 1u)) continue;
        const uint4* kv = reinterpret_cast<const uint4*>(keys + g * 32);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 k = kv[c];
          const int j = g * 32 + c * 4;
          rank += (k.x > key_e) || (k.x == key_e && j + 0 < e);
          rank += (k.y > key_e) || (k.y == key_e && j + 1 < e);
          rank += (k.z > key_e) || (k.z == key_e && j + 2 < e);
          rank += (k.w > key_e) || (k.w == key_e && j + 3 < e);
        }
      }
      if (rank < kTopK) { selidx[rank] = e; sels[rank] = s_e; }
    }
    __syncthreads();
    if (warp == 0) {
      const float sv = lane < kTopK ? sels[lane] : 0.0f;
      float sum = 0.0f;
#pragma unroll
      for (int k = 0; k < kTopK; ++k) sum += __shfl_sync(0xFFFFFFFFu, sv, k);
      sum += 1e-20f;
      uint32_t bit = 0;
      if (lane < kTopK) {
        const int idx = selidx[lane];
        a.topk_idx[t * kTopK + lane] = idx;
        a.topk_w[t * kTopK + lane] = (sv / sum) * a.routed_scaling_factor;
        const int le = idx - a.local_expert_offset;
        if (le >= 0 && le < kELocal) bit = 1u << le;
      }
      bit = __reduce_or_sync(0xFFFFFFFFu, bit);
      if (lane == 0) a.local_mask[t] = bit;
    }
    // the next token's keys / gscore are written before, selidx / sels after the next first barrier;
    // warp 0 has read selidx / sels before it reaches that barrier
  }
}

__global__ void __launch_bounds__(1024) permute_kernel(PermuteArgs a, bool counted) {
  griddep_launch_dependents();
  griddep_wait();
  permute_block(a, counted);
}

// Large batches: the histogram of every 32-token chunk by one warp each, over many CTAs, so that the single
// permutation CTA only scans 32 numbers per chunk instead of balloting through every token's mask.
__global__ void __launch_bounds__(256) chunk_count_kernel(PermuteArgs a) {
  griddep_launch_dependents();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  const int chunks = (a.T + 31) / 32;
  for (int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); c < chunks; c += gridDim.x * (blockDim.x >> 5))
    a.chunk_base[c * kELocal + lane] = chunk_counts(a, c, lane);
}

// Large batches: one warp per 32-token chunk fills the rows from the published chunk bases.
__global__ void __launch_bounds__(256) permute_fill_kernel(PermuteArgs a) {
  griddep_launch_dependents();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  const int chunks = (a.T + 31) / 32;
  for (int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); c < chunks; c += gridDim.x * (blockDim.x >> 5))
    fill_chunk(a, c, a.chunk_base[c * kELocal + lane], lane);
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
  permute_block(p, false);
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
  if (r.T <= 32) {
    launch_pdl(route_permute_kernel, dim3(1), dim3(1024), 0, stream, r, p);
  } else {
    launch_route_only(r, stream);
    const bool big = r.T > kPermuteFillInline;
    const int chunks = (r.T + 31) / 32;
    if (big) launch_pdl(chunk_count_kernel, dim3((chunks + 7) / 8), dim3(256), 0, stream, p);
    launch_pdl(permute_kernel, dim3(1), dim3(1024), 0, stream, p, big);
    if (big) launch_pdl(permute_fill_kernel, dim3((chunks + 7) / 8), dim3(256), 0, stream, p);
  }
}

void launch_route_only(const RouteArgs& r, cudaStream_t stream) {
  if (r.T <= 8 * kNumSMs) {          // one CTA per token while that is at most one wave of eight CTAs per SM
    launch_pdl(route_block_kernel, dim3(r.T), dim3(256), 0, stream, r);
  } else {
    const int grid = (r.T + 7) / 8 < 4 * kNumSMs ? (r.T + 7) / 8 : 4 * kNumSMs;
    launch_pdl(route_kernel, dim3(grid), dim3(256), 0, stream, r);
  }
}

void launch_gather_rows(const GatherArgs& a, int T, cudaStream_t stream) {
  long long chunks = static_cast<long long>(T) * kTopK * (kH / 16 + kKB1 / 4);
  long long blocks = (chunks + 255) / 256;
  if (blocks > 8 * kNumSMs) blocks = 8 * kNumSMs;
  if (blocks < 1) blocks = 1;
  launch_pdl(gather_rows_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, a);
}

}  // namespace moe
