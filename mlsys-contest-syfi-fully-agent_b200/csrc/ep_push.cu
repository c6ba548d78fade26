// Expert-parallel dispatch over peer memory: one kernel gathers, packs and SENDS.
//
// Every rank holds a symmetric receive area (same layout on all ranks, mapped into every
// peer's address space).  For each (token, selected shard) record this kernel reads the
// token's fp8 row, its 56 block scales (from the transposed [56, T] layout) and its 256
// routing logits, and stores them straight into the owner rank's receive area over NVLink
// (plain 16-byte peer stores; no multicast, no TMA to peer memory, nothing waits on a peer
// inside the kernel).  It replaces three index_select + three NCCL all-to-all-v of the
// host-driven dispatch.  The reference has no multi-rank code at all.
//
// Records are grouped in up to 8 segments (one per destination shard, ascending token inside);
// `seg` tells where each segment starts in `rec_token`, how long it is, and the base addresses
// of its three destination arrays at the owner.
#include <cuda_fp8.h>

#include "../../include/moe_b200.h"
#include "kernels.h"

namespace moe {
namespace {

struct SegTable {
  moe_ep_segment seg[8];
  int n_seg;
};

__global__ void __launch_bounds__(128) ep_dispatch_push_kernel(const uint8_t* __restrict__ hidden,
                                                               const float* __restrict__ hidden_scale,
                                                               const float* __restrict__ logits, int T,
                                                               const int64_t* __restrict__ rec_token, int n_rec,
                                                               SegTable tab) {
  griddep_launch_dependents();
  griddep_wait();
  constexpr int kRowChunks = kH / 16;          // 448 x 16 B
  constexpr int kLogitChunks = kEGlobal * 4 / 16;   // 64 x 16 B
  for (int r = blockIdx.x; r < n_rec; r += gridDim.x) {
    int s = 0;
#pragma unroll
    for (int k = 1; k < 8; ++k)
      if (k < tab.n_seg && r >= tab.seg[k].first_record) s = k;
    const moe_ep_segment sg = tab.seg[s];
    const long long k = r - sg.first_record;
    const int t = static_cast<int>(rec_token[r]);
    uint4* dst_h = reinterpret_cast<uint4*>(sg.dst_hidden + k * kH);
    const uint4* src_h = reinterpret_cast<const uint4*>(hidden + static_cast<size_t>(t) * kH);
    for (int c = threadIdx.x; c < kRowChunks; c += blockDim.x) dst_h[c] = __ldg(src_h + c);
    uint4* dst_l = reinterpret_cast<uint4*>(sg.dst_logits + k * kEGlobal);
    const uint4* src_l = reinterpret_cast<const uint4*>(logits + static_cast<size_t>(t) * kEGlobal);
    if (threadIdx.x < kLogitChunks) dst_l[threadIdx.x] = __ldg(src_l + threadIdx.x);
    if (threadIdx.x >= 64 && threadIdx.x < 64 + kKB1)
      sg.dst_scale[k * kKB1 + (threadIdx.x - 64)] = __ldg(hidden_scale + static_cast<size_t>(threadIdx.x - 64) * T + t);
  }
}

// Quantise, pack and send in one pass: the dispatch for activations that are still bf16.  One CTA per token
// quantises the row exactly as quantize_1x128_kernel does (scale = max(|x|, 1e-10) / 448 with IEEE division,
// e4m3 round-to-nearest-even saturating; one warp per 128-column block, eight blocks per warp), keeps the 7168
// bytes and 56 scales in shared memory, and stores them together with the token's logits to every shard the token
// selected: the record's place at the owner is its position among the rank's records for that shard
// (row_of[t][s] - first_record of the shard's segment).  The row is read from HBM once however many shards it
// goes to, and the fp8 copy never exists in this rank's memory.
struct SegByShard {
  moe_ep_segment seg[8];      // indexed by shard; count == 0: no record for that shard
};

constexpr int kQPushThreads = 224;   // 7 warps x 8 blocks = 56 blocks; 448 16-byte chunks = 2 per thread

__global__ void __launch_bounds__(kQPushThreads) ep_quantize_push_kernel(const uint16_t* __restrict__ x_bf16,
                                                                        const float* __restrict__ logits, int T,
                                                                        const int32_t* __restrict__ row_of,
                                                                        SegByShard tab) {
  griddep_launch_dependents();
  griddep_wait();
  __shared__ __align__(16) uint8_t q[kH];
  __shared__ float sc[kKB1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    int dest[8];
    bool any = false;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      dest[s] = __ldg(row_of + static_cast<size_t>(t) * 8 + s);
      any |= dest[s] >= 0;
    }
    if (!any) continue;      // (uniform over the CTA)
    for (int kb = warp; kb < kKB1; kb += kQPushThreads / 32) {
      const size_t off = static_cast<size_t>(t) * kH + kb * kBlock + lane * 4;
      const uint2 raw = __ldg(reinterpret_cast<const uint2*>(x_bf16 + off));
      float v[4];
      v[0] = __uint_as_float(raw.x << 16);
      v[1] = __uint_as_float(raw.x & 0xFFFF0000u);
      v[2] = __uint_as_float(raw.y << 16);
      v[3] = __uint_as_float(raw.y & 0xFFFF0000u);
      float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, d));
      const float scale = __fdiv_rn(fmaxf(amax, 1e-10f), 448.0f);
      uint32_t packed = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        packed |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(__fdiv_rn(v[i], scale), __NV_SATFINITE, __NV_E4M3)) << (8 * i);
      *reinterpret_cast<uint32_t*>(q + kb * kBlock + lane * 4) = packed;
      if (lane == 0) sc[kb] = scale;
    }
    __syncthreads();
    const uint4 row0 = reinterpret_cast<const uint4*>(q)[threadIdx.x];
    const uint4 row1 = reinterpret_cast<const uint4*>(q)[threadIdx.x + kQPushThreads];
    uint4 lg = make_uint4(0u, 0u, 0u, 0u);
    if (threadIdx.x < kEGlobal * 4 / 16)
      lg = __ldg(reinterpret_cast<const uint4*>(logits + static_cast<size_t>(t) * kEGlobal) + threadIdx.x);
    const float my_scale = threadIdx.x >= 64 && threadIdx.x < 64 + kKB1 ? sc[threadIdx.x - 64] : 0.0f;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (dest[s] < 0) continue;
      const moe_ep_segment sg = tab.seg[s];
      const long long k = dest[s] - sg.first_record;
      uint4* dst_h = reinterpret_cast<uint4*>(sg.dst_hidden + k * kH);
      dst_h[threadIdx.x] = row0;
      dst_h[threadIdx.x + kQPushThreads] = row1;
      if (threadIdx.x < kEGlobal * 4 / 16) reinterpret_cast<uint4*>(sg.dst_logits + k * kEGlobal)[threadIdx.x] = lg;
      if (threadIdx.x >= 64 && threadIdx.x < 64 + kKB1) sg.dst_scale[k * kKB1 + (threadIdx.x - 64)] = my_scale;
    }
    __syncthreads();      // the row buffer is reused by the next token
  }
  static_assert(kH / 16 == 2 * kQPushThreads && kKB1 == 8 * (kQPushThreads / 32), "chunks and blocks per thread");
}

// Final accumulation of the expert-parallel layer: out[t] = bf16(sum over shards s = 0..7, ascending, of
// fp32(back[pos[t][s]])) for the shards the token selected (pos >= 0).  One block per token; replaces
// eight index_add_ passes over fp32 copies of the returned rows.
__global__ void __launch_bounds__(224) ep_sum_shards_kernel(const uint16_t* __restrict__ back,
                                                            const int32_t* __restrict__ pos, int T,
                                                            uint16_t* __restrict__ out) {
  griddep_launch_dependents();
  griddep_wait();
  constexpr int kChunks = kH * 2 / 16;           // 896 x 16 B per row = 4 per thread
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    float acc[4][8];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[c][i] = 0.0f;
    for (int s = 0; s < 8; ++s) {
      const int row = pos[t * 8 + s];
      if (row < 0) continue;
      const uint4* src = reinterpret_cast<const uint4*>(back + static_cast<size_t>(row) * kH);
      uint4 v[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) v[c] = src[threadIdx.x + c * 224];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[c][2 * i] += __uint_as_float(w[i] << 16);
          acc[c][2 * i + 1] += __uint_as_float(w[i] & 0xFFFF0000u);
        }
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * kH);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w[i]) : "f"(acc[c][2 * i + 1]), "f"(acc[c][2 * i]));
      dst[threadIdx.x + c * 224] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  static_assert(kChunks == 4 * 224, "row chunks per thread");
}

// Dispatch plan of one rank: which (token, shard) records it sends, shard-major with ascending tokens inside a
// shard (the order torch.nonzero gives on the transposed hit mask), the per-shard counts, and for every
// (token, shard) the position of its record in that order (-1: not selected).  One CTA: every thread owns a run
// of consecutive tokens, counts its hits per shard, the CTA scans the counts, and the thread writes its records
// at the scanned positions.  Replaces about twenty host-launched tensor operations and the host stop inside
// torch.nonzero; the counts go to the peers without touching the host.
constexpr int kPlanThreads = 1024;

__device__ __forceinline__ uint32_t shard_mask_of(const int32_t* __restrict__ topk, int t) {
  const int4 a = __ldg(reinterpret_cast<const int4*>(topk + static_cast<size_t>(t) * kTopK));
  const int4 b = __ldg(reinterpret_cast<const int4*>(topk + static_cast<size_t>(t) * kTopK) + 1);
  const int e[kTopK] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  uint32_t m = 0;
#pragma unroll
  for (int k = 0; k < kTopK; ++k)
    if (e[k] >= 0 && e[k] < kEGlobal) m |= 1u << (e[k] / kELocal);
  return m;
}

__global__ void __launch_bounds__(kPlanThreads) ep_plan_kernel(const int32_t* __restrict__ topk, int T,
                                                              int64_t* __restrict__ counts9,
                                                              int64_t* __restrict__ send_order,
                                                              int64_t* __restrict__ send_shard,
                                                              int32_t* __restrict__ row_of) {
  griddep_launch_dependents();
  griddep_wait();
  constexpr int kShards = kEGlobal / kELocal;   // 8
  static_assert(kShards == 8 && kTopK == 8, "record layout");
  __shared__ int warp_tot[kPlanThreads / 32][kShards];
  __shared__ int warp_off[kPlanThreads / 32][kShards];
  __shared__ int base[kShards];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunk = (T + kPlanThreads - 1) / kPlanThreads;
  const int t0 = min(T, tid * chunk), t1 = min(T, t0 + chunk);
  int c[kShards];
#pragma unroll
  for (int s = 0; s < kShards; ++s) c[s] = 0;
  for (int t = t0; t < t1; ++t) {
    const uint32_t m = shard_mask_of(topk, t);
#pragma unroll
    for (int s = 0; s < kShards; ++s) c[s] += (m >> s) & 1u;
  }
  int excl[kShards];
#pragma unroll
  for (int s = 0; s < kShards; ++s) {
    int v = c[s];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int u = __shfl_up_sync(0xFFFFFFFFu, v, d);
      if (lane >= d) v += u;
    }
    excl[s] = v - c[s];
    if (lane == 31) warp_tot[warp][s] = v;
  }
  __syncthreads();
  if (tid < kShards) {
    int run = 0;
    for (int w = 0; w < kPlanThreads / 32; ++w) {
      warp_off[w][tid] = run;
      run += warp_tot[w][tid];
    }
    base[tid] = run;      // the shard's total, turned into its start below
  }
  __syncthreads();
  if (tid == 0) {
    int b = 0;
    for (int s = 0; s < kShards; ++s) {
      const int n = base[s];
      counts9[s] = n;
      base[s] = b;
      b += n;
    }
    counts9[kShards] = T;
  }
  __syncthreads();
  int pos[kShards];
#pragma unroll
  for (int s = 0; s < kShards; ++s) pos[s] = base[s] + warp_off[warp][s] + excl[s];
  for (int t = t0; t < t1; ++t) {
    const uint32_t m = shard_mask_of(topk, t);
#pragma unroll
    for (int s = 0; s < kShards; ++s) {
      int r = -1;
      if ((m >> s) & 1u) {
        r = pos[s]++;
        send_order[r] = t;
        send_shard[r] = s;
      }
      row_of[static_cast<size_t>(t) * kShards + s] = r;
    }
  }
}

// Destination address of every result row of this rank's shard operators: rows come in up to eight
// runs (owned shard x source rank), run k holding count[k] consecutive rows whose destinations start at base[k]
// and lie row_bytes apart.
struct PtrRuns {
  long long start[9];      // first row of run k (start[n] = total rows)
  long long base[8];
  int n;
};

__global__ void __launch_bounds__(256) ep_row_pointers_kernel(PtrRuns runs, long long row_bytes, int64_t* __restrict__ out,
                                                              int n_rows) {
  griddep_launch_dependents();
  griddep_wait();
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += gridDim.x * blockDim.x) {
    int k = 0;
#pragma unroll
    for (int j = 1; j < 8; ++j)
      if (j < runs.n && r >= runs.start[j]) k = j;
    out[r] = runs.base[k] + (r - runs.start[k]) * row_bytes;
  }
}

}  // namespace
}  // namespace moe

using namespace moe;

extern "C" int moe_ep_row_pointers(const int64_t* run_base_host, const int64_t* run_count_host, int n_runs,
                                   int64_t row_bytes, int64_t* out_ptrs, int n_rows, void* stream_v) {
  if (n_runs < 0 || n_runs > 8 || n_rows < 0 || row_bytes <= 0) return MOE_B200_EINVAL;
  if (n_rows == 0) return MOE_B200_OK;
  if (!run_base_host || !run_count_host || !out_ptrs || n_runs == 0) return MOE_B200_EINVAL;
  PtrRuns runs{};
  long long pos = 0;
  int n = 0;
  for (int k = 0; k < n_runs; ++k) {
    if (run_count_host[k] < 0) return MOE_B200_EINVAL;
    if (run_count_host[k] == 0) continue;       // empty runs own no row
    runs.start[n] = pos;
    runs.base[n] = run_base_host[k];
    pos += run_count_host[k];
    ++n;
  }
  if (pos != n_rows) return MOE_B200_EINVAL;
  runs.start[n] = pos;
  runs.n = n;
  const int blocks = (n_rows + 255) / 256 < 4 * kNumSMs ? (n_rows + 255) / 256 : 4 * kNumSMs;
  cudaError_t e = launch_pdl(ep_row_pointers_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream_v),
                             runs, static_cast<long long>(row_bytes), out_ptrs, n_rows);
  return e == cudaSuccess ? MOE_B200_OK : MOE_B200_ECUDA;
}

extern "C" int moe_ep_plan(const int32_t* topk_idx, int T, int64_t* counts9, int64_t* send_order, int64_t* send_shard,
                           int32_t* row_of, void* stream_v) {
  if (T < 0) return MOE_B200_EINVAL;
  if (!counts9 || (T > 0 && (!topk_idx || !send_order || !send_shard || !row_of))) return MOE_B200_EINVAL;
  if (reinterpret_cast<uintptr_t>(topk_idx) & 15u) return MOE_B200_EINVAL;
  cudaError_t e = launch_pdl(ep_plan_kernel, dim3(1), dim3(kPlanThreads), 0, static_cast<cudaStream_t>(stream_v),
                             topk_idx, T, counts9, send_order, send_shard, row_of);
  return e == cudaSuccess ? MOE_B200_OK : MOE_B200_ECUDA;
}

extern "C" int moe_ep_dispatch_push(const uint8_t* hidden_states, const float* hidden_states_scale,
                                    const float* routing_logits, int T, const int64_t* rec_token, int n_records,
                                    const moe_ep_segment* segments, int n_segments, void* stream_v) {
  if (T < 0 || n_records < 0 || n_segments < 0 || n_segments > 8) return MOE_B200_EINVAL;
  if (n_records == 0) return MOE_B200_OK;
  if (!hidden_states || !hidden_states_scale || !routing_logits || !rec_token || !segments || n_segments == 0)
    return MOE_B200_EINVAL;
  SegTable tab{};
  tab.n_seg = n_segments;
  for (int i = 0; i < n_segments; ++i) {
    tab.seg[i] = segments[i];
    if (!segments[i].dst_hidden || !segments[i].dst_scale || !segments[i].dst_logits) return MOE_B200_EINVAL;
    if ((reinterpret_cast<uintptr_t>(segments[i].dst_hidden) | reinterpret_cast<uintptr_t>(segments[i].dst_logits)) & 15u)
      return MOE_B200_EINVAL;
  }
  int blocks = n_records < 8 * kNumSMs ? n_records : 8 * kNumSMs;
  cudaError_t e = launch_pdl(ep_dispatch_push_kernel, dim3(blocks), dim3(128), 0, static_cast<cudaStream_t>(stream_v),
                             hidden_states, hidden_states_scale, routing_logits, T, rec_token, n_records, tab);
  return e == cudaSuccess ? MOE_B200_OK : MOE_B200_ECUDA;
}

extern "C" int moe_ep_quantize_push(const uint16_t* hidden_bf16, const float* routing_logits, int T,
                                    const int32_t* row_of, const moe_ep_segment* segments_by_shard, void* stream_v) {
  if (T < 0) return MOE_B200_EINVAL;
  if (T == 0) return MOE_B200_OK;
  if (!hidden_bf16 || !routing_logits || !row_of || !segments_by_shard) return MOE_B200_EINVAL;
  if ((reinterpret_cast<uintptr_t>(hidden_bf16) & 7u) || (reinterpret_cast<uintptr_t>(routing_logits) & 15u))
    return MOE_B200_EINVAL;
  SegByShard tab{};
  for (int s = 0; s < 8; ++s) {
    tab.seg[s] = segments_by_shard[s];
    if (segments_by_shard[s].count < 0) return MOE_B200_EINVAL;
    if (segments_by_shard[s].count == 0) continue;
    if (!segments_by_shard[s].dst_hidden || !segments_by_shard[s].dst_scale || !segments_by_shard[s].dst_logits)
      return MOE_B200_EINVAL;
    if ((reinterpret_cast<uintptr_t>(segments_by_shard[s].dst_hidden) |
         reinterpret_cast<uintptr_t>(segments_by_shard[s].dst_logits)) & 15u)
      return MOE_B200_EINVAL;
  }
  const int blocks = T < 8 * kNumSMs ? T : 8 * kNumSMs;
  cudaError_t e = launch_pdl(ep_quantize_push_kernel, dim3(blocks), dim3(kQPushThreads), 0,
                             static_cast<cudaStream_t>(stream_v), hidden_bf16, routing_logits, T, row_of, tab);
  return e == cudaSuccess ? MOE_B200_OK : MOE_B200_ECUDA;
}

extern "C" int moe_ep_sum_shards(const uint16_t* back_rows, const int32_t* row_of, int T, uint16_t* output,
                                 void* stream_v) {
  if (T < 0) return MOE_B200_EINVAL;
  if (T == 0) return MOE_B200_OK;
  if (!back_rows || !row_of || !output) return MOE_B200_EINVAL;
  if ((reinterpret_cast<uintptr_t>(back_rows) | reinterpret_cast<uintptr_t>(output)) & 15u) return MOE_B200_EINVAL;
  const int blocks = T < 16 * kNumSMs ? T : 16 * kNumSMs;
  cudaError_t e = launch_pdl(ep_sum_shards_kernel, dim3(blocks), dim3(224), 0, static_cast<cudaStream_t>(stream_v),
                             back_rows, row_of, T, output);
  return e == cudaSuccess ? MOE_B200_OK : MOE_B200_ECUDA;
}
