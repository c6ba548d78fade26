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

}  // namespace
}  // namespace moe

using namespace moe;

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
