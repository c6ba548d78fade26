// Routing + permutation entry point that allocates nothing.
//
// Some callers cannot obtain device memory at the moment they need the routing
// decision: a plugin running inside an engine that has already handed its whole
// memory budget to a pool it does not own, or code running while the process is
// in a phase where the allocator must not be touched.  For them this file offers
// the routing / histogram / prefix-sum / permutation stage of the operator with its
// scratch memory (the per-token local-expert bit mask, the per-token row lists and
// the schedule block) in a fixed device array that is part of the library image.
// Inputs and outputs are still the caller's buffers.  It has no counterpart in the
// reference solution.
//
// Limits and rules:
//  * at most MOE_B200_STATIC_MAX_TOKENS tokens per call (larger T is rejected with
//    MOE_B200_EINVAL); the array is ~160 KB and every GPU that loads the library
//    holds it until the process exits;
//  * the first call on a device looks the array's device address up
//    (cudaGetSymbolAddress) with that device current; make that first call before
//    starting any stream capture;
//  * all calls on a device share the one array, which keeps whatever the previous
//    call left in it.  Nothing has to be cleared: every word a call reads is written
//    earlier in the same call.  Two calls that overlap on the GPU (different
//    streams) race on it; serialise them.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/moe_b200.h"
#include "kernels.h"

namespace moe {
namespace {

constexpr int kStaticMaxTokens = MOE_B200_STATIC_MAX_TOKENS;
constexpr size_t kSchedBytes = (sizeof(MoeSched) + 1023) / 1024 * 1024;
constexpr size_t kMaskBytes = static_cast<size_t>(kStaticMaxTokens) * 4;
constexpr size_t kRowsBytes = static_cast<size_t>(kStaticMaxTokens) * kTopK * 4;
constexpr size_t kChunkBytes = static_cast<size_t>(kStaticMaxTokens / 32) * kELocal * 4;

// File-scope scratch.  In host code this name is only a handle for the runtime's
// symbol lookup, never a pointer a kernel may be given.
static __device__ __align__(256) unsigned char g_route_scratch[kSchedBytes + kMaskBytes + kRowsBytes + kChunkBytes];

std::mutex g_static_mu;
unsigned char* g_scratch_addr[16] = {};

// Device address of the scratch array on the current device (looked up once per device).
int scratch_address(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 16) return static_cast<int>(cudaErrorInvalidDevice);
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_route_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_scratch_addr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace
}  // namespace moe

using namespace moe;

extern "C" int moe_fp8_block_scale_route_static(const float* routing_logits, const uint16_t* routing_bias, int T,
                                                int local_expert_offset, float routed_scaling_factor,
                                                int32_t* topk_idx, float* topk_w, int32_t* expert_offsets,
                                                int32_t* perm_token, float* perm_weight, void* stream_v) {
  if (T < 0 || T > kStaticMaxTokens) return MOE_B200_EINVAL;   // beyond the fixed scratch
  if (T == 0) return MOE_B200_OK;
  if (!routing_logits || !routing_bias || !topk_idx || !topk_w || !expert_offsets || !perm_token || !perm_weight)
    return MOE_B200_EINVAL;
  if ((reinterpret_cast<uintptr_t>(routing_logits) & 15u) != 0) return MOE_B200_EINVAL;
  unsigned char* scratch = nullptr;
  if (const int e = scratch_address(&scratch)) {
    set_last_cuda_error(e);
    return MOE_B200_ECUDA;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  MoeSched* sched = reinterpret_cast<MoeSched*>(scratch);
  uint32_t* local_mask = reinterpret_cast<uint32_t*>(scratch + kSchedBytes);
  int* tok_rows = reinterpret_cast<int*>(scratch + kSchedBytes + kMaskBytes);
  int* chunk_base = reinterpret_cast<int*>(scratch + kSchedBytes + kMaskBytes + kRowsBytes);
  const int rows_cap = T * kTopK;
  RouteArgs ra{routing_logits, routing_bias, T, local_expert_offset, routed_scaling_factor, topk_idx, topk_w,
               local_mask};
  PermuteArgs pa{T, local_expert_offset, 128, 128, kNumSMs, 1, 1, rows_cap, rows_cap > kMinSlabRows ? rows_cap : kMinSlabRows,
                 local_mask, topk_idx, topk_w, sched, perm_token, perm_weight, tok_rows, chunk_base};
  launch_route_permute(ra, pa, stream);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) {
    count_launches(route_permute_launches(T));
    e = cudaMemcpyAsync(expert_offsets, sched->offs, (kELocal + 1) * sizeof(int), cudaMemcpyDeviceToDevice, stream);
  }
  if (e != cudaSuccess) {
    set_last_cuda_error(static_cast<int>(e));
    return MOE_B200_ECUDA;
  }
  return MOE_B200_OK;
}
