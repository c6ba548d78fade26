// Activation quantisation: the step before the operator.
//
// The operator takes hidden_states as e4m3 with one fp32 scale per (token, 128-column
// block), stored transposed [56, T] (full-agent-pipeline/references/moe.py:32-33, 95-104).
// The reference repository has no kernel for producing that layout (its harness
// generates it on the host); this kernel does it on the device from bf16 activations:
//     scale = max(|x| over the block, 1e-10) / 448      (IEEE division)
//     q     = e4m3(x / scale)                            (round to nearest even, saturating)
// which is bit-identical to the seeded generator's reference quantisation, so that an
// expert-parallel dispatch can quantise, pack and send in one pass.
// One warp per (token, block): lane owns 4 consecutive columns.  HBM-bound:
// reads 2 B and writes 1 B + 1/32 B per element.
#include <cuda_fp8.h>

#include "../../include/moe_b200.h"
#include "kernels.h"

namespace moe {
namespace {

__global__ void __launch_bounds__(256) quantize_1x128_kernel(const uint16_t* __restrict__ x_bf16, int T,
                                                             uint8_t* __restrict__ q, float* __restrict__ scale_T) {
  griddep_launch_dependents();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  const long long nblk = static_cast<long long>(T) * kKB1;
  const long long wstride = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long b = blockIdx.x * static_cast<long long>(blockDim.x >> 5) + (threadIdx.x >> 5); b < nblk; b += wstride) {
    const int t = static_cast<int>(b / kKB1), kb = static_cast<int>(b % kKB1);
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
    *reinterpret_cast<uint32_t*>(q + off) = packed;
    if (lane == 0) scale_T[static_cast<size_t>(kb) * T + t] = scale;
  }
}

}  // namespace
}  // namespace moe

using namespace moe;

extern "C" int moe_fp8_block_scale_quantize_activations(const uint16_t* hidden_bf16, int T, uint8_t* hidden_states,
                                                        float* hidden_states_scale, void* stream_v) {
  if (T < 0) return MOE_B200_EINVAL;
  if (T == 0) return MOE_B200_OK;
  if (!hidden_bf16 || !hidden_states || !hidden_states_scale) return MOE_B200_EINVAL;
  if ((reinterpret_cast<uintptr_t>(hidden_bf16) & 7u) || (reinterpret_cast<uintptr_t>(hidden_states) & 3u))
    return MOE_B200_EINVAL;
  long long warps = static_cast<long long>(T) * kKB1;
  long long blocks = (warps + 7) / 8;
  if (blocks > 16 * kNumSMs) blocks = 16 * kNumSMs;
  cudaError_t e = launch_pdl(quantize_1x128_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0,
                             static_cast<cudaStream_t>(stream_v), hidden_bf16, T, hidden_states, hidden_states_scale);
  return e == cudaSuccess ? MOE_B200_OK : MOE_B200_ECUDA;
}
