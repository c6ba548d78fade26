// SwiGLU + multi-term e4m3 split (between the two GEMMs) and the final weighted
// combine + bf16 cast.
//
// swiglu_split: sums the split-K slabs of GEMM1, applies
//   C = silu(G1[:, 2048:]) * G1[:, :2048]   (references/moe.py:187-193: the SECOND half
//   goes through silu), replacing swiglu_kernel (moe/solution/cuda/moe.cu:2125-2167),
//   and writes C as kNTerms e4m3 planes with one power-of-two scale per (row, 128 block):
//       C ~= scale * (t0 + t1 + ... ),  t_i = e4m3(residual after t_0..t_{i-1})
//   All planes share the scale, so GEMM2 accumulates the kNTerms products of a K-block
//   in the same TMEM accumulator.  Three terms carry ~12 significant bits of every element
//   and leave a relative error of ~2e-5 on the GEMM2 result, below the ~1e-5 fp32
//   summation-order noise of the definition itself by less than a factor of two and two
//   orders of magnitude inside the output tolerance; a single e4m3 rounding of C (what a
//   plain fp8 x fp8 GEMM2 would use) does not meet it.  The reference kernel keeps C in a
//   bf16 hi+lo pair for the same reason (moe.cu:1241-1251).  Each extra plane costs a
//   quarter more L2->SM traffic for GEMM2's token operand, which bounds it at large T.
// combine: out[t] = bf16( sum over the token's local experts, ascending, of
//   weight * (sum of GEMM2 split-K slabs) ), the accumulation order of
//   references/moe.py:168-200; replaces the fp32 atomics of the reference GEMM2
//   epilogue and fin_cast8_kernel (moe.cu:2404-2430, 2473-2496).  Tokens without a
//   local expert get zeros, so the output needs no memset.
#include "epilogue_device.cuh"
#include "kernels.h"

namespace moe {

namespace {

// One warp per (row, 128-column block).
__global__ void __launch_bounds__(256) swiglu_split_kernel(SwigluArgs a) {
  griddep_launch_dependents();
  griddep_wait();
  const MoeSched* sc = a.sched;
  const int n_sel = sc->n_sel, split = sc->split1;
  const size_t slab = static_cast<size_t>(sc->n_sel_pad) * k2I;
  const int lane = threadIdx.x & 31;
  constexpr int kNB = 1;   // blocks per warp; more per warp measured slower (fewer warps in flight)
  const long long nunit = static_cast<long long>(n_sel) * (kKB2 / kNB);
  const long long wstride = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long b = blockIdx.x * static_cast<long long>(blockDim.x >> 5) + (threadIdx.x >> 5); b < nunit; b += wstride)
    swiglu_split_blocks<kNB>(a.g1, slab, split, static_cast<int>(b / (kKB2 / kNB)),
                             static_cast<int>(b % (kKB2 / kNB)) * kNB, lane, a.cq, a.c_scale, a.rows_cap);
}

// One 256-thread block per token (grid-stride over tokens).
__global__ void __launch_bounds__(256) combine_kernel(CombineArgs a) {
  griddep_launch_dependents();
  griddep_wait();
  const MoeSched* sc = a.sched;
  const int split = sc->split2;
  const size_t slab = static_cast<size_t>(sc->n_sel_pad) * kH;
  for (int t = blockIdx.x; t < a.T; t += gridDim.x)
    combine_token(a.o, slab, split, __popc(a.local_mask[t]), a.tok_rows + t * kTopK, a.perm_weight,
                  a.out_rows ? a.out_rows[t] : a.out_bf16 + static_cast<size_t>(t) * kH);
}

}  // namespace

void launch_swiglu_split(const SwigluArgs& a, int T, cudaStream_t stream) {
  long long warps = static_cast<long long>(T) * kTopK * kKB2;
  long long blocks = (warps + 7) / 8;
  if (blocks > 8 * kNumSMs) blocks = 8 * kNumSMs;
  if (blocks < 1) blocks = 1;
  launch_pdl(swiglu_split_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, a);
}

void launch_combine(const CombineArgs& a, cudaStream_t stream) {
  long long blocks = a.T;
  if (blocks > 8 * kNumSMs) blocks = 8 * kNumSMs;
  if (blocks < 1) blocks = 1;
  launch_pdl(combine_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, a);
}

}  // namespace moe
