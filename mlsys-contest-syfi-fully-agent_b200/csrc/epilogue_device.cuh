// Device functions shared by the stand-alone SwiGLU / combine kernels and the
// decode-fused GEMM kernels (which run them as a tail phase after a grid barrier).
#pragma once
#include <cuda_fp8.h>

#include "kernels.h"

namespace moe {

__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float from_e4m3(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(__half(h));
}

// One element of the SwiGLU output: C = silu(x2) * x1 with IEEE exp and division
// (full-agent-pipeline/references/moe.py:187-193: the second half of GEMM1's result goes through silu).
__device__ __forceinline__ float swiglu_value(float x1, float x2) {
  return __fmul_rn(x2 / (1.0f + expf(-x2)), x1);
}

// Exponent e of the power-of-two plane scale 2^e of a 128-column block with |C| maximum `amax`:
// amax / 2^e lies in (224, 448]: e = floor(log2(amax / 448)) + 1, clamped to [-100, 100]; read from the
// exponent field (a denormal quotient clamps to -100 either way).  0 for an all-zero or non-finite block.
__device__ __forceinline__ int plane_scale_exponent(float amax) {
  int e = 0;
  if (amax > 0.0f && amax < 3.0e38f) {
    e = static_cast<int>((__float_as_uint(amax * (1.0f / 448.0f)) >> 23) & 0xFFu) - 127 + 1;
    e = max(-100, min(100, e));
  }
  return e;
}

// r (already divided by the plane scale) as kNTerms e4m3 terms: t_i = e4m3(residual after t_0 .. t_{i-1}).
__device__ __forceinline__ void split_e4m3_terms(float r, uint8_t* t) {
  if (!(fabsf(r) <= 448.0f)) r = r > 0.0f ? 448.0f : (r < 0.0f ? -448.0f : 0.0f);   // inf / nan guard
#pragma unroll
  for (int i = 0; i < kNTerms; ++i) {
    t[i] = to_e4m3(r);
    r -= from_e4m3(t[i]);
  }
}

// SwiGLU of 4 columns per lane of one (row, 128-column block), split of the result into kNTerms e4m3
// planes with one power-of-two scale for the block.
__device__ __forceinline__ void swiglu_finish_block(const float4 x1, const float4 x2, int row, int kb, int lane, uint8_t* cq,
                                                    float* c_scale, int rows_cap) {
  float c[4];
  c[0] = swiglu_value(x1.x, x2.x);
  c[1] = swiglu_value(x1.y, x2.y);
  c[2] = swiglu_value(x1.z, x2.z);
  c[3] = swiglu_value(x1.w, x2.w);
  float amax = fmaxf(fmaxf(fabsf(c[0]), fabsf(c[1])), fmaxf(fabsf(c[2]), fabsf(c[3])));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, d));
  const int e = plane_scale_exponent(amax);
  const float scale = __uint_as_float(static_cast<uint32_t>(e + 127) << 23);
  const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
  uint32_t packed[kNTerms];
#pragma unroll
  for (int t = 0; t < kNTerms; ++t) packed[t] = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint8_t q[kNTerms];
    split_e4m3_terms(c[i] * inv, q);
#pragma unroll
    for (int t = 0; t < kNTerms; ++t) packed[t] |= static_cast<uint32_t>(q[t]) << (8 * i);
  }
#pragma unroll
  for (int t = 0; t < kNTerms; ++t)
    *reinterpret_cast<uint32_t*>(cq + (static_cast<size_t>(t) * rows_cap + row) * kI + kb * kBlock + lane * 4) =
        packed[t];
  if (lane == 0) c_scale[static_cast<size_t>(row) * kKB2 + kb] = scale;
}

// SwiGLU + e4m3 split of NB consecutive 128-column blocks of one row by one warp; lane owns 4
// columns of each block.  `g1` points at the first split-K slab; slabs are `slab` floats apart.
// All loads of the NB blocks are issued before any arithmetic (memory-level parallelism), and they
// bypass L1 (the slabs may have been written by other SMs in the same kernel).
template <int NB>
__device__ __forceinline__ void swiglu_split_blocks(const float* g1, size_t slab, int split, int row, int kb0, int lane,
                                                    uint8_t* cq, float* c_scale, int rows_cap) {
  float4 x1[NB], x2[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) x1[b] = x2[b] = make_float4(0.f, 0.f, 0.f, 0.f);
  // four slabs' loads in flight at a time; the sum keeps the slab order
  constexpr int kAhead = 4;
  for (int s0 = 0; s0 < split; s0 += kAhead) {
    float4 u[kAhead][NB], v[kAhead][NB];
#pragma unroll
    for (int d = 0; d < kAhead; ++d) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        if (s0 + d < split) {
          const float* p = g1 + (s0 + d) * slab + static_cast<size_t>(row) * k2I + (kb0 + b) * kBlock + lane * 4;
          u[d][b] = __ldcg(reinterpret_cast<const float4*>(p));
          v[d][b] = __ldcg(reinterpret_cast<const float4*>(p + kI));
        } else {
          u[d][b] = v[d][b] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    }
#pragma unroll
    for (int d = 0; d < kAhead; ++d) {
      if (s0 + d < split) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          x1[b].x += u[d][b].x; x1[b].y += u[d][b].y; x1[b].z += u[d][b].z; x1[b].w += u[d][b].w;
          x2[b].x += v[d][b].x; x2[b].y += v[d][b].y; x2[b].z += v[d][b].z; x2[b].w += v[d][b].w;
        }
      }
    }
  }
#pragma unroll
  for (int b = 0; b < NB; ++b) swiglu_finish_block(x1[b], x2[b], row, kb0 + b, lane, cq, c_scale, rows_cap);
}

__device__ __forceinline__ void swiglu_split_unit(const float* g1, size_t slab, int split, int row, int kb, int lane,
                                                  uint8_t* cq, float* c_scale, int rows_cap) {
  swiglu_split_blocks<1>(g1, slab, split, row, kb, lane, cq, c_scale, rows_cap);
}

// The same for one block whose two halves have their own numbers of slabs (balanced partition of the
// decode kernel): x1 = sum of n1 slabs, x2 = sum of n2 slabs, each in slab order.
__device__ __forceinline__ void swiglu_split_unit2(const float* g1, size_t slab, int n1, int n2, int row, int kb, int lane,
                                                   uint8_t* cq, float* c_scale, int rows_cap) {
  constexpr int kMax = 8;
  const float* p = g1 + static_cast<size_t>(row) * k2I + kb * kBlock + lane * 4;
  float4 u[kMax], v[kMax];
#pragma unroll
  for (int s = 0; s < kMax; ++s) {
    u[s] = s < n1 ? __ldcg(reinterpret_cast<const float4*>(p + s * slab)) : make_float4(0.f, 0.f, 0.f, 0.f);
    v[s] = s < n2 ? __ldcg(reinterpret_cast<const float4*>(p + s * slab + kI)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float4 x1 = u[0], x2 = v[0];
#pragma unroll
  for (int s = 1; s < kMax; ++s) {
    if (s < n1) { x1.x += u[s].x; x1.y += u[s].y; x1.z += u[s].z; x1.w += u[s].w; }
    if (s < n2) { x2.x += v[s].x; x2.y += v[s].y; x2.z += v[s].z; x2.w += v[s].w; }
  }
  swiglu_finish_block(x1, x2, row, kb, lane, cq, c_scale, rows_cap);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Weighted combine of 4 output columns of one token: the token's local experts in ascending
// order, each the sum of its GEMM2 split-K slabs (in slab order), multiply then add (the definition's
// index_add_(O * w), references/moe.py:196-200), bf16 round-to-nearest-even.  `slabs(j)` gives the
// number of slabs (<= kMaxSlabs) of the token's j-th row.  Rows are taken two at a time with all their
// slab loads in flight: the loads are L2 round trips and would otherwise run one after the other.
template <int kMaxSlabs, typename SlabCount>
__device__ __forceinline__ void combine_unit(const float* o, size_t slab, SlabCount slabs, int n_local, const int* rows,
                                             const float* perm_weight, int c, uint16_t* out_row) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j0 = 0; j0 < n_local; j0 += 2) {
    float4 u[2][kMaxSlabs];
    float w[2];
    int ns[2];
#pragma unroll
    for (int d = 0; d < 2; ++d) {
      const bool on = j0 + d < n_local;
      const int row = on ? rows[j0 + d] : 0;
      w[d] = on ? perm_weight[row] : 0.0f;
      ns[d] = on ? slabs(j0 + d) : 0;
      const float* p = o + static_cast<size_t>(row) * kH + c * 4;
#pragma unroll
      for (int s = 0; s < kMaxSlabs; ++s)
        u[d][s] = s < ns[d] ? __ldcg(reinterpret_cast<const float4*>(p + s * slab)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int d = 0; d < 2; ++d) {
      if (j0 + d < n_local) {
        float4 v = u[d][0];
#pragma unroll
        for (int s = 1; s < kMaxSlabs; ++s)
          if (s < ns[d]) { v.x += u[d][s].x; v.y += u[d][s].y; v.z += u[d][s].z; v.w += u[d][s].w; }
        acc.x = __fadd_rn(acc.x, __fmul_rn(v.x, w[d]));
        acc.y = __fadd_rn(acc.y, __fmul_rn(v.y, w[d]));
        acc.z = __fadd_rn(acc.z, __fmul_rn(v.z, w[d]));
        acc.w = __fadd_rn(acc.w, __fmul_rn(v.w, w[d]));
      }
    }
  }
  uint2 q;
  q.x = pack_bf16x2(acc.x, acc.y);
  q.y = pack_bf16x2(acc.z, acc.w);
  *reinterpret_cast<uint2*>(out_row + c * 4) = q;
}

// Weighted combine of a whole token by one 256-thread block: thread owns the float4 columns
// tid, tid + 256, ... (7 of them), so every row contributes seven independent loads per thread.
__device__ __forceinline__ void combine_token(const float* o, size_t slab, int split, int n_local, const int* rows,
                                              const float* perm_weight, uint16_t* out_row) {
  constexpr int kPer = kH / 4 / 256;   // 7
  float4 acc[kPer];
#pragma unroll
  for (int x = 0; x < kPer; ++x) acc[x] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j = 0; j < n_local; ++j) {
    const int row = rows[j];
    const float w = perm_weight[row];
    const float* p = o + static_cast<size_t>(row) * kH + threadIdx.x * 4;
    float4 v[kPer];
#pragma unroll
    for (int x = 0; x < kPer; ++x) v[x] = __ldcg(reinterpret_cast<const float4*>(p + x * 1024));
    for (int s = 1; s < split; ++s) {
#pragma unroll
      for (int x = 0; x < kPer; ++x) {
        const float4 u = __ldcg(reinterpret_cast<const float4*>(p + s * slab + x * 1024));
        v[x].x += u.x; v[x].y += u.y; v[x].z += u.z; v[x].w += u.w;
      }
    }
#pragma unroll
    for (int x = 0; x < kPer; ++x) {
      acc[x].x = __fadd_rn(acc[x].x, __fmul_rn(v[x].x, w));
      acc[x].y = __fadd_rn(acc[x].y, __fmul_rn(v[x].y, w));
      acc[x].z = __fadd_rn(acc[x].z, __fmul_rn(v[x].z, w));
      acc[x].w = __fadd_rn(acc[x].w, __fmul_rn(v[x].w, w));
    }
  }
#pragma unroll
  for (int x = 0; x < kPer; ++x) {
    uint2 q;
    q.x = pack_bf16x2(acc[x].x, acc[x].y);
    q.y = pack_bf16x2(acc[x].z, acc[x].w);
    *reinterpret_cast<uint2*>(out_row + threadIdx.x * 4 + x * 1024) = q;
  }
}

}  // namespace moe
