// Large-batch grouped FP8 GEMMs (more than 1024 tokens per call: 128-token tiles) with the
// stages around them fused into the epilogues.
//
//   GEMM1 + SwiGLU:  replaces gemm_fp8_fp8_grouped_kernel + swiglu_kernel of the reference
//     (moe/solution/cuda/moe.cu:1373-1785, 2125-2167).  The fp32 GEMM1 result never exists in memory:
//     one work item owns a (128-token tile, 128-column block jb of the SwiGLU output) pair; its weight
//     operand is 256 rows made of TWO 128-row TMA boxes, rows [jb*128, +128) of the first half of W13
//     and the same rows of the second half, so that x1 and x2 of the same 128 output columns meet in
//     one 128 x 256 accumulator tile (UMMA N = 256).  After the K loop a thread holds
//     C = silu(x2) * x1 (full-agent-pipeline/references/moe.py:187-193: the SECOND half goes through
//     silu) of its token row, the four threads of a row agree on the block's power-of-two scale, and C
//     goes out as the three e4m3 planes + scale that GEMM2 reads.  The wide tile is also what the
//     hardware wants: an SM takes in about 45 bytes per clock from L2, a 128 x 128 x 128 fp8 tile needs
//     32 KB per 256 tensor-pipe clocks (128 B / clock), a 128 x 256 tile 48 KB per 512 (96 B / clock).
//   GEMM2 (+ combine):  replaces gemm_fp32_fp8w_fused_acc_grouped_kernel and fin_cast8_kernel
//     (moe.cu:2186-2431, 2473-2496).  COMBINE = false stores fp32 rows for the deterministic
//     combine kernel (ascending expert order, the order of references/moe.py:196-200).
//     COMBINE = true is the reference's own scheme (moe.cu:2404-2430): the epilogue multiplies by
//     the routing weight and adds into an fp32 [T, 7168] accumulator with 16-byte vector
//     reductions; a counter per (token, 128-column tile) tells the LAST contributor, which casts
//     the finished 128 columns to bf16 and writes them to the output.  No thread ever waits for
//     another one, but the fp32 summation order is whatever the hardware makes it.
//
// Orientation: the token tile is the UMMA M operand (TMEM lanes), the weight rows the N operand
// (TMEM columns), so a promotion thread owns ONE token row and the 128-block scale product of a
// K-block is one value per thread: f = a_scale[row, kb] * w_scale[e, block, kb].  The scales are
// arbitrary fp32, so every K-block is accumulated into its own TMEM columns and promoted with one
// FMA per element (they cannot ride on the hardware's power-of-two block scaling).
//
// Roles (640 threads, one CTA per SM):
//   warp 0      TMA producer (one thread; SWIZZLE_128B boxes, no multicast)
//   warps 1, 2  UMMA issuers (one thread each, alternate pipeline stages)
//   warps 4-19  promotion + epilogue: four warps per TMEM lane quarter, each owning a quarter of the
//               accumulator columns.  Sixteen warps (four per scheduler) so that the TMEM read-back
//               latency of one warp is covered by the FMAs of the others; with eight the read-back
//               latency was exposed in every K-block and the tensor pipe sat idle two thirds of the time.
// Every wait is bounded (ptx.cuh); a timeout raises the CTA's abort flag, all roles fall through to
// the normal teardown (TMEM freed) and an error bit is left in the schedule block.
#include "epilogue_device.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace moe {
namespace {

constexpr int kLEpiWarps = 16;
constexpr int kLFirstEpi = 4;
constexpr int kLEpiThreads = kLEpiWarps * 32;
constexpr int kLThreads = (kLFirstEpi + kLEpiWarps) * 32;   // 640
// setmaxnreg: the launch allocates kLRegsAtLaunch per thread (65536 / 640 rounded down to 8); the control
// warpgroup gives registers away, the four promotion warpgroups take them.
constexpr int kLRegsAtLaunch = 96;
constexpr int kLRegsControl = 32;
constexpr int kLRegsEpi = 112;
static_assert(128 * kLRegsControl + kLEpiThreads * kLRegsEpi <= kLRegsAtLaunch * kLThreads,
              "register reallocation would never complete");

template <int GEMM>
struct LCfg {
  static constexpr int KB = GEMM == 1 ? kKB1 : kKB2;             // K-blocks of the contraction
  static constexpr int J = GEMM == 1 ? kKB2 : kMT2 / 2;          // weight-side units per token tile: 16 / 28
  static constexpr int NTERMS = GEMM == 1 ? 1 : kNTerms;         // e4m3 planes of the token operand
  static constexpr int W_ROWS = 256;                             // weight rows of an item = UMMA N = TMEM columns per K-block
  static constexpr int W_BYTES = W_ROWS * 128;                   // one K-block of the weight operand
  static constexpr int TOK_BYTES = 128 * 128;                    // one K-block of 128 token rows (one plane)
  static constexpr int STAGE_BYTES = W_BYTES + NTERMS * TOK_BYTES;   // one K-block per pipeline stage: 48 KB / 80 KB
  static constexpr int STAGES = GEMM == 1 ? 4 : 2;
  static constexpr int BUF_COLS = W_ROWS;                        // TMEM columns of one stage's partial sums
  static constexpr int NBUF = 2;                                 // not deeper than the stage ring
  static constexpr int TMEM_COLS = 512;
  static constexpr int AUX_BYTES = 4096;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + AUX_BYTES + 1024;
  static_assert(NBUF * BUF_COLS <= TMEM_COLS && NBUF <= STAGES, "TMEM ring");
  static_assert(SMEM_BYTES <= 227 * 1024 && SMEM_BYTES > 116 * 1024, "one CTA per SM");
};

struct LAux {
  uint64_t full[4];        // TMA -> issuer
  uint64_t done[4];        // issuer -> producer and promotion warps
  uint64_t tempty[4];      // promotion warps -> issuer
  uint64_t esync;          // all promotion threads meet (bounded replacement of a named barrier)
  uint32_t tmem_base;
  int abort;
  int prefix[kELocal + 1];
  int offs[kELocal + 1];
  float amax[4][128];      // per column group and token row: |C| maximum of the thread's columns
};
static_assert(sizeof(LAux) <= 4096, "LAux must fit its slot");

struct LItem {
  int e, j, row0, valid;
};

// Item i -> (expert, weight-side unit j, token tile); token tiles of one weight unit are adjacent, so that
// CTAs working at the same time read the same weight rows (they come from HBM once, then from L2).
template <int GEMM>
__device__ __forceinline__ LItem decode_large(int i, const LAux* aux) {
  constexpr int J = LCfg<GEMM>::J;
  int e = 0;   // largest e with prefix[e] * J <= i (experts without tiles repeat the prefix value)
#pragma unroll 1
  for (int k = 16; k > 0; k >>= 1)
    if (e + k < kELocal && aux->prefix[e + k] * J <= i) e += k;
  const int r = i - aux->prefix[e] * J;
  const int tiles_e = aux->prefix[e + 1] - aux->prefix[e];
  const int n = r % tiles_e;
  LItem it;
  it.e = e;
  it.j = r / tiles_e;
  const int cnt = aux->offs[e + 1] - aux->offs[e];
  it.row0 = aux->offs[e] + n * 128;
  it.valid = min(128, cnt - n * 128);
  return it;
}

// acc[0..32) += v[0..32) * f with the packed two-element fp32 FMA of sm_100 (each element is one IEEE fma, the
// same result as fmaf): half the instructions of the scalar form, and the promotion warps are issue-bound.
__device__ __forceinline__ void fma32(float* acc, const float* v, float f) {
  const float2 ff = make_float2(f, f);
#pragma unroll
  for (int x = 0; x < 16; ++x) {
    const float2 r = __ffma2_rn(make_float2(v[2 * x], v[2 * x + 1]), ff, make_float2(acc[2 * x], acc[2 * x + 1]));
    acc[2 * x] = r.x;
    acc[2 * x + 1] = r.y;
  }
}

__device__ __forceinline__ void red_add_v4(float* p, float x, float y, float z, float w) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}

template <int GEMM, bool COMBINE>
__global__ void __launch_bounds__(kLThreads, 1)
grouped_gemm_large_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_b,
                          const __grid_constant__ GemmArgs a) {
  using C = LCfg<GEMM>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  LAux* aux = reinterpret_cast<LAux*>(smem + C::STAGES * C::STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  griddep_launch_dependents();
  MoeSched* sched = a.sched;
  // everything that does not depend on earlier kernels first: barriers, descriptors, TMEM
  if (threadIdx.x == 0) {
    aux->abort = 0;
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(smem_u32(&aux->full[s]), 1);
      mbar_init(smem_u32(&aux->done[s]), 1);
    }
    for (int b = 0; b < C::NBUF; ++b) mbar_init(smem_u32(&aux->tempty[b]), kLEpiWarps);
    mbar_init(smem_u32(&aux->esync), kLEpiThreads);
    fence_mbar_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&aux->tmem_base), C::TMEM_COLS);
    tmem_relinquish();
  }
  griddep_wait();   // the schedule, the operands and the outputs belong to earlier kernels until here
  const int items = GEMM == 1 ? sched->items1 : sched->items2;
  if (threadIdx.x <= kELocal) {
    aux->prefix[threadIdx.x] = GEMM == 1 ? sched->tile_prefix[threadIdx.x] : sched->tile_prefix2[threadIdx.x];
    aux->offs[threadIdx.x] = sched->offs[threadIdx.x];
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = aux->tmem_base;
  volatile int* abort_flag = &aux->abort;

  if (warp < kLFirstEpi) {
    setmaxnreg_dec<kLRegsControl>();
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        const uint32_t smem_base = smem_u32(smem);
        const uint32_t full_base = smem_u32(&aux->full[0]), done_base = smem_u32(&aux->done[0]);
        uint32_t stage = 0, ph = 0;
        bool ok = true;
        for (int i = blockIdx.x; ok && i < items; i += gridDim.x) {
          const LItem w = decode_large<GEMM>(i, aux);
#pragma unroll 1
          for (int kb = 0; kb < C::KB; ++kb) {
            if (!mbar_wait(done_base + stage * 8, ph ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t bar = full_base + stage * 8;
            mbar_arrive_expect_tx(bar, C::STAGE_BYTES);
            const uint32_t dst = smem_base + stage * C::STAGE_BYTES;
            if constexpr (GEMM == 1) {
              // weights: 128 rows of the first half of W13 | the same 128 rows of the second half
              const int y = w.e * k2I + w.j * 128;
              tma_load_3d(dst, &tm_w, 0, y, kb, bar);
              tma_load_3d(dst + 128 * 128, &tm_w, 0, y + kI, kb, bar);
              tma_load_3d(dst + C::W_BYTES, &tm_b, 0, w.row0, kb, bar);                   // [128 rows][128 B]
            } else {
              tma_load_3d(dst, &tm_w, 0, w.e * kH + w.j * 256, kb, bar);                  // 256 weight rows as two boxes
              tma_load_3d(dst + 128 * 128, &tm_w, 0, w.e * kH + w.j * 256 + 128, kb, bar);
              tma_load_4d(dst + C::W_BYTES, &tm_b, 0, w.row0, 0, kb, bar);                // [3 planes][128 rows][128 B]
            }
            if (++stage == C::STAGES) { stage = 0; ph ^= 1u; }
          }
        }
      }
      __syncwarp();   // block-wide barriers below need whole warps
    } else if (warp == 1 || warp == 2) {
      // ------------------------------------------------------------------ UMMA issuers (alternate stages)
      if (lane == 0) {
        constexpr uint32_t idesc = umma_idesc_e4m3(128, C::W_ROWS);
        const uint64_t desc_const = umma_desc_k_sw128(0);
        const uint32_t smem_base = smem_u32(smem);
        const uint32_t full_base = smem_u32(&aux->full[0]), done_base = smem_u32(&aux->done[0]);
        const uint32_t tempty_base = smem_u32(&aux->tempty[0]);
        uint32_t stage = 0, ph = 0, buf = 0, bph = 0;
        bool ok = true;
        int nst = 0;
        for (int i = blockIdx.x; ok && i < items; i += gridDim.x) {
#pragma unroll 1
          for (int s = 0; s < C::KB; ++s, ++nst) {
            if ((nst & 1) == warp - 1) {
              if (!mbar_wait(tempty_base + buf * 8, bph ^ 1u, abort_flag)) { ok = false; break; }
              if (!mbar_wait(full_base + stage * 8, ph, abort_flag)) { ok = false; break; }
              tc_fence_after_sync();
              const uint32_t sbase = smem_base + stage * C::STAGE_BYTES;
              const uint64_t wdesc = desc_const | (sbase >> 4);
              const uint32_t d = tmem_base + buf * C::BUF_COLS;
#pragma unroll
              for (int t = 0; t < C::NTERMS; ++t) {
                const uint64_t tdesc = desc_const | ((sbase + C::W_BYTES + t * C::TOK_BYTES) >> 4);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4)   // +32 bytes of K inside the 128-byte swizzle atom = +2 encoded units
                  umma_f8(d, tdesc + 2 * k4, wdesc + 2 * k4, idesc, (t | k4) != 0 ? 1u : 0u);
              }
              umma_commit(done_base + stage * 8);
            }
            if (++stage == C::STAGES) { stage = 0; ph ^= 1u; }
            if (++buf == C::NBUF) { buf = 0; bph ^= 1u; }
          }
        }
      }
      __syncwarp();
    }
  } else {
    setmaxnreg_inc<kLRegsEpi>();
    // ------------------------------------------------------------------ promotion + epilogue (warps 4..19)
    const int q = warp & 3;                       // TMEM lane quarter this warp may access
    const int cg = (warp - kLFirstEpi) >> 2;      // column group: a quarter of the accumulator columns
    const int trow = q * 32 + lane;               // token row inside the tile
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t done_base = smem_u32(&aux->done[0]), tempty_base = smem_u32(&aux->tempty[0]);
    uint32_t stage = 0, ph = 0, buf = 0, bph = 0;      // same ring positions as the issuers
    uint32_t eph = 0;
    bool ok = true;
    auto epi_sync = [&]() {
      mbar_arrive(smem_u32(&aux->esync));
      if (!mbar_wait(smem_u32(&aux->esync), eph, abort_flag)) ok = false;
      eph ^= 1u;
    };
    for (int i = blockIdx.x; ok && i < items; i += gridDim.x) {
      const LItem w = decode_large<GEMM>(i, aux);
      const int row = w.row0 + trow;
      const int lrow = min(row, a.rows_cap - 1);   // rows past the tile's last one are computed and dropped
      if constexpr (GEMM == 1) {
        // scales of this thread's token row and of the item's two weight blocks, read one K-block ahead
        const float* bsp = a.b_scale + static_cast<size_t>(lrow) * kKB1;
        const float* w1p = a.w_scale + (static_cast<size_t>(w.e) * kMT1 + w.j) * kKB1;
        const float* w2p = w1p + kKB2 * kKB1;   // the block 16 further: the second half of W13
        float acc[64];      // [0, 32): x1 of this thread's 32 columns, [32, 64): x2 of the same columns
#pragma unroll
        for (int x = 0; x < 64; ++x) acc[x] = 0.0f;
        float nb = __ldg(bsp), n1 = __ldg(w1p), n2 = __ldg(w2p);
#pragma unroll 1
        for (int s = 0; s < kKB1; ++s) {
          if (!mbar_wait(done_base + stage * 8, ph, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t taddr = tmem_base + lane_addr + buf * C::BUF_COLS + cg * 32;
          float v[32];
          tmem_ld32(taddr, v);                  // x1: columns cg*32 .. +32 of the first 128
          // (scale arithmetic and the next K-block's scale loads run under the read-back's latency)
          const float f1 = n1 * nb, f2 = n2 * nb;
          if (s + 1 < kKB1) { nb = __ldg(bsp + s + 1); n1 = __ldg(w1p + s + 1); n2 = __ldg(w2p + s + 1); }
          tmem_wait_ld();
          fma32(acc, v, f1);
          tmem_ld32(taddr + 128, v);            // x2: the same columns of the second 128
          tmem_wait_ld();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_base + buf * 8);
          fma32(acc + 32, v, f2);
          if (++stage == C::STAGES) { stage = 0; ph ^= 1u; }
          if (++buf == C::NBUF) { buf = 0; bph ^= 1u; }
        }
        if (!ok) break;
        float amax = 0.0f;
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          acc[x] = swiglu_value(acc[x], acc[32 + x]);
          amax = fmaxf(amax, fabsf(acc[x]));
        }
        aux->amax[cg][trow] = amax;
        epi_sync();      // the four threads of a row have published their maxima
        if (!ok) break;
        amax = fmaxf(fmaxf(aux->amax[0][trow], aux->amax[1][trow]), fmaxf(aux->amax[2][trow], aux->amax[3][trow]));
        const int ex = plane_scale_exponent(amax);
        const float inv = __uint_as_float(static_cast<uint32_t>(127 - ex) << 23);
        if (trow < w.valid) {
          uint32_t pk[kNTerms][8];
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            uint8_t t3[kNTerms];
            split_e4m3_terms(acc[x] * inv, t3);
#pragma unroll
            for (int t = 0; t < kNTerms; ++t) {
              if ((x & 3) == 0) pk[t][x >> 2] = 0;
              pk[t][x >> 2] |= static_cast<uint32_t>(t3[t]) << (8 * (x & 3));
            }
          }
#pragma unroll
          for (int t = 0; t < kNTerms; ++t) {
            uint4* dst = reinterpret_cast<uint4*>(a.cq + (static_cast<size_t>(t) * a.rows_cap + row) * kI + w.j * kBlock + cg * 32);
            dst[0] = make_uint4(pk[t][0], pk[t][1], pk[t][2], pk[t][3]);
            dst[1] = make_uint4(pk[t][4], pk[t][5], pk[t][6], pk[t][7]);
          }
          if (cg == 0) a.c_scale[static_cast<size_t>(row) * kKB2 + w.j] = __uint_as_float(static_cast<uint32_t>(ex + 127) << 23);
        }
      } else {
        // this thread's 64 columns lie in ONE 128-row weight block: 2 j + (cg >> 1)
        const int tile = 2 * w.j + (cg >> 1);
        const float* bsp = a.b_scale + static_cast<size_t>(lrow) * kKB2;
        const float* wsp = a.w_scale + (static_cast<size_t>(w.e) * kMT2 + tile) * kKB2;
        float acc[64];
#pragma unroll
        for (int x = 0; x < 64; ++x) acc[x] = 0.0f;
        float nb = __ldg(bsp), nw = __ldg(wsp);
#pragma unroll 1
        for (int s = 0; s < kKB2; ++s) {
          if (!mbar_wait(done_base + stage * 8, ph, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t taddr = tmem_base + lane_addr + buf * C::BUF_COLS + cg * 64;
          float v[32];
          tmem_ld32(taddr, v);
          const float f = nw * nb;
          if (s + 1 < kKB2) { nb = __ldg(bsp + s + 1); nw = __ldg(wsp + s + 1); }
          tmem_wait_ld();
          fma32(acc, v, f);
          tmem_ld32(taddr + 32, v);
          tmem_wait_ld();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_base + buf * 8);
          fma32(acc + 32, v, f);
          if (++stage == C::STAGES) { stage = 0; ph ^= 1u; }
          if (++buf == C::NBUF) { buf = 0; bph ^= 1u; }
        }
        if (!ok) break;
        if (trow < w.valid) {
          const int col0 = w.j * 256 + cg * 64;
          if constexpr (!COMBINE) {
            float* out = a.out + static_cast<size_t>(row) * kH + col0;
#pragma unroll
            for (int x = 0; x < 8; ++x) st_global_v8(out + 8 * x, acc + 8 * x);   // whole 32-byte sectors
          } else {
            const int t = __ldcg(a.perm_token + row);
            const float pw = __ldcg(a.perm_weight + row);
            float* dst = a.acc32 + static_cast<size_t>(t) * kH + col0;
#pragma unroll
            for (int x = 0; x < 16; ++x)
              red_add_v4(dst + 4 * x, __fmul_rn(acc[4 * x], pw), __fmul_rn(acc[4 * x + 1], pw), __fmul_rn(acc[4 * x + 2], pw),
                         __fmul_rn(acc[4 * x + 3], pw));
            __threadfence();      // the reductions above are performed before the arrival below is
            const int target = 2 * __popc(__ldcg(a.local_mask + t));   // two threads per (row, 128-column tile)
            const int old = atomicAdd(a.tile_cnt + static_cast<size_t>(t) * kMT2 + tile, 1);
            if (old == target - 1) {
              // last contributor of (token, column tile): all 128 sums are complete
              __threadfence();
              const float4* src = reinterpret_cast<const float4*>(a.acc32 + static_cast<size_t>(t) * kH + tile * 128);
              uint16_t* orow = (a.out_rows ? a.out_rows[t] : a.out_bf16 + static_cast<size_t>(t) * kH) + tile * 128;
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                float4 u[16];
#pragma unroll
                for (int x = 0; x < 16; ++x) u[x] = __ldcg(src + h * 16 + x);
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                  uint4 o;
                  o.x = pack_bf16x2(u[2 * x].x, u[2 * x].y);
                  o.y = pack_bf16x2(u[2 * x].z, u[2 * x].w);
                  o.z = pack_bf16x2(u[2 * x + 1].x, u[2 * x + 1].y);
                  o.w = pack_bf16x2(u[2 * x + 1].z, u[2 * x + 1].w);
                  reinterpret_cast<uint4*>(orow)[h * 8 + x] = o;
                }
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && aux->abort) atomicOr(&sched->status, GEMM == 1 ? kErrGemm1Timeout : kErrGemm2Timeout);
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// Before a GEMM2 launch with the fused combine: clears the fp32 accumulator and the arrival counters, and
// writes the output rows of tokens without a local expert (all zeros; nobody else will).
__global__ void __launch_bounds__(256) combine_prepare_kernel(float4* acc, size_t n_vec, const uint32_t* local_mask, int T,
                                                              uint16_t* out_bf16, uint16_t* const* out_rows) {
  griddep_launch_dependents();
  griddep_wait();
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    acc[i] = z;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    if (local_mask[t] != 0) continue;
    uint4* row = reinterpret_cast<uint4*>(out_rows ? out_rows[t] : out_bf16 + static_cast<size_t>(t) * kH);
    for (int c = threadIdx.x; c < kH * 2 / 16; c += blockDim.x) row[c] = make_uint4(0u, 0u, 0u, 0u);
  }
}

template <int GEMM, bool COMBINE>
int init_large() {
  return static_cast<int>(cudaFuncSetAttribute(grouped_gemm_large_kernel<GEMM, COMBINE>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, LCfg<GEMM>::SMEM_BYTES));
}

}  // namespace

int grouped_gemm_large_init() {
  int rc = 0;
  if ((rc = init_large<1, false>())) return rc;
  if ((rc = init_large<2, false>())) return rc;
  if ((rc = init_large<2, true>())) return rc;
  return 0;
}

int launch_grouped_gemm_large(int gemm_id, bool fused_combine, const CUtensorMap& tm_w, const CUtensorMap& tm_b,
                              const GemmArgs& a, int ctas, cudaStream_t stream) {
  if (gemm_id == 1)
    return static_cast<int>(launch_pdl(grouped_gemm_large_kernel<1, false>, dim3(ctas), dim3(kLThreads),
                                       LCfg<1>::SMEM_BYTES, stream, tm_w, tm_b, a));
  if (fused_combine)
    return static_cast<int>(launch_pdl(grouped_gemm_large_kernel<2, true>, dim3(ctas), dim3(kLThreads),
                                       LCfg<2>::SMEM_BYTES, stream, tm_w, tm_b, a));
  return static_cast<int>(launch_pdl(grouped_gemm_large_kernel<2, false>, dim3(ctas), dim3(kLThreads), LCfg<2>::SMEM_BYTES,
                                     stream, tm_w, tm_b, a));
}

int launch_combine_prepare(float* acc32, size_t acc_floats, const uint32_t* local_mask, int T, uint16_t* out_bf16,
                           uint16_t* const* out_rows, cudaStream_t stream) {
  const size_t n_vec = acc_floats / 4;
  size_t blocks = (n_vec + 255) / 256;
  if (blocks > 16 * kNumSMs) blocks = 16 * kNumSMs;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(launch_pdl(combine_prepare_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream,
                                     reinterpret_cast<float4*>(acc32), n_vec, local_mask, T, out_bf16, out_rows));
}

}  // namespace moe
