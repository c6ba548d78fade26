// Pieces shared by the grouped GEMM kernel and the single-launch decode kernel: the thread layout,
// the per-CTA barrier block, the grid barrier, and the in-kernel routing + schedule of the decode path.
#pragma once
#include "kernels.h"
#include "ptx.cuh"
#include "route_device.cuh"

#ifndef MOE_ROUTE_TRACE
#define MOE_ROUTE_TRACE(slot) do { } while (0)   // debug builds of an including file may stamp the routing phases
#endif

namespace moe {

// Three warpgroups: warpgroup 0 holds the TMA producer (warp 0) and the UMMA issuer (warp 1) and gives
// most of its registers away (setmaxnreg); warpgroups 1 and 2 are the eight promotion / epilogue warps
// (warp % 4 = the TMEM lane quarter a warp may access) and take them.
constexpr int kEpiWarps = 8;
constexpr int kFirstEpiWarp = 4;
constexpr int kGemmThreads = (kFirstEpiWarp + kEpiWarps) * 32;
constexpr int kRegsControl = 96;     // per thread in warpgroup 0 after the role split
constexpr int kRegsEpilogue = 200;   // per thread in warpgroups 1 and 2
// setmaxnreg.inc waits (unboundedly) for registers released by setmaxnreg.dec: the new total must fit
// in what the launch allocated, 168 registers (the launch-bounds cap for 384 threads) per thread.
constexpr int kRegsAtLaunch = 168;
static_assert(128 * kRegsControl + 256 * kRegsEpilogue <= kRegsAtLaunch * kGemmThreads, "register reallocation would never complete");
static_assert(kRegsControl % 8 == 0 && kRegsEpilogue % 8 == 0, "setmaxnreg takes multiples of 8");

struct Aux {
  uint64_t full[10];       // TMA -> issuer: the stage's operands have landed
  uint64_t done[10];       // issuer -> producer and promotion warps: the stage's UMMAs have completed
  uint64_t tempty[4];      // promotion warps -> issuer: the TMEM buffer has been read
  uint64_t esync;          // bounded replacement for a named barrier among the epilogue threads
  uint32_t tmem_base;
  int abort;
  int prefix[kELocal + 1];
  int offs[kELocal + 1];
};
static_assert(sizeof(Aux) <= 1024, "Aux must fit its slot");

// Extra shared state of the decode-fused kernels: every CTA routes all (<= 16) tokens itself.
struct FusedAux {
  uint32_t keys[kEGlobal];            // order-preserving keys of the biased scores of the token being routed
  float sval[kEGlobal];               // its unbiased sigmoid scores
  float gscore[kNGroup];
  int selidx[kTopK];
  float sels[kTopK];
  int tidx[kFusedMaxTokens][kTopK];
  float tw[kFusedMaxTokens][kTopK];
  uint32_t mask[kFusedMaxTokens];     // per token: selected local experts
  uint32_t colmask[kELocal];          // per local expert: tokens that selected it
  int items, split, n_sel_pad, n_sel;      // GEMM1 items / split-K factor, slab stride, rows
  int items2, split2;                      // GEMM2 items / split-K factor
};
static_assert(sizeof(FusedAux) <= 4096, "FusedAux must fit its slot");

// Grid-wide barrier for a grid whose CTAs are all resident (one per SM).  The 64-bit word holds
// {arrivals, call tag}.  CTA 0 installs {0, tag} when the kernel starts (after the wait on earlier
// kernels, long before anybody arrives); an arriving CTA first checks that the tag is the current
// call's, then adds one, then waits for `n` arrivals.  So the word needs no initialisation by the
// caller and no reset between calls, and an arrival is one atomic add.  Bounded like every other
// wait here: false on timeout.
__device__ __forceinline__ void grid_barrier_init(unsigned int* word2, unsigned int tag) {
  atomicExch(reinterpret_cast<unsigned long long*>(word2), static_cast<unsigned long long>(tag) << 32);
}

__device__ __forceinline__ bool grid_barrier(unsigned int* word2, unsigned int tag, unsigned int n) {
  unsigned long long* word = reinterpret_cast<unsigned long long*>(word2);
  __threadfence();
  const uint64_t t0 = globaltimer_ns();
  unsigned int spins = 0;
  while (static_cast<unsigned int>(*reinterpret_cast<volatile unsigned long long*>(word) >> 32) != tag)
    if ((++spins & 0xFFu) == 0 && globaltimer_ns() - t0 > MOE_WAIT_LIMIT_NS) return false;
  atomicAdd(word, 1ull);
  while (true) {
    const unsigned long long v = *reinterpret_cast<volatile unsigned long long*>(word);
    if (static_cast<unsigned int>(v) >= n) break;
    if ((++spins & 0xFFu) == 0 && globaltimer_ns() - t0 > MOE_WAIT_LIMIT_NS) return false;
  }
  __threadfence();
  return true;
}

// The same barrier in separate steps, for a word that serves several successive barriers of one launch
// (the k-th is complete at k * gridDim.x arrivals) and for waiters that do not arrive (a TMA producer).
// One thread per CTA calls them after a CTA-wide synchronisation: its release / acquire operations at
// GPU scope are cumulative over what the other threads of the CTA wrote before that synchronisation.
//
// Wait (bounded) until CTA 0 has installed this launch's tag; call once, early, off the critical path.
__device__ __forceinline__ bool grid_barrier_tag_wait(unsigned int* word2, unsigned int tag) {
  const uint64_t t0 = globaltimer_ns();
  unsigned int spins = 0;
  while (static_cast<unsigned int>(*reinterpret_cast<volatile unsigned long long*>(word2) >> 32) != tag)
    if ((++spins & 0xFFu) == 0 && globaltimer_ns() - t0 > MOE_WAIT_LIMIT_NS) return false;
  return true;
}

__device__ __forceinline__ void grid_barrier_arrive(unsigned int* word2) {
  asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(word2), "l"(1ull) : "memory");
}

// The tag is checked too: before CTA 0 has installed it the word still holds the previous launch's count.
__device__ __forceinline__ bool grid_barrier_wait(unsigned int* word2, unsigned int tag, unsigned int n) {
  const uint64_t t0 = globaltimer_ns();
  unsigned int spins = 0;
  while (true) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(word2) : "memory");
    if (static_cast<unsigned int>(v >> 32) == tag && static_cast<unsigned int>(v) >= n) return true;
    if ((++spins & 0xFFu) == 0 && globaltimer_ns() - t0 > MOE_WAIT_LIMIT_NS) return false;
  }
}

// K-blocks per pipeline stage of the 16-token kernels of both GEMMs (split-K granularity).
constexpr int kDecodeKps = 2;

// CPW fp32 columns of this warp's 32 TMEM lanes -> registers.
template <int CPW>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, float* v) {
  if constexpr (CPW == 8) {
    tmem_ld8(taddr, v);
  } else if constexpr (CPW == 16) {
    tmem_ld16(taddr, v);
  } else {
#pragma unroll
    for (int c = 0; c < CPW / 32; ++c) tmem_ld32(taddr + c * 32, v + c * 32);
  }
}

// Decode path (T <= 16): no routing / permutation / gather kernels run.  Every CTA routes all tokens
// and derives the same schedule in shared memory (aux->offs / prefix, fa->*); CTA 0 also publishes the
// selection, the permutation and the schedule block.  `smem` is shared memory that is idle until
// the first TMA load (the stage ring).  Called by all threads of the CTA.
__device__ __forceinline__ void decode_route_schedule(const GemmArgs& a, uint8_t* smem, Aux* aux, FusedAux* fa,
                                                      MoeSched* sched) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (a.T <= 2) {
    // Block-cooperative routing (same arithmetic and tie rules as route_token): thread e < 256 owns
    // expert e, so warp g is routing group g.  Per token: sigmoid + bias, the group's two best by
    // two warp reductions, then every kept expert counts how many kept experts beat it; the eight
    // with rank < 8 are the selection in descending order.  ~1k cycles per token instead of the
    // ~7k of one warp doing eight rounds of arg-max.
    const int e = threadIdx.x;
    float* xs = reinterpret_cast<float*>(smem);                 // [T][256] logits; the stage ring is still idle
    float bias_e = 0.0f;
    if (e < kEGlobal) {
      bias_e = __uint_as_float(static_cast<uint32_t>(a.bias_bf16[e]) << 16);
      for (int t = 0; t < a.T; ++t) xs[t * kEGlobal + e] = a.logits[static_cast<size_t>(t) * kEGlobal + e];
    }
    if (threadIdx.x == 0) MOE_ROUTE_TRACE(0);
    for (int t = 0; t < a.T; ++t) {
      float s_e = 0.0f;
      uint32_t key_e = 0;
      if (e < kEGlobal) {
        s_e = 1.0f / (1.0f + expf(-xs[t * kEGlobal + e]));
        key_e = order_key(s_e + bias_e);
        fa->keys[e] = key_e;
        fa->sval[e] = s_e;
        const uint32_t k1 = __reduce_max_sync(0xFFFFFFFFu, key_e);
        const int first = __ffs(__ballot_sync(0xFFFFFFFFu, key_e == k1)) - 1;
        const uint32_t k2 = __reduce_max_sync(0xFFFFFFFFu, lane == first ? 0u : key_e);
        const uint32_t u1 = (k1 & 0x80000000u) ? (k1 & 0x7FFFFFFFu) : ~k1;
        const uint32_t u2 = (k2 & 0x80000000u) ? (k2 & 0x7FFFFFFFu) : ~k2;
        if (lane == 0) fa->gscore[warp] = __uint_as_float(u1) + __uint_as_float(u2);
      }
      __syncthreads();
      if (e < kEGlobal) {
        uint32_t keep = 0;
#pragma unroll
        for (int g = 0; g < kNGroup; ++g) {
          int rank = 0;
#pragma unroll
          for (int h2 = 0; h2 < kNGroup; ++h2)
            rank += (fa->gscore[h2] > fa->gscore[g]) || (fa->gscore[h2] == fa->gscore[g] && h2 < g);
          keep |= (rank < kTopKGroup ? 1u : 0u) << g;
        }
        if ((keep >> warp) & 1u) {
          int rank = 0;
          for (int g = 0; g < kNGroup; ++g) {
            if (!((keep >> g) & 1u)) continue;
            const uint4* kv = reinterpret_cast<const uint4*>(fa->keys + g * 32);
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
          if (rank < kTopK) { fa->selidx[rank] = e; fa->sels[rank] = s_e; }
        }
      }
      __syncthreads();
      if (warp == 0) {
        const float sv = lane < kTopK ? fa->sels[lane] : 0.0f;
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < kTopK; ++k) sum += __shfl_sync(0xFFFFFFFFu, sv, k);
        sum += 1e-20f;
        uint32_t bit = 0;
        if (lane < kTopK) {
          const int idx = fa->selidx[lane];
          fa->tidx[t][lane] = idx;
          fa->tw[t][lane] = (sv / sum) * a.routed_scaling_factor;
          const int le = idx - a.local_expert_offset;
          if (le >= 0 && le < kELocal) bit = 1u << le;
        }
        bit = __reduce_or_sync(0xFFFFFFFFu, bit);
        if (lane == 0) fa->mask[t] = bit;
      }
    }
  } else {
    // More than two tokens: one warp per token (ten at a time), each doing the warp-level routing.
    float* bias_s = fa->sval;                                  // 256 floats, free on this path
    for (int i = threadIdx.x; i < kEGlobal; i += kGemmThreads)
      bias_s[i] = __uint_as_float(static_cast<uint32_t>(a.bias_bf16[i]) << 16);
    __syncthreads();
    for (int t = warp; t < a.T; t += kGemmThreads / 32) {
      int idx;
      float w;
      route_token(a.logits + static_cast<size_t>(t) * kEGlobal, bias_s, a.routed_scaling_factor, lane, idx, w);
      uint32_t bit = 0;
      if (lane < kTopK) {
        fa->tidx[t][lane] = idx;
        fa->tw[t][lane] = w;
        const int le = idx - a.local_expert_offset;
        if (le >= 0 && le < kELocal) bit = 1u << le;
      }
      bit = __reduce_or_sync(0xFFFFFFFFu, bit);
      if (lane == 0) fa->mask[t] = bit;
    }
  }
  if (threadIdx.x == 0) MOE_ROUTE_TRACE(1);
  fence_proxy_async_smem();   // the logits scratch is about to be overwritten by TMA (async proxy)
  __syncthreads();
  if (warp == 0) {                     // lane = local expert
    uint32_t cm = 0;
    for (int t = 0; t < a.T; ++t) cm |= ((fa->mask[t] >> lane) & 1u) << t;
    const int c = __popc(cm);
    int inc = c, tinc = c > 0 ? 1 : 0;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xFFFFFFFFu, inc, d);
      const int tv = __shfl_up_sync(0xFFFFFFFFu, tinc, d);
      if (lane >= d) { inc += v; tinc += tv; }
    }
    fa->colmask[lane] = cm;
    aux->offs[lane + 1] = inc;
    aux->prefix[lane + 1] = tinc;
    const uint32_t act = __ballot_sync(0xFFFFFFFFu, c > 0);
    const int n_sel = __shfl_sync(0xFFFFFFFFu, inc, 31), tiles_total = __shfl_sync(0xFFFFFFFFu, tinc, 31);
    const int pad = (n_sel + 15) & ~15;
    const int s1 = choose_split_warp(tiles_total * kMT1, kMaxSplit1, a.ctas, pad, a.slab_rows, lane, kKB1,
                                     kDecodeKps);
    const int s2 = choose_split_warp(tiles_total * kMT2, kMaxSplit2, a.ctas, pad, a.slab_rows, lane, kKB2,
                                     kDecodeKps);
    if (lane == 0) {
      aux->offs[0] = 0;
      aux->prefix[0] = 0;
      fa->items = tiles_total * kMT1 * s1;
      fa->split = s1;
      fa->n_sel_pad = pad;
      fa->n_sel = n_sel;
      fa->items2 = tiles_total * kMT2 * s2;
      fa->split2 = s2;
    }
    if (blockIdx.x == 0) {
      sched->counts[lane] = c;
      sched->offs[lane + 1] = inc;
      sched->tile_prefix[lane + 1] = tinc;
      sched->tile_prefix2[lane + 1] = tinc;
      if (lane == 0) {
        sched->offs[0] = 0;
        sched->tile_prefix[0] = 0;
        sched->tile_prefix2[0] = 0;
        sched->n_tile2 = kFusedMaxTokens;
        sched->status = 0;
        sched->n_sel = n_sel;
        sched->n_sel_pad = pad;
        sched->n_active = __popc(act);
        sched->n_tile = kFusedMaxTokens;
        sched->tiles_total = tiles_total;
        sched->split1 = s1;
        sched->split2 = s2;
        sched->items1 = tiles_total * kMT1 * s1;
        sched->items2 = tiles_total * kMT2 * s2;
      }
    }
  }
  if (threadIdx.x == 0) MOE_ROUTE_TRACE(2);
  __syncthreads();
  if (blockIdx.x == 0 && warp == kFirstEpiWarp && lane < a.T) {   // lane = token: selection, permutation, row lists
    const int t = lane;
    const uint32_t m = fa->mask[t];
    a.local_mask[t] = m;
#pragma unroll
    for (int k = 0; k < kTopK; ++k) {
      a.topk_idx[t * kTopK + k] = fa->tidx[t][k];
      a.topk_w[t * kTopK + k] = fa->tw[t][k];
    }
    int j = 0;
    for (uint32_t rest = m; rest; rest &= rest - 1, ++j) {
      const int le = __ffs(rest) - 1;
      const int row = aux->offs[le] + __popc(fa->colmask[le] & ((1u << t) - 1u));
      float w = 0.0f;
#pragma unroll
      for (int k = 0; k < kTopK; ++k)
        if (fa->tidx[t][k] - a.local_expert_offset == le) w = fa->tw[t][k];
      a.perm_token[row] = t;
      a.perm_weight[row] = w;
      a.tok_rows[t * kTopK + j] = row;
    }
  }
}

}  // namespace moe
