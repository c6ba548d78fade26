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
  float sval[kEGlobal];               // routing bias as fp32
  int tidx[kFusedMaxTokens][kTopK];   // selection of every token (global expert ids, descending score)
  float tw[kFusedMaxTokens][kTopK];   // and its combination weights
  uint32_t mask[kFusedMaxTokens];     // per token: selected local experts
  uint32_t colmask[kELocal];          // per local expert: tokens that selected it
  int rows[kFusedMaxTokens][kTopK];   // per token: its rows in ascending local expert order
  float permw[kFusedMaxTokens * kTopK];   // per row: combination weight
  int tiles, n_sel_pad, n_sel;        // active experts (one token tile each), slab stride, rows
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

// K-blocks per pipeline stage of the decode kernel.
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
  // Routing in two steps (same arithmetic and tie rules as route_token; the work is spread over all warps and
  // the instruction count per token is a third).  Step A, one warp per (token, routing group), lane = expert:
  // sigmoid + bias -> key (kept in shared memory with the unbiased score), two rounds of warp arg-max for the
  // group score.  Step B, one warp per token: the four best groups, then every lane holds its expert of each
  // kept group and eight rounds of arg-max over the 128 candidates give the selection in descending order.
  uint32_t* skey = reinterpret_cast<uint32_t*>(smem);             // [T][256] keys; the stage ring is still idle
  float* sval = reinterpret_cast<float*>(smem) + kFusedMaxTokens * kEGlobal;      // [T][256] unbiased scores
  float* gsc = reinterpret_cast<float*>(smem) + 2 * kFusedMaxTokens * kEGlobal;   // [T][8]   group scores
  float* bias_s = fa->sval;
  for (int i = threadIdx.x; i < kEGlobal; i += kGemmThreads)
    bias_s[i] = __uint_as_float(static_cast<uint32_t>(a.bias_bf16[i]) << 16);
  constexpr int kWarps = kGemmThreads / 32;
  constexpr int kMaxUnits = (kFusedMaxTokens * kNGroup + kWarps - 1) / kWarps;
  const int units = a.T * kNGroup;
  float x[kMaxUnits];
#pragma unroll
  for (int i = 0; i < kMaxUnits; ++i) {                            // all logits of this warp's units in flight
    const int u = warp + i * kWarps;
    x[i] = u < units ? a.logits[static_cast<size_t>(u) * 32 + lane] : 0.0f;      // [t][g][lane] = [u][lane]
  }
  __syncthreads();
  if (threadIdx.x == 0) MOE_ROUTE_TRACE(0);
#pragma unroll
  for (int i = 0; i < kMaxUnits; ++i) {
    const int u = warp + i * kWarps;
    if (u < units) {                                               // uniform over the warp
      const float s = 1.0f / (1.0f + expf(-x[i]));
      const uint32_t key = order_key(s + bias_s[(u & 7) * 32 + lane]);
      skey[u * 32 + lane] = key;
      sval[u * 32 + lane] = s;
      // group score = best + second best biased score (ties: any; undo the order-preserving map)
      const uint32_t k1 = __reduce_max_sync(0xFFFFFFFFu, key);
      const int first = __ffs(__ballot_sync(0xFFFFFFFFu, key == k1)) - 1;
      const uint32_t k2 = __reduce_max_sync(0xFFFFFFFFu, lane == first ? 0u : key);
      const uint32_t u1 = (k1 & 0x80000000u) ? (k1 & 0x7FFFFFFFu) : ~k1;
      const uint32_t u2 = (k2 & 0x80000000u) ? (k2 & 0x7FFFFFFFu) : ~k2;
      if (lane == 0) gsc[u] = __uint_as_float(u1) + __uint_as_float(u2);
    }
  }
  if (threadIdx.x == 0) MOE_ROUTE_TRACE(6);
  __syncthreads();
  if (threadIdx.x == 0) MOE_ROUTE_TRACE(7);
  // Step B for up to two tokens per warp (t and t + kWarps), interleaved: the rounds of a token are a
  // dependent chain of warp reductions, those of two tokens are independent.
  {
    constexpr int kTok = (kFusedMaxTokens + kWarps - 1) / kWarps;   // 2
    uint32_t kq[kTok][kTopKGroup];
    int gq[kTok][kTopKGroup];
#pragma unroll
    for (int b = 0; b < kTok; ++b) {
      const int t = warp + b * kWarps;
      if (t < a.T) {
        // the four best groups (ties: lower group first), ascending in gq
        const float gs = gsc[t * kNGroup + (lane & 7)];
        int grank = 0;
#pragma unroll
        for (int h = 0; h < kNGroup; ++h) {
          const float gh = __shfl_sync(0xFFFFFFFFu, gs, h);
          grank += (gh > gs) || (gh == gs && h < (lane & 7));
        }
        uint32_t keep = __ballot_sync(0xFFFFFFFFu, lane < kNGroup && grank < kTopKGroup);
#pragma unroll
        for (int q = 0; q < kTopKGroup; ++q) {
          gq[b][q] = __ffs(keep) - 1;
          keep &= keep - 1;
          kq[b][q] = skey[t * kEGlobal + gq[b][q] * 32 + lane];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kTopK; ++r) {
#pragma unroll
      for (int b = 0; b < kTok; ++b) {
        const int t = warp + b * kWarps;
        if (t < a.T) {
          // this lane's best candidate (ties: lower group), then the warp's (ties: lower expert index)
          uint32_t best = kq[b][0];
          int bq = 0;
#pragma unroll
          for (int q = 1; q < kTopKGroup; ++q)
            if (kq[b][q] > best) { best = kq[b][q]; bq = q; }
          const uint32_t m = __reduce_max_sync(0xFFFFFFFFu, best);
          const uint32_t who = __ballot_sync(0xFFFFFFFFu, best == m);
          int wl = __ffs(who) - 1;
          if (who & (who - 1)) {   // several lanes hold the maximum (rare): the lowest (group, lane) wins
            const uint32_t win = __reduce_min_sync(0xFFFFFFFFu, best == m ? static_cast<uint32_t>(bq * 32 + lane) : 0xFFFFFFFFu);
            wl = (win >> 5) == static_cast<uint32_t>(bq) && (win & 31) == static_cast<uint32_t>(lane) ? lane : -1;
            wl = __ffs(__ballot_sync(0xFFFFFFFFu, wl == lane)) - 1;
          }
          if (lane == wl) {       // the winner records itself; nobody else needs to know before the end
            int wg = gq[b][0];
#pragma unroll
            for (int q = 1; q < kTopKGroup; ++q) wg = (q == bq) ? gq[b][q] : wg;
            const int idx = wg * 32 + lane;
            fa->tidx[t][r] = idx;
            fa->tw[t][r] = sval[t * kEGlobal + idx];     // unbiased score for now, weight below
#pragma unroll
            for (int q = 0; q < kTopKGroup; ++q) kq[b][q] = (q == bq) ? 0u : kq[b][q];   // taken: below every real key
          }
        }
      }
    }
    __syncwarp();
#pragma unroll
    for (int b = 0; b < kTok; ++b) {
      const int t = warp + b * kWarps;
      if (t < a.T) {
        float total = 0.0f;                               // the normaliser is summed in selection order
#pragma unroll
        for (int k = 0; k < kTopK; ++k) total += fa->tw[t][k];
        total += 1e-20f;
        __syncwarp();
        uint32_t bit = 0;
        if (lane < kTopK) {
          fa->tw[t][lane] = (fa->tw[t][lane] / total) * a.routed_scaling_factor;
          const int le = fa->tidx[t][lane] - a.local_expert_offset;
          if (le >= 0 && le < kELocal) bit = 1u << le;
        }
        bit = __reduce_or_sync(0xFFFFFFFFu, bit);
        if (lane == 0) fa->mask[t] = bit;
      }
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
    if (lane == 0) {
      aux->offs[0] = 0;
      aux->prefix[0] = 0;
      fa->tiles = tiles_total;
      fa->n_sel_pad = pad;
      fa->n_sel = n_sel;
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
        sched->split1 = 0;
        sched->split2 = 0;
        sched->items1 = tiles_total * kMT1 * (kKB1 / kDecodeKps);
        sched->items2 = tiles_total * kMT2 * (kKB2 / kDecodeKps);
        sched->ctas = static_cast<int>(gridDim.x);
      }
    }
  }
  if (threadIdx.x == 0) MOE_ROUTE_TRACE(2);
  __syncthreads();
  if (warp == kFirstEpiWarp && lane < a.T) {   // lane = token: row lists and weights (CTA 0 also publishes them)
    const int t = lane;
    const uint32_t m = fa->mask[t];
    const bool pub = blockIdx.x == 0;
    if (pub) {
      a.local_mask[t] = m;
#pragma unroll
      for (int k = 0; k < kTopK; ++k) {
        a.topk_idx[t * kTopK + k] = fa->tidx[t][k];
        a.topk_w[t * kTopK + k] = fa->tw[t][k];
      }
    }
    int j = 0;
    for (uint32_t rest = m; rest; rest &= rest - 1, ++j) {
      const int le = __ffs(rest) - 1;
      const int row = aux->offs[le] + __popc(fa->colmask[le] & ((1u << t) - 1u));
      float w = 0.0f;
#pragma unroll
      for (int k = 0; k < kTopK; ++k)
        if (fa->tidx[t][k] - a.local_expert_offset == le) w = fa->tw[t][k];
      fa->rows[t][j] = row;
      fa->permw[row] = w;
      if (pub) {
        a.perm_token[row] = t;
        a.perm_weight[row] = w;
        a.tok_rows[t * kTopK + j] = row;
      }
    }
  }
}

}  // namespace moe
