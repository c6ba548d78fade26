// Pieces shared by the grouped GEMM kernel and the single-launch decode kernel: the thread layout,
// the per-CTA barrier block, the grid barrier, and the in-kernel routing + schedule of the decode path.
#pragma once
#include "kernels.h"
#include "ptx.cuh"
#include "route_device.cuh"

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
  unsigned int tag;        // decode kernel: this launch's grid-barrier tag
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
//
// The tag comes from the device, not from the host: an epoch word next to the barrier word.  Every CTA
// reads it when the kernel starts (tag = epoch + 1) and CTA 0 stores the tag back as the new epoch when
// it leaves, which it can only do after every CTA has read the old one (the last barrier needs all
// arrivals) or after a timeout (the launch has failed by then).  A launch recorded in a CUDA graph and
// replayed therefore tags every replay differently; a tag passed as a kernel argument would repeat.
__device__ __forceinline__ unsigned int grid_barrier_next_tag(const unsigned int* epoch) {
  unsigned int e;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(e) : "l"(epoch) : "memory");
  return e + 1u;
}

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

// Up to this many tokens the decode kernel routes with one thread per expert (see decode_route_schedule).
constexpr int kBlockRouteMaxTokens = 4;

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
  // Routing, one warp per token (same arithmetic and tie rules as route_token), organised around what is cheap
  // on this machine: shuffles and plain comparisons are, reduce / vote chains are not (a round of warp arg-max
  // costs ~300 cycles of latency).  Measured: ~2.5 us for one token, ~5.5 us for sixteen (two per warp).
  // Lane l holds the 8 consecutive experts 8l .. 8l+7, so a routing group is 4 adjacent lanes:
  //   * sigmoid + bias -> order-preserving keys; the lane's two best by plain comparisons; two xor-shuffle
  //     steps merge them over the group's 4 lanes -> group score (sum of its two best biased scores);
  //   * the four best groups by comparing against the 8 scores (8 shuffles);
  //   * candidates are 64-bit words {key, 255 - expert}: a larger word is a better candidate, ties on the key
  //     go to the lower expert; lanes of dropped groups hold zeros.  Every lane sorts its 8 words (19-exchange
  //     network), then five butterfly steps merge the lists: with the partner's list reversed, the element-wise
  //     maximum is the top 8 of both lists as a bitonic sequence, which a 3-stage merge network sorts.  After
  //     the last step every lane holds the selection in descending order.
  if (a.T <= kBlockRouteMaxTokens) {
    // A few tokens: thread = expert (warps 0..7, warp = routing group), one token after the other.  The sort
    // networks below take ~2500 cycles whatever the batch; counting, for every kept expert, the kept experts
    // that beat it takes a few hundred per token.  Same arithmetic and tie rules (route_block_kernel).
    uint32_t* keys = reinterpret_cast<uint32_t*>(smem);             // the stage ring is still idle
    float* gscore = reinterpret_cast<float*>(smem + 1024);
    int* selidx = reinterpret_cast<int*>(smem + 1024 + 64);
    float* sels = reinterpret_cast<float*>(smem + 1024 + 128);
    if (warp < kNGroup) {
      const int e = threadIdx.x;
      float x[kBlockRouteMaxTokens];
#pragma unroll
      for (int t = 0; t < kBlockRouteMaxTokens; ++t)                 // all tokens' logits in flight
        x[t] = t < a.T ? a.logits[static_cast<size_t>(t) * kEGlobal + e] : 0.0f;
      const float bias_e = __uint_as_float(static_cast<uint32_t>(a.bias_bf16[e]) << 16);
#pragma unroll 1
      for (int t = 0; t < a.T; ++t) {
        float xt = x[0];
#pragma unroll
        for (int u = 1; u < kBlockRouteMaxTokens; ++u) xt = u == t ? x[u] : xt;
        const float s_e = 1.0f / (1.0f + expf(-xt));
        const uint32_t key_e = order_key(s_e + bias_e);
        keys[e] = key_e;
        const uint32_t k1 = __reduce_max_sync(0xFFFFFFFFu, key_e);
        const int first = __ffs(__ballot_sync(0xFFFFFFFFu, key_e == k1)) - 1;
        const uint32_t k2 = __reduce_max_sync(0xFFFFFFFFu, lane == first ? 0u : key_e);
        const uint32_t u1 = (k1 & 0x80000000u) ? (k1 & 0x7FFFFFFFu) : ~k1;
        const uint32_t u2 = (k2 & 0x80000000u) ? (k2 & 0x7FFFFFFFu) : ~k2;
        if (lane == 0) gscore[warp] = __uint_as_float(u1) + __uint_as_float(u2);
        named_bar_sync(1, kNGroup * 32);
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
        named_bar_sync(1, kNGroup * 32);
        if (warp == 0) {
          const float sv = lane < kTopK ? sels[lane] : 0.0f;
          float sum = 0.0f;
#pragma unroll
          for (int k = 0; k < kTopK; ++k) sum += __shfl_sync(0xFFFFFFFFu, sv, k);   // selection order, like every other path
          sum += 1e-20f;
          uint32_t bit = 0;
          if (lane < kTopK) {
            const int idx = selidx[lane];
            fa->tidx[t][lane] = idx;
            fa->tw[t][lane] = (sv / sum) * a.routed_scaling_factor;
            const int le = idx - a.local_expert_offset;
            if (le >= 0 && le < kELocal) bit = 1u << le;
          }
          bit = __reduce_or_sync(0xFFFFFFFFu, bit);
          if (lane == 0) fa->mask[t] = bit;
        }
        // the next token's keys / gscore are written before, selidx / sels after the next first barrier;
        // warp 0 has read selidx / sels before it reaches that barrier
      }
    }
  } else {
  float* bias_s = fa->sval;
  for (int i = threadIdx.x; i < kEGlobal; i += kGemmThreads)
    bias_s[i] = __uint_as_float(static_cast<uint32_t>(a.bias_bf16[i]) << 16);
  float* sval = reinterpret_cast<float*>(smem);                   // [T][256] unbiased scores; the stage ring is still idle
  constexpr int kWarps = kGemmThreads / 32;
  constexpr int kTok = (kFusedMaxTokens + kWarps - 1) / kWarps;   // tokens per warp: t = warp, warp + kWarps
  static_assert(kTok == 2, "two tokens per warp at most");
  float4 xa[kTok], xb[kTok];
#pragma unroll
  for (int b = 0; b < kTok; ++b) {                                 // both tokens' logits in flight
    const int t = warp + b * kWarps;
    xa[b] = xb[b] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (t < a.T) {
      const float4* row = reinterpret_cast<const float4*>(a.logits + static_cast<size_t>(t) * kEGlobal + lane * 8);
      xa[b] = row[0];
      xb[b] = row[1];
    }
  }
  __syncthreads();
  // Both tokens of a warp go through every step together (b = 0, 1): the steps of one token are a chain of
  // dependent operations, those of two tokens are independent and overlap.  `on[b]` is uniform over the warp.
  if (warp < a.T) {
    const bool on[kTok] = {true, warp + kWarps < a.T};
    unsigned long long c[kTok][8];
#pragma unroll
    for (int b = 0; b < kTok; ++b) {
      if (!on[b]) continue;
      const int t = warp + b * kWarps;
      const float4 va = xa[b], vb = xb[b];
      const float x[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
      float s[8];
      uint32_t k[8];
      uint32_t m1 = 0u, m2 = 0u;                                   // the lane's two best keys (m1 >= m2)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        s[i] = 1.0f / (1.0f + expf(-x[i]));
        k[i] = order_key(s[i] + bias_s[lane * 8 + i]);
        if (k[i] > m1) { m2 = m1; m1 = k[i]; }
        else if (k[i] > m2) m2 = k[i];
      }
      float4* sv = reinterpret_cast<float4*>(sval + t * kEGlobal + lane * 8);
      sv[0] = make_float4(s[0], s[1], s[2], s[3]);
      sv[1] = make_float4(s[4], s[5], s[6], s[7]);
#pragma unroll
      for (int d = 1; d <= 2; d <<= 1) {                           // merge over the group's 4 lanes
        const uint32_t o1 = __shfl_xor_sync(0xFFFFFFFFu, m1, d), o2 = __shfl_xor_sync(0xFFFFFFFFu, m2, d);
        const uint32_t n2 = m1 >= o1 ? max(m2, o1) : max(o2, m1);
        m1 = max(m1, o1);
        m2 = n2;
      }
      const float gs = __uint_as_float((m1 & 0x80000000u) ? (m1 & 0x7FFFFFFFu) : ~m1) +
                       __uint_as_float((m2 & 0x80000000u) ? (m2 & 0x7FFFFFFFu) : ~m2);
      const int g = lane >> 2;
      int grank = 0;                                               // ties: lower group first
#pragma unroll
      for (int h = 0; h < kNGroup; ++h) {
        const float gh = __shfl_sync(0xFFFFFFFFu, gs, h * 4);
        grank += (gh > gs) || (gh == gs && h < g);
      }
      const bool kept = grank < kTopKGroup;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        c[b][i] = kept ? (static_cast<unsigned long long>(k[i]) << 32) | static_cast<unsigned int>(255 - (lane * 8 + i)) : 0ull;
    }
#define MOE_CX(p, q)                                               \
    {                                                              \
      const unsigned long long hi = max(c[b][p], c[b][q]);         \
      c[b][q] = min(c[b][p], c[b][q]);                             \
      c[b][p] = hi;                                                \
    }
#pragma unroll
    for (int b = 0; b < kTok; ++b) {                               // the lane's own list, descending
      if (!on[b]) continue;
      MOE_CX(0, 1) MOE_CX(2, 3) MOE_CX(4, 5) MOE_CX(6, 7)
      MOE_CX(0, 2) MOE_CX(1, 3) MOE_CX(4, 6) MOE_CX(5, 7)
      MOE_CX(1, 2) MOE_CX(5, 6) MOE_CX(0, 4) MOE_CX(3, 7)
      MOE_CX(1, 5) MOE_CX(2, 6)
      MOE_CX(1, 4) MOE_CX(3, 6)
      MOE_CX(2, 4) MOE_CX(3, 5)
      MOE_CX(3, 4)
    }
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {                             // butterfly merge over the warp
#pragma unroll
      for (int b = 0; b < kTok; ++b) {
        if (!on[b]) continue;
        unsigned long long o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __shfl_xor_sync(0xFFFFFFFFu, c[b][7 - i], d);
#pragma unroll
        for (int i = 0; i < 8; ++i) c[b][i] = max(c[b][i], o[i]);
        MOE_CX(0, 4) MOE_CX(1, 5) MOE_CX(2, 6) MOE_CX(3, 7)
        MOE_CX(0, 2) MOE_CX(1, 3) MOE_CX(4, 6) MOE_CX(5, 7)
        MOE_CX(0, 1) MOE_CX(2, 3) MOE_CX(4, 5) MOE_CX(6, 7)
      }
    }
#undef MOE_CX
    __syncwarp();                                                  // the warp's unbiased scores are in shared memory
#pragma unroll
    for (int b = 0; b < kTok; ++b) {
      if (!on[b]) continue;
      const int t = warp + b * kWarps;
      float total = 0.0f, mine = 0.0f;                             // the normaliser is summed in selection order
      int my_idx = 0;
#pragma unroll
      for (int q = 0; q < kTopK; ++q) {
        const int idx = 255 - static_cast<int>(static_cast<unsigned int>(c[b][q]) & 0xFFu);
        const float sq = sval[t * kEGlobal + idx];
        total += sq;
        if (lane == q) { mine = sq; my_idx = idx; }
      }
      total += 1e-20f;
      uint32_t bit = 0;
      if (lane < kTopK) {
        fa->tidx[t][lane] = my_idx;
        fa->tw[t][lane] = (mine / total) * a.routed_scaling_factor;
        const int le = my_idx - a.local_expert_offset;
        if (le >= 0 && le < kELocal) bit = 1u << le;
      }
      bit = __reduce_or_sync(0xFFFFFFFFu, bit);
      if (lane == 0) fa->mask[t] = bit;
    }
  }
  }   // T > kBlockRouteMaxTokens
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
