// Single-launch decode path of the MoE shard (T <= 16 tokens): routing, GEMM1, SwiGLU, GEMM2 and the
// weighted combine in ONE persistent kernel, one CTA per SM.
//
// Replaces, for small batches, the whole launch sequence of the reference's run()
// (moe/solution/cuda/moe.cu:2650-2896: route, histogram, scan, scatter, gather, two grouped GEMMs,
// activation and combine kernels); arithmetic contract from full-agent-pipeline/references/moe.py:95-200.
//
// The operator is a stream of 44 MB of fp8 weights per active expert.  With a kernel per GEMM the
// stream stops at every kernel boundary: the second GEMM cannot request its weights before the first
// has drained, the grid has been torn down and set up again, and the schedule has been re-read.  Here
// the TMA producer of every CTA goes straight from its last GEMM1 load to the WEIGHT tiles of its GEMM2
// items (they do not depend on GEMM1), so the ring is full of GEMM2 weights while the grid barrier and
// the SwiGLU tail run; only the token operand of GEMM2 (three e4m3 planes written by the tail) waits for
// the second grid barrier.  A stage's "full" barrier expects the bytes of both boxes, so the UMMA issuer
// needs no knowledge of the split.
//
//   warp 0      TMA producer (one thread)          warps 4-11  promotion + epilogue + tails
//   warp 1      UMMA issuer  (one thread)          (same roles and ring protocol as grouped_gemm.cu)
//
// Work split ("stream-K"): a GEMM's work is the sequence of pipeline stages (2 K-blocks) of all its
// (expert, weight-row tile) pairs, tile-major; CTA c takes the stages [c*G/n, (c+1)*G/n), i.e. a contiguous
// run that may cover the end of one tile and the start of the next.  Every CTA streams the same number of
// bytes (+-1 stage) whatever the number of active experts.  The pieces of a tile go to separate fp32 slabs
// (slab = ordinal of the piece in its tile, computable from the tile index alone), which the next phase
// sums in order: deterministic.
//
// Phases of a CTA:  setup | routing + schedule (every CTA, identical result) | GEMM1 items -> fp32
// split-K slabs | grid barrier 1 | SwiGLU + 3-plane e4m3 split of this CTA's share of (row, K-block)
// units | grid barrier 2 | GEMM2 items -> fp32 slabs | grid barrier 3 | weighted combine -> bf16.
// The three barriers are successive targets (n, 2n, 3n arrivals) of one tagged word.  Every wait is
// bounded; a timeout raises the CTA's abort flag, all roles leave through the normal teardown, and an
// error bit is left in the schedule block.
#include "ptx.cuh"
#include "epilogue_device.cuh"
#include "gemm_common.cuh"

namespace moe {

namespace {

constexpr int kNT = kFusedMaxTokens;   // all tokens are one token tile
constexpr int kL2PrefetchStages = 12;  // GEMM2 weight stages (32 KB each) a CTA asks into L2 behind its ring: <= 57 MB per GPU

struct DC {
  static constexpr int KPS = kDecodeKps;                  // K-blocks per stage
  static constexpr int A_BYTES = 128 * 128;               // one K-block of a weight tile
  static constexpr int B1_BYTES = kNT * 128;              // one K-block of the token rows (GEMM1)
  static constexpr int B2_BYTES = kNTerms * B1_BYTES;     // ... of the three planes (GEMM2)
  static constexpr int B_OFF = KPS * A_BYTES;
  static constexpr int STAGE_BYTES = KPS * (A_BYTES + B2_BYTES);
  static constexpr int TX1 = KPS * (A_BYTES + B1_BYTES);  // bytes a GEMM1 stage receives
  static constexpr int TX2 = STAGE_BYTES;                 // bytes a GEMM2 stage receives
  static constexpr int STAGES = 4;
  static constexpr int COLS1 = kNT;                       // TMEM columns of one K-block partial
  static constexpr int COLS2 = kNTerms * kNT;
  static constexpr int BUF_COLS = KPS * COLS2;
  static constexpr int NBUF = 4;
  static constexpr int TMEM_COLS = 512;
  static constexpr int SC_FLOATS = kKB1 * kNT;            // one scale-product table
  static constexpr int SC_BYTES = 2 * SC_FLOATS * 4;
  static constexpr int AUX_BYTES = 1024 + 4096;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SC_BYTES + AUX_BYTES + 1024;
  static_assert(STAGE_BYTES % 1024 == 0 && B1_BYTES % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
  static_assert(NBUF <= STAGES && NBUF * BUF_COLS <= TMEM_COLS, "ring depths");
  static_assert(SMEM_BYTES <= 227 * 1024 && SMEM_BYTES > 116 * 1024, "one CTA per SM");
  static_assert(kKB1 % KPS == 0 && kKB2 % KPS == 0, "stages hold whole K-blocks");
};

struct DItem {
  int e, m, s, row0, valid, kb0, kb1;
};

// CTA that owns stage g of a sequence of G stages cut into n contiguous runs [c*G/n, (c+1)*G/n).
__device__ __forceinline__ int stage_owner(int g, int G, int n) { return ((g + 1) * n - 1) / G; }

// Number of pieces (= slabs) of tile `tau` whose stages are [tau*U, tau*U + U).
__device__ __forceinline__ int tile_pieces(int tau, int U, int G, int n) {
  return stage_owner(tau * U + U - 1, G, n) - stage_owner(tau * U, G, n) + 1;
}

// This CTA's share of one GEMM, delivered piece by piece.
template <int GEMM>
struct Part {
  static constexpr int MT = GEMM == 1 ? kMT1 : kMT2;
  static constexpr int U = (GEMM == 1 ? kKB1 : kKB2) / DC::KPS;   // stages per tile
  int g, g1, G, cta, n;
  __device__ __forceinline__ void init(int tiles, int cta_, int n_) {
    G = tiles * MT * U;
    cta = cta_;
    n = n_;
    g = cta * G / n;
    g1 = (cta + 1) * G / n;
  }
  __device__ __forceinline__ bool next(const Aux* aux, DItem& it) {
    if (g >= g1) return false;
    const int tau = g / U, u0 = g - tau * U;
    const int len = min(U - u0, g1 - g);
    const int ord = tau / MT;   // ordinal of the expert among the active ones
    int e = 0;                  // largest e with prefix[e] <= ord: the ord-th active expert
#pragma unroll 1
    for (int k = 16; k > 0; k >>= 1)
      if (e + k < kELocal && aux->prefix[e + k] <= ord) e += k;
    it.e = e;
    it.m = tau - ord * MT;
    it.s = cta - stage_owner(tau * U, G, n);
    it.row0 = aux->offs[e];
    it.valid = aux->offs[e + 1] - aux->offs[e];
    it.kb0 = u0 * DC::KPS;
    it.kb1 = (u0 + len) * DC::KPS;
    g += len;
    return true;
  }
};

__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// Ring positions shared (by value, advanced identically) by the issuer and the promotion warps.
struct Ring {
  uint32_t stage = 0, ph = 0, buf = 0, bph = 0;
  __device__ __forceinline__ void advance() {
    if (++stage == DC::STAGES) { stage = 0; ph ^= 1u; }
    if (++buf == DC::NBUF) { buf = 0; bph ^= 1u; }
  }
};

// UMMA issue of one GEMM's items (one thread).
template <int GEMM>
__device__ __forceinline__ bool issue_items(int tiles, const Aux* aux, uint32_t smem_base, uint32_t tmem_base, Ring& r,
                                            volatile int* abort_flag) {
  constexpr int BB = GEMM == 1 ? DC::B1_BYTES : DC::B2_BYTES;
  constexpr int COLS = GEMM == 1 ? DC::COLS1 : DC::COLS2;
  constexpr uint32_t idesc = umma_idesc_e4m3(128, COLS);
  const uint64_t desc_const = umma_desc_k_sw128(0);
  const uint32_t full_base = smem_u32(&aux->full[0]), done_base = smem_u32(&aux->done[0]);
  const uint32_t tempty_base = smem_u32(&aux->tempty[0]);
  Part<GEMM> part;
  part.init(tiles, blockIdx.x, gridDim.x);
  DItem w;
  bool first = true;
  for (; part.next(aux, w); first = false) {
    for (int kb = w.kb0; kb < w.kb1; kb += DC::KPS) {
      if (!mbar_wait(tempty_base + r.buf * 8, r.bph ^ 1u, abort_flag)) return false;
      if (!mbar_wait(full_base + r.stage * 8, r.ph, abort_flag)) return false;
      tc_fence_after_sync();
      const uint32_t sbase = smem_base + r.stage * DC::STAGE_BYTES;
#pragma unroll
      for (int u = 0; u < DC::KPS; ++u) {
        const uint64_t adesc = desc_const | ((sbase + u * DC::A_BYTES) >> 4);
        const uint64_t bdesc = desc_const | ((sbase + DC::B_OFF + u * BB) >> 4);
        const uint32_t d = tmem_base + r.buf * DC::BUF_COLS + u * COLS;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) umma_f8(d, adesc + 2 * k4, bdesc + 2 * k4, idesc, k4 != 0 ? 1u : 0u);
      }
      umma_commit(done_base + r.stage * 8);
      r.advance();
    }
  }
  return true;
}

struct EpiCtx {
  Aux* aux;
  FusedAux* fa;
  float* sc_base;
  uint32_t tmem_base;
  volatile int* abort_flag;
  Ring r;
  uint32_t eph = 0;
  bool ok = true;
  int q, h, lane, etid;
  __device__ __forceinline__ void sync() {   // all promotion threads meet; bounded
    mbar_arrive(smem_u32(&aux->esync));
    if (!mbar_wait(smem_u32(&aux->esync), eph, abort_flag)) ok = false;
    eph ^= 1u;
  }
};

struct DecodeArgs {
  GemmArgs g;              // GEMM1 view: w_scale = gemm1 scales, out = GEMM1 slabs, plus the routing fields
  const float* w2_scale;   // [32, 56, 16]
  float* o;                // GEMM2 slabs
};

// Scale product of table entry idx = kbl * 16 + column of item w (0 for unused columns).
template <int GEMM>
__device__ __forceinline__ float scale_product(const DecodeArgs& a, const FusedAux* fa, const DItem& w, int idx) {
  const int nkb = w.kb1 - w.kb0;
  if (idx >= nkb * kNT) return 0.0f;
  const int kbl = idx / kNT, j = idx % kNT, kb = w.kb0 + kbl;
  if constexpr (GEMM == 1) {   // column j is token j; the scale table is the definition's [56, T]
    if (!((fa->colmask[w.e] >> j) & 1u)) return 0.0f;
    return __ldg(a.g.w_scale + (static_cast<size_t>(w.e) * kMT1 + w.m) * kKB1 + kb) *
           __ldg(a.g.hidden_scale + static_cast<size_t>(kb) * a.g.T + j);
  } else {                     // column j is row row0 + j; its plane scales were written by this launch
    if (j >= w.valid) return 0.0f;
    return __ldg(a.w2_scale + (static_cast<size_t>(w.e) * kMT2 + w.m) * kKB2 + kb) *
           __ldcg(a.g.c_scale + static_cast<size_t>(w.row0 + j) * kKB2 + kb);
  }
}

// Promotion + store of this CTA's pieces of one GEMM by the eight promotion warps.
template <int GEMM>
__device__ __forceinline__ void promote_items(const DecodeArgs& a, EpiCtx& c, int tiles, int n_sel_pad, float ws2_first) {
  constexpr int KB = GEMM == 1 ? kKB1 : kKB2;
  constexpr int M_TOTAL = GEMM == 1 ? k2I : kH;
  constexpr int COLS = GEMM == 1 ? DC::COLS1 : DC::COLS2;
  constexpr int PLANES = GEMM == 1 ? 1 : kNTerms;
  constexpr int CPW = kNT / 2;                        // token columns per warp
  constexpr int kEpiThreads = kEpiWarps * 32;
  constexpr int kMaxE = (KB * kNT + kEpiThreads - 1) / kEpiThreads;
  static_assert(GEMM == 1 || kMaxE == 1, "the GEMM2 table has one entry per promotion thread");
  const uint32_t done_base = smem_u32(&c.aux->done[0]), tempty_base = smem_u32(&c.aux->tempty[0]);
  const uint32_t lane_addr = static_cast<uint32_t>(c.q * 32) << 16;
  float* out_base = GEMM == 1 ? a.g.out : a.o;
  float pre[kMaxE];
  uint32_t nitem = 0;
  Part<GEMM> part;
  part.init(tiles, blockIdx.x, gridDim.x);
  DItem w, wn;
  bool have = part.next(c.aux, w);
  if (have) {
    const DItem& w0 = w;
#pragma unroll
    for (int x = 0; x < kMaxE; ++x) {
      const int idx = c.etid + x * kEpiThreads;
      if (idx >= KB * kNT) continue;
      if constexpr (GEMM == 2) {   // one entry per thread; the weight-scale factor was fetched ahead
        const int j = idx % kNT;
        c.sc_base[idx] = (idx < (w0.kb1 - w0.kb0) * kNT && j < w0.valid)
                             ? ws2_first * __ldcg(a.g.c_scale + static_cast<size_t>(w0.row0 + j) * kKB2 + w0.kb0 + idx / kNT)
                             : 0.0f;
      } else {
        c.sc_base[idx] = scale_product<GEMM>(a, c.fa, w0, idx);
      }
    }
  }
  for (; c.ok && have; ++nitem) {
    const int nkb = w.kb1 - w.kb0;
    const float* sc = c.sc_base + (nitem & 1u) * DC::SC_FLOATS;
    const bool have_next = part.next(c.aux, wn);
    c.sync();   // this piece's table is complete and the other one is free
    if (!c.ok) break;
    if (have_next) {
#pragma unroll
      for (int x = 0; x < kMaxE; ++x) pre[x] = scale_product<GEMM>(a, c.fa, wn, c.etid + x * kEpiThreads);
    }
    float acc[CPW];
#pragma unroll
    for (int j = 0; j < CPW; ++j) acc[j] = 0.0f;
    for (int kbl = 0; kbl < nkb; kbl += DC::KPS) {
      if (!mbar_wait(done_base + c.r.stage * 8, c.r.ph, c.abort_flag)) { c.ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = c.tmem_base + lane_addr + c.r.buf * DC::BUF_COLS + c.h * CPW;
      float v[DC::KPS][PLANES][CPW];
#pragma unroll
      for (int g = 0; g < DC::KPS; ++g)
#pragma unroll
        for (int p = 0; p < PLANES; ++p) tmem_ld8(taddr + g * COLS + p * kNT, v[g][p]);
      tmem_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (c.lane == 0) mbar_arrive(tempty_base + c.r.buf * 8);
#pragma unroll
      for (int g = 0; g < DC::KPS; ++g) {
        const float4* scv = reinterpret_cast<const float4*>(sc + (kbl + g) * kNT + c.h * CPW);
#pragma unroll
        for (int u = 0; u < CPW / 4; ++u) {
          const float4 f = scv[u];
          float s4[4];
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            float sum = v[g][PLANES - 1][u * 4 + x];
#pragma unroll
            for (int p = PLANES - 2; p >= 0; --p) sum += v[g][p][u * 4 + x];   // smallest terms first
            s4[x] = sum;
          }
          acc[u * 4 + 0] = fmaf(s4[0], f.x, acc[u * 4 + 0]);
          acc[u * 4 + 1] = fmaf(s4[1], f.y, acc[u * 4 + 1]);
          acc[u * 4 + 2] = fmaf(s4[2], f.z, acc[u * 4 + 2]);
          acc[u * 4 + 3] = fmaf(s4[3], f.w, acc[u * 4 + 3]);
        }
      }
      c.r.advance();
    }
    if (!c.ok) break;
    if constexpr (GEMM == 1) {      // token columns -> the expert's rows (ascending token)
      const uint32_t cm = c.fa->colmask[w.e];
      float* out = out_base + (static_cast<size_t>(w.s) * n_sel_pad + w.row0) * M_TOTAL + w.m * 128 + c.q * 32 + c.lane;
#pragma unroll
      for (int j = 0; j < CPW; ++j) {
        const int col = c.h * CPW + j;
        if ((cm >> col) & 1u) out[static_cast<size_t>(__popc(cm & ((1u << col) - 1u))) * M_TOTAL] = acc[j];
      }
    } else {
      float* out = out_base + (static_cast<size_t>(w.s) * n_sel_pad + w.row0 + c.h * CPW) * M_TOTAL + w.m * 128 +
                   c.q * 32 + c.lane;
#pragma unroll
      for (int j = 0; j < CPW; ++j)
        if (c.h * CPW + j < w.valid) out[static_cast<size_t>(j) * M_TOTAL] = acc[j];
    }
    if (have_next) {
      float* scn = c.sc_base + ((nitem + 1) & 1u) * DC::SC_FLOATS;
#pragma unroll
      for (int x = 0; x < kMaxE; ++x) {
        const int idx = c.etid + x * kEpiThreads;
        if (idx < KB * kNT) scn[idx] = pre[x];
      }
    }
    w = wn;
    have = have_next;
  }
}

__global__ void __launch_bounds__(kGemmThreads, 1)
decode_kernel(const __grid_constant__ CUtensorMap tm_w1, const __grid_constant__ CUtensorMap tm_x,
              const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_c,
              const __grid_constant__ DecodeArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sc_base = reinterpret_cast<float*>(smem + DC::STAGES * DC::STAGE_BYTES);
  Aux* aux = reinterpret_cast<Aux*>(smem + DC::STAGES * DC::STAGE_BYTES + DC::SC_BYTES);
  FusedAux* fa = reinterpret_cast<FusedAux*>(reinterpret_cast<uint8_t*>(aux) + 1024);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  griddep_launch_dependents();
  MoeSched* sched = a.g.sched;
  // everything that does not depend on earlier work in the stream first: barriers, descriptors, TMEM
  if (threadIdx.x == 0) {
    aux->abort = 0;
    for (int s = 0; s < DC::STAGES; ++s) {
      mbar_init(smem_u32(&aux->full[s]), 1);
      mbar_init(smem_u32(&aux->done[s]), 1);
    }
    for (int b = 0; b < DC::NBUF; ++b) mbar_init(smem_u32(&aux->tempty[b]), kEpiWarps);
    mbar_init(smem_u32(&aux->esync), kEpiWarps * 32);
    fence_mbar_init();
    tma_prefetch_desc(&tm_w1);
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_w2);
    tma_prefetch_desc(&tm_c);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&aux->tmem_base), DC::TMEM_COLS);
    tmem_relinquish();
  }
  griddep_wait();   // the workspace and the output belong to earlier launches until here
  unsigned int* bar = sched->bar1;
  unsigned int* epoch = sched->bar2;
  // (the epoch is requested here and first used after the routing, so its latency is not waited for)
  unsigned int tag_reg = 0;
  if (threadIdx.x == 0) tag_reg = grid_barrier_next_tag(epoch);
  decode_route_schedule(a.g, smem, aux, fa, sched);
  if (threadIdx.x == 0) {
    aux->tag = tag_reg;
    if (blockIdx.x == 0) grid_barrier_init(bar, tag_reg);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const unsigned int call_tag = aux->tag;
  const int tiles = fa->tiles;
  const int n_sel_pad = fa->n_sel_pad;
  const uint32_t tmem_base = aux->tmem_base;
  volatile int* abort_flag = &aux->abort;
  const unsigned int n_ctas = gridDim.x;

  if (warp < kFirstEpiWarp) {
    setmaxnreg_dec<kRegsControl>();
    if (warp == 0) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0) {
        const uint32_t smem_base = smem_u32(smem);
        const uint32_t full_base = smem_u32(&aux->full[0]), done_base = smem_u32(&aux->done[0]);
        uint32_t stage = 0, ph = 0;
        bool ok = true;
        {
          Part<1> part;
          part.init(tiles, blockIdx.x, gridDim.x);
          DItem w;
          while (ok && part.next(aux, w)) {
            const int wy = w.e * k2I + w.m * 128;
            for (int kb = w.kb0; kb < w.kb1; kb += DC::KPS) {
              if (!mbar_wait(done_base + stage * 8, ph ^ 1u, abort_flag)) { ok = false; break; }
              const uint32_t fb = full_base + stage * 8;
              mbar_arrive_expect_tx(fb, DC::TX1);
              const uint32_t dst = smem_base + stage * DC::STAGE_BYTES;
              tma_load_3d(dst, &tm_w1, 0, wy, kb, fb);                 // [2 K-blocks][128 rows][128 B]
              tma_load_3d(dst + DC::B_OFF, &tm_x, 0, 0, kb, fb);       // [2 K-blocks][16 tokens][128 B]
              if (++stage == DC::STAGES) { stage = 0; ph ^= 1u; }
            }
          }
        }
        // GEMM2: the weight box of a stage is requested as soon as the stage is free, up to a full ring
        // ahead of the token-operand boxes, which wait for the planes (grid barrier 2).
        Part<2> wpart, bpart;
        wpart.init(tiles, blockIdx.x, gridDim.x);
        bpart = wpart;
        DItem ww{}, bw{};
        bool whave = wpart.next(aux, ww), bhave = bpart.next(aux, bw);
        int wkb = ww.kb0, bkb = bw.kb0, ahead = 0;
        uint32_t bstage = stage;
        bool ready = false;
        while (ok && bhave) {
          if (ready ? ahead > 0 : (ahead == DC::STAGES || !whave)) {
            if (!ready) {
              // The ring is full of GEMM2 weights and HBM would now idle until the planes exist (two grid
              // barriers and the SwiGLU phase away): ask for the weight boxes behind the ring into L2, so that
              // after the barrier they arrive at L2 latency.  Bounded so that the slabs and planes stay in L2 too.
              {
                Part<2> ppart = wpart;
                DItem pw = ww;
                bool phave = whave;
                int pkb = wkb;
                for (int n = 0; phave && n < kL2PrefetchStages; ++n) {
                  tma_prefetch_l2_3d(&tm_w2, 0, pw.e * kH + pw.m * 128, pkb);
                  pkb += DC::KPS;
                  if (pkb >= pw.kb1) {
                    phave = ppart.next(aux, pw);
                    pkb = pw.kb0;
                  }
                }
              }
              if (!grid_barrier_wait(bar, call_tag, 2 * n_ctas)) { *abort_flag = 1; ok = false; break; }
              fence_proxy_async_global();   // the planes were written with ordinary stores by other SMs
              ready = true;
            }
            tma_load_4d(smem_base + bstage * DC::STAGE_BYTES + DC::B_OFF, &tm_c, 0, bw.row0, 0, bkb,
                        full_base + bstage * 8);                     // [2 K-blocks][3 planes][16 rows][128 B]
            if (++bstage == DC::STAGES) bstage = 0;
            --ahead;
            bkb += DC::KPS;
            if (bkb >= bw.kb1) {
              bhave = bpart.next(aux, bw);
              bkb = bw.kb0;
            }
          } else {
            if (!mbar_wait(done_base + stage * 8, ph ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t fb = full_base + stage * 8;
            mbar_arrive_expect_tx(fb, DC::TX2);
            tma_load_3d(smem_base + stage * DC::STAGE_BYTES, &tm_w2, 0, ww.e * kH + ww.m * 128, wkb, fb);
            if (++stage == DC::STAGES) { stage = 0; ph ^= 1u; }
            ++ahead;
            wkb += DC::KPS;
            if (wkb >= ww.kb1) {
              whave = wpart.next(aux, ww);
              wkb = ww.kb0;
            }
          }
        }
      }
      __syncwarp();   // block-wide barriers below need whole warps
    } else if (warp == 1) {
      // ---------------------------------------------------------------- UMMA issuer
      if (lane == 0) {
        Ring r;
        const uint32_t smem_base = smem_u32(smem);
        if (issue_items<1>(tiles, aux, smem_base, tmem_base, r, abort_flag))
          issue_items<2>(tiles, aux, smem_base, tmem_base, r, abort_flag);
      }
      __syncwarp();
    }
  } else {
    setmaxnreg_inc<kRegsEpilogue>();
    // ------------------------------------------------------------------ promotion, epilogue and tails
    EpiCtx c;
    c.aux = aux;
    c.fa = fa;
    c.sc_base = sc_base;
    c.tmem_base = tmem_base;
    c.abort_flag = abort_flag;
    c.q = warp & 3;                        // TMEM lane quarter this warp may access
    c.h = (warp - kFirstEpiWarp) >> 2;     // which half of the token columns
    c.lane = lane;
    c.etid = threadIdx.x - kFirstEpiWarp * 32;
    constexpr int kEpiThreads = kEpiWarps * 32;
    // arrivals are only valid once CTA 0 has installed this launch's tag; checked here, long before the first one
    if (c.etid == 0 && !grid_barrier_tag_wait(bar, call_tag)) *abort_flag = 1;

    promote_items<1>(a, c, tiles, n_sel_pad, 0.0f);

    // first GEMM2 item: the weight-scale factor of this thread's table entry does not depend on GEMM1;
    // fetching it here takes its DRAM latency off the path between grid barrier 2 and the first promotion
    float ws2_first = 0.0f;
    Part<2> first2;
    first2.init(tiles, blockIdx.x, gridDim.x);
    DItem w0;
    if (first2.next(aux, w0)) {
      const int kbl = c.etid / kNT;
      if (kbl < w0.kb1 - w0.kb0)
        // (volatile: the compiler would otherwise sink the load to its use, after both barriers)
        asm volatile("ld.global.nc.f32 %0, [%1];"
                     : "=f"(ws2_first)
                     : "l"(a.w2_scale + (static_cast<size_t>(w0.e) * kMT2 + w0.m) * kKB2 + w0.kb0 + kbl));
    }

    // grid barrier 1: every GEMM1 slab is complete
    c.sync();
    if (c.ok && c.etid == 0) {
      grid_barrier_arrive(bar);
      if (!grid_barrier_wait(bar, call_tag, n_ctas)) *abort_flag = 1;
    }
    c.sync();
    if (c.ok && !*abort_flag) {
      // SwiGLU + split of this CTA's share of the (row, K-block) units.  Up to 15 rows after the last one
      // are zero-filled: the 16-row token boxes of GEMM2 read them, and rows nobody has written would come
      // from DRAM instead of L2.
      const int n_sel = fa->n_sel;
      const int fill_rows = min(n_sel + kNT - 1, a.g.rows_cap);
      const int units = fill_rows * kKB2;
      const size_t slab = static_cast<size_t>(n_sel_pad) * k2I;
      constexpr int U1 = Part<1>::U;
      const int G1 = tiles * kMT1 * U1;
      for (int u = blockIdx.x * kEpiWarps + (warp - kFirstEpiWarp); u < units; u += gridDim.x * kEpiWarps) {
        const int row = u / kKB2, kb = u % kKB2;
        if (row < n_sel) {
          int e = 0;   // the row's expert: largest e with offs[e] <= row
#pragma unroll 1
          for (int k = 16; k > 0; k >>= 1)
            if (e + k < kELocal && aux->offs[e + k] <= row) e += k;
          const int tau = aux->prefix[e] * kMT1 + kb;   // weight tile of x1; x2's is 16 tiles further
          swiglu_split_unit2(a.g.out, slab, tile_pieces(tau, U1, G1, n_ctas), tile_pieces(tau + kKB2, U1, G1, n_ctas), row,
                             kb, lane, a.g.cq, a.g.c_scale, a.g.rows_cap);
        } else {
#pragma unroll
          for (int t = 0; t < kNTerms; ++t)
            *reinterpret_cast<uint32_t*>(a.g.cq + (static_cast<size_t>(t) * a.g.rows_cap + row) * kI + kb * kBlock +
                                         lane * 4) = 0u;
        }
      }
    }
    // grid barrier 2: the planes and their scales are complete (the producers' TMA loads read them)
    fence_proxy_async_global();
    c.sync();
    if (c.ok && c.etid == 0) {
      grid_barrier_arrive(bar);
      if (!grid_barrier_wait(bar, call_tag, 2 * n_ctas)) *abort_flag = 1;
    }
    c.sync();

    if (c.ok && !*abort_flag) promote_items<2>(a, c, tiles, n_sel_pad, ws2_first);

    // grid barrier 3: every GEMM2 slab is complete
    c.sync();
    if (c.ok && c.etid == 0) {
      grid_barrier_arrive(bar);
      if (!grid_barrier_wait(bar, call_tag, 3 * n_ctas)) *abort_flag = 1;
    }
    c.sync();
    if (c.ok && !*abort_flag) {
      constexpr int kVec = kH / 4;
      constexpr int U2 = Part<2>::U;
      const int G2 = tiles * kMT2 * U2;
      const size_t slab = static_cast<size_t>(n_sel_pad) * kH;
      const int total = a.g.T * kVec;
      for (int i = blockIdx.x * kEpiThreads + c.etid; i < total; i += gridDim.x * kEpiThreads) {
        const int t = i / kVec, col = i % kVec;
        const uint32_t mask = fa->mask[t];
        const int m = col / 32;   // weight-row tile of these four output columns
        auto slabs = [&](int j) {   // the token's j-th row belongs to its j-th local expert (ascending)
          uint32_t rest = mask;
          for (int x = 0; x < j; ++x) rest &= rest - 1;
          const int le = __ffs(rest) - 1;
          return tile_pieces(aux->prefix[le] * kMT2 + m, U2, G2, n_ctas);
        };
        combine_unit<6>(a.o, slab, slabs, __popc(mask), fa->rows[t], fa->permw, col,
                     a.g.out_rows ? a.g.out_rows[t] : a.g.out_bf16 + static_cast<size_t>(t) * kH);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && aux->abort) atomicOr(&sched->status, kErrGemm1Timeout | kErrGemm2Timeout);
  if (blockIdx.x == 0 && threadIdx.x == 0) *reinterpret_cast<volatile unsigned int*>(epoch) = call_tag;   // the next launch's tag differs
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, DC::TMEM_COLS);
  }
}

}  // namespace


int decode_kernel_init() {
  return static_cast<int>(cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DC::SMEM_BYTES));
}

int launch_decode(const CUtensorMap& tm_w1, const CUtensorMap& tm_x, const CUtensorMap& tm_w2, const CUtensorMap& tm_c,
                  const GemmArgs& g, const float* w2_scale, float* o, int ctas, cudaStream_t stream) {
  // A weight-row tile is cut into at most ctas / (tiles of its GEMM) + 2 pieces, and there is at least one
  // token tile; the SwiGLU phase sums up to 8 slabs (32 tiles per expert) and the combine up to 6 (56 tiles).
  if (ctas < 1 || ctas / kMT1 + 2 > 8 || ctas / kMT2 + 2 > 6) return static_cast<int>(cudaErrorInvalidConfiguration);
  DecodeArgs a{g, w2_scale, o};
  return static_cast<int>(launch_pdl(decode_kernel, dim3(ctas), dim3(kGemmThreads), DC::SMEM_BYTES, stream, tm_w1, tm_x,
                                     tm_w2, tm_c, a));
}

}  // namespace moe
