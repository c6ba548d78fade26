// Grouped FP8 GEMM on tcgen05 for both expert GEMMs of the MoE shard.
//
// Replaces gemm_fp8_fp8_grouped_kernel / gemm_fp8_fp8_native_grouped_kernel
// (moe/solution/cuda/moe.cu:1373-1785, GEMM1) and gemm_fp32_fp8w_fused_acc_grouped_kernel
// (moe.cu:2186-2431, GEMM2); arithmetic contract from
// full-agent-pipeline/references/moe.py:95-118 (block scales) and :183-196 (the two matmuls).
//
// Orientation ("swap-AB"): the expert's weight rows are the 128-row M operand of
// the UMMA and the tokens are the N operand, so a batch of 1..128 tokens per
// expert streams every weight byte through shared memory exactly once per token
// tile and the tensor core does all fp8 decoding.  The operator is HBM-bound on
// the weight stream in every single-GPU regime, so the kernel is organised around
// keeping TMA loads of 16 KB weight tiles in flight:
//
//   warp 0  producer: TMA (SWIZZLE_128B, no multicast) of one weight tile
//           [128 rows x 128 K-bytes] and the token tile(s) [N_TILE x 128] per K-block
//           into a ring of STAGES shared-memory stages.
//   warp 1 (and warp 2 from 32-token tiles up, alternate stages)  issuer: one thread issues the tcgen05.mma kind::f8f6f4 (M128, K32) of a
//           K-block into its own TMEM columns.  For GEMM2 the kNTerms e4m3 planes of
//           the token operand sit back to back in shared memory and, while they fit
//           N <= 256, are consumed as ONE operand of N = kNTerms * N_TILE rows, so the
//           weight tile is read from shared memory once per K32 step, not once per term.
//           G consecutive K-blocks form a hand-off group with one "full" barrier;
//           NBUF groups rotate through TMEM so that the hand-off latency between the
//           tensor core and the promotion warps is hidden.
//   warps 4-11 promotion + epilogue (two warps per TMEM lane quarter, each owning half
//           of the token columns): tcgen05.ld the partials of a group, release the TMEM
//           buffer, multiply by w_scale[e, m, kb] * b_scale[row, kb] and accumulate in
//           registers (the scales are arbitrary fp32 per 128-block, so they cannot ride
//           on the hardware's power-of-two block scaling); after the last K-block store
//           the fp32 tile transposed, i.e. token-major [row, m].
//
// Work items (expert, weight-row tile, K-split, token tile) are decoded from the
// device-resident schedule; CTAs are persistent and take items round-robin.
// Every mbarrier wait is bounded (ptx.cuh); on a timeout the CTA records an error
// bit in the schedule block and leaves through the normal teardown.
#include "epilogue_device.cuh"
#include "gemm_common.cuh"

namespace moe {

namespace {

constexpr int kThreads = kGemmThreads;

template <int GEMM, int N_TILE>
struct Cfg {
  static constexpr int KB = GEMM == 1 ? kKB1 : kKB2;
  static constexpr int MT = GEMM == 1 ? kMT1 : kMT2;
  static constexpr int M_TOTAL = MT * 128;
  static constexpr int NTERMS = GEMM == 1 ? 1 : kNTerms;
  static constexpr bool STACK = NTERMS > 1 && NTERMS * N_TILE <= 256;   // planes consumed as one N operand
  static constexpr int N_MMA = STACK ? NTERMS * N_TILE : N_TILE;        // UMMA N
  static constexpr int MMA_PER_K4 = STACK ? 1 : NTERMS;
  static constexpr int PLANES = STACK ? NTERMS : 1;                     // column planes the epilogue sums
  static constexpr int KB_COLS = N_MMA;                                 // TMEM columns of one K-block partial
  // 128-token tiles run un-swapped: tokens are the UMMA M operand (TMEM lanes), weight rows the N operand
  // (TMEM columns).  A promotion thread then owns one token row, so the scale product of a K-block is ONE
  // value per thread instead of one per token column, and the result row is contiguous in memory.
  // UMMA issuer threads (warps 1 and 2 of the control warpgroup), taking alternate stages.  A stage's UMMAs only
  // touch that stage's shared memory and TMEM columns and each thread commits its own, so stages are independent;
  // with one thread the waits and loop overhead between two stages (~500 cycles) leave the tensor pipe idle,
  // because the instruction queue behind the issuing thread is only an instruction or two deep.
  static constexpr int ISSUERS = N_TILE >= 32 ? 2 : 1;
  static constexpr bool TOK_ON_M = N_TILE == 128 && GEMM == 1;   // (GEMM2 measures the same either way)
  // Ragged token tiles (swapped orientation only): an item brings and multiplies the rows it has, rounded up to
  // RSTEP.  An SM takes in about 45 bytes per clock from L2 and HBM delivers a 16 KB weight tile every ~700
  // clocks per SM, so a K-block may cost 31 KB of operands before the weight stream stalls; GEMM2's three
  // planes of a full 64-token tile alone are 24 KB.
  static constexpr int RSTEP = N_TILE >= 64 ? N_TILE / 4 : 16;
  static constexpr int RMAPS = N_TILE / RSTEP;
  static_assert(RMAPS >= 1 && RMAPS <= 4 && RSTEP % 16 == 0, "token maps per kernel / UMMA N granularity");
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = N_TILE * 128;
  static constexpr int KB_BYTES = A_BYTES + NTERMS * B_BYTES;           // operands of one K-block
  // K-blocks per pipeline stage.  A stage is also the TMEM hand-off unit: ONE tcgen05.commit per
  // stage tells the producer that the stage's shared memory is free and the promotion warps that
  // its partial sums are in TMEM.  (A commit costs the tensor pipe roughly 400 cycles, about as
  // much as six UMMAs of a 128-token tile, so two K-blocks share one wherever shared memory and
  // TMEM allow two stages of two.)
  static constexpr int KPS = (2 * KB_BYTES <= 64 * 1024 && 2 * KB_COLS <= 256) ? 2 : 1;
  static constexpr int G = KPS;
  static constexpr int CPW = N_TILE / 2;                                // token columns per epilogue warp
  static constexpr int CH = CPW > 64 ? 32 : CPW;                        // columns read back per tcgen05.ld batch
  static constexpr int STAGE_BYTES = KPS * KB_BYTES;
  // Scale-product tables.  With two, the next item's products are fetched during the current item's K loop;
  // GEMM2's short items (16 K-blocks) on wide tiles measured faster with one table filled between two barriers.
  static constexpr int SC_BUFS = (N_TILE <= 32 || (GEMM == 1 && !TOK_ON_M)) ? 2 : 1;
  static constexpr int SC_BYTES = SC_BUFS * KB * N_TILE * 4;
  static constexpr int AUX_BYTES = 1024;
  static constexpr int BUDGET = 227 * 1024 - 1024;   // 1 KB slack for the 1024-byte alignment of the ring
  static constexpr int STAGES_FIT = (BUDGET - SC_BYTES - AUX_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 10 ? 10 : STAGES_FIT;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SC_BYTES + AUX_BYTES + 1024;
  static constexpr int NBUF_FIT = 512 / (G * KB_COLS);
  // TMEM buffers (one stage of partials each).  Not more than shared-memory stages: the promotion warps
  // and the producer wait on the same per-stage barrier, and a stage must not complete a second phase
  // before the promotion warps have seen the first; the issuer is at most NBUF stages ahead of them.
  static constexpr int NBUF_CAP = NBUF_FIT > 4 ? 4 : NBUF_FIT;
  static constexpr int NBUF = NBUF_CAP > STAGES ? STAGES : NBUF_CAP;
  static constexpr int TMEM_USED = NBUF * G * KB_COLS;
  static constexpr int TMEM_COLS = TMEM_USED <= 32 ? 32 : TMEM_USED <= 64 ? 64 : TMEM_USED <= 128 ? 128
                                   : TMEM_USED <= 256 ? 256 : 512;
  static_assert(STAGES >= 2 && CH <= CPW, "ring too small / read-back chunks");
  static_assert(KB % KPS == 0 && (KPS & (KPS - 1)) == 0, "K-blocks per stage: a power of two dividing the K extent");
  static_assert(NBUF >= 2 && NBUF <= STAGES && TMEM_USED <= 512, "TMEM budget / ring depths");
  static_assert(N_MMA % 16 == 0 && N_MMA >= 16 && N_MMA <= 256, "invalid UMMA N for M = 128");
  static_assert(SMEM_BYTES > 116 * 1024, "one CTA per SM is assumed (TMEM is allocated without contention)");
};

struct Item {
  int e, m, s, row0, valid, kb0, kb1;
  int nv;      // token rows the item brings and multiplies: `valid` rounded up to the row step
};

template <int GEMM, int N_TILE>
__device__ __forceinline__ Item decode_item(int i, int split, const Aux* aux) {
  using C = Cfg<GEMM, N_TILE>;
  const int per = C::MT * split;
  // largest e with prefix[e] * per <= i (experts without tiles repeat the prefix value, so
  // the largest such e is the one that owns tile i)
  int e = 0;
#pragma unroll 1
  for (int k = 16; k > 0; k >>= 1)
    if (e + k < kELocal && aux->prefix[e + k] * per <= i) e += k;
  int r = i - aux->prefix[e] * per;
  const int tiles_e = aux->prefix[e + 1] - aux->prefix[e];
  const int n = r % tiles_e;
  r /= tiles_e;
  Item it;
  it.e = e;
  it.s = r % split;
  it.m = r / split;
  const int cnt = aux->offs[e + 1] - aux->offs[e];
  it.row0 = aux->offs[e] + n * N_TILE;
  it.valid = min(N_TILE, cnt - n * N_TILE);
  it.nv = C::TOK_ON_M ? N_TILE : min(N_TILE, (it.valid + C::RSTEP - 1) / C::RSTEP * C::RSTEP);
  // split boundaries in units of one pipeline stage, so that no stage straddles two items
  constexpr int kUnits = C::KB / C::KPS;
  it.kb0 = ((it.s * kUnits) / split) * C::KPS;
  it.kb1 = (((it.s + 1) * kUnits) / split) * C::KPS;
  return it;
}

template <int GEMM, int N_TILE>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ TokenMaps tm_b, GemmArgs a) {
  using C = Cfg<GEMM, N_TILE>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sc_base = reinterpret_cast<float*>(smem + C::STAGES * C::STAGE_BYTES);
  Aux* aux = reinterpret_cast<Aux*>(smem + C::STAGES * C::STAGE_BYTES + C::SC_BYTES);

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
    for (int b = 0; b < C::NBUF; ++b) mbar_init(smem_u32(&aux->tempty[b]), kEpiWarps);
    mbar_init(smem_u32(&aux->esync), kEpiWarps * 32);
    fence_mbar_init();
    tma_prefetch_desc(&tm_w);
    for (int i = 0; i < C::RMAPS; ++i) tma_prefetch_desc(&tm_b.m[i]);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&aux->tmem_base), C::TMEM_COLS);
    tmem_relinquish();
  }
  griddep_wait();   // the schedule, the operands and the output slabs belong to earlier kernels until here
  int items, split, n_sel_pad;
  items = GEMM == 1 ? sched->items1 : sched->items2;
  split = GEMM == 1 ? sched->split1 : sched->split2;
  n_sel_pad = sched->n_sel_pad;
  if (threadIdx.x <= kELocal) {
    aux->prefix[threadIdx.x] = GEMM == 1 ? sched->tile_prefix[threadIdx.x] : sched->tile_prefix2[threadIdx.x];
    aux->offs[threadIdx.x] = sched->offs[threadIdx.x];
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = aux->tmem_base;
  volatile int* abort_flag = &aux->abort;

  if (warp < kFirstEpiWarp) {
  setmaxnreg_dec<kRegsControl>();
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint32_t smem_base = smem_u32(smem);
      const uint32_t full_base = smem_u32(&aux->full[0]), done_base = smem_u32(&aux->done[0]);
      uint32_t stage = 0, ph = 0;
      bool ok = true;
      for (int i = blockIdx.x; ok && i < items; i += gridDim.x) {
        const Item w = decode_item<GEMM, N_TILE>(i, split, aux);
        const int wy = w.e * C::M_TOTAL + w.m * 128;
        const int by = w.row0;
        for (int kb = w.kb0; kb < w.kb1; kb += C::KPS) {
          if (!mbar_wait(done_base + stage * 8, ph ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t bar = full_base + stage * 8;
          mbar_arrive_expect_tx(bar, C::KPS * (C::A_BYTES + C::NTERMS * w.nv * 128));
          const uint32_t dst = smem_base + stage * C::STAGE_BYTES;
          // weights: [KPS][128 rows][128 B]; tokens: [KPS][NTERMS planes][nv rows][128 B]
          tma_load_3d(dst, &tm_w, 0, wy, kb, bar);
          const CUtensorMap* mb = &tm_b.m[w.nv / C::RSTEP - 1];
          if (GEMM == 1) tma_load_3d(dst + C::KPS * C::A_BYTES, mb, 0, by, kb, bar);
          else tma_load_4d(dst + C::KPS * C::A_BYTES, mb, 0, by, 0, kb, bar);
          if (++stage == C::STAGES) { stage = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();   // block-wide barriers below need whole warps
  } else if (warp == 1 || (C::ISSUERS == 2 && warp == 2)) {
    // ------------------------------------------------------------------ UMMA issuer(s)
    // One thread; its loop is the critical path of the large-tile regimes (every instruction is
    // dependent-issue latency), so ring positions are kept incrementally and the descriptors are
    // formed with one add from constants.
    if (lane == 0) {
      const uint64_t desc_const = umma_desc_k_sw128(0);          // everything but the start address
      const uint32_t smem_base = smem_u32(smem);
      const uint32_t full_base = smem_u32(&aux->full[0]), done_base = smem_u32(&aux->done[0]);
      const uint32_t tempty_base = smem_u32(&aux->tempty[0]);
      uint32_t stage = 0, ph = 0, buf = 0, bph = 0;
      bool ok = true;
      [[maybe_unused]] int nst = 0;
      for (int i = blockIdx.x; ok && i < items; i += gridDim.x) {
        const Item w = decode_item<GEMM, N_TILE>(i, split, aux);
        const uint32_t idesc = umma_idesc_e4m3(128, C::STACK ? C::NTERMS * w.nv : w.nv);
        const uint32_t plane_bytes = static_cast<uint32_t>(w.nv) * 128;
        for (int kb = w.kb0; kb < w.kb1; kb += C::KPS, ++nst) {        // items span whole stages
          if (C::ISSUERS == 2 && (nst & 1) != warp - 1) {               // the other issuer's stage
            if (++stage == C::STAGES) { stage = 0; ph ^= 1u; }
            if (++buf == C::NBUF) { buf = 0; bph ^= 1u; }
            continue;
          }
          if (!mbar_wait(tempty_base + buf * 8, bph ^ 1u, abort_flag)) { ok = false; break; }
          if (!mbar_wait(full_base + stage * 8, ph, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sbase = smem_base + stage * C::STAGE_BYTES;
#pragma unroll
          for (int u = 0; u < C::KPS; ++u) {
            const uint64_t adesc = desc_const | ((sbase + u * C::A_BYTES) >> 4);
            const uint32_t sb = sbase + C::KPS * C::A_BYTES + u * (C::NTERMS * plane_bytes);
            const uint32_t d = tmem_base + buf * (C::G * C::KB_COLS) + u * C::KB_COLS;
#pragma unroll
            for (int t = 0; t < C::MMA_PER_K4; ++t) {
              const uint64_t bdesc = desc_const | ((sb + t * plane_bytes) >> 4);
#pragma unroll
              for (int k4 = 0; k4 < 4; ++k4) {  // +32 bytes of K inside the 128-byte swizzle atom = +2 encoded units
                if constexpr (C::TOK_ON_M) umma_f8(d, bdesc + 2 * k4, adesc + 2 * k4, idesc, (t | k4) != 0 ? 1u : 0u);
                else umma_f8(d, adesc + 2 * k4, bdesc + 2 * k4, idesc, (t | k4) != 0 ? 1u : 0u);
              }
            }
          }
          umma_commit(done_base + stage * 8);
          if (++stage == C::STAGES) { stage = 0; ph ^= 1u; }
          if (++buf == C::NBUF) { buf = 0; bph ^= 1u; }
        }
      }
    }
    __syncwarp();
  }
  } else {
    setmaxnreg_inc<kRegsEpilogue>();
    // ------------------------------------------------------------------ promotion + epilogue (warps 4..11)
    const int q = warp & 3;                       // TMEM lane quarter this warp may access
    const int h = (warp - kFirstEpiWarp) >> 2;    // which half of the token columns
    const int etid = threadIdx.x - kFirstEpiWarp * 32;   // 0..255
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    uint32_t eph = 0, nitem = 0;
    [[maybe_unused]] int nst = 0;
    uint32_t stage = 0, ph = 0, buf = 0, bph = 0;      // same ring positions as the issuer
    const uint32_t done_base = smem_u32(&aux->done[0]), tempty_base = smem_u32(&aux->tempty[0]);
    bool ok = true;
    // all epilogue threads meet here; bounded like every other wait in this kernel
    auto epi_sync = [&]() {
      mbar_arrive(smem_u32(&aux->esync));
      if (!mbar_wait(smem_u32(&aux->esync), eph, abort_flag)) ok = false;
      eph ^= 1u;
    };
    // Scale products sc[kbl][j] = w_scale[e, m, kb] * b_scale[row0 + j, kb] of one item.  With two
    // tables (small token tiles, short items) the next item's values are fetched into registers
    // before the current item's K loop, so their global-memory latency is off the critical path.
    constexpr int kEpiThreads = kEpiWarps * 32;
    constexpr int kMaxE = (C::KB * N_TILE + kEpiThreads - 1) / kEpiThreads;
    auto load_scale = [&](const Item& w, int idx) -> float {
      // branch-free (clamped addresses, result selected afterwards) so that a thread's loads can all be in flight
      const int nkb = w.kb1 - w.kb0;
      const bool in = idx < nkb * N_TILE;
      const int kbl = in ? idx / N_TILE : 0, j = idx % N_TILE, kb = w.kb0 + kbl;
      const bool valid = in && j < w.valid;
      const float ws = __ldg(a.w_scale + (static_cast<size_t>(w.e) * C::MT + w.m) * C::KB + kb);
      const float bs = __ldg(a.b_scale + static_cast<size_t>(w.row0 + (valid ? j : 0)) * C::KB + kb);
      return valid ? ws * bs : 0.0f;
    };
    // One table, next item's values prefetched into registers (un-swapped path: its promotion keeps no
    // per-column scale temporaries, so there is room for them during the K loop)
    constexpr bool kPrefetch1 = C::SC_BUFS == 1 && C::TOK_ON_M;
    float pre[(C::SC_BUFS == 2 || kPrefetch1) ? kMaxE : 1];
    if (C::SC_BUFS == 2 && static_cast<int>(blockIdx.x) < items) {
      const Item w0 = decode_item<GEMM, N_TILE>(blockIdx.x, split, aux);
#pragma unroll
      for (int x = 0; x < kMaxE; ++x) {
        const int idx = etid + x * kEpiThreads;
        if (idx < C::KB * N_TILE) sc_base[idx] = load_scale(w0, idx);
      }
    }
    for (int i = blockIdx.x; ok && i < items; i += gridDim.x, ++nitem) {
      const Item w = decode_item<GEMM, N_TILE>(i, split, aux);
      const int nkb = w.kb1 - w.kb0;
      float* sc = sc_base + (C::SC_BUFS == 2 ? (nitem & 1u) * (C::KB * N_TILE) : 0);
      const int inext = i + gridDim.x;
      if (C::SC_BUFS == 1) {
        epi_sync();   // the previous item's scale products are no longer being read
        if (!ok) break;
        if (kPrefetch1 && nitem > 0) {
#pragma unroll
          for (int x = 0; x < kMaxE; ++x) {
            const int idx = etid + x * kEpiThreads;
            if (idx < nkb * N_TILE) sc[idx] = pre[x];
          }
        } else {
          for (int idx = etid; idx < nkb * N_TILE; idx += kEpiThreads) sc[idx] = load_scale(w, idx);
        }
      }
      epi_sync();     // this item's table is complete (and, with two tables, the other one is free)
      if (!ok) break;
      if ((C::SC_BUFS == 2 || kPrefetch1) && inext < items) {
        const Item wn = decode_item<GEMM, N_TILE>(inext, split, aux);
#pragma unroll
        for (int x = 0; x < kMaxE; ++x) pre[x] = load_scale(wn, etid + x * kEpiThreads);
      }

      float acc[C::CPW];
#pragma unroll
      for (int j = 0; j < C::CPW; ++j) acc[j] = 0.0f;

      if constexpr (C::TOK_ON_M) {
        static_assert(C::PLANES == 1 && C::CPW == 64 && C::KB_COLS == 128, "un-swapped path: one 128 x 128 partial per K-block");
        // lane = token row (row0 + 32 q + lane), columns = this warp's half of the 128 weight rows
        const int trow = q * 32 + lane;
        for (int kbl = 0; kbl < nkb; kbl += C::G, ++nst) {
          if (!mbar_wait(done_base + stage * 8, ph, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t taddr = tmem_base + lane_addr + buf * (C::G * C::KB_COLS) + h * C::CPW;
#pragma unroll
          for (int g = 0; g < C::G; ++g) {
            float v[C::CPW];
            tmem_ld32(taddr + g * C::KB_COLS, v);
            tmem_ld32(taddr + g * C::KB_COLS + 32, v + 32);
            const float f = sc[(kbl + g) * N_TILE + trow];      // w_scale * b_scale of this token row and K-block
            tmem_wait_ld();
            if (g == C::G - 1) {
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(tempty_base + buf * 8);
            }
#pragma unroll
            for (int j = 0; j < C::CPW; ++j) acc[j] = fmaf(v[j], f, acc[j]);
          }
          if (++stage == C::STAGES) { stage = 0; ph ^= 1u; }
          if (++buf == C::NBUF) { buf = 0; bph ^= 1u; }
        }
      } else
      for (int kbl = 0; kbl < nkb; kbl += C::G, ++nst) {
        if (!mbar_wait(done_base + stage * 8, ph, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + lane_addr + buf * (C::G * C::KB_COLS) + h * C::CPW;
#pragma unroll
        for (int g = 0; g < C::G; ++g) {
          // one K-block's partial at a time, in chunks of at most 64 columns (register budget);
          // the buffer is released after the last read.  The stacked planes are w.nv columns apart.  A chunk
          // that starts past the item's rows is not read (its columns are never stored; whole warps skip it).
#pragma unroll
          for (int c0 = 0; c0 < C::CPW; c0 += C::CH) {
            float v[C::PLANES][C::CH];
            const bool live = h * C::CPW + c0 < w.nv;
            if (live) {
#pragma unroll
              for (int p = 0; p < C::PLANES; ++p) tmem_ld_cols<C::CH>(taddr + g * C::KB_COLS + p * w.nv + c0, v[p]);
              tmem_wait_ld();
            }
            if (g == C::G - 1 && c0 + C::CH >= C::CPW) {
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(tempty_base + buf * 8);
            }
            if (!live) continue;
            const float4* scv = reinterpret_cast<const float4*>(sc + (kbl + g) * N_TILE + h * C::CPW + c0);
#pragma unroll
            for (int u = 0; u < C::CH / 4; ++u) {
              const float4 f = scv[u];
              float s4[4];
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                float sum = v[C::PLANES - 1][u * 4 + x];
#pragma unroll
                for (int p = C::PLANES - 2; p >= 0; --p) sum += v[p][u * 4 + x];   // smallest terms first
                s4[x] = sum;
              }
              acc[c0 + u * 4 + 0] = fmaf(s4[0], f.x, acc[c0 + u * 4 + 0]);
              acc[c0 + u * 4 + 1] = fmaf(s4[1], f.y, acc[c0 + u * 4 + 1]);
              acc[c0 + u * 4 + 2] = fmaf(s4[2], f.z, acc[c0 + u * 4 + 2]);
              acc[c0 + u * 4 + 3] = fmaf(s4[3], f.w, acc[c0 + u * 4 + 3]);
            }
          }
        }
        if (++stage == C::STAGES) { stage = 0; ph ^= 1u; }
        if (++buf == C::NBUF) { buf = 0; bph ^= 1u; }
      }
      if (!ok) break;
      if constexpr (C::TOK_ON_M) {
        if (q * 32 + lane < w.valid) {      // one token row, 64 consecutive outputs
          float* out = a.out + (static_cast<size_t>(w.s) * n_sel_pad + w.row0 + q * 32 + lane) * C::M_TOTAL + w.m * 128 + h * C::CPW;
#pragma unroll
          for (int j = 0; j < C::CPW / 8; ++j) st_global_v8(out + 8 * j, acc + 8 * j);   // whole 32-byte sectors
        }
      } else {
        float* out = a.out + (static_cast<size_t>(w.s) * n_sel_pad + w.row0 + h * C::CPW) * C::M_TOTAL + w.m * 128 +
                     q * 32 + lane;
#pragma unroll
        for (int j = 0; j < C::CPW; ++j)
          if (h * C::CPW + j < w.valid) out[static_cast<size_t>(j) * C::M_TOTAL] = acc[j];
      }
      if (C::SC_BUFS == 2 && inext < items) {
        float* scn = sc_base + ((nitem + 1) & 1u) * (C::KB * N_TILE);
#pragma unroll
        for (int x = 0; x < kMaxE; ++x) {
          const int idx = etid + x * kEpiThreads;
          if (idx < C::KB * N_TILE) scn[idx] = pre[x];
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

template <int GEMM, int N_TILE>
int launch_one(const CUtensorMap& tm_w, const TokenMaps& tm_b, const GemmArgs& a, int ctas, cudaStream_t stream) {
  using C = Cfg<GEMM, N_TILE>;
  return static_cast<int>(launch_pdl(grouped_gemm_kernel<GEMM, N_TILE>, dim3(ctas), dim3(kThreads), C::SMEM_BYTES,
                                     stream, tm_w, tm_b, a));
}

template <int GEMM, int N_TILE>
int init_one() {
  using C = Cfg<GEMM, N_TILE>;
  return static_cast<int>(cudaFuncSetAttribute(grouped_gemm_kernel<GEMM, N_TILE>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
}

}  // namespace


int grouped_gemm_kblocks_per_stage(int gemm_id, int n_tile) {
#define MOE_CASE(G, N) \
  if (gemm_id == G && n_tile == N) return Cfg<G, N>::KPS;
  MOE_CASE(1, 32) MOE_CASE(1, 64) MOE_CASE(1, 128)
  MOE_CASE(2, 32) MOE_CASE(2, 64) MOE_CASE(2, 128)
#undef MOE_CASE
  return 1;
}

int grouped_gemm_init() {
  int rc = 0;
  if ((rc = init_one<1, 32>())) return rc;
  if ((rc = init_one<1, 64>())) return rc;
  if ((rc = init_one<1, 128>())) return rc;
  if ((rc = init_one<2, 32>())) return rc;
  if ((rc = init_one<2, 64>())) return rc;
  if ((rc = init_one<2, 128>())) return rc;
  return 0;
}

int grouped_gemm_row_step(int n_tile) { return n_tile >= 64 ? n_tile / 4 : 16; }

int launch_grouped_gemm(int gemm_id, int n_tile, const CUtensorMap& tm_w, const TokenMaps& tm_b, const GemmArgs& a,
                        int ctas, cudaStream_t stream) {
#define MOE_CASE(G, N) \
  if (gemm_id == G && n_tile == N) return launch_one<G, N>(tm_w, tm_b, a, ctas, stream);
  MOE_CASE(1, 32) MOE_CASE(1, 64) MOE_CASE(1, 128)
  MOE_CASE(2, 32) MOE_CASE(2, 64) MOE_CASE(2, 128)
#undef MOE_CASE
  return static_cast<int>(cudaErrorInvalidValue);
}

}  // namespace moe
