// Shapes of the operator, the device-resident schedule block and the workspace
// layout shared by all kernels and the host launcher.
//
// Shapes follow the definition (full-agent-pipeline/references/moe.py:56-78):
// H = 7168, I = 2048, 32 local of 256 global experts, 128-element scale blocks,
// top-8 experts out of the top-4 of 8 groups.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace moe {

constexpr int kH = 7168;
constexpr int kI = 2048;
constexpr int k2I = 4096;
constexpr int kELocal = 32;
constexpr int kEGlobal = 256;
constexpr int kBlock = 128;
constexpr int kTopK = 8;
constexpr int kNGroup = 8;
constexpr int kTopKGroup = 4;
constexpr int kKB1 = kH / kBlock;        // 56 K-blocks in GEMM1
constexpr int kKB2 = kI / kBlock;        // 16 K-blocks in GEMM2
constexpr int kMT1 = k2I / kBlock;       // 32 weight-row tiles per expert in GEMM1
constexpr int kMT2 = kH / kBlock;        // 56 weight-row tiles per expert in GEMM2
constexpr int kNTerms = 3;               // e4m3 terms the SwiGLU output is split into for GEMM2
constexpr int kMaxSplit1 = 14;           // split-K limits (>= 4 K-blocks per split)
constexpr int kMaxSplit2 = 8;
constexpr int kMinSlabRows = 2048;       // slab capacity floor so that small batches can split K
constexpr int kNumSMs = 148;

// Error bits of MoeSched::status.
enum : int {
  kErrGemm1Timeout = 1 << 0,
  kErrGemm2Timeout = 1 << 1,
  kErrSchedOverflow = 1 << 2,
};

// Device-resident schedule, written by the permutation kernel and read by every
// later kernel; nothing in it ever travels to the host on the hot path.
struct MoeSched {
  int status;              // error bits, sticky until the next call clears them
  int n_sel;               // number of (token, local expert) rows
  int n_sel_pad;           // n_sel rounded up to 16 (slab stride in rows)
  int n_active;            // local experts with at least one token
  int n_tile;              // token-tile width the GEMMs were scheduled for
  int tiles_total;         // sum over experts of ceil(count / n_tile)
  int split1, split2;      // split-K factors chosen for GEMM1 / GEMM2 (0: balanced partition of the decode path)
  int items1, items2;      // work items of GEMM1 / GEMM2 (decode path: pipeline stages)
  unsigned int bar1[2];    // grid barrier of the decode kernel: {arrivals, call tag}
  unsigned int bar2[2];    // [0]: epoch of the decode kernel's barrier tag (the last launch's tag); [1]: spare
  int n_tile2;             // token-tile width of GEMM2 (<= n_tile)
  int ctas;                // persistent CTAs of the launch that wrote this block (decode path; else 0)
  int counts[kELocal];
  int offs[kELocal + 1];       // exclusive prefix of counts
  int tile_prefix[kELocal + 1];  // exclusive prefix of GEMM1 token tiles (width n_tile)
  int tile_prefix2[kELocal + 1]; // exclusive prefix of GEMM2 token tiles (width n_tile2)
};

// Byte offsets of the workspace arrays for a given token count.
struct WorkspaceLayout {
  int T;
  int rows_cap;        // capacity in rows: 8*T rounded up to 128
  int slab_rows;       // rows of the fp32 slab areas: max(rows_cap, kMinSlabRows)
  size_t sched, topk_idx, topk_w, local_mask, perm_token, perm_weight, tok_rows, chunk_base;
  size_t a_packed, a_scale_rows, g1, cq, c_scale, o;
  size_t acc32, tile_cnt;   // fused combine of the large-batch GEMM2: fp32 output accumulator and arrival counters
  size_t total;
};

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

inline WorkspaceLayout make_layout(int T) {
  WorkspaceLayout L{};
  L.T = T;
  L.rows_cap = static_cast<int>(align_up(static_cast<size_t>(T) * kTopK, 128));
  if (L.rows_cap < 128) L.rows_cap = 128;
  L.slab_rows = L.rows_cap > kMinSlabRows ? L.rows_cap : kMinSlabRows;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off = align_up(off + bytes, 1024);
    return o;
  };
  const size_t Tz = static_cast<size_t>(T > 0 ? T : 1);
  L.sched = take(sizeof(MoeSched));
  L.topk_idx = take(Tz * kTopK * 4);
  L.topk_w = take(Tz * kTopK * 4);
  L.local_mask = take(Tz * 4);
  L.perm_token = take(static_cast<size_t>(L.rows_cap) * 4);
  L.perm_weight = take(static_cast<size_t>(L.rows_cap) * 4);
  L.tok_rows = take(Tz * kTopK * 4);
  L.chunk_base = take((Tz + 31) / 32 * kELocal * 4);   // first row of every (32-token chunk, expert)
  L.a_packed = take(static_cast<size_t>(L.rows_cap) * kH);
  L.a_scale_rows = take(static_cast<size_t>(L.rows_cap) * kKB1 * 4);
  L.g1 = take(static_cast<size_t>(L.slab_rows) * k2I * 4);
  L.cq = take(static_cast<size_t>(kNTerms) * L.rows_cap * kI);
  L.c_scale = take(static_cast<size_t>(L.rows_cap) * kKB2 * 4);
  L.o = take(static_cast<size_t>(L.slab_rows) * kH * 4);
  L.acc32 = take(Tz * kH * 4);
  L.tile_cnt = take(Tz * kMT2 * 4);
  L.total = off;
  return L;
}

}  // namespace moe
