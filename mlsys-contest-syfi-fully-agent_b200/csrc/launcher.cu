// Host launcher and C ABI (declared in include/moe_b200.h).
//
// Replaces run_impl and the process-global Workspace of the reference solution
// (moe/solution/cuda/moe.cu:2511-2589, 2650-2896).  One code path for every token
// count: route+permute -> gather -> GEMM1 -> SwiGLU/split -> GEMM2 -> combine,
// all asynchronous on the caller's stream, scratch memory owned by the caller.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/moe_b200.h"
#include "kernels.h"

namespace moe {
namespace {

thread_local int g_last_cuda_error = 0;

// Optional per-stage timing (CUDA events recorded on the caller's stream between the
// stages) and a count of the kernels this library has launched.
constexpr int kStages = 6;   // route+permute, gather, GEMM1, SwiGLU split, GEMM2, combine
std::atomic<long long> g_launches{0};
std::atomic<int> g_profiling{0};
std::atomic<unsigned> g_options{0};
struct StageEvents {
  cudaEvent_t ev[kStages + 1];
  bool created = false;
  bool recorded = false;
};
thread_local StageEvents g_events;

void stage_mark(int i, cudaStream_t stream) {
  if (!g_profiling.load(std::memory_order_relaxed)) return;
  if (!g_events.created) {
    for (auto& e : g_events.ev) cudaEventCreate(&e);
    g_events.created = true;
  }
  cudaEventRecord(g_events.ev[i], stream);
  if (i == kStages) g_events.recorded = true;
}

#define MOE_CUDA(expr)                                   \
  do {                                                   \
    cudaError_t e__ = (expr);                            \
    if (e__ != cudaSuccess) {                            \
      g_last_cuda_error = static_cast<int>(e__);         \
      return MOE_B200_ECUDA;                             \
    }                                                    \
  } while (0)

constexpr size_t kPackLimit = 256 * 1024;   // ..._run_host packs its inputs into one copy up to this size

// Staging area for ..._run_host, appended to the kernel workspace.
struct HostStage {
  size_t logits, bias, hidden, hscale, out, total;
};
HostStage make_stage(int T, size_t base) {
  HostStage s{};
  size_t off = base;
  auto take = [&](size_t b) { size_t o = off; off = align_up(off + b, 256); return o; };
  const size_t Tz = T > 0 ? T : 1;
  s.logits = take(Tz * kEGlobal * 4);
  s.bias = take(kEGlobal * 2);
  s.hidden = take(Tz * kH);
  s.hscale = take(Tz * kKB1 * 4);
  s.out = take(Tz * kH * 2);
  s.total = off;
  return s;
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int cc_major = 0;
  EncodeFn encode = nullptr;
};
std::mutex g_mu;
DeviceState g_dev[16];

struct MapKey {
  const void* ptr;
  uint32_t rank;
  uint64_t dims[4];
  uint64_t strides[3];
  uint32_t box[4];
  bool operator==(const MapKey& o) const {
    if (ptr != o.ptr || rank != o.rank) return false;
    for (uint32_t i = 0; i < rank; ++i)
      if (dims[i] != o.dims[i] || box[i] != o.box[i]) return false;
    for (uint32_t i = 0; i + 1 < rank; ++i)
      if (strides[i] != o.strides[i]) return false;
    return true;
  }
};
constexpr int kMapCache = 64;   // a call uses up to 12 maps; several batch-size classes stay cached side by side
struct MapEntry {
  MapKey key;
  CUtensorMap map;
  bool used;
};
MapEntry g_maps[kMapCache];
int g_map_next = 0;

int ensure_device(DeviceState** out) {
  int dev = 0;
  MOE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 16) return MOE_B200_EINVAL;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[dev];
  if (!d.ready) {
    MOE_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    MOE_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
    if (d.cc_major != 10) return MOE_B200_EDEVICE;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    MOE_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return MOE_B200_EDEVICE;
    d.encode = reinterpret_cast<EncodeFn>(fn);
    int rc = grouped_gemm_init();
    if (rc == 0) rc = grouped_gemm_large_init();
    if (rc == 0) rc = decode_kernel_init();
    if (rc != 0) {
      g_last_cuda_error = rc;
      return MOE_B200_ECUDA;
    }
    d.ready = true;
  }
  *out = &d;
  return MOE_B200_OK;
}

// u8 tensor map with the 128-byte swizzle; dims / box innermost first, strides in bytes for dims 1..rank-1.
int get_map(DeviceState* d, const MapKey& key, CUtensorMap* out) {
  std::lock_guard<std::mutex> lk(g_mu);
  for (auto& e : g_maps)
    if (e.used && e.key == key) {
      *out = e.map;
      return MOE_B200_OK;
    }
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
  for (uint32_t i = 0; i < key.rank; ++i) { dims[i] = key.dims[i]; box[i] = key.box[i]; }
  for (uint32_t i = 0; i + 1 < key.rank; ++i) strides[i] = key.strides[i];
  CUtensorMap m;
  CUresult r = d->encode(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, key.rank, const_cast<void*>(key.ptr), dims, strides, box,
                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = 100000 + static_cast<int>(r);
    return MOE_B200_ECUDA;
  }
  MapEntry& e = g_maps[g_map_next];
  g_map_next = (g_map_next + 1) % kMapCache;
  e.key = key;
  e.map = m;
  e.used = true;
  *out = m;
  return MOE_B200_OK;
}

// Operand [rows, K] (row-major, K in bytes) seen as [128 B inside a K-block, rows, K / 128 K-blocks]:
// one box brings `kps` consecutive K-blocks of `box_rows` rows as `kps` swizzled [box_rows x 128 B] tiles.
MapKey kblock_map(const void* ptr, uint64_t rows, uint64_t K, uint32_t box_rows, uint32_t kps) {
  MapKey k{};
  k.ptr = ptr;
  k.rank = 3;
  k.dims[0] = 128; k.dims[1] = rows; k.dims[2] = K / 128;
  k.strides[0] = K; k.strides[1] = 128;
  k.box[0] = 128; k.box[1] = box_rows; k.box[2] = kps;
  return k;
}

// The kNTerms e4m3 planes [plane][rows, 2048] of GEMM2's token operand as
// [128 B, rows, planes, K-blocks]: one box brings all planes of `kps` K-blocks, plane-major inside a K-block.
MapKey planes_map(const void* ptr, uint64_t rows, uint32_t box_rows, uint32_t kps) {
  MapKey k{};
  k.ptr = ptr;
  k.rank = 4;
  k.dims[0] = 128; k.dims[1] = rows; k.dims[2] = kNTerms; k.dims[3] = kI / 128;
  k.strides[0] = kI; k.strides[1] = rows * kI; k.strides[2] = 128;
  k.box[0] = 128; k.box[1] = box_rows; k.box[2] = kNTerms; k.box[3] = kps;
  return k;
}

// Token-tile width, chosen from T alone (no device read-back).  The tile is chosen for the rows an expert
// typically gets (T / 32 with balanced routing), not for the worst case: an expert with more rows simply takes
// several tiles.  Measured on balanced batches: 32-token tiles win up to T = 256, 64-token tiles up to T = 1024,
// 128-token tiles beyond; 33..64 tokens keep 64-token tiles, which also serve small batches that pile onto a
// few experts.
int pick_n_tile(int T) {
  return T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 256 ? 32 : T <= 1024 ? 64 : 128;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
bool aligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }
bool aligned2(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 1u) == 0; }

}  // namespace

void set_last_cuda_error(int cuda_error) { g_last_cuda_error = cuda_error; }
void count_launches(int n) { g_launches += n; }
int route_permute_launches(int T) { return T <= 32 ? 1 : T <= 1024 ? 2 : 4; }

}  // namespace moe

using namespace moe;

extern "C" size_t moe_fp8_block_scale_workspace_bytes(int T) {
  if (T < 0) return 0;
  const WorkspaceLayout L = make_layout(T);
  return make_stage(T, L.total).total;
}

extern "C" int moe_fp8_block_scale_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int moe_fp8_block_scale_layout(int T, moe_b200_layout* out) {
  if (T < 0 || out == nullptr) return MOE_B200_EINVAL;
  static_assert(sizeof(moe_b200_sched) == sizeof(MoeSched), "public and internal schedule structs differ");
  const WorkspaceLayout L = make_layout(T);
  out->T = T;
  out->rows_cap = L.rows_cap;
  out->slab_rows = L.slab_rows;
  out->n_terms = kNTerms;
  out->sched = L.sched;
  out->topk_idx = L.topk_idx;
  out->topk_w = L.topk_w;
  out->local_mask = L.local_mask;
  out->perm_token = L.perm_token;
  out->perm_weight = L.perm_weight;
  out->tok_rows = L.tok_rows;
  out->a_packed = L.a_packed;
  out->a_scale_rows = L.a_scale_rows;
  out->g1 = L.g1;
  out->cq = L.cq;
  out->c_scale = L.c_scale;
  out->o = L.o;
  out->acc32 = L.acc32;
  out->tile_cnt = L.tile_cnt;
  out->total = moe_fp8_block_scale_workspace_bytes(T);
  return MOE_B200_OK;
}

static int run_impl(const float* routing_logits, const uint16_t* routing_bias, const uint8_t* hidden_states,
                    const float* hidden_states_scale, const uint8_t* gemm1_weights, const float* gemm1_weights_scale,
                    const uint8_t* gemm2_weights, const float* gemm2_weights_scale, int T, int local_expert_offset,
                    float routed_scaling_factor, uint16_t* output, uint16_t* const* output_rows, void* workspace,
                    size_t workspace_bytes, void* stream_v) {
  if (T < 0) return MOE_B200_EINVAL;
  if (T == 0) return MOE_B200_OK;
  if (!routing_logits || !routing_bias || !hidden_states || !hidden_states_scale || !gemm1_weights ||
      !gemm1_weights_scale || !gemm2_weights || !gemm2_weights_scale || (!output && !output_rows) || !workspace)
    return MOE_B200_EINVAL;
  // vector loads and TMA: 16 bytes for the logits, the fp8 tensors, the weight scales and the output; natural
  // alignment for the rest
  if (!aligned16(routing_logits) || !aligned16(hidden_states) || !aligned16(gemm1_weights) || !aligned16(gemm2_weights) ||
      !aligned16(output) || !aligned2(routing_bias) || !aligned4(hidden_states_scale) || !aligned16(gemm1_weights_scale) ||
      !aligned16(gemm2_weights_scale) || (reinterpret_cast<uintptr_t>(workspace) & 1023u) != 0)
    return MOE_B200_EINVAL;
  if (workspace_bytes < moe_fp8_block_scale_workspace_bytes(T)) return MOE_B200_EWORKSPACE;
  DeviceState* dev = nullptr;
  int rc = ensure_device(&dev);
  if (rc != MOE_B200_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  const WorkspaceLayout L = make_layout(T);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  MoeSched* sched = reinterpret_cast<MoeSched*>(ws + L.sched);
  int* topk_idx = reinterpret_cast<int*>(ws + L.topk_idx);
  float* topk_w = reinterpret_cast<float*>(ws + L.topk_w);
  uint32_t* local_mask = reinterpret_cast<uint32_t*>(ws + L.local_mask);
  int* perm_token = reinterpret_cast<int*>(ws + L.perm_token);
  float* perm_weight = reinterpret_cast<float*>(ws + L.perm_weight);
  int* tok_rows = reinterpret_cast<int*>(ws + L.tok_rows);
  int* chunk_base = reinterpret_cast<int*>(ws + L.chunk_base);
  uint8_t* a_packed = ws + L.a_packed;
  float* a_scale_rows = reinterpret_cast<float*>(ws + L.a_scale_rows);
  float* g1 = reinterpret_cast<float*>(ws + L.g1);
  uint8_t* cq = ws + L.cq;
  float* c_scale = reinterpret_cast<float*>(ws + L.c_scale);
  float* o = reinterpret_cast<float*>(ws + L.o);
  float* acc32 = reinterpret_cast<float*>(ws + L.acc32);
  int* tile_cnt = reinterpret_cast<int*>(ws + L.tile_cnt);
  const unsigned opts = g_options.load(std::memory_order_relaxed);
  // more than 1024 tokens: 128-token tiles, SwiGLU in GEMM1's epilogue, optionally the combine in GEMM2's
  const bool large = T > 1024 && !(opts & MOE_B200_OPT_UNFUSED);
  const bool fast_combine = large && (opts & MOE_B200_OPT_FAST_COMBINE);

  const int n_tile = pick_n_tile(T);
  // GEMM2's three-plane token operand does not fit 256-token stages; and from 33 to 768 tokens it takes 32-token
  // tiles whatever GEMM1 takes (two K-blocks per TMEM hand-off): 4-7 % faster on the whole call for balanced
  // batches, 6 % slower on batches of 512+ tokens that pile 250+ rows onto each of a few experts.
  const int n_tile2 = (T > 32 && T <= 768) ? 32 : n_tile > 128 ? 128 : n_tile;
  const int ctas = dev->sm_count;

  CUtensorMap tm_w13, tm_w2, tm_a, tm_c;
  const bool decode = T <= kFusedMaxTokens;
  const uint32_t kps1 = decode ? kDecodeKps : grouped_gemm_kblocks_per_stage(1, n_tile);
  const uint32_t kps2 = decode ? kDecodeKps : grouped_gemm_kblocks_per_stage(2, n_tile2);
  // (the large-batch kernels take one K-block per box)
  if ((rc = get_map(dev, kblock_map(gemm1_weights, static_cast<uint64_t>(kELocal) * k2I, kH, 128, large ? 1 : kps1), &tm_w13)))
    return rc;
  if ((rc = get_map(dev, kblock_map(gemm2_weights, static_cast<uint64_t>(kELocal) * kH, kI, 128, kps2), &tm_w2)))
    return rc;
  if ((rc = get_map(dev, kblock_map(a_packed, L.rows_cap, kH, n_tile, large ? 1 : kps1), &tm_a))) return rc;
  if ((rc = get_map(dev, planes_map(cq, L.rows_cap, n_tile2, kps2), &tm_c))) return rc;

  if (T <= kFusedMaxTokens) {
    // Decode path: one launch.  The kernel routes, reads the token rows straight from hidden_states (all
    // tokens are one token tile), and runs both GEMMs with the SwiGLU and combine phases in between and after.
    CUtensorMap tm_h;
    if ((rc = get_map(dev, kblock_map(hidden_states, static_cast<uint64_t>(T), kH, kFusedMaxTokens, kps1), &tm_h)))
      return rc;
    GemmArgs fa{};
    fa.sched = sched; fa.w_scale = gemm1_weights_scale; fa.b_scale = nullptr; fa.out = g1;
    fa.logits = routing_logits; fa.bias_bf16 = routing_bias; fa.hidden_scale = hidden_states_scale;
    fa.T = T; fa.local_expert_offset = local_expert_offset; fa.routed_scaling_factor = routed_scaling_factor;
    fa.ctas = ctas; fa.rows_cap = L.rows_cap; fa.slab_rows = L.slab_rows;
    fa.topk_idx = topk_idx; fa.topk_w = topk_w; fa.local_mask = local_mask;
    fa.perm_token = perm_token; fa.perm_weight = perm_weight; fa.tok_rows = tok_rows;
    fa.cq = cq; fa.c_scale = c_scale; fa.out_bf16 = output; fa.out_rows = output_rows;
    stage_mark(0, stream); stage_mark(1, stream); stage_mark(2, stream);
    if ((rc = launch_decode(tm_w13, tm_h, tm_w2, tm_c, fa, gemm2_weights_scale, o, ctas, stream))) {
      g_last_cuda_error = rc;
      return MOE_B200_ECUDA;
    }
    stage_mark(3, stream); stage_mark(4, stream); stage_mark(5, stream); stage_mark(6, stream);
    g_launches += 1;
    return MOE_B200_OK;
  }

  RouteArgs ra{routing_logits, routing_bias, T, local_expert_offset, routed_scaling_factor, topk_idx, topk_w,
               local_mask};
  PermuteArgs pa{T, local_expert_offset, n_tile, n_tile2, ctas, static_cast<int>(kps1), static_cast<int>(kps2), L.rows_cap, L.slab_rows, local_mask, topk_idx, topk_w,
                 sched, perm_token, perm_weight, tok_rows, chunk_base, large ? 2 : 0};
  stage_mark(0, stream);
  launch_route_permute(ra, pa, stream);
  MOE_CUDA(cudaGetLastError());
  g_launches += route_permute_launches(T);
  stage_mark(1, stream);

  GatherArgs ga{sched, perm_token, hidden_states, hidden_states_scale, T, a_packed, a_scale_rows};
  launch_gather_rows(ga, T, stream);
  MOE_CUDA(cudaGetLastError());
  g_launches += 1;
  stage_mark(2, stream);

  GemmArgs g1a{};
  g1a.sched = sched; g1a.w_scale = gemm1_weights_scale; g1a.b_scale = a_scale_rows; g1a.out = g1;
  g1a.rows_cap = L.rows_cap; g1a.cq = cq; g1a.c_scale = c_scale;
  GemmArgs g2a{};
  g2a.sched = sched; g2a.w_scale = gemm2_weights_scale; g2a.b_scale = c_scale; g2a.out = o;
  g2a.rows_cap = L.rows_cap; g2a.perm_token = perm_token; g2a.perm_weight = perm_weight; g2a.local_mask = local_mask;
  g2a.acc32 = acc32; g2a.tile_cnt = tile_cnt; g2a.out_bf16 = output; g2a.out_rows = output_rows;

  if (large) {
    if (fast_combine) {
      // accumulator + counters are one span of the workspace
      const size_t span = (L.tile_cnt - L.acc32) + static_cast<size_t>(T) * kMT2 * 4;
      if ((rc = launch_combine_prepare(acc32, span / 4, local_mask, T, output, output_rows, stream))) {
        g_last_cuda_error = rc;
        return MOE_B200_ECUDA;
      }
      g_launches += 1;
    }
    if ((rc = launch_grouped_gemm_large(1, false, tm_w13, tm_a, g1a, ctas, stream))) {
      g_last_cuda_error = rc;
      return MOE_B200_ECUDA;
    }
    g_launches += 1;
    stage_mark(3, stream);
    stage_mark(4, stream);      // no SwiGLU kernel on this path
    if ((rc = launch_grouped_gemm_large(2, fast_combine, tm_w2, tm_c, g2a, ctas, stream))) {
      g_last_cuda_error = rc;
      return MOE_B200_ECUDA;
    }
    g_launches += 1;
    stage_mark(5, stream);
  } else {
    // token operands with boxes of 1..4 row steps (ragged token tiles bring only the rows they have)
    TokenMaps tms_a, tms_c;
    const int step1 = grouped_gemm_row_step(n_tile), step2 = grouped_gemm_row_step(n_tile2);
    for (int i = 0; i < 4; ++i) {
      const uint32_t r1 = static_cast<uint32_t>(std::min(n_tile, step1 * (i + 1)));
      const uint32_t r2 = static_cast<uint32_t>(std::min(n_tile2, step2 * (i + 1)));
      if ((rc = get_map(dev, kblock_map(a_packed, L.rows_cap, kH, r1, kps1), &tms_a.m[i]))) return rc;
      if ((rc = get_map(dev, planes_map(cq, L.rows_cap, r2, kps2), &tms_c.m[i]))) return rc;
    }
    if ((rc = launch_grouped_gemm(1, n_tile, tm_w13, tms_a, g1a, ctas, stream))) {
      g_last_cuda_error = rc;
      return MOE_B200_ECUDA;
    }
    g_launches += 1;
    stage_mark(3, stream);

    SwigluArgs sa{sched, g1, cq, c_scale, L.rows_cap};
    launch_swiglu_split(sa, T, stream);
    MOE_CUDA(cudaGetLastError());
    g_launches += 1;
    stage_mark(4, stream);

    if ((rc = launch_grouped_gemm(2, n_tile2, tm_w2, tms_c, g2a, ctas, stream))) {
      g_last_cuda_error = rc;
      return MOE_B200_ECUDA;
    }
    g_launches += 1;
    stage_mark(5, stream);
  }

  if (!fast_combine) {
    CombineArgs ca{sched, o, local_mask, tok_rows, perm_weight, output, T, output_rows};
    launch_combine(ca, stream);
    MOE_CUDA(cudaGetLastError());
    g_launches += 1;
  }
  stage_mark(6, stream);
  return MOE_B200_OK;
}

extern "C" int moe_fp8_block_scale_run(const float* routing_logits, const uint16_t* routing_bias,
                                       const uint8_t* hidden_states, const float* hidden_states_scale,
                                       const uint8_t* gemm1_weights, const float* gemm1_weights_scale,
                                       const uint8_t* gemm2_weights, const float* gemm2_weights_scale, int T,
                                       int local_expert_offset, float routed_scaling_factor, uint16_t* output,
                                       void* workspace, size_t workspace_bytes, void* stream_v) {
  if (T > 0 && !output) return MOE_B200_EINVAL;
  return run_impl(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
                  gemm2_weights, gemm2_weights_scale, T, local_expert_offset, routed_scaling_factor, output, nullptr,
                  workspace, workspace_bytes, stream_v);
}

extern "C" int moe_fp8_block_scale_run_rows(const float* routing_logits, const uint16_t* routing_bias,
                                            const uint8_t* hidden_states, const float* hidden_states_scale,
                                            const uint8_t* gemm1_weights, const float* gemm1_weights_scale,
                                            const uint8_t* gemm2_weights, const float* gemm2_weights_scale, int T,
                                            int local_expert_offset, float routed_scaling_factor,
                                            uint16_t* const* output_rows, void* workspace, size_t workspace_bytes,
                                            void* stream_v) {
  if (T > 0 && !output_rows) return MOE_B200_EINVAL;
  return run_impl(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
                  gemm2_weights, gemm2_weights_scale, T, local_expert_offset, routed_scaling_factor, nullptr,
                  output_rows, workspace, workspace_bytes, stream_v);
}

extern "C" int moe_fp8_block_scale_run_host(const float* routing_logits_host, const uint16_t* routing_bias_host,
                                            const uint8_t* hidden_states_host, const float* hidden_states_scale_host,
                                            const uint8_t* gemm1_weights, const float* gemm1_weights_scale,
                                            const uint8_t* gemm2_weights, const float* gemm2_weights_scale, int T,
                                            int local_expert_offset, float routed_scaling_factor,
                                            uint16_t* output_host, void* workspace, size_t workspace_bytes,
                                            void* stream_v) {
  if (T < 0) return MOE_B200_EINVAL;
  if (T == 0) return MOE_B200_OK;
  if (!routing_logits_host || !routing_bias_host || !hidden_states_host || !hidden_states_scale_host || !output_host ||
      !workspace)
    return MOE_B200_EINVAL;
  if (workspace_bytes < moe_fp8_block_scale_workspace_bytes(T)) return MOE_B200_EWORKSPACE;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const HostStage st = make_stage(T, make_layout(T).total);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* d_logits = reinterpret_cast<float*>(ws + st.logits);
  uint16_t* d_bias = reinterpret_cast<uint16_t*>(ws + st.bias);
  uint8_t* d_hidden = ws + st.hidden;
  float* d_hscale = reinterpret_cast<float*>(ws + st.hscale);
  uint16_t* d_out = reinterpret_cast<uint16_t*>(ws + st.out);
  const size_t Tz = static_cast<size_t>(T);
  const size_t in_bytes = st.out - st.logits;     // logits | bias | hidden | scales are contiguous in the staging area
  if (in_bytes <= kPackLimit) {
    // Small batches: one copy instead of four.  The inputs are packed into one of two pinned blocks owned by
    // this thread (allocated once) at the offsets of the device staging area.  The blocks alternate and each
    // has an event recorded behind the copy that read it, so a call only ever waits for the copy of the call
    // before the previous one, not for the stream.
    struct PinnedPair {
      uint8_t* block[2] = {nullptr, nullptr};
      cudaEvent_t copied[2] = {nullptr, nullptr};
      int next = 0;
    };
    static thread_local PinnedPair pairs[16];      // events belong to a device: one pair per device
    int cur = 0;
    MOE_CUDA(cudaGetDevice(&cur));
    if (cur < 0 || cur >= 16) return MOE_B200_EINVAL;
    PinnedPair& pp = pairs[cur];
    if (pp.block[0] == nullptr) {
      for (int b = 0; b < 2; ++b) {
        MOE_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&pp.block[b]), kPackLimit, cudaHostAllocDefault));
        MOE_CUDA(cudaEventCreateWithFlags(&pp.copied[b], cudaEventDisableTiming));
        MOE_CUDA(cudaEventRecord(pp.copied[b], stream));
      }
    }
    const int b = pp.next;
    pp.next ^= 1;
    MOE_CUDA(cudaEventSynchronize(pp.copied[b]));
    uint8_t* pinned = pp.block[b];
    std::memcpy(pinned, routing_logits_host, Tz * kEGlobal * 4);
    std::memcpy(pinned + (st.bias - st.logits), routing_bias_host, kEGlobal * 2);
    std::memcpy(pinned + (st.hidden - st.logits), hidden_states_host, Tz * kH);
    std::memcpy(pinned + (st.hscale - st.logits), hidden_states_scale_host, Tz * kKB1 * 4);
    MOE_CUDA(cudaMemcpyAsync(ws + st.logits, pinned, in_bytes, cudaMemcpyHostToDevice, stream));
    MOE_CUDA(cudaEventRecord(pp.copied[b], stream));
  } else {
    MOE_CUDA(cudaMemcpyAsync(d_logits, routing_logits_host, Tz * kEGlobal * 4, cudaMemcpyHostToDevice, stream));
    MOE_CUDA(cudaMemcpyAsync(d_bias, routing_bias_host, kEGlobal * 2, cudaMemcpyHostToDevice, stream));
    MOE_CUDA(cudaMemcpyAsync(d_hidden, hidden_states_host, Tz * kH, cudaMemcpyHostToDevice, stream));
    MOE_CUDA(cudaMemcpyAsync(d_hscale, hidden_states_scale_host, Tz * kKB1 * 4, cudaMemcpyHostToDevice, stream));
  }
  // Pinned (page-locked) host memory is addressable from the device, so the combine kernel can write
  // the bf16 result straight into the caller's buffer and the device-to-host copy disappears; pageable
  // buffers go through the staging area and one copy.
  cudaPointerAttributes attr{};
  const bool direct = Tz * kH * 2 <= kPackLimit && cudaPointerGetAttributes(&attr, output_host) == cudaSuccess &&
                      attr.type == cudaMemoryTypeHost && attr.devicePointer != nullptr && aligned16(attr.devicePointer);
  cudaGetLastError();   // a failed attribute query on pageable memory is not an error of this call
  uint16_t* out_dev = direct ? static_cast<uint16_t*>(attr.devicePointer) : d_out;
  int rc = moe_fp8_block_scale_run(d_logits, d_bias, d_hidden, d_hscale, gemm1_weights, gemm1_weights_scale,
                                   gemm2_weights, gemm2_weights_scale, T, local_expert_offset, routed_scaling_factor,
                                   out_dev, workspace, workspace_bytes, stream_v);
  if (rc != MOE_B200_OK) return rc;
  if (!direct) MOE_CUDA(cudaMemcpyAsync(output_host, d_out, Tz * kH * 2, cudaMemcpyDeviceToHost, stream));
  MOE_CUDA(cudaStreamSynchronize(stream));
  return MOE_B200_OK;
}

extern "C" int moe_fp8_block_scale_route(const float* routing_logits, const uint16_t* routing_bias, int T,
                                         int local_expert_offset, float routed_scaling_factor, int32_t* topk_idx,
                                         float* topk_w, uint32_t* local_mask, void* stream_v) {
  if (T < 0) return MOE_B200_EINVAL;
  if (T == 0) return MOE_B200_OK;
  if (!routing_logits || !routing_bias || !topk_idx || !topk_w || !local_mask) return MOE_B200_EINVAL;
  RouteArgs ra{routing_logits, routing_bias, T, local_expert_offset, routed_scaling_factor, topk_idx, topk_w,
               local_mask};
  launch_route_only(ra, static_cast<cudaStream_t>(stream_v));
  MOE_CUDA(cudaGetLastError());
  g_launches += 1;
  return MOE_B200_OK;
}

extern "C" int moe_fp8_block_scale_status(const void* workspace, void* stream_v, int* status) {
  if (!workspace || !status) return MOE_B200_EINVAL;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  MOE_CUDA(cudaStreamSynchronize(stream));
  const WorkspaceLayout L = make_layout(1);
  MOE_CUDA(cudaMemcpy(status, static_cast<const uint8_t*>(workspace) + L.sched, sizeof(int), cudaMemcpyDeviceToHost));
  return *status == 0 ? MOE_B200_OK : MOE_B200_EKERNEL;
}

extern "C" long long moe_fp8_block_scale_launch_count(void) { return g_launches.load(); }

extern "C" int moe_fp8_block_scale_set_options(unsigned int options) {
  if (options & ~(MOE_B200_OPT_FAST_COMBINE | MOE_B200_OPT_UNFUSED)) return MOE_B200_EINVAL;
  g_options.store(options);
  return MOE_B200_OK;
}

extern "C" unsigned int moe_fp8_block_scale_get_options(void) { return g_options.load(); }

extern "C" int moe_fp8_block_scale_set_profiling(int enable) {
  g_profiling.store(enable ? 1 : 0);
  return MOE_B200_OK;
}

extern "C" int moe_fp8_block_scale_stage_times(float* ms, int n) {
  if (!ms || n < kStages) return MOE_B200_EINVAL;
  if (!g_events.recorded) return MOE_B200_EINVAL;
  MOE_CUDA(cudaEventSynchronize(g_events.ev[kStages]));
  for (int i = 0; i < kStages; ++i) MOE_CUDA(cudaEventElapsedTime(&ms[i], g_events.ev[i], g_events.ev[i + 1]));
  return MOE_B200_OK;
}
