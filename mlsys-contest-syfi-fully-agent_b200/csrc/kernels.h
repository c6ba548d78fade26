// Argument blocks and host-side launch functions of the kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "moe_layout.h"

namespace moe {

// Programmatic dependent launch: every kernel of the operator is launched with the
// programmatic-stream-serialization attribute, signals `launch_dependents` as its first
// instruction (so the next kernel's launch latency, barrier initialisation and TMEM
// allocation overlap this kernel's execution) and executes `griddep_wait` before its first
// access to memory that an earlier kernel in the stream may still be writing.  Because the
// signal is given at CTA start, the dependent grid can only be scheduled once every CTA of
// this grid is resident, so early dependents never starve their prerequisite.
#ifdef __CUDACC__
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

struct RouteArgs {
  const float* logits;          // [T, 256]
  const uint16_t* bias_bf16;    // [256]
  int T;
  int local_expert_offset;
  float routed_scaling_factor;
  int* topk_idx;                // [T, 8] global expert ids, descending biased score
  float* topk_w;                // [T, 8] combination weights
  uint32_t* local_mask;         // [T] bit le set when local expert le is selected
};

struct PermuteArgs {
  int T;
  int local_expert_offset;
  int n_tile, n_tile2;          // token-tile widths GEMM1 / GEMM2 will use
  int ctas;                     // persistent CTAs the GEMMs will run
  int kps1, kps2;               // K-blocks per pipeline stage of the two GEMM kernels (split granularity)
  int rows_cap, slab_rows;
  const uint32_t* local_mask;
  const int* topk_idx;
  const float* topk_w;
  MoeSched* sched;
  int* perm_token;              // [n_sel] token of each row
  float* perm_weight;           // [n_sel] combination weight of each row
  int* tok_rows;                // [T, 8] rows of a token in ascending local expert order
  int* chunk_base;              // [ceil(T / 32), 32] first row of every (32-token chunk, expert); large T only
  int large;                    // 1: GEMM1 with the SwiGLU epilogue (no split-K, items are (token tile, 128-column block of C));
                                // 2: also the large-batch GEMM2 (no split-K either, items are (token tile, 256 weight rows))
};

struct GatherArgs {
  const MoeSched* sched;
  const int* perm_token;
  const uint8_t* hidden;        // [T, 7168] e4m3
  const float* hidden_scale;    // [56, T]
  int T;
  uint8_t* a_packed;            // [rows_cap, 7168]
  float* a_scale_rows;          // [rows_cap, 56] scales of each permuted row, row-major
};

// Grouped, swap-AB, split-K fp8 GEMM: out[slab][row, m] = sum_k W_e[m, k] * B[row, k] with the
// 128-block scales applied per K-block.  Used for GEMM1 (B = packed activations) and
// GEMM2 (B = kNTerms e4m3 planes of the SwiGLU output).
struct GemmArgs {
  MoeSched* sched;
  const float* w_scale;         // [32, M/128, K/128]
  const float* b_scale;         // per-row scales, row-major: GEMM1 [rows, 56]; GEMM2 [rows, 16]
  float* out;                   // fp32 slabs [split][n_sel_pad, M]
  // ---- only read by the single-launch decode kernel (T <= 16), see decode_kernel.cu
  const float* logits;          // [T, 256]
  const uint16_t* bias_bf16;    // [256]
  const float* hidden_scale;    // [56, T]
  int T, local_expert_offset;
  float routed_scaling_factor;
  int ctas, rows_cap, slab_rows;
  int* topk_idx; float* topk_w; uint32_t* local_mask;
  int* perm_token; float* perm_weight; int* tok_rows;
  uint8_t* cq; float* c_scale;  // SwiGLU planes and their scales
  uint16_t* out_bf16;           // final output
  uint16_t* const* out_rows;    // optional per-token destinations instead of out_bf16 (may be peer memory)
  // ---- only read by the large-batch GEMM2 with the fused combine (grouped_gemm_large.cu)
  float* acc32;                 // [T, 7168] fp32 accumulator of the output, zero before the launch
  int* tile_cnt;                // [T, 56] contributions that have arrived per (token, 128-column tile), zero before
};

struct SwigluArgs {
  const MoeSched* sched;
  const float* g1;              // slabs [split1][n_sel_pad, 4096]
  uint8_t* cq;                  // [kNTerms][rows_cap, 2048] e4m3 planes
  float* c_scale;               // [rows_cap, 16] power-of-two plane scale per 128 block
  int rows_cap;
};

struct CombineArgs {
  const MoeSched* sched;
  const float* o;               // slabs [split2][n_sel_pad, 7168]
  const uint32_t* local_mask;
  const int* tok_rows;
  const float* perm_weight;
  uint16_t* out_bf16;           // [T, 7168]
  int T;
  uint16_t* const* out_rows;    // optional: destination of every token's row (may be peer memory)
};

// Shared by every translation unit with an entry point: the calling thread's last cudaError_t (what
// moe_fp8_block_scale_last_cuda_error returns) and the library's launch counter.
void set_last_cuda_error(int cuda_error);
void count_launches(int n);
int route_permute_launches(int T);   // kernels launch_route_permute starts for T tokens

void launch_route_permute(const RouteArgs& r, const PermuteArgs& p, cudaStream_t stream);
void launch_route_only(const RouteArgs& r, cudaStream_t stream);
void launch_gather_rows(const GatherArgs& a, int T, cudaStream_t stream);
// gemm_id 1 or 2; n_tile in {16, 32, 64, 128}.  Returns a cudaError_t as int.
// Token-operand tensor maps of grouped_gemm_kernel: the same tensor with boxes of 1..4 row steps
// (grouped_gemm_row_step(n_tile) rows each), so that a token tile with few valid rows (the last tile of an
// expert, or an expert with a handful of tokens) brings only the rows it has, rounded up to a step.
struct TokenMaps {
  CUtensorMap m[4];
};
int grouped_gemm_row_step(int n_tile);   // rows per step: n_tile / 4 from 64-token tiles up, else 16
int launch_grouped_gemm(int gemm_id, int n_tile, const CUtensorMap& tm_w, const TokenMaps& tm_b, const GemmArgs& a,
                        int ctas, cudaStream_t stream);
constexpr int kFusedMaxTokens = 16;
constexpr int kDecodeKps = 2;   // K-blocks per pipeline stage (and per TMA box) of the decode kernel
// Decode path in one launch: routing, GEMM1, SwiGLU, GEMM2 and combine (decode_kernel.cu).  `g` is the GEMM1 view
// of the arguments with all routing / tail fields set; tm_x maps hidden_states, tm_c the SwiGLU planes.
int launch_decode(const CUtensorMap& tm_w1, const CUtensorMap& tm_x, const CUtensorMap& tm_w2, const CUtensorMap& tm_c,
                  const GemmArgs& g, const float* w2_scale, float* o, int ctas, cudaStream_t stream);
int decode_kernel_init();
int grouped_gemm_kblocks_per_stage(int gemm_id, int n_tile);   // K-blocks one TMA box of that kernel brings
int grouped_gemm_init();   // one-time function attributes (dynamic shared memory opt-in)
// Large batches (128-token tiles): GEMM1 with SwiGLU and the e4m3 plane split in its epilogue; GEMM2 storing fp32 rows
// for the deterministic combine kernel, or (fused_combine) adding weighted rows into acc32 with a last-arriver bf16 cast.
int grouped_gemm_large_init();
int launch_grouped_gemm_large(int gemm_id, bool fused_combine, const CUtensorMap& tm_w, const CUtensorMap& tm_b,
                              const GemmArgs& a, int ctas, cudaStream_t stream);
// Zeroes `acc_floats` floats at acc32 (the accumulator and the counters behind it) and writes zero output rows for
// tokens without a local expert.
int launch_combine_prepare(float* acc32, size_t acc_floats, const uint32_t* local_mask, int T, uint16_t* out_bf16,
                           uint16_t* const* out_rows, cudaStream_t stream);
void launch_swiglu_split(const SwigluArgs& a, int T, cudaStream_t stream);
void launch_combine(const CombineArgs& a, cudaStream_t stream);

}  // namespace moe
