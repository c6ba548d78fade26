/* C ABI of the B200-native FP8 block-scale DeepSeek-V3 MoE shard
 * (definition moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048).
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless its
 * name says host.  All functions return 0 on success or a negative MOE_B200_E*
 * code.  Scratch memory is the caller's `workspace`.  What the library keeps itself:
 * a per-process cache of TMA descriptors and kernel attributes (mutex protected);
 * one 256 KB pinned host block per calling thread of ..._run_host (allocated on its
 * first small-batch call); and the fixed ~160 KB device array of
 * ..._route_static (part of the library image on every GPU that loads it).
 *
 * Alignment (checked, MOE_B200_EINVAL otherwise): routing_logits, hidden_states,
 * both weight tensors, both weight-scale tensors and output 16 bytes; workspace
 * 1024 bytes; hidden_states_scale 4 bytes; routing_bias 2 bytes.
 */
#ifndef MOE_B200_H_
#define MOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOE_B200_OK 0
#define MOE_B200_EINVAL (-1)      /* null / misaligned pointer, negative size */
#define MOE_B200_EWORKSPACE (-2)  /* workspace smaller than moe_fp8_block_scale_workspace_bytes(T) */
#define MOE_B200_ECUDA (-3)       /* a CUDA call failed; see moe_fp8_block_scale_last_cuda_error() */
#define MOE_B200_EDEVICE (-4)     /* current device is not compute capability 10.x */
#define MOE_B200_EKERNEL (-5)     /* a kernel reported an error bit (bounded wait ran out, schedule overflow) */

/* Bytes of scratch the operator needs for T tokens (worst case: every token
 * selects 8 local experts).  Includes the staging area used by ..._run_host. */
size_t moe_fp8_block_scale_workspace_bytes(int T);

/* The operator.  Replaces the reference entry point `run`
 * (moe/solution/cuda/moe.cu:2650-2662, exported at :2898; semantics
 * full-agent-pipeline/references/moe.py:29-40), destination-passing:
 *   routing_logits        f32  [T, 256]
 *   routing_bias          bf16 [256]
 *   hidden_states         e4m3 [T, 7168]
 *   hidden_states_scale   f32  [56, T]          (transposed, as the definition has it)
 *   gemm1_weights         e4m3 [32, 4096, 7168]
 *   gemm1_weights_scale   f32  [32, 32, 56]
 *   gemm2_weights         e4m3 [32, 7168, 2048]
 *   gemm2_weights_scale   f32  [32, 56, 16]
 *   output                bf16 [T, 7168]        fully overwritten
 * Asynchronous on `stream` (a cudaStream_t); never synchronises with the host,
 * whatever T is (the reference blocks the host for T >= 512, moe.cu:2755-2759).
 * T == 0 returns at once, like the reference (moe.cu:2664).
 * T <= 16 runs as ONE persistent kernel of one CTA per SM whose phases meet at
 * grid-wide barriers; it needs every SM of the device to itself.  A kernel of
 * another stream (or process) that holds SMs for the whole call keeps some of its
 * CTAs from starting: the barrier waits then run out after 0.4 s and the call
 * ends with the error bits set (..._status returns MOE_B200_EKERNEL) -- no hang,
 * but no result either.  Keep decode-sized calls alone on the device.
 * CUDA graphs: the call may be recorded in a stream capture and replayed.  Everything
 * that changes from call to call (the schedule, the decode kernel's barrier tag) lives
 * in the workspace; tensor maps and addresses are baked into the recorded launches, so
 * a replay uses the buffers of the capture.  Make one ordinary call with the same T on
 * the device first (it sets the kernels' attributes), and do not switch
 * ..._set_profiling on around a capture. */
int moe_fp8_block_scale_run(const float* routing_logits, const uint16_t* routing_bias,
                            const uint8_t* hidden_states, const float* hidden_states_scale,
                            const uint8_t* gemm1_weights, const float* gemm1_weights_scale,
                            const uint8_t* gemm2_weights, const float* gemm2_weights_scale,
                            int T, int local_expert_offset, float routed_scaling_factor,
                            uint16_t* output, void* workspace, size_t workspace_bytes, void* stream);

/* Same operator for a caller whose token-side tensors live in HOST memory
 * (pinned for full speed): copies routing_logits, routing_bias, hidden_states and
 * hidden_states_scale to the device, runs, copies `output_host` back and waits
 * for the stream.  Weights are layer parameters and stay device resident.
 * The reference harness hands `run` device tensors only; this entry is what a
 * host-side caller of that harness would otherwise write itself. */
int moe_fp8_block_scale_run_host(const float* routing_logits_host, const uint16_t* routing_bias_host,
                                 const uint8_t* hidden_states_host, const float* hidden_states_scale_host,
                                 const uint8_t* gemm1_weights, const float* gemm1_weights_scale,
                                 const uint8_t* gemm2_weights, const float* gemm2_weights_scale,
                                 int T, int local_expert_offset, float routed_scaling_factor,
                                 uint16_t* output_host, void* workspace, size_t workspace_bytes, void* stream);

/* Routing alone (the first stage of the operator): the eight selected global
 * experts per token in descending biased-score order, their combination weights,
 * and a bit mask of the experts that fall in [local_expert_offset,
 * local_expert_offset + 32).  Same arithmetic as the operator's own routing
 * (reference route_kernel, moe/solution/cuda/moe.cu:60-186; definition
 * references/moe.py:123-158).  The expert-parallel layer uses it to decide where
 * each token is dispatched.  topk_idx i32 [T,8], topk_w f32 [T,8], local_mask u32 [T]. */
int moe_fp8_block_scale_route(const float* routing_logits, const uint16_t* routing_bias, int T,
                              int local_expert_offset, float routed_scaling_factor,
                              int32_t* topk_idx, float* topk_w, uint32_t* local_mask, void* stream);

/* The step before the operator: bf16 activations [T, 7168] -> e4m3 [T, 7168] plus one
 * fp32 scale per (token, 128-column block) in the definition's transposed layout
 * [56, T] (full-agent-pipeline/references/moe.py:32-33, 95-104): scale = amax / 448,
 * q = e4m3(x / scale).  The reference has no kernel for this step (its harness
 * generates the layout on the host).  Asynchronous on `stream`. */
int moe_fp8_block_scale_quantize_activations(const uint16_t* hidden_bf16, int T, uint8_t* hidden_states,
                                             float* hidden_states_scale, void* stream);

/* The operator with a per-token destination: row t of the result is written to
 * output_rows[t] (a device array of T device pointers, each 16-byte aligned and
 * addressing 7168 bf16) instead of output + t * 7168.  The pointers may address a PEER
 * GPU's memory (NVLink peer mapping): the expert-parallel layer uses this to let the
 * combine stage of the shard operator store every row directly into the receive area
 * of the rank that owns the token, i.e. the combine all-to-all happens inside the
 * operator's last kernel.  No counterpart in the reference (it has no multi-rank code). */
int moe_fp8_block_scale_run_rows(const float* routing_logits, const uint16_t* routing_bias,
                                 const uint8_t* hidden_states, const float* hidden_states_scale,
                                 const uint8_t* gemm1_weights, const float* gemm1_weights_scale,
                                 const uint8_t* gemm2_weights, const float* gemm2_weights_scale,
                                 int T, int local_expert_offset, float routed_scaling_factor,
                                 uint16_t* const* output_rows, void* workspace, size_t workspace_bytes, void* stream);

/* Expert-parallel dispatch over peer memory: for record r of segment s (records
 * first_record .. first_record + count of rec_token, a token index each) copy the token's
 * fp8 row, its 56 scales (gathered from the [56, T] layout) and its 256 logits to
 * dst_hidden + k * 7168, dst_scale + k * 56, dst_logits + k * 256 (k = r - first_record),
 * which may be peer-mapped memory of the rank that owns the segment's shard.  At most 8
 * segments (one per shard).  No counterpart in the reference. */
typedef struct moe_ep_segment {
  int64_t first_record;
  int64_t count;
  uint8_t* dst_hidden;
  float* dst_scale;
  float* dst_logits;
} moe_ep_segment;
int moe_ep_dispatch_push(const uint8_t* hidden_states, const float* hidden_states_scale,
                         const float* routing_logits, int T, const int64_t* rec_token, int n_records,
                         const moe_ep_segment* segments, int n_segments, void* stream);

/* The same dispatch for activations that are still bf16 [T, 7168] (8-byte aligned): every token is quantised
 * once (the arithmetic of ..._quantize_activations, bit for bit) and its e4m3 row, 56 scales and logits are
 * stored to every shard it selected.  segments_by_shard has EIGHT entries indexed by shard (count 0: none);
 * row_of [T, 8] is the table ..._plan leaves: the record of (t, s) goes to position
 * row_of[t][s] - segments_by_shard[s].first_record of the segment. */
int moe_ep_quantize_push(const uint16_t* hidden_bf16, const float* routing_logits, int T, const int32_t* row_of,
                         const moe_ep_segment* segments_by_shard, void* stream);

/* Dispatch plan of one rank of the expert-parallel layer from its routing result topk_idx [T, 8] (global
 * expert ids, 16-byte aligned): counts9[s] = records for shard s = 0..7 and counts9[8] = T; send_order /
 * send_shard [sum of counts] = token and shard of every record, shard-major with ascending tokens inside a
 * shard (capacity 8 T each); row_of [T, 8] = position of the record of (token, shard) in that order, -1 if
 * the token selected no expert of the shard.  One kernel, no host synchronisation. */
int moe_ep_plan(const int32_t* topk_idx, int T, int64_t* counts9, int64_t* send_order, int64_t* send_shard,
                int32_t* row_of, void* stream);

/* out_ptrs[r] for the n_rows result rows of a rank's shard operators (the output_rows argument of
 * ..._run_rows): the rows come in up to eight runs, run k of run_count_host[k] consecutive rows whose
 * destinations start at run_base_host[k] (a device address, possibly peer-mapped) and lie row_bytes apart.
 * The two run arrays are HOST arrays; their counts must add up to n_rows. */
int moe_ep_row_pointers(const int64_t* run_base_host, const int64_t* run_count_host, int n_runs, int64_t row_bytes,
                        int64_t* out_ptrs, int n_rows, void* stream);

/* Last step of the expert-parallel layer: output[t] = bf16(sum, in ascending shard order and in fp32, of the
 * bf16 rows back_rows[row_of[t][s]] for the shards s = 0..7 with row_of[t][s] >= 0).  The order and the
 * arithmetic are those in which the layer reference sums the eight shard outputs
 * (full-agent-pipeline/references/moe.py:196-200 per shard; the reference has no multi-rank code). */
int moe_ep_sum_shards(const uint16_t* back_rows, const int32_t* row_of, int T, uint16_t* output, void* stream);

/* Waits for `stream` and returns the error bits the kernels of the last call on
 * this workspace recorded (0 = none) in *status.  The reference checks no CUDA
 * return code at all (moe.cu:2729-2894); this is the replacement's error channel. */
int moe_fp8_block_scale_status(const void* workspace, void* stream, int* status);

/* Last cudaError_t seen by this library on the calling thread, as an int. */
int moe_fp8_block_scale_last_cuda_error(void);

/* Where the intermediate arrays of the last call live inside the workspace
 * (byte offsets), for parity tests that compare selection, permutation and
 * per-stage results with the definition.  Mirrors the reference's process-global
 * Workspace (moe.cu:2511-2589), owned by the caller instead. */
typedef struct moe_b200_layout {
  int32_t T, rows_cap, slab_rows, n_terms;
  uint64_t sched;        /* moe_b200_sched                                   */
  uint64_t topk_idx;     /* i32 [T, 8] selected global experts               */
  uint64_t topk_w;       /* f32 [T, 8] combination weights                   */
  uint64_t local_mask;   /* u32 [T]    bit le <=> local expert le selected   */
  uint64_t perm_token;   /* i32 [n_sel] token of each permuted row           */
  uint64_t perm_weight;  /* f32 [n_sel]                                      */
  uint64_t tok_rows;     /* i32 [T, 8] rows of each token, ascending expert  */
  uint64_t a_packed;     /* e4m3 [rows_cap, 7168] permuted activations       */
  uint64_t a_scale_rows; /* f32 [rows_cap, 56] block scales of each permuted row  */
  uint64_t g1;           /* f32 [split1][n_sel_pad, 4096] GEMM1 slabs        */
  uint64_t cq;           /* e4m3 [n_terms][rows_cap, 2048] SwiGLU planes     */
  uint64_t c_scale;      /* f32 [rows_cap, 16]                               */
  uint64_t o;            /* f32 [split2][n_sel_pad, 7168] GEMM2 slabs        */
  uint64_t acc32;        /* f32 [T, 7168] output accumulator (fast combine)  */
  uint64_t tile_cnt;     /* i32 [T, 56] arrivals per (token, column tile)    */
  uint64_t total;        /* == moe_fp8_block_scale_workspace_bytes(T)        */
} moe_b200_layout;

typedef struct moe_b200_sched {
  int32_t status, n_sel, n_sel_pad, n_active, n_tile, tiles_total, split1, split2, items1, items2;
  uint32_t bar1[2], bar2[2];
  int32_t n_tile2, ctas;
  int32_t counts[32];
  int32_t offs[33];
  int32_t tile_prefix[33];
  int32_t tile_prefix2[33];
} moe_b200_sched;

int moe_fp8_block_scale_layout(int T, moe_b200_layout* out);

/* Process-wide options of the operator (default 0).
 *  MOE_B200_OPT_FAST_COMBINE  For calls with more than 1024 tokens the GEMM2 epilogue multiplies by the routing
 *    weight and adds straight into an fp32 [T, 7168] accumulator (vector reductions) and the last contributor of
 *    every (token, 128-column tile) casts it to bf16: the scheme of the reference's own GEMM2 epilogue
 *    (moe/solution/cuda/moe.cu:2404-2430, 2473-2496).  Faster, same tolerance, but the fp32 summation order is no
 *    longer fixed: two runs may differ in the last bf16 bit of a few elements.  Without it the combine is a
 *    separate kernel that sums a token's experts in ascending order (bit-reproducible; the order of
 *    full-agent-pipeline/references/moe.py:196-200).
 *  MOE_B200_OPT_UNFUSED  Calls with more than 1024 tokens take the same multi-kernel path as smaller ones (GEMM1 ->
 *    SwiGLU kernel -> GEMM2 -> combine kernel) instead of the large-batch kernels that fuse SwiGLU into GEMM1's
 *    epilogue.  For A/B measurements and for tests that compare the two paths bit for bit. */
#define MOE_B200_OPT_FAST_COMBINE 1u
#define MOE_B200_OPT_UNFUSED 2u
int moe_fp8_block_scale_set_options(unsigned int options);
unsigned int moe_fp8_block_scale_get_options(void);

/* Kernels launched by this library since it was loaded (all threads). */
long long moe_fp8_block_scale_launch_count(void);

/* Per-stage device timing for benchmarks: when enabled, CUDA events are
 * recorded on the caller's stream between the six stages (route+permute, gather,
 * GEMM1, SwiGLU split, GEMM2, combine).  ..._stage_times waits for the calling
 * thread's last profiled call and writes the six durations in milliseconds.
 * The reference has no counterpart; its per-kernel times were read from a profiler. */
#define MOE_B200_STAGES 6
int moe_fp8_block_scale_set_profiling(int enable);
int moe_fp8_block_scale_stage_times(float* ms, int n);

/* No counterpart in the reference.  The routing / histogram / prefix-sum /
 * permutation stage for callers that cannot allocate device memory when they need
 * it (a plugin inside an engine that owns all memory, or code that runs while the
 * allocator is off limits): the stage's scratch lives in a fixed ~160 KB device
 * array inside the library instead of a caller workspace.
 *   in : routing_logits f32 [T, 256], routing_bias bf16 [256]
 *   out: topk_idx i32 [T, 8], topk_w f32 [T, 8], expert_offsets i32 [33] (exclusive
 *        prefix of tokens per local expert), perm_token i32 [8 T] and perm_weight
 *        f32 [8 T] (first expert_offsets[32] entries valid: ascending token inside
 *        ascending local expert)
 * T above MOE_B200_STATIC_MAX_TOKENS returns MOE_B200_EINVAL.  The first call on a
 * device resolves the array's address and should come before any stream capture.
 * All calls on a device share the array, so calls that overlap on the GPU race. */
#define MOE_B200_STATIC_MAX_TOKENS 4096
int moe_fp8_block_scale_route_static(const float* routing_logits, const uint16_t* routing_bias, int T,
                                     int local_expert_offset, float routed_scaling_factor,
                                     int32_t* topk_idx, float* topk_w, int32_t* expert_offsets,
                                     int32_t* perm_token, float* perm_weight, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_H_ */
