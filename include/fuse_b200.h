/*
 * fuse_b200 -- C ABI of the B200 (sm_100a) implementation of the fused Ulysses projection
 * operators.
 *
 * Every entry point takes plain pointers and sizes.  The parameter records are
 * layout-identical to the C++ records of the interface they replace (same members, same
 * order, enums as int32_t, bool as uint8_t), so a C++ caller of that interface can pass its
 * own struct through a reinterpret_cast; fuse_b200_abi_sizeof() lets a binding check this at
 * load time.  All functions return a cudaError_t value as int (0 = success, 1 = invalid
 * value, 801 = not supported, ...); nothing throws.
 *
 * Ownership is the caller's throughout: inputs, outputs, staging, ready/done flag arrays
 * (zeroed once; epochs start at 1 and must grow with every launch), peer mappings.  The
 * library allocates no device memory on the launch path.
 *
 * Each declaration cites the interface it replaces as file:line inside the reference
 * project (CyberSecurityErial/fuse).
 */
#ifndef FUSE_B200_H_
#define FUSE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FUSE_API __attribute__((visibility("default")))
#else
#define FUSE_API
#endif

#define FUSE_MAX_WORLD_SIZE 8      /* include/fuse/types.h:16 */
#define FUSE_READY_FLAG_STRIDE 32  /* include/fuse/types.h:18 : u32 words per flag */

typedef uint16_t fuse_bf16;            /* BF16 bit pattern */
typedef struct CUstream_st* fuse_stream; /* cudaStream_t */

/* include/fuse/layout/gemm.h:8-12 */
enum { FUSE_RASTER_HEURISTIC = 0, FUSE_RASTER_ALONG_M = 1, FUSE_RASTER_ALONG_N = 2 };
/* include/fuse/layout/gemm.h:14-17 */
enum { FUSE_DTYPE_BF16 = 0, FUSE_DTYPE_E4M3 = 1 };
/* include/fuse/layout/ulysses.h:14-22 */
enum { FUSE_ROUTE_HEAD_TO_SEQUENCE = 0, FUSE_ROUTE_QKV_GQA_PACK = 2 };
enum { FUSE_ROUTE_FORWARD = 0, FUSE_ROUTE_INVERSE = 1 };

/* include/fuse/layout/gemm.h:21-25.  Strides in elements; negative = packed. */
typedef struct fuse_matrix_stride {
  int64_t row, column, batch;
} fuse_matrix_stride;

/* include/fuse/layout/gemm.h:27-42 (GemmProblem / GemmShape4D). */
typedef struct fuse_gemm_problem {
  int32_t m, n, k, l;
  fuse_matrix_stride stride_a, stride_b, stride_d;
  int32_t input_dtype, weight_dtype, output_dtype;
  uint8_t transpose_a, transpose_b;
  int32_t raster;
  int32_t max_swizzle_size;
} fuse_gemm_problem;

/* include/fuse/layout/ulysses.h:24-63 (UlyssesRoute). */
typedef struct fuse_ulysses_route {
  int32_t world_size, rank, batch, global_seq, seq_local;
  int32_t q_heads, kv_heads, local_heads, head_dim, channel_count;
  uint8_t qkv_peer_interleaved, defer_v_a2a, causal_load_balanced, cyclic_peer_order;
  const int32_t* packed_source_row;
  int32_t packed_row_granularity;
  int32_t kind;
  int32_t direction;
} fuse_ulysses_route;

/* include/fuse/types.h:37-43 (KernelTraits). */
typedef struct fuse_kernel_traits {
  int32_t block_m, block_n, block_k, threads, dynamic_smem_bytes;
} fuse_kernel_traits;

/* include/fuse/operators/primitives/gemm_a2a.h:17-30 (GemmA2AParams): dense projection
 * Y[M,N] = alpha * X[M,K] W[N,K]^T followed by the sequence->head all-to-all.  peer_output[r]
 * is rank r's contiguous planar Q | K | V tensor ([B*S_global, q_local], [.., kv_local] x 2);
 * peer_route_done_epoch[r] is rank r's array of world_size completion flags (one
 * FUSE_READY_FLAG_STRIDE apart); ready has (M/block_m)*(N/block_n) flags of the same
 * stride. */
typedef struct fuse_gemm_a2a_params {
  const fuse_bf16* lhs;
  const fuse_bf16* rhs_nt;
  fuse_bf16* local_output;
  fuse_bf16* peer_output[FUSE_MAX_WORLD_SIZE];
  uint32_t* peer_route_done_epoch[FUSE_MAX_WORLD_SIZE];
  uint32_t* ready;
  uint32_t* completion_epoch;
  fuse_gemm_problem gemm;
  fuse_ulysses_route route;
  int32_t num_comm_ctas;
  uint32_t epoch;
  float alpha;
} fuse_gemm_a2a_params;

/* include/fuse/operators/primitives/a2a_gemm.h:47-61 (A2AGemmParams): head->sequence
 * all-to-all producing the row-major lhs [M,K] in input_staging, then
 * Y[M,N] = alpha * lhs W[N,K]^T.  peer_input[p] is rank p's head-sharded tensor
 * [B*S_global, K/world]; peer_input_ready[p] (optional) is the upstream epoch word of that
 * tensor; ready has fuse_a2a_lhs_gemm_ready_elements() words. */
typedef struct fuse_a2a_gemm_params {
  const fuse_bf16* peer_input[FUSE_MAX_WORLD_SIZE];
  fuse_bf16* input_staging;
  const uint32_t* peer_input_ready[FUSE_MAX_WORLD_SIZE];
  fuse_bf16* rhs_nt;
  fuse_bf16* output;
  uint32_t* ready;
  fuse_gemm_problem gemm;
  fuse_ulysses_route route;
  int32_t num_comm_ctas;
  int32_t lhs_policy;
  uint32_t epoch;
  uint32_t input_epoch;
  float alpha;
} fuse_a2a_gemm_params;

/* Additions of this implementation, all optional (pass NULL for defaults).  They have no
 * counterpart in the reference, whose device waits are unbounded. */
enum {
  /* Do not wait for the peers' completion epochs (used when several ranks are emulated by
   * consecutive launches on one GPU). */
  FUSE_B200_SKIP_PEER_WAIT = 1u,
  /* QKV operator: route the output from communication CTAs (the reference's structure) or
   * straight from every compute CTA's epilogue (num_comm_ctas then only has to be valid).
   * Neither flag: environment variable FUSE_B200_QKV_ROUTE = comm | direct, else comm. */
  FUSE_B200_QKV_ROUTE_COMM_CTAS = 2u,
  FUSE_B200_QKV_ROUTE_DIRECT = 4u,
  /* Output-projection operator: communication CTAs pull with 16-byte loads/stores instead of
   * the bulk-copy pipeline. */
  FUSE_B200_VECTOR_PULL = 8u,
  /* Write outputs with 16-byte stores from registers instead of tensor stores staged in
   * shared memory. */
  FUSE_B200_VECTOR_EPILOGUE = 16u,
  /* Run only the communication CTAs / only the compute CTAs of a fused kernel.  For emulating
   * several ranks on one GPU when the GEMM waits for data that other ranks push (QKV backward):
   * every rank pushes first, then every rank computes. */
  FUSE_B200_COMM_ONLY = 32u,
  FUSE_B200_COMPUTE_ONLY = 64u
};
typedef struct fuse_b200_options {
  uint64_t wait_budget_ns; /* per-wait limit; 0 = FUSE_B200_WAIT_MS env (default 2000 ms) */
  uint32_t flags;
  int32_t block_n;         /* 0 = choose; 128 or 256 */
  /* Optional %globaltimer trace of one CTA (device buffer of 1 + 2*trace_capacity uint64:
   * word 0 = record count, then (thread<<32 | site, nanoseconds) pairs).  NULL = off. */
  unsigned long long* trace;
  uint32_t trace_capacity;
  int32_t trace_cta;
} fuse_b200_options;

/* csrc/operators/sm103/api/forward.cuh:12-14 -> detail/launch.cuh:497-625. */
FUSE_API int fuse_launch_gemm_a2a_cutlass(const fuse_gemm_a2a_params* params, fuse_stream stream);
FUSE_API int fuse_launch_gemm_a2a_cutlass_ex(const fuse_gemm_a2a_params* params,
                                    const fuse_b200_options* options, fuse_stream stream);
/* csrc/operators/sm103/api/forward.cuh:6-10 -> detail/launch.cuh:364-485. */
FUSE_API int fuse_launch_a2a_gemm_cutlass(const fuse_a2a_gemm_params* params, fuse_stream stream);
FUSE_API int fuse_launch_a2a_gemm_cutlass_ex(const fuse_a2a_gemm_params* params,
                                    const fuse_b200_options* options, fuse_stream stream);
/* include/fuse/operators/primitives/gemm_a2a.h:107-110 (launch_batched_cutlass_reference):
 * the projection GEMM alone on (SMs - reserved_comm_ctas) CTAs; the full-SM denominator. */
FUSE_API int fuse_launch_batched_cutlass_reference(const fuse_gemm_a2a_params* params, fuse_stream stream,
                                          int32_t reserved_comm_ctas);
/* include/fuse/operators/primitives/a2a_gemm.h:126-129 (launch_a2a_gemm_cutlass_reference):
 * GEMM alone reading input_staging. */
FUSE_API int fuse_launch_a2a_gemm_cutlass_reference(const fuse_a2a_gemm_params* params, fuse_stream stream,
                                           int32_t reserved_comm_ctas);

/* include/fuse/operators/primitives/gemm_a2a.h:59-66 (qkv_cutlass_kernel_traits): the finest
 * publication geometry, for sizing `ready`. */
FUSE_API void fuse_qkv_cutlass_kernel_traits(const fuse_gemm_problem* problem, fuse_kernel_traits* out);
/* include/fuse/operators/primitives/a2a_gemm.h:86 (cutlass_kernel_traits). */
FUSE_API void fuse_cutlass_kernel_traits(fuse_kernel_traits* out);
/* include/fuse/operators/primitives/a2a_gemm.h:88-90. */
FUSE_API int64_t fuse_a2a_lhs_gemm_ready_elements(const fuse_gemm_problem* problem,
                                         const fuse_ulysses_route* route);
/* include/fuse/operators/primitives/gemm_a2a.h:76-78 and a2a_gemm.h:92-94: the communication-CTA
 * budget the host plan chooses when the operator runs with communication CTAs.
 *
 * Auto.  Every operator accepts num_comm_ctas == 0 (the reference's "Auto",
 * csrc/operators/sm103/detail/autotune.cuh:109-203): the host planner scores the candidates from an
 * offline B200 calibration of compute and copy rates (fuse_b200/csrc/calibration_b200.h, written by
 * `python -m fuse_b200.calibrate`) and takes the smallest makespan max(compute, transfer).  On B200
 * that is the epilogue push for the projections that route their OUTPUT (no communication CTA at
 * all) and, for the operators that move their INPUT, the copy warp embedded in every compute CTA or
 * a communication budget.  An explicit num_comm_ctas > 0 is used exactly: that many communication
 * CTAs. */
FUSE_API int32_t fuse_recommended_gemm_a2a_comm_ctas(const fuse_gemm_problem* problem,
                                            const fuse_ulysses_route* route);
FUSE_API int32_t fuse_recommended_a2a_lhs_gemm_comm_ctas(const fuse_gemm_problem* problem,
                                                const fuse_ulysses_route* route);

/* The planner itself (no counterpart in the reference's public interface; its scorer is
 * csrc/operators/sm103/detail/autotune.cuh).  kind: 0 BF16 lhs pull, 1 MXFP8 lhs pull, 2 BF16
 * gradient push, 3 MXFP8 gradient pull, 4 / 5 QKV push from communication CTAs (BF16 / MXFP8),
 * 6 MoE dispatch.  flops / bytes / tiles describe one launch, group = SMs per tile (2: CTA pairs).
 * out = {comm_ctas, embedded (0/1), makespan_us, compute_us, transfer_us}.  Host only. */
FUSE_API int fuse_b200_plan(int32_t kind, double flops, double bytes, int64_t tiles, int32_t sm_count, int32_t group,
                            int32_t explicit_comm_ctas, int32_t embedded_allowed, double out[5]);
/* The same with the share of the bytes that crosses NVLink, (world - 1) / world for the all-to-all
 * routes (fuse_b200_plan plans for local copies, share 0). */
FUSE_API int fuse_b200_plan_remote(int32_t kind, double flops, double bytes, int64_t tiles, int32_t sm_count,
                                   int32_t group, int32_t explicit_comm_ctas, int32_t embedded_allowed,
                                   double remote_share, double out[5]);

/* ---------------------------------------------------------------------------------------------
 * Backward (BF16).  include/fuse/operators/ulysses/{backward_common,qkv_backward,oproj_backward}.h
 * ------------------------------------------------------------------------------------------- */
/* backward_common.h:12-15 */
enum { FUSE_WEIGHT_GRADIENT_IMMEDIATE = 0, FUSE_WEIGHT_GRADIENT_DEFERRED = 1 };
/* backward_common.h:20-28 (BackwardGemmPolicy): 0 auto, 1..5 M128 x N{64,128,160,192,256}, 6 N64 cluster. */
/* backward_common.h:33-37 (BackwardGemmTuning). */
typedef struct fuse_backward_gemm_tuning {
  int32_t epilogue_n;
  int32_t max_swizzle_size;
  uint8_t along_m;
} fuse_backward_gemm_tuning;

/* qkv_backward.h:24-49 (QkvBackwardDataParams): grad_q/k/v are this rank's planar gradients
 * [B*S_global, local_heads*head_dim]; peer_dqkv_staging[r] is rank r's packed [M, (q+2kv)*d]
 * staging, peer_ready[r] its fuse_qkv_backward_ready_elements() flags, weight the stored
 * forward weight [QKV, H], grad_input dX [M, H]. */
typedef struct fuse_qkv_backward_data_params {
  const fuse_bf16* grad_q;
  const fuse_bf16* grad_k;
  const fuse_bf16* grad_v;
  fuse_bf16* peer_dqkv_staging[FUSE_MAX_WORLD_SIZE];
  uint32_t* peer_ready[FUSE_MAX_WORLD_SIZE];
  uint32_t* peer_done_epoch[FUSE_MAX_WORLD_SIZE];
  const fuse_bf16* weight;
  fuse_bf16* grad_input;
  int32_t local_tokens, hidden, batch, q_heads, kv_heads, head_dim, world_size, rank, num_comm_ctas;
  int32_t gemm_policy;
  fuse_backward_gemm_tuning gemm_tuning;
  uint32_t epoch;
  uint8_t causal_load_balanced;
  float alpha;
} fuse_qkv_backward_data_params;

/* qkv_backward.h:62-73 (QkvBackwardWeightParams): dW[QKV,H] = alpha dQKV^T X + beta dW. */
typedef struct fuse_qkv_backward_weight_params {
  const fuse_bf16* dqkv_staging;
  const fuse_bf16* saved_input;
  fuse_bf16* grad_weight;
  int32_t local_tokens, hidden, q_heads, kv_heads, head_dim;
  float alpha, beta;
} fuse_qkv_backward_weight_params;

/* qkv_backward.h:75-79 (QkvBackwardParams). */
typedef struct fuse_qkv_backward_params {
  fuse_qkv_backward_data_params data;
  fuse_qkv_backward_weight_params weight;
  int32_t weight_mode;
} fuse_qkv_backward_params;

/* oproj_backward.h:21-43 (OprojBackwardDataParams): dA[M,A] = alpha dY[M,H] Wo[H,A] into
 * local_grad_attention, routed to peer_grad_attention[r] = rank r's [B*S_global, local_heads*d]. */
typedef struct fuse_oproj_backward_data_params {
  const fuse_bf16* grad_output;
  const fuse_bf16* weight;
  fuse_bf16* local_grad_attention;
  fuse_bf16* peer_grad_attention[FUSE_MAX_WORLD_SIZE];
  uint32_t* peer_done_epoch[FUSE_MAX_WORLD_SIZE];
  uint32_t* ready;
  int32_t local_tokens, hidden, batch, q_heads, head_dim, world_size, rank, num_comm_ctas;
  int32_t gemm_policy;
  fuse_backward_gemm_tuning gemm_tuning;
  uint32_t epoch;
  uint8_t causal_load_balanced;
  float alpha;
} fuse_oproj_backward_data_params;

/* oproj_backward.h:54-64 (OprojBackwardWeightParams): dWo[H,A] = alpha dY^T A + beta dWo. */
typedef struct fuse_oproj_backward_weight_params {
  const fuse_bf16* grad_output;
  const fuse_bf16* saved_attention;
  fuse_bf16* grad_weight;
  int32_t local_tokens, hidden, q_heads, head_dim;
  float alpha, beta;
} fuse_oproj_backward_weight_params;

/* oproj_backward.h:66-70 (OprojBackwardParams). */
typedef struct fuse_oproj_backward_params {
  fuse_oproj_backward_data_params data;
  fuse_oproj_backward_weight_params weight;
  int32_t weight_mode;
} fuse_oproj_backward_params;

/* qkv_backward.h:145-167 / csrc/operators/sm103/api/backward.cuh:304-329. */
FUSE_API int fuse_launch_qkv_backward_data(const fuse_qkv_backward_data_params* params, fuse_stream stream);
FUSE_API int fuse_launch_qkv_backward_data_ex(const fuse_qkv_backward_data_params* params,
                                     const fuse_b200_options* options, fuse_stream stream);
FUSE_API int fuse_launch_qkv_backward_weight(const fuse_qkv_backward_weight_params* params, fuse_stream stream);
FUSE_API int fuse_launch_qkv_backward(const fuse_qkv_backward_params* params, fuse_stream stream);
/* oproj_backward.h:131-149. */
FUSE_API int fuse_launch_oproj_backward_data(const fuse_oproj_backward_data_params* params, fuse_stream stream);
FUSE_API int fuse_launch_oproj_backward_data_ex(const fuse_oproj_backward_data_params* params,
                                       const fuse_b200_options* options, fuse_stream stream);
FUSE_API int fuse_launch_oproj_backward_weight(const fuse_oproj_backward_weight_params* params, fuse_stream stream);
FUSE_API int fuse_launch_oproj_backward(const fuse_oproj_backward_params* params, fuse_stream stream);
/* api/backward.cuh:294-303. */
FUSE_API int64_t fuse_qkv_backward_ready_elements(const fuse_qkv_backward_data_params* params);
FUSE_API int64_t fuse_oproj_backward_ready_elements(const fuse_oproj_backward_data_params* params);
/* api/backward.cuh:270-271. */
FUSE_API int32_t fuse_recommended_qkv_backward_comm_ctas(const fuse_qkv_backward_data_params* params);
FUSE_API int32_t fuse_recommended_oproj_backward_comm_ctas(const fuse_oproj_backward_data_params* params);

/* ---------------------------------------------------------------------------------------------
 * MXFP8 forward.  include/fuse/operators/primitives/{gemm_a2a_mxfp8,a2a_gemm_mxfp8}.h
 * ------------------------------------------------------------------------------------------- */
/* include/fuse/types.h:22-26 (Mxfp8WeightPreparation). */
enum { FUSE_MXFP8_PREP_COMM_CTAS = 0, FUSE_MXFP8_PREP_ALL_CTAS = 1, FUSE_MXFP8_PREP_COMM_WARPS = 2 };
/* include/fuse/types.h:31-35 (Mxfp8Activation): packed row-major E4M3 [rows, K] + native K32
 * scale storage (512-byte atoms of 128 rows x 4 K-blocks, K atoms before row atoms, rows padded
 * to 128). */
typedef struct fuse_mxfp8_activation {
  const uint8_t* data;
  const uint8_t* scales;
  size_t data_bytes, scale_bytes;
} fuse_mxfp8_activation;
/* include/fuse/operators/semantics/attention_postprocess.h:19-27; must stay disabled (NULL). */
typedef struct fuse_qkv_postprocess {
  const fuse_bf16 *q_gamma, *k_gamma, *cos, *sin;
  float epsilon;
} fuse_qkv_postprocess;
/* gemm_a2a_mxfp8.h:23-39 (Mxfp8GemmA2AParams): prequantised activation, BF16 master weight in
 * projection.rhs_nt quantised inside the kernel on every call, BF16 routed output.
 * projection.lhs is unused.  workspace: fuse_gemm_a2a_mxfp8_workspace_size() bytes, 256-byte
 * aligned, device-local, private to the call. */
typedef struct fuse_mxfp8_gemm_a2a_params {
  fuse_gemm_a2a_params projection;
  void* workspace;
  size_t workspace_bytes;
  fuse_mxfp8_activation activation;
  int32_t weight_preparation;
  int32_t epilogue_n;
  fuse_qkv_postprocess postprocess;
} fuse_mxfp8_gemm_a2a_params;

/* gemm_a2a_mxfp8.h:50-58 / csrc/operators/sm103/api/forward_mxfp8.cuh:553-602. */
FUSE_API int fuse_gemm_a2a_mxfp8_activation_size(const fuse_gemm_problem* problem, size_t* data_bytes,
                                        size_t* scale_bytes);
FUSE_API int fuse_quantize_gemm_a2a_mxfp8_activation(const fuse_gemm_problem* problem, const fuse_bf16* source,
                                            const fuse_mxfp8_activation* output, fuse_stream stream);
FUSE_API int fuse_gemm_a2a_mxfp8_workspace_size(const fuse_gemm_problem* problem, size_t* bytes);
FUSE_API int fuse_launch_gemm_a2a_mxfp8_cutlass(const fuse_mxfp8_gemm_a2a_params* params, fuse_stream stream);
FUSE_API int fuse_launch_gemm_a2a_mxfp8_cutlass_ex(const fuse_mxfp8_gemm_a2a_params* params,
                                          const fuse_b200_options* options, fuse_stream stream);
/* gemm_a2a_mxfp8.h:77-80: weight preparation alone, then GEMM + route on the prepared weight. */
FUSE_API int fuse_prepare_gemm_a2a_mxfp8(const fuse_mxfp8_gemm_a2a_params* params, fuse_stream stream);
FUSE_API int fuse_launch_gemm_a2a_mxfp8_prequantized(const fuse_mxfp8_gemm_a2a_params* params, fuse_stream stream);
FUSE_API int fuse_launch_gemm_a2a_mxfp8_prequantized_ex(const fuse_mxfp8_gemm_a2a_params* params,
                                               const fuse_b200_options* options, fuse_stream stream);
/* gemm_a2a_mxfp8.h:93-94: the block-scaled GEMM alone on SMs - num_comm_ctas CTAs, prepared
 * weight, no quantisation and no communication. */
FUSE_API int fuse_launch_gemm_a2a_mxfp8_compute_reference(const fuse_mxfp8_gemm_a2a_params* params, fuse_stream stream);
/* No counterpart in the reference.  The MXFP8 QKV operator for callers that cannot supply
 * scratch memory -- code inside a stream capture or a latency-critical loop, where cudaMalloc is
 * illegal or stalls the device, and plug-ins whose host owns the allocator.  Same operator and
 * result as fuse_launch_gemm_a2a_mxfp8_cutlass, but params->workspace and workspace_bytes are
 * ignored: the quantised weight goes to a fixed array of FUSE_B200_STATIC_SCRATCH_BYTES inside
 * the library image (held by every GPU that loads the library, until exit).  The call allocates
 * and frees nothing.  A weight whose scratch (N*K bytes plus N*K/32 scale bytes, each rounded
 * up to 256) exceeds the array is rejected with cudaErrorInvalidValue and one line on stderr.
 * The first call on each device looks the array's device address up; make that call before
 * starting a stream capture.  All calls share the array and it keeps the previous call's
 * contents; nothing in it has to start at zero (each call rewrites every byte it later reads),
 * but two calls that overlap on the GPU race on it: keep them on one stream or order them. */
#define FUSE_B200_STATIC_SCRATCH_BYTES (8u << 20)
FUSE_API int fuse_b200_launch_gemm_a2a_mxfp8_static(const fuse_mxfp8_gemm_a2a_params* params, fuse_stream stream);

/* csrc/operators/sm103/detail/quantization.cuh:281-304,350-450: the standalone quantisers.
 * Row-major BF16 [rows, k] -> E4M3 [rows, k]; BF16 [rows, cols] -> E4M3 [cols, rows] quantised
 * along the source row axis (rows % 32 == 0).  Scales in native storage of the OUTPUT operand,
 * fuse_b200_mxfp8_scale_bytes(output rows, output k) bytes. */
FUSE_API int fuse_b200_quantize_mxfp8(const fuse_bf16* source, int64_t row_stride, int32_t rows, int32_t k,
                             uint8_t* data, uint8_t* scales, fuse_stream stream);
FUSE_API int fuse_b200_quantize_mxfp8_transposed(const fuse_bf16* source, int64_t row_stride, int32_t rows,
                                        int32_t cols, uint8_t* data, uint8_t* scales, fuse_stream stream);
FUSE_API size_t fuse_b200_mxfp8_scale_bytes(int64_t rows, int64_t k);

/* include/fuse/operators/semantics/attention_postprocess.h:36-42; must stay disabled (NULL). */
typedef struct fuse_residual_rms_norm {
  const fuse_bf16* residual;
  const fuse_bf16* gamma;
  fuse_bf16* residual_output;
  float epsilon;
} fuse_residual_rms_norm;
/* a2a_gemm_mxfp8.h:25-46 (Mxfp8A2AGemmParams): activation[p] is rank p's prequantised head shard
 * [B*S_global, K/world] (E4M3 + native scales of THAT shape); the all-to-all copies the bytes and
 * re-homes the scale atoms into the local [M, K] storage inside `workspace`; the BF16 master
 * weight projection.rhs_nt is quantised in-kernel; BF16 output.  projection.peer_input,
 * input_staging and ready are unused. */
typedef struct fuse_mxfp8_a2a_gemm_params {
  fuse_a2a_gemm_params projection;
  fuse_mxfp8_activation activation[FUSE_MAX_WORLD_SIZE];
  void* workspace;
  size_t workspace_bytes;
  int32_t epilogue_n, m_window_tiles, n_group_tiles;
  fuse_residual_rms_norm postprocess;
  uint8_t overlap_postnorm;
  int32_t weight_preparation;
} fuse_mxfp8_a2a_gemm_params;
/* a2a_gemm_mxfp8.h:48-61 / csrc/operators/sm103/api/forward_mxfp8.cuh:705-924. */
FUSE_API int fuse_a2a_gemm_mxfp8_activation_size(const fuse_gemm_problem* problem, const fuse_ulysses_route* route,
                                        size_t* data_bytes, size_t* scale_bytes);
FUSE_API int fuse_a2a_gemm_mxfp8_workspace_size(const fuse_gemm_problem* problem, size_t* bytes);
/* a2a_gemm_mxfp8.h:51: the overload that takes the whole parameter record (same answer for
 * params->projection.gemm; C has no overloads, hence the suffix). */
FUSE_API int fuse_a2a_gemm_mxfp8_workspace_size_for_params(const fuse_mxfp8_a2a_gemm_params* params, size_t* bytes);
/* gemm_a2a_mxfp8.h:41 and a2a_gemm_mxfp8.h:52: tile geometry of the block-scaled kernels (for
 * sizing `ready`).  epilogue_n and overlap_postnorm select among the reference's kernel
 * instances; this library has one tile shape per operand type, so both are accepted and
 * ignored (values outside {32, 64} leave *out zeroed, as the reference returns {}). */
FUSE_API void fuse_mxfp8_qkv_cutlass_kernel_traits(int32_t epilogue_n, fuse_kernel_traits* out);
FUSE_API void fuse_mxfp8_oproj_cutlass_kernel_traits(int32_t epilogue_n, uint8_t overlap_postnorm,
                                                     fuse_kernel_traits* out);
FUSE_API int fuse_a2a_gemm_mxfp8_staging_view(const fuse_mxfp8_a2a_gemm_params* params, fuse_mxfp8_activation* activation);
FUSE_API int fuse_launch_a2a_gemm_mxfp8_cutlass(const fuse_mxfp8_a2a_gemm_params* params, fuse_stream stream);
FUSE_API int fuse_launch_a2a_gemm_mxfp8_cutlass_ex(const fuse_mxfp8_a2a_gemm_params* params,
                                          const fuse_b200_options* options, fuse_stream stream);

/* ---------------------------------------------------------------------------------------------
 * MoE dispatch -> expert FC1 grouped GEMM.  include/fuse/operators/primitives/grouped_gemm.h
 * ------------------------------------------------------------------------------------------- */
/* grouped_gemm.h:10-12 (GroupedTokenSource): where a routed row comes from. */
typedef struct fuse_grouped_token_source {
  int32_t rank, token, slot;
} fuse_grouped_token_source;
/* grouped_gemm.h:17-53 (GroupedGemmPolicy).  This implementation honours num_comm_ctas,
 * num_compute_ctas and tile_n (128 or 256); mma_sm_count 1, or 2 = CTA pairs on
 * 256 x 256 tiles (needs tile_n 256 and an even num_comm_ctas); swap_ab must be false.
 * num_comm_ctas == 0 is Auto: on CTA pairs the dispatch then has no communication CTA (one thread
 * of every compute CTA pulls), on one-CTA tiles the host planner picks the budget for slabs half
 * full and the share of the rows that is remote. */
typedef struct fuse_grouped_gemm_policy {
  int32_t num_comm_ctas, num_compute_ctas, swizzle;
  uint8_t along_n;
  int32_t tile_n, tile_k;
  int32_t mma_sm_count;
  int32_t dispatch_copy;
  uint8_t balance_dispatch_tail, swap_ab, trim_swap_tokens;
  int32_t scheduler;
} fuse_grouped_gemm_policy;
/* grouped_gemm.h:62-85 (Bf16GroupedGemmParams): device arrays with one pointer per LOCAL expert
 * (lhs[e] / output[e] slabs of expert_row_capacity rows, weight_nt[e] = W_e[N,K]); row_offsets
 * (device, experts+1) and source (device) may change between launches; peer_started / peer_done
 * are caller-owned peer-visible arrays of world_size flags, zeroed once. */
typedef struct fuse_bf16_grouped_gemm_params {
  fuse_bf16* const* lhs;
  const fuse_bf16* const* weight_nt;
  fuse_bf16* const* output;
  const int64_t* row_offsets;
  const fuse_grouped_token_source* source;
  const fuse_bf16* peer_input[FUSE_MAX_WORLD_SIZE];
  fuse_bf16* peer_output[FUSE_MAX_WORLD_SIZE];
  uint32_t* peer_started[FUSE_MAX_WORLD_SIZE];
  uint32_t* peer_done[FUSE_MAX_WORLD_SIZE];
  int32_t experts, n, k;
  int32_t expert_row_capacity;
  int32_t rank, world_size, topk;
  fuse_grouped_gemm_policy policy;
  int32_t dispatch_buffer_rows;
} fuse_bf16_grouped_gemm_params;
/* grouped_gemm.h:87-98: opaque plan owning private device metadata; create outside stream
 * capture (it allocates and synchronises), launch allocates nothing and reads the row counts on
 * the device, destroy after the last use has finished. */
typedef struct fuse_bf16_grouped_gemm_plan fuse_bf16_grouped_gemm_plan;
FUSE_API int fuse_create_bf16_a2a_grouped_gemm(const fuse_bf16_grouped_gemm_params* params,
                                      fuse_bf16_grouped_gemm_plan** plan);
/* grouped_gemm.h:97-98 (create_bf16_grouped_gemm_a2a): the combine direction.  lhs[e] is local and
 * complete at launch; D_e = lhs_e W_e^T is written to output[e] and every routed row r to
 * peer_output[source.rank][(source.token * topk + source.slot) * n ...] (no weighting, no top-k
 * reduction: csrc/operators/sm103/detail/grouped/gemm_a2a.cuh:15-93).  Launched and destroyed
 * through the same two calls as the dispatch plan; every CTA computes (the epilogue scatters), so
 * policy.num_comm_ctas is only validated. */
FUSE_API int fuse_create_bf16_grouped_gemm_a2a(const fuse_bf16_grouped_gemm_params* params,
                                      fuse_bf16_grouped_gemm_plan** plan);
FUSE_API int fuse_launch_bf16_grouped_gemm(fuse_bf16_grouped_gemm_plan* plan, fuse_stream stream);
FUSE_API int fuse_launch_bf16_grouped_gemm_ex(fuse_bf16_grouped_gemm_plan* plan, const fuse_b200_options* options,
                                     fuse_stream stream);
FUSE_API int fuse_destroy_bf16_grouped_gemm(fuse_bf16_grouped_gemm_plan* plan);

/* ---------------------------------------------------------------------------------------------
 * MXFP8 backward.  include/fuse/operators/ulysses/qkv_backward.h:196-283, oproj_backward.h:186-240
 * ------------------------------------------------------------------------------------------- */
/* qkv_backward.h:199-204 (Mxfp8QkvBackwardInput): one source rank's prequantised planar dQ, dK,
 * dV (each with native scales of its OWN planar width) and their BF16 masters. */
typedef struct fuse_mxfp8_qkv_backward_input {
  fuse_mxfp8_activation grad_q, grad_k, grad_v;
  const fuse_bf16 *master_q, *master_k, *master_v;
} fuse_mxfp8_qkv_backward_input;
/* qkv_backward.h:219-224 (Mxfp8QkvBackwardDataParams): only projection.peer_dqkv_staging[rank]
 * and peer_ready[rank] are used locally; peer_input supplies the reads; head_dim must be 128. */
typedef struct fuse_mxfp8_qkv_backward_data_params {
  fuse_qkv_backward_data_params projection;
  fuse_mxfp8_qkv_backward_input peer_input[FUSE_MAX_WORLD_SIZE];
  void* workspace;
  size_t workspace_bytes;
} fuse_mxfp8_qkv_backward_data_params;
/* qkv_backward.h:241-246 (Mxfp8QkvBackwardWeightParams). */
typedef struct fuse_mxfp8_qkv_backward_weight_params {
  fuse_qkv_backward_weight_params projection;
  fuse_backward_gemm_tuning gemm_tuning;
  void* workspace;
  size_t workspace_bytes;
} fuse_mxfp8_qkv_backward_weight_params;
typedef struct fuse_mxfp8_qkv_backward_params {
  fuse_mxfp8_qkv_backward_data_params data;
  fuse_mxfp8_qkv_backward_weight_params weight;
  int32_t weight_mode;
} fuse_mxfp8_qkv_backward_params;
/* oproj_backward.h:191-196 (Mxfp8OprojBackwardDataParams): grad_output is the prequantised dY. */
typedef struct fuse_mxfp8_oproj_backward_data_params {
  fuse_oproj_backward_data_params projection;
  fuse_mxfp8_activation grad_output;
  void* workspace;
  size_t workspace_bytes;
} fuse_mxfp8_oproj_backward_data_params;
/* oproj_backward.h:205-210 (Mxfp8OprojBackwardWeightParams). */
typedef struct fuse_mxfp8_oproj_backward_weight_params {
  fuse_oproj_backward_weight_params projection;
  fuse_backward_gemm_tuning gemm_tuning;
  void* workspace;
  size_t workspace_bytes;
} fuse_mxfp8_oproj_backward_weight_params;
typedef struct fuse_mxfp8_oproj_backward_params {
  fuse_mxfp8_oproj_backward_data_params data;
  fuse_mxfp8_oproj_backward_weight_params weight;
  int32_t weight_mode;
} fuse_mxfp8_oproj_backward_params;
/* qkv_backward.h:252-280 / csrc/operators/sm103/api/backward_mxfp8.cuh:404-497. */
FUSE_API int fuse_qkv_backward_mxfp8_data_workspace_size(const fuse_qkv_backward_data_params* params, size_t* bytes);
FUSE_API int fuse_qkv_backward_mxfp8_weight_workspace_size(const fuse_qkv_backward_weight_params* params, size_t* bytes);
FUSE_API int fuse_launch_qkv_backward_mxfp8_data(const fuse_mxfp8_qkv_backward_data_params* params, fuse_stream stream);
FUSE_API int fuse_launch_qkv_backward_mxfp8_data_ex(const fuse_mxfp8_qkv_backward_data_params* params,
                                           const fuse_b200_options* options, fuse_stream stream);
FUSE_API int fuse_launch_qkv_backward_mxfp8_weight(const fuse_mxfp8_qkv_backward_weight_params* params, fuse_stream stream);
FUSE_API int fuse_launch_qkv_backward_mxfp8(const fuse_mxfp8_qkv_backward_params* params, fuse_stream stream);
/* oproj_backward.h:222-237. */
FUSE_API int fuse_oproj_backward_mxfp8_data_workspace_size(const fuse_oproj_backward_data_params* params, size_t* bytes);
FUSE_API int fuse_oproj_backward_mxfp8_weight_workspace_size(const fuse_oproj_backward_weight_params* params, size_t* bytes);
FUSE_API int fuse_launch_oproj_backward_mxfp8_data(const fuse_mxfp8_oproj_backward_data_params* params, fuse_stream stream);
FUSE_API int fuse_launch_oproj_backward_mxfp8_data_ex(const fuse_mxfp8_oproj_backward_data_params* params,
                                             const fuse_b200_options* options, fuse_stream stream);
FUSE_API int fuse_launch_oproj_backward_mxfp8_weight(const fuse_mxfp8_oproj_backward_weight_params* params, fuse_stream stream);
FUSE_API int fuse_launch_oproj_backward_mxfp8(const fuse_mxfp8_oproj_backward_params* params, fuse_stream stream);

/* The static tile order shared by compute and communication CTAs: linear index -> (m, n) tile
 * for a grid of m_tiles x n_tiles, swizzle in {1,2,4,8}, along_n = 0 (index runs down M inside
 * bands of `swizzle` N tiles) or 1 (transpose).  Same knobs as the reference scheduler
 * (csrc/operators/sm103/detail/persistent_gemm.cuh:27-182); returns 0, or 1 for bad input. */
FUSE_API int fuse_b200_tile_order_decode(int32_t m_tiles, int32_t n_tiles, int32_t swizzle, int32_t along_n,
                                int64_t linear, int32_t* m, int32_t* n);
/* benchmarks/sm103/fused_bf16.cu:196-206: swizzle actually used for a cap and a tile grid. */
FUSE_API int32_t fuse_b200_select_swizzle(int32_t max_swizzle, int32_t m_tiles, int32_t n_tiles);

/* Fills `count` BF16 values on the device from a seed: uniform in [-scale, scale) with the
 * reference harness's Philox4x32-10 element mapping and word->value map
 * (benchmarks/sm103/fused_inputs.cuh:22-29,117-141), or N(0, scale^2) when `normal` != 0. */
FUSE_API int fuse_b200_generate_bf16(fuse_bf16* out, uint64_t count, uint64_t seed, float scale, int normal,
                            fuse_stream stream);

/* Symmetric buffers for one-process-per-GPU ranks (harness helpers, not on the launch path;
 * the reference's harness does the same with cudaIpc*: benchmarks/sm103/fused_bf16.cu:1080-1139).
 * alloc: zero-filled cudaMalloc + 64-byte IPC handle; open: map a peer's handle (peer access is
 * enabled lazily); close / free undo them. */
FUSE_API int fuse_b200_symmetric_alloc(size_t bytes, void** ptr, unsigned char handle[64]);
FUSE_API int fuse_b200_symmetric_open(const unsigned char handle[64], void** ptr);
FUSE_API int fuse_b200_symmetric_close(void* ptr);
FUSE_API int fuse_b200_symmetric_free(void* ptr);

/* Device status record of the current device (16 words; see csrc/sync.cuh).  word 0 != 0
 * means a device-side wait gave up; `clear` resets the record.  No reference counterpart. */
FUSE_API int fuse_b200_read_status(uint32_t out[16], int clear);
/* sizeof of the ABI records as compiled: 0 gemm_problem, 1 ulysses_route, 2 gemm_a2a_params,
 * 3 a2a_gemm_params, 4 kernel_traits, 5 options, 6 qkv_backward_data_params,
 * 7 qkv_backward_weight_params, 8 qkv_backward_params, 9 oproj_backward_data_params,
 * 10 oproj_backward_weight_params, 11 oproj_backward_params, 12 mxfp8_activation,
 * 13 mxfp8_gemm_a2a_params, 14 mxfp8_a2a_gemm_params, 15 grouped_gemm_policy,
 * 16 bf16_grouped_gemm_params, 17 mxfp8_qkv_backward_data_params, 18 mxfp8_qkv_backward_weight_params,
 * 19 mxfp8_qkv_backward_params, 20 mxfp8_oproj_backward_data_params, 21 mxfp8_oproj_backward_weight_params,
 * 22 mxfp8_oproj_backward_params.  -1 for unknown ids. */
FUSE_API int fuse_b200_abi_sizeof(int record);
/* Number of kernels this library has launched in this process (all entry points). */
FUSE_API uint64_t fuse_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* FUSE_B200_H_ */
