/*
 * elsa_b200 -- C ABI of the B200-native two-pass monoid attention.
 *
 * Every entry point takes raw device pointers, explicit sizes and a CUDA stream handle
 * (a cudaStream_t passed as void*; NULL = the legacy default stream), launches on that
 * stream and returns immediately with 0 or one of the ELSA_ERR_* codes.  Nothing here
 * allocates or frees device memory, synchronises the device or throws: buffers belong to
 * the caller and are borrowed for the duration of the stream-ordered launch.  (Exceptions, both stated at
 * their declarations: elsa_twopass_forward_static keeps its scratch inside the library image, and the first
 * call of the process that needs the device status word makes one small pinned-host allocation.)
 *
 * The citations name the interface of the reference project (ming053l/ELSA, paths relative
 * to its root) that each entry point replaces.
 *
 * Tensor conventions
 *   q, k, v, out, dout, dq, dk, dv ... [B*H, N, D] contiguous, element type `dtype`
 *   row_m, row_z, row_d, row_lse ..... [B*H, N] fp32; row_m and row_lse in the log2 domain
 *   bias ............................. fp32, addressed as
 *                                      bias[b*stride_b + h*stride_h + q*stride_q + k*stride_k]
 *                                      (a zero stride broadcasts), NULL = no bias
 *   summaries ........................ m, z: [P, B*H, q_len] fp32; s: [P, B*H, q_len, D] in
 *                                      `summary_dtype`; P = number of K partitions; the rows
 *                                      are the queries q_start .. q_start+q_len-1
 */
#ifndef ELSA_B200_H_
#define ELSA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ELSA_B200_ABI_VERSION 2

enum elsa_dtype { ELSA_F32 = 0, ELSA_F16 = 1, ELSA_BF16 = 2 };

enum elsa_status {
  ELSA_OK = 0,
  ELSA_ERR_INVALID_ARGUMENT = 1, /* a size, pointer, dtype or alignment the ABI does not accept */
  ELSA_ERR_UNSUPPORTED = 2,      /* valid request that no kernel in this build covers */
  ELSA_ERR_CUDA = 3,             /* a CUDA runtime/driver call failed; see elsa_last_cuda_error */
  ELSA_ERR_WORKSPACE = 4,        /* workspace pointer missing, misaligned or too small */
  ELSA_ERR_DEVICE_TIMEOUT = 5    /* a bounded device-side wait gave up earlier (elsa_device_status is non-zero) */
};

/* flags for the forward / backward entry points */
#define ELSA_FLAG_FORCE_SIMT 1u   /* never take the tcgen05 kernels (debug / A-B checks) */
#define ELSA_FLAG_SCAN_STEPS 2u   /* causal: run the log-depth Hillis-Steele steps instead of the one-pass merge */
#define ELSA_FLAG_TREE_MERGE 4u   /* non-causal: run the Blelloch up-sweep levels instead of the one-pass merge */
#define ELSA_FLAG_FP32_FMA 16u     /* forward and backward, fp32 inputs: stay on the FP32-FMA kernels instead of the
                                     tensor-core kernels that work on two fp16 planes per operand (x * 2^e = h0 + h1,
                                     three cross products per fp32 product: the accuracy class of 3xTF32; the planes
                                     cost the size of q, k, v in forward workspace and of q, dout, k, v in backward
                                     workspace) */
#define ELSA_FLAG_REF_ROUNDING 8u /* forward, fp16 / head dim 64 / no bias / not causal only: reproduce the rounding points of
                                     the reference's fp16 d=64 kernels (q * log2(e)/8 formed in fp16, scores unscaled:
                                     attention_parallel_scan.py:153-154,160) instead of the exact fp32 scale; the workspace
                                     grows by one fp16 copy of q (elsa_forward_workspace_bytes accounts for it) */

int elsa_abi_version(void);
const char* elsa_strerror(int status);
/* cudaError_t of the most recent failing CUDA call made by this library on the calling thread */
int elsa_last_cuda_error(void);
/* Status word of the CURRENT device, written by the bounded device-side waits of the tensor-core kernels:
 * 0 = no wait gave up; otherwise (1 << 8) | id of the barrier.  The word lives in mapped pinned host memory
 * (one small host allocation, made by the first call of the process that needs it: make that call outside any
 * stream capture), so this read costs nothing and synchronises nothing; it describes the kernels that have
 * finished so far -- synchronise the stream first for a definite answer.  While the word is non-zero every entry
 * point that would launch a tensor-core kernel returns ELSA_ERR_DEVICE_TIMEOUT instead (the results of the
 * call whose wait gave up are undefined); clear != 0 resets it.  Returns -1 when the word cannot be set up. */
int elsa_device_status(int clear);
/* Test hook for the status path: one CTA waits on an mbarrier that nothing ever arrives at, gives up after
 * limit_ns nanoseconds, records (1 << 8) | 99 in the status word and returns normally.  It faults nothing and
 * leaves the context usable.  No counterpart in the reference. */
int elsa_debug_wait_timeout(uint64_t limit_ns, void* stream);
/* Measurement helper for benchmarks (no counterpart in the reference, on no product path): `blocks` CTAs of 256
 * threads each run `iters` rounds of 16 independent register-resident FP32 FMAs (scalar, or packed f32x2 when
 * packed != 0); the work is blocks * 256 * iters * 32 FLOP.  Timed by the caller with events, it gives the
 * FP32-FMA rate that bounds the fp32 kernels.  sink: one float of device memory. */
int elsa_debug_fma_rate(float* sink, int blocks, int64_t iters, int packed, void* stream);
/* number of kernels this library has launched in this process so far (all threads, all streams) */
int64_t elsa_kernel_launches(void);
/* 1 when the tcgen05 (tensor-core) kernels cover this problem, 0 when the FP32-FMA kernels run.  Covered, from 512
 * tokens on (see elsa_uses_tensor_cores_for for shorter sequences), with or without a bias (and its gradient): fp16 and bf16 inputs with a head dim that is a multiple of 8 up
 * to 128; fp32 inputs with a head dim that is a multiple of 8 up to 64.  Also covered: fp16 and bf16 sequences of at
 * most 64 tokens (attention windows) with a head dim that is a multiple of 8 up to 64, causal or not, with or without a bias
 * (and its gradient), two sequences per 128-row tile. */
int elsa_uses_tensor_cores(int dtype, int head_dim, int n_ctx, int has_bias, int is_causal, int backward);
/* The same question for a given batch size.  Sequences of 65 to 511 tokens also run on the tensor-core kernels when the
 * problem has at least 4096 rows in total (batch * heads * n_ctx): from there on 128-row tiles fill the machine; the
 * fp16 / bf16 backward runs there from 65 tokens on at every batch size.
 * elsa_uses_tensor_cores answers for batch = heads = 1, i.e. what holds whatever the batch size. */
int elsa_uses_tensor_cores_for(int dtype, int head_dim, int n_ctx, int has_bias, int is_causal, int backward, int batch,
                               int heads);

/* ---------------------------------------------------------------------------------------
 * Phase 1: per-K-partition (m, z, s) fold.
 * Replaces the Triton launches `_phase1_summary_kernel` (src/elsa_twopass_clean/attention.py:22-106),
 * `_phase1_d64_{fp16,fp32}_nomask_kernel` (attention_parallel_scan.py:123-224) and
 * `_phase1_d64_tiled_{fp16,fp32}_nomask_kernel` (attention_parallel_scan.py:227-372) together
 * with their grid set-up (attention_parallel_scan.py:486-563, 680-708, 881-909).
 * Partition p covers keys [p*part_width, min(N, (p+1)*part_width)).  Keys >= N never contribute
 * (the NEEDS_MASK rule, attention_parallel_scan.py:472); a partition with no valid key for a row
 * yields the identity (-inf, 0, 0).
 * ------------------------------------------------------------------------------------- */
int elsa_phase1_fold(const void* q, const void* k, const void* v,
                     const float* bias, int64_t bias_stride_b, int64_t bias_stride_h,
                     int64_t bias_stride_q, int64_t bias_stride_k,
                     float* m_buf, float* z_buf, void* s_buf,
                     int dtype, int summary_dtype,
                     int batch, int heads, int n_ctx, int head_dim,
                     int q_start, int q_len, int part_width, int n_parts,
                     int is_causal, unsigned flags, void* stream);

/* Phase 1 of ONE SEQUENCE SHARD: q holds all n_ctx query rows, k / v hold n_keys rows per
 * (batch*head) whose first row has global index key_offset (needed only by the causal mask).
 * Summaries cover all n_ctx rows: m, z [n_parts, B*H, n_ctx]; s [n_parts, B*H, n_ctx, D].
 * No counterpart in the reference, which is single-GPU: this is the per-GPU half of the
 * sequence-parallel forward; the partition layout is the reference's (attention.py:102-106). */
int elsa_phase1_fold_shard(const void* q, const void* k, const void* v,
                           float* m_buf, float* z_buf, void* s_buf,
                           int dtype, int summary_dtype, int batch, int heads, int n_ctx, int head_dim,
                           int n_keys, int key_offset, int part_width, int n_parts,
                           int is_causal, unsigned flags, void* stream);

/* The same with a workspace (elsa_phase1_fold_shard_workspace_bytes; 0 when none is needed): fp32 shards with head dim 64
 * then run on the tensor cores, the workspace holding the 16-bit planes of q, k_shard and v_shard.  No counterpart
 * in the reference. */
int64_t elsa_phase1_fold_shard_workspace_bytes(int dtype, int batch, int heads, int n_ctx, int head_dim, int n_keys,
                                               unsigned flags);
int elsa_phase1_fold_shard_ws(const void* q, const void* k, const void* v,
                              float* m_buf, float* z_buf, void* s_buf, void* workspace, int64_t workspace_bytes,
                              int dtype, int summary_dtype, int batch, int heads, int n_ctx, int head_dim,
                              int n_keys, int key_offset, int part_width, int n_parts,
                              int is_causal, unsigned flags, void* stream);

/* Merge the partitions of each row into ONE un-normalised fp32 summary (m_out, z_out [B*H, q_len],
 * s_out [B*H, q_len, D]): what a shard hands to the cross-GPU merge.  Same arithmetic as
 * elsa_merge_final (cuda/paper_scan_d64_kernel.cu:39-70) without the final division. */
int elsa_merge_partial(const float* m_buf, const float* z_buf, const void* s_buf,
                       float* s_out, float* m_out, float* z_out,
                       int summary_dtype, int n_parts, int bh, int q_len, int head_dim, void* stream);

/* Cross-GPU merge of sequence shards, the two local passes around the collective.  The reference is
 * single-GPU and has no counterpart; the arithmetic is that of its phase-2 reduce (weights 2^(m - M), weighted
 * sums of z and s, out = S / Z: cuda/paper_scan_d64_kernel.cu:54-95) with the partitions living on different GPUs.
 * Sequence: all_reduce(MAX) of m -> m_all; elsa_shard_pack; reduce_scatter(SUM) of `packed` (world equal chunks);
 * elsa_shard_finalize on the chunk this rank received.  n_ctx must divide by world; head_dim by 4.
 *   pack      m, z [B*H, N], s [B*H, N, D] fp32: this shard's merged un-normalised summary (elsa_merge_partial).
 *             packed: world chunks of elsa_shard_chunk_elems floats; chunk r covers rows [r*N/world, (r+1)*N/world)
 *             of every (batch*head): s*w as [B*H, N/world, D], then z*w as [B*H, N/world]; w = z > 0 ? 2^(m - m_all) : 0.
 *   finalize  chunk: the summed chunk `rank`; out [B*H, N/world, D] in out_dtype = S / Z (0 where Z == 0);
 *             row_m = Z > 0 ? m_all : -inf, row_z = Z, both [B*H, N/world].
 * world = 1 is the all_reduce form: one chunk with all rows, summed on every rank. */
int64_t elsa_shard_chunk_elems(int bh, int n_ctx, int head_dim, int world);
int elsa_shard_pack(const float* m, const float* z, const float* s, const float* m_all, float* packed,
                    int bh, int n_ctx, int head_dim, int world, void* stream);
int elsa_shard_finalize(const float* chunk, const float* m_all, void* out, float* row_m, float* row_z,
                        int out_dtype, int bh, int n_ctx, int head_dim, int world, int rank, void* stream);

/* ---------------------------------------------------------------------------------------
 * Phase 2, one pass: merge all partition summaries of each row, out = s / z, optional state.
 * Replaces pybind `final_reduce(m, z, s, out, row_m, row_z, q_start, n_ctx, k_blocks, q_blocks,
 * bh, block_m, store_state)` (src/elsa_twopass_clean/cuda/paper_scan_d64.cpp:3-20, kernel
 * cuda/paper_scan_d64_kernel.cu:9-96), generalised to any D <= 128 and to bf16.
 * out is [B*H, N, D] in `out_dtype`; rows q_start .. q_start+q_len-1 are written.
 * ------------------------------------------------------------------------------------- */
int elsa_merge_final(const float* m_buf, const float* z_buf, const void* s_buf,
                     void* out, float* row_m, float* row_z,
                     int summary_dtype, int out_dtype,
                     int n_parts, int bh, int q_start, int q_len, int n_ctx, int head_dim,
                     int store_state, void* stream);

/* One Hillis-Steele step out[p] = in[p-step] (+) in[p]; replaces `_summary_scan_step_kernel`
 * (attention_parallel_scan.py:13-64) and one iteration of the host loop at :713-733. */
int elsa_scan_step(const float* m_in, const float* z_in, const void* s_in,
                   float* m_out, float* z_out, void* s_out,
                   int summary_dtype, int n_parts, int bh, int q_len, int head_dim,
                   int step, void* stream);

/* One Blelloch up-sweep level out[i] = in[2i] (+) in[2i+1] (odd tail merges with the identity);
 * replaces `_summary_blelloch_upsweep_kernel` (attention_parallel_scan.py:67-120) and one
 * iteration of the host loop at :914-935.  Writes ceil(n_in/2) partitions. */
int elsa_upsweep_level(const float* m_in, const float* z_in, const void* s_in,
                       float* m_out, float* z_out, void* s_out,
                       int summary_dtype, int n_in, int bh, int q_len, int head_dim, void* stream);

/* Inclusive prefix scan over the partitions in ONE read + ONE write pass (each row's P
 * summaries are folded left to right in registers).  Same result as running elsa_scan_step for
 * step = 1, 2, 4, ... (attention_parallel_scan.py:710-733) with 1/log2(P) of the HBM traffic.
 * The output buffers must not alias the inputs. */
int elsa_prefix_scan(const float* m_in, const float* z_in, const void* s_in,
                     float* m_out, float* z_out, void* s_out,
                     int summary_dtype, int n_parts, int bh, int q_len, int head_dim, void* stream);

/* out = s / z from partition `final_part`, optional state; replaces `_scan_last_to_out_kernel`
 * (attention_parallel_scan.py:375-415). */
int elsa_finalize(const float* m_buf, const float* z_buf, const void* s_buf,
                  void* out, float* row_m, float* row_z,
                  int summary_dtype, int out_dtype,
                  int final_part, int bh, int q_start, int q_len, int n_ctx, int head_dim,
                  int store_state, void* stream);

/* ---------------------------------------------------------------------------------------
 * Whole forward = host orchestration of both passes, one call.
 * Replaces `twopass_attention_paper_scan` and the three host drivers under it
 * (attention_parallel_scan.py:443-584, 587-759, 762-961, 964-1018).
 * part_width / q_chunk <= 0 let the library choose.  row_m / row_z may be NULL.
 * ------------------------------------------------------------------------------------- */
int64_t elsa_forward_workspace_bytes(int dtype, int summary_dtype, int batch, int heads, int n_ctx,
                                     int head_dim, int has_bias, int is_causal, int part_width,
                                     int q_chunk, unsigned flags);
int elsa_twopass_forward(const void* q, const void* k, const void* v,
                         const float* bias, int64_t bias_stride_b, int64_t bias_stride_h,
                         int64_t bias_stride_q, int64_t bias_stride_k,
                         void* out, float* row_m, float* row_z,
                         void* workspace, int64_t workspace_bytes,
                         int dtype, int summary_dtype,
                         int batch, int heads, int n_ctx, int head_dim,
                         int is_causal, int part_width, int q_chunk, unsigned flags, void* stream);
/* The same forward on strided [B, H, N, D] VIEWS: every tensor comes with three element strides {batch, head, row}
 * (the D axis contiguous), e.g. q, k, v read in place from a packed [B, N, 3, H, D] projection output
 * (strides {3*N*H*D, D, 3*H*D}) and out written as [B, N, H*D] (strides {N*H*D, D, H*D}).  This removes the
 * `.contiguous()` copies the reference's hooks make before the call and the transpose after it
 * (src/elsa_twopass_clean/timm_dropin.py:46-55, timm_dropin_bwd.py:68-73).  Every stride must be a multiple of 8
 * elements and every base pointer 16-byte aligned (ELSA_ERR_INVALID_ARGUMENT otherwise: copy first).
 * row_m / row_z stay [B*H, N] contiguous.  ELSA_FLAG_REF_ROUNDING is not available here (ELSA_ERR_UNSUPPORTED). */
int elsa_twopass_forward_strided(const void* q, const void* k, const void* v,
                                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                                 const float* bias, int64_t bias_stride_b, int64_t bias_stride_h,
                                 int64_t bias_stride_q, int64_t bias_stride_k,
                                 void* out, const int64_t* out_strides, float* row_m, float* row_z,
                                 void* workspace, int64_t workspace_bytes,
                                 int dtype, int summary_dtype,
                                 int batch, int heads, int n_ctx, int head_dim,
                                 int is_causal, int part_width, int q_chunk, unsigned flags, void* stream);
/* how the forward above splits the work: fills part_width, n_parts, q_chunk (all may be NULL) */
int elsa_forward_plan(int dtype, int summary_dtype, int batch, int heads, int n_ctx, int head_dim,
                      int has_bias, int is_causal, int part_width_in, int q_chunk_in, unsigned flags,
                      int* part_width, int* n_parts, int* q_chunk);

/* Forward for callers that cannot provide or allocate a workspace (no counterpart in the reference, whose
 * buffers are always PyTorch allocations).  Meant for hosts that bind this library through a bare FFI and own
 * no device allocator, and for serving loops whose device memory is fixed at start-up and whose request
 * path must not allocate: the partition summaries go to a 64 MiB array that is part of the library image
 * (elsa_static_scratch_bytes) instead of a caller workspace.  No bias, library-chosen partitions, summaries
 * in the input dtype, fp32 inputs on the FP32-FMA kernel (as with ELSA_FLAG_FP32_FMA); out / row_m / row_z as in
 * elsa_twopass_forward (row_m, row_z may both be NULL).
 *   - Query rows are processed in chunks whose summaries fit the array; only a problem for which not even one
 *     query tile (256 rows on the tensor-core path, 64 otherwise) of summaries fits returns ELSA_ERR_WORKSPACE,
 *     and then nothing is launched.
 *   - The array stays resident on every GPU that loads the library, until the process exits.
 *   - All calls on a device share the array: two calls that overlap on the GPU (different streams, or
 *     different host threads) race on it.  Calls on one stream are safe back to back; nothing in the array
 *     needs clearing between calls.
 *   - The first call on each device looks the array's device address up; make that first call outside any
 *     stream capture.
 *   - The call itself never allocates or frees device memory. */
int64_t elsa_static_scratch_bytes(void);
int elsa_twopass_forward_static(const void* q, const void* k, const void* v,
                                void* out, float* row_m, float* row_z,
                                int dtype, int batch, int heads, int n_ctx, int head_dim,
                                int is_causal, void* stream);

/* ---------------------------------------------------------------------------------------
 * Backward.
 * ------------------------------------------------------------------------------------- */
/* D = sum_d out*dout, LSE = m + log2(max(z, 1e-30)); replaces `_bwd_preprocess_kernel`
 * (src/elsa_twopass_clean/attention_bwd.py:188-224). */
int elsa_bwd_preprocess(const void* out, const void* dout, const float* row_m, const float* row_z,
                        float* row_d, float* row_lse, int dtype, int bh, int n_ctx, int head_dim,
                        void* stream);

/* Row statistics (m, z) recomputed from q, k (and bias); replaces `_row_stats_kernel`
 * (attention_bwd.py:227-306).  workspace: elsa_row_stats_workspace_bytes. */
int64_t elsa_row_stats_workspace_bytes(int dtype, int batch, int heads, int n_ctx, int head_dim,
                                       int has_bias, int is_causal);
int elsa_row_stats(const void* q, const void* k,
                   const float* bias, int64_t bias_stride_b, int64_t bias_stride_h,
                   int64_t bias_stride_q, int64_t bias_stride_k,
                   float* row_m, float* row_z, void* workspace, int64_t workspace_bytes,
                   int dtype, int batch, int heads, int n_ctx, int head_dim, int is_causal,
                   void* stream);

/* dQ, dK, dV (and, when dbias != NULL, the bias gradient accumulated in fp32) by exact
 * recompute from the saved forward state (out, row_m, row_z).  Replaces the launches of
 * `_bwd_preprocess_kernel`, `_bwd_dq_kernel`, `_bwd_dkdv_kernel` and `_dbias_dense_kernel`
 * (attention_bwd.py:188-224, 309-412, 415-527, 529-624) made by `twopass_attention_backward`
 * and `_dense_bias_backward` (attention_bwd.py:765-838, 939-970).
 * dbias is fp32, addressed with the dbias_stride_* like bias; where a stride is 0 the
 * contributions of that axis are summed (atomically).  The caller ALWAYS zeroes dbias before the call: besides
 * the sums, entries of pairs that the causal rule or the sequence length excludes are never written.
 * workspace: elsa_backward_workspace_bytes (row_d, row_lse; on the tensor-core path also the fp32 dQ accumulator
 * for 16-bit inputs, or the 16-bit planes of q, dout, k, v for fp32 inputs). */
int64_t elsa_backward_workspace_bytes(int dtype, int batch, int heads, int n_ctx, int head_dim,
                                      int has_bias, int is_causal, unsigned flags);
int elsa_twopass_backward(const void* q, const void* k, const void* v, const void* out, const void* dout,
                          const float* row_m, const float* row_z,
                          const float* bias, int64_t bias_stride_b, int64_t bias_stride_h,
                          int64_t bias_stride_q, int64_t bias_stride_k,
                          void* dq, void* dk, void* dv,
                          float* dbias, int64_t dbias_stride_b, int64_t dbias_stride_h,
                          int64_t dbias_stride_q, int64_t dbias_stride_k,
                          void* workspace, int64_t workspace_bytes,
                          int dtype, int batch, int heads, int n_ctx, int head_dim,
                          int is_causal, unsigned flags, void* stream);

/* The same backward on strided [B, H, N, D] views.  `strides` holds 8 x 3 element strides {batch, head, row}, in the
 * order q, k, v, out, dout, dq, dk, dv: dq, dk, dv may be the three slices of one packed [B, N, 3, H, D] gradient,
 * dout the [B, N, H*D] gradient of the projection input.  Same rules as elsa_twopass_forward_strided. */
int elsa_twopass_backward_strided(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                  const int64_t* strides,
                                  const float* row_m, const float* row_z,
                                  const float* bias, int64_t bias_stride_b, int64_t bias_stride_h,
                                  int64_t bias_stride_q, int64_t bias_stride_k,
                                  void* dq, void* dk, void* dv,
                                  float* dbias, int64_t dbias_stride_b, int64_t dbias_stride_h,
                                  int64_t dbias_stride_q, int64_t dbias_stride_k,
                                  void* workspace, int64_t workspace_bytes,
                                  int dtype, int batch, int heads, int n_ctx, int head_dim,
                                  int is_causal, unsigned flags, void* stream);

/* Backward of ONE sequence shard (the K/V partitioning of the two-pass formulation, README.md:27-29,
 * carried across GPUs; the reference itself is single-GPU and has no counterpart).
 * k_shard, v_shard, dk_shard, dv_shard: [B*H, n_keys, D], rows key_offset .. key_offset + n_keys - 1
 * of the sequence; q, out, dout: [B*H, n_ctx, D]; row_m, row_z: the state of the MERGED forward.
 * dk_shard, dv_shard are complete; dq_partial ([B*H, n_ctx, D], fp32 whatever the input dtype) is this
 * shard's contribution: the caller sums it over the shards (all_reduce / reduce_scatter) and rounds.
 * No bias.  workspace: elsa_backward_shard_workspace_bytes. */
int64_t elsa_backward_shard_workspace_bytes(int dtype, int batch, int heads, int n_ctx, int head_dim,
                                            unsigned flags);
int elsa_twopass_backward_shard(const void* q, const void* k_shard, const void* v_shard, const void* out,
                                const void* dout, const float* row_m, const float* row_z, float* dq_partial,
                                void* dk_shard, void* dv_shard, void* workspace, int64_t workspace_bytes,
                                int dtype, int batch, int heads, int n_ctx, int head_dim, int n_keys,
                                int key_offset, int is_causal, unsigned flags, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ELSA_B200_H_ */
