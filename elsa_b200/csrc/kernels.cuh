// Internal interface between the C-ABI layer (api.cu) and the kernel translation units.
#pragma once

#include <mutex>
#include <set>
#include <utility>

#include "common.cuh"

namespace elsa {

// Element strides of the batch, head and row axes of a [B, H, rows, D] view; the D axis is contiguous.
struct Strides { int64_t b, h, r; };
inline Strides contiguous_strides(int heads, int64_t rows, int d) {
  return Strides{static_cast<int64_t>(heads) * rows * d, rows * d, static_cast<int64_t>(d)};
}

struct FoldParams {
  const void* q; const void* k; const void* v;
  Strides qs, ks, vs;
  const float* bias; int64_t bsb, bsh, bsq, bsk;
  float* m; float* z; void* s;
  int heads, n_ctx, head_dim, q_start, q_len, part_width, n_parts, bh;
  int n_keys, key_offset;   // rows of k/v per (batch*head) and the global index of their first row (sequence shards)
  int is_causal, summary_dtype, round_p;  // round_p: 0 keep P in fp32, 1 round to fp16, 2 to bf16
  float scale, scale_log2;
  // direct != 0 (FP32-FMA kernel, one partition, one query tile): the partition summary is the final state, so the
  // kernel writes out = s / z (element type = the input type, rows addressed through `os`) and, when row_m is
  // not null, the row state, instead of a summary -- phase 2 would merge a single element
  int direct;
  void* out; Strides os; float* row_m; float* row_z;
  // fp32 inputs on the tensor cores: the 16-bit planes of q, k, v written by fold_tc3_split (null otherwise)
  const void* q3; const void* k3; const void* v3;
};

struct BwdParams {
  const void* q; const void* k; const void* v; const void* dout;
  Strides qs, ks, vs, gs;          // q, k, v, dout
  Strides dqs, dks, dvs;           // dq (ignored when dq_f32: the fp32 partial is always contiguous), dk, dv
  const float* lse; const float* drow;
  const float* bias; int64_t bsb, bsh, bsq, bsk;
  void* dq; void* dk; void* dv;
  float* dbias; int64_t dsb, dsh, dsq, dsk; int dbias_atomic;
  int heads, n_ctx, head_dim, bh, is_causal;
  float scale, scale_log2;
  // sequence shard: k, v, dk, dv hold n_keys rows that are rows key_offset .. key_offset + n_keys - 1 of the
  // sequence (n_keys = n_ctx, key_offset = 0 for the whole problem); dq_f32: dq is an fp32 [BH, N, D] buffer
  int n_keys, key_offset, dq_f32;
  // single_tile != 0 (FP32-FMA kernels, n_ctx <= 64, whole problem): one launch computes D and LSE from out, dout and
  // the row state and then dQ, dK, dV (and dbias) of the only (query tile, key tile) pair
  int single_tile;
  const void* out; Strides os; const float* row_m; const float* row_z;
};

// opt-in to > 48 KB dynamic shared memory once per (function, device)
inline int ensure_dynamic_smem(const void* func, size_t bytes) {
  static std::mutex mu;
  static std::set<std::pair<const void*, int>> done;
  int dev = 0;
  ELSA_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  if (done.count({func, dev})) return ELSA_OK;
  ELSA_CUDA_CHECK(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
  done.insert({func, dev});
  return ELSA_OK;
}

// Status word of the CURRENT device for the bounded device-side waits: one int per device in mapped pinned host
// memory, allocated on first use (api.cu).  *dev_ptr is what a kernel stores through, *host_ptr what the host reads.
int device_status_word(int** dev_ptr, volatile int** host_ptr);
// number of SMs of the current device (cached per device; api.cu)
int sm_count();

// tcgen05 kernels (fold_tc.cu)
bool fold_tc_supported(int dtype, int head_dim, bool has_bias);
int fold_tc(const FoldParams& p, int dtype, cudaStream_t st);
int debug_wait_timeout(unsigned long long limit_ns, cudaStream_t st);
// sequences of at most 64 tokens (Swin windows), fp16 / bf16, on the tensor cores: two per tile, one launch (win_tc.cu)
bool win_tc_supported(int dtype, int head_dim, int n_ctx, bool is_causal);
int win_tc_fwd(const void* q, Strides qs, const void* k, Strides ks, const void* v, Strides vs, const float* bias,
               int64_t bsb, int64_t bsh, int64_t bsq, int64_t bsk, void* out, Strides os, float* row_m, float* row_z,
               int dtype, int summary_dtype, int batch, int heads, int n_ctx, int head_dim, float scale_log2,
               int is_causal, cudaStream_t st);
int win_tc_bwd(const BwdParams& p, int dtype, cudaStream_t st);
// tcgen05 fold for fp16 / bf16 inputs with 64 < head dim <= 128 (fold_tcw.cu)
bool fold_tcw_supported(int dtype, int head_dim, bool has_bias);
int fold_tcw(const FoldParams& p, int dtype, cudaStream_t st);
// tcgen05 fold for fp32 inputs split into 16-bit planes (fold_tc3.cu)
bool fold_tc3_supported(int dtype, int head_dim, bool has_bias);
int64_t fold_tc3_plane_bytes(int bh, int rows);
int fold_tc3_split(const void* x, Strides st, void* planes, int batch, int heads, int rows, int cols, cudaStream_t stream);
int fold_tc3_split_many(int n, const void* const* x, const Strides* st, void* const* planes, const int* rows, int batch,
                        int heads, int cols, cudaStream_t stream);
int fold_tc3(const FoldParams& p, cudaStream_t st);
// tcgen05 backward (bwd_tc.cu); workspace = padded D / LSE vectors + fp32 dQ accumulator
bool bwd_tc_supported(int dtype, int head_dim, bool has_bias);
int64_t bwd_tc_workspace_bytes(int bh, int n_ctx);
int bwd_tc(const BwdParams& p, const void* out, Strides os, const float* row_m, const float* row_z, void* workspace,
           int dtype, cudaStream_t st);
// tcgen05 backward for fp32 inputs split into 16-bit planes (bwd_tc3.cu); workspace = padded D / LSE vectors +
// the planes of q, dout (n_ctx rows) and k, v (n_keys rows)
bool bwd_tc3_supported(int dtype, int head_dim, bool has_bias);
int64_t bwd_tc3_workspace_bytes(int bh, int n_ctx, int n_keys);
int bwd_tc3(const BwdParams& p, const void* out, Strides os, const float* row_m, const float* row_z, void* workspace,
            cudaStream_t st);
// tcgen05 backward for fp16 / bf16 inputs with 64 < head dim <= 128 (bwd_tcw.cu); workspace = padded D / LSE vectors
bool bwd_tcw_supported(int dtype, int head_dim, bool has_bias);
int64_t bwd_tcw_workspace_bytes(int bh, int n_ctx);
int bwd_tcw(const BwdParams& p, const void* out, Strides os, const float* row_m, const float* row_z, void* workspace,
            int dtype, cudaStream_t st);
// D, LSE from out, dout (any strides) and the row state (bwd_simt.cu)
int bwd_preprocess_any(const void* out, Strides os, const void* dout, Strides gs, const float* row_m, const float* row_z,
                       float* row_d, float* row_lse, int dtype, int batch, int heads, int n_ctx, int head_dim, cudaStream_t st);

// FP32-FMA kernels (fold_simt.cu, bwd_simt.cu)
int fold_simt(const FoldParams& p, int dtype, cudaStream_t st);
int bwd_simt(const BwdParams& p, int dtype, cudaStream_t st);

// q' = fp16(q * fp16(c)), the product formed in fp16 (phase2.cu)
int prescale_q_f16(const void* q, void* q_scaled, int64_t n_elems, float c, cudaStream_t st);

// phase 2 (phase2.cu)
// out_strides == nullptr: out is [bh, n_ctx, head_dim] contiguous; else `heads` splits bh and out is addressed by strides
int merge_final_any(const float* m, const float* z, const void* s, void* out, float* row_m, float* row_z,
                    int summary_dtype, int out_dtype, int n_parts, int bh, int q_start, int q_len, int n_ctx,
                    int head_dim, int first_part, int store_state, cudaStream_t st, int normalize = 1,
                    int heads = 1, const Strides* out_strides = nullptr);

}  // namespace elsa
