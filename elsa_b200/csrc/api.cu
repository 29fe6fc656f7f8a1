// C-ABI layer: argument validation, work planning (partition width, query chunking), host
// orchestration of the two passes and of the backward.  Everything is stream-ordered; nothing
// here allocates device memory or synchronises.  Two things live inside the library instead of with the
// caller: the 64 MiB scratch array of elsa_twopass_forward_static, and one block of pinned host memory for
// the per-device status words (allocated once, at the first call that needs it).
#include <algorithm>
#include <cmath>

#include "kernels.cuh"

namespace elsa {

thread_local int g_last_cuda_error = 0;
std::atomic<long long> g_kernel_launches{0};

// sequences shorter than this run on the FP32-FMA kernels (the tensor-core kernels work on 128-row tiles)
#ifndef ELSA_TC_MIN_TOKENS
#define ELSA_TC_MIN_TOKENS 512
#endif
constexpr int kTcMinTokens = ELSA_TC_MIN_TOKENS;
// ... unless the problem has at least this many rows in total (batch * heads * tokens): from there on the 128-row tiles
// fill the machine, and the tensor-core kernels are 3-10 times faster from 65 tokens on (the window kernels take the
// 16-bit sequences of at most 64).  Below it both families are bound by the launch path.
#ifndef ELSA_TC_MIN_ROWS
#define ELSA_TC_MIN_ROWS 4096
#endif
static bool tc_tokens_ok(int n_ctx, int bh) {
  return n_ctx >= kTcMinTokens || (n_ctx > 64 && static_cast<int64_t>(bh) * n_ctx >= ELSA_TC_MIN_ROWS);
}

static int g_sm_count_cache[64] = {0};

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (g_sm_count_cache[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count_cache[dev] = n;
  }
  return g_sm_count_cache[dev];
}

// ---- device status word ------------------------------------------------------------------------
// One int per device in ONE block of mapped, portable pinned host memory, allocated at the first call that needs it
// (a host allocation, made once per process; it must not fall inside a stream capture).  Kernels store through the
// device-side alias, the host reads the word directly: no copy, no synchronisation on the call path.
int device_status_word(int** dev_ptr, volatile int** host_ptr) {
  static std::mutex mu;
  static int* host_block = nullptr;
  static int* dev_alias[64] = {nullptr};
  int dev = 0;
  ELSA_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return ELSA_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (!host_block) {
    void* p = nullptr;
    ELSA_CUDA_CHECK(cudaHostAlloc(&p, 64 * sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable));
    host_block = static_cast<int*>(p);
    for (int i = 0; i < 64; ++i) host_block[i] = 0;
  }
  if (!dev_alias[dev]) {
    void* d = nullptr;
    ELSA_CUDA_CHECK(cudaHostGetDevicePointer(&d, host_block + dev, 0));
    dev_alias[dev] = static_cast<int*>(d);
  }
  if (dev_ptr) *dev_ptr = dev_alias[dev];
  if (host_ptr) *host_ptr = host_block + dev;
  return ELSA_OK;
}

// A wait that gave up earlier leaves the word set until elsa_device_status(1) clears it: every later call that
// would launch a tensor-core kernel reports it instead of launching.
static int check_device_status() {
  volatile int* host = nullptr;
  const int rc = device_status_word(nullptr, &host);
  if (rc != ELSA_OK) return rc;
  return *host != 0 ? ELSA_ERR_DEVICE_TIMEOUT : ELSA_OK;
}

struct ForwardPlan {
  int part_width, n_parts, q_chunk, tile_m, tile_n;
  bool tensor_cores;
  bool split3;                // fp32 inputs on the tensor cores as 16-bit planes (fold_tc3.cu)
  int64_t mz_bytes, s_bytes;  // one summary set: m (== z) and s, 256-byte aligned
  int sets;                   // 1, or 2 when a ping-pong pass (scan steps / tree) was requested
};

static bool tc_forward_ok(int dtype, int head_dim, int n_ctx, int bh, bool has_bias, unsigned flags) {
  // tcgen05 fold: 16-bit inputs, head dim 64, no bias; short sequences stay on the FP32-FMA kernel
  // (one 64-row CTA per tile keeps more SMs busy than a 256-row CTA does when N is a few hundred).
  if (flags & ELSA_FLAG_FORCE_SIMT) return false;
  return tc_tokens_ok(n_ctx, bh) && fold_tc_supported(dtype, head_dim, has_bias);
}

// 16-bit inputs with 64 < head dim <= 128, or with a bias and any head dim up to 128, on the tensor cores
// (fold_tcw.cu / bwd_tcw.cu: one 128-row tile per CTA)
static bool tcw_forward_ok(int dtype, int head_dim, int n_ctx, int bh, bool has_bias, unsigned flags) {
  if (flags & ELSA_FLAG_FORCE_SIMT) return false;
  return tc_tokens_ok(n_ctx, bh) && fold_tcw_supported(dtype, head_dim, has_bias);
}

// fp32 on the tensor cores: head dim up to 64, and long enough that 128-row tiles fill the machine better than the
// FP32-FMA kernel's 64-row tiles do
static bool tc3_forward_ok(int dtype, int head_dim, int n_ctx, int bh, bool has_bias, unsigned flags) {
  if (flags & (ELSA_FLAG_FORCE_SIMT | ELSA_FLAG_FP32_FMA)) return false;
  return tc_tokens_ok(n_ctx, bh) && fold_tc3_supported(dtype, head_dim, has_bias);
}

static int plan_forward(int dtype, int summary_dtype, int batch, int heads, int n_ctx, int head_dim, int is_causal,
                        bool has_bias, int part_width_in, int q_chunk_in, unsigned flags, ForwardPlan* pl) {
  if (!dtype_ok(dtype) || !dtype_ok(summary_dtype) || batch < 1 || heads < 1 || n_ctx < 1 || head_dim < 1 ||
      head_dim > 128)
    return ELSA_ERR_INVALID_ARGUMENT;
  const int64_t bh = static_cast<int64_t>(batch) * heads;
  if (bh > 65535) return ELSA_ERR_UNSUPPORTED;
  pl->split3 = tc3_forward_ok(dtype, head_dim, n_ctx, batch * heads, has_bias, flags);
  const bool wide = tcw_forward_ok(dtype, head_dim, n_ctx, batch * heads, has_bias, flags);
  pl->tensor_cores = pl->split3 || wide || tc_forward_ok(dtype, head_dim, n_ctx, batch * heads, has_bias, flags);
  pl->tile_m = (pl->split3 || wide) ? 128 : (pl->tensor_cores ? 256 : 64);   // query rows per CTA
  pl->tile_n = pl->tensor_cores ? 128 : 64;                          // keys per tile
  const int tiles_n = static_cast<int>(cdiv64(n_ctx, pl->tile_n));
  int n_parts;
  if (part_width_in > 0) {
    pl->part_width = static_cast<int>(align_up(part_width_in, pl->tile_n));
  } else {
    // Every extra partition is one more summary to write and merge.  FP32-FMA kernels: the smallest partition count
    // whose CTA count fills the SMs in whole waves to >= 92 % (or the best seen).
    const int64_t q_ctas = cdiv64(n_ctx, pl->tile_m) * bh;
    const int64_t slots = static_cast<int64_t>(sm_count()) * (pl->tensor_cores ? 1 : 3);
    const int max_parts = static_cast<int>(std::min<int64_t>(tiles_n, pl->tensor_cores ? 8 : 16));
    int best = 1;
    if (pl->tensor_cores) {
      // Tensor-core kernels (one CTA per SM): time ~ waves x (key tiles per partition + fixed cost of a CTA) + the merge
      // pass over the partition summaries, in units of one key-tile step.  The fixed cost (barrier and TMEM set-up,
      // the first loads, the summary store) is about three steps; a step of the 256-row kernels takes ~1.8 us, so one
      // HBM pass over a summary set is bytes / 6.5 TB/s / 1.8 us steps.  (Measured at (8,3,4097,64): five partitions
      // fill the waves to 98 % but take 239 + 16 us; one partition fills them to 92 % and takes 190 us.)
      const double fixed_steps = 3.0;
      const double merge_steps_per_part = static_cast<double>(bh) * n_ctx * (head_dim * dtype_size(summary_dtype) + 8) / 6.5e6 / 1.8;
      double best_cost = 0.0;
      for (int cand = 1; cand <= max_parts; ++cand) {
        const int tiles_per_part = static_cast<int>(cdiv64(tiles_n, cand));
        const int64_t real_parts = cdiv64(tiles_n, tiles_per_part);
        if (real_parts != cand && cand > 1) continue;       // (the same split as a smaller candidate)
        const int64_t waves = cdiv64(q_ctas * real_parts, slots);
        double cost = static_cast<double>(waves) * (tiles_per_part + fixed_steps) + merge_steps_per_part * static_cast<double>(real_parts);
        if (is_causal) {
          // causal: a CTA's work grows with its first row (long CTAs are handed out first), half of the tile pairs are
          // skipped and (P - 1) / 2P of the (query tile, partition) pairs are empty: total work over the slots plus a
          // tail of a quarter of the longest CTA.  (Measured: (1,8,8192,64) one partition 0.156 ms, two 0.138.)
          const double p = static_cast<double>(real_parts);
          const double work = static_cast<double>(q_ctas) * (0.5 * tiles_n + 0.5 * pl->tile_m / pl->tile_n);
          const double ctas = static_cast<double>(q_ctas) * p * (p + 1.0) / (2.0 * p);
          cost = (work + ctas * (fixed_steps + 1.0)) / static_cast<double>(slots) + 0.25 * tiles_per_part + merge_steps_per_part * p;
        }
        if (cand == 1 || cost < best_cost - 1e-9) { best_cost = cost; best = cand; }
      }
    } else {
      double best_eff = 0.0;
      for (int cand = 1; cand <= max_parts; ++cand) {
        const int tiles_per_part = static_cast<int>(cdiv64(tiles_n, cand));
        const int64_t real_parts = cdiv64(tiles_n, tiles_per_part);
        const int64_t ctas = q_ctas * real_parts;
        const double eff = static_cast<double>(ctas) / static_cast<double>(cdiv64(ctas, slots) * slots);
        if (eff > best_eff + 1e-9) { best_eff = eff; best = cand; }
        if (eff >= 0.92) { best = cand; break; }
      }
    }
    pl->part_width = static_cast<int>(cdiv64(tiles_n, best)) * pl->tile_n;
  }
  n_parts = static_cast<int>(cdiv64(n_ctx, pl->part_width));
  if (n_parts > 65535) return ELSA_ERR_UNSUPPORTED;
  pl->n_parts = n_parts;
  pl->sets = (flags & (ELSA_FLAG_SCAN_STEPS | ELSA_FLAG_TREE_MERGE)) ? 2 : 1;
  const int64_t row_bytes = static_cast<int64_t>(n_parts) * bh * (static_cast<int64_t>(head_dim) * dtype_size(summary_dtype) + 8);
  int q_chunk;
  if (q_chunk_in > 0) {
    q_chunk = static_cast<int>(std::min<int64_t>(n_ctx, align_up(q_chunk_in, pl->tile_m)));
  } else {
    const int64_t cap = static_cast<int64_t>(1) << 30;  // keep one summary set under 1 GiB
    int64_t rows = std::max<int64_t>(pl->tile_m, (cap / row_bytes) / pl->tile_m * pl->tile_m);
    q_chunk = static_cast<int>(std::min<int64_t>(n_ctx, rows));
  }
  pl->q_chunk = q_chunk;
  const int64_t rows_total = static_cast<int64_t>(n_parts) * bh * q_chunk;
  pl->mz_bytes = align_up(rows_total * 4, 256);
  pl->s_bytes = align_up(rows_total * head_dim * dtype_size(summary_dtype), 256);
  return ELSA_OK;
}

static int64_t plan_bytes(const ForwardPlan& pl) { return pl.sets * (2 * pl.mz_bytes + pl.s_bytes); }

// ELSA_FLAG_REF_ROUNDING reproduces the rounding points of the reference's fp16 head-dim-64 kernels
// (attention_parallel_scan.py:153-154,160: q is multiplied by log2(e)/8 IN fp16 -- the constant rounded to fp16, the
// product rounded to fp16 -- and the scores get no further scale).  It applies where the reference takes those
// kernels: fp16, head dim 64, no bias, not causal; elsewhere the flag changes nothing.
static bool ref_rounding_applies(unsigned flags, int dtype, int head_dim, bool has_bias, int is_causal) {
  return (flags & ELSA_FLAG_REF_ROUNDING) && dtype == ELSA_F16 && head_dim == 64 && !has_bias && !is_causal;
}
static int64_t ref_rounding_bytes(int batch, int heads, int n_ctx, int head_dim) {
  return align_up(static_cast<int64_t>(batch) * heads * n_ctx * head_dim * 2, 256);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int phase1_dispatch(const void* q, const void* k, const void* v, const float* bias, int64_t bsb, int64_t bsh,
                           int64_t bsq, int64_t bsk, float* m_buf, float* z_buf, void* s_buf, int dtype,
                           int summary_dtype, int batch, int heads, int n_ctx, int head_dim, int q_start, int q_len,
                           int part_width, int n_parts, int is_causal, unsigned flags, cudaStream_t st,
                           int n_keys = -1, int key_offset = 0, bool q_prescaled = false,
                           const Strides* qs = nullptr, const Strides* ks = nullptr, const Strides* vs = nullptr,
                           void* direct_out = nullptr, const Strides* os = nullptr, float* row_m = nullptr,
                           float* row_z = nullptr, const void* q3 = nullptr, const void* k3 = nullptr,
                           const void* v3 = nullptr) {
  if (n_keys < 0) n_keys = n_ctx;
  if (!q || !k || !v || ((!m_buf || !z_buf || !s_buf) && !direct_out) || !dtype_ok(dtype) || !dtype_ok(summary_dtype) || batch < 1 ||
      heads < 1 || n_ctx < 1 || head_dim < 1 || head_dim > 128 || q_start < 0 || q_len < 0 ||
      q_start + q_len > n_ctx || part_width < 1 || n_parts < 1 ||
      static_cast<int64_t>(n_parts) * part_width < n_keys || n_keys < 1 || key_offset < 0)
    return ELSA_ERR_INVALID_ARGUMENT;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || (!direct_out && !aligned16(s_buf))) return ELSA_ERR_INVALID_ARGUMENT;
  if (static_cast<int64_t>(batch) * heads > 65535 || n_parts > 65535) return ELSA_ERR_UNSUPPORTED;
  if (q_len == 0) return ELSA_OK;
  if (part_width % 64 != 0) return ELSA_ERR_INVALID_ARGUMENT;
  FoldParams p;
  p.q = q; p.k = k; p.v = v;
  p.qs = qs ? *qs : contiguous_strides(heads, n_ctx, head_dim);
  p.ks = ks ? *ks : contiguous_strides(heads, n_keys, head_dim);
  p.vs = vs ? *vs : contiguous_strides(heads, n_keys, head_dim);
  p.bias = bias; p.bsb = bsb; p.bsh = bsh; p.bsq = bsq; p.bsk = bsk;
  p.m = m_buf; p.z = z_buf; p.s = s_buf;
  p.heads = heads; p.n_ctx = n_ctx; p.head_dim = head_dim; p.q_start = q_start; p.q_len = q_len;
  p.part_width = part_width; p.n_parts = n_parts; p.bh = batch * heads;
  p.n_keys = n_keys; p.key_offset = key_offset;
  p.is_causal = is_causal ? 1 : 0;
  p.summary_dtype = summary_dtype;
  p.q3 = q3; p.k3 = k3; p.v3 = v3;
  p.direct = direct_out ? 1 : 0;
  p.out = direct_out; p.os = os ? *os : contiguous_strides(heads, n_ctx, head_dim); p.row_m = row_m; p.row_z = row_z;
  // reference rounding point: P is cast to fp16 before P.V only for fp16 inputs whose summaries are
  // not fp32 (attention_parallel_scan.py:701, attention.py:96-99); bf16 and fp32 keep P in fp32.
  p.round_p = (dtype == ELSA_F16 && summary_dtype != ELSA_F32) ? 1 : 0;
  p.scale = 1.0f / std::sqrt(static_cast<float>(head_dim));
  p.scale_log2 = static_cast<float>((1.0 / std::sqrt(static_cast<double>(head_dim))) * 1.4426950408889634);
  if (q_prescaled) p.scale_log2 = 1.0f;   // q already carries log2(e)/sqrt(d) (reference-rounding mode, no bias)
  if (q3 && part_width % 128 == 0) {
    const int src = check_device_status();
    if (src != ELSA_OK) return src;
    return fold_tc3(p, st);
  }
  if (part_width % 128 == 0 && tc_forward_ok(dtype, head_dim, n_ctx, batch * heads, bias != nullptr, flags)) {
    const int src = check_device_status();
    if (src != ELSA_OK) return src;
    return fold_tc(p, dtype, st);
  }
  if (part_width % 128 == 0 && tcw_forward_ok(dtype, head_dim, n_ctx, batch * heads, bias != nullptr, flags)) {
    const int src = check_device_status();
    if (src != ELSA_OK) return src;
    return fold_tcw(p, dtype, st);
  }
  return fold_simt(p, dtype, st);
}

}  // namespace elsa

using namespace elsa;

extern "C" int elsa_abi_version(void) { return ELSA_B200_ABI_VERSION; }

extern "C" const char* elsa_strerror(int status) {
  switch (status) {
    case ELSA_OK: return "ok";
    case ELSA_ERR_INVALID_ARGUMENT: return "invalid argument (size, pointer, dtype or alignment)";
    case ELSA_ERR_UNSUPPORTED: return "unsupported problem for this build";
    case ELSA_ERR_CUDA: return "CUDA call failed (see elsa_last_cuda_error)";
    case ELSA_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case ELSA_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    default: return "unknown status";
  }
}

extern "C" int elsa_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int elsa_device_status(int clear) {
  volatile int* host = nullptr;
  if (device_status_word(nullptr, &host) != ELSA_OK) return -1;
  const int v = *host;
  if (clear && v != 0) *host = 0;
  return v;
}

extern "C" int elsa_debug_wait_timeout(uint64_t limit_ns, void* stream) {
  if (limit_ns == 0 || limit_ns > 1000000000ull) return ELSA_ERR_INVALID_ARGUMENT;   // at most one second
  return debug_wait_timeout(limit_ns, static_cast<cudaStream_t>(stream));
}

extern "C" int64_t elsa_kernel_launches(void) { return static_cast<int64_t>(g_kernel_launches.load()); }

static bool tc_backward_ok(int dtype, int head_dim, int n_ctx, int bh, bool has_bias, unsigned flags);
static bool tc3_backward_ok(int dtype, int head_dim, int n_ctx, int bh, bool has_bias, unsigned flags);
static bool tcw_backward_ok(int dtype, int head_dim, int n_ctx, int bh, bool has_bias, unsigned flags);

extern "C" int elsa_uses_tensor_cores_for(int dtype, int head_dim, int n_ctx, int has_bias, int is_causal, int backward,
                                          int batch, int heads) {
  if (batch < 1 || heads < 1) return 0;
  // sequences of at most 64 tokens, 16-bit: two per tensor-core tile, forward and backward (win_tc.cu)
  if (n_ctx >= 1 && n_ctx <= 64 && win_tc_supported(dtype, head_dim, n_ctx, is_causal != 0)) return 1;
  const int bh = static_cast<int>(std::min<int64_t>(static_cast<int64_t>(batch) * heads, 1 << 30));
  if (backward)
    return (tc_backward_ok(dtype, head_dim, n_ctx, bh, has_bias != 0, 0u) || tc3_backward_ok(dtype, head_dim, n_ctx, bh, has_bias != 0, 0u) ||
            tcw_backward_ok(dtype, head_dim, n_ctx, bh, has_bias != 0, 0u)) ? 1 : 0;
  return (tc_forward_ok(dtype, head_dim, n_ctx, bh, has_bias != 0, 0u) || tc3_forward_ok(dtype, head_dim, n_ctx, bh, has_bias != 0, 0u) ||
          tcw_forward_ok(dtype, head_dim, n_ctx, bh, has_bias != 0, 0u)) ? 1 : 0;
}

// the answer for a single (batch, head): what holds whatever the batch size
extern "C" int elsa_uses_tensor_cores(int dtype, int head_dim, int n_ctx, int has_bias, int is_causal, int backward) {
  return elsa_uses_tensor_cores_for(dtype, head_dim, n_ctx, has_bias, is_causal, backward, 1, 1);
}

extern "C" int elsa_phase1_fold(const void* q, const void* k, const void* v, const float* bias, int64_t bias_stride_b,
                                int64_t bias_stride_h, int64_t bias_stride_q, int64_t bias_stride_k, float* m_buf,
                                float* z_buf, void* s_buf, int dtype, int summary_dtype, int batch, int heads,
                                int n_ctx, int head_dim, int q_start, int q_len, int part_width, int n_parts,
                                int is_causal, unsigned flags, void* stream) {
  return phase1_dispatch(q, k, v, bias, bias_stride_b, bias_stride_h, bias_stride_q, bias_stride_k, m_buf, z_buf, s_buf,
                         dtype, summary_dtype, batch, heads, n_ctx, head_dim, q_start, q_len, part_width, n_parts,
                         is_causal, flags, static_cast<cudaStream_t>(stream));
}

extern "C" int elsa_phase1_fold_shard(const void* q, const void* k, const void* v, float* m_buf, float* z_buf,
                                      void* s_buf, int dtype, int summary_dtype, int batch, int heads, int n_ctx,
                                      int head_dim, int n_keys, int key_offset, int part_width, int n_parts,
                                      int is_causal, unsigned flags, void* stream) {
  return phase1_dispatch(q, k, v, nullptr, 0, 0, 0, 0, m_buf, z_buf, s_buf, dtype, summary_dtype, batch, heads, n_ctx,
                         head_dim, 0, n_ctx, part_width, n_parts, is_causal, flags, static_cast<cudaStream_t>(stream),
                         n_keys, key_offset);
}

// The shard fold with a workspace: fp32 inputs then run on the tensor cores (16-bit planes per operand, written
// into the workspace); every other case is the plain shard fold and needs no workspace.
extern "C" int64_t elsa_phase1_fold_shard_workspace_bytes(int dtype, int batch, int heads, int n_ctx, int head_dim,
                                                          int n_keys, unsigned flags) {
  if (!dtype_ok(dtype) || batch < 1 || heads < 1 || n_ctx < 1 || head_dim < 1 || head_dim > 128 || n_keys < 0) return -1;
  if (n_keys == 0 || !tc3_forward_ok(dtype, head_dim, n_ctx, batch * heads, false, flags)) return 0;
  return fold_tc3_plane_bytes(batch * heads, n_ctx) + 2 * fold_tc3_plane_bytes(batch * heads, n_keys);
}

extern "C" int elsa_phase1_fold_shard_ws(const void* q, const void* k, const void* v, float* m_buf, float* z_buf,
                                         void* s_buf, void* workspace, int64_t workspace_bytes, int dtype,
                                         int summary_dtype, int batch, int heads, int n_ctx, int head_dim, int n_keys,
                                         int key_offset, int part_width, int n_parts, int is_causal, unsigned flags,
                                         void* stream) {
  const int64_t need = elsa_phase1_fold_shard_workspace_bytes(dtype, batch, heads, n_ctx, head_dim, n_keys, flags);
  if (need < 0) return ELSA_ERR_INVALID_ARGUMENT;
  auto st = static_cast<cudaStream_t>(stream);
  const void *q3 = nullptr, *k3 = nullptr, *v3 = nullptr;
  if (need > 0 && part_width % 128 == 0) {
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < need) return ELSA_ERR_WORKSPACE;
    if (!q || !k || !v) return ELSA_ERR_INVALID_ARGUMENT;
    char* planes = static_cast<char*>(workspace);
    const int64_t qb = fold_tc3_plane_bytes(batch * heads, n_ctx), kb = fold_tc3_plane_bytes(batch * heads, n_keys);
    int rc;
    {
      const void* xs[3] = {q, k, v};
      const Strides sts[3] = {contiguous_strides(heads, n_ctx, head_dim), contiguous_strides(heads, n_keys, head_dim),
                              contiguous_strides(heads, n_keys, head_dim)};
      void* pls[3] = {planes, planes + qb, planes + qb + kb};
      const int rws[3] = {n_ctx, n_keys, n_keys};
      if ((rc = fold_tc3_split_many(3, xs, sts, pls, rws, batch, heads, head_dim, st)) != ELSA_OK) return rc;
    }
    q3 = planes; k3 = planes + qb; v3 = planes + qb + kb;
  }
  return phase1_dispatch(q, k, v, nullptr, 0, 0, 0, 0, m_buf, z_buf, s_buf, dtype, summary_dtype, batch, heads, n_ctx,
                         head_dim, 0, n_ctx, part_width, n_parts, is_causal, flags, st, n_keys, key_offset, false, nullptr,
                         nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, q3, k3, v3);
}

extern "C" int elsa_forward_plan(int dtype, int summary_dtype, int batch, int heads, int n_ctx, int head_dim,
                                 int has_bias, int is_causal, int part_width_in, int q_chunk_in, unsigned flags,
                                 int* part_width, int* n_parts, int* q_chunk) {
  ForwardPlan pl;
  int rc = plan_forward(dtype, summary_dtype, batch, heads, n_ctx, head_dim, is_causal, has_bias != 0, part_width_in,
                        q_chunk_in, flags, &pl);
  if (rc != ELSA_OK) return rc;
  if (part_width) *part_width = pl.part_width;
  if (n_parts) *n_parts = pl.n_parts;
  if (q_chunk) *q_chunk = pl.q_chunk;
  return ELSA_OK;
}

extern "C" int64_t elsa_forward_workspace_bytes(int dtype, int summary_dtype, int batch, int heads, int n_ctx,
                                                int head_dim, int has_bias, int is_causal, int part_width,
                                                int q_chunk, unsigned flags) {
  if (n_ctx == 0) return 0;
  ForwardPlan pl;
  if (plan_forward(dtype, summary_dtype, batch, heads, n_ctx, head_dim, is_causal, has_bias != 0, part_width, q_chunk, flags,
                   &pl) != ELSA_OK)
    return -1;
  return plan_bytes(pl) +
         (ref_rounding_applies(flags, dtype, head_dim, has_bias != 0, is_causal) ? ref_rounding_bytes(batch, heads, n_ctx, head_dim) : 0) +
         (pl.split3 ? 3 * fold_tc3_plane_bytes(batch * heads, n_ctx) : 0);
}

// strides given by the caller: every one a multiple of 8 elements, so that rows start on 16-byte boundaries
static bool strides_ok(const int64_t* st, int head_dim) {
  return st && st[0] >= 0 && st[1] >= 0 && st[2] >= head_dim && (st[0] | st[1] | st[2]) % 8 == 0;
}
static Strides to_strides(const int64_t* st) { return Strides{st[0], st[1], st[2]}; }

static int forward_impl(const void* q, const void* k, const void* v, const Strides* qs, const Strides* ks,
                        const Strides* vs, const float* bias, int64_t bias_stride_b, int64_t bias_stride_h,
                        int64_t bias_stride_q, int64_t bias_stride_k, void* out, const Strides* os, float* row_m,
                        float* row_z, void* workspace, int64_t workspace_bytes, int dtype, int summary_dtype, int batch,
                        int heads, int n_ctx, int head_dim, int is_causal, int part_width, int q_chunk, unsigned flags,
                        void* stream) {
  if (n_ctx == 0) return ELSA_OK;
  if (!q || !k || !v || !out) return ELSA_ERR_INVALID_ARGUMENT;
  if ((row_m == nullptr) != (row_z == nullptr)) return ELSA_ERR_INVALID_ARGUMENT;
  ForwardPlan pl;
  int rc = plan_forward(dtype, summary_dtype, batch, heads, n_ctx, head_dim, is_causal, bias != nullptr, part_width,
                        q_chunk, flags, &pl);
  if (rc != ELSA_OK) return rc;
  const bool ref_round = ref_rounding_applies(flags, dtype, head_dim, bias != nullptr, is_causal);
  const int64_t plane_bytes = pl.split3 ? fold_tc3_plane_bytes(batch * heads, n_ctx) : 0;
  const int64_t need_ws = plan_bytes(pl) + (ref_round ? ref_rounding_bytes(batch, heads, n_ctx, head_dim) : 0) + 3 * plane_bytes;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < need_ws)
    return ELSA_ERR_WORKSPACE;
  if (!aligned16(out)) return ELSA_ERR_INVALID_ARGUMENT;
  auto st = static_cast<cudaStream_t>(stream);
  char* ws = static_cast<char*>(workspace);
  if (ref_round) {
    // q' = fp16(q * fp16(log2(e) / sqrt(d))) behind the summaries in the workspace; phase 1 then runs on q' unscaled
    void* q_scaled = ws + plan_bytes(pl);
    if (!aligned16(q)) return ELSA_ERR_INVALID_ARGUMENT;
    if (qs) return ELSA_ERR_UNSUPPORTED;   // the pre-scaled copy is made from a contiguous q
    rc = prescale_q_f16(q, q_scaled, static_cast<int64_t>(batch) * heads * n_ctx * head_dim,
                        static_cast<float>((1.0 / std::sqrt(static_cast<double>(head_dim))) * 1.4426950408889634), st);
    if (rc != ELSA_OK) return rc;
    q = q_scaled;
  }
  float* m_a = reinterpret_cast<float*>(ws);
  float* z_a = reinterpret_cast<float*>(ws + pl.mz_bytes);
  void* s_a = ws + 2 * pl.mz_bytes;
  char* ws_b = ws + 2 * pl.mz_bytes + pl.s_bytes;
  float* m_b = reinterpret_cast<float*>(ws_b);
  float* z_b = reinterpret_cast<float*>(ws_b + pl.mz_bytes);
  void* s_b = ws_b + 2 * pl.mz_bytes;
  const int bh = batch * heads;
  const int store_state = row_m != nullptr;

  const void *q3 = nullptr, *k3 = nullptr, *v3 = nullptr;
  if (pl.split3) {
    // fp32 on the tensor cores: the 16-bit planes of q, k, v, written once behind the summaries
    char* planes = ws + plan_bytes(pl);
    const Strides cs = contiguous_strides(heads, n_ctx, head_dim);
    {
      const void* xs[3] = {q, k, v};
      const Strides sts[3] = {qs ? *qs : cs, ks ? *ks : cs, vs ? *vs : cs};
      void* pls[3] = {planes, planes + plane_bytes, planes + 2 * plane_bytes};
      const int rws[3] = {n_ctx, n_ctx, n_ctx};
      if ((rc = fold_tc3_split_many(3, xs, sts, pls, rws, batch, heads, head_dim, st)) != ELSA_OK) return rc;
    }
    q3 = planes; k3 = planes + plane_bytes; v3 = planes + 2 * plane_bytes;
  }
  // A problem that is a single (query tile, key partition) pair of the FP32-FMA kernel (49-token windows and other
  // sequences of at most 64 tokens): phase 2 would merge one summary per row, so phase 1 finalises the rows itself,
  // with the same rounding points, and the summaries never travel through memory.
  if (!pl.tensor_cores && pl.n_parts == 1 && n_ctx <= 64 && !(flags & (ELSA_FLAG_SCAN_STEPS | ELSA_FLAG_TREE_MERGE))) {
    // 16-bit inputs: two sequences per 128-row tensor-core tile, one launch (win_tc.cu)
    if (!(flags & ELSA_FLAG_FORCE_SIMT) && !ref_round && win_tc_supported(dtype, head_dim, n_ctx, is_causal != 0)) {
      const Strides cs0 = contiguous_strides(heads, n_ctx, head_dim);
      const int src = check_device_status();
      if (src != ELSA_OK) return src;
      const float sl2 = static_cast<float>((1.0 / std::sqrt(static_cast<double>(head_dim))) * 1.4426950408889634);
      return win_tc_fwd(q, qs ? *qs : cs0, k, ks ? *ks : cs0, v, vs ? *vs : cs0, bias, bias_stride_b, bias_stride_h,
                        bias_stride_q, bias_stride_k, out, os ? *os : cs0, row_m, row_z, dtype, summary_dtype, batch, heads,
                        n_ctx, head_dim, sl2, is_causal, st);
    }
    return phase1_dispatch(q, k, v, bias, bias_stride_b, bias_stride_h, bias_stride_q, bias_stride_k, nullptr, nullptr,
                           nullptr, dtype, summary_dtype, batch, heads, n_ctx, head_dim, 0, n_ctx, pl.part_width, 1,
                           is_causal, flags, st, -1, 0, ref_round, qs, ks, vs, out, os, row_m, row_z);
  }
  // One partition and one query chunk on the 16-bit d <= 64 tensor-core fold: the summary is the row's final state, so
  // the fold writes out and the row state itself (same rounding points as the merge pass) and no merge pass runs.
  if (pl.n_parts == 1 && pl.q_chunk >= n_ctx && !ref_round && !(flags & (ELSA_FLAG_SCAN_STEPS | ELSA_FLAG_TREE_MERGE)) &&
      pl.part_width % 128 == 0 && tc_forward_ok(dtype, head_dim, n_ctx, batch * heads, bias != nullptr, flags)) {
    return phase1_dispatch(q, k, v, bias, bias_stride_b, bias_stride_h, bias_stride_q, bias_stride_k, nullptr, nullptr,
                           nullptr, dtype, summary_dtype, batch, heads, n_ctx, head_dim, 0, n_ctx, pl.part_width, 1,
                           is_causal, flags, st, -1, 0, false, qs, ks, vs, out, os, row_m, row_z);
  }
  for (int q_start = 0; q_start < n_ctx; q_start += pl.q_chunk) {
    const int q_len = std::min(pl.q_chunk, n_ctx - q_start);
    rc = phase1_dispatch(q, k, v, bias, bias_stride_b, bias_stride_h, bias_stride_q, bias_stride_k, m_a, z_a, s_a, dtype,
                         summary_dtype, batch, heads, n_ctx, head_dim, q_start, q_len, pl.part_width, pl.n_parts,
                         is_causal, flags, st, -1, 0, ref_round, qs, ks, vs, nullptr, nullptr, nullptr, nullptr, q3, k3, v3);
    if (rc != ELSA_OK) return rc;
    if (is_causal && (flags & ELSA_FLAG_SCAN_STEPS)) {
      // log-depth Hillis-Steele inclusive scan, ping-pong between the two summary sets; the last
      // prefix is the row's answer (future partitions hold the identity).
      float *sm = m_a, *sz = z_a, *dm = m_b, *dz = z_b;
      void *ss = s_a, *ds = s_b;
      for (int step = 1; step < pl.n_parts; step *= 2) {
        rc = elsa_scan_step(sm, sz, ss, dm, dz, ds, summary_dtype, pl.n_parts, bh, q_len, head_dim, step, stream);
        if (rc != ELSA_OK) return rc;
        std::swap(sm, dm); std::swap(sz, dz); std::swap(ss, ds);
      }
      rc = merge_final_any(sm, sz, ss, out, row_m, row_z, summary_dtype, dtype, 1, bh, q_start, q_len, n_ctx, head_dim,
                           pl.n_parts - 1, store_state, st, 1, heads, os);
    } else if (!is_causal && (flags & ELSA_FLAG_TREE_MERGE)) {
      float *sm = m_a, *sz = z_a, *dm = m_b, *dz = z_b;
      void *ss = s_a, *ds = s_b;
      for (int n_in = pl.n_parts; n_in > 1; n_in = (n_in + 1) / 2) {
        rc = elsa_upsweep_level(sm, sz, ss, dm, dz, ds, summary_dtype, n_in, bh, q_len, head_dim, stream);
        if (rc != ELSA_OK) return rc;
        std::swap(sm, dm); std::swap(sz, dz); std::swap(ss, ds);
      }
      rc = merge_final_any(sm, sz, ss, out, row_m, row_z, summary_dtype, dtype, 1, bh, q_start, q_len, n_ctx, head_dim, 0,
                           store_state, st, 1, heads, os);
    } else {
      rc = merge_final_any(m_a, z_a, s_a, out, row_m, row_z, summary_dtype, dtype, pl.n_parts, bh, q_start, q_len, n_ctx,
                           head_dim, 0, store_state, st, 1, heads, os);
    }
    if (rc != ELSA_OK) return rc;
  }
  return ELSA_OK;
}

extern "C" int elsa_twopass_forward(const void* q, const void* k, const void* v, const float* bias,
                                    int64_t bias_stride_b, int64_t bias_stride_h, int64_t bias_stride_q,
                                    int64_t bias_stride_k, void* out, float* row_m, float* row_z, void* workspace,
                                    int64_t workspace_bytes, int dtype, int summary_dtype, int batch, int heads,
                                    int n_ctx, int head_dim, int is_causal, int part_width, int q_chunk, unsigned flags,
                                    void* stream) {
  return forward_impl(q, k, v, nullptr, nullptr, nullptr, bias, bias_stride_b, bias_stride_h, bias_stride_q, bias_stride_k,
                      out, nullptr, row_m, row_z, workspace, workspace_bytes, dtype, summary_dtype, batch, heads, n_ctx,
                      head_dim, is_causal, part_width, q_chunk, flags, stream);
}

extern "C" int elsa_twopass_forward_strided(const void* q, const void* k, const void* v, const int64_t* q_strides,
                                            const int64_t* k_strides, const int64_t* v_strides, const float* bias,
                                            int64_t bias_stride_b, int64_t bias_stride_h, int64_t bias_stride_q,
                                            int64_t bias_stride_k, void* out, const int64_t* out_strides, float* row_m,
                                            float* row_z, void* workspace, int64_t workspace_bytes, int dtype,
                                            int summary_dtype, int batch, int heads, int n_ctx, int head_dim,
                                            int is_causal, int part_width, int q_chunk, unsigned flags, void* stream) {
  if (!strides_ok(q_strides, head_dim) || !strides_ok(k_strides, head_dim) || !strides_ok(v_strides, head_dim) ||
      !strides_ok(out_strides, head_dim))
    return ELSA_ERR_INVALID_ARGUMENT;
  const Strides qs = to_strides(q_strides), ks = to_strides(k_strides), vs = to_strides(v_strides), os = to_strides(out_strides);
  return forward_impl(q, k, v, &qs, &ks, &vs, bias, bias_stride_b, bias_stride_h, bias_stride_q, bias_stride_k, out, &os,
                      row_m, row_z, workspace, workspace_bytes, dtype, summary_dtype, batch, heads, n_ctx, head_dim,
                      is_causal, part_width, q_chunk, flags, stream);
}

// ---- backward -------------------------------------------------------------------------------
static bool tc_backward_ok(int dtype, int head_dim, int n_ctx, int bh, bool has_bias, unsigned flags) {
  if (flags & ELSA_FLAG_FORCE_SIMT) return false;
  // (the 16-bit backward has no rounding points to keep in step with a forward plan, and from 65 tokens on it is faster
  // than the FP32-FMA kernels at every batch size: 0.048 against 0.095 ms at (1,8,197,64))
  (void)bh;
  return n_ctx > 64 && bwd_tc_supported(dtype, head_dim, has_bias);
}

// fp32 on the tensor cores (16-bit planes per operand): head dim up to 64, with or without a bias (and its gradient)
static bool tc3_backward_ok(int dtype, int head_dim, int n_ctx, int bh, bool has_bias, unsigned flags) {
  if (flags & (ELSA_FLAG_FORCE_SIMT | ELSA_FLAG_FP32_FMA)) return false;
  return tc_tokens_ok(n_ctx, bh) && bwd_tc3_supported(dtype, head_dim, has_bias);
}

// 16-bit inputs with 64 < head dim <= 128, or with a bias (and its gradient) and any head dim up to 128 (bwd_tcw.cu)
static bool tcw_backward_ok(int dtype, int head_dim, int n_ctx, int bh, bool has_bias, unsigned flags) {
  if (flags & ELSA_FLAG_FORCE_SIMT) return false;
  (void)bh;
  return n_ctx > 64 && bwd_tcw_supported(dtype, head_dim, has_bias);
}

static int64_t bwd_state_bytes(int batch, int heads, int n_ctx) {
  return align_up(static_cast<int64_t>(batch) * heads * n_ctx * 4, 256);
}

extern "C" int64_t elsa_backward_workspace_bytes(int dtype, int batch, int heads, int n_ctx, int head_dim,
                                                 int has_bias, int is_causal, unsigned flags) {
  (void)is_causal;
  if (!dtype_ok(dtype) || batch < 1 || heads < 1 || n_ctx < 0 || head_dim < 1 || head_dim > 128) return -1;
  if (tc_backward_ok(dtype, head_dim, n_ctx, batch * heads, has_bias != 0, flags)) return bwd_tc_workspace_bytes(batch * heads, n_ctx);
  // (the fp32 tensor-core route is not taken when dbias is asked for: the larger of the two needs covers both)
  if (tc3_backward_ok(dtype, head_dim, n_ctx, batch * heads, has_bias != 0, flags))
    return std::max(bwd_tc3_workspace_bytes(batch * heads, n_ctx, n_ctx), 2 * bwd_state_bytes(batch, heads, n_ctx));
  if (tcw_backward_ok(dtype, head_dim, n_ctx, batch * heads, has_bias != 0, flags))
    return std::max(bwd_tcw_workspace_bytes(batch * heads, n_ctx), 2 * bwd_state_bytes(batch, heads, n_ctx));
  return 2 * bwd_state_bytes(batch, heads, n_ctx);  // row_d, row_lse
}

// st8: strides of q, k, v, out, dout, dq, dk, dv in that order, or nullptr for contiguous [B*H, N, D] tensors
static int backward_impl(const void* q, const void* k, const void* v, const void* out, const void* dout,
                         const Strides* st8, const float* row_m, const float* row_z, const float* bias,
                         int64_t bias_stride_b, int64_t bias_stride_h, int64_t bias_stride_q, int64_t bias_stride_k,
                         void* dq, void* dk, void* dv, float* dbias, int64_t dbias_stride_b, int64_t dbias_stride_h,
                         int64_t dbias_stride_q, int64_t dbias_stride_k, void* workspace, int64_t workspace_bytes,
                         int dtype, int batch, int heads, int n_ctx, int head_dim, int is_causal, unsigned flags,
                         void* stream) {
  if (n_ctx == 0) return ELSA_OK;
  if (!q || !k || !v || !out || !dout || !row_m || !row_z || !dq || !dk || !dv || !dtype_ok(dtype) || batch < 1 ||
      heads < 1 || n_ctx < 0 || head_dim < 1 || head_dim > 128)
    return ELSA_ERR_INVALID_ARGUMENT;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !aligned16(dout) || !aligned16(dq) ||
      !aligned16(dk) || !aligned16(dv))
    return ELSA_ERR_INVALID_ARGUMENT;
  if (static_cast<int64_t>(batch) * heads > 65535) return ELSA_ERR_UNSUPPORTED;
  const int64_t need = elsa_backward_workspace_bytes(dtype, batch, heads, n_ctx, head_dim, bias != nullptr, is_causal, flags);
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < need) return ELSA_ERR_WORKSPACE;
  char* ws = static_cast<char*>(workspace);
  float* row_d = reinterpret_cast<float*>(ws);
  float* row_lse = reinterpret_cast<float*>(ws + bwd_state_bytes(batch, heads, n_ctx));
  const bool use_tc = dbias == nullptr && tc_backward_ok(dtype, head_dim, n_ctx, batch * heads, bias != nullptr, flags);
  const bool use_tc3 = (dbias == nullptr || bias != nullptr) && tc3_backward_ok(dtype, head_dim, n_ctx, batch * heads, bias != nullptr, flags);
  // (the wide-head kernels also take biased problems, with or without a bias gradient)
  const bool use_tcw = !use_tc && !use_tc3 && (dbias == nullptr || bias != nullptr) &&
                       tcw_backward_ok(dtype, head_dim, n_ctx, batch * heads, bias != nullptr, flags);
  const Strides cs = contiguous_strides(heads, n_ctx, head_dim);
  const Strides os = st8 ? st8[3] : cs;
  BwdParams p;
  p.qs = st8 ? st8[0] : cs; p.ks = st8 ? st8[1] : cs; p.vs = st8 ? st8[2] : cs; p.gs = st8 ? st8[4] : cs;
  p.dqs = st8 ? st8[5] : cs; p.dks = st8 ? st8[6] : cs; p.dvs = st8 ? st8[7] : cs;
  int rc = ELSA_OK;
  // a problem of at most 64 tokens is one (query tile, key tile) pair: one launch does the pre-pass and all gradients
  p.single_tile = (!use_tc && n_ctx <= 64 && head_dim <= 64) ? 1 : 0;
  p.out = out; p.os = os; p.row_m = row_m; p.row_z = row_z;
  if (!use_tc && !use_tc3 && !use_tcw && !p.single_tile)
    rc = bwd_preprocess_any(out, os, dout, p.gs, row_m, row_z, row_d, row_lse, dtype, batch, heads, n_ctx, head_dim,
                            static_cast<cudaStream_t>(stream));
  if (rc != ELSA_OK) return rc;
  p.q = q; p.k = k; p.v = v; p.dout = dout;
  p.lse = row_lse; p.drow = row_d;
  p.bias = bias; p.bsb = bias_stride_b; p.bsh = bias_stride_h; p.bsq = bias_stride_q; p.bsk = bias_stride_k;
  p.dq = dq; p.dk = dk; p.dv = dv;
  p.dbias = dbias; p.dsb = dbias_stride_b; p.dsh = dbias_stride_h; p.dsq = dbias_stride_q; p.dsk = dbias_stride_k;
  p.dbias_atomic = (dbias && ((dbias_stride_b == 0 && batch > 1) || (dbias_stride_h == 0 && heads > 1))) ? 1 : 0;
  p.heads = heads; p.n_ctx = n_ctx; p.head_dim = head_dim; p.bh = batch * heads; p.is_causal = is_causal ? 1 : 0;
  p.scale = 1.0f / std::sqrt(static_cast<float>(head_dim));
  p.scale_log2 = static_cast<float>((1.0 / std::sqrt(static_cast<double>(head_dim))) * 1.4426950408889634);
  p.n_keys = n_ctx; p.key_offset = 0; p.dq_f32 = 0;
  if (use_tc) {
    const int src = check_device_status();
    if (src != ELSA_OK) return src;
    return bwd_tc(p, out, os, row_m, row_z, workspace, dtype, static_cast<cudaStream_t>(stream));
  }
  // 16-bit sequences of at most 64 tokens: two per 128-row tensor-core tile, one launch (win_tc.cu)
  if (p.single_tile && !(flags & ELSA_FLAG_FORCE_SIMT) && (dbias == nullptr || bias != nullptr) &&
      win_tc_supported(dtype, head_dim, n_ctx, is_causal != 0)) {
    const int src = check_device_status();
    if (src != ELSA_OK) return src;
    return win_tc_bwd(p, dtype, static_cast<cudaStream_t>(stream));
  }
  if (use_tc3) {
    const int src = check_device_status();
    if (src != ELSA_OK) return src;
    return bwd_tc3(p, out, os, row_m, row_z, workspace, static_cast<cudaStream_t>(stream));
  }
  if (use_tcw) {
    const int src = check_device_status();
    if (src != ELSA_OK) return src;
    return bwd_tcw(p, out, os, row_m, row_z, workspace, dtype, static_cast<cudaStream_t>(stream));
  }
  return bwd_simt(p, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int elsa_twopass_backward(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                     const float* row_m, const float* row_z, const float* bias, int64_t bias_stride_b,
                                     int64_t bias_stride_h, int64_t bias_stride_q, int64_t bias_stride_k, void* dq,
                                     void* dk, void* dv, float* dbias, int64_t dbias_stride_b, int64_t dbias_stride_h,
                                     int64_t dbias_stride_q, int64_t dbias_stride_k, void* workspace,
                                     int64_t workspace_bytes, int dtype, int batch, int heads, int n_ctx, int head_dim,
                                     int is_causal, unsigned flags, void* stream) {
  return backward_impl(q, k, v, out, dout, nullptr, row_m, row_z, bias, bias_stride_b, bias_stride_h, bias_stride_q,
                       bias_stride_k, dq, dk, dv, dbias, dbias_stride_b, dbias_stride_h, dbias_stride_q, dbias_stride_k,
                       workspace, workspace_bytes, dtype, batch, heads, n_ctx, head_dim, is_causal, flags, stream);
}

extern "C" int elsa_twopass_backward_strided(const void* q, const void* k, const void* v, const void* out,
                                             const void* dout, const int64_t* strides, const float* row_m,
                                             const float* row_z, const float* bias, int64_t bias_stride_b,
                                             int64_t bias_stride_h, int64_t bias_stride_q, int64_t bias_stride_k,
                                             void* dq, void* dk, void* dv, float* dbias, int64_t dbias_stride_b,
                                             int64_t dbias_stride_h, int64_t dbias_stride_q, int64_t dbias_stride_k,
                                             void* workspace, int64_t workspace_bytes, int dtype, int batch, int heads,
                                             int n_ctx, int head_dim, int is_causal, unsigned flags, void* stream) {
  if (!strides) return ELSA_ERR_INVALID_ARGUMENT;
  Strides st8[8];
  for (int i = 0; i < 8; ++i) {
    if (!strides_ok(strides + 3 * i, head_dim)) return ELSA_ERR_INVALID_ARGUMENT;
    st8[i] = to_strides(strides + 3 * i);
  }
  return backward_impl(q, k, v, out, dout, st8, row_m, row_z, bias, bias_stride_b, bias_stride_h, bias_stride_q,
                       bias_stride_k, dq, dk, dv, dbias, dbias_stride_b, dbias_stride_h, dbias_stride_q, dbias_stride_k,
                       workspace, workspace_bytes, dtype, batch, heads, n_ctx, head_dim, is_causal, flags, stream);
}

// ---- backward of one sequence shard ---------------------------------------------------------------
// k, v hold rows key_offset .. key_offset + n_keys - 1 of the sequence; q, out, dout and the GLOBAL row state
// (row_m, row_z of the merged forward) cover all n_ctx rows.  dk, dv of the shard are complete; dq is this shard's
// contribution in fp32, to be summed over the shards by the caller (all_reduce / reduce_scatter) before rounding.
extern "C" int64_t elsa_backward_shard_workspace_bytes(int dtype, int batch, int heads, int n_ctx, int head_dim,
                                                       unsigned flags) {
  // (for the fp32 tensor-core route this covers a shard of up to n_ctx keys)
  return elsa_backward_workspace_bytes(dtype, batch, heads, n_ctx, head_dim, 0, 0, flags);
}

extern "C" int elsa_twopass_backward_shard(const void* q, const void* k_shard, const void* v_shard, const void* out,
                                           const void* dout, const float* row_m, const float* row_z, float* dq_partial,
                                           void* dk_shard, void* dv_shard, void* workspace, int64_t workspace_bytes,
                                           int dtype, int batch, int heads, int n_ctx, int head_dim, int n_keys,
                                           int key_offset, int is_causal, unsigned flags, void* stream) {
  if (n_ctx == 0) return ELSA_OK;
  if (!q || !out || !dout || !row_m || !row_z || !dq_partial || !dtype_ok(dtype) || batch < 1 || heads < 1 || n_ctx < 0 ||
      head_dim < 1 || head_dim > 128 || n_keys < 0 || key_offset < 0 || (n_keys > 0 && (!k_shard || !v_shard || !dk_shard || !dv_shard)))
    return ELSA_ERR_INVALID_ARGUMENT;
  if (!aligned16(q) || !aligned16(k_shard) || !aligned16(v_shard) || !aligned16(out) || !aligned16(dout) ||
      !aligned16(dq_partial) || !aligned16(dk_shard) || !aligned16(dv_shard))
    return ELSA_ERR_INVALID_ARGUMENT;
  if (static_cast<int64_t>(batch) * heads > 65535) return ELSA_ERR_UNSUPPORTED;
  const int64_t need = elsa_backward_shard_workspace_bytes(dtype, batch, heads, n_ctx, head_dim, flags);
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < need) return ELSA_ERR_WORKSPACE;
  char* ws = static_cast<char*>(workspace);
  float* row_d = reinterpret_cast<float*>(ws);
  float* row_lse = reinterpret_cast<float*>(ws + bwd_state_bytes(batch, heads, n_ctx));
  // (the tensor-core kernels address the fp32 dQ of a shard as 64-wide rows)
  const bool use_tc = n_keys > 0 && head_dim == 64 && tc_backward_ok(dtype, head_dim, n_ctx, batch * heads, false, flags);
  const bool use_tc3 = n_keys > 0 && n_keys <= n_ctx && tc3_backward_ok(dtype, head_dim, n_ctx, batch * heads, false, flags);
  const bool use_tcw = n_keys > 0 && tcw_backward_ok(dtype, head_dim, n_ctx, batch * heads, false, flags);
  int rc = ELSA_OK;
  if (!use_tc && !use_tc3 && !use_tcw) rc = elsa_bwd_preprocess(out, dout, row_m, row_z, row_d, row_lse, dtype, batch * heads, n_ctx, head_dim, stream);
  if (rc != ELSA_OK) return rc;
  BwdParams p;
  const Strides cs = contiguous_strides(heads, n_ctx, head_dim), cks = contiguous_strides(heads, n_keys, head_dim);
  p.qs = cs; p.gs = cs; p.dqs = cs; p.ks = cks; p.vs = cks; p.dks = cks; p.dvs = cks;
  p.q = q; p.k = k_shard; p.v = v_shard; p.dout = dout;
  p.lse = row_lse; p.drow = row_d;
  p.bias = nullptr; p.bsb = p.bsh = p.bsq = p.bsk = 0;
  p.dq = dq_partial; p.dk = dk_shard; p.dv = dv_shard;
  p.dbias = nullptr; p.dsb = p.dsh = p.dsq = p.dsk = 0; p.dbias_atomic = 0;
  p.heads = heads; p.n_ctx = n_ctx; p.head_dim = head_dim; p.bh = batch * heads; p.is_causal = is_causal ? 1 : 0;
  p.scale = 1.0f / std::sqrt(static_cast<float>(head_dim));
  p.scale_log2 = static_cast<float>((1.0 / std::sqrt(static_cast<double>(head_dim))) * 1.4426950408889634);
  p.n_keys = n_keys; p.key_offset = key_offset; p.dq_f32 = 1;
  p.single_tile = 0; p.out = out; p.os = cs; p.row_m = row_m; p.row_z = row_z;
  if (use_tc) {
    const int src = check_device_status();
    if (src != ELSA_OK) return src;
    return bwd_tc(p, out, cs, row_m, row_z, workspace, dtype, static_cast<cudaStream_t>(stream));
  }
  if (use_tc3) {
    const int src = check_device_status();
    if (src != ELSA_OK) return src;
    return bwd_tc3(p, out, cs, row_m, row_z, workspace, static_cast<cudaStream_t>(stream));
  }
  if (use_tcw) {
    const int src = check_device_status();
    if (src != ELSA_OK) return src;
    return bwd_tcw(p, out, cs, row_m, row_z, workspace, dtype, static_cast<cudaStream_t>(stream));
  }
  return bwd_simt(p, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int elsa_row_stats(const void* q, const void* k, const float* bias, int64_t bias_stride_b,
                              int64_t bias_stride_h, int64_t bias_stride_q, int64_t bias_stride_k, float* row_m,
                              float* row_z, void* workspace, int64_t workspace_bytes, int dtype, int batch, int heads,
                              int n_ctx, int head_dim, int is_causal, void* stream) {
  // (m, z) do not depend on V: run the forward with V := K into a scratch output placed behind the
  // summaries in the workspace, and keep only the state.
  if (n_ctx == 0) return ELSA_OK;
  if (!row_m || !row_z) return ELSA_ERR_INVALID_ARGUMENT;
  const int64_t fwd = elsa_forward_workspace_bytes(dtype, dtype, batch, heads, n_ctx, head_dim, bias != nullptr,
                                                   is_causal, 0, 0, 0u);
  if (fwd < 0) return ELSA_ERR_INVALID_ARGUMENT;
  const int64_t out_bytes = align_up(static_cast<int64_t>(batch) * heads * n_ctx * head_dim * dtype_size(dtype), 256);
  if (!workspace || workspace_bytes < fwd + out_bytes) return ELSA_ERR_WORKSPACE;
  void* scratch_out = static_cast<char*>(workspace) + fwd;
  return elsa_twopass_forward(q, k, k, bias, bias_stride_b, bias_stride_h, bias_stride_q, bias_stride_k, scratch_out,
                              row_m, row_z, workspace, fwd, dtype, dtype, batch, heads, n_ctx, head_dim, is_causal, 0, 0,
                              0u, stream);
}

extern "C" int64_t elsa_row_stats_workspace_bytes(int dtype, int batch, int heads, int n_ctx, int head_dim,
                                                  int has_bias, int is_causal) {
  const int64_t fwd = elsa_forward_workspace_bytes(dtype, dtype, batch, heads, n_ctx, head_dim, has_bias, is_causal,
                                                   0, 0, 0u);
  if (fwd < 0) return -1;
  return fwd + align_up(static_cast<int64_t>(batch) * heads * n_ctx * head_dim * dtype_size(dtype), 256);
}

// ---- forward without any caller-supplied or freshly allocated scratch --------------------------
// (The one exception to "buffers belong to the caller" in this file.)
// Some callers have no way to hand over a workspace: a host runtime that reaches this library through a
// minimal FFI and owns no device allocator, or a serving process whose device memory was carved up once at
// start-up and whose request path is forbidden to allocate.  For them the partition summaries of the forward
// live in one fixed array inside the library image.  The price: a hard size limit, the array is resident on
// every GPU that loads the library until the process exits, and all calls share it.
namespace elsa {
constexpr int64_t kStaticScratchBytes = 64ll << 20;   // 64 MiB: covers the fp16 16K-token, 8-head forward (35.6 MB)
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the CURRENT device (in host code the symbol itself is only a handle,
// not an address a kernel could use).  Looked up once per device and remembered.
static int static_scratch_ptr(void** out) {
  static std::mutex mu;
  static void* cached[64] = {nullptr};
  int dev = 0;
  ELSA_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return ELSA_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* p = nullptr;
    ELSA_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_scratch));
    if (!p || (reinterpret_cast<uintptr_t>(p) & 255u)) return ELSA_ERR_WORKSPACE;
    cached[dev] = p;
  }
  *out = cached[dev];
  return ELSA_OK;
}
}  // namespace elsa

extern "C" int64_t elsa_static_scratch_bytes(void) { return elsa::kStaticScratchBytes; }

extern "C" int elsa_twopass_forward_static(const void* q, const void* k, const void* v, void* out, float* row_m,
                                           float* row_z, int dtype, int batch, int heads, int n_ctx, int head_dim,
                                           int is_causal, void* stream) {
  if (n_ctx == 0) return ELSA_OK;
  // same plan as elsa_twopass_forward with library-chosen partitions, no bias, summaries in the input dtype; the
  // query chunk is the largest multiple of the kernel's query tile whose summaries fit the built-in array, so a
  // long problem runs as several chunks through the same array instead of being refused
  ForwardPlan pl;
  const unsigned sflags = ELSA_FLAG_FP32_FMA;   // the planes of an fp32 problem would not fit the built-in array
  int rc0 = plan_forward(dtype, dtype, batch, heads, n_ctx, head_dim, is_causal, false, 0, 0, sflags, &pl);
  if (rc0 != ELSA_OK) return rc0;
  int q_chunk = 0;   // 0: the automatic chunk already fits
  if (plan_bytes(pl) > elsa::kStaticScratchBytes) {
    const int64_t row_bytes = static_cast<int64_t>(pl.n_parts) * batch * heads * (static_cast<int64_t>(head_dim) * dtype_size(dtype) + 8);
    int64_t rows = (elsa::kStaticScratchBytes / row_bytes) / pl.tile_m * pl.tile_m;
    for (; rows >= pl.tile_m; rows -= pl.tile_m) {
      if (plan_forward(dtype, dtype, batch, heads, n_ctx, head_dim, is_causal, false, 0, static_cast<int>(rows), sflags, &pl) != ELSA_OK)
        return ELSA_ERR_INVALID_ARGUMENT;
      if (plan_bytes(pl) <= elsa::kStaticScratchBytes) break;
    }
    if (rows < pl.tile_m) return ELSA_ERR_WORKSPACE;   // not even one query tile of summaries fits
    q_chunk = static_cast<int>(rows);
  }
  void* scratch = nullptr;
  int rc = elsa::static_scratch_ptr(&scratch);
  if (rc != ELSA_OK) return rc;
  // Nothing in the scratch has to start at zero: phase 1 writes every summary that phase 2 reads.
  return elsa_twopass_forward(q, k, v, nullptr, 0, 0, 0, 0, out, row_m, row_z, scratch, elsa::kStaticScratchBytes, dtype,
                              dtype, batch, heads, n_ctx, head_dim, is_causal, 0, q_chunk, sflags, stream);
}
