// Phase 2 of the two-pass attention: HBM-bound passes over the partition summaries.
//
//   merge_final   all partitions of a row -> out = s/z (+ row_m, row_z)       1 read of the summaries
//   prefix_scan   inclusive prefix over partitions, one read + one write
//   scan_step     one Hillis-Steele step (kept for the log-depth formulation)
//   upsweep       one Blelloch up-sweep level
//   finalize      out = s/z from one partition
//
// Layout: m, z [P][R] fp32 and s [P][R][D] (R = B*H*q_len rows).  Each thread owns NV consecutive
// elements of one row (16 bytes of s where D allows), so a warp reads whole 128-byte lines; m and
// z of a row are read by the D/NV threads of that row as a warp broadcast.
#include "kernels.cuh"

namespace elsa {

template <typename T, int NV>
__device__ __forceinline__ void load_vec(const T* __restrict__ p, float (&o)[NV]) {
  if constexpr (NV == 1) {
    o[0] = to_f32<T>(p[0]);
  } else if constexpr (NV == 4) {
    Vec4<T>::load(p, o);
  } else {
    static_assert(NV == 8, "NV");
    if constexpr (sizeof(T) == 2) {
      uint4 t = *reinterpret_cast<const uint4*>(p);
      const T* e = reinterpret_cast<const T*>(&t);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = to_f32<T>(e[i]);
    } else {
      float a[4], b[4];
      Vec4<T>::load(p, a);
      Vec4<T>::load(p + 4, b);
#pragma unroll
      for (int i = 0; i < 4; ++i) { o[i] = a[i]; o[4 + i] = b[i]; }
    }
  }
}

template <typename T, int NV>
__device__ __forceinline__ void store_vec(T* __restrict__ p, const float (&o)[NV]) {
  if constexpr (NV == 1) {
    p[0] = from_f32<T>(o[0]);
  } else if constexpr (NV == 4) {
    Vec4<T>::store(p, o);
  } else {
    if constexpr (sizeof(T) == 2) {
      uint4 t;
      T* e = reinterpret_cast<T*>(&t);
#pragma unroll
      for (int i = 0; i < 8; ++i) e[i] = from_f32<T>(o[i]);
      *reinterpret_cast<uint4*>(p) = t;
    } else {
      float a[4] = {o[0], o[1], o[2], o[3]}, b[4] = {o[4], o[5], o[6], o[7]};
      Vec4<T>::store(p, a);
      Vec4<T>::store(p + 4, b);
    }
  }
}

// Thread -> (row, 16-byte chunk of the row).  blockIdx.y is the (batch*head) index and the x dimension covers
// q_len * chunks work items, so the only division left is a 32-bit one by `chunks` (a shift for power-of-two
// head dims): 64-bit divisions per thread cost more than the memory traffic of these passes.
struct RowChunk { int64_t row; int r; int c; bool ok; };
__device__ __forceinline__ RowChunk row_chunk(int q_len, int chunks, int chunk_shift) {
  const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
  RowChunk rc;
  const uint32_t r = chunk_shift >= 0 ? (idx >> chunk_shift) : (idx / static_cast<uint32_t>(chunks));
  rc.r = static_cast<int>(r);
  rc.c = static_cast<int>(idx - r * static_cast<uint32_t>(chunks));
  rc.ok = r < static_cast<uint32_t>(q_len);
  rc.row = static_cast<int64_t>(blockIdx.y) * q_len + r;
  return rc;
}
static inline int chunk_shift_of(int chunks) {
  for (int sft = 0; sft < 16; ++sft) if ((1 << sft) == chunks) return sft;
  return -1;
}

// ---- merge_final -----------------------------------------------------------------------
template <typename TS, typename TO, int NV>
__global__ void __launch_bounds__(256)
merge_final_kernel(const float* __restrict__ m, const float* __restrict__ z, const TS* __restrict__ s,
                   TO* __restrict__ out, float* __restrict__ row_m, float* __restrict__ row_z,
                   int n_parts, int64_t rows, int q_len, int q_start, int n_ctx, int head_dim,
                   int chunks, int chunk_shift, int first_part, int store_state, int normalize, int heads, Strides os) {
  const RowChunk rc = row_chunk(q_len, chunks, chunk_shift);
  if (!rc.ok) return;
  const int64_t row = rc.row;
  const int c = rc.c;
  float M = -CUDART_INF_F, Z = 0.f, acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) acc[i] = 0.f;
  const TS* sp = s + (static_cast<int64_t>(first_part) * rows + row) * head_dim + c * NV;
  const float* mp = m + static_cast<int64_t>(first_part) * rows + row;
  const float* zp = z + static_cast<int64_t>(first_part) * rows + row;
  // the first partition initialises the state (merging it into the identity would only cost two exponentials)
  {
    float sv[NV];
    load_vec<TS, NV>(sp, sv);
    M = mp[0];
    Z = zp[0];
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[i] = Z > 0.f ? sv[i] : 0.f;
    M = Z > 0.f ? M : -CUDART_INF_F;
  }
#pragma unroll 4
  for (int p = 1; p < n_parts; ++p) {
    float sv[NV];
    load_vec<TS, NV>(sp + static_cast<int64_t>(p) * rows * head_dim, sv);
    monoid_merge<NV>(M, Z, acc, mp[static_cast<int64_t>(p) * rows], zp[static_cast<int64_t>(p) * rows], sv);
  }
  const int64_t orow = static_cast<int64_t>(blockIdx.y) * n_ctx + q_start + rc.r;
  const float inv = normalize ? (Z > 0.f ? 1.0f / Z : 0.f) : 1.0f;   // normalize == 0: emit the merged, un-normalised s
  float o[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) o[i] = Z > 0.f ? acc[i] * inv : 0.f;
  // heads == 0: out is [BH][n_ctx][head_dim] contiguous; else rows are addressed through the strides
  const int bh_i = blockIdx.y;
  const int64_t ooff = heads == 0 ? orow * head_dim
                                  : (bh_i / heads) * os.b + (bh_i % heads) * os.h + static_cast<int64_t>(q_start + rc.r) * os.r;
  store_vec<TO, NV>(out + ooff + c * NV, o);
  if (store_state && c == 0) {
    row_m[orow] = Z > 0.f ? M : -CUDART_INF_F;
    row_z[orow] = Z;
  }
}

// ---- prefix_scan -----------------------------------------------------------------------
template <typename TS, int NV>
__global__ void __launch_bounds__(256)
prefix_scan_kernel(const float* m_in, const float* z_in, const TS* s_in, float* m_out, float* z_out, TS* s_out,
                   int n_parts, int64_t rows, int q_len, int head_dim, int chunks, int chunk_shift) {
  const RowChunk rc = row_chunk(q_len, chunks, chunk_shift);
  if (!rc.ok) return;
  const int64_t row = rc.row;
  const int c = rc.c;
  float M = -CUDART_INF_F, Z = 0.f, acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) acc[i] = 0.f;
#pragma unroll 2
  for (int p = 0; p < n_parts; ++p) {
    const int64_t ro = static_cast<int64_t>(p) * rows + row;
    float sv[NV];
    load_vec<TS, NV>(s_in + ro * head_dim + c * NV, sv);
    monoid_merge<NV>(M, Z, acc, m_in[ro], z_in[ro], sv);
    // the summary buffers hold s in TS: round the running value like a stored prefix would be
    store_vec<TS, NV>(s_out + ro * head_dim + c * NV, acc);
    if constexpr (sizeof(TS) == 2) {
#pragma unroll
      for (int i = 0; i < NV; ++i) acc[i] = round_to<TS>(acc[i]);
    }
    if (c == 0) { m_out[ro] = M; z_out[ro] = Z; }
  }
}

// ---- pairwise merges (scan step, up-sweep) -----------------------------------------------
// out[po] = in[pa] (+) in[pb]; pa < 0 or pb >= n_in means "identity".
template <typename TS, int NV, bool UPSWEEP>
__global__ void __launch_bounds__(256)
pair_merge_kernel(const float* __restrict__ m_in, const float* __restrict__ z_in, const TS* __restrict__ s_in,
                  float* __restrict__ m_out, float* __restrict__ z_out, TS* __restrict__ s_out,
                  int n_in, int step, int64_t rows, int q_len, int head_dim, int chunks, int chunk_shift) {
  const RowChunk rc = row_chunk(q_len, chunks, chunk_shift);
  if (!rc.ok) return;
  const int po = blockIdx.z;
  const int64_t row = rc.row;
  const int c = rc.c;
  int pa, pb;
  if (UPSWEEP) { pa = 2 * po; pb = 2 * po + 1; } else { pa = po - step; pb = po; }
  float M = -CUDART_INF_F, Z = 0.f, acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) acc[i] = 0.f;
  if (pa >= 0 && pa < n_in) {
    const int64_t ro = static_cast<int64_t>(pa) * rows + row;
    load_vec<TS, NV>(s_in + ro * head_dim + c * NV, acc);
    M = m_in[ro];
    Z = z_in[ro];
    // a stored summary may carry (m finite, z == 0)? No: producers always store m = -inf with z = 0.
  }
  if (pb >= 0 && pb < n_in) {
    const int64_t ro = static_cast<int64_t>(pb) * rows + row;
    float sv[NV];
    load_vec<TS, NV>(s_in + ro * head_dim + c * NV, sv);
    monoid_merge<NV>(M, Z, acc, m_in[ro], z_in[ro], sv);
  } else {
    float sv[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) sv[i] = 0.f;
    monoid_merge<NV>(M, Z, acc, -CUDART_INF_F, 0.f, sv);
  }
  const int64_t wo = static_cast<int64_t>(po) * rows + row;
  store_vec<TS, NV>(s_out + wo * head_dim + c * NV, acc);
  if (c == 0) { m_out[wo] = M; z_out[wo] = Z; }
}

// ---- cross-GPU merge of sequence shards: the two local passes around the reduce_scatter ---------
// pack: w = z > 0 ? 2^(m - m_all) : 0; chunk r of `packed` = rows [r*nl, (r+1)*nl) of every (batch*head):
// s*w as [BH][nl][D] followed by z*w as [BH][nl].  One thread per float4 of s.
__global__ void __launch_bounds__(256)
shard_pack_kernel(const float* __restrict__ m, const float* __restrict__ z, const float* __restrict__ s,
                  const float* __restrict__ m_all, float* __restrict__ packed, int bh, int n_ctx, int nl,
                  int head_dim, int chunks, int64_t chunk_elems) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t rows = static_cast<int64_t>(bh) * n_ctx;
  if (idx >= rows * chunks) return;
  const int64_t row = idx / chunks;
  const int c = static_cast<int>(idx - row * chunks);
  const int64_t b = row / n_ctx;
  const int i = static_cast<int>(row - b * n_ctx);
  const int r = i / nl, il = i - r * nl;
  const float zz = z[row];
  const float w = zz > 0.f ? exp2f(m[row] - m_all[row]) : 0.f;
  float4 v = *reinterpret_cast<const float4*>(s + row * head_dim + c * 4);
  v.x *= w; v.y *= w; v.z *= w; v.w *= w;
  float* chunk = packed + static_cast<int64_t>(r) * chunk_elems;
  *reinterpret_cast<float4*>(chunk + (b * nl + il) * head_dim + c * 4) = v;
  if (c == 0) chunk[static_cast<int64_t>(bh) * nl * head_dim + b * nl + il] = zz * w;
}

// finalize: out = S / Z (0 where Z == 0), row_m = Z > 0 ? m_all : -inf, row_z = Z for the nl rows of chunk `rank`
template <typename TO>
__global__ void __launch_bounds__(256)
shard_finalize_kernel(const float* __restrict__ chunk, const float* __restrict__ m_all, TO* __restrict__ out,
                      float* __restrict__ row_m, float* __restrict__ row_z, int bh, int n_ctx, int nl, int rank,
                      int head_dim, int chunks) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t rows = static_cast<int64_t>(bh) * nl;
  if (idx >= rows * chunks) return;
  const int64_t row = idx / chunks;           // b * nl + il
  const int c = static_cast<int>(idx - row * chunks);
  const float Z = chunk[rows * head_dim + row];
  const float inv = Z > 0.f ? 1.0f / Z : 0.f;
  float sv[4], o[4];
  Vec4<float>::load(chunk + row * head_dim + c * 4, sv);
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = Z > 0.f ? sv[i] * inv : 0.f;
  Vec4<TO>::store(out + row * head_dim + c * 4, o);
  if (c == 0) {
    const int64_t b = row / nl;
    const int il = static_cast<int>(row - b * nl);
    row_m[row] = Z > 0.f ? m_all[b * n_ctx + static_cast<int64_t>(rank) * nl + il] : -CUDART_INF_F;
    row_z[row] = Z;
  }
}

// ---- dispatch ----------------------------------------------------------------------------
static inline int pick_nv(int head_dim, int elem_bytes_a, int elem_bytes_b) {
  if (head_dim % 8 == 0 && elem_bytes_a == 2 && elem_bytes_b == 2) return 8;
  if (head_dim % 4 == 0) return 4;
  return 1;
}

template <typename TS, typename TO>
static int launch_merge_final(const float* m, const float* z, const void* s, void* out, float* row_m, float* row_z,
                              int n_parts, int bh, int q_start, int q_len, int n_ctx, int head_dim,
                              int first_part, int store_state, cudaStream_t st, int normalize, int heads, Strides os) {
  const int64_t rows = static_cast<int64_t>(bh) * q_len;
  const int nv = pick_nv(head_dim, sizeof(TS), sizeof(TO));
  const int chunks = head_dim / nv;
  const dim3 blocks(static_cast<unsigned>(cdiv64(static_cast<int64_t>(q_len) * chunks, 256)), static_cast<unsigned>(bh));
  const int cs = chunk_shift_of(chunks);
  auto ts = static_cast<const TS*>(s);
  auto to = static_cast<TO*>(out);
#define ELSA_MF(NV) merge_final_kernel<TS, TO, NV><<<blocks, 256, 0, st>>>(m, z, ts, to, row_m, row_z, n_parts, rows, \
                                                   q_len, q_start, n_ctx, head_dim, chunks, cs, first_part, store_state, normalize, heads, os)
  if (nv == 8) ELSA_MF(8); else if (nv == 4) ELSA_MF(4); else ELSA_MF(1);
#undef ELSA_MF
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

int merge_final_any(const float* m, const float* z, const void* s, void* out, float* row_m, float* row_z,
                           int summary_dtype, int out_dtype, int n_parts, int bh, int q_start, int q_len, int n_ctx,
                           int head_dim, int first_part, int store_state, cudaStream_t st, int normalize, int heads,
                           const Strides* out_strides) {
  const int heads_k = out_strides ? heads : 0;
  const Strides os = out_strides ? *out_strides : Strides{0, 0, 0};
  if (out_strides && (heads < 1 || bh % heads != 0)) return ELSA_ERR_INVALID_ARGUMENT;
  if (!dtype_ok(summary_dtype) || !dtype_ok(out_dtype)) return ELSA_ERR_INVALID_ARGUMENT;
  if (!m || !z || !s || !out || n_parts < 1 || bh < 1 || q_len < 0 || head_dim < 1 || head_dim > 128 ||
      q_start < 0 || q_start + q_len > n_ctx || first_part < 0)
    return ELSA_ERR_INVALID_ARGUMENT;
  if (store_state && (!row_m || !row_z)) return ELSA_ERR_INVALID_ARGUMENT;
  if (q_len == 0) return ELSA_OK;
#define ELSA_CASE(SD, OD, TS, TO)                 \
  if (summary_dtype == SD && out_dtype == OD)     \
    return launch_merge_final<TS, TO>(m, z, s, out, row_m, row_z, n_parts, bh, q_start, q_len, n_ctx, head_dim, \
                                      first_part, store_state, st, normalize, heads_k, os)
  ELSA_CASE(ELSA_F32, ELSA_F32, float, float);
  ELSA_CASE(ELSA_F16, ELSA_F16, __half, __half);
  ELSA_CASE(ELSA_BF16, ELSA_BF16, __nv_bfloat16, __nv_bfloat16);
  ELSA_CASE(ELSA_F32, ELSA_F16, float, __half);
  ELSA_CASE(ELSA_F32, ELSA_BF16, float, __nv_bfloat16);
  ELSA_CASE(ELSA_F16, ELSA_F32, __half, float);
  ELSA_CASE(ELSA_BF16, ELSA_F32, __nv_bfloat16, float);
  ELSA_CASE(ELSA_F16, ELSA_BF16, __half, __nv_bfloat16);
  ELSA_CASE(ELSA_BF16, ELSA_F16, __nv_bfloat16, __half);
#undef ELSA_CASE
  return ELSA_ERR_UNSUPPORTED;
}

template <typename TS>
static int launch_pair(const float* m_in, const float* z_in, const void* s_in, float* m_out, float* z_out, void* s_out,
                       int n_in, int n_out, int step, bool upsweep, int bh, int q_len, int head_dim, cudaStream_t st) {
  const int64_t rows = static_cast<int64_t>(bh) * q_len;
  const int nv = pick_nv(head_dim, sizeof(TS), sizeof(TS));
  const int chunks = head_dim / nv;
  dim3 grid(static_cast<unsigned>(cdiv64(static_cast<int64_t>(q_len) * chunks, 256)), static_cast<unsigned>(bh),
            static_cast<unsigned>(n_out));
  const int cs = chunk_shift_of(chunks);
  auto si = static_cast<const TS*>(s_in);
  auto so = static_cast<TS*>(s_out);
#define ELSA_PM(NV, UP) pair_merge_kernel<TS, NV, UP><<<grid, 256, 0, st>>>(m_in, z_in, si, m_out, z_out, so, n_in, step, \
                                                                          rows, q_len, head_dim, chunks, cs)
  if (upsweep) { if (nv == 8) ELSA_PM(8, true); else if (nv == 4) ELSA_PM(4, true); else ELSA_PM(1, true); }
  else         { if (nv == 8) ELSA_PM(8, false); else if (nv == 4) ELSA_PM(4, false); else ELSA_PM(1, false); }
#undef ELSA_PM
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

template <typename TS>
static int launch_prefix(const float* m_in, const float* z_in, const void* s_in, float* m_out, float* z_out,
                         void* s_out, int n_parts, int bh, int q_len, int head_dim, cudaStream_t st) {
  const int64_t rows = static_cast<int64_t>(bh) * q_len;
  const int nv = pick_nv(head_dim, sizeof(TS), sizeof(TS));
  const int chunks = head_dim / nv;
  const dim3 blocks(static_cast<unsigned>(cdiv64(static_cast<int64_t>(q_len) * chunks, 256)), static_cast<unsigned>(bh));
  const int cs = chunk_shift_of(chunks);
  auto si = static_cast<const TS*>(s_in);
  auto so = static_cast<TS*>(s_out);
#define ELSA_PS(NV) prefix_scan_kernel<TS, NV><<<blocks, 256, 0, st>>>(m_in, z_in, si, m_out, z_out, so, n_parts, rows, \
                                                                     q_len, head_dim, chunks, cs)
  if (nv == 8) ELSA_PS(8); else if (nv == 4) ELSA_PS(4); else ELSA_PS(1);
#undef ELSA_PS
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

// q' = q * c with c rounded to fp16 and the product formed and rounded in fp16 (8 elements per thread)
__global__ void __launch_bounds__(256) prescale_q_f16_kernel(const uint4* __restrict__ q, uint4* __restrict__ o, int64_t n_vec, __half c) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  uint4 v = q[i];
  __half2* h = reinterpret_cast<__half2*>(&v);
  const __half2 c2 = __half2half2(c);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __hmul2(h[j], c2);
  o[i] = v;
}

int prescale_q_f16(const void* q, void* q_scaled, int64_t n_elems, float c, cudaStream_t st) {
  if (n_elems % 8 != 0) return ELSA_ERR_INVALID_ARGUMENT;
  const int64_t n_vec = n_elems / 8;
  prescale_q_f16_kernel<<<static_cast<unsigned>(cdiv64(n_vec, 256)), 256, 0, st>>>(
      static_cast<const uint4*>(q), static_cast<uint4*>(q_scaled), n_vec, __float2half_rn(c));
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

static bool summary_args_ok(const void* a, const void* b, const void* c, const void* d, const void* e, const void* f,
                            int summary_dtype, int n, int bh, int q_len, int head_dim) {
  return a && b && c && d && e && f && dtype_ok(summary_dtype) && n >= 1 && bh >= 1 && q_len >= 0 && head_dim >= 1 &&
         head_dim <= 128;
}

}  // namespace elsa

using namespace elsa;

extern "C" int elsa_merge_final(const float* m_buf, const float* z_buf, const void* s_buf, void* out, float* row_m,
                                float* row_z, int summary_dtype, int out_dtype, int n_parts, int bh, int q_start,
                                int q_len, int n_ctx, int head_dim, int store_state, void* stream) {
  return merge_final_any(m_buf, z_buf, s_buf, out, row_m, row_z, summary_dtype, out_dtype, n_parts, bh, q_start, q_len,
                         n_ctx, head_dim, 0, store_state, static_cast<cudaStream_t>(stream));
}

extern "C" int elsa_finalize(const float* m_buf, const float* z_buf, const void* s_buf, void* out, float* row_m,
                             float* row_z, int summary_dtype, int out_dtype, int final_part, int bh, int q_start,
                             int q_len, int n_ctx, int head_dim, int store_state, void* stream) {
  // finalising partition `final_part` is a one-partition merge starting there
  return merge_final_any(m_buf, z_buf, s_buf, out, row_m, row_z, summary_dtype, out_dtype, 1, bh, q_start, q_len, n_ctx,
                         head_dim, final_part, store_state, static_cast<cudaStream_t>(stream));
}

extern "C" int elsa_scan_step(const float* m_in, const float* z_in, const void* s_in, float* m_out, float* z_out,
                              void* s_out, int summary_dtype, int n_parts, int bh, int q_len, int head_dim, int step,
                              void* stream) {
  if (!summary_args_ok(m_in, z_in, s_in, m_out, z_out, s_out, summary_dtype, n_parts, bh, q_len, head_dim) || step < 1)
    return ELSA_ERR_INVALID_ARGUMENT;
  if (m_in == m_out || s_in == s_out) return ELSA_ERR_INVALID_ARGUMENT;  // a step reads p-step after p may be written
  if (q_len == 0) return ELSA_OK;
  auto st = static_cast<cudaStream_t>(stream);
  if (summary_dtype == ELSA_F32) return launch_pair<float>(m_in, z_in, s_in, m_out, z_out, s_out, n_parts, n_parts, step, false, bh, q_len, head_dim, st);
  if (summary_dtype == ELSA_F16) return launch_pair<__half>(m_in, z_in, s_in, m_out, z_out, s_out, n_parts, n_parts, step, false, bh, q_len, head_dim, st);
  return launch_pair<__nv_bfloat16>(m_in, z_in, s_in, m_out, z_out, s_out, n_parts, n_parts, step, false, bh, q_len, head_dim, st);
}

extern "C" int elsa_upsweep_level(const float* m_in, const float* z_in, const void* s_in, float* m_out, float* z_out,
                                  void* s_out, int summary_dtype, int n_in, int bh, int q_len, int head_dim,
                                  void* stream) {
  if (!summary_args_ok(m_in, z_in, s_in, m_out, z_out, s_out, summary_dtype, n_in, bh, q_len, head_dim))
    return ELSA_ERR_INVALID_ARGUMENT;
  if (m_in == m_out || s_in == s_out) return ELSA_ERR_INVALID_ARGUMENT;
  if (q_len == 0) return ELSA_OK;
  auto st = static_cast<cudaStream_t>(stream);
  const int n_out = (n_in + 1) / 2;
  if (summary_dtype == ELSA_F32) return launch_pair<float>(m_in, z_in, s_in, m_out, z_out, s_out, n_in, n_out, 0, true, bh, q_len, head_dim, st);
  if (summary_dtype == ELSA_F16) return launch_pair<__half>(m_in, z_in, s_in, m_out, z_out, s_out, n_in, n_out, 0, true, bh, q_len, head_dim, st);
  return launch_pair<__nv_bfloat16>(m_in, z_in, s_in, m_out, z_out, s_out, n_in, n_out, 0, true, bh, q_len, head_dim, st);
}

extern "C" int elsa_prefix_scan(const float* m_in, const float* z_in, const void* s_in, float* m_out, float* z_out,
                                void* s_out, int summary_dtype, int n_parts, int bh, int q_len, int head_dim,
                                void* stream) {
  if (!summary_args_ok(m_in, z_in, s_in, m_out, z_out, s_out, summary_dtype, n_parts, bh, q_len, head_dim))
    return ELSA_ERR_INVALID_ARGUMENT;
  if (m_in == m_out || z_in == z_out || s_in == s_out) return ELSA_ERR_INVALID_ARGUMENT;
  if (q_len == 0) return ELSA_OK;
  auto st = static_cast<cudaStream_t>(stream);
  if (summary_dtype == ELSA_F32) return launch_prefix<float>(m_in, z_in, s_in, m_out, z_out, s_out, n_parts, bh, q_len, head_dim, st);
  if (summary_dtype == ELSA_F16) return launch_prefix<__half>(m_in, z_in, s_in, m_out, z_out, s_out, n_parts, bh, q_len, head_dim, st);
  return launch_prefix<__nv_bfloat16>(m_in, z_in, s_in, m_out, z_out, s_out, n_parts, bh, q_len, head_dim, st);
}

extern "C" int elsa_merge_partial(const float* m_buf, const float* z_buf, const void* s_buf, float* s_out, float* m_out,
                                  float* z_out, int summary_dtype, int n_parts, int bh, int q_len, int head_dim,
                                  void* stream) {
  // one un-normalised fp32 summary per row: the state a sequence shard contributes to the cross-GPU merge
  return merge_final_any(m_buf, z_buf, s_buf, s_out, m_out, z_out, summary_dtype, ELSA_F32, n_parts, bh, 0, q_len, q_len,
                         head_dim, 0, 1, static_cast<cudaStream_t>(stream), 0);
}

extern "C" int64_t elsa_shard_chunk_elems(int bh, int n_ctx, int head_dim, int world) {
  if (bh < 1 || n_ctx < 1 || head_dim < 1 || world < 1 || n_ctx % world != 0) return -1;
  return static_cast<int64_t>(bh) * (n_ctx / world) * (head_dim + 1);
}

extern "C" int elsa_shard_pack(const float* m, const float* z, const float* s, const float* m_all, float* packed, int bh,
                               int n_ctx, int head_dim, int world, void* stream) {
  if (!m || !z || !s || !m_all || !packed || bh < 1 || n_ctx < 1 || head_dim < 4 || head_dim > 128 || head_dim % 4 != 0 ||
      world < 1 || n_ctx % world != 0)
    return ELSA_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(packed)) & 15u) return ELSA_ERR_INVALID_ARGUMENT;
  const int nl = n_ctx / world, chunks = head_dim / 4;
  const int64_t chunk_elems = static_cast<int64_t>(bh) * nl * (head_dim + 1);
  if (world > 1 && (chunk_elems * 4) % 16 != 0) return ELSA_ERR_INVALID_ARGUMENT;   // chunk bases stay 16-byte aligned
  const int64_t total = static_cast<int64_t>(bh) * n_ctx * chunks;
  shard_pack_kernel<<<static_cast<unsigned>(cdiv64(total, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      m, z, s, m_all, packed, bh, n_ctx, nl, head_dim, chunks, chunk_elems);
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

extern "C" int elsa_shard_finalize(const float* chunk, const float* m_all, void* out, float* row_m, float* row_z,
                                   int out_dtype, int bh, int n_ctx, int head_dim, int world, int rank, void* stream) {
  if (!chunk || !m_all || !out || !row_m || !row_z || !dtype_ok(out_dtype) || bh < 1 || n_ctx < 1 || head_dim < 4 ||
      head_dim > 128 || head_dim % 4 != 0 || world < 1 || n_ctx % world != 0 || rank < 0 || rank >= world)
    return ELSA_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(chunk) | reinterpret_cast<uintptr_t>(out)) & 15u) return ELSA_ERR_INVALID_ARGUMENT;
  const int nl = n_ctx / world, chunks = head_dim / 4;
  const int64_t total = static_cast<int64_t>(bh) * nl * chunks;
  const unsigned blocks = static_cast<unsigned>(cdiv64(total, 256));
  auto st = static_cast<cudaStream_t>(stream);
  if (out_dtype == ELSA_F32)
    shard_finalize_kernel<float><<<blocks, 256, 0, st>>>(chunk, m_all, static_cast<float*>(out), row_m, row_z, bh, n_ctx, nl, rank, head_dim, chunks);
  else if (out_dtype == ELSA_F16)
    shard_finalize_kernel<__half><<<blocks, 256, 0, st>>>(chunk, m_all, static_cast<__half*>(out), row_m, row_z, bh, n_ctx, nl, rank, head_dim, chunks);
  else
    shard_finalize_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(chunk, m_all, static_cast<__nv_bfloat16*>(out), row_m, row_z, bh, n_ctx, nl, rank, head_dim, chunks);
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}
