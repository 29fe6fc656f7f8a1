// Phase 1 on the FP32-FMA pipe: the generic per-K-partition (m, z, s) fold.
//
// Covers what the tcgen05 kernel does not: fp32 inputs (exact FP32 FMA instead of 3xTF32),
// additive bias, head dims other than 64, and short / ragged problems.  One CTA of 256 threads
// (16 x 16) owns 64 query rows of one (batch*head) and one K partition; it walks the partition
// in 64-key tiles, keeps the running (m, z, s) of its rows in registers and merges each tile
// with the exp-rescale rule, then writes ONE summary per row to global memory.
//
// Shared memory (fp32, converted on load): Q[64][DP+4], K[64][DP+4], V[64][DP], P[64][68].
// The +4 padding makes the float4 reads of 8 consecutive rows hit 32 distinct banks.
#include "kernels.cuh"
#include "simt_tile.cuh"

namespace elsa {

template <typename T, int DP>
__global__ void __launch_bounds__(256, (DP == 32 ? ELSA_FOLD_MIN_CTAS_D32 : (DP == 64 ? ELSA_FOLD_MIN_CTAS_D64 : 1)))
fold_simt_kernel(const FoldParams prm) {
  constexpr int LD = DP + 4;
  constexpr int CPT = DP / 16;
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem;
  float* Ks = Qs + 64 * LD;
  float* Vs = Ks + 64 * LD;
  float* Ps = Vs + 64 * DP;

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int bh = blockIdx.z, part = blockIdx.y, qt = blockIdx.x;
  const int D = prm.head_dim, N = prm.n_ctx;
  const int q0 = prm.q_start + qt * 64;
  const int q_end = prm.q_start + prm.q_len;
  const int rows_valid = min(64, q_end - q0);
  const int k_begin = part * prm.part_width;
  const int koff = prm.key_offset;       // global index of local key 0
  int k_end = min(prm.n_keys, k_begin + prm.part_width);
  if (prm.is_causal) k_end = min(k_end, q0 + rows_valid - koff);  // keys beyond the tile's last row are masked for every row

  const int b = bh / prm.heads, h = bh - b * prm.heads;
  const T* qb = static_cast<const T*>(prm.q) + b * prm.qs.b + h * prm.qs.h;
  const T* kb = static_cast<const T*>(prm.k) + b * prm.ks.b + h * prm.ks.h;
  const T* vb = static_cast<const T*>(prm.v) + b * prm.vs.b + h * prm.vs.h;
  // vector loads need every row start on a vector boundary (the host only passes such strides with D % 4 == 0)
  const bool vec_ok = (D % 4) == 0 && ((prm.qs.r | prm.ks.r | prm.vs.r | prm.qs.h | prm.ks.h | prm.vs.h | prm.qs.b | prm.ks.b | prm.vs.b) % 4) == 0;
  const float* bias_bh = nullptr;
  if (prm.bias) bias_bh = prm.bias + b * prm.bsb + h * prm.bsh;

  load_tile<T, DP>(Qs, LD, qb + static_cast<int64_t>(q0) * prm.qs.r, prm.qs.r, rows_valid, D, vec_ok, tid);

  float m_run[4], z_part[4], acc[4][CPT];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m_run[i] = -CUDART_INF_F;
    z_part[i] = 0.f;
#pragma unroll
    for (int c = 0; c < CPT; ++c) acc[i][c] = 0.f;
  }

  for (int k0 = k_begin; k0 < k_end; k0 += 64) {
    __syncthreads();  // previous tile's PV has finished reading V and P
    const int kv = min(64, k_end - k0);
    load_tile<T, DP>(Ks, LD, kb + static_cast<int64_t>(k0) * prm.ks.r, prm.ks.r, kv, D, vec_ok, tid);
    load_tile<T, DP>(Vs, DP, vb + static_cast<int64_t>(k0) * prm.vs.r, prm.vs.r, kv, D, vec_ok, tid);
    __syncthreads();

    float S[4][4];
    tile_dot<DP>(Qs, Ks, LD, ty, tx, S);

    float lmax[4];
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const int qi = q0 + ty * 4 + ii;
      lmax[ii] = -CUDART_INF_F;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int kj = k0 + tx + 16 * jj;
        bool valid = kj < k_end && qi < q_end;
        if (prm.is_causal) valid = valid && (qi >= kj + koff);
        float sc;
        if (bias_bh) {
          float bv = valid ? bias_bh[static_cast<int64_t>(qi) * prm.bsq + static_cast<int64_t>(kj + koff) * prm.bsk] : 0.f;
          sc = (S[ii][jj] * prm.scale + bv) * kLog2e;
        } else {
          sc = S[ii][jj] * prm.scale_log2;
        }
        sc = valid ? sc : -CUDART_INF_F;
        S[ii][jj] = sc;
        lmax[ii] = fmaxf(lmax[ii], sc);
      }
    }
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
#pragma unroll
      for (int o = 8; o >= 1; o >>= 1) lmax[ii] = fmaxf(lmax[ii], __shfl_xor_sync(0xffffffffu, lmax[ii], o));
      const float m_new = fmaxf(m_run[ii], lmax[ii]);
      const float m_safe = (m_new == -CUDART_INF_F) ? 0.f : m_new;
      const float alpha = exp2f(m_run[ii] - m_safe);  // 0 when nothing has been seen yet
      float psum = 0.f;
      float pv[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const float p = exp2f(S[ii][jj] - m_safe);
        psum += p;
        pv[jj] = prm.round_p == 1 ? round_to<__half>(p) : (prm.round_p == 2 ? round_to<__nv_bfloat16>(p) : p);
      }
      z_part[ii] = z_part[ii] * alpha + psum;
#pragma unroll
      for (int c = 0; c < CPT; ++c) acc[ii][c] *= alpha;
      m_run[ii] = m_new;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) Ps[(ty * 4 + ii) * 68 + tx + 16 * jj] = pv[jj];
    }
    __syncthreads();
    tile_pv<DP>(Ps, Vs, DP, ty, tx, acc);
  }

  if (prm.direct) {
    // one partition, so (m, z, s) is the row's final state: out = s / z (0 for a row without admissible keys)
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      float zsum = z_part[ii];
#pragma unroll
      for (int o = 8; o >= 1; o >>= 1) zsum += __shfl_xor_sync(0xffffffffu, zsum, o);
      const int qi = q0 + ty * 4 + ii;
      if (qi >= q_end) continue;
      const float inv = zsum > 0.f ? 1.0f / zsum : 0.f;
      if (tx == 0 && prm.row_m) {
        prm.row_m[static_cast<int64_t>(bh) * N + qi] = zsum > 0.f ? m_run[ii] : -CUDART_INF_F;
        prm.row_z[static_cast<int64_t>(bh) * N + qi] = zsum;
      }
      T* orow = static_cast<T*>(prm.out) + b * prm.os.b + h * prm.os.h + static_cast<int64_t>(qi) * prm.os.r;
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        const int col = tile_col<DP>(tx, c);
        if (col >= D) continue;
        // same rounding points as the two-pass route: s is rounded to the summary type before the division
        float sval = acc[ii][c];
        if (prm.summary_dtype == ELSA_F16) sval = round_to<__half>(sval);
        else if (prm.summary_dtype == ELSA_BF16) sval = round_to<__nv_bfloat16>(sval);
        orow[col] = from_f32<T>(zsum > 0.f ? sval * inv : 0.f);
      }
    }
    return;
  }

  // write the partition summary
  const int64_t row_base = (static_cast<int64_t>(part) * prm.bh + bh) * prm.q_len;
#pragma unroll
  for (int ii = 0; ii < 4; ++ii) {
    float zsum = z_part[ii];
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) zsum += __shfl_xor_sync(0xffffffffu, zsum, o);
    const int r = qt * 64 + ty * 4 + ii;
    if (r >= prm.q_len) continue;
    const int64_t ro = row_base + r;
    if (tx == 0) {
      prm.m[ro] = zsum > 0.f ? m_run[ii] : -CUDART_INF_F;
      prm.z[ro] = zsum;
    }
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int col = tile_col<DP>(tx, c);
      if (col < D) {
        const float val = acc[ii][c];
        if (prm.summary_dtype == ELSA_F32) static_cast<float*>(prm.s)[ro * D + col] = val;
        else if (prm.summary_dtype == ELSA_F16) static_cast<__half*>(prm.s)[ro * D + col] = __float2half_rn(val);
        else static_cast<__nv_bfloat16*>(prm.s)[ro * D + col] = __float2bfloat16_rn(val);
      }
    }
  }
}

template <typename T, int DP>
static int launch_fold(const FoldParams& p, cudaStream_t st) {
  constexpr size_t smem = sizeof(float) * (2 * 64 * (DP + 4) + 64 * DP + 64 * 68);
  int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&fold_simt_kernel<T, DP>), smem);
  if (rc != ELSA_OK) return rc;
  dim3 grid(static_cast<unsigned>((p.q_len + 63) / 64), static_cast<unsigned>(p.n_parts), static_cast<unsigned>(p.bh));
  fold_simt_kernel<T, DP><<<grid, 256, smem, st>>>(p);
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

int fold_simt(const FoldParams& p, int dtype, cudaStream_t st) {
  const int dp = p.head_dim <= 32 ? 32 : (p.head_dim <= 64 ? 64 : 128);
#define ELSA_FOLD(T)                                  \
  do {                                                \
    if (dp == 32) return launch_fold<T, 32>(p, st);   \
    if (dp == 64) return launch_fold<T, 64>(p, st);   \
    return launch_fold<T, 128>(p, st);                \
  } while (0)
  if (dtype == ELSA_F32) ELSA_FOLD(float);
  if (dtype == ELSA_F16) ELSA_FOLD(__half);
  ELSA_FOLD(__nv_bfloat16);
#undef ELSA_FOLD
}

}  // namespace elsa
