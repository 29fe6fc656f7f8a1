// Register-tiled 64x64 building blocks shared by the FP32-FMA forward and backward kernels.
// Thread (ty, tx) of a 16x16 CTA owns rows ty*4+{0..3}; in a score tile it owns columns
// tx+16*{0..3}, in an output tile [64][DP] it owns the columns given by tile_col().
#pragma once

#include "kernels.cuh"

// Minimum resident CTAs per SM the FP32-FMA kernels are compiled for (this bounds the registers per thread).
// Measured on B200 (CUDA-graph replays, microseconds): the forward gains from three or four CTAs per SM (fp32
// N = 4096: 1155 -> 1050 at head dim 64; 49-token windows at head dim 32: 84 -> 47), the head-dim-32 backward from
// three (246 -> 162), while the head-dim-64 backward loses when squeezed below 128 registers (2710 -> 3360).
#ifndef ELSA_FOLD_MIN_CTAS_D32
#define ELSA_FOLD_MIN_CTAS_D32 4
#endif
#ifndef ELSA_FOLD_MIN_CTAS_D64
#define ELSA_FOLD_MIN_CTAS_D64 3
#endif
#ifndef ELSA_BWD_MIN_CTAS_D32
#define ELSA_BWD_MIN_CTAS_D32 3
#endif
#ifndef ELSA_BWD_MIN_CTAS_D64
#define ELSA_BWD_MIN_CTAS_D64 2
#endif

namespace elsa {

// global rows of D elements of T, `src_ld` elements apart  ->  shared fp32 [64][ld], zero-filled beyond rows_valid
// and beyond D
template <typename T, int DP>
__device__ __forceinline__ void load_tile(float* __restrict__ dst, int ld, const T* __restrict__ src, int64_t src_ld,
                                          int rows_valid, int D, bool vec_ok, int tid) {
  constexpr int C4 = DP / 4;
#pragma unroll 2
  for (int idx = tid; idx < 64 * C4; idx += 256) {
    const int r = idx / C4;
    const int c = (idx - r * C4) * 4;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (r < rows_valid) {
      const T* p = src + static_cast<int64_t>(r) * src_ld + c;
      if (vec_ok && c + 3 < D) {
        Vec4<T>::load(p, v);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (c + e < D) v[e] = to_f32<T>(p[e]);
      }
    }
    *reinterpret_cast<float4*>(dst + r * ld + c) = make_float4(v[0], v[1], v[2], v[3]);
  }
}

// S[ii][jj] = sum_d A[ty*4+ii][d] * B[tx+16*jj][d]
template <int DP>
__device__ __forceinline__ void tile_dot(const float* __restrict__ A, const float* __restrict__ B, int ld, int ty,
                                         int tx, float (&S)[4][4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) S[i][j] = 0.f;
#pragma unroll 4
  for (int d = 0; d < DP; d += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4*>(A + (ty * 4 + i) * ld + d);
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = *reinterpret_cast<const float4*>(B + (tx + 16 * j) * ld + d);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        S[i][j] = fmaf(a[i].x, b[j].x, S[i][j]);
        S[i][j] = fmaf(a[i].y, b[j].y, S[i][j]);
        S[i][j] = fmaf(a[i].z, b[j].z, S[i][j]);
        S[i][j] = fmaf(a[i].w, b[j].w, S[i][j]);
      }
  }
}

// column of output element c (0..DP/16-1) owned by lane tx
template <int DP>
__device__ __forceinline__ int tile_col(int tx, int c) {
  if constexpr (DP == 32) return tx * 2 + c;
  else if constexpr (DP == 64) return tx * 4 + c;
  else return (c >> 2) * 64 + tx * 4 + (c & 3);
}

// acc[ii][c] += sum_j P[ty*4+ii][j] * V[j][col(c)],  P is [64][68], V is [64][ldv]
template <int DP>
__device__ __forceinline__ void tile_pv(const float* __restrict__ P, const float* __restrict__ V, int ldv, int ty,
                                        int tx, float (&acc)[4][DP / 16]) {
  constexpr int CPT = DP / 16;
#pragma unroll 2
  for (int j = 0; j < 64; j += 4) {
    float4 pr[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pr[i] = *reinterpret_cast<const float4*>(P + (ty * 4 + i) * 68 + j);
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      float vv[CPT];
      const float* vr = V + (j + jj) * ldv;
      if constexpr (DP == 32) {
        float2 t = *reinterpret_cast<const float2*>(vr + tx * 2);
        vv[0] = t.x; vv[1] = t.y;
      } else {
#pragma unroll
        for (int g = 0; g < CPT / 4; ++g) {
          float4 t = *reinterpret_cast<const float4*>(vr + g * 64 + tx * 4);
          vv[g * 4 + 0] = t.x; vv[g * 4 + 1] = t.y; vv[g * 4 + 2] = t.z; vv[g * 4 + 3] = t.w;
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float pij = jj == 0 ? pr[i].x : (jj == 1 ? pr[i].y : (jj == 2 ? pr[i].z : pr[i].w));
#pragma unroll
        for (int c = 0; c < CPT; ++c) acc[i][c] = fmaf(pij, vv[c], acc[i][c]);
      }
    }
  }
}

// acc[ii][c] += sum_j PT[j][ty*4+ii] * V[j][col(c)]: as tile_pv with the left operand stored transposed
// (PT is [64][68], row = the contraction index), so the four rows of a thread come from one float4
template <int DP>
__device__ __forceinline__ void tile_ptv(const float* __restrict__ PT, const float* __restrict__ V, int ldv, int ty,
                                         int tx, float (&acc)[4][DP / 16]) {
  constexpr int CPT = DP / 16;
#pragma unroll 4
  for (int j = 0; j < 64; ++j) {
    const float4 p4 = *reinterpret_cast<const float4*>(PT + j * 68 + ty * 4);
    float vv[CPT];
    const float* vr = V + j * ldv;
    if constexpr (DP == 32) {
      float2 t = *reinterpret_cast<const float2*>(vr + tx * 2);
      vv[0] = t.x; vv[1] = t.y;
    } else {
#pragma unroll
      for (int g = 0; g < CPT / 4; ++g) {
        float4 t = *reinterpret_cast<const float4*>(vr + g * 64 + tx * 4);
        vv[g * 4 + 0] = t.x; vv[g * 4 + 1] = t.y; vv[g * 4 + 2] = t.z; vv[g * 4 + 3] = t.w;
      }
    }
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      acc[0][c] = fmaf(p4.x, vv[c], acc[0][c]);
      acc[1][c] = fmaf(p4.y, vv[c], acc[1][c]);
      acc[2][c] = fmaf(p4.z, vv[c], acc[2][c]);
      acc[3][c] = fmaf(p4.w, vv[c], acc[3][c]);
    }
  }
}

}  // namespace elsa
