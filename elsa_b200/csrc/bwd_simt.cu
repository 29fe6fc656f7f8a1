// Backward on the FP32-FMA pipe: exact recompute from the saved row statistics.
//
//   bwd_preprocess   D = sum_d out*dout, LSE = m + log2(max(z, 1e-30))        (HBM pass)
//   bwd_simt<MODE 0> one CTA per 64 query rows, streams key tiles:  dQ (+ dbias)
//   bwd_simt<MODE 1> one CTA per 64 key rows,   streams query tiles: dK, dV
//
//   bwd_simt<MODE 3> the whole problem is ONE (query tile, key tile) pair (n_ctx <= 64: 49-token windows): one launch
//                    forms D and LSE from out, dout and the row state, computes S and dP once and all of dQ, dK,
//                    dV (and dbias) from them -- five contractions, no atomics, no separate pre-pass
//   bwd_simt<MODE 2> MODE 1 plus dQ: the dQ contribution of each (key tile, query tile) pair, dS K, is formed from
//                    the dS^T tile that is already in shared memory and added into an fp32 dQ with vector
//                    reductions -- five contractions per pair instead of the seven of MODE 0 + MODE 1 (which
//                    compute S and dP twice).  Used where dQ is fp32 anyway (fp32 inputs, sequence shards) and no
//                    bias gradient is wanted; the order of the additions into dQ is then not fixed.
//
// All modes are the same register-tiled code with the operand roles swapped: the "row" operands
// stay in shared memory for the whole CTA, the "column" operands are streamed in 64-row tiles.
// MODE 1 / 2 compute the transposed tiles S^T = K Q^T and dP^T = V dO^T directly, so P^T and dS^T are
// produced in the layout the dV / dK contractions consume.  MODE 0 + MODE 1 use no atomics: bit-reproducible.
#include "kernels.cuh"
#include "simt_tile.cuh"

namespace elsa {

// global[0..3] += {a, b, c, d} as one 16-byte vector reduction (the address must be 16-byte aligned)
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <typename T, int DP, int MODE>
__global__ void __launch_bounds__(256, (DP == 32 ? ELSA_BWD_MIN_CTAS_D32 : (DP == 64 ? ELSA_BWD_MIN_CTAS_D64 : 1)))
bwd_simt_kernel(const BwdParams prm) {
  constexpr int LD = DP + 4;
  constexpr int CPT = DP / 16;
  constexpr bool QROWS = MODE == 0 || MODE == 3;   // the CTA's resident rows are queries (else keys)
  extern __shared__ __align__(16) float smem[];
  float* RA = smem;             // MODE 0: Q rows     MODE 1: K rows
  float* RB = RA + 64 * LD;     // MODE 0: dO rows    MODE 1: V rows
  float* CA = RB + 64 * LD;     // MODE 0: K tile     MODE 1: Q tile
  float* CB = CA + 64 * LD;     // MODE 0: V tile     MODE 1: dO tile
  float* Ps = CB + 64 * LD;     // MODE 0: dS         MODE 1: P^T
  float* Ss = Ps + 64 * 68;     //                    MODE 1: dS^T

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int bh = blockIdx.y;
  const int D = prm.head_dim, N = prm.n_ctx, NK = prm.n_keys, koff = prm.key_offset;
  const int NR = QROWS ? N : NK;       // rows of this launch: queries (dQ) or local keys (dK, dV)
  const int NC = QROWS ? NK : N;       // columns walked by the loop
  const int r0 = blockIdx.x * 64;
  const int rows_valid = min(64, NR - r0);
  const int b = bh / prm.heads, h = bh - b * prm.heads;
  const T* qb = static_cast<const T*>(prm.q) + b * prm.qs.b + h * prm.qs.h;
  const T* kb = static_cast<const T*>(prm.k) + b * prm.ks.b + h * prm.ks.h;
  const T* vb = static_cast<const T*>(prm.v) + b * prm.vs.b + h * prm.vs.h;
  const T* gb = static_cast<const T*>(prm.dout) + b * prm.gs.b + h * prm.gs.h;
  const int64_t ra_ld = QROWS ? prm.qs.r : prm.ks.r, rb_ld = QROWS ? prm.gs.r : prm.vs.r;   // resident operands
  const int64_t ca_ld = QROWS ? prm.ks.r : prm.qs.r, cb_ld = QROWS ? prm.vs.r : prm.gs.r;   // streamed operands
  const float* lse = prm.lse + static_cast<int64_t>(bh) * N;
  const float* drow = prm.drow + static_cast<int64_t>(bh) * N;
  const bool vec_ok = (D % 4) == 0 && ((prm.qs.r | prm.ks.r | prm.vs.r | prm.gs.r | prm.qs.h | prm.ks.h | prm.vs.h | prm.gs.h |
                                        prm.qs.b | prm.ks.b | prm.vs.b | prm.gs.b) % 4) == 0;
  const float* bias_bh = prm.bias ? prm.bias + b * prm.bsb + h * prm.bsh : nullptr;
  float* dbias_bh = (QROWS && prm.dbias) ? prm.dbias + b * prm.dsb + h * prm.dsh : nullptr;

  load_tile<T, DP>(RA, LD, (QROWS ? qb : kb) + static_cast<int64_t>(r0) * ra_ld, ra_ld, rows_valid, D, vec_ok, tid);
  load_tile<T, DP>(RB, LD, (QROWS ? gb : vb) + static_cast<int64_t>(r0) * rb_ld, rb_ld, rows_valid, D, vec_ok, tid);

  float lse_r[4], d_r[4];
  if (MODE == 0) {
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const int r = r0 + ty * 4 + ii;
      lse_r[ii] = r < N ? lse[r] : -CUDART_INF_F;
      d_r[ii] = r < N ? drow[r] : 0.f;
    }
  }
  if (MODE == 3) {
    // the pre-pass, inline: D = sum_d out * dout over the row (out staged in the K tile's buffer, dout already
    // resident), LSE = m + log2(max(z, 1e-30))
    const T* ob = static_cast<const T*>(prm.out) + b * prm.os.b + h * prm.os.h;
    const bool ovec = vec_ok && ((prm.os.r | prm.os.h | prm.os.b) % 4) == 0;
    load_tile<T, DP>(CA, LD, ob, prm.os.r, rows_valid, D, ovec, tid);
    __syncthreads();
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const int r = ty * 4 + ii;
      float part = 0.f;
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        const int col = tile_col<DP>(tx, c);
        part += CA[r * LD + col] * RB[r * LD + col];     // columns >= D are zero-filled in both tiles
      }
#pragma unroll
      for (int o = 8; o >= 1; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      d_r[ii] = r < N ? part : 0.f;
      const int64_t sr = static_cast<int64_t>(bh) * N + r;
      lse_r[ii] = r < N ? prm.row_m[sr] + log2f(fmaxf(prm.row_z[sr], 1.0e-30f)) : -CUDART_INF_F;
    }
    // (the loop below starts with a barrier before it overwrites the staging buffer)
  }
  float acc3[4][CPT];   // MODE 3: dK (unused, and removed by the compiler, in the other modes)
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < CPT; ++c) acc3[i][c] = 0.f;
  float acc1[4][CPT], acc2[4][CPT];  // MODE 0: acc1 = dQ; MODE 1: acc1 = dV, acc2 = dK
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < CPT; ++c) { acc1[i][c] = 0.f; acc2[i][c] = 0.f; }

  int c_begin = 0, c_end = NC;
  if (prm.is_causal) {
    if (QROWS) c_end = max(0, min(NK, r0 + rows_valid - koff));  // local keys whose sequence index <= last query row of the tile
    else c_begin = min(N, r0 + koff);                                // queries >= sequence index of the first key row of the tile
  }

  for (int c0 = c_begin; c0 < c_end; c0 += 64) {
    __syncthreads();
    const int cv = min(64, NC - c0);
    load_tile<T, DP>(CA, LD, (QROWS ? kb : qb) + static_cast<int64_t>(c0) * ca_ld, ca_ld, cv, D, vec_ok, tid);
    load_tile<T, DP>(CB, LD, (QROWS ? vb : gb) + static_cast<int64_t>(c0) * cb_ld, cb_ld, cv, D, vec_ok, tid);
    __syncthreads();

    float S[4][4], dP[4][4];
    tile_dot<DP>(RA, CA, LD, ty, tx, S);
    tile_dot<DP>(RB, CB, LD, ty, tx, dP);

    float lse_c[4], d_c[4];
    if (!QROWS) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int c = c0 + tx + 16 * jj;
        lse_c[jj] = c < N ? lse[c] : -CUDART_INF_F;
        d_c[jj] = c < N ? drow[c] : 0.f;
      }
    }
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int rr = r0 + ty * 4 + ii, cc = c0 + tx + 16 * jj;
        const int qi = QROWS ? rr : cc;
        const int kj = (QROWS ? cc : rr) + koff;       // sequence index of the key
        bool valid = rr < NR && cc < NC;
        if (prm.is_causal) valid = valid && (qi >= kj);
        const float l = QROWS ? lse_r[ii] : lse_c[jj];
        const float dd = QROWS ? d_r[ii] : d_c[jj];
        float sc;
        if (bias_bh) {
          const float bv = valid ? bias_bh[static_cast<int64_t>(qi) * prm.bsq + static_cast<int64_t>(kj) * prm.bsk] : 0.f;
          sc = (S[ii][jj] * prm.scale + bv) * kLog2e;
        } else {
          sc = S[ii][jj] * prm.scale_log2;
        }
        // a row with no admissible key has LSE = -inf: its probabilities are defined as 0
        const float p = (valid && l > -CUDART_INF_F) ? exp2f(sc - l) : 0.f;
        const float ds = p * (dP[ii][jj] - dd);
        if (QROWS && dbias_bh && valid) {
          float* dst = dbias_bh + static_cast<int64_t>(qi) * prm.dsq + static_cast<int64_t>(kj) * prm.dsk;
          if (prm.dbias_atomic) atomicAdd(dst, ds); else *dst = ds;
        }
        const int so = (ty * 4 + ii) * 68 + tx + 16 * jj;
        if (MODE == 0) {
          Ps[so] = round_to<T>(ds);
        } else if (MODE == 3) {
          Ps[so] = round_to<T>(ds);      // dS [query][key]
          Ss[so] = round_to<T>(p);       // P  [query][key]
        } else {
          Ps[so] = round_to<T>(p);
          Ss[so] = round_to<T>(ds);
        }
      }
    }
    __syncthreads();
    if (MODE == 0) {
      tile_pv<DP>(Ps, CA, LD, ty, tx, acc1);   // dQ += dS K
    } else if (MODE == 3) {
      tile_pv<DP>(Ps, CA, LD, ty, tx, acc1);    // dQ = dS K            (rows: queries)
      tile_ptv<DP>(Ss, RB, LD, ty, tx, acc2);   // dV = P^T dO          (rows: keys; the left operand is read transposed)
      tile_ptv<DP>(Ps, RA, LD, ty, tx, acc3);   // dK = dS^T Q
    } else {
      tile_pv<DP>(Ps, CB, LD, ty, tx, acc1);   // dV += P^T dO
      tile_pv<DP>(Ss, CA, LD, ty, tx, acc2);   // dK += dS^T Q
    }
    if (MODE == 2) {
      // dQ[c0 + q][:] += scale * sum_key dS^T[key][q] * K[key][:]   (dS^T in Ss, this CTA's K rows in RA)
      float dq[4][CPT];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < CPT; ++c) dq[i][c] = 0.f;
      tile_ptv<DP>(Ss, RA, LD, ty, tx, dq);
      float* dq_base = static_cast<float*>(prm.dq) + (static_cast<int64_t>(bh) * N + c0) * D;
#pragma unroll
      for (int ii = 0; ii < 4; ++ii) {
        const int qr = ty * 4 + ii;
        if (c0 + qr >= N) continue;
        float* dst = dq_base + static_cast<int64_t>(qr) * D;
        if constexpr (DP == 64) {
          if (D == 64) {        // four consecutive columns per thread: one 16-byte vector reduction
            red_add_v4(dst + tx * 4, dq[ii][0] * prm.scale, dq[ii][1] * prm.scale, dq[ii][2] * prm.scale, dq[ii][3] * prm.scale);
            continue;
          }
        }
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          const int col = tile_col<DP>(tx, c);
          if (col < D) atomicAdd(dst + col, dq[ii][c] * prm.scale);
        }
      }
    }
  }

#pragma unroll
  for (int ii = 0; ii < 4; ++ii) {
    const int r = r0 + ty * 4 + ii;
    if (r >= NR) continue;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int col = tile_col<DP>(tx, c);
      if (col >= D) continue;
      if (QROWS) {
        if (prm.dq_f32) static_cast<float*>(prm.dq)[(static_cast<int64_t>(bh) * N + r) * D + col] = acc1[ii][c] * prm.scale;
        else static_cast<T*>(prm.dq)[b * prm.dqs.b + h * prm.dqs.h + r * prm.dqs.r + col] = from_f32<T>(acc1[ii][c] * prm.scale);
        if (MODE == 3) {     // single tile: row r is also key r
          static_cast<T*>(prm.dv)[b * prm.dvs.b + h * prm.dvs.h + r * prm.dvs.r + col] = from_f32<T>(acc2[ii][c]);
          static_cast<T*>(prm.dk)[b * prm.dks.b + h * prm.dks.h + r * prm.dks.r + col] = from_f32<T>(acc3[ii][c] * prm.scale);
        }
      } else {
        static_cast<T*>(prm.dv)[b * prm.dvs.b + h * prm.dvs.h + r * prm.dvs.r + col] = from_f32<T>(acc1[ii][c]);
        static_cast<T*>(prm.dk)[b * prm.dks.b + h * prm.dks.h + r * prm.dks.r + col] = from_f32<T>(acc2[ii][c] * prm.scale);
      }
    }
  }
}

template <typename T, int DP, int MODE>
static int launch_bwd(const BwdParams& p, cudaStream_t st) {
  constexpr size_t smem = sizeof(float) * (4 * 64 * (DP + 4) + (MODE == 0 ? 1 : 2) * 64 * 68);
  static_assert(MODE >= 0 && MODE <= 3, "MODE");
  int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&bwd_simt_kernel<T, DP, MODE>), smem);
  if (rc != ELSA_OK) return rc;
  const int rows = (MODE == 0 || MODE == 3) ? p.n_ctx : p.n_keys;
  if (rows == 0) return ELSA_OK;
  dim3 grid(static_cast<unsigned>((rows + 63) / 64), static_cast<unsigned>(p.bh));
  bwd_simt_kernel<T, DP, MODE><<<grid, 256, smem, st>>>(p);
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

template <typename T>
static int bwd_simt_t(const BwdParams& p, cudaStream_t st) {
  const int dp = p.head_dim <= 32 ? 32 : (p.head_dim <= 64 ? 64 : 128);
  int rc;
  // one fused launch where dQ is fp32 (fp32 inputs with a contiguous dq, or the fp32 partial of a sequence shard) and
  // no bias gradient is wanted: dQ is zeroed and every (key tile, query tile) pair adds its contribution
  const bool dq_contig = p.dqs.r == p.head_dim && p.dqs.h == static_cast<int64_t>(p.n_ctx) * p.head_dim &&
                         (p.heads == 1 || p.bh == p.heads || p.dqs.b == p.dqs.h * p.heads);
  if (p.single_tile && dp <= 64) {
    if (dp == 32) return launch_bwd<T, 32, 3>(p, st);
    return launch_bwd<T, 64, 3>(p, st);
  }
  const bool fused = !p.dbias && (p.dq_f32 || (sizeof(T) == 4 && dq_contig)) && p.n_keys > 0;
  if (fused) {
    ELSA_CUDA_CHECK(cudaMemsetAsync(p.dq, 0, static_cast<size_t>(p.bh) * p.n_ctx * p.head_dim * sizeof(float), st));
    if (dp == 32) return launch_bwd<T, 32, 2>(p, st);
    if (dp == 64) return launch_bwd<T, 64, 2>(p, st);
    return launch_bwd<T, 128, 2>(p, st);
  }
  if (dp == 32) { rc = launch_bwd<T, 32, 0>(p, st); if (rc) return rc; return launch_bwd<T, 32, 1>(p, st); }
  if (dp == 64) { rc = launch_bwd<T, 64, 0>(p, st); if (rc) return rc; return launch_bwd<T, 64, 1>(p, st); }
  rc = launch_bwd<T, 128, 0>(p, st); if (rc) return rc; return launch_bwd<T, 128, 1>(p, st);
}

int bwd_simt(const BwdParams& p, int dtype, cudaStream_t st) {
  if (dtype == ELSA_F32) return bwd_simt_t<float>(p, st);
  if (dtype == ELSA_F16) return bwd_simt_t<__half>(p, st);
  return bwd_simt_t<__nv_bfloat16>(p, st);
}

// ---- preprocess --------------------------------------------------------------------------
// 8 lanes per row; blockIdx.y = (batch*head), x covers the rows; out / dout rows are addressed through their strides.
template <typename T>
__global__ void __launch_bounds__(256)
bwd_preprocess_kernel(const T* __restrict__ out, const T* __restrict__ dout, const float* __restrict__ row_m,
                      const float* __restrict__ row_z, float* __restrict__ row_d, float* __restrict__ row_lse,
                      int heads, int n_ctx, int D, Strides os, Strides gs, int vec_ok) {
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = static_cast<int>(gid >> 3);
  const int lane = static_cast<int>(gid & 7);
  const int bh = blockIdx.y;
  const int b = bh / heads, h = bh - b * heads;
  const bool ok = r < n_ctx;
  float part = 0.f;
  if (ok) {
    const T* o = out + b * os.b + h * os.h + static_cast<int64_t>(r) * os.r;
    const T* g = dout + b * gs.b + h * gs.h + static_cast<int64_t>(r) * gs.r;
    if (vec_ok == 2) {          // 16-bit elements, D % 8 == 0, rows 16-byte aligned: 16-byte loads
      if constexpr (sizeof(T) == 2) {
        for (int c = lane * 8; c < D; c += 64) {
          const uint4 ov = *reinterpret_cast<const uint4*>(o + c), gv = *reinterpret_cast<const uint4*>(g + c);
          const T* oe = reinterpret_cast<const T*>(&ov);
          const T* ge = reinterpret_cast<const T*>(&gv);
#pragma unroll
          for (int i = 0; i < 8; ++i) part += to_f32<T>(oe[i]) * to_f32<T>(ge[i]);
        }
      }
    } else if (vec_ok) {
      for (int c = lane * 4; c < D; c += 32) {
        float a[4], bb[4];
        Vec4<T>::load(o + c, a);
        Vec4<T>::load(g + c, bb);
        part += a[0] * bb[0] + a[1] * bb[1] + a[2] * bb[2] + a[3] * bb[3];
      }
    } else {
      for (int c = lane; c < D; c += 8) part += to_f32<T>(o[c]) * to_f32<T>(g[c]);
    }
  }
  part += __shfl_xor_sync(0xffffffffu, part, 4);
  part += __shfl_xor_sync(0xffffffffu, part, 2);
  part += __shfl_xor_sync(0xffffffffu, part, 1);
  if (ok && lane == 0) {
    const int64_t row = static_cast<int64_t>(bh) * n_ctx + r;
    row_d[row] = part;
    row_lse[row] = row_m[row] + log2f(fmaxf(row_z[row], 1.0e-30f));
  }
}

int bwd_preprocess_any(const void* out, Strides os, const void* dout, Strides gs, const float* row_m, const float* row_z,
                       float* row_d, float* row_lse, int dtype, int batch, int heads, int n_ctx, int head_dim,
                       cudaStream_t st) {
  if (!out || !dout || !row_m || !row_z || !row_d || !row_lse || !dtype_ok(dtype) || batch < 1 || heads < 1 || n_ctx < 0 ||
      head_dim < 1 || head_dim > 128 || static_cast<int64_t>(batch) * heads > 65535)
    return ELSA_ERR_INVALID_ARGUMENT;
  if (n_ctx == 0) return ELSA_OK;
  const int64_t all = os.b | os.h | os.r | gs.b | gs.h | gs.r;
  const bool al16 = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(dout)) & 15u) == 0;
  int vec_ok = 0;
  if (dtype != ELSA_F32 && head_dim % 8 == 0 && al16 && all % 8 == 0) vec_ok = 2;
  else if (head_dim % 4 == 0 && all % 4 == 0 && (dtype != ELSA_F32 || al16)) vec_ok = 1;
  const dim3 grid(static_cast<unsigned>(cdiv64(static_cast<int64_t>(n_ctx) * 8, 256)), static_cast<unsigned>(batch * heads));
  if (dtype == ELSA_F32)
    bwd_preprocess_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(out), static_cast<const float*>(dout),
                                                       row_m, row_z, row_d, row_lse, heads, n_ctx, head_dim, os, gs, vec_ok);
  else if (dtype == ELSA_F16)
    bwd_preprocess_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(out), static_cast<const __half*>(dout),
                                                        row_m, row_z, row_d, row_lse, heads, n_ctx, head_dim, os, gs, vec_ok);
  else
    bwd_preprocess_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(out),
                                                               static_cast<const __nv_bfloat16*>(dout), row_m, row_z,
                                                               row_d, row_lse, heads, n_ctx, head_dim, os, gs, vec_ok);
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

}  // namespace elsa

using namespace elsa;

extern "C" int elsa_bwd_preprocess(const void* out, const void* dout, const float* row_m, const float* row_z,
                                   float* row_d, float* row_lse, int dtype, int bh, int n_ctx, int head_dim,
                                   void* stream) {
  if (bh < 1 || head_dim < 1) return ELSA_ERR_INVALID_ARGUMENT;
  const Strides cs = contiguous_strides(1, n_ctx, head_dim);      // [bh, 1, n_ctx, head_dim]
  return bwd_preprocess_any(out, cs, dout, cs, row_m, row_z, row_d, row_lse, dtype, bh, 1, n_ctx, head_dim,
                            static_cast<cudaStream_t>(stream));
}
