// Backward on the 5th-generation tensor cores for fp16 / bf16 inputs with a WIDE head, 64 < d <= 128 (multiples of 8),
// causal or not, and for BIASED problems of any head dim up to 128 (bias and dbias are read / written in global memory
// by the fold warps of the dQ kernel; with d <= 64 only the first half below exists): exact recompute from the saved
// row statistics.  The head dim is handled as two 64-column
// halves of the same tensors (the second half zero-padded by the TMA box when d < 128).
//
// The kernel for d <= 64 (bwd_tc.cu) keeps S^T, dP^T, dV, dK and dQ of one key tile in TMEM; with 128 gradient columns
// that no longer fits, so the work is split the way the fp32 backward is (bwd_tc3.cu), seven contractions per tile
// pair, no atomics:
//
//   bwdw_dq_kernel    one CTA per 128-row QUERY tile, 128-key tiles streamed:
//                       S  = Q_lo K_lo^T + Q_hi K_hi^T,  dP = dO_lo V_lo^T + dO_hi V_hi^T        (N = 128)
//                       dS = P (dP - D), P = 2^(S c - LSE), rounded to the input type, into TMEM
//                       dQ_h += dS K_h, h = lo, hi       accumulated in TMEM over the key tiles  (N = 64 each)
//   bwdw_dkv_kernel   one CTA per 128-row KEY tile, 64-query tiles streamed:
//                       S^T = K_lo Q_lo^T + K_hi Q_hi^T, dP^T = V_lo dO_lo^T + V_hi dO_hi^T      (N = 64)
//                       P^T, dS^T rounded to the input type, into TMEM
//                       dV_h += P^T dO_h, dK_h += dS^T Q_h   accumulated in TMEM over the query tiles
//
// Gradients accumulate in TMEM (the 16-bit outputs do not see the tensor core's truncating accumulation; the fp32
// kernels keep their running sums in registers for that reason).  Both kernels: 16 fold warps (four threads per row),
// a TMA producer warp, an MMA-issuing warp; all waits bounded.
#include <type_traits>

#include "kernels.cuh"
#include "tc_common.cuh"

namespace elsa {

using namespace tc;

namespace {

constexpr int kSlotBytes = 64 * 64 * 2;      // one 64 x 64 16-bit tile (streamed operand of the dK/dV kernel)
constexpr int kTileBytes = 128 * 64 * 2;     // one 128 x 64 16-bit tile
constexpr int kFoldWarps = 16, kFoldThreads = kFoldWarps * 32;
constexpr int kThreads = kFoldThreads + 64;
constexpr int kProducerWarp = 16, kIssuerWarp = 17;
constexpr uint32_t kTmemCols = 512;
constexpr uint64_t kSlotStep = kSlotBytes >> 4;   // shared-memory descriptors count 16-byte units
constexpr uint64_t kTileStep = kTileBytes >> 4;

// dQ kernel: Q and dO halves resident (64 KB), a ring of 4 K tiles (two key tiles: a tile's halves stay until its dQ
// contraction has read them) and one of 4 V tiles
constexpr int kDqKSlots = 4, kDqVSlots = 4;
constexpr int kDqSmem = (4 + kDqKSlots + kDqVSlots) * kTileBytes + 1024;
// dK/dV kernel: K and V halves resident (64 KB), 15 ring slots of 8 KB, 8 stages of (-LSE, -D) vectors of 64 queries
constexpr int kKvSlots = 15, kVecStages = 8, kVecBytes = 2 * 64 * 4;   // (the ring runs up to 7 query tiles ahead when a tile has 2 entries)
constexpr int kKvSmem = 4 * kTileBytes + kKvSlots * kSlotBytes + kVecStages * kVecBytes + 1024;

enum BarId { BAR_STAGE = 61, BAR_FULL = 62, BAR_FREE = 63, BAR_SDP = 65, BAR_SFREE = 66, BAR_DS = 67, BAR_ACC = 68 };

struct BwdWParams {
  const float* nlse_pad; const float* nd_pad;   // [BH][n_pad]: -LSE, -D; padding rows hold -inf / 0
  void* dq; void* dk; void* dv;                 // dk, dv in the input type; dq too unless dq_f32
  Strides dqs, dks, dvs;
  int n_ctx, n_pad, bh, heads, is_causal;
  int n_keys, key_offset;                       // K/V rows of this launch and the sequence index of the first one
  int head_dim, dq_f32;
  int n_halves;                                 // 1 when head_dim <= 64 (biased problems), else 2
  float scale, scale_log2;
  const float* bias; int64_t bsb, bsh, bsq, bsk;      // additive bias [.., N, N] (natural-log units) or null
  float* dbias; int64_t dsb, dsh, dsq, dsk;           // its gradient (same addressing; zeroed by the caller) or null
  int dbias_atomic;                                   // a broadcast axis: contributions are added atomically
  int* status;                                  // the device's status word (mapped host memory)
};

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}

// the first n (a multiple of 8, possibly <= 0) of 16 consecutive gradient values, times f, in type TO
template <typename TO>
__device__ __forceinline__ void store16(TO* dst, const uint32_t (&r)[16], float f, int n) {
  if constexpr (sizeof(TO) == 4) {
#pragma unroll
    for (int i = 0; i < 16; i += 4)
      if (i < n) *reinterpret_cast<float4*>(dst + i) = make_float4(__uint_as_float(r[i]) * f, __uint_as_float(r[i + 1]) * f,
                                                                    __uint_as_float(r[i + 2]) * f, __uint_as_float(r[i + 3]) * f);
  } else {
#pragma unroll
    for (int i = 0; i < 16; i += 8) {
      if (i >= n) continue;
      uint4 t;
      t.x = pack2<TO>(__uint_as_float(r[i]) * f, __uint_as_float(r[i + 1]) * f);
      t.y = pack2<TO>(__uint_as_float(r[i + 2]) * f, __uint_as_float(r[i + 3]) * f);
      t.z = pack2<TO>(__uint_as_float(r[i + 4]) * f, __uint_as_float(r[i + 5]) * f);
      t.w = pack2<TO>(__uint_as_float(r[i + 6]) * f, __uint_as_float(r[i + 7]) * f);
      *reinterpret_cast<uint4*>(dst + i) = t;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// dQ: one CTA per 128-row query tile, 128-key tiles
// TMEM columns: S [0,128) dP [128,256) dQ_lo [256,320) dQ_hi [320,384) dS [384,448)
// ------------------------------------------------------------------------------------------------------------------
template <typename T, bool BIAS>
__global__ void __launch_bounds__(kThreads, 1)
bwdw_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
               const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
               const BwdWParams prm) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * (kDqKSlots + kDqVSlots) + 5];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.y;
  const int bi = bh / prm.heads, hi = bh - bi * prm.heads;   // tensor-map coordinates of this (batch*head)
  const int q0 = blockIdx.x * 128;
  const int N = prm.n_ctx, NK = prm.n_keys, koff = prm.key_offset;
  int ke = NK;
  if (prm.is_causal) ke = min(ke, min(q0 + 128, N) - koff);   // keys above the tile's last row are never admissible
  const int n_t = ke > 0 ? (ke + 127) / 128 : 0;              // 128-key tiles this query tile visits

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto sQ = [&](int h) { return smem_base + h * kTileBytes; };
  auto sDO = [&](int h) { return smem_base + (2 + h) * kTileBytes; };
  auto sKs = [&](int i) { return smem_base + (4 + i) * kTileBytes; };
  auto sVs = [&](int i) { return smem_base + (4 + kDqKSlots + i) * kTileBytes; };
  const uint32_t bar0 = smem_u32(bars);
  auto bar_kfull = [&](int i) { return bar0 + 8 * i; };
  auto bar_kfree = [&](int i) { return bar0 + 8 * (kDqKSlots + i); };
  auto bar_vfull = [&](int i) { return bar0 + 8 * (2 * kDqKSlots + i); };
  auto bar_vfree = [&](int i) { return bar0 + 8 * (2 * kDqKSlots + kDqVSlots + i); };
  const uint32_t barx = bar0 + 8 * 2 * (kDqKSlots + kDqVSlots);
  const uint32_t bar_stage = barx;            // the Q / dO halves are in shared memory
  const uint32_t bar_sdp = barx + 8;          // dP(j), S(j) are in TMEM
  const uint32_t bar_sfree = barx + 16;       // the fold warps hold them in registers
  const uint32_t bar_ds = barx + 24;          // dS of tile j has been delivered
  const uint32_t bar_dq = barx + 32;          // the dQ contractions of tile j have retired

  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < kDqKSlots; ++i) { mbar_init(bar_kfull(i), 1); mbar_init(bar_kfree(i), 1); }
    for (int i = 0; i < kDqVSlots; ++i) { mbar_init(bar_vfull(i), 1); mbar_init(bar_vfree(i), 1); }
    mbar_init(bar_stage, 1);
    mbar_init(bar_sdp, 1); mbar_init(bar_sfree, kFoldWarps);
    mbar_init(bar_ds, kFoldWarps); mbar_init(bar_dq, 1);
    fence_mbar_init();
  }
  if (warp == kProducerWarp) {
    tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdQ = tmem_base + 256, tDS = tmem_base + 384;

  if (warp == kProducerWarp) {
    if (n_t > 0 && lane == 0) {
      // ---------------- TMA producer ----------------
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_do); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      const int nh = BIAS ? prm.n_halves : 2;
      mbar_arrive_expect_tx(bar_stage, 2 * nh * kTileBytes);
      for (int h = 0; h < nh; ++h) {
        tma_load_4d(sQ(h), &tmap_q, bar_stage, 64 * h, q0, hi, bi);
        tma_load_4d(sDO(h), &tmap_do, bar_stage, 64 * h, q0, hi, bi);
      }
      bool ok = true;
      // per key tile: its K halves (ring sequence numbers 2 j, 2 j + 1), then its V halves.  A V slot is released by
      // the dP contraction that read it, a K slot by the dQ contraction.
      for (int j = 0; j < n_t && ok; ++j) {
        for (int h = 0; h < nh && ok; ++h) {
          const int seq = 2 * j + h, slot = seq % kDqKSlots;
          if (seq >= kDqKSlots && !(ok = mbar_wait(bar_kfree(slot), ((seq / kDqKSlots) - 1) & 1, &abort_flag, prm.status, BAR_FREE))) break;
          mbar_arrive_expect_tx(bar_kfull(slot), kTileBytes);
          tma_load_4d(sKs(slot), &tmap_k, bar_kfull(slot), 64 * h, j * 128, hi, bi);
        }
        for (int h = 0; h < nh && ok; ++h) {
          const int seq = 2 * j + h, slot = seq % kDqVSlots;
          if (seq >= kDqVSlots && !(ok = mbar_wait(bar_vfree(slot), ((seq / kDqVSlots) - 1) & 1, &abort_flag, prm.status, BAR_FREE))) break;
          mbar_arrive_expect_tx(bar_vfull(slot), kTileBytes);
          tma_load_4d(sVs(slot), &tmap_v, bar_vfull(slot), 64 * h, j * 128, hi, bi);
        }
      }
    }
  } else if (warp == kIssuerWarp) {
    if (n_t > 0 && lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc_k = make_idesc(fmt, 0, 0, 128, 128);   // S, dP: A, B K-major, N = 128 keys
      constexpr uint32_t idesc_mn = make_idesc(fmt, 0, 1, 128, 64);   // dQ_h: A in TMEM, B (K_h) MN-major, N = 64
      const uint64_t dQh[2] = {make_sdesc(sQ(0), 16, 1024), make_sdesc(sQ(1), 16, 1024)};
      const uint64_t dDOh[2] = {make_sdesc(sDO(0), 16, 1024), make_sdesc(sDO(1), 16, 1024)};
      const uint64_t dk_k0 = make_sdesc(sKs(0), 16, 1024), dk_mn0 = make_sdesc(sKs(0), 128 * 128, 1024);
      const uint64_t dv_k0 = make_sdesc(sVs(0), 16, 1024);
      const int nh = BIAS ? prm.n_halves : 2;
      bool ok = mbar_wait(bar_stage, 0, &abort_flag, prm.status, BAR_STAGE);
      auto issue_sdp = [&](int j) {
        for (int h = 0; h < nh && ok; ++h) {               // dP = sum over the halves of dO_h V_h^T
          const int seq = 2 * j + h, slot = seq % kDqVSlots;
          if (!(ok = mbar_wait(bar_vfull(slot), (seq / kDqVSlots) & 1, &abort_flag, prm.status, BAR_FULL))) return;
          tc_fence_after();
          mma_ss_x4<2, 2>(tdP, dDOh[h], dv_k0 + slot * kTileStep, idesc_k, h == 0 ? 0u : 1u);
          mma_commit(bar_vfree(slot));
        }
        for (int h = 0; h < nh && ok; ++h) {               // S = sum over the halves of Q_h K_h^T
          const int seq = 2 * j + h, slot = seq % kDqKSlots;
          if (!(ok = mbar_wait(bar_kfull(slot), (seq / kDqKSlots) & 1, &abort_flag, prm.status, BAR_FULL))) return;
          tc_fence_after();
          mma_ss_x4<2, 2>(tS, dQh[h], dk_k0 + slot * kTileStep, idesc_k, h == 0 ? 0u : 1u);
        }                                     // the K halves stay: the dQ contractions read them again
        if (ok) mma_commit(bar_sdp);
      };
      if (ok) {
        tc_fence_after();
        issue_sdp(0);
      }
      for (int j = 0; ok && j < n_t; ++j) {
        if (j + 1 < n_t) {
          if (!(ok = mbar_wait(bar_sfree, j & 1, &abort_flag, prm.status, BAR_SFREE))) break;
          tc_fence_after();
          issue_sdp(j + 1);
          if (!ok) break;
        }
        if (!(ok = mbar_wait(bar_ds, j & 1, &abort_flag, prm.status, BAR_DS))) break;
        tc_fence_after();
        for (int h = 0; h < nh; ++h) {                     // dQ_h += dS K_h over the 128 keys (eight K-steps)
          const int slot = (2 * j + h) % kDqKSlots;
          mma_ts_x4<8, 128>(tdQ + 64 * h, tDS, dk_mn0 + slot * kTileStep, idesc_mn, j == 0 ? 0u : 1u);
          mma_ts_x4<8, 128>(tdQ + 64 * h, tDS + 32, dk_mn0 + slot * kTileStep + 512, idesc_mn, 1u);
          mma_commit(bar_kfree(slot));
        }
        mma_commit(bar_dq);                   // dS may be overwritten
      }
    }
  } else {
    // ---------------- fold warps: four threads per query row ----------------
    const int qd = warp & 3, cq = warp >> 2;                // TMEM lane quadrant, column quarter (32 keys)
    const int row = qd * 32 + lane;
    const int qi = q0 + row;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float c = prm.scale_log2;
    const float nlse = prm.nlse_pad[static_cast<int64_t>(bh) * prm.n_pad + qi];   // q0 + 127 < n_pad
    const float nd = prm.nd_pad[static_cast<int64_t>(bh) * prm.n_pad + qi];
    const bool two_halves = BIAS ? prm.n_halves == 2 : true;   // (warp-uniform: tcgen05.ld is collective)
    const int qrow = min(qi, N - 1);                        // rows beyond N are never stored: any valid address will do
    const float* bias_row = BIAS ? prm.bias + bi * prm.bsb + hi * prm.bsh + static_cast<int64_t>(qrow) * prm.bsq : nullptr;
    float* dbias_row = (BIAS && prm.dbias) ? prm.dbias + bi * prm.dsb + hi * prm.dsh + static_cast<int64_t>(qrow) * prm.dsq : nullptr;
    bool alive = n_t > 0;

    for (int j = 0; alive && j < n_t; ++j) {
      if constexpr (BIAS) {
        // this thread's 128 bytes of the bias row for the NEXT key tile: on their way into L2 while this tile is worked on
        const int kn = (j + 1) * 128 + 32 * cq;
        if (kn + 32 <= NK) {
          const float* bn = bias_row + static_cast<int64_t>(kn + koff) * prm.bsk;
          prefetch_l2(bn);
          prefetch_l2(bn + 31 * prm.bsk);
        }
      }
      if (!__all_sync(0xffffffffu, mbar_wait(bar_sdp, j & 1, &abort_flag, prm.status, BAR_SDP))) { alive = false; break; }
      tc_fence_after();
      uint32_t pk[16];
      {
        uint32_t rs[32], rp[32];
        tmem_ld32(tS + lane_off + 32 * cq, rs);
        tmem_ld32(tdP + lane_off + 32 * cq, rp);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive_warp(bar_sfree, lane);      // S and dP may be overwritten with the next tile's
        const int kb = j * 128 + 32 * cq;                   // first (local) key of this thread's columns
        const bool masked = (j * 128 + 128 > NK) || (prm.is_causal && (j * 128 + koff + 127 > q0));
        const int lim = prm.is_causal ? min(NK - 1, qi - koff) : NK - 1;   // last admissible (local) key of this row
        float ab[32];                                       // bias log2(e) - LSE of this thread's 32 keys
#pragma unroll
        for (int i = 0; i < 32; ++i) ab[i] = nlse;
        bool vec = false;
        if constexpr (BIAS) {
          // bias in natural-log units: s c + b log2(e) - LSE; keys beyond the row's last admissible one are masked below
          const float* bp = bias_row + static_cast<int64_t>(kb + koff) * prm.bsk;
          vec = prm.bsk == 1 && kb + 32 <= NK && (reinterpret_cast<uintptr_t>(bp) & 31u) == 0;
          if (vec) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float b8[8];
              ld_global_v8(bp + 8 * g, b8);      // whole 32-byte sectors: see fold_tcw.cu
#pragma unroll
              for (int e = 0; e < 8; ++e) ab[8 * g + e] = fmaf(b8[e], 1.4426950408889634f, nlse);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (kb + i < NK) ab[i] = fmaf(bp[i * prm.bsk], 1.4426950408889634f, nlse);
          }
        }
        float dsv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float p = fast_exp2(fmaf(__uint_as_float(rs[i]), c, ab[i]));
          if (masked && kb + i > lim) p = 0.f;
          dsv[i] = p * (__uint_as_float(rp[i]) + nd);
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) pk[i >> 1] = pack2<T>(dsv[i], dsv[i + 1]);
        if constexpr (BIAS) {
          // dbias = dS (every (query, key) pair is visited exactly once by this kernel); pairs that the causal rule or
          // the sequence length excludes hold zeros here, as the caller zeroed them
          if (dbias_row && qi < N) {
            float* dp = dbias_row + static_cast<int64_t>(kb + koff) * prm.dsk;
            if (!prm.dbias_atomic && prm.dsk == 1 && kb + 32 <= NK && (reinterpret_cast<uintptr_t>(dp) & 31u) == 0) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                float d8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) d8[e] = dsv[8 * g + e];
                st_global_v8(dp + 8 * g, d8);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (kb + i > lim) continue;
                if (prm.dbias_atomic) atomicAdd(dp + i * prm.dsk, dsv[i]); else dp[i * prm.dsk] = dsv[i];
              }
            }
          }
        }
      }
      if (j > 0) {
        // the dQ contractions of the previous key tile have read dS
        if (!__all_sync(0xffffffffu, mbar_wait(bar_dq, (j - 1) & 1, &abort_flag, prm.status, BAR_ACC))) { alive = false; break; }
        tc_fence_after();
      }
      tmem_st16(tDS + lane_off + 16 * cq, pk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(bar_ds, lane);
    }
    uint32_t r0[16], r1[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) { r0[i] = 0u; r1[i] = 0u; }
    if (alive && n_t > 0) {
      if (!__all_sync(0xffffffffu, mbar_wait(bar_dq, (n_t - 1) & 1, &abort_flag, prm.status, BAR_ACC))) alive = false;
      if (alive) {
        tc_fence_after();
        tmem_ld16(tdQ + lane_off + 16 * cq, r0);
        if (two_halves) tmem_ld16(tdQ + 64 + lane_off + 16 * cq, r1);
        tmem_wait_ld();
      }
    }
    if (qi < N && (alive || n_t == 0)) {
      const int d = prm.head_dim, c0 = 16 * cq, c1 = 64 + 16 * cq;
      const int64_t off = bi * prm.dqs.b + hi * prm.dqs.h + static_cast<int64_t>(qi) * prm.dqs.r;
      if (prm.dq_f32) {
        store16<float>(static_cast<float*>(prm.dq) + off + c0, r0, prm.scale, d - c0);
        store16<float>(static_cast<float*>(prm.dq) + off + c1, r1, prm.scale, d - c1);
      } else {
        store16<T>(static_cast<T*>(prm.dq) + off + c0, r0, prm.scale, d - c0);
        store16<T>(static_cast<T*>(prm.dq) + off + c1, r1, prm.scale, d - c1);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------------------------------------------------
// dK, dV: one CTA per 128-row key tile, 64-query tiles
// TMEM columns: S^T [0,64) dP^T [64,128) P^T [128,160) dS^T [160,192) dV_lo dV_hi [192,320) dK_lo dK_hi [320,448)
// ------------------------------------------------------------------------------------------------------------------
template <typename T, bool BIAS>
__global__ void __launch_bounds__(kThreads, 1)
bwdw_dkv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                const BwdWParams prm) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kKvSlots + 5];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.y;
  const int bi = bh / prm.heads, hi = bh - bi * prm.heads;   // tensor-map coordinates of this (batch*head)
  const int k0 = blockIdx.x * 128;                  // first (local) key row of this CTA
  const int N = prm.n_ctx, NK = prm.n_keys;
  const int kseq0 = k0 + prm.key_offset;            // its index in the sequence
  const int n_q64 = (N + 63) / 64;
  const int it_begin = prm.is_causal ? min(n_q64, kseq0 / 64) : 0;   // query tiles above the diagonal see none of these keys
  const int n_it = n_q64 - it_begin;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  auto sK = [&](int h) { return smem_base + h * kTileBytes; };
  auto sV = [&](int h) { return smem_base + (2 + h) * kTileBytes; };
  auto sSlot = [&](int i) { return smem_base + 4 * kTileBytes + i * kSlotBytes; };
  const uint32_t vec_off = 4 * kTileBytes + kKvSlots * kSlotBytes;    // [stage][-LSE x 64 | -D x 64]
  const uint32_t bar0 = smem_u32(bars);
  auto bar_full = [&](int i) { return bar0 + 8 * i; };
  auto bar_free = [&](int i) { return bar0 + 8 * (kKvSlots + i); };
  const uint32_t barx = bar0 + 8 * 2 * kKvSlots;
  const uint32_t bar_kv = barx;               // the K / V halves are in shared memory
  const uint32_t bar_sdp = barx + 8;          // S^T(i), dP^T(i) are in TMEM
  const uint32_t bar_sfree = barx + 16;       // the fold warps hold them in registers
  const uint32_t bar_pl = barx + 24;          // P^T / dS^T of tile i have been delivered
  const uint32_t bar_acc = barx + 32;         // the dV / dK contractions of tile i have retired

  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < kKvSlots; ++i) { mbar_init(bar_full(i), 1); mbar_init(bar_free(i), 1); }
    mbar_init(bar_kv, 1);
    mbar_init(bar_sdp, 1); mbar_init(bar_sfree, kFoldWarps);
    mbar_init(bar_pl, kFoldWarps); mbar_init(bar_acc, 1);
    fence_mbar_init();
  }
  if (warp == kProducerWarp) {
    tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tS = tmem_base, tdP = tmem_base + 64, tP = tmem_base + 128, tDS = tmem_base + 160;
  const uint32_t tdV = tmem_base + 192, tdK = tmem_base + 320;

  if (warp == kProducerWarp) {
    if (n_it > 0 && lane == 0) {
      // ---------------- TMA producer ----------------
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_do); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      const int nh = BIAS ? prm.n_halves : 2;
      mbar_arrive_expect_tx(bar_kv, 2 * nh * kTileBytes);
      for (int h = 0; h < nh; ++h) {
        tma_load_4d(sK(h), &tmap_k, bar_kv, 64 * h, k0, hi, bi);
        tma_load_4d(sV(h), &tmap_v, bar_kv, 64 * h, k0, hi, bi);
      }
      int seq = 0;
      bool ok = true;
      // ring order of query tile i: its dO halves (sequence numbers 2 nh i ...), then its Q halves; the tile's first
      // slot also receives its -LSE / -D vectors
      for (int it = 0; it < n_it && ok; ++it) {
        const int qrow = (it_begin + it) * 64;
        for (int x = 0; x < 2 * nh && ok; ++x) {
          const int slot = seq % kKvSlots;
          if (seq >= kKvSlots && !(ok = mbar_wait(bar_free(slot), ((seq / kKvSlots) - 1) & 1, &abort_flag, prm.status, BAR_FREE))) break;
          mbar_arrive_expect_tx(bar_full(slot), kSlotBytes + (x == 0 ? kVecBytes : 0));
          tma_load_4d(sSlot(slot), x < nh ? &tmap_do : &tmap_q, bar_full(slot), 64 * (x % nh), qrow, hi, bi);
          if (x == 0) {
            const uint32_t dst = smem_base + vec_off + (it % kVecStages) * kVecBytes;
            bulk_load_1d(dst, prm.nlse_pad + static_cast<int64_t>(bh) * prm.n_pad + qrow, 256, bar_full(slot));
            bulk_load_1d(dst + 256, prm.nd_pad + static_cast<int64_t>(bh) * prm.n_pad + qrow, 256, bar_full(slot));
          }
          ++seq;
        }
      }
    }
  } else if (warp == kIssuerWarp) {
    if (n_it > 0 && lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc_k = make_idesc(fmt, 0, 0, 128, 64);    // S^T, dP^T: A, B K-major, N = 64 queries
      constexpr uint32_t idesc_mn = make_idesc(fmt, 0, 1, 128, 64);   // dV_h, dK_h: A in TMEM, B MN-major, N = 64
      const uint64_t dKh[2] = {make_sdesc(sK(0), 16, 1024), make_sdesc(sK(1), 16, 1024)};
      const uint64_t dVh[2] = {make_sdesc(sV(0), 16, 1024), make_sdesc(sV(1), 16, 1024)};
      const uint64_t dk_slot0 = make_sdesc(sSlot(0), 16, 1024), dmn_slot0 = make_sdesc(sSlot(0), 64 * 128, 1024);
      const int nh = BIAS ? prm.n_halves : 2;
      bool ok = mbar_wait(bar_kv, 0, &abort_flag, prm.status, BAR_STAGE);
      auto issue_sdp = [&](int it) {
        for (int h = 0; h < nh && ok; ++h) {               // dP^T = sum over the halves of V_h dO_h^T
          const int seq = 2 * nh * it + h, slot = seq % kKvSlots;
          if (!(ok = mbar_wait(bar_full(slot), (seq / kKvSlots) & 1, &abort_flag, prm.status, BAR_FULL))) return;
          tc_fence_after();
          mma_ss_x4<2, 2>(tdP, dVh[h], dk_slot0 + slot * kSlotStep, idesc_k, h == 0 ? 0u : 1u);
        }
        for (int h = 0; h < nh && ok; ++h) {               // S^T = sum over the halves of K_h Q_h^T
          const int seq = 2 * nh * it + nh + h, slot = seq % kKvSlots;
          if (!(ok = mbar_wait(bar_full(slot), (seq / kKvSlots) & 1, &abort_flag, prm.status, BAR_FULL))) return;
          tc_fence_after();
          mma_ss_x4<2, 2>(tS, dKh[h], dk_slot0 + slot * kSlotStep, idesc_k, h == 0 ? 0u : 1u);
        }
        if (ok) mma_commit(bar_sdp);
      };
      if (ok) {
        tc_fence_after();
        issue_sdp(0);
      }
      for (int it = 0; ok && it < n_it; ++it) {
        if (it + 1 < n_it) {
          if (!(ok = mbar_wait(bar_sfree, it & 1, &abort_flag, prm.status, BAR_SFREE))) break;
          tc_fence_after();
          issue_sdp(it + 1);
          if (!ok) break;
        }
        if (!(ok = mbar_wait(bar_pl, it & 1, &abort_flag, prm.status, BAR_DS))) break;
        tc_fence_after();
        const uint32_t acc = it == 0 ? 0u : 1u;
        for (int h = 0; h < nh; ++h) {                     // dV_h += P^T dO_h (64 queries: four K-steps)
          const int slot = (2 * nh * it + h) % kKvSlots;
          mma_ts_x4<8, 128>(tdV + 64 * h, tP, dmn_slot0 + slot * kSlotStep, idesc_mn, acc);
          mma_commit(bar_free(slot));
        }
        for (int h = 0; h < nh; ++h) {                     // dK_h += dS^T Q_h
          const int slot = (2 * nh * it + nh + h) % kKvSlots;
          mma_ts_x4<8, 128>(tdK + 64 * h, tDS, dmn_slot0 + slot * kSlotStep, idesc_mn, acc);
          mma_commit(bar_free(slot));
        }
        mma_commit(bar_acc);                  // P^T / dS^T may be overwritten
      }
    }
  } else {
    // ---------------- fold warps: four threads per key row ----------------
    const int qd = warp & 3, cq = warp >> 2;                // TMEM lane quadrant, column quarter (16 queries)
    const int row = qd * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const int key = k0 + row;                  // local key row
    const int key_seq = kseq0 + row;           // its index in the sequence (what the causal rule compares)
    const bool key_ok = key < NK;
    const bool cta_tail = k0 + 128 > NK;       // some key rows of this CTA do not exist
    const float c = prm.scale_log2;
    const int n_halves = BIAS ? prm.n_halves : 2;
    // bias[query, key] of this thread's key column; the query offset is added per element
    const float* bias_col = BIAS ? prm.bias + bi * prm.bsb + hi * prm.bsh + static_cast<int64_t>(min(key_seq, N - 1)) * prm.bsk : nullptr;
    bool alive = true;

    for (int it = 0; it < n_it; ++it) {
      const int q_tile0 = (it_begin + it) * 64;
      if constexpr (BIAS) {
        // the bias of the NEXT query tile (16 rows of this thread's column quarter, one 128-byte line per row and warp)
        // on its way into L2 while this tile is worked on
        const int qn = q_tile0 + 64 + 16 * cq + (lane & 15);
        if (it + 1 < n_it && qn < N) prefetch_l2(bias_col + static_cast<int64_t>(qn) * prm.bsq);
      }
      if (!__all_sync(0xffffffffu, mbar_wait(bar_sdp, it & 1, &abort_flag, prm.status, BAR_SDP))) { alive = false; break; }
      // the tile's row statistics were written by the bulk copies that complete on its first slot's barrier: observe
      // that barrier directly (it completed before the MMAs behind bar_sdp were issued, so this never spins)
      {
        const int seq = 2 * n_halves * it;
        if (!__all_sync(0xffffffffu, mbar_wait(bar_full(seq % kKvSlots), (seq / kKvSlots) & 1, &abort_flag, prm.status, BAR_FULL))) { alive = false; break; }
      }
      tc_fence_after();
      uint32_t pk[8], dsk[8];
      {
        uint32_t rs[16], rp[16];
        tmem_ld16(tS + lane_off + 16 * cq, rs);
        tmem_ld16(tdP + lane_off + 16 * cq, rp);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive_warp(bar_sfree, lane);      // S^T and dP^T may be overwritten with the next tile's
        const float4* nl4 = reinterpret_cast<const float4*>(smem_gen + vec_off + (it % kVecStages) * kVecBytes) + 4 * cq;
        const float4* nd4 = nl4 + 16;
        const bool masked = cta_tail || (prm.is_causal && q_tile0 < kseq0 + 128);   // only the diagonal tiles / the last key tile
        const int qc = q_tile0 + 16 * cq;                                           // first query of this thread's columns
        // The bias of this thread's 16 (query, key) pairs, fetched by unconditional loads (the query clamped into the
        // sequence) ahead of a branch-free element loop: with a conditional load inside, every element was a basic
        // block of its own and its chain of dependent instructions overlapped with nobody's.
        float bb[16];
        if constexpr (BIAS) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float bv = bias_col[static_cast<int64_t>(min(qc + i, N - 1)) * prm.bsq];
            bb[i] = (key_ok && qc + i < N) ? bv * 1.4426950408889634f : 0.f;
          }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const float4 nl = nl4[g], nd = nd4[g];            // -LSE, -D of 4 queries (warp-wide broadcast reads)
          const float nle[4] = {nl.x, nl.y, nl.z, nl.w}, nde[4] = {nd.x, nd.y, nd.z, nd.w};
          float pv[4], dv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = 4 * g + e;
            float a = nle[e];
            if constexpr (BIAS) a += bb[i];
            float x = fast_exp2(fmaf(__uint_as_float(rs[i]), c, a));
            if (masked && !(key_ok && (!prm.is_causal || qc + i >= key_seq))) x = 0.f;
            pv[e] = x;
            dv[e] = x * (__uint_as_float(rp[i]) + nde[e]);
          }
          pk[2 * g] = pack2<T>(pv[0], pv[1]); pk[2 * g + 1] = pack2<T>(pv[2], pv[3]);
          dsk[2 * g] = pack2<T>(dv[0], dv[1]); dsk[2 * g + 1] = pack2<T>(dv[2], dv[3]);
        }
      }
      if (it > 0) {
        // the dV / dK contractions of the previous query tile have read P^T and dS^T
        if (!__all_sync(0xffffffffu, mbar_wait(bar_acc, (it - 1) & 1, &abort_flag, prm.status, BAR_ACC))) { alive = false; break; }
        tc_fence_after();
      }
      tmem_st8(tP + lane_off + 8 * cq, pk);
      tmem_st8(tDS + lane_off + 8 * cq, dsk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(bar_pl, lane);
    }
    if (alive && n_it > 0 && !__all_sync(0xffffffffu, mbar_wait(bar_acc, (n_it - 1) & 1, &abort_flag, prm.status, BAR_ACC))) alive = false;
    if (alive) {
      // dK, dV of this key tile (tcgen05.ld is warp-collective: only the stores are predicated)
      const int d = prm.head_dim;
#pragma unroll
      for (int h = 0; h < n_halves; ++h) {
        uint32_t rk[16], rv[16];
        if (n_it > 0) {
          tc_fence_after();
          tmem_ld16(tdK + 64 * h + lane_off + 16 * cq, rk);
          tmem_ld16(tdV + 64 * h + lane_off + 16 * cq, rv);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) { rk[i] = 0u; rv[i] = 0u; }   // no query sees these keys: zero gradients
        }
        if (key_ok) {
          const int col = 64 * h + 16 * cq;
          store16<T>(static_cast<T*>(prm.dk) + bi * prm.dks.b + hi * prm.dks.h + static_cast<int64_t>(key) * prm.dks.r + col, rk, prm.scale, d - col);
          store16<T>(static_cast<T*>(prm.dv) + bi * prm.dvs.b + hi * prm.dvs.h + static_cast<int64_t>(key) * prm.dvs.r + col, rv, 1.f, d - col);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) tmem_dealloc(tmem_base, kTmemCols);
}

// -D = -sum_d out*dout, -LSE = -(m + log2(max(z, 1e-30))) into the padded layout; padding: -D = 0, -LSE = -inf
template <typename T>
__global__ void __launch_bounds__(256)
bwdw_preprocess_kernel(const T* __restrict__ out, const T* __restrict__ dout, const float* __restrict__ row_m,
                       const float* __restrict__ row_z, float* __restrict__ nd_pad, float* __restrict__ nlse_pad,
                       int heads, int n_ctx, int n_pad, int head_dim, Strides os, Strides gs) {
  // blockIdx.y = (batch*head); x covers the n_pad padded rows, 16 lanes (8 elements = 16 bytes each) per row
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = static_cast<int>(gid >> 4);
  const int lane = static_cast<int>(gid & 15);
  const int64_t b = blockIdx.y;
  const bool in_pad = r < n_pad;
  const bool real = in_pad && r < n_ctx;
  float part = 0.f;
  if (real && lane * 8 < head_dim) {
    const int bi = static_cast<int>(b) / heads, hi = static_cast<int>(b) - bi * heads;
    const uint4 ov = *reinterpret_cast<const uint4*>(out + bi * os.b + hi * os.h + static_cast<int64_t>(r) * os.r + lane * 8);
    const uint4 gv = *reinterpret_cast<const uint4*>(dout + bi * gs.b + hi * gs.h + static_cast<int64_t>(r) * gs.r + lane * 8);
    const T* oe = reinterpret_cast<const T*>(&ov);
    const T* ge = reinterpret_cast<const T*>(&gv);
#pragma unroll
    for (int i = 0; i < 8; ++i) part += to_f32<T>(oe[i]) * to_f32<T>(ge[i]);
  }
  part += __shfl_xor_sync(0xffffffffu, part, 8);
  part += __shfl_xor_sync(0xffffffffu, part, 4);
  part += __shfl_xor_sync(0xffffffffu, part, 2);
  part += __shfl_xor_sync(0xffffffffu, part, 1);
  if (in_pad && lane == 0) {
    const int64_t prow = b * n_pad + r;
    if (real) {
      nd_pad[prow] = -part;
      // (a row whose keys are all masked by the bias has m = -inf, z = 0: -LSE = -inf keeps its P at 0)
      const float rm = row_m[b * n_ctx + r], rz = row_z[b * n_ctx + r];
      nlse_pad[prow] = (rz > 0.f && rm > -CUDART_INF_F) ? -(rm + log2f(rz)) : -CUDART_INF_F;
    } else {
      nd_pad[prow] = 0.f;
      nlse_pad[prow] = -CUDART_INF_F;
    }
  }
}

}  // namespace

bool bwd_tcw_supported(int dtype, int head_dim, bool has_bias) { return fold_tcw_supported(dtype, head_dim, has_bias); }

int64_t bwd_tcw_workspace_bytes(int bh, int n_ctx) {
  const int64_t n_pad = align_up(n_ctx, 128);
  return 2 * align_up(static_cast<int64_t>(bh) * n_pad * 4, 256);
}

template <typename T>
static int bwd_tcw_t(const BwdParams& p, const void* out, Strides os, const float* row_m, const float* row_z,
                     void* workspace, int dtype, cudaStream_t st) {
  const int N = p.n_ctx, NK = p.n_keys, bh = p.bh, batch = bh / p.heads;
  const int n_pad = static_cast<int>(align_up(N, 128));
  const int64_t vec_bytes = align_up(static_cast<int64_t>(bh) * n_pad * 4, 256);
  char* ws = static_cast<char*>(workspace);
  float* nd_pad = reinterpret_cast<float*>(ws);
  float* nlse_pad = reinterpret_cast<float*>(ws + vec_bytes);
  int rc;
  {
    const dim3 pgrid(static_cast<unsigned>(cdiv64(static_cast<int64_t>(n_pad) * 16, 256)), static_cast<unsigned>(bh));
    bwdw_preprocess_kernel<T><<<pgrid, 256, 0, st>>>(static_cast<const T*>(out), static_cast<const T*>(p.dout), row_m, row_z,
                                                     nd_pad, nlse_pad, p.heads, N, n_pad, p.head_dim, os, p.gs);
    ELSA_LAUNCH_CHECK();
  }
  CUtensorMap mq128, mdo128, mq64, mdo64, mk128, mv128;
  if ((rc = make_tmap_rows64(&mq128, p.q, dtype, N, p.heads, batch, p.qs, 128, p.head_dim)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mdo128, p.dout, dtype, N, p.heads, batch, p.gs, 128, p.head_dim)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mq64, p.q, dtype, N, p.heads, batch, p.qs, 64, p.head_dim)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mdo64, p.dout, dtype, N, p.heads, batch, p.gs, 64, p.head_dim)) != ELSA_OK) return rc;
  BwdWParams prm;
  if ((rc = device_status_word(&prm.status, nullptr)) != ELSA_OK) return rc;
  prm.nlse_pad = nlse_pad; prm.nd_pad = nd_pad;
  prm.dq = p.dq; prm.dk = p.dk; prm.dv = p.dv;
  prm.dqs = p.dqs; prm.dks = p.dks; prm.dvs = p.dvs;
  prm.n_ctx = N; prm.n_pad = n_pad; prm.bh = bh; prm.heads = p.heads; prm.is_causal = p.is_causal;
  prm.n_keys = NK; prm.key_offset = p.key_offset; prm.head_dim = p.head_dim; prm.dq_f32 = p.dq_f32;
  prm.scale = p.scale; prm.scale_log2 = p.scale_log2;
  prm.n_halves = p.head_dim > 64 ? 2 : 1;
  prm.bias = p.bias; prm.bsb = p.bsb; prm.bsh = p.bsh; prm.bsq = p.bsq; prm.bsk = p.bsk;
  prm.dbias = p.dbias; prm.dsb = p.dsb; prm.dsh = p.dsh; prm.dsq = p.dsq; prm.dsk = p.dsk; prm.dbias_atomic = p.dbias_atomic;
  if (NK > 0) {
    if ((rc = make_tmap_rows64(&mk128, p.k, dtype, NK, p.heads, batch, p.ks, 128, p.head_dim)) != ELSA_OK) return rc;
    if ((rc = make_tmap_rows64(&mv128, p.v, dtype, NK, p.heads, batch, p.vs, 128, p.head_dim)) != ELSA_OK) return rc;
  } else {
    mk128 = mv128 = mq64;   // never dereferenced: no key tile is visited
  }
  const dim3 qgrid(static_cast<unsigned>((N + 127) / 128), static_cast<unsigned>(bh));
  const dim3 kgrid(static_cast<unsigned>((NK + 127) / 128), static_cast<unsigned>(bh));
  auto launch = [&](auto dq_kernel, auto dkv_kernel) -> int {
    int r;
    if ((r = ensure_dynamic_smem(reinterpret_cast<const void*>(dq_kernel), kDqSmem)) != ELSA_OK) return r;
    if ((r = ensure_dynamic_smem(reinterpret_cast<const void*>(dkv_kernel), kKvSmem)) != ELSA_OK) return r;
    dq_kernel<<<qgrid, kThreads, kDqSmem, st>>>(mq128, mdo128, mk128, mv128, prm);
    if (NK > 0) dkv_kernel<<<kgrid, kThreads, kKvSmem, st>>>(mq64, mdo64, mk128, mv128, prm);
    return ELSA_OK;
  };
  rc = p.bias ? launch(&bwdw_dq_kernel<T, true>, &bwdw_dkv_kernel<T, true>) : launch(&bwdw_dq_kernel<T, false>, &bwdw_dkv_kernel<T, false>);
  if (rc != ELSA_OK) return rc;
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

int bwd_tcw(const BwdParams& p, const void* out, Strides os, const float* row_m, const float* row_z, void* workspace,
            int dtype, cudaStream_t st) {
  if (!bwd_tcw_supported(dtype, p.head_dim, p.bias != nullptr) || (p.dbias && !p.bias)) return ELSA_ERR_UNSUPPORTED;
  if (dtype == ELSA_F16) return bwd_tcw_t<__half>(p, out, os, row_m, row_z, workspace, dtype, st);
  return bwd_tcw_t<__nv_bfloat16>(p, out, os, row_m, row_z, workspace, dtype, st);
}

}  // namespace elsa
