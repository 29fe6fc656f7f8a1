// Backward for fp32 inputs on the 5th-generation tensor cores at fp32-grade accuracy: exact recompute from the saved
// row statistics, head dim 64 (or a smaller multiple of 8: the planes are zero-padded to 64 columns), causal or not, no
// bias.  Every operand of every contraction is split into 16-bit planes (two fp16 planes and three cross products, or
// three bf16 planes and six: ELSA_FP32_PLANES, tc_common.cuh) exactly as in the forward kernel for fp32 inputs
// (fold_tc3.cu); Q, K, V, dO by the same pre-pass, P and dS inside the kernels.
//
// tcgen05.mma adds into its fp32 accumulator by truncation, so -- unlike the 16-bit backward -- no gradient is
// accumulated over tiles in TMEM: every (query tile, key tile) pair gets fresh accumulators, and the running sums live
// in the registers of the threads that drain them (ordinary round-to-nearest additions).  A resident dK / dV with a
// streamed dQ (one kernel, five contractions) would need global atomics for dQ and more TMEM than there is, so the
// work is done by two kernels of the same shape as the forward one, seven contractions per pair in all:
//
//   bwd3_dq_kernel    one CTA per 128-row QUERY tile, 128-key tiles streamed:
//                       S  = Q K^T, dP = dO V^T       A = Q / dO planes (shared memory), B = K / V planes
//                       dS = P (dP - D), P = 2^(S c - LSE)          four threads per query row
//                       dQ_j = dS K                    A = dS planes (TMEM), B = the same K planes, MN-major
//                     dQ = scale * sum_j dQ_j in registers, written once: no atomics, deterministic
//   bwd3_dkv_kernel   one CTA per 128-row KEY tile, 64-query tiles streamed:
//                       S^T = K Q^T, dP^T = V dO^T     A = K / V planes (shared memory), B = Q / dO planes
//                       P^T, dS^T                      four threads per key row; -LSE, -D of the tile's queries
//                                                      arrive with the tile (bulk copies into a small ring)
//                       dV_i = P^T dO, dK_i = dS^T Q   A = P^T / dS^T planes (TMEM), B = the same dO / Q planes, MN-major
//                     dV = sum_i dV_i, dK = scale * sum_i dK_i in registers
//
// Both kernels: 16 fold warps (warp w: TMEM lanes 32 (w % 4) ..., column quarter w / 4 of the streamed tile),
// a TMA producer warp and an MMA-issuing warp; plane tiles through shared-memory rings in the order the issuer
// consumes them (planes from the lightest to the leading one: the cross terms are added in order of increasing
// weight).  The score / dP tiles of pair t+1 are issued as soon as the fold warps hold those of pair t in registers,
// so the exponentials and the splits of one pair overlap the contractions of its neighbours.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace elsa {

using namespace tc;

namespace {

constexpr int kSlotBytes = 64 * 64 * 2;      // one 64 x 64 bf16 plane tile (streamed operand)
constexpr int kPlaneBytes = 128 * 64 * 2;    // one 128 x 64 bf16 plane tile (the CTA's own operand)
constexpr int kFoldWarps = 16, kFoldThreads = kFoldWarps * 32;
constexpr int kThreads = kFoldThreads + 64;
constexpr int kProducerWarp = 16, kIssuerWarp = 17;
constexpr uint32_t kTmemCols = 512;
constexpr uint64_t kSlotStep = kSlotBytes >> 4;   // shared-memory descriptors count 16-byte units

// dQ kernel: Q and dO planes resident (96 KB), a ring of 6 K plane tiles and one of 2 V plane tiles (16 KB each)
constexpr int kDqKSlots = 2 * kPlanes, kDqVSlots = kPlanes == 2 ? 4 : 2;
constexpr int kDqSmem = (2 * kPlanes + kDqKSlots + kDqVSlots) * kPlaneBytes + 1024;
// dK/dV kernel: K and V planes resident (96 KB), 15 ring slots, 4 stages of (-LSE, -D) vectors of 64 queries
constexpr int kKvSlots = 15, kVecStages = 4, kVecBytes = 2 * 64 * 4;
constexpr int kKvSmem = 2 * kPlanes * kPlaneBytes + kKvSlots * kSlotBytes + kVecStages * kVecBytes + 1024;

enum BarId { BAR_ROW = 40, BAR_STAGE = 41, BAR_FULL = 42, BAR_FREE = 43, BAR_SDP = 45, BAR_SFREE = 46, BAR_DS = 47, BAR_ACC = 48 };

struct Bwd3Params {
  const float* nlse_pad; const float* nd_pad;   // [BH][n_pad]: -LSE, -D; padding rows hold -inf / 0
  const uint32_t* amax_q; const uint32_t* amax_do; const uint32_t* amax_k; const uint32_t* amax_v;   // the plane headers
  float* dq; float* dk; float* dv;
  Strides dqs, dks, dvs;
  int n_ctx, n_pad, bh, heads, is_causal;
  int n_keys, key_offset;                       // K/V rows of this launch and the sequence index of the first one
  int head_dim;                                 // real columns of the gradients (<= 64; the planes are zero-padded to 64)
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

// the first n (a multiple of 4, possibly <= 0) of 16 consecutive values of a gradient row
__device__ __forceinline__ void store16(float* dst, const float (&v)[16], float f, int n) {
#pragma unroll
  for (int i = 0; i < 16; i += 4)
    if (i < n) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i] * f, v[i + 1] * f, v[i + 2] * f, v[i + 3] * f);
}

// 16 values -> their planes, 8 TMEM columns per plane starting at column `col` of plane base tp0 + STRIDE p
template <int STRIDE>
__device__ __forceinline__ void split_store16(const float* x, uint32_t tp0, uint32_t col) {
  uint32_t pk[kPlanes][8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint32_t w[kPlanes];
    split_planes_pair(x[2 * i], x[2 * i + 1], w);
#pragma unroll
    for (int p = 0; p < kPlanes; ++p) pk[p][i] = w[p];
  }
#pragma unroll
  for (int p = 0; p < kPlanes; ++p) tmem_st8(tp0 + STRIDE * p + col, pk[p]);
}

// The scaled quantities of the fp16-plane scheme (all factors are powers of two; 1 with bf16 planes), s_x being the
// plane scale of tensor x:
//   S' = s_q s_k S, dP' = s_do s_v dP        arrive in TMEM; the fold divides the factors out
//   P' = P * 2^kLog2Unit                     probabilities are at most 1 (the unit rides in the exponent)
//   dS' = dS * r                             r = the power of two that puts the largest |dS| of this ROW of this tile
//                                            pair in [2^13, 2^14): dS = P (dP - D) is orders of magnitude below any
//                                            a-priori bound on long rows (P ~ 1/N), and a fixed scale would push its
//                                            second fp16 term into the subnormals (measured: dQ 2.5e-5 relative at
//                                            N = 65536).  The four threads of a row exchange their maxima through
//                                            shared memory; the accumulator of the tile pair is divided by r (and by
//                                            the scale of the other operand) when it is taken into the running sum.
// With bf16 planes r = 1 and no exchange happens.
__device__ __forceinline__ float abs_max16(const float* x) {
  float m0 = fmaxf(fabsf(x[0]), fabsf(x[1])), m1 = fmaxf(fabsf(x[2]), fabsf(x[3]));
#pragma unroll
  for (int i = 4; i < 16; i += 4) {
    m0 = fmaxf(m0, fmaxf(fabsf(x[i]), fabsf(x[i + 1])));
    m1 = fmaxf(m1, fmaxf(fabsf(x[i + 2]), fabsf(x[i + 3])));
  }
  return fmaxf(m0, m1);
}

// ------------------------------------------------------------------------------------------------------------------
// dQ: one CTA per 128-row query tile, 128-key tiles (N = 128 for S and dP: a tcgen05.mma with N = 64 costs 48-70
// cycles for 32 cycles of math, one with N = 128 costs 64 for 64)
// TMEM columns: S [0,128) dP [128,256) dQ_j [256,320) dS planes [320,512) (plane p at 320 + 64 p)
// Shared memory: Q planes, dO planes (resident, 96 KB) | K ring, 6 slots of 16 KB (the planes of key tile j stay until
// dQ_j has read them, while S of tile j+1 needs the next three) | V ring, 2 slots
// ------------------------------------------------------------------------------------------------------------------
template <bool BIAS>
__global__ void __launch_bounds__(kThreads, 1)
bwd3_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
               const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
               const Bwd3Params prm) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * (kDqKSlots + kDqVSlots) + 9];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float row_max[2][4][128];   // [tile parity][column quarter][row]: the quarter-row maxima of |dS|

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.y;
  const int q0 = blockIdx.x * 128;
  const int N = prm.n_ctx, NK = prm.n_keys, koff = prm.key_offset;
  int ke = NK;
  if (prm.is_causal) ke = min(ke, min(q0 + 128, N) - koff);   // keys above the tile's last row are never admissible
  const int n_t = ke > 0 ? (ke + 127) / 128 : 0;              // 128-key tiles this query tile visits

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto sQ = [&](int p) { return smem_base + p * kPlaneBytes; };
  auto sDO = [&](int p) { return smem_base + (kPlanes + p) * kPlaneBytes; };
  auto sKs = [&](int i) { return smem_base + (2 * kPlanes + i) * kPlaneBytes; };
  auto sVs = [&](int i) { return smem_base + (2 * kPlanes + kDqKSlots + i) * kPlaneBytes; };
  const uint32_t bar0 = smem_u32(bars);
  auto bar_kfull = [&](int i) { return bar0 + 8 * i; };
  auto bar_kfree = [&](int i) { return bar0 + 8 * (kDqKSlots + i); };
  auto bar_vfull = [&](int i) { return bar0 + 8 * (2 * kDqKSlots + i); };
  auto bar_vfree = [&](int i) { return bar0 + 8 * (2 * kDqKSlots + kDqVSlots + i); };
  const uint32_t barx = bar0 + 8 * 2 * (kDqKSlots + kDqVSlots);
  const uint32_t bar_stage = barx;            // the Q / dO planes are in shared memory
  const uint32_t bar_sdp = barx + 8;          // dP(j), S(j) are in TMEM
  const uint32_t bar_sfree = barx + 16;       // the fold warps hold them in registers
  const uint32_t bar_ds = barx + 24;          // the dS planes of tile j have been delivered
  const uint32_t bar_dq = barx + 32;          // dQ_j is complete
  auto bar_row = [&](int qd) { return barx + 40 + 8 * qd; };   // the four threads of a row have exchanged their maxima

  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < kDqKSlots; ++i) { mbar_init(bar_kfull(i), 1); mbar_init(bar_kfree(i), 1); }
    for (int i = 0; i < kDqVSlots; ++i) { mbar_init(bar_vfull(i), 1); mbar_init(bar_vfree(i), 1); }
    mbar_init(bar_stage, 1);
    mbar_init(bar_sdp, 1); mbar_init(bar_sfree, kFoldWarps);
    mbar_init(bar_ds, kFoldWarps); mbar_init(bar_dq, 1);
    for (int qd = 0; qd < 4; ++qd) mbar_init(bar_row(qd), 4);
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
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdQ = tmem_base + 256, tDS = tmem_base + 320;

  if (warp == kProducerWarp) {
    if (n_t > 0 && lane == 0) {
      // ---------------- TMA producer ----------------
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_do); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      mbar_arrive_expect_tx(bar_stage, 2 * kPlanes * kPlaneBytes);
      for (int p = 0; p < kPlanes; ++p) {
        tma_load_4d(sQ(p), &tmap_q, bar_stage, 0, q0, bh, p);
        tma_load_4d(sDO(p), &tmap_do, bar_stage, 0, q0, bh, p);
      }
      bool ok = true;
      // per key tile: its K planes (ring sequence numbers kPlanes j ...), then its V planes; planes in the order of
      // increasing weight.  A V slot is released by the dP group that read it, a K slot by the dQ group.
      for (int j = 0; j < n_t && ok; ++j) {
        for (int x = 0; x < kPlanes && ok; ++x) {
          const int seq = kPlanes * j + x, slot = seq % kDqKSlots;
          if (seq >= kDqKSlots && !(ok = mbar_wait(bar_kfree(slot), ((seq / kDqKSlots) - 1) & 1, &abort_flag, prm.status, BAR_FREE))) break;
          mbar_arrive_expect_tx(bar_kfull(slot), kPlaneBytes);
          tma_load_4d(sKs(slot), &tmap_k, bar_kfull(slot), 0, j * 128, bh, kPlanes - 1 - x);
        }
        for (int x = 0; x < kPlanes && ok; ++x) {
          const int seq = kPlanes * j + x, slot = seq % kDqVSlots;
          if (seq >= kDqVSlots && !(ok = mbar_wait(bar_vfree(slot), ((seq / kDqVSlots) - 1) & 1, &abort_flag, prm.status, BAR_FREE))) break;
          mbar_arrive_expect_tx(bar_vfull(slot), kPlaneBytes);
          tma_load_4d(sVs(slot), &tmap_v, bar_vfull(slot), 0, j * 128, bh, kPlanes - 1 - x);
        }
      }
    }
  } else if (warp == kIssuerWarp) {
    if (n_t > 0 && lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc_k = make_idesc(kPlaneFmt, 0, 0, 128, 128);   // S, dP: A, B K-major, N = 128 keys
      constexpr uint32_t idesc_mn = make_idesc(kPlaneFmt, 0, 1, 128, 64);   // dQ_j: A in TMEM, B (K) MN-major, N = 64 = d
      uint64_t dQp[kPlanes], dDOp[kPlanes];
      for (int p = 0; p < kPlanes; ++p) { dQp[p] = make_sdesc(sQ(p), 16, 1024); dDOp[p] = make_sdesc(sDO(p), 16, 1024); }
      const uint64_t dk_k0 = make_sdesc(sKs(0), 16, 1024), dk_mn0 = make_sdesc(sKs(0), 128 * 128, 1024);
      const uint64_t dv_k0 = make_sdesc(sVs(0), 16, 1024);
      constexpr uint64_t kPlaneStep = kPlaneBytes >> 4;
      bool ok = mbar_wait(bar_stage, 0, &abort_flag, prm.status, BAR_STAGE);
      auto issue_sdp = [&](int j) {
        bool first = true;
        for (int vp = kPlanes - 1; vp >= 0 && ok; --vp) {  // dP = dO V^T
          const int seq = kPlanes * j + kPlanes - 1 - vp, slot = seq % kDqVSlots;
          if (!(ok = mbar_wait(bar_vfull(slot), (seq / kDqVSlots) & 1, &abort_flag, prm.status, BAR_FULL))) return;
          tc_fence_after();
          for (int gp = kPlanes - 1 - vp; gp >= 0; --gp) {
            mma_ss_x4<2, 2>(tdP, dDOp[gp], dv_k0 + slot * kPlaneStep, idesc_k, first ? 0u : 1u);
            first = false;
          }
          mma_commit(bar_vfree(slot));
        }
        first = true;
        for (int kp = kPlanes - 1; kp >= 0 && ok; --kp) {  // S = Q K^T
          const int seq = kPlanes * j + kPlanes - 1 - kp, slot = seq % kDqKSlots;
          if (!(ok = mbar_wait(bar_kfull(slot), (seq / kDqKSlots) & 1, &abort_flag, prm.status, BAR_FULL))) return;
          tc_fence_after();
          for (int qp = kPlanes - 1 - kp; qp >= 0; --qp) {
            mma_ss_x4<2, 2>(tS, dQp[qp], dk_k0 + slot * kPlaneStep, idesc_k, first ? 0u : 1u);
            first = false;
          }                                   // the K planes stay: dQ_j reads them again
        }
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
        bool first = true;
        for (int kp = kPlanes - 1; kp >= 0; --kp) {        // dQ_j = dS K over the 128 keys (eight K-steps)
          const int slot = (kPlanes * j + kPlanes - 1 - kp) % kDqKSlots;
          for (int sp = kPlanes - 1 - kp; sp >= 0; --sp) {
            mma_ts_x4<8, 128>(tdQ, tDS + 64 * sp, dk_mn0 + slot * kPlaneStep, idesc_mn, first ? 0u : 1u);
            mma_ts_x4<8, 128>(tdQ, tDS + 64 * sp + 32, dk_mn0 + slot * kPlaneStep + 512, idesc_mn, 1u);
            first = false;
          }
          mma_commit(bar_kfree(slot));
        }
        mma_commit(bar_dq);                   // dQ_j is complete; the dS planes may be overwritten
      }
    }
  } else {
    // ---------------- fold warps: four threads per query row ----------------
    const int qd = warp & 3, cq = warp >> 2;                // TMEM lane quadrant, column quarter (32 keys)
    const int row = qd * 32 + lane;
    const int qi = q0 + row;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    // plane scales (powers of two; see abs_max16): S arrives times s_q s_k, dP times s_do s_v, dS leaves times the row scale of the tile
    const float s_q = plane_scale(*prm.amax_q), s_do = plane_scale(*prm.amax_do);
    const float s_k = plane_scale(*prm.amax_k), s_v = plane_scale(*prm.amax_v);
    const float c = prm.scale_log2 / (s_q * s_k);
    const float idp = 1.f / (s_do * s_v);
    const float nlse = prm.nlse_pad[static_cast<int64_t>(bh) * prm.n_pad + qi];   // q0 + 127 < n_pad
    const float nd = prm.nd_pad[static_cast<int64_t>(bh) * prm.n_pad + qi];
    float inv_r = 1.f;                         // 1 / (r s_k) of the tile whose dQ_j is in flight
    const float* bias_row = nullptr;
    float* dbias_row = nullptr;
    if constexpr (BIAS) {
      const int bi = bh / prm.heads, hi = bh - bi * prm.heads;
      const int qrow = min(qi, N - 1);         // rows beyond N are never stored: any valid address will do
      bias_row = prm.bias + bi * prm.bsb + hi * prm.bsh + static_cast<int64_t>(qrow) * prm.bsq;
      if (prm.dbias) dbias_row = prm.dbias + bi * prm.dsb + hi * prm.dsh + static_cast<int64_t>(qrow) * prm.dsq;
    }
    float dq_run[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) dq_run[i] = 0.f;
    bool alive = n_t > 0;

    auto take_dq = [&]() {
      uint32_t r[16];
      tmem_ld16(tdQ + lane_off + 16 * cq, r);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 16; ++i) dq_run[i] = fmaf(__uint_as_float(r[i]), inv_r, dq_run[i]);
    };

    for (int j = 0; alive && j < n_t; ++j) {
      if (!__all_sync(0xffffffffu, mbar_wait(bar_sdp, j & 1, &abort_flag, prm.status, BAR_SDP))) { alive = false; break; }
      tc_fence_after();
      float ds[32];
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
        if constexpr (BIAS) {
          const float* bp = bias_row + static_cast<int64_t>(kb + koff) * prm.bsk;
          if (prm.bsk == 1 && kb + 32 <= NK && (reinterpret_cast<uintptr_t>(bp) & 31u) == 0) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float b8[8];
              ld_global_v8(bp + 8 * g, b8);      // whole 32-byte sectors (a warp's 32 rows are 32 different lines)
#pragma unroll
              for (int e = 0; e < 8; ++e) ab[8 * g + e] = fmaf(b8[e], 1.4426950408889634f, nlse);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (kb + i < NK) ab[i] = fmaf(bp[i * prm.bsk], 1.4426950408889634f, nlse);
          }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float p = fast_exp2(fmaf(__uint_as_float(rs[i]), c, ab[i]));
          if (masked && kb + i > lim) p = 0.f;
          ds[i] = p * fmaf(__uint_as_float(rp[i]), idp, nd);
        }
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
                for (int e = 0; e < 8; ++e) d8[e] = ds[8 * g + e];
                st_global_v8(dp + 8 * g, d8);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (kb + i > lim) continue;
                if (prm.dbias_atomic) atomicAdd(dp + i * prm.dsk, ds[i]); else dp[i * prm.dsk] = ds[i];
              }
            }
          }
        }
      }
      float r_scale = 1.f;
      if (kPlanes == 2) {
        // the row's scale for this tile: the largest |dS| over its 128 keys, exchanged between the row's four threads
        row_max[j & 1][cq][row] = fmaxf(abs_max16(ds), abs_max16(ds + 16));
        mbar_arrive_warp(bar_row(qd), lane);
        if (!__all_sync(0xffffffffu, mbar_wait(bar_row(qd), j & 1, &abort_flag, prm.status, BAR_ROW))) { alive = false; break; }
        const float mx = fmaxf(fmaxf(row_max[j & 1][0][row], row_max[j & 1][1][row]), fmaxf(row_max[j & 1][2][row], row_max[j & 1][3][row]));
        r_scale = plane_scale(__float_as_uint(mx));
#pragma unroll
        for (int i = 0; i < 32; ++i) ds[i] *= r_scale;
      }
      if (j > 0) {
        // dQ of the previous key tile has retired: it goes into the running sum, and the dS planes are free
        if (!__all_sync(0xffffffffu, mbar_wait(bar_dq, (j - 1) & 1, &abort_flag, prm.status, BAR_ACC))) { alive = false; break; }
        tc_fence_after();
        take_dq();
      }
      inv_r = 1.f / (r_scale * s_k);
      // the planes of dS: 16 keys (8 TMEM columns per plane) at a time
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) split_store16<64>(ds + 16 * ch, tDS + lane_off, 16 * cq + 8 * ch);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(bar_ds, lane);
    }
    if (alive && n_t > 0) {
      if (!__all_sync(0xffffffffu, mbar_wait(bar_dq, (n_t - 1) & 1, &abort_flag, prm.status, BAR_ACC))) alive = false;
      if (alive) {
        tc_fence_after();
        take_dq();
      }
    }
    if (qi < N && (alive || n_t == 0)) {
      const int bi = bh / prm.heads, hi = bh - bi * prm.heads;
      store16(prm.dq + bi * prm.dqs.b + hi * prm.dqs.h + static_cast<int64_t>(qi) * prm.dqs.r + 16 * cq, dq_run, prm.scale, prm.head_dim - 16 * cq);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------------------------------------------------
// dK, dV: one CTA per 128-row key tile
// TMEM columns: S^T [0,64) dP^T [64,128) P^T planes [128,224) dS^T planes [224,320) dV_i [320,384) dK_i [384,448)
// ------------------------------------------------------------------------------------------------------------------
template <bool BIAS>
__global__ void __launch_bounds__(kThreads, 1)
bwd3_dkv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                const Bwd3Params prm) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kKvSlots + 9];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float row_max[2][4][128];   // [tile parity][column quarter][key row]: the quarter-row maxima of |dS^T|

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.y;
  const int k0 = blockIdx.x * 128;                  // first (local) key row of this CTA
  const int N = prm.n_ctx, NK = prm.n_keys;
  const int kseq0 = k0 + prm.key_offset;            // its index in the sequence
  const int n_q64 = (N + 63) / 64;
  const int it_begin = prm.is_causal ? min(n_q64, kseq0 / 64) : 0;   // query tiles above the diagonal see none of these keys
  const int n_it = n_q64 - it_begin;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  auto sK = [&](int p) { return smem_base + p * kPlaneBytes; };
  auto sV = [&](int p) { return smem_base + (kPlanes + p) * kPlaneBytes; };
  auto sSlot = [&](int i) { return smem_base + 2 * kPlanes * kPlaneBytes + i * kSlotBytes; };
  const uint32_t vec_off = 2 * kPlanes * kPlaneBytes + kKvSlots * kSlotBytes;    // [stage][-LSE x 64 | -D x 64]
  const uint32_t bar0 = smem_u32(bars);
  auto bar_full = [&](int i) { return bar0 + 8 * i; };
  auto bar_free = [&](int i) { return bar0 + 8 * (kKvSlots + i); };
  const uint32_t barx = bar0 + 8 * 2 * kKvSlots;
  const uint32_t bar_kv = barx;               // the K / V planes are in shared memory
  const uint32_t bar_sdp = barx + 8;          // S^T(i), dP^T(i) are in TMEM
  const uint32_t bar_sfree = barx + 16;       // the fold warps hold them in registers
  const uint32_t bar_pl = barx + 24;          // the P^T / dS^T planes of tile i have been delivered
  const uint32_t bar_acc = barx + 32;         // dV_i, dK_i are complete
  auto bar_row = [&](int qd) { return barx + 40 + 8 * qd; };   // the four threads of a key row have exchanged their maxima

  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < kKvSlots; ++i) { mbar_init(bar_full(i), 1); mbar_init(bar_free(i), 1); }
    mbar_init(bar_kv, 1);
    mbar_init(bar_sdp, 1); mbar_init(bar_sfree, kFoldWarps);
    mbar_init(bar_pl, kFoldWarps); mbar_init(bar_acc, 1);
    for (int qd = 0; qd < 4; ++qd) mbar_init(bar_row(qd), 4);
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
  const uint32_t tS = tmem_base, tdP = tmem_base + 64, tP = tmem_base + 128, tDS = tmem_base + 224;
  const uint32_t tdV = tmem_base + 320, tdK = tmem_base + 384;

  if (warp == kProducerWarp) {
    if (n_it > 0 && lane == 0) {
      // ---------------- TMA producer ----------------
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_do); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      mbar_arrive_expect_tx(bar_kv, 2 * kPlanes * kPlaneBytes);
      for (int p = 0; p < kPlanes; ++p) {
        tma_load_4d(sK(p), &tmap_k, bar_kv, 0, k0, bh, p);
        tma_load_4d(sV(p), &tmap_v, bar_kv, 0, k0, bh, p);
      }
      int seq = 0;
      bool ok = true;
      // ring order of query tile i: its dO planes from the lightest to the leading one (sequence numbers
      // 2 kPlanes i ...), then its Q planes; the tile's first slot also receives its -LSE / -D vectors
      for (int it = 0; it < n_it && ok; ++it) {
        const int qrow = (it_begin + it) * 64;
        for (int x = 0; x < 2 * kPlanes && ok; ++x) {
          const int slot = seq % kKvSlots;
          if (seq >= kKvSlots && !(ok = mbar_wait(bar_free(slot), ((seq / kKvSlots) - 1) & 1, &abort_flag, prm.status, BAR_FREE))) break;
          mbar_arrive_expect_tx(bar_full(slot), kSlotBytes + (x == 0 ? kVecBytes : 0));
          tma_load_4d(sSlot(slot), x < kPlanes ? &tmap_do : &tmap_q, bar_full(slot), 0, qrow, bh, kPlanes - 1 - (x % kPlanes));
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
      constexpr uint32_t idesc_k = make_idesc(kPlaneFmt, 0, 0, 128, 64);    // S^T, dP^T: A, B K-major, N = 64 queries
      constexpr uint32_t idesc_mn = make_idesc(kPlaneFmt, 0, 1, 128, 64);   // dV_i, dK_i: A in TMEM, B MN-major, N = 64 = d
      uint64_t dKp[kPlanes], dVp[kPlanes];
      for (int p = 0; p < kPlanes; ++p) { dKp[p] = make_sdesc(sK(p), 16, 1024); dVp[p] = make_sdesc(sV(p), 16, 1024); }
      constexpr int kT = 2 * kPlanes;   // ring entries per query tile
      const uint64_t dk_slot0 = make_sdesc(sSlot(0), 16, 1024), dmn_slot0 = make_sdesc(sSlot(0), 64 * 128, 1024);
      bool ok = mbar_wait(bar_kv, 0, &abort_flag, prm.status, BAR_STAGE);
      auto issue_sdp = [&](int it) {
        bool first = true;
        for (int gp = kPlanes - 1; gp >= 0 && ok; --gp) {  // dP^T = V dO^T
          const int seq = kT * it + kPlanes - 1 - gp, slot = seq % kKvSlots;
          if (!(ok = mbar_wait(bar_full(slot), (seq / kKvSlots) & 1, &abort_flag, prm.status, BAR_FULL))) return;
          tc_fence_after();
          for (int vp = kPlanes - 1 - gp; vp >= 0; --vp) {
            mma_ss_x4<2, 2>(tdP, dVp[vp], dk_slot0 + slot * kSlotStep, idesc_k, first ? 0u : 1u);
            first = false;
          }
        }
        first = true;
        for (int qp = kPlanes - 1; qp >= 0 && ok; --qp) {  // S^T = K Q^T
          const int seq = kT * it + kT - 1 - qp, slot = seq % kKvSlots;
          if (!(ok = mbar_wait(bar_full(slot), (seq / kKvSlots) & 1, &abort_flag, prm.status, BAR_FULL))) return;
          tc_fence_after();
          for (int kp = kPlanes - 1 - qp; kp >= 0; --kp) {
            mma_ss_x4<2, 2>(tS, dKp[kp], dk_slot0 + slot * kSlotStep, idesc_k, first ? 0u : 1u);
            first = false;
          }
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
        bool first = true;
        for (int gp = kPlanes - 1; gp >= 0; --gp) {        // dV_i = P^T dO
          const int slot = (kT * it + kPlanes - 1 - gp) % kKvSlots;
          for (int pp = kPlanes - 1 - gp; pp >= 0; --pp) {
            mma_ts_x4<8, 128>(tdV, tP + 32 * pp, dmn_slot0 + slot * kSlotStep, idesc_mn, first ? 0u : 1u);
            first = false;
          }
          mma_commit(bar_free(slot));
        }
        first = true;
        for (int qp = kPlanes - 1; qp >= 0; --qp) {        // dK_i = dS^T Q
          const int slot = (kT * it + kT - 1 - qp) % kKvSlots;
          for (int sp = kPlanes - 1 - qp; sp >= 0; --sp) {
            mma_ts_x4<8, 128>(tdK, tDS + 32 * sp, dmn_slot0 + slot * kSlotStep, idesc_mn, first ? 0u : 1u);
            first = false;
          }
          mma_commit(bar_free(slot));
        }
        mma_commit(bar_acc);                  // dV_i, dK_i are complete; the planes may be overwritten
      }
    }
  } else {
    // ---------------- fold warps: four threads per key row ----------------
    const int qd = warp & 3, cq = warp >> 2;                // TMEM lane quadrant, column quarter
    const int row = qd * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const int key = k0 + row;                  // local key row
    const int key_seq = kseq0 + row;           // its index in the sequence (what the causal rule compares)
    const bool key_ok = key < NK;
    const bool cta_tail = k0 + 128 > NK;       // some key rows of this CTA do not exist
    // plane scales (powers of two; see abs_max16): S^T arrives times s_q s_k, dP^T times s_do s_v; P^T leaves times
    // 2^kLog2Unit (the unit rides in the exponent), dS^T times this key row's scale for the tile
    const float s_q = plane_scale(*prm.amax_q), s_do = plane_scale(*prm.amax_do);
    const float s_k = plane_scale(*prm.amax_k), s_v = plane_scale(*prm.amax_v);
    const float c = prm.scale_log2 / (s_q * s_k);
    const float k2 = exp2f(-kLog2Unit);                 // dS = P' * (dP + nd) * k2
    const float idp = k2 / (s_do * s_v);
    const float inv_v = k2 / s_do;                      // dV_i' = 2^kLog2Unit s_do dV_i
    float inv_r = 1.f;                                  // 1 / (r s_q) of the tile whose dK_i is in flight
    // bias[query, key] of this thread's key column; the query offset is added per element
    const float* bias_col = nullptr;
    if constexpr (BIAS) {
      const int bi = bh / prm.heads, hi = bh - bi * prm.heads;
      bias_col = prm.bias + bi * prm.bsb + hi * prm.bsh + static_cast<int64_t>(min(key_seq, N - 1)) * prm.bsk;
    }
    float dv_run[16], dk_run[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) { dv_run[i] = 0.f; dk_run[i] = 0.f; }
    bool alive = true;

    auto take_acc = [&]() {
      uint32_t rv[16], rk[16];
      tmem_ld16(tdV + lane_off + 16 * cq, rv);
      tmem_ld16(tdK + lane_off + 16 * cq, rk);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        dv_run[i] = fmaf(__uint_as_float(rv[i]), inv_v, dv_run[i]);
        dk_run[i] = fmaf(__uint_as_float(rk[i]), inv_r, dk_run[i]);
      }
    };

    for (int it = 0; it < n_it; ++it) {
      const int q_tile0 = (it_begin + it) * 64;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_sdp, it & 1, &abort_flag, prm.status, BAR_SDP))) { alive = false; break; }
      // the tile's row statistics were written by the bulk copies that complete on its first slot's barrier: observe
      // that barrier directly (it completed before the MMAs behind bar_sdp were issued, so this never spins)
      {
        const int seq = 2 * kPlanes * it;
        if (!__all_sync(0xffffffffu, mbar_wait(bar_full(seq % kKvSlots), (seq / kKvSlots) & 1, &abort_flag, prm.status, BAR_FULL))) { alive = false; break; }
      }
      tc_fence_after();
      float p[16], ds[16];
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
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = 4 * g + e;
            float a = nle[e] + kLog2Unit;
            if constexpr (BIAS) a += bb[i];
            float pv = fast_exp2(fmaf(__uint_as_float(rs[i]), c, a));
            if (masked && !(key_ok && (!prm.is_causal || qc + i >= key_seq))) pv = 0.f;
            p[i] = pv;
            ds[i] = pv * fmaf(__uint_as_float(rp[i]), idp, nde[e] * k2);
          }
        }
      }
      float r_scale = 1.f;
      if (kPlanes == 2) {
        // the key row's scale for this tile: the largest |dS^T| over its 64 queries, exchanged between its four threads
        row_max[it & 1][cq][row] = abs_max16(ds);
        mbar_arrive_warp(bar_row(qd), lane);
        if (!__all_sync(0xffffffffu, mbar_wait(bar_row(qd), it & 1, &abort_flag, prm.status, BAR_ROW))) { alive = false; break; }
        const float mx = fmaxf(fmaxf(row_max[it & 1][0][row], row_max[it & 1][1][row]), fmaxf(row_max[it & 1][2][row], row_max[it & 1][3][row]));
        r_scale = plane_scale(__float_as_uint(mx));
#pragma unroll
        for (int i = 0; i < 16; ++i) ds[i] *= r_scale;
      }
      if (it > 0) {
        // dV, dK of the previous query tile have retired: they go into the running sums, and the planes are free
        if (!__all_sync(0xffffffffu, mbar_wait(bar_acc, (it - 1) & 1, &abort_flag, prm.status, BAR_ACC))) { alive = false; break; }
        tc_fence_after();
        take_acc();
      }
      inv_r = 1.f / (r_scale * s_q);
      split_store16<32>(p, tP + lane_off, 8 * cq);
      split_store16<32>(ds, tDS + lane_off, 8 * cq);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(bar_pl, lane);
    }
    if (alive && n_it > 0) {
      if (!__all_sync(0xffffffffu, mbar_wait(bar_acc, (n_it - 1) & 1, &abort_flag, prm.status, BAR_ACC))) alive = false;
      if (alive) {
        tc_fence_after();
        take_acc();
      }
    }
    if (key_ok && alive) {
      const int bi = bh / prm.heads, hi = bh - bi * prm.heads;
      store16(prm.dk + bi * prm.dks.b + hi * prm.dks.h + static_cast<int64_t>(key) * prm.dks.r + 16 * cq, dk_run, prm.scale, prm.head_dim - 16 * cq);
      store16(prm.dv + bi * prm.dvs.b + hi * prm.dvs.h + static_cast<int64_t>(key) * prm.dvs.r + 16 * cq, dv_run, 1.f, prm.head_dim - 16 * cq);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) tmem_dealloc(tmem_base, kTmemCols);
}

// -D = -sum_d out*dout, -LSE = -(m + log2(max(z, 1e-30))) into the padded layout; padding: -D = 0, -LSE = -inf
__global__ void __launch_bounds__(256)
bwd3_preprocess_kernel(const float* __restrict__ out, const float* __restrict__ dout, const float* __restrict__ row_m,
                       const float* __restrict__ row_z, float* __restrict__ nd_pad, float* __restrict__ nlse_pad,
                       int heads, int n_ctx, int n_pad, int head_dim, Strides os, Strides gs) {
  // blockIdx.y = (batch*head); x covers the n_pad padded rows, 16 lanes (16 bytes each) per row
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = static_cast<int>(gid >> 4);
  const int lane = static_cast<int>(gid & 15);
  const int64_t b = blockIdx.y;
  const bool in_pad = r < n_pad;
  const bool real = in_pad && r < n_ctx;
  float part = 0.f;
  if (real && lane * 4 < head_dim) {
    const int bi = static_cast<int>(b) / heads, hi = static_cast<int>(b) - bi * heads;
    const float4 o = *reinterpret_cast<const float4*>(out + bi * os.b + hi * os.h + static_cast<int64_t>(r) * os.r + lane * 4);
    const float4 g = *reinterpret_cast<const float4*>(dout + bi * gs.b + hi * gs.h + static_cast<int64_t>(r) * gs.r + lane * 4);
    part = (o.x * g.x + o.y * g.y) + (o.z * g.z + o.w * g.w);
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

bool bwd_tc3_supported(int dtype, int head_dim, bool has_bias) { return fold_tc3_supported(dtype, head_dim, has_bias); }

int64_t bwd_tc3_workspace_bytes(int bh, int n_ctx, int n_keys) {
  const int64_t n_pad = align_up(n_ctx, 128);
  return 2 * align_up(static_cast<int64_t>(bh) * n_pad * 4, 256) + 2 * fold_tc3_plane_bytes(bh, n_ctx) +
         2 * fold_tc3_plane_bytes(bh, n_keys);
}

int bwd_tc3(const BwdParams& p, const void* out, Strides os, const float* row_m, const float* row_z, void* workspace,
            cudaStream_t st) {
  if (!bwd_tc3_supported(ELSA_F32, p.head_dim, p.bias != nullptr) || (p.dbias && !p.bias)) return ELSA_ERR_UNSUPPORTED;
  const int N = p.n_ctx, NK = p.n_keys, bh = p.bh, batch = bh / p.heads;
  const int n_pad = static_cast<int>(align_up(N, 128));
  const int64_t vec_bytes = align_up(static_cast<int64_t>(bh) * n_pad * 4, 256);
  const int64_t qb = fold_tc3_plane_bytes(bh, N), kb = fold_tc3_plane_bytes(bh, NK);
  char* ws = static_cast<char*>(workspace);
  float* nd_pad = reinterpret_cast<float*>(ws);
  float* nlse_pad = reinterpret_cast<float*>(ws + vec_bytes);
  char* q3 = ws + 2 * vec_bytes;
  char* do3 = q3 + qb;
  char* k3 = do3 + qb;
  char* v3 = k3 + kb;
  int rc;
  {
    const dim3 pgrid(static_cast<unsigned>(cdiv64(static_cast<int64_t>(n_pad) * 16, 256)), static_cast<unsigned>(bh));
    bwd3_preprocess_kernel<<<pgrid, 256, 0, st>>>(static_cast<const float*>(out), static_cast<const float*>(p.dout), row_m,
                                                  row_z, nd_pad, nlse_pad, p.heads, N, n_pad, p.head_dim, os, p.gs);
    ELSA_LAUNCH_CHECK();
  }
  {
    const void* xs[4] = {p.q, p.dout, p.k, p.v};
    const Strides sts[4] = {p.qs, p.gs, p.ks, p.vs};
    void* pls[4] = {q3, do3, k3, v3};
    const int rws[4] = {N, N, NK, NK};
    if ((rc = fold_tc3_split_many(4, xs, sts, pls, rws, batch, p.heads, p.head_dim, st)) != ELSA_OK) return rc;
  }

  // planes as [kPlanes, B*H, rows, 64] 16-bit tensors: the "head" coordinate is (batch*head), the "batch" coordinate the plane
  const Strides sq = contiguous_strides(bh, N, 64), sk = contiguous_strides(bh, NK, 64);
  CUtensorMap mq128, mdo128, mq64, mdo64, mk128, mv128;
  if ((rc = make_tmap_rows64(&mq128, q3 + kPlaneHeader, kPlaneDtype, N, bh, kPlanes, sq, 128)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mdo128, do3 + kPlaneHeader, kPlaneDtype, N, bh, kPlanes, sq, 128)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mq64, q3 + kPlaneHeader, kPlaneDtype, N, bh, kPlanes, sq, 64)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mdo64, do3 + kPlaneHeader, kPlaneDtype, N, bh, kPlanes, sq, 64)) != ELSA_OK) return rc;
  Bwd3Params prm;
  if ((rc = device_status_word(&prm.status, nullptr)) != ELSA_OK) return rc;
  prm.nlse_pad = nlse_pad; prm.nd_pad = nd_pad;
  prm.amax_q = reinterpret_cast<const uint32_t*>(q3) + kAmaxFinal; prm.amax_do = reinterpret_cast<const uint32_t*>(do3) + kAmaxFinal;
  prm.amax_k = reinterpret_cast<const uint32_t*>(k3) + kAmaxFinal; prm.amax_v = reinterpret_cast<const uint32_t*>(v3) + kAmaxFinal;
  prm.dq = static_cast<float*>(p.dq); prm.dk = static_cast<float*>(p.dk); prm.dv = static_cast<float*>(p.dv);
  prm.dqs = p.dqs; prm.dks = p.dks; prm.dvs = p.dvs;
  prm.n_ctx = N; prm.n_pad = n_pad; prm.bh = bh; prm.heads = p.heads; prm.is_causal = p.is_causal;
  prm.n_keys = NK; prm.key_offset = p.key_offset; prm.head_dim = p.head_dim;
  prm.scale = p.scale; prm.scale_log2 = p.scale_log2;
  prm.bias = p.bias; prm.bsb = p.bsb; prm.bsh = p.bsh; prm.bsq = p.bsq; prm.bsk = p.bsk;
  prm.dbias = p.dbias; prm.dsb = p.dsb; prm.dsh = p.dsh; prm.dsq = p.dsq; prm.dsk = p.dsk; prm.dbias_atomic = p.dbias_atomic;
  if (NK > 0) {
    if ((rc = make_tmap_rows64(&mk128, k3 + kPlaneHeader, kPlaneDtype, NK, bh, kPlanes, sk, 128)) != ELSA_OK) return rc;
    if ((rc = make_tmap_rows64(&mv128, v3 + kPlaneHeader, kPlaneDtype, NK, bh, kPlanes, sk, 128)) != ELSA_OK) return rc;
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
  rc = p.bias ? launch(&bwd3_dq_kernel<true>, &bwd3_dkv_kernel<true>) : launch(&bwd3_dq_kernel<false>, &bwd3_dkv_kernel<false>);
  if (rc != ELSA_OK) return rc;
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

}  // namespace elsa
