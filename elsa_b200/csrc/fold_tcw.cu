// Phase 1 on the 5th-generation tensor cores for fp16 / bf16 inputs with a WIDE head: 64 < d <= 128 (multiples of 8),
// and for BIASED problems of any head dim up to 128 (the additive bias is read from global memory by the fold warps;
// with d <= 64 only the first half below exists).
// The head dim is handled as two 64-column halves of the same tensors (the second half zero-padded by the TMA box
// when d < 128):
//     S   = Q_lo K_lo^T + Q_hi K_hi^T          two K = 64 contractions into one accumulator   (N = 128 keys)
//     O_h = P V_h,  h = lo, hi                 one contraction per half, own accumulator      (N = 64)
// The 16-bit kernel for d <= 64 (fold_tc.cu) keeps two query tiles with their S, O and P in TMEM; with 128 output
// columns per tile that no longer fits, so this kernel has the shape of the fp32 one (fold_tc3.cu): ONE 128-row query
// tile per CTA (576 threads, 1 per SM), walked in 128-key tiles,
//
//   warp 16     TMA producer   the two halves of the Q tile once; then 16 KB tiles through an 8-slot ring in the order
//                              the issuer consumes them: K halves of key tile j+1, V halves of key tile j
//   warp 17     MMA issuer     S(j+1) (8 x tcgen05.mma 128x128x16) as soon as the fold warps hold S(j) in registers;
//                              O_lo, O_hi of key tile j (2 x 8 x tcgen05.mma 128x64x16, P from TMEM, V MN-major)
//   warps 0-15  fold           four threads per query row (warp w: rows 32 (w % 4) ..., key columns 32 (w / 4) ...):
//                              scores into registers, row max exchanged through shared memory, exp2, row sum, P
//                              (16-bit) into its own TMEM columns; each thread keeps the running sum of 2 x 16 output
//                              columns in registers and takes in O of the previous key tile
//
// Exp-rescale merge as in fold_tc.cu: the reference max only moves when the tile max exceeds it by more than 2^8; the
// true running max is tracked separately and the summary is renormalised to it in the epilogue.
// TMEM columns: S [0,128) O_lo [128,192) O_hi [192,256) P [256,320).
#include <type_traits>

#include "kernels.cuh"
#include "tc_common.cuh"

namespace elsa {

using namespace tc;

namespace {

constexpr int kSlots = 8;
constexpr int kTileBytes = 128 * 64 * 2;                     // one 128 x 64 16-bit tile
constexpr int kFoldWSmem = (2 + kSlots) * kTileBytes + 1024;  // + alignment slack
constexpr int kFoldWarps = 16, kFoldThreads = kFoldWarps * 32;
constexpr int kThreads = kFoldThreads + 64;
constexpr uint32_t kTmemCols = 512;
constexpr int kProducerWarp = 16, kIssuerWarp = 17;
constexpr float kRescaleThreshold = 8.0f;

enum BarId { BAR_Q = 51, BAR_FULL = 52, BAR_FREE = 53, BAR_S = 54, BAR_P = 55, BAR_O = 56, BAR_SFREE = 57, BAR_PV = 58, BAR_ROW = 59 };

struct FoldWParams {
  float* m; float* z; void* s;
  int n_ctx, q_start, q_len, part_width, n_parts, bh, heads, is_causal, summary_dtype;
  int n_keys, key_offset, head_dim;
  int n_halves;                                 // 1 when head_dim <= 64 (biased problems), else 2
  float scale_log2;
  const float* bias; int64_t bsb, bsh, bsq, bsk;  // additive bias [.., N, N] (natural-log units) or null
  int* status;
};

__device__ __forceinline__ float max3w(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 16 consecutive values of a summary row, of which the first n (a multiple of 8, possibly <= 0) exist
template <typename TS>
__device__ __forceinline__ void store_row16(TS* dst, const float* v, int n) {
  if constexpr (sizeof(TS) == 4) {
#pragma unroll
    for (int i = 0; i < 16; i += 4)
      if (i < n) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; i += 8) {
      if (i >= n) continue;
      uint4 t;
      t.x = pack2<TS>(v[i], v[i + 1]); t.y = pack2<TS>(v[i + 2], v[i + 3]);
      t.z = pack2<TS>(v[i + 4], v[i + 5]); t.w = pack2<TS>(v[i + 6], v[i + 7]);
      *reinterpret_cast<uint4*>(dst + i) = t;
    }
  }
}

template <typename T, bool BIAS>
__global__ void __launch_bounds__(kThreads, 1)
fold_tcw_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const FoldWParams prm) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kSlots + 9];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float row_max[2][4][128];   // [key-tile parity][column quarter][row]: the quarter-row maxima
  __shared__ float row_sum[4][128];      // the quarter-row sums, exchanged once in the epilogue

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.z, part = blockIdx.y;
  const int bi = bh / prm.heads, hi = bh - bi * prm.heads;  // tensor-map coordinates of this (batch*head)
  // causal: a tile's work grows with its first row, so the tiles are handed out from the last one down -- the long
  // ones first, the short ones fill the end of the last wave
  const int bx = prm.is_causal ? static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
  const int q0 = prm.q_start + bx * 128;
  const int q_end = prm.q_start + prm.q_len;
  const int k_begin = part * prm.part_width;
  const int k_end = min(prm.n_keys, k_begin + prm.part_width);   // local key indices
  const int koff = prm.key_offset;
  int ke = k_end;
  if (prm.is_causal) ke = min(ke, min(q0 + 128, q_end) - koff);   // keys above the tile's last row are never admissible
  const int n_t = (q0 < q_end && ke > k_begin) ? (ke - k_begin + 127) / 128 : 0;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto sQ = [&](int h) { return smem_base + h * kTileBytes; };
  auto sSlot = [&](int i) { return smem_base + (2 + i) * kTileBytes; };
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_q = bar0;
  auto bar_full = [&](int i) { return bar0 + 8 * (1 + i); };
  auto bar_free = [&](int i) { return bar0 + 8 * (1 + kSlots + i); };
  const uint32_t bar_s = bar0 + 8 * (1 + 2 * kSlots);        // S(j) is in TMEM
  const uint32_t bar_sfree = bar0 + 8 * (2 + 2 * kSlots);    // the fold warps hold S(j) in registers
  const uint32_t bar_p = bar0 + 8 * (3 + 2 * kSlots);        // P of tile j has been delivered
  const uint32_t bar_pv = bar0 + 8 * (4 + 2 * kSlots);       // O_lo, O_hi of tile j are complete
  auto bar_row = [&](int qd) { return bar0 + 8 * (5 + 2 * kSlots + qd); };   // the four threads of a row have exchanged

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_q, 1);
    for (int i = 0; i < kSlots; ++i) { mbar_init(bar_full(i), 1); mbar_init(bar_free(i), 1); }
    mbar_init(bar_s, 1); mbar_init(bar_sfree, kFoldWarps);
    mbar_init(bar_p, kFoldWarps); mbar_init(bar_pv, 1);
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
  const uint32_t tS = tmem_base;
  const uint32_t tO = tmem_base + 128;                   // O_lo, O_hi at + 64 h
  const uint32_t tP = tmem_base + 256;

  if (warp == kProducerWarp) {
    if (n_t > 0 && lane == 0) {
      // ---------------- TMA producer ----------------
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      const int nh = BIAS ? prm.n_halves : 2;
      mbar_arrive_expect_tx(bar_q, nh * kTileBytes);
      for (int h = 0; h < nh; ++h) tma_load_4d(sQ(h), &tmap_q, bar_q, 64 * h, q0, hi, bi);
      int seq = 0;
      bool ok = true;
      auto load = [&](const CUtensorMap* map, int tile, int half) {
        const int slot = seq % kSlots;
        if (seq >= kSlots && !mbar_wait(bar_free(slot), ((seq / kSlots) - 1) & 1, &abort_flag, prm.status, BAR_FREE)) { ok = false; return; }
        mbar_arrive_expect_tx(bar_full(slot), kTileBytes);
        tma_load_4d(sSlot(slot), map, bar_full(slot), 64 * half, k_begin + tile * 128, hi, bi);
        ++seq;
      };
      for (int h = 0; h < nh && ok; ++h) load(&tmap_k, 0, h);
      for (int j = 0; j < n_t && ok; ++j) {
        if (j + 1 < n_t)
          for (int h = 0; h < nh && ok; ++h) load(&tmap_k, j + 1, h);
        for (int h = 0; h < nh && ok; ++h) load(&tmap_v, j, h);
      }
    }
  } else if (warp == kIssuerWarp) {
    if (n_t > 0 && lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc_s = make_idesc(fmt, 0, 0, 128, 128);   // S += Q_h K_h^T : A, B K-major
      constexpr uint32_t idesc_o = make_idesc(fmt, 0, 1, 128, 64);    // O_h = P V_h    : A in TMEM, B (V) MN-major
      const uint64_t dq[2] = {make_sdesc(sQ(0), 16, 1024), make_sdesc(sQ(1), 16, 1024)};
      const uint64_t dk_slot0 = make_sdesc(sSlot(0), 16, 1024), dv_slot0 = make_sdesc(sSlot(0), 128 * 128, 1024);
      constexpr uint64_t kSlotStep = kTileBytes >> 4;   // descriptor address field counts 16-byte units
      int seq = 0;
      const int nh = BIAS ? prm.n_halves : 2;
      bool ok = mbar_wait(bar_q, 0, &abort_flag, prm.status, BAR_Q);
      auto issue_s = [&]() {
        for (int h = 0; h < nh && ok; ++h) {
          const int slot = seq % kSlots;
          if (!(ok = mbar_wait(bar_full(slot), (seq / kSlots) & 1, &abort_flag, prm.status, BAR_FULL))) return;
          tc_fence_after();
          mma_ss_x4<2, 2>(tS, dq[h], dk_slot0 + slot * kSlotStep, idesc_s, h == 0 ? 0u : 1u);
          mma_commit(bar_free(slot));     // the tile is free again once these MMAs have retired
          ++seq;
        }
        if (ok) mma_commit(bar_s);
      };
      if (ok) issue_s();
      for (int j = 0; ok && j < n_t; ++j) {
        if (j + 1 < n_t) {
          // S(j+1) as soon as the fold warps hold S(j) in registers: it runs while they work on tile j
          if (!(ok = mbar_wait(bar_sfree, j & 1, &abort_flag, prm.status, BAR_SFREE))) break;
          tc_fence_after();
          issue_s();
          if (!ok) break;
        }
        if (!(ok = mbar_wait(bar_p, j & 1, &abort_flag, prm.status, BAR_P))) break;
        tc_fence_after();
        // O_lo, O_hi of this key tile start from zero (the fold warps took the previous ones into their registers)
        for (int h = 0; h < nh && ok; ++h) {
          const int slot = seq % kSlots;
          if (!(ok = mbar_wait(bar_full(slot), (seq / kSlots) & 1, &abort_flag, prm.status, BAR_FULL))) break;
          tc_fence_after();
          const uint64_t dv = dv_slot0 + slot * kSlotStep;
          mma_ts_x4<8, 128>(tO + 64 * h, tP, dv, idesc_o, 0u);
          mma_ts_x4<8, 128>(tO + 64 * h, tP + 32, dv + 512, idesc_o, 1u);
          mma_commit(bar_free(slot));
          ++seq;
        }
        if (ok) mma_commit(bar_pv);      // both halves are complete; P may be overwritten
      }
    }
  } else {
    // ---------------- fold warps: four threads per query row ----------------
    const int qd = warp & 3, cq = warp >> 2;                // TMEM lane quadrant, column quarter
    const int row = qd * 32 + lane;                         // row within the tile == TMEM lane
    const int qi = q0 + row;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float c = prm.scale_log2;
    const bool two_halves = BIAS ? prm.n_halves == 2 : true;   // (warp-uniform: tcgen05.ld is collective; unbiased problems here are wide)
    constexpr bool has_bias = BIAS;
    // with a bias the scores are moved to the log2 domain at once (s c + b log2 e) and the scale below becomes 1
    const float cc = has_bias ? 1.f : c;
    const float* bias_row = has_bias ? prm.bias + bi * prm.bsb + hi * prm.bsh + static_cast<int64_t>(min(qi, prm.n_ctx - 1)) * prm.bsq : nullptr;
    float m_ref = -CUDART_INF_F, m_true = -CUDART_INF_F, zsum = 0.f;   // zsum: this thread's 32 key columns only
    float o_run[32];        // running sums of output columns 16 cq ... (first 16) and 64 + 16 cq ... (last 16), relative to m_ref
#pragma unroll
    for (int i = 0; i < 32; ++i) o_run[i] = 0.f;
    bool alive = true;

    // o_run += O_lo, O_hi (the finished P V of one key tile)
    auto take_o = [&]() {
      uint32_t r0[16], r1[16];
      tmem_ld16(tO + lane_off + 16 * cq, r0);
      if (two_halves) tmem_ld16(tO + 64 + lane_off + 16 * cq, r1);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 16; ++i) o_run[i] += __uint_as_float(r0[i]);
      if (two_halves) {
#pragma unroll
        for (int i = 0; i < 16; ++i) o_run[16 + i] += __uint_as_float(r1[i]);
      }
    };

    for (int j = 0; j < n_t; ++j) {
      if constexpr (BIAS) {
        // this thread's 128 bytes of the bias row for the NEXT key tile: on their way into L2 while this tile is folded
        const int kn = k_begin + (j + 1) * 128 + 32 * cq;
        if (kn + 32 <= k_end) {
          const float* bn = bias_row + static_cast<int64_t>(kn + koff) * prm.bsk;
          prefetch_l2(bn);
          prefetch_l2(bn + 31 * prm.bsk);
        }
      }
      if (!__all_sync(0xffffffffu, mbar_wait(bar_s, j & 1, &abort_flag, prm.status, BAR_S))) { alive = false; break; }
      tc_fence_after();
      float sv[32];
      {
        uint32_t r[32];
        tmem_ld32(tS + lane_off + 32 * cq, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) sv[i] = __uint_as_float(r[i]);
      }
      tc_fence_before();
      mbar_arrive_warp(bar_sfree, lane);        // S may be overwritten with the next tile's scores
      const int k0 = k_begin + j * 128 + 32 * cq;           // first (local) key of this thread's columns
      if constexpr (BIAS) {
        const float* bp = bias_row + static_cast<int64_t>(k0 + koff) * prm.bsk;
        if (prm.bsk == 1 && k0 + 32 <= k_end && (reinterpret_cast<uintptr_t>(bp) & 31u) == 0) {
          // the thread's 128 bytes of the bias row as four whole sectors (a warp's 32 rows are 32 different lines:
          // 4-byte loads would fetch every sector eight times)
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float b8[8];
            ld_global_v8(bp + 8 * g, b8);
#pragma unroll
            for (int e = 0; e < 8; ++e) sv[8 * g + e] = fmaf(sv[8 * g + e], c, b8[e] * 1.4426950408889634f);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float b = (k0 + i < k_end) ? bp[i * prm.bsk] : 0.f;
            sv[i] = fmaf(sv[i], c, b * 1.4426950408889634f);
          }
        }
      }
      const bool tail = k_begin + j * 128 + 128 > k_end;
      const bool diag = prm.is_causal && (k_begin + j * 128 + koff + 127 > q0);
      if (tail || diag) {
        const int lim = prm.is_causal ? min(k_end - 1, qi - koff) : k_end - 1;   // last admissible (local) key of this row
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (k0 + i > lim) sv[i] = -CUDART_INF_F;
      }
      // ---- the row max: this quarter, then the exchange with the three other threads of the row ----
      float mx[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
      for (int i = 4; i < 28; i += 8) {
        mx[0] = max3w(mx[0], sv[i], sv[i + 1]); mx[1] = max3w(mx[1], sv[i + 2], sv[i + 3]);
        mx[2] = max3w(mx[2], sv[i + 4], sv[i + 5]); mx[3] = max3w(mx[3], sv[i + 6], sv[i + 7]);
      }
      mx[0] = max3w(mx[0], sv[28], sv[29]); mx[1] = max3w(mx[1], sv[30], sv[31]);
      row_max[j & 1][cq][row] = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      mbar_arrive_warp(bar_row(qd), lane);
      if (!__all_sync(0xffffffffu, mbar_wait(bar_row(qd), j & 1, &abort_flag, prm.status, BAR_ROW))) { alive = false; break; }
      float tmax = fmaxf(fmaxf(row_max[j & 1][0][row], row_max[j & 1][1][row]), fmaxf(row_max[j & 1][2][row], row_max[j & 1][3][row]));
      tmax *= cc;
      m_true = fmaxf(m_true, tmax);
      // the same decision in all four threads of the row (same tmax, same m_ref)
      const bool move = tmax > m_ref + kRescaleThreshold;   // also true for the first admissible tile (m_ref = -inf)
      float alpha = 1.f;
      if (move) {
        const float m_new = fmaxf(m_ref, tmax);
        alpha = (m_new == -CUDART_INF_F) ? 1.f : exp2f(m_ref - m_new);
        m_ref = m_new;
      }
      const float m_use = (m_ref == -CUDART_INF_F) ? 0.f : m_ref;
      // ---- p = 2^(s*c - m), the quarter-row sum and the 16-bit P (all of it overlaps P V of tile j-1) ----
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float p0 = fast_exp2(fmaf(sv[i], cc, -m_use));
        const float p1 = fast_exp2(fmaf(sv[i + 1], cc, -m_use));
        ps[(i >> 1) & 3] += p0 + p1;
        pk[i >> 1] = pack2<T>(p0, p1);
      }
      zsum = zsum * alpha + ((ps[0] + ps[1]) + (ps[2] + ps[3]));
      if (j > 0) {
        // P V of the previous key tile has retired: its O goes into the running sums (both are relative to the m_ref
        // of that tile) before P V of this tile starts the accumulators from zero again; P is free
        if (!__all_sync(0xffffffffu, mbar_wait(bar_pv, (j - 1) & 1, &abort_flag, prm.status, BAR_PV))) { alive = false; break; }
        tc_fence_after();
        take_o();
      }
      if (move) {
#pragma unroll
        for (int i = 0; i < 32; ++i) o_run[i] *= alpha;
      }
      tmem_st16(tP + lane_off + 16 * cq, pk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(bar_p, lane);
    }

    // epilogue: the last key tile's O, the row sum over the four quarters, renormalisation to the true max, the summary row
    const int r_chunk = bx * 128 + row;   // row within the query chunk
    const bool row_ok = r_chunk < prm.q_len;
    const int64_t ro = (static_cast<int64_t>(part) * prm.bh + bh) * prm.q_len + r_chunk;
    float m_out = -CUDART_INF_F, z_out = 0.f;
    if (n_t > 0) {
      if (alive && !__all_sync(0xffffffffu, mbar_wait(bar_pv, (n_t - 1) & 1, &abort_flag, prm.status, BAR_O))) alive = false;
      if (alive) {
        tc_fence_after();
        take_o();
        row_sum[cq][row] = zsum;
        mbar_arrive_warp(bar_row(qd), lane);
        if (!__all_sync(0xffffffffu, mbar_wait(bar_row(qd), n_t & 1, &abort_flag, prm.status, BAR_ROW))) alive = false;
      }
      if (alive) {
        const float ztot = (row_sum[0][row] + row_sum[1][row]) + (row_sum[2][row] + row_sum[3][row]);
        const float f = (m_true == -CUDART_INF_F) ? 0.f : exp2f(m_ref - m_true);
        z_out = ztot * f;
        m_out = z_out > 0.f ? m_true : -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < 32; ++i) o_run[i] = z_out > 0.f ? o_run[i] * f : 0.f;
      }
    }
    if (row_ok && (alive || n_t == 0)) {
      if (cq == 0) {
        prm.m[ro] = m_out;
        prm.z[ro] = z_out;
      }
      const int d = prm.head_dim;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int col = 64 * h + 16 * cq;
        if (prm.summary_dtype == ELSA_F32) store_row16<float>(static_cast<float*>(prm.s) + ro * d + col, o_run + 16 * h, d - col);
        else if (prm.summary_dtype == ELSA_F16) store_row16<__half>(static_cast<__half*>(prm.s) + ro * d + col, o_run + 16 * h, d - col);
        else store_row16<__nv_bfloat16>(static_cast<__nv_bfloat16*>(prm.s) + ro * d + col, o_run + 16 * h, d - col);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace

bool fold_tcw_supported(int dtype, int head_dim, bool has_bias) {
  // wide heads, and biased problems of any head dim up to 128 (unbiased ones up to 64 have their own kernel)
  return (dtype == ELSA_F16 || dtype == ELSA_BF16) && head_dim >= 8 && head_dim <= 128 && head_dim % 8 == 0 &&
         (head_dim > 64 || has_bias) && fold_tc_supported(dtype, 64, false);
}

int fold_tcw(const FoldParams& p, int dtype, cudaStream_t st) {
  if (!fold_tcw_supported(dtype, p.head_dim, p.bias != nullptr) || p.part_width % 128 != 0) return ELSA_ERR_UNSUPPORTED;
  CUtensorMap mq, mk, mv;
  int rc;
  const int batch = p.bh / p.heads;
  if ((rc = make_tmap_rows64(&mq, p.q, dtype, p.n_ctx, p.heads, batch, p.qs, 128, p.head_dim)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mk, p.k, dtype, p.n_keys, p.heads, batch, p.ks, 128, p.head_dim)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mv, p.v, dtype, p.n_keys, p.heads, batch, p.vs, 128, p.head_dim)) != ELSA_OK) return rc;
  FoldWParams prm;
  prm.m = p.m; prm.z = p.z; prm.s = p.s;
  if ((rc = device_status_word(&prm.status, nullptr)) != ELSA_OK) return rc;
  prm.n_ctx = p.n_ctx; prm.q_start = p.q_start; prm.q_len = p.q_len; prm.part_width = p.part_width;
  prm.n_parts = p.n_parts; prm.bh = p.bh; prm.heads = p.heads; prm.is_causal = p.is_causal; prm.summary_dtype = p.summary_dtype;
  prm.n_keys = p.n_keys; prm.key_offset = p.key_offset; prm.head_dim = p.head_dim;
  prm.scale_log2 = p.scale_log2;
  prm.n_halves = p.head_dim > 64 ? 2 : 1;
  prm.bias = p.bias; prm.bsb = p.bsb; prm.bsh = p.bsh; prm.bsq = p.bsq; prm.bsk = p.bsk;
  dim3 grid(static_cast<unsigned>((p.q_len + 127) / 128), static_cast<unsigned>(p.n_parts), static_cast<unsigned>(p.bh));
  auto launch = [&](auto kernel) -> int {
    const int r = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), kFoldWSmem);
    if (r != ELSA_OK) return r;
    kernel<<<grid, kThreads, kFoldWSmem, st>>>(mq, mk, mv, prm);
    return ELSA_OK;
  };
  if (dtype == ELSA_F16) rc = p.bias ? launch(&fold_tcw_kernel<__half, true>) : launch(&fold_tcw_kernel<__half, false>);
  else rc = p.bias ? launch(&fold_tcw_kernel<__nv_bfloat16, true>) : launch(&fold_tcw_kernel<__nv_bfloat16, false>);
  if (rc != ELSA_OK) return rc;
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

}  // namespace elsa
