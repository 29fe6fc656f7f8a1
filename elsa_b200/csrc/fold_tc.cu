// Phase 1 on the 5th-generation tensor cores (tcgen05 + TMEM + TMA): the per-K-partition
// (m, z, s) fold for fp16 / bf16 inputs with head dim 64 (or a smaller multiple of 8: the tensor maps describe the
// d real columns, the 64-column TMA box reads the rest as zeros, and only d summary columns are stored), causal or not.
//
// One CTA (1 per SM: 160 KB of shared memory, all 512 TMEM columns) owns TWO 128-row query tiles of one
// (batch*head) and one K partition, walked in 128-key tiles:
//
//   warp 8      TMA producer   Q tiles once; K and V tiles into a 4-stage ring (128-byte swizzle)
//   warp 9, 10  MMA issuers    one thread per query tile t:
//                              S_t = Q_t K^T   (4 x tcgen05.mma 128x128x16, both operands in smem)
//                              O_t += P_t V    (8 x tcgen05.mma 128x64x16, P from TMEM, V MN-major)
//   warps 0-3   fold of tile 0 one thread per query row: S row from TMEM into registers, running max, exp2,
//   warps 4-7   fold of tile 1 row sum, P (16-bit) into its own TMEM columns, exp-rescale of O when the max moved
//
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,320) O1 [320,384) P0 [384,448) P1 [448,512).  Because P has
// its own columns, S_t is free as soon as the fold warps hold the row in registers (bar_sfree): the tile's issuer
// produces S_t of the NEXT key tile right then, so the fold warps never wait for scores.  P is handed to the
// issuer once per key tile (bar_p); the fold warps wait for P V of the previous key tile (bar_pv) only before they
// overwrite P or rescale O.  The two tiles share nothing but the K/V ring (a stage is refilled when both issuers
// have released it) and the tensor pipe, so their chains scores -> exponentials -> P V run out of phase: one
// tile's exponentials overlap the other tile's P V and hand-offs instead of both tiles waiting at the same time.
//
// Exp-rescale merge: the fold keeps a reference max m_ref per row and only moves it (rescaling z
// and the O accumulator in TMEM) when the tile max exceeds it by more than 2^8; the true running
// max is tracked separately and the summary is renormalised to it in the epilogue, so the stored
// (m, z, s) is the same monoid element the FP32-FMA kernel produces.
//
// Measured alternatives at B=1 H=8 N=16384 (this design: 0.738 ms; with a P hand-off per 64-key half 0.755 ms and
// the variants below were measured against that): two threads per row (four fold
// warpgroups of 64 columns each, half-row max exchanged through shared memory) 0.77-0.79 ms; a fixed
// issue order that keeps the two tiles half a key tile apart 0.805 ms; half of the exponentials on the FMA
// pipe 0.81 ms; no exponentials at all (timing only) 0.72 ms -- the kernel is bound by the chain
// issuer -> TMEM -> fold warps -> TMEM -> issuer of each key tile, not by the ex2 unit.
#include <type_traits>

#include "kernels.cuh"
#include "tc_common.cuh"

namespace elsa {

using namespace tc;

namespace {

constexpr int kStages = 4;
constexpr int kTileBytes = 128 * 64 * 2;                          // one 128 x 64 16-bit tile
constexpr int kFoldSmem = (2 + 2 * kStages) * kTileBytes + 1024;  // + alignment slack
constexpr int kThreads = 384;   // 3 warpgroups: two fold groups + (producer, MMA issuer, 2 idle warps)
constexpr uint32_t kTmemCols = 512;
constexpr int kProducerWarp = 8, kIssuerWarp = 9;
constexpr float kRescaleThreshold = 8.0f;

enum BarId { BAR_Q = 1, BAR_KV_FULL = 2, BAR_KV_FREE = 3, BAR_S = 4, BAR_P = 5, BAR_O = 6, BAR_SFREE = 7, BAR_PV = 8 };

struct FoldTcParams {
  float* m; float* z; void* s;
  int n_ctx, q_start, q_len, part_width, n_parts, bh, heads, is_causal, summary_dtype;
  int n_keys, key_offset, head_dim;
  float scale_log2;
  int* status;   // the device's status word (mapped host memory)
  // direct != 0 (one partition, the whole query range in one launch): the partition summary is the row's final state,
  // so the kernel writes out = s / z (s rounded to the summary type first, as the merge pass would read it) through
  // `os` and, when row_m is not null, the row state -- no summary travels through memory and no merge pass runs
  int direct;
  void* out; Strides os; float* row_m; float* row_z;
};

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// the first d (a multiple of 8) of the 64 values of a summary row
template <typename TS>
__device__ __forceinline__ void store_row64(TS* dst, const float (&v)[64], int d) {
  if constexpr (sizeof(TS) == 4) {
#pragma unroll
    for (int i = 0; i < 64; i += 4)
      if (i < d) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 64; i += 8) {
      if (i >= d) continue;
      uint4 t;
      t.x = pack2<TS>(v[i], v[i + 1]); t.y = pack2<TS>(v[i + 2], v[i + 3]);
      t.z = pack2<TS>(v[i + 4], v[i + 5]); t.w = pack2<TS>(v[i + 6], v[i + 7]);
      *reinterpret_cast<uint4*>(dst + i) = t;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
fold_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const FoldTcParams prm) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kStages + 11];   // q, kv_full x4, kv_free x4, then 5 pairs
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.z, part = blockIdx.y;
  const int bi = bh / prm.heads, hi = bh - bi * prm.heads;  // tensor-map coordinates of this (batch*head)
  // causal: a tile's work grows with its first row, so the tiles are handed out from the last one down -- the long
  // ones first, the short ones fill the end of the last wave
  const int bx = prm.is_causal ? static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
  const int q0 = prm.q_start + bx * 256;           // first query row of tile 0
  const int q_end = prm.q_start + prm.q_len;
  const int k_begin = part * prm.part_width;
  const int k_end = min(prm.n_keys, k_begin + prm.part_width);   // local key indices
  const int koff = prm.key_offset;

  // number of 128-key tiles each query tile has to visit
  int n_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qt0 = q0 + t * 128;
    int ke = k_end;
    if (prm.is_causal) ke = min(ke, min(qt0 + 128, q_end) - koff);  // keys above the tile's last row are never admissible
    n_t[t] = (qt0 < q_end && ke > k_begin) ? (ke - k_begin + 127) / 128 : 0;
  }
  const int n_max = max(n_t[0], n_t[1]);

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ[2] = {smem_base, smem_base + kTileBytes};
  auto sK = [&](int st) { return smem_base + (2 + 2 * st) * kTileBytes; };
  auto sV = [&](int st) { return smem_base + (3 + 2 * st) * kTileBytes; };
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_q = bar0;
  auto bar_kv_full = [&](int st) { return bar0 + 8 * (1 + st); };
  auto bar_kv_free = [&](int st) { return bar0 + 8 * (1 + kStages + st); };
  auto bar_s = [&](int t) { return bar0 + 8 * (1 + 2 * kStages + t); };          // S_t(j) is in TMEM
  auto bar_p = [&](int t) { return bar0 + 8 * (3 + 2 * kStages + t); };          // P_t(j) has been delivered by the fold warps
  auto bar_o = [&](int t) { return bar0 + 8 * (5 + 2 * kStages + t); };          // every MMA of tile t has retired
  auto bar_sfree = [&](int t) { return bar0 + 8 * (7 + 2 * kStages + t); };      // the fold warps hold S_t in registers
  auto bar_pv = [&](int t) { return bar0 + 8 * (9 + 2 * kStages + t); };         // P_t V of the current key tile has retired

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_q, 1);
    // a K/V stage is free again when BOTH tiles' issuers have released it (a commit after the tile's P V, or a plain
    // arrival for a key tile that the tile does not visit)
    for (int st = 0; st < kStages; ++st) { mbar_init(bar_kv_full(st), 1); mbar_init(bar_kv_free(st), 2); }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_s(t), 1); mbar_init(bar_p(t), 128); mbar_init(bar_o(t), 1);
      mbar_init(bar_sfree(t), 128); mbar_init(bar_pv(t), 1);
    }
    fence_mbar_init();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 128};
  const uint32_t tO[2] = {tmem_base + 256, tmem_base + 320};
  const uint32_t tP[2] = {tmem_base + 384, tmem_base + 448};

  // register budget: the fold warps hold a whole 128-column score row per thread; the producer / issuer
  // warpgroup needs almost nothing (3 x 128 threads: 232 + 232 + 40 = 3 x 168, the launch allocation; setmaxnreg.inc waits, unbounded, until the pool has the registers, so the three budgets must never add up to more).  Each role
  // branch starts with its setmaxnreg and runs to the common exit, so the allocator sees one budget per branch.

  if (warp >= 8) {
    reg_dec<40>();
    if (n_max > 0 && warp == kProducerWarp) {
      // ---------------- TMA producer ----------------
      if (lane == 0) {
        prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
        mbar_arrive_expect_tx(bar_q, 2 * kTileBytes);
        tma_load_4d(sQ[0], &tmap_q, bar_q, 0, q0, hi, bi);
        tma_load_4d(sQ[1], &tmap_q, bar_q, 0, q0 + 128, hi, bi);
        for (int j = 0; j < n_max; ++j) {
          const int st = j % kStages;
          if (j >= kStages && !mbar_wait(bar_kv_free(st), ((j / kStages) - 1) & 1, &abort_flag, prm.status, BAR_KV_FREE)) break;
          mbar_arrive_expect_tx(bar_kv_full(st), 2 * kTileBytes);
          tma_load_4d(sK(st), &tmap_k, bar_kv_full(st), 0, k_begin + j * 128, hi, bi);
          tma_load_4d(sV(st), &tmap_v, bar_kv_full(st), 0, k_begin + j * 128, hi, bi);
        }
      }
    } else if (n_max > 0 && (warp == kIssuerWarp || warp == kIssuerWarp + 1)) {
      // ---------------- MMA issuers: one thread per query tile ----------------
      // Each tile has its own issuing thread, so the two tiles run their chains (scores -> exponentials -> P V)
      // independently and drift half a period apart by themselves: while one tile's P V and hand-offs are in
      // flight, the other tile's fold warps have the ex2 unit to themselves.  The only thing the tiles share is
      // the K/V ring (and the tensor pipe, which executes the MMAs of both threads in the order it receives them).
      const int t = warp - kIssuerWarp;
      if (lane == 0) {
        constexpr uint32_t fmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
        constexpr uint32_t idesc_s = make_idesc(fmt, 0, 0, 128, 128);   // S = Q K^T : A, B K-major
        constexpr uint32_t idesc_o = make_idesc(fmt, 0, 1, 128, 64);    // O += P V  : A in TMEM, B (V) MN-major
        // shared-memory descriptors are loop invariants: every instruction between two tcgen05.mma idles the pipe
        const uint64_t dq = make_sdesc(sQ[t], 16, 1024);
        const uint64_t dk0 = make_sdesc(sK(0), 16, 1024), dv0 = make_sdesc(sV(0), 128 * 128, 1024);
        constexpr uint64_t kStageStep = (2 * kTileBytes) >> 4;   // descriptor address field counts 16-byte units
        const int nt = n_t[t];
        bool ok = true;
        if (nt > 0) {
          ok = mbar_wait(bar_q, 0, &abort_flag, prm.status, BAR_Q) && mbar_wait(bar_kv_full(0), 0, &abort_flag, prm.status, BAR_KV_FULL);
          if (ok) {
            tc_fence_after();
            mma_ss_x4<2, 2>(tS[t], dq, dk0, idesc_s, 0u);
            mma_commit(bar_s(t));
          }
        }
        for (int j = 0; ok && j < nt; ++j) {
          const int u = j % kStages, un = (j + 1) % kStages;
          // S(j+1) as soon as the fold warps have pulled S(j) into registers: the next scores are computed while
          // the current exponentials run, so the fold warps never wait for the tensor pipe
          if (j + 1 < nt) {
            ok = mbar_wait(bar_kv_full(un), ((j + 1) / kStages) & 1, &abort_flag, prm.status, BAR_KV_FULL) &&
                 mbar_wait(bar_sfree(t), j & 1, &abort_flag, prm.status, BAR_SFREE);
            if (!ok) break;
            tc_fence_after();
            mma_ss_x4<2, 2>(tS[t], dq, dk0 + un * kStageStep, idesc_s, 0u);
            mma_commit(bar_s(t));
          }
          // O += P V once the fold warps have delivered P(j)
          if (!(ok = mbar_wait(bar_p(t), j & 1, &abort_flag, prm.status, BAR_P))) break;
          tc_fence_after();
          mma_ts_x4<8, 128>(tO[t], tP[t], dv0 + u * kStageStep, idesc_o, j > 0 ? 1u : 0u);
          mma_ts_x4<8, 128>(tO[t], tP[t] + 32, dv0 + u * kStageStep + 512, idesc_o, 1u);
          mma_commit(bar_pv(t));        // P_t may be overwritten, O_t may be rescaled
          mma_commit(bar_kv_free(u));   // this tile no longer reads K(j), V(j)
        }
        if (ok && nt > 0) mma_commit(bar_o(t));
        // key tiles this query tile does not visit (causal: the other tile reaches one tile further; a tile beyond
        // the last query row visits none): release their stages in order, each after the stage's previous use is over
        for (int j = nt; ok && j < n_max; ++j) {
          const int u = j % kStages;
          if (j >= kStages && !(ok = mbar_wait(bar_kv_free(u), ((j / kStages) - 1) & 1, &abort_flag, prm.status, BAR_KV_FREE))) break;
          mbar_arrive(bar_kv_free(u));
        }
      }
    }
  } else {
    reg_inc<232>();
    // ---------------- fold warps: one thread per query row ----------------
    const int t = warp >> 2;
    const int row = (warp & 3) * 32 + lane;                 // row within the tile == TMEM lane
    const int qi = q0 + t * 128 + row;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float c = prm.scale_log2;
    float m_ref = -CUDART_INF_F, m_true = -CUDART_INF_F, zsum = 0.f;
    bool alive = true;

    for (int j = 0; j < n_t[t]; ++j) {
      if (!__all_sync(0xffffffffu, mbar_wait(bar_s(t), j & 1, &abort_flag, prm.status, BAR_S))) { alive = false; break; }
      tc_fence_after();
      float sv[128];
#pragma unroll
      for (int cchunk = 0; cchunk < 4; ++cchunk) {
        uint32_t r[32];
        tmem_ld32(tS[t] + lane_off + 32 * cchunk, r);
#pragma unroll
        for (int i = 0; i < 32; ++i) sv[32 * cchunk + i] = __uint_as_float(r[i]);
      }
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bar_sfree(t));      // S_t may be overwritten with the next tile's scores
      const int k0 = k_begin + j * 128;
      const bool tail = k0 + 128 > k_end;
      const bool diag = prm.is_causal && (k0 + koff + 127 > q0 + t * 128);
      if (tail || diag) {
        const int lim = prm.is_causal ? min(k_end - 1, qi - koff) : k_end - 1;   // last admissible (local) key of this row
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (k0 + i > lim) sv[i] = -CUDART_INF_F;
      }
      // row max with four independent chains (a single 128-deep fmax chain costs ~500 cycles of latency)
      // (three-input max: 64 instructions instead of 128)
      float mx[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
      for (int i = 4; i < 124; i += 8) {
        mx[0] = max3(mx[0], sv[i], sv[i + 1]); mx[1] = max3(mx[1], sv[i + 2], sv[i + 3]);
        mx[2] = max3(mx[2], sv[i + 4], sv[i + 5]); mx[3] = max3(mx[3], sv[i + 6], sv[i + 7]);
      }
      mx[0] = max3(mx[0], sv[124], sv[125]);
      mx[1] = max3(mx[1], sv[126], sv[127]);
      float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      tmax *= c;
      m_true = fmaxf(m_true, tmax);
      if (j > 0) {
        // P_t V of the previous key tile must have retired before P_t is overwritten or O_t rescaled
        if (!__all_sync(0xffffffffu, mbar_wait(bar_pv(t), (j - 1) & 1, &abort_flag, prm.status, BAR_PV))) { alive = false; break; }
        tc_fence_after();
      }
      const bool move = tmax > m_ref + kRescaleThreshold;   // also true for the first admissible tile (m_ref = -inf)
      if (__any_sync(0xffffffffu, move)) {
        const float m_new = fmaxf(m_ref, tmax);
        const float alpha = (m_new == -CUDART_INF_F) ? 1.f : fast_exp2(m_ref - m_new);
        zsum *= alpha;
        if (j > 0) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld32(tO[t] + lane_off + 32 * h, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(tO[t] + lane_off + 32 * h, r);
          }
        }
        m_ref = m_new;
      }
      const float m_use = (m_ref == -CUDART_INF_F) ? 0.f : m_ref;
      // p = 2^(s*c - m) on packed pairs (fma.f32x2 / add.f32x2), row sum in four independent pair accumulators
      const float2 c2 = make_float2(c, c), nm2 = make_float2(-m_use, -m_use);
      float2 ps[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float2 x = __ffma2_rn(make_float2(sv[64 * h + 2 * i], sv[64 * h + 2 * i + 1]), c2, nm2);
          const float2 pp = make_float2(fast_exp2(x.x), fast_exp2(x.y));
          ps[i & 3] = __fadd2_rn(ps[i & 3], pp);
          pk[i] = pack2<T>(pp.x, pp.y);
        }
        tmem_st32(tP[t] + lane_off + 32 * h, pk);
      }
      // one hand-off per key tile: with the scores produced a tile ahead, P V need not start on the first half
      tmem_wait_st();               // (also covers the O rescale stores above)
      tc_fence_before();
      mbar_arrive(bar_p(t));
      {
        const float2 s01 = __fadd2_rn(ps[0], ps[1]), s23 = __fadd2_rn(ps[2], ps[3]);
        const float2 s = __fadd2_rn(s01, s23);
        zsum += s.x + s.y;
      }
    }

    // epilogue: renormalise to the true max and write the summary row
    const int r_chunk = bx * 256 + t * 128 + row;   // row within the query chunk
    const bool row_ok = r_chunk < prm.q_len;
    if (n_t[t] > 0) {
      if (alive && !__all_sync(0xffffffffu, mbar_wait(bar_o(t), 0, &abort_flag, prm.status, BAR_O))) alive = false;
      if (alive) {
        tc_fence_after();
        float ov[64];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld32(tO[t] + lane_off + 32 * h, r);
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[32 * h + i] = __uint_as_float(r[i]);
        }
        tmem_wait_ld();
        const float f = (m_true == -CUDART_INF_F) ? 0.f : fast_exp2(m_ref - m_true);
        const float zo = zsum * f;
        if (row_ok && prm.direct) {
          const int r_seq = prm.q_start + r_chunk;
          const float inv = zo > 0.f ? 1.0f / zo : 0.f;
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            float x = zo > 0.f ? ov[i] * f : 0.f;
            if (prm.summary_dtype == ELSA_F16) x = round_to<__half>(x);
            else if (prm.summary_dtype == ELSA_BF16) x = round_to<__nv_bfloat16>(x);
            ov[i] = zo > 0.f ? x * inv : 0.f;
          }
          T* dst = static_cast<T*>(prm.out) + static_cast<int64_t>(bh / prm.heads) * prm.os.b + static_cast<int64_t>(bh % prm.heads) * prm.os.h +
                   static_cast<int64_t>(r_seq) * prm.os.r;
          store_row64<T>(dst, ov, prm.head_dim);
          if (prm.row_m) {
            const int64_t ro = static_cast<int64_t>(bh) * prm.n_ctx + r_seq;
            prm.row_m[ro] = zo > 0.f ? m_true : -CUDART_INF_F;
            prm.row_z[ro] = zo;
          }
        } else if (row_ok) {
          const int64_t ro = (static_cast<int64_t>(part) * prm.bh + bh) * prm.q_len + r_chunk;
          prm.m[ro] = zo > 0.f ? m_true : -CUDART_INF_F;
          prm.z[ro] = zo;
#pragma unroll
          for (int i = 0; i < 64; ++i) ov[i] = zo > 0.f ? ov[i] * f : 0.f;
          if (prm.summary_dtype == ELSA_F32) store_row64<float>(static_cast<float*>(prm.s) + ro * prm.head_dim, ov, prm.head_dim);
          else if (prm.summary_dtype == ELSA_F16) store_row64<__half>(static_cast<__half*>(prm.s) + ro * prm.head_dim, ov, prm.head_dim);
          else store_row64<__nv_bfloat16>(static_cast<__nv_bfloat16*>(prm.s) + ro * prm.head_dim, ov, prm.head_dim);
        }
      }
    } else if (row_ok && prm.direct) {
      // nothing admissible for this tile at all: zeros and the empty state
      const int r_seq = prm.q_start + r_chunk;
      float ov[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) ov[i] = 0.f;
      T* dst = static_cast<T*>(prm.out) + static_cast<int64_t>(bh / prm.heads) * prm.os.b + static_cast<int64_t>(bh % prm.heads) * prm.os.h +
               static_cast<int64_t>(r_seq) * prm.os.r;
      store_row64<T>(dst, ov, prm.head_dim);
      if (prm.row_m) {
        const int64_t ro = static_cast<int64_t>(bh) * prm.n_ctx + r_seq;
        prm.row_m[ro] = -CUDART_INF_F;
        prm.row_z[ro] = 0.f;
      }
    } else if (row_ok) {
      // nothing admissible in this partition for this tile: the identity
      const int64_t ro = (static_cast<int64_t>(part) * prm.bh + bh) * prm.q_len + r_chunk;
      prm.m[ro] = -CUDART_INF_F;
      prm.z[ro] = 0.f;
      float ov[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) ov[i] = 0.f;
      if (prm.summary_dtype == ELSA_F32) store_row64<float>(static_cast<float*>(prm.s) + ro * prm.head_dim, ov, prm.head_dim);
      else if (prm.summary_dtype == ELSA_F16) store_row64<__half>(static_cast<__half*>(prm.s) + ro * prm.head_dim, ov, prm.head_dim);
      else store_row64<__nv_bfloat16>(static_cast<__nv_bfloat16*>(prm.s) + ro * prm.head_dim, ov, prm.head_dim);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem_base, kTmemCols);
}

// test hook: a bounded wait that runs out (nothing arrives at the barrier), in the form the product kernels use
__global__ void wait_timeout_kernel(int* status, unsigned long long limit_ns) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
    (void)mbar_wait(smem_u32(&bar), 0, &abort_flag, status, 99, limit_ns);
  }
}

}  // namespace

int debug_wait_timeout(unsigned long long limit_ns, cudaStream_t st) {
  int* status = nullptr;
  int rc = device_status_word(&status, nullptr);
  if (rc != ELSA_OK) return rc;
  wait_timeout_kernel<<<1, 32, 0, st>>>(status, limit_ns);
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

// ---- host ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// The driver's encode call wants a context current on the calling thread.  A thread that has made no runtime call yet
// (an autograd worker whose first CUDA work is this library's) has none: a null cudaFree binds the primary context of
// the thread's current device, after which the encode is repeated.
static bool bind_primary_context() { return cudaFree(nullptr) == cudaSuccess; }

int make_tmap_rows64(CUtensorMap* map, const void* base, int dtype, int64_t n_rows, int heads, int batch, Strides st,
                     int box_rows, int cols, int box_batch) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return ELSA_ERR_UNSUPPORTED;
  if ((st.b | st.h | st.r) % 8 != 0 || cols < 8 || cols > 128 || cols % 8 != 0 || st.r < cols || (reinterpret_cast<uintptr_t>(base) & 15u)) return ELSA_ERR_INVALID_ARGUMENT;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(n_rows), static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
  // a size-1 axis may come with any stride (PyTorch reports arbitrary ones): give it a valid dummy
  const cuuint64_t sh = heads > 1 ? static_cast<cuuint64_t>(st.h) * 2 : 128, sb = batch > 1 ? static_cast<cuuint64_t>(st.b) * 2 : 128;
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(st.r) * 2, sh, sb};
  const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, static_cast<cuuint32_t>(box_batch)};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == ELSA_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = fn(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_ERROR_INVALID_CONTEXT || !bind_primary_context()) break;
  }
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return ELSA_ERR_CUDA;
  }
  return ELSA_OK;
}

int make_tmap_f32_rows64(CUtensorMap* map, const void* base, int64_t n_rows, int64_t n_mats, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return ELSA_ERR_UNSUPPORTED;
  const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(n_rows), static_cast<cuuint64_t>(n_mats)};
  const cuuint64_t strides[2] = {256, static_cast<cuuint64_t>(n_rows) * 256};
  const cuuint32_t box[3] = {32, static_cast<cuuint32_t>(box_rows), 1};   // 32 floats = one 128-byte swizzle row
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_ERROR_INVALID_CONTEXT || !bind_primary_context()) break;
  }
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return ELSA_ERR_CUDA;
  }
  return ELSA_OK;
}

bool fold_tc_supported(int dtype, int head_dim, bool has_bias) {
  return (dtype == ELSA_F16 || dtype == ELSA_BF16) && head_dim >= 8 && head_dim <= 64 && head_dim % 8 == 0 && !has_bias &&
         encode_tiled_fn() != nullptr;
}

int fold_tc(const FoldParams& p, int dtype, cudaStream_t st) {
  if (!fold_tc_supported(dtype, p.head_dim, p.bias != nullptr) || p.part_width % 128 != 0) return ELSA_ERR_UNSUPPORTED;
  CUtensorMap mq, mk, mv;
  int rc;
  const int batch = p.bh / p.heads;
  if ((rc = make_tmap_rows64(&mq, p.q, dtype, p.n_ctx, p.heads, batch, p.qs, 128, p.head_dim)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mk, p.k, dtype, p.n_keys, p.heads, batch, p.ks, 128, p.head_dim)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mv, p.v, dtype, p.n_keys, p.heads, batch, p.vs, 128, p.head_dim)) != ELSA_OK) return rc;
  FoldTcParams prm;
  prm.n_keys = p.n_keys; prm.key_offset = p.key_offset; prm.head_dim = p.head_dim;
  prm.m = p.m; prm.z = p.z; prm.s = p.s;
  prm.direct = p.direct; prm.out = p.out; prm.os = p.os; prm.row_m = p.row_m; prm.row_z = p.row_z;
  if (p.direct && (p.n_parts != 1 || !p.out)) return ELSA_ERR_INVALID_ARGUMENT;
  if ((rc = device_status_word(&prm.status, nullptr)) != ELSA_OK) return rc;
  prm.n_ctx = p.n_ctx; prm.q_start = p.q_start; prm.q_len = p.q_len; prm.part_width = p.part_width;
  prm.n_parts = p.n_parts; prm.bh = p.bh; prm.heads = p.heads; prm.is_causal = p.is_causal; prm.summary_dtype = p.summary_dtype;
  prm.scale_log2 = p.scale_log2;
  dim3 grid(static_cast<unsigned>((p.q_len + 255) / 256), static_cast<unsigned>(p.n_parts), static_cast<unsigned>(p.bh));
  if (dtype == ELSA_F16) {
    rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&fold_tc_kernel<__half>), kFoldSmem);
    if (rc != ELSA_OK) return rc;
    fold_tc_kernel<__half><<<grid, kThreads, kFoldSmem, st>>>(mq, mk, mv, prm);
  } else {
    rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&fold_tc_kernel<__nv_bfloat16>), kFoldSmem);
    if (rc != ELSA_OK) return rc;
    fold_tc_kernel<__nv_bfloat16><<<grid, kThreads, kFoldSmem, st>>>(mq, mk, mv, prm);
  }
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}


}  // namespace elsa
