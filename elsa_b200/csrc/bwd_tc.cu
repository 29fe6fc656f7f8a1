// Backward on the 5th-generation tensor cores: exact recompute from the saved row statistics,
// fp16 / bf16 inputs, head dim 64, causal or not, no bias.  Five contractions per (key tile, query
// tile) pair -- the algorithmic minimum -- all as tcgen05.mma with TMEM accumulators:
//
//   S^T  = K Q^T          [128 keys x 128 queries]   smem x smem          -> TMEM tS
//   dP^T = V dO^T         [128 x 128]                smem x smem          -> TMEM tdP
//   dV  += P^T dO         [128 keys x 64]            TMEM (P^T over tS)  x smem (dO, MN-major)
//   dK  += dS^T Q         [128 keys x 64]            TMEM (dS^T over tdP) x smem (Q, MN-major)
//   dQ   = dS K           [128 queries x 64]         smem (dS^T, MN-major A) x smem (K, MN-major)
//
// One CTA (1 per SM) owns one 128-key tile of one (batch*head) and streams the query tiles.  Working
// on the transposed score tile puts one KEY per TMEM lane, so P^T and dS^T come out in exactly the
// layout the dV / dK contractions take as their TMEM A operand; dS^T is also written to shared
// memory (16-bit, 128-byte swizzle) where the dQ contraction reads it as an M-major A operand.
// dK and dV stay in TMEM for the whole CTA.  dQ of each pair is added into an fp32 accumulator in
// global memory with vector reductions (red.global.add.v4.f32); a last pass scales and rounds it.
//
//   warp 8      TMA producer   K, V once; Q_i, dO_i, LSE_i, D_i into a 2-stage ring
//   warp 9      MMA issuer
//   warps 0-7   256 threads: thread = (key row, half of the 128 query columns): exp2, dS, packing,
//               then (query row, half of the 64 dQ columns) for the reductions
//
// LSE and D are read from a padded [BH][ceil(N/128)*128] layout whose padding holds LSE = +inf,
// D = 0, so that query rows beyond N produce P = 0 without a branch.
#include <type_traits>

#include "kernels.cuh"
#include "tc_common.cuh"

namespace elsa {

using namespace tc;

static __device__ int g_bwd_status = 0;

namespace {

constexpr int kQStages = 2;
constexpr int kTile = 128 * 64 * 2;     // 16 KB: one 128 x 64 16-bit tile
constexpr int kVecBytes = 128 * 4;      // 128 fp32 row statistics
// smem: K, V | ring of (Q, dO, LSE, D) | dS^T (two 64-query blocks)
constexpr int kStageBytes = 2 * kTile + 2 * kVecBytes;
constexpr int kBwdSmem = 2 * kTile + kQStages * kStageBytes + 2 * kTile + 1024;
constexpr int kThreads = 320;
constexpr uint32_t kTmemCols = 512;

enum BarId { BAR_KV = 11, BAR_Q_FULL = 12, BAR_Q_FREE = 13, BAR_SP = 14, BAR_PDS = 15, BAR_DQ_FULL = 16, BAR_DQ_FREE = 17, BAR_DONE = 18 };

struct BwdTcParams {
  const float* lse_pad; const float* d_pad;   // [BH][n_pad]
  float* dq_acc;                              // [BH][N][64] fp32, zeroed by the caller
  void* dk; void* dv;                         // [BH][N][64] T
  int n_ctx, n_pad, bh, is_causal;
  float scale, scale_log2;
};

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
bwd_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
              const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
              const BwdTcParams prm) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kQStages + 6];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.y;
  const int k0 = blockIdx.x * 128;                  // first key row of this CTA
  const int N = prm.n_ctx;
  const int n_qtiles = (N + 127) / 128;
  const int it_begin = prm.is_causal ? blockIdx.x : 0;   // query tiles below the diagonal tile see none of these keys
  const int n_it = n_qtiles - it_begin;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = smem_base, sV = smem_base + kTile;
  auto sQ = [&](int st) { return smem_base + 2 * kTile + st * kStageBytes; };
  auto sDO = [&](int st) { return sQ(st) + kTile; };
  auto sLSE = [&](int st) { return sQ(st) + 2 * kTile; };
  auto sD = [&](int st) { return sQ(st) + 2 * kTile + kVecBytes; };
  const uint32_t sDS = smem_base + 2 * kTile + kQStages * kStageBytes;   // 2 x 16 KB
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));        // generic pointer to smem_base

  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_kv = bar0;
  auto bar_q_full = [&](int st) { return bar0 + 8 * (1 + st); };
  auto bar_q_free = [&](int st) { return bar0 + 8 * (1 + kQStages + st); };
  const uint32_t bar_sp = bar0 + 8 * (1 + 2 * kQStages);
  const uint32_t bar_pds = bar_sp + 8, bar_dq_full = bar_sp + 16, bar_dq_free = bar_sp + 24, bar_done = bar_sp + 32;

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_kv, 1);
    for (int st = 0; st < kQStages; ++st) { mbar_init(bar_q_full(st), 1); mbar_init(bar_q_free(st), 1); }
    mbar_init(bar_sp, 1);
    mbar_init(bar_pds, 256);
    mbar_init(bar_dq_full, 1);
    mbar_init(bar_dq_free, 256);
    mbar_init(bar_done, 1);
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
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 320, tdQ = tmem_base + 384;

  if (warp == 8) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_do);
      mbar_arrive_expect_tx(bar_kv, 2 * kTile);
      tma_load_3d(sK, &tmap_k, bar_kv, 0, k0, bh);
      tma_load_3d(sV, &tmap_v, bar_kv, 0, k0, bh);
      for (int it = 0; it < n_it; ++it) {
        const int st = it % kQStages;
        if (it >= kQStages && !mbar_wait(bar_q_free(st), ((it / kQStages) - 1) & 1, &abort_flag, &g_bwd_status, BAR_Q_FREE)) break;
        const int qrow = (it_begin + it) * 128;
        mbar_arrive_expect_tx(bar_q_full(st), kStageBytes);
        tma_load_3d(sQ(st), &tmap_q, bar_q_full(st), 0, qrow, bh);
        tma_load_3d(sDO(st), &tmap_do, bar_q_full(st), 0, qrow, bh);
        bulk_load_1d(sLSE(st), prm.lse_pad + static_cast<int64_t>(bh) * prm.n_pad + qrow, kVecBytes, bar_q_full(st));
        bulk_load_1d(sD(st), prm.d_pad + static_cast<int64_t>(bh) * prm.n_pad + qrow, kVecBytes, bar_q_full(st));
      }
    }
  } else if (warp == 9) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc_st = make_idesc(fmt, 0, 0, 128, 128);  // S^T, dP^T: A, B K-major
      constexpr uint32_t idesc_kv = make_idesc(fmt, 0, 1, 128, 64);   // dV, dK: A in TMEM, B MN-major
      constexpr uint32_t idesc_dq = make_idesc(fmt, 1, 1, 128, 64);   // dQ: A (dS^T) M-major, B (K) MN-major
      bool ok = mbar_wait(bar_kv, 0, &abort_flag, &g_bwd_status, BAR_KV);
      for (int it = 0; ok && it < n_it; ++it) {
        const int st = it % kQStages;
        ok = mbar_wait(bar_q_full(st), (it / kQStages) & 1, &abort_flag, &g_bwd_status, BAR_Q_FULL);
        if (!ok) break;
        tc_fence_after();
        {
          const uint64_t ak = make_sdesc(sK, 16, 1024), av = make_sdesc(sV, 16, 1024);
          const uint64_t bq = make_sdesc(sQ(st), 16, 1024), bdo = make_sdesc(sDO(st), 16, 1024);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) mma_ss(tS, ak + 2 * kk, bq + 2 * kk, idesc_st, kk > 0);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) mma_ss(tdP, av + 2 * kk, bdo + 2 * kk, idesc_st, kk > 0);
          mma_commit(bar_sp);
        }
        ok = mbar_wait(bar_pds, it & 1, &abort_flag, &g_bwd_status, BAR_PDS);
        if (ok && it > 0) ok = mbar_wait(bar_dq_free, (it - 1) & 1, &abort_flag, &g_bwd_status, BAR_DQ_FREE);
        if (!ok) break;
        tc_fence_after();
        {
          const uint64_t bdo = make_sdesc(sDO(st), 128 * 128, 1024), bq = make_sdesc(sQ(st), 128 * 128, 1024);
          const uint64_t ads = make_sdesc(sDS, 128 * 128, 1024), bk = make_sdesc(sK, 128 * 128, 1024);
#pragma unroll
          // 16 queries per step; queries 0-63 sit in columns [0,32), queries 64-127 in columns [64,96)
          for (int kk = 0; kk < 8; ++kk)
            mma_ts(tdV, tS + (kk < 4 ? 8 * kk : 32 + 8 * kk), bdo + 128 * kk, idesc_kv, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ts(tdK, tdP + (kk < 4 ? 8 * kk : 32 + 8 * kk), bq + 128 * kk, idesc_kv, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) mma_ss(tdQ, ads + 128 * kk, bk + 128 * kk, idesc_dq, kk > 0);
          mma_commit(bar_dq_full);
          mma_commit(bar_q_free(st));
        }
      }
      if (ok) mma_commit(bar_done);
    }
  } else {
    // ---------------- compute warps ----------------
    const int half = warp >> 2;                               // which 64 query columns / 32 dQ columns
    const int row = (warp & 3) * 32 + lane;                   // key row in phase A, query row in phase B
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int key = k0 + row;
    const bool key_ok = key < N;
    const float c = prm.scale_log2;
    bool alive = true;

    for (int it = 0; it < n_it; ++it) {
      const int st = it % kQStages;
      const int q_tile0 = (it_begin + it) * 128;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_sp, it & 1, &abort_flag, &g_bwd_status, BAR_SP))) { alive = false; break; }
      tc_fence_after();
      const float* lse_s = reinterpret_cast<const float*>(smem_gen + (sLSE(st) - smem_base));
      const float* d_s = reinterpret_cast<const float*>(smem_gen + (sD(st) - smem_base));
      const bool diag = prm.is_causal && (q_tile0 < k0 + 128);   // only the first visited tile crosses the diagonal
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        const int col0 = half * 64 + ch * 32;                 // first query column of this chunk
        uint32_t rs[32], rp[32];
        tmem_ld32(tS + lane_off + col0, rs);
        tmem_ld32(tdP + lane_off + col0, rp);
        tmem_wait_ld();
        uint32_t pk[16], dk_[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float pv[2], dv_[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = col0 + 2 * i + e;
            const float l = lse_s[col], dd = d_s[col];
            float p = fast_exp2(fmaf(__uint_as_float(rs[2 * i + e]), c, -l));
            bool valid = key_ok;
            if (diag) valid = valid && (q_tile0 + col >= key);
            p = valid ? p : 0.f;
            pv[e] = p;
            dv_[e] = p * (__uint_as_float(rp[2 * i + e]) - dd);
          }
          pk[i] = pack2<T>(pv[0], pv[1]);
          dk_[i] = pack2<T>(dv_[0], dv_[1]);
        }
        // P^T over S^T, dS^T over dP^T (16-bit pairs: 16 columns hold 32 query columns).  Each thread
        // overwrites only fp32 columns it has already consumed: the packed values of query half h go to
        // columns [64h + 16*ch, +16), inside this thread's own 64-column region.
        {
          uint32_t w[32];
#pragma unroll
          for (int i = 0; i < 16; ++i) { w[i] = pk[i]; w[16 + i] = dk_[i]; }
          const uint32_t pcol = static_cast<uint32_t>(half * 64 + ch * 16);
          asm volatile(
              "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
              ::"r"(tS + lane_off + pcol), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]),
                "r"(w[7]), "r"(w[8]), "r"(w[9]), "r"(w[10]), "r"(w[11]), "r"(w[12]), "r"(w[13]), "r"(w[14]), "r"(w[15]) : "memory");
          asm volatile(
              "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
              ::"r"(tdP + lane_off + pcol), "r"(w[16]), "r"(w[17]), "r"(w[18]), "r"(w[19]), "r"(w[20]), "r"(w[21]),
                "r"(w[22]), "r"(w[23]), "r"(w[24]), "r"(w[25]), "r"(w[26]), "r"(w[27]), "r"(w[28]), "r"(w[29]), "r"(w[30]),
                "r"(w[31]) : "memory");
        }
        // dS^T to shared memory: block `half` (64 queries), row = key, 16-byte chunk index XOR (key & 7)
        {
          uint8_t* blk = smem_gen + (sDS - smem_base) + half * kTile + row * 128;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int chunk = ch * 4 + g;                      // 8 queries per 16-byte chunk
            uint4 val = make_uint4(dk_[4 * g], dk_[4 * g + 1], dk_[4 * g + 2], dk_[4 * g + 3]);
            *reinterpret_cast<uint4*>(blk + ((chunk ^ (row & 7)) << 4)) = val;
          }
        }
      }
      fence_proxy_async_smem();
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_pds);

      // ---- dQ of this pair: TMEM -> registers -> global fp32 reductions ----
      if (!__all_sync(0xffffffffu, mbar_wait(bar_dq_full, it & 1, &abort_flag, &g_bwd_status, BAR_DQ_FULL))) { alive = false; break; }
      tc_fence_after();
      uint32_t rq[32];
      tmem_ld32(tdQ + lane_off + half * 32, rq);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bar_dq_free);
      const int qrow = q_tile0 + row;
      if (qrow < N) {
        float* dst = prm.dq_acc + (static_cast<int64_t>(bh) * N + qrow) * 64 + half * 32;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          red_add_v4(dst + 4 * i, __uint_as_float(rq[4 * i]), __uint_as_float(rq[4 * i + 1]), __uint_as_float(rq[4 * i + 2]),
                     __uint_as_float(rq[4 * i + 3]));
      }
    }

    // ---- epilogue: dK, dV of this key tile ----
    if (alive && n_it > 0 && !__all_sync(0xffffffffu, mbar_wait(bar_done, 0, &abort_flag, &g_bwd_status, BAR_DONE))) alive = false;
    // tcgen05.ld is warp-collective (.sync.aligned): every lane executes it, only the stores are predicated
    if (alive) {
      uint32_t rk[32], rv[32];
      if (n_it > 0) {
        tc_fence_after();
        tmem_ld32(tdK + lane_off + half * 32, rk);
        tmem_ld32(tdV + lane_off + half * 32, rv);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) { rk[i] = 0u; rv[i] = 0u; }   // no query sees these keys: zero gradients
      }
      if (key_ok) {
        T* dk_row = static_cast<T*>(prm.dk) + (static_cast<int64_t>(bh) * N + key) * 64 + half * 32;
        T* dv_row = static_cast<T*>(prm.dv) + (static_cast<int64_t>(bh) * N + key) * 64 + half * 32;
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 a, b;
          a.x = pack2<T>(__uint_as_float(rk[i]) * prm.scale, __uint_as_float(rk[i + 1]) * prm.scale);
          a.y = pack2<T>(__uint_as_float(rk[i + 2]) * prm.scale, __uint_as_float(rk[i + 3]) * prm.scale);
          a.z = pack2<T>(__uint_as_float(rk[i + 4]) * prm.scale, __uint_as_float(rk[i + 5]) * prm.scale);
          a.w = pack2<T>(__uint_as_float(rk[i + 6]) * prm.scale, __uint_as_float(rk[i + 7]) * prm.scale);
          b.x = pack2<T>(__uint_as_float(rv[i]), __uint_as_float(rv[i + 1]));
          b.y = pack2<T>(__uint_as_float(rv[i + 2]), __uint_as_float(rv[i + 3]));
          b.z = pack2<T>(__uint_as_float(rv[i + 4]), __uint_as_float(rv[i + 5]));
          b.w = pack2<T>(__uint_as_float(rv[i + 6]), __uint_as_float(rv[i + 7]));
          *reinterpret_cast<uint4*>(dk_row + i) = a;
          *reinterpret_cast<uint4*>(dv_row + i) = b;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem_base, kTmemCols);
}

// D = sum_d out*dout, LSE = m + log2(max(z, 1e-30)) into the padded layout; padding: D = 0, LSE = +inf
template <typename T>
__global__ void __launch_bounds__(256)
bwd_preprocess_pad_kernel(const T* __restrict__ out, const T* __restrict__ dout, const float* __restrict__ row_m,
                          const float* __restrict__ row_z, float* __restrict__ d_pad, float* __restrict__ lse_pad,
                          int bh, int n_ctx, int n_pad) {
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t prow = gid >> 3;                  // padded row index
  const int lane = static_cast<int>(gid & 7);
  const int64_t total = static_cast<int64_t>(bh) * n_pad;
  const int64_t b = prow / n_pad;
  const int r = static_cast<int>(prow - b * n_pad);
  const bool real = prow < total && r < n_ctx;
  float part = 0.f;
  if (real) {
    const T* o = out + (b * n_ctx + r) * 64 + lane * 8;
    const T* g = dout + (b * n_ctx + r) * 64 + lane * 8;
    uint4 ov = *reinterpret_cast<const uint4*>(o), gv = *reinterpret_cast<const uint4*>(g);
    const T* oe = reinterpret_cast<const T*>(&ov);
    const T* ge = reinterpret_cast<const T*>(&gv);
#pragma unroll
    for (int i = 0; i < 8; ++i) part += to_f32<T>(oe[i]) * to_f32<T>(ge[i]);
  }
  part += __shfl_xor_sync(0xffffffffu, part, 4);
  part += __shfl_xor_sync(0xffffffffu, part, 2);
  part += __shfl_xor_sync(0xffffffffu, part, 1);
  if (prow < total && lane == 0) {
    if (real) {
      d_pad[prow] = part;
      lse_pad[prow] = row_m[b * n_ctx + r] + log2f(fmaxf(row_z[b * n_ctx + r], 1.0e-30f));
    } else {
      d_pad[prow] = 0.f;
      lse_pad[prow] = CUDART_INF_F;
    }
  }
}

// dq = T(acc * scale)
template <typename T>
__global__ void __launch_bounds__(256)
dq_convert_kernel(const float* __restrict__ acc, T* __restrict__ dq, int64_t n_vec8, float scale) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec8) return;
  const float4 a = *reinterpret_cast<const float4*>(acc + i * 8);
  const float4 b = *reinterpret_cast<const float4*>(acc + i * 8 + 4);
  uint4 o;
  o.x = pack2<T>(a.x * scale, a.y * scale); o.y = pack2<T>(a.z * scale, a.w * scale);
  o.z = pack2<T>(b.x * scale, b.y * scale); o.w = pack2<T>(b.z * scale, b.w * scale);
  *reinterpret_cast<uint4*>(dq + i * 8) = o;
}

}  // namespace

bool bwd_tc_supported(int dtype, int head_dim, bool has_bias) { return fold_tc_supported(dtype, head_dim, has_bias); }

int64_t bwd_tc_workspace_bytes(int bh, int n_ctx) {
  const int64_t n_pad = align_up(n_ctx, 128);
  return 2 * align_up(static_cast<int64_t>(bh) * n_pad * 4, 256) + align_up(static_cast<int64_t>(bh) * n_ctx * 64 * 4, 256);
}

template <typename T>
static int bwd_tc_t(const BwdParams& p, const void* out, const float* row_m, const float* row_z, void* workspace,
                    int dtype, cudaStream_t st) {
  const int N = p.n_ctx, bh = p.bh;
  const int n_pad = static_cast<int>(align_up(N, 128));
  const int64_t vec_bytes = align_up(static_cast<int64_t>(bh) * n_pad * 4, 256);
  char* ws = static_cast<char*>(workspace);
  float* d_pad = reinterpret_cast<float*>(ws);
  float* lse_pad = reinterpret_cast<float*>(ws + vec_bytes);
  float* dq_acc = reinterpret_cast<float*>(ws + 2 * vec_bytes);
  const int64_t acc_elems = static_cast<int64_t>(bh) * N * 64;

  {
    const int64_t threads = static_cast<int64_t>(bh) * n_pad * 8;
    bwd_preprocess_pad_kernel<T><<<static_cast<unsigned>(cdiv64(threads, 256)), 256, 0, st>>>(
        static_cast<const T*>(out), static_cast<const T*>(p.dout), row_m, row_z, d_pad, lse_pad, bh, N, n_pad);
    ELSA_LAUNCH_CHECK();
  }
  ELSA_CUDA_CHECK(cudaMemsetAsync(dq_acc, 0, acc_elems * 4, st));

  CUtensorMap mq, mk, mv, mdo;
  int rc;
  if ((rc = make_tmap_rows64(&mq, p.q, dtype, N, bh, 128)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mk, p.k, dtype, N, bh, 128)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mv, p.v, dtype, N, bh, 128)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mdo, p.dout, dtype, N, bh, 128)) != ELSA_OK) return rc;
  BwdTcParams prm;
  prm.lse_pad = lse_pad; prm.d_pad = d_pad; prm.dq_acc = dq_acc; prm.dk = p.dk; prm.dv = p.dv;
  prm.n_ctx = N; prm.n_pad = n_pad; prm.bh = bh; prm.is_causal = p.is_causal;
  prm.scale = p.scale; prm.scale_log2 = p.scale_log2;
  rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&bwd_tc_kernel<T>), kBwdSmem);
  if (rc != ELSA_OK) return rc;
  dim3 grid(static_cast<unsigned>((N + 127) / 128), static_cast<unsigned>(bh));
  bwd_tc_kernel<T><<<grid, kThreads, kBwdSmem, st>>>(mq, mk, mv, mdo, prm);
  ELSA_LAUNCH_CHECK();
  dq_convert_kernel<T><<<static_cast<unsigned>(cdiv64(acc_elems / 8, 256)), 256, 0, st>>>(
      dq_acc, static_cast<T*>(p.dq), acc_elems / 8, p.scale);
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

int bwd_tc(const BwdParams& p, const void* out, const float* row_m, const float* row_z, void* workspace, int dtype,
           cudaStream_t st) {
  if (!bwd_tc_supported(dtype, p.head_dim, p.bias != nullptr) || p.dbias) return ELSA_ERR_UNSUPPORTED;
  if (dtype == ELSA_F16) return bwd_tc_t<__half>(p, out, row_m, row_z, workspace, dtype, st);
  return bwd_tc_t<__nv_bfloat16>(p, out, row_m, row_z, workspace, dtype, st);
}

int bwd_tc_status(int* status_out, int clear) {
  int v = 0;
  ELSA_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_bwd_status, sizeof(int)));
  if (clear && v != 0) {
    int zero = 0;
    ELSA_CUDA_CHECK(cudaMemcpyToSymbol(g_bwd_status, &zero, sizeof(int)));
  }
  *status_out = v;
  return ELSA_OK;
}

}  // namespace elsa
