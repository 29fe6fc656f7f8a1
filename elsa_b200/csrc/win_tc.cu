// Short sequences (49-token Swin windows and anything else of at most 64 tokens) on the 5th-generation tensor cores,
// fp16 / bf16, head dim <= 64 (multiples of 8), optional additive bias, causal or not: ONE launch, no partition summaries.
//
// A 128-row tcgen05 tile holds TWO sequences of the same head: one 4-D TMA box (64 columns x 64 rows x 1 head x 2
// batch entries) lands both in shared memory, each zero-padded to 64 rows and 64 columns by the box, as one 128 x 64
// operand tile.  One CTA (160 threads) per (pair of sequences, head):
//
//   warp 4 lane 0   TMA loads of the Q, K, V tiles; S = Q K^T (tcgen05.mma 128x128x16, only the two diagonal
//                   64 x 64 blocks are meaningful); after the fold warps have delivered P: O = P V (128x64x16 x 8)
//   warps 0-3       one thread per query row (rows 0-63: first sequence, 64-127: second): the row's own 64 scores from
//                   TMEM, scale + bias (read from global memory), softmax in registers, P (16-bit) into TMEM with
//                   zeros in the other sequence's columns, and after P V the row's output = O / z
//
// TMEM columns: S [0,128) O [128,192) P [192,256): two CTAs fit an SM.
#include <type_traits>

#include "kernels.cuh"
#include "tc_common.cuh"

namespace elsa {

using namespace tc;

namespace {

constexpr int kTileBytes = 128 * 64 * 2;          // two 64 x 64 16-bit sequences
constexpr int kBiasStride = 65;                   // floats per staged bias row: lanes that hold consecutive rows hit distinct banks
constexpr int kBiasBytes = 2 * 64 * kBiasStride * 4;   // the bias tiles of the two sequences
constexpr int kWinSmem = 3 * kTileBytes + kBiasBytes + 1024;   // Q, K, V, bias + alignment slack
constexpr int kThreads = 160;
constexpr uint32_t kTmemCols = 256;

enum BarId { BAR_LOAD = 71, BAR_S = 72, BAR_P = 73, BAR_O = 74 };

// The bias tiles [query][key] of the CTA's two sequences, copied into shared memory by `n_warps` warps (w = this warp's
// index among them): the lanes of a warp read consecutive keys of one query (coalesced when the key stride is 1), and
// afterwards a thread walks its own query row, or its own key column, without bank conflicts.
__device__ __forceinline__ void stage_bias(float* sb, const float* bias, int64_t bsb, int64_t bsh, int64_t bsq, int64_t bsk,
                                           int b0, int n_tiles, int batch, int hi, int N, int w, int n_warps, int lane) {
  for (int s2 = 0; s2 < n_tiles; ++s2) {
    if (b0 + s2 >= batch) break;
    const float* src = bias + static_cast<int64_t>(b0 + s2) * bsb + hi * bsh;
    float* dst = sb + s2 * 64 * kBiasStride;
    // eight rows of loads in flight per warp before the first store (N <= 64: two loads per row)
    for (int r0 = w; r0 < N; r0 += 8 * n_warps) {
      float t[8][2];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int r = r0 + j * n_warps;
        t[j][0] = (r < N && lane < N) ? src[static_cast<int64_t>(r) * bsq + lane * bsk] : 0.f;
        t[j][1] = (r < N && lane + 32 < N) ? src[static_cast<int64_t>(r) * bsq + (lane + 32) * bsk] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int r = r0 + j * n_warps;
        if (r < N) { dst[r * kBiasStride + lane] = t[j][0]; dst[r * kBiasStride + lane + 32] = t[j][1]; }
      }
    }
  }
}

struct WinParams {
  void* out; Strides os;
  float* row_m; float* row_z;                   // [B*H, N] row state (log2 domain), or null
  const float* bias; int64_t bsb, bsh, bsq, bsk;
  int batch, heads, n_ctx, head_dim, summary_dtype, causal;
  float scale_log2;
  int* status;
};

template <typename T>
__global__ void __launch_bounds__(kThreads, 2)
win_tc_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const WinParams prm) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b0 = blockIdx.x * 2, hi = blockIdx.y;
  const int N = prm.n_ctx, d = prm.head_dim;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base, sK = smem_base + kTileBytes, sV = smem_base + 2 * kTileBytes;
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_load = bar0, bar_s = bar0 + 8, bar_p = bar0 + 16, bar_o = bar0 + 24;

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_load, 1); mbar_init(bar_s, 1); mbar_init(bar_p, 4); mbar_init(bar_o, 1);
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tS = tmem_base, tO = tmem_base + 128, tP = tmem_base + 192;

  if (warp == 4) {
    if (lane == 0) {
      // ---------------- loads and MMAs ----------------
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      mbar_arrive_expect_tx(bar_load, 3 * kTileBytes);
      tma_load_4d(sQ, &tmap_q, bar_load, 0, 0, hi, b0);     // rows beyond N, columns beyond d, a batch entry beyond B: zeros
      tma_load_4d(sK, &tmap_k, bar_load, 0, 0, hi, b0);
      tma_load_4d(sV, &tmap_v, bar_load, 0, 0, hi, b0);
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc_s = make_idesc(fmt, 0, 0, 128, 128);   // S = Q K^T : A, B K-major
      constexpr uint32_t idesc_o = make_idesc(fmt, 0, 1, 128, 64);    // O = P V   : A in TMEM, B (V) MN-major
      bool ok = mbar_wait(bar_load, 0, &abort_flag, prm.status, BAR_LOAD);
      if (ok) {
        tc_fence_after();
        const uint64_t dq = make_sdesc(sQ, 16, 1024), dk = make_sdesc(sK, 16, 1024);
        const int ksteps = (d + 15) / 16;                     // the columns beyond d are zeros: their K-steps add nothing
        for (int ks = 0; ks < ksteps; ++ks) mma_ss(tS, dq + 2 * ks, dk + 2 * ks, idesc_s, ks > 0 ? 1u : 0u);
        mma_commit(bar_s);
        ok = mbar_wait(bar_p, 0, &abort_flag, prm.status, BAR_P);
      }
      if (ok) {
        tc_fence_after();
        const uint64_t dv = make_sdesc(sV, 128 * 128, 1024);
        mma_ts_x4<8, 128>(tO, tP, dv, idesc_o, 0u);
        mma_ts_x4<8, 128>(tO, tP + 32, dv + 512, idesc_o, 1u);
        mma_commit(bar_o);
      }
    }
  } else {
    // ---------------- fold warps: one thread per query row ----------------
    const int row = warp * 32 + lane;                       // row of the tile == TMEM lane
    const int seq = row >> 6, qi = row & 63;                // which of the two sequences, and the query index in it
    const int b = b0 + seq;
    const bool row_ok = b < prm.batch && qi < N;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    const float c = prm.scale_log2;
    float* sb = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)) + 3 * kTileBytes);
    if (prm.bias) {                                         // (while the loads and the S MMA are in flight)
      stage_bias(sb, prm.bias, prm.bsb, prm.bsh, prm.bsq, prm.bsk, b0, prm.bsb != 0 ? 2 : 1, prm.batch, hi, N, warp, 4, lane);
      named_barrier_sync(1, 128);
    }
    bool alive = __all_sync(0xffffffffu, mbar_wait(bar_s, 0, &abort_flag, prm.status, BAR_S));
    float z = 0.f, m = -CUDART_INF_F;
    if (alive) {
      tc_fence_after();
      float sv[64];
      {
        uint32_t r0[32], r1[32];
        tmem_ld32(tS + lane_off + 64 * seq, r0);            // the row's own sequence: the diagonal block
        tmem_ld32(tS + lane_off + 64 * seq + 32, r1);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) { sv[i] = __uint_as_float(r0[i]) * c; sv[32 + i] = __uint_as_float(r1[i]) * c; }
      }
      if (prm.bias) {                                        // (uniform; every load is inside the staged tile, a select drops what is not bias)
        const float* bp = sb + ((prm.bsb != 0 ? seq * 64 : 0) + (row_ok ? qi : 0)) * kBiasStride;   // (one tile when the bias ignores the batch index)
        const int n_b = row_ok ? N : 0;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          float bv = bp[i];
          bv = (i < n_b) ? bv : 0.f;
          sv[i] = fmaf(bv, 1.4426950408889634f, sv[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < 64; ++i)
        if (i >= N || (prm.causal && i > qi)) sv[i] = -CUDART_INF_F;
      float mx[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
      for (int i = 4; i < 64; i += 4) {
        mx[0] = fmaxf(mx[0], sv[i]); mx[1] = fmaxf(mx[1], sv[i + 1]);
        mx[2] = fmaxf(mx[2], sv[i + 2]); mx[3] = fmaxf(mx[3], sv[i + 3]);
      }
      m = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      const float m_use = (m == -CUDART_INF_F) ? 0.f : m;   // a row whose keys are all masked by the bias: p = 0 everywhere
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[32], zero[32];
#pragma unroll
      for (int i = 0; i < 64; i += 2) {
        const float p0 = fast_exp2(sv[i] - m_use), p1 = fast_exp2(sv[i + 1] - m_use);
        ps[(i >> 1) & 3] += p0 + p1;
        pk[i >> 1] = pack2<T>(p0, p1);
      }
      z = (ps[0] + ps[1]) + (ps[2] + ps[3]);
#pragma unroll
      for (int i = 0; i < 32; ++i) zero[i] = 0u;
      // P of this row over the 128 keys of the tile: its own sequence's 64 keys, zeros for the other sequence's
      tmem_st32(tP + lane_off + 32 * seq, pk);
      tmem_st32(tP + lane_off + 32 * (1 - seq), zero);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(bar_p, lane);
      alive = __all_sync(0xffffffffu, mbar_wait(bar_o, 0, &abort_flag, prm.status, BAR_O));
    }
    if (alive) {
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld32(tO + lane_off, r0);
      tmem_ld32(tO + lane_off + 32, r1);
      tmem_wait_ld();
      if (row_ok) {
        const float inv = z > 0.f ? 1.f / z : 0.f;
        T* dst = static_cast<T*>(prm.out) + static_cast<int64_t>(b) * prm.os.b + hi * prm.os.h + static_cast<int64_t>(qi) * prm.os.r;
#pragma unroll
        for (int i = 0; i < 64; i += 8) {
          if (i >= d) continue;
          float o[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float x = __uint_as_float(i + e < 32 ? r0[(i + e) & 31] : r1[(i + e) & 31]);
            // the two-pass path stores the partition summary in the summary type before dividing: same rounding points
            if (prm.summary_dtype == ELSA_F16) x = round_to<__half>(x);
            else if (prm.summary_dtype == ELSA_BF16) x = round_to<__nv_bfloat16>(x);
            o[e] = x * inv;
          }
          uint4 t;
          t.x = pack2<T>(o[0], o[1]); t.y = pack2<T>(o[2], o[3]); t.z = pack2<T>(o[4], o[5]); t.w = pack2<T>(o[6], o[7]);
          *reinterpret_cast<uint4*>(dst + i) = t;
        }
        if (prm.row_m) {
          const int64_t ro = (static_cast<int64_t>(b) * prm.heads + hi) * N + qi;
          prm.row_m[ro] = z > 0.f ? m : -CUDART_INF_F;
          prm.row_z[ro] = z;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, kTmemCols);
}


// ------------------------------------------------------------------------------------------------------------------
// Backward of the same problems, one launch: dQ, dK, dV (and dbias) of two sequences of one head per CTA.
//
//   first MMAs (issuer)   S^T = K Q^T, dP^T = V dO^T (the key side starts), S = Q K^T, dP = dO V^T (the query side starts):
//                      four 128 x 128 tiles = all 512 TMEM columns
//   query side (warps 0-3, thread = query row)   -LSE and -D of the row, published in shared memory;
//                      P = 2^(S c + bias - LSE), dS = P (dP - D) over the row's own sequence; dS (16-bit) written over
//                      the row's S columns
//   key side (warps 4-7, thread = key row, at the same time)   P^T, dS^T from S^T, dP^T with the queries' -LSE / -D;
//                      written over the S^T columns; dbias += dS^T (the lanes of a warp hold consecutive keys: coalesced)
//   second MMAs (issuer)  dQ = dS K -> the dP columns as soon as the query side is done; dV = P^T dO, dK = dS^T Q -> the
//                      dP^T columns as soon as the key side is done
//   epilogue           the query side stores dQ, the key side dV and dK
//
// TMEM columns: S [0,128) (later dS in [0,64)), dP [128,256) (later dQ in [128,192)), S^T [256,384) (later P^T in
// [256,320), dS^T in [320,384)), dP^T [384,512) (later dV in [384,448), dK in [448,512)).  A thread only ever touches its
// own TMEM lane, and it has read everything it needs from a column range before it writes there.
// ------------------------------------------------------------------------------------------------------------------
constexpr int kBwdStageBytes = 5 * kTileBytes;       // Q, K, V, dO, out of one pair of sequences
constexpr int kBiasTile = 64 * kBiasStride;          // floats of one staged bias (or dbias) tile
// two stages, three tiles (bias of the two sequences; or one bias tile and a dbias sum per sequence), alignment slack
constexpr int kWinBwdSmem = 2 * kBwdStageBytes + 3 * kBiasTile * 4 + 1024;
constexpr int kBwdThreads = 544;                     // 8 query-side warps, 8 key-side warps (two threads per row), 1 issuing warp

enum BwdBarId { BAR_BLOAD = 75, BAR_R1 = 76, BAR_PHQ = 77, BAR_PHK = 78, BAR_R2Q = 79, BAR_R2K = 80, BAR_EPI = 81, BAR_PUB = 82, BAR_BIAS = 83, BAR_R1K = 84 };

struct WinBwdParams {
  const void* out; Strides os; const void* dout; Strides gs;
  const float* row_m; const float* row_z;
  const float* bias; int64_t bsb, bsh, bsq, bsk;
  float* dbias; int64_t dsb, dsh, dsq, dsk; int dbias_atomic;
  void* dq; void* dk; void* dv; Strides dqs, dks, dvs;
  int batch, heads, n_ctx, head_dim, causal;
  float scale, scale_log2;
  int* status;
};

// half an accumulator row (32 fp32 columns at `src`) scaled by f and stored as up to 32 elements of T (n = how many of
// them exist: the head dim minus the half's first column)
template <typename T>
__device__ __forceinline__ void store_acc_half(uint32_t src, T* dst, int n, float f) {
  uint32_t r[32];
  tmem_ld32(src, r);
  tmem_wait_ld();
  if (!dst) return;
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    if (i >= n) continue;
    uint4 t;
    t.x = pack2<T>(__uint_as_float(r[i]) * f, __uint_as_float(r[i + 1]) * f);
    t.y = pack2<T>(__uint_as_float(r[i + 2]) * f, __uint_as_float(r[i + 3]) * f);
    t.z = pack2<T>(__uint_as_float(r[i + 4]) * f, __uint_as_float(r[i + 5]) * f);
    t.w = pack2<T>(__uint_as_float(r[i + 6]) * f, __uint_as_float(r[i + 7]) * f);
    *reinterpret_cast<uint4*>(dst + i) = t;
  }
}

// -D of a row = -sum(out * dout) over the row's 128 bytes in two 128-byte-swizzled tiles (chunk c of row r sits at
// chunk c ^ (r & 7)); columns beyond the head dim are zeros
template <typename T>
__device__ __forceinline__ float neg_row_dot(const uint8_t* t_out, const uint8_t* t_do, int r, int d) {
  float acc = 0.f;
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) {
    if (ch * 8 >= d) continue;
    const int off = r * 128 + ((ch ^ (r & 7)) << 4);
    const uint4 ov = *reinterpret_cast<const uint4*>(t_out + off), gv = *reinterpret_cast<const uint4*>(t_do + off);
    const T* oe = reinterpret_cast<const T*>(&ov);
    const T* ge = reinterpret_cast<const T*>(&gv);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc = fmaf(to_f32<T>(oe[e]), to_f32<T>(ge[e]), acc);
  }
  return -acc;
}

// Persistent: CTA c works on head c % heads and on the pairs of sequences c / heads, c / heads + G, ... (G = gridDim.x /
// heads).  The five tiles of the next pair are in flight while this one is computed (two stages of shared memory); a
// bias that does not depend on the batch index is staged once.
template <typename T>
__global__ void __launch_bounds__(kBwdThreads, 1)
win_tc_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                  const __grid_constant__ CUtensorMap tmap_o, const WinBwdParams prm) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[11];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float nlse_s[2][128], nd_s[2][128];   // -LSE and -D of the tile's 128 query rows, per iteration parity

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hi = blockIdx.x % prm.heads;
  const int pair0 = blockIdx.x / prm.heads, pair_step = gridDim.x / prm.heads;
  const int n_pairs = (prm.batch + 1) / 2;
  const int N = prm.n_ctx, d = prm.head_dim;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  // stage s: Q, K, V, dO, out at smem_base + s * kBwdStageBytes + {0..4} * kTileBytes
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_load = bar0 /* [2] */, bar_r1 = bar0 + 16, bar_phq = bar0 + 24, bar_phk = bar0 + 32, bar_r2q = bar0 + 40,
                 bar_r2k = bar0 + 48, bar_epi = bar0 + 56, bar_pub = bar0 + 64, bar_bias = bar0 + 72, bar_r1k = bar0 + 80;

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_load, 1); mbar_init(bar_load + 8, 1); mbar_init(bar_r1, 1); mbar_init(bar_phq, 8); mbar_init(bar_phk, 8);
    mbar_init(bar_r2q, 1); mbar_init(bar_r2k, 1); mbar_init(bar_epi, 16); mbar_init(bar_pub, 4); mbar_init(bar_bias, 8); mbar_init(bar_r1k, 1);
    fence_mbar_init();
  }
  if (warp == 16) {
    tmem_alloc(smem_u32(&tmem_base_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tST = tmem_base + 256, tdPT = tmem_base + 384;

  // Fold warps 0-7 are the query side, 8-15 the key side.  Two threads share a row of the tile (= a TMEM lane): warp w
  // works on lane quadrant w % 4 and on half (w / 4) % 2 of the row's 64 columns.
  const int wq = warp & 3, half = (warp >> 2) & 1;
  const int row = wq * 32 + lane;
  const int seq = row >> 6, ri = row & 63;                // which of the two sequences, and the row's index in it
  const uint32_t lane_off = static_cast<uint32_t>(wq * 32) << 16;
  const int pair_bar = 2 + (warp >> 3) * 4 + wq;          // named barrier of the two warps that share this quadrant
  const float c = prm.scale_log2;
  float* sb = reinterpret_cast<float*>(smem_al + 2 * kBwdStageBytes);
  const bool bias_per_batch = prm.bias && prm.bsb != 0;   // else one tile serves every pair of this head
  const float* sb_seq = sb + (bias_per_batch ? seq * kBiasTile : 0);

  if (warp == 16) {
    if (lane == 0 && pair0 < n_pairs) {
      // ---------------- loads and MMAs ----------------
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_do); prefetch_tmap(&tmap_o);
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc_s = make_idesc(fmt, 0, 0, 128, 128);   // A, B K-major, N = 128
      constexpr uint32_t idesc_o = make_idesc(fmt, 0, 1, 128, 64);    // A in TMEM, B MN-major, N = 64
      const int ksteps = (d + 15) / 16;                     // the columns beyond d are zeros: their K-steps add nothing
      auto issue_loads = [&](int pair, int stage) {         // rows beyond N, columns beyond d, a batch entry beyond B: zeros
        const uint32_t base = smem_base + stage * kBwdStageBytes, bar = bar_load + 8 * stage;
        mbar_arrive_expect_tx(bar, 5 * kTileBytes);
        tma_load_4d(base, &tmap_q, bar, 0, 0, hi, 2 * pair);
        tma_load_4d(base + kTileBytes, &tmap_k, bar, 0, 0, hi, 2 * pair);
        tma_load_4d(base + 2 * kTileBytes, &tmap_v, bar, 0, 0, hi, 2 * pair);
        tma_load_4d(base + 3 * kTileBytes, &tmap_do, bar, 0, 0, hi, 2 * pair);
        tma_load_4d(base + 4 * kTileBytes, &tmap_o, bar, 0, 0, hi, 2 * pair);
      };
      issue_loads(pair0, 0);
      int it = 0;
      for (int pair = pair0; pair < n_pairs; pair += pair_step, ++it) {
        const int stage = it & 1;
        const uint32_t ph = it & 1;
        const uint32_t sQ = smem_base + stage * kBwdStageBytes, sK = sQ + kTileBytes, sV = sQ + 2 * kTileBytes, sDO = sQ + 3 * kTileBytes;
        if (!mbar_wait(bar_load + 8 * stage, (it >> 1) & 1, &abort_flag, prm.status, BAR_BLOAD)) break;
        // the fold warps have read the gradients of the previous pair out of TMEM (and its tiles out of the other stage)
        if (it > 0 && !mbar_wait(bar_epi, (it - 1) & 1, &abort_flag, prm.status, BAR_EPI)) break;
        tc_fence_after();
        const uint64_t dq = make_sdesc(sQ, 16, 1024), dk = make_sdesc(sK, 16, 1024);
        const uint64_t dv = make_sdesc(sV, 16, 1024), ddo = make_sdesc(sDO, 16, 1024);
        // the key side has the longer way to go (two products, two gradients): its inputs first
        for (int ks = 0; ks < ksteps; ++ks) mma_ss(tST, dk + 2 * ks, dq + 2 * ks, idesc_s, ks > 0 ? 1u : 0u);
        for (int ks = 0; ks < ksteps; ++ks) mma_ss(tdPT, dv + 2 * ks, ddo + 2 * ks, idesc_s, ks > 0 ? 1u : 0u);
        mma_commit(bar_r1k);
        for (int ks = 0; ks < ksteps; ++ks) mma_ss(tS, dq + 2 * ks, dk + 2 * ks, idesc_s, ks > 0 ? 1u : 0u);
        for (int ks = 0; ks < ksteps; ++ks) mma_ss(tdP, ddo + 2 * ks, dv + 2 * ks, idesc_s, ks > 0 ? 1u : 0u);
        mma_commit(bar_r1);
        if (pair + pair_step < n_pairs) issue_loads(pair + pair_step, stage ^ 1);
        const uint64_t k_mn = make_sdesc(sK, 128 * 128, 1024), q_mn = make_sdesc(sQ, 128 * 128, 1024);
        const uint64_t do_mn = make_sdesc(sDO, 128 * 128, 1024);
        if (!mbar_wait(bar_phq, ph, &abort_flag, prm.status, BAR_PHQ)) break;
        tc_fence_after();
        mma_ts_x4<8, 128>(tdP, tS, k_mn, idesc_o, 0u);                 // dQ = dS K
        mma_ts_x4<8, 128>(tdP, tS + 32, k_mn + 512, idesc_o, 1u);
        mma_commit(bar_r2q);
        if (!mbar_wait(bar_phk, ph, &abort_flag, prm.status, BAR_PHK)) break;
        tc_fence_after();
        mma_ts_x4<8, 128>(tdPT, tST, do_mn, idesc_o, 0u);              // dV = P^T dO
        mma_ts_x4<8, 128>(tdPT, tST + 32, do_mn + 512, idesc_o, 1u);
        mma_ts_x4<8, 128>(tdPT + 64, tST + 64, q_mn, idesc_o, 0u);     // dK = dS^T Q
        mma_ts_x4<8, 128>(tdPT + 64, tST + 96, q_mn + 512, idesc_o, 1u);
        mma_commit(bar_r2k);
      }
    }
  } else if (warp < 8) {
    // ---------------- query-side warps: thread = (query row, half of its keys) ----------------
    auto load_state = [&](int pair, float& m, float& z) {
      const int bb = 2 * pair + seq;
      m = -CUDART_INF_F; z = 0.f;
      if (half == 0 && pair < n_pairs && bb < prm.batch && ri < N) {
        const int64_t ro = (static_cast<int64_t>(bb) * prm.heads + hi) * N + ri;
        m = prm.row_m[ro]; z = prm.row_z[ro];
      }
    };
    float m_next, z_next;
    load_state(pair0, m_next, z_next);
    int it = 0;
    for (int pair = pair0; pair < n_pairs; pair += pair_step, ++it) {
      const int stage = it & 1;
      const uint32_t ph = it & 1;
      const int b = 2 * pair + seq;
      const bool row_ok = b < prm.batch && ri < N;
      const uint8_t* tiles = smem_al + stage * kBwdStageBytes;
      if (half == 0) {
        // -LSE and -D of this row, published for the row's other thread and for the key-side warps
        float nl0 = -CUDART_INF_F;
        if (z_next > 0.f && m_next > -CUDART_INF_F) nl0 = -(m_next + log2f(z_next));   // (a row whose keys are all masked keeps P = 0)
        load_state(pair + pair_step, m_next, z_next);
        if (!__all_sync(0xffffffffu, mbar_wait(bar_load + 8 * stage, (it >> 1) & 1, &abort_flag, prm.status, BAR_BLOAD))) break;
        nlse_s[ph][row] = nl0;
        nd_s[ph][row] = neg_row_dot<T>(tiles + 4 * kTileBytes, tiles + 3 * kTileBytes, row, d);
        mbar_arrive_warp(bar_pub, lane);
      }
      if (prm.bias && !__all_sync(0xffffffffu, mbar_wait(bar_bias, ph, &abort_flag, prm.status, BAR_BIAS))) break;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_r1, ph, &abort_flag, prm.status, BAR_R1))) break;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_pub, ph, &abort_flag, prm.status, BAR_PUB))) break;
      tc_fence_after();
      {
        const float nlse = nlse_s[ph][row], nd = nd_s[ph][row];
        // this thread's 32 keys of the row's own sequence
        uint32_t rs[32], rp[32];
        tmem_ld32(tS + lane_off + 64 * seq + 32 * half, rs);
        tmem_ld32(tdP + lane_off + 64 * seq + 32 * half, rp);
        tmem_wait_ld();
        // dS goes over S columns that the row's other thread reads: both have their scores in registers from here on
        named_barrier_sync(pair_bar, 64);
        // The loops below are free of branches, so that the 32 independent chains (scale, exponential, mask, product)
        // overlap; with a conditional bias load inside, every element was a basic block of its own and ran in ~100 cycles.
        float t[32];                                        // s c + bias log2(e) - LSE
        if (prm.bias) {                                     // (uniform; every load is inside the staged tile, a select drops what is not bias)
          const float* bp = sb_seq + (row_ok ? ri : 0) * kBiasStride + 32 * half;
          const int n_b = row_ok ? N - 32 * half : 0;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float bv = bp[i];
            bv = (i < n_b) ? bv : 0.f;
            t[i] = fmaf(__uint_as_float(rs[i]), c, fmaf(bv, 1.4426950408889634f, nlse));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) t[i] = fmaf(__uint_as_float(rs[i]), c, nlse);
        }
        const int k_lim = prm.causal ? min(N, ri + 1) : N;  // keys kk < k_lim take part
        uint32_t zero[16];
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {                 // (stored as soon as eight are packed: fewer live registers)
          uint32_t dsk[8];
#pragma unroll
          for (int i = 16 * sub; i < 16 * sub + 16; i += 2) {
            float dsv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              float p = fast_exp2(t[i + e]);
              p = (32 * half + i + e < k_lim) ? p : 0.f;
              dsv[e] = p * (__uint_as_float(rp[i + e]) + nd);
            }
            dsk[(i >> 1) & 7] = pack2<T>(dsv[0], dsv[1]);
          }
          // dS of this query row over the 128 keys of the tile: its own sequence's 64 keys, zeros for the other's
          tmem_st8(tS + lane_off + 32 * seq + 16 * half + 8 * sub, dsk);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) zero[i] = 0u;
        tmem_st16(tS + lane_off + 32 * (1 - seq) + 16 * half, zero);
        tmem_wait_st();
      }
      tc_fence_before();
      mbar_arrive_warp(bar_phq, lane);
      if (!__all_sync(0xffffffffu, mbar_wait(bar_r2q, ph, &abort_flag, prm.status, BAR_R2Q))) break;
      tc_fence_after();
      T* dst = row_ok ? static_cast<T*>(prm.dq) + static_cast<int64_t>(b) * prm.dqs.b + hi * prm.dqs.h + static_cast<int64_t>(ri) * prm.dqs.r + 32 * half : nullptr;
      store_acc_half<T>(tdP + lane_off + 32 * half, dst, d - 32 * half, prm.scale);
      tc_fence_before();
      mbar_arrive_warp(bar_epi, lane);
      // the key side has consumed this pair's -LSE / -D (and the barrier phase that published them) before the next
      // pair's are published
      if (!__all_sync(0xffffffffu, mbar_wait(bar_r2k, ph, &abort_flag, prm.status, BAR_R2K))) break;
    }
  } else {
    // ---------------- key-side warps: thread = (key row, half of the queries) ----------------
    // A bias gradient shared by the batch (with a bias that is, so that two tiles of the bias buffer are free) is summed
    // over all the CTA's pairs in shared memory, one tile per sequence of the pair and every element by one thread only,
    // and added to global memory once, at the end.
    const bool dbias_local = prm.dbias && prm.dbias_atomic && prm.dsb == 0 && !bias_per_batch;
    float* dacc = sb + (1 + seq) * kBiasTile + ri + 32 * half * kBiasStride;   // this thread's half column of its sequence's tile
    if (dbias_local) {
      for (int qq = 0; qq < 32; ++qq) dacc[qq * kBiasStride] = 0.f;
    }
    bool completed = true;
    int it = 0;
    for (int pair = pair0; pair < n_pairs; pair += pair_step, ++it) {
      completed = false;
      const uint32_t ph = it & 1;
      const int b = 2 * pair + seq;
      const bool row_ok = b < prm.batch && ri < N;
      if (prm.bias) {
        // (the query side has finished with the tiles of the previous pair: its dS was an input of that pair's last MMAs)
        if (bias_per_batch) stage_bias(sb, prm.bias, prm.bsb, prm.bsh, prm.bsq, prm.bsk, 2 * pair, 2, prm.batch, hi, N, warp & 7, 8, lane);
        else if (it == 0) stage_bias(sb, prm.bias, 0, prm.bsh, prm.bsq, prm.bsk, 0, 1, prm.batch, hi, N, warp & 7, 8, lane);
        mbar_arrive_warp(bar_bias, lane);
        if (!__all_sync(0xffffffffu, mbar_wait(bar_bias, ph, &abort_flag, prm.status, BAR_BIAS))) break;   // all eight warps' rows
      }
      if (!__all_sync(0xffffffffu, mbar_wait(bar_pub, ph, &abort_flag, prm.status, BAR_PUB))) break;   // -LSE, -D of the 128 queries
      if (!__all_sync(0xffffffffu, mbar_wait(bar_r1k, ph, &abort_flag, prm.status, BAR_R1K))) break;
      tc_fence_after();
      {
        // this thread's 32 queries of the key's own sequence
        uint32_t rs[32], rp[32];
        tmem_ld32(tST + lane_off + 64 * seq + 32 * half, rs);
        tmem_ld32(tdPT + lane_off + 64 * seq + 32 * half, rp);
        tmem_wait_ld();
        // P^T and dS^T go over S^T columns that the row's other thread reads: both have them in registers from here on
        named_barrier_sync(pair_bar, 64);
        // bias[query, key] and dbias[query, key] of this key column: the lanes of a warp hold consecutive keys of one
        // query, so that every store or reduction of a warp is one coalesced access
        float* dbc = (prm.dbias && row_ok) ? prm.dbias + static_cast<int64_t>(b) * prm.dsb + hi * prm.dsh + static_cast<int64_t>(ri) * prm.dsk + static_cast<int64_t>(32 * half) * prm.dsq : nullptr;
        const float* nl = nlse_s[ph] + 64 * seq + 32 * half;
        const float* ndp = nd_s[ph] + 64 * seq + 32 * half;
        // branch-free loops (see the query side): P^T into pv, dS^T into dsv, then the bias gradient, then the packing
        float pv[32], dsv[32];
        if (prm.bias) {                                     // (uniform; loads inside the staged tile, see the query side)
          const float* bc = sb_seq + (row_ok ? ri : 0) + 32 * half * kBiasStride;
          const int n_b = row_ok ? N - 32 * half : 0;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float bv = bc[i * kBiasStride];
            bv = (i < n_b) ? bv : 0.f;
            pv[i] = fmaf(__uint_as_float(rs[i]), c, fmaf(bv, 1.4426950408889634f, nl[i]));   // (-inf for queries that do not exist)
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) pv[i] = fmaf(__uint_as_float(rs[i]), c, nl[i]);
        }
        const int q_min = !row_ok ? 64 : (prm.causal ? ri : 0);   // queries qq >= q_min see this key (none when it does not exist)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float p = fast_exp2(pv[i]);
          p = (32 * half + i >= q_min) ? p : 0.f;
          pv[i] = p;
          dsv[i] = p * (__uint_as_float(rp[i]) + ndp[i]);
        }
        if (dbc) {
          const int n_q = min(32, N - 32 * half);             // this thread's queries that exist
          if (dbias_local) {                                 // (all 32 rows of the half column exist in the tile)
#pragma unroll
            for (int i = 0; i < 32; ++i) dacc[i * kBiasStride] += (i < n_q) ? dsv[i] : 0.f;
          } else if (prm.dbias_atomic) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < n_q) atomicAdd(dbc + static_cast<int64_t>(i) * prm.dsq, dsv[i]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < n_q) dbc[static_cast<int64_t>(i) * prm.dsq] = dsv[i];
          }
        }
        uint32_t zero[16];
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
          uint32_t pk[8], dsk[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            pk[i] = pack2<T>(pv[16 * sub + 2 * i], pv[16 * sub + 2 * i + 1]);
            dsk[i] = pack2<T>(dsv[16 * sub + 2 * i], dsv[16 * sub + 2 * i + 1]);
          }
          tmem_st8(tST + lane_off + 32 * seq + 16 * half + 8 * sub, pk);             // P^T over the tile's 128 queries
          tmem_st8(tST + 64 + lane_off + 32 * seq + 16 * half + 8 * sub, dsk);       // dS^T
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) zero[i] = 0u;
        tmem_st16(tST + lane_off + 32 * (1 - seq) + 16 * half, zero);
        tmem_st16(tST + 64 + lane_off + 32 * (1 - seq) + 16 * half, zero);
        tmem_wait_st();
      }
      tc_fence_before();
      mbar_arrive_warp(bar_phk, lane);
      if (!__all_sync(0xffffffffu, mbar_wait(bar_r2k, ph, &abort_flag, prm.status, BAR_R2K))) break;
      tc_fence_after();
      T* dvp = row_ok ? static_cast<T*>(prm.dv) + static_cast<int64_t>(b) * prm.dvs.b + hi * prm.dvs.h + static_cast<int64_t>(ri) * prm.dvs.r + 32 * half : nullptr;
      T* dkp = row_ok ? static_cast<T*>(prm.dk) + static_cast<int64_t>(b) * prm.dks.b + hi * prm.dks.h + static_cast<int64_t>(ri) * prm.dks.r + 32 * half : nullptr;
      store_acc_half<T>(tdPT + lane_off + 32 * half, dvp, d - 32 * half, 1.f);
      store_acc_half<T>(tdPT + 64 + lane_off + 32 * half, dkp, d - 32 * half, prm.scale);
      tc_fence_before();
      mbar_arrive_warp(bar_epi, lane);
      completed = true;
    }
    if (dbias_local && completed && ri < N) {                // (nothing is added after a wait that gave up)
      float* dst = prm.dbias + hi * prm.dsh + static_cast<int64_t>(ri) * prm.dsk + static_cast<int64_t>(32 * half) * prm.dsq;
      for (int qq = 0; qq < 32 && 32 * half + qq < N; ++qq) atomicAdd(dst + static_cast<int64_t>(qq) * prm.dsq, dacc[qq * kBiasStride]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 16) tmem_dealloc(tmem_base, 512);
}

}  // namespace

bool win_tc_supported(int dtype, int head_dim, int n_ctx, bool is_causal) {
  (void)is_causal;   // both forms are covered
  return (dtype == ELSA_F16 || dtype == ELSA_BF16) && head_dim >= 8 && head_dim <= 64 && head_dim % 8 == 0 && n_ctx >= 1 &&
         n_ctx <= 64 && fold_tc_supported(dtype, 64, false);
}

// q, k, v, out: [B, H, N <= 64, D <= 64] views with element strides; bias (fp32, may be null) with its four strides;
// row_m / row_z may be null
int win_tc_fwd(const void* q, Strides qs, const void* k, Strides ks, const void* v, Strides vs, const float* bias,
               int64_t bsb, int64_t bsh, int64_t bsq, int64_t bsk, void* out, Strides os, float* row_m, float* row_z,
               int dtype, int summary_dtype, int batch, int heads, int n_ctx, int head_dim, float scale_log2,
               int is_causal, cudaStream_t st) {
  if (!win_tc_supported(dtype, head_dim, n_ctx, is_causal != 0)) return ELSA_ERR_UNSUPPORTED;
  CUtensorMap mq, mk, mv;
  int rc;
  // one box = 64 columns x 64 rows x 1 head x 2 batch entries: two sequences, each padded to 64 x 64 by the fill
  if ((rc = make_tmap_rows64(&mq, q, dtype, n_ctx, heads, batch, qs, 64, head_dim, 2)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mk, k, dtype, n_ctx, heads, batch, ks, 64, head_dim, 2)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mv, v, dtype, n_ctx, heads, batch, vs, 64, head_dim, 2)) != ELSA_OK) return rc;
  WinParams prm;
  prm.out = out; prm.os = os; prm.row_m = row_m; prm.row_z = row_z;
  prm.bias = bias; prm.bsb = bsb; prm.bsh = bsh; prm.bsq = bsq; prm.bsk = bsk;
  prm.batch = batch; prm.heads = heads; prm.n_ctx = n_ctx; prm.head_dim = head_dim; prm.summary_dtype = summary_dtype;
  prm.causal = is_causal ? 1 : 0;
  prm.scale_log2 = scale_log2;
  if ((rc = device_status_word(&prm.status, nullptr)) != ELSA_OK) return rc;
  const dim3 grid(static_cast<unsigned>((batch + 1) / 2), static_cast<unsigned>(heads));
  if (dtype == ELSA_F16) {
    if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&win_tc_fwd_kernel<__half>), kWinSmem)) != ELSA_OK) return rc;
    win_tc_fwd_kernel<__half><<<grid, kThreads, kWinSmem, st>>>(mq, mk, mv, prm);
  } else {
    if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&win_tc_fwd_kernel<__nv_bfloat16>), kWinSmem)) != ELSA_OK) return rc;
    win_tc_fwd_kernel<__nv_bfloat16><<<grid, kThreads, kWinSmem, st>>>(mq, mk, mv, prm);
  }
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

int win_tc_bwd(const BwdParams& p, int dtype, cudaStream_t st) {
  if (!win_tc_supported(dtype, p.head_dim, p.n_ctx, p.is_causal != 0) || p.n_keys != p.n_ctx || p.key_offset != 0 || p.dq_f32 ||
      !p.out || !p.row_m || !p.row_z || (p.dbias && !p.bias))
    return ELSA_ERR_UNSUPPORTED;
  const int batch = p.bh / p.heads;
  CUtensorMap mq, mk, mv, mdo, mo;
  int rc;
  if ((rc = make_tmap_rows64(&mo, p.out, dtype, p.n_ctx, p.heads, batch, p.os, 64, p.head_dim, 2)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mq, p.q, dtype, p.n_ctx, p.heads, batch, p.qs, 64, p.head_dim, 2)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mk, p.k, dtype, p.n_ctx, p.heads, batch, p.ks, 64, p.head_dim, 2)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mv, p.v, dtype, p.n_ctx, p.heads, batch, p.vs, 64, p.head_dim, 2)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mdo, p.dout, dtype, p.n_ctx, p.heads, batch, p.gs, 64, p.head_dim, 2)) != ELSA_OK) return rc;
  WinBwdParams prm;
  prm.out = p.out; prm.os = p.os; prm.dout = p.dout; prm.gs = p.gs;
  prm.row_m = p.row_m; prm.row_z = p.row_z;
  prm.bias = p.bias; prm.bsb = p.bsb; prm.bsh = p.bsh; prm.bsq = p.bsq; prm.bsk = p.bsk;
  prm.dbias = p.dbias; prm.dsb = p.dsb; prm.dsh = p.dsh; prm.dsq = p.dsq; prm.dsk = p.dsk; prm.dbias_atomic = p.dbias_atomic;
  prm.dq = p.dq; prm.dk = p.dk; prm.dv = p.dv; prm.dqs = p.dqs; prm.dks = p.dks; prm.dvs = p.dvs;
  prm.batch = batch; prm.heads = p.heads; prm.n_ctx = p.n_ctx; prm.head_dim = p.head_dim; prm.causal = p.is_causal ? 1 : 0;
  prm.scale = p.scale; prm.scale_log2 = p.scale_log2;
  if ((rc = device_status_word(&prm.status, nullptr)) != ELSA_OK) return rc;
  // persistent: one CTA per SM at most, a multiple of the head count (a CTA stays with one head)
  const int sms = sm_count();
  const int n_pairs = (batch + 1) / 2;
  const int groups = std::max(1, std::min(sms / p.heads, n_pairs));
  const dim3 grid(static_cast<unsigned>(groups * p.heads));
  if (dtype == ELSA_F16) {
    if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&win_tc_bwd_kernel<__half>), kWinBwdSmem)) != ELSA_OK) return rc;
    win_tc_bwd_kernel<__half><<<grid, kBwdThreads, kWinBwdSmem, st>>>(mq, mk, mv, mdo, mo, prm);
  } else {
    if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&win_tc_bwd_kernel<__nv_bfloat16>), kWinBwdSmem)) != ELSA_OK) return rc;
    win_tc_bwd_kernel<__nv_bfloat16><<<grid, kBwdThreads, kWinBwdSmem, st>>>(mq, mk, mv, mdo, mo, prm);
  }
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

}  // namespace elsa
