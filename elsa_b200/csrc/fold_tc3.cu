// Phase 1 for fp32 inputs on the 5th-generation tensor cores WITHOUT giving up fp32-grade accuracy: every operand is
// split into a few 16-bit planes and a product a*b is formed from the cross terms of the planes, each an exact
// 16-bit x 16-bit product accumulated in fp32 by tcgen05.mma (kind::f16).  Two forms, chosen at compile time
// (ELSA_FP32_PLANES, tc_common.cuh):
//   2 planes (default): x * 2^e = h0 + h1 in fp16 (11 + 11 significant bits; e puts the tensor's largest magnitude in
//     [2^13, 2^14)), a*b = h0 h0 + h0 h1 + h1 h0 (dropped: h1 h1 <= 2^-22 relative).  This is the accuracy class of
//     the reference's own fp32 route, 3xTF32 (src/elsa_twopass_clean/attention.py:280-282, 10 + 11 bits per operand),
//     at half its tensor-pipe cost: a tf32 instruction covers half the K extent of an fp16 one.
//   3 planes: x = b0 + b1 + b2 in bf16 (8 + 8 + 8 bits, no scaling needed), six cross terms of weight >= 2^-16
//     (dropped: <= 2^-24 relative).  Twice the instructions; 2-3 x closer to fp64 on the forward.
//
// A pre-pass (absmax_kernel + split_planes_kernel) writes the planes of q, k, v once per forward call.  One CTA (576
// threads, 1 per SM) owns ONE 128-row query tile of one (batch*head) and one K partition, walked in 128-key tiles:
//
//   warp 16     TMA producer   the planes of the Q tile once; then 16 KB plane tiles through an 8-slot ring in the
//                              order the issuer consumes them: K planes of key tile j+1, V planes of key tile j
//   warp 17     MMA issuer     S(j+1) = sum over the (q plane, k plane) pairs, 4 x tcgen05.mma 128x128x16 each,
//                              as soon as the fold warps hold S(j) in registers;
//                              O_j = sum over the (p plane, v plane) pairs, 8 x tcgen05.mma 128x64x16 each,
//                              into an accumulator that starts from zero for every key tile
//   warps 0-15  fold           FOUR threads per query row (warp w: rows 32 (w % 4) ..., key columns 32 (w / 4) ...):
//                              the thread's 32 scores go from TMEM into registers once, the row max is exchanged
//                              through shared memory, then exp2, row sum and -- after P V of the previous key tile
//                              has retired -- the split of P into its planes (own TMEM columns); the row's running
//                              output lives in registers (16 columns per thread) and takes in O_{j-1} with ordinary
//                              fp32 additions
//
// Scales.  The plane scales of q, k, v are powers of two, so they come out exactly: the scores arrive times s_q s_k
// (divided out together with the softmax scale), P is produced times 2^14 by adding 14 to the exponent of the
// exponential (so the row sum and the output carry 2^14, the output also s_v), and the epilogue takes all of it out.
// With fp16 planes a weight must not exceed 1, so the reference max follows every key tile (no lazy rescale).
//
// The per-element work of the fold is about a dozen instructions; with one thread per row (four warps, one per
// scheduler) every dependent instruction's latency was exposed and a key tile took 11.9 k cycles against 3.1 k of
// tensor-pipe work.  Four warps per scheduler hide it.
//
// Accuracy.  tcgen05.mma adds into its fp32 accumulator by truncation: every accumulating instruction loses up to one
// unit in the last place of the accumulator, always towards zero.  Accumulating P V of a whole partition in TMEM (as
// the 16-bit kernel does: invisible at 16-bit output precision) cost 1.6e-6 on an output of 0.1 after five key tiles,
// measured.  Therefore (a) every key tile gets a fresh accumulator and the running sum over key tiles is kept by the
// fold warps in registers, and (b) within a tile the cross terms are issued in order of increasing weight (the
// leading term x0*y0 last), so only its instructions work at full magnitude.
//
// TMEM columns: S [0,128) O [128,192) P planes [192 + 64 p, +64).
#include <algorithm>
#include <type_traits>

#include "kernels.cuh"
#include "tc_common.cuh"

namespace elsa {

using namespace tc;

namespace {

constexpr int kSlots = 8;
constexpr int kPlaneBytes = 128 * 64 * 2;                      // one 128 x 64 bf16 plane tile
constexpr int kFold3Smem = (kPlanes + kSlots) * kPlaneBytes + 1024;  // + alignment slack
constexpr int kFoldWarps = 16, kFoldThreads = kFoldWarps * 32;
constexpr int kThreads = kFoldThreads + 64;
constexpr uint32_t kTmemCols = 512;
constexpr int kProducerWarp = 16, kIssuerWarp = 17;
// lazy exp-rescale: with bf16 planes a weight may grow to 2^8 before the reference max moves; fp16 planes hold weights
// times 2^14, so there the reference max follows every tile (weights <= 1)
constexpr float kRescaleThreshold = kPlanes == 3 ? 8.0f : 0.0f;

enum BarId { BAR_Q = 31, BAR_FULL = 32, BAR_FREE = 33, BAR_S = 34, BAR_P = 35, BAR_O = 36, BAR_SFREE = 37, BAR_PV = 38, BAR_ROW = 39 };

struct Fold3Params {
  float* m; float* z; void* s;
  int n_ctx, q_start, q_len, part_width, n_parts, bh, is_causal, summary_dtype;
  int n_keys, key_offset, head_dim;
  float scale_log2;
  const uint32_t* amax_q; const uint32_t* amax_k; const uint32_t* amax_v;   // the plane headers
  const float* bias; int64_t bsb, bsh, bsq, bsk;   // additive bias [.., N, N] (natural-log units) or null
  int heads;
  int* status;
};

__device__ __forceinline__ float max3f(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}


// 16 consecutive values of a summary row, of which the first n (a multiple of 8) exist
template <typename TS>
__device__ __forceinline__ void store_row16(TS* dst, const float (&v)[16], int n) {
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

// ---- the plane pre-pass: up to four tensors per launch (blockIdx.z selects the tensor) ----
struct SplitJobs {
  const float* x[4]; Strides st[4]; uint32_t* header[4]; int rows[4];
};

// largest |x| of each [B, H, rows, cols] fp32 view: kAmaxBlocks blocks per tensor stride over its rows and write one
// partial maximum each into the tensor's plane header (bit patterns: non-negative floats order like integers); no
// atomics, nothing to zero beforehand
__global__ void __launch_bounds__(256)
absmax_kernel(const __grid_constant__ SplitJobs jobs, int heads, int bh, int cols) {
  __shared__ float wmax[8];
  const int job = blockIdx.z;
  const float* x = jobs.x[job];
  const Strides st = jobs.st[job];
  const int rows = jobs.rows[job];
  const int c = static_cast<int>(threadIdx.x & 15) * 4;          // 16 threads per row of 64
  float m = 0.f;
  if (c < cols) {
    const int64_t total = static_cast<int64_t>(bh) * rows;
    for (int64_t fr = blockIdx.x * 16 + static_cast<int>(threadIdx.x >> 4); fr < total; fr += gridDim.x * 16) {
      const int g = static_cast<int>(fr / rows), r = static_cast<int>(fr - static_cast<int64_t>(g) * rows);
      const int b = g / heads, h = g - b * heads;
      const float4 v = *reinterpret_cast<const float4*>(x + b * st.b + h * st.h + static_cast<int64_t>(r) * st.r + c);
      m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, wmax[w]);
    jobs.header[job][blockIdx.x] = (m > 0.f && m <= 3.0e38f) ? __float_as_uint(m) : 0u;
  }
}

// x (4 consecutive fp32 of a row of `cols` values, any strides) times the tensor's plane scale -> kPlanes 16-bit
// planes [kPlanes][B*H][rows][64] behind the header, contiguous; columns beyond `cols` are written as zeros (a head dim
// below 64 becomes a zero-padded 64-column operand).  The tensor's largest magnitude is the maximum of the partial
// maxima in its header; block (0, 0) also leaves it in header[kAmaxFinal] for the kernels that undo the scale.
__global__ void __launch_bounds__(256)
split_planes_kernel(const __grid_constant__ SplitJobs jobs, int heads, int bh, int cols) {
  __shared__ uint32_t amax_s;
  const int job = blockIdx.z;
  const int rows = jobs.rows[job];
  uint32_t* header = jobs.header[job];
  if (kPlanes == 2) {
    if (threadIdx.x < 32) {
      uint32_t m = max(header[threadIdx.x], header[threadIdx.x + 32]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
      if (threadIdx.x == 0) {
        amax_s = m;
        if (blockIdx.x == 0 && blockIdx.y == 0) header[kAmaxFinal] = m;
      }
    }
    __syncthreads();
  } else if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) {
    header[kAmaxFinal] = 0u;
  }
  const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;    // 16 threads per row of 64
  const int r = static_cast<int>(idx >> 4), c = static_cast<int>(idx & 15) * 4;
  if (r >= rows) return;
  const int g = blockIdx.y, b = g / heads, h = g - b * heads;
  const Strides st = jobs.st[job];
  const float sc = kPlanes == 2 ? plane_scale(amax_s) : 1.f;
  const float4 v = c < cols ? *reinterpret_cast<const float4*>(jobs.x[job] + b * st.b + h * st.h + static_cast<int64_t>(r) * st.r + c)
                            : make_float4(0.f, 0.f, 0.f, 0.f);
  uint32_t w0[kPlanes], w1[kPlanes];
  split_planes_pair(v.x * sc, v.y * sc, w0);
  split_planes_pair(v.z * sc, v.w * sc, w1);
  uint16_t* planes = reinterpret_cast<uint16_t*>(reinterpret_cast<char*>(header) + kPlaneHeader);
  const int64_t plane_elems = static_cast<int64_t>(bh) * rows * 64;
  const int64_t off = (static_cast<int64_t>(g) * rows + r) * 64 + c;
#pragma unroll
  for (int p = 0; p < kPlanes; ++p) *reinterpret_cast<uint2*>(planes + p * plane_elems + off) = make_uint2(w0[p], w1[p]);
}

template <bool BIAS>
__global__ void __launch_bounds__(kThreads, 1)
fold_tc3_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const Fold3Params prm) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kSlots + 9];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float row_max[2][4][128];   // [key-tile parity][column quarter][row]: the quarter-row maxima
  __shared__ float row_sum[4][128];      // the quarter-row sums, exchanged once in the epilogue

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.z, part = blockIdx.y;
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
  auto sQ = [&](int p) { return smem_base + p * kPlaneBytes; };
  auto sSlot = [&](int i) { return smem_base + (kPlanes + i) * kPlaneBytes; };
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_q = bar0;
  auto bar_full = [&](int i) { return bar0 + 8 * (1 + i); };
  auto bar_free = [&](int i) { return bar0 + 8 * (1 + kSlots + i); };
  const uint32_t bar_s = bar0 + 8 * (1 + 2 * kSlots);        // S(j) is in TMEM
  const uint32_t bar_sfree = bar0 + 8 * (2 + 2 * kSlots);    // the fold warps hold S(j) in registers
  const uint32_t bar_p = bar0 + 8 * (3 + 2 * kSlots);        // the P planes of tile j have been delivered
  const uint32_t bar_pv = bar0 + 8 * (4 + 2 * kSlots);       // O_j is complete
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
  const uint32_t tO = tmem_base + 128;
  const uint32_t tP0 = tmem_base + 192;                  // P plane p at tP0 + 64 p

  if (warp == kProducerWarp) {
    if (n_t > 0 && lane == 0) {
      // ---------------- TMA producer ----------------
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      mbar_arrive_expect_tx(bar_q, kPlanes * kPlaneBytes);
      for (int p = 0; p < kPlanes; ++p) tma_load_4d(sQ(p), &tmap_q, bar_q, 0, q0, bh, p);
      int seq = 0;
      bool ok = true;
      auto load = [&](const CUtensorMap* map, int tile, int plane) {
        const int slot = seq % kSlots;
        if (seq >= kSlots && !mbar_wait(bar_free(slot), ((seq / kSlots) - 1) & 1, &abort_flag, prm.status, BAR_FREE)) { ok = false; return; }
        mbar_arrive_expect_tx(bar_full(slot), kPlaneBytes);
        tma_load_4d(sSlot(slot), map, bar_full(slot), 0, k_begin + tile * 128, bh, plane);
        ++seq;
      };
      for (int p = kPlanes - 1; p >= 0 && ok; --p) load(&tmap_k, 0, p);       // planes in the order of increasing weight
      for (int j = 0; j < n_t && ok; ++j) {
        if (j + 1 < n_t)
          for (int p = kPlanes - 1; p >= 0 && ok; --p) load(&tmap_k, j + 1, p);
        for (int p = kPlanes - 1; p >= 0 && ok; --p) load(&tmap_v, j, p);
      }
    }
  } else if (warp == kIssuerWarp) {
    if (n_t > 0 && lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc_s = make_idesc(kPlaneFmt, 0, 0, 128, 128);   // S += Qp Kp^T : bf16, A, B K-major
      constexpr uint32_t idesc_o = make_idesc(kPlaneFmt, 0, 1, 128, 64);    // O += Pp Vp   : A in TMEM, B (V) MN-major
      uint64_t dq[kPlanes];
      for (int p = 0; p < kPlanes; ++p) dq[p] = make_sdesc(sQ(p), 16, 1024);
      const uint64_t dk_slot0 = make_sdesc(sSlot(0), 16, 1024), dv_slot0 = make_sdesc(sSlot(0), 128 * 128, 1024);
      constexpr uint64_t kSlotStep = kPlaneBytes >> 4;   // descriptor address field counts 16-byte units
      int seq = 0;
      bool ok = mbar_wait(bar_q, 0, &abort_flag, prm.status, BAR_Q);
      // the six (q plane, k plane) pairs of one key tile; K planes arrive in ring order 2, 1, 0 and within a plane
      // the q planes go from the lightest admissible one down to q0: the leading term q0 k0 is the last to be added
      auto issue_s = [&]() {
        bool first = true;
        for (int kp = kPlanes - 1; kp >= 0 && ok; --kp) {
          const int slot = seq % kSlots;
          if (!(ok = mbar_wait(bar_full(slot), (seq / kSlots) & 1, &abort_flag, prm.status, BAR_FULL))) return;
          tc_fence_after();
          const uint64_t dk = dk_slot0 + slot * kSlotStep;
          for (int qp = kPlanes - 1 - kp; qp >= 0; --qp) {
            mma_ss_x4<2, 2>(tS, dq[qp], dk, idesc_s, first ? 0u : 1u);
            first = false;
          }
          mma_commit(bar_free(slot));     // the plane tile is free again once these MMAs have retired
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
        // O_j starts from zero (the fold warps took O_{j-1} into their registers before they delivered P(j))
        bool first = true;
        for (int vp = kPlanes - 1; vp >= 0 && ok; --vp) {
          const int slot = seq % kSlots;
          if (!(ok = mbar_wait(bar_full(slot), (seq / kSlots) & 1, &abort_flag, prm.status, BAR_FULL))) break;
          tc_fence_after();
          const uint64_t dv = dv_slot0 + slot * kSlotStep;
          for (int pp = kPlanes - 1 - vp; pp >= 0; --pp) {
            mma_ts_x4<8, 128>(tO, tP0 + 64 * pp, dv, idesc_o, first ? 0u : 1u);
            mma_ts_x4<8, 128>(tO, tP0 + 64 * pp + 32, dv + 512, idesc_o, 1u);
            first = false;
          }
          mma_commit(bar_free(slot));
          ++seq;
        }
        if (ok) mma_commit(bar_pv);      // O_j is complete; the P planes may be overwritten
      }
    }
  } else {
    // ---------------- fold warps: four threads per query row ----------------
    const int qd = warp & 3, cq = warp >> 2;                // TMEM lane quadrant, column quarter
    const int row = qd * 32 + lane;                         // row within the tile == TMEM lane
    const int qi = q0 + row;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    // the scores arrive multiplied by the plane scales of q and k (powers of two): taken out with the softmax scale
    const float c = prm.scale_log2 / (plane_scale(*prm.amax_q) * plane_scale(*prm.amax_k));
    // with a bias the scores are moved to the log2 domain at once (s c + b log2 e) and the scale below becomes 1
    const float cc = BIAS ? 1.f : c;
    const float* bias_row = nullptr;
    if constexpr (BIAS) {
      const int bi = bh / prm.heads, hi = bh - bi * prm.heads;
      bias_row = prm.bias + bi * prm.bsb + hi * prm.bsh + static_cast<int64_t>(min(qi, prm.n_ctx - 1)) * prm.bsq;
    }
    float m_ref = -CUDART_INF_F, m_true = -CUDART_INF_F, zsum = 0.f;   // zsum: this thread's 32 columns only, times kPlaneUnit
    float o_run[16];                                        // running sum of O over the key tiles (columns 16 cq ...), relative to m_ref
#pragma unroll
    for (int i = 0; i < 16; ++i) o_run[i] = 0.f;
    bool alive = true;

    // o_run += O (the finished P V of one key tile)
    auto take_o = [&]() {
      uint32_t r[16];
      tmem_ld16(tO + lane_off + 16 * cq, r);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 16; ++i) o_run[i] += __uint_as_float(r[i]);
    };

    for (int j = 0; j < n_t; ++j) {
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
          // the thread's 128 bytes of the bias row as four whole sectors (a warp's 32 rows are 32 different lines)
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
        mx[0] = max3f(mx[0], sv[i], sv[i + 1]); mx[1] = max3f(mx[1], sv[i + 2], sv[i + 3]);
        mx[2] = max3f(mx[2], sv[i + 4], sv[i + 5]); mx[3] = max3f(mx[3], sv[i + 6], sv[i + 7]);
      }
      mx[0] = max3f(mx[0], sv[28], sv[29]); mx[1] = max3f(mx[1], sv[30], sv[31]);
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
      // ---- p = kPlaneUnit * 2^(s*c - m) in place of the scores (the unit rides in the exponent), and the quarter-row
      // sum (all of it overlaps P V of tile j-1) ----
      const float nm = kLog2Unit - m_use;
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        // ex2.approx: 2 units in the last place, i.e. 2.4e-7 relative on a weight
        sv[i] = fast_exp2(fmaf(sv[i], cc, nm));
        sv[i + 1] = fast_exp2(fmaf(sv[i + 1], cc, nm));
        ps[(i >> 1) & 3] += sv[i] + sv[i + 1];
      }
      zsum = zsum * alpha + ((ps[0] + ps[1]) + (ps[2] + ps[3]));
      if (j > 0) {
        // P V of the previous key tile has retired: its O goes into the running sum (both are relative to the m_ref
        // of that tile) before P V of this tile starts the accumulator from zero again; the P planes are free
        if (!__all_sync(0xffffffffu, mbar_wait(bar_pv, (j - 1) & 1, &abort_flag, prm.status, BAR_PV))) { alive = false; break; }
        tc_fence_after();
        take_o();
      }
      if (move) {
#pragma unroll
        for (int i = 0; i < 16; ++i) o_run[i] *= alpha;
      }
      // ---- the split of p into its planes, 16 keys (8 TMEM columns per plane) at a time ----
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t pk[kPlanes][8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint32_t w[kPlanes];
          split_planes_pair(sv[16 * ch + 2 * i], sv[16 * ch + 2 * i + 1], w);
#pragma unroll
          for (int p = 0; p < kPlanes; ++p) pk[p][i] = w[p];
        }
#pragma unroll
        for (int p = 0; p < kPlanes; ++p) tmem_st8(tP0 + 64 * p + lane_off + 16 * cq + 8 * ch, pk[p]);
      }
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
        // zsum carries kPlaneUnit, o_run kPlaneUnit and the plane scale of v (powers of two: taken out exactly)
        const float f = (m_true == -CUDART_INF_F) ? 0.f : exp2f(m_ref - m_true - kLog2Unit);
        const float fo = f / plane_scale(*prm.amax_v);
        z_out = ztot * f;
        m_out = z_out > 0.f ? m_true : -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < 16; ++i) o_run[i] = z_out > 0.f ? o_run[i] * fo : 0.f;
      }
    }
    if (row_ok && (alive || n_t == 0)) {
      if (cq == 0) {
        prm.m[ro] = m_out;
        prm.z[ro] = z_out;
      }
      if (prm.summary_dtype == ELSA_F32) store_row16<float>(static_cast<float*>(prm.s) + ro * prm.head_dim + 16 * cq, o_run, prm.head_dim - 16 * cq);
      else if (prm.summary_dtype == ELSA_F16) store_row16<__half>(static_cast<__half*>(prm.s) + ro * prm.head_dim + 16 * cq, o_run, prm.head_dim - 16 * cq);
      else store_row16<__nv_bfloat16>(static_cast<__nv_bfloat16*>(prm.s) + ro * prm.head_dim + 16 * cq, o_run, prm.head_dim - 16 * cq);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace

bool fold_tc3_supported(int dtype, int head_dim, bool has_bias) {
  (void)has_bias;   // the fold warps read an additive bias from global memory (BIAS variant of the kernel)
  return dtype == ELSA_F32 && head_dim >= 8 && head_dim <= 64 && head_dim % 8 == 0 && fold_tc_supported(ELSA_BF16, 64, false);
}

// a tensor's plane buffer: a header (kAmaxBlocks partial maxima and the final one) + [kPlanes][bh][rows][64] 16-bit
int64_t fold_tc3_plane_bytes(int bh, int rows) {
  return kPlaneHeader + align_up(static_cast<int64_t>(kPlanes) * bh * rows * 64 * 2, 256);
}

// the planes of up to four fp32 tensors ([B, H, rows[i], cols] views with strides st[i]) into planes[i]
// (fold_tc3_plane_bytes each): two launches for all of them
int fold_tc3_split_many(int n, const void* const* x, const Strides* st, void* const* planes, const int* rows, int batch,
                        int heads, int cols, cudaStream_t stream) {
  if (n < 1 || n > 4) return ELSA_ERR_INVALID_ARGUMENT;
  SplitJobs jobs;
  int n_jobs = 0, max_rows = 0;
  for (int i = 0; i < n; ++i) {
    if (rows[i] <= 0) continue;
    if ((st[i].b | st[i].h | st[i].r) % 4 != 0 || (reinterpret_cast<uintptr_t>(x[i]) & 15u)) return ELSA_ERR_INVALID_ARGUMENT;
    jobs.x[n_jobs] = static_cast<const float*>(x[i]); jobs.st[n_jobs] = st[i];
    jobs.header[n_jobs] = static_cast<uint32_t*>(planes[i]); jobs.rows[n_jobs] = rows[i];
    max_rows = std::max(max_rows, rows[i]);
    ++n_jobs;
  }
  if (n_jobs == 0) return ELSA_OK;
  for (int i = n_jobs; i < 4; ++i) { jobs.x[i] = jobs.x[0]; jobs.st[i] = jobs.st[0]; jobs.header[i] = jobs.header[0]; jobs.rows[i] = 0; }
  const int bh = batch * heads;
  if (kPlanes == 2) {
    absmax_kernel<<<dim3(kAmaxBlocks, 1, static_cast<unsigned>(n_jobs)), 256, 0, stream>>>(jobs, heads, bh, cols);
    ELSA_LAUNCH_CHECK();
  }
  const dim3 grid(static_cast<unsigned>(cdiv64(static_cast<int64_t>(max_rows) * 16, 256)), static_cast<unsigned>(bh),
                  static_cast<unsigned>(n_jobs));
  split_planes_kernel<<<grid, 256, 0, stream>>>(jobs, heads, bh, cols);
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

int fold_tc3_split(const void* x, Strides st, void* planes, int batch, int heads, int rows, int cols, cudaStream_t stream) {
  return fold_tc3_split_many(1, &x, &st, &planes, &rows, batch, heads, cols, stream);
}

// p.q3 / p.k3 / p.v3: the plane buffers written by fold_tc3_split for the whole problem (all query rows / this
// launch's key rows)
int fold_tc3(const FoldParams& p, cudaStream_t st) {
  if (!p.q3 || !p.k3 || !p.v3 || !fold_tc3_supported(ELSA_F32, p.head_dim, p.bias != nullptr) || p.part_width % 128 != 0)
    return ELSA_ERR_UNSUPPORTED;
  CUtensorMap mq, mk, mv;
  int rc;
  // planes as a [kPlanes, B*H, rows, 64] 16-bit tensor: the "head" coordinate is (batch*head), the "batch" coordinate the plane
  const Strides sq = contiguous_strides(p.bh, p.n_ctx, 64), sk = contiguous_strides(p.bh, p.n_keys, 64);
  if ((rc = make_tmap_rows64(&mq, static_cast<const char*>(p.q3) + kPlaneHeader, kPlaneDtype, p.n_ctx, p.bh, kPlanes, sq, 128)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mk, static_cast<const char*>(p.k3) + kPlaneHeader, kPlaneDtype, p.n_keys, p.bh, kPlanes, sk, 128)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mv, static_cast<const char*>(p.v3) + kPlaneHeader, kPlaneDtype, p.n_keys, p.bh, kPlanes, sk, 128)) != ELSA_OK) return rc;
  Fold3Params prm;
  prm.m = p.m; prm.z = p.z; prm.s = p.s;
  prm.amax_q = static_cast<const uint32_t*>(p.q3) + kAmaxFinal; prm.amax_k = static_cast<const uint32_t*>(p.k3) + kAmaxFinal;
  prm.amax_v = static_cast<const uint32_t*>(p.v3) + kAmaxFinal;
  if ((rc = device_status_word(&prm.status, nullptr)) != ELSA_OK) return rc;
  prm.n_ctx = p.n_ctx; prm.q_start = p.q_start; prm.q_len = p.q_len; prm.part_width = p.part_width;
  prm.n_parts = p.n_parts; prm.bh = p.bh; prm.is_causal = p.is_causal; prm.summary_dtype = p.summary_dtype;
  prm.n_keys = p.n_keys; prm.key_offset = p.key_offset; prm.head_dim = p.head_dim;
  prm.scale_log2 = p.scale_log2;
  prm.bias = p.bias; prm.bsb = p.bsb; prm.bsh = p.bsh; prm.bsq = p.bsq; prm.bsk = p.bsk; prm.heads = p.heads;
  rc = ensure_dynamic_smem(reinterpret_cast<const void*>(p.bias ? &fold_tc3_kernel<true> : &fold_tc3_kernel<false>), kFold3Smem);
  if (rc != ELSA_OK) return rc;
  dim3 grid(static_cast<unsigned>((p.q_len + 127) / 128), static_cast<unsigned>(p.n_parts), static_cast<unsigned>(p.bh));
  if (p.bias) fold_tc3_kernel<true><<<grid, kThreads, kFold3Smem, st>>>(mq, mk, mv, prm);
  else fold_tc3_kernel<false><<<grid, kThreads, kFold3Smem, st>>>(mq, mk, mv, prm);
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

}  // namespace elsa
