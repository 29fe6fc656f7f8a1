// Backward on the 5th-generation tensor cores: exact recompute from the saved row statistics,
// fp16 / bf16 inputs, head dim 64 (or a smaller multiple of 8, zero-padded to 64 columns by the TMA box), causal or
// not, no bias.  Five contractions per (key tile, query
// tile) pair -- the algorithmic minimum -- all as tcgen05.mma with TMEM accumulators:
//
//   S^T  = K Q^T          [128 keys x 128 queries]   TMEM (K) x smem (Q, K-major)          N = 128
//   dP^T = V dO^T         [128 x 128]                TMEM (V) x smem (dO, K-major)         N = 128
//   dV  += P^T dO         [128 keys x 64]            TMEM (P^T, in the dP^T columns)  x smem (dO, MN-major)
//   dK  += dS^T Q         [128 keys x 64]            TMEM (dS^T, in the dP^T columns) x smem (Q, MN-major)
//   dQ   = dS K           [128 queries x 64]         smem (dS^T, M-major A) x smem (K, MN-major)
//
// One CTA (1 per SM, 512 threads) owns one 128-key tile of one (batch*head) and streams the query
// tiles.  Working on the transposed score tile puts one KEY per TMEM lane, so P^T and dS^T come out
// in the layout the dV / dK contractions take as their TMEM A operand; dS^T also goes to shared
// memory (16-bit, 128-byte swizzle) where the dQ contraction reads it as an M-major A operand.
// dK and dV stay in TMEM for the whole CTA; dQ of each pair is added into an fp32 accumulator in
// global memory by a TMA reduce-add (cp.reduce.async.bulk.tensor) of the staged tile, and a last
// pass scales and rounds it.
//
// Pipeline.  A compute thread owns one key row and 64 of the 128 query columns and works in two phases:
//   A  load its S^T columns, release them (bar_lds), P^T = exp2(S^T c - LSE) kept in registers (fp32);
//   B  wait for dP^T, then per 32-query chunk: load dP^T, dS^T = P^T (dP^T - D), write the 16-bit P^T / dS^T
//      over the chunk's own dP^T columns (and dS^T to shared memory); every thread arrives once per tile on bar_pds.
// Because P^T no longer overlays S^T, the S^T columns are free as soon as phase A has loaded them: the issuer
// produces S^T of the NEXT query tile at the top of the iteration, so phase A of the next tile never waits
// and runs while the tensor pipe is busy with dV / dK / dP^T(next) / dQ of this one.  dP^T(next) follows the
// last dV / dK of this tile (same columns) and arrives during phase A.  The commit that announces dP^T(next)
// also tells the producer that dV / dK of this tile have retired, i.e. that its ring stage (Q, dO, -LSE, -D) may be
// refilled -- dQ reads only dS^T and K -- so the next-but-one tile's loads have a whole dQ + S^T of lead time.
//
//   warps 0-3   query columns 0-63  : one thread per key row (phases A and B above)
//   warps 4-7   query columns 64-127
//   warps 8-11  dQ drain: one thread per query row: TMEM -> registers -> swizzled smem -> TMA reduce-add
//   warp 12     TMA producer: K, V once; Q_i, dO_i, -LSE_i, -D_i into a 2-stage ring
//   warp 13     MMA issuer
//   (register budget re-balanced with setmaxnreg: 168 / 168 / 96 / 80 per thread = 4 x 128, the launch allocation)
//
// TMEM columns: S^T [0,128) dP^T [128,256) dV [256,320) dK [320,384) dQ [384,448) K [448,480) V [480,512).
// Within the 64 dP^T columns of a half, chunk ch keeps P^T in [32 ch, +16) and dS^T in [32 ch + 16, +16).
// K and V are copied once into TMEM (16-bit pairs, one key per lane) so that S^T and dP^T take their A operand
// from TMEM: the kernel is shared-memory-bandwidth sensitive and this removes 64 KB of operand reads per
// 128 x 128 pair.  (Measured alternatives at B=1 H=8 N=16384: P^T / dS^T as shared-memory A operands of dV / dK,
// 2.01 ms; two 64-query halves half an iteration apart with N = 64 S^T / dP^T, 1.80 ms; this design with a
// hand-off per 32-query chunk 1.64 ms, per half 1.59 ms.)
//
// -LSE and -D are read from a padded [BH][ceil(N/128)*128] layout whose padding holds -LSE = -inf,
// -D = 0, so that query rows beyond N produce P = 0 without a branch.
#include <type_traits>

#include "kernels.cuh"
#include "tc_common.cuh"

namespace elsa {

using namespace tc;

namespace {

constexpr int kQStages = 2;
constexpr int kPrefetchAhead = 3;   // query tiles between the ring's load and the L2 prefetch
constexpr int kTile = 128 * 64 * 2;     // 16 KB: one 128 x 64 16-bit tile
constexpr int kVecBytes = 128 * 4;      // 128 fp32 row statistics
// smem: K, V | ring of (Q, dO, -LSE, -D) | dS^T double buffer (each two 64-query blocks) | dQ staging (fp32, 2 x 16 KB)
constexpr int kStageBytes = 2 * kTile + 2 * kVecBytes;
constexpr int kBwdSmem = 2 * kTile + kQStages * kStageBytes + 4 * kTile + 2 * kTile + 1024;
constexpr int kThreads = 512;
constexpr uint32_t kTmemCols = 512;

enum BarId { BAR_KV = 11, BAR_Q_FULL = 12, BAR_Q_FREE = 13, BAR_SP = 14, BAR_PDS = 15, BAR_DQ_FULL = 16, BAR_DQ_FREE = 17, BAR_DONE = 18, BAR_KVT = 19, BAR_LDS = 20, BAR_DP = 21 };

struct BwdTcParams {
  const float* nlse_pad; const float* nd_pad;  // [BH][n_pad]: -LSE, -D
  float* dq_acc;                               // [BH][N][64] fp32, zeroed by the caller
  void* dk; void* dv;                          // T, rows addressed through dks / dvs
  Strides dks, dvs;
  int n_ctx, n_pad, bh, heads, is_causal;
  int n_keys, key_offset;                      // K/V rows of this launch and the sequence index of the first one
  int head_dim;                                // real columns of q, k, v, dout and the gradients (<= 64)
  float scale, scale_log2;
  int* status;   // the device's status word (mapped host memory)
};

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}


template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
bwd_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
              const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
              const __grid_constant__ CUtensorMap tmap_dq, const BwdTcParams prm) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kQStages + 13];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.y;
  const int bi = bh / prm.heads, hi = bh - bi * prm.heads;   // tensor-map coordinates of this (batch*head)
  const int k0 = blockIdx.x * 128;                  // first (local) key row of this CTA
  const int N = prm.n_ctx, NK = prm.n_keys;
  const int kseq0 = k0 + prm.key_offset;            // its index in the sequence
  const int n_qtiles = (N + 127) / 128;
  const int it_begin = prm.is_causal ? min(n_qtiles, kseq0 / 128) : 0;   // query tiles above the diagonal see none of these keys
  const int n_it = n_qtiles - it_begin;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = smem_base, sV = smem_base + kTile;
  auto sQ = [&](int st) { return smem_base + 2 * kTile + st * kStageBytes; };
  auto sDO = [&](int st) { return sQ(st) + kTile; };
  auto sNL = [&](int st) { return sQ(st) + 2 * kTile; };
  auto sND = [&](int st) { return sQ(st) + 2 * kTile + kVecBytes; };
  const uint32_t sDS0 = smem_base + 2 * kTile + kQStages * kStageBytes;   // buffer b at + b * 2 * kTile
  const uint32_t sDQ = sDS0 + 4 * kTile;                                   // dQ staging: two [128][32] fp32 blocks
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));         // generic pointer to smem_base

  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_kv = bar0;
  auto bar_q_full = [&](int st) { return bar0 + 8 * (1 + st); };
  auto bar_q_free = [&](int st) { return bar0 + 8 * (1 + kQStages + st); };
  const uint32_t barx = bar0 + 8 * (1 + 2 * kQStages);
  const uint32_t bar_s = barx;                             // S^T of the current query tile is in TMEM
  // bar_dpx(p): dP^T of a query tile of parity p is in TMEM -- and, the same arrival, dV / dK of the tile before it
  // have retired, so the ring stage of that tile (also parity-indexed) may be refilled
  auto bar_dpx = [&](int p) { return barx + 8 + 8 * 9 + 8 * p; };
  const uint32_t bar_pds = barx + 16;                      // P^T / dS^T of both halves are in TMEM / shared memory
  const uint32_t bar_dq_free = barx + 48, bar_done = barx + 56, bar_kvt = barx + 64;
  const uint32_t bar_lds = barx + 72;

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_kv, 1);
    for (int st = 0; st < kQStages; ++st) { mbar_init(bar_q_full(st), 1); mbar_init(bar_q_free(st), 1); }
    mbar_init(bar_s, 1); mbar_init(bar_dpx(0), 1); mbar_init(bar_dpx(1), 1); mbar_init(bar_lds, 256);
    mbar_init(bar_pds, 256);
    mbar_init(bar_dq_free, 128);
    mbar_init(bar_done, 1);
    mbar_init(bar_kvt, 256);
    fence_mbar_init();
  }
  if (warp == 12) {
    tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tdV = tmem_base + 256, tdK = tmem_base + 320, tdQ = tmem_base + 384;
  const uint32_t tK = tmem_base + 448, tV = tmem_base + 480;
  const uint32_t tS0 = tmem_base, tdP0 = tmem_base + 128;    // 128 query columns each
  auto tS = [&](int h) { return tmem_base + 64 * h; };
  auto tdP = [&](int h) { return tmem_base + 128 + 64 * h; };

  if (warp >= 12) {
    reg_dec<80>();
    if (warp == 12 && lane == 0) {
      // ---------------- TMA producer ----------------
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_do);
      mbar_arrive_expect_tx(bar_kv, 2 * kTile);
      tma_load_4d(sK, &tmap_k, bar_kv, 0, k0, hi, bi);
      tma_load_4d(sV, &tmap_v, bar_kv, 0, k0, hi, bi);
      for (int it = 0; it < n_it; ++it) {
        const int st = it % kQStages;
        // stage st held tile it-2: its dV / dK retired before the commit that announced dP^T of tile it-1
        if (it >= kQStages && !mbar_wait(bar_dpx((it - 1) & 1), ((it - 1) / 2) & 1, &abort_flag, prm.status, BAR_Q_FREE)) break;
        const int qrow = (it_begin + it) * 128;
        mbar_arrive_expect_tx(bar_q_full(st), kStageBytes);
        tma_load_4d(sQ(st), &tmap_q, bar_q_full(st), 0, qrow, hi, bi);
        tma_load_4d(sDO(st), &tmap_do, bar_q_full(st), 0, qrow, hi, bi);
        bulk_load_1d(sNL(st), prm.nlse_pad + static_cast<int64_t>(bh) * prm.n_pad + qrow, kVecBytes, bar_q_full(st));
        bulk_load_1d(sND(st), prm.nd_pad + static_cast<int64_t>(bh) * prm.n_pad + qrow, kVecBytes, bar_q_full(st));
        // the ring is only one tile ahead of the tensor pipe: pull the tiles after it into L2 now, so that a first
        // touch (inputs that are not L2-resident) costs an L2 hit instead of a DRAM round trip when its turn comes
        if (it + kPrefetchAhead < n_it) {
          tma_prefetch_l2_4d(&tmap_q, 0, qrow + kPrefetchAhead * 128, hi, bi);
          tma_prefetch_l2_4d(&tmap_do, 0, qrow + kPrefetchAhead * 128, hi, bi);
        }
      }
    } else if (warp == 13 && lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc_kv = make_idesc(fmt, 0, 1, 128, 64);   // dV, dK: A in TMEM, B MN-major
      constexpr uint32_t idesc_dq = make_idesc(fmt, 1, 1, 128, 64);   // dQ: A (dS^T) M-major, B (K) MN-major
      // Every shared-memory descriptor the loop needs, formed once: between two tcgen05.mma the issuing thread
      // should execute as little as possible (each instruction there is tensor-pipe idle time).
      const uint64_t bk_mn = make_sdesc(sK, 128 * 128, 1024);
      uint64_t dq_mn[2][2], ddo_mn[2][2], dds[2];
#pragma unroll
      for (int st = 0; st < 2; ++st) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          dq_mn[st][h] = make_sdesc(sQ(st) + h * 8192, 128 * 128, 1024);    // Q_h as MN-major B of dK
          ddo_mn[st][h] = make_sdesc(sDO(st) + h * 8192, 128 * 128, 1024);  // dO_h as MN-major B of dV
        }
        dds[st] = make_sdesc(sDS0 + st * 2 * kTile, 128 * 128, 1024);       // dS^T buffer as M-major A of dQ
      }
      static_assert(kQStages == 2, "the issuer loop is unrolled over the two ring stages");
      constexpr uint32_t idesc_st = make_idesc(fmt, 0, 0, 128, 128);  // S^T, dP^T: A (TMEM) and B K-major, N = 128 queries
      uint64_t dq_k[2], ddo_k[2];
#pragma unroll
      for (int st = 0; st < 2; ++st) {
        dq_k[st] = make_sdesc(sQ(st), 16, 1024);     // Q tile as K-major B of S^T
        ddo_k[st] = make_sdesc(sDO(st), 16, 1024);   // dO tile as K-major B of dP^T
      }
      using I0 = std::integral_constant<int, 0>;
      using I1 = std::integral_constant<int, 1>;
      // dV += P^T_h dO_h, dK += dS^T_h Q_h over the 64 queries of half h (four K-steps each); the 16-bit
      // P^T / dS^T of chunk ch sit in columns [32 ch, +16) / [32 ch + 16, +16) of the half's dP^T columns
      auto issue_dkv = [&](auto ST, auto H, uint32_t acc) {
        constexpr int st = decltype(ST)::value, h = decltype(H)::value;
        // K-steps of 16 queries: P^T at columns 0, 8 (chunk 0) and 32, 40 (chunk 1); dS^T 16 columns further
        mma_ts_x4_cols<8, 32, 40, 128>(tdV, tdP(h), ddo_mn[st][h], idesc_kv, acc);
        mma_ts_x4_cols<8, 32, 40, 128>(tdK, tdP(h) + 16, dq_mn[st][h], idesc_kv, acc);
      };
      bool ok = mbar_wait(bar_kv, 0, &abort_flag, prm.status, BAR_KV) &&
                mbar_wait(bar_kvt, 0, &abort_flag, prm.status, BAR_KVT) &&
                (n_it == 0 || mbar_wait(bar_q_full(0), 0, &abort_flag, prm.status, BAR_Q_FULL));
      if (ok && n_it > 0) {
        tc_fence_after();
        mma_ts_x4<8, 2>(tS0, tK, dq_k[0], idesc_st, 0u);
        mma_commit(bar_s);
        mma_ts_x4<8, 2>(tdP0, tV, ddo_k[0], idesc_st, 0u);
        mma_commit(bar_dpx(0));
      }
      // One iteration on ring stage ST (the next one is on the other stage).  S^T of the NEXT query tile is issued
      // as soon as the compute warps hold the current S^T in registers (their exp2 phase then overlaps the
      // contractions below); dP^T of the next tile follows dV / dK of this one, whose A operands live in the
      // dP^T columns; dQ comes last.  (dQ of the previous tile at the top of the iteration instead, so that only
      // dV / dK / dP^T stand between the halves' arrival and the next dS phase: measured 1.95 ms against 1.59 ms.)
      auto issue_dq = [&](int it_q, auto STQ) {       // dQ of tile it_q, whose dS^T sits in buffer STQ
        constexpr int stq = decltype(STQ)::value;
        if (it_q > 0 && !(ok = mbar_wait(bar_dq_free, (it_q - 1) & 1, &abort_flag, prm.status, BAR_DQ_FREE))) return;
        mma_ss_x4<128, 128>(tdQ, dds[stq], bk_mn, idesc_dq, 0u);
        mma_ss_x4<128, 128>(tdQ, dds[stq] + 512, bk_mn + 512, idesc_dq, 1u);
        mma_commit(bar_q_free(stq));   // dQ(it_q) is complete: the drain warps may read it
      };
      auto iteration = [&](int it, auto ST) {
        constexpr int st = decltype(ST)::value;
        const bool more = it + 1 < n_it;
        const uint32_t pit = it & 1;
        if (more) {
          ok = mbar_wait(bar_q_full(st ^ 1), ((it + 1) / kQStages) & 1, &abort_flag, prm.status, BAR_Q_FULL) &&
               mbar_wait(bar_lds, pit, &abort_flag, prm.status, BAR_LDS);
          if (!ok) return;
          tc_fence_after();
          mma_ts_x4<8, 2>(tS0, tK, dq_k[st ^ 1], idesc_st, 0u);
          mma_commit(bar_s);
        }
        if (!(ok = mbar_wait(bar_pds, pit, &abort_flag, prm.status, BAR_PDS))) return;
        tc_fence_after();
        issue_dkv(ST, I0{}, it == 0 ? 0u : 1u);
        issue_dkv(ST, I1{}, 1u);
        if (more) {
          // one commit for two facts: dP^T of the next tile is in TMEM, and dV / dK of this tile have retired, so
          // Q, dO and the row statistics of this tile are not read again (dQ takes dS^T and K) and the producer may
          // refill the ring stage
          mma_ts_x4<8, 2>(tdP0, tV, ddo_k[st ^ 1], idesc_st, 0u);
          mma_commit(bar_dpx(st ^ 1));
        }
        issue_dq(it, ST);
      };
      for (int it = 0; ok && it < n_it; it += 2) {
        iteration(it, I0{});
        if (ok && it + 1 < n_it) iteration(it + 1, I1{});
      }
      if (ok) mma_commit(bar_done);
    }
  } else if (warp >= 8) {
    // ---------------- dQ drain warps: one thread per query row ----------------
    reg_dec<96>();
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    for (int it = 0; it < n_it; ++it) {
      if (!__all_sync(0xffffffffu, mbar_wait(bar_q_free(it % kQStages), (it / kQStages) & 1, &abort_flag, prm.status, BAR_DQ_FULL))) break;
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld32(tdQ + lane_off, r0);
      tmem_ld32(tdQ + lane_off + 32, r1);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bar_dq_free);
      // Stage the 128 x 64 fp32 tile in shared memory (two 32-column blocks, 128-byte swizzle) and let the TMA
      // unit add it into the global accumulator: whole 128-byte lines per reduction instead of one 16-byte
      // piece per lane, and no LSU traffic that would delay the MMA issue slots of this scheduler.
      if (tid == 256) bulk_wait_group_read<0>();          // the previous tile has been read out of the staging buffer
      named_barrier_sync(1, 128);
      {
        uint8_t* stg = smem_gen + (sDQ - smem_base) + row * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          *reinterpret_cast<uint4*>(stg + ((c ^ (row & 7)) << 4)) = make_uint4(r0[4 * c], r0[4 * c + 1], r0[4 * c + 2], r0[4 * c + 3]);
          *reinterpret_cast<uint4*>(stg + kTile + ((c ^ (row & 7)) << 4)) = make_uint4(r1[4 * c], r1[4 * c + 1], r1[4 * c + 2], r1[4 * c + 3]);
        }
      }
      fence_proxy_async_smem();
      named_barrier_sync(1, 128);
      if (tid == 256) {
        const int qrow0 = (it_begin + it) * 128;
        tma_reduce_add_3d(&tmap_dq, sDQ, 0, qrow0, bh);           // rows beyond N are clipped by the tensor map
        tma_reduce_add_3d(&tmap_dq, sDQ + kTile, 32, qrow0, bh);
        bulk_commit_group();
      }
    }
    if (tid == 256) bulk_wait_group<0>();                 // reductions must have left shared memory before the CTA exits
  } else {
    // ---------------- compute warps: thread = (key row, query half) ----------------
    reg_inc<168>();
    const int half = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int key = k0 + row;                  // local key row
    const int key_seq = kseq0 + row;           // its index in the sequence (what the causal rule compares)
    const bool key_ok = key < NK;
    const bool cta_tail = k0 + 128 > NK;       // some key rows of this CTA do not exist
    const float2 c2 = make_float2(prm.scale_log2, prm.scale_log2);
    bool alive = true;

    // one-time copy of this CTA's K (warps 0-3) / V (warps 4-7) tile from shared memory into TMEM as the A operand
    // of S^T / dP^T: lane = key row, 32 columns of 16-bit pairs; the smem row is un-swizzled on the way
    if (!__all_sync(0xffffffffu, mbar_wait(bar_kv, 0, &abort_flag, prm.status, BAR_KV))) alive = false;
    if (alive) {
      const uint8_t* src = smem_gen + ((half == 0 ? sK : sV) - smem_base) + row * 128;
      uint32_t w[32];
#pragma unroll
      for (int cgrp = 0; cgrp < 8; ++cgrp) {
        const uint4 t = *reinterpret_cast<const uint4*>(src + ((cgrp ^ (row & 7)) << 4));
        w[4 * cgrp] = t.x; w[4 * cgrp + 1] = t.y; w[4 * cgrp + 2] = t.z; w[4 * cgrp + 3] = t.w;
      }
      tmem_st32((half == 0 ? tK : tV) + lane_off, w);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_kvt);
    }

    for (int it = 0; alive && it < n_it; ++it) {
      const int st = it % kQStages;
      const int q_tile0 = (it_begin + it) * 128;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_s, it & 1, &abort_flag, prm.status, BAR_SP))) { alive = false; break; }
      // the row statistics of this stage were written by the bulk copies that complete on q_full: observe that
      // barrier directly (it completed before the MMAs behind bar_s were issued, so this never spins)
      if (!__all_sync(0xffffffffu, mbar_wait(bar_q_full(st), (it / kQStages) & 1, &abort_flag, prm.status, BAR_Q_FULL))) { alive = false; break; }
      tc_fence_after();
      const float4* nl4 =reinterpret_cast<const float4*>(smem_gen + (sNL(st) - smem_base)) + half * 16;
      const float4* nd4 = reinterpret_cast<const float4*>(smem_gen + (sND(st) - smem_base)) + half * 16;
      const bool masked = cta_tail || (prm.is_causal && q_tile0 < kseq0 + 128);   // only the diagonal tile(s) / the last key tile
      uint8_t* ds_row = smem_gen + (sDS0 - smem_base) + (it & 1) * 2 * kTile + half * kTile + row * 128;

      // ---- phase A: P^T = exp2(S^T * c - LSE) for this thread's 64 queries, kept in registers as fp32 ----
      float p[64];
      {
        uint32_t r0[32], r1[32];
        tmem_ld32(tS(half) + lane_off, r0);
        tmem_ld32(tS(half) + lane_off + 32, r1);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(bar_lds);       // the S^T columns may be overwritten with the next query tile's scores
#pragma unroll
        for (int i = 0; i < 32; ++i) { p[i] = __uint_as_float(r0[i]); p[32 + i] = __uint_as_float(r1[i]); }
      }
#pragma unroll
      for (int g = 0; g < 16; ++g) {
        const float4 nl = nl4[g];                                   // -LSE of 4 queries (warp-wide broadcast read)
        const float2 x0 = __ffma2_rn(make_float2(p[4 * g], p[4 * g + 1]), c2, make_float2(nl.x, nl.y));
        const float2 x1 = __ffma2_rn(make_float2(p[4 * g + 2], p[4 * g + 3]), c2, make_float2(nl.z, nl.w));
        p[4 * g] = fast_exp2(x0.x); p[4 * g + 1] = fast_exp2(x0.y);
        p[4 * g + 2] = fast_exp2(x1.x); p[4 * g + 3] = fast_exp2(x1.y);
        if (masked) {
          const int qc = q_tile0 + half * 64 + 4 * g;               // first query of this group of 4
          const bool causal = prm.is_causal;
#pragma unroll
          for (int e = 0; e < 4; ++e)
            p[4 * g + e] = (key_ok && (!causal || qc + e >= key_seq)) ? p[4 * g + e] : 0.f;
        }
      }

      // ---- phase B: dS^T = P^T * (dP^T - D); P^T and dS^T (16-bit) handed to dV / dK in two 32-query chunks ----
      if (!__all_sync(0xffffffffu, mbar_wait(bar_dpx(it & 1), (it / 2) & 1, &abort_flag, prm.status, BAR_DP))) { alive = false; break; }
      tc_fence_after();
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t rp[32];
        tmem_ld32(tdP(half) + lane_off + 32 * ch, rp);
        tmem_wait_ld();
        uint32_t pk[16], dsk[16];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 nd = nd4[ch * 8 + g];                        // -D of 4 queries
          const float2 p0 = make_float2(p[32 * ch + 4 * g], p[32 * ch + 4 * g + 1]);
          const float2 p1 = make_float2(p[32 * ch + 4 * g + 2], p[32 * ch + 4 * g + 3]);
          const float2 t0 = __fadd2_rn(make_float2(__uint_as_float(rp[4 * g]), __uint_as_float(rp[4 * g + 1])), make_float2(nd.x, nd.y));
          const float2 t1 = __fadd2_rn(make_float2(__uint_as_float(rp[4 * g + 2]), __uint_as_float(rp[4 * g + 3])), make_float2(nd.z, nd.w));
          const float2 d0 = __fmul2_rn(p0, t0), d1 = __fmul2_rn(p1, t1);
          pk[2 * g] = pack2<T>(p0.x, p0.y);
          pk[2 * g + 1] = pack2<T>(p1.x, p1.y);
          dsk[2 * g] = pack2<T>(d0.x, d0.y);
          dsk[2 * g + 1] = pack2<T>(d1.x, d1.y);
        }
        // the 32 dP^T columns of this chunk are in registers: P^T goes over their first 16, dS^T over the other 16
        tmem_st16(tdP(half) + lane_off + 32 * ch, pk);
        tmem_st16(tdP(half) + lane_off + 32 * ch + 16, dsk);
        // dS^T to shared memory for dQ: block `half`, row = key, 16-byte piece (8 queries) index XOR (key & 7)
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = ch * 4 + g;
          *reinterpret_cast<uint4*>(ds_row + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(dsk[4 * g], dsk[4 * g + 1], dsk[4 * g + 2], dsk[4 * g + 3]);
        }
      }
      // hand the half to the MMA issuer: one wait for all four TMEM stores, one fence, one arrival (dP^T of the
      // next tile is only needed after the next exp2 phase, so dV / dK need not start on the first chunk)
      fence_proxy_async_smem();
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_pds);
    }

    // ---- epilogue: dK, dV of this key tile (tcgen05.ld is warp-collective: only the stores are predicated) ----
    if (alive && n_it > 0 && !__all_sync(0xffffffffu, mbar_wait(bar_done, 0, &abort_flag, prm.status, BAR_DONE))) alive = false;
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
        T* dk_row = static_cast<T*>(prm.dk) + bi * prm.dks.b + hi * prm.dks.h + key * prm.dks.r + half * 32;
        T* dv_row = static_cast<T*>(prm.dv) + bi * prm.dvs.b + hi * prm.dvs.h + key * prm.dvs.r + half * 32;
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          if (half * 32 + i >= prm.head_dim) continue;
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
  if (warp == 12) tmem_dealloc(tmem_base, kTmemCols);
}

// -D = -sum_d out*dout, -LSE = -(m + log2(max(z, 1e-30))) into the padded layout; padding: -D = 0, -LSE = -inf
template <typename T>
__global__ void __launch_bounds__(256)
bwd_preprocess_pad_kernel(const T* __restrict__ out, const T* __restrict__ dout, const float* __restrict__ row_m,
                          const float* __restrict__ row_z, float* __restrict__ nd_pad, float* __restrict__ nlse_pad,
                          int heads, int n_ctx, int n_pad, int head_dim, Strides os, Strides gs) {
  // blockIdx.y = (batch*head); x covers the n_pad padded rows, 8 lanes (16 bytes each) per row: no division
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = static_cast<int>(gid >> 3);        // padded row within this (batch*head)
  const int lane = static_cast<int>(gid & 7);
  const int64_t b = blockIdx.y;
  const int64_t prow = b * n_pad + r;
  const bool in_pad = r < n_pad;
  const bool real = in_pad && r < n_ctx;
  float part = 0.f;
  if (real && lane * 8 < head_dim) {
    const int bi = static_cast<int>(b) / heads, hi = static_cast<int>(b) - bi * heads;
    const T* o = out + bi * os.b + hi * os.h + static_cast<int64_t>(r) * os.r + lane * 8;
    const T* g = dout + bi * gs.b + hi * gs.h + static_cast<int64_t>(r) * gs.r + lane * 8;
    uint4 ov = *reinterpret_cast<const uint4*>(o), gv = *reinterpret_cast<const uint4*>(g);
    const T* oe = reinterpret_cast<const T*>(&ov);
    const T* ge = reinterpret_cast<const T*>(&gv);
#pragma unroll
    for (int i = 0; i < 8; ++i) part += to_f32<T>(oe[i]) * to_f32<T>(ge[i]);
  }
  part += __shfl_xor_sync(0xffffffffu, part, 4);
  part += __shfl_xor_sync(0xffffffffu, part, 2);
  part += __shfl_xor_sync(0xffffffffu, part, 1);
  if (in_pad && lane == 0) {
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

// acc *= scale (the fp32 dQ of a sequence shard stays fp32: the caller sums the shards before rounding)
__global__ void __launch_bounds__(256) dq_scale_kernel(float* __restrict__ acc, int64_t n_vec4, float scale) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec4) return;
  float4 a = *reinterpret_cast<float4*>(acc + i * 4);
  a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
  *reinterpret_cast<float4*>(acc + i * 4) = a;
}

// dq = T(acc * scale); acc is [BH][N][64] fp32, dq rows are addressed through their strides (blockIdx.y = batch*head)
template <typename T>
__global__ void __launch_bounds__(256)
dq_convert_kernel(const float* __restrict__ acc, T* __restrict__ dq, int n_ctx, int heads, int head_dim, Strides ds, float scale) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;        // 8 elements each: row = i / 8
  const int r = static_cast<int>(i >> 3), c = static_cast<int>(i & 7) * 8;
  if (r >= n_ctx || c >= head_dim) return;
  const int bh = blockIdx.y, bi = bh / heads, hi = bh - bi * heads;
  const float* src = acc + (static_cast<int64_t>(bh) * n_ctx + r) * 64 + c;
  const float4 a = *reinterpret_cast<const float4*>(src);
  const float4 b = *reinterpret_cast<const float4*>(src + 4);
  uint4 o;
  o.x = pack2<T>(a.x * scale, a.y * scale); o.y = pack2<T>(a.z * scale, a.w * scale);
  o.z = pack2<T>(b.x * scale, b.y * scale); o.w = pack2<T>(b.z * scale, b.w * scale);
  *reinterpret_cast<uint4*>(dq + bi * ds.b + hi * ds.h + static_cast<int64_t>(r) * ds.r + c) = o;
}

}  // namespace

bool bwd_tc_supported(int dtype, int head_dim, bool has_bias) { return fold_tc_supported(dtype, head_dim, has_bias); }

int64_t bwd_tc_workspace_bytes(int bh, int n_ctx) {
  const int64_t n_pad = align_up(n_ctx, 128);
  return 2 * align_up(static_cast<int64_t>(bh) * n_pad * 4, 256) + align_up(static_cast<int64_t>(bh) * n_ctx * 64 * 4, 256);
}

template <typename T>
static int bwd_tc_t(const BwdParams& p, const void* out, Strides os, const float* row_m, const float* row_z,
                    void* workspace, int dtype, cudaStream_t st) {
  const int N = p.n_ctx, NK = p.n_keys, bh = p.bh;
  const int n_pad = static_cast<int>(align_up(N, 128));
  const int64_t vec_bytes = align_up(static_cast<int64_t>(bh) * n_pad * 4, 256);
  char* ws = static_cast<char*>(workspace);
  float* nd_pad = reinterpret_cast<float*>(ws);
  float* nlse_pad = reinterpret_cast<float*>(ws + vec_bytes);
  // the fp32 accumulator the TMA reductions add into: the caller's fp32 dQ for a sequence shard, else workspace
  float* dq_acc = p.dq_f32 ? static_cast<float*>(p.dq) : reinterpret_cast<float*>(ws + 2 * vec_bytes);
  const int64_t acc_elems = static_cast<int64_t>(bh) * N * 64;

  {
    const dim3 pgrid(static_cast<unsigned>(cdiv64(static_cast<int64_t>(n_pad) * 8, 256)), static_cast<unsigned>(bh));
    bwd_preprocess_pad_kernel<T><<<pgrid, 256, 0, st>>>(
        static_cast<const T*>(out), static_cast<const T*>(p.dout), row_m, row_z, nd_pad, nlse_pad, p.heads, N, n_pad, p.head_dim, os, p.gs);
    ELSA_LAUNCH_CHECK();
  }
  ELSA_CUDA_CHECK(cudaMemsetAsync(dq_acc, 0, acc_elems * 4, st));

  CUtensorMap mq, mk, mv, mdo, mdq;
  int rc;
  if ((rc = make_tmap_f32_rows64(&mdq, dq_acc, N, bh, 128)) != ELSA_OK) return rc;
  const int batch = bh / p.heads;
  if ((rc = make_tmap_rows64(&mq, p.q, dtype, N, p.heads, batch, p.qs, 128, p.head_dim)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mk, p.k, dtype, NK, p.heads, batch, p.ks, 128, p.head_dim)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mv, p.v, dtype, NK, p.heads, batch, p.vs, 128, p.head_dim)) != ELSA_OK) return rc;
  if ((rc = make_tmap_rows64(&mdo, p.dout, dtype, N, p.heads, batch, p.gs, 128, p.head_dim)) != ELSA_OK) return rc;
  BwdTcParams prm;
  if ((rc = device_status_word(&prm.status, nullptr)) != ELSA_OK) return rc;
  prm.nlse_pad = nlse_pad; prm.nd_pad = nd_pad; prm.dq_acc = dq_acc; prm.dk = p.dk; prm.dv = p.dv;
  prm.n_ctx = N; prm.n_pad = n_pad; prm.bh = bh; prm.heads = p.heads; prm.is_causal = p.is_causal;
  prm.dks = p.dks; prm.dvs = p.dvs;
  prm.n_keys = NK; prm.key_offset = p.key_offset; prm.head_dim = p.head_dim;
  prm.scale = p.scale; prm.scale_log2 = p.scale_log2;
  rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&bwd_tc_kernel<T>), kBwdSmem);
  if (rc != ELSA_OK) return rc;
  if (NK > 0) {
    dim3 grid(static_cast<unsigned>((NK + 127) / 128), static_cast<unsigned>(bh));
    bwd_tc_kernel<T><<<grid, kThreads, kBwdSmem, st>>>(mq, mk, mv, mdo, mdq, prm);
    ELSA_LAUNCH_CHECK();
  }
  if (p.dq_f32) {
    dq_scale_kernel<<<static_cast<unsigned>(cdiv64(acc_elems / 4, 256)), 256, 0, st>>>(dq_acc, acc_elems / 4, p.scale);
  } else {
    const dim3 cgrid(static_cast<unsigned>(cdiv64(static_cast<int64_t>(N) * 8, 256)), static_cast<unsigned>(bh));
    dq_convert_kernel<T><<<cgrid, 256, 0, st>>>(dq_acc, static_cast<T*>(p.dq), N, p.heads, p.head_dim, p.dqs, p.scale);
  }
  ELSA_LAUNCH_CHECK();
  return ELSA_OK;
}

int bwd_tc(const BwdParams& p, const void* out, Strides os, const float* row_m, const float* row_z, void* workspace,
           int dtype, cudaStream_t st) {
  if (!bwd_tc_supported(dtype, p.head_dim, p.bias != nullptr) || p.dbias) return ELSA_ERR_UNSUPPORTED;
  if (p.dq_f32 && p.head_dim != 64) return ELSA_ERR_UNSUPPORTED;   // the caller's fp32 dQ is the accumulator: 64-wide rows
  if (dtype == ELSA_F16) return bwd_tc_t<__half>(p, out, os, row_m, row_z, workspace, dtype, st);
  return bwd_tc_t<__nv_bfloat16>(p, out, os, row_m, row_z, workspace, dtype, st);
}


}  // namespace elsa
