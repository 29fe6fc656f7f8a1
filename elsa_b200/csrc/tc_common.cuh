// sm_100a building blocks for the tensor-core kernels: mbarrier, TMA (cp.async.bulk.tensor),
// tcgen05 (TMEM allocation, MMA issue, commit, TMEM load/store) and the shared-memory / instruction
// descriptors, all as inline PTX.  No cluster launch and no multicast anywhere: every CTA loads
// its own tiles.
//
// Every wait on an mbarrier is bounded: after kWaitLimitNs it records an error in the device
// status word, raises the CTA's abort flag and returns false; callers then fall through to the
// common exit path (TMEM is released, the kernel returns, the host sees the status).
#pragma once

#include "common.cuh"

namespace elsa {
namespace tc {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

// device status word (one per device, in mapped pinned host memory, passed to the waits by pointer):
// 0 = ok, otherwise (1 << 8) | id of the barrier whose wait gave up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// one arrival for the whole warp: every lane's earlier operations (completed TMEM loads / stores, shared-memory
// writes) are ordered before it by the warp barrier, so a barrier that 16 warps feed counts 16 arrivals instead of 512
__device__ __forceinline__ void mbar_arrive_warp(uint32_t bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait; `abort_flag` lives in shared memory and is raised by whoever times out first.  `status` points at
// the device's status word, which lives in mapped pinned HOST memory (the host reads it without a copy or a
// synchronisation): a plain store followed by a system-scope fence, no atomics across the host link.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int bar_id, unsigned long long limit_ns = kWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        if (status) {
          *reinterpret_cast<volatile int*>(status) = (1 << 8) | bar_id;
          __threadfence_system();
        }
        return false;
      }
    }
  }
}

// ---- TMA ------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 4-D tiled load global -> shared, completion counted in bytes on `bar`.  Coordinates, innermost first:
// x = element within the row (must make x*elem_size a multiple of 16 bytes; always 0 here), row, head, batch.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int row, int h, int b) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(row), "r"(h), "r"(b)
      : "memory");
}
// the cache line at p into L2 (a hint: no register, nothing to wait for)
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
// 4-D tiled prefetch global -> L2 (no shared-memory destination, no completion to wait for)
__device__ __forceinline__ void tma_prefetch_l2_4d(const CUtensorMap* m, int x, int row, int h, int b) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(row), "r"(h), "r"(b) : "memory");
}
// 3-D tiled reduction shared -> global: global[tile] += smem tile (element type and add come from the tensor
// map / the .add qualifier); tracked by the thread's bulk async-group.  Coordinates out of range are skipped.
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, uint32_t src, int x, int y, int z) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the newest `N` groups of this thread have finished READING their shared-memory source
template <int N> __device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// arrive without waiting: the writes made before it are visible to the threads that `named_barrier_sync` on the same id
__device__ __forceinline__ void named_barrier_arrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// register re-balancing between warpgroups (every warp of the 128-thread warpgroup must execute it)
template <int N> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }

// ---- tcgen05 ----------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; M = 128, K = 16 per instruction, kind::f16 (fp16 or bf16 inputs, fp32 accumulate)
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Four consecutive K-steps in ONE asm block.  The issuing thread is blocked by each tcgen05.mma until the pipe
// accepts it, so every instruction executed between two MMAs is tensor-pipe idle time; here the operand
// addresses of all four steps are formed first and the four MMAs follow back to back.
// A_STEP: TMEM columns (TS form) or descriptor units of 16 bytes (SS form) per K-step; B_STEP: descriptor units.
template <int A_STEP, int B_STEP>
__device__ __forceinline__ void mma_ts_x4(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t first_accumulate) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t.reg .b64 b1, b2, b3;\n\t.reg .b32 a1, a2, a3;\n\t"
      "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
      "add.u32 a1, %1, %5;\n\tadd.u32 a2, %1, %6;\n\tadd.u32 a3, %1, %7;\n\t"
      "add.u64 b1, %2, %8;\n\tadd.u64 b2, %2, %9;\n\tadd.u64 b3, %2, %10;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %3, p1;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(first_accumulate), "n"(A_STEP), "n"(2 * A_STEP),
        "n"(3 * A_STEP), "n"(B_STEP), "n"(2 * B_STEP), "n"(3 * B_STEP)
      : "memory");
}
// four MMAs whose TMEM A slices sit at arbitrary column offsets A1..A3 from the first (B advances uniformly)
template <int A1, int A2, int A3, int B_STEP>
__device__ __forceinline__ void mma_ts_x4_cols(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t first_accumulate) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t.reg .b64 b1, b2, b3;\n\t.reg .b32 a1, a2, a3;\n\t"
      "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
      "add.u32 a1, %1, %5;\n\tadd.u32 a2, %1, %6;\n\tadd.u32 a3, %1, %7;\n\t"
      "add.u64 b1, %2, %8;\n\tadd.u64 b2, %2, %9;\n\tadd.u64 b3, %2, %10;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %3, p1;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(first_accumulate), "n"(A1), "n"(A2), "n"(A3),
        "n"(B_STEP), "n"(2 * B_STEP), "n"(3 * B_STEP)
      : "memory");
}
template <int A_STEP, int B_STEP>
__device__ __forceinline__ void mma_ss_x4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t first_accumulate) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
      "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
      "add.u64 a1, %1, %5;\n\tadd.u64 a2, %1, %6;\n\tadd.u64 a3, %1, %7;\n\t"
      "add.u64 b1, %2, %8;\n\tadd.u64 b2, %2, %9;\n\tadd.u64 b3, %2, %10;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, p1;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(first_accumulate), "n"(A_STEP), "n"(2 * A_STEP),
        "n"(3 * A_STEP), "n"(B_STEP), "n"(2 * B_STEP), "n"(3 * B_STEP)
      : "memory");
}
// the mbarrier receives one arrival when every tcgen05 operation issued so far by this thread is complete
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// shared-memory operand descriptor, 128-byte swizzle (what TMA SWIZZLE_128B writes; tile base 1024-byte aligned):
//   bits [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte offset >> 4,
//   bit 46 descriptor version (1 on sm_100), bits [61,64) layout type (2 = SWIZZLE_128B).
// K-major operand (rows of 64 16-bit elements, K contiguous): SBO = 1024 (8 rows x 128 B), LBO unused.
//   advancing K by 16 elements = +32 bytes on the start address.
// MN-major operand (rows are K, the 64 contiguous elements are M or N): SBO = 1024 between groups of 8 K-rows,
//   LBO = distance between 64-element column blocks; advancing K by 16 rows = +2048 bytes.
__device__ __forceinline__ uint64_t make_sdesc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// instruction descriptor for kind::f16: fp32 accumulate, A/B format (0 = fp16, 1 = bf16), operand majors, N, M
__host__ __device__ constexpr uint32_t make_idesc(uint32_t ab_format, uint32_t a_mn_major, uint32_t b_mn_major, uint32_t m, uint32_t n) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

// TMEM <-> registers: the warp's 32 lanes (32*(warp%4) ...) x 32 consecutive 32-bit columns; thread i gets lane i
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&w)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]), "r"(w[8]),
        "r"(w[9]), "r"(w[10]), "r"(w[11]), "r"(w[12]), "r"(w[13]), "r"(w[14]), "r"(w[15]) : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&w)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// 32-byte global loads / stores (one whole sector per thread; the address must be 32-byte aligned)
__device__ __forceinline__ void ld_global_v8(const float* p, float (&r)[8]) {
  asm volatile("ld.global.nc.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]) : "l"(p));
}
__device__ __forceinline__ void st_global_v8(float* p, const float (&r)[8]) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(p), "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]) : "memory");
}

// ---- fp32 operands as a few 16-bit planes -----------------------------------------------------------------------
// ELSA_FP32_PLANES == 3: x = a0 + a1 + a2 with three bf16 terms (8 + 8 + 8 significant bits, the full exponent range;
//   six cross products of weight >= 2^-16 per contraction).
// ELSA_FP32_PLANES == 2: x * 2^e = h0 + h1 with two fp16 terms (11 + 11 significant bits; three cross products
//   h0 h0 + h0 h1 + h1 h0 per contraction, the accuracy class of 3xTF32).  fp16 has five exponent bits, so every tensor
//   is multiplied by a power of two that puts its largest magnitude in [2^13, 2^14): elements down to 2^-16 of the
//   largest keep all 22 bits, smaller ones lose low bits gradually (absolute error below 2^-38 of the largest).
#ifndef ELSA_FP32_PLANES
#define ELSA_FP32_PLANES 2
#endif
constexpr int kPlanes = ELSA_FP32_PLANES;
static_assert(kPlanes == 2 || kPlanes == 3, "fp32 operands are split into two fp16 or three bf16 planes");
constexpr float kLog2Unit = kPlanes == 2 ? 14.f : 0.f;        // log2 of what a probability (<= 1) is multiplied by before its split
constexpr int kAmaxBlocks = 64, kAmaxFinal = 64;               // header words: partial |x| maxima (bit patterns), then the final one
constexpr int kPlaneHeader = 512;                              // bytes in front of a tensor's planes
constexpr uint32_t kPlaneFmt = kPlanes == 3 ? 1u : 0u;         // tcgen05 operand format: bf16 / fp16
constexpr int kPlaneDtype = kPlanes == 3 ? ELSA_BF16 : ELSA_F16;

// the power of two that scales a tensor whose largest magnitude has the bit pattern `absmax_bits` (0 for an all-zero
// tensor) into [2^13, 2^14); 1 for bf16 planes
__device__ __forceinline__ float plane_scale(uint32_t absmax_bits) {
  if (kPlanes == 3) return 1.f;
  int e = static_cast<int>(absmax_bits >> 23) - 127;         // floor(log2(absmax)) for a normal number
  if (absmax_bits == 0u) e = 13;
  e = max(-100, min(100, e));
  return __uint_as_float(static_cast<uint32_t>(127 + 13 - e) << 23);
}

// a pair of values -> its kPlanes packed 16-bit pairs (element 0 in the low half), leading plane first: round to
// nearest each time, remainders exact
__device__ __forceinline__ void split_planes_pair(float x0, float x1, uint32_t (&w)[kPlanes]) {
  if constexpr (kPlanes == 3) {
    const __nv_bfloat162 a0 = __floats2bfloat162_rn(x0, x1);
    const float2 f0 = __bfloat1622float2(a0);
    const float r0 = x0 - f0.x, r1 = x1 - f0.y;
    const __nv_bfloat162 a1 = __floats2bfloat162_rn(r0, r1);
    const float2 f1 = __bfloat1622float2(a1);
    const __nv_bfloat162 a2 = __floats2bfloat162_rn(r0 - f1.x, r1 - f1.y);
    w[0] = *reinterpret_cast<const uint32_t*>(&a0);
    w[1] = *reinterpret_cast<const uint32_t*>(&a1);
    w[kPlanes - 1] = *reinterpret_cast<const uint32_t*>(&a2);
  } else {
    const __half2 a0 = __floats2half2_rn(x0, x1);
    const float2 f0 = __half22float2(a0);
    const __half2 a1 = __floats2half2_rn(x0 - f0.x, x1 - f0.y);
    w[0] = *reinterpret_cast<const uint32_t*>(&a0);
    w[1] = *reinterpret_cast<const uint32_t*>(&a1);
  }
}

// two fp32 -> one packed pair of T (element 0 in the low half)
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

}  // namespace tc

// ---- host side: tensor maps -------------------------------------------------------------------
// 16-bit [B, H, n_rows, cols] view with element strides `st` (the elements of a row contiguous; cols a multiple of 8,
// at most 128) as a 4-D map (innermost first: cols, n_rows, H, B), box 64 x box_rows x 1 x 1, 128-byte swizzle:
// columns beyond `cols` and rows beyond n_rows read as zeros, so a narrower head dim lands in shared memory as a
// zero-padded 64-column tile; a head dim above 64 is loaded as two such tiles (x = 0 and x = 64).  box_batch = 2 takes
// two batch entries of one head in one box (short sequences: two of them fill a 128-row tile).  The strides must be multiples of 8 elements (16 bytes) and the base 16-byte aligned.
int make_tmap_rows64(CUtensorMap* map, const void* base, int dtype, int64_t n_rows, int heads, int batch, Strides st,
                     int box_rows, int cols = 64, int box_batch = 1);
// [n_mats][n_rows][64] fp32 tensor, box 32 x box_rows x 1 (two boxes cover the 64 columns), 128-byte swizzle
int make_tmap_f32_rows64(CUtensorMap* map, const void* base, int64_t n_rows, int64_t n_mats, int box_rows);

}  // namespace elsa
