// Thin inline-PTX wrappers for the sm_100a features the GEMM kernel uses:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (alloc / mma / commit / ld) and
// the proxy fences between them.  Every wait is bounded: a wait that runs out
// returns false and the caller records where it gave up and leaves cleanly.
#pragma once
#include <cstdint>
#include <cuda.h>

namespace gonn {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Non-blocking test of a phase (never suspends the thread).
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait.  `abort_flag` (shared memory) is polled so that one role that
// gave up takes the others down with it instead of each running out alone.
// Returns true when the phase completed.
constexpr uint32_t kSpinFast = 1u << 12;            // spins before backing off
constexpr uint64_t kWaitLimitNs = 1500ull * 1000 * 1000;  // 1.5 s, then give up
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile uint32_t* abort_flag) {
  for (uint32_t i = 0; i < kSpinFast; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 0; i < (1u << 24); ++i) {   // iteration cap as a second limit
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > kWaitLimitNs) return false;
    __nanosleep(64);
  }
  return false;
}

// ---------------------------------------------------------------- TMA
// Programmatic dependent launch: release lets the next kernel on the stream be scheduled
// early; wait holds this kernel until the previous one has completed (memory visible).
// Both are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void grid_dependency_release() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load global -> shared, completion counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* m,
                                            int32_t c0, int32_t c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
// 3-D tiled load (used for MN-major operands: all 128-byte-wide slabs of a tile in one box).
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* m, int32_t c0,
                                            int32_t c1, int32_t c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
// ---------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues for the CTA.  Each descriptor
// is given as two 32-bit halves: the issuing thread advances the start-address field with
// 32-bit adds.
__device__ __forceinline__ void mma_f16_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                             uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      ".reg .b64 DA, DB;\n\t"
      "mov.b64 DA, {%1, %2};\n\t"
      "mov.b64 DB, {%3, %4};\n\t"
      "setp.ne.b32 P, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], DA, DB, %5, P;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_tf32_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                              uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      ".reg .b64 DA, DB;\n\t"
      "mov.b64 DA, {%1, %2};\n\t"
      "mov.b64 DB, {%3, %4};\n\t"
      "setp.ne.b32 P, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], DA, DB, %5, P;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` once every tcgen05.mma issued so far by this thread retired.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar) : "memory");
}
// One warp reads its 32 TMEM lanes x 32 consecutive fp32 columns: thread t gets
// lane (lane_base + t), columns [col, col+32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// Same, 16 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster share one MMA: the leader (cluster rank 0) issues it,
// each CTA stages its own half of the operands and owns half of the rows of D.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank`.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// TMA load into this CTA's shared memory whose completion bytes are counted on
// a barrier that may live in the peer CTA (`bar_cluster` is a shared::cluster
// address).  No multicast: each CTA fetches its own boxes.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* m,
                                                 int32_t c0, int32_t c1, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(bar_cluster)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t smem_dst, const CUtensorMap* m,
                                                 int32_t c0, int32_t c1, int32_t c2,
                                                 uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(c2), "r"(bar_cluster)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t smem_dst, const CUtensorMap* m,
                                                 int32_t c0, int32_t c1, int32_t c2, int32_t c3,
                                                 uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
        "r"(bar_cluster)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// The pair's MMA (M = 256 over both CTAs), descriptors as low and high 32-bit words.
__device__ __forceinline__ void mma_f16_pair_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                                  uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      ".reg .b64 DA, DB;\n\t"
      "mov.b64 DA, {%1, %2};\n\t"
      "mov.b64 DB, {%3, %4};\n\t"
      "setp.ne.b32 P, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], DA, DB, %5, P;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_tf32_pair_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                                   uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                                   uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      ".reg .b64 DA, DB;\n\t"
      "mov.b64 DA, {%1, %2};\n\t"
      "mov.b64 DB, {%3, %4};\n\t"
      "setp.ne.b32 P, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], DA, DB, %5, P;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in every CTA of `cta_mask`
// once the pair's MMAs issued so far retired.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;"
      ::"r"(bar), "h"(cta_mask) : "memory");
}

// ------------------------------------------------- system-scope flags, multicast stores
// Flags that another GPU writes or reads (arrival of replicated data, acknowledgements).
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Orders this thread's earlier generic-proxy accesses to global memory (the acquire load of a
// flag) before its later asynchronous-proxy accesses (TMA loads of the data the flag covers).
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}
// 16 bytes to a multicast address: NVSwitch delivers a copy to every GPU bound to it.  A weak
// store carries no ordering of its own; a system-scope fence before the flag store orders it.
__device__ __forceinline__ void multimem_st_16(void* mc, const uint4& v) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// 16 bytes that are read once: no L1 allocation.
__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Epochs only grow; the comparison tolerates wrap-around of the 32-bit counter.
__device__ __forceinline__ bool epoch_reached(uint32_t seen, uint32_t wanted) {
  return int32_t(seen - wanted) >= 0;
}
// Polls `word` until it has reached `wanted`; false when the limit (`limit_ns` and an
// iteration cap) ran out or `abort_flag` (may be null) was raised.  Waits that feed one
// another get staggered limits, the innermost the shortest, so that the wait that names the
// cause runs out (and reports) before the waits that merely depend on it.
constexpr uint64_t kAckWaitLimitNs = 1000ull * 1000 * 1000;   // owner: acknowledgements of a slot
constexpr uint64_t kDataWaitLimitNs = 1250ull * 1000 * 1000;  // a rank: arrival of replicated data
__device__ __forceinline__ bool flag_wait(const uint32_t* word, uint32_t wanted,
                                          volatile uint32_t* abort_flag,
                                          uint64_t limit_ns = kWaitLimitNs) {
  for (uint32_t i = 0; i < 1024; ++i)
    if (epoch_reached(ld_acquire_sys(word), wanted)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 0; i < (1u << 24); ++i) {
    if (epoch_reached(ld_acquire_sys(word), wanted)) return true;
    if (abort_flag && *abort_flag) return false;
    if (globaltimer_ns() - t0 > limit_ns) return false;
    __nanosleep(100);
  }
  return false;
}

// ------------------------------------------------- descriptors (host+device)
// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle:
//   [0,14) start address >> 4, [16,30) leading byte offset >> 4,
//   [32,46) stride byte offset >> 4, [46,48) version = 1, [61,64) layout.
// `layout`: 2 = 128-byte swizzle of 16-byte chunks; 1 = 128-byte swizzle of
// 32-byte chunks, the only layout tf32 operands may use when MN-major; 4 = 64-byte
// swizzle (K-major tiles whose rows hold 64 bytes of K: groups of 8 rows, 512 bytes).
__host__ __device__ constexpr uint64_t smem_desc(uint32_t layout, uint32_t lbo_bytes,
                                                 uint32_t sbo_bytes) {
  return (uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16) | (uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32) |
         (uint64_t(1) << 46) | (uint64_t(layout) << 61);
}
// Instruction descriptor for kind::f16 / kind::tf32 with fp32 accumulation:
//   [4,6) D format (1 = f32), [7,10) A format, [10,13) B format (0 f16, 1 bf16,
//   2 tf32), bit 15 A is MN-major, bit 16 B is MN-major, [17,23) N >> 3,
//   [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t ab_format, bool a_mn_major,
                                                  bool b_mn_major, uint32_t m, uint32_t n) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | (uint32_t(a_mn_major) << 15) |
         (uint32_t(b_mn_major) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

}  // namespace ptx
}  // namespace gonn
