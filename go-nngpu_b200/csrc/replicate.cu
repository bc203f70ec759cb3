// Replication of the B operand of a row-sharded product over NVSwitch.
//
// In the row-sharded MatMul every GPU multiplies its own rows of A by the whole
// of B, so B has to reach every GPU before the products can start.  The rank
// that owns B pushes it ONCE into the switch with `multimem.st`: the store goes
// to a multicast address that is bound to the same buffer on every GPU of the
// group, and the switch delivers a copy to each of them.  The owner's NVLink
// carries B once instead of once per peer, and no GPU forwards anything.
//
// Two kernels:
//   replicate_send_kernel  (owner)    waits until every rank has finished with the
//                                     slot (acknowledgements), copies src -> multicast
//                                     dst, and when the last block is done publishes
//                                     the epoch in every rank's arrival flag.
//   replicate_wait_kernel  (everyone) acknowledges to the owner that its earlier
//                                     products are complete, then waits for the epoch.
// Both waits are bounded (1.5 s by %globaltimer plus an iteration cap): a wait
// that runs out writes a status word and the kernel returns; there is no trap
// and no endless spin.
//
// Memory order.  Data stores are relaxed multimem stores.  Each block then runs
// __syncthreads, one thread fences at system scope and counts the block in; the
// thread that sees the count complete fences again and writes the flags with
// st.release.sys through plain peer pointers.  A reader takes the flag with
// ld.acquire.sys.  No multicast LOAD of any kind is issued anywhere in this file.
#include <cstdint>
#include <cstdlib>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace gonn {
namespace {

constexpr uint64_t kReplicaWaitNs = 1500ull * 1000 * 1000;

// Blocks that have finished their share of the current send (zero between launches).
__device__ unsigned int g_send_blocks_done;

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// WEAK: a plain (weak) multicast store; else relaxed at system scope.  Either way the data
// stores carry no ordering of their own: the fences before the flag stores order them.
template <bool WEAK>
__device__ __forceinline__ void multimem_st_16(void* mc, const uint4& v) {
  if constexpr (WEAK) {
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x),
                 "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
  } else {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
  }
}
__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Epochs only grow; the comparison tolerates wrap-around of the 32-bit counter.
__device__ __forceinline__ bool reached(uint32_t seen, uint32_t wanted) {
  return int32_t(seen - wanted) >= 0;
}

// Polls `word` until it has reached `wanted`; false when the limit ran out.
__device__ bool bounded_wait(const uint32_t* word, uint32_t wanted) {
  for (uint32_t i = 0; i < 4096; ++i)
    if (reached(ld_acquire_sys(word), wanted)) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  for (uint32_t i = 0; i < (1u << 24); ++i) {
    if (reached(ld_acquire_sys(word), wanted)) return true;
    if (ptx::globaltimer_ns() - t0 > kReplicaWaitNs) return false;
    __nanosleep(128);
  }
  return false;
}

template <bool WEAK>
__global__ void __launch_bounds__(512)
replicate_send_kernel(const uint4* __restrict__ src, uint4* mc_dst, uint64_t n16,
                      void* const* __restrict__ bases, int world, int my_rank, uint64_t ctrl_offset,
                      int slot, uint32_t epoch, uint32_t ack_needed, GemmStatus* status) {
  ptx::grid_dependency_release();
  ptx::grid_dependency_wait();
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // the slot may be overwritten only when every rank's products of the epoch that
  // last used it are complete
  if (threadIdx.x < world) {
    const ReplicaControl* mine = reinterpret_cast<const ReplicaControl*>(
        static_cast<const char*>(bases[my_rank]) + ctrl_offset);
    if (!bounded_wait(&mine->ack[threadIdx.x], ack_needed)) {
      s_ok = 0;
      if (blockIdx.x == 0) {
        status->code = 4;
        status->where = threadIdx.x;
        status->tile = epoch;
        status->kblock = ack_needed;
      }
    }
  }
  __syncthreads();
  if (s_ok) {
    const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
    uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n16; i += 4 * stride) {
      const uint4 v0 = ld_stream_16(src + i);
      const uint4 v1 = ld_stream_16(src + i + stride);
      const uint4 v2 = ld_stream_16(src + i + 2 * stride);
      const uint4 v3 = ld_stream_16(src + i + 3 * stride);
      multimem_st_16<WEAK>(mc_dst + i, v0);
      multimem_st_16<WEAK>(mc_dst + i + stride, v1);
      multimem_st_16<WEAK>(mc_dst + i + 2 * stride, v2);
      multimem_st_16<WEAK>(mc_dst + i + 3 * stride, v3);
    }
    for (; i < n16; i += stride) multimem_st_16<WEAK>(mc_dst + i, ld_stream_16(src + i));
  }
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(&g_send_blocks_done, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) g_send_blocks_done = 0;
    // a send that gave up publishes nothing: the receivers' waits run out and report too
    if (s_ok && threadIdx.x < world) {
      __threadfence_system();
      ReplicaControl* theirs = reinterpret_cast<ReplicaControl*>(
          static_cast<char*>(bases[threadIdx.x]) + ctrl_offset);
      st_release_sys(&theirs->arrived[slot], epoch);
    }
  }
}

__global__ void __launch_bounds__(32)
replicate_wait_kernel(void* const* __restrict__ bases, int owner, int my_rank, uint64_t ctrl_offset,
                      int slot, uint32_t epoch, uint32_t ack_value, GemmStatus* status) {
  // No early release of the next kernel here: the product behind this wait is a persistent
  // grid that fills every SM, and the one behind that cannot be placed at all.  Scheduled
  // ahead of time, such a grid waits at the head of the block scheduler's queue and keeps the
  // owner's push (another stream) from getting SMs while this kernel waits for that push.
  // The next kernel is therefore released only when this one exits.
  ptx::grid_dependency_wait();  // everything earlier on this stream is complete from here on
  if (threadIdx.x != 0) return;
  ReplicaControl* owners = reinterpret_cast<ReplicaControl*>(static_cast<char*>(bases[owner]) +
                                                            ctrl_offset);
  st_release_sys(&owners->ack[my_rank], ack_value);
  const ReplicaControl* mine = reinterpret_cast<const ReplicaControl*>(
      static_cast<const char*>(bases[my_rank]) + ctrl_offset);
  if (!bounded_wait(&mine->arrived[slot], epoch)) {
    status->code = 5;
    status->where = uint32_t(slot);
    status->tile = epoch;
    status->kblock = ld_acquire_sys(&mine->arrived[slot]);
  }
}

}  // namespace

cudaError_t launch_replicate_send(const void* src, void* mc_dst, uint64_t bytes, void* const* bases,
                                  int world, int my_rank, uint64_t ctrl_offset, int slot,
                                  uint32_t epoch, uint32_t ack_needed, GemmStatus* status, int ctas,
                                  cudaStream_t stream) {
  // weak multicast stores; GONNGPU_REPLICATE_WEAK=0 (read once) makes them relaxed.sys
  static const bool weak = [] {
    const char* e = std::getenv("GONNGPU_REPLICATE_WEAK");
    return !(e && e[0] == '0');
  }();
  auto kern = weak ? replicate_send_kernel<true> : replicate_send_kernel<false>;
  return launch_kernel(kern, dim3(unsigned(ctas)), dim3(512), 0, stream,
                       static_cast<const uint4*>(src), static_cast<uint4*>(mc_dst), bytes / 16, bases,
                       world, my_rank, ctrl_offset, slot, epoch, ack_needed, status);
}

cudaError_t launch_replicate_wait(void* const* bases, int owner, int my_rank, uint64_t ctrl_offset,
                                  int slot, uint32_t epoch, uint32_t ack_value, GemmStatus* status,
                                  cudaStream_t stream) {
  return launch_kernel(replicate_wait_kernel, dim3(1), dim3(32), 0, stream, bases, owner, my_rank,
                       ctrl_offset, slot, epoch, ack_value, status);
}

}  // namespace gonn
