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
// Memory order.  Data stores are weak multimem stores.  Each block then runs
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

// Blocks that have finished their share of the current send, and whether one of them gave
// up waiting for the acknowledgements (both zero between launches).  One send at a time per
// GPU: two sends of one GPU must be ordered on one stream.
__device__ unsigned int g_send_blocks_done;
__device__ unsigned int g_send_gave_up;

using ptx::ld_acquire_sys;
using ptx::st_release_sys;

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
    if (!ptx::flag_wait(&mine->ack[threadIdx.x], ack_needed, nullptr)) {
      s_ok = 0;
      // whichever block runs out first reports; any block that ran out keeps the epoch
      // from being published, so that no receiver multiplies a partly written slot
      if (atomicOr(&g_send_gave_up, 1u) == 0u) {
        status->where = threadIdx.x;
        status->tile = epoch;
        status->kblock = ack_needed;
        status->code = 4;
      }
    }
  }
  __syncthreads();
  if (s_ok) {
    // The link only runs at full rate with enough bytes in flight (rate x latency is about
    // 1.5 MB towards 8 GPUs): every thread issues kDepth loads before its first store.
    constexpr int kDepth = 8;
    const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
    uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + (kDepth - 1) * stride < n16; i += kDepth * stride) {
      uint4 v[kDepth];
#pragma unroll
      for (int j = 0; j < kDepth; ++j) v[j] = ptx::ld_stream_16(src + i + j * stride);
#pragma unroll
      for (int j = 0; j < kDepth; ++j) ptx::multimem_st_16(mc_dst + i + j * stride, v[j]);
    }
    for (; i < n16; i += stride) ptx::multimem_st_16(mc_dst + i, ptx::ld_stream_16(src + i));
  }
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(&g_send_blocks_done, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last) {
    __shared__ unsigned int s_gave_up;
    if (threadIdx.x == 0) {
      g_send_blocks_done = 0;
      s_gave_up = atomicExch(&g_send_gave_up, 0u);
    }
    __syncthreads();
    // a send that gave up publishes nothing: the receivers' waits run out and report too
    if (!s_gave_up && threadIdx.x < world) {
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
  if (!ptx::flag_wait(&mine->arrived[slot], epoch, nullptr)) {
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
  return launch_kernel(replicate_send_kernel, dim3(unsigned(ctas)), dim3(512), 0, stream,
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
