// Dense GEMM for sm_100a: C[M,N] = act(alpha * A.B + beta * C_in + bias).
//
// This is the kernel behind the reference's MatMul
// (gpu/matrix/matrix.go:53-105 -> internal/cgo/metal_bridge_matrix.m:24-125),
// its alpha/beta variant (internal/cgo/metal_bridge_kernels.m:417-486) and the
// fused linear + bias + activation (internal/cgo/default.metal:459-509).
//
// Structure (one persistent CTA per SM, 6 warps):
//   warp 0    TMA producer: cp.async.bulk.tensor boxes of 128-byte rows with the
//             128-byte swizzle into a ring of shared-memory stages
//   warp 1    TMEM owner and MMA issuer: one lane issues tcgen05.mma from
//             shared-memory descriptors into one of two TMEM accumulators
//   warps 2-5 epilogue: tcgen05.ld of the finished accumulator, alpha/beta/bias/
//             activation in registers, stores to C; overlaps the next tile's
//             main loop because the accumulators are double-buffered
// Operands are fp16 (kind::f16) or pairs of tf32 planes (kind::tf32, three
// MMAs per k step: lo.hi + hi.lo + hi.hi) and may be K-major or MN-major, so
// A.B, At.B and A.Bt need no materialised transpose.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace gonn {

namespace {

constexpr uint32_t BLOCK_M = 128;
constexpr uint32_t SLAB_ROW_BYTES = 128;             // one swizzle row
constexpr uint32_t A_TILE_BYTES = BLOCK_M * SLAB_ROW_BYTES;  // 16 KiB per plane per k block
constexpr uint32_t KSTEPS = 4;                       // MMAs (per product) per k block
constexpr uint32_t NUM_THREADS = 192;
constexpr uint32_t GATED_THREADS = 320;   // row-sharded product: 4 more warps, used by the sending CTAs
constexpr uint32_t SENDER_GROUPS = 4;     // the slabs are dealt out to this many groups of sender warps
constexpr uint32_t SENDER_DEPTH = 16;     // 16-byte loads a sender lane keeps in flight
constexpr uint32_t SMEM_LIMIT = 227 * 1024;

// How one operand's k-block tile is fetched by TMA and described to the MMA.
struct OperandPlan {
  uint32_t slabs;        // TMA boxes per tile per k block
  uint32_t slab_bytes;   // shared-memory bytes per box
  int32_t c0_tile, c0_slab, c0_k;  // box coordinate 0 = tile*c0_tile + slab*c0_slab + kb*c0_k
  int32_t c1_tile, c1_k;           // box coordinate 1 = tile*c1_tile + kb*c1_k
  uint32_t kstep_bytes;  // descriptor start-address advance per MMA k step
  uint64_t desc;         // shared-memory descriptor without the start address
  // MN-major operands whose plane pitch allows it are loaded as ONE 3-D box per tile and
  // k block (128 bytes of MN, block_k rows of K, all slabs) instead of one 2-D box per
  // slab: coordinates (0, coordinate 1, tile * c2_tile).  Fewer, larger boxes load faster.
  uint32_t box3d;
  int32_t c2_tile;
  // K-major operands of the kernels whose stage holds several k blocks: ONE 3-D box
  // (128 bytes of K, the tile's rows, `kgroup` consecutive k blocks) per stage, so that
  // every row is fetched as kgroup x 128 contiguous bytes: coordinates
  // (0, tile * c1_tile, first k block).  0 = one box per k block.
  uint32_t kgroup;
};

// Device-side view of a ShardLink (row-sharded product that replicates B itself).
struct ShardParams {
  const uint4* src;      // owner: B in this GPU's memory, `row_chunks` 16-byte chunks per row
  uint4* mc_dst;         // multicast address of the slot, or null (plain peer stores)
  void* const* bases;    // every rank's symmetric buffer as this GPU maps it
  uint64_t slot_offset, ctrl_offset;
  uint32_t world, owner, rank, slot, epoch, ack_needed;
  uint32_t slab_tiles;   // column tiles per arrival flag
  uint32_t num_slabs;
  uint32_t rows;         // K
  uint32_t row_chunks;   // 16-byte chunks per row of B
  uint32_t slab_chunks;  // 16-byte chunks per row of one slab
  // On the owner the last `sender_pairs` CTA pairs push B with all their warps before they
  // multiply, and the tile order leaves them out of the first `late_rounds` rounds (both 0 on
  // the other ranks).
  uint32_t sender_pairs, late_rounds;
  // Optional timeline of one launch (device memory, 128 words of %globaltimer nanoseconds, or
  // null): [0] first CTA past its set-up, [1 + s] slab s published by the owner's senders,
  // [40 + s] slab s first seen by a producer of this rank (atomicMin: preset to ~0), [80] last
  // CTA leaving.
  unsigned long long* trace;
};

struct KernelParams {
  OperandPlan a, b;
  uint32_t M, N;
  uint32_t tiles_m, tiles_n, num_tiles, num_kblocks, group_m;
  // The first `group_m0` row tiles form one group of their own (0 = none): the gated product
  // sweeps them column slab by column slab while B is still arriving.
  uint32_t group_m0;
  uint32_t idesc;
  float* C;
  const float* c_in;
  const float* bias;
  uint64_t ldc;
  float alpha, beta, act_param;
  int act;
  uint32_t vec_store;  // C base and pitch allow 16-byte stores
  // batched products (stacked matrices): tiles per batch (0 = one product), and the
  // row-coordinate step per batch of the A and B tensor maps; M is then per batch
  uint32_t batch_tiles;
  int32_t a_batch_c1, b_batch_c1;
  // split-K (fp32 single-CTA kernel): a tile's k blocks are shared by `splits` work
  // units of `kb_per_split` k blocks each; partial sums go through `sk_ws`, and the
  // unit that arrives last on the tile's counter adds them up and writes C
  uint32_t splits, kb_per_split;
  float* sk_ws;
  uint32_t* sk_count;
  GemmStatus* status;
  // fp32 pair kernel with bf16 correction planes: the bf16 tiles' descriptors (without the
  // start address), their advance per K = 16 step, whether the operand is MN-major, and the
  // instruction descriptor of the bf16 MMAs
  uint64_t ax_desc, bx_desc;
  uint32_t ax_kstep, bx_kstep, ax_mn, bx_mn, idesc_x;
  ShardParams sh;
};

__device__ __forceinline__ void tile_coords(const KernelParams& p, uint32_t t, uint32_t& tm,
                                            uint32_t& tn) {
  // Groups of `group_m` row tiles sweep the columns together so that a wave of
  // CTAs shares A rows and B columns in L2.
  uint32_t base_m = 0;
  if (p.group_m0) {
    const uint32_t first = p.group_m0 * p.tiles_n;
    if (t < first) {
      // slab by slab, down the rows for even slabs and up for odd ones: the rows of A touched
      // last are touched first again, which is what an LRU-like L2 keeps
      tn = t / p.group_m0;
      const uint32_t r = t - tn * p.group_m0;
      tm = (tn & 1u) ? p.group_m0 - 1u - r : r;
      return;
    }
    t -= first;
    base_m = p.group_m0;
  }
  const uint32_t per_group = p.group_m * p.tiles_n;
  const uint32_t g = t / per_group;
  const uint32_t first_m = base_m + g * p.group_m;
  const uint32_t gm = min(p.group_m, p.tiles_m - first_m);
  const uint32_t r = t - g * per_group;
  tm = first_m + r % gm;
  tn = r / gm;
}

// Batched products: tiles are numbered batch by batch.
__device__ __forceinline__ void tile_coords(const KernelParams& p, uint32_t t, uint32_t& tm,
                                            uint32_t& tn, uint32_t& batch) {
  batch = p.batch_tiles ? t / p.batch_tiles : 0u;
  tile_coords(p, t - batch * p.batch_tiles, tm, tn);
}

// One operand tile's k block into shared memory at `dst` (completion bytes on `bar`).
template <bool PAIR>
__device__ __forceinline__ void load_operand(const OperandPlan& o, const CUtensorMap* m, uint32_t dst,
                                             int32_t tile, int32_t kb, int32_t c1_extra, uint32_t bar) {
  const int32_t c1 = tile * o.c1_tile + kb * o.c1_k + c1_extra;
  if (o.box3d) {
    if (PAIR) ptx::tma_load_3d_pair(dst, m, 0, c1, tile * o.c2_tile, bar);
    else ptx::tma_load_3d(dst, m, 0, c1, tile * o.c2_tile, bar);
    return;
  }
  for (uint32_t s = 0; s < o.slabs; ++s) {
    const int32_t c0 = tile * o.c0_tile + int32_t(s) * o.c0_slab + kb * o.c0_k;
    if (PAIR) ptx::tma_load_2d_pair(dst + s * o.slab_bytes, m, c0, c1, bar);
    else ptx::tma_load_2d(dst + s * o.slab_bytes, m, c0, c1, bar);
  }
}

// Both bf16 planes of one operand tile's k block (32 of K) in one box; `tile` counts 128 rows
// or columns.  See gemm_tf32x3_pair_kernel.
__device__ __forceinline__ void load_bf16_planes(uint32_t mn_major, const CUtensorMap* m, uint32_t dst,
                                                 int32_t tile, int32_t kb, uint32_t bar) {
  if (mn_major) ptx::tma_load_4d_pair(dst, m, 0, kb * 32, tile * 2, 0, bar);
  else ptx::tma_load_3d_pair(dst, m, kb * 32, tile * 128, 0, bar);
}

// The epilogues keep their accumulators in registers, so their loops are fully unrolled:
// 32 to 128 copies of whatever the activation inlines.  With expf / tanhf inlined in every
// copy the epilogue's code no longer fits the instruction cache, and even a ReLU, which
// only branches past them, took 11 us longer per launch (512 x 1024 x 1024: 27 against
// 16 us).  The transcendental activations are therefore one out-of-line function.
__device__ __noinline__ float apply_act_transcendental(float v, int act) {
  switch (act) {
    case ACT_SIGMOID: return 1.0f / (1.0f + expf(-v));
    case ACT_TANH: return tanhf(v);
    default: return 0.5f * v * (1.0f + tanhf(0.7978845608f * (v + 0.044715f * v * v * v)));  // ACT_GELU
  }
}
__device__ __forceinline__ float apply_act(float v, int act, float param) {
  if (act == ACT_RELU) return fmaxf(v, 0.0f);
  if (act == ACT_LEAKY) return v > 0.0f ? v : v * param;
  if (act == ACT_SIGMOID || act == ACT_TANH || act == ACT_GELU) return apply_act_transcendental(v, act);
  return v;
}

// Raises the CTA's abort flag; true for the one role that raised it.  Only that role reports:
// the roles that leave because they SAW the flag would otherwise overwrite the cause with
// their own, later, wait (the status words live in mapped host memory, where "write only if
// still zero" cannot tell a report of a microsecond ago from none).
__device__ __forceinline__ bool first_to_give_up(volatile uint32_t* abort_flag) {
  return atomicExch(const_cast<uint32_t*>(abort_flag), 1u) == 0u;
}

__device__ __forceinline__ void report(GemmStatus* st, uint32_t code, uint32_t where,
                                       uint32_t tile, uint32_t kb) {
  // `st` may be page-locked host memory mapped into the device: plain stores
  // only (the first reporter wins most of the time, which is all that is needed).
  volatile GemmStatus* v = st;
  if (v->code == 0u) {
    v->where = where;
    v->tile = tile;
    v->kblock = kb;
    v->code = code;
  }
}

// alpha * acc + beta * C_in + bias, then the activation, for four neighbouring columns;
// `cin` / `bias` point at the first of the four (16-byte aligned) or are null.
__device__ __forceinline__ float4 epilogue_value4(const KernelParams& p, float4 v, const float* cin,
                                                  const float* bias) {
  v.x *= p.alpha;
  v.y *= p.alpha;
  v.z *= p.alpha;
  v.w *= p.alpha;
  if (cin) {
    const float4 o = *reinterpret_cast<const float4*>(cin);
    v.x += p.beta * o.x;
    v.y += p.beta * o.y;
    v.z += p.beta * o.z;
    v.w += p.beta * o.w;
  }
  if (bias) {
    const float4 b = *reinterpret_cast<const float4*>(bias);
    v.x += b.x;
    v.y += b.y;
    v.z += b.z;
    v.w += b.w;
  }
  if (p.act >= 0) {
    v.x = apply_act(v.x, p.act, p.act_param);
    v.y = apply_act(v.y, p.act, p.act_param);
    v.z = apply_act(v.z, p.act, p.act_param);
    v.w = apply_act(v.w, p.act, p.act_param);
  }
  return v;
}
// The same for one column.
__device__ __forceinline__ float epilogue_value(const KernelParams& p, float v, const float* cin,
                                                const float* bias) {
  v *= p.alpha;
  if (cin) v += p.beta * *cin;
  if (bias) v += *bias;
  if (p.act >= 0) v = apply_act(v, p.act, p.act_param);
  return v;
}

// One thread's 32 consecutive accumulator columns of one output row:
// alpha/beta/bias/activation, then 16-byte stores (scalar at ragged edges).
__device__ __forceinline__ void epilogue_store32(const KernelParams& p, const uint32_t (&r)[32],
                                                 uint32_t row, uint32_t col0) {
  if (row >= p.M || col0 >= p.N) return;
  float* c_row = p.C + uint64_t(row) * p.ldc;
  const float* cin_row = p.c_in ? p.c_in + uint64_t(row) * p.ldc : nullptr;
  if (col0 + 32u <= p.N && p.vec_store) {
#pragma unroll
    for (uint32_t j = 0; j < 32; j += 4) {
      const float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                   __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
      *reinterpret_cast<float4*>(c_row + col0 + j) =
          epilogue_value4(p, v, cin_row ? cin_row + col0 + j : nullptr, p.bias ? p.bias + col0 + j : nullptr);
    }
  } else {
#pragma unroll
    for (uint32_t j = 0; j < 32; ++j) {
      const uint32_t col = col0 + j;
      if (col < p.N)
        c_row[col] = epilogue_value(p, __uint_as_float(r[j]), cin_row ? cin_row + col : nullptr,
                                    p.bias ? p.bias + col : nullptr);
    }
  }
}

template <int KIND, int BLOCK_N, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a0,
                    const __grid_constant__ CUtensorMap tm_a1,
                    const __grid_constant__ CUtensorMap tm_b0,
                    const __grid_constant__ CUtensorMap tm_b1,
                    const __grid_constant__ KernelParams p) {
  constexpr uint32_t PLANES = (KIND == int(Kind::TF32x3)) ? 2 : 1;
  constexpr uint32_t B_TILE_BYTES = BLOCK_N * SLAB_ROW_BYTES;
  constexpr uint32_t STAGE_BYTES = PLANES * (A_TILE_BYTES + B_TILE_BYTES);
  constexpr uint32_t TMEM_COLS = (2 * BLOCK_N < 32) ? 32 : 2 * BLOCK_N;
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns");

  extern __shared__ uint8_t smem_raw[];
  // Swizzled tiles need 1024-byte aligned bases.
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  // barrier slots: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (uint32_t a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tmap(&tm_a0);
    ptx::prefetch_tmap(&tm_b0);
    if (PLANES == 2) {
      ptx::prefetch_tmap(&tm_a1);
      ptx::prefetch_tmap(&tm_b1);
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above touched no global memory: from here on the previous kernel's results
  // are needed (and its reads of our output buffers must be over)
  ptx::grid_dependency_release();
  ptx::grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    uint32_t stage = 0, phase = 0;
    bool alive = true;
    for (uint32_t t = blockIdx.x; alive && t < p.num_tiles; t += gridDim.x) {
      uint32_t tm, tn;
      tile_coords(p, t, tm, tn);
      for (uint32_t kb = 0; kb < p.num_kblocks; ++kb) {
        bool ok = ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) {
            if (first_to_give_up(abort_flag)) report(p.status, 1, stage, t, kb);
          }
          alive = false;
          break;
        }
        if (lane == 0) {
          const uint32_t fb = full_bar(stage);
          ptx::mbar_arrive_expect_tx(fb, STAGE_BYTES);
          uint32_t dst = smem_base + stage * STAGE_BYTES;
#pragma unroll
          for (uint32_t pl = 0; pl < PLANES; ++pl) {
            load_operand<false>(p.a, pl ? &tm_a1 : &tm_a0, dst, int32_t(tm), int32_t(kb), 0, fb);
            dst += A_TILE_BYTES;
          }
#pragma unroll
          for (uint32_t pl = 0; pl < PLANES; ++pl) {
            load_operand<false>(p.b, pl ? &tm_b1 : &tm_b0, dst, int32_t(tn), int32_t(kb), 0, fb);
            dst += B_TILE_BYTES;
          }
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------- MMA issuer: one thread
    // (next stage's barrier tested without blocking, descriptors advanced by
    // 32-bit adds: see gemm_tf32x3_kernel)
    if (lane == 0) {
      const uint32_t a_hi32 = uint32_t(p.a.desc >> 32), b_hi32 = uint32_t(p.b.desc >> 32);
      const uint32_t a_lo0 = uint32_t(p.a.desc), b_lo0 = uint32_t(p.b.desc);
      const uint32_t a_step = p.a.kstep_bytes >> 4, b_step = p.b.kstep_bytes >> 4;
      uint32_t stage = 0, phase = 0;
      uint32_t local = 0;
      uint32_t ready = 0;
      bool alive = true;
      for (uint32_t t = blockIdx.x; alive && t < p.num_tiles; t += gridDim.x, ++local) {
        const uint32_t acc = local & 1u;
        const uint32_t acc_phase = (local >> 1) & 1u;
        if (!ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
          if (first_to_give_up(abort_flag)) report(p.status, 2, 0x100u | acc, t, 0);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
        for (uint32_t kb = 0; kb < p.num_kblocks; ++kb) {
          if (!ready && !ptx::mbar_wait(full_bar(stage), phase, abort_flag)) {
            if (first_to_give_up(abort_flag)) report(p.status, 2, stage, t, kb);
            alive = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t next_stage = (stage + 1 == STAGES) ? 0 : stage + 1;
          const uint32_t next_phase = (stage + 1 == STAGES) ? phase ^ 1u : phase;
          const uint32_t ready_next = ptx::mbar_test_wait(full_bar(next_stage), next_phase);
          const uint32_t st = smem_base + stage * STAGE_BYTES;
          const uint32_t ah = a_lo0 + (st >> 4);
          const uint32_t bh = b_lo0 + ((st + PLANES * A_TILE_BYTES) >> 4);
#pragma unroll
          for (uint32_t ks = 0; ks < KSTEPS; ++ks) {
            const uint32_t accum = (kb | ks) ? 1u : 0u;
            if (KIND == int(Kind::F16)) {
              ptx::mma_f16_lohi(d_tmem, ah + ks * a_step, a_hi32, bh + ks * b_step, b_hi32, p.idesc, accum);
            } else {
              const uint32_t al = ah + (A_TILE_BYTES >> 4), bl = bh + (B_TILE_BYTES >> 4);
              ptx::mma_tf32_lohi(d_tmem, al + ks * a_step, a_hi32, bh + ks * b_step, b_hi32, p.idesc, accum);
              ptx::mma_tf32_lohi(d_tmem, ah + ks * a_step, a_hi32, bl + ks * b_step, b_hi32, p.idesc, 1u);
              ptx::mma_tf32_lohi(d_tmem, ah + ks * a_step, a_hi32, bh + ks * b_step, b_hi32, p.idesc, 1u);
            }
          }
          ptx::mma_commit(empty_bar(stage));  // stage reusable once these MMAs retired
          if (kb + 1 == p.num_kblocks) ptx::mma_commit(tfull_bar(acc));
          stage = next_stage;
          phase = next_phase;
          ready = ready_next;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const uint32_t quarter = warp & 3u;  // TMEM lanes this warp may read
    uint32_t local = 0;
    for (uint32_t t = blockIdx.x; t < p.num_tiles; t += gridDim.x, ++local) {
      const uint32_t acc = local & 1u;
      const uint32_t acc_phase = (local >> 1) & 1u;
      uint32_t tm, tn;
      tile_coords(p, t, tm, tn);
      bool ok = ptx::mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) {
          if (first_to_give_up(abort_flag)) report(p.status, 3, acc, t, 0);
        }
        break;
      }
      ptx::tc_fence_after();
      const uint32_t row = tm * BLOCK_M + quarter * 32u + lane;
      const uint32_t col_tile = tn * BLOCK_N;
      const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * BLOCK_N;
#pragma unroll 1
      for (uint32_t ch = 0; ch < BLOCK_N / 32; ++ch) {
        const uint32_t col0 = col_tile + ch * 32u;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        ptx::tmem_ld_32x32(taddr + ch * 32u, r);
        ptx::tmem_ld_wait();
        epilogue_store32(p, r, row, col0);
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
    }
  }

  // ---------------------------------------------------------------- teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A role gave up: give copies and MMAs already in flight time to land
    // before shared memory and TMEM are handed back.
    const uint64_t t0 = ptx::globaltimer_ns();
    for (uint32_t i = 0; i < (1u << 16); ++i) {
      if (ptx::globaltimer_ns() - t0 > 2000000ull) break;
      __nanosleep(1000);
    }
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// Row-sharded product: the pieces that move B (see ShardLink in kernels.h).
__device__ __forceinline__ ShardControl* shard_ctrl(const ShardParams& s, uint32_t rank) {
  return reinterpret_cast<ShardControl*>(static_cast<char*>(s.bases[rank]) + s.ctrl_offset);
}

// Sending CTAs of the owner.  The sending CTAs form up to SENDER_GROUPS groups BY CTA (CTA c
// of the senders is in group c % groups); after slab 0, which all of them send together, group g
// sends the slabs 1 + g, 1 + g + groups, ...  Within a
// slab each warp takes whole rows (consecutive lanes, consecutive 16-byte chunks).  After a
// slab every lane fences at system scope and the warp counts itself in on the slab's counter.
// A system-scope fence waits for every store the SM still has in flight, not only the warp's
// own: with warps of one SM working on different slabs each fence waited for all of them
// (measured: 25 to 50 us per slab), which is why a whole CTA works on one slab at a time.
// The arrival flag itself is written by a watcher (see publish_slabs) on an SM that sends
// nothing, or, where every pair sends, by the warp that completes the count.
__device__ void push_b_slabs(const ShardParams& s, uint32_t group, uint32_t groups, uint32_t group_wid,
                             uint32_t group_nwarps, uint32_t all_wid, uint32_t all_nwarps, uint32_t lane,
                             bool publish, GemmStatus* status) {
  ShardControl* mine = shard_ctrl(s, s.rank);
  // the slot may be overwritten only when every rank has finished with the epoch that last used it
  bool ok = true;
  if (lane < s.world) ok = ptx::flag_wait(&mine->ack[lane], s.ack_needed, nullptr, ptx::kAckWaitLimitNs);
  if (!__all_sync(0xffffffffu, ok)) {
    // nothing is written and nothing published: the products' own waits run out and report
    if (!ok && (atomicOr(&mine->gave_up, 2u) & 2u) == 0u) report(status, 4, lane, s.epoch, s.ack_needed);
    return;
  }
  // Slab 0 is what every pair of every rank waits for when the kernel starts: all sending warps
  // push it together (`all_wid` of `all_nwarps`), then the groups take the slabs 1, 2, ... in turn.
  for (uint32_t k = 0; k == 0 || group + (k - 1u) * groups + 1u < s.num_slabs; ++k) {
    const uint32_t slab = k == 0 ? 0u : group + (k - 1u) * groups + 1u;
    const uint32_t wid = k == 0 ? all_wid : group_wid;
    const uint32_t nwarps = k == 0 ? all_nwarps : group_nwarps;
    const uint32_t c0 = slab * s.slab_chunks;
    const uint32_t width = min(s.slab_chunks, s.row_chunks - c0);
    // The link only runs at full rate with enough bytes in flight (rate x latency is about
    // 1.5 MB): every lane issues SENDER_DEPTH loads, one per row, before its first store.
    for (uint32_t ch = lane; ch < width; ch += 32u) {
      const uint64_t col = uint64_t(c0) + ch;
      for (uint32_t row = wid; row < s.rows; row += SENDER_DEPTH * nwarps) {
        uint4 v[SENDER_DEPTH];
#pragma unroll
        for (uint32_t j = 0; j < SENDER_DEPTH; ++j) {
          const uint32_t r = row + j * nwarps;
          if (r < s.rows) v[j] = ptx::ld_stream_16(s.src + uint64_t(r) * s.row_chunks + col);
        }
#pragma unroll
        for (uint32_t j = 0; j < SENDER_DEPTH; ++j) {
          const uint32_t r = row + j * nwarps;
          if (r >= s.rows) continue;
          const uint64_t off = uint64_t(r) * s.row_chunks + col;
          if (s.mc_dst) {
            ptx::multimem_st_16(s.mc_dst + off, v[j]);
          } else {
            for (uint32_t k = 0; k < s.world; ++k)
              reinterpret_cast<uint4*>(static_cast<char*>(s.bases[k]) + s.slot_offset)[off] = v[j];
          }
        }
      }
    }
    __threadfence_system();
    __syncwarp();
    uint32_t last = 0;
    if (lane == 0) last = (atomicAdd(&mine->sent[slab], 1u) == nwarps - 1u) ? 1u : 0u;
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last && publish) {
      if (lane == 0 && s.trace) s.trace[1 + slab] = ptx::globaltimer_ns();
      if (lane == 0) mine->sent[slab] = 0;  // zero again for the next launch
      if (lane < s.world) {
        __threadfence_system();
        ptx::st_release_sys(&shard_ctrl(s, lane)->arrived[s.slot][slab], s.epoch);
      }
    }
  }
}

// Sender warps of group g: the sending CTAs c with c % groups == g, `warps` warps each.
__device__ __forceinline__ uint32_t sender_group_warps(uint32_t sender_ctas, uint32_t groups, uint32_t g,
                                                       uint32_t warps) {
  return ((sender_ctas - g + groups - 1u) / groups) * warps;
}

// Watcher (one warp of the owner's first CTA, which sends nothing): polls the slabs' counters
// and writes a slab's arrival flag on every rank as soon as all its sender warps have counted
// themselves in.  The senders fenced before they counted in; the flag goes out with
// st.release.sys from an SM that has no stores of its own in flight, so its fence is short.
__device__ void publish_slabs(const ShardParams& s, uint32_t sender_ctas, uint32_t groups, uint32_t warps,
                              uint32_t lane) {
  ShardControl* mine = shard_ctrl(s, s.rank);
  uint32_t pending = s.num_slabs >= 32u ? 0xffffffffu : ((1u << s.num_slabs) - 1u);
  const uint64_t t0 = ptx::globaltimer_ns();
  // (a push that gave up never completes its counts: the limit ends the watch, and the
  // products' own waits report)
  while (pending && ptx::globaltimer_ns() - t0 < ptx::kAckWaitLimitNs + ptx::kDataWaitLimitNs) {
    for (uint32_t slab = 0; slab < s.num_slabs; ++slab) {
      if (!((pending >> slab) & 1u)) continue;
      uint32_t done = 0;
      if (lane == 0) {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(done) : "l"(&mine->sent[slab]) : "memory");
        done = done == (slab == 0 ? sender_ctas * warps
                                  : sender_group_warps(sender_ctas, groups, (slab - 1u) % groups, warps));
      }
      done = __shfl_sync(0xffffffffu, done, 0);
      if (!done) continue;
      if (lane == 0 && s.trace) s.trace[1 + slab] = ptx::globaltimer_ns();
      if (lane == 0) mine->sent[slab] = 0;  // zero again for the next launch
      if (lane < s.world) ptx::st_release_sys(&shard_ctrl(s, lane)->arrived[s.slot][slab], s.epoch);
      pending &= ~(1u << slab);
    }
    __nanosleep(200);
  }
}

// Last step of a CTA of the gated product: the CTA that leaves last tells the owner that this
// rank has finished reading the slot (unless some CTA gave up), and zeroes the scratch words.
__device__ __forceinline__ void shard_exit(const ShardParams& s, bool gave_up) {
  ShardControl* mine = shard_ctrl(s, s.rank);
  if (gave_up) atomicOr(&mine->gave_up, 1u);
  __threadfence();
  if (atomicAdd(&mine->exited, 1u) == gridDim.x - 1u) {
    if (s.trace) s.trace[80] = ptx::globaltimer_ns();
    mine->exited = 0;
    const uint32_t gave = atomicExch(&mine->gave_up, 0u);
    if (!gave) {
      __threadfence_system();
      ptx::st_release_sys(&shard_ctrl(s, s.owner)->ack[s.rank], s.epoch);
    }
  }
}

// The i-th tile of pair `pair` in the gated product.  Everywhere but on the owner that is the
// usual pair + i * num_pairs.  On the owner the last `sender_pairs` pairs are busy sending when
// the kernel starts: the first `late_rounds` rounds are dealt out among the other pairs only,
// and the sending pairs join behind them, so that they end up with about as many tiles fewer
// as the sending took.  A pair is done when the result reaches num_tiles.
__device__ __forceinline__ uint32_t gated_tile_at(const ShardParams& s, uint32_t pair,
                                                  uint32_t num_pairs, uint32_t i) {
  const uint32_t early = num_pairs - s.sender_pairs;
  if (pair >= early) return s.late_rounds * early + i * num_pairs + pair;
  return i < s.late_rounds ? i * early + pair : s.late_rounds * early + (i - s.late_rounds) * num_pairs + pair;
}

// ---------------------------------------------------------------------------
// fp16 kernel for large problems: CTA pairs (cta_group::2).
//
// A cluster of two CTAs computes a 256 x BLOCK_N tile.  CTA r of the pair
// stages rows [128r, 128r+128) of the A tile and columns [r*BLOCK_N/2, ..) of
// the B tile in its own shared memory; the leader (rank 0) issues one
// tcgen05.mma.cta_group::2 with M=256 that reads both CTAs' shared memory and
// writes 128 rows of D into each CTA's TMEM.  Per CTA this halves the B bytes
// that cross L2 -> SM and that are written to and read from shared memory,
// which is what limits the single-CTA kernel.  No multicast loads are used.
//
// Barriers (same offsets in both CTAs):
//   full[s]   leader only: 1 arrival (leader's producer, expecting both CTAs'
//             bytes) + the bytes of both CTAs' TMA loads
//   empty[s]  per CTA: tcgen05.commit from the leader, multicast to both
//   tfull[a]  per CTA: multicast commit when the tile's last MMA retired
//   tempty[a] leader only: 8 arrivals = 4 epilogue warps of each CTA
//
// A stage holds SUB k blocks (each laid out as A tile then B half tile); one
// barrier round (full wait, commit) therefore covers 4*SUB MMAs.
//
// GATED: the row-sharded product that replicates B itself.  On the owner the last pairs push B
// with all their warps (ten per CTA) before they join the product; every producer waits for
// the arrival flag of a tile's column slab before the tile's first load; the last CTA to leave
// acknowledges the epoch.
template <int BLOCK_N, int STAGES, int SUB, bool GATED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GATED ? GATED_THREADS : NUM_THREADS, 1)
gemm_f16_pair_kernel(const __grid_constant__ CUtensorMap tm_a,
                     const __grid_constant__ CUtensorMap tm_b,
                     const __grid_constant__ KernelParams p) {
  constexpr uint32_t B_TILE_BYTES = (BLOCK_N / 2) * SLAB_ROW_BYTES;  // this CTA's half
  constexpr uint32_t STAGE_BYTES = SUB * (A_TILE_BYTES + B_TILE_BYTES);  // SUB k blocks
  constexpr uint32_t TMEM_COLS = 2 * BLOCK_N;
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512 && TMEM_COLS >= 32, "TMEM");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t cta_rank = ptx::cluster_ctarank();
  const bool leader = (cta_rank == 0);
  const uint32_t pair = blockIdx.x >> 1;
  const uint32_t num_pairs = gridDim.x >> 1;
  const uint32_t rounds = (p.num_kblocks + SUB - 1) / SUB;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (uint32_t a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 8);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tmap(&tm_a);
    ptx::prefetch_tmap(&tm_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();  // the peer's barriers and TMEM exist before anyone signals them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above touched no global memory: from here on the previous kernel's results
  // are needed (and its reads of our output buffers must be over)
  ptx::grid_dependency_release();
  ptx::grid_dependency_wait();

  if constexpr (GATED) {
    if (p.sh.trace && blockIdx.x == 0 && threadIdx.x == 0) p.sh.trace[0] = ptx::globaltimer_ns();
  }
  // i-th tile of this pair (>= num_tiles: done)
  auto tile_at = [&](uint32_t i) -> uint32_t {
    if constexpr (GATED) return gated_tile_at(p.sh, pair, num_pairs, i);
    else return pair + i * num_pairs;
  };
  if constexpr (GATED) {
    // ------------------------------------------- sending pairs (owner of B only)
    constexpr uint32_t WARPS = GATED_THREADS / 32;
    const uint32_t early = num_pairs - p.sh.sender_pairs;
    const uint32_t sender_ctas = 2u * p.sh.sender_pairs;
    const uint32_t groups = min(SENDER_GROUPS, sender_ctas);
    const bool watched = early > 0;  // a CTA that sends nothing exists and watches the counters
    if (pair >= early) {
      const uint32_t c = (pair - early) * 2u + cta_rank;  // among the sending CTAs
      push_b_slabs(p.sh, c % groups, groups, (c / groups) * WARPS + warp,
                   sender_group_warps(sender_ctas, groups, c % groups, WARPS), c * WARPS + warp,
                   sender_ctas * WARPS, lane, !watched, p.status);
      __syncthreads();
    } else if (p.sh.sender_pairs && blockIdx.x == 0 && warp == 6) {
      publish_slabs(p.sh, sender_ctas, groups, WARPS, lane);
    }
  }

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    uint32_t stage = 0, phase = 0;
    bool alive = true;
    uint32_t slabs_seen = 0;  // GATED: column slabs of B known to have arrived (bit per slab)
    for (uint32_t i = 0, t = tile_at(0); alive && t < p.num_tiles; t = tile_at(++i)) {
      uint32_t tm, tn;
      tile_coords(p, t, tm, tn);
      const int32_t a_tile = int32_t(tm * 2 + cta_rank);  // in units of 128 rows
      const int32_t b_tile = int32_t(tn * 2 + cta_rank);  // in units of BLOCK_N/2 columns
      if constexpr (GATED) {
        const uint32_t slab = tn / p.sh.slab_tiles;
        if (!((slabs_seen >> slab) & 1u)) {
          bool here = true;
          if (lane == 0) {
            here = ptx::flag_wait(&shard_ctrl(p.sh, p.sh.rank)->arrived[p.sh.slot][slab], p.sh.epoch,
                                  abort_flag, ptx::kDataWaitLimitNs);
            // the slab was written by another GPU's stores: order the flag's acquire before
            // this thread's TMA loads of the slab
            ptx::fence_proxy_async_global();
            if (p.sh.trace) atomicMin(&p.sh.trace[40 + slab], ptx::globaltimer_ns());
          }
          if (!__all_sync(0xffffffffu, here)) {
            if (lane == 0) {
              if (first_to_give_up(abort_flag)) report(p.status, 6, slab, t, p.sh.epoch);
            }
            alive = false;
            break;
          }
          slabs_seen |= 1u << slab;
        }
      }
      for (uint32_t rd = 0; rd < rounds; ++rd) {
        bool ok = ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) {
            if (first_to_give_up(abort_flag)) report(p.status, 1, stage, t, rd);
          }
          alive = false;
          break;
        }
        if (lane == 0) {
          if (leader) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
          const uint32_t fb = ptx::mapa_shared(full_bar(stage), 0);  // the leader's barrier
          // stage layout: A of k blocks 0..SUB-1, then B of k blocks 0..SUB-1
          // (k blocks past the end of K are fetched too: TMA fills them with zeros)
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + SUB * A_TILE_BYTES;
          const int32_t kb0 = int32_t(rd * SUB);
          if (p.a.kgroup) {
            ptx::tma_load_3d_pair(a_dst, &tm_a, 0, a_tile * p.a.c1_tile, kb0, fb);
          } else {
#pragma unroll
            for (uint32_t j = 0; j < SUB; ++j)
              load_operand<true>(p.a, &tm_a, a_dst + j * A_TILE_BYTES, a_tile, kb0 + int32_t(j), 0, fb);
          }
          if (p.b.kgroup) {
            ptx::tma_load_3d_pair(b_dst, &tm_b, 0, b_tile * p.b.c1_tile, kb0, fb);
          } else {
#pragma unroll
            for (uint32_t j = 0; j < SUB; ++j)
              load_operand<true>(p.b, &tm_b, b_dst + j * B_TILE_BYTES, b_tile, kb0 + int32_t(j), 0, fb);
          }
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------- MMA issuer (leader CTA only)
    // One thread runs the loop: the next stage's barrier is tested (without
    // blocking) before this round's MMAs are issued and only waited on when
    // that test failed; descriptors advance by 32-bit adds on their low words.
    if (leader && lane == 0) {
      const uint32_t a_hi = uint32_t(p.a.desc >> 32), b_hi = uint32_t(p.b.desc >> 32);
      const uint32_t a_lo0 = uint32_t(p.a.desc), b_lo0 = uint32_t(p.b.desc);
      const uint32_t a_step = p.a.kstep_bytes >> 4, b_step = p.b.kstep_bytes >> 4;
      uint32_t stage = 0, phase = 0;
      uint32_t local = 0;
      uint32_t ready = 0;
      bool alive = true;
      for (uint32_t t = tile_at(0); alive && t < p.num_tiles; t = tile_at(++local)) {
        const uint32_t acc = local & 1u;
        const uint32_t acc_phase = (local >> 1) & 1u;
        if (!ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
          if (first_to_give_up(abort_flag)) report(p.status, 2, 0x100u | acc, t, 0);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
        for (uint32_t rd = 0; rd < rounds; ++rd) {
          if (!ready && !ptx::mbar_wait(full_bar(stage), phase, abort_flag)) {
            if (first_to_give_up(abort_flag)) report(p.status, 2, stage, t, rd);
            alive = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t next_stage = (stage + 1 == STAGES) ? 0 : stage + 1;
          const uint32_t next_phase = (stage + 1 == STAGES) ? phase ^ 1u : phase;
          const uint32_t ready_next = ptx::mbar_test_wait(full_bar(next_stage), next_phase);
#pragma unroll
          for (uint32_t j = 0; j < SUB; ++j) {
            const uint32_t st = smem_base + stage * STAGE_BYTES;
            const uint32_t a_lo = a_lo0 + ((st + j * A_TILE_BYTES) >> 4);
            const uint32_t b_lo = b_lo0 + ((st + SUB * A_TILE_BYTES + j * B_TILE_BYTES) >> 4);
#pragma unroll
            for (uint32_t ks = 0; ks < KSTEPS; ++ks) {
              ptx::mma_f16_pair_lohi(d_tmem, a_lo + ks * a_step, a_hi, b_lo + ks * b_step, b_hi,
                                     p.idesc, (rd | j | ks) ? 1u : 0u);
            }
          }
          ptx::mma_commit_pair(empty_bar(stage), 3);
          if (rd + 1 == rounds) ptx::mma_commit_pair(tfull_bar(acc), 3);
          stage = next_stage;
          phase = next_phase;
          ready = ready_next;
        }
      }
    }
  } else if (warp >= 6) {
    // (the extra warps of the gated product only take part in sending)
  } else {
    // ------------------------------------------------------------ epilogue
    const uint32_t quarter = warp & 3u;
    uint32_t local = 0;
    for (uint32_t t = tile_at(0); t < p.num_tiles; t = tile_at(++local)) {
      const uint32_t acc = local & 1u;
      const uint32_t acc_phase = (local >> 1) & 1u;
      uint32_t tm, tn;
      tile_coords(p, t, tm, tn);
      bool ok = ptx::mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) {
          if (first_to_give_up(abort_flag)) report(p.status, 3, acc, t, 0);
        }
        break;
      }
      ptx::tc_fence_after();
      const uint32_t row = (tm * 2 + cta_rank) * BLOCK_M + quarter * 32u + lane;
      const uint32_t col_tile = tn * BLOCK_N;
      const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * BLOCK_N;
#pragma unroll 1
      for (uint32_t ch = 0; ch < BLOCK_N / 32; ++ch) {
        const uint32_t col0 = col_tile + ch * 32u;
        if (col0 >= p.N) break;
        uint32_t r[32];
        ptx::tmem_ld_32x32(taddr + ch * 32u, r);
        ptx::tmem_ld_wait();
        epilogue_store32(p, r, row, col0);
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa_shared(tempty_bar(acc), 0));
    }
  }

  // ---------------------------------------------------------------- teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = ptx::globaltimer_ns();
    for (uint32_t i = 0; i < (1u << 16); ++i) {
      if (ptx::globaltimer_ns() - t0 > 2000000ull) break;
      __nanosleep(1000);
    }
    __syncthreads();
  }
  // Neither CTA may leave while the other can still signal its barriers or the
  // pair's MMAs can still touch its shared memory and TMEM.
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  // every load of B this CTA issued has landed and been consumed
  if (GATED && threadIdx.x == 0) shard_exit(p.sh, *abort_flag != 0u);
}

// The same 32 x 32 block of results, written so that a warp's store instruction
// covers whole rows: the 32 threads (one output row each) put their raw
// accumulators into a 4 KB staging tile in shared memory (16-byte chunks XOR-ed
// with the row, so neither side has bank conflicts), then each instruction takes
// four rows x 128 bytes back out, applies alpha/beta/bias/activation and stores.
// A row-per-thread store instruction touches 32 different lines and the
// load/store unit handles them one by one; for the one-tile-per-CTA products of
// the small shapes that serial tail was a fifth of the kernel.
// `row_base` is the first of the warp's 32 rows within M, `grow_base` the same
// row in the (possibly batch-stacked) C.  All 32 lanes must call.
__device__ __forceinline__ void epilogue_store32_coalesced(const KernelParams& p,
                                                           const uint32_t (&r)[32], uint32_t staging,
                                                           uint32_t row_base, uint64_t grow_base,
                                                           uint32_t col0, uint32_t lane) {
  if (row_base >= p.M || col0 >= p.N) return;  // the same for the whole warp
#pragma unroll
  for (uint32_t j = 0; j < 8; ++j) {
    const uint32_t addr = staging + lane * 128u + ((j ^ (lane & 7u)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(r[4 * j]), "r"(r[4 * j + 1]),
                 "r"(r[4 * j + 2]), "r"(r[4 * j + 3]) : "memory");
  }
  __syncwarp();
  if (p.vec_store) {
    const uint32_t q = lane & 7u, rsub = lane >> 3;
    const uint32_t col = col0 + q * 4u;
#pragma unroll
    for (uint32_t it = 0; it < 8; ++it) {
      const uint32_t rl = it * 4u + rsub;
      float4 v;
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                   : "r"(staging + rl * 128u + ((q ^ (rl & 7u)) << 4)));
      if (row_base + rl >= p.M || col >= p.N) continue;
      float* c = p.C + (grow_base + rl) * p.ldc + col;
      const float* cin = p.c_in ? p.c_in + (grow_base + rl) * p.ldc + col : nullptr;
      if (col + 4u <= p.N) {
        *reinterpret_cast<float4*>(c) = epilogue_value4(p, v, cin, p.bias ? p.bias + col : nullptr);
      } else {
        const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (uint32_t k = 0; k < 4; ++k) {
          if (col + k < p.N)
            c[k] = epilogue_value(p, e[k], cin ? cin + k : nullptr, p.bias ? p.bias + col + k : nullptr);
        }
      }
    }
  } else {
    const uint32_t col = col0 + lane;
#pragma unroll 4
    for (uint32_t rl = 0; rl < 32; ++rl) {
      float x;
      asm volatile("ld.shared.f32 %0, [%1];"
                   : "=f"(x)
                   : "r"(staging + rl * 128u + (((lane >> 2) ^ (rl & 7u)) << 4) + (lane & 3u) * 4u));
      if (row_base + rl >= p.M || col >= p.N) continue;
      p.C[(grow_base + rl) * p.ldc + col] =
          epilogue_value(p, x, p.c_in ? p.c_in + (grow_base + rl) * p.ldc + col : nullptr,
                         p.bias ? p.bias + col : nullptr);
    }
  }
  __syncwarp();  // the staging tile may be overwritten by the next block
}

// ---------------------------------------------------------------------------
// fp16 kernel for the largest problems: CTA pairs on 512 x 256 tiles.
//
// Measured on B200: TMA loads deliver at most ~46 bytes per clock per SM from
// L2 however many stages are in flight, and the 256 x 256 pair tile needs 64
// per clock at full tensor rate, so that kernel tops out near 70 % of the
// pipe.  Here each CTA of the pair carries TWO 128-row A sub-tiles against the
// same B half tile: 48 KB per k block feed 8 MMAs (1024 cycles), 48 bytes per
// clock.  The two 256-column accumulators fill TMEM, so they cannot be double
// buffered; instead sub-tile 0 is committed and drained first, and the next
// tile's sub-tile-0 MMAs start while sub-tile 1 is still draining.
//
// Barriers: full[s] (leader), empty[s] (both), tfull[u] (both, u = sub-tile),
// tempty[u] (leader, 8 arrivals = 4 epilogue warps of each CTA).
template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_f16_pair512_kernel(const __grid_constant__ CUtensorMap tm_a,
                        const __grid_constant__ CUtensorMap tm_b,
                        const __grid_constant__ KernelParams p) {
  constexpr uint32_t BN = 256;
  constexpr uint32_t B_TILE_BYTES = (BN / 2) * SLAB_ROW_BYTES;
  constexpr uint32_t STAGE_BYTES = 2 * A_TILE_BYTES + B_TILE_BYTES;  // A0, A1, B half
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t cta_rank = ptx::cluster_ctarank();
  const bool leader = (cta_rank == 0);
  const uint32_t pair = blockIdx.x >> 1;
  const uint32_t num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (uint32_t a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 8);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tmap(&tm_a);
    ptx::prefetch_tmap(&tm_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above touched no global memory: from here on the previous kernel's results
  // are needed (and its reads of our output buffers must be over)
  ptx::grid_dependency_release();
  ptx::grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    uint32_t stage = 0, phase = 0;
    bool alive = true;
    for (uint32_t t = pair; alive && t < p.num_tiles; t += num_pairs) {
      uint32_t tm, tn;
      tile_coords(p, t, tm, tn);
      const int32_t b_tile = int32_t(tn * 2 + cta_rank);  // units of 128 columns
      for (uint32_t kb = 0; kb < p.num_kblocks; ++kb) {
        bool ok = ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) {
            if (first_to_give_up(abort_flag)) report(p.status, 1, stage, t, kb);
          }
          alive = false;
          break;
        }
        if (lane == 0) {
          if (leader) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
          const uint32_t fb = ptx::mapa_shared(full_bar(stage), 0);
          uint32_t dst = smem_base + stage * STAGE_BYTES;
#pragma unroll
          for (uint32_t u = 0; u < 2; ++u) {
            const int32_t a_tile = int32_t(tm * 4 + u * 2 + cta_rank);  // units of 128 rows
            load_operand<true>(p.a, &tm_a, dst, a_tile, int32_t(kb), 0, fb);
            dst += A_TILE_BYTES;
          }
          load_operand<true>(p.b, &tm_b, dst, b_tile, int32_t(kb), 0, fb);
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  }
  else if (warp == 1) {
    // ------------------------------------------- MMA issuer (leader CTA only)
    // One thread runs the whole loop.  Issuing a tcgen05.mma is not free (about
    // 90 cycles each, measured), so everything else in a round has to fit in
    // the ~300 cycles that 8 MMAs of 128 cycles leave: the next stage's barrier
    // is peeked at with a non-blocking test BEFORE this round's MMAs are issued
    // and only waited on if that test failed; descriptors are advanced with
    // 32-bit adds on their low words.
    if (leader && lane == 0) {
      const uint32_t a_hi = uint32_t(p.a.desc >> 32), b_hi = uint32_t(p.b.desc >> 32);
      const uint32_t a_lo0 = uint32_t(p.a.desc), b_lo0 = uint32_t(p.b.desc);
      const uint32_t a_step = p.a.kstep_bytes >> 4, b_step = p.b.kstep_bytes >> 4;
      uint32_t stage = 0, phase = 0;
      uint32_t local = 0;
      bool alive = true;
      uint32_t ready = 0;
      for (uint32_t t = pair; alive && t < p.num_tiles; t += num_pairs, ++local) {
        const uint32_t tparity = local & 1u;
        for (uint32_t kb = 0; kb < p.num_kblocks; ++kb) {
          if (!ready && !ptx::mbar_wait(full_bar(stage), phase, abort_flag)) {
            if (first_to_give_up(abort_flag)) report(p.status, 2, stage, t, kb);
            alive = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t next_stage = (stage + 1 == STAGES) ? 0 : stage + 1;
          const uint32_t next_phase = (stage + 1 == STAGES) ? phase ^ 1u : phase;
          const uint32_t ready_next = ptx::mbar_test_wait(full_bar(next_stage), next_phase);
          const uint32_t stage_addr = smem_base + stage * STAGE_BYTES;
          const uint32_t b_lo = b_lo0 + ((stage_addr + 2 * A_TILE_BYTES) >> 4);
#pragma unroll
          for (uint32_t u = 0; u < 2; ++u) {
            if (kb == 0) {
              // accumulator u must have been drained of the previous tile
              if (!ptx::mbar_wait(tempty_bar(u), tparity ^ 1u, abort_flag)) {
                if (first_to_give_up(abort_flag)) report(p.status, 2, 0x100u | u, t, 0);
                alive = false;
                break;
              }
              ptx::tc_fence_after();
            }
            const uint32_t a_lo = a_lo0 + ((stage_addr + u * A_TILE_BYTES) >> 4);
            const uint32_t d_tmem = tmem_base + u * BN;
#pragma unroll
            for (uint32_t ks = 0; ks < KSTEPS; ++ks) {
              ptx::mma_f16_pair_lohi(d_tmem, a_lo + ks * a_step, a_hi, b_lo + ks * b_step, b_hi,
                                     p.idesc, (kb | ks) ? 1u : 0u);
            }
            if (kb + 1 == p.num_kblocks) ptx::mma_commit_pair(tfull_bar(u), 3);
          }
          if (!alive) break;
          ptx::mma_commit_pair(empty_bar(stage), 3);
          stage = next_stage;
          phase = next_phase;
          ready = ready_next;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const uint32_t quarter = warp & 3u;
    uint32_t local = 0;
    bool alive = true;
    for (uint32_t t = pair; alive && t < p.num_tiles; t += num_pairs, ++local) {
      uint32_t tm, tn;
      tile_coords(p, t, tm, tn);
#pragma unroll 1
      for (uint32_t u = 0; u < 2; ++u) {
        bool ok = ptx::mbar_wait(tfull_bar(u), local & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) {
            if (first_to_give_up(abort_flag)) report(p.status, 3, u, t, 0);
          }
          alive = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t row0 = (tm * 4 + u * 2 + cta_rank) * BLOCK_M + quarter * 32u;
        const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + u * BN;
#pragma unroll 1
        for (uint32_t ch = 0; ch < BN / 32; ++ch) {
          const uint32_t col0 = tn * BN + ch * 32u;
          if (col0 >= p.N) break;
          uint32_t r[32];
          ptx::tmem_ld_32x32(taddr + ch * 32u, r);
          ptx::tmem_ld_wait();
          epilogue_store32(p, r, row0 + lane, col0);
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa_shared(tempty_bar(u), 0));
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = ptx::globaltimer_ns();
    for (uint32_t i = 0; i < (1u << 16); ++i) {
      if (ptx::globaltimer_ns() - t0 > 2000000ull) break;
      __nanosleep(1000);
    }
    __syncthreads();
  }
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// fp32-accurate variant: three tf32 MMAs per k step on (hi, lo) planes, with
// the TMEM accumulator PROMOTED to fp32 registers every CHUNK_KB k blocks.
//
// Why: the tensor core adds into its fp32 accumulator with truncation, so the
// error of a long K loop grows linearly with the number of MMAs (measured:
// 3.6e-6 relative at K=512, which would pass 1e-5 near K=1500).  Here an
// accumulator only ever holds CHUNK_KB*32 values of K; the epilogue warps drain
// it with tcgen05.ld and add it to running sums with round-to-nearest fp32
// adds, so the error no longer depends on K.  The two TMEM accumulators
// alternate per chunk, which also overlaps the drain with the next chunk's MMAs.
//
// 10 warps: 0 producer, 1 MMA issuer, 2-9 drain/epilogue (warp w reads TMEM
// lanes 32*(w%4).., and columns half (w-2)/4 of the tile).
constexpr uint32_t TF32_THREADS = 320;
constexpr uint32_t CHUNK_KB = 4;  // k blocks (of 32) per TMEM accumulation chunk

template <int NC>
__device__ __forceinline__ void drain_add(uint32_t taddr, float (&sums)[NC]) {
  static_assert(NC % 32 == 0 || NC == 16, "columns per thread");
  if constexpr (NC == 16) {
    uint32_t r[16];
    ptx::tmem_ld_32x16(taddr, r);
    ptx::tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 16; ++i) sums[i] += __uint_as_float(r[i]);
  } else {
#pragma unroll
    for (int j = 0; j < NC / 32; ++j) {
      uint32_t r[32];
      ptx::tmem_ld_32x32(taddr + j * 32, r);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) sums[j * 32 + i] += __uint_as_float(r[i]);
    }
  }
}

template <int BLOCK_N, int STAGES>
__global__ void __launch_bounds__(TF32_THREADS, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tm_a0,
                   const __grid_constant__ CUtensorMap tm_a1,
                   const __grid_constant__ CUtensorMap tm_b0,
                   const __grid_constant__ CUtensorMap tm_b1,
                   const __grid_constant__ KernelParams p) {
  constexpr uint32_t B_TILE_BYTES = BLOCK_N * SLAB_ROW_BYTES;
  constexpr uint32_t STAGE_BYTES = 2 * (A_TILE_BYTES + B_TILE_BYTES);
  constexpr uint32_t TMEM_COLS = (2 * BLOCK_N < 64) ? 64 : 2 * BLOCK_N;
  constexpr int NC = BLOCK_N / 2;  // columns per drain thread
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t sk_all_bar = bar_base + 8u * (2 * STAGES + 4);   // split-K: partials written
  const uint32_t sk_lead_bar = bar_base + 8u * (2 * STAGES + 5);  // split-K: outcome published
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 6);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* sk_flag = tmem_slot + 2;
  // Epilogue staging, one 4 KB tile per drain warp: the first 32 KB of the pipeline
  // stages, used only by a CTA's LAST work unit (by then the producer has issued its
  // last load and every MMA that reads the stages has retired).
  const uint32_t staging_base = smem_base;
  static_assert(STAGES * STAGE_BYTES >= 8 * 4096, "staging tiles fit in the stages");

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (uint32_t a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 8);  // one arrival per drain warp
    }
    ptx::mbar_init(sk_all_bar, 8);
    ptx::mbar_init(sk_lead_bar, 1);
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tmap(&tm_a0);
    ptx::prefetch_tmap(&tm_a1);
    ptx::prefetch_tmap(&tm_b0);
    ptx::prefetch_tmap(&tm_b1);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Nothing above touched global memory.  The previous kernel's results are needed (and its
  // reads of our output buffers and of the split-K workspace must be over) only where a role
  // first touches global memory: the producer's first load, the drain warps' first store.
  // Each waits there, so that fetching the kernel parameters and the first tile's index
  // arithmetic (about 1.3 us between the end of the wait and the first load, measured with
  // %globaltimer) overlap the previous kernel's tail.
  ptx::grid_dependency_release();
  // work units: unit u is split (u % splits) of tile (u / splits); splits == 1 is one unit per tile
  const uint32_t num_units = p.num_tiles * p.splits;
  auto unit_range = [&](uint32_t u, uint32_t& t, uint32_t& kb_lo, uint32_t& kb_hi) {
    t = u / p.splits;
    kb_lo = (u - t * p.splits) * p.kb_per_split;
    kb_hi = min(kb_lo + p.kb_per_split, p.num_kblocks);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    uint32_t stage = 0, phase = 0;
    bool alive = true;
    bool waited = false;
    for (uint32_t u = blockIdx.x; alive && u < num_units; u += gridDim.x) {
      uint32_t t, kb_lo, kb_hi;
      unit_range(u, t, kb_lo, kb_hi);
      uint32_t tm, tn;
      uint32_t bt;
      tile_coords(p, t, tm, tn, bt);
      for (uint32_t kb = kb_lo; kb < kb_hi; ++kb) {
        bool ok = ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) {
            if (first_to_give_up(abort_flag)) report(p.status, 1, stage, t, kb);
          }
          alive = false;
          break;
        }
        if (lane == 0) {
          const uint32_t fb = full_bar(stage);
          if (!waited) {
            ptx::grid_dependency_wait();
            waited = true;
          }
          ptx::mbar_arrive_expect_tx(fb, STAGE_BYTES);
          uint32_t dst = smem_base + stage * STAGE_BYTES;
#pragma unroll
          for (uint32_t pl = 0; pl < 2; ++pl) {
            load_operand<false>(p.a, pl ? &tm_a1 : &tm_a0, dst, int32_t(tm), int32_t(kb),
                                int32_t(bt) * p.a_batch_c1, fb);
            dst += A_TILE_BYTES;
          }
#pragma unroll
          for (uint32_t pl = 0; pl < 2; ++pl) {
            load_operand<false>(p.b, pl ? &tm_b1 : &tm_b0, dst, int32_t(tn), int32_t(kb),
                                int32_t(bt) * p.b_batch_c1, fb);
            dst += B_TILE_BYTES;
          }
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------- MMA issuer: one thread
    // The next stage's barrier is tested without blocking before this stage's
    // MMAs go out, and descriptors advance by 32-bit adds, so that issuing a
    // 64-cycle MMA costs the thread less than the MMA takes.
    if (lane == 0) {
      const uint32_t a_hi32 = uint32_t(p.a.desc >> 32), b_hi32 = uint32_t(p.b.desc >> 32);
      const uint32_t a_lo0 = uint32_t(p.a.desc), b_lo0 = uint32_t(p.b.desc);
      const uint32_t a_step = p.a.kstep_bytes >> 4, b_step = p.b.kstep_bytes >> 4;
      uint32_t stage = 0, phase = 0;
      uint32_t chunk = 0;  // running chunk count: selects accumulator and barrier parity
      uint32_t ready = 0;
      bool alive = true;
      for (uint32_t u = blockIdx.x; alive && u < num_units; u += gridDim.x) {
        uint32_t t, kb_lo, kb_hi;
        unit_range(u, t, kb_lo, kb_hi);
        for (uint32_t kb0 = kb_lo; alive && kb0 < kb_hi; kb0 += CHUNK_KB, ++chunk) {
          const uint32_t acc = chunk & 1u;
          const uint32_t acc_phase = (chunk >> 1) & 1u;
          if (!ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
            if (first_to_give_up(abort_flag)) report(p.status, 2, 0x100u | acc, t, kb0);
            alive = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
          const uint32_t kb_end = min(kb0 + CHUNK_KB, kb_hi);
          for (uint32_t kb = kb0; kb < kb_end; ++kb) {
            if (!ready && !ptx::mbar_wait(full_bar(stage), phase, abort_flag)) {
              if (first_to_give_up(abort_flag)) report(p.status, 2, stage, t, kb);
              alive = false;
              break;
            }
            ptx::tc_fence_after();
            const uint32_t next_stage = (stage + 1 == STAGES) ? 0 : stage + 1;
            const uint32_t next_phase = (stage + 1 == STAGES) ? phase ^ 1u : phase;
            const uint32_t ready_next = ptx::mbar_test_wait(full_bar(next_stage), next_phase);
            const uint32_t st = smem_base + stage * STAGE_BYTES;
            const uint32_t ah = a_lo0 + (st >> 4), al = a_lo0 + ((st + A_TILE_BYTES) >> 4);
            const uint32_t bh = b_lo0 + ((st + 2 * A_TILE_BYTES) >> 4);
            const uint32_t bl = b_lo0 + ((st + 2 * A_TILE_BYTES + B_TILE_BYTES) >> 4);
#pragma unroll
            for (uint32_t ks = 0; ks < KSTEPS; ++ks) {
              const uint32_t accum = ((kb - kb0) | ks) ? 1u : 0u;
              ptx::mma_tf32_lohi(d_tmem, al + ks * a_step, a_hi32, bh + ks * b_step, b_hi32, p.idesc, accum);
              ptx::mma_tf32_lohi(d_tmem, ah + ks * a_step, a_hi32, bl + ks * b_step, b_hi32, p.idesc, 1u);
              ptx::mma_tf32_lohi(d_tmem, ah + ks * a_step, a_hi32, bh + ks * b_step, b_hi32, p.idesc, 1u);
            }
            ptx::mma_commit(empty_bar(stage));
            if (kb + 1 == kb_end) ptx::mma_commit(tfull_bar(acc));
            stage = next_stage;
            phase = next_phase;
            ready = ready_next;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------- drain + epilogue warps
    const uint32_t quarter = warp & 3u;
    const uint32_t half = (warp - 2u) >> 2;  // which half of the tile's columns
    uint32_t chunk = 0;
    uint32_t sk_parity = 0;
    const uint32_t tid_d = threadIdx.x - 64u;  // 0..255 among the drain threads
    bool alive = true;
    bool waited = false;
    for (uint32_t u = blockIdx.x; alive && u < num_units; u += gridDim.x) {
      uint32_t t, kb_lo, kb_hi;
      unit_range(u, t, kb_lo, kb_hi);
      const uint32_t chunks_per_tile = (kb_hi - kb_lo + CHUNK_KB - 1) / CHUNK_KB;
      uint32_t tm, tn;
      uint32_t bt;
      tile_coords(p, t, tm, tn, bt);
      float sums[NC];
#pragma unroll
      for (int i = 0; i < NC; ++i) sums[i] = 0.f;
      for (uint32_t c = 0; c < chunks_per_tile; ++c, ++chunk) {
        const uint32_t acc = chunk & 1u;
        const uint32_t acc_phase = (chunk >> 1) & 1u;
        bool ok = ptx::mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) {
            if (first_to_give_up(abort_flag)) report(p.status, 3, acc, t, c);
          }
          alive = false;
          break;
        }
        ptx::tc_fence_after();
        drain_add<NC>(tmem_base + ((quarter * 32u) << 16) + acc * BLOCK_N + half * NC, sums);
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
      }
      if (!alive) break;
      if (!waited) {
        ptx::grid_dependency_wait();
        waited = true;
      }
      if (p.splits > 1) {
        // Partial sums to the workspace, [unit][4 columns][thread] so that a warp's
        // 16-byte stores are contiguous; then the tile's counter says who came last.
        float4* mine = reinterpret_cast<float4*>(p.sk_ws) + size_t(u) * (NC / 4) * 256u;
#pragma unroll
        for (int j = 0; j < NC / 4; ++j)
          __stcg(mine + j * 256 + tid_d, make_float4(sums[4 * j], sums[4 * j + 1], sums[4 * j + 2], sums[4 * j + 3]));
        __threadfence();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(sk_all_bar);
        if (warp == 2) {
          bool all_in = ptx::mbar_wait(sk_all_bar, sk_parity, abort_flag);
          all_in = __all_sync(0xffffffffu, all_in);
          if (lane == 0) {
            uint32_t outcome = 2u;  // 2 = gave up
            if (all_in) {
              const uint32_t before = atomicAdd(p.sk_count + t, 1u);
              outcome = (before + 1u == p.splits) ? 1u : 0u;
              if (outcome) p.sk_count[t] = 0u;  // nobody else touches this tile again: ready for the next launch
            } else {
              if (first_to_give_up(abort_flag)) report(p.status, 3, 0x200u, t, 0);
            }
            *sk_flag = outcome;
            ptx::mbar_arrive(sk_lead_bar);
          }
        }
        bool ok = ptx::mbar_wait(sk_lead_bar, sk_parity, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        sk_parity ^= 1u;
        const uint32_t outcome = *sk_flag;
        if (!ok || outcome == 2u) {
          if (lane == 0 && !ok) {
            if (first_to_give_up(abort_flag)) report(p.status, 3, 0x201u, t, 0);
          }
          alive = false;
          break;
        }
        if (outcome == 0u) continue;  // another unit of this tile finishes it
        __threadfence();
        // the last unit adds the partial sums in split order: the result does not
        // depend on which unit came last
#pragma unroll
        for (int i = 0; i < NC; ++i) sums[i] = 0.f;
        const float4* part = reinterpret_cast<const float4*>(p.sk_ws) + size_t(t) * p.splits * (NC / 4) * 256u;
        for (uint32_t sp = 0; sp < p.splits; ++sp, part += (NC / 4) * 256u) {
#pragma unroll
          for (int j = 0; j < NC / 4; ++j) {
            const float4 v = __ldcg(part + j * 256 + tid_d);
            sums[4 * j] += v.x;
            sums[4 * j + 1] += v.y;
            sums[4 * j + 2] += v.z;
            sums[4 * j + 3] += v.w;
          }
        }
      }
      const uint32_t row_base = tm * BLOCK_M + quarter * 32u;        // within its batch
      const uint64_t grow_base = uint64_t(bt) * p.M + row_base;      // in the stacked C
      const uint32_t col0 = tn * BLOCK_N + half * NC;
      const uint32_t row = row_base + lane;
      if (col0 + NC <= p.N && p.vec_store) {
        // whole, aligned row segment: 16-byte stores from the row's own thread
        if (row < p.M) {
          float* c_row = p.C + (grow_base + lane) * p.ldc;
          const float* cin_row = p.c_in ? p.c_in + (grow_base + lane) * p.ldc : nullptr;
#pragma unroll
          for (int j = 0; j < NC; j += 4) {
            const float4 v = make_float4(sums[j + 0], sums[j + 1], sums[j + 2], sums[j + 3]);
            *reinterpret_cast<float4*>(c_row + col0 + j) =
                epilogue_value4(p, v, cin_row ? cin_row + col0 + j : nullptr,
                                p.bias ? p.bias + col0 + j : nullptr);
          }
        }
      } else if (NC >= 32 && u + gridDim.x >= num_units) {
        // Ragged or unaligned columns on the CTA's last unit: a row-per-thread scalar
        // store touches 32 lines per instruction, which the load/store unit handles one
        // by one (measured: 43 against 35 us for N = 784 against N = 768); the staging
        // tile turns them into whole-row stores.
        const uint32_t staging = staging_base + (warp - 2u) * 4096u;
#pragma unroll
        for (int j = 0; j < (NC >= 32 ? NC / 32 : 0); ++j) {
          uint32_t r[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(sums[(j * 32 + i) % NC]);
          epilogue_store32_coalesced(p, r, staging, row_base, grow_base, col0 + j * 32, lane);
        }
      } else if (row < p.M && col0 < p.N) {
        float* c_row = p.C + (grow_base + lane) * p.ldc;
        const float* cin_row = p.c_in ? p.c_in + (grow_base + lane) * p.ldc : nullptr;
#pragma unroll
        for (int j = 0; j < NC; ++j) {
          const uint32_t col = col0 + j;
          if (col < p.N)
            c_row[col] = epilogue_value(p, sums[j], cin_row ? cin_row + col : nullptr,
                                        p.bias ? p.bias + col : nullptr);
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = ptx::globaltimer_ns();
    for (uint32_t i = 0; i < (1u << 16); ++i) {
      if (ptx::globaltimer_ns() - t0 > 2000000ull) break;
      __nanosleep(1000);
    }
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// fp32-accurate variant on CTA pairs: chunked promotion as in gemm_tf32x3_kernel, the 2-SM MMA
// (M=256) of the fp16 pair kernel, and the two correction products (hi.lo + lo.hi) taken from
// bf16 planes instead of tf32 ones.  They are 2^-11 of the product, so 8 bits of them are
// enough for fp32-grade results (measured 8.8e-7 relative Frobenius error against float64 at
// K = 4096, the same as with tf32 corrections: the accumulation dominates), and the bf16 MMA
// runs at twice the tf32 rate: 4 tf32 + 4 bf16 MMAs per k block of 32 - the tensor-pipe time
// of 8 tf32 MMAs - instead of 12.  Each CTA stages its 128 rows of A and its half of the B
// tile: hi as fp32 (16 KB each) and, through one map per operand that covers both bf16 planes
// (last dimension = plane), bf16(hi) and bf16(lo) (8 KB each), one box per k block:
//   K-major operand: box (32 of K = 64 bytes, 128 rows, 2 planes), 64-byte swizzle;
//   MN-major:        box (64 of MN = 128 bytes, 32 rows of K, 2 slabs, 2 planes).
// 64 KB per k block and CTA.  8 drain warps per CTA.
//   full[s] leader; empty[s] both; tfull[a] both; tempty[a] leader, 16 arrivals.
template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TF32_THREADS, 1)
gemm_tf32x3_pair_kernel(const __grid_constant__ CUtensorMap tm_a0,
                        const __grid_constant__ CUtensorMap tm_a1,
                        const __grid_constant__ CUtensorMap tm_b0,
                        const __grid_constant__ CUtensorMap tm_b1,
                        const __grid_constant__ KernelParams p) {
  constexpr uint32_t BN = 256;
  constexpr uint32_t B_TILE_BYTES = (BN / 2) * SLAB_ROW_BYTES;  // this CTA's half, one plane
  constexpr uint32_t STAGE_BYTES = 2 * (A_TILE_BYTES + B_TILE_BYTES);
  constexpr uint32_t X_PLANE_BYTES = A_TILE_BYTES / 2;  // one bf16 tile: 128 rows/columns x 32 of K
  static_assert(A_TILE_BYTES == B_TILE_BYTES, "the bf16 planes of A and B tiles are the same size");
  constexpr uint32_t TMEM_COLS = 512;
  constexpr int NC = BN / 2;  // columns per drain thread

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](uint32_t a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t cta_rank = ptx::cluster_ctarank();
  const bool leader = (cta_rank == 0);
  const uint32_t pair = blockIdx.x >> 1;
  const uint32_t num_pairs = gridDim.x >> 1;
  const uint32_t chunks_per_tile = (p.num_kblocks + CHUNK_KB - 1) / CHUNK_KB;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (uint32_t a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 16);  // 8 drain warps of each CTA
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tmap(&tm_a0);
    ptx::prefetch_tmap(&tm_a1);
    ptx::prefetch_tmap(&tm_b0);
    ptx::prefetch_tmap(&tm_b1);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above touched no global memory: from here on the previous kernel's results
  // are needed (and its reads of our output buffers must be over)
  ptx::grid_dependency_release();
  ptx::grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    uint32_t stage = 0, phase = 0;
    bool alive = true;
    for (uint32_t t = pair; alive && t < p.num_tiles; t += num_pairs) {
      uint32_t tm, tn;
      tile_coords(p, t, tm, tn);
      const int32_t a_tile = int32_t(tm * 2 + cta_rank);
      const int32_t b_tile = int32_t(tn * 2 + cta_rank);
      for (uint32_t kb = 0; kb < p.num_kblocks; ++kb) {
        bool ok = ptx::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) {
            if (first_to_give_up(abort_flag)) report(p.status, 1, stage, t, kb);
          }
          alive = false;
          break;
        }
        if (lane == 0) {
          if (leader) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
          const uint32_t fb = ptx::mapa_shared(full_bar(stage), 0);
          uint32_t dst = smem_base + stage * STAGE_BYTES;
          load_operand<true>(p.a, &tm_a0, dst, a_tile, int32_t(kb), 0, fb);
          load_bf16_planes(p.ax_mn, &tm_a1, dst + A_TILE_BYTES, a_tile, int32_t(kb), fb);
          dst += 2 * A_TILE_BYTES;
          load_operand<true>(p.b, &tm_b0, dst, b_tile, int32_t(kb), 0, fb);
          load_bf16_planes(p.bx_mn, &tm_b1, dst + B_TILE_BYTES, b_tile, int32_t(kb), fb);
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------- MMA issuer: one thread of the leader
    if (leader && lane == 0) {
      const uint32_t a_hi32 = uint32_t(p.a.desc >> 32), b_hi32 = uint32_t(p.b.desc >> 32);
      const uint32_t a_lo0 = uint32_t(p.a.desc), b_lo0 = uint32_t(p.b.desc);
      const uint32_t a_step = p.a.kstep_bytes >> 4, b_step = p.b.kstep_bytes >> 4;
      const uint32_t ax_hi32 = uint32_t(p.ax_desc >> 32), bx_hi32 = uint32_t(p.bx_desc >> 32);
      const uint32_t ax_lo0 = uint32_t(p.ax_desc), bx_lo0 = uint32_t(p.bx_desc);
      const uint32_t ax_step = p.ax_kstep >> 4, bx_step = p.bx_kstep >> 4;
      uint32_t stage = 0, phase = 0;
      uint32_t chunk = 0;
      uint32_t ready = 0;
      bool alive = true;
      for (uint32_t t = pair; alive && t < p.num_tiles; t += num_pairs) {
        for (uint32_t kb0 = 0; alive && kb0 < p.num_kblocks; kb0 += CHUNK_KB, ++chunk) {
          const uint32_t acc = chunk & 1u;
          const uint32_t acc_phase = (chunk >> 1) & 1u;
          if (!ptx::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
            if (first_to_give_up(abort_flag)) report(p.status, 2, 0x100u | acc, t, kb0);
            alive = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN;
          const uint32_t kb_end = min(kb0 + CHUNK_KB, p.num_kblocks);
          for (uint32_t kb = kb0; kb < kb_end; ++kb) {
            if (!ready && !ptx::mbar_wait(full_bar(stage), phase, abort_flag)) {
              if (first_to_give_up(abort_flag)) report(p.status, 2, stage, t, kb);
              alive = false;
              break;
            }
            ptx::tc_fence_after();
            const uint32_t next_stage = (stage + 1 == STAGES) ? 0 : stage + 1;
            const uint32_t next_phase = (stage + 1 == STAGES) ? phase ^ 1u : phase;
            const uint32_t ready_next = ptx::mbar_test_wait(full_bar(next_stage), next_phase);
            const uint32_t st = smem_base + stage * STAGE_BYTES;
            const uint32_t ah = a_lo0 + (st >> 4);
            const uint32_t bh = b_lo0 + ((st + 2 * A_TILE_BYTES) >> 4);
            // the small terms first: bf16(lo_a).bf16(hi_b) + bf16(hi_a).bf16(lo_b), K = 16 each
            const uint32_t axh = ax_lo0 + ((st + A_TILE_BYTES) >> 4);
            const uint32_t axl = axh + (X_PLANE_BYTES >> 4);
            const uint32_t bxh = bx_lo0 + ((st + 2 * A_TILE_BYTES + B_TILE_BYTES) >> 4);
            const uint32_t bxl = bxh + (X_PLANE_BYTES >> 4);
#pragma unroll
            for (uint32_t ks = 0; ks < KSTEPS / 2; ++ks) {
              const uint32_t accum = ((kb - kb0) | ks) ? 1u : 0u;
              ptx::mma_f16_pair_lohi(d_tmem, axl + ks * ax_step, ax_hi32, bxh + ks * bx_step, bx_hi32,
                                     p.idesc_x, accum);
              ptx::mma_f16_pair_lohi(d_tmem, axh + ks * ax_step, ax_hi32, bxl + ks * bx_step, bx_hi32,
                                     p.idesc_x, 1u);
            }
#pragma unroll
            for (uint32_t ks = 0; ks < KSTEPS; ++ks)
              ptx::mma_tf32_pair_lohi(d_tmem, ah + ks * a_step, a_hi32, bh + ks * b_step, b_hi32,
                                      p.idesc, 1u);
            ptx::mma_commit_pair(empty_bar(stage), 3);
            if (kb + 1 == kb_end) ptx::mma_commit_pair(tfull_bar(acc), 3);
            stage = next_stage;
            phase = next_phase;
            ready = ready_next;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------- drain + epilogue warps
    const uint32_t quarter = warp & 3u;
    const uint32_t half = (warp - 2u) >> 2;
    uint32_t chunk = 0;
    bool alive = true;
    for (uint32_t t = pair; alive && t < p.num_tiles; t += num_pairs) {
      uint32_t tm, tn;
      tile_coords(p, t, tm, tn);
      float sums[NC];
#pragma unroll
      for (int i = 0; i < NC; ++i) sums[i] = 0.f;
      for (uint32_t c = 0; c < chunks_per_tile; ++c, ++chunk) {
        const uint32_t acc = chunk & 1u;
        const uint32_t acc_phase = (chunk >> 1) & 1u;
        bool ok = ptx::mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) {
            if (first_to_give_up(abort_flag)) report(p.status, 3, acc, t, c);
          }
          alive = false;
          break;
        }
        ptx::tc_fence_after();
        drain_add<NC>(tmem_base + ((quarter * 32u) << 16) + acc * BN + half * NC, sums);
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa_shared(tempty_bar(acc), 0));
      }
      if (!alive) break;
      const uint32_t row = (tm * 2 + cta_rank) * BLOCK_M + quarter * 32u + lane;
      const uint32_t colb = tn * BN + half * NC;
#pragma unroll
      for (int j = 0; j < NC / 32; ++j) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(sums[j * 32 + i]);
        epilogue_store32(p, r, row, colb + j * 32);
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = ptx::globaltimer_ns();
    for (uint32_t i = 0; i < (1u << 16); ++i) {
      if (ptx::globaltimer_ns() - t0 > 2000000ull) break;
      __nanosleep(1000);
    }
    __syncthreads();
  }
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------- host side

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_driver() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  });
  return fn;
}

// A tensor map is a pure function of its arguments (address, extents, strides, box, swizzle),
// and a layer chain multiplies the same buffers with the same shapes step after step, so the
// encoded maps are kept: a GEMM call then costs a table look-up per operand instead of a
// driver call.  Bounded: the table is emptied when it reaches kMapCacheMax entries.
struct MapKey {
  uint64_t w[16];
  bool operator==(const MapKey& o) const { return std::memcmp(w, o.w, sizeof(w)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t x : k.w) h = (h ^ x) * 1099511628211ull;
    return size_t(h);
  }
};
constexpr size_t kMapCacheMax = 1024;
std::mutex g_map_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;

CUresult encode_cached(CUtensorMap* map, CUtensorMapDataType dtype, cuuint32_t rank, void* base,
                       const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box,
                       const cuuint32_t* estr, CUtensorMapInterleave il, CUtensorMapSwizzle sw,
                       CUtensorMapL2promotion promo, CUtensorMapFloatOOBfill oob) {
  EncodeTiledFn fn = encode_tiled_driver();
  if (!fn) return CUDA_ERROR_NOT_SUPPORTED;
  if (rank > 4) return fn(map, dtype, rank, base, dims, strides, box, estr, il, sw, promo, oob);
  MapKey k{};
  k.w[0] = uint64_t(dtype) | (uint64_t(rank) << 8) | (uint64_t(il) << 16) | (uint64_t(sw) << 24) |
           (uint64_t(promo) << 32) | (uint64_t(oob) << 40);
  k.w[1] = reinterpret_cast<uint64_t>(base);
  for (cuuint32_t i = 0; i < rank; ++i) {
    k.w[2 + i] = dims[i];
    k.w[9 + i] = uint64_t(box[i]) | (uint64_t(estr[i]) << 32);
  }
  for (cuuint32_t i = 0; i + 1 < rank; ++i) k.w[6 + i] = strides[i];
  {
    std::lock_guard<std::mutex> lk(g_map_mu);
    auto it = g_map_cache.find(k);
    if (it != g_map_cache.end()) {
      *map = it->second;
      return CUDA_SUCCESS;
    }
  }
  const CUresult r = fn(map, dtype, rank, base, dims, strides, box, estr, il, sw, promo, oob);
  if (r == CUDA_SUCCESS) {
    std::lock_guard<std::mutex> lk(g_map_mu);
    if (g_map_cache.size() >= kMapCacheMax) g_map_cache.clear();
    g_map_cache.emplace(k, *map);
  }
  return r;
}

EncodeTiledFn encode_tiled() { return encode_tiled_driver() ? &encode_cached : nullptr; }

// 2-D map over a row-major plane: `inner` contiguous elements per row, `outer`
// rows, boxes of (128 bytes, box_rows) written with the 128-byte swizzle.
bool make_map(CUtensorMap* map, bool f32, const void* base, uint64_t inner, uint64_t outer,
              uint64_t pitch_elems, uint32_t box_rows, bool mn_major) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return false;
  const uint32_t esz = f32 ? 4 : 2;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_elems * esz};
  cuuint32_t box[2] = {SLAB_ROW_BYTES / esz, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  // MN-major tf32 tiles must use the 32-byte-chunk flavour of the swizzle.
                  (f32 && mn_major) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                    : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Plan for an operand whose tile spans `tile_mn` rows/columns of the output.
OperandPlan plan_operand(bool f32, bool mn_major, uint32_t tile_mn, uint32_t block_k) {
  const uint32_t esz = f32 ? 4 : 2;
  const uint32_t row_elems = SLAB_ROW_BYTES / esz;  // == block_k
  const uint32_t umma_k = 32 / esz;                 // 16 (f16) or 8 (tf32)
  OperandPlan o{};
  if (!mn_major) {
    // rows = MN index, 128 bytes of K per row: one box; 8-row groups 1024 B apart.
    o.slabs = 1;
    o.slab_bytes = tile_mn * SLAB_ROW_BYTES;
    o.c0_tile = 0;
    o.c0_slab = 0;
    o.c0_k = int32_t(block_k);
    o.c1_tile = int32_t(tile_mn);
    o.c1_k = 0;
    o.kstep_bytes = umma_k * esz;  // 32 bytes inside the swizzled row
    o.desc = ptx::smem_desc(2, 16, 1024);
  } else {
    // rows = K index, 128 bytes of MN per row: one box per 128 bytes of MN.
    o.slabs = tile_mn / row_elems;
    o.slab_bytes = block_k * SLAB_ROW_BYTES;
    o.c0_tile = int32_t(tile_mn);
    o.c0_slab = int32_t(row_elems);
    o.c0_k = 0;
    o.c1_tile = 0;
    o.c1_k = int32_t(block_k);
    o.kstep_bytes = umma_k * SLAB_ROW_BYTES;  // umma_k rows down
    // fp16: groups of 8 k rows are 1024 B apart (16-byte-chunk swizzle).  tf32:
    // the 32-byte-chunk swizzle repeats every 4 k rows, 512 B apart.
    o.desc = f32 ? ptx::smem_desc(1, o.slab_bytes, 512) : ptx::smem_desc(2, o.slab_bytes, 1024);
  }
  return o;
}

// 3-D map over an MN-major plane (rows = K, `inner` contiguous MN elements): dimension 0 is
// one 128-byte slab row, dimension 1 the K rows, dimension 2 the slab index, so that one box
// (128 bytes, block_k rows, all slabs of a tile) lands slab after slab in shared memory,
// exactly where the per-slab 2-D boxes would put it.  The last slab of a ragged MN extent
// reads the plane's row padding: those values only reach output rows / columns that are
// never stored.
bool make_map_3d(CUtensorMap* map, bool f32, const void* base, uint64_t inner, uint64_t outer,
                 uint64_t pitch_elems, uint32_t block_k, uint32_t tile_slabs) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return false;
  const uint32_t esz = f32 ? 4 : 2;
  const uint32_t row_elems = SLAB_ROW_BYTES / esz;
  cuuint64_t dims[3] = {row_elems, outer, (inner + row_elems - 1) / row_elems};
  cuuint64_t strides[2] = {pitch_elems * esz, SLAB_ROW_BYTES};
  cuuint32_t box[3] = {row_elems, block_k, tile_slabs};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  f32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// 3-D map over a K-major plane (rows = MN, `inner` contiguous K elements, a multiple of the
// 128-byte slab row): dimension 0 is 128 bytes of K, dimension 1 the rows, dimension 2 the k
// block index; one box of (128 bytes, tile rows, kgroup) lands as kgroup consecutive K-major
// tiles.  k blocks past the end of K are zero-filled.
bool make_map_kgroup(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
                     uint64_t pitch_elems, uint32_t tile_rows, uint32_t kgroup) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return false;
  const uint32_t row_elems = SLAB_ROW_BYTES / 2;
  cuuint64_t dims[3] = {row_elems, outer, inner / row_elems};
  cuuint64_t strides[2] = {pitch_elems * 2, SLAB_ROW_BYTES};
  cuuint32_t box[3] = {row_elems, tile_rows, kgroup};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Map over the two bf16 planes behind GemmOperand::plane1 (plane1_bf16), the plane index as the
// last dimension: K-major operands (rows = MN, `inner` = K) as boxes of (32 of K, tile rows,
// 2 planes) with the 64-byte swizzle; MN-major operands (rows = K, `inner` = MN) as boxes of
// (64 of MN, 32 rows of K, the tile's slabs, 2 planes) with the 128-byte swizzle.
bool make_map_bf16_planes(CUtensorMap* map, const GemmOperand& op, uint64_t inner, uint64_t outer,
                          uint32_t tile_mn) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return false;
  const uint64_t plane_bytes = outer * op.pitch * 2;
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (!op.mn_major) {
    cuuint64_t dims[3] = {inner, outer, 2};
    cuuint64_t strides[2] = {op.pitch * 2, plane_bytes};
    cuuint32_t box[3] = {32, tile_mn, 2};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(op.plane1), dims, strides, box,
              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  cuuint64_t dims[4] = {64, outer, (inner + 63) / 64, 2};
  cuuint64_t strides[3] = {op.pitch * 2, SLAB_ROW_BYTES, plane_bytes};
  cuuint32_t box[4] = {64, 32, tile_mn / 64, 2};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(op.plane1), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The tensor map(s) of one operand (plane1 only for the fp32 path) and, where the operand is
// MN-major with a pitch of whole slab rows, the switch of its plan to single 3-D boxes.
bool make_operand_maps(bool f32, const GemmOperand& op, uint64_t inner, uint64_t outer,
                       uint32_t box_rows, OperandPlan& plan, CUtensorMap* m0, CUtensorMap* m1,
                       uint32_t kgroup = 0) {
  const uint32_t row_elems = SLAB_ROW_BYTES / (f32 ? 4 : 2);
  plan.kgroup = 0;
  if (!f32 && !op.mn_major && kgroup > 1 && inner % row_elems == 0 &&
      make_map_kgroup(m0, op.plane0, inner, outer, op.pitch, box_rows, kgroup)) {
    plan.kgroup = kgroup;
    plan.box3d = 0;
    return true;
  }
  if (op.mn_major && plan.slabs > 1 && op.pitch % row_elems == 0) {
    if (make_map_3d(m0, f32, op.plane0, inner, outer, op.pitch, box_rows, plan.slabs) &&
        (!m1 || make_map_3d(m1, f32, op.plane1, inner, outer, op.pitch, box_rows, plan.slabs))) {
      plan.box3d = 1;
      plan.c2_tile = int32_t(plan.slabs);
      return true;
    }
  }
  plan.box3d = 0;
  return make_map(m0, f32, op.plane0, inner, outer, op.pitch, box_rows, op.mn_major) &&
         (!m1 || make_map(m1, f32, op.plane1, inner, outer, op.pitch, box_rows, op.mn_major));
}

// Shared memory behind the pipeline stages: the barrier words.
template <int KIND>
constexpr uint32_t extra_smem_for() {
  return 256u;
}

template <int KIND, int BLOCK_N>
constexpr int stages_for() {
  constexpr uint32_t planes = (KIND == int(Kind::TF32x3)) ? 2 : 1;
  constexpr uint32_t stage = planes * (A_TILE_BYTES + BLOCK_N * SLAB_ROW_BYTES);
  constexpr uint32_t avail = SMEM_LIMIT - 1024 /*align*/ - extra_smem_for<KIND>();
  constexpr int s = int(avail / stage);
  return s > 8 ? 8 : s;
}

template <int KIND, int BLOCK_N>
const char* launch_variant(const CUtensorMap* maps, const KernelParams& kp, uint32_t grid,
                           cudaStream_t stream) {
  constexpr int STAGES = stages_for<KIND, BLOCK_N>();
  constexpr uint32_t planes = (KIND == int(Kind::TF32x3)) ? 2 : 1;
  constexpr uint32_t smem =
      STAGES * planes * (A_TILE_BYTES + BLOCK_N * SLAB_ROW_BYTES) + 1024 + extra_smem_for<KIND>();
  static_assert(STAGES >= 2, "pipeline too shallow");
  static_assert(smem <= SMEM_LIMIT, "shared memory");
  void (*kern)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
               const KernelParams);
  uint32_t threads;
  if constexpr (KIND == int(Kind::TF32x3)) {
    kern = gemm_tf32x3_kernel<BLOCK_N, STAGES>;
    threads = TF32_THREADS;
  } else {
    kern = gemm_tcgen05_kernel<KIND, BLOCK_N, STAGES>;
    threads = NUM_THREADS;
  }
  static bool attr_done_dev[64] = {};  // per variant and device
  int dev = 0;
  cudaGetDevice(&dev);
  bool& attr_done = attr_done_dev[dev & 63];
  if (!attr_done) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) !=
        cudaSuccess) {
      return "cudaFuncSetAttribute(max dynamic shared memory) failed";
    }
    attr_done = true;
  }
  if (launch_kernel(kern, dim3(grid), dim3(threads), smem, stream, maps[0], maps[1], maps[2], maps[3], kp) !=
      cudaSuccess) {
    cudaGetLastError();
    return "GEMM kernel launch failed";
  }
  return nullptr;
}

// Tile width and split count with the cheapest estimated time.  A work unit costs,
// per k block, the largest of its tensor-pipe time, the MMAs' shared-memory read time
// and the time to load its operand bytes (one SM takes about 48 bytes per cycle from
// L2, measured), plus a fixed prologue/epilogue share; a split tile pays for the trip
// of its partial sums through the workspace.  Splits are whole accumulation chunks.
struct TileChoice {
  int bn;
  uint32_t splits, kb_per_split;
};
TileChoice choose_tiles(Kind kind, uint32_t M, uint32_t N, uint32_t K, int sms, uint32_t batch_count,
                        int forced_bn, int max_splits) {
  const bool f32 = (kind == Kind::TF32x3);
  const uint32_t tiles_m = (M + BLOCK_M - 1) / BLOCK_M;
  const uint32_t block_k = f32 ? 32u : 64u;
  const uint32_t kblocks = (K + block_k - 1) / block_k;
  const double mmas = f32 ? 12.0 : 4.0;        // per k block
  TileChoice best{32, 1u, kblocks};
  double best_cost = 1e300;
  const int cands[4] = {256, 128, 64, 32};
  for (int bn : cands) {
    if (forced_bn && bn != forced_bn) continue;
    if (!forced_bn && bn > 32 && uint32_t(bn) >= 2 * ((N + 31) / 32) * 32) continue;  // mostly padding
    const uint32_t tiles_n = (N + bn - 1) / bn;
    const double tiles = double(tiles_m) * tiles_n * batch_count;
    const double pipe = mmas * bn / 2.0;                          // 128 x bn x (8|16): bn/2 cycles
    const double smem = mmas * (4096.0 + bn * 32.0) / 128.0;
    const double load = 128.0 * (f32 ? 2.0 : 1.0) * (128.0 + bn) / 48.0;
    const double per_kb = std::max(pipe, std::max(smem, load));
    for (uint32_t want = 1; want <= uint32_t(std::max(1, max_splits)); ++want) {
      uint32_t per = (kblocks + want - 1) / want;
      if (want > 1) per = (per + CHUNK_KB - 1) / CHUNK_KB * CHUNK_KB;
      const uint32_t splits = (kblocks + per - 1) / per;
      if (splits != want) continue;  // rounding merged two candidates
      const double waves = std::ceil(tiles * splits / sms);
      double cost = waves * (per_kb * per + 2000.0 + 8.0 * bn);
      if (splits > 1) cost += 1500.0 + (splits + 1.0) * 128.0 * bn * 4.0 / 64.0;
      if (cost < best_cost) {
        best_cost = cost;
        best = TileChoice{bn, splits, per};
      }
    }
  }
  return best;
}

template <int BLOCK_N, int SUB, bool GATED = false>
const char* launch_pair_variant(const CUtensorMap& ma, const CUtensorMap& mb, const KernelParams& kp,
                                uint32_t pairs, cudaStream_t stream) {
  constexpr uint32_t stage = SUB * (A_TILE_BYTES + (BLOCK_N / 2) * SLAB_ROW_BYTES);
  constexpr uint32_t avail = SMEM_LIMIT - 1024 - 256;
  constexpr int STAGES = (avail / stage) > 8 ? 8 : int(avail / stage);
  constexpr uint32_t smem = STAGES * stage + 1024 + 256;
  static_assert(STAGES >= 1 && smem <= SMEM_LIMIT, "pair kernel shared memory");
  auto kern = gemm_f16_pair_kernel<BLOCK_N, STAGES, SUB, GATED>;
  static bool attr_done_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done_dev[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) !=
        cudaSuccess)
      return "cudaFuncSetAttribute(max dynamic shared memory) failed";
    attr_done_dev[dev & 63] = true;
  }
  // (cluster size 2 is compiled in)
  if (launch_kernel(kern, dim3(2 * pairs), dim3(GATED ? GATED_THREADS : NUM_THREADS), smem, stream, ma,
                    mb, kp) != cudaSuccess) {
    cudaGetLastError();
    return "GEMM pair kernel launch failed";
  }
  return nullptr;
}

const char* launch_pair512(const CUtensorMap& ma, const CUtensorMap& mb, const KernelParams& kp,
                           uint32_t pairs, cudaStream_t stream) {
  constexpr uint32_t stage = 2 * A_TILE_BYTES + 128 * SLAB_ROW_BYTES;
  constexpr uint32_t extra = 1024 /*align*/ + 1024 /*barriers*/;
  constexpr int STAGES = int((SMEM_LIMIT - extra) / stage);
  constexpr uint32_t smem = STAGES * stage + extra;
  static_assert(STAGES >= 3 && smem <= SMEM_LIMIT, "pair512 kernel shared memory");
  auto kern = gemm_f16_pair512_kernel<STAGES>;
  static bool attr_done_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done_dev[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) !=
        cudaSuccess)
      return "cudaFuncSetAttribute(max dynamic shared memory) failed";
    attr_done_dev[dev & 63] = true;
  }
  if (launch_kernel(kern, dim3(2 * pairs), dim3(NUM_THREADS), smem, stream, ma, mb, kp) != cudaSuccess) {
    cudaGetLastError();
    return "GEMM pair512 kernel launch failed";
  }
  return nullptr;
}

// fp16 GEMM on CTA pairs: (256 or 512) x bn tiles, one cluster of two CTAs per tile.
const char* launch_gemm_pair(uint32_t M, uint32_t N, uint32_t K, int bn, bool tall,
                             const GemmOperand& A, const GemmOperand& B, KernelParams kp,
                             int sm_count, int max_ctas, cudaStream_t stream, bool gated = false) {
  const uint32_t block_k = 64;
  const uint32_t tile_m = tall ? 4 * BLOCK_M : 2 * BLOCK_M;
  kp.a = plan_operand(false, A.mn_major, BLOCK_M, block_k);
  kp.b = plan_operand(false, B.mn_major, uint32_t(bn / 2), block_k);
  kp.tiles_m = (M + tile_m - 1) / tile_m;
  kp.tiles_n = (N + bn - 1) / bn;
  kp.num_tiles = kp.tiles_m * kp.tiles_n;
  kp.num_kblocks = (K + block_k - 1) / block_k;
  kp.group_m = tall ? 4 : 8;
  kp.group_m0 = gated ? std::min(kp.group_m0, kp.tiles_m) : 0u;
  kp.idesc = ptx::make_idesc(0u, A.mn_major, B.mn_major, 2 * BLOCK_M, uint32_t(bn));
  CUtensorMap ma, mb;
  std::memset(&ma, 0, sizeof(ma));
  std::memset(&mb, 0, sizeof(mb));
  const uint32_t a_box_rows = A.mn_major ? block_k : BLOCK_M;
  const uint32_t b_box_rows = B.mn_major ? block_k : uint32_t(bn / 2);
  const uint32_t kgroup = tall ? 0u : 2u;  // the 256-row kernel's stage holds two k blocks
  if (!make_operand_maps(false, A, A.mn_major ? M : K, A.mn_major ? K : M, a_box_rows, kp.a, &ma, nullptr, kgroup) ||
      !make_operand_maps(false, B, B.mn_major ? N : K, B.mn_major ? K : N, b_box_rows, kp.b, &mb, nullptr, kgroup))
    return "cuTensorMapEncodeTiled failed";
  const uint32_t limit = uint32_t(max_ctas > 0 ? max_ctas : sm_count) / 2;
  const uint32_t pairs = std::max<uint32_t>(1u, std::min<uint32_t>(kp.num_tiles, limit));
  if (tall) return launch_pair512(ma, mb, kp, pairs, stream);
  if (gated) return launch_pair_variant<256, 2, true>(ma, mb, kp, pairs, stream);
  if (bn == 256) return launch_pair_variant<256, 2>(ma, mb, kp, pairs, stream);
  return launch_pair_variant<128, 2>(ma, mb, kp, pairs, stream);
}

// fp32-accurate GEMM on CTA pairs (256 x 256 tiles).
const char* launch_tf32_pair(uint32_t M, uint32_t N, uint32_t K, const GemmOperand& A,
                             const GemmOperand& B, KernelParams kp, int sm_count, int max_ctas,
                             cudaStream_t stream) {
  constexpr uint32_t block_k = 32;
  constexpr uint32_t stage = 2 * (A_TILE_BYTES + 128 * SLAB_ROW_BYTES);
  constexpr int STAGES = int((SMEM_LIMIT - 1024 - 256) / stage);
  constexpr uint32_t smem = STAGES * stage + 1024 + 256;
  static_assert(STAGES >= 3 && smem <= SMEM_LIMIT, "tf32 pair kernel shared memory");
  if (!A.plane1_bf16 || !B.plane1_bf16) return "the fp32 CTA-pair kernel takes bf16 low planes";
  if (A.pitch % 64 || B.pitch % 64) return "bf16 low planes need a pitch of whole 64-element slabs";
  kp.a = plan_operand(true, A.mn_major, BLOCK_M, block_k);
  kp.b = plan_operand(true, B.mn_major, 128, block_k);
  kp.tiles_m = (M + 255) / 256;
  kp.tiles_n = (N + 255) / 256;
  kp.num_tiles = kp.tiles_m * kp.tiles_n;
  kp.num_kblocks = (K + block_k - 1) / block_k;
  kp.group_m = 8;
  kp.idesc = ptx::make_idesc(2u, A.mn_major, B.mn_major, 2 * BLOCK_M, 256);
  CUtensorMap maps[4];
  std::memset(maps, 0, sizeof(maps));
  const uint32_t a_box = A.mn_major ? block_k : BLOCK_M, b_box = B.mn_major ? block_k : 128;
  const uint64_t a_in = A.mn_major ? M : K, a_out = A.mn_major ? K : M;
  const uint64_t b_in = B.mn_major ? N : K, b_out = B.mn_major ? K : N;
  if (!make_operand_maps(true, A, a_in, a_out, a_box, kp.a, &maps[0], nullptr) ||
      !make_operand_maps(true, B, b_in, b_out, b_box, kp.b, &maps[2], nullptr) ||
      !make_map_bf16_planes(&maps[1], A, a_in, a_out, 128) ||
      !make_map_bf16_planes(&maps[3], B, b_in, b_out, 128))
    return "cuTensorMapEncodeTiled failed";
  // K-major bf16 tile: rows of 64 bytes, groups of 8 rows 512 bytes apart, 32 bytes per K = 16.
  // MN-major: as the fp16 kernels' (slabs of 64 columns, here 32 rows of K = 4 KB each).
  const OperandPlan xmn = plan_operand(false, true, 128, block_k);
  kp.ax_mn = A.mn_major;
  kp.bx_mn = B.mn_major;
  kp.ax_desc = A.mn_major ? xmn.desc : ptx::smem_desc(4, 16, 512);
  kp.bx_desc = B.mn_major ? xmn.desc : ptx::smem_desc(4, 16, 512);
  kp.ax_kstep = A.mn_major ? xmn.kstep_bytes : 32u;
  kp.bx_kstep = B.mn_major ? xmn.kstep_bytes : 32u;
  kp.idesc_x = ptx::make_idesc(1u, A.mn_major, B.mn_major, 2 * BLOCK_M, 256);
  auto kern = gemm_tf32x3_pair_kernel<STAGES>;
  static bool attr_done_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done_dev[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) !=
        cudaSuccess)
      return "cudaFuncSetAttribute(max dynamic shared memory) failed";
    attr_done_dev[dev & 63] = true;
  }
  const uint32_t limit = uint32_t(max_ctas > 0 ? max_ctas : sm_count) / 2;
  const uint32_t pairs = std::max<uint32_t>(1u, std::min<uint32_t>(kp.num_tiles, limit));
  if (launch_kernel(kern, dim3(2 * pairs), dim3(TF32_THREADS), smem, stream, maps[0], maps[1], maps[2],
                    maps[3], kp) != cudaSuccess) {
    cudaGetLastError();
    return "GEMM tf32 pair kernel launch failed";
  }
  return nullptr;
}

}  // namespace

bool tf32_takes_pair_kernel(uint32_t M, uint32_t N, uint32_t K, int sm_count, const GemmTuning& tune) {
  (void)K;
  if (tune.pair == 0 || !(tune.block_n == 0 || tune.block_n == 256)) return false;
  // Measured cross-over against the single-CTA kernel with split-K: level at 32 pair tiles
  // (2048 x 1024 x 1024: 34 against 37 us), 64 against 91 us at 2048^3 (64 tiles); below it
  // the pairs have too few tiles to fill the machine (1024^3, 16 tiles: 33 against 21 us).
  const uint64_t pair_tiles = uint64_t((M + 255) / 256) * ((N + 255) / 256);
  return tune.pair >= 1 || (M >= 256 && N >= 128 && pair_tiles >= uint64_t(sm_count) * 2 / 9);
}

const char* launch_gemm(Kind kind, uint32_t M, uint32_t N, uint32_t K, const GemmOperand& A,
                        const GemmOperand& B, float* C, uint64_t ldc, const GemmEpilogue& epi,
                        GemmStatus* status, int sm_count, const GemmTuning& tune,
                        cudaStream_t stream, const GemmBatch* batch) {
  if (M == 0 || N == 0 || K == 0) return "GEMM dimensions must be positive";
  if (batch && (kind != Kind::TF32x3 || A.mn_major || !B.mn_major || batch->count == 0))
    return "batched GEMM supports fp32 A[b,M,K].B[b,K,N] only";
  const bool f32 = (kind == Kind::TF32x3);
  const uint32_t esz = f32 ? 4 : 2;
  const uint32_t block_k = SLAB_ROW_BYTES / esz;
  if ((A.pitch * esz) % 16 || (B.pitch * esz) % 16) return "operand pitch must be a multiple of 16 bytes";
  if (reinterpret_cast<uintptr_t>(A.plane0) % 16 || reinterpret_cast<uintptr_t>(B.plane0) % 16)
    return "operand planes must be 16-byte aligned";
  if (f32 && (!A.plane1 || !B.plane1)) return "TF32x3 needs the low planes";

  // (for a batched product the tiles of all batches fill the machine together)
  if (tune.block_n && tune.block_n != 32 && tune.block_n != 64 && tune.block_n != 128 && tune.block_n != 256)
    return "unsupported BLOCK_N";
  // split-K only where the fp32 kernel has a workspace to put partial sums in
  int max_splits = 1;
  if (f32 && tune.split_k != 1 && tune.splitk_ws && tune.splitk_counters)
    max_splits = tune.split_k > 1 ? tune.split_k : 16;
  TileChoice choice = choose_tiles(kind, M, N, K, sm_count, batch ? batch->count : 1u, tune.block_n, max_splits);
  if (tune.split_k > 1 && max_splits > 1) {  // forced: as close to the asked count as whole chunks allow
    const uint32_t kblocks = (K + block_k - 1) / block_k;
    uint32_t per = (kblocks + uint32_t(tune.split_k) - 1) / uint32_t(tune.split_k);
    per = (per + CHUNK_KB - 1) / CHUNK_KB * CHUNK_KB;
    choice.kb_per_split = per;
    choice.splits = (kblocks + per - 1) / per;
  }
  int bn = choice.bn;
  // An N-major fp16 tile narrower than one 128-byte swizzle row (64 columns)
  // would need the 64-byte swizzle; use the 64-wide tile instead.
  if (!f32 && B.mn_major && bn == 32) bn = 64;

  KernelParams kp{};
  kp.a = plan_operand(f32, A.mn_major, BLOCK_M, block_k);
  kp.b = plan_operand(f32, B.mn_major, uint32_t(bn), block_k);
  kp.M = M;
  kp.N = N;
  kp.tiles_m = (M + BLOCK_M - 1) / BLOCK_M;
  kp.tiles_n = (N + bn - 1) / bn;
  kp.num_tiles = kp.tiles_m * kp.tiles_n;
  kp.num_kblocks = (K + block_k - 1) / block_k;
  kp.group_m = 16;
  kp.idesc = ptx::make_idesc(f32 ? 2u : 0u, A.mn_major, B.mn_major, BLOCK_M, uint32_t(bn));
  kp.C = C;
  kp.c_in = (epi.beta != 0.f) ? epi.c_in : nullptr;
  kp.bias = epi.bias;
  kp.ldc = ldc;
  kp.alpha = epi.alpha;
  kp.beta = epi.beta;
  kp.act = epi.act;
  kp.act_param = epi.act_param;
  kp.vec_store = (ldc % 4 == 0) && (reinterpret_cast<uintptr_t>(C) % 16 == 0) &&
                 (!kp.c_in || reinterpret_cast<uintptr_t>(kp.c_in) % 16 == 0) &&
                 (!kp.bias || reinterpret_cast<uintptr_t>(kp.bias) % 16 == 0);
  kp.status = status;
  kp.splits = 1;
  kp.kb_per_split = kp.num_kblocks;

  // Large fp16 problems run on CTA pairs (256-row tiles); small ones, where the
  // pair tiles would not fill the machine, stay on single-CTA tiles.
  if (kind == Kind::F16 && tune.pair != 0) {
    const uint64_t half_sms = uint64_t(sm_count) / 2;
    // 512-row tiles need a quarter fewer operand bytes per flop than 256-row
    // tiles but cannot overlap their epilogue with the next tile (TMEM is full),
    // so they pay off only for very deep K (measured with 3-D operand boxes: 4 % ahead at
    // K=16384, level at 8192^3, 4-10 % behind at K <= 8192 with N = 4096).
    const uint64_t tall_tiles = uint64_t((M + 511) / 512) * ((N + 255) / 256);
    const bool tall_ok = (tune.block_n == 0 || tune.block_n == 256);
    if (tall_ok && (tune.pair == 2 || (tune.pair < 0 && M >= 512 && N >= 128 && K >= 12288 && tall_tiles >= half_sms))) {
      return launch_gemm_pair(M, N, K, 256, true, A, B, kp, sm_count, tune.max_ctas, stream);
    }
    const int pbn = (tune.block_n == 128) ? 128 : 256;
    const uint64_t pair_tiles = uint64_t((M + 255) / 256) * ((N + pbn - 1) / pbn);
    const bool fits = (tune.block_n == 0 || tune.block_n == 128 || tune.block_n == 256);
    const bool worth = M >= 256 && N >= uint32_t(pbn) / 2 && pair_tiles >= half_sms;
    if (fits && (tune.pair == 1 || (tune.pair < 0 && worth))) {
      return launch_gemm_pair(M, N, K, pbn, false, A, B, kp, sm_count, tune.max_ctas, stream);
    }
  }

  if (kind == Kind::TF32x3 && !batch && tf32_takes_pair_kernel(M, N, K, sm_count, tune))
    return launch_tf32_pair(M, N, K, A, B, kp, sm_count, tune.max_ctas, stream);
  if (A.plane1_bf16 || B.plane1_bf16) return "bf16 low planes are for the CTA-pair kernel only";

  // Tensor maps: inner extent is the contiguous index, outer the row index.
  CUtensorMap maps[4];
  std::memset(maps, 0, sizeof(maps));
  const uint32_t a_box_rows = A.mn_major ? block_k : BLOCK_M;
  const uint32_t b_box_rows = B.mn_major ? block_k : uint32_t(bn);
  uint64_t a_inner = A.mn_major ? M : K, a_outer = A.mn_major ? K : M;
  uint64_t b_inner = B.mn_major ? N : K, b_outer = B.mn_major ? K : N;
  if (batch) {
    // stacked matrices: A is [count*M, K]; B is [count*b_rows, N] with b_rows >= K rows per
    // batch, the rows past K zero; tiles are numbered batch by batch
    a_outer = uint64_t(batch->count) * M;
    b_outer = uint64_t(batch->count) * batch->b_rows;
    kp.batch_tiles = kp.num_tiles;
    kp.num_tiles *= batch->count;
    kp.a_batch_c1 = int32_t(M);
    kp.b_batch_c1 = int32_t(batch->b_rows);
  }
  if (!make_operand_maps(f32, A, a_inner, a_outer, a_box_rows, kp.a, &maps[0], f32 ? &maps[1] : nullptr) ||
      !make_operand_maps(f32, B, b_inner, b_outer, b_box_rows, kp.b, &maps[2], f32 ? &maps[3] : nullptr))
    return "cuTensorMapEncodeTiled failed";
  if (!f32) {
    maps[1] = maps[0];
    maps[3] = maps[2];
  }

  if (f32 && choice.splits > 1) {
    const size_t need = size_t(kp.num_tiles) * choice.splits * BLOCK_M * size_t(bn) * sizeof(float);
    if (need <= tune.splitk_ws_bytes && kp.num_tiles <= tune.splitk_counter_slots) {
      kp.splits = choice.splits;
      kp.kb_per_split = choice.kb_per_split;
      kp.sk_ws = tune.splitk_ws;
      kp.sk_count = tune.splitk_counters;
    }
  }
  uint32_t grid = std::min<uint32_t>(kp.num_tiles * kp.splits,
                                     uint32_t(tune.max_ctas > 0 ? tune.max_ctas : sm_count));
  if (kind == Kind::F16) {
    switch (bn) {
      case 256: return launch_variant<0, 256>(maps, kp, grid, stream);
      case 128: return launch_variant<0, 128>(maps, kp, grid, stream);
      case 64: return launch_variant<0, 64>(maps, kp, grid, stream);
      default: return launch_variant<0, 32>(maps, kp, grid, stream);
    }
  } else {
    switch (bn) {
      case 256: return launch_variant<1, 256>(maps, kp, grid, stream);
      case 128: return launch_variant<1, 128>(maps, kp, grid, stream);
      case 64: return launch_variant<1, 64>(maps, kp, grid, stream);
      default: return launch_variant<1, 32>(maps, kp, grid, stream);
    }
  }
}

// Row-sharded product with the replication of B inside the kernel (see kernels.h).
const char* launch_gemm_sharded(uint32_t M, uint32_t N, uint32_t K, const void* a, uint64_t a_pitch,
                                const void* b_slot, float* C, uint64_t ldc, const ShardLink& link,
                                GemmStatus* status, int sm_count, cudaStream_t stream) {
  if (M == 0 || N == 0 || K == 0) return "GEMM dimensions must be positive";
  if (N % 8 || a_pitch % 8) return "operand pitch must be a multiple of 16 bytes";
  if (reinterpret_cast<uintptr_t>(a) % 16 || reinterpret_cast<uintptr_t>(b_slot) % 16 ||
      reinterpret_cast<uintptr_t>(link.b_src) % 16 || reinterpret_cast<uintptr_t>(link.slot_multicast) % 16 ||
      link.slot_offset % 16)
    return "operand planes must be 16-byte aligned";
  if (link.world < 1 || link.world > kShardMaxRanks || link.rank < 0 || link.rank >= link.world ||
      link.owner < 0 || link.owner >= link.world || (link.slot != 0 && link.slot != 1) || !link.bases)
    return "bad rank, owner, slot or group size";
  if (link.rank == link.owner && !link.b_src) return "the owner passes the source of B";
  constexpr uint32_t bn = 256;
  GemmOperand A, B;
  A.plane0 = a;
  A.pitch = a_pitch;
  A.mn_major = false;
  B.plane0 = b_slot;
  B.pitch = N;
  B.mn_major = true;
  KernelParams kp{};
  kp.M = M;
  kp.N = N;
  kp.C = C;
  kp.ldc = ldc;
  kp.alpha = 1.f;
  kp.act = ACT_NONE;
  kp.vec_store = (ldc % 4 == 0) && (reinterpret_cast<uintptr_t>(C) % 16 == 0);
  kp.status = status;
  kp.splits = 1;
  const uint32_t tiles_n = (N + bn - 1) / bn;
  ShardParams& sh = kp.sh;
  sh.src = static_cast<const uint4*>(link.b_src);
  sh.mc_dst = static_cast<uint4*>(link.slot_multicast);
  sh.bases = link.bases;
  sh.slot_offset = link.slot_offset;
  sh.ctrl_offset = link.ctrl_offset;
  sh.world = uint32_t(link.world);
  sh.owner = uint32_t(link.owner);
  sh.rank = uint32_t(link.rank);
  sh.slot = uint32_t(link.slot);
  sh.epoch = link.epoch;
  sh.ack_needed = link.epoch > 2u ? link.epoch - 2u : 0u;
  sh.slab_tiles = (tiles_n + kShardMaxSlabs - 1) / kShardMaxSlabs;
  sh.num_slabs = (tiles_n + sh.slab_tiles - 1) / sh.slab_tiles;
  sh.rows = K;
  sh.row_chunks = N / 8;
  sh.slab_chunks = sh.slab_tiles * bn / 8;
  sh.trace = static_cast<unsigned long long*>(link.trace);
  // Sending pairs of the owner: a quarter of the pairs, 8 at most (measured on 8 GPUs: 0.517 ms per
  // step with 8 sending pairs, 0.534 with 16, 0.546 with 24),
  // left out of as many rounds of tiles as the push is expected to take beyond the wait of the
  // other pairs for the first slabs: bytes at 400 GB/s plus 10 us (measured: 112 us for 32 MiB
  // to 2 GPUs beside the running product, first slab after 26 us), against 2 * 256 * 256 * K flop
  // per tile at the pair's share of 1.35 PFLOP/s.  A wrong guess only shifts a few tiles between
  // pairs.
  const uint32_t tiles_m = (M + 2 * BLOCK_M - 1) / (2 * BLOCK_M);
  const uint32_t pairs = std::max<uint32_t>(1u, std::min<uint32_t>(tiles_m * tiles_n, uint32_t(sm_count) / 2));
  if (link.rank == link.owner) {
    sh.sender_pairs = link.sender_pairs >= 0 ? uint32_t(link.sender_pairs)
                                             : (pairs >= 8 ? std::min<uint32_t>(8u, pairs / 4) : 1u);
    sh.sender_pairs = std::max<uint32_t>(1u, std::min<uint32_t>(sh.sender_pairs, pairs));
    const double push_s = double(K) * N * 2.0 / 400e9 + 10e-6;
    const double tile_s = 2.0 * 256 * 256 * K / (1.35e15 / (double(sm_count) / 2));
    sh.late_rounds = link.late_rounds >= 0 ? uint32_t(link.late_rounds)
                                           : uint32_t(std::min(64.0, std::floor(push_s / tile_s + 0.5)));
  }
  // Row tiles swept slab by slab while B arrives.  A slab must be consumed no faster than the
  // next one arrives: the group's tiles of one slab have to last as long as a slab's transfer.
  // Measured on B200s: the owner publishes a 2 MiB slab every 6 to 8 us (32 MiB in 110 us to 2
  // GPUs, 134 us to 8), a wave of 74 tiles with K = 4096 takes about 28 us, so 16 row tiles last
  // 6 us per slab; larger groups cost L2 reuse of A (8 GPUs: 0.517 ms per step with 16, 0.528
  // with 24, 0.536 with 32).
  kp.group_m0 = link.first_group ? link.first_group : 16u;
  return launch_gemm_pair(M, N, K, int(bn), false, A, B, kp, sm_count, 0, stream, true);
}

}  // namespace gonn
