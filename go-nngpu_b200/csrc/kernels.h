// Internal C++ interface between the C-ABI bridge and the sm_100a kernels.
// Nothing here is exported from the shared library.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace gonn {

// ---- dense GEMM on the 5th-generation tensor cores -------------------------
enum class Kind : int {
  F16 = 0,     // fp16 operands, fp32 accumulate in TMEM
  TF32x3 = 1,  // fp32 operands split hi+lo into two tf32 planes, 3 MMAs per k step
};

// Activation codes of the fused epilogue.  They are the codes the reference's
// fused_linear_activation kernel decodes (internal/cgo/default.metal:488-506);
// every other value means identity, as in its `default:` branch.
enum Act : int { ACT_RELU = 0, ACT_LEAKY = 1, ACT_SIGMOID = 2, ACT_TANH = 3, ACT_GELU = 4,
                 ACT_NONE = -1 };

// One GEMM operand as it lies in HBM.  `mn_major == false`: rows are the M (or
// N) index and K is contiguous ("K-major").  `mn_major == true`: rows are the K
// index and M (or N) is contiguous.  `pitch` is in elements and must make the
// row pitch a multiple of 16 bytes; `plane1` is the low tf32 plane (TF32x3 only).
// `plane1_bf16`: plane1 holds instead two bf16 planes of the same shape and pitch, one
// behind the other: bf16(hi), then bf16(x - hi) (launch_split_tf32_bf16); both operands of
// a product must agree, and only products that tf32_takes_pair_kernel() accepts may use it.
struct GemmOperand {
  const void* plane0 = nullptr;
  const void* plane1 = nullptr;
  uint64_t pitch = 0;
  bool mn_major = false;
  bool plane1_bf16 = false;
};

// C = act(alpha * A.B + beta * C_in + bias[n])
struct GemmEpilogue {
  float alpha = 1.f;
  float beta = 0.f;          // when non-zero, c_in is read with the same pitch as C
  const float* c_in = nullptr;
  const float* bias = nullptr;  // length N or null
  int act = ACT_NONE;
  float act_param = 0.f;
};

// Status words a kernel writes when a bounded wait ran out (all zero = fine).
struct GemmStatus {
  uint32_t code;   // 0 ok, 1 producer, 2 mma issuer, 3 epilogue gave up
  uint32_t where;  // stage / accumulator index
  uint32_t tile;
  uint32_t kblock;
};

struct GemmTuning {
  int block_n = 0;   // 0 = choose; else 32/64/128/256
  int max_ctas = 0;  // 0 = one per SM
  int pair = -1;     // fp16 CTA-pair kernel: -1 = choose by size, 0 = never, 1 = always
  // Split-K of the fp32 single-CTA kernel, for products with too few tiles to fill the
  // GPU: 0 = choose, 1 = never, n > 1 = n splits.  Needs the workspace below (device
  // memory, owned by the caller, used by one launch at a time; the counters start at
  // zero and every launch leaves them at zero).  Without it there is no split.
  int split_k = 0;
  float* splitk_ws = nullptr;
  size_t splitk_ws_bytes = 0;
  uint32_t* splitk_counters = nullptr;
  uint32_t splitk_counter_slots = 0;
};

// Batched product C[b] = A[b].B[b] over stacked matrices (fp32 path, A[b,M,K] and
// B[b,K,N] layouts only).  The B planes hold `b_rows` >= K rows per batch, a
// multiple of the 32-row k block, the rows past K zero.
struct GemmBatch {
  uint32_t count = 1;
  uint32_t b_rows = 0;
};

// Enqueues the GEMM on `stream`.  Returns nullptr on success, else a static
// message.  `status` is device memory holding one GemmStatus, zeroed by the
// caller before the launch.
const char* launch_gemm(Kind kind, uint32_t M, uint32_t N, uint32_t K, const GemmOperand& A,
                        const GemmOperand& B, float* C, uint64_t ldc, const GemmEpilogue& epi,
                        GemmStatus* status, int sm_count, const GemmTuning& tune,
                        cudaStream_t stream, const GemmBatch* batch = nullptr);

// True when launch_gemm(Kind::TF32x3, ...) with these sizes runs on the CTA-pair kernel, the
// one that also takes the correction terms from bf16 planes (GemmOperand::plane1_bf16).
bool tf32_takes_pair_kernel(uint32_t M, uint32_t N, uint32_t K, int sm_count, const GemmTuning& tune);

// ---- pre-pass: operand planes ---------------------------------------------
enum F16Mode : int { F16_RN = 0, F16_TRUNC = 1 };
// fp32 [rows, cols] (pitch cols) -> fp16 plane with `pitch` elements per row.
void launch_cvt_f16(const float* src, uint64_t rows, uint64_t cols, void* dst, uint64_t pitch,
                    int mode, cudaStream_t stream);
// fp32 -> (hi, lo) tf32 planes: hi = rna_tf32(x), lo = rna_tf32(x - hi).
// With `mask` (same shape as src): x is taken as 0 where mask <= 0 (ReLU derivative).
void launch_split_tf32(const float* src, uint64_t rows, uint64_t cols, float* hi, float* lo,
                       uint64_t pitch, cudaStream_t stream, const float* mask = nullptr);

// fp32 -> hi = rna_tf32(x) as fp32, and behind `x2` two bf16 planes [rows, pitch] one after the
// other: bf16(hi), then bf16(x - hi).  Same bytes as launch_split_tf32 writes.
void launch_split_tf32_bf16(const float* src, uint64_t rows, uint64_t cols, float* hi, void* x2,
                            uint64_t pitch, cudaStream_t stream, const float* mask = nullptr);

// Both of the above and the column sums of the same (masked) values in one pass, for the linear
// backward: `low` is the lo plane or, with `bf16x`, the two bf16 planes; `colsum` gets `cols`
// sums.  `ws` / `counters` as for launch_colsum.  Returns false without launching when the
// shape or an address does not allow 16-byte accesses (the caller then launches the two
// kernels separately).
bool launch_split_colsum(const float* src, uint64_t rows, uint64_t cols, float* hi, void* low, bool bf16x,
                         uint64_t pitch, float* colsum, cudaStream_t stream, const float* mask, float* ws,
                         size_t ws_floats, uint32_t* counters, uint32_t counter_slots);

// ---- HBM-bound kernels -----------------------------------------------------
void launch_transpose(const float* in, uint64_t rows, uint64_t cols, float* out, int sm_count,
                      cudaStream_t stream);
// mode 0: c[i,j] = a[i,j] + b[j]; 1: c = a[j] + b[i,j]; 2: c = a[i,j] + b[i]; 3: c = a[i] + b[i,j]
void launch_add_broadcast(const float* a, const float* b, float* c, uint64_t rows, uint64_t cols,
                          int mode, cudaStream_t stream);
void launch_relu_forward(const float* in, float* out, uint64_t n, cudaStream_t stream);
void launch_relu_backward(const float* grad_out, const float* act_out, float* grad_in, uint64_t n,
                          cudaStream_t stream);
// out[j] = sum_i in[i, j]   (bias gradient)
// With a workspace (`ws_floats` floats, `counter_slots` zeroed counters that every launch
// leaves at zero; one launch at a time) the rows are split over several blocks.
void launch_colsum(const float* in, uint64_t rows, uint64_t cols, float* out, cudaStream_t stream,
                   const float* mask = nullptr, float* ws = nullptr, size_t ws_floats = 0,
                   uint32_t* counters = nullptr, uint32_t counter_slots = 0);

// float64 <-> float32 (round to nearest even), for the gonum facade's host data.
void launch_f64_to_f32(const double* in, float* out, uint64_t n, cudaStream_t stream);
void launch_f32_to_f64(const float* in, double* out, uint64_t n, cudaStream_t stream);

// ---- element-wise family ----------------------------------------------------------
enum EwOp : int {
  EW_ADD = 0, EW_SUB, EW_MUL, EW_DIV, EW_SCALAR_ADD, EW_SCALAR_MUL,
  EW_SIGMOID, EW_SIGMOID_BWD, EW_TANH, EW_TANH_BWD, EW_LEAKY, EW_LEAKY_BWD,
  EW_ELU, EW_ELU_BWD, EW_SWISH, EW_SWISH_BWD, EW_GELU, EW_GELU_BWD,
};
// c[i] = op(a[i], b[i], scalar); b may be null for the one-operand ops.
void launch_elementwise(int op, const float* a, const float* b, float* c, uint64_t n, float scalar,
                        cudaStream_t stream);
// Row softmax over [rows, features].  Forward: out = softmax(in_or_grad) (act unused).
// Backward: out = act * (in_or_grad - dot(in_or_grad, act)) per row.
void launch_softmax(const float* in_or_grad, const float* act, float* out, uint64_t rows,
                    uint64_t features, bool backward, cudaStream_t stream);
// *out = min(*out, smallest i with b[i] == 0); the caller presets *out to ~0.
void launch_first_zero(const float* b, uint64_t n, unsigned long long* out, cudaStream_t stream);

// ---- replication of B over NVSwitch (row-sharded product) --------------------------
// Control words every rank keeps at the same offset of its symmetric buffer.  arrived[s] is
// the last epoch whose data is complete in slot s of this GPU (written by the owner);
// ack[r] on the OWNER's GPU is the last epoch whose products rank r has completed.
struct ReplicaControl {
  uint32_t arrived[2];
  uint32_t pad[14];
  uint32_t ack[16];
};
constexpr int kReplicaMaxRanks = 16;
// `bases` is a device array of each rank's buffer address as this GPU maps it; `mc_dst` the
// multicast address of the destination.  Both kernels report a wait that ran out in `status`
// (code 4: the owner waiting for acknowledgements, 5: a rank waiting for the data).
cudaError_t launch_replicate_send(const void* src, void* mc_dst, uint64_t bytes, void* const* bases,
                                  int world, int my_rank, uint64_t ctrl_offset, int slot,
                                  uint32_t epoch, uint32_t ack_needed, GemmStatus* status, int ctas,
                                  cudaStream_t stream);
cudaError_t launch_replicate_wait(void* const* bases, int owner, int my_rank, uint64_t ctrl_offset,
                                  int slot, uint32_t epoch, uint32_t ack_value, GemmStatus* status,
                                  cudaStream_t stream);

// ---- row-sharded product with the replication of B inside the kernel ---------------
// Every rank multiplies its rows of A by the whole of B, which only the owner holds.  The
// product kernel itself moves B: on the owner, a few CTA pairs first push B, column slab by
// column slab, into the current slot of every rank's symmetric buffer (multimem.st through
// NVSwitch, or plain peer stores when the group has no multicast address) and publish one
// arrival flag per slab, then join the product with correspondingly fewer tiles; on every rank the TMA producer of a tile waits for the flag of the
// tile's slab before its first load, and the last CTA to leave acknowledges the epoch to the
// owner, which may then overwrite the slot two epochs later.  Tiles are visited slab by slab
// while B is arriving, so the product runs beside the transfer instead of behind it.
constexpr int kShardMaxSlabs = 32;
constexpr int kShardMaxRanks = 16;
// Control words at the same offset of every rank's symmetric buffer, zero before the first
// epoch.  `sent`, `exited` and `gave_up` are scratch of the local kernel and zero between
// launches.
struct ShardControl {
  uint32_t arrived[2][kShardMaxSlabs];  // [slot][slab]: last epoch complete on this GPU
  uint32_t ack[kShardMaxRanks];         // on the owner: last epoch rank r has finished reading
  uint32_t sent[kShardMaxSlabs];        // owner: sender warps done with the slab
  uint32_t exited;                      // CTAs of the running product that have left
  uint32_t gave_up;                     // a CTA of the running product gave up
  uint32_t pad[14];
};
static_assert(sizeof(ShardControl) == 512, "ShardControl layout");

struct ShardLink {
  const void* b_src = nullptr;   // owner only: B [K, N] fp16, dense, in this GPU's memory
  void* slot_multicast = nullptr;  // multicast address of the slot, or null: plain peer stores
  void* const* bases = nullptr;  // device array: rank r's symmetric buffer as this GPU maps it
  uint64_t slot_offset = 0;      // byte offset of the slot inside every rank's buffer
  uint64_t ctrl_offset = 0;      // byte offset of the ShardControl inside every rank's buffer
  int world = 1, owner = 0, rank = 0;
  int slot = 0;
  uint32_t epoch = 1;
  uint32_t first_group = 0;      // row tiles (256 rows) visited slab by slab; 0 = choose
  int sender_pairs = -1;         // owner: CTA pairs that push B before they multiply; -1 = choose
  int late_rounds = -1;          // owner: rounds of tiles those pairs are left out of; -1 = choose
  void* trace = nullptr;         // optional timeline of the launch: 128 x uint64 of device memory
};

// C[M,N] = A[M,K] . B[K,N] for this rank's rows, fp16 operands, fp32 accumulate; `b_slot` is
// this rank's own copy of the slot (what the tensor map reads).  N must be a multiple of 8.
// Status codes beyond the GEMM's: 4 the owner ran out waiting for acknowledgements, 6 a
// producer ran out waiting for a slab of B.
const char* launch_gemm_sharded(uint32_t M, uint32_t N, uint32_t K, const void* a, uint64_t a_pitch,
                                const void* b_slot, float* C, uint64_t ldc, const ShardLink& link,
                                GemmStatus* status, int sm_count, cudaStream_t stream);


}  // namespace gonn
