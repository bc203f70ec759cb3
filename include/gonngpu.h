/* C ABI of libgonngpu_cuda.so: the dense-GEMM hot path of tsawler/go-nngpu on
 * NVIDIA B200 (sm_100a).
 *
 * Part 1 re-declares, with unchanged names, argument order and error
 * convention, the entry points of the reference's cgo bridge
 * (internal/cgo/metal_bridge.h) that its MatMul / Transpose / fused
 * linear+activation path binds; each declaration cites the reference line it
 * replaces.  A Go build of the reference links this library in place of the
 * Objective-C/Metal objects without touching its Go callers.
 *
 * Part 2 is additive: entry points (prefix gonngpu_) the reference has no
 * counterpart for - transposed operands, the fp16 path, device selection,
 * pinned staging, statistics.
 *
 * Conventions (same as the reference bridge):
 *   - every function returns 0 on success and a small negative int naming the
 *     failing step otherwise; on failure, when `err` is non-NULL,
 *     err->message is a malloc'ed C string the CALLER frees with
 *     free_c_error_message(); on success err is not touched;
 *   - dimensions are `long`; buffer sizes are in bytes; activation sizes are in
 *     elements; all matrix data is row-major float32;
 *   - every call is blocking: when it returns, the result is complete on the
 *     device (gonngpu_set_blocking(0) lifts that for pipelined callers);
 *   - a NULL DevicePtr means "the calling thread's current device".
 *
 * There is no CPU fallback: without a usable CUDA device every compute entry
 * point fails with -1.
 */
#ifndef GONNGPU_H_
#define GONNGPU_H_

#include <stdbool.h>
#include <stddef.h>

#if defined(__GNUC__)
#define GONNGPU_API __attribute__((visibility("default")))
#else
#define GONNGPU_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- Part 1: the reference bridge's hot-path subset ---------------------- */

typedef void *GPUPtr;          /* metal_bridge.h:9  - opaque buffer handle   */
typedef void *DevicePtr;       /* metal_bridge.h:10 - opaque device handle   */
typedef void *CommandQueuePtr; /* metal_bridge.h:11 - unused, kept for cgo   */

typedef struct {
  char *message;
} CError; /* metal_bridge.h:14-16 */

/* metal_bridge.h:23.  Registers `length_bytes` of caller memory at `data` as a
 * buffer.  The reference aliases that memory (zero copy); here the buffer owns
 * HBM of the same size and remembers `data`: the bytes are copied to the
 * device when the buffer is first used as an input (never, if it is only ever
 * written), so `data` must stay valid until then, as the reference requires
 * for the buffer's whole life.  Errors: -1 no device, -2 stream set-up,
 * -3 allocation. */
GONNGPU_API int create_gpu_buffer(float *data, long length_bytes, GPUPtr *outGPUPtr, DevicePtr *outDevicePtr,
                      CError *err);

/* metal_bridge.h:24.  Copies the buffer's current contents to `data`.
 * Errors: -1 bad handle, -2 length_bytes larger than the buffer, -3 copy. */
GONNGPU_API int retrieve_gpu_buffer_data(GPUPtr gpuPtr, float *data, long length_bytes, CError *err);

/* metal_bridge.h:25.  Frees the buffer; NULL is a no-op returning 0. */
GONNGPU_API int release_gpu_buffer(GPUPtr gpuPtr);

/* metal_bridge.h:250. */
GONNGPU_API void free_c_error_message(char *message);

/* metal_bridge.h:28-34.  C[M,N] = A[M,K] . B[K,N], fp32 in and out, computed
 * on the tensor cores as three tf32 products of hi/lo splits (fp32-level
 * accuracy).  Errors: -1 device, -2 bad buffer, -3 dimension/size mismatch,
 * -4 kernel set-up, -5 scratch allocation, -6 execution. */
GONNGPU_API int perform_mps_matrix_multiplication(GPUPtr aMatrixPtr, long aRows, long aCols, GPUPtr bMatrixPtr,
                                      long bRows, long bCols, GPUPtr resultMatrixPtr,
                                      long resultRows, long resultCols, DevicePtr mtlDevicePtr,
                                      CError *err);

/* metal_bridge.h:36-41.  out[j,i] = in[i,j], bit-exact.  Errors: -1 device,
 * -2 dimensions, -3 bad buffer, -6 execution. */
GONNGPU_API int perform_mps_matrix_transpose(GPUPtr inputMatrixPtr, long inputRows, long inputCols,
                                 GPUPtr outputMatrixPtr, long outputRows, long outputCols,
                                 DevicePtr mtlDevicePtr, CError *err);

/* metal_bridge.h:52-58.  The four bias-broadcast patterns [M,N]+[1,N],
 * [1,N]+[M,N], [M,N]+[M,1], [M,1]+[M,N].  Errors: -3 bad buffer, -2 any other
 * shape combination, -6 execution. */
GONNGPU_API int perform_mps_matrix_add_broadcast(GPUPtr aMatrixPtr, long aRows, long aCols, GPUPtr bMatrixPtr,
                                     long bRows, long bCols, GPUPtr resultMatrixPtr,
                                     long resultRows, long resultCols, DevicePtr mtlDevicePtr,
                                     CError *err);

/* metal_bridge.h:259-264.  out[i] = max(0, in[i]).  Errors: -1 bad buffer. */
GONNGPU_API int perform_activation_relu_forward(GPUPtr inputPtr, long size, GPUPtr outputPtr,
                                    DevicePtr mtlDevicePtr, CError *err);

/* metal_bridge.h:266-271.  gradIn[i] = actOut[i] > 0 ? gradOut[i] : 0. */
GONNGPU_API int perform_activation_relu_backward(GPUPtr gradOutputPtr, GPUPtr activationOutputPtr, long size,
                                     GPUPtr gradInputPtr, DevicePtr mtlDevicePtr, CError *err);

/* ---- element-wise family used between the GEMMs of eager layer chains -------
 * (CPU loops in the reference; streaming kernels here, so the data stays in HBM) */

/* metal_bridge.h:44-50, 60-82.  c = a (op) b for equal shapes.  Errors: -2
 * shapes differ, -1 device, -3 bad buffer, -6 execution; the divide also -4
 * "Division by zero encountered at element i" for the first zero divisor, with
 * the elements before i written and the rest left as they were, as the
 * reference's loop does (metal_bridge_matrix.m:470-479). */
GONNGPU_API int perform_mps_matrix_add(GPUPtr aMatrixPtr, long aRows, long aCols, GPUPtr bMatrixPtr, long bRows,
                           long bCols, GPUPtr resultMatrixPtr, long resultRows, long resultCols,
                           DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_mps_matrix_subtract(GPUPtr aMatrixPtr, long aRows, long aCols, GPUPtr bMatrixPtr, long bRows,
                                long bCols, GPUPtr resultMatrixPtr, long resultRows, long resultCols,
                                DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_mps_matrix_element_multiply(GPUPtr aMatrixPtr, long aRows, long aCols, GPUPtr bMatrixPtr,
                                        long bRows, long bCols, GPUPtr resultMatrixPtr, long resultRows,
                                        long resultCols, DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_mps_matrix_element_divide(GPUPtr aMatrixPtr, long aRows, long aCols, GPUPtr bMatrixPtr,
                                      long bRows, long bCols, GPUPtr resultMatrixPtr, long resultRows,
                                      long resultCols, DevicePtr mtlDevicePtr, CError *err);
/* metal_bridge.h:85-99.  result = input + scalar / input * scalar.  Errors: -1 bad buffer. */
GONNGPU_API int perform_mps_matrix_scalar_add(GPUPtr inputMatrixPtr, long rows, long cols, float scalar,
                                  GPUPtr resultMatrixPtr, DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_mps_matrix_scalar_multiply(GPUPtr inputMatrixPtr, long rows, long cols, float scalar,
                                       GPUPtr resultMatrixPtr, DevicePtr mtlDevicePtr, CError *err);
/* metal_bridge.h:274-301, 334-348.  Sigmoid and tanh clamp their input to
 * [-88, 88] (metal_bridge_activation.m:105, 166); the backward forms take the
 * activation OUTPUT.  Errors: -1 bad buffer. */
GONNGPU_API int perform_activation_sigmoid_forward(GPUPtr inputPtr, long size, GPUPtr outputPtr,
                                       DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_activation_sigmoid_backward(GPUPtr gradOutputPtr, GPUPtr activationOutputPtr, long size,
                                        GPUPtr gradInputPtr, DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_activation_tanh_forward(GPUPtr inputPtr, long size, GPUPtr outputPtr,
                                    DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_activation_tanh_backward(GPUPtr gradOutputPtr, GPUPtr activationOutputPtr, long size,
                                     GPUPtr gradInputPtr, DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_activation_leaky_relu_forward(GPUPtr inputPtr, long size, float alpha, GPUPtr outputPtr,
                                          DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_activation_leaky_relu_backward(GPUPtr gradOutputPtr, GPUPtr activationOutputPtr,
                                           long size, float alpha, GPUPtr gradInputPtr,
                                           DevicePtr mtlDevicePtr, CError *err);
/* metal_bridge.h:304-331.  Softmax of one vector (1d) or of each row of
 * [batchSize, features] (2d): exp(x - rowmax) / sum; backward is
 * grad_in = y * (grad_out - dot(grad_out, y)) per row.  Errors: -1 bad buffer. */
GONNGPU_API int perform_activation_softmax_1d_forward(GPUPtr inputPtr, long size, GPUPtr outputPtr,
                                          DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_activation_softmax_1d_backward(GPUPtr gradOutputPtr, GPUPtr activationOutputPtr,
                                           long size, GPUPtr gradInputPtr, DevicePtr mtlDevicePtr,
                                           CError *err);
GONNGPU_API int perform_activation_softmax_2d_forward(GPUPtr inputPtr, long batchSize, long features,
                                          GPUPtr outputPtr, DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_activation_softmax_2d_backward(GPUPtr gradOutputPtr, GPUPtr activationOutputPtr,
                                           long batchSize, long features, GPUPtr gradInputPtr,
                                           DevicePtr mtlDevicePtr, CError *err);
/* metal_bridge.h:351-395.  ELU(alpha), Swish and tanh-GELU.  The backward
 * forms take the activation OUTPUT; Swish and GELU recover the input from it
 * with three Newton steps, as metal_bridge_activation.m:570-600, 665-699 do. */
GONNGPU_API int perform_activation_elu_forward(GPUPtr inputPtr, long size, float alpha, GPUPtr outputPtr,
                                   DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_activation_elu_backward(GPUPtr gradOutputPtr, GPUPtr activationOutputPtr, long size,
                                    float alpha, GPUPtr gradInputPtr, DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_activation_swish_forward(GPUPtr inputPtr, long size, GPUPtr outputPtr,
                                     DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_activation_swish_backward(GPUPtr gradOutputPtr, GPUPtr activationOutputPtr, long size,
                                      GPUPtr gradInputPtr, DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_activation_gelu_forward(GPUPtr inputPtr, long size, GPUPtr outputPtr,
                                    DevicePtr mtlDevicePtr, CError *err);
GONNGPU_API int perform_activation_gelu_backward(GPUPtr gradOutputPtr, GPUPtr activationOutputPtr, long size,
                                     GPUPtr gradInputPtr, DevicePtr mtlDevicePtr, CError *err);

/* metal_bridge.h:1348-1353.  output[b,o] = act(sum_i input[b,i]*weight[i,o] +
 * bias[o]); `bias` may be NULL.  activation_type is decoded as the reference's
 * kernel decodes it (default.metal:488-506): 0 ReLU, 1 LeakyReLU(alpha),
 * 2 Sigmoid, 3 Tanh, 4 tanh-GELU, anything else identity.  Bias and activation
 * run in the GEMM epilogue.  Errors: -1 device or bad buffer, -3 sizes,
 * -4/-5/-6 as for the multiplication. */
GONNGPU_API int perform_fused_linear_activation(GPUPtr input, long batch_size, long input_size, GPUPtr weight,
                                    long output_size, GPUPtr bias, int activation_type, float alpha,
                                    GPUPtr output, DevicePtr device, CError *error);

/* metal_bridge.h:1423-1429.  C = alpha * A[M,K].B[K,N] + beta * C.
 * Errors: -1 device, -2 bad buffer, -3 sizes/kernel set-up, -6 execution. */
GONNGPU_API int perform_optimized_gemm(GPUPtr aPtr, GPUPtr bPtr, GPUPtr cPtr, long M, long N, long K,
                           float alpha, float beta, DevicePtr mtlDevicePtr, CError *err);

/* metal_bridge.h:1432-1437.  C[b] = A[b] . B[b] for b < batchSize over the
 * contiguous stacks A[batch,M,K], B[batch,K,N], C[batch,M,N] (fp32, computed like
 * the single product); one launch walks the tiles of every batch.
 * Errors: -1 device, -2 bad buffer, -3 dimensions or kernel set-up, -6 execution. */
GONNGPU_API int perform_batch_matmul_optimized(GPUPtr aPtr, GPUPtr bPtr, GPUPtr cPtr, long batchSize, long M,
                                   long N, long K, DevicePtr mtlDevicePtr, CError *err);

/* metal_bridge.h:1803.  Host memory for the reference's unified-memory
 * adapter: page-locked, zero-filled, 16 KiB aligned; NULL on failure.  Freed by
 * gonngpu_host_free(). */
GONNGPU_API void *allocateSharedMemory(long size);

/* metal_bridge.h:1804.  A buffer handle over memory from allocateSharedMemory
 * (same lazy-upload rule as create_gpu_buffer); NULL on failure. */
GONNGPU_API void *createGPUBufferFromSharedMemory(void *device, void *memory, long size);

/* ---- Part 2: additive entry points (no counterpart in the reference) ----- */

/* Precision of gonngpu_matmul_ex. */
#define GONNGPU_FP32_3XTF32 0 /* fp32 accuracy: x = hi + lo, three MMAs per product:
                                 hi.hi in tf32, hi.lo + lo.hi in tf32 (small products)
                                 or bf16 (large ones); <= 1e-5 rel. Frobenius vs float64 */
#define GONNGPU_FP16_RN 1     /* inputs rounded to fp16 (nearest even), fp32 accum. */
#define GONNGPU_FP16_TRUNC 2  /* inputs truncated to fp16 exactly as the reference's \
                                 Float32ToFloatMP16 (mixed-precision.go:106-151)    */
#define GONNGPU_ACT_NONE (-1)

/* C[M,N] = act(alpha * op(A).op(B) + beta * C + bias[N]) with op(X) = X or its
 * transpose (transX != 0; no transposed copy is made), any precision above.
 * `bias` may be NULL.  Replaces the Transpose+MatMul pairs of the reference's
 * backward passes (gpu/matrix/layers.go:77-96) and its ForwardFloat16
 * (gpu/matrix/mixed-precision.go:315-358).  Errors as
 * perform_mps_matrix_multiplication. */
GONNGPU_API int gonngpu_matmul_ex(GPUPtr a, long aRows, long aCols, int transA, GPUPtr b, long bRows,
                      long bCols, int transB, GPUPtr c, long cRows, long cCols, int precision,
                      float alpha, float beta, GPUPtr bias, int activation_type,
                      float activation_param, CError *err);

/* The same GEMM on device-resident fp16 operands, for callers that keep their
 * matrices in HBM as IEEE fp16 (what the reference's ForwardFloat16 simulates
 * with fp16-valued float32).  `a` and `b` are device pointers to the matrices
 * as stored ([rows, cols], pitch in elements); both pointers must be 16-byte
 * aligned and both pitches multiples of 8.  `c` is float32 [M,N] with leading
 * dimension ldc; `bias` (float32[N]) may be NULL.  All pointers belong to the
 * current device.  Errors: -1 device, -2 NULL pointer, -3 dimensions or
 * alignment, -4 kernel set-up, -6 execution. */
GONNGPU_API int gonngpu_gemm_f16_device(const void *a, long aRows, long aCols, long aPitch, int transA,
                            const void *b, long bRows, long bCols, long bPitch, int transB,
                            float *c, long ldc, float alpha, float beta, const float *bias,
                            int activation_type, float activation_param, CError *err);
/* float32 [rows, cols] (dense) -> fp16 [rows, dstPitch] on the device; mode is
 * GONNGPU_FP16_RN or GONNGPU_FP16_TRUNC. */
GONNGPU_API int gonngpu_convert_f16_device(const float *src, long rows, long cols, void *dst, long dstPitch,
                               int mode, CError *err);

/* Replication of B for the row-sharded MatMul (one process per GPU, A split by
 * rows, every GPU needs all of B).  The reference has one device and no such
 * step; these two calls are the NVLink replication the multi-GPU path adds
 * around gonngpu_gemm_f16_device.
 *
 * The ranks share a SYMMETRIC buffer: the same allocation on every GPU, mapped
 * into every process (`bases_dev` is a DEVICE array of `world` addresses: rank
 * r's buffer as the calling GPU maps it) and bound to an NVSwitch multicast
 * address.  It holds two destination slots and, at byte `ctrl_offset`, 128
 * bytes of control words that must be zero before the first call.  Allocation,
 * mapping and the multicast binding are the caller's (CUDA virtual-memory API,
 * or torch.distributed._symmetric_memory as bench.py does).
 *
 * gonngpu_replicate_send (owner of B only): copies `bytes` from `src` (device
 * memory of the current GPU) to `dst_multicast` (the multicast address of the
 * slot) with multimem.st, so every GPU of the group, the owner included,
 * receives a copy while the owner's NVLink carries B once; then marks the slot
 * as holding `epoch` on every rank.  Before writing it waits until every rank
 * has acknowledged epoch `ack_needed` (pass the last epoch that used this slot,
 * 0 if none).  `ctas`: thread blocks to use, 0 = one per SM (16 already reach the
 * link rate).  `stream`: cudaStream_t to enqueue on, NULL = the library's
 * stream; on a stream of its own the push runs beside the products of the
 * library's stream (B in column slabs: slab j+1 travels while slab j is being
 * multiplied) and needs no ordering against them, because the
 * acknowledgements already keep it from overwriting a slot that is still read.
 * Two sends of one GPU must not run at the same time (they share a counter):
 * keep them on one stream.
 * gonngpu_replicate_wait (every rank, the owner included, before the product
 * that reads the slot): tells the owner that all work queued earlier on this
 * library's stream is complete up to epoch `ack_value` (pass epoch - 1), then
 * holds the stream until the slot holds `epoch`.
 * Epochs start at 1 and grow by one per replication; slot = epoch % 2 lets the
 * owner fill one slot while products still read the other.
 *
 * Both are enqueued on the library's stream like every other call.  Their waits
 * are bounded (1.5 s): a wait that runs out is reported as -6 by this call (blocking
 * mode) or by gonngpu_synchronize, with status code 4 (owner, acknowledgements) or
 * 5 (data did not arrive).  Errors: -1 device, -2 NULL pointer, -3 arguments,
 * -4 launch, -6 execution. */
GONNGPU_API int gonngpu_replicate_send(const void *src, void *dst_multicast, long bytes,
                           void *const *bases_dev, int world, int rank, long ctrl_offset, int slot,
                           unsigned epoch, unsigned ack_needed, int ctas, void *stream, CError *err);
GONNGPU_API int gonngpu_replicate_wait(void *const *bases_dev, int world, int owner, int rank,
                           long ctrl_offset, int slot, unsigned epoch, unsigned ack_value,
                           CError *err);

/* The row-sharded MatMul as ONE call, for a process that sees several GPUs: the multi-GPU
 * form of matrix.MatMul (gpu/matrix/matrix.go:53-105; the reference has one device).
 * C[aRows, bCols] = A . B with all three matrices in HOST memory, float32, row-major, dense.
 * A is split into contiguous row blocks over devices 0 .. n_devices-1 (gonngpu_shard_plan;
 * n_devices 0 = every visible device), B crosses PCIe once (to device 0), is converted to
 * fp16 there and copied to the other devices over NVLink (peer copies), and every device
 * streams its own rows: upload, fp32 -> fp16, product on the tensor cores, and the rows of
 * C straight back into the caller's `c` at their row offset, block by block, so that both
 * PCIe directions of every GPU and the tensor cores overlap.  The kernels read their own
 * GPU's memory only.  `precision` is GONNGPU_FP16_RN or GONNGPU_FP16_TRUNC.
 * The host matrices should be page-locked (gonngpu_host_alloc); other memory is locked for
 * the duration of the call, which is slow.  Blocking: C is complete on return.
 * Errors: -1 device, -2 NULL pointer, -3 dimensions or precision, -4 kernel set-up,
 * -5 memory, -6 execution. */
GONNGPU_API int gonngpu_matmul_sharded(const float *a, long aRows, long aCols, const float *b, long bRows,
                           long bCols, float *c, int precision, int n_devices, CError *err);
/* The row block [*first_row, *end_row) of `device` when `rows` rows are split over
 * `n_devices` (blocks of ceil(rows / n_devices) rounded up to the 256-row tile; trailing
 * blocks may be short or empty).  Returns -3 on bad arguments. */
GONNGPU_API int gonngpu_shard_plan(long rows, int n_devices, int device, long *first_row, long *end_row);

/* The row-sharded MatMul with the replication of B INSIDE the product kernel: one
 * launch per rank and step, nothing else on the stream.  No counterpart in the
 * reference (one device); it is the multi-GPU form of matrix.MatMul
 * (gpu/matrix/matrix.go:53-105) for a tall A split by rows.
 *
 * Rank `rank` computes C[aRows, bCols] = A . B for its own rows of A (fp16,
 * [aRows, aCols], pitch aPitch elements) with B [aCols, bCols] (fp16, dense, bCols
 * a multiple of 8) that only rank `owner` holds, at `b_src` in its own memory
 * (NULL on the other ranks).  The ranks share a symmetric buffer as for
 * gonngpu_replicate_send: `local_base` is this rank's own mapping of it,
 * `bases_dev` the device array of every rank's mapping, `multicast_base` its
 * NVSwitch multicast address (NULL: the owner writes every rank's copy with plain
 * peer stores instead).  At `slots_offset` it holds two slots of aCols*bCols*2
 * bytes, at `ctrl_offset` 512 bytes of control words, zero before epoch 1.
 *
 * On the owner a few CTA pairs (32 of the 148 SMs) first push B into slot
 * epoch % 2 of every rank, 256-column slab by slab, raising one arrival flag per
 * slab, and then join the product with as many tiles fewer as the push took; on
 * every rank a tile's loads wait for the flag of its slab, and the first
 * `first_group` 256-row tiles (0 = chosen from the group size) are visited slab by
 * slab, so the product runs while B is still arriving.  The last CTA to leave acknowledges the
 * epoch to the owner, which overwrites a slot only when every rank has
 * acknowledged the epoch that used it before (epoch - 2).  Every rank calls this
 * once per step with the same epoch: 1, 2, 3 ...  The kernels read B from their
 * own GPU's memory only.
 *
 * Enqueued on the library's stream.  Every wait is bounded (1 to 1.5 s); one that ran
 * out is reported as -6 (blocking mode) or by gonngpu_synchronize, with status
 * code 4 (owner: acknowledgements missing) or 6 (a slab of B did not arrive;
 * where = slab, tile, k block = epoch); no acknowledgement is then sent.
 * Errors: -1 device, -2 NULL pointer, -3 arguments, -4 kernel set-up, -6 execution. */
GONNGPU_API int gonngpu_gemm_f16_sharded(const void *a, long aRows, long aCols, long aPitch,
                             const void *b_src, long bCols, void *local_base,
                             void *const *bases_dev, void *multicast_base, int world, int owner,
                             int rank, long slots_offset, long ctrl_offset, unsigned epoch, float *c,
                             long ldc, int first_group, CError *err);

/* No counterpart in the reference.  C[M,N] = A[M,K] . B[K,N] on the fp16 path
 * (inputs rounded to fp16, fp32 accumulate, as GONNGPU_FP16_RN) for callers
 * that must not allocate: programs that gave all of HBM to their own arena at
 * start-up, or that call from a loop where a cudaMalloc / cudaFree would stall
 * the whole device.  a, b, c are float32 DEVICE pointers of the current device
 * (row-major, dense); nothing is allocated or freed: the fp16 operand planes
 * live in a fixed array inside the library, GONNGPU_STATIC_SCRATCH_BYTES of HBM
 * on every GPU that loads it.  Operands whose planes (rows x columns padded to
 * 64, 2 bytes each, A and B together) exceed that are refused with -3.
 * `stream` is the cudaStream_t to run on (NULL: the default stream); every call
 * waits for its work with cudaStreamSynchronize before it returns.  The first
 * call on a device does the set-up: it looks up the array's address and makes
 * CUDA load the kernels, for which the driver itself takes device memory.  Make
 * one small warm-up call per device first: before the arena takes the rest of
 * HBM and before any stream capture is begun (or start the process with
 * CUDA_MODULE_LOADING=EAGER).  All calls share the array, so calls that overlap
 * on the GPU race; serialise them.
 * Errors: -1 device, -2 NULL pointer, -3 dimensions or size, -4 kernel set-up,
 * -6 execution. */
#define GONNGPU_STATIC_SCRATCH_BYTES (32l << 20)
GONNGPU_API int gonngpu_matmul_f16_static_scratch(const float *a, long aRows, long aCols, const float *b,
                                      long bRows, long bCols, float *c, void *stream, CError *err);

/* Backward pass of a linear layer Y = act(X.W + b), all three gradients in one
 * call (replaces, in gpu/matrix/layers.go:77-96,139-141 and
 * fused-operations.go:467-578, ReLUBackward + Transpose + MatMul + Transpose +
 * MatMul + sumAlongAxis):
 *   dAct = dY (.) [actOut > 0]   when actOut is non-NULL (ReLU derivative,
 *                                metal_bridge_activation.m:74-77), else dY
 *   dW[in,out] = X^T . dAct,  dX[batch,in] = dAct . W^T,  db[out] = column sums of dAct
 * x is [batch,in], w is [in,out], dy and actOut are [batch,out].  Any of dx, dw,
 * db may be NULL (x may be NULL when dw is, w when dx is).  The mask is applied
 * while the tensor-core operand planes of dY are written, so the masked
 * gradient is never materialised; both GEMMs read their operands transposed in
 * place (fp32 accuracy, 3xTF32).  Errors as perform_mps_matrix_multiplication. */
GONNGPU_API int gonngpu_linear_backward(GPUPtr x, GPUPtr w, GPUPtr dy, GPUPtr actOut, long batch, long in_size,
                            long out_size, GPUPtr dx, GPUPtr dw, GPUPtr db, CError *err);

/* out[j] = sum_i in[i,j] (bias gradient, gpu/matrix/layers.go:281-294). */
GONNGPU_API int gonngpu_column_sum(GPUPtr in, long rows, long cols, GPUPtr out, CError *err);

/* Device-only buffer of `length_bytes` (contents undefined). */
GONNGPU_API int gonngpu_alloc_device_buffer(long length_bytes, GPUPtr *out, CError *err);
/* Handle over device memory the caller owns (for example a torch tensor). */
GONNGPU_API int gonngpu_wrap_device_memory(void *device_ptr, long length_bytes, GPUPtr *out, CError *err);
/* Device address behind a handle (after any pending upload), or NULL. */
GONNGPU_API void *gonngpu_device_address(GPUPtr buffer);
/* Copies `length_bytes` from host `data` into the buffer now. */
GONNGPU_API int gonngpu_upload(GPUPtr buffer, const float *data, long length_bytes, CError *err);
/* float64 host data into / out of a float32 buffer, converted on the device
 * (round to nearest even, as Go's float32(x)).  They replace the per-element
 * host loops of FromGonum / ToGonum (gpu/matrix/gonum-compat.go:14-42, 322-334):
 * the Go side passes mat.Dense.RawMatrix().Data.  `count` is in elements.
 * Both return after the data has arrived.  Errors: -1 bad handle, -2 length,
 * -3 copy or memory failure. */
GONNGPU_API int gonngpu_upload_f64(GPUPtr buffer, const double *data, long count, CError *err);
GONNGPU_API int gonngpu_retrieve_f64(GPUPtr buffer, double *data, long count, CError *err);
/* Tells the library the caller changed the device contents behind a wrapped
 * handle, so cached operand planes are rebuilt. */
GONNGPU_API int gonngpu_mark_modified(GPUPtr buffer);

/* Page-locked host memory (fast, asynchronous copies). */
GONNGPU_API void *gonngpu_host_alloc(long bytes);
GONNGPU_API void gonngpu_host_free(void *p);

/* Host-side fault injection for tests of the error paths: the `nth` next device allocation
 * (`kind` "alloc"), host-to-device copy ("h2d") or device-to-host copy ("d2h") of this
 * library reports failure before the device is asked for anything; the entry point that
 * needed it returns its documented error code and message, and the library's state (handles,
 * cache, statistics) stays consistent.  nth 0 disarms.  No GPU is made to fail.  Returns -3
 * for an unknown kind. */
GONNGPU_API int gonngpu_inject_fault(const char *kind, int nth);

GONNGPU_API int gonngpu_device_count(void);
GONNGPU_API int gonngpu_set_device(int ordinal); /* device used by later calls of this process */
GONNGPU_API int gonngpu_get_device(void);
/* cudaStream_t every kernel and copy of the current device is enqueued on. */
GONNGPU_API void *gonngpu_stream(void);
/* 1 (default): every entry point waits for its work.  0: work is only enqueued;
 * call gonngpu_synchronize() before reading results. */
GONNGPU_API int gonngpu_set_blocking(int blocking);
GONNGPU_API int gonngpu_synchronize(CError *err);
/* Keeps (1, default) or drops (0) the converted operand planes of a buffer
 * between calls while its contents are unchanged. */
GONNGPU_API int gonngpu_set_plane_cache(int enabled);
/* GEMM tile override for experiments: block_n in {0 = auto, 32, 64, 128, 256},
 * max_ctas 0 = one per SM. */
GONNGPU_API int gonngpu_set_gemm_tuning(int block_n, int max_ctas);
/* fp16 GEMM on CTA pairs (2-SM MMA): -1 (default) chosen by problem size,
 * 0 never, 1 force 256-row tiles (block_n 0, 128 or 256), 2 force 512-row
 * tiles (block_n 0 or 256). */
GONNGPU_API int gonngpu_set_gemm_pair_mode(int mode);
/* gonngpu_gemm_f16_sharded on the owner of B: how many CTA pairs push B before they
 * multiply (1..74) and how many rounds of tiles they are left out of (0..64); -1 (default)
 * lets the library choose from the sizes.  For measurements. */
GONNGPU_API int gonngpu_set_sharded_tuning(int sender_pairs, int late_rounds);
/* Timeline of the next gonngpu_gemm_f16_sharded launches, for measurements: `device_words`
 * is device memory of the current GPU holding 128 64-bit words (NULL switches it off), which
 * every launch fills with %globaltimer nanoseconds: [0] start, [1 + s] slab s published by
 * the owner, [40 + s] slab s first seen by this rank (a minimum: preset the words to ~0),
 * [80] last CTA leaving. */
GONNGPU_API int gonngpu_set_sharded_trace(void *device_words);
/* Split-K of the fp32 GEMM (products with too few tiles to fill the GPU share a
 * tile's K range among several SMs and add the partial sums in a fixed order):
 * 0 (default) chosen by problem size, 1 never, n > 1 force n splits. */
GONNGPU_API int gonngpu_set_gemm_split_k(int splits);

/* Released buffers and operand planes are kept in a per-device cache (the
 * reference's callers create and release a result buffer per MatMul, and
 * cudaMalloc/cudaFree of gigabytes cost milliseconds).  This returns the cache
 * to the driver and reports the bytes freed. */
GONNGPU_API long gonngpu_trim_cache(void);

/* out[0] bytes of HBM held by live buffers and planes, [1] host->device bytes,
 * [2] device->host bytes, [3] kernels launched, [4] GEMM kernels launched,
 * [5] buffers alive, [6] scratch (operand plane) bytes held, [7] bytes in the
 * released-block cache. */
GONNGPU_API void gonngpu_get_stats(long out[8]);
/* Status words of the last GEMM kernel on the current device: code (0 fine,
 * 1 producer / 2 MMA issuer / 3 epilogue wait ran out), where, tile, k block. */
GONNGPU_API void gonngpu_last_kernel_status(unsigned out[4]);
GONNGPU_API const char *gonngpu_version(void);

#ifdef __cplusplus
}
#endif
#endif /* GONNGPU_H_ */
