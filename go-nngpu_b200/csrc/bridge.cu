// C-ABI bridge: buffer handles, host<->device staging, per-device streams, the
// reference's error convention, argument validation, and the dispatch of every
// exported entry point onto the sm_100a kernels.  It replaces the reference's
// Objective-C bridge files internal/cgo/metal_bridge_{buffer,matrix,fused,
// kernels,activation,common}.m for the dense-GEMM path.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <map>
#include <mutex>
#include <unordered_set>
#include <vector>

#include "../../include/gonngpu.h"
#include "kernels.h"

namespace {

using gonn::GemmStatus;

constexpr uint64_t kMagic = 0x676f6e6e67707562ull;  // "gonngpub"
constexpr int kMaxDevices = 16;
constexpr size_t kStageBytes = 16u << 20;  // pinned staging chunk

std::recursive_mutex g_mu;

// Waits for a stream with the library's lock released, so that other threads of the caller
// (the reference allows goroutine-concurrent calls) can enqueue their own uploads and kernels
// instead of queueing behind a wait.  The calling thread holds g_mu (every entry point takes it);
// everything the waiter touches afterwards is re-read under the lock.
cudaError_t wait_stream(cudaStream_t s) {
  g_mu.unlock();
  const cudaError_t e = cudaStreamSynchronize(s);
  g_mu.lock();
  return e;
}

// Converted copy of a buffer for the tensor cores ("operand plane").
struct Plane {
  void* p0 = nullptr;
  void* p1 = nullptr;
  size_t bytes = 0;  // per plane
  uint64_t version = ~0ull;
  uint64_t rows = 0, cols = 0, pitch = 0;
};

struct Buffer {
  uint64_t magic = kMagic;
  int device = 0;
  float* dptr = nullptr;
  size_t bytes = 0;
  bool owns = true;
  float* host = nullptr;      // caller memory registered by create_gpu_buffer
  bool host_pending = false;  // host bytes not yet copied to the device
  uint64_t version = 1;       // bumped whenever the device contents change
  bool host_current = false;  // the registered host memory already holds the device contents
  Plane f16[2];               // [F16_RN], [F16_TRUNC]
  Plane tf32;
  Plane tf32x;                // hi as fp32 + bf16(hi), bf16(lo): operands of the fp32 CTA-pair kernel
};

struct Device {
  int ordinal = -1;
  bool ready = false;
  cudaStream_t stream = nullptr;
  cudaStream_t copy_stream = nullptr;  // host -> device side stream of the streamed MatMul
  cudaStream_t d2h_stream = nullptr;   // device -> host side stream of the streamed MatMul
  int sm_count = 0;
  GemmStatus* status_host = nullptr;  // mapped pinned memory the kernels report into
  GemmStatus* status_dev = nullptr;
  GemmStatus last_status{};
  unsigned long long* first_zero_dev = nullptr;  // scratch word of the element-wise divide
  float* splitk_ws = nullptr;                    // partial sums of split fp32 products
  uint32_t* splitk_counters = nullptr;           // per-tile arrival counters (zero between launches)
  void* stage[2] = {nullptr, nullptr};
  cudaEvent_t stage_ev[2] = {nullptr, nullptr};
  // events of the streamed product (re-recorded block after block: a stream's wait keeps the
  // record that was current when the wait was enqueued)
  cudaEvent_t ev_start = nullptr, ev_up = nullptr, ev_done = nullptr;
};

Device g_dev[kMaxDevices];
int g_current = 0;
bool g_blocking = true;
bool g_plane_cache = true;
gonn::GemmTuning g_tune;
int g_shard_sender_pairs = -1, g_shard_late_rounds = -1;  // gonngpu_set_sharded_tuning
void* g_shard_trace = nullptr;                            // gonngpu_set_sharded_trace
// Split-K workspace per device: room for one wave of 128 x 256 partial tiles.
constexpr size_t kSplitKBytes = size_t(24) << 20;
constexpr uint32_t kSplitKSlots = 4096;

// The tuning of a launch on the device's own compute stream: the global settings
// plus that device's split-K workspace (launches on one stream never overlap).
gonn::GemmTuning tune_for(const Device& d) {
  gonn::GemmTuning t = g_tune;
  t.splitk_ws = d.splitk_ws;
  t.splitk_ws_bytes = kSplitKBytes;
  t.splitk_counters = d.splitk_counters;
  t.splitk_counter_slots = kSplitKSlots;
  return t;
}
std::unordered_set<Buffer*> g_buffers;
long g_stats[8] = {0, 0, 0, 0, 0, 0, 0, 0};

// Device-memory cache.  cudaMalloc / cudaFree cost from tens of microseconds to milliseconds
// and cudaFree waits for the device, and the reference's callers create and release a
// result buffer per operation (a layer stack: a dozen per step, many of them small: logits,
// bias gradients), so freed blocks are kept (per device, keyed by size, up to kPoolCapBytes;
// blocks below 1 MiB in 512-byte size classes, up to kSmallPoolCapBytes of them) and handed
// out again.  Measured on the MLP step of configuration 3 through the layer stack: with the
// small blocks freed and allocated every step the host spent the whole step waiting in
// cudaFree.
constexpr size_t kPoolCapBytes = size_t(24) << 30;
constexpr size_t kSmallBlock = size_t(1) << 20;
constexpr size_t kSmallPoolCapBytes = size_t(256) << 20;
std::multimap<size_t, void*> g_pool[kMaxDevices];
size_t g_pool_bytes[kMaxDevices] = {};
size_t g_small_pool_bytes[kMaxDevices] = {};
inline size_t pool_class(size_t bytes) {
  return bytes < kSmallBlock ? (bytes + 511) / 512 * 512 + (bytes == 0 ? 512 : 0) : bytes;
}

// Host-side fault injection (gonngpu_inject_fault): the n-th next allocation / host-to-device
// copy / device-to-host copy reports failure BEFORE anything is asked of the device, so that
// the error paths can be tested without making a GPU fail.  0 = disarmed.
enum FaultKind { FAULT_ALLOC = 0, FAULT_H2D = 1, FAULT_D2H = 2, FAULT_KINDS = 3 };
int g_fault_countdown[FAULT_KINDS] = {0, 0, 0};
bool fault_hit(FaultKind k) {
  if (g_fault_countdown[k] <= 0) return false;
  return --g_fault_countdown[k] == 0;
}

cudaError_t pool_alloc(int dev, void** out, size_t bytes) {
  if (fault_hit(FAULT_ALLOC)) {
    *out = nullptr;
    return cudaErrorMemoryAllocation;
  }
  bytes = pool_class(bytes);
  auto& pool = g_pool[dev];
  auto it = pool.find(bytes);
  if (it != pool.end()) {
    *out = it->second;
    g_pool_bytes[dev] -= bytes;
    if (bytes < kSmallBlock) g_small_pool_bytes[dev] -= bytes;
    pool.erase(it);
    return cudaSuccess;
  }
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess && !pool.empty()) {  // give the cache back and retry once
    cudaGetLastError();
    for (auto& kv : pool) cudaFree(kv.second);
    pool.clear();
    g_pool_bytes[dev] = 0;
    g_small_pool_bytes[dev] = 0;
    e = cudaMalloc(out, bytes);
  }
  return e;
}

// `dev` must be current.  The caller has made sure no work still uses `p`, or that
// whatever uses it next is queued behind that work on the device's compute stream.
void pool_free(int dev, void* p, size_t bytes) {
  if (!p) return;
  bytes = pool_class(bytes);
  const bool small = bytes < kSmallBlock;
  if (g_pool_bytes[dev] + bytes <= kPoolCapBytes &&
      (!small || g_small_pool_bytes[dev] + bytes <= kSmallPoolCapBytes)) {
    g_pool[dev].emplace(bytes, p);
    g_pool_bytes[dev] += bytes;
    if (small) g_small_pool_bytes[dev] += bytes;
  } else {
    cudaFree(p);
  }
}

void set_error(CError* err, const char* fmt, ...) {
  if (!err) return;
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  err->message = strdup(buf);
}

// Brings up the device's streams and staging memory once.
// 0 ok, -1 no usable device, -2 stream / staging set-up failed.
int ensure_device(int ordinal, CError* err) {
  if (ordinal < 0 || ordinal >= kMaxDevices) {
    set_error(err, "CUDA device ordinal %d out of range.", ordinal);
    return -1;
  }
  Device& d = g_dev[ordinal];
  if (cudaSetDevice(ordinal) != cudaSuccess) {
    cudaGetLastError();
    set_error(err, "Could not select CUDA device %d (no usable GPU).", ordinal);
    return -1;
  }
  if (d.ready) return 0;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, ordinal) != cudaSuccess) {
    cudaGetLastError();
    set_error(err, "Could not query CUDA device %d.", ordinal);
    return -1;
  }
  if (prop.major != 10) {
    set_error(err, "Device %d is sm_%d%d; this library contains sm_100a code only.", ordinal,
              prop.major, prop.minor);
    return -1;
  }
  d.ordinal = ordinal;
  d.sm_count = prop.multiProcessorCount;
  bool ok = cudaStreamCreateWithFlags(&d.stream, cudaStreamNonBlocking) == cudaSuccess &&
            cudaStreamCreateWithFlags(&d.copy_stream, cudaStreamNonBlocking) == cudaSuccess &&
            cudaStreamCreateWithFlags(&d.d2h_stream, cudaStreamNonBlocking) == cudaSuccess &&
            cudaHostAlloc(reinterpret_cast<void**>(&d.status_host), sizeof(GemmStatus),
                          cudaHostAllocMapped) == cudaSuccess &&
            cudaHostGetDevicePointer(reinterpret_cast<void**>(&d.status_dev), d.status_host, 0) ==
                cudaSuccess &&
            cudaMalloc(reinterpret_cast<void**>(&d.first_zero_dev), 8) == cudaSuccess &&
            cudaMalloc(reinterpret_cast<void**>(&d.splitk_ws), kSplitKBytes) == cudaSuccess &&
            cudaMalloc(reinterpret_cast<void**>(&d.splitk_counters), kSplitKSlots * 4) == cudaSuccess &&
            cudaMemset(d.splitk_counters, 0, kSplitKSlots * 4) == cudaSuccess &&
            cudaEventCreateWithFlags(&d.ev_start, cudaEventDisableTiming) == cudaSuccess &&
            cudaEventCreateWithFlags(&d.ev_up, cudaEventDisableTiming) == cudaSuccess &&
            cudaEventCreateWithFlags(&d.ev_done, cudaEventDisableTiming) == cudaSuccess;
  for (int i = 0; ok && i < 2; ++i) {
    ok = cudaHostAlloc(&d.stage[i], kStageBytes, cudaHostAllocDefault) == cudaSuccess &&
         cudaEventCreateWithFlags(&d.stage_ev[i], cudaEventDisableTiming) == cudaSuccess;
  }
  if (!ok) {
    cudaGetLastError();
    set_error(err, "Could not create CUDA streams / staging memory on device %d.", ordinal);
    return -2;
  }
  std::memset(d.status_host, 0, sizeof(GemmStatus));
  d.ready = true;
  return 0;
}

Buffer* as_buffer(GPUPtr p) {
  Buffer* b = static_cast<Buffer*>(p);
  if (!b || g_buffers.find(b) == g_buffers.end() || b->magic != kMagic) return nullptr;
  return b;
}

bool host_is_pinned(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return a.type == cudaMemoryTypeHost;
}

// Host -> device on the compute stream.  Page-locked sources go in one async
// copy; pageable sources are pipelined through two pinned staging chunks.
bool copy_h2d(Device& d, void* dst, const void* src, size_t bytes) {
  if (bytes == 0) return true;
  if (fault_hit(FAULT_H2D)) return false;
  g_stats[1] += long(bytes);
  if (host_is_pinned(src)) {
    return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, d.stream) == cudaSuccess;
  }
  size_t off = 0;
  int slot = 0;
  while (off < bytes) {
    const size_t n = bytes - off < kStageBytes ? bytes - off : kStageBytes;
    if (cudaEventSynchronize(d.stage_ev[slot]) != cudaSuccess) return false;
    std::memcpy(d.stage[slot], static_cast<const char*>(src) + off, n);
    if (cudaMemcpyAsync(static_cast<char*>(dst) + off, d.stage[slot], n, cudaMemcpyHostToDevice,
                        d.stream) != cudaSuccess)
      return false;
    if (cudaEventRecord(d.stage_ev[slot], d.stream) != cudaSuccess) return false;
    off += n;
    slot ^= 1;
  }
  return true;
}

// Device -> host, complete on return.
bool copy_d2h(Device& d, void* dst, const void* src, size_t bytes) {
  if (bytes == 0) return true;
  if (fault_hit(FAULT_D2H)) return false;
  g_stats[2] += long(bytes);
  if (host_is_pinned(dst)) {
    return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, d.stream) == cudaSuccess &&
           wait_stream(d.stream) == cudaSuccess;
  }
  // chunk i is copied out of staging while chunk i+1 crosses the bus
  size_t off = 0, pending_off = 0, pending_n = 0;
  int slot = 0, pending_slot = -1;
  while (off < bytes || pending_slot >= 0) {
    int issued_slot = -1;
    size_t n = 0;
    if (off < bytes) {
      n = bytes - off < kStageBytes ? bytes - off : kStageBytes;
      if (cudaMemcpyAsync(d.stage[slot], static_cast<const char*>(src) + off, n,
                          cudaMemcpyDeviceToHost, d.stream) != cudaSuccess)
        return false;
      if (cudaEventRecord(d.stage_ev[slot], d.stream) != cudaSuccess) return false;
      issued_slot = slot;
    }
    if (pending_slot >= 0) {
      if (cudaEventSynchronize(d.stage_ev[pending_slot]) != cudaSuccess) return false;
      std::memcpy(static_cast<char*>(dst) + pending_off, d.stage[pending_slot], pending_n);
    }
    pending_slot = issued_slot;
    pending_off = off;
    pending_n = n;
    off += n;
    slot ^= 1;
  }
  return true;
}

// Makes the device copy current (lazy upload of registered host memory).
bool make_resident(Device& d, Buffer* b) {
  if (!b->host_pending) return true;
  if (!copy_h2d(d, b->dptr, b->host, b->bytes)) return false;
  b->host_pending = false;
  ++b->version;
  return true;
}

void wrote(Buffer* b) {
  b->host_pending = false;
  b->host_current = false;
  ++b->version;
}

void free_plane(Plane& p) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (p.p0) {
    pool_free(dev, p.p0, p.bytes);
    g_stats[0] -= long(p.bytes);
    g_stats[6] -= long(p.bytes);
  }
  if (p.p1) {
    pool_free(dev, p.p1, p.bytes);
    g_stats[0] -= long(p.bytes);
    g_stats[6] -= long(p.bytes);
  }
  p = Plane{};
}

inline uint64_t round_up(uint64_t v, uint64_t m) { return (v + m - 1) / m * m; }

// Returns the operand plane(s) of `b` viewed as [rows, cols], converting when
// the cached copy is stale.  kind: 0 fp16 RN, 1 fp16 trunc, 2 tf32 hi/lo, 3 tf32 hi + the
// two bf16 planes of the CTA-pair kernel (same bytes as kind 2).
Plane* get_plane(Device& d, Buffer* b, uint64_t rows, uint64_t cols, int kind) {
  Plane& p = (kind == 3) ? b->tf32x : (kind == 2) ? b->tf32 : b->f16[kind];
  if (p.p0 && p.version == b->version && p.rows == rows && p.cols == cols) return &p;
  const uint64_t pitch = round_up(cols, 64);
  const size_t esz = (kind >= 2) ? 4 : 2;
  const size_t bytes = size_t(rows) * pitch * esz;
  if (!p.p0 || p.bytes < bytes) {
    free_plane(p);
    if (pool_alloc(d.ordinal, &p.p0, bytes) != cudaSuccess) {
      cudaGetLastError();
      p = Plane{};
      return nullptr;
    }
    g_stats[0] += long(bytes);
    g_stats[6] += long(bytes);
    if (kind >= 2) {
      if (pool_alloc(d.ordinal, &p.p1, bytes) != cudaSuccess) {
        cudaGetLastError();
        pool_free(d.ordinal, p.p0, bytes);
        g_stats[0] -= long(bytes);
        g_stats[6] -= long(bytes);
        p = Plane{};
        return nullptr;
      }
      g_stats[0] += long(bytes);
      g_stats[6] += long(bytes);
    }
    p.bytes = bytes;
  }
  p.rows = rows;
  p.cols = cols;
  p.pitch = pitch;
  if (kind == 3) {
    gonn::launch_split_tf32_bf16(b->dptr, rows, cols, static_cast<float*>(p.p0), p.p1, pitch, d.stream);
  } else if (kind == 2) {
    gonn::launch_split_tf32(b->dptr, rows, cols, static_cast<float*>(p.p0),
                            static_cast<float*>(p.p1), pitch, d.stream);
  } else {
    gonn::launch_cvt_f16(b->dptr, rows, cols, p.p0, pitch, kind, d.stream);
  }
  ++g_stats[3];
  p.version = b->version;
  return &p;
}

// Ends an entry point: waits when blocking, then turns CUDA errors and kernel
// status words into the reference-style error.  `exec_code` is the value the
// entry point returns for an execution failure.
int finish(Device& d, CError* err, int exec_code, const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && g_blocking) e = wait_stream(d.stream);
  if (e != cudaSuccess) {
    set_error(err, "%s: CUDA error: %s", what, cudaGetErrorString(e));
    return exec_code;
  }
  if (g_blocking && d.status_host->code != 0) {
    d.last_status = *d.status_host;
    std::memset(d.status_host, 0, sizeof(GemmStatus));
    // a kernel that gave up may have left split-K arrival counters half counted
    cudaMemsetAsync(d.splitk_counters, 0, kSplitKSlots * 4, d.stream);
    set_error(err,
              "%s: GEMM kernel gave up waiting (role %u, where 0x%x, tile %u, k block %u).", what,
              d.last_status.code, d.last_status.where, d.last_status.tile, d.last_status.kblock);
    return exec_code;
  }
  return 0;
}

struct MatmulArgs {
  GPUPtr a, b, c, bias;
  long aRows, aCols, bRows, bCols, cRows, cCols;
  bool transA, transB;
  int precision;
  float alpha, beta;
  int act;
  float act_param;
};

// Streamed MatMul for a product whose A still lies in page-locked host memory
// and whose C is registered over page-locked host memory: A is uploaded in row
// blocks on one stream, each block is converted and multiplied on the compute
// stream, and its rows of C go back to the host on a third stream, so that the
// two PCIe directions and the tensor cores overlap.  The host copy of C is then
// current, as it is with the reference's aliased buffers, and a later
// retrieve_gpu_buffer_data into the same memory has nothing left to do.
// Returns 1 when the product was done here, 0 when the caller should take the
// ordinary path, -1 on a CUDA error.
// Rows per block: small enough that the first upload and the last write-back, which
// nothing overlaps, are short; large enough that a block's product fills the GPU.
// GONNGPU_STREAM_ROWS (a multiple of 512, >= 1024) overrides it.
long stream_rows() {
  static const long rows = [] {
    const char* e = std::getenv("GONNGPU_STREAM_ROWS");
    const long v = e ? std::atol(e) : 0;
    return (v >= 1024 && v % 512 == 0) ? v : 4096l;
  }();
  return rows;
}
// One device's share of a streamed product: `rows` rows of A in page-locked host memory, the
// fp32 and fp16 device copies they pass through, the B plane on that device, and where the
// rows of C go (device and page-locked host).
struct StreamedShard {
  const float* host_a = nullptr;
  float* host_c = nullptr;
  float* dev_a = nullptr;
  float* dev_c = nullptr;
  void* plane_a = nullptr;
  uint64_t pitch = 0;
  long rows = 0, N = 0, K = 0;
  gonn::GemmOperand b;
  int pkind = 0;
  float alpha = 1.f;
  const float* bias = nullptr;
  int act = gonn::ACT_NONE;
  float act_param = 0.f;
  // the uploads of A wait for what is already queued on the compute stream (false: only the
  // products do, so the rows travel while B is still on its way)
  bool uploads_wait = true;
};

// Enqueues the shard's blocks on the device's three streams (the device must be current)
// without waiting for anything.  Returns false on a CUDA or launch error (*msg set for the latter).
bool streamed_issue(Device& d, const StreamedShard& s, const char** msg) {
  const long block = stream_rows();
  // the side streams start after everything already queued on the compute stream (B, bias)
  bool ok = cudaEventRecord(d.ev_start, d.stream) == cudaSuccess &&
            (!s.uploads_wait || cudaStreamWaitEvent(d.copy_stream, d.ev_start, 0) == cudaSuccess) &&
            cudaStreamWaitEvent(d.d2h_stream, d.ev_start, 0) == cudaSuccess;
  for (long r0 = 0; r0 < s.rows && ok; r0 += block) {
    const long rows = std::min(block, s.rows - r0);
    float* a_dev = s.dev_a + size_t(r0) * s.K;
    float* c_dev = s.dev_c + size_t(r0) * s.N;
    ok = cudaMemcpyAsync(a_dev, s.host_a + size_t(r0) * s.K, size_t(rows) * s.K * 4,
                         cudaMemcpyHostToDevice, d.copy_stream) == cudaSuccess &&
         cudaEventRecord(d.ev_up, d.copy_stream) == cudaSuccess &&
         cudaStreamWaitEvent(d.stream, d.ev_up, 0) == cudaSuccess;
    if (!ok) break;
    g_stats[1] += long(rows) * s.K * 4;
    char* plane_rows = static_cast<char*>(s.plane_a) + size_t(r0) * s.pitch * 2;
    gonn::launch_cvt_f16(a_dev, uint64_t(rows), uint64_t(s.K), plane_rows, s.pitch, s.pkind, d.stream);
    gonn::GemmOperand oa;
    oa.plane0 = plane_rows;
    oa.pitch = s.pitch;
    oa.mn_major = false;
    gonn::GemmEpilogue epi;
    epi.alpha = s.alpha;
    epi.bias = s.bias;
    epi.act = s.act;
    epi.act_param = s.act_param;
    *msg = gonn::launch_gemm(gonn::Kind::F16, uint32_t(rows), uint32_t(s.N), uint32_t(s.K), oa, s.b, c_dev,
                             uint64_t(s.N), epi, d.status_dev, d.sm_count, g_tune, d.stream);
    if (*msg) return false;
    g_stats[3] += 2;
    ++g_stats[4];
    ok = cudaEventRecord(d.ev_done, d.stream) == cudaSuccess &&
         cudaStreamWaitEvent(d.d2h_stream, d.ev_done, 0) == cudaSuccess &&
         cudaMemcpyAsync(s.host_c + size_t(r0) * s.N, c_dev, size_t(rows) * s.N * 4, cudaMemcpyDeviceToHost,
                         d.d2h_stream) == cudaSuccess;
    g_stats[2] += long(rows) * s.N * 4;
  }
  return ok;
}

// Everything a streamed_issue enqueued is complete on return.
bool streamed_wait(Device& d) {
  const bool a = wait_stream(d.copy_stream) == cudaSuccess;
  const bool b = wait_stream(d.stream) == cudaSuccess;
  const bool c = wait_stream(d.d2h_stream) == cudaSuccess;
  return a && b && c;
}

int matmul_streamed(Device& d, Buffer* A, Buffer* B, Buffer* C, Buffer* bias, long M, long N, long K,
                    bool transB, int pkind, float alpha, int act, float act_param, const char** msg) {
  const long kStreamRows = stream_rows();
  if (pkind == 2 || !g_blocking || !A->host_pending || !C->host || M < 2 * kStreamRows) return 0;
  if (!host_is_pinned(A->host) || !host_is_pinned(C->host)) return 0;
  if (!make_resident(d, B) || (bias && !make_resident(d, bias))) return -1;
  Plane* pb = get_plane(d, B, uint64_t(transB ? N : K), uint64_t(transB ? K : N), pkind);
  // the A plane is filled block by block below; take it without converting
  Plane& pa = A->f16[pkind];
  const uint64_t pitch = round_up(uint64_t(K), 64);
  const size_t pa_bytes = size_t(M) * pitch * 2;
  if (!pb) return -1;
  if (!pa.p0 || pa.bytes < pa_bytes) {
    free_plane(pa);
    if (pool_alloc(d.ordinal, &pa.p0, pa_bytes) != cudaSuccess) {
      cudaGetLastError();
      pa = Plane{};
      return -1;
    }
    pa.bytes = pa_bytes;
    g_stats[0] += long(pa_bytes);
    g_stats[6] += long(pa_bytes);
  }
  StreamedShard s;
  s.host_a = A->host;
  s.host_c = C->host;
  s.dev_a = A->dptr;
  s.dev_c = C->dptr;
  s.plane_a = pa.p0;
  s.pitch = pitch;
  s.rows = M;
  s.N = N;
  s.K = K;
  s.b.plane0 = pb->p0;
  s.b.pitch = pb->pitch;
  s.b.mn_major = !transB;
  s.pkind = pkind;
  s.alpha = alpha;
  s.bias = bias ? bias->dptr : nullptr;
  s.act = act;
  s.act_param = act_param;
  const bool ok = streamed_issue(d, s, msg);
  // everything is complete on return (the ABI is blocking)
  const bool synced = streamed_wait(d);
  if (!ok || !synced) return -1;
  A->host_pending = false;
  ++A->version;
  pa.version = A->version;  // the plane matches the uploaded rows
  pa.rows = uint64_t(M);
  pa.cols = uint64_t(K);
  pa.pitch = pitch;
  wrote(C);
  C->host_current = true;
  return 1;
}

// Shared body of every GEMM entry point.  `codes` maps the failing step to the
// caller's return value: {device, buffer, dims, setup, scratch, exec}.
int matmul_core(const MatmulArgs& m, const int codes[6], const char* what, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* A = as_buffer(m.a);
  Buffer* B = as_buffer(m.b);
  Buffer* C = as_buffer(m.c);
  Buffer* bias = m.bias ? as_buffer(m.bias) : nullptr;
  if (!A || !B || !C || (m.bias && !bias)) {
    set_error(err, "Invalid input or output buffer pointers.");
    return codes[1];
  }
  if (int rc = ensure_device(C->device, err)) return rc == -1 ? codes[0] : codes[0];
  Device& d = g_dev[C->device];
  if (A->device != C->device || B->device != C->device || (bias && bias->device != C->device)) {
    set_error(err, "%s: buffers live on different devices.", what);
    return codes[1];
  }
  if (m.aRows <= 0 || m.aCols <= 0 || m.bRows <= 0 || m.bCols <= 0 || m.cRows <= 0 ||
      m.cCols <= 0) {
    set_error(err, "%s: matrix dimensions must be positive.", what);
    return codes[2];
  }
  const long M = m.transA ? m.aCols : m.aRows, K = m.transA ? m.aRows : m.aCols;
  const long Kb = m.transB ? m.bCols : m.bRows, N = m.transB ? m.bRows : m.bCols;
  if (K != Kb || m.cRows != M || m.cCols != N) {
    set_error(err, "%s: incompatible dimensions: op(A) %ldx%ld, op(B) %ldx%ld, C %ldx%ld.", what, M,
              K, Kb, N, m.cRows, m.cCols);
    return codes[2];
  }
  if (M >= (1l << 31) || N >= (1l << 31) || K >= (1l << 31)) {
    set_error(err, "%s: dimensions beyond 2^31-1 are not supported.", what);
    return codes[2];
  }
  if (size_t(m.aRows) * m.aCols * 4 > A->bytes || size_t(m.bRows) * m.bCols * 4 > B->bytes ||
      size_t(M) * N * 4 > C->bytes || (bias && size_t(N) * 4 > bias->bytes)) {
    set_error(err, "%s: a buffer is smaller than its stated matrix.", what);
    return codes[2];
  }
  if (C == A || C == B || C->dptr == A->dptr || C->dptr == B->dptr) {
    set_error(err, "%s: the result buffer must not alias an input.", what);
    return codes[2];
  }
  if (m.precision < 0 || m.precision > 2) {
    set_error(err, "%s: unknown precision %d.", what, m.precision);
    return codes[2];
  }
  if (!m.transA && m.beta == 0.f && m.precision != GONNGPU_FP32_3XTF32) {
    const char* smsg = nullptr;
    const int sr = matmul_streamed(d, A, B, C, bias, M, N, K, m.transB,
                                   m.precision == GONNGPU_FP16_RN ? 0 : 1, m.alpha, m.act, m.act_param,
                                   &smsg);
    if (sr == 1) return finish(d, err, codes[5], what);
    if (sr < 0) {
      cudaGetLastError();
      set_error(err, "%s: %s", what, smsg ? smsg : "streamed transfer failed.");
      return smsg ? codes[3] : codes[5];
    }
  }
  if (!make_resident(d, A) || !make_resident(d, B) || (bias && !make_resident(d, bias)) ||
      (m.beta != 0.f && !make_resident(d, C))) {
    cudaGetLastError();
    set_error(err, "%s: host to device copy failed.", what);
    return codes[5];
  }
  const int pkind = (m.precision == GONNGPU_FP32_3XTF32) ? 2 : (m.precision == GONNGPU_FP16_RN ? 0 : 1);
  // large fp32 products run on the CTA-pair kernel, which takes its correction terms from bf16 planes
  const bool bf16x = pkind == 2 && gonn::tf32_takes_pair_kernel(uint32_t(M), uint32_t(N), uint32_t(K),
                                                                d.sm_count, tune_for(d));
  Plane* pa = get_plane(d, A, uint64_t(m.aRows), uint64_t(m.aCols), bf16x ? 3 : pkind);
  Plane* pb = get_plane(d, B, uint64_t(m.bRows), uint64_t(m.bCols), bf16x ? 3 : pkind);
  if (!pa || !pb) {
    set_error(err, "%s: could not allocate operand planes.", what);
    return codes[4];
  }
  gonn::GemmOperand oa, ob;
  oa.plane0 = pa->p0;
  oa.plane1 = pa->p1;
  oa.pitch = pa->pitch;
  oa.mn_major = m.transA;  // stored [K, M]: M contiguous
  oa.plane1_bf16 = bf16x;
  ob.plane0 = pb->p0;
  ob.plane1 = pb->p1;
  ob.pitch = pb->pitch;
  ob.mn_major = !m.transB;  // stored [K, N]: N contiguous
  ob.plane1_bf16 = bf16x;
  gonn::GemmEpilogue epi;
  epi.alpha = m.alpha;
  epi.beta = m.beta;
  epi.c_in = C->dptr;
  epi.bias = bias ? bias->dptr : nullptr;
  epi.act = m.act;
  epi.act_param = m.act_param;
  const char* msg = gonn::launch_gemm(pkind == 2 ? gonn::Kind::TF32x3 : gonn::Kind::F16, uint32_t(M),
                                      uint32_t(N), uint32_t(K), oa, ob, C->dptr, uint64_t(N), epi,
                                      d.status_dev, d.sm_count, tune_for(d), d.stream);
  if (msg) {
    cudaGetLastError();
    set_error(err, "%s: %s", what, msg);
    return codes[3];
  }
  ++g_stats[3];
  ++g_stats[4];
  wrote(C);
  const int rc = finish(d, err, codes[5], what);
  if (!g_plane_cache) {
    if (g_blocking || cudaStreamSynchronize(d.stream) == cudaSuccess) {
      free_plane(A->f16[0]); free_plane(A->f16[1]); free_plane(A->tf32); free_plane(A->tf32x);
      free_plane(B->f16[0]); free_plane(B->f16[1]); free_plane(B->tf32); free_plane(B->tf32x);
    }
  }
  return rc;
}

int new_buffer(int device, float* host, size_t bytes, void* wrap, Buffer** out, CError* err) {
  if (int rc = ensure_device(device, err)) return rc;
  Buffer* b = new Buffer();
  b->device = device;
  b->bytes = bytes;
  b->host = host;
  b->host_pending = (host != nullptr);
  if (wrap) {
    b->dptr = static_cast<float*>(wrap);
    b->owns = false;
  } else {
    if (pool_alloc(device, reinterpret_cast<void**>(&b->dptr), bytes ? bytes : 4) != cudaSuccess) {
      cudaGetLastError();
      delete b;
      set_error(err, "Could not allocate %zu bytes of device memory.", bytes);
      return -3;
    }
    g_stats[0] += long(bytes);
  }
  g_buffers.insert(b);
  ++g_stats[5];
  *out = b;
  return 0;
}

}  // namespace

// =========================================================================
// Part 1: the reference bridge's symbols
// =========================================================================
extern "C" {

int create_gpu_buffer(float* data, long length_bytes, GPUPtr* outGPUPtr, DevicePtr* outDevicePtr,
                      CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (!outGPUPtr || length_bytes < 0 || (length_bytes > 0 && !data)) {
    set_error(err, "Could not create buffer: invalid arguments.");
    return -3;
  }
  Buffer* b = nullptr;
  if (int rc = new_buffer(g_current, data, size_t(length_bytes), nullptr, &b, err)) return rc;
  *outGPUPtr = b;
  if (outDevicePtr) *outDevicePtr = &g_dev[g_current];
  return 0;
}

int retrieve_gpu_buffer_data(GPUPtr gpuPtr, float* data, long length_bytes, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* b = as_buffer(gpuPtr);
  if (!b) {
    set_error(err, "Invalid GPU buffer pointer.");
    return -1;
  }
  if (length_bytes < 0 || size_t(length_bytes) > b->bytes) {
    set_error(err, "Buffer length mismatch during retrieval.");
    return -2;
  }
  if (length_bytes == 0) return 0;
  if (!data) {
    set_error(err, "Retrieval into a NULL pointer.");
    return -3;
  }
  if (b->host_pending) {
    // Never uploaded, never written: the registered host bytes are the contents.
    if (data != b->host) std::memmove(data, b->host, size_t(length_bytes));
    return 0;
  }
  if (b->host_current && data == b->host) return 0;  // the streamed MatMul already wrote it back
  if (ensure_device(b->device, err)) return -3;
  Device& d = g_dev[b->device];
  if (!copy_d2h(d, data, b->dptr, size_t(length_bytes))) {
    cudaError_t e = cudaGetLastError();
    set_error(err, "Device to host copy failed: %s", cudaGetErrorString(e));
    return -3;
  }
  return 0;
}

int release_gpu_buffer(GPUPtr gpuPtr) {
  if (!gpuPtr) return 0;
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* b = as_buffer(gpuPtr);
  if (!b) return -1;
  // Memory the caller owns (registered host memory that an upload may still read, wrapped device
  // memory) must be out of use when this returns.  The library's own device memory goes back to
  // the cache without a wait: every kernel runs on the device's one compute stream, so whoever
  // gets the block next is ordered behind its last user, and cudaFree waits by itself.
  const bool callers_memory = !b->owns || b->host != nullptr;
  if (cudaSetDevice(b->device) == cudaSuccess && g_dev[b->device].ready && callers_memory) {
    cudaStreamSynchronize(g_dev[b->device].stream);
  }
  free_plane(b->f16[0]);
  free_plane(b->f16[1]);
  free_plane(b->tf32);
  free_plane(b->tf32x);
  if (b->owns && b->dptr) {
    pool_free(b->device, b->dptr, b->bytes ? b->bytes : 4);
    g_stats[0] -= long(b->bytes);
  }
  cudaGetLastError();
  g_buffers.erase(b);
  --g_stats[5];
  b->magic = 0;
  delete b;
  return 0;
}

void free_c_error_message(char* message) {
  if (message) free(message);
}

int perform_mps_matrix_multiplication(GPUPtr aMatrixPtr, long aRows, long aCols, GPUPtr bMatrixPtr,
                                      long bRows, long bCols, GPUPtr resultMatrixPtr,
                                      long resultRows, long resultCols, DevicePtr /*device*/,
                                      CError* err) {
  MatmulArgs m{aMatrixPtr, bMatrixPtr, resultMatrixPtr, nullptr, aRows, aCols, bRows, bCols,
               resultRows, resultCols, false, false, GONNGPU_FP32_3XTF32, 1.f, 0.f,
               GONNGPU_ACT_NONE, 0.f};
  static const int codes[6] = {-1, -2, -3, -4, -5, -6};
  return matmul_core(m, codes, "matrix multiplication", err);
}

int perform_optimized_gemm(GPUPtr aPtr, GPUPtr bPtr, GPUPtr cPtr, long M, long N, long K,
                           float alpha, float beta, DevicePtr /*device*/, CError* err) {
  MatmulArgs m{aPtr, bPtr, cPtr, nullptr, M, K, K, N, M, N, false, false, GONNGPU_FP32_3XTF32,
               alpha, beta, GONNGPU_ACT_NONE, 0.f};
  static const int codes[6] = {-1, -2, -3, -3, -3, -6};
  return matmul_core(m, codes, "optimized GEMM", err);
}

int perform_fused_linear_activation(GPUPtr input, long batch_size, long input_size, GPUPtr weight,
                                    long output_size, GPUPtr bias, int activation_type, float alpha,
                                    GPUPtr output, DevicePtr /*device*/, CError* error) {
  // The reference decodes 0..4 and treats every other code as identity.
  const int act = (activation_type >= 0 && activation_type <= 4) ? activation_type : GONNGPU_ACT_NONE;
  MatmulArgs m{input, weight, output, bias, batch_size, input_size, input_size, output_size,
               batch_size, output_size, false, false, GONNGPU_FP32_3XTF32, 1.f, 0.f, act, alpha};
  static const int codes[6] = {-1, -1, -3, -4, -5, -6};
  return matmul_core(m, codes, "fused linear+activation", error);
}

int gonngpu_matmul_ex(GPUPtr a, long aRows, long aCols, int transA, GPUPtr b, long bRows,
                      long bCols, int transB, GPUPtr c, long cRows, long cCols, int precision,
                      float alpha, float beta, GPUPtr bias, int activation_type,
                      float activation_param, CError* err) {
  const int act = (activation_type >= 0 && activation_type <= 4) ? activation_type : GONNGPU_ACT_NONE;
  MatmulArgs m{a, b, c, bias, aRows, aCols, bRows, bCols, cRows, cCols, transA != 0, transB != 0,
               precision, alpha, beta, act, activation_param};
  static const int codes[6] = {-1, -2, -3, -4, -5, -6};
  return matmul_core(m, codes, "matmul_ex", err);
}

int perform_mps_matrix_transpose(GPUPtr inputMatrixPtr, long inputRows, long inputCols,
                                 GPUPtr outputMatrixPtr, long outputRows, long outputCols,
                                 DevicePtr /*device*/, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (inputRows != outputCols || inputCols != outputRows || inputRows < 0 || inputCols < 0) {
    set_error(err, "Invalid transpose dimensions.");
    return -2;
  }
  Buffer* in = as_buffer(inputMatrixPtr);
  Buffer* out = as_buffer(outputMatrixPtr);
  if (!in || !out) {
    set_error(err, "Invalid input or output buffer pointers.");
    return -3;
  }
  const size_t need = size_t(inputRows) * size_t(inputCols) * 4;
  if (need > in->bytes || need > out->bytes || in->device != out->device || in == out ||
      inputRows >= (1l << 31) || inputCols >= (1l << 31)) {
    set_error(err, "Invalid transpose dimensions.");
    return -2;
  }
  if (ensure_device(out->device, err)) return -1;
  Device& d = g_dev[out->device];
  if (!make_resident(d, in)) {
    cudaGetLastError();
    set_error(err, "transpose: host to device copy failed.");
    return -6;
  }
  gonn::launch_transpose(in->dptr, uint64_t(inputRows), uint64_t(inputCols), out->dptr, d.sm_count,
                         d.stream);
  ++g_stats[3];
  wrote(out);
  return finish(d, err, -6, "transpose");
}

int perform_mps_matrix_add_broadcast(GPUPtr aMatrixPtr, long aRows, long aCols, GPUPtr bMatrixPtr,
                                     long bRows, long bCols, GPUPtr resultMatrixPtr,
                                     long resultRows, long resultCols, DevicePtr /*device*/,
                                     CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* A = as_buffer(aMatrixPtr);
  Buffer* B = as_buffer(bMatrixPtr);
  Buffer* C = as_buffer(resultMatrixPtr);
  if (!A || !B || !C) {
    set_error(err, "Invalid input or output buffer pointers.");
    return -3;
  }
  int mode = -1;
  if (aRows == resultRows && aCols == resultCols && bRows == 1 && bCols == resultCols) mode = 0;
  else if (bRows == resultRows && bCols == resultCols && aRows == 1 && aCols == resultCols) mode = 1;
  else if (aRows == resultRows && aCols == resultCols && bRows == resultRows && bCols == 1) mode = 2;
  else if (bRows == resultRows && bCols == resultCols && aRows == resultRows && aCols == 1) mode = 3;
  if (mode < 0 || resultRows < 0 || resultCols < 0 ||
      size_t(aRows) * aCols * 4 > A->bytes || size_t(bRows) * bCols * 4 > B->bytes ||
      size_t(resultRows) * resultCols * 4 > C->bytes || A->device != C->device ||
      B->device != C->device) {
    set_error(err, "Unsupported broadcasting pattern: A (%ldx%ld) + B (%ldx%ld) -> Result (%ldx%ld)",
              aRows, aCols, bRows, bCols, resultRows, resultCols);
    return -2;
  }
  if (ensure_device(C->device, err)) return -1;
  Device& d = g_dev[C->device];
  if (!make_resident(d, A) || !make_resident(d, B)) {
    cudaGetLastError();
    set_error(err, "add broadcast: host to device copy failed.");
    return -6;
  }
  gonn::launch_add_broadcast(A->dptr, B->dptr, C->dptr, uint64_t(resultRows), uint64_t(resultCols),
                             mode, d.stream);
  ++g_stats[3];
  wrote(C);
  return finish(d, err, -6, "add broadcast");
}

int perform_activation_relu_forward(GPUPtr inputPtr, long size, GPUPtr outputPtr,
                                    DevicePtr /*device*/, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* in = as_buffer(inputPtr);
  Buffer* out = as_buffer(outputPtr);
  if (!in || !out || size < 0 || size_t(size) * 4 > in->bytes || size_t(size) * 4 > out->bytes ||
      in->device != out->device) {
    set_error(err, "Invalid buffer pointers for ReLU forward.");
    return -1;
  }
  if (ensure_device(out->device, err)) return -1;
  Device& d = g_dev[out->device];
  if (!make_resident(d, in)) {
    cudaGetLastError();
    set_error(err, "ReLU forward: host to device copy failed.");
    return -6;
  }
  gonn::launch_relu_forward(in->dptr, out->dptr, uint64_t(size), d.stream);
  ++g_stats[3];
  wrote(out);
  return finish(d, err, -6, "ReLU forward");
}

int perform_activation_relu_backward(GPUPtr gradOutputPtr, GPUPtr activationOutputPtr, long size,
                                     GPUPtr gradInputPtr, DevicePtr /*device*/, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* go = as_buffer(gradOutputPtr);
  Buffer* act = as_buffer(activationOutputPtr);
  Buffer* gi = as_buffer(gradInputPtr);
  if (!go || !act || !gi || size < 0 || size_t(size) * 4 > go->bytes ||
      size_t(size) * 4 > act->bytes || size_t(size) * 4 > gi->bytes || go->device != gi->device ||
      act->device != gi->device) {
    set_error(err, "Invalid buffer pointers for ReLU backward.");
    return -1;
  }
  if (ensure_device(gi->device, err)) return -1;
  Device& d = g_dev[gi->device];
  if (!make_resident(d, go) || !make_resident(d, act)) {
    cudaGetLastError();
    set_error(err, "ReLU backward: host to device copy failed.");
    return -6;
  }
  gonn::launch_relu_backward(go->dptr, act->dptr, gi->dptr, uint64_t(size), d.stream);
  ++g_stats[3];
  wrote(gi);
  return finish(d, err, -6, "ReLU backward");
}

void* allocateSharedMemory(long size) {
  if (size <= 0) return nullptr;
  return gonngpu_host_alloc(size);
}

void* createGPUBufferFromSharedMemory(void* /*device*/, void* memory, long size) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (!memory || size <= 0) return nullptr;
  Buffer* b = nullptr;
  if (new_buffer(g_current, static_cast<float*>(memory), size_t(size), nullptr, &b, nullptr))
    return nullptr;
  return b;
}

// =========================================================================
// Part 2: additive entry points
// =========================================================================

int gonngpu_gemm_f16_device(const void* a, long aRows, long aCols, long aPitch, int transA,
                            const void* b, long bRows, long bCols, long bPitch, int transB,
                            float* c, long ldc, float alpha, float beta, const float* bias,
                            int activation_type, float activation_param, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (!a || !b || !c) {
    set_error(err, "gemm_f16_device: NULL operand pointer.");
    return -2;
  }
  if (ensure_device(g_current, err)) return -1;
  Device& d = g_dev[g_current];
  const long M = transA ? aCols : aRows, K = transA ? aRows : aCols;
  const long Kb = transB ? bCols : bRows, N = transB ? bRows : bCols;
  if (aRows <= 0 || aCols <= 0 || bRows <= 0 || bCols <= 0 || K != Kb || aPitch < aCols ||
      bPitch < bCols || ldc < N || aPitch % 8 || bPitch % 8 || M >= (1l << 31) || N >= (1l << 31) ||
      K >= (1l << 31)) {
    set_error(err, "gemm_f16_device: incompatible dimensions or pitches (op(A) %ldx%ld, op(B) %ldx%ld).",
              M, K, Kb, N);
    return -3;
  }
  gonn::GemmOperand oa, ob;
  oa.plane0 = a;
  oa.pitch = uint64_t(aPitch);
  oa.mn_major = transA != 0;
  ob.plane0 = b;
  ob.pitch = uint64_t(bPitch);
  ob.mn_major = transB == 0;
  gonn::GemmEpilogue epi;
  epi.alpha = alpha;
  epi.beta = beta;
  epi.c_in = c;
  epi.bias = bias;
  epi.act = (activation_type >= 0 && activation_type <= 4) ? activation_type : GONNGPU_ACT_NONE;
  epi.act_param = activation_param;
  const char* msg = gonn::launch_gemm(gonn::Kind::F16, uint32_t(M), uint32_t(N), uint32_t(K), oa, ob, c,
                                      uint64_t(ldc), epi, d.status_dev, d.sm_count, g_tune, d.stream);
  if (msg) {
    cudaGetLastError();
    set_error(err, "gemm_f16_device: %s", msg);
    return (std::strstr(msg, "pitch") || std::strstr(msg, "aligned")) ? -3 : -4;
  }
  ++g_stats[3];
  ++g_stats[4];
  return finish(d, err, -6, "gemm_f16_device");
}

int gonngpu_convert_f16_device(const float* src, long rows, long cols, void* dst, long dstPitch,
                               int mode, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (!src || !dst || rows < 0 || cols < 0 || dstPitch < cols ||
      (mode != GONNGPU_FP16_RN && mode != GONNGPU_FP16_TRUNC)) {
    set_error(err, "convert_f16_device: invalid arguments.");
    return -3;
  }
  if (ensure_device(g_current, err)) return -1;
  Device& d = g_dev[g_current];
  gonn::launch_cvt_f16(src, uint64_t(rows), uint64_t(cols), dst, uint64_t(dstPitch),
                       mode == GONNGPU_FP16_RN ? gonn::F16_RN : gonn::F16_TRUNC, d.stream);
  ++g_stats[3];
  return finish(d, err, -6, "convert_f16_device");
}

// ---- replication of B for the row-sharded product ----------------------------------
int gonngpu_replicate_send(const void* src, void* dst_multicast, long bytes, void* const* bases_dev,
                           int world, int rank, long ctrl_offset, int slot, unsigned epoch,
                           unsigned ack_needed, int ctas, void* stream, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (!src || !dst_multicast || !bases_dev) {
    set_error(err, "replicate_send: NULL pointer.");
    return -2;
  }
  if (bytes <= 0 || bytes % 16 || (reinterpret_cast<uintptr_t>(src) & 15) ||
      (reinterpret_cast<uintptr_t>(dst_multicast) & 15) || world < 1 ||
      world > gonn::kReplicaMaxRanks || rank < 0 || rank >= world || ctrl_offset < 0 ||
      ctrl_offset % 16 || (slot != 0 && slot != 1) || ctas < 0 || ctas > 4096) {
    set_error(err, "replicate_send: sizes and addresses must be multiples of 16 bytes, 1..%d ranks, "
                   "slot 0 or 1.", gonn::kReplicaMaxRanks);
    return -3;
  }
  if (ensure_device(g_current, err)) return -1;
  Device& d = g_dev[g_current];
  cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : d.stream;
  cudaError_t e = gonn::launch_replicate_send(src, dst_multicast, uint64_t(bytes), bases_dev, world, rank,
                                              uint64_t(ctrl_offset), slot, epoch, ack_needed,
                                              d.status_dev, ctas ? ctas : d.sm_count, s);
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error(err, "replicate_send: launch failed: %s", cudaGetErrorString(e));
    return -4;
  }
  ++g_stats[3];
  if (stream && g_blocking && cudaStreamSynchronize(s) != cudaSuccess) {
    set_error(err, "replicate_send: CUDA error: %s", cudaGetErrorString(cudaGetLastError()));
    return -6;
  }
  return finish(d, err, -6, "replicate_send");
}

int gonngpu_replicate_wait(void* const* bases_dev, int world, int owner, int rank, long ctrl_offset,
                           int slot, unsigned epoch, unsigned ack_value, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (!bases_dev) {
    set_error(err, "replicate_wait: NULL pointer.");
    return -2;
  }
  if (world < 1 || world > gonn::kReplicaMaxRanks || rank < 0 || rank >= world || owner < 0 ||
      owner >= world || ctrl_offset < 0 || ctrl_offset % 16 || (slot != 0 && slot != 1)) {
    set_error(err, "replicate_wait: 1..%d ranks, owner and rank inside the group, slot 0 or 1.",
              gonn::kReplicaMaxRanks);
    return -3;
  }
  if (ensure_device(g_current, err)) return -1;
  Device& d = g_dev[g_current];
  cudaError_t e = gonn::launch_replicate_wait(bases_dev, owner, rank, uint64_t(ctrl_offset), slot, epoch,
                                              ack_value, d.status_dev, d.stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error(err, "replicate_wait: launch failed: %s", cudaGetErrorString(e));
    return -4;
  }
  ++g_stats[3];
  return finish(d, err, -6, "replicate_wait");
}

int gonngpu_gemm_f16_sharded(const void* a, long aRows, long aCols, long aPitch, const void* b_src,
                             long bCols, void* local_base, void* const* bases_dev,
                             void* multicast_base, int world, int owner, int rank,
                             long slots_offset, long ctrl_offset, unsigned epoch, float* c, long ldc,
                             int first_group, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (!a || !c || !local_base || !bases_dev || (rank == owner && !b_src)) {
    set_error(err, "gemm_f16_sharded: NULL pointer (the owner of B passes its source).");
    return -2;
  }
  if (aRows <= 0 || aCols <= 0 || bCols <= 0 || aPitch < aCols || aPitch % 8 || bCols % 8 ||
      ldc < bCols || aRows >= (1l << 31) || aCols >= (1l << 31) || bCols >= (1l << 31) ||
      world < 1 || world > gonn::kShardMaxRanks || rank < 0 || rank >= world || owner < 0 ||
      owner >= world || slots_offset < 0 || slots_offset % 16 || ctrl_offset < 0 || ctrl_offset % 16 ||
      epoch == 0 || first_group < 0) {
    set_error(err, "gemm_f16_sharded: bad dimensions (B needs a multiple of 8 columns), pitches, "
                   "offsets (multiples of 16 bytes), group (1..%d ranks) or epoch (starts at 1).",
              gonn::kShardMaxRanks);
    return -3;
  }
  const uint64_t slot_bytes = uint64_t(aCols) * uint64_t(bCols) * 2;
  const uint64_t lo = uint64_t(slots_offset), hi = lo + 2 * slot_bytes;
  if (uint64_t(ctrl_offset) + sizeof(gonn::ShardControl) > lo && uint64_t(ctrl_offset) < hi) {
    set_error(err, "gemm_f16_sharded: the control words lie inside the slots.");
    return -3;
  }
  if (ensure_device(g_current, err)) return -1;
  Device& d = g_dev[g_current];
  gonn::ShardLink link;
  link.slot = int(epoch & 1u);
  link.slot_offset = lo + uint64_t(link.slot) * slot_bytes;
  link.b_src = b_src;
  link.slot_multicast = multicast_base ? static_cast<char*>(multicast_base) + link.slot_offset : nullptr;
  link.bases = bases_dev;
  link.ctrl_offset = uint64_t(ctrl_offset);
  link.world = world;
  link.owner = owner;
  link.rank = rank;
  link.epoch = epoch;
  link.first_group = uint32_t(first_group);
  link.sender_pairs = g_shard_sender_pairs;
  link.late_rounds = g_shard_late_rounds;
  link.trace = g_shard_trace;
  const char* msg = gonn::launch_gemm_sharded(uint32_t(aRows), uint32_t(bCols), uint32_t(aCols), a,
                                              uint64_t(aPitch), static_cast<char*>(local_base) + link.slot_offset,
                                              c, uint64_t(ldc), link, d.status_dev, d.sm_count, d.stream);
  if (msg) {
    cudaGetLastError();
    set_error(err, "gemm_f16_sharded: %s", msg);
    return (std::strstr(msg, "pitch") || std::strstr(msg, "aligned") || std::strstr(msg, "bad ")) ? -3 : -4;
  }
  ++g_stats[3];
  ++g_stats[4];
  return finish(d, err, -6, "gemm_f16_sharded");
}

// ---- row-sharded MatMul over the GPUs of one process ----------------------------------
namespace {
// Rows [lo, hi) of device `i` of `n`: contiguous blocks of ceil(M / n) rows rounded up to the
// 256-row tile of the pair kernel; the last blocks may be short or empty.
void shard_rows(long M, int n, int i, long* lo, long* hi) {
  long per = (M + n - 1) / n;
  per = (per + 255) / 256 * 256;
  *lo = std::min(long(i) * per, M);
  *hi = std::min(*lo + per, M);
}

struct ShardScratch {
  int dev = -1;
  long lo = 0, hi = 0;
  void* dev_a = nullptr;
  void* dev_c = nullptr;
  void* plane_a = nullptr;
  void* plane_b = nullptr;
  size_t a_bytes = 0, c_bytes = 0, pa_bytes = 0, pb_bytes = 0;
};
}  // namespace

int gonngpu_shard_plan(long rows, int n_devices, int device, long* first_row, long* end_row) {
  if (rows < 0 || n_devices < 1 || device < 0 || device >= n_devices || !first_row || !end_row) return -3;
  shard_rows(rows, n_devices, device, first_row, end_row);
  return 0;
}

int gonngpu_matmul_sharded(const float* a, long aRows, long aCols, const float* b, long bRows,
                           long bCols, float* c, int precision, int n_devices, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (!a || !b || !c) {
    set_error(err, "matmul_sharded: NULL matrix pointer.");
    return -2;
  }
  if (aRows <= 0 || aCols <= 0 || bRows <= 0 || bCols <= 0 || aCols != bRows || aRows >= (1l << 31) ||
      aCols >= (1l << 31) || bCols >= (1l << 31)) {
    set_error(err, "matmul_sharded: incompatible dimensions: A %ldx%ld, B %ldx%ld.", aRows, aCols, bRows,
              bCols);
    return -3;
  }
  if (precision != GONNGPU_FP16_RN && precision != GONNGPU_FP16_TRUNC) {
    set_error(err, "matmul_sharded: precision must be GONNGPU_FP16_RN or GONNGPU_FP16_TRUNC.");
    return -3;
  }
  const int visible = gonngpu_device_count();
  if (n_devices == 0) n_devices = visible;
  if (n_devices < 1 || n_devices > visible || n_devices > kMaxDevices) {
    set_error(err, "matmul_sharded: %d devices asked for, %d visible.", n_devices, visible);
    return -1;
  }
  const long M = aRows, K = aCols, N = bCols;
  const int pkind = precision == GONNGPU_FP16_RN ? 0 : 1;
  // The rows travel by asynchronous copies: the host matrices must be page-locked.  Memory that
  // is not (a Go slice, a malloc) is locked for the duration of the call, which costs far more
  // than the product; callers that care allocate with gonngpu_host_alloc.
  void* locked[3] = {nullptr, nullptr, nullptr};
  const void* host[3] = {a, c, b};
  const size_t host_bytes[3] = {size_t(M) * K * 4, size_t(M) * N * 4, size_t(K) * N * 4};
  bool lock_ok = true;
  for (int i = 0; i < 3 && lock_ok; ++i) {
    if (host_is_pinned(host[i])) continue;
    if (cudaHostRegister(const_cast<void*>(host[i]), host_bytes[i], cudaHostRegisterPortable) == cudaSuccess) {
      locked[i] = const_cast<void*>(host[i]);
    } else {
      cudaGetLastError();
      lock_ok = false;
    }
  }
  std::vector<ShardScratch> sh;
  const uint64_t pitch = round_up(uint64_t(K), 64), pitch_b = round_up(uint64_t(N), 64);
  int rc = 0;
  const char* msg = nullptr;
  void* b32 = nullptr;
  auto fail = [&](int code, const char* what) {
    if (rc == 0) {
      rc = code;
      cudaError_t e = cudaGetLastError();
      set_error(err, "matmul_sharded: %s%s%s", what, e != cudaSuccess ? ": " : "",
                e != cudaSuccess ? cudaGetErrorString(e) : "");
    }
  };
  if (!lock_ok) fail(-5, "could not page-lock a host matrix");
  // ---- plan and scratch
  for (int i = 0; i < n_devices && rc == 0; ++i) {
    ShardScratch x;
    x.dev = i;
    shard_rows(M, n_devices, i, &x.lo, &x.hi);
    if (x.hi <= x.lo) continue;
    if (ensure_device(i, nullptr)) {
      fail(-1, "a device of the group is not a usable sm_100 GPU");
      break;
    }
    // the uploads below do not wait for the compute stream: blocks from the cache must be idle
    cudaStreamSynchronize(g_dev[i].stream);
    const size_t rows = size_t(x.hi - x.lo);
    x.a_bytes = rows * K * 4;
    x.c_bytes = rows * N * 4;
    x.pa_bytes = rows * pitch * 2;
    x.pb_bytes = size_t(K) * pitch_b * 2;
    if (pool_alloc(i, &x.dev_a, x.a_bytes) != cudaSuccess || pool_alloc(i, &x.dev_c, x.c_bytes) != cudaSuccess ||
        pool_alloc(i, &x.plane_a, x.pa_bytes) != cudaSuccess || pool_alloc(i, &x.plane_b, x.pb_bytes) != cudaSuccess)
      fail(-5, "could not allocate device memory for a shard");
    sh.push_back(x);
  }
  // ---- B: to the first device over PCIe, converted there, then to every other device over NVLink
  if (rc == 0 && !sh.empty()) {
    ShardScratch& s0 = sh[0];
    Device& d0 = g_dev[s0.dev];
    cudaSetDevice(s0.dev);
    if (pool_alloc(s0.dev, &b32, host_bytes[2]) != cudaSuccess) fail(-5, "could not allocate device memory for B");
    if (rc == 0) {
      if (cudaMemcpyAsync(b32, b, host_bytes[2], cudaMemcpyHostToDevice, d0.stream) != cudaSuccess)
        fail(-6, "host to device copy of B failed");
      g_stats[1] += long(host_bytes[2]);
      gonn::launch_cvt_f16(static_cast<const float*>(b32), uint64_t(K), uint64_t(N), s0.plane_b, pitch_b, pkind,
                           d0.stream);
      ++g_stats[3];
      if (cudaEventRecord(d0.ev_done, d0.stream) != cudaSuccess) fail(-6, "event record failed");
    }
    for (size_t i = 1; i < sh.size() && rc == 0; ++i) {
      Device& di = g_dev[sh[i].dev];
      cudaSetDevice(sh[i].dev);
      int can = 0;
      if (cudaDeviceCanAccessPeer(&can, sh[i].dev, s0.dev) == cudaSuccess && can) {
        if (cudaDeviceEnablePeerAccess(s0.dev, 0) != cudaSuccess) cudaGetLastError();  // already enabled is fine
      }
      if (cudaStreamWaitEvent(di.stream, d0.ev_done, 0) != cudaSuccess ||
          cudaMemcpyPeerAsync(sh[i].plane_b, sh[i].dev, s0.plane_b, s0.dev, s0.pb_bytes, di.stream) != cudaSuccess)
        fail(-6, "peer copy of B failed");
    }
  }
  // ---- every device's rows: upload, convert, multiply, write back, block by block
  for (size_t i = 0; i < sh.size() && rc == 0; ++i) {
    ShardScratch& x = sh[i];
    Device& d = g_dev[x.dev];
    cudaSetDevice(x.dev);
    StreamedShard s;
    s.host_a = a + size_t(x.lo) * K;
    s.host_c = c + size_t(x.lo) * N;
    s.dev_a = static_cast<float*>(x.dev_a);
    s.dev_c = static_cast<float*>(x.dev_c);
    s.plane_a = x.plane_a;
    s.pitch = pitch;
    s.rows = x.hi - x.lo;
    s.N = N;
    s.K = K;
    s.b.plane0 = x.plane_b;
    s.b.pitch = pitch_b;
    s.b.mn_major = true;
    s.pkind = pkind;
    s.uploads_wait = false;  // the scratch is this call's own; only the products need B
    if (!streamed_issue(d, s, &msg)) fail(msg ? -4 : -6, msg ? msg : "a copy or launch of a shard failed");
  }
  // ---- wait for every device, collect kernel status, hand the scratch back to the cache
  for (auto& x : sh) {
    Device& d = g_dev[x.dev];
    cudaSetDevice(x.dev);
    if (!streamed_wait(d)) fail(-6, "execution failed");
    if (d.status_host->code != 0) {
      d.last_status = *d.status_host;
      std::memset(d.status_host, 0, sizeof(GemmStatus));
      if (rc == 0) {
        rc = -6;
        set_error(err, "matmul_sharded: GEMM kernel on device %d gave up waiting (role %u, tile %u, k block %u).",
                  x.dev, d.last_status.code, d.last_status.tile, d.last_status.kblock);
      }
    }
    pool_free(x.dev, x.dev_a, x.a_bytes);
    pool_free(x.dev, x.dev_c, x.c_bytes);
    pool_free(x.dev, x.plane_a, x.pa_bytes);
    pool_free(x.dev, x.plane_b, x.pb_bytes);
  }
  if (b32 && !sh.empty()) {
    cudaSetDevice(sh[0].dev);
    pool_free(sh[0].dev, b32, host_bytes[2]);
  }
  for (void* p : locked)
    if (p) cudaHostUnregister(p);
  cudaSetDevice(g_current);
  cudaGetLastError();
  return rc;
}

// ---- element-wise family (internal/cgo/metal_bridge_matrix.m:172-543) -------------
namespace {
// Equal-shaped binary op.  Order of checks and codes as in the reference:
// dimensions (-2), device (-1), buffers (-3).
int ew_binary(int op, const char* noun, GPUPtr aPtr, long aRows, long aCols, GPUPtr bPtr, long bRows,
              long bCols, GPUPtr cPtr, long cRows, long cCols, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (aRows != bRows || aCols != bCols || aRows != cRows || aCols != cCols || aRows < 0 || aCols < 0) {
    set_error(err, "Matrices must have the same dimensions for element-wise %s.", noun);
    return -2;
  }
  Buffer* A = as_buffer(aPtr);
  Buffer* B = as_buffer(bPtr);
  Buffer* C = as_buffer(cPtr);
  const size_t n = size_t(aRows) * size_t(aCols);
  if (!A || !B || !C || n * 4 > A->bytes || n * 4 > B->bytes || n * 4 > C->bytes ||
      A->device != C->device || B->device != C->device) {
    set_error(err, "Invalid input or output buffer pointers.");
    return -3;
  }
  if (ensure_device(C->device, err)) return -1;
  Device& d = g_dev[C->device];
  if (!make_resident(d, A) || !make_resident(d, B)) {
    cudaGetLastError();
    set_error(err, "element-wise %s: host to device copy failed.", noun);
    return -6;
  }
  size_t count = n;
  long zero_at = -1;
  if (op == gonn::EW_DIV && n > 0) {
    // The reference stops at the first zero divisor: the elements before it are
    // written, the rest are not, and the call fails with -4.
    unsigned long long idx = ~0ull;
    bool ok = cudaMemsetAsync(d.first_zero_dev, 0xFF, 8, d.stream) == cudaSuccess;
    if (ok) gonn::launch_first_zero(B->dptr, n, d.first_zero_dev, d.stream);
    ok = ok && cudaMemcpyAsync(&idx, d.first_zero_dev, 8, cudaMemcpyDeviceToHost, d.stream) == cudaSuccess &&
         cudaStreamSynchronize(d.stream) == cudaSuccess;
    ++g_stats[3];
    if (!ok) {
      cudaGetLastError();
      set_error(err, "element-wise division: CUDA error.");
      return -6;
    }
    if (idx < n) {
      zero_at = long(idx);
      count = size_t(idx);
    }
  }
  if (count > 0) {
    if (C->host_pending && count < n && !make_resident(d, C)) {  // keep the untouched tail
      cudaGetLastError();
      set_error(err, "element-wise %s: host to device copy failed.", noun);
      return -6;
    }
    gonn::launch_elementwise(op, A->dptr, B->dptr, C->dptr, count, 0.f, d.stream);
    ++g_stats[3];
    wrote(C);
  }
  const int rc = finish(d, err, -6, "element-wise operation");
  if (rc == 0 && zero_at >= 0) {
    set_error(err, "Division by zero encountered at element %ld.", zero_at);
    return -4;
  }
  return rc;
}

// One-operand op with a scalar, or activation forward (b == nullptr), or
// activation backward (a = gradient, b = activation output).  Bad buffers: -1.
// `softmax_rows` >= 0 selects the row softmax over [softmax_rows, n / softmax_rows]
// instead of `op` (forward when b == nullptr, else backward).
int ew_unary(int op, const char* what, GPUPtr aPtr, GPUPtr bPtr, GPUPtr cPtr, long n, float scalar,
             CError* err, long softmax_rows = -1) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* A = as_buffer(aPtr);
  Buffer* B = bPtr ? as_buffer(bPtr) : nullptr;
  Buffer* C = as_buffer(cPtr);
  if (!A || !C || (bPtr && !B) || n < 0 || size_t(n) * 4 > A->bytes || size_t(n) * 4 > C->bytes ||
      (B && size_t(n) * 4 > B->bytes) || A->device != C->device || (B && B->device != C->device)) {
    set_error(err, "Invalid %s.", what);
    return -1;
  }
  if (ensure_device(C->device, err)) return -1;
  Device& d = g_dev[C->device];
  if (!make_resident(d, A) || (B && !make_resident(d, B))) {
    cudaGetLastError();
    set_error(err, "%s: host to device copy failed.", what);
    return -6;
  }
  if (softmax_rows > 0)
    gonn::launch_softmax(A->dptr, B ? B->dptr : nullptr, C->dptr, uint64_t(softmax_rows),
                         uint64_t(n / softmax_rows), B != nullptr, d.stream);
  else if (softmax_rows < 0)
    gonn::launch_elementwise(op, A->dptr, B ? B->dptr : nullptr, C->dptr, uint64_t(n), scalar, d.stream);
  ++g_stats[3];
  wrote(C);
  return finish(d, err, -6, what);
}
}  // namespace

int perform_mps_matrix_add(GPUPtr a, long aRows, long aCols, GPUPtr b, long bRows, long bCols, GPUPtr c,
                           long cRows, long cCols, DevicePtr, CError* err) {
  return ew_binary(gonn::EW_ADD, "addition", a, aRows, aCols, b, bRows, bCols, c, cRows, cCols, err);
}
int perform_mps_matrix_subtract(GPUPtr a, long aRows, long aCols, GPUPtr b, long bRows, long bCols,
                                GPUPtr c, long cRows, long cCols, DevicePtr, CError* err) {
  return ew_binary(gonn::EW_SUB, "subtraction", a, aRows, aCols, b, bRows, bCols, c, cRows, cCols, err);
}
int perform_mps_matrix_element_multiply(GPUPtr a, long aRows, long aCols, GPUPtr b, long bRows,
                                        long bCols, GPUPtr c, long cRows, long cCols, DevicePtr,
                                        CError* err) {
  return ew_binary(gonn::EW_MUL, "multiplication", a, aRows, aCols, b, bRows, bCols, c, cRows, cCols, err);
}
int perform_mps_matrix_element_divide(GPUPtr a, long aRows, long aCols, GPUPtr b, long bRows, long bCols,
                                      GPUPtr c, long cRows, long cCols, DevicePtr, CError* err) {
  return ew_binary(gonn::EW_DIV, "division", a, aRows, aCols, b, bRows, bCols, c, cRows, cCols, err);
}
int perform_mps_matrix_scalar_add(GPUPtr in, long rows, long cols, float scalar, GPUPtr out, DevicePtr,
                                  CError* err) {
  return ew_unary(gonn::EW_SCALAR_ADD, "input or output buffer pointers", in, nullptr, out,
                  rows < 0 || cols < 0 ? -1 : rows * cols, scalar, err);
}
int perform_mps_matrix_scalar_multiply(GPUPtr in, long rows, long cols, float scalar, GPUPtr out,
                                       DevicePtr, CError* err) {
  return ew_unary(gonn::EW_SCALAR_MUL, "input or output buffer pointers", in, nullptr, out,
                  rows < 0 || cols < 0 ? -1 : rows * cols, scalar, err);
}
int perform_activation_sigmoid_forward(GPUPtr in, long size, GPUPtr out, DevicePtr, CError* err) {
  return ew_unary(gonn::EW_SIGMOID, "buffer pointers for Sigmoid forward", in, nullptr, out, size, 0.f, err);
}
int perform_activation_sigmoid_backward(GPUPtr gradOut, GPUPtr actOut, long size, GPUPtr gradIn,
                                        DevicePtr, CError* err) {
  return ew_unary(gonn::EW_SIGMOID_BWD, "buffer pointers for Sigmoid backward", gradOut, actOut, gradIn,
                  size, 0.f, err);
}
int perform_activation_tanh_forward(GPUPtr in, long size, GPUPtr out, DevicePtr, CError* err) {
  return ew_unary(gonn::EW_TANH, "buffer pointers for Tanh forward", in, nullptr, out, size, 0.f, err);
}
int perform_activation_tanh_backward(GPUPtr gradOut, GPUPtr actOut, long size, GPUPtr gradIn, DevicePtr,
                                     CError* err) {
  return ew_unary(gonn::EW_TANH_BWD, "buffer pointers for Tanh backward", gradOut, actOut, gradIn, size,
                  0.f, err);
}
int perform_activation_leaky_relu_forward(GPUPtr in, long size, float alpha, GPUPtr out, DevicePtr,
                                          CError* err) {
  return ew_unary(gonn::EW_LEAKY, "buffer pointers for Leaky ReLU forward", in, nullptr, out, size, alpha,
                  err);
}
int perform_activation_leaky_relu_backward(GPUPtr gradOut, GPUPtr actOut, long size, float alpha,
                                           GPUPtr gradIn, DevicePtr, CError* err) {
  return ew_unary(gonn::EW_LEAKY_BWD, "buffer pointers for Leaky ReLU backward", gradOut, actOut, gradIn,
                  size, alpha, err);
}

int perform_activation_softmax_1d_forward(GPUPtr in, long size, GPUPtr out, DevicePtr, CError* err) {
  return ew_unary(0, "buffer pointers for Softmax 1D forward", in, nullptr, out, size, 0.f, err,
                  size > 0 ? 1 : 0);
}
int perform_activation_softmax_1d_backward(GPUPtr gradOut, GPUPtr actOut, long size, GPUPtr gradIn,
                                           DevicePtr, CError* err) {
  return ew_unary(0, "buffer pointers for Softmax 1D backward", gradOut, actOut, gradIn, size, 0.f, err,
                  size > 0 ? 1 : 0);
}
int perform_activation_softmax_2d_forward(GPUPtr in, long batchSize, long features, GPUPtr out, DevicePtr,
                                          CError* err) {
  const bool bad = batchSize < 0 || features < 0;
  return ew_unary(0, "buffer pointers for Softmax 2D forward", in, nullptr, out,
                  bad ? -1 : batchSize * features, 0.f, err, bad || features == 0 ? 0 : batchSize);
}
int perform_activation_softmax_2d_backward(GPUPtr gradOut, GPUPtr actOut, long batchSize, long features,
                                           GPUPtr gradIn, DevicePtr, CError* err) {
  const bool bad = batchSize < 0 || features < 0;
  return ew_unary(0, "buffer pointers for Softmax 2D backward", gradOut, actOut, gradIn,
                  bad ? -1 : batchSize * features, 0.f, err, bad || features == 0 ? 0 : batchSize);
}
int perform_activation_elu_forward(GPUPtr in, long size, float alpha, GPUPtr out, DevicePtr, CError* err) {
  return ew_unary(gonn::EW_ELU, "buffer pointers for ELU forward", in, nullptr, out, size, alpha, err);
}
int perform_activation_elu_backward(GPUPtr gradOut, GPUPtr actOut, long size, float alpha, GPUPtr gradIn,
                                    DevicePtr, CError* err) {
  return ew_unary(gonn::EW_ELU_BWD, "buffer pointers for ELU backward", gradOut, actOut, gradIn, size,
                  alpha, err);
}
int perform_activation_swish_forward(GPUPtr in, long size, GPUPtr out, DevicePtr, CError* err) {
  return ew_unary(gonn::EW_SWISH, "buffer pointers for Swish forward", in, nullptr, out, size, 0.f, err);
}
int perform_activation_swish_backward(GPUPtr gradOut, GPUPtr actOut, long size, GPUPtr gradIn, DevicePtr,
                                      CError* err) {
  return ew_unary(gonn::EW_SWISH_BWD, "buffer pointers for Swish backward", gradOut, actOut, gradIn, size,
                  0.f, err);
}
int perform_activation_gelu_forward(GPUPtr in, long size, GPUPtr out, DevicePtr, CError* err) {
  return ew_unary(gonn::EW_GELU, "buffer pointers for GELU forward", in, nullptr, out, size, 0.f, err);
}
int perform_activation_gelu_backward(GPUPtr gradOut, GPUPtr actOut, long size, GPUPtr gradIn, DevicePtr,
                                     CError* err) {
  return ew_unary(gonn::EW_GELU_BWD, "buffer pointers for GELU backward", gradOut, actOut, gradIn, size,
                  0.f, err);
}

int perform_batch_matmul_optimized(GPUPtr aPtr, GPUPtr bPtr, GPUPtr cPtr, long batchSize, long M,
                                   long N, long K, DevicePtr /*device*/, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* A = as_buffer(aPtr);
  Buffer* B = as_buffer(bPtr);
  Buffer* C = as_buffer(cPtr);
  if (!A || !B || !C) {
    set_error(err, "Invalid buffer pointers");
    return -2;
  }
  if (batchSize <= 0 || M <= 0 || N <= 0 || K <= 0 || M >= (1l << 31) || N >= (1l << 31) ||
      K >= (1l << 31) || batchSize * M >= (1l << 31) || batchSize * (K + 32) >= (1l << 31) ||
      size_t(batchSize) * M * K * 4 > A->bytes || size_t(batchSize) * K * N * 4 > B->bytes ||
      size_t(batchSize) * M * N * 4 > C->bytes || A->device != C->device || B->device != C->device ||
      C == A || C == B) {
    set_error(err, "batch matmul: invalid dimensions (batch %ld, M %ld, N %ld, K %ld).", batchSize, M, N,
              K);
    return -3;
  }
  if (ensure_device(C->device, err)) return -1;
  Device& d = g_dev[C->device];
  if (!make_resident(d, A) || !make_resident(d, B)) {
    cudaGetLastError();
    set_error(err, "batch matmul: host to device copy failed.");
    return -6;
  }
  Plane* pa = get_plane(d, A, uint64_t(batchSize) * M, uint64_t(K), 2);
  if (!pa) {
    set_error(err, "batch matmul: could not allocate operand planes.");
    return -3;
  }
  gonn::GemmOperand oa, ob;
  oa.plane0 = pa->p0;
  oa.plane1 = pa->p1;
  oa.pitch = pa->pitch;
  oa.mn_major = false;
  ob.mn_major = true;
  gonn::GemmBatch gb;
  gb.count = uint32_t(batchSize);
  void *thi = nullptr, *tlo = nullptr;
  size_t tbytes = 0;
  if (K % 32 == 0) {
    // the stacked B is its own padded layout
    Plane* pb = get_plane(d, B, uint64_t(batchSize) * K, uint64_t(N), 2);
    if (!pb) {
      set_error(err, "batch matmul: could not allocate operand planes.");
      return -3;
    }
    ob.plane0 = pb->p0;
    ob.plane1 = pb->p1;
    ob.pitch = pb->pitch;
    gb.b_rows = uint32_t(K);
  } else {
    // K is not a multiple of the k block: each batch of B gets zero rows up to the next
    // multiple, so that a k block never reads into the following batch
    const uint64_t kp = round_up(uint64_t(K), 32), pitch = round_up(uint64_t(N), 64);
    tbytes = size_t(batchSize) * kp * pitch * 4;
    if (pool_alloc(C->device, &thi, tbytes) != cudaSuccess ||
        pool_alloc(C->device, &tlo, tbytes) != cudaSuccess) {
      cudaGetLastError();
      if (thi) pool_free(C->device, thi, tbytes);
      set_error(err, "batch matmul: could not allocate operand planes.");
      return -3;
    }
    cudaMemsetAsync(thi, 0, tbytes, d.stream);
    cudaMemsetAsync(tlo, 0, tbytes, d.stream);
    for (long b = 0; b < batchSize; ++b) {
      gonn::launch_split_tf32(B->dptr + size_t(b) * K * N, uint64_t(K), uint64_t(N),
                              static_cast<float*>(thi) + size_t(b) * kp * pitch,
                              static_cast<float*>(tlo) + size_t(b) * kp * pitch, pitch, d.stream);
      ++g_stats[3];
    }
    ob.plane0 = thi;
    ob.plane1 = tlo;
    ob.pitch = pitch;
    gb.b_rows = uint32_t(kp);
  }
  gonn::GemmEpilogue epi;
  const char* msg = gonn::launch_gemm(gonn::Kind::TF32x3, uint32_t(M), uint32_t(N), uint32_t(K), oa, ob,
                                      C->dptr, uint64_t(N), epi, d.status_dev, d.sm_count, tune_for(d),
                                      d.stream, &gb);
  if (thi) {
    pool_free(C->device, thi, tbytes);
    pool_free(C->device, tlo, tbytes);
  }
  if (msg) {
    cudaGetLastError();
    set_error(err, "batch matmul: %s", msg);
    return -3;
  }
  ++g_stats[3];
  ++g_stats[4];
  wrote(C);
  return finish(d, err, -6, "batch matmul");
}

int gonngpu_linear_backward(GPUPtr xPtr, GPUPtr wPtr, GPUPtr dyPtr, GPUPtr actOutPtr, long batch,
                            long in_size, long out_size, GPUPtr dxPtr, GPUPtr dwPtr, GPUPtr dbPtr,
                            CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* X = as_buffer(xPtr);
  Buffer* W = as_buffer(wPtr);
  Buffer* dY = as_buffer(dyPtr);
  Buffer* act = actOutPtr ? as_buffer(actOutPtr) : nullptr;
  Buffer* dX = dxPtr ? as_buffer(dxPtr) : nullptr;
  Buffer* dW = dwPtr ? as_buffer(dwPtr) : nullptr;
  Buffer* db = dbPtr ? as_buffer(dbPtr) : nullptr;
  if (!dY || (actOutPtr && !act) || (dxPtr && !dX) || (dwPtr && !dW) || (dbPtr && !db) ||
      (dW && !X) || (dX && !W)) {
    set_error(err, "Invalid input or output buffer pointers.");
    return -2;
  }
  if (batch <= 0 || in_size <= 0 || out_size <= 0 || batch >= (1l << 31) || in_size >= (1l << 31) ||
      out_size >= (1l << 31)) {
    set_error(err, "linear backward: dimensions must be positive.");
    return -3;
  }
  const size_t by = size_t(batch) * out_size * 4;
  if (dY->bytes < by || (act && act->bytes < by) || (X && X->bytes < size_t(batch) * in_size * 4) ||
      (W && W->bytes < size_t(in_size) * out_size * 4) ||
      (dX && dX->bytes < size_t(batch) * in_size * 4) ||
      (dW && dW->bytes < size_t(in_size) * out_size * 4) || (db && db->bytes < size_t(out_size) * 4)) {
    set_error(err, "linear backward: a buffer is smaller than its stated matrix.");
    return -3;
  }
  const int dev = dY->device;
  for (Buffer* b : {X, W, act, dX, dW, db}) {
    if (b && b->device != dev) {
      set_error(err, "linear backward: buffers live on different devices.");
      return -2;
    }
  }
  if (ensure_device(dev, err)) return -1;
  Device& d = g_dev[dev];
  if (!make_resident(d, dY) || (act && !make_resident(d, act)) || (X && dW && !make_resident(d, X)) ||
      (W && dX && !make_resident(d, W))) {
    cudaGetLastError();
    set_error(err, "linear backward: host to device copy failed.");
    return -6;
  }
  // bias gradient: column sums of the masked gradient (in the same pass as the operand planes
  // of that gradient when the products are asked for too, see below)
  auto bias_gradient = [&] {
    gonn::launch_colsum(dY->dptr, uint64_t(batch), uint64_t(out_size), db->dptr, d.stream,
                        act ? act->dptr : nullptr, d.splitk_ws, kSplitKBytes / 4, d.splitk_counters,
                        kSplitKSlots);
    ++g_stats[3];
    wrote(db);
  };
  if (db && !dX && !dW) bias_gradient();
  int rc = 0;
  if (dX || dW) {
    // operand planes of dAct = dY (.) [actOut > 0]: the mask is applied while the
    // planes are written, the masked gradient itself is never stored
    const uint64_t pitch = round_up(uint64_t(out_size), 64);
    const size_t pbytes = size_t(batch) * pitch * 4;
    // each product takes the low planes of the kernel it will run on: bf16 planes on the
    // CTA-pair kernel, tf32 planes otherwise (a layer can need both: a small batch makes dX
    // a small product and dW a large one)
    const gonn::GemmTuning tune = tune_for(d);
    const bool dw_x = dW && gonn::tf32_takes_pair_kernel(uint32_t(in_size), uint32_t(out_size),
                                                         uint32_t(batch), d.sm_count, tune);
    const bool dx_x = dX && gonn::tf32_takes_pair_kernel(uint32_t(batch), uint32_t(in_size),
                                                         uint32_t(out_size), d.sm_count, tune);
    const bool need_lo = (dW && !dw_x) || (dX && !dx_x), need_x2 = dw_x || dx_x;
    void *hi = nullptr, *lo = nullptr, *x2 = nullptr;
    if (pool_alloc(dev, &hi, pbytes) != cudaSuccess ||
        (need_lo && pool_alloc(dev, &lo, pbytes) != cudaSuccess) ||
        (need_x2 && pool_alloc(dev, &x2, pbytes) != cudaSuccess)) {
      cudaGetLastError();
      if (hi) pool_free(dev, hi, pbytes);
      if (lo) pool_free(dev, lo, pbytes);
      set_error(err, "linear backward: could not allocate operand planes.");
      return -5;
    }
    // one kind of low planes and the bias gradient wanted: one kernel writes the planes and
    // the column sums
    bool summed = false;
    if (db && need_lo != need_x2) {
      summed = gonn::launch_split_colsum(dY->dptr, uint64_t(batch), uint64_t(out_size), static_cast<float*>(hi),
                                         need_x2 ? x2 : lo, need_x2, pitch, db->dptr, d.stream,
                                         act ? act->dptr : nullptr, d.splitk_ws, kSplitKBytes / 4,
                                         d.splitk_counters, kSplitKSlots);
      if (summed) {
        ++g_stats[3];
        wrote(db);
      }
    }
    if (db && !summed) bias_gradient();
    if (need_lo && !summed) {
      gonn::launch_split_tf32(dY->dptr, uint64_t(batch), uint64_t(out_size), static_cast<float*>(hi),
                              static_cast<float*>(lo), pitch, d.stream, act ? act->dptr : nullptr);
      ++g_stats[3];
    }
    if (need_x2 && !summed) {  // writes the same hi
      gonn::launch_split_tf32_bf16(dY->dptr, uint64_t(batch), uint64_t(out_size), static_cast<float*>(hi),
                                   x2, pitch, d.stream, act ? act->dptr : nullptr);
      ++g_stats[3];
    }
    auto dact = [&](bool bf16x) {  // dAct stored [batch, out]
      gonn::GemmOperand g;
      g.plane0 = hi;
      g.plane1 = bf16x ? x2 : lo;
      g.pitch = pitch;
      g.plane1_bf16 = bf16x;
      return g;
    };
    gonn::GemmEpilogue epi;
    const char* msg = nullptr;
    if (dW) {
      // dW[in, out] = X^T . dAct : A = X stored [batch(K), in(M)], B = dAct stored [batch(K), out(N)]
      Plane* px = get_plane(d, X, uint64_t(batch), uint64_t(in_size), dw_x ? 3 : 2);
      if (!px) {
        msg = "could not allocate operand planes";
      } else {
        gonn::GemmOperand a;
        a.plane0 = px->p0;
        a.plane1 = px->p1;
        a.pitch = px->pitch;
        a.mn_major = true;
        a.plane1_bf16 = dw_x;
        gonn::GemmOperand b = dact(dw_x);
        b.mn_major = true;
        msg = gonn::launch_gemm(gonn::Kind::TF32x3, uint32_t(in_size), uint32_t(out_size),
                                uint32_t(batch), a, b, dW->dptr, uint64_t(out_size), epi, d.status_dev,
                                d.sm_count, tune, d.stream);
        if (!msg) {
          ++g_stats[3];
          ++g_stats[4];
          wrote(dW);
        }
      }
    }
    if (!msg && dX) {
      // dX[batch, in] = dAct . W^T : A = dAct stored [batch(M), out(K)], B = W stored [in(N), out(K)]
      Plane* pw = get_plane(d, W, uint64_t(in_size), uint64_t(out_size), dx_x ? 3 : 2);
      if (!pw) {
        msg = "could not allocate operand planes";
      } else {
        gonn::GemmOperand a = dact(dx_x);
        a.mn_major = false;
        gonn::GemmOperand b;
        b.plane0 = pw->p0;
        b.plane1 = pw->p1;
        b.pitch = pw->pitch;
        b.mn_major = false;
        b.plane1_bf16 = dx_x;
        msg = gonn::launch_gemm(gonn::Kind::TF32x3, uint32_t(batch), uint32_t(in_size),
                                uint32_t(out_size), a, b, dX->dptr, uint64_t(in_size), epi,
                                d.status_dev, d.sm_count, tune, d.stream);
        if (!msg) {
          ++g_stats[3];
          ++g_stats[4];
          wrote(dX);
        }
      }
    }
    // The planes go back to the cache; later work on the same stream may reuse them
    // only after the GEMMs above (stream order).
    pool_free(dev, hi, pbytes);
    if (lo) pool_free(dev, lo, pbytes);
    if (x2) pool_free(dev, x2, pbytes);
    if (msg) {
      cudaGetLastError();
      set_error(err, "linear backward: %s", msg);
      rc = -4;
    }
  }
  const int frc = finish(d, err && rc == 0 ? err : nullptr, -6, "linear backward");
  return rc ? rc : frc;
}

int gonngpu_column_sum(GPUPtr inPtr, long rows, long cols, GPUPtr outPtr, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* in = as_buffer(inPtr);
  Buffer* out = as_buffer(outPtr);
  if (!in || !out) {
    set_error(err, "Invalid input or output buffer pointers.");
    return -2;
  }
  if (rows < 0 || cols < 0 || size_t(rows) * cols * 4 > in->bytes || size_t(cols) * 4 > out->bytes ||
      in->device != out->device) {
    set_error(err, "column sum: invalid dimensions.");
    return -3;
  }
  if (ensure_device(out->device, err)) return -1;
  Device& d = g_dev[out->device];
  if (!make_resident(d, in)) {
    cudaGetLastError();
    set_error(err, "column sum: host to device copy failed.");
    return -6;
  }
  gonn::launch_colsum(in->dptr, uint64_t(rows), uint64_t(cols), out->dptr, d.stream, nullptr, d.splitk_ws,
                      kSplitKBytes / 4, d.splitk_counters, kSplitKSlots);
  ++g_stats[3];
  wrote(out);
  return finish(d, err, -6, "column sum");
}

int gonngpu_alloc_device_buffer(long length_bytes, GPUPtr* out, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (!out || length_bytes < 0) {
    set_error(err, "Could not create buffer: invalid arguments.");
    return -3;
  }
  Buffer* b = nullptr;
  if (int rc = new_buffer(g_current, nullptr, size_t(length_bytes), nullptr, &b, err)) return rc;
  *out = b;
  return 0;
}

int gonngpu_wrap_device_memory(void* device_ptr, long length_bytes, GPUPtr* out, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (!out || !device_ptr || length_bytes < 0) {
    set_error(err, "Could not wrap device memory: invalid arguments.");
    return -3;
  }
  Buffer* b = nullptr;
  if (int rc = new_buffer(g_current, nullptr, size_t(length_bytes), device_ptr, &b, err)) return rc;
  *out = b;
  return 0;
}

void* gonngpu_device_address(GPUPtr buffer) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* b = as_buffer(buffer);
  if (!b) return nullptr;
  if (b->host_pending) {
    if (ensure_device(b->device, nullptr)) return nullptr;
    Device& d = g_dev[b->device];
    if (!make_resident(d, b) || cudaStreamSynchronize(d.stream) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
  }
  return b->dptr;
}

int gonngpu_upload(GPUPtr buffer, const float* data, long length_bytes, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* b = as_buffer(buffer);
  if (!b) {
    set_error(err, "Invalid GPU buffer pointer.");
    return -1;
  }
  if (length_bytes < 0 || size_t(length_bytes) > b->bytes || (length_bytes > 0 && !data)) {
    set_error(err, "Buffer length mismatch during upload.");
    return -2;
  }
  if (ensure_device(b->device, err)) return -3;
  Device& d = g_dev[b->device];
  if (size_t(length_bytes) < b->bytes && !make_resident(d, b)) {
    cudaGetLastError();
    set_error(err, "Host to device copy failed.");
    return -3;
  }
  if (!copy_h2d(d, b->dptr, data, size_t(length_bytes))) {
    cudaGetLastError();
    set_error(err, "Host to device copy failed.");
    return -3;
  }
  wrote(b);
  // Pageable sources were staged synchronously except for the last chunks in
  // flight; blocking mode waits for them too.
  if (g_blocking || !host_is_pinned(data)) {
    if (cudaStreamSynchronize(d.stream) != cudaSuccess) {
      cudaGetLastError();
      set_error(err, "Host to device copy failed.");
      return -3;
    }
  }
  return 0;
}

// float64 host data <-> float32 device buffer; the conversion runs on the device,
// one scratch chunk at a time (stream order makes the reuse of the chunk safe).
namespace {
constexpr size_t kF64ChunkElems = size_t(32) << 20;  // 256 MiB of float64 per chunk
}

int gonngpu_upload_f64(GPUPtr buffer, const double* data, long count, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* b = as_buffer(buffer);
  if (!b) {
    set_error(err, "Invalid GPU buffer pointer.");
    return -1;
  }
  if (count < 0 || size_t(count) * 4 > b->bytes || (count > 0 && !data)) {
    set_error(err, "Buffer length mismatch during float64 upload.");
    return -2;
  }
  if (ensure_device(b->device, err)) return -3;
  Device& d = g_dev[b->device];
  if (size_t(count) * 4 < b->bytes && !make_resident(d, b)) {
    cudaGetLastError();
    set_error(err, "Host to device copy failed.");
    return -3;
  }
  const size_t n = size_t(count);
  const size_t chunk = n < kF64ChunkElems ? n : kF64ChunkElems;
  void* scratch = nullptr;
  if (n > 0 && pool_alloc(b->device, &scratch, chunk * 8) != cudaSuccess) {
    cudaGetLastError();
    set_error(err, "Out of device memory for the float64 staging chunk (%zu bytes).", chunk * 8);
    return -3;
  }
  bool ok = true;
  for (size_t off = 0; ok && off < n; off += chunk) {
    const size_t m = n - off < chunk ? n - off : chunk;
    ok = copy_h2d(d, scratch, data + off, m * 8);
    if (ok) {
      gonn::launch_f64_to_f32(static_cast<const double*>(scratch), b->dptr + off, m, d.stream);
      ++g_stats[3];
    }
  }
  wrote(b);
  // the scratch chunk goes back to the pool only once the stream is done with it
  ok = ok && cudaStreamSynchronize(d.stream) == cudaSuccess && cudaGetLastError() == cudaSuccess;
  if (scratch) pool_free(b->device, scratch, chunk * 8);
  if (!ok) {
    cudaGetLastError();
    set_error(err, "Host to device copy failed.");
    return -3;
  }
  return 0;
}

int gonngpu_retrieve_f64(GPUPtr buffer, double* data, long count, CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* b = as_buffer(buffer);
  if (!b) {
    set_error(err, "Invalid GPU buffer pointer.");
    return -1;
  }
  if (count < 0 || size_t(count) * 4 > b->bytes || (count > 0 && !data)) {
    set_error(err, "Buffer length mismatch during float64 retrieval.");
    return -2;
  }
  if (ensure_device(b->device, err)) return -3;
  Device& d = g_dev[b->device];
  if (!make_resident(d, b)) {
    cudaGetLastError();
    set_error(err, "Host to device copy failed.");
    return -3;
  }
  const size_t n = size_t(count);
  const size_t chunk = n < kF64ChunkElems ? n : kF64ChunkElems;
  void* scratch = nullptr;
  if (n > 0 && pool_alloc(b->device, &scratch, chunk * 8) != cudaSuccess) {
    cudaGetLastError();
    set_error(err, "Out of device memory for the float64 staging chunk (%zu bytes).", chunk * 8);
    return -3;
  }
  bool ok = true;
  for (size_t off = 0; ok && off < n; off += chunk) {
    const size_t m = n - off < chunk ? n - off : chunk;
    gonn::launch_f32_to_f64(b->dptr + off, static_cast<double*>(scratch), m, d.stream);
    ++g_stats[3];
    ok = copy_d2h(d, data + off, scratch, m * 8);  // complete on return
  }
  ok = ok && cudaGetLastError() == cudaSuccess;
  if (scratch) {
    cudaStreamSynchronize(d.stream);
    pool_free(b->device, scratch, chunk * 8);
  }
  if (!ok) {
    cudaGetLastError();
    set_error(err, "Device to host copy failed.");
    return -3;
  }
  return 0;
}

int gonngpu_mark_modified(GPUPtr buffer) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  Buffer* b = as_buffer(buffer);
  if (!b) return -1;
  wrote(b);
  return 0;
}

void* gonngpu_host_alloc(long bytes) {
  if (bytes <= 0) return nullptr;
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (ensure_device(g_current, nullptr)) return nullptr;
  void* p = nullptr;
  if (cudaHostAlloc(&p, size_t(bytes), cudaHostAllocPortable) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  std::memset(p, 0, size_t(bytes));
  return p;
}

void gonngpu_host_free(void* p) {
  if (!p) return;
  cudaFreeHost(p);
  cudaGetLastError();
}

int gonngpu_inject_fault(const char* kind, int nth) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (!kind || nth < 0) return -3;
  int k = -1;
  if (std::strcmp(kind, "alloc") == 0) k = FAULT_ALLOC;
  else if (std::strcmp(kind, "h2d") == 0) k = FAULT_H2D;
  else if (std::strcmp(kind, "d2h") == 0) k = FAULT_D2H;
  if (k < 0) return -3;
  g_fault_countdown[k] = nth;
  return 0;
}

int gonngpu_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int gonngpu_set_device(int ordinal) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (int rc = ensure_device(ordinal, nullptr)) return rc;
  g_current = ordinal;
  return 0;
}

int gonngpu_get_device(void) { return g_current; }

void* gonngpu_stream(void) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (ensure_device(g_current, nullptr)) return nullptr;
  return g_dev[g_current].stream;
}

int gonngpu_set_blocking(int blocking) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  g_blocking = blocking != 0;
  return 0;
}

int gonngpu_synchronize(CError* err) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (int rc = ensure_device(g_current, err)) return rc;
  Device& d = g_dev[g_current];
  const bool was = g_blocking;
  g_blocking = true;
  const int rc = finish(d, err, -6, "synchronize");
  g_blocking = was;
  return rc;
}

int gonngpu_set_plane_cache(int enabled) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  g_plane_cache = enabled != 0;
  return 0;
}

int gonngpu_set_gemm_tuning(int block_n, int max_ctas) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (block_n != 0 && block_n != 32 && block_n != 64 && block_n != 128 && block_n != 256) return -1;
  g_tune.block_n = block_n;
  g_tune.max_ctas = max_ctas < 0 ? 0 : max_ctas;
  return 0;
}

int gonngpu_set_sharded_tuning(int sender_pairs, int late_rounds) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (sender_pairs < -1 || sender_pairs > 74 || late_rounds < -1 || late_rounds > 64) return -1;
  g_shard_sender_pairs = sender_pairs;
  g_shard_late_rounds = late_rounds;
  return 0;
}

int gonngpu_set_sharded_trace(void* device_words) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  g_shard_trace = device_words;
  return 0;
}

int gonngpu_set_gemm_split_k(int splits) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (splits < 0 || splits > 64) return -1;
  g_tune.split_k = splits;
  return 0;
}

int gonngpu_set_gemm_pair_mode(int mode) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  if (mode < -1 || mode > 2) return -1;
  g_tune.pair = mode;
  return 0;
}

long gonngpu_trim_cache(void) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  long freed = 0;
  int prev = 0;
  cudaGetDevice(&prev);
  for (int dev = 0; dev < kMaxDevices; ++dev) {
    if (g_pool[dev].empty()) continue;
    if (cudaSetDevice(dev) != cudaSuccess) continue;
    if (g_dev[dev].ready) cudaStreamSynchronize(g_dev[dev].stream);
    for (auto& kv : g_pool[dev]) {
      cudaFree(kv.second);
      freed += long(kv.first);
    }
    g_pool[dev].clear();
    g_pool_bytes[dev] = 0;
    g_small_pool_bytes[dev] = 0;
  }
  cudaSetDevice(prev);
  cudaGetLastError();
  return freed;
}

void gonngpu_get_stats(long out[8]) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  for (int i = 0; i < 8; ++i) out[i] = g_stats[i];
  long cached = 0;
  for (int dev = 0; dev < kMaxDevices; ++dev) cached += long(g_pool_bytes[dev]);
  out[7] = cached;
}

void gonngpu_last_kernel_status(unsigned out[4]) {
  std::lock_guard<std::recursive_mutex> lk(g_mu);
  const GemmStatus& s = g_dev[g_current].last_status;
  out[0] = s.code;
  out[1] = s.where;
  out[2] = s.tile;
  out[3] = s.kblock;
}

const char* gonngpu_version(void) { return "gonngpu-cuda 0.1 (sm_100a)"; }

}  // extern "C"
