// gonngpu_matmul_f16_static_scratch: the fp16-path MatMul for callers that
// must not allocate.
//
// Every other GEMM entry point of this library converts its float32 operands
// into fp16 "operand planes" that it cudaMalloc's on demand.  Some callers
// cannot live with that: a host program that hands all of HBM to its own arena
// at start-up (a later cudaMalloc then fails), or one that calls MatMul from a
// latency-critical loop where cudaMalloc / cudaFree would synchronise the whole
// device under it.  For them this file keeps the planes in a fixed array that
// is part of the library image: `g_scratch` below, kScratchBytes of HBM on
// every GPU that loads the library, held until the process exits.
//
// The entry point calls no cudaMalloc, cudaFree, cudaHostAlloc, stream or event
// creation, and no library routine that allocates; it touches none of the
// state the other entry points share.
//
// Set-up: `g_scratch` as named in host code is only a host-side stand-in for
// the symbol, not a device address.  The first call on each device (with that
// device current) asks the runtime for the real address with
// cudaGetSymbolAddress and caches it.  With CUDA's lazy module loading that
// first call is also when the driver loads this library's kernels and the
// array, taking device memory of its own for them.  A caller that reserves the
// rest of HBM for itself therefore makes one small warm-up call per device
// first (or sets CUDA_MODULE_LOADING=EAGER), and makes it before any stream
// capture is begun.  Every call ends with cudaStreamSynchronize on its stream.
//
// Sharing: all calls use the same array and it keeps the previous call's
// contents.  Nothing in it has to start at zero except the kernel's status
// words, which every call clears.  Two calls whose device work overlaps (two
// streams, two threads) race on the array; serialise them.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/gonngpu.h"
#include "kernels.h"

namespace {

constexpr size_t kScratchBytes = size_t(GONNGPU_STATIC_SCRATCH_BYTES);
constexpr size_t kStatusBytes = 256;  // first 256 bytes: GemmStatus, then the planes
constexpr int kMaxDevices = 16;

static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

std::mutex g_ss_mu;
void* g_scratch_addr[kMaxDevices] = {};  // device address of g_scratch, per device
int g_sm_count[kMaxDevices] = {};

void ss_error(CError* err, const char* fmt, ...) {
  if (!err) return;
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  err->message = strdup(buf);
}

inline size_t round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }

}  // namespace

extern "C" int gonngpu_matmul_f16_static_scratch(const float* a, long aRows, long aCols,
                                                  const float* b, long bRows, long bCols, float* c,
                                                  void* stream_handle, CError* err) {
  std::lock_guard<std::mutex> lk(g_ss_mu);
  if (!a || !b || !c) {
    ss_error(err, "static-scratch matmul: NULL operand pointer.");
    return -2;
  }
  if (aRows <= 0 || aCols <= 0 || bRows <= 0 || bCols <= 0 || aCols != bRows ||
      aRows >= (1l << 31) || bCols >= (1l << 31) || aCols >= (1l << 31)) {
    ss_error(err, "static-scratch matmul: incompatible dimensions A %ldx%ld, B %ldx%ld.", aRows,
             aCols, bRows, bCols);
    return -3;
  }
  // Plane layout inside the array: [status | A as fp16, pitch padded to 64 | B likewise].
  const size_t pitch_a = round_up(size_t(aCols), 64), pitch_b = round_up(size_t(bCols), 64);
  const size_t bytes_a = round_up(size_t(aRows) * pitch_a * 2, 256);
  const size_t bytes_b = round_up(size_t(bRows) * pitch_b * 2, 256);
  if (kStatusBytes + bytes_a + bytes_b > kScratchBytes) {
    ss_error(err,
             "static-scratch matmul: operands need %zu bytes of fp16 planes but the built-in "
             "scratch holds %zu; use gonngpu_matmul_ex for this size.",
             bytes_a + bytes_b, kScratchBytes - kStatusBytes);
    return -3;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    ss_error(err, "static-scratch matmul: no current CUDA device.");
    return -1;
  }
  if (!g_scratch_addr[dev]) {
    // once per device, with that device current
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_scratch);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      ss_error(err, "static-scratch matmul: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return -1;
    }
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        major != 10) {
      cudaGetLastError();
      ss_error(err, "static-scratch matmul: device %d is not an sm_100 GPU.", dev);
      return -1;
    }
    g_sm_count[dev] = sms;
    g_scratch_addr[dev] = p;
  }
  unsigned char* base = static_cast<unsigned char*>(g_scratch_addr[dev]);
  gonn::GemmStatus* status = reinterpret_cast<gonn::GemmStatus*>(base);
  void* plane_a = base + kStatusBytes;
  void* plane_b = base + kStatusBytes + bytes_a;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);

  if (cudaMemsetAsync(status, 0, sizeof(gonn::GemmStatus), stream) != cudaSuccess) {
    cudaGetLastError();
    ss_error(err, "static-scratch matmul: could not clear the status words.");
    return -6;
  }
  gonn::launch_cvt_f16(a, uint64_t(aRows), uint64_t(aCols), plane_a, pitch_a, gonn::F16_RN, stream);
  gonn::launch_cvt_f16(b, uint64_t(bRows), uint64_t(bCols), plane_b, pitch_b, gonn::F16_RN, stream);
  gonn::GemmOperand oa, ob;
  oa.plane0 = plane_a;
  oa.pitch = pitch_a;
  oa.mn_major = false;  // A stored [M, K]
  ob.plane0 = plane_b;
  ob.pitch = pitch_b;
  ob.mn_major = true;  // B stored [K, N]
  gonn::GemmEpilogue epi;
  gonn::GemmTuning tune;
  const char* msg = gonn::launch_gemm(gonn::Kind::F16, uint32_t(aRows), uint32_t(bCols),
                                      uint32_t(aCols), oa, ob, c, uint64_t(bCols), epi, status,
                                      g_sm_count[dev], tune, stream);
  if (msg) {
    cudaGetLastError();
    ss_error(err, "static-scratch matmul: %s", msg);
    return -4;
  }
  gonn::GemmStatus host_status;
  cudaError_t e = cudaMemcpyAsync(&host_status, status, sizeof(host_status), cudaMemcpyDeviceToHost,
                                  stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    ss_error(err, "static-scratch matmul: CUDA error: %s", cudaGetErrorString(e));
    return -6;
  }
  if (host_status.code != 0) {
    ss_error(err, "static-scratch matmul: GEMM kernel gave up waiting (role %u, tile %u, k block %u).",
             host_status.code, host_status.tile, host_status.kblock);
    return -6;
  }
  return 0;
}
