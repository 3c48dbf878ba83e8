// mlxr_q_gemm_dequant_static: the decode linear without any allocation.
//
// The regular entry points keep a workspace per (device, stream) that they cudaMalloc on first
// use.  Some callers cannot afford that: a serving engine that has handed all free device memory
// to its own pool (the KV-cache arena) may find cudaMalloc failing at an arbitrary later moment,
// and on a latency-critical path the device-wide synchronisation an allocation implies stalls
// every other stream.  This variant runs the same persistent decode kernel with its scratch
// (split-K partial sums, barrier and tile-counter words, status word) in a fixed array that is
// part of the loaded module, so no call here - first or later - allocates or frees device memory.
//
// Consequences of the fixed array:
//   * sizes are limited (MLXR_STATIC_MAX_N rows; anything larger is refused, not truncated);
//   * the array exists once per device: two calls in flight at the same time on one device
//     (different streams) would share counters and partial sums and race.  Calls on one stream,
//     or otherwise ordered one after the other, are fine;
//   * the first call on a device looks up the array's address, clears the words that must start
//     at zero and sets the kernel's attributes.  Make that first call outside any stream capture.
#include <mutex>

#include "../../include/mlxr_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace mlxr {
namespace {

constexpr size_t kStaticPartialBytes = (size_t)4 << 20;        // split-K partial sums
constexpr size_t kStaticSyncBytes = kSyncWords * sizeof(uint32_t);
constexpr size_t kStaticBytes = kStaticPartialBytes + kStaticSyncBytes + 256;

// [partials 4 MiB][sync words 16 KiB][status word, padded]
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

struct PerDevice {
  unsigned char* base = nullptr;
  uint32_t bar_host = 0;
};
std::mutex g_mu;
PerDevice g_dev[64];

// Address of the array on the current device; on the first call per device also zero the
// barrier / counter / status words (the kernel leaves them at zero after every clean run).
int static_scratch(cudaStream_t st, PerDevice** out) {
  int dev = 0;
  MLXR_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) { set_error("device index %d outside 0..63", dev); return MLXR_ERR_INVALID_ARGUMENT; }
  std::lock_guard<std::mutex> lk(g_mu);
  PerDevice& d = g_dev[dev];
  if (!d.base) {
    unsigned char* ptr = nullptr;
    MLXR_CUDA_TRY(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
    MLXR_CUDA_TRY(cudaMemsetAsync(ptr + kStaticPartialBytes, 0, kStaticSyncBytes + 256, st));
    d.base = ptr;
  }
  *out = &d;
  return MLXR_OK;
}

}  // namespace
}  // namespace mlxr

using namespace mlxr;

extern "C" int mlxr_q_gemm_dequant_static(const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                                          int quant_type, int dtype, void* stream) {
  if (dtype != MLXR_F16 && dtype != MLXR_BF16 && dtype != MLXR_F32) {
    set_error("dtype must be MLXR_F16, MLXR_BF16 or MLXR_F32 (got %d)", dtype);
    return MLXR_ERR_INVALID_ARGUMENT;
  }
  if (M < 0 || N < 0 || K <= 0) { set_error("bad dimensions M=%d N=%d K=%d", M, N, K); return MLXR_ERR_SHAPE; }
  if (M == 0 || N == 0) return MLXR_OK;
  if (!x || !w || !y) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (N > MLXR_STATIC_MAX_N) {
    set_error("mlxr_q_gemm_dequant_static: N = %d exceeds the limit of %d rows its fixed scratch is sized for; "
              "use mlxr_q_gemm_dequant", N, MLXR_STATIC_MAX_N);
    return MLXR_ERR_WORKSPACE;
  }
  if (!decode_supported(quant_type, M, K, &w, 1)) {
    set_error("mlxr_q_gemm_dequant_static takes the decode shapes only: Q4_K or Q4_0, 1 <= M <= 8, K a multiple "
              "of 256 and >= 512, weights 16-byte aligned (got %s, M=%d, K=%d)", mlxr_quant_type_name(quant_type), M, K);
    return MLXR_ERR_UNSUPPORTED;
  }
  cudaStream_t st = (cudaStream_t)stream;
  PerDevice* d = nullptr;
  if (int r = static_scratch(st, &d)) return r;
  uint32_t* sync = reinterpret_cast<uint32_t*>(d->base + kStaticPartialBytes);
  int* status = reinterpret_cast<int*>(d->base + kStaticPartialBytes + kStaticSyncBytes);
  DecodeLinear L;
  memset(&L, 0, sizeof(L));
  L.w[0] = w; L.rows[0] = N; L.nmat = 1; L.K = K; L.x = x; L.y[0] = y; L.bias[0] = bias;
  const int rc = launch_decode(&L, 1, M, quant_type, dtype, d->base, kStaticPartialBytes, sync, &d->bar_host, status, st);
  if (rc == MLXR_ERR_WORKSPACE)
    set_error("mlxr_q_gemm_dequant_static: this shape (M=%d N=%d K=%d) needs more split-K scratch than the fixed "
              "%zu bytes; use mlxr_q_gemm_dequant", M, N, K, kStaticPartialBytes);
  return rc;
}

extern "C" int mlxr_static_status(void* stream, int* status_out) {
  cudaStream_t st = (cudaStream_t)stream;
  PerDevice* d = nullptr;
  if (int r = static_scratch(st, &d)) return r;
  int* status = reinterpret_cast<int*>(d->base + kStaticPartialBytes + kStaticSyncBytes);
  int value = 0;
  // pageable destination: the copy is staged by the driver and complete when the call returns
  MLXR_CUDA_TRY(cudaMemcpyAsync(&value, status, sizeof(int), cudaMemcpyDeviceToHost, st));
  MLXR_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int), st));
  MLXR_CUDA_TRY(cudaStreamSynchronize(st));
  if (status_out) *status_out = value;
  if (value == MLXR_ERR_TIMEOUT) set_error("a bounded device-side wait expired in an earlier mlxr_q_gemm_dequant_static call on this device");
  return MLXR_OK;
}
