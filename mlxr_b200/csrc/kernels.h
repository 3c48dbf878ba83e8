// Host-side launchers of the CUDA kernels (one per .cu file) and shared constants.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace mlxr {

// Zero-initialised 32-bit words per workspace for counters and barriers.
constexpr int kSyncWords = 4096;

int launch_dequantize(const void* w, void* out, int N, int K, int qt, int out_dtype, int flags,
                      cudaStream_t st);
int launch_qgemm_generic(const void* x, const void* w, const void* bias, void* y, int M, int N,
                         int K, int qt, int dtype, cudaStream_t st);
int launch_rmsnorm(const void* x, const void* w, const void* res, void* y, int rows, int hidden,
                   float eps, int dtype, cudaStream_t st);
int launch_swiglu(const void* g, const void* u, void* o, size_t n, int dtype, cudaStream_t st);
int launch_rope(const void* x, const uint16_t* cos_t, const uint16_t* sin_t,
                const int32_t* positions, void* y, size_t tokens, int heads, int head_dim,
                int max_seq, int mode, float scale, int offset, int dtype, int* status,
                cudaStream_t st);

}  // namespace mlxr
