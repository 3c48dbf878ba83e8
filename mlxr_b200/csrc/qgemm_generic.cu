// Shape-generic quantized GEMM: Y[M,N] = X[M,K] * dequant(W[N,K])^T (+ bias).
//
// This is the kernel for shapes the specialised kernels do not take (K not a multiple of
// 256, rows whose byte length is not a multiple of 16, formats without a fast path).  It
// uses exactly the reference's dequantized weight values (dequant_unit) and accumulates
// in fp32, the arithmetic of kernel q_gemm_dequant (q_gemm_dequant.metal:443-461).
#include "common.cuh"

namespace mlxr {

// One warp per weight row, MT activation rows at a time.  Lane l dequantizes units
// l, l+32, ... of the row (32 weights each) and multiplies them with MT rows of X; the
// lanes' partial sums meet in a shuffle reduction.
template <int QT, typename T, int MT>
__global__ void __launch_bounds__(128) qgemm_generic_kernel(
    const T* __restrict__ x, const uint8_t* __restrict__ w, const T* __restrict__ bias,
    T* __restrict__ y, int M, int N, int K, size_t row_bytes) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 4 + warp;
  if (n >= N) return;
  const uint8_t* row = w + (size_t)n * row_bytes;
  const int units = K >> 5;
  for (int m0 = blockIdx.y * MT; m0 < M; m0 += gridDim.y * MT) {
    float acc[MT];
#pragma unroll
    for (int i = 0; i < MT; i++) acc[i] = 0.0f;
    for (int u = lane; u < units; u += 32) {
      float wv[32];
      dequant_unit<QT>(row, u, wv);
#pragma unroll
      for (int i = 0; i < MT; i++) {
        if (m0 + i < M) {
          const T* xp = x + (size_t)(m0 + i) * K + (size_t)u * 32;
          float s = 0.0f;
#pragma unroll
          for (int k = 0; k < 32; k++) s = fmaf(Act<T>::to_f(xp[k]), wv[k], s);
          acc[i] += s;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < MT; i++) {
      const float r = warp_sum(acc[i]);
      if (lane == 0 && m0 + i < M) {
        float v = r;
        if (bias) v += Act<T>::to_f(bias[n]);
        y[(size_t)(m0 + i) * N + n] = Act<T>::from_f(v);
      }
    }
  }
}

// Dense weights W[N,K] of the activation dtype (the unquantized Linear / swiglu_mlp of the
// reference): same one-warp-per-row scheme, fp32 accumulation.
template <typename T, int MT>
__global__ void __launch_bounds__(128) linear_dense_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                           const T* __restrict__ bias, T* __restrict__ y,
                                                           int M, int N, int K) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 4 + warp;
  if (n >= N) return;
  const T* row = w + (size_t)n * K;
  for (int m0 = blockIdx.y * MT; m0 < M; m0 += gridDim.y * MT) {
    float acc[MT];
#pragma unroll
    for (int i = 0; i < MT; i++) acc[i] = 0.0f;
    for (int k = lane; k < K; k += 32) {
      const float wv = Act<T>::to_f(row[k]);
#pragma unroll
      for (int i = 0; i < MT; i++)
        if (m0 + i < M) acc[i] = fmaf(Act<T>::to_f(x[(size_t)(m0 + i) * K + k]), wv, acc[i]);
    }
#pragma unroll
    for (int i = 0; i < MT; i++) {
      const float r = warp_sum(acc[i]);
      if (lane == 0 && m0 + i < M) {
        float v = r;
        if (bias) v += Act<T>::to_f(bias[n]);
        y[(size_t)(m0 + i) * N + n] = Act<T>::from_f(v);
      }
    }
  }
}

int launch_linear_dense(const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                        int dtype, cudaStream_t st) {
  if (M == 0 || N == 0) return MLXR_OK;
  constexpr int MT = 4;
  int gy = (M + MT - 1) / MT;
  if (gy > 4096) gy = 4096;
  dim3 grid((N + 3) / 4, gy);
  MLXR_DISPATCH_DTYPE(dtype, T, {
    linear_dense_kernel<T, MT><<<grid, 128, 0, st>>>((const T*)x, (const T*)w, (const T*)bias, (T*)y, M, N, K);
  });
  MLXR_LAUNCH_CHECK("linear_dense_kernel");
  return MLXR_OK;
}

int launch_qgemm_generic(const void* x, const void* w, const void* bias, void* y, int M, int N,
                         int K, int qt, int dtype, cudaStream_t st) {
  if (M == 0 || N == 0) return MLXR_OK;
  const size_t row_bytes = (size_t)(K / block_elems(qt)) * block_bytes(qt);
  constexpr int MT = 4;
  int gy = (M + MT - 1) / MT;
  if (gy > 4096) gy = 4096;
  dim3 grid((N + 3) / 4, gy);
  MLXR_DISPATCH_QT(qt, QT, {
    MLXR_DISPATCH_DTYPE(dtype, T, {
      qgemm_generic_kernel<QT, T, MT><<<grid, 128, 0, st>>>(
          (const T*)x, (const uint8_t*)w, (const T*)bias, (T*)y, M, N, K, row_bytes);
    });
  });
  MLXR_LAUNCH_CHECK("qgemm_generic_kernel");
  return MLXR_OK;
}

}  // namespace mlxr
