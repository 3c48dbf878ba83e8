// Shape-generic quantized GEMM: Y[M,N] = X[M,K] * dequant(W[N,K])^T (+ bias).
//
// This is the kernel for shapes the specialised kernels do not take (K not a multiple of
// 256, rows whose byte length is not a multiple of 16, formats without a fast path).  It
// uses exactly the reference's dequantized weight values (dequant_unit) and accumulates
// in fp32, the arithmetic of kernel q_gemm_dequant (q_gemm_dequant.metal:443-461).
#include "common.cuh"
#include <atomic>

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


// ---- small-batch GEMV for the 32-/64-element block formats ----------------------------------------
// Q4_0, Q4_1, Q8_0 and NF4 at batch <= 8 (Q4_K and Q4_0 with K >= 512 go to the persistent decode
// kernel instead).  HBM-bound: one warp per weight row, eight rows per CTA.  The row is staged into
// shared memory in chunks of 4096 weights with coalesced 16-byte loads (block boundaries of 18 /
// 20 / 34 bytes do not line up with vector loads), then the warp walks the chunk 128 weights at a
// time: lane l takes weights 4l .. 4l+3, so the activations are read conflict-free and the block
// scale is a broadcast.  Values are the reference's fp32 products (q_gemm_dequant_primitive.mm:
// 189-225), accumulated in fp32.
constexpr int kGemvChunk = 4096;

// 16-bit read from the staged row in shared memory (ld_u16 is a read-only GLOBAL load)
__device__ __forceinline__ uint16_t sm_u16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }

template <int QT>
__device__ __forceinline__ void gemv_weights4(const uint8_t* chunk, int step, int lane, const float* nf4, float (&wv)[4]) {
  if constexpr (QT == MLXR_Q8_0) {
    const uint8_t* blk = chunk + (size_t)(4 * step + (lane >> 3)) * 34;
    const float s = __half2float(h_from_bits(sm_u16(blk)));
    const uint32_t v = (uint32_t)sm_u16(blk + 2 + 4 * (lane & 7)) | ((uint32_t)sm_u16(blk + 4 + 4 * (lane & 7)) << 16);
#pragma unroll
    for (int j = 0; j < 4; j++) wv[j] = (float)(int)(int8_t)((v >> (8 * j)) & 0xFFu) * s;
  } else if constexpr (QT == MLXR_Q4_0) {
    const uint8_t* blk = chunk + (size_t)(4 * step + (lane >> 3)) * 18;
    const float s = __half2float(h_from_bits(sm_u16(blk)));
    const uint32_t v = sm_u16(blk + 2 + 2 * (lane & 7));
#pragma unroll
    for (int j = 0; j < 4; j++) wv[j] = (float)((int)((v >> (4 * j)) & 15u) - 8) * s;
  } else if constexpr (QT == MLXR_Q4_1) {
    const uint8_t* blk = chunk + (size_t)(4 * step + (lane >> 3)) * 20;
    const float s = __half2float(h_from_bits(sm_u16(blk))), m = __half2float(h_from_bits(sm_u16(blk + 2)));
    const uint32_t v = sm_u16(blk + 4 + 2 * (lane & 7));
#pragma unroll
    for (int j = 0; j < 4; j++) wv[j] = __fadd_rn(__fmul_rn((float)((v >> (4 * j)) & 15u), s), m);
  } else {  // NF4: 64 weights per 34-byte block
    const uint8_t* blk = chunk + (size_t)(2 * step + (lane >> 4)) * 34;
    const float a = __half2float(h_from_bits(sm_u16(blk)));
    const uint32_t v = sm_u16(blk + 2 + 2 * (lane & 15));
#pragma unroll
    for (int j = 0; j < 4; j++) wv[j] = nf4[(v >> (4 * j)) & 15u] * a;
  }
}

template <int QT, typename T, int MB>
__global__ void __launch_bounds__(256) gemv_rows_kernel(const T* __restrict__ x, const uint8_t* __restrict__ w,
                                                        const T* __restrict__ bias, T* __restrict__ y, int M, int N,
                                                        int K, size_t row_bytes) {
  extern __shared__ __align__(16) uint8_t gsm[];
  constexpr int be = (QT == MLXR_NF4) ? 64 : 32;
  constexpr int bb = (QT == MLXR_Q4_0) ? 18 : (QT == MLXR_Q4_1) ? 20 : 34;
  constexpr int kChunkBytes = kGemvChunk / be * bb;                 // multiple of 16
  T* xs = reinterpret_cast<T*>(gsm);                                 // [MB][kGemvChunk]
  uint8_t* wrows = gsm + (size_t)MB * kGemvChunk * sizeof(T);        // [8][kChunkBytes]
  float* nf4 = reinterpret_cast<float*>(wrows + 8 * kChunkBytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (QT == MLXR_NF4 && tid < 16) nf4[tid] = kNF4[tid];
  const int n = blockIdx.x * 8 + warp;
  const bool live = n < N;
  const uint8_t* row = w + (size_t)(live ? n : 0) * row_bytes;
  uint8_t* mine = wrows + (size_t)warp * kChunkBytes;
  float acc[MB];
#pragma unroll
  for (int m = 0; m < MB; m++) acc[m] = 0.0f;
  for (int k0 = 0; k0 < K; k0 += kGemvChunk) {
    const int kc = min(kGemvChunk, K - k0);                          // a multiple of 256
    __syncthreads();                                                  // previous chunk fully consumed
    for (int m = 0; m < MB; m++)
      if (m < M)
        for (int i = tid * 8; i < kc; i += 256 * 8) {
          if constexpr (sizeof(T) == 2) *reinterpret_cast<uint4*>(xs + (size_t)m * kGemvChunk + i) = __ldg(reinterpret_cast<const uint4*>(x + (size_t)m * K + k0 + i));
          else {
            *reinterpret_cast<uint4*>(xs + (size_t)m * kGemvChunk + i) = __ldg(reinterpret_cast<const uint4*>(x + (size_t)m * K + k0 + i));
            *reinterpret_cast<uint4*>(xs + (size_t)m * kGemvChunk + i + 4) = __ldg(reinterpret_cast<const uint4*>(x + (size_t)m * K + k0 + i + 4));
          }
        }
    if (live) {
      const int nb16 = kc / be * bb / 16;
      const uint4* src = reinterpret_cast<const uint4*>(row + (size_t)(k0 / be) * bb);
      for (int i = lane; i < nb16; i += 32) reinterpret_cast<uint4*>(mine)[i] = __ldcs(src + i);   // streamed once
    }
    __syncthreads();
    if (live) {
      for (int step = 0; step < kc / 128; step++) {
        float wv[4];
        gemv_weights4<QT>(mine, step, lane, nf4, wv);
#pragma unroll
        for (int m = 0; m < MB; m++) {
          if (m < M) {
            const T* xp = xs + (size_t)m * kGemvChunk + step * 128 + 4 * lane;
            float s = acc[m];
#pragma unroll
            for (int j = 0; j < 4; j++) s = fmaf(Act<T>::to_f(xp[j]), wv[j], s);
            acc[m] = s;
          }
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MB; m++) {
    const float r = warp_sum(acc[m]);
    if (live && lane == 0 && m < M) {
      float v = r;
      if (bias) v += Act<T>::to_f(bias[n]);
      y[(size_t)m * N + n] = Act<T>::from_f(v);
    }
  }
}

bool gemv_rows_supported(int qt, int M, int K, const void* x, const void* w) {
  if (qt != MLXR_Q4_0 && qt != MLXR_Q4_1 && qt != MLXR_Q8_0 && qt != MLXR_NF4) return false;
  if (M < 1 || M > 8 || K % 256 != 0) return false;
  // rows (and with them the 4096-weight chunks) must start on 16-byte boundaries: NF4 needs K % 512
  if (((size_t)(K / block_elems(qt)) * block_bytes(qt)) % 16 != 0) return false;
  return ((((uintptr_t)x) | ((uintptr_t)w)) & 15u) == 0;
}

template <int QT, typename T, int MB>
static int launch_gemv_inst(const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                            size_t row_bytes, cudaStream_t st) {
  constexpr int be = (QT == MLXR_NF4) ? 64 : 32;
  constexpr int bb = (QT == MLXR_Q4_0) ? 18 : (QT == MLXR_Q4_1) ? 20 : 34;
  constexpr size_t smem = (size_t)MB * kGemvChunk * sizeof(T) + 8 * (size_t)(kGemvChunk / be * bb) + 64;
  auto kern = gemv_rows_kernel<QT, T, MB>;
  // set once per device; the call is idempotent, the flags are atomic so that concurrent first
  // launches from several host threads do not race on them
  static std::atomic<bool> attr_done[64] = {};
  int dev = 0;
  MLXR_CUDA_TRY(cudaGetDevice(&dev));
  if (smem > 48 * 1024 && !attr_done[dev & 63].load(std::memory_order_acquire)) {
    MLXR_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done[dev & 63].store(true, std::memory_order_release);
  }
  kern<<<(N + 7) / 8, 256, smem, st>>>((const T*)x, (const uint8_t*)w, (const T*)bias, (T*)y, M, N, K, row_bytes);
  MLXR_LAUNCH_CHECK("gemv_rows_kernel");
  return MLXR_OK;
}

int launch_gemv_rows(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int qt, int dtype,
                     cudaStream_t st) {
  if (M == 0 || N == 0) return MLXR_OK;
  const size_t row_bytes = (size_t)(K / block_elems(qt)) * block_bytes(qt);
  int rc = MLXR_ERR_UNSUPPORTED;
#define MLXR_GEMV_MB(QTV, T)                                                                              \
  do {                                                                                                    \
    if (M == 1) rc = launch_gemv_inst<QTV, T, 1>(x, w, bias, y, M, N, K, row_bytes, st);                  \
    else if (M == 2) rc = launch_gemv_inst<QTV, T, 2>(x, w, bias, y, M, N, K, row_bytes, st);             \
    else if (M <= 4) rc = launch_gemv_inst<QTV, T, 4>(x, w, bias, y, M, N, K, row_bytes, st);             \
    else rc = launch_gemv_inst<QTV, T, 8>(x, w, bias, y, M, N, K, row_bytes, st);                         \
  } while (0)
#define MLXR_GEMV_QT(QTV)                                                           \
  do {                                                                              \
    if (dtype == MLXR_F16) MLXR_GEMV_MB(QTV, __half);                               \
    else if (dtype == MLXR_BF16) MLXR_GEMV_MB(QTV, __nv_bfloat16);                  \
    else MLXR_GEMV_MB(QTV, float);                                                  \
  } while (0)
  switch (qt) {
    case MLXR_Q4_0: MLXR_GEMV_QT(MLXR_Q4_0); break;
    case MLXR_Q4_1: MLXR_GEMV_QT(MLXR_Q4_1); break;
    case MLXR_Q8_0: MLXR_GEMV_QT(MLXR_Q8_0); break;
    case MLXR_NF4: MLXR_GEMV_QT(MLXR_NF4); break;
    default: set_error("gemv_rows: no code for %d", qt); break;
  }
#undef MLXR_GEMV_QT
#undef MLXR_GEMV_MB
  return rc;
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
