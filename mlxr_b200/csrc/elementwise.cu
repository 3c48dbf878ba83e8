// RMSNorm, SwiGLU and RoPE as standalone kernels (the fused decode kernels carry their
// own copies of this arithmetic; these serve the primitives called on their own and the
// prefill path, where the GEMM dominates and the elementwise work is one HBM pass).
#include "common.cuh"

namespace mlxr {

// ---- RMSNorm ---------------------------------------------------------------------------
// One CTA per row: y = (x * rsqrt(mean(x^2) + eps)) * w (+ residual), fp32 throughout, one
// rounding at the store (rmsnorm.metal:105-156, :165-217).  The row is read once from
// HBM and kept in registers for the second pass (the reference reads it twice).
template <typename T, int THREADS, int PER_THREAD>
__global__ void __launch_bounds__(THREADS) rmsnorm_kernel(const T* __restrict__ x,
                                                          const T* __restrict__ w,
                                                          const T* __restrict__ res,
                                                          T* __restrict__ y, int hidden,
                                                          float eps) {
  __shared__ float red[THREADS / 32];
  // A kernel launched behind this one with programmatic stream serialization (the linears of the
  // MLP block) may start its set-up and its weight stream now; it waits for this kernel's
  // completion before it reads y.  Without such a dependent the instruction does nothing.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const size_t row = blockIdx.x;
  const T* xr = x + row * hidden;
  float v[PER_THREAD];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < PER_THREAD; i++) {
    const int c = threadIdx.x + i * THREADS;
    v[i] = c < hidden ? Act<T>::to_f(xr[c]) : 0.0f;
    ss = fmaf(v[i], v[i], ss);
  }
  // columns beyond THREADS * PER_THREAD (very wide rows) are streamed without caching
  for (int c = threadIdx.x + PER_THREAD * THREADS; c < hidden; c += THREADS) {
    const float t = Act<T>::to_f(xr[c]);
    ss = fmaf(t, t, ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; i++) tot += red[i];
  const float rms = rsqrtf(tot / (float)hidden + eps);
#pragma unroll
  for (int i = 0; i < PER_THREAD; i++) {
    const int c = threadIdx.x + i * THREADS;
    if (c < hidden) {
      float o = (v[i] * rms) * Act<T>::to_f(w[c]);
      if (res) o += Act<T>::to_f(res[row * hidden + c]);
      y[row * hidden + c] = Act<T>::from_f(o);
    }
  }
  for (int c = threadIdx.x + PER_THREAD * THREADS; c < hidden; c += THREADS) {
    float o = (Act<T>::to_f(xr[c]) * rms) * Act<T>::to_f(w[c]);
    if (res) o += Act<T>::to_f(res[row * hidden + c]);
    y[row * hidden + c] = Act<T>::from_f(o);
  }
}

int launch_rmsnorm(const void* x, const void* w, const void* res, void* y, int rows, int hidden,
                   float eps, int dtype, cudaStream_t st) {
  if (rows == 0 || hidden == 0) return MLXR_OK;
  MLXR_DISPATCH_DTYPE(dtype, T, {
    if (hidden <= 1024)
      rmsnorm_kernel<T, 128, 8><<<rows, 128, 0, st>>>((const T*)x, (const T*)w, (const T*)res,
                                                      (T*)y, hidden, eps);
    else
      rmsnorm_kernel<T, 512, 16><<<rows, 512, 0, st>>>((const T*)x, (const T*)w, (const T*)res,
                                                       (T*)y, hidden, eps);
  });
  MLXR_LAUNCH_CHECK("rmsnorm_kernel");
  return MLXR_OK;
}

// ---- swish / swiglu --------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ g,
                                                     const T* __restrict__ u, T* __restrict__ o,
                                                     size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    float s = swish_f(Act<T>::to_f(g[i]));
    if (u) s *= Act<T>::to_f(u[i]);
    o[i] = Act<T>::from_f(s);
  }
}

int launch_swiglu(const void* g, const void* u, void* o, size_t n, int dtype, cudaStream_t st) {
  if (n == 0) return MLXR_OK;
  size_t blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  MLXR_DISPATCH_DTYPE(dtype, T, {
    swiglu_kernel<T><<<(int)blocks, 256, 0, st>>>((const T*)g, (const T*)u, (T*)o, n);
  });
  MLXR_LAUNCH_CHECK("swiglu_kernel");
  return MLXR_OK;
}

// ---- widening cast (partial sums of a sharded linear on the generic path) ------------------
template <typename T>
__global__ void __launch_bounds__(256) cast_f32_kernel(const T* __restrict__ x, float* __restrict__ y, size_t n) {
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) y[i] = Act<T>::to_f(x[i]);
}

template <typename T>
__global__ void __launch_bounds__(256) cast_from_f32_kernel(const float* __restrict__ x, T* __restrict__ y, size_t n) {
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) y[i] = Act<T>::from_f(x[i]);
}

int launch_cast_from_f32(const float* x, void* y, size_t n, int dtype, cudaStream_t st) {
  if (n == 0) return MLXR_OK;
  size_t blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  MLXR_DISPATCH_DTYPE(dtype, T, { cast_from_f32_kernel<T><<<(int)blocks, 256, 0, st>>>(x, (T*)y, n); });
  MLXR_LAUNCH_CHECK("cast_from_f32_kernel");
  return MLXR_OK;
}

int launch_cast_to_f32(const void* x, float* y, size_t n, int dtype, cudaStream_t st) {
  if (n == 0) return MLXR_OK;
  size_t blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  MLXR_DISPATCH_DTYPE(dtype, T, { cast_f32_kernel<T><<<(int)blocks, 256, 0, st>>>((const T*)x, y, n); });
  MLXR_LAUNCH_CHECK("cast_f32_kernel");
  return MLXR_OK;
}

// ---- RoPE ------------------------------------------------------------------------------
// One thread per (token, head, pair): interleaved pairs (2p, 2p+1), binary16 tables, fp32
// math, one rounding at the store (rope_apply.metal:103-172).  A token whose position
// falls outside the table is left untouched and flagged in *status.
template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const T* __restrict__ x,
                                                   const __half* __restrict__ cos_t,
                                                   const __half* __restrict__ sin_t,
                                                   const int32_t* __restrict__ positions,
                                                   T* __restrict__ y, size_t tokens, int heads,
                                                   int pairs, int max_seq, int linear,
                                                   float scale, int offset, int* status) {
  const size_t total = tokens * heads * pairs;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int p = (int)(i % pairs);
    const size_t th = i / pairs;  // token * heads + head
    const size_t tok = th / heads;
    const long long pos = (long long)positions[tok] + offset;
    if (pos < 0 || pos >= max_seq) {
      if (status) atomicExch(status, 1);
      continue;
    }
    const float c = __half2float(cos_t[(size_t)pos * pairs + p]);
    const float s = __half2float(sin_t[(size_t)pos * pairs + p]);
    const size_t e = th * (size_t)(2 * pairs) + 2 * p;
    const float xe = Act<T>::to_f(x[e]), xo = Act<T>::to_f(x[e + 1]);
    float ye = __fsub_rn(__fmul_rn(xe, c), __fmul_rn(xo, s));
    float yo = __fadd_rn(__fmul_rn(xo, c), __fmul_rn(xe, s));
    if (linear) { ye *= scale; yo *= scale; }
    y[e] = Act<T>::from_f(ye);
    y[e + 1] = Act<T>::from_f(yo);
  }
}

int launch_rope(const void* x, const uint16_t* cos_t, const uint16_t* sin_t,
                const int32_t* positions, void* y, size_t tokens, int heads, int head_dim,
                int max_seq, int mode, float scale, int offset, int dtype, int* status,
                cudaStream_t st) {
  const size_t total = tokens * heads * (head_dim / 2);
  if (total == 0) return MLXR_OK;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  MLXR_DISPATCH_DTYPE(dtype, T, {
    rope_kernel<T><<<(int)blocks, 256, 0, st>>>(
        (const T*)x, (const __half*)cos_t, (const __half*)sin_t, positions, (T*)y, tokens, heads,
        head_dim / 2, max_seq, mode == MLXR_ROPE_LINEAR, scale, offset, status);
  });
  MLXR_LAUNCH_CHECK("rope_kernel");
  return MLXR_OK;
}

// ---- RoPE, split-half convention --------------------------------------------------------
// graph::RotaryEmbedding::forward (core/graph/layers.cpp:157-225): the head is split in two
// halves (x1 = first d/2 elements, x2 = the rest), positions are the contiguous range
// offset .. offset + seq, tables are float32 [max_seq, d/2]:
//   y1 = x1 * cos - x2 * sin,  y2 = x2 * cos + x1 * sin
// as four products and two sums, each rounded to float32 (the composition materialises every
// product as an array); one rounding to T at the store.  One thread per (token, head, p).
template <typename T>
__global__ void __launch_bounds__(256) rope_split_half_kernel(const T* __restrict__ x, const float* __restrict__ cos_t,
                                                              const float* __restrict__ sin_t, T* __restrict__ y,
                                                              size_t batch, int seq, int heads, int half, int offset) {
  const size_t total = batch * seq * heads * half;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int p = (int)(i % half);
    const size_t th = i / half;            // (batch * seq + t) * heads + head
    const int t = (int)((th / heads) % seq);
    const size_t tab = (size_t)(offset + t) * half + p;
    const float c = cos_t[tab], sn = sin_t[tab];
    const size_t e = th * (size_t)(2 * half) + p;
    const float x1 = Act<T>::to_f(x[e]), x2 = Act<T>::to_f(x[e + half]);
    y[e] = Act<T>::from_f(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn)));
    y[e + half] = Act<T>::from_f(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sn)));
  }
}

int launch_rope_split_half(const void* x, const float* cos_t, const float* sin_t, void* y, size_t batch, int seq,
                           int heads, int head_dim, int offset, int dtype, cudaStream_t st) {
  const size_t total = batch * seq * heads * (head_dim / 2);
  if (total == 0) return MLXR_OK;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  MLXR_DISPATCH_DTYPE(dtype, T, {
    rope_split_half_kernel<T><<<(int)blocks, 256, 0, st>>>((const T*)x, cos_t, sin_t, (T*)y, batch, seq, heads,
                                                           head_dim / 2, offset);
  });
  MLXR_LAUNCH_CHECK("rope_split_half_kernel");
  return MLXR_OK;
}

}  // namespace mlxr
