// Standalone dequantizer: packed [N, K] blocks -> dense [N, K] fp16 or fp32, bit for bit
// what MLXR's dequantizers produce (q_gemm_dequant_primitive.mm:189-225 for fp32,
// q_gemm_dequant.metal:142-286 for half).
#include "common.cuh"

namespace mlxr {

// One thread per 32-element unit.  A unit's 32 outputs are contiguous, so each thread
// stores 64 B (half) or 128 B (float) with 16-byte vector stores.
template <int QT, bool FUSED, typename OutT>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* __restrict__ w,
                                                         OutT* __restrict__ out, int N,
                                                         int units_per_row, size_t row_bytes) {
  const size_t total = (size_t)N * units_per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t n = idx / units_per_row;
    const int u = (int)(idx % units_per_row);
    float v[32];
    dequant_unit<QT, FUSED, sizeof(OutT) == 2>(w + n * row_bytes, u, v);
    OutT* o = out + (n * units_per_row + u) * 32;
    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
      for (int i = 0; i < 8; i++)
        reinterpret_cast<float4*>(o)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
      // For Q4_0 / Q4_1 / Q8_0 / NF4 the half result is the fp32 product rounded once
      // (the product itself is exact in fp32, so this equals the shader's half
      // multiply); for Q4_1 / Q4_K / Q6_K v already holds half values (half arithmetic
      // in dequant_unit), so the conversion is exact.
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const __half2 h0 = __floats2half2_rn(v[8 * i + 0], v[8 * i + 1]);
        const __half2 h1 = __floats2half2_rn(v[8 * i + 2], v[8 * i + 3]);
        const __half2 h2 = __floats2half2_rn(v[8 * i + 4], v[8 * i + 5]);
        const __half2 h3 = __floats2half2_rn(v[8 * i + 6], v[8 * i + 7]);
        uint4 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&h0);
        pk.y = *reinterpret_cast<const uint32_t*>(&h1);
        pk.z = *reinterpret_cast<const uint32_t*>(&h2);
        pk.w = *reinterpret_cast<const uint32_t*>(&h3);
        reinterpret_cast<uint4*>(o)[i] = pk;
      }
    }
  }
}

// Canonical ggml Q4_0 -> MLXR Q4_0: one thread per block; element i (low nibble of qs[i]) and
// element i + 16 (high nibble) go to byte i/2 / (i+16)/2 as the low (even element) or high nibble.
__global__ void __launch_bounds__(256) repack_ggml_q4_0_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, size_t nblocks) {
  for (size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += (size_t)gridDim.x * blockDim.x) {
    const uint8_t* s = src + b * 18;
    uint8_t* d = dst + b * 18;
    uint8_t q[16];
#pragma unroll
    for (int i = 0; i < 8; i++) { const uint32_t v = ld_u16(s + 2 + 2 * i); q[2 * i] = (uint8_t)(v & 0xFFu); q[2 * i + 1] = (uint8_t)(v >> 8); }
    *reinterpret_cast<uint16_t*>(d) = ld_u16(s);
    uint8_t o[16];
#pragma unroll
    for (int i = 0; i < 8; i++) {
      o[i] = (uint8_t)((q[2 * i] & 0x0F) | ((q[2 * i + 1] & 0x0F) << 4));          // elements 2i, 2i+1 (< 16): low nibbles
      o[8 + i] = (uint8_t)((q[2 * i] >> 4) | ((q[2 * i + 1] >> 4) << 4));          // elements 16+2i, 17+2i: high nibbles
    }
#pragma unroll
    for (int i = 0; i < 8; i++) *reinterpret_cast<uint16_t*>(d + 2 + 2 * i) = (uint16_t)(o[2 * i] | (o[2 * i + 1] << 8));
  }
}

int launch_repack_ggml_q4_0(const void* src, void* dst, size_t nblocks, cudaStream_t st) {
  if (nblocks == 0) return MLXR_OK;
  size_t blocks = (nblocks + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  repack_ggml_q4_0_kernel<<<(int)blocks, 256, 0, st>>>((const uint8_t*)src, (uint8_t*)dst, nblocks);
  MLXR_LAUNCH_CHECK("repack_ggml_q4_0_kernel");
  return MLXR_OK;
}

int launch_dequantize(const void* w, void* out, int N, int K, int qt, int out_dtype, int flags,
                      cudaStream_t st) {
  const int units = K / 32;
  const size_t row_bytes = (size_t)(K / block_elems(qt)) * block_bytes(qt);
  const size_t total = (size_t)N * units;
  if (total == 0) return MLXR_OK;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 32) blocks = 148 * 32;
  const bool fused = (flags & 1) != 0;
#define LAUNCH(QT, FU, OT)                                                          \
  dequantize_kernel<QT, FU, OT><<<blocks, 256, 0, st>>>((const uint8_t*)w, (OT*)out, N, units, row_bytes)
  MLXR_DISPATCH_QT(qt, QT, {
    if (out_dtype == MLXR_F32) {
      if (fused && QT == MLXR_Q4_K) LAUNCH(QT, true, float); else LAUNCH(QT, false, float);
    } else {
      if (fused && (QT == MLXR_Q4_K || QT == MLXR_Q4_1)) LAUNCH(QT, true, __half);
      else LAUNCH(QT, false, __half);
    }
  });
#undef LAUNCH
  MLXR_LAUNCH_CHECK("dequantize_kernel");
  return MLXR_OK;
}

}  // namespace mlxr
