// Test oracle: MLXR's Metal dequantizer functions, compiled from the reference tree as host
// C++ through ref_shim/metal_stdlib and exported with a C interface.
//   core/kernels/metal/q_gemm_dequant.metal:142-259  dequant_q4_0/_q4_1/_q8_0/_q4_k
//   core/kernels/metal/swiglu_mlp_fused.metal:92-99   swish
// REF_METAL_DIR is given by the Makefile; no reference source is copied into this repo.
#include <metal_stdlib>
#include <cstdint>

#define MLXR_STR2(x) #x
#define MLXR_STR(x) MLXR_STR2(x)

namespace ref_qgemm {
#include MLXR_STR(REF_QGEMM_METAL)
}

extern "C" {
#define EXPORT __attribute__((visibility("default")))

// Dequantize nblocks blocks of format qt (MLXR QuantType value) into binary16 bits.
// Q4_K: all 8 sub-blocks of each super-block.
EXPORT int ref_shader_dequant(int qt, const void* blocks, long nblocks, uint16_t* out) {
  using namespace ref_qgemm;
  static_assert(sizeof(metal::half) == 2, "half must be 2 bytes");
  static_assert(sizeof(BlockQ4_0) == 18 && sizeof(BlockQ4_1) == 20 && sizeof(BlockQ8_0) == 34 &&
                sizeof(BlockQ4_K) == 144, "block layout");
  metal::half* o = reinterpret_cast<metal::half*>(out);
  for (long b = 0; b < nblocks; b++) {
    switch (qt) {
      case 0: dequant_q4_0(reinterpret_cast<const BlockQ4_0*>(blocks) + b, o, (metal::uint)(b * 32)); break;
      case 1: dequant_q4_1(reinterpret_cast<const BlockQ4_1*>(blocks) + b, o, (metal::uint)(b * 32)); break;
      case 2: dequant_q8_0(reinterpret_cast<const BlockQ8_0*>(blocks) + b, o, (metal::uint)(b * 32)); break;
      case 3:
        for (metal::uint s = 0; s < 8; s++)
          dequant_q4_k(reinterpret_cast<const BlockQ4_K*>(blocks) + b, o, (metal::uint)(b * 256 + s * 32), s);
        break;
      default: return -1;
    }
  }
  return 0;
}
}
