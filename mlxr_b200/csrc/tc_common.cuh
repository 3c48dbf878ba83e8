// Device-side building blocks shared by the tensor-core kernels: mbarrier and TMA wrappers,
// tcgen05 (MMA, tensor memory) wrappers, shared-memory and instruction descriptors, and the Q4_K
// sub-block conversions to 16-bit pairs.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace mlxr {
namespace tc {

constexpr uint32_t kSpin = 1u << 22;   // bound of every mbarrier wait, in polls
constexpr int kUmmaK = 16;             // K of one kind::f16 MMA

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// The same poll, but the hardware may park the thread for up to `ns` nanoseconds while the phase
// is incomplete (it resumes as soon as the phase completes): a waiting warp then issues no
// instructions instead of competing for issue slots with the warps that have work.
__device__ __forceinline__ bool mbar_try_park(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
  return ok != 0;
}
// Bounded wait; false when it gave up or another role already did.  kParkPolls polls of up to
// kParkNs each bound it to about a quarter of a second.
constexpr uint32_t kParkNs = 2000, kParkPolls = 1u << 17;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* dead) {
  if (mbar_try(bar, parity)) return true;
  for (uint32_t i = 0; i < kParkPolls; i++) {
    if (mbar_try_park(bar, parity, kParkNs)) return true;
    if ((i & 7u) == 7u && *dead) return false;
  }
  *dead = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// ---- tcgen05 wrappers ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrive on an mbarrier once every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives lane (base + i)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile with the 128-byte swizzle: rows are 128
// bytes, groups of 8 rows are 1024 bytes apart (stride byte offset), descriptor version 1
// (sm_100), layout type 2 (SWIZZLE_128B).  The tile base is 1024-byte aligned; a K step of 16
// elements inside the swizzle row advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);        // start address, bits 0-13
  d |= (uint64_t)0 << 16;                         // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024u >> 4) << 32;              // stride byte offset, bits 32-45
  d |= (uint64_t)1 << 46;                         // descriptor version
  d |= (uint64_t)2 << 61;                         // SWIZZLE_128B
  return d;
}
// Instruction descriptor of kind::f16: fp32 accumulate, A and B of format `fmt` (0 fp16, 1 bf16),
// both K-major, N and M of the MMA.
__host__ __device__ constexpr uint32_t instr_desc(int afmt, int bfmt, int m, int n) {
  return (1u << 4) | ((uint32_t)afmt << 7) | ((uint32_t)bfmt << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <typename T> struct Fmt;
template <> struct Fmt<__half> { static constexpr int v = 0; };
template <> struct Fmt<__nv_bfloat16> { static constexpr int v = 1; };

// Eight consecutive weights of a Q4_K sub-block (one 32-bit word of nibbles, element order =
// nibble order) -> four packed pairs of the activation dtype.
//
// fp16 activations: the shader's arithmetic exactly (q_gemm_dequant.metal:244-256).  1024 + n as
// fp16 is 0x6400 | n; subtracting 1032 gives n - 8 exactly; then rn16(rn16((n - 8) * ss) + sm).
__device__ __forceinline__ uint4 dequant8_f16(uint32_t v, __half2 ss, __half2 sm) {
  const uint32_t lo = v & 0x0F0F0F0Fu, hi = (v >> 4) & 0x0F0F0F0Fu;
  const __half2 off = __half2half2(__ushort_as_half((unsigned short)0x6408));   // 1032
  uint32_t out[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const uint32_t sel = (uint32_t)j | ((uint32_t)j << 4) | ((uint32_t)(4 + j) << 8) | ((uint32_t)(4 + j) << 12);
    uint32_t bits = (__byte_perm(lo, hi, sel) & 0x00FF00FFu) | 0x64006400u;
    const __half2 q = __hsub2(*reinterpret_cast<__half2*>(&bits), off);
    const __half2 r = __hadd2_rn(__hmul2_rn(q, ss), sm);
    out[j] = *reinterpret_cast<const uint32_t*>(&r);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}
// bf16 activations: the weight is rounded to bf16 for the MMA anyway (2^-9 relative), so the two
// fp16 roundings of the shader are not reproduced; one fp32 multiply-add per weight from the
// exact fp16 scale and min, then one rounding to bf16.  The nibble becomes the fp32 number
// 128 + n by a byte permute (bits 0x4300'0000 | n << 16), so w = (128 + n) * ss + (sm - 136 ss).
__device__ __forceinline__ uint4 dequant8_bf16(uint32_t v, float ss, float c) {
  const uint32_t lo = v & 0x0F0F0F0Fu, hi = (v >> 4) & 0x0F0F0F0Fu;
  uint32_t out[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    // result bytes (0, 0, nibble, 0x43): sources 6/7 are the zero bytes of 0x00004300, 5 is 0x43
    const float fe = __uint_as_float(__byte_perm(lo, 0x00004300u, 0x5066u | ((uint32_t)j << 8)));
    const float fo = __uint_as_float(__byte_perm(hi, 0x00004300u, 0x5066u | ((uint32_t)j << 8)));
    __nv_bfloat162 b = __floats2bfloat162_rn(fmaf(fe, ss, c), fmaf(fo, ss, c));
    out[j] = *reinterpret_cast<const uint32_t*>(&b);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

}  // namespace tc
}  // namespace mlxr
