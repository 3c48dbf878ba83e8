// Minimal stand-in for <mlx/dtype.h>: the subset of mlx::core::Dtype that MLXR's kernel
// primitives and graph layers touch.  MLX itself is Apple-only and is not a dependency
// of this build; these headers keep MLXR's call sites source-compatible.
#pragma once
#include <cstdint>
#include <cstring>

namespace mlx {
namespace core {

struct Dtype {
  enum class Val { bool_, uint8, uint16, uint32, uint64, int8, int16, int32, int64, float16, float32, float64, bfloat16 };
  constexpr Dtype(Val v, uint8_t s) : val_(v), size_(s) {}
  constexpr operator Val() const { return val_; }
  constexpr Val val() const { return val_; }
  constexpr uint8_t size() const { return size_; }
  Val val_;
  uint8_t size_;
};
inline constexpr bool operator==(const Dtype& a, const Dtype& b) { return a.val_ == b.val_; }
inline constexpr bool operator!=(const Dtype& a, const Dtype& b) { return a.val_ != b.val_; }

inline constexpr Dtype bool_{Dtype::Val::bool_, 1};
inline constexpr Dtype uint8{Dtype::Val::uint8, 1};
inline constexpr Dtype uint16{Dtype::Val::uint16, 2};
inline constexpr Dtype uint32{Dtype::Val::uint32, 4};
inline constexpr Dtype uint64{Dtype::Val::uint64, 8};
inline constexpr Dtype int8{Dtype::Val::int8, 1};
inline constexpr Dtype int16{Dtype::Val::int16, 2};
inline constexpr Dtype int32{Dtype::Val::int32, 4};
inline constexpr Dtype int64{Dtype::Val::int64, 8};
inline constexpr Dtype float16{Dtype::Val::float16, 2};
inline constexpr Dtype float32{Dtype::Val::float32, 4};
inline constexpr Dtype float64{Dtype::Val::float64, 8};
inline constexpr Dtype bfloat16{Dtype::Val::bfloat16, 2};

inline const char* dtype_name(Dtype d) {
  switch (d.val()) {
    case Dtype::Val::bool_: return "bool";
    case Dtype::Val::uint8: return "uint8";
    case Dtype::Val::uint16: return "uint16";
    case Dtype::Val::uint32: return "uint32";
    case Dtype::Val::uint64: return "uint64";
    case Dtype::Val::int8: return "int8";
    case Dtype::Val::int16: return "int16";
    case Dtype::Val::int32: return "int32";
    case Dtype::Val::int64: return "int64";
    case Dtype::Val::float16: return "float16";
    case Dtype::Val::float32: return "float32";
    case Dtype::Val::float64: return "float64";
    case Dtype::Val::bfloat16: return "bfloat16";
  }
  return "?";
}

// Storage-only 16-bit float types with round-to-nearest-even conversion from float.
struct float16_t {
  uint16_t bits = 0;
  float16_t() = default;
  float16_t(float f);
  operator float() const;
};
struct bfloat16_t {
  uint16_t bits = 0;
  bfloat16_t() = default;
  bfloat16_t(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) { bits = (uint16_t)((u >> 16) | 0x40u); return; }
    u += 0x7FFFu + ((u >> 16) & 1u);
    bits = (uint16_t)(u >> 16);
  }
  operator float() const {
    uint32_t u = (uint32_t)bits << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
  }
};

inline float16_t::float16_t(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7FFFFFFFu;
  if (x >= 0x7F800000u) { bits = (uint16_t)(sign | (x > 0x7F800000u ? 0x7E00u : 0x7C00u)); return; }
  if (x >= 0x477FF000u) { bits = (uint16_t)(sign | 0x7C00u); return; }
  if (x < 0x33000001u) { bits = (uint16_t)sign; return; }
  const int e = (int)(x >> 23) - 127;
  const uint32_t m = (x & 0x7FFFFFu) | 0x800000u;
  const int shift = e < -14 ? (13 + (-14 - e)) : 13;
  uint32_t r = m >> shift;
  const uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (r & 1u))) r++;
  bits = e < -14 ? (uint16_t)(sign | r) : (uint16_t)(sign | (((uint32_t)(e + 15) << 10) + (r - 0x400u)));
}
inline float16_t::operator float() const {
  const uint32_t sign = ((uint32_t)bits & 0x8000u) << 16;
  uint32_t e = (bits >> 10) & 0x1Fu, m = bits & 0x3FFu, u;
  if (e == 0) {
    if (m == 0) { u = sign; }
    else {
      int sh = 0;
      while (!(m & 0x400u)) { m <<= 1; sh++; }
      u = sign | ((uint32_t)(113 - sh) << 23) | ((m & 0x3FFu) << 13);
    }
  } else if (e == 31) {
    u = sign | 0x7F800000u | (m << 13);
  } else {
    u = sign | ((e + 112u) << 23) | (m << 13);
  }
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

template <typename T> struct TypeToDtype;
#define MLX_SHIM_T2D(T, D) template <> struct TypeToDtype<T> { constexpr operator Dtype() const { return D; } }
MLX_SHIM_T2D(bool, bool_);
MLX_SHIM_T2D(uint8_t, uint8);
MLX_SHIM_T2D(uint16_t, uint16);
MLX_SHIM_T2D(uint32_t, uint32);
MLX_SHIM_T2D(uint64_t, uint64);
MLX_SHIM_T2D(int8_t, int8);
MLX_SHIM_T2D(int16_t, int16);
MLX_SHIM_T2D(int32_t, int32);
MLX_SHIM_T2D(int64_t, int64);
MLX_SHIM_T2D(float16_t, float16);
MLX_SHIM_T2D(float, float32);
MLX_SHIM_T2D(double, float32);
MLX_SHIM_T2D(bfloat16_t, bfloat16);
#undef MLX_SHIM_T2D

}  // namespace core
}  // namespace mlx
