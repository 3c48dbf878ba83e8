// Stand-in for <mlx/device.h>.
#pragma once
namespace mlx {
namespace core {

struct Device {
  enum class DeviceType { cpu, gpu };
  static constexpr DeviceType cpu = DeviceType::cpu;
  static constexpr DeviceType gpu = DeviceType::gpu;
  Device(DeviceType type, int index = 0) : type(type), index(index) {}
  DeviceType type;
  int index;
};
inline bool operator==(const Device& a, const Device& b) { return a.type == b.type && a.index == b.index; }
inline bool operator!=(const Device& a, const Device& b) { return !(a == b); }

// The default device is the GPU (CUDA device `index`) in the product build and the CPU in
// a host-only build (MLX_SHIM_HOST_ONLY).
const Device& default_device();
void set_default_device(const Device& d);

}  // namespace core
}  // namespace mlx
