// Test-oracle stub of MLX's Metal backend device: compiles eval_gpu bodies, runs nothing.
#pragma once
#include <Metal/Metal.hpp>
#include <mlx/device.h>
#include <cstddef>
namespace mlx { namespace core { namespace metal {
class CommandEncoder {
 public:
  void set_compute_pipeline_state(MTL::ComputePipelineState*) {}
  void set_bytes(const void*, size_t, int) {}
  void set_threadgroup_memory_length(size_t, int) {}
  void dispatch_threadgroups(MTL::Size, MTL::Size) {}
};
class Device {
 public:
  MTL::Device* mtl_device() { static MTL::Device d; return &d; }
  MTL::ComputePipelineState* get_kernel(const char*, MTL::Library*) { return nullptr; }
  template <typename S> MTL::ComputePipelineState* get_kernel(const S&, MTL::Library*) { return nullptr; }
  CommandEncoder& get_command_encoder(int) { static CommandEncoder e; return e; }
};
inline Device& device(mlx::core::Device) { static Device d; return d; }
}}}  // namespace mlx::core::metal
