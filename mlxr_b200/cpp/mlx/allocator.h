// Stand-in for <mlx/allocator.h>.  Memory is "unified" as in MLX: in the product build an
// allocation is CUDA managed memory (valid on host and device); in a host-only build
// (MLX_SHIM_HOST_ONLY) it is plain heap memory.
#pragma once
#include <cstddef>

namespace mlx {
namespace core {
namespace allocator {

class Buffer {
 public:
  explicit Buffer(void* p = nullptr) : ptr_(p) {}
  void* raw_ptr() const { return ptr_; }
  void* ptr() const { return ptr_; }

 private:
  void* ptr_;
};

Buffer malloc(size_t size);  // throws std::runtime_error on failure
void free(Buffer buffer);

}  // namespace allocator
}  // namespace core
}  // namespace mlx
