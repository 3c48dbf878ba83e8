// Stand-in for <mlx/primitives.h>: the Primitive base class MLXR's kernels subclass.
#pragma once
#include <stdexcept>
#include <utility>
#include <vector>

#include "array.h"
#include "device.h"
#include "stream.h"

namespace mlx {
namespace core {

class Primitive {
 public:
  explicit Primitive(Stream stream) : stream_(stream) {}
  virtual ~Primitive() = default;
  Primitive(const Primitive&) = delete;
  Primitive& operator=(const Primitive&) = delete;

  const Device& device() { return stream_.device; }
  const Stream& stream() { return stream_; }

  virtual void eval_cpu(const std::vector<array>& inputs, std::vector<array>& outputs) = 0;
  virtual void eval_gpu(const std::vector<array>& inputs, std::vector<array>& outputs) = 0;

  virtual std::vector<array> jvp(const std::vector<array>&, const std::vector<array>&, const std::vector<int>&) {
    throw std::invalid_argument("Primitive's jvp not implemented.");
  }
  virtual std::vector<array> vjp(const std::vector<array>&, const std::vector<array>&, const std::vector<int>&,
                                 const std::vector<array>&) {
    throw std::invalid_argument("Primitive's vjp not implemented.");
  }
  virtual std::pair<std::vector<array>, std::vector<int>> vmap(const std::vector<array>&, const std::vector<int>&) {
    throw std::invalid_argument("Primitive's vmap not implemented.");
  }
  virtual const char* name() const = 0;
  virtual bool is_equivalent(const Primitive&) const { return false; }
  virtual std::vector<Shape> output_shapes(const std::vector<array>&) {
    throw std::invalid_argument("Primitive's output_shapes not implemented.");
  }

 private:
  Stream stream_;
};

}  // namespace core
}  // namespace mlx
