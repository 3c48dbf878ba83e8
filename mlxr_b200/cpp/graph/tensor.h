// mlxr::graph::Tensor on the B200 path: the thin wrapper over mlx::core::array that the
// reference's graph layer passes around (core/graph/tensor.h:36-181).  Same class and free
// function names and argument order, reduced to what the layers on the quantized-linear path
// use (construction, shape access, reshape, from_data / zeros / ones); element-wise operators
// and matmul on Tensors are not on this path and are not provided.
#pragma once
#include <string>
#include <vector>

#include <mlx/mlx.h>

namespace mlxr {
namespace graph {

inline mlx::core::Shape to_shape(const std::vector<int>& vec) { return mlx::core::Shape(vec.begin(), vec.end()); }
inline std::vector<int> from_shape(const mlx::core::Shape& shape) { return std::vector<int>(shape.begin(), shape.end()); }

class Tensor {
 public:
  Tensor();                                                      // empty tensor (tensor.h:41)
  explicit Tensor(const mlx::core::array& array);                // wrap an array (tensor.h:47)
  Tensor(const std::vector<int>& shape, mlx::core::Dtype dtype);  // uninitialised (tensor.h:54)
  mlx::core::array& array();
  const mlx::core::array& array() const;
  std::vector<int> shape() const;
  mlx::core::Dtype dtype() const;
  int ndim() const;
  size_t size() const;
  bool empty() const;
  Tensor reshape(const std::vector<int>& new_shape) const;
  std::string to_string() const;
  void eval();

 private:
  mlx::core::array array_;
  bool empty_ = false;
};

Tensor zeros(const std::vector<int>& shape, mlx::core::Dtype dtype = mlx::core::float32);
Tensor ones(const std::vector<int>& shape, mlx::core::Dtype dtype = mlx::core::float32);
// `data` holds elements of `dtype` (tensor.h:163-164)
Tensor from_data(const void* data, const std::vector<int>& shape, mlx::core::Dtype dtype);

}  // namespace graph
}  // namespace mlxr
