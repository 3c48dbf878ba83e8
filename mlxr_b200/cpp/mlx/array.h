// Stand-in for <mlx/array.h>: a reference-counted n-d array handle with lazy evaluation
// through a Primitive, reduced to what MLXR's kernel primitives and graph layers use.
//
// Differences from MLX, on purpose:
//  * array(Shape, Dtype) allocates an uninitialised array of that shape.  MLXR writes
//    `mlx::core::array({M, N}, float32)` meaning exactly that
//    (q_gemm_dequant_primitive.mm:314,382,510); in MLX proper that spelling builds a 1-D
//    array holding the two numbers.  The initializer-list-of-values constructor therefore
//    does not exist here.
//  * array::wrap() adopts caller-owned (device) memory without copying.
//  * arrays are always row-contiguous; there are no strided views.
#pragma once
#include <cstring>
#include <memory>
#include <stdexcept>
#include <type_traits>
#include <vector>

#include "allocator.h"
#include "dtype.h"
#include "stream.h"

namespace mlx {
namespace core {

using Shape = std::vector<int32_t>;
using ShapeElem = int32_t;
class Primitive;

class array {
 public:
  struct Flags {
    bool contiguous = true;
    bool row_contiguous = true;
    bool col_contiguous = false;
  };

  // scalar
  template <typename T, typename = std::enable_if_t<std::is_arithmetic_v<T>>>
  explicit array(T val, Dtype dtype = TypeToDtype<T>()) : array(Shape{}, dtype) {
    set_scalar(static_cast<double>(val));
  }
  // uninitialised [shape] (see header comment)
  array(Shape shape, Dtype dtype);
  // copy from host data of element type T, converted to dtype
  template <typename T>
  array(const T* data, Shape shape, Dtype dtype = TypeToDtype<T>()) : array(std::move(shape), dtype) {
    copy_from(data, TypeToDtype<T>());
  }
  // shim extension: adopt memory owned by the caller (device or managed); never freed here
  static array wrap(void* data, Shape shape, Dtype dtype);

  // lazy outputs of a primitive (evaluated by eval())
  static std::vector<array> make_arrays(std::vector<Shape> shapes, const std::vector<Dtype>& dtypes,
                                        const std::shared_ptr<Primitive>& primitive,
                                        const std::vector<array>& inputs);

  const Shape& shape() const { return d_->shape; }
  int32_t shape(int dim) const { return d_->shape.at(dim < 0 ? dim + (int)d_->shape.size() : dim); }
  size_t ndim() const { return d_->shape.size(); }
  size_t size() const { return d_->size; }
  size_t itemsize() const { return d_->dtype.size(); }
  size_t nbytes() const { return d_->size * d_->dtype.size(); }
  Dtype dtype() const { return d_->dtype; }
  Flags flags() const { return Flags{}; }

  bool is_available() const { return d_->data != nullptr; }
  bool has_primitive() const { return d_->primitive != nullptr; }
  Primitive& primitive() const { return *d_->primitive; }
  const std::vector<array>& inputs() const { return d_->inputs; }
  const std::vector<array>& siblings() const { return d_->siblings; }

  // Evaluate if needed (and wait for the stream when the data is about to be read on the
  // host through item()).
  void eval();

  template <typename T> T* data() { return static_cast<T*>(raw()); }
  template <typename T> const T* data() const { return static_cast<const T*>(raw()); }
  template <typename T> T item();

  void set_data(allocator::Buffer buffer);
  // replace this handle's contents by another array's (used by primitives that build
  // their output as a fresh array)
  void overwrite_descriptor(const array& other) { d_ = other.d_; }
  // shim internals
  int sibling_index_() const { return d_->sibling_index; }
  void keep_alive_(const array& owner) { d_->inputs.push_back(owner); }

  struct Data {
    Shape shape;
    Dtype dtype{float32};
    size_t size = 0;
    void* data = nullptr;
    bool owned = false;
    std::shared_ptr<Primitive> primitive;
    std::vector<array> inputs;
    std::vector<array> siblings;  // other outputs of the same primitive
    int sibling_index = 0;
    ~Data();
  };

 private:
  void* raw() const;
  void set_scalar(double v);
  void copy_from(const void* src, Dtype src_dtype);
  std::shared_ptr<Data> d_;
};

void eval(std::vector<array> outputs);
inline void eval(const array& a) { eval(std::vector<array>{a}); }

template <typename T>
T array::item() {
  if (size() != 1) throw std::invalid_argument("item can only be called on arrays of size 1.");
  eval();
  synchronize();
  return *data<T>();
}

}  // namespace core
}  // namespace mlx
