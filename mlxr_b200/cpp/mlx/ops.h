// Stand-in for <mlx/ops.h>: the few array functions MLXR's primitives call around their
// kernels.  They run on the host over unified memory (tables, dtype casts, reshapes of
// evaluated arrays); none of them is on the hot path.
#pragma once
#include "array.h"
#include "utils.h"

namespace mlx {
namespace core {

array zeros(const Shape& shape, Dtype dtype, StreamOrDevice s = {});
array zeros_like(const array& a, StreamOrDevice s = {});
array ones(const Shape& shape, Dtype dtype, StreamOrDevice s = {});
array astype(array a, Dtype dtype, StreamOrDevice s = {});
array reshape(const array& a, Shape shape, StreamOrDevice s = {});
array contiguous(const array& a, bool allow_col_major = false, StreamOrDevice s = {});

}  // namespace core
}  // namespace mlx
