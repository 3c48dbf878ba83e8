// Stand-in for <mlx/utils.h>: StreamOrDevice and to_stream.
#pragma once
#include <variant>

#include "device.h"
#include "stream.h"

namespace mlx {
namespace core {

using StreamOrDevice = std::variant<std::monostate, Stream, Device>;

inline Stream to_stream(StreamOrDevice s) {
  if (std::holds_alternative<std::monostate>(s)) return default_stream(default_device());
  if (std::holds_alternative<Device>(s)) return default_stream(std::get<Device>(s));
  return std::get<Stream>(s);
}

}  // namespace core
}  // namespace mlx
