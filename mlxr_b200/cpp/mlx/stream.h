// Stand-in for <mlx/stream.h>.  A gpu Stream maps to one cudaStream_t owned by the shim
// runtime (index 0 of a device = the CUDA legacy default stream).
#pragma once
#include "device.h"

namespace mlx {
namespace core {

struct Stream {
  int index;
  Device device;
  explicit Stream(int index, Device device) : index(index), device(device) {}
};
inline bool operator==(const Stream& a, const Stream& b) { return a.index == b.index && a.device == b.device; }
inline bool operator!=(const Stream& a, const Stream& b) { return !(a == b); }

Stream default_stream(Device d);
void set_default_stream(Stream s);
Stream new_stream(Device d);
inline Stream new_stream() { return new_stream(default_device()); }
// Block until everything queued on s has finished.
void synchronize(Stream s);
void synchronize();

// Shim extension: the native handle (cudaStream_t as void*) behind a gpu stream; nullptr
// for cpu streams and for index 0.
void* native_stream(const Stream& s);

}  // namespace core
}  // namespace mlx
