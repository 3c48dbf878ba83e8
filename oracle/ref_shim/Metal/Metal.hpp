// Test-oracle stub of metal-cpp's Metal (see Foundation.hpp).
#pragma once
#include <Foundation/Foundation.hpp>
namespace MTL {
class Library {
 public:
  void release() {}
};
class ComputePipelineState {};
class Device {
 public:
  Library* newLibrary(NS::String*, NS::Error**) { return nullptr; }  // no Metal here
};
struct Size {
  Size(unsigned long w, unsigned long h, unsigned long d) : width(w), height(h), depth(d) {}
  unsigned long width, height, depth;
};
}  // namespace MTL
