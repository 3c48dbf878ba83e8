// Test-oracle stub of metal-cpp's Foundation: just enough for MLXR's primitives to
// compile as host C++.  Nothing here can load a Metal library: newLibrary() reports failure.
#pragma once
namespace NS {
enum StringEncoding { UTF8StringEncoding = 4 };
class String {
 public:
  static String* string(const char* s, StringEncoding) { static String one; one.s_ = s; return &one; }
  const char* utf8String() const { return s_; }
 private:
  const char* s_ = "";
};
class Error {
 public:
  String* localizedDescription() { static String d; return &d; }
};
}  // namespace NS
