// Runtime of the MLX stand-in headers (mlx/*.h): devices, streams, unified memory, the
// array handle, lazy evaluation and a handful of host-side array functions.
//
// Product build: allocations are CUDA managed memory and a gpu Stream owns a
// cudaStream_t.  Host-only build (MLX_SHIM_HOST_ONLY, used to compile the reference's own
// CPU code for the test oracle): heap memory, no CUDA.
#include <cmath>
#include <cstdlib>
#include <mutex>
#include <string>

#include "mlx/mlx.h"

#ifndef MLX_SHIM_HOST_ONLY
#include <cuda_runtime.h>
#endif

namespace mlx {
namespace core {

// ---- devices and streams ---------------------------------------------------------------
namespace {
#ifdef MLX_SHIM_HOST_ONLY
Device g_default_device{Device::cpu, 0};
#else
Device g_default_device{Device::gpu, 0};
#endif
std::mutex g_mu;
struct StreamRec {
  Device device;
  void* native;
};
std::vector<StreamRec>& streams() {
  // index 0: default gpu stream (CUDA legacy default stream); index 1: default cpu stream
  static std::vector<StreamRec> v = {{Device(Device::gpu, 0), nullptr}, {Device(Device::cpu, 0), nullptr}};
  return v;
}
int g_default_gpu_stream = 0;
int g_default_cpu_stream = 1;
}  // namespace

const Device& default_device() { return g_default_device; }
void set_default_device(const Device& d) { g_default_device = d; }

Stream default_stream(Device d) {
  std::lock_guard<std::mutex> lk(g_mu);
  const int idx = d.type == Device::gpu ? g_default_gpu_stream : g_default_cpu_stream;
  return Stream(idx, streams()[idx].device);
}
void set_default_stream(Stream s) {
  std::lock_guard<std::mutex> lk(g_mu);
  (s.device.type == Device::gpu ? g_default_gpu_stream : g_default_cpu_stream) = s.index;
}
Stream new_stream(Device d) {
  std::lock_guard<std::mutex> lk(g_mu);
  void* native = nullptr;
#ifndef MLX_SHIM_HOST_ONLY
  if (d.type == Device::gpu) {
    cudaStream_t st;
    cudaSetDevice(d.index);
    if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess)
      throw std::runtime_error("new_stream: cudaStreamCreate failed");
    native = st;
  }
#endif
  streams().push_back({d, native});
  return Stream((int)streams().size() - 1, d);
}
void* native_stream(const Stream& s) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (s.index < 0 || s.index >= (int)streams().size()) throw std::invalid_argument("unknown stream");
  return streams()[s.index].native;
}
void synchronize(Stream s) {
#ifndef MLX_SHIM_HOST_ONLY
  if (s.device.type == Device::gpu) {
    if (cudaStreamSynchronize((cudaStream_t)native_stream(s)) != cudaSuccess)
      throw std::runtime_error(std::string("synchronize: ") + cudaGetErrorString(cudaGetLastError()));
  }
#else
  (void)s;
#endif
}
void synchronize() { synchronize(default_stream(default_device())); }

// ---- unified memory ----------------------------------------------------------------------
namespace allocator {
Buffer malloc(size_t size) {
  if (size == 0) size = 1;
  void* p = nullptr;
#ifdef MLX_SHIM_HOST_ONLY
  p = std::malloc(size);
#else
  if (cudaMallocManaged(&p, size) != cudaSuccess) p = nullptr;
#endif
  if (!p) throw std::runtime_error("[malloc] Unable to allocate " + std::to_string(size) + " bytes.");
  return Buffer(p);
}
void free(Buffer b) {
  if (!b.raw_ptr()) return;
#ifdef MLX_SHIM_HOST_ONLY
  std::free(b.raw_ptr());
#else
  cudaFree(b.raw_ptr());
#endif
}
}  // namespace allocator

// ---- array -------------------------------------------------------------------------------
array::Data::~Data() {
  if (owned && data) allocator::free(allocator::Buffer(data));
}

static size_t shape_size(const Shape& s) {
  size_t n = 1;
  for (auto d : s) {
    if (d < 0) throw std::invalid_argument("negative dimension in shape");
    n *= (size_t)d;
  }
  return n;
}

array::array(Shape shape, Dtype dtype) : d_(std::make_shared<Data>()) {
  d_->size = shape_size(shape);
  d_->shape = std::move(shape);
  d_->dtype = dtype;
  d_->data = allocator::malloc(d_->size * dtype.size()).raw_ptr();
  d_->owned = true;
}

array array::wrap(void* data, Shape shape, Dtype dtype) {
  array a(Shape{0}, dtype);  // tiny placeholder allocation, replaced below
  auto d = std::make_shared<Data>();
  d->size = shape_size(shape);
  d->shape = std::move(shape);
  d->dtype = dtype;
  d->data = data;
  d->owned = false;
  a.d_ = d;
  return a;
}

std::vector<array> array::make_arrays(std::vector<Shape> shapes, const std::vector<Dtype>& dtypes,
                                      const std::shared_ptr<Primitive>& primitive,
                                      const std::vector<array>& inputs) {
  std::vector<array> outs;
  for (size_t i = 0; i < shapes.size(); i++) {
    array a = wrap(nullptr, shapes[i], dtypes[i]);
    a.d_->primitive = primitive;
    a.d_->inputs = inputs;
    a.d_->sibling_index = (int)i;
    outs.push_back(a);
  }
  for (size_t i = 0; i < outs.size(); i++)
    for (size_t j = 0; j < outs.size(); j++)
      if (i != j) outs[i].d_->siblings.push_back(outs[j]);
  return outs;
}

void array::set_data(allocator::Buffer buffer) {
  if (d_->owned && d_->data) allocator::free(allocator::Buffer(d_->data));
  d_->data = buffer.raw_ptr();
  d_->owned = true;
}

void* array::raw() const {
  if (!d_->data && d_->size != 0)
    throw std::runtime_error("array data accessed before evaluation (call mlx::core::eval first)");
  return d_->data;
}

void array::eval() { mlx::core::eval(std::vector<array>{*this}); }

static void eval_one(array& a) {
  if (a.is_available() || !a.has_primitive()) return;
  for (auto in : a.inputs()) eval_one(in);
  // outputs in primitive order: siblings() lists the other outputs in creation order
  std::vector<array> outs;
  const size_t n = a.siblings().size() + 1, self = (size_t)a.sibling_index_();
  size_t k = 0;
  for (size_t i = 0; i < n; i++) outs.push_back(i == self ? a : a.siblings()[k++]);
  Primitive& p = a.primitive();
  if (p.stream().device.type == Device::gpu) p.eval_gpu(a.inputs(), outs);
  else p.eval_cpu(a.inputs(), outs);
}

void eval(std::vector<array> outputs) {
  for (auto& a : outputs) eval_one(a);
}

static double load_as_double(const void* p, size_t i, Dtype dt) {
  switch (dt.val()) {
    case Dtype::Val::bool_: return ((const bool*)p)[i];
    case Dtype::Val::uint8: return ((const uint8_t*)p)[i];
    case Dtype::Val::uint16: return ((const uint16_t*)p)[i];
    case Dtype::Val::uint32: return ((const uint32_t*)p)[i];
    case Dtype::Val::uint64: return (double)((const uint64_t*)p)[i];
    case Dtype::Val::int8: return ((const int8_t*)p)[i];
    case Dtype::Val::int16: return ((const int16_t*)p)[i];
    case Dtype::Val::int32: return ((const int32_t*)p)[i];
    case Dtype::Val::int64: return (double)((const int64_t*)p)[i];
    case Dtype::Val::float16: return (float)((const float16_t*)p)[i];
    case Dtype::Val::float32: return ((const float*)p)[i];
    case Dtype::Val::float64: return ((const double*)p)[i];
    case Dtype::Val::bfloat16: return (float)((const bfloat16_t*)p)[i];
  }
  return 0;
}
static void store_from_double(void* p, size_t i, Dtype dt, double v) {
  switch (dt.val()) {
    case Dtype::Val::bool_: ((bool*)p)[i] = v != 0; break;
    case Dtype::Val::uint8: ((uint8_t*)p)[i] = (uint8_t)v; break;
    case Dtype::Val::uint16: ((uint16_t*)p)[i] = (uint16_t)v; break;
    case Dtype::Val::uint32: ((uint32_t*)p)[i] = (uint32_t)v; break;
    case Dtype::Val::uint64: ((uint64_t*)p)[i] = (uint64_t)v; break;
    case Dtype::Val::int8: ((int8_t*)p)[i] = (int8_t)v; break;
    case Dtype::Val::int16: ((int16_t*)p)[i] = (int16_t)v; break;
    case Dtype::Val::int32: ((int32_t*)p)[i] = (int32_t)v; break;
    case Dtype::Val::int64: ((int64_t*)p)[i] = (int64_t)v; break;
    case Dtype::Val::float16: ((float16_t*)p)[i] = float16_t((float)v); break;
    case Dtype::Val::float32: ((float*)p)[i] = (float)v; break;
    case Dtype::Val::float64: ((double*)p)[i] = v; break;
    case Dtype::Val::bfloat16: ((bfloat16_t*)p)[i] = bfloat16_t((float)v); break;
  }
}

void array::set_scalar(double v) { store_from_double(d_->data, 0, d_->dtype, v); }

void array::copy_from(const void* src, Dtype src_dtype) {
  if (src_dtype == d_->dtype) {
    std::memcpy(d_->data, src, nbytes());
    return;
  }
  for (size_t i = 0; i < d_->size; i++) store_from_double(d_->data, i, d_->dtype, load_as_double(src, i, src_dtype));
}

// ---- host-side array functions -----------------------------------------------------------
array zeros(const Shape& shape, Dtype dtype, StreamOrDevice) {
  array a(shape, dtype);
  std::memset(a.data<void>(), 0, a.nbytes());
  return a;
}
array zeros_like(const array& a, StreamOrDevice s) { return zeros(a.shape(), a.dtype(), s); }
array ones(const Shape& shape, Dtype dtype, StreamOrDevice) {
  array a(shape, dtype);
  for (size_t i = 0; i < a.size(); i++) store_from_double(a.data<void>(), i, dtype, 1.0);
  return a;
}
array astype(array a, Dtype dtype, StreamOrDevice) {
  a.eval();
  if (a.dtype() == dtype) return a;
  synchronize();
  array out(a.shape(), dtype);
  // float32 -> float16/bfloat16 is one rounding to nearest even (float16_t / bfloat16_t)
  for (size_t i = 0; i < a.size(); i++)
    store_from_double(out.data<void>(), i, dtype, load_as_double(a.data<void>(), i, a.dtype()));
  return out;
}
array reshape(const array& a, Shape shape, StreamOrDevice) {
  size_t known = 1;
  int infer = -1;
  for (size_t i = 0; i < shape.size(); i++) {
    if (shape[i] == -1) { if (infer >= 0) throw std::invalid_argument("[reshape] only one dimension can be inferred"); infer = (int)i; }
    else known *= (size_t)shape[i];
  }
  if (infer >= 0) shape[infer] = known ? (int32_t)(a.size() / known) : 0;
  if (shape_size(shape) != a.size()) throw std::invalid_argument("[reshape] Cannot reshape array into the requested shape.");
  array src = a;
  src.eval();
  // arrays are always row-contiguous here, so a reshape is a view of the same memory
  array out = array::wrap(src.size() ? src.data<void>() : nullptr, shape, a.dtype());
  out.keep_alive_(src);
  return out;
}
array contiguous(const array& a, bool, StreamOrDevice) { return a; }

}  // namespace core
}  // namespace mlx
