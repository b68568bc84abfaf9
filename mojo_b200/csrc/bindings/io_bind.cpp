// Bindings of the checkpoint IO layer (b2/io.h) and the process context (b2/runtime.h).
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <stdexcept>

#include "b2/io.h"
#include "b2/runtime.h"

namespace py = pybind11;
using b2::io::SafetensorsFile;

namespace {

at::ScalarType scalar_type_of(const std::string& d) {
  if (d == "BF16") return at::kBFloat16;
  if (d == "F16") return at::kHalf;
  if (d == "F32") return at::kFloat;
  if (d == "F64") return at::kDouble;
  if (d == "I64") return at::kLong;
  if (d == "I32") return at::kInt;
  if (d == "I16") return at::kShort;
  if (d == "I8") return at::kChar;
  if (d == "U8") return at::kByte;
  if (d == "BOOL") return at::kBool;
  if (d == "F8_E4M3") return at::kFloat8_e4m3fn;
  if (d == "F8_E5M2") return at::kFloat8_e5m2;
  throw std::invalid_argument("mojo_b200: safetensors dtype '" + d + "' is not supported");
}

// Two pinned staging buffers per process for host -> device streaming; released when the context goes away.
struct Staging {
  static constexpr size_t kBytes = 32u << 20;
  void* buf[2];
  cudaEvent_t done[2];
  bool ok;
};
void staging_init(void* p) {
  auto* s = static_cast<Staging*>(p);
  s->ok = cudaHostAlloc(&s->buf[0], Staging::kBytes, cudaHostAllocDefault) == cudaSuccess &&
          cudaHostAlloc(&s->buf[1], Staging::kBytes, cudaHostAllocDefault) == cudaSuccess &&
          cudaEventCreateWithFlags(&s->done[0], cudaEventDisableTiming) == cudaSuccess &&
          cudaEventCreateWithFlags(&s->done[1], cudaEventDisableTiming) == cudaSuccess;
}
void staging_fini(void* p) {
  auto* s = static_cast<Staging*>(p);
  if (!s->ok) return;
  for (int i = 0; i < 2; ++i) {
    cudaFreeHost(s->buf[i]);
    cudaEventDestroy(s->done[i]);
  }
}

// mapped bytes -> device memory through the pinned pair: the pool fills one buffer while the copy engine drains the other
void copy_to_device(void* dst, const uint8_t* src, size_t n, cudaStream_t stream) {
  auto* st = static_cast<Staging*>(b2::rt::Context::instance().global("io.staging", sizeof(Staging), staging_init, staging_fini));
  if (st == nullptr || !st->ok) throw std::runtime_error("mojo_b200: cannot allocate pinned staging buffers");
  size_t off = 0;
  int turn = 0;
  bool used[2] = {false, false};
  while (off < n) {
    const size_t m = std::min(Staging::kBytes, n - off);
    if (used[turn]) cudaEventSynchronize(st->done[turn]);
    b2::io::parallel_copy(st->buf[turn], src + off, m);
    if (cudaMemcpyAsync(static_cast<uint8_t*>(dst) + off, st->buf[turn], m, cudaMemcpyHostToDevice, stream) != cudaSuccess)
      throw std::runtime_error("mojo_b200: host to device copy failed");
    cudaEventRecord(st->done[turn], stream);
    used[turn] = true;
    off += m;
    turn ^= 1;
  }
  for (int i = 0; i < 2; ++i)
    if (used[i]) cudaEventSynchronize(st->done[i]);   // the buffers are shared: leave them idle
}

}  // namespace

void bind_io(py::module_& m) {
  py::class_<SafetensorsFile, std::shared_ptr<SafetensorsFile>>(m, "SafetensorsFile")
      .def(py::init([](const std::string& path) { return std::make_shared<SafetensorsFile>(path); }))
      .def("keys", [](const SafetensorsFile& f) { return f.names(); })
      .def("has", &SafetensorsFile::has)
      .def("metadata", [](const SafetensorsFile& f) { return f.metadata(); })
      .def("info",
           [](const SafetensorsFile& f, const std::string& name) {
             if (!f.has(name)) throw py::key_error(name);
             const auto& t = f.info(name);
             return py::make_tuple(t.dtype, t.shape, t.nbytes());
           })
      .def("get",
           [](std::shared_ptr<SafetensorsFile> f, const std::string& name) {
             // A tensor over the mapping itself: no copy. The memory is read-only; callers convert, slice and move it.
             if (!f->has(name)) throw py::key_error(name);
             const auto& t = f->info(name);
             auto keep = f->file();
             return at::from_blob(const_cast<uint8_t*>(f->tensor_data(name)), t.shape, [keep](void*) {},
                                  at::TensorOptions().dtype(scalar_type_of(t.dtype)).device(at::kCPU));
           })
      .def("read_into",
           [](std::shared_ptr<SafetensorsFile> f, const std::string& name, at::Tensor& dst) {
             // Copy a whole tensor into `dst` (same dtype, element count and contiguous): host memory through the worker
             // pool, device memory through pinned staging on the current stream.
             if (!f->has(name)) throw py::key_error(name);
             const auto& t = f->info(name);
             if (!dst.is_contiguous() || dst.scalar_type() != scalar_type_of(t.dtype) ||
                 static_cast<size_t>(dst.numel()) * dst.element_size() != t.nbytes())
               throw std::invalid_argument("mojo_b200: read_into: destination must be contiguous with the tensor's dtype and size");
             const uint8_t* src = f->tensor_data(name);
             f->file()->will_need(static_cast<size_t>(src - f->file()->data()), t.nbytes());
             if (dst.is_cuda()) {
               c10::cuda::CUDAGuard g(dst.device());
               cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
               py::gil_scoped_release nogil;
               copy_to_device(dst.data_ptr(), src, t.nbytes(), stream);
             } else {
               py::gil_scoped_release nogil;
               b2::io::parallel_copy(dst.data_ptr(), src, t.nbytes());
             }
           });

  m.def("context_info", [] {
    auto& ctx = b2::rt::Context::instance();
    py::dict d;
    d["hardware_threads"] = ctx.hardware_threads();
    d["pool_threads"] = ctx.pool().size();
    d["globals"] = ctx.num_globals();
    d["failed_tasks"] = ctx.pool().failed_tasks();
    return d;
  });
  m.def("parallel_copy", [](at::Tensor& dst, const at::Tensor& src, int max_threads) {
    if (dst.is_cuda() || src.is_cuda() || !dst.is_contiguous() || !src.is_contiguous() || dst.nbytes() != src.nbytes())
      throw std::invalid_argument("mojo_b200: parallel_copy: contiguous host tensors of equal byte size");
    py::gil_scoped_release nogil;
    b2::io::parallel_copy(dst.data_ptr(), src.data_ptr(), src.nbytes(), max_threads);
  }, py::arg("dst"), py::arg("src"), py::arg("max_threads") = 0);
}
