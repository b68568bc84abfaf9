// Bindings of the standalone symmetric-memory collectives (csrc/kernels/symm_coll.cu).
#include <torch/extension.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/cuda/CUDAGuard.h>
#include "b2/api.h"
#include "b2/launch.h"
#include "b2/coll.h"
#include "b2/symm_heap.h"
namespace py = pybind11;

namespace {
cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }
void check(int rc, const char* what) {
  if (rc == 0) return;
  if (b2::is_cuda_rc(rc)) {
    // the CUDA runtime refused the launch or its set-up: say which error, not a generic "bad argument"
    const cudaError_t e = b2::cuda_error_of(rc);
    throw std::runtime_error(std::string("mojo_b200: ") + what + " failed: CUDA error " + std::to_string(static_cast<int>(e)) + " (" +
                             cudaGetErrorName(e) + ": " + cudaGetErrorString(e) + ")");
  }
  throw std::runtime_error(std::string("mojo_b200: ") + what + " rejected its arguments: " + b2::status_code_name(-rc));
}
void need(bool cond, const char* msg) {
  if (!cond) throw std::invalid_argument(std::string("mojo_b200: ") + msg);
}
b2::Status* status_ptr(const c10::optional<at::Tensor>& s) {
  return s.has_value() ? reinterpret_cast<b2::Status*>(s->data_ptr()) : nullptr;
}
B2TpRegion make_region(int rank, const std::vector<int64_t>& ptrs) {
  need(!ptrs.empty() && ptrs.size() <= 8 && rank >= 0 && rank < static_cast<int>(ptrs.size()), "region: 1..8 peer pointers and a valid rank");
  B2TpRegion r{};
  r.rank = rank;
  r.tp = static_cast<int>(ptrs.size());
  for (size_t i = 0; i < ptrs.size(); ++i) r.peer[i] = reinterpret_cast<void*>(ptrs[i]);
  return r;
}
}  // namespace

void bind_coll(py::module_& m) {
  // VMM-based symmetric heap segment (csrc/runtime/symm_heap.cpp). Errors surface as RuntimeError with the driver's code.
  py::class_<b2::symm::HeapSegment>(m, "SymmHeapSegment")
      .def(py::init<>())
      .def("create",
           [](b2::symm::HeapSegment& h, int device, int rank, int world, size_t bytes, bool multicast) {
             const std::string e = h.create(device, rank, world, bytes, multicast);
             if (!e.empty()) throw std::runtime_error(e);
           })
      .def("export_fd",
           [](b2::symm::HeapSegment& h) {
             std::string e;
             const int fd = h.export_fd(&e);
             if (fd < 0) throw std::runtime_error(e);
             return fd;
           })
      .def("map_peer",
           [](b2::symm::HeapSegment& h, int peer, int fd) {
             const std::string e = h.map_peer(peer, fd);
             if (!e.empty()) throw std::runtime_error(e);
           })
      .def("multicast_supported", &b2::symm::HeapSegment::multicast_supported)
      .def("mc_create",
           [](b2::symm::HeapSegment& h) {
             std::string e;
             const int fd = h.mc_create(&e);
             if (fd < 0) throw std::runtime_error(e);
             return fd;
           })
      .def("mc_import",
           [](b2::symm::HeapSegment& h, int fd) {
             const std::string e = h.mc_import(fd);
             if (!e.empty()) throw std::runtime_error(e);
           })
      .def("mc_add_device",
           [](b2::symm::HeapSegment& h) {
             const std::string e = h.mc_add_device();
             if (!e.empty()) throw std::runtime_error(e);
           })
      .def("mc_bind_and_map",
           [](b2::symm::HeapSegment& h) {
             const std::string e = h.mc_bind_and_map();
             if (!e.empty()) throw std::runtime_error(e);
           })
      .def("bytes", &b2::symm::HeapSegment::bytes)
      .def("ptr", &b2::symm::HeapSegment::ptr)
      .def("mc_ptr", &b2::symm::HeapSegment::mc_ptr)
      .def("close", &b2::symm::HeapSegment::close);

  py::class_<B2CollLayout>(m, "CollLayout")
      .def(py::init([]() { return B2CollLayout{}; }))
      .def_readwrite("off_buf", &B2CollLayout::off_buf)
      .def_readwrite("buf_half_bytes", &B2CollLayout::buf_half_bytes)
      .def_readwrite("off_out", &B2CollLayout::off_out)
      .def_readwrite("out_half_bytes", &B2CollLayout::out_half_bytes)
      .def_readwrite("off_flags_a", &B2CollLayout::off_flags_a)
      .def_readwrite("off_flags_b", &B2CollLayout::off_flags_b)
      .def_readwrite("off_counts", &B2CollLayout::off_counts)
      .def_readwrite("off_done", &B2CollLayout::off_done)
      .def_readwrite("off_epoch", &B2CollLayout::off_epoch)
      .def_readwrite("total_bytes", &B2CollLayout::total_bytes);

  m.def("coll_all_reduce",
        [](int rank, const std::vector<int64_t>& peers, const B2CollLayout& lay, int64_t mc_base, c10::optional<at::Tensor> out, int64_t n,
           int algo, int slot, uint64_t timeout_ns, c10::optional<at::Tensor> status) {
          const B2TpRegion reg = make_region(rank, peers);
          if (algo == 0) need(out.has_value() && out->is_cuda() && out->scalar_type() == at::kBFloat16 && out->is_contiguous() && out->numel() >= n, "coll_all_reduce: out bf16, contiguous, n elements");
          check(b2_coll_all_reduce_bf16(&reg, &lay, reinterpret_cast<void*>(mc_base), out.has_value() ? out->data_ptr() : nullptr, n, algo, slot,
                                        timeout_ns, status_ptr(status), cur_stream()),
                "coll_all_reduce");
        });
  m.def("coll_all_reduce_rmsnorm",
        [](int rank, const std::vector<int64_t>& peers, const B2CollLayout& lay, c10::optional<at::Tensor> residual, const at::Tensor& weight,
           at::Tensor& out, double eps, int slot, uint64_t timeout_ns, c10::optional<at::Tensor> status) {
          const B2TpRegion reg = make_region(rank, peers);
          need(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.is_contiguous() && out.dim() == 2, "coll_all_reduce_rmsnorm: out bf16 [rows, hidden]");
          need(weight.scalar_type() == at::kBFloat16 && weight.is_contiguous() && weight.numel() == out.size(1), "coll_all_reduce_rmsnorm: weight bf16 [hidden]");
          if (residual.has_value())
            need(residual->scalar_type() == at::kBFloat16 && residual->is_contiguous() && residual->sizes() == out.sizes(), "coll_all_reduce_rmsnorm: residual bf16 [rows, hidden]");
          c10::cuda::CUDAGuard g(out.device());
          check(b2_coll_all_reduce_rmsnorm_bf16(&reg, &lay, residual.has_value() ? residual->data_ptr() : nullptr, weight.data_ptr(), out.data_ptr(),
                                                static_cast<int>(out.size(0)), static_cast<int>(out.size(1)), static_cast<float>(eps), slot,
                                                timeout_ns, status_ptr(status), cur_stream()),
                "coll_all_reduce_rmsnorm");
        });
  m.def("coll_all_reduce_rmsnorm_nvls",
        [](int rank, const std::vector<int64_t>& peers, const B2CollLayout& lay, int64_t mc_base, c10::optional<at::Tensor> residual,
           const at::Tensor& weight, int rows, double eps, int slot, uint64_t timeout_ns, c10::optional<at::Tensor> status) {
          const B2TpRegion reg = make_region(rank, peers);
          need(weight.is_cuda() && weight.scalar_type() == at::kBFloat16 && weight.is_contiguous(), "coll_all_reduce_rmsnorm_nvls: weight bf16 [hidden]");
          const int hidden = static_cast<int>(weight.numel());
          if (residual.has_value())
            need(residual->scalar_type() == at::kBFloat16 && residual->is_contiguous() && residual->numel() == static_cast<int64_t>(rows) * hidden,
                 "coll_all_reduce_rmsnorm_nvls: residual bf16 [rows, hidden]");
          c10::cuda::CUDAGuard g(weight.device());
          check(b2_coll_all_reduce_rmsnorm_nvls_bf16(&reg, &lay, reinterpret_cast<void*>(mc_base), residual.has_value() ? residual->data_ptr() : nullptr,
                                                     weight.data_ptr(), rows, hidden, static_cast<float>(eps), slot, timeout_ns, status_ptr(status),
                                                     cur_stream()),
                "coll_all_reduce_rmsnorm_nvls");
        });
  m.def("coll_p2p_probe",
        [](int rank, const std::vector<int64_t>& peers, const B2CollLayout& lay, int64_t bytes, int n_peers, uint32_t senders, bool pull, int ctas,
           int slot, uint64_t timeout_ns, c10::optional<at::Tensor> status) {
          const B2TpRegion reg = make_region(rank, peers);
          check(b2_coll_p2p_probe(&reg, &lay, bytes, n_peers, senders, pull ? 1 : 0, ctas, slot, timeout_ns, status_ptr(status), cur_stream()),
                "coll_p2p_probe");
        });
  m.def("coll_reduce_scatter",
        [](int rank, const std::vector<int64_t>& peers, const B2CollLayout& lay, at::Tensor& out, int64_t n, int slot, uint64_t timeout_ns,
           c10::optional<at::Tensor> status) {
          const B2TpRegion reg = make_region(rank, peers);
          need(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.is_contiguous() && out.numel() * reg.tp >= n, "coll_reduce_scatter: out bf16, contiguous, n / tp elements");
          check(b2_coll_reduce_scatter_bf16(&reg, &lay, out.data_ptr(), n, slot, timeout_ns, status_ptr(status), cur_stream()), "coll_reduce_scatter");
        });
  m.def("coll_all_gather",
        [](int rank, const std::vector<int64_t>& peers, const B2CollLayout& lay, const at::Tensor& in, int slot, uint64_t timeout_ns,
           c10::optional<at::Tensor> status) {
          const B2TpRegion reg = make_region(rank, peers);
          need(in.is_cuda() && in.is_contiguous(), "coll_all_gather: contiguous CUDA input");
          check(b2_coll_all_gather(&reg, &lay, in.data_ptr(), static_cast<int64_t>(in.numel()) * in.element_size(), slot, timeout_ns,
                                   status_ptr(status), cur_stream()),
                "coll_all_gather");
        });
  m.def("coll_all_to_all",
        [](int rank, const std::vector<int64_t>& peers, const B2CollLayout& lay, const at::Tensor& in, const std::vector<int>& send_counts,
           int slot, uint64_t timeout_ns, c10::optional<at::Tensor> status) {
          const B2TpRegion reg = make_region(rank, peers);
          need(in.is_cuda() && in.is_contiguous() && in.dim() == 3 && in.size(0) == reg.tp && static_cast<int>(send_counts.size()) == reg.tp,
               "coll_all_to_all: in [tp, max_rows, row], one count per peer");
          check(b2_coll_all_to_all(&reg, &lay, in.data_ptr(), send_counts.data(), static_cast<int>(in.size(1)),
                                   static_cast<int64_t>(in.size(2)) * in.element_size(), slot, timeout_ns, status_ptr(status), cur_stream()),
                "coll_all_to_all");
        });
  m.def("coll_vocab_argmax",
        [](int rank, const std::vector<int64_t>& peers, const B2CollLayout& lay, const at::Tensor& logits, const at::Tensor& local_idx,
           at::Tensor& tokens, int v_stride, int slot, uint64_t timeout_ns, c10::optional<at::Tensor> status) {
          const B2TpRegion reg = make_region(rank, peers);
          need(logits.is_cuda() && logits.scalar_type() == at::kBFloat16 && logits.dim() == 2 && logits.stride(1) == 1, "coll_vocab_argmax: logits bf16 [S, V/tp]");
          const int S = static_cast<int>(logits.size(0));
          need(local_idx.scalar_type() == at::kLong && local_idx.is_contiguous() && local_idx.numel() == S && tokens.scalar_type() == at::kLong &&
                   tokens.is_contiguous() && tokens.numel() == S,
               "coll_vocab_argmax: int64 [S] indices and tokens");
          c10::cuda::CUDAGuard g(logits.device());
          check(b2_coll_vocab_argmax(&reg, &lay, logits.data_ptr(), logits.stride(0), local_idx.data_ptr<int64_t>(), tokens.data_ptr<int64_t>(), S,
                                     static_cast<int>(logits.size(1)), v_stride, slot, timeout_ns, status_ptr(status), cur_stream()),
                "coll_vocab_argmax");
        });
}
