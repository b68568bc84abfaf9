// Bindings of the second kernel group: fused tensor-parallel ops over symmetric memory (more groups register
// themselves below as they are added).
#include <torch/extension.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/cuda/CUDAGuard.h>
#include "b2/api.h"
#include "b2/launch.h"
#include "b2/tp.h"
#include "b2/ep.h"
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
  need(!ptrs.empty() && ptrs.size() <= 8 && rank >= 0 && rank < static_cast<int>(ptrs.size()), "tp region: 1..8 peer pointers and a valid rank");
  B2TpRegion r{};
  r.rank = rank;
  r.tp = static_cast<int>(ptrs.size());
  for (size_t i = 0; i < ptrs.size(); ++i) r.peer[i] = reinterpret_cast<void*>(ptrs[i]);
  return r;
}
bool is_bf16_2d(const at::Tensor& t) { return t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.stride(1) == 1; }
}  // namespace

void bind_ops_extra(py::module_& m) {
  py::class_<B2TpLayout>(m, "TpLayout")
      .def(py::init([]() { return B2TpLayout{}; }))
      .def_readwrite("off_staging", &B2TpLayout::off_staging)
      .def_readwrite("staging_half_bytes", &B2TpLayout::staging_half_bytes)
      .def_readwrite("off_yall", &B2TpLayout::off_yall)
      .def_readwrite("yall_half_bytes", &B2TpLayout::yall_half_bytes)
      .def_readwrite("off_xall", &B2TpLayout::off_xall)
      .def_readwrite("xall_half_bytes", &B2TpLayout::xall_half_bytes)
      .def_readwrite("off_rs_flags", &B2TpLayout::off_rs_flags)
      .def_readwrite("rs_flags_bytes", &B2TpLayout::rs_flags_bytes)
      .def_readwrite("off_ag_flags", &B2TpLayout::off_ag_flags)
      .def_readwrite("ag_flags_bytes", &B2TpLayout::ag_flags_bytes)
      .def_readwrite("off_res_flags", &B2TpLayout::off_res_flags)
      .def_readwrite("off_done", &B2TpLayout::off_done)
      .def_readwrite("off_barrier", &B2TpLayout::off_barrier)
      .def_readwrite("off_epoch_rs", &B2TpLayout::off_epoch_rs)
      .def_readwrite("off_epoch_ag", &B2TpLayout::off_epoch_ag)
      .def_readwrite("off_epoch_bar", &B2TpLayout::off_epoch_bar)
      .def_readwrite("total_bytes", &B2TpLayout::total_bytes);

  m.def("tp_gemm_rs",
        [](const at::Tensor& x, const at::Tensor& w, int rank, const std::vector<int64_t>& peers, const B2TpLayout& lay,
           c10::optional<at::Tensor> out, c10::optional<at::Tensor> residual, int mode, int slot, uint64_t timeout_ns,
           int config, c10::optional<at::Tensor> status, int64_t mc_base) {
          need(is_bf16_2d(x) && is_bf16_2d(w) && x.size(1) == w.size(1), "tp_gemm_rs: x [M, K/tp], w [N, K/tp] bf16");
          const int M = static_cast<int>(x.size(0)), K = static_cast<int>(x.size(1)), N = static_cast<int>(w.size(0));
          B2TpRegion reg = make_region(rank, peers);
          reg.mc_base = reinterpret_cast<void*>(mc_base);   // multicast mapping of the region: the reduction runs in the switch
          if (mode == 0) need(out.has_value() && is_bf16_2d(*out) && out->is_contiguous() && out->size(0) * reg.tp == M && out->size(1) == N, "tp_gemm_rs: out must be contiguous [M/tp, N]");
          if (residual.has_value()) need(is_bf16_2d(*residual) && residual->is_contiguous() && residual->size(1) == N, "tp_gemm_rs: residual must be contiguous [rows, N]");
          c10::cuda::CUDAGuard g(x.device());
          check(b2_tp_gemm_rs_bf16(x.data_ptr(), w.data_ptr(), &reg, &lay, out.has_value() ? out->data_ptr() : nullptr,
                                   residual.has_value() ? residual->data_ptr() : nullptr, M, N, K, x.stride(0), w.stride(0), mode,
                                   slot, timeout_ns, config, status_ptr(status), cur_stream()),
                "tp_gemm_rs");
        },
        py::arg("x"), py::arg("w"), py::arg("rank"), py::arg("peers"), py::arg("layout"), py::arg("out"), py::arg("residual"),
        py::arg("mode"), py::arg("slot"), py::arg("timeout_ns"), py::arg("config") = 0, py::arg("status") = py::none(), py::arg("mc_base") = 0);

  m.def("tp_gemm_rs_fp8",
        [](const at::Tensor& xq, const at::Tensor& xs, const at::Tensor& wq, const at::Tensor& ws, int rank,
           const std::vector<int64_t>& peers, const B2TpLayout& lay, c10::optional<at::Tensor> out,
           c10::optional<at::Tensor> residual, int mode, int slot, uint64_t timeout_ns, c10::optional<at::Tensor> status) {
          need(xq.is_cuda() && xq.element_size() == 1 && wq.element_size() == 1 && xq.dim() == 2 && wq.dim() == 2 && xq.is_contiguous() && wq.is_contiguous(),
               "tp_gemm_rs_fp8: xq [M, K/tp], wq [N, K/tp] contiguous 8-bit");
          const int M = static_cast<int>(xq.size(0)), K = static_cast<int>(xq.size(1)), N = static_cast<int>(wq.size(0));
          need(wq.size(1) == K && K % 128 == 0, "tp_gemm_rs_fp8: K must match and be a multiple of 128");
          need(xs.scalar_type() == at::kFloat && xs.is_contiguous() && xs.numel() == static_cast<int64_t>(M) * (K / 128), "tp_gemm_rs_fp8: xs f32 [M, K/128]");
          need(ws.scalar_type() == at::kFloat && ws.is_contiguous() && ws.numel() == static_cast<int64_t>((N + 127) / 128) * (K / 128), "tp_gemm_rs_fp8: ws f32 [ceil(N/128), K/128]");
          const B2TpRegion reg = make_region(rank, peers);
          if (mode == 0) need(out.has_value() && is_bf16_2d(*out) && out->is_contiguous() && out->size(0) * reg.tp == M && out->size(1) == N, "tp_gemm_rs_fp8: out must be contiguous [M/tp, N]");
          if (residual.has_value()) need(is_bf16_2d(*residual) && residual->is_contiguous() && residual->size(1) == N, "tp_gemm_rs_fp8: residual must be contiguous [rows, N]");
          c10::cuda::CUDAGuard g(xq.device());
          check(b2_tp_gemm_rs_fp8(xq.data_ptr(), xs.data_ptr<float>(), wq.data_ptr(), ws.data_ptr<float>(), &reg, &lay,
                                  out.has_value() ? out->data_ptr() : nullptr, residual.has_value() ? residual->data_ptr() : nullptr, M, N,
                                  K, mode, slot, timeout_ns, status_ptr(status), cur_stream()),
                "tp_gemm_rs_fp8");
        },
        py::arg("xq"), py::arg("xs"), py::arg("wq"), py::arg("ws"), py::arg("rank"), py::arg("peers"), py::arg("layout"), py::arg("out"),
        py::arg("residual"), py::arg("mode"), py::arg("slot"), py::arg("timeout_ns"), py::arg("status") = py::none());

  m.def("tp_ag_gemm",
        [](const at::Tensor& w, int rank, const std::vector<int64_t>& peers, const B2TpLayout& lay, at::Tensor& y, int M,
           int slot, uint64_t timeout_ns, int n_comm, int config, c10::optional<at::Tensor> status) {
          need(is_bf16_2d(w) && is_bf16_2d(y) && y.size(0) == M && y.size(1) == w.size(0), "tp_ag_gemm: w [N/tp, K], y [M, N/tp] bf16");
          const B2TpRegion reg = make_region(rank, peers);
          c10::cuda::CUDAGuard g(w.device());
          check(b2_tp_ag_gemm_bf16(w.data_ptr(), &reg, &lay, y.data_ptr(), M, static_cast<int>(w.size(0)), static_cast<int>(w.size(1)),
                                   w.stride(0), y.stride(0), slot, timeout_ns, n_comm, config, status_ptr(status), cur_stream()),
                "tp_ag_gemm");
        },
        py::arg("w"), py::arg("rank"), py::arg("peers"), py::arg("layout"), py::arg("y"), py::arg("M"), py::arg("slot"),
        py::arg("timeout_ns"), py::arg("n_comm") = 0, py::arg("config") = 0, py::arg("status") = py::none());

  m.def("tp_ag_gemm_fp8",
        [](const at::Tensor& wq, const at::Tensor& ws, int rank, const std::vector<int64_t>& peers, const B2TpLayout& lay, at::Tensor& y,
           int M, int slot, uint64_t timeout_ns, int n_comm, c10::optional<at::Tensor> status) {
          need(wq.is_cuda() && wq.element_size() == 1 && wq.dim() == 2 && wq.is_contiguous(), "tp_ag_gemm_fp8: wq [N/tp, K] contiguous 8-bit");
          const int N = static_cast<int>(wq.size(0)), K = static_cast<int>(wq.size(1));
          need(ws.scalar_type() == at::kFloat && ws.is_contiguous() && ws.numel() == static_cast<int64_t>((N + 127) / 128) * (K / 128), "tp_ag_gemm_fp8: ws f32 [ceil(N/128), K/128]");
          need(is_bf16_2d(y) && y.size(0) == M && y.size(1) == N, "tp_ag_gemm_fp8: y bf16 [M, N/tp]");
          const B2TpRegion reg = make_region(rank, peers);
          c10::cuda::CUDAGuard g(wq.device());
          check(b2_tp_ag_gemm_fp8(wq.data_ptr(), ws.data_ptr<float>(), &reg, &lay, y.data_ptr(), M, N, K, y.stride(0), slot, timeout_ns, n_comm,
                                  status_ptr(status), cur_stream()),
                "tp_ag_gemm_fp8");
        },
        py::arg("wq"), py::arg("ws"), py::arg("rank"), py::arg("peers"), py::arg("layout"), py::arg("y"), py::arg("M"), py::arg("slot"),
        py::arg("timeout_ns"), py::arg("n_comm") = 0, py::arg("status") = py::none());

  m.def("tp_all_gather",
        [](int rank, const std::vector<int64_t>& peers, const B2TpLayout& lay, int M, int K, int slot, uint64_t timeout_ns,
           c10::optional<at::Tensor> status) {
          const B2TpRegion reg = make_region(rank, peers);
          check(b2_tp_all_gather(&reg, &lay, M, K, slot, timeout_ns, status_ptr(status), cur_stream()), "tp_all_gather");
        });

  m.def("symm_barrier",
        [](int rank, const std::vector<int64_t>& peers, const B2TpLayout& lay, uint64_t timeout_ns,
           c10::optional<at::Tensor> status) {
          const B2TpRegion reg = make_region(rank, peers);
          check(b2_symm_barrier(&reg, &lay, timeout_ns, status_ptr(status), cur_stream()), "symm_barrier");
        });

  m.def("gemm_fp8",
        [](const at::Tensor& xq, const at::Tensor& xs, const at::Tensor& wq, const at::Tensor& ws, at::Tensor& y, int config,
           c10::optional<at::Tensor> status, c10::optional<at::Tensor> workspace) {
          need(xq.is_cuda() && xq.element_size() == 1 && wq.element_size() == 1 && xq.dim() == 2 && wq.dim() == 2 && xq.is_contiguous() && wq.is_contiguous(),
               "gemm_fp8: xq [M, K], wq [N, K] contiguous 8-bit");
          const int M = static_cast<int>(xq.size(0)), K = static_cast<int>(xq.size(1)), N = static_cast<int>(wq.size(0));
          need(wq.size(1) == K && K % 128 == 0, "gemm_fp8: K must match and be a multiple of 128");
          need(xs.scalar_type() == at::kFloat && xs.is_contiguous() && xs.numel() == static_cast<int64_t>(M) * (K / 128), "gemm_fp8: xs f32 [M, K/128]");
          need(ws.scalar_type() == at::kFloat && ws.is_contiguous() && ws.numel() == static_cast<int64_t>((N + 127) / 128) * (K / 128), "gemm_fp8: ws f32 [ceil(N/128), K/128]");
          need(is_bf16_2d(y) && y.size(0) == M && y.size(1) == N, "gemm_fp8: y bf16 [M, N]");
          c10::cuda::CUDAGuard g(xq.device());
          check(b2_gemm_fp8_block_ws(xq.data_ptr(), xs.data_ptr<float>(), wq.data_ptr(), ws.data_ptr<float>(), y.data_ptr(), M, N, K,
                                     y.stride(0), config, workspace.has_value() ? workspace->data_ptr() : nullptr,
                                     workspace.has_value() ? workspace->numel() * workspace->element_size() : 0, status_ptr(status),
                                     cur_stream()),
                "gemm_fp8");
        },
        py::arg("xq"), py::arg("xs"), py::arg("wq"), py::arg("ws"), py::arg("y"), py::arg("config") = 0, py::arg("status") = py::none(),
        py::arg("workspace") = py::none());

  m.def("mla_decode",
        [](const at::Tensor& q_lat, const at::Tensor& q_rope, const at::Tensor& kv_cache, at::Tensor& out_lat, const at::Tensor& ctx_lens,
           const at::Tensor& block_tables, c10::optional<at::Tensor> workspace, int num_splits, double scale,
           c10::optional<at::Tensor> status) {
          need(q_lat.is_cuda() && q_lat.scalar_type() == at::kBFloat16 && q_lat.is_contiguous() && q_lat.dim() == 3 && q_lat.size(2) == 512, "mla_decode: q_lat bf16 [B, H, 512]");
          need(q_rope.is_contiguous() && q_rope.scalar_type() == at::kBFloat16 && q_rope.dim() == 3 && q_rope.size(2) == 64 && q_rope.size(1) == q_lat.size(1), "mla_decode: q_rope bf16 [B, H, 64]");
          need(kv_cache.is_contiguous() && kv_cache.scalar_type() == at::kBFloat16 && kv_cache.dim() == 3 && kv_cache.size(2) == 576, "mla_decode: cache bf16 [pages, page, 576]");
          need(out_lat.is_contiguous() && out_lat.sizes() == q_lat.sizes() && out_lat.scalar_type() == at::kBFloat16, "mla_decode: out bf16 [B, H, 512]");
          need(ctx_lens.scalar_type() == at::kInt && block_tables.scalar_type() == at::kInt && block_tables.dim() == 2 && block_tables.is_contiguous(), "mla_decode: int32 metadata");
          const int B = static_cast<int>(q_lat.size(0)), H = static_cast<int>(q_lat.size(1));
          float* ws = nullptr;
          if (num_splits > 1) {
            need(workspace.has_value() && workspace->numel() * 4 >= b2_mla_decode_workspace(B, H, num_splits), "mla_decode: workspace too small");
            ws = workspace->data_ptr<float>();
          }
          c10::cuda::CUDAGuard g(q_lat.device());
          check(b2_mla_decode_bf16(q_lat.data_ptr(), q_rope.data_ptr(), kv_cache.data_ptr(), out_lat.data_ptr(), ctx_lens.data_ptr<int32_t>(),
                                   block_tables.data_ptr<int32_t>(), ws, B, static_cast<int>(block_tables.size(1)), H,
                                   static_cast<int>(kv_cache.size(1)), num_splits, static_cast<float>(scale), kv_cache.size(0),
                                   status_ptr(status), cur_stream()),
                "mla_decode");
        });

  m.def("mla_attend",
        [](const at::Tensor& q_lat, const at::Tensor& q_rope, const at::Tensor& kv_cache, at::Tensor& out_lat, const at::Tensor& row_ctx,
           const at::Tensor& block_tables, c10::optional<at::Tensor> row_seq, c10::optional<at::Tensor> workspace, int num_splits,
           double scale, c10::optional<at::Tensor> status) {
          need(q_lat.is_cuda() && q_lat.scalar_type() == at::kBFloat16 && q_lat.dim() == 3 && q_lat.size(2) == 512 && q_lat.stride(2) == 1 && q_lat.stride(1) == 512,
               "mla_attend: q_lat bf16 [R, H, 512] (rows may be strided)");
          need(q_rope.is_cuda() && q_rope.scalar_type() == at::kBFloat16 && q_rope.dim() == 3 && q_rope.size(2) == 64 && q_rope.stride(2) == 1 && q_rope.stride(1) == 64 &&
                   q_rope.size(0) == q_lat.size(0) && q_rope.size(1) == q_lat.size(1),
               "mla_attend: q_rope bf16 [R, H, 64] (rows may be strided)");
          need(kv_cache.is_contiguous() && kv_cache.scalar_type() == at::kBFloat16 && kv_cache.dim() == 3 && kv_cache.size(2) == 576, "mla_attend: cache bf16 [pages, page, 576]");
          need(out_lat.is_contiguous() && out_lat.sizes() == q_lat.sizes() && out_lat.scalar_type() == at::kBFloat16, "mla_attend: out bf16 [R, H, 512] contiguous");
          const int R = static_cast<int>(q_lat.size(0)), H = static_cast<int>(q_lat.size(1));
          need(row_ctx.scalar_type() == at::kInt && row_ctx.is_contiguous() && row_ctx.numel() >= R, "mla_attend: row_ctx int32 [R]");
          need(block_tables.scalar_type() == at::kInt && block_tables.dim() == 2 && block_tables.is_contiguous(), "mla_attend: block_tables int32 [S, max_blocks]");
          if (row_seq.has_value()) need(row_seq->scalar_type() == at::kInt && row_seq->is_contiguous() && row_seq->numel() >= R, "mla_attend: row_seq int32 [R]");
          else need(block_tables.size(0) >= R, "mla_attend: one block table per row when row_seq is not given");
          float* ws = nullptr;
          if (num_splits > 1) {
            need(workspace.has_value() && workspace->numel() * 4 >= b2_mla_decode_workspace(R, H, num_splits), "mla_attend: workspace too small");
            ws = workspace->data_ptr<float>();
          }
          c10::cuda::CUDAGuard g(q_lat.device());
          check(b2_mla_attend_bf16(q_lat.data_ptr(), q_rope.data_ptr(), kv_cache.data_ptr(), out_lat.data_ptr(), row_ctx.data_ptr<int32_t>(),
                                   block_tables.data_ptr<int32_t>(), row_seq.has_value() ? row_seq->data_ptr<int32_t>() : nullptr, ws, R,
                                   static_cast<int>(block_tables.size(1)), H, static_cast<int>(kv_cache.size(1)), num_splits,
                                   static_cast<float>(scale), kv_cache.size(0), q_lat.stride(0), q_rope.stride(0), status_ptr(status), cur_stream()),
                "mla_attend");
        },
        py::arg("q_lat"), py::arg("q_rope"), py::arg("kv_cache"), py::arg("out_lat"), py::arg("row_ctx"), py::arg("block_tables"),
        py::arg("row_seq") = py::none(), py::arg("workspace") = py::none(), py::arg("num_splits") = 1, py::arg("scale") = 1.0,
        py::arg("status") = py::none());

  m.def("mla_rows_meta", [](const at::Tensor& cu_q, const at::Tensor& ctx_lens, at::Tensor& row_ctx, at::Tensor& row_seq) {
    need(cu_q.is_cuda() && cu_q.scalar_type() == at::kInt && ctx_lens.scalar_type() == at::kInt && cu_q.is_contiguous() && ctx_lens.is_contiguous() &&
             cu_q.numel() == ctx_lens.numel() + 1,
         "mla_rows_meta: cu_q int32 [S + 1], ctx_lens int32 [S]");
    need(row_ctx.scalar_type() == at::kInt && row_seq.scalar_type() == at::kInt && row_ctx.is_contiguous() && row_seq.is_contiguous(), "mla_rows_meta: int32 outputs");
    c10::cuda::CUDAGuard g(cu_q.device());
    check(b2_mla_rows_meta(cu_q.data_ptr<int32_t>(), ctx_lens.data_ptr<int32_t>(), static_cast<int>(ctx_lens.numel()), row_ctx.data_ptr<int32_t>(),
                           row_seq.data_ptr<int32_t>(), cur_stream()),
          "mla_rows_meta");
  });

  py::class_<B2EpLayout>(m, "EpLayout")
      .def(py::init([]() { return B2EpLayout{}; }))
      .def_readwrite("off_recv_x", &B2EpLayout::off_recv_x)
      .def_readwrite("off_recv_meta", &B2EpLayout::off_recv_meta)
      .def_readwrite("off_recv_count", &B2EpLayout::off_recv_count)
      .def_readwrite("off_ret_y", &B2EpLayout::off_ret_y)
      .def_readwrite("off_disp_done", &B2EpLayout::off_disp_done)
      .def_readwrite("off_comb_done", &B2EpLayout::off_comb_done)
      .def_readwrite("off_epoch", &B2EpLayout::off_epoch)
      .def_readwrite("total_bytes", &B2EpLayout::total_bytes)
      .def_readwrite("cap", &B2EpLayout::cap)
      .def_readwrite("e_local", &B2EpLayout::e_local)
      .def_readwrite("hidden", &B2EpLayout::hidden)
      .def_readwrite("top_k", &B2EpLayout::top_k)
      .def_readwrite("t_cap", &B2EpLayout::t_cap);

  m.def("ep_dispatch",
        [](const at::Tensor& x, const at::Tensor& logits, at::Tensor& weights, at::Tensor& ids, int rank, const std::vector<int64_t>& peers,
           const B2EpLayout& lay, int top_k, bool norm_topk, double route_scale, int slot, uint64_t timeout_ns,
           c10::optional<at::Tensor> status) {
          need(is_bf16_2d(x) && x.is_contiguous() && is_bf16_2d(logits) && logits.is_contiguous() && logits.size(0) == x.size(0), "ep_dispatch: x [T, H], logits [T, E] contiguous bf16");
          need(weights.scalar_type() == at::kFloat && weights.is_contiguous() && ids.scalar_type() == at::kInt && ids.is_contiguous() &&
                   weights.numel() == x.size(0) * top_k && ids.numel() == x.size(0) * top_k, "ep_dispatch: weights f32 / ids i32 [T, k]");
          need(x.size(1) == lay.hidden, "ep_dispatch: hidden mismatch");
          const B2TpRegion reg = make_region(rank, peers);
          c10::cuda::CUDAGuard g(x.device());
          check(b2_ep_dispatch(x.data_ptr(), logits.data_ptr(), weights.data_ptr<float>(), ids.data_ptr<int32_t>(), &reg, &lay,
                               static_cast<int>(x.size(0)), static_cast<int>(logits.size(1)), top_k, norm_topk ? 1 : 0,
                               static_cast<float>(route_scale), slot, timeout_ns, status_ptr(status), cur_stream()),
                "ep_dispatch");
        });

  m.def("moe_grouped_gemm",
        [](const at::Tensor& x, const at::Tensor& w, const at::Tensor& counts, at::Tensor& y, int cap, bool swiglu, int bn,
           c10::optional<at::Tensor> status) {
          need(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 2, "moe_grouped_gemm: x bf16 [e_local * cap, K]");
          need(w.scalar_type() == at::kBFloat16 && w.is_contiguous() && w.dim() == 3 && w.size(2) == x.size(1), "moe_grouped_gemm: w bf16 [e_local, N, K]");
          need(counts.element_size() == 4 && counts.is_contiguous() && counts.numel() >= w.size(0), "moe_grouped_gemm: counts 32-bit [e_local]");
          const int e_local = static_cast<int>(w.size(0)), N = static_cast<int>(w.size(1)), K = static_cast<int>(w.size(2));
          need(x.size(0) == static_cast<int64_t>(e_local) * cap, "moe_grouped_gemm: x rows must be e_local * cap");
          const int64_t ldy = swiglu ? N / 2 : N;
          need(y.scalar_type() == at::kBFloat16 && y.is_contiguous() && y.numel() == static_cast<int64_t>(e_local) * cap * ldy, "moe_grouped_gemm: y bf16 [e_local * cap, N or N/2]");
          c10::cuda::CUDAGuard g(x.device());
          check(b2_moe_grouped_gemm(x.data_ptr(), w.data_ptr(), reinterpret_cast<const uint32_t*>(counts.data_ptr()), y.data_ptr(), e_local,
                                    cap, N, K, ldy, swiglu ? 1 : 0, bn, status_ptr(status), cur_stream()),
                "moe_grouped_gemm");
        });

  m.def("ep_combine",
        [](const at::Tensor& y_local, const at::Tensor& weights, c10::optional<at::Tensor> shared, at::Tensor& out, int rank,
           const std::vector<int64_t>& peers, const B2EpLayout& lay, int top_k, int slot, uint64_t timeout_ns,
           c10::optional<at::Tensor> status) {
          need(y_local.is_cuda() && y_local.scalar_type() == at::kBFloat16 && y_local.is_contiguous(), "ep_combine: y_local contiguous bf16");
          need(weights.scalar_type() == at::kFloat && weights.is_contiguous(), "ep_combine: weights f32 [T, k]");
          need(is_bf16_2d(out) && out.is_contiguous() && out.size(1) == lay.hidden && weights.numel() == out.size(0) * top_k, "ep_combine: out bf16 [T, H]");
          if (shared.has_value()) need(is_bf16_2d(*shared) && shared->is_contiguous() && shared->sizes() == out.sizes(), "ep_combine: shared must match out");
          const B2TpRegion reg = make_region(rank, peers);
          c10::cuda::CUDAGuard g(out.device());
          check(b2_ep_combine(y_local.data_ptr(), weights.data_ptr<float>(), shared.has_value() ? shared->data_ptr() : nullptr, out.data_ptr(),
                              &reg, &lay, static_cast<int>(out.size(0)), top_k, slot, timeout_ns, status_ptr(status), cur_stream()),
                "ep_combine");
        });

  m.def("gguf_dequant", [](const at::Tensor& wq, int ggml_type, at::Tensor& out) {
    need(wq.is_cuda() && wq.element_size() == 1 && wq.is_contiguous(), "gguf_dequant: packed weights as contiguous CUDA bytes");
    need(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.is_contiguous(), "gguf_dequant: out contiguous bf16");
    c10::cuda::CUDAGuard g(wq.device());
    check(b2_dequant_gguf(wq.data_ptr(), ggml_type, out.data_ptr(), out.numel(), cur_stream()), "gguf_dequant");
  });
  m.def("gemm_gguf", [](const at::Tensor& x, const at::Tensor& wq, int ggml_type, at::Tensor& y, c10::optional<at::Tensor> status) {
    need(is_bf16_2d(x) && x.is_contiguous() && is_bf16_2d(y) && y.is_contiguous() && y.size(0) == x.size(0), "gemm_gguf: x [M, K], y [M, N] contiguous bf16");
    need(wq.is_cuda() && wq.element_size() == 1 && wq.is_contiguous(), "gemm_gguf: packed weights as contiguous CUDA bytes");
    c10::cuda::CUDAGuard g(x.device());
    check(b2_gemm_gguf(x.data_ptr(), wq.data_ptr(), ggml_type, y.data_ptr(), static_cast<int>(x.size(0)), static_cast<int>(y.size(1)),
                       static_cast<int>(x.size(1)), status_ptr(status), cur_stream()),
          "gemm_gguf");
  });

  m.def("wait_flag", [](const at::Tensor& flag, uint32_t want, uint64_t timeout_ns, c10::optional<at::Tensor> status) {
    need(flag.is_cuda() && flag.element_size() == 4, "wait_flag: 32-bit CUDA flag tensor");
    c10::cuda::CUDAGuard g(flag.device());
    check(b2_wait_flag(reinterpret_cast<const uint32_t*>(flag.data_ptr()), want, timeout_ns, status_ptr(status), cur_stream()), "wait_flag");
  });
}
