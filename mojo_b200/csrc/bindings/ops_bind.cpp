// PyTorch bindings: thin argument checking around the C launch API (b2/api.h). Tensors are passed through as
// raw pointers on the current CUDA stream; nothing here allocates.
#include <torch/extension.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/cuda/CUDAGuard.h>
#include "b2/api.h"
#include "b2/launch.h"

namespace py = pybind11;
void bind_engine(py::module_& m);

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
bool is_bf16(const at::Tensor& t) { return t.scalar_type() == at::kBFloat16; }
b2::Status* status_ptr(const c10::optional<at::Tensor>& s) {
  if (!s.has_value()) return nullptr;
  need(s->is_cuda() && s->numel() * s->element_size() >= 32, "status tensor must be a CUDA tensor of >= 32 bytes");
  return reinterpret_cast<b2::Status*>(s->data_ptr());
}
void* opt_ptr(const c10::optional<at::Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }

void rmsnorm(const at::Tensor& x, c10::optional<at::Tensor> residual, const at::Tensor& weight, at::Tensor& out,
             c10::optional<at::Tensor> q_out, c10::optional<at::Tensor> q_scale, double eps) {
  need(x.is_cuda() && is_bf16(x) && x.is_contiguous() && out.is_contiguous() && is_bf16(out), "rmsnorm: x/out must be contiguous CUDA bf16");
  need(is_bf16(weight) && weight.is_contiguous(), "rmsnorm: weight must be contiguous bf16");
  const int hidden = static_cast<int>(x.size(-1));
  const int rows = static_cast<int>(x.numel() / hidden);
  need(weight.numel() == hidden && out.numel() == x.numel(), "rmsnorm: shape mismatch");
  if (residual.has_value()) need(residual->is_contiguous() && is_bf16(*residual) && residual->numel() == x.numel(), "rmsnorm: bad residual");
  c10::cuda::CUDAGuard g(x.device());
  check(b2_rmsnorm_bf16(x.data_ptr(), opt_ptr(residual), weight.data_ptr(), out.data_ptr(), opt_ptr(q_out),
                        q_scale.has_value() ? q_scale->data_ptr<float>() : nullptr, rows, hidden, static_cast<float>(eps),
                        cur_stream()),
        "rmsnorm");
}

void quant_e4m3(const at::Tensor& x, at::Tensor& q_out, at::Tensor& scale_out) {
  need(x.is_cuda() && is_bf16(x) && x.is_contiguous() && x.dim() == 2, "quant_e4m3: x must be 2-D contiguous CUDA bf16");
  need(q_out.is_contiguous() && q_out.element_size() == 1 && q_out.numel() == x.numel(), "quant_e4m3: bad q_out");
  need(scale_out.scalar_type() == at::kFloat && scale_out.is_contiguous() && scale_out.numel() == x.size(0) * (x.size(1) / 128), "quant_e4m3: bad scale_out");
  c10::cuda::CUDAGuard g(x.device());
  check(b2_quant_e4m3_1x128(x.data_ptr(), q_out.data_ptr(), scale_out.data_ptr<float>(), static_cast<int>(x.size(0)),
                            static_cast<int>(x.size(1)), cur_stream()),
        "quant_e4m3");
}

void rope_kvwrite(at::Tensor& q, at::Tensor& k, c10::optional<at::Tensor> v, const at::Tensor& cos_sin,
                  const at::Tensor& positions, c10::optional<at::Tensor> slots, c10::optional<at::Tensor> k_cache,
                  c10::optional<at::Tensor> v_cache, int64_t head_dim, bool interleaved,
                  c10::optional<at::Tensor> status) {
  need(q.is_cuda() && is_bf16(q) && is_bf16(k) && q.dim() == 2 && k.dim() == 2, "rope: q, k must be 2-D CUDA bf16 [T, heads*D]");
  need(q.stride(1) == 1 && k.stride(1) == 1, "rope: q, k must have unit inner stride");
  need(cos_sin.scalar_type() == at::kFloat && cos_sin.is_contiguous() && cos_sin.dim() == 2, "rope: cos_sin must be f32 [max_pos, rot_dim]");
  need(positions.scalar_type() == at::kInt && positions.is_contiguous(), "rope: positions must be int32");
  const int tokens = static_cast<int>(q.size(0));
  const int n_q = static_cast<int>(q.size(1) / head_dim), n_kv = static_cast<int>(k.size(1) / head_dim);
  int page_size = 1;
  int64_t num_slots = 0;
  if (k_cache.has_value()) {
    need(k_cache->dim() == 4 && k_cache->is_contiguous() && is_bf16(*k_cache), "rope: k_cache must be contiguous bf16 [pages, n_kv, page, D]");
    need(k_cache->size(1) == n_kv && k_cache->size(3) == head_dim, "rope: cache head geometry mismatch");
    need(slots.has_value() && slots->scalar_type() == at::kLong && slots->is_contiguous(), "rope: slots must be int64");
    page_size = static_cast<int>(k_cache->size(2));
    num_slots = k_cache->size(0) * page_size;
  }
  if (v.has_value()) need(is_bf16(*v) && v->stride(1) == 1 && v->size(1) == k.size(1), "rope: bad v");
  c10::cuda::CUDAGuard g(q.device());
  check(b2_rope_kvwrite_bf16(q.data_ptr(), k.data_ptr(), v.has_value() ? v->data_ptr() : nullptr, cos_sin.data_ptr<float>(),
                             positions.data_ptr<int32_t>(), slots.has_value() ? slots->data_ptr<int64_t>() : nullptr,
                             opt_ptr(k_cache), opt_ptr(v_cache), tokens, n_q, n_kv, static_cast<int>(head_dim),
                             static_cast<int>(cos_sin.size(1)), interleaved ? 1 : 0, q.stride(0), k.stride(0),
                             v.has_value() ? v->stride(0) : 0, page_size, num_slots, static_cast<int>(cos_sin.size(0)),
                             status_ptr(status), cur_stream()),
        "rope_kvwrite");
}

void swiglu(const at::Tensor& gate_up, at::Tensor& out, bool interleaved) {
  need(gate_up.is_cuda() && is_bf16(gate_up) && gate_up.is_contiguous() && out.is_contiguous() && is_bf16(out), "swiglu: contiguous CUDA bf16 required");
  const int ffn = static_cast<int>(out.size(-1));
  need(gate_up.size(-1) == 2 * ffn, "swiglu: gate_up last dim must be 2 * ffn");
  c10::cuda::CUDAGuard g(out.device());
  check(b2_swiglu_bf16(gate_up.data_ptr(), out.data_ptr(), static_cast<int>(out.numel() / ffn), ffn, interleaved ? 1 : 0, cur_stream()), "swiglu");
}

void embedding(const at::Tensor& ids, const at::Tensor& table, at::Tensor& out, int64_t vocab_start) {
  need(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "embedding: ids must be contiguous CUDA int64");
  need(is_bf16(table) && table.is_contiguous() && is_bf16(out) && out.is_contiguous(), "embedding: bf16 contiguous table/out required");
  need(out.size(-1) == table.size(1) && out.numel() == ids.numel() * table.size(1), "embedding: shape mismatch");
  c10::cuda::CUDAGuard g(out.device());
  check(b2_embedding_bf16(ids.data_ptr<int64_t>(), table.data_ptr(), out.data_ptr(), static_cast<int>(ids.numel()),
                          static_cast<int>(table.size(1)), vocab_start, table.size(0), cur_stream()),
        "embedding");
}

void patch_tokens(at::Tensor& tok, const at::Tensor& rows, const at::Tensor& src, const at::Tensor& prev, int64_t n, c10::optional<at::Tensor> status) {
  need(tok.is_cuda() && tok.scalar_type() == at::kLong && tok.is_contiguous() && prev.is_cuda() && prev.scalar_type() == at::kLong && prev.is_contiguous(),
       "patch_tokens: tok and prev must be contiguous CUDA int64");
  need(rows.is_cuda() && src.is_cuda() && rows.scalar_type() == at::kInt && src.scalar_type() == at::kInt && rows.is_contiguous() && src.is_contiguous() &&
           rows.numel() >= n && src.numel() >= n,
       "patch_tokens: rows and src must be contiguous CUDA int32 with at least n entries");
  c10::cuda::CUDAGuard g(tok.device());
  check(b2_patch_tokens(tok.data_ptr<int64_t>(), rows.data_ptr<int32_t>(), src.data_ptr<int32_t>(), prev.data_ptr<int64_t>(), static_cast<int>(n),
                        tok.numel(), prev.numel(), status_ptr(status), cur_stream()),
        "patch_tokens");
}

void gather_rows(const at::Tensor& src, const at::Tensor& index, at::Tensor& out, c10::optional<at::Tensor> status) {
  need(src.is_cuda() && is_bf16(src) && src.is_contiguous() && src.dim() == 2 && out.is_contiguous() && is_bf16(out), "gather_rows: bf16 contiguous 2-D required");
  need(index.scalar_type() == at::kLong && index.is_contiguous(), "gather_rows: index must be int64");
  c10::cuda::CUDAGuard g(out.device());
  check(b2_gather_rows_bf16(src.data_ptr(), index.data_ptr<int64_t>(), out.data_ptr(), static_cast<int>(index.numel()),
                            static_cast<int>(src.size(1)), src.size(0), status_ptr(status), cur_stream()),
        "gather_rows");
}

void scatter_rows(const at::Tensor& src, const at::Tensor& slots, at::Tensor& dst, c10::optional<at::Tensor> status) {
  need(src.is_cuda() && is_bf16(src) && src.is_contiguous() && src.dim() == 2 && is_bf16(dst) && dst.is_contiguous() && dst.dim() == 2 && dst.size(1) == src.size(1), "scatter_rows: bf16 contiguous 2-D src/dst with equal width");
  need(slots.scalar_type() == at::kLong && slots.is_contiguous() && slots.numel() == src.size(0), "scatter_rows: int64 slots [rows]");
  c10::cuda::CUDAGuard g(src.device());
  check(b2_scatter_rows_bf16(src.data_ptr(), slots.data_ptr<int64_t>(), dst.data_ptr(), static_cast<int>(src.size(0)),
                             static_cast<int>(src.size(1)), dst.size(0), status_ptr(status), cur_stream()),
        "scatter_rows");
}

void copy_pages(at::Tensor& cache, const at::Tensor& src_pages, const at::Tensor& dst_pages, c10::optional<at::Tensor> status) {
  need(cache.is_cuda() && cache.is_contiguous() && cache.dim() >= 2, "copy_pages: cache must be contiguous CUDA");
  need(src_pages.scalar_type() == at::kLong && dst_pages.scalar_type() == at::kLong && src_pages.numel() == dst_pages.numel(), "copy_pages: int64 page lists of equal length");
  const int64_t page_bytes = cache.stride(0) * cache.element_size();
  c10::cuda::CUDAGuard g(cache.device());
  check(b2_copy_pages(cache.data_ptr(), src_pages.data_ptr<int64_t>(), dst_pages.data_ptr<int64_t>(),
                      static_cast<int>(src_pages.numel()), page_bytes, cache.size(0), status_ptr(status), cur_stream()),
        "copy_pages");
}

void argmax(const at::Tensor& logits, at::Tensor& ids, c10::optional<at::Tensor> max_out) {
  need(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "argmax: logits must be 2-D CUDA with unit inner stride");
  need(is_bf16(logits) || logits.scalar_type() == at::kFloat, "argmax: logits must be bf16 or f32");
  need(ids.scalar_type() == at::kLong && ids.is_contiguous() && ids.numel() == logits.size(0), "argmax: ids must be int64 [rows]");
  c10::cuda::CUDAGuard g(logits.device());
  check(b2_argmax(logits.data_ptr(), is_bf16(logits) ? 1 : 0, ids.data_ptr<int64_t>(),
                  max_out.has_value() ? max_out->data_ptr<float>() : nullptr, static_cast<int>(logits.size(0)),
                  static_cast<int>(logits.size(1)), logits.stride(0), cur_stream()),
        "argmax");
}

void sample(const at::Tensor& logits, at::Tensor& ids, c10::optional<at::Tensor> temperature, c10::optional<at::Tensor> top_k,
            c10::optional<at::Tensor> top_p, c10::optional<at::Tensor> uniforms, uint64_t seed, uint64_t step) {
  need(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "sample: logits must be 2-D CUDA with unit inner stride");
  need(is_bf16(logits) || logits.scalar_type() == at::kFloat, "sample: logits must be bf16 or f32");
  need(ids.scalar_type() == at::kLong && ids.is_contiguous() && ids.numel() == logits.size(0), "sample: ids must be int64 [rows]");
  const int64_t rows = logits.size(0);
  if (temperature.has_value()) need(temperature->scalar_type() == at::kFloat && temperature->numel() == rows, "sample: temperature f32 [rows]");
  if (top_k.has_value()) need(top_k->scalar_type() == at::kInt && top_k->numel() == rows, "sample: top_k int32 [rows]");
  if (top_p.has_value()) need(top_p->scalar_type() == at::kFloat && top_p->numel() == rows, "sample: top_p f32 [rows]");
  if (uniforms.has_value()) need(uniforms->scalar_type() == at::kFloat && uniforms->numel() == rows, "sample: uniforms f32 [rows]");
  c10::cuda::CUDAGuard g(logits.device());
  check(b2_sample(logits.data_ptr(), is_bf16(logits) ? 1 : 0, ids.data_ptr<int64_t>(),
                  temperature.has_value() ? temperature->data_ptr<float>() : nullptr,
                  top_k.has_value() ? top_k->data_ptr<int32_t>() : nullptr,
                  top_p.has_value() ? top_p->data_ptr<float>() : nullptr,
                  uniforms.has_value() ? uniforms->data_ptr<float>() : nullptr, seed, step, static_cast<int>(rows),
                  static_cast<int>(logits.size(1)), logits.stride(0), cur_stream()),
        "sample");
}

void check_cache(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache, int64_t head_dim) {
  need(q.is_cuda() && is_bf16(q) && q.dim() == 2 && q.stride(1) == 1, "attention: q must be 2-D CUDA bf16 [T, n_q*D]");
  need(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous() && is_bf16(k_cache) && is_bf16(v_cache), "attention: caches must be contiguous bf16 [pages, n_kv, page, D]");
  need(k_cache.size(3) == head_dim && v_cache.sizes() == k_cache.sizes(), "attention: cache geometry mismatch");
}

void attn_prefill(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache, at::Tensor& out,
                  const at::Tensor& cu_q, const at::Tensor& ctx_lens, const at::Tensor& block_tables, int64_t head_dim,
                  int64_t max_q_len, double scale, c10::optional<at::Tensor> status) {
  check_cache(q, k_cache, v_cache, head_dim);
  need(out.dim() == 2 && out.stride(1) == 1 && is_bf16(out) && out.size(0) == q.size(0), "attention: bad out");
  need(cu_q.scalar_type() == at::kInt && ctx_lens.scalar_type() == at::kInt && block_tables.scalar_type() == at::kInt, "attention: metadata must be int32");
  need(block_tables.dim() == 2 && block_tables.is_contiguous() && cu_q.is_contiguous() && ctx_lens.is_contiguous(), "attention: metadata must be contiguous");
  const int batch = static_cast<int>(ctx_lens.numel());
  need(cu_q.numel() == batch + 1 && block_tables.size(0) == batch, "attention: metadata batch mismatch");
  c10::cuda::CUDAGuard g(q.device());
  check(b2_attn_prefill_bf16(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), cu_q.data_ptr<int32_t>(),
                             ctx_lens.data_ptr<int32_t>(), block_tables.data_ptr<int32_t>(), batch,
                             static_cast<int>(block_tables.size(1)), static_cast<int>(q.size(1) / head_dim),
                             static_cast<int>(k_cache.size(1)), static_cast<int>(head_dim), static_cast<int>(k_cache.size(2)),
                             static_cast<int>(max_q_len), static_cast<float>(scale), q.stride(0), out.stride(0),
                             k_cache.size(0), status_ptr(status), cur_stream()),
        "attn_prefill");
}

void gemm_bf16_pair(const at::Tensor& x, const at::Tensor& w, at::Tensor& y, int64_t epilogue, int64_t bn, c10::optional<at::Tensor> status) {
  need(x.is_cuda() && is_bf16(x) && is_bf16(w) && is_bf16(y) && x.dim() == 2 && w.dim() == 2 && y.dim() == 2, "gemm_bf16_pair: 2-D CUDA bf16 tensors");
  need(x.stride(1) == 1 && w.stride(1) == 1 && y.stride(1) == 1 && x.size(1) == w.size(1) && y.size(0) == x.size(0) &&
           y.size(1) == (epilogue == B2_EPI_SWIGLU ? w.size(0) / 2 : w.size(0)),
       "gemm_bf16_pair: x [M, K], w [N, K], y [M, N] (or [M, N / 2] with the SwiGLU epilogue), unit inner strides");
  c10::cuda::CUDAGuard g(x.device());
  check(b2_gemm_bf16_pair(x.data_ptr(), w.data_ptr(), y.data_ptr(), static_cast<int>(x.size(0)), static_cast<int>(w.size(0)),
                          static_cast<int>(x.size(1)), x.stride(0), w.stride(0), y.stride(0), static_cast<int>(epilogue), static_cast<int>(bn), status_ptr(status), cur_stream()),
        "gemm_bf16_pair");
}

void attn_prefill_tc(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache, at::Tensor& out,
                     const at::Tensor& cu_q, const at::Tensor& ctx_lens, const at::Tensor& block_tables, int64_t max_q_len,
                     double scale, int64_t variant, c10::optional<at::Tensor> status, c10::optional<at::Tensor> work,
                     c10::optional<at::Tensor> n_work, int64_t work_items) {
  check_cache(q, k_cache, v_cache, 128);
  if (work.has_value()) {
    need(work->is_cuda() && work->scalar_type() == at::kInt && work->is_contiguous() && work->numel() >= 2 * work_items, "attn_prefill_tc: work must be CUDA int32 [items, 2]");
    if (n_work.has_value()) need(n_work->is_cuda() && n_work->scalar_type() == at::kInt && n_work->numel() >= 1, "attn_prefill_tc: n_work must be a CUDA int32 scalar");
  }
  need(k_cache.size(2) == 128 && k_cache.size(3) == 128, "attn_prefill_tc: head_dim 128 and page_size 128 only");
  need(out.dim() == 2 && out.stride(1) == 1 && is_bf16(out) && out.size(0) == q.size(0), "attention: bad out");
  need(cu_q.scalar_type() == at::kInt && ctx_lens.scalar_type() == at::kInt && block_tables.scalar_type() == at::kInt, "attention: metadata must be int32");
  need(block_tables.dim() == 2 && block_tables.is_contiguous() && cu_q.is_contiguous() && ctx_lens.is_contiguous(), "attention: metadata must be contiguous");
  const int batch = static_cast<int>(ctx_lens.numel());
  need(cu_q.numel() == batch + 1 && block_tables.size(0) == batch, "attention: metadata batch mismatch");
  c10::cuda::CUDAGuard g(q.device());
  check(b2_attn_prefill_tc_bf16(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), cu_q.data_ptr<int32_t>(),
                                ctx_lens.data_ptr<int32_t>(), block_tables.data_ptr<int32_t>(), batch,
                                static_cast<int>(block_tables.size(1)), static_cast<int>(q.size(1) / 128),
                                static_cast<int>(k_cache.size(1)), static_cast<int>(max_q_len), static_cast<float>(scale), q.size(0),
                                q.stride(0), out.stride(0), k_cache.size(0), static_cast<int>(variant),
                                work.has_value() ? work->data_ptr<int32_t>() : nullptr,
                                work.has_value() && n_work.has_value() ? n_work->data_ptr<int32_t>() : nullptr,
                                static_cast<int>(work_items), status_ptr(status), cur_stream()),
        "attn_prefill_tc");
}

void attn_decode(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache, at::Tensor& out,
                 const at::Tensor& ctx_lens, const at::Tensor& block_tables, c10::optional<at::Tensor> workspace,
                 int64_t head_dim, int64_t num_splits, double scale, c10::optional<at::Tensor> status,
                 c10::optional<at::Tensor> counters) {
  check_cache(q, k_cache, v_cache, head_dim);
  need(out.dim() == 2 && out.stride(1) == 1 && is_bf16(out) && out.size(0) == q.size(0), "attention: bad out");
  need(ctx_lens.scalar_type() == at::kInt && block_tables.scalar_type() == at::kInt && block_tables.dim() == 2 && block_tables.is_contiguous(), "attention: metadata must be contiguous int32");
  const int batch = static_cast<int>(ctx_lens.numel());
  need(q.size(0) == batch && block_tables.size(0) == batch, "attention: decode expects one query row per sequence");
  const int n_q = static_cast<int>(q.size(1) / head_dim);
  float* ws = nullptr;
  if (num_splits > 1) {
    need(workspace.has_value() && workspace->scalar_type() == at::kFloat, "attention: split decode needs an f32 workspace");
    need(workspace->numel() * 4 >= b2_attn_decode_workspace(batch, n_q, static_cast<int>(head_dim), static_cast<int>(num_splits)), "attention: workspace too small");
    ws = workspace->data_ptr<float>();
  }
  uint32_t* cnt = nullptr;
  if (num_splits > 1 && counters.has_value()) {
    need(counters->is_cuda() && counters->scalar_type() == at::kInt && counters->is_contiguous(), "attention: split counters must be a contiguous CUDA int32 tensor");
    if (counters->numel() * 4 >= b2_attn_decode_counter_bytes(batch, static_cast<int>(k_cache.size(1))))
      cnt = reinterpret_cast<uint32_t*>(counters->data_ptr());
  }
  c10::cuda::CUDAGuard g(q.device());
  check(b2_attn_decode_bf16(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), ctx_lens.data_ptr<int32_t>(),
                            block_tables.data_ptr<int32_t>(), ws, batch, static_cast<int>(block_tables.size(1)), n_q,
                            static_cast<int>(k_cache.size(1)), static_cast<int>(head_dim), static_cast<int>(k_cache.size(2)),
                            static_cast<int>(num_splits), static_cast<float>(scale), q.stride(0), out.stride(0),
                            k_cache.size(0), cnt, status_ptr(status), cur_stream()),
        "attn_decode");
}

void gemm_bf16(const at::Tensor& x, const at::Tensor& w, at::Tensor& y, c10::optional<at::Tensor> residual,
               int64_t epilogue, int64_t config, c10::optional<at::Tensor> workspace, c10::optional<at::Tensor> status) {
  need(x.is_cuda() && is_bf16(x) && is_bf16(w) && is_bf16(y) && x.dim() == 2 && w.dim() == 2 && y.dim() == 2, "gemm: 2-D CUDA bf16 x [M,K], w [N,K], y [M,N]");
  need(x.stride(1) == 1 && w.stride(1) == 1 && y.stride(1) == 1, "gemm: unit inner strides required");
  const int M = static_cast<int>(x.size(0)), K = static_cast<int>(x.size(1)), N = static_cast<int>(w.size(0));
  need(w.size(1) == K, "gemm: K mismatch");
  const int64_t out_cols = epilogue == B2_EPI_SWIGLU ? N / 2 : N;
  need(y.size(0) == M && y.size(1) == out_cols, "gemm: output shape mismatch");
  if (residual.has_value()) need(is_bf16(*residual) && residual->sizes() == y.sizes() && residual->stride(1) == 1 && residual->stride(0) == y.stride(0), "gemm: residual must match y");
  c10::cuda::CUDAGuard g(x.device());
  check(b2_gemm_bf16(x.data_ptr(), w.data_ptr(), y.data_ptr(), opt_ptr(residual), M, N, K, x.stride(0), w.stride(0),
                     y.stride(0), static_cast<int>(epilogue), static_cast<int>(config), opt_ptr(workspace),
                     workspace.has_value() ? workspace->numel() * workspace->element_size() : 0, status_ptr(status),
                     cur_stream()),
        "gemm_bf16");
}

py::dict device_caps(int device) {
  B2DeviceCaps c;
  py::dict d;
  if (b2_device_caps(device, &c) != 0) return d;
  d["name"] = std::string(c.name);
  d["cc_major"] = c.cc_major;
  d["cc_minor"] = c.cc_minor;
  d["sm_count"] = c.sm_count;
  d["smem_per_block_optin"] = c.smem_per_block_optin;
  d["l2_bytes"] = c.l2_bytes;
  d["total_mem"] = c.total_mem;
  d["can_map_peer"] = c.can_map_peer != 0;
  d["multicast_supported"] = c.multicast_supported != 0;
  d["clock_khz"] = c.clock_khz;
  d["mem_clock_khz"] = c.mem_clock_khz;
  d["max_cluster"] = c.max_cluster;
  return d;
}

}  // namespace

void bind_ops_extra(py::module_& m);
void bind_coll(py::module_& m);
void bind_io(py::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "mojo_b200 native extension: sm_100a kernels + engine runtime";
  bind_engine(m);
  m.def("rmsnorm", &rmsnorm, py::arg("x"), py::arg("residual"), py::arg("weight"), py::arg("out"), py::arg("q_out") = py::none(),
        py::arg("q_scale") = py::none(), py::arg("eps") = 1e-5);
  m.def("quant_e4m3", &quant_e4m3);
  m.def("rope_kvwrite", &rope_kvwrite, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("cos_sin"), py::arg("positions"),
        py::arg("slots"), py::arg("k_cache"), py::arg("v_cache"), py::arg("head_dim"), py::arg("interleaved") = false,
        py::arg("status") = py::none());
  m.def("swiglu", &swiglu, py::arg("gate_up"), py::arg("out"), py::arg("interleaved") = false);
  m.def("embedding", &embedding, py::arg("ids"), py::arg("table"), py::arg("out"), py::arg("vocab_start") = 0);
  m.def("patch_tokens", &patch_tokens, py::arg("tok"), py::arg("rows"), py::arg("src"), py::arg("prev"), py::arg("n"), py::arg("status") = py::none());
  m.def("gather_rows", &gather_rows, py::arg("src"), py::arg("index"), py::arg("out"), py::arg("status") = py::none());
  m.def("scatter_rows", &scatter_rows, py::arg("src"), py::arg("slots"), py::arg("dst"), py::arg("status") = py::none());
  m.def("copy_pages", &copy_pages, py::arg("cache"), py::arg("src_pages"), py::arg("dst_pages"), py::arg("status") = py::none());
  m.def("argmax", &argmax, py::arg("logits"), py::arg("ids"), py::arg("max_out") = py::none());
  m.def("sample", &sample, py::arg("logits"), py::arg("ids"), py::arg("temperature") = py::none(), py::arg("top_k") = py::none(),
        py::arg("top_p") = py::none(), py::arg("uniforms") = py::none(), py::arg("seed") = 0, py::arg("step") = 0);
  m.def("attn_prefill", &attn_prefill, py::arg("q"), py::arg("k_cache"), py::arg("v_cache"), py::arg("out"), py::arg("cu_q"),
        py::arg("ctx_lens"), py::arg("block_tables"), py::arg("head_dim"), py::arg("max_q_len"), py::arg("scale"),
        py::arg("status") = py::none());
  m.def("gemm_bf16_pair", &gemm_bf16_pair, py::arg("x"), py::arg("w"), py::arg("y"), py::arg("epilogue") = 0, py::arg("bn") = 256, py::arg("status") = py::none());
  m.def("attn_prefill_tc", &attn_prefill_tc, py::arg("q"), py::arg("k_cache"), py::arg("v_cache"), py::arg("out"), py::arg("cu_q"),
        py::arg("ctx_lens"), py::arg("block_tables"), py::arg("max_q_len"), py::arg("scale"), py::arg("variant") = 0,
        py::arg("status") = py::none(), py::arg("work") = py::none(), py::arg("n_work") = py::none(), py::arg("work_items") = 0);
  m.def("attn_decode", &attn_decode, py::arg("q"), py::arg("k_cache"), py::arg("v_cache"), py::arg("out"), py::arg("ctx_lens"),
        py::arg("block_tables"), py::arg("workspace"), py::arg("head_dim"), py::arg("num_splits"), py::arg("scale"),
        py::arg("status") = py::none(), py::arg("counters") = py::none());
  m.def("gemm_bf16", &gemm_bf16, py::arg("x"), py::arg("w"), py::arg("y"), py::arg("residual") = py::none(),
        py::arg("epilogue") = 0, py::arg("config") = 0, py::arg("workspace") = py::none(), py::arg("status") = py::none());
  m.def("gemm_workspace_bytes", [](int M, int N, int K) { return b2_gemm_workspace_bytes(M, N, K); });
  m.def("attn_decode_workspace_bytes", [](int batch, int n_q, int d, int splits) { return b2_attn_decode_workspace(batch, n_q, d, splits); });
  m.def("device_caps", &device_caps, py::arg("device") = 0);
  bind_ops_extra(m);
  bind_coll(m);
  bind_io(m);
}
