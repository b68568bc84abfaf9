// pybind11 bindings of the host engine runtime (KV manager, scheduler). No PyTorch dependency.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include "b2/dtype.h"
#include "b2/engine.h"
#include "b2/symm_sim.h"

namespace py = pybind11;
using namespace b2::engine;

namespace {
template <typename T>
py::array_t<T> to_array(const std::vector<T>& v) {
  py::array_t<T> a(static_cast<py::ssize_t>(v.size()));
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(T));
  return a;
}
}  // namespace

void bind_engine(py::module_& m) {
  // CPU-rank simulator of the symmetric-memory collective protocol, with host-side fault injection
  m.def(
      "symm_sim_run",
      [](int world, int n, int steps, const std::string& algo, const std::string& fault, int timeout_ms) {
        b2::sim::Fault f;
        if (!b2::sim::parse_fault(fault, &f)) throw std::invalid_argument("mojo_b200: malformed fault spec '" + fault + "'");
        b2::sim::Algo a;
        if (algo == "one_shot") a = b2::sim::Algo::kOneShot;
        else if (algo == "two_shot") a = b2::sim::Algo::kTwoShot;
        else if (algo == "all_to_all") a = b2::sim::Algo::kAllToAll;
        else throw std::invalid_argument("mojo_b200: symm_sim_run: algo must be one_shot, two_shot or all_to_all");
        if (world < 1 || world > 8 || n < 1 || steps < 0 || timeout_ms < 1) throw std::invalid_argument("mojo_b200: symm_sim_run: bad sizes");
        b2::sim::SimResult r;
        {
          py::gil_scoped_release nogil;
          r = b2::sim::run(world, n, steps, a, f, timeout_ms);
        }
        py::list ranks;
        for (const auto& rr : r.ranks) {
          py::dict d;
          d["code"] = rr.code;
          d["step"] = rr.step;
          d["peer"] = rr.peer;
          d["which"] = rr.which;
          d["wrong_steps"] = rr.wrong_steps;
          d["timeouts"] = rr.timeouts;
          ranks.append(d);
        }
        py::dict out;
        out["ranks"] = ranks;
        out["elapsed_ms"] = r.elapsed_ms;
        return out;
      },
      py::arg("world"), py::arg("n"), py::arg("steps"), py::arg("algo") = "one_shot", py::arg("fault") = "", py::arg("timeout_ms") = 2000);
  m.def("hash_page", [](uint64_t parent, py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens) {
    return hash_page(parent, tokens.data(), static_cast<int>(tokens.size()));
  });
  m.def("f32_to_bf16_bits", [](float f) { return b2::f32_to_bf16_bits(f); });
  m.def("bf16_bits_to_f32", [](uint16_t h) { return b2::bf16_bits_to_f32(h); });
  m.def("e4m3_bits_to_f32", [](uint8_t v) { return b2::e4m3_bits_to_f32(v); });
  m.def("e5m2_bits_to_f32", [](uint8_t v) { return b2::e5m2_bits_to_f32(v); });
  m.def("f32_to_e4m3_bits", [](float f) { return b2::f32_to_e4m3_bits(f); });

  py::class_<KVStats>(m, "KVStats")
      .def_readonly("num_pages", &KVStats::num_pages)
      .def_readonly("free_pages", &KVStats::free_pages)
      .def_readonly("cached_pages", &KVStats::cached_pages)
      .def_readonly("prefix_hits", &KVStats::prefix_hits)
      .def_readonly("prefix_queries", &KVStats::prefix_queries)
      .def_readonly("evictions", &KVStats::evictions);

  py::class_<KVCacheManager>(m, "KVCacheManager")
      .def(py::init<int64_t, int, bool>(), py::arg("num_pages"), py::arg("page_size"), py::arg("enable_prefix_cache") = false)
      .def_property_readonly("page_size", &KVCacheManager::page_size)
      .def_property_readonly("num_pages", &KVCacheManager::num_pages)
      .def("available_pages", &KVCacheManager::available_pages)
      .def("pages_needed", &KVCacheManager::pages_needed)
      .def("has_sequence", &KVCacheManager::has_sequence)
      .def("add_sequence",
           [](KVCacheManager& k, int64_t id, py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens) {
             return k.add_sequence(id, tokens.data(), static_cast<int64_t>(tokens.size()));
           })
      .def("reserve", &KVCacheManager::reserve)
      .def("commit",
           [](KVCacheManager& k, int64_t id, py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens, int64_t n) {
             k.commit(id, tokens.data(), std::min<int64_t>(n, tokens.size()));
           })
      .def("free_sequence", &KVCacheManager::free_sequence)
      .def("fork",
           [](KVCacheManager& k, int64_t src, int64_t dst) {
             std::vector<std::pair<int64_t, int64_t>> copies;
             const bool ok = k.fork(src, dst, &copies);
             return py::make_tuple(ok, copies);
           })
      .def("block_table", [](const KVCacheManager& k, int64_t id) { return to_array(k.block_table(id)); })
      .def("slot", &KVCacheManager::slot)
      .def("num_tokens_reserved", &KVCacheManager::num_tokens_reserved)
      .def("stats", &KVCacheManager::stats)
      .def("check_invariants", &KVCacheManager::check_invariants);

  py::class_<SchedulerConfig>(m, "SchedulerConfig")
      .def(py::init<>())
      .def_readwrite("max_num_seqs", &SchedulerConfig::max_num_seqs)
      .def_readwrite("max_num_batched_tokens", &SchedulerConfig::max_num_batched_tokens)
      .def_readwrite("max_model_len", &SchedulerConfig::max_model_len)
      .def_readwrite("enable_chunked_prefill", &SchedulerConfig::enable_chunked_prefill)
      .def_readwrite("decode_reserve_pages", &SchedulerConfig::decode_reserve_pages);

  py::class_<Batch>(m, "Batch")
      .def_property_readonly("seq_ids", [](const Batch& b) { return to_array(b.seq_ids); })
      .def_property_readonly("q_lens", [](const Batch& b) { return to_array(b.q_lens); })
      .def_property_readonly("ctx_lens", [](const Batch& b) { return to_array(b.ctx_lens); })
      .def_property_readonly("cu_q", [](const Batch& b) { return to_array(b.cu_q); })
      .def_property_readonly("token_ids", [](const Batch& b) { return to_array(b.token_ids); })
      .def_property_readonly("positions", [](const Batch& b) { return to_array(b.positions); })
      .def_property_readonly("slots", [](const Batch& b) { return to_array(b.slots); })
      .def_property_readonly("block_tables",
                             [](const Batch& b) {
                               auto a = to_array(b.block_tables);
                               a.resize({static_cast<py::ssize_t>(b.seq_ids.size()), static_cast<py::ssize_t>(b.max_blocks)});
                               return a;
                             })
      .def_property_readonly("sample_rows", [](const Batch& b) { return to_array(b.sample_rows); })
      .def_property_readonly("sample_seq_ids", [](const Batch& b) { return to_array(b.sample_seq_ids); })
      .def_property_readonly("preempted", [](const Batch& b) { return to_array(b.preempted); })
      .def_readonly("max_blocks", &Batch::max_blocks)
      .def_readonly("num_decode", &Batch::num_decode)
      .def_readonly("num_prefill", &Batch::num_prefill)
      .def_readonly("max_q_len", &Batch::max_q_len)
      .def_readonly("num_tokens", &Batch::num_tokens)
      .def_property_readonly("num_seqs", [](const Batch& b) { return b.seq_ids.size(); });

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<SchedulerConfig, KVCacheManager*>(), py::keep_alive<1, 3>())
      .def("add_request",
           [](Scheduler& s, int64_t id, py::array_t<int32_t, py::array::c_style | py::array::forcecast> prompt,
              int64_t max_new_tokens, double arrival) {
             s.add_request(id, prompt.data(), static_cast<int64_t>(prompt.size()), max_new_tokens, arrival);
           },
           py::arg("id"), py::arg("prompt"), py::arg("max_new_tokens"), py::arg("arrival") = 0.0)
      .def("step", &Scheduler::step)
      .def("append_token", &Scheduler::append_token)
      .def("finish", &Scheduler::finish)
      .def("abort", &Scheduler::abort)
      .def("commit_step", &Scheduler::commit_step)
      .def("set_auto_commit", &Scheduler::set_auto_commit)
      .def("set_token", &Scheduler::set_token)
      .def("num_tokens", &Scheduler::num_tokens)
      .def("has_unfinished", &Scheduler::has_unfinished)
      .def("num_waiting", &Scheduler::num_waiting)
      .def("num_running", &Scheduler::num_running)
      .def("total_preemptions", &Scheduler::total_preemptions)
      .def("tokens",
           [](const Scheduler& s, int64_t id) {
             const Request* r = s.request(id);
             if (r == nullptr) throw py::key_error("unknown request");
             return to_array(r->tokens);
           })
      .def("request_info", [](const Scheduler& s, int64_t id) {
        const Request* r = s.request(id);
        if (r == nullptr) throw py::key_error("unknown request");
        py::dict d;
        d["prompt_len"] = r->prompt_len;
        d["generated"] = r->generated;
        d["computed"] = r->computed;
        d["preemptions"] = r->preemptions;
        d["status"] = static_cast<int>(r->status);
        return d;
      });
}
