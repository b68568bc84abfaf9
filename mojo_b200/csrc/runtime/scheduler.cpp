// Iteration-level (continuous-batching) scheduler with chunked prefill and recompute preemption.
//
// Every step spends one token budget: each running sequence that has exactly one uncomputed token (decode)
// takes one token; sequences in the middle of their prompt take a chunk of what is left; then waiting
// requests are admitted with whatever budget and KV pages remain. When a running sequence cannot get a page
// the most recently admitted sequence is pushed back to the head of the waiting queue and recomputed later.
#include <algorithm>
#include <stdexcept>
#include "b2/engine.h"

namespace b2 {
namespace engine {

Scheduler::Scheduler(SchedulerConfig cfg, KVCacheManager* kv) : cfg_(cfg), kv_(kv) {
  if (kv == nullptr) throw std::invalid_argument("Scheduler: kv manager is null");
  if (cfg_.max_num_seqs <= 0 || cfg_.max_num_batched_tokens <= 0) throw std::invalid_argument("Scheduler: bad limits");
}

void Scheduler::add_request(int64_t id, const int32_t* prompt, int64_t prompt_len, int64_t max_new_tokens,
                            double arrival) {
  if (reqs_.count(id)) throw std::invalid_argument("Scheduler: duplicate request id");
  if (prompt_len <= 0) throw std::invalid_argument("Scheduler: empty prompt");
  if (prompt_len + 1 > cfg_.max_model_len) throw std::invalid_argument("Scheduler: prompt longer than max_model_len");
  // Without chunked prefill a prompt must fit one step's token budget, or it would sit at the head of the queue forever.
  if (!cfg_.enable_chunked_prefill && prompt_len > cfg_.max_num_batched_tokens)
    throw std::invalid_argument("Scheduler: prompt longer than max_num_batched_tokens and chunked prefill is off");
  const int64_t max_pages = (std::min<int64_t>(prompt_len + max_new_tokens, cfg_.max_model_len) + kv_->page_size() - 1) / kv_->page_size();
  if (max_pages > kv_->num_pages()) throw std::invalid_argument("Scheduler: request can never fit in the KV cache");
  Request r;
  r.id = id;
  r.tokens.assign(prompt, prompt + prompt_len);
  r.prompt_len = prompt_len;
  r.max_new_tokens = max_new_tokens;
  r.arrival = arrival;
  reqs_.emplace(id, std::move(r));
  waiting_.push_back(id);
}

const Request* Scheduler::request(int64_t id) const {
  auto it = reqs_.find(id);
  return it == reqs_.end() ? nullptr : &it->second;
}

bool Scheduler::preempt_one(int64_t keep_id, Batch* b) {
  if (running_.empty()) return false;
  const int64_t victim = running_.back();
  running_.pop_back();
  Request& r = reqs_.at(victim);
  drop_pending_commit(victim);
  kv_->free_sequence(victim);
  r.computed = 0;
  r.status = SeqStatus::kWaiting;
  ++r.preemptions;
  ++total_preemptions_;
  waiting_.push_front(victim);
  b->preempted.push_back(victim);
  return victim != keep_id;
}

namespace {
struct Entry {
  int64_t id;
  int64_t n;
};
}  // namespace

void Scheduler::emit(Request& r, int64_t n, Batch* b) {
  const int64_t start = r.computed;
  b->seq_ids.push_back(r.id);
  b->q_lens.push_back(static_cast<int32_t>(n));
  b->ctx_lens.push_back(static_cast<int32_t>(start + n));
  for (int64_t i = 0; i < n; ++i) {
    b->token_ids.push_back(r.tokens[start + i]);
    b->positions.push_back(static_cast<int32_t>(start + i));
    b->slots.push_back(kv_->slot(r.id, start + i));
  }
  b->cu_q.push_back(static_cast<int32_t>(b->token_ids.size()));
  if (start + n == static_cast<int64_t>(r.tokens.size())) {
    b->sample_rows.push_back(static_cast<int32_t>(b->token_ids.size()) - 1);
    b->sample_seq_ids.push_back(r.id);
  }
  r.computed = start + n;
  // The pages become prefix-cache entries only once the step that writes their KV has completed (commit_step).
  if (pending_commits_.empty()) pending_commits_.emplace_back();
  pending_commits_.back().push_back({r.id, r.computed});
  b->max_q_len = std::max<int>(b->max_q_len, static_cast<int>(n));
}

void Scheduler::commit_step() {
  if (pending_commits_.empty()) return;
  for (const auto& pc : pending_commits_.front()) {
    auto it = reqs_.find(pc.first);
    if (it == reqs_.end()) continue;
    kv_->commit(pc.first, it->second.tokens.data(), std::min<int64_t>(pc.second, static_cast<int64_t>(it->second.tokens.size())));
  }
  pending_commits_.pop_front();
}

void Scheduler::drop_pending_commit(int64_t id) {
  for (auto& batch : pending_commits_)
    batch.erase(std::remove_if(batch.begin(), batch.end(), [id](const std::pair<int64_t, int64_t>& pc) { return pc.first == id; }), batch.end());
}

Batch Scheduler::step() {
  // Asking for the next batch says that the previous one ran to completion: its pages may now be shared. A pipelined
  // engine schedules ahead of the device, turns this off and confirms each batch itself when it has read its tokens.
  if (auto_commit_)
    while (!pending_commits_.empty()) commit_step();
  pending_commits_.emplace_back();
  Batch b;
  int64_t budget = cfg_.max_num_batched_tokens;
  std::vector<Entry> entries;

  // ---- 1. sequences already running ----
  size_t i = 0;
  while (i < running_.size()) {
    const int64_t id = running_[i];
    Request& r = reqs_.at(id);
    const int64_t pending = static_cast<int64_t>(r.tokens.size()) - r.computed;
    int64_t n = pending == 1 ? 1 : std::min(pending, budget);
    // chunked prefill off: wait for a step with room for the whole run, unless no step ever has it (a preempted
    // sequence recomputes prompt + generated tokens, which may exceed the budget): that run is chunked after all
    if (pending > 1 && !cfg_.enable_chunked_prefill && n < pending && pending <= cfg_.max_num_batched_tokens) n = 0;
    if (n <= 0 || budget <= 0) { ++i; continue; }
    bool self_preempted = false;
    while (!kv_->reserve(id, r.computed + n)) {
      if (!preempt_one(id, &b)) { self_preempted = true; break; }
    }
    if (self_preempted) continue;  // running_[i] is now a different sequence (or the end)
    entries.push_back({id, n});
    budget -= n;
    ++i;
  }

  // ---- 2. admit waiting requests ----
  while (!waiting_.empty() && static_cast<int>(running_.size()) < cfg_.max_num_seqs && budget > 0) {
    const int64_t id = waiting_.front();
    // a sequence preempted in this very step waits for the next one
    if (std::find(b.preempted.begin(), b.preempted.end(), id) != b.preempted.end()) break;
    Request& r = reqs_.at(id);
    if (!kv_->has_sequence(id)) r.computed = kv_->add_sequence(id, r.tokens.data(), static_cast<int64_t>(r.tokens.size()));
    const int64_t pending = static_cast<int64_t>(r.tokens.size()) - r.computed;
    int64_t n = std::min(pending, budget);
    if (!cfg_.enable_chunked_prefill && n < pending && pending <= cfg_.max_num_batched_tokens) break;
    // Admission needs the pages of the whole known sequence, not just this chunk: a request that can
    // start but not finish its prompt would only be preempted again.
    const int64_t need_all = kv_->pages_needed(id, static_cast<int64_t>(r.tokens.size()) + 1);
    if (need_all + cfg_.decode_reserve_pages > kv_->available_pages()) break;
    if (!kv_->reserve(id, r.computed + n)) break;
    waiting_.pop_front();
    running_.push_back(id);
    r.status = SeqStatus::kRunning;
    entries.push_back({id, n});
    budget -= n;
  }

  // ---- 3. flatten: decode sequences first ----
  std::stable_partition(entries.begin(), entries.end(), [](const Entry& e) { return e.n == 1; });
  b.cu_q.push_back(0);
  for (const Entry& e : entries) {
    Request& r = reqs_.at(e.id);
    if (e.n == 1) ++b.num_decode; else ++b.num_prefill;
    emit(r, e.n, &b);
  }
  b.num_tokens = static_cast<int64_t>(b.token_ids.size());
  for (int64_t id : b.seq_ids) b.max_blocks = std::max<int>(b.max_blocks, static_cast<int>(kv_->block_table(id).size()));
  b.block_tables.assign(b.seq_ids.size() * static_cast<size_t>(b.max_blocks), 0);
  for (size_t s = 0; s < b.seq_ids.size(); ++s) {
    const auto& t = kv_->block_table(b.seq_ids[s]);
    std::copy(t.begin(), t.end(), b.block_tables.begin() + s * b.max_blocks);
  }
  if (b.seq_ids.empty()) pending_commits_.pop_back();   // nothing was scheduled: no batch to confirm later
  return b;
}

bool Scheduler::append_token(int64_t id, int32_t token) {
  auto it = reqs_.find(id);
  if (it == reqs_.end()) throw std::invalid_argument("Scheduler::append_token: unknown request");
  Request& r = it->second;
  r.tokens.push_back(token);
  ++r.generated;
  return r.generated >= r.max_new_tokens || static_cast<int64_t>(r.tokens.size()) >= cfg_.max_model_len;
}

bool Scheduler::set_token(int64_t id, int64_t pos, int32_t token) {
  auto it = reqs_.find(id);
  if (it == reqs_.end()) return false;
  Request& r = it->second;
  if (pos < 0 || pos >= static_cast<int64_t>(r.tokens.size())) return false;
  r.tokens[pos] = token;
  return true;
}

int64_t Scheduler::num_tokens(int64_t id) const {
  auto it = reqs_.find(id);
  return it == reqs_.end() ? -1 : static_cast<int64_t>(it->second.tokens.size());
}

void Scheduler::finish(int64_t id) {
  auto it = reqs_.find(id);
  if (it == reqs_.end()) return;
  drop_pending_commit(id);   // a step that was not confirmed leaves no prefix-cache entry behind
  kv_->free_sequence(id);
  running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
  waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
  reqs_.erase(it);
}

}  // namespace engine
}  // namespace b2
