// Host runtime of the serving engine: paged KV-cache manager and continuous-batching scheduler.
//
// The reference ships containers, not an engine; the pieces used here follow its library types where they
// fit: the per-request table is an insertion-ordered hash map like `Dict`
// (stdlib/src/collections/dict.mojo:13-30, 352-1060), waiting/running queues and the free-page list are ring
// deques like `Deque` (stdlib/src/collections/deque.mojo:34-1036), and the prefix-cache key is a 64-bit
// folded-multiply hash like `AHasher` (stdlib/src/hashlib/_ahash.mojo:87-202). All of it is plain C++17 with
// no CUDA dependency, so it is unit-tested on CPU.
#pragma once
#include <cstdint>
#include <deque>
#include <list>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace b2 {
namespace engine {

// ---- hashing ------------------------------------------------------------------------------------
inline uint64_t folded_multiply(uint64_t a, uint64_t b) {
  const unsigned __int128 r = static_cast<unsigned __int128>(a) * b;
  return static_cast<uint64_t>(r) ^ static_cast<uint64_t>(r >> 64);
}
// Hash of one page of token ids chained to the hash of everything before it.
uint64_t hash_page(uint64_t parent, const int32_t* tokens, int n);

// ---- KV cache -----------------------------------------------------------------------------------
struct KVStats {
  int64_t num_pages, free_pages, cached_pages, prefix_hits, prefix_queries, evictions;
};

class KVCacheManager {
 public:
  KVCacheManager(int64_t num_pages, int page_size, bool enable_prefix_cache);

  int page_size() const { return page_size_; }
  int64_t num_pages() const { return num_pages_; }
  // Pages that can be handed out right now (free + evictable cached pages).
  int64_t available_pages() const { return static_cast<int64_t>(free_.size() + evictable_.size()); }
  int64_t pages_needed(int64_t seq_id, int64_t total_tokens) const;

  bool has_sequence(int64_t seq_id) const { return seqs_.count(seq_id) != 0; }
  // Create a sequence; with prefix caching on, reuse cached pages matching the longest full-page prefix of
  // `tokens`. Returns the number of tokens whose KV is already present.
  int64_t add_sequence(int64_t seq_id, const int32_t* tokens, int64_t n_tokens);
  // Make sure the sequence owns pages for `total_tokens` positions. False (and no change) if pages run out.
  bool reserve(int64_t seq_id, int64_t total_tokens);
  // Register the sequence's full pages in the prefix cache (call after their KV has been written).
  void commit(int64_t seq_id, const int32_t* tokens, int64_t n_tokens);
  void free_sequence(int64_t seq_id);
  // Share all pages of `src` with a new sequence `dst` (parallel sampling). Last partial page is copied lazily:
  // the (src_page, dst_page) pair to copy is appended to `copies`.
  bool fork(int64_t src, int64_t dst, std::vector<std::pair<int64_t, int64_t>>* copies);

  const std::vector<int32_t>& block_table(int64_t seq_id) const;
  int64_t slot(int64_t seq_id, int64_t pos) const;
  int64_t num_tokens_reserved(int64_t seq_id) const;
  KVStats stats() const;
  // Invariant check used by tests: every page is in exactly one of {free, evictable, referenced}.
  std::string check_invariants() const;

 private:
  struct Seq {
    std::vector<int32_t> pages;
    int64_t reserved_tokens = 0;
    int64_t committed_pages = 0;
    uint64_t last_hash = 0;
  };
  int32_t take_page();
  void release_page(int32_t page);

  int64_t num_pages_;
  int page_size_;
  bool prefix_;
  std::deque<int32_t> free_;
  std::list<int32_t> evictable_;               // cached pages with refcount 0, oldest first
  std::vector<std::list<int32_t>::iterator> evict_pos_;
  std::vector<uint8_t> in_evictable_;
  std::vector<int32_t> refcount_;
  std::vector<uint64_t> page_hash_;            // 0 = not cached
  std::unordered_map<uint64_t, int32_t> cache_;  // hash -> page
  std::unordered_map<int64_t, Seq> seqs_;
  int64_t prefix_hits_ = 0, prefix_queries_ = 0, evictions_ = 0;
};

// ---- scheduler ----------------------------------------------------------------------------------
enum class SeqStatus : int32_t { kWaiting = 0, kRunning = 1, kFinished = 2 };

struct SchedulerConfig {
  int max_num_seqs = 256;
  int max_num_batched_tokens = 8192;  // per-iteration token budget (decode tokens + prefill chunk tokens)
  int max_model_len = 8192;
  bool enable_chunked_prefill = true;
  int decode_reserve_pages = 0;       // pages kept back from admission so running sequences can grow
};

struct Request {
  int64_t id = 0;
  std::vector<int32_t> tokens;  // prompt + generated
  int64_t prompt_len = 0;
  int64_t max_new_tokens = 0;
  int64_t computed = 0;         // tokens whose KV is in the cache
  int64_t generated = 0;
  double arrival = 0.0;
  SeqStatus status = SeqStatus::kWaiting;
  int64_t preemptions = 0;
};

// One engine iteration, flattened for the device: decode sequences first, then prefill chunks.
struct Batch {
  std::vector<int64_t> seq_ids;
  std::vector<int32_t> q_lens;      // tokens processed this step per sequence
  std::vector<int32_t> ctx_lens;    // context length after this step per sequence
  std::vector<int32_t> cu_q;        // [B + 1] offsets into the flat token arrays
  std::vector<int64_t> token_ids;   // [T]
  std::vector<int32_t> positions;   // [T]
  std::vector<int64_t> slots;       // [T] physical KV slots
  std::vector<int32_t> block_tables;  // [B, max_blocks], padded with 0
  std::vector<int32_t> sample_rows; // indices (into the flat token arrays) whose logits are sampled
  std::vector<int64_t> sample_seq_ids;
  int max_blocks = 0;
  int num_decode = 0;               // first num_decode sequences have q_len == 1 and full context
  int num_prefill = 0;
  int max_q_len = 0;
  int64_t num_tokens = 0;
  std::vector<int64_t> preempted;   // sequences pushed back to the waiting queue this step
};

class Scheduler {
 public:
  Scheduler(SchedulerConfig cfg, KVCacheManager* kv);

  void add_request(int64_t id, const int32_t* prompt, int64_t prompt_len, int64_t max_new_tokens, double arrival);
  // Build the next batch; empty batch when nothing is runnable.
  Batch step();
  // Record the token sampled for a sequence after the step. Returns true when the sequence hit
  // max_new_tokens (the caller may also finish it earlier, e.g. on EOS or a stop string).
  bool append_token(int64_t id, int32_t token);
  // Pipelined engines append a placeholder (-1) when a step is launched and fill in the sampled token one step later:
  // `set_token` overwrites position `pos` of the sequence (false if the request is gone or `pos` is out of range);
  // `num_tokens` is the current length (prompt + generated, placeholders included; -1 for an unknown request).
  bool set_token(int64_t id, int64_t pos, int32_t token);
  int64_t num_tokens(int64_t id) const;
  void finish(int64_t id);
  void abort(int64_t id) { finish(id); }
  // Register the full pages written by the last batch in the prefix cache. The engine calls it when the step has
  // completed; `step()` calls it for the previous batch as well. A sequence that is finished, aborted or preempted
  // before that keeps no entry for the unconfirmed step, so a failed step cannot leave half-written pages shared.
  void commit_step();
  // With auto-commit off, `step()` no longer confirms earlier batches: every `commit_step()` confirms the oldest
  // unconfirmed batch, in launch order (engines that schedule one step ahead of the device).
  void set_auto_commit(bool on) { auto_commit_ = on; }

  bool has_unfinished() const { return !waiting_.empty() || !running_.empty(); }
  int64_t num_waiting() const { return static_cast<int64_t>(waiting_.size()); }
  int64_t num_running() const { return static_cast<int64_t>(running_.size()); }
  const Request* request(int64_t id) const;
  int64_t total_preemptions() const { return total_preemptions_; }

 private:
  bool preempt_one(int64_t keep_id, Batch* b);
  void emit(Request& r, int64_t n_tokens, Batch* b);
  void drop_pending_commit(int64_t id);

  SchedulerConfig cfg_;
  KVCacheManager* kv_;
  std::unordered_map<int64_t, Request> reqs_;
  std::deque<int64_t> waiting_;
  std::vector<int64_t> running_;  // admission order
  int64_t total_preemptions_ = 0;
  std::deque<std::vector<std::pair<int64_t, int64_t>>> pending_commits_;  // per unconfirmed batch: (sequence, tokens computed)
  bool auto_commit_ = true;
};

}  // namespace engine
}  // namespace b2
