// Paged KV-cache bookkeeping: fixed-size pages, per-sequence block tables, reference counts, and an optional
// prefix cache keyed by a chained hash of whole pages of token ids. Host-only; the device sees block tables.
#include <algorithm>
#include <sstream>
#include <stdexcept>
#include "b2/engine.h"

namespace b2 {
namespace engine {

uint64_t hash_page(uint64_t parent, const int32_t* tokens, int n) {
  // Folded multiply with two odd constants (pi digits), the mixing step of the reference's AHasher
  // (stdlib/src/hashlib/_ahash.mojo:87-202), applied to 64-bit lanes of token pairs.
  constexpr uint64_t kMul = 6364136223846793005ull;
  constexpr uint64_t kPad0 = 0x243f6a8885a308d3ull, kPad1 = 0x13198a2e03707344ull;
  uint64_t h = parent ^ kPad0;
  int i = 0;
  for (; i + 1 < n; i += 2) {
    const uint64_t v = (static_cast<uint64_t>(static_cast<uint32_t>(tokens[i])) << 32) | static_cast<uint32_t>(tokens[i + 1]);
    h = folded_multiply(h ^ v, kMul);
  }
  if (i < n) h = folded_multiply(h ^ static_cast<uint32_t>(tokens[i]), kMul);
  h = folded_multiply(h, kPad1 ^ static_cast<uint64_t>(n));
  const int rot = static_cast<int>(h & 63);
  h = (h << rot) | (h >> ((64 - rot) & 63));
  return h == 0 ? 1 : h;  // 0 is reserved for "not cached"
}

KVCacheManager::KVCacheManager(int64_t num_pages, int page_size, bool enable_prefix_cache)
    : num_pages_(num_pages), page_size_(page_size), prefix_(enable_prefix_cache) {
  if (num_pages <= 0 || page_size <= 0) throw std::invalid_argument("KVCacheManager: num_pages and page_size must be positive");
  refcount_.assign(num_pages, 0);
  page_hash_.assign(num_pages, 0);
  evict_pos_.resize(num_pages);
  in_evictable_.assign(num_pages, 0);
  for (int64_t p = 0; p < num_pages; ++p) free_.push_back(static_cast<int32_t>(p));
}

int32_t KVCacheManager::take_page() {
  if (!free_.empty()) {
    const int32_t p = free_.front();
    free_.pop_front();
    refcount_[p] = 1;
    return p;
  }
  if (!evictable_.empty()) {
    const int32_t p = evictable_.front();
    evictable_.pop_front();
    in_evictable_[p] = 0;
    auto it = cache_.find(page_hash_[p]);
    if (it != cache_.end() && it->second == p) cache_.erase(it);
    page_hash_[p] = 0;
    ++evictions_;
    refcount_[p] = 1;
    return p;
  }
  return -1;
}

void KVCacheManager::release_page(int32_t p) {
  if (--refcount_[p] > 0) return;
  if (page_hash_[p] != 0) {
    evictable_.push_back(p);
    evict_pos_[p] = std::prev(evictable_.end());
    in_evictable_[p] = 1;
  } else {
    free_.push_back(p);
  }
}

int64_t KVCacheManager::pages_needed(int64_t seq_id, int64_t total_tokens) const {
  const int64_t want = (total_tokens + page_size_ - 1) / page_size_;
  auto it = seqs_.find(seq_id);
  const int64_t have = it == seqs_.end() ? 0 : static_cast<int64_t>(it->second.pages.size());
  return std::max<int64_t>(0, want - have);
}

int64_t KVCacheManager::add_sequence(int64_t seq_id, const int32_t* tokens, int64_t n_tokens) {
  if (seqs_.count(seq_id)) throw std::invalid_argument("KVCacheManager: sequence already exists");
  Seq s;
  int64_t matched = 0;
  if (prefix_ && tokens != nullptr) {
    // Never match the whole prompt: at least one token must be computed to produce logits.
    const int64_t max_pages = (n_tokens - 1) / page_size_;
    uint64_t h = 0;
    for (int64_t i = 0; i < max_pages; ++i) {
      ++prefix_queries_;
      h = hash_page(h, tokens + i * page_size_, page_size_);
      auto it = cache_.find(h);
      if (it == cache_.end()) break;
      const int32_t p = it->second;
      if (in_evictable_[p]) {
        evictable_.erase(evict_pos_[p]);
        in_evictable_[p] = 0;
      }
      ++refcount_[p];
      s.pages.push_back(p);
      s.last_hash = h;
      ++matched;
      ++prefix_hits_;
    }
  }
  s.committed_pages = matched;
  s.reserved_tokens = matched * page_size_;
  seqs_.emplace(seq_id, std::move(s));
  return matched * page_size_;
}

bool KVCacheManager::reserve(int64_t seq_id, int64_t total_tokens) {
  auto it = seqs_.find(seq_id);
  if (it == seqs_.end()) throw std::invalid_argument("KVCacheManager::reserve: unknown sequence");
  Seq& s = it->second;
  const int64_t need = pages_needed(seq_id, total_tokens);
  if (need > available_pages()) return false;
  for (int64_t i = 0; i < need; ++i) s.pages.push_back(take_page());
  s.reserved_tokens = std::max(s.reserved_tokens, total_tokens);
  return true;
}

void KVCacheManager::commit(int64_t seq_id, const int32_t* tokens, int64_t n_tokens) {
  if (!prefix_) return;
  auto it = seqs_.find(seq_id);
  if (it == seqs_.end()) return;
  Seq& s = it->second;
  const int64_t full = std::min<int64_t>(n_tokens / page_size_, static_cast<int64_t>(s.pages.size()));
  for (int64_t i = s.committed_pages; i < full; ++i) {
    const uint64_t h = hash_page(s.last_hash, tokens + i * page_size_, page_size_);
    const int32_t p = s.pages[i];
    if (cache_.find(h) == cache_.end() && page_hash_[p] == 0) {
      cache_.emplace(h, p);
      page_hash_[p] = h;
    }
    s.last_hash = h;
    s.committed_pages = i + 1;
  }
}

void KVCacheManager::free_sequence(int64_t seq_id) {
  auto it = seqs_.find(seq_id);
  if (it == seqs_.end()) return;
  // Leaves first, so that eviction (oldest first) drops the end of a cached prefix before its root.
  for (auto p = it->second.pages.rbegin(); p != it->second.pages.rend(); ++p) release_page(*p);
  seqs_.erase(it);
}

bool KVCacheManager::fork(int64_t src, int64_t dst, std::vector<std::pair<int64_t, int64_t>>* copies) {
  auto it = seqs_.find(src);
  if (it == seqs_.end() || seqs_.count(dst)) throw std::invalid_argument("KVCacheManager::fork: bad sequence ids");
  const Seq& a = it->second;
  Seq b;
  b.reserved_tokens = a.reserved_tokens;
  b.committed_pages = a.committed_pages;
  b.last_hash = a.last_hash;
  const bool partial_tail = !a.pages.empty() && (a.reserved_tokens % page_size_ != 0);
  if (partial_tail && available_pages() < 1) return false;
  const size_t shared = a.pages.size() - (partial_tail ? 1 : 0);
  for (size_t i = 0; i < shared; ++i) {
    ++refcount_[a.pages[i]];
    b.pages.push_back(a.pages[i]);
  }
  if (partial_tail) {
    const int32_t np = take_page();
    b.pages.push_back(np);
    if (copies) copies->emplace_back(a.pages.back(), np);
    b.committed_pages = std::min<int64_t>(b.committed_pages, static_cast<int64_t>(shared));
  }
  seqs_.emplace(dst, std::move(b));
  return true;
}

const std::vector<int32_t>& KVCacheManager::block_table(int64_t seq_id) const {
  auto it = seqs_.find(seq_id);
  if (it == seqs_.end()) throw std::invalid_argument("KVCacheManager::block_table: unknown sequence");
  return it->second.pages;
}

int64_t KVCacheManager::slot(int64_t seq_id, int64_t pos) const {
  const auto& pages = block_table(seq_id);
  const int64_t idx = pos / page_size_;
  if (pos < 0 || idx >= static_cast<int64_t>(pages.size())) throw std::out_of_range("KVCacheManager::slot: position not reserved");
  return static_cast<int64_t>(pages[idx]) * page_size_ + pos % page_size_;
}

int64_t KVCacheManager::num_tokens_reserved(int64_t seq_id) const {
  auto it = seqs_.find(seq_id);
  return it == seqs_.end() ? 0 : it->second.reserved_tokens;
}

KVStats KVCacheManager::stats() const {
  KVStats s{};
  s.num_pages = num_pages_;
  s.free_pages = static_cast<int64_t>(free_.size());
  s.cached_pages = static_cast<int64_t>(cache_.size());
  s.prefix_hits = prefix_hits_;
  s.prefix_queries = prefix_queries_;
  s.evictions = evictions_;
  return s;
}

std::string KVCacheManager::check_invariants() const {
  std::vector<int> seen(num_pages_, 0);
  std::vector<int> refs(num_pages_, 0);
  for (int32_t p : free_) seen[p] += 1;
  for (int32_t p : evictable_) seen[p] += 1;
  for (const auto& kv : seqs_)
    for (int32_t p : kv.second.pages) refs[p] += 1;
  std::ostringstream err;
  for (int64_t p = 0; p < num_pages_; ++p) {
    if (refs[p] != refcount_[p]) err << "page " << p << ": refcount " << refcount_[p] << " but " << refs[p] << " owners; ";
    const int places = seen[p] + (refs[p] > 0 ? 1 : 0);
    if (places != 1) err << "page " << p << ": in " << places << " places; ";
    if (seen[p] && refs[p]) err << "page " << p << ": free and referenced; ";
  }
  for (const auto& kv : cache_)
    if (page_hash_[kv.second] != kv.first) err << "cache entry for page " << kv.second << " has stale hash; ";
  return err.str();
}

}  // namespace engine
}  // namespace b2
