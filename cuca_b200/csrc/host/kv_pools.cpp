#include "kv_pools.hpp"

#include <algorithm>
#include <set>

namespace cuca {

// FNV-1a over the previous hash and the ids of one page (src/provider/local/model/paged.rs:257-272).
uint64_t chain_hash(uint64_t prev, const int* ids, int n) {
  const uint64_t prime = 0x00000100000001b3ull;
  uint64_t h = 0xcbf29ce484222325ull;
  for (int i = 0; i < 8; ++i) h = (h ^ ((prev >> (8 * i)) & 0xff)) * prime;
  for (int k = 0; k < n; ++k) {
    const uint32_t id = (uint32_t)ids[k];
    for (int i = 0; i < 4; ++i) h = (h ^ ((id >> (8 * i)) & 0xff)) * prime;
  }
  return h;
}

// ------------------------------------------------------------------ BlockPool
BlockPool::BlockPool(int n_blocks) : refcount_(n_blocks > 0 ? n_blocks : 0, 0) { reset(); }

void BlockPool::reset() {
  const int n = (int)refcount_.size();
  free_.resize(n);
  for (int i = 0; i < n; ++i) free_[i] = n - 1 - i;  // page 0 is handed out first
  std::fill(refcount_.begin(), refcount_.end(), 0);
  named_.assign(n, 0);
  key_.assign(n, BlockKey());
  lru_.clear();
  stamp_.assign(n, 0);
  next_stamp_ = 1;
  cached_ = 0;
  by_hash_.clear();
}

int BlockPool::alloc() {
  if (!free_.empty()) {
    const int b = free_.back();
    free_.pop_back();
    if (refcount_[b] != 0) return -2;
    refcount_[b] = 1;
    return b;
  }
  while (!lru_.empty()) {
    const std::pair<int, uint64_t> e = lru_.front();
    lru_.pop_front();
    const int b = e.first;
    if (stamp_[b] != e.second) continue;  // a stale entry: the page was taken out of the cache meanwhile
    stamp_[b] = 0;
    --cached_;
    if (named_[b]) {
      auto it = by_hash_.find(key_[b].hash);
      if (it != by_hash_.end() && it->second == b) by_hash_.erase(it);
      named_[b] = 0;
      key_[b] = BlockKey();
    }
    refcount_[b] = 1;
    return b;
  }
  return -1;
}

bool BlockPool::release(int b) {
  if (b < 0 || b >= (int)refcount_.size() || refcount_[b] == 0) return false;
  if (--refcount_[b] > 0) return true;
  if (named_[b]) {
    stamp_[b] = next_stamp_;
    lru_.emplace_back(b, next_stamp_);
    ++next_stamp_;
    ++cached_;
  } else {
    free_.push_back(b);
  }
  return true;
}

bool BlockPool::register_key(int b, const BlockKey& key) {
  if (b < 0 || b >= (int)refcount_.size() || refcount_[b] == 0 || named_[b] || by_hash_.count(key.hash)) return false;
  named_[b] = 1;
  key_[b] = key;
  by_hash_[key.hash] = b;
  return true;
}

bool BlockPool::holds(const BlockKey& key) const {
  auto it = by_hash_.find(key.hash);
  return it != by_hash_.end() && named_[it->second] && key_[it->second] == key;
}

int BlockPool::lookup(const BlockKey& key) {
  if (!holds(key)) return -1;
  const int b = by_hash_[key.hash];
  if (refcount_[b] == 0) {  // out of the cache
    stamp_[b] = 0;
    --cached_;
  }
  ++refcount_[b];
  return b;
}

// ------------------------------------------------------------------ KvPools
KvPools::KvPools(const std::vector<Group>& groups, int block_size) : groups_(groups), block_size_(block_size) {
  for (const Group& g : groups_) pools_.emplace_back(g.n_blocks);
}

int KvPools::new_seq() {
  int h;
  if (!spare_.empty()) {
    h = spare_.back();
    spare_.pop_back();
  } else {
    h = (int)seqs_.size();
    seqs_.emplace_back();
  }
  SeqBlocks& s = seqs_[h];
  s.tables.assign(groups_.size(), {});
  s.length = 0;
  s.released = false;
  s.in_use = true;
  s.first_live.assign(groups_.size(), 0);
  s.dirty_from.assign(groups_.size(), 0);
  s.chain.clear();
  ++live_;
  return h;
}

SeqBlocks* KvPools::seq(int handle) {
  if (handle < 0 || handle >= (int)seqs_.size() || !seqs_[handle].in_use) return nullptr;
  return &seqs_[handle];
}

void KvPools::drop_seq(int handle) {
  SeqBlocks* s = seq(handle);
  if (!s) return;
  if (!s->released) release(handle);
  s->in_use = false;
  spare_.push_back(handle);
}

void KvPools::owed(int handle, int tokens, int* out) {
  const int need = blocks_for(tokens);
  SeqBlocks* s = handle >= 0 ? seq(handle) : nullptr;
  for (size_t g = 0; g < groups_.size(); ++g) {
    const int have = s ? (int)s->tables[g].size() : 0;
    out[g] = need > have ? need - have : 0;
  }
}

bool KvPools::can_give(const int* owed) const {
  for (size_t g = 0; g < groups_.size(); ++g)
    if (pools_[g].free_count() < owed[g]) return false;
  return true;
}

Status KvPools::reserve(int handle, int upto) {
  SeqBlocks* s = seq(handle);
  if (!s) return fail(BOOKKEEPING, "reserve on an unknown request");
  if (s->released) return fail(BOOKKEEPING, "reserve on a released request");
  std::vector<int> need(groups_.size());
  owed(handle, upto, need.data());
  if (!can_give(need.data())) return fail(EXHAUSTED, "the K/V page pool is exhausted");
  for (size_t g = 0; g < groups_.size(); ++g)
    for (int i = 0; i < need[g]; ++i) {
      const int b = pools_[g].alloc();
      if (b < 0) return fail(BOOKKEEPING, "a page was on the free list while held");
      s->tables[g].push_back(b);
    }
  return OK;
}

int KvPools::release_window(int handle) {
  SeqBlocks* s = seq(handle);
  if (!s || s->released) return 0;
  int n = 0;
  for (size_t g = 0; g < groups_.size(); ++g) {
    const int window = groups_[g].window;
    if (window < 0) continue;
    // the next query sits at position `length` and sees keys >= length - (window - 1)
    const int first_needed = std::max(0, s->length - (window - 1));
    std::vector<int>& table = s->tables[g];
    const int upto = std::min(first_needed / block_size_, (int)table.size());
    for (int i = s->first_live[g]; i < upto; ++i) {
      if (table[i] == NO_BLOCK) continue;
      if (!pools_[g].release(table[i])) {
        fail(BOOKKEEPING, "page " + std::to_string(table[i]) + " is freed but not held");
        return -1;
      }
      table[i] = NO_BLOCK;
      ++n;
    }
    s->first_live[g] = std::max(s->first_live[g], upto);
  }
  return n;
}

Status KvPools::truncate(int handle, int length) {
  SeqBlocks* s = seq(handle);
  if (!s) return fail(BOOKKEEPING, "truncate on an unknown request");
  length = std::min(length, s->length);
  if (length < s->length && length % block_size_ != 0) {
    // a named page is read-only: when the new end falls into one, only whole pages are kept
    const int tail = length / block_size_;
    for (size_t g = 0; g < groups_.size(); ++g) {
      const std::vector<int>& table = s->tables[g];
      if (tail < (int)table.size() && table[tail] != NO_BLOCK && pools_[g].is_named(table[tail])) length = tail * block_size_;
    }
  }
  const int keep = blocks_for(length);
  if ((int)s->chain.size() > length / block_size_) s->chain.resize(length / block_size_);
  for (size_t g = 0; g < groups_.size(); ++g) {
    std::vector<int>& table = s->tables[g];
    while ((int)table.size() > keep) {
      const int b = table.back();
      table.pop_back();
      if (b != NO_BLOCK && !pools_[g].release(b)) return fail(BOOKKEEPING, "page " + std::to_string(b) + " is freed but not held");
    }
    s->dirty_from[g] = std::min(s->dirty_from[g], (int)table.size());
  }
  s->length = std::min(s->length, length);
  return OK;
}

Status KvPools::release(int handle) {
  SeqBlocks* s = seq(handle);
  if (!s) return fail(BOOKKEEPING, "release of an unknown request");
  if (s->released) return fail(BOOKKEEPING, "a request's pages are released twice");
  for (size_t g = 0; g < groups_.size(); ++g) {
    for (int b : s->tables[g])
      if (b != NO_BLOCK && !pools_[g].release(b)) return fail(BOOKKEEPING, "page " + std::to_string(b) + " is freed but not held");
    s->tables[g].clear();
  }
  s->released = true;
  s->chain.clear();
  --live_;
  return OK;
}

void KvPools::reset() {
  for (BlockPool& p : pools_) p.reset();
  for (SeqBlocks& s : seqs_) {
    if (!s.in_use || s.released) continue;
    s.released = true;
    for (auto& t : s.tables) t.clear();
  }
  live_ = 0;
}

Status KvPools::publish(int handle, const int* ids, int n) {
  SeqBlocks* s = seq(handle);
  if (!s || s->released) return fail(BOOKKEEPING, "publish on a request without pages");
  const int full = std::min(s->length, n) / block_size_;
  while ((int)s->chain.size() < full) {
    const int i = (int)s->chain.size();
    s->chain.push_back(chain_hash(i ? s->chain[i - 1] : 0, ids + (size_t)i * block_size_, block_size_));
  }
  for (size_t g = 0; g < groups_.size(); ++g) {
    const std::vector<int>& table = s->tables[g];
    for (int i = 0; i < (int)table.size() && i < (int)s->chain.size(); ++i) {
      if (table[i] == NO_BLOCK || pools_[g].is_named(table[i])) continue;
      BlockKey key;
      key.hash = s->chain[i];
      key.parent = i ? s->chain[i - 1] : 0;
      key.ids.assign(ids + (size_t)i * block_size_, ids + (size_t)(i + 1) * block_size_);
      pools_[g].register_key(table[i], key);
    }
  }
  return OK;
}

Status KvPools::finish(int handle, const int* ids, int n) {
  const Status st = publish(handle, ids, n);
  if (st != OK) return st;
  return release(handle);
}

int KvPools::new_seq_with_prefix(const int* prompt, int n) {
  const int max_blocks = n > 0 ? (n - 1) / block_size_ : 0;  // the last prompt token is always computed
  std::vector<BlockKey> keys(max_blocks);
  uint64_t prev = 0;
  for (int i = 0; i < max_blocks; ++i) {
    keys[i].parent = prev;
    keys[i].hash = chain_hash(prev, prompt + (size_t)i * block_size_, block_size_);
    keys[i].ids.assign(prompt + (size_t)i * block_size_, prompt + (size_t)(i + 1) * block_size_);
    prev = keys[i].hash;
  }
  // the longest chain every full-attention group holds
  int nb = max_blocks;
  for (size_t g = 0; g < groups_.size(); ++g) {
    if (groups_[g].window >= 0) continue;
    int have = 0;
    while (have < nb && pools_[g].holds(keys[have])) ++have;
    nb = have;
  }
  // a windowed group must hold the pages of the window before the prefix's end
  auto first_needed = [&](int window, int blocks) { return std::max(0, blocks * block_size_ - (window - 1)) / block_size_; };
  while (nb > 0) {
    bool ok = true;
    for (size_t g = 0; g < groups_.size() && ok; ++g) {
      if (groups_[g].window < 0) continue;
      for (int i = first_needed(groups_[g].window, nb); i < nb && ok; ++i) ok = pools_[g].holds(keys[i]);
    }
    if (ok) break;
    --nb;
  }
  const int h = new_seq();
  SeqBlocks& s = seqs_[h];
  for (size_t g = 0; g < groups_.size(); ++g) {
    const int from = groups_[g].window >= 0 ? first_needed(groups_[g].window, nb) : 0;
    s.tables[g].assign(from, NO_BLOCK);
    for (int i = from; i < nb; ++i) {
      const int b = pools_[g].lookup(keys[i]);
      if (b < 0) { nb = i; break; }  // cannot happen after the checks above; never hand out a hole
      s.tables[g].push_back(b);
    }
    s.first_live[g] = from;
  }
  for (size_t g = 0; g < groups_.size(); ++g)  // (only after a miss above: keep the groups equally long)
    while ((int)s.tables[g].size() > nb) {
      const int b = s.tables[g].back();
      s.tables[g].pop_back();
      if (b != NO_BLOCK) pools_[g].release(b);
    }
  s.length = nb * block_size_;
  s.chain.clear();
  for (int i = 0; i < nb; ++i) s.chain.push_back(keys[i].hash);
  return h;
}

Status KvPools::check() {
  for (size_t g = 0; g < groups_.size(); ++g) {
    const int n = pools_[g].n_blocks();
    std::vector<int> holders(n, 0);
    for (const SeqBlocks& s : seqs_) {
      if (!s.in_use || s.released) continue;
      for (int b : s.tables[g]) {
        if (b == NO_BLOCK) continue;
        if (b < 0 || b >= n) return fail(BOOKKEEPING, "group " + std::to_string(g) + ": page id " + std::to_string(b) + " is out of range");
        ++holders[b];
        if (holders[b] > 1 && !pools_[g].is_named(b))
          return fail(BOOKKEEPING, "group " + std::to_string(g) + ": page " + std::to_string(b) + " is held twice");
      }
    }
    std::vector<int> on_free(n, 0);
    for (int b : pools_[g].free_list()) {
      if (++on_free[b] > 1) return fail(BOOKKEEPING, "group " + std::to_string(g) + ": a page is on the free list twice");
      if (holders[b]) return fail(BOOKKEEPING, "group " + std::to_string(g) + ": page " + std::to_string(b) + " is free and held");
    }
    for (int b = 0; b < n; ++b) {
      if (holders[b] != pools_[g].refcount(b))
        return fail(BOOKKEEPING, "group " + std::to_string(g) + ": page " + std::to_string(b) + " has " + std::to_string(pools_[g].refcount(b)) +
                                     " references but " + std::to_string(holders[b]) + " tables name it");
      const bool cached = pools_[g].in_cache(b);
      if (cached && (holders[b] || on_free[b])) return fail(BOOKKEEPING, "group " + std::to_string(g) + ": page " + std::to_string(b) + " is cached and also held or free");
      if (!on_free[b] && !holders[b] && !cached) return fail(BOOKKEEPING, "group " + std::to_string(g) + ": page " + std::to_string(b) + " is lost");
    }
  }
  return OK;
}

// ------------------------------------------------------------------ StateSlots
StateSlots::StateSlots(int n) : held_(n > 0 ? n : 0, 0) { reset(); }

void StateSlots::reset() {
  const int n = (int)held_.size();
  free_.resize(n);
  for (int i = 0; i < n; ++i) free_[i] = i;  // the highest slot is handed out first
  std::fill(held_.begin(), held_.end(), 0);
}

int StateSlots::alloc() {
  if (free_.empty()) return -1;
  const int s = free_.back();
  free_.pop_back();
  held_[s] = 1;
  return s;
}

bool StateSlots::release(int s) {
  if (s < 0 || s >= (int)held_.size() || !held_[s]) return false;
  held_[s] = 0;
  free_.push_back(s);
  return true;
}

}  // namespace cuca
