#include "kv_pools.hpp"

#include <algorithm>
#include <set>

namespace cuca {

// ------------------------------------------------------------------ BlockPool
BlockPool::BlockPool(int n_blocks) : held_(n_blocks > 0 ? n_blocks : 0, 0) { reset(); }

void BlockPool::reset() {
  const int n = (int)held_.size();
  free_.resize(n);
  for (int i = 0; i < n; ++i) free_[i] = n - 1 - i;  // page 0 is handed out first
  std::fill(held_.begin(), held_.end(), 0);
}

int BlockPool::alloc() {
  if (free_.empty()) return -1;
  const int b = free_.back();
  free_.pop_back();
  if (held_[b]) return -2;
  held_[b] = 1;
  return b;
}

bool BlockPool::release(int b) {
  if (b < 0 || b >= (int)held_.size() || !held_[b]) return false;
  held_[b] = 0;
  free_.push_back(b);
  return true;
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
  const int keep = blocks_for(length);
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

Status KvPools::check() {
  for (size_t g = 0; g < groups_.size(); ++g) {
    const int n = pools_[g].n_blocks();
    std::vector<int> holders(n, 0);
    for (const SeqBlocks& s : seqs_) {
      if (!s.in_use || s.released) continue;
      for (int b : s.tables[g]) {
        if (b == NO_BLOCK) continue;
        if (b < 0 || b >= n) return fail(BOOKKEEPING, "group " + std::to_string(g) + ": page id " + std::to_string(b) + " is out of range");
        if (++holders[b] > 1) return fail(BOOKKEEPING, "group " + std::to_string(g) + ": page " + std::to_string(b) + " is held twice");
      }
    }
    std::vector<int> on_free(n, 0);
    for (int b : pools_[g].free_list()) {
      if (++on_free[b] > 1) return fail(BOOKKEEPING, "group " + std::to_string(g) + ": a page is on the free list twice");
      if (holders[b]) return fail(BOOKKEEPING, "group " + std::to_string(g) + ": page " + std::to_string(b) + " is free and held");
    }
    for (int b = 0; b < n; ++b)
      if (!on_free[b] && !holders[b]) return fail(BOOKKEEPING, "group " + std::to_string(g) + ": page " + std::to_string(b) + " is lost");
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
