#include "kv_pools.hpp"

#include <algorithm>

namespace cuca {

// FNV-1a over the previous page's hash (eight bytes, low first) and then the ids of the page (four bytes each,
// low first): the hash the reference names its pages by (src/provider/local/model/paged.rs:257-272).
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
BlockPool::BlockPool(int n_blocks) : refs_(n_blocks > 0 ? n_blocks : 0, 0) { reset(); }

void BlockPool::reset() {
  const int n = n_blocks();
  std::fill(refs_.begin(), refs_.end(), 0);
  named_.assign(n, 0);
  link_.assign(n, -1);
  back_.assign(n, -1);
  hash_.assign(n, 0);
  parent_.assign(n, 0);
  ids_.assign(n, {});
  size_t cap = 8;
  while (cap < 2 * (size_t)n) cap <<= 1;  // at most half full, so probes stay short
  table_.assign(cap, -1);
  free_top_ = -1;
  for (int b = n - 1; b >= 0; --b) { link_[b] = free_top_; free_top_ = b; }  // page 0 on top
  n_free_ = n;
  oldest_ = newest_ = -1;
  n_cached_ = 0;
}

size_t BlockPool::slot_of(uint64_t hash, uint64_t parent) const {
  uint64_t x = hash ^ (parent * 0x9E3779B97F4A7C15ull);
  x ^= x >> 29;
  return (size_t)x & (table_.size() - 1);
}

int BlockPool::find(const PageName& name) const {
  for (size_t i = slot_of(name.hash, name.parent);; i = (i + 1) & (table_.size() - 1)) {
    const int b = table_[i];
    if (b < 0) return -1;
    if (hash_[b] == name.hash && parent_[b] == name.parent) {
      const std::vector<int>& ids = ids_[b];
      if ((int)ids.size() == name.n_ids && std::equal(ids.begin(), ids.end(), name.ids)) return b;
      return -1;  // same hashes, other tokens: the name belongs to the page that took it first
    }
  }
}

// Takes the page's entry out of the name table, closing the gap so that later entries of the same run of probes
// stay reachable (backward-shift deletion: no tombstones).
void BlockPool::forget_name(int b) {
  const size_t mask = table_.size() - 1;
  size_t i = slot_of(hash_[b], parent_[b]);
  while (table_[i] != b) {
    if (table_[i] < 0) { named_[b] = 0; ids_[b].clear(); return; }  // (not reachable: a named page is in the table)
    i = (i + 1) & mask;
  }
  size_t hole = i;
  for (size_t j = (i + 1) & mask; table_[j] >= 0; j = (j + 1) & mask) {
    const size_t home = slot_of(hash_[table_[j]], parent_[table_[j]]);
    // entry j may move into the hole unless its home lies cyclically in (hole, j]
    const bool stays = hole <= j ? (home > hole && home <= j) : (home > hole || home <= j);
    if (!stays) { table_[hole] = table_[j]; hole = j; }
  }
  table_[hole] = -1;
  named_[b] = 0;
  ids_[b].clear();
}

void BlockPool::unlink_cached(int b) {
  const int older = back_[b], newer = link_[b];
  if (older >= 0) link_[older] = newer; else oldest_ = newer;
  if (newer >= 0) back_[newer] = older; else newest_ = older;
  link_[b] = back_[b] = -1;
  --n_cached_;
}

int BlockPool::alloc() {
  int b;
  if (free_top_ >= 0) {
    b = free_top_;
    if (refs_[b] != 0 || named_[b]) return -2;  // a held or cached page on the free stack: the books are wrong
    free_top_ = link_[b];
    link_[b] = -1;
    --n_free_;
  } else if (oldest_ >= 0) {
    b = oldest_;
    unlink_cached(b);
    forget_name(b);  // whoever gets the page writes new tokens into it
  } else {
    return -1;
  }
  refs_[b] = 1;
  return b;
}

bool BlockPool::release(int b) {
  if (b < 0 || b >= n_blocks() || refs_[b] == 0) return false;
  if (--refs_[b] > 0) return true;
  if (named_[b]) {  // keeps its tokens and its name until an allocation needs the page
    back_[b] = newest_;
    link_[b] = -1;
    if (newest_ >= 0) link_[newest_] = b; else oldest_ = b;
    newest_ = b;
    ++n_cached_;
  } else {
    link_[b] = free_top_;
    free_top_ = b;
    ++n_free_;
  }
  return true;
}

bool BlockPool::give_name(int b, const PageName& name) {
  if (b < 0 || b >= n_blocks() || refs_[b] == 0 || named_[b]) return false;
  const size_t mask = table_.size() - 1;
  size_t i = slot_of(name.hash, name.parent);
  for (; table_[i] >= 0; i = (i + 1) & mask)
    if (hash_[table_[i]] == name.hash && parent_[table_[i]] == name.parent) return false;  // the name is taken
  table_[i] = b;
  hash_[b] = name.hash;
  parent_[b] = name.parent;
  ids_[b].assign(name.ids, name.ids + name.n_ids);
  named_[b] = 1;
  return true;
}

int BlockPool::take(const PageName& name) {
  const int b = find(name);
  if (b < 0) return -1;
  if (refs_[b] == 0) unlink_cached(b);
  ++refs_[b];
  return b;
}

bool BlockPool::walk_free(std::vector<int>& seen) const {
  int steps = 0;
  for (int b = free_top_; b >= 0; b = link_[b]) {
    if (++steps > n_blocks() || !is_free(b)) return false;
    ++seen[b];
  }
  return steps == n_free_;
}

bool BlockPool::walk_cached(std::vector<int>& seen) const {
  int steps = 0, prev = -1;
  for (int b = oldest_; b >= 0; prev = b, b = link_[b]) {
    if (++steps > n_blocks() || !is_cached(b) || back_[b] != prev) return false;
    ++seen[b];
  }
  return steps == n_cached_ && prev == newest_;
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

// The names of a token sequence's whole pages, one after the other: each page's hash chains from the one before.
namespace {
struct NameWalker {
  const int* ids;
  int page_tokens;
  uint64_t prev = 0;
  int index = 0;
  PageName next() {
    PageName nm;
    nm.parent = prev;
    nm.ids = ids + (size_t)index * page_tokens;
    nm.n_ids = page_tokens;
    nm.hash = chain_hash(prev, nm.ids, page_tokens);
    prev = nm.hash;
    ++index;
    return nm;
  }
};
}  // namespace

Status KvPools::publish(int handle, const int* ids, int n) {
  SeqBlocks* s = seq(handle);
  if (!s || s->released) return fail(BOOKKEEPING, "publish on a request without pages");
  const int whole = std::min(s->length, n) / block_size_;  // pages that are full and whose tokens are known
  NameWalker walk{ids, block_size_};
  for (int i = 0; i < whole; ++i) {
    if (i < (int)s->chain.size()) {  // named at an earlier call: only move the walker on
      walk.prev = s->chain[i];
      walk.index = i + 1;
      continue;
    }
    const PageName nm = walk.next();
    s->chain.push_back(nm.hash);
    for (size_t g = 0; g < groups_.size(); ++g) {
      const std::vector<int>& table = s->tables[g];
      if (i < (int)table.size() && table[i] != NO_BLOCK) pools_[g].give_name(table[i], nm);  // refused if taken
    }
  }
  return OK;
}

Status KvPools::finish(int handle, const int* ids, int n) {
  const Status st = publish(handle, ids, n);
  return st == OK ? release(handle) : st;
}

int KvPools::new_seq_with_prefix(const int* prompt, int n) {
  // Whole pages strictly below the last prompt token: that token's logits are what the request is after, so it
  // is always computed.
  const int limit = n > 0 ? (n - 1) / block_size_ : 0;
  std::vector<PageName> names;
  names.reserve(limit);
  NameWalker walk{prompt, block_size_};
  // as deep as every group that keeps all keys can follow
  while ((int)names.size() < limit) {
    const PageName nm = walk.next();
    bool everywhere = true;
    for (size_t g = 0; g < groups_.size() && everywhere; ++g)
      if (groups_[g].window < 0) everywhere = pools_[g].holds(nm);
    if (!everywhere) break;
    names.push_back(nm);
  }
  // a windowed group needs only the pages its window still reaches from the prefix's end; pages before that
  // may be gone. Shrink the prefix until every windowed group has the tail it needs.
  auto tail_begin = [&](int g, int depth) {
    return std::max(0, depth * block_size_ - (groups_[g].window - 1)) / block_size_;
  };
  int depth = (int)names.size();
  for (; depth > 0; --depth) {
    bool tails = true;
    for (size_t g = 0; g < groups_.size() && tails; ++g) {
      if (groups_[g].window < 0) continue;
      for (int i = tail_begin((int)g, depth); i < depth && tails; ++i) tails = pools_[g].holds(names[i]);
    }
    if (tails) break;
  }
  const int h = new_seq();
  SeqBlocks& s = seqs_[h];
  for (size_t g = 0; g < groups_.size(); ++g) {
    const int from = groups_[g].window >= 0 ? tail_begin((int)g, depth) : 0;
    s.tables[g].assign(from, NO_BLOCK);
    for (int i = from; i < depth; ++i) s.tables[g].push_back(pools_[g].take(names[i]));  // found above: never -1
    s.first_live[g] = from;
  }
  s.length = depth * block_size_;
  for (int i = 0; i < depth; ++i) s.chain.push_back(names[i].hash);
  return h;
}

Status KvPools::check() {
  for (size_t g = 0; g < groups_.size(); ++g) {
    const BlockPool& pool = pools_[g];
    const int n = pool.n_blocks();
    const std::string where = "group " + std::to_string(g) + ": ";
    std::vector<int> holders(n, 0);
    for (const SeqBlocks& s : seqs_) {
      if (!s.in_use || s.released) continue;
      for (int b : s.tables[g]) {
        if (b == NO_BLOCK) continue;
        if (b < 0 || b >= n) return fail(BOOKKEEPING, where + "page id " + std::to_string(b) + " is out of range");
        if (++holders[b] > 1 && !pool.is_named(b))
          return fail(BOOKKEEPING, where + "page " + std::to_string(b) + " is held twice");
      }
    }
    std::vector<int> on_free(n, 0), in_cache(n, 0);
    if (!pool.walk_free(on_free)) return fail(BOOKKEEPING, where + "the free pages' links are broken, or a page that is held or cached is among them");
    if (!pool.walk_cached(in_cache)) return fail(BOOKKEEPING, where + "the cached pages' links are broken, or a page that is held or free is among them");
    for (int b = 0; b < n; ++b) {
      const std::string page = where + "page " + std::to_string(b);
      if (on_free[b] > 1) return fail(BOOKKEEPING, page + " is on the free list twice");
      if (on_free[b] && holders[b]) return fail(BOOKKEEPING, page + " is free and held");
      if (holders[b] != pool.refcount(b))
        return fail(BOOKKEEPING, page + " has " + std::to_string(pool.refcount(b)) + " references but " +
                                     std::to_string(holders[b]) + " tables name it");
      if (in_cache[b] && (holders[b] || on_free[b])) return fail(BOOKKEEPING, page + " is cached and also held or free");
      if (!on_free[b] && !holders[b] && !in_cache[b]) return fail(BOOKKEEPING, page + " is lost");
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
