// Host-side bookkeeping of the paged key/value cache: which request holds which page.
//
// A page (block) is `block_size` consecutive positions of one request, for every cache of a group; layers whose
// mixers have equal needs share a group, each group has a pool of its own, and each request has one block table
// per group (src/provider/local/model/paged.rs:6-16,52-103,344-489 of the reference). Pages go back to the pool
// when a request ends and, in a windowed group, as soon as the window has passed them (model/paged.rs:736-761).
// No device memory lives here: the page ids index slabs that the Python side allocates.
//
// Prefix store (model/paged.rs:18-35,257-321,344-480,831-928): a full page is named by a hash chain over the
// token ids it holds (FNV-1a over the previous page's hash, then the page's ids; the first page chains from 0), so
// two requests with the same token prefix name the same pages. `publish` files a request's full pages under
// their names; a named page whose last reference goes stays in the pool as *cached* (least recently used first
// out) and is what an allocation takes when no free page is left. `lookup` finds the longest page-aligned prefix
// of a prompt whose pages every group still holds, at most prompt - 1 positions, and takes a reference to each.
// A name is the hash, the parent's hash and the ids themselves, so a collision of hashes never shares pages.
// A named page is read-only: a hit covers whole pages below the prompt's last token, and the request appends
// after them.
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

namespace cuca {

constexpr int NO_BLOCK = -1;  // a table entry whose page was given back (behind a window)

uint64_t chain_hash(uint64_t prev, const int* ids, int n);

// What names a full page: its chain hash, the hash of the page before it, and its token ids.
struct BlockKey {
  uint64_t hash = 0, parent = 0;
  std::vector<int> ids;
  bool operator==(const BlockKey& o) const { return hash == o.hash && parent == o.parent && ids == o.ids; }
};

// One group's pages: free list (popped from the back, as the reference's), reference counts, names, and the
// least-recently-used order of unreferenced named pages.
class BlockPool {
 public:
  explicit BlockPool(int n_blocks);
  int n_blocks() const { return (int)refcount_.size(); }
  int free_count() const { return (int)free_.size() + cached_; }  // what allocations can still get
  int cached_count() const { return cached_; }
  int alloc();            // a page with one reference: a free one, else the least recently used cached one; -1: none
  bool release(int b);    // drops one reference; false: the page has none (freed twice, or out of range)
  bool register_key(int b, const BlockKey& key);  // false: already named, or the name is taken
  bool holds(const BlockKey& key) const;
  int lookup(const BlockKey& key);                // takes a reference; -1 unless holds(key)
  bool is_named(int b) const { return named_[b] != 0; }
  int refcount(int b) const { return refcount_[b]; }
  void reset();
  const std::vector<int>& free_list() const { return free_; }
  bool in_cache(int b) const { return stamp_[b] != 0; }

 private:
  std::vector<int> free_;
  std::vector<int> refcount_;
  std::vector<char> named_;
  std::vector<BlockKey> key_;
  std::deque<std::pair<int, uint64_t>> lru_;  // (page, stamp): an entry is live while the page's stamp equals it
  std::vector<uint64_t> stamp_;               // 0: not in the cache
  uint64_t next_stamp_ = 1;
  int cached_ = 0;
  std::unordered_map<uint64_t, int> by_hash_;
};

struct Group {
  int n_blocks;
  int window;  // positions a query of this group sees, itself included; < 0: all
};

// One request's block tables (one per group) and how many positions it has cached.
struct SeqBlocks {
  std::vector<std::vector<int>> tables;
  int length = 0;
  bool released = false;
  bool in_use = false;              // the record belongs to a live handle
  std::vector<int> first_live;      // per group: index of the first table entry still held
  std::vector<int> dirty_from;      // per group: table entries from here on are not yet on the device
  std::vector<uint64_t> chain;      // chain hashes of the full pages named so far
};

enum Status { OK = 0, EXHAUSTED = 1, BOOKKEEPING = 2, INVALID = 3, TOO_SMALL = 4 };

class KvPools {
 public:
  KvPools(const std::vector<Group>& groups, int block_size);
  int n_groups() const { return (int)groups_.size(); }
  int block_size() const { return block_size_; }
  const Group& group(int g) const { return groups_[g]; }
  BlockPool& pool(int g) { return pools_[g]; }

  int new_seq();                       // a handle
  void drop_seq(int seq);              // the handle's owner is gone: pages still held go back, the record is reused
  SeqBlocks* seq(int handle);          // nullptr for a handle that is not in use
  int blocks_for(int tokens) const { return (tokens + block_size_ - 1) / block_size_; }
  void owed(int seq, int tokens, int* out);      // seq < 0: a request that holds nothing yet
  bool can_give(const int* owed) const;
  Status reserve(int seq, int upto);             // all or nothing
  int release_window(int seq);                   // pages given back, or -1 on a bookkeeping error
  Status truncate(int seq, int length);
  Status release(int seq);
  // Name every full page of the request (its first `length` positions hold `ids`) so that later prompts find them.
  Status publish(int seq, const int* ids, int n);
  Status finish(int seq, const int* ids, int n);  // publish, then release: the full pages stay cached
  // A new request that starts with the longest cached prefix of `prompt` (at most n - 1 positions, whole pages):
  // its tables hold a reference to each shared page and `length` says how many positions they cover.
  int new_seq_with_prefix(const int* prompt, int n);
  void reset();
  Status check();                                // every page is free or held by exactly one live request
  int live() const { return live_; }
  const std::string& error() const { return error_; }

 private:
  Status fail(Status s, const std::string& msg) { error_ = msg; return s; }
  std::vector<Group> groups_;
  int block_size_;
  std::vector<BlockPool> pools_;
  std::vector<SeqBlocks> seqs_;
  std::vector<int> spare_;   // records free for reuse
  int live_ = 0;             // requests that hold tables (new_seq .. release)
  std::string error_;
};

// Fixed-size per-request state: slot ids 0..n-1, handed out last-in first-out
// (src/provider/local/model/mod.rs:247-251, engine/scheduler.rs:741-750,890-891).
class StateSlots {
 public:
  explicit StateSlots(int n);
  int free_count() const { return (int)free_.size(); }
  int capacity() const { return (int)held_.size(); }
  int alloc();           // -1: none free
  bool release(int s);   // false: not held
  void reset();

 private:
  std::vector<int> free_;
  std::vector<char> held_;
};

}  // namespace cuca
