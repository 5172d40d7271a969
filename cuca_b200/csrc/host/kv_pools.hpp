// Host-side bookkeeping of the paged key/value cache: which request holds which page.
//
// A page (block) is `block_size` consecutive positions of one request, for every cache of a group; layers whose
// mixers have equal needs share a group, each group has a pool of its own, and each request has one block table
// per group (src/provider/local/model/paged.rs:6-16,52-103,344-489 of the reference). Pages go back to the pool
// when a request ends and, in a windowed group, as soon as the window has passed them (model/paged.rs:736-761).
// No device memory lives here: the page ids index slabs that the Python side allocates.
//
// Prefix store (behaviour of model/paged.rs:18-35,257-321,344-480,831-928): a full page is named by a hash chain over the
// token ids it holds (FNV-1a over the previous page's hash, then the page's ids; the first page chains from 0), so
// two requests with the same token prefix name the same pages. `publish` files a request's full pages under
// their names; a named page whose last reference goes stays in the pool as *cached* (least recently used first
// out) and is what an allocation takes when no free page is left. `new_seq_with_prefix` finds the longest page-aligned prefix
// of a prompt whose pages every group still holds, at most prompt - 1 positions, and takes a reference to each.
// A name is the hash, the parent's hash and the ids themselves, so a collision of hashes never shares pages.
// A named page is read-only: a hit covers whole pages below the prompt's last token, and the request appends
// after them.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace cuca {

constexpr int NO_BLOCK = -1;  // a table entry whose page was given back (behind a window)

uint64_t chain_hash(uint64_t prev, const int* ids, int n);

// What names a full page: its chain hash, the hash of the page before it, and (a view of) its token ids.
struct PageName {
  uint64_t hash = 0, parent = 0;
  const int* ids = nullptr;
  int n_ids = 0;
};

// One group's pages. A page is in exactly one of three states: free (on an intrusive last-in first-out stack
// through `link_`), held (one or more tables name it; `refs_` says how many), or cached (it carries a name, nothing
// holds it; it sits in an intrusive doubly linked list in least-recently-used order, so taking it out on a hit and
// evicting the oldest are both O(1) with no stale entries to skip). Names live in one open-addressed table keyed by
// (hash, parent) that stores page numbers; a hit also compares the token ids, so equal hashes never share pages.
class BlockPool {
 public:
  explicit BlockPool(int n_blocks);
  int n_blocks() const { return (int)refs_.size(); }
  int free_count() const { return n_free_ + n_cached_; }  // what allocations can still get
  int cached_count() const { return n_cached_; }
  int alloc();            // a page with one reference: a free one, else the least recently used cached one; -1: none
  bool release(int b);    // drops one reference; false: the page has none (freed twice, or out of range)
  bool give_name(int b, const PageName& name);  // false: not held, already named, or another page has the name
  bool holds(const PageName& name) const { return find(name) >= 0; }
  int take(const PageName& name);               // one more reference to the page of this name; -1 if there is none
  bool is_named(int b) const { return named_[b] != 0; }
  int refcount(int b) const { return refs_[b]; }
  bool is_cached(int b) const { return named_[b] && refs_[b] == 0; }
  bool is_free(int b) const { return !named_[b] && refs_[b] == 0; }
  // Walks the free stack and the cached list and counts every page it meets into `seen`; false when a walk does
  // not end after n_blocks() pages (a loop in the links) or meets a page in the wrong state.
  bool walk_free(std::vector<int>& seen) const;
  bool walk_cached(std::vector<int>& seen) const;
  void reset();

 private:
  int find(const PageName& name) const;          // the page of this name, or -1
  size_t slot_of(uint64_t hash, uint64_t parent) const;
  void forget_name(int b);
  void unlink_cached(int b);
  std::vector<int> refs_;
  std::vector<char> named_;
  std::vector<int> link_, back_;                 // free stack: link_ = next; cached list: link_ = newer, back_ = older
  int free_top_ = -1, n_free_ = 0;
  int oldest_ = -1, newest_ = -1, n_cached_ = 0;
  std::vector<uint64_t> hash_, parent_;          // per page: its name
  std::vector<std::vector<int>> ids_;
  std::vector<int> table_;                       // open addressing, linear probing; -1 empty
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
