// Host-side bookkeeping of the paged key/value cache: which request holds which page.
//
// A page (block) is `block_size` consecutive positions of one request, for every cache of a group; layers whose
// mixers have equal needs share a group, each group has a pool of its own, and each request has one block table
// per group (src/provider/local/model/paged.rs:6-16,52-103,344-489 of the reference). Pages go back to the pool
// when a request ends and, in a windowed group, as soon as the window has passed them (model/paged.rs:736-761).
// No device memory lives here: the page ids index slabs that the Python side allocates.
#pragma once
#include <string>
#include <vector>

namespace cuca {

constexpr int NO_BLOCK = -1;  // a table entry whose page was given back (behind a window)

// Free list of one group's pages; pops from the back, as the reference's does.
class BlockPool {
 public:
  explicit BlockPool(int n_blocks);
  int n_blocks() const { return (int)held_.size(); }
  int free_count() const { return (int)free_.size(); }
  int alloc();            // a page, or -1 when none is free; -2 if the free list names a held page
  bool release(int b);    // false: the page is not held (freed twice, or out of range)
  void reset();
  const std::vector<int>& free_list() const { return free_; }

 private:
  std::vector<int> free_;
  std::vector<char> held_;
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
