// Continuous batching above the step function: admit, cut prompts into portions, decode, finish, free.
//
// One turn is at most one step (src/provider/local/engine/scheduler.rs:515-535,793-876,1032-1107 of the
// reference): admission is first-in first-out with head-of-line blocking; a step has at most `max_step_tokens`
// rows, decoding requests first (oldest first, one pending token each), then portions of prompts in admission
// order; a request finishes on an end id, on its budget or on a full context; when pages run out while decoding
// the youngest running request is preempted and re-prefills everything it had (engine/scheduler.rs:970-1008).
// This class decides and keeps the books; it touches no device. The caller runs the planned step, samples, and
// hands the tokens back. Whatever changed is reported as events.
#pragma once
#include <deque>
#include <string>
#include <vector>

#include "kv_pools.hpp"

namespace cuca {

enum Phase { PH_PREFILL = 0, PH_DECODE = 1, PH_ENDED = 2 };
enum FinishReason { FIN_NONE = 0, FIN_STOP = 1, FIN_LENGTH = 2, FIN_ERROR = 3, FIN_CANCELLED = 4 };
enum EventKind {
  EV_ADMITTED = 1,   // value = slot, extra = handle of its block tables
  EV_TOKEN = 2,      // value = the token appended to the completion
  EV_FINISHED = 3,   // value = FinishReason
  EV_PREEMPTED = 4,  // back at the front of the queue; its prompt is now prompt + completion
  EV_PREFILLED = 5,  // value = prompt tokens cached so far
  EV_DECODING = 6,   // the prompt is done; the request decodes from now on
};

struct Event { int kind, seq, value, extra; };

struct SchedulerConfig {
  int max_sequences = 4, max_step_tokens = 256, prefill_chunk = 256, context_length = 8192;
  std::vector<int> eos_token_ids;
  bool prefix_cache = false;  // requests start from the longest cached prefix of their prompt and leave their pages named
};

// A request's share of the coming step: prompt[offset, offset + n) while prefilling, else its one pending `token`.
struct PlanItem { int seq, offset, n, want_last, slot, blocks, start, token; };  // start = positions cached before the step

struct Sequence {
  int id = 0;
  std::vector<int> request_prompt, prompt, completion, stop_ids;
  int budget = 0, phase = PH_PREFILL, pos = 0, pending = -1, blocks = -1, slot = -1;
  int finish_reason = FIN_NONE, preemptions = 0;
  long long draws = 0;
  bool draws_random = false;  // temperature > 0: each token advances the request's generator
  std::string error;
};

class Scheduler {
 public:
  Scheduler(KvPools& pools, StateSlots& slots, const SchedulerConfig& cfg) : pools_(pools), slots_(slots), cfg_(cfg) {}
  // A new request; max_tokens < 0: as many as the context allows. Returns its id, or -1 with error() set.
  int submit(const int* prompt, int n, long long max_tokens, bool draws_random, const int* stop_ids, int n_stop);
  void admit();
  void plan(std::vector<PlanItem>& out);
  // `tokens`: one per planned request that asked for its last logits, in plan order.
  bool apply(const std::vector<PlanItem>& plans, const int* tokens, int n_tokens);
  void cancel(int id);                        // the caller dropped the request: pages and slot go back
  void fail_running(const std::string& why);  // every running request fails, pools and slots start over
  bool has_work() const { return !waiting_.empty() || !running_.empty(); }
  int n_running() const { return (int)running_.size(); }
  int n_waiting() const { return (int)waiting_.size(); }
  Sequence* seq(int id) { return id >= 0 && id < (int)seqs_.size() ? &seqs_[id] : nullptr; }
  void forget(int id);  // an ended request's record is cleared and its id may be used again
  std::vector<Event>& events() { return events_; }
  const std::string& error() const { return error_; }
  const std::vector<int>& running() const { return running_; }
  const std::deque<int>& waiting() const { return waiting_; }
  long long preemptions = 0, admissions = 0, generated_tokens = 0, prefix_hit_tokens = 0;

 private:
  void committed(std::vector<int>& total);
  bool ensure_block(int id);
  bool ensure_portion(int id, int upto);
  void preempt(int id);
  void take_token(int id, int tok);
  void release(int id, bool share);  // share: with the prefix cache on, its full pages stay findable
  void tokens_cached(const Sequence& s, std::vector<int>& ids) const;
  void finish(int id, int reason, const std::string& error = std::string());
  bool is_running(int id) const;
  void emit(int kind, int seq, int value = 0, int extra = 0) { events_.push_back(Event{kind, seq, value, extra}); }

  KvPools& pools_;
  StateSlots& slots_;
  SchedulerConfig cfg_;
  std::vector<Sequence> seqs_;
  std::vector<int> spare_ids_;
  std::deque<int> waiting_;
  std::vector<int> running_;  // admission order: oldest first
  std::vector<Event> events_;
  std::string error_;
};

}  // namespace cuca
