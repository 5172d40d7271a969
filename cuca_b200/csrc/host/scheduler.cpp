#include "scheduler.hpp"

#include <algorithm>

namespace cuca {

int Scheduler::submit(const int* prompt, int n, long long max_tokens, bool draws_random, const int* stop_ids, int n_stop) {
  if (n <= 0) { error_ = "the prompt is empty"; return -1; }
  if (n >= cfg_.context_length) {
    // src/provider/local/mod.rs:3252, engine/scheduler.rs:471-482
    error_ = "the prompt has " + std::to_string(n) + " tokens; the context holds " + std::to_string(cfg_.context_length);
    return -1;
  }
  const long long room = cfg_.context_length - n;
  int id;
  if (!spare_ids_.empty()) {
    id = spare_ids_.back();
    spare_ids_.pop_back();
  } else {
    id = (int)seqs_.size();
    seqs_.emplace_back();
  }
  Sequence s;
  s.id = id;
  s.request_prompt.assign(prompt, prompt + n);
  s.prompt = s.request_prompt;
  s.stop_ids.assign(stop_ids, stop_ids + n_stop);
  s.budget = (int)(max_tokens < 0 ? room : std::min(max_tokens, room));
  s.draws_random = draws_random;
  seqs_[id] = std::move(s);
  if (seqs_[id].budget <= 0) finish(id, FIN_LENGTH);
  else waiting_.push_back(id);
  return id;
}

void Scheduler::forget(int id) {
  Sequence* s = seq(id);
  if (!s || s->phase != PH_ENDED) return;
  if (s->blocks >= 0) pools_.drop_seq(s->blocks);
  *s = Sequence();
  s->phase = PH_ENDED;
  spare_ids_.push_back(id);
}

bool Scheduler::is_running(int id) const { return std::find(running_.begin(), running_.end(), id) != running_.end(); }

// Pages the prompts being prefilled still need (per group).
void Scheduler::committed(std::vector<int>& total) {
  const int G = pools_.n_groups();
  total.assign(G, 0);
  std::vector<int> owed(G);
  for (int id : running_) {
    const Sequence& s = seqs_[id];
    if (s.phase != PH_PREFILL) continue;
    pools_.owed(s.blocks, (int)s.prompt.size() + 1, owed.data());
    for (int g = 0; g < G; ++g) total[g] += owed[g];
  }
}

void Scheduler::admit() {
  const int G = pools_.n_groups();
  std::vector<int> com, owed(G), need(G);
  while (!waiting_.empty() && (int)running_.size() < cfg_.max_sequences && slots_.free_count() > 0) {
    const int id = waiting_.front();
    Sequence& s = seqs_[id];
    committed(com);
    // with the prefix cache the request starts from the pages that already hold the head of its prompt
    // (src/provider/local/engine/scheduler.rs:805-813)
    const int blocks = cfg_.prefix_cache ? pools_.new_seq_with_prefix(s.prompt.data(), (int)s.prompt.size()) : pools_.new_seq();
    pools_.owed(blocks, (int)s.prompt.size() + 1, owed.data());
    for (int g = 0; g < G; ++g) need[g] = com[g] + owed[g];
    if (!pools_.can_give(need.data())) {
      const bool never = running_.empty() && !pools_.can_give(owed.data());
      pools_.drop_seq(blocks);
      if (never) {
        // nothing runs and it still does not fit: it never will
        waiting_.pop_front();
        finish(id, FIN_ERROR, "the prompt needs more pages than the pool has");
        continue;
      }
      break;  // head-of-line blocking
    }
    waiting_.pop_front();
    s.slot = slots_.alloc();
    s.blocks = blocks;
    s.phase = PH_PREFILL;
    s.pos = pools_.seq(blocks)->length;
    s.pending = -1;
    running_.push_back(id);
    ++admissions;
    prefix_hit_tokens += s.pos;
    emit(EV_ADMITTED, id, s.slot, s.blocks);
    if (s.pos > 0) emit(EV_PREFILLED, id, s.pos);
  }
}

void Scheduler::plan(std::vector<PlanItem>& out) {
  out.clear();
  const int budget = cfg_.max_step_tokens;
  int used = 0;
  // decoding requests, oldest first; a preemption may take requests (planned ones too) out of `running_`
  const std::vector<int> snapshot = running_;
  for (int id : snapshot) {
    Sequence& s = seqs_[id];
    if (s.phase != PH_DECODE || !is_running(id)) continue;
    if (used >= budget) break;
    if (!ensure_block(id)) continue;
    out.push_back(PlanItem{id, 0, 1, 1, s.slot, s.blocks, 0, s.pending});
    ++used;
  }
  out.erase(std::remove_if(out.begin(), out.end(), [&](const PlanItem& p) { return !is_running(p.seq); }), out.end());
  used = (int)out.size();
  // prompts, in admission order
  const std::vector<int> snapshot2 = running_;
  for (int id : snapshot2) {
    Sequence& s = seqs_[id];
    if (s.phase != PH_PREFILL || !is_running(id)) continue;
    const int room = budget - used;
    if (room <= 0) break;
    const int n = std::min(std::min((int)s.prompt.size() - s.pos, cfg_.prefill_chunk), room);
    if (!ensure_portion(id, s.pos + n)) continue;
    const int last = s.pos + n == (int)s.prompt.size() ? 1 : 0;
    out.push_back(PlanItem{id, s.pos, n, last, s.slot, s.blocks, 0, -1});
    used += n;
  }
  // a portion that found no page may have sent younger requests, planned ones among them, back to the queue
  out.erase(std::remove_if(out.begin(), out.end(), [&](const PlanItem& p) { return !is_running(p.seq); }), out.end());
  for (PlanItem& p : out) {
    SeqBlocks* b = pools_.seq(p.blocks);
    p.start = b ? b->length : 0;
  }
}

// Pages for a prompt portion up to position `upto`. When the pool is exhausted the youngest running request gives
// way: it goes back to the head of the queue and starts again when pages are free. If that is this request, it
// waits there itself. Only a request that runs alone and still finds no page fails: the pool is too small for it.
// (The reference fails the request at once, src/provider/local/engine/scheduler.rs:1260-1263; admission only counts
// the prompts being prefilled, so there a request could fail because others had grown while it was cut into
// portions, although it would have fitted a moment later.)
bool Scheduler::ensure_portion(int id, int upto) {
  while (true) {
    Sequence& s = seqs_[id];
    if (pools_.reserve(s.blocks, upto) == OK) return true;
    if (running_.size() == 1) {
      release(id, false);
      finish(id, FIN_ERROR, "the K/V page pool is exhausted");
      return false;
    }
    const int victim = running_.back();  // youngest
    preempt(victim);
    if (victim == id) return false;
  }
}

// Pages for the pending token's position; preempts the youngest on exhaustion.
bool Scheduler::ensure_block(int id) {
  while (true) {
    Sequence& s = seqs_[id];
    SeqBlocks* b = pools_.seq(s.blocks);
    const Status st = pools_.reserve(s.blocks, (b ? b->length : 0) + 1);
    if (st == OK) return true;
    if (running_.size() == 1) {
      release(id, false);
      finish(id, FIN_ERROR, "the K/V page pool is exhausted by one request");
      return false;
    }
    int victim = running_.back();  // youngest
    if (victim == running_.front()) victim = id;
    preempt(victim);
    if (victim == id) return false;
  }
}

// Free the request's pages; it goes back to the front of the queue with all it had as its prompt.
void Scheduler::preempt(int id) {
  release(id, true);  // what it computed stays findable: its re-prefill starts from there if the pages survive
  Sequence& s = seqs_[id];
  s.prompt = s.request_prompt;
  s.prompt.insert(s.prompt.end(), s.completion.begin(), s.completion.end());
  // the pending token is the last of the completion; it is part of the new prompt and its logits will be asked
  // for again at the end of the re-prefill
  s.phase = PH_PREFILL;
  s.pos = 0;
  s.pending = -1;
  ++s.preemptions;
  ++preemptions;
  waiting_.push_front(id);
  emit(EV_PREEMPTED, id);
}

bool Scheduler::apply(const std::vector<PlanItem>& plans, const int* tokens, int n_tokens) {
  int it = 0;
  for (const PlanItem& p : plans) {
    Sequence& s = seqs_[p.seq];
    if (s.phase == PH_PREFILL) {
      s.pos += p.n;
      emit(EV_PREFILLED, p.seq, s.pos);
      if (!p.want_last) continue;
      // (a preempted request re-prefilled its own completion too: the logits just computed follow its last
      // emitted token, so decoding simply goes on)
      s.phase = PH_DECODE;
      emit(EV_DECODING, p.seq);
      if (cfg_.prefix_cache) {
        // a full page is never written again: requests that arrive while this one decodes may share its prompt
        std::vector<int> ids;
        tokens_cached(s, ids);
        pools_.publish(s.blocks, ids.data(), (int)ids.size());
      }
    }
    if (it >= n_tokens) { error_ = "the step returned fewer tokens than requests that asked for one"; return false; }
    take_token(p.seq, tokens[it++]);
  }
  return true;
}

// Rules of src/provider/local/engine/scheduler.rs:1287-1316.
void Scheduler::take_token(int id, int tok) {
  Sequence& s = seqs_[id];
  if (s.draws_random) ++s.draws;
  const bool stop = std::find(cfg_.eos_token_ids.begin(), cfg_.eos_token_ids.end(), tok) != cfg_.eos_token_ids.end() ||
                    std::find(s.stop_ids.begin(), s.stop_ids.end(), tok) != s.stop_ids.end();
  if (stop) {
    release(id, true);
    finish(id, FIN_STOP);
    return;
  }
  s.completion.push_back(tok);
  ++generated_tokens;
  emit(EV_TOKEN, id, tok);
  const int total = (int)s.request_prompt.size() + (int)s.completion.size();
  if ((int)s.completion.size() >= s.budget || total >= cfg_.context_length) {
    release(id, true);
    finish(id, FIN_LENGTH);
    return;
  }
  s.pending = tok;
}

// The tokens at the positions the request has cached: its prompt, then what it generated and forwarded.
void Scheduler::tokens_cached(const Sequence& s, std::vector<int>& ids) const {
  ids = s.request_prompt;
  ids.insert(ids.end(), s.completion.begin(), s.completion.end());
}

void Scheduler::release(int id, bool share) {
  Sequence& s = seqs_[id];
  running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
  if (s.blocks >= 0) {
    SeqBlocks* b = pools_.seq(s.blocks);
    if (b && !b->released) {
      if (share && cfg_.prefix_cache) {
        // src/provider/local/engine/scheduler.rs:884-896: the full pages are filed in the prefix store
        std::vector<int> ids;
        tokens_cached(s, ids);
        pools_.finish(s.blocks, ids.data(), (int)ids.size());
      } else {
        pools_.release(s.blocks);
      }
    }
  }
  if (s.slot >= 0) {
    slots_.release(s.slot);
    s.slot = -1;
  }
}

void Scheduler::finish(int id, int reason, const std::string& error) {
  Sequence& s = seqs_[id];
  s.phase = PH_ENDED;
  s.finish_reason = reason;
  s.error = error;
  emit(EV_FINISHED, id, reason);
}

// src/provider/local/engine/scheduler.rs:663-678
void Scheduler::cancel(int id) {
  Sequence* s = seq(id);
  if (!s || s->phase == PH_ENDED) return;
  waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
  release(id, true);
  finish(id, FIN_CANCELLED);
}

// src/provider/local/engine/scheduler.rs:950-966
void Scheduler::fail_running(const std::string& why) {
  const std::vector<int> snapshot = running_;
  running_.clear();
  for (int id : snapshot) {
    seqs_[id].slot = -1;
    finish(id, FIN_ERROR, why);
  }
  pools_.reset();
  slots_.reset();
}

}  // namespace cuca
