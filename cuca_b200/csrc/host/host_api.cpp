// The C interface of the host core (loaded with ctypes): pools, state slots, step packing, scheduler.
// Every function that can fail returns a Status (0 = fine) and leaves its reason in cuca_host_last_error().
#include <cstring>
#include <string>
#include <vector>

#include "kv_pools.hpp"
#include "scheduler.hpp"
#include "step_pack.hpp"

using namespace cuca;

#define HOST_API extern "C" __attribute__((visibility("default")))

static thread_local std::string g_error;
static int fail(int code, const std::string& msg) { g_error = msg; return code; }

HOST_API const char* cuca_host_last_error() { return g_error.c_str(); }

// ------------------------------------------------------------------ a single pool (tests)
HOST_API void* cuca_host_blockpool_new(int n) { return n > 0 ? new BlockPool(n) : nullptr; }
HOST_API void cuca_host_blockpool_free(void* h) { delete (BlockPool*)h; }
HOST_API int cuca_host_blockpool_alloc(void* h) { return ((BlockPool*)h)->alloc(); }
HOST_API int cuca_host_blockpool_release(void* h, int b) { return ((BlockPool*)h)->release(b) ? 0 : BOOKKEEPING; }
HOST_API int cuca_host_blockpool_free_count(void* h) { return ((BlockPool*)h)->free_count(); }
HOST_API void cuca_host_blockpool_reset(void* h) { ((BlockPool*)h)->reset(); }

// ------------------------------------------------------------------ pools
HOST_API void* cuca_host_pools_new(int n_groups, const int* n_blocks, const int* windows, int block_size) {
  if (n_groups < 0 || block_size <= 0) return nullptr;
  std::vector<Group> groups;
  for (int g = 0; g < n_groups; ++g) {
    if (n_blocks[g] <= 0) return nullptr;
    groups.push_back(Group{n_blocks[g], windows[g]});
  }
  return new KvPools(groups, block_size);
}
HOST_API void cuca_host_pools_free(void* h) { delete (KvPools*)h; }
HOST_API int cuca_host_pools_new_seq(void* h) { return ((KvPools*)h)->new_seq(); }
HOST_API void cuca_host_pools_drop_seq(void* h, int seq) { ((KvPools*)h)->drop_seq(seq); }
HOST_API void cuca_host_pools_owed(void* h, int seq, int tokens, int* out) { ((KvPools*)h)->owed(seq, tokens, out); }
HOST_API int cuca_host_pools_can_give(void* h, const int* owed) { return ((KvPools*)h)->can_give(owed) ? 1 : 0; }
static int pool_status(KvPools* p, Status s) { return s == OK ? 0 : fail(s, p->error()); }
static bool group_ok(void* h, int g) { return g >= 0 && g < ((KvPools*)h)->n_groups(); }
HOST_API int cuca_host_pools_reserve(void* h, int seq, int upto) { return pool_status((KvPools*)h, ((KvPools*)h)->reserve(seq, upto)); }
HOST_API int cuca_host_pools_release_window(void* h, int seq) {
  const int n = ((KvPools*)h)->release_window(seq);
  if (n < 0) fail(BOOKKEEPING, ((KvPools*)h)->error());
  return n;
}
HOST_API int cuca_host_pools_truncate(void* h, int seq, int length) { return pool_status((KvPools*)h, ((KvPools*)h)->truncate(seq, length)); }
HOST_API int cuca_host_pools_release(void* h, int seq) { return pool_status((KvPools*)h, ((KvPools*)h)->release(seq)); }
HOST_API int cuca_host_pools_publish(void* h, int seq, const int* ids, int n) { return pool_status((KvPools*)h, ((KvPools*)h)->publish(seq, ids, n)); }
HOST_API int cuca_host_pools_finish(void* h, int seq, const int* ids, int n) { return pool_status((KvPools*)h, ((KvPools*)h)->finish(seq, ids, n)); }
HOST_API int cuca_host_pools_new_seq_with_prefix(void* h, const int* prompt, int n) { return ((KvPools*)h)->new_seq_with_prefix(prompt, n); }
HOST_API int cuca_host_pools_cached_blocks(void* h, int g) { return group_ok(h, g) ? ((KvPools*)h)->pool(g).cached_count() : -1; }
HOST_API void cuca_host_pools_reset(void* h) { ((KvPools*)h)->reset(); }
HOST_API int cuca_host_pools_check(void* h) { return pool_status((KvPools*)h, ((KvPools*)h)->check()); }
HOST_API int cuca_host_pools_live(void* h) { return ((KvPools*)h)->live(); }
HOST_API int cuca_host_pools_free_blocks(void* h, int g) { return group_ok(h, g) ? ((KvPools*)h)->pool(g).free_count() : -1; }
HOST_API int cuca_host_pools_total_blocks(void* h, int g) { return group_ok(h, g) ? ((KvPools*)h)->pool(g).n_blocks() : -1; }

// a request's record: field 0 length, 1 released, 2 + g first_live, 2 + G + g dirty_from (get / set)
HOST_API int cuca_host_seq_get(void* h, int seq, int field) {
  KvPools* p = (KvPools*)h;
  SeqBlocks* s = p->seq(seq);
  if (!s) return -1;
  const int G = p->n_groups();
  if (field == 0) return s->length;
  if (field == 1) return s->released ? 1 : 0;
  if (field < 2 + G) return s->first_live[field - 2];
  if (field < 2 + 2 * G) return s->dirty_from[field - 2 - G];
  return -1;
}
HOST_API int cuca_host_seq_set(void* h, int seq, int field, int value) {
  KvPools* p = (KvPools*)h;
  SeqBlocks* s = p->seq(seq);
  if (!s) return fail(BOOKKEEPING, "unknown request");
  const int G = p->n_groups();
  if (field == 0) s->length = value;
  else if (field >= 2 && field < 2 + G) s->first_live[field - 2] = value;
  else if (field >= 2 + G && field < 2 + 2 * G) s->dirty_from[field - 2 - G] = value;
  else return fail(INVALID, "this field cannot be set");
  return 0;
}
// the request's table in group g: its length; entries copied into `out` (up to cap)
HOST_API int cuca_host_seq_table(void* h, int seq, int g, int* out, int cap) {
  SeqBlocks* s = ((KvPools*)h)->seq(seq);
  if (!s || !group_ok(h, g)) return -1;
  const std::vector<int>& t = s->tables[g];
  for (int i = 0; i < (int)t.size() && i < cap; ++i) out[i] = t[i];
  return (int)t.size();
}

// ------------------------------------------------------------------ state slots
HOST_API void* cuca_host_slots_new(int n) { return new StateSlots(n); }
HOST_API void cuca_host_slots_free(void* h) { delete (StateSlots*)h; }
HOST_API int cuca_host_slots_alloc(void* h) { return ((StateSlots*)h)->alloc(); }
HOST_API int cuca_host_slots_release(void* h, int s) { return ((StateSlots*)h)->release(s) ? 0 : BOOKKEEPING; }
HOST_API int cuca_host_slots_free_count(void* h) { return ((StateSlots*)h)->free_count(); }
HOST_API void cuca_host_slots_reset(void* h) { ((StateSlots*)h)->reset(); }

// ------------------------------------------------------------------ the step
static void entries_of(int n, const int* seqs, const int* slots, const int* n_tokens, const int* tokens, const int* n_want,
                       const int* want, std::vector<StepEntryView>& out) {
  out.resize(n);
  int ta = 0, wa = 0;
  for (int i = 0; i < n; ++i) {
    out[i] = StepEntryView{seqs[i], slots[i], tokens + ta, n_tokens[i], want + wa, n_want[i]};
    ta += n_tokens[i] > 0 ? n_tokens[i] : 0;
    wa += n_want[i] > 0 ? n_want[i] : 0;
  }
}

// Validates the batch, then packs it. meta: rows, requests, wanted, total. sizes: one per section (8 fixed, then
// two per group).
HOST_API int cuca_host_step_pack(void* pools, int n, const int* seqs, const int* slots, const int* n_tokens, const int* tokens,
                                 const int* n_want, const int* want, int context_length, int vocab, int max_sequences,
                                 int table_width, int* out, int cap, int* sizes, int* meta) {
  std::vector<StepEntryView> entries;
  entries_of(n, seqs, slots, n_tokens, tokens, n_want, want, entries);
  std::string why;
  Status st = validate_step(*(KvPools*)pools, entries, context_length, vocab, max_sequences, why);
  if (st != OK) return fail(st, why);
  StepMeta m;
  st = pack_step(*(KvPools*)pools, entries, table_width, out, cap, sizes, m);
  const int mm[4] = {m.rows, m.requests, m.wanted, m.total};
  std::memcpy(meta, mm, sizeof(mm));
  return st == OK ? 0 : fail(st, "the staging buffer is too small for this step");
}
// Validation alone, for a step whose rows already live on the device (a captured decode step): one token per
// request. Same refusals as cuca_host_step_pack; nothing is packed or marked.
HOST_API int cuca_host_step_validate(void* pools, int n, const int* seqs, const int* slots, const int* n_tokens,
                                     const int* tokens, int context_length, int vocab, int max_sequences) {
  std::vector<StepEntryView> entries;
  std::vector<int> none(n > 0 ? n : 1, 0);
  entries_of(n, seqs, slots, n_tokens, tokens, none.data(), none.data(), entries);
  std::string why;
  const Status st = validate_step(*(KvPools*)pools, entries, context_length, vocab, max_sequences, why);
  return st == OK ? 0 : fail(st, why);
}
HOST_API int cuca_host_table_updates(void* pools, const int* seqs, const int* slots, int n, int table_width, int group, int* out, int cap) {
  if (!group_ok(pools, group)) {  // -2: not the "buffer too small" answer
    fail(INVALID, "no such group of caches");
    return -2;
  }
  return table_updates(*(KvPools*)pools, seqs, slots, n, table_width, group, out, cap);
}
HOST_API int cuca_host_step_advance(void* pools, const int* seqs, const int* n_tokens, int n) {
  const Status st = advance_step(*(KvPools*)pools, seqs, n_tokens, n);
  return st == OK ? 0 : fail(st, ((KvPools*)pools)->error());
}

// ------------------------------------------------------------------ scheduler
struct SchedulerBox {
  Scheduler sched;
  std::vector<PlanItem> plans;
  SchedulerBox(KvPools& p, StateSlots& s, const SchedulerConfig& c) : sched(p, s, c) {}
};

HOST_API void* cuca_host_sched_new(void* pools, void* slots, int max_sequences, int max_step_tokens, int prefill_chunk,
                                   int context_length, const int* eos, int n_eos, int prefix_cache) {
  SchedulerConfig c;
  c.prefix_cache = prefix_cache != 0;
  c.max_sequences = max_sequences; c.max_step_tokens = max_step_tokens; c.prefill_chunk = prefill_chunk;
  c.context_length = context_length;
  c.eos_token_ids.assign(eos, eos + n_eos);
  return new SchedulerBox(*(KvPools*)pools, *(StateSlots*)slots, c);
}
HOST_API void cuca_host_sched_free(void* h) { delete (SchedulerBox*)h; }
HOST_API int cuca_host_sched_submit(void* h, const int* prompt, int n, long long max_tokens, int draws_random, const int* stop_ids, int n_stop) {
  Scheduler& s = ((SchedulerBox*)h)->sched;
  const int id = s.submit(prompt, n, max_tokens, draws_random != 0, stop_ids, n_stop);
  if (id < 0) fail(INVALID, s.error());
  return id;
}
HOST_API void cuca_host_sched_admit(void* h) { ((SchedulerBox*)h)->sched.admit(); }
// Plans the coming step; returns the number of items (8 integers each, see PlanItem) copied into `out`.
HOST_API int cuca_host_sched_plan(void* h, int* out, int cap_items) {
  SchedulerBox* b = (SchedulerBox*)h;
  b->sched.plan(b->plans);
  const int n = (int)b->plans.size();
  if (n > cap_items) return -1;
  for (int i = 0; i < n; ++i) {
    const PlanItem& p = b->plans[i];
    const int v[8] = {p.seq, p.offset, p.n, p.want_last, p.slot, p.blocks, p.start, p.token};
    std::memcpy(out + 8 * i, v, sizeof(v));
  }
  return n;
}
HOST_API int cuca_host_sched_apply(void* h, const int* tokens, int n_tokens) {
  SchedulerBox* b = (SchedulerBox*)h;
  return b->sched.apply(b->plans, tokens, n_tokens) ? 0 : fail(INVALID, b->sched.error());
}
HOST_API void cuca_host_sched_fail_running(void* h, const char* why) { ((SchedulerBox*)h)->sched.fail_running(why ? why : ""); }
HOST_API void cuca_host_sched_cancel(void* h, int id) { ((SchedulerBox*)h)->sched.cancel(id); }
HOST_API void cuca_host_sched_forget(void* h, int id) { ((SchedulerBox*)h)->sched.forget(id); }
// Events since the last call: 4 integers each (kind, request, value, extra); returns how many there were.
HOST_API int cuca_host_sched_events(void* h, int* out, int cap_events) {
  std::vector<Event>& ev = ((SchedulerBox*)h)->sched.events();
  const int n = (int)ev.size();
  if (n > cap_events) return -n;  // nothing consumed: call again with room for n
  for (int i = 0; i < n; ++i) {
    const int v[4] = {ev[i].kind, ev[i].seq, ev[i].value, ev[i].extra};
    std::memcpy(out + 4 * i, v, sizeof(v));
  }
  ev.clear();
  return n;
}
// counters: 0 running, 1 waiting, 2 preemptions, 3 admissions, 4 generated tokens, 5 prompt tokens found cached
HOST_API long long cuca_host_sched_counter(void* h, int which) {
  Scheduler& s = ((SchedulerBox*)h)->sched;
  switch (which) {
    case 0: return s.n_running();
    case 1: return s.n_waiting();
    case 2: return s.preemptions;
    case 3: return s.admissions;
    case 4: return s.generated_tokens;
    case 5: return s.prefix_hit_tokens;
  }
  return -1;
}
// a request's record: 0 phase, 1 pos, 2 pending, 3 blocks, 4 slot, 5 finish reason, 6 preemptions, 7 budget,
// 8 completion length, 9 prompt length (what is prefilled)
HOST_API long long cuca_host_sched_seq_get(void* h, int id, int field) {
  Sequence* s = ((SchedulerBox*)h)->sched.seq(id);
  if (!s) return -1;
  switch (field) {
    case 0: return s->phase;
    case 1: return s->pos;
    case 2: return s->pending;
    case 3: return s->blocks;
    case 4: return s->slot;
    case 5: return s->finish_reason;
    case 6: return s->preemptions;
    case 7: return s->budget;
    case 8: return (long long)s->completion.size();
    case 9: return (long long)s->prompt.size();
    case 10: return s->draws;
  }
  return -1;
}
HOST_API const char* cuca_host_sched_seq_error(void* h, int id) {
  Sequence* s = ((SchedulerBox*)h)->sched.seq(id);
  return s ? s->error.c_str() : "";
}
// ids of the running requests (admission order) or of the queue; returns the count
HOST_API int cuca_host_sched_list(void* h, int which, int* out, int cap) {
  Scheduler& s = ((SchedulerBox*)h)->sched;
  int n = 0;
  if (which == 0) { for (int id : s.running()) { if (n < cap) out[n] = id; ++n; } }
  else { for (int id : s.waiting()) { if (n < cap) out[n] = id; ++n; } }
  return n;
}
