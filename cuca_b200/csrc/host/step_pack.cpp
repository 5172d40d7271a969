#include "step_pack.hpp"

#include <algorithm>

namespace cuca {

Status validate_step(KvPools& pools, const std::vector<StepEntryView>& entries, int context_length, int vocab,
                     int max_sequences, std::string& error) {
  if (entries.empty()) { error = "a step needs at least one request"; return INVALID; }
  const int bs = pools.block_size();
  std::vector<char> seen(max_sequences > 0 ? max_sequences : 0, 0);
  for (const StepEntryView& e : entries) {
    const int t = e.n_tokens;
    if (t <= 0) { error = "a request in a step brings no tokens"; return INVALID; }
    SeqBlocks* s = pools.seq(e.seq);
    if (!s || s->released) { error = "a request in a step has given its pages back already"; return INVALID; }
    if (e.slot < 0 || e.slot >= max_sequences) {
      error = "state slot " + std::to_string(e.slot) + " is outside 0.." + std::to_string(max_sequences - 1);
      return INVALID;
    }
    if (seen[e.slot]) { error = "state slot " + std::to_string(e.slot) + " appears twice in one step"; return INVALID; }
    seen[e.slot] = 1;
    const int start = s->length;
    if (start + t > context_length) {
      error = "positions " + std::to_string(start) + ".." + std::to_string(start + t - 1) + " exceed the context length " +
              std::to_string(context_length);
      return INVALID;
    }
    for (int i = 0; i < t; ++i)
      if (e.tokens[i] < 0 || e.tokens[i] >= vocab) {
        error = "token id " + std::to_string(e.tokens[i]) + " is outside the vocabulary of " + std::to_string(vocab);
        return INVALID;
      }
    for (const std::vector<int>& table : s->tables) {
      if ((long long)table.size() * bs < start + t) {
        error = "the request holds pages for " + std::to_string(table.size() * bs) + " positions but the step writes up to position " +
                std::to_string(start + t - 1);
        return INVALID;
      }
      for (int i = start / bs; i <= (start + t - 1) / bs; ++i)
        if (table[i] == NO_BLOCK) { error = "a page the step writes was given back already"; return INVALID; }
    }
    for (int i = 0; i < e.n_want; ++i)
      if (e.want[i] < 0 || e.want[i] >= t) {
        error = "wanted place " + std::to_string(e.want[i]) + " is outside the request's " + std::to_string(t) + " tokens";
        return INVALID;
      }
  }
  return OK;
}

// Appends, for one group, the page-table entries of these requests that changed since they were last sent
// (index into the device table, page id) and marks them as sent. The one routine behind both `pack_step` and
// `table_updates`.
static int append_table_updates(KvPools& pools, const int* seqs, const int* slots, int n, int table_width, int g,
                                int* idx, int* val) {
  int k = 0;
  for (int i = 0; i < n; ++i) {
    SeqBlocks* s = pools.seq(seqs[i]);
    if (!s) continue;
    const std::vector<int>& table = s->tables[g];
    for (int j = s->dirty_from[g]; j < (int)table.size(); ++j, ++k) {
      idx[k] = slots[i] * table_width + j;
      val[k] = table[j];
    }
    s->dirty_from[g] = std::max(s->dirty_from[g], (int)table.size());
  }
  return k;
}

static int count_table_updates(KvPools& pools, const int* seqs, int n, int g) {
  int count = 0;
  for (int i = 0; i < n; ++i) {
    SeqBlocks* s = pools.seq(seqs[i]);
    if (s) count += std::max(0, (int)s->tables[g].size() - s->dirty_from[g]);
  }
  return count;
}

Status pack_step(KvPools& pools, const std::vector<StepEntryView>& entries, int table_width, int* out, int cap,
                 int* sizes, StepMeta& meta) {
  const int G = pools.n_groups();
  const int n = (int)entries.size();
  int rows = 0, wanted = 0;
  std::vector<int> seqs(n), slot_list(n);
  for (int i = 0; i < n; ++i) {
    if (!pools.seq(entries[i].seq)) return INVALID;
    rows += entries[i].n_tokens;
    wanted += entries[i].n_want;
    seqs[i] = entries[i].seq;
    slot_list[i] = entries[i].slot;
  }
  sizes[SEC_TOKENS] = sizes[SEC_POSITIONS] = sizes[SEC_SLOT_OF_ROW] = rows;
  sizes[SEC_SLOTS] = sizes[SEC_REQ_ROW0] = sizes[SEC_REQ_COUNT] = sizes[SEC_REQ_START] = n;
  sizes[SEC_LOGIT_ROWS] = wanted;
  for (int g = 0; g < G; ++g)
    sizes[SEC_FIXED + 2 * g] = sizes[SEC_FIXED + 2 * g + 1] = count_table_updates(pools, seqs.data(), n, g);
  const int n_sections = SEC_FIXED + 2 * G;
  int total = 0;
  std::vector<int> at(n_sections);
  for (int i = 0; i < n_sections; ++i) { at[i] = total; total += sizes[i]; }
  meta = StepMeta{rows, n, wanted, total};
  if (total > cap) return TOO_SMALL;

  int* tokens = out + at[SEC_TOKENS];
  int* positions = out + at[SEC_POSITIONS];
  int* slot_of_row = out + at[SEC_SLOT_OF_ROW];
  int* logit_rows = out + at[SEC_LOGIT_ROWS];
  int row = 0, w = 0;
  for (int i = 0; i < n; ++i) {
    const StepEntryView& e = entries[i];
    const int start = pools.seq(e.seq)->length, t = e.n_tokens;
    for (int k = 0; k < t; ++k) {
      tokens[row + k] = e.tokens[k];
      positions[row + k] = start + k;
      slot_of_row[row + k] = e.slot;
    }
    out[at[SEC_SLOTS] + i] = e.slot;
    out[at[SEC_REQ_ROW0] + i] = row;
    out[at[SEC_REQ_COUNT] + i] = t;
    out[at[SEC_REQ_START] + i] = start;
    for (int k = 0; k < e.n_want; ++k) logit_rows[w++] = row + e.want[k];
    row += t;
  }
  for (int g = 0; g < G; ++g)
    append_table_updates(pools, seqs.data(), slot_list.data(), n, table_width, g, out + at[SEC_FIXED + 2 * g],
                         out + at[SEC_FIXED + 2 * g + 1]);
  return OK;
}

int table_updates(KvPools& pools, const int* seqs, const int* slots, int n, int table_width, int group, int* out, int cap) {
  const int count = count_table_updates(pools, seqs, n, group);
  if (2 * count > cap) return -1;
  append_table_updates(pools, seqs, slots, n, table_width, group, out, out + count);
  return count;
}

Status advance_step(KvPools& pools, const int* seqs, const int* n_tokens, int n) {
  for (int i = 0; i < n; ++i) {
    SeqBlocks* s = pools.seq(seqs[i]);
    if (!s) return INVALID;
    s->length += n_tokens[i];
    if (pools.release_window(seqs[i]) < 0) return BOOKKEEPING;
  }
  return OK;
}

}  // namespace cuca
