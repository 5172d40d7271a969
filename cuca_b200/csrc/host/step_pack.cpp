#include "step_pack.hpp"

#include <algorithm>
#include <numeric>

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

Status pack_step(KvPools& pools, const std::vector<StepEntryView>& entries, int table_width, int* out, int cap,
                 int* sizes, StepMeta& meta) {
  const int G = pools.n_groups();
  int rows = 0, wanted = 0, n_decode = 0, n_tiles = 0, n_tiles128 = 0, max_len = 1;
  std::vector<int> upd(G, 0);
  for (const StepEntryView& e : entries) {
    SeqBlocks* s = pools.seq(e.seq);
    if (!s) return INVALID;
    rows += e.n_tokens;
    wanted += e.n_want;
    if (e.n_tokens == 1) {
      ++n_decode;
      max_len = std::max(max_len, s->length + 1);
    } else {
      n_tiles += (e.n_tokens + 63) / 64;
      n_tiles128 += (e.n_tokens + 127) / 128;
    }
    for (int g = 0; g < G; ++g) upd[g] += std::max(0, (int)s->tables[g].size() - s->dirty_from[g]);
  }
  const bool identity = n_decode == rows;
  sizes[SEC_TOKENS] = sizes[SEC_POSITIONS] = sizes[SEC_SLOT_OF_ROW] = rows;
  sizes[SEC_SLOTS] = (int)entries.size();
  sizes[SEC_LOGIT_ROWS] = wanted;
  sizes[SEC_DECODE_ROWS] = identity ? 0 : n_decode;
  sizes[SEC_TILE_ROW0] = sizes[SEC_TILE_NROWS] = n_tiles;
  sizes[SEC_TILE128_ROW0] = sizes[SEC_TILE128_NROWS] = n_tiles128;
  for (int g = 0; g < G; ++g) sizes[SEC_FIXED + 2 * g] = sizes[SEC_FIXED + 2 * g + 1] = upd[g];
  const int n_sections = SEC_FIXED + 2 * G;
  int total = 0;
  std::vector<int> at(n_sections);
  for (int i = 0; i < n_sections; ++i) { at[i] = total; total += sizes[i]; }
  meta = StepMeta{rows, (int)entries.size(), wanted, n_decode, max_len, identity ? 1 : 0, n_tiles, n_tiles128, total};
  if (total > cap) return TOO_SMALL;

  int* tokens = out + at[SEC_TOKENS];
  int* positions = out + at[SEC_POSITIONS];
  int* slot_of_row = out + at[SEC_SLOT_OF_ROW];
  int* slots = out + at[SEC_SLOTS];
  int* logit_rows = out + at[SEC_LOGIT_ROWS];
  int* decode_rows = out + at[SEC_DECODE_ROWS];
  struct Tile { int row0, n, pos; };
  std::vector<Tile> tiles, tiles128;
  tiles.reserve(n_tiles);
  tiles128.reserve(n_tiles128);
  int row = 0, w = 0, d = 0;
  for (size_t i = 0; i < entries.size(); ++i) {
    const StepEntryView& e = entries[i];
    SeqBlocks* s = pools.seq(e.seq);
    const int start = s->length, t = e.n_tokens;
    for (int k = 0; k < t; ++k) {
      tokens[row + k] = e.tokens[k];
      positions[row + k] = start + k;
      slot_of_row[row + k] = e.slot;
    }
    slots[i] = e.slot;
    for (int k = 0; k < e.n_want; ++k) logit_rows[w++] = row + e.want[k];
    if (t == 1) {
      if (!identity) decode_rows[d++] = row;
    } else {
      for (int off = 0; off < t; off += 64) tiles.push_back({row + off, std::min(64, t - off), start + off});
      for (int off = 0; off < t; off += 128) tiles128.push_back({row + off, std::min(128, t - off), start + off});
    }
    row += t;
  }
  // heavy tiles (late positions see most keys) first; equal positions keep their order
  auto heavy_first = [](const Tile& a, const Tile& b) { return a.pos > b.pos; };
  std::stable_sort(tiles.begin(), tiles.end(), heavy_first);
  std::stable_sort(tiles128.begin(), tiles128.end(), heavy_first);
  for (int i = 0; i < n_tiles; ++i) {
    out[at[SEC_TILE_ROW0] + i] = tiles[i].row0;
    out[at[SEC_TILE_NROWS] + i] = tiles[i].n;
  }
  for (int i = 0; i < n_tiles128; ++i) {
    out[at[SEC_TILE128_ROW0] + i] = tiles128[i].row0;
    out[at[SEC_TILE128_NROWS] + i] = tiles128[i].n;
  }
  // page-table entries that changed since they were last sent
  for (int g = 0; g < G; ++g) {
    int* idx = out + at[SEC_FIXED + 2 * g];
    int* val = out + at[SEC_FIXED + 2 * g + 1];
    int n = 0;
    for (const StepEntryView& e : entries) {
      SeqBlocks* s = pools.seq(e.seq);
      const std::vector<int>& table = s->tables[g];
      for (int i = s->dirty_from[g]; i < (int)table.size(); ++i, ++n) {
        idx[n] = e.slot * table_width + i;
        val[n] = table[i];
      }
      s->dirty_from[g] = std::max(s->dirty_from[g], (int)table.size());
    }
  }
  return OK;
}

int table_updates(KvPools& pools, const int* seqs, const int* slots, int n, int table_width, int group, int* out, int cap) {
  int count = 0;
  for (int i = 0; i < n; ++i) {
    SeqBlocks* s = pools.seq(seqs[i]);
    if (s) count += std::max(0, (int)s->tables[group].size() - s->dirty_from[group]);
  }
  if (2 * count > cap) return -1;
  int k = 0;
  for (int i = 0; i < n; ++i) {
    SeqBlocks* s = pools.seq(seqs[i]);
    if (!s) continue;
    const std::vector<int>& table = s->tables[group];
    for (int j = s->dirty_from[group]; j < (int)table.size(); ++j, ++k) {
      out[k] = slots[i] * table_width + j;
      out[count + k] = table[j];
    }
    s->dirty_from[group] = std::max(s->dirty_from[group], (int)table.size());
  }
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
