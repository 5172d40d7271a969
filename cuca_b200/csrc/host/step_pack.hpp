// Validation and packing of one step: everything the device needs of a batch of (request, its next tokens) as one
// run of 32-bit integers, ready for a single copy from pinned memory.
#pragma once
#include <string>
#include <vector>

#include "kv_pools.hpp"

namespace cuca {

struct StepEntryView {
  int seq;            // handle of the request's block tables
  int slot;           // its state slot
  const int* tokens;  // its next tokens
  int n_tokens;
  const int* want;    // places among the tokens whose logits are wanted
  int n_want;
};

// Sections of the packed buffer, in order; `sizes` of pack_step has one entry per section. Per row: its token,
// position and request slot. Per request, in the order given: its slot, the row its tokens start at, how many
// tokens it brings and how many positions it had cached before. How the rows are handed to kernels (tiles,
// lists of single-token rows, scans) is not decided here: every mixer plans that for itself from the
// per-request sections.
enum Section {
  SEC_TOKENS = 0, SEC_POSITIONS, SEC_SLOT_OF_ROW, SEC_SLOTS, SEC_LOGIT_ROWS, SEC_REQ_ROW0, SEC_REQ_COUNT, SEC_REQ_START,
  SEC_FIXED  // then, per group: indices into the device page table, and the page ids that go there
};

struct StepMeta {
  int rows, requests, wanted, total;
};

// Empty batch, empty token list, context overflow, token id out of range, missing or returned pages, wanted
// places, duplicate slots (src/provider/local/model/cpu.rs:1822-1837, model/cpu/paged_attn.rs:42-65): nothing
// has been changed when this fails. `error` gets the reason.
Status validate_step(KvPools& pools, const std::vector<StepEntryView>& entries, int context_length, int vocab,
                     int max_sequences, std::string& error);

// Packs the step into `out` (capacity `cap` integers). Page-table entries that changed since they were last sent
// are appended per group and marked as sent. TOO_SMALL: meta.total says what is needed and nothing was marked.
Status pack_step(KvPools& pools, const std::vector<StepEntryView>& entries, int table_width, int* out, int cap,
                 int* sizes, StepMeta& meta);

// Page-table entries of these requests that changed, for one group: indices then values, `2 * count` integers.
// Returns the count, or -1 if `cap` is too small (nothing marked then).
int table_updates(KvPools& pools, const int* seqs, const int* slots, int n, int table_width, int group, int* out, int cap);

// After the step ran: every request has `n_tokens` more positions cached; pages behind windows go back.
Status advance_step(KvPools& pools, const int* seqs, const int* n_tokens, int n);

}  // namespace cuca
