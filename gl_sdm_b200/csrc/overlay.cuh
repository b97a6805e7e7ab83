// Undo logs of copy-free commits, as the kernels that read an older bank version see them.
//
// A commit that updates the bank in place (glsdm_commit_undo) writes down, for every address it
// touches, the row that address held before. A row of an OLDER version is the row recorded by
// the earliest later commit that touched its address, or the bank's current row if none did
// (the reference plans this as "immutable base + versioned touched-row updates",
// projects/gl-sdm/OPTIMIZATION_PLAN.md, "Represent commits as compact overlays").
#pragma once

#include <cstdint>

#include "glsdm.h"

namespace glsdm {

constexpr int kMaxLogs = GLSDM_MAX_UNDO_LOGS;

struct UndoChain {
  int count;
  const int64_t* addresses[kMaxLogs];  // sorted flat addresses of one commit (runs of equal values)
  const void* rows[kMaxLogs];          // [entries, dim]; the first position of a run holds the row
  int64_t entries[kMaxLogs];
};

// First position whose address is >= key.
__device__ __forceinline__ int64_t lower_bound(const int64_t* __restrict__ sorted, int64_t n, int64_t key) {
  int64_t lo = 0, hi = n;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (sorted[mid] < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// Where the older version's row `flat` lives: in the oldest log that holds the address, else in
// the bank (`current`).
template <typename T>
__device__ __forceinline__ const T* version_row(const UndoChain& chain, int64_t flat, int dim, const T* current) {
  for (int l = 0; l < chain.count; ++l) {
    const int64_t pos = lower_bound(chain.addresses[l], chain.entries[l], flat);
    if (pos < chain.entries[l] && chain.addresses[l][pos] == flat)
      return static_cast<const T*>(chain.rows[l]) + pos * dim;
  }
  return current;
}

// Host side: the logs a caller passed (oldest commit first; empty ones dropped) as a chain.
// `rows_aligned` reports whether every log's rows start on a 16-byte boundary.
inline int make_chain(int32_t n_logs, const int64_t* const* log_addresses, const void* const* log_rows,
                      const int64_t* log_entries, UndoChain* chain, bool* rows_aligned) {
  if (n_logs < 0) return GLSDM_ERR_ARGUMENT;
  if (n_logs > kMaxLogs) return GLSDM_ERR_LIMIT;
  if (n_logs > 0 && (log_addresses == nullptr || log_rows == nullptr || log_entries == nullptr))
    return GLSDM_ERR_ARGUMENT;
  chain->count = 0;
  bool aligned = true;
  for (int l = 0; l < n_logs; ++l) {
    if (log_entries[l] < 0) return GLSDM_ERR_ARGUMENT;
    if (log_entries[l] == 0) continue;
    if (log_addresses[l] == nullptr || log_rows[l] == nullptr) return GLSDM_ERR_ARGUMENT;
    chain->addresses[chain->count] = log_addresses[l];
    chain->rows[chain->count] = log_rows[l];
    chain->entries[chain->count] = log_entries[l];
    aligned = aligned && (reinterpret_cast<uintptr_t>(log_rows[l]) & 15u) == 0;
    ++chain->count;
  }
  if (rows_aligned != nullptr) *rows_aligned = aligned;
  return GLSDM_OK;
}

}  // namespace glsdm
