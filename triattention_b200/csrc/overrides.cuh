// Effective-length overrides for the forward pass after compaction: a compressed request attends over
// `effective_base + query_len` cached tokens instead of its absolute length, and (debug option of the
// reference) its query positions can be shifted by a per-request delta.  Per-request values live in dense
// arrays indexed by the request-state row (idx_mapping[r]); a negative base / zero delta means "no override".
#pragma once

#include "common.cuh"

namespace triattn {

struct OverrideParams {
  const int32_t* idx_mapping;      // [R] request-state row of batch entry r
  const int32_t* query_start_loc;  // [R + 1]
  int num_reqs;
  const int32_t* effective_base;   // [num_rows] or null
  const int32_t* pos_delta;        // [num_rows] or null
  int num_rows;
  int32_t* seq_lens;               // [>= R] in/out, or null
  const int64_t* positions;        // [num_tokens] or null
  int64_t* positions_out;          // [num_tokens]
  int num_tokens;
  int32_t* counters;               // [4]: rows with a base override, rows with a non-zero delta,
                                   //      1 if query_start_loc is not non-decreasing, 1 if a segment leaves [0, num_tokens]
  int apply;                       // 0: only fill `counters`; 1: also write seq_lens / positions_out
};

__global__ void apply_effective_overrides_kernel(const __grid_constant__ OverrideParams p) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int R = p.num_reqs;
  if (i < R) {
    const int row = p.idx_mapping[i];
    const int q0 = p.query_start_loc[i], q1 = p.query_start_loc[i + 1];
    if (q1 < q0) atomicOr(reinterpret_cast<unsigned int*>(p.counters + 2), 1u);
    if (p.positions != nullptr && (q0 < 0 || q1 > p.num_tokens)) atomicOr(reinterpret_cast<unsigned int*>(p.counters + 3), 1u);
    const bool in_rows = row >= 0 && row < p.num_rows;
    if (p.effective_base != nullptr && in_rows) {
      const int base = p.effective_base[row];
      if (base >= 0) {
        atomicAdd(p.counters + 0, 1);
        if (p.apply && p.seq_lens != nullptr) p.seq_lens[i] = base + (q1 - q0);
      }
    }
    if (p.pos_delta != nullptr && in_rows && p.pos_delta[row] != 0) atomicAdd(p.counters + 1, 1);
  }
  if (p.apply && p.positions != nullptr && i < p.num_tokens) {
    int64_t v = p.positions[i];
    if (p.pos_delta != nullptr && R > 0) {
      // batch entry r with query_start_loc[r] <= i < query_start_loc[r + 1] (upper_bound - 1)
      int lo = 0, hi = R + 1;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (p.query_start_loc[mid] <= i) lo = mid + 1; else hi = mid;
      }
      const int r = lo - 1;
      if (r >= 0 && r < R) {
        const int row = p.idx_mapping[r];
        if (row >= 0 && row < p.num_rows) v += (int64_t)p.pos_delta[row];
      }
    }
    p.positions_out[i] = v;
  }
}

}  // namespace triattn
