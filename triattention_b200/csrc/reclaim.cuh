// Block-table rewrite after compaction: every request keeps the first ceil(len_after / block_size) blocks of
// its row; the rest are appended, request by request and in row order, to a list of freed block ids.
// One CTA handles the whole batch: counts per request -> exclusive scan (offsets into the freed list) ->
// each warp copies the tails of its requests (lanes along the row).  Deterministic order, no atomics.
#pragma once

#include "common.cuh"

namespace triattn {

constexpr int kReclaimThreads = 1024;

struct ReclaimParams {
  int32_t* block_table;         // [B, max_blocks], tails are overwritten with fill_value
  const int32_t* blocks_before; // [B] valid entries per row before the rewrite
  const int32_t* lens_after;    // [B] cached tokens per request after compaction
  int32_t* blocks_after;        // [B] out
  int32_t* freed_ids;           // [freed_capacity] out
  int32_t* freed_count;         // [1] out: total freed blocks (may exceed the capacity: then the list is truncated)
  uint32_t* status;
  int B, max_blocks, block_size, freed_capacity, fill_value;
};

__global__ void __launch_bounds__(kReclaimThreads) rewrite_block_tables_kernel(const __grid_constant__ ReclaimParams p) {
  __shared__ unsigned int warp_tot[32];
  __shared__ unsigned int s_carry;
  __shared__ unsigned int s_off[kReclaimThreads];
  __shared__ int s_after[kReclaimThreads], s_removed[kReclaimThreads];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  if (tid == 0) s_carry = 0u;
  __syncthreads();
  for (int b0 = 0; b0 < p.B; b0 += kReclaimThreads) {
    const int b = b0 + tid;
    int before = 0, after = 0;
    if (b < p.B) {
      before = min(max(p.blocks_before[b], 0), p.max_blocks);
      const int len = max(p.lens_after[b], 0);
      after = min((len + p.block_size - 1) / p.block_size, before);
      p.blocks_after[b] = after;
    }
    const unsigned removed = (unsigned)(before - after);
    // exclusive scan of `removed` over the CTA
    unsigned incl = removed;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const unsigned u = __shfl_up_sync(0xffffffffu, incl, s);
      if (lane >= s) incl += u;
    }
    if (lane == 31) warp_tot[wid] = incl;
    __syncthreads();
    const unsigned wv = warp_tot[lane];
    unsigned winc = wv;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const unsigned u = __shfl_up_sync(0xffffffffu, winc, s);
      if (lane >= s) winc += u;
    }
    const unsigned total = __shfl_sync(0xffffffffu, winc, 31);
    const unsigned carry = s_carry;
    const unsigned off = carry + __shfl_sync(0xffffffffu, winc - wv, wid) + incl - removed;
    s_off[tid] = off;
    s_after[tid] = after;
    s_removed[tid] = (int)removed;
    __syncthreads();
    // the tail of row b goes to freed_ids[off .. off+removed): one warp per row, lanes along the row
    const int rows_here = min(kReclaimThreads, p.B - b0);
    for (int r = wid; r < rows_here; r += kReclaimThreads / 32) {
      int32_t* row = p.block_table + (size_t)(b0 + r) * p.max_blocks + s_after[r];
      const unsigned o = s_off[r];
      for (int j = lane; j < s_removed[r]; j += 32) {
        const int32_t id = row[j];
        if (o + j < (unsigned)p.freed_capacity) p.freed_ids[o + j] = id;
        row[j] = p.fill_value;
      }
    }
    __syncthreads();
    if (tid == 0) s_carry = carry + total;
    __syncthreads();
  }
  if (tid == 0) {
    *p.freed_count = (int32_t)s_carry;
    if (s_carry > (unsigned)p.freed_capacity && p.status != nullptr) flag_status(p.status, TRIATTN_DEV_BAD_LENGTH);
  }
}

}  // namespace triattn
