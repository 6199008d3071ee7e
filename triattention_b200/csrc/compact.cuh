// In-place paged K/V compaction: token keep[r] of each (layer, request, KV head) moves to slot r.
//
// Hazard handling: keep rows are strictly ascending, so keep[r] >= r and a destination slot r is a
// source only for some r' <= r.  One CTA owns one (layer, request, head, K-or-V) stream and walks
// destination tiles in ascending order: load the whole tile's sources into registers, barrier,
// store.  Sources of later tiles lie at or beyond the current tile's end, so nothing a tile
// overwrites is still needed; distinct streams touch disjoint memory.
#pragma once

#include "common.cuh"

namespace triattn {

#ifndef TRIATTN_COMPACT_THREADS
#define TRIATTN_COMPACT_THREADS 256
#endif
constexpr int kCompactThreads = TRIATTN_COMPACT_THREADS;
#ifndef TRIATTN_COMPACT_UNROLL
#define TRIATTN_COMPACT_UNROLL 2
#endif
constexpr int kCompactUnroll = TRIATTN_COMPACT_UNROLL;

struct CompactParams {
  void* const* k_ptrs;  // [L]
  void* const* v_ptrs;  // [L]
  const int32_t* block_table;
  const int32_t* seq_lens;
  const int32_t* keep;
  long long keep_ls, keep_rs, keep_hs;
  const int32_t* keep_counts;
  uint32_t* status;
  int L, B, Hkv, bs, num_blocks, max_blocks;
  long long block_stride, token_stride, head_stride;  // elements
  int row_bytes;                                      // D*2
  // preserve-dropped variant
  unsigned char* scratch;
  long long scratch_stream_bytes;  // per (l, b, h, which) stream
  int scratch_rows;                // rows each stream's scratch can hold
};

__device__ __forceinline__ unsigned char* slot_ptr(const CompactParams& p, unsigned char* base, const int32_t* bt,
                                                   int tok, int head, unsigned& err) {
  int blk = bt[tok / p.bs];
  if ((unsigned)blk >= (unsigned)p.num_blocks) {
    err |= TRIATTN_DEV_BAD_BLOCK_ID;
    blk = 0;
  }
  return base + ((long long)blk * p.block_stride + (long long)(tok % p.bs) * p.token_stride +
                 (long long)head * p.head_stride) * 2;
}

// lanes_per_row = row_bytes/16; rows handled per pass = kCompactThreads / lanes_per_row
template <bool PRESERVE>
__global__ void __launch_bounds__(kCompactThreads) compact_paged_kernel(const __grid_constant__ CompactParams p) {
  const int which = blockIdx.x & 1;  // 0: K, 1: V
  const int head = blockIdx.x >> 1;
  const int l = blockIdx.y, b = blockIdx.z;
  const int seq_len = min(p.seq_lens[b], p.max_blocks * p.bs);
  const int k = min(p.keep_counts[b], seq_len);
  if (k <= 0) return;
  const int32_t* keep = p.keep + l * p.keep_ls + b * p.keep_rs + head * p.keep_hs;
  const int32_t* bt = p.block_table + (size_t)b * p.max_blocks;
  unsigned char* base = reinterpret_cast<unsigned char*>(which ? p.v_ptrs[l] : p.k_ptrs[l]);
  const int lpr = p.row_bytes / 16;
  const int rows_per_pass = kCompactThreads / lpr;
  const int tid = threadIdx.x;
  const int rsub = tid / lpr, lsub = tid % lpr;
  const bool active_lane = rsub < rows_per_pass;
  unsigned err = 0u;

  if constexpr (PRESERVE) {
    // phase A: stage every dropped row, in ascending token order, into this stream's scratch
    unsigned char* scr = p.scratch + ((((size_t)l * p.B + b) * p.Hkv + head) * 2 + which) * p.scratch_stream_bytes;
    for (int t0 = 0; t0 < seq_len; t0 += rows_per_pass) {
      const int t = t0 + rsub;
      if (active_lane && t < seq_len) {
        // lower_bound(keep, t)
        int lo = 0, hi = k;
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (keep[mid] < t) lo = mid + 1; else hi = mid;
        }
        const bool kept = lo < k && keep[lo] == t;
        if (!kept) {
          const int d = t - lo;  // rank among dropped tokens
          if (d >= p.scratch_rows) {
            err |= TRIATTN_DEV_BAD_LENGTH;
            continue;
          }
          const uint4 v = *reinterpret_cast<const uint4*>(slot_ptr(p, base, bt, t, head, err) + lsub * 16);
          *reinterpret_cast<uint4*>(scr + (size_t)d * p.row_bytes + lsub * 16) = v;
        }
      }
    }
    __syncthreads();
  }

  // first position that actually moves: keep[r] - r is non-decreasing, binary search for keep[r] != r
  int r_begin;
  {
    int lo = 0, hi = k;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (keep[mid] == mid) lo = mid + 1; else hi = mid;
    }
    r_begin = lo;
  }

  const int tile_rows = rows_per_pass * kCompactUnroll;
  for (int r0 = r_begin; r0 < k; r0 += tile_rows) {
    uint4 v[kCompactUnroll];
    bool mv[kCompactUnroll];
#pragma unroll
    for (int u = 0; u < kCompactUnroll; ++u) {
      const int r = r0 + u * rows_per_pass + rsub;
      mv[u] = false;
      if (active_lane && r < k) {
        const int src = keep[r];
        if (src < r || src >= seq_len || (r > 0 && src <= keep[r - 1])) {
          err |= TRIATTN_DEV_BAD_KEEP_INDEX;  // not a strictly ascending in-range keep row: skip the element
        } else if (src != r) {
          v[u] = *reinterpret_cast<const uint4*>(slot_ptr(p, base, bt, src, head, err) + lsub * 16);
          mv[u] = true;
        }
      }
    }
    __syncthreads();  // all sources of this tile are in registers before any slot of it is overwritten
#pragma unroll
    for (int u = 0; u < kCompactUnroll; ++u) {
      const int r = r0 + u * rows_per_pass + rsub;
      if (mv[u]) *reinterpret_cast<uint4*>(slot_ptr(p, base, bt, r, head, err) + lsub * 16) = v[u];
    }
  }

  if constexpr (PRESERVE) {
    __syncthreads();
    // phase C: dropped rows go to slots k .. seq_len-1
    const unsigned char* scr = p.scratch + ((((size_t)l * p.B + b) * p.Hkv + head) * 2 + which) * p.scratch_stream_bytes;
    const int nd = min(seq_len - k, p.scratch_rows);
    for (int d0 = 0; d0 < nd; d0 += rows_per_pass) {
      const int d = d0 + rsub;
      if (active_lane && d < nd) {
        const uint4 v = *reinterpret_cast<const uint4*>(scr + (size_t)d * p.row_bytes + lsub * 16);
        *reinterpret_cast<uint4*>(slot_ptr(p, base, bt, k + d, head, err) + lsub * 16) = v;
      }
    }
  }
  if (err) flag_status(p.status, err);
}

}  // namespace triattn
