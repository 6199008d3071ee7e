// In-place paged K/V compaction: token keep[r] of each (layer, request, KV head) moves to slot r.
//
// Hazard handling: keep rows are strictly ascending, so keep[r] >= r and a destination slot r is a
// source only for some r' <= r.  One CTA owns one (layer, request, head, K-or-V) stream and walks
// destination tiles in ascending order: load the whole tile's sources into registers, barrier,
// store.  Sources of later tiles lie at or beyond the current tile's end, so nothing a tile
// overwrites is still needed; distinct streams touch disjoint memory.
//
// Work split inside a warp: the address of a row (keep lookup, block-table lookup, division by the
// block size) is computed once, by one lane per row, as a 32-bit offset in 16-byte units; the copy
// then runs with all lanes on 16-byte pieces (32/lpr rows per instruction, lpr = pieces per row),
// each row's offset broadcast by a shuffle.  A warp tile is up to 8 such instructions, so a CTA
// keeps 8 warps x 8 x 512 bytes of reads in flight per barrier.  A step with few streams (a single short request)
// leaves most SMs empty and is bound by the serial chain of load-barrier-store round trips of one stream, so
// such grids run 1024-thread CTAs: four times fewer round trips per stream.
#pragma once

#include "common.cuh"

namespace triattn {

constexpr int kCompactThreads = 256;        // grids that fill the device
constexpr int kCompactThreadsSmall = 1024;  // grids of fewer CTAs than kCompactSmallGrid
constexpr int kCompactSmallGrid = 512;
constexpr int kCompactIters = 8;  // 16-byte pieces a lane holds per tile
constexpr uint32_t kNoMove = 0xffffffffu;

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
  long long block_stride, token_stride, head_stride;  // elements (multiples of 8)
  int row_bytes;                                      // D*2
  int nsub;  // a row wider than 512 bytes is handled as nsub sub-rows of row_bytes/nsub bytes
  // preserve-dropped variant
  unsigned char* scratch;
  long long scratch_stream_bytes;  // per (l, b, h, which) stream
  int scratch_rows;                // rows each stream's scratch can hold
};

// offset of (token, head) from the layer's base pointer, in 16-byte units
__device__ __forceinline__ uint32_t slot_off16(const CompactParams& p, const int32_t* bt, int tok, int head,
                                               unsigned& err) {
  const int bi = tok / p.bs;
  int blk = bt[bi];
  if ((unsigned)blk >= (unsigned)p.num_blocks) {
    err |= TRIATTN_DEV_BAD_BLOCK_ID;
    blk = 0;
  }
  return (uint32_t)(((long long)blk * p.block_stride + (long long)(tok - bi * p.bs) * p.token_stride +
                     (long long)head * p.head_stride) >> 3);
}

template <bool PRESERVE, int THREADS>
__global__ void __launch_bounds__(THREADS) compact_paged_kernel(const __grid_constant__ CompactParams p) {
  constexpr int kCompactWarps = THREADS / 32;
  grid_dependency_wait();  // no global access before the preceding kernel of the stream has completed
  trigger_dependents();
  const int which = blockIdx.x & 1;  // 0: K, 1: V
  const int head = blockIdx.x >> 1;
  const int l = blockIdx.y, b = blockIdx.z;
  const int seq_len = min(p.seq_lens[b], p.max_blocks * p.bs);
  const int k = min(p.keep_counts[b], seq_len);
  if (k <= 0) return;
  const int32_t* keep = p.keep + l * p.keep_ls + b * p.keep_rs + head * p.keep_hs;
  const int32_t* bt = p.block_table + (size_t)b * p.max_blocks;
  unsigned char* base = reinterpret_cast<unsigned char*>(which ? p.v_ptrs[l] : p.k_ptrs[l]);
  constexpr unsigned kFull = 0xffffffffu;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nsub = p.nsub;
  const int ppr = p.row_bytes / 16;                    // 16-byte pieces per row
  const int lpr = ppr / nsub;                          // lanes per (sub-)row, <= 32
  const int rpi = 32 / lpr;                            // (sub-)rows per copy instruction
  const int rows_w = min(32, kCompactIters * rpi);     // (sub-)rows per warp tile: one address lane each
  const int nit = rows_w / rpi;                        // copy instructions per warp tile
  const int sub_row = lane / lpr, piece = lane - sub_row * lpr;
  const bool lane_active = sub_row < rpi;
  const int tile_v = kCompactWarps * rows_w;
  unsigned err = 0u;

  // copy the warp tile whose (sub-)row j has source offset so (lane j) and destination offset dof (lane j)
  auto warp_copy = [&](const unsigned char* srcb, uint32_t so, unsigned char* dstb, uint32_t dof) {
#pragma unroll
    for (int j = 0; j < kCompactIters; ++j) {
      if (j < nit) {
        const int row = (j * rpi + sub_row) & 31;
        const uint32_t o1 = __shfl_sync(kFull, so, row), o2 = __shfl_sync(kFull, dof, row);
        if (lane_active && o1 != kNoMove)
          *reinterpret_cast<uint4*>(dstb + ((size_t)o2 + piece) * 16) =
              *reinterpret_cast<const uint4*>(srcb + ((size_t)o1 + piece) * 16);
      }
    }
  };

  unsigned char* scr = nullptr;
  if constexpr (PRESERVE) {
    // phase A: stage every dropped row, in ascending token order, into this stream's scratch
    scr = p.scratch + ((((size_t)l * p.B + b) * p.Hkv + head) * 2 + which) * p.scratch_stream_bytes;
    const int nv = seq_len * nsub;
    for (int v0 = 0; v0 < nv; v0 += tile_v) {
      const int vr = v0 + wid * rows_w + lane;
      uint32_t so = kNoMove, dof = kNoMove;
      if (lane < rows_w && vr < nv) {
        const int t = vr / nsub, s = vr - t * nsub;
        int lo = 0, hi = k;  // lower_bound(keep, t)
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (keep[mid] < t) lo = mid + 1; else hi = mid;
        }
        if (!(lo < k && keep[lo] == t)) {
          const int d = t - lo;  // rank among dropped tokens
          if (d >= p.scratch_rows) {
            err |= TRIATTN_DEV_BAD_LENGTH;
          } else {
            so = slot_off16(p, bt, t, head, err) + s * lpr;
            dof = (uint32_t)(d * ppr + s * lpr);
          }
        }
      }
      warp_copy(base, so, scr, dof);
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

  const int nv = (k - r_begin) * nsub;
  for (int v0 = 0; v0 < nv; v0 += tile_v) {
    const int vr = v0 + wid * rows_w + lane;
    uint32_t so = kNoMove, dof = kNoMove;
    if (lane < rows_w && vr < nv) {
      const int q = vr / nsub, s = vr - q * nsub;
      const int r = r_begin + q;
      const int src = keep[r];
      if (src < r || src >= seq_len || (r > 0 && src <= keep[r - 1])) {
        err |= TRIATTN_DEV_BAD_KEEP_INDEX;  // not a strictly ascending in-range keep row: skip the element
      } else if (src != r) {
        so = slot_off16(p, bt, src, head, err) + s * lpr;
        dof = slot_off16(p, bt, r, head, err) + s * lpr;
      }
    }
    uint4 v[kCompactIters];
#pragma unroll
    for (int j = 0; j < kCompactIters; ++j) {
      if (j < nit) {
        const uint32_t o = __shfl_sync(kFull, so, (j * rpi + sub_row) & 31);
        if (lane_active && o != kNoMove) v[j] = *reinterpret_cast<const uint4*>(base + ((size_t)o + piece) * 16);
      }
    }
    __syncthreads();  // all sources of this tile are in registers before any slot of it is overwritten
#pragma unroll
    for (int j = 0; j < kCompactIters; ++j) {
      if (j < nit) {
        const uint32_t o = __shfl_sync(kFull, dof, (j * rpi + sub_row) & 31);
        if (lane_active && o != kNoMove) *reinterpret_cast<uint4*>(base + ((size_t)o + piece) * 16) = v[j];
      }
    }
  }

  if constexpr (PRESERVE) {
    __syncthreads();
    // phase C: dropped rows go to slots k .. seq_len-1
    const int nd = min(seq_len - k, p.scratch_rows);
    const int nvd = nd * nsub;
    for (int v0 = 0; v0 < nvd; v0 += tile_v) {
      const int vr = v0 + wid * rows_w + lane;
      uint32_t so = kNoMove, dof = kNoMove;
      if (lane < rows_w && vr < nvd) {
        const int d = vr / nsub, s = vr - d * nsub;
        so = (uint32_t)(d * ppr + s * lpr);
        dof = slot_off16(p, bt, k + d, head, err) + s * lpr;
      }
      warp_copy(scr, so, base, dof);
    }
  }
  if (err) flag_status(p.status, err);
}

}  // namespace triattn
