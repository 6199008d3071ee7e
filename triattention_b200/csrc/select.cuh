// Per-row top-k by radix select on order-preserving keys, with deterministic lowest-index
// tie-break and ascending index output (stable compaction by prefix sums in index order).
// One CTA per row: rows are few (requests x KV heads) and each row stays in L2 across passes.
// Every thread handles 4 consecutive scores per step (one 16-byte load when the row is aligned).
#pragma once

#include "common.cuh"

namespace triattn {

constexpr int kSelectThreads = 1024;
constexpr int kSelectVec = 4;
constexpr int kSelectChunk = kSelectThreads * kSelectVec;
constexpr int kSelectSubHists = 8;  // histogram copies, indexed by warp, to spread shared-memory atomics

struct SelectParams {
  const float* scores;  // [rows, row_stride]
  long long row_stride;
  const int32_t* seq_lens;
  const int32_t* keep_counts;
  int num_reqs, rows_inner;
  int32_t* keep_out;  // [rows, keep_pitch]
  int keep_pitch;
  uint32_t* status;
};

// 4 consecutive keys starting at i (keys of positions >= n come back as 0 with valid=false)
__device__ __forceinline__ void load_keys4(const float* __restrict__ x, int i, int n, bool aligned, unsigned (&key)[4],
                                           bool (&valid)[4]) {
  if (aligned && i + 3 < n) {
    const float4 v = *reinterpret_cast<const float4*>(x + i);
    key[0] = float_to_ordered(v.x);
    key[1] = float_to_ordered(v.y);
    key[2] = float_to_ordered(v.z);
    key[3] = float_to_ordered(v.w);
    valid[0] = valid[1] = valid[2] = valid[3] = true;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      valid[j] = i + j < n;
      key[j] = valid[j] ? float_to_ordered(x[i + j]) : 0u;
    }
  }
}

// exclusive prefix of `v` over the whole CTA (threads in index order) and the CTA total; 2 barriers
__device__ __forceinline__ unsigned block_exclusive_scan(unsigned v, unsigned* warp_tot, unsigned& total) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  unsigned incl = v;
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    const unsigned u = __shfl_up_sync(0xffffffffu, incl, s);
    if (lane >= s) incl += u;
  }
  if (lane == 31) warp_tot[wid] = incl;
  __syncthreads();
  unsigned wv = warp_tot[lane];  // 32 warps: one value per lane
  unsigned winc = wv;
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    const unsigned u = __shfl_up_sync(0xffffffffu, winc, s);
    if (lane >= s) winc += u;
  }
  total = __shfl_sync(0xffffffffu, winc, 31);
  const unsigned warp_excl = __shfl_sync(0xffffffffu, winc - wv, wid);
  __syncthreads();  // warp_tot may be reused by the caller
  return warp_excl + incl - v;
}

__global__ void __launch_bounds__(kSelectThreads) select_topk_kernel(const __grid_constant__ SelectParams p) {
  __shared__ unsigned int hist[kSelectSubHists][256];
  __shared__ unsigned int s_prefix, s_remaining;
  __shared__ unsigned int warp_tot[32];

  grid_dependency_wait();  // no global access before the preceding kernel of the stream has completed
  trigger_dependents();
  const int row = blockIdx.x;
  const int b = (row / p.rows_inner) % p.num_reqs;
  // a length beyond the row (bad metadata) is clamped and reported, like the scorer and the compaction do
  int n = p.seq_lens[b];
  if ((long long)n > p.row_stride) {
    if (threadIdx.x == 0) flag_status(p.status, TRIATTN_DEV_BAD_LENGTH);
    n = (int)p.row_stride;
  }
  const int k = min(p.keep_counts[b], min(n, p.keep_pitch));
  const float* x = p.scores + (size_t)row * p.row_stride;
  int32_t* out = p.keep_out + (size_t)row * p.keep_pitch;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);

  if (k <= 0 || n <= 0) {
    for (int i = tid; i < p.keep_pitch; i += kSelectThreads) out[i] = -1;
    return;
  }
  for (int i = k + tid; i < p.keep_pitch; i += kSelectThreads) out[i] = -1;
  if (k >= n) {
    for (int i = tid; i < n; i += kSelectThreads) out[i] = i;
    return;
  }

  // ---- radix select: key value of the k-th largest element, 8 bits per pass from the top
  if (tid == 0) {
    s_prefix = 0u;
    s_remaining = (unsigned)k;
  }
  unsigned int* my_hist = hist[wid & (kSelectSubHists - 1)];
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    const unsigned himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < kSelectSubHists * 256; i += kSelectThreads) (&hist[0][0])[i] = 0u;
    __syncthreads();
    const unsigned prefix = s_prefix;
    for (int i0 = 0; i0 < n; i0 += kSelectChunk) {
      unsigned key[4];
      bool valid[4];
      load_keys4(x, i0 + tid * kSelectVec, n, aligned, key, valid);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (valid[j] && ((key[j] ^ prefix) & himask) == 0u) atomicAdd(&my_hist[(key[j] >> shift) & 0xffu], 1u);
      }
    }
    __syncthreads();
    if (tid < 256) {
      unsigned s = 0;
#pragma unroll
      for (int h = 0; h < kSelectSubHists; ++h) s += hist[h][tid];
      hist[0][tid] = s;
    }
    __syncthreads();
    if (wid == 0) {
      // lane owns 8 consecutive bins in descending order; find the bin where the count from the top crosses
      unsigned local[8];
      unsigned tot = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        local[j] = hist[0][255 - (lane * 8 + j)];
        tot += local[j];
      }
      unsigned incl = tot;
#pragma unroll
      for (int s = 1; s < 32; s <<= 1) {
        const unsigned v = __shfl_up_sync(0xffffffffu, incl, s);
        if (lane >= s) incl += v;
      }
      unsigned above = incl - tot;  // elements in bins above this lane's first bin
      const unsigned remaining = s_remaining;
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (above < remaining && above + local[j] >= remaining) {
          const unsigned bin = 255u - (unsigned)(lane * 8 + j);
          s_prefix = prefix | (bin << shift);
          s_remaining = remaining - above;
        }
        above += local[j];
      }
    }
    __syncthreads();
  }
  const unsigned kth = s_prefix;         // key of the k-th largest element
  const unsigned need_eq = s_remaining;  // elements equal to kth that are kept (lowest indices first)
  __syncthreads();

  // ---- stable compaction in index order: keys > kth, plus the first need_eq keys == kth
  unsigned base_eq = 0u, base_out = 0u;
  for (int i0 = 0; i0 < n; i0 += kSelectChunk) {
    const int i = i0 + tid * kSelectVec;
    unsigned key[4];
    bool valid[4];
    load_keys4(x, i, n, aligned, key, valid);
    bool gt[4], eq[4];
    unsigned ce = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      gt[j] = valid[j] && key[j] > kth;
      eq[j] = valid[j] && key[j] == kth;
      ce += eq[j] ? 1u : 0u;
    }
    unsigned tot_eq;
    unsigned eq_rank = base_eq + block_exclusive_scan(ce, warp_tot, tot_eq);
    bool sel[4];
    unsigned cs = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      sel[j] = gt[j] || (eq[j] && eq_rank < need_eq);
      eq_rank += eq[j] ? 1u : 0u;
      cs += sel[j] ? 1u : 0u;
    }
    unsigned tot_sel;
    unsigned pos = base_out + block_exclusive_scan(cs, warp_tot, tot_sel);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (sel[j]) {
        if (pos < (unsigned)k) out[pos] = i + j;
        ++pos;
      }
    }
    base_eq += tot_eq;
    base_out += tot_sel;
  }
}

}  // namespace triattn
