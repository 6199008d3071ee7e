// Per-row top-k by radix select on order-preserving keys, with deterministic lowest-index
// tie-break and ascending index output (stable compaction by ballot/popc prefix sums).
// One CTA per row: rows are few (requests x KV heads) and each row fits in L2.
#pragma once

#include "common.cuh"

namespace triattn {

constexpr int kSelectThreads = 1024;

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

__global__ void __launch_bounds__(kSelectThreads) select_topk_kernel(const __grid_constant__ SelectParams p) {
  __shared__ unsigned int hist[256];
  __shared__ unsigned int s_prefix, s_remaining;
  __shared__ unsigned int warp_tot[2][32];
  __shared__ unsigned int s_base_eq, s_base_out;

  const int row = blockIdx.x;
  const int b = (row / p.rows_inner) % p.num_reqs;
  const int n = p.seq_lens[b];
  int k = min(p.keep_counts[b], min(n, p.keep_pitch));
  const float* x = p.scores + (size_t)row * p.row_stride;
  int32_t* out = p.keep_out + (size_t)row * p.keep_pitch;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;

  if (k <= 0 || n <= 0) {
    for (int i = tid; i < p.keep_pitch; i += kSelectThreads) out[i] = -1;
    return;
  }
  for (int i = k + tid; i < p.keep_pitch; i += kSelectThreads) out[i] = -1;
  if (k >= n) {
    for (int i = tid; i < n; i += kSelectThreads) out[i] = i;
    return;
  }

  // ---- radix select: find the key value of the k-th largest element, 8 bits per pass
  if (tid == 0) {
    s_prefix = 0u;
    s_remaining = (unsigned)k;
  }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    const unsigned himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    if (tid < 256) hist[tid] = 0u;
    __syncthreads();
    const unsigned prefix = s_prefix;
    for (int i0 = 0; i0 < n; i0 += kSelectThreads) {
      const int i = i0 + tid;
      bool on = false;
      unsigned bin = 0;
      if (i < n) {
        const unsigned key = float_to_ordered(x[i]);
        on = ((key ^ prefix) & himask) == 0u;
        bin = (key >> shift) & 0xffu;
      }
      // warp-aggregated histogram update: one atomic per distinct bin per warp
      const unsigned active = __ballot_sync(0xffffffffu, on);
      if (on) {
        const unsigned peers = __match_any_sync(active, bin);
        if (lane == __ffs(peers) - 1) atomicAdd(&hist[bin], (unsigned)__popc(peers));
      }
    }
    __syncthreads();
    // thread 0..255: suffix count above my bin; the bin where the running count crosses `remaining` wins
    if (wid == 0) {
      // each lane owns 8 consecutive bins, descending order
      unsigned local[8];
      unsigned tot = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        local[j] = hist[255 - (lane * 8 + j)];
        tot += local[j];
      }
      unsigned incl = tot;
#pragma unroll
      for (int s = 1; s < 32; s <<= 1) {
        const unsigned v = __shfl_up_sync(0xffffffffu, incl, s);
        if (lane >= s) incl += v;
      }
      unsigned above = incl - tot;  // elements in bins strictly greater than my first bin
      const unsigned remaining = s_remaining;
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
  const unsigned kth = s_prefix;        // key of the k-th largest element
  const unsigned need_eq = s_remaining;  // how many elements equal to kth are kept (lowest indices first)
  if (tid == 0) {
    s_base_eq = 0u;
    s_base_out = 0u;
  }
  __syncthreads();

  // ---- stable compaction in index order
  for (int i0 = 0; i0 < n; i0 += kSelectThreads) {
    const int i = i0 + tid;
    bool gt = false, eq = false;
    if (i < n) {
      const unsigned key = float_to_ordered(x[i]);
      gt = key > kth;
      eq = key == kth;
    }
    const unsigned beq = __ballot_sync(0xffffffffu, eq);
    const unsigned lt_mask = (1u << lane) - 1u;
    if (lane == 0) warp_tot[0][wid] = (unsigned)__popc(beq);
    __syncthreads();
    unsigned eq_before = s_base_eq;
    for (int w = 0; w < wid; ++w) eq_before += warp_tot[0][w];
    const unsigned eq_rank = eq_before + (unsigned)__popc(beq & lt_mask);
    const bool sel = gt || (eq && eq_rank < need_eq);
    const unsigned bsel = __ballot_sync(0xffffffffu, sel);
    if (lane == 0) warp_tot[1][wid] = (unsigned)__popc(bsel);
    __syncthreads();
    unsigned out_before = s_base_out;
    for (int w = 0; w < wid; ++w) out_before += warp_tot[1][w];
    if (sel) {
      const unsigned pos = out_before + (unsigned)__popc(bsel & lt_mask);
      if (pos < (unsigned)k) out[pos] = i;
    }
    __syncthreads();
    if (tid == 0) {
      unsigned te = 0, to = 0;
      for (int w = 0; w < 32; ++w) {
        te += warp_tot[0][w];
        to += warp_tot[1][w];
      }
      s_base_eq += te;
      s_base_out += to;
    }
    __syncthreads();
  }
}

}  // namespace triattn
