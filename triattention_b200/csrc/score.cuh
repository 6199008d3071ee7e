// Key scorer, shared definitions and the generic kernel.
//
// The scorer streams paged bf16 K once from HBM and writes raw fp32 scores for the g query heads of each KV
// head, plus per-(layer, request, query head) sum / sum of squares.  The streaming tensor-core kernel for
// offset aggregation = mean lives in score_mma.cuh; this file holds the launch parameters, the pipeline
// constants and the generic kernel (any head_dim / group size, mean or max aggregation).
#pragma once

#include "common.cuh"

namespace triattn {

struct ScoreParams {
  const void* const* k_ptrs;   // [L]
  const int32_t* block_table;  // [B, max_blocks]
  const int32_t* seq_lens;     // [B]
  const float* weights;        // [L, B, Hq, rows, F]
  float* raw;                  // [L, B, Hkv, t_pad, GP]
  double* moments;             // [L, B, Hq, 2]
  uint32_t* status;
  int L, B, Hkv, g, bs, num_blocks, max_blocks, t_pad;
  long long block_stride_bytes;
  int token_stride, head_stride;  // elements
  int block_bytes;                // bs*Hkv*D*2
  int mb;                         // cache blocks per pipeline stage
  int stages;
  int tiles_per_cta;
  int gp_total;  // query-head slots per KV head in the raw layout
  int nhd;       // 1: token-major blocks (head_stride == D, token_stride == Hkv*D)
  int block_group;  // > 0: 16-token blocks, Hkv * mb == 8: block j of a stage is read only by the Hkv warps j*Hkv..(j+1)*Hkv-1
  const unsigned char* tmaps;  // [L] stamped tensor maps of the layers' K caches (tcgen05 scorer only)
  int tmap_slots_per_block;    // head slots (head_stride apart) per cache block in those maps
  int num_offsets;
  int agg_max;
};

constexpr int kScoreConsumerWarps = 8;
constexpr int kScoreThreadsWS = kScoreConsumerWarps * 32;  // every warp consumes; the last one to release a stage refills it
constexpr int kMaxStages = 8;
constexpr int kMaxPrefetchedBlocks = 1024;  // block ids of a CTA's tiles kept in shared memory

// Generic scorer: any head_dim / group size / offset aggregation (mean or max).  One thread per
// (token, KV head); K is read straight from global memory (cache resident between passes).
// Weight rows: MEAN {w_re, w_im, w_mag}; MAX {w_re[o]..., w_im[o]..., w_mag}.
__global__ void score_paged_generic_kernel(const __grid_constant__ ScoreParams p, int D, int interleaved) {
  grid_dependency_wait();  // no global access before the preceding kernel of the stream has completed
  trigger_dependents();
  const int GP = p.gp_total;
  const int F = D / 2;
  const int l = blockIdx.z / p.B, b = blockIdx.z % p.B;
  const int head = blockIdx.y;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  int seq_len = p.seq_lens[b];
  if (seq_len > p.t_pad) {
    if (threadIdx.x == 0 && blockIdx.x == 0) flag_status(p.status, TRIATTN_DEV_BAD_LENGTH);
    seq_len = p.t_pad;
  }
  const bool valid = t < seq_len;
  const int Hq = p.Hkv * p.g;
  const int rows = p.agg_max ? 2 * p.num_offsets + 1 : 3;
  const uint16_t* krow = nullptr;
  if (valid) {
    int blk = p.block_table[(size_t)b * p.max_blocks + t / p.bs];
    if ((unsigned)blk >= (unsigned)p.num_blocks) {
      flag_status(p.status, TRIATTN_DEV_BAD_BLOCK_ID);
      blk = 0;
    }
    krow = reinterpret_cast<const uint16_t*>(reinterpret_cast<const unsigned char*>(p.k_ptrs[l]) +
                                             (long long)blk * p.block_stride_bytes) +
           (size_t)(t % p.bs) * p.token_stride + (size_t)head * p.head_stride;
  }
  for (int h = 0; h < p.g; ++h) {
    const float* w = p.weights + (((size_t)l * p.B + b) * Hq + (size_t)head * p.g + h) * rows * F;
    float score = 0.f;
    if (valid) {
      float extra = 0.f;
      const float* wm = w + (size_t)(rows - 1) * F;
      for (int f = 0; f < F; ++f) {
        const float kr = bf16_to_float(interleaved ? krow[2 * f] : krow[f]);
        const float ki = bf16_to_float(interleaved ? krow[2 * f + 1] : krow[F + f]);
        extra = fmaf(sqrtf(fmaf(ki, ki, kr * kr)), __ldg(wm + f), extra);
      }
      if (!p.agg_max) {
        float base = 0.f;
        for (int f = 0; f < F; ++f) {
          const float kr = bf16_to_float(interleaved ? krow[2 * f] : krow[f]);
          const float ki = bf16_to_float(interleaved ? krow[2 * f + 1] : krow[F + f]);
          base = fmaf(kr, __ldg(w + f), base);
          base = fmaf(ki, __ldg(w + F + f), base);
        }
        score = base + extra;
      } else {
        float best = -INFINITY;
        for (int o0 = 0; o0 < p.num_offsets; o0 += 4) {
          float a[4] = {0.f, 0.f, 0.f, 0.f};
          for (int f = 0; f < F; ++f) {
            const float kr = bf16_to_float(interleaved ? krow[2 * f] : krow[f]);
            const float ki = bf16_to_float(interleaved ? krow[2 * f + 1] : krow[F + f]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int o = min(o0 + j, p.num_offsets - 1);
              a[j] = fmaf(kr, __ldg(w + (size_t)o * F + f), a[j]);
              a[j] = fmaf(ki, __ldg(w + (size_t)(p.num_offsets + o) * F + f), a[j]);
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) best = fmaxf(best, a[j]);
        }
        score = best + extra;
      }
      p.raw[((((size_t)l * p.B + b) * p.Hkv + head) * (size_t)p.t_pad + t) * GP + h] = score;
    }
    // block-wide moments of this query head
    float s1 = valid ? score : 0.f, s2 = valid ? score * score : 0.f;
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
      s1 += __shfl_xor_sync(0xffffffffu, s1, s);
      s2 += __shfl_xor_sync(0xffffffffu, s2, s);
    }
    if ((threadIdx.x & 31) == 0 && (s1 != 0.f || s2 != 0.f)) {
      double* m = p.moments + (((size_t)l * p.B + b) * Hq + (size_t)head * p.g + h) * 2;
      atomicAdd(m, (double)s1);
      atomicAdd(m + 1, (double)s2);
    }
  }
}

}  // namespace triattn
