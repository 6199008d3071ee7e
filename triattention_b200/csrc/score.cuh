// Key scorer: streams paged bf16 K once from HBM and writes raw fp32 scores for the g query
// heads of each KV head, plus per-(layer, request, query head) sum / sum of squares.
//
// Fast kernel (offset aggregation = mean, head_dim 64 or 128, g <= 8):
//   * a CTA owns a run of consecutive cache blocks of one (layer, request); each pipeline stage
//     holds `mb` whole cache blocks (all KV heads) fetched by 1-D bulk async copies (TMA) that
//     complete on an mbarrier; stages are recycled with one __syncthreads per stage;
//   * 16 lanes share a key: lane j owns frequencies [j*FPT, (j+1)*FPT) and keeps the folded
//     weights of its frequencies for all GP query heads in registers (packed as fp32x2 over
//     adjacent frequencies, so the inner loop is fma.rn.f32x2 on naturally paired bf16 data);
//   * a batch of NT = 16/GP tokens gives 16 partial sums per lane, combined across the 16 lanes
//     with a select-free reduce-scatter: lane j accumulates logical value (token, head) in
//     register slot (idx ^ j), so every lane sends slots with bit s set and keeps the others;
//     after 4 steps lane j holds the finished score of token j/GP, head j%GP and the 16 lanes
//     store 64 contiguous bytes.
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
  int num_offsets;  // generic kernel only
  int agg_max;      // generic kernel only
};

constexpr int kScoreThreads = 256;
constexpr int kLPK = 16;  // lanes per key

template <int D, int GP, bool INTERLEAVED>
__global__ void __launch_bounds__(kScoreThreads, (GP * D >= 8 * 128) ? 1 : 2)
score_paged_mean_kernel(const __grid_constant__ ScoreParams p) {
  constexpr int F = D / 2;
  constexpr int FPT = F / kLPK;  // frequencies per lane: 4 (D=128) or 2 (D=64)
  constexpr int P2 = FPT / 2;    // fp32x2 pairs per lane per component
  constexpr int NT = kLPK / GP;  // tokens per batch
  constexpr int NG = kScoreThreads / kLPK;
  static_assert(FPT >= 2 && (FPT % 2) == 0, "head_dim must be 64 or 128");
  static_assert(NT >= 1 && NT * GP == kLPK, "GP must divide 16");

  extern __shared__ __align__(128) unsigned char smem_tiles[];
  __shared__ __align__(8) uint64_t full_bar[8];
  __shared__ int s_err;

  const int tid = threadIdx.x;
  const int lg = tid & (kLPK - 1);  // lane within the key group
  const int gid = tid / kLPK;
  const int lane_lo = lg % GP;      // permutes head slots
  const int lane_hi = lg / GP;      // permutes token slots
  const unsigned gmask = 0xffffu << (((tid & 31) / kLPK) * kLPK);
  const int l = blockIdx.y, b = blockIdx.z;

  int seq_len = p.seq_lens[b];
  if (seq_len > p.t_pad) {
    if (tid == 0) flag_status(p.status, TRIATTN_DEV_BAD_LENGTH);
    seq_len = p.t_pad;
  }
  const int nblk = (seq_len + p.bs - 1) / p.bs;
  const int ntiles = (nblk + p.mb - 1) / p.mb;
  const int tile0 = blockIdx.x * p.tiles_per_cta;
  if (tile0 >= ntiles) return;
  const int my_tiles = min(p.tiles_per_cta, ntiles - tile0);
  const int stage_bytes = p.mb * p.block_bytes;
  const unsigned char* kbase = reinterpret_cast<const unsigned char*>(p.k_ptrs[l]);
  const int32_t* bt = p.block_table + (size_t)b * p.max_blocks;
  const int Hq = p.Hkv * p.g;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) mbar_init(smem_u32(&full_bar[s]), 1);
    mbar_fence_init();
    s_err = 0;
  }
  __syncthreads();

  // producer (thread 0): fetch the cache blocks of stage-tile `it`
  auto issue = [&](int it) {
    const int stage = it % p.stages;
    const uint32_t bar = smem_u32(&full_bar[stage]);
    const int blk0 = (tile0 + it) * p.mb;
    const int nb = min(p.mb, nblk - blk0);
    mbar_arrive_expect_tx(bar, (uint32_t)(nb * p.block_bytes));
    for (int j = 0; j < nb; ++j) {
      int blk = bt[blk0 + j];
      if ((unsigned)blk >= (unsigned)p.num_blocks) {
        flag_status(p.status, TRIATTN_DEV_BAD_BLOCK_ID);
        blk = 0;
      }
      bulk_copy_g2s(smem_u32(smem_tiles + (size_t)stage * stage_bytes + (size_t)j * p.block_bytes),
                    kbase + (long long)blk * p.block_stride_bytes, (uint32_t)p.block_bytes, bar);
    }
  };
  if (tid == 0) {
    const int pre = min(p.stages, my_tiles);
    for (int it = 0; it < pre; ++it) issue(it);
  }

  // register-resident weights of the current KV head: [pair][head slot] for re / im / magnitude
  float2 wre[P2][GP], wim[P2][GP], wmg[P2][GP];
  int cur_head = -1;
  float s1 = 0.f, s2 = 0.f;  // running sum / sum of squares of this lane's (head, query slot)

  auto flush_moments = [&]() {
    if (cur_head < 0) return;
    // lanes with equal lg % GP inside the 16-lane group hold the same query head
#pragma unroll
    for (int s = GP; s < kLPK; s <<= 1) {
      s1 += __shfl_xor_sync(gmask, s1, s);
      s2 += __shfl_xor_sync(gmask, s2, s);
    }
    if (lg < GP && lg < p.g) {
      double* m = p.moments + (((size_t)l * p.B + b) * Hq + (size_t)cur_head * p.g + lg) * 2;
      atomicAdd(m, (double)s1);
      atomicAdd(m + 1, (double)s2);
    }
    s1 = 0.f;
    s2 = 0.f;
  };
  auto load_weights = [&](int head) {
#pragma unroll
    for (int hp = 0; hp < GP; ++hp) {
      const int h = hp ^ lane_lo;
      const bool on = h < p.g;
      const float* w = p.weights + ((((size_t)l * p.B + b) * Hq + (size_t)head * p.g + (on ? h : 0)) * 3) * F + lg * FPT;
#pragma unroll
      for (int c = 0; c < P2; ++c) {
        const float2 z = make_float2(0.f, 0.f);
        wre[c][hp] = on ? __ldg(reinterpret_cast<const float2*>(w + 2 * c)) : z;
        wim[c][hp] = on ? __ldg(reinterpret_cast<const float2*>(w + F + 2 * c)) : z;
        wmg[c][hp] = on ? __ldg(reinterpret_cast<const float2*>(w + 2 * F + 2 * c)) : z;
      }
    }
  };

  const int bph = (p.bs + NT - 1) / NT;        // token batches per cache block
  const int items_per_block = p.Hkv * bph;
  const int n_items = p.mb * items_per_block;

  for (int it = 0; it < my_tiles; ++it) {
    const int stage = it % p.stages;
    const uint32_t parity = (uint32_t)((it / p.stages) & 1);
    const bool ready = mbar_wait_bounded(smem_u32(&full_bar[stage]), parity);
    if (!ready) {
      s_err = 1;
      flag_status(p.status, TRIATTN_DEV_WAIT_TIMEOUT);
    }
    const unsigned char* tile = smem_tiles + (size_t)stage * stage_bytes;
    const int blk0 = (tile0 + it) * p.mb;

    if (ready) {
      for (int item = gid; item < n_items; item += NG) {
        const int head = item % p.Hkv;
        const int q = item / p.Hkv;
        const int batch = q % bph;
        const int mbi = q / bph;
        if (head != cur_head) {
          flush_moments();
          load_weights(head);
          cur_head = head;
        }
        const int tok_base = batch * NT;
        const int gtok_base = (blk0 + mbi) * p.bs;
        const unsigned char* blkp = tile + (size_t)mbi * p.block_bytes + (size_t)head * p.head_stride * 2;

        float2 acc[NT][GP];
#pragma unroll
        for (int tp = 0; tp < NT; ++tp)
#pragma unroll
          for (int hp = 0; hp < GP; ++hp) acc[tp][hp] = make_float2(0.f, 0.f);

#pragma unroll
        for (int tp = 0; tp < NT; ++tp) {
          const int tok = tok_base + (tp ^ lane_hi);
          const bool valid = (tok < p.bs) && (gtok_base + tok < seq_len);
          const unsigned char* row = blkp + (size_t)(valid ? tok : 0) * p.token_stride * 2;
          float2 kre[P2], kim[P2];
          if constexpr (!INTERLEAVED) {
            if constexpr (FPT == 4) {
              const uint2 a = *reinterpret_cast<const uint2*>(row + lg * 8);
              const uint2 c = *reinterpret_cast<const uint2*>(row + F * 2 + lg * 8);
              kre[0] = bf16x2_to_float2(a.x);
              kre[1] = bf16x2_to_float2(a.y);
              kim[0] = bf16x2_to_float2(c.x);
              kim[1] = bf16x2_to_float2(c.y);
            } else {
              kre[0] = bf16x2_to_float2(*reinterpret_cast<const uint32_t*>(row + lg * 4));
              kim[0] = bf16x2_to_float2(*reinterpret_cast<const uint32_t*>(row + F * 2 + lg * 4));
            }
          } else {
            if constexpr (FPT == 4) {
              const uint4 a = *reinterpret_cast<const uint4*>(row + lg * 16);
              const float2 p0 = bf16x2_to_float2(a.x), p1 = bf16x2_to_float2(a.y);
              const float2 p2 = bf16x2_to_float2(a.z), p3 = bf16x2_to_float2(a.w);
              kre[0] = make_float2(p0.x, p1.x);
              kim[0] = make_float2(p0.y, p1.y);
              kre[1] = make_float2(p2.x, p3.x);
              kim[1] = make_float2(p2.y, p3.y);
            } else {
              const uint2 a = *reinterpret_cast<const uint2*>(row + lg * 8);
              const float2 p0 = bf16x2_to_float2(a.x), p1 = bf16x2_to_float2(a.y);
              kre[0] = make_float2(p0.x, p1.x);
              kim[0] = make_float2(p0.y, p1.y);
            }
          }
#pragma unroll
          for (int c = 0; c < P2; ++c) {
            if (!valid) {
              kre[c] = make_float2(0.f, 0.f);
              kim[c] = make_float2(0.f, 0.f);
            }
            float2 m2 = ffma2(kim[c], kim[c], fmul2(kre[c], kre[c]));
            m2.x = sqrt_approx(m2.x);
            m2.y = sqrt_approx(m2.y);
#pragma unroll
            for (int hp = 0; hp < GP; ++hp) {
              float2 a2 = acc[tp][hp];
              a2 = ffma2(kre[c], wre[c][hp], a2);
              a2 = ffma2(kim[c], wim[c][hp], a2);
              a2 = ffma2(m2, wmg[c][hp], a2);
              acc[tp][hp] = a2;
            }
          }
        }

        // collapse the frequency pairs, then reduce-scatter across the 16 lanes
        float v[kLPK];
#pragma unroll
        for (int tp = 0; tp < NT; ++tp)
#pragma unroll
          for (int hp = 0; hp < GP; ++hp) v[tp * GP + hp] = acc[tp][hp].x + acc[tp][hp].y;
#pragma unroll
        for (int s = kLPK / 2; s >= 1; s >>= 1) {
#pragma unroll
          for (int i = 0; i < kLPK; ++i) {
            if ((i & s) == 0 && i < 2 * s) v[i] += __shfl_xor_sync(gmask, v[i | s], s);
          }
        }
        // lane lg now owns token tok_base + lg/GP, query slot lg%GP
        const int tok = tok_base + lane_hi;
        const int gtok = gtok_base + tok;
        if (tok < p.bs && gtok < seq_len && lane_lo < p.g) {
          const float sc = v[0];
          p.raw[((((size_t)l * p.B + b) * p.Hkv + head) * (size_t)p.t_pad + gtok) * GP + lane_lo] = sc;
          s1 += sc;
          s2 = fmaf(sc, sc, s2);
        }
      }
    }
    __syncthreads();  // every lane is done reading this stage
    if (s_err) break;
    if (tid == 0 && it + p.stages < my_tiles) issue(it + p.stages);
  }
  flush_moments();

  if (s_err && tid == 0) {
    // give copies that may still be in flight into this CTA's shared memory a bounded chance to land
    for (int it = 0; it < my_tiles && it < p.stages; ++it) {
      (void)mbar_wait_bounded(smem_u32(&full_bar[it % p.stages]), 0u);
    }
  }
}

// Generic scorer: any head_dim / group size / offset aggregation (mean or max).  One thread per
// (token, KV head); K is read straight from global memory (cache resident between passes).
// Weight rows: MEAN {w_re, w_im, w_mag}; MAX {w_re[o]..., w_im[o]..., w_mag}.
__global__ void score_paged_generic_kernel(const __grid_constant__ ScoreParams p, int D, int GP, int interleaved) {
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
