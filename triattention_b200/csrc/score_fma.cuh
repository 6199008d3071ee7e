// Key scorer on the CUDA cores only (no tensor cores), offset aggregation = mean, head_dim 64 or 128.
// Selected with TRIATTN_SCORE_PATH=fma; the default streaming kernel is the tensor-core one (score_mma.cuh),
// which does the same contraction with mma.sync and is bound by HBM instead of fp32 issue slots.
//
//   * a CTA owns a run of consecutive cache blocks of one (layer, request); each pipeline stage holds `mb`
//     whole cache blocks (all KV heads) fetched by 1-D bulk async copies (TMA) that complete on an mbarrier;
//     the last of the 8 warps to release a stage refills it (no CTA-wide barrier in the loop);
//   * 16 lanes share a key: lane j owns frequencies [j*FPT, (j+1)*FPT) and keeps the folded weights of its
//     frequencies for all GP query heads in registers (packed as fp32x2 over adjacent frequencies, so the
//     inner loop is fma.rn.f32x2 on naturally paired bf16 data);
//   * a batch of NT = 16/GP tokens gives 16 partial sums per lane, combined across the 16 lanes with a
//     select-free reduce-scatter: lane j accumulates logical value (token, head) in register slot (idx ^ j),
//     so every lane sends the slots with the exchanged bits set and keeps the others; after two radix-4
//     steps (15 shuffles) lane j holds the finished score of token j/GP, head j%GP and the 16 lanes store
//     64 contiguous bytes.
#pragma once

#include <type_traits>

#include "score.cuh"

namespace triattn {

constexpr int kLPK = 16;  // lanes per key
constexpr int kScoreConsumerThreads = kScoreConsumerWarps * 32;
constexpr int kScoreFmaMinCtas = 2;  // CTAs per SM the register budget is held to

// One (virtual head, token-batch) work item of a pipeline stage; the table is identical for every stage.
// A KV head with g > 4 query heads is split into ceil(g/4) virtual heads of <= 4 query heads that read
// the same K rows, so the register-resident weight set never exceeds 4 query heads.
struct ScoreItem {
  int smem_off;  // byte offset of (cache block, KV head, first token of the batch) inside the stage
  int tok_rel;   // token index of the batch's first token relative to the stage's first token
  int vhead;     // virtual head = kv_head * nsub + sub
  int pad;
};
constexpr int kMaxScoreItems = 256;

// GP = query-head slots per virtual head (1, 2 or 4).  p.gp_total = slots per KV head in the raw layout.
template <int D, int GP, bool INTERLEAVED>
__global__ void __launch_bounds__(kScoreThreadsWS, kScoreFmaMinCtas)
score_paged_mean_kernel(const __grid_constant__ ScoreParams p) {
  constexpr int F = D / 2;
  constexpr int FPT = F / kLPK;  // frequencies per lane: 4 (D=128) or 2 (D=64)
  constexpr int P2 = FPT / 2;    // fp32x2 pairs per lane per component
  constexpr int NT = kLPK / GP;  // tokens per batch
  constexpr int NG = kScoreConsumerThreads / kLPK;
  static_assert(FPT >= 2 && (FPT % 2) == 0, "head_dim must be 64 or 128");
  static_assert(NT >= 1 && NT * GP == kLPK, "GP must divide 16");

  extern __shared__ __align__(128) unsigned char smem_tiles[];
  __shared__ __align__(16) ScoreItem s_items[kMaxScoreItems];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];  // reader warps done with each stage
  __shared__ unsigned int s_issued[kMaxStages];    // copies armed so far, per stage barrier
  __shared__ int s_bt[kMaxPrefetchedBlocks];  // this CTA's slice of the block table
  __shared__ int s_err;

  const int tid = threadIdx.x;
  const int l = blockIdx.y, b = blockIdx.z;

  grid_dependency_wait();  // no global access before the preceding kernel of the stream has completed
  trigger_dependents();
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
  const int stage_tokens = p.mb * p.bs;
  const int Hq = p.Hkv * p.g;
  const int nsub = p.gp_total / GP;  // virtual heads per KV head (1 unless g > 4)
  const int nvh = p.Hkv * nsub;
  // Token batches of a stage.  In NHD order the blocks of a stage sit back to back with one uniform token
  // stride, so the stage is a dense [mb*bs tokens, heads, D] array and batches may span cache blocks (this
  // covers blocks smaller than a batch, down to token-granular pools with block_size 1).  Otherwise batches
  // stay inside a block (the host guarantees block_size % NT == 0 then).
  const int bph = p.nhd ? stage_tokens / NT : p.bs / NT;
  const int n_items = (p.nhd ? 1 : p.mb) * nvh * bph;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), kScoreConsumerWarps);
      s_issued[s] = 0u;
    }
    mbar_fence_init();
    s_err = 0;
  }
  for (int i = tid; i < n_items; i += kScoreThreadsWS) {
    const int vh = i % nvh;
    const int q = i / nvh;
    const int batch = q % bph;
    const int mbi = q / bph;  // always 0 in NHD order
    ScoreItem it;
    it.smem_off = mbi * p.block_bytes + ((vh / nsub) * p.head_stride + batch * NT * p.token_stride) * 2;
    it.tok_rel = mbi * p.bs + batch * NT;
    it.vhead = vh;
    it.pad = 0;
    s_items[i] = it;
  }
  // block ids of this CTA's tiles (bounds-checked once here), so the refill path never waits on global memory
  const int32_t* bt = p.block_table + (size_t)b * p.max_blocks;
  const int my_blocks = min(my_tiles * p.mb, nblk - tile0 * p.mb);
  const bool bt_in_smem = my_blocks <= kMaxPrefetchedBlocks;
  if (bt_in_smem) {
    for (int i = tid; i < my_blocks; i += kScoreThreadsWS) {
      int blk = bt[tile0 * p.mb + i];
      if ((unsigned)blk >= (unsigned)p.num_blocks) {
        flag_status(p.status, TRIATTN_DEV_BAD_BLOCK_ID);
        blk = 0;
      }
      s_bt[i] = blk;
    }
  }
  __syncthreads();

  // fetch the cache blocks of stage-tile `it` (called by one lane)
  const unsigned char* kbase = reinterpret_cast<const unsigned char*>(p.k_ptrs[l]);
  // Fetch the cache blocks of stage-tile `it`.  Called by a whole (converged) warp: lane 0 arms the barrier
  // with the byte count, then lane j issues the copy of block j, so a stage made of several small cache
  // blocks costs one issue slot per lane instead of a serial loop.
  auto issue = [&](int it, int stage, int lane_id) {
    const uint32_t bar = smem_u32(&full_bar[stage]);
    const int blk0 = (tile0 + it) * p.mb;
    const int nb = min(p.mb, nblk - blk0);
    if (lane_id == 0) {
      mbar_arrive_expect_tx(bar, (uint32_t)(nb * p.block_bytes) + kTestExtraTxBytes);
      s_issued[stage] += 1u;  // one issuer at a time: the issuers of a stage are ordered by its reader barrier
    }
    __syncwarp();
    for (int j = lane_id; j < nb; j += 32) {
      int blk;
      if (bt_in_smem) {
        blk = s_bt[it * p.mb + j];
      } else {
        blk = bt[blk0 + j];
        if ((unsigned)blk >= (unsigned)p.num_blocks) {
          flag_status(p.status, TRIATTN_DEV_BAD_BLOCK_ID);
          blk = 0;
        }
      }
      bulk_copy_g2s(smem_u32(smem_tiles + (size_t)stage * stage_bytes + (size_t)j * p.block_bytes),
                    kbase + (long long)blk * p.block_stride_bytes, (uint32_t)p.block_bytes, bar);
    }
  };
  if (tid < 32) {
    const int pre = min(p.stages, my_tiles);
    for (int it = 0; it < pre; ++it) issue(it, it, tid);
  }

  // ---------------------------------------------------------------- consumers (all 8 warps)
  // The two 16-lane key groups of a warp run in lockstep (same trip counts, warp-uniform branches), so
  // every shuffle uses the full-warp mask; xor distances < 16 never cross the group boundary.
  constexpr unsigned kFull = 0xffffffffu;
  const int lane = tid & 31;
  const int lg = tid & (kLPK - 1);  // lane within the key group
  const int gid = tid / kLPK;
  const int lane_lo = lg % GP;      // permutes head slots
  const int lane_hi = lg / GP;      // permutes token slots

  // register-resident weights of the current virtual head: [pair][head slot] for re / im / magnitude
  float2 wre[P2][GP], wim[P2][GP], wmg[P2][GP];
  int cur_vh = -1;
  int cur_qbase = 0;           // first query head (within the layer) of the current virtual head
  int cur_nq = 0;              // valid query slots of the current virtual head
  float s1 = 0.f, s2 = 0.f;    // running sum / sum of squares of this lane's (virtual head, query slot)
  float* raw_head = nullptr;   // raw-score rows of (l, b, kv head), pre-offset by sub*GP and this lane's slot

  // 32-bit byte offsets into smem_tiles of this lane's slice of token slot tp (slot tp holds token tp ^ lane_hi)
  const unsigned lane_byte = (unsigned)lg * (INTERLEAVED ? FPT * 4 : FPT * 2);
  unsigned lane_off[NT];
#pragma unroll
  for (int tp = 0; tp < NT; ++tp) lane_off[tp] = (unsigned)((tp ^ lane_hi) * p.token_stride * 2) + lane_byte;
  const int gp_total = p.gp_total;

  auto flush_moments = [&]() {
    if (cur_vh < 0) return;
    // lanes with equal lg % GP inside the 16-lane group hold the same query head
#pragma unroll
    for (int s = GP; s < kLPK; s <<= 1) {
      s1 += __shfl_xor_sync(kFull, s1, s);
      s2 += __shfl_xor_sync(kFull, s2, s);
    }
    if (lg < GP && lg < cur_nq) {
      double* m = p.moments + (((size_t)l * p.B + b) * Hq + (size_t)cur_qbase + lg) * 2;
      atomicAdd(m, (double)s1);
      atomicAdd(m + 1, (double)s2);
    }
    s1 = 0.f;
    s2 = 0.f;
  };
  auto load_weights = [&](int vh) {
    const int kvh = vh / nsub, sub = vh - kvh * nsub;
    cur_qbase = kvh * p.g + sub * GP;
    cur_nq = min(GP, p.g - sub * GP);
#pragma unroll
    for (int hp = 0; hp < GP; ++hp) {
      const int h = hp ^ lane_lo;
      const bool on = h < cur_nq;
      const float* w = p.weights + ((((size_t)l * p.B + b) * Hq + (size_t)cur_qbase + (on ? h : 0)) * 3) * F + lg * FPT;
#pragma unroll
      for (int c = 0; c < P2; ++c) {
        const float2 z = make_float2(0.f, 0.f);
        wre[c][hp] = on ? __ldg(reinterpret_cast<const float2*>(w + 2 * c)) : z;
        wim[c][hp] = on ? __ldg(reinterpret_cast<const float2*>(w + F + 2 * c)) : z;
        wmg[c][hp] = on ? __ldg(reinterpret_cast<const float2*>(w + 2 * F + 2 * c)) : z;
      }
    }
    raw_head = p.raw + (((size_t)l * p.B + b) * p.Hkv + kvh) * (size_t)p.t_pad * gp_total + sub * GP +
               lane_hi * gp_total + lane_lo;
  };

  // one (virtual head, batch of NT tokens) item; `checked` = the stage may hold tokens beyond seq_len.
  // `live` is false only for the padding item of a group when n_items is not a multiple of the group count.
  auto compute_item = [&](const unsigned base, const int gtok0, bool live, auto checked) {
    constexpr bool CHECK = decltype(checked)::value;

    float2 acc[NT][GP];
#pragma unroll
    for (int tp = 0; tp < NT; ++tp)
#pragma unroll
      for (int hp = 0; hp < GP; ++hp) acc[tp][hp] = make_float2(0.f, 0.f);

#pragma unroll
    for (int tp = 0; tp < NT; ++tp) {
      bool valid = true;
      if constexpr (CHECK) valid = gtok0 + (tp ^ lane_hi) < seq_len;
      const unsigned char* row = smem_tiles + (base + (valid ? lane_off[tp] : lane_byte));  // invalid: token 0, zeroed
      float2 kre[P2], kim[P2];
      if constexpr (!INTERLEAVED) {
        if constexpr (FPT == 4) {
          const uint2 a = *reinterpret_cast<const uint2*>(row);
          const uint2 c = *reinterpret_cast<const uint2*>(row + F * 2);
          kre[0] = bf16x2_to_float2(a.x);
          kre[1] = bf16x2_to_float2(a.y);
          kim[0] = bf16x2_to_float2(c.x);
          kim[1] = bf16x2_to_float2(c.y);
        } else {
          kre[0] = bf16x2_to_float2(*reinterpret_cast<const uint32_t*>(row));
          kim[0] = bf16x2_to_float2(*reinterpret_cast<const uint32_t*>(row + F * 2));
        }
      } else {
        if constexpr (FPT == 4) {
          const uint4 a = *reinterpret_cast<const uint4*>(row);
          const float2 p0 = bf16x2_to_float2(a.x), p1 = bf16x2_to_float2(a.y);
          const float2 p2 = bf16x2_to_float2(a.z), p3 = bf16x2_to_float2(a.w);
          kre[0] = make_float2(p0.x, p1.x);
          kim[0] = make_float2(p0.y, p1.y);
          kre[1] = make_float2(p2.x, p3.x);
          kim[1] = make_float2(p2.y, p3.y);
        } else {
          const uint2 a = *reinterpret_cast<const uint2*>(row);
          const float2 p0 = bf16x2_to_float2(a.x), p1 = bf16x2_to_float2(a.y);
          kre[0] = make_float2(p0.x, p1.x);
          kim[0] = make_float2(p0.y, p1.y);
        }
      }
#pragma unroll
      for (int c = 0; c < P2; ++c) {
        if constexpr (CHECK) {
          if (!valid) {
            kre[c] = make_float2(0.f, 0.f);
            kim[c] = make_float2(0.f, 0.f);
          }
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
    // radix-4 reduce-scatter: two latency levels instead of four, still 15 shuffles.  Slot p holds logical value
    // p ^ lg, so for every xor distance d a lane keeps the slots with the d-bits clear and sends slot p | d.
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float t1 = __shfl_xor_sync(kFull, v[q | 4], 4);
      const float t2 = __shfl_xor_sync(kFull, v[q | 8], 8);
      const float t3 = __shfl_xor_sync(kFull, v[q | 12], 12);
      v[q] = (v[q] + t1) + (t2 + t3);
    }
    {
      const float t1 = __shfl_xor_sync(kFull, v[1], 1);
      const float t2 = __shfl_xor_sync(kFull, v[2], 2);
      const float t3 = __shfl_xor_sync(kFull, v[3], 3);
      v[0] = (v[0] + t1) + (t2 + t3);
    }
    // lane lg now owns token gtok0 + lg/GP, query slot lg%GP
    bool store = live && (lane_lo < cur_nq);
    if constexpr (CHECK) store = store && (gtok0 + lane_hi < seq_len);
    if (store) {
      const float sc = v[0];
      raw_head[(size_t)gtok0 * gp_total] = sc;
      s1 += sc;
      s2 = fmaf(sc, sc, s2);
    }
  };

  // general path: the virtual head may change from item to item
  auto process_item = [&](unsigned tile_off, const ScoreItem it, int tile_tok0, bool live, auto checked) {
    if (__any_sync(kFull, it.vhead != cur_vh)) {  // warp-uniform: both key groups switch together
      flush_moments();
      load_weights(it.vhead);
      cur_vh = it.vhead;
    }
    compute_item(tile_off + (unsigned)it.smem_off, tile_tok0 + it.tok_rel, live, checked);
  };

  const int slots = (n_items + NG - 1) / NG;  // items per key group and stage (uniform over the CTA)
  // common case: every key group keeps one virtual head for the whole CTA and has at most kMaxFixedSlots items
  // per stage; its item descriptors and weights then live in registers for the whole kernel
  constexpr int kMaxFixedSlots = 4;
  const bool fixed = (NG % nvh) == 0 && slots <= kMaxFixedSlots && slots * NG == n_items;
  unsigned f_off[kMaxFixedSlots];
  int f_tok[kMaxFixedSlots];
#pragma unroll
  for (int sl = 0; sl < kMaxFixedSlots; ++sl) {
    const ScoreItem d = s_items[min(gid + sl * NG, n_items - 1)];
    f_off[sl] = (unsigned)d.smem_off;
    f_tok[sl] = d.tok_rel;
  }
  if (fixed) {
    cur_vh = gid % nvh;
    load_weights(cur_vh);
  }
  int stage = 0;
  uint32_t parity = 0;
  for (int it = 0; it < my_tiles; ++it) {
    // warp-uniform outcome, so that the shuffles below never see a split warp
    const bool ready = __all_sync(kFull, mbar_wait_bounded(smem_u32(&full_bar[stage]), parity, &s_err));
    if (!ready) {
      if (lane == 0) {
        if (s_err == 0) flag_status(p.status, TRIATTN_DEV_WAIT_TIMEOUT);
        s_err = 1;
      }
      break;
    }
    const unsigned tile_off = (unsigned)(stage * stage_bytes);
    const int tile_tok0 = (tile0 + it) * stage_tokens;
    if (fixed && tile_tok0 + stage_tokens <= seq_len) {
#pragma unroll
      for (int sl = 0; sl < kMaxFixedSlots; ++sl)
        if (sl < slots) compute_item(tile_off + f_off[sl], tile_tok0 + f_tok[sl], true, std::false_type{});
    } else if (tile_tok0 + stage_tokens <= seq_len && slots * NG == n_items) {
      for (int sl = 0; sl < slots; ++sl)
        process_item(tile_off, s_items[gid + sl * NG], tile_tok0, true, std::false_type{});
    } else {
      for (int sl = 0; sl < slots; ++sl) {
        const int item = gid + sl * NG;
        const bool live = item < n_items;
        process_item(tile_off, s_items[live ? item : 0], tile_tok0, live, std::true_type{});
      }
    }
    // Release the stage: the warp whose release is the last of the 8 refills it with the tile `stages` ahead -
    // nobody waits for it.
    __syncwarp();
    unsigned refill = 0u;
    if (lane == 0 && release_and_check_last(smem_u32(&empty_bar[stage])) && it + p.stages < my_tiles) refill = 1u;
    if (__shfl_sync(kFull, refill, 0)) {
      fence_proxy_async();  // generic-proxy reads of the stage before this lane's async-proxy refill copies
      issue(it + p.stages, stage, lane);
    }
    if (++stage == p.stages) {
      stage = 0;
      parity ^= 1u;
    }
  }
  flush_moments();
  // No thread leaves while a copy may still be on its way into this CTA's shared memory: after a timeout
  // (and only then) one lane per stage waits once more, bounded, for every copy that was armed.
  __syncthreads();
  if (s_err != 0 && tid < p.stages) {
    const unsigned n = s_issued[tid];
    if (n > 0u) mbar_wait_bounded(smem_u32(&full_bar[tid]), (n - 1u) & 1u);
  }
}

}  // namespace triattn
