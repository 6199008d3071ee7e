// Key scorer on the warp-level tensor-core path (mma.sync m16n8k16 bf16), offset aggregation = mean.
//
// With the offsets folded into per-frequency weights the score of a key for the query heads of its KV head is
// a small matrix product: [16 keys x 3F] x [3F x heads], where the 3F entries are re(k), im(k) and |k|.
//   * g <= 4: keys are the A operand (M = 16 keys per MMA), weights the B operand: the 8 output columns of an
//     MMA are 4 query heads x {high, low} part of the fp32 weight (column n = 2*head + part; bf16 high part and
//     bf16 of the remainder, accurate to ~2^-17).
//   * 5 <= g <= 8 (per virtual head of 8): the product is transposed.  The weights are the A operand - M = 16
//     rows = 8 query heads x {high, low} part, loop-invariant registers - and 8 keys are the B operand, whose
//     two registers per thread are adjacent words of ONE 16-byte shared-memory load of one key row, so no
//     register is moved between the load and the MMA (with keys as the A operand every A quad interleaves the
//     words of two loads, which cost 57 moves per 16 keys and made this shape issue-bound).
//   * re / im are the cached bf16 values themselves, so they go from shared memory into the MMA unchanged.
//   * |k| = sqrt(re^2 + im^2) is computed in fp32 on the CUDA cores (re^2 + im^2 by mixed-precision FMAs straight
//     from the packed bf16 pair) and split into its bf16 rounding and the bf16 of the exact remainder (four
//     instructions per pair of values); both parts extend the K dimension of the magnitude MMAs.
//   * The K dimension of a dot product may be visited in any order, so every thread reads whole 16-byte chunks
//     of "its" two keys (rows lane/4 and lane/4+8 of the tile, chunks lane%4 + 4q) and the weight fragments are
//     permuted once per CTA to match: no ldmatrix and no cross-lane reduction; a thread ends up with the two
//     parts of query head lane%4 for its two keys, and their sum is the finished score.
// Data movement: a CTA owns a run of consecutive cache blocks of one (layer, request); each pipeline stage holds
// `mb` whole cache blocks (all KV heads) fetched by 1-D bulk async copies (TMA) that complete on an mbarrier
// (bounded waits).  There is no CTA-wide barrier in the loop: a warp that finishes a stage bumps a shared
// counter and the last of the 8 warps to do so refills the stage with the tile `stages` ahead.  In token-major
// (NHD) order the blocks of a stage form one dense token array, so 16-key tiles may span cache blocks (block
// sizes down to 1).
#pragma once

#include "score.cuh"

namespace triattn {

constexpr int kScoreMmaMinCtas = 2;  // CTAs per SM the register budget is held to

constexpr int kMmaKeys = 16;  // keys per MMA tile and work item

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// d = a * b (no accumulator input: the first MMA of a chain needs no zeroed registers)
__device__ __forceinline__ void mma_bf16_16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                     uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// bf16 (round to nearest even) of x, as the upper 16 bits of an fp32 pattern
__device__ __forceinline__ uint32_t bf16_bits_rn(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
}
// x = hi + lo with hi = bf16(x), lo = bf16(x - hi); both returned in the low 16 bits
__device__ __forceinline__ void bf16_split(float x, uint32_t& hi16, uint32_t& lo16) {
  const uint32_t hi = bf16_bits_rn(x);
  hi16 = hi >> 16;
  lo16 = bf16_bits_rn(x - __uint_as_float(hi)) >> 16;
}
// two fp32 -> bf16x2 (round to nearest even), `lo` in the low half
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}


// NT = column tiles of 4 query heads per virtual head (1: g <= 4, 2: g <= 8; larger groups are split into
// virtual heads of 8 that read the same K rows).
template <int D, bool INTERLEAVED, int NT>
__global__ void __launch_bounds__(kScoreThreadsWS, kScoreMmaMinCtas)
score_paged_mma_kernel(const __grid_constant__ ScoreParams p) {
  constexpr int F = D / 2;
  constexpr int NQ = D / 32;  // 16-byte chunks per key and thread: chunk index lane%4 + 4q
  constexpr int GP = 4 * NT;  // query-head slots per virtual head
  static_assert(D == 64 || D == 128, "head_dim must be 64 or 128");

  extern __shared__ __align__(128) unsigned char smem_tiles[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t blk_bar[kMaxStages][kScoreConsumerWarps];  // block-group mode: one per block
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];                           // readers done, per stage
  __shared__ __align__(8) uint64_t blk_empty_bar[kMaxStages][kScoreConsumerWarps];  // readers done, per block
  __shared__ unsigned int s_blk_issued[kMaxStages][kScoreConsumerWarps];  // copies armed so far, per barrier
  __shared__ unsigned int s_issued[kMaxStages];
  __shared__ int s_bt[kMaxPrefetchedBlocks];
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
  const int nsub = (p.gp_total + GP - 1) / GP;  // virtual heads per KV head
  const int nvh = p.Hkv * nsub;
  const int ntt = (stage_tokens + kMmaKeys - 1) / kMmaKeys;  // 16-key items per stage and virtual head
  const int n_items = ntt * nvh;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), kScoreConsumerWarps);
      s_issued[s] = 0u;
      for (int w = 0; w < kScoreConsumerWarps; ++w) {
        mbar_init(smem_u32(&blk_bar[s][w]), 1);
        mbar_init(smem_u32(&blk_empty_bar[s][w]), (uint32_t)max(p.block_group, 1));
        s_blk_issued[s][w] = 0u;
      }
    }
    mbar_fence_init();
    s_err = 0;
  }
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

  const unsigned char* kbase = reinterpret_cast<const unsigned char*>(p.k_ptrs[l]);
  // Fetch the cache blocks of stage-tile `it`: lane 0 arms the barrier, lane j copies block j.
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
  // Block-group mode (16-token blocks, Hkv * mb == 8, one virtual head per KV head): block j of every stage is
  // read only by the Hkv warps that own its heads, so every block has its own barrier and release counter and is
  // refilled as soon as ITS readers are done - a single-head shard runs 8 independent per-warp rings, two heads
  // 4 rings of 2 warps, and nobody waits for the slowest warp of the CTA.  Called by one lane.
  auto issue_block = [&](int it, int stage, int j) {
    const int bi = (tile0 + it) * p.mb + j;
    if (bi >= nblk) return;
    int blk;
    if (bt_in_smem) {
      blk = s_bt[it * p.mb + j];
    } else {
      blk = bt[bi];
      if ((unsigned)blk >= (unsigned)p.num_blocks) {
        flag_status(p.status, TRIATTN_DEV_BAD_BLOCK_ID);
        blk = 0;
      }
    }
    const uint32_t bar = smem_u32(&blk_bar[stage][j]);
    mbar_arrive_expect_tx(bar, (uint32_t)p.block_bytes + kTestExtraTxBytes);
    s_blk_issued[stage][j] += 1u;
    bulk_copy_g2s(smem_u32(smem_tiles + (size_t)stage * stage_bytes + (size_t)j * p.block_bytes),
                  kbase + (long long)blk * p.block_stride_bytes, (uint32_t)p.block_bytes, bar);
  };
  if (p.block_group > 0) {
    // the first warp of each reader group starts its block's ring
    const int w0 = tid >> 5;
    if ((tid & 31) == 0 && (w0 % p.block_group) == 0) {
      const int pre = min(p.stages, my_tiles);
      for (int it = 0; it < pre; ++it) issue_block(it, it, w0 / p.block_group);
    }
  } else if (tid < 32) {
    const int pre = min(p.stages, my_tiles);
    for (int it = 0; it < pre; ++it) issue(it, it, tid);
  }

  constexpr unsigned kFull = 0xffffffffu;
  const int lane = tid & 31, wid = tid >> 5;
  const int rg = lane >> 2;  // this thread owns keys (rows) rg and rg + 8 of a tile; in B: output column rg
  const int rt = lane & 3;   // chunk selector; in the result: query-head slot rt of each column tile
  const int b_head = rg >> 1, b_part = rg & 1;  // column rg of a weight fragment = (head within the tile, part)

  // weight fragments (B operands) of the current virtual head, permuted to the chunk order of the loads
  uint32_t bri[NT][NQ][2][2];  // re/im: [column tile][chunk][half of the chunk][b0, b1]
  uint32_t bmg[NT][NQ][2];     // magnitude: [column tile][4 consecutive frequencies][b0, b1]
  // transposed form (NT == 2): A fragments of query head rg, rows rg (high part) and rg + 8 (low part)
  uint32_t ari[NQ][2][4];      // re/im: [chunk][half of the chunk][a0..a3]
  uint32_t amg[NQ][4];         // magnitude: [4 consecutive frequencies][a0..a3]
  int cur_vh = -1, cur_qbase = 0, cur_nq = 0;
  // Running sum / sum of squares of this thread's query slot(s) over its keys, in double: the scores of one
  // 16-key tile are summed in fp32 in a fixed order, and a double accumulates such fp32 sums exactly, so the
  // moments - and with them every later stage - do not depend on how the tiles were split over CTAs and warps
  // (the same request gives the same keep set whatever else is in the batch).
  double s1[NT], s2[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) s1[nt] = s2[nt] = 0.0;
  float* raw_head = nullptr;
  const uint32_t smem_base = smem_u32(smem_tiles);
  const int gp_total = p.gp_total;

  auto flush_moments = [&]() {
    if (cur_vh < 0) return;
    if constexpr (NT == 2) {
      // the thread's sums belong to query head rg: combine the 4 lanes of the head, one atomic pair per head
      s1[0] += __shfl_xor_sync(kFull, s1[0], 1);
      s2[0] += __shfl_xor_sync(kFull, s2[0], 1);
      s1[0] += __shfl_xor_sync(kFull, s1[0], 2);
      s2[0] += __shfl_xor_sync(kFull, s2[0], 2);
      // (sums of squares round in double; their order over lanes is fixed)
      if (rt == 0 && rg < cur_nq) {
        double* m = p.moments + (((size_t)l * p.B + b) * Hq + (size_t)cur_qbase + rg) * 2;
        atomicAdd(m, s1[0]);
        atomicAdd(m + 1, s2[0]);
      }
      s1[0] = s2[0] = 0.0;
    } else {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int s = 4; s < 32; s <<= 1) {
          s1[nt] += __shfl_xor_sync(kFull, s1[nt], s);
          s2[nt] += __shfl_xor_sync(kFull, s2[nt], s);
        }
        if (lane < 4 && 4 * nt + lane < cur_nq) {
          double* m = p.moments + (((size_t)l * p.B + b) * Hq + (size_t)cur_qbase + 4 * nt + lane) * 2;
          atomicAdd(m, s1[nt]);
          atomicAdd(m + 1, s2[nt]);
        }
        s1[nt] = 0.0;
        s2[nt] = 0.0;
      }
    }
  };
  // 4 consecutive weights starting at w -> this thread's column part, packed as (b0, b1)
  auto pack_part = [&](const float (&x)[4], bool on, uint32_t& b0, uint32_t& b1) {
    uint32_t v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      uint32_t hi, lo;
      bf16_split(on ? x[e] : 0.f, hi, lo);
      v[e] = b_part ? lo : hi;
    }
    b0 = v[0] | (v[1] << 16);
    b1 = v[2] | (v[3] << 16);
  };
  auto load_weights = [&](int vh) {
    const int kvh = vh / nsub, sub = vh - kvh * nsub;
    cur_qbase = kvh * p.g + sub * GP;
    cur_nq = min(GP, p.g - sub * GP);
    if constexpr (NT == 2) {
      // rows rg / rg + 8 of every A fragment: high / low bf16 part of query head rg's weights
      const bool on = rg < cur_nq;
      const float* w = p.weights + ((((size_t)l * p.B + b) * Hq + (size_t)cur_qbase + (on ? rg : 0)) * 3) * F;
      auto pack4 = [&](const float (&x)[4], uint32_t (&a)[4]) {
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) bf16_split(on ? x[e] : 0.f, hi[e], lo[e]);
        a[0] = hi[0] | (hi[1] << 16);  // row rg,     k = 2t, 2t+1
        a[1] = lo[0] | (lo[1] << 16);  // row rg + 8, k = 2t, 2t+1
        a[2] = hi[2] | (hi[3] << 16);  // row rg,     k = 2t+8, 2t+9
        a[3] = lo[2] | (lo[3] << 16);  // row rg + 8, k = 2t+8, 2t+9
      };
#pragma unroll
      for (int c = 0; c < NQ; ++c)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int d0 = 8 * (rt + 4 * c) + 4 * h;
          float x[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int d = d0 + e;
            x[e] = INTERLEAVED ? __ldg(w + (d & 1) * F + (d >> 1)) : __ldg(w + d);
          }
          pack4(x, ari[c][h]);
        }
      const float* wm = w + 2 * F;
#pragma unroll
      for (int j = 0; j < NQ; ++j) {
        const int f0 = INTERLEAVED ? 4 * (rt + 4 * j) : 8 * (rt + 4 * (j >> 1)) + 4 * (j & 1);
        float x[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) x[e] = __ldg(wm + f0 + e);
        pack4(x, amg[j]);
      }
      // the thread's results: query head rg, keys 2*rt and 2*rt + 1 of each 8-key group
      raw_head = p.raw + (((size_t)l * p.B + b) * p.Hkv + kvh) * (size_t)p.t_pad * gp_total + sub * GP + rg;
    } else {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int head = 4 * nt + b_head;
        const bool on = head < cur_nq;
        const float* w = p.weights + ((((size_t)l * p.B + b) * Hq + (size_t)cur_qbase + (on ? head : 0)) * 3) * F;
#pragma unroll
        for (int c = 0; c < NQ; ++c) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int d0 = 8 * (rt + 4 * c) + 4 * h;  // the thread's 4 consecutive dims of this MMA
            float x[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int d = d0 + e;
              // half layout: rows re | im of the weight record are contiguous, so dim d is element d
              x[e] = INTERLEAVED ? __ldg(w + (d & 1) * F + (d >> 1)) : __ldg(w + d);
            }
            pack_part(x, on, bri[nt][c][h][0], bri[nt][c][h][1]);
          }
        }
        const float* wm = w + 2 * F;
#pragma unroll
        for (int j = 0; j < NQ; ++j) {
          // 4 consecutive frequencies per magnitude MMA, in the order compute_item produces |k|
          const int f0 = INTERLEAVED ? 4 * (rt + 4 * j) : 8 * (rt + 4 * (j >> 1)) + 4 * (j & 1);
          float x[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) x[e] = __ldg(wm + f0 + e);
          pack_part(x, on, bmg[nt][j][0], bmg[nt][j][1]);
        }
      }
      raw_head = p.raw + (((size_t)l * p.B + b) * p.Hkv + kvh) * (size_t)p.t_pad * gp_total + sub * GP + rt;
    }
  };

  // shared-memory byte offset (inside a stage) of token `tk` of the stage for KV head `kvh`
  auto row_offset = [&](int tk, int kvh) -> uint32_t {
    if (p.nhd) return (uint32_t)((tk * p.token_stride + kvh * p.head_stride) * 2);
    const int j = tk / p.bs, in = tk - j * p.bs;
    return (uint32_t)(j * p.block_bytes + (kvh * p.head_stride + in * p.token_stride) * 2);
  };

  // One work item: 16 keys of the current virtual head.  rowA / rowB = shared-memory address of this thread's 16-byte
  // chunk `rt` of the item's key rg / rg + 8, tok0 = token index (in the request) of the item's first key, valid =
  // how many of the 16 keys exist (inside the stage and below seq_len); with all 16 the stores need no per-key test.
  auto compute_rows = [&](uint32_t rowA, uint32_t rowB, int tok0, int valid) {
    const bool full = valid >= kMmaKeys;
    if constexpr (NT == 2) {
      // Transposed form.  Group A = keys tt*16 + 0..7, group B = keys tt*16 + 8..15; this thread feeds key rg of each
      // group as column rg of the B operand and ends with query head rg's score for keys 2*rt, 2*rt + 1 of each group.
      float accA[2][4], accB[2][4];
      auto mma_t = [&](float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        mma_bf16_16816(d, a[0], a[1], a[2], a[3], b0, b1);
      };
      auto mma_t0 = [&](bool first, float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        if (first) mma_bf16_16816_first(d, a[0], a[1], a[2], a[3], b0, b1);
        else mma_bf16_16816(d, a[0], a[1], a[2], a[3], b0, b1);
      };
      auto split_pair = [&](float m0, float m1, uint32_t& hi, uint32_t& lo) { split_bf16x2_hi_lo(m0, m1, hi, lo); };
      if constexpr (!INTERLEAVED) {
#pragma unroll
        for (int q = 0; q < NQ / 2; ++q) {
          constexpr int QI = NQ / 2;
          const uint4 reA = lds128(rowA + 64u * q), reB = lds128(rowB + 64u * q);
          const uint4 imA = lds128(rowA + 64u * q + D), imB = lds128(rowB + 64u * q + D);
          mma_t0(q == 0, accA[0], ari[q][0], reA.x, reA.y);
          mma_t0(q == 0, accB[0], ari[q][0], reB.x, reB.y);
          mma_t0(q == 0, accA[1], ari[q][1], reA.z, reA.w);
          mma_t0(q == 0, accB[1], ari[q][1], reB.z, reB.w);
          mma_t(accA[0], ari[q + QI][0], imA.x, imA.y);
          mma_t(accB[0], ari[q + QI][0], imB.x, imB.y);
          mma_t(accA[1], ari[q + QI][1], imA.z, imA.w);
          mma_t(accB[1], ari[q + QI][1], imB.z, imB.w);
          const uint32_t rA[4] = {reA.x, reA.y, reA.z, reA.w}, rB[4] = {reB.x, reB.y, reB.z, reB.w};
          const uint32_t iA[4] = {imA.x, imA.y, imA.z, imA.w}, iB[4] = {imB.x, imB.y, imB.z, imB.w};
          uint32_t hA[4], lA[4], hB[4], lB[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 ma = sq_mag_bf16x2(rA[i], iA[i]);
            const float2 mb = sq_mag_bf16x2(rB[i], iB[i]);
            split_pair(sqrt_approx(ma.x), sqrt_approx(ma.y), hA[i], lA[i]);
            split_pair(sqrt_approx(mb.x), sqrt_approx(mb.y), hB[i], lB[i]);
          }
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int j = 2 * q + hh;
            mma_t(accA[hh], amg[j], hA[2 * hh], hA[2 * hh + 1]);
            mma_t(accB[hh], amg[j], hB[2 * hh], hB[2 * hh + 1]);
            mma_t(accA[hh ^ 1], amg[j], lA[2 * hh], lA[2 * hh + 1]);
            mma_t(accB[hh ^ 1], amg[j], lB[2 * hh], lB[2 * hh + 1]);
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < NQ; ++c) {
          const uint4 xA = lds128(rowA + 64u * c), xB = lds128(rowB + 64u * c);
          mma_t0(c == 0, accA[0], ari[c][0], xA.x, xA.y);
          mma_t0(c == 0, accB[0], ari[c][0], xB.x, xB.y);
          mma_t0(c == 0, accA[1], ari[c][1], xA.z, xA.w);
          mma_t0(c == 0, accB[1], ari[c][1], xB.z, xB.w);
          const uint32_t wA[4] = {xA.x, xA.y, xA.z, xA.w}, wB[4] = {xB.x, xB.y, xB.z, xB.w};
          float mA[4], mB[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            mA[i] = sqrt_approx(sq_mag_bf16_pair(wA[i]));
            mB[i] = sqrt_approx(sq_mag_bf16_pair(wB[i]));
          }
          uint32_t hA[2], lA[2], hB[2], lB[2];
          split_pair(mA[0], mA[1], hA[0], lA[0]);
          split_pair(mA[2], mA[3], hA[1], lA[1]);
          split_pair(mB[0], mB[1], hB[0], lB[0]);
          split_pair(mB[2], mB[3], hB[1], lB[1]);
          mma_t(accA[0], amg[c], hA[0], hA[1]);
          mma_t(accB[0], amg[c], hB[0], hB[1]);
          mma_t(accA[1], amg[c], lA[0], lA[1]);
          mma_t(accB[1], amg[c], lB[0], lB[1]);
        }
      }
      // d0/d1 = row rg (high part), d2/d3 = row rg + 8 (low part), columns = keys 2*rt, 2*rt + 1
      if (rg < cur_nq) {
        // this thread's keys: 2*rt, 2*rt + 1 of group A and of group B (8 keys further)
        const float sc[4] = {(accA[0][0] + accA[1][0]) + (accA[0][2] + accA[1][2]),
                             (accA[0][1] + accA[1][1]) + (accA[0][3] + accA[1][3]),
                             (accB[0][0] + accB[1][0]) + (accB[0][2] + accB[1][2]),
                             (accB[0][1] + accB[1][1]) + (accB[0][3] + accB[1][3])};
        float* out = raw_head + (size_t)(tok0 + 2 * rt) * gp_total;
        float t1 = 0.f, t2 = 0.f;  // this tile's share, fixed order (the same in both branches)
        if (full) {
          if (gp_total == 8) {  // the usual record of 8 query heads: constant store offsets
            out[0] = sc[0];
            out[8] = sc[1];
            out[64] = sc[2];
            out[72] = sc[3];
          } else {
            out[0] = sc[0];
            out[gp_total] = sc[1];
            out[(size_t)8 * gp_total] = sc[2];
            out[(size_t)9 * gp_total] = sc[3];
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            t1 += sc[e];
            t2 = fmaf(sc[e], sc[e], t2);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int ki = (e & 1) + 8 * (e >> 1);
            if (2 * rt + ki < valid) {
              out[(size_t)ki * gp_total] = sc[e];
              t1 += sc[e];
              t2 = fmaf(sc[e], sc[e], t2);
            }
          }
        }
        s1[0] += (double)t1;
        s2[0] += (double)t2;
      }
    } else {
      constexpr int NCH = NT == 1 ? 2 : 1;  // accumulator chains per column tile (two independent chains in total)
      float acc[NT][NCH][4];
      auto mma_k0 = [&](bool first, float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                        uint32_t b1) {
        if (first) mma_bf16_16816_first(d, a0, a1, a2, a3, b0, b1);
        else mma_bf16_16816(d, a0, a1, a2, a3, b0, b1);
      };

      // (hi, lo) bf16x2 pairs of two adjacent |k| values; lo is the bf16 of the exact remainder
      auto split_pair = [&](float m0, float m1, uint32_t& hi, uint32_t& lo) { split_bf16x2_hi_lo(m0, m1, hi, lo); };

      if constexpr (!INTERLEAVED) {
#pragma unroll
        for (int q = 0; q < NQ / 2; ++q) {
          constexpr int QI = NQ / 2;
          const uint4 reA = lds128(rowA + 64u * q), reB = lds128(rowB + 64u * q);
          const uint4 imA = lds128(rowA + 64u * q + D), imB = lds128(rowB + 64u * q + D);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            mma_k0(q == 0, acc[nt][0], reA.x, reB.x, reA.y, reB.y, bri[nt][q][0][0], bri[nt][q][0][1]);
            mma_k0(q == 0 && NCH == 2, acc[nt][NCH - 1], reA.z, reB.z, reA.w, reB.w, bri[nt][q][1][0], bri[nt][q][1][1]);
            mma_bf16_16816(acc[nt][0], imA.x, imB.x, imA.y, imB.y, bri[nt][q + QI][0][0], bri[nt][q + QI][0][1]);
            mma_bf16_16816(acc[nt][NCH - 1], imA.z, imB.z, imA.w, imB.w, bri[nt][q + QI][1][0], bri[nt][q + QI][1][1]);
          }
          const uint32_t rA[4] = {reA.x, reA.y, reA.z, reA.w}, rB[4] = {reB.x, reB.y, reB.z, reB.w};
          const uint32_t iA[4] = {imA.x, imA.y, imA.z, imA.w}, iB[4] = {imB.x, imB.y, imB.z, imB.w};
          uint32_t hA[4], lA[4], hB[4], lB[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 ma = sq_mag_bf16x2(rA[i], iA[i]);
            const float2 mb = sq_mag_bf16x2(rB[i], iB[i]);
            split_pair(sqrt_approx(ma.x), sqrt_approx(ma.y), hA[i], lA[i]);
            split_pair(sqrt_approx(mb.x), sqrt_approx(mb.y), hB[i], lB[i]);
          }
#pragma unroll
          for (int hh = 0; hh < 2; ++hh)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const int j = 2 * q + hh;
              mma_bf16_16816(acc[nt][hh % NCH], hA[2 * hh], hB[2 * hh], hA[2 * hh + 1], hB[2 * hh + 1], bmg[nt][j][0],
                             bmg[nt][j][1]);
              mma_bf16_16816(acc[nt][(hh ^ 1) % NCH], lA[2 * hh], lB[2 * hh], lA[2 * hh + 1], lB[2 * hh + 1], bmg[nt][j][0],
                             bmg[nt][j][1]);
            }
        }
      } else {
#pragma unroll
        for (int c = 0; c < NQ; ++c) {
          const uint4 xA = lds128(rowA + 64u * c), xB = lds128(rowB + 64u * c);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            mma_k0(c == 0, acc[nt][0], xA.x, xB.x, xA.y, xB.y, bri[nt][c][0][0], bri[nt][c][0][1]);
            mma_k0(c == 0 && NCH == 2, acc[nt][NCH - 1], xA.z, xB.z, xA.w, xB.w, bri[nt][c][1][0], bri[nt][c][1][1]);
          }
          const uint32_t wA[4] = {xA.x, xA.y, xA.z, xA.w}, wB[4] = {xB.x, xB.y, xB.z, xB.w};
          float mA[4], mB[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            mA[i] = sqrt_approx(sq_mag_bf16_pair(wA[i]));
            mB[i] = sqrt_approx(sq_mag_bf16_pair(wB[i]));
          }
          uint32_t hA[2], lA[2], hB[2], lB[2];
          split_pair(mA[0], mA[1], hA[0], lA[0]);
          split_pair(mA[2], mA[3], hA[1], lA[1]);
          split_pair(mB[0], mB[1], hB[0], lB[0]);
          split_pair(mB[2], mB[3], hB[1], lB[1]);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            mma_bf16_16816(acc[nt][0], hA[0], hB[0], hA[1], hB[1], bmg[nt][c][0], bmg[nt][c][1]);
            mma_bf16_16816(acc[nt][NCH - 1], lA[0], lB[0], lA[1], lB[1], bmg[nt][c][0], bmg[nt][c][1]);
          }
        }
      }
      // columns 2*rt and 2*rt+1 of a column tile are the two weight parts of query slot 4*nt + rt
      const int gA = tok0 + rg;
      const bool okA = full || rg < valid;
      const bool okB = full || rg + 8 < valid;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float c4[4];  // the column tile's accumulator, chains summed
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if constexpr (NCH == 2) c4[e] = acc[nt][0][e] + acc[nt][1][e];
          else c4[e] = acc[nt][0][e];
        }
        const float scA = c4[0] + c4[1];
        const float scB = c4[2] + c4[3];
        if (4 * nt + rt < cur_nq) {
          float* out = raw_head + (size_t)gA * gp_total + 4 * nt;
          float t1 = 0.f, t2 = 0.f;  // this tile's share, fixed order
          if (okA) {
            out[0] = scA;
            t1 = scA;
            t2 = scA * scA;
          }
          if (okB) {
            out[(size_t)8 * gp_total] = scB;
            t1 += scB;
            t2 = fmaf(scB, scB, t2);
          }
          s1[nt] += (double)t1;
          s2[nt] += (double)t2;
        }
      }
    }
  };
  // Item tt (keys tt*16 .. tt*16 + 15 of the stage) of KV head kvh, any block geometry.
  auto compute_item = [&](uint32_t stage_addr, int tt, int kvh, int stage_tok0, int tok_end) {
    const int tkA = tt * kMmaKeys + rg, tkB = tkA + 8;
    const uint32_t rowA = stage_addr + row_offset(min(tkA, stage_tokens - 1), kvh) + 16u * rt;
    const uint32_t rowB = stage_addr + row_offset(min(tkB, stage_tokens - 1), kvh) + 16u * rt;
    compute_rows(rowA, rowB, stage_tok0 + tt * kMmaKeys, tok_end - tt * kMmaKeys);
  };

  const int slots = (n_items + kScoreConsumerWarps - 1) / kScoreConsumerWarps;
  // common case: every warp keeps one virtual head for the whole CTA
  const bool fixed = (kScoreConsumerWarps % nvh) == 0;
  const int tt_first = fixed ? wid / nvh : 0, tt_step = fixed ? kScoreConsumerWarps / nvh : 1;
  if (fixed) {
    cur_vh = wid % nvh;
    load_weights(cur_vh);
  }
  const int fixed_kvh = cur_vh >= 0 ? cur_vh / nsub : 0;
  int stage = 0;
  uint32_t parity = 0;
  if (p.block_group > 0) {
    // 16-token blocks: item = block, and everything but the stage base is fixed for the warp.
    const int G = p.block_group;           // warps (KV heads) per block
    const int j = wid / G, kvh = wid - j * G;
    const int first_blk = tile0 * p.mb + j;  // this warp's block in the CTA's first stage-tile
    const int my_n = first_blk < nblk ? min(my_tiles, (nblk - first_blk + p.mb - 1) / p.mb) : 0;
    const int refill_n = my_n - p.stages;    // iterations below this one hand their block to a later iteration
    const uint32_t blk_rel = (uint32_t)(j * p.block_bytes);
    const uint32_t row_rel = blk_rel + (uint32_t)((kvh * p.head_stride + rg * p.token_stride) * 2) + 16u * rt;
    const uint32_t rowB_delta = (uint32_t)(16 * p.token_stride);
    uint32_t stage_off = 0u;                 // stage * stage_bytes
    unsigned round = 0u;                     // it / stages
    int tok0 = first_blk * kMmaKeys;
    int bt_next = p.stages * p.mb + j;       // position (in the CTA's block list) of the block that refills this slot
    for (int it = 0; it < my_n; ++it) {
      const bool ready = __all_sync(kFull, mbar_wait_bounded(smem_u32(&blk_bar[stage][j]), parity, &s_err));
      if (!ready) {
        if (lane == 0) {
          if (s_err == 0) flag_status(p.status, TRIATTN_DEV_WAIT_TIMEOUT);
          s_err = 1;
        }
        break;
      }
      const uint32_t rowA = smem_base + stage_off + row_rel;
      compute_rows(rowA, rowA + rowB_delta, tok0, seq_len - tok0);
      // Hand the block back; the last of the block's G reader warps refills it (a single reader needs no count).
      __syncwarp();
      if (lane == 0) {
        const bool last = G == 1 ? true : release_and_check_last(smem_u32(&blk_empty_bar[stage][j]));
        if (last && it < refill_n) {
          fence_proxy_async();  // generic-proxy reads of the block before the async-proxy refill
          int blk;
          if (bt_in_smem) {
            blk = s_bt[bt_next];
          } else {
            blk = bt[tile0 * p.mb + bt_next];
            if ((unsigned)blk >= (unsigned)p.num_blocks) {
              flag_status(p.status, TRIATTN_DEV_BAD_BLOCK_ID);
              blk = 0;
            }
          }
          const uint32_t bar = smem_u32(&blk_bar[stage][j]);
          mbar_arrive_expect_tx(bar, (uint32_t)p.block_bytes + kTestExtraTxBytes);
          s_blk_issued[stage][j] = round + 2u;  // armed once before the loop and once per earlier round
          bulk_copy_g2s(smem_base + stage_off + blk_rel, kbase + (long long)blk * p.block_stride_bytes,
                        (uint32_t)p.block_bytes, bar);
        }
      }
      tok0 += stage_tokens;
      bt_next += p.mb;
      stage_off += (uint32_t)stage_bytes;
      if (++stage == p.stages) {
        stage = 0;
        stage_off = 0u;
        parity ^= 1u;
        ++round;
      }
    }
  } else {
    for (int it = 0; it < my_tiles; ++it) {
      const bool ready = __all_sync(kFull, mbar_wait_bounded(smem_u32(&full_bar[stage]), parity, &s_err));
      if (!ready) {
        if (lane == 0) {
          if (s_err == 0) flag_status(p.status, TRIATTN_DEV_WAIT_TIMEOUT);
          s_err = 1;
        }
        break;
      }
      const uint32_t stage_addr = smem_base + (uint32_t)(stage * stage_bytes);
      const int stage_tok0 = (tile0 + it) * stage_tokens;
      const int tok_end = min(seq_len - stage_tok0, stage_tokens);  // keys of this stage that exist
      if (fixed) {
        for (int tt = tt_first; tt * kMmaKeys < tok_end; tt += tt_step)
          compute_item(stage_addr, tt, fixed_kvh, stage_tok0, tok_end);
      } else {
        for (int sl = 0; sl < slots; ++sl) {
          const int item = wid + sl * kScoreConsumerWarps;  // warp-uniform
          if (item >= n_items) break;
          const int vh = item % nvh, tt = item / nvh;
          if (tt * kMmaKeys >= tok_end) break;  // items are ordered by token
          if (vh != cur_vh) {
            flush_moments();
            load_weights(vh);
            cur_vh = vh;
          }
          compute_item(stage_addr, tt, vh / nsub, stage_tok0, tok_end);
        }
      }
      // release the stage; the warp whose release is the last of the 8 refills it with the tile `stages` ahead
      __syncwarp();
      unsigned refill = 0u;
      if (lane == 0 && release_and_check_last(smem_u32(&empty_bar[stage])) && it + p.stages < my_tiles) refill = 1u;
      if (__shfl_sync(kFull, refill, 0)) {
        fence_proxy_async();  // every lane issues copies: each orders the (acquired) generic reads before its own
        issue(it + p.stages, stage, lane);
      }
      if (++stage == p.stages) {
        stage = 0;
        parity ^= 1u;
      }
    }
  }
  flush_moments();
  // No thread leaves while a copy may still be on its way into this CTA's shared memory: after a timeout
  // (and only then) the first warp waits once more, bounded, for every copy that was armed.
  __syncthreads();
  if (s_err != 0 && tid < 32) {
    if (p.block_group > 0) {
      for (int i = tid; i < p.stages * kScoreConsumerWarps; i += 32) {
        const int s = i / kScoreConsumerWarps, w = i - s * kScoreConsumerWarps;
        const unsigned n = s_blk_issued[s][w];
        if (n > 0u) mbar_wait_bounded(smem_u32(&blk_bar[s][w]), (n - 1u) & 1u);
      }
    } else if (tid < p.stages) {
      const unsigned n = s_issued[tid];
      if (n > 0u) mbar_wait_bounded(smem_u32(&full_bar[tid]), (n - 1u) & 1u);
    }
  }
}

}  // namespace triattn
