// Key scorer for offset aggregation = max on the warp-level tensor-core path.
//
// score(key, head) = max over the O offsets of sum_d k_d * W[o][head][d]  +  sum_f |k_f| * w_mag[head][f]
// is O dot products of length D per (key, head): [16 keys x D] x [D x (O x 4 heads x 2 parts)] on m16n8k16 bf16
// MMAs, one column tile per offset (column n = 2*head + part, bf16 high part and bf16 of the remainder of the
// fp32 weight, as in score_mma.cuh), so a thread sees the finished dot product of query head lane%4 for its two
// keys after every offset and keeps a running maximum in registers.  The magnitude term is the one of
// score_mma.cuh (|k| in fp32 on the CUDA cores, split into two bf16 parts).
//
// The work is bound by the tensor pipe (8*O + 8 MMAs per 16 keys), not by HBM, so the data movement is chosen for
// simplicity: a CTA works on ONE (layer, request, virtual head); its weight fragments for all offsets live in
// shared memory in fragment order (conflict-free 16-byte loads), and every warp streams its own 16-key tiles of
// that head, two at a time (one load of an offset's weight fragments feeds both), through private 16-row slots
// fetched row by row with 1-D bulk async copies on the warp's own mbarriers (bounded waits).  Rows are padded by
// 16 bytes, so ldmatrix.x4 delivers the key fragments conflict-free and already in MMA register order; the tiles
// move to registers, the slots are refilled at once and the copies land during the 17 offsets.  No warp waits for
// another.
#pragma once

#include "score_mma.cuh"

namespace triattn {

constexpr int kMaxAggWarps = 12;
constexpr int kMaxAggThreads = kMaxAggWarps * 32;
constexpr int kMaxAggOffsets = 1;  // offsets a warp works on at once
constexpr int kMaxAggTiles = 2;   // 16-key tiles a warp works on at once (independent accumulator chains)
constexpr int kMaxAggSlots = kMaxAggTiles;  // ring slots per warp: the tiles move to registers, then the slots refill

// dynamic shared memory: weight fragments [O][KS/2][32 lanes][4 words] + rings [warps][slots][16 rows][D*2 bytes]
// (rows are padded by 16 bytes so that the 8 row addresses of an ldmatrix phase fall into 8 different bank groups)
inline size_t max_agg_smem_bytes(int D, int num_offsets) {
  return (size_t)num_offsets * (D / 32) * 32 * 16 + (size_t)kMaxAggWarps * kMaxAggSlots * kMmaKeys * (D * 2 + 16);
}

// four 8x8 b16 matrices -> the A fragment (a0..a3) of one m16n8k16 MMA, straight in fragment order
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&a)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
               : "r"(addr));
}

template <int D, bool INTERLEAVED>
__global__ void __launch_bounds__(kMaxAggThreads, 1) score_paged_mma_max_kernel(const __grid_constant__ ScoreParams p) {
  constexpr int F = D / 2;
  constexpr int KS = D / 16;   // k-steps (MMAs) per offset
  constexpr int GP = 4;
  constexpr int ROW_BYTES = D * 2;
  constexpr int ROW_STRIDE = ROW_BYTES + 16;  // padded row pitch inside a slot
  constexpr int SLOT_BYTES = kMmaKeys * ROW_STRIDE;
  constexpr int NMG = KS / 2;                 // magnitude MMAs per part (16 frequencies each)

  extern __shared__ __align__(128) unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t bars[kMaxAggWarps][kMaxAggSlots];

  const int O = p.num_offsets;
  uint4* s_w = reinterpret_cast<uint4*>(smem_dyn);  // [O][KS/2][32]
  unsigned char* s_ring = smem_dyn + (size_t)O * (KS / 2) * 32 * 16;

  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int l = blockIdx.y, b = blockIdx.z;
  grid_dependency_wait();  // no global access before the preceding kernel of the stream has completed
  trigger_dependents();
  const int nsub = (p.gp_total + GP - 1) / GP;
  const int nvh = p.Hkv * nsub;
  const int vh = blockIdx.x % nvh, chunk = blockIdx.x / nvh;
  const int kvh = vh / nsub, sub = vh - kvh * nsub;
  int seq_len = p.seq_lens[b];
  if (seq_len > p.t_pad) {
    if (tid == 0 && blockIdx.x == 0) flag_status(p.status, TRIATTN_DEV_BAD_LENGTH);
    seq_len = p.t_pad;
  }
  const int n_tiles = (seq_len + kMmaKeys - 1) / kMmaKeys;  // 16-key tiles of the request
  const int tile0 = chunk * p.tiles_per_cta;
  if (tile0 >= n_tiles) return;
  const int my_tiles = min(p.tiles_per_cta, n_tiles - tile0);
  const int Hq = p.Hkv * p.g;
  const int rows_w = 2 * O + 1;  // weight rows per query head: re[o]..., im[o]..., magnitude
  const int qbase = kvh * p.g + sub * GP;
  const int nq = min(GP, p.g - sub * GP);
  const int rg = lane >> 2, rt = lane & 3;

  if (tid < kMaxAggWarps * kMaxAggSlots) mbar_init(smem_u32(&bars[tid / kMaxAggSlots][tid % kMaxAggSlots]), 1);
  if (tid == 0) mbar_fence_init();

  // weight fragments of all offsets -> shared memory, fragment order: entry (o, ks, lane') = (b0, b1) of k-step ks
  for (int e = tid; e < O * KS * 32; e += kMaxAggThreads) {
    const int ln = e & 31, ks = (e >> 5) % KS, o = e / (32 * KS);
    const int crg = ln >> 2, crt = ln & 3;
    const int head = crg >> 1, part = crg & 1;
    const bool on = head < nq;
    const float* w = p.weights + (((size_t)l * p.B + b) * Hq + (size_t)qbase + (on ? head : 0)) * rows_w * F;
    uint32_t v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int d = 16 * ks + 8 * (i >> 1) + 2 * crt + (i & 1);  // b0: k = 2t, 2t+1; b1: k = 2t+8, 2t+9
      const int comp = INTERLEAVED ? (d & 1) : (d >= F ? 1 : 0);
      const int f = INTERLEAVED ? (d >> 1) : (d >= F ? d - F : d);
      const float x = on ? __ldg(w + (size_t)(comp * O + o) * F + f) : 0.f;
      uint32_t hi, lo;
      bf16_split(x, hi, lo);
      v[i] = part ? lo : hi;
    }
    uint32_t* dst = reinterpret_cast<uint32_t*>(s_w + ((size_t)o * (KS / 2) + (ks >> 1)) * 32 + ln) + 2 * (ks & 1);
    dst[0] = v[0] | (v[1] << 16);
    dst[1] = v[2] | (v[3] << 16);
  }
  // magnitude fragments stay in registers
  uint32_t bmg[NMG][2];
  {
    const int head = rg >> 1, part = rg & 1;
    const bool on = head < nq;
    const float* wm = p.weights + ((((size_t)l * p.B + b) * Hq + (size_t)qbase + (on ? head : 0)) * rows_w + 2 * O) * F;
#pragma unroll
    for (int j = 0; j < NMG; ++j) {
      uint32_t v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // the 4 frequencies this thread feeds into magnitude MMA j, in the order load_tile packs |k|
        const int f = INTERLEAVED ? 16 * j + 4 * i + rt : 16 * j + 8 * (i >> 1) + 2 * rt + (i & 1);
        uint32_t hi, lo;
        bf16_split(on ? __ldg(wm + f) : 0.f, hi, lo);
        v[i] = part ? lo : hi;
      }
      bmg[j][0] = v[0] | (v[1] << 16);
      bmg[j][1] = v[2] | (v[3] << 16);
    }
  }
  __syncthreads();

  const unsigned char* kbase = reinterpret_cast<const unsigned char*>(p.k_ptrs[l]);
  const int32_t* bt = p.block_table + (size_t)b * p.max_blocks;
  unsigned char* my_ring = s_ring + (size_t)wid * kMaxAggSlots * SLOT_BYTES;
  constexpr unsigned kFull = 0xffffffffu;

  unsigned armed[kMaxAggTiles];  // copies armed so far on each of this warp's barriers (warp-uniform)
#pragma unroll
  for (int t = 0; t < kMaxAggTiles; ++t) armed[t] = 0u;
  // fetch the 16 rows of this warp's tile `i` (tile index within the CTA's range): lane r copies row r
  auto fetch = [&](int i, int slot) {
    armed[slot] += 1u;
    const int tok0 = (tile0 + i) * kMmaKeys;
    const int rows = min(kMmaKeys, seq_len - tok0);
    const uint32_t bar = smem_u32(&bars[wid][slot]);
    if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)(rows * ROW_BYTES) + kTestExtraTxBytes);
    __syncwarp();
    if (lane < rows) {
      const int t = tok0 + lane;
      const int bi = t / p.bs;
      int blk = bt[bi];
      if ((unsigned)blk >= (unsigned)p.num_blocks) {
        flag_status(p.status, TRIATTN_DEV_BAD_BLOCK_ID);
        blk = 0;
      }
      const unsigned char* src = kbase + (long long)blk * p.block_stride_bytes +
                                 ((long long)(t - bi * p.bs) * p.token_stride + (long long)kvh * p.head_stride) * 2;
      bulk_copy_g2s(smem_u32(my_ring + (size_t)slot * SLOT_BYTES + (size_t)lane * ROW_STRIDE), src, ROW_BYTES, bar);
    }
  };

  // this warp's tiles: wid, wid + W, ... of the CTA's range, taken kMaxAggTiles at a time: the weight fragments
  // of an offset are loaded from shared memory once and used for all of them
  const int n_mine = my_tiles > wid ? (my_tiles - wid + kMaxAggWarps - 1) / kMaxAggWarps : 0;
#pragma unroll
  for (int i = 0; i < kMaxAggTiles; ++i)
    if (i < n_mine) fetch(wid + i * kMaxAggWarps, i);

  auto split_pair = [&](float m0, float m1, uint32_t& hi, uint32_t& lo) { split_bf16x2_hi_lo(m0, m1, hi, lo); };
  // A fragments of one tile (kept for all offsets) and its magnitude term for this thread's two keys
  auto load_tile = [&](uint32_t base, uint32_t (&a)[KS][4], float& magA, float& magB) {
    // lane -> (row, 8-column block) of the 8x8 matrix it addresses: matrices 0..3 = (rows 0-7 | 8-15) x (k 0-7 | 8-15)
    const uint32_t lm = base + (uint32_t)(((lane & 7) + 8 * ((lane >> 3) & 1)) * ROW_STRIDE) + 16u * (lane >> 4);
    float accm[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) ldmatrix_x4(a[ks], lm + 32u * ks);
    // a[ks] = {(key rg, dims 16ks+2rt,+1), (key rg+8, same), (key rg, dims 16ks+8+2rt,+1), (key rg+8, same)}
    if constexpr (!INTERLEAVED) {
#pragma unroll
      for (int j = 0; j < NMG; ++j) {
        // k-step j holds re of 16 frequencies, k-step j + NMG their im: |k| comes out in fragment order
        uint32_t h[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 m = sq_mag_bf16x2(a[j][e], a[j + NMG][e]);
          split_pair(sqrt_approx(m.x), sqrt_approx(m.y), h[e], lo[e]);
        }
        mma_bf16_16816(accm[0], h[0], h[1], h[2], h[3], bmg[j][0], bmg[j][1]);
        mma_bf16_16816(accm[1], lo[0], lo[1], lo[2], lo[3], bmg[j][0], bmg[j][1]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < NMG; ++j) {
        // a word is (re, im) of one frequency: k-steps 2j, 2j+1 give this thread 4 frequencies per key
        float m[2][4];  // [k-step of the pair][fragment element]
#pragma unroll
        for (int s2 = 0; s2 < 2; ++s2)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            m[s2][e] = sqrt_approx(sq_mag_bf16_pair(a[2 * j + s2][e]));
          }
        uint32_t h[4], lo[4];
        split_pair(m[0][0], m[0][2], h[0], lo[0]);  // key rg:   frequencies 16j + rt, 16j + 4 + rt
        split_pair(m[0][1], m[0][3], h[1], lo[1]);  // key rg+8
        split_pair(m[1][0], m[1][2], h[2], lo[2]);  // key rg:   frequencies 16j + 8 + rt, 16j + 12 + rt
        split_pair(m[1][1], m[1][3], h[3], lo[3]);  // key rg+8
        mma_bf16_16816(accm[0], h[0], h[1], h[2], h[3], bmg[j][0], bmg[j][1]);
        mma_bf16_16816(accm[1], lo[0], lo[1], lo[2], lo[3], bmg[j][0], bmg[j][1]);
      }
    }
    magA = (accm[0][0] + accm[1][0]) + (accm[0][1] + accm[1][1]);
    magB = (accm[0][2] + accm[1][2]) + (accm[0][3] + accm[1][3]);
  };

  float s1 = 0.f, s2 = 0.f;
  float* raw_head = p.raw + (((size_t)l * p.B + b) * p.Hkv + kvh) * (size_t)p.t_pad * p.gp_total + sub * GP + rt;
  uint32_t parity = 0;
  bool failed = false;
  for (int i = 0; i < n_mine && !failed; i += kMaxAggTiles) {
    uint32_t a[kMaxAggTiles][KS][4];
    float mag[kMaxAggTiles][2];
    bool have[kMaxAggTiles];
#pragma unroll
    for (int t = 0; t < kMaxAggTiles; ++t) {
      have[t] = i + t < n_mine;  // warp-uniform
      mag[t][0] = mag[t][1] = 0.f;
      if (have[t]) {
        const bool ready = __all_sync(kFull, mbar_wait_bounded(smem_u32(&bars[wid][t]), parity));
        if (!ready) {
          if (lane == 0) flag_status(p.status, TRIATTN_DEV_WAIT_TIMEOUT);
          failed = true;
          have[t] = false;
        }
      }
      if (have[t]) {
        load_tile(smem_u32(my_ring + (size_t)t * SLOT_BYTES), a[t], mag[t][0], mag[t][1]);
      } else {
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
          for (int e = 0; e < 4; ++e) a[t][ks][e] = 0u;
      }
    }
    if (failed) break;
    // every shared-memory value of the slots is in registers: refill them with the next tiles of this warp
    __syncwarp();
    if (i + kMaxAggTiles < n_mine) {
      fence_proxy_async();  // every lane copies a row: each orders the warp's (synchronised) reads before its own copy
#pragma unroll
      for (int t = 0; t < kMaxAggTiles; ++t)
        if (i + kMaxAggTiles + t < n_mine) fetch(wid + (i + kMaxAggTiles + t) * kMaxAggWarps, t);
    }
    parity ^= 1u;

    // offsets: one column tile each; the weight fragments of an offset feed all tiles
    float best[kMaxAggTiles][2];
#pragma unroll
    for (int t = 0; t < kMaxAggTiles; ++t) best[t][0] = best[t][1] = -INFINITY;
    // kMaxAggOffsets offsets at a time: with the tiles that gives tiles x offsets independent accumulator chains
    for (int o = 0; o < O; o += kMaxAggOffsets) {
      float c[kMaxAggOffsets][kMaxAggTiles][4];
      const uint4* w[kMaxAggOffsets];
#pragma unroll
      for (int n = 0; n < kMaxAggOffsets; ++n) {
        w[n] = s_w + (size_t)min(o + n, O - 1) * (KS / 2) * 32 + lane;  // past the end: the last offset again (max unchanged)
#pragma unroll
        for (int t = 0; t < kMaxAggTiles; ++t)
#pragma unroll
          for (int e = 0; e < 4; ++e) c[n][t][e] = 0.f;
      }
#pragma unroll
      for (int r = 0; r < KS / 2; ++r) {
        uint4 u[kMaxAggOffsets];
#pragma unroll
        for (int n = 0; n < kMaxAggOffsets; ++n) u[n] = w[n][r * 32];
#pragma unroll
        for (int n = 0; n < kMaxAggOffsets; ++n)
#pragma unroll
          for (int t = 0; t < kMaxAggTiles; ++t)
            mma_bf16_16816(c[n][t], a[t][2 * r][0], a[t][2 * r][1], a[t][2 * r][2], a[t][2 * r][3], u[n].x, u[n].y);
#pragma unroll
        for (int n = 0; n < kMaxAggOffsets; ++n)
#pragma unroll
          for (int t = 0; t < kMaxAggTiles; ++t)
            mma_bf16_16816(c[n][t], a[t][2 * r + 1][0], a[t][2 * r + 1][1], a[t][2 * r + 1][2], a[t][2 * r + 1][3],
                           u[n].z, u[n].w);
      }
#pragma unroll
      for (int n = 0; n < kMaxAggOffsets; ++n)
#pragma unroll
        for (int t = 0; t < kMaxAggTiles; ++t) {
          best[t][0] = fmaxf(best[t][0], c[n][t][0] + c[n][t][1]);
          best[t][1] = fmaxf(best[t][1], c[n][t][2] + c[n][t][3]);
        }
    }
#pragma unroll
    for (int t = 0; t < kMaxAggTiles; ++t) {
      if (have[t] && rt < nq) {
        const int gA = (tile0 + wid + (i + t) * kMaxAggWarps) * kMmaKeys + rg;
        float* out = raw_head + (size_t)gA * p.gp_total;
        const float scA = best[t][0] + mag[t][0], scB = best[t][1] + mag[t][1];
        if (gA < seq_len) {
          out[0] = scA;
          s1 += scA;
          s2 = fmaf(scA, scA, s2);
        }
        if (gA + 8 < seq_len) {
          out[(size_t)8 * p.gp_total] = scB;
          s1 += scB;
          s2 = fmaf(scB, scB, s2);
        }
      }
    }
  }
  if (failed) {
    // a wait ran out: before leaving, wait once more (bounded) for every copy this warp armed, so that no copy
    // is still on its way into the CTA's shared memory when the CTA retires
#pragma unroll
    for (int t = 0; t < kMaxAggTiles; ++t)
      if (armed[t] > 0u) mbar_wait_bounded(smem_u32(&bars[wid][t]), (armed[t] - 1u) & 1u);
  }
  // moments of query slot rt over this warp's keys
#pragma unroll
  for (int s = 4; s < 32; s <<= 1) {
    s1 += __shfl_xor_sync(kFull, s1, s);
    s2 += __shfl_xor_sync(kFull, s2, s);
  }
  if (lane < 4 && lane < nq && n_mine > 0) {
    double* m = p.moments + (((size_t)l * p.B + b) * Hq + (size_t)qbase + lane) * 2;
    atomicAdd(m, (double)s1);
    atomicAdd(m + 1, (double)s2);
  }
}

}  // namespace triattn
