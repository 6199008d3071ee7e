// Key scorer for offset aggregation = max on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory), head_dim 128.
//
// With max aggregation every (query head, offset) pair is its own dot product against the key, so a tile of
// 128 keys times the O offsets of 4 query heads is a [128 x 128] x [128 x 4*O] matrix product.  The fp32 weights
// are carried as a bf16 high part and the bf16 of the remainder, side by side as columns of one operand
// (D = K x [W_hi | W_lo]), so the accumulator of a tile is [128 keys x 2 x 4*O] fp32 (2 x 68 columns for 17
// offsets, each part padded to 80), a tile costs eight tcgen05.mma of shape M = 128, N = 160, K = 16 - the keys
// are read from shared memory once per K step - and the epilogue adds the two parts.
//
// A CTA (one per SM, 18 warps) works on a run of 128-key tiles of one (layer, request, virtual head of <= 4
// query heads); the weights go to shared memory once, in the K-major 128-byte-swizzled operand layout (40 KB).
//   * One producer warp streams the keys with tiled TMA loads (cp.async.bulk.tensor, no multicast): the layer's
//     K cache is described by a rank-5 tensor map (64 dims, token mod 8, half of the head vector, token / 8 in
//     the block, head slot) with the 128-byte swizzle, so ONE box brings the 16 tokens of a head that a cache
//     block holds - 4 KB - and lands in the ring as complete 8-row operand atoms: [8-key group][real | imaginary]
//     [8 rows x 128 B].  8 loads per tile into a 5-stage ring, completing on an mbarrier.  The producer starts
//     streaming right after the mbarriers are set up, while the other warps still build the weight operand.
//     The engine hands the per-layer base pointers over in DEVICE memory, so the host encodes one template map
//     for the geometry and a one-warp kernel stamps each layer's address into a copy of it (tensormap.replace)
//     before the scorer starts.
//   * The MMA warp issues the 8 MMAs of a tile (through one elected lane) into one of two TMEM accumulators and
//     commits to two mbarriers (accumulator complete; stage no longer read by the tensor core).
//   * 8 magnitude warps (two per tile, four tiles in flight) form sum_f |k_f| * w_mag in fp32 straight from
//     the shared-memory tile - no bf16 split of |k| - with 2 keys per thread, so that one load of a frequency's
//     weights serves 2 keys; the work is latency-bound, hence the many warps.
//   * 8 epilogue warps in two groups (even / odd tiles).  A thread owns one key (= one TMEM lane): it reads its
//     accumulator row with tcgen05.ld, adds the two weight parts, takes the max over the offsets of each head,
//     adds the magnitude term and stores the 4 scores of its key as one 16-byte store.
// Every wait is bounded; a wait that runs out sets TRIATTN_DEV_WAIT_TIMEOUT, all roles leave their loops, the
// producer drains its copies, and the tensor memory is freed before the CTA exits.
// What limits it (measured with per-role cycle counters and with builds in which one consumer at a time does
// nothing): with every consumer idle the ring alone streams the keys at 0.91 of the measured HBM bandwidth; the
// whole kernel reaches 0.64, and leaving out the MMAs, the magnitude pass or the epilogue's TMEM reads lifts that
// to 0.76, 0.75 and 0.68.  The gains rank like the shared-memory bytes each of them moves per 128-key tile
// (operand reads of the tensor core 72 KB, magnitude pass 48 KB, epilogue 4 KB, on top of the 32 KB the TMA
// writes): the shared-memory pipe, 128 bytes per cycle, is what the roles compete for.  Halving the MMAs per tile
// (which removed 32 KB of operand re-reads), halving the loads per tile, a second producer warp, releasing stages
// earlier and an L2 prefetch ahead of the loads did not change the rate by themselves.
#pragma once

#include "score_mma.cuh"

namespace triattn {

constexpr int kUmmaEpiWarps = 8;     // two groups of 4: warp w may only touch TMEM lanes 32*(w % 4) .. +31
constexpr int kUmmaMagWarps = 8;     // two per tile (64 keys each), four tiles in flight
constexpr int kUmmaProdWarps = 1;
constexpr int kUmmaMmaWarp = kUmmaEpiWarps + kUmmaMagWarps;  // warp order: epilogue, magnitude, MMA, producers
constexpr int kUmmaWarps = kUmmaMmaWarp + 1 + kUmmaProdWarps;
constexpr int kUmmaThreads = kUmmaWarps * 32;
constexpr int kUmmaSetupThreads = (kUmmaMmaWarp + 1) * 32;  // every warp but the producers prepares the weights
constexpr int kUmmaTileKeys = 128;
constexpr int kUmmaStages = 5;      // 160 KB of keys in flight or in use per SM
constexpr int kUmmaStageBytes = kUmmaTileKeys * 256;  // 32 KB: 16 groups of 8 keys, each [real | imaginary][8 rows x 128 B]
constexpr int kUmmaGroupBytes = 2048;                 // one 8-key group: the 1 KB atom of the real parts, then the imaginary parts
constexpr int kUmmaHalfBytes = 1024;
constexpr int kUmmaMaxN = 256;
constexpr int kUmmaAccStride = 256;  // TMEM columns between the two accumulators
constexpr int kUmmaTmemCols = 512;
constexpr int kUmmaMaxBlocks = 1152; // block ids of a CTA's keys kept in shared memory

// accumulator columns: 4 heads x O offsets, padded to a multiple of 16
inline int umma_max_cols(int num_offsets) { return (4 * num_offsets + 15) / 16 * 16; }
inline size_t umma_max_smem_bytes(int n_cols) {
  return 1024 /* alignment slack */ + (size_t)kUmmaStages * kUmmaStageBytes + 2 * (size_t)n_cols * 256 +
         64 * sizeof(float4) + (size_t)kUmmaStages * kUmmaTileKeys * sizeof(float4) +
         (size_t)kUmmaMaxBlocks * sizeof(int);
}

// ---- tcgen05 / cp.async wrappers
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(addr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// One lane of a fully converged warp.  The warp runs the surrounding loop as a whole (barrier waits, descriptor and
// coordinate arithmetic stay warp-uniform) and only the asynchronous instruction itself is issued by the elected lane.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0u;
}
// tiled TMA load of one box (coordinates innermost first) into this CTA's shared memory; no multicast
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}

// One tensor map per layer: a copy of the host-encoded template with that layer's K base pointer stamped in.
// The stamped maps live in global memory; a kernel that loads through them acquires them with
// fence.proxy.tensormap before its first load.
struct TensorMapBytes {
  alignas(64) unsigned long long q[16];
};
__global__ void stamp_tensor_maps_kernel(const __grid_constant__ TensorMapBytes tmpl, const void* const* k_ptrs,
                                         unsigned char* slots, int num_layers) {
  grid_dependency_wait();  // no global access before the preceding kernel of the stream has completed
  trigger_dependents();
  const int l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= num_layers) return;
  unsigned long long* dst = reinterpret_cast<unsigned long long*>(slots + (size_t)l * 128);
#pragma unroll
  for (int i = 0; i < 16; ++i) dst[i] = tmpl.q[i];
  const unsigned long long addr = reinterpret_cast<unsigned long long>(k_ptrs[l]);
  asm volatile("tensormap.replace.tile.global_address.global.b1024.b64 [%0], %1;" ::"l"(dst), "l"(addr) : "memory");
  asm volatile("fence.proxy.tensormap::generic.release.gpu;" ::: "memory");
}

// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups `sbo_bytes` apart
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t sbo_bytes) {
  uint64_t d = (uint64_t)((smem_addr & 0x3ffffu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                                 // leading byte offset (unused with swizzled K-major): 1
  d |= (uint64_t)(sbo_bytes >> 4) << 32;                  // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                                 // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                                 // SWIZZLE_128B
  return d;
}
// byte offset of 16-byte chunk `c` (0..7) of row `r` inside a [rows x 128 B] swizzled K block
__device__ __forceinline__ uint32_t swz128(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }
// the same for key row `r` (0..127) of a stage, half `h` (0 real, 1 imaginary parts)
__device__ __forceinline__ uint32_t key_chunk(int r, int h, int c) {
  return (uint32_t)((r >> 3) * kUmmaGroupBytes + h * kUmmaHalfBytes + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}

template <bool INTERLEAVED>
__global__ void __launch_bounds__(kUmmaThreads, 1) score_paged_umma_max_kernel(const __grid_constant__ ScoreParams p) {
  constexpr int F = 64, GP = 4;
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kUmmaStages], empty_bar[kUmmaStages], mag_bar[kUmmaStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_err;
  // Tile each stage was last armed for.  A barrier wait names its phase by one parity bit, so it is only exact for a
  // waiter that is at most one phase away.  The MMA warp, the producer and the epilogue groups visit a stage's
  // barriers in step with its reuse; the magnitude warps do not: a pair takes every fourth tile, and the copies of
  // two tiles may land out of order, so a pair can finish tile i - 4 and ask for tile i while tile i - 5 - the
  // previous user of the same stage - has not even landed.  Its parity wait would then pass at once (the barrier
  // is still in the phase BEFORE the one it wants) and it would read and release a stage that is not its own.
  // It therefore first waits until the producer has armed the stage for its tile.
  __shared__ int s_armed[kUmmaStages];

  grid_dependency_wait();  // no global access before the preceding kernel of the stream has completed
  trigger_dependents();
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int l = blockIdx.y, b = blockIdx.z;
  const int O = p.num_offsets;
  const int n_cols = (4 * O + 15) / 16 * 16;
  const int nsub = (p.gp_total + GP - 1) / GP;
  const int nvh = p.Hkv * nsub;
  const int vh = blockIdx.x % nvh, chunk = blockIdx.x / nvh;
  const int kvh = vh / nsub, sub = vh - kvh * nsub;
  int seq_len = p.seq_lens[b];
  if (seq_len > p.t_pad) {
    if (tid == 0 && blockIdx.x == 0) flag_status(p.status, TRIATTN_DEV_BAD_LENGTH);
    seq_len = p.t_pad;
  }
  const int n_tiles_req = (seq_len + kUmmaTileKeys - 1) / kUmmaTileKeys;
  const int tile0 = chunk * p.tiles_per_cta;
  if (tile0 >= n_tiles_req) return;  // CTA-uniform: nothing allocated yet
  const int my_tiles = min(p.tiles_per_cta, n_tiles_req - tile0);
  const int Hq = p.Hkv * p.g;
  const int qbase = kvh * p.g + sub * GP;
  const int nq = min(GP, p.g - sub * GP);
  const int rows_w = 2 * O + 1;

  // carve the dynamic shared memory (operands 1024-byte aligned: the swizzle pattern repeats every 1024 bytes)
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_base = base;                                    // [stages][2 K blocks][128 rows][128 B]
  const uint32_t b_base = a_base + kUmmaStages * kUmmaStageBytes;  // [2 parts][2 K blocks][n_cols rows][128 B]
  unsigned char* gen = smem_raw + (base - smem_u32(smem_raw)) + kUmmaStages * kUmmaStageBytes + 2 * (size_t)n_cols * 256;
  float4* s_wmag = reinterpret_cast<float4*>(gen);                 // [64 f]: magnitude weights of the 4 heads
  float4* s_mag = s_wmag + 64;                                     // [stages][128 keys]: magnitude terms of a tile
  int* s_bt = reinterpret_cast<int*>(s_mag + kUmmaStages * kUmmaTileKeys);

  if (tid == 0) {
    for (int s = 0; s < kUmmaStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);  // the producer's arrive with the byte count of the tile
      mbar_init(smem_u32(&empty_bar[s]), 2 + 1 + 4);  // 2 magnitude warps, tensor-core commit, 4 epilogue warps
      mbar_init(smem_u32(&mag_bar[s]), 2);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), 4);
    }
    mbar_fence_init();
    s_err = 0;
    for (int st = 0; st < kUmmaStages; ++st) s_armed[st] = st;  // the first round needs no check
  }
  if (wid == 0) {  // one warp allocates the accumulator columns and gives up the permit
    tmem_alloc(smem_u32(&s_tmem), kUmmaTmemCols);
    tmem_relinquish();
  }
  // block ids of this CTA's keys
  const int tok0 = tile0 * kUmmaTileKeys;
  const int tok1 = min(seq_len, tok0 + my_tiles * kUmmaTileKeys);
  const int bi0 = tok0 / p.bs, bi1 = (tok1 + p.bs - 1) / p.bs;
  const int32_t* bt = p.block_table + (size_t)b * p.max_blocks;
  for (int i = tid; i < bi1 - bi0; i += kUmmaThreads) {
    int blk = bt[bi0 + i];
    if ((unsigned)blk >= (unsigned)p.num_blocks) {
      flag_status(p.status, TRIATTN_DEV_BAD_BLOCK_ID);
      blk = 0;
    }
    s_bt[i] = blk;
  }
  // First barrier: mbarriers, TMEM address and block ids are in place.  The producers start streaming keys right
  // away; the other warps build the weight operands meanwhile and meet at a barrier of their own.
  __syncthreads();
  const uint32_t tmem_base = s_tmem;
  const volatile int* err = &s_err;
  auto fail = [&]() {
    if (*err == 0) flag_status(p.status, TRIATTN_DEV_WAIT_TIMEOUT);
    s_err = 1;
  };
  if (wid <= kUmmaMmaWarp) {
  // B operand: rows 0 .. n_cols-1 = high bf16 parts, rows n_cols .. 2*n_cols-1 = remainders, so that one MMA of
  // N = 2 * n_cols covers both and the keys (the A operand) are read once per K step; row n = o * 4 + q inside a part
  // (offset-major, so the head of a column is a compile-time constant in the epilogue), column k = key dimension;
  // 16-byte chunks of 8 dimensions
  for (int e = tid; e < 2 * n_cols * 16; e += kUmmaSetupThreads) {
    const int part = e / (n_cols * 16), r = e - part * n_cols * 16;
    const int n = r >> 4, c16 = r & 15;  // chunk c16 covers key dims 8*c16 .. 8*c16+7
    const int o = n >> 2, q = n & 3;
    const bool on = o < O && q < nq;
    const float* w = p.weights + (((size_t)l * p.B + b) * Hq + (size_t)qbase + (on ? q : 0)) * rows_w * F;
    uint32_t v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = 8 * c16 + i;
      const int comp = INTERLEAVED ? (d & 1) : (d >= F ? 1 : 0);
      const int f = INTERLEAVED ? (d >> 1) : (d >= F ? d - F : d);
      const float x = on ? __ldg(w + (size_t)(comp * O + min(o, O - 1)) * F + f) : 0.f;
      uint32_t hi, lo;
      bf16_split(x, hi, lo);
      v[i] = part ? lo : hi;
    }
    const uint32_t dst = b_base + (uint32_t)(c16 >> 3) * (uint32_t)(2 * n_cols * 128) + swz128(part * n_cols + n, c16 & 7);
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(v[0] | (v[1] << 16)), "r"(v[2] | (v[3] << 16)),
                 "r"(v[4] | (v[5] << 16)), "r"(v[6] | (v[7] << 16))
                 : "memory");
  }
  // magnitude weights, fp32, [f][4 heads]
  for (int f = tid; f < F; f += kUmmaSetupThreads) {
    float m[4];
#pragma unroll
    for (int q = 0; q < 4; ++q)
      m[q] = q < nq ? __ldg(p.weights + ((((size_t)l * p.B + b) * Hq + (size_t)qbase + q) * rows_w + 2 * O) * F + f) : 0.f;
    s_wmag[f] = make_float4(m[0], m[1], m[2], m[3]);
  }
  fence_proxy_async();  // the B operands were written through the generic proxy; the tensor core reads them through the async proxy
  tc_fence_before();
  asm volatile("bar.sync 1, %0;" ::"r"(kUmmaSetupThreads) : "memory");
  tc_fence_after();
  }

  if (wid < kUmmaEpiWarps) {
    // ------------------------------------------------------------------ epilogue: tiles with (i & 1) == group
    const int group = wid >> 2, quad = wid & 3;
    const int r = quad * 32 + lane;  // key row inside the tile = TMEM lane
    double s1[4] = {0.0, 0.0, 0.0, 0.0}, s2[4] = {0.0, 0.0, 0.0, 0.0};
    float* raw_head = p.raw + (((size_t)l * p.B + b) * p.Hkv + kvh) * (size_t)p.t_pad * p.gp_total + sub * GP;
    const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(group * kUmmaAccStride);
    const int n_used = 4 * O;  // columns beyond it are padding (zero weights): they must not enter the max
    for (int i = group; i < my_tiles; i += 2) {
      const int stage = i % kUmmaStages;
      const int use = i >> 1;  // how often this group's accumulator has been filled before
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&acc_full[group]), (uint32_t)use & 1u, err))) {
        if (lane == 0) fail();
        break;
      }
      tc_fence_after();
      float best[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      for (int c0 = 0; c0 < n_cols; c0 += 32) {
        // columns c0 .. c0+31 of the high part and of the remainder part: up to four 16-column loads per wait
        uint32_t vh[2][16], vl[2][16];
        const bool second = c0 + 16 < n_cols;
        tmem_ld16(t_row + (uint32_t)c0, vh[0]);
        tmem_ld16(t_row + (uint32_t)(n_cols + c0), vl[0]);
        if (second) {
          tmem_ld16(t_row + (uint32_t)c0 + 16u, vh[1]);
          tmem_ld16(t_row + (uint32_t)(n_cols + c0) + 16u, vl[1]);
        }
        tmem_ld_wait();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (h == 1 && !second) break;
          const int cb = c0 + 16 * h;
          const bool whole = cb + 16 <= n_used;
#pragma unroll
          for (int j = 0; j < 16; ++j)  // column cb + j = (offset, head j & 3)
            if (whole || cb + j < n_used)
              best[j & 3] = fmaxf(best[j & 3], __uint_as_float(vh[h][j]) + __uint_as_float(vl[h][j]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty[group]));
      // magnitude term of this key from the magnitude warp of the tile
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&mag_bar[stage]), (uint32_t)(i / kUmmaStages) & 1u, err))) {
        if (lane == 0) fail();
        break;
      }
      const float4 mg = s_mag[stage * kUmmaTileKeys + r];
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[stage]));  // this warp no longer reads the stage's magnitude row
      const int key = (tile0 + i) * kUmmaTileKeys + r;
      if (key < seq_len) {
        const float sc[4] = {best[0] + mg.x, best[1] + mg.y, best[2] + mg.z, best[3] + mg.w};
        float* out = raw_head + (size_t)key * p.gp_total;
        if (nq == 4) {
          *reinterpret_cast<float4*>(out) = make_float4(sc[0], sc[1], sc[2], sc[3]);
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (q < nq) out[q] = sc[q];
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          s1[q] += (double)sc[q];
          s2[q] += (double)(sc[q] * sc[q]);
        }
      }
    }
    // Moments: one pair of atomics per warp and head.  A thread's own sums are formed in a fixed order (its keys
    // are fixed by the tile split) but are not exact; snapping them to a grid (2^-20 for the sum, 2^-10 for the
    // sum of squares, both far below the fp32 rounding of a single score) makes every later addition - the
    // shuffles, the atomics of other warps and CTAs in whatever order - exact, so the moments are reproducible.
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      s1[q] = (s1[q] + 4294967296.0) - 4294967296.0;            // 2^32: unit in the last place 2^-20
      s2[q] = (s2[q] + 4398046511104.0) - 4398046511104.0;      // 2^42: unit in the last place 2^-10
#pragma unroll
      for (int s = 16; s >= 1; s >>= 1) {
        s1[q] += __shfl_xor_sync(0xffffffffu, s1[q], s);
        s2[q] += __shfl_xor_sync(0xffffffffu, s2[q], s);
      }
      if (lane == 0 && q < nq) {
        double* m = p.moments + (((size_t)l * p.B + b) * Hq + (size_t)qbase + q) * 2;
        atomicAdd(m, s1[q]);
        atomicAdd(m + 1, s2[q]);
      }
    }
  } else if (wid < kUmmaEpiWarps + kUmmaMagWarps) {
    // ------------------------------------------------------------------ magnitude: warp pair m takes tiles m, m + 4, ...
    const int mw = wid - kUmmaEpiWarps;
    const int row0 = (mw & 1) * 64 + lane;  // this thread's 2 keys: rows row0 and row0 + 32 of the tile
    for (int i = mw >> 1; i < my_tiles; i += kUmmaMagWarps / 2) {
      const int stage = i % kUmmaStages;
      if (i >= kUmmaStages) {
        // bounded: the producer arms tile i as soon as the stage's previous tile has been released
        bool armed = false;
        for (uint32_t n = 0; n < (kWaitLimit << 4) && !armed; ++n) {  // ~0.2 s of 200 ns naps
          int a;
          asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(a) : "r"(smem_u32(&s_armed[stage])) : "memory");
          armed = a == i;
          if (!armed) {
            if (*err != 0) break;
            __nanosleep(200);
          }
        }
        if (!__all_sync(0xffffffffu, armed)) {
          if (lane == 0) fail();
          break;
        }
      }
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&full_bar[stage]), (uint32_t)(i / kUmmaStages) & 1u, err))) {
        if (lane == 0) fail();
        break;
      }
      const uint32_t a_st = a_base + (uint32_t)stage * kUmmaStageBytes;
      float2 m01[2], m23[2];  // per key: heads (0,1) and (2,3)
#pragma unroll
      for (int j = 0; j < 2; ++j) m01[j] = m23[j] = make_float2(0.f, 0.f);
      auto add_freq = [&](int j, float kabs, const float4 w) {
        const float2 kk = make_float2(kabs, kabs);
        m01[j] = ffma2(kk, make_float2(w.x, w.y), m01[j]);
        m23[j] = ffma2(kk, make_float2(w.z, w.w), m23[j]);
      };
      if constexpr (!INTERLEAVED) {
#pragma unroll 4
        for (int c = 0; c < 8; ++c) {
          uint4 re[2], im[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            re[j] = lds128(a_st + key_chunk(row0 + 32 * j, 0, c));
            im[j] = lds128(a_st + key_chunk(row0 + 32 * j, 1, c));
          }
#pragma unroll
          for (int wd = 0; wd < 4; ++wd) {
            const float4 w0 = s_wmag[8 * c + 2 * wd], w1 = s_wmag[8 * c + 2 * wd + 1];  // one load serves both keys
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const uint32_t rw = wd == 0 ? re[j].x : wd == 1 ? re[j].y : wd == 2 ? re[j].z : re[j].w;
              const uint32_t iw = wd == 0 ? im[j].x : wd == 1 ? im[j].y : wd == 2 ? im[j].z : im[j].w;
              const float2 m2 = sq_mag_bf16x2(rw, iw);
              add_freq(j, sqrt_approx(m2.x), w0);
              add_freq(j, sqrt_approx(m2.y), w1);
            }
          }
        }
      } else {
#pragma unroll 2
        for (int c = 0; c < 16; ++c) {
          uint4 x[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) x[j] = lds128(a_st + key_chunk(row0 + 32 * j, c >> 3, c & 7));
#pragma unroll
          for (int wd = 0; wd < 4; ++wd) {
            const float4 w0 = s_wmag[4 * c + wd];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const uint32_t xw = wd == 0 ? x[j].x : wd == 1 ? x[j].y : wd == 2 ? x[j].z : x[j].w;
              add_freq(j, sqrt_approx(sq_mag_bf16_pair(xw)), w0);
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 2; ++j)
        s_mag[stage * kUmmaTileKeys + row0 + 32 * j] = make_float4(m01[j].x, m01[j].y, m23[j].x, m23[j].y);
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&mag_bar[stage]));    // this half of the tile's magnitude terms is written
        mbar_arrive(smem_u32(&empty_bar[stage]));  // this warp's reads of the stage's keys are done
      }
    }
  } else if (wid > kUmmaMmaWarp) {
    // ------------------------------------------------------------------ producer: boxes of keys -> ring (tiled TMA)
    const void* tmap = p.tmaps + (size_t)l * 128;
    // the map was stamped by another kernel through the generic proxy: acquire it for the tensor-map proxy
    asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(tmap) : "memory");
    int issued = 0;
    for (int i = 0; i < my_tiles; ++i, ++issued) {
      const int stage = i % kUmmaStages;
      if (i >= kUmmaStages) {
        const uint32_t ph = (uint32_t)(i / kUmmaStages - 1) & 1u;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&empty_bar[stage]), ph, err))) {
          if (lane == 0) fail();
          break;
        }
        fence_proxy_async();  // the readers' generic-proxy accesses (acquired above) before the async-proxy refill
      }
      const uint32_t a_st = a_base + (uint32_t)stage * kUmmaStageBytes;
      const uint32_t bar = smem_u32(&full_bar[stage]);
      const int t_base = (tile0 + i) * kUmmaTileKeys;
      // 16-token groups of the tile that hold at least one key of the request (whole boxes are loaded: the rows of
      // a group beyond the request's length come from its last block and are not used)
      const int groups = min(kUmmaTileKeys / 16, (seq_len - t_base + 15) / 16);
      // position of the tile's first token: block (relative to the CTA's first) and offset inside it
      int bi = t_base / p.bs;
      int in_blk = t_base - bi * p.bs;
      bi -= bi0;
      if (elect_one()) {
        // published before the arming: whoever reads i here finds the barrier in the phase of tile i or later
        asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(&s_armed[stage])), "r"(i) : "memory");
        mbar_arrive_expect_tx(bar, (uint32_t)groups * 4096u + kTestExtraTxBytes);
      }
      __syncwarp();
      for (int gi = 0; gi < groups; ++gi) {
        // one box = 16 tokens of this head, both halves: 4 KB = two 8-key groups of the stage
        const int slot = s_bt[bi] * p.tmap_slots_per_block + kvh;
        if (elect_one()) tma_load_5d(a_st + (uint32_t)gi * 4096u, tmap, bar, 0, 0, 0, in_blk >> 3, slot);
        in_blk += 16;
        if (in_blk >= p.bs) {
          in_blk = 0;
          ++bi;
        }
      }
    }
    // Nothing may still be landing when the CTA retires: the copies of the last tiles (one per stage) have
    // completed long ago on the normal path; after a timeout this is one more bounded wait for each of them.
    if (*err != 0)
      for (int j = max(0, issued - kUmmaStages); j < issued; ++j)
        mbar_wait_bounded(smem_u32(&full_bar[j % kUmmaStages]), (uint32_t)(j / kUmmaStages) & 1u);
  } else {
    // ------------------------------------------------------------------ MMA issue (one thread)
    // The whole warp runs the loop; one elected lane issues the MMAs and commits of a tile.
    // instruction descriptor: D fp32, A and B bf16, both K-major, N = n_cols, M = 128
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((2 * n_cols) >> 3) << 17) | ((128u >> 4) << 24);
    const uint64_t desc_b0 = umma_smem_desc(b_base, 1024u);
    const uint64_t b_kblock = (uint64_t)((2 * n_cols * 128) >> 4);
    for (int i = 0; i < my_tiles; ++i) {
      const int stage = i % kUmmaStages, acc = i & 1, use = i >> 1;
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&full_bar[stage]), (uint32_t)(i / kUmmaStages) & 1u, err))) {
        if (lane == 0) fail();
        break;
      }
      if (use > 0 &&
          !__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&acc_empty[acc]), (uint32_t)(use - 1) & 1u, err))) {
        if (lane == 0) fail();
        break;
      }
      fence_proxy_async();
      tc_fence_after();
      const uint64_t desc_a0 = umma_smem_desc(a_base + (uint32_t)stage * kUmmaStageBytes, (uint32_t)kUmmaGroupBytes);
      const uint32_t d_addr = tmem_base + (uint32_t)(acc * kUmmaAccStride);
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // K step of 16 dims = 32 bytes inside the 128-byte swizzle span; dims 64..127 live in the second K block
          const uint64_t ka = (uint64_t)((k & 3) * 2) + (k >= 4 ? (uint64_t)(kUmmaHalfBytes >> 4) : 0);
          const uint64_t kb = (uint64_t)((k & 3) * 2) + (k >= 4 ? b_kblock : 0);
          umma_bf16(d_addr, desc_a0 + ka, desc_b0 + kb, idesc, k ? 1u : 0u);
        }
        umma_commit(smem_u32(&acc_full[acc]));      // accumulator complete
        umma_commit(smem_u32(&empty_bar[stage]));   // the tensor core no longer reads the stage
      }
      __syncwarp();
    }
  }
  // all roles are done (or gave up): free the tensor memory
  tc_fence_before();
  __syncthreads();
  if (wid == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kUmmaTmemCols);
  }
}

}  // namespace triattn
