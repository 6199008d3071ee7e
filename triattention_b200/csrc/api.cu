// C ABI of libtriattn_b200.so: argument validation, launch geometry and kernel launches.
// No allocation, no synchronisation, no exceptions: every entry returns a triattn_status.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <mutex>

#include "../../include/triattn_b200.h"
#include "common.cuh"
#include "compact.cuh"
#include "finalize.cuh"
#include "overrides.cuh"
#include "prep.cuh"
#include "reclaim.cuh"
#include "score.cuh"
#include "score_fma.cuh"
#include "score_mma.cuh"
#include "score_mma_max.cuh"
#include "select.cuh"

using namespace triattn;

namespace {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// tuning knob read from the environment (unset or unparsable -> the built-in choice)
int env_int(const char* name, int fallback, int lo, int hi) {
  const char* v = std::getenv(name);
  if (v == nullptr || *v == 0) return fallback;
  const long x = std::strtol(v, nullptr, 10);
  return (x < lo || x > hi) ? fallback : (int)x;
}

int check_launch() { return cudaGetLastError() == cudaSuccess ? TRIATTN_OK : TRIATTN_ERR_CUDA; }

// Opt a kernel in to `smem` bytes of dynamic shared memory; the attribute call is made only when a device has
// not yet been raised to that size for this kernel.
constexpr int kMaxDevicesSmem = 64;
template <auto Kern>
bool ensure_dynamic_smem(size_t smem) {
  static std::atomic<size_t> raised[kMaxDevicesSmem];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevicesSmem) return false;
  if (raised[dev].load(std::memory_order_relaxed) >= smem) return true;
  if (cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return false;
  raised[dev].store(smem, std::memory_order_relaxed);
  return true;
}

int validate_layout(const triattn_paged_layout* L) {
  if (L == nullptr) return TRIATTN_ERR_INVALID_ARGUMENT;
  if (L->num_layers <= 0 || L->num_reqs <= 0 || L->num_kv_heads <= 0 || L->group_size <= 0 || L->head_dim <= 0 ||
      L->block_size <= 0 || L->num_blocks <= 0 || L->max_blocks_per_req <= 0)
    return TRIATTN_ERR_INVALID_ARGUMENT;
  if (L->head_dim % 8 != 0) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  if (L->num_reqs > 65535 || L->num_layers > 65535) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  if (L->block_stride % 8 != 0 || L->token_stride % 8 != 0 || L->head_stride % 8 != 0) return TRIATTN_ERR_MISALIGNED;
  return TRIATTN_OK;
}

// true when the K region of a block is one dense run of bs*Hkv*D elements in NHD or HND order
bool block_is_dense(const triattn_paged_layout* L) {
  const int64_t D = L->head_dim, H = L->num_kv_heads, bs = L->block_size;
  const bool nhd = L->head_stride == D && L->token_stride == H * D;
  const bool hnd = L->token_stride == D && L->head_stride == bs * D;
  return nhd || hnd || (H == 1 && L->token_stride == D) || (bs == 1 && L->head_stride == D);
}

template <int D, bool IL>
int launch_score_fma(const ScoreParams& p, int gp, dim3 grid, size_t smem, cudaStream_t st) {
#define TRIATTN_LAUNCH(GP)                                                                                  \
  {                                                                                                         \
    if (!ensure_dynamic_smem<score_paged_mean_kernel<D, GP, IL>>(smem)) return TRIATTN_ERR_CUDA;             \
    score_paged_mean_kernel<D, GP, IL><<<grid, kScoreThreadsWS, smem, st>>>(p);                             \
    return check_launch();                                                                                  \
  }
  switch (gp) {
    case 1: TRIATTN_LAUNCH(1)
    case 2: TRIATTN_LAUNCH(2)
    case 4: TRIATTN_LAUNCH(4)
    default: return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  }
#undef TRIATTN_LAUNCH
}

// TRIATTN_SCORE_PATH=fma selects the CUDA-core streaming kernel (no tensor cores); anything else the default.
bool score_path_is_fma() {
  const char* v = std::getenv("TRIATTN_SCORE_PATH");
  return v != nullptr && v[0] == 'f' && v[1] == 'm' && v[2] == 'a' && v[3] == 0;
}

template <int D, bool IL>
int launch_score_mma(const ScoreParams& p, dim3 grid, size_t smem, cudaStream_t st) {
#define TRIATTN_LAUNCH(NT)                                                                                  \
  {                                                                                                         \
    if (!ensure_dynamic_smem<score_paged_mma_kernel<D, IL, NT>>(smem)) return TRIATTN_ERR_CUDA;              \
    score_paged_mma_kernel<D, IL, NT><<<grid, kScoreThreadsWS, smem, st>>>(p);                              \
    return check_launch();                                                                                  \
  }
  if (p.gp_total <= 4) TRIATTN_LAUNCH(1)
  TRIATTN_LAUNCH(2)
#undef TRIATTN_LAUNCH
}

}  // namespace

extern "C" {

int triattn_abi_version(void) { return TRIATTN_ABI_VERSION; }

const char* triattn_status_string(int status) {
  switch (status) {
    case TRIATTN_OK: return "ok";
    case TRIATTN_ERR_INVALID_ARGUMENT: return "invalid argument";
    case TRIATTN_ERR_UNSUPPORTED_SHAPE: return "unsupported shape";
    case TRIATTN_ERR_MISALIGNED: return "pointer or stride not 16-byte aligned";
    case TRIATTN_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case TRIATTN_ERR_CUDA: return "CUDA runtime error";
    case TRIATTN_ERR_LIMIT_EXCEEDED: return "size exceeds the fixed maximum of this entry point";
    default: return "unknown status";
  }
}

int triattn_padded_group(int g) {
  if (g <= 0 || g > 64) return 0;
  if (g > 4) return (g + 3) / 4 * 4;
  int gp = 1;
  while (gp < g) gp <<= 1;
  return gp;
}

int triattn_weight_rows(int offset_agg, int num_offsets) {
  return offset_agg == TRIATTN_OFFSETS_MAX ? 2 * num_offsets + 1 : 3;
}

size_t triattn_prep_scratch_floats(int num_reqs, int num_freqs, int num_offsets, int offset_agg) {
  const size_t rows = offset_agg == TRIATTN_OFFSETS_MAX ? 2 * (size_t)num_offsets : 2;
  return (size_t)num_reqs * rows * (size_t)num_freqs;
}

int triattn_prep_weights(const float* q_mean_real, const float* q_mean_imag, const float* q_abs_mean,
                         const float* freq_scale_sq, const float* omega, const float* offsets,
                         const int32_t* round_start, int num_layers, int num_reqs, int num_q_heads, int num_freqs,
                         int num_offsets, int offset_agg, int flags, float* scratch, float* weights_out,
                         void* stream) {
  if (!q_mean_real || !q_mean_imag || !q_abs_mean || !freq_scale_sq || !omega || !offsets || !round_start ||
      !scratch || !weights_out)
    return TRIATTN_ERR_INVALID_ARGUMENT;
  if (num_layers <= 0 || num_reqs <= 0 || num_q_heads <= 0 || num_freqs <= 0 || num_offsets <= 0)
    return TRIATTN_ERR_INVALID_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int agg_max = offset_agg == TRIATTN_OFFSETS_MAX ? 1 : 0;
  trig_table_kernel<<<num_reqs, 64, 0, st>>>(omega, offsets, round_start, num_freqs, num_offsets, agg_max, scratch);
  const size_t n = (size_t)num_layers * num_reqs * num_q_heads * num_freqs;
  fold_weights_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(q_mean_real, q_mean_imag, q_abs_mean, freq_scale_sq,
                                                                   scratch, num_layers, num_reqs, num_q_heads,
                                                                   num_freqs, num_offsets, agg_max, flags, weights_out);
  return check_launch();
}

// ------------------------------------------------------------------------- allocation-free prep
// Trig-table scratch that lives in the library image, for callers that cannot allocate.  In host
// code the name below is only a host-side stand-in for the device array, never a device address:
// the pointer handed to kernels comes from cudaGetSymbolAddress, looked up once per device.
static __device__ __align__(256) float g_noalloc_prep_scratch[TRIATTN_NOALLOC_PREP_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mutex;
float* g_noalloc_prep_ptr[kMaxDevices] = {};
}  // namespace

int triattn_prep_weights_noalloc(const float* q_mean_real, const float* q_mean_imag, const float* q_abs_mean,
                                 const float* freq_scale_sq, const float* omega, const float* offsets,
                                 const int32_t* round_start, int num_layers, int num_reqs, int num_q_heads,
                                 int num_freqs, int num_offsets, int offset_agg, int flags, float* weights_out,
                                 void* stream) {
  if (num_layers <= 0 || num_reqs <= 0 || num_q_heads <= 0 || num_freqs <= 0 || num_offsets <= 0)
    return TRIATTN_ERR_INVALID_ARGUMENT;
  if (triattn_prep_scratch_floats(num_reqs, num_freqs, num_offsets, offset_agg) >
      (size_t)TRIATTN_NOALLOC_PREP_SCRATCH_FLOATS)
    return TRIATTN_ERR_LIMIT_EXCEEDED;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return TRIATTN_ERR_CUDA;
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_prep_ptr[dev] == nullptr) {
      // set-up, once per device, with that device current
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_noalloc_prep_scratch) != cudaSuccess || p == nullptr) return TRIATTN_ERR_CUDA;
      g_noalloc_prep_ptr[dev] = static_cast<float*>(p);
    }
    scratch = g_noalloc_prep_ptr[dev];
  }
  return triattn_prep_weights(q_mean_real, q_mean_imag, q_abs_mean, freq_scale_sq, omega, offsets, round_start,
                              num_layers, num_reqs, num_q_heads, num_freqs, num_offsets, offset_agg, flags, scratch,
                              weights_out, stream);
}

int triattn_score_paged(const triattn_paged_layout* layout, const void* const* k_layer_ptrs,
                        const int32_t* block_table, const int32_t* seq_lens, const float* weights, int offset_agg,
                        int num_offsets, float* raw_scores, double* moments, uint32_t* device_status, void* stream) {
  int rc = validate_layout(layout);
  if (rc != TRIATTN_OK) return rc;
  if (!k_layer_ptrs || !block_table || !seq_lens || !weights || !raw_scores || !moments)
    return TRIATTN_ERR_INVALID_ARGUMENT;
  const triattn_paged_layout& Y = *layout;
  const int gp = triattn_padded_group(Y.group_size);
  if (gp == 0) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int Hq = Y.num_kv_heads * Y.group_size;
  if (cudaMemsetAsync(moments, 0, sizeof(double) * 2 * (size_t)Y.num_layers * Y.num_reqs * Hq, st) != cudaSuccess)
    return TRIATTN_ERR_CUDA;

  ScoreParams p{};
  p.k_ptrs = k_layer_ptrs;
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.weights = weights;
  p.raw = raw_scores;
  p.moments = moments;
  p.status = device_status;
  p.L = Y.num_layers;
  p.B = Y.num_reqs;
  p.Hkv = Y.num_kv_heads;
  p.g = Y.group_size;
  p.bs = Y.block_size;
  p.num_blocks = Y.num_blocks;
  p.max_blocks = Y.max_blocks_per_req;
  p.t_pad = Y.max_blocks_per_req * Y.block_size;
  p.block_stride_bytes = (long long)Y.block_stride * 2;
  p.token_stride = (int)Y.token_stride;
  p.head_stride = (int)Y.head_stride;
  p.num_offsets = num_offsets;
  p.agg_max = offset_agg == TRIATTN_OFFSETS_MAX ? 1 : 0;

  const long long block_bytes = (long long)Y.block_size * Y.num_kv_heads * Y.head_dim * 2;
  p.gp_total = gp;
  const bool nhd = Y.head_stride == Y.head_dim && Y.token_stride == (int64_t)Y.num_kv_heads * Y.head_dim;
  p.nhd = nhd ? 1 : 0;
  // Streaming tensor-core kernel: mean aggregation, head_dim 64/128, K region of a block one dense run.
  const bool streamable = !p.agg_max && (Y.head_dim == 64 || Y.head_dim == 128) && block_is_dense(layout) &&
                          block_bytes <= 64 * 1024 && (block_bytes % 16) == 0 && (p.block_stride_bytes % 16) == 0;
  if (streamable) {
    // cache blocks per pipeline stage: a power of two filling ~32 KB (8 work items of 16 keys for 8 KV heads)
    int mb = 1;
    while ((mb * 2) * block_bytes <= 32 * 1024) mb *= 2;
    mb = env_int("TRIATTN_SCORE_MB", mb, 1, 64);
    while (mb > 1 && (long long)mb * block_bytes > 96 * 1024) mb /= 2;
    const long long stage_bytes = (long long)mb * block_bytes;
    // two CTAs per SM share ~200 KB of shared memory
    const long long budget = 100 * 1024;
    int stages = (int)std::min<long long>(4, budget / stage_bytes);
    stages = env_int("TRIATTN_SCORE_STAGES", stages, 1, kMaxStages);
    if (stages < 2) stages = 2;
    while (stages > 2 && stages * stage_bytes > 200 * 1024) --stages;
    p.block_bytes = (int)block_bytes;
    p.mb = mb;
    p.stages = stages;
    p.block_group = (gp <= 8 && Y.block_size == 16 && Y.num_kv_heads * mb == kScoreConsumerWarps &&
                     !score_path_is_fma() && env_int("TRIATTN_SCORE_BLOCK_GROUPS", 1, 0, 1) == 1)
                        ? Y.num_kv_heads : 0;
    const int max_tiles = (Y.max_blocks_per_req + mb - 1) / mb;
    // Tiles per CTA: every CTA pays a fixed start-up (weight fragments, first copies: about two tiles' worth) and
    // the CTAs run in waves of 2 per SM, so the launch takes about waves(tpc) * (tpc + 2) tile times; take the
    // tpc that minimises it.  At least ~64 KB and at most ~2 MB of keys per CTA, and the CTA's block ids must
    // fit its shared-memory table.
    const int min_tpc = (int)std::max<long long>(1, (64 * 1024) / stage_bytes);
    int max_tpc = (int)std::max<long long>(min_tpc, (2 * 1024 * 1024) / stage_bytes);
    max_tpc = std::max(1, std::min(max_tpc, kMaxPrefetchedBlocks / mb));
    const int lo_tpc = std::min(min_tpc, max_tpc);
    int tpc = lo_tpc;
    {
      const long long slots = (long long)kSMs * 2;
      const long long lb = (long long)Y.num_layers * Y.num_reqs;
      long long best = -1;
      for (int c = lo_tpc; c <= std::min(max_tpc, max_tiles); ++c) {
        const long long per_lb = (max_tiles + c - 1) / c;
        const int share = (int)((max_tiles + per_lb - 1) / per_lb);  // equal shares for the CTAs of one (layer, request)
        const long long waves = (per_lb * lb + slots - 1) / slots;
        const long long cost = waves * (share + 2);
        if (best < 0 || cost < best) {
          best = cost;
          tpc = share;
        }
      }
    }
    tpc = env_int("TRIATTN_SCORE_TILES_PER_CTA", tpc, 1, 1 << 20);
    p.tiles_per_cta = tpc;
    dim3 grid((unsigned)((max_tiles + tpc - 1) / tpc), (unsigned)Y.num_layers, (unsigned)Y.num_reqs);
    const size_t smem = (size_t)stages * stage_bytes;
    if (score_path_is_fma()) {
      // the CUDA-core kernel works on batches of 16/gpv tokens and keeps a table of work items per stage
      const int gpv = std::min(gp, 4), nsub = gp / gpv, nt = kLPK / gpv;
      const long long stage_tok = (long long)mb * Y.block_size;
      const long long n_items = nhd ? (long long)Y.num_kv_heads * nsub * (stage_tok / nt)
                                    : (long long)mb * Y.num_kv_heads * nsub * (Y.block_size / nt);
      const bool ok = (nhd ? (stage_tok % nt) == 0 : (Y.block_size % nt) == 0) && n_items > 0 && n_items <= kMaxScoreItems;
      if (ok) {
        if (Y.head_dim == 128)
          return Y.rope_interleaved ? launch_score_fma<128, true>(p, gpv, grid, smem, st)
                                    : launch_score_fma<128, false>(p, gpv, grid, smem, st);
        return Y.rope_interleaved ? launch_score_fma<64, true>(p, gpv, grid, smem, st)
                                  : launch_score_fma<64, false>(p, gpv, grid, smem, st);
      }
    }
    if (Y.head_dim == 128)
      return Y.rope_interleaved ? launch_score_mma<128, true>(p, grid, smem, st)
                                : launch_score_mma<128, false>(p, grid, smem, st);
    return Y.rope_interleaved ? launch_score_mma<64, true>(p, grid, smem, st)
                              : launch_score_mma<64, false>(p, grid, smem, st);
  }
  // max over offsets on the tensor cores: one CTA per (layer, request, virtual head, run of 16-key tiles)
  if (p.agg_max && (Y.head_dim == 64 || Y.head_dim == 128) && (p.block_stride_bytes % 16) == 0 &&
      max_agg_smem_bytes(Y.head_dim, num_offsets) <= 220 * 1024 && env_int("TRIATTN_SCORE_MAX_MMA", 1, 0, 1) == 1) {
    const int nvh = Y.num_kv_heads * ((gp + 3) / 4);
    const int n_tiles = (p.t_pad + kMmaKeys - 1) / kMmaKeys;
    p.tiles_per_cta = std::min(n_tiles, 16 * kMaxAggWarps);
    const int chunks = (n_tiles + p.tiles_per_cta - 1) / p.tiles_per_cta;
    dim3 grid((unsigned)(nvh * chunks), (unsigned)Y.num_layers, (unsigned)Y.num_reqs);
    const size_t smem = max_agg_smem_bytes(Y.head_dim, num_offsets);
#define TRIATTN_LAUNCH(D, IL)                                                                      \
  {                                                                                                \
    if (!ensure_dynamic_smem<score_paged_mma_max_kernel<D, IL>>(smem)) return TRIATTN_ERR_CUDA;    \
    score_paged_mma_max_kernel<D, IL><<<grid, kMaxAggThreads, smem, st>>>(p);                      \
    return check_launch();                                                                         \
  }
    if (Y.head_dim == 128) {
      if (Y.rope_interleaved) TRIATTN_LAUNCH(128, true) else TRIATTN_LAUNCH(128, false)
    } else {
      if (Y.rope_interleaved) TRIATTN_LAUNCH(64, true) else TRIATTN_LAUNCH(64, false)
    }
#undef TRIATTN_LAUNCH
  }
  dim3 grid((unsigned)((p.t_pad + 127) / 128), (unsigned)Y.num_kv_heads, (unsigned)(Y.num_layers * Y.num_reqs));
  if ((long long)Y.num_layers * Y.num_reqs > 65535) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  score_paged_generic_kernel<<<grid, 128, 0, st>>>(p, Y.head_dim, Y.rope_interleaved);
  return check_launch();
}

int triattn_finalize_scores(const triattn_paged_layout* layout, const float* raw_scores, const double* moments,
                            const int32_t* seq_lens, const int32_t* prefill_lens, int window, int normalize,
                            int group_reduce, int head_reduce, int layer_reduce, float* mean_std_scratch,
                            float* scores_out, void* stream) {
  int rc = validate_layout(layout);
  if (rc != TRIATTN_OK) return rc;
  if (!raw_scores || !moments || !seq_lens || !mean_std_scratch || !scores_out) return TRIATTN_ERR_INVALID_ARGUMENT;
  if (group_reduce != TRIATTN_REDUCE_MAX && group_reduce != TRIATTN_REDUCE_MEAN) return TRIATTN_ERR_INVALID_ARGUMENT;
  if (head_reduce != TRIATTN_REDUCE_NONE && head_reduce != TRIATTN_REDUCE_MAX) return TRIATTN_ERR_INVALID_ARGUMENT;
  if (layer_reduce < TRIATTN_REDUCE_NONE || layer_reduce > TRIATTN_REDUCE_MAX) return TRIATTN_ERR_INVALID_ARGUMENT;
  const triattn_paged_layout& Y = *layout;
  const int gp = triattn_padded_group(Y.group_size);
  if (gp == 0) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int Hq = Y.num_kv_heads * Y.group_size;
  const int t_pad = Y.max_blocks_per_req * Y.block_size;
  const int n = Y.num_layers * Y.num_reqs * Hq;
  moments_to_mean_std_kernel<<<(n + 127) / 128, 128, 0, st>>>(moments, seq_lens, Y.num_layers, Y.num_reqs, Hq, t_pad,
                                                             mean_std_scratch);
  FinalizeParams p{};
  p.raw = raw_scores;
  p.mean_std = mean_std_scratch;
  p.seq_lens = seq_lens;
  p.prefill_lens = prefill_lens;
  p.out = scores_out;
  p.L = Y.num_layers;
  p.B = Y.num_reqs;
  p.Hkv = Y.num_kv_heads;
  p.g = Y.group_size;
  p.t_pad = t_pad;
  p.window = window;
  p.normalize = normalize;
  p.group_reduce = group_reduce;
  p.head_reduce = head_reduce;
  p.layer_reduce = layer_reduce;
  const int Ho = head_reduce != TRIATTN_REDUCE_NONE ? 1 : Y.num_kv_heads;
  dim3 grid((unsigned)((t_pad + 255) / 256), (unsigned)Ho, (unsigned)Y.num_reqs);
  p.gp = gp;
  if (head_reduce == TRIATTN_REDUCE_NONE && Y.group_size <= 8 && (gp == 4 || gp == 8)) {
#define TRIATTN_FIN(G)                                                                                \
  case G:                                                                                             \
    if (layer_reduce == TRIATTN_REDUCE_NONE)                                                          \
      finalize_scores_fast_kernel<G, TRIATTN_REDUCE_NONE><<<grid, 256, 0, st>>>(p);                   \
    else if (layer_reduce == TRIATTN_REDUCE_MAX)                                                      \
      finalize_scores_fast_kernel<G, TRIATTN_REDUCE_MAX><<<grid, 256, 0, st>>>(p);                    \
    else                                                                                              \
      finalize_scores_fast_kernel<G, TRIATTN_REDUCE_MEAN><<<grid, 256, 0, st>>>(p);                   \
    break;
    switch (Y.group_size) {
      TRIATTN_FIN(3) TRIATTN_FIN(4) TRIATTN_FIN(5) TRIATTN_FIN(6) TRIATTN_FIN(7) TRIATTN_FIN(8)
      default: finalize_scores_kernel<<<grid, 256, 0, st>>>(p);
    }
#undef TRIATTN_FIN
  } else {
    finalize_scores_kernel<<<grid, 256, 0, st>>>(p);
  }
  return check_launch();
}

int triattn_select_topk(const float* scores, int num_rows, int64_t row_stride, const int32_t* seq_lens,
                        const int32_t* keep_counts, int num_reqs, int rows_per_req_inner, int32_t* keep_out,
                        int keep_pitch, uint32_t* device_status, void* stream) {
  if (!scores || !seq_lens || !keep_counts || !keep_out) return TRIATTN_ERR_INVALID_ARGUMENT;
  if (num_rows <= 0 || row_stride <= 0 || num_reqs <= 0 || rows_per_req_inner <= 0 || keep_pitch <= 0)
    return TRIATTN_ERR_INVALID_ARGUMENT;
  SelectParams p{};
  p.scores = scores;
  p.row_stride = row_stride;
  p.seq_lens = seq_lens;
  p.keep_counts = keep_counts;
  p.num_reqs = num_reqs;
  p.rows_inner = rows_per_req_inner;
  p.keep_out = keep_out;
  p.keep_pitch = keep_pitch;
  p.status = device_status;
  select_topk_kernel<<<num_rows, kSelectThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_launch();
}

static int compact_common(const triattn_paged_layout* layout, void* const* k_layer_ptrs, void* const* v_layer_ptrs,
                          const int32_t* block_table, const int32_t* seq_lens, const int32_t* keep,
                          int64_t keep_ls, int64_t keep_rs, int64_t keep_hs, const int32_t* keep_counts,
                          void* scratch, long long scratch_stream_bytes, int scratch_rows, bool preserve,
                          uint32_t* device_status, void* stream) {
  int rc = validate_layout(layout);
  if (rc != TRIATTN_OK) return rc;
  if (!k_layer_ptrs || !v_layer_ptrs || !block_table || !seq_lens || !keep || !keep_counts)
    return TRIATTN_ERR_INVALID_ARGUMENT;
  const triattn_paged_layout& Y = *layout;
  const int row_bytes = Y.head_dim * 2;
  if (row_bytes % 16 != 0) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  const int ppr = row_bytes / 16, nsub = (ppr + 31) / 32;
  if (ppr % nsub != 0) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  // row offsets inside a layer's pool are kept as 32-bit counts of 16 bytes: pools up to 64 GB per layer
  if (((long long)Y.num_blocks * Y.block_stride >> 3) >= (1ll << 32) - (1ll << 20)) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  CompactParams p{};
  p.nsub = nsub;
  p.k_ptrs = k_layer_ptrs;
  p.v_ptrs = v_layer_ptrs;
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.keep = keep;
  p.keep_ls = keep_ls;
  p.keep_rs = keep_rs;
  p.keep_hs = keep_hs;
  p.keep_counts = keep_counts;
  p.status = device_status;
  p.L = Y.num_layers;
  p.B = Y.num_reqs;
  p.Hkv = Y.num_kv_heads;
  p.bs = Y.block_size;
  p.num_blocks = Y.num_blocks;
  p.max_blocks = Y.max_blocks_per_req;
  p.block_stride = Y.block_stride;
  p.token_stride = Y.token_stride;
  p.head_stride = Y.head_stride;
  p.row_bytes = row_bytes;
  p.scratch = static_cast<unsigned char*>(scratch);
  p.scratch_stream_bytes = scratch_stream_bytes;
  p.scratch_rows = scratch_rows;
  dim3 grid((unsigned)(Y.num_kv_heads * 2), (unsigned)Y.num_layers, (unsigned)Y.num_reqs);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (preserve)
    compact_paged_kernel<true><<<grid, kCompactThreads, 0, st>>>(p);
  else
    compact_paged_kernel<false><<<grid, kCompactThreads, 0, st>>>(p);
  return check_launch();
}

int triattn_compact_paged(const triattn_paged_layout* layout, void* const* k_layer_ptrs, void* const* v_layer_ptrs,
                          const int32_t* block_table, const int32_t* seq_lens, const int32_t* keep,
                          int64_t keep_layer_stride, int64_t keep_req_stride, int64_t keep_head_stride,
                          const int32_t* keep_counts, uint32_t* device_status, void* stream) {
  return compact_common(layout, k_layer_ptrs, v_layer_ptrs, block_table, seq_lens, keep, keep_layer_stride,
                        keep_req_stride, keep_head_stride, keep_counts, nullptr, 0, 0, false, device_status, stream);
}

size_t triattn_compact_preserve_scratch_bytes(const triattn_paged_layout* layout, int max_dropped_rows) {
  if (validate_layout(layout) != TRIATTN_OK || max_dropped_rows < 0) return 0;
  const size_t per_stream = round_up((size_t)max_dropped_rows * layout->head_dim * 2, 256);
  return per_stream * 2 * (size_t)layout->num_layers * layout->num_reqs * layout->num_kv_heads;
}

int triattn_compact_paged_preserve(const triattn_paged_layout* layout, void* const* k_layer_ptrs,
                                   void* const* v_layer_ptrs, const int32_t* block_table, const int32_t* seq_lens,
                                   const int32_t* keep, int64_t keep_layer_stride, int64_t keep_req_stride,
                                   int64_t keep_head_stride, const int32_t* keep_counts, int max_dropped_rows,
                                   void* scratch, size_t scratch_bytes, uint32_t* device_status, void* stream) {
  int rc = validate_layout(layout);
  if (rc != TRIATTN_OK) return rc;
  if (!scratch || !aligned16(scratch) || max_dropped_rows < 0) return TRIATTN_ERR_INVALID_ARGUMENT;
  const size_t need = triattn_compact_preserve_scratch_bytes(layout, max_dropped_rows);
  if (scratch_bytes < need) return TRIATTN_ERR_WORKSPACE_TOO_SMALL;
  const size_t per_stream = round_up((size_t)max_dropped_rows * layout->head_dim * 2, 256);
  return compact_common(layout, k_layer_ptrs, v_layer_ptrs, block_table, seq_lens, keep, keep_layer_stride,
                        keep_req_stride, keep_head_stride, keep_counts, scratch, (long long)per_stream,
                        max_dropped_rows, true, device_status, stream);
}

int triattn_rewrite_block_tables(int32_t* block_table, int num_reqs, int max_blocks_per_req, int block_size,
                                 const int32_t* blocks_before, const int32_t* lens_after, int32_t* blocks_after,
                                 int32_t* freed_ids, int freed_capacity, int32_t* freed_count, int32_t fill_value,
                                 uint32_t* device_status, void* stream) {
  if (!block_table || !blocks_before || !lens_after || !blocks_after || !freed_count) return TRIATTN_ERR_INVALID_ARGUMENT;
  if (num_reqs <= 0 || max_blocks_per_req <= 0 || block_size <= 0 || freed_capacity < 0) return TRIATTN_ERR_INVALID_ARGUMENT;
  if (freed_capacity > 0 && !freed_ids) return TRIATTN_ERR_INVALID_ARGUMENT;
  ReclaimParams p{};
  p.block_table = block_table;
  p.blocks_before = blocks_before;
  p.lens_after = lens_after;
  p.blocks_after = blocks_after;
  p.freed_ids = freed_ids;
  p.freed_count = freed_count;
  p.status = device_status;
  p.B = num_reqs;
  p.max_blocks = max_blocks_per_req;
  p.block_size = block_size;
  p.freed_capacity = freed_capacity;
  p.fill_value = fill_value;
  rewrite_block_tables_kernel<<<1, kReclaimThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_launch();
}

int triattn_apply_effective_overrides(const int32_t* idx_mapping, const int32_t* query_start_loc, int num_reqs,
                                      const int32_t* effective_base, const int32_t* pos_delta, int num_rows,
                                      int32_t* seq_lens, const int64_t* positions, int64_t* positions_out,
                                      int num_tokens, int32_t* counters, int apply, void* stream) {
  if (!idx_mapping || !query_start_loc || !counters || num_reqs <= 0 || num_rows < 0 || num_tokens < 0)
    return TRIATTN_ERR_INVALID_ARGUMENT;
  if (positions != nullptr && positions_out == nullptr) return TRIATTN_ERR_INVALID_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(counters, 0, 4 * sizeof(int32_t), st) != cudaSuccess) return TRIATTN_ERR_CUDA;
  OverrideParams p{};
  p.idx_mapping = idx_mapping;
  p.query_start_loc = query_start_loc;
  p.num_reqs = num_reqs;
  p.effective_base = effective_base;
  p.pos_delta = pos_delta;
  p.num_rows = num_rows;
  p.seq_lens = seq_lens;
  p.positions = positions;
  p.positions_out = positions_out;
  p.num_tokens = num_tokens;
  p.counters = counters;
  p.apply = apply ? 1 : 0;
  const int n = std::max(num_reqs, positions != nullptr ? num_tokens : 0);
  apply_effective_overrides_kernel<<<(n + 255) / 256, 256, 0, st>>>(p);
  return check_launch();
}

// ------------------------------------------------------------------------- fused step
namespace {
struct CompressWs {
  size_t trig, weights, raw, moments, mean_std, final_scores, total;
};
CompressWs compress_ws_layout(const triattn_paged_layout& Y, int num_offsets, int offset_agg) {
  CompressWs w{};
  const int F = Y.head_dim / 2;
  const int Hq = Y.num_kv_heads * Y.group_size;
  const int gp = std::max(1, triattn_padded_group(Y.group_size));
  const size_t t_pad = (size_t)Y.max_blocks_per_req * Y.block_size;
  size_t off = 0;
  w.trig = off;
  off += round_up(sizeof(float) * triattn_prep_scratch_floats(Y.num_reqs, F, num_offsets, offset_agg), 256);
  w.weights = off;
  off += round_up(sizeof(float) * (size_t)Y.num_layers * Y.num_reqs * Hq * triattn_weight_rows(offset_agg, num_offsets) * F, 256);
  w.raw = off;
  off += round_up(sizeof(float) * (size_t)Y.num_layers * Y.num_reqs * Y.num_kv_heads * t_pad * gp, 256);
  w.moments = off;
  off += round_up(sizeof(double) * 2 * (size_t)Y.num_layers * Y.num_reqs * Hq, 256);
  w.mean_std = off;
  off += round_up(sizeof(float) * 2 * (size_t)Y.num_layers * Y.num_reqs * Hq, 256);
  w.final_scores = off;
  off += round_up(sizeof(float) * (size_t)Y.num_reqs * Y.num_kv_heads * t_pad, 256);
  w.total = off;
  return w;
}
}  // namespace

size_t triattn_compress_workspace_bytes(const triattn_paged_layout* layout, int num_offsets, int offset_agg,
                                        int keep_pitch) {
  (void)keep_pitch;
  if (validate_layout(layout) != TRIATTN_OK || num_offsets <= 0) return 0;
  return compress_ws_layout(*layout, num_offsets, offset_agg).total;
}

int triattn_compress_paged(const triattn_paged_layout* layout, void* const* k_layer_ptrs, void* const* v_layer_ptrs,
                           const int32_t* block_table, const int32_t* seq_lens, const int32_t* round_start,
                           const int32_t* prefill_lens, const int32_t* keep_counts, const float* q_mean_real,
                           const float* q_mean_imag, const float* q_abs_mean, const float* freq_scale_sq,
                           const float* omega, const float* offsets, int num_offsets, int offset_agg, int flags,
                           int window, int normalize, int layer_reduce, void* workspace, size_t workspace_bytes,
                           int32_t* keep_out, int keep_pitch, uint32_t* device_status, void* stream) {
  int rc = validate_layout(layout);
  if (rc != TRIATTN_OK) return rc;
  if (!workspace || !aligned16(workspace) || !keep_out || keep_pitch <= 0 || num_offsets <= 0)
    return TRIATTN_ERR_INVALID_ARGUMENT;
  if (layer_reduce != TRIATTN_REDUCE_MEAN && layer_reduce != TRIATTN_REDUCE_MAX) return TRIATTN_ERR_INVALID_ARGUMENT;
  const triattn_paged_layout& Y = *layout;
  const CompressWs w = compress_ws_layout(Y, num_offsets, offset_agg);
  if (workspace_bytes < w.total) return TRIATTN_ERR_WORKSPACE_TOO_SMALL;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  float* trig = reinterpret_cast<float*>(ws + w.trig);
  float* weights = reinterpret_cast<float*>(ws + w.weights);
  float* raw = reinterpret_cast<float*>(ws + w.raw);
  double* moments = reinterpret_cast<double*>(ws + w.moments);
  float* mean_std = reinterpret_cast<float*>(ws + w.mean_std);
  float* fin = reinterpret_cast<float*>(ws + w.final_scores);
  const int Hq = Y.num_kv_heads * Y.group_size;
  const int64_t t_pad = (int64_t)Y.max_blocks_per_req * Y.block_size;

  rc = triattn_prep_weights(q_mean_real, q_mean_imag, q_abs_mean, freq_scale_sq, omega, offsets, round_start,
                            Y.num_layers, Y.num_reqs, Hq, Y.head_dim / 2, num_offsets, offset_agg, flags, trig,
                            weights, stream);
  if (rc != TRIATTN_OK) return rc;
  rc = triattn_score_paged(layout, reinterpret_cast<const void* const*>(k_layer_ptrs), block_table, seq_lens,
                           weights, offset_agg, num_offsets, raw, moments, device_status, stream);
  if (rc != TRIATTN_OK) return rc;
  rc = triattn_finalize_scores(layout, raw, moments, seq_lens, prefill_lens, window, normalize, TRIATTN_REDUCE_MAX,
                               TRIATTN_REDUCE_NONE, layer_reduce, mean_std, fin, stream);
  if (rc != TRIATTN_OK) return rc;
  rc = triattn_select_topk(fin, Y.num_reqs * Y.num_kv_heads, t_pad, seq_lens, keep_counts, Y.num_reqs,
                           Y.num_kv_heads, keep_out, keep_pitch, device_status, stream);
  if (rc != TRIATTN_OK) return rc;
  return triattn_compact_paged(layout, k_layer_ptrs, v_layer_ptrs, block_table, seq_lens, keep_out, 0,
                               (int64_t)Y.num_kv_heads * keep_pitch, keep_pitch, keep_counts, device_status, stream);
}

}  // extern "C"
