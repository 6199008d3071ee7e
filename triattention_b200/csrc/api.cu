// C ABI of libtriattn_b200.so: argument validation, launch geometry and kernel launches.
// No allocation, no synchronisation, no exceptions: every entry returns a triattn_status.
#include <cuda.h>  // tensor-map types; cuTensorMapEncodeTiled itself is looked up at run time (no link against libcuda)
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <utility>

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
#include "score_umma_max.cuh"
#include "select.cuh"

using namespace triattn;

namespace {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int check_launch() { return cudaGetLastError() == cudaSuccess ? TRIATTN_OK : TRIATTN_ERR_CUDA; }

// Kernel launch, optionally as a programmatic dependent of the preceding kernel in the stream: the launch is
// processed and its CTAs become resident while that kernel drains (every kernel of this library starts with
// griddepcontrol.wait, so nothing is read or written before the predecessor has completed).
template <typename... KArgs, typename... Args>
int launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...) == cudaSuccess ? TRIATTN_OK : TRIATTN_ERR_CUDA;
}

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
int launch_score_fma(const ScoreParams& p, int gp, dim3 grid, size_t smem, cudaStream_t st, bool pdl) {
#define TRIATTN_LAUNCH(GP)                                                                                  \
  {                                                                                                         \
    if (!ensure_dynamic_smem<score_paged_mean_kernel<D, GP, IL>>(smem)) return TRIATTN_ERR_CUDA;             \
    return launch_kernel(score_paged_mean_kernel<D, GP, IL>, grid, dim3(kScoreThreadsWS), smem, st, pdl, p); \
  }
  switch (gp) {
    case 1: TRIATTN_LAUNCH(1)
    case 2: TRIATTN_LAUNCH(2)
    case 4: TRIATTN_LAUNCH(4)
    default: return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  }
#undef TRIATTN_LAUNCH
}

template <int D, bool IL>
int launch_score_mma(const ScoreParams& p, dim3 grid, size_t smem, cudaStream_t st, bool pdl) {
#define TRIATTN_LAUNCH(NT)                                                                                  \
  {                                                                                                         \
    if (!ensure_dynamic_smem<score_paged_mma_kernel<D, IL, NT>>(smem)) return TRIATTN_ERR_CUDA;              \
    return launch_kernel(score_paged_mma_kernel<D, IL, NT>, grid, dim3(kScoreThreadsWS), smem, st, pdl, p);  \
  }
  if (p.gp_total <= 4) TRIATTN_LAUNCH(1)
  TRIATTN_LAUNCH(2)
#undef TRIATTN_LAUNCH
}

// ------------------------------------------------------------------------- tensor maps for the tcgen05 scorer
// Per-layer tensor maps live in a ring of slots inside the library image (the entry points allocate nothing):
// kTmapRing consecutive scoring calls each get their own kTmapMaxLayers slots, so a call's maps are overwritten
// only after kTmapRing later max-aggregation calls on the same device have been issued.
constexpr int kTmapRing = 8;
constexpr int kTmapMaxLayers = 128;
static __device__ __align__(128) unsigned char g_tmap_slots[kTmapRing * kTmapMaxLayers * 128];
std::mutex g_tmap_mutex;
unsigned char* g_tmap_ptr[kMaxDevicesSmem] = {};
std::atomic<unsigned> g_tmap_call{0};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static std::atomic<void*> cached{nullptr};
  void* f = cached.load(std::memory_order_acquire);
  if (f == nullptr) {
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    cached.store(f, std::memory_order_release);
  }
  return reinterpret_cast<EncodeTiledFn>(f);
}

// Slots of this call (device pointer) or nullptr; also stamps the layers' K pointers into them on `st`.
const unsigned char* stamp_layer_tensor_maps(const triattn_paged_layout& Y, const void* const* k_layer_ptrs,
                                             cudaStream_t st, bool pdl) {
  if (Y.num_layers > kTmapMaxLayers) return nullptr;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevicesSmem) return nullptr;
  unsigned char* slots = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    if (g_tmap_ptr[dev] == nullptr) {
      void* ptr = nullptr;
      if (cudaGetSymbolAddress(&ptr, g_tmap_slots) != cudaSuccess || ptr == nullptr) return nullptr;
      g_tmap_ptr[dev] = static_cast<unsigned char*>(ptr);
    }
    slots = g_tmap_ptr[dev];
  }
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return nullptr;
  slots += (size_t)(g_tmap_call.fetch_add(1) % kTmapRing) * kTmapMaxLayers * 128;
  // Rank 5, innermost first: (64 dims = 128 bytes, token mod 8, half of the head vector, token / 8 inside the block,
  // head slot).  A head slot is one (block, KV head) pair: slots are head_stride apart and a block holds
  // block_stride / head_stride of them, which covers token-major and head-major blocks alike.  The box is 16 tokens
  // of one head, 4 KB; in shared memory it reads [8-token group][half][token mod 8][128 B], i.e. complete 8-row
  // swizzle atoms of the real parts and of the imaginary parts in turn.  (Strides need not ascend.)
  const cuuint64_t slots_per_block = (cuuint64_t)(Y.block_stride / Y.head_stride);
  const cuuint64_t dims[5] = {64, 8, 2, (cuuint64_t)Y.block_size / 8, (cuuint64_t)Y.num_blocks * slots_per_block};
  const cuuint64_t strides[4] = {(cuuint64_t)Y.token_stride * 2, 128, (cuuint64_t)Y.token_stride * 16,
                                 (cuuint64_t)Y.head_stride * 2};
  const cuuint32_t box[5] = {64, 8, 2, 2, 1};
  const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
  TensorMapBytes tmpl;
  static_assert(sizeof(CUtensorMap) == sizeof(TensorMapBytes), "tensor map is 128 bytes");
  // the base address of the template is a placeholder (its own slot: valid device memory, 128-byte aligned)
  if (encode(reinterpret_cast<CUtensorMap*>(&tmpl), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, slots, dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return nullptr;
  if (launch_kernel(stamp_tensor_maps_kernel, dim3(1), dim3((unsigned)((Y.num_layers + 31) / 32 * 32)), 0, st, pdl, tmpl,
                    k_layer_ptrs, slots, (int)Y.num_layers) != TRIATTN_OK)
    return nullptr;
  return slots;
}

// How an internal stage is launched: after the preceding kernel as a programmatic dependent or in plain stream
// order; the scorer can leave the clearing of the moments to whoever ran before it.
struct StageOpts {
  bool pdl = false;
  bool cuda_core_scorer = false;  // the all-fp32 CUDA-core scorer instead of the tensor-core one
  bool moments_cleared = false;   // moments already zero: skip the memset
};

int score_paged_impl(const triattn_paged_layout* layout, const void* const* k_layer_ptrs, const int32_t* block_table,
                     const int32_t* seq_lens, const float* weights, int offset_agg, int num_offsets,
                     float* raw_scores, double* moments, uint32_t* device_status, cudaStream_t st,
                     const StageOpts& opt);
struct ScatterOut {
  float* const* ptrs = nullptr;  // [ranks] device pointers to the ranks' receive buffers
  int rows = 0, rank = 0;        // output rows per rank; this rank
  int shift = 0;                 // first layer this rank visits
};
int finalize_scores_impl(const triattn_paged_layout* layout, const float* raw_scores, const double* moments,
                         const int32_t* seq_lens, const int32_t* prefill_lens, int window, int normalize,
                         int group_reduce, int head_reduce, int layer_reduce, int l_total, bool first_chunk,
                         bool last_chunk, float* scores_out, cudaStream_t st, bool pdl,
                         const ScatterOut& scatter = ScatterOut{});

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
  return score_paged_impl(layout, k_layer_ptrs, block_table, seq_lens, weights, offset_agg, num_offsets, raw_scores,
                          moments, device_status, static_cast<cudaStream_t>(stream), StageOpts{});
}

int triattn_score_paged_cuda_cores(const triattn_paged_layout* layout, const void* const* k_layer_ptrs,
                                   const int32_t* block_table, const int32_t* seq_lens, const float* weights,
                                   int offset_agg, int num_offsets, float* raw_scores, double* moments,
                                   uint32_t* device_status, void* stream) {
  StageOpts opt;
  opt.cuda_core_scorer = true;
  return score_paged_impl(layout, k_layer_ptrs, block_table, seq_lens, weights, offset_agg, num_offsets, raw_scores,
                          moments, device_status, static_cast<cudaStream_t>(stream), opt);
}

int triattn_finalize_scores(const triattn_paged_layout* layout, const float* raw_scores, const double* moments,
                            const int32_t* seq_lens, const int32_t* prefill_lens, int window, int normalize,
                            int group_reduce, int head_reduce, int layer_reduce, float* scores_out, void* stream) {
  if (validate_layout(layout) != TRIATTN_OK) return validate_layout(layout);
  return finalize_scores_impl(layout, raw_scores, moments, seq_lens, prefill_lens, window, normalize, group_reduce,
                              head_reduce, layer_reduce, layout->num_layers, true, true, scores_out,
                              static_cast<cudaStream_t>(stream), false);
}

int triattn_finalize_scores_scatter(const triattn_paged_layout* layout, const float* raw_scores, const double* moments,
                                    const int32_t* seq_lens, const int32_t* prefill_lens, int window, int normalize,
                                    int group_reduce, int head_reduce, float* const* recv_ptrs, int num_ranks, int rank,
                                    void* stream) {
  int rc = validate_layout(layout);
  if (rc != TRIATTN_OK) return rc;
  if (!recv_ptrs || num_ranks <= 0 || rank < 0 || rank >= num_ranks) return TRIATTN_ERR_INVALID_ARGUMENT;
  const long long rows = (long long)layout->num_layers * layout->num_reqs *
                         (head_reduce != TRIATTN_REDUCE_NONE ? 1 : layout->num_kv_heads);
  if (rows % num_ranks != 0) return TRIATTN_ERR_INVALID_ARGUMENT;
  ScatterOut sc;
  sc.ptrs = recv_ptrs;
  sc.rows = (int)(rows / num_ranks);
  sc.rank = rank;
  // start with the layers of the next rank: at any moment the ranks store into different owners
  sc.shift = (int)(((long long)((rank + 1) % num_ranks) * layout->num_layers) / num_ranks);
  return finalize_scores_impl(layout, raw_scores, moments, seq_lens, prefill_lens, window, normalize, group_reduce,
                              head_reduce, TRIATTN_REDUCE_NONE, layout->num_layers, true, true, nullptr,
                              static_cast<cudaStream_t>(stream), false, sc);
}

int triattn_max_over_slots(const float* slots, int num_slots, int64_t elems_per_slot, float* out, void* stream) {
  if (!slots || !out || num_slots <= 0 || elems_per_slot <= 0) return TRIATTN_ERR_INVALID_ARGUMENT;
  if (!aligned16(slots) || !aligned16(out)) return TRIATTN_ERR_MISALIGNED;
  const size_t n = (size_t)elems_per_slot;
  const size_t work = (n & 3) == 0 ? n / 4 : n;
  const unsigned blocks = (unsigned)std::min<size_t>((work + 255) / 256, (size_t)kSMs * 8);
  max_over_slots_kernel<<<std::max(1u, blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(slots, num_slots, n, out);
  return check_launch();
}

static int select_topk_impl(const float* scores, int num_rows, int64_t row_stride, const int32_t* seq_lens,
                            const int32_t* keep_counts, int num_reqs, int rows_per_req_inner, int32_t* keep_out,
                            int keep_pitch, uint32_t* device_status, cudaStream_t st, bool pdl) {
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
  return launch_kernel(select_topk_kernel, dim3((unsigned)num_rows), dim3(kSelectThreads), 0, st, pdl, p);
}

int triattn_select_topk(const float* scores, int num_rows, int64_t row_stride, const int32_t* seq_lens,
                        const int32_t* keep_counts, int num_reqs, int rows_per_req_inner, int32_t* keep_out,
                        int keep_pitch, uint32_t* device_status, void* stream) {
  return select_topk_impl(scores, num_rows, row_stride, seq_lens, keep_counts, num_reqs, rows_per_req_inner, keep_out,
                          keep_pitch, device_status, static_cast<cudaStream_t>(stream), false);
}

static int compact_common(const triattn_paged_layout* layout, void* const* k_layer_ptrs, void* const* v_layer_ptrs,
                          const int32_t* block_table, const int32_t* seq_lens, const int32_t* keep,
                          int64_t keep_ls, int64_t keep_rs, int64_t keep_hs, const int32_t* keep_counts,
                          void* scratch, long long scratch_stream_bytes, int scratch_rows, bool preserve,
                          uint32_t* device_status, void* stream, bool pdl = false) {
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
  const bool small = (long long)grid.x * grid.y * grid.z < kCompactSmallGrid;
  if (preserve) {
    if (small) return launch_kernel(compact_paged_kernel<true, kCompactThreadsSmall>, grid, dim3(kCompactThreadsSmall), 0, st, pdl, p);
    return launch_kernel(compact_paged_kernel<true, kCompactThreads>, grid, dim3(kCompactThreads), 0, st, pdl, p);
  }
  if (small) return launch_kernel(compact_paged_kernel<false, kCompactThreadsSmall>, grid, dim3(kCompactThreadsSmall), 0, st, pdl, p);
  return launch_kernel(compact_paged_kernel<false, kCompactThreads>, grid, dim3(kCompactThreads), 0, st, pdl, p);
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

// ------------------------------------------------------------------------- one-launch weight prep
static int prep_weights_fused_impl(const float* q_mean_real, const float* q_mean_imag, const float* q_abs_mean,
                                   const float* freq_scale_sq, const float* omega, const float* offsets,
                                   const int32_t* round_start, int num_layers, int num_reqs, int num_q_heads,
                                   int num_freqs, int num_offsets, int offset_agg, int flags, float* weights_out,
                                   double* moments_to_clear, cudaStream_t st, bool pdl) {
  if (!q_mean_real || !q_mean_imag || !q_abs_mean || !freq_scale_sq || !omega || !offsets || !round_start || !weights_out)
    return TRIATTN_ERR_INVALID_ARGUMENT;
  if (num_layers <= 0 || num_reqs <= 0 || num_q_heads <= 0 || num_freqs <= 0 || num_offsets <= 0)
    return TRIATTN_ERR_INVALID_ARGUMENT;
  if (num_reqs > 65535) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  const size_t smem = sizeof(float) * (2 * (size_t)num_offsets * num_freqs + 2 * (size_t)num_freqs);
  if (smem > 200 * 1024) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  if (!ensure_dynamic_smem<prep_weights_fused_kernel>(smem)) return TRIATTN_ERR_CUDA;
  PrepFusedParams p{};
  p.q_re = q_mean_real;
  p.q_im = q_mean_imag;
  p.q_abs = q_abs_mean;
  p.fs = freq_scale_sq;
  p.omega = omega;
  p.offsets = offsets;
  p.round_start = round_start;
  p.weights = weights_out;
  p.moments = moments_to_clear;
  p.L = num_layers;
  p.B = num_reqs;
  p.Hq = num_q_heads;
  p.F = num_freqs;
  p.O = num_offsets;
  p.agg_max = offset_agg == TRIATTN_OFFSETS_MAX ? 1 : 0;
  p.flags = flags;
  // Every CTA re-evaluates its request's O x F trig values, so few CTAs per request would be cheapest, but the
  // launch should still fill the GPU: about four CTAs per SM in total, at least 4 rows of weights per CTA.
  const int n_rows = num_layers * num_q_heads;
  const int want_ctas = std::max(1, (4 * kSMs + num_reqs - 1) / num_reqs);
  const int chunks = std::max(1, std::min((n_rows + 3) / 4, want_ctas));
  p.rows_per_cta = (n_rows + chunks - 1) / chunks;
  dim3 grid((unsigned)((n_rows + p.rows_per_cta - 1) / p.rows_per_cta), (unsigned)num_reqs);
  return launch_kernel(prep_weights_fused_kernel, grid, dim3(kPrepThreads), smem, st, pdl, p);
}

int triattn_prep_weights_fused(const float* q_mean_real, const float* q_mean_imag, const float* q_abs_mean,
                               const float* freq_scale_sq, const float* omega, const float* offsets,
                               const int32_t* round_start, int num_layers, int num_reqs, int num_q_heads,
                               int num_freqs, int num_offsets, int offset_agg, int flags, float* weights_out,
                               double* moments_to_clear, void* stream) {
  return prep_weights_fused_impl(q_mean_real, q_mean_imag, q_abs_mean, freq_scale_sq, omega, offsets, round_start,
                                 num_layers, num_reqs, num_q_heads, num_freqs, num_offsets, offset_agg, flags,
                                 weights_out, moments_to_clear, static_cast<cudaStream_t>(stream), false);
}

// ------------------------------------------------------------------------- fused step
namespace {
// Workspace of the fused step: folded weights and moments of all layers, raw scores of ONE chunk of layers,
// the final score rows.  The raw scores dominate (4 * Gp bytes per key); a smaller workspace means fewer layers
// per chunk, down to one.
struct CompressWs {
  size_t weights, moments, final_scores, raw, fixed, raw_per_layer;
};
CompressWs compress_ws_layout(const triattn_paged_layout& Y, int num_offsets, int offset_agg) {
  CompressWs w{};
  const int F = Y.head_dim / 2;
  const int Hq = Y.num_kv_heads * Y.group_size;
  const int gp = std::max(1, triattn_padded_group(Y.group_size));
  const size_t t_pad = (size_t)Y.max_blocks_per_req * Y.block_size;
  size_t off = 0;
  w.weights = off;
  off += round_up(sizeof(float) * (size_t)Y.num_layers * Y.num_reqs * Hq * triattn_weight_rows(offset_agg, num_offsets) * F, 256);
  w.moments = off;
  off += round_up(sizeof(double) * 2 * (size_t)Y.num_layers * Y.num_reqs * Hq, 256);
  w.final_scores = off;
  off += round_up(sizeof(float) * (size_t)Y.num_reqs * Y.num_kv_heads * t_pad, 256);
  w.raw = off;
  w.fixed = off;
  w.raw_per_layer = round_up(sizeof(float) * (size_t)Y.num_reqs * Y.num_kv_heads * t_pad * gp, 256);
  return w;
}
}  // namespace

size_t triattn_compress_workspace_bytes(const triattn_paged_layout* layout, int num_offsets, int offset_agg,
                                        int keep_pitch) {
  (void)keep_pitch;
  if (validate_layout(layout) != TRIATTN_OK || num_offsets <= 0) return 0;
  const CompressWs w = compress_ws_layout(*layout, num_offsets, offset_agg);
  return w.fixed + w.raw_per_layer * (size_t)layout->num_layers;
}

size_t triattn_compress_workspace_bytes_min(const triattn_paged_layout* layout, int num_offsets, int offset_agg,
                                            int keep_pitch) {
  (void)keep_pitch;
  if (validate_layout(layout) != TRIATTN_OK || num_offsets <= 0) return 0;
  const CompressWs w = compress_ws_layout(*layout, num_offsets, offset_agg);
  return w.fixed + w.raw_per_layer;
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
  if (workspace_bytes < w.fixed + w.raw_per_layer) return TRIATTN_ERR_WORKSPACE_TOO_SMALL;
  const int chunk_layers = (int)std::min<size_t>((size_t)Y.num_layers, (workspace_bytes - w.fixed) / w.raw_per_layer);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  float* weights = reinterpret_cast<float*>(ws + w.weights);
  float* raw = reinterpret_cast<float*>(ws + w.raw);
  double* moments = reinterpret_cast<double*>(ws + w.moments);
  float* fin = reinterpret_cast<float*>(ws + w.final_scores);
  const int Hq = Y.num_kv_heads * Y.group_size;
  const int F = Y.head_dim / 2;
  const int64_t t_pad = (int64_t)Y.max_blocks_per_req * Y.block_size;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  // prep (also clears the moments) -> per chunk of layers: score -> finalize into the running rows -> top-k ->
  // compaction.  Score, top-k and compaction are programmatic dependents of the launch before them; finalize is
  // launched normally: with an unbroken chain of programmatic launches from the scorer to the compaction, the
  // compaction ran 5 - 19 % slower on B200 (measured on shapes where it dominates), with any link normal it did not
  // (an SM that never runs empty between the kernels may keep the scorer's large shared-memory carve-out).
  rc = prep_weights_fused_impl(q_mean_real, q_mean_imag, q_abs_mean, freq_scale_sq, omega, offsets, round_start,
                               Y.num_layers, Y.num_reqs, Hq, F, num_offsets, offset_agg, flags, weights, moments, st,
                               false);
  if (rc != TRIATTN_OK) return rc;
  const size_t w_layer = (size_t)Y.num_reqs * Hq * triattn_weight_rows(offset_agg, num_offsets) * F;
  const size_t m_layer = (size_t)Y.num_reqs * Hq * 2;
  StageOpts opt;
  opt.pdl = true;
  opt.moments_cleared = true;
  for (int l0 = 0; l0 < Y.num_layers; l0 += chunk_layers) {
    triattn_paged_layout C = Y;
    C.num_layers = std::min(chunk_layers, Y.num_layers - l0);
    rc = score_paged_impl(&C, reinterpret_cast<const void* const*>(k_layer_ptrs) + l0, block_table, seq_lens,
                          weights + (size_t)l0 * w_layer, offset_agg, num_offsets, raw, moments + (size_t)l0 * m_layer,
                          device_status, st, opt);
    if (rc != TRIATTN_OK) return rc;
    rc = finalize_scores_impl(&C, raw, moments + (size_t)l0 * m_layer, seq_lens, prefill_lens, window, normalize,
                              TRIATTN_REDUCE_MAX, TRIATTN_REDUCE_NONE, layer_reduce, Y.num_layers, l0 == 0,
                              l0 + C.num_layers >= Y.num_layers, fin, st, false);
    if (rc != TRIATTN_OK) return rc;
  }
  rc = select_topk_impl(fin, Y.num_reqs * Y.num_kv_heads, t_pad, seq_lens, keep_counts, Y.num_reqs, Y.num_kv_heads,
                        keep_out, keep_pitch, device_status, st, true);
  if (rc != TRIATTN_OK) return rc;
  return compact_common(layout, k_layer_ptrs, v_layer_ptrs, block_table, seq_lens, keep_out, 0,
                        (int64_t)Y.num_kv_heads * keep_pitch, keep_pitch, keep_counts, nullptr, 0, 0, false,
                        device_status, stream, true);
}

}  // extern "C"

// ------------------------------------------------------------------------- stage implementations
namespace {

int score_paged_impl(const triattn_paged_layout* layout, const void* const* k_layer_ptrs, const int32_t* block_table,
                     const int32_t* seq_lens, const float* weights, int offset_agg, int num_offsets,
                     float* raw_scores, double* moments, uint32_t* device_status, cudaStream_t st,
                     const StageOpts& opt) {
  int rc = validate_layout(layout);
  if (rc != TRIATTN_OK) return rc;
  if (!k_layer_ptrs || !block_table || !seq_lens || !weights || !raw_scores || !moments)
    return TRIATTN_ERR_INVALID_ARGUMENT;
  const triattn_paged_layout& Y = *layout;
  const int gp = triattn_padded_group(Y.group_size);
  if (gp == 0) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  const int Hq = Y.num_kv_heads * Y.group_size;
  if (!opt.moments_cleared &&
      cudaMemsetAsync(moments, 0, sizeof(double) * 2 * (size_t)Y.num_layers * Y.num_reqs * Hq, st) != cudaSuccess)
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
  // Streaming kernels: mean aggregation, head_dim 64/128, K region of a block one dense run.
  const bool streamable = !p.agg_max && (Y.head_dim == 64 || Y.head_dim == 128) && block_is_dense(layout) &&
                          block_bytes <= 64 * 1024 && (block_bytes % 16) == 0 && (p.block_stride_bytes % 16) == 0;
  if (streamable) {
    // cache blocks per pipeline stage: a power of two filling ~32 KB (8 work items of 16 keys for 8 KV heads)
    int mb = 1;
    while ((mb * 2) * block_bytes <= 32 * 1024) mb *= 2;
    const long long stage_bytes = (long long)mb * block_bytes;
    // two CTAs per SM share ~200 KB of shared memory
    int stages = (int)std::min<long long>(4, (100 * 1024) / stage_bytes);
    if (stages < 2) stages = 2;
    p.block_bytes = (int)block_bytes;
    p.mb = mb;
    p.stages = stages;
    p.block_group = (gp <= 8 && Y.block_size == 16 && Y.num_kv_heads * mb == kScoreConsumerWarps && !opt.cuda_core_scorer)
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
    p.tiles_per_cta = tpc;
    dim3 grid((unsigned)((max_tiles + tpc - 1) / tpc), (unsigned)Y.num_layers, (unsigned)Y.num_reqs);
    const size_t smem = (size_t)stages * stage_bytes;
    if (opt.cuda_core_scorer) {
      // the CUDA-core kernel works on batches of 16/gpv tokens and keeps a table of work items per stage
      const int gpv = std::min(gp, 4), nsub = gp / gpv, nt = kLPK / gpv;
      const long long stage_tok = (long long)mb * Y.block_size;
      const long long n_items = nhd ? (long long)Y.num_kv_heads * nsub * (stage_tok / nt)
                                    : (long long)mb * Y.num_kv_heads * nsub * (Y.block_size / nt);
      const bool ok = (nhd ? (stage_tok % nt) == 0 : (Y.block_size % nt) == 0) && n_items > 0 && n_items <= kMaxScoreItems;
      if (!ok) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
      if (Y.head_dim == 128)
        return Y.rope_interleaved ? launch_score_fma<128, true>(p, gpv, grid, smem, st, opt.pdl)
                                  : launch_score_fma<128, false>(p, gpv, grid, smem, st, opt.pdl);
      return Y.rope_interleaved ? launch_score_fma<64, true>(p, gpv, grid, smem, st, opt.pdl)
                                : launch_score_fma<64, false>(p, gpv, grid, smem, st, opt.pdl);
    }
    if (Y.head_dim == 128)
      return Y.rope_interleaved ? launch_score_mma<128, true>(p, grid, smem, st, opt.pdl)
                                : launch_score_mma<128, false>(p, grid, smem, st, opt.pdl);
    return Y.rope_interleaved ? launch_score_mma<64, true>(p, grid, smem, st, opt.pdl)
                              : launch_score_mma<64, false>(p, grid, smem, st, opt.pdl);
  }
  if (opt.cuda_core_scorer) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  // max over offsets, head_dim 128: tcgen05 kernel, one CTA per (layer, request, virtual head, run of 128-key tiles)
  if (p.agg_max && Y.head_dim == 128 && num_offsets >= 1 && 2 * umma_max_cols(num_offsets) <= kUmmaMaxN &&
      umma_max_smem_bytes(umma_max_cols(num_offsets)) <= 220 * 1024 && (Y.block_size % 16) == 0 &&
      Y.num_layers <= kTmapMaxLayers && (p.block_stride_bytes % 16) == 0 && (Y.token_stride % 8) == 0 &&
      (Y.head_stride % 8) == 0 && Y.head_stride > 0 && (Y.block_stride % Y.head_stride) == 0 &&
      (long long)Y.num_blocks * (Y.block_stride / Y.head_stride) < (1ll << 31)) {
    const int n_cols = umma_max_cols(num_offsets);
    const int nvh = Y.num_kv_heads * ((gp + 3) / 4);
    const int n_tiles = (p.t_pad + kUmmaTileKeys - 1) / kUmmaTileKeys;
    // a CTA keeps the block ids of its keys in shared memory; 128 tiles (16384 keys) amortise the weight set-up
    const int fit = (int)std::max<long long>(1, ((long long)(kUmmaMaxBlocks - 1) * Y.block_size) / kUmmaTileKeys);
    p.tiles_per_cta = std::min(n_tiles, std::min(128, fit));
    const int chunks = (n_tiles + p.tiles_per_cta - 1) / p.tiles_per_cta;
    dim3 grid((unsigned)(nvh * chunks), (unsigned)Y.num_layers, (unsigned)Y.num_reqs);
    const size_t smem = umma_max_smem_bytes(n_cols);
    // the layers' tensor maps are stamped by a one-warp kernel in front of the scorer (its programmatic dependent)
    p.tmap_slots_per_block = (int)(Y.block_stride / Y.head_stride);
    p.tmaps = stamp_layer_tensor_maps(Y, k_layer_ptrs, st, opt.pdl);
    if (p.tmaps == nullptr) return TRIATTN_ERR_CUDA;
    if (Y.rope_interleaved) {
      if (!ensure_dynamic_smem<score_paged_umma_max_kernel<true>>(smem)) return TRIATTN_ERR_CUDA;
      return launch_kernel(score_paged_umma_max_kernel<true>, grid, dim3(kUmmaThreads), smem, st, true, p);
    }
    if (!ensure_dynamic_smem<score_paged_umma_max_kernel<false>>(smem)) return TRIATTN_ERR_CUDA;
    return launch_kernel(score_paged_umma_max_kernel<false>, grid, dim3(kUmmaThreads), smem, st, true, p);
  }
  // max over offsets on mma.sync (head_dim 64): one CTA per (layer, request, virtual head, run of 16-key tiles)
  if (p.agg_max && (Y.head_dim == 64 || Y.head_dim == 128) && (p.block_stride_bytes % 16) == 0 &&
      max_agg_smem_bytes(Y.head_dim, num_offsets) <= 220 * 1024) {
    const int nvh = Y.num_kv_heads * ((gp + 3) / 4);
    const int n_tiles = (p.t_pad + kMmaKeys - 1) / kMmaKeys;
    p.tiles_per_cta = std::min(n_tiles, 16 * kMaxAggWarps);
    const int chunks = (n_tiles + p.tiles_per_cta - 1) / p.tiles_per_cta;
    dim3 grid((unsigned)(nvh * chunks), (unsigned)Y.num_layers, (unsigned)Y.num_reqs);
    const size_t smem = max_agg_smem_bytes(Y.head_dim, num_offsets);
#define TRIATTN_LAUNCH(D, IL)                                                                      \
  {                                                                                                \
    if (!ensure_dynamic_smem<score_paged_mma_max_kernel<D, IL>>(smem)) return TRIATTN_ERR_CUDA;    \
    return launch_kernel(score_paged_mma_max_kernel<D, IL>, grid, dim3(kMaxAggThreads), smem, st, opt.pdl, p); \
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
  return launch_kernel(score_paged_generic_kernel, grid, dim3(128), 0, st, opt.pdl, p, (int)Y.head_dim,
                       (int)Y.rope_interleaved);
}

int finalize_scores_impl(const triattn_paged_layout* layout, const float* raw_scores, const double* moments,
                         const int32_t* seq_lens, const int32_t* prefill_lens, int window, int normalize,
                         int group_reduce, int head_reduce, int layer_reduce, int l_total, bool first_chunk,
                         bool last_chunk, float* scores_out, cudaStream_t st, bool pdl, const ScatterOut& scatter) {
  if (!raw_scores || !moments || !seq_lens || (!scores_out && !scatter.ptrs)) return TRIATTN_ERR_INVALID_ARGUMENT;
  if (scatter.ptrs && (layer_reduce != TRIATTN_REDUCE_NONE || scatter.rows <= 0 || scatter.rank < 0))
    return TRIATTN_ERR_INVALID_ARGUMENT;
  if (group_reduce != TRIATTN_REDUCE_MAX && group_reduce != TRIATTN_REDUCE_MEAN) return TRIATTN_ERR_INVALID_ARGUMENT;
  if (head_reduce != TRIATTN_REDUCE_NONE && head_reduce != TRIATTN_REDUCE_MAX) return TRIATTN_ERR_INVALID_ARGUMENT;
  if (layer_reduce < TRIATTN_REDUCE_NONE || layer_reduce > TRIATTN_REDUCE_MAX) return TRIATTN_ERR_INVALID_ARGUMENT;
  const triattn_paged_layout& Y = *layout;
  const int gp = triattn_padded_group(Y.group_size);
  if (gp == 0) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  const int t_pad = Y.max_blocks_per_req * Y.block_size;
  FinalizeParams p{};
  p.raw = raw_scores;
  p.moments = moments;
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
  p.l_total = l_total;
  p.first_chunk = first_chunk ? 1 : 0;
  p.last_chunk = last_chunk ? 1 : 0;
  p.gp = gp;
  p.scatter_out = scatter.ptrs;
  p.scatter_rows = scatter.rows;
  p.scatter_rank = scatter.rank;
  p.scatter_shift = scatter.shift;
  const int Ho = head_reduce != TRIATTN_REDUCE_NONE ? 1 : Y.num_kv_heads;
  dim3 grid((unsigned)((t_pad + 255) / 256), (unsigned)Ho, (unsigned)Y.num_reqs);
  // (mean, 1/std) of the rows a CTA normalises with live in its shared memory
  const size_t heads_per_cta = (size_t)(head_reduce != TRIATTN_REDUCE_NONE ? Y.num_kv_heads : 1) * Y.group_size;
  const size_t smem = sizeof(float2) * (size_t)Y.num_layers * heads_per_cta;
  if (smem > 200 * 1024) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
  if (head_reduce == TRIATTN_REDUCE_NONE && Y.group_size <= 8 && (gp == 4 || gp == 8)) {
#define TRIATTN_FIN_LR(G, LR)                                                                         \
  {                                                                                                   \
    if (!ensure_dynamic_smem<finalize_scores_fast_kernel<G, LR>>(smem)) return TRIATTN_ERR_CUDA;      \
    return launch_kernel(finalize_scores_fast_kernel<G, LR>, grid, dim3(256), smem, st, pdl, p);      \
  }
#define TRIATTN_FIN(G)                                                                                \
  case G:                                                                                             \
    if (layer_reduce == TRIATTN_REDUCE_NONE) TRIATTN_FIN_LR(G, TRIATTN_REDUCE_NONE)                   \
    if (layer_reduce == TRIATTN_REDUCE_MAX) TRIATTN_FIN_LR(G, TRIATTN_REDUCE_MAX)                     \
    TRIATTN_FIN_LR(G, TRIATTN_REDUCE_MEAN)
    switch (Y.group_size) {
      TRIATTN_FIN(3) TRIATTN_FIN(4) TRIATTN_FIN(5) TRIATTN_FIN(6) TRIATTN_FIN(7) TRIATTN_FIN(8)
      default: break;
    }
#undef TRIATTN_FIN
#undef TRIATTN_FIN_LR
  }
  // general kernel: without a layer reduction every layer is its own output row, so the layers go into the grid
  // (one layer per CTA: more loads in flight than a per-thread loop over the layers, and less shared memory)
  size_t smem_gen = smem;
  if (layer_reduce == TRIATTN_REDUCE_NONE) {
    if ((long long)Ho * Y.num_layers > 65535) return TRIATTN_ERR_UNSUPPORTED_SHAPE;
    grid.y = (unsigned)(Ho * Y.num_layers);
    smem_gen = sizeof(float2) * heads_per_cta;
  }
  if (!ensure_dynamic_smem<finalize_scores_kernel>(smem_gen)) return TRIATTN_ERR_CUDA;
  return launch_kernel(finalize_scores_kernel, grid, dim3(256), smem_gen, st, pdl, p);
}

}  // namespace
