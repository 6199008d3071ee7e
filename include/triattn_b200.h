/*
 * triattn_b200.h - C ABI of libtriattn_b200.so: TriAttention runtime KV compression
 * (score -> select -> compact on a paged bf16 KV cache) for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its comment says "host";
 *   - every function enqueues work on `stream` (a cudaStream_t passed as void*) and
 *     returns without synchronising; it allocates nothing and frees nothing;
 *   - the return value is a triattn_status; kernels never trap: bad metadata seen on
 *     the device (block id out of range, keep index out of range, a bounded wait that
 *     ran out) sets bits in the caller's `device_status` word (may be NULL) and the
 *     offending element is skipped;
 *   - strides are in ELEMENTS (bf16) unless named *_bytes.
 *
 * Each entry point names the function of the reference implementation
 * (WeianMao/triattention, paths relative to that project) whose work it replaces.
 */
#ifndef TRIATTN_B200_H
#define TRIATTN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRIATTN_ABI_VERSION 2

typedef enum triattn_status {
  TRIATTN_OK = 0,
  TRIATTN_ERR_INVALID_ARGUMENT = 1,   /* NULL pointer, non-positive size, inconsistent sizes      */
  TRIATTN_ERR_UNSUPPORTED_SHAPE = 2,  /* head_dim / group size / block geometry outside the build */
  TRIATTN_ERR_MISALIGNED = 3,         /* base pointer or stride breaks the 16-byte copy rule      */
  TRIATTN_ERR_WORKSPACE_TOO_SMALL = 4,
  TRIATTN_ERR_CUDA = 5,               /* a CUDA runtime call or launch failed                     */
  TRIATTN_ERR_LIMIT_EXCEEDED = 6      /* size beyond a fixed maximum of a no-allocation entry     */
} triattn_status;

/* bits of the device status word */
#define TRIATTN_DEV_BAD_BLOCK_ID   0x1u  /* block_table entry outside [0, num_blocks)          */
#define TRIATTN_DEV_BAD_KEEP_INDEX 0x2u  /* keep index outside [0, seq_len) or not ascending   */
#define TRIATTN_DEV_WAIT_TIMEOUT   0x4u  /* a bounded wait on an async copy ran out            */
#define TRIATTN_DEV_BAD_LENGTH     0x8u  /* seq_len exceeds the request's block-table capacity */

typedef enum triattn_offset_agg { TRIATTN_OFFSETS_MEAN = 0, TRIATTN_OFFSETS_MAX = 1 } triattn_offset_agg;
typedef enum triattn_reduce { TRIATTN_REDUCE_NONE = 0, TRIATTN_REDUCE_MEAN = 1, TRIATTN_REDUCE_MAX = 2 } triattn_reduce;

#define TRIATTN_FLAG_DISABLE_MLR  0x1  /* magnitude coefficient = q_abs_mean (scoring.py:346-348) */
#define TRIATTN_FLAG_DISABLE_TRIG 0x2  /* drop the trigonometric series (scoring.py:321-329)      */

/*
 * Geometry of one worker's paged KV cache as the kernels see it.  One K (and one V)
 * base pointer per layer; inside a layer, element (block, token, head, d) lives at
 * block*block_stride + token*token_stride + head*head_stride + d.  Covers vLLM's
 * [2, nb, bs, H, D] and [nb, 2, bs, H, D] tensors in NHD or HND stride order
 * (kv_compaction.py:94-117 _split_kv_axes).  The K region of a block must be one dense
 * run of block_size*num_kv_heads*head_dim elements.
 */
typedef struct triattn_paged_layout {
  int32_t num_layers;          /* L: layers sharing the block table (one KV-cache group)    */
  int32_t num_reqs;            /* B: requests compressed by this call                      */
  int32_t num_kv_heads;        /* Hkv on this rank                                          */
  int32_t group_size;          /* g: statistic (query) heads per KV head                    */
  int32_t head_dim;            /* D (64 or 128 for the fast scorer)                         */
  int32_t block_size;          /* tokens per cache block                                    */
  int32_t num_blocks;          /* blocks in the cache (bound for block_table entries)       */
  int32_t max_blocks_per_req;  /* row pitch of block_table                                  */
  int64_t block_stride;
  int64_t token_stride;
  int64_t head_stride;
  int32_t rope_interleaved;    /* 0: [r0..,i0..] "half" layout, 1: [r0,i0,r1,i1,..]         */
  int32_t reserved;
} triattn_paged_layout;

/* ABI version of the loaded library (== TRIATTN_ABI_VERSION it was built with). */
int triattn_abi_version(void);

/* Static, human-readable text for a triattn_status. */
const char* triattn_status_string(int status);

/* Query-head slots per KV head in the raw-score layout: group_size rounded up to 1, 2 or 4, and
 * above 4 to the next multiple of 4 (the scorers split such groups into virtual heads), up to 64.
 * Returns 0 for group_size <= 0 or > 64. */
int triattn_padded_group(int group_size);

/* Number of weight rows per (layer, request, query head): 3 for MEAN (w_re, w_im, w_mag),
 * 2*num_offsets + 1 for MAX. */
int triattn_weight_rows(int offset_agg, int num_offsets);

/* Floats of scratch triattn_prep_weights needs. */
size_t triattn_prep_scratch_floats(int num_reqs, int num_freqs, int num_offsets, int offset_agg);

/*
 * Fold the calibrated query statistics and the future-offset phases of each request into
 * per-(layer, request, query head) weight rows, so that a key's score is a dot product:
 *   MEAN: s = sum_f k_re*w_re + k_im*w_im + |k|*w_mag, with
 *         w_re = fs*(q_re*C - q_im*S), w_im = fs*(q_im*C + q_re*S), C/S = mean over offsets of
 *         cos/sin(fl32(round_start+offset)*omega_f), w_mag = (q_abs - sqrt(q_re^2+q_im^2+1e-8))*fs;
 *   MAX : one (w_re, w_im) row pair per offset and one w_mag row.
 * Replaces the per-call statistics handling of compute_scores_pytorch
 * (triattention/vllm/core/scoring.py:258-271, :313-332, :346-356) and the trig tables of
 * triattention/vllm/core/kernels/triton_scoring.py:38-122.
 *   q_mean_real/q_mean_imag/q_abs_mean/freq_scale_sq : [L, Hq, F] fp32
 *   omega [F], offsets [num_offsets] fp32; round_start [B] int32
 *   weights_out : [L, B, Hq, triattn_weight_rows(), F] fp32
 */
int triattn_prep_weights(const float* q_mean_real, const float* q_mean_imag, const float* q_abs_mean,
                         const float* freq_scale_sq, const float* omega, const float* offsets,
                         const int32_t* round_start, int num_layers, int num_reqs, int num_q_heads,
                         int num_freqs, int num_offsets, int offset_agg, int flags,
                         float* scratch, float* weights_out, void* stream);

/*
 * triattn_prep_weights in ONE launch and without scratch: each CTA evaluates the offset phases of its request
 * into shared memory (the O x F double-precision sincos calls run in parallel) and folds a slice of the
 * (layer, query head) rows.  weights_out is bit-identical to triattn_prep_weights.  If moments_to_clear is not
 * NULL, the [L, B, Hq, 2] fp64 array it names is zeroed by the same launch (the scorer accumulates into it).
 * Replaces the same reference code as triattn_prep_weights (scoring.py:258-271, :313-332, :346-356).
 */
int triattn_prep_weights_fused(const float* q_mean_real, const float* q_mean_imag, const float* q_abs_mean,
                               const float* freq_scale_sq, const float* omega, const float* offsets,
                               const int32_t* round_start, int num_layers, int num_reqs, int num_q_heads,
                               int num_freqs, int num_offsets, int offset_agg, int flags, float* weights_out,
                               double* moments_to_clear, void* stream);

/* Capacity, in floats, of the built-in scratch of triattn_prep_weights_noalloc (256 KiB). */
#define TRIATTN_NOALLOC_PREP_SCRATCH_FLOATS 65536

/*
 * triattn_prep_weights for callers that must not allocate device memory.  (No counterpart in the
 * reference: its scorer allocates torch temporaries on every call.)
 *
 * Who needs it: a serving worker that has already handed every free byte of HBM to its KV-cache
 * pool, so a late cudaMalloc can fail or fragment the pool; and a hook that runs inside the
 * engine's step loop, where cudaMalloc / cudaFree synchronise the whole device and would stall the
 * other streams.  Such callers still pass their own inputs and `weights_out`; only the trig-table
 * scratch (triattn_prep_scratch_floats() floats) is taken from an array that lives inside the
 * library image.  Every GPU that loads the library holds those 256 KiB until the process exits.
 *
 * Limits and rules:
 *   - triattn_prep_scratch_floats(num_reqs, num_freqs, num_offsets, offset_agg) must not exceed
 *     TRIATTN_NOALLOC_PREP_SCRATCH_FLOATS (MEAN, 64 frequencies: up to 512 requests per call; MAX with
 *     17 offsets: up to 30); larger requests return TRIATTN_ERR_LIMIT_EXCEEDED and launch nothing;
 *   - the first call on a device looks up the array's device address (once per device, with that
 *     device current); make that first call before starting any stream capture;
 *   - all calls share the one array, which keeps the previous call's contents.  Nothing in it has
 *     to start at zero - each call overwrites every entry it later reads - but two calls whose
 *     kernels can overlap on the GPU (different streams, no ordering between them) race on it:
 *     order them on one stream or with events;
 *   - calls no cudaMalloc, cudaFree or allocating library routine.
 * Arguments and results are those of triattn_prep_weights without `scratch`.
 */
int triattn_prep_weights_noalloc(const float* q_mean_real, const float* q_mean_imag, const float* q_abs_mean,
                                 const float* freq_scale_sq, const float* omega, const float* offsets,
                                 const int32_t* round_start, int num_layers, int num_reqs, int num_q_heads,
                                 int num_freqs, int num_offsets, int offset_agg, int flags,
                                 float* weights_out, void* stream);

/*
 * Score every cached key of every (layer, request, KV head) against the g query heads of its
 * group: streams each cache block once with bulk async copies into shared memory and writes
 *   raw_scores [L, B, Hkv, t_pad, Gp] fp32 (Gp = triattn_padded_group(g); slot q of token t is
 *              query head kvh*g + q; t_pad = max_blocks_per_req*block_size)
 *   moments    [L, B, Hkv*g, 2] fp64: sum and sum of squares over the request's tokens
 *              (zeroed by this call).
 * Replaces gather_request_k_dense_range (triattention/vllm/runtime/kv_compaction.py:322-352),
 * the repeat_interleave expansion and scorer call (triattention/vllm/runtime/selector_hf.py:299-328),
 * the Triton kernels (triattention/vllm/core/kernels/triton_scoring.py:160-490) and the moment
 * accumulation (selector_hf.py:884-894).
 *   k_layer_ptrs : [L] device array of per-layer K base pointers (bf16)
 *   block_table  : [B, max_blocks_per_req] int32; seq_lens : [B] int32
 *   weights      : output of triattn_prep_weights with the same offset_agg / num_offsets
 * TRIATTN_OFFSETS_MAX with head_dim 128, a block size that is a multiple of 16, at most 128 layers and
 * block_stride a multiple of head_stride runs on the tcgen05 tensor cores: the call then also launches a
 * one-warp kernel that writes one 128-byte TMA tensor map per layer into a ring inside the library image
 * (8 calls deep per device, no allocation).  Calls on one stream are ordered and may be issued without limit;
 * more than 8 such calls in flight on DIFFERENT streams of one device must be serialised by the caller.
 */
int triattn_score_paged(const triattn_paged_layout* layout /* host */, const void* const* k_layer_ptrs,
                        const int32_t* block_table, const int32_t* seq_lens, const float* weights,
                        int offset_agg, int num_offsets, float* raw_scores, double* moments,
                        uint32_t* device_status, void* stream);

/*
 * triattn_score_paged on the CUDA cores only: every product is an fp32 FMA (fma.rn.f32x2), no operand is split
 * into bf16 parts.  Same arguments, same outputs.  It exists as the all-fp32 cross-check of the tensor-core
 * scorer's error budget (the parity tests run both) and covers mean aggregation with head_dim 64/128 on dense
 * blocks; other shapes return TRIATTN_ERR_UNSUPPORTED_SHAPE.  Replaces the same reference code as
 * triattn_score_paged.
 */
int triattn_score_paged_cuda_cores(const triattn_paged_layout* layout /* host */, const void* const* k_layer_ptrs,
                                   const int32_t* block_table, const int32_t* seq_lens, const float* weights,
                                   int offset_agg, int num_offsets, float* raw_scores, double* moments,
                                   uint32_t* device_status, void* stream);

/*
 * Turn raw scores into the scores the top-k runs on: z-normalise per (layer, query head) with the
 * unbiased streaming variance (sigma < 1e-8 -> 1), force +inf on the last `window` tokens and on
 * tokens < prefill_lens[b] (prefill_lens may be NULL), reduce the g query heads of each KV head
 * (group_reduce: MAX or MEAN), optionally the KV heads (head_reduce: NONE or MAX) and the layers
 * (layer_reduce: NONE, MEAN, MAX).
 *   scores_out : [Lo, B, Ho, t_pad] fp32, Lo = 1 if layer_reduce != NONE else L,
 *                Ho = 1 if head_reduce != NONE else Hkv.
 * Replaces selector_hf.py:896-913 (mean/std), :916-989 (normalise, guards, group max, layer mean)
 * and, with layer_reduce NONE, the per-layer path :584-602 / :636-637.
 */
int triattn_finalize_scores(const triattn_paged_layout* layout /* host */, const float* raw_scores,
                            const double* moments, const int32_t* seq_lens, const int32_t* prefill_lens,
                            int window, int normalize, int group_reduce, int head_reduce, int layer_reduce,
                            float* scores_out, void* stream);

/*
 * triattn_finalize_scores with layer_reduce NONE for tensor-parallel layer-shared selection, exchange included:
 * the L*B*Ho output rows are dealt to the ranks in runs of rows/num_ranks, and every row is stored straight into
 * the receive buffer of the rank that owns it - recv_ptrs[owner], a device array of num_ranks pointers, each to
 * a [num_ranks, rows/num_ranks, t_pad] fp32 buffer (peer memory reachable from this device; the own buffer
 * included) - at slot [rank][row % (rows/num_ranks)], by plain stores.  After a barrier across the ranks each
 * owner holds everybody's values of its rows; triattn_max_over_slots folds them.  rows must divide by num_ranks.
 * Replaces the all-reduce / reduce-scatter of score rows a layer-shared step would otherwise need
 * (the reference runs this mode on one device: selector_hf.py:636-667).
 */
int triattn_finalize_scores_scatter(const triattn_paged_layout* layout /* host */, const float* raw_scores,
                                    const double* moments, const int32_t* seq_lens, const int32_t* prefill_lens,
                                    int window, int normalize, int group_reduce, int head_reduce,
                                    float* const* recv_ptrs /* device array */, int num_ranks, int rank, void* stream);

/* out[i] = max over s < num_slots of slots[s * elems_per_slot + i]; both pointers 16-byte aligned. */
int triattn_max_over_slots(const float* slots, int num_slots, int64_t elems_per_slot, float* out, void* stream);

/*
 * Per-row top-k with deterministic lowest-index tie-break; indices come out ascending.
 * Row r belongs to request b = (r / rows_per_req_inner) % num_reqs, has seq_lens[b] valid scores and
 * keeps keep_counts[b] of them (clamped to the row length).
 *   scores : [num_rows, row_stride] fp32;  keep_out : [num_rows, keep_pitch] int32 (tail filled with -1)
 * A seq_lens[b] larger than row_stride is clamped to it and raises TRIATTN_DEV_BAD_LENGTH.
 * Replaces the chunked torch.topk / merge / torch.sort of selector_hf.py:990-1025 (and :604-677, :721-747).
 */
int triattn_select_topk(const float* scores, int num_rows, int64_t row_stride, const int32_t* seq_lens,
                        const int32_t* keep_counts, int num_reqs, int rows_per_req_inner,
                        int32_t* keep_out, int keep_pitch, uint32_t* device_status, void* stream);

/*
 * In-place compaction of K and V: for every (layer, request, KV head) move token keep[r] to slot r,
 * r < keep_counts[b], inside the request's own blocks.  The keep rows must be strictly ascending.
 * Row used for (layer l, request b, head h) is keep + l*keep_layer_stride + b*keep_req_stride +
 * h*keep_head_stride (a stride of 0 shares the row: 0 layer stride = one keep set for all layers,
 * 0 head stride = the "shared" mode).  Slots >= keep_counts[b] are left untouched.
 * Replaces compact_request_kv_in_place_per_head (triattention/vllm/runtime/kv_compaction.py:461-599)
 * and compact_request_kv_in_place (:355-458) for the kept prefix.
 */
int triattn_compact_paged(const triattn_paged_layout* layout /* host */, void* const* k_layer_ptrs,
                          void* const* v_layer_ptrs, const int32_t* block_table, const int32_t* seq_lens,
                          const int32_t* keep, int64_t keep_layer_stride, int64_t keep_req_stride,
                          int64_t keep_head_stride, const int32_t* keep_counts, uint32_t* device_status,
                          void* stream);

/* Bytes of scratch triattn_compact_paged_preserve needs when no request drops more than
 * max_dropped_rows = max_b (seq_lens[b] - keep_counts[b]) tokens. */
size_t triattn_compact_preserve_scratch_bytes(const triattn_paged_layout* layout /* host */, int max_dropped_rows);

/*
 * Same as triattn_compact_paged but additionally writes the dropped tokens, in ascending order,
 * to slots keep_counts[b] .. seq_lens[b]-1, i.e. the full [kept..., dropped...] permutation of
 * kv_compaction.py:518-546 (preserve_dropped_tokens=True).  Uses `scratch` to stage dropped rows.
 */
int triattn_compact_paged_preserve(const triattn_paged_layout* layout /* host */, void* const* k_layer_ptrs,
                                   void* const* v_layer_ptrs, const int32_t* block_table,
                                   const int32_t* seq_lens, const int32_t* keep, int64_t keep_layer_stride,
                                   int64_t keep_req_stride, int64_t keep_head_stride,
                                   const int32_t* keep_counts, int max_dropped_rows, void* scratch,
                                   size_t scratch_bytes, uint32_t* device_status, void* stream);

/*
 * Block-table rewrite after compaction, on the device and for all requests of a step at once:
 * request b keeps the first ceil(lens_after[b] / block_size) entries of its block_table row
 * (blocks_after[b], never more than blocks_before[b]); the removed tail entries are appended to
 * freed_ids in request order, then row order, and overwritten with fill_value.  *freed_count
 * receives the number of removed blocks; if it exceeds freed_capacity the list is truncated and
 * TRIATTN_DEV_BAD_LENGTH is raised in *device_status.
 * Replaces truncate_tail_reclaim_group (triattention/vllm/runtime/layout_engine.py:209-227) and the
 * num_blocks_per_row shrink of apply_worker_block_reclaim_events
 * (triattention/vllm/runtime/worker_reclaim_sync.py:95-112) for engines that keep block tables on the device.
 */
int triattn_rewrite_block_tables(int32_t* block_table, int num_reqs, int max_blocks_per_req, int block_size,
                                 const int32_t* blocks_before, const int32_t* lens_after, int32_t* blocks_after,
                                 int32_t* freed_ids, int freed_capacity, int32_t* freed_count, int32_t fill_value,
                                 uint32_t* device_status, void* stream);

/*
 * Effective-length overrides for the step after a compaction, one launch for the whole batch:
 *   seq_lens[r]      = effective_base[idx_mapping[r]] + (query_start_loc[r+1] - query_start_loc[r])
 *                      for every batch entry r whose row has effective_base >= 0 (others untouched);
 *   positions_out[i] = positions[i] + pos_delta[idx_mapping[r]] for the tokens i of entry r
 *                      (tokens outside every segment are copied).
 * effective_base / pos_delta are dense int32 arrays over request-state rows (null = absent);
 * seq_lens or positions may be null.  counters[4] (device, zeroed by the call) receives: rows with a
 * base override, rows with a non-zero delta, 1 if query_start_loc decreases somewhere, 1 if a
 * segment leaves [0, num_tokens].  apply = 0 only fills the counters.
 * Replaces overwrite_seq_lens_from_effective_lengths / overwrite_seq_lens_from_effective_base_map /
 * shift_positions_from_sparse_deltas (triattention/vllm/runtime/input_patch_ops.py:66-215).
 */
int triattn_apply_effective_overrides(const int32_t* idx_mapping, const int32_t* query_start_loc, int num_reqs,
                                      const int32_t* effective_base, const int32_t* pos_delta, int num_rows,
                                      int32_t* seq_lens, const int64_t* positions, int64_t* positions_out,
                                      int num_tokens, int32_t* counters, int apply, void* stream);

/* Bytes of workspace with which triattn_compress_paged scores all layers in one launch (the raw scores of
 * every layer, 4 * triattn_padded_group(g) bytes per key, dominate it). */
size_t triattn_compress_workspace_bytes(const triattn_paged_layout* layout /* host */, int num_offsets,
                                        int offset_agg, int keep_pitch);

/* Smallest workspace triattn_compress_paged accepts: raw scores of ONE layer at a time.  Any size between this
 * and triattn_compress_workspace_bytes() works; the step is then cut into chunks of as many layers as fit, each
 * scored and folded into the running per-KV-head rows before the next (results are bit-identical). */
size_t triattn_compress_workspace_bytes_min(const triattn_paged_layout* layout /* host */, int num_offsets,
                                            int offset_agg, int keep_pitch);

/*
 * The whole default-mode step for a batch of requests in one call and no host synchronisation:
 * prep -> score -> finalize (z-norm, window/prefill guards, group max, layer mean) -> per-KV-head
 * top-k -> in-place compaction of every layer with the shared keep set.
 * keep_out [B, Hkv, keep_pitch] int32 receives the ascending keep indices.
 * workspace_bytes selects how many layers are scored per launch (see triattn_compress_workspace_bytes_min).
 * The score, top-k and compaction launches are programmatic dependents of their predecessors (each kernel
 * starts with griddepcontrol.wait), so the tail of one kernel overlaps the launch of the next.
 * Replaces, for all requests of a step at once, select_keep_indices_for_group
 * (selector_hf.py:749-1033) followed by execute_group_compaction's per-layer calls
 * (triattention/vllm/runtime/layout_engine.py:112-139).
 */
int triattn_compress_paged(const triattn_paged_layout* layout /* host */, void* const* k_layer_ptrs,
                           void* const* v_layer_ptrs, const int32_t* block_table, const int32_t* seq_lens,
                           const int32_t* round_start, const int32_t* prefill_lens,
                           const int32_t* keep_counts, const float* q_mean_real, const float* q_mean_imag,
                           const float* q_abs_mean, const float* freq_scale_sq, const float* omega,
                           const float* offsets, int num_offsets, int offset_agg, int flags, int window,
                           int normalize, int layer_reduce, void* workspace, size_t workspace_bytes,
                           int32_t* keep_out, int keep_pitch, uint32_t* device_status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TRIATTN_B200_H */
