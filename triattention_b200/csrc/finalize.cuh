// Score finalisation: moments -> (mean, std), z-normalisation, window / prefill guards, reduction
// over the query heads of a KV head, over KV heads (optional) and over layers (optional).
#pragma once

#include "common.cuh"

namespace triattn {

// (mean, 1/std_safe) of one (layer, request, query head) row from its (sum, sum of squares): mean = S1/n,
// var = (S2 - n*mean^2)/(n-1) clamped at 0, std < 1e-8 -> 1 (the streaming formula of the reference selector,
// selector_hf.py:896-913), evaluated in double; the finalize kernels multiply by the reciprocal.
__device__ __forceinline__ float2 mean_rstd_from_moments(const double* __restrict__ m, int n) {
  const double s1 = m[0], s2 = m[1];
  double mean = 0.0, var = 0.0;
  if (n > 0) mean = s1 / (double)n;
  if (n > 1) var = (s2 - (double)n * mean * mean) / (double)(n - 1);
  if (var < 0.0) var = 0.0;
  float sd = (float)sqrt(var);
  if (sd < 1e-8f) sd = 1.0f;
  return make_float2((float)mean, 1.0f / sd);
}

constexpr int kFinalizeUnroll = 4;

struct FinalizeParams {
  const float* raw;        // [L, B, Hkv, t_pad, gp]
  const double* moments;   // [L, B, Hq, 2]: (sum, sum of squares) from the scorer
  const int32_t* seq_lens;
  const int32_t* prefill_lens;  // may be null
  float* out;              // [Lo, B, Ho, t_pad]
  int L, B, Hkv, g, gp, t_pad;
  int window, normalize, group_reduce, head_reduce, layer_reduce;
  // A step may be cut into chunks of layers (raw scores of one chunk at a time): L counts the layers of this
  // call, l_total those of the whole step.  With a layer reduction, every call but the first continues from
  // the value already in `out` and only the last one divides the mean.
  int l_total, first_chunk, last_chunk;
  // Scatter mode (layer_reduce NONE, tensor-parallel layer-shared selection): output row r = (l * B + b) * Ho + ho
  // belongs to rank r / scatter_rows and is stored straight into THAT rank's receive buffer - a peer pointer, plain
  // stores over NVLink - at slot [scatter_rank][r % scatter_rows], so the exchange rides on the stores of this kernel.
  float* const* scatter_out;  // [ranks] device pointers to the ranks' [ranks, scatter_rows, t_pad] buffers, or null
  int scatter_rows, scatter_rank;
  // Layers are visited starting at scatter_shift (and wrapping): each rank begins with the layers of a different
  // owner, so that at no time all ranks store into the same GPU (its NVLink ingress would carry the whole exchange).
  // 0 unless scatter_out is set: with a layer reduction the order of the layers is part of the result.
  int scatter_shift;
};

// where the value of output row `row` (layer_reduce NONE), token t, goes
__device__ __forceinline__ float* finalize_row_dst(const FinalizeParams& p, size_t row, int t) {
  if (p.scatter_out == nullptr) return p.out + row * (size_t)p.t_pad + t;
  const size_t owner = row / (size_t)p.scatter_rows, local = row - owner * (size_t)p.scatter_rows;
  return p.scatter_out[owner] + ((size_t)p.scatter_rank * p.scatter_rows + local) * (size_t)p.t_pad + t;
}

// one thread per (request, output head, token); gp = query-head slots per KV head in the raw layout.
// Dynamic shared memory: (mean, 1/std) of the L x (heads this CTA reduces) rows it normalises with.
__global__ void __launch_bounds__(256) finalize_scores_kernel(const __grid_constant__ FinalizeParams p) {
  extern __shared__ float2 s_ms[];
  grid_dependency_wait();
  trigger_dependents();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.z;
  const int seq_len = min(p.seq_lens[b], p.t_pad);
  const int gp = p.gp;
  const int Hq = p.Hkv * p.g;
  const int Ho = p.head_reduce != TRIATTN_REDUCE_NONE ? 1 : p.Hkv;
  // with a layer reduction a CTA walks all layers of its output row; without one blockIdx.y also names the layer
  int ho = blockIdx.y, l_lo = 0, l_hi = p.L;
  if (p.layer_reduce == TRIATTN_REDUCE_NONE) {
    l_lo = blockIdx.y / Ho;
    ho = blockIdx.y - l_lo * Ho;
    l_lo += p.scatter_shift;
    if (l_lo >= p.L) l_lo -= p.L;
    l_hi = l_lo + 1;
  }
  const int h_begin = p.head_reduce != TRIATTN_REDUCE_NONE ? 0 : ho;
  const int h_end = p.head_reduce != TRIATTN_REDUCE_NONE ? p.Hkv : ho + 1;
  const int nh = (h_end - h_begin) * p.g;  // query heads this CTA reads
  if (blockIdx.x * blockDim.x >= seq_len) return;  // whole CTA beyond the request
  for (int i = threadIdx.x; i < (l_hi - l_lo) * nh; i += blockDim.x) {
    const int l = l_lo + i / nh, hq = h_begin * p.g + i % nh;
    s_ms[i] = mean_rstd_from_moments(p.moments + (((size_t)l * p.B + b) * Hq + hq) * 2, seq_len);
  }
  __syncthreads();
  if (t >= seq_len) return;
  const int recent = p.window > 0 ? min(p.window, seq_len) : 0;
  bool guarded = recent > 0 && t >= seq_len - recent;
  if (p.prefill_lens != nullptr && t < p.prefill_lens[b]) guarded = true;
  const bool vec4 = (gp & 3) == 0;
  float* out_red = p.out + ((size_t)b * Ho + ho) * (size_t)p.t_pad + t;
  float acc = (p.layer_reduce != TRIATTN_REDUCE_NONE && !p.first_chunk) ? *out_red : 0.f;
#pragma unroll(kFinalizeUnroll)
  for (int l = l_lo; l < l_hi; ++l) {
    float lv = -INFINITY;
    for (int kvh = h_begin; kvh < h_end; ++kvh) {
      float gv;
      if (guarded) {
        gv = INFINITY;
      } else {
        const float* r = p.raw + ((((size_t)l * p.B + b) * p.Hkv + kvh) * (size_t)p.t_pad + t) * gp;
        const float2* ms = s_ms + (size_t)(l - l_lo) * nh + (size_t)(kvh - h_begin) * p.g;
        float mx = -INFINITY, sum = 0.f;
        for (int j0 = 0; j0 < p.g; j0 += 4) {
          float s[4];
          if (vec4) {
            const float4 q = *reinterpret_cast<const float4*>(r + j0);
            s[0] = q.x; s[1] = q.y; s[2] = q.z; s[3] = q.w;
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) s[j] = (j0 + j < gp) ? r[j0 + j] : 0.f;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (j0 + j < p.g) {
              float z = s[j];
              if (p.normalize) z = __fmul_rn(__fsub_rn(z, ms[j0 + j].x), ms[j0 + j].y);
              mx = fmaxf(mx, z);
              sum = __fadd_rn(sum, z);
            }
          }
        }
        gv = p.group_reduce == TRIATTN_REDUCE_MEAN ? __fdiv_rn(sum, (float)p.g) : mx;
      }
      lv = fmaxf(lv, gv);  // single head unless head_reduce == MAX
    }
    const bool first = l == 0 && p.first_chunk;
    if (p.layer_reduce == TRIATTN_REDUCE_NONE) {
      *finalize_row_dst(p, ((size_t)l * p.B + b) * Ho + ho, t) = lv;
    } else if (p.layer_reduce == TRIATTN_REDUCE_MAX) {
      acc = first ? lv : fmaxf(acc, lv);
    } else {
      acc = first ? lv : __fadd_rn(acc, lv);
    }
  }
  if (p.layer_reduce == TRIATTN_REDUCE_MEAN && p.last_chunk) acc = __fdiv_rn(acc, (float)p.l_total);
  if (p.layer_reduce != TRIATTN_REDUCE_NONE) *out_red = acc;
}

// Fast path for one KV head per output row (head_reduce == NONE): group size G and the layer reduction are
// compile-time, the per-layer arithmetic is branch-free, and the raw rows of kFinalizePrefetch layers are
// requested before any of them is used, so a thread keeps that many 16-byte loads in flight.  The arithmetic
// per layer and the order over layers are those of the kernel above.
constexpr int kFinalizePrefetch = 6;

template <int G, int LR>
__global__ void __launch_bounds__(256) finalize_scores_fast_kernel(const __grid_constant__ FinalizeParams p) {
  constexpr int NQ = (G + 3) / 4;  // float4 loads per layer; the raw layout has 4*NQ slots per KV head
  extern __shared__ float2 s_ms[];  // [L][G]: (mean, 1/std) of this CTA's query heads
  grid_dependency_wait();
  trigger_dependents();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int seq_len = min(p.seq_lens[b], p.t_pad);
  if (blockIdx.x * blockDim.x >= seq_len) return;  // whole CTA beyond the request
  const int Hq = p.Hkv * G;
  const bool normalize = p.normalize != 0, group_mean = p.group_reduce == TRIATTN_REDUCE_MEAN;
  for (int i = threadIdx.x; i < p.L * G; i += blockDim.x) {
    const int l = i / G, j = i - l * G;
    float2 m = mean_rstd_from_moments(p.moments + (((size_t)l * p.B + b) * Hq + (size_t)kvh * G + j) * 2, seq_len);
    if (!normalize) m = make_float2(0.f, 1.f);  // (s - 0) * 1 == s exactly
    s_ms[i] = m;
  }
  __syncthreads();
  if (t >= seq_len) return;
  const int recent = p.window > 0 ? min(p.window, seq_len) : 0;
  bool guarded = recent > 0 && t >= seq_len - recent;
  if (p.prefill_lens != nullptr && t < p.prefill_lens[b]) guarded = true;
  float* out = p.out + ((size_t)b * p.Hkv + kvh) * (size_t)p.t_pad + t;
  const size_t out_layer_stride = (size_t)p.B * p.Hkv * (size_t)p.t_pad;
  if (guarded) {
    // +inf survives max and sum over layers and the division of the mean
    if (LR == TRIATTN_REDUCE_NONE) {
      for (int l = 0; l < p.L; ++l) *finalize_row_dst(p, ((size_t)l * p.B + b) * p.Hkv + kvh, t) = INFINITY;
    } else {
      *out = INFINITY;
    }
    return;
  }
  const size_t raw_layer_stride = (size_t)p.B * p.Hkv * (size_t)p.t_pad * NQ;  // in float4
  const float4* r = reinterpret_cast<const float4*>(p.raw) + (((size_t)b * p.Hkv + kvh) * (size_t)p.t_pad + t) * NQ;
  const bool first_chunk = p.first_chunk != 0;
  float acc = (LR != TRIATTN_REDUCE_NONE && !first_chunk) ? *out : 0.f;

  // the layer visited at step l of the loops below (identity unless the scatter mode rotates the order)
  auto at = [&](int l) {
    const int m = l + p.scatter_shift;
    return m >= p.L ? m - p.L : m;
  };
  // z-normalise, reduce over the G query heads; then fold layer l into the accumulator / the output
  auto layer = [&](const float4 (&q)[NQ], int l) {
    const float2* msl = s_ms + (size_t)l * G;
    float mx = -INFINITY, sum = 0.f;
#pragma unroll
    for (int j = 0; j < G; ++j) {
      const float4 v = q[j >> 2];
      const float sj = (j & 3) == 0 ? v.x : (j & 3) == 1 ? v.y : (j & 3) == 2 ? v.z : v.w;
      const float2 m = msl[j];
      const float z = __fmul_rn(__fsub_rn(sj, m.x), m.y);
      mx = fmaxf(mx, z);
      sum = __fadd_rn(sum, z);
    }
    const float lv = group_mean ? __fdiv_rn(sum, (float)G) : mx;
    const bool first = l == 0 && first_chunk;
    if (LR == TRIATTN_REDUCE_NONE) {
      *finalize_row_dst(p, ((size_t)l * p.B + b) * p.Hkv + kvh, t) = lv;
    } else if (LR == TRIATTN_REDUCE_MAX) {
      acc = first ? lv : fmaxf(acc, lv);
    } else {
      acc = first ? lv : __fadd_rn(acc, lv);
    }
  };

  int l0 = 0;
  for (; l0 + kFinalizePrefetch <= p.L; l0 += kFinalizePrefetch) {
    float4 q[kFinalizePrefetch][NQ];
#pragma unroll
    for (int i = 0; i < kFinalizePrefetch; ++i)
#pragma unroll
      for (int n = 0; n < NQ; ++n) q[i][n] = r[(size_t)at(l0 + i) * raw_layer_stride + n];
#pragma unroll
    for (int i = 0; i < kFinalizePrefetch; ++i) layer(q[i], at(l0 + i));
  }
  for (; l0 < p.L; ++l0) {
    float4 q[NQ];
#pragma unroll
    for (int n = 0; n < NQ; ++n) q[n] = r[(size_t)at(l0) * raw_layer_stride + n];
    layer(q, at(l0));
  }
  if (LR == TRIATTN_REDUCE_MEAN && p.last_chunk) acc = __fdiv_rn(acc, (float)p.l_total);
  if (LR != TRIATTN_REDUCE_NONE) *out = acc;
}

// out[i] = max over the `slots` receive slots of x[s * n + i]: the owner's half of the scattered exchange.
__global__ void __launch_bounds__(256) max_over_slots_kernel(const float* __restrict__ x, int slots, size_t n,
                                                             float* __restrict__ out) {
  grid_dependency_wait();
  trigger_dependents();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  if ((n & 3) == 0) {
    const size_t n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
      float4 m = __ldcs(x4 + i);
      for (int s = 1; s < slots; ++s) {
        const float4 v = __ldcs(x4 + (size_t)s * n4 + i);
        m.x = fmaxf(m.x, v.x); m.y = fmaxf(m.y, v.y); m.z = fmaxf(m.z, v.z); m.w = fmaxf(m.w, v.w);
      }
      reinterpret_cast<float4*>(out)[i] = m;
    }
  } else {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
      float m = x[i];
      for (int s = 1; s < slots; ++s) m = fmaxf(m, x[(size_t)s * n + i]);
      out[i] = m;
    }
  }
}

}  // namespace triattn
