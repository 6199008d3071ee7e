// Weight preparation: offset-phase trig tables and folding of the calibrated query
// statistics into per-(layer, request, query head) dot-product weights.
#pragma once

#include "common.cuh"

namespace triattn {

// trig[b][row][f]: MEAN -> rows {C, S} (means over offsets); MAX -> rows {cos_0..cos_{O-1}, sin_0..sin_{O-1}}.
// phase = fl32(round_start + offset) * omega_f rounded to fp32 (the reference multiplies an fp32 tensor by
// the scalar t, scoring.py:313,322); cos/sin of that fp32 value are evaluated in double and rounded once.
__global__ void trig_table_kernel(const float* __restrict__ omega, const float* __restrict__ offsets,
                                  const int32_t* __restrict__ round_start, int F, int O, int agg_max,
                                  float* __restrict__ trig) {
  const int b = blockIdx.x;
  const float rs = (float)((double)round_start[b]);
  const int rows = agg_max ? 2 * O : 2;
  for (int f = threadIdx.x; f < F; f += blockDim.x) {
    const float w = omega[f];
    double csum = 0.0, ssum = 0.0;
    for (int o = 0; o < O; ++o) {
      const float t = (float)((double)rs + (double)offsets[o]);
      const float phase = __fmul_rn(t, w);
      double s, c;
      sincos((double)phase, &s, &c);
      if (agg_max) {
        trig[((size_t)b * rows + o) * F + f] = (float)c;
        trig[((size_t)b * rows + O + o) * F + f] = (float)s;
      } else {
        // the reference averages per-offset scores in fp32; averaging fp32-rounded cos/sin keeps the
        // same per-offset rounding and only reorders the (linear) sum
        csum += (double)(float)c;
        ssum += (double)(float)s;
      }
    }
    if (!agg_max) {
      trig[((size_t)b * rows + 0) * F + f] = (float)(csum / (double)O);
      trig[((size_t)b * rows + 1) * F + f] = (float)(ssum / (double)O);
    }
  }
}

// weights[l][b][h][row][f]; one thread per (l, b, h, f).
__global__ void fold_weights_kernel(const float* __restrict__ q_re, const float* __restrict__ q_im,
                                    const float* __restrict__ q_abs, const float* __restrict__ fs,
                                    const float* __restrict__ trig, int L, int B, int Hq, int F, int O,
                                    int agg_max, int flags, float* __restrict__ weights) {
  const size_t n = (size_t)L * B * Hq * F;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int f = (int)(i % F);
  const int h = (int)((i / F) % Hq);
  const int b = (int)((i / ((size_t)F * Hq)) % B);
  const int l = (int)(i / ((size_t)F * Hq * B));
  const size_t si = ((size_t)l * Hq + h) * F + f;
  const float qr = q_re[si], qi = q_im[si], qa = q_abs[si], sc = fs[si];
  const int rows = agg_max ? 2 * O + 1 : 3;
  const int trows = agg_max ? 2 * O : 2;
  float* w = weights + (((size_t)l * B + b) * Hq + h) * rows * F + f;
  const float* tr = trig + (size_t)b * trows * F + f;
  const bool no_trig = (flags & TRIATTN_FLAG_DISABLE_TRIG) != 0;
  // |q_mean| exactly as the reference forms it in fp32: sqrt(qr*qr + qi*qi + 1e-8)
  const float qma = __fsqrt_rn(__fadd_rn(__fadd_rn(__fmul_rn(qr, qr), __fmul_rn(qi, qi)), 1e-8f));
  const float coef = (flags & TRIATTN_FLAG_DISABLE_MLR) ? qa : __fsub_rn(qa, qma);
  const float wmag = __fmul_rn(coef, sc);
  if (!agg_max) {
    const double C = (double)tr[0], S = (double)tr[(size_t)F];
    w[0] = no_trig ? 0.f : (float)((double)sc * ((double)qr * C - (double)qi * S));
    w[(size_t)F] = no_trig ? 0.f : (float)((double)sc * ((double)qi * C + (double)qr * S));
    w[2 * (size_t)F] = wmag;
  } else {
    for (int o = 0; o < O; ++o) {
      const double C = (double)tr[(size_t)o * F], S = (double)tr[(size_t)(O + o) * F];
      w[(size_t)o * F] = no_trig ? 0.f : (float)((double)sc * ((double)qr * C - (double)qi * S));
      w[(size_t)(O + o) * F] = no_trig ? 0.f : (float)((double)sc * ((double)qi * C + (double)qr * S));
    }
    w[(size_t)(2 * O) * F] = wmag;
  }
}

// ---------------------------------------------------------------------------------------- one-launch variant
// Same results as trig_table_kernel followed by fold_weights_kernel, without the table in global memory:
// CTA (chunk, request) evaluates the O x F cos/sin values of its request into shared memory (one value per
// thread and round, so the double-precision sincos calls run in parallel instead of O in a row per thread),
// reduces them exactly as trig_table_kernel does, and then folds the rows [row0, row1) of the (layer, query
// head) list.  It can also clear a moments array for the scorer that follows (saves a memset between launches).
constexpr int kPrepThreads = 256;

struct PrepFusedParams {
  const float *q_re, *q_im, *q_abs, *fs;  // [L, Hq, F]
  const float *omega, *offsets;           // [F], [O]
  const int32_t* round_start;             // [B]
  float* weights;                         // [L, B, Hq, rows, F]
  double* moments;                        // [L, B, Hq, 2] to clear, or null
  int L, B, Hq, F, O, agg_max, flags;
  int rows_per_cta;                       // (layer, head) rows one CTA folds
};

__global__ void __launch_bounds__(kPrepThreads) prep_weights_fused_kernel(const __grid_constant__ PrepFusedParams p) {
  extern __shared__ float s_trig[];  // cos [O][F], sin [O][F]; MEAN keeps its two reduced rows behind them
  grid_dependency_wait();
  trigger_dependents();
  const int b = blockIdx.y, tid = threadIdx.x;
  const int F = p.F, O = p.O;
  float* s_cos = s_trig;
  float* s_sin = s_trig + (size_t)O * F;
  float* s_mean = s_trig + 2 * (size_t)O * F;  // C [F], S [F]
  const float rs = (float)((double)p.round_start[b]);
  for (int i = tid; i < O * F; i += kPrepThreads) {
    const int o = i / F, f = i - o * F;
    const float t = (float)((double)rs + (double)p.offsets[o]);
    const float phase = __fmul_rn(t, p.omega[f]);
    double sn, cs;
    sincos((double)phase, &sn, &cs);
    s_cos[i] = (float)cs;
    s_sin[i] = (float)sn;
  }
  __syncthreads();
  if (!p.agg_max) {
    for (int f = tid; f < F; f += kPrepThreads) {
      double csum = 0.0, ssum = 0.0;
      for (int o = 0; o < O; ++o) {  // same order as trig_table_kernel
        csum += (double)s_cos[o * F + f];
        ssum += (double)s_sin[o * F + f];
      }
      s_mean[f] = (float)(csum / (double)O);
      s_mean[F + f] = (float)(ssum / (double)O);
    }
    __syncthreads();
  }
  const int n_rows = p.L * p.Hq;
  const int row0 = blockIdx.x * p.rows_per_cta;
  const int row1 = min(row0 + p.rows_per_cta, n_rows);
  const int rows = p.agg_max ? 2 * O + 1 : 3;
  const bool no_trig = (p.flags & TRIATTN_FLAG_DISABLE_TRIG) != 0;
  for (int i = row0 * F + tid; i < row1 * F; i += kPrepThreads) {
    const int r = i / F, f = i - r * F;
    const int l = r / p.Hq, h = r - l * p.Hq;
    const size_t si = (size_t)r * F + f;
    const float qr = p.q_re[si], qi = p.q_im[si], qa = p.q_abs[si], sc = p.fs[si];
    float* w = p.weights + (((size_t)l * p.B + b) * p.Hq + h) * rows * F + f;
    const float qma = __fsqrt_rn(__fadd_rn(__fadd_rn(__fmul_rn(qr, qr), __fmul_rn(qi, qi)), 1e-8f));
    const float coef = (p.flags & TRIATTN_FLAG_DISABLE_MLR) ? qa : __fsub_rn(qa, qma);
    const float wmag = __fmul_rn(coef, sc);
    if (!p.agg_max) {
      const double C = (double)s_mean[f], S = (double)s_mean[F + f];
      w[0] = no_trig ? 0.f : (float)((double)sc * ((double)qr * C - (double)qi * S));
      w[(size_t)F] = no_trig ? 0.f : (float)((double)sc * ((double)qi * C + (double)qr * S));
      w[2 * (size_t)F] = wmag;
    } else {
      for (int o = 0; o < O; ++o) {
        const double C = (double)s_cos[o * F + f], S = (double)s_sin[o * F + f];
        w[(size_t)o * F] = no_trig ? 0.f : (float)((double)sc * ((double)qr * C - (double)qi * S));
        w[(size_t)(O + o) * F] = no_trig ? 0.f : (float)((double)sc * ((double)qi * C + (double)qr * S));
      }
      w[(size_t)(2 * O) * F] = wmag;
    }
  }
  if (p.moments != nullptr) {
    for (int r = row0 + tid; r < row1; r += kPrepThreads) {
      const int l = r / p.Hq, h = r - l * p.Hq;
      double* m = p.moments + (((size_t)l * p.B + b) * p.Hq + h) * 2;
      m[0] = 0.0;
      m[1] = 0.0;
    }
  }
}

}  // namespace triattn
