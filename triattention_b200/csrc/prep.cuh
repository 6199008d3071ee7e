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

}  // namespace triattn
