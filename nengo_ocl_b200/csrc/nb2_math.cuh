// Correctly rounded float32 elementary functions for the neuron updates.
#pragma once
#include "nb2_common.cuh"

// expm1 / log1p of a float argument, correctly rounded to float (evaluated in double and
// rounded once): the float32 result no longer depends on whose math library computed it, so
// the neuron state is bit-identical to a CPU evaluation of the reference kernel done the same
// way.  In the LIF update both arguments lie in [-dt / tau, 0] (a step integrates over at most
// dt, and the overshoot of a spiking neuron is at most the step's relative voltage change), so
// for |x| <= 1/16 the Taylor series in double is exact to double round-off with a dozen fused
// multiply-adds; anything else goes to the double-precision library function.
__device__ __forceinline__ double nb2_expm1_series(double x) {
  double q = 1.0 / 3628800.0;            // x^10 / 10!
  q = fma(q, x, 1.0 / 362880.0);
  q = fma(q, x, 1.0 / 40320.0);
  q = fma(q, x, 1.0 / 5040.0);
  q = fma(q, x, 1.0 / 720.0);
  q = fma(q, x, 1.0 / 120.0);
  q = fma(q, x, 1.0 / 24.0);
  q = fma(q, x, 1.0 / 6.0);
  q = fma(q, x, 0.5);
  return fma(x * x, q, x);
}
__device__ __forceinline__ float nb2_expm1_cr(float xf) {
  const double x = (double)xf;
  if (fabsf(xf) > 0.0625f) return (float)expm1(x);
  return (float)nb2_expm1_series(x);
}
__device__ __forceinline__ double nb2_log1p_series(double x) {
  double q = 1.0 / 16.0;                 // -x^16 / 16
  q = fma(-q, x, 1.0 / 15.0);
  q = fma(-q, x, 1.0 / 14.0);
  q = fma(-q, x, 1.0 / 13.0);
  q = fma(-q, x, 1.0 / 12.0);
  q = fma(-q, x, 1.0 / 11.0);
  q = fma(-q, x, 1.0 / 10.0);
  q = fma(-q, x, 1.0 / 9.0);
  q = fma(-q, x, 1.0 / 8.0);
  q = fma(-q, x, 1.0 / 7.0);
  q = fma(-q, x, 1.0 / 6.0);
  q = fma(-q, x, 1.0 / 5.0);
  q = fma(-q, x, 1.0 / 4.0);
  q = fma(-q, x, 1.0 / 3.0);
  q = fma(-q, x, 0.5);                   // 1/2 - x/3 + x^2/4 - ...
  return fma(-(x * x), q, x);
}
__device__ __forceinline__ float nb2_log1p_cr(float xf) {
  const double x = (double)xf;
  if (!(fabsf(xf) <= 0.0625f)) return (float)log1p(x);
  return (float)nb2_log1p_series(x);
}
// N independent evaluations at once: the series of the arguments interleave in the
// pipeline (one dependent chain of fused multiply-adds each), and the library fallback is one
// rarely taken branch for all of them.
// (the library calls stay out of line: they are almost never taken, and inlined they would be
// most of the instructions of the kernels that use them)
static __device__ __noinline__ float nb2_expm1_library(float x) { return (float)expm1((double)x); }
static __device__ __noinline__ float nb2_log1p_library(float x) { return (float)log1p((double)x); }

template <int N>
__device__ __forceinline__ void nb2_expm1_crN(const float (&x)[N], float (&out)[N]) {
  float big = 0.0f;
#pragma unroll
  for (int j = 0; j < N; ++j) big = fmaxf(big, fabsf(x[j]));
  if (!(big <= 0.0625f)) {
#pragma unroll
    for (int j = 0; j < N; ++j) out[j] = nb2_expm1_library(x[j]);
    return;
  }
#pragma unroll
  for (int j = 0; j < N; ++j) out[j] = (float)nb2_expm1_series((double)x[j]);
}
template <int N>
__device__ __forceinline__ void nb2_log1p_crN(const float (&x)[N], float (&out)[N]) {
  float big = 0.0f;
#pragma unroll
  for (int j = 0; j < N; ++j) big = fmaxf(big, fabsf(x[j]));
  if (!(big <= 0.0625f)) {
#pragma unroll
    for (int j = 0; j < N; ++j) out[j] = nb2_log1p_library(x[j]);
    return;
  }
#pragma unroll
  for (int j = 0; j < N; ++j) out[j] = (float)nb2_log1p_series((double)x[j]);
}

__device__ __forceinline__ float nb2_exp_cr(float x) { return (float)exp((double)x); }
