// White-noise processes: plan_whitenoise (nengo_ocl/clra_nonlinearities.py:1573-1675).
//
// The reference keeps a RANLUX state per work-item (create_rngs / init_rngs,
// :1486-1532, generator from pyopencl-ranluxcl.cl) and advances it every step.
// Here the generator is counter-based -- Philox4x32-10 (Salmon, Moraes, Dror,
// Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11) -- so there is no
// state to store, initialise, reset or checkpoint: the four words for elements
// 4q .. 4q+3 of a process at a step are philox(counter = (step, q, 0, 0),
// key = the process's 64-bit seed), whatever thread computes them.  The random
// STREAM therefore differs from the reference's (RANLUX cannot be restated: its
// source is not part of the reference tree); the use made of a sample is the
// reference's (:1536-1551, :1625-1637):
//   uniform   low + (high - low) * u,  u = (word >> 8) * 2^-24 in [0, 1)
//   gaussian  mean + std * z,  z by Box-Muller in double on the word pairs
//             (0, 1) and (2, 3), rounded to float once
//   if scale: sample = (float)(sample * (1 / sqrt(dt)))   (a double literal there)
//   y += sample  or  y = sample
// This translation unit is compiled with -fmad=false.
#include "nb2_common.cuh"
#include "../../include/nengo_b200.h"

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t (&k)[2]) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k[0], n2 = hi0 ^ c[3] ^ k[1];
  c[0] = n0;
  c[1] = lo1;
  c[2] = n2;
  c[3] = lo0;
  k[0] += 0x9E3779B9u;
  k[1] += 0xBB67AE85u;
}

__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  uint32_t k[2] = {k0, k1};
#pragma unroll
  for (int r = 0; r < 10; ++r) philox_round(c, k);
}

// grid (items, ceil(max quads / 256)): one thread per four elements
__global__ void nb2_whitenoise_kernel(const int* __restrict__ shape0s, const int* __restrict__ Ystarts, float* Y,
                                      const int* __restrict__ Tstarts, const float* T,
                                      const int* __restrict__ enums, const float* __restrict__ params,
                                      const int* __restrict__ scales, const int* __restrict__ incs,
                                      const unsigned* __restrict__ seeds, double sqrt_dt_inv) {
  nb2_pdl_enter();
  const int k = blockIdx.x;
  const int q = blockIdx.y * blockDim.x + threadIdx.x;
  const int m = shape0s[k];
  if (4 * q >= m) return;
  uint32_t c[4] = {(uint32_t)(int)T[Tstarts[k]], (uint32_t)q, 0u, 0u};
  philox4x32_10(c, seeds[2 * k], seeds[2 * k + 1]);
  const float p0 = params[2 * k], p1 = params[2 * k + 1];
  float v[4];
  if (enums[k] == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = p0 + (p1 - p0) * ((float)(c[j] >> 8) * 5.9604644775390625e-8f);
  } else {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const double u1 = ((double)(c[2 * h] >> 8) + 1.0) * 5.9604644775390625e-8;  // (0, 1]
      const double u2 = (double)(c[2 * h + 1] >> 8) * 5.9604644775390625e-8;      // [0, 1)
      const double r = sqrt(-2.0 * log(u1));
      double sn, cs;
      sincos(6.283185307179586 * u2, &sn, &cs);
      v[2 * h] = p0 + p1 * (float)(r * cs);
      v[2 * h + 1] = p0 + p1 * (float)(r * sn);
    }
  }
  float* y = Y + Ystarts[k];
  const bool scale = scales[k] != 0, inc = incs[k] != 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = 4 * q + j;
    if (i >= m) break;
    float s = v[j];
    if (scale) s = (float)((double)s * sqrt_dt_inv);
    y[i] = inc ? y[i] + s : s;
  }
}

extern "C" int nb2_whitenoise(void* stream, int n_items, int max_len, const int* shape0s, const int* Ystarts, float* Y,
                              const int* Tstarts, const float* T, const int* enums, const float* params,
                              const int* scales, const int* incs, const unsigned* seeds, double dt) {
  if (n_items == 0) return NB2_OK;
  NB2_REQUIRE(shape0s && Ystarts && Y && Tstarts && T && enums && params && scales && incs && seeds, "null pointer");
  NB2_REQUIRE(max_len >= 1 && dt > 0, "sizes");
  const int quads = (max_len + 3) / 4;
  NB2_REQUIRE((quads + 255) / 256 <= 65535, "an item of more than 67 M elements");
  nb2_launch(nb2_whitenoise_kernel, dim3(n_items, (quads + 255) / 256), dim3(256), 0, nb2_stream(stream), shape0s,
             Ystarts, Y, Tstarts, T, enums, params, scales, incs, seeds, 1.0 / sqrt(dt));
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
