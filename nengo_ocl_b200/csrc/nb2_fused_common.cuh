// Tables and neuron update shared by the fused ensemble kernels (nb2_fused.cu,
// nb2_fused_stream.cu).
#pragma once
#include "nb2_common.cuh"

// table layouts (ints; floats stored as bit patterns)
enum { E_N = 0, E_J, E_V, E_W, E_S, E_BIAS, E_NTERMS, E_TERM0, E_NCONN, E_CONN0, E_TAU, E_REF, E_AMP, E_FLAGS, E_STRIDE = 16 };
enum { T_A = 0, T_D, T_X, T_XS, T_STRIDE = 4 };
enum { C_W = 0, C_D, C_WEIGHTED, C_FILT, C_B0, C_A0, C_PES, C_ERR, C_PF, C_PFB0, C_PFA0, C_ALPHA, C_STRIDE = 16 };

__device__ __forceinline__ float bits(int v) { return __int_as_float(v); }

// LIF step with exact spike-time refractory handling, upsample = 1
// (clra_nonlinearities.py:1087-1132); returns the output spike value.
__device__ __forceinline__ float fused_lif(float J, float& V, float& W, float tau, float ref, float amp,
                                           float dt, float dt_inv) {
  W -= dt;
  const float delta_t = (W > dt) ? 0.0f : (W < 0.0f) ? dt : dt - W;
  const float dV = -expm1f(-delta_t / tau) * (J - V);
  V += dV;
  bool spiked = false;
  if (V > 1.0f) {
    const float t_spike = dt + tau * log1pf(-(V - 1.0f) / (J - 1.0f));
    W = ref + t_spike;
    V = 0.0f;
    spiked = true;
  } else if (V < 0.0f) {
    V = 0.0f;
  }
  return spiked ? amp * dt_inv : 0.0f;
}

