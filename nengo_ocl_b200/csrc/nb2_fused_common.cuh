// Tables and neuron update shared by the fused ensemble kernels (nb2_fused.cu,
// nb2_fused_stream.cu).
#pragma once
#include "nb2_common.cuh"

// table layouts (ints; floats stored as bit patterns)
enum { E_N = 0, E_J, E_V, E_W, E_S, E_BIAS, E_NTERMS, E_TERM0, E_NCONN, E_CONN0, E_TAU, E_REF, E_AMP, E_FLAGS, E_EM1, E_STRIDE = 16 };
enum { T_A = 0, T_D, T_X, T_XS, T_STRIDE = 4 };
enum { C_W = 0, C_D, C_WEIGHTED, C_FILT, C_B0, C_A0, C_PES, C_ERR, C_PF, C_PFB0, C_PFA0, C_ALPHA, C_STRIDE = 16 };

__device__ __forceinline__ float bits(int v) { return __int_as_float(v); }

// expm1 / log1p of a float argument, correctly rounded to float (evaluated in double and
// rounded once): the float32 result no longer depends on whose math library computed it, so
// the neuron state is bit-identical to a CPU evaluation of the reference kernel done the same
// way.
__device__ __forceinline__ float nb2_expm1_cr(float x) { return (float)expm1((double)x); }
__device__ __forceinline__ float nb2_log1p_cr(float x) { return (float)log1p((double)x); }

// LIF step with exact spike-time refractory handling, upsample = 1
// (clra_nonlinearities.py:1087-1132); returns the output spike value.
// em1_dt = expm1(-dt / tau) rounded to float, formed once per ensemble on the host: a
// neuron outside its refractory period integrates over the whole step, so delta_t == dt
// for almost every neuron and the double-precision evaluation is needed only for the few
// that leave the refractory period inside this step.
__device__ __forceinline__ float fused_lif(float J, float& V, float& W, float tau, float ref, float amp,
                                           float dt, float dt_inv, float em1_dt) {
  W -= dt;
  const float delta_t = (W > dt) ? 0.0f : (W < 0.0f) ? dt : dt - W;
  float em1 = em1_dt;
  if (delta_t != dt) em1 = (delta_t == 0.0f) ? 0.0f : nb2_expm1_cr(-delta_t / tau);
  const float dV = -em1 * (J - V);
  V += dV;
  bool spiked = false;
  if (V > 1.0f) {
    const float t_spike = dt + tau * nb2_log1p_cr(-(V - 1.0f) / (J - 1.0f));
    W = ref + t_spike;
    V = 0.0f;
    spiked = true;
  } else if (V < 0.0f) {
    V = 0.0f;
  }
  return spiked ? amp * dt_inv : 0.0f;
}
