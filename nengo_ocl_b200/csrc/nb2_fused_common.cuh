// Tables and neuron update shared by the fused ensemble kernels (nb2_fused.cu,
// nb2_fused_stream.cu).
#pragma once
#include "nb2_common.cuh"
#include "nb2_math.cuh"

// table layouts (ints; floats stored as bit patterns)
enum { E_N = 0, E_J, E_V, E_W, E_S, E_BIAS, E_NTERMS, E_TERM0, E_NCONN, E_CONN0, E_TAU, E_REF, E_AMP, E_FLAGS, E_EM1, E_STRIDE = 16 };
enum { T_A = 0, T_D, T_X, T_XS, T_STRIDE = 4 };
enum { C_W = 0, C_D, C_WEIGHTED, C_FILT, C_B0, C_A0, C_PES, C_ERR, C_PF, C_PFB0, C_PFA0, C_ALPHA, C_STRIDE = 16 };

__device__ __forceinline__ float bits(int v) { return __int_as_float(v); }

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

// The same update for N neurons of one lane.  The rare double-precision evaluations (a
// neuron leaving its refractory period inside the step; a neuron that spikes) are taken out of
// the per-neuron flow: if any of them needs one, all the arguments are evaluated together,
// so the warp pays the latency of one series instead of up to four in sequence.  Values are
// identical to N calls of fused_lif.
template <int N>
__device__ __forceinline__ void fused_lifN(const float (&J)[N], float (&V)[N], float (&W)[N], float (&S)[N],
                                           float tau, float ref, float amp, float dt, float dt_inv,
                                           float em1_dt) {
  float em1[N], arg[N];
  bool need = false;
#pragma unroll
  for (int j = 0; j < N; ++j) {
    W[j] -= dt;
    const float delta_t = (W[j] > dt) ? 0.0f : (W[j] < 0.0f) ? dt : dt - W[j];
    em1[j] = (delta_t == 0.0f) ? 0.0f : em1_dt;
    arg[j] = 0.0f;
    if (delta_t != dt && delta_t != 0.0f) {
      need = true;
      arg[j] = -delta_t / tau;
    }
  }
  if (need) {
    float v[N];
    nb2_expm1_crN<N>(arg, v);
#pragma unroll
    for (int j = 0; j < N; ++j)
      if (arg[j] != 0.0f) em1[j] = v[j];
  }
  float y[N];
  bool spiked[N], any = false;
#pragma unroll
  for (int j = 0; j < N; ++j) {
    const float dV = -em1[j] * (J[j] - V[j]);
    V[j] += dV;
    y[j] = 0.0f;
    spiked[j] = V[j] > 1.0f;
    if (spiked[j]) {
      any = true;
      y[j] = -(V[j] - 1.0f) / (J[j] - 1.0f);
    } else if (V[j] < 0.0f) {
      V[j] = 0.0f;
    }
  }
  if (any) {
    float l[N];
    nb2_log1p_crN<N>(y, l);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      if (spiked[j]) {
        const float t_spike = dt + tau * l[j];
        W[j] = ref + t_spike;
        V[j] = 0.0f;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < N; ++j) S[j] = spiked[j] ? amp * dt_inv : 0.0f;
}
