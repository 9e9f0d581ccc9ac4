// Neuron-model kernels: one thread per neuron over a blocked ragged layout.
// Follows the element-wise template of the reference
// (nengo_ocl/clra_nonlinearities.py:1367-1417): grid = (block_size, n_blocks),
// thread (gind0, gind1) handles element starts[gind1] + gind0 of every
// variable when gind0 < sizes[gind1].
//
// Compiled with -fmad=false so that the LIF update keeps the reference's
// operation order (no fused multiply-add contraction).  expm1 / log1p / exp are
// evaluated in double and rounded once to float (correctly rounded float32
// results, independent of the math library), like the CPU evaluation of the
// reference kernels this path is checked against.
#include "nb2_common.cuh"
#include "nb2_math.cuh"
#include "../../include/nengo_b200.h"

__device__ __forceinline__ float nb2_var_load(const nb2_var& v, int block, int i) {
  return v.buf ? v.buf[v.starts[block] + i] : v.value;
}
__device__ __forceinline__ void nb2_var_store(const nb2_var& v, int block, int i, float x) {
  v.buf[v.starts[block] + i] = x;
}

// LIF with exact spike-time refractory handling (plan_lif, :1071-1133); `fastlif` selects the
// cheaper variant of the same kernel text (:1079-1114): the whole substep is integrated, a
// refractory neuron's voltage is scaled afterwards, the spike time is interpolated linearly.
__device__ __forceinline__ void nb2_lif_core(float J, float& V, float& W, float& S, float tau, float ref,
                                             float amp, float dtu, float dtu_inv, float dt_inv, int upsample,
                                             float Nadapt, bool adaptive, bool fastlif) {
  const float V_threshold = 1.0f;
  bool spiked = false;
  for (int ii = 0; ii < upsample; ++ii) {
    W -= dtu;
    const float delta_t = fastlif ? dtu : (W > dtu) ? 0.0f : (W < 0.0f) ? dtu : dtu - W;
    float dV;
    if (adaptive) dV = -nb2_expm1_cr(-delta_t / tau) * (J - Nadapt - V);
    else dV = -nb2_expm1_cr(-delta_t / tau) * (J - V);
    V += dV;
    if (fastlif) {
      if (V < 0.0f || W > dtu) V = 0.0f;
      else if (W >= 0.0f) V *= 1.0f - W * dtu_inv;
    }
    if (V > V_threshold) {
      if (fastlif) {
        const float overshoot = dtu * (V - V_threshold) / dV;
        W = ref - overshoot + dtu;
      } else {
        const float t_spike = dtu + tau * nb2_log1p_cr(-(V - V_threshold) / (J - V_threshold));
        W = ref + t_spike;
      }
      V = 0.0f;
      spiked = true;
    } else if (!fastlif && V < 0.0f) {
      V = 0.0f;
    }
  }
  S = spiked ? amp * dt_inv : 0.0f;
}

__global__ void nb2_neurons_kernel(int kind, int n_blocks, const int* __restrict__ sizes,
                                   const nb2_neuron_args a) {
  nb2_pdl_enter();
  const int gind0 = threadIdx.x;
  const int gind1 = blockIdx.x;
  if (gind1 >= n_blocks || gind0 >= sizes[gind1]) return;
  // dt-derived constants are double expressions rounded once to float, as the
  // reference renders them into `const float dtu = ..., dt_inv = ...;`
  const float dt = (float)a.dt;
  const float dtu = (float)(a.dt / a.upsample);
  const float dt_inv = (float)(1.0 / a.dt);
  const float dtu_inv = (float)(a.upsample / a.dt);

  if (kind == NB2_NEURON_LIF) {
    const float J = nb2_var_load(a.J, gind1, gind0);
    float V = nb2_var_load(a.V, gind1, gind0);
    float W = nb2_var_load(a.W, gind1, gind0);
    const float tau = nb2_var_load(a.tau, gind1, gind0);
    const float ref = nb2_var_load(a.ref, gind1, gind0);
    const float amp = nb2_var_load(a.amp, gind1, gind0);
    float N = 0.0f, S;
    if (a.adaptive) N = nb2_var_load(a.N, gind1, gind0);
    nb2_lif_core(J, V, W, S, tau, ref, amp, dtu, dtu_inv, dt_inv, a.upsample, N, a.adaptive != 0, a.fastlif != 0);
    nb2_var_store(a.V, gind1, gind0, V);
    nb2_var_store(a.W, gind1, gind0, W);
    nb2_var_store(a.S, gind1, gind0, S);
    if (a.adaptive) {
      const float tau_n = nb2_var_load(a.tau_n, gind1, gind0);
      const float inc_n = nb2_var_load(a.inc_n, gind1, gind0);
      nb2_var_store(a.N, gind1, gind0, N + (dt / tau_n) * (inc_n * S - N));
    }
  } else if (kind == NB2_NEURON_LIF_RATE) {
    // plan_lif_rate (:1168-1184): relies on 1/0 = inf -> log1p(inf) = inf -> R = 0
    float J = nb2_var_load(a.J, gind1, gind0);
    const float tau = nb2_var_load(a.tau, gind1, gind0);
    const float ref = nb2_var_load(a.ref, gind1, gind0);
    const float amp = nb2_var_load(a.amp, gind1, gind0);
    float N = 0.0f;
    if (a.adaptive) {
      N = nb2_var_load(a.N, gind1, gind0);
      J = fmaxf(J - N - 1.0f, 0.0f);
    } else {
      J = fmaxf(J - 1.0f, 0.0f);
    }
    const float R = amp / (ref + tau * nb2_log1p_cr(1.0f / J));
    nb2_var_store(a.S, gind1, gind0, R);
    if (a.adaptive) {
      const float tau_n = nb2_var_load(a.tau_n, gind1, gind0);
      const float inc_n = nb2_var_load(a.inc_n, gind1, gind0);
      nb2_var_store(a.N, gind1, gind0, N + (dt / tau_n) * (inc_n * R - N));
    }
  } else if (kind == NB2_NEURON_RELU) {
    // plan_rectified_linear (:1244-1245)
    const float J = nb2_var_load(a.J, gind1, gind0);
    const float amp = nb2_var_load(a.amp, gind1, gind0);
    nb2_var_store(a.S, gind1, gind0, amp * fmaxf(J, 0.0f));
  } else if (kind == NB2_NEURON_SPIKING_RELU) {
    // plan_spiking_rectified_linear (:1216-1222)
    const float J = nb2_var_load(a.J, gind1, gind0);
    float V = nb2_var_load(a.V, gind1, gind0);
    const float amp = nb2_var_load(a.amp, gind1, gind0);
    V += (J > 0.0f) ? dt * J : 0.0f;
    const float n_spikes = floorf(V);
    nb2_var_store(a.V, gind1, gind0, V - n_spikes);
    nb2_var_store(a.S, gind1, gind0, amp * n_spikes * dt_inv);
  } else if (kind == NB2_NEURON_SIGMOID) {
    // plan_sigmoid (:1267-1268)
    const float J = nb2_var_load(a.J, gind1, gind0);
    const float ref = nb2_var_load(a.ref, gind1, gind0);
    const float R = J < -88.0f ? 0.0f : J > 15.0f ? 1.0f / ref : 1.0f / (ref * (1.0f + nb2_exp_cr(-J)));
    nb2_var_store(a.S, gind1, gind0, R);
  }
}

extern "C" int nb2_neurons(void* stream, int kind, int n_blocks, int block_size, const int* sizes,
                           const nb2_neuron_args* args) {
  if (n_blocks == 0) return NB2_OK;
  NB2_REQUIRE(args && sizes, "null pointer");
  NB2_REQUIRE(block_size >= 1 && block_size <= 1024, "block_size");
  NB2_REQUIRE(kind >= NB2_NEURON_LIF && kind <= NB2_NEURON_SIGMOID, "kind");
  NB2_REQUIRE(args->J.buf && args->S.buf, "J and output buffers required");
  NB2_REQUIRE(args->upsample >= 1 || kind != NB2_NEURON_LIF, "upsample");
  if (kind == NB2_NEURON_LIF) NB2_REQUIRE(args->V.buf && args->W.buf, "V/W buffers required");
  if (kind == NB2_NEURON_SPIKING_RELU) NB2_REQUIRE(args->V.buf, "V buffer required");
  if (args->adaptive) NB2_REQUIRE(args->N.buf, "N buffer required");
  nb2_neuron_args a = *args;
  if (a.upsample < 1) a.upsample = 1;
  nb2_launch(nb2_neurons_kernel, dim3(n_blocks), dim3(block_size), 0, nb2_stream(stream), kind, n_blocks, sizes, a);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
