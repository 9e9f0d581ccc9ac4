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
#include "nb2_fused_common.cuh"
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

// The common LIF case -- one substep, no adaptation, tau / ref / amp one scalar each -- with four
// neurons per thread (elements i, i + T, i + 2T, i + 3T of the block, T = threads per block, so
// every load is contiguous across the warp).  The arithmetic is that of nb2_lif_core; what changes
// is how often the expensive parts run: expm1(-dt / tau) for a neuron outside its refractory
// period is one number per launch (em1_dt, rounded once from double on the host), and the
// double-precision series for the neurons that leave the refractory period or spike is entered
// once for the 128 neurons of a warp instead of once for every 32 (fused_lifN).
#define LIF4_NB 4
__global__ void __launch_bounds__(256) nb2_lif4_kernel(int n_blocks, const int* __restrict__ sizes,
                                                       const nb2_neuron_args a, float em1_dt) {
  nb2_pdl_enter();
  const int block = blockIdx.x;
  if (block >= n_blocks) return;
  const int n = sizes[block];
  const int t = threadIdx.x, T = blockDim.x;
  const float dt = (float)a.dt, dt_inv = (float)(1.0 / a.dt);
  const float tau = a.tau.value, ref = a.ref.value, amp = a.amp.value;
  const float* J = a.J.buf + a.J.starts[block];
  float* V = a.V.buf + a.V.starts[block];
  float* W = a.W.buf + a.W.starts[block];
  float* S = a.S.buf + a.S.starts[block];
  for (int i0 = t; i0 < n; i0 += LIF4_NB * T) {
    float Jv[LIF4_NB], Vv[LIF4_NB], Wv[LIF4_NB], Sv[LIF4_NB];
#pragma unroll
    for (int j = 0; j < LIF4_NB; ++j) {
      const int i = i0 + j * T;
      const bool ok = i < n;
      Jv[j] = ok ? J[i] : 0.0f;  // (an idle slot holds a neuron at rest: it neither integrates nor spikes)
      Vv[j] = ok ? V[i] : 0.0f;
      Wv[j] = ok ? W[i] : 0.0f;
    }
    fused_lifN<LIF4_NB>(Jv, Vv, Wv, Sv, tau, ref, amp, dt, dt_inv, em1_dt);
#pragma unroll
    for (int j = 0; j < LIF4_NB; ++j) {
      const int i = i0 + j * T;
      if (i < n) {
        V[i] = Vv[j];
        W[i] = Wv[j];
        S[i] = Sv[j];
      }
    }
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
  if (kind == NB2_NEURON_LIF && a.upsample == 1 && !a.adaptive && !a.fastlif && !a.tau.buf && !a.ref.buf &&
      !a.amp.buf && a.J.starts && a.V.starts && a.W.starts && a.S.starts) {
    // expm1 of the float quotient, evaluated in double and rounded once: what nb2_expm1_cr returns
    const float em1_dt = (float)expm1((double)(-(float)a.dt / a.tau.value));
    int threads = (block_size + LIF4_NB - 1) / LIF4_NB;
    threads = threads < 32 ? 32 : (threads + 31) & ~31;
    nb2_launch(nb2_lif4_kernel, dim3(n_blocks), dim3(threads), 0, nb2_stream(stream), n_blocks, sizes, a, em1_dt);
    NB2_LAUNCH_CHECK();
    return NB2_OK;
  }
  nb2_launch(nb2_neurons_kernel, dim3(n_blocks), dim3(block_size), 0, nb2_stream(stream), kind, n_blocks, sizes, a);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
