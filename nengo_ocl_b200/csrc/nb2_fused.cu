// Fused ensemble step: encoder GEMV + LIF update + decoder GEMV (+ lowpass
// synapse) (+ PES decoder update) in ONE kernel per time step.
//
// Replaces, for every population whose operators match the pattern, the
// sequence the reference launches as separate kernels each step:
//   plan_copy (bias -> J)                     clra_nonlinearities.py:217-304
//   plan_block_gemv (J += encoders . x)       clra_gemv.py:861-1175 (2 kernels)
//   plan_lif                                  clra_nonlinearities.py:1028-1146
//   plan_reset (decoded value)                clra_nonlinearities.py:147-214
//   plan_block_gemv (decoded = decoders . s)  clra_gemv.py:861-1175 (2 kernels)
//   plan_linearfilter (lowpass synapse)       clra_nonlinearities.py:577-803
//   plan_linearfilter (PES activity filter), plan_elementwise_inc(outer) (PES
//   delta, simulator.py:1334-1345), plan_copy (decoders += delta)
// The input current J, the PES delta and (unless something else reads them)
// the spikes never touch HBM.  Per step and ensemble the kernel streams the
// encoders, the neuron state and every decoder matrix exactly once (decoders
// are written back once when PES is active): it is HBM-bound, and all streams
// are contiguous, so threads map to consecutive neurons.
//
// One thread group per ensemble: a CTA of 256 threads for large populations, a
// warp for small ones (8 per CTA).  Phase 1: each thread computes J for its
// neurons (x staged in shared memory, encoder rows read with 128-bit loads when
// aligned), runs the LIF update (same operation order as the reference kernel;
// this file is compiled with -fmad=false, dot products use explicit fmaf) and
// keeps the spikes in shared memory.  Phase 2: for every outgoing connection,
// 16 decoder rows at a time, each thread accumulates w[r][i] * s[i] over its
// neurons while applying the PES update to the same element, then the group
// reduces the 16 partial sums in a fixed order and one thread per row runs the
// synapse.  All index tables are int32 element offsets into the one packed
// signal buffer.
#include "nb2_common.cuh"
#include "nb2_fused_common.cuh"
#include "../../include/nengo_b200.h"

#define FUSED_THREADS 256
#ifndef FUSED_MIN_BLOCKS
#define FUSED_MIN_BLOCKS 3  // CTAs per SM the register budget is sized for
#endif
#define FUSED_RCH 16                         // decoder rows per pass
#define FUSED_MAX_N NB2_FUSED_MAX_NEURONS    // neurons per ensemble (spikes staged in smem)
#define FUSED_MAX_X NB2_FUSED_MAX_INPUT      // total encoder columns per ensemble
#define FUSED_SMALL_N NB2_FUSED_SMALL_NEURONS

// TPE = threads per ensemble (32 or 256); NEMAX = staged neurons per ensemble
template <int TPE, int NEMAX>
__global__ void __launch_bounds__(FUSED_THREADS, FUSED_MIN_BLOCKS)
nb2_ensemble_step_kernel(int n_ens, const int* __restrict__ ens_ids, const int* __restrict__ ens_table,
                         const int* __restrict__ term_table, const int* __restrict__ conn_table,
                         float* data, float dt, float dt_inv) {
  constexpr int GROUPS = FUSED_THREADS / TPE;     // ensembles per CTA
  constexpr int WARPS = TPE / 32;                 // warps per ensemble
  __shared__ __align__(16) float s_spk[GROUPS][NEMAX];
  __shared__ __align__(16) float s_x[GROUPS][FUSED_MAX_X];
  __shared__ float s_red[GROUPS][WARPS][FUSED_RCH];
  __shared__ float s_ae[GROUPS][FUSED_RCH];

  const int grp = threadIdx.x / TPE;
  const int t = threadIdx.x % TPE;
  const int lane = threadIdx.x & 31;
  const int wig = t >> 5;  // warp within group
  const int slot = blockIdx.x * GROUPS + grp;
  const bool active = slot < n_ens;
  const int* e = ens_table + (size_t)(active ? ens_ids[slot] : 0) * E_STRIDE;
  const int n = active ? e[E_N] : 0;
  // 128-bit path: n, every encoder width and every array start are multiples of 4 (set by the host)
  const bool vec = active && (e[E_FLAGS] & 1);

  auto group_sync = [&]() {
    if (TPE == 32) __syncwarp();
    else __syncthreads();
  };

  // ---- stage the input vectors of all encoder terms ----
  const int n_terms = e[E_NTERMS];
  const int* terms = term_table + (size_t)e[E_TERM0] * T_STRIDE;
  if (active) {
    int xoff = 0;
    for (int k = 0; k < n_terms; ++k) {
      const int d = terms[k * T_STRIDE + T_D];
      const float* x = data + terms[k * T_STRIDE + T_X];
      const int xs = terms[k * T_STRIDE + T_XS];
      for (int c = t; c < d; c += TPE) s_x[grp][xoff + c] = x[(size_t)c * xs];
      xoff += d;
    }
  }
  group_sync();

  // ---- phase 1: J = bias + enc . x ; LIF ----
  if (active) {
    const float tau = bits(e[E_TAU]), ref = bits(e[E_REF]), amp = bits(e[E_AMP]);
    const float* bias = data + e[E_BIAS];
    float* V = data + e[E_V];
    float* W = data + e[E_W];
    float* S = e[E_S] >= 0 ? data + e[E_S] : nullptr;
    float* Jout = e[E_J] >= 0 ? data + e[E_J] : nullptr;
    if (vec) {
      // four consecutive neurons per thread: 16 independent 128-bit encoder loads in flight
      const int n4 = n >> 2;
      for (int i4 = t; i4 < n4; i4 += TPE) {
        const int i = i4 << 2;
        float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        int xoff = 0;
        for (int k = 0; k < n_terms; ++k) {
          const int d4 = terms[k * T_STRIDE + T_D] >> 2;
          const float4* rows =
              reinterpret_cast<const float4*>(data + terms[k * T_STRIDE + T_A]) + (size_t)i * d4;
          const float4* xv = reinterpret_cast<const float4*>(&s_x[grp][xoff]);
          for (int c = 0; c < d4; ++c) {
            const float4 x4 = xv[c];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float4 a = __ldg(rows + (size_t)j * d4 + c);
              sum[j] = fmaf(a.x, x4.x, sum[j]);
              sum[j] = fmaf(a.y, x4.y, sum[j]);
              sum[j] = fmaf(a.z, x4.z, sum[j]);
              sum[j] = fmaf(a.w, x4.w, sum[j]);
            }
          }
          xoff += d4 << 2;
        }
        const float4 b4 = *reinterpret_cast<const float4*>(bias + i);
        float4 v4 = *reinterpret_cast<float4*>(V + i);
        float4 w4 = *reinterpret_cast<float4*>(W + i);
        float4 J4, s4;
        J4.x = b4.x + sum[0]; J4.y = b4.y + sum[1]; J4.z = b4.z + sum[2]; J4.w = b4.w + sum[3];
        s4.x = fused_lif(J4.x, v4.x, w4.x, tau, ref, amp, dt, dt_inv);
        s4.y = fused_lif(J4.y, v4.y, w4.y, tau, ref, amp, dt, dt_inv);
        s4.z = fused_lif(J4.z, v4.z, w4.z, tau, ref, amp, dt, dt_inv);
        s4.w = fused_lif(J4.w, v4.w, w4.w, tau, ref, amp, dt, dt_inv);
        *reinterpret_cast<float4*>(V + i) = v4;
        *reinterpret_cast<float4*>(W + i) = w4;
        if (S) *reinterpret_cast<float4*>(S + i) = s4;
        if (Jout) *reinterpret_cast<float4*>(Jout + i) = J4;
        *reinterpret_cast<float4*>(&s_spk[grp][i]) = s4;
      }
    } else
    for (int i = t; i < n; i += TPE) {
      float sum = 0.0f;
      int xoff = 0;
      for (int k = 0; k < n_terms; ++k) {
        const int d = terms[k * T_STRIDE + T_D];
        const int a0 = terms[k * T_STRIDE + T_A];
        const float* row = data + a0 + (size_t)i * d;
        const float* xv = &s_x[grp][xoff];
        if (((d | a0) & 3) == 0) {
          const float4* row4 = reinterpret_cast<const float4*>(row);
          for (int c = 0; c < (d >> 2); ++c) {
            const float4 a = __ldg(row4 + c);
            sum = fmaf(a.x, xv[4 * c + 0], sum);
            sum = fmaf(a.y, xv[4 * c + 1], sum);
            sum = fmaf(a.z, xv[4 * c + 2], sum);
            sum = fmaf(a.w, xv[4 * c + 3], sum);
          }
        } else {
          for (int c = 0; c < d; ++c) sum = fmaf(__ldg(row + c), xv[c], sum);
        }
        xoff += d;
      }
      const float J = bias[i] + sum;
      float v = V[i], w = W[i];
      const float s = fused_lif(J, v, w, tau, ref, amp, dt, dt_inv);
      V[i] = v;
      W[i] = w;
      if (S) S[i] = s;
      if (Jout) Jout[i] = J;
      s_spk[grp][i] = s;
    }
  }
  group_sync();

  // ---- phase 2: decode, synapse, PES ----
  const int n_conn = active ? e[E_NCONN] : 0;
  for (int ci = 0; ci < n_conn; ++ci) {
    const int* c = conn_table + (size_t)(e[E_CONN0] + ci) * C_STRIDE;
    // A run of single-row connections without PES (e.g. scalar edges of a recurrent graph):
    // decode up to FUSED_RCH of them in one pass, one row each, instead of one pass per connection.
    int run = 0;
    while (ci + run < n_conn && run < FUSED_RCH && c[run * C_STRIDE + C_D] == 1 && c[run * C_STRIDE + C_PES] == 0)
      ++run;
    if (run >= 2) {
      float acc[FUSED_RCH];
      int woff[FUSED_RCH];
#pragma unroll
      for (int r = 0; r < FUSED_RCH; ++r) {
        acc[r] = 0.0f;
        woff[r] = c[(r < run ? r : 0) * C_STRIDE + C_W];
      }
      for (int i = t; i < n; i += TPE) {
        const float s = s_spk[grp][i];
#pragma unroll
        for (int r = 0; r < FUSED_RCH; ++r)
          if (r < run) acc[r] = fmaf(data[woff[r] + i], s, acc[r]);
      }
#pragma unroll
      for (int r = 0; r < FUSED_RCH; ++r) {
        float v = acc[r];
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) s_red[grp][wig][r] = v;
      }
      group_sync();
      if (t < run) {
        const int* cr = c + t * C_STRIDE;
        float total = 0.0f;
        for (int w = 0; w < WARPS; ++w) total += s_red[grp][w][t];
        data[cr[C_WEIGHTED]] = total;
        if (cr[C_FILT] >= 0) {
          float* y = data + cr[C_FILT];
          if (cr[C_A0] == 0) *y = bits(cr[C_B0]) * total;
          else *y = bits(cr[C_B0]) * total - bits(cr[C_A0]) * *y;
        }
      }
      group_sync();
      ci += run - 1;
      continue;
    }
    const int d_c = active ? c[C_D] : 0;
    float* Wd = data + c[C_W];
    const bool pes = active && c[C_PES] != 0;
    float* pf = pes ? data + c[C_PF] : nullptr;
    for (int r0 = 0; r0 < d_c; r0 += FUSED_RCH) {
      const int nr = min(FUSED_RCH, d_c - r0);
      if (pes) {
        // alpha * error, formed once per row as in `alpha * aa * xx` (left to right)
        if (t < nr) s_ae[grp][t] = bits(c[C_ALPHA]) * data[c[C_ERR] + r0 + t];
        group_sync();
      }
      float acc[FUSED_RCH];
#pragma unroll
      for (int r = 0; r < FUSED_RCH; ++r) acc[r] = 0.0f;
      if (vec) {
        // 128-bit loads of 8 decoder rows at a time: all loads of a half-pass are issued
        // before the (possibly aliasing) PES stores of the same rows
        const int n4 = n >> 2;
        for (int i4 = t; i4 < n4; i4 += TPE) {
          const float4 s4 = *reinterpret_cast<const float4*>(&s_spk[grp][i4 << 2]);
          float4 p4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          if (pes) p4 = *reinterpret_cast<const float4*>(pf + (i4 << 2));
#pragma unroll
          for (int h = 0; h < FUSED_RCH; h += 8) {
            float4 wv[8];
#pragma unroll
            for (int r = 0; r < 8; ++r)
              if (h + r < nr) wv[r] = *(reinterpret_cast<const float4*>(Wd + (size_t)(r0 + h + r) * n) + i4);
#pragma unroll
            for (int r = 0; r < 8; ++r) {
              if (h + r < nr) {
                float a = acc[h + r];
                a = fmaf(wv[r].x, s4.x, a);
                a = fmaf(wv[r].y, s4.y, a);
                a = fmaf(wv[r].z, s4.z, a);
                a = fmaf(wv[r].w, s4.w, a);
                acc[h + r] = a;
                if (pes) {
                  const float ae = s_ae[grp][h + r];
                  float4 o;
                  o.x = wv[r].x + ae * p4.x;
                  o.y = wv[r].y + ae * p4.y;
                  o.z = wv[r].z + ae * p4.z;
                  o.w = wv[r].w + ae * p4.w;
                  *(reinterpret_cast<float4*>(Wd + (size_t)(r0 + h + r) * n) + i4) = o;
                }
              }
            }
          }
        }
      } else
      for (int i = t; i < n; i += TPE) {
        const float s = s_spk[grp][i];
        const float p = pes ? pf[i] : 0.0f;
#pragma unroll
        for (int r = 0; r < FUSED_RCH; ++r) {
          if (r < nr) {
            float* wp = Wd + (size_t)(r0 + r) * n + i;
            const float w = *wp;
            acc[r] = fmaf(w, s, acc[r]);
            if (pes) *wp = w + s_ae[grp][r] * p;
          }
        }
      }
      // fixed-order reduction: lanes (xor tree), then warps in index order
#pragma unroll
      for (int r = 0; r < FUSED_RCH; ++r) {
        float v = acc[r];
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) s_red[grp][wig][r] = v;
      }
      group_sync();
      if (active && t < nr) {
        float total = 0.0f;
        for (int w = 0; w < WARPS; ++w) total += s_red[grp][w][t];
        data[c[C_WEIGHTED] + r0 + t] = total;
        if (c[C_FILT] >= 0) {
          float* y = data + c[C_FILT] + r0 + t;
          // plan_linearfilter fast path (clra_nonlinearities.py:657-660)
          if (c[C_A0] == 0) *y = bits(c[C_B0]) * total;
          else *y = bits(c[C_B0]) * total - bits(c[C_A0]) * *y;
        }
      }
      group_sync();
    }
    if (pes) {
      const float b0 = bits(c[C_PFB0]), a0 = bits(c[C_PFA0]);
      for (int i = t; i < n; i += TPE) pf[i] = b0 * s_spk[grp][i] - a0 * pf[i];
    }
  }
}

extern "C" int nb2_ensemble_step(void* stream, int n_large, const int* large_ids, int n_small,
                                 const int* small_ids, const int* ens_table, const int* term_table,
                                 const int* conn_table, float* data, double dt) {
  NB2_REQUIRE(ens_table && term_table && conn_table && data, "null pointer");
  NB2_REQUIRE(dt > 0, "dt");
  cudaStream_t s = nb2_stream(stream);
  const float dtf = (float)dt;
  const float dt_inv = (float)(1.0 / dt);
  if (n_large > 0) {
    NB2_REQUIRE(large_ids != NULL, "large_ids");
    nb2_ensemble_step_kernel<256, FUSED_MAX_N><<<n_large, FUSED_THREADS, 0, s>>>(
        n_large, large_ids, ens_table, term_table, conn_table, data, dtf, dt_inv);
    NB2_LAUNCH_CHECK();
  }
  if (n_small > 0) {
    NB2_REQUIRE(small_ids != NULL, "small_ids");
    const int blocks = (n_small + 7) / 8;
    nb2_ensemble_step_kernel<32, FUSED_SMALL_N><<<blocks, FUSED_THREADS, 0, s>>>(
        n_small, small_ids, ens_table, term_table, conn_table, data, dtf, dt_inv);
    NB2_LAUNCH_CHECK();
  }
  return NB2_OK;
}
