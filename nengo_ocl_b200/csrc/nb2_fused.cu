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
// warp for small ones (8 per CTA).  All dot products are summed in the order of
// the reference's block GEMV (nb2_blockdot.cuh: tiles of 128 columns, four
// column-strided partial sums per tile, no fused multiply-add), so J and the
// decoded values are bit-identical to that kernel.  Phase 1: each thread computes
// J for its neurons (x staged in shared memory, encoder rows read with 128-bit
// loads when aligned), runs the LIF update (operation order of the reference
// kernel, -fmad=false, expm1 / log1p correctly rounded) and keeps the spikes in
// shared memory.  Phase 2: up to 16 decoder rows at a time (rows of one
// connection, or one row each of a run of single-row connections); every thread
// owns one partial sum of one (row, tile), walks it in order and applies the PES
// update to the same elements; one thread per row then combines the partial sums
// tile by tile and runs the synapse.  All index tables are int32 element offsets
// into the one packed signal buffer.
#include "nb2_common.cuh"
#include "nb2_blockdot.cuh"
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

// One encoder row (d columns, contiguous) times x (shared memory), added tile by tile to total.
__device__ __forceinline__ float fused_row_dot(const float* __restrict__ row, const float* __restrict__ xv, int d,
                                               bool vec, float total) {
  for (int c0 = 0; c0 < d; c0 += 128) {
    const int wt = min(128, d - c0);
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    int c = 0;
    if (vec) {
      const float4* row4 = reinterpret_cast<const float4*>(row + c0);
      const float4* x4 = reinterpret_cast<const float4*>(xv + c0);
      for (; c + 4 <= wt; c += 4) {
        const float4 a = __ldg(row4 + (c >> 2));
        const float4 x = x4[c >> 2];
        s0 = bd_add(s0, bd_mul(a.x, x.x));
        s1 = bd_add(s1, bd_mul(a.y, x.y));
        s2 = bd_add(s2, bd_mul(a.z, x.z));
        s3 = bd_add(s3, bd_mul(a.w, x.w));
      }
    } else {
      for (; c + 4 <= wt; c += 4) {
        s0 = bd_add(s0, bd_mul(__ldg(row + c0 + c + 0), xv[c0 + c + 0]));
        s1 = bd_add(s1, bd_mul(__ldg(row + c0 + c + 1), xv[c0 + c + 1]));
        s2 = bd_add(s2, bd_mul(__ldg(row + c0 + c + 2), xv[c0 + c + 2]));
        s3 = bd_add(s3, bd_mul(__ldg(row + c0 + c + 3), xv[c0 + c + 3]));
      }
    }
    if (c < wt) s0 = bd_add(s0, bd_mul(__ldg(row + c0 + c), xv[c0 + c]));
    if (c + 1 < wt) s1 = bd_add(s1, bd_mul(__ldg(row + c0 + c + 1), xv[c0 + c + 1]));
    if (c + 2 < wt) s2 = bd_add(s2, bd_mul(__ldg(row + c0 + c + 2), xv[c0 + c + 2]));
    total = bd_add(total, bd_tile(s0, s1, s2, s3));
  }
  return total;
}

// TPE = threads per ensemble (32 or 256); NEMAX = staged neurons per ensemble
template <int TPE, int NEMAX>
__global__ void __launch_bounds__(FUSED_THREADS, FUSED_MIN_BLOCKS)
nb2_ensemble_step_kernel(int n_ens, const int* __restrict__ ens_ids, const int* __restrict__ ens_table,
                         const int* __restrict__ term_table, const int* __restrict__ conn_table,
                         float* data, float dt, float dt_inv) {
  nb2_pdl_enter();
  constexpr int GROUPS = FUSED_THREADS / TPE;     // ensembles per CTA
  constexpr int CHAINS = FUSED_RCH * ((NEMAX + 127) / 128) * 4;  // partial sums of one pass
  __shared__ __align__(16) float s_spk[GROUPS][NEMAX];
  __shared__ __align__(16) float s_x[GROUPS][FUSED_MAX_X];
  __shared__ float s_chain[GROUPS][CHAINS];
  __shared__ float s_ae[GROUPS][FUSED_RCH];

  const int grp = threadIdx.x / TPE;
  const int t = threadIdx.x % TPE;
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

  // ---- phase 1: J = ((bias + enc_0 . x_0) + enc_1 . x_1) ... ; LIF ----
  if (active) {
    const float tau = bits(e[E_TAU]), ref = bits(e[E_REF]), amp = bits(e[E_AMP]);
    const float em1_dt = bits(e[E_EM1]);
    const float* bias = data + e[E_BIAS];
    float* V = data + e[E_V];
    float* W = data + e[E_W];
    float* S = e[E_S] >= 0 ? data + e[E_S] : nullptr;
    float* Jout = e[E_J] >= 0 ? data + e[E_J] : nullptr;
    for (int i = t; i < n; i += TPE) {
      float J = bias[i];
      int xoff = 0;
      for (int k = 0; k < n_terms; ++k) {
        const int d = terms[k * T_STRIDE + T_D];
        const int a0 = terms[k * T_STRIDE + T_A];
        J = fused_row_dot(data + a0 + (size_t)i * d, &s_x[grp][xoff], d, vec || ((d | a0 | xoff) & 3) == 0, J);
        xoff += d;
      }
      float v = V[i], w = W[i];
      const float s = fused_lif(J, v, w, tau, ref, amp, dt, dt_inv, em1_dt);
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
  const int ntile = (n + 127) >> 7;
  const int per_row = ntile * 4;  // partial sums of one row
  const float* spk = s_spk[grp];
  for (int ci = 0; ci < n_conn;) {
    const int* c = conn_table + (size_t)(e[E_CONN0] + ci) * C_STRIDE;
    // A run of single-row connections without PES (e.g. the scalar edges of a recurrent graph) is
    // decoded in one pass, one row each, instead of one pass per connection.
    int run = 0;
    while (ci + run < n_conn && run < FUSED_RCH && c[run * C_STRIDE + C_D] == 1 && c[run * C_STRIDE + C_PES] == 0)
      ++run;
    const bool single = run >= 2;
    const int d_c = single ? run : c[C_D];
    const bool pes = !single && c[C_PES] != 0;
    float* pf = pes ? data + c[C_PF] : nullptr;
    for (int r0 = 0; r0 < d_c; r0 += FUSED_RCH) {
      const int nr = min(FUSED_RCH, d_c - r0);
      if (pes) {
        // alpha * error, formed once per row as in `alpha * aa * xx` (left to right)
        if (t < nr) s_ae[grp][t] = bits(c[C_ALPHA]) * data[c[C_ERR] + r0 + t];
        group_sync();
      }
      for (int u = t; u < nr * per_row; u += TPE) {
        const int r = u / per_row, rem = u - r * per_row;
        const int tile = rem >> 2, j = rem & 3;
        float* w = single ? data + c[r * C_STRIDE + C_W] : data + c[C_W] + (size_t)(r0 + r) * n;
        const int end = min(n, (tile + 1) << 7);
        float acc = 0.0f;
        if (pes) {
          const float ae = s_ae[grp][r];
#pragma unroll 4
          for (int i = (tile << 7) + j; i < end; i += 4) {
            const float wv = w[i];
            acc = bd_add(acc, bd_mul(wv, spk[i]));
            w[i] = wv + ae * pf[i];
          }
        } else {
#pragma unroll 8
          for (int i = (tile << 7) + j; i < end; i += 4) acc = bd_add(acc, bd_mul(w[i], spk[i]));
        }
        s_chain[grp][u] = acc;
      }
      group_sync();
      if (active && t < nr) {
        const float* ch = &s_chain[grp][t * per_row];
        float total = 0.0f;
        for (int tile = 0; tile < ntile; ++tile)
          total = bd_add(total, bd_tile(ch[4 * tile], ch[4 * tile + 1], ch[4 * tile + 2], ch[4 * tile + 3]));
        const int* cr = single ? c + t * C_STRIDE : c;
        const int row = single ? 0 : r0 + t;
        data[cr[C_WEIGHTED] + row] = total;
        if (cr[C_FILT] >= 0) {
          float* y = data + cr[C_FILT] + row;
          // plan_linearfilter fast path (clra_nonlinearities.py:657-660)
          if (cr[C_A0] == 0) *y = bits(cr[C_B0]) * total;
          else *y = bits(cr[C_B0]) * total - bits(cr[C_A0]) * *y;
        }
      }
      group_sync();
    }
    if (pes) {
      const float b0 = bits(c[C_PFB0]), a0 = bits(c[C_PFA0]);
      for (int i = t; i < n; i += TPE) pf[i] = b0 * spk[i] - a0 * pf[i];
    }
    ci += single ? run : 1;
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
    nb2_launch(nb2_ensemble_step_kernel<256, FUSED_MAX_N>, dim3(n_large), dim3(FUSED_THREADS), 0, s, n_large, large_ids, ens_table, term_table, conn_table, data, dtf, dt_inv);
    NB2_LAUNCH_CHECK();
  }
  if (n_small > 0) {
    NB2_REQUIRE(small_ids != NULL, "small_ids");
    const int blocks = (n_small + 7) / 8;
    nb2_launch(nb2_ensemble_step_kernel<32, FUSED_SMALL_N>, dim3(blocks), dim3(FUSED_THREADS), 0, s, n_small, small_ids, ens_table, term_table, conn_table, data, dtf, dt_inv);
    NB2_LAUNCH_CHECK();
  }
  return NB2_OK;
}
