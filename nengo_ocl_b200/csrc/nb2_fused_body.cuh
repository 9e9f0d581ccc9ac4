// Body of the fused ensemble step (encoder GEMV + LIF + decoder GEMV + synapse + PES)
// as a device function over a virtual block index: nb2_fused.cu launches it as its own
// kernel (virtual block = blockIdx.x), nb2_step_loop.cu runs it as one phase of the
// persistent step loop.  See nb2_fused.cu for the operators it replaces and the
// summation order.  NC: encoder rows may be read through the non-coherent path
// (only valid when nothing inside the same kernel launch writes them).
#pragma once
#include "nb2_common.cuh"
#include "nb2_blockdot.cuh"
#include "nb2_fused_common.cuh"
#include "../../include/nengo_b200.h"

#define FUSED_THREADS 256
#ifndef FUSED_MIN_BLOCKS
#define FUSED_MIN_BLOCKS 4  // CTAs per SM the register budget is sized for (the populations left to these kernels are latency-bound)
#endif
#ifndef FUSED_MIN_BLOCKS_SMALL
#define FUSED_MIN_BLOCKS_SMALL 4  // the warp-per-ensemble variant is latency-bound: more resident warps
#endif
#define FUSED_RCH 16                         // decoder rows per pass
#define FUSED_MAX_N NB2_FUSED_MAX_NEURONS    // neurons per ensemble (spikes staged in smem)
#define FUSED_MAX_X NB2_FUSED_MAX_INPUT      // total encoder columns per ensemble
#define FUSED_SMALL_N NB2_FUSED_SMALL_NEURONS
#define FUSED_CONN_STAGED 16  // connection-table rows per ensemble prefetched into shared memory
#ifndef FUSED_PREFETCH_BYTES
#define FUSED_PREFETCH_BYTES 4096  // decoder matrices up to this size are prefetched into L1
#endif
#define FUSED_BATCH 4         // neurons per thread whose loads are issued together

template <int V> struct FusedInt { static constexpr int value = V; };

template <bool NC> __device__ __forceinline__ float fused_ld(const float* p) { return NC ? __ldg(p) : *p; }
template <bool NC> __device__ __forceinline__ float4 fused_ld4(const float4* p) { return NC ? __ldg(p) : *p; }

// One encoder row (d columns, contiguous) times x (shared memory), added tile by tile to total.
template <bool NC>
__device__ __forceinline__ float fused_row_dot(const float* row, const float* xv, int d,
                                               bool vec, float total) {
  for (int c0 = 0; c0 < d; c0 += 128) {
    const int wt = min(128, d - c0);
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    int c = 0;
    if (vec) {
      const float4* row4 = reinterpret_cast<const float4*>(row + c0);
      const float4* x4 = reinterpret_cast<const float4*>(xv + c0);
      for (; c + 4 <= wt; c += 4) {
        const float4 a = fused_ld4<NC>(row4 + (c >> 2));
        const float4 x = x4[c >> 2];
        s0 = bd_add(s0, bd_mul(a.x, x.x));
        s1 = bd_add(s1, bd_mul(a.y, x.y));
        s2 = bd_add(s2, bd_mul(a.z, x.z));
        s3 = bd_add(s3, bd_mul(a.w, x.w));
      }
    } else {
      for (; c + 4 <= wt; c += 4) {
        s0 = bd_add(s0, bd_mul(fused_ld<NC>(row + c0 + c + 0), xv[c0 + c + 0]));
        s1 = bd_add(s1, bd_mul(fused_ld<NC>(row + c0 + c + 1), xv[c0 + c + 1]));
        s2 = bd_add(s2, bd_mul(fused_ld<NC>(row + c0 + c + 2), xv[c0 + c + 2]));
        s3 = bd_add(s3, bd_mul(fused_ld<NC>(row + c0 + c + 3), xv[c0 + c + 3]));
      }
    }
    if (c < wt) s0 = bd_add(s0, bd_mul(fused_ld<NC>(row + c0 + c), xv[c0 + c]));
    if (c + 1 < wt) s1 = bd_add(s1, bd_mul(fused_ld<NC>(row + c0 + c + 1), xv[c0 + c + 1]));
    if (c + 2 < wt) s2 = bd_add(s2, bd_mul(fused_ld<NC>(row + c0 + c + 2), xv[c0 + c + 2]));
    total = bd_add(total, bd_tile(s0, s1, s2, s3));
  }
  return total;
}

// Shared memory of one CTA of the fused step (TPE = threads per ensemble, 32 or 256;
// NEMAX = staged neurons per ensemble).
template <int TPE, int NEMAX>
struct FusedSmem {
  static constexpr int GROUPS = FUSED_THREADS / TPE;                    // ensembles per CTA
  static constexpr int CHAINS = FUSED_RCH * ((NEMAX + 127) / 128) * 4;  // partial sums of one pass
  float spk[GROUPS][NEMAX];
  float x[GROUPS][FUSED_MAX_X];
  float chain[GROUPS][CHAINS];
  float ae[GROUPS][FUSED_RCH];
  int conn[GROUPS][FUSED_CONN_STAGED * C_STRIDE];  // first rows of the ensemble's connection table
};

// One virtual block: FUSED_THREADS / TPE ensembles.  `smem` is 16-byte aligned and holds a
// FusedSmem<TPE, NEMAX>; every thread of the CTA calls this (it synchronises the CTA).
template <int TPE, int NEMAX, bool NC>
__device__ __forceinline__ void nb2_ensemble_step_body(void* smem, int vblock, int n_ens, const int* __restrict__ ens_ids,
                                                       const int* __restrict__ ens_table,
                                                       const int* __restrict__ term_table,
                                                       const int* __restrict__ conn_table, float* data, float dt,
                                                       float dt_inv) {
  typedef FusedSmem<TPE, NEMAX> Smem;
  constexpr int GROUPS = Smem::GROUPS;
  Smem& sm = *reinterpret_cast<Smem*>(smem);
  float(*s_spk)[NEMAX] = sm.spk;
  float(*s_x)[FUSED_MAX_X] = sm.x;
  float(*s_chain)[Smem::CHAINS] = sm.chain;
  float(*s_ae)[FUSED_RCH] = sm.ae;

  const int grp = threadIdx.x / TPE;
  int* s_conn = sm.conn[grp];
  const int t = threadIdx.x % TPE;
  const int slot = vblock * GROUPS + grp;
  const bool active = slot < n_ens;
  const int* e = ens_table + (size_t)(active ? __ldg(&ens_ids[slot]) : 0) * E_STRIDE;
  const int n = active ? __ldg(&e[E_N]) : 0;
  // 128-bit path: n, every encoder width and every array start are multiples of 4 (set by the host)
  const bool vec = active && (__ldg(&e[E_FLAGS]) & 1);

  auto group_sync = [&]() {
    if (TPE == 32) __syncwarp();
    else __syncthreads();
  };

  // ---- stage the input vectors of all encoder terms ----
  const int n_terms = __ldg(&e[E_NTERMS]);
  const int* terms = term_table + (size_t)__ldg(&e[E_TERM0]) * T_STRIDE;
  const int n_conn = active ? __ldg(&e[E_NCONN]) : 0;
  const int* conn_rows = conn_table + (size_t)__ldg(&e[E_CONN0]) * C_STRIDE;
  if (active) {
    // the connection rows are needed only after the neuron update: fetch them now, so that their
    // latency overlaps phase 1 (consumed after the barrier that ends phase 1)
    for (int q = t; q < min(n_conn, FUSED_CONN_STAGED) * C_STRIDE; q += TPE) s_conn[q] = __ldg(&conn_rows[q]);
    int xoff = 0;
    for (int k = 0; k < n_terms; ++k) {
      const int d = __ldg(&terms[k * T_STRIDE + T_D]);
      const float* x = data + __ldg(&terms[k * T_STRIDE + T_X]);
      const int xs = __ldg(&terms[k * T_STRIDE + T_XS]);
      for (int c = t; c < d; c += TPE) s_x[grp][xoff + c] = x[(size_t)c * xs];
      xoff += d;
    }
  }
  group_sync();
  // row i of this ensemble's connection table (generic pointer: shared or global memory)
  auto conn_row = [&](int i) -> const int* {
    return i < FUSED_CONN_STAGED ? s_conn + i * C_STRIDE : conn_rows + (size_t)i * C_STRIDE;
  };
  // Small decoder matrices (the many one-row connections of a graph model) are asked into L1 now:
  // they are needed only after the neuron update, whose latency then hides the fetch.
  for (int k = 0; k < min(n_conn, FUSED_CONN_STAGED); ++k) {
    const int* c = s_conn + k * C_STRIDE;
    const int bytes = c[C_D] * n * 4;
    if (bytes > FUSED_PREFETCH_BYTES) continue;
    const char* base = reinterpret_cast<const char*>(data + c[C_W]);
    for (int off = t * 128; off < bytes + 124; off += TPE * 128)
      asm volatile("prefetch.global.L1 [%0];" ::"l"(base + min(off, bytes - 4)));
    if (t == TPE - 1 && c[C_FILT] >= 0) asm volatile("prefetch.global.L1 [%0];" ::"l"(data + c[C_FILT]));
  }

  // ---- phase 1: J = ((bias + enc_0 . x_0) + enc_1 . x_1) ... ; LIF ----
  if (active) {
    const float tau = bits(__ldg(&e[E_TAU])), ref = bits(__ldg(&e[E_REF])), amp = bits(__ldg(&e[E_AMP]));
    const float em1_dt = bits(__ldg(&e[E_EM1]));
    const float* bias = data + __ldg(&e[E_BIAS]);
    float* V = data + __ldg(&e[E_V]);
    float* W = data + __ldg(&e[E_W]);
    float* S = __ldg(&e[E_S]) >= 0 ? data + __ldg(&e[E_S]) : nullptr;
    float* Jout = __ldg(&e[E_J]) >= 0 ? data + __ldg(&e[E_J]) : nullptr;
    // NB neurons per thread at a time (1, 2 or FUSED_BATCH, whichever covers the population with
    // the fewest idle slots): all their loads are issued before the first use, so a thread with
    // several neurons pays the memory latency once per batch
    auto phase1 = [&](auto nb_tag) {
      constexpr int NB = decltype(nb_tag)::value;
      for (int i0 = t; i0 < n; i0 += NB * TPE) {
        float J[NB], v[NB], w[NB], s[NB];
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          const int i = i0 + j * TPE;
          const bool ok = i < n;
          J[j] = ok ? bias[i] : 0.0f;
          v[j] = ok ? V[i] : 0.0f;
          w[j] = ok ? W[i] : 0.0f;
        }
        int xoff = 0;
        for (int k = 0; k < n_terms; ++k) {
          const int d = __ldg(&terms[k * T_STRIDE + T_D]);
          const int a0 = __ldg(&terms[k * T_STRIDE + T_A]);
          const bool v4 = vec || ((d | a0 | xoff) & 3) == 0;
#pragma unroll
          for (int j = 0; j < NB; ++j) {
            const int i = i0 + j * TPE;
            if (i < n) J[j] = fused_row_dot<NC>(data + a0 + (size_t)i * d, &s_x[grp][xoff], d, v4, J[j]);
          }
          xoff += d;
        }
        fused_lifN<NB>(J, v, w, s, tau, ref, amp, dt, dt_inv, em1_dt);
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          const int i = i0 + j * TPE;
          if (i < n) {
            V[i] = v[j];
            W[i] = w[j];
            if (S) S[i] = s[j];
            if (Jout) Jout[i] = J[j];
            s_spk[grp][i] = s[j];
          }
        }
      }
    };
    if (n <= TPE) phase1(FusedInt<1>());
    else if (n <= 2 * TPE) phase1(FusedInt<2>());
    else phase1(FusedInt<FUSED_BATCH>());
  }
  group_sync();

  // ---- phase 2: decode, synapse, PES ----
  const int ntile = (n + 127) >> 7;
  const int per_row = ntile * 4;  // partial sums of one row
  const float* spk = s_spk[grp];
  for (int ci = 0; ci < n_conn;) {
    const int* c = conn_row(ci);
    // A run of single-row connections without PES (e.g. the scalar edges of a recurrent graph) is
    // decoded in one pass, one row each, instead of one pass per connection.
    int run = 0;
    while (ci + run < n_conn && run < FUSED_RCH && conn_row(ci + run)[C_D] == 1 && conn_row(ci + run)[C_PES] == 0)
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
        float* w = single ? data + conn_row(ci + r)[C_W] : data + c[C_W] + (size_t)(r0 + r) * n;
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
        const int* cr = single ? conn_row(ci + t) : c;
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

