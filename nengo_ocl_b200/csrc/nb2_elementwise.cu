// Elementwise ragged kernels: clock, reset, copy, sliced copy, elementwise
// increment (incl. the PES outer product), linear filters, probes and table
// playback.  Each kernel consumes the index tables that the matching
// reference plan function uploads (nengo_ocl/clra_nonlinearities.py), so the
// host-side plans are interchangeable.  This translation unit is compiled
// with -fmad=false: every a*b+c below is a separate multiply and add, as in
// the CPU restatement the results are checked against.
#include <mutex>
#include "nb2_common.cuh"
#include "nb2_phase_bodies.cuh"
#include "../../include/nengo_b200.h"

// ---- plan_timeupdate (clra_nonlinearities.py:119-133) ----------------------
__global__ void nb2_timeupdate_kernel(float* step, float* time, double dt) {
  nb2_pdl_enter();
  const Nb2TimeupdateArgs a = {step, time, dt};
  nb2_timeupdate_body(a, 0, 0);
}

extern "C" int nb2_timeupdate(void* stream, float* step, float* time, double dt) {
  NB2_REQUIRE(step && time, "null pointer");
  nb2_launch(nb2_timeupdate_kernel, dim3(1), dim3(1), 0, nb2_stream(stream), step, time, dt);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}

// ---- plan_reset (:154-172) --------------------------------------------------
__global__ void nb2_reset_kernel(int n_blocks, const float* __restrict__ values,
                                 const int* __restrict__ sizes, const int* __restrict__ starts,
                                 float* Y) {
  nb2_pdl_enter();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = t >> 4;
  const int i = t & 15;
  if (n < n_blocks && i < sizes[n]) Y[starts[n] + i] = values[n];
}

extern "C" int nb2_reset(void* stream, int n_blocks, const float* values, const int* sizes,
                         const int* starts, float* Y) {
  if (n_blocks == 0) return NB2_OK;
  NB2_REQUIRE(values && sizes && starts && Y, "null pointer");
  const long long threads = (long long)n_blocks * 16;
  nb2_launch(nb2_reset_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, nb2_stream(stream), n_blocks, values, sizes, starts, Y);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}

// ---- plan_copy (:225-262) ---------------------------------------------------
__global__ void nb2_copy_kernel(int inc_mode, const int* __restrict__ incdata,
                                const int* __restrict__ offsets, const int* __restrict__ shape0s,
                                const int* __restrict__ shape1s, const int* __restrict__ Xstride0s,
                                const int* __restrict__ Xstarts, const float* X,
                                const int* __restrict__ Ystride0s, const int* __restrict__ Ystarts,
                                float* Y) {
  nb2_pdl_enter();
  const int n = blockIdx.x;
  const int ij = threadIdx.x + offsets[n];
  const int shape1 = shape1s[n];
  const int i = ij / shape1;
  const int j = ij - i * shape1;
  if (i >= shape0s[n]) return;
  const int xo = Xstarts[n] + i * Xstride0s[n] + j;
  const int yo = Ystarts[n] + i * Ystride0s[n] + j;
  const bool inc = inc_mode == 1 || (inc_mode == 2 && incdata[n]);
  if (inc) Y[yo] += X[xo];
  else Y[yo] = X[xo];
}

extern "C" int nb2_copy(void* stream, int n_blocks, int inc_mode, const int* incdata,
                        const int* offsets, const int* shape0s, const int* shape1s,
                        const int* Xstride0s, const int* Xstarts, const float* X,
                        const int* Ystride0s, const int* Ystarts, float* Y) {
  if (n_blocks == 0) return NB2_OK;
  NB2_REQUIRE(offsets && shape0s && shape1s && Xstride0s && Xstarts && X && Ystride0s && Ystarts && Y,
              "null pointer");
  NB2_REQUIRE(inc_mode != 2 || incdata, "incdata required for inc_mode 2");
  nb2_launch(nb2_copy_kernel, dim3(n_blocks), dim3(256), 0, nb2_stream(stream), inc_mode, incdata, offsets, shape0s, shape1s,
                                                           Xstride0s, Xstarts, X, Ystride0s, Ystarts, Y);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}

// ---- plan_slicedcopy (:321-364) ---------------------------------------------
__global__ void nb2_slicedcopy_kernel(int n_blocks, int inc_mode, const int* __restrict__ incdata,
                                      const int* __restrict__ Xstride0s,
                                      const int* __restrict__ Xstarts, const float* X,
                                      const int* __restrict__ Ystride0s,
                                      const int* __restrict__ Ystarts, float* Y,
                                      const int* __restrict__ Isizes,
                                      const int* __restrict__ XIstarts,
                                      const int* __restrict__ XIdata,
                                      const int* __restrict__ YIstarts,
                                      const int* __restrict__ YIdata) {
  nb2_pdl_enter();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = t >> 4;
  const int i = t & 15;
  if (n >= n_blocks || i >= Isizes[n]) return;
  const float* a = X + Xstarts[n];
  float* b = Y + Ystarts[n];
  const int ai = XIdata[XIstarts[n] + i] * Xstride0s[n];
  const int bi = YIdata[YIstarts[n] + i] * Ystride0s[n];
  const bool inc = inc_mode == 1 || (inc_mode == 2 && incdata[n]);
  if (inc) b[bi] += a[ai];
  else b[bi] = a[ai];
}

extern "C" int nb2_slicedcopy(void* stream, int n_blocks, int inc_mode, const int* incdata,
                              const int* Xstride0s, const int* Xstarts, const float* X,
                              const int* Ystride0s, const int* Ystarts, float* Y, const int* Isizes,
                              const int* XIstarts, const int* XIdata, const int* YIstarts,
                              const int* YIdata) {
  if (n_blocks == 0) return NB2_OK;
  NB2_REQUIRE(Xstride0s && Xstarts && X && Ystride0s && Ystarts && Y && Isizes && XIstarts && XIdata &&
                  YIstarts && YIdata,
              "null pointer");
  NB2_REQUIRE(inc_mode != 2 || incdata, "incdata required for inc_mode 2");
  const long long threads = (long long)n_blocks * 16;
  nb2_launch(nb2_slicedcopy_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, nb2_stream(stream), n_blocks, inc_mode, incdata, Xstride0s, Xstarts, X, Ystride0s, Ystarts, Y, Isizes, XIstarts, XIdata,
      YIstarts, YIdata);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}

// ---- plan_elementwise_inc (:449-525) ----------------------------------------
__device__ __forceinline__ float nb2_get_element(const float* data, int shape0, int shape1, int stride0,
                                                 int i, int j) {
  if (shape0 == 1 && shape1 == 1) return data[0];
  if (shape0 == 1) return data[j];
  if (shape1 == 1) return data[i * stride0];
  return data[i * stride0 + j];
}

__global__ void nb2_elementwise_inc_kernel(
    int outer, int inc, const float* __restrict__ alphas, const int* __restrict__ offsets,
    const int* __restrict__ Ashape0s, const int* __restrict__ Ashape1s,
    const int* __restrict__ Astride0s, const int* __restrict__ Astarts, const float* A,
    const int* __restrict__ Xshape0s, const int* __restrict__ Xshape1s,
    const int* __restrict__ Xstride0s, const int* __restrict__ Xstarts, const float* X,
    const int* __restrict__ Yshape0s, const int* __restrict__ Yshape1s,
    const int* __restrict__ Ystride0s, const int* __restrict__ Ystarts, float* Y) {
  nb2_pdl_enter();
  const int n = blockIdx.x;
  const int ij = threadIdx.x + offsets[n];
  const float* a = A + Astarts[n];
  const float* x = X + Xstarts[n];
  float* y = Y + Ystarts[n];
  const int Ystride0 = Ystride0s[n];
  const int Yshape0 = Yshape0s[n];
  const int Yshape1 = Yshape1s[n];
  const int i = ij / Yshape1;
  const int j = ij - i * Yshape1;
  if (i >= Yshape0) return;
  float aa, xx;
  if (outer) {
    aa = nb2_get_element(a, Ashape0s[n], 1, Astride0s[n], i, 0);
    xx = nb2_get_element(x, Xshape0s[n], 1, Xstride0s[n], j, 0);
  } else {
    aa = nb2_get_element(a, Ashape0s[n], Ashape1s[n], Astride0s[n], i, j);
    xx = nb2_get_element(x, Xshape0s[n], Xshape1s[n], Xstride0s[n], i, j);
  }
  const float alpha = alphas ? alphas[n] : 1.0f;
  const float v = alpha * aa * xx;
  if (inc) y[i * Ystride0 + j] += v;
  else y[i * Ystride0 + j] = v;
}

extern "C" int nb2_elementwise_inc(void* stream, int n_blocks, int outer, int inc, const float* alphas,
                                   const int* offsets, const int* Ashape0s, const int* Ashape1s,
                                   const int* Astride0s, const int* Astarts, const float* A,
                                   const int* Xshape0s, const int* Xshape1s, const int* Xstride0s,
                                   const int* Xstarts, const float* X, const int* Yshape0s,
                                   const int* Yshape1s, const int* Ystride0s, const int* Ystarts,
                                   float* Y) {
  if (n_blocks == 0) return NB2_OK;
  NB2_REQUIRE(offsets && Ashape0s && Ashape1s && Astride0s && Astarts && A && Xshape0s && Xshape1s &&
                  Xstride0s && Xstarts && X && Yshape0s && Yshape1s && Ystride0s && Ystarts && Y,
              "null pointer");
  nb2_launch(nb2_elementwise_inc_kernel, dim3(n_blocks), dim3(256), 0, nb2_stream(stream), outer, inc, alphas, offsets, Ashape0s, Ashape1s, Astride0s, Astarts, A, Xshape0s, Xshape1s, Xstride0s,
      Xstarts, X, Yshape0s, Yshape1s, Ystride0s, Ystarts, Y);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}

// ---- plan_linearfilter (:604-711) -------------------------------------------
__global__ void nb2_linearfilter_kernel(
    int uses_buf, const int* __restrict__ offsets, const int* __restrict__ shape0s,
    const int* __restrict__ shape1s, const int* __restrict__ Xstride0s,
    const int* __restrict__ Xstride1s, const int* __restrict__ Xstarts, const float* x,
    const int* __restrict__ Ystride0s, const int* __restrict__ Ystride1s,
    const int* __restrict__ Ystarts, float* y, const int* __restrict__ Ashape0s,
    const int* __restrict__ Astarts, const float* __restrict__ Adata,
    const int* __restrict__ Bshape0s, const int* __restrict__ Bstarts,
    const float* __restrict__ Bdata, const int* __restrict__ Xbufstarts, float* Xbufdata,
    const int* __restrict__ Ybufstarts, float* Ybufdata, const int* __restrict__ Xbufpos,
    const int* __restrict__ Ybufpos) {
  nb2_pdl_enter();
  const int k = blockIdx.x;
  const int ij = threadIdx.x + offsets[k];
  const int shape0 = shape0s[k];
  const int shape1 = shape1s[k];
  const int i = ij / shape1;
  const int j = ij - i * shape1;
  if (i >= shape0) return;
  const int xij = Xstarts[k] + i * Xstride0s[k] + j * Xstride1s[k];
  const int yij = Ystarts[k] + i * Ystride0s[k] + j * Ystride1s[k];
  const int na = Ashape0s[k];
  const int nb = Bshape0s[k];
  const float* a = Adata + Astarts[k];
  const float* b = Bdata + Bstarts[k];

  if (na == 0 && nb == 1) {
    y[yij] = b[0] * x[xij];
  } else if (na == 1 && nb == 1) {
    y[yij] = b[0] * x[xij] - a[0] * y[yij];
  } else if (uses_buf) {
    float* xbuf = Xbufdata + Xbufstarts[k];
    float* ybuf = Ybufdata + Ybufstarts[k];
    const int ix = Xbufpos[k];
    const int iy = Ybufpos[k];
    const int iy1 = (iy > 0) ? iy - 1 : na - 1;
    const int size = shape0 * shape1;
    float yi = b[0] * x[xij];
    if (nb > 1) {
      xbuf[ix * size + ij] = x[xij];
      for (int p = 1; p < nb; p++) yi += b[p] * xbuf[((ix + p) % nb) * size + ij];
    }
    if (na > 0) {
      yi -= a[0] * y[yij];
      if (na > 1) {
        for (int p = 1; p < na; p++) yi -= a[p] * ybuf[((iy + p) % na) * size + ij];
        ybuf[iy1 * size + ij] = yi;
      }
    }
    y[yij] = yi;
  }
}

__global__ void nb2_linearfilter_inc_kernel(int n, const int* __restrict__ Ashape0s,
                                            const int* __restrict__ Bshape0s, int* Xbufpos,
                                            int* Ybufpos) {
  nb2_pdl_enter();
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  const int ix = Xbufpos[k];
  const int iy = Ybufpos[k];
  Xbufpos[k] = (ix > 0) ? ix - 1 : Bshape0s[k] - 1;
  Ybufpos[k] = (iy > 0) ? iy - 1 : Ashape0s[k] - 1;
}

extern "C" int nb2_linearfilter(void* stream, int n_blocks, int block_size, int uses_buf,
                                const int* offsets, const int* shape0s, const int* shape1s,
                                const int* Xstride0s, const int* Xstride1s, const int* Xstarts,
                                const float* X, const int* Ystride0s, const int* Ystride1s,
                                const int* Ystarts, float* Y, const int* Ashape0s, const int* Astarts,
                                const float* A, const int* Bshape0s, const int* Bstarts, const float* B,
                                const int* Xbufstarts, float* Xbuf, const int* Ybufstarts, float* Ybuf,
                                int* Xbufpos, int* Ybufpos) {
  if (n_blocks == 0) return NB2_OK;
  NB2_REQUIRE(block_size >= 1 && block_size <= 1024, "block_size");
  NB2_REQUIRE(offsets && shape0s && shape1s && Xstride0s && Xstride1s && Xstarts && X && Ystride0s &&
                  Ystride1s && Ystarts && Y && Ashape0s && Astarts && A && Bshape0s && Bstarts && B,
              "null pointer");
  NB2_REQUIRE(!uses_buf || (Xbufstarts && Xbuf && Ybufstarts && Ybuf && Xbufpos && Ybufpos),
              "ring buffers required when uses_buf");
  cudaStream_t s = nb2_stream(stream);
  nb2_launch(nb2_linearfilter_kernel, dim3(n_blocks), dim3(block_size), 0, s, uses_buf, offsets, shape0s, shape1s, Xstride0s, Xstride1s, Xstarts, X, Ystride0s, Ystride1s, Ystarts, Y,
      Ashape0s, Astarts, A, Bshape0s, Bstarts, B, Xbufstarts, Xbuf, Ybufstarts, Ybuf, Xbufpos, Ybufpos);
  NB2_LAUNCH_CHECK();
  if (uses_buf) {
    nb2_launch(nb2_linearfilter_inc_kernel, dim3((n_blocks + 255) / 256), dim3(256), 0, s, n_blocks, Ashape0s, Bshape0s, Xbufpos,
                                                                       Ybufpos);
    NB2_LAUNCH_CHECK();
  }
  return NB2_OK;
}

// ---- weight deltas of the unsupervised learning rules --------------------------
// plan_bcm (clra_nonlinearities.py:2082-2169), plan_oja (:2172-2277), plan_voja
// (:2280-2405): one thread per element (i, j) of delta item k,
//   BCM : delta = alpha * post_i * (post_i - theta_i) * pre_j
//   Oja : delta = alpha * post_i * (pre_j - beta * w_ij * post_i)
//   Voja: delta = alpha * learn * post_i * (scale_i * pre_j - enc_ij)
// evaluated left to right as in the reference kernels (this file is compiled
// with -fmad=false).  `aux` is theta (a vector), the weights or the encoders.
struct LearnArgs {
  const int *shape0s, *shape1s;
  const int *pre_stride0s, *pre_starts;
  const float* pre;
  const int *post_stride0s, *post_starts;
  const float* post;
  const int *aux_stride0s, *aux_starts;
  const float* aux;
  const int *delta_stride0s, *delta_starts;
  float* delta;
  const float *alphas, *betas;
  const int* learn_starts;
  const float* learn;
  const int *scale_stride0s, *scale_starts;
  const float* scale;
};

template <int RULE>
__global__ void nb2_learning_delta_kernel(const LearnArgs a) {
  nb2_pdl_enter();
  const int ij = blockIdx.x * blockDim.x + threadIdx.x;
  const int k = blockIdx.y;
  const int shape0 = a.shape0s[k];
  const int shape1 = a.shape1s[k];
  const int i = ij / shape1;
  const int j = ij - i * shape1;
  if (i >= shape0) return;
  const float pre = a.pre[a.pre_starts[k] + j * a.pre_stride0s[k]];
  const float post = a.post[a.post_starts[k] + i * a.post_stride0s[k]];
  const float alpha = a.alphas[k];
  float out;
  if (RULE == NB2_RULE_BCM) {
    const float theta = a.aux[a.aux_starts[k] + i * a.aux_stride0s[k]];
    out = alpha * post * (post - theta) * pre;
  } else if (RULE == NB2_RULE_OJA) {
    const float weight = a.aux[a.aux_starts[k] + i * a.aux_stride0s[k] + j];
    out = alpha * post * (pre - a.betas[k] * weight * post);
  } else {
    const float enc = a.aux[a.aux_starts[k] + i * a.aux_stride0s[k] + j];
    const float learn = a.learn[a.learn_starts[k]];
    const float scale = a.scale[a.scale_starts[k] + i * a.scale_stride0s[k]];
    out = alpha * learn * post * (scale * pre - enc);
  }
  a.delta[a.delta_starts[k] + i * a.delta_stride0s[k] + j] = out;
}

extern "C" int nb2_learning_delta(void* stream, int rule, int n_items, int max_size, const int* shape0s,
                                  const int* shape1s, const int* pre_stride0s, const int* pre_starts,
                                  const float* pre, const int* post_stride0s, const int* post_starts,
                                  const float* post, const int* aux_stride0s, const int* aux_starts,
                                  const float* aux, const int* delta_stride0s, const int* delta_starts,
                                  float* delta, const float* alphas, const float* betas, const int* learn_starts,
                                  const float* learn, const int* scale_stride0s, const int* scale_starts,
                                  const float* scale) {
  if (n_items == 0 || max_size == 0) return NB2_OK;
  NB2_REQUIRE(rule == NB2_RULE_BCM || rule == NB2_RULE_OJA || rule == NB2_RULE_VOJA, "rule");
  NB2_REQUIRE(n_items > 0 && n_items <= 65535 && max_size > 0, "n_items / max_size");
  NB2_REQUIRE(shape0s && shape1s && pre_stride0s && pre_starts && pre && post_stride0s && post_starts && post &&
                  aux_stride0s && aux_starts && aux && delta_stride0s && delta_starts && delta && alphas,
              "null pointer");
  NB2_REQUIRE(rule != NB2_RULE_OJA || betas, "Oja needs betas");
  NB2_REQUIRE(rule != NB2_RULE_VOJA || (learn_starts && learn && scale_stride0s && scale_starts && scale),
              "Voja needs the learning signal and the scale");
  LearnArgs a = {shape0s, shape1s, pre_stride0s, pre_starts, pre, post_stride0s, post_starts, post,
                 aux_stride0s, aux_starts, aux, delta_stride0s, delta_starts, delta, alphas, betas,
                 learn_starts, learn, scale_stride0s, scale_starts, scale};
  const dim3 grid((max_size + 255) / 256, n_items);
  cudaStream_t s = nb2_stream(stream);
  if (rule == NB2_RULE_BCM) nb2_launch(nb2_learning_delta_kernel<NB2_RULE_BCM>, dim3(grid), dim3(256), 0, s, a);
  else if (rule == NB2_RULE_OJA) nb2_launch(nb2_learning_delta_kernel<NB2_RULE_OJA>, dim3(grid), dim3(256), 0, s, a);
  else nb2_launch(nb2_learning_delta_kernel<NB2_RULE_VOJA>, dim3(grid), dim3(256), 0, s, a);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}

// ---- plan_probes (:831-902) -------------------------------------------------
__global__ void nb2_probes_kernel(float* countdowns, int* bufpositions,
                                  const float* __restrict__ periods, const int* __restrict__ Xstarts,
                                  const int* __restrict__ Xshape0s, const int* __restrict__ Xshape1s,
                                  const int* __restrict__ Xstride0s,
                                  const int* __restrict__ Xstride1s, const float* X,
                                  const int* __restrict__ Ystarts, float* Y) {
  nb2_pdl_enter();
  const int n = blockIdx.x;
  const float countdown = countdowns[n];
  const int bufpos = bufpositions[n];
  __syncthreads();  // everyone has read the counters before thread 0 rewrites them
  const Nb2ProbesArgs a = {countdowns, bufpositions, periods, Xstarts, Xshape0s, Xshape1s, Xstride0s, Xstride1s, X,
                           Ystarts, Y};
  nb2_probes_body(a, n, threadIdx.x, blockDim.x, countdown, bufpos);
}

extern "C" int nb2_probes(void* stream, int n_probes, int block_size, float* countdowns,
                          int* bufpositions, const float* periods, const int* Xstarts,
                          const int* Xshape0s, const int* Xshape1s, const int* Xstride0s,
                          const int* Xstride1s, const float* X, const int* Ystarts, float* Y) {
  if (n_probes == 0) return NB2_OK;
  NB2_REQUIRE(block_size >= 1 && block_size <= 1024, "block_size");
  NB2_REQUIRE(countdowns && bufpositions && periods && Xstarts && Xshape0s && Xshape1s && Xstride0s &&
                  Xstride1s && X && Ystarts && Y,
              "null pointer");
  nb2_launch(nb2_probes_kernel, dim3(n_probes), dim3(block_size), 0, nb2_stream(stream), countdowns, bufpositions, periods, Xstarts, Xshape0s, Xshape1s, Xstride0s, Xstride1s, X, Ystarts, Y);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}

// Large probes (a whole population's spikes): `chunks` CTAs share one probe.  Every CTA
// reads the probe's counters before it copies its part; the counters may only advance when
// all of them have done so, so the CTAs count their arrivals in `arrive[n]` (zero between
// launches) and the last one advances the counters and clears the count.
#define PROBE_THREADS 256
__global__ void __launch_bounds__(PROBE_THREADS) nb2_probes_wide_kernel(
    float* countdowns, int* bufpositions, const float* __restrict__ periods, const int* __restrict__ Xstarts,
    const int* __restrict__ Xshape0s, const int* __restrict__ Xshape1s, const int* __restrict__ Xstride0s,
    const int* __restrict__ Xstride1s, const float* X, const int* __restrict__ Ystarts, float* Y, int* arrive) {
  nb2_pdl_enter();
  const int n = blockIdx.y;
  const float countdown = countdowns[n];
  const int bufpos = bufpositions[n];
  if (countdown <= 0.0f) {
    const int ni = Xshape0s[n];
    const int nj = Xshape1s[n];
    const int n_dims = ni * nj;
    const int sti = Xstride0s[n];
    const int stj = Xstride1s[n];
    const float* x = X + Xstarts[n];
    float* y = Y + Ystarts[n] + (size_t)bufpos * n_dims;
    for (int ij = blockIdx.x * PROBE_THREADS + threadIdx.x; ij < n_dims; ij += gridDim.x * PROBE_THREADS) {
      const int i = ij / nj;
      const int j = ij - i * nj;
      y[ij] = x[i * sti + j * stj];
    }
  }
  __syncthreads();  // every thread of this CTA has read the counters
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(arrive + n, 1) + 1 == (int)gridDim.x) {
      arrive[n] = 0;
      if (countdown <= 0.0f) {
        countdowns[n] = countdown + periods[n] - 1.0f;
        bufpositions[n] = bufpos + 1;
      } else {
        countdowns[n] = countdown - 1.0f;
      }
    }
  }
}

static int nb2_probes_wide_launch(void* stream, int n_probes, int chunks, float* countdowns, int* bufpositions,
                                  const float* periods, const int* Xstarts, const int* Xshape0s,
                                  const int* Xshape1s, const int* Xstride0s, const int* Xstride1s, const float* X,
                                  const int* Ystarts, float* Y, int* arrive) {
  NB2_REQUIRE(chunks >= 1 && chunks <= 65535 && n_probes <= 65535, "chunks / n_probes");
  NB2_REQUIRE(countdowns && bufpositions && periods && Xstarts && Xshape0s && Xshape1s && Xstride0s &&
                  Xstride1s && X && Ystarts && Y && arrive,
              "null pointer");
  nb2_launch(nb2_probes_wide_kernel, dim3(dim3(chunks, n_probes)), dim3(PROBE_THREADS), 0, nb2_stream(stream), countdowns, bufpositions, periods, Xstarts, Xshape0s, Xshape1s, Xstride0s, Xstride1s, X, Ystarts, Y, arrive);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}

extern "C" int nb2_probes_wide(void* stream, int n_probes, int chunks, float* countdowns, int* bufpositions,
                               const float* periods, const int* Xstarts, const int* Xshape0s,
                               const int* Xshape1s, const int* Xstride0s, const int* Xstride1s, const float* X,
                               const int* Ystarts, float* Y, int* arrive) {
  if (n_probes == 0) return NB2_OK;
  return nb2_probes_wide_launch(stream, n_probes, chunks, countdowns, bufpositions, periods, Xstarts, Xshape0s,
                                Xshape1s, Xstride0s, Xstride1s, X, Ystarts, Y, arrive);
}

// The same launch with the arrival counters in a device array of this library instead of
// caller memory: nothing is allocated, by the caller or here.  The array is zero at load
// time and every launch leaves it zero; its address is looked up once per device.
static __device__ __align__(256) int g_probe_arrive[NB2_PROBES_STATIC_MAX];

extern "C" int nb2_probes_wide_noalloc(void* stream, int n_probes, int chunks, float* countdowns,
                                       int* bufpositions, const float* periods, const int* Xstarts,
                                       const int* Xshape0s, const int* Xshape1s, const int* Xstride0s,
                                       const int* Xstride1s, const float* X, const int* Ystarts, float* Y) {
  if (n_probes == 0) return NB2_OK;
  NB2_REQUIRE(n_probes <= NB2_PROBES_STATIC_MAX, "more probes than the static arrival counters cover");
  // Set-up, once per device and with that device current: the array's name is only a host-side
  // stand-in, the kernel needs its device address.  Done by the first call on a device (under a
  // lock, so that two host threads cannot both be "first"); that call should come before any
  // stream capture.
  static int* arrive_of_device[64] = {};
  static std::mutex setup_lock;
  int dev = 0;
  NB2_CUDA(cudaGetDevice(&dev));
  NB2_REQUIRE(dev >= 0 && dev < 64, "device ordinal");
  {
    std::lock_guard<std::mutex> guard(setup_lock);
    if (arrive_of_device[dev] == NULL) {
      void* sym = NULL;
      NB2_CUDA(cudaGetSymbolAddress(&sym, g_probe_arrive));
      arrive_of_device[dev] = static_cast<int*>(sym);
    }
  }
  return nb2_probes_wide_launch(stream, n_probes, chunks, countdowns, bufpositions, periods, Xstarts, Xshape0s,
                                Xshape1s, Xstride0s, Xstride1s, X, Ystarts, Y, arrive_of_device[dev]);
}

// ---- plan_presentinput (:1694-1730) -----------------------------------------
__global__ void nb2_presentinput_kernel(int n_items, int width, const float* __restrict__ pres_t, float dt,
                                        const int* __restrict__ Yshape0s,
                                        const int* __restrict__ Ystarts, float* Y,
                                        const int* __restrict__ Tstarts, const float* T,
                                        const int* __restrict__ Sshape0s,
                                        const int* __restrict__ Sstarts,
                                        const int* __restrict__ Sstride0s,
                                        const float* __restrict__ S) {
  nb2_pdl_enter();
  // `width` threads per item (a power of two): a CTA takes blockDim.x / width items, so that
  // many short tables do not cost one nearly empty CTA each
  const Nb2PresentArgs a = {n_items, width, pres_t, dt, Yshape0s, Ystarts, Y, Tstarts, T, Sshape0s, Sstarts, Sstride0s, S};
  nb2_presentinput_body(a, blockIdx.x * (blockDim.x / width) + threadIdx.x / width, threadIdx.x % width, width);
}

extern "C" int nb2_presentinput(void* stream, int n_items, int block_size, const float* pres_t, double dt,
                                const int* Yshape0s, const int* Ystarts, float* Y, const int* Tstarts,
                                const float* T, const int* Sshape0s, const int* Sstarts,
                                const int* Sstride0s, const float* S) {
  if (n_items == 0) return NB2_OK;
  NB2_REQUIRE(block_size >= 1 && block_size <= 1024, "block_size");
  NB2_REQUIRE(Yshape0s && Ystarts && Y && Tstarts && T && Sshape0s && Sstarts && S, "null pointer");
  int width = 1;
  while (width < block_size) width <<= 1;
  const int threads = width < 256 ? 256 : width;
  const int per_cta = threads / width;
  nb2_launch(nb2_presentinput_kernel, dim3((n_items + per_cta - 1) / per_cta), dim3(threads), 0, nb2_stream(stream),
             n_items, width, pres_t, (float)dt, Yshape0s, Ystarts, Y, Tstarts, T, Sshape0s, Sstarts, Sstride0s, S);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}

// ---- gather-sum: Y = sum of sources ------------------------------------------
// One launch for the pattern "reset a signal to zero, then increment it by
// several whole-signal copies" (plan_reset :147-214 followed by one plan_copy
// :217-304 per group of non-overlapping targets in the reference).  Sources are
// added in operator order starting from zero, so the result is bit-identical to
// the reset + sequential increments.
// blocks: [n_blocks][4] = {dst start, element count (<= 256), first source, source count};
// src_starts: element offset of every (block, source) pair.
__global__ void nb2_gather_sum_kernel(int n_blocks, int width, const int4* __restrict__ blocks,
                                      const int* __restrict__ src_starts, float* data) {
  nb2_pdl_enter();
  // `width` threads per table block (a power of two >= the longest block): 256 / width blocks
  // per CTA, so that thousands of one- or sixteen-element targets fill their CTAs
  const Nb2GatherArgs a = {n_blocks, width, blocks, src_starts, data};
  nb2_gather_sum_body(a, blockIdx.x, threadIdx.x);
}

extern "C" int nb2_gather_sum(void* stream, int n_blocks, int width, const int* blocks, const int* src_starts,
                              float* data) {
  if (n_blocks == 0) return NB2_OK;
  NB2_REQUIRE(blocks && src_starts && data, "null pointer");
  NB2_REQUIRE(width >= 1 && width <= 256 && (width & (width - 1)) == 0, "width must be a power of two <= 256");
  const int per_cta = 256 / width;
  nb2_launch(nb2_gather_sum_kernel, dim3((n_blocks + per_cta - 1) / per_cta), dim3(256), 0, nb2_stream(stream), n_blocks,
             width, reinterpret_cast<const int4*>(blocks), src_starts, data);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
