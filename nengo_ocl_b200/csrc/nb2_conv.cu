// 2-D convolution / local filtering and average pooling on one image:
// plan_conv2d (nengo_ocl/clra_nonlinearities.py:1762-1969) and plan_pool2d
// (:1972-2079).
//
// One thread per output element (filter k, row i, column j).  The reference
// stages an image patch and the filter of one channel in local memory per
// work-group; the images of a simulated network are a few thousand elements
// and live in L2/L1, so the threads read them directly and the kernel needs no
// barrier.  The sum runs over channels, then kernel rows, then kernel columns,
// starting from zero, each product rounded before it is added (this translation
// unit is compiled with -fmad=false): the order of the reference's loop nest
// (:1836-1868).  The reference kernel STORES the result into y (:1871-1872);
// `inc` adds it instead, which is what the ConvInc operator means when its
// target was not reset in the same step.  Padding reads as zero.
// Pooling averages the elements of the window that lie inside the image
// (:2013-2026: out-of-range positions are NaN-marked there and skipped).
#include "nb2_common.cuh"
#include "../../include/nengo_b200.h"

struct ConvGeom {
  int nc, nxi, nxj;  // input channels, rows, columns
  int nf, nyi, nyj;  // filters, output rows, columns
  int si, sj, sti, stj, pi, pj;
  int xs_c, xs_i, xs_j;  // element strides of x
  int ys_f, ys_i, ys_j;  // element strides of y
  int inc;               // 0: store the result (the reference kernel), 1: add it to y
  int conv;              // 1: shared filters [si][sj][nc][nf]; 0: local filters [nf][nc][si][sj][nyi][nyj]
};

__global__ void nb2_conv2d_kernel(const ConvGeom g, const float* x, const float* __restrict__ f, float* y) {
  nb2_pdl_enter();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int per_f = g.nyi * g.nyj;
  if (idx >= g.nf * per_f) return;
  const int k = idx / per_f, ij = idx - k * per_f;
  const int i = ij / g.nyj, j = ij - i * g.nyj;
  const int i0 = i * g.sti - g.pi, j0 = j * g.stj - g.pj;
  float out = 0.0f;
  for (int c = 0; c < g.nc; ++c) {
    const float* xc = x + (size_t)c * g.xs_c;
    for (int ii = 0; ii < g.si; ++ii) {
      const int xi = i0 + ii;
      for (int jj = 0; jj < g.sj; ++jj) {
        const int xj = j0 + jj;
        const float p = (xi >= 0 && xi < g.nxi && xj >= 0 && xj < g.nxj) ? xc[(size_t)xi * g.xs_i + (size_t)xj * g.xs_j]
                                                                           : 0.0f;
        const float w = g.conv ? f[((size_t)(ii * g.sj + jj) * g.nc + c) * g.nf + k]
                               : f[(((size_t)k * g.nc + c) * (g.si * g.sj) + ii * g.sj + jj) * per_f + ij];
        out = out + w * p;
      }
    }
  }
  float* yo = y + (size_t)k * g.ys_f + (size_t)i * g.ys_i + (size_t)j * g.ys_j;
  *yo = g.inc ? *yo + out : out;
}

extern "C" int nb2_conv2d(void* stream, const float* x, const float* filters, float* y, int nc, int nxi, int nxj, int nf,
                          int nyi, int nyj, int si, int sj, int sti, int stj, int pi, int pj, int channels_last,
                          int conv, int inc) {
  NB2_REQUIRE(x && filters && y, "null pointer");
  NB2_REQUIRE(nc >= 1 && nxi >= 1 && nxj >= 1 && nf >= 1 && nyi >= 1 && nyj >= 1 && si >= 1 && sj >= 1 && sti >= 1 &&
                  stj >= 1 && pi >= 0 && pj >= 0,
              "shape");
  NB2_REQUIRE((long long)nf * nyi * nyj < (1ll << 31) && (long long)nc * nxi * nxj < (1ll << 31), "image too large");
  ConvGeom g;
  g.nc = nc; g.nxi = nxi; g.nxj = nxj; g.nf = nf; g.nyi = nyi; g.nyj = nyj;
  g.si = si; g.sj = sj; g.sti = sti; g.stj = stj; g.pi = pi; g.pj = pj;
  g.xs_i = nxj * (channels_last ? nc : 1);
  g.xs_j = channels_last ? nc : 1;
  g.xs_c = channels_last ? 1 : nxi * nxj;
  g.ys_i = nyj * (channels_last ? nf : 1);
  g.ys_j = channels_last ? nf : 1;
  g.ys_f = channels_last ? 1 : nyi * nyj;
  g.conv = conv ? 1 : 0;
  g.inc = inc ? 1 : 0;
  const int n = nf * nyi * nyj;
  nb2_launch(nb2_conv2d_kernel, dim3((n + 255) / 256), dim3(256), 0, nb2_stream(stream), g, x, filters, y);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}

__global__ void nb2_pool2d_kernel(const float* x, float* y, int nc, int nyi, int nyj, int nxi, int nxj, int si, int sj,
                                  int sti, int stj) {
  nb2_pdl_enter();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int per_c = nyi * nyj;
  if (idx >= nc * per_c) return;
  const int c = idx / per_c, ij = idx - c * per_c;
  const int i = ij / nyj, j = ij - i * nyj;
  const float* xc = x + (size_t)c * nxi * nxj;
  float out = 0.0f;
  int n = 0;
  for (int ii = 0; ii < si; ++ii) {
    const int xi = i * sti + ii;
    for (int jj = 0; jj < sj; ++jj) {
      const int xj = j * stj + jj;
      if (xi < nxi && xj < nxj) {
        const float v = xc[(size_t)xi * nxj + xj];
        if (!isnan(v)) {  // (a NaN in the image is skipped like a position outside it, :2020-2024)
          out = out + v;
          ++n;
        }
      }
    }
  }
  y[(size_t)c * per_c + ij] = out / (float)n;
}

extern "C" int nb2_pool2d(void* stream, const float* x, float* y, int nc, int nyi, int nyj, int nxi, int nxj, int si,
                          int sj, int sti, int stj) {
  NB2_REQUIRE(x && y, "null pointer");
  NB2_REQUIRE(nc >= 1 && nyi >= 1 && nyj >= 1 && nxi >= 1 && nxj >= 1 && si >= 1 && sj >= 1 && sti >= 1 && stj >= 1,
              "shape");
  NB2_REQUIRE((long long)nc * nyi * nyj < (1ll << 31) && (long long)nc * nxi * nxj < (1ll << 31), "image too large");
  const int n = nc * nyi * nyj;
  nb2_launch(nb2_pool2d_kernel, dim3((n + 255) / 256), dim3(256), 0, nb2_stream(stream), x, y, nc, nyi, nyj, nxi, nxj,
             si, sj, sti, stj);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
