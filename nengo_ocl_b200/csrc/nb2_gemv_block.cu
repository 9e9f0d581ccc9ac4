// Ragged gather-GEMV with the summation order of the reference's block_impl
// (nengo_ocl/clra_gemv.py:861-1175), the variant its simulator plans for every
// MultiDotInc (simulator.py:803):
//
//     Y[k] = ((beta * Y_in[k] + alpha * tile_0) + alpha * tile_1) + ... + gamma
//
// where the tiles are the 128-column blocks of every term in list order and a
// tile is four column-strided partial sums combined as (s0 + s2) + (s1 + s3)
// (nb2_blockdot.cuh).  Results are bit-identical to that kernel pair; there is
// no scratch buffer and no second kernel.
//
// Work units (host-built, int4 = item row of the index table, first output row,
// row count <= 32, 0) mirror the reference's 32-row blocks.  Four lanes own the
// four partial sums of one row of one tile and walk them in order; two shuffles
// give the tile value.
//  * nb2_gemv_block_cta_kernel: one CTA (8 warps) per unit.  The (8-row group,
//    tile) pairs of the unit are dealt to the warps; tile values meet in shared
//    memory and one thread per row adds them in order.
//  * nb2_gemv_block_warp_kernel: one warp per unit of at most 8 rows and a few
//    tiles (the many tiny products of a model: scalar gains, 1 x n decoders).
// Matrices are read straight from global memory (these products are small and
// L2-resident inside a model step; the HBM-bound products of a model run in the
// fused ensemble kernels).
#include "nb2_common.cuh"
#include "nb2_blockdot.cuh"
#include "../../include/nengo_b200.h"

#define GB_THREADS 256
#define GB_WARPS (GB_THREADS / 32)
#define GB_ROWS 32   // rows per unit
#define GB_TMAX 64   // tile values per row held in shared memory at a time

struct GemvBlockParams {
  const int* gstructure;  // [n_items][gstride]
  const int* xstrides;    // [n_items][D] or NULL (all 1)
  const int4* worklist;
  int n_units;
  int gstride;
  int D;
  const float* A;
  const float* X;
  const float* Yin;
  float* Y;
  double alpha, beta, gamma;
};

// The four lanes (row, j = 0..3) of a row: partial sum j of the tile starting at column c0
// of term k, combined to the tile value (valid in all four lanes).
__device__ __forceinline__ float gb_tile_value(const GemvBlockParams& p, const int* g, const int* xst, int k, int c0,
                                               int row, bool valid, int j) {
  const int D = p.D;
  const int N = g[3 * D + k];
  const int len = min(128, N - c0);
  float acc = 0.0f;
  if (valid) {
    const float* a = p.A + g[1 * D + k] + (size_t)row * g[2 * D + k] + c0;
    const int xs = xst ? xst[k] : 1;
    const float* x = p.X + g[0 * D + k] + (ptrdiff_t)c0 * xs;
    if (xs == 1) {
#pragma unroll 8
      for (int c = j; c < len; c += 4) acc = bd_add(acc, bd_mul(__ldg(a + c), __ldg(x + c)));
    } else {
#pragma unroll 4
      for (int c = j; c < len; c += 4) acc = bd_add(acc, bd_mul(__ldg(a + c), __ldg(x + (ptrdiff_t)c * xs)));
    }
  }
  acc = bd_add(acc, __shfl_xor_sync(0xffffffffu, acc, 2));  // s0 + s2 | s1 + s3
  acc = bd_add(acc, __shfl_xor_sync(0xffffffffu, acc, 1));  // (s0 + s2) + (s1 + s3)
  return bd_scale(acc, p.alpha);
}

__global__ void __launch_bounds__(GB_THREADS) nb2_gemv_block_cta_kernel(const GemvBlockParams p) {
  nb2_pdl_enter();
  __shared__ float s_tile[GB_ROWS][GB_TMAX + 1];
  __shared__ float s_total[GB_ROWS];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int4 unit = p.worklist[blockIdx.x];
  const int D = p.D;
  const int* g = p.gstructure + (size_t)unit.x * p.gstride;
  const int* xst = p.xstrides ? p.xstrides + (size_t)unit.x * D : nullptr;
  const int r0 = unit.y, R = unit.z;
  const int n_dots = g[4 * D + 2];
  const int y_in = g[4 * D + 0] + r0, y = g[4 * D + 1] + r0;
  if (tid < R) s_total[tid] = (float)(p.beta * (double)p.Yin[y_in + tid]);
  const int n_groups = (R + 7) >> 3;
  const int rl = lane >> 2, j = lane & 3;
  // walk the tiles of all terms in order, GB_TMAX at a time
  int k = 0, c0 = 0;  // next tile: term k, first column c0
  while (k < n_dots) {
    // this pass: tiles tt = 0 .. n_pass - 1 starting at (k, c0)
    int kk = k, cc = c0, tt = 0, task = 0;
    for (; kk < n_dots && tt < GB_TMAX; ++tt) {
      for (int grp = 0; grp < n_groups; ++grp, ++task) {
        if (task % GB_WARPS == wid) {
          const int row_l = grp * 8 + rl;
          const float v = gb_tile_value(p, g, xst, kk, cc, r0 + row_l, row_l < R, j);
          if (j == 0 && row_l < R) s_tile[row_l][tt] = v;
        }
      }
      cc += 128;
      if (cc >= g[3 * D + kk]) {
        cc = 0;
        ++kk;
      }
    }
    __syncthreads();
    if (tid < R) {
      float total = s_total[tid];
      for (int q = 0; q < tt; ++q) total = bd_add(total, s_tile[tid][q]);
      s_total[tid] = total;
    }
    __syncthreads();
    k = kk;
    c0 = cc;
  }
  if (tid < R) p.Y[y + tid] = (float)((double)s_total[tid] + p.gamma);
}

__global__ void __launch_bounds__(GB_THREADS) nb2_gemv_block_warp_kernel(const GemvBlockParams p) {
  nb2_pdl_enter();
  const int lane = threadIdx.x & 31;
  const int u = blockIdx.x * GB_WARPS + (threadIdx.x >> 5);
  if (u >= p.n_units) return;
  const int4 unit = p.worklist[u];
  const int D = p.D;
  const int* g = p.gstructure + (size_t)unit.x * p.gstride;
  const int* xst = p.xstrides ? p.xstrides + (size_t)unit.x * D : nullptr;
  const int r0 = unit.y, R = unit.z;  // R <= 8
  const int n_dots = g[4 * D + 2];
  const int rl = lane >> 2, j = lane & 3;
  const bool valid = rl < R;
  float total = valid ? (float)(p.beta * (double)p.Yin[g[4 * D + 0] + r0 + rl]) : 0.0f;
  for (int k = 0; k < n_dots; ++k) {
    const int N = g[3 * D + k];
    for (int c0 = 0; c0 < N; c0 += 128) total = bd_add(total, gb_tile_value(p, g, xst, k, c0, r0 + rl, valid, j));
  }
  if (valid && j == 0) p.Y[g[4 * D + 1] + r0 + rl] = (float)((double)total + p.gamma);
}

extern "C" int nb2_gemv_block(void* stream, const int* gstructure, int gstride, int D, const int* xstrides,
                              const int* cta_units, int n_cta, const int* warp_units, int n_warp, const float* A,
                              const float* X, const float* Yin, float* Y, double alpha, double beta,
                              double gamma) {
  if (n_cta == 0 && n_warp == 0) return NB2_OK;
  NB2_REQUIRE(gstructure && A && X && Yin && Y, "null pointer");
  NB2_REQUIRE(D >= 0 && gstride >= 4 * D + 5, "table layout");
  GemvBlockParams p;
  p.gstructure = gstructure; p.xstrides = xstrides; p.gstride = gstride; p.D = D;
  p.A = A; p.X = X; p.Yin = Yin; p.Y = Y;
  p.alpha = alpha; p.beta = beta; p.gamma = gamma;
  cudaStream_t s = nb2_stream(stream);
  if (n_cta > 0) {
    NB2_REQUIRE(cta_units != NULL, "cta_units");
    p.worklist = reinterpret_cast<const int4*>(cta_units);
    p.n_units = n_cta;
    nb2_launch(nb2_gemv_block_cta_kernel, dim3(n_cta), dim3(GB_THREADS), 0, s, p);
    NB2_LAUNCH_CHECK();
  }
  if (n_warp > 0) {
    NB2_REQUIRE(warp_units != NULL, "warp_units");
    p.worklist = reinterpret_cast<const int4*>(warp_units);
    p.n_units = n_warp;
    nb2_launch(nb2_gemv_block_warp_kernel, dim3((n_warp + GB_WARPS - 1) / GB_WARPS), dim3(GB_THREADS), 0, s, p);
    NB2_LAUNCH_CHECK();
  }
  return NB2_OK;
}
