// Bodies of the block-order ragged GEMV (see nb2_gemv_block.cu) as device functions over a
// virtual block index, shared by its own kernels and the persistent step loop
// (nb2_step_loop.cu).  NC: matrices and vectors may be read through the non-coherent path
// (only valid when nothing inside the same kernel launch writes them).
#pragma once
#include "nb2_common.cuh"
#include "nb2_blockdot.cuh"

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
template <bool NC> __device__ __forceinline__ float gb_ld(const float* p) { return NC ? __ldg(p) : *p; }

template <bool NC>
__device__ __forceinline__ float gb_tile_value(const GemvBlockParams& p, const int* g, const int* xst, int k, int c0,
                                               int row, bool valid, int j) {
  const int D = p.D;
  const int N = __ldg(&g[3 * D + k]);
  const int len = min(128, N - c0);
  float acc = 0.0f;
  if (valid) {
    const float* a = p.A + __ldg(&g[1 * D + k]) + (size_t)row * __ldg(&g[2 * D + k]) + c0;
    const int xs = xst ? __ldg(&xst[k]) : 1;
    const float* x = p.X + __ldg(&g[0 * D + k]) + (ptrdiff_t)c0 * xs;
    if (xs == 1) {
#pragma unroll 16
      for (int c = j; c < len; c += 4) acc = bd_add(acc, bd_mul(gb_ld<NC>(a + c), gb_ld<NC>(x + c)));
    } else {
#pragma unroll 4
      for (int c = j; c < len; c += 4) acc = bd_add(acc, bd_mul(gb_ld<NC>(a + c), gb_ld<NC>(x + (ptrdiff_t)c * xs)));
    }
  }
  acc = bd_add(acc, __shfl_xor_sync(0xffffffffu, acc, 2));  // s0 + s2 | s1 + s3
  acc = bd_add(acc, __shfl_xor_sync(0xffffffffu, acc, 1));  // (s0 + s2) + (s1 + s3)
  return bd_scale(acc, p.alpha);
}

struct GemvBlockSmem {
  float tile[GB_ROWS][GB_TMAX + 1];
  float total[GB_ROWS];
};

// One CTA (GB_THREADS threads, all of which call this) per 32-row unit `vblock`.
template <bool NC>
__device__ __forceinline__ void nb2_gemv_block_cta_body(void* smem, const GemvBlockParams& p, int vblock) {
  GemvBlockSmem& sm = *reinterpret_cast<GemvBlockSmem*>(smem);
  float(*s_tile)[GB_TMAX + 1] = sm.tile;
  float* s_total = sm.total;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int4 unit = __ldg(&p.worklist[vblock]);
  const int D = p.D;
  const int* g = p.gstructure + (size_t)unit.x * p.gstride;
  const int* xst = p.xstrides ? p.xstrides + (size_t)unit.x * D : nullptr;
  const int r0 = unit.y, R = unit.z;
  const int n_dots = __ldg(&g[4 * D + 2]);
  const int y_in = __ldg(&g[4 * D + 0]) + r0, y = __ldg(&g[4 * D + 1]) + r0;
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
          const float v = gb_tile_value<NC>(p, g, xst, kk, cc, r0 + row_l, row_l < R, j);
          if (j == 0 && row_l < R) s_tile[row_l][tt] = v;
        }
      }
      cc += 128;
      if (cc >= __ldg(&g[3 * D + kk])) {
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

// One warp per unit of at most 8 rows: virtual block `vblock` covers GB_WARPS units.
template <bool NC>
__device__ __forceinline__ void nb2_gemv_block_warp_body(const GemvBlockParams& p, int vblock) {
  const int lane = threadIdx.x & 31;
  const int u = vblock * GB_WARPS + (threadIdx.x >> 5);
  if (u >= p.n_units) return;
  const int4 unit = __ldg(&p.worklist[u]);
  const int D = p.D;
  const int* g = p.gstructure + (size_t)unit.x * p.gstride;
  const int* xst = p.xstrides ? p.xstrides + (size_t)unit.x * D : nullptr;
  const int r0 = unit.y, R = unit.z;  // R <= 8
  const int n_dots = __ldg(&g[4 * D + 2]);
  const int rl = lane >> 2, j = lane & 3;
  const bool valid = rl < R;
  float total = valid ? (float)(p.beta * (double)p.Yin[__ldg(&g[4 * D + 0]) + r0 + rl]) : 0.0f;
  for (int k = 0; k < n_dots; ++k) {
    const int N = __ldg(&g[3 * D + k]);
    for (int c0 = 0; c0 < N; c0 += 128) total = bd_add(total, gb_tile_value<NC>(p, g, xst, k, c0, r0 + rl, valid, j));
  }
  if (valid && j == 0) p.Y[__ldg(&g[4 * D + 1]) + r0 + rl] = (float)((double)total + p.gamma);
}

