// Dot products in the summation order of the reference's block GEMV, the kernel
// its simulator plans for every MultiDotInc (nengo_ocl/simulator.py:803,
// clra_gemv.py:1018-1058 and :1137-1153): a row is cut into tiles of 128
// columns; inside a tile four partial sums take the columns j, j + 4, j + 8, ...
// (j = 0..3) in ascending order, each product rounded before it is added (no
// fused multiply-add); the tile is (s0 + s2) + (s1 + s3), scaled by alpha, and
// the tiles are added to the running output value in order.  Results are
// therefore bit-identical to that kernel, whatever the thread mapping.
//
// Two mappings are provided.
//  * lane per row (block_rows_*): a lane walks its own rows; the four partial
//    sums are four registers per row.  Rows staged in shared memory with a pitch
//    that is a multiple of 4 floats are read with 128-bit loads.  Optionally the
//    lanes whose rows fall into the same banks start a few iterations later than
//    their neighbours ("time skew"; walking the columns in a rotated order
//    instead would change the summation order); measured on the fused step the
//    skew's extra iterations cost slightly more than the bank conflicts it
//    removes, so the default is off.
//  * lane per partial sum: for short, wide matrices (decoders) every lane owns
//    one or two of the 4 partial sums of one (row, tile) and walks them
//    sequentially; the tile value is formed with two shuffles (see the D records
//    of nb2_fused_stream.cu, nb2_fused.cu and nb2_gemv_block.cu).
#pragma once
#include "nb2_common.cuh"

__device__ __forceinline__ float bd_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float bd_add(float a, float b) { return __fadd_rn(a, b); }

// (s0 + s2) + (s1 + s3), then alpha as the double literal of the kernel text
__device__ __forceinline__ float bd_tile(float s0, float s1, float s2, float s3) {
  return bd_add(bd_add(s0, s2), bd_add(s1, s3));
}
__device__ __forceinline__ float bd_scale(float tile, double alpha) {
  return alpha == 1.0 ? tile : (float)(alpha * (double)tile);
}

// gcd(v, 8) for v >= 1
__device__ __forceinline__ int bd_gcd8(int v) { return (v & 1) ? 1 : (v & 2) ? 2 : (v & 4) ? 4 : 8; }

// Lane per row, rows staged in shared memory with pitch w (w % 4 == 0, rows and x
// 16-byte aligned).  total[j] += alpha * tile for every tile of the w columns, for
// the NR rows roff[0..NR) of this lane.
template <int NR>
__device__ __forceinline__ void block_rows_staged4(const float* __restrict__ a, const float* __restrict__ x, int w,
                                                   int lane, const int (&roff)[4], float (&total)[4],
                                                   double alpha, bool use_skew = false) {
  const int chunks_row = w >> 2;  // float4 per row
  const float4* x4 = reinterpret_cast<const float4*>(x);
  const float4* a4[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) a4[j] = reinterpret_cast<const float4*>(a) + (size_t)roff[j < NR ? j : 0] * chunks_row;
  // A 128-bit shared load is served 8 lanes at a time; those lanes read rows 8 apart at
  // most, i.e. chunk indices row * chunks_row + q: g = gcd(chunks_row, 8) of them collide
  // unless they are g different q apart.
  const int g = use_skew ? bd_gcd8(chunks_row) : 1;
  const int skew = ((lane & 7) * g) >> 3;
  for (int c0 = 0; c0 < chunks_row; c0 += 32) {  // one tile = 32 chunks
    const int nch = min(32, chunks_row - c0);
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
    for (int k = 0; k < nch + g - 1; ++k) {
      const int q = k - skew;
      if (q >= 0 && q < nch) {
        const float4 xv = x4[c0 + q];
#pragma unroll
        for (int j = 0; j < NR; ++j) {
          const float4 av = a4[j][c0 + q];
          s[j][0] = bd_add(s[j][0], bd_mul(av.x, xv.x));
          s[j][1] = bd_add(s[j][1], bd_mul(av.y, xv.y));
          s[j][2] = bd_add(s[j][2], bd_mul(av.z, xv.z));
          s[j][3] = bd_add(s[j][3], bd_mul(av.w, xv.w));
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NR; ++j)
      total[j] = bd_add(total[j], bd_scale(bd_tile(s[j][0], s[j][1], s[j][2], s[j][3]), alpha));
  }
}
