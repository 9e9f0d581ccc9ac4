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
//  * CTA units (nb2_gemv_block_cta_body): one CTA (8 warps) per unit.  The (8-row group,
//    tile) pairs of the unit are dealt to the warps; tile values meet in shared
//    memory and one thread per row adds them in order.
//  * warp units (nb2_gemv_block_warp_body): one warp per unit of at most 8 rows and a few
//    tiles (the many tiny products of a model: scalar gains, 1 x n decoders).
// Matrices are read straight from global memory (these products are small and
// L2-resident inside a model step; the HBM-bound products of a model run in the
// fused ensemble kernels).
#include "nb2_gemv_block_body.cuh"
#include "../../include/nengo_b200.h"

// One launch for both kinds of unit: the first n_cta blocks take a 32-row unit each, the blocks
// after them eight warp units each.
__global__ void __launch_bounds__(GB_THREADS) nb2_gemv_block_kernel(const GemvBlockParams pc, const GemvBlockParams pw,
                                                                    int n_cta) {
  nb2_pdl_enter();
  __shared__ __align__(16) unsigned char smem[sizeof(GemvBlockSmem)];
  if ((int)blockIdx.x < n_cta) nb2_gemv_block_cta_body<true>(smem, pc, blockIdx.x);
  else nb2_gemv_block_warp_body<true>(pw, blockIdx.x - n_cta);
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
  NB2_REQUIRE((n_cta == 0 || cta_units != NULL) && (n_warp == 0 || warp_units != NULL), "units");
  GemvBlockParams pc = p, pw = p;
  pc.worklist = reinterpret_cast<const int4*>(cta_units);
  pc.n_units = n_cta;
  pw.worklist = reinterpret_cast<const int4*>(warp_units);
  pw.n_units = n_warp;
  const int warp_blocks = (n_warp + GB_WARPS - 1) / GB_WARPS;
  nb2_launch(nb2_gemv_block_kernel, dim3(n_cta + warp_blocks), dim3(GB_THREADS), 0, s, pc, pw, n_cta);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
