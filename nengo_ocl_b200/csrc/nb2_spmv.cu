// Sparse matrix-vector products  y (+)= A x  for sparse transforms.
//
// Replaces the reference's three OpenCL SpMV kernels: spmv_csr_impl
// (nengo_ocl/clra_gemv.py:1570-1646, one work-item per row walking the row
// serially), spmv_ellpack_impl (:1649-1755, one work-group per row with a tree
// reduction in local memory) and spmv_ellpacktwostep_impl (:1758-1916, partial
// sums in a scratch buffer and a second reduction kernel).  Both formats are
// streams of (column, value) pairs read exactly once, i.e. HBM-bound at
// 8 bytes per nonzero plus the gathered x values (served by L2):
//
//  * CSR: 2^k lanes per row (k chosen by the host from the mean row length:
//    about 8 nonzeros per lane, several rows per warp) so that a warp's loads
//    of `data` and `indices` cover whole sectors and many are in flight; partial sums
//    meet in a shuffle reduction.  No scratch buffer, one launch.
//  * ELLPACK, many rows or narrow: the host stores the padded arrays column-
//    major (entry (row, k) at k * n_rows + row), one thread per row, so every
//    load instruction of a warp is one contiguous line.
//  * ELLPACK, few wide rows: row-major as the reference stores it, one warp per row.
//    Row lengths bound every loop, so padding is never read.
#include "nb2_common.cuh"
#include "../../include/nengo_b200.h"

#define SPMV_THREADS 256

template <int LOGG>
__global__ void __launch_bounds__(SPMV_THREADS) nb2_spmv_csr_kernel(const int* __restrict__ indices,
                                                                     const int* __restrict__ indptr,
                                                                     const float* __restrict__ data, int n_rows,
                                                                     const float* __restrict__ x, float* y, int inc) {
  nb2_pdl_enter();
  constexpr int G = 1 << LOGG;
  const int row = (int)(((size_t)blockIdx.x * SPMV_THREADS + threadIdx.x) >> LOGG);
  const int g = threadIdx.x & (G - 1);
  float sum = 0.0f;
  if (row < n_rows) {
    const int end = __ldg(indptr + row + 1);
#pragma unroll 8
    for (int k = __ldg(indptr + row) + g; k < end; k += G)
      sum = fmaf(__ldcs(data + k), __ldg(x + __ldcs(indices + k)), sum);
  }
#pragma unroll
  for (int off = G >> 1; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if (row < n_rows && g == 0) y[row] = inc ? y[row] + sum : sum;
}

// narrow ELLPACK, column-major, thread per row
__global__ void __launch_bounds__(SPMV_THREADS) nb2_spmv_ell_cm_kernel(const int* __restrict__ columns,
                                                                        const float* __restrict__ entries,
                                                                        const int* __restrict__ rowlens, int n_rows,
                                                                        const float* __restrict__ x, float* y,
                                                                        int inc) {
  nb2_pdl_enter();
  const int row = blockIdx.x * SPMV_THREADS + threadIdx.x;
  if (row >= n_rows) return;
  const int len = __ldg(rowlens + row);
  float sum = 0.0f;
#pragma unroll 8
  for (int k = 0; k < len; ++k) {
    const size_t at = (size_t)k * n_rows + row;
    sum = fmaf(__ldcs(entries + at), __ldg(x + __ldcs(columns + at)), sum);
  }
  y[row] = inc ? y[row] + sum : sum;
}

// wide ELLPACK, row-major, warp per row
__global__ void __launch_bounds__(SPMV_THREADS) nb2_spmv_ell_rm_kernel(const int* __restrict__ columns,
                                                                        const float* __restrict__ entries,
                                                                        const int* __restrict__ rowlens, int n_rows,
                                                                        int width, const float* __restrict__ x,
                                                                        float* y, int inc) {
  nb2_pdl_enter();
  const int row = (int)(((size_t)blockIdx.x * SPMV_THREADS + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  float sum = 0.0f;
  if (row < n_rows) {
    const int len = __ldg(rowlens + row);
    const size_t base = (size_t)row * width;
    for (int k = lane; k < len; k += 32)
      sum = fmaf(__ldcs(entries + base + k), __ldg(x + __ldcs(columns + base + k)), sum);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if (row < n_rows && lane == 0) y[row] = inc ? y[row] + sum : sum;
}

extern "C" int nb2_spmv_csr(void* stream, const int* indices, const int* indptr, const float* data, int n_rows,
                            int lanes_log2, const float* x, float* y, int inc) {
  if (n_rows == 0) return NB2_OK;
  NB2_REQUIRE(indices && indptr && data && x && y, "null pointer");
  NB2_REQUIRE(n_rows > 0 && lanes_log2 >= 0 && lanes_log2 <= 5, "n_rows / lanes_log2");
  cudaStream_t s = nb2_stream(stream);
  const long long threads = (long long)n_rows << lanes_log2;
  const unsigned blocks = (unsigned)((threads + SPMV_THREADS - 1) / SPMV_THREADS);
  switch (lanes_log2) {
    case 0: nb2_launch(nb2_spmv_csr_kernel<0>, dim3(blocks), dim3(SPMV_THREADS), 0, s, indices, indptr, data, n_rows, x, y, inc); break;
    case 1: nb2_launch(nb2_spmv_csr_kernel<1>, dim3(blocks), dim3(SPMV_THREADS), 0, s, indices, indptr, data, n_rows, x, y, inc); break;
    case 2: nb2_launch(nb2_spmv_csr_kernel<2>, dim3(blocks), dim3(SPMV_THREADS), 0, s, indices, indptr, data, n_rows, x, y, inc); break;
    case 3: nb2_launch(nb2_spmv_csr_kernel<3>, dim3(blocks), dim3(SPMV_THREADS), 0, s, indices, indptr, data, n_rows, x, y, inc); break;
    case 4: nb2_launch(nb2_spmv_csr_kernel<4>, dim3(blocks), dim3(SPMV_THREADS), 0, s, indices, indptr, data, n_rows, x, y, inc); break;
    default: nb2_launch(nb2_spmv_csr_kernel<5>, dim3(blocks), dim3(SPMV_THREADS), 0, s, indices, indptr, data, n_rows, x, y, inc); break;
  }
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}

extern "C" int nb2_spmv_ell(void* stream, const int* columns, const float* entries, const int* rowlens, int n_rows,
                            int width, int row_major, const float* x, float* y, int inc) {
  if (n_rows == 0) return NB2_OK;
  NB2_REQUIRE(columns && entries && rowlens && x && y, "null pointer");
  NB2_REQUIRE(n_rows > 0 && width >= 0, "n_rows / width");
  cudaStream_t s = nb2_stream(stream);
  if (row_major) {
    const unsigned blocks = (unsigned)(((long long)n_rows * 32 + SPMV_THREADS - 1) / SPMV_THREADS);
    nb2_launch(nb2_spmv_ell_rm_kernel, dim3(blocks), dim3(SPMV_THREADS), 0, s, columns, entries, rowlens, n_rows, width, x, y, inc);
  } else {
    const unsigned blocks = (unsigned)((n_rows + SPMV_THREADS - 1) / SPMV_THREADS);
    nb2_launch(nb2_spmv_ell_cm_kernel, dim3(blocks), dim3(SPMV_THREADS), 0, s, columns, entries, rowlens, n_rows, x, y, inc);
  }
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
