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
#include "nb2_fused_body.cuh"

// TPE = threads per ensemble (32 or 256); NEMAX = staged neurons per ensemble
template <int TPE, int NEMAX>
__global__ void __launch_bounds__(FUSED_THREADS, TPE == 32 ? FUSED_MIN_BLOCKS_SMALL : FUSED_MIN_BLOCKS)
nb2_ensemble_step_kernel(int n_ens, const int* __restrict__ ens_ids, const int* __restrict__ ens_table,
                         const int* __restrict__ term_table, const int* __restrict__ conn_table,
                         float* data, float dt, float dt_inv) {
  nb2_pdl_enter();
  __shared__ __align__(16) unsigned char smem[sizeof(FusedSmem<TPE, NEMAX>)];
  nb2_ensemble_step_body<TPE, NEMAX, true>(smem, blockIdx.x, n_ens, ens_ids, ens_table, term_table, conn_table, data,
                                           dt, dt_inv);
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
