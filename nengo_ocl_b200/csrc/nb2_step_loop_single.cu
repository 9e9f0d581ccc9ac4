// The persistent step loop on ONE CTA, for models so small that every phase is a block or
// two: a barrier is then __syncthreads(), every signal stays in this multiprocessor's L1
// between phases and steps, and a step costs a few L1 round trips instead of one launch
// gap per plan.  Compiled with the default caching of global loads (the multi-CTA kernel in
// nb2_step_loop.cu needs L2-only loads); everything else is shared (nb2_step_loop_device.cuh).
#include "nb2_step_loop_device.cuh"

__global__ void __launch_bounds__(LOOP_THREADS, 1)
nb2_step_loop_single_kernel(const StepPhase* __restrict__ phases, int n_phases, int n_steps, unsigned* counter,
                            int* status) {
  extern __shared__ __align__(16) unsigned char dyn[];
  nb2_step_loop_device<true>(dyn, phases, n_phases, n_steps, counter, status);
}

cudaError_t nb2_step_loop_single_prepare(size_t smem) {
  return cudaFuncSetAttribute(nb2_step_loop_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

cudaError_t nb2_step_loop_single_launch(const StepPhase* phases, int n_phases, int n_steps, unsigned* counter,
                                        int* status, size_t smem, cudaStream_t s) {
  // (an ordinary launch: the loop starts only when everything before it on the stream has finished)
  nb2_step_loop_single_kernel<<<1, LOOP_THREADS, smem, s>>>(phases, n_phases, n_steps, counter, status);
  return cudaGetLastError();
}
