// Device evaluation of translated Python node functions.
//
// The reference turns a Python function into OpenCL C text and compiles one
// program per function (plan_direct, nengo_ocl/clra_nonlinearities.py:954-1025,
// with nengo_ocl/ast_conversion.py:845-931 producing the text).  Here the
// translator emits a postfix program instead and a single interpreter kernel
// evaluates it, one thread per function instance, so no run-time compiler is
// needed and the launch is capturable in a CUDA graph like any other plan.
//
// The program is evaluated in double precision (inputs widened, the constant
// pool held in double, results rounded to float when stored): that is how the
// Python function itself computes, so a node's float32 output is the correctly
// rounded value of the Python expression rather than a chain of float32
// roundings.  The evaluation stack holds NB2_DIRECT_STACK values; the translator
// computes the depth a program needs and the entry point rejects deeper ones.
#include "nb2_common.cuh"
#include "../../include/nengo_b200.h"
#include "nb2_direct_ops.h"
#include "nb2_phase_bodies.cuh"

__global__ void nb2_direct_kernel(int n_items, const int2* __restrict__ prog, int n_ops,
                                  const double* __restrict__ consts, const int* __restrict__ in0_starts,
                                  const float* in0, const int* __restrict__ in1_starts, const float* in1,
                                  const int* __restrict__ out_starts, float* out) {
  nb2_pdl_enter();
  const Nb2DirectArgs a = {n_items, prog, n_ops, consts, in0_starts, in0, in1_starts, in1, out_starts, out};
  nb2_direct_body(a, blockIdx.x * blockDim.x + threadIdx.x);
}

extern "C" int nb2_direct(void* stream, int n_items, const int* prog, int n_ops, int max_depth,
                          const double* consts, int out_dim, const int* in0_starts, const float* in0, const int* in1_starts,
                          const float* in1, const int* out_starts, float* out) {
  if (n_items == 0) return NB2_OK;
  NB2_REQUIRE(prog && out_starts && out && out_dim >= 1, "null pointer");
  NB2_REQUIRE(max_depth >= 0 && max_depth <= NB2_DIRECT_STACK, "program needs a deeper evaluation stack");
  NB2_REQUIRE((in0 == NULL) == (in0_starts == NULL) && (in1 == NULL) == (in1_starts == NULL),
              "input buffer/starts mismatch");
  nb2_launch(nb2_direct_kernel, dim3((n_items + 127) / 128), dim3(128), 0, nb2_stream(stream), n_items, reinterpret_cast<const int2*>(prog), n_ops, consts, in0_starts, in0, in1_starts, in1,
      out_starts, out);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
