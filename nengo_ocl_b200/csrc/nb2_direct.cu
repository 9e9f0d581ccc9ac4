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

__global__ void nb2_direct_kernel(int n_items, const int2* __restrict__ prog, int n_ops,
                                  const double* __restrict__ consts, const int* __restrict__ in0_starts,
                                  const float* in0, const int* __restrict__ in1_starts, const float* in1,
                                  const int* __restrict__ out_starts, float* out) {
  nb2_pdl_enter();
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= n_items) return;
  const float* x0 = in0 ? in0 + in0_starts[n] : nullptr;
  const float* x1 = in1 ? in1 + in1_starts[n] : nullptr;
  float* y = out + out_starts[n];
  double st[NB2_DIRECT_STACK];
  int sp = 0;
#define POP() (st[--sp])
#define PUSH(v) (st[sp++] = (v))
#define UN(expr) { double a = POP(); PUSH(expr); } break
#define BIN(expr) { double b = POP(); double a = POP(); PUSH(expr); } break
  for (int pc = 0; pc < n_ops; ++pc) {
    const int2 op = prog[pc];
    switch (op.x) {
      case NB2_OP_CONST: PUSH(consts[op.y]); break;
      case NB2_OP_IN0: PUSH((double)x0[op.y]); break;
      case NB2_OP_IN1: PUSH((double)x1[op.y]); break;
      case NB2_OP_STORE: y[op.y] = (float)POP(); break;
      case NB2_OP_ADD: BIN(a + b);
      case NB2_OP_SUB: BIN(a - b);
      case NB2_OP_MUL: BIN(a * b);
      case NB2_OP_DIV: BIN(a / b);
      case NB2_OP_POW: BIN(pow(a, b));
      case NB2_OP_MOD: BIN(a - floor(a / b) * b);
      case NB2_OP_MIN: BIN(fmin(a, b));
      case NB2_OP_MAX: BIN(fmax(a, b));
      case NB2_OP_ATAN2: BIN(atan2(a, b));
      case NB2_OP_LT: BIN(a < b ? 1.0 : 0.0);
      case NB2_OP_LE: BIN(a <= b ? 1.0 : 0.0);
      case NB2_OP_GT: BIN(a > b ? 1.0 : 0.0);
      case NB2_OP_GE: BIN(a >= b ? 1.0 : 0.0);
      case NB2_OP_EQ: BIN(a == b ? 1.0 : 0.0);
      case NB2_OP_NE: BIN(a != b ? 1.0 : 0.0);
      case NB2_OP_AND: BIN((a != 0.0 && b != 0.0) ? 1.0 : 0.0);
      case NB2_OP_OR: BIN((a != 0.0 || b != 0.0) ? 1.0 : 0.0);
      case NB2_OP_NEG: UN(-a);
      case NB2_OP_NOT: UN(a == 0.0 ? 1.0 : 0.0);
      case NB2_OP_SIN: UN(sin(a));
      case NB2_OP_COS: UN(cos(a));
      case NB2_OP_TAN: UN(tan(a));
      case NB2_OP_ASIN: UN(asin(a));
      case NB2_OP_ACOS: UN(acos(a));
      case NB2_OP_ATAN: UN(atan(a));
      case NB2_OP_SINH: UN(sinh(a));
      case NB2_OP_COSH: UN(cosh(a));
      case NB2_OP_TANH: UN(tanh(a));
      case NB2_OP_EXP: UN(exp(a));
      case NB2_OP_EXPM1: UN(expm1(a));
      case NB2_OP_LOG: UN(log(a));
      case NB2_OP_LOG2: UN(log2(a));
      case NB2_OP_LOG10: UN(log10(a));
      case NB2_OP_LOG1P: UN(log1p(a));
      case NB2_OP_SQRT: UN(sqrt(a));
      case NB2_OP_ABS: UN(fabs(a));
      case NB2_OP_FLOOR: UN(floor(a));
      case NB2_OP_CEIL: UN(ceil(a));
      case NB2_OP_ROUND: UN(rint(a));
      case NB2_OP_SIGN: UN(a > 0.0 ? 1.0 : (a < 0.0 ? -1.0 : 0.0));
      case NB2_OP_ACOSH: UN(acosh(a));
      case NB2_OP_ASINH: UN(asinh(a));
      case NB2_OP_ATANH: UN(atanh(a));
      case NB2_OP_EXP2: UN(exp2(a));
      case NB2_OP_ISINF: UN(isinf(a) ? 1.0 : 0.0);
      case NB2_OP_ISNAN: UN(isnan(a) ? 1.0 : 0.0);
      case NB2_OP_ISFINITE: UN(isfinite(a) ? 1.0 : 0.0);
      case NB2_OP_ERF: UN(erf(a));
      case NB2_OP_ERFC: UN(erfc(a));
      case NB2_OP_LGAMMA: UN(lgamma(a));
      case NB2_OP_FMOD: BIN(fmod(a, b));
      case NB2_OP_SELECT: {
        double b = POP(); double a = POP(); double c = POP();
        PUSH(c != 0.0 ? a : b);
      } break;
      default: break;
    }
  }
#undef POP
#undef PUSH
#undef UN
#undef BIN
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
