// Device evaluation of translated Python node functions.
//
// The reference turns a Python function into OpenCL C text and compiles one
// program per function (plan_direct, nengo_ocl/clra_nonlinearities.py:954-1025,
// with nengo_ocl/ast_conversion.py:845-931 producing the text).  Here the
// translator emits a postfix program instead and a single interpreter kernel
// evaluates it, one thread per function instance, so no run-time compiler is
// needed and the launch is capturable in a CUDA graph like any other plan.
#include "nb2_common.cuh"
#include "../../include/nengo_b200.h"
#include "nb2_direct_ops.h"

#define DIRECT_STACK 32

__global__ void nb2_direct_kernel(int n_items, const int2* __restrict__ prog, int n_ops,
                                  const float* __restrict__ consts, const int* __restrict__ in0_starts,
                                  const float* in0, const int* __restrict__ in1_starts, const float* in1,
                                  const int* __restrict__ out_starts, float* out) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= n_items) return;
  const float* x0 = in0 ? in0 + in0_starts[n] : nullptr;
  const float* x1 = in1 ? in1 + in1_starts[n] : nullptr;
  float* y = out + out_starts[n];
  float st[DIRECT_STACK];
  int sp = 0;
#define POP() (st[--sp])
#define PUSH(v) (st[sp++] = (v))
#define UN(expr) { float a = POP(); PUSH(expr); } break
#define BIN(expr) { float b = POP(); float a = POP(); PUSH(expr); } break
  for (int pc = 0; pc < n_ops; ++pc) {
    const int2 op = prog[pc];
    switch (op.x) {
      case NB2_OP_CONST: PUSH(consts[op.y]); break;
      case NB2_OP_IN0: PUSH(x0[op.y]); break;
      case NB2_OP_IN1: PUSH(x1[op.y]); break;
      case NB2_OP_STORE: y[op.y] = POP(); break;
      case NB2_OP_ADD: BIN(a + b);
      case NB2_OP_SUB: BIN(a - b);
      case NB2_OP_MUL: BIN(a * b);
      case NB2_OP_DIV: BIN(a / b);
      case NB2_OP_POW: BIN(powf(a, b));
      case NB2_OP_MOD: BIN(a - floorf(a / b) * b);
      case NB2_OP_MIN: BIN(fminf(a, b));
      case NB2_OP_MAX: BIN(fmaxf(a, b));
      case NB2_OP_ATAN2: BIN(atan2f(a, b));
      case NB2_OP_LT: BIN(a < b ? 1.0f : 0.0f);
      case NB2_OP_LE: BIN(a <= b ? 1.0f : 0.0f);
      case NB2_OP_GT: BIN(a > b ? 1.0f : 0.0f);
      case NB2_OP_GE: BIN(a >= b ? 1.0f : 0.0f);
      case NB2_OP_EQ: BIN(a == b ? 1.0f : 0.0f);
      case NB2_OP_NE: BIN(a != b ? 1.0f : 0.0f);
      case NB2_OP_AND: BIN((a != 0.0f && b != 0.0f) ? 1.0f : 0.0f);
      case NB2_OP_OR: BIN((a != 0.0f || b != 0.0f) ? 1.0f : 0.0f);
      case NB2_OP_NEG: UN(-a);
      case NB2_OP_NOT: UN(a == 0.0f ? 1.0f : 0.0f);
      case NB2_OP_SIN: UN(sinf(a));
      case NB2_OP_COS: UN(cosf(a));
      case NB2_OP_TAN: UN(tanf(a));
      case NB2_OP_ASIN: UN(asinf(a));
      case NB2_OP_ACOS: UN(acosf(a));
      case NB2_OP_ATAN: UN(atanf(a));
      case NB2_OP_SINH: UN(sinhf(a));
      case NB2_OP_COSH: UN(coshf(a));
      case NB2_OP_TANH: UN(tanhf(a));
      case NB2_OP_EXP: UN(expf(a));
      case NB2_OP_EXPM1: UN(expm1f(a));
      case NB2_OP_LOG: UN(logf(a));
      case NB2_OP_LOG2: UN(log2f(a));
      case NB2_OP_LOG10: UN(log10f(a));
      case NB2_OP_LOG1P: UN(log1pf(a));
      case NB2_OP_SQRT: UN(sqrtf(a));
      case NB2_OP_ABS: UN(fabsf(a));
      case NB2_OP_FLOOR: UN(floorf(a));
      case NB2_OP_CEIL: UN(ceilf(a));
      case NB2_OP_ROUND: UN(rintf(a));
      case NB2_OP_SIGN: UN(a > 0.0f ? 1.0f : (a < 0.0f ? -1.0f : 0.0f));
      case NB2_OP_SELECT: {
        float b = POP(); float a = POP(); float c = POP();
        PUSH(c != 0.0f ? a : b);
      } break;
      default: break;
    }
  }
#undef POP
#undef PUSH
#undef UN
#undef BIN
}

extern "C" int nb2_direct(void* stream, int n_items, const int* prog, int n_ops, const float* consts,
                          int out_dim, const int* in0_starts, const float* in0, const int* in1_starts,
                          const float* in1, const int* out_starts, float* out) {
  if (n_items == 0) return NB2_OK;
  NB2_REQUIRE(prog && out_starts && out && out_dim >= 1, "null pointer");
  NB2_REQUIRE((in0 == NULL) == (in0_starts == NULL) && (in1 == NULL) == (in1_starts == NULL),
              "input buffer/starts mismatch");
  nb2_direct_kernel<<<(n_items + 127) / 128, 128, 0, nb2_stream(stream)>>>(
      n_items, reinterpret_cast<const int2*>(prog), n_ops, consts, in0_starts, in0, in1_starts, in1,
      out_starts, out);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
