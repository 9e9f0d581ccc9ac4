// Bodies of the small per-step kernels as device functions over a VIRTUAL block
// index, so that the same code runs either as its own launch (virtual block =
// blockIdx.x; nb2_elementwise.cu, nb2_direct.cu) or as one phase of the persistent
// step-loop kernel (nb2_step_loop.cu), where every CTA walks the virtual blocks of
// a phase with a stride of the grid size.  Index tables and programs are constant for
// the life of a launch and are read through the non-coherent path (__ldg); signal data,
// which an earlier phase of the same launch may have written, never is.  `tid` / `nthreads`: this thread's index
// in the CTA and the CTA size.  Reference counterparts are cited at each body.
#pragma once
#include "nb2_common.cuh"
#include "nb2_direct_ops.h"

// ---- plan_timeupdate (clra_nonlinearities.py:119-133) ----------------------
struct Nb2TimeupdateArgs {
  float* step;
  float* time;
  double dt;
};
__device__ __forceinline__ void nb2_timeupdate_body(const Nb2TimeupdateArgs& a, int vb, int tid) {
  if (vb != 0 || tid != 0) return;
  const float s = a.step[0] + 1.0f;
  a.step[0] = s;
  a.time[0] = (float)(a.dt * (double)s);  // dt is a double literal in the reference source
}

// ---- gather-sum: reset to zero + whole-signal increments in operator order ----
// (plan_reset :147-214 followed by plan_copy(inc) :217-304 in the reference)
// blocks: [n_blocks][4] = {dst start, element count (<= width), first source, source count};
// `width` threads per table block, 256 / width table blocks per virtual block.
struct Nb2GatherArgs {
  int n_blocks;
  int width;
  const int4* blocks;
  const int* src_starts;
  float* data;
};
__device__ __forceinline__ void nb2_gather_sum_body(const Nb2GatherArgs& a, int vb, int tid) {
  const int k = vb * (256 / a.width) + tid / a.width;
  if (tid >= 256 || k >= a.n_blocks) return;
  const int4 b = __ldg(&a.blocks[k]);
  const int i = tid % a.width;
  if (i >= b.y) return;
  // sources are added one by one in list order, starting from zero; their loads are issued four at
  // a time (an index and a value each: two dependent memory round trips per group instead of per source)
  float sum = 0.0f;
  int q = 0;
  for (; q + 4 <= b.w; q += 4) {
    const int s0 = __ldg(&a.src_starts[b.z + q]), s1 = __ldg(&a.src_starts[b.z + q + 1]);
    const int s2 = __ldg(&a.src_starts[b.z + q + 2]), s3 = __ldg(&a.src_starts[b.z + q + 3]);
    const float v0 = a.data[s0 + i], v1 = a.data[s1 + i], v2 = a.data[s2 + i], v3 = a.data[s3 + i];
    sum += v0;
    sum += v1;
    sum += v2;
    sum += v3;
  }
  for (; q < b.w; ++q) sum += a.data[__ldg(&a.src_starts[b.z + q]) + i];
  a.data[b.x + i] = sum;
}

// ---- plan_probes (:831-902): one virtual block per probe -----------------------
struct Nb2ProbesArgs {
  float* countdowns;
  int* bufpositions;
  const float* periods;
  const int* Xstarts;
  const int* Xshape0s;
  const int* Xshape1s;
  const int* Xstride0s;
  const int* Xstride1s;
  const float* X;
  const int* Ystarts;
  float* Y;
};
// The caller reads countdowns[n] and bufpositions[n] in every thread and synchronises the CTA
// before this call, so that thread 0 cannot rewrite them under a slower thread.
__device__ __forceinline__ void nb2_probes_body(const Nb2ProbesArgs& a, int n, int tid, int nthreads,
                                                float countdown, int bufpos) {
  if (countdown <= 0.0f) {
    const int ni = __ldg(&a.Xshape0s[n]);
    const int nj = __ldg(&a.Xshape1s[n]);
    const int n_dims = ni * nj;
    const int sti = __ldg(&a.Xstride0s[n]);
    const int stj = __ldg(&a.Xstride1s[n]);
    const float* x = a.X + __ldg(&a.Xstarts[n]);
    float* y = a.Y + __ldg(&a.Ystarts[n]) + bufpos * n_dims;
    for (int ij = tid; ij < n_dims; ij += nthreads) {
      const int i = ij / nj;
      const int j = ij - i * nj;
      y[ij] = x[i * sti + j * stj];
    }
    if (tid == 0) {
      a.countdowns[n] = countdown + __ldg(&a.periods[n]) - 1.0f;
      a.bufpositions[n] = bufpos + 1;
    }
  } else if (tid == 0) {
    a.countdowns[n] = countdown - 1.0f;
  }
}

// ---- plan_linearfilter (:604-711), paths without ring buffers ------------------
// (order-0 gain and first-order lowpass: y = b0 x [- a0 y])
struct Nb2FilterArgs {
  int block_size;
  const int* offsets;
  const int* shape0s;
  const int* shape1s;
  const int* Xstride0s;
  const int* Xstride1s;
  const int* Xstarts;
  const float* x;
  const int* Ystride0s;
  const int* Ystride1s;
  const int* Ystarts;
  float* y;
  const int* Ashape0s;
  const int* Astarts;
  const float* Adata;
  const int* Bshape0s;
  const int* Bstarts;
  const float* Bdata;
};
__device__ __forceinline__ void nb2_filter_fast_body(const Nb2FilterArgs& a, int k, int tid, int nthreads) {
  const int shape0 = __ldg(&a.shape0s[k]);
  const int shape1 = __ldg(&a.shape1s[k]);
  const int na = __ldg(&a.Ashape0s[k]);
  const int nb = __ldg(&a.Bshape0s[k]);
  if (nb != 1 || na > 1) return;  // (ring-buffer filters are not planned as a phase)
  const float b0 = __ldg(&a.Bdata[__ldg(&a.Bstarts[k])]);
  const float a0 = na ? __ldg(&a.Adata[__ldg(&a.Astarts[k])]) : 0.0f;
  for (int t = tid; t < a.block_size; t += nthreads) {
    const int ij = t + __ldg(&a.offsets[k]);
    const int i = ij / shape1;
    const int j = ij - i * shape1;
    if (i >= shape0) continue;
    const int xij = __ldg(&a.Xstarts[k]) + i * __ldg(&a.Xstride0s[k]) + j * __ldg(&a.Xstride1s[k]);
    const int yij = __ldg(&a.Ystarts[k]) + i * __ldg(&a.Ystride0s[k]) + j * __ldg(&a.Ystride1s[k]);
    if (na == 0) a.y[yij] = b0 * a.x[xij];
    else a.y[yij] = b0 * a.x[xij] - a0 * a.y[yij];
  }
}

// ---- plan_presentinput (:1694-1730): row `step-derived index` of item k's table ----
struct Nb2PresentArgs {
  int n_items;
  int width;  // threads per item, a power of two
  const float* pres_t;
  float dt;
  const int* Yshape0s;
  const int* Ystarts;
  float* Y;
  const int* Tstarts;
  const float* T;
  const int* Sshape0s;
  const int* Sstarts;
  const int* Sstride0s;
  const float* S;
};
// item k, elements i0, i0 + stride, ...
__device__ __forceinline__ void nb2_presentinput_body(const Nb2PresentArgs& a, int k, int i0, int stride) {
  if (k >= a.n_items) return;
  const int m = __ldg(&a.Yshape0s[k]);
  float* y = a.Y + __ldg(&a.Ystarts[k]);
  const float* s = a.S + __ldg(&a.Sstarts[k]);
  const int it = (int)a.T[__ldg(&a.Tstarts[k])];
  const int nt = __ldg(&a.Sshape0s[k]);
  int ti;
  if (a.pres_t) ti = (int)(((float)it - 0.5f) * (a.dt / __ldg(&a.pres_t[k]))) % nt;
  else ti = it % nt;
  const int row = a.Sstride0s ? __ldg(&a.Sstride0s[k]) : m;  // table rows are packed unless a stride table is given
  for (int i = i0; i < m; i += stride) y[i] = __ldg(&s[(size_t)row * ti + i]);  // (the tables are constants)
}

// ---- plan_direct (:954-1025): postfix program, one thread per function instance -
struct Nb2DirectArgs {
  int n_items;
  const int2* prog;
  int n_ops;
  const double* consts;
  const int* in0_starts;
  const float* in0;
  const int* in1_starts;
  const float* in1;
  const int* out_starts;
  float* out;
};
__device__ __forceinline__ void nb2_direct_body(const Nb2DirectArgs& a, int n) {
  if (n >= a.n_items) return;
  const float* x0 = a.in0 ? a.in0 + __ldg(&a.in0_starts[n]) : nullptr;
  const float* x1 = a.in1 ? a.in1 + __ldg(&a.in1_starts[n]) : nullptr;
  float* y = a.out + __ldg(&a.out_starts[n]);
  double st[NB2_DIRECT_STACK];
  int sp = 0;
#define POP() (st[--sp])
#define PUSH(v) (st[sp++] = (v))
#define UN(expr) { double a_ = POP(); PUSH(expr); } break
#define BIN(expr) { double b_ = POP(); double a_ = POP(); PUSH(expr); } break
  for (int pc = 0; pc < a.n_ops; ++pc) {
    const int2 op = __ldg(&a.prog[pc]);
    switch (op.x) {
      case NB2_OP_CONST: PUSH(__ldg(&a.consts[op.y])); break;
      case NB2_OP_IN0: PUSH((double)x0[op.y]); break;
      case NB2_OP_IN1: PUSH((double)x1[op.y]); break;
      case NB2_OP_STORE: y[op.y] = (float)POP(); break;
      case NB2_OP_ADD: BIN(a_ + b_);
      case NB2_OP_SUB: BIN(a_ - b_);
      case NB2_OP_MUL: BIN(a_ * b_);
      case NB2_OP_DIV: BIN(a_ / b_);
      case NB2_OP_POW: BIN(pow(a_, b_));
      case NB2_OP_MOD: BIN(a_ - floor(a_ / b_) * b_);
      case NB2_OP_MIN: BIN(fmin(a_, b_));
      case NB2_OP_MAX: BIN(fmax(a_, b_));
      case NB2_OP_ATAN2: BIN(atan2(a_, b_));
      case NB2_OP_LT: BIN(a_ < b_ ? 1.0 : 0.0);
      case NB2_OP_LE: BIN(a_ <= b_ ? 1.0 : 0.0);
      case NB2_OP_GT: BIN(a_ > b_ ? 1.0 : 0.0);
      case NB2_OP_GE: BIN(a_ >= b_ ? 1.0 : 0.0);
      case NB2_OP_EQ: BIN(a_ == b_ ? 1.0 : 0.0);
      case NB2_OP_NE: BIN(a_ != b_ ? 1.0 : 0.0);
      case NB2_OP_AND: BIN((a_ != 0.0 && b_ != 0.0) ? 1.0 : 0.0);
      case NB2_OP_OR: BIN((a_ != 0.0 || b_ != 0.0) ? 1.0 : 0.0);
      case NB2_OP_NEG: UN(-a_);
      case NB2_OP_NOT: UN(a_ == 0.0 ? 1.0 : 0.0);
      case NB2_OP_SIN: UN(sin(a_));
      case NB2_OP_COS: UN(cos(a_));
      case NB2_OP_TAN: UN(tan(a_));
      case NB2_OP_ASIN: UN(asin(a_));
      case NB2_OP_ACOS: UN(acos(a_));
      case NB2_OP_ATAN: UN(atan(a_));
      case NB2_OP_SINH: UN(sinh(a_));
      case NB2_OP_COSH: UN(cosh(a_));
      case NB2_OP_TANH: UN(tanh(a_));
      case NB2_OP_EXP: UN(exp(a_));
      case NB2_OP_EXPM1: UN(expm1(a_));
      case NB2_OP_LOG: UN(log(a_));
      case NB2_OP_LOG2: UN(log2(a_));
      case NB2_OP_LOG10: UN(log10(a_));
      case NB2_OP_LOG1P: UN(log1p(a_));
      case NB2_OP_SQRT: UN(sqrt(a_));
      case NB2_OP_ABS: UN(fabs(a_));
      case NB2_OP_FLOOR: UN(floor(a_));
      case NB2_OP_CEIL: UN(ceil(a_));
      case NB2_OP_ROUND: UN(rint(a_));
      case NB2_OP_SIGN: UN(a_ > 0.0 ? 1.0 : (a_ < 0.0 ? -1.0 : 0.0));
      case NB2_OP_ACOSH: UN(acosh(a_));
      case NB2_OP_ASINH: UN(asinh(a_));
      case NB2_OP_ATANH: UN(atanh(a_));
      case NB2_OP_EXP2: UN(exp2(a_));
      case NB2_OP_ISINF: UN(isinf(a_) ? 1.0 : 0.0);
      case NB2_OP_ISNAN: UN(isnan(a_) ? 1.0 : 0.0);
      case NB2_OP_ISFINITE: UN(isfinite(a_) ? 1.0 : 0.0);
      case NB2_OP_ERF: UN(erf(a_));
      case NB2_OP_ERFC: UN(erfc(a_));
      case NB2_OP_LGAMMA: UN(lgamma(a_));
      case NB2_OP_FMOD: BIN(fmod(a_, b_));
      case NB2_OP_SELECT: {
        double b_ = POP(); double a_ = POP(); double c_ = POP();
        PUSH(c_ != 0.0 ? a_ : b_);
      } break;
      default: break;
    }
  }
#undef POP
#undef PUSH
#undef UN
#undef BIN
}
