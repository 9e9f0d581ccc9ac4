// Shared pieces of the bulk-copy pipelines (nb2_gemv_pipe.cu, nb2_fused_stream.cu):
// bounded mbarrier waits, 1-D bulk async copies, and the lane-per-row dot product
// over rows staged in shared memory.
#pragma once
#include "nb2_common.cuh"

#ifndef PIPE_UNROLL
#define PIPE_UNROLL 8
#endif
constexpr int kPipeUnroll = PIPE_UNROLL;
#define PIPE_WAIT_NS 1000000000ull  // limit of one barrier wait
#ifndef PIPE_SUSPEND_NS
#define PIPE_SUSPEND_NS 20000u  // a waiting thread is suspended by the hardware for up to this long per poll
#endif


__device__ __forceinline__ uint32_t pipe_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long pipe_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool mbar_try(unsigned long long* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n .reg .pred q;\n mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2, %3;\n selp.u32 %0, 1, 0, q;\n}"
      : "=r"(done)
      : "r"(pipe_smem(bar)), "r"(parity), "r"(PIPE_SUSPEND_NS)
      : "memory");
  return done != 0;
}

// Bounded parity wait.  Returns false on timeout.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t parity) {
  unsigned long long t0 = 0;
  for (int spins = 0;; ++spins) {
    if (mbar_try(bar, parity)) return true;
    if ((spins & 3) == 3) {
      const unsigned long long t = pipe_timer();
      if (t0 == 0) t0 = t;
      else if (t - t0 > PIPE_WAIT_NS) return false;
    }
  }
}

__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   pipe_smem(dst)),
               "l"(src), "r"(bytes), "r"(pipe_smem(bar))
               : "memory");
}

// One staged block of rows for one lane: NR rows (roff, in rows of w floats), all w columns.
// MODE 0: x staged in shared memory, columns in order (the x load is a broadcast);
// MODE 1: x staged, diagonal walk (lane l starts at column l mod w) for widths
//         whose row pitch would put all lanes into a few banks;
// MODE 2: x read from global memory with a stride.
template <int NR, int MODE>
__device__ __forceinline__ void pipe_segment(const float* __restrict__ a, const float* __restrict__ x, int xstride,
                                             int w, int lane, const int (&roff)[4], float (&acc)[4]) {
  const float* a0 = a + roff[0] * w;
  const float* a1 = a + roff[NR > 1 ? 1 : 0] * w;
  const float* a2 = a + roff[NR > 2 ? 2 : 0] * w;
  const float* a3 = a + roff[NR > 3 ? 3 : 0] * w;
  if (MODE == 1) {
    int cc = lane % w;
#pragma unroll 4
    for (int c = 0; c < w; ++c) {
      const float xv = x[cc];
      acc[0] = fmaf(a0[cc], xv, acc[0]);
      if (NR > 1) acc[1] = fmaf(a1[cc], xv, acc[1]);
      if (NR > 2) acc[2] = fmaf(a2[cc], xv, acc[2]);
      if (NR > 3) acc[3] = fmaf(a3[cc], xv, acc[3]);
      ++cc;
      if (cc == w) cc = 0;
    }
  } else {
#pragma unroll kPipeUnroll
    for (int c = 0; c < w; ++c) {
      const float xv = MODE == 0 ? x[c] : __ldg(x + (size_t)c * xstride);
      acc[0] = fmaf(a0[c], xv, acc[0]);
      if (NR > 1) acc[1] = fmaf(a1[c], xv, acc[1]);
      if (NR > 2) acc[2] = fmaf(a2[c], xv, acc[2]);
      if (NR > 3) acc[3] = fmaf(a3[c], xv, acc[3]);
    }
  }
}

template <int NR>
__device__ __forceinline__ void pipe_segment_mode(const float* a, const float* xs, const float* xg, int xstride,
                                                  int w, int lane, const int (&roff)[4], float (&acc)[4]) {
  if (xs == nullptr) pipe_segment<NR, 2>(a, xg, xstride, w, lane, roff, acc);
  else if ((w & 7) == 0) pipe_segment<NR, 1>(a, xs, 1, w, lane, roff, acc);
  else pipe_segment<NR, 0>(a, xs, 1, w, lane, roff, acc);
}

__device__ __forceinline__ void l2_prefetch(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

