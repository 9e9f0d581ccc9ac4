// Control block and system-scope flag accesses of the per-step exchange between
// GPUs (nb2_exchange.cu, and the push folded into nb2_fused_stream.cu).
#pragma once
#include "nb2_common.cuh"

// control block (ints) in local device memory
enum { X_EPOCH = 0, X_DONE_BLOCKS, X_STATUS, X_WORDS = 8 };

__device__ __forceinline__ unsigned long long nb2_globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

