// Shared helpers for the sm_100a kernels and the C-ABI entry points.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define NB2_OK 0
#define NB2_ERR_CUDA (-1)
#define NB2_ERR_ARG (-2)
#define NB2_ERR_LIMIT (-3)
#define NB2_ERR_TIMEOUT (-4)

// Records a message retrievable through nb2_last_error().
void nb2_set_error(const char* fmt, ...);

#define NB2_CUDA(call)                                                         \
  do {                                                                         \
    cudaError_t e__ = (call);                                                  \
    if (e__ != cudaSuccess) {                                                  \
      nb2_set_error("%s:%d %s -> %s", __FILE__, __LINE__, #call,               \
                    cudaGetErrorString(e__));                                  \
      return NB2_ERR_CUDA;                                                     \
    }                                                                          \
  } while (0)

#define NB2_LAUNCH_CHECK()                                                     \
  do {                                                                         \
    cudaError_t e__ = cudaGetLastError();                                      \
    if (e__ != cudaSuccess) {                                                  \
      nb2_set_error("%s:%d launch -> %s", __FILE__, __LINE__,                  \
                    cudaGetErrorString(e__));                                  \
      return NB2_ERR_CUDA;                                                     \
    }                                                                          \
  } while (0)

#define NB2_REQUIRE(cond, msg)                                                 \
  do {                                                                         \
    if (!(cond)) {                                                             \
      nb2_set_error("%s:%d argument check failed: %s (%s)", __FILE__,          \
                    __LINE__, #cond, msg);                                     \
      return NB2_ERR_ARG;                                                      \
    }                                                                          \
  } while (0)

static inline cudaStream_t nb2_stream(void* s) { return (cudaStream_t)s; }

// ---- programmatic dependent launch -----------------------------------------------------
// A simulation step is a chain of small dependent launches; most of a tiny kernel's cost is
// the launch gap before it.  Every kernel of this library is launched with the
// programmatic-stream-serialization attribute and starts with nb2_pdl_enter(): the next
// kernel of the stream (or of the captured graph) may be scheduled while this one still runs
// and then waits, at its first instruction, until every kernel before it has completed and
// flushed its memory.  The data dependencies are exactly those of an ordinary in-order
// stream; only the launch latency overlaps.  nb2_set_programmatic_launch(0) (or the
// environment variable NENGO_B200_PDL=0) turns the attribute off; the device-side
// instructions are then no-ops.
extern "C" int nb2_programmatic_launch_enabled();

#ifdef __CUDACC__
__device__ __forceinline__ void nb2_pdl_enter() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
static inline cudaError_t nb2_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                     Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = nb2_programmatic_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

// B200: 148 SMs. Grid sizes for grid-stride kernels are multiples of this.
#define NB2_NUM_SMS 148

// Streaming (read-once) global loads: bypass L1 allocation.
__device__ __forceinline__ float nb2_ldg_stream(const float* p) {
  float v;
  asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float4 nb2_ldg_stream4(const float4* p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
