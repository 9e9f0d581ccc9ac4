// Per-step exchange of decoded signals between the GPUs of one box.
//
// The reference is single-device (nengo_ocl/simulator.py:215-219), so this has
// no counterpart there.  A model is sharded by ensemble block, one rank per
// GPU; every rank holds a full replica of one `exchange` signal and owns one
// contiguous segment of it.  After a step each rank PUSHES its segment into a
// staging buffer of every peer with plain peer stores over NVLink (no NCCL
// launch on the step path, no multicast loads) and then publishes the step
// number in the peer's flag array; before the next step each rank waits (with
// a time limit) until every peer's flag has reached the step it needs and copies
// the staged segments into its replica.
//
// Two staging buffers alternate by step parity: a rank can start step s+2 only
// after every peer published s+1, and a peer publishes s+1 only after it has
// consumed the parity-s buffer, so a push never overwrites data still to be read.
// Both kernels are captured in the step's CUDA graph; the step counter lives on
// the device.  A wait that runs out of time records NB2_ERR_TIMEOUT in the
// control block, stops waiting and lets the kernel finish, so the context stays
// usable and the host can report the failure.
#include "nb2_common.cuh"
#include "nb2_exchange_common.cuh"
#include "../../include/nengo_b200.h"

#define EXCH_THREADS 256

// Before step epoch+1: wait until every peer published `epoch`, then copy the
// peers' staged segments (parity epoch & 1) into the local replica.
__global__ void nb2_exchange_wait_kernel(int* ctl, const int* flags, const float* staging, float* replica,
                                         int rank, int world, int seg, long long timeout_ns) {
  nb2_pdl_enter();
  const int epoch = ctl[X_EPOCH];
  if (epoch == 0) return;  // nothing has been exchanged yet: replicas hold the initial values
  // thread p watches peer p's flag (the flags live in this GPU's memory; the peers store into
  // them), so the block waits for the slowest peer, not for the peers one after the other
  int ok = 1;
  if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
    const unsigned long long t0 = nb2_globaltimer();
    while (ld_acquire_sys(flags + threadIdx.x) < epoch) {
      if ((long long)(nb2_globaltimer() - t0) > timeout_ns) {
        ok = 0;
        atomicExch(ctl + X_STATUS, NB2_ERR_TIMEOUT);
        break;
      }
      __nanosleep(100);
    }
  }
  if (!__syncthreads_and(ok)) return;
  const float* src = staging + (size_t)(epoch & 1) * world * seg;
  const size_t total = (size_t)world * seg;
  const size_t lo = (size_t)rank * seg, hi = lo + seg;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    if (i < lo || i >= hi) replica[i] = src[i];
}

// After step epoch+1: store the local segment into every peer's staging buffer
// of parity (epoch+1) & 1, then (last block) publish epoch+1 to every peer.
__global__ void nb2_exchange_push_kernel(int* ctl, float* const* peer_staging, int* const* peer_flags,
                                         const float* replica, int rank, int world, int seg) {
  nb2_pdl_enter();
  const int next = ctl[X_EPOCH] + 1;
  const size_t off = (size_t)(next & 1) * world * seg + (size_t)rank * seg;
  const float* src = replica + (size_t)rank * seg;
  for (int p = 0; p < world; ++p) {
    if (p == rank) continue;
    float* dst = peer_staging[p] + off;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < seg; i += gridDim.x * blockDim.x) dst[i] = src[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(ctl + X_DONE_BLOCKS, 1) + 1;
    if (done == (int)gridDim.x) {
      ctl[X_DONE_BLOCKS] = 0;
      __threadfence_system();
      for (int p = 0; p < world; ++p)
        if (p != rank) st_release_sys(peer_flags[p] + rank, next);
      ctl[X_EPOCH] = next;
    }
  }
}

extern "C" int nb2_exchange_wait(void* stream, int* ctl, const int* flags, const float* staging,
                                 float* replica, int rank, int world, int seg, double timeout_s) {
  NB2_REQUIRE(ctl && flags && staging && replica, "null pointer");
  NB2_REQUIRE(world >= 1 && world <= EXCH_THREADS && rank >= 0 && rank < world && seg > 0, "rank/world/seg");
  if (world == 1) return NB2_OK;
  const long long total = (long long)world * seg;
  int blocks = (int)((total + EXCH_THREADS * 8 - 1) / (EXCH_THREADS * 8));
  if (blocks > 2 * NB2_NUM_SMS) blocks = 2 * NB2_NUM_SMS;
  if (blocks < 1) blocks = 1;
  nb2_launch(nb2_exchange_wait_kernel, dim3(blocks), dim3(EXCH_THREADS), 0, nb2_stream(stream), ctl, flags, staging, replica, rank, world, seg, (long long)(timeout_s * 1e9));
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}

extern "C" int nb2_exchange_push(void* stream, int* ctl, float* const* peer_staging, int* const* peer_flags,
                                 const float* replica, int rank, int world, int seg) {
  NB2_REQUIRE(ctl && peer_staging && peer_flags && replica, "null pointer");
  NB2_REQUIRE(world >= 1 && rank >= 0 && rank < world && seg > 0, "rank/world/seg");
  if (world == 1) return NB2_OK;
  int blocks = (seg + EXCH_THREADS * 4 - 1) / (EXCH_THREADS * 4);
  if (blocks > NB2_NUM_SMS) blocks = NB2_NUM_SMS;
  if (blocks < 1) blocks = 1;
  nb2_launch(nb2_exchange_push_kernel, dim3(blocks), dim3(EXCH_THREADS), 0, nb2_stream(stream), ctl, peer_staging, peer_flags,
                                                                            replica, rank, world, seg);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
