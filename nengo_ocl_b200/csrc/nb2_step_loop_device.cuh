// Device side of the persistent step loop (see nb2_step_loop.cu): phase records, the bounded
// grid barrier and the loop itself, shared by the multi-CTA kernel (nb2_step_loop.cu, global
// loads cached in L2 only) and the single-CTA kernel (nb2_step_loop_single.cu).
#pragma once
#include "nb2_common.cuh"
#include "nb2_phase_bodies.cuh"
#include "nb2_fused_body.cuh"
#include "nb2_gemv_block_body.cuh"

#define LOOP_THREADS 256
#define LOOP_MIN_BLOCKS 3
#define NB2_LOOP_SPIN_LIMIT (1u << 22)
#ifndef NB2_STEP_LOOP_MAX_PHASES
#define NB2_STEP_LOOP_MAX_PHASES 64
#endif

enum {
  PH_TIMEUPDATE = 0,
  PH_GATHER_SUM,
  PH_DIRECT,
  PH_FUSED_LARGE,
  PH_FUSED_SMALL,
  PH_GEMV_CTA,
  PH_GEMV_WARP,
  PH_PROBES,
  PH_FILTER,
  PH_PRESENT,
};

struct Nb2FusedArgs {
  int n_ens;
  const int* ids;
  const int* ens_table;
  const int* term_table;
  const int* conn_table;
  float* data;
  float dt, dt_inv;
};

struct StepPhase {
  int kind;
  int n_vblocks;
  int barrier;  // a grid barrier stands before this phase
  int pad;
  union Args {
    Nb2TimeupdateArgs timeupdate;
    Nb2GatherArgs gather;
    Nb2DirectArgs direct;
    Nb2FusedArgs fused;
    GemvBlockParams gemv;
    Nb2ProbesArgs probes;
    Nb2FilterArgs filter;
    Nb2PresentArgs present;
    __host__ __device__ Args() {}
  } a;
  __host__ __device__ StepPhase() {}
};

union LoopPool {
  FusedSmem<256, FUSED_MAX_N> large;
  FusedSmem<32, FUSED_SMALL_N> small;
  GemvBlockSmem gemv;
  __device__ LoopPool() {}
};

// All CTAs of the grid meet here.  Returns false when the wait ran out (or another CTA's did).
// `extra`: arrivals expected beyond the grid's own (0 in every real run; the self-test of the
// time-out path passes 1, so that the wait can only run out).
__device__ __forceinline__ bool loop_barrier(unsigned* counter, unsigned& target, int* status, int* s_flag,
                                             int extra) {
  __syncthreads();
  if (threadIdx.x == 0) {
    target += gridDim.x + extra;
    __threadfence();
    atomicAdd(counter, 1u);
    unsigned spins = 0;
    bool ok = true;
    while ((int)(*(volatile unsigned*)counter - target) < 0) {
      if (++spins > NB2_LOOP_SPIN_LIMIT || *(volatile int*)status != 0) {
        atomicCAS(status, 0, NB2_ERR_TIMEOUT);
        ok = false;
        break;
      }
    }
    __threadfence();
    *s_flag = ok ? 1 : 0;
  }
  __syncthreads();
  return *s_flag != 0;
}

// SINGLE: the grid is one CTA; a barrier is then a CTA barrier and nothing is read that another
// multiprocessor wrote, so the translation unit may keep the default (L1) caching of global loads.
template <bool SINGLE>
__device__ __forceinline__ void nb2_step_loop_device(unsigned char* dyn, const StepPhase* __restrict__ phases,
                                                     int n_phases, int n_steps, unsigned* counter, int* status,
                                                     int barrier_extra = 0) {
  LoopPool* pool = reinterpret_cast<LoopPool*>(dyn);
  StepPhase* s_ph = reinterpret_cast<StepPhase*>(dyn + ((sizeof(LoopPool) + 15) & ~size_t(15)));
  __shared__ int s_flag;
  const int tid = threadIdx.x;
  {  // the phase list is read every step: keep it in shared memory
    const int* src = reinterpret_cast<const int*>(phases);
    int* dst = reinterpret_cast<int*>(s_ph);
    for (int i = tid; i < n_phases * (int)(sizeof(StepPhase) / 4); i += LOOP_THREADS) dst[i] = src[i];
  }
  __syncthreads();
  unsigned target = 0;
  const int G = SINGLE ? 1 : gridDim.x;
  for (int step = 0; step < n_steps; ++step) {
    for (int ph = 0; ph < n_phases; ++ph) {
      const StepPhase& P = s_ph[ph];
      if (P.barrier && !(step == 0 && ph == 0)) {
        if (SINGLE) __syncthreads();
        else if (!loop_barrier(counter, target, status, &s_flag, barrier_extra)) return;
      }
      const int nvb = P.n_vblocks;
      switch (P.kind) {
        case PH_TIMEUPDATE:
          if (blockIdx.x == 0) nb2_timeupdate_body(P.a.timeupdate, 0, tid);
          break;
        case PH_GATHER_SUM:
          for (int vb = blockIdx.x; vb < nvb; vb += G) nb2_gather_sum_body(P.a.gather, vb, tid);
          break;
        case PH_DIRECT:
          for (int vb = blockIdx.x; vb < nvb; vb += G) nb2_direct_body(P.a.direct, vb * LOOP_THREADS + tid);
          break;
        case PH_FUSED_LARGE: {
          const Nb2FusedArgs& f = P.a.fused;
          for (int vb = blockIdx.x; vb < nvb; vb += G) {
            nb2_ensemble_step_body<256, FUSED_MAX_N, false>(&pool->large, vb, f.n_ens, f.ids, f.ens_table, f.term_table,
                                                            f.conn_table, f.data, f.dt, f.dt_inv);
            __syncthreads();
          }
        } break;
        case PH_FUSED_SMALL: {
          const Nb2FusedArgs& f = P.a.fused;
          for (int vb = blockIdx.x; vb < nvb; vb += G) {
            nb2_ensemble_step_body<32, FUSED_SMALL_N, false>(&pool->small, vb, f.n_ens, f.ids, f.ens_table, f.term_table,
                                                             f.conn_table, f.data, f.dt, f.dt_inv);
            __syncthreads();
          }
        } break;
        case PH_GEMV_CTA:
          for (int vb = blockIdx.x; vb < nvb; vb += G) {
            nb2_gemv_block_cta_body<false>(&pool->gemv, P.a.gemv, vb);
            __syncthreads();
          }
          break;
        case PH_GEMV_WARP:
          for (int vb = blockIdx.x; vb < nvb; vb += G) nb2_gemv_block_warp_body<false>(P.a.gemv, vb);
          break;
        case PH_PROBES:
          for (int vb = blockIdx.x; vb < nvb; vb += G) {
            const float countdown = P.a.probes.countdowns[vb];
            const int bufpos = P.a.probes.bufpositions[vb];
            __syncthreads();  // every thread has read the counters before thread 0 rewrites them
            nb2_probes_body(P.a.probes, vb, tid, LOOP_THREADS, countdown, bufpos);
          }
          break;
        case PH_FILTER:
          for (int vb = blockIdx.x; vb < nvb; vb += G) nb2_filter_fast_body(P.a.filter, vb, tid, LOOP_THREADS);
          break;
        case PH_PRESENT: {
          // min(width, 256) threads per item; an item wider than the CTA is walked with a stride
          const int w = min(P.a.present.width, LOOP_THREADS);
          for (int vb = blockIdx.x; vb < nvb; vb += G)
            nb2_presentinput_body(P.a.present, vb * (LOOP_THREADS / w) + tid / w, tid % w, w);
        } break;
        default:
          break;
      }
    }
  }
}

