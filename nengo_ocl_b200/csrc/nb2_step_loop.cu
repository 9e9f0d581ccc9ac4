// Persistent step loop: a whole simulation step, repeated n times, in ONE
// cooperative kernel launch.
//
// The reference replays its plan list once per step (nengo_ocl/plan.py:137-149:
// enqueue every kernel of every plan, n times); a captured CUDA graph does the
// same with one submission per step, but every kernel of the step still pays a
// launch gap of a few microseconds, which is most of the step for a model that
// fits in L2.  Here the plans of a step become PHASES of one kernel: every CTA
// walks the virtual blocks of a phase (the blocks the plan's own kernel would
// launch) with a stride of the grid size, and a grid-wide barrier stands only
// where a phase depends on one before it (the host marks those).  The phase
// bodies are the same device functions that the plans' own kernels call
// (nb2_phase_bodies.cuh, nb2_fused_body.cuh, nb2_gemv_block_body.cuh), so a step
// computes bit-identical values either way.
//
// Memory visibility: a phase reads what other CTAs wrote in earlier phases of
// the same launch.  The barrier is a release/acquire pair through one counter
// (fence, atomic add, wait, fence, CTA barrier), no body uses the non-coherent
// load path for signal data (template argument NC = false), and this
// translation unit is compiled with global loads cached in L2 only
// (-Xptxas -dlcm=cg), so no load can be served from a stale L1 line.
//
// The barrier wait is bounded: a CTA that does not see all arrivals within
// NB2_LOOP_SPIN_LIMIT polls records NB2_ERR_TIMEOUT in the loop's status word and
// returns (the others follow at their next barrier).  The launch is cooperative,
// so all CTAs of the grid are resident and the wait normally lasts a microsecond.
#include <string.h>
#include <vector>
#include "nb2_step_loop_device.cuh"
#include "../../include/nengo_b200.h"

__global__ void __launch_bounds__(LOOP_THREADS, LOOP_MIN_BLOCKS)
nb2_step_loop_kernel(const StepPhase* __restrict__ phases, int n_phases, int n_steps, unsigned* counter, int* status,
                     int barrier_extra) {
  extern __shared__ __align__(16) unsigned char dyn[];
  nb2_step_loop_device<false>(dyn, phases, n_phases, n_steps, counter, status, barrier_extra);
}

// defined in nb2_step_loop_single.cu (compiled with the default load caching)
cudaError_t nb2_step_loop_single_prepare(size_t smem);
cudaError_t nb2_step_loop_single_launch(const StepPhase* phases, int n_phases, int n_steps, unsigned* counter,
                                        int* status, size_t smem, cudaStream_t s);

// ---- host side -----------------------------------------------------------------------
struct Nb2StepLoop {
  std::vector<StepPhase> phases;
  StepPhase* d_phases = nullptr;
  unsigned* d_counter = nullptr;  // [0] barrier counter, [1] status word
  int grid = 0;  // 1: the single-CTA kernel
  size_t smem = 0;
  int device = -1;
};

static Nb2StepLoop* loop_of(void* h) { return static_cast<Nb2StepLoop*>(h); }

static StepPhase& new_phase(Nb2StepLoop* L, int kind, int n_vblocks, int barrier) {
  StepPhase p;
  memset(&p, 0, sizeof(p));
  p.kind = kind;
  p.n_vblocks = n_vblocks;
  p.barrier = barrier ? 1 : 0;
  L->phases.push_back(p);
  return L->phases.back();
}

#define LOOP_OPEN(L)                                    \
  NB2_REQUIRE((L) != NULL, "loop");                     \
  NB2_REQUIRE((L)->d_phases == NULL, "the loop is already finalized")

extern "C" int nb2_step_loop_create(void** loop) {
  NB2_REQUIRE(loop != NULL, "loop");
  *loop = new Nb2StepLoop();
  return NB2_OK;
}

extern "C" int nb2_step_loop_destroy(void* loop) {
  Nb2StepLoop* L = loop_of(loop);
  if (!L) return NB2_OK;
  if (L->d_phases) cudaFree(L->d_phases);
  if (L->d_counter) cudaFree(L->d_counter);
  delete L;
  return NB2_OK;
}

extern "C" int nb2_step_loop_add_timeupdate(void* loop, int barrier, float* step, float* time, double dt) {
  Nb2StepLoop* L = loop_of(loop);
  LOOP_OPEN(L);
  NB2_REQUIRE(step && time, "null pointer");
  StepPhase& p = new_phase(L, PH_TIMEUPDATE, 1, barrier);
  p.a.timeupdate.step = step;
  p.a.timeupdate.time = time;
  p.a.timeupdate.dt = dt;
  return NB2_OK;
}

extern "C" int nb2_step_loop_add_gather_sum(void* loop, int barrier, int n_blocks, int width, const int* blocks,
                                            const int* src_starts, float* data) {
  Nb2StepLoop* L = loop_of(loop);
  LOOP_OPEN(L);
  NB2_REQUIRE(blocks && src_starts && data, "null pointer");
  NB2_REQUIRE(width >= 1 && width <= 256 && (width & (width - 1)) == 0, "width must be a power of two <= 256");
  const int per_cta = 256 / width;
  StepPhase& p = new_phase(L, PH_GATHER_SUM, (n_blocks + per_cta - 1) / per_cta, barrier);
  p.a.gather.n_blocks = n_blocks;
  p.a.gather.width = width;
  p.a.gather.blocks = reinterpret_cast<const int4*>(blocks);
  p.a.gather.src_starts = src_starts;
  p.a.gather.data = data;
  return NB2_OK;
}

extern "C" int nb2_step_loop_add_direct(void* loop, int barrier, int n_items, const int* prog, int n_ops, int max_depth,
                                        const double* consts, int out_dim, const int* in0_starts, const float* in0,
                                        const int* in1_starts, const float* in1, const int* out_starts, float* out) {
  Nb2StepLoop* L = loop_of(loop);
  LOOP_OPEN(L);
  NB2_REQUIRE(prog && out_starts && out && out_dim >= 1, "null pointer");
  NB2_REQUIRE(max_depth >= 0 && max_depth <= NB2_DIRECT_STACK, "program needs a deeper evaluation stack");
  NB2_REQUIRE((in0 == NULL) == (in0_starts == NULL) && (in1 == NULL) == (in1_starts == NULL),
              "input buffer/starts mismatch");
  StepPhase& p = new_phase(L, PH_DIRECT, (n_items + LOOP_THREADS - 1) / LOOP_THREADS, barrier);
  Nb2DirectArgs& a = p.a.direct;
  a.n_items = n_items;
  a.prog = reinterpret_cast<const int2*>(prog);
  a.n_ops = n_ops;
  a.consts = consts;
  a.in0_starts = in0_starts;
  a.in0 = in0;
  a.in1_starts = in1_starts;
  a.in1 = in1;
  a.out_starts = out_starts;
  a.out = out;
  return NB2_OK;
}

extern "C" int nb2_step_loop_add_ensemble_step(void* loop, int barrier, int n_large, const int* large_ids, int n_small,
                                               const int* small_ids, const int* ens_table, const int* term_table,
                                               const int* conn_table, float* data, double dt) {
  Nb2StepLoop* L = loop_of(loop);
  LOOP_OPEN(L);
  NB2_REQUIRE(ens_table && term_table && conn_table && data, "null pointer");
  NB2_REQUIRE(dt > 0, "dt");
  NB2_REQUIRE((n_large == 0 || large_ids) && (n_small == 0 || small_ids), "ids");
  for (int variant = 0; variant < 2; ++variant) {
    const int n = variant == 0 ? n_large : n_small;
    if (n <= 0) continue;
    StepPhase& p = new_phase(L, variant == 0 ? PH_FUSED_LARGE : PH_FUSED_SMALL, variant == 0 ? n : (n + 7) / 8, barrier);
    barrier = 0;  // the two variants update different ensembles
    Nb2FusedArgs& a = p.a.fused;
    a.n_ens = n;
    a.ids = variant == 0 ? large_ids : small_ids;
    a.ens_table = ens_table;
    a.term_table = term_table;
    a.conn_table = conn_table;
    a.data = data;
    a.dt = (float)dt;
    a.dt_inv = (float)(1.0 / dt);
  }
  return NB2_OK;
}

extern "C" int nb2_step_loop_add_gemv_block(void* loop, int barrier, const int* gstructure, int gstride, int D,
                                            const int* xstrides, const int* cta_units, int n_cta, const int* warp_units,
                                            int n_warp, const float* A, const float* X, const float* Yin, float* Y,
                                            double alpha, double beta, double gamma) {
  Nb2StepLoop* L = loop_of(loop);
  LOOP_OPEN(L);
  if (n_cta == 0 && n_warp == 0) return NB2_OK;
  NB2_REQUIRE(gstructure && A && X && Yin && Y, "null pointer");
  NB2_REQUIRE(D >= 0 && gstride >= 4 * D + 5, "table layout");
  NB2_REQUIRE((n_cta == 0 || cta_units) && (n_warp == 0 || warp_units), "units");
  for (int variant = 0; variant < 2; ++variant) {
    const int n = variant == 0 ? n_cta : n_warp;
    if (n <= 0) continue;
    StepPhase& p = new_phase(L, variant == 0 ? PH_GEMV_CTA : PH_GEMV_WARP,
                             variant == 0 ? n : (n + GB_WARPS - 1) / GB_WARPS, barrier);
    barrier = 0;  // the two unit lists cover different output rows
    GemvBlockParams& g = p.a.gemv;
    g.gstructure = gstructure;
    g.xstrides = xstrides;
    g.worklist = reinterpret_cast<const int4*>(variant == 0 ? cta_units : warp_units);
    g.n_units = n;
    g.gstride = gstride;
    g.D = D;
    g.A = A;
    g.X = X;
    g.Yin = Yin;
    g.Y = Y;
    g.alpha = alpha;
    g.beta = beta;
    g.gamma = gamma;
  }
  return NB2_OK;
}

extern "C" int nb2_step_loop_add_probes(void* loop, int barrier, int n_probes, int block_size, float* countdowns,
                                        int* bufpositions, const float* periods, const int* Xstarts,
                                        const int* Xshape0s, const int* Xshape1s, const int* Xstride0s,
                                        const int* Xstride1s, const float* X, const int* Ystarts, float* Y) {
  Nb2StepLoop* L = loop_of(loop);
  LOOP_OPEN(L);
  (void)block_size;
  if (n_probes == 0) return NB2_OK;
  NB2_REQUIRE(countdowns && bufpositions && periods && Xstarts && Xshape0s && Xshape1s && Xstride0s && Xstride1s &&
                  X && Ystarts && Y,
              "null pointer");
  StepPhase& p = new_phase(L, PH_PROBES, n_probes, barrier);
  Nb2ProbesArgs& a = p.a.probes;
  a.countdowns = countdowns;
  a.bufpositions = bufpositions;
  a.periods = periods;
  a.Xstarts = Xstarts;
  a.Xshape0s = Xshape0s;
  a.Xshape1s = Xshape1s;
  a.Xstride0s = Xstride0s;
  a.Xstride1s = Xstride1s;
  a.X = X;
  a.Ystarts = Ystarts;
  a.Y = Y;
  return NB2_OK;
}

extern "C" int nb2_step_loop_add_linearfilter(void* loop, int barrier, int n_blocks, int block_size, int uses_buf,
                                              const int* offsets, const int* shape0s, const int* shape1s,
                                              const int* Xstride0s, const int* Xstride1s, const int* Xstarts,
                                              const float* X, const int* Ystride0s, const int* Ystride1s,
                                              const int* Ystarts, float* Y, const int* Ashape0s, const int* Astarts,
                                              const float* A, const int* Bshape0s, const int* Bstarts, const float* B,
                                              const int* Xbufstarts, float* Xbuf, const int* Ybufstarts, float* Ybuf,
                                              int* Xbufpos, int* Ybufpos) {
  Nb2StepLoop* L = loop_of(loop);
  LOOP_OPEN(L);
  (void)Xbufstarts; (void)Xbuf; (void)Ybufstarts; (void)Ybuf; (void)Xbufpos; (void)Ybufpos;
  if (n_blocks == 0) return NB2_OK;
  if (uses_buf) {
    nb2_set_error("filters with ring buffers run as their own launches, not as a phase of the step loop");
    return NB2_ERR_LIMIT;
  }
  NB2_REQUIRE(block_size >= 1 && block_size <= 1024, "block_size");
  NB2_REQUIRE(offsets && shape0s && shape1s && Xstride0s && Xstride1s && Xstarts && X && Ystride0s && Ystride1s &&
                  Ystarts && Y && Ashape0s && Astarts && A && Bshape0s && Bstarts && B,
              "null pointer");
  StepPhase& p = new_phase(L, PH_FILTER, n_blocks, barrier);
  Nb2FilterArgs& a = p.a.filter;
  a.block_size = block_size;
  a.offsets = offsets;
  a.shape0s = shape0s;
  a.shape1s = shape1s;
  a.Xstride0s = Xstride0s;
  a.Xstride1s = Xstride1s;
  a.Xstarts = Xstarts;
  a.x = X;
  a.Ystride0s = Ystride0s;
  a.Ystride1s = Ystride1s;
  a.Ystarts = Ystarts;
  a.y = Y;
  a.Ashape0s = Ashape0s;
  a.Astarts = Astarts;
  a.Adata = A;
  a.Bshape0s = Bshape0s;
  a.Bstarts = Bstarts;
  a.Bdata = B;
  return NB2_OK;
}

extern "C" int nb2_step_loop_add_presentinput(void* loop, int barrier, int n_items, int block_size, const float* pres_t,
                                              double dt, const int* Yshape0s, const int* Ystarts, float* Y,
                                              const int* Tstarts, const float* T, const int* Sshape0s,
                                              const int* Sstarts, const int* Sstride0s, const float* S) {
  Nb2StepLoop* L = loop_of(loop);
  LOOP_OPEN(L);
  if (n_items == 0) return NB2_OK;
  NB2_REQUIRE(block_size >= 1 && block_size <= 1024, "block_size");
  NB2_REQUIRE(Yshape0s && Ystarts && Y && Tstarts && T && Sshape0s && Sstarts && S, "null pointer");
  int width = 1;
  while (width < block_size) width <<= 1;
  const int per_vb = width < LOOP_THREADS ? LOOP_THREADS / width : 1;
  StepPhase& p = new_phase(L, PH_PRESENT, (n_items + per_vb - 1) / per_vb, barrier);
  Nb2PresentArgs& a = p.a.present;
  a.n_items = n_items;
  a.width = width;
  a.pres_t = pres_t;
  a.dt = (float)dt;
  a.Yshape0s = Yshape0s;
  a.Ystarts = Ystarts;
  a.Y = Y;
  a.Tstarts = Tstarts;
  a.T = T;
  a.Sshape0s = Sshape0s;
  a.Sstarts = Sstarts;
  a.Sstride0s = Sstride0s;
  a.S = S;
  return NB2_OK;
}

extern "C" int nb2_step_loop_finalize(void* loop, int max_ctas) {
  Nb2StepLoop* L = loop_of(loop);
  LOOP_OPEN(L);
  NB2_REQUIRE(!L->phases.empty() && L->phases.size() <= NB2_STEP_LOOP_MAX_PHASES, "number of phases");
  NB2_CUDA(cudaGetDevice(&L->device));
  L->smem = ((sizeof(LoopPool) + 15) & ~size_t(15)) + L->phases.size() * sizeof(StepPhase);
  // the attribute belongs to the kernel, not to this loop: always ask for what the longest phase list needs
  const size_t smem_max = ((sizeof(LoopPool) + 15) & ~size_t(15)) + NB2_STEP_LOOP_MAX_PHASES * sizeof(StepPhase);
  int widest = 1;
  for (const StepPhase& p : L->phases) widest = p.n_vblocks > widest ? p.n_vblocks : widest;
  if (widest == 1 || max_ctas == 1) {
    L->grid = 1;
    NB2_CUDA(nb2_step_loop_single_prepare(smem_max));
  } else {
    int coop = 0, sms = 0;
    NB2_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, L->device));
    NB2_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, L->device));
    if (!coop) {
      nb2_set_error("the device does not support cooperative launches");
      return NB2_ERR_LIMIT;
    }
    NB2_CUDA(cudaFuncSetAttribute(nb2_step_loop_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
    int per_sm = 0;
    NB2_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, nb2_step_loop_kernel, LOOP_THREADS, L->smem));
    NB2_REQUIRE(per_sm >= 1, "the step loop kernel does not fit on a multiprocessor");
    int grid = per_sm * sms;  // every CTA must be resident: the barrier waits for all of them
    if (widest < grid) grid = widest;
    if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
    L->grid = grid;
  }
  NB2_CUDA(cudaMalloc(&L->d_phases, L->phases.size() * sizeof(StepPhase)));
  NB2_CUDA(cudaMemcpy(L->d_phases, L->phases.data(), L->phases.size() * sizeof(StepPhase), cudaMemcpyHostToDevice));
  NB2_CUDA(cudaMalloc(&L->d_counter, 2 * sizeof(unsigned)));
  NB2_CUDA(cudaMemset(L->d_counter, 0, 2 * sizeof(unsigned)));
  return NB2_OK;
}

static int step_loop_launch(Nb2StepLoop* L, cudaStream_t s, int n_steps, int barrier_extra) {
  const StepPhase* phases = L->d_phases;
  int n_phases = (int)L->phases.size();
  unsigned* counter = L->d_counter;
  int* status = reinterpret_cast<int*>(L->d_counter + 1);
  if (L->grid == 1) {
    NB2_CUDA(nb2_step_loop_single_launch(phases, n_phases, n_steps, counter, status, L->smem, s));
    return NB2_OK;
  }
  NB2_CUDA(cudaMemsetAsync(L->d_counter, 0, sizeof(unsigned), s));  // the barrier counter; the status word is sticky
  void* args[] = {&phases, &n_phases, &n_steps, &counter, &status, &barrier_extra};
  NB2_CUDA(cudaLaunchCooperativeKernel((const void*)nb2_step_loop_kernel, dim3(L->grid), dim3(LOOP_THREADS), args,
                                       L->smem, s));
  return NB2_OK;
}

extern "C" int nb2_step_loop_run(void* loop, void* stream, int n_steps) {
  Nb2StepLoop* L = loop_of(loop);
  NB2_REQUIRE(L != NULL && L->d_phases != NULL, "the loop is not finalized");
  if (n_steps <= 0) return NB2_OK;
  return step_loop_launch(L, nb2_stream(stream), n_steps, 0);
}

extern "C" int nb2_step_loop_wait_selftest(void* loop, void* stream) {
  Nb2StepLoop* L = loop_of(loop);
  NB2_REQUIRE(L != NULL && L->d_phases != NULL, "the loop is not finalized");
  NB2_REQUIRE(L->grid > 1, "the single-CTA form has no grid barrier");
  return step_loop_launch(L, nb2_stream(stream), 2, 1);
}

extern "C" int nb2_step_loop_clear_status(void* loop, void* stream) {
  Nb2StepLoop* L = loop_of(loop);
  NB2_REQUIRE(L != NULL && L->d_counter != NULL, "the loop is not finalized");
  NB2_CUDA(cudaMemsetAsync(L->d_counter, 0, 2 * sizeof(unsigned), nb2_stream(stream)));
  return NB2_OK;
}

extern "C" int nb2_step_loop_info(void* loop, int* n_phases, int* n_barriers, int* grid, int* total_vblocks) {
  Nb2StepLoop* L = loop_of(loop);
  NB2_REQUIRE(L != NULL, "loop");
  int nb = 0, total = 0;
  for (const StepPhase& p : L->phases) {
    nb += p.barrier;
    total += p.n_vblocks;
  }
  if (total_vblocks) *total_vblocks = total;
  if (n_phases) *n_phases = (int)L->phases.size();
  if (n_barriers) *n_barriers = nb;
  if (grid) *grid = L->grid;
  return NB2_OK;
}

extern "C" int nb2_step_loop_status(void* loop, void* stream, int* status) {
  Nb2StepLoop* L = loop_of(loop);
  NB2_REQUIRE(L != NULL && L->d_counter != NULL && status != NULL, "the loop is not finalized");
  cudaStream_t s = nb2_stream(stream);
  NB2_CUDA(cudaMemcpyAsync(status, L->d_counter + 1, sizeof(int), cudaMemcpyDeviceToHost, s));
  NB2_CUDA(cudaStreamSynchronize(s));
  if (*status != 0) nb2_set_error("the step loop gave up waiting at a grid barrier (status %d)", *status);
  return NB2_OK;
}
