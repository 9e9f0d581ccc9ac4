// Pipelined ragged gather-GEMV for sm_100a (the main GEMV path).
//
//     Y[k] = gamma + beta * Y_in[k] + alpha * sum_j A[a_kj] . X[x_kj]
//
// Same math as the reference's four OpenCL GEMV variants (nengo_ocl/
// clra_gemv.py:264-1175).  The kernel is bandwidth-bound (0.5 flop/byte), so
// the design is about keeping HBM busy:
//
//  * The host cuts every output item into work records of roughly equal bytes
//    (<= NB2_PIPE_STAGE_FLOATS staged matrix elements, <= 4 (term, column
//    chunk) segments).  Records of one row range form a chain (several records
//    when an item has many terms or long rows).
//  * Persistent CTAs (a multiple of the SM count) each own a contiguous range
//    of records, balanced by bytes, so neighbouring CTAs stream neighbouring
//    memory.
//  * Inside a CTA eight producer warps and eight consumer warps share a ring of
//    16 shared-memory stages; every consumer warp works on records of its own
//    and owns two stages, so one can load while the other is consumed.  A
//    producer reads the next record and launches its copies into shared memory
//    without waiting for them: the contiguous matrix rows go
//    through 1-D bulk async copies (cp.async.bulk, completion counted in bytes
//    on an mbarrier), ragged heads/tails, gathered X segments and the Y_in rows
//    through 4-byte cp.async copies tracked by the same mbarrier.
//  * Each consumer thread owns up to four output rows and a strided subset of
//    the columns, loads each x value once for its four rows, reads the staged
//    rows with a per-thread column rotation (bank-conflict avoidance), keeps
//    the running sums in registers across all segments and records of a chain
//    and finishes with one shuffle reduction and a single-pass epilogue.  There
//    is no scratch buffer and no second reduction kernel.
//
// Every mbarrier wait is bounded; on timeout the CTA records NB2_ERR_TIMEOUT
// in the status word, stops issuing, drains its own cp.async copies and exits.
#include "nb2_common.cuh"
#include "../../include/nengo_b200.h"

#define PIPE_STAGES NB2_PIPE_STAGES
#define PIPE_NW NB2_PIPE_CONSUMER_WARPS  // consumer warps, each works on its own record
#define PIPE_NP 8                        // producer warps (record i is issued by warp i % NP)
#define PIPE_CONSUMERS 32                // threads that share one record
#define PIPE_ROWS_PER_THREAD 4
#define PIPE_THREADS (32 * (PIPE_NW + PIPE_NP))
#define PIPE_A NB2_PIPE_STAGE_FLOATS  // staged matrix floats per stage
#define PIPE_X NB2_PIPE_XBUF          // staged x floats per stage
#define PIPE_R NB2_PIPE_RMAX          // max rows per record
#define PIPE_REC 32                   // ints per record
#define PIPE_MAXSEG 4
#define PIPE_SPIN_LIMIT (1 << 22)

// Record i uses stage i % STAGES and is consumed by warp i % NW.  With STAGES a
// multiple of NW every stage is always consumed by the same warp, so a warp can
// only wait for phase r of a stage after it has itself consumed phase r-1:
// parity waits can never be a whole round behind.
static_assert(PIPE_STAGES % PIPE_NW == 0, "each stage must belong to one consumer warp");
static_assert(PIPE_STAGES % PIPE_NP == 0, "each stage must belong to one producer warp");

struct PipeParams {
  const int* records;  // [n_records][32]
  const int2* ranges;  // per CTA: [begin, end) record indices
  const float* A;
  const float* X;
  const float* Yin;
  float* Y;
  double alpha, beta, gamma;
  const float* alphas;
  const float* betas;
  const float* gammas;
  int* status;
};

struct __align__(128) PipeStage {
  float a[PIPE_A];
  float x[PIPE_X];
  float yin[PIPE_R];
  int rec[PIPE_REC];
};

__device__ __forceinline__ uint32_t pipe_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(pipe_smem(dst)), "l"(src) : "memory");
}

// Bounded parity wait. Returns false on timeout.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t parity) {
  uint32_t done = 0;
  for (int spins = 0; spins < PIPE_SPIN_LIMIT; ++spins) {
    asm volatile(
        "{\n .reg .pred q;\n mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n selp.u32 %0, 1, 0, q;\n}"
        : "=r"(done)
        : "r"(pipe_smem(bar)), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ float pipe_epilogue(const PipeParams& p, int bb, float yin, float sum) {
  float pre;
  if (p.betas) pre = p.betas[bb] * yin;
  else pre = (p.beta != 0.0) ? (float)(p.beta * (double)yin) : 0.0f;
  if (p.gammas) pre += p.gammas[bb];
  else if (p.gamma != 0.0) pre = (float)((double)pre + p.gamma);
  if (p.alphas) return pre + p.alphas[bb] * sum;
  return (float)((double)pre + p.alpha * (double)sum);
}

__global__ void __launch_bounds__(PIPE_THREADS, 1) nb2_gemv_pipe_kernel(const PipeParams p) {
  extern __shared__ __align__(128) unsigned char pipe_raw[];
  PipeStage* stages = reinterpret_cast<PipeStage*>(pipe_raw);
  __shared__ __align__(8) unsigned long long full_bar[PIPE_STAGES];
  __shared__ __align__(8) unsigned long long empty_bar[PIPE_STAGES];
  __shared__ int s_abort;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int2 range = p.ranges[blockIdx.x];
  const int n = range.y - range.x;

  if (tid == 0) {
    for (int s = 0; s < PIPE_STAGES; ++s) {
      // full: 32 producer lanes (cp.async completion arrivals) + 1 expect_tx arrival
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pipe_smem(&full_bar[s])), "r"(33));
      // empty: one arrival by the consumer warp that owned the record
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pipe_smem(&empty_bar[s])), "r"(1));
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int wid = tid >> 5;
  if (wid >= PIPE_NW) {
    // ======================= producer warps =======================
    const int first = wid - PIPE_NW;
    int next = first < n ? __ldg(p.records + (size_t)(range.x + first) * PIPE_REC + lane) : 0;
    for (int i = first; i < n; i += PIPE_NP) {
      const int s = i % PIPE_STAGES;
      const int round = i / PIPE_STAGES;
      const int my = next;  // record i; this warp's next record is fetched while this one is issued
      if (i + PIPE_NP < n) next = __ldg(p.records + (size_t)(range.x + i + PIPE_NP) * PIPE_REC + lane);
      if (round > 0) {
        if (!mbar_wait(&empty_bar[s], (uint32_t)((round - 1) & 1)) || *(volatile int*)&s_abort) {
          if (lane == 0) { s_abort = 1; if (p.status) atomicExch(p.status, NB2_ERR_TIMEOUT); }
          break;
        }
      }
      PipeStage& st = stages[s];
      st.rec[lane] = my;
      const int flags = __shfl_sync(0xffffffffu, my, 0);
      const int R = __shfl_sync(0xffffffffu, my, 1);
      const int y_in = __shfl_sync(0xffffffffu, my, 2);
      const int nseg = __shfl_sync(0xffffffffu, my, 5);
      uint32_t bulk_bytes = 0;
      for (int q = 0; q < nseg; ++q) {
        const int gidx = __shfl_sync(0xffffffffu, my, 8 + 6 * q + 0);
        const int w = __shfl_sync(0xffffffffu, my, 8 + 6 * q + 1);
        const int s0 = __shfl_sync(0xffffffffu, my, 8 + 6 * q + 2);
        const int xstart = __shfl_sync(0xffffffffu, my, 8 + 6 * q + 3);
        const int xstride = __shfl_sync(0xffffffffu, my, 8 + 6 * q + 4);
        const int aoff_xoff = __shfl_sync(0xffffffffu, my, 8 + 6 * q + 5);
        const int aoff = aoff_xoff & 0xffff;
        const int xoff = aoff_xoff >> 16;
        for (int c = lane; c < w; c += 32) cp_async4(&st.x[xoff + c], p.X + xstart + (size_t)c * xstride);
        const int len = R * w;
        const float* src = p.A + gidx;
        float* dst = st.a + aoff;
        if (s0 == w || R == 1) {
          const int head = min(len, (4 - (gidx & 3)) & 3);
          const int body = (len - head) & ~3;
          const int tail0 = head + body;
          if (lane < head) cp_async4(dst + lane, src + lane);
          if (lane >= 8 && lane - 8 < len - tail0) cp_async4(dst + tail0 + lane - 8, src + tail0 + lane - 8);
          if (body > 0 && lane == 0) {
            asm volatile(
                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
                    "r"(pipe_smem(dst + head)), "l"(src + head), "r"((uint32_t)body * 4u),
                "r"(pipe_smem(&full_bar[s]))
                : "memory");
          }
          bulk_bytes += (uint32_t)body * 4u;
        } else {
          for (int e = lane; e < len; e += 32) {
            const int r = e / w;
            const int c = e - r * w;
            cp_async4(dst + e, src + (size_t)r * s0 + c);
          }
        }
      }
      if (flags & 2)
        for (int r = lane; r < R; r += 32) cp_async4(&st.yin[r], p.Yin + y_in + r);
      // this lane's cp.async copies arrive on the barrier when they land
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(pipe_smem(&full_bar[s]))
                   : "memory");
      __syncwarp();  // record words of all lanes are written before the release below
      if (lane == 0) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pipe_smem(&full_bar[s])),
                     "r"(bulk_bytes)
                     : "memory");
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    return;
  }

  // ========================= consumer warps =========================
  // Thread mapping per record (rows R <= 512, fixed along a chain so the sums
  // stay in registers): record i of the CTA's list belongs to consumer warp
  // i % NW (the host interleaves the chains accordingly); each lane owns up to
  // 4 rows row0 + j*P and the columns g, g+G, g+2G, ... of every segment, with
  // G * P = 32 lanes.  The
  // x value of a column is loaded once and used for the thread's 4 rows.  The
  // column order is rotated per thread so that lanes working on different rows
  // of a warp hit different shared-memory banks.
  float acc[PIPE_ROWS_PER_THREAD] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (int i = wid; i < n; i += PIPE_NW) {
    const int s = i % PIPE_STAGES;
    const uint32_t parity = (uint32_t)((i / PIPE_STAGES) & 1);
    if (!mbar_wait(&full_bar[s], parity)) {
      if (lane == 0) { s_abort = 1; if (p.status) atomicExch(p.status, NB2_ERR_TIMEOUT); }
      break;
    }
    const PipeStage& st = stages[s];
    const int flags = st.rec[0];
    const int R = st.rec[1];
    const int nseg = st.rec[5];
    // G = lanes per row: largest power of two with ceil(R/4) * G <= 128 (at most 32)
    const int quarter = (R + PIPE_ROWS_PER_THREAD - 1) / PIPE_ROWS_PER_THREAD;
    int logG = 0;
    while (logG < 5 && (quarter << (logG + 1)) <= PIPE_CONSUMERS) ++logG;
    const int G = 1 << logG;
    const int P = PIPE_CONSUMERS >> logG;  // rows per pass
    const int g = lane & (G - 1);
    const int row0 = lane >> logG;
    if (flags & 1) {
#pragma unroll
      for (int j = 0; j < PIPE_ROWS_PER_THREAD; ++j) acc[j] = 0.0f;
    }
    if (row0 < R) {
      // rows beyond R re-read the last valid row; their sums are discarded
      int roff[PIPE_ROWS_PER_THREAD];
#pragma unroll
      for (int j = 0; j < PIPE_ROWS_PER_THREAD; ++j) roff[j] = min(row0 + j * P, R - 1);
      for (int q = 0; q < nseg; ++q) {
        const int w = st.rec[8 + 6 * q + 1];
        const int aoff_xoff = st.rec[8 + 6 * q + 5];
        const float* a = st.a + (aoff_xoff & 0xffff) + g;
        const float* x = st.x + (aoff_xoff >> 16) + g;
        const int K = (w - g + G - 1) >> logG;  // columns of this lane
        if (K <= 0) continue;
        const int shift = row0 & ((1 << (31 - __clz(K))) - 1);
        const float* a0 = a + roff[0] * w;
        const float* a1 = a + roff[1] * w;
        const float* a2 = a + roff[2] * w;
        const float* a3 = a + roff[3] * w;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          const int kbeg = half ? 0 : shift;
          const int kend = half ? shift : K;
#pragma unroll 4
          for (int k = kbeg; k < kend; ++k) {
            const int col = k << logG;
            const float xv = x[col];
            acc[0] = fmaf(a0[col], xv, acc[0]);
            acc[1] = fmaf(a1[col], xv, acc[1]);
            acc[2] = fmaf(a2[col], xv, acc[2]);
            acc[3] = fmaf(a3[col], xv, acc[3]);
          }
        }
      }
    }
    if (flags & 2) {
      const int y = st.rec[3];
      const int bb = st.rec[4];
#pragma unroll
      for (int j = 0; j < PIPE_ROWS_PER_THREAD; ++j) {
        float t = acc[j];
        for (int off = G >> 1; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
        const int r = row0 + j * P;
        if (g == 0 && r < R) p.Y[y + r] = pipe_epilogue(p, bb, st.yin[r], t);
      }
    }
    __syncwarp();
    if (lane == 0) {
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pipe_smem(&empty_bar[s])) : "memory");
    }
  }
}

static const size_t kPipeSmem = sizeof(PipeStage) * PIPE_STAGES;

extern "C" int nb2_gemv_pipelined(void* stream, const int* records, int n_records, const int* ranges,
                                  int n_ctas, const float* A, const float* X, const float* Yin, float* Y,
                                  double alpha, double beta, double gamma, const float* alphas,
                                  const float* betas, const float* gammas, int* status) {
  if (n_records == 0 || n_ctas == 0) return NB2_OK;
  NB2_REQUIRE(records && ranges && A && X && Yin && Y, "null pointer");
  static bool optin[64] = {};
  int dev = 0;
  NB2_CUDA(cudaGetDevice(&dev));
  if (dev >= 64 || !optin[dev]) {
    NB2_CUDA(cudaFuncSetAttribute(nb2_gemv_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)kPipeSmem));
    if (dev < 64) optin[dev] = true;
  }
  PipeParams p;
  p.records = records; p.ranges = reinterpret_cast<const int2*>(ranges);
  p.A = A; p.X = X; p.Yin = Yin; p.Y = Y;
  p.alpha = alpha; p.beta = beta; p.gamma = gamma;
  p.alphas = alphas; p.betas = betas; p.gammas = gammas;
  p.status = status;
  nb2_gemv_pipe_kernel<<<n_ctas, PIPE_THREADS, kPipeSmem, nb2_stream(stream)>>>(p);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
