// Pipelined ragged gather-GEMV for sm_100a (the main GEMV path).
//
//     Y[k] = gamma + beta * Y_in[k] + alpha * sum_j A[a_kj] . X[x_kj]
//
// Same math as the reference's four OpenCL GEMV variants (nengo_ocl/
// clra_gemv.py:264-1175).  The kernel is bandwidth-bound (0.5 flop/byte), so
// the design is about keeping as many bytes in flight per SM as shared memory
// allows, with as few instructions per byte as possible:
//
//  * The host cuts every output item into work records of roughly equal bytes
//    (<= NB2_PIPE_STAGE_FLOATS staged floats, <= 4 terms or column chunks,
//    whole rows whenever a row fits).  Records of one row range form a chain
//    (several records when an item has many terms or very long rows).
//  * Persistent CTAs (one per SM) own contiguous ranges of records, balanced
//    by bytes, so neighbouring CTAs stream neighbouring memory.
//  * Every warp of a CTA owns one shared-memory stage and the records
//    i = warp, warp + WARPS, ... of the CTA's range.  Lane 0 fills the stage
//    with nothing but 1-D bulk async copies (cp.async.bulk, completion counted
//    in bytes on the stage's mbarrier): one copy per matrix segment, one per
//    gathered X segment, one for the Y_in rows, and the NEXT record of this
//    warp (so the work description is read from shared memory and never held
//    in registers).  Sources that do not start or end on a 16-byte boundary
//    are copied as the enclosing 16-byte-aligned window and indexed from the
//    remainder, so there are no per-element copies at all.  While one warp
//    waits for its copies the others compute: the 12 stages of a CTA keep
//    about 200 KB in flight per SM.
//  * The warp maps one lane to one output row (up to 4 rows per lane, 32 lanes
//    apart) and walks the row's columns linearly: the x value of a column is one
//    broadcast shared-memory load for the whole warp, row elements are loaded
//    with immediate offsets, the running sums stay in registers across all
//    segments and records of a chain, and the epilogue needs no reduction.
//    Segments whose width is a multiple of 8 would put the lanes of a warp in
//    the same few banks; those walk the columns diagonally instead (lane l
//    starts at column l mod w).  There is no scratch buffer and no second
//    reduction kernel.
//
// Every mbarrier wait is bounded by the global timer; on timeout the warp
// records NB2_ERR_TIMEOUT in the status word and leaves.
#include "nb2_common.cuh"
#include "nb2_pipe.cuh"
#include "../../include/nengo_b200.h"

#define PIPE_NW NB2_PIPE_WARPS  // warps per CTA = stages per CTA; record i belongs to warp i % NW
#define PIPE_ROWS_PER_THREAD 4
#define PIPE_THREADS (32 * PIPE_NW)
#define PIPE_A NB2_PIPE_STAGE_FLOATS  // staged floats per stage (matrix rows and x segments share the pool)
#define PIPE_R NB2_PIPE_RMAX          // max rows per record
#define PIPE_REC 32                   // ints per record
#define PIPE_MAXSEG 4
static_assert(PIPE_R == 32 * PIPE_ROWS_PER_THREAD, "rows per record = 4 rows per lane");
static_assert(PIPE_THREADS <= 1024, "CTA size");

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
  float buf[PIPE_A];
  float yin[PIPE_R + 8];
  int rec[3][PIPE_REC];  // record of turn m in slot m % 3
};

__device__ __forceinline__ float pipe_epilogue(const PipeParams& p, int bb, float yin, float sum) {
  float pre;
  if (p.betas) pre = p.betas[bb] * yin;
  else pre = (p.beta != 0.0) ? (float)(p.beta * (double)yin) : 0.0f;
  if (p.gammas) pre += p.gammas[bb];
  else if (p.gamma != 0.0) pre = (float)((double)pre + p.gamma);
  if (p.alphas) return pre + p.alphas[bb] * sum;
  return (float)((double)pre + p.alpha * (double)sum);
}

// Lane 0 of a warp: fill the warp's stage for turn m (record index i of the CTA's range).
// The record itself is already in st.rec[m % 3] and the warp's next record in the slot after
// it: the matrix windows of that next record are prefetched into L2 now, one whole turn
// before they are copied, so that more bytes are in flight than the stages alone can hold.
// The record two turns ahead rides along with the copies of this turn.
__device__ __forceinline__ void pipe_issue(const PipeParams& p, PipeStage& st, unsigned long long* full,
                                           const int4* rp, int i, int m, int n) {
  const int slot = m % 3;
  const int* r = st.rec[slot];
  const int nseg = r[5];
  const int yin_bytes = r[7];
  const bool more = i + 2 * PIPE_NW < n;
  uint32_t tx = (uint32_t)yin_bytes + (more ? PIPE_REC * 4u : 0u);
  int4 sg[PIPE_MAXSEG];  // window index and bytes of A and X
  int offs[PIPE_MAXSEG];
#pragma unroll
  for (int q = 0; q < PIPE_MAXSEG; ++q) {
    if (q < nseg) {
      const int2 lo = *reinterpret_cast<const int2*>(r + 8 + 6 * q);
      const int2 hi = *reinterpret_cast<const int2*>(r + 8 + 6 * q + 2);
      sg[q] = make_int4(lo.x, lo.y, hi.x, hi.y);
      offs[q] = r[8 + 6 * q + 5];
      tx += (uint32_t)lo.y + (uint32_t)max(hi.y, 0);
    }
  }
  // the stage was read through the generic proxy; order those reads before the async-proxy writes
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pipe_smem(full)), "r"(tx) : "memory");
#pragma unroll
  for (int q = 0; q < PIPE_MAXSEG; ++q) {
    if (q < nseg) {
      bulk_copy(st.buf + ((offs[q] & 0xffff) & ~3), p.A + sg[q].x, (uint32_t)sg[q].y, full);
      if (sg[q].w > 0) bulk_copy(st.buf + ((offs[q] >> 16) & ~3), p.X + sg[q].z, (uint32_t)sg[q].w, full);
    }
  }
  if (yin_bytes > 0) bulk_copy(st.yin, p.Yin + (r[2] & ~3), (uint32_t)yin_bytes, full);
  if (more) bulk_copy(st.rec[(m + 2) % 3], rp + (size_t)(i + 2 * PIPE_NW) * 8, PIPE_REC * 4u, full);
  if (i + PIPE_NW < n) {
    const int* rn = st.rec[(m + 1) % 3];
    const int nn = rn[5];
#pragma unroll
    for (int q = 0; q < PIPE_MAXSEG; ++q) {
      if (q < nn) {
        const int2 lo = *reinterpret_cast<const int2*>(rn + 8 + 6 * q);
        l2_prefetch(p.A + lo.x, (uint32_t)lo.y);
      }
    }
  }
}

__global__ void __launch_bounds__(PIPE_THREADS, NB2_PIPE_CTAS_PER_SM) nb2_gemv_pipe_kernel(const PipeParams p) {
  nb2_pdl_enter();
  extern __shared__ __align__(128) unsigned char pipe_raw[];
  PipeStage* stages = reinterpret_cast<PipeStage*>(pipe_raw);
  __shared__ __align__(8) unsigned long long full_bar[PIPE_NW];

  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  const int2 range = p.ranges[blockIdx.x];
  const int n = range.y - range.x;
  if (wid >= n) return;  // (no CTA-wide barrier below: every warp works on its own stage)

  PipeStage& st = stages[wid];
  unsigned long long* full = &full_bar[wid];
  const int4* rp = reinterpret_cast<const int4*>(p.records + (size_t)range.x * PIPE_REC);
  if (lane == 0) {
    // the copies complete the byte count; the single arrival is lane 0's expect_tx
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pipe_smem(full)), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // the first two records of this warp come straight from global memory
    int4* dst = reinterpret_cast<int4*>(st.rec[0]);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = __ldg(rp + (size_t)wid * 8 + j);
    if (wid + PIPE_NW < n) {
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[8 + j] = __ldg(rp + (size_t)(wid + PIPE_NW) * 8 + j);
    }
    pipe_issue(p, st, full, rp, wid, 0, n);
  }
  __syncwarp();

  // Lane l takes the rows l, l + 32, l + 64, l + 96 of the record.  The row count is
  // fixed along a chain, so the sums stay in registers.
  float acc[PIPE_ROWS_PER_THREAD] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (int m = 0, i = wid; i < n; ++m, i += PIPE_NW) {
    if (!mbar_wait(full, (uint32_t)(m & 1))) {
      if (lane == 0 && p.status) atomicExch(p.status, NB2_ERR_TIMEOUT);
      return;
    }
    const int* rec = st.rec[m % 3];
    const int4 h0 = *reinterpret_cast<const int4*>(rec);      // flags, rows, y_in, y
    const int4 h1 = *reinterpret_cast<const int4*>(rec + 4);  // item, segments, -, yin bytes
    const int flags = h0.x, R = h0.y, nseg = h1.y;
    if (flags & 1) {
#pragma unroll
      for (int j = 0; j < PIPE_ROWS_PER_THREAD; ++j) acc[j] = 0.0f;
    }
    if (R > 0) {
      // lanes beyond the last row re-read it; their sums are discarded
      int roff[PIPE_ROWS_PER_THREAD];
#pragma unroll
      for (int j = 0; j < PIPE_ROWS_PER_THREAD; ++j) roff[j] = min(lane + 32 * j, R - 1);
      const int NR = (R + 31) >> 5;
      for (int q = 0; q < nseg; ++q) {
        const int2 xf = *reinterpret_cast<const int2*>(rec + 8 + 6 * q + 2);  // x index, x bytes / -stride
        const int2 wf = *reinterpret_cast<const int2*>(rec + 8 + 6 * q + 4);  // columns, offsets
        const float* a = st.buf + (wf.y & 0xffff);
        const float* xs = xf.y > 0 ? st.buf + (wf.y >> 16) : nullptr;
        const float* xg = p.X + xf.x;
        if (NR == 1) pipe_segment_mode<1>(a, xs, xg, -xf.y, wf.x, lane, roff, acc);
        else if (NR == 2) pipe_segment_mode<2>(a, xs, xg, -xf.y, wf.x, lane, roff, acc);
        else pipe_segment_mode<4>(a, xs, xg, -xf.y, wf.x, lane, roff, acc);
      }
      if (flags & 2) {
        const int y_in = h0.z, y = h0.w, bb = h1.x;
        const bool staged = h1.w > 0;
#pragma unroll
        for (int j = 0; j < PIPE_ROWS_PER_THREAD; ++j) {
          const int r = lane + 32 * j;
          if (r < R) {
            const float yin = staged ? st.yin[(y_in & 3) + r] : p.Yin[y_in + r];
            p.Y[y + r] = pipe_epilogue(p, bb, yin, acc[j]);
          }
        }
      }
    }
    __syncwarp();  // every lane is done with the stage
    if (lane == 0 && i + PIPE_NW < n) pipe_issue(p, st, full, rp, i + PIPE_NW, m + 1, n);
  }
}

static const size_t kPipeSmem = sizeof(PipeStage) * PIPE_NW;

extern "C" int nb2_gemv_pipelined(void* stream, const int* records, int n_records, const int* ranges,
                                  int n_ctas, const float* A, const float* X, const float* Yin, float* Y,
                                  double alpha, double beta, double gamma, const float* alphas,
                                  const float* betas, const float* gammas, int* status) {
  if (n_records == 0 || n_ctas == 0) return NB2_OK;
  NB2_REQUIRE(records && ranges && A && X && Yin && Y, "null pointer");
  NB2_REQUIRE((((uintptr_t)records | (uintptr_t)A | (uintptr_t)X | (uintptr_t)Yin) & 15) == 0,
              "records, A, X and Y_in must be 16-byte aligned");
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
  nb2_launch(nb2_gemv_pipe_kernel, dim3(n_ctas), dim3(PIPE_THREADS), kPipeSmem, nb2_stream(stream), p);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
