// Ragged gather-GEMV for sm_100a:
//     Y[k] = gamma + beta * Y_in[k] + alpha * sum_j A[a_kj] . X[x_kj]
//
// One single-pass kernel family replaces the reference's four OpenCL variants
// (nengo_ocl/clra_gemv.py: ref_impl :264-444, reduce_impl :447-670,
// many_dots_impl :673-858, block_impl + reduce :861-1175).  The kernels read
// the same per-item int32 index table that the reference uploads
// (cl_geometry_and_textconf, clra_gemv.py:211-261): for item row `g` and
// D = max dots, g[0*D+i] = X start, g[1*D+i] = A start, g[2*D+i] = A stride0,
// g[3*D+i] = A shape1, g[4*D+0..4] = Y_in start, Y start, n dots, y_len, item id.
//
// Work decomposition (host-built work list, int4 per unit = item row, first
// output row, row count, unused):
//  * nb2_gemv_cta_kernel: one CTA per unit.  The A rows of every term of the
//    unit are staged into shared memory as flat, fully coalesced streams
//    (128-bit loads, or 1-D bulk async copies completed on an mbarrier), the
//    gathered X segments are staged once, and a lane group per row reduces
//    with warp shuffles.  Terms accumulate in list order into one value per
//    row; the epilogue applies alpha/beta/gamma in a single pass, so there is
//    no scratch buffer and no second reduce kernel.
//  * nb2_gemv_warp_kernel: one warp per unit for tiny items (a few hundred
//    floats), reading A straight from global memory.
//
// The kernel is HBM-bound (0.5 flop/byte); no tensor cores are involved.
#include "nb2_common.cuh"
#include "../../include/nengo_b200.h"

#define GEMV_THREADS 256
#define GEMV_WARPS (GEMV_THREADS / 32)
#define GEMV_ABUF NB2_GEMV_ABUF      // floats of staged A per CTA
#define GEMV_XBUF NB2_GEMV_XBUF      // floats of staged X per CTA
#define GEMV_RMAX NB2_GEMV_RMAX      // max rows per unit
#define GEMV_MAXSEG 32               // staged (term, column chunk) segments per batch
#define GEMV_SPIN_LIMIT (1 << 24)

struct GemvParams {
  const int* gstructure;   // [n_items][gstride]
  const int* xstrides;     // [n_items][D] or NULL (all 1)
  const int4* worklist;    // [n_units]
  int n_units;
  int gstride;
  int D;
  const float* A;
  const float* X;
  const float* Yin;
  float* Y;
  double alpha, beta, gamma;
  const float* alphas;     // per item id, or NULL
  const float* betas;
  const float* gammas;
  int* status;             // device status word (bounded-wait timeouts)
};

struct Segment {
  int w;        // columns in this segment
  int aoff;     // smem offset of (row 0, col 0)
  int xoff;     // smem offset of x[col 0]
  int gidx;     // global element index of (row r0, col c0)
  int s0;       // global row stride
  int xstart;   // global index of x[c0]
  int xstride;
  int contiguous;
};

__device__ __forceinline__ int pow2ceil_le32(int w) {
  if (w >= 32) return 32;
  int g = 1;
  while (g < w) g <<= 1;
  return g;
}

// Epilogue shared by both kernels.  The scalar forms are evaluated in double
// and rounded once, like the reference's rendered double literals
// (clra_gemv.py:782-824); the per-item vector forms are float arithmetic.
__device__ __forceinline__ float gemv_epilogue(const GemvParams& p, int bb, float yin, float sum) {
  float pre;
  if (p.betas) pre = p.betas[bb] * yin;
  else pre = (p.beta != 0.0) ? (float)(p.beta * (double)yin) : 0.0f;
  if (p.gammas) pre += p.gammas[bb];
  else if (p.gamma != 0.0) pre = (float)((double)pre + p.gamma);
  if (p.alphas) return pre + p.alphas[bb] * sum;
  return (float)((double)pre + p.alpha * (double)sum);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

template <int BULK>
__global__ void __launch_bounds__(GEMV_THREADS)
nb2_gemv_cta_kernel(const GemvParams p) {
  nb2_pdl_enter();
  extern __shared__ __align__(128) float smem[];
  float* sA = smem;                       // GEMV_ABUF
  float* sX = sA + GEMV_ABUF;             // GEMV_XBUF
  float* sY = sX + GEMV_XBUF;             // GEMV_RMAX
  __shared__ Segment segs[GEMV_MAXSEG];
  __shared__ int s_nseg, s_next_ii, s_next_c0;
  __shared__ __align__(8) unsigned long long s_bar;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int wid = tid >> 5;

  const int4 unit = p.worklist[blockIdx.x];
  const int* g = p.gstructure + (size_t)unit.x * p.gstride;
  const int r0 = unit.y;
  const int R = unit.z;
  const int D = p.D;
  const int n_dots = g[4 * D + 2];
  const int* xst = p.xstrides ? p.xstrides + (size_t)unit.x * D : nullptr;

  for (int r = tid; r < R; r += GEMV_THREADS) sY[r] = 0.0f;
  uint32_t phase = 0;
  if (BULK && tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_bar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid == 0) { s_next_ii = 0; s_next_c0 = 0; }
  __syncthreads();

  const int RW = (R + GEMV_WARPS - 1) / GEMV_WARPS;
  const int wbeg = wid * RW;
  const int wend = min(R, wbeg + RW);

  while (true) {
    // ---- plan one batch of segments (thread 0) ----
    if (tid == 0) {
      int ii = s_next_ii, c0 = s_next_c0, used_a = 0, used_x = 0, nseg = 0;
      while (ii < n_dots && nseg < GEMV_MAXSEG) {
        const int N = g[3 * D + ii];
        const int s0 = g[2 * D + ii];
        const int gidx = g[1 * D + ii] + r0 * s0 + c0;
        const int base = ((used_a + 3) & ~3) + (gidx & 3);
        const int avail = GEMV_ABUF - base;
        int w = min(N - c0, min(avail / R, GEMV_XBUF - used_x));
        if (w <= 0) break;
        Segment s;
        s.w = w; s.aoff = base; s.xoff = used_x; s.gidx = gidx; s.s0 = s0;
        s.xstride = xst ? xst[ii] : 1;
        s.xstart = g[ii] + c0 * s.xstride;
        s.contiguous = (s0 == w) || (R == 1);
        segs[nseg++] = s;
        used_a = base + R * w;
        used_x += w;
        c0 += w;
        if (c0 >= N) { ii++; c0 = 0; }
      }
      s_nseg = nseg; s_next_ii = ii; s_next_c0 = c0;
    }
    __syncthreads();
    const int nseg = s_nseg;
    if (nseg == 0) break;

    // ---- stage X and A ----
    uint32_t bulk_bytes = 0;
    for (int s = 0; s < nseg; ++s) {
      const Segment sg = segs[s];
      for (int c = tid; c < sg.w; c += GEMV_THREADS)
        sX[sg.xoff + c] = __ldg(p.X + sg.xstart + (size_t)c * sg.xstride);
      const int len = R * sg.w;
      if (sg.contiguous) {
        const float* src = p.A + sg.gidx;
        float* dst = sA + sg.aoff;
        const int head = min(len, (4 - (sg.gidx & 3)) & 3);
        const int body = (len - head) & ~3;
        if (tid < head) dst[tid] = nb2_ldg_stream(src + tid);
        const int tail0 = head + body;
        if (tid >= 32 && tid - 32 < len - tail0) dst[tail0 + tid - 32] = nb2_ldg_stream(src + tail0 + tid - 32);
        if (BULK) {
          if (tid == 0 && body > 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile(
                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
                    "r"(smem_u32(dst + head)), "l"(src + head), "r"((uint32_t)body * 4u),
                "r"(smem_u32(&s_bar))
                : "memory");
          }
          bulk_bytes += (uint32_t)body * 4u;
        } else {
          const float4* src4 = reinterpret_cast<const float4*>(src + head);
          float4* dst4 = reinterpret_cast<float4*>(dst + head);
          const int n4 = body >> 2;
          int i = tid;
          for (; i + 3 * GEMV_THREADS < n4; i += 4 * GEMV_THREADS) {
            float4 v0 = nb2_ldg_stream4(src4 + i);
            float4 v1 = nb2_ldg_stream4(src4 + i + GEMV_THREADS);
            float4 v2 = nb2_ldg_stream4(src4 + i + 2 * GEMV_THREADS);
            float4 v3 = nb2_ldg_stream4(src4 + i + 3 * GEMV_THREADS);
            dst4[i] = v0; dst4[i + GEMV_THREADS] = v1;
            dst4[i + 2 * GEMV_THREADS] = v2; dst4[i + 3 * GEMV_THREADS] = v3;
          }
          for (; i < n4; i += GEMV_THREADS) dst4[i] = nb2_ldg_stream4(src4 + i);
        }
      } else {
        // strided rows or a column chunk: generic 2-D copy into packed rows
        for (int e = tid; e < len; e += GEMV_THREADS) {
          const int r = e / sg.w;
          const int c = e - r * sg.w;
          sA[sg.aoff + e] = nb2_ldg_stream(p.A + sg.gidx + (size_t)r * sg.s0 + c);
        }
      }
    }
    if (BULK) {
      if (tid == 0) {
        // thread 0 issued every bulk copy above, so the expected byte count is complete here
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&s_bar)),
                     "r"(bulk_bytes)
                     : "memory");
      }
      __syncthreads();
      uint32_t done = 0;
      int spins = 0;
      while (!done && spins < GEMV_SPIN_LIMIT) {
        asm volatile(
            "{\n .reg .pred q;\n mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n selp.u32 %0, 1, 0, q;\n}"
            : "=r"(done)
            : "r"(smem_u32(&s_bar)), "r"(phase)
            : "memory");
        ++spins;
      }
      if (!done && tid == 0 && p.status) atomicExch(p.status, NB2_ERR_TIMEOUT);
      phase ^= 1;
    }
    __syncthreads();

    // ---- compute: lane group per row, warp owns rows [wbeg, wend) ----
    for (int s = 0; s < nseg; ++s) {
      const Segment sg = segs[s];
      const int w = sg.w;
      const int G = pow2ceil_le32(w);
      const int rpp = 32 / G;
      const int lg = lane & (G - 1);
      const int lr = lane / G;
      const float* a = sA + sg.aoff;
      const float* x = sX + sg.xoff;
      for (int rb = wbeg; rb < wend; rb += rpp) {
        const int r = rb + lr;
        float sum = 0.0f;
        if (r < wend) {
          const float* ar = a + r * w;
          for (int c = lg; c < w; c += G) sum = fmaf(ar[c], x[c], sum);
        }
        for (int off = G >> 1; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (lg == 0 && r < wend) sY[r] += sum;
      }
      __syncwarp();
    }
    __syncthreads();
  }

  // ---- epilogue ----
  const int y_in_start = g[4 * D + 0];
  const int y_start = g[4 * D + 1];
  const int bb = g[4 * D + 4];
  for (int r = tid; r < R; r += GEMV_THREADS) {
    const float yin = p.Yin[y_in_start + r0 + r];
    p.Y[y_start + r0 + r] = gemv_epilogue(p, bb, yin, sY[r]);
  }
}

// One warp per unit, at most 32 rows, A read directly from global memory.
__global__ void __launch_bounds__(GEMV_THREADS)
nb2_gemv_warp_kernel(const GemvParams p) {
  nb2_pdl_enter();
  __shared__ float acc[GEMV_WARPS][32];
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  const int u = blockIdx.x * GEMV_WARPS + wid;
  if (u >= p.n_units) return;
  const int4 unit = p.worklist[u];
  const int* g = p.gstructure + (size_t)unit.x * p.gstride;
  const int r0 = unit.y;
  const int R = unit.z;  // <= 32
  const int D = p.D;
  const int n_dots = g[4 * D + 2];
  const int* xst = p.xstrides ? p.xstrides + (size_t)unit.x * D : nullptr;
  acc[wid][lane] = 0.0f;
  __syncwarp();
  for (int ii = 0; ii < n_dots; ++ii) {
    const int N = g[3 * D + ii];
    const int s0 = g[2 * D + ii];
    const float* a = p.A + g[1 * D + ii] + (size_t)r0 * s0;
    const int xs = xst ? xst[ii] : 1;
    const float* x = p.X + g[ii];
    const int G = pow2ceil_le32(N);
    const int rpp = 32 / G;
    const int lg = lane & (G - 1);
    const int lr = lane / G;
    for (int rb = 0; rb < R; rb += rpp) {
      const int r = rb + lr;
      float sum = 0.0f;
      if (r < R)
        for (int c = lg; c < N; c += G) sum = fmaf(__ldg(a + (size_t)r * s0 + c), __ldg(x + (size_t)c * xs), sum);
      for (int off = G >> 1; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      if (lg == 0 && r < R) acc[wid][r] += sum;
    }
    __syncwarp();
  }
  if (lane < R) {
    const int y_in_start = g[4 * D + 0];
    const int y_start = g[4 * D + 1];
    const int bb = g[4 * D + 4];
    const float yin = p.Yin[y_in_start + r0 + lane];
    p.Y[y_start + r0 + lane] = gemv_epilogue(p, bb, yin, acc[wid][lane]);
  }
}


// ---- row-group kernel -------------------------------------------------------
// One CTA per unit of up to 8 * P rows (P = 256 / G).  G = 2^logG lanes share a
// row and stride over its columns, so a warp reads 32 / G contiguous row
// chunks; every thread owns 8 rows (8 independent accumulators, 8 loads in
// flight per column step) and loads each gathered x value once for all of
// them.  A is read straight from global memory: with ~2048 resident threads
// per SM each holding >= 8 outstanding 4-byte loads, enough bytes are in flight
// to cover HBM latency without a shared-memory ring.
#define ROWS_PER_THREAD 8
__global__ void __launch_bounds__(GEMV_THREADS)
nb2_gemv_rows_kernel(const GemvParams p) {
  nb2_pdl_enter();
  const int tid = threadIdx.x;
  const int4 unit = p.worklist[blockIdx.x];
  const int* __restrict__ g = p.gstructure + (size_t)unit.x * p.gstride;
  const int r0 = unit.y;
  const int R = unit.z;
  const int logG = unit.w;
  const int G = 1 << logG;
  const int P = GEMV_THREADS >> logG;
  const int lg = tid & (G - 1);
  const int row0 = tid >> logG;
  const int D = p.D;
  const int n_dots = __ldg(g + 4 * D + 2);
  const int* xst = p.xstrides ? p.xstrides + (size_t)unit.x * D : nullptr;

  float acc[ROWS_PER_THREAD];
  int roff[ROWS_PER_THREAD];
#pragma unroll
  for (int j = 0; j < ROWS_PER_THREAD; ++j) {
    acc[j] = 0.0f;
    roff[j] = r0 + min(row0 + j * P, R - 1);  // rows past the end re-read the last row
  }
  if (row0 < R) {
    for (int ii = 0; ii < n_dots; ++ii) {
      const int N = __ldg(g + 3 * D + ii);
      const int s0 = __ldg(g + 2 * D + ii);
      const float* __restrict__ a = p.A + __ldg(g + 1 * D + ii) + lg;
      const int xs = xst ? __ldg(xst + ii) : 1;
      const float* __restrict__ x = p.X + __ldg(g + ii) + (size_t)lg * xs;
      const float* ap[ROWS_PER_THREAD];
#pragma unroll
      for (int j = 0; j < ROWS_PER_THREAD; ++j) ap[j] = a + (size_t)roff[j] * s0;
#pragma unroll 2
      for (int c = lg; c < N; c += G) {
        const float xv = __ldg(x);
        x += (size_t)G * xs;
#pragma unroll
        for (int j = 0; j < ROWS_PER_THREAD; ++j) {
          acc[j] = fmaf(__ldg(ap[j]), xv, acc[j]);
          ap[j] += G;
        }
      }
    }
  }
  const int y_in_start = __ldg(g + 4 * D + 0);
  const int y_start = __ldg(g + 4 * D + 1);
  const int bb = __ldg(g + 4 * D + 4);
#pragma unroll
  for (int j = 0; j < ROWS_PER_THREAD; ++j) {
    float t = acc[j];
    for (int off = G >> 1; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
    const int r = row0 + j * P;
    if (lg == 0 && r < R) {
      const float yin = p.Yin[y_in_start + r0 + r];
      p.Y[y_start + r0 + r] = gemv_epilogue(p, bb, yin, t);
    }
  }
}

static const size_t kGemvSmem = (size_t)(GEMV_ABUF + GEMV_XBUF + GEMV_RMAX) * sizeof(float);

// Opt in to >48 KB dynamic shared memory once per device and kernel variant.
static cudaError_t gemv_optin_smem(int bulk) {
  static bool done[2][64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && done[bulk][dev]) return cudaSuccess;
  e = bulk ? cudaFuncSetAttribute(nb2_gemv_cta_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)kGemvSmem)
           : cudaFuncSetAttribute(nb2_gemv_cta_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)kGemvSmem);
  if (e == cudaSuccess && dev < 64) done[bulk][dev] = true;
  return e;
}

extern "C" int nb2_gemv_ragged(void* stream, int kind, const int* gstructure, int gstride, int D,
                               const int* xstrides, const int* worklist, int n_units, const float* A,
                               const float* X, const float* Yin, float* Y, double alpha, double beta,
                               double gamma, const float* alphas, const float* betas,
                               const float* gammas, int* status) {
  if (n_units == 0) return NB2_OK;
  NB2_REQUIRE(gstructure && worklist && A && X && Yin && Y, "null pointer");
  NB2_REQUIRE(D >= 0 && gstride >= 4 * D + 5, "gstride < 4*D+5");
  GemvParams p;
  p.gstructure = gstructure; p.xstrides = xstrides;
  p.worklist = reinterpret_cast<const int4*>(worklist);
  p.n_units = n_units; p.gstride = gstride; p.D = D;
  p.A = A; p.X = X; p.Yin = Yin; p.Y = Y;
  p.alpha = alpha; p.beta = beta; p.gamma = gamma;
  p.alphas = alphas; p.betas = betas; p.gammas = gammas;
  p.status = status;
  cudaStream_t s = nb2_stream(stream);
  if (kind == NB2_GEMV_WARP) {
    const int blocks = (n_units + GEMV_WARPS - 1) / GEMV_WARPS;
    nb2_launch(nb2_gemv_warp_kernel, dim3(blocks), dim3(GEMV_THREADS), 0, s, p);
  } else if (kind == NB2_GEMV_CTA_BULK) {
    NB2_CUDA(gemv_optin_smem(1));
    nb2_launch(nb2_gemv_cta_kernel<1>, dim3(n_units), dim3(GEMV_THREADS), kGemvSmem, s, p);
  } else if (kind == NB2_GEMV_CTA) {
    NB2_CUDA(gemv_optin_smem(0));
    nb2_launch(nb2_gemv_cta_kernel<0>, dim3(n_units), dim3(GEMV_THREADS), kGemvSmem, s, p);
  } else if (kind == NB2_GEMV_ROWS) {
    nb2_launch(nb2_gemv_rows_kernel, dim3(n_units), dim3(GEMV_THREADS), 0, s, p);
  } else {
    NB2_REQUIRE(false, "unknown gemv kind");
  }
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
