// Streamed fused ensemble step for large populations: the same operator
// sequence as nb2_fused.cu (encoder GEMV + LIF + decoder GEMV + lowpass synapse
// + PES decoder update in one kernel per time step; reference counterparts
// listed there), organised as a bulk-copy pipeline so that every SM always has
// about 200 KB of loads in flight.
//
//  * The host cuts every ensemble into work records: E records (a block of
//    neurons: their encoder rows, bias, voltage, refractory time and PES
//    activity trace) and D records (a few whole rows of one decoder matrix), each
//    at most one stage (8 KB) of data.  A CTA
//    (one per SM, persistent) owns a list of whole ensembles; its records are
//    ordered E(0), E(1), D(0), E(2), D(1), ... so that the spikes a D record
//    needs were produced one pass over the warps earlier.
//  * Every warp owns one shared-memory stage and the records i = warp,
//    warp + WARPS, ... .  Lane 0 fills the stage with 1-D bulk async copies
//    (cp.async.bulk, completion counted in bytes on the stage's mbarrier); all
//    sources are 16-byte aligned by construction (the host only streams
//    ensembles whose arrays start on multiples of 4 floats).  The warp's next
//    record rides along with the copies.
//  * All dot products are summed in the order of the reference's block GEMV
//    (nb2_blockdot.cuh), so J and the decoded values are bit-identical to it.
//  * E record: one lane per neuron (4 neurons per lane); J = bias + enc . x from
//    the staged rows (128-bit shared loads, columns in order), LIF update in the operation order of the reference kernel
//    (this file is compiled with -fmad=false; expm1 / log1p correctly rounded),
//    V / W / spikes / new activity trace written straight to global memory,
//    spikes and the OLD trace kept in a per-ensemble slot of shared memory for
//    the D records.
//  * D record: PES update w += (alpha * err) * trace: elementwise, lanes over
//    groups of 4 neurons, 128-bit shared loads and 128-bit global stores.
//    Decode: a pair of lanes owns the four partial sums of one (row, 128-column
//    tile) and walks them in column order (64-bit shared loads; the pairs start
//    one iteration apart so that the tiles, 128 floats apart, do not meet in the
//    same banks); two shuffles form the tile value, the tiles of a row are added
//    in order, then the synapse.
//  * Slots are handed from E to D records and back through two counters per slot
//    in shared memory; a record only ever waits for records that precede it in
//    the CTA's list, so the lowest unfinished record can always run.
//
//  * Multi-GPU: when the model is sharded, the decoded (filtered) values of a
//    CTA's ensembles are one contiguous run of this rank's segment of the
//    exchange signal; the CTA's last warp stores that run into every peer's
//    staging buffer (plain peer stores over NVLink, whole lines; no multicast)
//    as soon as the CTA is done, and the last CTA of the grid publishes the
//    step number in the peers' flag words (st.release.sys).  The compute step
//    and its push are one kernel; the peers' nb2_exchange_wait is the other
//    half.
//
// Every wait (mbarrier, counters) is bounded by the global timer; on timeout
// the warp records NB2_ERR_TIMEOUT in the status word, raises the CTA's abort
// flag and leaves.
#include "nb2_common.cuh"
#include "nb2_pipe.cuh"
#include "nb2_blockdot.cuh"
#include "nb2_fused_common.cuh"
#include "nb2_exchange_common.cuh"
#include "../../include/nengo_b200.h"

#define ST_NW NB2_STREAM_WARPS
#define ST_THREADS (32 * ST_NW)
#define ST_A NB2_STREAM_STAGE_FLOATS
#define ST_X NB2_STREAM_MAX_INPUT
#define ST_N NB2_STREAM_MAX_NEURONS
#define ST_SLOTS NB2_STREAM_SLOTS
#define ST_REC 32
#define ST_MAXCOPY 8
#ifndef ST_L2_PREFETCH
#define ST_L2_PREFETCH 1
#endif
#ifndef ST_ROWS
#define ST_ROWS 4  // neurons per lane and pass of an E record (3 measured no faster for the 96-neuron records of the PES model)
#endif
#define ST_DITEMS 16  // (row, 128-column tile) pairs of a D record: two lanes each

struct StreamParams {
  const int* records;  // [n_records][32]
  const int2* ranges;  // per CTA: [begin, end) record indices
  const int* ens_table;
  const int* term_table;
  const int* conn_table;
  float* data;
  float dt, dt_inv;
  int* status;
  nb2_exchange_desc x;  // x.peer_staging == NULL: no exchange
};

struct __align__(128) StreamStage {
  float buf[ST_A];
  float x[ST_X];
  int rec[2][ST_REC];  // record of turn m in slot m & 1
  float ae[ST_DITEMS];  // alpha * error of the rows of a D record
};

struct __align__(16) StreamSlot {
  float spk[ST_N];  // spikes of this step
  float pfo[ST_N];  // PES activity trace before this step's update
};

// record words
enum { R_TYPE = 0, R_ENS, R_SLOT, R_A, R_B, R_NCOPY, R_TARGET, R_C, R_COPY0 = 8, R_TX = 31 };
// D records: R_A connection, R_B first row, R_C rows; everything else the record needs is written
// into it by the host (one shared-memory read instead of a table lookup in global memory):
enum { RD_NE = 11, RD_PES, RD_ALPHA, RD_ERR, RD_WEIGHTED, RD_FILT, RD_B0, RD_A0 };  // neurons, PES flag, alpha
// (float bits), element index of the error / decoded / filtered value of the first row (filtered: -1 = none),
// synapse coefficients (float bits; a0 == 0: pure gain)

// All lanes: fill the stage for turn m (record index i); the record is in st.rec[m & 1].
// Every copy is issued by a lane of its own; the warp's next record rides along.
__device__ __forceinline__ void stream_issue(const StreamParams& p, StreamStage& st, unsigned long long* full,
                                             const int4* rp, int i, int m, int n, int lane) {
  const int* r = st.rec[m & 1];
  const bool more = i + ST_NW < n;
  // the stage was read through the generic proxy; order those reads before the async-proxy writes
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  const float* src = nullptr;
  float* dst = nullptr;
  uint32_t bytes = 0;
  if (lane < r[R_NCOPY]) {
    src = p.data + r[R_COPY0 + 3 * lane];
    bytes = (uint32_t)r[R_COPY0 + 3 * lane + 1];
    dst = st.buf + r[R_COPY0 + 3 * lane + 2];
  }
  if (lane == 0) {
    const uint32_t tx = (uint32_t)r[R_TX] + (more ? ST_REC * 4u : 0u);  // (the host added up the copies)
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pipe_smem(full)), "r"(tx) : "memory");
  }
  __syncwarp();
  if (bytes) bulk_copy(dst, src, bytes, full);
  if (more && lane == 31) bulk_copy(st.rec[(m + 1) & 1], rp + (size_t)(i + ST_NW) * 8, ST_REC * 4u, full);
}

// All lanes: stage the input vectors of an E record's ensemble (read from global memory, L2-hot).
__device__ __forceinline__ void stream_stage_x(const StreamParams& p, StreamStage& st, const int* r, int lane) {
  if (r[R_TYPE] != 1) return;
  const int* e = p.ens_table + (size_t)r[R_ENS] * E_STRIDE;
  const int n_terms = __ldg(e + E_NTERMS);
  const int* terms = p.term_table + (size_t)__ldg(e + E_TERM0) * T_STRIDE;
  int xoff = 0;
  for (int k = 0; k < n_terms; ++k) {
    const int d = __ldg(terms + k * T_STRIDE + T_D);
    const float* x = p.data + __ldg(terms + k * T_STRIDE + T_X);
    const int xs = __ldg(terms + k * T_STRIDE + T_XS);
    for (int c = lane; c < d; c += 32) st.x[xoff + c] = x[(size_t)c * xs];
    xoff += d;
  }
}

// w + (alpha * error) * trace for 4 neighbouring columns (two roundings per element, as the
// reference's delta kernel followed by its increment)
__device__ __forceinline__ float4 pes_update(float4 w, float ae, float4 p) {
  float4 o;
  o.x = w.x + ae * p.x;
  o.y = w.y + ae * p.y;
  o.z = w.z + ae * p.z;
  o.w = w.w + ae * p.w;
  return o;
}

// Lane 0 polls a counter of the CTA; the whole warp gets the answer.
__device__ __forceinline__ bool stream_wait_count(const volatile int* ctr, int target, volatile int* abort_flag,
                                                  int lane) {
  int ok = 1;
  if (lane == 0 && *ctr < target) {
    const unsigned long long t0 = pipe_timer();
    for (int spins = 0; *ctr < target; ++spins) {
      __nanosleep(100);
      if ((spins & 15) == 15 && (*abort_flag || pipe_timer() - t0 > PIPE_WAIT_NS)) {
        ok = 0;
        break;
      }
    }
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  __threadfence_block();  // the other warps' shared-memory writes before their count
  return ok != 0;
}

__global__ void __launch_bounds__(ST_THREADS, 1) nb2_ensemble_stream_kernel(const StreamParams p) {
  nb2_pdl_enter();
  extern __shared__ __align__(128) unsigned char stream_raw[];
  StreamStage* stages = reinterpret_cast<StreamStage*>(stream_raw);
  StreamSlot* slots = reinterpret_cast<StreamSlot*>(stream_raw + sizeof(StreamStage) * ST_NW);
  __shared__ __align__(8) unsigned long long full_bar[ST_NW];
  __shared__ int e_done[ST_SLOTS];  // E records finished per slot (cumulative)
  __shared__ int d_done[ST_SLOTS];  // D records finished per slot (cumulative)
  __shared__ int s_abort;
  __shared__ int warps_left;  // warps of this CTA that still work (exchange push only)

  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  const int2 range = p.ranges[blockIdx.x];
  const int n = range.y - range.x;
  if (threadIdx.x < ST_SLOTS) e_done[threadIdx.x] = d_done[threadIdx.x] = 0;
  if (threadIdx.x == 0) {
    s_abort = 0;
    warps_left = min(ST_NW, n);
  }
  __syncthreads();
  if (wid >= n) return;
  // exchange push: this step's values go into the staging half of parity (epoch + 1) & 1
  const bool xpush = p.x.peer_staging != nullptr;
  const int epoch = xpush ? p.x.ctl[X_EPOCH] : 0;
  const size_t xoff = (size_t)((epoch + 1) & 1) * p.x.world * p.x.seg;

  StreamStage& st = stages[wid];
  unsigned long long* full = &full_bar[wid];
  const int4* rp = reinterpret_cast<const int4*>(p.records + (size_t)range.x * ST_REC);
  if (lane == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pipe_smem(full)), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    int4* dst = reinterpret_cast<int4*>(st.rec[0]);  // the first record comes straight from global memory
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = __ldg(rp + (size_t)wid * 8 + j);
  }
  __syncwarp();
  stream_issue(p, st, full, rp, wid, 0, n, lane);
  stream_stage_x(p, st, st.rec[0], lane);
  __syncwarp();

  float* const data = p.data;
  for (int m = 0, i = wid; i < n; ++m, i += ST_NW) {
    bool ok = mbar_wait(full, (uint32_t)(m & 1));
    const int* rec = st.rec[m & 1];
#if ST_L2_PREFETCH
    // The warp's next record arrived with this one: ask its arrays into L2 now, so that the bulk
    // copies issued after this record's arithmetic find them there (a stage is then empty for the
    // L2 latency instead of the DRAM latency).
    if (ok && i + ST_NW < n) {
      const int* rn = st.rec[(m + 1) & 1];
      if (lane < rn[R_NCOPY]) l2_prefetch(p.data + rn[R_COPY0 + 3 * lane], (uint32_t)rn[R_COPY0 + 3 * lane + 1]);
    }
#endif
    const int4 h0 = *reinterpret_cast<const int4*>(rec);      // type, ensemble, slot, a
    const int4 h1 = *reinterpret_cast<const int4*>(rec + 4);  // b, copies, target, c
    const int* e = p.ens_table + (size_t)h0.y * E_STRIDE;
    StreamSlot& slot = slots[h0.z];
    if (ok && h0.x == 1) {
      // ---------------- E record: neurons [i0, i0 + ne) ----------------
      const int i0 = h0.w, ne = h1.x, pf_conn = h1.w;
      const int n_terms = __ldg(e + E_NTERMS);
      const int* terms = p.term_table + (size_t)__ldg(e + E_TERM0) * T_STRIDE;
      const float tau = bits(__ldg(e + E_TAU)), ref = bits(__ldg(e + E_REF)), amp = bits(__ldg(e + E_AMP));
      const int eV = __ldg(e + E_V), eW = __ldg(e + E_W), eS = __ldg(e + E_S);
      const float* s_bias = st.buf + rec[R_COPY0 + 3 * n_terms + 2];
      const float* s_V = st.buf + rec[R_COPY0 + 3 * (n_terms + 1) + 2];
      const float* s_W = st.buf + rec[R_COPY0 + 3 * (n_terms + 2) + 2];
      const float* s_pf = st.buf + rec[R_COPY0 + 3 * (n_terms + 3) + 2];  // (only read when pf_conn >= 0)
      float pb0 = 0.0f, pa0 = 0.0f;
      int gpf = 0;
      if (pf_conn >= 0) {
        const int* c = p.conn_table + (size_t)pf_conn * C_STRIDE;
        pb0 = bits(__ldg(c + C_PFB0));
        pa0 = bits(__ldg(c + C_PFA0));
        gpf = __ldg(c + C_PF);
      }
      // the slot's previous ensemble must have been decoded completely
      ok = stream_wait_count(&d_done[h0.z], h1.z, &s_abort, lane);
      const float em1_dt = bits(__ldg(e + E_EM1));
      // blocks of 32 * ST_ROWS neurons: ST_ROWS per lane
      for (int base = 0; ok && base < ne; base += 32 * ST_ROWS) {
        const int nb = min(32 * ST_ROWS, ne - base);
        float tot[4];  // (block_rows_staged4 takes arrays of four; ST_ROWS of them are used)
        int roff[4];
#pragma unroll
        for (int j = 0; j < ST_ROWS; ++j) {
          roff[j] = base + min(lane + 32 * j, nb - 1);
          tot[j] = s_bias[roff[j]];  // J = ((bias + term 0) + term 1) + ...
        }
        int xoff = 0;
        for (int k = 0; k < n_terms; ++k) {
          const int d = __ldg(terms + k * T_STRIDE + T_D);
          const float* a = st.buf + rec[R_COPY0 + 3 * k + 2];
          // (always ST_ROWS rows per lane: a short last block repeats its last neuron, which keeps
          // the kernel's code small)
          block_rows_staged4<ST_ROWS>(a, st.x + xoff, d, lane, roff, tot, 1.0);
          xoff += d;
        }
        // (lanes beyond the last neuron of the block recompute it; nothing of theirs is stored)
        float Jv[ST_ROWS], Vv[ST_ROWS], Wv[ST_ROWS], Sv[ST_ROWS], Pv[ST_ROWS];
#pragma unroll
        for (int j = 0; j < ST_ROWS; ++j) {
          Jv[j] = tot[j];
          Vv[j] = s_V[roff[j]];
          Wv[j] = s_W[roff[j]];
          Pv[j] = pf_conn >= 0 ? s_pf[roff[j]] : 0.0f;
        }
        fused_lifN<ST_ROWS>(Jv, Vv, Wv, Sv, tau, ref, amp, p.dt, p.dt_inv, em1_dt);
        // row j of this lane is neuron i0 + base + lane + 32 j: every array is walked with immediates
        const int first = i0 + base + lane;
        float* gV = data + eV + first;
        float* gW = data + eW + first;
        float* gS = eS >= 0 ? data + eS + first : nullptr;
        float* sspk = slot.spk + first;
        if (pf_conn >= 0) {
          float* spfo = slot.pfo + first;
          float* gPF = data + gpf + first;
#pragma unroll
          for (int j = 0; j < ST_ROWS; ++j) {
            if (lane + 32 * j < nb) {
              spfo[32 * j] = Pv[j];
              gPF[32 * j] = pb0 * Sv[j] - pa0 * Pv[j];
            }
          }
        }
#pragma unroll
        for (int j = 0; j < ST_ROWS; ++j) {
          if (lane + 32 * j < nb) {
            gV[32 * j] = Vv[j];
            gW[32 * j] = Wv[j];
            if (gS) gS[32 * j] = Sv[j];
            sspk[32 * j] = Sv[j];
          }
        }
      }
      if (ok) {
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          atomicAdd(&e_done[h0.z], 1);
        }
      }
    } else if (ok && h0.x == 2) {
      // ---------------- D record: rows [r0, r0 + nr) of one decoder matrix ----------------
      const int nr = h1.w;  // nr * ntile <= ST_DITEMS by construction
      const int4 k0 = *reinterpret_cast<const int4*>(rec + 8);   // W element index, bytes, 0, neurons
      const int4 k1 = *reinterpret_cast<const int4*>(rec + 12);  // PES, alpha, error, decoded
      const int4 k2 = *reinterpret_cast<const int4*>(rec + 16);  // filtered, b0, a0, -
      const int n_e = k0.w;
      const int n4 = n_e >> 2;
      const int ntile = (n_e + 127) >> 7;
      const bool pes = k1.x != 0;
      // every E record of this ensemble must have delivered its spikes
      ok = stream_wait_count(&e_done[h0.z], h1.z, &s_abort, lane);
      if (ok) {
        if (pes) {
          // w += (alpha * error) * trace, with alpha * error formed once per row as in
          // `alpha * aa * xx` (left to right); the stage keeps the old values for the decode
          if (lane < nr) st.ae[lane] = bits(k1.y) * data[k1.z + lane];
          __syncwarp();
          // (pointers advance by immediates: the loop body is loads, 8 flops per row and stores)
          const float4* pf4 = reinterpret_cast<const float4*>(slot.pfo) + lane;
          const float4* w4p = reinterpret_cast<const float4*>(st.buf) + lane;
          float4* g4p = reinterpret_cast<float4*>(data + k0.x) + lane;
          const int iters = (n4 - lane + 31) >> 5;  // this lane's groups of 4 columns
          if (nr == 2) {
            const float a0 = st.ae[0], a1 = st.ae[1];
#pragma unroll 2
            for (int it = 0; it < iters; ++it) {
              const float4 p4 = pf4[32 * it];
              const float4 u = w4p[32 * it], v = w4p[n4 + 32 * it];
              g4p[32 * it] = pes_update(u, a0, p4);
              g4p[n4 + 32 * it] = pes_update(v, a1, p4);
            }
          } else {
            for (int rr = 0; rr < nr; ++rr) {
              const float a = st.ae[rr];
              const float4* wr = w4p + rr * n4;
              float4* gr = g4p + (size_t)rr * n4;
#pragma unroll 4
              for (int it = 0; it < iters; ++it) gr[32 * it] = pes_update(wr[32 * it], a, pf4[32 * it]);
            }
          }
        }
        // lanes 2 i and 2 i + 1 own pair i = row * ntile + tile: the even lane the partial sums 0
        // and 1 of the tile (columns 4 q and 4 q + 1, q ascending), the odd lane 2 and 3.  Tiles are
        // 128 floats apart, i.e. in the same banks: pair i starts i mod 8 iterations late, so the
        // 16 lanes that a 64-bit shared load serves at a time read 16 different bank pairs.
        const int item = lane >> 1, jp = lane & 1;
        const int rr = item / ntile, tt = item - rr * ntile;
        const bool valid = rr < nr;
        const int len = valid ? min(32, (n_e - (tt << 7)) >> 2) : 0;
        const int skew = item & 7;
        const float* wi = st.buf + (valid ? rr * n_e : 0) + (tt << 7) + 2 * jp - 4 * skew;
        const float* si = slot.spk + (tt << 7) + 2 * jp - 4 * skew;
        float ca = 0.0f, cb = 0.0f;
        {
          const int kmax = min(32, n4) + 7;
#pragma unroll 8
          for (int k = 0; k < kmax; ++k) {
            if ((unsigned)(k - skew) < (unsigned)len) {
              const float2 w2 = *reinterpret_cast<const float2*>(wi + 4 * k);
              const float2 s2 = *reinterpret_cast<const float2*>(si + 4 * k);
              ca = bd_add(ca, bd_mul(w2.x, s2.x));
              cb = bd_add(cb, bd_mul(w2.y, s2.y));
            }
          }
        }
        // tile = (s0 + s2) + (s1 + s3); the tiles of a row are added in order
        const float xa = bd_add(ca, __shfl_xor_sync(0xffffffffu, ca, 1));
        const float xb = bd_add(cb, __shfl_xor_sync(0xffffffffu, cb, 1));
        const float tile = bd_add(xa, xb);
        const int lane_t0 = 2 * (valid ? rr : 0) * ntile;
        float total = 0.0f;
        for (int t = 0; t < ntile; ++t) total = bd_add(total, __shfl_sync(0xffffffffu, tile, lane_t0 + 2 * t));
        if (valid && tt == 0 && jp == 0) {
          data[k1.w + rr] = total;
          if (k2.x >= 0) {
            const int yi = k2.x + rr;
            // plan_linearfilter fast path (clra_nonlinearities.py:657-660)
            float out = bits(k2.y) * total;
            if (k2.z != 0) out = out - bits(k2.z) * data[yi];
            data[yi] = out;
          }
        }
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          atomicAdd(&d_done[h0.z], 1);
        }
      }
    }
    if (!ok) {
      if (lane == 0) {
        s_abort = 1;
        if (p.status) atomicExch(p.status, NB2_ERR_TIMEOUT);
      }
      return;
    }
    __syncwarp();  // every lane is done with the stage
    if (i + ST_NW < n) {
      stream_issue(p, st, full, rp, i + ST_NW, m + 1, n, lane);
      stream_stage_x(p, st, st.rec[(m + 1) & 1], lane);
    }
  }
  if (xpush) {
    // The decoded values of this CTA's ensembles form one contiguous run of this rank's
    // segment (the host checked): its last warp stores the run into every peer's staging
    // buffer with whole-line stores (per-value peer stores would be one NVLink packet each),
    // and the last CTA of the grid publishes the step number to every peer.
    __threadfence();  // this warp's results before its count
    __syncwarp();
    int last = 0;
    if (lane == 0) last = atomicSub(&warps_left, 1) == 1;
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      __threadfence();  // the other warps' results after their counts
      const int2 run = reinterpret_cast<const int2*>(p.x.cta_runs)[blockIdx.x];  // first element (in the signal buffer), length
      const float* src = data + run.x;
      const size_t dst0 = xoff + (size_t)(run.x - p.x.x_base);
      for (int q = 0; q < p.x.world; ++q) {
        if (q == p.x.rank) continue;
        float* dst = p.x.peer_staging[q] + dst0;
        if (((run.x | run.y | (int)(dst0 & 3)) & 3) == 0) {
          for (int i = lane; i < (run.y >> 2); i += 32)
            reinterpret_cast<float4*>(dst)[i] = __ldcg(reinterpret_cast<const float4*>(src) + i);
        } else {
          for (int i = lane; i < run.y; i += 32) dst[i] = __ldcg(src + i);
        }
      }
      __threadfence_system();  // the peer stores before the flags
      __syncwarp();
      if (lane == 0 && atomicAdd(p.x.ctl + X_DONE_BLOCKS, 1) + 1 == (int)gridDim.x) {
        p.x.ctl[X_DONE_BLOCKS] = 0;
        __threadfence_system();
        for (int q = 0; q < p.x.world; ++q)
          if (q != p.x.rank) st_release_sys(p.x.peer_flags[q] + p.x.rank, epoch + 1);
        p.x.ctl[X_EPOCH] = epoch + 1;
      }
    }
  }
}

static const size_t kStreamSmem = sizeof(StreamStage) * ST_NW + sizeof(StreamSlot) * ST_SLOTS;

extern "C" int nb2_ensemble_stream(void* stream, const int* records, int n_records, const int* ranges, int n_ctas,
                                   const int* ens_table, const int* term_table, const int* conn_table, float* data,
                                   double dt, int* status, const nb2_exchange_desc* xch) {
  if (n_records == 0 || n_ctas == 0) return NB2_OK;
  NB2_REQUIRE(records && ranges && ens_table && term_table && conn_table && data, "null pointer");
  NB2_REQUIRE(dt > 0, "dt");
  NB2_REQUIRE((((uintptr_t)records | (uintptr_t)data) & 15) == 0, "records and data must be 16-byte aligned");
  static bool optin[64] = {};
  int dev = 0;
  NB2_CUDA(cudaGetDevice(&dev));
  if (dev >= 64 || !optin[dev]) {
    NB2_CUDA(cudaFuncSetAttribute(nb2_ensemble_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)kStreamSmem));
    if (dev < 64) optin[dev] = true;
  }
  StreamParams p;
  p.records = records; p.ranges = reinterpret_cast<const int2*>(ranges);
  p.ens_table = ens_table; p.term_table = term_table; p.conn_table = conn_table;
  p.data = data; p.dt = (float)dt; p.dt_inv = (float)(1.0 / dt); p.status = status;
  if (xch != NULL && xch->world > 1) {
    NB2_REQUIRE(xch->peer_staging && xch->peer_flags && xch->ctl && xch->cta_runs, "exchange descriptor");
    NB2_REQUIRE(xch->rank >= 0 && xch->rank < xch->world && xch->seg > 0 && xch->x_lo <= xch->x_hi,
                "exchange descriptor");
    p.x = *xch;
  } else {
    p.x = nb2_exchange_desc();
  }
  nb2_launch(nb2_ensemble_stream_kernel, dim3(n_ctas), dim3(ST_THREADS), kStreamSmem, nb2_stream(stream), p);
  NB2_LAUNCH_CHECK();
  return NB2_OK;
}
