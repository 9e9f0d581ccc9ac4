/* C ABI of libnengo_b200.so: the sm_100a device layer behind the
 * nengo_ocl-compatible Python planning surface.
 *
 * The reference (nengo_ocl) has no FFI of its own: its device boundary is
 * PyOpenCL.  Each entry point below names the reference interface it stands
 * in for (paths relative to the nengo-ocl source tree).  A maintainer of the
 * reference binds these with ctypes exactly as nengo_ocl_b200/_capi.py does.
 *
 * Conventions: every function returns 0 on success or a negative NB2_ERR_*
 * code (nb2_last_error() then holds a message for the calling thread); no
 * ownership crosses the boundary; pointers named d_* / without prefix in
 * kernel entry points are DEVICE pointers owned by the caller; `stream` is a
 * cudaStream_t passed as void* (NULL = legacy default stream); index tables
 * are int32 in element units, as in the reference's ragged arrays.
 */
#ifndef NENGO_B200_H
#define NENGO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NB2_ABI_VERSION 1

/* ---- runtime: replaces pyopencl Context/CommandQueue/Array --------------
 * nengo_ocl/simulator.py:209-219 (context + queue), clraggedarray.py:36-62,
 * 128-196 (to_device, to_host, enqueue_copy), plan.py:85-149 (enqueue loop). */
const char* nb2_last_error(void);
int nb2_abi_version(void);
/* Kernels are launched with the programmatic-stream-serialization attribute
 * (the next kernel of a stream or captured graph is scheduled while the
 * current one runs and waits, at its first instruction, for everything before
 * it to complete): the launch gaps of a step's chain of small kernels overlap
 * with execution, data dependencies are those of an in-order stream.  On by
 * default; 0 turns it off (also: environment variable NENGO_B200_PDL=0).  No
 * counterpart in the reference (one OpenCL in-order queue, plan.py:85-91). */
int nb2_set_programmatic_launch(int enabled);
int nb2_device_count(int* count);
int nb2_set_device(int ordinal);
int nb2_device_info(int ordinal, int* sm_count, int* max_threads_per_block, size_t* global_mem,
                    size_t* shared_mem_per_block_optin, int* cc_major, int* cc_minor);
int nb2_malloc(void** dptr, size_t bytes); /* 256-byte aligned, size rounded up to 256 bytes */
int nb2_free(void* dptr);
int nb2_host_alloc(void** hptr, size_t bytes); /* pinned host memory */
int nb2_host_free(void* hptr);
int nb2_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream, int sync);
int nb2_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream, int sync);
int nb2_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream);
int nb2_memset(void* dst, int byte_value, size_t bytes, void* stream);
int nb2_stream_create(void** stream);
int nb2_stream_destroy(void* stream);
int nb2_stream_sync(void* stream);
int nb2_device_sync(void);
int nb2_event_create(void** event);
int nb2_event_destroy(void* event);
int nb2_event_record(void* event, void* stream);
/* the work submitted to `stream` after this call waits for `event` (while capturing: a graph edge) */
int nb2_stream_wait_event(void* stream, void* event);
int nb2_event_sync(void* event);
int nb2_event_elapsed_ms(void* start, void* stop, float* ms);
/* Step-loop replay: Plans.call_n_times (plan.py:128-149) becomes a captured
 * CUDA graph of one (or several) steps launched n times. */
int nb2_graph_begin(void* stream);
int nb2_graph_end(void* stream, void** graph_exec);
int nb2_graph_abort(void* stream);
int nb2_graph_launch(void* graph_exec, void* stream, int n_times);
int nb2_graph_destroy(void* graph_exec);
/* Peer mapping for the multi-GPU exchange (no counterpart: the reference is
 * single-device, simulator.py:215-219). handle64 is a 64-byte opaque blob. */
int nb2_ipc_get_handle(void* dptr, void* handle64);
int nb2_ipc_open_handle(const void* handle64, void** dptr);
int nb2_ipc_close_handle(void* dptr);

/* ---- ragged gather-GEMV --------------------------------------------------
 * Replaces clra_gemv.py ref_impl :264-444, reduce_impl :447-670,
 * many_dots_impl :673-858, block_impl :861-1175 (all four compute
 * Y = gamma + beta*Y_in + alpha*sum_j A_j X_j).  `gstructure` is the int32
 * table of cl_geometry_and_textconf (clra_gemv.py:211-261), row stride
 * `gstride`, D = max dots.  `xstrides` ([n_items][D], may be NULL = all 1)
 * carries X element strides (honoured by ref_impl/block_impl :371-376,1037).
 * `worklist` holds n_units int4 = {item row, first row, row count, 0};
 * row count <= NB2_GEMV_RMAX (CTA kinds) or <= 32 (warp kind).
 * alphas/betas/gammas: optional per-item float vectors indexed by the item id
 * stored in the table (float_cl_clra, clra_gemv.py:17-32); NULL = use the
 * scalar.  `status` (may be NULL) receives NB2_ERR_TIMEOUT if a bounded wait
 * inside the kernel gave up. */
#define NB2_GEMV_CTA 0      /* CTA per unit, 128-bit global loads into smem */
#define NB2_GEMV_CTA_BULK 1 /* CTA per unit, cp.async.bulk + mbarrier staging */
#define NB2_GEMV_WARP 2     /* warp per unit, tiny items */
#define NB2_GEMV_ROWS 4     /* CTA per row group, direct global loads, 8 rows per thread;
                               worklist .w = log2(lanes per row), row count <= 8 * (256 >> .w) */
#define NB2_GEMV_ABUF 8192
#define NB2_GEMV_XBUF 2048
#define NB2_GEMV_RMAX 1024
int nb2_gemv_ragged(void* stream, int kind, const int* gstructure, int gstride, int D,
                    const int* xstrides, const int* worklist, int n_units, const float* A,
                    const float* X, const float* Yin, float* Y, double alpha, double beta,
                    double gamma, const float* alphas, const float* betas, const float* gammas,
                    int* status);

/* plan_block_gemv (clra_gemv.py:861-1175; the variant the reference simulator
 * plans for every MultiDotInc, simulator.py:803) with that kernel pair's exact
 * float32 summation order: 128-column tiles, four column-strided partial sums
 * per tile combined as (s0 + s2) + (s1 + s3), tiles added in order to
 * beta * Y_in, gamma last; scalar alpha / beta / gamma only (as block_impl,
 * :863-880).  Same index table as nb2_gemv_ragged.  cta_units / warp_units:
 * int4 {item row, first row, row count, 0}; row count <= 32 for CTA units,
 * <= 8 for warp units.  Results are bit-identical to the reference kernels
 * evaluated without fused multiply-add. */
int nb2_gemv_block(void* stream, const int* gstructure, int gstride, int D, const int* xstrides,
                   const int* cta_units, int n_cta, const int* warp_units, int n_warp, const float* A,
                   const float* X, const float* Yin, float* Y, double alpha, double beta, double gamma);

/* The main GEMV path: persistent CTAs whose warps each own one shared-memory
 * stage fed by 1-D bulk async copies (cp.async.bulk) only.  Same math and
 * reference counterparts as nb2_gemv_ragged.  `records`: n_records x 32 int32
 * work records (layout documented in
 * nengo_ocl_b200/cura_gemv.py:build_pipe_records); `ranges`: n_ctas x 2 int32
 * [begin, end) record ranges, one per CTA; record i of a range is worked on by
 * warp i % NB2_PIPE_WARPS (chains are interleaved accordingly).
 * `records`, `A`, `X` and `Yin` must be 16-byte aligned and readable up to the
 * next 16-byte boundary past their last element (any nb2_malloc buffer is):
 * unaligned sources are staged as their enclosing 16-byte-aligned window. */
#ifndef NB2_PIPE_STAGE_FLOATS
#define NB2_PIPE_STAGE_FLOATS 4300 /* floats of one stage's pool */
#define NB2_PIPE_WARPS 12          /* warps per CTA, one stage each */
#define NB2_PIPE_CTAS_PER_SM 1
#endif
#define NB2_PIPE_RMAX 128 /* rows per record */
int nb2_gemv_pipelined(void* stream, const int* records, int n_records, const int* ranges, int n_ctas,
                       const float* A, const float* X, const float* Yin, float* Y, double alpha,
                       double beta, double gamma, const float* alphas, const float* betas,
                       const float* gammas, int* status);

/* ---- sparse transforms (clra_gemv.py:1242-1997) ---------------------------
 * y (+)= A x for one sparse matrix; x and y are contiguous vectors.
 * nb2_spmv_csr: spmv_csr_impl :1570-1646; `lanes_log2` (0..5) lanes share a row.
 * nb2_spmv_ell: spmv_ellpack_impl :1649-1755 and spmv_ellpacktwostep_impl
 * :1758-1916 (no scratch buffer, one launch); `rowlens` bounds every row;
 * `row_major` = 1: entry (row, k) at row * width + k (one warp per row),
 * 0: at k * n_rows + row (one thread per row, for narrow matrices). */
int nb2_spmv_csr(void* stream, const int* indices, const int* indptr, const float* data, int n_rows,
                 int lanes_log2, const float* x, float* y, int inc);
int nb2_spmv_ell(void* stream, const int* columns, const float* entries, const int* rowlens, int n_rows,
                 int width, int row_major, const float* x, float* y, int inc);

/* ---- elementwise family (clra_nonlinearities.py) -------------------------
 * All index tables have the layout the reference's plan functions upload. */
/* plan_timeupdate :113-144 */
int nb2_timeupdate(void* stream, float* step, float* time, double dt);
/* plan_reset :147-214; blocks of <=16 elements */
int nb2_reset(void* stream, int n_blocks, const float* values, const int* sizes, const int* starts,
              float* Y);
/* plan_copy :217-304; blocks of 256; inc_mode 0 = set, 1 = inc, 2 = per-block incdata */
int nb2_copy(void* stream, int n_blocks, int inc_mode, const int* incdata, const int* offsets,
             const int* shape0s, const int* shape1s, const int* Xstride0s, const int* Xstarts,
             const float* X, const int* Ystride0s, const int* Ystarts, float* Y);
/* plan_slicedcopy :307-411; blocks of 16 */
int nb2_slicedcopy(void* stream, int n_blocks, int inc_mode, const int* incdata,
                   const int* Xstride0s, const int* Xstarts, const float* X, const int* Ystride0s,
                   const int* Ystarts, float* Y, const int* Isizes, const int* XIstarts,
                   const int* XIdata, const int* YIstarts, const int* YIdata);
/* plan_elementwise_inc :414-574 (outer=1 is the PES delta, simulator.py:1334-1345) */
int nb2_elementwise_inc(void* stream, int n_blocks, int outer, int inc, const float* alphas,
                        const int* offsets, const int* Ashape0s, const int* Ashape1s,
                        const int* Astride0s, const int* Astarts, const float* A,
                        const int* Xshape0s, const int* Xshape1s, const int* Xstride0s,
                        const int* Xstarts, const float* X, const int* Yshape0s,
                        const int* Yshape1s, const int* Ystride0s, const int* Ystarts, float* Y);
/* plan_bcm :2082-2169, plan_oja :2172-2277, plan_voja :2280-2405: weight deltas of the
 * unsupervised learning rules, one thread per delta element; `aux` = theta (vector) for
 * BCM, the weights for Oja, the scaled encoders for Voja; `betas` only for Oja, the
 * learning signal and `scale` only for Voja (NULL otherwise). */
#define NB2_RULE_BCM 0
#define NB2_RULE_OJA 1
#define NB2_RULE_VOJA 2
int nb2_learning_delta(void* stream, int rule, int n_items, int max_size, const int* shape0s,
                       const int* shape1s, const int* pre_stride0s, const int* pre_starts, const float* pre,
                       const int* post_stride0s, const int* post_starts, const float* post,
                       const int* aux_stride0s, const int* aux_starts, const float* aux,
                       const int* delta_stride0s, const int* delta_starts, float* delta, const float* alphas,
                       const float* betas, const int* learn_starts, const float* learn,
                       const int* scale_stride0s, const int* scale_starts, const float* scale);
/* plan_linearfilter :577-803 (+ linearfilter_inc ring-position kernel when uses_buf) */
int nb2_linearfilter(void* stream, int n_blocks, int block_size, int uses_buf, const int* offsets,
                     const int* shape0s, const int* shape1s, const int* Xstride0s,
                     const int* Xstride1s, const int* Xstarts, const float* X,
                     const int* Ystride0s, const int* Ystride1s, const int* Ystarts, float* Y,
                     const int* Ashape0s, const int* Astarts, const float* A, const int* Bshape0s,
                     const int* Bstarts, const float* B, const int* Xbufstarts, float* Xbuf,
                     const int* Ybufstarts, float* Ybuf, int* Xbufpos, int* Ybufpos);
/* plan_probes :806-951; one CTA of `block_size` threads per probe */
int nb2_probes(void* stream, int n_probes, int block_size, float* countdowns, int* bufpositions,
               const float* periods, const int* Xstarts, const int* Xshape0s, const int* Xshape1s,
               const int* Xstride0s, const int* Xstride1s, const float* X, const int* Ystarts,
               float* Y);
/* plan_probes for large probes: `chunks` CTAs share one probe; `arrive`: n_probes ints of
 * scratch, zero before the first launch (the kernel leaves them zero). */
int nb2_probes_wide(void* stream, int n_probes, int chunks, float* countdowns, int* bufpositions,
                    const float* periods, const int* Xstarts, const int* Xshape0s, const int* Xshape1s,
                    const int* Xstride0s, const int* Xstride1s, const float* X, const int* Ystarts,
                    float* Y, int* arrive);
/* nb2_probes_wide without any allocation (no reference counterpart): for callers
 * that cannot allocate device memory at this point (inside a stream capture, or
 * with a fixed memory budget handed out elsewhere), the arrival counters live in
 * a 16 KB device array of the library (NB2_PROBES_STATIC_MAX probes at most; more
 * are rejected with NB2_ERR_ARG).  The first call on a device looks the array's
 * device address up (once per device, under a lock); make that first call before
 * any stream capture.  Every call shares the one array: the kernel leaves the
 * counters zero, but two launches that overlap in time on one GPU (two streams,
 * two host threads) race on them and must not be issued. */
#define NB2_PROBES_STATIC_MAX 4096
int nb2_probes_wide_noalloc(void* stream, int n_probes, int chunks, float* countdowns, int* bufpositions,
                            const float* periods, const int* Xstarts, const int* Xshape0s,
                            const int* Xshape1s, const int* Xstride0s, const int* Xstride1s,
                            const float* X, const int* Ystarts, float* Y);
/* plan_presentinput :1678-1759; pres_t may be NULL (table indexed by step);
 * Sstride0s may be NULL (table rows packed, as in the reference) or give the
 * row stride of every table (tables that are column blocks of one buffer) */
int nb2_presentinput(void* stream, int n_items, int block_size, const float* pres_t, double dt,
                     const int* Yshape0s, const int* Ystarts, float* Y, const int* Tstarts,
                     const float* T, const int* Sshape0s, const int* Sstarts, const int* Sstride0s,
                     const float* S);

/* plan_whitenoise (:1573-1675), with a counter-based generator (Philox4x32-10)
 * in place of the reference's per-work-item RANLUX states (create_rngs /
 * init_rngs, :1486-1532): element e of item k at a step is word e % 4 of
 * philox(counter = (step, e / 4, 0, 0), key = seeds[2k], seeds[2k+1]); the step
 * is read from T[Tstarts[k]].  enums[k]: 0 uniform (params[2k] = low, [2k+1] =
 * high), 1 gaussian (mean, std); scales[k]: multiply by 1/sqrt(dt); incs[k]: add
 * to Y instead of overwriting it.  The random stream differs from RANLUX; what
 * is done with a sample does not. */
int nb2_whitenoise(void* stream, int n_items, int max_len, const int* shape0s, const int* Ystarts, float* Y,
                   const int* Tstarts, const float* T, const int* enums, const float* params, const int* scales,
                   const int* incs, const unsigned* seeds, double dt);

/* plan_conv2d (:1762-1969) on one image: y[k,i,j] = sum over c, ii, jj (in that
 * order, from zero) of filter * x[c, i*sti - pi + ii, j*stj - pj + jj], zero
 * outside the image; the result is stored (inc == 0, the reference kernel) or
 * added to y (inc != 0).  conv != 0: shared filters laid out
 * [si][sj][nc][nf]; conv == 0 (local filtering): [nf][nc][si][sj][nyi][nyj].
 * channels_last selects [rows][cols][channels] against [channels][rows][cols]
 * for x and y.  Biases are not supported (the reference asserts them absent). */
int nb2_conv2d(void* stream, const float* x, const float* filters, float* y, int nc, int nxi, int nxj, int nf,
               int nyi, int nyj, int si, int sj, int sti, int stj, int pi, int pj, int channels_last, int conv, int inc);
/* plan_pool2d (:1972-2079): average over the part of each si x sj window (stride
 * sti, stj) that lies inside the image; x [nc][nxi][nxj], y [nc][nyi][nyj]. */
int nb2_pool2d(void* stream, const float* x, float* y, int nc, int nyi, int nyj, int nxi, int nxj, int si, int sj,
               int sti, int stj);

/* Reset-then-accumulate in one launch: the reference runs plan_reset (:147-214)
 * and then one plan_copy(inc) (:217-304) per group of non-overlapping targets.
 * blocks [n_blocks][4] = {dst start, elements (<= 256), first source, n sources};
 * src_starts holds the element offset of every (block, source) pair; sources are
 * added in order starting from zero.  width: threads per block of the table, a
 * power of two >= the longest block (256 / width blocks share one CTA). */
int nb2_gather_sum(void* stream, int n_blocks, int width, const int* blocks, const int* src_starts,
                   float* data);

/* Neuron models generated by _plan_template (:1286-1483): plan_lif :1028-1146,
 * plan_lif_rate :1149-1197, plan_spiking_rectified_linear :1200-1235,
 * plan_rectified_linear :1238-1259, plan_sigmoid :1262-1283.  Each variable is
 * a per-block starts table plus a buffer; a parameter with buf == NULL is the
 * constant `value` (the reference's static_params). */
typedef struct {
  const int* starts;
  float* buf;
  float value;
} nb2_var;
typedef struct {
  nb2_var J, V, W, S, N;              /* S = output (spikes or rates); N = adaptation */
  nb2_var tau, ref, amp, tau_n, inc_n; /* parameters */
  double dt;
  int upsample;
  int adaptive;
  int fastlif; /* LIF only: the `fastlif` variant of the kernel text (:1079-1114) */
} nb2_neuron_args;
#define NB2_NEURON_LIF 0
#define NB2_NEURON_LIF_RATE 1
#define NB2_NEURON_RELU 2
#define NB2_NEURON_SPIKING_RELU 3
#define NB2_NEURON_SIGMOID 4
int nb2_neurons(void* stream, int kind, int n_blocks, int block_size, const int* sizes,
                const nb2_neuron_args* args);

/* plan_direct :954-1025: the reference compiles a translated Python function
 * per node; here the translation is a postfix program run by one interpreter
 * kernel.  prog: n_ops int32 pairs {opcode, operand}; consts: double pool (the
 * program is evaluated in double and results rounded to float when stored, as
 * the Python function itself computes); max_depth: evaluation-stack depth the
 * program needs, at most NB2_DIRECT_STACK (csrc/nb2_direct_ops.h) or the call
 * is rejected.  Inputs: up to 2 ragged inputs (starts table + buffer + dim);
 * one output. */
int nb2_direct(void* stream, int n_items, const int* prog, int n_ops, int max_depth, const double* consts,
               int out_dim, const int* in0_starts, const float* in0, const int* in1_starts,
               const float* in1, const int* out_starts, float* out);

/* ---- fused ensemble step --------------------------------------------------
 * One launch replaces, for every population matching the pattern, the
 * reference's per-step sequence plan_copy (bias) + plan_block_gemv (encoders,
 * clra_gemv.py:861-1175) + plan_lif (clra_nonlinearities.py:1028-1146) +
 * plan_reset + plan_block_gemv (decoders) + plan_linearfilter (:577-803) and,
 * with PES, plan_linearfilter (activity filter) + plan_elementwise_inc(outer)
 * (simulator.py:1334-1345) + plan_copy (decoders += delta).
 * `data` is the one packed signal buffer; all table entries are int32 element
 * offsets into it (floats stored as bit patterns):
 *   ens_table  [n][16]: n, J (-1 = not stored), V, W, S (-1 = not stored), bias,
 *                       n_terms, first term, n_conns, first conn, tau_rc, tau_ref,
 *                       amplitude, 0, 0, 0
 *   term_table [..][4]: encoder start (row-major n x d), d, x start, x stride
 *   conn_table [..][16]: decoder start (row-major d_c x n), d_c, decoded start,
 *                       filtered start (-1 = no synapse), b0, a0, pes flag, error
 *                       start, activity-filter state start, its b0, its a0, alpha
 * large_ids / small_ids list the ensembles run by a 256-thread CTA (n <=
 * NB2_FUSED_MAX_NEURONS) or by one warp (n <= NB2_FUSED_SMALL_NEURONS); the sum
 * of the d of an ensemble's terms must be <= NB2_FUSED_MAX_INPUT. */
#define NB2_FUSED_MAX_NEURONS 4096
#define NB2_FUSED_SMALL_NEURONS 256
#define NB2_FUSED_MAX_INPUT 512
int nb2_ensemble_step(void* stream, int n_large, const int* large_ids, int n_small, const int* small_ids,
                      const int* ens_table, const int* term_table, const int* conn_table, float* data,
                      double dt);

/* The same fused step for large populations as a bulk-copy pipeline (persistent
 * CTAs, one shared-memory stage per warp, cp.async.bulk + mbarrier).  `records`:
 * n_records x 32 int32 work records and `ranges`: n_ctas x 2 int32 [begin, end)
 * record ranges, one per CTA, as built by
 * nengo_ocl_b200/fusion.py:stream_records; the three tables are those of
 * nb2_ensemble_step.  Only ensembles whose arrays start on multiples of 4 floats,
 * with n % 4 == 0, n <= NB2_STREAM_MAX_NEURONS, total encoder width <=
 * NB2_STREAM_MAX_INPUT and at most one PES connection may be streamed.
 * `status` (may be NULL) receives NB2_ERR_TIMEOUT if a bounded wait gave up. */
#ifndef NB2_STREAM_STAGE_FLOATS
#define NB2_STREAM_STAGE_FLOATS 2048 /* floats of one stage */
#define NB2_STREAM_WARPS 20          /* warps per CTA, one stage each */
#endif
#ifndef NB2_STREAM_SLOTS
#define NB2_STREAM_SLOTS 3 /* ensembles in flight per CTA (spikes + PES trace in shared memory) */
#endif
#define NB2_STREAM_MAX_NEURONS 1024
#define NB2_STREAM_MAX_INPUT 64
/* Optional push of the step's decoded values to the other GPUs, folded into
 * nb2_ensemble_stream (the counterpart of nb2_exchange_push): CTA b stores the
 * run cta_runs[b] = {first element in the signal buffer, length} (its share of
 * this rank's segment [x_lo, x_hi) of the exchange signal, which starts at
 * element x_base and has world * seg floats) into every peer's staging buffer
 * when it is done; the last CTA publishes the step in the peers' flag words.
 * `peer_staging`, `peer_flags`: device arrays of `world` pointers; `ctl`: the
 * control block shared with nb2_exchange_wait. */
typedef struct nb2_exchange_desc {
  float* const* peer_staging;
  int* const* peer_flags;
  int* ctl;
  const int* cta_runs; /* n_ctas x 2 */
  int x_base, x_lo, x_hi;
  int rank, world, seg;
} nb2_exchange_desc;
int nb2_ensemble_stream(void* stream, const int* records, int n_records, const int* ranges, int n_ctas,
                        const int* ens_table, const int* term_table, const int* conn_table, float* data,
                        double dt, int* status, const nb2_exchange_desc* xch /* NULL: none */);

/* ---- multi-GPU exchange of decoded signals ---------------------------------
 * No counterpart in the reference (single device, simulator.py:215-219).  Every
 * rank holds a replica of one exchange signal of world*seg floats and owns
 * segment `rank`.  nb2_exchange_push (end of a step) stores the local segment
 * into every peer's staging buffer (2 * world * seg floats, alternating by step
 * parity) through peer pointers and publishes the step number in the peer's
 * flag array (world ints); nb2_exchange_wait (start of the next step) waits at
 * most timeout_s for all peers' flags and copies the staged segments into the
 * replica.  `ctl`: 8 ints of local device memory, zero-initialised (step
 * counter, block counter, status = NB2_ERR_TIMEOUT after a timed-out wait).
 * peer_staging / peer_flags: device arrays of `world` pointers (entry `rank`
 * unused) obtained with nb2_ipc_open_handle. */
int nb2_exchange_wait(void* stream, int* ctl, const int* flags, const float* staging, float* replica,
                      int rank, int world, int seg, double timeout_s);
int nb2_exchange_push(void* stream, int* ctl, float* const* peer_staging, int* const* peer_flags,
                      const float* replica, int rank, int world, int seg);

/* ---- persistent step loop ---------------------------------------------------
 * Replaces Plans.call_n_times / enqueue_n_times (nengo_ocl/plan.py:137-149: every
 * kernel of every plan enqueued n times) for models whose plans all have a phase
 * form: ONE cooperative launch runs n whole steps.  A loop is built once:
 * create, one add call per plan in plan order (same arguments as the launch
 * entry point of that name without the stream; `barrier` != 0 puts a grid-wide
 * barrier before the phase - required whenever the phase reads or writes what
 * an earlier phase since the last barrier wrote, or writes what one read,
 * counting the previous step's phases as earlier), finalize, then run any
 * number of times.  Results are bit-identical to the separate launches: the
 * phases execute the same device code.  Ring-buffer filters, wide probes and
 * the streamed ensemble kernel have no phase form (the add call returns
 * NB2_ERR_LIMIT or does not exist): such models keep the launch-per-plan path.
 * finalize: max_ctas > 0 caps the grid (0: as many CTAs as are co-resident, at
 * most the widest phase).  A grid of ONE CTA (max_ctas == 1, or no phase wider
 * than one block) runs a variant whose barrier is a CTA barrier and whose loads
 * stay in that multiprocessor's L1: the form that pays for very small models
 * (nb2_step_loop_info: total_vblocks = blocks of all phases of one step).  A barrier wait is bounded (about a second); if it
 * runs out the kernel returns and nb2_step_loop_status reports NB2_ERR_TIMEOUT
 * (sticky) after synchronising the stream. */
#define NB2_STEP_LOOP_MAX_PHASES 64
int nb2_step_loop_create(void** loop);
int nb2_step_loop_destroy(void* loop);
int nb2_step_loop_add_timeupdate(void* loop, int barrier, float* step, float* time, double dt);
int nb2_step_loop_add_gather_sum(void* loop, int barrier, int n_blocks, int width, const int* blocks,
                                 const int* src_starts, float* data);
int nb2_step_loop_add_direct(void* loop, int barrier, int n_items, const int* prog, int n_ops, int max_depth,
                             const double* consts, int out_dim, const int* in0_starts, const float* in0,
                             const int* in1_starts, const float* in1, const int* out_starts, float* out);
int nb2_step_loop_add_ensemble_step(void* loop, int barrier, int n_large, const int* large_ids, int n_small,
                                    const int* small_ids, const int* ens_table, const int* term_table,
                                    const int* conn_table, float* data, double dt);
int nb2_step_loop_add_gemv_block(void* loop, int barrier, const int* gstructure, int gstride, int D,
                                 const int* xstrides, const int* cta_units, int n_cta, const int* warp_units,
                                 int n_warp, const float* A, const float* X, const float* Yin, float* Y,
                                 double alpha, double beta, double gamma);
int nb2_step_loop_add_probes(void* loop, int barrier, int n_probes, int block_size, float* countdowns,
                             int* bufpositions, const float* periods, const int* Xstarts, const int* Xshape0s,
                             const int* Xshape1s, const int* Xstride0s, const int* Xstride1s, const float* X,
                             const int* Ystarts, float* Y);
int nb2_step_loop_add_linearfilter(void* loop, int barrier, int n_blocks, int block_size, int uses_buf,
                                   const int* offsets, const int* shape0s, const int* shape1s,
                                   const int* Xstride0s, const int* Xstride1s, const int* Xstarts, const float* X,
                                   const int* Ystride0s, const int* Ystride1s, const int* Ystarts, float* Y,
                                   const int* Ashape0s, const int* Astarts, const float* A, const int* Bshape0s,
                                   const int* Bstarts, const float* B, const int* Xbufstarts, float* Xbuf,
                                   const int* Ybufstarts, float* Ybuf, int* Xbufpos, int* Ybufpos);
int nb2_step_loop_add_presentinput(void* loop, int barrier, int n_items, int block_size, const float* pres_t,
                                   double dt, const int* Yshape0s, const int* Ystarts, float* Y,
                                   const int* Tstarts, const float* T, const int* Sshape0s, const int* Sstarts,
                                   const int* Sstride0s, const float* S);
int nb2_step_loop_finalize(void* loop, int max_ctas);
int nb2_step_loop_run(void* loop, void* stream, int n_steps);
int nb2_step_loop_info(void* loop, int* n_phases, int* n_barriers, int* grid, int* total_vblocks);
/* Self-test of the bounded wait: runs the cooperative loop with every barrier expecting one arrival
 * more than the grid has CTAs, so that the first barrier can only run out; the kernel must return
 * within the wait limit with NB2_ERR_TIMEOUT in the status word (then nb2_step_loop_clear_status).
 * The model's state is advanced by part of a step: call it on a scratch model only. */
int nb2_step_loop_wait_selftest(void* loop, void* stream);
int nb2_step_loop_clear_status(void* loop, void* stream);
int nb2_step_loop_status(void* loop, void* stream, int* status);

#ifdef __cplusplus
}
#endif
#endif /* NENGO_B200_H */
