/* Plain-C restatement of the reference's device kernels on the simulator's hot
 * path (paths below are relative to the nengo-ocl source tree).
 *
 * TEST INFRASTRUCTURE ONLY: this file is the compiled half of the CPU oracle.
 * The tests, the smoke check and the CPU-baseline leg of the benchmark load it
 * through oracle/cport.py; nothing in the product links or calls it.
 *
 * Arithmetic is IEEE float32 without fused multiply-add (compile with
 * -ffp-contract=off); expm1/log1p are evaluated in double and rounded once,
 * exactly as oracle/kernels.py does.  Every loop nest below is one kernel
 * launch of the reference; the OpenMP pragmas parallelise over the ragged
 * items of a launch, which is what the device does.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Thread count of the OpenMP loops below (a launcher may have exported OMP_NUM_THREADS=1 for its
 * workers; the timed baseline asks for the cores it is allowed to use).  Returns the count in use. */
int nb2o_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/* ---- block GEMV (clra_gemv.py:1018-1058 tile kernel, :1137-1153 reduce) ----
 * One item: total[i] (already beta * y_in[i]) += alpha * tile for every
 * 128-column tile of A (M x N, strides s0/s1) times x (stride xs), where a
 * tile is reduced by 4 column-strided partial sums combined as
 * (s0 + s2) + (s1 + s3).  alpha is a double literal in the kernel text. */
void nb2o_block_rows(const float* A, long s0, long s1, int M, int N, const float* x, long xs, float* total,
                     long ts, double alpha) {
  for (int i = 0; i < M; ++i) {
    const float* Ai = A + (long)i * s0;
    float tot = total[(long)i * ts];
    for (int j0 = 0; j0 < N; j0 += 128) {
      const int w = N - j0 < 128 ? N - j0 : 128;
      float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      for (int jj = 0; jj < w; ++jj) {
        const float p = Ai[(long)(j0 + jj) * s1] * x[(long)(j0 + jj) * xs];
        s[jj & 3] = s[jj & 3] + p;
      }
      const float a = s[0] + s[2];
      const float b = s[1] + s[3];
      const float tile = (float)(alpha * (double)(a + b));
      tot = tot + tile;
    }
    total[(long)i * ts] = tot;
  }
}

/* ---- LIF (clra_nonlinearities.py:1087-1132, upsample 1, not adaptive) ---- */
static inline float lif_one(float J, float* V, float* W, float tau, float ref, float amp, float dt, float dt_inv) {
  float v = *V, w = *W;
  w = w - dt;
  const float delta_t = (w > dt) ? 0.0f : (w < 0.0f) ? dt : dt - w;
  const float dV = -(float)expm1((double)(-delta_t / tau)) * (J - v);
  v = v + dV;
  int spiked = 0;
  if (v > 1.0f) {
    const float t_spike = dt + tau * (float)log1p((double)(-(v - 1.0f) / (J - 1.0f)));
    w = ref + t_spike;
    v = 0.0f;
    spiked = 1;
  } else if (v < 0.0f) {
    v = 0.0f;
  }
  *V = v;
  *W = w;
  return spiked ? amp * dt_inv : 0.0f;
}

void nb2o_lif(int n, double dt, const float* J, float* V, float* W, float* S, float tau, float ref, float amp) {
  const float dtf = (float)dt, dt_inv = (float)(1.0 / dt);
  for (int i = 0; i < n; ++i) S[i] = lif_one(J[i], V + i, W + i, tau, ref, amp, dtf, dt_inv);
}

/* ---- one time step of a batch of identical-shape PES ensembles, operator by
 * operator in the order the reference schedules them (nengo_ocl/simulator.py:
 * 352-356 with the greedy planner): every block below is one kernel launch
 * over all ensembles.  Arrays are [ensemble][...] contiguous.
 *   x[e][d]        input of the ensemble (already gathered)
 *   enc[e][n][d], bias[e][n], J/V/W/S[e][n]
 *   dec[e][dc][n], delta[e][dc][n], weighted/filtered/err[e][dc], pf[e][n]
 * Returns nothing; all state is updated in place. */
void nb2o_pes_step(int n_ens, int n, int d, int dc, double dt, const float* x, const float* enc,
                   const float* bias, float* J, float* V, float* W, float* S, float* dec, float* delta,
                   float* weighted, float* filtered, const float* err, float* pf, float tau, float ref,
                   float amp, float b0, float a0, float pb0, float pa0, float alpha) {
  const long nn = n, dd = d, cc = dc;
  /* plan_copy inc (clra_nonlinearities.py:242-260): decoders += delta of the previous step */
#pragma omp parallel for schedule(static)
  for (int e = 0; e < n_ens; ++e) {
    float* w = dec + e * cc * nn;
    const float* dl = delta + e * cc * nn;
    for (long i = 0; i < cc * nn; ++i) w[i] = w[i] + dl[i];
  }
  /* plan_copy (bias -> J) */
#pragma omp parallel for schedule(static)
  for (int e = 0; e < n_ens; ++e) memcpy(J + e * nn, bias + e * nn, sizeof(float) * nn);
  /* plan_block_gemv: J += enc . x */
#pragma omp parallel for schedule(static)
  for (int e = 0; e < n_ens; ++e)
    nb2o_block_rows(enc + e * nn * dd, dd, 1, n, d, x + e * dd, 1, J + e * nn, 1, 1.0);
  /* plan_lif */
#pragma omp parallel for schedule(static)
  for (int e = 0; e < n_ens; ++e)
    nb2o_lif(n, dt, J + e * nn, V + e * nn, W + e * nn, S + e * nn, tau, ref, amp);
  /* plan_reset (decoded value) */
#pragma omp parallel for schedule(static)
  for (int e = 0; e < n_ens; ++e)
    for (int r = 0; r < dc; ++r) weighted[e * cc + r] = 0.0f;
  /* plan_block_gemv: weighted += dec . S */
#pragma omp parallel for schedule(static)
  for (int e = 0; e < n_ens; ++e)
    nb2o_block_rows(dec + e * cc * nn, nn, 1, dc, n, S + e * nn, 1, weighted + e * cc, 1, 1.0);
  /* SimPES: delta = (alpha * err) outer pf  (plan_elementwise_inc, outer, :489-523) -- reads the
   * activity trace before this step's filter update */
#pragma omp parallel for schedule(static)
  for (int e = 0; e < n_ens; ++e)
    for (int r = 0; r < dc; ++r) {
      const float ae = alpha * err[e * cc + r];
      float* dl = delta + (e * cc + r) * nn;
      const float* p = pf + e * nn;
      for (int i = 0; i < n; ++i) dl[i] = ae * p[i];
    }
  /* plan_linearfilter, first order (:657-660): synapse and PES activity trace */
#pragma omp parallel for schedule(static)
  for (int e = 0; e < n_ens; ++e) {
    for (int r = 0; r < dc; ++r)
      filtered[e * cc + r] = b0 * weighted[e * cc + r] - a0 * filtered[e * cc + r];
    float* p = pf + e * nn;
    const float* s = S + e * nn;
    for (int i = 0; i < n; ++i) p[i] = pb0 * s[i] - pa0 * p[i];
  }
}

/* ---- one whole time step of the PES learning model on a batch of ensembles -------
 * (benchmark configuration 5).  Ensemble e has one decoded connection with a PES rule into
 * ensemble targets[e]; its error is played back from a table.  Operator order as the reference
 * schedules it: gather of the inputs (reset + one increment per incoming connection, in
 * connection order), table playback (plan_presentinput, clra_nonlinearities.py:1710-1728:
 * row `step % nt`), then the operators of nb2o_pes_step.  err_tables: [ensemble][nt][dc]. */
void nb2o_pes_model_step(int n_ens, int n, int d, int dc, double dt, int step, int nt, const int* targets,
                         const float* err_tables, float* x, const float* enc, const float* bias, float* J,
                         float* V, float* W, float* S, float* dec, float* delta, float* weighted,
                         float* filtered, float* err, float* pf, float tau, float ref, float amp, float b0,
                         float a0, float pb0, float pa0, float alpha) {
  /* plan_reset + plan_copy(inc): inputs = sum of the filtered outputs that target them */
  memset(x, 0, sizeof(float) * (size_t)n_ens * d);
  for (int e = 0; e < n_ens; ++e) {
    float* xt = x + (long)targets[e] * d;
    const float* f = filtered + (long)e * dc;
    for (int k = 0; k < d; ++k) xt[k] = xt[k] + f[k];
  }
  /* plan_presentinput + reset + copy(inc) into the error signal: 0 + table row */
  const int ti = step % nt;
#pragma omp parallel for schedule(static)
  for (int e = 0; e < n_ens; ++e)
    for (int k = 0; k < dc; ++k) err[(long)e * dc + k] = 0.0f + err_tables[((long)e * nt + ti) * dc + k];
  nb2o_pes_step(n_ens, n, d, dc, dt, x, enc, bias, J, V, W, S, dec, delta, weighted, filtered, err, pf, tau, ref,
                amp, b0, a0, pb0, pa0, alpha);
}
