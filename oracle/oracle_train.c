/*
 * CPU oracle (C, OpenMP) for the FlyVec train step and hashing rule.
 * TEST INFRASTRUCTURE ONLY: it checks the CUDA library and serves as the timed
 * CPU baseline of the benchmark.  Nothing in the product links or calls it.
 *
 * It restates the reference's live training path literally, dense `ds` matrix
 * included, one "device" after the other (paths relative to the reference
 * project root):
 *   activations        flyvec/src/cuda_funcs.cu:248-263, 289-305
 *   winner / m-th max  flyvec/src/cuda_funcs.cu:488-561
 *   xx                 flyvec/src/cuda_funcs.cu:722-744
 *   ds = -xx * W       flyvec/src/cuda_funcs.cu:394-406
 *   scatter            flyvec/src/cuda_funcs.cu:657-672
 *   combine + abs-max  flyvec/src/cu_special_reduction.cu:26-99
 *   step size          flyvec/src/cuda_funcs.cu:1797-1799
 *   update             flyvec/src/cu_special_reduction.cu:316-354
 * Pinning: checked bit for bit against the numpy restatement (oracle/flyvec_oracle.py) and
 * against the reference's own kernel text executed on the host (oracle/ref_kernels_host.cpp,
 * built from a reference checkout) in tests/test_oracle.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <omp.h>

/* Tie order of get_max_and_m_max_kernel_2 (flyvec/src/cuda_funcs.cu:488-561), 64 threads per window:
 * a thread keeps its lowest index (strict '>', 507-512); the __shfl_down_sync tree with offsets
 * 16..1 keeps the lower lane at every level (515-522), so among tied lanes the one with the smallest
 * bit-reversed lane number reaches lane 0; warp 0 is preferred over warp 1 (535-540). */
static int tie_key(int i) {
  const int t = i & 63, lane = t & 31;
  const int rev = ((lane & 1) << 4) | ((lane & 2) << 2) | (lane & 4) | ((lane & 8) >> 2) | ((lane & 16) >> 4);
  return (((t >> 5) << 5 | rev) << 20) | i;
}

/* arg-max with the reference's tie order: smallest tie_key among equal maxima */
static int argmax_ref(const float* a, int K) {
  int best = 0;
  for (int i = 1; i < K; ++i) {
    if (a[i] > a[best] || (a[i] == a[best] && tie_key(i) < tie_key(best))) best = i;
  }
  return best;
}

/*
 * One global step over G devices.
 *   Wm    [K][N]  synapses, updated in place
 *   idx   [G][B][W] input ids (token, centre token + V, -1 = padding)
 *   nwin  [G]     windows actually present on each device (<= B)
 *   f     [V]     inverse word frequency
 *   win   [G][B]  winners out (may be NULL)      xx [G][K] out (may be NULL)
 *   scratch: (G+1)*K*N floats provided by the caller
 * Returns nc through *nc_out and the step size through *s_out.
 */
int orc_train_step(int K, int N, int V, int W, int B, int G, float* Wm, const int32_t* idx, const int32_t* nwin,
                   const float* f, float eps, float prec, int32_t* win, float* xx, float* nc_out, float* s_out,
                   float* scratch) {
  const size_t KN = (size_t)K * N;
  float* D = scratch;             /* combined update direction */
  float* ds_all = scratch + KN;   /* G dense ds matrices */
  float* xx_all = (float*)calloc((size_t)G * K, sizeof(float));
  int32_t* win_all = (int32_t*)malloc((size_t)G * B * sizeof(int32_t));
  float* aw_all = (float*)malloc((size_t)G * B * sizeof(float));
  if (!xx_all || !win_all || !aw_all) return 1;

  for (int g = 0; g < G; ++g) {
    const int nb = nwin[g];
    const int32_t* gi = idx + (size_t)g * B * W;
    /* activations + winner: double running sums over c = 0..W-1, float store */
#pragma omp parallel
    {
      float* ar = (float*)malloc((size_t)K * sizeof(float));
      double* acc = (double*)malloc((size_t)K * sizeof(double));
#pragma omp for schedule(static)
      for (int j = 0; j < nb; ++j) {
        for (int mu = 0; mu < K; ++mu) acc[mu] = 0.0;
        for (int c = 0; c < W; ++c) {
          const int id = gi[(size_t)j * W + c];
          if (id == -1) continue;
          for (int mu = 0; mu < K; ++mu) acc[mu] += (double)Wm[(size_t)mu * N + id]; /* ds = W for p = 2 */
        }
        for (int mu = 0; mu < K; ++mu) ar[mu] = (float)acc[mu];
        const int w = argmax_ref(ar, K);
        double s = 0.0;
        for (int c = 0; c < W; ++c) {
          const int id = gi[(size_t)j * W + c];
          if (id == -1) continue;
          const float prod = Wm[(size_t)w * N + id] * f[id % V]; /* float product */
          s += (double)prod;
        }
        win_all[(size_t)g * B + j] = w;
        aw_all[(size_t)g * B + j] = (float)s;
      }
      free(ar);
      free(acc);
    }
    /* xx: float adds in window order (one admissible order of the reference's atomics) */
    float* xg = xx_all + (size_t)g * K;
    for (int j = 0; j < nb; ++j) xg[win_all[(size_t)g * B + j]] += aw_all[(size_t)g * B + j];
    /* ds = -xx * W, or 0 where xx == 0 */
    float* ds = ds_all + (size_t)g * KN;
#pragma omp parallel for schedule(static)
    for (int mu = 0; mu < K; ++mu) {
      const float x = xg[mu];
      float* row = ds + (size_t)mu * N;
      const float* wrow = Wm + (size_t)mu * N;
      if (x != 0.0f)
        for (int i = 0; i < N; ++i) row[i] = -x * wrow[i];
      else
        memset(row, 0, (size_t)N * sizeof(float));
    }
    /* scatter: ds[win][id] += f[id % V], one float add per occurrence */
    for (int j = 0; j < nb; ++j) {
      float* row = ds + (size_t)win_all[(size_t)g * B + j] * N;
      for (int c = 0; c < W; ++c) {
        const int id = gi[(size_t)j * W + c];
        if (id != -1) row[id] += f[id % V];
      }
    }
  }

  /* combine: mean over the devices where the row was active; abs-max */
  float nc = 0.0f;
#pragma omp parallel for schedule(static) reduction(max : nc)
  for (int mu = 0; mu < K; ++mu) {
    int nnz = 0;
    for (int g = 0; g < G; ++g) nnz += (xx_all[(size_t)g * K + mu] != 0.0f);
    float* drow = D + (size_t)mu * N;
    if (nnz == 0) {
      memset(drow, 0, (size_t)N * sizeof(float));
      continue;
    }
    const double inv = 1.0 / (double)nnz;
    for (int i = 0; i < N; ++i) {
      double sum = 0.0;
      for (int g = 0; g < G; ++g)
        if (xx_all[(size_t)g * K + mu] != 0.0f) sum += (double)ds_all[(size_t)g * KN + (size_t)mu * N + i];
      const float sum_f = (float)((double)(float)sum * inv);
      drow[i] = sum_f;
      const float a = fabsf(sum_f);
      if (a > nc) nc = a;
    }
  }
  const float s = (prec > nc) ? eps / prec : eps / nc;
  /* update */
#pragma omp parallel for schedule(static)
  for (int mu = 0; mu < K; ++mu) {
    int nnz = 0;
    for (int g = 0; g < G; ++g) nnz += (xx_all[(size_t)g * K + mu] != 0.0f);
    if (nnz == 0) continue;
    float* wrow = Wm + (size_t)mu * N;
    const float* drow = D + (size_t)mu * N;
    for (int i = 0; i < N; ++i) {
      const float val = s * drow[i];
      if (fabs((double)val) > 1.e-10) wrow[i] = wrow[i] + val;
    }
  }
  if (win) memcpy(win, win_all, (size_t)G * B * sizeof(int32_t));
  if (xx) memcpy(xx, xx_all, (size_t)G * K * sizeof(float));
  if (nc_out) *nc_out = nc;
  if (s_out) *s_out = s;
  free(xx_all);
  free(win_all);
  free(aw_all);
  return 0;
}

static int cmp_desc(const void* a, const void* b) {
  const float x = *(const float*)a, y = *(const float*)b;
  return (x < y) - (x > y);
}

/*
 * Context-independent codes (flyvec/core.py:139-185): activation = column V+id
 * of syn [K][N]; threshold at the float midpoint of the h-th and (h+1)-th
 * largest; strict '>'; id 0 gives zeros.  codes: [n][K] bytes.
 */
int orc_hash_tokens(const float* syn, int K, int N, int V, const int32_t* ids, int64_t n, int h, int8_t* codes) {
  if (h < 1 || h >= K) return 1;
#pragma omp parallel
  {
    float* act = (float*)malloc((size_t)K * sizeof(float));
    float* srt = (float*)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t t = 0; t < n; ++t) {
      int8_t* out = codes + (size_t)t * K;
      const int id = ids[t];
      if (id == 0) {
        memset(out, 0, (size_t)K);
        continue;
      }
      for (int mu = 0; mu < K; ++mu) act[mu] = syn[(size_t)mu * N + V + id];
      memcpy(srt, act, (size_t)K * sizeof(float));
      qsort(srt, (size_t)K, sizeof(float), cmp_desc);
      const float thr = (srt[h - 1] + srt[h]) / 2.0f;
      for (int mu = 0; mu < K; ++mu) out[mu] = act[mu] > thr;
    }
    free(act);
    free(srt);
  }
  return 0;
}

int orc_num_threads(void) { return omp_get_max_threads(); }
void orc_set_num_threads(int n) { omp_set_num_threads(n > 0 ? n : 1); }
