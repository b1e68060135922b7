/*
 * norm_oracle.c -- CPU restatement of TritonHub's LayerNorm / RMSNorm forward and backward.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are compared with and
 * the CPU baseline that the benchmark times; no product code path may call it.
 *
 * Every function follows the reference's algorithm step by step (file:line cited at each
 * function).  Storage types are handled by the caller: inputs arrive as fp32 arrays holding
 * values already rounded to the storage type (widening fp16 / bf16 to fp32 is exact; fp64
 * inputs are narrowed first, which is what the reference's `.to(tl.float32)` does,
 * layernorm.py:31), and outputs leave as un-rounded fp32 for the caller to round once.
 *
 * Row sums are marked `omp simd reduction` (compiled with -fopenmp-simd, no OpenMP runtime):
 * like the reference's tl.sum, their association order is not the sequential one.
 *
 * acc64 = 0: all arithmetic in fp32, like the reference's kernels.
 * acc64 = 1: the same formulas evaluated in fp64 ("truth", used to scale tolerances).
 *
 * Pinned against (tests/test_oracle.py): outputs of the reference's own Triton kernel
 * bodies executed by Triton's interpreter (tests/golden/, made by tests/golden/make_golden.py)
 * and torch.nn.functional.layer_norm / rms_norm on CPU, the comparator the reference's
 * UnitTests use (UnitTests/Normalization/layernorm_unittest.py:17,37,46).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

/* ---- a minimal parallel-for over [0, n) on `g_threads` POSIX threads -------------------- */
static int g_threads = 1;
API void oracle_set_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }
API int oracle_get_threads(void) { return g_threads; }

typedef void (*range_fn)(int64_t begin, int64_t end, void* ctx);
typedef struct { range_fn fn; void* ctx; int64_t begin, end; } range_job;
static void* range_thread(void* a) {
  range_job* j = (range_job*)a;
  j->fn(j->begin, j->end, j->ctx);
  return NULL;
}
static void parallel_for(int64_t n, range_fn fn, void* ctx) {
  int t = g_threads;
  if (t > n) t = (int)(n > 0 ? n : 1);
  if (t <= 1) { fn(0, n, ctx); return; }
  pthread_t tid[256];
  range_job job[256];
  const int64_t chunk = (n + t - 1) / t;
  for (int i = 0; i < t; ++i) {
    job[i].fn = fn; job[i].ctx = ctx;
    job[i].begin = i * chunk;
    job[i].end = (i + 1) * chunk > n ? n : (i + 1) * chunk;
    if (job[i].begin > n) job[i].begin = n;
    pthread_create(&tid[i], NULL, range_thread, &job[i]);
  }
  for (int i = 0; i < t; ++i) pthread_join(tid[i], NULL);
}

/* One row of _layernorm_kernel_fwd (TritonHub/Normalization/layernorm.py:27-46) or, with
 * rms != 0, of _rmsnorm_kernel_fwd (TritonHub/Normalization/rmsnorm.py:24-38). */
#define ROW_FWD(ACC)                                                                     \
  do {                                                                                   \
    ACC mean = 0;                                                                        \
    if (!rms) {                                                                          \
      ACC s = 0;                                                                         \
      _Pragma("omp simd reduction(+ : s)")                                               \
      for (int64_t c = 0; c < N; ++c) s += (ACC)xr[c];                                   \
      mean = s / (ACC)N;                                  /* layernorm.py:32 */          \
    }                                                                                    \
    ACC q = 0;                                                                           \
    _Pragma("omp simd reduction(+ : q)")                                                 \
    for (int64_t c = 0; c < N; ++c) {                                                    \
      ACC d = (ACC)xr[c] - mean;                          /* layernorm.py:34 */          \
      q += d * d;                                                                        \
    }                                                                                    \
    ACC var = q / (ACC)N;                                 /* layernorm.py:35, rmsnorm.py:30 */ \
    ACC rs = (ACC)1 / (ACC)sqrt((double)(var + (ACC)eps)); /* layernorm.py:36 */          \
    if (sizeof(ACC) == 4) rs = (ACC)(1.0f / sqrtf((float)var + eps));                    \
    if (mean_out) mean_out[r] = (float)mean;              /* layernorm.py:33 */          \
    rstd_out[r] = (float)rs;                              /* layernorm.py:37 */          \
    for (int64_t c = 0; c < N; ++c) {                                                    \
      ACC yv = ((ACC)xr[c] - mean) * rs;                  /* layernorm.py:38 */          \
      if (w) yv = yv * (ACC)w[c];                         /* layernorm.py:40-42 */       \
      if (b) yv = yv + (ACC)b[c];                         /* layernorm.py:43-45 */       \
      yr[c] = (float)yv;                                                                 \
    }                                                                                    \
  } while (0)

/* Forward over M rows (host glue of _layernorm_fwd, layernorm.py:48-87: one program per row).
 * x: (M, N) with row stride xs; y: (M, N) contiguous; mean_out may be NULL for RMSNorm. */
typedef struct {
  const float *x, *w, *b;
  float *y, *mean_out, *rstd_out;
  int64_t xs, N;
  float eps;
  int rms, acc64;
} fwd_ctx;

static void fwd_rows(int64_t begin, int64_t end, void* vctx) {
  const fwd_ctx* k = (const fwd_ctx*)vctx;
  const float *w = k->w, *b = k->b;
  float *mean_out = k->mean_out, *rstd_out = k->rstd_out;
  const int64_t N = k->N;
  const float eps = k->eps;
  const int rms = k->rms;
  for (int64_t r = begin; r < end; ++r) {
    const float* xr = k->x + r * k->xs;
    float* yr = k->y + r * N;
    if (k->acc64) ROW_FWD(double);
    else ROW_FWD(float);
  }
}

API void oracle_norm_fwd(const float* x, int64_t xs, const float* w, const float* b, float* y, float* mean_out,
                         float* rstd_out, int64_t M, int64_t N, float eps, int rms, int acc64) {
  fwd_ctx k = {x, w, b, y, mean_out, rstd_out, xs, N, eps, rms, acc64};
  parallel_for(M, fwd_rows, &k);
}

/* One program of _layernorm_kernel_bwd (layernorm.py:113-153) / _rmsnorm_kernel_bwd
 * (rmsnorm.py:92-122): rows [row_start, row_end), dweight / dbias accumulated across them. */
#define PROG_BWD(ACC)                                                                    \
  do {                                                                                   \
    ACC* dwp = (ACC*)calloc((size_t)N, sizeof(ACC));                                     \
    ACC* dbp = (ACC*)calloc((size_t)N, sizeof(ACC));                                     \
    ACC* xh = (ACC*)malloc((size_t)N * sizeof(ACC));                                     \
    ACC* wdy = (ACC*)malloc((size_t)N * sizeof(ACC));                                    \
    for (int64_t r = row_start; r < row_end; ++r) {                                      \
      const float* xr = x + r * xs;                                                      \
      const float* gr = dy + r * dys;                                                    \
      float* dxr = dx + r * N;                                                           \
      ACC mu = rms ? (ACC)0 : (ACC)mean[r];                                              \
      ACC rs = (ACC)rstd[r];                                                             \
      ACC s1 = 0, s2 = 0;                                                                \
      _Pragma("omp simd reduction(+ : s1, s2)")                                          \
      for (int64_t c = 0; c < N; ++c) {                                                  \
        xh[c] = ((ACC)xr[c] - mu) * rs;                   /* layernorm.py:132 */         \
        wdy[c] = w ? (ACC)w[c] * (ACC)gr[c] : (ACC)gr[c]; /* layernorm.py:135,141 */     \
        dwp[c] += (ACC)gr[c] * xh[c];                     /* layernorm.py:136 */         \
        dbp[c] += (ACC)gr[c];                             /* layernorm.py:145 */         \
        s1 += xh[c] * wdy[c];                                                            \
        s2 += wdy[c];                                                                    \
      }                                                                                  \
      ACC c1 = s1 / (ACC)N;                               /* layernorm.py:137 */         \
      ACC c2 = rms ? (ACC)0 : s2 / (ACC)N;                /* layernorm.py:138 */         \
      for (int64_t c = 0; c < N; ++c)                                                    \
        dxr[c] = (float)((wdy[c] - (xh[c] * c1 + c2)) * rs); /* layernorm.py:139 */      \
    }                                                                                    \
    for (int64_t c = 0; c < N; ++c) {                     /* layernorm.py:150-153 */     \
      dw_part[(size_t)prog * N + c] = (double)dwp[c];                                    \
      db_part[(size_t)prog * N + c] = (double)dbp[c];                                    \
    }                                                                                    \
    free(dwp); free(dbp); free(xh); free(wdy);                                           \
  } while (0)

/* Backward over M rows with the reference's work split (host glue of _layernorm_bwd,
 * layernorm.py:155-209): `programs` programs (sm_count there) of ceil(M/programs) consecutive
 * rows each, one fp32 partial row per program, then the column sum of the partial rows
 * (`_dw.sum(0)`, layernorm.py:207-208) -- left to right here, in the accumulation type.
 * dw / db (N,) may be NULL.  The cast to the parameter dtype is the caller's. */
typedef struct {
  const float *x, *dy, *w, *mean, *rstd;
  float* dx;
  double *dw_part, *db_part;
  int64_t xs, dys, M, N, rows_per_program;
  int rms, acc64;
} bwd_ctx;

static void bwd_programs(int64_t begin, int64_t end, void* vctx) {
  const bwd_ctx* k = (const bwd_ctx*)vctx;
  const float *x = k->x, *dy = k->dy, *w = k->w, *mean = k->mean, *rstd = k->rstd;
  float* dx = k->dx;
  double *dw_part = k->dw_part, *db_part = k->db_part;
  const int64_t xs = k->xs, dys = k->dys, N = k->N;
  const int rms = k->rms;
  for (int64_t prog = begin; prog < end; ++prog) {
    const int64_t row_start = prog * k->rows_per_program;
    int64_t row_end = row_start + k->rows_per_program;
    if (row_end > k->M) row_end = k->M;                            /* layernorm.py:126 */
    if (k->acc64) PROG_BWD(double);
    else PROG_BWD(float);
  }
}

API int oracle_norm_bwd(const float* x, int64_t xs, const float* dy, int64_t dys, const float* w, const float* mean,
                        const float* rstd, float* dx, float* dw, float* db, int64_t M, int64_t N, int programs,
                        int rms, int acc64) {
  if (programs < 1) return 1;
  double* dw_part = (double*)calloc((size_t)programs * N, sizeof(double));
  double* db_part = (double*)calloc((size_t)programs * N, sizeof(double));
  if (!dw_part || !db_part) return 2;
  const int64_t rows_per_program = (M + programs - 1) / programs; /* layernorm.py:185 */
  bwd_ctx k = {x, dy, w, mean, rstd, dx, dw_part, db_part, xs, dys, M, N, rows_per_program, rms, acc64};
  parallel_for(programs, bwd_programs, &k);
  for (int64_t c = 0; c < N; ++c) {
    if (acc64) {
      double a = 0, bsum = 0;
      for (int p = 0; p < programs; ++p) { a += dw_part[(size_t)p * N + c]; bsum += db_part[(size_t)p * N + c]; }
      if (dw) dw[c] = (float)a;
      if (db) db[c] = (float)bsum;
    } else {
      float a = 0, bsum = 0;
      for (int p = 0; p < programs; ++p) { a += (float)dw_part[(size_t)p * N + c]; bsum += (float)db_part[(size_t)p * N + c]; }
      if (dw) dw[c] = a;
      if (db) db[c] = bsum;
    }
  }
  free(dw_part);
  free(db_part);
  return 0;
}

/* ---- GeLU: the activation that follows the norm in the reference's Quick Start ----------- */

/* One element of _gelu_kernel_fwd (TritonHub/Activations/gelu.py:20-28).  approx != 0: tanh form. */
#define GELU_FWD(ACC, X)                                                                  \
  (approx ? ({ ACC x_ = (X);                                                              \
               ACC inner_ = (ACC)sqrt(2.0 / M_PI) * (x_ + (ACC)0.044715 * x_ * x_ * x_);  /* gelu.py:22 */ \
               ACC e_ = (ACC)exp((double)((ACC)2 * inner_));                              /* gelu.py:23 */ \
               ACC t_ = (e_ - (ACC)1) / (e_ + (ACC)1);                                    /* gelu.py:24 */ \
               (ACC)0.5 * x_ * ((ACC)1 + t_); })                                          /* gelu.py:25 */ \
          : ({ ACC x_ = (X);                                                              \
               (ACC)0.5 * x_ * ((ACC)1 + (ACC)erf((double)(x_ / (ACC)sqrt(2.0)))); }))   /* gelu.py:27 */

/* One element of the derivative in _gelu_kernel_bwd (gelu.py:67-79). */
#define GELU_GRAD(ACC, X)                                                                 \
  (approx ? ({ ACC x_ = (X);                                                              \
               ACC k_ = (ACC)sqrt(2.0 / M_PI);                                            \
               ACC g_ = k_ * (x_ + (ACC)0.044715 * x_ * x_ * x_);                         /* gelu.py:69 */ \
               ACC e_ = (ACC)exp((double)((ACC)2 * g_));                                  /* gelu.py:70 */ \
               ACC t_ = (e_ - (ACC)1) / (e_ + (ACC)1);                                    /* gelu.py:71 */ \
               ACC gp_ = k_ * ((ACC)1 + (ACC)3 * (ACC)0.044715 * x_ * x_);                /* gelu.py:72 */ \
               (ACC)0.5 * ((ACC)1 + t_ + x_ * ((ACC)1 - t_ * t_) * gp_); })               /* gelu.py:73 */ \
          : ({ ACC x_ = (X);                                                              \
               ACC cdf_ = (ACC)0.5 * ((ACC)1 + (ACC)erf((double)(x_ / (ACC)sqrt(2.0))));  /* gelu.py:76 */ \
               ACC pdf_ = (ACC)exp((double)((ACC)-0.5 * x_ * x_)) / (ACC)sqrt(2.0 * M_PI);/* gelu.py:77 */ \
               cdf_ + x_ * pdf_; }))                                                      /* gelu.py:78 */

/* y = gelu(x) over n elements (_gelu_kernel_fwd, gelu.py:12-29). */
API void oracle_gelu_fwd(const float* x, float* y, int64_t n, int approx, int acc64) {
  for (int64_t i = 0; i < n; ++i)
    y[i] = acc64 ? (float)GELU_FWD(double, (double)x[i]) : (float)GELU_FWD(float, x[i]);
}

/* dx = dout * gelu'(x) over n elements (_gelu_kernel_bwd, gelu.py:56-81). */
API void oracle_gelu_bwd(const float* x, const float* dout, float* dx, int64_t n, int approx, int acc64) {
  for (int64_t i = 0; i < n; ++i)
    dx[i] = acc64 ? (float)((double)dout[i] * GELU_GRAD(double, (double)x[i])) : dout[i] * (float)GELU_GRAD(float, x[i]);
}

/* ---- Softmax / LogSoftmax over rows -------------------------------------------------------- */

/* _softmax_kernel_fwd (TritonHub/Activations/softmax.py:11-22) and _logsoftmax_kernel_fwd
 * (logsoftmax.py:11-24), one program per row. */
API void oracle_softmax_fwd(const float* x, float* y, int64_t M, int64_t N, int log_softmax, int acc64) {
  for (int64_t r = 0; r < M; ++r) {
    const float* xr = x + r * N;
    float* yr = y + r * N;
    float mx = -INFINITY;
    for (int64_t c = 0; c < N; ++c) mx = xr[c] > mx ? xr[c] : mx;          /* softmax.py:19 */
    if (acc64) {
      double den = 0;
      for (int64_t c = 0; c < N; ++c) den += exp((double)xr[c] - (double)mx); /* softmax.py:20-21 */
      for (int64_t c = 0; c < N; ++c) {
        const double z = (double)xr[c] - (double)mx;
        yr[c] = (float)(log_softmax ? z - log(den) : exp(z) / den);        /* softmax.py:22, logsoftmax.py:21-22 */
      }
    } else {
      float den = 0;
      for (int64_t c = 0; c < N; ++c) den += expf(xr[c] - mx);
      for (int64_t c = 0; c < N; ++c) {
        const float z = xr[c] - mx;
        yr[c] = log_softmax ? z - logf(den) : expf(z) / den;
      }
    }
  }
}

/* _softmax_kernel_bwd (softmax.py:48-62) and _logsoftmax_kernel_bwd (logsoftmax.py:51-68); `y` is
 * the forward's output (softmax.py:93-96). */
API void oracle_softmax_bwd(const float* y, const float* dout, float* dx, int64_t M, int64_t N, int log_softmax,
                            int acc64) {
  for (int64_t r = 0; r < M; ++r) {
    const float *yr = y + r * N, *gr = dout + r * N;
    float* dr = dx + r * N;
    if (acc64) {
      double s = 0;
      for (int64_t c = 0; c < N; ++c) s += log_softmax ? (double)gr[c] : (double)gr[c] * yr[c];
      for (int64_t c = 0; c < N; ++c)
        dr[c] = (float)(log_softmax ? (double)gr[c] - exp((double)yr[c]) * s      /* logsoftmax.py:63-65 */
                                    : -(double)yr[c] * s + (double)gr[c] * yr[c]); /* softmax.py:59 */
    } else {
      float s = 0;
      for (int64_t c = 0; c < N; ++c) s += log_softmax ? gr[c] : gr[c] * yr[c];
      for (int64_t c = 0; c < N; ++c) dr[c] = log_softmax ? gr[c] - expf(yr[c]) * s : -yr[c] * s + gr[c] * yr[c];
    }
  }
}

/* ---- p-norm / normalize over rows ---------------------------------------------------------- */

static double sgn(double v) { return v > 0 ? 1.0 : (v < 0 ? -1.0 : 0.0); }

/* _norm_fwd_kernel (TritonHub/Ops/norm.py:11-45): norms[r] = max((sum |x|^p)^(1/p), eps).  The
 * caller rounds the result to the storage type, as the kernel's store does (norm.py:41). */
API void oracle_pnorm_fwd(const float* x, float* norms, int64_t M, int64_t N, float p, float eps, int acc64) {
  for (int64_t r = 0; r < M; ++r) {
    const float* xr = x + r * N;
    if (acc64) {
      double acc = 0;
      for (int64_t c = 0; c < N; ++c)
        acc += p == 1.f ? fabs((double)xr[c]) : (p == 2.f ? (double)xr[c] * xr[c] : pow(fabs((double)xr[c]), (double)p)); /* :26-32 */
      double n = p == 2.f ? sqrt(acc) : (p == 1.f ? acc : pow(acc, 1.0 / (double)p));                                   /* :36-39 */
      norms[r] = (float)(n > (double)eps ? n : (double)eps);                                                             /* :40 */
    } else {
      float acc = 0;
      for (int64_t c = 0; c < N; ++c) acc += p == 1.f ? fabsf(xr[c]) : (p == 2.f ? xr[c] * xr[c] : powf(fabsf(xr[c]), p));
      float n = p == 2.f ? sqrtf(acc) : (p == 1.f ? acc : powf(acc, 1.0f / p));
      norms[r] = n > eps ? n : eps;
    }
  }
}

/* _norm_bwd_kernel (norm.py:66-101); `norms` as stored by the forward. */
API void oracle_pnorm_bwd(const float* x, const float* norms, const float* dout, float* dx, int64_t M, int64_t N,
                          float p, int acc64) {
  for (int64_t r = 0; r < M; ++r) {
    const float* xr = x + r * N;
    float* dr = dx + r * N;
    const double g = dout[r], n = norms[r];
    const double np1 = (p != 1.f && p != 2.f) ? pow(n, (double)p - 1.0) : n;                  /* norm.py:86-87 */
    for (int64_t c = 0; c < N; ++c) {
      const double v = xr[c];
      double d;
      if (p == 1.f) d = g * sgn(v);                                                          /* :93-95 */
      else if (p == 2.f) d = (g * v) / n;                                                    /* :96-97 */
      else d = (g * sgn(v) * pow(fabs(v), (double)p - 1.0)) / np1;                           /* :98-100 */
      dr[c] = acc64 ? (float)d : (float)d;
    }
  }
}

/* _normalize_bwd_kernel (TritonHub/Ops/normalize.py:61-117): x the input, y the forward's output,
 * norms as stored by the forward. */
API void oracle_normalize_bwd(const float* x, const float* y, const float* norms, const float* dout, float* dx,
                              int64_t M, int64_t N, float p, int acc64) {
  (void)acc64;
  for (int64_t r = 0; r < M; ++r) {
    const float *xr = x + r * N, *yr = y + r * N, *gr = dout + r * N;
    float* dr = dx + r * N;
    const double n = norms[r];
    double proj = 0;
    for (int64_t c = 0; c < N; ++c) proj += (p == 1.f ? (double)xr[c] : (double)yr[c]) * gr[c];   /* :87-95 */
    for (int64_t c = 0; c < N; ++c) {
      const double g = gr[c];
      double d;
      if (p == 1.f) d = g / n - sgn(xr[c]) * (proj / (n * n));                                    /* :101-105 */
      else if (p == 2.f) d = (g - yr[c] * proj) / n;                                              /* :106-108 */
      else d = g / n - sgn(xr[c]) * pow(fabs((double)xr[c]), (double)p - 1.0) * (proj / (pow(n, (double)p - 1.0) * n)); /* :109-113 */
      dr[c] = (float)d;
    }
  }
}
