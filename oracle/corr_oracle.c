/*
 * CPU oracle for the Theano CorrMM path (test infrastructure, not product code).
 *
 * A plain-C restatement of the algorithm in the reference file
 * theano/tensor/nnet/c_code/corr_gemm.c: unfold the image into a column
 * matrix (im2col), multiply with BLAS-style gemm once per image and group,
 * and for the input gradient fold the column matrix back (col2im).
 *
 *   forward      corr_gemm.c:305-336   top   = weight . col(bottom)
 *   gradWeights  corr_gemm.c:398-455   dW    = sum_n top_n . col(bottom_n)^T
 *   gradInputs   corr_gemm.c:489-527   dX_n  = col2im(weight^T . top_n)
 *   im2col       corr_gemm.c:31-59,    col2im corr_gemm.c:64-92
 *
 * Tensors are C-contiguous NCHW (bottom, top) and OIHW (weight), like the
 * arrays the reference makes contiguous at corr_gemm.c:149-151.  Pads are the
 * resolved values (no half/full sentinels), as computed by the caller.
 *
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may
 * call into this file; the CUDA library never does.
 *
 * Build: see oracle/build_oracle.py (REAL=float -> liboracle_f32.so,
 * REAL=double -> liboracle_f64.so).
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#ifndef REAL
#define REAL float
#endif

/* Fortran-style gemm: C(m x n, ldc) = alpha * op(A) * op(B) + beta * C, column major. */
typedef void (*gemm_fn)(const char *ta, const char *tb, const int *m, const int *n, const int *k,
                        const REAL *alpha, const REAL *a, const int *lda, const REAL *b,
                        const int *ldb, const REAL *beta, REAL *c, const int *ldc);
typedef void (*set_threads_fn)(int);

static gemm_fn g_ext_gemm = NULL;          /* optional external BLAS gemm */
static set_threads_fn g_ext_set_threads = NULL;

void oracle_set_gemm(void *fn, void *set_threads) {
  g_ext_gemm = (gemm_fn)fn;
  g_ext_set_threads = (set_threads_fn)set_threads;
}

int oracle_has_ext_gemm(void) { return g_ext_gemm != NULL; }

void oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Portable column-major gemm used when no BLAS was handed in.  Accumulates in
 * REAL like BLAS does; the loop order keeps the innermost access unit-stride. */
static void plain_gemm(char ta, char tb, int m, int n, int k, REAL alpha, const REAL *a, int lda,
                       const REAL *b, int ldb, REAL beta, REAL *c, int ldc) {
  for (int j = 0; j < n; ++j) {
    REAL *cj = c + (size_t)j * ldc;
    if (beta == (REAL)0) {
      for (int i = 0; i < m; ++i) cj[i] = 0;
    } else if (beta != (REAL)1) {
      for (int i = 0; i < m; ++i) cj[i] *= beta;
    }
    for (int p = 0; p < k; ++p) {
      const REAL bpj = alpha * ((tb == 'N') ? b[(size_t)j * ldb + p] : b[(size_t)p * ldb + j]);
      if (ta == 'N') {
        const REAL *ap = a + (size_t)p * lda;
        for (int i = 0; i < m; ++i) cj[i] += ap[i] * bpj;
      } else {
        for (int i = 0; i < m; ++i) cj[i] += a[(size_t)i * lda + p] * bpj;
      }
    }
  }
}

static void do_gemm(char ta, char tb, int m, int n, int k, REAL alpha, const REAL *a, int lda,
                    const REAL *b, int ldb, REAL beta, REAL *c, int ldc) {
  if (g_ext_gemm) {
    g_ext_gemm(&ta, &tb, &m, &n, &k, &alpha, a, &lda, b, &ldb, &beta, c, &ldc);
  } else {
    plain_gemm(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
  }
}

/* Python-style floor division (corr_gemm.c:180-185 needs it for negative sizes). */
static int floordiv(int x, int y) {
  int q = x / y;
  if ((x % y != 0) && ((x < 0) != (y < 0))) --q;
  return q;
}

int oracle_out_size(int in, int k, int dil, int pad_l, int pad_r, int stride) {
  return floordiv(in + pad_l + pad_r - ((k - 1) * dil + 1), stride) + 1;
}

/* col[(c*kH*kW + i*kW + j), oh, ow] = im[c, oh*sH - pH + i*dilH, ow*sW - pW + j*dilW] or 0. */
static void unfold(const REAL *im, int C, int H, int W, int kH, int kW, int dilH, int dilW,
                   int pH, int pW, int sH, int sW, int Ho, int Wo, REAL *col) {
  const int rows = C * kH * kW;
  for (int r = 0; r < rows; ++r) {
    const int j = r % kW, i = (r / kW) % kH, c = r / (kW * kH);
    for (int oh = 0; oh < Ho; ++oh) {
      const int h = oh * sH - pH + i * dilH;
      REAL *dst = col + ((size_t)r * Ho + oh) * Wo;
      if (h < 0 || h >= H) {
        for (int ow = 0; ow < Wo; ++ow) dst[ow] = 0;
        continue;
      }
      const REAL *src = im + ((size_t)c * H + h) * W;
      for (int ow = 0; ow < Wo; ++ow) {
        const int w = ow * sW - pW + j * dilW;
        dst[ow] = (w >= 0 && w < W) ? src[w] : (REAL)0;
      }
    }
  }
}

/* Inverse scatter of unfold(): accumulates into im, which the caller zeroed. */
static void fold(const REAL *col, int C, int H, int W, int kH, int kW, int dilH, int dilW, int pH,
                 int pW, int sH, int sW, int Ho, int Wo, REAL *im) {
  const int rows = C * kH * kW;
  for (int r = 0; r < rows; ++r) {
    const int j = r % kW, i = (r / kW) % kH, c = r / (kW * kH);
    for (int oh = 0; oh < Ho; ++oh) {
      const int h = oh * sH - pH + i * dilH;
      if (h < 0 || h >= H) continue;
      const REAL *src = col + ((size_t)r * Ho + oh) * Wo;
      REAL *dst = im + ((size_t)c * H + h) * W;
      for (int ow = 0; ow < Wo; ++ow) {
        const int w = ow * sW - pW + j * dilW;
        if (w >= 0 && w < W) dst[w] += src[ow];
      }
    }
  }
}

/*
 * direction 0: top <- corr(bottom, weight); 1: weight <- grad; 2: bottom <- grad.
 * Shapes: bottom [N,C,H,W], weight [K,C/g,kH,kW], top [N,K,Ho,Wo].
 * Returns 0, or -1 shape inconsistency (the reference's ValueError at
 * corr_gemm.c:164-237), -2 allocation failure.
 */
int oracle_corr(int direction, REAL *bottom, REAL *weight, REAL *top, int N, int C, int H, int W,
                int K, int kH, int kW, int Ho, int Wo, int sH, int sW, int dilH, int dilW,
                int padH_l, int padH_r, int padW_l, int padW_r, int groups) {
  if (groups < 1 || C % groups || K % groups) return -1;
  if (Ho != oracle_out_size(H, kH, dilH, padH_l, padH_r, sH) ||
      Wo != oracle_out_size(W, kW, dilW, padW_l, padW_r, sW))
    return -1;
  const size_t nb = (size_t)N * C * H * W, nw = (size_t)K * (C / groups) * kH * kW,
               nt = (size_t)N * K * Ho * Wo;
  if (N == 0 || C == 0 || K == 0) { /* corr_gemm.c:281-296: zero-fill the output */
    if (direction == 0) memset(top, 0, nt * sizeof(REAL));
    if (direction == 1) memset(weight, 0, nw * sizeof(REAL));
    if (direction == 2) memset(bottom, 0, nb * sizeof(REAL));
    return 0;
  }
  const int M_ = K / groups;                /* filters per group            */
  const int K_ = (C / groups) * kH * kW;    /* unfolded rows per group      */
  const int N_ = Ho * Wo;                   /* output pixels per image      */
  int nthreads = oracle_max_threads();
  if (nthreads > N) nthreads = N;
  const size_t col_elems = (size_t)K_ * groups * N_;
  REAL *col = (REAL *)malloc(sizeof(REAL) * col_elems * nthreads);
  REAL *wpart = NULL;
  if (!col) return -2;
  if (direction == 1) {
    wpart = (REAL *)calloc(nw * nthreads, sizeof(REAL));
    if (!wpart) { free(col); return -2; }
  }
  if (direction == 2) memset(bottom, 0, nb * sizeof(REAL));
  if (g_ext_set_threads) g_ext_set_threads(1); /* one BLAS thread per OpenMP thread, corr_gemm.c:303 */

#pragma omp parallel for schedule(static) num_threads(nthreads)
  for (int n = 0; n < N; ++n) {
#ifdef _OPENMP
    const int tid = omp_get_thread_num();
#else
    const int tid = 0;
#endif
    REAL *mycol = col + col_elems * tid;
    REAL *bn = bottom + (size_t)n * C * H * W;
    REAL *tn = top + (size_t)n * K * N_;
    if (direction != 2)
      unfold(bn, C, H, W, kH, kW, dilH, dilW, padH_l, padW_l, sH, sW, Ho, Wo, mycol);
    for (int g = 0; g < groups; ++g) {
      REAL *colg = mycol + (size_t)g * K_ * N_;
      REAL *wg = weight + (size_t)g * M_ * K_;
      REAL *tg = tn + (size_t)g * M_ * N_;
      if (direction == 0) {
        /* row-major top[M_,N_] = W[M_,K_] col[K_,N_]  ==  col-major (N_ x M_) = col * W */
        do_gemm('N', 'N', N_, M_, K_, 1, colg, N_, wg, K_, 0, tg, N_);
      } else if (direction == 1) {
        /* row-major dW[M_,K_] += top[M_,N_] col[K_,N_]^T */
        REAL *wp = wpart + nw * tid + (size_t)g * M_ * K_;
        do_gemm('T', 'N', K_, M_, N_, 1, colg, N_, tg, N_, 1, wp, K_);
      } else {
        /* row-major col[K_,N_] = W[M_,K_]^T top[M_,N_] */
        do_gemm('N', 'T', N_, K_, M_, 1, tg, N_, wg, K_, 0, colg, N_);
      }
    }
    if (direction == 2)
      fold(mycol, C, H, W, kH, kW, dilH, dilW, padH_l, padW_l, sH, sW, Ho, Wo, bn);
  }

  if (direction == 1) { /* thread-ordered sum of partials, corr_gemm.c:443-455 */
#pragma omp parallel for schedule(static)
    for (ptrdiff_t e = 0; e < (ptrdiff_t)nw; ++e) {
      REAL s = 0;
      for (int t = 0; t < nthreads; ++t) s += wpart[nw * t + e];
      weight[e] = s;
    }
    free(wpart);
  }
  free(col);
  return 0;
}

/* Pool(ignore_border=True, mode='max') with ws == stride == (2,2), pad 0
 * (theano/tensor/signal/pool.py:524-574): out[n,c,i,j] = max of the 2x2 window. */
void oracle_maxpool2x2(const REAL *x, REAL *y, int N, int C, int H, int W) {
  const int Ho = H / 2, Wo = W / 2;
#pragma omp parallel for schedule(static)
  for (ptrdiff_t nc = 0; nc < (ptrdiff_t)N * C; ++nc) {
    const REAL *xi = x + (size_t)nc * H * W;
    REAL *yo = y + (size_t)nc * Ho * Wo;
    for (int i = 0; i < Ho; ++i)
      for (int j = 0; j < Wo; ++j) {
        REAL m = xi[(size_t)(2 * i) * W + 2 * j];
        const REAL b = xi[(size_t)(2 * i) * W + 2 * j + 1];
        const REAL c = xi[(size_t)(2 * i + 1) * W + 2 * j];
        const REAL d = xi[(size_t)(2 * i + 1) * W + 2 * j + 1];
        if (b > m) m = b;
        if (c > m) m = c;
        if (d > m) m = d;
        yo[(size_t)i * Wo + j] = m;
      }
  }
}
