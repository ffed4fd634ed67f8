/* Type-generic body of the CPU oracle.  Included twice by pb_oracle.c with
 * T / SUF defined (double/_f64 and float/_f32).  TEST INFRASTRUCTURE ONLY.
 *
 * Every kernel restates one PolyBench/C 4.2 loop nest of the reference
 * (paths relative to tools/cgeist/Test/polybench/) with run-time sizes and
 * leading dimensions.  Statement order, loop order and the association of
 * each product are kept exactly as in the source, so that for equal inputs
 * the result is bit-identical to the reference compiled without FP
 * contraction. */

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUF)

/* linear-algebra/blas/gemm/gemm.c:104-113
 *   for i { for j C[i][j] *= beta;
 *           for k for j C[i][j] += alpha * A[i][k] * B[k][j]; } */
void FN(pbo_gemm)(int64_t ni, int64_t nj, int64_t nk, T alpha, T beta,
                  T *C, int64_t ldc, const T *A, int64_t lda,
                  const T *B, int64_t ldb)
{
  for (int64_t i = 0; i < ni; i++) {
    for (int64_t j = 0; j < nj; j++)
      C[i * ldc + j] *= beta;
    for (int64_t k = 0; k < nk; k++) {
      for (int64_t j = 0; j < nj; j++)
        C[i * ldc + j] += alpha * A[i * lda + k] * B[k * ldb + j];
    }
  }
}

/* linear-algebra/kernels/2mm/2mm.c:103-119
 *   nest 1: tmp[i][j] = 0; for k tmp[i][j] += alpha * A[i][k] * B[k][j];
 *   nest 2: D[i][j] *= beta; for k D[i][j] += tmp[i][k] * C[k][j]; */
void FN(pbo_2mm)(int64_t ni, int64_t nj, int64_t nk, int64_t nl, T alpha,
                 T beta, T *tmp, int64_t ldtmp, const T *A, int64_t lda,
                 const T *B, int64_t ldb, const T *C, int64_t ldcc, T *D,
                 int64_t ldd)
{
  for (int64_t i = 0; i < ni; i++)
    for (int64_t j = 0; j < nj; j++) {
      tmp[i * ldtmp + j] = (T)0.0;
      for (int64_t k = 0; k < nk; ++k)
        tmp[i * ldtmp + j] += alpha * A[i * lda + k] * B[k * ldb + j];
    }
  for (int64_t i = 0; i < ni; i++)
    for (int64_t j = 0; j < nl; j++) {
      D[i * ldd + j] *= beta;
      for (int64_t k = 0; k < nj; ++k)
        D[i * ldd + j] += tmp[i * ldtmp + k] * C[k * ldcc + j];
    }
}

/* linear-algebra/kernels/mvt/mvt.c:102-109
 *   nest 1: x1[i] = x1[i] + A[i][j] * y_1[j];
 *   nest 2: x2[i] = x2[i] + A[j][i] * y_2[j];
 * [row0,row1) restricts the outer i of both nests (the full kernel is
 * row0=0,row1=n); each x[i] depends on no other x, so a restricted run is
 * bit-identical to the full one on those entries. */
void FN(pbo_mvt_range)(int64_t n, int64_t row0, int64_t row1, T *x1, T *x2,
                       const T *y1, const T *y2, const T *A, int64_t lda)
{
  for (int64_t i = row0; i < row1; i++)
    for (int64_t j = 0; j < n; j++)
      x1[i] = x1[i] + A[i * lda + j] * y1[j];
  for (int64_t i = row0; i < row1; i++)
    for (int64_t j = 0; j < n; j++)
      x2[i] = x2[i] + A[j * lda + i] * y2[j];
}

void FN(pbo_mvt)(int64_t n, T *x1, T *x2, const T *y1, const T *y2,
                 const T *A, int64_t lda)
{
  FN(pbo_mvt_range)(n, 0, n, x1, x2, y1, y2, A, lda);
}

/* linear-algebra/blas/syrk/syrk.c:97-106
 *   for i { for j<=i C[i][j] *= beta;
 *           for k for j<=i C[i][j] += alpha * A[i][k] * A[j][k]; }
 * The strict upper triangle of C is never touched.  [row0,row1) restricts i;
 * A must still hold rows 0..row1-1. */
void FN(pbo_syrk_range)(int64_t row0, int64_t row1, int64_t m, T alpha,
                        T beta, T *C, int64_t ldc, const T *A, int64_t lda)
{
  for (int64_t i = row0; i < row1; i++) {
    for (int64_t j = 0; j <= i; j++)
      C[i * ldc + j] *= beta;
    for (int64_t k = 0; k < m; k++) {
      for (int64_t j = 0; j <= i; j++)
        C[i * ldc + j] += alpha * A[i * lda + k] * A[j * lda + k];
    }
  }
}

void FN(pbo_syrk)(int64_t n, int64_t m, T alpha, T beta, T *C, int64_t ldc,
                  const T *A, int64_t lda)
{
  FN(pbo_syrk_range)(0, n, m, alpha, beta, C, ldc, A, lda);
}

/* linear-algebra/kernels/3mm/3mm.c:99-124
 *   E = A*B ; F = C*D ; G = E*F, each as  X[i][j] = 0; for k X[i][j] += L[i][k]*R[k][j] */
void FN(pbo_3mm)(int64_t ni, int64_t nj, int64_t nk, int64_t nl, int64_t nm, T *E,
                 const T *A, const T *B, T *F, const T *C, const T *D, T *G)
{
  for (int64_t i = 0; i < ni; i++)
    for (int64_t j = 0; j < nj; j++) {
      E[i * nj + j] = (T)0.0;
      for (int64_t k = 0; k < nk; ++k)
        E[i * nj + j] += A[i * nk + k] * B[k * nj + j];
    }
  for (int64_t i = 0; i < nj; i++)
    for (int64_t j = 0; j < nl; j++) {
      F[i * nl + j] = (T)0.0;
      for (int64_t k = 0; k < nm; ++k)
        F[i * nl + j] += C[i * nm + k] * D[k * nl + j];
    }
  for (int64_t i = 0; i < ni; i++)
    for (int64_t j = 0; j < nl; j++) {
      G[i * nl + j] = (T)0.0;
      for (int64_t k = 0; k < nj; ++k)
        G[i * nl + j] += E[i * nj + k] * F[k * nl + j];
    }
}

/* linear-algebra/kernels/atax/atax.c:89-99
 *   y = 0; for i { tmp[i] = 0; for j tmp[i] += A[i][j]*x[j];
 *                  for j y[j] += A[i][j]*tmp[i]; }          A is m x n */
void FN(pbo_atax)(int64_t m, int64_t n, const T *A, int64_t lda, const T *x, T *y,
                  T *tmp)
{
  for (int64_t i = 0; i < n; i++)
    y[i] = 0;
  for (int64_t i = 0; i < m; i++) {
    tmp[i] = (T)0.0;
    for (int64_t j = 0; j < n; j++)
      tmp[i] = tmp[i] + A[i * lda + j] * x[j];
    for (int64_t j = 0; j < n; j++)
      y[j] = y[j] + A[i * lda + j] * tmp[i];
  }
}

/* linear-algebra/kernels/bicg/bicg.c:97-108
 *   s = 0; for i { q[i] = 0; for j { s[j] += r[i]*A[i][j]; q[i] += A[i][j]*p[j]; } }
 *   A is n x m */
void FN(pbo_bicg)(int64_t m, int64_t n, const T *A, int64_t lda, T *s, T *q,
                  const T *p, const T *r)
{
  for (int64_t i = 0; i < m; i++)
    s[i] = 0;
  for (int64_t i = 0; i < n; i++) {
    q[i] = (T)0.0;
    for (int64_t j = 0; j < m; j++) {
      s[j] = s[j] + r[i] * A[i * lda + j];
      q[i] = q[i] + A[i * lda + j] * p[j];
    }
  }
}

/* linear-algebra/blas/gesummv/gesummv.c:99-109
 *   for i { tmp[i] = 0; y[i] = 0;
 *           for j { tmp[i] = A[i][j]*x[j] + tmp[i]; y[i] = B[i][j]*x[j] + y[i]; }
 *           y[i] = alpha*tmp[i] + beta*y[i]; } */
void FN(pbo_gesummv)(int64_t n, T alpha, T beta, const T *A, int64_t lda, const T *B,
                     int64_t ldb, T *tmp, const T *x, T *y)
{
  for (int64_t i = 0; i < n; i++) {
    tmp[i] = (T)0.0;
    y[i] = (T)0.0;
    for (int64_t j = 0; j < n; j++) {
      tmp[i] = A[i * lda + j] * x[j] + tmp[i];
      y[i] = B[i * ldb + j] * x[j] + y[i];
    }
    y[i] = alpha * tmp[i] + beta * y[i];
  }
}

/* linear-algebra/blas/syr2k/syr2k.c:100-109
 *   for i { for j<=i C[i][j] *= beta;
 *           for k for j<=i C[i][j] += A[j][k]*alpha*B[i][k] + B[j][k]*alpha*A[i][k]; } */
void FN(pbo_syr2k)(int64_t n, int64_t m, T alpha, T beta, T *C, int64_t ldc, const T *A,
                   int64_t lda, const T *B, int64_t ldb)
{
  for (int64_t i = 0; i < n; i++) {
    for (int64_t j = 0; j <= i; j++)
      C[i * ldc + j] *= beta;
    for (int64_t k = 0; k < m; k++)
      for (int64_t j = 0; j <= i; j++)
        C[i * ldc + j] += A[j * lda + k] * alpha * B[i * ldb + k] + B[j * ldb + k] * alpha * A[i * lda + k];
  }
}

/* linear-algebra/blas/gemver/gemver.c:114-131 (four nests, in order) */
void FN(pbo_gemver)(int64_t n, T alpha, T beta, T *A, int64_t lda, const T *u1, const T *v1,
                    const T *u2, const T *v2, T *w, T *x, const T *y, const T *z)
{
  for (int64_t i = 0; i < n; i++)
    for (int64_t j = 0; j < n; j++)
      A[i * lda + j] = A[i * lda + j] + u1[i] * v1[j] + u2[i] * v2[j];
  for (int64_t i = 0; i < n; i++)
    for (int64_t j = 0; j < n; j++)
      x[i] = x[i] + beta * A[j * lda + i] * y[j];
  for (int64_t i = 0; i < n; i++)
    x[i] = x[i] + z[i];
  for (int64_t i = 0; i < n; i++)
    for (int64_t j = 0; j < n; j++)
      w[i] = w[i] + alpha * A[i * lda + j] * x[j];
}

/* linear-algebra/blas/symm/symm.c:108-117
 *   for i for j { temp2 = 0;
 *                 for k<i { C[k][j] += alpha*B[i][j] * A[i][k]; temp2 += B[k][j] * A[i][k]; }
 *                 C[i][j] = beta*C[i][j] + alpha*B[i][j]*A[i][i] + alpha*temp2; }
 * Only the lower triangle of A (diagonal included) is read. */
void FN(pbo_symm)(int64_t m, int64_t n, T alpha, T beta, T *C, int64_t ldc, const T *A,
                  int64_t lda, const T *B, int64_t ldb)
{
  for (int64_t i = 0; i < m; i++)
    for (int64_t j = 0; j < n; j++) {
      T temp2 = (T)0;
      for (int64_t k = 0; k < i; k++) {
        C[k * ldc + j] += alpha * B[i * ldb + j] * A[i * lda + k];
        temp2 += B[k * ldb + j] * A[i * lda + k];
      }
      C[i * ldc + j] = beta * C[i * ldc + j] + alpha * B[i * ldb + j] * A[i * lda + i] + alpha * temp2;
    }
}

/* linear-algebra/blas/trmm/trmm.c:101-106
 *   for i for j { for k>i B[i][j] += A[k][i] * B[k][j];  B[i][j] = alpha * B[i][j]; }
 * Only the strict lower triangle of A is read (unit diagonal). */
void FN(pbo_trmm)(int64_t m, int64_t n, T alpha, const T *A, int64_t lda, T *B, int64_t ldb)
{
  for (int64_t i = 0; i < m; i++)
    for (int64_t j = 0; j < n; j++) {
      for (int64_t k = i + 1; k < m; k++)
        B[i * ldb + j] += A[k * lda + i] * B[k * ldb + j];
      B[i * ldb + j] = alpha * B[i * ldb + j];
    }
}

/* linear-algebra/kernels/doitgen/doitgen.c:88-97, with (r,q) flattened to one
 * row index (A is nr*nq rows of np entries, contiguous in the source):
 *   for row { for p { sum[p] = 0; for s sum[p] += A[row][s] * C4[s][p]; }
 *             for p A[row][p] = sum[p]; } */
void FN(pbo_doitgen)(int64_t rows, int64_t np, T *A, int64_t lda, const T *C4, int64_t ldc4,
                     T *sum)
{
  for (int64_t r = 0; r < rows; r++) {
    for (int64_t p = 0; p < np; p++) {
      sum[p] = (T)0.0;
      for (int64_t s = 0; s < np; s++)
        sum[p] += A[r * lda + s] * C4[s * ldc4 + p];
    }
    for (int64_t p = 0; p < np; p++)
      A[r * lda + p] = sum[p];
  }
}

/* Same statements as pbo_gemm, but with a double accumulator per output and
 * the fp32 inputs promoted: the "truth" that fp32 results are also gated on
 * (the sequential fp32 sum itself drifts from it as K grows). */
void FN(pbo_gemm_acc64)(int64_t ni, int64_t nj, int64_t nk, T alpha, T beta,
                        double *Cout, int64_t ldo, const T *C, int64_t ldc,
                        const T *A, int64_t lda, const T *B, int64_t ldb)
{
  for (int64_t i = 0; i < ni; i++) {
    for (int64_t j = 0; j < nj; j++)
      Cout[i * ldo + j] = (double)beta * (double)C[i * ldc + j];
    for (int64_t k = 0; k < nk; k++) {
      const double a = (double)alpha * (double)A[i * lda + k];
      for (int64_t j = 0; j < nj; j++)
        Cout[i * ldo + j] += a * (double)B[k * ldb + j];
    }
  }
}

void FN(pbo_syrk_range_acc64)(int64_t row0, int64_t row1, int64_t m, T alpha,
                              T beta, double *Cout, int64_t ldo, const T *C,
                              int64_t ldc, const T *A, int64_t lda)
{
  for (int64_t i = row0; i < row1; i++) {
    for (int64_t j = 0; j <= i; j++)
      Cout[i * ldo + j] = (double)beta * (double)C[i * ldc + j];
    for (int64_t k = 0; k < m; k++) {
      const double a = (double)alpha * (double)A[i * lda + k];
      for (int64_t j = 0; j <= i; j++)
        Cout[i * ldo + j] += a * (double)A[j * lda + k];
    }
  }
}

#undef FN
#undef CAT
#undef CAT_
