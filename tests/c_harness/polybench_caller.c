/* A plain C99 caller of libpgb200, written the way a PolyBench source would
 * opt in by hand: malloc'd row-major arrays, the reference's init formulas
 * (gemm.c:42-63, mvt.c:39-58, MINI-like extents scaled up), the drop-in call in
 * place of the scop, and the original loop nest beside it as the check.
 *
 *   polybench_caller            : link/ABI check only (no device needed)
 *   polybench_caller --compute  : runs the drop-ins on the GPU and compares
 *
 * TEST CODE: the loop nests below are the checker, not a product path. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "pgb200.h"

static int check_gemm(int ni, int nj, int nk)
{
  double alpha = 1.5, beta = 1.2;
  double *A = malloc(sizeof(double) * ni * nk), *B = malloc(sizeof(double) * nk * nj);
  double *C = malloc(sizeof(double) * ni * nj), *R = malloc(sizeof(double) * ni * nj);
  int i, j, k;
  for (i = 0; i < ni; i++)
    for (j = 0; j < nj; j++)
      R[i * nj + j] = C[i * nj + j] = (double)((i * j + 1) % ni) / ni;
  for (i = 0; i < ni; i++)
    for (j = 0; j < nk; j++)
      A[i * nk + j] = (double)(i * (j + 1) % nk) / nk;
  for (i = 0; i < nk; i++)
    for (j = 0; j < nj; j++)
      B[i * nj + j] = (double)(i * (j + 2) % nj) / nj;

  int32_t st = pgb200_kernel_gemm(ni, nj, nk, alpha, beta, C, A, B);
  if (st != PGB200_OK) {
    fprintf(stderr, "pgb200_kernel_gemm: %d %s\n", (int)st, pgb200GetLastErrorString());
    return 1;
  }
  for (i = 0; i < ni; i++) {
    for (j = 0; j < nj; j++)
      R[i * nj + j] *= beta;
    for (k = 0; k < nk; k++)
      for (j = 0; j < nj; j++)
        R[i * nj + j] += alpha * A[i * nk + k] * B[k * nj + j];
  }
  double worst = 0.0, scale = 0.0;
  for (i = 0; i < ni * nj; i++) {
    worst = fmax(worst, fabs(C[i] - R[i]));
    scale = fmax(scale, fabs(R[i]));
  }
  printf("gemm %dx%dx%d max |diff| / max |ref| = %.3e\n", ni, nj, nk, worst / scale);
  free(A); free(B); free(C); free(R);
  return !(worst <= 1e-12 * scale);
}

static int check_mvt(int n)
{
  double *A = malloc(sizeof(double) * n * n);
  double *x1 = malloc(sizeof(double) * n), *x2 = malloc(sizeof(double) * n);
  double *y1 = malloc(sizeof(double) * n), *y2 = malloc(sizeof(double) * n);
  double *r1 = malloc(sizeof(double) * n), *r2 = malloc(sizeof(double) * n);
  int i, j;
  for (i = 0; i < n; i++) {
    r1[i] = x1[i] = (double)(i % n) / n;
    r2[i] = x2[i] = (double)((i + 1) % n) / n;
    y1[i] = (double)((i + 3) % n) / n;
    y2[i] = (double)((i + 4) % n) / n;
    for (j = 0; j < n; j++)
      A[i * n + j] = (double)(i * j % n) / n;
  }
  int32_t st = pgb200_kernel_mvt(n, x1, x2, y1, y2, A);
  if (st != PGB200_OK) {
    fprintf(stderr, "pgb200_kernel_mvt: %d %s\n", (int)st, pgb200GetLastErrorString());
    return 1;
  }
  for (i = 0; i < n; i++)
    for (j = 0; j < n; j++)
      r1[i] = r1[i] + A[i * n + j] * y1[j];
  for (i = 0; i < n; i++)
    for (j = 0; j < n; j++)
      r2[i] = r2[i] + A[j * n + i] * y2[j];
  double worst = 0.0, scale = 0.0;
  for (i = 0; i < n; i++) {
    worst = fmax(worst, fmax(fabs(x1[i] - r1[i]), fabs(x2[i] - r2[i])));
    scale = fmax(scale, fmax(fabs(r1[i]), fabs(r2[i])));
  }
  printf("mvt %d max |diff| / max |ref| = %.3e\n", n, worst / scale);
  free(A); free(x1); free(x2); free(y1); free(y2); free(r1); free(r2);
  return !(worst <= 1e-12 * scale);
}

int main(int argc, char **argv)
{
  printf("libpgb200 version %d\n", (int)pgb200Version());
  if (argc < 2 || strcmp(argv[1], "--compute") != 0)
    return 0;
  int bad = 0;
  bad |= check_gemm(200, 220, 240); /* PolyBench MEDIUM */
  bad |= check_gemm(384, 512, 256); /* aligned: tensor-core path */
  bad |= check_mvt(400);            /* PolyBench MEDIUM */
  if (pgb200LastPath() == 0) {
    fprintf(stderr, "no kernel ran\n");
    bad = 1;
  }
  pgb200Shutdown();
  puts(bad ? "FAILED" : "OK");
  return bad;
}
