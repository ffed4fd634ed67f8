// RUN: cgeist %s --function=gemm_nest --raise-scf-to-affine --raise-affine-to-pgb200 -S | FileCheck %s
// RUN: cgeist %s --function=gemm_nest --raise-scf-to-affine -S | FileCheck %s --check-prefix=PLAIN

// A GEMM loop nest in the statement order of PolyBench's kernel_gemm
// (tools/cgeist/Test/polybench/linear-algebra/blas/gemm/gemm.c:104-113): with
// the flag the whole nest becomes one call into libpgb200, without it the
// affine nest is what comes out today.
#define NJ 1100
#define NK 1200

void gemm_nest(int ni, int nj, int nk, double alpha, double beta,
               double C[][NJ], double A[][NK], double B[][NJ]) {
  for (int i = 0; i < ni; i++) {
    for (int j = 0; j < nj; j++)
      C[i][j] *= beta;
    for (int k = 0; k < nk; k++)
      for (int j = 0; j < nj; j++)
        C[i][j] += alpha * A[i][k] * B[k][j];
  }
}

// CHECK:       func.func private @pgb200Dgemm(!llvm.ptr, i64, i64, i64, f64, !llvm.ptr, i64, !llvm.ptr, i64, f64, !llvm.ptr, i64) -> i32
// CHECK:       func @gemm_nest(%[[NI:.+]]: i32, %[[NJ:.+]]: i32, %[[NK:.+]]: i32, %[[ALPHA:.+]]: f64, %[[BETA:.+]]: f64, %[[C:.+]]: memref<?x1100xf64>, %[[A:.+]]: memref<?x1200xf64>, %[[B:.+]]: memref<?x1100xf64>)
// CHECK-NOT:     affine.for
// CHECK:         call @pgb200Dgemm(%{{.*}}, %{{.*}}, %{{.*}}, %{{.*}}, %[[ALPHA]], %{{.*}}, %{{.*}}, %{{.*}}, %{{.*}}, %[[BETA]], %{{.*}}, %{{.*}})
// CHECK-NEXT:    return

// PLAIN:       func @gemm_nest(
// PLAIN:         affine.for
// PLAIN-NOT:     pgb200
