// RUN: cgeist %s --function=run_gemm -S | FileCheck %s

// Opting one function into libpgb200 without the matcher pass: the pragma
// that tools/cgeist/Test/Verification/lower_to.c:1-10 pins for single ops,
// with a "func.call @<symbol>" target, redirects every call of kernel_gemm
// to the library's host-array drop-in of the same signature
// (include/pgb200.h: pgb200_kernel_gemm <- kernel_gemm gemm.c:88-115).
#define NI 1000
#define NJ 1100
#define NK 1200

#pragma lower_to(kernel_gemm, "func.call @pgb200_kernel_gemm")
extern void kernel_gemm(int ni, int nj, int nk, double alpha, double beta,
                        double C[NI][NJ], double A[NI][NK], double B[NK][NJ]);

void run_gemm(double alpha, double beta, double C[NI][NJ], double A[NI][NK],
              double B[NK][NJ]) {
  kernel_gemm(NI, NJ, NK, alpha, beta, C, A, B);
}

// CHECK:       func @run_gemm(%[[ALPHA:.+]]: f64, %[[BETA:.+]]: f64, %[[C:.+]]: memref<?x1100xf64>, %[[A:.+]]: memref<?x1200xf64>, %[[B:.+]]: memref<?x1100xf64>)
// CHECK-DAG:     %[[NI:.+]] = arith.constant 1000 : i32
// CHECK-DAG:     %[[NJ:.+]] = arith.constant 1100 : i32
// CHECK-DAG:     %[[NK:.+]] = arith.constant 1200 : i32
// CHECK:         call @pgb200_kernel_gemm(%[[NI]], %[[NJ]], %[[NK]], %[[ALPHA]], %[[BETA]], %[[C]], %[[A]], %[[B]]) : (i32, i32, i32, f64, f64, memref<?x1100xf64>, memref<?x1200xf64>, memref<?x1100xf64>) -> ()
// CHECK-NEXT:    return
// CHECK:       func private @pgb200_kernel_gemm(i32, i32, i32, f64, f64, memref<?x1100xf64>, memref<?x1200xf64>, memref<?x1100xf64>)
// CHECK-NOT:   @kernel_gemm
