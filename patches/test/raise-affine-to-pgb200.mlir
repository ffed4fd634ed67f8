// RUN: polygeist-opt --raise-affine-to-pgb200 --split-input-file %s | FileCheck %s

// The affine form of kernel_gemm that
// tools/cgeist/Test/polybench/linear-algebra/blas/gemm/gemm.c:164-189 pins:
// for i { for j: C *= beta;  for k: for j: C += (alpha * A[i][k]) * B[k][j] }.
module {
  func.func @kernel_gemm(%arg0: i32, %arg1: i32, %arg2: i32, %arg3: f64, %arg4: f64, %arg5: memref<?x1100xf64>, %arg6: memref<?x1200xf64>, %arg7: memref<?x1100xf64>) {
    %0 = arith.index_cast %arg0 : i32 to index
    %1 = arith.index_cast %arg1 : i32 to index
    %2 = arith.index_cast %arg2 : i32 to index
    affine.for %arg8 = 0 to %0 {
      affine.for %arg9 = 0 to %1 {
        %3 = affine.load %arg5[%arg8, %arg9] : memref<?x1100xf64>
        %4 = arith.mulf %3, %arg4 : f64
        affine.store %4, %arg5[%arg8, %arg9] : memref<?x1100xf64>
      }
      affine.for %arg9 = 0 to %2 {
        affine.for %arg10 = 0 to %1 {
          %3 = affine.load %arg6[%arg8, %arg9] : memref<?x1200xf64>
          %4 = arith.mulf %arg3, %3 : f64
          %5 = affine.load %arg7[%arg9, %arg10] : memref<?x1100xf64>
          %6 = arith.mulf %4, %5 : f64
          %7 = affine.load %arg5[%arg8, %arg10] : memref<?x1100xf64>
          %8 = arith.addf %7, %6 : f64
          affine.store %8, %arg5[%arg8, %arg10] : memref<?x1100xf64>
        }
      }
    }
    return
  }
}

// CHECK:       func.func private @pgb200Dgemm(!llvm.ptr, i64, i64, i64, f64, !llvm.ptr, i64, !llvm.ptr, i64, f64, !llvm.ptr, i64) -> i32
// CHECK-LABEL: func.func @kernel_gemm(
// CHECK-SAME:    %[[NI:.+]]: i32, %[[NJ:.+]]: i32, %[[NK:.+]]: i32, %[[ALPHA:.+]]: f64, %[[BETA:.+]]: f64, %[[C:.+]]: memref<?x1100xf64>, %[[A:.+]]: memref<?x1200xf64>, %[[B:.+]]: memref<?x1100xf64>)
// CHECK-DAG:     %[[M:.+]] = arith.index_cast %[[NI]] : i32 to index
// CHECK-DAG:     %[[N:.+]] = arith.index_cast %[[NJ]] : i32 to index
// CHECK-DAG:     %[[K:.+]] = arith.index_cast %[[NK]] : i32 to index
// CHECK-NOT:     affine.for
// CHECK:         %[[STREAM:.+]] = llvm.mlir.zero : !llvm.ptr
// CHECK-DAG:     %[[M64:.+]] = arith.index_cast %[[M]] : index to i64
// CHECK-DAG:     %[[N64:.+]] = arith.index_cast %[[N]] : index to i64
// CHECK-DAG:     %[[K64:.+]] = arith.index_cast %[[K]] : index to i64
// CHECK-DAG:     %[[PA:.+]] = "polygeist.memref2pointer"(%[[A]]) : (memref<?x1200xf64>) -> !llvm.ptr
// CHECK-DAG:     %[[PB:.+]] = "polygeist.memref2pointer"(%[[B]]) : (memref<?x1100xf64>) -> !llvm.ptr
// CHECK-DAG:     %[[PC:.+]] = "polygeist.memref2pointer"(%[[C]]) : (memref<?x1100xf64>) -> !llvm.ptr
// CHECK-DAG:     %[[LDA:.+]] = arith.constant 1200 : i64
// CHECK-DAG:     %[[LDBC:.+]] = arith.constant 1100 : i64
// CHECK:         call @pgb200Dgemm(%[[STREAM]], %[[M64]], %[[N64]], %[[K64]], %[[ALPHA]], %[[PA]], %[[LDA]], %[[PB]], %{{.*}}, %[[BETA]], %[[PC]], %{{.*}}) : (!llvm.ptr, i64, i64, i64, f64, !llvm.ptr, i64, !llvm.ptr, i64, f64, !llvm.ptr, i64) -> i32
// CHECK-NOT:     affine.for
// CHECK:         return

// -----

// The two nests of kernel_2mm as
// tools/cgeist/Test/polybench/linear-algebra/kernels/2mm/2mm.c:177-200 pins them:
// tmp = alpha*A*B written as i-j-k with a zero store, then D = tmp*C + beta*D.
module {
  func.func @kernel_2mm(%arg0: i32, %arg1: i32, %arg2: i32, %arg3: i32, %arg4: f64, %arg5: f64, %arg6: memref<?x900xf64>, %arg7: memref<?x1100xf64>, %arg8: memref<?x900xf64>, %arg9: memref<?x1200xf64>, %arg10: memref<?x1200xf64>) {
    %cst = arith.constant 0.000000e+00 : f64
    %0 = arith.index_cast %arg0 : i32 to index
    %1 = arith.index_cast %arg1 : i32 to index
    %2 = arith.index_cast %arg2 : i32 to index
    %3 = arith.index_cast %arg3 : i32 to index
    affine.for %arg11 = 0 to %0 {
      affine.for %arg12 = 0 to %1 {
        affine.store %cst, %arg6[%arg11, %arg12] : memref<?x900xf64>
        affine.for %arg13 = 0 to %2 {
          %4 = affine.load %arg7[%arg11, %arg13] : memref<?x1100xf64>
          %5 = arith.mulf %arg4, %4 : f64
          %6 = affine.load %arg8[%arg13, %arg12] : memref<?x900xf64>
          %7 = arith.mulf %5, %6 : f64
          %8 = affine.load %arg6[%arg11, %arg12] : memref<?x900xf64>
          %9 = arith.addf %8, %7 : f64
          affine.store %9, %arg6[%arg11, %arg12] : memref<?x900xf64>
        }
      }
    }
    affine.for %arg11 = 0 to %0 {
      affine.for %arg12 = 0 to %3 {
        %4 = affine.load %arg10[%arg11, %arg12] : memref<?x1200xf64>
        %5 = arith.mulf %4, %arg5 : f64
        affine.store %5, %arg10[%arg11, %arg12] : memref<?x1200xf64>
        affine.for %arg13 = 0 to %1 {
          %6 = affine.load %arg6[%arg11, %arg13] : memref<?x900xf64>
          %7 = affine.load %arg9[%arg13, %arg12] : memref<?x1200xf64>
          %8 = arith.mulf %6, %7 : f64
          %9 = affine.load %arg10[%arg11, %arg12] : memref<?x1200xf64>
          %10 = arith.addf %9, %8 : f64
          affine.store %10, %arg10[%arg11, %arg12] : memref<?x1200xf64>
        }
      }
    }
    return
  }
}

// CHECK-LABEL: func.func @kernel_2mm(
// CHECK-SAME:    %{{.*}}: i32, %{{.*}}: i32, %{{.*}}: i32, %{{.*}}: i32, %[[ALPHA:.+]]: f64, %[[BETA:.+]]: f64, %[[TMP:.+]]: memref<?x900xf64>, %[[A:.+]]: memref<?x1100xf64>, %[[B:.+]]: memref<?x900xf64>, %[[C:.+]]: memref<?x1200xf64>, %[[D:.+]]: memref<?x1200xf64>)
// CHECK-NOT:     affine.for
// tmp = alpha*A*B + 0*tmp
// CHECK:         %[[ZERO:.+]] = arith.constant 0.000000e+00 : f64
// CHECK:         %[[PTMP1:.+]] = "polygeist.memref2pointer"(%[[TMP]])
// CHECK:         call @pgb200Dgemm(%{{.*}}, %{{.*}}, %{{.*}}, %{{.*}}, %[[ALPHA]], %{{.*}}, %{{.*}}, %{{.*}}, %{{.*}}, %{{.*}}, %[[PTMP1]], %{{.*}})
// D = 1*tmp*C + beta*D
// CHECK:         %[[ONE:.+]] = arith.constant 1.000000e+00 : f64
// CHECK:         %[[PD:.+]] = "polygeist.memref2pointer"(%[[D]])
// CHECK:         call @pgb200Dgemm(%{{.*}}, %{{.*}}, %{{.*}}, %{{.*}}, %[[ONE]], %{{.*}}, %{{.*}}, %{{.*}}, %{{.*}}, %[[BETA]], %[[PD]], %{{.*}})
// CHECK-NOT:     affine.for
// CHECK:         return

// -----

// fp32 `C += A*B` (the matmul nest of tools/cgeist/Test/Verification/raiseToAffine.c:12-27)
// and a mat-vec nest with a zero store.  A nest that is not a contraction stays.
module {
  func.func @matmul_f32(%A: memref<?x400xf32>, %B: memref<?x300xf32>, %C: memref<?x300xf32>) {
    affine.for %i = 0 to 200 {
      affine.for %j = 0 to 300 {
        affine.for %k = 0 to 400 {
          %a = affine.load %A[%i, %k] : memref<?x400xf32>
          %b = affine.load %B[%k, %j] : memref<?x300xf32>
          %p = arith.mulf %a, %b : f32
          %c = affine.load %C[%i, %j] : memref<?x300xf32>
          %s = arith.addf %c, %p : f32
          affine.store %s, %C[%i, %j] : memref<?x300xf32>
        }
      }
    }
    return
  }
  func.func @matvec(%n: index, %A: memref<?x28xf64>, %x: memref<?xf64>, %y: memref<?xf64>) {
    %cst = arith.constant 0.000000e+00 : f64
    affine.for %i = 0 to %n {
      affine.store %cst, %y[%i] : memref<?xf64>
      affine.for %j = 0 to %n {
        %a = affine.load %A[%i, %j] : memref<?x28xf64>
        %b = affine.load %x[%j] : memref<?xf64>
        %p = arith.mulf %a, %b : f64
        %c = affine.load %y[%i] : memref<?xf64>
        %s = arith.addf %p, %c : f64
        affine.store %s, %y[%i] : memref<?xf64>
      }
    }
    return
  }
  func.func @not_a_contraction(%A: memref<?x64xf64>, %B: memref<?x64xf64>) {
    affine.for %i = 0 to 64 {
      affine.for %j = 0 to 64 {
        %a = affine.load %A[%i, %j] : memref<?x64xf64>
        %b = arith.addf %a, %a : f64
        affine.store %b, %B[%j, %i] : memref<?x64xf64>
      }
    }
    return
  }
}

// CHECK-LABEL: func.func @matmul_f32(
// CHECK-NOT:     affine.for
// CHECK-DAG:     %[[M:.+]] = arith.constant 200 : index
// CHECK-DAG:     %[[N:.+]] = arith.constant 300 : index
// CHECK-DAG:     %[[K:.+]] = arith.constant 400 : index
// CHECK:         call @pgb200Sgemm(
// CHECK-SAME:      -> i32
// CHECK-LABEL: func.func @matvec(
// CHECK-NOT:     affine.for
// CHECK:         %[[NOTRANS:.+]] = arith.constant 0 : i32
// CHECK:         call @pgb200Dgemv(%{{.*}}, %[[NOTRANS]],
// CHECK-LABEL: func.func @not_a_contraction(
// CHECK:         affine.for
// CHECK:           affine.for
// CHECK-NOT:     call @pgb200

// -----

// The two nests of kernel_mvt
// (tools/cgeist/Test/polybench/linear-algebra/kernels/mvt/mvt.c:102-109): both
// accumulate into their result (no zero store -> beta = 1); the second walks A
// by columns (A[j][i] -> transA = 1).
module {
  func.func @kernel_mvt(%arg0: i32, %arg1: memref<?xf64>, %arg2: memref<?xf64>, %arg3: memref<?xf64>, %arg4: memref<?xf64>, %arg5: memref<?x2000xf64>) {
    %0 = arith.index_cast %arg0 : i32 to index
    affine.for %arg6 = 0 to %0 {
      affine.for %arg7 = 0 to %0 {
        %1 = affine.load %arg1[%arg6] : memref<?xf64>
        %2 = affine.load %arg5[%arg6, %arg7] : memref<?x2000xf64>
        %3 = affine.load %arg3[%arg7] : memref<?xf64>
        %4 = arith.mulf %2, %3 : f64
        %5 = arith.addf %1, %4 : f64
        affine.store %5, %arg1[%arg6] : memref<?xf64>
      }
    }
    affine.for %arg6 = 0 to %0 {
      affine.for %arg7 = 0 to %0 {
        %1 = affine.load %arg2[%arg6] : memref<?xf64>
        %2 = affine.load %arg5[%arg7, %arg6] : memref<?x2000xf64>
        %3 = affine.load %arg4[%arg7] : memref<?xf64>
        %4 = arith.mulf %2, %3 : f64
        %5 = arith.addf %1, %4 : f64
        affine.store %5, %arg2[%arg6] : memref<?xf64>
      }
    }
    return
  }
}

// CHECK-LABEL: func.func @kernel_mvt(
// CHECK-SAME:    %{{.*}}: i32, %[[X1:.+]]: memref<?xf64>, %[[X2:.+]]: memref<?xf64>, %[[Y1:.+]]: memref<?xf64>, %[[Y2:.+]]: memref<?xf64>, %[[A:.+]]: memref<?x2000xf64>)
// CHECK-NOT:     affine.for
// CHECK:         %[[NOTRANS:.+]] = arith.constant 0 : i32
// CHECK-DAG:     %[[PY1:.+]] = "polygeist.memref2pointer"(%[[Y1]])
// CHECK-DAG:     %[[PX1:.+]] = "polygeist.memref2pointer"(%[[X1]])
// CHECK:         call @pgb200Dgemv(%{{.*}}, %[[NOTRANS]], %{{.*}}, %{{.*}}, %{{.*}}, %{{.*}}, %{{.*}}, %[[PY1]], %{{.*}}, %[[PX1]])
// CHECK-NOT:     affine.for
// CHECK:         %[[TRANS:.+]] = arith.constant 1 : i32
// CHECK-DAG:     %[[PY2:.+]] = "polygeist.memref2pointer"(%[[Y2]])
// CHECK-DAG:     %[[PX2:.+]] = "polygeist.memref2pointer"(%[[X2]])
// CHECK:         call @pgb200Dgemv(%{{.*}}, %[[TRANS]], %{{.*}}, %{{.*}}, %{{.*}}, %{{.*}}, %{{.*}}, %[[PY2]], %{{.*}}, %[[PX2]])
// CHECK-NOT:     affine.for
// CHECK:         return

// -----

// kernel_syrk (tools/cgeist/Test/polybench/linear-algebra/blas/syrk/syrk.c:97-106):
// both inner loops run to j <= i, i.e. to #map(%i) with #map = (d0) -> (d0 + 1).
// A nest with the same triangular bound that multiplies two different arrays
// (the update of trmm / a triangular gemm) is not a rank-k update and stays.
#map = affine_map<(d0) -> (d0 + 1)>
module {
  func.func @kernel_syrk(%arg0: i32, %arg1: i32, %arg2: f64, %arg3: f64, %arg4: memref<?x1200xf64>, %arg5: memref<?x1000xf64>) {
    %0 = arith.index_cast %arg0 : i32 to index
    %1 = arith.index_cast %arg1 : i32 to index
    affine.for %arg6 = 0 to %0 {
      affine.for %arg7 = 0 to #map(%arg6) {
        %2 = affine.load %arg4[%arg6, %arg7] : memref<?x1200xf64>
        %3 = arith.mulf %2, %arg3 : f64
        affine.store %3, %arg4[%arg6, %arg7] : memref<?x1200xf64>
      }
      affine.for %arg7 = 0 to %1 {
        affine.for %arg8 = 0 to #map(%arg6) {
          %2 = affine.load %arg5[%arg6, %arg7] : memref<?x1000xf64>
          %3 = arith.mulf %arg2, %2 : f64
          %4 = affine.load %arg5[%arg8, %arg7] : memref<?x1000xf64>
          %5 = arith.mulf %3, %4 : f64
          %6 = affine.load %arg4[%arg6, %arg8] : memref<?x1200xf64>
          %7 = arith.addf %6, %5 : f64
          affine.store %7, %arg4[%arg6, %arg8] : memref<?x1200xf64>
        }
      }
    }
    return
  }
  func.func @triangular_product(%n: index, %beta: f64, %C: memref<?x64xf64>, %A: memref<?x64xf64>, %B: memref<?x64xf64>) {
    affine.for %i = 0 to %n {
      affine.for %j = 0 to #map(%i) {
        %2 = affine.load %C[%i, %j] : memref<?x64xf64>
        %3 = arith.mulf %2, %beta : f64
        affine.store %3, %C[%i, %j] : memref<?x64xf64>
      }
      affine.for %k = 0 to %n {
        affine.for %j = 0 to #map(%i) {
          %2 = affine.load %A[%i, %k] : memref<?x64xf64>
          %4 = affine.load %B[%k, %j] : memref<?x64xf64>
          %5 = arith.mulf %2, %4 : f64
          %6 = affine.load %C[%i, %j] : memref<?x64xf64>
          %7 = arith.addf %6, %5 : f64
          affine.store %7, %C[%i, %j] : memref<?x64xf64>
        }
      }
    }
    return
  }
}

// CHECK:       func.func private @pgb200Dsyrk(!llvm.ptr, i64, i64, f64, !llvm.ptr, i64, f64, !llvm.ptr, i64) -> i32
// CHECK-LABEL: func.func @kernel_syrk(
// CHECK-SAME:    %[[NN:.+]]: i32, %[[NM:.+]]: i32, %[[ALPHA:.+]]: f64, %[[BETA:.+]]: f64, %[[C:.+]]: memref<?x1200xf64>, %[[A:.+]]: memref<?x1000xf64>)
// CHECK-DAG:     %[[N:.+]] = arith.index_cast %[[NN]] : i32 to index
// CHECK-DAG:     %[[K:.+]] = arith.index_cast %[[NM]] : i32 to index
// CHECK-NOT:     affine.for
// CHECK:         %[[STREAM:.+]] = llvm.mlir.zero : !llvm.ptr
// CHECK-DAG:     %[[N64:.+]] = arith.index_cast %[[N]] : index to i64
// CHECK-DAG:     %[[K64:.+]] = arith.index_cast %[[K]] : index to i64
// CHECK-DAG:     %[[PA:.+]] = "polygeist.memref2pointer"(%[[A]]) : (memref<?x1000xf64>) -> !llvm.ptr
// CHECK-DAG:     %[[PC:.+]] = "polygeist.memref2pointer"(%[[C]]) : (memref<?x1200xf64>) -> !llvm.ptr
// CHECK-DAG:     %[[LDA:.+]] = arith.constant 1000 : i64
// CHECK-DAG:     %[[LDC:.+]] = arith.constant 1200 : i64
// CHECK:         call @pgb200Dsyrk(%[[STREAM]], %[[N64]], %[[K64]], %[[ALPHA]], %[[PA]], %[[LDA]], %[[BETA]], %[[PC]], %[[LDC]]) : (!llvm.ptr, i64, i64, f64, !llvm.ptr, i64, f64, !llvm.ptr, i64) -> i32
// CHECK-NOT:     affine.for
// CHECK:         return
// CHECK-LABEL: func.func @triangular_product(
// CHECK:         affine.for
// CHECK:           affine.for
// CHECK-NOT:     call @pgb200

// -----

// kernel_syr2k as tools/cgeist/Test/polybench/linear-algebra/blas/syr2k/syr2k.c:162-190
// pins it: two products in one statement, the factors that do not depend on j
// (B[i][k], A[i][k]) already hoisted into the k loop's body.  kernel_syrk in the
// same hoisted form (syrk.c:147-170: alpha * A[i][k] computed in the k body).
#map = affine_map<(d0) -> (d0 + 1)>
module {
  func.func @kernel_syr2k(%arg0: i32, %arg1: i32, %arg2: f64, %arg3: f64, %arg4: memref<?x1200xf64>, %arg5: memref<?x1000xf64>, %arg6: memref<?x1000xf64>) {
    %0 = arith.index_cast %arg0 : i32 to index
    %1 = arith.index_cast %arg1 : i32 to index
    affine.for %arg7 = 0 to %0 {
      affine.for %arg8 = 0 to #map(%arg7) {
        %2 = affine.load %arg4[%arg7, %arg8] : memref<?x1200xf64>
        %3 = arith.mulf %2, %arg3 : f64
        affine.store %3, %arg4[%arg7, %arg8] : memref<?x1200xf64>
      }
      affine.for %arg8 = 0 to %1 {
        %2 = affine.load %arg6[%arg7, %arg8] : memref<?x1000xf64>
        %3 = affine.load %arg5[%arg7, %arg8] : memref<?x1000xf64>
        affine.for %arg9 = 0 to #map(%arg7) {
          %4 = affine.load %arg5[%arg9, %arg8] : memref<?x1000xf64>
          %5 = arith.mulf %4, %arg2 : f64
          %6 = arith.mulf %5, %2 : f64
          %7 = affine.load %arg6[%arg9, %arg8] : memref<?x1000xf64>
          %8 = arith.mulf %7, %arg2 : f64
          %9 = arith.mulf %8, %3 : f64
          %10 = arith.addf %6, %9 : f64
          %11 = affine.load %arg4[%arg7, %arg9] : memref<?x1200xf64>
          %12 = arith.addf %11, %10 : f64
          affine.store %12, %arg4[%arg7, %arg9] : memref<?x1200xf64>
        }
      }
    }
    return
  }
  func.func @kernel_syrk_hoisted(%arg0: i32, %arg1: i32, %arg2: f64, %arg3: f64, %arg4: memref<?x1200xf64>, %arg5: memref<?x1000xf64>) {
    %0 = arith.index_cast %arg0 : i32 to index
    %1 = arith.index_cast %arg1 : i32 to index
    affine.for %arg6 = 0 to %0 {
      affine.for %arg7 = 0 to #map(%arg6) {
        %2 = affine.load %arg4[%arg6, %arg7] : memref<?x1200xf64>
        %3 = arith.mulf %2, %arg3 : f64
        affine.store %3, %arg4[%arg6, %arg7] : memref<?x1200xf64>
      }
      affine.for %arg7 = 0 to %1 {
        %2 = affine.load %arg5[%arg6, %arg7] : memref<?x1000xf64>
        %3 = arith.mulf %arg2, %2 : f64
        affine.for %arg8 = 0 to #map(%arg6) {
          %4 = affine.load %arg5[%arg8, %arg7] : memref<?x1000xf64>
          %5 = arith.mulf %3, %4 : f64
          %6 = affine.load %arg4[%arg6, %arg8] : memref<?x1200xf64>
          %7 = arith.addf %6, %5 : f64
          affine.store %7, %arg4[%arg6, %arg8] : memref<?x1200xf64>
        }
      }
    }
    return
  }
}

// CHECK:       func.func private @pgb200Dsyr2k(!llvm.ptr, i64, i64, f64, !llvm.ptr, i64, !llvm.ptr, i64, f64, !llvm.ptr, i64) -> i32
// CHECK-LABEL: func.func @kernel_syr2k(
// CHECK-SAME:    %[[NN:.+]]: i32, %[[NM:.+]]: i32, %[[ALPHA:.+]]: f64, %[[BETA:.+]]: f64, %[[C:.+]]: memref<?x1200xf64>, %[[A:.+]]: memref<?x1000xf64>, %[[B:.+]]: memref<?x1000xf64>)
// CHECK-NOT:     affine.for
// CHECK:         %[[STREAM:.+]] = llvm.mlir.zero : !llvm.ptr
// CHECK-DAG:     %[[PA:.+]] = "polygeist.memref2pointer"(%[[A]]) : (memref<?x1000xf64>) -> !llvm.ptr
// CHECK-DAG:     %[[PB:.+]] = "polygeist.memref2pointer"(%[[B]]) : (memref<?x1000xf64>) -> !llvm.ptr
// CHECK-DAG:     %[[PC:.+]] = "polygeist.memref2pointer"(%[[C]]) : (memref<?x1200xf64>) -> !llvm.ptr
// CHECK:         call @pgb200Dsyr2k(%[[STREAM]], %{{.*}}, %{{.*}}, %[[ALPHA]], %[[PA]], %{{.*}}, %[[PB]], %{{.*}}, %[[BETA]], %[[PC]], %{{.*}}) : (!llvm.ptr, i64, i64, f64, !llvm.ptr, i64, !llvm.ptr, i64, f64, !llvm.ptr, i64) -> i32
// CHECK-NOT:     affine.for
// CHECK:         return
// CHECK-LABEL: func.func @kernel_syrk_hoisted(
// CHECK-SAME:    %{{.*}}: i32, %{{.*}}: i32, %[[ALPHA:.+]]: f64, %[[BETA:.+]]: f64, %[[C:.+]]: memref<?x1200xf64>, %[[A:.+]]: memref<?x1000xf64>)
// CHECK-NOT:     affine.for
// CHECK-DAG:     %[[PA:.+]] = "polygeist.memref2pointer"(%[[A]])
// CHECK-DAG:     %[[PC:.+]] = "polygeist.memref2pointer"(%[[C]])
// CHECK:         call @pgb200Dsyrk(%{{.*}}, %{{.*}}, %{{.*}}, %[[ALPHA]], %[[PA]], %{{.*}}, %[[BETA]], %[[PC]], %{{.*}})
// CHECK-NOT:     affine.for
// CHECK:         return
