// Plain SIMT contraction kernels: the any-shape, any-alignment path that the
// tensor-core kernels fall back to (odd leading dimensions, unaligned bases,
// sizes that break a TMA rule).  Still a GPU path - there is no CPU fallback.
//
// 64x64 output tile per CTA, 16x16 threads, 4x4 outputs per thread, K staged
// through shared memory 16 at a time with bounds-checked loads.
#include "pgb200_internal.h"

namespace pgb200 {

template <typename T, bool TRANSB>
__global__ void __launch_bounds__(256)
simt_gemm_kernel(int64_t M, int64_t N, int64_t K, T alpha, const T *__restrict__ A, int64_t lda,
                 const T *__restrict__ B, int64_t ldb, T beta, T *__restrict__ C, int64_t ldc,
                 int lower, int64_t row0, int64_t tiles_n) {
  constexpr int TM = 64, TN = 64, TK = 16;
  __shared__ T As[TK][TM + 4];
  __shared__ T Bs[TK][TN + 4];
  const int64_t tile_m = blockIdx.x / tiles_n, tile_n = blockIdx.x % tiles_n;
  const int64_t m0 = tile_m * TM, n0 = tile_n * TN;
  // A tile wholly above the diagonal has nothing to compute.
  if (lower && n0 > m0 + TM - 1 + row0) return;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = (T)0;

  for (int64_t k0 = 0; k0 < K; k0 += TK) {
    // A tile: 64 rows x 16 k; thread loads 4 elements, k fastest (contiguous).
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int idx = threadIdx.x + e * 256;
      const int r = idx / TK, kk = idx % TK;
      const int64_t gr = m0 + r, gk = k0 + kk;
      As[kk][r] = (gr < M && gk < K) ? A[gr * lda + gk] : (T)0;
    }
    if (TRANSB) {
      // B(k,j) = B[j*ldb + k]: k contiguous.
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int idx = threadIdx.x + e * 256;
        const int c = idx / TK, kk = idx % TK;
        const int64_t gc = n0 + c, gk = k0 + kk;
        Bs[kk][c] = (gc < N && gk < K) ? B[gc * ldb + gk] : (T)0;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int idx = threadIdx.x + e * 256;
        const int kk = idx / TN, c = idx % TN;
        const int64_t gc = n0 + c, gk = k0 + kk;
        Bs[kk][c] = (gc < N && gk < K) ? B[gk * ldb + gc] : (T)0;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk++) {
      T a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int64_t r = m0 + ty * 4 + i;
    if (r >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int64_t c = n0 + tx * 4 + j;
      if (c >= N || (lower && c > r + row0)) continue;
      T v = alpha * acc[i][j];
      if (beta != (T)0) v += beta * C[r * ldc + c];
      C[r * ldc + c] = v;
    }
  }
}

template <typename T>
int32_t simt_gemm(cudaStream_t s, int64_t M, int64_t N, int64_t K, T alpha, const T *A,
                  int64_t lda, const T *B, int64_t ldb, bool transB, T beta, T *C, int64_t ldc,
                  bool lower, int64_t row0) {
  const int64_t tm = (M + 63) / 64, tn = (N + 63) / 64;
  PGB_REQUIRE(tm * tn < (int64_t(1) << 31), "simt_gemm: too many tiles");
  const unsigned grid = (unsigned)(tm * tn);
  if (transB)
    simt_gemm_kernel<T, true><<<grid, 256, 0, s>>>(M, N, K, alpha, A, lda, B, ldb, beta, C, ldc,
                                                    lower ? 1 : 0, row0, tn);
  else
    simt_gemm_kernel<T, false><<<grid, 256, 0, s>>>(M, N, K, alpha, A, lda, B, ldb, beta, C, ldc,
                                                     lower ? 1 : 0, row0, tn);
  note_launch(PATH_SIMT);
  PGB_CUDA(cudaGetLastError());
  return PGB200_OK;
}

template int32_t simt_gemm<double>(cudaStream_t, int64_t, int64_t, int64_t, double, const double *,
                                   int64_t, const double *, int64_t, bool, double, double *,
                                   int64_t, bool, int64_t);
template int32_t simt_gemm<float>(cudaStream_t, int64_t, int64_t, int64_t, float, const float *,
                                  int64_t, const float *, int64_t, bool, float, float *, int64_t,
                                  bool, int64_t);

}  // namespace pgb200
