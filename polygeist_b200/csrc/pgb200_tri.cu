// Contractions with a triangular or symmetric operand (PolyBench symm and trmm)
// and the flattened tensor contraction of doitgen.  Each is brought to the
// dense GEMM kernels by one cheap reshaping pass over the M x M operand:
//
//   symm    C = beta*C + alpha*S*B,  S = the symmetric matrix whose lower
//           triangle is stored in A        (blas/symm/symm.c:108-117)
//   trmm    B = alpha*(I + L^T)*B,   L = the strict lower triangle of A
//                                          (blas/trmm/trmm.c:101-106)
//   doitgen A[r][q][:] = A[r][q][:] * C4   (kernels/doitgen/doitgen.c:88-97)
//
// The reshaping kernels move M*M elements through 32x32 shared-memory tiles so
// that both the read of A and the write of the dense operand are coalesced;
// the 2*M*M*N flops that follow dominate for every N of interest.
#include "pgb200_internal.h"

namespace pgb200 {
namespace {

constexpr int TILE = 32;
constexpr int TROWS = 8;

// S[i][j] = A[max(i,j)][min(i,j)]; the strict upper triangle of A is never read.
template <typename T>
__global__ void symmetrize_lower_kernel(int64_t M, const T *__restrict__ A, int64_t lda,
                                        T *__restrict__ S, int64_t lds) {
  __shared__ T tile[TILE][TILE + 1];
  const int64_t bi = blockIdx.y, bj = blockIdx.x;
  if (bj > bi) return;
  const int tx = threadIdx.x;
  for (int r = threadIdx.y; r < TILE; r += TROWS) {
    const int64_t i = bi * TILE + r, j = bj * TILE + tx;
    T v = (T)0;
    if (i < M && j <= i) {
      v = A[i * lda + j];
      S[i * lds + j] = v;
    }
    tile[r][tx] = v;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < TILE; r += TROWS) {
    const int64_t i = bj * TILE + r, j = bi * TILE + tx;
    if (j < M && j > i) S[i * lds + j] = tile[tx][r];
  }
}

// U[i][k] = A[k][i] for i < k < M, 1 for k == i, 0 elsewhere (k up to Kp, the
// padded inner extent).  Neither the diagonal nor the upper triangle of A is read.
template <typename T>
__global__ void unit_upper_from_lower_kernel(int64_t M, int64_t Kp, const T *__restrict__ A,
                                             int64_t lda, T *__restrict__ U, int64_t ldu) {
  __shared__ T tile[TILE][TILE + 1];
  const int64_t ti = blockIdx.y, tk = blockIdx.x;
  const int tx = threadIdx.x;
  const bool has_data = tk >= ti;
  if (has_data) {
    for (int r = threadIdx.y; r < TILE; r += TROWS) {
      const int64_t k = tk * TILE + r, i = ti * TILE + tx;
      tile[r][tx] = (k < M && i < k) ? A[k * lda + i] : (T)0;
    }
    __syncthreads();
  }
  for (int r = threadIdx.y; r < TILE; r += TROWS) {
    const int64_t i = ti * TILE + r, k = tk * TILE + tx;
    if (i >= M || k >= Kp) continue;
    T v = has_data ? tile[tx][r] : (T)0;
    if (k == i) v = (T)1;
    U[i * ldu + k] = v;
  }
}

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

template <typename T>
int32_t symm_device(cudaStream_t s, int64_t M, int64_t N, T alpha, const T *A, int64_t lda,
                    const T *B, int64_t ldb, T beta, T *C, int64_t ldc) {
  const int64_t lds = round_up(M, 4);
  PoolBuffer sbuf;
  PGB_CUDA(sbuf.alloc((size_t)M * lds * sizeof(T), s));
  T *S = sbuf.as<T>();
  const unsigned nt = (unsigned)((M + TILE - 1) / TILE);
  symmetrize_lower_kernel<T><<<dim3(nt, nt), dim3(TILE, TROWS), 0, s>>>(M, A, lda, S, lds);
  PGB_CUDA(cudaGetLastError());
  note_launch(PATH_STREAM);
  return gemm_device<T>(s, M, N, M, alpha, S, lds, B, ldb, false, beta, C, ldc, false, 0);
}

// B = alpha * U * Bold on the tensor-core kernel of the element type, with the
// hint that U is upper triangular.
inline int32_t triangular_product(cudaStream_t s, int64_t M, int64_t N, int64_t K, double alpha,
                                  const double *U, int64_t ldu, const double *Bold, int64_t ldo,
                                  double *B, int64_t ldb) {
  return dmma_gemm(s, M, N, K, alpha, U, ldu, Bold, ldo, false, 0.0, B, ldb, false, true);
}
inline int32_t triangular_product(cudaStream_t s, int64_t M, int64_t N, int64_t K, float alpha,
                                  const float *U, int64_t ldu, const float *Bold, int64_t ldo,
                                  float *B, int64_t ldb) {
  return tf32x3_gemm(s, M, N, K, alpha, U, ldu, Bold, ldo, false, 0.0f, B, ldb, false, 0, true);
}

template <typename T>
int32_t trmm_device(Runtime *rt, cudaStream_t s, int64_t M, int64_t N, T alpha, const T *A,
                    int64_t lda, T *B, int64_t ldb) {
  // The inner extent is padded to a multiple of four (zero columns of U, zero
  // rows of the copy of B) so the tensor-core kernels' K rule always holds.
  const int64_t Kp = round_up(M, 4), ldu = Kp, ldo = round_up(N, 4);
  PoolBuffer ubuf, bbuf;
  PGB_CUDA(ubuf.alloc((size_t)M * ldu * sizeof(T), s));
  PGB_CUDA(bbuf.alloc((size_t)Kp * ldo * sizeof(T), s));
  T *U = ubuf.as<T>(), *Bold = bbuf.as<T>();
  const unsigned nti = (unsigned)((M + TILE - 1) / TILE), ntk = (unsigned)((Kp + TILE - 1) / TILE);
  unit_upper_from_lower_kernel<T><<<dim3(ntk, nti), dim3(TILE, TROWS), 0, s>>>(M, Kp, A, lda, U, ldu);
  PGB_CUDA(cudaGetLastError());
  note_launch(PATH_STREAM);
  // Every row of the result reads rows of the old B at and below it, and the
  // row blocks run concurrently, so the products read a copy.
  PGB_CUDA(cudaMemcpy2DAsync(Bold, ldo * sizeof(T), B, ldb * sizeof(T), N * sizeof(T), M,
                             cudaMemcpyDeviceToDevice, s));
  if (Kp > M) PGB_CUDA(cudaMemsetAsync(Bold + M * ldo, 0, (size_t)(Kp - M) * ldo * sizeof(T), s));
  // One launch on the tensor-core kernels, which start each tile row's K loop
  // at its diagonal block: the zero half of U is neither loaded nor multiplied.
  int32_t st = PGB200_ERR_UNSUPPORTED;
  if (!rt->cfg.force_generic) st = triangular_product(s, M, N, Kp, alpha, U, ldu, Bold, ldo, B, ldb);
  if (st == PGB200_ERR_UNSUPPORTED) {
    // Generic kernels (operands that miss the tensor-core alignment rules):
    // row block [r0, r1) of U is zero left of column r0, so its product starts
    // there.  At least 256 rows per block, at most 16 blocks.
    int64_t rb = round_up((M + 15) / 16 < 256 ? 256 : (M + 15) / 16, 128);
    st = PGB200_OK;
    for (int64_t r0 = 0; r0 < M && st == PGB200_OK; r0 += rb) {
      const int64_t rows = (M - r0 < rb) ? M - r0 : rb;
      st = gemm_device<T>(s, rows, N, Kp - r0, alpha, U + r0 * ldu + r0, ldu, Bold + r0 * ldo, ldo,
                          false, (T)0, B + r0 * ldb, ldb, false, 0);
    }
  }
  return st;
}

template <typename T>
int32_t symm_entry(void *stream, int64_t M, int64_t N, T alpha, const T *A, int64_t lda,
                   const T *B, int64_t ldb, T beta, T *C, int64_t ldc) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(M >= 0 && N >= 0, "symm: negative size");
  if (M == 0 || N == 0) return PGB200_OK;
  PGB_REQUIRE(A && B && C, "symm: null pointer");
  PGB_REQUIRE(lda >= M && ldb >= N && ldc >= N,
              "symm: lda (%lld) < M (%lld) or ldb (%lld) / ldc (%lld) < N (%lld)", (long long)lda,
              (long long)M, (long long)ldb, (long long)ldc, (long long)N);
  cudaStream_t s = (cudaStream_t)stream;
  Staged<T> sa, sb, sc;
  PGB_TRY(stage<T>(s, A, M, M, lda, true, false, &sa));
  PGB_TRY(stage<T>(s, B, M, N, ldb, true, false, &sb));
  PGB_TRY(stage<T>(s, C, M, N, ldc, beta != (T)0, true, &sc));
  const bool staged = sa.host || sb.host || sc.host;
  const int32_t st =
      symm_device<T>(s, M, N, alpha, sa.dev, sa.ld, sb.dev, sb.ld, beta, sc.dev, sc.ld);
  if (st != PGB200_OK) return st;  // staged copies are released, nothing is copied back
  if (staged) PGB_TRY(sync_check(rt, s));  // a kernel that gave up: nothing is copied back either
  PGB_TRY(finish(s, &sa));
  PGB_TRY(finish(s, &sb));
  PGB_TRY(finish(s, &sc));
  if (staged) PGB_CUDA(cudaStreamSynchronize(s));
  return st;
}

template <typename T>
int32_t trmm_entry(void *stream, int64_t M, int64_t N, T alpha, const T *A, int64_t lda, T *B,
                   int64_t ldb) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(M >= 0 && N >= 0, "trmm: negative size");
  if (M == 0 || N == 0) return PGB200_OK;
  PGB_REQUIRE(A && B, "trmm: null pointer");
  PGB_REQUIRE(lda >= M && ldb >= N, "trmm: lda (%lld) < M (%lld) or ldb (%lld) < N (%lld)",
              (long long)lda, (long long)M, (long long)ldb, (long long)N);
  cudaStream_t s = (cudaStream_t)stream;
  Staged<T> sa, sb;
  PGB_TRY(stage<T>(s, A, M, M, lda, true, false, &sa));
  PGB_TRY(stage<T>(s, B, M, N, ldb, true, true, &sb));
  const bool staged = sa.host || sb.host;
  const int32_t st = trmm_device<T>(rt, s, M, N, alpha, sa.dev, sa.ld, sb.dev, sb.ld);
  if (st != PGB200_OK) return st;  // staged copies are released, nothing is copied back
  if (staged) PGB_TRY(sync_check(rt, s));  // a kernel that gave up: nothing is copied back either
  PGB_TRY(finish(s, &sa));
  PGB_TRY(finish(s, &sb));
  if (staged) PGB_CUDA(cudaStreamSynchronize(s));
  return st;
}

// A (R x P, row-major with lda) := A * C4 (P x P); `sum` (P entries, may be
// null) receives the last row of the result, as the nest leaves it.
int32_t doitgen_entry(void *stream, int64_t R, int64_t P, double *A, int64_t lda,
                      const double *C4, int64_t ldc4, double *sum) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(R >= 0 && P >= 0, "doitgen: negative size");
  if (R == 0 || P == 0) return PGB200_OK;
  PGB_REQUIRE(A && C4 && lda >= P && ldc4 >= P, "doitgen: null pointer or lda/ldc4 < NP (%lld)",
              (long long)P);
  cudaStream_t s = (cudaStream_t)stream;
  Staged<double> sa, sc, ss;
  // `out` = true only marks a registered (pgb200Pin) A as written; a staged A
  // receives the result by the explicit copy below instead of finish().
  PGB_TRY(stage<double>(s, A, R, P, lda, true, true, &sa));
  sa.copy_back = false;
  PGB_TRY(stage<double>(s, C4, P, P, ldc4, true, false, &sc));
  if (sum) PGB_TRY(stage<double>(s, sum, 1, P, P, false, true, &ss));
  // The product cannot be formed in place; the result goes to a second buffer
  // and from there to the caller's A (host array: by the copy-back itself).
  const int64_t ldo = round_up(P, 2);
  PoolBuffer obuf;
  PGB_CUDA(obuf.alloc((size_t)R * ldo * sizeof(double), s));
  double *out = obuf.as<double>();
  const int32_t st = gemm_device<double>(s, R, P, P, 1.0, sa.dev, sa.ld, sc.dev, sc.ld, false, 0.0,
                                         out, ldo, false, 0);
  const bool staged = sa.host || sc.host || ss.host;
  if (st != PGB200_OK) return st;  // staged copies are released, nothing is copied back
  if (staged) PGB_TRY(sync_check(rt, s));  // a kernel that gave up: nothing is copied back either
  if (sa.host) {
    PGB_CUDA(cudaMemcpy2DAsync(A, lda * sizeof(double), out, ldo * sizeof(double),
                               P * sizeof(double), R, cudaMemcpyDeviceToHost, s));
    count_d2h((size_t)R * P * sizeof(double));
  } else {
    PGB_CUDA(cudaMemcpy2DAsync(sa.dev, sa.ld * sizeof(double), out, ldo * sizeof(double),
                               P * sizeof(double), R, cudaMemcpyDeviceToDevice, s));
  }
  if (sum)
    PGB_CUDA(cudaMemcpyAsync(ss.dev, out + (R - 1) * ldo, P * sizeof(double),
                             cudaMemcpyDeviceToDevice, s));
  PGB_TRY(finish(s, &sa));
  PGB_TRY(finish(s, &sc));
  PGB_TRY(finish(s, &ss));
  if (staged) PGB_CUDA(cudaStreamSynchronize(s));
  return st;
}

}  // namespace
}  // namespace pgb200

using namespace pgb200;

extern "C" {

int32_t pgb200Dsymm(void *stream, int64_t M, int64_t N, double alpha, const double *A, int64_t lda,
                    const double *B, int64_t ldb, double beta, double *C, int64_t ldc) {
  PGB_ENTRY(stream);
  return symm_entry<double>(stream, M, N, alpha, A, lda, B, ldb, beta, C, ldc);
}

int32_t pgb200Ssymm(void *stream, int64_t M, int64_t N, float alpha, const float *A, int64_t lda,
                    const float *B, int64_t ldb, float beta, float *C, int64_t ldc) {
  PGB_ENTRY(stream);
  return symm_entry<float>(stream, M, N, alpha, A, lda, B, ldb, beta, C, ldc);
}

int32_t pgb200Dtrmm(void *stream, int64_t M, int64_t N, double alpha, const double *A, int64_t lda,
                    double *B, int64_t ldb) {
  PGB_ENTRY(stream);
  return trmm_entry<double>(stream, M, N, alpha, A, lda, B, ldb);
}

int32_t pgb200Strmm(void *stream, int64_t M, int64_t N, float alpha, const float *A, int64_t lda,
                    float *B, int64_t ldb) {
  PGB_ENTRY(stream);
  return trmm_entry<float>(stream, M, N, alpha, A, lda, B, ldb);
}

int32_t pgb200Ddoitgen(void *stream, int64_t R, int64_t P, double *A, int64_t lda,
                       const double *C4, int64_t ldc4, double *sum) {
  PGB_ENTRY(stream);
  return doitgen_entry(stream, R, P, A, lda, C4, ldc4, sum);
}

int32_t pgb200_kernel_symm(int m, int n, double alpha, double beta, double *C, const double *A,
                           const double *B) {
  PGB_ENTRY(nullptr);
  return pgb200Dsymm(nullptr, m, n, alpha, A, m, B, n, beta, C, n);
}

int32_t pgb200_kernel_symm_f32(int m, int n, float alpha, float beta, float *C, const float *A,
                               const float *B) {
  PGB_ENTRY(nullptr);
  return pgb200Ssymm(nullptr, m, n, alpha, A, m, B, n, beta, C, n);
}

int32_t pgb200_kernel_trmm(int m, int n, double alpha, const double *A, double *B) {
  PGB_ENTRY(nullptr);
  return pgb200Dtrmm(nullptr, m, n, alpha, A, m, B, n);
}

int32_t pgb200_kernel_trmm_f32(int m, int n, float alpha, const float *A, float *B) {
  PGB_ENTRY(nullptr);
  return pgb200Strmm(nullptr, m, n, alpha, A, m, B, n);
}

int32_t pgb200_kernel_doitgen(int nr, int nq, int np, double *A, const double *C4, double *sum) {
  PGB_ENTRY(nullptr);
  PGB_REQUIRE(nr >= 0 && nq >= 0 && np >= 0, "kernel_doitgen: negative size");
  return pgb200Ddoitgen(nullptr, (int64_t)nr * nq, np, A, np, C4, np, sum);
}

}  // extern "C"
