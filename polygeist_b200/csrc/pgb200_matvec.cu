// HBM-streaming fp64 matrix-vector kernels.
//
// One pass over A[MxN] (row-major) produces, per tile, partial row dots
// (for y1 = A*x1) and partial column sums (for y2 = A^T*x2); a second tiny
// kernel adds the partials in a fixed order, so the result is deterministic
// (no floating-point atomics).  With both outputs requested the pair of
// PolyBench mvt nests (kernels/mvt/mvt.c:102-109) costs one read of A instead
// of two.
//
// Tile = TR rows x TC columns per CTA iteration, 8 warps.  Warp w owns rows
// w, w+8, ... of the tile; within a row, lane l loads 128-bit pairs at columns
// 2l + 64q (q < Q), so every load instruction of a warp covers 512 contiguous
// bytes.  Row dots are reduced with shuffles once per row; column sums stay in
// registers for all rows of the tile and are combined across the 8 warps
// through shared memory at the end of the tile.
#include <mutex>

#include "pgb200_internal.h"

namespace pgb200 {

namespace {

constexpr int MV_WARPS = 8;
constexpr int MV_Q = 4;                    // 128-bit loads per lane per row
constexpr int MV_TC = 64 * MV_Q;           // 256 columns per tile
constexpr int MV_ROWS_PER_WARP = 32;
constexpr int MV_TR = MV_WARPS * MV_ROWS_PER_WARP;  // 256 rows per tile
constexpr int MV_RU = 4;                   // rows in flight per warp

__device__ __forceinline__ double2 ldg_stream_v2(const double *p) {
  double2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.f64 {%0,%1}, [%2];"
               : "=d"(v.x), "=d"(v.y)
               : "l"(p));
  return v;
}

// Optional rank-2 update fused into the pass (gemver's first nest): when R2,
// every element becomes A + u1[r]*v1[c] + u2[r]*v2[c] (each product and sum
// rounded separately, like the C statement compiled without contraction), is
// written back, and the updated value feeds the dot products.
struct Rank2 {
  double *Aw;
  const double *u1, *v1, *u2, *v2;
};

template <bool VEC, bool R2 = false>
__global__ void __launch_bounds__(MV_WARPS * 32, 2)
matvec_tile_kernel(const double *__restrict__ A, int64_t lda, int64_t M, int64_t N,
                   const double *__restrict__ x1, const double *__restrict__ x2,
                   double *__restrict__ p1 /* [tiles_c][M] */,
                   double *__restrict__ p2 /* [tiles_r][N] */, int64_t tiles_r, int64_t tiles_c,
                   Rank2 r2 = Rank2{nullptr, nullptr, nullptr, nullptr, nullptr}) {
  __shared__ double red[MV_WARPS][MV_TC];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t ntiles = tiles_r * tiles_c;
  for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int64_t tr = tile / tiles_c, tc = tile - tr * tiles_c;
    const int64_t r0 = tr * MV_TR, c0 = tc * MV_TC;
    double xv[MV_Q][2];
    double colacc[MV_Q][2];
    double v1v[MV_Q][2], v2v[MV_Q][2];
#pragma unroll
    for (int q = 0; q < MV_Q; q++) {
      const int64_t c = c0 + 64 * q + 2 * lane;
      xv[q][0] = (x1 && c < N) ? x1[c] : 0.0;
      xv[q][1] = (x1 && c + 1 < N) ? x1[c + 1] : 0.0;
      colacc[q][0] = 0.0;
      colacc[q][1] = 0.0;
      if (R2) {
        v1v[q][0] = c < N ? r2.v1[c] : 0.0;
        v1v[q][1] = c + 1 < N ? r2.v1[c + 1] : 0.0;
        v2v[q][0] = c < N ? r2.v2[c] : 0.0;
        v2v[q][1] = c + 1 < N ? r2.v2[c + 1] : 0.0;
      }
    }
    for (int it = 0; it < MV_ROWS_PER_WARP / MV_RU; it++) {
      double a[MV_RU][MV_Q][2];
      double w[MV_RU];
#pragma unroll
      for (int u = 0; u < MV_RU; u++) {
        const int64_t r = r0 + warp + MV_WARPS * (it * MV_RU + u);
        const bool rok = r < M;
        w[u] = (x2 && rok) ? x2[r] : 0.0;
        const double *row = A + r * lda;
        const double u1r = (R2 && rok) ? r2.u1[r] : 0.0, u2r = (R2 && rok) ? r2.u2[r] : 0.0;
#pragma unroll
        for (int q = 0; q < MV_Q; q++) {
          const int64_t c = c0 + 64 * q + 2 * lane;
          if (R2) {
            // Read-modify-write of A: plain loads (the data is written back).
#pragma unroll
            for (int e = 0; e < 2; e++) {
              if (rok && c + e < N) {
                double v = r2.Aw[r * lda + c + e];  // not through the restrict/const view of A
                v = __dadd_rn(__dadd_rn(v, __dmul_rn(u1r, v1v[q][e])), __dmul_rn(u2r, v2v[q][e]));
                r2.Aw[r * lda + c + e] = v;
                a[u][q][e] = v;
              } else {
                a[u][q][e] = 0.0;
              }
            }
          } else if (VEC) {
            if (rok && c < N) {  // N even on this path: c+1 < N too
              const double2 v = ldg_stream_v2(row + c);
              a[u][q][0] = v.x;
              a[u][q][1] = v.y;
            } else {
              a[u][q][0] = 0.0;
              a[u][q][1] = 0.0;
            }
          } else {
            a[u][q][0] = (rok && c < N) ? __ldg(row + c) : 0.0;
            a[u][q][1] = (rok && c + 1 < N) ? __ldg(row + c + 1) : 0.0;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < MV_RU; u++) {
        double dot = 0.0;
#pragma unroll
        for (int q = 0; q < MV_Q; q++) {
          dot = fma(a[u][q][0], xv[q][0], dot);
          dot = fma(a[u][q][1], xv[q][1], dot);
          colacc[q][0] = fma(a[u][q][0], w[u], colacc[q][0]);
          colacc[q][1] = fma(a[u][q][1], w[u], colacc[q][1]);
        }
        if (p1) {
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
          const int64_t r = r0 + warp + MV_WARPS * (it * MV_RU + u);
          if (lane == 0 && r < M) p1[tc * M + r] = dot;
        }
      }
    }
    if (p2) {
#pragma unroll
      for (int q = 0; q < MV_Q; q++) {
        red[warp][64 * q + 2 * lane] = colacc[q][0];
        red[warp][64 * q + 2 * lane + 1] = colacc[q][1];
      }
      __syncthreads();
      {
        const int c = threadIdx.x;  // 256 threads, 256 columns
        double sum = 0.0;
#pragma unroll
        for (int ww = 0; ww < MV_WARPS; ww++) sum += red[ww][c];
        if (c0 + c < N) p2[tr * N + c0 + c] = sum;
      }
      __syncthreads();
    }
  }
}

// y[i] = beta*y[i] + alpha * sum_p part[p*len + i], p ascending.
__global__ void matvec_reduce_kernel(double *__restrict__ y, const double *__restrict__ part,
                                     int64_t nparts, int64_t len, double alpha, double beta) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= len) return;
  double sum = 0.0;
  for (int64_t p = 0; p < nparts; p++) sum += part[p * len + i];
  double v = alpha * sum;
  if (beta != 0.0) v = fma(beta, y[i], v);
  y[i] = v;
}

// Both results of the fused pair in one launch: blocks [0,blocks1) reduce the
// row-dot partials into y1, the rest reduce the column-sum partials into y2.
__global__ void matvec_reduce_pair_kernel(double *__restrict__ y1, const double *__restrict__ p1,
                                          int64_t parts1, int64_t len1, int blocks1,
                                          double *__restrict__ y2, const double *__restrict__ p2,
                                          int64_t parts2, int64_t len2, double alpha,
                                          double beta) {
  const bool first = (int)blockIdx.x < blocks1;
  double *y = first ? y1 : y2;
  const double *part = first ? p1 : p2;
  const int64_t nparts = first ? parts1 : parts2, len = first ? len1 : len2;
  const int64_t i = (first ? blockIdx.x : blockIdx.x - blocks1) * (int64_t)blockDim.x + threadIdx.x;
  if (i >= len) return;
  double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
  int64_t p = 0;
  // Four independent partial sums keep four loads in flight; they are combined
  // in a fixed order, so the result is still deterministic.
  for (; p + 3 < nparts; p += 4) {
    s0 += part[p * len + i];
    s1 += part[(p + 1) * len + i];
    s2 += part[(p + 2) * len + i];
    s3 += part[(p + 3) * len + i];
  }
  for (; p < nparts; p++) s0 += part[p * len + i];
  double v = alpha * ((s0 + s1) + (s2 + s3));
  if (beta != 0.0) v = fma(beta, y[i], v);
  y[i] = v;
}

__global__ void vec_scale_kernel(double *y, int64_t len, double beta) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < len) y[i] = (beta == 0.0) ? 0.0 : beta * y[i];
}

}  // namespace

int32_t stream_matvec(cudaStream_t s, int64_t M, int64_t N, const double *A, int64_t lda,
                      double alpha, double beta, const double *x1, double *y1, const double *x2,
                      double *y2) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  if (!y1 && !y2) return PGB200_OK;
  if (M == 0 || N == 0) {
    // Empty sum: y = beta*y.
    if (y1 && M > 0) {
      vec_scale_kernel<<<(unsigned)((M + 255) / 256), 256, 0, s>>>(y1, M, beta);
      note_launch(PATH_STREAM);
    }
    if (y2 && N > 0) {
      vec_scale_kernel<<<(unsigned)((N + 255) / 256), 256, 0, s>>>(y2, N, beta);
      note_launch(PATH_STREAM);
    }
    PGB_CUDA(cudaGetLastError());
    return PGB200_OK;
  }
  const int64_t tiles_r = (M + MV_TR - 1) / MV_TR, tiles_c = (N + MV_TC - 1) / MV_TC;
  const size_t n1 = y1 ? (size_t)tiles_c * M : 0, n2 = y2 ? (size_t)tiles_r * N : 0;
  PoolBuffer scratch;  // this call's own partial sums, released in stream order
  PGB_CUDA(scratch.alloc((n1 + n2) * sizeof(double), s));
  void *ws = scratch.ptr;
  double *p1 = y1 ? static_cast<double *>(ws) : nullptr;
  double *p2 = y2 ? static_cast<double *>(ws) + n1 : nullptr;
  const int64_t ntiles = tiles_r * tiles_c;
  const int64_t cap = (int64_t)rt->num_sms * 2;
  const unsigned grid = (unsigned)(ntiles < cap ? ntiles : cap);
  const bool vec = aligned16(A) && (lda % 2 == 0) && (N % 2 == 0);
  if (vec)
    matvec_tile_kernel<true><<<grid, MV_WARPS * 32, 0, s>>>(A, lda, M, N, y1 ? x1 : nullptr,
                                                            y2 ? x2 : nullptr, p1, p2, tiles_r,
                                                            tiles_c);
  else
    matvec_tile_kernel<false><<<grid, MV_WARPS * 32, 0, s>>>(A, lda, M, N, y1 ? x1 : nullptr,
                                                             y2 ? x2 : nullptr, p1, p2, tiles_r,
                                                             tiles_c);
  note_launch(PATH_STREAM);
  if (y1 && y2) {
    const int b1 = (int)((M + 255) / 256), b2 = (int)((N + 255) / 256);
    matvec_reduce_pair_kernel<<<(unsigned)(b1 + b2), 256, 0, s>>>(y1, p1, tiles_c, M, b1, y2, p2,
                                                                  tiles_r, N, alpha, beta);
    note_launch(PATH_STREAM);
    PGB_CUDA(cudaGetLastError());
    return PGB200_OK;
  }
  if (y1) {
    matvec_reduce_kernel<<<(unsigned)((M + 255) / 256), 256, 0, s>>>(y1, p1, tiles_c, M, alpha,
                                                                     beta);
    note_launch(PATH_STREAM);
  }
  if (y2) {
    matvec_reduce_kernel<<<(unsigned)((N + 255) / 256), 256, 0, s>>>(y2, p2, tiles_r, N, alpha,
                                                                     beta);
    note_launch(PATH_STREAM);
  }
  PGB_CUDA(cudaGetLastError());
  return PGB200_OK;
}

}  // namespace pgb200

namespace pgb200 {
namespace {
__global__ void vec_axpby_kernel(double *y, const double *x, int64_t n, double alpha, double beta) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) y[i] = alpha * x[i] + beta * y[i];
}
}  // namespace

// gemver (blas/gemver/gemver.c:114-131) in two passes over A instead of four:
//   pass 1: A += u1 v1^T + u2 v2^T fused with x += beta * A^T y (then x += z)
//   pass 2: w += alpha * A x
int32_t stream_gemver(cudaStream_t s, int64_t N, double alpha, double beta, double *A, int64_t lda,
                      const double *u1, const double *v1, const double *u2, const double *v2,
                      double *w, double *x, const double *y, const double *z) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  if (N == 0) return PGB200_OK;
  const int64_t tiles_r = (N + MV_TR - 1) / MV_TR, tiles_c = (N + MV_TC - 1) / MV_TC;
  PoolBuffer scratch;
  PGB_CUDA(scratch.alloc((size_t)tiles_r * N * sizeof(double), s));
  void *ws = scratch.ptr;
  double *p2 = static_cast<double *>(ws);
  const int64_t ntiles = tiles_r * tiles_c, cap = (int64_t)rt->num_sms * 2;
  const unsigned grid = (unsigned)(ntiles < cap ? ntiles : cap);
  Rank2 r2{A, u1, v1, u2, v2};
  matvec_tile_kernel<false, true><<<grid, MV_WARPS * 32, 0, s>>>(A, lda, N, N, nullptr, y, nullptr,
                                                                 p2, tiles_r, tiles_c, r2);
  matvec_reduce_kernel<<<(unsigned)((N + 255) / 256), 256, 0, s>>>(x, p2, tiles_r, N, beta, 1.0);
  note_launch(PATH_STREAM, 2);
  PGB_CUDA(cudaGetLastError());
  PGB_TRY(stream_axpby(s, N, 1.0, z, 1.0, x));
  return stream_matvec(s, N, N, A, lda, alpha, 1.0, x, w, nullptr, nullptr);
}

int32_t stream_axpby(cudaStream_t s, int64_t n, double alpha, const double *x, double beta,
                     double *y) {
  if (n <= 0) return PGB200_OK;
  vec_axpby_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(y, x, n, alpha, beta);
  note_launch(PATH_STREAM);
  PGB_CUDA(cudaGetLastError());
  return PGB200_OK;
}
}  // namespace pgb200

// ---------------------------------------------------------------------------
// pgb200DmvtNoAlloc: the fused mat-vec pair for callers that must not allocate.
//
// Same two kernels as pgb200Dmvt, but the per-tile partial sums go to a fixed
// array that is part of the library image instead of the grown-on-demand
// workspace, and nothing in the call path reserves or releases memory (no
// cudaMalloc / cudaFree / stream-ordered pool, no pinned host block).  Every
// GPU that loads the library carries the array (1 MiB) until the process exits.
// ---------------------------------------------------------------------------
namespace pgb200 {
namespace {

constexpr int64_t NOALLOC_MAX_N = 4096;
constexpr int64_t NOALLOC_TILES = (NOALLOC_MAX_N + MV_TC - 1) / MV_TC;
constexpr size_t NOALLOC_DOUBLES = (size_t)2 * NOALLOC_TILES * NOALLOC_MAX_N;  // 1 MiB

static __device__ __align__(256) double g_noalloc_scratch[NOALLOC_DOUBLES];

constexpr int NOALLOC_MAX_DEVICES = 64;
struct NoAllocDevice {
  double *scratch = nullptr;  // device address of g_noalloc_scratch on this GPU
  int num_sms = 0;
};
std::mutex g_noalloc_mu;
NoAllocDevice g_noalloc_dev[NOALLOC_MAX_DEVICES];

// One-time set-up for the current device.  In host code the name of a
// __device__ array is only a handle; the address a kernel can use has to be
// asked for, with the owning device current.
int32_t noalloc_device(NoAllocDevice **out) {
  int dev = 0;
  PGB_CUDA(cudaGetDevice(&dev));
  PGB_REQUIRE(dev >= 0 && dev < NOALLOC_MAX_DEVICES, "DmvtNoAlloc: device index %d out of range",
              dev);
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  NoAllocDevice &d = g_noalloc_dev[dev];
  if (!d.scratch) {
    int major = 0, sms = 0;
    PGB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    PGB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (major != 10) {
      set_error("DmvtNoAlloc: device %d is not sm_100", dev);
      return PGB200_ERR_UNSUPPORTED;
    }
    double *ptr = nullptr;
    PGB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_noalloc_scratch));
    PGB_REQUIRE(ptr != nullptr, "DmvtNoAlloc: no device address for the static scratch array");
    d.num_sms = sms;
    d.scratch = ptr;
  }
  *out = &d;
  return PGB200_OK;
}

}  // namespace
}  // namespace pgb200

extern "C" int32_t pgb200DmvtNoAlloc(void *stream, int64_t N, const double *A, int64_t lda,
                                     const double *y1, const double *y2, double *x1, double *x2) {
  using namespace pgb200;
  PGB_REQUIRE(N >= 0, "DmvtNoAlloc: negative size");
  if (N == 0) return PGB200_OK;
  PGB_REQUIRE(N <= NOALLOC_MAX_N,
              "DmvtNoAlloc: N = %lld exceeds the static scratch limit of %lld; use pgb200Dmvt",
              (long long)N, (long long)NOALLOC_MAX_N);
  PGB_REQUIRE(A && y1 && y2 && x1 && x2 && lda >= N,
              "DmvtNoAlloc: null pointer or lda (%lld) < N (%lld)", (long long)lda, (long long)N);
  // Host arrays would need a staging buffer, i.e. an allocation.
  PGB_REQUIRE(!is_host_pointer(A) && !is_host_pointer(y1) && !is_host_pointer(y2) &&
                  !is_host_pointer(x1) && !is_host_pointer(x2),
              "DmvtNoAlloc: all arrays must be device memory (staging host arrays would allocate)");
  NoAllocDevice *d = nullptr;
  PGB_TRY(noalloc_device(&d));
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t tiles_r = (N + MV_TR - 1) / MV_TR, tiles_c = (N + MV_TC - 1) / MV_TC;
  // Every partial that the second pass reads is written by the first pass of
  // the same call, so nothing left over from an earlier call is ever consumed
  // and nothing needs clearing.
  double *p1 = d->scratch;
  double *p2 = d->scratch + (size_t)tiles_c * N;
  const int64_t ntiles = tiles_r * tiles_c;
  const int64_t cap = (int64_t)d->num_sms * 2;
  const unsigned grid = (unsigned)(ntiles < cap ? ntiles : cap);
  const bool vec = aligned16(A) && (lda % 2 == 0) && (N % 2 == 0);
  if (vec)
    matvec_tile_kernel<true><<<grid, MV_WARPS * 32, 0, s>>>(A, lda, N, N, y1, y2, p1, p2, tiles_r,
                                                            tiles_c);
  else
    matvec_tile_kernel<false><<<grid, MV_WARPS * 32, 0, s>>>(A, lda, N, N, y1, y2, p1, p2,
                                                             tiles_r, tiles_c);
  // The same second pass as pgb200Dmvt (one launch for both vectors, the same
  // four interleaved partial sums), so the two entry points agree bit for bit.
  const int blocks = (int)((N + 255) / 256);
  matvec_reduce_pair_kernel<<<(unsigned)(2 * blocks), 256, 0, s>>>(x1, p1, tiles_c, N, blocks, x2,
                                                                   p2, tiles_r, N, 1.0, 1.0);
  note_launch(PATH_STREAM, 2);
  PGB_CUDA(cudaGetLastError());
  return PGB200_OK;
}
