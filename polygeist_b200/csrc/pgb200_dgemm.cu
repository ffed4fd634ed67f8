// fp64 GEMM / SYRK on the DMMA tensor path (tcgen05 has no f64 kind, so the
// fp64 tensor instruction on sm_100a is the warp-level mma.sync .f64).
//
// Persistent kernel, one CTA per SM, 128x128 output tile per CTA iteration:
//   warp 8      producer: one elected lane issues two 3-D TMA loads per K-step
//               into a STAGES-deep shared-memory ring guarded by mbarriers;
//   warps 0-7   consumers: 2x4 warp grid, each a 64x32 sub-tile held as
//               4x4 m16n8 accumulator fragments (128 registers), fed by
//               conflict-free 64-bit shared loads, then the alpha/beta epilogue.
//
// Shared-memory layout.  A 2-D row-major operand with 8-byte elements cannot be
// read conflict-free in the mma fragment pattern (8 rows x 4 k) from a 128-byte
// swizzled tile, so each operand is described to TMA as a 3-D tensor
//   A[M][K]   -> dims (4, M, K/4), strides (lda*8, 32)  box (4, 128, BK/4)
//   B[K][N]   -> dims (4, K, N/4), strides (ldb*8, 32)  box (4, BK, 32)
//   B^T[N][K] -> like A (for the rank-k update, B(k,n) = A[n][k])
// which lands as [k/4][row][4] resp. [n/4][k][4] doubles: the 16 lanes of a
// half-warp then read 128 contiguous bytes.  The innermost TMA coordinate is
// always 0, so every copy starts on a 16-byte boundary.  Out-of-range rows,
// columns and K are zero-filled by TMA; the epilogue masks the stores.
#include <vector>

#include "pgb200_internal.h"

namespace pgb200 {

namespace {

constexpr int BM = 128, BN = 128, BK = 16;
constexpr int STAGES = 6;
constexpr int CONSUMER_WARPS = 8;
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int A_STAGE_BYTES = BM * BK * 8;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 8;  // 16 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
constexpr uint32_t WAIT_LIMIT = 1u << 22;  // try_wait rounds before giving up

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait: false when the limit was reached.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
// Records a failure code where the host can read it (mapped pinned memory).
__device__ __forceinline__ void report_status(int32_t *status, int32_t code, int32_t detail) {
  volatile int32_t *s = status;
  s[1] = detail;
  s[0] = code;
  __threadfence_system();
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void dmma_m16n8k4(double (&d)[4], const double (&a)[2], double b) {
  asm volatile(
      "mma.sync.aligned.m16n8k4.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5}, {%6}, "
      "{%0,%1,%2,%3};"
      : "+d"(d[0]), "+d"(d[1]), "+d"(d[2]), "+d"(d[3])
      : "d"(a[0]), "d"(a[1]), "d"(b));
}

// Tile enumeration.  Full: tiles walk down groups of 8 tile-rows so that the
// CTAs running together share A row panels and B column panels in L2.
// Lower: only tiles that intersect j <= i, row by row.
struct TileMap {
  int64_t tiles_m, tiles_n, total;
  int lower;
  // A is upper triangular (zero left of its diagonal): the K loop of tile row
  // tm starts at the diagonal block instead of 0.
  int a_upper;
  // Split-K (problems with few tiles): the K-blocks of a tile are dealt to
  // `splits` CTAs, `kper` each; work item w = tile * splits + sp writes its raw
  // partial product to partial[sp][M][ldp], added up by a second kernel.
  int splits;
  int64_t kper;
  double *partial;
  int64_t ldp;
  __host__ __device__ int64_t first_kblock(int64_t tm) const {
    return a_upper ? (tm * BM) / BK : 0;
  }
  // Tile of CTA `cta` in its round-th turn.  Tiles come in descending K length
  // when A is triangular, so odd rounds hand them out in reverse CTA order
  // (each CTA's long and short tiles pair up); otherwise plain round-robin.
  // May return an index >= total in the last round.
  __device__ int64_t index(int64_t round, int64_t cta, int64_t ctas) const {
    return round * ctas + ((a_upper && (round & 1)) ? ctas - 1 - cta : cta);
  }
  __host__ __device__ void get(int64_t idx, int64_t *tm, int64_t *tn) const {
    if (lower) {
      // idx = tm*(tm+1)/2 + tn with tn <= tm (BM == BN).
      int64_t r = (int64_t)((sqrt(8.0 * (double)idx + 1.0) - 1.0) * 0.5);
      while (r * (r + 1) / 2 > idx) r--;
      while ((r + 1) * (r + 2) / 2 <= idx) r++;
      *tm = r;
      *tn = idx - r * (r + 1) / 2;
    } else {
      constexpr int64_t G = 8;
      const int64_t per_group = G * tiles_n;
      const int64_t grp = idx / per_group;
      const int64_t first = grp * G;
      const int64_t rows = (tiles_m - first < G) ? (tiles_m - first) : G;
      const int64_t in = idx - grp * per_group;
      *tm = first + in % rows;
      *tn = in / rows;
    }
  }
};

// The tiles of this CTA, in order: from the host-built schedule when SCHED,
// else round-robin (reversed in odd rounds when A is triangular).  Returns
// false when the CTA is done; *t < 0 means "no tile in this turn".
template <bool SCHED>
__device__ __forceinline__ bool next_tile(const TileMap &tiles, const TileSchedule *sched,
                                          int64_t work, int64_t turn, int64_t *t) {
  if (SCHED) {
    const int64_t i = (int64_t)sched->off[blockIdx.x] + turn;
    if (i >= (int64_t)sched->off[blockIdx.x + 1]) return false;
    *t = sched->idx[i];
    return true;
  }
  if (turn * gridDim.x >= work) return false;
  const int64_t x = tiles.index(turn, blockIdx.x, gridDim.x);
  *t = x < work ? x : -1;
  return true;
}

template <bool TRANSB, bool SCHED, bool SPLITK>
__device__ __forceinline__ void dmma_gemm_body(const CUtensorMap *mapA, const CUtensorMap *mapB,
                                               int64_t M, int64_t N, int64_t K, double alpha,
                                               double beta, double *__restrict__ C, int64_t ldc,
                                               const TileMap &tiles, const TileSchedule *sched,
                                               int32_t *status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * STAGES];
  // 1024-byte aligned ring base.
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 32) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(mapA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(mapB) : "memory");
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, CONSUMER_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int64_t nkb = (K + BK - 1) / BK;
  const int64_t work = SPLITK ? tiles.total * tiles.splits : tiles.total;  // (tile, K range) items

  if (warp == CONSUMER_WARPS) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int64_t turn = 0; ok; turn++) {
        int64_t w;
        if (!next_tile<SCHED>(tiles, sched, work, turn, &w)) break;
        if (w < 0) continue;
        int64_t tm, tn;
        tiles.get(SPLITK ? w / tiles.splits : w, &tm, &tn);
        const int64_t kb_lo = SPLITK ? (w % tiles.splits) * tiles.kper : tiles.first_kblock(tm);
        const int64_t kb_hi = SPLITK ? (kb_lo + tiles.kper < nkb ? kb_lo + tiles.kper : nkb) : nkb;
        for (int64_t kb = kb_lo; kb < kb_hi; kb++) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1)) {
            report_status(status, 1, (int32_t)blockIdx.x);
            ok = false;
            break;
          }
          const uint32_t dstA = ring + stage * STAGE_BYTES;
          const uint32_t dstB = dstA + A_STAGE_BYTES;
          mbar_expect_tx(full0 + 8 * stage, STAGE_BYTES);
          tma_load_3d(dstA, mapA, full0 + 8 * stage, 0, (int)(tm * BM), (int)(kb * (BK / 4)));
          if (TRANSB)
            tma_load_3d(dstB, mapB, full0 + 8 * stage, 0, (int)(tn * BN), (int)(kb * (BK / 4)));
          else
            tma_load_3d(dstB, mapB, full0 + 8 * stage, 0, (int)(kb * BK), (int)(tn * (BN / 4)));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    return;
  }

  // -------------------------------- consumers --------------------------------
  const int g = lane >> 2, t4 = lane & 3;
  const int wm = warp >> 2, wn = warp & 3;  // 2 x 4 warps -> 64 x 32 sub-tiles
  uint32_t stage = 0, phase = 0;
  for (int64_t turn = 0;; turn++) {
    int64_t w;
    if (!next_tile<SCHED>(tiles, sched, work, turn, &w)) break;
    if (w < 0) continue;
    int64_t tm, tn;
    tiles.get(SPLITK ? w / tiles.splits : w, &tm, &tn);
    const int sp = SPLITK ? (int)(w % tiles.splits) : 0;
    const int kb_lo = SPLITK ? sp * (int)tiles.kper : (int)tiles.first_kblock(tm);
    const int kb_hi = SPLITK ? (kb_lo + (int)tiles.kper < (int)nkb ? kb_lo + (int)tiles.kper : (int)nkb)
                             : (int)nkb;
    double acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++)
#pragma unroll
        for (int r = 0; r < 4; r++) acc[i][j][r] = 0.0;

    for (int kb = kb_lo; kb < kb_hi; kb++) {
      if (!mbar_wait(full0 + 8 * stage, phase)) {
        report_status(status, 2, (int32_t)blockIdx.x);
        return;
      }
      const double *As = reinterpret_cast<const double *>(ring_ptr + stage * STAGE_BYTES);
      const double *Bs = reinterpret_cast<const double *>(ring_ptr + stage * STAGE_BYTES +
                                                          A_STAGE_BYTES);
#pragma unroll
      for (int kk = 0; kk < BK / 4; kk++) {
        double a[4][2], b[4];
#pragma unroll
        for (int mt = 0; mt < 4; mt++) {
          const int row = wm * 64 + mt * 16 + g;
          a[mt][0] = As[(kk * BM + row) * 4 + t4];
          a[mt][1] = As[(kk * BM + row + 8) * 4 + t4];
        }
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
          const int col = wn * 32 + nt * 8 + g;
          if (TRANSB)
            b[nt] = Bs[(kk * BN + col) * 4 + t4];
          else
            b[nt] = Bs[((col >> 2) * BK + kk * 4 + t4) * 4 + (col & 3)];
        }
#pragma unroll
        for (int mt = 0; mt < 4; mt++)
#pragma unroll
          for (int nt = 0; nt < 4; nt++) dmma_m16n8k4(acc[mt][nt], a[mt], b[nt]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * stage);
      if (++stage == STAGES) {
        stage = 0;
        phase ^= 1;
      }
    }

    // Epilogue: C = alpha*acc + beta*C (split-K: the raw partial product to
    // scratch); each thread owns pairs of adjacent columns (16-byte accesses
    // when the destination allows it).
    double *const Cw = SPLITK ? tiles.partial + (int64_t)sp * M * tiles.ldp : C;
    const int64_t ldw = SPLITK ? tiles.ldp : ldc;
    const double aw = SPLITK ? 1.0 : alpha, bw = SPLITK ? 0.0 : beta;
    const int64_t m_base = tm * BM + wm * 64, n_base = tn * BN + wn * 32;
    const bool vec_ok = ((ldw & 1) == 0) && ((reinterpret_cast<uintptr_t>(Cw) & 15) == 0);
#pragma unroll
    for (int mt = 0; mt < 4; mt++)
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const int64_t r = m_base + mt * 16 + g + 8 * h;
        if (r >= M) continue;
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
          const int64_t c = n_base + nt * 8 + 2 * t4;
          if (c >= N) continue;
          // lower: columns beyond the diagonal of this row are not touched.
          const int64_t lim = tiles.lower ? (r < N - 1 ? r : N - 1) : N - 1;
          if (c > lim) continue;
          double v0 = aw * acc[mt][nt][2 * h], v1 = aw * acc[mt][nt][2 * h + 1];
          double *dst = Cw + r * ldw + c;
          if (c + 1 <= lim) {
            if (vec_ok) {
              if (bw != 0.0) {
                const double2 old = *reinterpret_cast<const double2 *>(dst);
                v0 = fma(bw, old.x, v0);
                v1 = fma(bw, old.y, v1);
              }
              *reinterpret_cast<double2 *>(dst) = make_double2(v0, v1);
            } else {
              if (bw != 0.0) {
                v0 = fma(bw, dst[0], v0);
                v1 = fma(bw, dst[1], v1);
              }
              dst[0] = v0;
              dst[1] = v1;
            }
          } else {
            if (bw != 0.0) v0 = fma(bw, dst[0], v0);
            dst[0] = v0;
          }
        }
      }
  }
}

template <bool TRANSB>
__global__ void __launch_bounds__(THREADS, 1)
dmma_gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                 int64_t M, int64_t N, int64_t K, double alpha, double beta,
                 double *__restrict__ C, int64_t ldc, TileMap tiles, int32_t *status) {
  dmma_gemm_body<TRANSB, false, false>(&mapA, &mapB, M, N, K, alpha, beta, C, ldc, tiles, nullptr,
                                       status);
}

// Same kernel with its tiles taken from a host-built schedule (triangular A).
__global__ void __launch_bounds__(THREADS, 1)
dmma_gemm_sched_kernel(const __grid_constant__ CUtensorMap mapA,
                       const __grid_constant__ CUtensorMap mapB, int64_t M, int64_t N, int64_t K,
                       double alpha, double beta, double *__restrict__ C, int64_t ldc,
                       TileMap tiles, const __grid_constant__ TileSchedule sched,
                       int32_t *status) {
  dmma_gemm_body<false, true, false>(&mapA, &mapB, M, N, K, alpha, beta, C, ldc, tiles, &sched,
                                     status);
}

// Same kernel over (tile, K range) work items; partial products go to scratch.
template <bool TRANSB>
__global__ void __launch_bounds__(THREADS, 1)
dmma_gemm_splitk_kernel(const __grid_constant__ CUtensorMap mapA,
                        const __grid_constant__ CUtensorMap mapB, int64_t M, int64_t N, int64_t K,
                        TileMap tiles, int32_t *status) {
  dmma_gemm_body<TRANSB, false, true>(&mapA, &mapB, M, N, K, 1.0, 0.0, nullptr, 0, tiles, nullptr,
                                      status);
}

// C = beta*C + alpha*(P[0] + P[1] + ...) in split order, two columns per thread
// (lower: only columns up to the diagonal).
constexpr int MAX_SPLITS = 16;
__global__ void dsplitk_reduce_kernel(const double *__restrict__ P, int64_t ldp, int splits,
                                      int64_t M, int64_t N, double alpha, double beta,
                                      double *__restrict__ C, int64_t ldc, int lower) {
  const int64_t pairs = ldp / 2;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * pairs) return;
  const int64_t r = i / pairs, c = (i - r * pairs) * 2;
  if (c >= N || (lower && c > r)) return;  // lower: nothing right of the diagonal is touched
  double2 v[MAX_SPLITS];
  const double *src = P + r * ldp + c;
#pragma unroll
  for (int sp = 0; sp < MAX_SPLITS; sp++)
    if (sp < splits) v[sp] = __ldcs(reinterpret_cast<const double2 *>(src + (int64_t)sp * M * ldp));
  double *dst = C + r * ldc + c;
  const bool two = c + 1 < N && (!lower || c + 1 <= r);
  double old0 = 0.0, old1 = 0.0;
  if (beta != 0.0) {
    old0 = dst[0];
    if (two) old1 = dst[1];
  }
  double2 sum = v[0];
#pragma unroll
  for (int sp = 1; sp < MAX_SPLITS; sp++)
    if (sp < splits) {
      sum.x += v[sp].x;
      sum.y += v[sp].y;
    }
  const double o0 = alpha * sum.x, o1 = alpha * sum.y;
  dst[0] = (beta != 0.0) ? fma(beta, old0, o0) : o0;
  if (two) dst[1] = (beta != 0.0) ? fma(beta, old1, o1) : o1;
}

// dst[rows][ldp] = src[rows][cols] followed by zeros up to column colsP: the
// repacking pass for operands that break a TMA rule.
__global__ void pad_rows_kernel(const double *__restrict__ src, int64_t ld, int64_t rows,
                                int64_t cols, double *__restrict__ dst, int64_t colsP) {
  const int64_t total = rows * colsP;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / colsP, c = i - r * colsP;
    dst[i] = c < cols ? src[r * ld + c] : 0.0;
  }
}

}  // namespace

int32_t dmma_gemm(cudaStream_t s, int64_t M, int64_t N, int64_t K, double alpha, const double *A,
                  int64_t lda, const double *B, int64_t ldb, bool transB, double beta, double *C,
                  int64_t ldc, bool lower, bool a_upper) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  if (K == 0) return PGB200_ERR_UNSUPPORTED;  // nothing to contract: the SIMT path scales C
  if (M >= (int64_t(1) << 31) || N >= (int64_t(1) << 31) || K >= (int64_t(1) << 31))
    return PGB200_ERR_UNSUPPORTED;
  if (lower && M != N) return PGB200_ERR_UNSUPPORTED;  // square lower-triangular update only
  // TMA rules: 16-byte aligned bases and row pitches; the 3-D views need the
  // inner extent (K; N for a row-major B) to be a multiple of 4 elements.  An
  // operand that breaks one is repacked once into scratch with its inner extent
  // padded to a multiple of 4 by zero columns (an O(M*K + K*N) pass beside the
  // O(M*N*K) product), so every shape runs on the tensor-core kernel.
  const int64_t K4 = (K + 3) / 4 * 4, N4 = (N + 3) / 4 * 4;
  const bool a_ok = K == K4 && (lda % 2) == 0 && aligned16(A);
  const bool b_ok = (ldb % 2) == 0 && aligned16(B) && (transB ? K == K4 : N == N4);
  const bool b_is_a = transB && B == A && ldb == lda && N <= M;  // the rank-k update
  PoolBuffer a_pack, b_pack;
  const int64_t pad_cap = (int64_t)rt->num_sms * 16;
  auto pad_grid = [&](int64_t total) {
    const int64_t g = (total + 255) / 256;
    return (unsigned)(g < 1 ? 1 : (g > pad_cap ? pad_cap : g));
  };
  if (!a_ok) {
    PGB_CUDA(a_pack.alloc((size_t)M * K4 * sizeof(double), s));
    pad_rows_kernel<<<pad_grid(M * K4), 256, 0, s>>>(A, lda, M, K, a_pack.as<double>(), K4);
    note_launch(PATH_DMMA);
    if (b_is_a) {
      B = a_pack.as<double>();
      ldb = K4;
    }
    A = a_pack.as<double>();
    lda = K4;
  }
  if (!(b_is_a ? a_ok : b_ok)) {
    if (!b_is_a) {
      const int64_t rows = transB ? N : K, cols = transB ? K : N, colsP = transB ? K4 : N4;
      PGB_CUDA(b_pack.alloc((size_t)rows * colsP * sizeof(double), s));
      pad_rows_kernel<<<pad_grid(rows * colsP), 256, 0, s>>>(B, ldb, rows, cols, b_pack.as<double>(),
                                                             colsP);
      note_launch(PATH_DMMA);
      B = b_pack.as<double>();
      ldb = colsP;
    }
  }
  PGB_CUDA(cudaGetLastError());
  // From here on K is the padded inner extent (the added columns of A are zero;
  // rows of a row-major B past the true K are zero-filled by TMA).
  const int64_t n_map = N4;   // columns of a row-major B the tensor map may address
  const int64_t k_rows = K;  // rows a row-major B really has
  K = K4;

  CUtensorMap mapA, mapB;
  {
    const uint64_t dims[3] = {4, (uint64_t)M, (uint64_t)(K / 4)};
    const uint64_t str[2] = {(uint64_t)lda * 8, 32};
    const uint32_t box[3] = {4, BM, BK / 4};
    PGB_TRY(encode_tensor_map(&mapA, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 3, A, dims, str, box,
                              CU_TENSOR_MAP_SWIZZLE_NONE));
  }
  if (transB) {
    const uint64_t dims[3] = {4, (uint64_t)N, (uint64_t)(K / 4)};
    const uint64_t str[2] = {(uint64_t)ldb * 8, 32};
    const uint32_t box[3] = {4, BN, BK / 4};
    PGB_TRY(encode_tensor_map(&mapB, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 3, B, dims, str, box,
                              CU_TENSOR_MAP_SWIZZLE_NONE));
  } else {
    const uint64_t dims[3] = {4, (uint64_t)k_rows, (uint64_t)(n_map / 4)};
    const uint64_t str[2] = {(uint64_t)ldb * 8, 32};
    const uint32_t box[3] = {4, BK, BN / 4};
    PGB_TRY(encode_tensor_map(&mapB, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 3, B, dims, str, box,
                              CU_TENSOR_MAP_SWIZZLE_NONE));
  }
  TileMap tiles;
  tiles.tiles_m = (M + BM - 1) / BM;
  tiles.tiles_n = (N + BN - 1) / BN;
  tiles.lower = lower ? 1 : 0;
  tiles.a_upper = a_upper ? 1 : 0;
  tiles.splits = 1;
  tiles.kper = 0;
  tiles.partial = nullptr;
  tiles.ldp = 0;
  if (lower) {
    tiles.total = tiles.tiles_m * (tiles.tiles_m + 1) / 2;
  } else {
    tiles.total = tiles.tiles_m * tiles.tiles_n;
  }
  int64_t ctas = rt->num_sms - (rt->cfg.reserve_sms > 0 ? rt->cfg.reserve_sms : 0);
  if (ctas < 1) ctas = 1;
  const unsigned grid = (unsigned)(tiles.total < ctas ? tiles.total : ctas);
  // Few tiles (less than half of the SMs would get one): deal the K-blocks of
  // every tile to several CTAs (at least 8 K-blocks each) and add the partial
  // products afterwards in split order.  A tile's time is K / (one SM's DMMA
  // rate) however many SMs idle beside it.
  if (!a_upper && tiles.total * 2 <= ctas && !rt->cfg.no_split_k) {
    const int64_t nkb = (K + BK - 1) / BK;
    int64_t sp = ctas / tiles.total;
    if (sp > nkb / 8) sp = nkb / 8;
    if (sp > MAX_SPLITS) sp = MAX_SPLITS;
    if (sp >= 2) {
      const int64_t kper = (nkb + sp - 1) / sp;
      const int splits = (int)((nkb + kper - 1) / kper);
      const int64_t ldp = (N + 1) / 2 * 2;
      PoolBuffer scratch;  // this call's own partial products, released in stream order
      PGB_CUDA(scratch.alloc((size_t)splits * M * ldp * sizeof(double), s));
      void *ws = scratch.ptr;
      tiles.splits = splits;
      tiles.kper = kper;
      tiles.partial = static_cast<double *>(ws);
      tiles.ldp = ldp;
      const int64_t work = tiles.total * splits;
      const unsigned g2 = (unsigned)(work < ctas ? work : ctas);
      if (transB) {
        PGB_TRY(ensure_dynamic_smem((const void *)dmma_gemm_splitk_kernel<true>, SMEM_BYTES));
        dmma_gemm_splitk_kernel<true><<<g2, THREADS, SMEM_BYTES, s>>>(mapA, mapB, M, N, K, tiles,
                                                                       rt->status_dev);
      } else {
        PGB_TRY(ensure_dynamic_smem((const void *)dmma_gemm_splitk_kernel<false>, SMEM_BYTES));
        dmma_gemm_splitk_kernel<false><<<g2, THREADS, SMEM_BYTES, s>>>(mapA, mapB, M, N, K, tiles,
                                                                        rt->status_dev);
      }
      PGB_CUDA(cudaGetLastError());
      const int64_t items = M * (ldp / 2);
      dsplitk_reduce_kernel<<<(unsigned)((items + 127) / 128), 128, 0, s>>>(
          tiles.partial, ldp, splits, M, N, alpha, beta, C, ldc, lower ? 1 : 0);
      PGB_CUDA(cudaGetLastError());
      note_launch(PATH_DMMA, 2);
      return PGB200_OK;
    }
  }
  // Triangular A: tiles differ in length.  With few tiles per CTA a static
  // round-robin leaves SMs idle at the end (13 % at 4096 x 4096), so the tiles
  // are handed out longest-first on the host when the table fits.
  if (a_upper && !transB && !lower && tiles.total > (int64_t)grid) {
    const int64_t nkb = (K + BK - 1) / BK;
    std::vector<int64_t> cost((size_t)tiles.total);
    for (int64_t t = 0; t < tiles.total; t++) {
      int64_t tm, tn;
      tiles.get(t, &tm, &tn);
      const int64_t len = nkb - tiles.first_kblock(tm);
      cost[(size_t)t] = (len > 0 ? len : 0) + 2;  // + the tile's epilogue
    }
    TileSchedule sched;
    if (build_lpt_schedule(cost.data(), tiles.total, (int)grid, &sched)) {
      PGB_TRY(ensure_dynamic_smem((const void *)dmma_gemm_sched_kernel, SMEM_BYTES));
      dmma_gemm_sched_kernel<<<grid, THREADS, SMEM_BYTES, s>>>(mapA, mapB, M, N, K, alpha, beta, C,
                                                               ldc, tiles, sched, rt->status_dev);
      note_launch(PATH_DMMA);
      PGB_CUDA(cudaGetLastError());
      return PGB200_OK;
    }
  }
  if (transB) {
    PGB_TRY(ensure_dynamic_smem((const void *)dmma_gemm_kernel<true>, SMEM_BYTES));
    dmma_gemm_kernel<true><<<grid, THREADS, SMEM_BYTES, s>>>(mapA, mapB, M, N, K, alpha, beta, C,
                                                              ldc, tiles, rt->status_dev);
  } else {
    PGB_TRY(ensure_dynamic_smem((const void *)dmma_gemm_kernel<false>, SMEM_BYTES));
    dmma_gemm_kernel<false><<<grid, THREADS, SMEM_BYTES, s>>>(mapA, mapB, M, N, K, alpha, beta, C,
                                                               ldc, tiles, rt->status_dev);
  }
  note_launch(PATH_DMMA);
  PGB_CUDA(cudaGetLastError());
  return PGB200_OK;
}

// Test hook (host only): the (tile row, tile column) of every linear tile
// index of the fp64 kernel, as TileMap::get yields them.  Returns the count,
// or -1 when `cap` pairs do not hold them.
int64_t enumerate_dmma_tiles_for_test(int64_t tiles_m, int64_t tiles_n, int lower, int64_t *tm_out,
                                      int64_t *tn_out, int64_t cap) {
  TileMap t = {};
  t.tiles_m = tiles_m;
  t.tiles_n = tiles_n;
  t.lower = lower;
  t.total = lower ? tiles_m * (tiles_m + 1) / 2 : tiles_m * tiles_n;
  if (t.total > cap) return -1;
  for (int64_t i = 0; i < t.total; i++) t.get(i, &tm_out[i], &tn_out[i]);
  return t.total;
}

}  // namespace pgb200
