// Internal declarations shared by the translation units of libpgb200.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "pgb200.h"

namespace pgb200 {

// ---------------------------------------------------------------------------
// Error convention: same message shape as the reference runtime wrappers
// ("'<expr>' failed with '<msg>'", CudaRuntimeWrappers.cpp:29-50); the call
// returns a status instead of aborting.
// ---------------------------------------------------------------------------
void set_error(const char *fmt, ...);
int32_t report_cuda(cudaError_t e, const char *expr);

#define PGB_CUDA(expr)                                              \
  do {                                                              \
    cudaError_t e__ = (expr);                                       \
    if (e__ != cudaSuccess) return ::pgb200::report_cuda(e__, #expr); \
  } while (0)

#define PGB_TRY(expr)                      \
  do {                                     \
    int32_t s__ = (expr);                  \
    if (s__ != PGB200_OK) return s__;      \
  } while (0)

#define PGB_REQUIRE(cond, ...)             \
  do {                                     \
    if (!(cond)) {                         \
      ::pgb200::set_error(__VA_ARGS__);    \
      return PGB200_ERR_INVALID;           \
    }                                      \
  } while (0)

enum Path : int32_t { PATH_NONE = 0, PATH_SIMT = 1, PATH_DMMA = 2, PATH_TCGEN05 = 3, PATH_STREAM = 4 };

struct StageRing;  // page-locked staging ring (pgb200_hostio.cu)

struct Runtime {
  pgb200Config cfg;
  int num_sms;
  int cc_major;
  // Device-visible status word in mapped pinned host memory: kernels store a
  // non-zero code there when a bounded wait expires.
  volatile int32_t *status_host;
  int32_t *status_dev;
  // Side streams of the host-array path: uploads and downloads of row blocks
  // run beside the products of the blocks already on the device.
  cudaStream_t copy_in, copy_out;
  // Page-locked rings through which pageable host arrays travel, one per
  // direction (4 x 32 MiB each, allocated on first use).
  StageRing *ring_up, *ring_down;
};

StageRing *new_stage_ring();
void delete_stage_ring(StageRing *r);
// Unregistered (malloc'd) host memory, as opposed to page-locked or device memory.
bool is_pageable_host(const void *p);
// Contiguous copies between pageable host memory and the device through the
// rings, the host side done by several threads.  Upload: returns when the host
// range has been read (device copies may still be in flight on `stream`).
// Download: ordered after the work on `stream`, returns when the host range is
// complete.
int32_t staged_upload(Runtime *rt, void *dev, const void *host, size_t bytes, cudaStream_t stream);
int32_t staged_download(Runtime *rt, void *host, const void *dev, size_t bytes,
                        cudaStream_t stream);

// Lazily initialises the runtime for the current device; fails (no CPU
// fallback) when there is no sm_100 GPU.
int32_t get_runtime(Runtime **rt);
void note_launch(Path p, int n = 1);
int log_level();

// stderr logging by level (pgb200Config.log_level / PGB200_LOG): errors are
// always printed; level 1 adds life-cycle lines, level 2 one line per call.
void log_line(int level, const char *fmt, ...);

// Waits for `s`, then reads the device status word: an expired device-side
// wait becomes PGB200_ERR_TIMEOUT here (word cleared, message set).  Every
// path that copies results back to a host array calls this before the copy,
// so a kernel that gave up never hands a half-written result to the caller.
int32_t sync_check(Runtime *rt, cudaStream_t s);
int32_t take_device_status(Runtime *rt);

// Transfer accounting behind pgb200TransferCounters().
void count_h2d(size_t bytes);
void count_d2h(size_t bytes);

// Device-residency registry (pgb200Pin): when `p` lies inside a registered host
// range owned by the current device, *dev receives the matching address in the
// device copy; `written` marks the device copy as newer than the host array.
bool registry_lookup(const void *p, void **dev, bool written);

// One of these at the top of every exported compute entry: per-call event
// timing when profiling is on (outermost entry only), and the level-2 log line
// when the call returns.
struct EntryScope {
  const char *name;
  cudaStream_t stream;
  int slot;  // ring slot holding this call's event pair, -1 when not timed
  bool outer;
  EntryScope(const char *name, void *stream);
  ~EntryScope();
  EntryScope(const EntryScope &) = delete;
  EntryScope &operator=(const EntryScope &) = delete;
};
#define PGB_ENTRY(stream) ::pgb200::EntryScope entry_scope__(__func__, (stream))
void profile_enable(bool on);
int32_t profile_dump(const char *path);  // null: stderr
void profile_reset();                    // drops events and totals (shutdown)

// Destroys the communicators and streams of the multi-GPU entry points.
void mg_shutdown();

// cuTensorMapEncodeTiled looked up through the runtime (no link against
// libcuda).  `dims`/`box` innermost first; `strides_bytes` for dims 1..rank-1.
int32_t encode_tensor_map(CUtensorMap *map, CUtensorMapDataType dtype, int rank,
                          const void *base, const uint64_t *dims,
                          const uint64_t *strides_bytes, const uint32_t *box,
                          CUtensorMapSwizzle swizzle);

// Static schedule for kernels whose tiles differ in length (triangular K
// loops): the tile indices of every worker (a CTA, or a CTA pair), assigned
// longest-processing-time-first on the host and passed by value as a kernel
// parameter, so nothing is allocated or copied for it.
struct TileSchedule {
  static constexpr int MAX_TILES = 1408, MAX_WORKERS = 160;
  uint16_t off[MAX_WORKERS + 1];  // tiles of worker w: idx[off[w]] .. idx[off[w+1]-1]
  uint16_t idx[MAX_TILES];
};
// cost[t] > 0 is the relative length of tile t.  Tiles go, longest first (ties:
// lowest index), to the worker with the least work so far (ties: lowest id).
// Returns false when the problem does not fit the fixed-size table.
bool build_lpt_schedule(const int64_t *cost, int64_t tiles, int workers, TileSchedule *out);

// Raises a kernel's dynamic shared-memory limit once per (device, kernel); the
// attribute call is not free and the kernels are launched many times.
int32_t ensure_dynamic_smem(const void *kernel, int bytes);

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// A caller array that may live on the host: staged to the device on demand.
// finish() copies an output back and releases the device copy; a Staged that
// goes out of scope unfinished (an error return) only releases it, so a failed
// call never overwrites the caller's array.
template <typename T>
struct Staged {
  T *dev = nullptr;       // pointer the kernels use
  int64_t ld = 0;         // its leading dimension
  T *host = nullptr;      // non-null while a device copy is held
  int64_t host_ld = 0;
  int64_t rows = 0, cols = 0;
  bool copy_back = false;
  cudaStream_t stream = nullptr;
  Staged() = default;
  Staged(const Staged &) = delete;
  Staged &operator=(const Staged &) = delete;
  ~Staged() {
    if (host && dev) cudaFreeAsync(dev, stream);
  }
};

// Scratch memory of one call: hi/lo planes, split-K partial products, mat-vec
// partial sums.  No two calls that can run at the same time ever share a block:
//  * small requests (<= 64 MiB) come from a cache private to the calling host
//    thread, one block per (device, stream, nesting depth): a thread's calls on
//    one stream are ordered on that stream, so reusing its block is safe, and
//    other threads - on the same stream or another - have blocks of their own.
//    Holders are stack objects, so the k-th holder alive in a thread always
//    maps to block k and two holders alive at once never share one.  No driver
//    call at all after the first use, which matters for products of a few
//    microseconds;
//  * larger requests come from the stream-ordered pool and go back to it (in
//    stream order) when the holder goes out of scope; the pool keeps freed
//    blocks (release threshold: never), so this costs no device allocation
//    after the first call of a size either.
// Cached blocks are released by pgb200Shutdown().
struct PoolBuffer {
  void *ptr = nullptr;
  cudaStream_t stream = nullptr;
  bool owned = false;  // from the pool: returned by the destructor
  bool cached = false; // from the thread's cache: its depth slot is given back
  PoolBuffer() = default;
  PoolBuffer(const PoolBuffer &) = delete;
  PoolBuffer &operator=(const PoolBuffer &) = delete;
  ~PoolBuffer();
  cudaError_t alloc(size_t bytes, cudaStream_t s);
  template <typename T>
  T *as() const { return static_cast<T *>(ptr); }
};

bool is_host_pointer(const void *p);
// Host memory that is not covered by a pgb200Pin registration: has to be
// staged through the device for the duration of the call.
bool needs_staging(const void *p);

// in: copy host->device when staged; out: copy device->host in finish().
template <typename T>
int32_t stage(cudaStream_t s, const T *p, int64_t rows, int64_t cols, int64_t ld,
              bool in, bool out, Staged<T> *st);
template <typename T>
int32_t finish(cudaStream_t s, Staged<T> *st);

// ---------------------------------------------------------------------------
// Kernel families (each in its own .cu).  All pointers are device pointers.
// ---------------------------------------------------------------------------
// Plain SIMT kernels: any size, any alignment.  transB: B(k,j) = B[j*ldb+k].
// lower: only rows [row0,row1) x columns j<=i are computed and written.
template <typename T>
int32_t simt_gemm(cudaStream_t s, int64_t M, int64_t N, int64_t K, T alpha, const T *A,
                  int64_t lda, const T *B, int64_t ldb, bool transB, T beta, T *C,
                  int64_t ldc, bool lower, int64_t row0);

// fp64 DMMA path.  Returns PGB200_ERR_UNSUPPORTED when the operands do not
// meet its alignment rules (the caller then takes the SIMT path).  a_upper:
// A(i,k) is zero for k < i, and the K-blocks left of each tile row's diagonal
// are skipped (neither loaded nor multiplied).
int32_t dmma_gemm(cudaStream_t s, int64_t M, int64_t N, int64_t K, double alpha,
                  const double *A, int64_t lda, const double *B, int64_t ldb, bool transB,
                  double beta, double *C, int64_t ldc, bool lower, bool a_upper = false);

// fp32 3xTF32 tcgen05 path; rows [row0,row0+M) of a lower-triangular update
// when `lower`.  Same UNSUPPORTED convention.  a_upper: A(i,k) is zero for
// k < i; large products then skip the K-blocks left of each tile row's
// diagonal (a pure optimisation: the zeros are in A either way).
int32_t tf32x3_gemm(cudaStream_t s, int64_t M, int64_t N, int64_t K, float alpha,
                    const float *A, int64_t lda, const float *B, int64_t ldb, bool transB,
                    float beta, float *C, int64_t ldc, bool lower, int64_t row0,
                    bool a_upper = false);

// Device-pointer GEMM core on the current device: picks the tensor-core path,
// falls back to the SIMT kernels.  C[MxN] = alpha*A*op(B) + beta*C; `lower` and
// `row0` as in simt_gemm.
template <typename T>
int32_t gemm_device(cudaStream_t s, int64_t M, int64_t N, int64_t K, T alpha, const T *A,
                    int64_t lda, const T *B, int64_t ldb, bool transB, T beta, T *C, int64_t ldc,
                    bool lower, int64_t row0);

// kind::tf32 tensor-pipe issue-rate probe (dense GFLOP/s).
int32_t tf32_peak_probe(cudaStream_t s, double *gflops);

// Launches a one-CTA kernel whose wait can never be satisfied, bounded by
// `limit_cycles`; it must record status code 99 and return.
int32_t wait_timeout_selftest(cudaStream_t s, long long limit_cycles);

// HBM-streaming mat-vec: y1 = beta*y1 + alpha*A*x1 (if y1) and
// y2 = beta*y2 + alpha*A^T*x2 (if y2) in one pass over A[MxN].
int32_t stream_matvec(cudaStream_t s, int64_t M, int64_t N, const double *A, int64_t lda,
                      double alpha, double beta, const double *x1, double *y1,
                      const double *x2, double *y2);

// gemver in two passes over A (device pointers; A is updated in place).
int32_t stream_gemver(cudaStream_t s, int64_t N, double alpha, double beta, double *A, int64_t lda,
                      const double *u1, const double *v1, const double *u2, const double *v2,
                      double *w, double *x, const double *y, const double *z);

// y = alpha*x + beta*y on n doubles (device pointers).
int32_t stream_axpby(cudaStream_t s, int64_t n, double alpha, const double *x, double beta,
                     double *y);

}  // namespace pgb200
