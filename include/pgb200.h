/* libpgb200 - B200 (sm_100a) runtime library for the dense contractions that
 * appear as C loop nests in Polygeist's PolyBench workloads.
 *
 * Calling convention.  The entry points take exactly what Polygeist's C-style
 * memref lowering hands to an external callee: one bare pointer to element
 * (0,0) of each row-major array (lib/polygeist/Passes/ConvertPolygeistToLLVM.cpp
 * :2802-2810, pinned by test/polygeist-opt/cconv-func.mlir:3-18), sizes and
 * leading dimensions as explicit integers, floating scalars by value, and an
 * opaque `void*` stream whose null value means the default stream
 * (lib/polygeist/Passes/RuntimeWrapperUtils.h:124,139;
 * ConvertPolygeistToLLVM.cpp:2315-2318).  Like the reference runtime's `*Err`
 * wrappers (lib/polygeist/ExecutionEngine/CudaRuntimeWrappers.cpp:29-50,90-97)
 * every function returns an int32_t status (0 = success), prints
 * "'<expr>' failed with '<msg>'" to stderr on a CUDA error and returns: no
 * abort, no exception.
 *
 * Pointers.  Each array pointer may be device, managed or host memory.  Device
 * and managed arrays are used in place and the call is asynchronous on
 * `stream`.  Host arrays (what the PolyBench nests operate on,
 * tools/cgeist/Test/polybench/utilities/polybench.h:233-235) are staged to the
 * GPU and back inside the call, which then synchronises `stream` before
 * returning because the C caller reads the result immediately.
 *
 * There is no CPU fallback: without a usable sm_100 GPU every compute entry
 * point fails with PGB200_ERR_CUDA / PGB200_ERR_UNSUPPORTED.
 */
#ifndef PGB200_H
#define PGB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  PGB200_OK = 0,
  PGB200_ERR_INVALID = 1,     /* bad size, leading dimension or null pointer */
  PGB200_ERR_CUDA = 2,        /* a CUDA runtime/driver call failed           */
  PGB200_ERR_NCCL = 3,        /* reserved for the multi-GPU entry points     */
  PGB200_ERR_TIMEOUT = 4,     /* a bounded device-side wait expired          */
  PGB200_ERR_UNSUPPORTED = 5  /* no sm_100 device / feature unavailable      */
};

/* Optional tuning knobs; pgb200Init(NULL) and lazy initialisation use the
 * defaults.  A zero field means "default". */
typedef struct pgb200Config {
  int32_t log_level;          /* stderr verbosity: 0 errors only, 1 also one line
                                 per initialised device and per Pin/Unpin, 2 also
                                 one line per compute call (entry, sizes, kernel
                                 family).  The environment variable PGB200_LOG,
                                 when set, takes precedence.  Errors always have
                                 the "'<expr>' failed with '<msg>'" form of
                                 CudaRuntimeWrappers.cpp:29-50.                 */
  int32_t sgemm_chunk_kblocks;/* 3xTF32: K-blocks (of 16) accumulated in the
                                 tensor-core accumulator before it is drained
                                 into fp32 registers; bounds the truncation
                                 bias of tensor-core accumulation             */
  int32_t force_generic;      /* 1: always take the plain SIMT kernels        */
  int32_t sgemm_planes_only;  /* 1: the 3xTF32 path never reads an operand in
                                 place (always writes both hi and lo planes)  */
  int32_t reserve_sms;        /* SMs the persistent GEMM kernels leave free, so
                                 that a concurrent collective (NCCL broadcast
                                 of the next operand chunk) can run beside them */
  int32_t no_two_cta;         /* 1: never use the two-CTA (cta_group::2) fp32
                                 kernel (default: whenever a product has >= 512
                                 rows and enough tiles)                        */
  int32_t no_split_k;         /* 1: never split K over several CTAs (default:
                                 whenever fewer than half of the SMs would get
                                 a tile and K is long enough)                  */
  int32_t sgemm_b_in_place;   /* 1: fp32 row-major B always used in place,
                                 whatever M (default: transposed once into
                                 K-major planes for tall products)             */
  int32_t no_step_sync;       /* 1: the CTAs of the two-CTA fp32 kernel do not
                                 meet between rounds of tiles (default: they
                                 do, which keeps the CTAs that share an operand
                                 panel close together in K so that one DRAM
                                 read serves all of them)                      */
} pgb200Config;

/* Runtime life cycle.  Replaces nothing in the reference one-to-one; plays the
 * role of the lazily created primary context of
 * lib/polygeist/ExecutionEngine/CudaRuntimeWrappers.cpp:52-76.  Initialisation
 * is also done lazily by the first compute call. */
int32_t pgb200Init(const pgb200Config *cfg);
int32_t pgb200Shutdown(void);
const char *pgb200GetLastErrorString(void);
int32_t pgb200Version(void);

/* C[MxN] = alpha * A[MxK] * B[KxN] + beta * C, all row-major.
 * Replaces the loop nest kernel_gemm,
 * tools/cgeist/Test/polybench/linear-algebra/blas/gemm/gemm.c:104-113, and each
 * of the two nests of kernel_2mm,
 * tools/cgeist/Test/polybench/linear-algebra/kernels/2mm/2mm.c:103-119
 * (beta == 0 never reads C, like `tmp[i][j] = 0` at 2mm.c:108).
 * fp64 runs on the DMMA tensor path. */
int32_t pgb200Dgemm(void *stream, int64_t M, int64_t N, int64_t K, double alpha,
                    const double *A, int64_t lda, const double *B, int64_t ldb,
                    double beta, double *C, int64_t ldc);

/* fp32 version of the same nest (gemm.c built with -DDATA_TYPE_IS_FLOAT,
 * gemm.h:70-77) on the tcgen05 tensor path with an error-compensated 3xTF32
 * split. */
int32_t pgb200Sgemm(void *stream, int64_t M, int64_t N, int64_t K, float alpha,
                    const float *A, int64_t lda, const float *B, int64_t ldb,
                    float beta, float *C, int64_t ldc);

/* C[MxN] = alpha * A[MxK] * B[NxK]^T + beta * C: the product of two row-major
 * arrays over their common inner dimension, the statement shape
 * `C[i][j] += alpha*A[i][k]*B[j][k]` of the rank-k / rank-2k nests
 * (tools/cgeist/Test/polybench/linear-algebra/blas/syrk/syrk.c:102-105 with two
 * different arrays).  Also the unit a GPU computes per column block when the
 * rows of a triangular update are partitioned across devices. */
int32_t pgb200DgemmNT(void *stream, int64_t M, int64_t N, int64_t K, double alpha,
                      const double *A, int64_t lda, const double *B, int64_t ldb,
                      double beta, double *C, int64_t ldc);
int32_t pgb200SgemmNT(void *stream, int64_t M, int64_t N, int64_t K, float alpha,
                      const float *A, int64_t lda, const float *B, int64_t ldb,
                      float beta, float *C, int64_t ldc);

/* Lower triangle of C[NxN] = alpha * (A * B^T + B * A^T) + beta * C with A, B
 * [NxK]; the strict upper triangle is untouched.  Replaces kernel_syr2k,
 * tools/cgeist/Test/polybench/linear-algebra/blas/syr2k/syr2k.c:100-109. */
int32_t pgb200Dsyr2k(void *stream, int64_t N, int64_t K, double alpha,
                     const double *A, int64_t lda, const double *B, int64_t ldb,
                     double beta, double *C, int64_t ldc);
int32_t pgb200Ssyr2k(void *stream, int64_t N, int64_t K, float alpha,
                     const float *A, int64_t lda, const float *B, int64_t ldb,
                     float beta, float *C, int64_t ldc);

/* C[MxN] = beta * C + alpha * S * B[MxN], S the symmetric M x M matrix whose
 * lower triangle (diagonal included) is stored in A; the strict upper triangle
 * of A is never read.  Replaces kernel_symm,
 * tools/cgeist/Test/polybench/linear-algebra/blas/symm/symm.c:108-117.  One pass
 * expands A to the dense S in scratch memory, then the dense product runs. */
int32_t pgb200Dsymm(void *stream, int64_t M, int64_t N, double alpha, const double *A,
                    int64_t lda, const double *B, int64_t ldb, double beta, double *C,
                    int64_t ldc);
int32_t pgb200Ssymm(void *stream, int64_t M, int64_t N, float alpha, const float *A,
                    int64_t lda, const float *B, int64_t ldb, float beta, float *C,
                    int64_t ldc);

/* B[MxN] = alpha * (I + L^T) * B in place, L the strict lower triangle of the
 * M x M array A (unit diagonal: neither A's diagonal nor its upper triangle is
 * read).  Replaces kernel_trmm,
 * tools/cgeist/Test/polybench/linear-algebra/blas/trmm/trmm.c:101-106.  The
 * products read a copy of the old B and skip the zero part of I + L^T by row
 * blocks.  Entries of B are expected to be finite: inside a diagonal block a
 * zero of the triangular factor still multiplies the rows above it. */
int32_t pgb200Dtrmm(void *stream, int64_t M, int64_t N, double alpha, const double *A,
                    int64_t lda, double *B, int64_t ldb);
int32_t pgb200Strmm(void *stream, int64_t M, int64_t N, float alpha, const float *A,
                    int64_t lda, float *B, int64_t ldb);

/* A[RxP] = A * C4[PxP] in place (R = NR*NQ rows of the flattened 3-D array);
 * `sum` (P entries, may be null) receives the last row of the result, which is
 * what the nest leaves there.  Replaces kernel_doitgen,
 * tools/cgeist/Test/polybench/linear-algebra/kernels/doitgen/doitgen.c:88-97. */
int32_t pgb200Ddoitgen(void *stream, int64_t R, int64_t P, double *A, int64_t lda,
                       const double *C4, int64_t ldc4, double *sum);

/* Lower triangle of C[NxN] = alpha * A[NxK] * A^T + beta * C; the strict upper
 * triangle of C is neither read nor written.  Replaces kernel_syrk,
 * tools/cgeist/Test/polybench/linear-algebra/blas/syrk/syrk.c:97-106. */
int32_t pgb200Dsyrk(void *stream, int64_t N, int64_t K, double alpha,
                    const double *A, int64_t lda, double beta, double *C,
                    int64_t ldc);
int32_t pgb200Ssyrk(void *stream, int64_t N, int64_t K, float alpha,
                    const float *A, int64_t lda, float beta, float *C,
                    int64_t ldc);

/* Rows [row0,row1) of the same lower-triangular update: the unit one GPU owns
 * when the rows of C are partitioned across devices.  A must hold rows
 * [0,row1).  No counterpart loop in the reference (it has no multi-GPU path);
 * the statements are those of syrk.c:97-106 with the outer i restricted. */
int32_t pgb200SsyrkRows(void *stream, int64_t N, int64_t K, int64_t row0,
                        int64_t row1, float alpha, const float *A, int64_t lda,
                        float beta, float *C, int64_t ldc);

/* The same GEMM / rank-k update on `ndev` GPUs of one box (devices 0..ndev-1)
 * from a single host thread: the rows of the output are partitioned across the
 * GPUs (equal heights for the GEMM, equal triangular areas for the update) and
 * the shared operand is broadcast from device 0 by NCCL in K-slices, each
 * slice's product running while the next slice travels.  Arrays are host
 * memory or memory of device 0; the call returns when the result is back in
 * C.  NCCL is loaded at run time (libnccl.so.2); ndev == 1 makes no NCCL call.
 * The reference has no multi-GPU path: the nests are those of gemm.c:104-113 and
 * syrk.c:97-106, whose rows are independent. */
int32_t pgb200DgemmMg(int32_t ndev, int64_t M, int64_t N, int64_t K, double alpha,
                      const double *A, int64_t lda, const double *B, int64_t ldb,
                      double beta, double *C, int64_t ldc);
int32_t pgb200SgemmMg(int32_t ndev, int64_t M, int64_t N, int64_t K, float alpha,
                      const float *A, int64_t lda, const float *B, int64_t ldb,
                      float beta, float *C, int64_t ldc);
int32_t pgb200SsyrkMg(int32_t ndev, int64_t N, int64_t K, float alpha,
                      const float *A, int64_t lda, float beta, float *C,
                      int64_t ldc);

/* y[.] = alpha * op(A) * x + beta * y with A[MxN] row-major;
 * transA == 0: op(A) = A (y has M entries), transA != 0: op(A) = A^T (y has N).
 * Replaces either nest of kernel_mvt taken alone,
 * tools/cgeist/Test/polybench/linear-algebra/kernels/mvt/mvt.c:102-105 and
 * :106-109, and the same-shaped nests of atax/bicg/gesummv. */
int32_t pgb200Dgemv(void *stream, int32_t transA, int64_t M, int64_t N,
                    double alpha, const double *A, int64_t lda, const double *x,
                    double beta, double *y);

/* y1[M] = alpha * A * x1 + beta * y1 and y2[N] = alpha * A^T * x2 + beta * y2
 * with A[MxN] read ONCE for both results (beta == 0 never reads y1 / y2).
 * Replaces the scop of kernel_bicg,
 * tools/cgeist/Test/polybench/linear-algebra/kernels/bicg/bicg.c:97-108
 * (s = A^T r and q = A p accumulated in the same i-j nest). */
int32_t pgb200DgemvPair(void *stream, int64_t M, int64_t N, double alpha,
                        const double *A, int64_t lda, const double *x1,
                        const double *x2, double beta, double *y1, double *y2);

/* The four nests of kernel_gemver,
 * tools/cgeist/Test/polybench/linear-algebra/blas/gemver/gemver.c:114-131:
 *   A += u1 v1^T + u2 v2^T;  x += beta * A^T y;  x += z;  w += alpha * A x
 * in two passes over A[NxN] instead of four (the rank-2 update is fused with
 * the transposed product; A is updated in place like in the C source). */
int32_t pgb200Dgemver(void *stream, int64_t N, double alpha, double beta,
                      double *A, int64_t lda, const double *u1, const double *v1,
                      const double *u2, const double *v2, double *w, double *x,
                      const double *y, const double *z);

/* x1 += A * y1 and x2 += A^T * y2 with A[NxN] read ONCE for both results.
 * Replaces the whole scop of kernel_mvt, mvt.c:102-109. */
int32_t pgb200Dmvt(void *stream, int64_t N, const double *A, int64_t lda,
                   const double *y1, const double *y2, double *x1, double *x2);

/* The same fused pair, x1 += A*y1 and x2 += A^T*y2, for callers that are not
 * allowed to allocate.  This entry point has no counterpart in the reference.
 *
 * Who needs it: a host program that hands all GPU memory to its own arena at
 * start-up (any later cudaMalloc by a library would simply fail), and code in a
 * latency-critical section, where cudaMalloc / cudaFree would stall every stream
 * of the device.  pgb200Dmvt keeps its per-tile partial sums in a workspace that
 * it grows on demand; this variant keeps them in a fixed 1 MiB array inside the
 * library image, so the call reserves and releases nothing - no cudaMalloc, no
 * cudaFree, no memory pool, no pinned host block.  Every GPU that loads the
 * library holds that 1 MiB until the process exits.
 *
 * Limits and rules:
 *  - N <= 4096 (what the fixed array can hold); larger N is rejected with
 *    PGB200_ERR_INVALID and a message that names the limit.
 *  - A, y1, y2, x1, x2 must all be device (or managed) memory: host arrays would
 *    need a staging buffer, so they are rejected too.
 *  - The first call on each device looks up the device address of the array
 *    (once, with that device current).  Make that first call outside any
 *    stream capture.
 *  - All calls on a device share the one array.  It still holds the previous
 *    call's partial sums when the next call starts; that is harmless because
 *    each call overwrites every entry before reading it (nothing has to start
 *    at zero).  Two calls that overlap on the GPU - different streams, or two
 *    host threads - would overwrite each other's partial sums: serialise them.
 *  - The looked-up address is remembered per device for the life of the
 *    process; after a cudaDeviceReset() it is stale, so do not reset a device
 *    between calls of this entry point.
 * The result equals pgb200Dmvt's bit for bit (same two kernels, same summation
 * order). */
int32_t pgb200DmvtNoAlloc(void *stream, int64_t N, const double *A, int64_t lda,
                          const double *y1, const double *y2, double *x1,
                          double *x2);

/* Device residency across calls.  pgb200Pin registers the host range
 * [host, host + bytes) and keeps a device copy of it (uploaded once, now);
 * until pgb200Unpin every entry point that is handed a pointer inside the
 * range computes on the device copy and moves nothing over PCIe, and a call
 * whose arrays are all registered (or device memory) is asynchronous on its
 * stream like a call on device arrays.  The device copy is the current one
 * while the range is registered: the host array is stale after a call that
 * wrote into it, until pgb200PinSync (download if a call wrote to it, stay
 * registered) or pgb200Unpin (download if written, then release).  Host
 * writes to a registered range are not seen by the device copy; unpin, write,
 * pin again.  Ranges must not overlap; `host` given to Unpin / PinSync is the
 * pointer that was registered.  The downloads synchronise the device.
 * This is how the reference's own CUDA variant of the kernels keeps operands
 * in cudaMalloc buffers across the kernel call and copies only the result
 * back (tools/cgeist/Test/CUDA/polybench-cuda/gemm/gemm.cu:89-100); here the
 * generated host code keeps its host arrays and brackets the calls instead. */
int32_t pgb200Pin(const void *host, uint64_t bytes);
int32_t pgb200PinSync(const void *host);
int32_t pgb200Unpin(const void *host);

/* Bytes this library has copied host->device and device->host so far in this
 * process (staging of host arrays, row-block pipeline, Pin/PinSync/Unpin, the
 * multi-GPU scatter and gather).  Either pointer may be null.  No counterpart
 * in the reference. */
int32_t pgb200TransferCounters(int64_t *h2d_bytes, int64_t *d2h_bytes);

/* Per-call device timing.  With the environment variable PGB200_PROFILE=1 (or
 * after pgb200ProfileEnable(1)) every compute entry point brackets its work on
 * the stream with a pair of CUDA events taken from a ring of 512; the oldest
 * pair is resolved and added to its entry's totals when the ring wraps.
 * pgb200ProfileDump synchronises the device, resolves what is pending and
 * writes one line per entry point - name, calls, total and mean milliseconds -
 * to `path`, or to stderr when path is null; it is also called at
 * pgb200Shutdown when PGB200_PROFILE_FILE names a file.  Plays the role of the
 * reference's profile-guided timing runtime, which brackets a region with
 * device synchronisations and clock_gettime and appends the elapsed time to a
 * file per kernel id at exit
 * (lib/polygeist/ExecutionEngine/PGORuntime.h:58-113). */
int32_t pgb200ProfileEnable(int32_t on);
int32_t pgb200ProfileDump(const char *path);

/* Counter-based uniform generator used by the test and benchmark harness
 * (device pointer only).  Element (r,c) of the logical rows x cols array, for
 * r in [row0,row0+rows), written at dst[(r-row0)*ld + c]:
 *   h = splitmix64(seed ^ (array_id << 56)); x = splitmix64(h + r*cols + c);
 *   fp64: u = (x >> 11) * 2^-53; fp32: u = (x >> 40) * 2^-24;
 *   value = lo + (hi - lo) * u.
 * No counterpart in the reference (PolyBench's init_array is a modular
 * formula, e.g. gemm.c:42-63). */
int32_t pgb200FillUniformF64(void *stream, double *dst, int64_t row0,
                             int64_t rows, int64_t cols, int64_t ld,
                             uint64_t seed, uint32_t array_id, double lo,
                             double hi);
int32_t pgb200FillUniformF32(void *stream, float *dst, int64_t row0,
                             int64_t rows, int64_t cols, int64_t ld,
                             uint64_t seed, uint32_t array_id, float lo,
                             float hi);

/* Which kernel family served the last compute call of this thread:
 * 0 none yet, 1 plain SIMT kernels, 2 DMMA tensor path, 3 tcgen05 3xTF32 path,
 * 4 HBM-streaming mat-vec.  Lets tests assert that the fast path ran. */
int32_t pgb200LastPath(void);

/* Every device-side wait in the tensor-core kernels (mbarrier, tensor-memory
 * handshakes) has an iteration limit; a kernel whose wait expires records a code
 * in a host-visible status word and returns instead of hanging.  This reads
 * and clears that word: PGB200_OK or PGB200_ERR_TIMEOUT.  Call it after the
 * stream has been synchronised.  (The reference runtime has no such check: its
 * wrappers only report launch errors, CudaRuntimeWrappers.cpp:90-97.) */
int32_t pgb200PollDeviceStatus(void);

/* Measured peak of the current GPU, the denominators of the fp64 rooflines:
 * kind 0 = fp64 tensor (best of the mma.sync .f64 shapes; 10/11/12/13 select
 * m16n8k4 / k8 / k16 / m8n8k4), 1 = fp64 FMA, in GFLOP/s from register-only
 * issue loops; 2 = read-only HBM sweep over 2 GiB in GB/s; 3 = dense TF32
 * tensor rate (tcgen05.mma kind::tf32 issue loop) in GFLOP/s, of which the
 * 3xTF32 fp32 path can deliver at most a third.  Synchronises the stream.  No counterpart in the reference. */
int32_t pgb200ProbePeak(void *stream, int32_t kind, double *out);

/* Exercises that path without any fault: launches one CTA that waits on a
 * barrier nothing ever signals, for at most `limit_cycles` SM cycles (clamped
 * to about one second), after which it records a code and returns.  A
 * following synchronise + pgb200PollDeviceStatus() must report
 * PGB200_ERR_TIMEOUT, and the context stays usable.  No counterpart in the
 * reference. */
int32_t pgb200SelfTestWaitTimeout(void *stream, int64_t limit_cycles);

/* How many of this library's kernels this thread has launched so far. */
int64_t pgb200LaunchCount(void);

/* Host-array drop-ins with the reference's own function names, argument order
 * and array extents (C99 prototypes of PolyBench: inner dimension = the size
 * argument).  Arrays are host memory, exactly what the C nests receive; each
 * call stages operands to the GPU, runs the contraction(s) and copies the
 * results back before returning.
 *   pgb200_kernel_gemm  <- kernel_gemm  gemm.c:88-115
 *   pgb200_kernel_2mm   <- kernel_2mm   2mm.c:92-121  (tmp is written too)
 *   pgb200_kernel_mvt   <- kernel_mvt   mvt.c:93-111
 *   pgb200_kernel_syrk  <- kernel_syrk  syrk.c:83-108
 * The `_f32` forms are the -DDATA_TYPE_IS_FLOAT builds of the same sources. */
int32_t pgb200_kernel_gemm(int ni, int nj, int nk, double alpha, double beta,
                           double *C, const double *A, const double *B);
int32_t pgb200_kernel_gemm_f32(int ni, int nj, int nk, float alpha, float beta,
                               float *C, const float *A, const float *B);
int32_t pgb200_kernel_2mm(int ni, int nj, int nk, int nl, double alpha,
                          double beta, double *tmp, const double *A,
                          const double *B, const double *C, double *D);
int32_t pgb200_kernel_mvt(int n, double *x1, double *x2, const double *y_1,
                          const double *y_2, const double *A);
int32_t pgb200_kernel_syrk(int n, int m, double alpha, double beta, double *C,
                           const double *A);
int32_t pgb200_kernel_syrk_f32(int n, int m, float alpha, float beta, float *C,
                               const float *A);
/* Same-shaped nests served by the same kernels:
 *   pgb200_kernel_3mm      <- kernel_3mm      kernels/3mm/3mm.c:87-127   (three GEMMs;
 *                             E and F are live-out like G)
 *   pgb200_kernel_atax     <- kernel_atax     kernels/atax/atax.c:80-102 (tmp = A x, then
 *                             y = A^T tmp: two passes, the second depends on the first)
 *   pgb200_kernel_bicg     <- kernel_bicg     kernels/bicg/bicg.c:86-111 (one fused pass)
 *   pgb200_kernel_gesummv  <- kernel_gesummv  blas/gesummv/gesummv.c:86-112 */
/*   pgb200_kernel_syr2k    <- kernel_syr2k    blas/syr2k/syr2k.c:84-112
 *   pgb200_kernel_gemver   <- kernel_gemver   blas/gemver/gemver.c:97-133 */
int32_t pgb200_kernel_gemver(int n, double alpha, double beta, double *A,
                             const double *u1, const double *v1, const double *u2,
                             const double *v2, double *w, double *x,
                             const double *y, const double *z);
int32_t pgb200_kernel_syr2k(int n, int m, double alpha, double beta, double *C,
                            const double *A, const double *B);
int32_t pgb200_kernel_syr2k_f32(int n, int m, float alpha, float beta, float *C,
                                const float *A, const float *B);
int32_t pgb200_kernel_3mm(int ni, int nj, int nk, int nl, int nm, double *E,
                          const double *A, const double *B, double *F,
                          const double *C, const double *D, double *G);
int32_t pgb200_kernel_atax(int m, int n, const double *A, const double *x,
                           double *y, double *tmp);
int32_t pgb200_kernel_bicg(int m, int n, const double *A, double *s, double *q,
                           const double *p, const double *r);
int32_t pgb200_kernel_gesummv(int n, double alpha, double beta, const double *A,
                              const double *B, double *tmp, const double *x,
                              double *y);
/*   pgb200_kernel_symm     <- kernel_symm     blas/symm/symm.c:89-120
 *   pgb200_kernel_trmm     <- kernel_trmm     blas/trmm/trmm.c:85-109
 *   pgb200_kernel_doitgen  <- kernel_doitgen  kernels/doitgen/doitgen.c:80-100 */
int32_t pgb200_kernel_symm(int m, int n, double alpha, double beta, double *C,
                           const double *A, const double *B);
int32_t pgb200_kernel_symm_f32(int m, int n, float alpha, float beta, float *C,
                               const float *A, const float *B);
int32_t pgb200_kernel_trmm(int m, int n, double alpha, const double *A, double *B);
int32_t pgb200_kernel_trmm_f32(int m, int n, float alpha, const float *A, float *B);
int32_t pgb200_kernel_doitgen(int nr, int nq, int np, double *A, const double *C4,
                              double *sum);

#ifdef __cplusplus
}
#endif
#endif /* PGB200_H */
