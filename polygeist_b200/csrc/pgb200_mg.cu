// Single-process multi-GPU entry points: one host thread drives the GPUs of one
// box, the output rows are partitioned across them and the shared operand is
// broadcast by NCCL over NVLink in K-slices, each slice's product (or rank-k
// update) running while the next slice is in flight.  The reference has no
// multi-GPU path; the split is exact because the rows of every nest are
// independent (gemm.c:104-113, syrk.c:97-106).
//
// NCCL is bound at run time (dlopen of libnccl.so.2), so the library itself has
// no link-time dependency on it; with one device no NCCL call is made at all.
#include <dlfcn.h>
#include <math.h>
#include <nccl.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <mutex>
#include <thread>
#include <vector>

#include "pgb200_internal.h"

namespace pgb200 {
namespace {

struct NcclApi {
  ncclResult_t (*CommInitAll)(ncclComm_t *, int, const int *) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
  // Optional (failure detection): absent from very old libraries.
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  bool ok = false;
};

// Host-side failure injection for tests: the table entries are replaced by
// stubs that report a failure without touching any GPU.
ncclResult_t failing_broadcast(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t,
                               cudaStream_t) {
  return ncclSystemError;
}
ncclResult_t failing_async_error(ncclComm_t, ncclResult_t *out) {
  *out = ncclSystemError;
  return ncclSuccess;
}

struct MgState {
  int ndev = 0;
  bool links_checked = false;  // this call's link streams have been drained (or found failed)
  bool comm_failed = false;    // a collective failed or is overdue: communicators to be aborted
  std::vector<ncclComm_t> comm;
  std::vector<cudaStream_t> compute, link;
};

std::mutex g_mg_mu;
NcclApi g_nccl;
MgState g_mg;

int32_t load_nccl() {
  if (g_nccl.ok) return PGB200_OK;
  void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) {
    set_error("multi-GPU entry: cannot load libnccl.so.2 (%s)", dlerror());
    return PGB200_ERR_NCCL;
  }
  g_nccl.CommInitAll = (decltype(g_nccl.CommInitAll))dlsym(h, "ncclCommInitAll");
  g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))dlsym(h, "ncclCommDestroy");
  g_nccl.Broadcast = (decltype(g_nccl.Broadcast))dlsym(h, "ncclBroadcast");
  g_nccl.GroupStart = (decltype(g_nccl.GroupStart))dlsym(h, "ncclGroupStart");
  g_nccl.GroupEnd = (decltype(g_nccl.GroupEnd))dlsym(h, "ncclGroupEnd");
  g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))dlsym(h, "ncclGetErrorString");
  if (!g_nccl.CommInitAll || !g_nccl.CommDestroy || !g_nccl.Broadcast || !g_nccl.GroupStart ||
      !g_nccl.GroupEnd || !g_nccl.GetErrorString) {
    set_error("multi-GPU entry: libnccl.so.2 lacks a required symbol");
    return PGB200_ERR_NCCL;
  }
  g_nccl.CommGetAsyncError =
      (decltype(g_nccl.CommGetAsyncError))dlsym(h, "ncclCommGetAsyncError");
  g_nccl.CommAbort = (decltype(g_nccl.CommAbort))dlsym(h, "ncclCommAbort");
  // PGB200_FAULT_NCCL=broadcast | async (read when the library is bound): every
  // broadcast call fails / every asynchronous-error poll reports a failure.
  if (const char *f = getenv("PGB200_FAULT_NCCL")) {
    if (!strcmp(f, "broadcast")) g_nccl.Broadcast = failing_broadcast;
    if (!strcmp(f, "async")) g_nccl.CommGetAsyncError = failing_async_error;
  }
  g_nccl.ok = true;
  return PGB200_OK;
}

// Releases the streams and communicators; `abort` after a failed or overdue
// collective (ncclCommAbort also ends kernels that still wait for a peer).
void mg_destroy(bool abort) {
  for (int d = 0; d < g_mg.ndev; d++) {
    cudaSetDevice(d);
    if (!g_mg.comm.empty() && g_mg.comm[d]) {
      if (abort && g_nccl.CommAbort)
        g_nccl.CommAbort(g_mg.comm[d]);
      else
        g_nccl.CommDestroy(g_mg.comm[d]);
    }
    if (g_mg.compute[d]) cudaStreamDestroy(g_mg.compute[d]);
    if (g_mg.link[d]) cudaStreamDestroy(g_mg.link[d]);
  }
  g_mg = MgState();
}

#define PGB_NCCL(expr)                                                             \
  do {                                                                             \
    ncclResult_t r__ = (expr);                                                     \
    if (r__ != ncclSuccess) {                                                      \
      set_error("'%s' failed with '%s'", #expr, g_nccl.GetErrorString(r__));       \
      return PGB200_ERR_NCCL;                                                      \
    }                                                                              \
  } while (0)

// Streams and (for ndev > 1) communicators for devices 0..ndev-1, created once.
int32_t mg_state(int ndev, MgState **out) {
  if (g_mg.ndev == ndev) {
    *out = &g_mg;
    return PGB200_OK;
  }
  int count = 0;
  PGB_CUDA(cudaGetDeviceCount(&count));
  PGB_REQUIRE(ndev >= 1 && ndev <= count, "multi-GPU entry: ndev = %d but %d device(s) visible",
              ndev, count);
  if (g_mg.ndev != 0) mg_destroy(false);  // different device count than last time: rebuild
  MgState st;
  st.compute.resize(ndev);
  st.link.resize(ndev);
  for (int d = 0; d < ndev; d++) {
    PGB_CUDA(cudaSetDevice(d));
    Runtime *rt = nullptr;
    PGB_TRY(get_runtime(&rt));
    PGB_CUDA(cudaStreamCreateWithFlags(&st.compute[d], cudaStreamNonBlocking));
    PGB_CUDA(cudaStreamCreateWithFlags(&st.link[d], cudaStreamNonBlocking));
  }
  // Direct peer copies (row blocks of device-resident operands travel over
  // NVLink instead of being staged through the host).
  for (int d = 0; d < ndev; d++) {
    PGB_CUDA(cudaSetDevice(d));
    for (int p = 0; p < ndev; p++) {
      if (p == d) continue;
      int can = 0;
      PGB_CUDA(cudaDeviceCanAccessPeer(&can, d, p));
      if (can) {
        cudaError_t e = cudaDeviceEnablePeerAccess(p, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
          return report_cuda(e, "cudaDeviceEnablePeerAccess");
        cudaGetLastError();
      }
    }
  }
  if (ndev > 1) {
    PGB_TRY(load_nccl());
    st.comm.resize(ndev);
    std::vector<int> devs(ndev);
    for (int d = 0; d < ndev; d++) devs[d] = d;
    PGB_NCCL(g_nccl.CommInitAll(st.comm.data(), ndev, devs.data()));
  }
  st.ndev = ndev;
  g_mg = st;
  *out = &g_mg;
  return PGB200_OK;
}

template <typename T>
ncclDataType_t nccl_type();
template <>
ncclDataType_t nccl_type<float>() { return ncclFloat; }
template <>
ncclDataType_t nccl_type<double>() { return ncclDouble; }

int64_t round_to(int64_t x, int64_t a) { return (x + a / 2) / a * a; }

// rows x cols elements between any two memories (host, this device, a peer):
// one linear copy when both sides are dense, a pitched copy otherwise.
template <typename T>
cudaError_t copy_block(T *dst, int64_t dst_ld, const T *src, int64_t src_ld, int64_t rows,
                       int64_t cols, cudaStream_t s) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  if (dst_ld == cols && src_ld == cols)
    return cudaMemcpyAsync(dst, src, (size_t)rows * cols * sizeof(T), cudaMemcpyDefault, s);
  return cudaMemcpy2DAsync(dst, dst_ld * sizeof(T), src, src_ld * sizeof(T), cols * sizeof(T), rows,
                           cudaMemcpyDefault, s);
}

// Broadcast rows [0, rows) x `pitch` elements of `bufs[d]` from device 0 to all.
template <typename T>
int32_t bcast(MgState *st, std::vector<T *> &bufs, size_t offset, size_t count) {
  PGB_NCCL(g_nccl.GroupStart());
  // A failing call must not leave the group open: close it, then report.
  ncclResult_t first = ncclSuccess;
  for (int d = 0; d < st->ndev && first == ncclSuccess; d++)
    first = g_nccl.Broadcast(bufs[0] + offset, bufs[d] + offset, count, nccl_type<T>(), 0,
                             st->comm[d], st->link[d]);
  const ncclResult_t end = g_nccl.GroupEnd();
  if (first == ncclSuccess) first = end;
  if (first != ncclSuccess) {
    set_error("'ncclBroadcast' failed with '%s'", g_nccl.GetErrorString(first));
    return PGB200_ERR_NCCL;
  }
  return PGB200_OK;
}

// Waits for the link stream of device d with a host deadline, polling the
// communicator's asynchronous error state meanwhile (a peer that died, a
// network error).  False: the collective failed or is overdue.
bool drain_link(MgState *st, int d) {
  static const double limit_s = [] {
    const char *e = getenv("PGB200_NCCL_TIMEOUT_S");
    const double v = e ? atof(e) : 0.0;
    return v > 0.0 ? v : 300.0;
  }();
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    if (!st->comm.empty() && g_nccl.CommGetAsyncError) {
      ncclResult_t r = ncclSuccess;
      if (g_nccl.CommGetAsyncError(st->comm[d], &r) != ncclSuccess ||
          (r != ncclSuccess && r != ncclInProgress)) {
        set_error("'ncclCommGetAsyncError' reported '%s' on device %d",
                  g_nccl.GetErrorString(r), d);
        return false;
      }
    }
    const cudaError_t q = cudaStreamQuery(st->link[d]);
    if (q == cudaSuccess) return true;
    if (q != cudaErrorNotReady) {
      report_cuda(q, "cudaStreamQuery(link stream)");
      return false;
    }
    const double el =
        std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (el > limit_s) {
      set_error("the broadcast on device %d did not finish within %.0f s", d, limit_s);
      return false;
    }
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

// Drains the link streams of all devices (once per call), polling for
// collective failures; false when a collective failed or is overdue.
bool mg_links_ok(MgState *st) {
  if (st->links_checked) return !st->comm_failed;
  st->links_checked = true;
  st->comm_failed = false;
  if (st->ndev > 1)
    for (int d = 0; d < st->ndev && !st->comm_failed; d++) {
      cudaSetDevice(d);
      if (!drain_link(st, d)) st->comm_failed = true;
    }
  return !st->comm_failed;
}

// Common exit of the multi-GPU entries, also taken after a failure: drain both
// streams of every device, release the scratch, destroy the events and make
// the caller's device current again.  Returns `status`, or the first error of
// the drain when `status` was PGB200_OK.
int32_t mg_release(MgState *st, int entry_dev, int32_t status,
                   const std::vector<std::vector<void *>> &bufs,
                   std::vector<std::vector<cudaEvent_t>> &ev) {
  cudaError_t drain = cudaSuccess;
  auto note = [&](cudaError_t e) {
    if (e != cudaSuccess && drain == cudaSuccess) drain = e;
  };
  // Link streams first: when a collective failed or is overdue the
  // communicators are aborted, which also ends kernels still waiting on a peer,
  // so the synchronisations below cannot hang.
  const bool comm_ok = mg_links_ok(st);
  st->links_checked = false;  // per call
  st->comm_failed = false;
  if (!comm_ok && status == PGB200_OK) status = PGB200_ERR_NCCL;
  if (!comm_ok && g_nccl.CommAbort) {
    for (int d = 0; d < st->ndev; d++) {
      cudaSetDevice(d);
      if (st->comm[d]) g_nccl.CommAbort(st->comm[d]);
      st->comm[d] = nullptr;
    }
  }
  for (int d = 0; d < st->ndev; d++) {
    note(cudaSetDevice(d));
    note(cudaStreamSynchronize(st->compute[d]));
    note(cudaStreamSynchronize(st->link[d]));
    Runtime *rt = nullptr;
    if (get_runtime(&rt) == PGB200_OK) {
      const int32_t dst = take_device_status(rt);
      if (status == PGB200_OK) status = dst;
    }
    for (void *p : bufs[d])
      if (p) note(cudaFreeAsync(p, st->compute[d]));
    for (auto e : ev[d])
      if (e) cudaEventDestroy(e);
    note(cudaStreamSynchronize(st->compute[d]));
  }
  if (!comm_ok) mg_destroy(false);  // communicators are gone: rebuilt by the next call
  note(cudaSetDevice(entry_dev));
  if (status == PGB200_OK && drain != cudaSuccess) return report_cuda(drain, "multi-GPU drain");
  return status;
}

// Before the results travel back: wait for every device's products and read
// its status word, so a kernel that gave up is reported instead of copied.
int32_t mg_products_done(MgState *st) {
  // A failed or overdue broadcast means the products ran on incomplete data.
  if (!mg_links_ok(st)) return PGB200_ERR_NCCL;
  int32_t status = PGB200_OK;
  for (int d = 0; d < st->ndev; d++) {
    PGB_CUDA(cudaSetDevice(d));
    PGB_CUDA(cudaStreamSynchronize(st->compute[d]));
    Runtime *rt = nullptr;
    PGB_TRY(get_runtime(&rt));
    const int32_t dst = take_device_status(rt);
    if (status == PGB200_OK) status = dst;
  }
  return status;
}

// Arrays in device-0 memory may still be being written by work the caller
// queued on its own streams; the entry's private non-blocking streams are not
// ordered after that work by anything else.
template <typename T>
int32_t mg_wait_for_caller(const T *a, const T *b, const T *c) {
  if (is_host_pointer(a) && is_host_pointer(b) && is_host_pointer(c)) return PGB200_OK;
  PGB_CUDA(cudaSetDevice(0));
  PGB_CUDA(cudaDeviceSynchronize());
  return PGB200_OK;
}

// C = alpha*A*B + beta*C, rows of A and C split over ndev GPUs, B broadcast in
// K-slices from device 0.  Arrays may be host memory or memory of device 0.
template <typename T>
int32_t gemm_mg(int ndev, int64_t M, int64_t N, int64_t K, T alpha, const T *A, int64_t lda,
                const T *B, int64_t ldb, T beta, T *C, int64_t ldc) {
  PGB_REQUIRE(M >= 0 && N >= 0 && K >= 0, "gemm (multi-GPU): negative size");
  if (M == 0 || N == 0) return PGB200_OK;
  PGB_REQUIRE(C && ldc >= N && (K == 0 || (A && B && lda >= K && ldb >= N)),
              "gemm (multi-GPU): null pointer or leading dimension too small");
  std::lock_guard<std::mutex> lk(g_mg_mu);
  int entry_dev = 0;
  PGB_CUDA(cudaGetDevice(&entry_dev));
  MgState *st = nullptr;
  PGB_TRY(mg_state(ndev, &st));
  const int64_t per16 = 16 / (int64_t)sizeof(T);
  const int64_t pA = (K + per16 - 1) / per16 * per16, pB = (N + per16 - 1) / per16 * per16;
  const int64_t pC = pB;
  std::vector<int64_t> b(ndev + 1, 0);
  for (int d = 1; d < ndev; d++) {
    int64_t x = round_to(M * d / ndev, 128);
    if (x > M) x = M;
    b[d] = x < b[d - 1] ? b[d - 1] : x;
  }
  b[ndev] = M;
  const int nslice = (ndev > 1 && K >= 2048) ? 8 : 1;
  std::vector<T *> dA(ndev, nullptr), dB(ndev, nullptr), dC(ndev, nullptr);
  std::vector<std::vector<cudaEvent_t>> ev(ndev);
  int32_t status = PGB200_OK;
  auto run = [&]() -> int32_t {
    PGB_TRY(mg_wait_for_caller<T>(A, B, C));
    if (is_host_pointer(A)) count_h2d((size_t)M * K * sizeof(T));
    if (is_host_pointer(B)) count_h2d((size_t)K * N * sizeof(T));
    if (is_host_pointer(C)) {
      if (beta != (T)0) count_h2d((size_t)M * N * sizeof(T));
      count_d2h((size_t)M * N * sizeof(T));
    }
    // Stage: every device takes its rows of A and C; device 0 takes B.
    for (int d = 0; d < ndev; d++) {
      PGB_CUDA(cudaSetDevice(d));
      const int64_t rows = b[d + 1] - b[d];
      cudaStream_t cs = st->compute[d];
      PGB_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&dB[d]), (size_t)(K > 0 ? K : 1) * pB * sizeof(T), st->link[d]));
      if (rows > 0) {
        PGB_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&dA[d]), (size_t)rows * pA * sizeof(T), cs));
        PGB_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&dC[d]), (size_t)rows * pC * sizeof(T), cs));
        PGB_CUDA(copy_block<T>(dA[d], pA, A + b[d] * lda, lda, rows, K, cs));
        if (beta != (T)0) PGB_CUDA(copy_block<T>(dC[d], pC, C + b[d] * ldc, ldc, rows, N, cs));
      }
      ev[d].resize(nslice);
      for (int c = 0; c < nslice; c++)
        PGB_CUDA(cudaEventCreateWithFlags(&ev[d][c], cudaEventDisableTiming));
    }
    PGB_CUDA(cudaSetDevice(0));
    PGB_CUDA(copy_block<T>(dB[0], pB, B, ldb, K, N, st->link[0]));
    // The receive buffers must exist before device 0 starts sending into them.
    for (int d = 0; d < ndev; d++) {
      PGB_CUDA(cudaSetDevice(d));
      PGB_CUDA(cudaStreamSynchronize(st->link[d]));
    }
    // K-slices: broadcast slice c (all of them queued up front on the link
    // streams), multiply slice c as soon as it has landed.
    std::vector<int64_t> kb(nslice + 1, 0);
    for (int c = 1; c < nslice; c++) kb[c] = round_to(K * c / nslice, 16);
    kb[nslice] = K;
    for (int c = 0; c < nslice && status == PGB200_OK; c++) {
      if (ndev > 1 && kb[c + 1] > kb[c])
        status = bcast<T>(st, dB, (size_t)kb[c] * pB, (size_t)(kb[c + 1] - kb[c]) * pB);
      for (int d = 0; d < ndev; d++) {
        PGB_CUDA(cudaSetDevice(d));
        PGB_CUDA(cudaEventRecord(ev[d][c], st->link[d]));
      }
    }
    for (int c = 0; c < nslice && status == PGB200_OK; c++) {
      for (int d = 0; d < ndev && status == PGB200_OK; d++) {
        const int64_t rows = b[d + 1] - b[d];
        if (rows == 0) continue;
        PGB_CUDA(cudaSetDevice(d));
        PGB_CUDA(cudaStreamWaitEvent(st->compute[d], ev[d][c], 0));
        if (kb[c + 1] == kb[c] && !(c == 0 && K == 0)) continue;
        status = gemm_device<T>(st->compute[d], rows, N, kb[c + 1] - kb[c], alpha, dA[d] + kb[c], pA,
                                dB[d] + kb[c] * pB, pB, false, c == 0 ? beta : (T)1, dC[d], pC,
                                false, 0);
      }
    }
    if (status == PGB200_OK) status = mg_products_done(st);
    for (int d = 0; d < ndev; d++) {
      PGB_CUDA(cudaSetDevice(d));
      const int64_t rows = b[d + 1] - b[d];
      if (rows > 0 && status == PGB200_OK)
        PGB_CUDA(copy_block<T>(C + b[d] * ldc, ldc, dC[d], pC, rows, N, st->compute[d]));
    }
    return status;
  };
  status = run();
  std::vector<std::vector<void *>> bufs(ndev);
  for (int d = 0; d < ndev; d++) bufs[d] = {dA[d], dB[d], dC[d]};
  return mg_release(st, entry_dev, status, bufs, ev);
}

// Lower triangle of C = alpha*A*A^T + beta*C, rows split by equal triangular
// area; A is broadcast as packed K-slices (columns [k0,k1) of all rows).
int32_t ssyrk_mg(int ndev, int64_t N, int64_t K, float alpha, const float *A, int64_t lda,
                 float beta, float *C, int64_t ldc) {
  PGB_REQUIRE(N >= 0 && K >= 0, "syrk (multi-GPU): negative size");
  if (N == 0) return PGB200_OK;
  PGB_REQUIRE(C && ldc >= N && (K == 0 || (A && lda >= K)),
              "syrk (multi-GPU): null pointer or leading dimension too small");
  std::lock_guard<std::mutex> lk(g_mg_mu);
  int entry_dev = 0;
  PGB_CUDA(cudaGetDevice(&entry_dev));
  MgState *st = nullptr;
  PGB_TRY(mg_state(ndev, &st));
  std::vector<int64_t> b(ndev + 1, 0);
  for (int d = 1; d < ndev; d++) {
    int64_t x = round_to((int64_t)llround((double)N * sqrt((double)d / ndev)), 128);
    if (x > N) x = N;
    b[d] = x < b[d - 1] ? b[d - 1] : x;
  }
  b[ndev] = N;
  const int nslice = (K >= 2048) ? 4 : 1;
  std::vector<int64_t> kb(nslice + 1, 0);
  for (int c = 1; c < nslice; c++) kb[c] = round_to(K * c / nslice, 16);
  kb[nslice] = K;
  const int64_t pC = (N + 3) / 4 * 4;
  std::vector<float *> dP(ndev, nullptr), dC(ndev, nullptr);
  std::vector<std::vector<cudaEvent_t>> ev(ndev);
  // Packed slices: slice c holds columns [kb[c],kb[c+1]) of all N rows, pitch wc.
  std::vector<size_t> off(nslice + 1, 0);
  for (int c = 0; c < nslice; c++) {
    const int64_t wc = (kb[c + 1] - kb[c] + 3) / 4 * 4;
    off[c + 1] = off[c] + (size_t)N * wc;
  }
  int32_t status = PGB200_OK;
  auto run = [&]() -> int32_t {
    PGB_TRY(mg_wait_for_caller<float>(A, A, C));
    if (is_host_pointer(A)) count_h2d((size_t)N * K * sizeof(float));
    if (is_host_pointer(C)) {
      count_h2d((size_t)N * N * sizeof(float));
      count_d2h((size_t)N * N * sizeof(float));
    }
    for (int d = 0; d < ndev; d++) {
      PGB_CUDA(cudaSetDevice(d));
      const int64_t rows = b[d + 1] - b[d];
      PGB_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&dP[d]), (off[nslice] ? off[nslice] : 4) * sizeof(float), st->link[d]));
      if (rows > 0) {
        PGB_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&dC[d]), (size_t)rows * pC * sizeof(float), st->compute[d]));
        PGB_CUDA(copy_block<float>(dC[d], pC, C + b[d] * ldc, ldc, rows, N, st->compute[d]));
      }
      ev[d].resize(nslice);
      for (int c = 0; c < nslice; c++)
        PGB_CUDA(cudaEventCreateWithFlags(&ev[d][c], cudaEventDisableTiming));
    }
    for (int d = 0; d < ndev; d++) {
      PGB_CUDA(cudaSetDevice(d));
      PGB_CUDA(cudaStreamSynchronize(st->link[d]));
    }
    for (int c = 0; c < nslice && status == PGB200_OK; c++) {
      const int64_t w = kb[c + 1] - kb[c], wc = (w + 3) / 4 * 4;
      PGB_CUDA(cudaSetDevice(0));
      if (w > 0)  // pack columns [kb[c],kb[c+1]) of A on device 0
        PGB_CUDA(copy_block<float>(dP[0] + off[c], wc, A + kb[c], lda, N, w, st->link[0]));
      if (ndev > 1 && w > 0) status = bcast<float>(st, dP, off[c], (size_t)N * wc);
      for (int d = 0; d < ndev; d++) {
        PGB_CUDA(cudaSetDevice(d));
        PGB_CUDA(cudaEventRecord(ev[d][c], st->link[d]));
      }
    }
    for (int c = 0; c < nslice && status == PGB200_OK; c++) {
      const int64_t w = kb[c + 1] - kb[c], wc = (w + 3) / 4 * 4;
      for (int d = 0; d < ndev && status == PGB200_OK; d++) {
        const int64_t r0 = b[d], r1 = b[d + 1];
        if (r1 == r0) continue;
        PGB_CUDA(cudaSetDevice(d));
        PGB_CUDA(cudaStreamWaitEvent(st->compute[d], ev[d][c], 0));
        if (w == 0 && !(c == 0 && K == 0)) continue;
        // Rows [r0,r1) against columns [0,r1): A_p * A[0:r1]^T masked to j <= i.
        status = gemm_device<float>(st->compute[d], r1 - r0, r1, w, alpha, dP[d] + off[c] + r0 * wc,
                                    wc, dP[d] + off[c], wc, true, c == 0 ? beta : 1.0f, dC[d], pC,
                                    true, r0);
      }
    }
    if (status == PGB200_OK) status = mg_products_done(st);
    for (int d = 0; d < ndev; d++) {
      PGB_CUDA(cudaSetDevice(d));
      const int64_t rows = b[d + 1] - b[d];
      if (rows > 0 && status == PGB200_OK)
        PGB_CUDA(copy_block<float>(C + b[d] * ldc, ldc, dC[d], pC, rows, N, st->compute[d]));
    }
    return status;
  };
  status = run();
  std::vector<std::vector<void *>> bufs(ndev);
  for (int d = 0; d < ndev; d++) bufs[d] = {dP[d], dC[d]};
  return mg_release(st, entry_dev, status, bufs, ev);
}

}  // namespace

void mg_shutdown() {
  std::lock_guard<std::mutex> lk(g_mg_mu);
  if (g_mg.ndev != 0) mg_destroy(false);
}

}  // namespace pgb200

using namespace pgb200;

extern "C" {

int32_t pgb200DgemmMg(int32_t ndev, int64_t M, int64_t N, int64_t K, double alpha, const double *A,
                      int64_t lda, const double *B, int64_t ldb, double beta, double *C,
                      int64_t ldc) {
  PGB_ENTRY(nullptr);
  return gemm_mg<double>(ndev, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}

int32_t pgb200SgemmMg(int32_t ndev, int64_t M, int64_t N, int64_t K, float alpha, const float *A,
                      int64_t lda, const float *B, int64_t ldb, float beta, float *C,
                      int64_t ldc) {
  PGB_ENTRY(nullptr);
  return gemm_mg<float>(ndev, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}

int32_t pgb200SsyrkMg(int32_t ndev, int64_t N, int64_t K, float alpha, const float *A, int64_t lda,
                      float beta, float *C, int64_t ldc) {
  PGB_ENTRY(nullptr);
  return ssyrk_mg(ndev, N, K, alpha, A, lda, beta, C, ldc);
}

}  // extern "C"
