// Host-array traffic for pageable memory.
//
// The arrays of the C loop nests come from malloc / posix_memalign
// (tools/cgeist/Test/polybench/utilities/polybench.c:519-525): pageable memory.
// A cudaMemcpyAsync from such memory is staged by the driver through its own
// bounce buffer by one host thread, blocks the caller, and reaches a fraction
// of the PCIe rate.  Here the staging is done by the library: a ring of
// page-locked slots per direction and device, filled (upload) or drained
// (download) by several host threads with plain memcpy while the copy engine
// moves the slots that are already full.  The row-block GEMM pipeline runs an
// uploader and a downloader thread on top of this, so uploads, products and
// downloads overlap for pageable arrays as they do for page-locked ones.
#include <string.h>

#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include "pgb200_internal.h"

namespace pgb200 {

namespace {

// ---------------------------------------------------------------------------
// A few persistent host threads that split a memcpy between them.
// ---------------------------------------------------------------------------
class CopyPool {
 public:
  static CopyPool &get() {
    static CopyPool pool;
    return pool;
  }
  // dst[0,bytes) = src[0,bytes), split over the workers; returns when done.
  void copy(void *dst, const void *src, size_t bytes) {
    const size_t min_part = size_t(1) << 20;
    size_t parts = workers_.size();
    if (bytes / min_part < parts) parts = bytes / min_part;
    if (parts <= 1) {
      memcpy(dst, src, bytes);
      return;
    }
    Job job;
    job.left = (int)parts;
    const size_t per = (bytes / parts + 4095) & ~size_t(4095);
    {
      std::lock_guard<std::mutex> lk(mu_);
      for (size_t p = 0; p < parts; p++) {
        const size_t off = p * per;
        const size_t n = off >= bytes ? 0 : (bytes - off < per ? bytes - off : per);
        tasks_.push_back(Task{static_cast<char *>(dst) + off, static_cast<const char *>(src) + off, n,
                              &job});
      }
    }
    cv_.notify_all();
    std::unique_lock<std::mutex> lk(job.mu);
    job.cv.wait(lk, [&] { return job.left == 0; });
  }

 private:
  struct Job {
    std::mutex mu;
    std::condition_variable cv;
    int left = 0;
  };
  struct Task {
    char *dst;
    const char *src;
    size_t bytes;
    Job *job;
  };
  CopyPool() {
    unsigned hw = std::thread::hardware_concurrency();
    int n = (int)(hw / 2);
    if (n < 2) n = 2;
    if (n > 8) n = 8;
    for (int i = 0; i < n; i++) workers_.emplace_back([this] { run(); });
  }
  ~CopyPool() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    for (auto &t : workers_) t.join();
  }
  void run() {
    for (;;) {
      Task t;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return stop_ || !tasks_.empty(); });
        if (tasks_.empty()) return;  // stop requested and nothing left
        t = tasks_.front();
        tasks_.pop_front();
      }
      if (t.bytes) memcpy(t.dst, t.src, t.bytes);
      std::lock_guard<std::mutex> lk(t.job->mu);
      if (--t.job->left == 0) t.job->cv.notify_all();
    }
  }
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<Task> tasks_;
  std::vector<std::thread> workers_;
  bool stop_ = false;
};

}  // namespace

// ---------------------------------------------------------------------------
// Page-locked ring of one direction on one device.
// ---------------------------------------------------------------------------
struct StageRing {
  static constexpr int SLOTS = 4;
  static constexpr size_t SLOT_BYTES = size_t(32) << 20;
  std::mutex mu;  // one transfer at a time per ring
  void *buf[SLOTS] = {};
  cudaEvent_t ev[SLOTS] = {};
  bool busy[SLOTS] = {};
  bool ready = false;

  int32_t init() {
    if (ready) return PGB200_OK;
    for (int i = 0; i < SLOTS; i++) {
      PGB_CUDA(cudaHostAlloc(&buf[i], SLOT_BYTES, cudaHostAllocDefault));
      PGB_CUDA(cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming));
    }
    ready = true;
    return PGB200_OK;
  }
  void release() {
    for (int i = 0; i < SLOTS; i++) {
      if (ev[i]) cudaEventDestroy(ev[i]);
      if (buf[i]) cudaFreeHost(buf[i]);
      ev[i] = nullptr;
      buf[i] = nullptr;
      busy[i] = false;
    }
    ready = false;
  }
};

StageRing *new_stage_ring() { return new StageRing(); }
void delete_stage_ring(StageRing *r) {
  if (!r) return;
  r->release();
  delete r;
}

bool is_pageable_host(const void *p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return true;
  }
  return a.type == cudaMemoryTypeUnregistered;
}

// dev[0,bytes) = host[0,bytes) on `stream`.  Returns once the host range has
// been read completely (the device copies may still be in flight on `stream`).
int32_t staged_upload(Runtime *rt, void *dev, const void *host, size_t bytes, cudaStream_t stream) {
  StageRing *ring = rt->ring_up;
  std::lock_guard<std::mutex> lk(ring->mu);
  PGB_TRY(ring->init());
  CopyPool &pool = CopyPool::get();
  int k = 0;
  for (size_t off = 0; off < bytes; off += StageRing::SLOT_BYTES, k = (k + 1) % StageRing::SLOTS) {
    const size_t n = bytes - off < StageRing::SLOT_BYTES ? bytes - off : StageRing::SLOT_BYTES;
    if (ring->busy[k]) PGB_CUDA(cudaEventSynchronize(ring->ev[k]));  // its last copy has left the slot
    pool.copy(ring->buf[k], static_cast<const char *>(host) + off, n);
    PGB_CUDA(cudaMemcpyAsync(static_cast<char *>(dev) + off, ring->buf[k], n, cudaMemcpyHostToDevice,
                             stream));
    PGB_CUDA(cudaEventRecord(ring->ev[k], stream));
    ring->busy[k] = true;
  }
  count_h2d(bytes);
  return PGB200_OK;
}

// host[0,bytes) = dev[0,bytes), ordered after the work already on `stream`.
// Returns when the host range is complete.
int32_t staged_download(Runtime *rt, void *host, const void *dev, size_t bytes,
                        cudaStream_t stream) {
  StageRing *ring = rt->ring_down;
  std::lock_guard<std::mutex> lk(ring->mu);
  PGB_TRY(ring->init());
  CopyPool &pool = CopyPool::get();
  const size_t chunks = (bytes + StageRing::SLOT_BYTES - 1) / StageRing::SLOT_BYTES;
  auto issue = [&](size_t c) -> int32_t {
    const int k = (int)(c % StageRing::SLOTS);
    const size_t off = c * StageRing::SLOT_BYTES;
    const size_t n = bytes - off < StageRing::SLOT_BYTES ? bytes - off : StageRing::SLOT_BYTES;
    PGB_CUDA(cudaMemcpyAsync(ring->buf[k], static_cast<const char *>(dev) + off, n,
                             cudaMemcpyDeviceToHost, stream));
    PGB_CUDA(cudaEventRecord(ring->ev[k], stream));
    return PGB200_OK;
  };
  // Keep SLOTS - 1 device copies in flight ahead of the slot being drained.
  size_t issued = 0;
  for (; issued < chunks && issued < (size_t)StageRing::SLOTS - 1; issued++) PGB_TRY(issue(issued));
  for (size_t c = 0; c < chunks; c++) {
    if (issued < chunks) PGB_TRY(issue(issued++));  // slot (c - 1) % SLOTS was drained last round
    const int k = (int)(c % StageRing::SLOTS);
    const size_t off = c * StageRing::SLOT_BYTES;
    const size_t n = bytes - off < StageRing::SLOT_BYTES ? bytes - off : StageRing::SLOT_BYTES;
    PGB_CUDA(cudaEventSynchronize(ring->ev[k]));
    pool.copy(static_cast<char *>(host) + off, ring->buf[k], n);
  }
  for (int i = 0; i < StageRing::SLOTS; i++) ring->busy[i] = false;
  count_d2h(bytes);
  return PGB200_OK;
}

}  // namespace pgb200
