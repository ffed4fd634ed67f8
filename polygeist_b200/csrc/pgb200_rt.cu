// libpgb200 runtime: life cycle, error reporting, pointer classification and
// staging, scratch memory, tensor-map encoding, the harness generator, and the
// exported C ABI that dispatches to the kernel families.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <condition_variable>
#include <map>
#include <mutex>
#include <thread>
#include <string>
#include <tuple>
#include <utility>

#include <algorithm>
#include <functional>
#include <queue>
#include <set>
#include <vector>

#include "pgb200_internal.h"

namespace pgb200 {

static thread_local char tls_error[512] = "";
static thread_local int32_t tls_path = PATH_NONE;
static thread_local int64_t tls_launches = 0;

static std::mutex g_mu;
static bool g_have_cfg = false;
static pgb200Config g_cfg = {};
static std::map<int, Runtime *> g_rt;  // per device
static std::atomic<int64_t> g_h2d{0}, g_d2h{0};

// pgb200Pin registry: host base address -> device copy.
struct PinEntry {
  size_t bytes = 0;
  void *dev = nullptr;
  int device = 0;
  bool written = false;  // a call wrote into the device copy since the last download
};
static std::mutex g_pin_mu;
static std::map<uintptr_t, PinEntry> g_pins;
static std::atomic<int> g_pin_count{0};
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tls_error, sizeof(tls_error), fmt, ap);
  va_end(ap);
  fprintf(stderr, "pgb200: %s\n", tls_error);
}

int32_t report_cuda(cudaError_t e, const char *expr) {
  snprintf(tls_error, sizeof(tls_error), "'%s' failed with '%s'", expr, cudaGetErrorName(e));
  fprintf(stderr, "%s\n", tls_error);
  return PGB200_ERR_CUDA;
}

int log_level() {
  // PGB200_LOG, read once, takes precedence over the configured level.
  static const int env = [] {
    const char *e = getenv("PGB200_LOG");
    return (e && *e) ? atoi(e) : -1;
  }();
  if (env >= 0) return env;
  return g_have_cfg ? g_cfg.log_level : 0;
}

void log_line(int level, const char *fmt, ...) {
  if (log_level() < level) return;
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  fprintf(stderr, "pgb200: %s\n", buf);
}

void count_h2d(size_t bytes) { g_h2d.fetch_add((int64_t)bytes, std::memory_order_relaxed); }
void count_d2h(size_t bytes) { g_d2h.fetch_add((int64_t)bytes, std::memory_order_relaxed); }

int32_t take_device_status(Runtime *rt) {
  const int32_t v = rt->status_host[0];
  if (v == 0) return PGB200_OK;
  const int32_t detail = rt->status_host[1];
  rt->status_host[0] = 0;
  rt->status_host[1] = 0;
  set_error("a device-side bounded wait expired (code %d, detail %d)", v, detail);
  return PGB200_ERR_TIMEOUT;
}

int32_t sync_check(Runtime *rt, cudaStream_t s) {
  PGB_CUDA(cudaStreamSynchronize(s));
  return take_device_status(rt);
}

// ---------------------------------------------------------------------------
// Per-call device timing (PGB200_PROFILE): a ring of event pairs; a pair is
// resolved into its entry's totals when its slot comes round again or at dump.
// ---------------------------------------------------------------------------
namespace {
constexpr int PROF_RING = 512;
struct ProfSlot {
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  int device = -1;
  const char *name = nullptr;
  bool pending = false;
};
struct ProfTotal {
  int64_t calls = 0;
  double ms = 0.0;
};
std::mutex g_prof_mu;
ProfSlot g_prof_ring[PROF_RING];
int64_t g_prof_next = 0;
std::map<std::string, ProfTotal> g_prof_totals;
std::atomic<int> g_prof_on{-1};  // -1: not decided yet (environment not read)
thread_local int tls_entry_depth = 0;

bool profile_on() {
  int v = g_prof_on.load(std::memory_order_relaxed);
  if (v < 0) {
    const char *e = getenv("PGB200_PROFILE");
    v = (e && *e && atoi(e) != 0) ? 1 : 0;
    g_prof_on.store(v, std::memory_order_relaxed);
  }
  return v == 1;
}

// Caller holds g_prof_mu.
void prof_resolve(ProfSlot &sl) {
  if (!sl.pending) return;
  sl.pending = false;
  float ms = 0.0f;
  if (cudaEventSynchronize(sl.e1) == cudaSuccess &&
      cudaEventElapsedTime(&ms, sl.e0, sl.e1) == cudaSuccess) {
    ProfTotal &t = g_prof_totals[sl.name];
    t.calls++;
    t.ms += ms;
  } else {
    cudaGetLastError();
  }
}
}  // namespace

void profile_enable(bool on) { g_prof_on.store(on ? 1 : 0, std::memory_order_relaxed); }

void profile_reset() {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (ProfSlot &sl : g_prof_ring) {
    if (sl.e0) cudaEventDestroy(sl.e0);
    if (sl.e1) cudaEventDestroy(sl.e1);
    sl = ProfSlot();
  }
  g_prof_totals.clear();
  g_prof_next = 0;
}

int32_t profile_dump(const char *path) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (ProfSlot &sl : g_prof_ring) prof_resolve(sl);
  FILE *f = path ? fopen(path, "a") : stderr;
  if (!f) {
    set_error("ProfileDump: cannot open '%s'", path);
    return PGB200_ERR_INVALID;
  }
  for (auto &kv : g_prof_totals)
    fprintf(f, "%s calls %lld total_ms %.6f mean_ms %.6f\n", kv.first.c_str(),
            (long long)kv.second.calls, kv.second.ms, kv.second.ms / (double)kv.second.calls);
  if (path) fclose(f);
  return PGB200_OK;
}

EntryScope::EntryScope(const char *n, void *st)
    : name(n), stream((cudaStream_t)st), slot(-1), outer(tls_entry_depth++ == 0) {
  if (!outer || !profile_on()) return;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  const int i = (int)(g_prof_next++ % PROF_RING);
  ProfSlot &sl = g_prof_ring[i];
  prof_resolve(sl);
  if (sl.device != dev) {  // events belong to the device they were created on
    if (sl.e0) cudaEventDestroy(sl.e0);
    if (sl.e1) cudaEventDestroy(sl.e1);
    sl.e0 = sl.e1 = nullptr;
    if (cudaEventCreate(&sl.e0) != cudaSuccess || cudaEventCreate(&sl.e1) != cudaSuccess) {
      cudaGetLastError();
      sl.device = -1;
      return;
    }
    sl.device = dev;
  }
  sl.name = name;
  if (cudaEventRecord(sl.e0, stream) == cudaSuccess) slot = i;
}

EntryScope::~EntryScope() {
  tls_entry_depth--;
  if (slot >= 0) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    ProfSlot &sl = g_prof_ring[slot];
    if (cudaEventRecord(sl.e1, stream) == cudaSuccess) sl.pending = true;
  }
  if (outer && log_level() >= 2) {
    static const char *const paths[] = {"none", "SIMT", "DMMA", "tcgen05 3xTF32", "HBM-streaming"};
    const int32_t pth = tls_path;
    log_line(2, "%s -> %s kernels, %lld launches by this thread so far", name,
             paths[(pth >= 0 && pth <= 4) ? pth : 0], (long long)tls_launches);
  }
}

bool registry_lookup(const void *p, void **dev, bool written) {
  if (g_pin_count.load(std::memory_order_acquire) == 0 || !p) return false;
  int cur = 0;
  if (cudaGetDevice(&cur) != cudaSuccess) return false;
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  std::lock_guard<std::mutex> lk(g_pin_mu);
  auto it = g_pins.upper_bound(a);
  if (it == g_pins.begin()) return false;
  --it;
  if (a >= it->first + it->second.bytes || it->second.device != cur) return false;
  *dev = static_cast<char *>(it->second.dev) + (a - it->first);
  if (written) it->second.written = true;
  return true;
}

void note_launch(Path p, int n) {
  tls_path = p;
  tls_launches += n;
}

int32_t get_runtime(Runtime **out) {
  int dev = 0;
  PGB_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_rt.find(dev);
  if (it != g_rt.end()) {
    *out = it->second;
    return PGB200_OK;
  }
  cudaDeviceProp prop;
  PGB_CUDA(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10) {
    set_error("device %d is sm_%d%d; libpgb200 kernels are built for sm_100a only", dev,
              prop.major, prop.minor);
    return PGB200_ERR_UNSUPPORTED;
  }
  {
    // Keep staging buffers of the host-array path cached in the stream-ordered
    // pool instead of returning them to the driver at every synchronisation.
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
      uint64_t keep = UINT64_MAX;
      cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    cudaGetLastError();
  }
  Runtime *rt = new Runtime();
  rt->cfg = g_cfg;
  rt->num_sms = prop.multiProcessorCount;
  rt->cc_major = prop.major;
  void *h = nullptr;
  PGB_CUDA(cudaHostAlloc(&h, sizeof(int32_t) * 4, cudaHostAllocMapped));
  memset(h, 0, sizeof(int32_t) * 4);
  rt->status_host = static_cast<volatile int32_t *>(h);
  void *d = nullptr;
  PGB_CUDA(cudaHostGetDevicePointer(&d, h, 0));
  rt->status_dev = static_cast<int32_t *>(d);
  PGB_CUDA(cudaStreamCreateWithFlags(&rt->copy_in, cudaStreamNonBlocking));
  PGB_CUDA(cudaStreamCreateWithFlags(&rt->copy_out, cudaStreamNonBlocking));
  rt->ring_up = new_stage_ring();
  rt->ring_down = new_stage_ring();
  if (!g_encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    PGB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (!fn || q != cudaDriverEntryPointSuccess) {
      set_error("cuTensorMapEncodeTiled is not available from this driver");
      return PGB200_ERR_UNSUPPORTED;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  g_rt[dev] = rt;
  *out = rt;
  log_line(1, "device %d: %s, %d SMs, runtime initialised", dev, prop.name, prop.multiProcessorCount);
  return PGB200_OK;
}

// ---------------------------------------------------------------------------
// Per-call scratch (see PoolBuffer in pgb200_internal.h).
// ---------------------------------------------------------------------------
namespace {
constexpr size_t SMALL_SCRATCH = size_t(64) << 20;
struct CachedBlock {
  void *ptr = nullptr;
  size_t bytes = 0;
  int device = 0;
};
// Every cached block is also listed here so that pgb200Shutdown can release the
// blocks of all threads; a thread notices through the epoch that its cache is gone.
std::mutex g_cache_mu;
std::vector<CachedBlock *> g_cache_all;
std::atomic<uint64_t> g_cache_epoch{1};
struct ThreadCache {
  uint64_t epoch = 0;
  int live = 0;  // cached holders alive in this thread = depth of the next one
  std::map<std::tuple<int, cudaStream_t, int>, CachedBlock *> blocks;
};
thread_local ThreadCache tls_cache;
}  // namespace

cudaError_t PoolBuffer::alloc(size_t bytes, cudaStream_t s) {
  stream = s;
  if (bytes == 0) bytes = 16;
  if (bytes > SMALL_SCRATCH) {
    owned = true;
    return cudaMallocAsync(&ptr, bytes, s);
  }
  owned = false;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const uint64_t epoch = g_cache_epoch.load(std::memory_order_acquire);
  if (tls_cache.epoch != epoch) {  // first use, or a shutdown released everything
    tls_cache.blocks.clear();
    tls_cache.epoch = epoch;
  }
  CachedBlock *&slot = tls_cache.blocks[std::make_tuple(dev, s, tls_cache.live)];
  if (!slot) {
    slot = new CachedBlock();
    slot->device = dev;
    std::lock_guard<std::mutex> lk(g_cache_mu);
    g_cache_all.push_back(slot);
  }
  if (slot->bytes < bytes) {
    // The old block may still be read by this thread's earlier calls on `s`:
    // release it in stream order.
    if (slot->ptr) cudaFreeAsync(slot->ptr, s);
    slot->ptr = nullptr;
    slot->bytes = 0;
    const size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    e = cudaMallocAsync(&slot->ptr, want, s);
    if (e != cudaSuccess) return e;
    slot->bytes = want;
  }
  ptr = slot->ptr;
  cached = true;
  tls_cache.live++;
  return cudaSuccess;
}

PoolBuffer::~PoolBuffer() {
  if (ptr && owned) cudaFreeAsync(ptr, stream);
  if (cached) tls_cache.live--;
}

static void release_cached_scratch() {
  std::lock_guard<std::mutex> lk(g_cache_mu);
  for (CachedBlock *b : g_cache_all) {
    if (b->ptr) {
      cudaSetDevice(b->device);
      cudaDeviceSynchronize();
      cudaFree(b->ptr);
    }
    delete b;
  }
  g_cache_all.clear();
  g_cache_epoch.fetch_add(1, std::memory_order_acq_rel);
}

int32_t encode_tensor_map(CUtensorMap *map, CUtensorMapDataType dtype, int rank,
                          const void *base, const uint64_t *dims,
                          const uint64_t *strides_bytes, const uint32_t *box,
                          CUtensorMapSwizzle swizzle) {
  cuuint64_t d[5], st[5];
  cuuint32_t b[5], es[5];
  for (int i = 0; i < rank; i++) {
    d[i] = dims[i];
    b[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) st[i] = strides_bytes[i];
  }
  CUresult r = g_encode(map, dtype, (cuuint32_t)rank, const_cast<void *>(base), d, st, b, es,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("'cuTensorMapEncodeTiled' failed with 'CUresult %d'", (int)r);
    return PGB200_ERR_CUDA;
  }
  return PGB200_OK;
}

static std::mutex g_attr_mu;
static std::set<std::pair<int, const void *>> g_attr_done;

int32_t ensure_dynamic_smem(const void *kernel, int bytes) {
  int dev = 0;
  PGB_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_attr_mu);
  if (g_attr_done.count({dev, kernel})) return PGB200_OK;
  PGB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  g_attr_done.insert({dev, kernel});
  return PGB200_OK;
}

bool build_lpt_schedule(const int64_t *cost, int64_t tiles, int workers, TileSchedule *out) {
  if (tiles < 0 || tiles > TileSchedule::MAX_TILES || workers < 1 ||
      workers > TileSchedule::MAX_WORKERS)
    return false;
  std::vector<int32_t> order((size_t)tiles);
  for (int64_t t = 0; t < tiles; t++) order[(size_t)t] = (int32_t)t;
  std::stable_sort(order.begin(), order.end(),
                   [&](int32_t a, int32_t b) { return cost[a] > cost[b]; });
  // Min-heap of (work so far, worker id).
  using Slot = std::pair<int64_t, int>;
  std::priority_queue<Slot, std::vector<Slot>, std::greater<Slot>> heap;
  for (int w = 0; w < workers; w++) heap.push({0, w});
  std::vector<std::vector<uint16_t>> mine((size_t)workers);
  for (int32_t t : order) {
    Slot top = heap.top();
    heap.pop();
    mine[(size_t)top.second].push_back((uint16_t)t);
    top.first += cost[t];
    heap.push(top);
  }
  int64_t n = 0;
  for (int w = 0; w < workers; w++) {
    out->off[w] = (uint16_t)n;
    for (uint16_t t : mine[(size_t)w]) out->idx[n++] = t;
  }
  for (int w = workers; w <= TileSchedule::MAX_WORKERS; w++) out->off[w] = (uint16_t)n;
  return true;
}

bool is_host_pointer(const void *p) {
  cudaPointerAttributes a;
  cudaError_t e = cudaPointerGetAttributes(&a, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return true;
  }
  return a.type == cudaMemoryTypeUnregistered || a.type == cudaMemoryTypeHost;
}

// Pageable arrays of at least this size travel through the page-locked rings.
static constexpr size_t STAGED_MIN_BYTES = size_t(64) << 20;

bool needs_staging(const void *p) {
  void *d = nullptr;
  return is_host_pointer(p) && !registry_lookup(p, &d, false);
}

template <typename T>
int32_t stage(cudaStream_t s, const T *p, int64_t rows, int64_t cols, int64_t ld, bool in,
              bool out, Staged<T> *st) {
  st->rows = rows;
  st->cols = cols;
  void *resident = nullptr;
  if (rows > 0 && cols > 0 && registry_lookup(p, &resident, out)) {
    // Inside a pgb200Pin range: the device copy is the array, same layout.
    st->dev = static_cast<T *>(resident);
    st->ld = ld;
    st->host = nullptr;
    return PGB200_OK;
  }
  if (rows == 0 || cols == 0 || !is_host_pointer(p)) {
    st->dev = const_cast<T *>(p);
    st->ld = ld;
    st->host = nullptr;
    return PGB200_OK;
  }
  st->host_ld = ld;
  st->copy_back = out;
  st->stream = s;
  // Pad the device pitch to 16 bytes so staged operands always meet the
  // alignment rules of the tensor-core paths.
  const int64_t per16 = 16 / (int64_t)sizeof(T);
  st->ld = (cols + per16 - 1) / per16 * per16;
  void *d = nullptr;
  PGB_CUDA(cudaMallocAsync(&d, (size_t)rows * st->ld * sizeof(T), s));
  st->dev = static_cast<T *>(d);
  st->host = const_cast<T *>(p);  // from here on the destructor owns the device copy
  if (in) {
    const size_t bytes = (size_t)rows * ld * sizeof(T);
    Runtime *rt = nullptr;
    if (st->ld == ld && bytes >= STAGED_MIN_BYTES && is_pageable_host(p) &&
        get_runtime(&rt) == PGB200_OK) {
      PGB_TRY(staged_upload(rt, st->dev, p, bytes, s));
      return PGB200_OK;  // counted by staged_upload
    }
    if (st->ld == ld)
      PGB_CUDA(cudaMemcpyAsync(st->dev, p, bytes, cudaMemcpyHostToDevice, s));
    else
      PGB_CUDA(cudaMemcpy2DAsync(st->dev, st->ld * sizeof(T), p, ld * sizeof(T), cols * sizeof(T),
                                 rows, cudaMemcpyHostToDevice, s));
    count_h2d((size_t)rows * cols * sizeof(T));
  }
  return PGB200_OK;
}

template <typename T>
int32_t finish(cudaStream_t s, Staged<T> *st) {
  if (!st->host) return PGB200_OK;
  if (st->copy_back) {
    const size_t bytes = (size_t)st->rows * st->ld * sizeof(T);
    Runtime *rt = nullptr;
    if (st->ld == st->host_ld && st->ld == st->cols && bytes >= STAGED_MIN_BYTES &&
        is_pageable_host(st->host) && get_runtime(&rt) == PGB200_OK) {
      PGB_TRY(staged_download(rt, st->host, st->dev, bytes, s));
      T *d = st->dev;
      st->host = nullptr;
      PGB_CUDA(cudaFreeAsync(d, s));
      return PGB200_OK;  // counted by staged_download
    }
    if (st->ld == st->host_ld && st->ld == st->cols)
      PGB_CUDA(cudaMemcpyAsync(st->host, st->dev, bytes, cudaMemcpyDeviceToHost, s));
    else
      PGB_CUDA(cudaMemcpy2DAsync(st->host, st->host_ld * sizeof(T), st->dev, st->ld * sizeof(T),
                                 st->cols * sizeof(T), st->rows, cudaMemcpyDeviceToHost, s));
    count_d2h((size_t)st->rows * st->cols * sizeof(T));
  }
  T *d = st->dev;
  st->host = nullptr;  // released below, whatever cudaFreeAsync answers
  PGB_CUDA(cudaFreeAsync(d, s));
  return PGB200_OK;
}

template int32_t stage<double>(cudaStream_t, const double *, int64_t, int64_t, int64_t, bool,
                               bool, Staged<double> *);
template int32_t stage<float>(cudaStream_t, const float *, int64_t, int64_t, int64_t, bool, bool,
                              Staged<float> *);
template int32_t finish<double>(cudaStream_t, Staged<double> *);
template int32_t finish<float>(cudaStream_t, Staged<float> *);

// ---------------------------------------------------------------------------
// Harness generator (see pgb200.h for the recurrence).
// ---------------------------------------------------------------------------
__host__ __device__ inline uint64_t splitmix64(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

__global__ void fill_f64_kernel(double *dst, int64_t row0, int64_t rows, int64_t cols,
                                int64_t ld, uint64_t h, double lo, double span) {
  const int64_t total = rows * cols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    const uint64_t x = splitmix64(h + (uint64_t)((row0 + r) * cols + c));
    const double u = __dmul_rn((double)(x >> 11), 0x1.0p-53);
    dst[r * ld + c] = __dadd_rn(lo, __dmul_rn(span, u));
  }
}

__global__ void fill_f32_kernel(float *dst, int64_t row0, int64_t rows, int64_t cols, int64_t ld,
                                uint64_t h, float lo, float span) {
  const int64_t total = rows * cols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    const uint64_t x = splitmix64(h + (uint64_t)((row0 + r) * cols + c));
    const float u = __fmul_rn((float)(uint32_t)(x >> 40), 0x1.0p-24f);
    dst[r * ld + c] = __fadd_rn(lo, __fmul_rn(span, u));
  }
}

static int fill_grid(int64_t total, int sms) {
  int64_t g = (total + 255) / 256;
  int64_t cap = (int64_t)sms * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace pgb200

using namespace pgb200;

// ===========================================================================
// Exported C ABI
// ===========================================================================
extern "C" {

int32_t pgb200Init(const pgb200Config *cfg) {
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (cfg) g_cfg = *cfg;
    g_have_cfg = true;
    for (auto &kv : g_rt) kv.second->cfg = g_cfg;
  }
  Runtime *rt = nullptr;
  return get_runtime(&rt);
}

int32_t pgb200Shutdown(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  int cur = 0;
  cudaGetDevice(&cur);
  if (const char *f = getenv("PGB200_PROFILE_FILE")) profile_dump(f);
  mg_shutdown();
  release_cached_scratch();
  profile_reset();
  {
    // Registered ranges that were never unpinned: their device copies go,
    // nothing is downloaded (pgb200Unpin is the call that brings data back).
    std::lock_guard<std::mutex> pl(g_pin_mu);
    for (auto &kv : g_pins) {
      cudaSetDevice(kv.second.device);
      cudaDeviceSynchronize();
      cudaFree(kv.second.dev);
    }
    g_pins.clear();
    g_pin_count.store(0, std::memory_order_release);
  }
  for (auto &kv : g_rt) {
    cudaSetDevice(kv.first);
    cudaDeviceSynchronize();
    cudaFreeHost(const_cast<int32_t *>(kv.second->status_host));
    cudaStreamDestroy(kv.second->copy_in);
    cudaStreamDestroy(kv.second->copy_out);
    delete_stage_ring(kv.second->ring_up);
    delete_stage_ring(kv.second->ring_down);
    delete kv.second;
  }
  g_rt.clear();
  {
    std::lock_guard<std::mutex> lk2(g_attr_mu);
    g_attr_done.clear();
  }
  cudaSetDevice(cur);
  return PGB200_OK;
}

const char *pgb200GetLastErrorString(void) { return tls_error; }
int32_t pgb200Version(void) { return 100; }
int32_t pgb200LastPath(void) { return tls_path; }
int64_t pgb200LaunchCount(void) { return tls_launches; }

int32_t pgb200PollDeviceStatus(void) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  return take_device_status(rt);
}

int32_t pgb200TransferCounters(int64_t *h2d_bytes, int64_t *d2h_bytes) {
  if (h2d_bytes) *h2d_bytes = g_h2d.load(std::memory_order_relaxed);
  if (d2h_bytes) *d2h_bytes = g_d2h.load(std::memory_order_relaxed);
  return PGB200_OK;
}

int32_t pgb200Pin(const void *host, uint64_t bytes) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(host && bytes > 0, "Pin: null pointer or empty range");
  PGB_REQUIRE(is_host_pointer(host), "Pin: the range must be host memory");
  const uintptr_t a = reinterpret_cast<uintptr_t>(host);
  int dev = 0;
  PGB_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lk(g_pin_mu);
    auto it = g_pins.upper_bound(a);
    const bool hits_next = it != g_pins.end() && it->first < a + bytes;
    bool hits_prev = false;
    if (it != g_pins.begin()) {
      auto pv = std::prev(it);
      hits_prev = a < pv->first + pv->second.bytes;
    }
    PGB_REQUIRE(!hits_next && !hits_prev, "Pin: the range overlaps a registered range");
  }
  PinEntry e;
  e.bytes = (size_t)bytes;
  e.device = dev;
  PGB_CUDA(cudaMalloc(&e.dev, e.bytes));
  if (e.bytes >= STAGED_MIN_BYTES && is_pageable_host(host)) {
    int32_t st = staged_upload(rt, e.dev, host, e.bytes, rt->copy_in);
    if (st == PGB200_OK && cudaStreamSynchronize(rt->copy_in) != cudaSuccess) st = PGB200_ERR_CUDA;
    if (st != PGB200_OK) {
      cudaFree(e.dev);
      return st;
    }
  } else {
    cudaError_t ce = cudaMemcpy(e.dev, host, e.bytes, cudaMemcpyHostToDevice);
    if (ce != cudaSuccess) {
      cudaFree(e.dev);
      return report_cuda(ce, "cudaMemcpy(Pin upload)");
    }
    count_h2d(e.bytes);
  }
  {
    std::lock_guard<std::mutex> lk(g_pin_mu);
    g_pins[a] = e;
    g_pin_count.store((int)g_pins.size(), std::memory_order_release);
  }
  log_line(1, "Pin %p: %llu bytes resident on device %d", host, (unsigned long long)bytes, dev);
  return PGB200_OK;
}

static int32_t pin_download(const void *host, bool release) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(host);
  PinEntry e;
  {
    std::lock_guard<std::mutex> lk(g_pin_mu);
    auto it = g_pins.find(a);
    PGB_REQUIRE(it != g_pins.end(), "%s: %p is not the start of a registered range",
                release ? "Unpin" : "PinSync", host);
    e = it->second;
    it->second.written = false;
    if (release) {
      g_pins.erase(it);
      g_pin_count.store((int)g_pins.size(), std::memory_order_release);
    }
  }
  int cur = 0;
  PGB_CUDA(cudaGetDevice(&cur));
  if (cur != e.device) PGB_CUDA(cudaSetDevice(e.device));
  int32_t st = PGB200_OK;
  cudaError_t ce = cudaDeviceSynchronize();  // every call that used the copy has finished
  if (ce == cudaSuccess) {
    Runtime *rt = nullptr;
    st = get_runtime(&rt);
    if (st == PGB200_OK) st = take_device_status(rt);
  }
  if (ce == cudaSuccess && st == PGB200_OK && e.written) {
    Runtime *rt = nullptr;
    if (e.bytes >= STAGED_MIN_BYTES && is_pageable_host(host) && get_runtime(&rt) == PGB200_OK) {
      st = staged_download(rt, const_cast<void *>(host), e.dev, e.bytes, rt->copy_out);
    } else {
      ce = cudaMemcpy(const_cast<void *>(host), e.dev, e.bytes, cudaMemcpyDeviceToHost);
      if (ce == cudaSuccess) count_d2h(e.bytes);
    }
  }
  if (release) cudaFree(e.dev);
  if (cur != e.device) cudaSetDevice(cur);
  if (ce != cudaSuccess) return report_cuda(ce, release ? "Unpin download" : "PinSync download");
  if (st == PGB200_OK)
    log_line(1, "%s %p: %s", release ? "Unpin" : "PinSync", host,
             e.written ? "downloaded" : "host copy was current");
  return st;
}

int32_t pgb200PinSync(const void *host) { return pin_download(host, false); }
int32_t pgb200Unpin(const void *host) { return pin_download(host, true); }

int32_t pgb200ProfileEnable(int32_t on) {
  profile_enable(on != 0);
  return PGB200_OK;
}
int32_t pgb200ProfileDump(const char *path) { return profile_dump(path); }

int32_t pgb200SelfTestWaitTimeout(void *stream, int64_t limit_cycles) {
  return wait_timeout_selftest((cudaStream_t)stream, (long long)limit_cycles);
}

int32_t pgb200FillUniformF64(void *stream, double *dst, int64_t row0, int64_t rows, int64_t cols,
                             int64_t ld, uint64_t seed, uint32_t array_id, double lo, double hi) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(dst && rows >= 0 && cols >= 0 && ld >= cols, "FillUniformF64: bad arguments");
  if (rows * cols == 0) return PGB200_OK;
  PGB_REQUIRE(!is_host_pointer(dst), "FillUniformF64: dst must be device memory");
  const uint64_t h = splitmix64(seed ^ ((uint64_t)array_id << 56));
  fill_f64_kernel<<<fill_grid(rows * cols, rt->num_sms), 256, 0, (cudaStream_t)stream>>>(
      dst, row0, rows, cols, ld, h, lo, hi - lo);
  note_launch(PATH_SIMT);
  PGB_CUDA(cudaGetLastError());
  return PGB200_OK;
}

int32_t pgb200FillUniformF32(void *stream, float *dst, int64_t row0, int64_t rows, int64_t cols,
                             int64_t ld, uint64_t seed, uint32_t array_id, float lo, float hi) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(dst && rows >= 0 && cols >= 0 && ld >= cols, "FillUniformF32: bad arguments");
  if (rows * cols == 0) return PGB200_OK;
  PGB_REQUIRE(!is_host_pointer(dst), "FillUniformF32: dst must be device memory");
  const uint64_t h = splitmix64(seed ^ ((uint64_t)array_id << 56));
  fill_f32_kernel<<<fill_grid(rows * cols, rt->num_sms), 256, 0, (cudaStream_t)stream>>>(
      dst, row0, rows, cols, ld, h, lo, hi - lo);
  note_launch(PATH_SIMT);
  PGB_CUDA(cudaGetLastError());
  return PGB200_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// GEMM / SYRK dispatch: validate, stage host operands, pick the kernel family.
// ---------------------------------------------------------------------------
namespace pgb200 {

static int32_t fast_gemm(cudaStream_t s, int64_t M, int64_t N, int64_t K, double alpha,
                         const double *A, int64_t lda, const double *B, int64_t ldb, bool transB,
                         double beta, double *C, int64_t ldc, bool lower, int64_t row0) {
  if (row0 != 0) return PGB200_ERR_UNSUPPORTED;
  return dmma_gemm(s, M, N, K, alpha, A, lda, B, ldb, transB, beta, C, ldc, lower);
}
static int32_t fast_gemm(cudaStream_t s, int64_t M, int64_t N, int64_t K, float alpha,
                         const float *A, int64_t lda, const float *B, int64_t ldb, bool transB,
                         float beta, float *C, int64_t ldc, bool lower, int64_t row0) {
  return tf32x3_gemm(s, M, N, K, alpha, A, lda, B, ldb, transB, beta, C, ldc, lower, row0);
}

// Device-pointer core shared by gemm and syrk.
template <typename T>
int32_t gemm_device(cudaStream_t s, int64_t M, int64_t N, int64_t K, T alpha, const T *A,
                           int64_t lda, const T *B, int64_t ldb, bool transB, T beta, T *C,
                           int64_t ldc, bool lower, int64_t row0) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  if (M == 0 || N == 0) return PGB200_OK;
  if (!rt->cfg.force_generic) {
    int32_t st = fast_gemm(s, M, N, K, alpha, A, lda, B, ldb, transB, beta, C, ldc, lower, row0);
    if (st != PGB200_ERR_UNSUPPORTED) return st;
  }
  return simt_gemm<T>(s, M, N, K, alpha, A, lda, B, ldb, transB, beta, C, ldc, lower, row0);
}

template int32_t gemm_device<double>(cudaStream_t, int64_t, int64_t, int64_t, double, const double *,
                                     int64_t, const double *, int64_t, bool, double, double *,
                                     int64_t, bool, int64_t);
template int32_t gemm_device<float>(cudaStream_t, int64_t, int64_t, int64_t, float, const float *,
                                    int64_t, const float *, int64_t, bool, float, float *, int64_t,
                                    bool, int64_t);

template <typename T>
static cudaError_t copy_rows(T *dst, int64_t dst_ld, const T *src, int64_t src_ld, int64_t rows,
                             int64_t cols, cudaMemcpyKind kind, cudaStream_t s) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  if (dst_ld == src_ld && (dst_ld == cols || rows == 1))
    return cudaMemcpyAsync(dst, src, (size_t)rows * cols * sizeof(T), kind, s);
  return cudaMemcpy2DAsync(dst, dst_ld * sizeof(T), src, src_ld * sizeof(T), cols * sizeof(T),
                           rows, kind, s);
}

// The same row-block pipeline for pageable arrays (malloc'd, what the C nests
// hold): an uploader thread stages B and then the blocks of A and C through the
// page-locked upload ring, the calling thread launches each block's product as
// soon as its rows are queued, and a downloader thread drains finished blocks
// through the download ring - three actors, so the host-side memcpy of one
// direction never holds up the other direction or the launches.  Needs dense
// arrays (leading dimension = row length, a multiple of 16 bytes).
template <typename T>
static int32_t gemm_host_staged(Runtime *rt, cudaStream_t s, int64_t M, int64_t N, int64_t K,
                                T alpha, const T *A, const T *B, T beta, T *C, bool transB) {
  const int64_t b_rows = transB ? N : K, b_cols = transB ? K : N;
  PoolBuffer bufA, bufB, bufC;
  PGB_CUDA(bufA.alloc((size_t)M * K * sizeof(T), s));
  PGB_CUDA(bufB.alloc((size_t)b_rows * b_cols * sizeof(T), s));
  PGB_CUDA(bufC.alloc((size_t)M * N * sizeof(T), s));
  T *dA = bufA.as<T>(), *dB = bufB.as<T>(), *dC = bufC.as<T>();
  constexpr int MAXB = 32;
  int nb = (int)(M / 512);
  if (nb > MAXB) nb = MAXB;
  if (nb < 1) nb = 1;
  const int64_t rows_per = ((M + nb - 1) / nb + 127) / 128 * 128;
  nb = (int)((M + rows_per - 1) / rows_per);
  int dev = 0;
  PGB_CUDA(cudaGetDevice(&dev));
  std::vector<cudaEvent_t> ev((size_t)2 * nb + 1, nullptr);
  std::mutex mu;
  std::condition_variable cv;
  int uploaded = 0, computed = 0;  // blocks whose copies are queued / whose product is queued
  int32_t up_st = PGB200_OK, down_st = PGB200_OK, main_st = PGB200_OK;
  bool stop = false;
  auto block = [&](int i, int64_t *r0, int64_t *rows) {
    *r0 = i * rows_per;
    *rows = (M - *r0 < rows_per) ? (M - *r0) : rows_per;
  };
  auto fail = [&](int32_t *slot, int32_t st) {
    std::lock_guard<std::mutex> lk(mu);
    *slot = st;
    stop = true;
    cv.notify_all();
  };
  auto run = [&]() -> int32_t {
    for (auto &e : ev) PGB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    cudaEvent_t ev_start = ev[0], *ev_in = ev.data() + 1, *ev_c = ev.data() + 1 + nb;
    PGB_CUDA(cudaEventRecord(ev_start, s));  // buffers exist, earlier work on s is done
    PGB_CUDA(cudaStreamWaitEvent(rt->copy_in, ev_start, 0));
    PGB_CUDA(cudaStreamWaitEvent(rt->copy_out, ev_start, 0));
    std::thread uploader([&] {
      if (cudaSetDevice(dev) != cudaSuccess) return fail(&up_st, PGB200_ERR_CUDA);
      int32_t st = staged_upload(rt, dB, B, (size_t)b_rows * b_cols * sizeof(T), rt->copy_in);
      for (int i = 0; i < nb && st == PGB200_OK; i++) {
        int64_t r0, rows;
        block(i, &r0, &rows);
        st = staged_upload(rt, dA + r0 * K, A + r0 * K, (size_t)rows * K * sizeof(T), rt->copy_in);
        if (st == PGB200_OK && beta != (T)0)
          st = staged_upload(rt, dC + r0 * N, C + r0 * N, (size_t)rows * N * sizeof(T), rt->copy_in);
        if (st == PGB200_OK && cudaEventRecord(ev_in[i], rt->copy_in) != cudaSuccess)
          st = PGB200_ERR_CUDA;
        if (st != PGB200_OK) break;
        std::lock_guard<std::mutex> lk(mu);
        if (stop) return;
        uploaded = i + 1;
        cv.notify_all();
      }
      if (st != PGB200_OK) fail(&up_st, st);
    });
    std::thread downloader([&] {
      if (cudaSetDevice(dev) != cudaSuccess) return fail(&down_st, PGB200_ERR_CUDA);
      for (int i = 0; i < nb; i++) {
        {
          std::unique_lock<std::mutex> lk(mu);
          cv.wait(lk, [&] { return stop || computed > i; });
          if (computed <= i) return;  // stopped before this block's product was queued
        }
        int64_t r0, rows;
        block(i, &r0, &rows);
        int32_t st = PGB200_OK;
        if (cudaStreamWaitEvent(rt->copy_out, ev_c[i], 0) != cudaSuccess) st = PGB200_ERR_CUDA;
        if (st == PGB200_OK)
          st = staged_download(rt, C + r0 * N, dC + r0 * N, (size_t)rows * N * sizeof(T),
                               rt->copy_out);
        if (st != PGB200_OK) return fail(&down_st, st);
      }
    });
    for (int i = 0; i < nb; i++) {
      {
        std::unique_lock<std::mutex> lk(mu);
        cv.wait(lk, [&] { return stop || uploaded > i; });
        if (uploaded <= i) break;
      }
      int64_t r0, rows;
      block(i, &r0, &rows);
      int32_t st = PGB200_OK;
      if (cudaStreamWaitEvent(s, ev_in[i], 0) != cudaSuccess) st = PGB200_ERR_CUDA;
      if (st == PGB200_OK)
        st = gemm_device<T>(s, rows, N, K, alpha, dA + r0 * K, K, dB, b_cols, transB, beta,
                            dC + r0 * N, N, false, 0);
      if (st == PGB200_OK && cudaEventRecord(ev_c[i], s) != cudaSuccess) st = PGB200_ERR_CUDA;
      if (st != PGB200_OK) {
        fail(&main_st, st);
        break;
      }
      std::lock_guard<std::mutex> lk(mu);
      computed = i + 1;
      cv.notify_all();
    }
    {
      // Whatever happened, let the helpers run out and collect them.
      std::lock_guard<std::mutex> lk(mu);
      if (main_st != PGB200_OK || up_st != PGB200_OK) stop = true;
      cv.notify_all();
    }
    uploader.join();
    downloader.join();
    if (main_st != PGB200_OK) return main_st;
    if (up_st != PGB200_OK || down_st != PGB200_OK) {
      set_error("host-array pipeline: the %s thread failed (status %d)",
                up_st != PGB200_OK ? "upload" : "download", up_st != PGB200_OK ? up_st : down_st);
      return up_st != PGB200_OK ? up_st : down_st;
    }
    return PGB200_OK;
  };
  const int32_t st = run();
  const cudaError_t e1 = cudaStreamSynchronize(rt->copy_in);
  const cudaError_t e2 = cudaStreamSynchronize(rt->copy_out);
  const cudaError_t e3 = cudaStreamSynchronize(s);
  for (auto e : ev)
    if (e) cudaEventDestroy(e);
  if (st != PGB200_OK) return st;
  PGB_CUDA(e1);
  PGB_CUDA(e2);
  PGB_CUDA(e3);
  // Row blocks are downloaded as they finish, so a block whose kernel gave up
  // may already be in C: the status tells the caller that C is not valid.
  return take_device_status(rt);
}

// Host-array GEMM for large problems: the rows of A and C travel in blocks, so
// that block i+1 is uploaded and block i-1 downloaded (PCIe is full duplex)
// while block i is being multiplied.  B goes first, whole.  The result is what
// the plain staged path gives; only the schedule differs.
template <typename T>
static int32_t gemm_host_pipelined(Runtime *rt, cudaStream_t s, int64_t M, int64_t N, int64_t K,
                                   T alpha, const T *A, int64_t lda, const T *B, int64_t ldb,
                                   T beta, T *C, int64_t ldc, bool transB) {
  const int64_t per16 = 16 / (int64_t)sizeof(T);
  auto pad = [&](int64_t c) { return (c + per16 - 1) / per16 * per16; };
  const int64_t b_rows = transB ? N : K, b_cols = transB ? K : N;
  const int64_t dlda = pad(K), dldb = pad(b_cols), dldc = pad(N);
  PoolBuffer bufA, bufB, bufC;
  PGB_CUDA(bufA.alloc((size_t)M * dlda * sizeof(T), s));
  PGB_CUDA(bufB.alloc((size_t)b_rows * dldb * sizeof(T), s));
  PGB_CUDA(bufC.alloc((size_t)M * dldc * sizeof(T), s));
  T *dA = bufA.as<T>(), *dB = bufB.as<T>(), *dC = bufC.as<T>();
  constexpr int MAXB = 16;
  int nb = (int)(M / 512);
  if (nb > MAXB) nb = MAXB;
  if (nb < 1) nb = 1;
  int64_t rows_per = ((M + nb - 1) / nb + 127) / 128 * 128;
  nb = (int)((M + rows_per - 1) / rows_per);
  cudaEvent_t ev[2 * MAXB + 2] = {};
  int nev = 0;
  // The pipeline proper; any failure falls through to the common exit below,
  // which drains the side streams before the buffers and events go away.
  auto run = [&]() -> int32_t {
    for (; nev < 2 * nb + 2; nev++)
      PGB_CUDA(cudaEventCreateWithFlags(&ev[nev], cudaEventDisableTiming));
    cudaEvent_t ev_start = ev[0], ev_done = ev[1], *ev_in = ev + 2, *ev_c = ev + 2 + nb;
    PGB_CUDA(cudaEventRecord(ev_start, s));  // buffers exist, earlier work on s is done
    PGB_CUDA(cudaStreamWaitEvent(rt->copy_in, ev_start, 0));
    PGB_CUDA(cudaStreamWaitEvent(rt->copy_out, ev_start, 0));
    PGB_CUDA(copy_rows(dB, dldb, B, ldb, b_rows, b_cols, cudaMemcpyHostToDevice, rt->copy_in));
    count_h2d((size_t)(b_rows * b_cols + M * K + (beta != (T)0 ? M * N : 0)) * sizeof(T));
    count_d2h((size_t)M * N * sizeof(T));
    for (int i = 0; i < nb; i++) {
      const int64_t r0 = i * rows_per, rows = (M - r0 < rows_per) ? (M - r0) : rows_per;
      PGB_CUDA(copy_rows(dA + r0 * dlda, dlda, A + r0 * lda, lda, rows, K, cudaMemcpyHostToDevice,
                         rt->copy_in));
      if (beta != (T)0)
        PGB_CUDA(copy_rows(dC + r0 * dldc, dldc, C + r0 * ldc, ldc, rows, N, cudaMemcpyHostToDevice,
                           rt->copy_in));
      PGB_CUDA(cudaEventRecord(ev_in[i], rt->copy_in));
    }
    for (int i = 0; i < nb; i++) {
      const int64_t r0 = i * rows_per, rows = (M - r0 < rows_per) ? (M - r0) : rows_per;
      PGB_CUDA(cudaStreamWaitEvent(s, ev_in[i], 0));
      // A block whose product failed is not copied back.
      PGB_TRY(gemm_device<T>(s, rows, N, K, alpha, dA + r0 * dlda, dlda, dB, dldb, transB, beta,
                             dC + r0 * dldc, dldc, false, 0));
      PGB_CUDA(cudaEventRecord(ev_c[i], s));
      PGB_CUDA(cudaStreamWaitEvent(rt->copy_out, ev_c[i], 0));
      PGB_CUDA(copy_rows(C + r0 * ldc, ldc, dC + r0 * dldc, dldc, rows, N, cudaMemcpyDeviceToHost,
                         rt->copy_out));
    }
    PGB_CUDA(cudaEventRecord(ev_done, rt->copy_out));
    PGB_CUDA(cudaStreamWaitEvent(s, ev_done, 0));
    return PGB200_OK;
  };
  const int32_t st = run();
  const cudaError_t e1 = cudaStreamSynchronize(rt->copy_in);
  const cudaError_t e2 = cudaStreamSynchronize(rt->copy_out);
  const cudaError_t e3 = cudaStreamSynchronize(s);
  for (int i = 0; i < nev; i++) cudaEventDestroy(ev[i]);
  if (st != PGB200_OK) return st;
  PGB_CUDA(e1);
  PGB_CUDA(e2);
  PGB_CUDA(e3);
  // Row blocks are downloaded as they finish, so a block whose kernel gave up
  // may already be in C: the status tells the caller that C is not valid.
  return take_device_status(rt);
}

template <typename T>
static int32_t gemm_entry(void *stream, int64_t M, int64_t N, int64_t K, T alpha, const T *A,
                          int64_t lda, const T *B, int64_t ldb, T beta, T *C, int64_t ldc,
                          bool transB = false) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(M >= 0 && N >= 0 && K >= 0, "gemm: negative size (M=%lld N=%lld K=%lld)",
              (long long)M, (long long)N, (long long)K);
  if (M == 0 || N == 0) return PGB200_OK;
  PGB_REQUIRE(C && ldc >= N, "gemm: C is null or ldc (%lld) < N (%lld)", (long long)ldc,
              (long long)N);
  PGB_REQUIRE(K == 0 || (A && B && lda >= K && ldb >= (transB ? K : N)),
              "gemm: A/B null or lda (%lld) < K (%lld) or ldb (%lld) too small for N (%lld)",
              (long long)lda, (long long)K, (long long)ldb, (long long)N);
  cudaStream_t s = (cudaStream_t)stream;
  if (K > 0 && M >= 1024 && (double)M * (double)N * (double)K >= 1e9 && needs_staging(A) &&
      needs_staging(B) && needs_staging(C)) {
    const int64_t per16 = 16 / (int64_t)sizeof(T), b_cols = transB ? K : N;
    const bool dense = lda == K && ldb == b_cols && ldc == N && K % per16 == 0 && N % per16 == 0;
    if (dense && is_pageable_host(A) && is_pageable_host(B) && is_pageable_host(C))
      return gemm_host_staged<T>(rt, s, M, N, K, alpha, A, B, beta, C, transB);
    return gemm_host_pipelined<T>(rt, s, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, transB);
  }
  Staged<T> sa, sb, sc;
  PGB_TRY(stage<T>(s, A, M, K, lda, true, false, &sa));
  if (transB)
    PGB_TRY(stage<T>(s, B, N, K, ldb, true, false, &sb));
  else
    PGB_TRY(stage<T>(s, B, K, N, ldb, true, false, &sb));
  PGB_TRY(stage<T>(s, C, M, N, ldc, beta != (T)0, true, &sc));
  const bool staged = sa.host || sb.host || sc.host;
  int32_t st = gemm_device<T>(s, M, N, K, alpha, sa.dev, sa.ld, sb.dev, sb.ld, transB, beta,
                              sc.dev, sc.ld, false, 0);
  if (st != PGB200_OK) return st;  // staged copies are released, nothing is copied back
  if (staged) PGB_TRY(sync_check(rt, s));  // a kernel that gave up: nothing is copied back either
  PGB_TRY(finish(s, &sa));
  PGB_TRY(finish(s, &sb));
  PGB_TRY(finish(s, &sc));
  if (staged) PGB_CUDA(cudaStreamSynchronize(s));
  return st;
}

template <typename T>
static int32_t syrk_entry(void *stream, int64_t N, int64_t K, int64_t row0, int64_t row1, T alpha,
                          const T *A, int64_t lda, T beta, T *C, int64_t ldc) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(N >= 0 && K >= 0 && row0 >= 0 && row0 <= row1 && row1 <= N,
              "syrk: bad sizes (N=%lld K=%lld rows [%lld,%lld))", (long long)N, (long long)K,
              (long long)row0, (long long)row1);
  if (row1 == row0) return PGB200_OK;
  PGB_REQUIRE(C && ldc >= N, "syrk: C is null or ldc (%lld) < N (%lld)", (long long)ldc,
              (long long)N);
  PGB_REQUIRE(K == 0 || (A && lda >= K), "syrk: A is null or lda (%lld) < K (%lld)",
              (long long)lda, (long long)K);
  cudaStream_t s = (cudaStream_t)stream;
  Staged<T> sa, sc;
  PGB_TRY(stage<T>(s, A, row1, K, lda, true, false, &sa));
  // The whole row block of C travels both ways; its strict upper triangle is
  // never touched on the device, so it comes back unchanged.
  PGB_TRY(stage<T>(s, C + row0 * ldc, row1 - row0, N, ldc, true, true, &sc));
  const bool staged = sa.host || sc.host;
  // Rows [row0,row1) of C against columns [0,row1): an (row1-row0) x row1
  // product A[row0:row1,:] * A[0:row1,:]^T masked to j <= i.
  int32_t st = gemm_device<T>(s, row1 - row0, row1, K, alpha, sa.dev + row0 * sa.ld, sa.ld,
                              sa.dev, sa.ld, true, beta, sc.dev, sc.ld, true, row0);
  if (st != PGB200_OK) return st;  // staged copies are released, nothing is copied back
  if (staged) PGB_TRY(sync_check(rt, s));  // a kernel that gave up: nothing is copied back either
  PGB_TRY(finish(s, &sa));
  PGB_TRY(finish(s, &sc));
  if (staged) PGB_CUDA(cudaStreamSynchronize(s));
  return st;
}

// Lower triangle of C = alpha*(A*B^T + B*A^T) + beta*C: two masked NT products.
template <typename T>
static int32_t syr2k_entry(void *stream, int64_t N, int64_t K, T alpha, const T *A, int64_t lda,
                           const T *B, int64_t ldb, T beta, T *C, int64_t ldc) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(N >= 0 && K >= 0, "syr2k: negative size");
  if (N == 0) return PGB200_OK;
  PGB_REQUIRE(C && ldc >= N, "syr2k: C is null or ldc (%lld) < N (%lld)", (long long)ldc,
              (long long)N);
  PGB_REQUIRE(K == 0 || (A && B && lda >= K && ldb >= K), "syr2k: A/B null or lda/ldb < K (%lld)",
              (long long)K);
  cudaStream_t s = (cudaStream_t)stream;
  Staged<T> sa, sb, sc;
  PGB_TRY(stage<T>(s, A, N, K, lda, true, false, &sa));
  PGB_TRY(stage<T>(s, B, N, K, ldb, true, false, &sb));
  PGB_TRY(stage<T>(s, C, N, N, ldc, true, true, &sc));
  const bool staged = sa.host || sb.host || sc.host;
  int32_t st = gemm_device<T>(s, N, N, K, alpha, sb.dev, sb.ld, sa.dev, sa.ld, true, beta, sc.dev,
                              sc.ld, true, 0);
  if (st == PGB200_OK)
    st = gemm_device<T>(s, N, N, K, alpha, sa.dev, sa.ld, sb.dev, sb.ld, true, (T)1, sc.dev, sc.ld,
                        true, 0);
  if (st != PGB200_OK) return st;  // staged copies are released, nothing is copied back
  if (staged) PGB_TRY(sync_check(rt, s));  // a kernel that gave up: nothing is copied back either
  PGB_TRY(finish(s, &sa));
  PGB_TRY(finish(s, &sb));
  PGB_TRY(finish(s, &sc));
  if (staged) PGB_CUDA(cudaStreamSynchronize(s));
  return st;
}

static int32_t matvec_entry(void *stream, int64_t M, int64_t N, const double *A, int64_t lda,
                            double alpha, double beta, const double *x1, double *y1,
                            const double *x2, double *y2) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(M >= 0 && N >= 0, "matvec: negative size");
  PGB_REQUIRE(M == 0 || N == 0 || (A && lda >= N), "matvec: A is null or lda (%lld) < N (%lld)",
              (long long)lda, (long long)N);
  PGB_REQUIRE((!y1 || x1 || N == 0) && (!y2 || x2 || M == 0), "matvec: null vector");
  cudaStream_t s = (cudaStream_t)stream;
  Staged<double> sa, sx1, sy1, sx2, sy2;
  PGB_TRY(stage<double>(s, A, M, N, lda, true, false, &sa));
  if (y1) {
    PGB_TRY(stage<double>(s, x1, 1, N, N, true, false, &sx1));
    PGB_TRY(stage<double>(s, y1, 1, M, M, beta != 0.0, true, &sy1));
  }
  if (y2) {
    PGB_TRY(stage<double>(s, x2, 1, M, M, true, false, &sx2));
    PGB_TRY(stage<double>(s, y2, 1, N, N, beta != 0.0, true, &sy2));
  }
  const bool staged = sa.host || sx1.host || sy1.host || sx2.host || sy2.host;
  int32_t st = stream_matvec(s, M, N, sa.dev, sa.ld, alpha, beta, y1 ? sx1.dev : nullptr,
                             y1 ? sy1.dev : nullptr, y2 ? sx2.dev : nullptr,
                             y2 ? sy2.dev : nullptr);
  if (st != PGB200_OK) return st;  // staged copies are released, nothing is copied back
  if (staged) PGB_TRY(sync_check(rt, s));  // a kernel that gave up: nothing is copied back either
  PGB_TRY(finish(s, &sa));
  PGB_TRY(finish(s, &sx1));
  PGB_TRY(finish(s, &sy1));
  PGB_TRY(finish(s, &sx2));
  PGB_TRY(finish(s, &sy2));
  if (staged) PGB_CUDA(cudaStreamSynchronize(s));
  return st;
}

}  // namespace pgb200

extern "C" {

int32_t pgb200Dgemm(void *stream, int64_t M, int64_t N, int64_t K, double alpha, const double *A,
                    int64_t lda, const double *B, int64_t ldb, double beta, double *C,
                    int64_t ldc) {
  PGB_ENTRY(stream);
  return gemm_entry<double>(stream, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}

int32_t pgb200Sgemm(void *stream, int64_t M, int64_t N, int64_t K, float alpha, const float *A,
                    int64_t lda, const float *B, int64_t ldb, float beta, float *C, int64_t ldc) {
  PGB_ENTRY(stream);
  return gemm_entry<float>(stream, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}

int32_t pgb200DgemmNT(void *stream, int64_t M, int64_t N, int64_t K, double alpha,
                      const double *A, int64_t lda, const double *B, int64_t ldb, double beta,
                      double *C, int64_t ldc) {
  PGB_ENTRY(stream);
  return gemm_entry<double>(stream, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, true);
}

int32_t pgb200SgemmNT(void *stream, int64_t M, int64_t N, int64_t K, float alpha, const float *A,
                      int64_t lda, const float *B, int64_t ldb, float beta, float *C,
                      int64_t ldc) {
  PGB_ENTRY(stream);
  return gemm_entry<float>(stream, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, true);
}

int32_t pgb200Dsyr2k(void *stream, int64_t N, int64_t K, double alpha, const double *A,
                     int64_t lda, const double *B, int64_t ldb, double beta, double *C,
                     int64_t ldc) {
  PGB_ENTRY(stream);
  return syr2k_entry<double>(stream, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}

int32_t pgb200Ssyr2k(void *stream, int64_t N, int64_t K, float alpha, const float *A, int64_t lda,
                     const float *B, int64_t ldb, float beta, float *C, int64_t ldc) {
  PGB_ENTRY(stream);
  return syr2k_entry<float>(stream, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}

int32_t pgb200Dsyrk(void *stream, int64_t N, int64_t K, double alpha, const double *A,
                    int64_t lda, double beta, double *C, int64_t ldc) {
  PGB_ENTRY(stream);
  return syrk_entry<double>(stream, N, K, 0, N, alpha, A, lda, beta, C, ldc);
}

int32_t pgb200Ssyrk(void *stream, int64_t N, int64_t K, float alpha, const float *A, int64_t lda,
                    float beta, float *C, int64_t ldc) {
  PGB_ENTRY(stream);
  return syrk_entry<float>(stream, N, K, 0, N, alpha, A, lda, beta, C, ldc);
}

int32_t pgb200SsyrkRows(void *stream, int64_t N, int64_t K, int64_t row0, int64_t row1,
                        float alpha, const float *A, int64_t lda, float beta, float *C,
                        int64_t ldc) {
  PGB_ENTRY(stream);
  return syrk_entry<float>(stream, N, K, row0, row1, alpha, A, lda, beta, C, ldc);
}

int32_t pgb200Dgemv(void *stream, int32_t transA, int64_t M, int64_t N, double alpha,
                    const double *A, int64_t lda, const double *x, double beta, double *y) {
  PGB_ENTRY(stream);
  PGB_REQUIRE(y || (transA ? N : M) == 0, "gemv: y is null");
  if (transA) return matvec_entry(stream, M, N, A, lda, alpha, beta, nullptr, nullptr, x, y);
  return matvec_entry(stream, M, N, A, lda, alpha, beta, x, y, nullptr, nullptr);
}

int32_t pgb200DgemvPair(void *stream, int64_t M, int64_t N, double alpha, const double *A,
                        int64_t lda, const double *x1, const double *x2, double beta, double *y1,
                        double *y2) {
  PGB_ENTRY(stream);
  PGB_REQUIRE((y1 || M == 0) && (y2 || N == 0), "gemv pair: null output vector");
  return matvec_entry(stream, M, N, A, lda, alpha, beta, x1, y1, x2, y2);
}

int32_t pgb200Dgemver(void *stream, int64_t N, double alpha, double beta, double *A, int64_t lda,
                      const double *u1, const double *v1, const double *u2, const double *v2,
                      double *w, double *x, const double *y, const double *z) {
  PGB_ENTRY(stream);
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(N >= 0, "gemver: negative size");
  if (N == 0) return PGB200_OK;
  PGB_REQUIRE(A && u1 && v1 && u2 && v2 && w && x && y && z && lda >= N,
              "gemver: null pointer or lda (%lld) < N (%lld)", (long long)lda, (long long)N);
  cudaStream_t s = (cudaStream_t)stream;
  Staged<double> sa, su1, sv1, su2, sv2, sw, sx, sy, sz;
  PGB_TRY(stage<double>(s, A, N, N, lda, true, true, &sa));
  PGB_TRY(stage<double>(s, u1, 1, N, N, true, false, &su1));
  PGB_TRY(stage<double>(s, v1, 1, N, N, true, false, &sv1));
  PGB_TRY(stage<double>(s, u2, 1, N, N, true, false, &su2));
  PGB_TRY(stage<double>(s, v2, 1, N, N, true, false, &sv2));
  PGB_TRY(stage<double>(s, w, 1, N, N, true, true, &sw));
  PGB_TRY(stage<double>(s, x, 1, N, N, true, true, &sx));
  PGB_TRY(stage<double>(s, y, 1, N, N, true, false, &sy));
  PGB_TRY(stage<double>(s, z, 1, N, N, true, false, &sz));
  const bool staged = sa.host || su1.host || sv1.host || su2.host || sv2.host || sw.host ||
                      sx.host || sy.host || sz.host;
  int32_t st = stream_gemver(s, N, alpha, beta, sa.dev, sa.ld, su1.dev, sv1.dev, su2.dev, sv2.dev,
                             sw.dev, sx.dev, sy.dev, sz.dev);
  if (st != PGB200_OK) return st;  // staged copies are released, nothing is copied back
  if (staged) PGB_TRY(sync_check(rt, s));  // a kernel that gave up: nothing is copied back either
  PGB_TRY(finish(s, &sa));
  PGB_TRY(finish(s, &su1));
  PGB_TRY(finish(s, &sv1));
  PGB_TRY(finish(s, &su2));
  PGB_TRY(finish(s, &sv2));
  PGB_TRY(finish(s, &sw));
  PGB_TRY(finish(s, &sx));
  PGB_TRY(finish(s, &sy));
  PGB_TRY(finish(s, &sz));
  if (staged) PGB_CUDA(cudaStreamSynchronize(s));
  return st;
}

int32_t pgb200Dmvt(void *stream, int64_t N, const double *A, int64_t lda, const double *y1,
                   const double *y2, double *x1, double *x2) {
  PGB_ENTRY(stream);
  PGB_REQUIRE(N == 0 || (x1 && x2 && y1 && y2), "mvt: null vector");
  return matvec_entry(stream, N, N, A, lda, 1.0, 1.0, y1, x1, y2, x2);
}

// ---- host-array drop-ins with the reference's signatures -------------------

int32_t pgb200_kernel_gemm(int ni, int nj, int nk, double alpha, double beta, double *C,
                           const double *A, const double *B) {
  PGB_ENTRY(nullptr);
  return pgb200Dgemm(nullptr, ni, nj, nk, alpha, A, nk, B, nj, beta, C, nj);
}

int32_t pgb200_kernel_gemm_f32(int ni, int nj, int nk, float alpha, float beta, float *C,
                               const float *A, const float *B) {
  PGB_ENTRY(nullptr);
  return pgb200Sgemm(nullptr, ni, nj, nk, alpha, A, nk, B, nj, beta, C, nj);
}

int32_t pgb200_kernel_2mm(int ni, int nj, int nk, int nl, double alpha, double beta, double *tmp,
                          const double *A, const double *B, const double *C, double *D) {
  PGB_ENTRY(nullptr);
  // tmp = alpha*A*B stays in HBM between the two contractions; it is copied
  // back once because the C source leaves it as a live-out array.
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(ni >= 0 && nj >= 0 && nk >= 0 && nl >= 0, "kernel_2mm: negative size");
  cudaStream_t s = nullptr;
  Staged<double> sa, sb, sc, sd, st;
  PGB_TRY(stage<double>(s, A, ni, nk, nk, true, false, &sa));
  PGB_TRY(stage<double>(s, B, nk, nj, nj, true, false, &sb));
  PGB_TRY(stage<double>(s, C, nj, nl, nl, true, false, &sc));
  PGB_TRY(stage<double>(s, D, ni, nl, nl, beta != 0.0, true, &sd));
  PGB_TRY(stage<double>(s, tmp, ni, nj, nj, false, true, &st));
  int32_t r = pgb200Dgemm(s, ni, nj, nk, alpha, sa.dev, sa.ld, sb.dev, sb.ld, 0.0, st.dev, st.ld);
  if (r == PGB200_OK)
    r = pgb200Dgemm(s, ni, nl, nj, 1.0, st.dev, st.ld, sc.dev, sc.ld, beta, sd.dev, sd.ld);
  if (r != PGB200_OK) return r;  // staged copies are released, nothing is copied back
  PGB_TRY(sync_check(rt, s));  // a kernel that gave up: nothing is copied back either
  PGB_TRY(finish(s, &sa));
  PGB_TRY(finish(s, &sb));
  PGB_TRY(finish(s, &sc));
  PGB_TRY(finish(s, &sd));
  PGB_TRY(finish(s, &st));
  PGB_CUDA(cudaStreamSynchronize(s));
  return r;
}

int32_t pgb200_kernel_mvt(int n, double *x1, double *x2, const double *y_1, const double *y_2,
                          const double *A) {
  PGB_ENTRY(nullptr);
  return pgb200Dmvt(nullptr, n, A, n, y_1, y_2, x1, x2);
}

int32_t pgb200_kernel_3mm(int ni, int nj, int nk, int nl, int nm, double *E, const double *A,
                          const double *B, double *F, const double *C, const double *D,
                          double *G) {
  PGB_ENTRY(nullptr);
  // E = A*B and F = C*D stay in HBM for G = E*F; all three are copied back
  // because the C source leaves them as live-out arrays.
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(ni >= 0 && nj >= 0 && nk >= 0 && nl >= 0 && nm >= 0, "kernel_3mm: negative size");
  cudaStream_t s = nullptr;
  Staged<double> sa, sb, sc, sd, se, sf, sg;
  PGB_TRY(stage<double>(s, A, ni, nk, nk, true, false, &sa));
  PGB_TRY(stage<double>(s, B, nk, nj, nj, true, false, &sb));
  PGB_TRY(stage<double>(s, C, nj, nm, nm, true, false, &sc));
  PGB_TRY(stage<double>(s, D, nm, nl, nl, true, false, &sd));
  PGB_TRY(stage<double>(s, E, ni, nj, nj, false, true, &se));
  PGB_TRY(stage<double>(s, F, nj, nl, nl, false, true, &sf));
  PGB_TRY(stage<double>(s, G, ni, nl, nl, false, true, &sg));
  int32_t r = pgb200Dgemm(s, ni, nj, nk, 1.0, sa.dev, sa.ld, sb.dev, sb.ld, 0.0, se.dev, se.ld);
  if (r == PGB200_OK)
    r = pgb200Dgemm(s, nj, nl, nm, 1.0, sc.dev, sc.ld, sd.dev, sd.ld, 0.0, sf.dev, sf.ld);
  if (r == PGB200_OK)
    r = pgb200Dgemm(s, ni, nl, nj, 1.0, se.dev, se.ld, sf.dev, sf.ld, 0.0, sg.dev, sg.ld);
  if (r != PGB200_OK) return r;  // staged copies are released, nothing is copied back
  PGB_TRY(sync_check(rt, s));  // a kernel that gave up: nothing is copied back either
  PGB_TRY(finish(s, &sa));
  PGB_TRY(finish(s, &sb));
  PGB_TRY(finish(s, &sc));
  PGB_TRY(finish(s, &sd));
  PGB_TRY(finish(s, &se));
  PGB_TRY(finish(s, &sf));
  PGB_TRY(finish(s, &sg));
  PGB_CUDA(cudaStreamSynchronize(s));
  return r;
}

int32_t pgb200_kernel_atax(int m, int n, const double *A, const double *x, double *y,
                           double *tmp) {
  PGB_ENTRY(nullptr);
  // tmp = A x, then y = A^T tmp.  A is staged once and read twice on the GPU.
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(m >= 0 && n >= 0, "kernel_atax: negative size");
  cudaStream_t s = nullptr;
  Staged<double> sa, sx, sy, st;
  PGB_TRY(stage<double>(s, A, m, n, n, true, false, &sa));
  PGB_TRY(stage<double>(s, x, 1, n, n, true, false, &sx));
  PGB_TRY(stage<double>(s, y, 1, n, n, false, true, &sy));
  PGB_TRY(stage<double>(s, tmp, 1, m, m, false, true, &st));
  int32_t r = pgb200Dgemv(s, 0, m, n, 1.0, sa.dev, sa.ld, sx.dev, 0.0, st.dev);
  if (r == PGB200_OK) r = pgb200Dgemv(s, 1, m, n, 1.0, sa.dev, sa.ld, st.dev, 0.0, sy.dev);
  if (r != PGB200_OK) return r;  // staged copies are released, nothing is copied back
  PGB_TRY(sync_check(rt, s));  // a kernel that gave up: nothing is copied back either
  PGB_TRY(finish(s, &sa));
  PGB_TRY(finish(s, &sx));
  PGB_TRY(finish(s, &sy));
  PGB_TRY(finish(s, &st));
  PGB_CUDA(cudaStreamSynchronize(s));
  return r;
}

int32_t pgb200_kernel_bicg(int m, int n, const double *A, double *s_out, double *q,
                           const double *p, const double *r) {
  PGB_ENTRY(nullptr);
  // A is n x m: q = A p (n entries), s = A^T r (m entries), one pass.
  return pgb200DgemvPair(nullptr, n, m, 1.0, A, m, p, r, 0.0, q, s_out);
}

int32_t pgb200_kernel_gesummv(int n, double alpha, double beta, const double *A, const double *B,
                              double *tmp, const double *x, double *y) {
  PGB_ENTRY(nullptr);
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  PGB_REQUIRE(n >= 0, "kernel_gesummv: negative size");
  cudaStream_t s = nullptr;
  Staged<double> sa, sb, sx, sy, st;
  PGB_TRY(stage<double>(s, A, n, n, n, true, false, &sa));
  PGB_TRY(stage<double>(s, B, n, n, n, true, false, &sb));
  PGB_TRY(stage<double>(s, x, 1, n, n, true, false, &sx));
  PGB_TRY(stage<double>(s, y, 1, n, n, false, true, &sy));
  PGB_TRY(stage<double>(s, tmp, 1, n, n, false, true, &st));
  int32_t r = pgb200Dgemv(s, 0, n, n, 1.0, sa.dev, sa.ld, sx.dev, 0.0, st.dev);  // tmp = A x
  if (r == PGB200_OK) r = pgb200Dgemv(s, 0, n, n, 1.0, sb.dev, sb.ld, sx.dev, 0.0, sy.dev);  // y = B x
  if (r == PGB200_OK) r = stream_axpby(s, n, alpha, st.dev, beta, sy.dev);  // y = alpha*tmp + beta*y
  if (r != PGB200_OK) return r;  // staged copies are released, nothing is copied back
  PGB_TRY(sync_check(rt, s));  // a kernel that gave up: nothing is copied back either
  PGB_TRY(finish(s, &sa));
  PGB_TRY(finish(s, &sb));
  PGB_TRY(finish(s, &sx));
  PGB_TRY(finish(s, &sy));
  PGB_TRY(finish(s, &st));
  PGB_CUDA(cudaStreamSynchronize(s));
  return r;
}

int32_t pgb200_kernel_syrk(int n, int m, double alpha, double beta, double *C, const double *A) {
  PGB_ENTRY(nullptr);
  return pgb200Dsyrk(nullptr, n, m, alpha, A, m, beta, C, n);
}

int32_t pgb200_kernel_gemver(int n, double alpha, double beta, double *A, const double *u1,
                             const double *v1, const double *u2, const double *v2, double *w,
                             double *x, const double *y, const double *z) {
  PGB_ENTRY(nullptr);
  return pgb200Dgemver(nullptr, n, alpha, beta, A, n, u1, v1, u2, v2, w, x, y, z);
}

int32_t pgb200_kernel_syr2k(int n, int m, double alpha, double beta, double *C, const double *A,
                            const double *B) {
  PGB_ENTRY(nullptr);
  return pgb200Dsyr2k(nullptr, n, m, alpha, A, m, B, m, beta, C, n);
}

int32_t pgb200_kernel_syr2k_f32(int n, int m, float alpha, float beta, float *C, const float *A,
                                const float *B) {
  PGB_ENTRY(nullptr);
  return pgb200Ssyr2k(nullptr, n, m, alpha, A, m, B, m, beta, C, n);
}

int32_t pgb200_kernel_syrk_f32(int n, int m, float alpha, float beta, float *C, const float *A) {
  PGB_ENTRY(nullptr);
  return pgb200Ssyrk(nullptr, n, m, alpha, A, m, beta, C, n);
}

}  // extern "C"
