// Host runtime behind the C ABI: error reporting, devices, the per-device stream pool, events,
// the stream-ordered caching allocator, host<->device copies through pinned staging, and the
// iteration-descriptor helpers.  No kernels live here.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>
#include <set>
#include <unordered_map>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "twg_launch.cuh"

namespace twg {

// ------------------------------------------------------------------------------------------
// errors, counters
// ------------------------------------------------------------------------------------------
static thread_local char g_error[1024] = "";
thread_local int g_last_path = 0;
static std::atomic<long long> g_launches{0};

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
  const char* base = strrchr(file, '/');
  // cudaErrorMemoryAllocation and launch-configuration errors are not sticky; clear them so the
  // next call starts clean.
  cudaGetLastError();
  return set_error(e == cudaErrorMemoryAllocation ? TWG_ERR_OOM : TWG_ERR_CUDA, "%s failed: %s (%s) at %s:%d", what,
                   cudaGetErrorString(e), cudaGetErrorName(e), base ? base + 1 : file, line);
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// -1: not decided yet (the environment is read on first use), 0 off, 1 on
static std::atomic<int> g_tracing{-1};
static bool tracing_on() {
  int v = g_tracing.load(std::memory_order_relaxed);
  if (v < 0) {
    const char* env = getenv("TWG_NVTX");
    v = (env && *env && *env != '0') ? 1 : 0;
    int expected = -1;
    g_tracing.compare_exchange_strong(expected, v);
    v = g_tracing.load();
  }
  return v == 1;
}
TraceRange::TraceRange(const char* name) : active(tracing_on()) {
  if (active) nvtxRangePushA(name);
}
TraceRange::~TraceRange() {
  if (active) nvtxRangePop();
}

constexpr int kMaxDevices = 64;

int sm_count() {
  static std::atomic<int> cache[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int v = cache[dev].load();
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    cache[dev].store(v);
  }
  return v;
}

// ------------------------------------------------------------------------------------------
// descriptors
// ------------------------------------------------------------------------------------------
int check_desc(const TwgIterDesc* d, int ntensors) {
  TWG_REQUIRE(d != nullptr, "iteration descriptor is null");
  TWG_REQUIRE(d->ndim >= 0 && d->ndim <= TWG_MAX_DIMS, "descriptor has %d dimensions; at most %d are supported",
              d->ndim, TWG_MAX_DIMS);
  TWG_REQUIRE(ntensors <= TWG_MAX_TENSORS, "too many operands (%d)", ntensors);
  TWG_REQUIRE(d->ntensors >= ntensors, "descriptor describes %d operands, the op needs %d", d->ntensors, ntensors);
  int64_t n = 1;
  for (int k = 0; k < d->ndim; ++k) {
    TWG_REQUIRE(d->shape[k] >= 0, "descriptor shape[%d] is negative", k);
    n *= d->shape[k];
  }
  TWG_REQUIRE(n == d->numel, "descriptor numel %lld does not match its shape (%lld)", (long long)d->numel,
              (long long)n);
  return TWG_OK;
}

int64_t max_offset(const TwgIterDesc& d, int t) {
  int64_t off = 0;
  for (int k = 0; k < d.ndim; ++k) {
    const int64_t s = d.strides[t][k] < 0 ? -d.strides[t][k] : d.strides[t][k];
    if (d.shape[k] > 0) off += (d.shape[k] - 1) * s;
  }
  return off;
}

void make_fastdiv(uint32_t d, uint32_t* m, uint32_t* s) {
  if (d == 0) d = 1;
  uint32_t shift = 0;
  while (shift < 32 && (1ull << shift) < d) ++shift;
  const uint64_t one = 1;
  const uint64_t magic = ((one << 32) * ((one << shift) - d)) / d + 1;
  *m = (uint32_t)magic;
  *s = shift;
}

// ------------------------------------------------------------------------------------------
// launch planning for the pointwise kernels
// ------------------------------------------------------------------------------------------
bool fits_32bit(const TwgIterDesc& d, int nt) {
  if (d.numel >= (int64_t(1) << 31)) return false;
  for (int t = 0; t < nt; ++t) {
    for (int k = 0; k < d.ndim; ++k)
      if (d.strides[t][k] < 0) return false;
    if (max_offset(d, t) >= (int64_t(1) << 31)) return false;
  }
  return true;
}

bool plan_tile(const TwgIterDesc& d, int nt, int tile_edge, PwPlan* plan) {
  if (d.ndim != 2 || d.shape[0] < 16 || d.shape[1] < 16) return false;
  uint32_t mask = 0;
  for (int t = 0; t < nt; ++t) {
    const int64_t s0 = d.strides[t][0], s1 = d.strides[t][1];
    if (s0 == 1) continue;  // dense along dimension 0: accessed directly
    if (s1 == 1 && s0 >= 0) { mask |= 1u << t; continue; }
    return false;
  }
  if (mask == 0) return false;
  plan->dim1_mask = mask;
  plan->tiles0 = (d.shape[0] + tile_edge - 1) / tile_edge;
  plan->tiles1 = (d.shape[1] + tile_edge - 1) / tile_edge;
  plan->ntiles = plan->tiles0 * plan->tiles1;
  if (tile_edge == kPwTile) {
    // the functor kernels walk tiles in 8x8 super-blocks; partial super-blocks leave idle slots
    plan->sb0 = (plan->tiles0 + kTileSuper - 1) / kTileSuper;
    plan->ntiles = plan->sb0 * ((plan->tiles1 + kTileSuper - 1) / kTileSuper) * kTileSuper * kTileSuper;
  }
  if (plan->ntiles > 0x7fffffff) return false;  // the kernels index tiles with 32 bits
  plan->grid = (unsigned)plan->ntiles;
  return true;
}

int plan_pointwise(const PwSig& sig, const TwgIterDesc* desc, void* const* ptrs, PwPlan* plan) {
  const int nt = sig.nt();
  g_last_path = kPathNone;
  plan->path = kPathNone;
  if (int rc = check_desc(desc, nt)) return rc;
  if (desc->numel == 0) return TWG_OK;
  for (int t = 0; t < nt; ++t) TWG_REQUIRE(ptrs[t] != nullptr, "operand %d is a null pointer", t);
  for (int t = 0; t < nt; ++t)
    TWG_REQUIRE(sig.byte(t) || is_aligned(ptrs[t], 4), "operand %d is not aligned to its 4-byte element", t);
  plan->d = *desc;
  plan->d.ntensors = nt;
  if (int rc = twg_iter_coalesce(&plan->d)) return rc;
  const TwgIterDesc& d = plan->d;

  bool dense = d.ndim <= 1;
  const int vec = sig.vec();
  for (int t = 0; t < nt && dense; ++t) {
    if (d.ndim == 1 && d.numel > 1 && d.strides[t][0] != 1) dense = false;
    if (!is_aligned(ptrs[t], (size_t)vec * (sig.byte(t) ? 1 : 4))) dense = false;
  }
  if (dense) {
    plan->nunits = d.numel / vec;
    const int64_t chunk = (int64_t)kBlock * dense_unroll(sig.nin);
    plan->grid = (unsigned)std::min<int64_t>(std::max<int64_t>(1, (plan->nunits + chunk - 1) / chunk), 0x7fffffff);
    plan->path = kPathDense;
    return TWG_OK;
  }
  if (plan_tile(d, nt, kPwTile, plan)) {
    plan->path = kPathTile;
    return TWG_OK;
  }
  const int64_t per_cta = (int64_t)kBlock * kStridedUnroll;
  plan->grid = (unsigned)std::min<int64_t>((d.numel + per_cta - 1) / per_cta, 0x7fffffff);
  plan->path = fits_32bit(d, nt) ? kPathStrided32 : kPathStrided64;
  return TWG_OK;
}

// ------------------------------------------------------------------------------------------
// devices, streams
// ------------------------------------------------------------------------------------------
struct DeviceState {
  std::mutex mu;
  cudaStream_t streams[TWG_NUM_STREAMS] = {};
  bool created[TWG_NUM_STREAMS] = {};
};
static DeviceState g_devices[kMaxDevices];

static int device_count_cached(int* n) {
  static std::atomic<int> cached{-1};
  int v = cached.load();
  if (v < 0) {
    cudaError_t e = cudaGetDeviceCount(&v);
    if (e != cudaSuccess) {
      cudaGetLastError();
      if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) {
        *n = 0;
        return TWG_OK;  // no GPU is a count of zero, not an error; the result is not cached
      }
      return cuda_fail(e, "cudaGetDeviceCount", __FILE__, __LINE__);
    }
    cached.store(v);
  }
  *n = v;
  return TWG_OK;
}

struct ScopedDevice {
  int prev = -1;
  bool switched = false;
  cudaError_t err = cudaSuccess;
  explicit ScopedDevice(int dev) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != dev) {
      err = cudaSetDevice(dev);
      switched = err == cudaSuccess;
    }
  }
  ~ScopedDevice() {
    if (switched) cudaSetDevice(prev);
  }
};

// ------------------------------------------------------------------------------------------
// caching allocator
//
// Sizes are rounded to 512 B.  Requests up to 1 MiB are carved from 2 MiB segments (small pool);
// larger ones from segments of 20 MiB (requests below 10 MiB) or the request rounded to 2 MiB
// (large pool).  Free blocks are kept per (stream, size) and reused best-fit by the stream that
// allocated them; a block that was also used on other streams (twg_record_stream) becomes
// reusable only after an event recorded on each of those streams has completed.  Neighbouring
// free blocks of a segment merge.  When cudaMalloc fails, every cached segment is released and
// the request retried once.
// ------------------------------------------------------------------------------------------
constexpr size_t kRound = 512;
constexpr size_t kSmallLimit = 1u << 20;
constexpr size_t kSmallSegment = 2u << 20;
constexpr size_t kLargeSegment = 20u << 20;
constexpr size_t kMidLimit = 10u << 20;

struct Block {
  int device = 0;
  cudaStream_t stream = nullptr;
  char* ptr = nullptr;
  size_t size = 0;
  bool small = false;
  bool allocated = false;
  Block* prev = nullptr;
  Block* next = nullptr;
  int pending_events = 0;
  std::vector<cudaStream_t> extra_streams;
  size_t user_bytes = 0;  // bytes the caller asked for (guard words start behind them)
  bool guarded = false;
};

// Guard words (a debugging aid, off by default): while enabled, every new block is allocated
// kGuardBytes larger than asked for and the bytes behind the caller's are filled with a pattern;
// twg_check_guard_words compares them later.  A kernel that writes a little past its output lands
// in the guard (inside the block, so nothing faults) and is reported with the block's address.
constexpr size_t kGuardBytes = 512;
constexpr unsigned char kGuardPattern = 0xA5;
static std::atomic<int> g_guard_words{0};

struct BlockLess {
  bool operator()(const Block* a, const Block* b) const {
    if (a->stream != b->stream) return (uintptr_t)a->stream < (uintptr_t)b->stream;
    if (a->size != b->size) return a->size < b->size;
    return (uintptr_t)a->ptr < (uintptr_t)b->ptr;
  }
};

struct Pool {
  std::set<Block*, BlockLess> small_free, large_free;
  std::deque<std::pair<cudaEvent_t, Block*>> pending;
  TwgMemStats stats = {};
  size_t budget = 0;
};

static std::mutex g_alloc_mu;
static Pool g_pools[kMaxDevices];
static std::unordered_map<void*, Block*> g_live;

static void bump_allocated(Pool& p, int64_t delta) {
  p.stats.allocated_bytes += delta;
  if (p.stats.allocated_bytes > p.stats.peak_allocated_bytes) p.stats.peak_allocated_bytes = p.stats.allocated_bytes;
}
static void bump_reserved(Pool& p, int64_t delta) {
  p.stats.reserved_bytes += delta;
  if (p.stats.reserved_bytes > p.stats.peak_reserved_bytes) p.stats.peak_reserved_bytes = p.stats.reserved_bytes;
}

static void insert_free(Pool& p, Block* b) {
  // merge with free neighbours of the same segment
  auto& set = b->small ? p.small_free : p.large_free;
  Block* n = b->next;
  if (n && !n->allocated && n->pending_events == 0 && set.count(n)) {
    set.erase(n);
    b->size += n->size;
    b->next = n->next;
    if (n->next) n->next->prev = b;
    delete n;
  }
  Block* q = b->prev;
  if (q && !q->allocated && q->pending_events == 0 && set.count(q)) {
    set.erase(q);
    q->size += b->size;
    q->next = b->next;
    if (b->next) b->next->prev = q;
    delete b;
    b = q;
  }
  set.insert(b);
}

static void process_pending(Pool& p, bool wait) {
  while (!p.pending.empty()) {
    auto& front = p.pending.front();
    cudaError_t e = wait ? cudaEventSynchronize(front.first) : cudaEventQuery(front.first);
    if (e == cudaErrorNotReady) {
      cudaGetLastError();
      break;
    }
    cudaEventDestroy(front.first);
    Block* b = front.second;
    p.pending.pop_front();
    if (--b->pending_events == 0) insert_free(p, b);
  }
}

// Release every fully free segment back to the driver.  Caller holds g_alloc_mu.
static void release_cached(Pool& p, int device) {
  ScopedDevice guard(device);
  process_pending(p, true);
  for (auto* set : {&p.small_free, &p.large_free}) {
    for (auto it = set->begin(); it != set->end();) {
      Block* b = *it;
      if (b->prev == nullptr && b->next == nullptr) {
        cudaFree(b->ptr);
        p.stats.num_device_frees++;
        bump_reserved(p, -(int64_t)b->size);
        it = set->erase(it);
        delete b;
      } else {
        ++it;
      }
    }
  }
}

static size_t round_size(size_t n) { return (n + kRound - 1) / kRound * kRound; }
static size_t segment_size(size_t size) {
  if (size <= kSmallLimit) return kSmallSegment;
  if (size < kMidLimit) return kLargeSegment;
  return (size + kSmallSegment - 1) / kSmallSegment * kSmallSegment;
}

static int device_malloc(Pool& p, void** out, size_t bytes) {
  if (p.budget != 0 && (size_t)p.stats.reserved_bytes + bytes > p.budget)
    return set_error(TWG_ERR_OOM, "allocation of %zu bytes exceeds the configured memory budget of %zu bytes "
                     "(%lld reserved)", bytes, p.budget, (long long)p.stats.reserved_bytes);
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return set_error(TWG_ERR_OOM, "cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
  }
  p.stats.num_device_mallocs++;
  bump_reserved(p, (int64_t)bytes);
  return TWG_OK;
}

}  // namespace twg

using namespace twg;

// ------------------------------------------------------------------------------------------
// C ABI: library / device / stream / event
// ------------------------------------------------------------------------------------------
extern "C" const char* twg_last_error(void) { return g_error; }
extern "C" const char* twg_version(void) { return "twg 0.1 (sm_100a)"; }
extern "C" int twg_last_launch_path(void) { return g_last_path; }
extern "C" int64_t twg_launch_count(void) { return g_launches.load(); }
extern "C" void twg_reset_launch_count(void) { g_launches.store(0); }

extern "C" int twg_set_tracing(int enabled) {
  g_tracing.store(enabled ? 1 : 0);
  return TWG_OK;
}
extern "C" int twg_get_tracing(void) { return tracing_on() ? 1 : 0; }

extern "C" int twg_device_count(int* count) {
  TWG_REQUIRE(count != nullptr, "twg_device_count: null argument");
  return device_count_cached(count);
}

static int check_device(int device) {
  int n = 0;
  if (int rc = device_count_cached(&n)) return rc;
  if (n == 0) return set_error(TWG_ERR_CUDA, "no CUDA device is available");
  TWG_REQUIRE(device >= 0 && device < n && device < kMaxDevices, "device %d is out of range (%d available)", device, n);
  return TWG_OK;
}

extern "C" int twg_set_device(int device) {
  if (int rc = check_device(device)) return rc;
  TWG_CUDA(cudaSetDevice(device));
  return TWG_OK;
}

extern "C" int twg_get_device(int* device) {
  TWG_REQUIRE(device != nullptr, "twg_get_device: null argument");
  TWG_CUDA(cudaGetDevice(device));
  return TWG_OK;
}

extern "C" int twg_get_stream(int device, int index, void** stream) {
  TWG_REQUIRE(stream != nullptr, "twg_get_stream: null argument");
  TWG_REQUIRE(index >= 0 && index < TWG_NUM_STREAMS, "stream index %d out of range", index);
  if (int rc = check_device(device)) return rc;
  DeviceState& st = g_devices[device];
  std::lock_guard<std::mutex> lock(st.mu);
  if (!st.created[index]) {
    ScopedDevice guard(device);
    TWG_CUDA(guard.err);
    TWG_CUDA(cudaStreamCreateWithFlags(&st.streams[index], cudaStreamNonBlocking));
    st.created[index] = true;
  }
  *stream = st.streams[index];
  return TWG_OK;
}

extern "C" int twg_stream_sync(void* stream) {
  TWG_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return TWG_OK;
}

extern "C" int twg_device_sync(int device) {
  if (int rc = check_device(device)) return rc;
  ScopedDevice guard(device);
  TWG_CUDA(guard.err);
  TWG_CUDA(cudaDeviceSynchronize());
  return TWG_OK;
}

extern "C" int twg_stream_query(void* stream, int* done) {
  TWG_REQUIRE(done != nullptr, "twg_stream_query: null argument");
  cudaError_t e = cudaStreamQuery(static_cast<cudaStream_t>(stream));
  if (e == cudaErrorNotReady) {
    cudaGetLastError();
    *done = 0;
    return TWG_OK;
  }
  TWG_CUDA(e);
  *done = 1;
  return TWG_OK;
}

extern "C" int twg_event_create(void** event) {
  TWG_REQUIRE(event != nullptr, "twg_event_create: null argument");
  cudaEvent_t ev;
  TWG_CUDA(cudaEventCreate(&ev));
  *event = ev;
  return TWG_OK;
}
extern "C" int twg_event_destroy(void* event) {
  if (event) TWG_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  return TWG_OK;
}
extern "C" int twg_event_record(void* event, void* stream) {
  TWG_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
  return TWG_OK;
}
extern "C" int twg_event_wait(void* event, void* stream) {
  TWG_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
  return TWG_OK;
}
extern "C" int twg_event_query(void* event, int* done) {
  TWG_REQUIRE(done != nullptr, "twg_event_query: null argument");
  cudaError_t e = cudaEventQuery(static_cast<cudaEvent_t>(event));
  if (e == cudaErrorNotReady) {
    cudaGetLastError();
    *done = 0;
    return TWG_OK;
  }
  TWG_CUDA(e);
  *done = 1;
  return TWG_OK;
}
extern "C" int twg_event_sync(void* event) {
  TWG_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
  return TWG_OK;
}
extern "C" int twg_event_elapsed_ms(void* start, void* stop, float* ms) {
  TWG_REQUIRE(ms != nullptr, "twg_event_elapsed_ms: null argument");
  TWG_CUDA(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
  return TWG_OK;
}

// ------------------------------------------------------------------------------------------
// C ABI: descriptors
// ------------------------------------------------------------------------------------------
extern "C" int twg_iter_contiguous(TwgIterDesc* d, int ntensors, int64_t numel) {
  TWG_REQUIRE(d != nullptr, "twg_iter_contiguous: null descriptor");
  TWG_REQUIRE(ntensors >= 1 && ntensors <= TWG_MAX_TENSORS, "twg_iter_contiguous: %d operands", ntensors);
  TWG_REQUIRE(numel >= 0, "twg_iter_contiguous: negative numel");
  memset(d, 0, sizeof(*d));
  d->ndim = 1;
  d->ntensors = ntensors;
  d->numel = numel;
  d->shape[0] = numel;
  for (int t = 0; t < ntensors; ++t) d->strides[t][0] = 1;
  return TWG_OK;
}

extern "C" int twg_iter_coalesce(TwgIterDesc* d) {
  if (int rc = check_desc(d, d ? d->ntensors : 0)) return rc;
  if (d->numel == 0) return TWG_OK;
  const int nt = d->ntensors;
  // drop size-1 dimensions
  int nd = 0;
  for (int k = 0; k < d->ndim; ++k) {
    if (d->shape[k] == 1) continue;
    if (nd != k) {
      d->shape[nd] = d->shape[k];
      for (int t = 0; t < nt; ++t) d->strides[t][nd] = d->strides[t][k];
    }
    ++nd;
  }
  // merge dimension k+1 into k when every operand continues seamlessly
  int w = 0;
  for (int k = 1; k < nd; ++k) {
    bool mergeable = true;
    for (int t = 0; t < nt; ++t)
      if (d->strides[t][k] != d->strides[t][w] * d->shape[w]) { mergeable = false; break; }
    if (mergeable) {
      d->shape[w] *= d->shape[k];
    } else {
      ++w;
      d->shape[w] = d->shape[k];
      for (int t = 0; t < nt; ++t) d->strides[t][w] = d->strides[t][k];
    }
  }
  d->ndim = nd == 0 ? 0 : w + 1;
  for (int k = d->ndim; k < TWG_MAX_DIMS; ++k) {
    d->shape[k] = 0;
    for (int t = 0; t < nt; ++t) d->strides[t][k] = 0;
  }
  return TWG_OK;
}

// ------------------------------------------------------------------------------------------
// C ABI: allocator
// ------------------------------------------------------------------------------------------
extern "C" int twg_malloc(void** ptr, size_t nbytes, int device, void* stream) {
  TWG_REQUIRE(ptr != nullptr, "twg_malloc: null result pointer");
  *ptr = nullptr;
  if (nbytes == 0) return TWG_OK;
  if (int rc = check_device(device)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool guarded = g_guard_words.load(std::memory_order_relaxed) != 0;
  const size_t size = round_size(nbytes + (guarded ? kGuardBytes : 0));
  const bool small = size <= kSmallLimit;

  std::lock_guard<std::mutex> lock(g_alloc_mu);
  Pool& p = g_pools[device];
  ScopedDevice guard(device);
  TWG_CUDA(guard.err);
  process_pending(p, false);
  auto& set = small ? p.small_free : p.large_free;

  Block key;
  key.stream = s;
  key.size = size;
  key.ptr = nullptr;
  Block* b = nullptr;
  auto it = set.lower_bound(&key);
  if (it != set.end() && (*it)->stream == s) {
    // do not hand a huge cached block to a much smaller large-pool request
    if (small || (*it)->size < kMidLimit || (*it)->size <= size + size / 4 + kLargeSegment) {
      b = *it;
      set.erase(it);
      p.stats.num_cache_hits++;
    }
  }
  if (!b) {
    const size_t seg = segment_size(size);
    void* mem = nullptr;
    int rc = device_malloc(p, &mem, seg);
    if (rc != TWG_OK) {
      release_cached(p, device);
      rc = device_malloc(p, &mem, seg);
      if (rc != TWG_OK) return rc;
    }
    b = new Block();
    b->device = device;
    b->stream = s;
    b->ptr = static_cast<char*>(mem);
    b->size = seg;
    b->small = small;
  }
  // split
  const size_t remaining = b->size - size;
  if ((small && remaining >= kRound) || (!small && remaining > kSmallLimit)) {
    Block* rest = new Block();
    rest->device = device;
    rest->stream = s;
    rest->ptr = b->ptr + size;
    rest->size = remaining;
    rest->small = small;
    rest->prev = b;
    rest->next = b->next;
    if (b->next) b->next->prev = rest;
    b->next = rest;
    b->size = size;
    set.insert(rest);
  }
  b->allocated = true;
  b->user_bytes = nbytes;
  b->guarded = false;
  g_live[b->ptr] = b;
  p.stats.num_allocs++;
  bump_allocated(p, (int64_t)b->size);
  *ptr = b->ptr;
  if (guarded) {
    // everything behind the caller's bytes, on the block's stream (ordered before its first use)
    TWG_CUDA(cudaMemsetAsync(b->ptr + nbytes, kGuardPattern, b->size - nbytes, s));
    b->guarded = true;
  }
  return TWG_OK;
}

extern "C" int twg_free(void* ptr) {
  if (!ptr) return TWG_OK;
  std::lock_guard<std::mutex> lock(g_alloc_mu);
  auto it = g_live.find(ptr);
  TWG_REQUIRE(it != g_live.end(), "twg_free: %p was not allocated by twg_malloc", ptr);
  Block* b = it->second;
  g_live.erase(it);
  Pool& p = g_pools[b->device];
  b->allocated = false;
  bump_allocated(p, -(int64_t)b->size);
  if (!b->extra_streams.empty()) {
    ScopedDevice guard(b->device);
    for (cudaStream_t s : b->extra_streams) {
      cudaEvent_t ev;
      if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) == cudaSuccess && cudaEventRecord(ev, s) == cudaSuccess) {
        b->pending_events++;
        p.pending.emplace_back(ev, b);
      } else {
        cudaGetLastError();
        cudaStreamSynchronize(s);  // fall back to waiting here
      }
    }
    b->extra_streams.clear();
    if (b->pending_events > 0) return TWG_OK;
  }
  insert_free(p, b);
  return TWG_OK;
}

extern "C" int twg_record_stream(void* ptr, void* stream) {
  if (!ptr) return TWG_OK;
  std::lock_guard<std::mutex> lock(g_alloc_mu);
  auto it = g_live.find(ptr);
  TWG_REQUIRE(it != g_live.end(), "twg_record_stream: %p was not allocated by twg_malloc", ptr);
  Block* b = it->second;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (s == b->stream) return TWG_OK;
  for (cudaStream_t e : b->extra_streams)
    if (e == s) return TWG_OK;
  b->extra_streams.push_back(s);
  return TWG_OK;
}

extern "C" int twg_trim(void* ptr, size_t new_nbytes) {
  if (!ptr) return TWG_OK;
  std::lock_guard<std::mutex> lock(g_alloc_mu);
  auto it = g_live.find(ptr);
  TWG_REQUIRE(it != g_live.end(), "twg_trim: %p was not allocated by twg_malloc", ptr);
  Block* b = it->second;
  const size_t keep = round_size(new_nbytes == 0 ? 1 : new_nbytes);
  if (keep >= b->size) return TWG_OK;
  const size_t remaining = b->size - keep;
  if ((b->small && remaining < kRound) || (!b->small && remaining <= kSmallLimit)) return TWG_OK;
  if (b->guarded) return TWG_OK;  // the guard words sit in the tail
  // A block that other streams also use (twg_record_stream) keeps its tail: those streams may
  // still touch it, and only twg_free orders a block's reuse after them.
  if (!b->extra_streams.empty()) return TWG_OK;
  Pool& p = g_pools[b->device];
  Block* rest = new Block();
  rest->device = b->device;
  rest->stream = b->stream;
  rest->ptr = b->ptr + keep;
  rest->size = remaining;
  rest->small = b->small;
  rest->prev = b;
  rest->next = b->next;
  if (b->next) b->next->prev = rest;
  b->next = rest;
  b->size = keep;
  bump_allocated(p, -(int64_t)remaining);
  // The tail may still be written by work already queued on the block's own stream, and a later
  // allocation on that stream is ordered after it, so it can go straight back to the free list.
  insert_free(p, rest);
  return TWG_OK;
}

extern "C" int twg_set_guard_words(int enabled) {
  g_guard_words.store(enabled ? 1 : 0);
  return TWG_OK;
}

extern "C" int twg_check_guard_words(int device, int64_t* corrupted_blocks, void** first_block) {
  if (int rc = check_device(device)) return rc;
  if (corrupted_blocks) *corrupted_blocks = 0;
  if (first_block) *first_block = nullptr;
  std::lock_guard<std::mutex> lock(g_alloc_mu);
  ScopedDevice guard(device);
  TWG_CUDA(guard.err);
  TWG_CUDA(cudaDeviceSynchronize());
  std::vector<unsigned char> host;
  int64_t bad = 0;
  void* first = nullptr;
  for (const auto& kv : g_live) {
    const Block* b = kv.second;
    if (b->device != device || !b->guarded) continue;
    const size_t n = b->size - b->user_bytes;
    host.resize(n);
    TWG_CUDA(cudaMemcpy(host.data(), b->ptr + b->user_bytes, n, cudaMemcpyDeviceToHost));
    bool ok = true;
    for (size_t i = 0; i < n && ok; ++i) ok = host[i] == kGuardPattern;
    if (!ok) {
      ++bad;
      if (first == nullptr || b->ptr < static_cast<char*>(first)) first = b->ptr;
    }
  }
  if (corrupted_blocks) *corrupted_blocks = bad;
  if (first_block) *first_block = first;
  return TWG_OK;
}

extern "C" int twg_block_size(void* ptr, size_t* nbytes, int* device) {
  std::lock_guard<std::mutex> lock(g_alloc_mu);
  auto it = g_live.find(ptr);
  TWG_REQUIRE(it != g_live.end(), "twg_block_size: %p was not allocated by twg_malloc", ptr);
  if (nbytes) *nbytes = it->second->size;
  if (device) *device = it->second->device;
  return TWG_OK;
}

extern "C" int twg_empty_cache(int device) {
  int n = 0;
  if (int rc = device_count_cached(&n)) return rc;
  std::lock_guard<std::mutex> lock(g_alloc_mu);
  for (int d = 0; d < n && d < kMaxDevices; ++d)
    if (device < 0 || device == d) release_cached(g_pools[d], d);
  return TWG_OK;
}

extern "C" int twg_memory_stats(int device, TwgMemStats* stats) {
  TWG_REQUIRE(stats != nullptr, "twg_memory_stats: null argument");
  TWG_REQUIRE(device >= 0 && device < kMaxDevices, "twg_memory_stats: device %d out of range", device);
  std::lock_guard<std::mutex> lock(g_alloc_mu);
  *stats = g_pools[device].stats;
  return TWG_OK;
}

extern "C" int twg_reset_peak_stats(int device) {
  TWG_REQUIRE(device >= 0 && device < kMaxDevices, "twg_reset_peak_stats: device %d out of range", device);
  std::lock_guard<std::mutex> lock(g_alloc_mu);
  Pool& p = g_pools[device];
  p.stats.peak_allocated_bytes = p.stats.allocated_bytes;
  p.stats.peak_reserved_bytes = p.stats.reserved_bytes;
  return TWG_OK;
}

extern "C" int twg_set_memory_budget(int device, size_t max_reserved_bytes) {
  TWG_REQUIRE(device >= 0 && device < kMaxDevices, "twg_set_memory_budget: device %d out of range", device);
  std::lock_guard<std::mutex> lock(g_alloc_mu);
  g_pools[device].budget = max_reserved_bytes;
  return TWG_OK;
}

// ------------------------------------------------------------------------------------------
// C ABI: copies
// ------------------------------------------------------------------------------------------
namespace twg {

constexpr size_t kStageBytes = 16u << 20;
constexpr int kStageSlots = 4;

struct Staging {
  std::mutex mu;
  char* buf[kStageSlots] = {};
  cudaEvent_t ev[kStageSlots] = {};
  bool busy[kStageSlots] = {};
  bool ready = false;
  int next = 0;
};
// one ring per device: CUDA events belong to the device they were created on
static Staging g_stage[kMaxDevices];

static Staging& staging_for_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
  return g_stage[dev];
}

static int staging_init(Staging& st) {
  if (st.ready) return TWG_OK;
  for (int i = 0; i < kStageSlots; ++i) {
    TWG_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&st.buf[i]), kStageBytes, cudaHostAllocPortable));
    TWG_CUDA(cudaEventCreateWithFlags(&st.ev[i], cudaEventDisableTiming));
  }
  st.ready = true;
  return TWG_OK;
}

static bool is_pinned(const void* p) {
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeHost || attr.type == cudaMemoryTypeManaged;
}

}  // namespace twg

extern "C" int twg_memcpy_h2d(void* dst_dev, const void* src_host, size_t nbytes, void* stream) {
  TWG_TRACE("twg_memcpy_h2d");
  if (nbytes == 0) return TWG_OK;
  TWG_REQUIRE(dst_dev && src_host, "twg_memcpy_h2d: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_pinned(src_host)) {
    TWG_CUDA(cudaMemcpyAsync(dst_dev, src_host, nbytes, cudaMemcpyHostToDevice, s));
    return TWG_OK;
  }
  Staging& st = staging_for_current_device();
  std::lock_guard<std::mutex> lock(st.mu);
  if (int rc = staging_init(st)) return rc;
  const char* src = static_cast<const char*>(src_host);
  char* dst = static_cast<char*>(dst_dev);
  for (size_t off = 0; off < nbytes; off += kStageBytes) {
    const size_t len = nbytes - off < kStageBytes ? nbytes - off : kStageBytes;
    const int slot = st.next;
    st.next = (st.next + 1) % kStageSlots;
    if (st.busy[slot]) TWG_CUDA(cudaEventSynchronize(st.ev[slot]));
    memcpy(st.buf[slot], src + off, len);
    TWG_CUDA(cudaMemcpyAsync(dst + off, st.buf[slot], len, cudaMemcpyHostToDevice, s));
    TWG_CUDA(cudaEventRecord(st.ev[slot], s));
    st.busy[slot] = true;
  }
  return TWG_OK;
}

extern "C" int twg_memcpy_d2h(void* dst_host, const void* src_dev, size_t nbytes, void* stream, int blocking) {
  TWG_TRACE("twg_memcpy_d2h");
  if (nbytes == 0) return TWG_OK;
  TWG_REQUIRE(dst_host && src_dev, "twg_memcpy_d2h: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_pinned(dst_host)) {
    TWG_CUDA(cudaMemcpyAsync(dst_host, src_dev, nbytes, cudaMemcpyDeviceToHost, s));
    if (blocking) TWG_CUDA(cudaStreamSynchronize(s));
    return TWG_OK;
  }
  Staging& st = staging_for_current_device();
  std::lock_guard<std::mutex> lock(st.mu);
  if (int rc = staging_init(st)) return rc;
  const char* src = static_cast<const char*>(src_dev);
  char* dst = static_cast<char*>(dst_host);
  // software pipeline: DMA of chunk i+1 overlaps the host memcpy of chunk i
  struct InFlight { int slot; size_t off, len; };
  std::deque<InFlight> flight;
  size_t off = 0;
  while (off < nbytes || !flight.empty()) {
    while (off < nbytes && (int)flight.size() < kStageSlots - 1) {
      const size_t len = nbytes - off < kStageBytes ? nbytes - off : kStageBytes;
      const int slot = st.next;
      st.next = (st.next + 1) % kStageSlots;
      if (st.busy[slot]) TWG_CUDA(cudaEventSynchronize(st.ev[slot]));
      TWG_CUDA(cudaMemcpyAsync(st.buf[slot], src + off, len, cudaMemcpyDeviceToHost, s));
      TWG_CUDA(cudaEventRecord(st.ev[slot], s));
      st.busy[slot] = true;
      flight.push_back({slot, off, len});
      off += len;
    }
    const InFlight f = flight.front();
    flight.pop_front();
    TWG_CUDA(cudaEventSynchronize(st.ev[f.slot]));
    memcpy(dst + f.off, st.buf[f.slot], f.len);
    st.busy[f.slot] = false;
  }
  return TWG_OK;
}

extern "C" int twg_memcpy_d2d(void* dst_dev, const void* src_dev, size_t nbytes, void* stream) {
  TWG_TRACE("twg_memcpy_d2d");
  if (nbytes == 0) return TWG_OK;
  TWG_REQUIRE(dst_dev && src_dev, "twg_memcpy_d2d: null pointer");
  TWG_CUDA(cudaMemcpyAsync(dst_dev, src_dev, nbytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
  return TWG_OK;
}

extern "C" int twg_memset(void* dst_dev, int value, size_t nbytes, void* stream) {
  if (nbytes == 0) return TWG_OK;
  TWG_REQUIRE(dst_dev != nullptr, "twg_memset: null pointer");
  TWG_CUDA(cudaMemsetAsync(dst_dev, value, nbytes, static_cast<cudaStream_t>(stream)));
  return TWG_OK;
}

extern "C" int twg_host_alloc_pinned(void** ptr, size_t nbytes) {
  TWG_REQUIRE(ptr != nullptr, "twg_host_alloc_pinned: null result pointer");
  *ptr = nullptr;
  if (nbytes == 0) return TWG_OK;
  TWG_CUDA(cudaHostAlloc(ptr, nbytes, cudaHostAllocPortable));
  return TWG_OK;
}

extern "C" int twg_host_free_pinned(void* ptr) {
  if (ptr) TWG_CUDA(cudaFreeHost(ptr));
  return TWG_OK;
}
