// The one exchange of the batch-sharded op path: every rank (one GPU each) tells every other rank
// how many elements its masked_select produced, so that each can place its segment in the global
// (concatenated) result.  16 bytes per rank and step.  Two ways to do it live here:
//
//   * NCCL: ncclAllGather on a communicator created through this C ABI.  libnccl is loaded lazily
//     with dlopen, so the library loads and every other entry point works without it.
//   * Peer stores: each rank owns a small "mailbox" in its own HBM; a rank's publish kernel
//     writes {count, sequence|status} straight into its slot of every peer's mailbox with plain
//     stores over NVLink (the second word is a release store at system scope), and a one-warp
//     collect kernel on the receiving GPU polls its own mailbox (acquire loads, bounded by a
//     time limit), computes the rank's offset and hands the gathered counts to the host through
//     mapped pinned memory.  No library call, no multicast, no TMA; nothing reads a peer's memory.
//     A step costs a sub-microsecond NVLink store instead of a collective launch, and the host
//     learns the counts by polling its own memory instead of waiting on an event.
//
// Slot reuse rule of the mailbox ring: slot = seq % ring.  A rank may publish sequence number s
// only after twg_exchange_wait has returned for sequence s - ring/2 on that rank.  Then a slot is
// never overwritten while a peer's collect kernel for the previous use is still reading it (the
// peer finished collecting s - ring before it published s - ring/2, which the publisher has
// observed).
#include <dlfcn.h>
#include <sched.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <mutex>
#include <string>

#include "twg_internal.h"

namespace twg {

using u64 = unsigned long long;
using i64 = long long;

// ------------------------------------------------------------------------------------------
// NCCL through dlopen
// ------------------------------------------------------------------------------------------
struct NcclId { char bytes[TWG_COMM_ID_BYTES]; };   // ncclUniqueId: 128 opaque bytes, passed by value
struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(NcclId*) = nullptr;
  int (*CommInitRank)(void**, int, NcclId, int) = nullptr;
  int (*CommDestroy)(void*) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  int (*GetVersion)(int*) = nullptr;
};
constexpr int kNcclInt64 = 4;  // ncclInt64 in ncclDataType_t

static std::mutex g_nccl_mu;
static NcclApi g_nccl;
static std::string g_nccl_path;

static int nccl_api(NcclApi** out) {
  std::lock_guard<std::mutex> lock(g_nccl_mu);
  if (g_nccl.handle == nullptr) {
    // an explicit path is the only candidate; otherwise the loader's search path
    const bool forced = !g_nccl_path.empty();
    const char* candidates[] = {forced ? g_nccl_path.c_str() : "libnccl.so.2", forced ? nullptr : "libnccl.so"};
    void* h = nullptr;
    std::string tried;
    for (const char* c : candidates) {
      if (c == nullptr) continue;
      h = dlopen(c, RTLD_NOW | RTLD_GLOBAL);
      if (h) break;
      tried += std::string(tried.empty() ? "" : ", ") + c;
    }
    if (!h) return set_error(TWG_ERR_UNSUPPORTED, "NCCL is not available: could not load %s", tried.c_str());
    NcclApi api;
    api.handle = h;
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(h, "ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
    api.GetVersion = reinterpret_cast<decltype(api.GetVersion)>(dlsym(h, "ncclGetVersion"));
    if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllGather || !api.GetErrorString) {
      dlclose(h);
      return set_error(TWG_ERR_UNSUPPORTED, "the NCCL library that was found lacks a required symbol");
    }
    g_nccl = api;
  }
  *out = &g_nccl;
  return TWG_OK;
}

static int nccl_fail(NcclApi* api, int rc, const char* what) {
  return set_error(TWG_ERR_CUDA, "%s failed: %s (ncclResult %d)", what, api->GetErrorString(rc), rc);
}

struct Comm {
  unsigned magic;
  void* nccl;
  int rank, nranks, device;
};
constexpr unsigned kCommMagic = 0x54574743u;  // "TWGC"

// ------------------------------------------------------------------------------------------
// peer-store exchange
// ------------------------------------------------------------------------------------------
constexpr int kXchgMaxRanks = TWG_EXCHANGE_MAX_RANKS;
constexpr unsigned kXchgMagic = 0x54574758u;  // "TWGX"

struct PeerSlots { u64* p[kXchgMaxRanks]; };

struct Xchg {
  unsigned magic;
  int rank, nranks, ring, device;
  u64* mailbox;                  // device: ring x nranks x {count, sequence << 8 | status}
  u64* peer[kXchgMaxRanks];      // every rank's mailbox as seen from this device
  bool opened[kXchgMaxRanks];    // peer[r] came from cudaIpcOpenMemHandle
  i64* gathered;                 // device: ring x record
  i64* host;                     // mapped pinned: ring x record
  i64* host_dev;                 // device alias of `host`
  i64 timeout_ns;
  int record() const { return 2 * nranks + 4; }  // counts, statuses, offset, total, done sequence, spare
};

__device__ __forceinline__ void st_release_sys(u64* p, u64 v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ u64 ld_acquire_sys(const u64* p) {
  u64 v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ u64 ld_relaxed_sys(const u64* p) {
  u64 v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ u64 global_timer_ns() {
  u64 t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Lane r stores this rank's {count, sequence | status} into rank r's mailbox.
__global__ void xchg_publish_kernel(PeerSlots peers, int nranks, int my_rank, int slot, u64 seq, const i64* result) {
  const int r = threadIdx.x;
  if (r >= nranks) return;
  u64* p = peers.p[r] + ((size_t)slot * nranks + my_rank) * 2;
  const u64 count = (u64)result[0];
  const u64 status = (u64)result[1] & 0xffull;
  p[0] = count;
  st_release_sys(p + 1, (seq << 8) | status);  // orders the count before the flag
}

// One warp.  Lane r waits until rank r's publication of `seq` has landed in this rank's mailbox
// (or the time limit runs out: that lane reports TWG_ERR_TIMEOUT), then the warp writes
// {counts, statuses, this rank's offset, total} to device memory and to the host record, whose
// last word (the sequence number) tells the polling host that the record is complete.
__global__ void xchg_collect_kernel(const u64* mailbox_slot, int nranks, int my_rank, u64 seq, i64 timeout_ns,
                                    i64* gathered, i64* host) {
  const int lane = threadIdx.x;
  i64 count = 0, status = 0;
  if (lane < nranks) {
    const u64* p = mailbox_slot + 2 * lane;
    const u64 t0 = global_timer_ns();
    unsigned polls = 0;
    while (true) {
      const u64 flag = ld_acquire_sys(p + 1);
      if ((flag >> 8) == seq) {
        count = (i64)ld_relaxed_sys(p);
        status = (i64)(signed char)(flag & 0xffull);
        break;
      }
      if (++polls > 16u) {
        if ((i64)(global_timer_ns() - t0) > timeout_ns) {
          status = TWG_ERR_TIMEOUT;
          break;
        }
        __nanosleep(200);
      }
    }
  }
  i64 before = lane < my_rank ? count : 0, total = count;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    before += __shfl_xor_sync(0xffffffffu, before, o);
    total += __shfl_xor_sync(0xffffffffu, total, o);
  }
  if (lane < nranks) {
    gathered[lane] = count;
    gathered[nranks + lane] = status;
    host[lane] = count;
    host[nranks + lane] = status;
  }
  if (lane == 0) {
    gathered[2 * nranks] = before;
    gathered[2 * nranks + 1] = total;
    host[2 * nranks] = before;
    host[2 * nranks + 1] = total;
  }
  __threadfence_system();
  __syncwarp();
  if (lane == 0) st_release_sys(reinterpret_cast<u64*>(host + 2 * nranks + 2), seq);
}

// Makes `dev` current for the lifetime of the object (peers are opened from the owning device).
struct ScopedDeviceGuard {
  int prev = -1;
  bool switched = false;
  explicit ScopedDeviceGuard(int dev) {
    if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) switched = cudaSetDevice(dev) == cudaSuccess;
  }
  ~ScopedDeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

static Xchg* as_xchg(void* p) {
  Xchg* x = static_cast<Xchg*>(p);
  return (x != nullptr && x->magic == kXchgMagic) ? x : nullptr;
}

}  // namespace twg

using namespace twg;

// ---- NCCL ----------------------------------------------------------------------------------
extern "C" int twg_comm_set_nccl_path(const char* path) {
  std::lock_guard<std::mutex> lock(g_nccl_mu);
  g_nccl_path = path ? path : "";
  return TWG_OK;
}

extern "C" int twg_comm_unique_id(void* out128) {
  TWG_REQUIRE(out128 != nullptr, "twg_comm_unique_id: output is null");
  NcclApi* api = nullptr;
  if (int rc = nccl_api(&api)) return rc;
  NcclId id;
  std::memset(&id, 0, sizeof(id));
  if (int rc = api->GetUniqueId(&id)) return nccl_fail(api, rc, "ncclGetUniqueId");
  std::memcpy(out128, id.bytes, sizeof(id.bytes));
  return TWG_OK;
}

extern "C" int twg_comm_init_rank(const void* unique_id, int rank, int nranks, void** comm) {
  TWG_REQUIRE(comm != nullptr, "twg_comm_init_rank: comm is null");
  *comm = nullptr;
  TWG_REQUIRE(unique_id != nullptr, "twg_comm_init_rank: unique_id is null");
  TWG_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, "twg_comm_init_rank: rank %d is outside a world of %d", rank,
              nranks);
  bool any = false;
  for (int i = 0; i < TWG_COMM_ID_BYTES; ++i) any = any || static_cast<const char*>(unique_id)[i] != 0;
  TWG_REQUIRE(any, "twg_comm_init_rank: the unique id is all zeros (not produced by twg_comm_unique_id)");
  NcclApi* api = nullptr;
  if (int rc = nccl_api(&api)) return rc;
  int dev = 0;
  TWG_CUDA(cudaGetDevice(&dev));
  NcclId id;
  std::memcpy(id.bytes, unique_id, sizeof(id.bytes));
  void* nc = nullptr;
  if (int rc = api->CommInitRank(&nc, nranks, id, rank)) return nccl_fail(api, rc, "ncclCommInitRank");
  *comm = new Comm{kCommMagic, nc, rank, nranks, dev};
  return TWG_OK;
}

extern "C" int twg_comm_destroy(void* comm) {
  if (comm == nullptr) return TWG_OK;
  Comm* c = static_cast<Comm*>(comm);
  TWG_REQUIRE(c->magic == kCommMagic, "twg_comm_destroy: not a communicator");
  NcclApi* api = nullptr;
  if (int rc = nccl_api(&api)) return rc;
  const int rc = api->CommDestroy(c->nccl);
  c->magic = 0;
  delete c;
  if (rc) return nccl_fail(api, rc, "ncclCommDestroy");
  return TWG_OK;
}

extern "C" int twg_allgather_i64(void* comm, const int64_t* send_dev, int64_t* recv_dev, int n, void* stream) {
  TWG_TRACE("twg_allgather_i64");
  Comm* c = static_cast<Comm*>(comm);
  TWG_REQUIRE(c != nullptr && c->magic == kCommMagic, "twg_allgather_i64: not a communicator");
  TWG_REQUIRE(n >= 0, "twg_allgather_i64: negative count");
  if (n == 0) return TWG_OK;
  TWG_REQUIRE(send_dev != nullptr && recv_dev != nullptr, "twg_allgather_i64: null buffer");
  NcclApi* api = nullptr;
  if (int rc = nccl_api(&api)) return rc;
  if (int rc = api->AllGather(send_dev, recv_dev, (size_t)n, kNcclInt64, c->nccl, static_cast<cudaStream_t>(stream)))
    return nccl_fail(api, rc, "ncclAllGather");
  return TWG_OK;
}

// ---- peer-store exchange ---------------------------------------------------------------------
extern "C" int twg_exchange_create(int rank, int nranks, int ring, void** xchg) {
  TWG_REQUIRE(xchg != nullptr, "twg_exchange_create: output is null");
  *xchg = nullptr;
  TWG_REQUIRE(nranks >= 1 && nranks <= kXchgMaxRanks, "twg_exchange_create: %d ranks (1..%d supported)", nranks,
              kXchgMaxRanks);
  TWG_REQUIRE(rank >= 0 && rank < nranks, "twg_exchange_create: rank %d is outside a world of %d", rank, nranks);
  TWG_REQUIRE(ring >= 2 && ring <= 1024 && ring % 2 == 0, "twg_exchange_create: ring must be even, 2..1024 (got %d)", ring);
  Xchg* x = new Xchg();
  std::memset(x, 0, sizeof(*x));
  x->rank = rank;
  x->nranks = nranks;
  x->ring = ring;
  x->timeout_ns = 2000000000ll;
  auto fail = [&](int rc) {
    if (x->mailbox) cudaFree(x->mailbox);
    if (x->gathered) cudaFree(x->gathered);
    if (x->host) cudaFreeHost(x->host);
    delete x;
    return rc;
  };
  cudaError_t e = cudaGetDevice(&x->device);
  if (e != cudaSuccess) return fail(cuda_fail(e, "cudaGetDevice", __FILE__, __LINE__));
  const size_t mailbox_bytes = (size_t)ring * nranks * 2 * sizeof(u64);
  const size_t record_bytes = (size_t)ring * x->record() * sizeof(i64);
  // a dedicated cudaMalloc: the block is exported whole through an IPC handle
  if ((e = cudaMalloc(reinterpret_cast<void**>(&x->mailbox), mailbox_bytes)) != cudaSuccess)
    return fail(cuda_fail(e, "cudaMalloc(mailbox)", __FILE__, __LINE__));
  if ((e = cudaMemset(x->mailbox, 0, mailbox_bytes)) != cudaSuccess) return fail(cuda_fail(e, "cudaMemset", __FILE__, __LINE__));
  if ((e = cudaMalloc(reinterpret_cast<void**>(&x->gathered), record_bytes)) != cudaSuccess)
    return fail(cuda_fail(e, "cudaMalloc(gathered)", __FILE__, __LINE__));
  if ((e = cudaMemset(x->gathered, 0, record_bytes)) != cudaSuccess) return fail(cuda_fail(e, "cudaMemset", __FILE__, __LINE__));
  if ((e = cudaHostAlloc(reinterpret_cast<void**>(&x->host), record_bytes, cudaHostAllocMapped)) != cudaSuccess)
    return fail(cuda_fail(e, "cudaHostAlloc", __FILE__, __LINE__));
  std::memset(x->host, 0, record_bytes);
  if ((e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&x->host_dev), x->host, 0)) != cudaSuccess)
    return fail(cuda_fail(e, "cudaHostGetDevicePointer", __FILE__, __LINE__));
  if ((e = cudaDeviceSynchronize()) != cudaSuccess) return fail(cuda_fail(e, "cudaDeviceSynchronize", __FILE__, __LINE__));
  x->peer[rank] = x->mailbox;
  x->magic = kXchgMagic;
  *xchg = x;
  return TWG_OK;
}

extern "C" int twg_exchange_handle(void* xchg, void* out64) {
  Xchg* x = as_xchg(xchg);
  TWG_REQUIRE(x != nullptr && out64 != nullptr, "twg_exchange_handle: bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == TWG_EXCHANGE_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  TWG_CUDA(cudaIpcGetMemHandle(&h, x->mailbox));
  std::memcpy(out64, &h, sizeof(h));
  return TWG_OK;
}

extern "C" int twg_exchange_connect_ipc(void* xchg, int peer_rank, const void* handle64) {
  Xchg* x = as_xchg(xchg);
  TWG_REQUIRE(x != nullptr && handle64 != nullptr, "twg_exchange_connect_ipc: bad argument");
  TWG_REQUIRE(peer_rank >= 0 && peer_rank < x->nranks, "twg_exchange_connect_ipc: rank %d is outside a world of %d",
              peer_rank, x->nranks);
  if (peer_rank == x->rank) return TWG_OK;
  TWG_REQUIRE(x->peer[peer_rank] == nullptr, "twg_exchange_connect_ipc: rank %d is already connected", peer_rank);
  ScopedDeviceGuard guard(x->device);
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  TWG_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  x->peer[peer_rank] = static_cast<u64*>(p);
  x->opened[peer_rank] = true;
  return TWG_OK;
}

extern "C" int twg_exchange_connect_local(void* xchg, int peer_rank, void* peer_xchg) {
  Xchg* x = as_xchg(xchg);
  Xchg* y = as_xchg(peer_xchg);
  TWG_REQUIRE(x != nullptr && y != nullptr, "twg_exchange_connect_local: bad argument");
  TWG_REQUIRE(peer_rank >= 0 && peer_rank < x->nranks && y->rank == peer_rank && y->nranks == x->nranks &&
                  y->ring == x->ring,
              "twg_exchange_connect_local: the peer object is not rank %d of the same world", peer_rank);
  if (peer_rank == x->rank) return TWG_OK;
  if (y->device != x->device) {
    ScopedDeviceGuard guard(x->device);
    int can = 0;
    TWG_CUDA(cudaDeviceCanAccessPeer(&can, x->device, y->device));
    if (!can)
      return set_error(TWG_ERR_UNSUPPORTED, "twg_exchange_connect_local: device %d cannot access device %d", x->device,
                       y->device);
    cudaError_t e = cudaDeviceEnablePeerAccess(y->device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
    else if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceEnablePeerAccess", __FILE__, __LINE__);
  }
  x->peer[peer_rank] = y->mailbox;
  return TWG_OK;
}

static int xchg_ready(Xchg* x, const char* who) {
  for (int r = 0; r < x->nranks; ++r)
    if (x->peer[r] == nullptr) return set_error(TWG_ERR_INVALID, "%s: rank %d is not connected yet", who, r);
  return TWG_OK;
}

namespace twg {
int xchg_publish_slots(void* xchg, int64_t seq, MsPublish* out) {
  Xchg* x = as_xchg(xchg);
  TWG_REQUIRE(x != nullptr && out != nullptr, "count exchange: not an exchange object");
  TWG_REQUIRE(seq >= 1 && seq < (int64_t(1) << 55), "count exchange: sequence numbers start at 1 (got %lld)", (long long)seq);
  if (int rc = xchg_ready(x, "count exchange")) return rc;
  const int slot = (int)(seq % x->ring);
  for (int r = 0; r < kXchgMaxRanks; ++r)
    out->slot[r] = r < x->nranks ? x->peer[r] + ((size_t)slot * x->nranks + x->rank) * 2 : nullptr;
  out->nranks = x->nranks;
  out->seq = (u64)seq;
  return TWG_OK;
}
}  // namespace twg

extern "C" int twg_exchange_publish(void* xchg, int64_t seq, const int64_t* result_dev, void* stream) {
  TWG_TRACE("twg_exchange_publish");
  Xchg* x = as_xchg(xchg);
  TWG_REQUIRE(x != nullptr && result_dev != nullptr, "twg_exchange_publish: bad argument");
  TWG_REQUIRE(seq >= 1 && seq < (int64_t(1) << 55), "twg_exchange_publish: sequence numbers start at 1 (got %lld)",
              (long long)seq);
  if (int rc = xchg_ready(x, "twg_exchange_publish")) return rc;
  PeerSlots peers;
  for (int r = 0; r < kXchgMaxRanks; ++r) peers.p[r] = r < x->nranks ? x->peer[r] : nullptr;
  xchg_publish_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(peers, x->nranks, x->rank, (int)(seq % x->ring),
                                                                        (u64)seq, reinterpret_cast<const i64*>(result_dev));
  TWG_CHECK_LAUNCH();
  return TWG_OK;
}

extern "C" int twg_exchange_collect(void* xchg, int64_t seq, void* stream) {
  TWG_TRACE("twg_exchange_collect");
  Xchg* x = as_xchg(xchg);
  TWG_REQUIRE(x != nullptr, "twg_exchange_collect: bad argument");
  TWG_REQUIRE(seq >= 1 && seq < (int64_t(1) << 55), "twg_exchange_collect: sequence numbers start at 1 (got %lld)",
              (long long)seq);
  const int slot = (int)(seq % x->ring);
  xchg_collect_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      x->mailbox + (size_t)slot * x->nranks * 2, x->nranks, x->rank, (u64)seq, x->timeout_ns,
      x->gathered + (size_t)slot * x->record(), x->host_dev + (size_t)slot * x->record());
  TWG_CHECK_LAUNCH();
  return TWG_OK;
}

extern "C" int twg_exchange_wait(void* xchg, int64_t seq, int64_t* counts, int64_t* statuses, int64_t* offset,
                                 int64_t* total, int timeout_ms) {
  TWG_TRACE("twg_exchange_wait");
  Xchg* x = as_xchg(xchg);
  TWG_REQUIRE(x != nullptr, "twg_exchange_wait: bad argument");
  TWG_REQUIRE(seq >= 1, "twg_exchange_wait: sequence numbers start at 1");
  const int n = x->nranks;
  const i64* rec = x->host + (size_t)(seq % x->ring) * x->record();
  const volatile i64* done = rec + 2 * n + 2;
  const auto t0 = std::chrono::steady_clock::now();
  unsigned spins = 0;
  while (*done != (i64)seq) {
    if ((++spins & 0x3ffu) == 0u) {
      const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
      if (timeout_ms >= 0 && ms > timeout_ms)
        return set_error(TWG_ERR_TIMEOUT, "twg_exchange_wait: sequence %lld did not complete within %d ms (slot holds %lld)",
                         (long long)seq, timeout_ms, (long long)*done);
      if (ms > 2) sched_yield();
    }
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  }
  std::atomic_thread_fence(std::memory_order_acquire);
  int worst = TWG_OK;
  for (int r = 0; r < n; ++r) {
    if (counts) counts[r] = rec[r];
    if (statuses) statuses[r] = rec[n + r];
    if (rec[n + r] != 0 && worst == TWG_OK) worst = (int)rec[n + r];
  }
  if (offset) *offset = rec[2 * n];
  if (total) *total = rec[2 * n + 1];
  if (worst != TWG_OK)
    return set_error(worst, "twg_exchange_wait: sequence %lld completed with a device status of %d on some rank",
                     (long long)seq, worst);
  return TWG_OK;
}

extern "C" int twg_exchange_gathered(void* xchg, int64_t seq, const int64_t** dev_record) {
  Xchg* x = as_xchg(xchg);
  TWG_REQUIRE(x != nullptr && dev_record != nullptr && seq >= 1, "twg_exchange_gathered: bad argument");
  *dev_record = reinterpret_cast<const int64_t*>(x->gathered + (size_t)(seq % x->ring) * x->record());
  return TWG_OK;
}

extern "C" int twg_exchange_set_timeout_ns(void* xchg, int64_t timeout_ns) {
  Xchg* x = as_xchg(xchg);
  TWG_REQUIRE(x != nullptr, "twg_exchange_set_timeout_ns: bad argument");
  x->timeout_ns = timeout_ns > 0 ? timeout_ns : 2000000000ll;
  return TWG_OK;
}

extern "C" int twg_exchange_destroy(void* xchg) {
  if (xchg == nullptr) return TWG_OK;
  Xchg* x = as_xchg(xchg);
  TWG_REQUIRE(x != nullptr, "twg_exchange_destroy: not an exchange object");
  ScopedDeviceGuard guard(x->device);
  cudaDeviceSynchronize();
  for (int r = 0; r < x->nranks; ++r)
    if (x->opened[r] && x->peer[r]) cudaIpcCloseMemHandle(x->peer[r]);
  cudaFree(x->mailbox);
  cudaFree(x->gathered);
  cudaFreeHost(x->host);
  cudaGetLastError();
  x->magic = 0;
  delete x;
  return TWG_OK;
}
