// masked_select as a single-pass stream compaction.
//
// One CTA owns one tile of 4096 logical elements.  Inside the tile, selected elements are ranked
// with popc on the packed mask bytes plus a warp scan (dense path) or with warp ballots (strided
// path); the tile's base offset in the output comes from a decoupled look-back over the
// preceding tiles' published counts, so the input is read exactly once and no second pass or
// global scan is needed.  Selected values are first packed into shared memory in output order and
// then written as contiguous runs.
//
// Forward progress: a tile's index is a ticket drawn from a global counter when its CTA starts,
// not blockIdx, so every tile a CTA may wait for belongs to a CTA that is already running.  The
// wait is nevertheless bounded: after `poll_budget` polls the tile gives up, records
// TWG_ERR_TIMEOUT in result[1], publishes a prefix so that later tiles do not wait on it, and the
// kernel drains normally.
#include "twg_launch.cuh"

#include <atomic>

namespace twg {

constexpr int kMsThreads = 256;
constexpr int kMsWarps = kMsThreads / 32;
constexpr int kMsPerThread = 16;
constexpr int kMsTile = kMsThreads * kMsPerThread;  // 4096
constexpr size_t kMsHeaderBytes = 256;              // ticket counter, padded

constexpr u64 kMsAggregate = 1ull << 62;
constexpr u64 kMsPrefix = 2ull << 62;
constexpr u64 kMsValueMask = (1ull << 62) - 1ull;

static std::atomic<long long> g_poll_budget{4000000};

__device__ __forceinline__ u64 ld_relaxed_u64(const u64* p) {
  u64 v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_u64(u64* p, u64 v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ u64 warp_sum_u64(u64 v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct MsShared {
  float stage[kMsTile];
  u32 warp_total[kMsWarps];
  i64 tile;
  i64 excl;
};

// Executed by warp 0 only.  Publishes this tile's count, resolves the number of selected
// elements in all earlier tiles, publishes the inclusive prefix and returns the exclusive one.
__device__ __forceinline__ i64 lookback(i64 tile, u32 tile_total, u64* desc, i64* result, i64 poll_budget) {
  const int lane = threadIdx.x & 31;
  // A negative budget is the test hook "tile 0 never publishes": every wait that depends on it
  // must run out after |budget| polls and report TWG_ERR_TIMEOUT instead of hanging.
  const bool withhold_first = poll_budget < 0;
  if (withhold_first) poll_budget = -poll_budget;
  if (tile == 0) {
    if (lane == 0 && !withhold_first) st_relaxed_u64(desc, kMsPrefix | (u64)tile_total);
    return 0;
  }
  if (lane == 0) st_relaxed_u64(desc + tile, kMsAggregate | (u64)tile_total);
  u64 excl = 0;
  i64 look = tile - 1;  // nearest predecessor not yet accounted for
  i64 polls = 0;
  bool timed_out = false;
  while (true) {
    const i64 idx = look - lane;
    const u64 d = idx >= 0 ? ld_relaxed_u64(desc + idx) : kMsPrefix;  // before tile 0: prefix of 0
    const u32 status = (u32)(d >> 62);
    const u32 invalid = __ballot_sync(0xffffffffu, status == 0u);
    const u32 prefix = __ballot_sync(0xffffffffu, status == 2u);
    if (prefix != 0u) {
      const int p = __ffs(prefix) - 1;  // nearest tile that already knows its inclusive prefix
      const u32 need = p == 31 ? 0xffffffffu : ((1u << (p + 1)) - 1u);
      if ((invalid & need) == 0u) {
        excl += warp_sum_u64(lane <= p ? (d & kMsValueMask) : 0ull);
        break;
      }
    } else if (invalid == 0u) {
      excl += warp_sum_u64(d & kMsValueMask);  // 32 aggregates, keep walking back
      look -= 32;
      continue;
    }
    if (++polls > poll_budget) { timed_out = true; break; }
    if (polls > 64) __nanosleep(100);
  }
  if (timed_out) {
    excl = 0;
    if (lane == 0) result[1] = (i64)TWG_ERR_TIMEOUT;
  }
  if (lane == 0) st_relaxed_u64(desc + tile, kMsPrefix | ((excl + (u64)tile_total) & kMsValueMask));
  return (i64)excl;
}

// Common tail of both kernels: turn per-warp totals into a tile total, run the look-back, and
// return (exclusive global prefix, this warp's offset in the tile, tile total).
__device__ __forceinline__ void tile_offsets(MsShared& sm, u32 warp_total, i64 tile, i64 ntiles, u64* desc,
                                             i64* result, i64 poll_budget, u32* warp_off, u32* tile_total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sm.warp_total[warp] = warp_total;
  __syncthreads();
  u32 off = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kMsWarps; ++w) {
    const u32 t = sm.warp_total[w];
    if (w < warp) off += t;
    tot += t;
  }
  *warp_off = off;
  *tile_total = tot;
  if (warp == 0) {
    const i64 excl = lookback(tile, tot, desc, result, poll_budget);
    if (lane == 0) {
      sm.excl = excl;
      if (tile == ntiles - 1) result[0] = excl + (i64)tot;
    }
  }
}

__device__ __forceinline__ void flush_stage(const MsShared& sm, float* out, u32 tile_total) {
  const i64 excl = sm.excl;
  for (u32 i = threadIdx.x; i < tile_total; i += kMsThreads) out[excl + i] = sm.stage[i];
}

// ------------------------------------------------------------------------------------------
// Dense path: src and mask contiguous, src 16-byte and mask 4-byte aligned.  A warp covers 512
// consecutive elements as 4 rounds of 32 quads; lane l owns quad j*32+l of round j, so the mask
// is read as one 128-byte run and src as one 512-byte run per round.  src quads whose four mask
// bytes are all zero are not read at all.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kMsThreads)
    ms_dense_kernel(const float* src, const u8* mask, float* out, i64 n, i64 ntiles, u64* ticket, u64* desc,
                    i64* result, i64 poll_budget) {
  __shared__ MsShared sm;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) sm.tile = (i64)atomicAdd(ticket, 1ull);
  __syncthreads();
  const i64 tile = sm.tile;
  if (tile >= ntiles) return;
  const i64 warp_base = tile * kMsTile + (i64)warp * (32 * kMsPerThread);

  u32 m[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const i64 e = warp_base + (i64)(j * 32 + lane) * 4;
    u32 w = 0;
    if (e + 3 < n) {
      w = ld_b32(mask + e);
    } else {
      for (int b = 0; b < 4; ++b)
        if (e + b < n) w |= ld_b8(mask + e + b) << (8 * b);
    }
    m[j] = __vcmpne4(w, 0u) & 0x01010101u;
  }
  u32 v[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const i64 e = warp_base + (i64)(j * 32 + lane) * 4;
    if (m[j] != 0u) {
      if (e + 3 < n) {
        const uint4 q = ld_v4(src + e);
        v[j][0] = q.x; v[j][1] = q.y; v[j][2] = q.z; v[j][3] = q.w;
      } else {
#pragma unroll
        for (int b = 0; b < 4; ++b) v[j][b] = (e + b < n) ? ld_b32(src + e + b) : 0u;
      }
    }
  }

  // ranks: per-round counts packed into one word (each field <= 128 after the warp scan)
  const u32 cnt = __popc(m[0]) | (__popc(m[1]) << 8) | (__popc(m[2]) << 16) | (__popc(m[3]) << 24);
  u32 incl = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const u32 t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  const u32 tot = __shfl_sync(0xffffffffu, incl, 31);
  const u32 t0 = tot & 0xffu, t1 = (tot >> 8) & 0xffu, t2 = (tot >> 16) & 0xffu, t3 = tot >> 24;
  const u32 excl_w = incl - cnt;  // per-field exclusive scan across lanes
  u32 warp_off, tile_total;
  tile_offsets(sm, t0 + t1 + t2 + t3, tile, ntiles, desc, result, poll_budget, &warp_off, &tile_total);

  const u32 round_base[4] = {0u, t0, t0 + t1, t0 + t1 + t2};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (m[j] != 0u) {
      u32 r = warp_off + round_base[j] + ((excl_w >> (8 * j)) & 0xffu);
#pragma unroll
      for (int b = 0; b < 4; ++b)
        if ((m[j] >> (8 * b)) & 1u) sm.stage[r++] = __uint_as_float(v[j][b]);
    }
  }
  __syncthreads();
  flush_stage(sm, out, tile_total);
}

// ------------------------------------------------------------------------------------------
// Strided / broadcast path.  Logical element e (row-major over the broadcast shape) is mapped to
// a src offset and a mask offset with the descriptor's strides (0 = broadcast).  Lane l of a warp
// owns elements warp_base + i*32 + l, i = 0..15, so that a ballot over the warp is the selection
// bitmap of 32 consecutive elements and popc of its low bits is the rank.
// ------------------------------------------------------------------------------------------
template <class IDX>
__global__ void __launch_bounds__(kMsThreads)
    ms_strided_kernel(const float* src, const u8* mask, float* out, StridedDesc<2, IDX> d, i64 n, i64 ntiles,
                      u64* ticket, u64* desc, i64* result, i64 poll_budget) {
  __shared__ MsShared sm;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) sm.tile = (i64)atomicAdd(ticket, 1ull);
  __syncthreads();
  const i64 tile = sm.tile;
  if (tile >= ntiles) return;
  const i64 warp_base = tile * kMsTile + (i64)warp * (32 * kMsPerThread);

  u32 flags = 0;                 // bit i: element i of this lane is selected
  u32 v[kMsPerThread];
  u32 before[kMsPerThread];      // selected elements of this warp that precede element i of this lane
  u32 running = 0;
#pragma unroll
  for (int i = 0; i < kMsPerThread; ++i) {
    const i64 e = warp_base + i * 32 + lane;
    bool sel = false;
    if (e < n) {
      i64 off[2];
      linear_to_offsets<2>(d, (IDX)e, off);
      sel = ld_b8(mask + off[1]) != 0u;
      if (sel) v[i] = ld_b32(src + off[0]);
    }
    const u32 b = __ballot_sync(0xffffffffu, sel);
    before[i] = running + __popc(b & ((1u << lane) - 1u));
    running += __popc(b);
    if (sel) flags |= 1u << i;
  }
  u32 warp_off, tile_total;
  tile_offsets(sm, running, tile, ntiles, desc, result, poll_budget, &warp_off, &tile_total);
#pragma unroll
  for (int i = 0; i < kMsPerThread; ++i)
    if ((flags >> i) & 1u) sm.stage[warp_off + before[i]] = __uint_as_float(v[i]);
  __syncthreads();
  flush_stage(sm, out, tile_total);
}

}  // namespace twg

using namespace twg;

extern "C" size_t twg_masked_select_workspace_bytes(int64_t numel) {
  if (numel < 0) numel = 0;
  const int64_t ntiles = (numel + kMsTile - 1) / kMsTile;
  return kMsHeaderBytes + (size_t)ntiles * sizeof(u64);
}

extern "C" int twg_masked_select_set_poll_budget(int64_t polls) {
  g_poll_budget.store(polls != 0 ? polls : 4000000);
  return TWG_OK;
}

extern "C" int twg_masked_select_f32(const TwgIterDesc* desc, const float* src, const uint8_t* mask, float* out,
                                     int64_t* result_dev, void* workspace, size_t workspace_bytes, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  g_last_path = kPathNone;
  if (int rc = check_desc(desc, 2)) return rc;
  TWG_REQUIRE(result_dev != nullptr, "twg_masked_select_f32: result_dev is null");
  TWG_CUDA(cudaMemsetAsync(result_dev, 0, 2 * sizeof(int64_t), s));
  const int64_t n = desc->numel;
  if (n == 0) return TWG_OK;
  TWG_REQUIRE(src && mask && out, "twg_masked_select_f32: null operand");
  const size_t need = twg_masked_select_workspace_bytes(n);
  TWG_REQUIRE(workspace != nullptr && workspace_bytes >= need,
              "twg_masked_select_f32: workspace of %zu bytes is smaller than the %zu required", workspace_bytes, need);
  TWG_REQUIRE(is_aligned(workspace, 256), "twg_masked_select_f32: workspace is not 256-byte aligned");
  TWG_REQUIRE(is_aligned(src, 4) && is_aligned(out, 4), "twg_masked_select_f32: src/out not 4-byte aligned");

  TwgIterDesc d = *desc;
  d.ntensors = 2;
  if (int rc = twg_iter_coalesce(&d)) return rc;
  const int64_t ntiles = (n + kMsTile - 1) / kMsTile;
  TWG_REQUIRE(ntiles <= 0x7fffffff, "twg_masked_select_f32: %lld elements exceed the tile limit", (long long)n);
  TWG_CUDA(cudaMemsetAsync(workspace, 0, need, s));
  u64* ticket = static_cast<u64*>(workspace);
  u64* tdesc = reinterpret_cast<u64*>(static_cast<char*>(workspace) + kMsHeaderBytes);
  const long long budget = g_poll_budget.load();

  const bool dense = (d.ndim == 0 || (d.ndim == 1 && (n == 1 || (d.strides[0][0] == 1 && d.strides[1][0] == 1)))) &&
                     is_aligned(src, 16) && is_aligned(mask, 4);
  if (dense) {
    ms_dense_kernel<<<(unsigned)ntiles, kMsThreads, 0, s>>>(src, mask, out, n, ntiles, ticket, tdesc, reinterpret_cast<i64*>(result_dev), budget);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathDense;
    return TWG_OK;
  }
  if (fits_32bit(d, 2)) {
    StridedDesc<2, u32> sd;
    fill_strided_desc<2>(d, &sd);
    ms_strided_kernel<u32><<<(unsigned)ntiles, kMsThreads, 0, s>>>(src, mask, out, sd, n, ntiles, ticket, tdesc,
                                                                   reinterpret_cast<i64*>(result_dev), budget);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathStrided32;
  } else {
    StridedDesc<2, u64> sd;
    fill_strided_desc<2>(d, &sd);
    ms_strided_kernel<u64><<<(unsigned)ntiles, kMsThreads, 0, s>>>(src, mask, out, sd, n, ntiles, ticket, tdesc,
                                                                   reinterpret_cast<i64*>(result_dev), budget);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathStrided64;
  }
  return TWG_OK;
}
