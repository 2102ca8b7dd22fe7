// masked_select as a single-pass stream compaction.
//
// One CTA owns one tile of consecutive logical elements.  Inside the tile, selected elements are
// ranked with popc on the packed mask bytes plus a warp scan (dense path) or with warp ballots
// (strided path); the tile's base offset in the output comes from a decoupled look-back over the
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
#include <cstdlib>

namespace twg {

constexpr int kMsThreads = 256;
constexpr int kMsWarps = kMsThreads / 32;
constexpr int kMsRound = kMsThreads * 16;           // 4096 elements: what one staging pass holds
constexpr int kMsMaxRounds = 4;                     // dense tiles are 1, 2 or 4 rounds
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
  float stage[kMsRound];
  u32 warp_total[kMsMaxRounds][kMsWarps];
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
    // lanes nearer than the first unpublished tile can be consumed right away
    const int first_invalid = invalid ? __ffs(invalid) - 1 : 32;
    const int first_prefix = prefix ? __ffs(prefix) - 1 : 32;
    if (first_prefix < first_invalid) {
      excl += warp_sum_u64(lane <= first_prefix ? (d & kMsValueMask) : 0ull);
      break;
    }
    if (first_invalid > 0) {
      // consume the published aggregates in front of the gap and continue from the gap
      excl += warp_sum_u64(lane < first_invalid ? (d & kMsValueMask) : 0ull);
      look -= first_invalid;
      if (first_invalid == 32) continue;
    }
    if (++polls > poll_budget) { timed_out = true; break; }
    if (polls > 32) __nanosleep(64);
  }
  if (timed_out) {
    excl = 0;
    if (lane == 0) result[1] = (i64)TWG_ERR_TIMEOUT;
  }
  if (lane == 0) st_relaxed_u64(desc + tile, kMsPrefix | ((excl + (u64)tile_total) & kMsValueMask));
  return (i64)excl;
}

// Write `count` staged values to out[base ...].  Runs of a tile are contiguous, so everything
// between the first and last 16-byte boundary goes out as 128-bit stores.
__device__ __forceinline__ void flush_stage(const float* stage, float* out, i64 base, u32 count) {
  float* dst = out + base;
  const u32 head = min(count, (u32)(((16u - (u32)(reinterpret_cast<unsigned long long>(dst) & 15ull)) & 15u) >> 2));
  if (threadIdx.x < head) dst[threadIdx.x] = stage[threadIdx.x];
  const u32 nvec = (count - head) >> 2;
  float4* dst4 = reinterpret_cast<float4*>(dst + head);
  for (u32 i = threadIdx.x; i < nvec; i += kMsThreads) {
    const float* s = stage + head + 4 * i;
    dst4[i] = make_float4(s[0], s[1], s[2], s[3]);
  }
  const u32 tail0 = head + 4 * nvec;
  if (tail0 + threadIdx.x < count) dst[tail0 + threadIdx.x] = stage[tail0 + threadIdx.x];
}

// ------------------------------------------------------------------------------------------
// Dense path: src contiguous and 16-byte aligned; the mask is either a dense bool array (4-byte
// aligned) or, with ROWMASK, one bool per row of `row_len` elements (a [R,1] mask broadcast over
// [R,C] with C % 4 == 0).  A tile is ROUNDS rounds of 4096 elements.  In a round a warp covers
// 512 consecutive elements as 4 sub-rounds of 32 quads; lane l owns quad j*32+l of sub-round j, so
// the mask is read as 128-byte runs and src as 512-byte runs.  Every load of the tile is issued
// before the first use: with a dense mask src does not wait for the mask; with a row mask the
// (cached) row flag is read first and unselected rows are never fetched.
// ------------------------------------------------------------------------------------------
template <int ROUNDS, bool ROWMASK>
__global__ void __launch_bounds__(kMsThreads)
    ms_dense_kernel(const float* src, const u8* mask, float* out, i64 n, i64 ntiles, u64* ticket, u64* desc,
                    i64* result, i64 poll_budget, FastDiv32 row_len) {
  __shared__ MsShared sm;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) sm.tile = (i64)atomicAdd(ticket, 1ull);
  __syncthreads();
  const i64 tile = sm.tile;
  if (tile >= ntiles) return;
  const i64 tile_base = tile * (i64)(ROUNDS * kMsRound) + (i64)warp * 512;

  u32 m[ROUNDS][4];
  u32 v[ROUNDS][4][4];
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const i64 e = tile_base + (i64)r * kMsRound + (i64)(j * 32 + lane) * 4;
      u32 w = 0;
      if constexpr (ROWMASK) {
        if (e < n) w = ld_b8(mask + row_len.div((u32)e)) != 0u ? 0x01010101u : 0u;  // n < 2^31 here
        if (e + 3 >= n && w) w &= (e + 2 < n) ? 0x00ffffffu : (e + 1 < n) ? 0x0000ffffu : 0x000000ffu;
      } else {
        if (e + 3 < n) {
          w = ld_b32(mask + e);
        } else {
          for (int b = 0; b < 4; ++b)
            if (e + b < n) w |= ld_b8(mask + e + b) << (8 * b);
        }
        w = __vcmpne4(w, 0u) & 0x01010101u;
      }
      m[r][j] = w;
      const bool want = ROWMASK ? (w != 0u) : true;
      if (want) {
        if (e + 3 < n) {
          const uint4 q = ld_v4(src + e);
          v[r][j][0] = q.x; v[r][j][1] = q.y; v[r][j][2] = q.z; v[r][j][3] = q.w;
        } else {
#pragma unroll
          for (int b = 0; b < 4; ++b) v[r][j][b] = (e + b < n) ? ld_b32(src + e + b) : 0u;
        }
      }
    }
  }

  // ranks inside a round: per-sub-round counts packed into one word (each field <= 128 after
  // the warp scan), one scan per round
  u32 excl_w[ROUNDS], sub_base[ROUNDS][4];
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    const u32 cnt = __popc(m[r][0]) | (__popc(m[r][1]) << 8) | (__popc(m[r][2]) << 16) | (__popc(m[r][3]) << 24);
    u32 incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const u32 t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const u32 tot = __shfl_sync(0xffffffffu, incl, 31);
    const u32 t0 = tot & 0xffu, t1 = (tot >> 8) & 0xffu, t2 = (tot >> 16) & 0xffu, t3 = tot >> 24;
    excl_w[r] = incl - cnt;
    sub_base[r][0] = 0u; sub_base[r][1] = t0; sub_base[r][2] = t0 + t1; sub_base[r][3] = t0 + t1 + t2;
    if (lane == 0) sm.warp_total[r][warp] = t0 + t1 + t2 + t3;
  }
  __syncthreads();
  u32 warp_off[ROUNDS], round_total[ROUNDS], tile_total = 0;
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    u32 off = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < kMsWarps; ++w) {
      const u32 t = sm.warp_total[r][w];
      if (w < warp) off += t;
      tot += t;
    }
    warp_off[r] = off;
    round_total[r] = tot;
    tile_total += tot;
  }
  if (warp == 0) {
    const i64 excl = lookback(tile, tile_total, desc, result, poll_budget);
    if (lane == 0) {
      sm.excl = excl;
      if (tile == ntiles - 1) result[0] = excl + (i64)tile_total;
    }
  }

  u32 round_base = 0;
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (m[r][j] != 0u) {
        u32 pos = warp_off[r] + sub_base[r][j] + ((excl_w[r] >> (8 * j)) & 0xffu);
#pragma unroll
        for (int b = 0; b < 4; ++b)
          if ((m[r][j] >> (8 * b)) & 1u) sm.stage[pos++] = __uint_as_float(v[r][j][b]);
      }
    }
    __syncthreads();  // stage complete (and, in round 0, sm.excl published)
    flush_stage(sm.stage, out, sm.excl + (i64)round_base, round_total[r]);
    round_base += round_total[r];
    if (r + 1 < ROUNDS) __syncthreads();  // stage free again
  }
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
  const i64 warp_base = tile * kMsRound + (i64)warp * 512;

  u32 flags = 0;       // bit i: element i of this lane is selected
  u32 v[16];
  u32 before[16];      // selected elements of this warp that precede element i of this lane
  u32 running = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
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
  if (lane == 0) sm.warp_total[0][warp] = running;
  __syncthreads();
  u32 warp_off = 0, tile_total = 0;
#pragma unroll
  for (int w = 0; w < kMsWarps; ++w) {
    const u32 t = sm.warp_total[0][w];
    if (w < warp) warp_off += t;
    tile_total += t;
  }
  if (warp == 0) {
    const i64 excl = lookback(tile, tile_total, desc, result, poll_budget);
    if (lane == 0) {
      sm.excl = excl;
      if (tile == ntiles - 1) result[0] = excl + (i64)tile_total;
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i)
    if ((flags >> i) & 1u) sm.stage[warp_off + before[i]] = __uint_as_float(v[i]);
  __syncthreads();
  flush_stage(sm.stage, out, sm.excl, tile_total);
}

// rounds per dense tile; TWG_MS_ROUNDS (1, 2 or 4) overrides it for experiments
static int dense_rounds() {
  static const int rounds = [] {
    const char* env = getenv("TWG_MS_ROUNDS");
    const int r = env ? atoi(env) : 0;
    return (r == 1 || r == 2 || r == 4) ? r : 2;
  }();
  return rounds;
}

template <bool ROWMASK>
static void launch_dense(int rounds, unsigned ntiles, cudaStream_t s, const float* src, const u8* mask, float* out, i64 n,
                         u64* ticket, u64* tdesc, i64* result, i64 budget, FastDiv32 row_len) {
  if (rounds == 1)
    ms_dense_kernel<1, ROWMASK><<<ntiles, kMsThreads, 0, s>>>(src, mask, out, n, ntiles, ticket, tdesc, result, budget, row_len);
  else if (rounds == 2)
    ms_dense_kernel<2, ROWMASK><<<ntiles, kMsThreads, 0, s>>>(src, mask, out, n, ntiles, ticket, tdesc, result, budget, row_len);
  else
    ms_dense_kernel<4, ROWMASK><<<ntiles, kMsThreads, 0, s>>>(src, mask, out, n, ntiles, ticket, tdesc, result, budget, row_len);
}

}  // namespace twg

using namespace twg;

extern "C" size_t twg_masked_select_workspace_bytes(int64_t numel) {
  if (numel < 0) numel = 0;
  const int64_t ntiles = (numel + kMsRound - 1) / kMsRound;  // the smallest tile any path uses
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
  u64* ticket = static_cast<u64*>(workspace);
  u64* tdesc = reinterpret_cast<u64*>(static_cast<char*>(workspace) + kMsHeaderBytes);
  i64* result = reinterpret_cast<i64*>(result_dev);
  const long long budget = g_poll_budget.load();

  const bool dense = (d.ndim == 0 || (d.ndim == 1 && (n == 1 || (d.strides[0][0] == 1 && d.strides[1][0] == 1)))) &&
                     is_aligned(src, 16) && is_aligned(mask, 4);
  // [R,C] source with a [R,1] mask: dimension 0 is the row (src stride 1, mask stride 0),
  // dimension 1 walks rows in both
  const bool rowmask = d.ndim == 2 && d.strides[0][0] == 1 && d.strides[1][0] == 0 && d.strides[0][1] == d.shape[0] &&
                       d.strides[1][1] == 1 && d.shape[0] % 4 == 0 && n < (int64_t(1) << 31) && is_aligned(src, 16);
  if (dense || rowmask) {
    const int rounds = dense_rounds();
    const int64_t tile_elems = (int64_t)rounds * kMsRound;
    const int64_t ntiles = (n + tile_elems - 1) / tile_elems;
    TWG_REQUIRE(ntiles <= 0x7fffffff, "twg_masked_select_f32: %lld elements exceed the tile limit", (long long)n);
    TWG_CUDA(cudaMemsetAsync(workspace, 0, kMsHeaderBytes + (size_t)ntiles * sizeof(u64), s));
    FastDiv32 row_len;
    row_len.d = rowmask ? (uint32_t)d.shape[0] : 1u;
    make_fastdiv(row_len.d, &row_len.m, &row_len.s);
    if (rowmask) launch_dense<true>(rounds, (unsigned)ntiles, s, src, mask, out, n, ticket, tdesc, result, budget, row_len);
    else launch_dense<false>(rounds, (unsigned)ntiles, s, src, mask, out, n, ticket, tdesc, result, budget, row_len);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathDense;
    return TWG_OK;
  }

  const int64_t ntiles = (n + kMsRound - 1) / kMsRound;
  TWG_REQUIRE(ntiles <= 0x7fffffff, "twg_masked_select_f32: %lld elements exceed the tile limit", (long long)n);
  TWG_CUDA(cudaMemsetAsync(workspace, 0, need, s));
  if (fits_32bit(d, 2)) {
    StridedDesc<2, u32> sd;
    fill_strided_desc<2>(d, &sd);
    ms_strided_kernel<u32><<<(unsigned)ntiles, kMsThreads, 0, s>>>(src, mask, out, sd, n, ntiles, ticket, tdesc, result, budget);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathStrided32;
  } else {
    StridedDesc<2, u64> sd;
    fill_strided_desc<2>(d, &sd);
    ms_strided_kernel<u64><<<(unsigned)ntiles, kMsThreads, 0, s>>>(src, mask, out, sd, n, ntiles, ticket, tdesc, result, budget);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathStrided64;
  }
  return TWG_OK;
}
