// Device-side building blocks of the single-pass stream compaction: the tile-descriptor protocol
// of the decoupled look-back and the fused "predicate + select" kernel body.  Like
// twg_pointwise.cuh this header is compiled by nvcc into the library and, as text, by NVRTC, so it
// includes nothing from the host.
#pragma once

#include "twg_pointwise.cuh"

namespace twg {

constexpr int kMsThreads = 256;
constexpr int kMsWarps = kMsThreads / 32;
constexpr int kMsRound = kMsThreads * 16;  // 4096 elements: what one staging pass of masked_select holds
constexpr unsigned kMsHeaderBytes = 256;    // workspace header: ticket counter, padded
constexpr int kErrTimeout = -4;            // TWG_ERR_TIMEOUT (checked against twg.h where both are visible)

constexpr u64 kMsAggregate = 1ull << 62;
constexpr u64 kMsPrefix = 2ull << 62;
constexpr u64 kMsValueMask = (1ull << 62) - 1ull;

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

// Decoupled look-back in two steps.  lookback_publish (one thread) announces this run's count as
// soon as it is known; lookback_resolve (warp 0, later) adds up the counts of all earlier runs,
// publishes the inclusive prefix and returns the exclusive one.  Each poll reads the 32 nearest
// unresolved predecessors; published aggregates in front of the first unpublished descriptor are
// consumed at once.
//
// A negative poll budget is the test hook "run 0 never publishes": every wait that depends on it
// must run out after |budget| polls and report TWG_ERR_TIMEOUT instead of hanging.
__device__ __forceinline__ void lookback_publish(i64 tile, u32 tile_total, u64* desc, i64 poll_budget) {
  if (tile == 0) {
    if (poll_budget >= 0) st_relaxed_u64(desc, kMsPrefix | (u64)tile_total);
  } else {
    st_relaxed_u64(desc + tile, kMsAggregate | (u64)tile_total);
  }
}

__device__ __forceinline__ i64 lookback_resolve(i64 tile, u32 tile_total, u64* desc, i64* result, i64 poll_budget) {
  const int lane = threadIdx.x & 31;
  if (tile == 0) return 0;
  if (poll_budget < 0) poll_budget = -poll_budget;
  u64 excl = 0;
  i64 look = tile - 1;  // nearest predecessor not yet accounted for
  i64 polls = 0;
  bool timed_out = false;
  while (true) {
    const i64 idx = look - lane;
    const u64 d = idx >= 0 ? ld_relaxed_u64(desc + idx) : kMsPrefix;  // before run 0: prefix of 0
    const u32 status = (u32)(d >> 62);
    const u32 invalid = __ballot_sync(0xffffffffu, status == 0u);
    const u32 prefix = __ballot_sync(0xffffffffu, status == 2u);
    const int first_invalid = invalid ? __ffs(invalid) - 1 : 32;
    const int first_prefix = prefix ? __ffs(prefix) - 1 : 32;
    if (first_prefix < first_invalid) {
      excl += warp_sum_u64(lane <= first_prefix ? (d & kMsValueMask) : 0ull);
      break;
    }
    if (first_invalid > 0) {
      excl += warp_sum_u64(lane < first_invalid ? (d & kMsValueMask) : 0ull);
      look -= first_invalid;
      if (first_invalid == 32) continue;  // 32 aggregates, no prefix yet: keep walking
    }
    if (++polls > poll_budget) { timed_out = true; break; }
    if (polls > 64) __nanosleep(64);
  }
  if (timed_out) {
    excl = 0;
    if (lane == 0) {
      result[1] = (i64)kErrTimeout;
      __threadfence();  // the status is visible before the prefix that lets later runs finish
    }
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


// Look-back for callers whose runs are short compared with an L2 round trip: as many runs are in
// flight as there are CTAs, so the nearest resolved prefix is typically a hundred or more
// descriptors back.  One poll fetches DEPTH * 32 descriptors at once (DEPTH coalesced loads in
// flight together) and consumes them 32 at a time with the same rules as lookback_resolve.
template <int DEPTH>
__device__ __forceinline__ i64 lookback_resolve_deep(i64 tile, u32 tile_total, u64* desc, i64* result, i64 poll_budget) {
  const int lane = threadIdx.x & 31;
  if (tile == 0) return 0;
  if (poll_budget < 0) poll_budget = -poll_budget;
  u64 excl = 0;
  i64 look = tile - 1;  // nearest predecessor not yet accounted for
  i64 polls = 0;
  bool done = false, timed_out = false;
  while (!done) {
    u64 d[DEPTH];
#pragma unroll
    for (int q = 0; q < DEPTH; ++q) {
      const i64 idx = look - q * 32 - lane;
      d[q] = idx >= 0 ? ld_relaxed_u64(desc + idx) : kMsPrefix;  // before run 0: prefix of 0
    }
    bool stalled = false;
#pragma unroll
    for (int q = 0; q < DEPTH; ++q) {
      if (done || stalled) continue;
      const u32 status = (u32)(d[q] >> 62);
      const u32 invalid = __ballot_sync(0xffffffffu, status == 0u);
      const u32 prefix = __ballot_sync(0xffffffffu, status == 2u);
      const int first_invalid = invalid ? __ffs(invalid) - 1 : 32;
      const int first_prefix = prefix ? __ffs(prefix) - 1 : 32;
      if (first_prefix < first_invalid) {
        excl += warp_sum_u64(lane <= first_prefix ? (d[q] & kMsValueMask) : 0ull);
        done = true;
      } else {
        if (first_invalid > 0) {
          excl += warp_sum_u64(lane < first_invalid ? (d[q] & kMsValueMask) : 0ull);
          look -= first_invalid;
        }
        if (first_invalid < 32) stalled = true;  // an unpublished run: poll again from there
      }
    }
    if (done) break;
    if (stalled) {
      if (++polls > poll_budget) { timed_out = true; break; }
      if (polls > 64) __nanosleep(64);
    }
  }
  if (timed_out) {
    excl = 0;
    if (lane == 0) {
      result[1] = (i64)kErrTimeout;
      __threadfence();  // the status is visible before the prefix that lets later runs finish
    }
  }
  if (lane == 0) st_relaxed_u64(desc + tile, kMsPrefix | ((excl + (u64)tile_total) & kMsValueMask));
  return (i64)excl;
}

// ------------------------------------------------------------------------------------------
// Fused predicate + select: out = src[pred(inputs)] in one pass, where `pred` is a pointwise
// functor over dense f32 inputs with one bool output and src is one of its inputs.  The boolean
// mask never exists in memory: HBM sees every input element once (4 * NIN bytes) and the selected
// values once (4k bytes), instead of writing the mask, reading it back and reading src again.
//
// Persistent CTAs of 16 warps, three per SM, draw chunks of 16384 consecutive elements from a
// ticket counter.  Warp w owns the contiguous span [w*1024, (w+1)*1024) of the chunk and walks it
// in steps of 128 elements (one float4 quad per lane and input, the loads of kSelUnroll steps in
// flight together).  Per step the warp evaluates the predicate, ranks its selected elements with
// four independent ballots + popc and appends their src values to its own region of a 64 KB
// shared-memory stage - no CTA-wide barrier inside the loop.  The sixteen warp totals give the
// chunk count; it is published for the decoupled look-back (one link per chunk), warp 0 resolves
// the exclusive prefix (bounded wait), and every warp writes its run to out[prefix + offset of
// the warp ...] with 128-bit stores where aligned.
//
// Why these sizes (measured on B200, 2^28 elements, the three-input silu chain): a look-back
// costs several L2 round trips whatever the chunk size - the nearest predecessors are staged at
// the same moment by other SMs - so small chunks are look-back bound (2048 elements: 1.47 ms,
// 4096: 0.99, 8192: 0.86, 16384: 0.78); the two other CTAs of the SM and their 32 warps cover the
// wait.  A warp-specialised variant (one CTA per SM, TMA bulk loads into an mbarrier ring, scan
// warps resolving several units at once) kept HBM busy but left only 16 warps for the predicate
// arithmetic and measured 1.03 ms.
// ------------------------------------------------------------------------------------------
constexpr int kSelWarps = 16;
constexpr int kSelThreads = kSelWarps * 32;
constexpr int kSelChunk = 16384;
constexpr int kSelSpan = kSelChunk / kSelWarps;  // 1024 elements per warp
constexpr int kSelSteps = kSelSpan / 128;        // 8 steps of 32 quads
constexpr int kSelCtasPerSm = 3;
constexpr unsigned kSelSmemBytes = kSelChunk * 4u;  // dynamic: the stage
constexpr int kSelLookDepth = 4;                    // 128 descriptors per poll
// Steps whose loads are issued together: about 24 registers of loaded data per thread.
__host__ __device__ constexpr int sel_unroll(int nin) { return nin == 1 ? 4 : (nin <= 3 ? 2 : 1); }

struct SelShared {
  u32 warp_total[kSelWarps];
  i64 chunk;
  i64 excl;
};

template <class F, int SRC>
__device__ __forceinline__ void select_fused_body(const PwPtrs<F::NIN>& in, const F& f, float* out, i64 n, i64 nchunks,
                                                  u64* ticket, u64* desc, i64* result, i64 poll_budget) {
  static_assert(F::NOUT == 1 && F::kOutByteMask == 1u && F::kInByteMask == 0u, "predicate over f32 inputs");
  static_assert(SRC >= 0 && SRC < F::NIN, "src is one of the inputs");
  constexpr int NIN = F::NIN;
  constexpr int U = sel_unroll(NIN);
  __shared__ SelShared sm;
  extern __shared__ float sel_stage[];  // [kSelWarps][kSelSpan]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const u32 below = (1u << lane) - 1u;
  float* region = sel_stage + warp * kSelSpan;

  for (i64 iter = 0;; ++iter) {
    i64 chunk = (i64)blockIdx.x + iter * (i64)gridDim.x;
    if (ticket != nullptr) {
      if (threadIdx.x == 0) sm.chunk = (i64)atomicAdd(ticket, 1ull);
      __syncthreads();
      chunk = sm.chunk;
    }
    if (chunk >= nchunks) return;
    const i64 span_base = chunk * (i64)kSelChunk + (i64)warp * kSelSpan;
    u32 running = 0;
#pragma unroll 1
    for (int s0 = 0; s0 < kSelSteps; s0 += U) {
      u32 v[U][NIN][4];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const i64 e = span_base + (i64)(s0 + u) * 128 + lane * 4;
#pragma unroll
        for (int k = 0; k < NIN; ++k) {
          if (e + 3 < n) {
            const uint4 q = ld_v4(reinterpret_cast<const float*>(in.p[k]) + e);
            v[u][k][0] = q.x; v[u][k][1] = q.y; v[u][k][2] = q.z; v[u][k][3] = q.w;
          } else {
#pragma unroll
            for (int b = 0; b < 4; ++b)
              v[u][k][b] = (e + b < n) ? ld_b32(reinterpret_cast<const float*>(in.p[k]) + e + b) : 0u;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        // elements of this lane's quad that exist: 4 everywhere except at the very end of the data
        const i64 left = n - (span_base + (i64)(s0 + u) * 128 + lane * 4);
        const int live = left >= 4 ? 4 : (left > 0 ? (int)left : 0);
        u32 flags = 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          u32 x[NIN], y[1];
#pragma unroll
          for (int k = 0; k < NIN; ++k) x[k] = v[u][k][q];
          f(x, y);
          if ((y[0] & 1u) && q < live) flags |= 1u << q;
        }
        // rank = selected elements of the lanes below (four independent ballots) + own earlier ones
        u32 pos = running;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const u32 bal = __ballot_sync(0xffffffffu, (flags >> q) & 1u);
          pos += __popc(bal & below);
          running += __popc(bal);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
          if ((flags >> q) & 1u) region[pos++] = __uint_as_float(v[u][SRC][q]);
      }
    }
    if (lane == 0) sm.warp_total[warp] = running;
    __syncthreads();
    // offset of this warp's run inside the chunk, and the chunk count
    u32 t = lane < kSelWarps ? sm.warp_total[lane] : 0u;
    u32 warp_off = lane < warp ? t : 0u;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      t += __shfl_xor_sync(0xffffffffu, t, o);
      warp_off += __shfl_xor_sync(0xffffffffu, warp_off, o);
    }
    if (warp == 0) {
      if (lane == 0) lookback_publish(chunk, t, desc, poll_budget);
      const i64 excl = lookback_resolve_deep<kSelLookDepth>(chunk, t, desc, result, poll_budget);
      if (lane == 0) {
        sm.excl = excl;
        if (chunk == nchunks - 1) result[0] = excl + (i64)t;
      }
    }
    __syncthreads();
    // every warp writes its own run: 128-bit stores between the first and last 16-byte boundary
    float* dst = out + sm.excl + warp_off;
    const u32 head = min(running, (u32)(((16u - (u32)(reinterpret_cast<unsigned long long>(dst) & 15ull)) & 15u) >> 2));
    if ((u32)lane < head) dst[lane] = region[lane];
    const u32 nvec = (running - head) >> 2;
    float4* dst4 = reinterpret_cast<float4*>(dst + head);
    for (u32 i = lane; i < nvec; i += 32) {
      const float* r = region + head + 4 * i;
      dst4[i] = make_float4(r[0], r[1], r[2], r[3]);
    }
    const u32 tail0 = head + 4 * nvec;
    if (tail0 + lane < running) dst[tail0 + lane] = region[tail0 + lane];
    __syncthreads();  // the stage, warp_total and excl are rewritten by the next chunk
  }
}

template <class F, int SRC>
__global__ void __launch_bounds__(kSelThreads, kSelCtasPerSm)
    select_fused_kernel(PwPtrs<F::NIN> in, F f, float* out, i64 n, i64 nchunks, u64* ticket, u64* desc, i64* result,
                        i64 poll_budget) {
  select_fused_body<F, SRC>(in, f, out, n, nchunks, ticket, desc, result, poll_budget);
}

}  // namespace twg
