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
    if (lane == 0) result[1] = (i64)kErrTimeout;
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
// Fused predicate + select: out = src[pred(inputs)] in one pass, where `pred` is a pointwise
// functor over dense f32 inputs with one bool output and src is one of its inputs.  The boolean
// mask never exists in memory: HBM sees every input element once (4 * NIN bytes) and the selected
// values once (4k bytes), instead of writing the mask, reading it back and reading src again.
//
// Persistent CTAs (a few per SM) draw chunks of 8192 consecutive elements from a ticket counter.
// Warp w owns the contiguous span [w*1024, (w+1)*1024) of the chunk and walks it in steps of 128
// elements (one float4 quad per lane and input, kSelUnroll steps in flight).  Per step the warp
// evaluates the predicate, ranks its selected elements with popc + a warp scan and appends their
// src values to its private region of shared memory - no CTA-wide barrier inside the loop.  The
// eight warp totals give the chunk count, which is published at once for the decoupled look-back
// (one link per chunk, bounded wait).
//
// The count of a chunk is only known when all of its inputs have been read, so resolving the
// look-back right away would leave the CTA idle for several round trips per chunk.  Instead the
// stage is double-buffered: after publishing chunk i the CTA streams chunk i+1 into the other
// buffer, and only then resolves chunk i's prefix - by that time its predecessors have resolved
// theirs, so one poll usually suffices - and flushes chunk i to out[prefix + offset of the warp].
// ------------------------------------------------------------------------------------------
constexpr int kSelChunk = 8192;
constexpr int kSelWarpSpan = kSelChunk / kMsWarps;  // 1024 elements
constexpr int kSelSteps = kSelWarpSpan / 128;       // 8 steps of 32 quads
constexpr int kSelUnroll = 2;
constexpr int kSelCtasPerSm = 3;
constexpr unsigned kSelSmemBytes = 2u * kSelChunk * 4u;  // dynamic: two stage buffers

struct SelShared {
  u32 warp_total[kMsWarps];
  i64 tile;
  i64 excl;
};

template <class F, int SRC>
__device__ __forceinline__ void select_fused_body(const PwPtrs<F::NIN>& in, const F& f, float* out, i64 n, i64 nchunks,
                                                  u64* ticket, u64* desc, i64* result, i64 poll_budget) {
  static_assert(F::NOUT == 1 && F::kOutByteMask == 1u && F::kInByteMask == 0u, "predicate over f32 inputs");
  static_assert(SRC >= 0 && SRC < F::NIN, "src is one of the inputs");
  __shared__ SelShared sm;
  extern __shared__ float sel_stage[];  // [2][kMsWarps][kSelWarpSpan]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  int buf = 0;
  bool pending = false;          // a staged chunk is waiting for its prefix (uniform over the CTA)
  i64 pend_chunk = 0;
  u32 pend_running = 0, pend_warp_off = 0, pend_total = 0;

  for (i64 iter = 0;; ++iter) {
    i64 chunk = (i64)blockIdx.x + iter * (i64)gridDim.x;
    if (ticket != nullptr) {
      if (threadIdx.x == 0) sm.tile = (i64)atomicAdd(ticket, 1ull);
      __syncthreads();
      chunk = sm.tile;
    }
    const bool has = chunk < nchunks;
    float* region = sel_stage + ((size_t)buf * kMsWarps + warp) * kSelWarpSpan;
    u32 running = 0;
    if (has) {
      const i64 span_base = chunk * (i64)kSelChunk + (i64)warp * kSelWarpSpan;
#pragma unroll 1
      for (int s0 = 0; s0 < kSelSteps; s0 += kSelUnroll) {
        u32 v[kSelUnroll][F::NIN][4];
#pragma unroll
        for (int u = 0; u < kSelUnroll; ++u) {
          const i64 e = span_base + (i64)(s0 + u) * 128 + lane * 4;
#pragma unroll
          for (int k = 0; k < F::NIN; ++k) {
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
        for (int u = 0; u < kSelUnroll; ++u) {
          const i64 e = span_base + (i64)(s0 + u) * 128 + lane * 4;
          u32 flags = 0;
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            u32 x[F::NIN], y[1];
#pragma unroll
            for (int k = 0; k < F::NIN; ++k) x[k] = v[u][k][b];
            f(x, y);
            if ((y[0] & 1u) && e + b < n) flags |= 1u << b;
          }
          const u32 cnt = __popc(flags);
          u32 incl = cnt;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const u32 t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
          }
          u32 pos = running + incl - cnt;
#pragma unroll
          for (int b = 0; b < 4; ++b)
            if ((flags >> b) & 1u) region[pos++] = __uint_as_float(v[u][SRC][b]);
          running += __shfl_sync(0xffffffffu, incl, 31);
        }
      }
      if (lane == 0) sm.warp_total[warp] = running;
    }
    __syncthreads();
    u32 warp_off = 0, chunk_total = 0;
    if (has) {
#pragma unroll
      for (int w = 0; w < kMsWarps; ++w) {
        const u32 t = sm.warp_total[w];
        if (w < warp) warp_off += t;
        chunk_total += t;
      }
      if (threadIdx.x == 0) lookback_publish(chunk, chunk_total, desc, poll_budget);
    }
    if (pending) {
      // the chunk staged one iteration ago: its predecessors have had a whole chunk time to resolve
      if (warp == 0) {
        const i64 excl = lookback_resolve(pend_chunk, pend_total, desc, result, poll_budget);
        if (lane == 0) {
          sm.excl = excl;
          if (pend_chunk == nchunks - 1) result[0] = excl + (i64)pend_total;
        }
      }
      __syncthreads();
      // every warp writes its own run: out[prefix + offset of the warp ...], 128-bit where aligned
      const float* src_region = sel_stage + ((size_t)(buf ^ 1) * kMsWarps + warp) * kSelWarpSpan;
      float* dst = out + sm.excl + pend_warp_off;
      const u32 head =
          min(pend_running, (u32)(((16u - (u32)(reinterpret_cast<unsigned long long>(dst) & 15ull)) & 15u) >> 2));
      if ((u32)lane < head) dst[lane] = src_region[lane];
      const u32 nvec = (pend_running - head) >> 2;
      float4* dst4 = reinterpret_cast<float4*>(dst + head);
      for (u32 i = lane; i < nvec; i += 32) {
        const float* s = src_region + head + 4 * i;
        dst4[i] = make_float4(s[0], s[1], s[2], s[3]);
      }
      const u32 tail0 = head + 4 * nvec;
      if (tail0 + lane < pend_running) dst[tail0 + lane] = src_region[tail0 + lane];
    }
    if (!has) break;
    pending = true;
    pend_chunk = chunk;
    pend_running = running;
    pend_warp_off = warp_off;
    pend_total = chunk_total;
    buf ^= 1;
    __syncthreads();  // warp_total and excl may be rewritten by the next iteration
  }
}

template <class F, int SRC>
__global__ void __launch_bounds__(kMsThreads)
    select_fused_kernel(PwPtrs<F::NIN> in, F f, float* out, i64 n, i64 nchunks, u64* ticket, u64* desc, i64* result,
                        i64 poll_budget) {
  select_fused_body<F, SRC>(in, f, out, n, nchunks, ticket, desc, result, poll_budget);
}

}  // namespace twg
