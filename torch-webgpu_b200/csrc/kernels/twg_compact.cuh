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


// ------------------------------------------------------------------------------------------
// Fused predicate + select, first half: a pointwise predicate over dense f32 inputs, written as
// ONE BIT per element.  The compaction kernel (masked_select.cu) reads those bits instead of a
// byte mask, so a predicate that feeds nothing but masked_select of one of its inputs costs
// 4 NIN + 1/8 bytes per element here and 4 1/8 + 4 k/N there, instead of 4 NIN + 1 and 5 + 4 k/N
// with a bool tensor in between: 1.75 bytes per element less, and both launches are the dense
// streaming kernels that run at the memory roofline.
//
// A warp takes 128 U consecutive elements (U = 4, 2, 1 for 1, 2, more inputs).  In each of its U rounds a lane takes one quad (4
// consecutive elements, one 128-bit load per input; all rounds' loads are issued before the first
// predicate is evaluated), evaluates the predicate four times and holds a nibble; the eight lanes
// of a group OR their shifted nibbles into the word of their 32 elements (one redux per group).
// Lane 8 g + t (t < U) then stores word g of round t, so the warp writes its 16 U bytes of bits
// with one store instruction.  Bit i of word w is element 32 w + i; bits at and beyond n are
// zero, and the buffer is written in whole 16-byte vectors (128 elements).
// (An earlier one-launch kernel evaluated the predicate and staged the selected values in one
// sweep over 16384-element chunks with a CTA-wide barrier around every look-back; it was no faster
// than writing a byte mask and compacting in a second launch: 0.85 ms against 0.83 ms for the
// three-input silu chain at 2^28 elements.)
// ------------------------------------------------------------------------------------------
// Bytes of the bit buffer for n elements.
__host__ __device__ constexpr unsigned long long predicate_bits_bytes(long long n) {
  return (unsigned long long)((n + 127) / 128) * 16ull;
}
// Rounds per warp: the unroll the dense pointwise kernel uses for as many inputs (one round with
// three or more inputs keeps the kernel near 32 registers, i.e. eight CTAs per SM, which this
// issue-bound loop needs more than it needs loads in flight per thread).
__host__ __device__ constexpr int predicate_bits_rounds(int nin) { return nin <= 1 ? 4 : (nin == 2 ? 2 : 1); }
// CTAs that cover n elements: every warp takes exactly one stretch.
__host__ __device__ constexpr long long predicate_bits_ctas(long long n, int nin) {
  const long long per_cta = 128ll * predicate_bits_rounds(nin) * (kBlock / 32);
  return (n + per_cta - 1) / per_cta;
}

// The predicate over one quad as a nibble (bit b = element b).
template <class F>
__device__ __forceinline__ u32 predicate_nibble(const F& f, const u32 (&x)[4][F::NIN]) {
  u32 nib = 0;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    u32 y[1];
    f(x[b], y);
    nib |= (y[0] & 1u) << b;
  }
  return nib;
}

template <class F>
__device__ __forceinline__ void predicate_bits_body(const PwPtrs<F::NIN>& in, const F& f, u32* bits, i64 n) {
  static_assert(F::NOUT == 1 && F::kOutByteMask == 1u && F::kInByteMask == 0u, "predicate over f32 inputs");
  constexpr int NIN = F::NIN;
  constexpr int U = predicate_bits_rounds(NIN);
  const int lane = threadIdx.x & 31;
  const int group = lane >> 3, t = lane & 7;
  const u32 members = 0xffu << (lane & 24);   // the eight lanes of a group hold the 32 elements of one word
  const i64 nquads = ((n + 127) / 128) * 32;  // whole rounds: 32 quads = 128 elements = one 16-byte vector of bits
  {  // the grid covers every stretch (predicate_bits_ctas)
    const i64 q0 = ((i64)blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5)) * (32 * U);
    if (q0 >= nquads) return;
    u32 x[U][4][NIN];
    u32 mine = 0;  // word `group` of round t
    if ((q0 + 32 * U) * 4 <= n) {
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int k = 0; k < NIN; ++k) {
          const uint4 v = ld_v4(static_cast<const float*>(in.p[k]) + 4 * (q0 + lane) + 128 * u);
          x[u][0][k] = v.x; x[u][1][k] = v.y; x[u][2][k] = v.z; x[u][3][k] = v.w;
        }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const u32 word = __reduce_or_sync(members, predicate_nibble<F>(f, x[u]) << (t * 4));
        if (t == u) mine = word;
      }
    } else {  // the stretch that holds element n - 1
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const i64 e = 4 * (q0 + u * 32 + lane);
#pragma unroll
        for (int k = 0; k < NIN; ++k) {
          const float* p = static_cast<const float*>(in.p[k]);
#pragma unroll
          for (int b = 0; b < 4; ++b) x[u][b][k] = (e + b < n) ? ld_b32(p + e + b) : 0u;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const i64 left = n - 4 * (q0 + u * 32 + lane);  // elements of this quad that exist
        const u32 valid = left >= 4 ? 0xfu : (left <= 0 ? 0u : (1u << (int)left) - 1u);
        const u32 word = __reduce_or_sync(members, (predicate_nibble<F>(f, x[u]) & valid) << (t * 4));
        if (t == u) mine = word;
      }
    }
    if (t < U && q0 + t * 32 < nquads) bits[(q0 >> 3) + 4 * t + group] = mine;
  }
}

template <class F>
__global__ void __launch_bounds__(kBlock) predicate_bits_kernel(PwPtrs<F::NIN> in, F f, u32* bits, i64 n) {
  predicate_bits_body<F>(in, f, bits, n);
}

}  // namespace twg
