// masked_select as a single-pass stream compaction.
//
// One CTA owns a run of consecutive logical elements (a chunk of tiles in the chunked kernel, one
// tile in the kernel for 64-bit offsets).  Selected elements are ranked with popc on mask words
// that are warp ballots of 32 consecutive elements; the run's base offset in the output comes from
// a decoupled look-back over the preceding runs' published counts, so one launch does everything,
// src is read exactly once and no global scan kernel is needed.  Selected values are first packed
// into shared memory in output order and then written as contiguous, aligned runs.
//
// Forward progress: a run's index is a ticket drawn from a global counter when its CTA starts,
// not blockIdx, so every run a CTA may wait for belongs to a CTA that is already running.  The
// wait is nevertheless bounded: after `poll_budget` polls the run gives up, records
// TWG_ERR_TIMEOUT in result[1], publishes a prefix so that later runs do not wait on it, and the
// kernel drains normally.
#include "twg_launch.cuh"
#include "twg_compact.cuh"

#include <atomic>
#include <mutex>
#include <cstdlib>
#include <cstring>
#include <string>

namespace twg {

static_assert(kErrTimeout == TWG_ERR_TIMEOUT, "twg_compact.cuh and twg.h disagree");

constexpr int kMsMaxRounds = 2;                     // double-buffered per-warp totals

static std::atomic<long long> g_poll_budget{4000000};

struct MsShared {
  float stage[kMsRound];
  u32 warp_total[kMsMaxRounds][kMsWarps];
  u32 reduce[kMsWarps];
  i64 tile;
  i64 excl;
};

// ------------------------------------------------------------------------------------------
// The chunked kernel.  src contiguous and 16-byte aligned; the mask is either a dense bool array
// (16-byte aligned) or, with kMsRowMask, one bool per row of `row_len` elements (a [R,1] mask
// broadcast over [R,C] with C % 4 == 0).  A third mode walks both operands through the iteration
// descriptor (element index -> offsets with 32-bit multiply-shift division): slices, broadcast
// masks and other non-dense layouts get the same chunking, at one index computation per mask byte
// and per selected element.
//
// A CTA owns a chunk of CH consecutive tiles of 4096 elements; warp w owns the CH consecutive
// spans (512 elements each) [w CH, (w + 1) CH) of it, so its output is one contiguous run.
//   Phase A  turns the chunk's mask into one bit per element in shared memory and counts the
//            selected elements of every span.  In the dense mode every warp does this for its own
//            stretch and starts fetching its first span right away.  The chunk count is published
//            at once: the chain of dependent CTAs has one link per chunk, and warp 0 resolves it
//            while those first loads are in flight.
//   Phase B  Lane l owns elements 32 k + l (k = 0..15) of a span: a warp-wide access is one
//            128-byte run, word k of the span's bits is the selection bitmap of row k, and popc of
//            its low bits is a lane's rank in the row - consecutive selected lanes get consecutive
//            stage slots, so the staging stores are free of bank conflicts whatever the density.
//            The staged run leaves as aligned 128-bit vectors; spans that select everything are
//            copied straight from registers; the next span's loads are in flight while the current
//            one is ranked and written out.
// HBM sees every mask byte once and every selected sector of src once.  (Earlier forms, measured
// on 2^27 elements at 41 % density: eight warps ranking a tile together with two barriers per tile
// 169.7 us; lanes owning quads of four consecutive elements with a packed warp scan 165.8 us and
// 32 instructions per element; this form 149.5 us and 20.)
// ------------------------------------------------------------------------------------------
// four arbitrary bytes -> four 0/1 bytes (non-zero counts as true): the carry of (b & 0x7f) + 0x7f
// reaches bit 7 exactly when the low seven bits are non-zero
__device__ __forceinline__ u32 nonzero_bytes(u32 w) {
  return ((((w & 0x7f7f7f7fu) + 0x7f7f7f7fu) | w) >> 7) & 0x01010101u;
}
// four arbitrary bytes -> their "non-zero" flags in bits 28..31 (byte 0 in bit 28): bit 7 of every byte is
// set as above, and the multiplier moves bits 7, 15, 23 and 31 to bits 28, 29, 30 and 31 (the partial
// products land on distinct bits, so nothing carries)
__device__ __forceinline__ u32 nonzero_nibble(u32 w) {
  return ((((w & 0x7f7f7f7fu) + 0x7f7f7f7fu) | w) & 0x80808080u) * 0x00204081u;
}
// How the chunked kernel addresses its operands.
constexpr int kMsDense = 0;    // src and mask dense
constexpr int kMsRowMask = 1;  // src dense, one mask byte per row
constexpr int kMsStrided = 2;  // both through the iteration descriptor (32-bit index math)
constexpr int kMsBits = 3;     // src dense; `mask` points at one BIT per element (predicate_bits_body's output)

// Offsets of logical element `lin` in src and mask; returns its coordinate along dimension 0, so
// that a caller walking consecutive elements can step by the dimension-0 strides until the
// coordinate wraps.
__device__ __forceinline__ u32 ms_offsets(const StridedDesc<2, u32>& d, u32 lin, u32& osrc, u32& omask) {
  u32 q = d.shape[0].div(lin);
  const u32 c0 = lin - q * d.shape[0].d;
  osrc = c0 * d.strides[0][0];
  omask = c0 * d.strides[1][0];
#pragma unroll
  for (int k = 1; k < kMaxDims; ++k) {
    if (k >= d.ndim) break;
    const u32 q2 = d.shape[k].div(q);
    const u32 c = q - q2 * d.shape[k].d;
    q = q2;
    osrc += c * d.strides[0][k];
    omask += c * d.strides[1][k];
  }
  return c0;
}

template <int MODE>
__device__ __forceinline__ u32 mask_quad(const u8* mask, i64 e, i64 n, const FastDiv32& row_len,
                                         const StridedDesc<2, u32>& sd) {
  u32 w = 0;
  if constexpr (MODE == kMsStrided) {
    if (e < n) {
      u32 os, om;
      u32 c0 = ms_offsets(sd, (u32)e, os, om);
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        if (e + b < n) w |= (ld_b8(mask + om) != 0u ? 1u : 0u) << (8 * b);
        if (b < 3) {
          if (++c0 == sd.shape[0].d) {
            if (e + b + 1 < n) c0 = ms_offsets(sd, (u32)(e + b + 1), os, om);
          } else {
            om += sd.strides[1][0];
          }
        }
      }
    }
    return w;
  } else if constexpr (MODE == kMsRowMask) {
    if (e < n) w = ld_b8(mask + row_len.div((u32)e)) != 0u ? 0x01010101u : 0u;  // n < 2^31 on this path
    if (e + 3 >= n && w) w &= (e + 2 < n) ? 0x00ffffffu : (e + 1 < n) ? 0x0000ffffu : 0x000000ffu;
  } else {
    if (e + 3 < n) {
      w = ld_b32(mask + e);
    } else {
      for (int b = 0; b < 4; ++b)
        if (e + b < n) w |= ld_b8(mask + e + b) << (8 * b);
    }
    w = nonzero_bytes(w);
  }
  return w;
}
// four 0/1 bytes -> one nibble (the product has no colliding partial terms, so no carries)
__device__ __forceinline__ u32 bytes_to_nibble(u32 w) { return ((w * 0x01020408u) >> 24) & 0xfu; }

// Floats of a warp's staging buffer: one span (512) plus the at most three elements that wait for
// the rest of their 16-byte vector.
constexpr int kMsStageFloats = 516;

template <int CH>
struct MsDenseShared {
  alignas(16) float stage[kMsWarps][kMsStageFloats];
  alignas(16) unsigned short cnt[CH * kMsWarps];  // selected elements of span s (512 elements at chunk offset 512 s)
  u32 reduce[kMsWarps];
  i64 tile;
  i64 excl;
};

// A lane's sixteen elements of a span: element 32 i + lane, i = 0..15 (loaded only where needed).
struct MsSpanRegs {
  u32 v[16];
};

// The compaction's last chunk knows the total; when a count exchange rides along, the thread that
// writes it also stores {count, sequence | status} into this rank's slot of every rank's mailbox -
// plain stores to peer memory over NVLink, the flag word with release semantics at system scope -
// so the exchange costs no launch of its own.  A status written by a chunk that gave up waiting is
// fenced before that chunk's prefix becomes visible, so it is seen here.
__device__ __forceinline__ void ms_publish(const MsPublish& pub, i64 count, const i64* result) {
  if (pub.nranks == 0) return;
  __threadfence();
  const u64 status = (u64)(*reinterpret_cast<const volatile i64*>(result + 1)) & 0xffull;
  for (int r = 0; r < pub.nranks; ++r) {
    u64* p = pub.slot[r];
    p[0] = (u64)count;
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p + 1), "l"((pub.seq << 8) | status) : "memory");
  }
}

template <int CH, int MODE>
__global__ void __launch_bounds__(kMsThreads, 4)
    ms_dense_kernel(const float* src, const u8* mask, float* out, i64 n, i64 nchunks, u64* ticket, u64* desc,
                     i64* result, i64 poll_budget, FastDiv32 row_len, StridedDesc<2, u32> sd, MsPublish pub) {
  constexpr bool ROWMASK = MODE == kMsRowMask;
  constexpr int kSpans = CH * kMsWarps;  // spans of 512 elements in a chunk
  __shared__ MsDenseShared<CH> sm;
  __shared__ __align__(16) u32 bits[CH * (kMsRound / 32)];  // the chunk's mask, one bit per element
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) sm.tile = (i64)atomicAdd(ticket, 1ull);
  __syncthreads();
  const i64 chunk = sm.tile;
  if (chunk >= nchunks) return;
  const i64 chunk_base = chunk * (i64)(CH * kMsRound);
  const bool full_chunk = chunk_base + (i64)(CH * kMsRound) <= n;

  // ---- phase A: mask -> bits, count per span, chunk count ----
  u32 c = 0;
  // In phase B warp w owns the CH consecutive spans [w CH, (w + 1) CH) of the chunk, i.e. one
  // contiguous stretch of CH * 512 elements, so its output is one contiguous run.
  const int span0 = warp * CH;
  if (MODE == kMsDense && full_chunk) {
    // every warp reads the mask of its own stretch: it knows its bits and counts without waiting
    // for anybody and can start fetching src before the CTA meets at the barrier
    unsigned short* bits16 = reinterpret_cast<unsigned short*>(bits);
    const u8* mp = mask + chunk_base + (i64)span0 * 512 + lane * 16;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      uint4 q = ld_v4(mp + i * 512);
      const u32 sixteen = (nonzero_nibble(q.x) >> 28) | ((nonzero_nibble(q.y) >> 24) & 0xf0u) |
                          ((nonzero_nibble(q.z) >> 20) & 0xf00u) | ((nonzero_nibble(q.w) >> 16) & 0xf000u);
      const u32 ci = __popc(sixteen);
      c += ci;
      bits16[(span0 + i) * 32 + lane] = (unsigned short)sixteen;
      const u32 span = __reduce_add_sync(0xffffffffu, ci);
      if (lane == 0) sm.cnt[span0 + i] = (unsigned short)span;
    }
    __syncwarp();
  } else if constexpr (MODE == kMsBits) {
    // the mask already is one bit per element: every warp copies the words of its own stretch
    // (16 per span, 128-byte runs) and counts them, half a warp per span
    const u32* gbits = reinterpret_cast<const u32*>(mask);
    const i64 total_words = ((n + 127) / 128) * 4;  // what the producer wrote (zero at and beyond n)
    const i64 gw0 = chunk_base / 32 + (i64)span0 * 16;
    constexpr int kWords = CH * 16;
#pragma unroll
    for (int j0 = 0; j0 < kWords; j0 += 32) {
      const int idx = j0 + lane;
      u32 word = 0;
      if (idx < kWords && gw0 + idx < total_words) word = ld_b32(gbits + gw0 + idx);
      if (idx < kWords) bits[span0 * 16 + idx] = word;
      u32 cw = __popc(word);
      c += cw;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) cw += __shfl_xor_sync(0xffffffffu, cw, o);
      if ((lane & 15) == 0 && idx < kWords) sm.cnt[span0 + (idx >> 4)] = (unsigned short)cw;
    }
    __syncwarp();
  } else if constexpr (MODE == kMsStrided) {
    // a warp takes whole spans; lane l looks at element 32 g + l of word g, so that neighbouring
    // lanes read neighbouring mask bytes, and a ballot is the word
    for (int sidx = warp; sidx < kSpans; sidx += kMsWarps) {
      u32 span_count = 0;
#pragma unroll 4
      for (int k = 0; k < 16; ++k) {
        const int g = sidx * 16 + k;
        const i64 e = chunk_base + (i64)g * 32 + lane;
        bool nz = false;
        if (e < n) {
          u32 os, om;
          ms_offsets(sd, (u32)e, os, om);
          nz = ld_b8(mask + om) != 0u;
        }
        const u32 word = __ballot_sync(0xffffffffu, nz);
        if (lane == 0) bits[g] = word;
        span_count += __popc(word);
      }
      if (lane == 0) {
        sm.cnt[sidx] = (unsigned short)span_count;
        c += span_count;
      }
    }
  } else {
    // one word of bits = 32 consecutive elements, 16 words = one span: half a warp per span
    const bool row_words = ROWMASK && full_chunk && (row_len.d % 32u) == 0u;
    for (int g = threadIdx.x; g < CH * (kMsRound / 32); g += kMsThreads) {
      u32 word = 0, cw = 0;
      if (row_words) {
        word = ld_b8(mask + row_len.div((u32)(chunk_base + (i64)g * 32))) != 0u ? 0xffffffffu : 0u;
        cw = word & 32u;
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const u32 w = mask_quad<MODE>(mask, chunk_base + ((i64)g * 8 + k) * 4, n, row_len, sd);
          cw += __popc(w);
          word |= bytes_to_nibble(w) << (4 * k);
        }
      }
      bits[g] = word;
      c += cw;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) cw += __shfl_xor_sync(0xffffffffu, cw, o);
      if ((lane & 15) == 0) sm.cnt[g >> 4] = (unsigned short)cw;
    }
  }
  // ---- phase B: every warp compacts its stretch of the chunk on its own ----
  // Lane l owns elements 32 i + l (i = 0..15) of a span: a warp-wide access is one 128-byte run,
  // word i of the span's mask bits is the selection bitmap of row i, and popc of its low bits is a
  // lane's rank in the row - consecutive selected lanes get consecutive stage slots, so the
  // staging stores are free of bank conflicts whatever the density.  Spans that select a quarter
  // of their elements or more are loaded whole (nearly every sector is needed anyway); sparser
  // ones load selected elements only, so untouched sectors are never fetched.
  auto load_span = [&](MsSpanRegs& r, int s) {
    const i64 e0 = chunk_base + (i64)s * 512 + lane;
    if constexpr (MODE == kMsStrided) {
      u32 os = 0, om, c0 = 0;
      bool have = false;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if ((bits[s * 16 + i] >> lane) & 1u) {  // set bits only exist below n
          if (!have || c0 >= sd.shape[0].d) {
            c0 = ms_offsets(sd, (u32)(e0 + i * 32), os, om);
            have = true;
          }
          r.v[i] = __float_as_uint(__ldg(src + os));
        }
        if (have) {  // the next row lies 32 elements further along dimension 0 (or wraps: recomputed on use)
          c0 += 32u;
          os += 32u * sd.strides[0][0];
        }
      }
    } else if (full_chunk && sm.cnt[s] >= 128u) {
#pragma unroll
      for (int i = 0; i < 16; ++i) r.v[i] = ld_b32(src + e0 + i * 32);
    } else {
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const uint4 q = reinterpret_cast<const uint4*>(bits + s * 16)[h];
        const u32 w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if ((w[k] >> lane) & 1u) r.v[4 * h + k] = ld_b32(src + e0 + (4 * h + k) * 32);  // 0 bits beyond n
      }
    }
  };
  // A warp that made its own bits (dense mode) starts fetching its first span right away: the
  // loads are in flight across the barrier and the look-back below.
  MsSpanRegs next;
  const bool early = (MODE == kMsDense && full_chunk) || MODE == kMsBits;  // the warp made its own bits
  if (early) load_span(next, span0);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if (lane == 0) sm.reduce[warp] = c;
  __syncthreads();
  u32 chunk_total = 0;
#pragma unroll
  for (int w = 0; w < kMsWarps; ++w) chunk_total += sm.reduce[w];
  if (threadIdx.x == 0) lookback_publish(chunk, chunk_total, desc, poll_budget);

  // the warp's run starts `before` elements into the chunk's output
  u32 before = 0;
  for (int k = lane; k < span0; k += 32) before += sm.cnt[k];
  before = __reduce_add_sync(0xffffffffu, before);

  // ---- phase B for sparse chunks (fewer than one element in sixteen selected) ----
  // Ranking, staging and quad loads cost the same whether anything is selected or not; here a
  // lane walks the set bits of its 16 elements instead: one scalar load and one store per selected
  // element, and spans that select nothing are skipped with one look at the table of phase A.
  if (chunk_total * 16u < (u32)(CH * kMsRound)) {
    if (warp == 0) {
      const i64 excl = lookback_resolve(chunk, chunk_total, desc, result, poll_budget);
      if (lane == 0) {
        sm.excl = excl;
        if (chunk == nchunks - 1) {
          result[0] = excl + (i64)chunk_total;
          ms_publish(pub, excl + (i64)chunk_total, result);
        }
      }
    }
    __syncthreads();
    float* to_span = out + sm.excl + before;
    for (int i = 0; i < CH; ++i) {
      const int s = span0 + i;
      const u32 mine = sm.cnt[s];
      if (mine == 0u) continue;
      const u32 word = bits[s * 16 + (lane >> 1)];
      u32 half = (word >> ((lane & 1) * 16)) & 0xffffu;  // this lane's 16 consecutive elements
      const u32 cnt = __popc(half);
      u32 incl = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const u32 x = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += x;
      }
      const i64 first = chunk_base + (i64)s * 512 + lane * 16;
      float* to = to_span + (incl - cnt);
      u32 first_os = 0, first_c0 = 0;
      if constexpr (MODE == kMsStrided) {
        u32 om;
        if (half != 0u) first_c0 = ms_offsets(sd, (u32)first, first_os, om);
      }
      while (half != 0u) {
        const int bit = __ffs(half) - 1;
        half &= half - 1u;
        if constexpr (MODE == kMsStrided) {
          u32 o = first_os + bit * sd.strides[0][0], om;
          if (first_c0 + bit >= sd.shape[0].d) ms_offsets(sd, (u32)(first + bit), o, om);
          *to++ = __uint_as_float(ld_b32(src + o));
        } else {
          *to++ = __uint_as_float(ld_b32(src + first + bit));
        }
      }
      to_span += mine;
    }
    return;
  }

  if (!early) load_span(next, span0);  // in flight while warp 0 walks the look-back
  if (warp == 0) {
    const i64 excl = lookback_resolve(chunk, chunk_total, desc, result, poll_budget);
    if (lane == 0) {
      sm.excl = excl;
      if (chunk == nchunks - 1) {
        result[0] = excl + (i64)chunk_total;
        ms_publish(pub, excl + (i64)chunk_total, result);
      }
    }
  }
  __syncthreads();

  // Output positions are counted in a "virtual" index v = a0 + position inside the chunk's output,
  // where a0 is the misalignment (in elements) of the chunk's first output element: out_v + v is
  // 16-byte aligned exactly when v is a multiple of 4.  A staged element with virtual index v sits
  // at stage[v - vbase] (vbase a multiple of 4), so aligned vectors of the output are aligned
  // vectors of the stage and go out as one 128-bit shared load and one 128-bit store.  Elements
  // below vf are already in global memory; after every span the complete vectors are written and
  // the at most three elements left over ride in a register to the front of the next span's stage.
  float* const chunk_out = out + sm.excl;
  const u32 a0 = (u32)(reinterpret_cast<unsigned long long>(chunk_out) >> 2) & 3u;
  float* const out_v = chunk_out - a0;
  float* const stage = sm.stage[warp];
  const u32 below = (1u << lane) - 1u;
  u32 v = a0 + before, vf = v, vbase = v & ~3u;
  float carry = 0.f;  // lane i < v - vf holds the element with virtual index vf + i
  for (int i = 0; i < CH; ++i) {
    const int s = span0 + i;
    const MsSpanRegs cur = next;
    if (i + 1 < CH) load_span(next, s + 1);  // in flight while this span is ranked and written out
    const u32 run = sm.cnt[s];
    if (run == 0u) continue;
    if (run == 512u) {
      // everything selected: after the few elements still waiting the span is a straight copy
      if ((u32)lane < v - vf) out_v[vf + lane] = carry;
#pragma unroll
      for (int k = 0; k < 16; ++k) out_v[v + k * 32 + lane] = __uint_as_float(cur.v[k]);
      v += 512u;
      vf = v;
      vbase = v & ~3u;
      continue;
    }
    if ((u32)lane < v - vf) stage[vf - vbase + lane] = carry;
    u32 pos = v - vbase;  // stage index of the span's first selected element
#pragma unroll
    for (int h = 0; h < 2; ++h) {  // the span's mask words, eight at a time (two 128-bit broadcast loads)
      const uint4 qa = reinterpret_cast<const uint4*>(bits + s * 16)[2 * h];
      const uint4 qb = reinterpret_cast<const uint4*>(bits + s * 16)[2 * h + 1];
      const u32 w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if ((w[k] >> lane) & 1u) stage[pos + __popc(w[k] & below)] = __uint_as_float(cur.v[8 * h + k]);
        pos += __popc(w[k]);
      }
    }
    const u32 v_end = v + run;
    __syncwarp();
    if (vf & 3u) {  // the run starts inside a vector that earlier output shares: scalars up to the boundary
      const u32 head_end = min((vf + 3u) & ~3u, v_end);
      if ((u32)lane < head_end - vf) out_v[vf + lane] = stage[vf - vbase + lane];
      vf = head_end;
    }
    if ((vf & 3u) == 0u) {
      const u32 nvec = (v_end - vf) >> 2;
      const float4* from = reinterpret_cast<const float4*>(stage + (vf - vbase));
      float4* to4 = reinterpret_cast<float4*>(out_v + vf);
      for (u32 k = lane; k < nvec; k += 64) {  // two rounds per trip: both loads are issued before the stores
        const float4 x0 = from[k];
        float4 x1 = x0;
        if (k + 32 < nvec) x1 = from[k + 32];
        to4[k] = x0;
        if (k + 32 < nvec) to4[k + 32] = x1;
      }
      vf += 4u * nvec;
      if ((u32)lane < v_end - vf) carry = stage[vf - vbase + lane];  // 0..3 elements wait for the rest of their vector
      vbase = vf;
    }
    v = v_end;
    __syncwarp();  // the stage is rewritten by the next span
  }
  if ((u32)lane < v - vf) out_v[vf + lane] = carry;  // the stretch's last partial vector
}

// ------------------------------------------------------------------------------------------
// Strided / broadcast path for iterations whose offsets need 64 bits (and flipped views).  Logical element e (row-major over the broadcast shape) is mapped to
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
  i64 tile = blockIdx.x;
  if (ticket != nullptr) {
    if (threadIdx.x == 0) sm.tile = (i64)atomicAdd(ticket, 1ull);
    __syncthreads();
    tile = sm.tile;
  }
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
  if (threadIdx.x == 0) lookback_publish(tile, tile_total, desc, poll_budget);
  if (warp == 0) {
    const i64 excl = lookback_resolve(tile, tile_total, desc, result, poll_budget);
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

// Zeroes the part of the workspace a call uses (ticket header + descriptors) and the two result
// words with ONE small kernel.  Two cudaMemsetAsync calls in front of the compaction kernel cost
// about 20 us per call on B200 (measured: 196 us from event to event for a kernel that runs 174 us);
// a kernel in front of a kernel on the same stream costs a microsecond or two.
__global__ void __launch_bounds__(256) ms_clear_kernel(u64* workspace, unsigned nwords, i64* result) {
  const unsigned i = blockIdx.x * 256u + threadIdx.x;  // one 16-byte pair of words per thread
  if (2u * i + 1u < nwords) *reinterpret_cast<uint4*>(workspace + 2u * i) = make_uint4(0u, 0u, 0u, 0u);
  else if (2u * i < nwords) workspace[2u * i] = 0ull;
  if (i < 2u) result[i] = 0;
}
// workspace == nullptr: only the result words
int ms_clear(void* workspace, size_t nbytes, int64_t* result, cudaStream_t s) {
  const unsigned nwords = workspace ? (unsigned)(nbytes / 8) : 0u;  // sized in 8-byte words, 256-byte aligned
  const unsigned threads = (nwords + 1u) / 2u > 2u ? (nwords + 1u) / 2u : 2u;
  ms_clear_kernel<<<(threads + 255u) / 256u, 256, 0, s>>>(static_cast<u64*>(workspace), nwords, reinterpret_cast<i64*>(result));
  TWG_CHECK_LAUNCH();
  return TWG_OK;
}

// Tiles per dense chunk.  Two costs pull in opposite directions (measured on B200, 41 - 50 % of
// the elements selected): every chunk costs a CTA about 5.5 us that do not overlap with its own
// copying (ticket, mask latency, barrier, look-back), which favours long chunks, and the last wave
// of chunks runs on a partly idle device, which favours many.  The longest chunk that still leaves
// two waves of four CTAs per SM, capped at 16 tiles below 2^29 elements, was the best of the
// candidates at every size tried (2^27: 16 tiles 0.170 ms, 8 tiles 0.179 ms; 2^28: 16 tiles
// 0.329 ms, 32 tiles 0.331 ms; 2^30: 32 tiles).
static int dense_chunk_tiles(int64_t n) {
  const int64_t tiles = (n + kMsRound - 1) / kMsRound;
  const int64_t want_chunks = 2ll * 4 * sm_count();
  int ch = n < (int64_t(1) << 29) ? 16 : 32;
  while (ch > 1 && tiles / ch < want_chunks) ch >>= 1;
  return ch;
}

long long ms_poll_budget() { return g_poll_budget.load(); }

template <int MODE>
static void launch_dense(int chunk_tiles, unsigned nchunks, cudaStream_t s, const float* src, const u8* mask, float* out,
                         i64 n, u64* ticket, u64* tdesc, i64* result, i64 budget, FastDiv32 row_len,
                         const StridedDesc<2, u32>& sd, const MsPublish& pub) {
#define TWG_MS_LAUNCH(CH) \
  ms_dense_kernel<CH, MODE><<<nchunks, kMsThreads, 0, s>>>(src, mask, out, n, nchunks, ticket, tdesc, result, budget, row_len, sd, pub)
  switch (chunk_tiles) {
    case 1: TWG_MS_LAUNCH(1); break;
    case 2: TWG_MS_LAUNCH(2); break;
    case 4: TWG_MS_LAUNCH(4); break;
    case 8: TWG_MS_LAUNCH(8); break;
    case 16: TWG_MS_LAUNCH(16); break;
    default: TWG_MS_LAUNCH(32); break;
  }
#undef TWG_MS_LAUNCH
}

// Compaction of dense src by a bit mask (one bit per element, as predicate_bits_body writes it).
// `workspace` holds the ticket header and the chunk descriptors (twg_masked_select_workspace_bytes).
int ms_select_from_bits(const float* src, const unsigned* bits, float* out, int64_t n, int64_t* result_dev,
                        void* workspace, cudaStream_t s, const MsPublish& pub) {
  const int chunk_tiles = dense_chunk_tiles(n);
  const int64_t tile_elems = (int64_t)chunk_tiles * kMsRound;
  const int64_t nchunks = (n + tile_elems - 1) / tile_elems;
  TWG_REQUIRE(nchunks <= 0x7fffffff, "fused select: %lld elements exceed the chunk limit", (long long)n);
  if (int rc = ms_clear(workspace, kMsHeaderBytes + (size_t)nchunks * sizeof(u64), result_dev, s)) return rc;
  FastDiv32 row_len;
  row_len.d = 1u;
  make_fastdiv(row_len.d, &row_len.m, &row_len.s);
  StridedDesc<2, u32> sd;
  std::memset(&sd, 0, sizeof(sd));
  launch_dense<kMsBits>(chunk_tiles, (unsigned)nchunks, s, src, reinterpret_cast<const u8*>(bits), out, n,
                        static_cast<u64*>(workspace), reinterpret_cast<u64*>(static_cast<char*>(workspace) + kMsHeaderBytes),
                        reinterpret_cast<i64*>(result_dev), ms_poll_budget(), row_len, sd, pub);
  TWG_CHECK_LAUNCH();
  return TWG_OK;
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

// `fused_publish` in: the caller wants this rank's count published to `pub`; out: whether the
// compaction kernel did it (false: the caller launches the publish kernel behind this call).
static int masked_select_impl(const TwgIterDesc* desc, const float* src, const uint8_t* mask, float* out,
                              int64_t* result_dev, void* workspace, size_t workspace_bytes, void* stream,
                              const MsPublish& pub_in, bool* fused_publish) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  g_last_path = kPathNone;
  MsPublish pub = pub_in;
  if (fused_publish) *fused_publish = false;
  if (int rc = check_desc(desc, 2)) return rc;
  TWG_REQUIRE(result_dev != nullptr, "twg_masked_select_f32: result_dev is null");
  const int64_t n = desc->numel;
  if (n == 0) return ms_clear(nullptr, 0, result_dev, s);
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
                     is_aligned(src, 16) && is_aligned(mask, 16);
  // [R,C] source with a [R,1] mask: dimension 0 is the row (src stride 1, mask stride 0),
  // dimension 1 walks rows in both
  const bool rowmask = d.ndim == 2 && d.strides[0][0] == 1 && d.strides[1][0] == 0 && d.strides[0][1] == d.shape[0] &&
                       d.strides[1][1] == 1 && d.shape[0] % 4 == 0 && n < (int64_t(1) << 31) && is_aligned(src, 16);
  // anything else whose element count and offsets fit 32 bits goes through the same chunked
  // kernel with index math per element; only the rest keeps the one-tile-per-CTA kernel
  const bool strided32 = !dense && !rowmask && n < (int64_t(1) << 31) && fits_32bit(d, 2);
  if (dense || rowmask || strided32) {
    const int chunk_tiles = dense_chunk_tiles(n);
    const int64_t tile_elems = (int64_t)chunk_tiles * kMsRound;
    const int64_t ntiles = (n + tile_elems - 1) / tile_elems;
    TWG_REQUIRE(ntiles <= 0x7fffffff, "twg_masked_select_f32: %lld elements exceed the tile limit", (long long)n);
    if (int rc = ms_clear(workspace, kMsHeaderBytes + (size_t)ntiles * sizeof(u64), result_dev, s)) return rc;
    FastDiv32 row_len;
    row_len.d = rowmask ? (uint32_t)d.shape[0] : 1u;
    make_fastdiv(row_len.d, &row_len.m, &row_len.s);
    StridedDesc<2, u32> sd;
    std::memset(&sd, 0, sizeof(sd));
    if (strided32) fill_strided_desc<2>(d, &sd);
    if (dense) launch_dense<kMsDense>(chunk_tiles, (unsigned)ntiles, s, src, mask, out, n, ticket, tdesc, result, budget, row_len, sd, pub);
    else if (rowmask) launch_dense<kMsRowMask>(chunk_tiles, (unsigned)ntiles, s, src, mask, out, n, ticket, tdesc, result, budget, row_len, sd, pub);
    else launch_dense<kMsStrided>(chunk_tiles, (unsigned)ntiles, s, src, mask, out, n, ticket, tdesc, result, budget, row_len, sd, pub);
    TWG_CHECK_LAUNCH();
    if (fused_publish) *fused_publish = pub.nranks != 0;
    g_last_path = strided32 ? kPathStrided32 : kPathDense;
    return TWG_OK;
  }

  const int64_t ntiles = (n + kMsRound - 1) / kMsRound;
  TWG_REQUIRE(ntiles <= 0x7fffffff, "twg_masked_select_f32: %lld elements exceed the tile limit", (long long)n);
  if (int rc = ms_clear(workspace, need, result_dev, s)) return rc;
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

extern "C" int twg_masked_select_f32(const TwgIterDesc* desc, const float* src, const uint8_t* mask, float* out,
                                     int64_t* result_dev, void* workspace, size_t workspace_bytes, void* stream) {
  TWG_TRACE("twg_masked_select_f32");
  MsPublish none;
  std::memset(&none, 0, sizeof(none));
  return masked_select_impl(desc, src, mask, out, result_dev, workspace, workspace_bytes, stream, none, nullptr);
}

extern "C" int twg_masked_select_f32_publish(const TwgIterDesc* desc, const float* src, const uint8_t* mask, float* out,
                                             int64_t* result_dev, void* workspace, size_t workspace_bytes, void* xchg,
                                             int64_t seq, void* stream) {
  TWG_TRACE("twg_masked_select_f32_publish");
  MsPublish pub;
  std::memset(&pub, 0, sizeof(pub));
  if (int rc = xchg_publish_slots(xchg, seq, &pub)) return rc;
  bool fused = false;
  if (int rc = masked_select_impl(desc, src, mask, out, result_dev, workspace, workspace_bytes, stream, pub, &fused)) return rc;
  // layouts served by the one-tile-per-CTA kernel, and empty inputs: the publish kernel behind the compaction
  if (!fused) return twg_exchange_publish(xchg, seq, result_dev, stream);
  return TWG_OK;
}

// masked_select of dense src by a bit mask (bit i of 32-bit word w = element 32 w + i), as
// twg_fused_predicate_bits writes it.
static int select_bits_impl(const float* src, const uint32_t* bits, int64_t numel, float* out, int64_t* result_dev,
                            void* workspace, size_t workspace_bytes, void* stream, const MsPublish& pub, bool* published) {
  if (published) *published = false;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TWG_REQUIRE(result_dev != nullptr && numel >= 0, "twg_masked_select_bits_f32: null result or negative numel");
  g_last_path = kPathNone;
  if (numel == 0) return ms_clear(nullptr, 0, result_dev, s);
  TWG_REQUIRE(src && bits && out, "twg_masked_select_bits_f32: null argument");
  TWG_REQUIRE(is_aligned(src, 16) && is_aligned(bits, 16) && is_aligned(out, 4),
              "twg_masked_select_bits_f32: src and bits must be 16-byte aligned, out 4-byte aligned");
  const size_t need = twg_masked_select_workspace_bytes(numel);
  TWG_REQUIRE(workspace != nullptr && workspace_bytes >= need && is_aligned(workspace, 256),
              "twg_masked_select_bits_f32: workspace of %zu bytes is smaller than the %zu required or not 256-byte aligned",
              workspace_bytes, need);
  if (int rc = ms_select_from_bits(src, bits, out, numel, result_dev, workspace, s, pub)) return rc;
  g_last_path = kPathDense;
  if (published) *published = pub.nranks != 0;
  return TWG_OK;
}

extern "C" size_t twg_predicate_bits_bytes(int64_t numel) { return (size_t)predicate_bits_bytes(numel < 0 ? 0 : numel); }

extern "C" int twg_masked_select_bits_f32(const float* src, const uint32_t* bits, int64_t numel, float* out,
                                          int64_t* result_dev, void* workspace, size_t workspace_bytes, void* stream) {
  TWG_TRACE("twg_masked_select_bits_f32");
  MsPublish none;
  std::memset(&none, 0, sizeof(none));
  return select_bits_impl(src, bits, numel, out, result_dev, workspace, workspace_bytes, stream, none, nullptr);
}

extern "C" int twg_masked_select_bits_f32_publish(const float* src, const uint32_t* bits, int64_t numel, float* out,
                                                  int64_t* result_dev, void* workspace, size_t workspace_bytes, void* xchg,
                                                  int64_t seq, void* stream) {
  TWG_TRACE("twg_masked_select_bits_f32_publish");
  MsPublish pub;
  std::memset(&pub, 0, sizeof(pub));
  if (int rc = xchg_publish_slots(xchg, seq, &pub)) return rc;
  bool published = false;
  if (int rc = select_bits_impl(src, bits, numel, out, result_dev, workspace, workspace_bytes, stream, pub, &published)) return rc;
  if (!published) return twg_exchange_publish(xchg, seq, result_dev, stream);  // empty input
  return TWG_OK;
}

// ------------------------------------------------------------------------------------------
// masked_select without any allocation by anybody.
//
// twg_masked_select_f32 needs a scratch buffer (ticket counter + one descriptor per chunk) that
// the caller has to provide, which normally means the caller allocates device memory.  Some
// callers cannot: a host framework whose own allocator has reserved the whole device and which
// treats a foreign cudaMalloc as a failure; a plugin that is handed input and output buffers and
// nothing else, with no way to ask its host for more; a latency-critical loop that must not hit
// the implicit device synchronisation of cudaMalloc / cudaFree.  For them the scratch lives in
// the library image itself, as a file-scope __device__ array of fixed size.  Every GPU that loads
// the library holds these 513 KB until the process exits, used or not.
//
// The array's name below is only meaningful in device code.  On the host it is a stand-in symbol,
// not a device address, so its address is looked up once per device with cudaGetSymbolAddress
// (with that device current) and the looked-up pointer is what the kernels receive.
// ------------------------------------------------------------------------------------------
namespace twg {

constexpr int64_t kMsStaticMaxNumel = int64_t(1) << 28;
constexpr size_t kMsStaticBytes = kMsHeaderBytes + (size_t)(kMsStaticMaxNumel / kMsRound) * sizeof(u64);

static __device__ __align__(256) unsigned char g_ms_static_scratch[kMsStaticBytes];

static std::mutex g_ms_static_mu;
static void* g_ms_static_ptr[64] = {};  // per device ordinal; nullptr = not looked up yet

// Device address of the scratch array on the current device (looked up on first use).
static int ms_static_scratch(void** out) {
  int dev = 0;
  TWG_CUDA(cudaGetDevice(&dev));
  TWG_REQUIRE(dev >= 0 && dev < 64, "twg_masked_select_f32_static: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_ms_static_mu);
  if (g_ms_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    TWG_CUDA(cudaGetSymbolAddress(&p, g_ms_static_scratch));
    TWG_REQUIRE(p != nullptr && is_aligned(p, 256), "twg_masked_select_f32_static: bad scratch address %p", p);
    g_ms_static_ptr[dev] = p;
  }
  *out = g_ms_static_ptr[dev];
  return TWG_OK;
}

}  // namespace twg

extern "C" int64_t twg_masked_select_static_max_numel(void) { return twg::kMsStaticMaxNumel; }

extern "C" int twg_masked_select_f32_static(const TwgIterDesc* desc, const float* src, const uint8_t* mask, float* out,
                                            int64_t* result_dev, void* stream) {
  TWG_TRACE("twg_masked_select_f32_static");
  if (int rc = check_desc(desc, 2)) return rc;
  if (desc->numel > kMsStaticMaxNumel)
    return set_error(TWG_ERR_UNSUPPORTED,
                     "twg_masked_select_f32_static: %lld elements exceed the %lld this entry point's built-in scratch "
                     "is sized for; use twg_masked_select_f32 with a caller-provided workspace",
                     (long long)desc->numel, (long long)kMsStaticMaxNumel);
  void* scratch = nullptr;
  if (int rc = ms_static_scratch(&scratch)) return rc;
  // Same kernels, same clearing of the part of the scratch that must start at zero (done on
  // `stream` by the call below); only where the scratch comes from differs.
  return twg_masked_select_f32(desc, src, mask, out, result_dev, scratch, kMsStaticBytes, stream);
}
