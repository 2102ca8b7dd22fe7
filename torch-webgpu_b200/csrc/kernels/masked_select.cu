// masked_select as a single-pass stream compaction.
//
// One CTA owns a run of consecutive logical elements (a chunk of tiles on the dense path, one tile
// on the strided path).  Inside a tile, selected elements are ranked with popc on the packed mask
// bytes plus a warp scan (dense path) or with warp ballots (strided path); the run's base offset in
// the output comes from a decoupled look-back over the preceding runs' published counts, so one
// launch does everything, src is read exactly once and no global scan kernel is needed.  Selected values are first packed into shared memory in output order and
// then written as contiguous runs.
//
// Forward progress: a tile's index is a ticket drawn from a global counter when its CTA starts,
// not blockIdx, so every tile a CTA may wait for belongs to a CTA that is already running.  The
// wait is nevertheless bounded: after `poll_budget` polls the tile gives up, records
// TWG_ERR_TIMEOUT in result[1], publishes a prefix so that later tiles do not wait on it, and the
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
// Dense path: src contiguous and 16-byte aligned; the mask is either a dense bool array (16-byte
// aligned) or, with ROWMASK, one bool per row of `row_len` elements (a [R,1] mask broadcast over
// [R,C] with C % 4 == 0).  A third mode walks both operands through the iteration descriptor
// (element index -> offsets with 32-bit multiply-shift division): slices, broadcast masks and
// other non-dense layouts get the same chunking, at one index computation per mask byte and per
// selected element.
//
// A CTA owns a chunk of CH consecutive tiles of 4096 elements.
//   Phase A  reads the chunk's mask (1 byte per element), keeps it in shared memory packed to one
//            bit per element, and counts the selected elements of every warp span (512 elements)
//            of every tile.  The chunk count is published at once: the chain of dependent CTAs has
//            one link per chunk, not per tile, and its latency is amortised over CH tiles.
//   Phase B  With the table of phase A each warp knows where its run of every tile starts inside
//            the chunk before it has looked at a single src value, so there is no barrier and no
//            exchange between warps: a warp loads its span (src quads whose four mask bits are
//            all zero are never fetched; the next tile's loads are issued before the current one
//            is ranked), ranks it with popc + a warp scan, stages into its own 2 KB region and
//            writes its run out, tile after tile.  The look-back is resolved as late as possible
//            - after tile 0 is staged, right before its flush - so that most predecessors have
//            published by then; the two barriers around it are the only CTA-wide ones.
// In a tile a warp covers 512 consecutive elements as 4 sub-rounds of 32 quads; lane l owns quad
// j*32+l of sub-round j, so src is read as 512-byte runs.  HBM sees every mask byte and every
// selected sector of src once.  (An earlier form ranked across the eight warps of a tile with two
// barriers per tile; ncu showed it issue-bound at 31 instructions per element with the barrier
// among the top stalls.  Measured, 2^30 elements at 41 % density: 1.246 ms -> 1.197 ms.)
// ------------------------------------------------------------------------------------------
// four arbitrary bytes -> four 0/1 bytes (non-zero counts as true): the carry of (b & 0x7f) + 0x7f
// reaches bit 7 exactly when the low seven bits are non-zero
__device__ __forceinline__ u32 nonzero_bytes(u32 w) {
  return ((((w & 0x7f7f7f7fu) + 0x7f7f7f7fu) | w) >> 7) & 0x01010101u;
}
// How the chunked kernel addresses its operands.
constexpr int kMsDense = 0;    // src and mask dense
constexpr int kMsRowMask = 1;  // src dense, one mask byte per row
constexpr int kMsStrided = 2;  // both through the iteration descriptor (32-bit index math)

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

template <int CH>
struct MsDenseShared {
  float stage[kMsRound];  // warp w stages into [w*512, (w+1)*512)
  alignas(16) unsigned short cnt[CH][kMsWarps];
  u32 reduce[kMsWarps];
  i64 tile;
  i64 excl;
};

template <int CH, int MODE>
__global__ void __launch_bounds__(kMsThreads, 4)
    ms_dense_kernel(const float* src, const u8* mask, float* out, i64 n, i64 nchunks, u64* ticket, u64* desc,
                     i64* result, i64 poll_budget, FastDiv32 row_len, StridedDesc<2, u32> sd) {
  constexpr bool ROWMASK = MODE == kMsRowMask;
  __shared__ MsDenseShared<CH> sm;
  __shared__ u32 bits[CH * (kMsRound / 32)];  // the chunk's mask, one bit per element
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  i64 chunk = blockIdx.x;
  if (ticket != nullptr) {
    if (threadIdx.x == 0) sm.tile = (i64)atomicAdd(ticket, 1ull);
    __syncthreads();
    chunk = sm.tile;
  }
  if (chunk >= nchunks) return;
  const i64 chunk_base = chunk * (i64)(CH * kMsRound);
  const bool full_chunk = chunk_base + (i64)(CH * kMsRound) <= n;

  // ---- phase A: mask -> bits, counts per (tile, warp span), chunk count ----
  u32 c = 0;
  if (MODE == kMsDense && full_chunk) {
    unsigned short* bits16 = reinterpret_cast<unsigned short*>(bits);
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      uint4 q = ld_v4(mask + chunk_base + (i64)i * kMsRound + threadIdx.x * 16);
      const u32 sixteen = bytes_to_nibble(nonzero_bytes(q.x)) | (bytes_to_nibble(nonzero_bytes(q.y)) << 4) |
                          (bytes_to_nibble(nonzero_bytes(q.z)) << 8) | (bytes_to_nibble(nonzero_bytes(q.w)) << 12);
      const u32 ci = __popc(sixteen);
      c += ci;
      bits16[i * kMsThreads + threadIdx.x] = (unsigned short)sixteen;
      const u32 span = __reduce_add_sync(0xffffffffu, ci);  // this warp's 512 bytes are exactly its span of tile i
      if (lane == 0) sm.cnt[i][warp] = (unsigned short)span;
    }
  } else if constexpr (MODE == kMsStrided) {
    // a warp takes whole spans; lane l looks at element 32 g + l of word g, so that neighbouring
    // lanes read neighbouring mask bytes, and a ballot is the word
    for (int sidx = warp; sidx < CH * kMsWarps; sidx += kMsWarps) {
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
        sm.cnt[sidx >> 3][sidx & 7] = (unsigned short)span_count;
        c += span_count;
      }
    }
  } else {
    // one word of bits = 32 consecutive elements, 16 words = one warp span: half a warp per span
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
      if ((lane & 15) == 0) sm.cnt[g >> 7][(g & 127) >> 4] = (unsigned short)cw;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if (lane == 0) sm.reduce[warp] = c;
  __syncthreads();
  u32 chunk_total = 0;
#pragma unroll
  for (int w = 0; w < kMsWarps; ++w) chunk_total += sm.reduce[w];
  if (threadIdx.x == 0) lookback_publish(chunk, chunk_total, desc, poll_budget);
  const int tiles_here = full_chunk ? CH : (int)((n - chunk_base + kMsRound - 1) / kMsRound);

  // ---- phase B for sparse chunks (fewer than one element in sixteen selected) ----
  // Ranking, staging and quad loads cost the same whether anything is selected or not; here a
  // lane walks the set bits of its 16 elements instead: one scalar load and one store per selected
  // element, and spans that select nothing are skipped with one look at the table of phase A.
  if (chunk_total * 16u < (u32)(CH * kMsRound)) {
    if (warp == 0) {
      const i64 excl = lookback_resolve(chunk, chunk_total, desc, result, poll_budget);
      if (lane == 0) {
        sm.excl = excl;
        if (chunk == nchunks - 1) result[0] = excl + (i64)chunk_total;
      }
    }
    __syncthreads();
    float* chunk_out = out + sm.excl;
    u32 tile_off = 0;
    for (int t = 0; t < tiles_here; ++t) {
      const u32 mine = sm.cnt[t][warp];
      u32 before = 0, tile_total = 0;  // selected by the spans in front of this one / by the whole tile
#pragma unroll
      for (int w = 0; w < kMsWarps; ++w) {
        const u32 x = sm.cnt[t][w];
        if (w < warp) before += x;
        tile_total += x;
      }
      if (mine != 0u) {
        const u32 word = bits[t * (kMsRound / 32) + warp * 16 + (lane >> 1)];
        u32 half = (word >> ((lane & 1) * 16)) & 0xffffu;  // this lane's 16 consecutive elements
        const u32 cnt = __popc(half);
        u32 incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const u32 x = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += x;
        }
        const i64 first = chunk_base + (i64)t * kMsRound + (i64)warp * 512 + lane * 16;
        float* to = chunk_out + tile_off + before + (incl - cnt);
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
      }
      tile_off += tile_total;
    }
    return;
  }

  // ---- phase B: every warp compacts its span of every tile on its own ----
  struct TileRegs {
    u32 m[4];     // the four mask bits of this lane's quad in each sub-round
    u32 v[4][4];  // its src values (loaded only where a bit is set)
  };
  auto load_tile = [&](TileRegs& r, int t) {
    const i64 tb = chunk_base + (i64)t * kMsRound + (i64)warp * 512;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int q = warp * 128 + j * 32 + lane;
      const i64 e = tb + (i64)(j * 32 + lane) * 4;
      r.m[j] = (bits[t * (kMsRound / 32) + (q >> 3)] >> ((q & 7) * 4)) & 0xfu;  // 0 beyond n
      if constexpr (MODE == kMsStrided) {
        if (r.m[j] != 0u) {  // set bits only exist below n
          u32 os0, om;
          const u32 c0 = ms_offsets(sd, (u32)e, os0, om);
          if (sd.strides[0][0] == 1u && c0 + 3 < sd.shape[0].d && ((reinterpret_cast<unsigned long long>(src + os0) & 15ull) == 0)) {
            const uint4 x = ld_v4(src + os0);  // the quad is one aligned 16-byte piece of src
            r.v[j][0] = x.x; r.v[j][1] = x.y; r.v[j][2] = x.z; r.v[j][3] = x.w;
          } else {
            // neighbouring elements share sectors: let L1 serve the repeats
#pragma unroll
            for (int b = 0; b < 4; ++b)
              if ((r.m[j] >> b) & 1u) {
                u32 o = os0 + b * sd.strides[0][0];
                if (c0 + b >= sd.shape[0].d) ms_offsets(sd, (u32)(e + b), o, om);  // the quad runs into the next row
                r.v[j][b] = __float_as_uint(__ldg(src + o));
              }
          }
        }
      } else if (r.m[j] != 0u) {
        if (full_chunk || e + 3 < n) {
          const uint4 x = ld_v4(src + e);
          r.v[j][0] = x.x; r.v[j][1] = x.y; r.v[j][2] = x.z; r.v[j][3] = x.w;
        } else {
#pragma unroll
          for (int b = 0; b < 4; ++b) r.v[j][b] = (e + b < n) ? ld_b32(src + e + b) : 0u;
        }
      }
    }
  };
  float* region = sm.stage + warp * 512;
  u32 tile_off = 0;  // selected elements of the chunk's earlier tiles
  auto compact_tile = [&](const TileRegs& r, int t) {
    // where this warp's run starts inside the chunk: the table of phase A
    const uint4 row = *reinterpret_cast<const uint4*>(sm.cnt[t]);
    const u32 c01 = row.x, c23 = row.y, c45 = row.z, c67 = row.w;
    const u32 pair[4] = {(c01 & 0xffffu) + (c01 >> 16), (c23 & 0xffffu) + (c23 >> 16), (c45 & 0xffffu) + (c45 >> 16),
                         (c67 & 0xffffu) + (c67 >> 16)};
    u32 warp_off = 0;
#pragma unroll
    for (int p = 0; p < 4; ++p)
      if (2 * p + 1 < warp) warp_off += pair[p];
    if (warp & 1) {
      const u32 lo[4] = {c01 & 0xffffu, c23 & 0xffffu, c45 & 0xffffu, c67 & 0xffffu};
      warp_off += lo[warp >> 1];
    }
    const u32 tile_total = pair[0] + pair[1] + pair[2] + pair[3];

    // ranks inside the warp: per-sub-round counts packed into one word (each field <= 128)
    const u32 cnt = __popc(r.m[0]) | (__popc(r.m[1]) << 8) | (__popc(r.m[2]) << 16) | (__popc(r.m[3]) << 24);
    u32 incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const u32 x = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += x;
    }
    const u32 tot = __shfl_sync(0xffffffffu, incl, 31);
    const u32 t0 = tot & 0xffu, t1 = (tot >> 8) & 0xffu, t2 = (tot >> 16) & 0xffu, t3 = tot >> 24;
    const u32 excl_w = incl - cnt;
    const u32 sub_base[4] = {0u, t0, t0 + t1, t0 + t1 + t2};
    const u32 run = t0 + t1 + t2 + t3;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (r.m[j] != 0u) {
        u32 pos = sub_base[j] + ((excl_w >> (8 * j)) & 0xffu);
#pragma unroll
        for (int b = 0; b < 4; ++b)
          if ((r.m[j] >> b) & 1u) region[pos++] = __uint_as_float(r.v[j][b]);
      }
    }
    if (t == 0) {
      // the look-back as late as possible: tile 0 is staged, most predecessors have published
      if (warp == 0) {
        const i64 excl = lookback_resolve(chunk, chunk_total, desc, result, poll_budget);
        if (lane == 0) {
          sm.excl = excl;
          if (chunk == nchunks - 1) result[0] = excl + (i64)chunk_total;
        }
      }
      __syncthreads();
    } else {
      __syncwarp();
    }
    // this warp's run: 128-bit stores between the first and last 16-byte boundary
    float* dst = out + sm.excl + tile_off + warp_off;
    const u32 head = min(run, (u32)(((16u - (u32)(reinterpret_cast<unsigned long long>(dst) & 15ull)) & 15u) >> 2));
    if ((u32)lane < head) dst[lane] = region[lane];
    const u32 nvec = (run - head) >> 2;
    float4* dst4 = reinterpret_cast<float4*>(dst + head);
    for (u32 i = lane; i < nvec; i += 32) {
      const float* s4 = region + head + 4 * i;
      dst4[i] = make_float4(s4[0], s4[1], s4[2], s4[3]);
    }
    const u32 tail0 = head + 4 * nvec;
    if (tail0 + lane < run) dst[tail0 + lane] = region[tail0 + lane];
    tile_off += tile_total;
    __syncwarp();  // the region is rewritten by the next tile
  };
  TileRegs next;
  load_tile(next, 0);
  for (int t = 0; t < tiles_here; ++t) {
    const TileRegs cur = next;
    if (t + 1 < tiles_here) load_tile(next, t + 1);  // in flight while this tile is ranked and written out
    compact_tile(cur, t);
  }
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

// Tiles per dense chunk: the largest power of two up to 32 that still leaves about four waves
// of chunks on the device, so that large tensors amortise the look-back over long chunks and small
// ones still fill every SM.  TWG_MS_CHUNK (1..32, power of two) overrides it for experiments.
static int dense_chunk_tiles(int64_t n) {
  static const int forced = [] {
    const char* env = getenv("TWG_MS_CHUNK");
    const int r = env ? atoi(env) : 0;
    return (r == 1 || r == 2 || r == 4 || r == 8 || r == 16 || r == 32) ? r : 0;
  }();
  if (forced) return forced;
  const int64_t tiles = (n + kMsRound - 1) / kMsRound;
  const int64_t want_chunks = 4ll * 4 * sm_count();
  int ch = 32;
  while (ch > 1 && tiles / ch < want_chunks) ch >>= 1;
  return ch;
}

long long ms_poll_budget() { return g_poll_budget.load(); }

// Tile order.  Default: tickets from a global counter (forward progress does not depend on the
// order in which the hardware starts CTAs).  TWG_MS_ORDER=blockidx uses blockIdx.x instead, for
// measuring what the ticket costs.
bool ms_use_ticket() {
  static const bool v = [] {
    const char* env = getenv("TWG_MS_ORDER");
    return !(env && std::string(env) == "blockidx");
  }();
  return v;
}

template <int MODE>
static void launch_dense(int chunk_tiles, unsigned nchunks, cudaStream_t s, const float* src, const u8* mask, float* out,
                         i64 n, u64* ticket, u64* tdesc, i64* result, i64 budget, FastDiv32 row_len,
                         const StridedDesc<2, u32>& sd) {
#define TWG_MS_LAUNCH(CH) \
  ms_dense_kernel<CH, MODE><<<nchunks, kMsThreads, 0, s>>>(src, mask, out, n, nchunks, ticket, tdesc, result, budget, row_len, sd)
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
  u64* ticket = ms_use_ticket() ? static_cast<u64*>(workspace) : nullptr;
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
    TWG_CUDA(cudaMemsetAsync(workspace, 0, kMsHeaderBytes + (size_t)ntiles * sizeof(u64), s));
    FastDiv32 row_len;
    row_len.d = rowmask ? (uint32_t)d.shape[0] : 1u;
    make_fastdiv(row_len.d, &row_len.m, &row_len.s);
    StridedDesc<2, u32> sd;
    std::memset(&sd, 0, sizeof(sd));
    if (strided32) fill_strided_desc<2>(d, &sd);
    if (dense) launch_dense<kMsDense>(chunk_tiles, (unsigned)ntiles, s, src, mask, out, n, ticket, tdesc, result, budget, row_len, sd);
    else if (rowmask) launch_dense<kMsRowMask>(chunk_tiles, (unsigned)ntiles, s, src, mask, out, n, ticket, tdesc, result, budget, row_len, sd);
    else launch_dense<kMsStrided>(chunk_tiles, (unsigned)ntiles, s, src, mask, out, n, ticket, tdesc, result, budget, row_len, sd);
    TWG_CHECK_LAUNCH();
    g_last_path = strided32 ? kPathStrided32 : kPathDense;
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
