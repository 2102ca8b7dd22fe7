// Device-side building blocks of every pointwise kernel in the library: the element functions,
// the three launch shapes (dense 128-bit vector path, 2-D permuted tile path, generic
// strided/broadcast index-math path) and the functor protocol that binds them.
//
// The same header is compiled ahead of time by nvcc into the library and, as text, by NVRTC for
// fused programs built at torch.compile time, so it must not include any host header.
//
// Functor protocol (type F):
//   static constexpr int NIN, NOUT            number of inputs / outputs
//   static constexpr unsigned kInByteMask     bit k set: input k is 1-byte (bool/u8), else f32
//   static constexpr unsigned kOutByteMask    same for outputs
//   __device__ void operator()(const u32* in, u32* out) const
// Values travel in 32-bit registers: f32 as its bit pattern, bool as 0/1.
#pragma once

namespace twg {

typedef unsigned int u32;
typedef unsigned char u8;
typedef long long i64;
typedef unsigned long long u64;

constexpr int kMaxDims = 8;
constexpr int kBlock = 256;  // threads per CTA of the dense and strided kernels

// ------------------------------------------------------------------------------------------
// Element functions.  They restate PyTorch's CPU kernels, which is what the reference's tests
// assert against and what its CPU-fallback ops execute; explicit _rn intrinsics keep the
// compiler from contracting or reassociating anything.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float f_add(float a, float b, float alpha) { return __fmaf_rn(alpha, b, a); }
__device__ __forceinline__ float f_mul(float a, float b) { return __fmul_rn(a, b); }
// max(0,x) that keeps NaN and -0.0 (clamp_min semantics of the CPU kernel).
__device__ __forceinline__ float f_div(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float f_relu(float x) { return (x < 0.0f) ? 0.0f : x; }
__device__ __forceinline__ float f_abs(float x) { return fabsf(x); }
__device__ __forceinline__ float f_silu(float x) {
  return __fdiv_rn(x, __fadd_rn(1.0f, expf(-x)));
}
__device__ __forceinline__ float f_gelu_erf(float x) {
  // x * 0.5 * (1 + erf(x / sqrt(2)))
  const float kAlpha = 0.70710678118654752440f;
  return __fmul_rn(__fmul_rn(x, 0.5f), __fadd_rn(1.0f, erff(__fmul_rn(x, kAlpha))));
}
__device__ __forceinline__ float f_gelu_tanh(float x) {
  // 0.5 * x * (1 + tanh(sqrt(2/pi) * (x + 0.044715 x^3)))
  const float kBeta = 0.79788456080286535588f;  // sqrt(2) * (2/sqrt(pi)) * 0.5
  const float kKappa = 0.044715f;
  float x3 = __fmul_rn(__fmul_rn(x, x), x);
  float inner = __fmul_rn(kBeta, __fadd_rn(x, __fmul_rn(kKappa, x3)));
  return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, tanhf(inner)));
}
__device__ __forceinline__ u32 f_eq(float a, float b) { return a == b ? 1u : 0u; }
__device__ __forceinline__ u32 f_ne(float a, float b) { return a != b ? 1u : 0u; }
__device__ __forceinline__ u32 f_lt(float a, float b) { return a < b ? 1u : 0u; }
__device__ __forceinline__ u32 f_le(float a, float b) { return a <= b ? 1u : 0u; }
__device__ __forceinline__ u32 f_gt(float a, float b) { return a > b ? 1u : 0u; }
__device__ __forceinline__ u32 f_ge(float a, float b) { return a >= b ? 1u : 0u; }
__device__ __forceinline__ u32 f_and(u32 a, u32 b) { return a & b; }

__device__ __forceinline__ float as_f(u32 v) { return __uint_as_float(v); }
__device__ __forceinline__ u32 as_u(float v) { return __float_as_uint(v); }

// ------------------------------------------------------------------------------------------
// Memory access helpers.  Streaming hints: every byte is touched once, so loads do not
// allocate in L1 and stores are marked evict-first.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ u32 ld_b32(const void* p) {
  u32 r;
  asm volatile("ld.global.L1::no_allocate.u32 %0, [%1];" : "=r"(r) : "l"(p));
  return r;
}
__device__ __forceinline__ u32 ld_b8(const void* p) {
  u32 r;
  asm volatile("ld.global.L1::no_allocate.u8 %0, [%1];" : "=r"(r) : "l"(p));
  return r;
}
__device__ __forceinline__ void st_v4(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_b32(void* p, u32 v) {
  asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_b8(void* p, u32 v) {
  asm volatile("st.global.cs.u8 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One "unit" is VEC consecutive elements: 4 when any operand is f32 (float4 / uchar4 accesses),
// 16 when every operand is a byte type (uint4 accesses).
template <int VEC, bool BYTE>
__device__ __forceinline__ void load_unit(const void* base, i64 unit, u32 (&r)[VEC]) {
  if constexpr (!BYTE) {
    static_assert(VEC == 4, "f32 units are 4 wide");
    uint4 v = ld_v4(reinterpret_cast<const uint4*>(base) + unit);
    r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
  } else if constexpr (VEC == 4) {
    u32 w = ld_b32(reinterpret_cast<const u32*>(base) + unit);
    w = __vcmpne4(w, 0u) & 0x01010101u;  // any non-zero byte counts as true
    r[0] = w & 0xffu; r[1] = (w >> 8) & 0xffu; r[2] = (w >> 16) & 0xffu; r[3] = w >> 24;
  } else {
    static_assert(VEC == 16, "byte units are 4 or 16 wide");
    uint4 v = ld_v4(reinterpret_cast<const uint4*>(base) + unit);
    u32 w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      r[4 * i + 0] = w[i] & 0xffu; r[4 * i + 1] = (w[i] >> 8) & 0xffu;
      r[4 * i + 2] = (w[i] >> 16) & 0xffu; r[4 * i + 3] = w[i] >> 24;
    }
  }
}
template <int VEC, bool BYTE>
__device__ __forceinline__ void store_unit(void* base, i64 unit, const u32 (&r)[VEC]) {
  if constexpr (!BYTE) {
    st_v4(reinterpret_cast<uint4*>(base) + unit, make_uint4(r[0], r[1], r[2], r[3]));
  } else if constexpr (VEC == 4) {
    st_b32(reinterpret_cast<u32*>(base) + unit, r[0] | (r[1] << 8) | (r[2] << 16) | (r[3] << 24));
  } else {
    uint4 v;
    v.x = r[0] | (r[1] << 8) | (r[2] << 16) | (r[3] << 24);
    v.y = r[4] | (r[5] << 8) | (r[6] << 16) | (r[7] << 24);
    v.z = r[8] | (r[9] << 8) | (r[10] << 16) | (r[11] << 24);
    v.w = r[12] | (r[13] << 8) | (r[14] << 16) | (r[15] << 24);
    st_v4(reinterpret_cast<uint4*>(base) + unit, v);
  }
}
template <bool BYTE>
__device__ __forceinline__ u32 load_elem(const void* base, i64 idx) {
  if constexpr (BYTE) return ld_b8(reinterpret_cast<const u8*>(base) + idx);
  else return ld_b32(reinterpret_cast<const u32*>(base) + idx);
}
template <bool BYTE>
__device__ __forceinline__ void store_elem(void* base, i64 idx, u32 v) {
  if constexpr (BYTE) st_b8(reinterpret_cast<u8*>(base) + idx, v);
  else st_b32(reinterpret_cast<u32*>(base) + idx, v);
}

template <int NT>
struct PwPtrs {
  void* p[NT];  // outputs first, then inputs
};

template <class F>
struct PwTraits {
  static constexpr int NIN = F::NIN, NOUT = F::NOUT, NT = F::NIN + F::NOUT;
  __host__ __device__ static constexpr bool in_byte(int k) { return (F::kInByteMask >> k) & 1u; }
  __host__ __device__ static constexpr bool out_byte(int k) { return (F::kOutByteMask >> k) & 1u; }
  __host__ __device__ static constexpr bool all_bytes() {
    return F::kInByteMask == ((1u << F::NIN) - 1u) && F::kOutByteMask == ((1u << F::NOUT) - 1u);
  }
  static constexpr int VEC = all_bytes() ? 16 : 4;
};

// compile-time loops over operands (operand type is a template argument of load/store)
template <class F, int VEC, int K = 0>
__device__ __forceinline__ void load_inputs_unit(const PwPtrs<PwTraits<F>::NT>& ptrs, i64 unit,
                                                 u32 (&v)[F::NIN][VEC]) {
  if constexpr (K < F::NIN) {
    load_unit<VEC, PwTraits<F>::in_byte(K)>(ptrs.p[F::NOUT + K], unit, v[K]);
    load_inputs_unit<F, VEC, K + 1>(ptrs, unit, v);
  }
}
template <class F, int VEC, int K = 0>
__device__ __forceinline__ void store_outputs_unit(const PwPtrs<PwTraits<F>::NT>& ptrs, i64 unit,
                                                   const u32 (&v)[F::NOUT][VEC]) {
  if constexpr (K < F::NOUT) {
    store_unit<VEC, PwTraits<F>::out_byte(K)>(ptrs.p[K], unit, v[K]);
    store_outputs_unit<F, VEC, K + 1>(ptrs, unit, v);
  }
}
template <class F, int K = 0>
__device__ __forceinline__ void load_inputs_elem(const PwPtrs<PwTraits<F>::NT>& ptrs, const i64* off,
                                                 u32* v) {
  if constexpr (K < F::NIN) {
    u32 x = load_elem<PwTraits<F>::in_byte(K)>(ptrs.p[F::NOUT + K], off[F::NOUT + K]);
    if constexpr (PwTraits<F>::in_byte(K)) x = (x != 0u) ? 1u : 0u;
    v[K] = x;
    load_inputs_elem<F, K + 1>(ptrs, off, v);
  }
}
template <class F, int K = 0>
__device__ __forceinline__ void store_outputs_elem(const PwPtrs<PwTraits<F>::NT>& ptrs, const i64* off,
                                                   const u32* v) {
  if constexpr (K < F::NOUT) {
    store_elem<PwTraits<F>::out_byte(K)>(ptrs.p[K], off[K], v[K]);
    store_outputs_elem<F, K + 1>(ptrs, off, v);
  }
}

template <class F, int VEC>
__device__ __forceinline__ void apply_unit(const F& f, const u32 (&vin)[F::NIN][VEC], u32 (&vout)[F::NOUT][VEC]) {
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    u32 in[F::NIN > 0 ? F::NIN : 1], out[F::NOUT];
#pragma unroll
    for (int k = 0; k < F::NIN; ++k) in[k] = vin[k][e];
    f(in, out);
#pragma unroll
    for (int k = 0; k < F::NOUT; ++k) vout[k][e] = out[k];
  }
}

// ------------------------------------------------------------------------------------------
// Dense path.  All operands are contiguous and aligned to their unit size.  Each CTA walks
// chunks of kBlock*U units; inside a chunk a thread owns units threadIdx.x + u*kBlock, so every
// warp-wide access is one contiguous 512-byte (f32) or 128-byte (bool) run.  All loads of a
// chunk are issued before the first use to keep U*NIN 128-bit requests in flight per thread.
// `n` is the element count; the < VEC leftover elements are handled by CTA 0.
// ------------------------------------------------------------------------------------------
template <class F, int U>
__device__ __forceinline__ void pw_contig_body(const PwPtrs<PwTraits<F>::NT>& ptrs, const F& f, i64 nunits, i64 n) {
  constexpr int VEC = PwTraits<F>::VEC;
  const i64 chunk_units = (i64)kBlock * U;
  const i64 nchunks = (nunits + chunk_units - 1) / chunk_units;
  for (i64 c = blockIdx.x; c < nchunks; c += gridDim.x) {
    const i64 u0 = c * chunk_units + threadIdx.x;
    u32 vin[U][F::NIN > 0 ? F::NIN : 1][VEC];
    u32 vout[U][F::NOUT][VEC];
    if (u0 + (i64)(U - 1) * kBlock < nunits) {
#pragma unroll
      for (int u = 0; u < U; ++u) load_inputs_unit<F, VEC>(ptrs, u0 + (i64)u * kBlock, vin[u]);
#pragma unroll
      for (int u = 0; u < U; ++u) apply_unit<F, VEC>(f, vin[u], vout[u]);
#pragma unroll
      for (int u = 0; u < U; ++u) store_outputs_unit<F, VEC>(ptrs, u0 + (i64)u * kBlock, vout[u]);
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (u0 + (i64)u * kBlock < nunits) load_inputs_unit<F, VEC>(ptrs, u0 + (i64)u * kBlock, vin[u]);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (u0 + (i64)u * kBlock < nunits) {
          apply_unit<F, VEC>(f, vin[u], vout[u]);
          store_outputs_unit<F, VEC>(ptrs, u0 + (i64)u * kBlock, vout[u]);
        }
    }
  }
  const i64 tail0 = nunits * VEC;
  if (blockIdx.x == 0 && tail0 + threadIdx.x < n) {
    i64 off[PwTraits<F>::NT];
#pragma unroll
    for (int t = 0; t < PwTraits<F>::NT; ++t) off[t] = tail0 + threadIdx.x;
    u32 in[F::NIN > 0 ? F::NIN : 1], out[F::NOUT];
    load_inputs_elem<F>(ptrs, off, in);
    f(in, out);
    store_outputs_elem<F>(ptrs, off, out);
  }
}

// ------------------------------------------------------------------------------------------
// Generic path: up to 8 dimensions, any strides including 0 (broadcast).  Consecutive threads
// take consecutive linear indices, i.e. they walk dimension 0 (the fastest one), so accesses
// coalesce whenever an operand's dimension-0 stride is 1.  IDX is u32 when the element count
// and every operand's largest offset stay below 2^31 (division by multiply-shift), else u64.
// ------------------------------------------------------------------------------------------
struct FastDiv32 {
  u32 d, m, s;
  __device__ __forceinline__ u32 div(u32 n) const { return (__umulhi(n, m) + n) >> s; }  // n < 2^31
};

template <int NT, class IDX>
struct StridedDesc;
template <int NT>
struct StridedDesc<NT, u32> {
  int ndim;
  FastDiv32 shape[kMaxDims];
  u32 strides[NT][kMaxDims];
};
template <int NT>
struct StridedDesc<NT, u64> {
  int ndim;
  u64 shape[kMaxDims];
  i64 strides[NT][kMaxDims];
};

template <int NT>
__device__ __forceinline__ void linear_to_offsets(const StridedDesc<NT, u32>& d, u32 lin, i64* off) {
  u32 o[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) o[t] = 0;
#pragma unroll
  for (int k = 0; k < kMaxDims; ++k) {
    if (k >= d.ndim) break;
    u32 q = d.shape[k].div(lin);
    u32 c = lin - q * d.shape[k].d;
    lin = q;
#pragma unroll
    for (int t = 0; t < NT; ++t) o[t] += c * d.strides[t][k];
  }
#pragma unroll
  for (int t = 0; t < NT; ++t) off[t] = (i64)o[t];
}
template <int NT>
__device__ __forceinline__ void linear_to_offsets(const StridedDesc<NT, u64>& d, u64 lin, i64* off) {
#pragma unroll
  for (int t = 0; t < NT; ++t) off[t] = 0;
#pragma unroll
  for (int k = 0; k < kMaxDims; ++k) {
    if (k >= d.ndim) break;
    u64 q = lin / d.shape[k];
    i64 c = (i64)(lin - q * d.shape[k]);
    lin = q;
#pragma unroll
    for (int t = 0; t < NT; ++t) off[t] += c * d.strides[t][k];
  }
}

template <class F, int U, class IDX>
__device__ __forceinline__ void pw_strided_body(const PwPtrs<PwTraits<F>::NT>& ptrs, const F& f,
                                                const StridedDesc<PwTraits<F>::NT, IDX>& d, i64 n) {
  constexpr int NT = PwTraits<F>::NT;
  const i64 step = (i64)gridDim.x * kBlock * U;
  for (i64 base = (i64)blockIdx.x * kBlock * U + threadIdx.x; base < n; base += step) {
    i64 off[U][NT];
    u32 in[U][F::NIN > 0 ? F::NIN : 1], out[U][F::NOUT];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const i64 e = base + (i64)u * kBlock;
      if (e < n) {
        linear_to_offsets<NT>(d, (IDX)e, off[u]);
        load_inputs_elem<F>(ptrs, off[u], in[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const i64 e = base + (i64)u * kBlock;
      if (e < n) {
        f(in[u], out[u]);
        store_outputs_elem<F>(ptrs, off[u], out[u]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// 2-D permuted path (a true transpose: some operands are dense along dimension 0, the others
// along dimension 1).  A CTA of 32x8 threads owns a 64x64 tile, 16 elements per thread, so that a
// CTA has 16 KB per operand in flight.  (Measured: 512 threads with 8 elements each - more warps,
// fewer bytes in flight per SM - is slower for every functor: 0.92 / 0.76 / 0.70 of the copy peak
// for relu / silu / gelu on a 16384^2 transpose against 0.97 / 0.83 / 0.76; what this shape needs
// is bytes in flight, not warps.)  In registers a thread holds the tile in "dimension-0 order":
// elements (tx + 32a, ty + 8r).  Operands dense along dimension 0 are accessed directly
// in that order; operands dense along dimension 1 are accessed with tx running along dimension 1
// and pass through one padded shared-memory tile (row pitch 65: both the row-wise writes and
// the column-wise reads are conflict-free), so every global access is a 128-byte run.
// bit t of `dim1_mask` set: operand t is dense along dimension 1.
// ------------------------------------------------------------------------------------------
constexpr int kTile = 32;      // tile edge of the element-size-generic kernels (copy.cu)
constexpr int kPwTile = 64;    // tile edge of the functor kernels
constexpr int kTileX = 32;
constexpr int kTileRows = 8;                  // thread rows of the element-size-generic kernels (copy.cu)
constexpr int kPwRows = 8;                    // thread rows of the functor kernels: 32 x 8 = 256 threads
constexpr int kTileXR = kPwTile / kTileX;     // 2
constexpr int kTileYR = kPwTile / kPwRows;    // 8
constexpr int kTileElems = kTileXR * kTileYR; // 16 per thread
constexpr int kTileVecRows = kTileX * kPwRows / 16;  // rows one pass of the 128-bit path covers (16 threads per row)
constexpr int kTilePersistCtas = 4;           // CTAs per SM of the pipelined tile kernel (heavy one-input functors)
constexpr int kTileSuper = 8;                 // tiles per super-block edge

template <int NT>
struct TileDesc {
  i64 shape0, shape1;
  i64 tiles0, tiles1;  // ceil(shape / tile edge) along dimension 0 / 1
  i64 sb0;             // super-blocks along dimension 0 (functor kernels)
  FastDiv32 sb0_div;   // the same as a multiply-shift divisor
  i64 ntiles;          // CTAs' worth of work: tiles, or padded super-block slots
  i64 s0[NT], s1[NT];
  u32 dim1_mask;
  u32 vec;  // every operand is 4 bytes wide, 16-byte aligned, unit stride along its dense dimension
            // and a multiple of 4 along the other: interior tiles may use 128-bit accesses
};

typedef u32 (*PwTileSmem)[kPwTile + 1];

// INTERIOR: the whole 64x64 tile lies inside the tensor, so no element needs a bounds check.
// Offsets advance by precomputed per-step deltas instead of two 64-bit multiplies per element.
template <class F, bool INTERIOR, int K = 0>
__device__ __forceinline__ void tile_load_inputs(const PwPtrs<PwTraits<F>::NT>& ptrs, const TileDesc<PwTraits<F>::NT>& d,
                                                 i64 t0, i64 t1, PwTileSmem smem,
                                                 u32 (&v)[kTileElems][F::NIN > 0 ? F::NIN : 1]) {
  if constexpr (K < F::NIN) {
    constexpr int T = F::NOUT + K;
    constexpr bool BYTE = PwTraits<F>::in_byte(K);
    const int tx = threadIdx.x, ty = threadIdx.y;
    const i64 s0 = d.s0[T], s1 = d.s1[T];
    if ((d.dim1_mask >> T) & 1u) {
      // tx runs along dimension 1: element (i0 = t0 + ty + 8r, i1 = t1 + tx + 32a)
      const i64 base = (t0 + ty) * s0 + (t1 + tx) * s1;
      const i64 step_r = kPwRows * s0, step_a = kTileX * s1;
      __syncthreads();  // the tile is free (previous operand gathered, previous tile stored)
#pragma unroll
      for (int a = 0; a < kTileXR; ++a)
#pragma unroll
        for (int r = 0; r < kTileYR; ++r) {
          u32 x = 0;
          if (INTERIOR || (t0 + ty + r * kPwRows < d.shape0 && t1 + tx + a * kTileX < d.shape1))
            x = load_elem<BYTE>(ptrs.p[T], base + r * step_r + a * step_a);
          smem[ty + r * kPwRows][tx + a * kTileX] = x;
        }
      __syncthreads();
#pragma unroll
      for (int a = 0; a < kTileXR; ++a)
#pragma unroll
        for (int r = 0; r < kTileYR; ++r) v[a * kTileYR + r][K] = smem[tx + a * kTileX][ty + r * kPwRows];
    } else {
      // tx runs along dimension 0: element (i0 = t0 + tx + 32a, i1 = t1 + ty + 8r)
      const i64 base = (t0 + tx) * s0 + (t1 + ty) * s1;
      const i64 step_a = kTileX * s0, step_r = kPwRows * s1;
#pragma unroll
      for (int a = 0; a < kTileXR; ++a)
#pragma unroll
        for (int r = 0; r < kTileYR; ++r) {
          u32 x = 0;
          if (INTERIOR || (t0 + tx + a * kTileX < d.shape0 && t1 + ty + r * kPwRows < d.shape1))
            x = load_elem<BYTE>(ptrs.p[T], base + a * step_a + r * step_r);
          v[a * kTileYR + r][K] = x;
        }
    }
    if constexpr (BYTE) {
#pragma unroll
      for (int e = 0; e < kTileElems; ++e) v[e][K] = v[e][K] != 0u ? 1u : 0u;
    }
    tile_load_inputs<F, INTERIOR, K + 1>(ptrs, d, t0, t1, smem, v);
  }
}
template <class F, bool INTERIOR, int K = 0>
__device__ __forceinline__ void tile_store_outputs(const PwPtrs<PwTraits<F>::NT>& ptrs, const TileDesc<PwTraits<F>::NT>& d,
                                                   i64 t0, i64 t1, PwTileSmem smem, const u32 (&v)[kTileElems][F::NOUT]) {
  if constexpr (K < F::NOUT) {
    constexpr bool BYTE = PwTraits<F>::out_byte(K);
    const int tx = threadIdx.x, ty = threadIdx.y;
    const i64 s0 = d.s0[K], s1 = d.s1[K];
    if ((d.dim1_mask >> K) & 1u) {
      const i64 base = (t0 + ty) * s0 + (t1 + tx) * s1;
      const i64 step_r = kPwRows * s0, step_a = kTileX * s1;
      __syncthreads();  // previous use of the tile is finished
#pragma unroll
      for (int a = 0; a < kTileXR; ++a)
#pragma unroll
        for (int r = 0; r < kTileYR; ++r) smem[tx + a * kTileX][ty + r * kPwRows] = v[a * kTileYR + r][K];
      __syncthreads();
#pragma unroll
      for (int a = 0; a < kTileXR; ++a)
#pragma unroll
        for (int r = 0; r < kTileYR; ++r)
          if (INTERIOR || (t0 + ty + r * kPwRows < d.shape0 && t1 + tx + a * kTileX < d.shape1))
            store_elem<BYTE>(ptrs.p[K], base + r * step_r + a * step_a, smem[ty + r * kPwRows][tx + a * kTileX]);
    } else {
      const i64 base = (t0 + tx) * s0 + (t1 + ty) * s1;
      const i64 step_a = kTileX * s0, step_r = kPwRows * s1;
#pragma unroll
      for (int a = 0; a < kTileXR; ++a)
#pragma unroll
        for (int r = 0; r < kTileYR; ++r)
          if (INTERIOR || (t0 + tx + a * kTileX < d.shape0 && t1 + ty + r * kPwRows < d.shape1))
            store_elem<BYTE>(ptrs.p[K], base + a * step_a + r * step_r, v[a * kTileYR + r][K]);
    }
    tile_store_outputs<F, INTERIOR, K + 1>(ptrs, d, t0, t1, smem, v);
  }
}

template <class F, bool INTERIOR>
__device__ __forceinline__ void pw_tile_one(const PwPtrs<PwTraits<F>::NT>& ptrs, const F& f,
                                            const TileDesc<PwTraits<F>::NT>& d, i64 t0, i64 t1, PwTileSmem smem) {
  constexpr int NS = F::NIN > 0 ? F::NIN : 1;
  u32 vin[kTileElems][NS], vout[kTileElems][F::NOUT];
  tile_load_inputs<F, INTERIOR>(ptrs, d, t0, t1, smem, vin);
#pragma unroll
  for (int e = 0; e < kTileElems; ++e) f(vin[e], vout[e]);
  tile_store_outputs<F, INTERIOR>(ptrs, d, t0, t1, smem, vout);
}

// Interior tile with 128-bit global accesses (TileDesc::vec).  The 256 threads are seen as 16x16:
// thread (vx, vy) holds elements (i0 = 4 vx + c, i1 = vy + 16 r), c, r = 0..3 - four float4 along
// dimension 0.  Operands dense along dimension 0 are loaded and stored in exactly that shape (a
// warp access is two 256-byte runs).  Operands dense along dimension 1 are accessed as float4
// along dimension 1 - thread (vx, vy) takes (i1 = 4 vx .. 4 vx + 3, i0 = vy + 16 r) - and turned
// through a 64x64 shared tile whose 16-byte chunks are XOR-swizzled with (i0 >> 2), which makes
// both the float4 row accesses and the scalar column accesses conflict-free without padding.
constexpr int kTileVecR = kTileElems / 4;  // float4 per thread and operand

// The float4 of operand t that thread (vx, vy) touches in pass r lies at base + r * step.
template <int NT>
__device__ __forceinline__ void tile_vec_address(const TileDesc<NT>& d, int t, i64 t0, i64 t1, int vx, int vy, i64& base,
                                                 i64& step) {
  if ((d.dim1_mask >> t) & 1u) {
    base = (t0 + vy) * d.s0[t] + (t1 + 4 * vx);
    step = kTileVecRows * d.s0[t];
  } else {
    base = (t0 + 4 * vx) + (t1 + vy) * d.s1[t];
    step = kTileVecRows * d.s1[t];
  }
}
// Raw float4 of an input tile -> the thread's 16 elements (through the shared tile if the operand
// is dense along dimension 1).
template <int NS>
__device__ __forceinline__ void tile_vec_unpack(const uint4 (&q)[kTileVecR], bool along1, int vx, int vy, u32* smem,
                                                u32 (&vin)[kTileElems][NS], int k) {
  if (along1) {
    __syncthreads();  // the tile is free (previous operand gathered, previous tile stored)
#pragma unroll
    for (int r = 0; r < kTileVecR; ++r) {
      const int i0 = vy + kTileVecRows * r;
      *reinterpret_cast<uint4*>(smem + i0 * kPwTile + ((vx ^ ((i0 >> 2) & 15)) << 2)) = q[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kTileVecR; ++r) {
      const int i1 = vy + kTileVecRows * r;
#pragma unroll
      for (int c = 0; c < 4; ++c)  // row i0 = 4 vx + c, whose swizzle key is vx
        vin[r * 4 + c][k] = smem[(4 * vx + c) * kPwTile + ((((i1 >> 2) ^ vx) & 15) << 2) + (i1 & 3)];
    }
  } else {
#pragma unroll
    for (int r = 0; r < kTileVecR; ++r) {
      vin[r * 4 + 0][k] = q[r].x; vin[r * 4 + 1][k] = q[r].y; vin[r * 4 + 2][k] = q[r].z; vin[r * 4 + 3][k] = q[r].w;
    }
  }
}
template <class F>
__device__ __forceinline__ void tile_vec_store(const PwPtrs<PwTraits<F>::NT>& ptrs, const TileDesc<PwTraits<F>::NT>& d,
                                               i64 t0, i64 t1, int vx, int vy, u32* smem,
                                               const u32 (&vout)[kTileElems][F::NOUT]) {
#pragma unroll
  for (int k = 0; k < F::NOUT; ++k) {
    u32* p = static_cast<u32*>(ptrs.p[k]);
    i64 base, step;
    tile_vec_address(d, k, t0, t1, vx, vy, base, step);
    if ((d.dim1_mask >> k) & 1u) {
      __syncthreads();  // previous use of the tile is finished
#pragma unroll
      for (int r = 0; r < kTileVecR; ++r) {
        const int i1 = vy + kTileVecRows * r;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          smem[(4 * vx + c) * kPwTile + ((((i1 >> 2) ^ vx) & 15) << 2) + (i1 & 3)] = vout[r * 4 + c][k];
      }
      __syncthreads();
#pragma unroll
      for (int r = 0; r < kTileVecR; ++r) {
        const int i0 = vy + kTileVecRows * r;
        const uint4 q = *reinterpret_cast<const uint4*>(smem + i0 * kPwTile + ((vx ^ ((i0 >> 2) & 15)) << 2));
        st_v4(p + base + r * step, q);
      }
    } else {
#pragma unroll
      for (int r = 0; r < kTileVecR; ++r)
        st_v4(p + base + r * step, make_uint4(vout[r * 4 + 0][k], vout[r * 4 + 1][k], vout[r * 4 + 2][k], vout[r * 4 + 3][k]));
    }
  }
}

template <class F>
__device__ __forceinline__ void pw_tile_one_vec(const PwPtrs<PwTraits<F>::NT>& ptrs, const F& f,
                                                const TileDesc<PwTraits<F>::NT>& d, i64 t0, i64 t1, u32* smem) {
  constexpr int NS = F::NIN > 0 ? F::NIN : 1;
  const int lin = threadIdx.y * kTileX + threadIdx.x;
  const int vx = lin & 15, vy = lin >> 4;
  u32 vin[kTileElems][NS], vout[kTileElems][F::NOUT];  // element r * 4 + c
#pragma unroll
  for (int k = 0; k < F::NIN; ++k) {
    const int t = F::NOUT + k;
    const u32* p = static_cast<const u32*>(ptrs.p[t]);
    i64 base, step;
    tile_vec_address(d, t, t0, t1, vx, vy, base, step);
    uint4 q[kTileVecR];
#pragma unroll
    for (int r = 0; r < kTileVecR; ++r) q[r] = ld_v4(p + base + r * step);
    tile_vec_unpack<NS>(q, (d.dim1_mask >> t) & 1u, vx, vy, smem, vin, k);
  }
#pragma unroll
  for (int e = 0; e < kTileElems; ++e) f(vin[e], vout[e]);
  tile_vec_store<F>(ptrs, d, t0, t1, vx, vy, smem, vout);
}

// Tile coordinates of a slot.  Tiles are walked in super-blocks of 8x8, so that the CTAs running
// side by side touch neighbouring pieces of the rows they share along dimension 0 and dimension 1
// alike.  Slots fit 32 bits (the planner refuses more), so the coordinates come from shifts and
// one multiply-shift division.  Returns 0 for a padding slot, 1 for a tile that lies wholly inside
// the tensor, 2 for an edge tile.
template <int NT>
__device__ __forceinline__ int tile_coords(const TileDesc<NT>& d, u32 slot, i64& t0, i64& t1) {
  static_assert(kTileSuper == 8, "the shifts below assume 8x8 super-blocks");
  const u32 sb = slot >> 6, within = slot & 63u;
  const u32 sb_hi = d.sb0_div.div(sb);
  const i64 b0 = (i64)(sb - sb_hi * d.sb0_div.d) * kTileSuper + (within & 7u);
  const i64 b1 = (i64)sb_hi * kTileSuper + (within >> 3);
  if (b0 >= d.tiles0 || b1 >= d.tiles1) return 0;
  t0 = b0 * kPwTile;
  t1 = b1 * kPwTile;
  return (t0 + kPwTile <= d.shape0 && t1 + kPwTile <= d.shape1) ? 1 : 2;
}

// One-input functors on 128-bit-capable layouts: a CTA walks several tiles and issues the global
// loads of its next tile before it computes and stores the current one, so a tile's worth of
// loads is in flight per CTA at all times - also while the transcendental functors (silu, gelu)
// keep the warps busy.  Launched with kTilePersistCtas CTAs per SM.
template <class F>
__device__ __forceinline__ void pw_tile_pipelined(const PwPtrs<PwTraits<F>::NT>& ptrs, const F& f,
                                                  const TileDesc<PwTraits<F>::NT>& d, PwTileSmem smem2d) {
  static_assert(F::NIN == 1, "one input");
  constexpr int T = F::NOUT;  // operand index of the input
  u32* smem = &smem2d[0][0];
  const int lin = threadIdx.y * kTileX + threadIdx.x;
  const int vx = lin & 15, vy = lin >> 4;
  const u32* p = static_cast<const u32*>(ptrs.p[T]);
  const bool along1 = (d.dim1_mask >> T) & 1u;
  const u32 nslots = (u32)d.ntiles;
  uint4 q[kTileVecR];
  auto prefetch = [&](i64 t0, i64 t1) {
    i64 base, step;
    tile_vec_address(d, T, t0, t1, vx, vy, base, step);
#pragma unroll
    for (int r = 0; r < kTileVecR; ++r) q[r] = ld_v4(p + base + r * step);
  };
  u32 slot = blockIdx.x;
  i64 t0 = 0, t1 = 0;
  int kind = slot < nslots ? tile_coords(d, slot, t0, t1) : 0;
  if (kind == 1) prefetch(t0, t1);
  while (slot < nslots) {
    const u32 nslot = slot + gridDim.x;
    i64 n0 = 0, n1 = 0;
    const int nkind = nslot < nslots ? tile_coords(d, nslot, n0, n1) : 0;
    if (kind == 1) {
      u32 vin[kTileElems][1], vout[kTileElems][F::NOUT];
      tile_vec_unpack<1>(q, along1, vx, vy, smem, vin, 0);
      if (nkind == 1) prefetch(n0, n1);  // in flight while this tile is computed and stored
#pragma unroll
      for (int e = 0; e < kTileElems; ++e) f(vin[e], vout[e]);
      tile_vec_store<F>(ptrs, d, t0, t1, vx, vy, smem, vout);
    } else {
      if (kind == 2) pw_tile_one<F, false>(ptrs, f, d, t0, t1, smem2d);
      if (nkind == 1) prefetch(n0, n1);
    }
    slot = nslot;
    kind = nkind;
    t0 = n0;
    t1 = n1;
  }
}

// Functors that cost tens of instructions per element (silu, gelu) say so with
// `static constexpr bool kHeavy = true`; the tile kernel then prefetches the next tile's loads into
// registers (pw_tile_pipelined).  Measured on a 16384^2 transpose, fractions of the copy peak for
// relu / silu / gelu(erf): one tile per CTA, 5 CTAs per SM 0.97 / 0.88 / 0.80; register prefetch,
// 4 persistent CTAs per SM 0.91 / 0.90 / 0.86; a three-stage cp.async ring in shared memory
// 0.86 / 0.78 / 0.85 (dropped).  Cheap functors want CTAs, expensive ones want the loads of the next
// tile in flight while the arithmetic runs.
template <class F, class = void>
struct PwHeavy {
  static constexpr bool value = false;
};
template <class F>
struct PwHeavy<F, decltype((void)F::kHeavy)> {
  static constexpr bool value = F::kHeavy;
};
template <class F>
struct TilePipelined {
  static constexpr bool value = F::NIN == 1 && F::kInByteMask == 0u && F::kOutByteMask == 0u && PwHeavy<F>::value;
};

template <class F>
__device__ __forceinline__ void pw_tile_body(const PwPtrs<PwTraits<F>::NT>& ptrs, const F& f,
                                             const TileDesc<PwTraits<F>::NT>& d) {
  __shared__ __align__(16) u32 smem[kPwTile][kPwTile + 1];
  if constexpr (TilePipelined<F>::value) {
    if (d.vec) {
      pw_tile_pipelined<F>(ptrs, f, d, smem);
      return;
    }
  }
  const u32 nslots = (u32)d.ntiles;
  for (u32 slot = blockIdx.x; slot < nslots; slot += gridDim.x) {
    i64 t0, t1;
    const int kind = tile_coords(d, slot, t0, t1);
    if (kind == 0) continue;
    if (kind == 1) {
      if constexpr (F::kInByteMask == 0u && F::kOutByteMask == 0u) {
        if (d.vec) {
          pw_tile_one_vec<F>(ptrs, f, d, t0, t1, &smem[0][0]);
          continue;
        }
      }
      pw_tile_one<F, true>(ptrs, f, d, t0, t1, smem);
    } else {
      pw_tile_one<F, false>(ptrs, f, d, t0, t1, smem);
    }
  }
}

// __global__ wrappers (templates for ahead-of-time instantiation)
template <class F, int U>
__global__ void __launch_bounds__(kBlock) pw_contig_kernel(PwPtrs<PwTraits<F>::NT> ptrs, F f, i64 nunits, i64 n) {
  pw_contig_body<F, U>(ptrs, f, nunits, n);
}
template <class F, int U, class IDX>
__global__ void __launch_bounds__(kBlock)
    pw_strided_kernel(PwPtrs<PwTraits<F>::NT> ptrs, F f, StridedDesc<PwTraits<F>::NT, IDX> d, i64 n) {
  pw_strided_body<F, U, IDX>(ptrs, f, d, n);
}
// CTAs per SM the tile kernels are compiled for: the pipelined kernel keeps a second tile in
// registers (64 registers, 4 CTAs); one-input kernels otherwise fit 48 registers (5 CTAs),
// two-input ones get 64 and larger ones 80 (3 CTAs), which keeps all of them clear of spills.
template <class F>
__host__ __device__ constexpr int tile_min_ctas() {
  return TilePipelined<F>::value ? kTilePersistCtas : (F::NIN <= 1 ? 5 : (F::NIN == 2 ? 4 : 3));
}

template <class F>
__global__ void __launch_bounds__(kTileX* kPwRows, tile_min_ctas<F>())
    pw_tile_kernel(PwPtrs<PwTraits<F>::NT> ptrs, F f, TileDesc<PwTraits<F>::NT> d) {
  pw_tile_body<F>(ptrs, f, d);
}

}  // namespace twg
