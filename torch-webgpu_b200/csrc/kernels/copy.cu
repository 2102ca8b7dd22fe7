// Element-size-generic kernels: strided/broadcast device copy (any dtype is just 1/2/4/8/16
// bytes per element here) and the integer bitwise-and, which is the same byte-wise operation
// for every integer width.  They share the index math of the pointwise kernels but move raw
// bytes, so nothing is normalised or reinterpreted.
#include <cstring>

#include "twg_launch.cuh"

namespace twg {

int and_bool(const TwgIterDesc* d, const void* a, const void* b, void* out, cudaStream_t s);

template <class T>
__device__ __forceinline__ T bits_and(T a, T b) { return a & b; }
template <>
__device__ __forceinline__ uint4 bits_and<uint4>(uint4 a, uint4 b) {
  return make_uint4(a.x & b.x, a.y & b.y, a.z & b.z, a.w & b.w);
}

// NIN == 1: out = a.  NIN == 2: out = a & b.
template <class T, int NIN, class IDX>
__global__ void __launch_bounds__(kBlock)
    sized_strided_kernel(T* out, const T* a, const T* b, StridedDesc<NIN + 1, IDX> d, i64 n) {
  constexpr int U = kStridedUnroll;
  const i64 step = (i64)gridDim.x * kBlock * U;
  for (i64 base = (i64)blockIdx.x * kBlock * U + threadIdx.x; base < n; base += step) {
    i64 off[U][NIN + 1];
    T va[U], vb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const i64 e = base + (i64)u * kBlock;
      if (e < n) {
        linear_to_offsets<NIN + 1>(d, (IDX)e, off[u]);
        va[u] = a[off[u][1]];
        if constexpr (NIN == 2) vb[u] = b[off[u][2]];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const i64 e = base + (i64)u * kBlock;
      if (e < n) {
        if constexpr (NIN == 2) out[off[u][0]] = bits_and(va[u], vb[u]);
        else out[off[u][0]] = va[u];
      }
    }
  }
}

// 2-D permuted copy / and through a padded shared-memory tile (see pw_tile_body).
template <class T, int NIN>
__global__ void __launch_bounds__(kTile* kTileRows)
    sized_tile_kernel(T* out, const T* a, const T* b, TileDesc<NIN + 1> d) {
  constexpr int R = kTile / kTileRows;
  __shared__ T smem[NIN][kTile][kTile + 1];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const T* in[2] = {a, b};
  for (i64 tile = blockIdx.x; tile < d.ntiles; tile += gridDim.x) {
    const i64 t0 = (tile % d.tiles0) * kTile, t1 = (tile / d.tiles0) * kTile;
    T v[R][NIN];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < NIN; ++k) {
      const int t = 1 + k;
      if ((d.dim1_mask >> t) & 1u) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const i64 i0 = t0 + ty + r * kTileRows, i1 = t1 + tx;
          if (i0 < d.shape0 && i1 < d.shape1) smem[k][ty + r * kTileRows][tx] = in[k][i0 * d.s0[t] + i1 * d.s1[t]];
        }
      } else {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const i64 i0 = t0 + tx, i1 = t1 + ty + r * kTileRows;
          if (i0 < d.shape0 && i1 < d.shape1) v[r][k] = in[k][i0 * d.s0[t] + i1 * d.s1[t]];
        }
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < NIN; ++k)
      if ((d.dim1_mask >> (1 + k)) & 1u) {
#pragma unroll
        for (int r = 0; r < R; ++r) v[r][k] = smem[k][tx][ty + r * kTileRows];
      }
    T y[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if constexpr (NIN == 2) y[r] = bits_and(v[r][0], v[r][1]);
      else y[r] = v[r][0];
    }
    if (d.dim1_mask & 1u) {
      __syncthreads();
#pragma unroll
      for (int r = 0; r < R; ++r) smem[0][tx][ty + r * kTileRows] = y[r];
      __syncthreads();
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const i64 i0 = t0 + ty + r * kTileRows, i1 = t1 + tx;
        if (i0 < d.shape0 && i1 < d.shape1) out[i0 * d.s0[0] + i1 * d.s1[0]] = smem[0][ty + r * kTileRows][tx];
      }
    } else {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const i64 i0 = t0 + tx, i1 = t1 + ty + r * kTileRows;
        if (i0 < d.shape0 && i1 < d.shape1) out[i0 * d.s0[0] + i1 * d.s1[0]] = y[r];
      }
    }
  }
}

// Dense and over raw bytes: 128-bit words plus a byte tail.
__global__ void __launch_bounds__(kBlock)
    and_dense_kernel(uint4* out, const uint4* a, const uint4* b, i64 nvec, i64 nbytes) {
  constexpr int U = kDenseUnrollBytes;
  const i64 chunk = (i64)kBlock * U;
  const i64 nchunks = (nvec + chunk - 1) / chunk;
  for (i64 c = blockIdx.x; c < nchunks; c += gridDim.x) {
    const i64 u0 = c * chunk + threadIdx.x;
    uint4 va[U], vb[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (u0 + (i64)u * kBlock < nvec) { va[u] = ld_v4(a + u0 + (i64)u * kBlock); vb[u] = ld_v4(b + u0 + (i64)u * kBlock); }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (u0 + (i64)u * kBlock < nvec) st_v4(out + u0 + (i64)u * kBlock, bits_and(va[u], vb[u]));
  }
  const i64 tail0 = nvec * 16;
  if (blockIdx.x == 0 && tail0 + threadIdx.x < nbytes) {
    const u8* pa = reinterpret_cast<const u8*>(a);
    const u8* pb = reinterpret_cast<const u8*>(b);
    reinterpret_cast<u8*>(out)[tail0 + threadIdx.x] = pa[tail0 + threadIdx.x] & pb[tail0 + threadIdx.x];
  }
}

template <class T, int NIN>
int launch_sized(const TwgIterDesc& d, const void* a, const void* b, void* out, cudaStream_t stream) {
  constexpr int NT = NIN + 1;
  T* po = static_cast<T*>(out);
  const T* pa = static_cast<const T*>(a);
  const T* pb = static_cast<const T*>(b);
  PwPlan plan;
  plan.d = d;
  if (plan_tile(d, NT, kTile, &plan)) {
    TileDesc<NT> td;
    fill_tile_desc<NT>(plan, &td);
    sized_tile_kernel<T, NIN><<<plan.grid, dim3(kTile, kTileRows), 0, stream>>>(po, pa, pb, td);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathTile;
    return TWG_OK;
  }
  const int64_t per_cta = (int64_t)kBlock * kStridedUnroll;
  const unsigned grid = (unsigned)std::min<int64_t>((d.numel + per_cta - 1) / per_cta, 0x7fffffff);
  if (fits_32bit(d, NT)) {
    StridedDesc<NT, u32> sd;
    fill_strided_desc<NT>(d, &sd);
    sized_strided_kernel<T, NIN, u32><<<grid, kBlock, 0, stream>>>(po, pa, pb, sd, d.numel);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathStrided32;
  } else {
    StridedDesc<NT, u64> sd;
    fill_strided_desc<NT>(d, &sd);
    sized_strided_kernel<T, NIN, u64><<<grid, kBlock, 0, stream>>>(po, pa, pb, sd, d.numel);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathStrided64;
  }
  return TWG_OK;
}

template <int NIN>
int dispatch_sized(const TwgIterDesc& d, int itemsize, const void* a, const void* b, void* out, cudaStream_t s) {
  switch (itemsize) {
    case 1: return launch_sized<uint8_t, NIN>(d, a, b, out, s);
    case 2: return launch_sized<uint16_t, NIN>(d, a, b, out, s);
    case 4: return launch_sized<uint32_t, NIN>(d, a, b, out, s);
    case 8: return launch_sized<unsigned long long, NIN>(d, a, b, out, s);
    case 16: return launch_sized<uint4, NIN>(d, a, b, out, s);
    default: return set_error(TWG_ERR_UNSUPPORTED, "element size %d is not 1, 2, 4, 8 or 16 bytes", itemsize);
  }
}

// fill: every element of `out` becomes the low `sizeof(T)` bytes of `pattern`.  Dense outputs are
// written as 16-byte vectors between the first and last 16-byte boundary; anything else walks the
// descriptor.
template <class T>
__global__ void __launch_bounds__(kBlock) fill_dense_kernel(T* out, T value, uint4 vec, i64 n) {
  const unsigned long long addr = reinterpret_cast<unsigned long long>(out);
  const i64 per = 16 / (i64)sizeof(T);
  i64 head = (i64)(((16ull - (addr & 15ull)) & 15ull) / sizeof(T));
  if (head > n) head = n;
  const i64 nvec = (n - head) / per;
  uint4* out4 = reinterpret_cast<uint4*>(out + head);
  const i64 step = (i64)gridDim.x * kBlock;
  for (i64 i = (i64)blockIdx.x * kBlock + threadIdx.x; i < nvec; i += step) st_v4(out4 + i, vec);
  if (blockIdx.x == 0) {
    if ((i64)threadIdx.x < head) out[threadIdx.x] = value;
    const i64 tail0 = head + nvec * per;
    if (tail0 + (i64)threadIdx.x < n) out[tail0 + threadIdx.x] = value;
  }
}
template <class T, class IDX>
__global__ void __launch_bounds__(kBlock) fill_strided_kernel(T* out, T value, StridedDesc<1, IDX> d, i64 n) {
  const i64 step = (i64)gridDim.x * kBlock;
  for (i64 e = (i64)blockIdx.x * kBlock + threadIdx.x; e < n; e += step) {
    i64 off[1];
    linear_to_offsets<1>(d, (IDX)e, off);
    out[off[0]] = value;
  }
}
template <class T>
int launch_fill(const TwgIterDesc& d, unsigned long long pattern, void* out, cudaStream_t s) {
  T value;
  std::memcpy(&value, &pattern, sizeof(T));
  const int64_t n = d.numel;
  if (all_dense(d, 1)) {
    unsigned long long two[2];
    unsigned char* bytes = reinterpret_cast<unsigned char*>(two);
    for (size_t i = 0; i < 16; i += sizeof(T)) std::memcpy(bytes + i, &value, sizeof(T));
    uint4 vec;
    std::memcpy(&vec, two, 16);
    const int64_t nvec = n / (16 / (int64_t)sizeof(T)) + 1;
    const unsigned grid = (unsigned)std::min<int64_t>((nvec + kBlock - 1) / kBlock, (int64_t)sm_count() * 16);
    fill_dense_kernel<T><<<grid, kBlock, 0, s>>>(static_cast<T*>(out), value, vec, n);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathDense;
    return TWG_OK;
  }
  const unsigned grid = (unsigned)std::min<int64_t>((n + kBlock - 1) / kBlock, (int64_t)sm_count() * 32);
  if (fits_32bit(d, 1)) {
    StridedDesc<1, u32> sd;
    fill_strided_desc<1>(d, &sd);
    fill_strided_kernel<T, u32><<<grid, kBlock, 0, s>>>(static_cast<T*>(out), value, sd, n);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathStrided32;
  } else {
    StridedDesc<1, u64> sd;
    fill_strided_desc<1>(d, &sd);
    fill_strided_kernel<T, u64><<<grid, kBlock, 0, s>>>(static_cast<T*>(out), value, sd, n);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathStrided64;
  }
  return TWG_OK;
}

bool all_dense(const TwgIterDesc& d, int nt) {
  if (d.ndim > 1) return false;
  if (d.ndim == 1 && d.numel > 1)
    for (int t = 0; t < nt; ++t)
      if (d.strides[t][0] != 1) return false;
  return true;
}

}  // namespace twg

using namespace twg;

extern "C" int twg_copy_strided(const TwgIterDesc* desc, int itemsize, const void* in, void* out, void* stream) {
  TWG_TRACE("twg_copy_strided");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  g_last_path = kPathNone;
  if (int rc = check_desc(desc, 2)) return rc;
  if (desc->numel == 0) return TWG_OK;
  TWG_REQUIRE(in && out, "twg_copy_strided: null operand");
  TwgIterDesc d = *desc;
  d.ntensors = 2;
  if (int rc = twg_iter_coalesce(&d)) return rc;
  if (all_dense(d, 2)) {
    TWG_CUDA(cudaMemcpyAsync(out, in, (size_t)d.numel * (size_t)itemsize, cudaMemcpyDeviceToDevice, s));
    g_last_path = kPathDense;
    return TWG_OK;
  }
  TWG_REQUIRE(is_aligned(in, (size_t)itemsize) && is_aligned(out, (size_t)itemsize),
              "twg_copy_strided: operands are not aligned to the element size %d", itemsize);
  // 4-byte elements move through the f32 functor kernels (a bit-exact 32-bit copy) and get their
  // larger tiles; the other widths use the generic kernels of this file
  if (itemsize == 4)
    return twg_unary_f32(TWG_UNARY_COPY, desc, static_cast<const float*>(in), static_cast<float*>(out), stream);
  return dispatch_sized<1>(d, itemsize, in, nullptr, out, s);
}

extern "C" int twg_fill(const TwgIterDesc* desc, int itemsize, uint64_t pattern, void* out, void* stream) {
  TWG_TRACE("twg_fill");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  g_last_path = kPathNone;
  if (int rc = check_desc(desc, 1)) return rc;
  if (desc->numel == 0) return TWG_OK;
  TWG_REQUIRE(out != nullptr, "twg_fill: null operand");
  TWG_REQUIRE(itemsize == 1 || itemsize == 2 || itemsize == 4 || itemsize == 8,
              "twg_fill: element size %d is not 1, 2, 4 or 8 bytes", itemsize);
  TWG_REQUIRE(is_aligned(out, (size_t)itemsize), "twg_fill: the operand is not aligned to the element size %d", itemsize);
  TwgIterDesc d = *desc;
  d.ntensors = 1;
  if (int rc = twg_iter_coalesce(&d)) return rc;
  switch (itemsize) {
    case 1: return launch_fill<uint8_t>(d, pattern, out, s);
    case 2: return launch_fill<uint16_t>(d, pattern, out, s);
    case 4: return launch_fill<uint32_t>(d, pattern, out, s);
    default: return launch_fill<unsigned long long>(d, pattern, out, s);
  }
}

extern "C" int twg_bitwise_and(const TwgIterDesc* desc, int itemsize, int is_bool, const void* a, const void* b,
                               void* out, void* stream) {
  TWG_TRACE("twg_bitwise_and");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_bool) {
    TWG_REQUIRE(itemsize == 1, "twg_bitwise_and: bool operands are 1 byte, got itemsize %d", itemsize);
    return and_bool(desc, a, b, out, s);
  }
  g_last_path = kPathNone;
  if (int rc = check_desc(desc, 3)) return rc;
  if (desc->numel == 0) return TWG_OK;
  TWG_REQUIRE(a && b && out, "twg_bitwise_and: null operand");
  TwgIterDesc d = *desc;
  d.ntensors = 3;
  if (int rc = twg_iter_coalesce(&d)) return rc;
  if (all_dense(d, 3) && is_aligned(a, 16) && is_aligned(b, 16) && is_aligned(out, 16)) {
    const int64_t nbytes = d.numel * itemsize, nvec = nbytes / 16;
    const int64_t chunk = (int64_t)kBlock * kDenseUnrollBytes;
    const int64_t grid = std::min<int64_t>(std::max<int64_t>(1, (nvec + chunk - 1) / chunk), 0x7fffffff);
    and_dense_kernel<<<(unsigned)grid, kBlock, 0, s>>>(static_cast<uint4*>(out), static_cast<const uint4*>(a),
                                                        static_cast<const uint4*>(b), nvec, nbytes);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathDense;
    return TWG_OK;
  }
  TWG_REQUIRE(is_aligned(a, (size_t)itemsize) && is_aligned(b, (size_t)itemsize) && is_aligned(out, (size_t)itemsize),
              "twg_bitwise_and: operands are not aligned to the element size %d", itemsize);
  return dispatch_sized<2>(d, itemsize, a, b, out, s);
}
