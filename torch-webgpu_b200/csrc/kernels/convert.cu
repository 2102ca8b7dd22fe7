// Element-type conversion on the device: out[i] = (Dst)in[i] for any pair of the ten element
// types the copy path moves.  The reference converts nothing (its copies assert float32,
// csrc/ops/copy.cpp:22); this is what copy_ between two device tensors of different dtypes runs
// instead of a round trip through host memory.
//
// Dense, suitably aligned operands take four elements per thread as one load and one store (4 to
// 32 bytes wide depending on the types); everything else takes the strided index path with 64-bit
// offsets.  Conversions follow C++ static_cast, which is what ATen's CPU copy kernel does: floats
// to integers truncate toward zero, anything to bool is "!= 0", float32 to float16 / bfloat16
// rounds to nearest even.  Float values outside the integer target's range are undefined there
// and saturate here.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <type_traits>

#include "twg_launch.cuh"

namespace twg {

struct BoolByte {
  uint8_t v;
};

template <class T>
struct CvtTraits {
  static constexpr bool is_float = false;
};
template <>
struct CvtTraits<__half> {
  static constexpr bool is_float = true;
};
template <>
struct CvtTraits<__nv_bfloat16> {
  static constexpr bool is_float = true;
};
template <>
struct CvtTraits<float> {
  static constexpr bool is_float = true;
};
template <>
struct CvtTraits<double> {
  static constexpr bool is_float = true;
};

// Source value as the widest type that holds it exactly: double for floats, 64-bit integer else.
template <class S>
__device__ __forceinline__ auto widen(S v) {
  if constexpr (std::is_same<S, __half>::value) return (double)__half2float(v);
  else if constexpr (std::is_same<S, __nv_bfloat16>::value) return (double)__bfloat162float(v);
  else if constexpr (std::is_same<S, float>::value || std::is_same<S, double>::value) return (double)v;
  else if constexpr (std::is_same<S, BoolByte>::value) return (long long)(v.v != 0);
  else return (long long)v;
}

template <class S, class D>
__device__ __forceinline__ D convert_one(S v) {
  if constexpr (std::is_same<S, D>::value) {
    return v;
  } else if constexpr (std::is_same<D, BoolByte>::value) {
    return BoolByte{(uint8_t)(widen(v) != 0)};
  } else if constexpr (std::is_same<D, __half>::value) {
    // float32 is the stepping stone for every source: exact for all sources but float64 and
    // 64-bit integers, whose double rounding is what a static_cast chain on the host does too
    return __float2half_rn((float)widen(v));
  } else if constexpr (std::is_same<D, __nv_bfloat16>::value) {
    return __float2bfloat16_rn((float)widen(v));
  } else if constexpr (std::is_same<D, float>::value || std::is_same<D, double>::value) {
    return (D)widen(v);
  } else {  // integer target
    if constexpr (CvtTraits<S>::is_float) return (D)(long long)widen(v);  // truncation toward zero
    else return (D)widen(v);                                              // wraps like a C cast
  }
}

template <class T>
struct alignas(sizeof(T) * 4 > 16 ? 16 : sizeof(T) * 4) Pack4 {
  T v[4];
};

constexpr int kCvtBlock = 256;

template <class S, class D>
__global__ void __launch_bounds__(kCvtBlock) convert_dense_kernel(const S* in, D* out, i64 n) {
  const i64 npacks = n >> 2;
  const i64 step = (i64)gridDim.x * kCvtBlock;
  for (i64 p = (i64)blockIdx.x * kCvtBlock + threadIdx.x; p < npacks; p += step) {
    const Pack4<S> x = reinterpret_cast<const Pack4<S>*>(in)[p];
    Pack4<D> y;
#pragma unroll
    for (int k = 0; k < 4; ++k) y.v[k] = convert_one<S, D>(x.v[k]);
    reinterpret_cast<Pack4<D>*>(out)[p] = y;
  }
  const i64 tail = (npacks << 2) + (i64)blockIdx.x * kCvtBlock + threadIdx.x;
  if (tail < n) out[tail] = convert_one<S, D>(in[tail]);
}

template <class S, class D>
__global__ void __launch_bounds__(kCvtBlock) convert_strided_kernel(const S* in, D* out, StridedDesc<2, u64> d, i64 n) {
  const i64 step = (i64)gridDim.x * kCvtBlock;
  for (i64 e = (i64)blockIdx.x * kCvtBlock + threadIdx.x; e < n; e += step) {
    i64 off[2];
    linear_to_offsets<2>(d, (u64)e, off);
    out[off[0]] = convert_one<S, D>(in[off[1]]);
  }
}

template <class S, class D>
static int run_convert(const TwgIterDesc& d, const void* in, void* out, cudaStream_t s) {
  const S* src = static_cast<const S*>(in);
  D* dst = static_cast<D*>(out);
  const i64 n = d.numel;
  const i64 max_grid = (i64)sm_count() * 16;
  if (all_dense(d, 2) && is_aligned(in, alignof(Pack4<S>)) && is_aligned(out, alignof(Pack4<D>))) {
    const i64 grid = std::max<i64>(1, std::min<i64>(max_grid, ((n >> 2) + kCvtBlock - 1) / kCvtBlock));
    convert_dense_kernel<S, D><<<(unsigned)grid, kCvtBlock, 0, s>>>(src, dst, n);
    TWG_CHECK_LAUNCH();
    g_last_path = kPathDense;
    return TWG_OK;
  }
  StridedDesc<2, u64> sd;
  fill_strided_desc<2>(d, &sd);
  const i64 grid = std::max<i64>(1, std::min<i64>(max_grid, (n + kCvtBlock - 1) / kCvtBlock));
  convert_strided_kernel<S, D><<<(unsigned)grid, kCvtBlock, 0, s>>>(src, dst, sd, n);
  TWG_CHECK_LAUNCH();
  g_last_path = kPathStrided64;
  return TWG_OK;
}

template <class S>
static int run_convert_from(int dst_dtype, const TwgIterDesc& d, const void* in, void* out, cudaStream_t s) {
  switch (dst_dtype) {
    case TWG_DTYPE_U8: return run_convert<S, uint8_t>(d, in, out, s);
    case TWG_DTYPE_I8: return run_convert<S, int8_t>(d, in, out, s);
    case TWG_DTYPE_I16: return run_convert<S, int16_t>(d, in, out, s);
    case TWG_DTYPE_I32: return run_convert<S, int32_t>(d, in, out, s);
    case TWG_DTYPE_I64: return run_convert<S, long long>(d, in, out, s);
    case TWG_DTYPE_F16: return run_convert<S, __half>(d, in, out, s);
    case TWG_DTYPE_BF16: return run_convert<S, __nv_bfloat16>(d, in, out, s);
    case TWG_DTYPE_F32: return run_convert<S, float>(d, in, out, s);
    case TWG_DTYPE_F64: return run_convert<S, double>(d, in, out, s);
    case TWG_DTYPE_BOOL: return run_convert<S, BoolByte>(d, in, out, s);
    default: return set_error(TWG_ERR_INVALID, "twg_convert: unknown destination dtype %d", dst_dtype);
  }
}

static int dtype_size(int dtype) {
  switch (dtype) {
    case TWG_DTYPE_U8: case TWG_DTYPE_I8: case TWG_DTYPE_BOOL: return 1;
    case TWG_DTYPE_I16: case TWG_DTYPE_F16: case TWG_DTYPE_BF16: return 2;
    case TWG_DTYPE_I32: case TWG_DTYPE_F32: return 4;
    case TWG_DTYPE_I64: case TWG_DTYPE_F64: return 8;
    default: return 0;
  }
}

}  // namespace twg

using namespace twg;

extern "C" int twg_convert(const TwgIterDesc* desc, int src_dtype, int dst_dtype, const void* in, void* out, void* stream) {
  TWG_TRACE("twg_convert");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  g_last_path = kPathNone;
  if (int rc = check_desc(desc, 2)) return rc;
  const int ssz = dtype_size(src_dtype), dsz = dtype_size(dst_dtype);
  TWG_REQUIRE(ssz != 0 && dsz != 0, "twg_convert: unknown dtype %d -> %d", src_dtype, dst_dtype);
  if (desc->numel == 0) return TWG_OK;
  TWG_REQUIRE(in && out, "twg_convert: null operand");
  TWG_REQUIRE(is_aligned(in, (size_t)ssz) && is_aligned(out, (size_t)dsz),
              "twg_convert: operands are not aligned to their element sizes (%d, %d)", ssz, dsz);
  TwgIterDesc d = *desc;
  d.ntensors = 2;
  if (int rc = twg_iter_coalesce(&d)) return rc;
  switch (src_dtype) {
    case TWG_DTYPE_U8: return run_convert_from<uint8_t>(dst_dtype, d, in, out, s);
    case TWG_DTYPE_I8: return run_convert_from<int8_t>(dst_dtype, d, in, out, s);
    case TWG_DTYPE_I16: return run_convert_from<int16_t>(dst_dtype, d, in, out, s);
    case TWG_DTYPE_I32: return run_convert_from<int32_t>(dst_dtype, d, in, out, s);
    case TWG_DTYPE_I64: return run_convert_from<long long>(dst_dtype, d, in, out, s);
    case TWG_DTYPE_F16: return run_convert_from<__half>(dst_dtype, d, in, out, s);
    case TWG_DTYPE_BF16: return run_convert_from<__nv_bfloat16>(dst_dtype, d, in, out, s);
    case TWG_DTYPE_F32: return run_convert_from<float>(dst_dtype, d, in, out, s);
    case TWG_DTYPE_F64: return run_convert_from<double>(dst_dtype, d, in, out, s);
    default: return run_convert_from<BoolByte>(dst_dtype, d, in, out, s);
  }
}
