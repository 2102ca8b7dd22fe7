// C-ABI entry points of the single-op pointwise kernels: unary f32, binary f32, f32 comparisons
// producing bool bytes, and bool logical-and.  Each one is the launcher template of
// twg_launch.cuh instantiated with a small functor.
#include "twg_launch.cuh"

namespace twg {

template <int OP>
struct UnaryF32 {
  static constexpr int NIN = 1, NOUT = 1;
  static constexpr unsigned kInByteMask = 0u, kOutByteMask = 0u;
  // the transcendental activations cost tens of instructions per element
  static constexpr bool kHeavy = OP == TWG_UNARY_GELU_TANH || OP == TWG_UNARY_SILU || OP == TWG_UNARY_GELU_ERF;
  __device__ __forceinline__ void operator()(const u32* in, u32* out) const {
    const float x = as_f(in[0]);
    float y;
    if constexpr (OP == TWG_UNARY_COPY) y = x;
    else if constexpr (OP == TWG_UNARY_RELU) y = f_relu(x);
    else if constexpr (OP == TWG_UNARY_GELU_TANH) y = f_gelu_tanh(x);
    else if constexpr (OP == TWG_UNARY_SILU) y = f_silu(x);
    else if constexpr (OP == TWG_UNARY_GELU_ERF) y = f_gelu_erf(x);
    else y = f_abs(x);
    out[0] = as_u(y);
  }
};

template <int OP>
struct BinaryF32 {
  static constexpr int NIN = 2, NOUT = 1;
  static constexpr unsigned kInByteMask = 0u, kOutByteMask = 0u;
  float alpha;
  __device__ __forceinline__ void operator()(const u32* in, u32* out) const {
    const float a = as_f(in[0]), b = as_f(in[1]);
    float y;
    if constexpr (OP == TWG_BINARY_ADD) y = f_add(a, b, alpha);
    else if constexpr (OP == TWG_BINARY_MUL) y = f_mul(a, b);
    else if constexpr (OP == TWG_BINARY_DIV) y = f_div(a, b);
    else y = f_relu(f_add(a, b, 1.0f));
    out[0] = as_u(y);
  }
};

// The same ops with a scalar right operand (x + 2, x * 0.5, x / 3): one stream in, one out.
template <int OP>
struct BinaryScalarF32 {
  static constexpr int NIN = 1, NOUT = 1;
  static constexpr unsigned kInByteMask = 0u, kOutByteMask = 0u;
  float scalar, alpha;
  __device__ __forceinline__ void operator()(const u32* in, u32* out) const {
    const float a = as_f(in[0]);
    float y;
    if constexpr (OP == TWG_BINARY_ADD) y = f_add(a, scalar, alpha);
    else if constexpr (OP == TWG_BINARY_MUL) y = f_mul(a, scalar);
    else if constexpr (OP == TWG_BINARY_DIV) y = f_div(a, scalar);
    else y = f_relu(f_add(a, scalar, 1.0f));
    out[0] = as_u(y);
  }
};

template <int OP>
__device__ __forceinline__ u32 compare(float a, float b) {
  if constexpr (OP == TWG_CMP_EQ) return f_eq(a, b);
  else if constexpr (OP == TWG_CMP_NE) return f_ne(a, b);
  else if constexpr (OP == TWG_CMP_LT) return f_lt(a, b);
  else if constexpr (OP == TWG_CMP_LE) return f_le(a, b);
  else if constexpr (OP == TWG_CMP_GT) return f_gt(a, b);
  else return f_ge(a, b);
}
template <int OP>
struct CompareTensorF32 {
  static constexpr int NIN = 2, NOUT = 1;
  static constexpr unsigned kInByteMask = 0u, kOutByteMask = 1u;
  __device__ __forceinline__ void operator()(const u32* in, u32* out) const {
    out[0] = compare<OP>(as_f(in[0]), as_f(in[1]));
  }
};
template <int OP>
struct CompareScalarF32 {
  static constexpr int NIN = 1, NOUT = 1;
  static constexpr unsigned kInByteMask = 0u, kOutByteMask = 1u;
  float scalar;
  __device__ __forceinline__ void operator()(const u32* in, u32* out) const {
    out[0] = compare<OP>(as_f(in[0]), scalar);
  }
};

// out = cond ? a : b with a bool-byte condition (any non-zero byte counts as true, like ATen).
struct WhereF32 {
  static constexpr int NIN = 3, NOUT = 1;
  static constexpr unsigned kInByteMask = 1u, kOutByteMask = 0u;
  __device__ __forceinline__ void operator()(const u32* in, u32* out) const { out[0] = in[0] != 0u ? in[1] : in[2]; }
};
// out = mask ? value : self.
struct MaskedFillF32 {
  static constexpr int NIN = 2, NOUT = 1;
  static constexpr unsigned kInByteMask = 2u, kOutByteMask = 0u;
  float value;
  __device__ __forceinline__ void operator()(const u32* in, u32* out) const { out[0] = in[1] != 0u ? as_u(value) : in[0]; }
};

struct AndBool {
  static constexpr int NIN = 2, NOUT = 1;
  static constexpr unsigned kInByteMask = 3u, kOutByteMask = 1u;
  __device__ __forceinline__ void operator()(const u32* in, u32* out) const { out[0] = f_and(in[0], in[1]); }
};

template <int OP>
int run_unary(const TwgIterDesc* d, const float* in, float* out, cudaStream_t s) {
  void* ptrs[2] = {out, const_cast<float*>(in)};
  return launch_pointwise(UnaryF32<OP>{}, d, ptrs, s);
}
template <int OP>
int run_binary(const TwgIterDesc* d, const float* a, const float* b, float alpha, float* out, cudaStream_t s) {
  void* ptrs[3] = {out, const_cast<float*>(a), const_cast<float*>(b)};
  return launch_pointwise(BinaryF32<OP>{alpha}, d, ptrs, s);
}
template <int OP>
int run_binary_scalar(const TwgIterDesc* d, const float* a, float scalar, float alpha, float* out, cudaStream_t s) {
  void* ptrs[2] = {out, const_cast<float*>(a)};
  return launch_pointwise(BinaryScalarF32<OP>{scalar, alpha}, d, ptrs, s);
}
template <int OP>
int run_compare(const TwgIterDesc* d, const float* a, const float* b, float scalar, uint8_t* out, cudaStream_t s) {
  if (b) {
    void* ptrs[3] = {out, const_cast<float*>(a), const_cast<float*>(b)};
    return launch_pointwise(CompareTensorF32<OP>{}, d, ptrs, s);
  }
  void* ptrs[2] = {out, const_cast<float*>(a)};
  return launch_pointwise(CompareScalarF32<OP>{scalar}, d, ptrs, s);
}

int and_bool(const TwgIterDesc* d, const void* a, const void* b, void* out, cudaStream_t s) {
  void* ptrs[3] = {out, const_cast<void*>(a), const_cast<void*>(b)};
  return launch_pointwise(AndBool{}, d, ptrs, s);
}

}  // namespace twg

using namespace twg;

extern "C" int twg_unary_f32(int op, const TwgIterDesc* desc, const float* in, float* out, void* stream) {
  TWG_TRACE("twg_unary_f32");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (op) {
    case TWG_UNARY_COPY: return run_unary<TWG_UNARY_COPY>(desc, in, out, s);
    case TWG_UNARY_RELU: return run_unary<TWG_UNARY_RELU>(desc, in, out, s);
    case TWG_UNARY_GELU_TANH: return run_unary<TWG_UNARY_GELU_TANH>(desc, in, out, s);
    case TWG_UNARY_SILU: return run_unary<TWG_UNARY_SILU>(desc, in, out, s);
    case TWG_UNARY_GELU_ERF: return run_unary<TWG_UNARY_GELU_ERF>(desc, in, out, s);
    case TWG_UNARY_ABS: return run_unary<TWG_UNARY_ABS>(desc, in, out, s);
    default: return set_error(TWG_ERR_INVALID, "twg_unary_f32: unknown op %d", op);
  }
}

extern "C" int twg_binary_f32(int op, const TwgIterDesc* desc, const float* a, const float* b, float alpha,
                              float* out, void* stream) {
  TWG_TRACE("twg_binary_f32");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (op) {
    case TWG_BINARY_ADD: return run_binary<TWG_BINARY_ADD>(desc, a, b, alpha, out, s);
    case TWG_BINARY_MUL: return run_binary<TWG_BINARY_MUL>(desc, a, b, alpha, out, s);
    case TWG_BINARY_FUSED_ADD_RELU: return run_binary<TWG_BINARY_FUSED_ADD_RELU>(desc, a, b, alpha, out, s);
    case TWG_BINARY_DIV: return run_binary<TWG_BINARY_DIV>(desc, a, b, alpha, out, s);
    default: return set_error(TWG_ERR_INVALID, "twg_binary_f32: unknown op %d", op);
  }
}

extern "C" int twg_binary_scalar_f32(int op, const TwgIterDesc* desc, const float* a, float scalar, float alpha,
                                     float* out, void* stream) {
  TWG_TRACE("twg_binary_scalar_f32");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (op) {
    case TWG_BINARY_ADD: return run_binary_scalar<TWG_BINARY_ADD>(desc, a, scalar, alpha, out, s);
    case TWG_BINARY_MUL: return run_binary_scalar<TWG_BINARY_MUL>(desc, a, scalar, alpha, out, s);
    case TWG_BINARY_FUSED_ADD_RELU: return run_binary_scalar<TWG_BINARY_FUSED_ADD_RELU>(desc, a, scalar, alpha, out, s);
    case TWG_BINARY_DIV: return run_binary_scalar<TWG_BINARY_DIV>(desc, a, scalar, alpha, out, s);
    default: return set_error(TWG_ERR_INVALID, "twg_binary_scalar_f32: unknown op %d", op);
  }
}

extern "C" int twg_where_f32(const TwgIterDesc* desc, const uint8_t* cond, const float* a, const float* b, float* out,
                             void* stream) {
  TWG_TRACE("twg_where_f32");
  void* ptrs[4] = {out, const_cast<uint8_t*>(cond), const_cast<float*>(a), const_cast<float*>(b)};
  return launch_pointwise(WhereF32{}, desc, ptrs, static_cast<cudaStream_t>(stream));
}

extern "C" int twg_masked_fill_f32(const TwgIterDesc* desc, const float* self, const uint8_t* mask, float value,
                                   float* out, void* stream) {
  TWG_TRACE("twg_masked_fill_f32");
  void* ptrs[3] = {out, const_cast<float*>(self), const_cast<uint8_t*>(mask)};
  return launch_pointwise(MaskedFillF32{value}, desc, ptrs, static_cast<cudaStream_t>(stream));
}

extern "C" int twg_compare_f32(int op, const TwgIterDesc* desc, const float* a, const float* b, float scalar,
                               uint8_t* out, void* stream) {
  TWG_TRACE("twg_compare_f32");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (op) {
    case TWG_CMP_EQ: return run_compare<TWG_CMP_EQ>(desc, a, b, scalar, out, s);
    case TWG_CMP_NE: return run_compare<TWG_CMP_NE>(desc, a, b, scalar, out, s);
    case TWG_CMP_LT: return run_compare<TWG_CMP_LT>(desc, a, b, scalar, out, s);
    case TWG_CMP_LE: return run_compare<TWG_CMP_LE>(desc, a, b, scalar, out, s);
    case TWG_CMP_GT: return run_compare<TWG_CMP_GT>(desc, a, b, scalar, out, s);
    case TWG_CMP_GE: return run_compare<TWG_CMP_GE>(desc, a, b, scalar, out, s);
    default: return set_error(TWG_ERR_INVALID, "twg_compare_f32: unknown op %d", op);
  }
}
