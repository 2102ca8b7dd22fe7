/*
 * twg_oracle.c - CPU restatement of torch-webgpu's data-parallel op path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are compared against and
 * the CPU baseline the benchmark times beside them.  Nothing in the shipped package links,
 * imports or calls it, and the package has no CPU fallback.
 *
 * What is restated, and from where (paths inside the torch-webgpu project):
 *   - index math of the two compute shaders: linear invocation id -> coordinates -> per-operand
 *     element offsets (csrc/ops/binary.cpp:56-83, csrc/ops/unary.cpp:50-74);
 *   - the op expressions the shaders substitute (csrc/ops/binary.cpp:97-103,
 *     csrc/ops/unary.cpp:88-97): copy, add with alpha, mul, fused add+relu, relu, tanh-GELU, SiLU;
 *   - eq.Tensor / ne.Scalar / bitwise_and.Tensor / masked_select, which the reference runs as
 *     PyTorch CPU ATen kernels through at::native::cpu_fallback (csrc/bindings.cpp:27-42).
 *
 * Third-party dependency holding part of the algorithm: PyTorch (pinned torch==2.9.0 in the
 * reference's pyproject.toml:12; 2.11.0 installed here).  Where the WGSL text leaves a result
 * implementation-defined (NaN / -0.0 through max(), pow of a negative base, contraction of
 * a + alpha*b) the restatement follows the ATen CPU kernel, because that is what every reference
 * test asserts against (tests/ops/test_add.py:10, test_gelu.py:11-14, test_silu.py:10-13):
 *     add   : fmaf(alpha, b, a)        (one rounding, like at::native add with alpha)
 *     relu  : x < 0 ? 0 : x            (NaN and -0.0 pass through, clamp_min semantics)
 *     silu  : x / (1 + expf(-x))       (ATen form; *_SHADER is the literal WGSL form)
 *     gelu  : erf form per ATen/native/cpu/Gelu.h; tanh form per unary.cpp:94 / Gelu.h
 * Pinned against the reference tests' known-answer vectors and against outputs of the ATen CPU
 * kernels committed as fixtures (tests/golden/); see tests/test_oracle.py.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define TWGO_MAX_DIMS 8

/* Same layout idea as the shaders' Params blocks (binary.h:108-124, unary.h:88-101), 64-bit.
 * Dimension ndim-1 is peeled first, exactly like the shader loop `for d = ndim-1 .. 0`. */
typedef struct TwgoIter {
  int32_t ndim;
  int32_t pad;
  int64_t length;
  int64_t shape[TWGO_MAX_DIMS];
  int64_t out_strides[TWGO_MAX_DIMS];
  int64_t a_strides[TWGO_MAX_DIMS];
  int64_t b_strides[TWGO_MAX_DIMS];
  int64_t out_offset, a_offset, b_offset;
} TwgoIter;

enum {
  TWGO_COPY = 0, TWGO_RELU = 1, TWGO_GELU_TANH = 2, TWGO_SILU = 3, TWGO_GELU_ERF = 4, TWGO_ABS = 5,
  TWGO_SILU_SHADER = 6, TWGO_GELU_TANH_SHADER = 7
};
enum { TWGO_ADD = 0, TWGO_MUL = 1, TWGO_FUSED_ADD_RELU = 2, TWGO_DIV = 3 };
enum { TWGO_EQ = 0, TWGO_NE = 1, TWGO_LT = 2, TWGO_LE = 3, TWGO_GT = 4, TWGO_GE = 5 };

int twgo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void twgo_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* binary.cpp:60-83 / unary.cpp:54-74: coordinates from the linear index, then dot with strides. */
static inline void offsets(const TwgoIter* it, int64_t i, int64_t* o, int64_t* a, int64_t* b) {
  int64_t remaining = i, io = 0, ia = 0, ib = 0;
  for (int d = it->ndim - 1; d >= 0; --d) {
    const int64_t s = it->shape[d];
    const int64_t c = remaining % s;
    remaining /= s;
    io += c * it->out_strides[d];
    ia += c * it->a_strides[d];
    ib += c * it->b_strides[d];
  }
  *o = io + it->out_offset;
  *a = ia + it->a_offset;
  *b = ib + it->b_offset;
}

static inline float relu1(float x) { return x < 0.0f ? 0.0f : x; }

static inline float unary1(int op, float x) {
  switch (op) {
    case TWGO_COPY: return x;
    case TWGO_RELU: return relu1(x);
    case TWGO_ABS: return fabsf(x);
    case TWGO_SILU: return x / (1.0f + expf(-x));
    case TWGO_SILU_SHADER: return x * (1.0f / (1.0f + expf(-1.0f * x)));          /* unary.cpp:97 */
    case TWGO_GELU_ERF: return x * 0.5f * (1.0f + erff(x * 0.70710678118654752440f));
    case TWGO_GELU_TANH: {
      const float kBeta = 0.79788456080286535588f, kKappa = 0.044715f;
      const float x3 = x * x * x;
      const float inner = kBeta * (x + kKappa * x3);
      return 0.5f * x * (1.0f + tanhf(inner));
    }
    case TWGO_GELU_TANH_SHADER: {                                                    /* unary.cpp:94 */
      const float c = sqrtf(2.0f / 3.14159265358979323846f);
      return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * (x * x * x))));
    }
    default: return NAN;
  }
}

int twgo_unary_f32(int op, const TwgoIter* it, const float* in, float* out) {
  if (op < 0 || op > TWGO_GELU_TANH_SHADER) return -1;
  const int64_t n = it->length;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    int64_t o, a, b;
    offsets(it, i, &o, &a, &b);
    out[o] = unary1(op, in[a]);
  }
  return 0;
}

int twgo_binary_f32(int op, const TwgoIter* it, const float* x, const float* y, float alpha, float* out) {
  if (op < 0 || op > TWGO_DIV) return -1;
  const int64_t n = it->length;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    int64_t o, a, b;
    offsets(it, i, &o, &a, &b);
    float r;
    if (op == TWGO_ADD) r = fmaf(alpha, y[b], x[a]);            /* binary.cpp:97  */
    else if (op == TWGO_MUL) r = x[a] * y[b];                   /* binary.cpp:100 */
    else if (op == TWGO_DIV) r = x[a] / y[b];                   /* README.md:107 (div, unchecked) */
    else r = relu1(x[a] + y[b]);                                /* binary.cpp:103 */
    out[o] = r;
  }
  return 0;
}

static inline uint8_t cmp1(int op, float a, float b) {
  switch (op) {
    case TWGO_EQ: return a == b;
    case TWGO_NE: return a != b;
    case TWGO_LT: return a < b;
    case TWGO_LE: return a <= b;
    case TWGO_GT: return a > b;
    default: return a >= b;
  }
}

/* y == NULL compares against `scalar` (ne.Scalar / eq.Scalar). */
int twgo_compare_f32(int op, const TwgoIter* it, const float* x, const float* y, float scalar, uint8_t* out) {
  if (op < 0 || op > TWGO_GE) return -1;
  const int64_t n = it->length;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    int64_t o, a, b;
    offsets(it, i, &o, &a, &b);
    out[o] = cmp1(op, x[a], y ? y[b] : scalar);
  }
  return 0;
}

/* bool & bool: logical and of 0/1 bytes (any non-zero byte is true). */
/* Element-type conversion with C cast rules (ATen's copy kernel is a static_cast per element).
 * dtype codes: 0 u8, 1 i8, 2 i16, 3 i32, 4 i64, 5 f16, 6 bf16 (bit pattern), 7 f32, 8 f64, 9 bool.
 * Every source is first widened exactly (double for floats, int64 else), then narrowed the way a
 * cast does: through float for f16 / bf16 (round to nearest even), truncation toward zero for
 * float -> integer. */
static inline float bf16_to_f32(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;                    /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);                                        /* round to nearest even */
  return (uint16_t)(u >> 16);
}
int twgo_convert(int64_t n, int src, int dst, const void* in, void* out) {
  if (src < 0 || src > 9 || dst < 0 || dst > 9) return -1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    double fv = 0.0; int64_t iv = 0; int is_f = 0;
    switch (src) {
      case 0: iv = ((const uint8_t*)in)[i]; break;
      case 1: iv = ((const int8_t*)in)[i]; break;
      case 2: iv = ((const int16_t*)in)[i]; break;
      case 3: iv = ((const int32_t*)in)[i]; break;
      case 4: iv = ((const int64_t*)in)[i]; break;
      case 5: fv = (double)(float)((const _Float16*)in)[i]; is_f = 1; break;
      case 6: fv = (double)bf16_to_f32(((const uint16_t*)in)[i]); is_f = 1; break;
      case 7: fv = (double)((const float*)in)[i]; is_f = 1; break;
      case 8: fv = ((const double*)in)[i]; is_f = 1; break;
      default: iv = ((const uint8_t*)in)[i] != 0; break;
    }
    const int64_t as_int = is_f ? (int64_t)fv : iv;
    switch (dst) {
      case 0: ((uint8_t*)out)[i] = (uint8_t)as_int; break;
      case 1: ((int8_t*)out)[i] = (int8_t)as_int; break;
      case 2: ((int16_t*)out)[i] = (int16_t)as_int; break;
      case 3: ((int32_t*)out)[i] = (int32_t)as_int; break;
      case 4: ((int64_t*)out)[i] = as_int; break;
      case 5: ((_Float16*)out)[i] = (_Float16)(is_f ? (float)fv : (float)iv); break;
      case 6: ((uint16_t*)out)[i] = f32_to_bf16(is_f ? (float)fv : (float)iv); break;
      case 7: ((float*)out)[i] = is_f ? (float)fv : (float)iv; break;
      case 8: ((double*)out)[i] = is_f ? fv : (double)iv; break;
      default: ((uint8_t*)out)[i] = is_f ? (fv != 0.0) : (iv != 0); break;
    }
  }
  return 0;
}

/* where.self and masked_fill.Scalar (README.md:128-166, unchecked: the reference has no kernel;
 * semantics are ATen's).  Operands are dense and of one length: the caller has broadcast them. */
int twgo_where_f32(int64_t n, const uint8_t* cond, const float* x, const float* y, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = cond[i] != 0 ? x[i] : y[i];
  return 0;
}

int twgo_masked_fill_f32(int64_t n, const float* self, const uint8_t* mask, float value, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = mask[i] != 0 ? value : self[i];
  return 0;
}

int twgo_and_bool(const TwgoIter* it, const uint8_t* x, const uint8_t* y, uint8_t* out) {
  const int64_t n = it->length;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    int64_t o, a, b;
    offsets(it, i, &o, &a, &b);
    out[o] = (uint8_t)((x[a] != 0) & (y[b] != 0));
  }
  return 0;
}

/* integer bitwise and, any width: byte-wise over itemsize-byte elements. */
int twgo_and_bytes(const TwgoIter* it, int itemsize, const uint8_t* x, const uint8_t* y, uint8_t* out) {
  const int64_t n = it->length;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    int64_t o, a, b;
    offsets(it, i, &o, &a, &b);
    for (int k = 0; k < itemsize; ++k) out[o * itemsize + k] = x[a * itemsize + k] & y[b * itemsize + k];
  }
  return 0;
}

/* strided copy of itemsize-byte elements (UnaryOp::Copy, copy.cpp:123-134) */
int twgo_copy_bytes(const TwgoIter* it, int itemsize, const uint8_t* x, uint8_t* out) {
  const int64_t n = it->length;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    int64_t o, a, b;
    offsets(it, i, &o, &a, &b);
    memcpy(out + o * itemsize, x + a * itemsize, (size_t)itemsize);
  }
  return 0;
}

/* masked_select: walk the broadcast shape in row-major order (the iterator's dimension ndim-1 is
 * peeled first, so callers pass the logical shape as-is), a_strides = self, b_strides = mask
 * (0 where broadcast); append self[...] wherever mask[...] != 0.  Returns the count.
 * Parallel version: count per chunk, exclusive scan, scatter - same output as the serial loop. */
int64_t twgo_masked_select_f32(const TwgoIter* it, const float* self, const uint8_t* mask, float* out) {
  const int64_t n = it->length;
  int nt = twgo_num_threads();
  if (n < (1 << 16)) nt = 1;
  int64_t* counts = (int64_t*)calloc((size_t)nt + 1, sizeof(int64_t));
  if (!counts) return -1;
  const int64_t chunk = (n + nt - 1) / nt;
#pragma omp parallel for schedule(static, 1) num_threads(nt)
  for (int t = 0; t < nt; ++t) {
    const int64_t lo = t * chunk, hi = lo + chunk < n ? lo + chunk : n;
    int64_t c = 0;
    for (int64_t i = lo; i < hi; ++i) {
      int64_t o, a, b;
      offsets(it, i, &o, &a, &b);
      c += mask[b] != 0;
    }
    counts[t + 1] = c;
  }
  for (int t = 0; t < nt; ++t) counts[t + 1] += counts[t];
#pragma omp parallel for schedule(static, 1) num_threads(nt)
  for (int t = 0; t < nt; ++t) {
    const int64_t lo = t * chunk, hi = lo + chunk < n ? lo + chunk : n;
    int64_t k = counts[t];
    for (int64_t i = lo; i < hi; ++i) {
      int64_t o, a, b;
      offsets(it, i, &o, &a, &b);
      if (mask[b] != 0) out[k++] = self[a];
    }
  }
  const int64_t total = counts[nt];
  free(counts);
  return total;
}

/* The torch.compile chain of the benchmark, op by op with every intermediate rounded to f32 as
 * separate kernels would: y = relu(silu(a + b) + c); m = (y == 0) & (a != 0).
 * y may be NULL.  Dense 1-D operands. */
int twgo_chain_mask(int64_t n, const float* a, const float* b, const float* c, float* y, uint8_t* m) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float s = fmaf(1.0f, b[i], a[i]);
    const float t = unary1(TWGO_SILU, s);
    const float u = fmaf(1.0f, c[i], t);
    const float yy = relu1(u);
    if (y) y[i] = yy;
    m[i] = (uint8_t)((yy == 0.0f) & (a[i] != 0.0f));
  }
  return 0;
}
