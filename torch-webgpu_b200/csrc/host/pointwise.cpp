// ATen pointwise ops under the PrivateUse1 key.
//
// Same registrations as the reference: add.out (csrc/ops/arithmetic.cpp:393-399), relu / gelu /
// silu and their .out forms (csrc/ops/activation_functions.cpp:116-126), and the ops the reference
// routes to at::native::cpu_fallback - ne.Scalar(_out), eq.Tensor(_out), bitwise_and.Tensor(_out),
// abs (csrc/bindings.cpp:32-43) - which are real kernels here.  Added because the configurations
// need them: eq.Scalar(_out) (torch.eq(y, 0)), mul.out (the launcher exists in the reference but
// its registration is commented out, arithmetic.cpp:396), relu_.
//
// Each wrapper builds the at::TensorIterator the reference builds, turns it into a TwgIterDesc and
// calls the C ABI; the library picks the dense / tile / strided kernel.
#include <ATen/NativeFunctions.h>
#include <ATen/native/BinaryOps.h>
#include <ATen/native/DispatchStub.h>
#include <torch/library.h>

#include "twg_host.h"

namespace torch_webgpu {
namespace ops {

TwgIterDesc desc_from_iter(const at::TensorIteratorBase& iter) {
  TORCH_CHECK(iter.ndim() <= TWG_MAX_DIMS, "torch_webgpu: tensors that do not coalesce to at most ", TWG_MAX_DIMS,
              " dimensions are not supported (got ", iter.ndim(), ")");
  TORCH_CHECK(iter.ntensors() <= TWG_MAX_TENSORS, "torch_webgpu: too many operands");
  TwgIterDesc d;
  std::memset(&d, 0, sizeof(d));
  d.ndim = iter.ndim();
  d.ntensors = iter.ntensors();
  d.numel = iter.numel();
  const auto shape = iter.shape();
  for (int k = 0; k < d.ndim; ++k) d.shape[k] = shape[k];
  for (int t = 0; t < d.ntensors; ++t) {
    const auto strides = iter.strides(t);  // bytes
    const int64_t es = static_cast<int64_t>(iter.element_size(t));
    for (int k = 0; k < d.ndim; ++k) {
      TORCH_INTERNAL_ASSERT(strides[k] % es == 0);
      d.strides[t][k] = strides[k] / es;
    }
  }
  return d;
}

c10::DeviceIndex iter_device(const at::TensorIteratorBase& iter) {
  c10::DeviceIndex dev = -1;
  for (int t = 0; t < iter.ntensors(); ++t) {
    const c10::Device d = iter.device(t);
    TORCH_CHECK(d.is_privateuseone(), "torch_webgpu: operand ", t, " lives on ", d, ", expected a webgpu tensor");
    const c10::DeviceIndex i = d.index() < 0 ? core::current_device() : d.index();
    TORCH_CHECK(dev < 0 || dev == i, "torch_webgpu: operands live on different webgpu devices");
    dev = i;
  }
  return dev < 0 ? core::current_device() : dev;
}

at::Tensor to_device_if_cpu_scalar(const at::Tensor& t, c10::Device device, at::ScalarType dtype) {
  // Python numbers arrive as 0-dim CPU tensors (float64 / int64); they take the tensor operand's dtype.
  if (t.device().is_cpu() && t.dim() == 0) return t.to(dtype).to(device);
  return t;
}

static void check_all_float(const at::TensorIteratorBase& iter, const char* name) {
  for (int t = 0; t < iter.ntensors(); ++t)
    TORCH_CHECK(iter.dtype(t) == at::kFloat, "torch_webgpu: ", name, " supports float32 tensors only, operand ", t,
                " is ", iter.dtype(t));
}

void unary_kernel(int op, at::TensorIteratorBase& iter) {
  TORCH_CHECK(iter.ntensors() == 2, "torch_webgpu: unary kernel expects 1 output and 1 input");
  check_all_float(iter, "this unary op");
  if (iter.numel() == 0) return;
  const c10::DeviceIndex dev = iter_device(iter);
  core::DeviceScope scope(dev);
  TwgIterDesc desc = desc_from_iter(iter);
  TWG_TORCH_CHECK(twg_unary_f32(op, &desc, static_cast<const float*>(iter.data_ptr(1)),
                                static_cast<float*>(iter.data_ptr(0)), core::current_stream(dev)));
}

void binary_kernel(int op, at::TensorIteratorBase& iter, const at::Scalar& alpha) {
  TORCH_CHECK(iter.ntensors() == 3, "torch_webgpu: binary kernel expects 1 output and 2 inputs");
  check_all_float(iter, "this binary op");
  if (iter.numel() == 0) return;
  const c10::DeviceIndex dev = iter_device(iter);
  core::DeviceScope scope(dev);
  TwgIterDesc desc = desc_from_iter(iter);
  TWG_TORCH_CHECK(twg_binary_f32(op, &desc, static_cast<const float*>(iter.data_ptr(1)),
                                 static_cast<const float*>(iter.data_ptr(2)), alpha.to<float>(),
                                 static_cast<float*>(iter.data_ptr(0)), core::current_stream(dev)));
}

// ---- add / mul ---------------------------------------------------------------------------
// Python numbers on the right (x + 2, x * 0.5) arrive as 0-dim CPU tensors: they ride in the kernel's
// arguments instead of being uploaded and read back as a broadcast operand.
static bool binary_scalar_out(int op, const at::Tensor& self, const at::Tensor& other, const at::Scalar& alpha,
                              at::Tensor& out) {
  if (!(other.device().is_cpu() && other.dim() == 0 && self.device().is_privateuseone())) return false;
  if (self.scalar_type() != at::kFloat || out.scalar_type() != at::kFloat) return false;
  at::TensorIteratorConfig config;
  config.set_check_mem_overlap(true).add_output(out).add_const_input(self).check_all_same_dtype(true);
  auto iter = config.build();
  if (iter.numel() == 0) return true;
  const c10::DeviceIndex dev = iter_device(iter);
  core::DeviceScope scope(dev);
  TwgIterDesc desc = desc_from_iter(iter);
  TWG_TORCH_CHECK(twg_binary_scalar_f32(op, &desc, static_cast<const float*>(iter.data_ptr(1)), other.item<float>(),
                                        alpha.to<float>(), static_cast<float*>(iter.data_ptr(0)), core::current_stream(dev)));
  return true;
}

static at::Tensor& binary_out(int op, const at::Tensor& self, const at::Tensor& other, const at::Scalar& alpha,
                              at::Tensor& out) {
  if (binary_scalar_out(op, self, other, alpha, out)) return out;
  const at::Tensor a = to_device_if_cpu_scalar(self, out.device(), out.scalar_type());
  const at::Tensor b = to_device_if_cpu_scalar(other, out.device(), out.scalar_type());
  at::TensorIteratorConfig config;
  config.set_check_mem_overlap(true);
  config.add_output(out);
  config.add_const_input(a);
  config.add_const_input(b);
  config.check_all_same_dtype(true);
  auto iter = config.build();
  binary_kernel(op, iter, alpha);
  return out;
}

at::Tensor& add_out_webgpu(const at::Tensor& self, const at::Tensor& other, const at::Scalar& alpha, at::Tensor& out) {
  return binary_out(TWG_BINARY_ADD, self, other, alpha, out);
}
at::Tensor& mul_out_webgpu(const at::Tensor& self, const at::Tensor& other, at::Tensor& out) {
  return binary_out(TWG_BINARY_MUL, self, other, 1, out);
}

// sub is add with the negated alpha (what ATen does: one fused multiply-add, one rounding)
at::Tensor& sub_out_webgpu(const at::Tensor& self, const at::Tensor& other, const at::Scalar& alpha, at::Tensor& out) {
  return binary_out(TWG_BINARY_ADD, self, other, -alpha.to<double>(), out);
}
// true division only; floor / trunc rounding modes are not part of this path
at::Tensor& div_out_webgpu(const at::Tensor& self, const at::Tensor& other, at::Tensor& out) {
  return binary_out(TWG_BINARY_DIV, self, other, 1, out);
}

// ---- where / masked_fill -------------------------------------------------------------------
at::Tensor& where_self_out(const at::Tensor& condition, const at::Tensor& self, const at::Tensor& other, at::Tensor& out) {
  TORCH_CHECK(condition.scalar_type() == at::kBool, "where expected condition to be a boolean tensor, but got a tensor with dtype ",
              condition.scalar_type());
  const at::Tensor a = to_device_if_cpu_scalar(self, condition.device(), at::kFloat);
  const at::Tensor b = to_device_if_cpu_scalar(other, condition.device(), at::kFloat);
  TORCH_CHECK(a.scalar_type() == at::kFloat && b.scalar_type() == at::kFloat && out.scalar_type() == at::kFloat,
              "torch_webgpu: where supports float32 values only, got ", a.scalar_type(), " and ", b.scalar_type());
  at::TensorIteratorConfig config;
  config.set_check_mem_overlap(true).check_all_same_dtype(false);
  config.add_output(out).add_const_input(condition).add_const_input(a).add_const_input(b);
  auto iter = config.build();
  if (iter.numel() == 0) return out;
  const c10::DeviceIndex dev = iter_device(iter);
  core::DeviceScope scope(dev);
  TwgIterDesc desc = desc_from_iter(iter);
  TWG_TORCH_CHECK(twg_where_f32(&desc, static_cast<const uint8_t*>(iter.data_ptr(1)), static_cast<const float*>(iter.data_ptr(2)),
                                static_cast<const float*>(iter.data_ptr(3)), static_cast<float*>(iter.data_ptr(0)),
                                core::current_stream(dev)));
  return out;
}
at::Tensor where_self(const at::Tensor& condition, const at::Tensor& self, const at::Tensor& other) {
  auto shape = at::infer_size(condition.sizes(), at::infer_size(self.sizes(), other.sizes()));
  at::Tensor out = at::empty(shape, condition.options().dtype(at::kFloat));
  return where_self_out(condition, self, other, out);
}
at::Tensor& masked_fill_scalar_(at::Tensor& self, const at::Tensor& mask, const at::Scalar& value) {
  TORCH_CHECK(mask.scalar_type() == at::kBool, "masked_fill_ only supports boolean masks, but got mask with dtype ",
              mask.scalar_type());
  TORCH_CHECK(self.scalar_type() == at::kFloat, "torch_webgpu: masked_fill_ supports float32 tensors only, got ",
              self.scalar_type());
  at::TensorIteratorConfig config;
  config.set_check_mem_overlap(false).check_all_same_dtype(false).resize_outputs(false);
  config.add_output(self).add_const_input(self).add_const_input(mask);
  auto iter = config.build();
  if (iter.numel() == 0) return self;
  const c10::DeviceIndex dev = iter_device(iter);
  core::DeviceScope scope(dev);
  TwgIterDesc desc = desc_from_iter(iter);
  TWG_TORCH_CHECK(twg_masked_fill_f32(&desc, static_cast<const float*>(iter.data_ptr(1)), static_cast<const uint8_t*>(iter.data_ptr(2)),
                                      value.to<float>(), static_cast<float*>(iter.data_ptr(0)), core::current_stream(dev)));
  return self;
}

// ---- relu / gelu / silu / abs ----------------------------------------------------------------
static at::Tensor& unary_out(int op, const at::Tensor& self, at::Tensor& out) {
  at::TensorIteratorConfig config;
  config.set_check_mem_overlap(true);
  config.add_output(out);
  config.add_const_input(self);
  config.check_all_same_dtype(true);
  auto iter = config.build();
  unary_kernel(op, iter);
  return out;
}
static at::Tensor unary_functional(int op, const at::Tensor& self) {
  at::Tensor out = at::empty_like(self);
  return unary_out(op, self, out);
}
static int gelu_op(std::string_view approximate) {
  if (approximate == "none") return TWG_UNARY_GELU_ERF;
  TORCH_CHECK(approximate == "tanh", "approximate argument must be either none or tanh.");
  return TWG_UNARY_GELU_TANH;
}

at::Tensor relu(const at::Tensor& self) { return unary_functional(TWG_UNARY_RELU, self); }
at::Tensor& relu_out(const at::Tensor& self, at::Tensor& out) { return unary_out(TWG_UNARY_RELU, self, out); }
at::Tensor& relu_(at::Tensor& self) { return unary_out(TWG_UNARY_RELU, self, self); }
at::Tensor gelu(const at::Tensor& self, std::string_view approximate) { return unary_functional(gelu_op(approximate), self); }
at::Tensor& gelu_out(const at::Tensor& self, std::string_view approximate, at::Tensor& out) {
  return unary_out(gelu_op(approximate), self, out);
}
at::Tensor silu(const at::Tensor& self) { return unary_functional(TWG_UNARY_SILU, self); }
at::Tensor& silu_out(const at::Tensor& self, at::Tensor& out) { return unary_out(TWG_UNARY_SILU, self, out); }
at::Tensor abs(const at::Tensor& self) { return unary_functional(TWG_UNARY_ABS, self); }
at::Tensor& abs_out(const at::Tensor& self, at::Tensor& out) { return unary_out(TWG_UNARY_ABS, self, out); }

// ---- comparisons ---------------------------------------------------------------------------------
static at::Tensor& compare_tensor_out(int op, const at::Tensor& self, const at::Tensor& other, at::Tensor& out) {
  TORCH_CHECK(out.scalar_type() == at::kBool, "torch_webgpu: comparison output must be a bool tensor");
  if (other.device().is_cpu() && other.dim() == 0) {
    // wrapped number: compare against the scalar directly
    at::TensorIteratorConfig config;
    config.set_check_mem_overlap(true).add_output(out).add_const_input(self).check_all_same_dtype(false);
    auto iter = config.build();
    TORCH_CHECK(iter.dtype(1) == at::kFloat, "torch_webgpu: comparisons support float32 inputs only");
    if (iter.numel() == 0) return out;
    const c10::DeviceIndex dev = iter_device(iter);
    core::DeviceScope scope(dev);
    TwgIterDesc desc = desc_from_iter(iter);
    TWG_TORCH_CHECK(twg_compare_f32(op, &desc, static_cast<const float*>(iter.data_ptr(1)), nullptr,
                                    other.item<float>(), static_cast<uint8_t*>(iter.data_ptr(0)), core::current_stream(dev)));
    return out;
  }
  at::TensorIteratorConfig config;
  config.set_check_mem_overlap(true).add_output(out).add_const_input(self).add_const_input(other).check_all_same_dtype(false);
  auto iter = config.build();
  TORCH_CHECK(iter.dtype(1) == at::kFloat && iter.dtype(2) == at::kFloat,
              "torch_webgpu: comparisons support float32 inputs only");
  if (iter.numel() == 0) return out;
  const c10::DeviceIndex dev = iter_device(iter);
  core::DeviceScope scope(dev);
  TwgIterDesc desc = desc_from_iter(iter);
  TWG_TORCH_CHECK(twg_compare_f32(op, &desc, static_cast<const float*>(iter.data_ptr(1)),
                                  static_cast<const float*>(iter.data_ptr(2)), 0.0f,
                                  static_cast<uint8_t*>(iter.data_ptr(0)), core::current_stream(dev)));
  return out;
}

static at::Tensor& compare_scalar_out(int op, const at::Tensor& self, const at::Scalar& other, at::Tensor& out) {
  TORCH_CHECK(out.scalar_type() == at::kBool, "torch_webgpu: comparison output must be a bool tensor");
  at::TensorIteratorConfig config;
  config.set_check_mem_overlap(true).add_output(out).add_const_input(self).check_all_same_dtype(false);
  auto iter = config.build();
  TORCH_CHECK(iter.dtype(1) == at::kFloat, "torch_webgpu: comparisons support float32 inputs only");
  if (iter.numel() == 0) return out;
  const c10::DeviceIndex dev = iter_device(iter);
  core::DeviceScope scope(dev);
  TwgIterDesc desc = desc_from_iter(iter);
  // the scalar is compared in the tensor's dtype, like the CPU kernel does
  TWG_TORCH_CHECK(twg_compare_f32(op, &desc, static_cast<const float*>(iter.data_ptr(1)), nullptr, other.to<float>(),
                                  static_cast<uint8_t*>(iter.data_ptr(0)), core::current_stream(dev)));
  return out;
}

static at::Tensor compare_tensor(int op, const at::Tensor& self, const at::Tensor& other) {
  const auto shape = at::infer_size(self.sizes(), other.sizes());
  at::Tensor out = at::empty(shape, self.options().dtype(at::kBool));
  return compare_tensor_out(op, self, other, out);
}
static at::Tensor compare_scalar(int op, const at::Tensor& self, const at::Scalar& other) {
  at::Tensor out = at::empty(self.sizes(), self.options().dtype(at::kBool));
  return compare_scalar_out(op, self, other, out);
}

#define TWG_DEFINE_COMPARE(name, OP)                                                                              \
  at::Tensor name##_tensor(const at::Tensor& a, const at::Tensor& b) { return compare_tensor(OP, a, b); }         \
  at::Tensor& name##_tensor_out(const at::Tensor& a, const at::Tensor& b, at::Tensor& out) {                      \
    return compare_tensor_out(OP, a, b, out);                                                                     \
  }                                                                                                               \
  at::Tensor name##_scalar(const at::Tensor& a, const at::Scalar& b) { return compare_scalar(OP, a, b); }         \
  at::Tensor& name##_scalar_out(const at::Tensor& a, const at::Scalar& b, at::Tensor& out) {                      \
    return compare_scalar_out(OP, a, b, out);                                                                     \
  }
TWG_DEFINE_COMPARE(eq, TWG_CMP_EQ)
TWG_DEFINE_COMPARE(ne, TWG_CMP_NE)
TWG_DEFINE_COMPARE(lt, TWG_CMP_LT)
TWG_DEFINE_COMPARE(le, TWG_CMP_LE)
TWG_DEFINE_COMPARE(gt, TWG_CMP_GT)
TWG_DEFINE_COMPARE(ge, TWG_CMP_GE)
#undef TWG_DEFINE_COMPARE

// ---- bitwise_and -------------------------------------------------------------------------------
at::Tensor& bitwise_and_out(const at::Tensor& self, const at::Tensor& other, at::Tensor& out) {
  TORCH_CHECK(self.scalar_type() == other.scalar_type() && self.scalar_type() == out.scalar_type(),
              "torch_webgpu: bitwise_and expects operands of one dtype, got ", self.scalar_type(), ", ",
              other.scalar_type(), " -> ", out.scalar_type());
  TORCH_CHECK(self.scalar_type() == at::kBool || at::isIntegralType(self.scalar_type(), false),
              "bitwise_and is only defined for integral and bool tensors");
  at::TensorIteratorConfig config;
  config.set_check_mem_overlap(true).add_output(out).add_const_input(self).add_const_input(other).check_all_same_dtype(true);
  auto iter = config.build();
  if (iter.numel() == 0) return out;
  const c10::DeviceIndex dev = iter_device(iter);
  core::DeviceScope scope(dev);
  TwgIterDesc desc = desc_from_iter(iter);
  TWG_TORCH_CHECK(twg_bitwise_and(&desc, static_cast<int>(out.dtype().itemsize()), self.scalar_type() == at::kBool ? 1 : 0,
                                  iter.data_ptr(1), iter.data_ptr(2), iter.data_ptr(0), core::current_stream(dev)));
  return out;
}
at::Tensor bitwise_and(const at::Tensor& self, const at::Tensor& other) {
  const auto shape = at::infer_size(self.sizes(), other.sizes());
  at::Tensor out = at::empty(shape, self.options());
  return bitwise_and_out(self, other, out);
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("add.out", TORCH_FN(add_out_webgpu));
  m.impl("mul.out", TORCH_FN(mul_out_webgpu));
  m.impl("sub.out", TORCH_FN(sub_out_webgpu));
  m.impl("div.out", TORCH_FN(div_out_webgpu));
  m.impl("where.self", TORCH_FN(where_self));
  m.impl("where.self_out", TORCH_FN(where_self_out));
  m.impl("masked_fill_.Scalar", TORCH_FN(masked_fill_scalar_));
  m.impl("relu", TORCH_FN(relu));
  m.impl("relu.out", TORCH_FN(relu_out));
  m.impl("relu_", TORCH_FN(relu_));
  m.impl("gelu", TORCH_FN(gelu));
  m.impl("gelu.out", TORCH_FN(gelu_out));
  m.impl("silu", TORCH_FN(silu));
  m.impl("silu.out", TORCH_FN(silu_out));
  m.impl("abs", TORCH_FN(abs));
  m.impl("abs.out", TORCH_FN(abs_out));
#define TWG_REGISTER_COMPARE(name)                             \
  m.impl(#name ".Tensor", TORCH_FN(name##_tensor));            \
  m.impl(#name ".Tensor_out", TORCH_FN(name##_tensor_out));    \
  m.impl(#name ".Scalar", TORCH_FN(name##_scalar));            \
  m.impl(#name ".Scalar_out", TORCH_FN(name##_scalar_out));
  TWG_REGISTER_COMPARE(eq)
  TWG_REGISTER_COMPARE(ne)
  TWG_REGISTER_COMPARE(lt)
  TWG_REGISTER_COMPARE(le)
  TWG_REGISTER_COMPARE(gt)
  TWG_REGISTER_COMPARE(ge)
#undef TWG_REGISTER_COMPARE
  m.impl("bitwise_and.Tensor", TORCH_FN(bitwise_and));
  m.impl("bitwise_and.Tensor_out", TORCH_FN(bitwise_and_out));
}

}  // namespace ops
}  // namespace torch_webgpu

// The reference also plugs its launchers into ATen's add/mul dispatch stubs
// (csrc/ops/arithmetic.cpp:403-418), which is what serves code paths that reach the stub through
// a structured kernel rather than add.out.
namespace at {
namespace native {
static void add_kernel_webgpu(TensorIteratorBase& iter, const Scalar& alpha) {
  torch_webgpu::ops::binary_kernel(TWG_BINARY_ADD, iter, alpha);
}
REGISTER_PRIVATEUSE1_DISPATCH(add_stub, &add_kernel_webgpu);
static void mul_kernel_webgpu(TensorIteratorBase& iter) { torch_webgpu::ops::binary_kernel(TWG_BINARY_MUL, iter, 1); }
REGISTER_PRIVATEUSE1_DISPATCH(mul_stub, &mul_kernel_webgpu);
}  // namespace native
}  // namespace at
