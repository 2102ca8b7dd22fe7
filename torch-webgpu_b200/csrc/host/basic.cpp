// Tensor creation and metadata ops.  Mirrors the registrations of the reference's
// csrc/ops/basic.cpp:294-307 (empty.memory_format, empty_strided, as_strided, view, resize_,
// reshape); none of them launches a kernel.  Zero-element tensors get a null DataPtr and work
// (the reference segfaults on them, tests/ops/test_silu.py:55).
#include <cstring>

#include <ATen/EmptyTensor.h>
#include <ATen/NativeFunctions.h>
#include <ATen/native/Resize.h>
#include <torch/library.h>

#include "twg_host.h"

namespace torch_webgpu {
namespace ops {

static c10::DeviceIndex resolve_device(const std::optional<at::Device>& device_opt) {
  if (device_opt.has_value()) {
    TORCH_CHECK(device_opt->is_privateuseone(), "torch_webgpu: expected a webgpu device, got ", *device_opt);
    if (device_opt->has_index()) {
      TORCH_CHECK(device_opt->index() < core::device_count(), "torch_webgpu: invalid device ordinal ",
                  static_cast<int>(device_opt->index()));
      return device_opt->index();
    }
  }
  return core::current_device();
}

at::Tensor empty_memory_format(c10::IntArrayRef size, std::optional<at::ScalarType> dtype_opt,
                               std::optional<at::Layout> layout_opt, std::optional<at::Device> device_opt,
                               std::optional<bool> pin_memory_opt, std::optional<c10::MemoryFormat> memory_format_opt) {
  TORCH_CHECK(!layout_opt.has_value() || *layout_opt == at::kStrided, "torch_webgpu: only strided tensors are supported");
  TORCH_CHECK(!pin_memory_opt.value_or(false), "torch_webgpu: pin_memory is a host-tensor option");
  core::DeviceScope scope(resolve_device(device_opt));
  constexpr c10::DispatchKeySet ks(c10::DispatchKey::PrivateUse1);
  return at::detail::empty_generic(size, core::getWebGPUCachingAllocator(), ks, c10::dtype_or_default(dtype_opt),
                                   memory_format_opt);
}

at::Tensor empty_strided(c10::IntArrayRef size, c10::IntArrayRef stride, std::optional<at::ScalarType> dtype_opt,
                         std::optional<at::Layout> layout_opt, std::optional<at::Device> device_opt,
                         std::optional<bool> pin_memory_opt) {
  TORCH_CHECK(!layout_opt.has_value() || *layout_opt == at::kStrided, "torch_webgpu: only strided tensors are supported");
  TORCH_CHECK(!pin_memory_opt.value_or(false), "torch_webgpu: pin_memory is a host-tensor option");
  core::DeviceScope scope(resolve_device(device_opt));
  constexpr c10::DispatchKeySet ks(c10::DispatchKey::PrivateUse1);
  return at::detail::empty_strided_generic(size, stride, core::getWebGPUCachingAllocator(), ks,
                                           c10::dtype_or_default(dtype_opt));
}

at::Tensor view(const at::Tensor& self, c10::IntArrayRef size) { return at::native::view(self, size); }

at::Tensor as_strided(const at::Tensor& self, c10::IntArrayRef size, c10::IntArrayRef stride,
                      std::optional<int64_t> storage_offset) {
  return at::native::as_strided_tensorimpl(self, size, stride, storage_offset);
}

at::Tensor _reshape_alias(const at::Tensor& self, c10::IntArrayRef size, c10::IntArrayRef stride) {
  return at::native::_reshape_alias(self, size, stride);
}

// Grow (never shrink) the storage so that `size` contiguous elements fit, keeping old contents.
const at::Tensor& resize_(const at::Tensor& self, c10::IntArrayRef size, std::optional<c10::MemoryFormat> format) {
  TORCH_CHECK(!format.has_value() || *format == c10::MemoryFormat::Contiguous || *format == c10::MemoryFormat::Preserve,
              "torch_webgpu: resize_ supports only the contiguous memory format");
  auto* impl = self.unsafeGetTensorImpl();
  int64_t numel = 1;
  for (auto s : size) {
    TORCH_CHECK(s >= 0, "torch_webgpu: resize_ got a negative dimension");
    numel *= s;
  }
  const size_t itemsize = self.dtype().itemsize();
  const size_t need = (static_cast<size_t>(impl->storage_offset()) + static_cast<size_t>(numel)) * itemsize;
  const c10::Storage& storage = impl->unsafe_storage();
  if (numel > 0 && need > storage.nbytes()) {
    TORCH_CHECK(storage.resizable(), "Trying to resize storage that is not resizable");
    const c10::DeviceIndex dev = self.device().index() < 0 ? core::current_device() : self.device().index();
    core::DeviceScope scope(dev);
    c10::DataPtr fresh = core::getWebGPUCachingAllocator()->allocate(need);
    if (storage.nbytes() > 0 && storage.data() != nullptr)
      TWG_TORCH_CHECK(twg_memcpy_d2d(fresh.get(), storage.data(), storage.nbytes(), core::current_stream(dev)));
    storage.unsafeGetStorageImpl()->set_data_ptr_noswap(std::move(fresh));
    storage.unsafeGetStorageImpl()->set_nbytes(need);
  }
  impl->set_sizes_contiguous(size);
  return self;
}

at::Tensor& set_source_storage_offset(at::Tensor& self, at::Storage source, int64_t storage_offset, c10::IntArrayRef size,
                                      c10::IntArrayRef stride) {
  return at::native::set_storage_cpu_(self, std::move(source), storage_offset, size, stride);
}
at::Tensor& set_source_storage(at::Tensor& self, at::Storage source) {
  const int64_t n = static_cast<int64_t>(source.nbytes() / self.dtype().itemsize());
  return at::native::set_storage_cpu_(self, std::move(source), 0, {n}, {});
}
at::Tensor& set_source_tensor(at::Tensor& self, const at::Tensor& source) {
  return at::native::set_tensor_(self, source);
}

// Scalars leave the device through a one-element read-back.
at::Scalar _local_scalar_dense(const at::Tensor& self) {
  TORCH_CHECK(self.numel() == 1, "a Tensor with ", self.numel(), " elements cannot be converted to Scalar");
  return at::_local_scalar_dense(self.cpu());
}

// fill_.Scalar on the device for every dtype: the scalar is converted to the tensor's dtype on the
// host (one element, PyTorch's own conversion rules) and its bit pattern is what the kernel writes.
at::Tensor& fill_scalar(at::Tensor& self, const at::Scalar& value) {
  if (self.numel() == 0) return self;
  const size_t itemsize = self.dtype().itemsize();
  TORCH_CHECK(itemsize == 1 || itemsize == 2 || itemsize == 4 || itemsize == 8, "torch_webgpu: fill_ supports element sizes 1, 2, 4 and 8, got ",
              itemsize, " (", self.scalar_type(), ")");
  TORCH_CHECK(self.dim() <= TWG_MAX_DIMS, "torch_webgpu: fill_ supports at most ", TWG_MAX_DIMS, " dimensions");
  at::Tensor one = at::scalar_tensor(value, self.options().device(at::kCPU));
  uint64_t pattern = 0;
  std::memcpy(&pattern, one.const_data_ptr(), itemsize);
  TwgIterDesc d;
  std::memset(&d, 0, sizeof(d));
  d.ndim = static_cast<int32_t>(self.dim());
  d.ntensors = 1;
  d.numel = self.numel();
  for (int k = 0; k < d.ndim; ++k) {  // dimension 0 of the descriptor is the last logical dimension
    const int64_t dim = d.ndim - 1 - k;
    d.shape[k] = self.size(dim);
    d.strides[0][k] = self.size(dim) == 1 ? 0 : self.stride(dim);
  }
  const c10::DeviceIndex dev = self.device().index() < 0 ? core::current_device() : self.device().index();
  core::DeviceScope scope(dev);
  TWG_TORCH_CHECK(twg_fill(&d, static_cast<int>(itemsize), pattern, self.data_ptr(), core::current_stream(dev)));
  return self;
}

// reshape is registered by name like the reference does (csrc/ops/basic.cpp:296-307, under both
// PrivateUse1 and AutogradPrivateUse1); the work is PyTorch's own composite: a view where the
// strides allow one, a copy otherwise, and its shape inference and error messages.
at::Tensor reshape(const at::Tensor& self, c10::SymIntArrayRef shape) { return at::native::reshape_symint(self, shape); }

at::Tensor& zero_(at::Tensor& self) {
  if (self.numel() == 0) return self;
  if (self.is_non_overlapping_and_dense()) {
    const c10::DeviceIndex dev = self.device().index() < 0 ? core::current_device() : self.device().index();
    core::DeviceScope scope(dev);
    TWG_TORCH_CHECK(twg_memset(self.data_ptr(), 0, static_cast<size_t>(self.numel()) * self.dtype().itemsize(),
                               core::current_stream(dev)));
    return self;
  }
  return fill_scalar(self, 0);
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("zero_", TORCH_FN(zero_));
  m.impl("empty.memory_format", TORCH_FN(empty_memory_format));
  m.impl("empty_strided", TORCH_FN(empty_strided));
  m.impl("view", TORCH_FN(view));
  m.impl("as_strided", TORCH_FN(as_strided));
  m.impl("_reshape_alias", TORCH_FN(_reshape_alias));
  m.impl("resize_", TORCH_FN(resize_));
  m.impl("reshape", TORCH_FN(reshape));
  m.impl("set_.source_Storage_storage_offset", TORCH_FN(set_source_storage_offset));
  m.impl("set_.source_Storage", TORCH_FN(set_source_storage));
  m.impl("set_.source_Tensor", TORCH_FN(set_source_tensor));
  m.impl("_local_scalar_dense", TORCH_FN(_local_scalar_dense));
  m.impl("fill_.Scalar", TORCH_FN(fill_scalar));
}

TORCH_LIBRARY_IMPL(aten, AutogradPrivateUse1, m) { m.impl("reshape", TORCH_FN(reshape)); }

}  // namespace ops
}  // namespace torch_webgpu
