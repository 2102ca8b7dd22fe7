// copy_ / _copy_from / _copy_from_and_resize / to.device (the reference's csrc/ops/copy.cpp:69-189).
//
// Host->device and device->host transfers are cudaMemcpyAsync on the tensor's stream through the
// library (pinned memory directly, pageable memory through a pinned staging ring); device->device
// is a dense async copy or the strided copy kernel.  Differences from the reference, on purpose:
// every dtype can be moved (it asserts Float on read-back, copy.cpp:22), storage offsets are
// honoured in both directions (copy.cpp:42 ignores the source offset), non-contiguous device
// tensors can be the destination of an upload, and the aten CPU `copy_` kernel is left alone -
// the dispatcher already routes a mixed CPU/webgpu copy_ to the PrivateUse1 kernel.
#include <ATen/NativeFunctions.h>
#include <torch/library.h>

#include "twg_host.h"

namespace torch_webgpu {
namespace ops {

static c10::DeviceIndex dev_of(const at::Tensor& t) {
  return t.device().index() < 0 ? core::current_device() : t.device().index();
}

static void device_strided_copy(at::Tensor& dst, const at::Tensor& src) {
  at::TensorIteratorConfig config;
  config.set_check_mem_overlap(true);
  config.add_output(dst);
  config.add_const_input(src);
  config.check_all_same_dtype(true);
  config.check_all_same_device(true);
  auto iter = config.build();
  if (iter.numel() == 0) return;
  const c10::DeviceIndex dev = dev_of(dst);
  core::DeviceScope scope(dev);
  TwgIterDesc desc = desc_from_iter(iter);
  TWG_TORCH_CHECK(twg_copy_strided(&desc, static_cast<int>(dst.dtype().itemsize()), iter.data_ptr(1), iter.data_ptr(0),
                                   core::current_stream(dev)));
}

static void host_to_device(at::Tensor& dst, const at::Tensor& src, bool non_blocking) {
  at::Tensor host = src;
  if (host.scalar_type() != dst.scalar_type()) host = host.to(dst.scalar_type());
  if (!host.sizes().equals(dst.sizes())) host = host.expand(dst.sizes());
  host = host.contiguous();
  const c10::DeviceIndex dev = dev_of(dst);
  core::DeviceScope scope(dev);
  void* stream = core::current_stream(dev);
  const size_t nbytes = static_cast<size_t>(host.numel()) * host.dtype().itemsize();
  if (nbytes == 0) return;
  if (dst.is_contiguous()) {
    TWG_TORCH_CHECK(twg_memcpy_h2d(dst.data_ptr(), host.const_data_ptr(), nbytes, stream));
  } else {
    at::Tensor staged = at::empty(dst.sizes(), dst.options());
    TWG_TORCH_CHECK(twg_memcpy_h2d(staged.data_ptr(), host.const_data_ptr(), nbytes, stream));
    device_strided_copy(dst, staged);
  }
  // A pinned source is read by the DMA engine after the library call returns; a blocking copy_
  // must have consumed its source, so wait unless the caller asked for non_blocking.
  if (!non_blocking) TWG_TORCH_CHECK(twg_stream_sync(stream));
}

static void device_to_host(at::Tensor& dst, const at::Tensor& src, bool non_blocking) {
  const c10::DeviceIndex dev = dev_of(src);
  core::DeviceScope scope(dev);
  void* stream = core::current_stream(dev);
  at::Tensor dense = src;
  if (!dense.sizes().equals(dst.sizes())) dense = dense.expand(dst.sizes());
  if (!dense.is_contiguous()) {
    at::Tensor tmp = at::empty(dense.sizes(), src.options());
    device_strided_copy(tmp, dense);
    dense = tmp;
  }
  const size_t nbytes = static_cast<size_t>(dense.numel()) * dense.dtype().itemsize();
  if (nbytes == 0) return;
  if (dst.is_contiguous() && dst.scalar_type() == src.scalar_type()) {
    // non_blocking only takes effect for pinned destinations; the library blocks for pageable ones
    TWG_TORCH_CHECK(twg_memcpy_d2h(dst.data_ptr(), dense.const_data_ptr(), nbytes, stream, non_blocking ? 0 : 1));
  } else {
    at::Tensor host = at::empty(dense.sizes(), dst.options().dtype(src.scalar_type()).memory_format(c10::MemoryFormat::Contiguous));
    TWG_TORCH_CHECK(twg_memcpy_d2h(host.data_ptr(), dense.const_data_ptr(), nbytes, stream, 1));
    dst.copy_(host);
  }
}

static int twg_dtype(at::ScalarType t) {
  switch (t) {
    case at::kByte: return TWG_DTYPE_U8;
    case at::kChar: return TWG_DTYPE_I8;
    case at::kShort: return TWG_DTYPE_I16;
    case at::kInt: return TWG_DTYPE_I32;
    case at::kLong: return TWG_DTYPE_I64;
    case at::kHalf: return TWG_DTYPE_F16;
    case at::kBFloat16: return TWG_DTYPE_BF16;
    case at::kFloat: return TWG_DTYPE_F32;
    case at::kDouble: return TWG_DTYPE_F64;
    case at::kBool: return TWG_DTYPE_BOOL;
    default: return -1;
  }
}

// dst = src with an element-type conversion, any layouts, both on one device
static void device_convert(at::Tensor& dst, const at::Tensor& src) {
  const int st = twg_dtype(src.scalar_type()), dt = twg_dtype(dst.scalar_type());
  TORCH_CHECK(st >= 0 && dt >= 0, "torch_webgpu: copy_ cannot convert ", src.scalar_type(), " to ", dst.scalar_type());
  at::TensorIteratorConfig config;
  config.set_check_mem_overlap(true).check_all_same_dtype(false).promote_inputs_to_common_dtype(false);
  config.cast_common_dtype_to_outputs(false).resize_outputs(false);
  config.add_output(dst).add_const_input(src);
  auto iter = config.build();
  if (iter.numel() == 0) return;
  const c10::DeviceIndex dev = dev_of(dst);
  core::DeviceScope scope(dev);
  TwgIterDesc desc = desc_from_iter(iter);
  TWG_TORCH_CHECK(twg_convert(&desc, st, dt, iter.data_ptr(1), iter.data_ptr(0), core::current_stream(dev)));
}

static void device_to_device(at::Tensor& dst, const at::Tensor& src) {
  if (dst.scalar_type() != src.scalar_type()) {
    if (dev_of(dst) == dev_of(src)) {
      device_convert(dst, src);
    } else {  // move first, convert where the result lives
      at::Tensor landed = at::empty(src.sizes(), dst.options().dtype(src.scalar_type()));
      device_to_device(landed, src);
      device_convert(dst, landed);
    }
    return;
  }
  if (dev_of(dst) != dev_of(src)) {
    at::Tensor dense = src.contiguous();
    at::Tensor landed = at::empty(dense.sizes(), dst.options());
    const size_t nbytes = static_cast<size_t>(dense.numel()) * dense.dtype().itemsize();
    void* src_stream = core::current_stream(dev_of(src));
    void* dst_stream = core::current_stream(dev_of(dst));
    // The peer copy runs on the destination's stream.  It is ordered after the producer of `dense`
    // by an event on the source stream, and everything the source stream does afterwards (reuse of
    // the temporary `dense` once it is freed, in-place writes to `src`) is ordered after the copy
    // by a second event; neither side's host thread waits.
    // (an event belongs to the device that was current when it was created: one per side)
    void *produced = nullptr, *copied = nullptr;
    int rc;
    {
      core::DeviceScope scope(dev_of(src));
      rc = twg_event_create(&produced);
      if (rc == TWG_OK) rc = twg_event_record(produced, src_stream);
    }
    if (rc == TWG_OK) {
      core::DeviceScope scope(dev_of(dst));
      rc = twg_event_create(&copied);
      if (rc == TWG_OK) rc = twg_event_wait(produced, dst_stream);
      if (rc == TWG_OK) rc = twg_memcpy_d2d(landed.data_ptr(), dense.const_data_ptr(), nbytes, dst_stream);
      if (rc == TWG_OK) rc = twg_event_record(copied, dst_stream);
    }
    if (rc == TWG_OK) {
      core::DeviceScope scope(dev_of(src));
      rc = twg_event_wait(copied, src_stream);
    }
    // destroying a recorded event is safe: its resources are released once it has completed
    if (produced) twg_event_destroy(produced);
    if (copied) twg_event_destroy(copied);
    TWG_TORCH_CHECK(rc);
    core::DeviceScope scope(dev_of(dst));
    device_strided_copy(dst, landed);
    return;
  }
  device_strided_copy(dst, src);
}

at::Tensor& copy_(at::Tensor& self, const at::Tensor& src, bool non_blocking) {
  if (self.is_same(src)) return self;
  TORCH_CHECK(self.defined() && src.defined(), "copy_: undefined tensor");
  if (src.device().is_cpu() && self.device().is_privateuseone()) {
    host_to_device(self, src, non_blocking);
  } else if (src.device().is_privateuseone() && self.device().is_cpu()) {
    device_to_host(self, src, non_blocking);
  } else if (src.device().is_privateuseone() && self.device().is_privateuseone()) {
    device_to_device(self, src);
  } else {
    TORCH_CHECK(false, "torch_webgpu: copy_ between ", src.device(), " and ", self.device(), " is not supported");
  }
  return self;
}

at::Tensor _copy_from(const at::Tensor& self, const at::Tensor& dst, bool non_blocking) {
  at::Tensor& out = const_cast<at::Tensor&>(dst);
  copy_(out, self, non_blocking);
  return dst;
}

at::Tensor _copy_from_and_resize(const at::Tensor& self, const at::Tensor& dst) {
  dst.resize_(self.sizes());
  at::Tensor& out = const_cast<at::Tensor&>(dst);
  copy_(out, self, false);
  return dst;
}

at::Tensor to_device(const at::Tensor& self, at::Device device, at::ScalarType dtype, bool non_blocking, bool copy,
                     std::optional<c10::MemoryFormat> memory_format) {
  return at::native::to(self, device, dtype, non_blocking, copy, memory_format);
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("copy_", TORCH_FN(copy_));
  m.impl("_copy_from", TORCH_FN(_copy_from));
  m.impl("_copy_from_and_resize", TORCH_FN(_copy_from_and_resize));
  m.impl("to.device", TORCH_FN(to_device));
}

}  // namespace ops
}  // namespace torch_webgpu
