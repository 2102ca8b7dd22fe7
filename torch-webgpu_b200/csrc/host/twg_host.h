// Shared declarations of the PyTorch-facing host layer.  Everything below this layer is reached
// through the C ABI in twg.h; nothing here touches CUDA directly.
#pragma once

#include <ATen/ATen.h>
#include <ATen/TensorIterator.h>
#include <c10/core/Allocator.h>
#include <c10/core/Stream.h>

#include "twg.h"

namespace torch_webgpu {

// Turn a C-ABI status into a c10::Error (Python RuntimeError) carrying the library's message.
#define TWG_TORCH_CHECK(expr)                                                       \
  do {                                                                              \
    const int twg_rc_ = (expr);                                                     \
    TORCH_CHECK(twg_rc_ == TWG_OK, "torch_webgpu: ", twg_last_error(), " [", #expr, " -> ", twg_rc_, "]"); \
  } while (0)

namespace core {

// Device / stream bookkeeping shared by the guard, the allocator and the ops.
c10::DeviceIndex device_count();
c10::DeviceIndex current_device();
void set_current_device(c10::DeviceIndex index);
// Thread-local current stream of `device` as an index into the library's per-device pool.
int current_stream_index(c10::DeviceIndex device);
int exchange_stream_index(c10::DeviceIndex device, int index);
// cudaStream_t (as void*) of the current stream of `device`.
void* current_stream(c10::DeviceIndex device);
void* stream_handle(c10::DeviceIndex device, int index);

c10::Allocator* getWebGPUCachingAllocator();

struct DeviceScope {
  c10::DeviceIndex prev;
  // Always re-asserts the CUDA current device: other libraries in the process (torch.cuda) may
  // have changed it behind this thread's back.
  explicit DeviceScope(c10::DeviceIndex d) : prev(current_device()) {
    if (d >= 0) set_current_device(d);
  }
  ~DeviceScope() {
    if (current_device() != prev) set_current_device(prev);
  }
};

}  // namespace core

namespace ops {

// Describe a built TensorIterator to the C ABI: operand order, shape and element strides exactly
// as the iterator reports them (dimension 0 fastest).
TwgIterDesc desc_from_iter(const at::TensorIteratorBase& iter);
// Device index all PrivateUse1 operands of the iterator live on (checked to agree).
c10::DeviceIndex iter_device(const at::TensorIteratorBase& iter);
// Replace CPU scalar operands (wrapped numbers) by one-element device tensors.
at::Tensor to_device_if_cpu_scalar(const at::Tensor& t, c10::Device device, at::ScalarType dtype);

void unary_kernel(int op, at::TensorIteratorBase& iter);
void binary_kernel(int op, at::TensorIteratorBase& iter, const at::Scalar& alpha);

}  // namespace ops
}  // namespace torch_webgpu
