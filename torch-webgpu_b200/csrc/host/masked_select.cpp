// masked_select / masked_select.out under PrivateUse1.  The reference boxes this op to
// at::native::cpu_fallback (csrc/bindings.cpp:42): two device->host copies, the CPU kernel, one
// host->device copy.  Here it is one compaction kernel; the only host round trip is the 16-byte
// read-back of the element count that sizes the result.
#include <torch/library.h>

#include "twg_host.h"

namespace torch_webgpu {
namespace ops {

// Describe self and mask over their broadcast shape in logical row-major order (dimension 0 of
// the descriptor = last logical dimension).  Nothing is reordered, so the output order is the
// order torch.masked_select defines.
static TwgIterDesc rowmajor_desc(c10::IntArrayRef shape, const at::Tensor& self, const at::Tensor& mask) {
  TORCH_CHECK(shape.size() <= TWG_MAX_DIMS, "torch_webgpu: masked_select supports at most ", TWG_MAX_DIMS,
              " dimensions, got ", shape.size());
  TwgIterDesc d;
  std::memset(&d, 0, sizeof(d));
  d.ndim = static_cast<int32_t>(shape.size());
  d.ntensors = 2;
  d.numel = 1;
  const at::Tensor ops[2] = {self.expand(shape), mask.expand(shape)};
  for (int k = 0; k < d.ndim; ++k) {
    const int64_t dim = d.ndim - 1 - k;
    d.shape[k] = shape[dim];
    d.numel *= shape[dim];
    for (int t = 0; t < 2; ++t) d.strides[t][k] = shape[dim] == 1 ? 0 : ops[t].stride(dim);
  }
  return d;
}

// A permuted operand (no broadcast dimension, not contiguous) would be walked in logical order
// with one useful element per 32-byte sector.  Copying it into logical order first runs at copy
// bandwidth (the 2-D tile kernels) and lets the compaction take its dense path, which is several
// times cheaper than the sector over-fetch for anything that does not fit in L2.  Broadcast
// operands are left alone: their strided walk re-reads cached rows and materialising them would
// multiply the traffic.
static at::Tensor logical_order(const at::Tensor& t) {
  if (t.is_contiguous() || t.numel() < (1 << 16)) return t;
  for (int64_t d = 0; d < t.dim(); ++d)
    if (t.size(d) > 1 && t.stride(d) == 0) return t;
  return t.contiguous();
}

// Runs the compaction into `out_storage` (room for numel elements) and returns the count.
static int64_t run_masked_select(const at::Tensor& self_in, const at::Tensor& mask_in, at::Tensor& out_storage,
                                 c10::IntArrayRef shape) {
  const at::Tensor self = logical_order(self_in), mask = logical_order(mask_in);
  const c10::DeviceIndex dev = self.device().index() < 0 ? core::current_device() : self.device().index();
  core::DeviceScope scope(dev);
  void* stream = core::current_stream(dev);
  TwgIterDesc desc = rowmajor_desc(shape, self, mask);
  // one block holds the kernel's workspace and, behind it, the two result words
  const size_t ws_bytes = (twg_masked_select_workspace_bytes(desc.numel) + 255) / 256 * 256;
  at::Tensor scratch = at::empty({static_cast<int64_t>(ws_bytes + 2 * sizeof(int64_t))}, self.options().dtype(at::kByte));
  auto* result = reinterpret_cast<int64_t*>(static_cast<char*>(scratch.data_ptr()) + ws_bytes);
  TWG_TORCH_CHECK(twg_masked_select_f32(&desc, static_cast<const float*>(self.const_data_ptr()),
                                        static_cast<const uint8_t*>(mask.const_data_ptr()),
                                        static_cast<float*>(out_storage.data_ptr()), result, scratch.data_ptr(), ws_bytes,
                                        stream));
  int64_t host[2] = {0, 0};
  TWG_TORCH_CHECK(twg_memcpy_d2h(host, result, sizeof(host), stream, 1));
  TORCH_CHECK(host[1] == 0, "torch_webgpu: masked_select's device-side scan failed with status ", host[1],
              host[1] == TWG_ERR_TIMEOUT ? " (a tile gave up waiting for its predecessors)" : "");
  return host[0];
}

static void check_args(const at::Tensor& self, const at::Tensor& mask) {
  TORCH_CHECK(mask.scalar_type() == at::kBool, "masked_select: expected BoolTensor for mask");
  TORCH_CHECK(self.scalar_type() == at::kFloat, "torch_webgpu: masked_select supports float32 tensors only, got ",
              self.scalar_type());
  TORCH_CHECK(self.device() == mask.device(), "masked_select: expected self and mask to be on the same device, but got mask on ",
              mask.device(), " and self on ", self.device());
}

at::Tensor masked_select(const at::Tensor& self, const at::Tensor& mask) {
  check_args(self, mask);
  const auto shape = at::infer_size(self.sizes(), mask.sizes());
  int64_t numel = 1;
  for (auto s : shape) numel *= s;
  if (numel == 0) return at::empty({0}, self.options());
  // Worst case first, then hand the unused tail of the block back to the allocator.
  at::Tensor out = at::empty({numel}, self.options());
  const int64_t k = run_masked_select(self, mask, out, shape);
  if (k < numel) {
    TWG_TORCH_CHECK(twg_trim(out.data_ptr(), static_cast<size_t>(k) * sizeof(float)));
    out.unsafeGetTensorImpl()->set_sizes_contiguous({k});
    out.storage().unsafeGetStorageImpl()->set_nbytes(static_cast<size_t>(k) * sizeof(float));
  }
  return out;
}

at::Tensor& masked_select_out(const at::Tensor& self, const at::Tensor& mask, at::Tensor& out) {
  check_args(self, mask);
  TORCH_CHECK(out.scalar_type() == self.scalar_type(), "masked_select(): self and result must have the same scalar type");
  const auto shape = at::infer_size(self.sizes(), mask.sizes());
  int64_t numel = 1;
  for (auto s : shape) numel *= s;
  if (numel == 0) {
    out.resize_({0});
    return out;
  }
  at::Tensor tmp = at::empty({numel}, self.options());
  const int64_t k = run_masked_select(self, mask, tmp, shape);
  out.resize_({k});
  out.copy_(tmp.narrow(0, 0, k));
  return out;
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("masked_select", TORCH_FN(masked_select));
  m.impl("masked_select.out", TORCH_FN(masked_select_out));
}

}  // namespace ops
}  // namespace torch_webgpu
