// The `webgpu::` custom-op library the compile backend's runtime calls.
//
// Schemas kept from the reference (csrc/ops/webgpu_ops.cpp:47-62): create_buffer, write_buffer,
// fused_add_relu, plus the global AutogradPrivateUse1 fallthrough.  Added for the fused-pointwise
// backend: compile_fused (SSA program -> kernel handle) and run_fused (one launch for a whole
// pointwise subgraph).
#include <torch/library.h>

#include "twg_host.h"

namespace torch_webgpu {
namespace ops {

at::Tensor create_buffer(c10::IntArrayRef size, c10::IntArrayRef stride, std::optional<at::ScalarType> dtype_opt) {
  return at::empty_strided(size, stride, at::TensorOptions().dtype(dtype_opt).device(c10::Device(c10::kPrivateUse1)));
}

at::Tensor write_buffer(at::Tensor& self, const at::Tensor& src) {
  self.copy_(src);
  return self;
}

at::Tensor fused_add_relu(const at::Tensor& self, const at::Tensor& other) {
  const auto shape = at::infer_size(self.sizes(), other.sizes());
  at::Tensor out = at::empty(shape, self.options());
  at::TensorIteratorConfig config;
  config.set_check_mem_overlap(true);
  config.add_output(out);
  config.add_const_input(self);
  config.add_const_input(other);
  config.check_all_same_dtype(true);
  auto iter = config.build();
  binary_kernel(TWG_BINARY_FUSED_ADD_RELU, iter, 1.0f);
  return out;
}

// Program encoding: four parallel lists, one entry per SSA instruction (TwgFusedInstr fields).
int64_t compile_fused(c10::IntArrayRef opcodes, c10::IntArrayRef a, c10::IntArrayRef b, c10::ArrayRef<double> imm) {
  const size_t n = opcodes.size();
  TORCH_CHECK(a.size() == n && b.size() == n && imm.size() == n, "compile_fused: the four lists must have one length");
  std::vector<TwgFusedInstr> prog(n);
  for (size_t i = 0; i < n; ++i) {
    prog[i].opcode = static_cast<int32_t>(opcodes[i]);
    prog[i].a = static_cast<int32_t>(a[i]);
    prog[i].b = static_cast<int32_t>(b[i]);
    prog[i].imm = static_cast<float>(imm[i]);
  }
  TwgFusedProgram* handle = nullptr;
  TWG_TORCH_CHECK(twg_fused_compile(prog.data(), static_cast<int>(n), &handle));
  return static_cast<int64_t>(reinterpret_cast<intptr_t>(handle));
}

int64_t fused_kind(int64_t handle) {
  int kind = 0;
  TWG_TORCH_CHECK(twg_fused_kind(reinterpret_cast<TwgFusedProgram*>(static_cast<intptr_t>(handle)), &kind));
  return kind;
}

// Inputs broadcast against each other; outputs are freshly allocated dense tensors of the
// broadcast shape with the dtypes in `out_dtypes` (float32 or bool).
std::vector<at::Tensor> run_fused(int64_t handle, at::TensorList inputs, c10::IntArrayRef out_dtypes) {
  TORCH_CHECK(!inputs.empty() && !out_dtypes.empty(), "run_fused: needs at least one input and one output");
  const c10::Device device = inputs[0].device();
  std::vector<int64_t> shape(inputs[0].sizes().begin(), inputs[0].sizes().end());
  for (size_t i = 1; i < inputs.size(); ++i) shape = at::infer_size(shape, inputs[i].sizes());
  std::vector<at::Tensor> outs;
  at::TensorIteratorConfig config;
  config.set_check_mem_overlap(true).check_all_same_dtype(false);
  for (auto dt : out_dtypes) {
    const auto st = static_cast<at::ScalarType>(dt);
    TORCH_CHECK(st == at::kFloat || st == at::kBool, "run_fused: outputs are float32 or bool");
    outs.push_back(at::empty(shape, inputs[0].options().dtype(st)));
  }
  for (auto& o : outs) config.add_output(o);
  for (const auto& in : inputs) {
    TORCH_CHECK(in.device() == device, "run_fused: inputs live on different devices");
    TORCH_CHECK(in.scalar_type() == at::kFloat || in.scalar_type() == at::kBool, "run_fused: inputs are float32 or bool");
    config.add_const_input(in);
  }
  auto iter = config.build();
  if (iter.numel() == 0) return outs;
  const c10::DeviceIndex dev = iter_device(iter);
  core::DeviceScope scope(dev);
  TwgIterDesc desc = desc_from_iter(iter);
  std::vector<void*> ptrs(iter.ntensors());
  for (int t = 0; t < iter.ntensors(); ++t) ptrs[t] = iter.data_ptr(t);
  TWG_TORCH_CHECK(twg_fused_launch(reinterpret_cast<TwgFusedProgram*>(static_cast<intptr_t>(handle)), &desc, ptrs.data(),
                                   core::current_stream(dev)));
  return outs;
}

// masked_select(inputs[src_index], program(inputs)) with the mask kept as one bit per element in
// scratch memory.  The fused path needs dense, equally shaped float32 inputs; any other case (and programs the library has
// no select form for) runs the program and masked_select one after the other - same result.
at::Tensor run_fused_select(int64_t handle, at::TensorList inputs, int64_t src_index) {
  TORCH_CHECK(!inputs.empty() && src_index >= 0 && src_index < static_cast<int64_t>(inputs.size()),
              "run_fused_select: src_index out of range");
  auto* program = reinterpret_cast<TwgFusedProgram*>(static_cast<intptr_t>(handle));
  const at::Tensor& src = inputs[src_index];
  bool dense = true;
  for (const auto& t : inputs)
    dense = dense && t.scalar_type() == at::kFloat && t.is_contiguous() && t.sizes().equals(src.sizes()) &&
            t.device() == src.device();
  const int64_t numel = src.numel();
  if (dense && numel > 0) {
    const c10::DeviceIndex dev = src.device().index() < 0 ? core::current_device() : src.device().index();
    core::DeviceScope scope(dev);
    void* stream = core::current_stream(dev);
    // one block holds the kernel's workspace and, behind it, the two result words
    const size_t ws_bytes = (twg_fused_select_workspace_bytes(numel) + 255) / 256 * 256;
    at::Tensor scratch = at::empty({static_cast<int64_t>(ws_bytes + 2 * sizeof(int64_t))}, src.options().dtype(at::kByte));
    auto* result = reinterpret_cast<int64_t*>(static_cast<char*>(scratch.data_ptr()) + ws_bytes);
    at::Tensor out = at::empty({numel}, src.options());
    std::vector<const void*> ptrs;
    for (const auto& t : inputs) ptrs.push_back(t.const_data_ptr());
    const int rc = twg_fused_select_f32(program, static_cast<int>(src_index), numel, ptrs.data(),
                                        static_cast<float*>(out.data_ptr()), result, scratch.data_ptr(), ws_bytes, stream);
    if (rc == TWG_OK) {
      int64_t host[2] = {0, 0};
      TWG_TORCH_CHECK(twg_memcpy_d2h(host, result, sizeof(host), stream, 1));
      TORCH_CHECK(host[1] == 0, "torch_webgpu: the fused select's device-side scan failed with status ", host[1]);
      if (host[0] < numel) {
        TWG_TORCH_CHECK(twg_trim(out.data_ptr(), static_cast<size_t>(host[0]) * sizeof(float)));
        out.unsafeGetTensorImpl()->set_sizes_contiguous({host[0]});
        out.storage().unsafeGetStorageImpl()->set_nbytes(static_cast<size_t>(host[0]) * sizeof(float));
      }
      return out;
    }
    TORCH_CHECK(rc == TWG_ERR_UNSUPPORTED, "torch_webgpu: ", twg_last_error());
  }
  std::vector<at::Tensor> mask = run_fused(handle, inputs, {static_cast<int64_t>(at::kBool)});
  return at::masked_select(src, mask[0]);
}

}  // namespace ops

TORCH_LIBRARY(webgpu, m) {
  m.def("create_buffer(int[] size, int[] stride, ScalarType? dtype=None) -> Tensor");
  m.def("write_buffer(Tensor self, Tensor src) -> Tensor");
  m.def("fused_add_relu(Tensor self, Tensor src) -> Tensor");
  m.def("compile_fused(int[] opcodes, int[] a, int[] b, float[] imm) -> int");
  m.def("fused_kind(int handle) -> int");
  m.def("run_fused(int handle, Tensor[] inputs, int[] out_dtypes) -> Tensor[]");
  m.def("run_fused_select(int handle, Tensor[] inputs, int src_index) -> Tensor");
}
TORCH_LIBRARY_IMPL(webgpu, PrivateUse1, m) {
  m.impl("create_buffer", TORCH_FN(ops::create_buffer));
  m.impl("write_buffer", TORCH_FN(ops::write_buffer));
  m.impl("fused_add_relu", TORCH_FN(ops::fused_add_relu));
  m.impl("run_fused", TORCH_FN(ops::run_fused));
  m.impl("run_fused_select", TORCH_FN(ops::run_fused_select));
}
TORCH_LIBRARY_IMPL(webgpu, CatchAll, m) {
  m.impl("create_buffer", TORCH_FN(ops::create_buffer));
  m.impl("compile_fused", TORCH_FN(ops::compile_fused));
  m.impl("fused_kind", TORCH_FN(ops::fused_kind));
}
TORCH_LIBRARY_IMPL(_, AutogradPrivateUse1, m) { m.fallback(torch::CppFunction::makeFallthrough()); }

}  // namespace torch_webgpu
