// Python module torch_webgpu._C.  Loading it runs the static registrations of this extension:
// the PrivateUse1 device guard and allocator (core.cpp) and every TORCH_LIBRARY_IMPL block.  The
// reference's module is empty (csrc/bindings.cpp:46-58); this one also exposes what the
// `torch.webgpu` device module needs on current PyTorch (device count / selection, synchronise,
// allocator statistics) as plain functions.  No GPU work happens at import time.
#include <torch/extension.h>

#include "twg_host.h"

namespace py = pybind11;
using namespace torch_webgpu;

static py::dict memory_stats(int device) {
  TwgMemStats s;
  TWG_TORCH_CHECK(twg_memory_stats(device, &s));
  py::dict d;
  d["allocated_bytes"] = s.allocated_bytes;
  d["reserved_bytes"] = s.reserved_bytes;
  d["peak_allocated_bytes"] = s.peak_allocated_bytes;
  d["peak_reserved_bytes"] = s.peak_reserved_bytes;
  d["num_allocs"] = s.num_allocs;
  d["num_cache_hits"] = s.num_cache_hits;
  d["num_device_mallocs"] = s.num_device_mallocs;
  d["num_device_frees"] = s.num_device_frees;
  return d;
}

PYBIND11_MODULE(_C, m) {
  m.doc() = "torch_webgpu native extension (PrivateUse1 backend over the twg C ABI)";
  m.def("device_count", []() { return static_cast<int>(core::device_count()); });
  m.def("current_device", []() { return static_cast<int>(core::current_device()); });
  m.def("set_device", [](int d) { core::set_current_device(static_cast<c10::DeviceIndex>(d)); });
  m.def("synchronize", [](int d) { TWG_TORCH_CHECK(twg_device_sync(d < 0 ? core::current_device() : d)); },
        py::arg("device") = -1, py::call_guard<py::gil_scoped_release>());
  m.def("current_stream_handle", [](int d) {
    const c10::DeviceIndex dev = d < 0 ? core::current_device() : static_cast<c10::DeviceIndex>(d);
    return reinterpret_cast<uintptr_t>(core::current_stream(dev));
  }, py::arg("device") = -1);
  m.def("current_stream_index", [](int d) {
    return core::current_stream_index(d < 0 ? core::current_device() : static_cast<c10::DeviceIndex>(d));
  }, py::arg("device") = -1);
  m.def("memory_stats", &memory_stats, py::arg("device") = 0);
  m.def("reset_peak_memory_stats", [](int d) { TWG_TORCH_CHECK(twg_reset_peak_stats(d)); }, py::arg("device") = 0);
  m.def("empty_cache", []() { TWG_TORCH_CHECK(twg_empty_cache(-1)); });
  m.def("set_memory_budget", [](int d, size_t bytes) { TWG_TORCH_CHECK(twg_set_memory_budget(d, bytes)); });
  m.def("launch_count", []() { return twg_launch_count(); });
  m.def("reset_launch_count", []() { twg_reset_launch_count(); });
  m.def("last_launch_path", []() { return twg_last_launch_path(); });
  m.def("set_nvrtc_path", [](const std::string& p) { TWG_TORCH_CHECK(twg_fused_set_nvrtc_path(p.c_str())); });
  m.def("masked_select_set_poll_budget", [](int64_t polls) { TWG_TORCH_CHECK(twg_masked_select_set_poll_budget(polls)); });
  m.def("version", []() { return std::string(twg_version()); });
}
