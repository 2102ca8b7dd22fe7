// Core runtime objects PyTorch needs from a PrivateUse1 backend: the allocator and the device
// guard.  They replace the reference's csrc/core/webgpu_allocator.{h,cpp} (one wgpu::Buffer per
// tensor, "not really caching, yet") and csrc/core/webgpu_device_guard.{h,cpp} (one device, one
// default stream) with thin shims over the library's stream-ordered caching allocator, its
// per-device stream pool and CUDA events.
#include <c10/core/impl/DeviceGuardImplInterface.h>
#include <c10/macros/Macros.h>

#include <array>

#include "twg_host.h"

namespace torch_webgpu {
namespace core {

constexpr int kMaxDevices = 64;

static thread_local c10::DeviceIndex tl_device = 0;
static thread_local std::array<int8_t, kMaxDevices> tl_stream = {};

c10::DeviceIndex device_count() {
  int n = 0;
  TWG_TORCH_CHECK(twg_device_count(&n));
  return static_cast<c10::DeviceIndex>(n);
}

c10::DeviceIndex current_device() { return tl_device; }

void set_current_device(c10::DeviceIndex index) {
  TORCH_CHECK(index >= 0, "torch_webgpu: negative device index ", static_cast<int>(index));
  TWG_TORCH_CHECK(twg_set_device(index));
  tl_device = index;
}

int current_stream_index(c10::DeviceIndex device) {
  TORCH_CHECK(device >= 0 && device < kMaxDevices, "torch_webgpu: device index out of range");
  return tl_stream[device];
}

int exchange_stream_index(c10::DeviceIndex device, int index) {
  TORCH_CHECK(device >= 0 && device < kMaxDevices, "torch_webgpu: device index out of range");
  TORCH_CHECK(index >= 0 && index < TWG_NUM_STREAMS, "torch_webgpu: stream id ", index, " out of range");
  const int prev = tl_stream[device];
  tl_stream[device] = static_cast<int8_t>(index);
  return prev;
}

void* stream_handle(c10::DeviceIndex device, int index) {
  void* s = nullptr;
  TWG_TORCH_CHECK(twg_get_stream(device, index, &s));
  return s;
}

void* current_stream(c10::DeviceIndex device) { return stream_handle(device, current_stream_index(device)); }

// ------------------------------------------------------------------------------------------
// allocator: DataPtr{data, ctx=data, deleter, Device(PrivateUse1, index)} over twg_malloc.
// The data pointer is a real device address (the reference stores a host-side handle,
// webgpu_allocator.h:9-13), so ops read it directly and views are plain pointer arithmetic.
// ------------------------------------------------------------------------------------------
static void WebGPUCachingDeleter(void* ptr) {
  if (ptr) twg_free(ptr);  // never throws; a failure here can only be a double free
}

struct WebGPUCachingAllocator final : public c10::Allocator {
  c10::DataPtr allocate(size_t nbytes) override {
    const c10::DeviceIndex dev = current_device();
    if (nbytes == 0) return {nullptr, nullptr, &WebGPUCachingDeleter, c10::Device(c10::DeviceType::PrivateUse1, dev)};
    void* p = nullptr;
    TWG_TORCH_CHECK(twg_malloc(&p, nbytes, dev, current_stream(dev)));
    return {p, p, &WebGPUCachingDeleter, c10::Device(c10::DeviceType::PrivateUse1, dev)};
  }
  c10::DeleterFnPtr raw_deleter() const override { return &WebGPUCachingDeleter; }
  void copy_data(void* dest, const void* src, std::size_t count) const override {
    const c10::DeviceIndex dev = current_device();
    TWG_TORCH_CHECK(twg_memcpy_d2d(dest, src, count, current_stream(dev)));
  }
};

c10::Allocator* getWebGPUCachingAllocator() {
  static WebGPUCachingAllocator allocator;
  return &allocator;
}
REGISTER_ALLOCATOR(c10::DeviceType::PrivateUse1, getWebGPUCachingAllocator());

// ------------------------------------------------------------------------------------------
// device guard
// ------------------------------------------------------------------------------------------
struct WebGPUGuardImpl final : public c10::impl::DeviceGuardImplInterface {
  static constexpr c10::DeviceType static_type = c10::DeviceType::PrivateUse1;
  WebGPUGuardImpl() = default;
  explicit WebGPUGuardImpl(c10::DeviceType t) { TORCH_INTERNAL_ASSERT(t == static_type); }

  c10::DeviceType type() const override { return static_type; }
  c10::Device exchangeDevice(c10::Device d) const override {
    const c10::Device old = getDevice();
    if (d.index() != old.index()) setDevice(d);
    return old;
  }
  c10::Device getDevice() const override { return c10::Device(static_type, current_device()); }
  void setDevice(c10::Device d) const override {
    TORCH_INTERNAL_ASSERT(d.type() == static_type);
    set_current_device(d.index() < 0 ? 0 : d.index());
  }
  void uncheckedSetDevice(c10::Device d) const noexcept override {
    const c10::DeviceIndex i = d.index() < 0 ? 0 : d.index();
    if (twg_set_device(i) == TWG_OK) tl_device = i;
  }
  c10::DeviceIndex deviceCount() const noexcept override {
    int n = 0;
    return twg_device_count(&n) == TWG_OK ? static_cast<c10::DeviceIndex>(n) : 0;
  }

  static c10::Stream make_stream(c10::DeviceIndex dev, int index) {
    return c10::Stream(c10::Stream::UNSAFE, c10::Device(static_type, dev), static_cast<c10::StreamId>(index));
  }
  static c10::DeviceIndex index_of(c10::Device d) { return d.index() < 0 ? current_device() : d.index(); }
  static void* native(const c10::Stream& s) {
    return stream_handle(s.device_index() < 0 ? current_device() : s.device_index(), static_cast<int>(s.id()));
  }

  c10::Stream getStream(c10::Device d) const override {
    const c10::DeviceIndex dev = index_of(d);
    return make_stream(dev, current_stream_index(dev));
  }
  c10::Stream getDefaultStream(c10::Device d) const override { return make_stream(index_of(d), 0); }
  c10::Stream getStreamFromGlobalPool(c10::Device d, bool /*isHighPriority*/ = false) const override {
    return getNewStream(d, 0);
  }
  c10::Stream getNewStream(c10::Device d, int /*priority*/ = 0) const override {
    // round-robin over the spare streams of the pool (indices 2..)
    static std::atomic<unsigned> next{0};
    const int index = 2 + static_cast<int>(next.fetch_add(1) % (TWG_NUM_STREAMS - 2));
    return make_stream(index_of(d), index);
  }
  c10::Stream exchangeStream(c10::Stream s) const override {
    const c10::DeviceIndex dev = s.device_index() < 0 ? current_device() : s.device_index();
    const int prev = exchange_stream_index(dev, static_cast<int>(s.id()));
    return make_stream(dev, prev);
  }
  void* getStreamNativeHandle(const c10::Stream s) const override { return native(s); }

  void destroyEvent(void* event, const c10::DeviceIndex /*device_index*/) const noexcept override {
    if (event) twg_event_destroy(event);
  }
  void record(void** event, const c10::Stream& stream, const c10::DeviceIndex device_index,
              const c10::EventFlag /*flag*/) const override {
    TORCH_CHECK(device_index == -1 || device_index == stream.device_index(), "Event device index ",
                static_cast<int>(device_index), " does not match recording stream's device index ",
                static_cast<int>(stream.device_index()), ".");
    DeviceScope scope(stream.device_index());
    if (*event == nullptr) TWG_TORCH_CHECK(twg_event_create(event));
    TWG_TORCH_CHECK(twg_event_record(*event, native(stream)));
  }
  void block(void* event, const c10::Stream& stream) const override {
    if (!event) return;
    DeviceScope scope(stream.device_index());
    TWG_TORCH_CHECK(twg_event_wait(event, native(stream)));
  }
  bool queryEvent(void* event) const override {
    if (!event) return true;
    int done = 0;
    TWG_TORCH_CHECK(twg_event_query(event, &done));
    return done != 0;
  }
  bool queryStream(const c10::Stream& stream) const override {
    int done = 0;
    TWG_TORCH_CHECK(twg_stream_query(native(stream), &done));
    return done != 0;
  }
  void synchronizeStream(const c10::Stream& stream) const override { TWG_TORCH_CHECK(twg_stream_sync(native(stream))); }
  void synchronizeEvent(void* event) const override {
    if (event) TWG_TORCH_CHECK(twg_event_sync(event));
  }
  void synchronizeDevice(const c10::DeviceIndex device_index) const override {
    TWG_TORCH_CHECK(twg_device_sync(device_index < 0 ? current_device() : device_index));
  }
  void recordDataPtrOnStream(const c10::DataPtr& data_ptr, const c10::Stream& stream) const override {
    if (data_ptr.get()) TWG_TORCH_CHECK(twg_record_stream(data_ptr.get(), native(stream)));
  }
  double elapsedTime(void* event1, void* event2, const c10::DeviceIndex /*device_index*/) const override {
    float ms = 0.f;
    TWG_TORCH_CHECK(twg_event_elapsed_ms(event1, event2, &ms));
    return static_cast<double>(ms);
  }
};

C10_REGISTER_GUARD_IMPL(PrivateUse1, WebGPUGuardImpl);

}  // namespace core
}  // namespace torch_webgpu
