// Host-side helpers shared by the translation units of the library: error reporting,
// launch accounting, descriptor lowering and the generic pointwise launcher.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "twg.h"

namespace twg {

// Store a formatted message for twg_last_error() on this thread and return `code`.
int set_error(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what, const char* file, int line);
void count_launch(int n = 1);
// NVTX range around a C-ABI call, emitted only while tracing is on (twg_set_tracing / TWG_NVTX=1):
// a profiler's timeline then shows which library call every kernel and copy belongs to.
struct TraceRange {
  bool active;
  explicit TraceRange(const char* name);
  ~TraceRange();
  TraceRange(const TraceRange&) = delete;
  TraceRange& operator=(const TraceRange&) = delete;
};
#define TWG_TRACE(name) ::twg::TraceRange twg_trace_range_(name)
// Properties of the current device (cached per ordinal).
int sm_count();

#define TWG_CUDA(expr)                                                          \
  do {                                                                          \
    cudaError_t twg_e_ = (expr);                                                \
    if (twg_e_ != cudaSuccess) return ::twg::cuda_fail(twg_e_, #expr, __FILE__, __LINE__); \
  } while (0)

#define TWG_CHECK_LAUNCH()                                                      \
  do {                                                                          \
    cudaError_t twg_e_ = cudaGetLastError();                                    \
    if (twg_e_ != cudaSuccess) return ::twg::cuda_fail(twg_e_, "kernel launch", __FILE__, __LINE__); \
    ::twg::count_launch();                                                      \
  } while (0)

#define TWG_REQUIRE(cond, ...)                                                  \
  do {                                                                          \
    if (!(cond)) return ::twg::set_error(TWG_ERR_INVALID, __VA_ARGS__);         \
  } while (0)

// Validate a descriptor for `ntensors` operands.
int check_desc(const TwgIterDesc* d, int ntensors);
// Largest element offset operand t can reach (strides are non-negative in TensorIterator order
// except for flipped views, which take the 64-bit path through the absolute value).
int64_t max_offset(const TwgIterDesc& d, int t);
// Settings of the look-back shared by masked_select and the fused select (masked_select.cu).
long long ms_poll_budget();
// Where the last chunk of a compaction stores this rank's {count, sequence | status} for the count
// exchange: this rank's slot of every rank's mailbox (comm.cu fills it, masked_select.cu uses it).
struct MsPublish {
  unsigned long long* slot[TWG_EXCHANGE_MAX_RANKS];
  int nranks;  // 0: no publication
  unsigned long long seq;
};
int xchg_publish_slots(void* xchg, int64_t seq, MsPublish* out);
// Second half of the fused predicate + select (masked_select.cu): compaction by a bit mask.
int ms_select_from_bits(const float* src, const unsigned* bits, float* out, int64_t n, int64_t* result_dev,
                        void* workspace, cudaStream_t s, const MsPublish& pub);
// Zero a compaction workspace prefix and the two result words with one kernel (masked_select.cu).
int ms_clear(void* workspace, size_t nbytes, int64_t* result, cudaStream_t s);
// After coalescing: every one of the first `nt` operands is one contiguous run (copy.cu).
bool all_dense(const TwgIterDesc& d, int nt);
// Host-side multiply-shift divisor for u32 numerators below 2^31.
void make_fastdiv(uint32_t d, uint32_t* m, uint32_t* s);

}  // namespace twg
