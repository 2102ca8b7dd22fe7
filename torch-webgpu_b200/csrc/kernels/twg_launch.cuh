// Host-side launcher for the pointwise functor kernels: lowers a TwgIterDesc to one of the three
// launch shapes of twg_pointwise.cuh and enqueues it.  The planning step works on a run-time
// operand signature so that kernels instantiated ahead of time and kernels compiled by NVRTC
// take exactly the same decisions.
#pragma once

#include <algorithm>
#include <cstdlib>

#include "twg_internal.h"
#include "twg_pointwise.cuh"

namespace twg {

// Shape chosen for a launch; twg_last_launch_path() reports it so tests can assert which kernel
// served a layout.
enum PwPath { kPathNone = 0, kPathDense = 1, kPathTile = 2, kPathStrided32 = 3, kPathStrided64 = 4 };
extern thread_local int g_last_path;

// 128-bit units a thread handles per input on the dense path.  Measured on B200 with the kernels
// of this library on random data (2^28 elements): about four 16-byte loads in flight per thread
// saturate HBM; fewer starve it (add with one unit: 6.0 TB/s instead of 7.0), more only cost
// registers and occupancy (the three-input chain with four units: 5.9 TB/s instead of 7.0).
constexpr int dense_unroll(int nin) { return nin >= 3 ? 1 : (nin == 2 ? 2 : 4); }
constexpr int kDenseUnrollBytes = 2;  // raw-byte kernels of copy.cu
constexpr int kStridedUnroll = 4;

inline bool is_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Operand signature of a pointwise kernel: outputs first, then inputs; bit set = 1-byte operand.
struct PwSig {
  int nin, nout;
  unsigned in_byte_mask, out_byte_mask;
  int nt() const { return nin + nout; }
  bool byte(int t) const { return t < nout ? (out_byte_mask >> t) & 1u : (in_byte_mask >> (t - nout)) & 1u; }
  int vec() const {
    return (in_byte_mask == ((1u << nin) - 1u) && out_byte_mask == ((1u << nout) - 1u)) ? 16 : 4;
  }
};
template <class F>
PwSig sig_of() { return PwSig{F::NIN, F::NOUT, F::kInByteMask, F::kOutByteMask}; }

struct PwPlan {
  int path = kPathNone;
  TwgIterDesc d;         // coalesced
  int64_t nunits = 0;    // dense path
  uint32_t dim1_mask = 0;
  int64_t tiles0 = 0, tiles1 = 0, sb0 = 1, ntiles = 0;
  unsigned grid = 1;
};

// Decide the launch shape.  Returns TWG_OK with plan->path == kPathNone for an empty iteration.
int plan_pointwise(const PwSig& sig, const TwgIterDesc* desc, void* const* ptrs, PwPlan* plan);
// Shared by the element-size-generic kernels in copy.cu.
bool plan_tile(const TwgIterDesc& d, int nt, int tile_edge, PwPlan* plan);
bool fits_32bit(const TwgIterDesc& d, int nt);

// `ptrs` and `four_byte` (every operand is 4 bytes wide) decide whether interior tiles may use
// 128-bit accesses; callers that leave them out get the scalar tile code.
template <int NT>
void fill_tile_desc(const PwPlan& p, TileDesc<NT>* td, void* const* ptrs = nullptr, bool four_byte = false) {
  td->shape0 = p.d.shape[0];
  td->shape1 = p.d.shape[1];
  td->tiles0 = p.tiles0;
  td->tiles1 = p.tiles1;
  td->sb0 = p.sb0;
  td->sb0_div.d = (uint32_t)p.sb0;
  make_fastdiv(td->sb0_div.d, &td->sb0_div.m, &td->sb0_div.s);
  td->ntiles = p.ntiles;
  for (int t = 0; t < NT; ++t) { td->s0[t] = p.d.strides[t][0]; td->s1[t] = p.d.strides[t][1]; }
  td->dim1_mask = p.dim1_mask;
  bool vec = four_byte && ptrs != nullptr;
  for (int t = 0; vec && t < NT; ++t) {
    const bool along1 = (p.dim1_mask >> t) & 1u;
    const i64 dense = along1 ? td->s1[t] : td->s0[t], other = along1 ? td->s0[t] : td->s1[t];
    vec = dense == 1 && other % 4 == 0 && (reinterpret_cast<uintptr_t>(ptrs[t]) & 15u) == 0;
  }
  td->vec = vec ? 1u : 0u;
}
// Grid of a tile launch: one CTA per slot, except for the pipelined kernel (a heavy one-input f32
// functor on a 128-bit capable layout), whose CTAs stay resident and walk the slots with a grid stride.
inline unsigned tile_grid(bool pipelined, bool vec, unsigned slots) {
  if (pipelined && vec) return std::min<unsigned>(slots, (unsigned)(sm_count() * kTilePersistCtas));
  return slots;
}
template <int NT>
void fill_strided_desc(const TwgIterDesc& d, StridedDesc<NT, u32>* sd) {
  sd->ndim = d.ndim;
  for (int k = 0; k < kMaxDims; ++k) {
    const uint32_t s = k < d.ndim ? (uint32_t)d.shape[k] : 1u;
    sd->shape[k].d = s;
    make_fastdiv(s, &sd->shape[k].m, &sd->shape[k].s);
    for (int t = 0; t < NT; ++t) sd->strides[t][k] = k < d.ndim ? (uint32_t)d.strides[t][k] : 0u;
  }
}
template <int NT>
void fill_strided_desc(const TwgIterDesc& d, StridedDesc<NT, u64>* sd) {
  sd->ndim = d.ndim;
  for (int k = 0; k < kMaxDims; ++k) {
    sd->shape[k] = k < d.ndim ? (u64)d.shape[k] : 1ull;
    for (int t = 0; t < NT; ++t) sd->strides[t][k] = k < d.ndim ? d.strides[t][k] : 0;
  }
}

template <class F>
int launch_pointwise(const F& f, const TwgIterDesc* desc, void* const* ptrs_in, cudaStream_t stream) {
  constexpr int NT = PwTraits<F>::NT;
  PwPlan plan;
  if (int rc = plan_pointwise(sig_of<F>(), desc, ptrs_in, &plan)) return rc;
  if (plan.path == kPathNone) return TWG_OK;
  PwPtrs<NT> ptrs;
  for (int t = 0; t < NT; ++t) ptrs.p[t] = ptrs_in[t];
  switch (plan.path) {
    case kPathDense:
      pw_contig_kernel<F, dense_unroll(F::NIN)><<<plan.grid, kBlock, 0, stream>>>(ptrs, f, plan.nunits, plan.d.numel);
      break;
    case kPathTile: {
      TileDesc<NT> td;
      fill_tile_desc<NT>(plan, &td, ptrs_in, F::kInByteMask == 0u && F::kOutByteMask == 0u);
      pw_tile_kernel<F><<<tile_grid(TilePipelined<F>::value, td.vec != 0u, plan.grid), dim3(kTileX, kPwRows), 0, stream>>>(ptrs, f, td);
      break;
    }
    case kPathStrided32: {
      StridedDesc<NT, u32> sd;
      fill_strided_desc<NT>(plan.d, &sd);
      pw_strided_kernel<F, kStridedUnroll, u32><<<plan.grid, kBlock, 0, stream>>>(ptrs, f, sd, plan.d.numel);
      break;
    }
    default: {
      StridedDesc<NT, u64> sd;
      fill_strided_desc<NT>(plan.d, &sd);
      pw_strided_kernel<F, kStridedUnroll, u64><<<plan.grid, kBlock, 0, stream>>>(ptrs, f, sd, plan.d.numel);
      break;
    }
  }
  TWG_CHECK_LAUNCH();
  g_last_path = plan.path;
  return TWG_OK;
}

}  // namespace twg
