// Fused pointwise programs for the torch.compile backend.
//
// A program is a straight-line SSA list over f32 / bool values (TwgFusedInstr).  It becomes ONE
// kernel: the generated functor is plugged into the same dense / tile / strided launch shapes as
// the single ops (twg_pointwise.cuh), so intermediates live in registers and never touch HBM.
// Programs that the library instantiates ahead of time are matched by value; anything else is
// turned into a small CUDA translation unit around the same header and compiled for sm_100a with
// NVRTC on first use (loaded with the driver API, cached per device).
#include <dlfcn.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "twg_compact.cuh"
#include "twg_launch.cuh"

namespace twg {

// The text of twg_pointwise.cuh, embedded at build time for NVRTC.
static const char kPointwiseHeader[] =
#include "twg_pointwise_src.inc"
    ;
// The text of twg_compact.cuh (fused predicate + select), likewise.
static const char kCompactHeader[] =
#include "twg_compact_src.inc"
    ;

// ------------------------------------------------------------------------------------------
// program analysis
// ------------------------------------------------------------------------------------------
enum ValType { kF32 = 0, kBool = 1, kNone = 2 };

struct Analysis {
  int nin = 0, nout = 0;
  unsigned in_byte_mask = 0, out_byte_mask = 0;
  bool heavy = false;  // the program contains a transcendental activation
  std::vector<int> type;  // per instruction
  // a predicate: one bool output over f32 inputs - can drive the fused select
  bool is_predicate() const { return nout == 1 && out_byte_mask == 1u && in_byte_mask == 0u && nin >= 1; }
};

static int analyse(const TwgFusedInstr* prog, int n, Analysis* a) {
  TWG_REQUIRE(prog != nullptr && n > 0 && n <= 4096, "fused program: bad instruction count %d", n);
  a->type.assign(n, kNone);
  std::vector<int> in_seen, out_seen;
  for (int i = 0; i < n; ++i) {
    const TwgFusedInstr& I = prog[i];
    auto operand = [&](int idx, int want) -> int {
      if (idx < 0 || idx >= i || a->type[idx] == kNone)
        return set_error(TWG_ERR_INVALID, "fused program: instruction %d reads value %d which is not defined before it", i, idx);
      if (a->type[idx] != want)
        return set_error(TWG_ERR_INVALID, "fused program: instruction %d expects a %s operand", i, want == kF32 ? "f32" : "bool");
      return TWG_OK;
    };
    switch (I.opcode) {
      case TWG_F_INPUT_F32:
      case TWG_F_INPUT_BOOL: {
        TWG_REQUIRE(I.a >= 0 && I.a < TWG_MAX_TENSORS, "fused program: input slot %d out of range", I.a);
        if ((int)in_seen.size() <= I.a) in_seen.resize(I.a + 1, 0);
        TWG_REQUIRE(!in_seen[I.a], "fused program: input slot %d is declared twice", I.a);
        in_seen[I.a] = 1;
        if (I.opcode == TWG_F_INPUT_BOOL) a->in_byte_mask |= 1u << I.a;
        a->type[i] = I.opcode == TWG_F_INPUT_BOOL ? kBool : kF32;
        break;
      }
      case TWG_F_CONST_F32: a->type[i] = kF32; break;
      case TWG_F_ADD:
      case TWG_F_MUL:
        if (int rc = operand(I.a, kF32)) return rc;
        if (int rc = operand(I.b, kF32)) return rc;
        a->type[i] = kF32;
        break;
      case TWG_F_RELU:
      case TWG_F_SILU:
      case TWG_F_GELU_ERF:
      case TWG_F_GELU_TANH:
      case TWG_F_ABS:
        if (int rc = operand(I.a, kF32)) return rc;
        a->type[i] = kF32;
        if (I.opcode == TWG_F_SILU || I.opcode == TWG_F_GELU_ERF || I.opcode == TWG_F_GELU_TANH) a->heavy = true;
        break;
      case TWG_F_EQ:
      case TWG_F_NE:
      case TWG_F_LT:
      case TWG_F_LE:
      case TWG_F_GT:
      case TWG_F_GE:
        if (int rc = operand(I.a, kF32)) return rc;
        if (int rc = operand(I.b, kF32)) return rc;
        a->type[i] = kBool;
        break;
      case TWG_F_AND:
        if (int rc = operand(I.a, kBool)) return rc;
        if (int rc = operand(I.b, kBool)) return rc;
        a->type[i] = kBool;
        break;
      case TWG_F_OUTPUT: {
        TWG_REQUIRE(I.a >= 0 && I.a < i && a->type[I.a] != kNone, "fused program: output %d stores an undefined value", i);
        TWG_REQUIRE(I.b >= 0 && I.b < TWG_MAX_TENSORS, "fused program: output slot %d out of range", I.b);
        if ((int)out_seen.size() <= I.b) out_seen.resize(I.b + 1, 0);
        TWG_REQUIRE(!out_seen[I.b], "fused program: output slot %d is stored twice", I.b);
        out_seen[I.b] = 1;
        if (a->type[I.a] == kBool) a->out_byte_mask |= 1u << I.b;
        break;
      }
      default: return set_error(TWG_ERR_INVALID, "fused program: unknown opcode %d at instruction %d", I.opcode, i);
    }
  }
  for (size_t k = 0; k < in_seen.size(); ++k) TWG_REQUIRE(in_seen[k], "fused program: input slot %zu is never declared", k);
  for (size_t k = 0; k < out_seen.size(); ++k) TWG_REQUIRE(out_seen[k], "fused program: output slot %zu is never stored", k);
  a->nin = (int)in_seen.size();
  a->nout = (int)out_seen.size();
  TWG_REQUIRE(a->nout >= 1, "fused program: no output");
  TWG_REQUIRE(a->nin + a->nout <= TWG_MAX_TENSORS, "fused program: %d operands exceed the limit of %d",
              a->nin + a->nout, TWG_MAX_TENSORS);
  return TWG_OK;
}

// ------------------------------------------------------------------------------------------
// source generation
// ------------------------------------------------------------------------------------------
static std::string hexf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  char buf[48];
  snprintf(buf, sizeof(buf), "__uint_as_float(0x%08xu)", u);
  return buf;
}

static std::string generate_source(const TwgFusedInstr* prog, int n, const Analysis& a) {
  std::string s;
  char line[512];
  s += "#include \"twg_pointwise.cuh\"\nnamespace twg {\nstruct Prog {\n";
  snprintf(line, sizeof(line),
           "  static constexpr int NIN = %d, NOUT = %d;\n  static constexpr unsigned kInByteMask = %uu, kOutByteMask = %uu;\n",
           a.nin, a.nout, a.in_byte_mask, a.out_byte_mask);
  s += line;
  s += a.heavy ? "  static constexpr bool kHeavy = true;\n" : "  static constexpr bool kHeavy = false;\n";
  s += "  __device__ __forceinline__ void operator()(const u32* in, u32* out) const {\n";
  static const char* unary[] = {"f_relu", "f_silu", "f_gelu_erf", "f_gelu_tanh", "f_abs"};
  static const char* cmp[] = {"f_eq", "f_ne", "f_lt", "f_le", "f_gt", "f_ge"};
  for (int i = 0; i < n; ++i) {
    const TwgFusedInstr& I = prog[i];
    switch (I.opcode) {
      case TWG_F_INPUT_F32: snprintf(line, sizeof(line), "    const float v%d = as_f(in[%d]);\n", i, I.a); break;
      case TWG_F_INPUT_BOOL: snprintf(line, sizeof(line), "    const u32 v%d = in[%d];\n", i, I.a); break;
      case TWG_F_CONST_F32: snprintf(line, sizeof(line), "    const float v%d = %s;\n", i, hexf(I.imm).c_str()); break;
      case TWG_F_ADD:
        snprintf(line, sizeof(line), "    const float v%d = f_add(v%d, v%d, %s);\n", i, I.a, I.b, hexf(I.imm).c_str());
        break;
      case TWG_F_MUL: snprintf(line, sizeof(line), "    const float v%d = f_mul(v%d, v%d);\n", i, I.a, I.b); break;
      case TWG_F_RELU:
      case TWG_F_SILU:
      case TWG_F_GELU_ERF:
      case TWG_F_GELU_TANH:
      case TWG_F_ABS:
        snprintf(line, sizeof(line), "    const float v%d = %s(v%d);\n", i, unary[I.opcode - TWG_F_RELU], I.a);
        break;
      case TWG_F_EQ:
      case TWG_F_NE:
      case TWG_F_LT:
      case TWG_F_LE:
      case TWG_F_GT:
      case TWG_F_GE:
        snprintf(line, sizeof(line), "    const u32 v%d = %s(v%d, v%d);\n", i, cmp[I.opcode - TWG_F_EQ], I.a, I.b);
        break;
      case TWG_F_AND: snprintf(line, sizeof(line), "    const u32 v%d = f_and(v%d, v%d);\n", i, I.a, I.b); break;
      case TWG_F_OUTPUT:
        if (a.type[I.a] == kBool) snprintf(line, sizeof(line), "    out[%d] = v%d;\n", I.b, I.a);
        else snprintf(line, sizeof(line), "    out[%d] = as_u(v%d);\n", I.b, I.a);
        break;
      default: line[0] = 0;
    }
    s += line;
  }
  s += "  }\n};\n}  // namespace twg\nusing namespace twg;\n";
  snprintf(line, sizeof(line), "constexpr int NT = %d;\n", a.nin + a.nout);
  s += line;
  snprintf(line, sizeof(line),
           "extern \"C\" __global__ void __launch_bounds__(kBlock) twg_fused_dense(PwPtrs<NT> p, i64 nunits, i64 n) "
           "{ pw_contig_body<Prog, %d>(p, Prog{}, nunits, n); }\n", dense_unroll(a.nin));
  s += line;
  s += "extern \"C\" __global__ void __launch_bounds__(kTileX * kPwRows, tile_min_ctas<Prog>()) twg_fused_tile(PwPtrs<NT> p, TileDesc<NT> d) "
       "{ pw_tile_body<Prog>(p, Prog{}, d); }\n";
  snprintf(line, sizeof(line),
           "extern \"C\" __global__ void __launch_bounds__(kBlock) twg_fused_strided32(PwPtrs<NT> p, StridedDesc<NT, u32> d, i64 n) "
           "{ pw_strided_body<Prog, %d, u32>(p, Prog{}, d, n); }\n", kStridedUnroll);
  s += line;
  snprintf(line, sizeof(line),
           "extern \"C\" __global__ void __launch_bounds__(kBlock) twg_fused_strided64(PwPtrs<NT> p, StridedDesc<NT, u64> d, i64 n) "
           "{ pw_strided_body<Prog, %d, u64>(p, Prog{}, d, n); }\n", kStridedUnroll);
  s += line;
  if (a.is_predicate()) {
    s += "#include \"twg_compact.cuh\"\n";
    snprintf(line, sizeof(line),
             "extern \"C\" __global__ void __launch_bounds__(kBlock) twg_fused_bits(PwPtrs<%d> in, u32* bits, i64 n) "
             "{ predicate_bits_body<Prog>(in, Prog{}, bits, n); }\n", a.nin);
    s += line;
  }
  return s;
}

// ------------------------------------------------------------------------------------------
// programs instantiated ahead of time
// ------------------------------------------------------------------------------------------
// relu(a + b): the reference's only fusion (python/torch_webgpu/compiler/high_ir.py:108-120).
struct AotAddRelu {
  static constexpr int NIN = 2, NOUT = 1;
  static constexpr unsigned kInByteMask = 0u, kOutByteMask = 0u;
  __device__ __forceinline__ void operator()(const u32* in, u32* out) const {
    out[0] = as_u(f_relu(f_add(as_f(in[0]), as_f(in[1]), 1.0f)));
  }
};
// m = (relu(silu(a + b) + c) == 0) & (a != 0): three f32 streams in, one bool stream out.
struct AotChainMask {
  static constexpr int NIN = 3, NOUT = 1;
  static constexpr unsigned kInByteMask = 0u, kOutByteMask = 1u;
  __device__ __forceinline__ void operator()(const u32* in, u32* out) const {
    const float a = as_f(in[0]), b = as_f(in[1]), c = as_f(in[2]);
    const float y = f_relu(f_add(f_silu(f_add(a, b, 1.0f)), c, 1.0f));
    out[0] = f_and(f_eq(y, 0.0f), f_ne(a, 0.0f));
  }
};
// The same predicate, decided from a fast evaluation wherever that is provably the decision of the
// exact chain; used where only the mask is wanted as bits (predicate_bits_kernel is close to
// issue-bound with the exact chain's 46 instructions per element).
//   y == 0  <=>  silu(a + b) + c <= 0  (relu), so only the sign of q = silu(t) + c matters.
// Fast silu: ex2.approx and rcp.approx.  Error of __expf(x): 2 + 1.173 |x| ulp; of the division
// and of 1 + e: 3 ulp; the exact path's own silu: 3 ulp.  So both evaluations lie within
// 6e-8 (8 + 1.2 |t|) |s| of the true value, and when |q| exceeds twice that (plus a floor that
// covers flushed denormals) both sums have the sign of q.  Everything else - the band around
// zero, NaN, infinities (every comparison with NaN is false) - takes the exact path.
struct AotChainMaskQuick {
  static constexpr int NIN = 3, NOUT = 1;
  static constexpr unsigned kInByteMask = 0u, kOutByteMask = 1u;
  __device__ __forceinline__ void operator()(const u32* in, u32* out) const {
    const float a = as_f(in[0]), b = as_f(in[1]), c = as_f(in[2]);
    const float t = f_add(a, b, 1.0f);
    const float s = __fdividef(t, 1.0f + __expf(-t));
    const float q = s + c;
    const float band = fabsf(s) * fmaf(fabsf(t), 3.0e-7f, 2.0e-6f) + 1e-30f;
    u32 y_is_zero;
    if (fabsf(q) > band) {
      y_is_zero = q < 0.0f ? 1u : 0u;
    } else {
      const float y = f_relu(f_add(f_silu(t), c, 1.0f));
      y_is_zero = f_eq(y, 0.0f);
    }
    out[0] = f_and(y_is_zero, f_ne(a, 0.0f));
  }
};
// Same chain that also keeps y.
struct AotChainMaskY {
  static constexpr int NIN = 3, NOUT = 2;
  static constexpr unsigned kInByteMask = 0u, kOutByteMask = 2u;
  __device__ __forceinline__ void operator()(const u32* in, u32* out) const {
    const float a = as_f(in[0]), b = as_f(in[1]), c = as_f(in[2]);
    const float y = f_relu(f_add(f_silu(f_add(a, b, 1.0f)), c, 1.0f));
    out[0] = as_u(y);
    out[1] = f_and(f_eq(y, 0.0f), f_ne(a, 0.0f));
  }
};

static const TwgFusedInstr kProgAddRelu[] = {
    {TWG_F_INPUT_F32, 0, 0, 0.f}, {TWG_F_INPUT_F32, 1, 0, 0.f}, {TWG_F_ADD, 0, 1, 1.f},
    {TWG_F_RELU, 2, 0, 0.f},      {TWG_F_OUTPUT, 3, 0, 0.f}};
static const TwgFusedInstr kProgChainMask[] = {
    {TWG_F_INPUT_F32, 0, 0, 0.f}, {TWG_F_INPUT_F32, 1, 0, 0.f}, {TWG_F_INPUT_F32, 2, 0, 0.f},
    {TWG_F_ADD, 0, 1, 1.f},       {TWG_F_SILU, 3, 0, 0.f},      {TWG_F_ADD, 4, 2, 1.f},
    {TWG_F_RELU, 5, 0, 0.f},      {TWG_F_CONST_F32, 0, 0, 0.f}, {TWG_F_EQ, 6, 7, 0.f},
    {TWG_F_CONST_F32, 0, 0, 0.f}, {TWG_F_NE, 0, 9, 0.f},        {TWG_F_AND, 8, 10, 0.f},
    {TWG_F_OUTPUT, 11, 0, 0.f}};
static const TwgFusedInstr kProgChainMaskY[] = {
    {TWG_F_INPUT_F32, 0, 0, 0.f}, {TWG_F_INPUT_F32, 1, 0, 0.f}, {TWG_F_INPUT_F32, 2, 0, 0.f},
    {TWG_F_ADD, 0, 1, 1.f},       {TWG_F_SILU, 3, 0, 0.f},      {TWG_F_ADD, 4, 2, 1.f},
    {TWG_F_RELU, 5, 0, 0.f},      {TWG_F_CONST_F32, 0, 0, 0.f}, {TWG_F_EQ, 6, 7, 0.f},
    {TWG_F_CONST_F32, 0, 0, 0.f}, {TWG_F_NE, 0, 9, 0.f},        {TWG_F_AND, 8, 10, 0.f},
    {TWG_F_OUTPUT, 6, 0, 0.f},    {TWG_F_OUTPUT, 11, 1, 0.f}};

typedef int (*AotLaunch)(const TwgIterDesc*, void* const*, cudaStream_t);
template <class F>
int aot_launch(const TwgIterDesc* d, void* const* ptrs, cudaStream_t s) { return launch_pointwise(F{}, d, ptrs, s); }

// first half of the fused predicate + select: the predicate as one bit per element
static unsigned bits_grid(i64 n, int nin) {
  return (unsigned)std::min<i64>(std::max<i64>(predicate_bits_ctas(n, nin), 1), 0x7fffffff);
}
typedef int (*AotBits)(const void* const*, unsigned*, i64, cudaStream_t);
template <class F>
int aot_bits(const void* const* inputs, unsigned* bits, i64 n, cudaStream_t s) {
  PwPtrs<F::NIN> in;
  for (int k = 0; k < F::NIN; ++k) in.p[k] = const_cast<void*>(inputs[k]);
  predicate_bits_kernel<F><<<bits_grid(n, F::NIN), kBlock, 0, s>>>(in, F{}, bits, n);
  TWG_CHECK_LAUNCH();
  return TWG_OK;
}

struct AotEntry {
  const TwgFusedInstr* prog;
  int n;
  AotLaunch launch;
  AotBits bits;  // nullptr: not a predicate
};
static const AotEntry kAot[] = {
    {kProgAddRelu, (int)(sizeof(kProgAddRelu) / sizeof(TwgFusedInstr)), &aot_launch<AotAddRelu>, nullptr},
    {kProgChainMask, (int)(sizeof(kProgChainMask) / sizeof(TwgFusedInstr)), &aot_launch<AotChainMask>, &aot_bits<AotChainMaskQuick>},
    {kProgChainMaskY, (int)(sizeof(kProgChainMaskY) / sizeof(TwgFusedInstr)), &aot_launch<AotChainMaskY>, nullptr},
};

static bool same_program(const TwgFusedInstr* a, int na, const TwgFusedInstr* b, int nb) {
  if (na != nb) return false;
  for (int i = 0; i < na; ++i) {
    if (a[i].opcode != b[i].opcode) return false;
    const int op = a[i].opcode;
    const bool uses_b = op == TWG_F_ADD || op == TWG_F_MUL || (op >= TWG_F_EQ && op <= TWG_F_OUTPUT);
    const bool uses_a = op != TWG_F_CONST_F32;
    const bool uses_imm = op == TWG_F_CONST_F32 || op == TWG_F_ADD;
    if (uses_a && a[i].a != b[i].a) return false;
    if (uses_b && a[i].b != b[i].b) return false;
    if (uses_imm && memcmp(&a[i].imm, &b[i].imm, 4) != 0) return false;
  }
  return true;
}

// ------------------------------------------------------------------------------------------
// NVRTC + driver API, loaded lazily with dlopen so that the library itself has no link-time
// dependency on either (it must load on machines without a GPU driver).
// ------------------------------------------------------------------------------------------
typedef struct _nvrtcProgram* nvrtcProgram;
typedef int nvrtcResult;
typedef struct CUmod_st* CUmodule;
typedef struct CUfunc_st* CUfunction;
typedef struct CUstream_st* CUstream;
typedef int CUresult;

struct Dyn {
  std::mutex mu;
  std::string nvrtc_path;
  void* nvrtc = nullptr;
  void* cuda = nullptr;
  nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*);
  nvrtcResult (*DestroyProgram)(nvrtcProgram*);
  nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*);
  nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*);
  nvrtcResult (*GetCUBIN)(nvrtcProgram, char*);
  nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*);
  nvrtcResult (*GetProgramLog)(nvrtcProgram, char*);
  const char* (*GetErrorString)(nvrtcResult);
  CUresult (*ModuleLoadData)(CUmodule*, const void*);
  CUresult (*ModuleUnload)(CUmodule);
  CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*);
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                           void**, void**);
  CUresult (*CuGetErrorString)(CUresult, const char**);
  CUresult (*FuncSetAttribute)(CUfunction, int, int);
};
static Dyn g_dyn;

template <class T>
static bool sym(void* lib, const char* name, T* out) {
  *out = reinterpret_cast<T>(dlsym(lib, name));
  return *out != nullptr;
}

static int load_nvrtc() {
  Dyn& d = g_dyn;
  std::lock_guard<std::mutex> lock(d.mu);
  if (d.nvrtc) return TWG_OK;
  std::vector<std::string> candidates;
  if (!d.nvrtc_path.empty()) candidates.push_back(d.nvrtc_path);
  if (const char* env = getenv("TWG_NVRTC_PATH")) candidates.push_back(env);
  candidates.push_back("libnvrtc.so.12");
  candidates.push_back("/usr/local/cuda/lib64/libnvrtc.so.12");
  candidates.push_back("libnvrtc.so");
  void* lib = nullptr;
  for (const auto& c : candidates) {
    lib = dlopen(c.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (lib) break;
  }
  if (!lib) return set_error(TWG_ERR_UNSUPPORTED, "cannot load NVRTC (libnvrtc.so.12): %s", dlerror());
  bool ok = sym(lib, "nvrtcCreateProgram", &d.CreateProgram) && sym(lib, "nvrtcDestroyProgram", &d.DestroyProgram) &&
            sym(lib, "nvrtcCompileProgram", &d.CompileProgram) && sym(lib, "nvrtcGetCUBINSize", &d.GetCUBINSize) &&
            sym(lib, "nvrtcGetCUBIN", &d.GetCUBIN) && sym(lib, "nvrtcGetProgramLogSize", &d.GetProgramLogSize) &&
            sym(lib, "nvrtcGetProgramLog", &d.GetProgramLog) && sym(lib, "nvrtcGetErrorString", &d.GetErrorString);
  if (!ok) return set_error(TWG_ERR_UNSUPPORTED, "the NVRTC library lacks a required entry point");
  d.nvrtc = lib;
  return TWG_OK;
}

static int load_driver() {
  Dyn& d = g_dyn;
  std::lock_guard<std::mutex> lock(d.mu);
  if (d.cuda) return TWG_OK;
  void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_LOCAL);
  if (!lib) return set_error(TWG_ERR_CUDA, "cannot load the CUDA driver library libcuda.so.1: %s", dlerror());
  bool ok = sym(lib, "cuModuleLoadData", &d.ModuleLoadData) && sym(lib, "cuModuleUnload", &d.ModuleUnload) &&
            sym(lib, "cuModuleGetFunction", &d.ModuleGetFunction) && sym(lib, "cuLaunchKernel", &d.LaunchKernel) &&
            sym(lib, "cuGetErrorString", &d.CuGetErrorString) && sym(lib, "cuFuncSetAttribute", &d.FuncSetAttribute);
  if (!ok) return set_error(TWG_ERR_UNSUPPORTED, "the CUDA driver library lacks a required entry point");
  d.cuda = lib;
  return TWG_OK;
}

static int cu_fail(CUresult r, const char* what) {
  const char* msg = nullptr;
  if (g_dyn.CuGetErrorString) g_dyn.CuGetErrorString(r, &msg);
  return set_error(TWG_ERR_CUDA, "%s failed: %s (CUresult %d)", what, msg ? msg : "unknown", r);
}

static int nvrtc_compile(const std::string& source, std::vector<char>* cubin) {
  if (int rc = load_nvrtc()) return rc;
  Dyn& d = g_dyn;
  nvrtcProgram prog = nullptr;
  const char* headers[] = {kPointwiseHeader, kCompactHeader};
  const char* names[] = {"twg_pointwise.cuh", "twg_compact.cuh"};
  nvrtcResult r = d.CreateProgram(&prog, source.c_str(), "twg_fused.cu", 2, headers, names);
  if (r != 0) return set_error(TWG_ERR_CUDA, "nvrtcCreateProgram failed: %s", d.GetErrorString(r));
  const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo"};
  r = d.CompileProgram(prog, 3, opts);
  if (r != 0) {
    size_t n = 0;
    d.GetProgramLogSize(prog, &n);
    std::string log(n, '\0');
    if (n) d.GetProgramLog(prog, &log[0]);
    d.DestroyProgram(&prog);
    return set_error(TWG_ERR_CUDA, "NVRTC compilation failed: %s\n%.800s", d.GetErrorString(r), log.c_str());
  }
  size_t size = 0;
  r = d.GetCUBINSize(prog, &size);
  if (r == 0) {
    cubin->resize(size);
    r = d.GetCUBIN(prog, cubin->data());
  }
  d.DestroyProgram(&prog);
  if (r != 0 || size == 0) return set_error(TWG_ERR_CUDA, "NVRTC produced no cubin: %s", d.GetErrorString(r));
  return TWG_OK;
}

// ------------------------------------------------------------------------------------------
// On-disk cache of the cubins NVRTC produced.  A program's generated source includes the device
// headers only by name, so the key hashes the source text, both header texts and the library
// version; the file holds the hash key's source length, and the cubin.  Files are written to a
// temporary name and renamed, so concurrent processes (one per GPU) never see half a file.  The
// cache is off until a directory is given (twg_fused_set_cache_dir, or TWG_CACHE_DIR in the
// environment when the library is first used).
// ------------------------------------------------------------------------------------------
static std::mutex g_disk_mu;
static std::string g_disk_dir;
static bool g_disk_env_read = false;
static std::atomic<long long> g_disk_hits{0}, g_disk_misses{0};

static std::string disk_dir() {
  std::lock_guard<std::mutex> lock(g_disk_mu);
  if (!g_disk_env_read) {
    g_disk_env_read = true;
    if (g_disk_dir.empty()) {
      const char* env = getenv("TWG_CACHE_DIR");
      if (env && *env) g_disk_dir = env;
    }
  }
  return g_disk_dir;
}
static unsigned long long fnv1a(const char* data, size_t n, unsigned long long h) {
  for (size_t i = 0; i < n; ++i) {
    h ^= (unsigned char)data[i];
    h *= 1099511628211ull;
  }
  return h;
}
static std::string disk_path(const std::string& dir, const std::string& source) {
  unsigned long long h1 = 14695981039346656037ull, h2 = 0x9e3779b97f4a7c15ull;
  const char* parts[] = {source.c_str(), kPointwiseHeader, kCompactHeader, twg_version()};
  for (const char* part : parts) {
    const size_t n = strlen(part);
    h1 = fnv1a(part, n, h1);
    h2 = fnv1a(part, n, h2 ^ n);
  }
  char name[64];
  snprintf(name, sizeof(name), "/twg_%016llx%016llx.cubin", h1, h2);
  return dir + name;
}
static bool disk_load(const std::string& path, size_t source_len, std::vector<char>* cubin) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return false;
  unsigned long long head[2] = {0, 0};  // source length, cubin size
  bool ok = fread(head, sizeof(head), 1, f) == 1 && head[0] == source_len && head[1] > 0 && head[1] < (1ull << 30);
  if (ok) {
    cubin->resize((size_t)head[1]);
    ok = fread(cubin->data(), 1, cubin->size(), f) == cubin->size() && fgetc(f) == EOF;
  }
  fclose(f);
  if (!ok) cubin->clear();
  return ok;
}
static void disk_store(const std::string& path, size_t source_len, const std::vector<char>& cubin) {
  char tmp_suffix[48];
  snprintf(tmp_suffix, sizeof(tmp_suffix), ".tmp.%ld.%p", (long)getpid(), (const void*)&cubin);
  const std::string tmp = path + tmp_suffix;
  FILE* f = fopen(tmp.c_str(), "wb");
  if (!f) return;  // an unwritable directory only means: no cache
  const unsigned long long head[2] = {source_len, cubin.size()};
  const bool ok = fwrite(head, sizeof(head), 1, f) == 1 && fwrite(cubin.data(), 1, cubin.size(), f) == cubin.size();
  if (fclose(f) != 0 || !ok || rename(tmp.c_str(), path.c_str()) != 0) remove(tmp.c_str());
}
// nvrtc_compile behind the disk cache.
static int compile_cached(const std::string& source, std::vector<char>* cubin) {
  const std::string dir = disk_dir();
  if (dir.empty()) return nvrtc_compile(source, cubin);
  const std::string path = disk_path(dir, source);
  if (disk_load(path, source.size(), cubin)) {
    g_disk_hits.fetch_add(1);
    return TWG_OK;
  }
  g_disk_misses.fetch_add(1);
  if (int rc = nvrtc_compile(source, cubin)) return rc;
  disk_store(path, source.size(), *cubin);
  return TWG_OK;
}

struct DeviceModule {
  CUmodule mod = nullptr;
  CUfunction dense = nullptr, tile = nullptr, strided32 = nullptr, strided64 = nullptr;
  CUfunction bits = nullptr;  // twg_fused_bits, predicates only
};

}  // namespace twg

using namespace twg;

struct TwgFusedProgram {
  std::vector<TwgFusedInstr> prog;
  Analysis an;
  std::string source;
  int kind = 0;  // 0 ahead-of-time, 1 NVRTC
  AotLaunch aot = nullptr;
  AotBits aot_bits = nullptr;
  std::vector<char> cubin;
  std::mutex mu;
  std::map<int, DeviceModule> modules;  // per device ordinal
  int refs = 0;                         // handles handed out by twg_fused_compile and not yet released
};

namespace twg {

static int get_module(TwgFusedProgram* p, DeviceModule** out) {
  if (int rc = load_driver()) return rc;
  int dev = 0;
  TWG_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(p->mu);
  auto it = p->modules.find(dev);
  if (it == p->modules.end()) {
    TWG_CUDA(cudaFree(nullptr));  // make sure the primary context exists and is current
    DeviceModule m;
    CUresult r = g_dyn.ModuleLoadData(&m.mod, p->cubin.data());
    if (r != 0) return cu_fail(r, "cuModuleLoadData");
    struct { const char* name; CUfunction* fn; } want[] = {{"twg_fused_dense", &m.dense}, {"twg_fused_tile", &m.tile},
                                                           {"twg_fused_strided32", &m.strided32},
                                                           {"twg_fused_strided64", &m.strided64}};
    for (auto& w : want) {
      r = g_dyn.ModuleGetFunction(w.fn, m.mod, w.name);
      if (r != 0) return cu_fail(r, "cuModuleGetFunction");
    }
    if (p->an.is_predicate()) {
      r = g_dyn.ModuleGetFunction(&m.bits, m.mod, "twg_fused_bits");
      if (r != 0) return cu_fail(r, "cuModuleGetFunction");
    }
    it = p->modules.emplace(dev, m).first;
  }
  *out = &it->second;
  return TWG_OK;
}

template <int NT>
static int jit_launch(TwgFusedProgram* p, const TwgIterDesc* desc, void* const* ptrs_in, cudaStream_t stream) {
  PwSig sig{p->an.nin, p->an.nout, p->an.in_byte_mask, p->an.out_byte_mask};
  PwPlan plan;
  if (int rc = plan_pointwise(sig, desc, ptrs_in, &plan)) return rc;
  if (plan.path == kPathNone) return TWG_OK;
  DeviceModule* m = nullptr;
  if (int rc = get_module(p, &m)) return rc;
  PwPtrs<NT> ptrs;
  for (int t = 0; t < NT; ++t) ptrs.p[t] = ptrs_in[t];
  i64 n = plan.d.numel, nunits = plan.nunits;
  CUresult r;
  CUstream cs = reinterpret_cast<CUstream>(stream);
  switch (plan.path) {
    case kPathDense: {
      void* args[] = {&ptrs, &nunits, &n};
      r = g_dyn.LaunchKernel(m->dense, plan.grid, 1, 1, kBlock, 1, 1, 0, cs, args, nullptr);
      break;
    }
    case kPathTile: {
      TileDesc<NT> td;
      fill_tile_desc<NT>(plan, &td, ptrs_in, p->an.in_byte_mask == 0u && p->an.out_byte_mask == 0u);
      void* args[] = {&ptrs, &td};
      const bool pipelined = p->an.heavy && p->an.nin == 1 && p->an.in_byte_mask == 0u && p->an.out_byte_mask == 0u;  // TilePipelined<Prog>
      r = g_dyn.LaunchKernel(m->tile, tile_grid(pipelined, td.vec != 0u, plan.grid), 1, 1, kTileX, kPwRows, 1, 0, cs, args, nullptr);
      break;
    }
    case kPathStrided32: {
      StridedDesc<NT, u32> sd;
      fill_strided_desc<NT>(plan.d, &sd);
      void* args[] = {&ptrs, &sd, &n};
      r = g_dyn.LaunchKernel(m->strided32, plan.grid, 1, 1, kBlock, 1, 1, 0, cs, args, nullptr);
      break;
    }
    default: {
      StridedDesc<NT, u64> sd;
      fill_strided_desc<NT>(plan.d, &sd);
      void* args[] = {&ptrs, &sd, &n};
      r = g_dyn.LaunchKernel(m->strided64, plan.grid, 1, 1, kBlock, 1, 1, 0, cs, args, nullptr);
      break;
    }
  }
  if (r != 0) return cu_fail(r, "cuLaunchKernel");
  count_launch();
  g_last_path = plan.path;
  return TWG_OK;
}

// cache of compiled programs, keyed by generated source
static std::mutex g_cache_mu;
static std::map<std::string, TwgFusedProgram*> g_cache;

}  // namespace twg

extern "C" int twg_fused_set_nvrtc_path(const char* path) {
  std::lock_guard<std::mutex> lock(g_dyn.mu);
  g_dyn.nvrtc_path = path ? path : "";
  return TWG_OK;
}

extern "C" int twg_fused_compile(const TwgFusedInstr* prog, int ninstr, TwgFusedProgram** out) {
  TWG_TRACE("twg_fused_compile");
  TWG_REQUIRE(out != nullptr, "twg_fused_compile: null result pointer");
  *out = nullptr;
  Analysis an;
  if (int rc = analyse(prog, ninstr, &an)) return rc;
  std::string source = generate_source(prog, ninstr, an);
  std::lock_guard<std::mutex> lock(g_cache_mu);
  auto it = g_cache.find(source);
  if (it != g_cache.end()) {
    it->second->refs++;
    *out = it->second;
    return TWG_OK;
  }
  TwgFusedProgram* p = new TwgFusedProgram();
  p->prog.assign(prog, prog + ninstr);
  p->an = an;
  p->source = source;
  for (const AotEntry& e : kAot)
    if (same_program(prog, ninstr, e.prog, e.n)) { p->aot = e.launch; p->aot_bits = e.bits; break; }
  if (p->aot) {
    p->kind = 0;
  } else {
    p->kind = 1;
    if (int rc = compile_cached(source, &p->cubin)) {
      delete p;
      return rc;
    }
  }
  p->refs = 1;
  g_cache[source] = p;
  *out = p;
  return TWG_OK;
}

extern "C" int twg_fused_set_cache_dir(const char* dir) {
  std::lock_guard<std::mutex> lock(g_disk_mu);
  g_disk_env_read = true;  // an explicit setting wins over the environment
  g_disk_dir = dir ? dir : "";
  return TWG_OK;
}

extern "C" int twg_fused_cache_stats(int64_t* hits, int64_t* misses) {
  if (hits) *hits = g_disk_hits.load();
  if (misses) *misses = g_disk_misses.load();
  return TWG_OK;
}

extern "C" int twg_fused_kind(const TwgFusedProgram* p, int* kind) {
  TWG_REQUIRE(p && kind, "twg_fused_kind: null argument");
  *kind = p->kind;
  return TWG_OK;
}

extern "C" int twg_fused_source(const TwgFusedProgram* p, const char** source) {
  TWG_REQUIRE(p && source, "twg_fused_source: null argument");
  *source = p->source.c_str();
  return TWG_OK;
}

extern "C" int twg_fused_launch(const TwgFusedProgram* cp, const TwgIterDesc* desc, void* const* ptrs, void* stream) {
  TWG_TRACE("twg_fused_launch");
  TWG_REQUIRE(cp && ptrs, "twg_fused_launch: null argument");
  TwgFusedProgram* p = const_cast<TwgFusedProgram*>(cp);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p->aot) return p->aot(desc, ptrs, s);
  switch (p->an.nin + p->an.nout) {
    case 1: return jit_launch<1>(p, desc, ptrs, s);
    case 2: return jit_launch<2>(p, desc, ptrs, s);
    case 3: return jit_launch<3>(p, desc, ptrs, s);
    case 4: return jit_launch<4>(p, desc, ptrs, s);
    case 5: return jit_launch<5>(p, desc, ptrs, s);
    case 6: return jit_launch<6>(p, desc, ptrs, s);
    case 7: return jit_launch<7>(p, desc, ptrs, s);
    case 8: return jit_launch<8>(p, desc, ptrs, s);
    default: return set_error(TWG_ERR_INVALID, "twg_fused_launch: bad operand count");
  }
}

// Programs are shared through the cache and counted: every twg_fused_compile hands out one
// reference, the last twg_fused_release drops the program from the cache, waits for the devices
// that loaded its module (a kernel of it may still be running), unloads the modules and frees the
// cubin and the generated source.
extern "C" int twg_fused_release(TwgFusedProgram* p) {
  if (p == nullptr) return TWG_OK;
  {
    std::lock_guard<std::mutex> lock(g_cache_mu);
    auto it = g_cache.begin();
    for (; it != g_cache.end(); ++it)
      if (it->second == p) break;
    TWG_REQUIRE(it != g_cache.end(), "twg_fused_release: %p is not a live program handle", (void*)p);
    if (--p->refs > 0) return TWG_OK;
    g_cache.erase(it);
  }
  int rc = TWG_OK;
  if (!p->modules.empty()) {
    int prev = 0;
    cudaGetDevice(&prev);
    for (auto& kv : p->modules) {
      if (kv.second.mod == nullptr) continue;
      if (cudaSetDevice(kv.first) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        cudaGetLastError();
        rc = set_error(TWG_ERR_CUDA, "twg_fused_release: could not quiesce device %d before unloading the module", kv.first);
        continue;  // the module stays loaded rather than being pulled from under a kernel
      }
      g_dyn.ModuleUnload(kv.second.mod);
    }
    cudaSetDevice(prev);
  }
  delete p;
  return rc;
}

// ------------------------------------------------------------------------------------------
// fused predicate + select: the predicate as one bit per element, then the compaction by bits
// ------------------------------------------------------------------------------------------
namespace twg {
template <int NIN>
static int jit_bits(TwgFusedProgram* p, const void* const* inputs, unsigned* bits, i64 n, cudaStream_t stream) {
  DeviceModule* m = nullptr;
  if (int rc = get_module(p, &m)) return rc;
  PwPtrs<NIN> in;
  for (int k = 0; k < NIN; ++k) in.p[k] = const_cast<void*>(inputs[k]);
  void* args[] = {&in, &bits, &n};
  CUresult r = g_dyn.LaunchKernel(m->bits, bits_grid(n, NIN), 1, 1, kBlock, 1, 1, 0, reinterpret_cast<CUstream>(stream), args, nullptr);
  if (r != 0) return cu_fail(r, "cuLaunchKernel");
  count_launch();
  return TWG_OK;
}

// Layout of the fused select's workspace: ticket header and chunk descriptors (as masked_select's),
// rounded to 256 bytes, then the bit mask.
static size_t select_bits_offset(int64_t numel) { return (twg_masked_select_workspace_bytes(numel) + 255) / 256 * 256; }

static int predicate_bits_impl(const TwgFusedProgram* cp, int64_t numel, const void* const* inputs, unsigned* bits,
                               void* stream) {
  TWG_REQUIRE(cp && inputs, "twg_fused_predicate_bits: null argument");
  TwgFusedProgram* p = const_cast<TwgFusedProgram*>(cp);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!p->an.is_predicate())
    return set_error(TWG_ERR_UNSUPPORTED, "twg_fused_predicate_bits: the program is not a predicate (one bool output over f32 inputs)");
  TWG_REQUIRE(numel >= 0, "twg_fused_predicate_bits: negative numel");
  if (numel == 0) return TWG_OK;
  TWG_REQUIRE(bits != nullptr && is_aligned(bits, 16), "twg_fused_predicate_bits: bits is null or not 16-byte aligned");
  for (int k = 0; k < p->an.nin; ++k) {
    TWG_REQUIRE(inputs[k] != nullptr, "twg_fused_predicate_bits: input %d is null", k);
    if (!is_aligned(inputs[k], 16))
      return set_error(TWG_ERR_UNSUPPORTED, "twg_fused_predicate_bits: input %d is not 16-byte aligned", k);
  }
  TWG_REQUIRE(predicate_bits_ctas(numel, p->an.nin) <= 0x7fffffff, "twg_fused_predicate_bits: %lld elements exceed the grid limit",
              (long long)numel);
  if (p->aot_bits) return p->aot_bits(inputs, bits, numel, s);
  if (p->kind != 1)
    return set_error(TWG_ERR_UNSUPPORTED, "twg_fused_predicate_bits: this ahead-of-time program has no predicate form");
  switch (p->an.nin) {
    case 1: return jit_bits<1>(p, inputs, bits, numel, s);
    case 2: return jit_bits<2>(p, inputs, bits, numel, s);
    case 3: return jit_bits<3>(p, inputs, bits, numel, s);
    case 4: return jit_bits<4>(p, inputs, bits, numel, s);
    case 5: return jit_bits<5>(p, inputs, bits, numel, s);
    case 6: return jit_bits<6>(p, inputs, bits, numel, s);
    default: return jit_bits<7>(p, inputs, bits, numel, s);
  }
}

// Checks shared by the two forms of the fused select; *bits is where the predicate's bits go.
static int fused_select_check(const TwgFusedProgram* p, int src_input, int64_t numel, const void* const* inputs,
                              void* workspace, size_t workspace_bytes, unsigned** bits) {
  TWG_REQUIRE(p && inputs, "twg_fused_select_f32: null argument");
  if (!p->an.is_predicate())
    return set_error(TWG_ERR_UNSUPPORTED, "twg_fused_select_f32: the program is not a predicate (one bool output over f32 inputs)");
  TWG_REQUIRE(src_input >= 0 && src_input < p->an.nin, "twg_fused_select_f32: src_input %d out of range", src_input);
  TWG_REQUIRE(numel >= 0, "twg_fused_select_f32: negative numel");
  *bits = nullptr;
  if (numel == 0) return TWG_OK;
  const size_t need = twg_fused_select_workspace_bytes(numel);
  TWG_REQUIRE(workspace != nullptr && workspace_bytes >= need && is_aligned(workspace, 256),
              "twg_fused_select_f32: workspace of %zu bytes is smaller than the %zu required or not 256-byte aligned",
              workspace_bytes, need);
  *bits = reinterpret_cast<unsigned*>(static_cast<char*>(workspace) + select_bits_offset(numel));
  return TWG_OK;
}
}  // namespace twg

extern "C" int twg_fused_predicate_bits(const TwgFusedProgram* p, int64_t numel, const void* const* inputs, uint32_t* bits,
                                        void* stream) {
  TWG_TRACE("twg_fused_predicate_bits");
  return predicate_bits_impl(p, numel, inputs, bits, stream);
}

extern "C" size_t twg_fused_select_workspace_bytes(int64_t numel) {
  if (numel < 0) numel = 0;
  return select_bits_offset(numel) + (size_t)predicate_bits_bytes(numel);
}

extern "C" int twg_fused_select_f32(const TwgFusedProgram* p, int src_input, int64_t numel, const void* const* inputs,
                                    float* out, int64_t* result_dev, void* workspace, size_t workspace_bytes,
                                    void* stream) {
  TWG_TRACE("twg_fused_select_f32");
  unsigned* bits = nullptr;
  if (int rc = fused_select_check(p, src_input, numel, inputs, workspace, workspace_bytes, &bits)) return rc;
  if (int rc = predicate_bits_impl(p, numel, inputs, bits, stream)) return rc;
  return twg_masked_select_bits_f32(static_cast<const float*>(inputs[src_input]), bits, numel, out, result_dev, workspace,
                                    select_bits_offset(numel), stream);
}

extern "C" int twg_fused_select_f32_publish(const TwgFusedProgram* p, int src_input, int64_t numel,
                                            const void* const* inputs, float* out, int64_t* result_dev, void* workspace,
                                            size_t workspace_bytes, void* xchg, int64_t seq, void* stream) {
  TWG_TRACE("twg_fused_select_f32_publish");
  unsigned* bits = nullptr;
  if (int rc = fused_select_check(p, src_input, numel, inputs, workspace, workspace_bytes, &bits)) return rc;
  if (int rc = predicate_bits_impl(p, numel, inputs, bits, stream)) return rc;
  return twg_masked_select_bits_f32_publish(static_cast<const float*>(inputs[src_input]), bits, numel, out, result_dev,
                                            workspace, select_bits_offset(numel), xchg, seq, stream);
}
