/*
 * twg.h - C ABI of the B200 (sm_100a) data-parallel op path behind torch-webgpu's
 * PrivateUse1 operator interface.
 *
 * Every entry point is extern "C", takes plain pointers and sizes, returns an int
 * status (TWG_OK == 0, negative == TwgStatus error), never throws, never aborts and
 * never blocks the host unless its comment says "blocks".  twg_last_error() returns
 * a thread-local message for the most recent failing call on the calling thread.
 *
 * Each declaration names the reference interface (path inside the torch-webgpu
 * project : line) that it replaces.  The reference reaches its GPU through two
 * launcher templates, binary_kernel<Op>(iter, alpha) and unary_kernel<Op>(iter)
 * (csrc/ops/binary.h:29-30, csrc/ops/unary.h:30-31), an allocator
 * (csrc/core/webgpu_allocator.h:17) and Queue.WriteBuffer / CopyBufferToBuffer /
 * MapAsync calls in csrc/ops/copy.cpp; this header is what a foreign-function
 * binding for that path would bind instead.
 *
 * Conventions
 *   - "stream" is a cudaStream_t passed as void*; NULL is the legacy default stream.
 *   - Device pointers must belong to the device that is current on the calling
 *     thread (twg_set_device), except for twg_malloc which takes the ordinal.
 *   - bool tensors are arrays of bytes holding exactly 0x00 or 0x01.
 */
#ifndef TWG_H_
#define TWG_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TWG_MAX_DIMS 8      /* same limit as the reference (csrc/ops/binary.h:105-106) */
#define TWG_MAX_TENSORS 8   /* operands of one pointwise launch: outputs first, then inputs */

typedef enum TwgStatus {
  TWG_OK = 0,
  TWG_ERR_INVALID = -1,      /* bad argument (null pointer, ndim > 8, unknown op ...) */
  TWG_ERR_CUDA = -2,         /* a CUDA runtime/driver call failed; see twg_last_error() */
  TWG_ERR_OOM = -3,          /* device allocation failed even after emptying the cache */
  TWG_ERR_TIMEOUT = -4,      /* a bounded device-side wait gave up (masked_select look-back) */
  TWG_ERR_UNSUPPORTED = -5,  /* valid request that this build has no kernel for */
  TWG_ERR_INJECTED = -6      /* host-side fault injection hook fired (tests only) */
} TwgStatus;

/* ------------------------------------------------------------------------------------------
 * Iteration descriptor.  Same information the reference packs into its `Params` uniform
 * (csrc/ops/binary.h:108-124, csrc/ops/unary.h:88-101) but 64-bit, in ELEMENTS, and passed
 * by value to the kernel.  Dimension 0 varies fastest (at::TensorIterator order).
 * strides[t][d] is operand t's stride along dimension d; operands are ordered outputs
 * first, then inputs, matching iter.tensor(i).  A stride of 0 broadcasts.  Data pointers
 * handed to the entry points already include the tensor's storage offset.
 * ---------------------------------------------------------------------------------------- */
typedef struct TwgIterDesc {
  int32_t ndim;      /* 0..TWG_MAX_DIMS; 0 with numel==1 is a scalar */
  int32_t ntensors;  /* number of operand rows of `strides` that are valid */
  int64_t numel;     /* product of shape[0..ndim) */
  int64_t shape[TWG_MAX_DIMS];
  int64_t strides[TWG_MAX_TENSORS][TWG_MAX_DIMS];
} TwgIterDesc;

/* Fill `d` for `ntensors` dense 1-D operands of `numel` elements. */
int twg_iter_contiguous(TwgIterDesc* d, int ntensors, int64_t numel);
/* Merge adjacent dimensions that every operand walks as one dense run and drop size-1
 * dimensions, preserving element order (what at::TensorIterator::coalesce_dimensions does
 * before the reference reads iter.shape()/strides(), csrc/ops/binary.h:43-47). */
int twg_iter_coalesce(TwgIterDesc* d);

/* ---- library / device / stream (replaces WebGPUContext, csrc/core/webgpu_context.cpp:9-68,
 *      and the guard's device bookkeeping, csrc/core/webgpu_device_guard.cpp:9-49) -------- */
const char* twg_last_error(void);
const char* twg_version(void);
int twg_device_count(int* count);
int twg_set_device(int device);
int twg_get_device(int* device);
/* Per-device stream pool.  index 0 is the device's compute stream, 1 its copy stream,
 * 2..TWG_NUM_STREAMS-1 spare streams handed out by the guard's getNewStream. */
#define TWG_NUM_STREAMS 8
int twg_get_stream(int device, int index, void** stream);
int twg_stream_sync(void* stream);           /* blocks */
int twg_device_sync(int device);             /* blocks */
int twg_stream_query(void* stream, int* done);
/* events (c10::DeviceGuardImplInterface record/block/queryEvent; the reference has none) */
int twg_event_create(void** event);
int twg_event_destroy(void* event);
int twg_event_record(void* event, void* stream);
int twg_event_wait(void* event, void* stream);       /* stream waits; host does not */
int twg_event_query(void* event, int* done);
int twg_event_sync(void* event);                     /* blocks */
int twg_event_elapsed_ms(void* start, void* stop, float* ms);

/* ---- caching allocator (replaces WebGPUAllocator::allocate / WebGPUCachingAllocator,
 *      csrc/core/webgpu_allocator.cpp:10-49, which creates one wgpu::Buffer per tensor) ---- */
typedef struct TwgMemStats {
  int64_t allocated_bytes;      /* bytes in live blocks */
  int64_t reserved_bytes;       /* bytes obtained from cudaMalloc and still held */
  int64_t peak_allocated_bytes;
  int64_t peak_reserved_bytes;
  int64_t num_allocs;           /* twg_malloc calls served */
  int64_t num_cache_hits;       /* ... of which from the free lists */
  int64_t num_device_mallocs;   /* cudaMalloc calls */
  int64_t num_device_frees;     /* cudaFree calls */
} TwgMemStats;
int twg_malloc(void** ptr, size_t nbytes, int device, void* stream);  /* nbytes==0 -> *ptr=NULL */
int twg_free(void* ptr);                                   /* NULL is a no-op */
int twg_record_stream(void* ptr, void* stream);            /* block is also in use on `stream` */
int twg_trim(void* ptr, size_t new_nbytes);                /* give the tail of a block back */
int twg_block_size(void* ptr, size_t* nbytes, int* device);
int twg_empty_cache(int device);                           /* device < 0: all devices; blocks */
int twg_memory_stats(int device, TwgMemStats* stats);
int twg_reset_peak_stats(int device);
/* Debugging aid (the pool offers no memory checker): while enabled, every block allocated from then
 * on carries at least 512 guard bytes behind the caller's, filled with a pattern.
 * twg_check_guard_words (blocks: synchronises the device, reads every live guarded block's guard)
 * reports how many blocks have had their guard overwritten and the lowest such block's address.
 * A write that lands in the guard stays inside the block, so nothing faults.  Off by default. */
int twg_set_guard_words(int enabled);
int twg_check_guard_words(int device, int64_t* corrupted_blocks, void** first_block);
/* Host-side fault injection for tests: cap on reserved bytes per device (0 = no cap). */
int twg_set_memory_budget(int device, size_t max_reserved_bytes);

/* ---- copies (replaces Queue.WriteBuffer, copy.cpp:90; CopyBufferToBuffer, copy.cpp:113-120;
 *      the MapAsync read-back, copy.cpp:27-55) ---------------------------------------------- */
/* Host -> device.  Pinned sources are one cudaMemcpyAsync; pageable sources are staged through
 * a ring of pinned buffers and the call returns once the source has been consumed. */
int twg_memcpy_h2d(void* dst_dev, const void* src_host, size_t nbytes, void* stream);
/* Device -> host.  If `blocking` is non-zero, or the destination is pageable, the call returns
 * after the bytes are in `dst_host` (blocks); otherwise it is a single cudaMemcpyAsync. */
int twg_memcpy_d2h(void* dst_host, const void* src_dev, size_t nbytes, void* stream, int blocking);
int twg_memcpy_d2d(void* dst_dev, const void* src_dev, size_t nbytes, void* stream);
int twg_memset(void* dst_dev, int value, size_t nbytes, void* stream);
int twg_host_alloc_pinned(void** ptr, size_t nbytes);
int twg_host_free_pinned(void* ptr);
/* Strided / broadcasting device copy of `itemsize`-byte elements (1, 2, 4, 8 or 16).
 * Replaces unary_kernel<UnaryOp::Copy> (csrc/ops/copy.cpp:123-134, unary.cpp:88).
 * desc operands: [0] = out, [1] = in. */
int twg_copy_strided(const TwgIterDesc* desc, int itemsize, const void* in, void* out, void* stream);

/* fill_.Scalar / zero_ for any dtype: every element of `out` becomes the low `itemsize` bytes
 * (1, 2, 4 or 8) of `pattern`, i.e. the value's bit pattern in the tensor's dtype.  The reference
 * has no fill: its tensors are born uninitialised (csrc/ops/basic.cpp:51-96) and are written by
 * Queue.WriteBuffer from a host copy (copy.cpp:90).  desc operands: [0]=out. */
int twg_fill(const TwgIterDesc* desc, int itemsize, uint64_t pattern, void* out, void* stream);

/* ---- pointwise kernels ------------------------------------------------------------------- */
typedef enum TwgUnaryOp {
  TWG_UNARY_COPY = 0,       /* unary.cpp:88  */
  TWG_UNARY_RELU = 1,       /* unary.cpp:91  */
  TWG_UNARY_GELU_TANH = 2,  /* unary.cpp:94 (the only GELU the reference computes) */
  TWG_UNARY_SILU = 3,       /* unary.cpp:97  */
  TWG_UNARY_GELU_ERF = 4,   /* approximate='none'; the reference ignores the argument
                               (activation_functions.cpp:56) and its tests compare against
                               the erf form (tests/ops/test_gelu.py:11-14) */
  TWG_UNARY_ABS = 5         /* CPU fallback in the reference (bindings.cpp:35) */
} TwgUnaryOp;
typedef enum TwgBinaryOp {
  TWG_BINARY_ADD = 0,             /* out = a + alpha*b, one rounding (binary.cpp:97) */
  TWG_BINARY_MUL = 1,             /* binary.cpp:100 */
  TWG_BINARY_FUSED_ADD_RELU = 2,  /* binary.cpp:103 */
  TWG_BINARY_DIV = 3              /* true division, IEEE round-to-nearest; unchecked in the
                                     reference's op list (README.md:106-114) */
} TwgBinaryOp;
typedef enum TwgCompareOp { TWG_CMP_EQ = 0, TWG_CMP_NE = 1, TWG_CMP_LT = 2, TWG_CMP_LE = 3,
                            TWG_CMP_GT = 4, TWG_CMP_GE = 5 } TwgCompareOp;

/* unary_kernel<Op>(iter) (csrc/ops/unary.h:30-181).  desc operands: [0]=out, [1]=in. */
int twg_unary_f32(int op, const TwgIterDesc* desc, const float* in, float* out, void* stream);
/* binary_kernel<Op>(iter, alpha) (csrc/ops/binary.h:29-215).  desc: [0]=out, [1]=a, [2]=b. */
int twg_binary_f32(int op, const TwgIterDesc* desc, const float* a, const float* b, float alpha,
                   float* out, void* stream);
/* Element types of twg_convert (the ten dtypes the copy path moves). */
typedef enum TwgDtype {
  TWG_DTYPE_U8 = 0, TWG_DTYPE_I8 = 1, TWG_DTYPE_I16 = 2, TWG_DTYPE_I32 = 3, TWG_DTYPE_I64 = 4,
  TWG_DTYPE_F16 = 5, TWG_DTYPE_BF16 = 6, TWG_DTYPE_F32 = 7, TWG_DTYPE_F64 = 8, TWG_DTYPE_BOOL = 9
} TwgDtype;
/* out[i] = (dst type)in[i] with C++ static_cast rules (what ATen's copy kernel applies); floats
 * to float16 / bfloat16 round to nearest even.  The reference has no conversion: its copies
 * assert float32 (csrc/ops/copy.cpp:22).  desc operands: [0]=out, [1]=in, strides in elements of
 * each operand's own type. */
int twg_convert(const TwgIterDesc* desc, int src_dtype, int dst_dtype, const void* in, void* out, void* stream);

/* where.self and masked_fill.Scalar: unchecked entries of the reference's op list
 * (README.md:128-166), no kernel there.  cond / mask are bool bytes (non-zero = true).
 * twg_where_f32:       desc operands [0]=out, [1]=cond, [2]=a, [3]=b;  out = cond ? a : b.
 * twg_masked_fill_f32: desc operands [0]=out, [1]=self, [2]=mask;      out = mask ? value : self
 *                      (out may be self itself: in-place masked_fill_). */
int twg_where_f32(const TwgIterDesc* desc, const uint8_t* cond, const float* a, const float* b, float* out,
                  void* stream);
int twg_masked_fill_f32(const TwgIterDesc* desc, const float* self, const uint8_t* mask, float value,
                        float* out, void* stream);
/* The binary ops with a scalar right operand (add.Scalar, mul.Scalar, ... reach the reference's
 * add / mul stubs as 0-dim tensors, csrc/ops/arithmetic.cpp:413-417).  desc: [0]=out, [1]=a;
 * out = a + alpha*scalar, a * scalar, relu(a + scalar), a / scalar. */
int twg_binary_scalar_f32(int op, const TwgIterDesc* desc, const float* a, float scalar, float alpha,
                          float* out, void* stream);
/* eq.Tensor / ne.Scalar ..., CPU fallbacks in the reference (csrc/bindings.cpp:36-39).
 * b == NULL compares against `scalar`; then desc has operands [0]=out, [1]=a only,
 * otherwise [0]=out, [1]=a, [2]=b.  out is bool bytes. */
int twg_compare_f32(int op, const TwgIterDesc* desc, const float* a, const float* b, float scalar,
                    uint8_t* out, void* stream);
/* bitwise_and.Tensor(_out), CPU fallback in the reference (csrc/bindings.cpp:40-41).
 * itemsize 1 with is_bool != 0 is logical and of bool bytes; itemsize 1/2/4/8 otherwise is the
 * integer bitwise and.  desc: [0]=out, [1]=a, [2]=b. */
int twg_bitwise_and(const TwgIterDesc* desc, int itemsize, int is_bool, const void* a, const void* b,
                    void* out, void* stream);

/* ---- masked_select, CPU fallback in the reference (csrc/bindings.cpp:42) ------------------
 * Single-pass stream compaction.  desc describes the BROADCAST shape in logical row-major
 * order reversed (dimension 0 = last logical dimension, fastest): operand [0] = src strides,
 * [1] = mask strides (0 where broadcast).  out receives the selected values in row-major order
 * and must have room for desc->numel elements.  result_dev points at two int64 on the device:
 * [0] = number of selected elements, [1] = TwgStatus of the device-side scan (TWG_ERR_TIMEOUT
 * if the bounded look-back wait gave up).  workspace must hold at least
 * twg_masked_select_workspace_bytes(numel) bytes, 256-byte aligned; the call clears it. */
size_t twg_masked_select_workspace_bytes(int64_t numel);
int twg_masked_select_f32(const TwgIterDesc* desc, const float* src, const uint8_t* mask, float* out,
                          int64_t* result_dev, void* workspace, size_t workspace_bytes, void* stream);
/* No counterpart in the reference.  masked_select for callers that cannot allocate device memory
 * and therefore have no workspace to hand to twg_masked_select_f32: a host framework whose own
 * allocator owns the whole device and rejects a foreign cudaMalloc, a plugin that receives input
 * and output buffers and nothing else, a latency-critical loop that must stay clear of
 * cudaMalloc's implicit synchronisation.  The scratch is a fixed array inside the library image
 * (about 513 KB of every GPU that loads the library, held until the process exits), sized for at
 * most twg_masked_select_static_max_numel() = 2^28 broadcast elements; larger requests fail with
 * TWG_ERR_UNSUPPORTED and a message naming the limit.  The call allocates nothing (no cudaMalloc,
 * no cudaFree, no allocating library routine); inputs, `out` (room for numel elements) and
 * `result_dev` (two int64) still come from the caller, with the same meaning as above.
 * The first call on a device looks up the array's device address; make that first call outside
 * any stream capture.  All calls on a device share the one array, which keeps the previous
 * call's contents: each call clears what it needs on `stream` before its kernel, so calls that
 * are ordered on the GPU are fine, while two calls that can overlap on the GPU (different
 * streams without a dependency, different host threads) race on it and corrupt each other. */
int64_t twg_masked_select_static_max_numel(void);
int twg_masked_select_f32_static(const TwgIterDesc* desc, const float* src, const uint8_t* mask, float* out,
                                 int64_t* result_dev, void* stream);
/* Test hook for the bounded wait.  polls > 0: every look-back wait gives up after `polls` polls.
 * polls < 0: additionally the first tile never publishes its count (a flag nothing sets), so the
 * tiles that depend on it run out of polls after |polls| and result[1] becomes TWG_ERR_TIMEOUT;
 * the kernel still terminates and the context stays usable.  0 restores the default budget. */
int twg_masked_select_set_poll_budget(int64_t polls);

/* ---- fused pointwise programs for the torch.compile backend ---------------------------------
 * Replaces the reference's FX -> HighIR -> LowIR -> RUN_SHADER lowering whose only fusion is
 * ADD,RELU -> webgpu::fused_add_relu (python/torch_webgpu/compiler/high_ir.py:108-120,
 * lowering.py:36-48).  A program is a straight-line SSA list over f32 / bool values; value i
 * is the result of instruction i. */
typedef enum TwgFusedOpcode {
  TWG_F_INPUT_F32 = 0,   /* a = input slot                      -> f32  */
  TWG_F_INPUT_BOOL = 1,  /* a = input slot                      -> bool */
  TWG_F_CONST_F32 = 2,   /* imm                                 -> f32  */
  TWG_F_ADD = 3,         /* v[a] + imm*v[b], one rounding       -> f32  */
  TWG_F_MUL = 4,         /* v[a] * v[b]                         -> f32  */
  TWG_F_RELU = 5,
  TWG_F_SILU = 6,
  TWG_F_GELU_ERF = 7,
  TWG_F_GELU_TANH = 8,
  TWG_F_ABS = 9,
  TWG_F_EQ = 10,         /* v[a] == v[b]                        -> bool */
  TWG_F_NE = 11,
  TWG_F_LT = 12,
  TWG_F_LE = 13,
  TWG_F_GT = 14,
  TWG_F_GE = 15,
  TWG_F_AND = 16,        /* bool & bool                         -> bool */
  TWG_F_OUTPUT = 17      /* store v[a] to output slot b (f32 or bool by v[a]'s type) */
} TwgFusedOpcode;
typedef struct TwgFusedInstr {
  int32_t opcode;
  int32_t a;
  int32_t b;
  float imm;
} TwgFusedInstr;
typedef struct TwgFusedProgram TwgFusedProgram;  /* opaque */
/* Build (or fetch from the cache) the kernel for `prog`.  Programs that match a kernel
 * instantiated ahead of time in the library are served from it; others are generated from the
 * same C++ templates and compiled for sm_100a with NVRTC on first use (blocks). */
int twg_fused_compile(const TwgFusedInstr* prog, int ninstr, TwgFusedProgram** out);
/* 0 = ahead-of-time instantiation, 1 = NVRTC. */
int twg_fused_kind(const TwgFusedProgram* p, int* kind);
/* desc operands: outputs (slot order) first, then inputs (slot order).  ptrs likewise. */
int twg_fused_launch(const TwgFusedProgram* p, const TwgIterDesc* desc, void* const* ptrs, void* stream);
/* Drops one reference; the last one unloads the program's modules (blocks until the devices that
 * ran it are idle) and frees it.  A handle must not be used after its release. */
int twg_fused_release(TwgFusedProgram* p);
/* Fused predicate + select: out = inputs[src_input][ prog(inputs) ], for a program that is a
 * predicate (exactly one bool output over dense f32 inputs of `numel` elements each, 16-byte
 * aligned).  Two launches: the predicate kernel reads every input once and writes ONE BIT per
 * element into the workspace, and the compaction reads those bits and src and writes only the
 * selected values - instead of the fused kernel writing a byte mask and masked_select (CPU
 * fallback in the reference, csrc/bindings.cpp:42) reading it back: 0.25 bytes of mask traffic
 * per element rather than 2.  out, result_dev and the bounded look-back behave as in
 * twg_masked_select_f32; the workspace holds masked_select's plus the bits
 * (twg_fused_select_workspace_bytes, 256-byte aligned).
 * TWG_ERR_UNSUPPORTED (program is not a predicate, an input is misaligned) means: run
 * twg_fused_launch followed by twg_masked_select_f32 instead. */
size_t twg_fused_select_workspace_bytes(int64_t numel);
/* The two halves on their own.  twg_fused_predicate_bits writes the predicate of `numel` elements
 * as bits (bit i of 32-bit word w = element 32 w + i; twg_predicate_bits_bytes(numel) bytes, whole
 * 16-byte vectors, zero at and beyond numel; `bits` 16-byte aligned).  twg_masked_select_bits_f32
 * is masked_select of dense, 16-byte aligned `src` by such a mask; workspace
 * (twg_masked_select_workspace_bytes(numel), 256-byte aligned) and result words as
 * twg_masked_select_f32. */
size_t twg_predicate_bits_bytes(int64_t numel);
int twg_fused_predicate_bits(const TwgFusedProgram* p, int64_t numel, const void* const* inputs, uint32_t* bits,
                             void* stream);
int twg_masked_select_bits_f32(const float* src, const uint32_t* bits, int64_t numel, float* out, int64_t* result_dev,
                               void* workspace, size_t workspace_bytes, void* stream);
int twg_fused_select_f32(const TwgFusedProgram* p, int src_input, int64_t numel, const void* const* inputs,
                         float* out, int64_t* result_dev, void* workspace, size_t workspace_bytes, void* stream);
/* Path of the NVRTC shared library to load on first use (default: the loader's search path for
 * libnvrtc.so.12, then /usr/local/cuda/lib64).  Honoured only before the first NVRTC build. */
int twg_fused_set_nvrtc_path(const char* path);
/* Directory for an on-disk cache of NVRTC results (one file per program, keyed by a hash of the
 * generated source, the device headers and the library version; written atomically, safe to share
 * between processes).  NULL or "" turns the cache off, which is the default unless TWG_CACHE_DIR
 * is set in the environment when the library is first used.  The reference compiles its WGSL on
 * every process start and keeps pipelines in a per-process map (csrc/ops/binary.cpp:23-54). */
int twg_fused_set_cache_dir(const char* dir);
/* Programs served from / added to that directory by this process. */
int twg_fused_cache_stats(int64_t* hits, int64_t* misses);
/* Generated CUDA source of a program (ahead-of-time programs report the same text NVRTC would
 * be given); the pointer stays valid until twg_fused_release. */
int twg_fused_source(const TwgFusedProgram* p, const char** source);

/* ---- the count exchange of the batch-sharded path ---------------------------------------------
 * No counterpart in the reference: it drives one device (`webgpu_device_count = 1`,
 * csrc/core/webgpu_device_guard.h:9).  When a batch is cut over several GPUs, masked_select of
 * the whole batch is the concatenation of the per-rank results in rank order, and the only thing
 * the ranks have to tell each other is how many elements each produced (one int64 + one status
 * per rank and step).  Two transports:
 *
 * (1) NCCL.  libnccl.so.2 is loaded on first use (dlopen); without it these calls return
 *     TWG_ERR_UNSUPPORTED and everything else keeps working.  The 128-byte unique id made on one
 *     rank must reach the others through the host's own channel (a file, a socket, a key-value
 *     store).  Plain ncclAllGather on the caller's stream; `n` int64 per rank. */
#define TWG_COMM_ID_BYTES 128
int twg_comm_set_nccl_path(const char* path);   /* honoured only before the first NCCL call */
int twg_comm_unique_id(void* out128);
int twg_comm_init_rank(const void* unique_id, int rank, int nranks, void** comm);  /* blocks: all ranks must call */
int twg_comm_destroy(void* comm);
int twg_allgather_i64(void* comm, const int64_t* send_dev, int64_t* recv_dev, int n, void* stream);
/* (2) Peer stores over NVLink, no library call on the step.  Every rank creates an exchange object
 *     on its device (current device of the calling thread), hands its 64-byte handle to every other
 *     rank and connects theirs (twg_exchange_connect_ipc for ranks in other processes,
 *     twg_exchange_connect_local for ranks of the same process).  Per step, with a sequence number
 *     seq = 1, 2, 3 ... that all ranks use for the same step:
 *       twg_exchange_publish(x, seq, result_dev, stream)   after masked_select on `stream`:
 *           a one-warp kernel stores {result_dev[0], seq, result_dev[1]} into this rank's slot of
 *           every rank's mailbox (plain stores to peer memory, the flag word a release store);
 *       twg_exchange_collect(x, seq, stream2)   on any stream ordered after the publish:
 *           a one-warp kernel waits until every rank's slot of the local mailbox carries `seq`
 *           (bounded: after the time limit a missing rank is reported as TWG_ERR_TIMEOUT in its
 *           status and the kernel returns), then writes counts, statuses, this rank's exclusive
 *           offset and the total to device memory (twg_exchange_gathered) and to pinned host memory;
 *       twg_exchange_wait(x, seq, counts, statuses, &offset, &total, timeout_ms)   blocks:
 *           the host polls that pinned record; returns the worst status (TWG_OK when every rank
 *           reported 0).  counts / statuses hold nranks entries; any output may be NULL.
 *     Rule for reusing mailbox slots (slot = seq % ring): publish seq only after twg_exchange_wait
 *     has returned for seq - ring/2 on this rank.  Nothing reads a peer's memory, there is no
 *     multicast and no TMA; a rank that never publishes costs the others one time limit, not a hang. */
#define TWG_EXCHANGE_HANDLE_BYTES 64
#define TWG_EXCHANGE_MAX_RANKS 16
int twg_exchange_create(int rank, int nranks, int ring, void** xchg);   /* blocks (allocates, clears) */
int twg_exchange_handle(void* xchg, void* out64);
int twg_exchange_connect_ipc(void* xchg, int peer_rank, const void* handle64);
int twg_exchange_connect_local(void* xchg, int peer_rank, void* peer_xchg);
int twg_exchange_publish(void* xchg, int64_t seq, const int64_t* result_dev, void* stream);
int twg_exchange_collect(void* xchg, int64_t seq, void* stream);
/* twg_masked_select_f32 and twg_exchange_publish as ONE call: the compaction kernel's last chunk,
 * which knows the total, stores {count, seq, status} into every rank's mailbox itself, so the
 * exchange costs no launch of its own.  (Layouts that the chunked kernel does not serve, and empty
 * inputs, get the publish kernel behind the compaction - same effect.)  Arguments as the two calls. */
int twg_masked_select_f32_publish(const TwgIterDesc* desc, const float* src, const uint8_t* mask, float* out,
                                  int64_t* result_dev, void* workspace, size_t workspace_bytes, void* xchg, int64_t seq,
                                  void* stream);
/* The same for the compaction by a bit mask and for the fused predicate + select. */
int twg_masked_select_bits_f32_publish(const float* src, const uint32_t* bits, int64_t numel, float* out,
                                       int64_t* result_dev, void* workspace, size_t workspace_bytes, void* exchange,
                                       int64_t seq, void* stream);
int twg_fused_select_f32_publish(const TwgFusedProgram* p, int src_input, int64_t numel, const void* const* inputs,
                                 float* out, int64_t* result_dev, void* workspace, size_t workspace_bytes,
                                 void* exchange, int64_t seq, void* stream);
int twg_exchange_wait(void* xchg, int64_t seq, int64_t* counts, int64_t* statuses, int64_t* offset, int64_t* total,
                      int timeout_ms);
/* Device copy of the record of `seq`: int64[2*nranks + 2] = counts, statuses, offset, total; valid
 * for work ordered after that step's twg_exchange_collect. */
int twg_exchange_gathered(void* xchg, int64_t seq, const int64_t** dev_record);
/* Time limit of the collect kernel's wait (default 2 s; <= 0 restores the default). */
int twg_exchange_set_timeout_ns(void* xchg, int64_t timeout_ns);
int twg_exchange_destroy(void* xchg);   /* blocks */

/* ---- tracing: NVTX ranges named after the entry points around the compute, copy and exchange
 *      calls, so that a profiler's timeline shows which library call a kernel or copy belongs to.
 *      Off by default (TWG_NVTX=1 in the environment turns it on at first use); without a profiler
 *      attached a range costs a function call.  The reference has no tracing. */
int twg_set_tracing(int enabled);
int twg_get_tracing(void);

/* ---- launch accounting: number of kernels this library launched on the calling thread's
 *      behalf since the last reset (all threads), used by the benchmark's gpu_launches ----- */
int64_t twg_launch_count(void);
void twg_reset_launch_count(void);
/* Launch shape the most recent pointwise / copy / masked_select call on this thread used:
 * 0 none (empty tensor), 1 dense vector path, 2 2-D permuted tile path, 3 strided 32-bit index
 * path, 4 strided 64-bit index path. */
int twg_last_launch_path(void);

#ifdef __cplusplus
}
#endif
#endif /* TWG_H_ */
