// Shared internals of liblogos_b200: status/error plumbing, the handle
// registry, and small device helpers.  Nothing here is part of the C ABI.
#pragma once
#include <utility>

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <string>

#include "../../include/logos_b200.h"

namespace logos {

// ---------------------------------------------------------------- errors
// Per-thread message store, read through logos_b200_last_error(); same contract as
// the reference's thread-keyed store (crates/logicaffeine_compile/src/codegen/ffi.rs:214-251).
void set_last_error(const std::string& msg);
const char* last_error_text();  // null when the calling thread has no pending message
void clear_last_error();
logos_status_t fail(logos_status_t code, const char* fmt, ...);
logos_status_t cuda_fail(cudaError_t e, const char* what);

#define LOGOS_CUDA_TRY(expr)                                            \
  do {                                                                  \
    cudaError_t _e = (expr);                                            \
    if (_e != cudaSuccess) return ::logos::cuda_fail(_e, #expr);        \
  } while (0)

#define LOGOS_TRY(expr)                                                 \
  do {                                                                  \
    logos_status_t _s = (expr);                                         \
    if (_s != LOGOS_OK) return _s;                                      \
  } while (0)

// Every extern "C" body runs inside this guard: a C++ exception never crosses
// the ABI (the reference wraps each export in catch_unwind, ffi.rs:329-345).
template <class F>
logos_status_t guarded(F&& f) {
  try {
    return f();
  } catch (const std::bad_alloc&) {
    return fail(LOGOS_MEMORY_EXHAUSTED, "host allocation failed");
  } catch (const std::exception& e) {
    return fail(LOGOS_THREAD_PANIC, "internal exception: %s", e.what());
  } catch (...) {
    return fail(LOGOS_THREAD_PANIC, "internal exception");
  }
}

// ---------------------------------------------------------------- handles
enum class ObjKind : uint32_t { DevBuf = 1, Model = 2 };

struct DevBuf {
  void*   ptr = nullptr;
  int64_t bytes = 0;
  int32_t device = 0;
};

// Registers an object and returns its id (never 0).  The id packs a slot
// counter; a freed id is never reused, so stale handles stay invalid.
logos_handle_t registry_put(ObjKind kind, void* obj);
// Looks an id up; nullptr when unknown or of another kind.
void* registry_get(logos_handle_t h, ObjKind kind);
// Removes the id and returns the object, nullptr when unknown.
void* registry_take(logos_handle_t h, ObjKind kind);

// Resolves a device buffer handle, checking that [offset, offset+need) fits.
logos_status_t buf_resolve(logos_handle_t h, int64_t offset, int64_t need, const char* name, DevBuf** out);

template <class T>
logos_status_t buf_ptr(logos_handle_t h, int64_t elems, const char* name, T** out, int32_t* device = nullptr) {
  DevBuf* b = nullptr;
  LOGOS_TRY(buf_resolve(h, 0, elems * (int64_t)sizeof(T), name, &b));
  *out = reinterpret_cast<T*>(b->ptr);
  if (device) *device = b->device;
  return LOGOS_OK;
}

// Per-device scratch the library owns, for the stand-alone operators (activation planes and
// split-K partials of logos_q8_gemm*, split-KV partials of logos_gqa_decode_attn*).  One block
// per (device, slot), shared by every caller on that device: calls that use it must be ordered
// on the GPU (one stream, or the caller's own events).  Grows on demand, outside any stream
// capture; outgrown blocks are kept until the process exits.  A model never uses it: what a
// captured decode step points at is owned by the model.
logos_status_t scratch_get(int32_t device, int slot, int64_t bytes, void** out);

int sm_count(int device);

// Per-device status word in device memory: kernels store a non-zero code when
// a bounded wait gives up.  0 = fine.
int* kernel_status_ptr(int device);
logos_status_t kernel_status_read(int device, int* out, bool clear);

// ---------------------------------------------------------------- launch helpers
logos_status_t check_launch(const char* kernel);

// Process-wide count of kernel launches by kind (read through logos_launch_counts).
enum LaunchKind : int {
  LK_GEMV = 0, LK_GEMM_TC = 1, LK_GEMM_SIMT = 2, LK_ATTN = 3, LK_ATTN_MERGE = 4, LK_ELEMWISE = 5, LK_SYNTH = 6,
  LK_KINDS = 8
};
void count_launch(int kind, int64_t n = 1);

static inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// ---------------------------------------------------------------- programmatic dependent launch
// Inside a PdlScope (the decode step opens one) kernels are launched so that the next kernel in
// the stream may start while the previous one is still running: its CTAs are scheduled, do the
// work that depends on nothing (barrier set-up, tensor-memory allocation, fetching WEIGHTS, which
// nothing in a decode step writes) and then block in pdl_wait() until the previous kernel has
// completed and its writes are visible.  The contract every kernel of the step keeps:
//   * no read or write of anything another kernel of the step writes before pdl_wait();
//   * at least the threads that do such accesses call pdl_wait(), and every path through the
//     kernel has some thread calling it (so "this kernel completed" implies "its predecessor did");
//   * pdl_trigger() after the point where a successor's CTAs may take up SM resources.
// Outside a scope the launch is an ordinary one and both calls are no-ops.
bool pdl_active();
struct PdlScope {
  bool prev;
  explicit PdlScope(bool on);
  ~PdlScope();
};

#if defined(__CUDACC__)
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_active() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#endif

}  // namespace logos
