// Runtime half of the C ABI: status and last-error store, handle registry,
// device buffers.  Mirrors the behaviour of the reference's generated preamble
// (crates/logicaffeine_compile/src/codegen/ffi.rs:190-327): thread-keyed error
// text, ids instead of addresses, invalid ids reported instead of dereferenced.
#include "common.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace logos {

namespace {
thread_local std::string t_error;
thread_local bool t_has_error = false;

struct Entry {
  ObjKind kind;
  void*   obj;
};
std::mutex g_reg_mu;
std::unordered_map<uint64_t, Entry> g_reg;
uint64_t g_counter = 0;

struct Scratch {
  void*   ptr = nullptr;
  int64_t bytes = 0;
  std::vector<void*> retired;  // outgrown blocks: kept, since launches already enqueued may still use them
};
std::mutex g_scratch_mu;
std::unordered_map<uint64_t, Scratch> g_scratch;
}  // namespace

void set_last_error(const std::string& msg) {
  t_error = msg;
  t_has_error = true;
}
const char* last_error_text() { return t_has_error ? t_error.c_str() : nullptr; }
void clear_last_error() {
  t_has_error = false;
  t_error.clear();
}

logos_status_t fail(logos_status_t code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  set_last_error(buf);
  return code;
}

logos_status_t cuda_fail(cudaError_t e, const char* what) {
  logos_status_t code = (e == cudaErrorMemoryAllocation) ? LOGOS_MEMORY_EXHAUSTED : LOGOS_ERROR;
  return fail(code, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

static std::atomic<int64_t> g_launches[LK_KINDS];
void count_launch(int kind, int64_t n) { g_launches[kind].fetch_add(n, std::memory_order_relaxed); }

thread_local bool g_pdl = false;
bool pdl_active() { return g_pdl; }
PdlScope::PdlScope(bool on) : prev(g_pdl) { g_pdl = on; }
PdlScope::~PdlScope() { g_pdl = prev; }

logos_status_t check_launch(const char* kernel) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(LOGOS_ERROR, "launch of %s failed: %s", kernel, cudaGetErrorString(e));
  return LOGOS_OK;
}

logos_handle_t registry_put(ObjKind kind, void* obj) {
  std::lock_guard<std::mutex> lk(g_reg_mu);
  uint64_t id = ++g_counter;
  g_reg[id] = Entry{kind, obj};
  return reinterpret_cast<logos_handle_t>(static_cast<uintptr_t>(id));
}

void* registry_get(logos_handle_t h, ObjKind kind) {
  std::lock_guard<std::mutex> lk(g_reg_mu);
  auto it = g_reg.find(static_cast<uint64_t>(reinterpret_cast<uintptr_t>(h)));
  if (it == g_reg.end() || it->second.kind != kind) return nullptr;
  return it->second.obj;
}

void* registry_take(logos_handle_t h, ObjKind kind) {
  std::lock_guard<std::mutex> lk(g_reg_mu);
  auto it = g_reg.find(static_cast<uint64_t>(reinterpret_cast<uintptr_t>(h)));
  if (it == g_reg.end() || it->second.kind != kind) return nullptr;
  void* obj = it->second.obj;
  g_reg.erase(it);
  return obj;
}

logos_status_t buf_resolve(logos_handle_t h, int64_t offset, int64_t need, const char* name, DevBuf** out) {
  if (h == nullptr) return fail(LOGOS_NULL_POINTER, "%s: null handle", name);
  DevBuf* b = static_cast<DevBuf*>(registry_get(h, ObjKind::DevBuf));
  if (!b) return fail(LOGOS_INVALID_HANDLE, "%s: invalid or freed device-buffer handle", name);
  if (offset < 0 || need < 0 || offset > b->bytes || need > b->bytes - offset)
    return fail(LOGOS_OUT_OF_BOUNDS, "%s: needs bytes [%lld,%lld) but the buffer holds %lld", name,
                (long long)offset, (long long)(offset + need), (long long)b->bytes);
  *out = b;
  return LOGOS_OK;
}

logos_status_t scratch_get(int32_t device, int slot, int64_t bytes, void** out) {
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  uint64_t key = (static_cast<uint64_t>(static_cast<uint32_t>(device)) << 8) | static_cast<uint64_t>(slot);
  Scratch& s = g_scratch[key];
  if (s.bytes < bytes) {
    int prev = 0;
    LOGOS_CUDA_TRY(cudaGetDevice(&prev));
    LOGOS_CUDA_TRY(cudaSetDevice(device));
    // An outgrown block is never freed: kernels already enqueued (on any stream) may still
    // write to it.  Growing at least geometrically bounds what the retired blocks hold to the
    // size of the live one.
    int64_t want = bytes > 2 * s.bytes ? bytes : 2 * s.bytes;
    want = (want + 255) & ~int64_t(255);
    void* fresh = nullptr;
    cudaError_t e = cudaMalloc(&fresh, want);
    if (e != cudaSuccess && want > bytes) {  // no room for the doubled block: take what is needed
      cudaGetLastError();
      want = (bytes + 255) & ~int64_t(255);
      e = cudaMalloc(&fresh, want);
    }
    if (e != cudaSuccess) {
      cudaSetDevice(prev);
      return cuda_fail(e, "cudaMalloc (library scratch)");
    }
    if (s.ptr) s.retired.push_back(s.ptr);
    s.ptr = fresh;
    s.bytes = want;
    LOGOS_CUDA_TRY(cudaSetDevice(prev));
  }
  *out = s.ptr;
  return LOGOS_OK;
}

int sm_count(int device) {
  static std::mutex mu;
  static std::unordered_map<int, int> cache;
  std::lock_guard<std::mutex> lk(mu);
  auto it = cache.find(device);
  if (it != cache.end()) return it->second;
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
  cache[device] = n;
  return n;
}

}  // namespace logos

using namespace logos;

extern "C" {

const char* logos_b200_last_error(void) { return last_error_text(); }
const char* logos_b200_get_last_error(void) { return last_error_text(); }
void logos_b200_clear_error(void) { clear_last_error(); }
// Strings handed out with ownership would come from malloc; none is handed out today.
void logos_b200_free_string(char* str) { free(str); }
uint32_t logos_b200_abi_version(void) { return LOGOS_ABI_VERSION; }
const char* logos_b200_version(void) { return "0.2.0-b200"; }

// The reference preamble's names, for hosts that do not define them themselves.  Weak: a LOGOS
// program that links this library statically keeps its own definitions without a clash.
#define LOGOS_WEAK __attribute__((weak, visibility("default")))
LOGOS_WEAK const char* logos_last_error(void) { return last_error_text(); }
LOGOS_WEAK const char* logos_get_last_error(void) { return last_error_text(); }
LOGOS_WEAK void logos_clear_error(void) { clear_last_error(); }
LOGOS_WEAK void logos_free_string(char* str) { free(str); }
LOGOS_WEAK uint32_t logos_abi_version(void) { return LOGOS_ABI_VERSION; }
LOGOS_WEAK const char* logos_version(void) { return logos_b200_version(); }

int32_t logos_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

logos_status_t logos_launch_counts(int64_t* out8) {
  if (!out8) return fail(LOGOS_NULL_POINTER, "logos_launch_counts: out is null");
  for (int i = 0; i < LK_KINDS; ++i) out8[i] = g_launches[i].load(std::memory_order_relaxed);
  return LOGOS_OK;
}

logos_status_t logos_dev_alloc(int64_t bytes, int32_t device, logos_handle_t* out) {
  return guarded([&]() -> logos_status_t {
    if (!out) return fail(LOGOS_NULL_POINTER, "logos_dev_alloc: out is null");
    *out = nullptr;
    if (bytes < 0) return fail(LOGOS_OUT_OF_BOUNDS, "logos_dev_alloc: negative size");
    int n = logos_device_count();
    if (n == 0) return fail(LOGOS_ERROR, "logos_dev_alloc: no CUDA device (this library has no CPU path)");
    if (device < 0 || device >= n) return fail(LOGOS_OUT_OF_BOUNDS, "logos_dev_alloc: device %d of %d", device, n);
    LOGOS_CUDA_TRY(cudaSetDevice(device));
    DevBuf* b = new DevBuf();
    b->bytes = bytes;
    b->device = device;
    if (bytes > 0) {
      cudaError_t e = cudaMalloc(&b->ptr, static_cast<size_t>(bytes));
      if (e != cudaSuccess) {
        delete b;
        return cuda_fail(e, "cudaMalloc");
      }
    }
    *out = registry_put(ObjKind::DevBuf, b);
    return LOGOS_OK;
  });
}

logos_status_t logos_dev_upload(logos_handle_t dst, int64_t dst_offset, const void* src_host, int64_t bytes) {
  return guarded([&]() -> logos_status_t {
    if (!src_host && bytes > 0) return fail(LOGOS_NULL_POINTER, "logos_dev_upload: src_host is null");
    DevBuf* b = nullptr;
    LOGOS_TRY(buf_resolve(dst, dst_offset, bytes, "logos_dev_upload dst", &b));
    if (bytes == 0) return LOGOS_OK;
    LOGOS_CUDA_TRY(cudaSetDevice(b->device));
    LOGOS_CUDA_TRY(cudaMemcpy(static_cast<char*>(b->ptr) + dst_offset, src_host, bytes, cudaMemcpyHostToDevice));
    return LOGOS_OK;
  });
}

logos_status_t logos_dev_download(void* dst_host, logos_handle_t src, int64_t src_offset, int64_t bytes) {
  return guarded([&]() -> logos_status_t {
    if (!dst_host && bytes > 0) return fail(LOGOS_NULL_POINTER, "logos_dev_download: dst_host is null");
    DevBuf* b = nullptr;
    LOGOS_TRY(buf_resolve(src, src_offset, bytes, "logos_dev_download src", &b));
    if (bytes == 0) return LOGOS_OK;
    LOGOS_CUDA_TRY(cudaSetDevice(b->device));
    LOGOS_CUDA_TRY(cudaMemcpy(dst_host, static_cast<char*>(b->ptr) + src_offset, bytes, cudaMemcpyDeviceToHost));
    return LOGOS_OK;
  });
}

logos_status_t logos_dev_memset(logos_handle_t dst, int32_t byte_value, int64_t bytes) {
  return guarded([&]() -> logos_status_t {
    DevBuf* b = nullptr;
    LOGOS_TRY(buf_resolve(dst, 0, bytes, "logos_dev_memset dst", &b));
    if (bytes == 0) return LOGOS_OK;
    LOGOS_CUDA_TRY(cudaSetDevice(b->device));
    LOGOS_CUDA_TRY(cudaMemset(b->ptr, byte_value, bytes));
    return LOGOS_OK;
  });
}

logos_status_t logos_dev_ptr(logos_handle_t h, void** out_ptr, int64_t* out_bytes) {
  return guarded([&]() -> logos_status_t {
    if (!out_ptr) return fail(LOGOS_NULL_POINTER, "logos_dev_ptr: out_ptr is null");
    DevBuf* b = nullptr;
    LOGOS_TRY(buf_resolve(h, 0, 0, "logos_dev_ptr", &b));
    *out_ptr = b->ptr;
    if (out_bytes) *out_bytes = b->bytes;
    return LOGOS_OK;
  });
}

logos_status_t logos_dev_mem_info(int32_t device, int64_t* free_out, int64_t* total_out) {
  return guarded([&]() -> logos_status_t {
    int n = logos_device_count();
    if (device < 0 || device >= n) return fail(LOGOS_OUT_OF_BOUNDS, "logos_dev_mem_info: device %d of %d", device, n);
    LOGOS_CUDA_TRY(cudaSetDevice(device));
    size_t f = 0, t = 0;
    LOGOS_CUDA_TRY(cudaMemGetInfo(&f, &t));
    if (free_out) *free_out = (int64_t)f;
    if (total_out) *total_out = (int64_t)t;
    return LOGOS_OK;
  });
}

logos_status_t logos_dev_sync(int32_t device) {
  return guarded([&]() -> logos_status_t {
    int n = logos_device_count();
    if (device < 0 || device >= n) return fail(LOGOS_OUT_OF_BOUNDS, "logos_dev_sync: device %d of %d", device, n);
    LOGOS_CUDA_TRY(cudaSetDevice(device));
    LOGOS_CUDA_TRY(cudaDeviceSynchronize());
    return LOGOS_OK;
  });
}

logos_status_t logos_dev_free(logos_handle_t h) {
  return guarded([&]() -> logos_status_t {
    if (!h) return fail(LOGOS_NULL_POINTER, "logos_dev_free: null handle");
    DevBuf* b = static_cast<DevBuf*>(registry_take(h, ObjKind::DevBuf));
    if (!b) return fail(LOGOS_INVALID_HANDLE, "logos_dev_free: invalid or already freed handle");
    if (b->ptr) {
      cudaSetDevice(b->device);
      cudaFree(b->ptr);
    }
    delete b;
    return LOGOS_OK;
  });
}

}  // extern "C"

// Opens (on != 0) or closes a dependent-launch scope for the calling thread's later operator
// calls; returns the previous setting through prev_out when that is not null.
extern "C" logos_status_t logos_dependent_launch_scope(int32_t on, int32_t* prev_out) {
  return logos::guarded([&]() -> logos_status_t {
    if (prev_out) *prev_out = logos::g_pdl ? 1 : 0;
    logos::g_pdl = on != 0;
    return LOGOS_OK;
  });
}
