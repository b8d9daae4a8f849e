// Host helpers for TMA tensor maps and the device-visible kernel status word.
#include "ptx.cuh"

#include <mutex>
#include <string>
#include <unordered_map>

namespace logos {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}
}  // namespace

logos_status_t make_tensor_map_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, uint32_t elem_bytes,
                                  uint64_t inner, uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner,
                                  uint32_t box_outer, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(LOGOS_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || (row_pitch_bytes & 15u))
    return fail(LOGOS_ERROR, "tensor map: base address and row pitch must be multiples of 16 bytes");
  if (((uint64_t)box_inner * elem_bytes) & 15u)
    return fail(LOGOS_ERROR, "tensor map: inner box extent must be a multiple of 16 bytes");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LOGOS_ERROR, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return LOGOS_OK;
}

logos_status_t make_tensor_map_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, uint32_t elem_bytes,
                                  uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1_bytes, uint64_t pitch2_bytes,
                                  uint32_t box0, uint32_t box1, uint32_t box2) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(LOGOS_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || (pitch1_bytes & 15u) || (pitch2_bytes & 15u))
    return fail(LOGOS_ERROR, "tensor map: base address and pitches must be multiples of 16 bytes");
  if (((uint64_t)box0 * elem_bytes) & 15u)
    return fail(LOGOS_ERROR, "tensor map: inner box extent must be a multiple of 16 bytes");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {pitch1_bytes, pitch2_bytes};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dtype, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LOGOS_ERROR, "cuTensorMapEncodeTiled (3d) failed with code %d", (int)r);
  return LOGOS_OK;
}

int* kernel_status_ptr(int device) {
  static std::mutex mu;
  static std::unordered_map<int, int*> words;
  std::lock_guard<std::mutex> lk(mu);
  auto it = words.find(device);
  if (it != words.end()) return it->second;
  // Device memory, not mapped host memory: every CTA reads this word once, and a read that
  // crosses PCIe costs about a microsecond and serialises.
  int prev = 0;
  cudaGetDevice(&prev);
  int* p = nullptr;
  if (cudaSetDevice(device) != cudaSuccess || cudaMalloc(reinterpret_cast<void**>(&p), 256) != cudaSuccess ||
      cudaMemset(p, 0, 256) != cudaSuccess) {
    cudaGetLastError();
    cudaSetDevice(prev);
    return nullptr;
  }
  cudaSetDevice(prev);
  words[device] = p;
  return p;
}

logos_status_t static_attn_status_read(int device, int words_out[8], bool clear, bool* used);  // attention.cu

logos_status_t kernel_status_read(int device, int* out, bool clear) {
  int* p = kernel_status_ptr(device);
  if (!p) return fail(LOGOS_ERROR, "no kernel status word (no CUDA device?)");
  LOGOS_CUDA_TRY(cudaSetDevice(device));
  int words[8];
  LOGOS_CUDA_TRY(cudaMemcpy(words, p, sizeof(words), cudaMemcpyDeviceToHost));
  if (words[0] == 0) {
    // the word of the entry point that keeps its scratch inside the library image
    int sw[8];
    bool used = false;
    LOGOS_TRY(static_attn_status_read(device, sw, clear, &used));
    if (used && sw[0] != 0) {
      *out = sw[0];
      set_last_error("device-side wait gave up in logos_gqa_decode_attn_fixed_scratch: code " + std::to_string(sw[0]));
      return LOGOS_OK;
    }
  }
  *out = words[0];
  if (words[0] != 0) {
    // where the first kernel to give up was: block (x, y), K stage, stages of that block, warp
    set_last_error("device-side wait gave up: code " + std::to_string(words[0]) + " block (" + std::to_string(words[1]) +
                   "," + std::to_string(words[2]) + ") stage " + std::to_string(words[3]) + " of " +
                   std::to_string(words[4]) + " warp " + std::to_string(words[5]));
    if (clear) LOGOS_CUDA_TRY(cudaMemset(p, 0, sizeof(words)));
  }
  return LOGOS_OK;
}

}  // namespace logos

using namespace logos;

// Reads and clears the status word kernels set when a bounded wait gives up
// (0 = no kernel reported a problem since the last read).
extern "C" logos_status_t logos_kernel_status(int32_t device, int32_t* out_code) {
  return guarded([&]() -> logos_status_t {
    if (!out_code) return fail(LOGOS_NULL_POINTER, "logos_kernel_status: out_code is null");
    int n = logos_device_count();
    if (device < 0 || device >= n) return fail(LOGOS_OUT_OF_BOUNDS, "logos_kernel_status: device %d of %d", device, n);
    int code = 0;
    LOGOS_TRY(kernel_status_read(device, &code, true));
    *out_code = code;
    return LOGOS_OK;
  });
}
