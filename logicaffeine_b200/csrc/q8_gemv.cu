// Q8 GEMV: y[n] = sum_kb s[n,kb] * sum_{k in kb} q[n,k] * x[k].
//
// HBM-bound: 1.125 bytes of weights per multiply-add, so the kernel is a
// coalesced stream.  One warp owns one row at a time; every lane issues 128-bit
// read-only loads of 16 consecutive int8 (a half block), so a warp covers 512
// columns per load and keeps eight such loads in flight.  int8 -> f32 uses
// the 2^23 mantissa trick (one byte-permute and one subtract), the half-block
// dot product is scaled by its block's f32 scale in registers, and the row sum
// is a warp-shuffle reduction.  x lives in shared memory, laid out so the
// four 128-bit reads a lane needs are bank-conflict free.
#include "ops.cuh"

namespace logos {

namespace {

constexpr int GEMV_WARPS = 8;

__device__ __forceinline__ uint4 ldg_nc_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// byte `sel` of the bias-flipped word -> exact float value of the int8
__device__ __forceinline__ float byte_to_f32(uint32_t w_xor80, uint32_t selector) {
  // 0x4B0000bb = 2^23 + bb ; bb = q + 128
  uint32_t bits = __byte_perm(w_xor80, 0x4B000000u, selector);
  return __uint_as_float(bits) - 8388736.0f;
}

__device__ __forceinline__ float dot4(uint32_t w, float4 x, float acc) {
  uint32_t u = w ^ 0x80808080u;
  acc = fmaf(byte_to_f32(u, 0x7650), x.x, acc);
  acc = fmaf(byte_to_f32(u, 0x7651), x.y, acc);
  acc = fmaf(byte_to_f32(u, 0x7652), x.z, acc);
  acc = fmaf(byte_to_f32(u, 0x7653), x.w, acc);
  return acc;
}

// xs4 layout: chunk c (16 floats) is split into 4 float4; float4 j of chunk c
// sits at index (c/32)*128 + j*32 + (c%32), so the 32 lanes of a warp reading
// the same j of consecutive chunks touch consecutive 16-byte slots.
__device__ __forceinline__ int xs4_index(int chunk, int j) { return (chunk >> 5) * 128 + j * 32 + (chunk & 31); }

// A warp owns one row.  For each super-chunk of 4096 columns a lane first issues
// all of its eight 128-bit weight loads (and the eight scales), and only then
// waits for x to be staged, so the HBM stream starts at the first instruction.
// What decides the speed is the bytes an SM keeps in flight: the launch bound caps the
// kernel at 64 registers so that four CTAs share an SM (128 KB of loads in flight, and the
// 512 CTAs of a 4096-row matrix are one wave); with three CTAs per SM the same code
// measured 3.2 instead of 3.4 TB/s at 4096 x 4096 and 4.05 instead of 4.3 TB/s at
// 152064 x 5120.
template <bool X_IN_SMEM>
__global__ void __launch_bounds__(GEMV_WARPS * 32, 4)
q8_gemv_kernel(const int8_t* __restrict__ q, const float* __restrict__ s, const float* __restrict__ x,
               float* __restrict__ y, int64_t n, int64_t k) {
  extern __shared__ float4 xs4[];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int chunks = (int)(k >> 4);  // 16-element chunks per row
  const int64_t kb_per_row = k >> 5;
  // Dependent launch: the weights are read before the previous kernel of the stream has
  // finished (the caller's scope promises nothing in it writes them); x and y wait for it.
  pdl_trigger();
  bool waited = false;
  bool x_ready = !X_IN_SMEM;
  for (int64_t row0 = (int64_t)blockIdx.x * GEMV_WARPS; row0 < n; row0 += (int64_t)gridDim.x * GEMV_WARPS) {
    const int64_t row = row0 + warp;
    const bool row_ok = row < n;
    const uint4* qr = reinterpret_cast<const uint4*>(q + (row_ok ? row : 0) * k);
    const float* sr = s + (row_ok ? row : 0) * kb_per_row;
    float acc = 0.f;
    for (int c0 = 0; c0 < chunks; c0 += 256) {
      uint4 w[8];
      float sc[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        int c = c0 + lane + 32 * u;
        if (row_ok && c < chunks) {
          w[u] = ldg_nc_v4(qr + c);
          sc[u] = __ldg(sr + (c >> 1));
        } else {
          w[u] = make_uint4(0x0, 0x0, 0x0, 0x0);
          sc[u] = 0.f;
        }
      }
      if (!waited) {
        pdl_wait();
        waited = true;
      }
      if (!x_ready) {
        const float4* xg = reinterpret_cast<const float4*>(x);
        for (int i = tid; i < chunks * 4; i += GEMV_WARPS * 32) {
          int c = i >> 2, j = i & 3;
          xs4[xs4_index(c, j)] = __ldcg(xg + i);
        }
        __syncthreads();
        x_ready = true;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        int c = c0 + lane + 32 * u;
        if (c < chunks) {
          float4 x0, x1, x2, x3;
          if (X_IN_SMEM) {
            x0 = xs4[xs4_index(c, 0)]; x1 = xs4[xs4_index(c, 1)];
            x2 = xs4[xs4_index(c, 2)]; x3 = xs4[xs4_index(c, 3)];
          } else {
            const float4* xg = reinterpret_cast<const float4*>(x) + c * 4;
            x0 = __ldcg(xg); x1 = __ldcg(xg + 1); x2 = __ldcg(xg + 2); x3 = __ldcg(xg + 3);
          }
          float p = 0.f;
          p = dot4(w[u].x, x0, p);
          p = dot4(w[u].y, x1, p);
          p = dot4(w[u].z, x2, p);
          p = dot4(w[u].w, x3, p);
          acc = fmaf(sc[u], p, acc);
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0 && row_ok) y[row] = acc;
  }
}


}  // namespace

logos_status_t launch_q8_gemv(const int8_t* q, const float* s, const float* x, float* y, int64_t n, int64_t k,
                              int device, cudaStream_t st) {
  if (n == 0) return LOGOS_OK;
  if (k == 0) {
    LOGOS_CUDA_TRY(cudaMemsetAsync(y, 0, sizeof(float) * n, st));
    return LOGOS_OK;
  }
  int64_t ctas = (n + GEMV_WARPS - 1) / GEMV_WARPS;
  int64_t cap = (int64_t)sm_count(device) * 8;
  int grid = (int)(ctas < cap ? ctas : cap);
  // x padded to whole groups of 32 chunks (512 floats)
  size_t smem = (size_t)((k / 16 + 31) / 32) * 128 * sizeof(float4);
  if (smem <= 96 * 1024) {
    if (smem > 48 * 1024)
      LOGOS_CUDA_TRY(cudaFuncSetAttribute(q8_gemv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    LOGOS_CUDA_TRY(launch_kernel(q8_gemv_kernel<true>, dim3((unsigned)grid), dim3(GEMV_WARPS * 32), smem, st, q, s, x, y, n, k));
  } else {
    LOGOS_CUDA_TRY(launch_kernel(q8_gemv_kernel<false>, dim3((unsigned)grid), dim3(GEMV_WARPS * 32), 0, st, q, s, x, y, n, k));
  }
  count_launch(LK_GEMV);
  return check_launch("q8_gemv_kernel");
}

}  // namespace logos

using namespace logos;

extern "C" logos_status_t logos_q8_gemv(logos_handle_t q, logos_handle_t s, logos_handle_t x, logos_handle_t y,
                                        int64_t n, int64_t k, void* stream_or_null) {
  return guarded([&]() -> logos_status_t {
    if (n < 0 || k < 0) return fail(LOGOS_OUT_OF_BOUNDS, "logos_q8_gemv: negative extent");
    if (k % 32) return fail(LOGOS_OUT_OF_BOUNDS, "logos_q8_gemv: K=%lld is not a multiple of the block size 32", (long long)k);
    int8_t* qp; float* sp; float* xp; float* yp;
    int32_t dev = 0;
    LOGOS_TRY(buf_ptr<int8_t>(q, n * k, "q", &qp, &dev));
    LOGOS_TRY(buf_ptr<float>(s, n * (k / 32), "s", &sp));
    LOGOS_TRY(buf_ptr<float>(x, k, "x", &xp));
    LOGOS_TRY(buf_ptr<float>(y, n, "y", &yp));
    LOGOS_CUDA_TRY(cudaSetDevice(dev));
    return launch_q8_gemv(qp, sp, xp, yp, n, k, dev, as_stream(stream_or_null));
  });
}
