// Seeded synthetic inputs and Q8 weight preparation.
//   logos_synth_fill        — fill a device buffer from the counter-based generator
//   logos_q8_quantize       — f32 [N][K] -> int8 [N][K] + f32 scale per 32-block
//   logos_q8_synth_weights  — generate N(0,std) and quantise in one pass
// Q8 block rule: s = max|w| / 127 (IEEE division), q = round-half-even(w / s),
// an all-zero block stores s = 0, q = 0.
#include "ops.cuh"
#include "synth.cuh"

namespace logos {

__global__ void synth_fill_kernel(void* dst, int dtype, int kind, uint64_t seed, uint64_t stream,
                                  int64_t first, int64_t count, float a, float b) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < count; i += step) {
    uint64_t idx = (uint64_t)(first + i);
    if (kind == 0) {
      reinterpret_cast<int8_t*>(dst)[i] = (int8_t)synth::uniform_i8(seed, stream, idx);
    } else if (kind == 1) {
      reinterpret_cast<float*>(dst)[i] = synth::uniform_f32(seed, stream, idx, a, b);
    } else if (kind == 2) {
      float v = synth::normal_scaled(seed, stream, idx, a, b);
      if (dtype == LOGOS_F32) reinterpret_cast<float*>(dst)[i] = v;
      else if (dtype == LOGOS_F16) reinterpret_cast<__half*>(dst)[i] = __float2half_rn(v);
      else reinterpret_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn(v);
    } else if (kind == 4) {
      reinterpret_cast<float*>(dst)[i] = synth::gumbel_f32(seed, stream, idx);
    } else {
      reinterpret_cast<int32_t*>(dst)[i] = synth::uniform_i32(seed, stream, idx, (uint32_t)b);
    }
  }
}

// Positions [0,t) of a [B][Hkv_local][Lmax][D] fp16 cache, valued by their index in the
// unsharded [B][Hkv_total][Lmax][D] cache, so every rank fills its heads with the same bits.
__global__ void synth_kv_kernel(__half* __restrict__ cache, uint64_t seed, uint64_t stream, int64_t b, int64_t hkv_local,
                                int64_t h0, int64_t hkv_total, int64_t l_max, int64_t d, int64_t t) {
  const int64_t per_head = t * d;
  const int64_t total = b * hkv_local * per_head;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    int64_t bh = i / per_head, r = i - bh * per_head;
    int64_t bb = bh / hkv_local, h = bh - bb * hkv_local;
    int64_t logical = ((bb * hkv_total + h0 + h) * l_max) * d + r;
    int64_t local = ((bb * hkv_local + h) * l_max) * d + r;
    cache[local] = __float2half_rn(synth::normal_scaled(seed, stream, (uint64_t)logical, 0.f, 1.f));
  }
}

logos_status_t launch_synth_kv(__half* cache, uint64_t seed, uint64_t stream, int64_t b, int64_t hkv_local, int64_t h0,
                               int64_t hkv_total, int64_t l_max, int64_t d, int64_t t, int device, cudaStream_t st) {
  int64_t total = b * hkv_local * t * d;
  if (total == 0) return LOGOS_OK;
  int64_t want = (total + 255) / 256;
  int64_t cap = (int64_t)sm_count(device) * 16;
  synth_kv_kernel<<<(int)(want < cap ? want : cap), 256, 0, st>>>(cache, seed, stream, b, hkv_local, h0, hkv_total, l_max,
                                                                  d, t);
  count_launch(LK_SYNTH);
  return check_launch("synth_kv_kernel");
}

// One warp per 32-element block: lane l owns element l.
template <bool GENERATE>
__global__ void q8_quantize_kernel(const float* __restrict__ w, int8_t* __restrict__ q, float* __restrict__ s,
                                   int64_t n, int64_t k, int64_t row0, int64_t col0, int64_t k_total,
                                   int64_t out_row_mul, int64_t out_row_add, uint64_t seed, uint64_t stream,
                                   float std) {
  const int lane = threadIdx.x & 31;
  const int64_t kb_per_row = k / 32;
  const int64_t blocks = n * kb_per_row;
  int64_t blk = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t step = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (; blk < blocks; blk += step) {
    int64_t row = blk / kb_per_row;
    int64_t kb = blk - row * kb_per_row;
    int64_t col = kb * 32 + lane;
    int64_t src = (row0 + row) * k_total + col0 + col;
    float v;
    if (GENERATE) {
      v = __fmul_rn(std, synth::normal_f32(seed, stream, (uint64_t)src));
    } else {
      v = w[src];
    }
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float sc = __fdiv_rn(amax, 127.0f);
    int qi = 0;
    if (amax > 0.0f) {
      qi = __float2int_rn(__fdiv_rn(v, sc));
      qi = max(-127, min(127, qi));
    }
    int64_t orow = row * out_row_mul + out_row_add;
    q[orow * k + col] = (int8_t)qi;
    if (lane == 0) s[orow * kb_per_row + kb] = sc;
  }
}

// Row-major int8 [n][k] <-> the tile-major layout the tcgen05 GEMM streams: tiles of 128 rows x
// 128 columns, each 16 KB contiguous, ordered (row tile, K tile), so that the stages a CTA reads
// one after the other form one contiguous run in HBM instead of 128 lines a row pitch apart.
// Rows n .. ceil128(n) of the tiled form hold the value zero.  One thread moves 16 bytes.
__global__ void q8_retile_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ out, int64_t n, int64_t k,
                                 int to_tiled) {
  const int64_t ktiles = k >> 7, rtiles = (n + 127) >> 7;
  const int64_t total = rtiles * ktiles * 128 * 8;  // 16-byte chunks of the tiled form
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c16 = i & 7, r = (i >> 3) & 127, ts = i >> 10;
    const int64_t t = ts / ktiles, st = ts - t * ktiles;
    const int64_t row = t * 128 + r;
    const int64_t rm = row * k + st * 128 + c16 * 16;   // offset in the row-major form
    // the tiled form holds q + 128 as unsigned bytes (every byte's top bit flipped): the GEMM's
    // int8 -> fp16 conversion wants that form and then needs no flip of its own
    const uint32_t f = 0x80808080u;
    if (to_tiled) {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (row < n) v = *reinterpret_cast<const uint4*>(in + rm);
      *reinterpret_cast<uint4*>(out + i * 16) = make_uint4(v.x ^ f, v.y ^ f, v.z ^ f, v.w ^ f);
    } else if (row < n) {
      const uint4 v = *reinterpret_cast<const uint4*>(in + i * 16);
      *reinterpret_cast<uint4*>(out + rm) = make_uint4(v.x ^ f, v.y ^ f, v.z ^ f, v.w ^ f);
    }
  }
}

// The scales of the same tiles: f32 [n][k/32] row-major <-> [row tile][K tile][128 rows][4], so the
// 128 rows' scales of one GEMM stage are 2 contiguous KB.  One thread moves one row's four scales.
__global__ void q8_retile_scales_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t n, int64_t k,
                                        int to_tiled) {
  const int64_t ktiles = k >> 7, rtiles = (n + 127) >> 7, kb_per_row = k >> 5;
  const int64_t total = rtiles * ktiles * 128;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i & 127, ts = i >> 7;
    const int64_t t = ts / ktiles, st = ts - t * ktiles;
    const int64_t row = t * 128 + r;
    const int64_t rm = row * kb_per_row + st * 4;
    if (to_tiled) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row < n) v = *reinterpret_cast<const float4*>(in + rm);
      *reinterpret_cast<float4*>(out + i * 4) = v;
    } else if (row < n) {
      *reinterpret_cast<float4*>(out + rm) = *reinterpret_cast<const float4*>(in + i * 4);
    }
  }
}

logos_status_t launch_q8_retile_scales(const float* in, float* out, int64_t n, int64_t k, bool to_tiled, int device,
                                       cudaStream_t st) {
  if (n == 0 || k == 0) return LOGOS_OK;
  if (k % 128) return fail(LOGOS_ERROR, "q8_retile: K=%lld is not a multiple of 128", (long long)k);
  const int64_t total = ((n + 127) / 128) * (k / 128) * 128;
  const int64_t want = (total + 255) / 256, cap = (int64_t)sm_count(device) * 32;
  q8_retile_scales_kernel<<<(int)(want < cap ? want : cap), 256, 0, st>>>(in, out, n, k, to_tiled ? 1 : 0);
  count_launch(LK_SYNTH);
  return check_launch("q8_retile_scales_kernel");
}

logos_status_t launch_q8_retile(const int8_t* in, int8_t* out, int64_t n, int64_t k, bool to_tiled, int device,
                                cudaStream_t st) {
  if (n == 0 || k == 0) return LOGOS_OK;
  if (k % 128) return fail(LOGOS_ERROR, "q8_retile: K=%lld is not a multiple of 128", (long long)k);
  const int64_t total = ((n + 127) / 128) * (k / 128) * 1024;
  const int64_t want = (total + 255) / 256, cap = (int64_t)sm_count(device) * 32;
  q8_retile_kernel<<<(int)(want < cap ? want : cap), 256, 0, st>>>(in, out, n, k, to_tiled ? 1 : 0);
  count_launch(LK_SYNTH);
  return check_launch("q8_retile_kernel");
}

logos_status_t launch_synth_fill(void* dst, int dtype, int kind, uint64_t seed, uint64_t stream, int64_t first,
                                 int64_t count, float a, float b, int device, cudaStream_t st) {
  if (count == 0) return LOGOS_OK;
  int threads = 256;
  int64_t want = (count + threads - 1) / threads;
  int64_t cap = (int64_t)sm_count(device) * 16;
  int grid = (int)(want < cap ? want : cap);
  synth_fill_kernel<<<grid, threads, 0, st>>>(dst, dtype, kind, seed, stream, first, count, a, b);
  count_launch(LK_SYNTH);
  return check_launch("synth_fill_kernel");
}

logos_status_t launch_q8_quantize(bool generate, const float* w, int8_t* q, float* s, int64_t n, int64_t k,
                                  int64_t row0, int64_t col0, int64_t k_total, int64_t out_row_mul,
                                  int64_t out_row_add, uint64_t seed, uint64_t stream, float std, int device,
                                  cudaStream_t st) {
  if (n == 0 || k == 0) return LOGOS_OK;
  int64_t blocks = n * (k / 32);
  int threads = 256;
  int64_t want = (blocks * 32 + threads - 1) / threads;
  int64_t cap = (int64_t)sm_count(device) * 32;
  int grid = (int)(want < cap ? want : cap);
  if (generate)
    q8_quantize_kernel<true><<<grid, threads, 0, st>>>(nullptr, q, s, n, k, row0, col0, k_total, out_row_mul,
                                                       out_row_add, seed, stream, std);
  else
    q8_quantize_kernel<false><<<grid, threads, 0, st>>>(w, q, s, n, k, row0, col0, k_total, out_row_mul,
                                                        out_row_add, 0, 0, 0.f);
  count_launch(LK_SYNTH);
  return check_launch("q8_quantize_kernel");
}

}  // namespace logos

using namespace logos;

extern "C" {

logos_status_t logos_synth_fill(logos_handle_t dst, int64_t dst_offset_bytes, int32_t dtype, int32_t kind,
                                uint64_t seed, uint64_t stream, int64_t first_index, int64_t count,
                                float a, float b, void* stream_or_null) {
  return guarded([&]() -> logos_status_t {
    if (count < 0 || first_index < 0) return fail(LOGOS_OUT_OF_BOUNDS, "logos_synth_fill: negative extent");
    int64_t esz;
    switch (kind) {
      case 0: esz = 1; if (dtype != LOGOS_I8) return fail(LOGOS_ERROR, "logos_synth_fill: kind 0 writes i8"); break;
      case 1: esz = 4; if (dtype != LOGOS_F32) return fail(LOGOS_ERROR, "logos_synth_fill: kind 1 writes f32"); break;
      case 2:
        if (dtype == LOGOS_F32) esz = 4;
        else if (dtype == LOGOS_F16 || dtype == LOGOS_BF16) esz = 2;
        else return fail(LOGOS_ERROR, "logos_synth_fill: kind 2 writes f32, f16 or bf16");
        break;
      case 3:
        esz = 4;
        if (dtype != LOGOS_I32) return fail(LOGOS_ERROR, "logos_synth_fill: kind 3 writes i32");
        if (!(b >= 1.0f)) return fail(LOGOS_OUT_OF_BOUNDS, "logos_synth_fill: kind 3 needs b >= 1");
        break;
      case 4: esz = 4; if (dtype != LOGOS_F32) return fail(LOGOS_ERROR, "logos_synth_fill: kind 4 writes f32"); break;
      default: return fail(LOGOS_ERROR, "logos_synth_fill: unknown kind %d", kind);
    }
    if (dst_offset_bytes % esz) return fail(LOGOS_ERROR, "logos_synth_fill: offset not aligned to the element size");
    DevBuf* buf = nullptr;
    LOGOS_TRY(buf_resolve(dst, dst_offset_bytes, count * esz, "logos_synth_fill dst", &buf));
    LOGOS_CUDA_TRY(cudaSetDevice(buf->device));
    return launch_synth_fill(static_cast<char*>(buf->ptr) + dst_offset_bytes, dtype, kind, seed, stream,
                             first_index, count, a, b, buf->device, as_stream(stream_or_null));
  });
}

static logos_status_t quantize_abi(bool generate, logos_handle_t w, logos_handle_t q, logos_handle_t s,
                                   int64_t n, int64_t k, int64_t row0, uint64_t seed, uint64_t stream,
                                   float std, void* cu_stream, const char* who) {
  if (n < 0 || k < 0 || row0 < 0) return fail(LOGOS_OUT_OF_BOUNDS, "%s: negative extent", who);
  if (k % 32) return fail(LOGOS_OUT_OF_BOUNDS, "%s: K=%lld is not a multiple of the block size 32", who, (long long)k);
  int8_t* qp = nullptr;
  float* sp = nullptr;
  float* wp = nullptr;
  int32_t dev = 0;
  LOGOS_TRY(buf_ptr<int8_t>(q, n * k, "q", &qp, &dev));
  LOGOS_TRY(buf_ptr<float>(s, n * (k / 32), "s", &sp));
  if (!generate) LOGOS_TRY(buf_ptr<float>(w, n * k, "w", &wp));
  LOGOS_CUDA_TRY(cudaSetDevice(dev));
  return launch_q8_quantize(generate, wp, qp, sp, n, k, row0, 0, k, 1, 0, seed, stream, std, dev,
                            as_stream(cu_stream));
}

logos_status_t logos_q8_quantize(logos_handle_t w, logos_handle_t q, logos_handle_t s,
                                 int64_t n, int64_t k, void* stream_or_null) {
  return guarded([&]() -> logos_status_t {
    return quantize_abi(false, w, q, s, n, k, 0, 0, 0, 0.f, stream_or_null, "logos_q8_quantize");
  });
}

logos_status_t logos_q8_synth_weights(logos_handle_t q, logos_handle_t s, int64_t n, int64_t k,
                                      int64_t row0, uint64_t seed, uint64_t stream, float std,
                                      void* stream_or_null) {
  return guarded([&]() -> logos_status_t {
    return quantize_abi(true, nullptr, q, s, n, k, row0, seed, stream, std, stream_or_null,
                        "logos_q8_synth_weights");
  });
}

}  // extern "C"
