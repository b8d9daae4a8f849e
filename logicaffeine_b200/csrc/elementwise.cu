// Norms and element-wise pieces of the decode step.
//   rmsnorm            y = x * rsqrt(mean(x^2) + eps) * g
//   swiglu             y = silu(gate) * up
//   embed              h[row] = dequantised Q8 row of the token
//   residual_rmsnorm   h += delta (split-K partials summed in ascending order),
//                      xn = 16-bit( rmsnorm(h) )  — one pass over the row
//   argmax             lowest index wins ties
// Row reductions run in a fixed shape (per-thread strided partials, shuffle
// tree, then warps in ascending order), so results do not depend on timing.
#include "ops.cuh"

#include <cooperative_groups.h>

namespace logos {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the CTA; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  __syncthreads();
  return t;
}

__global__ void rmsnorm_f32_kernel(const float* __restrict__ x, const float* __restrict__ g, float* __restrict__ y,
                                   int64_t h, float eps) {
  __shared__ float red[32];
  const float* xr = x + (int64_t)blockIdx.x * h;
  float* yr = y + (int64_t)blockIdx.x * h;
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < h; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
  ss = block_sum(ss, red);
  float inv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)h), eps)));
  for (int64_t i = threadIdx.x; i < h; i += blockDim.x) yr[i] = __fmul_rn(__fmul_rn(xr[i], inv), g[i]);
}

__global__ void swiglu_f32_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                  float* __restrict__ y, int64_t count) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < count; i += step) {
    float g = gate[i];
    float sg = __fdiv_rn(g, 1.0f + expf(-g));
    y[i] = __fmul_rn(sg, up[i]);
  }
}

__global__ void embed_kernel(const int32_t* __restrict__ tokens, const int8_t* __restrict__ q,
                             const float* __restrict__ s, float* __restrict__ h, int64_t hidden) {
  pdl_wait();
  pdl_trigger();
  int64_t row = blockIdx.x;
  int64_t t = __ldcg(tokens + row);
  const int8_t* qr = q + t * hidden;
  const float* sr = s + t * (hidden / 32);
  for (int64_t e = threadIdx.x; e < hidden; e += blockDim.x)
    h[row * hidden + e] = __fmul_rn(sr[e >> 5], (float)qr[e]);
}

// One CTA per row, 128-bit accesses: fold the split-K partials into the residual
// stream in ascending order, keep the updated row in shared memory, reduce the
// sum of squares, then write the normalised row as activation planes.
__global__ void __launch_bounds__(512)
residual_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta, int parts, int64_t part_stride,
                        const float* __restrict__ g, ActOut xn, int64_t hidden, float eps) {
  __shared__ float red[32];
  extern __shared__ float4 row_cache4[];  // hidden floats
  float* row_cache = reinterpret_cast<float*>(row_cache4);
  // h and the partials come from kernels of the same step: wait for them, and read them past L1
  pdl_wait();
  pdl_trigger();
  const int64_t row = blockIdx.x;
  float* hr = h + row * hidden;
  float ss = 0.f;
  if ((hidden & 3) == 0) {
    const int64_t n4 = hidden >> 2;
    float4* hr4 = reinterpret_cast<float4*>(hr);
    for (int64_t i = threadIdx.x; i < n4; i += blockDim.x) {
      float4 v = __ldcg(hr4 + i);
      for (int p = 0; p < parts; ++p) {
        const float4 d = __ldcg(reinterpret_cast<const float4*>(delta + (int64_t)p * part_stride + row * hidden) + i);
        v.x = __fadd_rn(v.x, d.x); v.y = __fadd_rn(v.y, d.y); v.z = __fadd_rn(v.z, d.z); v.w = __fadd_rn(v.w, d.w);
      }
      if (parts > 0) hr4[i] = v;
      row_cache4[i] = v;
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
  } else {
    for (int64_t i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = __ldcg(hr + i);
      for (int p = 0; p < parts; ++p) v = __fadd_rn(v, __ldcg(delta + (int64_t)p * part_stride + row * hidden + i));
      if (parts > 0) hr[i] = v;
      row_cache[i] = v;
      ss = fmaf(v, v, ss);
    }
  }
  ss = block_sum(ss, red);
  float inv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)hidden), eps)));
  for (int64_t i = threadIdx.x; i < hidden; i += blockDim.x)
    act_store(xn, row * hidden + i, __fmul_rn(__fmul_rn(row_cache[i], inv), g[i]));
}

// ---- residual + RMSNorm with the tensor-parallel all-reduce folded in (see ops.cuh)
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded: false when the flag did not reach `target` within about ten seconds of SM clock (a
// peer is another process on another GPU: it may lag by a graph instantiation or a page-in).
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* p, uint32_t target) {
  if ((int32_t)(ld_acquire_sys(p) - target) >= 0) return true;
  const long long start = clock64();
  for (;;) {
#pragma unroll 1
    for (int k = 0; k < 64; ++k)
      if ((int32_t)(ld_acquire_sys(p) - target) >= 0) return true;
    if (clock64() - start > 20000000000ll) return false;
  }
}

constexpr int TP_MAX_SRC = 64;  // degree x parts
constexpr int TP_CLUSTER = 4;   // CTAs per row: at decode batch sizes a rank owns fewer rows than there are SMs

// A row is spread over a cluster of TP_CLUSTER CTAs (one float4 per thread where the row is
// short enough), so that every peer load of a row is in flight at once; the slices' sums of
// squares meet through distributed shared memory, summed in rank order by every CTA.
__global__ void __launch_bounds__(512)
tp_residual_rmsnorm_kernel(float* __restrict__ h, const TpFusedArgs t, int parts, int64_t part_stride,
                           const float* __restrict__ g, int64_t rows_own, int64_t hidden, float eps, int* status) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float red[32];
  __shared__ float slice_ss;
  __shared__ uint32_t epoch_s;
  __shared__ int last_s;
  __shared__ const float* src[TP_MAX_SRC];
  extern __shared__ float4 row_cache4[];  // this CTA's slice of the row
  const int tid = threadIdx.x;
  pdl_wait();  // this rank's own GEMM has completed: its partials are in this GPU's memory
  pdl_trigger();
  uint32_t* my = t.flags[t.rank];
  if (tid == 0) epoch_s = ld_acquire_sys(my + 16) + 1u;
  const int nsrc = t.degree * parts;
  if (tid < nsrc) src[tid] = t.partials[tid / parts] + (int64_t)(tid % parts) * part_stride;  // rank-major, then split
  __syncthreads();
  const uint32_t e = epoch_s;
  // ---- barrier 1: every rank's partials are complete.  One CTA announces this rank to all
  // (itself included); every CTA polls its own rank's words, which are local memory.
  if (blockIdx.x == 0 && tid < t.degree) st_release_sys(t.flags[tid] + t.rank, e);
  if (tid < t.degree && !wait_flag_ge(my + tid, e)) atomicExch(status, 3010);
  __syncthreads();

  const unsigned crank = cluster.block_rank();
  const int64_t row = (int64_t)t.rank * rows_own + blockIdx.x / TP_CLUSTER;
  const int64_t per = (hidden >> 2) / TP_CLUSTER;  // float4 per CTA
  const int64_t off4 = row * (hidden >> 2) + (int64_t)crank * per;  // this slice, in float4 units from a buffer's base
  float4* hr4 = reinterpret_cast<float4*>(h) + off4;
  float ss = 0.f;
  for (int64_t i = tid; i < per; i += blockDim.x) {
    float4 v = __ldcg(hr4 + i);
    // peers' buffers are read past L1 (ld.global.cg): the lines are rewritten every call.
    // Eight loads are issued before their sums are taken, so a row costs few NVLink round trips.
    for (int q0 = 0; q0 < nsrc; q0 += 8) {
      float4 d[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        d[u] = (q0 + u < nsrc) ? __ldcg(reinterpret_cast<const float4*>(src[q0 + u]) + off4 + i)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (q0 + u < nsrc) {
          v.x = __fadd_rn(v.x, d[u].x); v.y = __fadd_rn(v.y, d[u].y);
          v.z = __fadd_rn(v.z, d[u].z); v.w = __fadd_rn(v.w, d[u].w);
        }
      }
    }
    hr4[i] = v;
    row_cache4[i] = v;
    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
  }
  ss = block_sum(ss, red);
  if (tid == 0) slice_ss = ss;
  cluster.sync();
  float total = 0.f;
  for (unsigned r = 0; r < TP_CLUSTER; ++r) total += *cluster.map_shared_rank(&slice_ss, r);
  const float inv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)hidden), eps)));
  const float4* g4 = reinterpret_cast<const float4*>(g) + (int64_t)crank * per;
  for (int64_t i = tid; i < per; i += blockDim.x) {
    const float4 v = row_cache4[i], gg = g4[i];
    const float o[4] = {__fmul_rn(__fmul_rn(v.x, inv), gg.x), __fmul_rn(__fmul_rn(v.y, inv), gg.y),
                        __fmul_rn(__fmul_rn(v.z, inv), gg.z), __fmul_rn(__fmul_rn(v.w, inv), gg.w)};
    __half hh[4], ll[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float x = o[k];
      if (t.act_mode == LOGOS_BF16) x = __bfloat162float(__float2bfloat16_rn(x));
      x = act_clamp(x);
      hh[k] = __float2half_rn(x);
      ll[k] = __float2half_rn((x - __half2float(hh[k])) * 2048.f);
    }
    const uint2 hp = *reinterpret_cast<const uint2*>(hh), lp = *reinterpret_cast<const uint2*>(ll);
    for (int r = 0; r < t.degree; ++r) {
      reinterpret_cast<uint2*>(t.xn_hi[r])[off4 + i] = hp;
      if (t.xn_lo[r]) reinterpret_cast<uint2*>(t.xn_lo[r])[off4 + i] = lp;
    }
  }
  // ---- barrier 2: the last CTA of this rank to finish tells every rank that this rank's rows
  // have been delivered, and holds the kernel until every peer's rows are here.
  cluster.sync();  // also: no CTA leaves while a peer of its cluster may still read its slice_ss
  if (tid == 0) {
    __threadfence_system();
    const uint32_t ticket = atomicAdd(my + 17, 1u);
    last_s = (ticket == gridDim.x - 1) ? 1 : 0;
    if (last_s) {
      __threadfence_system();
      my[17] = 0u;
    }
  }
  __syncthreads();
  if (last_s) {
    if (tid < t.degree) st_release_sys(t.flags[tid] + 8 + t.rank, e);
    if (tid < t.degree && !wait_flag_ge(my + 8 + tid, e)) atomicExch(status, 3020);
    __syncthreads();
    if (tid == 0) st_release_sys(my + 16, e);
  }
}

__global__ void bf16_to_f16_kernel(const __nv_bfloat16* __restrict__ x, __half* __restrict__ y, int64_t count) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) y[i] = __float2half_rn(act_clamp(__bfloat162float(x[i])));
}

__global__ void act_split_kernel(const float* __restrict__ x, ActOut o, int64_t count) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) act_store(o, i, x[i]);
}

// history (optional): row `*step_counter` of a [history_rows][rows] log also receives the ids,
// so a captured step needs no per-step pointer.
__global__ void argmax_kernel(const float* __restrict__ logits, int32_t* __restrict__ tokens,
                              int32_t* __restrict__ history, const int32_t* __restrict__ step_counter,
                              int64_t history_rows, int64_t vocab) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  pdl_wait();
  pdl_trigger();
  const int64_t row = blockIdx.x;
  const float* lr = logits + row * vocab;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int64_t i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = __ldcg(lr + i);
    if (v > best || (v == best && (int)i < idx)) {
      best = v;
      idx = (int)i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) {
      best = ov;
      idx = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) {
    bv[warp] = best;
    bi[warp] = idx;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < nw; ++w)
      if (bv[w] > best || (bv[w] == best && bi[w] < idx)) {
        best = bv[w];
        idx = bi[w];
      }
    if (idx == 0x7fffffff) idx = 0;  // all NaN / empty row
    tokens[row] = idx;
    if (history) {
      int64_t slot = step_counter ? __ldcg(step_counter) : 0;
      if (slot < history_rows) history[slot * gridDim.x + row] = idx;
    }
  }
}

}  // namespace

logos_status_t launch_rmsnorm_f32(const float* x, const float* g, float* y, int64_t rows, int64_t h, float eps,
                                  cudaStream_t st) {
  if (rows == 0 || h == 0) return LOGOS_OK;
  rmsnorm_f32_kernel<<<(unsigned)rows, 256, 0, st>>>(x, g, y, h, eps);
  count_launch(LK_ELEMWISE);
  return check_launch("rmsnorm_f32_kernel");
}

logos_status_t launch_swiglu_f32(const float* gate, const float* up, float* y, int64_t count, cudaStream_t st) {
  if (count == 0) return LOGOS_OK;
  int64_t want = (count + 255) / 256;
  int grid = (int)(want < 148 * 8 ? want : 148 * 8);
  swiglu_f32_kernel<<<grid, 256, 0, st>>>(gate, up, y, count);
  count_launch(LK_ELEMWISE);
  return check_launch("swiglu_f32_kernel");
}

logos_status_t launch_embed(const int32_t* tokens, const int8_t* q, const float* s, float* h, int64_t rows,
                            int64_t hidden, cudaStream_t st) {
  if (rows == 0) return LOGOS_OK;
  LOGOS_CUDA_TRY(launch_kernel(embed_kernel, dim3((unsigned)rows), dim3(256), 0, st, tokens, q, s, h, hidden));
  count_launch(LK_ELEMWISE);
  return check_launch("embed_kernel");
}

logos_status_t launch_bf16_to_f16(const __nv_bfloat16* x, __half* y, int64_t count, cudaStream_t st) {
  if (count == 0) return LOGOS_OK;
  bf16_to_f16_kernel<<<(unsigned)((count + 255) / 256), 256, 0, st>>>(x, y, count);
  count_launch(LK_ELEMWISE);
  return check_launch("bf16_to_f16_kernel");
}

logos_status_t launch_act_split(const float* x, ActOut o, int64_t count, cudaStream_t st) {
  if (count == 0) return LOGOS_OK;
  act_split_kernel<<<(unsigned)((count + 255) / 256), 256, 0, st>>>(x, o, count);
  count_launch(LK_ELEMWISE);
  return check_launch("act_split_kernel");
}

logos_status_t launch_residual_rmsnorm(float* h, const float* delta, int parts, int64_t part_stride,
                                       const float* g, ActOut xn, int64_t rows, int64_t hidden, float eps,
                                       cudaStream_t st) {
  if (rows == 0) return LOGOS_OK;
  size_t smem = sizeof(float) * (size_t)hidden;
  if (smem > 48 * 1024)
    LOGOS_CUDA_TRY(cudaFuncSetAttribute(residual_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  LOGOS_CUDA_TRY(launch_kernel(residual_rmsnorm_kernel, dim3((unsigned)rows), dim3(512), smem, st, h, delta, parts,
                               part_stride, g, xn, hidden, eps));
  count_launch(LK_ELEMWISE);
  return check_launch("residual_rmsnorm_kernel");
}

logos_status_t launch_tp_residual_rmsnorm(float* h, const TpFusedArgs& t, int parts, int64_t part_stride, const float* g,
                                          int64_t rows, int64_t hidden, float eps, int device, cudaStream_t st) {
  if (rows == 0) return LOGOS_OK;
  if (t.degree < 2 || t.degree > 8 || rows % t.degree || hidden % (4 * TP_CLUSTER) || parts < 1 ||
      t.degree * parts > TP_MAX_SRC)
    return fail(LOGOS_ERROR, "tp_residual_rmsnorm: unsupported shape (rows %lld, hidden %lld, degree %d, parts %d)",
                (long long)rows, (long long)hidden, t.degree, parts);
  int* status = kernel_status_ptr(device);
  if (!status) return fail(LOGOS_ERROR, "tp_residual_rmsnorm: no kernel status word");
  const int64_t per = (hidden >> 2) / TP_CLUSTER;
  const int64_t rows_own = rows / t.degree;
  int threads = (int)(((per + 31) / 32) * 32);
  if (threads > 512) threads = 512;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows_own * TP_CLUSTER));
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = sizeof(float4) * (size_t)per;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = TP_CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_active() ? 2 : 1;
  if (cfg.dynamicSmemBytes > 48 * 1024)
    LOGOS_CUDA_TRY(cudaFuncSetAttribute(tp_residual_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)cfg.dynamicSmemBytes));
  LOGOS_CUDA_TRY(cudaLaunchKernelEx(&cfg, tp_residual_rmsnorm_kernel, h, t, parts, part_stride, g, rows_own, hidden, eps,
                                    status));
  count_launch(LK_ELEMWISE);
  return check_launch("tp_residual_rmsnorm_kernel");
}

logos_status_t launch_argmax(const float* logits, int32_t* tokens, int32_t* history_or_null,
                             const int32_t* step_counter_or_null, int64_t history_rows, int64_t rows, int64_t vocab,
                             cudaStream_t st) {
  if (rows == 0) return LOGOS_OK;
  LOGOS_CUDA_TRY(launch_kernel(argmax_kernel, dim3((unsigned)rows), dim3(1024), 0, st, logits, tokens, history_or_null,
                               step_counter_or_null, history_rows, vocab));
  count_launch(LK_ELEMWISE);
  return check_launch("argmax_kernel");
}

}  // namespace logos

using namespace logos;

extern "C" {

logos_status_t logos_rmsnorm(logos_handle_t x, logos_handle_t g, logos_handle_t y, int64_t rows, int64_t h,
                             float eps, void* stream_or_null) {
  return guarded([&]() -> logos_status_t {
    if (rows < 0 || h < 0) return fail(LOGOS_OUT_OF_BOUNDS, "logos_rmsnorm: negative extent");
    float *xp, *gp, *yp;
    int32_t dev = 0;
    LOGOS_TRY(buf_ptr<float>(x, rows * h, "x", &xp, &dev));
    LOGOS_TRY(buf_ptr<float>(g, h, "g", &gp));
    LOGOS_TRY(buf_ptr<float>(y, rows * h, "y", &yp));
    LOGOS_CUDA_TRY(cudaSetDevice(dev));
    return launch_rmsnorm_f32(xp, gp, yp, rows, h, eps, as_stream(stream_or_null));
  });
}

logos_status_t logos_swiglu(logos_handle_t gate, logos_handle_t up, logos_handle_t y, int64_t count,
                            void* stream_or_null) {
  return guarded([&]() -> logos_status_t {
    if (count < 0) return fail(LOGOS_OUT_OF_BOUNDS, "logos_swiglu: negative extent");
    float *gp, *up_p, *yp;
    int32_t dev = 0;
    LOGOS_TRY(buf_ptr<float>(gate, count, "gate", &gp, &dev));
    LOGOS_TRY(buf_ptr<float>(up, count, "up", &up_p));
    LOGOS_TRY(buf_ptr<float>(y, count, "y", &yp));
    LOGOS_CUDA_TRY(cudaSetDevice(dev));
    return launch_swiglu_f32(gp, up_p, yp, count, as_stream(stream_or_null));
  });
}

}  // extern "C"
