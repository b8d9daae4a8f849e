// Q8 GEMM front: C[m,n] = sum_kb s[n,kb] * sum_k A[m,k] * q[n,k].
//
// Dispatch between two kernels:
//   * q8_gemm_tc.cu — the tcgen05 / TMA kernel used for every shape the decode
//     step produces (K a multiple of 128, N a multiple of 128, M <= 256);
//   * the SIMT kernel below — any other shape, and the on-device cross-check
//     the tests hold the tensor-core kernel against.
// Plus the split-K reduction + epilogue kernel shared by both.
#include "ops.cuh"
#include "q8_gemm_tc.cuh"

namespace logos {

namespace {

__device__ __forceinline__ float load_act(const void* a, int dtype, int64_t i, const __half* lo = nullptr) {
  if (dtype == LOGOS_F16) return act_load(reinterpret_cast<const __half*>(a), lo, i);
  if (dtype == LOGOS_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a)[i]);
  return reinterpret_cast<const float*>(a)[i];
}
__device__ __forceinline__ void store_out(void* c, int dtype, int64_t i, float v, const ActOut& planes) {
  if (dtype == LOGOS_ACT_PLANES) act_store(planes, i, v);
  else if (dtype == LOGOS_F16) reinterpret_cast<__half*>(c)[i] = __float2half_rn(v);
  else if (dtype == LOGOS_BF16) reinterpret_cast<__nv_bfloat16*>(c)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(c)[i] = v;
}
__device__ __forceinline__ float silu_f(float g) { return __fdiv_rn(g, 1.0f + expf(-g)); }

constexpr int SIMT_TN = 32;  // weight rows per CTA
constexpr int SIMT_TM = 32;  // tokens per CTA

// 256 threads: lane = weight row inside the tile, warp w owns tokens 4w..4w+3.
__global__ void __launch_bounds__(256)
q8_gemm_simt_kernel(const void* __restrict__ a, const __half* __restrict__ a_lo, int a_dtype, int64_t lda,
                    const int8_t* __restrict__ q, const float* __restrict__ s, void* __restrict__ c, int c_dtype,
                    ActOut c_act, int64_t ldc,
                    const void* __restrict__ aux, float* __restrict__ partials, int64_t m, int64_t n, int64_t k,
                    int epilogue, int splits) {
  __shared__ float as[SIMT_TM][33];
  __shared__ float qs[SIMT_TN][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t n0 = (int64_t)blockIdx.x * SIMT_TN, m0 = (int64_t)blockIdx.y * SIMT_TM;
  const int64_t kb_total = k / 32;
  const int split = blockIdx.z;
  const int64_t kb_per = (kb_total + splits - 1) / splits;
  const int64_t kb_begin = split * kb_per;
  const int64_t kb_end = kb_begin + kb_per < kb_total ? kb_begin + kb_per : kb_total;
  const int64_t row = n0 + lane;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int64_t kb = kb_begin; kb < kb_end; ++kb) {
    for (int i = threadIdx.x; i < SIMT_TM * 32; i += 256) {
      int r = i >> 5, cidx = i & 31;
      as[r][cidx] = (m0 + r < m) ? load_act(a, a_dtype, (m0 + r) * lda + kb * 32 + cidx, a_lo) : 0.f;
      qs[r][cidx] = (n0 + r < n) ? (float)q[(n0 + r) * k + kb * 32 + cidx] : 0.f;
    }
    __syncthreads();
    float p[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kk = 0; kk < 32; ++kk) {
      float qv = qs[lane][kk];
#pragma unroll
      for (int j = 0; j < 4; ++j) p[j] = fmaf(as[warp * 4 + j][kk], qv, p[j]);
    }
    float sc = (row < n) ? s[row * kb_total + kb] : 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = fmaf(sc, p[j], acc[j]);
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int64_t mm = m0 + warp * 4 + j;
    float v = acc[j];
    if (splits > 1) {
      if (mm < m && row < n) partials[((int64_t)split * m + mm) * n + row] = v;
      continue;
    }
    if (epilogue == EPI_SWIGLU) {
      float other = __shfl_xor_sync(0xffffffffu, v, 1);
      if (!(lane & 1) && mm < m && row + 1 < n) store_out(c, c_dtype, mm * ldc + (row >> 1), __fmul_rn(silu_f(v), other), c_act);
    } else if (mm < m && row < n) {
      if (epilogue == EPI_RESIDUAL) v = __fadd_rn(v, load_act(aux, c_dtype, mm * ldc + row));
      store_out(c, c_dtype, mm * ldc + row, v, c_act);
    }
  }
}

// Sum split-K partials in ascending split order, then apply the epilogue.
__global__ void splitk_reduce_kernel(const float* __restrict__ partials, int splits, void* __restrict__ c, int c_dtype,
                                     ActOut c_act, int64_t ldc, const void* __restrict__ aux, int64_t m, int64_t n,
                                     int epilogue) {
  pdl_wait();  // the partials are the previous kernel's output: wait for it, read them past L1
  pdl_trigger();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (epilogue == EPI_SWIGLU) {
    int64_t half_n = n / 2;
    if (i >= m * half_n) return;
    int64_t mm = i / half_n, j = i - mm * half_n;
    float g = 0.f, u = 0.f;
    for (int sp = 0; sp < splits; ++sp) {
      const float2 gu = __ldcg(reinterpret_cast<const float2*>(partials + ((int64_t)sp * m + mm) * n + 2 * j));
      g = __fadd_rn(g, gu.x);
      u = __fadd_rn(u, gu.y);
    }
    store_out(c, c_dtype, mm * ldc + j, __fmul_rn(silu_f(g), u), c_act);
    return;
  }
  if (i >= m * n) return;
  int64_t mm = i / n, nn = i - mm * n;
  float v = 0.f;
  for (int sp = 0; sp < splits; ++sp) v = __fadd_rn(v, __ldcg(partials + ((int64_t)sp * m + mm) * n + nn));
  if (epilogue == EPI_RESIDUAL) v = __fadd_rn(v, load_act(aux, c_dtype, mm * ldc + nn));
  store_out(c, c_dtype, mm * ldc + nn, v, c_act);
}

}  // namespace

int gemm_pick_splits(int64_t m, int64_t n, int64_t k, int device) {
  // Work units are (tile of 128 weight rows) x (K split); a CTA's time is a fixed part (pipeline
  // fill, epilogue: about twelve stage times, measured) plus its K stages, and CTAs run in
  // rounds of one per SM.  Take the split count with the smallest rounds x (fixed + stages);
  // ties go to fewer splits (fewer partials to write and fold).
  // (a row tile for each token tile of 64 is a unit of its own: with many tokens there are enough)
  const int64_t tiles = ((n + 127) / 128) * ((m + 63) / 64 > 0 ? (m + 63) / 64 : 1);
  const int64_t stages = k / 128;
  const int sms = sm_count(device);
  if (tiles >= sms || stages < 8) return 1;
  const int64_t fixed = 12;
  int64_t max_splits = stages / 4;  // at least 4 stages (512 columns) per split
  if (max_splits > 16) max_splits = 16;
  int best = 1;
  int64_t best_cost = INT64_MAX;
  for (int64_t sp = 1; sp <= max_splits; ++sp) {
    const int64_t rounds = (tiles * sp + sms - 1) / sms;
    const int64_t per = (stages + sp - 1) / sp;
    const int64_t cost = rounds * (fixed + per) * 8 + sp;
    if (cost < best_cost) { best_cost = cost; best = (int)sp; }
  }
  return best;
}

logos_status_t launch_splitk_reduce(const float* partials, int splits, void* c, int c_dtype, ActOut c_act,
                                    int64_t ldc, const void* aux, int64_t m, int64_t n, int epilogue,
                                    cudaStream_t st) {
  int64_t total = (epilogue == EPI_SWIGLU) ? m * (n / 2) : m * n;
  if (total == 0) return LOGOS_OK;
  LOGOS_CUDA_TRY(launch_kernel(splitk_reduce_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, partials, splits,
                               c, c_dtype, c_act, ldc, aux, m, n, epilogue));
  count_launch(LK_ELEMWISE);
  return check_launch("splitk_reduce_kernel");
}

logos_status_t launch_q8_gemm(const GemmArgs& g, cudaStream_t st) {
  if (g.m == 0 || g.n == 0) return LOGOS_OK;
  if (g.k % 32) return fail(LOGOS_OUT_OF_BOUNDS, "q8_gemm: K=%lld is not a multiple of the block size 32", (long long)g.k);
  if (g.epilogue == EPI_SWIGLU && (g.n & 1)) return fail(LOGOS_OUT_OF_BOUNDS, "q8_gemm: swiglu epilogue needs even N");
  if (g.splits > 1 && (!g.partials || g.epilogue != EPI_NONE))
    return fail(LOGOS_ERROR, "q8_gemm: split-K writes raw partials; the caller reduces them");
  if (!g.force_simt && gemm_tc_applicable(g)) return launch_q8_gemm_tc(g, st);
  if (g.q_tiled) return fail(LOGOS_ERROR, "q8_gemm: tile-major weights need the tensor-core kernel, which does not take this call");
  dim3 grid((unsigned)((g.n + SIMT_TN - 1) / SIMT_TN), (unsigned)((g.m + SIMT_TM - 1) / SIMT_TM),
            (unsigned)(g.splits > 1 ? g.splits : 1));
  q8_gemm_simt_kernel<<<grid, 256, 0, st>>>(g.a, g.a_lo, g.a_dtype, g.lda, g.q, g.s, g.c, g.c_dtype, g.c_act, g.ldc,
                                            g.aux, g.partials, g.m, g.n, g.k, g.epilogue,
                                            g.splits > 1 ? g.splits : 1);
  count_launch(LK_GEMM_SIMT);
  return check_launch("q8_gemm_simt_kernel");
}

}  // namespace logos

using namespace logos;

static logos_status_t gemm_abi(logos_handle_t a, logos_handle_t q, logos_handle_t s, logos_handle_t c, int64_t m,
                               int64_t n, int64_t k, int32_t epilogue, logos_handle_t aux, void* stream,
                               int force_simt) {
  if (m < 0 || n < 0 || k < 0) return fail(LOGOS_OUT_OF_BOUNDS, "logos_q8_gemm: negative extent");
  if (k % 32) return fail(LOGOS_OUT_OF_BOUNDS, "logos_q8_gemm: K=%lld is not a multiple of the block size 32", (long long)k);
  if (epilogue < 0 || epilogue > 2) return fail(LOGOS_ERROR, "logos_q8_gemm: unknown epilogue %d", epilogue);
  if (epilogue == EPI_SWIGLU && (n & 1)) return fail(LOGOS_OUT_OF_BOUNDS, "logos_q8_gemm: swiglu epilogue needs even N");
  int64_t n_out = epilogue == EPI_SWIGLU ? n / 2 : n;
  __nv_bfloat16 *ap, *cp, *xp = nullptr;
  int8_t* qp;
  float* sp;
  int32_t dev = 0;
  LOGOS_TRY(buf_ptr<__nv_bfloat16>(a, m * k, "a", &ap, &dev));
  LOGOS_TRY(buf_ptr<int8_t>(q, n * k, "q", &qp));
  LOGOS_TRY(buf_ptr<float>(s, n * (k / 32), "s", &sp));
  LOGOS_TRY(buf_ptr<__nv_bfloat16>(c, m * n_out, "c", &cp));
  if (epilogue == EPI_RESIDUAL) {
    if (!aux) return fail(LOGOS_NULL_POINTER, "logos_q8_gemm: residual epilogue needs aux");
    LOGOS_TRY(buf_ptr<__nv_bfloat16>(aux, m * n, "aux", &xp));
  }
  LOGOS_CUDA_TRY(cudaSetDevice(dev));
  GemmArgs g;
  g.a = ap; g.a_dtype = LOGOS_BF16; g.lda = k;
  g.q = qp; g.s = sp;
  g.c = cp; g.c_dtype = LOGOS_BF16; g.ldc = n_out;
  g.aux = xp;
  g.m = m; g.n = n; g.k = k;
  g.epilogue = epilogue;
  g.device = dev;
  g.force_simt = force_simt;
  cudaStream_t st = as_stream(stream);
  if (force_simt) return launch_q8_gemm(g, st);
  // Tensor-core path: the kernel multiplies fp16 planes.  A bf16 value is exactly
  // representable in fp16 inside fp16's normal range, so one plane is enough.
  GemmArgs t = g;
  t.a_dtype = LOGOS_F16;
  t.a = reinterpret_cast<const void*>(uintptr_t(16));  // placeholder so applicability can be asked first
  if (!gemm_tc_applicable(t)) return launch_q8_gemm(g, st);
  int splits = gemm_pick_splits(m, n, k, dev);
  void* scratch = nullptr;
  int64_t plane_bytes = ((m * k * 2 + 255) / 256) * 256;
  int64_t part_bytes = splits > 1 ? (int64_t)splits * m * n * (int64_t)sizeof(float) : 0;
  LOGOS_TRY(scratch_get(dev, 0, plane_bytes + part_bytes, &scratch));
  __half* plane = reinterpret_cast<__half*>(scratch);
  LOGOS_TRY(launch_bf16_to_f16(ap, plane, m * k, st));
  t.a = plane;
  if (splits > 1) {
    GemmArgs gp = t;
    gp.splits = splits;
    gp.partials = reinterpret_cast<float*>(static_cast<char*>(scratch) + plane_bytes);
    gp.epilogue = EPI_NONE;
    gp.c = nullptr;
    LOGOS_TRY(launch_q8_gemm(gp, st));
    return launch_splitk_reduce(gp.partials, splits, cp, LOGOS_BF16, ActOut(), n_out, xp, m, n, epilogue, st);
  }
  return launch_q8_gemm(t, st);
}

extern "C" {

#ifdef LOGOS_TC_TRACE
// Development builds only: CTA (0,0,0) of every tcgen05 GEMM launch stores SM-clock timestamps of
// its pipeline roles per K stage ([stage][16]) into this buffer of at least 64*16 int64; null
// turns it off.
__attribute__((visibility("default"))) logos_status_t logos_gemm_trace_buffer(logos_handle_t buf_or_null) {
  return guarded([&]() -> logos_status_t {
    if (!buf_or_null) {
      gemm_set_trace(nullptr);
      return LOGOS_OK;
    }
    long long* p = nullptr;
    LOGOS_TRY(buf_ptr<long long>(buf_or_null, 64 * 16, "trace", &p));
    gemm_set_trace(p);
    return LOGOS_OK;
  });
}
#endif

// f32 activations, f32 output: the form the decode step uses internally (the
// activations are split into two fp16 planes so the tensor-core product keeps
// f32-class accuracy).
logos_status_t logos_q8_gemm_f32(logos_handle_t a, logos_handle_t q, logos_handle_t s, logos_handle_t c, int64_t m,
                                 int64_t n, int64_t k, void* stream_or_null) {
  return guarded([&]() -> logos_status_t {
    if (m < 0 || n < 0 || k < 0) return fail(LOGOS_OUT_OF_BOUNDS, "logos_q8_gemm_f32: negative extent");
    if (k % 32) return fail(LOGOS_OUT_OF_BOUNDS, "logos_q8_gemm_f32: K=%lld is not a multiple of the block size 32", (long long)k);
    float *ap, *sp, *cp;
    int8_t* qp;
    int32_t dev = 0;
    LOGOS_TRY(buf_ptr<float>(a, m * k, "a", &ap, &dev));
    LOGOS_TRY(buf_ptr<int8_t>(q, n * k, "q", &qp));
    LOGOS_TRY(buf_ptr<float>(s, n * (k / 32), "s", &sp));
    LOGOS_TRY(buf_ptr<float>(c, m * n, "c", &cp));
    LOGOS_CUDA_TRY(cudaSetDevice(dev));
    cudaStream_t st = as_stream(stream_or_null);
    GemmArgs g;
    g.a = ap; g.a_dtype = LOGOS_F32; g.lda = k;
    g.q = qp; g.s = sp;
    g.c = cp; g.c_dtype = LOGOS_F32; g.ldc = n;
    g.m = m; g.n = n; g.k = k;
    g.device = dev;
    GemmArgs t = g;
    t.a_dtype = LOGOS_F16;
    t.a = reinterpret_cast<const void*>(uintptr_t(16));
    if (m == 0 || n == 0 || !gemm_tc_applicable(t)) return launch_q8_gemm(g, st);
    int splits = gemm_pick_splits(m, n, k, dev);
    int64_t plane_bytes = ((m * k * 2 + 255) / 256) * 256;
    int64_t part_bytes = splits > 1 ? (int64_t)splits * m * n * (int64_t)sizeof(float) : 0;
    void* scratch = nullptr;
    LOGOS_TRY(scratch_get(dev, 0, 2 * plane_bytes + part_bytes, &scratch));
    ActOut planes;
    planes.hi = reinterpret_cast<__half*>(scratch);
    planes.lo = reinterpret_cast<__half*>(static_cast<char*>(scratch) + plane_bytes);
    planes.mode = LOGOS_F32;
    LOGOS_TRY(launch_act_split(ap, planes, m * k, st));
    t.a = planes.hi;
    t.a_lo = planes.lo;
    if (splits > 1) {
      t.splits = splits;
      t.partials = reinterpret_cast<float*>(static_cast<char*>(scratch) + 2 * plane_bytes);
      t.c = nullptr;
      LOGOS_TRY(launch_q8_gemm(t, st));
      return launch_splitk_reduce(t.partials, splits, cp, LOGOS_F32, ActOut(), n, nullptr, m, n, EPI_NONE, st);
    }
    return launch_q8_gemm(t, st);
  });
}

logos_status_t logos_q8_gemm(logos_handle_t a, logos_handle_t q, logos_handle_t s, logos_handle_t c, int64_t m,
                             int64_t n, int64_t k, int32_t epilogue, logos_handle_t aux_or_null,
                             void* stream_or_null) {
  return guarded([&]() -> logos_status_t {
    return gemm_abi(a, q, s, c, m, n, k, epilogue, aux_or_null, stream_or_null, 0);
  });
}

// Same contract as logos_q8_gemm, always on the SIMT kernel: the on-device
// cross-check for the tensor-core path.
logos_status_t logos_q8_gemm_simt(logos_handle_t a, logos_handle_t q, logos_handle_t s, logos_handle_t c, int64_t m,
                                  int64_t n, int64_t k, int32_t epilogue, logos_handle_t aux_or_null,
                                  void* stream_or_null) {
  return guarded([&]() -> logos_status_t {
    return gemm_abi(a, q, s, c, m, n, k, epilogue, aux_or_null, stream_or_null, 1);
  });
}

}  // extern "C"
