// Prompt processing (prefill): the two kernels between the qkv and o_proj GEMMs when a chunk of
// prompt positions of every sequence runs through a layer at once.
//
//   prefill_rope_kv_kernel    rotates q and k of every (sequence, position) of the chunk with the
//                             same f32 arithmetic as the decode path (product and sum rounded
//                             separately, fp16 result), writes the K and V rows into the cache and
//                             the rotated queries into an fp16 buffer
//   gqa_prefill_attn_kernel   causal attention of the chunk's queries over the cache: one CTA
//                             per (block of query positions, KV head, sequence); a producer
//                             thread streams 64-position K/V tiles through a 3-stage TMA ring
//                             (128-byte swizzle, no multicast); each of four warps owns 16 query
//                             rows = 16 / G positions x the G heads of the group, walks the four
//                             16-position slices of every tile with m16n8k16 MMAs, keeps scores,
//                             online softmax and output in f32 registers, and feeds the
//                             probabilities to the second MMA as fp16 high part + residual, as
//                             the decode kernel does.
// Rows of the chunk are ordered (sequence, position): row = b * chunk + j.
#include "ops.cuh"
#include "ptx.cuh"

#include <math.h>

namespace logos {

namespace {

using namespace ptx;

constexpr int PF_TILE = 64;
constexpr int PF_STAGES = 3;
constexpr int PF_CWARPS = 4;
constexpr int PF_CTHREADS = PF_CWARPS * 32;
constexpr int PF_THREADS = (PF_CWARPS + 1) * 32;
constexpr int PF_BOX_BYTES = 64 * 128;

struct PrefillAttnParams {
  const __half* q16;     // [rows][Hq * D] rotated queries
  __half*       k_cache; // [B][Hkv][Lmax][D]
  __half*       v_cache;
  ActOut        o;       // planes [rows][Hq * D]
  int           b, h_q, h_kv, l_max, chunk, pos0;
  float         scale_log2;
  int*          status;
};

__device__ __forceinline__ uint32_t pack_half2_pf(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// One thread per pair (e, e + D/2) of one head of one row.
__global__ void prefill_rope_kv_kernel(const float* __restrict__ qkv, int64_t ld, const float* __restrict__ bias,
                                       const float* __restrict__ rope, __half* __restrict__ q16,
                                       __half* __restrict__ k_cache, __half* __restrict__ v_cache, int h_q, int h_kv,
                                       int d, int l_max, int chunk, int pos0) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;                 // b * chunk + j
  const int b = row / chunk, j = row - b * chunk;
  const int pos = pos0 + j;
  const int half_d = d >> 1;
  const float* src = qkv + (int64_t)row * ld;
  const float* tab = rope + (int64_t)pos * half_d * 2;
  const int nq = h_q * d;
  const int heads = h_q + 2 * h_kv;
  for (int i = threadIdx.x; i < heads * half_d; i += blockDim.x) {
    const int head = i / half_d, e = i - head * half_d;
    const int col = head * d + e;            // q | k | v heads follow each other in the row
    float x1 = __ldcg(src + col), x2 = __ldcg(src + col + half_d);
    if (bias) {
      x1 = __fadd_rn(x1, __ldg(bias + col));
      x2 = __fadd_rn(x2, __ldg(bias + col + half_d));
    }
    if (head < h_q + h_kv) {                  // q and k heads are rotated, v is not
      const float c = tab[2 * e], s = tab[2 * e + 1];
      const float r1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
      const float r2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
      x1 = r1;
      x2 = r2;
    }
    const __half h1 = __float2half_rn(x1), h2 = __float2half_rn(x2);
    if (head < h_q) {
      __half* dst = q16 + (int64_t)row * nq + head * d;
      dst[e] = h1;
      dst[e + half_d] = h2;
    } else if (pos < l_max) {
      const int kvh = head < h_q + h_kv ? head - h_q : head - h_q - h_kv;
      __half* cache = head < h_q + h_kv ? k_cache : v_cache;
      __half* dst = cache + (((int64_t)b * h_kv + kvh) * l_max + pos) * d;
      dst[e] = h1;
      dst[e + half_d] = h2;
    }
  }
}

template <int D>
__global__ void __launch_bounds__(PF_THREADS)
gqa_prefill_attn_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const PrefillAttnParams p) {
  constexpr int NBOX = D / 64;
  constexpr int STAGE_BYTES = 2 * NBOX * PF_BOX_BYTES;
  constexpr int QS_STRIDE = D + 8;
  constexpr int KSTEPS = D / 16;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  __half* qs = reinterpret_cast<__half*>(stages + PF_STAGES * STAGE_BYTES);   // [warp][16][QS_STRIDE]
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(qs + PF_CWARPS * 16 * QS_STRIDE);
  uint64_t* bar_empty = bar_full + PF_STAGES;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.h_q / p.h_kv;
  const int PW = 16 / G;                       // query positions in a warp's 16 rows
  const int qpb = PF_CWARPS * PW;              // query positions of the CTA
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int j0 = blockIdx.x * qpb;             // first query position of the CTA inside the chunk
  const int j_end = min(j0 + qpb, p.chunk);    // one past its last
  // the CTA's last query attends to positions [0, pos0 + j_end): that many tiles are streamed
  const int ntiles = (p.pos0 + j_end + PF_TILE - 1) / PF_TILE;
  const int64_t row_base = ((int64_t)b * p.h_kv + kvh) * p.l_max;

  pdl_wait();
  pdl_trigger();
  __shared__ int prior_status;
  if (tid == 0) {
    prior_status = *reinterpret_cast<volatile int*>(p.status);
    for (int i = 0; i < PF_STAGES; ++i) {
      mbar_init(&bar_full[i], 1);
      mbar_init(&bar_empty[i], PF_CWARPS);
    }
    fence_barrier_init();
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  __syncthreads();
  if (prior_status != 0) return;

  if (warp == PF_CWARPS) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      bool ok = true;
      for (int t = 0; t < ntiles && ok; ++t) {
        const int st = t % PF_STAGES;
        const uint32_t ph = (uint32_t)(t / PF_STAGES) & 1u;
        ok = mbar_wait(&bar_empty[st], ph ^ 1u);
        if (!ok) break;
        uint8_t* sb = stages + st * STAGE_BYTES;
        mbar_arrive_expect_tx(&bar_full[st], STAGE_BYTES);
        const int y = (int)(row_base + (int64_t)t * PF_TILE);
#pragma unroll
        for (int jb = 0; jb < NBOX; ++jb) {
          tma_load_2d(sb + jb * PF_BOX_BYTES, &map_k, &bar_full[st], jb * 64, y);
          tma_load_2d(sb + (NBOX + jb) * PF_BOX_BYTES, &map_v, &bar_full[st], jb * 64, y);
        }
      }
      if (!ok) atomicExch(p.status, 111);
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  const int g4 = lane >> 2, t4 = lane & 3;
  // row r of the warp's tile: query position j0 + warp * PW + r / G, head r % G of the group
  __half* qw = qs + warp * 16 * QS_STRIDE;
  for (int i = lane; i < 16 * (D / 8); i += 32) {
    const int r = i / (D / 8), c8 = i - r * (D / 8);
    const int jj = r / G, g = r - jj * G;
    const int j = j0 + warp * PW + jj;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (jj < PW && j < p.chunk)
      v = __ldcg(reinterpret_cast<const uint4*>(p.q16 + ((int64_t)b * p.chunk + j) * p.h_q * D + (kvh * G + g) * D) + c8);
    *reinterpret_cast<uint4*>(qw + r * QS_STRIDE + c8 * 8) = v;
  }
  __syncwarp();
  uint32_t qa[KSTEPS][4];
  {
    const int row = (lane & 7) + 8 * ((lane >> 3) & 1);
    const int colh = 8 * (lane >> 4);
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
      ldmatrix_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], smem_u32(qw + row * QS_STRIDE + ks * 16 + colh));
  }
  // causal limits of this thread's two rows (g4 and g4 + 8): positions [0, lim) are attended to
  int lim[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g4 + 8 * h, jj = r / G;
    const int j = j0 + warp * PW + jj;
    lim[h] = (jj < PW && j < p.chunk) ? p.pos0 + j + 1 : 0;
  }
  // the furthest position any row of this warp attends to (rows of the warp are uniform per jj)
  int warp_lim = 0;
  {
    const int j_last = min(j0 + warp * PW + PW, p.chunk);
    warp_lim = j_last > j0 + warp * PW ? p.pos0 + j_last : 0;
  }

  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  bool ok = true;
  for (int t = 0; t < ntiles; ++t) {
    const int st = t % PF_STAGES;
    const uint32_t ph = (uint32_t)(t / PF_STAGES) & 1u;
    if (!mbar_wait(&bar_full[st], ph)) {
      ok = false;
      break;
    }
    uint8_t* kb = stages + st * STAGE_BYTES;
    uint8_t* vb = kb + NBOX * PF_BOX_BYTES;
#pragma unroll 1
    for (int sb = 0; sb < 4; ++sb) {
      const int pos_base = t * PF_TILE + 16 * sb;
      if (pos_base >= warp_lim) break;   // nothing left for this warp in the tile (warp-uniform)
      // ---- S = Q K^T for 16 positions
      float s[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      {
        const uint32_t row = 16 * sb + (lane & 7) + 8 * (lane >> 4);
        const int ch = (lane >> 3) & 1;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          const int chunk = ks * 2 + ch;
          uint32_t r0, r1, r2, r3;
          ldmatrix_x4(r0, r1, r2, r3, smem_u32(kb + (chunk >> 3) * PF_BOX_BYTES + swz128(row, chunk & 7)));
          mma_f16_16816(s[0], qa[ks], r0, r1);
          mma_f16_16816(s[1], qa[ks], r2, r3);
        }
      }
      // ---- causal mask, scale, online softmax
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int jx = 0; jx < 4; ++jx) {
          const int pos = pos_base + nt * 8 + 2 * t4 + (jx & 1);
          const float v = (pos < lim[jx >> 1]) ? s[nt][jx] * p.scale_log2 : -INFINITY;
          s[nt][jx] = v;
          mx[jx >> 1] = fmaxf(mx[jx >> 1], v);
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      }
      float corr[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float m_new = fmaxf(m_run[r], mx[r]);
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
        corr[r] = exp2f(m_run[r] - m_use[r]);
        m_run[r] = m_new;
      }
      float pr[2][4];
      float psum[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int jx = 0; jx < 4; ++jx) {
          const float e = exp2f(s[nt][jx] - m_use[jx >> 1]);
          pr[nt][jx] = e;
          psum[jx >> 1] += e;
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * corr[r] + psum[r];
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= corr[0]; o[i][1] *= corr[0];
        o[i][2] *= corr[1]; o[i][3] *= corr[1];
      }
      // ---- P as fp16 high part + fp16 residual
      uint32_t a_hi[4], a_lo[4];
      {
        const float h[8] = {pr[0][0], pr[0][1], pr[0][2], pr[0][3], pr[1][0], pr[1][1], pr[1][2], pr[1][3]};
        float lo[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) lo[i] = h[i] - __half2float(__float2half_rn(h[i]));
        a_hi[0] = pack_half2_pf(h[0], h[1]); a_hi[1] = pack_half2_pf(h[2], h[3]);
        a_hi[2] = pack_half2_pf(h[4], h[5]); a_hi[3] = pack_half2_pf(h[6], h[7]);
        a_lo[0] = pack_half2_pf(lo[0], lo[1]); a_lo[1] = pack_half2_pf(lo[2], lo[3]);
        a_lo[2] = pack_half2_pf(lo[4], lo[5]); a_lo[3] = pack_half2_pf(lo[6], lo[7]);
      }
      // ---- O += P V
      {
        const uint32_t row = 16 * sb + (lane & 7) + 8 * ((lane >> 3) & 1);
        const int ch = lane >> 4;
#pragma unroll
        for (int dn = 0; dn < D / 16; ++dn) {
          const int chunk = dn * 2 + ch;
          uint32_t r0, r1, r2, r3;
          ldmatrix_x4_trans(r0, r1, r2, r3, smem_u32(vb + (chunk >> 3) * PF_BOX_BYTES + swz128(row, chunk & 7)));
          mma_f16_16816(o[2 * dn], a_hi, r0, r1);
          mma_f16_16816(o[2 * dn], a_lo, r0, r1);
          mma_f16_16816(o[2 * dn + 1], a_hi, r2, r3);
          mma_f16_16816(o[2 * dn + 1], a_lo, r2, r3);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&bar_empty[st]);
  }
  if (!ok) {
    if (lane == 0) atomicExch(p.status, 112);
    return;
  }

  // ---- normalise and write: thread (g4, t4) holds columns 8 i + 2 t4, + 1 of rows g4 and g4 + 8
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g4 + 8 * h, jj = r / G, g = r - jj * G;
    const int j = j0 + warp * PW + jj;
    if (jj >= PW || j >= p.chunk) continue;
    const int64_t base = ((int64_t)b * p.chunk + j) * p.h_q * D + (kvh * G + g) * D;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int col = i * 8 + 2 * t4;
      act_store(p.o, base + col, __fdiv_rn(o[i][2 * h], l_run[h]));
      act_store(p.o, base + col + 1, __fdiv_rn(o[i][2 * h + 1], l_run[h]));
    }
  }
}

template <int D>
logos_status_t launch_prefill_attn_t(const PrefillAttnArgs& a, cudaStream_t st) {
  const int64_t rows_total = a.b * a.h_kv * a.l_max;
  CUtensorMap mk, mv;
  LOGOS_TRY(make_tensor_map_2d(&mk, a.k_cache, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, D, rows_total, D * 2, 64, PF_TILE,
                               CU_TENSOR_MAP_SWIZZLE_128B));
  LOGOS_TRY(make_tensor_map_2d(&mv, a.v_cache, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, D, rows_total, D * 2, 64, PF_TILE,
                               CU_TENSOR_MAP_SWIZZLE_128B));
  PrefillAttnParams p{};
  p.q16 = a.q16; p.k_cache = a.k_cache; p.v_cache = a.v_cache; p.o = a.o;
  p.b = (int)a.b; p.h_q = (int)a.h_q; p.h_kv = (int)a.h_kv; p.l_max = (int)a.l_max;
  p.chunk = (int)a.chunk; p.pos0 = (int)a.pos0;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.status = kernel_status_ptr(a.device);
  if (!p.status) return fail(LOGOS_ERROR, "prefill attention: no kernel status word");
  const int G = (int)(a.h_q / a.h_kv);
  const int qpb = PF_CWARPS * (16 / G);
  constexpr size_t smem = 1024 + (size_t)PF_STAGES * 2 * (D / 64) * PF_BOX_BYTES + (size_t)PF_CWARPS * 16 * (D + 8) * 2 +
                          2 * PF_STAGES * 8 + 64;
  LOGOS_CUDA_TRY(cudaFuncSetAttribute(gqa_prefill_attn_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)((a.chunk + qpb - 1) / qpb), (unsigned)a.h_kv, (unsigned)a.b);
  LOGOS_CUDA_TRY(launch_kernel(gqa_prefill_attn_kernel<D>, grid, dim3(PF_THREADS), smem, st, mk, mv, p));
  count_launch(LK_ATTN);
  return check_launch("gqa_prefill_attn_kernel");
}

}  // namespace

logos_status_t launch_prefill_attn(const PrefillAttnArgs& a, cudaStream_t st) {
  if (a.b == 0 || a.chunk == 0 || a.h_q == 0) return LOGOS_OK;
  if (a.h_kv <= 0 || a.h_q % a.h_kv) return fail(LOGOS_ERROR, "prefill attention: h_q must be a multiple of h_kv");
  if (a.h_q / a.h_kv > 16) return fail(LOGOS_ERROR, "prefill attention: at most 16 query heads per KV head");
  if (a.pos0 < 0 || a.pos0 + a.chunk > a.l_max)
    return fail(LOGOS_OUT_OF_BOUNDS, "prefill attention: positions [%lld, %lld) exceed l_max = %lld", (long long)a.pos0,
                (long long)(a.pos0 + a.chunk), (long long)a.l_max);
  // rotate q and k, write the chunk's K/V rows and the fp16 queries
  {
    const int64_t rows = a.b * a.chunk;
    const int64_t pairs = (a.h_q + 2 * a.h_kv) * (a.d / 2);
    const int threads = (int)(pairs < 256 ? ((pairs + 31) / 32) * 32 : 256);
    LOGOS_CUDA_TRY(launch_kernel(prefill_rope_kv_kernel, dim3((unsigned)rows), dim3((unsigned)threads), 0, st, a.qkv,
                                 a.qkv_ld, a.qkv_bias, a.rope, a.q16, a.k_cache, a.v_cache, (int)a.h_q, (int)a.h_kv,
                                 (int)a.d, (int)a.l_max, (int)a.chunk, (int)a.pos0));
    count_launch(LK_ELEMWISE);
    LOGOS_TRY(check_launch("prefill_rope_kv_kernel"));
  }
  if (a.d == 128) return launch_prefill_attn_t<128>(a, st);
  if (a.d == 64) return launch_prefill_attn_t<64>(a, st);
  return fail(LOGOS_ERROR, "prefill attention: head_dim %lld is not supported (64 or 128)", (long long)a.d);
}

}  // namespace logos
