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
#include "synth.cuh"

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
                             const float* __restrict__ s, float* __restrict__ h, int64_t hidden, int tiled) {
  pdl_wait();
  pdl_trigger();
  int64_t row = blockIdx.x;
  int64_t t = __ldcg(tokens + row);
  if (tiled) {
    // element (t, e) of the tile-major form: tile (t / 128, e / 128), row t % 128, byte e % 128;
    // its scale: the same tile's [128 rows][4] block, row t % 128, entry (e % 128) / 32
    const int64_t tile0 = ((t >> 7) * (hidden >> 7) * 128 + (t & 127));
    const int8_t* base = q + tile0 * 128;
    const float* sbase = s + tile0 * 4;
    for (int64_t e = threadIdx.x; e < hidden; e += blockDim.x)
      h[row * hidden + e] = __fmul_rn(sbase[(e >> 7) * 512 + ((e & 127) >> 5)],
                                      (float)((int)(uint8_t)base[(e >> 7) * 16384 + (e & 127)] - 128));  // bytes hold q + 128
    return;
  }
  const float* sr = s + t * (hidden / 32);
  const int8_t* qr = q + t * hidden;
  for (int64_t e = threadIdx.x; e < hidden; e += blockDim.x)
    h[row * hidden + e] = __fmul_rn(sr[e >> 5], (float)qr[e]);
}

// One CTA per row, 128-bit accesses: fold the split-K partials into the residual
// stream in ascending order, keep the updated row on chip, reduce the sum of squares,
// then write the normalised row as activation planes.  Rows of up to 8192 floats stay in
// registers (IN_REGS): the kernel then uses no dynamic shared memory, so under a dependent
// launch the next GEMM's CTAs, which take nearly a whole SM's shared memory, can start beside
// it and fetch their first weights while the norm finishes.  Longer rows go through shared memory.
template <bool IN_REGS>
__global__ void __launch_bounds__(512)
residual_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta, int parts, int64_t part_stride,
                        const float* __restrict__ g, ActOut xn, int64_t hidden, float eps) {
  __shared__ float red[32];
  extern __shared__ float4 row_cache4[];  // hidden floats (not IN_REGS)
  float* row_cache = reinterpret_cast<float*>(row_cache4);
  // h and the partials come from kernels of the same step: wait for them, and read them past L1
  pdl_wait();
  pdl_trigger();
  const int64_t row = blockIdx.x;
  float* hr = h + row * hidden;
  float ss = 0.f;
  if (IN_REGS) {
    constexpr int PER = 4;   // float4 per thread: 512 threads x 4 x 4 floats = 8192
    const int64_t n4 = hidden >> 2;
    float4* hr4 = reinterpret_cast<float4*>(hr);
    float4 v[PER];
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int64_t i = threadIdx.x + (int64_t)u * 512;
      v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < n4) {
        v[u] = __ldcg(hr4 + i);
        for (int p = 0; p < parts; ++p) {
          const float4 d = __ldcg(reinterpret_cast<const float4*>(delta + (int64_t)p * part_stride + row * hidden) + i);
          v[u].x = __fadd_rn(v[u].x, d.x); v[u].y = __fadd_rn(v[u].y, d.y);
          v[u].z = __fadd_rn(v[u].z, d.z); v[u].w = __fadd_rn(v[u].w, d.w);
        }
        if (parts > 0) hr4[i] = v[u];
      }
    }
    // the same order of additions as the strided loop over the row: element i of thread t is t + 512 u
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      ss = fmaf(v[u].x, v[u].x, ss); ss = fmaf(v[u].y, v[u].y, ss);
      ss = fmaf(v[u].z, v[u].z, ss); ss = fmaf(v[u].w, v[u].w, ss);
    }
    ss = block_sum(ss, red);
    const float inv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)hidden), eps)));
    const float4* g4 = reinterpret_cast<const float4*>(g);
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int64_t i = threadIdx.x + (int64_t)u * 512;
      if (i < n4) {
        const float4 gg = g4[i];
        const int64_t e = row * hidden + 4 * i;
        act_store(xn, e + 0, __fmul_rn(__fmul_rn(v[u].x, inv), gg.x));
        act_store(xn, e + 1, __fmul_rn(__fmul_rn(v[u].y, inv), gg.y));
        act_store(xn, e + 2, __fmul_rn(__fmul_rn(v[u].z, inv), gg.z));
        act_store(xn, e + 3, __fmul_rn(__fmul_rn(v[u].w, inv), gg.w));
      }
    }
    return;
  }
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

// ---- residual + RMSNorm with the tensor-parallel exchange folded in (see ops.cuh)
// Data travels between ranks as 16-byte slots {word, epoch, word, epoch}, each written by ONE
// 16-byte store: a reader that finds both epoch words equal to the current call's number has
// the two data words of that same store, so no flag, fence or barrier separates the payload
// from its arrival, and every transfer is a one-way push over NVLink.
__device__ __forceinline__ void ll_store(uint4* p, uint32_t a, uint32_t b, uint32_t epoch) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(epoch), "r"(b), "r"(epoch)
               : "memory");
}
// Bounded poll.  The sender is another process on another GPU and may lag (by a graph
// instantiation, say), so a thread's waits of one kernel share ONE budget of about four seconds
// of SM clock counted from the thread's first unsuccessful poll: `*deadline` is 0 until then.
// False when the slot did not carry this epoch in time; the caller then stops waiting
// altogether (a launch with a dead peer costs one budget, not one per slot).
constexpr long long kPeerWaitCycles = 8000000000ll;
__device__ __forceinline__ bool ll_load(const uint4* p, uint32_t epoch, uint32_t* a, uint32_t* b, long long* deadline) {
  uint4 v;
  for (int spin = 0;; ++spin) {
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    if (v.y == epoch && v.w == epoch) {
      *a = v.x;
      *b = v.z;
      return true;
    }
    if ((spin & 255) == 255) {
      const long long now = clock64();
      if (*deadline == 0) *deadline = now + kPeerWaitCycles;
      else if (now > *deadline) return false;
    }
  }
}

constexpr int TP_CLUSTER = 4;  // CTAs per row: a rank owns fewer rows than there are SMs

// grid = rows x TP_CLUSTER, cluster = the TP_CLUSTER slices of one row.  Every rank runs it:
//   A  each CTA sums its slice of this rank's split-K partials and pushes it to the row's owner;
//   B  the owner's CTAs wait for every rank's slice, add them (rank order) to the residual
//      stream, reduce the sum of squares across the cluster, normalise, and push the row's
//      activation words to every rank;
//   C  each CTA waits for its slice of the normalised row and unpacks it into this rank's planes.
// No CTA waits before it has pushed, so the waits cannot form a cycle.
__global__ void __launch_bounds__(512)
tp_residual_rmsnorm_kernel(float* __restrict__ h, const TpFusedArgs t, int parts, int64_t part_stride,
                           const float* __restrict__ g, int64_t rows_own, int64_t hidden, float eps, int* status) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float red[32];
  __shared__ float slice_ss;
  __shared__ uint32_t epoch_s;
  extern __shared__ float4 row_cache4[];  // this CTA's slice of the row
  const int tid = threadIdx.x;
  pdl_wait();  // this rank's own GEMM has completed: its partials are in this GPU's memory
  pdl_trigger();
  if (tid == 0) epoch_s = *reinterpret_cast<volatile uint32_t*>(t.flags + 16) + 1u;
  __syncthreads();
  const uint32_t e = epoch_s;
  const unsigned crank = cluster.block_rank();
  const int64_t row = blockIdx.x / TP_CLUSTER;
  const int owner = (int)(row / rows_own);
  const int64_t row_local = row - (int64_t)owner * rows_own;
  const bool mine = owner == t.rank;
  const int64_t n4 = hidden >> 2, per = n4 / TP_CLUSTER;  // float4 per row, per CTA
  const int64_t slots_per_row = hidden >> 1;               // 16-byte slots per row (two words each)
  // A code left behind by an earlier kernel (a wait that gave up, here or in a GEMM) means the
  // ranks are no longer in step: push as usual, so that no peer waits for this rank longer
  // than it must, but wait for nobody.
  bool ok = *reinterpret_cast<volatile int*>(status) == 0;
  const bool ok_at_entry = ok;
  long long deadline = 0;

  // ---- A: push this rank's contribution to the row's owner
  {
    uint4* inbox = t.inbox_part[owner] + ((int64_t)t.rank * rows_own + row_local) * slots_per_row;
    for (int64_t i = tid; i < per; i += blockDim.x) {
      const int64_t i4 = (int64_t)crank * per + i;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < parts; ++p) {
        const float4 d = __ldcg(reinterpret_cast<const float4*>(t.partials + (int64_t)p * part_stride + row * hidden) + i4);
        v.x = __fadd_rn(v.x, d.x); v.y = __fadd_rn(v.y, d.y); v.z = __fadd_rn(v.z, d.z); v.w = __fadd_rn(v.w, d.w);
      }
      ll_store(inbox + 2 * i4, __float_as_uint(v.x), __float_as_uint(v.y), e);
      ll_store(inbox + 2 * i4 + 1, __float_as_uint(v.z), __float_as_uint(v.w), e);
    }
  }

  // ---- B: the owner folds, normalises and publishes
  if (mine) {
    float4* hr4 = reinterpret_cast<float4*>(h) + row * n4;
    float ss = 0.f;
    for (int64_t i = tid; i < per; i += blockDim.x) {
      const int64_t i4 = (int64_t)crank * per + i;
      float4 v = __ldcg(hr4 + i4);
      for (int src = 0; src < t.degree; ++src) {
        const uint4* in = t.inbox_part[t.rank] + ((int64_t)src * rows_own + row_local) * slots_per_row + 2 * i4;
        uint32_t a0, a1, a2, a3;
        if (!ok || !ll_load(in, e, &a0, &a1, &deadline) || !ll_load(in + 1, e, &a2, &a3, &deadline)) {
          ok = false;
          a0 = a1 = a2 = a3 = 0u;
        }
        v.x = __fadd_rn(v.x, __uint_as_float(a0)); v.y = __fadd_rn(v.y, __uint_as_float(a1));
        v.z = __fadd_rn(v.z, __uint_as_float(a2)); v.w = __fadd_rn(v.w, __uint_as_float(a3));
      }
      hr4[i4] = v;
      row_cache4[i] = v;
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = block_sum(ss, red);
    if (tid == 0) slice_ss = ss;
    cluster.sync();
    float total = 0.f;
    for (unsigned r = 0; r < TP_CLUSTER; ++r) total += *cluster.map_shared_rank(&slice_ss, r);
    const float inv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)hidden), eps)));
    const float4* g4 = reinterpret_cast<const float4*>(g);
    for (int64_t i = tid; i < per; i += blockDim.x) {
      const int64_t i4 = (int64_t)crank * per + i;
      const float4 v = row_cache4[i], gg = g4[i4];
      const float o[4] = {__fmul_rn(__fmul_rn(v.x, inv), gg.x), __fmul_rn(__fmul_rn(v.y, inv), gg.y),
                          __fmul_rn(__fmul_rn(v.z, inv), gg.z), __fmul_rn(__fmul_rn(v.w, inv), gg.w)};
      uint32_t pk[4];  // low half: hi plane, high half: lo plane
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float x = o[k];
        if (t.act_mode == LOGOS_BF16) x = __bfloat162float(__float2bfloat16_rn(x));
        x = act_clamp(x);
        const __half hh = __float2half_rn(x);
        const __half ll = __float2half_rn((x - __half2float(hh)) * 2048.f);
        pk[k] = (uint32_t)__half_as_ushort(hh) | ((uint32_t)__half_as_ushort(ll) << 16);
      }
      for (int r = 0; r < t.degree; ++r) {
        uint4* out = t.inbox_xn[r] + row * slots_per_row + 2 * i4;
        ll_store(out, pk[0], pk[1], e);
        ll_store(out + 1, pk[2], pk[3], e);
      }
    }
    cluster.sync();  // no CTA leaves while a peer of its cluster may still read its slice_ss
  }

  // ---- C: unpack this CTA's slice of the normalised row into the plain planes
  {
    const uint4* in = t.inbox_xn[t.rank] + row * slots_per_row;
    for (int64_t i = tid; i < per; i += blockDim.x) {
      const int64_t i4 = (int64_t)crank * per + i;
      uint32_t pk[4];
      if (!ok || !ll_load(in + 2 * i4, e, &pk[0], &pk[1], &deadline) ||
          !ll_load(in + 2 * i4 + 1, e, &pk[2], &pk[3], &deadline)) {
        ok = false;
        pk[0] = pk[1] = pk[2] = pk[3] = 0u;
      }
      uint2 hi2, lo2;
      hi2.x = (pk[0] & 0xffffu) | (pk[1] << 16);
      hi2.y = (pk[2] & 0xffffu) | (pk[3] << 16);
      lo2.x = (pk[0] >> 16) | (pk[1] & 0xffff0000u);
      lo2.y = (pk[2] >> 16) | (pk[3] & 0xffff0000u);
      reinterpret_cast<uint2*>(t.xn_hi + row * hidden)[i4] = hi2;
      if (t.xn_lo) reinterpret_cast<uint2*>(t.xn_lo + row * hidden)[i4] = lo2;
    }
  }
  if (!ok && ok_at_entry) atomicCAS(status, 0, 3030);
  // the last CTA to finish advances this rank's epoch
  __syncthreads();
  if (tid == 0) {
    const uint32_t ticket = atomicAdd(t.flags + 17, 1u);
    if (ticket == gridDim.x - 1) {
      t.flags[17] = 0u;
      *reinterpret_cast<volatile uint32_t*>(t.flags + 16) = e;
    }
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

// Order-preserving map of a float onto unsigned integers, and back.
__device__ __forceinline__ uint32_t float_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// The k-th largest value of row[0 .. n) (1 <= k <= n), by the whole block: radix select on the
// ordered keys, eight bits a round, each round one pass over the row and one 256-bin histogram.
__device__ float block_kth_largest(const float* __restrict__ row, int64_t n, int k) {
  __shared__ unsigned hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_k;
  uint32_t prefix = 0u, mask = 0u;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0u;
    __syncthreads();
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
      const uint32_t key = float_key(__ldcg(row + i));
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int cum = 0, b = 255;
      for (; b > 0; --b) {
        if (cum + (int)hist[b] >= k) break;
        cum += (int)hist[b];
      }
      s_prefix = prefix | ((uint32_t)b << shift);
      s_k = k - cum;
    }
    __syncthreads();
    prefix = s_prefix;
    k = s_k;
    mask |= 255u << shift;
    __syncthreads();
  }
  return key_float(prefix);
}

// history (optional): row `*step_counter` of a [history_rows][rows] log also receives the ids,
// so a captured step needs no per-step pointer.
__global__ void argmax_kernel(const float* __restrict__ logits, int32_t* __restrict__ tokens,
                              int32_t* __restrict__ history, const int32_t* __restrict__ step_counter,
                              int64_t history_rows, int64_t vocab, const SamplingParams* __restrict__ sampling,
                              const int32_t* __restrict__ positions, const int32_t* __restrict__ only_ending,
                              int prompt_step) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  pdl_wait();
  pdl_trigger();
  const int64_t row = blockIdx.x;
  if (only_ending && only_ending[row] - 1 != prompt_step) return;  // this sequence's prompt does not end here
  const float* lr = logits + row * vocab;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  const bool sample = sampling && positions && __ldcg(&sampling->enabled) != 0;
  const float inv_t = sample ? __ldcg(&sampling->inv_temperature) : 1.f;
  const uint64_t seed = sample ? __ldcg(&sampling->seed) : 0ull;
  const uint64_t first = sample ? (uint64_t)__ldcg(positions + row) * (uint64_t)vocab : 0ull;
  const int top_k = sample ? __ldcg(&sampling->top_k) : 0;
  // candidates: everything, or the logits that reach the row's k-th largest (ties at it included)
  const float least = (top_k > 0 && (int64_t)top_k < vocab) ? block_kth_largest(lr, vocab, top_k) : -INFINITY;
  for (int64_t i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = __ldcg(lr + i);
    if (v < least) continue;
    if (sample) v = __fadd_rn(__fmul_rn(v, inv_t), synth::gumbel_f32(seed, (uint64_t)row, first + (uint64_t)i));
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
  int dev = 0;
  cudaGetDevice(&dev);
  const int64_t cap = (int64_t)sm_count(dev) * 8;
  int grid = (int)(want < cap ? want : cap);
  swiglu_f32_kernel<<<grid, 256, 0, st>>>(gate, up, y, count);
  count_launch(LK_ELEMWISE);
  return check_launch("swiglu_f32_kernel");
}

logos_status_t launch_embed(const int32_t* tokens, const int8_t* q, const float* s, float* h, int64_t rows,
                            int64_t hidden, int tiled, cudaStream_t st) {
  if (rows == 0) return LOGOS_OK;
  LOGOS_CUDA_TRY(launch_kernel(embed_kernel, dim3((unsigned)rows), dim3(256), 0, st, tokens, q, s, h, hidden, tiled));
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
  if ((hidden & 3) == 0 && hidden <= 8192) {
    LOGOS_CUDA_TRY(launch_kernel(residual_rmsnorm_kernel<true>, dim3((unsigned)rows), dim3(512), 0, st, h, delta, parts,
                                 part_stride, g, xn, hidden, eps));
  } else {
    size_t smem = sizeof(float) * (size_t)hidden;
    if (smem > 48 * 1024)
      LOGOS_CUDA_TRY(cudaFuncSetAttribute(residual_rmsnorm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LOGOS_CUDA_TRY(launch_kernel(residual_rmsnorm_kernel<false>, dim3((unsigned)rows), dim3(512), smem, st, h, delta, parts,
                                 part_stride, g, xn, hidden, eps));
  }
  count_launch(LK_ELEMWISE);
  return check_launch("residual_rmsnorm_kernel");
}

logos_status_t launch_tp_residual_rmsnorm(float* h, const TpFusedArgs& t, int parts, int64_t part_stride, const float* g,
                                          int64_t rows, int64_t hidden, float eps, int device, cudaStream_t st) {
  if (rows == 0) return LOGOS_OK;
  if (t.degree < 2 || t.degree > 8 || rows % t.degree || hidden % (4 * TP_CLUSTER) || parts < 1)
    return fail(LOGOS_ERROR, "tp_residual_rmsnorm: unsupported shape (rows %lld, hidden %lld, degree %d, parts %d)",
                (long long)rows, (long long)hidden, t.degree, parts);
  // every CTA must be resident at once: CTAs that wait for a peer's push must not keep the
  // CTAs that peers wait for off the SMs
  if (rows * TP_CLUSTER > 2 * (int64_t)sm_count(device))
    return fail(LOGOS_ERROR, "tp_residual_rmsnorm: %lld rows are more than the grid can hold resident", (long long)rows);
  int* status = kernel_status_ptr(device);
  if (!status) return fail(LOGOS_ERROR, "tp_residual_rmsnorm: no kernel status word");
  const int64_t per = (hidden >> 2) / TP_CLUSTER;
  const int64_t rows_own = rows / t.degree;
  int threads = (int)(((per + 31) / 32) * 32);
  if (threads > 512) threads = 512;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * TP_CLUSTER));
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
                             const SamplingParams* sampling_or_null, const int32_t* positions_or_null,
                             const int32_t* only_ending_or_null, int prompt_step, cudaStream_t st) {
  if (rows == 0) return LOGOS_OK;
  LOGOS_CUDA_TRY(launch_kernel(argmax_kernel, dim3((unsigned)rows), dim3(1024), 0, st, logits, tokens, history_or_null,
                               step_counter_or_null, history_rows, vocab, sampling_or_null, positions_or_null,
                               only_ending_or_null, prompt_step));
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
