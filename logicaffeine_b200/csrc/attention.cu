// GQA decode attention over an fp16 KV cache, with the rotary embedding and
// the KV-cache append fused in.
//
// HBM-bound: every step streams the whole K and V history once (512 bytes per
// position per KV head at D=128), so the kernel is built around that stream:
//   * the work is the sequence of 64-position K/V tiles of all (sequence, KV head)
//     pairs, in order; the grid is persistent (two CTAs per SM) and CTA c takes the
//     c-th equal share of that sequence, whatever pairs it crosses: every CTA streams
//     the same number of tiles, and a pair is cut only where a share ends;
//   * a producer thread moves the tiles into a 3-stage shared-memory ring with TMA
//     tile loads (128-byte swizzle, no multicast) signalled on mbarriers; the ring
//     keeps running across pairs, so the loads of the next pair are in flight while
//     the consumers finish and write out the previous one; four consumer warps each
//     own 16 positions of every tile;
//   * all query heads that share the KV head (up to 16) form the M side of
//     m16n8k16 tensor-core MMAs, so a K/V tile is read from shared memory once
//     for the whole group; scores, softmax and the running output stay in f32
//     registers; the probabilities enter the second MMA as an fp16 high part
//     plus an fp16 residual so the product keeps f32-class accuracy;
//   * the CTA whose share holds the position being appended rotates the new key
//     (f32 multiply and add rounded separately, fp16 store), writes the new
//     K/V row to the cache and patches it into its own shared-memory tile;
//   * a pair that lies inside one share is normalised and written by that CTA; the
//     parts of a pair that was cut are merged by a second small kernel in a fixed order.
#include "ops.cuh"
#include "ptx.cuh"

#include <math.h>

#include <mutex>

namespace logos {

namespace {

using namespace ptx;

constexpr int ATT_TILE = 64;
constexpr int ATT_STAGES = 3;
constexpr int ATT_CWARPS = 4;
constexpr int ATT_CTHREADS = ATT_CWARPS * 32;
constexpr int ATT_THREADS = (ATT_CWARPS + 1) * 32;
constexpr int ATT_BOX_BYTES = 64 * 128;  // 64 rows x 128 bytes
constexpr int ATT_MAX_BATCH = 2048;      // sequences whose tile counts a CTA keeps in shared memory

struct AttnParams {
  const __half* q_f16;
  const float*  q_f32;
  int64_t       q_ld;
  int           rotate_q;
  const __half* k_new_f16;
  const __half* v_new_f16;
  const float*  k_new_f32;
  const float*  v_new_f32;
  int64_t       kv_ld;
  int           f32_parts;        // split-K partial copies of the f32 inputs, summed while staging
  int64_t       f32_part_stride;
  const float*  q_bias;           // f32 inputs only: added after the partial copies (null = none)
  const float*  k_bias;
  const float*  v_bias;
  int           fused;
  __half*       k_cache;
  __half*       v_cache;
  const float*  rope;
  const int32_t* seq_len;
  // Parts of cut pairs.  Only the first and the last pair of a share can be cut, so a share writes
  // at most two: slot 0 for a part that begins at the share's first tile, slot 1 otherwise.
  float*        part_o;   // [shares][2][16][D]   unnormalised outputs
  float*        part_ml;  // [shares][2][16][2]   their (max, sum)
  // [shares][2] descriptors, rewritten by every launch: the slot that holds the FIRST part of a
  // cut pair names the pair and its shares {b, kvh, first share, last share}; every other slot
  // says -1.  The merge kernel runs one CTA per slot and query row and acts on the named ones.
  int4*         part_desc;
  int64_t*      tiles_total;   // [1] the launch's tile count, for the merge kernel's share arithmetic
  void*         o;        // [B][Hq][D]
  int           o_dtype;
  ActOut        o_act;
  int           b, h_q, h_kv, l_max;
  int           shares;   // the persistent grid's size: the tile sequence is cut into this many shares
  float         scale_log2;
  int*          status;
};

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ int attn_len_eff(const AttnParams& p, int len0) {
  int len_eff = p.fused ? len0 + 1 : len0;
  if (len_eff > p.l_max) len_eff = p.l_max;
  return len_eff < 0 ? 0 : len_eff;
}

// Share c of `shares` takes tiles [c * total / shares, (c + 1) * total / shares); the share that
// holds tile g is the largest c whose first tile is <= g.
__device__ __forceinline__ int64_t share_begin(int64_t c, int64_t total, int shares) { return c * total / shares; }
__device__ __forceinline__ int share_of_tile(int64_t g, int64_t total, int shares) {
  return (int)(((g + 1) * shares - 1) / total);
}

__device__ __forceinline__ void store_out(const AttnParams& p, int64_t oi, float v) {
  if (p.o_dtype == LOGOS_ACT_PLANES) act_store(p.o_act, oi, v);
  else if (p.o_dtype == LOGOS_F16) reinterpret_cast<__half*>(p.o)[oi] = __float2half_rn(v);
  else if (p.o_dtype == LOGOS_BF16) reinterpret_cast<__nv_bfloat16*>(p.o)[oi] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(p.o)[oi] = v;
}

template <int D>
__global__ void __launch_bounds__(ATT_THREADS)
gqa_decode_attn_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const AttnParams p) {
  constexpr int NBOX = D / 64;
  constexpr int STAGE_BYTES = 2 * NBOX * ATT_BOX_BYTES;
  constexpr int QS_STRIDE = D + 8;  // halfs; +16 bytes keeps ldmatrix rows on distinct banks
  constexpr int KSTEPS = D / 16;
  static_assert(STAGE_BYTES >= ATT_CWARPS * 16 * D * 4, "a ring stage doubles as the scratch that combines the warps");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;                                            // ATT_STAGES * STAGE_BYTES
  __half* qs = reinterpret_cast<__half*>(stages + ATT_STAGES * STAGE_BYTES);  // [16][QS_STRIDE]
  __half* new_k = qs + 16 * QS_STRIDE;                               // [D]
  __half* new_v = new_k + D;                                         // [D]
  float* mml = reinterpret_cast<float*>(new_v + D);                  // [warp][16][2]
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(mml + ATT_CWARPS * 16 * 2);
  uint64_t* bar_empty = bar_full + ATT_STAGES;
  int32_t* s_tiles = reinterpret_cast<int32_t*>(bar_empty + ATT_STAGES);  // [B] tiles of a sequence
  int32_t* s_pref = s_tiles + p.b;                                         // [B + 1] tiles before it

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int G = p.h_q / p.h_kv;

  // The lengths, the query and the new K/V rows come from kernels of the same step: wait for
  // them (the launch may have let this kernel start early), and read them past L1.
  pdl_wait();
  pdl_trigger();
  // a kernel that gave up earlier left a code behind: do not start new work on top of it
  // (one thread reads, everyone takes the same decision)
  __shared__ int prior_status;
  if (tid == 0) {
    prior_status = *reinterpret_cast<volatile int*>(p.status);
    for (int i = 0; i < ATT_STAGES; ++i) {
      mbar_init(&bar_full[i], 1);
      mbar_init(&bar_empty[i], ATT_CWARPS);
    }
    fence_barrier_init();
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  for (int b = tid; b < p.b; b += ATT_THREADS)
    s_tiles[b] = (attn_len_eff(p, __ldcg(p.seq_len + b)) + ATT_TILE - 1) / ATT_TILE;
  if (tid < 2) p.part_desc[blockIdx.x * 2 + tid] = make_int4(-1, -1, -1, -1);
  __syncthreads();
  if (prior_status != 0) return;
  // a sequence without any position to attend to has no tile, hence no CTA: its output rows are zero
  for (int b = blockIdx.x; b < p.b; b += gridDim.x)
    if (s_tiles[b] == 0)
      for (int e = tid; e < p.h_q * D; e += ATT_THREADS) store_out(p, (int64_t)b * p.h_q * D + e, 0.f);
  if (warp == 0) {  // exclusive prefix over the sequences: lane l sums a contiguous run, then a warp scan
    const int per = (p.b + 31) / 32;
    int run = 0;
    for (int i = 0; i < per; ++i) {
      const int b = lane * per + i;
      if (b < p.b) run += s_tiles[b];
    }
    int incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int acc = incl - run;
    for (int i = 0; i < per; ++i) {
      const int b = lane * per + i;
      if (b < p.b) {
        s_pref[b] = acc;
        acc += s_tiles[b];
      }
    }
    if (lane == 31) s_pref[p.b] = incl;
  }
  __syncthreads();
  const int64_t total = (int64_t)p.h_kv * s_pref[p.b];
  if (blockIdx.x == 0 && tid == 0) *p.tiles_total = total;
  if (total == 0) return;
  const int64_t g_lo = share_begin(blockIdx.x, total, p.shares), g_hi = share_begin(blockIdx.x + 1, total, p.shares);
  if (g_lo >= g_hi) return;

  // Both roles walk the share the same way: tile g belongs to sequence b (the one with
  // h_kv * pref[b] <= g < h_kv * pref[b + 1]), KV head (g - h_kv * pref[b]) / tiles[b], tile
  // (g - h_kv * pref[b]) % tiles[b] of that pair.
  int b_cur = 0;
  {
    int lo = 0, hi = p.b;  // last b with h_kv * pref[b] <= g_lo
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if ((int64_t)p.h_kv * s_pref[mid] <= g_lo) lo = mid; else hi = mid;
    }
    b_cur = lo;
  }

  bool ok = true;

  if (warp == ATT_CWARPS) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      int t_ring = 0;
      int b = b_cur;
      for (int64_t g = g_lo; g < g_hi && ok;) {
        while ((int64_t)p.h_kv * s_pref[b + 1] <= g) ++b;
        const int tiles_b = s_tiles[b];
        const int64_t within = g - (int64_t)p.h_kv * s_pref[b];
        const int kvh = (int)(within / tiles_b), t0 = (int)(within - (int64_t)kvh * tiles_b);
        const int t1 = (int)min((int64_t)tiles_b, t0 + (g_hi - g));
        const int64_t row_base = ((int64_t)b * p.h_kv + kvh) * p.l_max;
        for (int t = t0; t < t1 && ok; ++t, ++t_ring) {
          const int st = t_ring % ATT_STAGES;
          const uint32_t ph = (uint32_t)(t_ring / ATT_STAGES) & 1u;
          ok = mbar_wait(&bar_empty[st], ph ^ 1u);
          if (!ok) break;
          uint8_t* sb = stages + st * STAGE_BYTES;
          mbar_arrive_expect_tx(&bar_full[st], STAGE_BYTES);
          const int y = (int)(row_base + (int64_t)t * ATT_TILE);
#pragma unroll
          for (int j = 0; j < NBOX; ++j) {
            tma_load_2d(sb + j * ATT_BOX_BYTES, &map_k, &bar_full[st], j * 64, y);
            tma_load_2d(sb + (NBOX + j) * ATT_BOX_BYTES, &map_v, &bar_full[st], j * 64, y);
          }
        }
        g += t1 - t0;
      }
      if (!ok) atomicExch(p.status, 101);
    }
  } else {
    // ---------------------------------------------------------------- consumers
    const int g4 = lane >> 2, t4 = lane & 3;
    const int ctid = tid;  // 0 .. ATT_CTHREADS - 1
    int t_ring = 0;
    int b = b_cur;
    for (int64_t g = g_lo; g < g_hi && ok;) {
      while ((int64_t)p.h_kv * s_pref[b + 1] <= g) ++b;
      const int tiles_b = s_tiles[b];
      const int64_t pair0 = (int64_t)p.h_kv * s_pref[b];
      const int64_t within = g - pair0;
      const int kvh = (int)(within / tiles_b), t0 = (int)(within - (int64_t)kvh * tiles_b);
      const int t1 = (int)min((int64_t)tiles_b, t0 + (g_hi - g));
      const int64_t pair_g0 = pair0 + (int64_t)kvh * tiles_b;  // first tile of the pair in the whole sequence
      const int share_first = share_of_tile(pair_g0, total, p.shares);
      const int share_last = share_of_tile(pair_g0 + tiles_b - 1, total, p.shares);
      const bool whole = share_first == share_last;   // the pair lies inside this share: write the result itself
      const int slot = g == g_lo ? 0 : 1;
      const int len0 = __ldcg(p.seq_len + b);
      const int len_eff = attn_len_eff(p, len0);
      const int64_t row_base = ((int64_t)b * p.h_kv + kvh) * p.l_max;
      const int pos_new = len0;  // where the appended row goes
      const bool append = p.fused && len0 < p.l_max;
      const bool owns_new = append && pos_new >= t0 * ATT_TILE && pos_new < t1 * ATT_TILE;

      // ---- stage the query heads (rotated when asked), zero the padding rows
      {
        const int half_d = D / 2;
        int pos_q = len0 < p.l_max ? len0 : p.l_max - 1;
        if (pos_q < 0) pos_q = 0;
        const float* tab = p.rope + (int64_t)pos_q * half_d * 2;
        for (int i = ctid; i < 16 * half_d; i += ATT_CTHREADS) {
          int g = i / half_d, e = i - g * half_d;
          float x1 = 0.f, x2 = 0.f;
          if (g < G) {
            int hq = kvh * G + g;
            if (p.q_f16) {
              const __half* qp = p.q_f16 + ((int64_t)b * p.h_q + hq) * D;
              x1 = __half2float(__ldcg(qp + e));
              x2 = __half2float(__ldcg(qp + e + half_d));
            } else {
              const float* qp = p.q_f32 + (int64_t)b * p.q_ld + (int64_t)hq * D;
              x1 = __ldcg(qp + e);
              x2 = __ldcg(qp + e + half_d);
              for (int sp = 1; sp < p.f32_parts; ++sp) {
                x1 = __fadd_rn(x1, __ldcg(qp + sp * p.f32_part_stride + e));
                x2 = __fadd_rn(x2, __ldcg(qp + sp * p.f32_part_stride + e + half_d));
              }
              if (p.q_bias) {
                x1 = __fadd_rn(x1, __ldg(p.q_bias + hq * D + e));
                x2 = __fadd_rn(x2, __ldg(p.q_bias + hq * D + e + half_d));
              }
            }
            if (p.rotate_q) {
              float c = tab[2 * e], s = tab[2 * e + 1];
              float r1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
              float r2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
              x1 = r1;
              x2 = r2;
            }
          }
          qs[g * QS_STRIDE + e] = __float2half_rn(x1);
          qs[g * QS_STRIDE + e + half_d] = __float2half_rn(x2);
        }
        // ---- the appended row: rotate k, round to fp16, write the cache, keep a copy
        if (owns_new) {
          const float* tabn = p.rope + (int64_t)pos_new * half_d * 2;
          for (int e = ctid; e < half_d; e += ATT_CTHREADS) {
            float k1, k2, v1, v2;
            if (p.k_new_f16) {
              const __half* kp = p.k_new_f16 + ((int64_t)b * p.h_kv + kvh) * D;
              const __half* vp = p.v_new_f16 + ((int64_t)b * p.h_kv + kvh) * D;
              k1 = __half2float(__ldcg(kp + e)); k2 = __half2float(__ldcg(kp + e + half_d));
              v1 = __half2float(__ldcg(vp + e)); v2 = __half2float(__ldcg(vp + e + half_d));
            } else {
              const float* kp = p.k_new_f32 + (int64_t)b * p.kv_ld + (int64_t)kvh * D;
              const float* vp = p.v_new_f32 + (int64_t)b * p.kv_ld + (int64_t)kvh * D;
              k1 = __ldcg(kp + e); k2 = __ldcg(kp + e + half_d);
              v1 = __ldcg(vp + e); v2 = __ldcg(vp + e + half_d);
              for (int sp = 1; sp < p.f32_parts; ++sp) {
                const int64_t o = sp * p.f32_part_stride;
                k1 = __fadd_rn(k1, __ldcg(kp + o + e)); k2 = __fadd_rn(k2, __ldcg(kp + o + e + half_d));
                v1 = __fadd_rn(v1, __ldcg(vp + o + e)); v2 = __fadd_rn(v2, __ldcg(vp + o + e + half_d));
              }
              if (p.k_bias) {
                k1 = __fadd_rn(k1, __ldg(p.k_bias + kvh * D + e)); k2 = __fadd_rn(k2, __ldg(p.k_bias + kvh * D + e + half_d));
              }
              if (p.v_bias) {
                v1 = __fadd_rn(v1, __ldg(p.v_bias + kvh * D + e)); v2 = __fadd_rn(v2, __ldg(p.v_bias + kvh * D + e + half_d));
              }
            }
            float c = tabn[2 * e], s = tabn[2 * e + 1];
            __half r1 = __float2half_rn(__fsub_rn(__fmul_rn(k1, c), __fmul_rn(k2, s)));
            __half r2 = __float2half_rn(__fadd_rn(__fmul_rn(k2, c), __fmul_rn(k1, s)));
            __half h1 = __float2half_rn(v1), h2 = __float2half_rn(v2);
            new_k[e] = r1; new_k[e + half_d] = r2;
            new_v[e] = h1; new_v[e + half_d] = h2;
            __half* kd = p.k_cache + (row_base + pos_new) * D;
            __half* vd = p.v_cache + (row_base + pos_new) * D;
            kd[e] = r1; kd[e + half_d] = r2;
            vd[e] = h1; vd[e + half_d] = h2;
          }
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(ATT_CTHREADS));

      uint32_t qa[KSTEPS][4];
      {
        int row = (lane & 7) + 8 * ((lane >> 3) & 1);
        int colh = 8 * (lane >> 4);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          uint32_t addr = smem_u32(qs + row * QS_STRIDE + ks * 16 + colh);
          ldmatrix_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], addr);
        }
      }
      float m_run[2] = {-INFINITY, -INFINITY};
      float l_run[2] = {0.f, 0.f};
      float o[D / 8][4];
#pragma unroll
      for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

      int st = 0;
      for (int t = t0; t < t1; ++t, ++t_ring) {
        st = t_ring % ATT_STAGES;
        uint32_t ph = (uint32_t)(t_ring / ATT_STAGES) & 1u;
        if (!mbar_wait(&bar_full[st], ph)) {
          ok = false;
          break;
        }
        uint8_t* kb = stages + st * STAGE_BYTES;
        uint8_t* vb = kb + NBOX * ATT_BOX_BYTES;
        const int tile_pos0 = t * ATT_TILE;
        const int my_pos0 = tile_pos0 + 16 * warp;

        // patch the appended row / clear rows past the end (only this warp reads its 16 rows)
        if (my_pos0 + 16 > len_eff || (owns_new && pos_new >= my_pos0 && pos_new < my_pos0 + 16)) {
          for (int r = 0; r < 16; ++r) {
            int pos = my_pos0 + r;
            uint32_t row = 16 * warp + r;
            if (owns_new && pos == pos_new) {
              for (int c = lane; c < 2 * (D / 8); c += 32) {
                bool is_v = c >= D / 8;
                int cc = is_v ? c - D / 8 : c;
                const uint4 val = *reinterpret_cast<const uint4*>((is_v ? new_v : new_k) + cc * 8);
                uint8_t* base = (is_v ? vb : kb) + (cc >> 3) * ATT_BOX_BYTES;
                *reinterpret_cast<uint4*>(base + swz128(row, cc & 7)) = val;
              }
            } else if (pos >= len_eff) {
              for (int c = lane; c < D / 8; c += 32) {
                uint8_t* base = vb + (c >> 3) * ATT_BOX_BYTES;
                *reinterpret_cast<uint4*>(base + swz128(row, c & 7)) = make_uint4(0, 0, 0, 0);
              }
            }
          }
          __syncwarp();
        }

        // ---- S = Q K^T for 16 positions
        float s[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        {
          uint32_t row = 16 * warp + (lane & 7) + 8 * (lane >> 4);
          int ch = (lane >> 3) & 1;
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ++ks) {
            int chunk = ks * 2 + ch;
            uint32_t addr = smem_u32(kb + (chunk >> 3) * ATT_BOX_BYTES + swz128(row, chunk & 7));
            uint32_t r0, r1, r2, r3;
            ldmatrix_x4(r0, r1, r2, r3, addr);
            mma_f16_16816(s[0], qa[ks], r0, r1);
            mma_f16_16816(s[1], qa[ks], r2, r3);
          }
        }
        // ---- mask, scale, online softmax
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            int pos = my_pos0 + nt * 8 + 2 * t4 + (j & 1);
            float v = (pos < len_eff) ? s[nt][j] * p.scale_log2 : -INFINITY;
            s[nt][j] = v;
            mx[j >> 1] = fmaxf(mx[j >> 1], v);
          }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          float m_new = fmaxf(m_run[r], mx[r]);
          m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
          corr[r] = exp2f(m_run[r] - m_use[r]);
          m_run[r] = m_new;
        }
        float pr[2][4];
        float psum[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float e = exp2f(s[nt][j] - m_use[j >> 1]);
            pr[nt][j] = e;
            psum[j >> 1] += e;
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
          const float (*q)[4] = pr;
          float h[8] = {q[0][0], q[0][1], q[0][2], q[0][3], q[1][0], q[1][1], q[1][2], q[1][3]};
          float lo[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float hi = __half2float(__float2half_rn(h[i]));
            lo[i] = h[i] - hi;
          }
          a_hi[0] = pack_half2(h[0], h[1]); a_hi[1] = pack_half2(h[2], h[3]);
          a_hi[2] = pack_half2(h[4], h[5]); a_hi[3] = pack_half2(h[6], h[7]);
          a_lo[0] = pack_half2(lo[0], lo[1]); a_lo[1] = pack_half2(lo[2], lo[3]);
          a_lo[2] = pack_half2(lo[4], lo[5]); a_lo[3] = pack_half2(lo[6], lo[7]);
        }
        // ---- O += P V
        {
          uint32_t row = 16 * warp + (lane & 7) + 8 * ((lane >> 3) & 1);
          int ch = lane >> 4;
#pragma unroll
          for (int dn = 0; dn < D / 16; ++dn) {
            int chunk = dn * 2 + ch;
            uint32_t addr = smem_u32(vb + (chunk >> 3) * ATT_BOX_BYTES + swz128(row, chunk & 7));
            uint32_t r0, r1, r2, r3;
            ldmatrix_x4_trans(r0, r1, r2, r3, addr);
            mma_f16_16816(o[2 * dn], a_hi, r0, r1);
            mma_f16_16816(o[2 * dn], a_lo, r0, r1);
            mma_f16_16816(o[2 * dn + 1], a_hi, r2, r3);
            mma_f16_16816(o[2 * dn + 1], a_lo, r2, r3);
          }
        }
        __syncwarp();
        // the last tile of this part keeps its ring stage: it is the scratch the warps are combined in
        if (t + 1 < t1 && lane == 0) mbar_arrive(&bar_empty[st]);
      }
      // ---- combine the four warps in the ring stage of the part's last tile (every warp has
      // read its rows of it once all four have passed the barrier), then hand the stage back.
      // The barrier also carries the outcome: a warp whose wait gave up takes the others with it.
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
      }
      {
        int all_ok;
        asm volatile(
            "{\n\t.reg .pred q, r;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred r, 1, %2, q;\n\tselp.u32 %0, 1, 0, r;\n\t}"
            : "=r"(all_ok)
            : "r"((uint32_t)ok), "n"(ATT_CTHREADS)
            : "memory");
        if (!all_ok) {
          if (!ok && lane == 0) atomicExch(p.status, 102);
          ok = false;
          break;
        }
      }
      float* mo = reinterpret_cast<float*>(stages + st * STAGE_BYTES);   // [warp][16][D]
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        int col = i * 8 + 2 * t4;
        float* r0p = mo + ((warp * 16 + g4) * D) + col;
        float* r1p = mo + ((warp * 16 + g4 + 8) * D) + col;
        r0p[0] = o[i][0]; r0p[1] = o[i][1];
        r1p[0] = o[i][2]; r1p[1] = o[i][3];
      }
      if (t4 == 0) {
        mml[(warp * 16 + g4) * 2 + 0] = m_run[0];
        mml[(warp * 16 + g4) * 2 + 1] = l_run[0];
        mml[(warp * 16 + g4 + 8) * 2 + 0] = m_run[1];
        mml[(warp * 16 + g4 + 8) * 2 + 1] = l_run[1];
      }
      asm volatile("bar.sync 1, %0;" ::"n"(ATT_CTHREADS));
      const int64_t pi = ((int64_t)blockIdx.x * 2 + slot) * 16;   // row 0 of this part's slot
      for (int e = ctid; e < G * D; e += ATT_CTHREADS) {
        int r = e / D, d = e - r * D;
        float mstar = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATT_CWARPS; ++w) mstar = fmaxf(mstar, mml[(w * 16 + r) * 2]);
        float muse = (mstar == -INFINITY) ? 0.f : mstar;
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_CWARPS; ++w) {
          float wgt = exp2f(mml[(w * 16 + r) * 2] - muse);
          acc = fmaf(mo[(w * 16 + r) * D + d], wgt, acc);
          L = fmaf(mml[(w * 16 + r) * 2 + 1], wgt, L);
        }
        if (whole) {
          store_out(p, ((int64_t)b * p.h_q + kvh * G + r) * D + d, __fdiv_rn(acc, L));
        } else {
          if (e == 0 && t0 == 0) p.part_desc[blockIdx.x * 2 + slot] = make_int4(b, kvh, share_first, share_last);
          p.part_o[(pi + r) * D + d] = acc;
          if (d == 0) {
            p.part_ml[(pi + r) * 2 + 0] = mstar;
            p.part_ml[(pi + r) * 2 + 1] = L;
          }
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(ATT_CTHREADS));   // everyone has read the scratch and qs
      if (lane == 0) mbar_arrive(&bar_empty[st]);
      g += t1 - t0;
    }
  }
}

// One CTA per part slot: where the slot holds the first part of a pair that the main kernel cut,
// fold the pair's parts in ascending order of their shares, for every query row of the group.
// (Most slots name no pair: the grid is small and those CTAs leave after one load.)
// The parts of a pair are listed once (a lane per share: which shares hold tiles), every row's
// maximum, weights and normaliser are computed once by a warp, and the threads then sum the
// parts' output rows with all their loads independent of one another: a fold is three rounds of
// global loads whatever the number of parts.  A pair cut into more than ATT_MERGE_PARTS parts
// (more shares than tiles) goes through a plain loop.
constexpr int ATT_MERGE_PARTS = 64;
template <int D>
__global__ void __launch_bounds__(256) attn_merge_kernel(const AttnParams p) {
  pdl_wait();
  pdl_trigger();
  const int4 desc = __ldcg(p.part_desc + blockIdx.x);
  if (desc.x < 0) return;
  const int G = p.h_q / p.h_kv;
  const int b = desc.x, kvh = desc.y, first = desc.z, last = desc.w;
  const int64_t total = __ldcg(p.tiles_total);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // the first part sits in this very slot; every later share holds its part in slot 0 (it begins
  // at the share's first tile); with more shares than tiles some shares in between hold no tile
  auto empty = [&](int c) { return share_begin(c, total, p.shares) == share_begin(c + 1, total, p.shares); };
  auto row0_of = [&](int c) -> int { return (c == first ? (int)blockIdx.x : c * 2) * 16; };
  const int span = last - first + 1;
  if (span > ATT_MERGE_PARTS) {
    for (int e = tid; e < G * D; e += blockDim.x) {
      const int r = e / D, d = e - r * D;
      float mstar = -INFINITY;
      for (int c = first; c <= last; ++c)
        if (!empty(c)) mstar = fmaxf(mstar, __ldcg(p.part_ml + (int64_t)(row0_of(c) + r) * 2));
      float muse = (mstar == -INFINITY) ? 0.f : mstar;
      float acc = 0.f, L = 0.f;
      for (int c = first; c <= last; ++c) {
        if (empty(c)) continue;
        const int64_t row = row0_of(c) + r;
        float wgt = exp2f(__ldcg(p.part_ml + row * 2) - muse);
        acc = fmaf(__ldcg(p.part_o + row * D + d), wgt, acc);
        L = fmaf(__ldcg(p.part_ml + row * 2 + 1), wgt, L);
      }
      store_out(p, ((int64_t)b * p.h_q + kvh * G + r) * D + d, __fdiv_rn(acc, L));
    }
    return;
  }
  __shared__ int s_row0[ATT_MERGE_PARTS];       // first of the 16 rows of each part that holds tiles
  __shared__ float s_w[ATT_MERGE_PARTS][16];    // weight of a part for a query row
  __shared__ float s_l[16];                     // the row's normaliser
  __shared__ int s_np;
  if (warp == 0) {  // list the parts in ascending order of their shares
    int np = 0;
    for (int c0 = first; c0 <= last; c0 += 32) {
      const int c = c0 + lane;
      const bool has = c <= last && !empty(c);
      const uint32_t m = __ballot_sync(0xffffffffu, has);
      if (has) s_row0[np + __popc(m & ((1u << lane) - 1u))] = row0_of(c);
      np += __popc(m);
    }
    if (lane == 0) s_np = np;
  }
  __syncthreads();
  const int np = s_np;
  // per query row (a warp each): maximum, weights in part order, normaliser summed in part order
  for (int r = warp; r < G; r += 8) {
    float mloc = -INFINITY;
    for (int pi = lane; pi < np; pi += 32) mloc = fmaxf(mloc, __ldcg(p.part_ml + (int64_t)(s_row0[pi] + r) * 2));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
    const float muse = (mloc == -INFINITY) ? 0.f : mloc;
    for (int pi = lane; pi < np; pi += 32)
      s_w[pi][r] = exp2f(__ldcg(p.part_ml + (int64_t)(s_row0[pi] + r) * 2) - muse);
    __syncwarp();
    if (lane == 0) {
      float L = 0.f;
      for (int pi = 0; pi < np; ++pi) L = fmaf(__ldcg(p.part_ml + (int64_t)(s_row0[pi] + r) * 2 + 1), s_w[pi][r], L);
      s_l[r] = L;
    }
  }
  __syncthreads();
  // a thread's elements (tid + 256 k) together, so that a part costs one round of loads for all of them
  constexpr int EPT = 16 * D / 256;
  float acc[EPT];
#pragma unroll
  for (int k = 0; k < EPT; ++k) acc[k] = 0.f;
  for (int pi = 0; pi < np; ++pi) {
    const float* po = p.part_o + (int64_t)s_row0[pi] * D;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      const int e = tid + k * 256;   // row e / D, column e % D: the part's rows are contiguous
      if (e < G * D) acc[k] = fmaf(__ldcg(po + e), s_w[pi][e / D], acc[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const int e = tid + k * 256;
    if (e < G * D) store_out(p, ((int64_t)b * p.h_q + kvh * G) * D + e, __fdiv_rn(acc[k], s_l[e / D]));
  }
}

__global__ void bump_seq_len_kernel(int32_t* seq_len, int b, int l_max) {
  pdl_wait();
  pdl_trigger();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < b && seq_len[i] < l_max) seq_len[i] += 1;
}

// Stand-alone append (no attention): one CTA per (sequence, KV head).
__global__ void kv_append_rope_kernel(__half* k_cache, __half* v_cache, const __half* k_new, const __half* v_new,
                                      const float* rope, const int32_t* seq_len, int h_kv, int d, int l_max) {
  const int kvh = blockIdx.x, b = blockIdx.y;
  const int pos = seq_len[b];
  if (pos < 0 || pos >= l_max) return;
  const int half_d = d / 2;
  const float* tab = rope + (int64_t)pos * half_d * 2;
  const __half* kp = k_new + ((int64_t)b * h_kv + kvh) * d;
  const __half* vp = v_new + ((int64_t)b * h_kv + kvh) * d;
  __half* kd = k_cache + (((int64_t)b * h_kv + kvh) * l_max + pos) * d;
  __half* vd = v_cache + (((int64_t)b * h_kv + kvh) * l_max + pos) * d;
  for (int e = threadIdx.x; e < half_d; e += blockDim.x) {
    float k1 = __half2float(kp[e]), k2 = __half2float(kp[e + half_d]);
    float c = tab[2 * e], s = tab[2 * e + 1];
    kd[e] = __float2half_rn(__fsub_rn(__fmul_rn(k1, c), __fmul_rn(k2, s)));
    kd[e + half_d] = __float2half_rn(__fadd_rn(__fmul_rn(k2, c), __fmul_rn(k1, s)));
    vd[e] = vp[e];
    vd[e + half_d] = vp[e + half_d];
  }
}

template <int D>
size_t attn_smem_bytes(int64_t batch) {
  return 1024 + (size_t)ATT_STAGES * 2 * (D / 64) * ATT_BOX_BYTES + (size_t)16 * (D + 8) * 2 + (size_t)2 * D * 2 +
         (size_t)ATT_CWARPS * 16 * 2 * 4 + 2 * ATT_STAGES * 8 + (size_t)(2 * batch + 1) * 4 + 64;
}

// The persistent grid: the tile sequence is cut into this many shares, one per CTA.
int attn_shares(const AttnArgs& a) {
  const int sms = sm_count(a.device);
  const int64_t tiles_max = (a.l_max + ATT_TILE - 1) / ATT_TILE;
  int64_t g = 2ll * sms;   // two CTAs of about 113 KB of shared memory fit an SM
  // With no more (sequence, KV head) pairs than CTAs, a whole number of shares per pair: where the
  // sequences are equally long every share boundary then falls on a pair boundary or cuts a pair
  // into equal pieces, and a CTA stages one pair's query instead of two (measured 4-8 % on the
  // operator at the shapes a rank of four or eight holds; neutral for ragged lengths).
  const int64_t pairs = a.b * a.h_kv;
  if (pairs > 0 && pairs <= g) g = g / pairs * pairs;
  const int64_t most = a.b * a.h_kv * tiles_max;
  if (g > most) g = most > 0 ? most : 1;
  return (int)g;
}

template <int D>
logos_status_t launch_attn_t(const AttnArgs& a, cudaStream_t st) {
  if (a.b > ATT_MAX_BATCH)
    return fail(LOGOS_OUT_OF_BOUNDS, "attention: batch %lld exceeds %d sequences per call", (long long)a.b, ATT_MAX_BATCH);
  const int64_t rows_total = a.b * a.h_kv * a.l_max;
  CUtensorMap mk, mv;
  LOGOS_TRY(make_tensor_map_2d(&mk, a.k_cache, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, D, rows_total, D * 2, 64, ATT_TILE,
                               CU_TENSOR_MAP_SWIZZLE_128B));
  LOGOS_TRY(make_tensor_map_2d(&mv, a.v_cache, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, D, rows_total, D * 2, 64, ATT_TILE,
                               CU_TENSOR_MAP_SWIZZLE_128B));
  const int shares = attn_shares(a);

  void* scratch = nullptr;
  const int64_t po_bytes = (int64_t)shares * 2 * 16 * D * (int64_t)sizeof(float);
  const int64_t pml_bytes = (int64_t)shares * 2 * 16 * 2 * (int64_t)sizeof(float);
  const int64_t desc_bytes = (int64_t)shares * 2 * (int64_t)sizeof(int4) + 16;
  if (a.ext_scratch) {
    if (po_bytes + pml_bytes + desc_bytes > a.ext_scratch_bytes)
      return fail(LOGOS_OUT_OF_BOUNDS,
                  "attention: this shape needs %lld bytes of split-KV scratch, the fixed scratch holds %lld",
                  (long long)(po_bytes + pml_bytes + desc_bytes), (long long)a.ext_scratch_bytes);
    scratch = a.ext_scratch;
  } else {
    LOGOS_TRY(scratch_get(a.device, 1, po_bytes + pml_bytes + desc_bytes, &scratch));
  }

  AttnParams p{};
  p.q_f16 = a.q_f16; p.q_f32 = a.q_f32; p.q_ld = a.q_ld; p.rotate_q = a.rotate_q;
  p.k_new_f16 = a.k_new_f16; p.v_new_f16 = a.v_new_f16; p.k_new_f32 = a.k_new_f32; p.v_new_f32 = a.v_new_f32;
  p.kv_ld = a.kv_ld;
  p.f32_parts = a.f32_parts > 1 ? a.f32_parts : 1;
  p.f32_part_stride = a.f32_part_stride;
  p.q_bias = a.q_bias; p.k_bias = a.k_bias; p.v_bias = a.v_bias;
  p.fused = (a.k_new_f16 || a.k_new_f32) ? 1 : 0;
  p.k_cache = a.k_cache; p.v_cache = a.v_cache; p.rope = a.rope; p.seq_len = a.seq_len;
  p.part_o = reinterpret_cast<float*>(scratch);
  p.part_ml = reinterpret_cast<float*>(static_cast<char*>(scratch) + po_bytes);
  p.part_desc = reinterpret_cast<int4*>(static_cast<char*>(scratch) + po_bytes + pml_bytes);
  p.tiles_total = reinterpret_cast<int64_t*>(static_cast<char*>(scratch) + po_bytes + pml_bytes + desc_bytes - 16);
  p.o = a.o; p.o_dtype = a.o_dtype; p.o_act = a.o_act;
  p.b = (int)a.b; p.h_q = (int)a.h_q; p.h_kv = (int)a.h_kv; p.l_max = (int)a.l_max;
  p.shares = shares;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.status = a.ext_status ? a.ext_status : kernel_status_ptr(a.device);
  if (!p.status) return fail(LOGOS_ERROR, "attention: no kernel status word");

  const size_t smem = attn_smem_bytes<D>(a.b);
  LOGOS_CUDA_TRY(cudaFuncSetAttribute(gqa_decode_attn_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  LOGOS_CUDA_TRY(launch_kernel(gqa_decode_attn_kernel<D>, dim3((unsigned)shares), dim3(ATT_THREADS), smem, st, mk, mv, p));
  count_launch(LK_ATTN);
  LOGOS_TRY(check_launch("gqa_decode_attn_kernel"));
  LOGOS_CUDA_TRY(launch_kernel(attn_merge_kernel<D>, dim3((unsigned)(2 * shares)), dim3(256), 0, st, p));
  count_launch(LK_ATTN_MERGE);
  LOGOS_TRY(check_launch("attn_merge_kernel"));
  if (a.bump_seq_len) {
    LOGOS_CUDA_TRY(launch_kernel(bump_seq_len_kernel, dim3((unsigned)((a.b + 127) / 128)), dim3(128), 0, st, a.seq_len,
                                 (int)a.b, (int)a.l_max));
    LOGOS_TRY(check_launch("bump_seq_len_kernel"));
  }
  return LOGOS_OK;
}

}  // namespace

void rope_table_host(float* out, int64_t l_max, int64_t d, double theta) {
  int64_t half = d / 2;
  for (int64_t pos = 0; pos < l_max; ++pos)
    for (int64_t i = 0; i < half; ++i) {
      double inv = pow(theta, -2.0 * (double)i / (double)d);
      double ang = (double)pos * inv;
      out[(pos * half + i) * 2 + 0] = (float)cos(ang);
      out[(pos * half + i) * 2 + 1] = (float)sin(ang);
    }
}

int64_t attn_scratch_bytes(const AttnArgs& a) {
  return (int64_t)attn_shares(a) * 2 * (16 * (a.d + 2) * (int64_t)sizeof(float) + (int64_t)sizeof(int4)) + 16;
}

logos_status_t launch_gqa_decode_attn(const AttnArgs& a, cudaStream_t st) {
  if (a.b == 0 || a.h_q == 0) return LOGOS_OK;
  if (a.h_kv <= 0 || a.h_q % a.h_kv) return fail(LOGOS_ERROR, "attention: h_q must be a multiple of h_kv");
  if (a.h_q / a.h_kv > 16) return fail(LOGOS_ERROR, "attention: at most 16 query heads per KV head");
  if (a.l_max <= 0) return fail(LOGOS_OUT_OF_BOUNDS, "attention: l_max must be positive");
  if (a.d == 128) return launch_attn_t<128>(a, st);
  if (a.d == 64) return launch_attn_t<64>(a, st);
  return fail(LOGOS_ERROR, "attention: head_dim %lld is not supported (64 or 128)", (long long)a.d);
}

logos_status_t launch_kv_append_rope(__half* k_cache, __half* v_cache, const __half* k_new, const __half* v_new,
                                     const float* rope, int32_t* seq_len, int64_t b, int64_t h_kv, int64_t d,
                                     int64_t l_max, int device, cudaStream_t st) {
  (void)device;
  if (b == 0 || h_kv == 0) return LOGOS_OK;
  dim3 grid((unsigned)h_kv, (unsigned)b);
  kv_append_rope_kernel<<<grid, 64, 0, st>>>(k_cache, v_cache, k_new, v_new, rope, seq_len, (int)h_kv, (int)d, (int)l_max);
  LOGOS_TRY(check_launch("kv_append_rope_kernel"));
  bump_seq_len_kernel<<<(unsigned)((b + 127) / 128), 128, 0, st>>>(seq_len, (int)b, (int)l_max);
  return check_launch("bump_seq_len_kernel");
}

// ---------------------------------------------------------------- fixed-scratch variant
// Scratch that lives in the library image instead of coming from cudaMalloc: every GPU
// that loads the library holds these 6 MiB (+ one status word) until the process exits.
// The kernel needs two part slots of 16 x (D + 2) floats per CTA of its persistent grid (two
// CTAs per SM): 4.7 MiB on a 148-SM B200 at D = 128; 6 MiB provide for 189 SMs.
constexpr int64_t kStaticScratchBytes = 6ll << 20;
static __device__ __align__(256) unsigned char g_static_attn_scratch[kStaticScratchBytes];
static __device__ __align__(256) int g_static_attn_status[8];

namespace {
constexpr int kMaxStaticDevices = 64;
struct StaticAddr {
  void* scratch = nullptr;
  int*  status = nullptr;
  bool  ready = false;
};
StaticAddr g_static_addr[kMaxStaticDevices];
std::mutex g_static_mu;

// In host code the array names above are host-side stand-ins, not device addresses: the
// address a kernel may use comes from cudaGetSymbolAddress, asked once per device with
// that device current.
logos_status_t static_scratch_for(int device, StaticAddr* out) {
  if (device < 0 || device >= kMaxStaticDevices)
    return fail(LOGOS_OUT_OF_BOUNDS, "fixed-scratch attention: device %d is beyond the %d this build tracks", device,
                kMaxStaticDevices);
  std::lock_guard<std::mutex> lk(g_static_mu);
  StaticAddr& sa = g_static_addr[device];
  if (!sa.ready) {
    void* p = nullptr;
    void* q = nullptr;
    LOGOS_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_attn_scratch));
    LOGOS_CUDA_TRY(cudaGetSymbolAddress(&q, g_static_attn_status));
    sa.scratch = p;
    sa.status = static_cast<int*>(q);
    sa.ready = true;
  }
  *out = sa;
  return LOGOS_OK;
}
}  // namespace

// The fixed-scratch entry point's own status word, for logos_kernel_status: copies the eight
// words out (and zeroes them when asked) if that entry point has run on `device`; *used tells
// whether it has.  A device-to-host copy of eight words: no allocation here either.
logos_status_t static_attn_status_read(int device, int words_out[8], bool clear, bool* used) {
  *used = false;
  if (device < 0 || device >= kMaxStaticDevices) return LOGOS_OK;
  StaticAddr sa;
  {
    std::lock_guard<std::mutex> lk(g_static_mu);
    sa = g_static_addr[device];
  }
  if (!sa.ready) return LOGOS_OK;
  LOGOS_CUDA_TRY(cudaSetDevice(device));
  LOGOS_CUDA_TRY(cudaMemcpy(words_out, sa.status, sizeof(int) * 8, cudaMemcpyDeviceToHost));
  if (clear && words_out[0] != 0) LOGOS_CUDA_TRY(cudaMemset(sa.status, 0, sizeof(int) * 8));
  *used = true;
  return LOGOS_OK;
}

}  // namespace logos

using namespace logos;

extern "C" {

logos_status_t logos_gqa_decode_attn_fixed_scratch(logos_handle_t q, logos_handle_t k_cache, logos_handle_t v_cache,
                                                   logos_handle_t seq_len, logos_handle_t o, int64_t b, int64_t h_q,
                                                   int64_t h_kv, int64_t d, int64_t l_max, float softmax_scale,
                                                   void* stream_or_null) {
  return guarded([&]() -> logos_status_t {
    if (b < 0 || h_q < 0 || h_kv <= 0 || d <= 0 || l_max <= 0)
      return fail(LOGOS_OUT_OF_BOUNDS, "logos_gqa_decode_attn_fixed_scratch: bad extents");
    AttnArgs a;
    __half *qp, *kc, *vc, *op;
    int32_t* sl;
    int32_t dev = 0;
    LOGOS_TRY(buf_ptr<__half>(q, b * h_q * d, "q", &qp, &dev));
    LOGOS_TRY(buf_ptr<__half>(k_cache, b * h_kv * l_max * d, "k_cache", &kc));
    LOGOS_TRY(buf_ptr<__half>(v_cache, b * h_kv * l_max * d, "v_cache", &vc));
    LOGOS_TRY(buf_ptr<int32_t>(seq_len, b, "seq_len", &sl));
    LOGOS_TRY(buf_ptr<__half>(o, b * h_q * d, "o", &op));
    LOGOS_CUDA_TRY(cudaSetDevice(dev));
    StaticAddr sa;
    LOGOS_TRY(static_scratch_for(dev, &sa));
    cudaStream_t st = as_stream(stream_or_null);
    // Nothing in the array has to be cleared.  The partials: every entry the merge reads is
    // written by this call first.  The status word starts at zero with the library image and is
    // sticky like the per-device one: a kernel that gave up leaves its code there, later calls
    // on this entry point do no work on top of it, and logos_kernel_status reports and clears it.
    a.q_f16 = qp; a.k_cache = kc; a.v_cache = vc; a.seq_len = sl; a.o = op; a.o_dtype = LOGOS_F16;
    a.b = b; a.h_q = h_q; a.h_kv = h_kv; a.d = d; a.l_max = l_max; a.scale = softmax_scale; a.device = dev;
    a.ext_scratch = sa.scratch;
    a.ext_scratch_bytes = kStaticScratchBytes;
    a.ext_status = sa.status;
    return launch_gqa_decode_attn(a, st);
  });
}

logos_status_t logos_rope_table(float* out_host, int64_t l_max, int64_t d, double theta) {
  return guarded([&]() -> logos_status_t {
    if (!out_host) return fail(LOGOS_NULL_POINTER, "logos_rope_table: out_host is null");
    if (l_max < 0 || d <= 0 || (d & 1)) return fail(LOGOS_OUT_OF_BOUNDS, "logos_rope_table: bad extents");
    rope_table_host(out_host, l_max, d, theta);
    return LOGOS_OK;
  });
}

logos_status_t logos_kv_append_rope(logos_handle_t k_cache, logos_handle_t v_cache, logos_handle_t k_new,
                                    logos_handle_t v_new, logos_handle_t rope_table, logos_handle_t seq_len,
                                    int64_t b, int64_t h_kv, int64_t d, int64_t l_max, void* stream_or_null) {
  return guarded([&]() -> logos_status_t {
    if (b < 0 || h_kv < 0 || d <= 0 || l_max <= 0 || (d & 1))
      return fail(LOGOS_OUT_OF_BOUNDS, "logos_kv_append_rope: bad extents");
    __half *kc, *vc, *kn, *vn;
    float* rt;
    int32_t* sl;
    int32_t dev = 0;
    LOGOS_TRY(buf_ptr<__half>(k_cache, b * h_kv * l_max * d, "k_cache", &kc, &dev));
    LOGOS_TRY(buf_ptr<__half>(v_cache, b * h_kv * l_max * d, "v_cache", &vc));
    LOGOS_TRY(buf_ptr<__half>(k_new, b * h_kv * d, "k_new", &kn));
    LOGOS_TRY(buf_ptr<__half>(v_new, b * h_kv * d, "v_new", &vn));
    LOGOS_TRY(buf_ptr<float>(rope_table, l_max * d, "rope_table", &rt));
    LOGOS_TRY(buf_ptr<int32_t>(seq_len, b, "seq_len", &sl));
    LOGOS_CUDA_TRY(cudaSetDevice(dev));
    return launch_kv_append_rope(kc, vc, kn, vn, rt, sl, b, h_kv, d, l_max, dev, as_stream(stream_or_null));
  });
}

static logos_status_t attn_abi(bool fused, logos_handle_t q, logos_handle_t k_new, logos_handle_t v_new,
                               logos_handle_t k_cache, logos_handle_t v_cache, logos_handle_t rope_table,
                               logos_handle_t seq_len, logos_handle_t o, int64_t b, int64_t h_q, int64_t h_kv,
                               int64_t d, int64_t l_max, float scale, void* stream) {
  if (b < 0 || h_q < 0 || h_kv <= 0 || d <= 0 || l_max <= 0)
    return fail(LOGOS_OUT_OF_BOUNDS, "gqa_decode_attn: bad extents");
  AttnArgs a;
  __half *qp, *kc, *vc, *op;
  int32_t* sl;
  int32_t dev = 0;
  LOGOS_TRY(buf_ptr<__half>(q, b * h_q * d, "q", &qp, &dev));
  LOGOS_TRY(buf_ptr<__half>(k_cache, b * h_kv * l_max * d, "k_cache", &kc));
  LOGOS_TRY(buf_ptr<__half>(v_cache, b * h_kv * l_max * d, "v_cache", &vc));
  LOGOS_TRY(buf_ptr<int32_t>(seq_len, b, "seq_len", &sl));
  LOGOS_TRY(buf_ptr<__half>(o, b * h_q * d, "o", &op));
  a.q_f16 = qp; a.k_cache = kc; a.v_cache = vc; a.seq_len = sl; a.o = op; a.o_dtype = LOGOS_F16;
  if (fused) {
    __half *kn, *vn;
    float* rt;
    LOGOS_TRY(buf_ptr<__half>(k_new, b * h_kv * d, "k_new", &kn));
    LOGOS_TRY(buf_ptr<__half>(v_new, b * h_kv * d, "v_new", &vn));
    LOGOS_TRY(buf_ptr<float>(rope_table, l_max * d, "rope_table", &rt));
    a.k_new_f16 = kn; a.v_new_f16 = vn; a.rope = rt; a.rotate_q = 1; a.bump_seq_len = 1;
  }
  a.b = b; a.h_q = h_q; a.h_kv = h_kv; a.d = d; a.l_max = l_max; a.scale = scale; a.device = dev;
  LOGOS_CUDA_TRY(cudaSetDevice(dev));
  return launch_gqa_decode_attn(a, as_stream(stream));
}

logos_status_t logos_gqa_decode_attn(logos_handle_t q, logos_handle_t k_cache, logos_handle_t v_cache,
                                     logos_handle_t seq_len, logos_handle_t o, int64_t b, int64_t h_q, int64_t h_kv,
                                     int64_t d, int64_t l_max, float softmax_scale, void* stream_or_null) {
  return guarded([&]() -> logos_status_t {
    return attn_abi(false, q, nullptr, nullptr, k_cache, v_cache, nullptr, seq_len, o, b, h_q, h_kv, d, l_max,
                    softmax_scale, stream_or_null);
  });
}

logos_status_t logos_gqa_decode_attn_fused(logos_handle_t q_raw, logos_handle_t k_new, logos_handle_t v_new,
                                           logos_handle_t k_cache, logos_handle_t v_cache, logos_handle_t rope_table,
                                           logos_handle_t seq_len, logos_handle_t o, int64_t b, int64_t h_q,
                                           int64_t h_kv, int64_t d, int64_t l_max, float softmax_scale,
                                           void* stream_or_null) {
  return guarded([&]() -> logos_status_t {
    return attn_abi(true, q_raw, k_new, v_new, k_cache, v_cache, rope_table, seq_len, o, b, h_q, h_kv, d, l_max,
                    softmax_scale, stream_or_null);
  });
}

}  // extern "C"
