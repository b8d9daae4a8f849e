// Q8 GEMM on the 5th-generation tensor cores (tcgen05) for small token counts.
//
//   acc[n, m] = sum_kb s[n,kb] * ( sum_{k in kb} q[n,k] * a[m,k] )
//
// The problem is laid out "weights on the M side": one CTA owns 128 weight
// rows (MMA M = 128, one TMEM lane per row) and MT tokens (MMA N), so the f32
// scale of a (row, K-block) pair is one scalar per thread when the block's
// partial sum is drained from tensor memory.
//
// Data flow per 128-column K stage (4 Q8 blocks):
//   TMA  int8 weights [128 rows][128 B], 128-byte swizzle  -> smem ring   (warp 0)
//   TMA  fp16 activation planes [MT][64] x 2 halves x limbs -> smem ring   (warp 1)
//   TMA  the stage's f32 scales [128 rows][4]               -> smem ring   (warp 0)
//   4 converter warps (one per TMEM lane quarter): smem int8 -> fp16 (exact: 0x6400|b trick)
//        -> tcgen05.st into a TMEM operand ring; the weights never go back to shared memory
//   2 MMA warps (one per half of a stage): per Q8 block two tcgen05.mma kind::f16 (K=16
//        each) per plane, A from TMEM, B = activations from smem, into a fresh TMEM
//        accumulator: first q*lo', then q*hi + D*2^-11 through the MMA's own
//        accumulator scaling, so hi + lo*2^-11 is recombined on the tensor core
//   8 drain warps: tcgen05.ld the block's partial sums (two blocks per wait),
//        acc += s * partial in f32 registers (scales from the shared-memory ring: a global load
//        under this kernel's own traffic takes several stage times), then the epilogue.
// A CTA is persistent: it takes work items (tile of 128 weight rows x K split) in turn,
// and the rings keep running across items, so the next item's weights stream in, are
// converted and multiplied while the drain warps finish the previous item's epilogue.
// The epilogue forms the output tile in shared memory in its final type and hands it to
// one TMA store (split-K partials, plain outputs, SwiGLU into activation planes); other
// output forms go through a plain loop of global stores.
// All hand-offs are mbarriers; every wait is bounded and reports through the
// device status word instead of spinning for ever.
//
// HBM roofline: 1.125 bytes per weight (int8 + f32/32); activations and
// outputs are small next to that at decode batch sizes.
#include "q8_gemm_tc.cuh"

#include "ptx.cuh"

#include <stdlib.h>

#include <mutex>
#include <unordered_map>

namespace logos {

namespace {

using namespace ptx;

constexpr int TC_ROWS = 128;     // weight rows per CTA (MMA M)
constexpr int TC_KSTAGE = 128;   // K per stage
constexpr int RAW_STAGES = 4;
constexpr int RAW_PREFETCH = 12;  // L2 prefetch distance of the weight stream, in stages
constexpr int ACT_STAGES = 3;
constexpr int TA_STAGES = 4;
constexpr int TA_LIMB_COLS = 64; // TMEM columns per converted stage and copy: 128 fp16 per row
constexpr int CONV_WARPS = 4;     // one per TMEM lane quarter
constexpr int CONV_WARP0 = 4, DRAIN_WARP0 = CONV_WARP0 + CONV_WARPS;
constexpr int TC_THREADS = (DRAIN_WARP0 + 8) * 32;  // 4 single-role warps, converter warps, 8 drain warps
constexpr int ACC_PAIRS = 2;     // TMEM accumulator ring: each entry holds two Q8 blocks
constexpr uint32_t TMEM_COLS = 512;
constexpr int RAW_BYTES = TC_ROWS * TC_KSTAGE;  // 16 KB
constexpr int SC_STAGES = 12;                   // scale ring: longer than the way from the producer to the drain
constexpr int SC_BYTES = TC_ROWS * 16;          // four f32 per row and stage

template <int MT, int LIMBS>
struct TcCfg {
  static constexpr int NB = MT * LIMBS;                 // activation rows staged per stage (planes stacked)
  static constexpr int TA_COLS = TA_LIMB_COLS;
  static constexpr int ACC_COL0 = TA_STAGES * TA_COLS;
  static constexpr int ACT_ATOM_BYTES = NB * 128;       // one 64-column half: NB rows x 128 B
  static constexpr int ACT_BYTES = 2 * ACT_ATOM_BYTES;
  static constexpr int EPI_BYTES = MT * TC_ROWS * 4;    // output tile staged for the store: [MT][128] f32 at most
  static constexpr size_t SMEM_NEED =
      1024 + (size_t)RAW_STAGES * RAW_BYTES + (size_t)ACT_STAGES * ACT_BYTES + EPI_BYTES + SC_STAGES * SC_BYTES + 1024;
  // the CTA allocates all of tensor memory, so ask for enough shared memory that only one CTA fits an SM
  static constexpr size_t SMEM = SMEM_NEED > 120 * 1024 ? SMEM_NEED : 120 * 1024;
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
  static_assert(ACC_COL0 + ACC_PAIRS * 2 * MT <= (int)TMEM_COLS, "TMEM budget");
  static_assert(MT % 16 == 0 && MT <= 64, "MMA N");
};

// How a finished tile leaves the CTA.
enum : int {
  STORE_GENERIC = 0,      // loop of global stores (any epilogue and output type)
  STORE_TMA_PARTIAL = 1,  // f32 split-K partials [splits][M][N], one 3-D TMA store
  STORE_TMA_PLAIN = 2,    // f32 / f16 / bf16 [M][ldc], no epilogue, one TMA store
  STORE_TMA_SWIGLU = 3,   // SwiGLU into fp16 activation planes [M][ldc], one TMA store per plane
};

struct TcParams {
  const float* s;
  int64_t n, k, m;
  void* c;
  int c_dtype;
  ActOut c_act;
  int64_t ldc;
  const void* aux;
  int epilogue;
  float* partials;
  int splits;
  int stages_total;
  int items;        // (row tile, K split) pairs
  int mtiles;       // token tiles of MT rows; a work unit is (item, token tile), token tile fastest
  int store_mode;
  int tiled;        // weights are tile-major: the map is [row tiles x K tiles x 128][128 B]
  int* status;
#ifdef LOGOS_TC_TRACE
  long long* trace;  // SM-clock timestamps of CTA (0,0,0), first item, [stage][16]
#endif
};

// Work item w = (row tile, K split): the splits of a tile are neighbours.
struct TcItem { int tile, split, st_begin, nst; };
__device__ __forceinline__ TcItem tc_item(const TcParams& p, int w) {
  TcItem it;
  it.tile = w / p.splits;
  it.split = w - it.tile * p.splits;
  it.st_begin = (int)(((int64_t)it.split * p.stages_total) / p.splits);
  it.nst = (int)(((int64_t)(it.split + 1) * p.stages_total) / p.splits) - it.st_begin;
  return it;
}

// First failure wins: code in word 0, where it happened in words 1..5.
__device__ __forceinline__ void tc_report(int* status, int code, int stage, int nst) {
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = blockIdx.x; status[2] = blockIdx.y; status[3] = stage; status[4] = nst; status[5] = threadIdx.x >> 5;
  }
}

// Timestamp slot `ev` of stage `i` (development builds with -DLOGOS_TC_TRACE only; CTA 0, its
// first item, one lane per role).  Compiled out otherwise.
#ifdef LOGOS_TC_TRACE
#define TC_TRACE(i, ev)                                                                          \
  do {                                                                                           \
    if (trace_on && (i) < 64) p.trace[(i) * 16 + (ev)] = clock64();                              \
  } while (0)
#define TC_TRACE_ITEM(w) trace_on = cta0 && (w) == 0
#else
#define TC_TRACE(i, ev) do { } while (0)
#define TC_TRACE_ITEM(w) do { } while (0)
#endif

__device__ __forceinline__ float silu_f(float g) { return __fdiv_rn(g, 1.0f + expf(-g)); }

__device__ __forceinline__ void store_c(const TcParams& p, int64_t i, float v) {
  if (p.c_dtype == LOGOS_ACT_PLANES) act_store(p.c_act, i, v);
  else if (p.c_dtype == LOGOS_F16) reinterpret_cast<__half*>(p.c)[i] = __float2half_rn(v);
  else if (p.c_dtype == LOGOS_BF16) reinterpret_cast<__nv_bfloat16*>(p.c)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(p.c)[i] = v;
}
__device__ __forceinline__ float load_aux(const TcParams& p, int64_t i) {
  if (p.c_dtype == LOGOS_F16) return __half2float(reinterpret_cast<const __half*>(p.aux)[i]);
  if (p.c_dtype == LOGOS_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.aux)[i]);
  return reinterpret_cast<const float*>(p.aux)[i];
}

// two int8 (bytes sel_lo / sel_hi of w ^ 0x80808080, i.e. of q + 128 as unsigned bytes) -> packed
// fp16 pair, exact
__device__ __forceinline__ uint32_t cvt_pair(uint32_t w_xor80, uint32_t selector) {
  uint32_t bits = __byte_perm(w_xor80, 0x64646464u, selector);   // 0x64bb = 1024 + (q + 128)
  __half2 h = *reinterpret_cast<__half2*>(&bits);
  const uint32_t bias_bits = 0x64806480u;                        // 1152 = 1024 + 128
  __half2 r = __hsub2(h, *reinterpret_cast<const __half2*>(&bias_bits));
  return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pack2(float v) { return pack2(__float_as_uint(v), __float_as_uint(v)); }
// two f32 FMAs in one instruction (sm_100): d = a * b + c on both halves, round to nearest
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier; both addresses and the
// size are multiples of 16
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <int N>
__device__ __forceinline__ void tc_ld_cols(uint32_t taddr, uint32_t (&r)[N]) {
  if constexpr (N == 32) tc_ld_32x32b_x32(taddr, r);
  else if constexpr (N == 16) tc_ld_32x32b_x16(taddr, r);
  else tc_ld_32x32b_x8(taddr, r);
}

// fp32 -> the value(s) an activation plane pair stores (same rounding as act_store)
__device__ __forceinline__ void act_split_planes(int mode, float x, __half* h, __half* l) {
  if (mode == LOGOS_BF16) x = __bfloat162float(__float2bfloat16_rn(x));
  x = act_clamp(x);
  *h = __float2half_rn(x);
  *l = __float2half_rn((x - __half2float(*h)) * 2048.f);
}

template <int MT, int LIMBS, bool TILED>
__global__ void __launch_bounds__(TC_THREADS, 1)
q8_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_ahi,
                  const __grid_constant__ CUtensorMap map_alo, const __grid_constant__ CUtensorMap map_o0,
                  const __grid_constant__ CUtensorMap map_o1, const __grid_constant__ CUtensorMap map_s,
                  const TcParams p) {
  using Cfg = TcCfg<MT, LIMBS>;
  constexpr int TA_COLS = Cfg::TA_COLS;
  constexpr int ACC_COL0 = Cfg::ACC_COL0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* raw = smem;
  uint8_t* act = raw + RAW_STAGES * RAW_BYTES;
  uint8_t* epi = act + ACT_STAGES * Cfg::ACT_BYTES;  // 1024-aligned: all sizes before it are multiples of 1024
  uint8_t* scl = epi + Cfg::EPI_BYTES;               // scale ring
  uint64_t* bars = reinterpret_cast<uint64_t*>(scl + SC_STAGES * SC_BYTES);
  uint64_t* raw_full = bars;                    // [RAW_STAGES]
  uint64_t* raw_empty = raw_full + RAW_STAGES;  // [RAW_STAGES]
  uint64_t* act_full = raw_empty + RAW_STAGES;  // [ACT_STAGES]
  uint64_t* act_empty = act_full + ACT_STAGES;  // [ACT_STAGES]
  uint64_t* ta_full = act_empty + ACT_STAGES;   // [TA_STAGES]
  uint64_t* ta_empty = ta_full + TA_STAGES;     // [TA_STAGES]
  uint64_t* acc_full = ta_empty + TA_STAGES;    // [ACC_PAIRS]
  uint64_t* acc_empty = acc_full + ACC_PAIRS;   // [ACC_PAIRS]
  uint64_t* sc_full = acc_empty + ACC_PAIRS;    // [SC_STAGES]
  uint64_t* sc_empty = sc_full + SC_STAGES;     // [SC_STAGES]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sc_empty + SC_STAGES);

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  // Work units u = item * mtiles + token tile: CTAs that run side by side hold consecutive units,
  // i.e. the same weight tile for neighbouring token tiles, so with many tokens (prefill) a
  // weight tile crosses HBM once and is served to the other token tiles by L2.
  const int units = p.items * p.mtiles;
#ifdef LOGOS_TC_TRACE
  const bool cta0 = p.trace && blockIdx.x == 0;
  bool trace_on = cta0;
#endif

  if (tid == 0) TC_TRACE(63, 0);  // kernel entry
  // a kernel that gave up earlier left a code behind: do not start new work on top of it
  // (one thread reads, everyone takes the same decision)
  __shared__ int prior_status;
  if (tid == 0) prior_status = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (prior_status != 0) {
    pdl_wait();  // "this kernel completed" must keep implying "its predecessor did"
    return;
  }

  if (tid == 0) {
    for (int i = 0; i < RAW_STAGES; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], CONV_WARPS); }
    for (int i = 0; i < ACT_STAGES; ++i) { mbar_init(&act_full[i], 1); mbar_init(&act_empty[i], 2); }
    for (int i = 0; i < TA_STAGES; ++i) { mbar_init(&ta_full[i], CONV_WARPS); mbar_init(&ta_empty[i], 2); }
    for (int i = 0; i < ACC_PAIRS; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 8); }
    for (int i = 0; i < SC_STAGES; ++i) { mbar_init(&sc_full[i], 1); mbar_init(&sc_empty[i], 8); }
    fence_barrier_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_ahi);
    if (LIMBS == 2) prefetch_tensormap(&map_alo);
    if (p.store_mode != STORE_GENERIC) prefetch_tensormap(&map_o0);
    if (p.store_mode == STORE_TMA_SWIGLU) prefetch_tensormap(&map_o1);
    if (!TILED) prefetch_tensormap(&map_s);
  }
  if (warp == 3) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Dependent launch: this CTA holds its SM's shared and tensor memory by now, so a successor's
  // CTAs may be scheduled wherever room is left.  Weights and scales are read without waiting
  // for the previous kernel (nothing in a decode step writes them); the activation producer
  // and the drain warps (the only ones that touch what other kernels write) wait first.
  pdl_trigger();

  bool ok = true;
  if (tid == 0) TC_TRACE(63, 1);  // set-up done

  // Every role walks the same sequence of (item, stage) pairs; `gs` counts stages across items
  // and alone decides ring slots and barrier phases, so the rings never drain between items.
  if (warp == 0) {
    // ------------------------------------------------------------ weight producer
    if (lane == 0) {
      const uint64_t pol = policy_evict_first();
      int gs = 0;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int w = u / p.mtiles;
        const TcItem it = tc_item(p, w);
        const int n0 = it.tile * TC_ROWS, nst = it.nst, st_begin = it.st_begin;
        TC_TRACE_ITEM(w);
        // The smem ring alone (RAW_STAGES x 16 KB per SM) does not cover HBM latency under load:
        // L2 prefetches run RAW_PREFETCH stages ahead of the TMA loads.  They start only after
        // the item's first loads are on their way, so that nothing queues in front of those.
        for (int i = 0; i < nst; ++i, ++gs) {
          {
            // the stage's scales, four per row: tile-major they are 2 contiguous KB, row-major a
            // [128 rows][4] box of the [N][K/32] matrix (rows past N read as zero)
            const int ss = gs % SC_STAGES;
            if (!mbar_wait(&sc_empty[ss], ((uint32_t)(gs / SC_STAGES) & 1u) ^ 1u)) { ok = false; tc_report(p.status, 2011, i, nst); break; }
            mbar_arrive_expect_tx(&sc_full[ss], SC_BYTES);
            if (TILED)
              bulk_load(scl + ss * SC_BYTES, p.s + ((int64_t)it.tile * p.stages_total + st_begin + i) * TC_ROWS * 4, SC_BYTES, &sc_full[ss]);
            else
              tma_load_2d(scl + ss * SC_BYTES, &map_s, &sc_full[ss], (st_begin + i) * 4, n0);
          }
          const int st = gs % RAW_STAGES;
          const uint32_t ph = (uint32_t)(gs / RAW_STAGES) & 1u;
          if (!mbar_wait(&raw_empty[st], ph ^ 1u)) { ok = false; tc_report(p.status, 2010, i, nst); break; }
          TC_TRACE(i, 0);
          mbar_arrive_expect_tx(&raw_full[st], RAW_BYTES);
          // row-major weights: tile (n0, stage) of a [N][K] map; tile-major: 128 rows of 128 bytes at
          // row ((tile * stages + stage) * 128) of a [tiles * stages * 128][128 B] map
          const int tbase = it.tile * p.stages_total + st_begin;
          if (TILED) tma_load_2d_hint(raw + st * RAW_BYTES, &map_q, &raw_full[st], 0, (tbase + i) * TC_ROWS, pol);
          else tma_load_2d_hint(raw + st * RAW_BYTES, &map_q, &raw_full[st], (st_begin + i) * TC_KSTAGE, n0, pol);
          if (i + 1 >= RAW_STAGES) {
            // after the first fill: stages RAW_STAGES .. RAW_PREFETCH in one go, then one per stage
            const int first = (i + 1 == RAW_STAGES) ? RAW_STAGES : i + RAW_PREFETCH;
            for (int j = first; j <= i + RAW_PREFETCH && j < nst; ++j) {
              if (TILED) tma_prefetch_l2_2d(&map_q, 0, (tbase + j) * TC_ROWS);
              else tma_prefetch_l2_2d(&map_q, (st_begin + j) * TC_KSTAGE, n0);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ activation producer
    if (lane == 0) {
      pdl_wait();  // the activations are the previous kernel's output
      const uint64_t pol = policy_evict_last();
      int gs = 0;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int w = u / p.mtiles;
        const int m0 = (u - w * p.mtiles) * MT;
        const TcItem it = tc_item(p, w);
        const int nst = it.nst, st_begin = it.st_begin;
        TC_TRACE_ITEM(w);
        for (int i = 0; i < nst; ++i, ++gs) {
          const int st = gs % ACT_STAGES;
          const uint32_t ph = (uint32_t)(gs / ACT_STAGES) & 1u;
          if (!mbar_wait(&act_empty[st], ph ^ 1u)) { ok = false; tc_report(p.status, 2020, i, nst); break; }
          TC_TRACE(i, 1);
          mbar_arrive_expect_tx(&act_full[st], Cfg::ACT_BYTES);
          uint8_t* sb = act + st * Cfg::ACT_BYTES;
          const int x = (st_begin + i) * TC_KSTAGE;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            tma_load_2d_hint(sb + h * Cfg::ACT_ATOM_BYTES, &map_ahi, &act_full[st], x + h * 64, (int)m0, pol);
            if (LIMBS == 2)
              tma_load_2d_hint(sb + h * Cfg::ACT_ATOM_BYTES + MT * 128, &map_alo, &act_full[st], x + h * 64, (int)m0, pol);
          }
        }
      }
    }
  } else if (warp == 2 || warp == 3) {
    // ------------------------------------------------------------ MMA issuers
    // Two warps, one per half of a stage: warp 2 issues the first pair of Q8 blocks of every
    // stage, warp 3 the second.  What bounds the kernel is the round trip of an accumulator entry
    // (MMAs execute -> completion seen by the drain -> tcgen05.ld -> entry released -> next
    // stage's MMAs), so the two pairs' round trips run side by side; and every barrier is
    // waited on, phase after phase, by the same warp, which the odd/even phase test needs.
    // A warp runs its loop with all lanes (addresses and descriptors stay warp-uniform) and one
    // elected lane issues the tcgen05 instructions.  A pair owns accumulator ring entry `pr`.
    constexpr int NSPLIT = 1;   // an M=128, K=16 MMA costs the same at N=32 and N=64: one MMA per block and plane
    constexpr int MN = MT;      // tokens per MMA (MMA N, a multiple of 16)
    constexpr uint32_t idesc = make_idesc_f16(0, 0, TC_ROWS, MN);
    static_assert(ACC_PAIRS == 2, "one accumulator ring entry per MMA warp");
    const int pr = warp - 2;
    int gs = 0;
    int as = 0;           // slot and phase of the activation ring, counted
    uint32_t aph = 0;
    for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
      const int w = u / p.mtiles;
      const int nst = tc_item(p, w).nst;
      TC_TRACE_ITEM(w);
      for (int i = 0; i < nst && ok; ++i, ++gs) {
        const int ts = gs % TA_STAGES;
        const uint32_t tph = (uint32_t)(gs / TA_STAGES) & 1u;
        if (!mbar_wait(&ta_full[ts], tph)) { ok = false; if (lane == 0) tc_report(p.status, 2031, i, nst); break; }
        if (lane == 0 && pr == 0) TC_TRACE(i, 2);
        if (!mbar_wait(&act_full[as], aph)) { ok = false; if (lane == 0) tc_report(p.status, 2032, i, nst); break; }
        const uint32_t act_base = smem_u32(act + as * Cfg::ACT_BYTES);
        const uint32_t sph = (uint32_t)gs & 1u;
        if (pr == 1 && lane == 0) TC_TRACE(i, 11);
        if (!mbar_wait(&acc_empty[pr], sph ^ 1u)) { ok = false; if (lane == 0) tc_report(p.status, 2033, i, nst); break; }
        if (pr == 1 && lane == 0) TC_TRACE(i, 12);
        tc_fence_after();
        if (elect_one()) {
          // Per block: d = q * lo' first, then d = q * hi + d * 2^-11 (the residual plane is folded
          // in by the accumulator scaling of the MMA itself, from one copy of the weights).
          // The two blocks' chains are issued interleaved (measured neutral: the pipe runs
          // dependent and independent accumulations at the same rate).
#pragma unroll
          for (int u = 0; u < 2 * LIMBS; ++u) {
#pragma unroll
            for (int bb = 0; bb < 2; ++bb) {
#pragma unroll
              for (int hh = 0; hh < NSPLIT; ++hh) {
                const int blk = 2 * pr + bb;
                const uint32_t d = tmem_base + ACC_COL0 + blk * MT + hh * MN;
                const int l = (LIMBS == 2) ? 1 - (u >> 1) : 0, j = u & 1;
                const int kk = blk * 2 + j;  // K=16 step inside the stage
                const uint32_t a = tmem_base + ts * TA_COLS + kk * 8;
                const uint64_t bdesc = make_desc_sw128(act_base + (kk >> 2) * Cfg::ACT_ATOM_BYTES + l * MT * 128 +
                                                       hh * MN * 128 + (kk & 3) * 32);
                if (LIMBS == 2 && u == 2) tc_mma_f16_ts_scaled_d<11>(d, a, bdesc, idesc);
                else tc_mma_f16_ts(d, a, bdesc, idesc, (uint32_t)(u != 0));
              }
            }
          }
          if (pr == 1) TC_TRACE(i, 13);
          tc_commit(&acc_full[pr]);
          // the stage's operands are free once both warps' MMAs have completed
          tc_commit(&ta_empty[ts]);
          tc_commit(&act_empty[as]);
        }
        __syncwarp();
        if (lane == 0 && pr == 0) TC_TRACE(i, 4);
        if (++as == ACT_STAGES) { as = 0; aph ^= 1u; }
      }
    }

  } else if (warp >= CONV_WARP0 && warp < DRAIN_WARP0) {
    // ------------------------------------------------------------ converters: int8 smem -> fp16 TMEM
    // One or two warps per lane quarter; each converts its share of the stage's eight 16-byte
    // chunks per row.
    const int qd = warp & 3;
    const int chalf = (warp - CONV_WARP0) >> 2;
    const uint32_t row = qd * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(qd * 32) << 16);
    int gs = 0;
    for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
      const int w = u / p.mtiles;
      const int nst = tc_item(p, w).nst;
      TC_TRACE_ITEM(w);
      for (int i = 0; i < nst; ++i, ++gs) {
        const int rs = gs % RAW_STAGES, ts = gs % TA_STAGES;
        const uint32_t rph = (uint32_t)(gs / RAW_STAGES) & 1u, tph = (uint32_t)(gs / TA_STAGES) & 1u;
        if (!mbar_wait(&raw_full[rs], rph)) { ok = false; if (lane == 0) tc_report(p.status, 2041, i, nst); break; }
        if (warp == CONV_WARP0 && lane == 0) TC_TRACE(i, 5);
        if (!mbar_wait(&ta_empty[ts], tph ^ 1u)) { ok = false; if (lane == 0) tc_report(p.status, 2042, i, nst); break; }
        if (warp == CONV_WARP0 && lane == 0) TC_TRACE(i, 6);
        tc_fence_after();
        const uint8_t* rb = raw + rs * RAW_BYTES;
#pragma unroll
        for (int cc = 0; cc < 32 / CONV_WARPS; ++cc) {
          const int c = chalf * (32 / CONV_WARPS) + cc;
          const uint4 wv = *reinterpret_cast<const uint4*>(rb + swz128(row, c));
          uint32_t r[8];
          const uint32_t ws[4] = {wv.x, wv.y, wv.z, wv.w};
          if (TILED) {  // tile-major weights are stored as q + 128 already (compile-time branch: two
                        // copies of this loop in one kernel cost 10 % of its speed)
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
              r[2 * wi] = cvt_pair(ws[wi], 0x4140);
              r[2 * wi + 1] = cvt_pair(ws[wi], 0x4342);
            }
          } else {
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
              const uint32_t u = ws[wi] ^ 0x80808080u;
              r[2 * wi] = cvt_pair(u, 0x4140);
              r[2 * wi + 1] = cvt_pair(u, 0x4342);
            }
          }
          tc_st_32x32b_x8(t_lane + ts * TA_COLS + c * 8, r);
        }
        tc_wait_st();
        if (warp == CONV_WARP0 && lane == 0) TC_TRACE(i, 7);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&raw_empty[rs]);
          mbar_arrive(&ta_full[ts]);
        }
      }
    }

  } else if (warp >= DRAIN_WARP0) {
    // ------------------------------------------------------------ drain + epilogue
    // Two warps per lane quarter, each owning half of the token columns.  Blocks are taken two
    // at a time so one tcgen05.wait::ld covers both loads: the TMEM read latency, not the
    // arithmetic, is what bounds this role.
    const int qd = warp & 3;
    const int half = (warp - DRAIN_WARP0) >> 2;
    constexpr int HC = MT / 2;  // token columns per drain warp
    const int nl = qd * 32 + lane;  // row of the tile this thread drains
    const uint32_t t_lane = tmem_base + ((uint32_t)(qd * 32) << 16) + ACC_COL0 + half * HC;
    const int et = tid - DRAIN_WARP0 * 32;  // 0..255 among the drain warps
    pdl_wait();  // before any write to global memory (nothing to drain before the activations are in anyway)
    bool stored = false;  // thread et == 0: a TMA store of this CTA may still be reading the staging tile
    int gs = 0;
    int ss = 0;           // slot and phase of the scale ring (SC_STAGES is not a power of two: counted, not divided)
    uint32_t sph = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const int w = u / p.mtiles;
      const int64_t m0 = (int64_t)(u - w * p.mtiles) * MT;
      const int64_t rows_here = (p.m - m0 < MT) ? (p.m - m0) : MT;
      const TcItem it = tc_item(p, w);
      const int nst = it.nst;
      const int64_t n0 = (int64_t)it.tile * TC_ROWS;
      TC_TRACE_ITEM(w);
      uint64_t acc2[HC / 2];  // packed f32 pairs: the drain arithmetic uses two-wide f32 FMAs
#pragma unroll
      for (int j = 0; j < HC / 2; ++j) acc2[j] = 0ull;
      for (int i = 0; i < nst && ok; ++i, ++gs) {
        // the stage's four scales of this row, from the ring
        if (!mbar_wait(&sc_full[ss], sph)) { ok = false; if (lane == 0) tc_report(p.status, 2051, i, nst); break; }
        const float4 sc4 = *reinterpret_cast<const float4*>(scl + ss * SC_BYTES + nl * 16);
        __syncwarp();
        if (lane == 0) mbar_arrive(&sc_empty[ss]);
        if (++ss == SC_STAGES) { ss = 0; sph ^= 1u; }
        const float scs[4] = {sc4.x, sc4.y, sc4.z, sc4.w};
        const uint32_t fph = (uint32_t)gs & 1u;
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {
          if (!mbar_wait(&acc_full[pr], fph)) { ok = false; if (lane == 0) tc_report(p.status, 2050, i, nst); break; }
          if (warp == DRAIN_WARP0 && lane == 0 && pr == 0) TC_TRACE(i, 8);
          tc_fence_after();
          uint32_t b0[HC], b1[HC];
          tc_ld_cols<HC>(t_lane + (pr * 2) * MT, b0);
          tc_ld_cols<HC>(t_lane + (pr * 2 + 1) * MT, b1);
          tc_wait_ld();
          if (warp == DRAIN_WARP0 && lane == 0) TC_TRACE(i, pr == 0 ? 9 : 14);
#ifdef LOGOS_TC_TRACE
          if (trace_on && lane == 0 && i < 64)  // the last of the eight drain warps to get here
            atomicMax(reinterpret_cast<unsigned long long*>(&p.trace[i * 16 + (pr == 0 ? 3 : 15)]), (unsigned long long)clock64());
#endif
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[pr]);
          const uint64_t sc0 = pack2(scs[2 * pr]), sc1 = pack2(scs[2 * pr + 1]);
#pragma unroll
          for (int j = 0; j < HC / 2; ++j) {
            acc2[j] = ffma2(sc0, pack2(b0[2 * j], b0[2 * j + 1]), acc2[j]);
            acc2[j] = ffma2(sc1, pack2(b1[2 * j], b1[2 * j + 1]), acc2[j]);
          }
          if (warp == DRAIN_WARP0 && lane == 0 && pr == 0) TC_TRACE(i, 10);
        }
      }
      if (warp == DRAIN_WARP0 && lane == 0) TC_TRACE(63, 2);  // main loop of the first item done

      // ---- epilogue.  The tile goes to shared memory in the form it will have in global
      // memory, and one thread hands it to the TMA; the next item's stages are already being
      // loaded, converted and multiplied meanwhile.  The staging tile is free again once the
      // previous store has read it.
      if (et == 0 && stored) bulk_wait_read_all();
      int all_ok;
      asm volatile(
          "{\n\t.reg .pred q, r;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred r, 2, 256, q;\n\tselp.u32 %0, 1, 0, r;\n\t}"
          : "=r"(all_ok)
          : "r"((uint32_t)ok)
          : "memory");  // the eight drain warps agree on leaving
      if (!all_ok) { ok = false; break; }
      // element x (0..HC-1) of this thread's row: token half * HC + x
#define TC_ACC(x) __uint_as_float((uint32_t)(((x) & 1) ? (acc2[(x) >> 1] >> 32) : acc2[(x) >> 1]))
      const int mode = p.store_mode;
      if (mode == STORE_TMA_SWIGLU) {
        // rows (2j, 2j+1) of the tile are (gate_j, up_j): neighbouring lanes.  The even lane
        // takes the first half of this warp's tokens, the odd lane the second half.
        __half* eh = reinterpret_cast<__half*>(epi);   // [MT][64] hi plane
        __half* el = eh + MT * (TC_ROWS / 2);           // [MT][64] lo plane
        const int par = lane & 1, jj = nl >> 1;
#pragma unroll
        for (int t = 0; t < HC / 2; ++t) {
          const float a = TC_ACC(t), b = TC_ACC(t + HC / 2);
          const float recv = __shfl_xor_sync(0xffffffffu, par ? a : b, 1);
          const float mine = par ? b : a;
          const float g = par ? recv : mine, u = par ? mine : recv;
          const int mm = half * HC + (par ? t + HC / 2 : t);
          __half h, l;
          act_split_planes(p.c_act.mode, __fmul_rn(silu_f(g), u), &h, &l);
          eh[mm * (TC_ROWS / 2) + jj] = h;
          el[mm * (TC_ROWS / 2) + jj] = l;
        }
      } else if (mode == STORE_TMA_PLAIN && p.c_dtype != LOGOS_F32) {
        __half* e16 = reinterpret_cast<__half*>(epi);  // [MT][128] f16 or bf16
#pragma unroll
        for (int x = 0; x < HC; ++x) {
          const float v = TC_ACC(x);
          if (p.c_dtype == LOGOS_F16) e16[(half * HC + x) * TC_ROWS + nl] = __float2half_rn(v);
          else reinterpret_cast<__nv_bfloat16*>(e16)[(half * HC + x) * TC_ROWS + nl] = __float2bfloat16_rn(v);
        }
      } else {
        float* e32 = reinterpret_cast<float*>(epi);    // [MT][128] f32
#pragma unroll
        for (int x = 0; x < HC; ++x) e32[(half * HC + x) * TC_ROWS + nl] = TC_ACC(x);
      }
#undef TC_ACC
      if (mode != STORE_GENERIC) fence_proxy_async_smem();
      if (warp == DRAIN_WARP0 && lane == 0) TC_TRACE(63, 5);  // staged
      asm volatile("bar.sync 2, 256;" ::: "memory");
      if (mode != STORE_GENERIC) {
        if (et == 0) {
          if (mode == STORE_TMA_PARTIAL) {
            tma_store_3d(&map_o0, epi, (int)n0, (int)m0, it.split);
          } else if (mode == STORE_TMA_PLAIN) {
            tma_store_2d(&map_o0, epi, (int)n0, (int)m0);
          } else {
            tma_store_2d(&map_o0, epi, (int)(n0 >> 1), (int)m0);
            if (p.c_act.mode == LOGOS_F32) tma_store_2d(&map_o1, epi + MT * TC_ROWS, (int)(n0 >> 1), (int)m0);
          }
          bulk_commit();
          stored = true;
        }
      } else {
        const float* stage_c = reinterpret_cast<const float*>(epi);
        if (p.splits <= 1 && p.epilogue == EPI_SWIGLU) {
          // rows (2j, 2j+1) of the tile are (gate_j, up_j): 64 outputs per token
          const int64_t out0 = n0 >> 1;
          const int64_t outs = ((p.n - n0 < TC_ROWS ? p.n - n0 : TC_ROWS)) >> 1;
#pragma unroll 4
          for (int e = et; e < MT * (TC_ROWS / 2); e += 256) {
            const int mm = e / (TC_ROWS / 2), jj = e % (TC_ROWS / 2);
            if (mm < rows_here && jj < outs) {
              const float g = stage_c[mm * TC_ROWS + 2 * jj], u = stage_c[mm * TC_ROWS + 2 * jj + 1];
              store_c(p, (m0 + mm) * p.ldc + out0 + jj, __fmul_rn(silu_f(g), u));
            }
          }
        } else {
          const int64_t cols_here = (p.n - n0 < TC_ROWS) ? (p.n - n0) : TC_ROWS;
#pragma unroll 4
          for (int e = et; e < MT * TC_ROWS; e += 256) {
            const int mm = e / TC_ROWS, nn = e % TC_ROWS;
            if (mm < rows_here && nn < cols_here) {
              float v = stage_c[mm * TC_ROWS + nn];
              if (p.splits > 1) {
                p.partials[((int64_t)it.split * p.m + m0 + mm) * p.n + n0 + nn] = v;
              } else {
                const int64_t ci = (m0 + mm) * p.ldc + n0 + nn;
                if (p.epilogue == EPI_RESIDUAL) v = __fadd_rn(v, load_aux(p, ci));
                store_c(p, ci, v);
              }
            }
          }
        }
      }
      if (warp == DRAIN_WARP0 && lane == 0) TC_TRACE(63, 3);  // first item's stores issued
    }
    // global writes of the TMA stores are complete before the CTA ends
    if (et == 0 && stored) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
#ifdef LOGOS_TC_TRACE
  if (tid == 0) { trace_on = cta0; TC_TRACE(63, 4); }
#endif
  if (warp == 3) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------- host side
#ifdef LOGOS_TC_TRACE
long long* g_trace = nullptr;  // set through logos_gemm_trace_buffer; null = tracing off
#endif

struct MapKey {
  const void* base;
  uint64_t d0, d1, d2, pitch1, pitch2;
  uint32_t box0, box1, elem, swizzle;
  bool operator==(const MapKey& o) const {
    return base == o.base && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && pitch1 == o.pitch1 && pitch2 == o.pitch2 &&
           box0 == o.box0 && box1 == o.box1 && elem == o.elem && swizzle == o.swizzle;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = reinterpret_cast<uint64_t>(k.base);
    for (uint64_t v : {k.d0, k.d1, k.d2, k.pitch1, k.pitch2, ((uint64_t)k.box0 << 32) | k.box1,
                       ((uint64_t)k.elem << 32) | k.swizzle})
      h = h * 0x9E3779B97F4A7C15ull + v;
    return (size_t)h;
  }
};

}  // namespace

// Tensor maps are pure functions of (address, shape, box): encode once, reuse.  d2 == 0 asks
// for a 2-D map [d1][d0] with the given swizzle; otherwise a 3-D map [d2][d1][d0], box depth 1,
// no swizzle.
logos_status_t cached_map(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint32_t elem, uint64_t d0,
                          uint64_t d1, uint64_t pitch1, uint32_t box0, uint32_t box1, CUtensorMapSwizzle swizzle,
                          uint64_t d2, uint64_t pitch2) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{base, d0, d1, d2, pitch1, pitch2, box0, box1, elem, (uint32_t)swizzle};
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return LOGOS_OK;
    }
  }
  if (d2 == 0) LOGOS_TRY(make_tensor_map_2d(out, base, dt, elem, d0, d1, pitch1, box0, box1, swizzle));
  else LOGOS_TRY(make_tensor_map_3d(out, base, dt, elem, d0, d1, d2, pitch1, pitch2, box0, box1, 1));
  std::lock_guard<std::mutex> lk(mu);
  if (cache.size() > 8192) cache.clear();
  cache[key] = *out;
  return LOGOS_OK;
}

namespace {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int MT, int LIMBS>
logos_status_t launch_t(const GemmArgs& g, cudaStream_t st) {
  using Cfg = TcCfg<MT, LIMBS>;
  CUtensorMap mq, mhi, mlo, mo0, mo1, ms;
  if (g.q_tiled) {
    const uint64_t rows = (uint64_t)((g.n + TC_ROWS - 1) / TC_ROWS) * (uint64_t)(g.k / TC_KSTAGE) * TC_ROWS;
    LOGOS_TRY(cached_map(&mq, g.q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, TC_KSTAGE, rows, TC_KSTAGE, TC_KSTAGE, TC_ROWS));
  } else {
    LOGOS_TRY(cached_map(&mq, g.q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)g.k, (uint64_t)g.n, (uint64_t)g.k, TC_KSTAGE, TC_ROWS));
  }
  LOGOS_TRY(cached_map(&mhi, g.a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)g.k, (uint64_t)g.m, (uint64_t)g.lda * 2, 64, MT));
  if (LIMBS == 2)
    LOGOS_TRY(cached_map(&mlo, g.a_lo, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)g.k, (uint64_t)g.m, (uint64_t)g.lda * 2, 64, MT));
  else
    mlo = mhi;
  ms = mhi;
  if (!g.q_tiled)
    LOGOS_TRY(cached_map(&ms, g.s, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)(g.k / 32), (uint64_t)g.n, (uint64_t)(g.k / 32) * 4, 4,
                         TC_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE));
  TcParams p{};
  p.s = g.s; p.n = g.n; p.k = g.k; p.m = g.m;
  p.c = g.c; p.c_dtype = g.c_dtype; p.c_act = g.c_act; p.ldc = g.ldc; p.aux = g.aux; p.epilogue = g.epilogue;
  p.partials = g.partials;
  p.tiled = g.q_tiled;
  p.splits = g.splits > 1 ? g.splits : 1;
  p.stages_total = (int)(g.k / TC_KSTAGE);
  const int64_t tiles = (g.n + TC_ROWS - 1) / TC_ROWS;
  if (tiles * p.splits > INT32_MAX) return fail(LOGOS_OUT_OF_BOUNDS, "q8_gemm: too many work items");
  p.items = (int)(tiles * p.splits);
  p.status = kernel_status_ptr(g.device);
#ifdef LOGOS_TC_TRACE
  p.trace = g_trace;
  if (g_trace) {
    // optional filter: trace only launches whose grid has this many row tiles
    static const char* f = getenv("LOGOS_B200_TRACE_TILES");
    if (f && atoi(f) != (int)tiles) p.trace = nullptr;
  }
#endif
  if (!p.status) return fail(LOGOS_ERROR, "q8_gemm: no kernel status word");
  if (p.splits > p.stages_total) return fail(LOGOS_ERROR, "q8_gemm: more K splits than 128-column stages");

  // How the tile is stored: through the TMA where the destination allows a tensor map
  // (16-byte aligned base and row pitch), else by a loop of plain stores.
  static const bool no_tma_store = getenv("LOGOS_B200_GEMM_PLAIN_STORES") != nullptr;
  p.store_mode = STORE_GENERIC;
  mo0 = mq;
  mo1 = mq;
  if (no_tma_store) {
  } else if (p.splits > 1) {
    if (aligned16(g.partials) && g.n % 4 == 0) {
      LOGOS_TRY(cached_map(&mo0, g.partials, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)g.n, (uint64_t)g.m,
                           (uint64_t)g.n * 4, TC_ROWS, MT, CU_TENSOR_MAP_SWIZZLE_NONE, (uint64_t)p.splits,
                           (uint64_t)g.m * g.n * 4));
      p.store_mode = STORE_TMA_PARTIAL;
    }
  } else if (g.epilogue == EPI_NONE &&
             (g.c_dtype == LOGOS_F32 || g.c_dtype == LOGOS_F16 || g.c_dtype == LOGOS_BF16)) {
    const uint32_t eb = g.c_dtype == LOGOS_F32 ? 4 : 2;
    const CUtensorMapDataType dt = g.c_dtype == LOGOS_F32   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : g.c_dtype == LOGOS_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                            : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    if (aligned16(g.c) && (g.ldc * eb) % 16 == 0) {
      LOGOS_TRY(cached_map(&mo0, g.c, dt, eb, (uint64_t)g.n, (uint64_t)g.m, (uint64_t)g.ldc * eb, TC_ROWS, MT,
                           CU_TENSOR_MAP_SWIZZLE_NONE));
      p.store_mode = STORE_TMA_PLAIN;
    }
  } else if (g.epilogue == EPI_SWIGLU && g.c_dtype == LOGOS_ACT_PLANES && g.n % 2 == 0) {
    const bool two = g.c_act.mode == LOGOS_F32;
    if (aligned16(g.c_act.hi) && (!two || aligned16(g.c_act.lo)) && (g.ldc * 2) % 16 == 0) {
      LOGOS_TRY(cached_map(&mo0, g.c_act.hi, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)(g.n / 2), (uint64_t)g.m,
                           (uint64_t)g.ldc * 2, TC_ROWS / 2, MT, CU_TENSOR_MAP_SWIZZLE_NONE));
      if (two)
        LOGOS_TRY(cached_map(&mo1, g.c_act.lo, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)(g.n / 2),
                             (uint64_t)g.m, (uint64_t)g.ldc * 2, TC_ROWS / 2, MT, CU_TENSOR_MAP_SWIZZLE_NONE));
      p.store_mode = STORE_TMA_SWIGLU;
    }
  }

  auto kernel = g.q_tiled ? q8_gemm_tc_kernel<MT, LIMBS, true> : q8_gemm_tc_kernel<MT, LIMBS, false>;
  LOGOS_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM));
  // persistent CTAs: one per SM at most, each takes units blockIdx.x, blockIdx.x + gridDim.x, ...
  const int sms = sm_count(g.device);
  const int64_t mtiles = (g.m + MT - 1) / MT;
  if ((int64_t)p.items * mtiles > INT32_MAX) return fail(LOGOS_OUT_OF_BOUNDS, "q8_gemm: too many work units");
  p.mtiles = (int)mtiles;
  const int64_t units = (int64_t)p.items * mtiles;
  dim3 grid((unsigned)(units < sms ? units : sms), 1u, 1u);
  LOGOS_CUDA_TRY(launch_kernel(kernel, grid, dim3(TC_THREADS), Cfg::SMEM, st, mq, mhi, mlo, mo0, mo1, ms, p));
  count_launch(LK_GEMM_TC);
  return check_launch("q8_gemm_tc_kernel");
}

}  // namespace

#ifdef LOGOS_TC_TRACE
void gemm_set_trace(long long* buf) { g_trace = buf; }
#endif

bool gemm_tc_applicable(const GemmArgs& g) {
  if (g.a_dtype != LOGOS_F16) return false;
  if (g.k < TC_KSTAGE || g.k % TC_KSTAGE) return false;
  if (g.m < 1 || g.n < 1) return false;
  if (g.lda % 8) return false;
  if ((reinterpret_cast<uintptr_t>(g.a) & 15u) || (reinterpret_cast<uintptr_t>(g.a_lo) & 15u) ||
      (reinterpret_cast<uintptr_t>(g.q) & 15u) || (reinterpret_cast<uintptr_t>(g.s) & 15u))
    return false;
  return true;
}

logos_status_t launch_q8_gemm_tc(const GemmArgs& g, cudaStream_t st) {
  const bool two = g.a_lo != nullptr;
  if (g.m <= 16) return two ? launch_t<16, 2>(g, st) : launch_t<16, 1>(g, st);
  if (g.m <= 32) return two ? launch_t<32, 2>(g, st) : launch_t<32, 1>(g, st);
  return two ? launch_t<64, 2>(g, st) : launch_t<64, 1>(g, st);
}

}  // namespace logos
