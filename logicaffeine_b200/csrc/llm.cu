// Batched Qwen-architecture greedy decode on Q8 weights.
//
// One step, per layer (all sequences in lock step):
//   residual add + RMSNorm -> 16-bit x          (one kernel; also folds split-K partials)
//   Q8 GEMM  x -> [q | k | v]  (f32)
//   RoPE + KV append + GQA attention           (one kernel + merge) -> 16-bit
//   Q8 GEMM  o_proj  -> f32 partials           [all-reduce when tensor parallel]
//   residual add + RMSNorm -> 16-bit x
//   Q8 GEMM  gate/up with the SwiGLU epilogue -> 16-bit
//   Q8 GEMM  down_proj -> f32 partials         [all-reduce when tensor parallel]
// then final norm, lm_head GEMM (f32 logits), argmax.
//
// Memory: weights are int8 [N][K] + f32 [N][K/32]; the residual stream is f32;
// GEMM inputs are fp16 planes: a high and a residual plane that together keep
// f32-class precision (cfg.act_dtype = LOGOS_F32, the default), or one plane of
// values rounded to fp16 / bf16 when the configuration asks; the KV cache is fp16
// [B][Hkv][Lmax][D] per layer.  Tensor parallelism shards q/k/v/gate/up by
// output rows (heads, FFN columns) and o_proj/down_proj by input columns, so
// the only exchanges are the two sum all-reduces per layer.
#include "ops.cuh"
#include "q8_gemm_tc.cuh"
#include "tp.cuh"
#include "weights.cuh"

#include <errno.h>
#include <fcntl.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <algorithm>
#include <vector>

namespace logos {

namespace {

// int8 [n][k] + f32 [n][k/32].  q is allocated for ceil128(n) rows and is either row-major (as
// generated, loaded and saved) or tile-major (as the GEMM streams it, see launch_q8_retile);
// matrices whose K is not a multiple of 128 stay row-major (the SIMT kernel takes them).
struct Q8Mat {
  int8_t* q = nullptr;
  float*  s = nullptr;
  int64_t n = 0, k = 0;
  bool tiled = false;
};

struct Layer {
  Q8Mat wqkv, wo, wgu, wd;
  float* bqkv = nullptr;  // cfg.qkv_bias only: f32 [nqkv], the biases of this rank's q | k | v rows
  __half *kc = nullptr, *vc = nullptr;
};

// Buffers of the chunked prompt pass: one row per (sequence, position of the chunk).
struct PrefillWs {
  int64_t rows = 0;          // capacity
  float*  h = nullptr;       // [rows][H] residual stream
  float*  delta = nullptr;   // [rows][H] output of the last row-parallel GEMM, folded in by the next norm
  ActOut  xn;                // [rows][H]
  float*  qkv = nullptr;     // [rows][nqkv]
  __half* q16 = nullptr;     // [rows][nq] rotated queries
  ActOut  att;               // [rows][nq]
  ActOut  ffn;               // [rows][f_local]
  int32_t* tok = nullptr;    // [rows]
};

struct Model {
  logos_llm_config_t cfg;
  int device = 0;
  cudaStream_t stream = nullptr;
  TpGroup tp;
  int64_t nq = 0, nkv = 0, nqkv = 0, f_local = 0, hkv_local = 0, hq_local = 0;
  std::vector<Layer> layers;
  Q8Mat embed, head;
  float* gains = nullptr;    // RMSNorm gains [2 * layers + 1][H]: attn_norm and mlp_norm of every layer, final_norm; 1 at creation
  float* rope = nullptr;
  float* h = nullptr;        // [B][H] residual stream
  ActOut xn;                 // [B][H] fp16 plane(s)
  float* qkv = nullptr;      // [B][nqkv]
  ActOut att;                // [B][nq]
  ActOut ffn;                // [B][f_local]
  float* partials = nullptr; // [max_splits][B][H]
  float* dpart = nullptr;    // split-K partials of the GEMMs with a direct output (qkv, gate/up)
  int64_t dpart_floats = 0;
  void*  attn_scratch = nullptr;  // split-KV partials of the attention kernel: owned here, so the captured step
  int64_t attn_scratch_bytes = 0; // never points at the library's shared scratch
  // tensor parallelism with peer-addressable memory: partials, xn planes and flag words live in
  // one block per rank that every rank maps; the all-reduce is folded into residual + RMSNorm
  TpSymm symm;
  bool tp_fused = false;
  TpFusedArgs tpf;
  int    max_splits = 1;
  float* logits = nullptr;   // [B][V]
  int32_t* tokens = nullptr; // [B] current input / last output
  int32_t* seq_len = nullptr;
  SamplingParams* sampling = nullptr;  // device: temperature sampling state (zeroed = greedy)
  int32_t* history = nullptr; // [history_cap][B] token log of the current decode_steps call
  int64_t  history_cap = 0;
  int32_t* step_counter = nullptr;  // device: steps taken since the current decode_steps call began
  // one decode step captured as a CUDA graph (launch-bound at small per-step times)
  cudaGraphExec_t step_graph = nullptr;
  bool graph_failed = false;
  int64_t eager_sample_steps = 0;
  int32_t* prompt = nullptr;  // [T][B]
  int64_t  prompt_cap = 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  double last_ms = 0.0;
  int64_t launches_per_step = 0;
  int64_t launch_counter = 0;
  std::vector<void*> allocs;
  PrefillWs pf;
  // per-class device timing of one step (logos_llm_profile_step)
  bool profiling = false;
  std::vector<cudaEvent_t> prof_events;
  std::vector<int> prof_class;
  size_t prof_used = 0;
};

enum ProfClass : int { PROF_GEMM = 0, PROF_ATTN = 1, PROF_ELEMWISE = 2, PROF_COMM = 3, PROF_CLASSES = 4 };

// Brackets a group of launches with an event pair when a profiled step is running.
struct ProfScope {
  Model* m;
  bool on;
  ProfScope(Model* model, int cls) : m(model), on(model->profiling) {
    if (!on) return;
    if (m->prof_used + 2 > m->prof_events.size()) {
      for (int i = 0; i < 2; ++i) {
        cudaEvent_t e;
        cudaEventCreate(&e);
        m->prof_events.push_back(e);
      }
    }
    m->prof_class.push_back(cls);
    cudaEventRecord(m->prof_events[m->prof_used], m->stream);
  }
  ~ProfScope() {
    if (!on) return;
    cudaEventRecord(m->prof_events[m->prof_used + 1], m->stream);
    m->prof_used += 2;
  }
};

logos_status_t dmalloc(Model* m, void** p, int64_t bytes) {
  *p = nullptr;
  if (bytes <= 0) bytes = 16;
  cudaError_t e = cudaMalloc(p, (size_t)bytes);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc (model)");
  m->allocs.push_back(*p);
  return LOGOS_OK;
}

logos_status_t alloc_mat(Model* m, Q8Mat* w, int64_t n, int64_t k) {
  w->n = n;
  w->k = k;
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&w->q), ((n + 127) / 128 * 128) * k));
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&w->s), ((n + 127) / 128 * 128) * (k / 32) * (int64_t)sizeof(float)));
  return LOGOS_OK;
}

void destroy(Model* m) {
  cudaSetDevice(m->device);
  if (m->stream) cudaStreamSynchronize(m->stream);
  // The captured step holds NCCL nodes: it has to go before the communicator does, or the
  // communicator's destruction waits on it.
  if (m->step_graph) cudaGraphExecDestroy(m->step_graph);
  m->step_graph = nullptr;
  tp_symm_free(&m->symm);
  tp_destroy(&m->tp);
  for (void* p : m->allocs) cudaFree(p);
  for (cudaEvent_t e : m->prof_events) cudaEventDestroy(e);
  if (m->ev0) cudaEventDestroy(m->ev0);
  if (m->ev1) cudaEventDestroy(m->ev1);
  if (m->stream) cudaStreamDestroy(m->stream);
  delete m;
}

bool tiling_enabled() {
  const char* e = getenv("LOGOS_B200_TILED_WEIGHTS");
  return !(e && e[0] == '0');
}

// Every GEMM weight of the model into the tile-major layout (or back to row-major, which is what
// the generator, the weight-file loader and the writer address).  One pass per matrix through a
// scratch buffer of the largest matrix's size, allocated for the call.
logos_status_t set_layout(Model* m, bool tiled) {
  if (tiled && !tiling_enabled()) return LOGOS_OK;
  std::vector<Q8Mat*> mats;
  for (Layer& L : m->layers) {
    mats.push_back(&L.wqkv); mats.push_back(&L.wo); mats.push_back(&L.wgu); mats.push_back(&L.wd);
  }
  mats.push_back(&m->embed);
  if (!m->cfg.tied_embeddings) mats.push_back(&m->head);
  int64_t biggest = 0;
  for (Q8Mat* w : mats)
    if (w->k % 128 == 0 && w->tiled != tiled) biggest = std::max(biggest, ((w->n + 127) / 128 * 128) * w->k);
  if (biggest == 0) return LOGOS_OK;
  int8_t* tmp = nullptr;
  LOGOS_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&tmp), (size_t)biggest));
  logos_status_t rc = LOGOS_OK;
  for (Q8Mat* w : mats) {
    if (w->k % 128 || w->tiled == tiled) continue;
    const int64_t bytes = (tiled ? (w->n + 127) / 128 * 128 : w->n) * w->k;
    rc = launch_q8_retile(w->q, tmp, w->n, w->k, tiled, m->device, m->stream);
    if (rc != LOGOS_OK) break;
    if (cudaMemcpyAsync(w->q, tmp, (size_t)bytes, cudaMemcpyDeviceToDevice, m->stream) != cudaSuccess) {
      rc = fail(LOGOS_ERROR, "set_layout: device copy failed");
      break;
    }
    rc = launch_q8_retile_scales(w->s, reinterpret_cast<float*>(tmp), w->n, w->k, tiled, m->device, m->stream);
    if (rc != LOGOS_OK) break;
    if (cudaMemcpyAsync(w->s, tmp, (size_t)(bytes / 8), cudaMemcpyDeviceToDevice, m->stream) != cudaSuccess) {
      rc = fail(LOGOS_ERROR, "set_layout: device copy failed");
      break;
    }
    w->tiled = tiled;
  }
  cudaStreamSynchronize(m->stream);
  cudaFree(tmp);
  if (m->cfg.tied_embeddings) m->head = m->embed;
  return rc;
}

logos_status_t gen(Model* m, Q8Mat* w, int64_t n, int64_t row0, int64_t col0, int64_t k_total, int64_t mul, int64_t add,
                   uint64_t stream_id) {
  return launch_q8_quantize(true, nullptr, w->q, w->s, n, w->k, row0, col0, k_total, mul, add, m->cfg.seed, stream_id,
                            m->cfg.init_std, m->device, m->stream);
}

logos_status_t build(Model* m, const void* nccl_id) {
  const logos_llm_config_t& c = m->cfg;
  const int g = c.tp_degree, r = c.tp_rank;
  const int64_t H = c.hidden, D = c.head_dim, B = c.batch;
  m->hq_local = c.h_q / g;
  m->hkv_local = c.h_kv / g;
  m->nq = m->hq_local * D;
  m->nkv = m->hkv_local * D;
  m->nqkv = m->nq + 2 * m->nkv;
  m->f_local = c.ffn / g;
  const int64_t nq_total = c.h_q * D;

  LOGOS_CUDA_TRY(cudaSetDevice(m->device));
  LOGOS_CUDA_TRY(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
  LOGOS_CUDA_TRY(cudaEventCreate(&m->ev0));
  LOGOS_CUDA_TRY(cudaEventCreate(&m->ev1));
  LOGOS_TRY(tp_init(&m->tp, g, r, nccl_id));

  m->layers.resize((size_t)c.layers);
  const int64_t kv_elems = B * m->hkv_local * c.l_max * D;
  for (int64_t l = 0; l < c.layers; ++l) {
    Layer& L = m->layers[(size_t)l];
    const uint64_t st = (uint64_t)l * 16;
    LOGOS_TRY(alloc_mat(m, &L.wqkv, m->nqkv, H));
    LOGOS_TRY(alloc_mat(m, &L.wo, H, m->nq));
    LOGOS_TRY(alloc_mat(m, &L.wgu, 2 * m->f_local, H));
    LOGOS_TRY(alloc_mat(m, &L.wd, H, m->f_local));
    LOGOS_TRY(gen(m, &L.wqkv, m->nq, r * m->nq, 0, H, 1, 0, st + 0));
    LOGOS_TRY(gen(m, &L.wqkv, m->nkv, r * m->nkv, 0, H, 1, m->nq, st + 1));
    LOGOS_TRY(gen(m, &L.wqkv, m->nkv, r * m->nkv, 0, H, 1, m->nq + m->nkv, st + 2));
    LOGOS_TRY(gen(m, &L.wo, H, 0, r * m->nq, nq_total, 1, 0, st + 3));
    LOGOS_TRY(gen(m, &L.wgu, m->f_local, r * m->f_local, 0, H, 2, 0, st + 4));
    LOGOS_TRY(gen(m, &L.wgu, m->f_local, r * m->f_local, 0, H, 2, 1, st + 5));
    LOGOS_TRY(gen(m, &L.wd, H, 0, r * m->f_local, c.ffn, 1, 0, st + 6));
    if (c.qkv_bias) {  // streams 7, 8, 9 of the layer, valued by the row's index in the whole projection
      LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&L.bqkv), m->nqkv * 4));
      LOGOS_TRY(launch_synth_fill(L.bqkv, LOGOS_F32, 2, c.seed, st + 7, r * m->nq, m->nq, 0.f, c.init_std, m->device, m->stream));
      LOGOS_TRY(launch_synth_fill(L.bqkv + m->nq, LOGOS_F32, 2, c.seed, st + 8, r * m->nkv, m->nkv, 0.f, c.init_std, m->device,
                                  m->stream));
      LOGOS_TRY(launch_synth_fill(L.bqkv + m->nq + m->nkv, LOGOS_F32, 2, c.seed, st + 9, r * m->nkv, m->nkv, 0.f, c.init_std,
                                  m->device, m->stream));
    }
    LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&L.kc), kv_elems * 2));
    LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&L.vc), kv_elems * 2));
    LOGOS_CUDA_TRY(cudaMemsetAsync(L.kc, 0, (size_t)kv_elems * 2, m->stream));
    LOGOS_CUDA_TRY(cudaMemsetAsync(L.vc, 0, (size_t)kv_elems * 2, m->stream));
  }
  LOGOS_TRY(alloc_mat(m, &m->embed, c.vocab, H));
  LOGOS_TRY(gen(m, &m->embed, c.vocab, 0, 0, H, 1, 0, (uint64_t)1 << 20));
  if (c.tied_embeddings) {
    m->head = m->embed;
  } else {
    LOGOS_TRY(alloc_mat(m, &m->head, c.vocab, H));
    LOGOS_TRY(gen(m, &m->head, c.vocab, 0, 0, H, 1, 0, ((uint64_t)1 << 20) + 1));
  }

  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->gains), (2 * c.layers + 1) * H * 4));
  LOGOS_TRY(launch_synth_fill(m->gains, LOGOS_F32, 1, 0, 0, 0, (2 * c.layers + 1) * H, 1.0f, 1.0f, m->device, m->stream));
  {
    std::vector<float> tab((size_t)(c.l_max * D));
    rope_table_host(tab.data(), c.l_max, D, (double)c.rope_theta);
    LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->rope), c.l_max * D * 4));
    LOGOS_CUDA_TRY(cudaMemcpyAsync(m->rope, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, m->stream));
    LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
  }
  m->max_splits = 1;
  {
    int s1 = gemm_pick_splits(B, H, m->nq, m->device);
    int s2 = gemm_pick_splits(B, H, m->f_local, m->device);
    m->max_splits = s1 > s2 ? s1 : s2;
  }
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->h), B * H * 4));
  auto planes = [&](ActOut* a, int64_t elems) -> logos_status_t {
    a->mode = c.act_dtype;
    LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&a->hi), elems * 2));
    if (c.act_dtype == LOGOS_F32) LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&a->lo), elems * 2));
    return LOGOS_OK;
  };
  LOGOS_TRY(planes(&m->xn, B * H));
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->partials), (int64_t)m->max_splits * B * H * 4));
  // The block the ranks of a TP group map from each other: the two inboxes of the folded
  // exchange ([partial rows of the rows this rank owns, from every rank] and [normalised rows],
  // 16-byte slots of two words each) and the flag words, 256-byte aligned.
  {
    auto up = [](int64_t v) { return (v + 255) / 256 * 256; };
    const int64_t inbox_bytes = up(B * H * 8);  // both inboxes: rows x hidden / 2 slots of 16 bytes
    const int64_t off_xn = inbox_bytes, off_flags = 2 * inbox_bytes;
    const int64_t total = off_flags + up(TP_FLAG_WORDS * 4);
    const char* e = getenv("LOGOS_B200_TP_FUSED");
    // the default wherever the shapes allow it (measured faster than NCCL at 2, 4 and 8 GPUs);
    // LOGOS_B200_TP_FUSED=0 keeps the NCCL all-reduce
    const bool want = g > 1 && g <= 8 && B % g == 0 && H % 16 == 0 && B * 4 <= 2 * (int64_t)sm_count(m->device) &&
                      !(e && e[0] == '0');
    if (want) LOGOS_TRY(tp_symm_alloc(&m->tp, (size_t)total, &m->symm, m->stream));
    m->tp_fused = want && m->symm.ok;
    if (m->tp_fused) {
      m->tpf.degree = g;
      m->tpf.rank = r;
      m->tpf.act_mode = c.act_dtype;
      for (int k = 0; k < g; ++k) {
        char* base = static_cast<char*>(m->symm.base[k]);
        m->tpf.inbox_part[k] = reinterpret_cast<uint4*>(base);
        m->tpf.inbox_xn[k] = reinterpret_cast<uint4*>(base + off_xn);
      }
      m->tpf.flags = reinterpret_cast<uint32_t*>(static_cast<char*>(m->symm.base[r]) + off_flags);
      m->tpf.partials = m->partials;
      m->tpf.xn_hi = m->xn.hi;
      m->tpf.xn_lo = m->xn.lo;
    }
  }
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->qkv), B * m->nqkv * 4));
  LOGOS_TRY(planes(&m->att, B * m->nq));
  LOGOS_TRY(planes(&m->ffn, B * m->f_local));
  {
    // qkv and gate/up split K too when their row tiles alone would leave most SMs idle (the
    // per-rank shapes of a TP group): room for the larger of the two sets of partials
    const int s_qkv = gemm_pick_splits(B, m->nqkv, H, m->device), s_gu = gemm_pick_splits(B, 2 * m->f_local, H, m->device);
    const int64_t need_qkv = s_qkv > 1 ? (int64_t)s_qkv * B * m->nqkv : 0;
    const int64_t need_gu = s_gu > 1 ? (int64_t)s_gu * B * 2 * m->f_local : 0;
    m->dpart_floats = need_qkv > need_gu ? need_qkv : need_gu;
    if (m->dpart_floats > 0) LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->dpart), m->dpart_floats * 4));
  }
  {
    AttnArgs a;
    a.b = B; a.h_q = m->hq_local; a.h_kv = m->hkv_local; a.d = D; a.l_max = c.l_max; a.device = m->device;
    m->attn_scratch_bytes = attn_scratch_bytes(a);
    LOGOS_TRY(dmalloc(m, &m->attn_scratch, m->attn_scratch_bytes));
  }
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->logits), B * c.vocab * 4));
  m->history_cap = c.l_max;
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->history), m->history_cap * B * 4));
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->step_counter), 256));
  LOGOS_CUDA_TRY(cudaMemsetAsync(m->step_counter, 0, 256, m->stream));
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->tokens), B * 4));
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->seq_len), B * 4));
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->sampling), 256));
  LOGOS_CUDA_TRY(cudaMemsetAsync(m->sampling, 0, 256, m->stream));
  LOGOS_CUDA_TRY(cudaMemsetAsync(m->tokens, 0, (size_t)B * 4, m->stream));
  LOGOS_CUDA_TRY(cudaMemsetAsync(m->seq_len, 0, (size_t)B * 4, m->stream));
  LOGOS_CUDA_TRY(cudaMemsetAsync(m->logits, 0, (size_t)(B * c.vocab) * 4, m->stream));
  LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
  return set_layout(m, true);
}

__global__ void sum_partials_kernel(float* __restrict__ p, int parts, int64_t stride, int64_t count) {
  pdl_wait();
  pdl_trigger();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  float v = __ldcg(p + i);
  for (int s = 1; s < parts; ++s) v = __fadd_rn(v, __ldcg(p + (int64_t)s * stride + i));
  p[i] = v;
}

// prompt_len (ragged prompts, null otherwise): only sequences with prompt_step < prompt_len[i] advance
__global__ void bump_len_kernel(int32_t* seq_len, int32_t* step_counter, int b, int l_max,
                                const int32_t* __restrict__ prompt_len, int prompt_step) {
  pdl_wait();
  pdl_trigger();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < b && seq_len[i] < l_max && (!prompt_len || prompt_step < prompt_len[i])) seq_len[i] += 1;
  if (i == 0) *step_counter += 1;
}

// GEMM with its own output and epilogue (qkv, gate/up, lm_head): K is split, and a small kernel
// folds the partials and applies the epilogue, where the cost model prefers that.
// unfolded_splits (may be null): the caller's consumer folds the partials itself; it receives the
// split count (1 = the output is in g.c as usual) and the fold kernel is not launched.
logos_status_t gemm_direct(Model* m, const GemmArgs& g, int* unfolded_splits = nullptr) {
  ProfScope ps(m, PROF_GEMM);
  if (unfolded_splits) *unfolded_splits = 1;
  int splits = gemm_pick_splits(g.m, g.n, g.k, m->device);
  if (splits > 1 && (int64_t)splits * g.m * g.n <= m->dpart_floats && gemm_tc_applicable(g)) {
    GemmArgs gp = g;
    gp.splits = splits;
    gp.partials = m->dpart;
    gp.epilogue = EPI_NONE;
    gp.c = nullptr;
    gp.c_dtype = LOGOS_F32;
    gp.aux = nullptr;
    LOGOS_TRY(launch_q8_gemm(gp, m->stream));
    m->launch_counter += 1;
    if (unfolded_splits && g.epilogue == EPI_NONE && g.ldc == g.n) {
      *unfolded_splits = splits;
      return LOGOS_OK;
    }
    LOGOS_TRY(launch_splitk_reduce(m->dpart, splits, g.c, g.c_dtype, g.c_act, g.ldc, g.aux, g.m, g.n, g.epilogue,
                                   m->stream));
    m->launch_counter += 1;
    return LOGOS_OK;
  }
  LOGOS_TRY(launch_q8_gemm(g, m->stream));
  m->launch_counter += 1;
  return LOGOS_OK;
}

// GEMM producing f32 partials [splits][B][N] in m->partials; returns the split count.
logos_status_t gemm_partials(Model* m, const ActOut& a, const Q8Mat& w, int* splits_out) {
  const int64_t B = m->cfg.batch;
  GemmArgs g;
  g.a = a.hi; g.a_lo = a.lo; g.a_dtype = LOGOS_F16; g.lda = w.k;
  g.q = w.q; g.s = w.s; g.q_tiled = w.tiled;
  g.m = B; g.n = w.n; g.k = w.k;
  g.device = m->device;
  int splits = gemm_pick_splits(B, w.n, w.k, m->device);
  if (splits > m->max_splits) splits = m->max_splits;
  if (splits > 1 && gemm_tc_applicable(g)) {
    g.splits = splits;
    g.partials = m->partials;
  } else {
    splits = 1;
    g.c = m->partials; g.c_dtype = LOGOS_F32; g.ldc = w.n;
  }
  m->launch_counter += 1;
  {
    ProfScope ps(m, PROF_GEMM);
    LOGOS_TRY(launch_q8_gemm(g, m->stream));
  }
  if (m->tp.degree > 1 && !m->tp_fused) {
    ProfScope ps(m, PROF_COMM);
    const int64_t count = B * w.n;
    if (splits > 1) {
      LOGOS_CUDA_TRY(launch_kernel(sum_partials_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), 0, m->stream,
                                   m->partials, splits, count, count));
      LOGOS_TRY(check_launch("sum_partials_kernel"));
      m->launch_counter += 1;
      splits = 1;
    }
    LOGOS_TRY(tp_allreduce_sum_f32(&m->tp, m->partials, count, m->stream));
  }
  *splits_out = splits;
  return LOGOS_OK;
}

bool debug_sync();
bool pdl_enabled();
logos_status_t debug_check(Model* m, const char* what, int64_t layer) {
  if (!debug_sync()) return LOGOS_OK;
  LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
  int code = 0;
  LOGOS_TRY(kernel_status_read(m->device, &code, false));
  if (code != 0) {
    std::string detail = last_error_text() ? last_error_text() : "";
    return fail(LOGOS_ERROR, "kernel status %d first seen after %s of layer %lld [%s]", code, what, (long long)layer, detail.c_str());
  }
  return LOGOS_OK;
}

// Fold the pending partial sums into the residual stream and normalise: h += sum(partials),
// xn = planes(rmsnorm(h)).  With a peer-mapped TP group the sum runs over every rank's partials
// (the all-reduce is part of the kernel) and each rank updates only the rows it owns.
logos_status_t norm_step(Model* m, int parts, int64_t gain_row) {
  const logos_llm_config_t& c = m->cfg;
  const int64_t B = c.batch, H = c.hidden;
  const float* g = m->gains + gain_row * H;
  if (m->tp_fused && parts > 0) {
    ProfScope ps(m, PROF_COMM);
    return launch_tp_residual_rmsnorm(m->h, m->tpf, parts, B * H, g, B, H, c.rms_eps, m->device, m->stream);
  }
  ProfScope ps(m, PROF_ELEMWISE);
  return launch_residual_rmsnorm(m->h, m->partials, parts, B * H, g, m->xn, B, H, c.rms_eps, m->stream);
}

// The end of a step: final norm (folding `parts` pending partial sums), lm_head, token choice (when
// `sample`), then the lengths advance.
logos_status_t step_tail(Model* m, int parts, bool sample, bool log_tokens, const int32_t* prompt_len, int prompt_step) {
  const logos_llm_config_t& c = m->cfg;
  const int64_t B = c.batch, H = c.hidden;
  cudaStream_t st = m->stream;
  if (sample) {
    LOGOS_TRY(norm_step(m, parts, 2 * c.layers));
    GemmArgs g;
    g.a = m->xn.hi; g.a_lo = m->xn.lo; g.a_dtype = LOGOS_F16; g.lda = H;
    g.q = m->head.q; g.s = m->head.s; g.q_tiled = m->head.tiled;
    g.c = m->logits; g.c_dtype = LOGOS_F32; g.ldc = c.vocab;
    g.m = B; g.n = c.vocab; g.k = H;
    g.device = m->device;
    {
      ProfScope ps(m, PROF_GEMM);
      LOGOS_TRY(launch_q8_gemm(g, st));
    }
    ProfScope ps(m, PROF_ELEMWISE);
    // seq_len still holds the position of the token this step consumed (bump_len_kernel runs last)
    LOGOS_TRY(launch_argmax(m->logits, m->tokens, log_tokens ? m->history : nullptr, m->step_counter, m->history_cap, B,
                            c.vocab, m->sampling, m->seq_len, prompt_len, prompt_step, st));
    m->launch_counter += 3;
  }
  ProfScope ps_tail(m, PROF_ELEMWISE);
  LOGOS_CUDA_TRY(launch_kernel(bump_len_kernel, dim3((unsigned)((B + 127) / 128)), dim3(128), 0, st, m->seq_len,
                               m->step_counter, (int)B, (int)c.l_max, prompt_len, prompt_step));
  LOGOS_TRY(check_launch("bump_len_kernel"));
  m->launch_counter += 1;
  m->launches_per_step = m->launch_counter;
  return LOGOS_OK;
}

// One lock-step decode step on the model's stream.  tokens_in: [B] device.
// prompt_len ([B] device, ragged prompts only) with prompt_step: sequences whose prompt is over
// (prompt_step >= prompt_len[i]) run through the step without advancing - their K/V row lands at
// their next free position and is overwritten when they do advance - and only sequences whose
// prompt ends at this step take the sampled token.
logos_status_t step(Model* m, const int32_t* tokens_in, bool sample, bool log_tokens,
                    const int32_t* prompt_len = nullptr, int prompt_step = 0) {
  const logos_llm_config_t& c = m->cfg;
  const int64_t B = c.batch, H = c.hidden, D = c.head_dim;
  cudaStream_t st = m->stream;
  m->launch_counter = 0;
  // Every kernel of a step keeps the dependent-launch contract (common.cuh): weights are the
  // only thing a kernel touches before it has waited for its predecessor.
  PdlScope pdl(pdl_enabled());
  {
    ProfScope ps(m, PROF_ELEMWISE);
    LOGOS_TRY(launch_embed(tokens_in, m->embed.q, m->embed.s, m->h, B, H, m->embed.tiled ? 1 : 0, st));
  }
  m->launch_counter += 1;
  int parts = 0;
  for (int64_t l = 0; l < c.layers; ++l) {
    Layer& L = m->layers[(size_t)l];
    int qkv_parts = 1;
    LOGOS_TRY(norm_step(m, parts, 2 * l));
    m->launch_counter += 1;
    {
      GemmArgs g;
      g.a = m->xn.hi; g.a_lo = m->xn.lo; g.a_dtype = LOGOS_F16; g.lda = H;
      g.q = L.wqkv.q; g.s = L.wqkv.s; g.q_tiled = L.wqkv.tiled;
      g.c = m->qkv; g.c_dtype = LOGOS_F32; g.ldc = m->nqkv;
      g.m = B; g.n = m->nqkv; g.k = H;
      g.device = m->device;
      LOGOS_TRY(gemm_direct(m, g, &qkv_parts));  // split-K partials, if any, are folded by the attention kernel
    }
    LOGOS_TRY(debug_check(m, "qkv gemm", l));
    {
      ProfScope ps(m, PROF_ATTN);
      AttnArgs a;
      const float* qkv_src = qkv_parts > 1 ? m->dpart : m->qkv;
      a.q_f32 = qkv_src; a.q_ld = m->nqkv; a.rotate_q = 1;
      a.k_new_f32 = qkv_src + m->nq; a.v_new_f32 = qkv_src + m->nq + m->nkv; a.kv_ld = m->nqkv;
      a.f32_parts = qkv_parts; a.f32_part_stride = B * m->nqkv;
      if (L.bqkv) {
        a.q_bias = L.bqkv; a.k_bias = L.bqkv + m->nq; a.v_bias = L.bqkv + m->nq + m->nkv;
      }
      a.k_cache = L.kc; a.v_cache = L.vc; a.rope = m->rope; a.seq_len = m->seq_len;
      a.bump_seq_len = 0;
      a.o_dtype = LOGOS_ACT_PLANES; a.o_act = m->att;
      a.b = B; a.h_q = m->hq_local; a.h_kv = m->hkv_local; a.d = D; a.l_max = c.l_max;
      a.scale = 1.0f / sqrtf((float)D);
      a.device = m->device;
      a.ext_scratch = m->attn_scratch; a.ext_scratch_bytes = m->attn_scratch_bytes;
      LOGOS_TRY(launch_gqa_decode_attn(a, st));
      m->launch_counter += 2;
    }
    LOGOS_TRY(debug_check(m, "attention", l));
    LOGOS_TRY(gemm_partials(m, m->att, L.wo, &parts));
    LOGOS_TRY(debug_check(m, "o_proj gemm", l));
    LOGOS_TRY(norm_step(m, parts, 2 * l + 1));
    m->launch_counter += 1;
    {
      GemmArgs g;
      g.a = m->xn.hi; g.a_lo = m->xn.lo; g.a_dtype = LOGOS_F16; g.lda = H;
      g.q = L.wgu.q; g.s = L.wgu.s; g.q_tiled = L.wgu.tiled;
      g.c_dtype = LOGOS_ACT_PLANES; g.c_act = m->ffn; g.ldc = m->f_local;
      g.m = B; g.n = 2 * m->f_local; g.k = H;
      g.epilogue = EPI_SWIGLU;
      g.device = m->device;
      LOGOS_TRY(gemm_direct(m, g));
    }
    LOGOS_TRY(debug_check(m, "gate/up gemm", l));
    LOGOS_TRY(gemm_partials(m, m->ffn, L.wd, &parts));
    LOGOS_TRY(debug_check(m, "down_proj gemm", l));
  }
  return step_tail(m, parts, sample, log_tokens, prompt_len, prompt_step);
}

// h[b] = ws.h[row(b)] + ws.delta[row(b)] for the last prompt position of every sequence: the rows the
// end of the step (final norm, lm_head, token choice) runs on.
__global__ void gather_last_rows_kernel(float* __restrict__ h, const float* __restrict__ src, const float* __restrict__ delta,
                                        int64_t hidden, int64_t chunk) {
  pdl_wait();
  pdl_trigger();
  const int64_t b = blockIdx.x, row = b * chunk + chunk - 1;
  for (int64_t e = threadIdx.x; e < hidden; e += blockDim.x)
    h[b * hidden + e] = __fadd_rn(__ldcg(src + row * hidden + e), __ldcg(delta + row * hidden + e));
}

bool chunked_prefill_enabled() {
  const char* e = getenv("LOGOS_B200_PREFILL");
  return !(e && (e[0] == 'l' || e[0] == '0'));   // "loop" or "0": prompts run through the decode step token by token
}

logos_status_t prefill_workspace(Model* m, int64_t rows) {
  PrefillWs& w = m->pf;
  if (w.rows >= rows) return LOGOS_OK;
  const logos_llm_config_t& c = m->cfg;
  const int64_t H = c.hidden;
  auto planes = [&](ActOut* a, int64_t elems) -> logos_status_t {
    a->mode = c.act_dtype;
    LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&a->hi), elems * 2));
    if (c.act_dtype == LOGOS_F32) LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&a->lo), elems * 2));
    return LOGOS_OK;
  };
  // (a model is given one workspace, sized by the first prompt pass: later passes use chunks that fit it)
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&w.h), rows * H * 4));
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&w.delta), rows * H * 4));
  LOGOS_TRY(planes(&w.xn, rows * H));
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&w.qkv), rows * m->nqkv * 4));
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&w.q16), rows * m->nq * 2));
  LOGOS_TRY(planes(&w.att, rows * m->nq));
  LOGOS_TRY(planes(&w.ffn, rows * m->f_local));
  LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&w.tok), rows * 4));
  w.rows = rows;
  return LOGOS_OK;
}

// The prompt pass proper: chunks of positions, every sequence's chunk at once (rows = batch x chunk),
// so that each weight matrix is streamed once per chunk instead of once per token.  Per layer:
// norm -> qkv GEMM -> RoPE + KV write + causal attention -> o_proj GEMM -> norm -> gate/up GEMM
// with SwiGLU -> down GEMM, the same kernels and the same arithmetic as a decode step, on more rows.
// tokens_host: [B][t].  Leaves the cache filled for positions [0, t), the lengths at t and the
// token chosen after the last prompt position as the current token.
logos_status_t prefill_chunked(Model* m, const int32_t* tokens_host, int64_t t) {
  const logos_llm_config_t& c = m->cfg;
  const int64_t B = c.batch, H = c.hidden, D = c.head_dim;
  cudaStream_t st = m->stream;
  // rows per chunk: enough token tiles that the GEMMs fill the GPU several times over while the
  // chunk's activations stay inside L2 (LOGOS_B200_PREFILL_ROWS overrides: tests use small chunks)
  int64_t target_rows = 4096;
  if (const char* e = getenv("LOGOS_B200_PREFILL_ROWS")) target_rows = std::max<int64_t>(1, atoll(e));
  int64_t chunk = std::max<int64_t>(1, target_rows / B);
  if (m->pf.rows > 0 && chunk * B > m->pf.rows) chunk = std::max<int64_t>(1, m->pf.rows / B);
  if (chunk > t) chunk = t;
  if (chunk < 1) chunk = 1;
  LOGOS_TRY(prefill_workspace(m, B * chunk));
  PrefillWs& w = m->pf;
  PdlScope pdl(pdl_enabled());
  LOGOS_CUDA_TRY(cudaMemsetAsync(m->seq_len, 0, (size_t)B * 4, st));
  std::vector<int32_t> rows_tok;
  for (int64_t p0 = 0; p0 < t; p0 += chunk) {
    const int64_t cn = std::min(chunk, t - p0), M = B * cn;
    rows_tok.assign((size_t)M, 0);
    for (int64_t b = 0; b < B; ++b)
      for (int64_t j = 0; j < cn; ++j) rows_tok[(size_t)(b * cn + j)] = tokens_host[b * t + p0 + j];
    LOGOS_CUDA_TRY(cudaMemcpyAsync(w.tok, rows_tok.data(), (size_t)M * 4, cudaMemcpyHostToDevice, st));
    LOGOS_CUDA_TRY(cudaStreamSynchronize(st));   // rows_tok is reused by the next chunk
    LOGOS_TRY(launch_embed(w.tok, m->embed.q, m->embed.s, w.h, M, H, m->embed.tiled ? 1 : 0, st));
    auto gemm = [&](const ActOut& a, const Q8Mat& wt, int64_t k, GemmArgs g) -> logos_status_t {
      g.a = a.hi; g.a_lo = a.lo; g.a_dtype = LOGOS_F16; g.lda = k;
      g.q = wt.q; g.s = wt.s; g.q_tiled = wt.tiled;
      g.m = M; g.n = wt.n; g.k = k;
      g.device = m->device;
      return launch_q8_gemm(g, st);
    };
    auto reduce_delta = [&]() -> logos_status_t {
      if (m->tp.degree > 1) return tp_allreduce_sum_f32(&m->tp, w.delta, M * H, st);
      return LOGOS_OK;
    };
    for (int64_t l = 0; l < c.layers; ++l) {
      Layer& L = m->layers[(size_t)l];
      LOGOS_TRY(launch_residual_rmsnorm(w.h, w.delta, l == 0 ? 0 : 1, M * H, m->gains + (2 * l) * H, w.xn, M, H, c.rms_eps, st));
      {
        GemmArgs g;
        g.c = w.qkv; g.c_dtype = LOGOS_F32; g.ldc = m->nqkv;
        LOGOS_TRY(gemm(w.xn, L.wqkv, H, g));
      }
      {
        PrefillAttnArgs a;
        a.qkv = w.qkv; a.qkv_ld = m->nqkv; a.qkv_bias = L.bqkv; a.rope = m->rope; a.q16 = w.q16;
        a.k_cache = L.kc; a.v_cache = L.vc; a.o = w.att;
        a.b = B; a.h_q = m->hq_local; a.h_kv = m->hkv_local; a.d = D; a.l_max = c.l_max; a.chunk = cn; a.pos0 = p0;
        a.scale = 1.0f / sqrtf((float)D);
        a.device = m->device;
        LOGOS_TRY(launch_prefill_attn(a, st));
      }
      {
        GemmArgs g;
        g.c = w.delta; g.c_dtype = LOGOS_F32; g.ldc = H;
        LOGOS_TRY(gemm(w.att, L.wo, m->nq, g));
        LOGOS_TRY(reduce_delta());
      }
      LOGOS_TRY(launch_residual_rmsnorm(w.h, w.delta, 1, M * H, m->gains + (2 * l + 1) * H, w.xn, M, H, c.rms_eps, st));
      {
        GemmArgs g;
        g.c_dtype = LOGOS_ACT_PLANES; g.c_act = w.ffn; g.ldc = m->f_local;
        g.epilogue = EPI_SWIGLU;
        LOGOS_TRY(gemm(w.xn, L.wgu, H, g));
      }
      {
        GemmArgs g;
        g.c = w.delta; g.c_dtype = LOGOS_F32; g.ldc = H;
        LOGOS_TRY(gemm(w.ffn, L.wd, m->f_local, g));
        LOGOS_TRY(reduce_delta());
      }
      LOGOS_TRY(debug_check(m, "prefill layer", l));
    }
    if (p0 + cn >= t) {
      // the last position of every sequence: fold the pending delta, then the ordinary end of a step
      LOGOS_CUDA_TRY(launch_kernel(gather_last_rows_kernel, dim3((unsigned)B), dim3(256), 0, st, m->h, (const float*)w.h,
                                   (const float*)w.delta, H, cn));
      LOGOS_TRY(check_launch("gather_last_rows_kernel"));
    }
  }
  {
    std::vector<int32_t> len((size_t)B, (int32_t)(t - 1));   // the position the last prompt token sits at
    LOGOS_CUDA_TRY(cudaMemcpyAsync(m->seq_len, len.data(), (size_t)B * 4, cudaMemcpyHostToDevice, st));
    LOGOS_CUDA_TRY(cudaStreamSynchronize(st));
  }
  m->launch_counter = 0;
  LOGOS_TRY(step_tail(m, 0, true, false, nullptr, 0));
  LOGOS_CUDA_TRY(cudaStreamSynchronize(st));
  int code = 0;
  LOGOS_TRY(kernel_status_read(m->device, &code, false));
  if (code != 0) return fail(LOGOS_ERROR, "a device-side wait gave up during the prompt pass (kernel status %d)", code);
  return LOGOS_OK;
}

// LOGOS_B200_DEBUG_SYNC=1: synchronise after every launch group of a step and name the first
// one after which the device status word is set.
bool debug_sync() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LOGOS_B200_DEBUG_SYNC");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v == 1;
}

bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LOGOS_B200_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

bool graphs_enabled() {
  const char* e = getenv("LOGOS_B200_GRAPH");
  return !(e && e[0] == '0');
}

logos_status_t check_cfg(const logos_llm_config_t& c) {
  if (c.layers <= 0 || c.hidden <= 0 || c.h_q <= 0 || c.h_kv <= 0 || c.head_dim <= 0 || c.ffn <= 0 || c.vocab <= 0 ||
      c.l_max <= 0 || c.batch <= 0)
    return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_create: every extent must be positive");
  if (c.tp_degree < 1 || c.tp_rank < 0 || c.tp_rank >= c.tp_degree)
    return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_create: tp_rank %d of tp_degree %d", c.tp_rank, c.tp_degree);
  if (c.h_q % c.h_kv) return fail(LOGOS_ERROR, "logos_llm_create: h_q must be a multiple of h_kv");
  if (c.h_kv % c.tp_degree || c.ffn % c.tp_degree)
    return fail(LOGOS_ERROR, "logos_llm_create: h_kv and ffn must divide by tp_degree");
  if (c.head_dim != 64 && c.head_dim != 128) return fail(LOGOS_ERROR, "logos_llm_create: head_dim must be 64 or 128");
  if (c.hidden % 32 || (c.ffn / c.tp_degree) % 32 || ((c.h_q / c.tp_degree) * c.head_dim) % 32)
    return fail(LOGOS_ERROR, "logos_llm_create: hidden, ffn/tp and q width/tp must be multiples of the Q8 block 32");
  if (c.qkv_bias != 0 && c.qkv_bias != 1) return fail(LOGOS_ERROR, "logos_llm_create: qkv_bias must be 0 or 1");
  if (c.act_dtype != LOGOS_F32 && c.act_dtype != LOGOS_F16 && c.act_dtype != LOGOS_BF16)
    return fail(LOGOS_ERROR, "logos_llm_create: act_dtype must be LOGOS_F32, LOGOS_F16 or LOGOS_BF16");
  return LOGOS_OK;
}

// Streams host memory to the device (and back) through two pinned buffers, so that reading the
// next chunk out of the mapped file overlaps the copy of the previous one.
struct Stager {
  static constexpr size_t BYTES = (size_t)32 << 20;
  uint8_t* buf[2] = {nullptr, nullptr};
  cudaEvent_t ev[2] = {nullptr, nullptr};
  bool busy[2] = {false, false};
  int next = 0;
  cudaStream_t st = nullptr;

  logos_status_t init(cudaStream_t stream) {
    st = stream;
    for (int i = 0; i < 2; ++i) {
      LOGOS_CUDA_TRY(cudaMallocHost(reinterpret_cast<void**>(&buf[i]), BYTES));
      LOGOS_CUDA_TRY(cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming));
    }
    return LOGOS_OK;
  }
  ~Stager() {
    for (int i = 0; i < 2; ++i) {
      if (busy[i]) cudaEventSynchronize(ev[i]);
      if (ev[i]) cudaEventDestroy(ev[i]);
      if (buf[i]) cudaFreeHost(buf[i]);
    }
  }
  // host rows of `width` bytes, src_pitch apart -> device rows dst_pitch apart
  logos_status_t put(void* dst, size_t dst_pitch, const uint8_t* src, size_t src_pitch, size_t width, int64_t rows) {
    if (width == 0 || rows <= 0) return LOGOS_OK;
    if (width > BYTES) return fail(LOGOS_ERROR, "weight row of %zu bytes exceeds the staging buffer", width);
    const int64_t per = (int64_t)(BYTES / width);
    for (int64_t r0 = 0; r0 < rows; r0 += per) {
      const int64_t n = rows - r0 < per ? rows - r0 : per;
      if (busy[next]) LOGOS_CUDA_TRY(cudaEventSynchronize(ev[next]));
      if (src_pitch == width) {
        memcpy(buf[next], src + (size_t)r0 * src_pitch, (size_t)n * width);
      } else {
        for (int64_t i = 0; i < n; ++i) memcpy(buf[next] + (size_t)i * width, src + (size_t)(r0 + i) * src_pitch, width);
      }
      LOGOS_CUDA_TRY(cudaMemcpy2DAsync(static_cast<uint8_t*>(dst) + (size_t)r0 * dst_pitch, dst_pitch, buf[next], width, width,
                                       (size_t)n, cudaMemcpyHostToDevice, st));
      LOGOS_CUDA_TRY(cudaEventRecord(ev[next], st));
      busy[next] = true;
      next ^= 1;
    }
    return LOGOS_OK;
  }
  // device rows src_pitch apart -> `width` bytes per row written to the file at `off`, rows packed
  logos_status_t get_to_file(int fd, int64_t off, const void* src, size_t src_pitch, size_t width, int64_t rows) {
    if (width == 0 || rows <= 0) return LOGOS_OK;
    if (width > BYTES) return fail(LOGOS_ERROR, "weight row of %zu bytes exceeds the staging buffer", width);
    const int64_t per = (int64_t)(BYTES / width);
    for (int64_t r0 = 0; r0 < rows; r0 += per) {
      const int64_t n = rows - r0 < per ? rows - r0 : per;
      LOGOS_CUDA_TRY(cudaMemcpy2DAsync(buf[0], width, static_cast<const uint8_t*>(src) + (size_t)r0 * src_pitch, src_pitch,
                                       width, (size_t)n, cudaMemcpyDeviceToHost, st));
      LOGOS_CUDA_TRY(cudaStreamSynchronize(st));
      size_t done = 0, total = (size_t)n * width;
      while (done < total) {
        ssize_t k = pwrite(fd, buf[0] + done, total - done, (off_t)(off + r0 * (int64_t)width + (int64_t)done));
        if (k < 0 && errno == EINTR) continue;
        if (k <= 0) return fail(LOGOS_ERROR, "logos_llm_save_weights: write failed: %s", strerror(errno));
        done += (size_t)k;
      }
    }
    return LOGOS_OK;
  }
};

// Where one tensor of the file lives in the model: device rows and their pitches, for the int8
// part and for the scales (a gain vector: q only).
struct TensorHome {
  void* q = nullptr;
  size_t q_pitch = 0;
  void* s = nullptr;
  size_t s_pitch = 0;
};

TensorHome tensor_home(Model* m, int64_t l, int kind) {
  const int64_t H = m->cfg.hidden, hb = H / 32;
  TensorHome t;
  Layer* L = (kind <= LOGOS_W_DOWN || kind >= LOGOS_W_Q_BIAS) ? &m->layers[(size_t)l] : nullptr;
  auto rows_of = [&](Q8Mat& w, int64_t row0, int64_t mul) {
    t.q = w.q + row0 * w.k; t.q_pitch = (size_t)(mul * w.k);
    t.s = w.s + row0 * (w.k / 32); t.s_pitch = (size_t)(mul * (w.k / 32) * 4);
  };
  switch (kind) {
    case LOGOS_W_ATTN_NORM:  t.q = m->gains + (2 * l) * H; t.q_pitch = (size_t)H * 4; break;
    case LOGOS_W_MLP_NORM:   t.q = m->gains + (2 * l + 1) * H; t.q_pitch = (size_t)H * 4; break;
    case LOGOS_W_FINAL_NORM: t.q = m->gains + (2 * m->cfg.layers) * H; t.q_pitch = (size_t)H * 4; break;
    case LOGOS_W_Q_BIAS: t.q = L->bqkv; t.q_pitch = (size_t)m->nq * 4; break;
    case LOGOS_W_K_BIAS: t.q = L->bqkv + m->nq; t.q_pitch = (size_t)m->nkv * 4; break;
    case LOGOS_W_V_BIAS: t.q = L->bqkv + m->nq + m->nkv; t.q_pitch = (size_t)m->nkv * 4; break;
    case LOGOS_W_Q:    rows_of(L->wqkv, 0, 1); break;
    case LOGOS_W_K:    rows_of(L->wqkv, m->nq, 1); break;
    case LOGOS_W_V:    rows_of(L->wqkv, m->nq + m->nkv, 1); break;
    case LOGOS_W_O:    rows_of(L->wo, 0, 1); break;
    // gate row i and up row i are neighbours (rows 2i and 2i+1), which is what the SwiGLU epilogue pairs
    case LOGOS_W_GATE: rows_of(L->wgu, 0, 2); break;
    case LOGOS_W_UP:   rows_of(L->wgu, 0, 2); t.q = L->wgu.q + H; t.s = L->wgu.s + hb; break;
    case LOGOS_W_DOWN: rows_of(L->wd, 0, 1); break;
    case LOGOS_W_EMBED: rows_of(m->embed, 0, 1); break;
    case LOGOS_W_HEAD:  rows_of(m->head, 0, 1); break;
  }
  return t;
}

logos_status_t same_arch(const WeightsArch& f, const WeightsArch& a, const char* who) {
  if (f.layers != a.layers || f.hidden != a.hidden || f.h_q != a.h_q || f.h_kv != a.h_kv || f.head_dim != a.head_dim ||
      f.ffn != a.ffn || f.vocab != a.vocab || f.tied != a.tied || f.qkv_bias != a.qkv_bias)
    return fail(LOGOS_ERROR,
                "%s: the file holds layers %lld hidden %lld heads %lld/%lld x %lld ffn %lld vocab %lld tied %d qkv_bias %d, "
                "the model layers %lld hidden %lld heads %lld/%lld x %lld ffn %lld vocab %lld tied %d qkv_bias %d",
                who, (long long)f.layers, (long long)f.hidden, (long long)f.h_q, (long long)f.h_kv, (long long)f.head_dim,
                (long long)f.ffn, (long long)f.vocab, f.tied, f.qkv_bias, (long long)a.layers, (long long)a.hidden,
                (long long)a.h_q, (long long)a.h_kv, (long long)a.head_dim, (long long)a.ffn, (long long)a.vocab, a.tied,
                a.qkv_bias);
  return LOGOS_OK;
}

// Every tensor of the file in storage order: fn(layer, kind).
template <class F>
logos_status_t for_each_tensor(const WeightsArch& a, F&& fn) {
  for (int64_t l = 0; l < a.layers; ++l) {
    for (int kind = LOGOS_W_ATTN_NORM; kind <= LOGOS_W_V; ++kind) LOGOS_TRY(fn(l, kind));
    if (a.qkv_bias)
      for (int kind = LOGOS_W_Q_BIAS; kind <= LOGOS_W_V_BIAS; ++kind) LOGOS_TRY(fn(l, kind));
    for (int kind = LOGOS_W_O; kind <= LOGOS_W_DOWN; ++kind) LOGOS_TRY(fn(l, kind));
  }
  LOGOS_TRY(fn((int64_t)0, (int)LOGOS_W_FINAL_NORM));
  LOGOS_TRY(fn((int64_t)0, (int)LOGOS_W_EMBED));
  if (!a.tied) LOGOS_TRY(fn((int64_t)0, (int)LOGOS_W_HEAD));
  return LOGOS_OK;
}

logos_status_t load_weights(Model* m, const MappedWeights& w) {
  const char* who = "logos_llm_load_weights";
  const WeightsArch a = arch_of(m->cfg);
  LOGOS_TRY(same_arch(w.arch, a, who));
  LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));  // no step reads the weights while they change
  Stager stg;
  LOGOS_TRY(stg.init(m->stream));
  LOGOS_TRY(for_each_tensor(a, [&](int64_t l, int kind) -> logos_status_t {
    TensorSpan t;
    ShardRect r;
    LOGOS_TRY(weights_span(a, l, kind, &t, who));
    LOGOS_TRY(weights_shard(a, kind, m->cfg.tp_degree, m->cfg.tp_rank, &r, who));
    const TensorHome home = tensor_home(m, l, kind);
    if (is_vector(kind))  // a gain whole, a bias this rank's slice
      return stg.put(home.q, home.q_pitch, w.base + t.q_off + r.col0 * 4, (size_t)r.cols * 4, (size_t)r.cols * 4, 1);
    const int64_t kb = t.k / 32;
    LOGOS_TRY(stg.put(home.q, home.q_pitch, w.base + t.q_off + r.row0 * t.k + r.col0, (size_t)t.k, (size_t)r.cols, r.rows));
    return stg.put(home.s, home.s_pitch, w.base + t.s_off + (r.row0 * kb + r.col0 / 32) * 4, (size_t)kb * 4,
                   (size_t)(r.cols / 32) * 4, r.rows);
  }));
  LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
  return LOGOS_OK;
}

logos_status_t save_weights(Model* m, int fd) {
  const char* who = "logos_llm_save_weights";
  const WeightsArch a = arch_of(m->cfg);
  const int64_t total = weights_file_bytes(a);
  if (ftruncate(fd, (off_t)total) != 0) return fail(LOGOS_ERROR, "%s: cannot size the file: %s", who, strerror(errno));
  uint8_t header[256];
  LOGOS_TRY(logos_llm_weights_header(&m->cfg, header));
  if (pwrite(fd, header, sizeof(header), 0) != (ssize_t)sizeof(header))
    return fail(LOGOS_ERROR, "%s: write failed: %s", who, strerror(errno));
  LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
  Stager stg;
  LOGOS_TRY(stg.init(m->stream));
  return for_each_tensor(a, [&](int64_t l, int kind) -> logos_status_t {
    TensorSpan t;
    LOGOS_TRY(weights_span(a, l, kind, &t, who));
    const TensorHome home = tensor_home(m, l, kind);
    if (is_vector(kind)) return stg.get_to_file(fd, t.q_off, home.q, home.q_pitch, (size_t)t.q_bytes, 1);
    LOGOS_TRY(stg.get_to_file(fd, t.q_off, home.q, home.q_pitch, (size_t)t.k, t.n));
    return stg.get_to_file(fd, t.s_off, home.s, home.s_pitch, (size_t)(t.k / 32) * 4, t.n);
  });
}

Model* get_model(logos_handle_t h) { return static_cast<Model*>(registry_get(h, ObjKind::Model)); }

#define MODEL_OR_FAIL(m, h, who)                                                           \
  if (!(h)) return fail(LOGOS_NULL_POINTER, who ": null model handle");                    \
  Model* m = get_model(h);                                                                 \
  if (!m) return fail(LOGOS_INVALID_HANDLE, who ": invalid or freed model handle");        \
  LOGOS_CUDA_TRY(cudaSetDevice(m->device));

}  // namespace
}  // namespace logos

using namespace logos;

extern "C" {

logos_status_t logos_llm_create(const logos_llm_config_t* cfg, const void* nccl_unique_id_or_null, logos_handle_t* out) {
  return guarded([&]() -> logos_status_t {
    if (!out) return fail(LOGOS_NULL_POINTER, "logos_llm_create: out is null");
    *out = nullptr;
    if (!cfg) return fail(LOGOS_NULL_POINTER, "logos_llm_create: cfg is null");
    LOGOS_TRY(check_cfg(*cfg));
    int ndev = logos_device_count();
    if (ndev == 0) return fail(LOGOS_ERROR, "logos_llm_create: no CUDA device (this library has no CPU path)");
    if (cfg->device < 0 || cfg->device >= ndev)
      return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_create: device %d of %d", cfg->device, ndev);
    Model* m = new Model();
    m->cfg = *cfg;
    m->device = cfg->device;
    logos_status_t s = build(m, nccl_unique_id_or_null);
    if (s != LOGOS_OK) {
      std::string keep = last_error_text() ? last_error_text() : "";
      destroy(m);
      set_last_error(keep);
      return s;
    }
    *out = registry_put(ObjKind::Model, m);
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_prefill(logos_handle_t model, const int32_t* tokens_host, int64_t t) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_prefill");
    if (!tokens_host) return fail(LOGOS_NULL_POINTER, "logos_llm_prefill: tokens_host is null");
    const int64_t B = m->cfg.batch;
    if (t <= 0 || t > m->cfg.l_max) return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_prefill: t=%lld outside [1,%lld]", (long long)t, (long long)m->cfg.l_max);
    for (int64_t i = 0; i < B * t; ++i)
      if (tokens_host[i] < 0 || tokens_host[i] >= m->cfg.vocab)
        return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_prefill: token id %d outside the vocabulary", tokens_host[i]);
    if (chunked_prefill_enabled()) return prefill_chunked(m, tokens_host, t);
    if (m->prompt_cap < B * t) {
      LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->prompt), B * t * 4));
      m->prompt_cap = B * t;
    }
    std::vector<int32_t> tr((size_t)(B * t));
    for (int64_t b = 0; b < B; ++b)
      for (int64_t p = 0; p < t; ++p) tr[(size_t)(p * B + b)] = tokens_host[b * t + p];
    LOGOS_CUDA_TRY(cudaMemcpyAsync(m->prompt, tr.data(), tr.size() * 4, cudaMemcpyHostToDevice, m->stream));
    LOGOS_CUDA_TRY(cudaMemsetAsync(m->seq_len, 0, (size_t)B * 4, m->stream));
    for (int64_t p = 0; p < t; ++p) LOGOS_TRY(step(m, m->prompt + p * B, p == t - 1, false));
    LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_prefill_ragged(logos_handle_t model, const int32_t* tokens_host, int64_t t_max,
                                        const int32_t* lens_host) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_prefill_ragged");
    if (!tokens_host || !lens_host) return fail(LOGOS_NULL_POINTER, "logos_llm_prefill_ragged: null argument");
    const int64_t B = m->cfg.batch;
    if (t_max <= 0 || t_max > m->cfg.l_max)
      return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_prefill_ragged: t_max=%lld outside [1,%lld]", (long long)t_max,
                  (long long)m->cfg.l_max);
    int64_t longest = 0;
    for (int64_t b = 0; b < B; ++b) {
      if (lens_host[b] < -1 || lens_host[b] > t_max)
        return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_prefill_ragged: length %d of sequence %lld outside [-1,%lld]", lens_host[b],
                    (long long)b, (long long)t_max);
      if (lens_host[b] > longest) longest = lens_host[b];
      for (int64_t p = 0; p < lens_host[b]; ++p)
        if (tokens_host[b * t_max + p] < 0 || tokens_host[b * t_max + p] >= m->cfg.vocab)
          return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_prefill_ragged: token id %d outside the vocabulary",
                      tokens_host[b * t_max + p]);
    }
    // device: [longest][B] prompt tokens (0 past a sequence's end), then the [B] lengths
    const int64_t need = (longest + 1) * B;
    if (m->prompt_cap < need) {
      LOGOS_TRY(dmalloc(m, reinterpret_cast<void**>(&m->prompt), need * 4));
      m->prompt_cap = need;
    }
    std::vector<int32_t> tr((size_t)need, 0);
    for (int64_t b = 0; b < B; ++b) {
      for (int64_t p = 0; p < lens_host[b]; ++p) tr[(size_t)(p * B + b)] = tokens_host[b * t_max + p];
      tr[(size_t)(longest * B + b)] = lens_host[b];
    }
    LOGOS_CUDA_TRY(cudaMemcpyAsync(m->prompt, tr.data(), tr.size() * 4, cudaMemcpyHostToDevice, m->stream));
    // restarted sequences begin empty with token 0 (what an empty prompt leaves); length -1 keeps a
    // sequence's cache, length and current token
    std::vector<int32_t> len_now((size_t)B), tok_now((size_t)B);
    LOGOS_CUDA_TRY(cudaMemcpyAsync(len_now.data(), m->seq_len, (size_t)B * 4, cudaMemcpyDeviceToHost, m->stream));
    LOGOS_CUDA_TRY(cudaMemcpyAsync(tok_now.data(), m->tokens, (size_t)B * 4, cudaMemcpyDeviceToHost, m->stream));
    LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
    for (int64_t b = 0; b < B; ++b)
      if (lens_host[b] >= 0) len_now[(size_t)b] = tok_now[(size_t)b] = 0;
    LOGOS_CUDA_TRY(cudaMemcpyAsync(m->seq_len, len_now.data(), (size_t)B * 4, cudaMemcpyHostToDevice, m->stream));
    LOGOS_CUDA_TRY(cudaMemcpyAsync(m->tokens, tok_now.data(), (size_t)B * 4, cudaMemcpyHostToDevice, m->stream));
    const int32_t* lens_dev = m->prompt + longest * B;
    for (int64_t p = 0; p < longest; ++p) {
      bool ends_here = false;
      for (int64_t b = 0; b < B; ++b) ends_here = ends_here || lens_host[b] - 1 == p;
      LOGOS_TRY(step(m, m->prompt + p * B, ends_here, false, lens_dev, (int)p));
    }
    LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_synth_kv(logos_handle_t model, int64_t t, uint64_t seed) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_synth_kv");
    const logos_llm_config_t& c = m->cfg;
    if (t < 0 || t > c.l_max) return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_synth_kv: t outside [0,l_max]");
    const int64_t D = c.head_dim, B = c.batch;
    for (int64_t l = 0; l < c.layers; ++l) {
      const int64_t h0 = (int64_t)c.tp_rank * m->hkv_local;
      LOGOS_TRY(launch_synth_kv(m->layers[(size_t)l].kc, seed, (uint64_t)(2 * l), B, m->hkv_local, h0, c.h_kv, c.l_max, D,
                                t, m->device, m->stream));
      LOGOS_TRY(launch_synth_kv(m->layers[(size_t)l].vc, seed, (uint64_t)(2 * l + 1), B, m->hkv_local, h0, c.h_kv, c.l_max,
                                D, t, m->device, m->stream));
    }
    std::vector<int32_t> len((size_t)B, (int32_t)t);
    LOGOS_CUDA_TRY(cudaMemcpyAsync(m->seq_len, len.data(), (size_t)B * 4, cudaMemcpyHostToDevice, m->stream));
    LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_set_tokens(logos_handle_t model, const int32_t* tokens_host) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_set_tokens");
    if (!tokens_host) return fail(LOGOS_NULL_POINTER, "logos_llm_set_tokens: tokens_host is null");
    for (int64_t i = 0; i < m->cfg.batch; ++i)
      if (tokens_host[i] < 0 || tokens_host[i] >= m->cfg.vocab)
        return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_set_tokens: token id %d outside the vocabulary", tokens_host[i]);
    LOGOS_CUDA_TRY(cudaMemcpyAsync(m->tokens, tokens_host, (size_t)m->cfg.batch * 4, cudaMemcpyHostToDevice, m->stream));
    LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_decode_steps(logos_handle_t model, int64_t steps, int32_t* tokens_host_or_null) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_decode_steps");
    const int64_t B = m->cfg.batch;
    if (steps < 0) return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_decode_steps: negative step count");
    if (steps == 0) return LOGOS_OK;
    if (steps > m->history_cap)
      return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_decode_steps: %lld steps exceed l_max = %lld", (long long)steps,
                  (long long)m->history_cap);
    LOGOS_CUDA_TRY(cudaMemsetAsync(m->step_counter, 0, sizeof(int32_t), m->stream));
    LOGOS_CUDA_TRY(cudaEventRecord(m->ev0, m->stream));
    for (int64_t i = 0; i < steps; ++i) {
      // The first step of a model runs eagerly; after that one step is captured once and
      // replayed: all of its arguments are device-resident and every buffer it names is owned
      // by the model.
      if (!m->step_graph && !m->graph_failed && m->eager_sample_steps >= 1 && graphs_enabled()) {
        cudaGraph_t graph = nullptr;
        bool good = cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
        logos_status_t cs = good ? step(m, m->tokens, true, true) : LOGOS_ERROR;
        cudaError_t ee = good ? cudaStreamEndCapture(m->stream, &graph) : cudaErrorUnknown;
        good = good && cs == LOGOS_OK && ee == cudaSuccess && graph &&
               cudaGraphInstantiate(&m->step_graph, graph, 0) == cudaSuccess;
        if (graph) cudaGraphDestroy(graph);
        if (!good) {
          cudaGetLastError();
          m->step_graph = nullptr;
          m->graph_failed = true;  // stay on the eager path
        }
      }
      if (m->step_graph) {
        LOGOS_CUDA_TRY(cudaGraphLaunch(m->step_graph, m->stream));
      } else {
        LOGOS_TRY(step(m, m->tokens, true, true));
        m->eager_sample_steps += 1;
      }
    }
    LOGOS_CUDA_TRY(cudaEventRecord(m->ev1, m->stream));
    if (tokens_host_or_null)
      LOGOS_CUDA_TRY(cudaMemcpyAsync(tokens_host_or_null, m->history, (size_t)(steps * B) * 4, cudaMemcpyDeviceToHost, m->stream));
    LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
    float ms = 0.f;
    LOGOS_CUDA_TRY(cudaEventElapsedTime(&ms, m->ev0, m->ev1));
    m->last_ms = ms;
    int code = 0;
    LOGOS_TRY(kernel_status_read(m->device, &code, false));
    if (code != 0) return fail(LOGOS_ERROR, "a device-side wait gave up (kernel status %d)", code);
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_profile_step(logos_handle_t model, double* ms_by_class_out) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_profile_step");
    if (!ms_by_class_out) return fail(LOGOS_NULL_POINTER, "logos_llm_profile_step: null output");
    m->profiling = true;
    m->prof_used = 0;
    m->prof_class.clear();
    logos_status_t s = step(m, m->tokens, true, false);
    m->profiling = false;
    LOGOS_TRY(s);
    LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
    for (int i = 0; i < PROF_CLASSES; ++i) ms_by_class_out[i] = 0.0;
    for (size_t i = 0; i < m->prof_class.size(); ++i) {
      float ms = 0.f;
      LOGOS_CUDA_TRY(cudaEventElapsedTime(&ms, m->prof_events[2 * i], m->prof_events[2 * i + 1]));
      ms_by_class_out[m->prof_class[i]] += ms;
    }
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_decode_step(logos_handle_t model, int32_t* next_tokens_host) {
  return logos_llm_decode_steps(model, 1, next_tokens_host);
}

logos_status_t logos_llm_read_kv(logos_handle_t model, int64_t layer, void* k_host, void* v_host) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_read_kv");
    if (!k_host || !v_host) return fail(LOGOS_NULL_POINTER, "logos_llm_read_kv: null output");
    if (layer < 0 || layer >= m->cfg.layers) return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_read_kv: layer %lld", (long long)layer);
    size_t bytes = (size_t)(m->cfg.batch * m->hkv_local * m->cfg.l_max * m->cfg.head_dim) * 2;
    LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
    LOGOS_CUDA_TRY(cudaMemcpy(k_host, m->layers[(size_t)layer].kc, bytes, cudaMemcpyDeviceToHost));
    LOGOS_CUDA_TRY(cudaMemcpy(v_host, m->layers[(size_t)layer].vc, bytes, cudaMemcpyDeviceToHost));
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_read_logits(logos_handle_t model, float* logits_host) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_read_logits");
    if (!logits_host) return fail(LOGOS_NULL_POINTER, "logos_llm_read_logits: null output");
    LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
    LOGOS_CUDA_TRY(cudaMemcpy(logits_host, m->logits, (size_t)(m->cfg.batch * m->cfg.vocab) * 4, cudaMemcpyDeviceToHost));
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_read_seq_len(logos_handle_t model, int32_t* seq_len_host) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_read_seq_len");
    if (!seq_len_host) return fail(LOGOS_NULL_POINTER, "logos_llm_read_seq_len: null output");
    LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
    LOGOS_CUDA_TRY(cudaMemcpy(seq_len_host, m->seq_len, (size_t)m->cfg.batch * 4, cudaMemcpyDeviceToHost));
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_set_seq_len(logos_handle_t model, int64_t t) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_set_seq_len");
    if (t < 0 || t > m->cfg.l_max) return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_set_seq_len: t outside [0,l_max]");
    std::vector<int32_t> len((size_t)m->cfg.batch, (int32_t)t);
    LOGOS_CUDA_TRY(cudaMemcpyAsync(m->seq_len, len.data(), len.size() * 4, cudaMemcpyHostToDevice, m->stream));
    LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_set_sampling(logos_handle_t model, float temperature, int64_t top_k, uint64_t seed) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_set_sampling");
    if (!(temperature >= 0.0f) || temperature > 1e6f)
      return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_set_sampling: temperature %g outside [0, 1e6]", (double)temperature);
    if (top_k < 0) return fail(LOGOS_OUT_OF_BOUNDS, "logos_llm_set_sampling: top_k %lld is negative", (long long)top_k);
    SamplingParams p;
    p.enabled = temperature > 0.0f ? 1 : 0;
    p.inv_temperature = p.enabled ? 1.0f / temperature : 1.0f;
    p.seed = seed;
    p.top_k = top_k >= m->cfg.vocab ? 0 : (int32_t)top_k;  // the whole vocabulary: no filter
    p.reserved = 0;
    LOGOS_CUDA_TRY(cudaMemcpyAsync(m->sampling, &p, sizeof(p), cudaMemcpyHostToDevice, m->stream));
    LOGOS_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_last_timing(logos_handle_t model, double* ms_out, int64_t* launches_per_step_out) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_last_timing");
    if (ms_out) *ms_out = m->last_ms;
    if (launches_per_step_out) *launches_per_step_out = m->launches_per_step;
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_get_config(logos_handle_t model, logos_llm_config_t* cfg_out) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_get_config");
    if (!cfg_out) return fail(LOGOS_NULL_POINTER, "logos_llm_get_config: cfg_out is null");
    *cfg_out = m->cfg;
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_tp_exchange(logos_handle_t model, int32_t* mode_out) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_tp_exchange");
    if (!mode_out) return fail(LOGOS_NULL_POINTER, "logos_llm_tp_exchange: mode_out is null");
    *mode_out = m->tp.degree <= 1 ? 0 : (m->tp_fused ? 2 : 1);
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_load_weights(logos_handle_t model, const char* path) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_load_weights");
    if (!path) return fail(LOGOS_NULL_POINTER, "logos_llm_load_weights: path is null");
    MappedWeights w;
    LOGOS_TRY(weights_open(path, &w, "logos_llm_load_weights"));
    logos_status_t s = set_layout(m, false);   // the loader addresses rows
    if (s == LOGOS_OK) s = load_weights(m, w);
    weights_close(&w);
    std::string keep = s != LOGOS_OK && last_error_text() ? last_error_text() : "";
    logos_status_t t = set_layout(m, true);
    if (s != LOGOS_OK) set_last_error(keep);
    return s != LOGOS_OK ? s : t;
  });
}

logos_status_t logos_llm_save_weights(logos_handle_t model, const char* path) {
  return guarded([&]() -> logos_status_t {
    MODEL_OR_FAIL(m, model, "logos_llm_save_weights");
    if (!path) return fail(LOGOS_NULL_POINTER, "logos_llm_save_weights: path is null");
    if (m->cfg.tp_degree != 1)
      return fail(LOGOS_ERROR, "logos_llm_save_weights: a rank of a tensor-parallel group holds no whole matrix (tp_degree %d)",
                  m->cfg.tp_degree);
    int fd = open(path, O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) return fail(LOGOS_ERROR, "logos_llm_save_weights: cannot create '%s': %s", path, strerror(errno));
    logos_status_t s = set_layout(m, false);   // the writer addresses rows
    if (s == LOGOS_OK) s = save_weights(m, fd);
    std::string keep = s != LOGOS_OK && last_error_text() ? last_error_text() : "";
    {
      logos_status_t t = set_layout(m, true);
      if (s == LOGOS_OK && t != LOGOS_OK) { s = t; keep = last_error_text() ? last_error_text() : ""; }
    }
    if (close(fd) != 0 && s == LOGOS_OK) s = fail(LOGOS_ERROR, "logos_llm_save_weights: close failed: %s", strerror(errno));
    else if (s != LOGOS_OK) set_last_error(keep);
    return s;
  });
}

logos_status_t logos_llm_free(logos_handle_t model) {
  return guarded([&]() -> logos_status_t {
    if (!model) return fail(LOGOS_NULL_POINTER, "logos_llm_free: null handle");
    Model* m = static_cast<Model*>(registry_take(model, ObjKind::Model));
    if (!m) return fail(LOGOS_INVALID_HANDLE, "logos_llm_free: invalid or already freed handle");
    destroy(m);
    return LOGOS_OK;
  });
}

}  // extern "C"
