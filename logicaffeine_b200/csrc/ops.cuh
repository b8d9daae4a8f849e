// Internal launchers: raw device pointers in, kernels enqueued on a stream.
// The extern "C" wrappers and the decode step both go through these.
#pragma once
#include "act.cuh"
#include "common.cuh"

namespace logos {

// ---- synthetic inputs / weight prep (synth.cu)
logos_status_t launch_synth_fill(void* dst, int dtype, int kind, uint64_t seed, uint64_t stream, int64_t first,
                                 int64_t count, float a, float b, int device, cudaStream_t st);
// Rows [row0,row0+n) x columns [col0,col0+k) of a logical [.][k_total] N(0,std)
// matrix (or of `w`, ld k_total, when generate is false).  Output row r goes to
// physical row r*out_row_mul + out_row_add of q/s, whose row length is k.
logos_status_t launch_q8_quantize(bool generate, const float* w, int8_t* q, float* s, int64_t n, int64_t k,
                                  int64_t row0, int64_t col0, int64_t k_total, int64_t out_row_mul,
                                  int64_t out_row_add, uint64_t seed, uint64_t stream, float std, int device,
                                  cudaStream_t st);

// int8 [n][k] row-major <-> tile-major (128 x 128 tiles of 16 contiguous KB, ordered (row tile, K tile),
// ceil128(n) rows; K a multiple of 128): the layout a model keeps its GEMM weights in.  The tiled
// bytes hold q + 128 (top bit flipped), the form the GEMM's int8 -> fp16 conversion starts from.
// in != out.
logos_status_t launch_q8_retile(const int8_t* in, int8_t* out, int64_t n, int64_t k, bool to_tiled, int device,
                                cudaStream_t st);
// and their scales: f32 [n][k/32] row-major <-> [row tile][K tile][128 rows][4 scales]
logos_status_t launch_q8_retile_scales(const float* in, float* out, int64_t n, int64_t k, bool to_tiled, int device,
                                       cudaStream_t st);

logos_status_t launch_synth_kv(__half* cache, uint64_t seed, uint64_t stream, int64_t b, int64_t hkv_local, int64_t h0,
                               int64_t hkv_total, int64_t l_max, int64_t d, int64_t t, int device, cudaStream_t st);

// ---- GEMV (q8_gemv.cu)
logos_status_t launch_q8_gemv(const int8_t* q, const float* s, const float* x, float* y, int64_t n, int64_t k,
                              int device, cudaStream_t st);

// ---- GEMM (q8_gemm.cu)
enum GemmEpilogue : int {
  EPI_NONE = 0,      // C = acc
  EPI_RESIDUAL = 1,  // C = acc + aux
  EPI_SWIGLU = 2,    // rows (2j,2j+1) = (gate_j, up_j); C[m][j] = silu(gate)*up
};

struct GemmArgs {
  const void*   a = nullptr;   // activations [M][K], row stride lda elements
  const __half* a_lo = nullptr;  // second fp16 plane (see act.cuh); only with a_dtype LOGOS_F16
  int           a_dtype = LOGOS_BF16;  // LOGOS_F16 plane(s), LOGOS_BF16 or LOGOS_F32
  int64_t       lda = 0;
  const int8_t* q = nullptr;   // [N][K] row-major, or tile-major when q_tiled (launch_q8_retile)
  int           q_tiled = 0;   // tcgen05 kernel only; s is then tile-major too (launch_q8_retile_scales)
  const float*  s = nullptr;   // [N][K/32]
  void*         c = nullptr;   // [M][N] (or [M][N/2] for EPI_SWIGLU), row stride ldc elements
  int           c_dtype = LOGOS_BF16;  // LOGOS_BF16, LOGOS_F16, LOGOS_F32 or LOGOS_ACT_PLANES
  ActOut        c_act;         // destination planes when c_dtype == LOGOS_ACT_PLANES
  int64_t       ldc = 0;
  const void*   aux = nullptr; // EPI_RESIDUAL: same type and stride as c
  int64_t       m = 0, n = 0, k = 0;
  int           epilogue = EPI_NONE;
  // split-K: when > 1 the kernel writes f32 partials [splits][M][N] to
  // `partials` and the caller reduces them; epilogue must be EPI_NONE.
  int           splits = 1;
  float*        partials = nullptr;
  int           device = 0;
  int           force_simt = 0;  // use the SIMT kernel even where the tensor-core one applies
};
logos_status_t launch_q8_gemm(const GemmArgs& g, cudaStream_t st);
// How many K-splits launch_q8_gemm would like for this shape (1 = none).
int gemm_pick_splits(int64_t m, int64_t n, int64_t k, int device);
// Whether the tcgen05 kernel accepts this call (else the SIMT kernel runs).
bool gemm_tc_applicable(const GemmArgs& g);

// ---- attention (attention.cu)
struct AttnArgs {
  // query: either f16 [B][Hq][D] (q_f16) or f32 rows inside a wider matrix
  // (q_f32, row stride q_ld floats per sequence, head h at column h*D).
  const __half* q_f16 = nullptr;
  const float*  q_f32 = nullptr;
  int64_t       q_ld = 0;
  int           rotate_q = 0;        // apply rotary embedding at position seq_len[b]
  // new row to append before attending (fused form); null = none
  const __half* k_new_f16 = nullptr;
  const __half* v_new_f16 = nullptr;
  const float*  k_new_f32 = nullptr; // f32 rows, stride kv_ld per sequence
  const float*  v_new_f32 = nullptr;
  int64_t       kv_ld = 0;
  // The f32 inputs (q_f32, k_new_f32, v_new_f32) may be split-K partial sums: f32_parts copies,
  // f32_part_stride floats apart, added in ascending order where the kernel stages them (the
  // fold the GEMM's reduce kernel would have done, without its launch).
  int           f32_parts = 1;
  int64_t       f32_part_stride = 0;
  // Bias vectors of the q, k and v projections (f32 [Hq*D], [Hkv*D], [Hkv*D]; f32 inputs only),
  // added after the partial copies where the kernel stages its inputs.  Null = none.
  const float*  q_bias = nullptr;
  const float*  k_bias = nullptr;
  const float*  v_bias = nullptr;
  __half*       k_cache = nullptr;   // [B][Hkv][Lmax][D]
  __half*       v_cache = nullptr;
  const float*  rope = nullptr;      // [Lmax][D/2][2]
  int32_t*      seq_len = nullptr;   // [B]
  int           bump_seq_len = 0;    // seq_len[b] += 1 after the call
  void*         o = nullptr;         // [B][Hq][D]
  int           o_dtype = LOGOS_F16; // LOGOS_F16 / LOGOS_BF16 / LOGOS_F32 / LOGOS_ACT_PLANES
  ActOut        o_act;               // destination planes when o_dtype == LOGOS_ACT_PLANES
  int64_t       b = 0, h_q = 0, h_kv = 0, d = 0, l_max = 0;
  float         scale = 1.f;
  int           device = 0;
  // Caller-provided scratch for the split-KV partials and the status word (both device
  // addresses).  Null = the library's own per-device scratch, allocated on first use and shared
  // by every stand-alone call on the device (a model passes its own: a captured step must not
  // point at memory another caller can outgrow).
  void*         ext_scratch = nullptr;
  int64_t       ext_scratch_bytes = 0;
  int*          ext_status = nullptr;
};
logos_status_t launch_gqa_decode_attn(const AttnArgs& a, cudaStream_t st);
// Bytes of split-KV scratch a call with these extents (b, h_q, h_kv, d, l_max, device) needs:
// what a caller that passes ext_scratch has to provide.
int64_t attn_scratch_bytes(const AttnArgs& a);
logos_status_t launch_kv_append_rope(__half* k_cache, __half* v_cache, const __half* k_new, const __half* v_new,
                                     const float* rope, int32_t* seq_len, int64_t b, int64_t h_kv, int64_t d,
                                     int64_t l_max, int device, cudaStream_t st);
void rope_table_host(float* out, int64_t l_max, int64_t d, double theta);

// ---- prompt processing (prefill.cu): RoPE + KV write + causal attention for a chunk of prompt
// positions [pos0, pos0 + chunk) of every sequence; rows are ordered (sequence, position).
struct PrefillAttnArgs {
  const float*  qkv = nullptr;       // [b * chunk][qkv_ld] f32: q | k | v heads of a row, un-rotated
  int64_t       qkv_ld = 0;
  const float*  qkv_bias = nullptr;  // f32 [(Hq + 2 Hkv) * D] or null
  const float*  rope = nullptr;      // [Lmax][D/2][2]
  __half*       q16 = nullptr;       // scratch [b * chunk][Hq * D]: the rotated queries
  __half*       k_cache = nullptr;   // [B][Hkv][Lmax][D]
  __half*       v_cache = nullptr;
  ActOut        o;                   // planes [b * chunk][Hq * D]
  int64_t       b = 0, h_q = 0, h_kv = 0, d = 0, l_max = 0, chunk = 0, pos0 = 0;
  float         scale = 1.f;
  int           device = 0;
};
logos_status_t launch_prefill_attn(const PrefillAttnArgs& a, cudaStream_t st);

// ---- norms and element-wise (elementwise.cu)
logos_status_t launch_rmsnorm_f32(const float* x, const float* g, float* y, int64_t rows, int64_t h, float eps,
                                  cudaStream_t st);
logos_status_t launch_swiglu_f32(const float* gate, const float* up, float* y, int64_t count, cudaStream_t st);
// h[row] = dequantised embedding row tokens[row]
// (q tile-major when `tiled`: see launch_q8_retile)
logos_status_t launch_embed(const int32_t* tokens, const int8_t* q, const float* s, float* h, int64_t rows,
                            int64_t hidden, int tiled, cudaStream_t st);
// h += sum over `parts` partial deltas (each [rows][hidden] f32, spaced
// part_stride floats, added in ascending order; parts may be 0), then
// xn = act16( h * rsqrt(mean(h^2)+eps) * g ).
logos_status_t launch_residual_rmsnorm(float* h, const float* delta, int parts, int64_t part_stride,
                                       const float* g, ActOut xn, int64_t rows, int64_t hidden, float eps,
                                       cudaStream_t st);
// The same operator for a tensor-parallel group whose ranks can address each other's memory:
// the all-reduce of the row-parallel GEMM's partial sums is folded in.  Rank r owns rows
// [r * rows / degree, (r + 1) * rows / degree): every rank pushes its partial sums of a row to
// the row's owner, the owner adds them (rank order) to its slice of the residual stream,
// normalises and pushes the resulting activation row to every rank, and every rank unpacks
// it into its own plane buffers.  The payload travels in 16-byte slots that carry the call's
// number (see elementwise.cu), so there is no barrier and no flag besides the data itself.
// Only the owner keeps a row of h up to date.
constexpr int TP_FLAG_WORDS = 64;  // u32 per rank: [16] call number (epoch), [17] CTA ticket
struct TpFusedArgs {
  int degree = 1, rank = 0;
  const float* partials = nullptr;  // this rank's [parts][rows][hidden] f32
  uint4* inbox_part[8] = {};        // each rank's inbox of partial rows: [source rank][rows / degree][hidden / 2] slots
  uint4* inbox_xn[8] = {};          // each rank's inbox of normalised rows: [rows][hidden / 2] slots
  __half* xn_hi = nullptr;          // this rank's planes [rows][hidden]
  __half* xn_lo = nullptr;          // null in the one-plane modes
  uint32_t* flags = nullptr;        // this rank's TP_FLAG_WORDS words, zero at creation
  int act_mode = LOGOS_F32;
};
logos_status_t launch_tp_residual_rmsnorm(float* h, const TpFusedArgs& t, int parts, int64_t part_stride, const float* g,
                                          int64_t rows, int64_t hidden, float eps, int device, cudaStream_t st);
// bf16 [count] -> fp16 plane (exact inside fp16's normal range, saturating outside)
logos_status_t launch_bf16_to_f16(const __nv_bfloat16* x, __half* y, int64_t count, cudaStream_t st);
// f32 [count] -> activation planes
logos_status_t launch_act_split(const float* x, ActOut o, int64_t count, cudaStream_t st);
// Sampling state of a model, in device memory so that a captured step follows changes to it.
struct SamplingParams {
  float inv_temperature;  // 1 / T
  int32_t enabled;        // 0: plain argmax
  uint64_t seed;
  int32_t top_k;          // > 0: only logits >= the k-th largest of their row are candidates
  int32_t reserved;
};
// tokens[row] = argmax(logits[row]) with the lowest index winning ties.  With sampling enabled
// (sampling_or_null and positions non-null) the compared value is
// logit * inv_temperature + gumbel(seed, row, positions[row] * vocab + index), over the logits
// that are >= the row's top_k-th largest when top_k is set.
// only_ending_or_null (ragged prompts): a row is written only if only_ending[row] - 1 == prompt_step.
logos_status_t launch_argmax(const float* logits, int32_t* tokens, int32_t* history_or_null,
                             const int32_t* step_counter_or_null, int64_t history_rows, int64_t rows, int64_t vocab,
                             const SamplingParams* sampling_or_null, const int32_t* positions_or_null,
                             const int32_t* only_ending_or_null, int prompt_step, cudaStream_t st);

}  // namespace logos
