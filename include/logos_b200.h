/*
 * logos_b200.h — C ABI of liblogos_b200.so: the Q8 LLM-decode hot path as
 * hand-written sm_100a CUDA kernels behind logicaffeine's native-operator /
 * "Universal ABI" conventions.
 *
 * The reference (logicaffeine v0.10.1) ships no GPU operators; what it does
 * fix, and what this header follows, is the shape of its C boundary:
 *   - every exported symbol is `logos_<name>`
 *       (crates/logicaffeine_compile/src/codegen/marshal.rs:143-146)
 *   - every fallible entry returns a LogosStatus with these exact codes
 *       (crates/logicaffeine_compile/src/codegen/ffi.rs:196-209, C mirror :1364-1375)
 *   - the message of the last failure on the calling thread is read with
 *     logos_last_error() / logos_get_last_error() and dropped with
 *     logos_clear_error()            (ffi.rs:214-264)
 *   - logos_abi_version() / logos_version()            (ffi.rs:275-285)
 *   - objects cross as opaque logos_handle_t ids held in a mutex-guarded
 *     registry; a stale or double-freed id is InvalidHandle, never UB
 *                                                       (ffi.rs:212,288-324,368-388)
 *   - out-parameters are null-checked before any work   (marshal.rs:355-358)
 *   - LOGOS `Int` is i64, so extents are int64_t
 *       (crates/logicaffeine_compile/src/codegen/types.rs:277)
 * A Rust host binds these with one `extern "C"` block inside a
 * `logicaffeine_system::llm` module shaped like `logicaffeine_system::ntt`
 * (crates/logicaffeine_system/src/ntt.rs:330-335) and reaches them from LOGOS
 * through rows in `map_native_function`
 * (crates/logicaffeine_compile/src/codegen/program.rs:1936-2003).
 *
 * Threading: error state is per thread; the registry is behind a mutex; one
 * model handle is driven by one host thread at a time.  `stream` arguments
 * take a cudaStream_t cast to void* (NULL = the legacy default stream).
 * There is no CPU fallback: without a CUDA device every compute entry
 * returns LOGOS_ERROR.
 */
#ifndef LOGOS_B200_H
#define LOGOS_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes: the Rust enum LogosStatus (ffi.rs:196-209) with the enumerator spelling of
 * the C header the reference generates (ffi.rs:1364-1375).  A translation unit that also
 * includes such a generated header defines LOGOS_B200_NO_RUNTIME_DECLS first: the typedefs and
 * the unprefixed runtime functions below then come from that header alone. */
#ifndef LOGOS_B200_NO_RUNTIME_DECLS
typedef enum {
  LOGOS_STATUS_OK = 0,
  LOGOS_STATUS_ERROR = 1,
  LOGOS_STATUS_REFINEMENT_VIOLATION = 2,
  LOGOS_STATUS_NULL_POINTER = 3,
  LOGOS_STATUS_OUT_OF_BOUNDS = 4,
  LOGOS_STATUS_DESERIALIZATION_FAILED = 5,
  LOGOS_STATUS_INVALID_HANDLE = 6,
  LOGOS_STATUS_CONTAINS_NULL_BYTE = 7,
  LOGOS_STATUS_THREAD_PANIC = 8,
  LOGOS_STATUS_MEMORY_EXHAUSTED = 9
} logos_status_t;
#endif
/* short spellings used inside this library */
#define LOGOS_OK LOGOS_STATUS_OK
#define LOGOS_ERROR LOGOS_STATUS_ERROR
#define LOGOS_REFINEMENT_VIOLATION LOGOS_STATUS_REFINEMENT_VIOLATION
#define LOGOS_NULL_POINTER LOGOS_STATUS_NULL_POINTER
#define LOGOS_OUT_OF_BOUNDS LOGOS_STATUS_OUT_OF_BOUNDS
#define LOGOS_DESERIALIZATION_FAILED LOGOS_STATUS_DESERIALIZATION_FAILED
#define LOGOS_INVALID_HANDLE LOGOS_STATUS_INVALID_HANDLE
#define LOGOS_CONTAINS_NULL_BYTE LOGOS_STATUS_CONTAINS_NULL_BYTE
#define LOGOS_THREAD_PANIC LOGOS_STATUS_THREAD_PANIC
#define LOGOS_MEMORY_EXHAUSTED LOGOS_STATUS_MEMORY_EXHAUSTED

/* ffi.rs:212 and :1376 — an id, not an address */
#ifndef LOGOS_B200_NO_RUNTIME_DECLS
typedef void* logos_handle_t;
#endif

#ifndef LOGOS_ABI_VERSION
#define LOGOS_ABI_VERSION 1 /* ffi.rs:275, :1382 */
#endif

#if defined(__GNUC__)
#define LOGOS_API __attribute__((visibility("default")))
#else
#define LOGOS_API
#endif

/* element types of device buffers named in operator signatures */
typedef enum {
  LOGOS_F32 = 0,
  LOGOS_F16 = 1,
  LOGOS_BF16 = 2,
  LOGOS_I8 = 3,
  LOGOS_I32 = 4
} logos_dtype_t;

/* ---- runtime ----
 * The library's own copies carry the logos_b200_ prefix.  Every LOGOS program with C exports
 * defines logos_last_error, logos_get_last_error, logos_clear_error, logos_free_string,
 * logos_version and logos_abi_version itself (#[no_mangle], ffi.rs:234-285), so inside such a
 * program the unprefixed names resolve to the PROGRAM's error store, not to this library's:
 * a host that is (or links) a LOGOS program reads this library's errors through the prefixed
 * names.  The unprefixed names (the reference preamble's, ffi.rs:1377-1384) are exported as
 * weak symbols for stand-alone C / Python hosts; the library never calls through them. */
LOGOS_API const char* logos_b200_last_error(void);     /* valid until the next failing call on this thread */
LOGOS_API const char* logos_b200_get_last_error(void); /* alias, as in the reference */
LOGOS_API void logos_b200_clear_error(void);
/* Releases a string the library handed out with ownership.  No entry point hands one out
 * today (error text stays owned by the library), so this only accepts NULL or such a future
 * string; it exists because the reference's C boundary has it (ffi.rs:268-273, :1380). */
LOGOS_API void logos_b200_free_string(char* str);
LOGOS_API uint32_t logos_b200_abi_version(void);
LOGOS_API const char* logos_b200_version(void);
#ifndef LOGOS_B200_NO_RUNTIME_DECLS
LOGOS_API const char* logos_last_error(void);
LOGOS_API const char* logos_get_last_error(void);
LOGOS_API void logos_clear_error(void);
LOGOS_API void logos_free_string(char* str);
LOGOS_API uint32_t logos_abi_version(void);
LOGOS_API const char* logos_version(void);
#endif
/* number of CUDA devices visible to the library; 0 when there is none */
LOGOS_API int32_t logos_device_count(void);

/* ---- device buffers (handles, ffi.rs:288-324; create/free pairs, ffi.rs:368-388) ---- */
LOGOS_API logos_status_t logos_dev_alloc(int64_t bytes, int32_t device, logos_handle_t* out);
LOGOS_API logos_status_t logos_dev_upload(logos_handle_t dst, int64_t dst_offset, const void* src_host, int64_t bytes);
LOGOS_API logos_status_t logos_dev_download(void* dst_host, logos_handle_t src, int64_t src_offset, int64_t bytes);
LOGOS_API logos_status_t logos_dev_memset(logos_handle_t dst, int32_t byte_value, int64_t bytes);
/* raw device address and size of a buffer, for hosts that share it with other CUDA code */
LOGOS_API logos_status_t logos_dev_ptr(logos_handle_t h, void** out_ptr, int64_t* out_bytes);
LOGOS_API logos_status_t logos_dev_sync(int32_t device);
/* free and total bytes of device memory as the driver reports them (cudaMemGetInfo) */
LOGOS_API logos_status_t logos_dev_mem_info(int32_t device, int64_t* free_out, int64_t* total_out);
LOGOS_API logos_status_t logos_dev_free(logos_handle_t h);
/* Every device-side wait in the library is bounded; a kernel that gives up
 * stores a non-zero code in a status word instead of hanging, and later kernels that
 * share the word do no work on top of it.  This reads and clears the device's words
 * (the per-device one, and the one logos_gqa_decode_attn_fixed_scratch keeps inside the
 * library image once that entry point has run on the device); 0 = nothing reported.
 * Call after a synchronisation.  The first call on a device allocates the 256-byte
 * per-device word; later calls allocate nothing. */
LOGOS_API logos_status_t logos_kernel_status(int32_t device, int32_t* out_code);

/* Kernel launches this process has made through the library, by kind:
 * out8 = {q8_gemv, q8_gemm tcgen05, q8_gemm SIMT, attention, attention merge,
 * norm/element-wise, synth/quantize, 0}.  Evidence that the CUDA path ran. */
LOGOS_API logos_status_t logos_launch_counts(int64_t* out8);

/* ---- seeded synthetic inputs, generated on the device ----
 * One counter-based generator (SplitMix64 finaliser over seed/stream/index, the
 * mixer the reference seeds with: crates/logicaffeine_runtime/src/seed.rs:15-28)
 * gives every element of every tensor from (seed, stream, index) alone, so a
 * shard can be produced on the rank that owns it.
 *   kind 0: int8 uniform in [-127,127]           (dst i8)
 *   kind 1: f32 uniform in [a,b)                 (dst f32)
 *   kind 2: normal, mean a, std b                (dst f32 / f16 / bf16 by `dtype`)
 *   kind 3: int32 uniform in [0,(int)b)          (dst i32)
 *   kind 4: standard Gumbel -ln(-ln u)           (dst f32; the noise of temperature sampling)
 * `first_index` offsets the counter (element i uses first_index+i). */
LOGOS_API logos_status_t logos_synth_fill(logos_handle_t dst, int64_t dst_offset_bytes, int32_t dtype, int32_t kind,
                                uint64_t seed, uint64_t stream, int64_t first_index, int64_t count,
                                float a, float b, void* stream_or_null);

/* Weight prep: per 32-element block along K, s = max|w|/127, q = rint(w/s).
 * w f32 [N][K] -> q i8 [N][K], s f32 [N][K/32]. */
LOGOS_API logos_status_t logos_q8_quantize(logos_handle_t w, logos_handle_t q, logos_handle_t s,
                                 int64_t n, int64_t k, void* stream_or_null);
/* Generate w ~ N(0,std) with the generator above (element (r,c) of the full
 * [rows_total][K] matrix uses index r*K+c) and quantise rows [row0,row0+n) in
 * one pass, never holding f32 weights in memory. */
LOGOS_API logos_status_t logos_q8_synth_weights(logos_handle_t q, logos_handle_t s, int64_t n, int64_t k,
                                      int64_t row0, uint64_t seed, uint64_t stream, float std,
                                      void* stream_or_null);

/* ---- single operators ---- */

/* y[n] = sum_kb s[n,kb] * sum_{k in kb} q[n,k] * x[k]   (f32 x, f32 accumulate, f32 y) */
LOGOS_API logos_status_t logos_q8_gemv(logos_handle_t q /*i8 [N][K]*/, logos_handle_t s /*f32 [N][K/32]*/,
                             logos_handle_t x /*f32 [K]*/, logos_handle_t y /*f32 [N]*/,
                             int64_t n, int64_t k, void* stream_or_null);

/* C[m,n] = bf16( sum_kb s[n,kb] * sum_k A[m,k] * q[n,k] )  (bf16 A, f32 accumulate)
 * epilogue 0: plain.  1: C = bf16(acc + aux[m,n]) with aux bf16 [M][N] (residual).
 * 2: rows of q interleave gate (even) and up (odd); C is [M][N/2] =
 *    bf16( silu(acc_gate) * acc_up ).
 * The stand-alone operators logos_q8_gemm, logos_q8_gemm_f32 and logos_gqa_decode_attn(_fused)
 * keep activation planes, split-K and split-KV partials in one library-owned scratch block per
 * device, grown on demand and shared by every caller on that device: calls that use it must
 * be ordered on the GPU (one stream, or events).  A model (logos_llm_*) owns its own. */
LOGOS_API logos_status_t logos_q8_gemm(logos_handle_t a /*bf16 [M][K]*/, logos_handle_t q, logos_handle_t s,
                             logos_handle_t c /*bf16*/, int64_t m, int64_t n, int64_t k,
                             int32_t epilogue, logos_handle_t aux_or_null, void* stream_or_null);

/* C[m,n] = sum_kb s[n,kb] * sum_k A[m,k] * q[n,k] with f32 A [M][K] and f32 C [M][N]:
 * the form the decode step uses between its kernels.  The activations are split into
 * two fp16 planes so the tensor-core product keeps f32-class accuracy. */
LOGOS_API logos_status_t logos_q8_gemm_f32(logos_handle_t a /*f32 [M][K]*/, logos_handle_t q, logos_handle_t s,
                                 logos_handle_t c /*f32 [M][N]*/, int64_t m, int64_t n, int64_t k,
                                 void* stream_or_null);

/* Same contract as logos_q8_gemm, always on the plain SIMT kernel (no tensor
 * cores, no split-K): the on-device cross-check the tests hold the tcgen05
 * kernel against, and the path for shapes the tcgen05 kernel does not take. */
LOGOS_API logos_status_t logos_q8_gemm_simt(logos_handle_t a, logos_handle_t q, logos_handle_t s,
                                  logos_handle_t c, int64_t m, int64_t n, int64_t k,
                                  int32_t epilogue, logos_handle_t aux_or_null, void* stream_or_null);

/* cos/sin table for rotary embedding, computed on the host in double and
 * rounded to f32: tab[pos][i] = {cos,sin}(pos * theta^(-2i/d)), i < d/2.
 * `out_host` holds l_max*(d/2)*2 floats. */
LOGOS_API logos_status_t logos_rope_table(float* out_host, int64_t l_max, int64_t d, double theta);

/* Rotate k_new by its position (= seq_len[b]) and write k,v rows at that index;
 * then seq_len[b] += 1.  f32 multiply and add rounded separately, fp16 store. */
LOGOS_API logos_status_t logos_kv_append_rope(logos_handle_t k_cache, logos_handle_t v_cache /*f16 [B][Hkv][Lmax][D]*/,
                                    logos_handle_t k_new, logos_handle_t v_new /*f16 [B][Hkv][D]*/,
                                    logos_handle_t rope_table /*f32 [Lmax][D/2][2]*/,
                                    logos_handle_t seq_len /*i32 [B]*/,
                                    int64_t b, int64_t h_kv, int64_t d, int64_t l_max, void* stream_or_null);

/* o = softmax(scale * q K^T) V over positions [0, seq_len[b]) for each of h_q
 * query heads (h_q/h_kv query heads share a KV head); q is used as given (already
 * rotated), f32 softmax.  q, o: f16 [B][Hq][D]. */
LOGOS_API logos_status_t logos_gqa_decode_attn(logos_handle_t q, logos_handle_t k_cache, logos_handle_t v_cache,
                                     logos_handle_t seq_len, logos_handle_t o,
                                     int64_t b, int64_t h_q, int64_t h_kv, int64_t d, int64_t l_max,
                                     float softmax_scale, void* stream_or_null);

/* No counterpart in the reference.  Same contract and same kernels as
 * logos_gqa_decode_attn, for hosts that must not trigger a device allocation when they
 * call an operator: a serving process that hands the whole GPU to its own KV-cache and
 * weight arena at start-up (a later cudaMalloc from inside the library would fail or
 * fragment that arena), or a decode loop with a latency budget that an allocation's
 * device-wide synchronisation would break.  The partial results of (sequence, KV head) pairs
 * that the kernel's persistent grid cuts go to a fixed 6 MiB array inside the library image
 * instead of library-allocated scratch, so every GPU that loads the library holds those 6 MiB
 * until the process exits.  What the kernel needs depends on the GPU, not on the shape: two
 * slots of 16 * (d + 2) floats and a 16-byte descriptor per CTA, two CTAs per SM (4.7 MiB on a
 * 148-SM B200 at d = 128);
 * a GPU with so many SMs that this exceeds the array is refused with LOGOS_OUT_OF_BOUNDS and
 * a message giving both sizes, and so is a call with more than 2048 sequences (the limit of
 * both attention entry points: a CTA keeps one tile count per sequence in shared memory).
 * The call itself makes no
 * cudaMalloc / cudaFree.  The first call on a device looks up the array's device address;
 * make that first call outside any stream capture.  All calls share the one array and one
 * status word.  Nothing is cleared between calls: the partials are always written before
 * they are read, and the status word is zero until a bounded wait inside the kernel gives up,
 * after which calls on this entry point leave `o` untouched until logos_kernel_status has
 * reported and cleared the code (call logos_kernel_status once at start-up if it must not
 * allocate later).  Two calls that overlap on the GPU race on the array: keep calls on this
 * entry point ordered, for instance on one stream. */
LOGOS_API logos_status_t logos_gqa_decode_attn_fixed_scratch(logos_handle_t q, logos_handle_t k_cache,
                                     logos_handle_t v_cache, logos_handle_t seq_len, logos_handle_t o,
                                     int64_t b, int64_t h_q, int64_t h_kv, int64_t d, int64_t l_max,
                                     float softmax_scale, void* stream_or_null);

/* The fused form the decode step uses: rotate q and k_new at position seq_len[b],
 * append k,v, attend over [0, seq_len[b]] including the new row, then
 * seq_len[b] += 1.  q_raw / k_new / v_new are un-rotated f16. */
LOGOS_API logos_status_t logos_gqa_decode_attn_fused(logos_handle_t q_raw, logos_handle_t k_new, logos_handle_t v_new,
                                           logos_handle_t k_cache, logos_handle_t v_cache,
                                           logos_handle_t rope_table, logos_handle_t seq_len, logos_handle_t o,
                                           int64_t b, int64_t h_q, int64_t h_kv, int64_t d, int64_t l_max,
                                           float softmax_scale, void* stream_or_null);

/* y = x * rsqrt(mean(x^2) + eps) * g, rows of length h.  x,y f32 [rows][h], g f32 [h]. */
LOGOS_API logos_status_t logos_rmsnorm(logos_handle_t x, logos_handle_t g, logos_handle_t y,
                             int64_t rows, int64_t h, float eps, void* stream_or_null);
/* y = silu(gate) * up, f32 element-wise over `count` elements. */
LOGOS_API logos_status_t logos_swiglu(logos_handle_t gate, logos_handle_t up, logos_handle_t y,
                            int64_t count, void* stream_or_null);

/* ---- model level: batched Qwen-architecture greedy decode ---- */
typedef struct {
  int64_t layers, hidden, h_q, h_kv, head_dim, ffn, vocab, l_max, batch;
  float   rms_eps, rope_theta;
  int32_t tied_embeddings;   /* 1: lm_head shares the embedding matrix */
  int32_t tp_degree, tp_rank; /* tensor-parallel group size and this rank */
  int32_t device;
  int32_t act_dtype;         /* precision of GEMM inputs: LOGOS_F32 (default: no rounding), LOGOS_F16 or LOGOS_BF16 */
  uint64_t seed;             /* random-init weights: N(0, init_std) -> Q8 blocks of 32 */
  float   init_std;
  int32_t qkv_bias;          /* 1: the q, k and v projections add a bias vector (Qwen2); N(0, init_std) at creation */
} logos_llm_config_t;

/* 128-byte NCCL unique id for the tensor-parallel group (rank 0 makes it, the
 * host carries it to the other ranks).  Not needed when tp_degree == 1. */
LOGOS_API logos_status_t logos_tp_unique_id(void* out_128_bytes);
LOGOS_API logos_status_t logos_llm_create(const logos_llm_config_t* cfg, const void* nccl_unique_id_or_null,
                                logos_handle_t* out);
/* The configuration the model was created with (a host that holds only the handle learns the
 * batch size, the vocabulary, ... from here). */
LOGOS_API logos_status_t logos_llm_get_config(logos_handle_t model, logos_llm_config_t* cfg_out);
/* Process t prompt tokens per sequence ([B][T] row-major, host) and fill the KV
 * cache; sequence lengths become t.  Starts from an empty cache.  The prompt runs in chunks of
 * positions, every sequence's chunk through a layer at once (rows = batch x chunk; the first call
 * allocates the chunk's workspace, about 4096 rows), with the decode step's arithmetic: weights
 * are streamed once per chunk, not once per token.  LOGOS_B200_PREFILL=loop in the environment
 * selects the token-by-token pass through the decode step instead (what
 * logos_llm_prefill_ragged always uses). */
LOGOS_API logos_status_t logos_llm_prefill(logos_handle_t model, const int32_t* tokens_host, int64_t t);
/* Prompts of different lengths: sequence b consumes tokens_host[b][0 .. lens_host[b]) of a
 * [B][t_max] array, 0 <= lens_host[b] <= t_max.  Afterwards its length is lens_host[b] and its
 * current token is the one chosen after its last prompt token (token 0 for an empty prompt);
 * decode steps then run all sequences in lock step, each at its own position.
 * lens_host[b] == -1 leaves sequence b as it is (cache, length, current token): a finished
 * sequence's slot takes a new prompt while the others of the running batch keep their state. */
LOGOS_API logos_status_t logos_llm_prefill_ragged(logos_handle_t model, const int32_t* tokens_host, int64_t t_max,
                                                  const int32_t* lens_host);
/* Fill the KV cache for positions [0,t) with seeded N(0,1) fp16 values instead
 * of running a prompt (measurement of decode at a given context length). */
LOGOS_API logos_status_t logos_llm_synth_kv(logos_handle_t model, int64_t t, uint64_t seed);
/* Set the tokens the next decode step consumes ([B], host). */
LOGOS_API logos_status_t logos_llm_set_tokens(logos_handle_t model, const int32_t* tokens_host);
/* One greedy step for every sequence: consumes the current tokens, appends to the
 * KV cache, writes argmax ids (lowest index wins ties) to next_tokens_host [B]
 * and keeps them as the next step's input. */
LOGOS_API logos_status_t logos_llm_decode_step(logos_handle_t model, int32_t* next_tokens_host);
/* `steps` greedy steps without a host round trip in between; tokens_host
 * receives [steps][B].  May be NULL to skip the read-back. */
LOGOS_API logos_status_t logos_llm_decode_steps(logos_handle_t model, int64_t steps, int32_t* tokens_host_or_null);
/* Parity-test accessors. K/V of one layer as stored on this rank:
 * f16 [B][Hkv/tp][Lmax][D]; logits of the last step f32 [B][vocab]; lengths [B]. */
LOGOS_API logos_status_t logos_llm_read_kv(logos_handle_t model, int64_t layer, void* k_host, void* v_host);
LOGOS_API logos_status_t logos_llm_read_logits(logos_handle_t model, float* logits_host);
LOGOS_API logos_status_t logos_llm_read_seq_len(logos_handle_t model, int32_t* seq_len_host);
/* Rewind every sequence to length t (t <= current length): decode can be re-run
 * from a prefilled state. */
LOGOS_API logos_status_t logos_llm_set_seq_len(logos_handle_t model, int64_t t);
/* Temperature sampling instead of greedy argmax: the next token of sequence b at position p
 * is argmax_i(logit_i / temperature + G(seed, b, p * vocab + i)) with G the generator's Gumbel
 * variate (logos_synth_fill kind 4), i.e. a draw from softmax(logits / temperature) that is a
 * pure function of (seed, sequence, position): the same on every rank of a tensor-parallel
 * group, under graph replay, and in the CPU oracle.  temperature 0 (the state after create)
 * is greedy.  top_k > 0 restricts the draw to the logits that reach the k-th largest of their
 * sequence (ties at that value included; 0 or >= vocab: no filter).  Takes effect from the
 * next step. */
LOGOS_API logos_status_t logos_llm_set_sampling(logos_handle_t model, float temperature, int64_t top_k, uint64_t seed);
/* Device-side time of the last logos_llm_decode_steps call, milliseconds
 * (CUDA events on the model's stream), and kernels launched per step. */
LOGOS_API logos_status_t logos_llm_last_timing(logos_handle_t model, double* ms_out, int64_t* launches_per_step_out);
/* Dependent-launch scope (no counterpart in the reference).  While it is open for the calling
 * thread (on != 0), the operators it launches may start before the previous kernel of their
 * stream has finished: they fetch their WEIGHT operands (q, s) right away and wait for the
 * previous kernel only before touching activations and outputs.  The caller promises that no
 * operator launched inside the scope writes weights that another one inside it reads.
 * prev_out (may be null) receives the previous setting. */
LOGOS_API logos_status_t logos_dependent_launch_scope(int32_t on, int32_t* prev_out);
/* How the ranks of the model's tensor-parallel group exchange the partial products of the
 * row-parallel GEMMs: 0 = no group (tp_degree 1), 1 = NCCL all-reduce, 2 = folded into the
 * residual + RMSNorm kernel over peer-mapped memory (one process per GPU, one node). */
LOGOS_API logos_status_t logos_llm_tp_exchange(logos_handle_t model, int32_t* mode_out);
/* ---- weight file: one flat file [256-byte header | tensors] that the library maps read-only
 * and copies from, the device-side counterpart of the reference's memory-mapped zone
 * (`Inside a zone called "D" mapped from "f.bin"`, crates/logicaffeine_language/src/ast/stmt.rs:405-418;
 * Zone::new_mapped, crates/logicaffeine_system/src/memory.rs:97-103).  Regions start on
 * 256-byte boundaries in this order: per layer attn_norm, q, k, v, (q_bias, k_bias, v_bias: f32
 * vectors, only with qkv_bias, header flag bit 0), o, mlp_norm, gate, up, down;
 * then final_norm, embed and (untied only) head.  A matrix is int8 [n][k] followed by f32
 * [n][k/32]; a norm gain is f32 [hidden].  Matrices are stored whole: a tensor-parallel rank
 * takes its rows (q, k, v, gate, up) or columns (o, down), so one file serves every group size.
 * A malformed or truncated file is LOGOS_DESERIALIZATION_FAILED, an unreadable one LOGOS_ERROR. */
typedef enum {
  LOGOS_W_ATTN_NORM = 0, LOGOS_W_Q = 1, LOGOS_W_K = 2, LOGOS_W_V = 3, LOGOS_W_O = 4, LOGOS_W_MLP_NORM = 5,
  LOGOS_W_GATE = 6, LOGOS_W_UP = 7, LOGOS_W_DOWN = 8, LOGOS_W_FINAL_NORM = 9, LOGOS_W_EMBED = 10, LOGOS_W_HEAD = 11,
  LOGOS_W_Q_BIAS = 12, LOGOS_W_K_BIAS = 13, LOGOS_W_V_BIAS = 14 /* only with cfg.qkv_bias; stored after v */
} logos_weight_tensor_t;
/* Layout queries (no GPU needed; only the architecture fields of cfg are read): size of the
 * file; place of one tensor (for a gain: q_off/q_bytes = the f32 vector, s_bytes = 0); the
 * header a writer puts at offset 0. */
LOGOS_API logos_status_t logos_llm_weights_file_bytes(const logos_llm_config_t* cfg, int64_t* bytes_out);
LOGOS_API logos_status_t logos_llm_weights_span(const logos_llm_config_t* cfg, int64_t layer, int32_t tensor,
                                                int64_t* q_off_out, int64_t* q_bytes_out, int64_t* s_off_out,
                                                int64_t* s_bytes_out);
LOGOS_API logos_status_t logos_llm_weights_header(const logos_llm_config_t* cfg, void* out_256_bytes);
/* Map a file, validate header and length, and (cfg_out non-null) report its architecture:
 * layers, hidden, h_q, h_kv, head_dim, ffn, vocab, tied_embeddings, qkv_bias; other fields are untouched. */
LOGOS_API logos_status_t logos_llm_weights_check(const char* path, logos_llm_config_t* cfg_out);
/* Host-side read of what rank tp_rank of a group of tp_degree holds of one tensor: int8
 * [rows][cols] into q_out and f32 [rows][cols/32] into s_out (a gain: f32 [hidden] into q_out,
 * s_out unused).  Capacities are in bytes.  The device loader copies the same rectangles. */
LOGOS_API logos_status_t logos_llm_weights_read_shard(const char* path, int32_t tp_degree, int32_t tp_rank, int64_t layer,
                                                      int32_t tensor, void* q_out, int64_t q_capacity, float* s_out,
                                                      int64_t s_capacity, int64_t* rows_out, int64_t* cols_out);
/* Replace the model's weights and norm gains with this rank's part of the file (architecture
 * must match the model's; the KV cache and sequence state are left alone).  The file is mapped
 * and streamed to the GPU through two pinned staging buffers. */
LOGOS_API logos_status_t logos_llm_load_weights(logos_handle_t model, const char* path);
/* Write the model's weights and gains as a weight file (tp_degree 1 only: a rank of a group
 * holds no whole matrix). */
LOGOS_API logos_status_t logos_llm_save_weights(logos_handle_t model, const char* path);
/* One greedy step with CUDA events around every launch group; ms_by_class_out
 * receives 4 doubles: Q8 GEMMs, attention (+merge), norms/element-wise, and
 * tensor-parallel exchange.  Advances the model like logos_llm_decode_step. */
LOGOS_API logos_status_t logos_llm_profile_step(logos_handle_t model, double* ms_by_class_out);
LOGOS_API logos_status_t logos_llm_free(logos_handle_t model);

#ifdef __cplusplus
}
#endif
#endif /* LOGOS_B200_H */
