/*
 * logos_oracle.c — CPU restatement of the Q8 LLM-decode arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is
 * compared against (tests/, the smoke check, and the CPU-baseline legs of the
 * benchmark).  Nothing in the shipped library includes, links or calls it.
 *
 * PARITY UNPINNED.  logicaffeine v0.10.1 contains no implementation of this
 * path (no Q8, attention, KV-cache or decode code and no golden vectors for
 * them; its only dense kernel is the i64 triple loop of
 * benchmarks/programs/matrix_mult/main.lg:20-29).  The normative text is the
 * arithmetic of the five benchmark configurations: int8 weights in row-major
 * blocks of 32 along K with one f32 scale per block, f32 accumulation, fp16 KV
 * cache, rotary embedding with theta 1e6, softmax scale 1/sqrt(d), RMSNorm
 * eps 1e-6, SwiGLU, greedy argmax.  What is borrowed from the reference is its
 * numeric discipline: float reductions are never re-associated
 * (crates/logicaffeine_forge/src/vectorize.rs:1-16) and a multiply followed by
 * an add rounds twice (crates/logicaffeine_jit/src/lib.rs:5225-5231).  So this
 * file must be built with -ffp-contract=off, every sum below runs in ascending
 * index order, and the order is part of the definition.
 *
 * Independent cross-check: tests/golden/make_golden.py restates the same
 * operators, the sampler and the whole decode model in numpy (float64 sums,
 * explicit float32 steps where bits are defined) and commits small
 * input/output vectors; tests/test_oracle_golden.py holds this file to them.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

enum { ORC_F32 = 0, ORC_F16 = 1, ORC_BF16 = 2, ORC_I8 = 3, ORC_I32 = 4 };

/* ------------------------------------------------------------ 16-bit floats */
static inline float h2f(uint16_t h) {
  _Float16 v;
  memcpy(&v, &h, 2);
  return (float)v;
}
static inline uint16_t f2h(float f) {
  _Float16 v = (_Float16)f; /* round to nearest even */
  uint16_t h;
  memcpy(&h, &v, 2);
  return h;
}
static inline float bf2f(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f2bf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u); /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u); /* round to nearest even */
  return (uint16_t)(u >> 16);
}
static inline float round_act(float v, int act_dtype) {
  if (act_dtype == ORC_F16) return h2f(f2h(v));
  if (act_dtype == ORC_BF16) return bf2f(f2bf(v));
  return v;
}

ORC_API int orc_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
ORC_API float orc_h2f(uint16_t h) { return h2f(h); }
ORC_API uint16_t orc_f2h(float f) { return f2h(f); }
ORC_API float orc_bf2f(uint16_t h) { return bf2f(h); }
ORC_API uint16_t orc_f2bf(float f) { return f2bf(f); }

/* ------------------------------------------------------------ generator
 * SplitMix64 finaliser (the mixer of crates/logicaffeine_runtime/src/seed.rs:15-28)
 * over (seed, stream, index).  Normals: Box-Muller on 24-bit uniforms with
 * polynomial log / sin / cos in f32, so that no libm call decides a bit. */
static inline uint64_t mix64(uint64_t z) {
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z;
}
static inline uint64_t ctr_hash(uint64_t seed, uint64_t stream, uint64_t idx) {
  const uint64_t G = 0x9E3779B97F4A7C15ull;
  return mix64(mix64(seed + G * (stream + 1)) + G * (idx + 1));
}
static inline int gen_i8(uint64_t seed, uint64_t stream, uint64_t idx) {
  uint32_t r = (uint32_t)(ctr_hash(seed, stream, idx) >> 32);
  return (int)(r % 255u) - 127;
}
static inline float gen_uniform(uint64_t seed, uint64_t stream, uint64_t idx, float a, float b) {
  uint32_t r = (uint32_t)(ctr_hash(seed, stream, idx) >> 40);
  float u = (float)r * 5.9604644775390625e-08f;
  float w = b - a;
  float t = u * w;
  return a + t;
}
static inline float gen_normal(uint64_t seed, uint64_t stream, uint64_t idx) {
  uint64_t h = ctr_hash(seed, stream, idx >> 1);
  uint32_t k1 = (uint32_t)(h >> 40);
  uint32_t k2 = (uint32_t)(h >> 16) & 0xFFFFFFu;
  uint32_t v = k1 + 1u;
  int e = 31 - __builtin_clz(v);
  uint32_t pw = (uint32_t)(127 - e) << 23;
  float scale;
  memcpy(&scale, &pw, 4);
  float m = (float)v * scale;
  if (m > 1.41421354f) {
    m = m * 0.5f;
    e += 1;
  }
  float num = m - 1.0f, den = m + 1.0f;
  float t = num / den;
  float t2 = t * t;
  float p = 0.111111111f;
  p = p * t2; p = p + 0.142857143f;
  p = p * t2; p = p + 0.2f;
  p = p * t2; p = p + 0.333333343f;
  p = p * t2; p = p + 1.0f;
  float two_t = 2.0f * t;
  float ln_m = two_t * p;
  float ek = (float)(e - 24) * 0.693147182f;
  float ln_u = ln_m + ek;
  float arg = -2.0f * ln_u;
  float r = sqrtf(arg);
  uint32_t quad = k2 >> 22;
  float f = (float)(k2 & 0x3FFFFFu) * 2.384185791015625e-07f;
  float x = f * 1.57079637f;
  float x2 = x * x;
  float c = 2.08767570e-09f;
  c = c * x2; c = c + -2.75573192e-07f;
  c = c * x2; c = c + 2.48015873e-05f;
  c = c * x2; c = c + -1.38888889e-03f;
  c = c * x2; c = c + 4.16666667e-02f;
  c = c * x2; c = c + -0.5f;
  c = c * x2; c = c + 1.0f;
  float s = 1.60590438e-10f;
  s = s * x2; s = s + -2.50521084e-08f;
  s = s * x2; s = s + 2.75573192e-06f;
  s = s * x2; s = s + -1.98412698e-04f;
  s = s * x2; s = s + 8.33333333e-03f;
  s = s * x2; s = s + -1.66666667e-01f;
  s = s * x2; s = s + 1.0f;
  s = s * x;
  float cq, sq;
  switch (quad) {
    case 0: cq = c; sq = s; break;
    case 1: cq = -s; sq = c; break;
    case 2: cq = -c; sq = -s; break;
    default: cq = s; sq = -c; break;
  }
  return r * ((idx & 1ull) ? sq : cq);
}

/* ln of a positive normal float (exponent by bits, atanh series on the mantissa) and the
 * standard Gumbel variate -ln(-ln u), u = (2k+1) * 2^-24 for a 23-bit k. */
static inline float ln_pos(float x) {
  uint32_t bits;
  memcpy(&bits, &x, 4);
  int e = (int)(bits >> 23) - 127;
  uint32_t mb = (bits & 0x007FFFFFu) | 0x3F800000u;
  float m;
  memcpy(&m, &mb, 4);
  if (m > 1.41421354f) {
    m = m * 0.5f;
    e += 1;
  }
  float num = m - 1.0f, den = m + 1.0f;
  float t = num / den;
  float t2 = t * t;
  float p = 0.111111111f;
  p = p * t2; p = p + 0.142857143f;
  p = p * t2; p = p + 0.2f;
  p = p * t2; p = p + 0.333333343f;
  p = p * t2; p = p + 1.0f;
  float two_t = 2.0f * t;
  float ln_m = two_t * p;
  float ek = (float)e * 0.693147182f;
  return ln_m + ek;
}
static inline float gen_gumbel(uint64_t seed, uint64_t stream, uint64_t idx) {
  uint32_t k = (uint32_t)(ctr_hash(seed, stream, idx) >> 41);
  float u = (float)(2u * k + 1u) * 5.9604644775390625e-08f;
  float l = -ln_pos(u);
  return -ln_pos(l);
}

ORC_API void orc_synth_fill(void* dst, int dtype, int kind, uint64_t seed, uint64_t stream,
                            int64_t first, int64_t count, float a, float b) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; ++i) {
    uint64_t idx = (uint64_t)(first + i);
    if (kind == 0) {
      ((int8_t*)dst)[i] = (int8_t)gen_i8(seed, stream, idx);
    } else if (kind == 1) {
      ((float*)dst)[i] = gen_uniform(seed, stream, idx, a, b);
    } else if (kind == 2) {
      float z = gen_normal(seed, stream, idx);
      float sz = b * z;
      float v = a + sz;
      if (dtype == ORC_F32) ((float*)dst)[i] = v;
      else if (dtype == ORC_F16) ((uint16_t*)dst)[i] = f2h(v);
      else ((uint16_t*)dst)[i] = f2bf(v);
    } else if (kind == 4) {
      ((float*)dst)[i] = gen_gumbel(seed, stream, idx);
    } else {
      uint32_t r = (uint32_t)(ctr_hash(seed, stream, idx) >> 32);
      ((int32_t*)dst)[i] = (int32_t)(r % (uint32_t)b);
    }
  }
}

/* ------------------------------------------------------------ Q8 blocks
 * s = max|w| / 127, q = round-half-even(w / s); an all-zero block has s = 0. */
static inline void quantize_block(const float* w, int8_t* q, float* s) {
  float amax = 0.0f;
  for (int i = 0; i < 32; ++i) {
    float a = fabsf(w[i]);
    if (a > amax) amax = a;
  }
  float sc = amax / 127.0f;
  *s = sc;
  for (int i = 0; i < 32; ++i) {
    int v = 0;
    if (amax > 0.0f) {
      float r = w[i] / sc;
      v = (int)lrintf(r);
      if (v > 127) v = 127;
      if (v < -127) v = -127;
    }
    q[i] = (int8_t)v;
  }
}

ORC_API void orc_q8_quantize(const float* w, int8_t* q, float* s, int64_t n, int64_t k) {
  int64_t kb = k / 32;
#pragma omp parallel for schedule(static)
  for (int64_t blk = 0; blk < n * kb; ++blk) quantize_block(w + blk * 32, q + blk * 32, s + blk);
}

/* Rows [row0,row0+n) x columns [col0,col0+k) of the logical [.][k_total] matrix
 * whose element (r,c) is std * normal(seed, stream, r*k_total + c). */
ORC_API void orc_q8_synth_weights(int8_t* q, float* s, int64_t n, int64_t k, int64_t row0, int64_t col0,
                                  int64_t k_total, uint64_t seed, uint64_t stream, float std) {
  int64_t kb = k / 32;
#pragma omp parallel for schedule(static)
  for (int64_t blk = 0; blk < n * kb; ++blk) {
    int64_t r = blk / kb, b = blk - r * kb;
    float w[32];
    for (int i = 0; i < 32; ++i) {
      uint64_t idx = (uint64_t)((row0 + r) * k_total + col0 + b * 32 + i);
      w[i] = std * gen_normal(seed, stream, idx);
    }
    quantize_block(w, q + r * k + b * 32, s + blk);
  }
}

/* ------------------------------------------------------------ Q8 GEMV (config 0)
 * y[n] = sum_kb s[n,kb] * (sum_{k in kb} q[n,k] * x[k]); k ascending inside a
 * block, blocks ascending, every product and sum rounded to f32. */
ORC_API void orc_q8_gemv(const int8_t* q, const float* s, const float* x, float* y, int64_t n, int64_t k) {
  int64_t kb = k / 32;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r) {
    const int8_t* qr = q + r * k;
    float acc = 0.0f;
    for (int64_t b = 0; b < kb; ++b) {
      float p = 0.0f;
      for (int i = 0; i < 32; ++i) {
        float t = (float)qr[b * 32 + i] * x[b * 32 + i];
        p = p + t;
      }
      float sp = s[r * kb + b] * p;
      acc = acc + sp;
    }
    y[r] = acc;
  }
}

/* ------------------------------------------------------------ Q8 GEMM core
 * acc[m,n] = sum_kb s[n,kb] * (sum_k a[m,k] * q[n,k]), same order as the GEMV.
 * `at` is the activation matrix transposed to [K][M] so the m loop vectorises
 * without touching the k order. */
static int g_perturb = 0;
/* Sensitivity probe for the tests: 1 sums the K-blocks of every GEMM in
 * descending order, an f32-level re-association of the same arithmetic.  It
 * measures how far greedy token ids move under rounding-order noise of the
 * size a GPU kernel introduces.  0 (the definition) is the default. */
ORC_API void orc_set_perturb(int mode) { g_perturb = mode; }

static void gemm_core(const float* at, const int8_t* q, const float* s, float* c, int64_t ldc,
                      int64_t m, int64_t n, int64_t k) {
  int64_t kb = k / 32;
  const int rev = g_perturb;
#pragma omp parallel
  {
    float* acc = (float*)malloc(sizeof(float) * (size_t)m * 2);
    float* p = acc + m;
#pragma omp for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
      const int8_t* qr = q + r * k;
      for (int64_t j = 0; j < m; ++j) acc[j] = 0.0f;
      for (int64_t bb = 0; bb < kb; ++bb) {
        int64_t b = rev ? kb - 1 - bb : bb;
        for (int64_t j = 0; j < m; ++j) p[j] = 0.0f;
        for (int i = 0; i < 32; ++i) {
          float qv = (float)qr[b * 32 + i];
          const float* ar = at + (b * 32 + i) * m;
          for (int64_t j = 0; j < m; ++j) {
            float t = ar[j] * qv;
            p[j] = p[j] + t;
          }
        }
        float sc = s[r * kb + b];
        for (int64_t j = 0; j < m; ++j) {
          float sp = sc * p[j];
          acc[j] = acc[j] + sp;
        }
      }
      for (int64_t j = 0; j < m; ++j) c[j * ldc + r] = acc[j];
    }
    free(acc);
  }
}

static float* transpose_act(const void* a, int dtype, int64_t m, int64_t k) {
  float* at = (float*)malloc(sizeof(float) * (size_t)m * (size_t)k);
  for (int64_t j = 0; j < m; ++j)
    for (int64_t i = 0; i < k; ++i) {
      float v;
      if (dtype == ORC_F32) v = ((const float*)a)[j * k + i];
      else if (dtype == ORC_F16) v = h2f(((const uint16_t*)a)[j * k + i]);
      else v = bf2f(((const uint16_t*)a)[j * k + i]);
      at[i * m + j] = v;
    }
  return at;
}

static inline float silu(float g) { return g / (1.0f + expf(-g)); }

/* f32-output GEMM on activations of any storage type. */
ORC_API void orc_q8_gemm_f32(const void* a, int a_dtype, const int8_t* q, const float* s, float* c,
                             int64_t m, int64_t n, int64_t k) {
  float* at = transpose_act(a, a_dtype, m, k);
  gemm_core(at, q, s, c, n, m, n, k);
  free(at);
}

/* Config 1: bf16 A, bf16 C.  epilogue 0 plain; 1 adds aux (bf16 [M][N]) before
 * the final rounding; 2 treats rows (2j, 2j+1) of q as (gate_j, up_j) and
 * writes bf16(silu(gate) * up) to C [M][N/2]. */
ORC_API void orc_q8_gemm(const uint16_t* a, const int8_t* q, const float* s, uint16_t* c,
                         int64_t m, int64_t n, int64_t k, int epilogue, const uint16_t* aux) {
  float* tmp = (float*)malloc(sizeof(float) * (size_t)m * (size_t)n);
  orc_q8_gemm_f32(a, ORC_BF16, q, s, tmp, m, n, k);
  if (epilogue == 2) {
    int64_t h = n / 2;
    for (int64_t j = 0; j < m; ++j)
      for (int64_t r = 0; r < h; ++r) {
        float g = tmp[j * n + 2 * r], u = tmp[j * n + 2 * r + 1];
        float sg = silu(g);
        c[j * h + r] = f2bf(sg * u);
      }
  } else {
    for (int64_t i = 0; i < m * n; ++i) {
      float v = tmp[i];
      if (epilogue == 1) v = v + bf2f(aux[i]);
      c[i] = f2bf(v);
    }
  }
  free(tmp);
}

/* ------------------------------------------------------------ rotary embedding
 * tab[pos][i] = {cos,sin}(pos * theta^(-2i/d)) evaluated in double, rounded to
 * f32.  Pairing is half-split: element i rotates with element i + d/2. */
ORC_API void orc_rope_table(float* out, int64_t l_max, int64_t d, double theta) {
  int64_t half = d / 2;
  for (int64_t pos = 0; pos < l_max; ++pos)
    for (int64_t i = 0; i < half; ++i) {
      double inv = pow(theta, -2.0 * (double)i / (double)d);
      double ang = (double)pos * inv;
      out[(pos * half + i) * 2 + 0] = (float)cos(ang);
      out[(pos * half + i) * 2 + 1] = (float)sin(ang);
    }
}

/* out[i] = x[i]*c - x[i+h]*s ; out[i+h] = x[i+h]*c + x[i]*s ; each product and
 * each sum rounded to f32, result rounded to fp16. */
static inline void rope_row_f16out(const float* x, const float* tab_pos, int64_t d, uint16_t* out) {
  int64_t half = d / 2;
  for (int64_t i = 0; i < half; ++i) {
    float c = tab_pos[2 * i], s = tab_pos[2 * i + 1];
    float x1 = x[i], x2 = x[i + half];
    float a1 = x1 * c, b1 = x2 * s;
    float a2 = x2 * c, b2 = x1 * s;
    out[i] = f2h(a1 - b1);
    out[i + half] = f2h(a2 + b2);
  }
}

ORC_API void orc_kv_append_rope(uint16_t* k_cache, uint16_t* v_cache, const uint16_t* k_new,
                                const uint16_t* v_new, const float* tab, int32_t* seq_len,
                                int64_t b, int64_t h_kv, int64_t d, int64_t l_max) {
  float tmp[1024];
  for (int64_t i = 0; i < b; ++i) {
    int64_t pos = seq_len[i];
    if (pos < 0 || pos >= l_max) continue; /* full sequence: nothing is written */
    for (int64_t h = 0; h < h_kv; ++h) {
      const uint16_t* kn = k_new + (i * h_kv + h) * d;
      const uint16_t* vn = v_new + (i * h_kv + h) * d;
      uint16_t* kd = k_cache + ((i * h_kv + h) * l_max + pos) * d;
      uint16_t* vd = v_cache + ((i * h_kv + h) * l_max + pos) * d;
      for (int64_t e = 0; e < d; ++e) tmp[e] = h2f(kn[e]);
      rope_row_f16out(tmp, tab + pos * (d / 2) * 2, d, kd);
      memcpy(vd, vn, sizeof(uint16_t) * (size_t)d);
    }
    seq_len[i] = (int32_t)(pos + 1);
  }
}

/* One (sequence, query head): scores in f32 with d ascending, scale applied to
 * the finished dot product, p = expf(s - max), sums over positions ascending,
 * o = (sum p*v) / (sum p). */
static void attn_one(const uint16_t* qh, const uint16_t* kc, const uint16_t* vc, int64_t len, int64_t d,
                     float scale, float* sc_buf, float* o) {
  float mx = -INFINITY;
  for (int64_t j = 0; j < len; ++j) {
    float acc = 0.0f;
    for (int64_t e = 0; e < d; ++e) {
      float t = h2f(qh[e]) * h2f(kc[j * d + e]);
      acc = acc + t;
    }
    acc = acc * scale;
    sc_buf[j] = acc;
    if (acc > mx) mx = acc;
  }
  float l = 0.0f;
  for (int64_t e = 0; e < d; ++e) o[e] = 0.0f;
  for (int64_t j = 0; j < len; ++j) {
    float p = expf(sc_buf[j] - mx);
    l = l + p;
    for (int64_t e = 0; e < d; ++e) {
      float t = p * h2f(vc[j * d + e]);
      o[e] = o[e] + t;
    }
  }
  for (int64_t e = 0; e < d; ++e) o[e] = (len > 0) ? o[e] / l : 0.0f;
}

/* q, o: [B][Hq][D]; o written as f32 into o_f32 (when given) and/or rounded to
 * fp16 into o_f16 (when given). */
static void attn_all(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, const int32_t* seq_len,
                     float* o_f32, uint16_t* o_f16, int64_t b, int64_t h_q, int64_t h_kv, int64_t d,
                     int64_t l_max, float scale) {
  int64_t group = h_q / h_kv;
#pragma omp parallel
  {
    float* sc_buf = (float*)malloc(sizeof(float) * (size_t)(l_max + 1));
    float* o = (float*)malloc(sizeof(float) * (size_t)d);
#pragma omp for schedule(dynamic, 1) collapse(2)
    for (int64_t i = 0; i < b; ++i)
      for (int64_t h = 0; h < h_q; ++h) {
        int64_t kvh = h / group;
        int64_t len = seq_len[i];
        if (len > l_max) len = l_max;
        attn_one(q + (i * h_q + h) * d, k_cache + (i * h_kv + kvh) * l_max * d,
                 v_cache + (i * h_kv + kvh) * l_max * d, len, d, scale, sc_buf, o);
        for (int64_t e = 0; e < d; ++e) {
          if (o_f32) o_f32[(i * h_q + h) * d + e] = o[e];
          if (o_f16) o_f16[(i * h_q + h) * d + e] = f2h(o[e]);
        }
      }
    free(sc_buf);
    free(o);
  }
}

ORC_API void orc_gqa_decode_attn(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache,
                                 const int32_t* seq_len, uint16_t* o, int64_t b, int64_t h_q, int64_t h_kv,
                                 int64_t d, int64_t l_max, float scale) {
  attn_all(q, k_cache, v_cache, seq_len, NULL, o, b, h_q, h_kv, d, l_max, scale);
}

/* Fused form: rotate q and k_new at position seq_len[b], append, attend over
 * [0, seq_len[b]] (new row included), then bump the lengths. */
ORC_API void orc_gqa_decode_attn_fused(const uint16_t* q_raw, const uint16_t* k_new, const uint16_t* v_new,
                                       uint16_t* k_cache, uint16_t* v_cache, const float* tab, int32_t* seq_len,
                                       uint16_t* o, int64_t b, int64_t h_q, int64_t h_kv, int64_t d,
                                       int64_t l_max, float scale) {
  uint16_t* q_rot = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)(b * h_q * d));
  float tmp[1024];
  for (int64_t i = 0; i < b; ++i) {
    int64_t pos = seq_len[i];
    if (pos >= l_max) pos = l_max - 1;
    for (int64_t h = 0; h < h_q; ++h) {
      for (int64_t e = 0; e < d; ++e) tmp[e] = h2f(q_raw[(i * h_q + h) * d + e]);
      rope_row_f16out(tmp, tab + pos * (d / 2) * 2, d, q_rot + (i * h_q + h) * d);
    }
  }
  orc_kv_append_rope(k_cache, v_cache, k_new, v_new, tab, seq_len, b, h_kv, d, l_max);
  attn_all(q_rot, k_cache, v_cache, seq_len, NULL, o, b, h_q, h_kv, d, l_max, scale);
  free(q_rot);
}

/* ------------------------------------------------------------ norms, SwiGLU */
ORC_API void orc_rmsnorm(const float* x, const float* g, float* y, int64_t rows, int64_t h, float eps) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * h;
    float ss = 0.0f;
    for (int64_t i = 0; i < h; ++i) {
      float t = xr[i] * xr[i];
      ss = ss + t;
    }
    float mean = ss / (float)h;
    float den = sqrtf(mean + eps);
    float inv = 1.0f / den;
    for (int64_t i = 0; i < h; ++i) {
      float t = xr[i] * inv;
      y[r * h + i] = t * g[i];
    }
  }
}

ORC_API void orc_swiglu(const float* gate, const float* up, float* y, int64_t count) {
  for (int64_t i = 0; i < count; ++i) {
    float sg = silu(gate[i]);
    y[i] = sg * up[i];
  }
}

/* ------------------------------------------------------------ model
 * Batched Qwen-architecture greedy decode: f32 residual stream, GEMM inputs
 * rounded to the 16-bit activation type, fp16 KV cache, f32 logits, argmax
 * with the lowest index winning ties.  Weight streams: layer*16 + {0:q 1:k 2:v
 * 3:o 4:gate 5:up 6:down}; embedding (1<<20); lm_head (1<<20)+1.  Norm gains
 * [2*layers+1][hidden] (attn_norm and mlp_norm per layer, final_norm) are 1 until
 * orc_llm_set_tensor replaces them. */
typedef struct {
  int64_t layers, hidden, h_q, h_kv, head_dim, ffn, vocab, l_max, batch;
  float rms_eps, rope_theta;
  int32_t tied_embeddings, tp_degree, tp_rank, device, act_dtype;
  uint64_t seed;
  float init_std;
  int32_t qkv_bias; /* 1: the q, k and v projections add a bias vector (Qwen2) */
} orc_llm_config_t;

typedef struct {
  int8_t* q;
  float* s;
  int64_t n, k;
} q8mat;

typedef struct {
  orc_llm_config_t cfg;
  q8mat *wq, *wk, *wv, *wo, *wg, *wu, *wd;
  float **bq, **bk, **bv; /* per layer, only with cfg.qkv_bias: f32 [h_q*D], [h_kv*D], [h_kv*D] */
  q8mat embed, head;
  uint16_t **kc, **vc; /* per layer [B][Hkv][Lmax][D] */
  float* rope;
  float* gains;
  int32_t* seq_len;
  int32_t* tokens;
  float* logits;
  float* h; /* residual stream [B][H] */
  int sampling; /* 0: greedy argmax */
  int64_t top_k; /* > 0: only logits >= the k-th largest of the row are candidates */
  float inv_temperature;
  uint64_t sample_seed;
} orc_llm;

static q8mat make_mat(int64_t n, int64_t k, uint64_t seed, uint64_t stream, float std) {
  q8mat m;
  m.n = n;
  m.k = k;
  m.q = (int8_t*)malloc((size_t)(n * k));
  m.s = (float*)malloc(sizeof(float) * (size_t)(n * (k / 32)));
  orc_q8_synth_weights(m.q, m.s, n, k, 0, 0, k, seed, stream, std);
  return m;
}
static void free_mat(q8mat* m) {
  free(m->q);
  free(m->s);
}

ORC_API void* orc_llm_create(const orc_llm_config_t* cfg) {
  orc_llm* M = (orc_llm*)calloc(1, sizeof(orc_llm));
  M->cfg = *cfg;
  int64_t L = cfg->layers, H = cfg->hidden, D = cfg->head_dim, F = cfg->ffn;
  int64_t nq = cfg->h_q * D, nkv = cfg->h_kv * D;
  M->wq = calloc((size_t)L, sizeof(q8mat)); M->wk = calloc((size_t)L, sizeof(q8mat));
  M->wv = calloc((size_t)L, sizeof(q8mat)); M->wo = calloc((size_t)L, sizeof(q8mat));
  M->wg = calloc((size_t)L, sizeof(q8mat)); M->wu = calloc((size_t)L, sizeof(q8mat));
  M->wd = calloc((size_t)L, sizeof(q8mat));
  M->bq = calloc((size_t)L, sizeof(float*)); M->bk = calloc((size_t)L, sizeof(float*));
  M->bv = calloc((size_t)L, sizeof(float*));
  M->kc = calloc((size_t)L, sizeof(uint16_t*));
  M->vc = calloc((size_t)L, sizeof(uint16_t*));
  for (int64_t l = 0; l < L; ++l) {
    uint64_t st = (uint64_t)l * 16;
    M->wq[l] = make_mat(nq, H, cfg->seed, st + 0, cfg->init_std);
    M->wk[l] = make_mat(nkv, H, cfg->seed, st + 1, cfg->init_std);
    M->wv[l] = make_mat(nkv, H, cfg->seed, st + 2, cfg->init_std);
    M->wo[l] = make_mat(H, nq, cfg->seed, st + 3, cfg->init_std);
    M->wg[l] = make_mat(F, H, cfg->seed, st + 4, cfg->init_std);
    M->wu[l] = make_mat(F, H, cfg->seed, st + 5, cfg->init_std);
    M->wd[l] = make_mat(H, F, cfg->seed, st + 6, cfg->init_std);
    if (cfg->qkv_bias) { /* streams 7, 8, 9 of the layer: N(0, init_std) */
      M->bq[l] = (float*)malloc(sizeof(float) * (size_t)nq);
      M->bk[l] = (float*)malloc(sizeof(float) * (size_t)nkv);
      M->bv[l] = (float*)malloc(sizeof(float) * (size_t)nkv);
      orc_synth_fill(M->bq[l], ORC_F32, 2, cfg->seed, st + 7, 0, nq, 0.0f, cfg->init_std);
      orc_synth_fill(M->bk[l], ORC_F32, 2, cfg->seed, st + 8, 0, nkv, 0.0f, cfg->init_std);
      orc_synth_fill(M->bv[l], ORC_F32, 2, cfg->seed, st + 9, 0, nkv, 0.0f, cfg->init_std);
    }
    size_t kv = (size_t)(cfg->batch * cfg->h_kv * cfg->l_max * D);
    M->kc[l] = (uint16_t*)calloc(kv, 2);
    M->vc[l] = (uint16_t*)calloc(kv, 2);
  }
  M->embed = make_mat(cfg->vocab, H, cfg->seed, (uint64_t)1 << 20, cfg->init_std);
  if (!cfg->tied_embeddings) M->head = make_mat(cfg->vocab, H, cfg->seed, ((uint64_t)1 << 20) + 1, cfg->init_std);
  M->rope = (float*)malloc(sizeof(float) * (size_t)(cfg->l_max * D));
  orc_rope_table(M->rope, cfg->l_max, D, (double)cfg->rope_theta);
  M->gains = (float*)malloc(sizeof(float) * (size_t)((2 * L + 1) * H));
  for (int64_t i = 0; i < (2 * L + 1) * H; ++i) M->gains[i] = 1.0f;
  M->seq_len = (int32_t*)calloc((size_t)cfg->batch, 4);
  M->tokens = (int32_t*)calloc((size_t)cfg->batch, 4);
  M->logits = (float*)calloc((size_t)(cfg->batch * cfg->vocab), 4);
  M->h = (float*)calloc((size_t)(cfg->batch * H), 4);
  return M;
}

ORC_API void orc_llm_free(void* model) {
  orc_llm* M = (orc_llm*)model;
  for (int64_t l = 0; l < M->cfg.layers; ++l) {
    free_mat(&M->wq[l]); free_mat(&M->wk[l]); free_mat(&M->wv[l]); free_mat(&M->wo[l]);
    free_mat(&M->wg[l]); free_mat(&M->wu[l]); free_mat(&M->wd[l]);
    free(M->bq[l]); free(M->bk[l]); free(M->bv[l]);
    free(M->kc[l]); free(M->vc[l]);
  }
  free(M->wq); free(M->wk); free(M->wv); free(M->wo); free(M->wg); free(M->wu); free(M->wd);
  free(M->bq); free(M->bk); free(M->bv);
  free(M->kc); free(M->vc);
  free_mat(&M->embed);
  if (!M->cfg.tied_embeddings) free_mat(&M->head);
  free(M->rope); free(M->gains); free(M->seq_len); free(M->tokens); free(M->logits); free(M->h);
  free(M);
}

static void round_rows(float* x, int64_t n, int act_dtype) {
  for (int64_t i = 0; i < n; ++i) x[i] = round_act(x[i], act_dtype);
}

/* Next token per row: argmax with the lowest index winning ties; with sampling enabled the
 * compared value is logit * inv_temperature + gumbel(seed, row, position * vocab + index)
 * (Gumbel-max: a draw from softmax(logits / temperature) that depends only on seed, row and
 * position). */
static int cmp_float_desc(const void* a, const void* b) {
  float x = *(const float*)a, y = *(const float*)b;
  return (x < y) - (x > y);
}
/* top_k > 0 (with sampling enabled): only logits >= the k-th largest of the row are candidates
 * (ties at that value included); 0 or >= vocab: all of them. */
ORC_API void orc_sample_rows(const float* logits, int64_t rows, int64_t vocab, int enabled, float inv_temperature,
                             int64_t top_k, uint64_t seed, const int32_t* positions, int32_t* tokens) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < rows; ++i) {
    const float* lg = logits + i * vocab;
    uint64_t first = enabled ? (uint64_t)positions[i] * (uint64_t)vocab : 0;
    float least = -INFINITY;
    if (enabled && top_k > 0 && top_k < vocab) {
      float* sorted = (float*)malloc(sizeof(float) * (size_t)vocab);
      memcpy(sorted, lg, sizeof(float) * (size_t)vocab);
      qsort(sorted, (size_t)vocab, sizeof(float), cmp_float_desc);
      least = sorted[top_k - 1];
      free(sorted);
    }
    int64_t best = -1;
    float best_v = 0.0f;
    for (int64_t v = 0; v < vocab; ++v) {
      float x = lg[v];
      if (x < least) continue;
      if (enabled) {
        float scaled = x * inv_temperature;
        float g = gen_gumbel(seed, (uint64_t)i, first + (uint64_t)v);
        x = scaled + g;
      }
      if (best < 0 || x > best_v) {
        best = v;
        best_v = x;
      }
    }
    tokens[i] = (int32_t)(best < 0 ? 0 : best);
  }
}

/* One step for all sequences.  `sample` 0 skips the lm_head (prompt tokens).  With `lens`
 * (ragged prompts, step p of the prefill): only sequences with p < lens[i] advance, and only
 * those whose prompt ends here (lens[i] - 1 == p) take the sampled token; the others keep
 * theirs.  A sequence that does not advance still runs through the step - its K/V row lands
 * at its next free position and is overwritten when the sequence does advance.
 * A sequence whose cache is full (length == l_max) still steps: its query is rotated for the
 * last position, nothing is appended, it attends over the l_max cached rows and its length
 * stays. */
static void llm_step(orc_llm* M, int sample, const int32_t* lens, int64_t p) {
  const orc_llm_config_t* c = &M->cfg;
  int64_t B = c->batch, H = c->hidden, D = c->head_dim, F = c->ffn;
  int64_t nq = c->h_q * D, nkv = c->h_kv * D;
  int act = c->act_dtype;
  float scale = 1.0f / sqrtf((float)D);
  float* xn = (float*)malloc(sizeof(float) * (size_t)(B * (H > F ? H : F)));
  float* qf = (float*)malloc(sizeof(float) * (size_t)(B * nq));
  float* kf = (float*)malloc(sizeof(float) * (size_t)(B * nkv));
  float* vf = (float*)malloc(sizeof(float) * (size_t)(B * nkv));
  uint16_t* qh = (uint16_t*)malloc(2 * (size_t)(B * nq));
  float* att = (float*)malloc(sizeof(float) * (size_t)(B * nq));
  float* delta = (float*)malloc(sizeof(float) * (size_t)(B * H));
  float* gate = (float*)malloc(sizeof(float) * (size_t)(B * F));
  float* up = (float*)malloc(sizeof(float) * (size_t)(B * F));
  int32_t* len1 = (int32_t*)malloc(4 * (size_t)B);
  int32_t* pos0 = (int32_t*)malloc(4 * (size_t)B); /* lengths when the step began = positions of the consumed tokens */
  for (int64_t i = 0; i < B; ++i) pos0[i] = M->seq_len[i];

  /* embedding row = dequantised Q8 row */
  for (int64_t i = 0; i < B; ++i) {
    int64_t t = M->tokens[i];
    for (int64_t e = 0; e < H; ++e)
      M->h[i * H + e] = M->embed.s[t * (H / 32) + e / 32] * (float)M->embed.q[t * H + e];
  }
  for (int64_t l = 0; l < c->layers; ++l) {
    orc_rmsnorm(M->h, M->gains + (2 * l) * H, xn, B, H, c->rms_eps);
    round_rows(xn, B * H, act);
    orc_q8_gemm_f32(xn, ORC_F32, M->wq[l].q, M->wq[l].s, qf, B, nq, H);
    orc_q8_gemm_f32(xn, ORC_F32, M->wk[l].q, M->wk[l].s, kf, B, nkv, H);
    orc_q8_gemm_f32(xn, ORC_F32, M->wv[l].q, M->wv[l].s, vf, B, nkv, H);
    if (c->qkv_bias)
      for (int64_t i = 0; i < B; ++i) {
        for (int64_t j = 0; j < nq; ++j) qf[i * nq + j] = qf[i * nq + j] + M->bq[l][j];
        for (int64_t j = 0; j < nkv; ++j) kf[i * nkv + j] = kf[i * nkv + j] + M->bk[l][j];
        for (int64_t j = 0; j < nkv; ++j) vf[i * nkv + j] = vf[i * nkv + j] + M->bv[l][j];
      }
    for (int64_t i = 0; i < B; ++i) {
      int64_t pos = pos0[i];
      int full = pos >= c->l_max;
      if (full) pos = c->l_max - 1;
      const float* tab = M->rope + pos * (D / 2) * 2;
      for (int64_t h = 0; h < c->h_q; ++h) rope_row_f16out(qf + (i * c->h_q + h) * D, tab, D, qh + (i * c->h_q + h) * D);
      for (int64_t h = 0; h < c->h_kv && !full; ++h) {
        uint16_t* kd = M->kc[l] + ((i * c->h_kv + h) * c->l_max + pos) * D;
        uint16_t* vd = M->vc[l] + ((i * c->h_kv + h) * c->l_max + pos) * D;
        rope_row_f16out(kf + (i * c->h_kv + h) * D, tab, D, kd);
        for (int64_t e = 0; e < D; ++e) vd[e] = f2h(vf[(i * c->h_kv + h) * D + e]);
      }
      len1[i] = (int32_t)(pos + 1);
    }
    attn_all(qh, M->kc[l], M->vc[l], len1, att, NULL, B, c->h_q, c->h_kv, D, c->l_max, scale);
    round_rows(att, B * nq, act);
    orc_q8_gemm_f32(att, ORC_F32, M->wo[l].q, M->wo[l].s, delta, B, H, nq);
    for (int64_t i = 0; i < B * H; ++i) M->h[i] = M->h[i] + delta[i];
    orc_rmsnorm(M->h, M->gains + (2 * l + 1) * H, xn, B, H, c->rms_eps);
    round_rows(xn, B * H, act);
    orc_q8_gemm_f32(xn, ORC_F32, M->wg[l].q, M->wg[l].s, gate, B, F, H);
    orc_q8_gemm_f32(xn, ORC_F32, M->wu[l].q, M->wu[l].s, up, B, F, H);
    orc_swiglu(gate, up, gate, B * F);
    round_rows(gate, B * F, act);
    orc_q8_gemm_f32(gate, ORC_F32, M->wd[l].q, M->wd[l].s, delta, B, H, F);
    for (int64_t i = 0; i < B * H; ++i) M->h[i] = M->h[i] + delta[i];
  }
  for (int64_t i = 0; i < B; ++i)
    if ((!lens || p < lens[i]) && M->seq_len[i] < c->l_max) M->seq_len[i] += 1;
  if (sample) {
    orc_rmsnorm(M->h, M->gains + (2 * c->layers) * H, xn, B, H, c->rms_eps);
    round_rows(xn, B * H, act);
    const q8mat* hd = c->tied_embeddings ? &M->embed : &M->head;
    orc_q8_gemm_f32(xn, ORC_F32, hd->q, hd->s, M->logits, B, c->vocab, H);
    int32_t* tok = (int32_t*)malloc(4 * (size_t)B);
    orc_sample_rows(M->logits, B, c->vocab, M->sampling, M->inv_temperature, M->top_k, M->sample_seed, pos0, tok);
    for (int64_t i = 0; i < B; ++i)
      if (!lens || lens[i] - 1 == p) M->tokens[i] = tok[i];
    free(tok);
  }
  free(xn); free(qf); free(kf); free(vf); free(qh); free(att); free(delta); free(gate); free(up); free(len1); free(pos0);
}

/* One tensor of the model, named as the weight file names them: 0 attn_norm, 1 q, 2 k, 3 v,
 * 4 o, 5 mlp_norm, 6 gate, 7 up, 8 down, 9 final_norm, 10 embed, 11 head, 12 q_bias, 13 k_bias,
 * 14 v_bias.  A matrix is int8 [n][k] plus f32 [n][k/32]; a vector (gain [hidden], bias [rows of
 * its projection]) is f32 behind `q`.  Returns 0, or -1 for a tensor the model does not have. */
static int llm_tensor(orc_llm* M, int64_t layer, int kind, q8mat** mat, float** gain, int64_t* gain_len) {
  const orc_llm_config_t* c = &M->cfg;
  *mat = NULL;
  *gain = NULL;
  *gain_len = c->hidden;
  if ((kind <= 8 || kind >= 12) && (layer < 0 || layer >= c->layers)) return -1;
  switch (kind) {
    case 0: *gain = M->gains + (2 * layer) * c->hidden; return 0;
    case 5: *gain = M->gains + (2 * layer + 1) * c->hidden; return 0;
    case 9: *gain = M->gains + (2 * c->layers) * c->hidden; return 0;
    case 12: if (!c->qkv_bias) return -1; *gain = M->bq[layer]; *gain_len = c->h_q * c->head_dim; return 0;
    case 13: if (!c->qkv_bias) return -1; *gain = M->bk[layer]; *gain_len = c->h_kv * c->head_dim; return 0;
    case 14: if (!c->qkv_bias) return -1; *gain = M->bv[layer]; *gain_len = c->h_kv * c->head_dim; return 0;
    case 1: *mat = &M->wq[layer]; return 0;
    case 2: *mat = &M->wk[layer]; return 0;
    case 3: *mat = &M->wv[layer]; return 0;
    case 4: *mat = &M->wo[layer]; return 0;
    case 6: *mat = &M->wg[layer]; return 0;
    case 7: *mat = &M->wu[layer]; return 0;
    case 8: *mat = &M->wd[layer]; return 0;
    case 10: *mat = &M->embed; return 0;
    case 11: if (c->tied_embeddings) return -1; *mat = &M->head; return 0;
    default: return -1;
  }
}
ORC_API int orc_llm_set_tensor(void* model, int64_t layer, int kind, const void* q, const float* s) {
  orc_llm* M = (orc_llm*)model;
  q8mat* mat;
  float* gain;
  int64_t gain_len;
  if (llm_tensor(M, layer, kind, &mat, &gain, &gain_len) != 0) return -1;
  if (gain) {
    memcpy(gain, q, sizeof(float) * (size_t)gain_len);
  } else {
    memcpy(mat->q, q, (size_t)(mat->n * mat->k));
    memcpy(mat->s, s, sizeof(float) * (size_t)(mat->n * (mat->k / 32)));
  }
  return 0;
}
ORC_API int orc_llm_get_tensor(void* model, int64_t layer, int kind, void* q, float* s) {
  orc_llm* M = (orc_llm*)model;
  q8mat* mat;
  float* gain;
  int64_t gain_len;
  if (llm_tensor(M, layer, kind, &mat, &gain, &gain_len) != 0) return -1;
  if (gain) {
    memcpy(q, gain, sizeof(float) * (size_t)gain_len);
  } else {
    memcpy(q, mat->q, (size_t)(mat->n * mat->k));
    memcpy(s, mat->s, sizeof(float) * (size_t)(mat->n * (mat->k / 32)));
  }
  return 0;
}

/* temperature 0 = greedy */
ORC_API void orc_llm_set_sampling(void* model, float temperature, int64_t top_k, uint64_t seed) {
  orc_llm* M = (orc_llm*)model;
  M->top_k = top_k;
  M->sampling = temperature > 0.0f ? 1 : 0;
  M->inv_temperature = M->sampling ? 1.0f / temperature : 1.0f;
  M->sample_seed = seed;
}

ORC_API void orc_llm_prefill(void* model, const int32_t* tokens, int64_t t) {
  orc_llm* M = (orc_llm*)model;
  int64_t B = M->cfg.batch;
  for (int64_t i = 0; i < B; ++i) M->seq_len[i] = 0;
  for (int64_t p = 0; p < t; ++p) {
    for (int64_t i = 0; i < B; ++i) M->tokens[i] = tokens[i * t + p];
    llm_step(M, p == t - 1, NULL, 0);
  }
}
/* Prompts of different lengths: sequence i consumes tokens[i][0 .. lens[i]) of a [B][t_max]
 * array (0 <= lens[i] <= t_max); afterwards its length is lens[i] and its current token is the
 * one sampled after its last prompt token (token 0 for an empty prompt).  lens[i] == -1 keeps
 * sequence i as it is (cache, length, current token). */
ORC_API void orc_llm_prefill_ragged(void* model, const int32_t* tokens, int64_t t_max, const int32_t* lens) {
  orc_llm* M = (orc_llm*)model;
  int64_t B = M->cfg.batch;
  int32_t* next = (int32_t*)calloc((size_t)B, 4);
  for (int64_t i = 0; i < B; ++i) {
    if (lens[i] < 0) next[i] = M->tokens[i];
    else M->seq_len[i] = 0;
  }
  for (int64_t p = 0; p < t_max; ++p) {
    int ends_here = 0, active = 0;
    for (int64_t i = 0; i < B; ++i) {
      M->tokens[i] = p < lens[i] ? tokens[i * t_max + p] : 0;
      if (lens[i] - 1 == p) ends_here = 1;
      if (p < lens[i]) active = 1;
    }
    if (!active) break;
    llm_step(M, ends_here, lens, p);
    for (int64_t i = 0; i < B; ++i)
      if (lens[i] - 1 == p) next[i] = M->tokens[i];
  }
  memcpy(M->tokens, next, 4 * (size_t)B);
  free(next);
}
/* Fill positions [0,t) of every layer's cache with seeded N(0,1) fp16 values
 * (streams 2l for K, 2l+1 for V, index = flat index in the [B][Hkv][Lmax][D]
 * cache) and set every length to t: decode at a given context length without
 * running a prompt. */
ORC_API void orc_llm_synth_kv(void* model, int64_t t, uint64_t seed) {
  orc_llm* M = (orc_llm*)model;
  const orc_llm_config_t* c = &M->cfg;
  int64_t D = c->head_dim;
  for (int64_t l = 0; l < c->layers; ++l)
    for (int64_t b = 0; b < c->batch; ++b)
      for (int64_t h = 0; h < c->h_kv; ++h) {
        int64_t first = ((b * c->h_kv + h) * c->l_max) * D;
        orc_synth_fill(M->kc[l] + first, ORC_F16, 2, seed, (uint64_t)(2 * l), first, t * D, 0.0f, 1.0f);
        orc_synth_fill(M->vc[l] + first, ORC_F16, 2, seed, (uint64_t)(2 * l + 1), first, t * D, 0.0f, 1.0f);
      }
  for (int64_t i = 0; i < c->batch; ++i) M->seq_len[i] = (int32_t)t;
}
ORC_API void orc_llm_set_tokens(void* model, const int32_t* tokens) {
  orc_llm* M = (orc_llm*)model;
  memcpy(M->tokens, tokens, 4 * (size_t)M->cfg.batch);
}
ORC_API void orc_llm_decode_step(void* model, int32_t* next_tokens) {
  orc_llm* M = (orc_llm*)model;
  llm_step(M, 1, NULL, 0);
  if (next_tokens) memcpy(next_tokens, M->tokens, 4 * (size_t)M->cfg.batch);
}
ORC_API void orc_llm_read_kv(void* model, int64_t layer, uint16_t* k, uint16_t* v) {
  orc_llm* M = (orc_llm*)model;
  size_t kv = (size_t)(M->cfg.batch * M->cfg.h_kv * M->cfg.l_max * M->cfg.head_dim);
  memcpy(k, M->kc[layer], kv * 2);
  memcpy(v, M->vc[layer], kv * 2);
}
ORC_API void orc_llm_read_logits(void* model, float* logits) {
  orc_llm* M = (orc_llm*)model;
  memcpy(logits, M->logits, 4 * (size_t)(M->cfg.batch * M->cfg.vocab));
}
ORC_API void orc_llm_read_seq_len(void* model, int32_t* out) {
  orc_llm* M = (orc_llm*)model;
  memcpy(out, M->seq_len, 4 * (size_t)M->cfg.batch);
}
ORC_API void orc_llm_set_seq_len(void* model, int64_t t) {
  orc_llm* M = (orc_llm*)model;
  for (int64_t i = 0; i < M->cfg.batch; ++i) M->seq_len[i] = (int32_t)t;
}
