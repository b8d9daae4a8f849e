// Weight file: layout arithmetic, the read-only mapping, and the host-side entry points that need
// no GPU (layout queries, header check, reading one rank's shard into host memory).  The copy
// into a model's device buffers lives with the model (llm.cu) and uses the same shard rectangles.
#include "weights.cuh"

#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace logos {

namespace {

const char MAGIC[8] = {'L', 'O', 'G', 'O', 'S', 'Q', '8', 'W'};

int64_t align_up(int64_t v) { return (v + WEIGHTS_ALIGN - 1) / WEIGHTS_ALIGN * WEIGHTS_ALIGN; }

// Walks the file in storage order and stops at (layer, kind); kind < 0 walks to the end and
// returns the file size in out->q_off.
void walk(const WeightsArch& a, int64_t layer, int kind, TensorSpan* out) {
  const int64_t H = a.hidden, nq = a.h_q * a.head_dim, nkv = a.h_kv * a.head_dim, F = a.ffn;
  int64_t off = (int64_t)sizeof(WeightsHeader);
  bool found = false;
  auto vec = [&](int64_t l, int k, int64_t len) {
    if (found) return;
    if (l == layer && k == kind) {
      out->q_off = off; out->q_bytes = len * 4; out->s_off = 0; out->s_bytes = 0; out->n = 1; out->k = len;
      found = true;
    }
    off = align_up(off + len * 4);
  };
  auto gain = [&](int64_t l, int k) { vec(l, k, H); };
  auto mat = [&](int64_t l, int k, int64_t n, int64_t kk) {
    if (found) return;
    const int64_t qb = n * kk, sb = n * (kk / 32) * 4;
    if (l == layer && k == kind) {
      out->q_off = off; out->q_bytes = qb; out->s_off = align_up(off + qb); out->s_bytes = sb; out->n = n; out->k = kk;
      found = true;
    }
    off = align_up(align_up(off + qb) + sb);
  };
  for (int64_t l = 0; l < a.layers && !found; ++l) {
    gain(l, LOGOS_W_ATTN_NORM);
    mat(l, LOGOS_W_Q, nq, H);
    mat(l, LOGOS_W_K, nkv, H);
    mat(l, LOGOS_W_V, nkv, H);
    if (a.qkv_bias) {
      vec(l, LOGOS_W_Q_BIAS, nq);
      vec(l, LOGOS_W_K_BIAS, nkv);
      vec(l, LOGOS_W_V_BIAS, nkv);
    }
    mat(l, LOGOS_W_O, H, nq);
    gain(l, LOGOS_W_MLP_NORM);
    mat(l, LOGOS_W_GATE, F, H);
    mat(l, LOGOS_W_UP, F, H);
    mat(l, LOGOS_W_DOWN, H, F);
  }
  gain(layer, LOGOS_W_FINAL_NORM);
  mat(layer, LOGOS_W_EMBED, a.vocab, H);
  if (!a.tied) mat(layer, LOGOS_W_HEAD, a.vocab, H);
  if (!found) { out->q_off = off; out->q_bytes = 0; }
}

}  // namespace

WeightsArch arch_of(const logos_llm_config_t& c) {
  WeightsArch a;
  a.layers = c.layers; a.hidden = c.hidden; a.h_q = c.h_q; a.h_kv = c.h_kv; a.head_dim = c.head_dim;
  a.ffn = c.ffn; a.vocab = c.vocab; a.tied = c.tied_embeddings ? 1 : 0;
  a.qkv_bias = c.qkv_bias ? 1 : 0;
  return a;
}

logos_status_t check_arch(const WeightsArch& a, const char* who) {
  if (a.layers <= 0 || a.hidden <= 0 || a.h_q <= 0 || a.h_kv <= 0 || a.head_dim <= 0 || a.ffn <= 0 || a.vocab <= 0)
    return fail(LOGOS_OUT_OF_BOUNDS, "%s: every extent must be positive", who);
  if (a.hidden % 32 || a.ffn % 32 || (a.h_q * a.head_dim) % 32)
    return fail(LOGOS_ERROR, "%s: hidden, ffn and the q width must be multiples of the Q8 block 32", who);
  // extents a 64-bit file offset cannot overflow with
  if (a.layers > (1 << 20) || a.hidden > (1 << 24) || a.ffn > (1 << 26) || a.vocab > (1 << 28) || a.h_q > (1 << 16) ||
      a.h_kv > (1 << 16) || a.head_dim > (1 << 12))
    return fail(LOGOS_OUT_OF_BOUNDS, "%s: extent too large", who);
  return LOGOS_OK;
}

bool is_vector(int kind) {
  return kind == LOGOS_W_ATTN_NORM || kind == LOGOS_W_MLP_NORM || kind == LOGOS_W_FINAL_NORM || kind == LOGOS_W_Q_BIAS ||
         kind == LOGOS_W_K_BIAS || kind == LOGOS_W_V_BIAS;
}

int64_t weights_file_bytes(const WeightsArch& a) {
  TensorSpan end;
  walk(a, -1, -1, &end);
  return end.q_off;
}

logos_status_t weights_span(const WeightsArch& a, int64_t layer, int kind, TensorSpan* out, const char* who) {
  if (kind < LOGOS_W_ATTN_NORM || kind > LOGOS_W_V_BIAS) return fail(LOGOS_OUT_OF_BOUNDS, "%s: tensor kind %d", who, kind);
  const bool per_layer = kind <= LOGOS_W_DOWN || kind >= LOGOS_W_Q_BIAS;
  if (kind >= LOGOS_W_Q_BIAS && !a.qkv_bias) return fail(LOGOS_ERROR, "%s: the architecture has no q/k/v biases", who);
  if (per_layer && (layer < 0 || layer >= a.layers))
    return fail(LOGOS_OUT_OF_BOUNDS, "%s: layer %lld of %lld", who, (long long)layer, (long long)a.layers);
  if (kind == LOGOS_W_HEAD && a.tied) return fail(LOGOS_ERROR, "%s: tied embeddings: the file has no separate lm_head", who);
  *out = TensorSpan();
  walk(a, per_layer ? layer : -1, kind, out);
  return LOGOS_OK;
}

logos_status_t weights_shard(const WeightsArch& a, int kind, int g, int r, ShardRect* out, const char* who) {
  if (g < 1 || r < 0 || r >= g) return fail(LOGOS_OUT_OF_BOUNDS, "%s: tp_rank %d of tp_degree %d", who, r, g);
  if (a.h_kv % g || a.h_q % g || a.ffn % g) return fail(LOGOS_ERROR, "%s: heads and ffn must divide by tp_degree", who);
  const int64_t H = a.hidden, nq = a.h_q * a.head_dim, nkv = a.h_kv * a.head_dim, F = a.ffn;
  if ((nq / g) % 32 || (F / g) % 32) return fail(LOGOS_ERROR, "%s: a rank's column slice must keep whole Q8 blocks", who);
  ShardRect s;
  switch (kind) {
    case LOGOS_W_Q:    s = {r * (nq / g), nq / g, 0, H}; break;
    case LOGOS_W_K:
    case LOGOS_W_V:    s = {r * (nkv / g), nkv / g, 0, H}; break;
    case LOGOS_W_O:    s = {0, H, r * (nq / g), nq / g}; break;
    case LOGOS_W_GATE:
    case LOGOS_W_UP:   s = {r * (F / g), F / g, 0, H}; break;
    case LOGOS_W_DOWN: s = {0, H, r * (F / g), F / g}; break;
    case LOGOS_W_EMBED:
    case LOGOS_W_HEAD: s = {0, a.vocab, 0, H}; break;
    case LOGOS_W_ATTN_NORM:
    case LOGOS_W_MLP_NORM:
    case LOGOS_W_FINAL_NORM: s = {0, 1, 0, H}; break;
    case LOGOS_W_Q_BIAS: s = {0, 1, r * (nq / g), nq / g}; break;
    case LOGOS_W_K_BIAS:
    case LOGOS_W_V_BIAS: s = {0, 1, r * (nkv / g), nkv / g}; break;
    default: return fail(LOGOS_OUT_OF_BOUNDS, "%s: tensor kind %d", who, kind);
  }
  *out = s;
  return LOGOS_OK;
}

logos_status_t weights_open(const char* path, MappedWeights* out, const char* who) {
  *out = MappedWeights();
  int fd = open(path, O_RDONLY);
  if (fd < 0) return fail(LOGOS_ERROR, "%s: cannot open '%s': %s", who, path, strerror(errno));
  struct stat st;
  if (fstat(fd, &st) != 0) {
    int e = errno;
    close(fd);
    return fail(LOGOS_ERROR, "%s: cannot stat '%s': %s", who, path, strerror(e));
  }
  if ((size_t)st.st_size < sizeof(WeightsHeader)) {
    close(fd);
    return fail(LOGOS_DESERIALIZATION_FAILED, "%s: '%s' is shorter than a weight-file header", who, path);
  }
  void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  int e = errno;
  close(fd);  // the mapping keeps the file
  if (p == MAP_FAILED) return fail(LOGOS_ERROR, "%s: cannot map '%s': %s", who, path, strerror(e));
  out->base = static_cast<const uint8_t*>(p);
  out->bytes = (size_t)st.st_size;
  WeightsHeader h;
  memcpy(&h, p, sizeof(h));
  logos_status_t s = LOGOS_OK;
  if (memcmp(h.magic, MAGIC, 8) != 0)
    s = fail(LOGOS_DESERIALIZATION_FAILED, "%s: '%s' is not a weight file (magic)", who, path);
  else if (h.version != WEIGHTS_VERSION || h.header_bytes != sizeof(WeightsHeader) || h.block != 32)
    s = fail(LOGOS_DESERIALIZATION_FAILED, "%s: '%s' has version %u, header %u bytes, block %u; this library reads %u / %u / 32",
             who, path, h.version, h.header_bytes, h.block, WEIGHTS_VERSION, (unsigned)sizeof(WeightsHeader));
  if (s == LOGOS_OK) {
    WeightsArch a;
    a.layers = h.layers; a.hidden = h.hidden; a.h_q = h.h_q; a.h_kv = h.h_kv; a.head_dim = h.head_dim;
    a.ffn = h.ffn; a.vocab = h.vocab; a.tied = h.tied_embeddings ? 1 : 0;
    a.qkv_bias = (h.flags & 1u) ? 1 : 0;
    if (h.flags & ~1u) {
      s = fail(LOGOS_DESERIALIZATION_FAILED, "%s: '%s' sets header flags 0x%x this library does not know", who, path, h.flags);
    } else if (check_arch(a, who) != LOGOS_OK) {
      s = fail(LOGOS_DESERIALIZATION_FAILED, "%s: '%s' names an architecture this library cannot hold", who, path);
    } else {
      const int64_t need = weights_file_bytes(a);
      if (h.file_bytes != (uint64_t)need)
        s = fail(LOGOS_DESERIALIZATION_FAILED, "%s: '%s' says %llu bytes, its architecture needs %lld", who, path,
                 (unsigned long long)h.file_bytes, (long long)need);
      else if ((int64_t)out->bytes < need)
        s = fail(LOGOS_DESERIALIZATION_FAILED, "%s: '%s' is truncated: %lld of %lld bytes", who, path, (long long)out->bytes,
                 (long long)need);
      else
        out->arch = a;
    }
  }
  if (s != LOGOS_OK) weights_close(out);
  return s;
}

void weights_close(MappedWeights* w) {
  if (w->base) munmap(const_cast<uint8_t*>(w->base), w->bytes);
  *w = MappedWeights();
}

}  // namespace logos

using namespace logos;

extern "C" {

logos_status_t logos_llm_weights_file_bytes(const logos_llm_config_t* cfg, int64_t* bytes_out) {
  return guarded([&]() -> logos_status_t {
    if (!cfg || !bytes_out) return fail(LOGOS_NULL_POINTER, "logos_llm_weights_file_bytes: null argument");
    const WeightsArch a = arch_of(*cfg);
    LOGOS_TRY(check_arch(a, "logos_llm_weights_file_bytes"));
    *bytes_out = weights_file_bytes(a);
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_weights_span(const logos_llm_config_t* cfg, int64_t layer, int32_t tensor, int64_t* q_off_out,
                                      int64_t* q_bytes_out, int64_t* s_off_out, int64_t* s_bytes_out) {
  return guarded([&]() -> logos_status_t {
    if (!cfg || !q_off_out || !q_bytes_out || !s_off_out || !s_bytes_out)
      return fail(LOGOS_NULL_POINTER, "logos_llm_weights_span: null argument");
    const WeightsArch a = arch_of(*cfg);
    LOGOS_TRY(check_arch(a, "logos_llm_weights_span"));
    TensorSpan t;
    LOGOS_TRY(weights_span(a, layer, tensor, &t, "logos_llm_weights_span"));
    *q_off_out = t.q_off; *q_bytes_out = t.q_bytes; *s_off_out = t.s_off; *s_bytes_out = t.s_bytes;
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_weights_header(const logos_llm_config_t* cfg, void* out_256_bytes) {
  return guarded([&]() -> logos_status_t {
    if (!cfg || !out_256_bytes) return fail(LOGOS_NULL_POINTER, "logos_llm_weights_header: null argument");
    const WeightsArch a = arch_of(*cfg);
    LOGOS_TRY(check_arch(a, "logos_llm_weights_header"));
    WeightsHeader h;
    memset(&h, 0, sizeof(h));
    memcpy(h.magic, "LOGOSQ8W", 8);
    h.version = WEIGHTS_VERSION;
    h.header_bytes = (uint32_t)sizeof(WeightsHeader);
    h.layers = a.layers; h.hidden = a.hidden; h.h_q = a.h_q; h.h_kv = a.h_kv; h.head_dim = a.head_dim;
    h.ffn = a.ffn; h.vocab = a.vocab; h.tied_embeddings = (uint32_t)a.tied;
    h.block = 32;
    h.flags = a.qkv_bias ? 1u : 0u;
    h.file_bytes = (uint64_t)weights_file_bytes(a);
    memcpy(out_256_bytes, &h, sizeof(h));
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_weights_check(const char* path, logos_llm_config_t* cfg_out) {
  return guarded([&]() -> logos_status_t {
    if (!path) return fail(LOGOS_NULL_POINTER, "logos_llm_weights_check: path is null");
    MappedWeights w;
    LOGOS_TRY(weights_open(path, &w, "logos_llm_weights_check"));
    if (cfg_out) {
      cfg_out->layers = w.arch.layers; cfg_out->hidden = w.arch.hidden; cfg_out->h_q = w.arch.h_q;
      cfg_out->h_kv = w.arch.h_kv; cfg_out->head_dim = w.arch.head_dim; cfg_out->ffn = w.arch.ffn;
      cfg_out->vocab = w.arch.vocab; cfg_out->tied_embeddings = w.arch.tied;
      cfg_out->qkv_bias = w.arch.qkv_bias;
    }
    weights_close(&w);
    return LOGOS_OK;
  });
}

logos_status_t logos_llm_weights_read_shard(const char* path, int32_t tp_degree, int32_t tp_rank, int64_t layer,
                                            int32_t tensor, void* q_out, int64_t q_capacity, float* s_out,
                                            int64_t s_capacity, int64_t* rows_out, int64_t* cols_out) {
  return guarded([&]() -> logos_status_t {
    const char* who = "logos_llm_weights_read_shard";
    if (!path || !q_out) return fail(LOGOS_NULL_POINTER, "%s: null argument", who);
    MappedWeights w;
    LOGOS_TRY(weights_open(path, &w, who));
    TensorSpan t;
    ShardRect r;
    logos_status_t s = weights_span(w.arch, layer, tensor, &t, who);
    if (s == LOGOS_OK) s = weights_shard(w.arch, tensor, tp_degree, tp_rank, &r, who);
    if (s == LOGOS_OK) {
      if (is_vector(tensor)) {  // a gain is whole on every rank, a bias is the rank's slice
        if (q_capacity < r.cols * 4) s = fail(LOGOS_OUT_OF_BOUNDS, "%s: the vector needs %lld bytes", who, (long long)(r.cols * 4));
        else memcpy(q_out, w.base + t.q_off + r.col0 * 4, (size_t)r.cols * 4);
      } else if (!s_out) {
        s = fail(LOGOS_NULL_POINTER, "%s: s_out is null", who);
      } else if (q_capacity < r.rows * r.cols || s_capacity < r.rows * (r.cols / 32) * 4) {
        s = fail(LOGOS_OUT_OF_BOUNDS, "%s: the shard needs %lld + %lld bytes", who, (long long)(r.rows * r.cols),
                 (long long)(r.rows * (r.cols / 32) * 4));
      } else {
        const int8_t* q = reinterpret_cast<const int8_t*>(w.base + t.q_off);
        const float* sc = reinterpret_cast<const float*>(w.base + t.s_off);
        const int64_t kb = t.k / 32, cb = r.cols / 32;
        for (int64_t i = 0; i < r.rows; ++i) {
          memcpy(static_cast<int8_t*>(q_out) + i * r.cols, q + (r.row0 + i) * t.k + r.col0, (size_t)r.cols);
          memcpy(s_out + i * cb, sc + (r.row0 + i) * kb + r.col0 / 32, (size_t)cb * 4);
        }
      }
    }
    if (s == LOGOS_OK) {
      if (rows_out) *rows_out = r.rows;
      if (cols_out) *cols_out = r.cols;
    }
    weights_close(&w);
    return s;
  });
}

}  // extern "C"
