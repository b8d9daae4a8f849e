// Weight file of the decode model: one flat file, [header | tensors], that the library maps
// read-only and copies from.  It is the device-side counterpart of the reference's memory-mapped
// zone (`Inside a zone called "D" mapped from "f.bin"`, crates/logicaffeine_language/src/ast/stmt.rs:405-418;
// Zone::new_mapped, crates/logicaffeine_system/src/memory.rs:97-103): the file is the format,
// there is no parsing step between the bytes on disk and the bytes in HBM.
//
// Layout (little endian; every region starts on a 256-byte boundary, gaps are zero):
//   header, 256 bytes (WeightsHeader)
//   per layer l = 0..layers-1, in this order:
//     attn_norm  f32 [hidden]
//     q  k  v    each: int8 [rows][hidden] then f32 [rows][hidden/32]   (rows = h_q*D, h_kv*D, h_kv*D)
//     q_bias  k_bias  v_bias   f32 [rows] each, present only when header flag bit 0 (qkv_bias) is set
//     o          int8 [hidden][h_q*D]     then f32 [hidden][h_q*D/32]
//     mlp_norm   f32 [hidden]
//     gate  up   each: int8 [ffn][hidden] then f32 [ffn][hidden/32]
//     down       int8 [hidden][ffn]       then f32 [hidden][ffn/32]
//   final_norm   f32 [hidden]
//   embed        int8 [vocab][hidden] then f32 [vocab][hidden/32]
//   head         the same shape, present only when tied_embeddings == 0
// The matrices are stored whole; a tensor-parallel rank copies its rows (q, k, v, gate, up) or
// its columns (o, down) out of them, so one file serves every group size.
#pragma once

#include <stddef.h>
#include <stdint.h>

#include "common.cuh"

namespace logos {

constexpr uint32_t WEIGHTS_VERSION = 1;
constexpr int64_t WEIGHTS_ALIGN = 256;

struct WeightsHeader {
  char     magic[8];  // "LOGOSQ8W"
  uint32_t version;
  uint32_t header_bytes;  // 256
  int64_t  layers, hidden, h_q, h_kv, head_dim, ffn, vocab;
  uint32_t tied_embeddings;
  uint32_t block;       // elements per scale along K: 32
  uint64_t file_bytes;  // header + payload, as laid out above
  uint32_t flags;       // bit 0: q/k/v bias vectors are present
  uint8_t  pad[256 - 8 - 4 - 4 - 7 * 8 - 4 - 4 - 8 - 4];
};
static_assert(sizeof(WeightsHeader) == 256, "the header is 256 bytes");

struct WeightsArch {
  int64_t layers = 0, hidden = 0, h_q = 0, h_kv = 0, head_dim = 0, ffn = 0, vocab = 0;
  int32_t tied = 0;
  int32_t qkv_bias = 0;
};

// One tensor's place in the file.  Matrices: q_off/q_bytes = the int8 part [n][k], s_off/s_bytes
// = the scales [n][k/32].  Vectors (gains, biases): q_off/q_bytes = the f32 vector, n = 1,
// k = its length, no scales.
struct TensorSpan {
  int64_t q_off = 0, q_bytes = 0, s_off = 0, s_bytes = 0, n = 0, k = 0;
};

// The rectangle of a whole matrix that one rank of a tensor-parallel group holds.
struct ShardRect {
  int64_t row0 = 0, rows = 0, col0 = 0, cols = 0;
};

WeightsArch arch_of(const logos_llm_config_t& c);
logos_status_t check_arch(const WeightsArch& a, const char* who);
bool is_vector(int kind);
// kind: logos_weight_tensor_t.  layer is ignored for final_norm, embed and head.
logos_status_t weights_span(const WeightsArch& a, int64_t layer, int kind, TensorSpan* out, const char* who);
int64_t weights_file_bytes(const WeightsArch& a);
logos_status_t weights_shard(const WeightsArch& a, int kind, int tp_degree, int tp_rank, ShardRect* out, const char* who);

// A weight file mapped read-only.
struct MappedWeights {
  const uint8_t* base = nullptr;
  size_t bytes = 0;
  WeightsArch arch;
};
// Error (1): the file cannot be opened or mapped.  DeserializationFailed (5): it is not a weight
// file of this version, its header is inconsistent, or it is shorter than its header says.
logos_status_t weights_open(const char* path, MappedWeights* out, const char* who);
void weights_close(MappedWeights* w);

}  // namespace logos
