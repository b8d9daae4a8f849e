"""Weight file of the decode model: layout, writer and host-side reader.

One flat file `[256-byte header | tensors]` that the library maps read-only and
streams to the GPU (`Llm.loadWeights`).  It is the device-side counterpart of the
reference's memory-mapped zone (`Inside a zone called "D" mapped from "f.bin"`,
crates/logicaffeine_language/src/ast/stmt.rs:405-418; Zone::new_mapped,
crates/logicaffeine_system/src/memory.rs:97-103): the bytes on disk are the bytes
in HBM, there is nothing to parse.

Regions start on 256-byte boundaries, in this order: per layer attn_norm, q, k, v,
(q_bias, k_bias, v_bias when the architecture has them: header flag bit 0), o,
mlp_norm, gate, up, down; then final_norm, embed and (untied only) head.  A matrix
is int8 [n][k] followed by f32 [n][k/32]; a gain is f32 [hidden], a bias f32 [rows
of its projection].

`layout()` restates the arithmetic in Python, independently of the library's
`logos_llm_weights_span`; the tests hold the two against each other.
"""
import ctypes as C
import struct

import numpy as np

from ._lib import LlmConfig, call

ATTN_NORM, Q, K, V, O, MLP_NORM, GATE, UP, DOWN, FINAL_NORM, EMBED, HEAD, Q_BIAS, K_BIAS, V_BIAS = range(15)
TENSOR_NAMES = ("attn_norm", "q", "k", "v", "o", "mlp_norm", "gate", "up", "down", "final_norm", "embed", "head",
                "q_bias", "k_bias", "v_bias")
GAINS = (ATTN_NORM, MLP_NORM, FINAL_NORM)
BIASES = (Q_BIAS, K_BIAS, V_BIAS)
VECTORS = GAINS + BIASES
MAGIC = b"LOGOSQ8W"
VERSION = 1
HEADER_BYTES = 256
ALIGN = 256
_ARCH = ("layers", "hidden", "h_q", "h_kv", "head_dim", "ffn", "vocab")


def _up(v):
    return (v + ALIGN - 1) // ALIGN * ALIGN


def _arch(cfg):
    """(layers, hidden, h_q, h_kv, head_dim, ffn, vocab, tied, qkv_bias) from a dict or an LlmConfig."""
    get = (lambda k: cfg[k]) if isinstance(cfg, dict) else (lambda k: getattr(cfg, k))
    tied = cfg.get("tied_embeddings", 1) if isinstance(cfg, dict) else cfg.tied_embeddings
    bias = cfg.get("qkv_bias", 0) if isinstance(cfg, dict) else cfg.qkv_bias
    return tuple(int(get(k)) for k in _ARCH) + (1 if tied else 0, 1 if bias else 0)


def shape(cfg, kind):
    """(n, k) of a whole tensor; a vector is (1, length)."""
    _, hidden, h_q, h_kv, d, ffn, vocab, _, _ = _arch(cfg)
    return {
        ATTN_NORM: (1, hidden), MLP_NORM: (1, hidden), FINAL_NORM: (1, hidden),
        Q_BIAS: (1, h_q * d), K_BIAS: (1, h_kv * d), V_BIAS: (1, h_kv * d),
        Q: (h_q * d, hidden), K: (h_kv * d, hidden), V: (h_kv * d, hidden), O: (hidden, h_q * d),
        GATE: (ffn, hidden), UP: (ffn, hidden), DOWN: (hidden, ffn), EMBED: (vocab, hidden), HEAD: (vocab, hidden),
    }[kind]


def tensors(cfg):
    """(layer, kind) of every tensor in storage order (layer is 0 for the model-level ones)."""
    layers, tied, bias = _arch(cfg)[0], _arch(cfg)[7], _arch(cfg)[8]
    per_layer = [ATTN_NORM, Q, K, V] + (list(BIASES) if bias else []) + [O, MLP_NORM, GATE, UP, DOWN]
    out = [(l, kind) for l in range(layers) for kind in per_layer]
    out += [(0, FINAL_NORM), (0, EMBED)]
    if not tied:
        out.append((0, HEAD))
    return out


def layout(cfg):
    """{(layer, kind): (q_off, q_bytes, s_off, s_bytes)} and the file size."""
    off = HEADER_BYTES
    spans = {}
    for layer, kind in tensors(cfg):
        n, k = shape(cfg, kind)
        if kind in VECTORS:
            spans[(layer, kind)] = (off, k * 4, 0, 0)
            off = _up(off + k * 4)
        else:
            s_off = _up(off + n * k)
            spans[(layer, kind)] = (off, n * k, s_off, n * (k // 32) * 4)
            off = _up(s_off + n * (k // 32) * 4)
    return spans, off


def header(cfg):
    layers, hidden, h_q, h_kv, d, ffn, vocab, tied, bias = _arch(cfg)
    _, total = layout(cfg)
    h = MAGIC + struct.pack("<II7qIIQI", VERSION, HEADER_BYTES, layers, hidden, h_q, h_kv, d, ffn, vocab, tied, 32, total,
                            bias)
    return h + bytes(HEADER_BYTES - len(h))


def writeWeightsFile(path, cfg, get_tensor):
    """Write a weight file.  get_tensor(layer, kind) returns (q int8 [n][k], s f32 [n][k/32]) for a
    matrix and an f32 vector for a gain (None: all ones) or a bias (None: all zeros)."""
    spans, total = layout(cfg)
    with open(path, "wb") as f:
        f.truncate(total)
        f.write(header(cfg))
        for (layer, kind), (q_off, q_bytes, s_off, s_bytes) in spans.items():
            n, k = shape(cfg, kind)
            got = get_tensor(layer, kind)
            if kind in VECTORS:
                default = np.ones if kind in GAINS else np.zeros
                g = default(k, np.float32) if got is None else np.ascontiguousarray(got, np.float32).reshape(k)
                f.seek(q_off)
                f.write(g.tobytes())
                continue
            q, s = got
            q = np.ascontiguousarray(q, np.int8)
            s = np.ascontiguousarray(s, np.float32)
            if q.shape != (n, k) or s.shape != (n, k // 32):
                raise ValueError("%s of layer %d: got %s / %s, the file holds %s / %s"
                                 % (TENSOR_NAMES[kind], layer, q.shape, s.shape, (n, k), (n, k // 32)))
            f.seek(q_off)
            f.write(q.tobytes())
            f.seek(s_off)
            f.write(s.tobytes())
    return total


def q8QuantizeHost(w):
    """Q8 blocks of a float matrix on the host, for converting a float checkpoint into a weight
    file: per 32 elements along k, s = max|w| / 127 (f32 division), q = round-half-even(w / s),
    an all-zero block stores s = 0.  The same rule, bit for bit, as the library's
    logos_q8_quantize kernel.  Returns (q int8 [n][k], s f32 [n][k/32])."""
    w = np.ascontiguousarray(w, np.float32)
    n, k = w.shape
    if k % 32:
        raise ValueError("k = %d is not a multiple of the Q8 block 32" % k)
    blocks = w.reshape(n, k // 32, 32)
    amax = np.abs(blocks).max(axis=2)
    s = (amax / np.float32(127.0)).astype(np.float32)
    safe = np.where(amax > 0, s, np.float32(1.0)).astype(np.float32)
    q = np.rint((blocks / safe[:, :, None]).astype(np.float32))
    q = np.where(amax[:, :, None] > 0, np.clip(q, -127, 127), 0).astype(np.int8)
    return q.reshape(n, k), s


def _cfg_struct(cfg):
    if isinstance(cfg, LlmConfig):
        return cfg
    fields = {name for name, _ in LlmConfig._fields_}
    return LlmConfig(**{k: v for k, v in cfg.items() if k in fields})


def weightsFileBytes(cfg):
    """File size by the library's own arithmetic (logos_llm_weights_file_bytes)."""
    out = C.c_int64()
    call("logos_llm_weights_file_bytes", C.byref(_cfg_struct(cfg)), C.byref(out))
    return out.value


def weightsSpan(cfg, layer, kind):
    """(q_off, q_bytes, s_off, s_bytes) by the library's own arithmetic (logos_llm_weights_span)."""
    v = [C.c_int64() for _ in range(4)]
    call("logos_llm_weights_span", C.byref(_cfg_struct(cfg)), int(layer), int(kind), *[C.byref(x) for x in v])
    return tuple(x.value for x in v)


def weightsHeader(cfg):
    buf = (C.c_uint8 * HEADER_BYTES)()
    call("logos_llm_weights_header", C.byref(_cfg_struct(cfg)), C.cast(buf, C.c_void_p))
    return bytes(buf)


def weightsCheck(path):
    """Validate a file and return its architecture as a dict (LogosError: DeserializationFailed /
    Error as the library reports them)."""
    cfg = LlmConfig()
    call("logos_llm_weights_check", str(path).encode(), C.byref(cfg))
    out = {k: int(getattr(cfg, k)) for k in _ARCH}
    out["tied_embeddings"] = int(cfg.tied_embeddings)
    out["qkv_bias"] = int(cfg.qkv_bias)
    return out


def weightsReadShard(path, layer, kind, tp_degree=1, tp_rank=0):
    """What one rank of a tensor-parallel group holds of a tensor, read on the host:
    (q int8 [rows][cols], s f32 [rows][cols/32]), or an f32 vector for a gain (whole) or a
    bias (the rank's slice)."""
    arch = weightsCheck(path)
    n, k = shape(arch, kind)
    if kind in VECTORS:
        g = np.empty(k // tp_degree if kind in BIASES else k, np.float32)
        call("logos_llm_weights_read_shard", str(path).encode(), int(tp_degree), int(tp_rank), int(layer), int(kind),
             g.ctypes.data_as(C.c_void_p), g.nbytes, None, 0, None, None)
        return g
    q = np.empty(n * k // tp_degree if kind not in (EMBED, HEAD) else n * k, np.int8)
    s = np.empty(q.size // 32, np.float32)
    rows, cols = C.c_int64(), C.c_int64()
    call("logos_llm_weights_read_shard", str(path).encode(), int(tp_degree), int(tp_rank), int(layer), int(kind),
         q.ctypes.data_as(C.c_void_p), q.nbytes, s.ctypes.data_as(C.c_void_p), s.nbytes, C.byref(rows), C.byref(cols))
    return q.reshape(rows.value, cols.value), s.reshape(rows.value, cols.value // 32)

