"""ctypes front of the CPU oracle (oracle/logos_oracle.c).

Test infrastructure: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline legs only.  The shipped package never imports it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liblogos_oracle.so")

F32, F16, BF16, I8, I32 = 0, 1, 2, 3, 4


def build(force=False):
    """Compile the oracle with the committed Makefile."""
    src = os.path.join(_HERE, "logos_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


class LlmConfig(C.Structure):
    _fields_ = [
        ("layers", C.c_int64), ("hidden", C.c_int64), ("h_q", C.c_int64), ("h_kv", C.c_int64),
        ("head_dim", C.c_int64), ("ffn", C.c_int64), ("vocab", C.c_int64), ("l_max", C.c_int64),
        ("batch", C.c_int64),
        ("rms_eps", C.c_float), ("rope_theta", C.c_float),
        ("tied_embeddings", C.c_int32), ("tp_degree", C.c_int32), ("tp_rank", C.c_int32),
        ("device", C.c_int32), ("act_dtype", C.c_int32),
        ("seed", C.c_uint64), ("init_std", C.c_float), ("qkv_bias", C.c_int32),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        L.orc_threads.restype = C.c_int
        L.orc_h2f.restype = C.c_float
        L.orc_h2f.argtypes = [C.c_uint16]
        L.orc_bf2f.restype = C.c_float
        L.orc_bf2f.argtypes = [C.c_uint16]
        L.orc_f2h.restype = C.c_uint16
        L.orc_f2h.argtypes = [C.c_float]
        L.orc_f2bf.restype = C.c_uint16
        L.orc_f2bf.argtypes = [C.c_float]
        L.orc_llm_create.restype = C.c_void_p
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def threads():
    return lib().orc_threads()


def set_threads(n):
    lib().orc_set_threads(C.c_int(n))


_NP = {F32: np.float32, F16: np.uint16, BF16: np.uint16, I8: np.int8, I32: np.int32}


def synth_fill(dtype, kind, seed, stream, first, count, a=0.0, b=1.0):
    out = np.empty(count, dtype=_NP[dtype])
    lib().orc_synth_fill(_p(out), C.c_int(dtype), C.c_int(kind), C.c_uint64(seed), C.c_uint64(stream),
                         C.c_int64(first), C.c_int64(count), C.c_float(a), C.c_float(b))
    return out


def q8_quantize(w):
    n, k = w.shape
    w = np.ascontiguousarray(w, dtype=np.float32)
    q = np.empty((n, k), np.int8)
    s = np.empty((n, k // 32), np.float32)
    lib().orc_q8_quantize(_p(w), _p(q), _p(s), C.c_int64(n), C.c_int64(k))
    return q, s


def q8_synth_weights(n, k, seed, stream, std, row0=0, col0=0, k_total=None):
    q = np.empty((n, k), np.int8)
    s = np.empty((n, k // 32), np.float32)
    lib().orc_q8_synth_weights(_p(q), _p(s), C.c_int64(n), C.c_int64(k), C.c_int64(row0), C.c_int64(col0),
                               C.c_int64(k if k_total is None else k_total), C.c_uint64(seed),
                               C.c_uint64(stream), C.c_float(std))
    return q, s


def q8_gemv(q, s, x):
    n, k = q.shape
    y = np.empty(n, np.float32)
    lib().orc_q8_gemv(_p(q), _p(s), _p(np.ascontiguousarray(x, np.float32)), _p(y), C.c_int64(n), C.c_int64(k))
    return y


def q8_gemm(a_bf16, q, s, epilogue=0, aux=None):
    m, k = a_bf16.shape
    n = q.shape[0]
    c = np.empty((m, n // 2 if epilogue == 2 else n), np.uint16)
    lib().orc_q8_gemm(_p(a_bf16), _p(q), _p(s), _p(c), C.c_int64(m), C.c_int64(n), C.c_int64(k),
                      C.c_int(epilogue), _p(aux) if aux is not None else None)
    return c


def q8_gemm_f32(a, a_dtype, q, s):
    m, k = a.shape
    n = q.shape[0]
    c = np.empty((m, n), np.float32)
    lib().orc_q8_gemm_f32(_p(a), C.c_int(a_dtype), _p(q), _p(s), _p(c), C.c_int64(m), C.c_int64(n), C.c_int64(k))
    return c


def rope_table(l_max, d, theta):
    out = np.empty((l_max, d // 2, 2), np.float32)
    lib().orc_rope_table(_p(out), C.c_int64(l_max), C.c_int64(d), C.c_double(theta))
    return out


def kv_append_rope(k_cache, v_cache, k_new, v_new, tab, seq_len):
    b, h_kv, l_max, d = k_cache.shape
    lib().orc_kv_append_rope(_p(k_cache), _p(v_cache), _p(k_new), _p(v_new), _p(tab), _p(seq_len),
                             C.c_int64(b), C.c_int64(h_kv), C.c_int64(d), C.c_int64(l_max))


def gqa_decode_attn(q, k_cache, v_cache, seq_len, scale):
    b, h_q, d = q.shape
    _, h_kv, l_max, _ = k_cache.shape
    o = np.empty((b, h_q, d), np.uint16)
    lib().orc_gqa_decode_attn(_p(q), _p(k_cache), _p(v_cache), _p(seq_len), _p(o), C.c_int64(b), C.c_int64(h_q),
                              C.c_int64(h_kv), C.c_int64(d), C.c_int64(l_max), C.c_float(scale))
    return o


def gqa_decode_attn_fused(q_raw, k_new, v_new, k_cache, v_cache, tab, seq_len, scale):
    b, h_q, d = q_raw.shape
    _, h_kv, l_max, _ = k_cache.shape
    o = np.empty((b, h_q, d), np.uint16)
    lib().orc_gqa_decode_attn_fused(_p(q_raw), _p(k_new), _p(v_new), _p(k_cache), _p(v_cache), _p(tab),
                                    _p(seq_len), _p(o), C.c_int64(b), C.c_int64(h_q), C.c_int64(h_kv),
                                    C.c_int64(d), C.c_int64(l_max), C.c_float(scale))
    return o


def sample_rows(logits, temperature, seed, positions, top_k=0):
    """Next token per row by Gumbel-max on the seeded generator (temperature 0: plain argmax),
    over the logits that reach the row's top_k-th largest when top_k > 0."""
    logits = np.ascontiguousarray(logits, np.float32)
    rows, vocab = logits.shape
    pos = np.ascontiguousarray(positions, np.int32)
    out = np.empty(rows, np.int32)
    on = 1 if temperature > 0 else 0
    inv = np.float32(1.0) / np.float32(temperature) if on else np.float32(1.0)
    lib().orc_sample_rows(_p(logits), C.c_int64(rows), C.c_int64(vocab), C.c_int(on), C.c_float(inv), C.c_int64(top_k),
                          C.c_uint64(seed), _p(pos), _p(out))
    return out


def rmsnorm(x, g, eps):
    rows, h = x.shape
    y = np.empty((rows, h), np.float32)
    lib().orc_rmsnorm(_p(np.ascontiguousarray(x, np.float32)), _p(g), _p(y), C.c_int64(rows), C.c_int64(h),
                      C.c_float(eps))
    return y


def swiglu(gate, up):
    y = np.empty(gate.shape, np.float32)
    lib().orc_swiglu(_p(gate), _p(up), _p(y), C.c_int64(gate.size))
    return y


def f32_to_bf16(a):
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_to_f32(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def f32_to_f16(a):
    return np.ascontiguousarray(a, np.float32).astype(np.float16).view(np.uint16)


def f16_to_f32(h):
    return h.view(np.float16).astype(np.float32)


class Llm:
    """The oracle's model: unsharded, same seeded weights as the library's."""

    def __init__(self, **kw):
        self.cfg = LlmConfig(**kw)
        self._h = C.c_void_p(lib().orc_llm_create(C.byref(self.cfg)))

    def close(self):
        if self._h:
            lib().orc_llm_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def prefill(self, tokens):
        tokens = np.ascontiguousarray(tokens, np.int32)
        lib().orc_llm_prefill(self._h, _p(tokens), C.c_int64(tokens.shape[1]))

    def prefill_ragged(self, tokens, lens):
        """tokens [B][t_max]; sequence i consumes tokens[i, :lens[i]]."""
        tokens = np.ascontiguousarray(tokens, np.int32)
        lens = np.ascontiguousarray(lens, np.int32)
        lib().orc_llm_prefill_ragged(self._h, _p(tokens), C.c_int64(tokens.shape[1]), _p(lens))

    def synth_kv(self, t, seed=0):
        lib().orc_llm_synth_kv(self._h, C.c_int64(t), C.c_uint64(seed))

    def set_tokens(self, tokens):
        lib().orc_llm_set_tokens(self._h, _p(np.ascontiguousarray(tokens, np.int32)))

    def decode_step(self):
        out = np.empty(self.cfg.batch, np.int32)
        lib().orc_llm_decode_step(self._h, _p(out))
        return out

    def read_kv(self, layer):
        c = self.cfg
        shape = (c.batch, c.h_kv, c.l_max, c.head_dim)
        k = np.empty(shape, np.uint16)
        v = np.empty(shape, np.uint16)
        lib().orc_llm_read_kv(self._h, C.c_int64(layer), _p(k), _p(v))
        return k, v

    def _tensor_shape(self, kind):
        c = self.cfg
        nq, nkv = c.h_q * c.head_dim, c.h_kv * c.head_dim
        return {1: (nq, c.hidden), 2: (nkv, c.hidden), 3: (nkv, c.hidden), 4: (c.hidden, nq), 6: (c.ffn, c.hidden),
                7: (c.ffn, c.hidden), 8: (c.hidden, c.ffn), 10: (c.vocab, c.hidden), 11: (c.vocab, c.hidden)}.get(kind)

    def _vector_len(self, kind):
        c = self.cfg
        return {12: c.h_q * c.head_dim, 13: c.h_kv * c.head_dim, 14: c.h_kv * c.head_dim}.get(kind, c.hidden)

    def get_tensor(self, layer, kind):
        """A tensor by the weight file's numbering (0 attn_norm, 1 q, 2 k, 3 v, 4 o, 5 mlp_norm, 6 gate,
        7 up, 8 down, 9 final_norm, 10 embed, 11 head, 12 q_bias, 13 k_bias, 14 v_bias): (q, s) for a matrix,
        an f32 vector for a gain or a bias."""
        shape = self._tensor_shape(kind)
        if shape is None:
            g = np.empty(self._vector_len(kind), np.float32)
            if lib().orc_llm_get_tensor(self._h, C.c_int64(layer), C.c_int(kind), _p(g), None) != 0:
                raise KeyError((layer, kind))
            return g
        q = np.empty(shape, np.int8)
        s = np.empty((shape[0], shape[1] // 32), np.float32)
        if lib().orc_llm_get_tensor(self._h, C.c_int64(layer), C.c_int(kind), _p(q), _p(s)) != 0:
            raise KeyError((layer, kind))
        return q, s

    def set_tensor(self, layer, kind, q, s=None):
        shape = self._tensor_shape(kind)
        if shape is None:
            g = np.ascontiguousarray(q, np.float32).reshape(self._vector_len(kind))
            rc = lib().orc_llm_set_tensor(self._h, C.c_int64(layer), C.c_int(kind), _p(g), None)
        else:
            q = np.ascontiguousarray(q, np.int8).reshape(shape)
            s = np.ascontiguousarray(s, np.float32).reshape(shape[0], shape[1] // 32)
            rc = lib().orc_llm_set_tensor(self._h, C.c_int64(layer), C.c_int(kind), _p(q), _p(s))
        if rc != 0:
            raise KeyError((layer, kind))

    def set_sampling(self, temperature, seed=0, top_k=0):
        lib().orc_llm_set_sampling(self._h, C.c_float(temperature), C.c_int64(top_k), C.c_uint64(seed))

    def read_logits(self):
        out = np.empty((self.cfg.batch, self.cfg.vocab), np.float32)
        lib().orc_llm_read_logits(self._h, _p(out))
        return out

    def read_seq_len(self):
        out = np.empty(self.cfg.batch, np.int32)
        lib().orc_llm_read_seq_len(self._h, _p(out))
        return out

    def set_seq_len(self, t):
        lib().orc_llm_set_seq_len(self._h, C.c_int64(t))
