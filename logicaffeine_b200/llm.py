"""Host-side mirror of the LOGOS operator family `llm` over the C ABI.

In the reference a native operator is declared in LOGOS as
`## To native mlkemNtt (a: Seq of Int) -> Seq of Int`
(crates/logicaffeine_compile/assets/std/crypto.lg:120), lowered by name through
`map_native_function` to `logicaffeine_system::<module>::<fn>`
(crates/logicaffeine_compile/src/codegen/program.rs:1517-1522,1936-2003) and
implemented as a thin function over slices
(crates/logicaffeine_system/src/ntt.rs:330-335).  The functions below are that
layer for the new `llm` module, with the same camelCase operator names a LOGOS
program would use; tensors travel as opaque device handles (LOGOS `Int`), never
as `Seq of Real`.  Errors surface as LogosError carrying the LogosStatus code,
where the Rust wrapper would return `Err`.
"""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import BF16, F16, F32, I8, I32, LlmConfig, LogosError, call, load  # noqa: F401

EPI_NONE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2


def deviceCount():
    return int(load().logos_device_count())


def abiVersion():
    return int(load().logos_b200_abi_version())


def devMemInfo(device=0):
    """(free, total) bytes of device memory as the driver reports them."""
    f, t = C.c_int64(), C.c_int64()
    call("logos_dev_mem_info", int(device), C.byref(f), C.byref(t))
    return f.value, t.value


def _host_ptr(a):
    return a.ctypes.data_as(C.c_void_p)


class DeviceBuffer:
    """An owned device allocation behind a logos_handle_t id."""

    def __init__(self, nbytes, device=0):
        h = _lib.H()
        call("logos_dev_alloc", int(nbytes), int(device), C.byref(h))
        self.handle = h
        self.nbytes = int(nbytes)
        self.device = int(device)

    @classmethod
    def from_host(cls, array, device=0):
        array = np.ascontiguousarray(array)
        buf = cls(array.nbytes, device)
        buf.upload(array)
        return buf

    def upload(self, array, offset=0):
        array = np.ascontiguousarray(array)
        call("logos_dev_upload", self.handle, int(offset), _host_ptr(array), array.nbytes)

    def download(self, dtype, shape, offset=0):
        out = np.empty(shape, dtype=dtype)
        call("logos_dev_download", _host_ptr(out), self.handle, int(offset), out.nbytes)
        return out

    def memset(self, byte_value=0):
        call("logos_dev_memset", self.handle, int(byte_value), self.nbytes)

    def ptr(self):
        p = C.c_void_p()
        n = C.c_int64()
        call("logos_dev_ptr", self.handle, C.byref(p), C.byref(n))
        return p.value

    def free(self):
        if self.handle is not None:
            call("logos_dev_free", self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def devSync(device=0):
    call("logos_dev_sync", int(device))


def kernelStatus(device=0):
    code = C.c_int32()
    call("logos_kernel_status", int(device), C.byref(code))
    return code.value


def launchCounts():
    """Kernel launches made through the library so far, by kind."""
    out = (C.c_int64 * 8)()
    call("logos_launch_counts", out)
    names = ("q8_gemv", "q8_gemm_tc", "q8_gemm_simt", "attention", "attention_merge", "elementwise", "synth")
    return dict(zip(names, (int(v) for v in out)))


def _h(buf):
    return buf.handle if buf is not None else None


def _s(stream):
    return C.c_void_p(stream) if stream else None


# ---------------------------------------------------------------- synthetic inputs
def synthFill(dst, dtype, kind, seed, stream_id, first, count, a=0.0, b=1.0, offset_bytes=0, stream=None):
    call("logos_synth_fill", dst.handle, int(offset_bytes), int(dtype), int(kind), int(seed), int(stream_id),
         int(first), int(count), float(a), float(b), _s(stream))


def q8Quantize(w, q, s, n, k, stream=None):
    call("logos_q8_quantize", w.handle, q.handle, s.handle, int(n), int(k), _s(stream))


def q8SynthWeights(q, s, n, k, row0, seed, stream_id, std, stream=None):
    call("logos_q8_synth_weights", q.handle, s.handle, int(n), int(k), int(row0), int(seed), int(stream_id),
         float(std), _s(stream))


# ---------------------------------------------------------------- single operators
def q8Gemv(q, s, x, y, n, k, stream=None):
    call("logos_q8_gemv", q.handle, s.handle, x.handle, y.handle, int(n), int(k), _s(stream))


def q8Gemm(a, q, s, c, m, n, k, epilogue=EPI_NONE, aux=None, stream=None):
    call("logos_q8_gemm", a.handle, q.handle, s.handle, c.handle, int(m), int(n), int(k), int(epilogue), _h(aux),
         _s(stream))


def dependentLaunchScope(on):
    """Open or close the calling thread's dependent-launch scope; returns the previous setting."""
    prev = C.c_int32()
    call("logos_dependent_launch_scope", 1 if on else 0, C.byref(prev))
    return bool(prev.value)


def q8GemmF32(a, q, s, c, m, n, k, stream=None):
    call("logos_q8_gemm_f32", a.handle, q.handle, s.handle, c.handle, int(m), int(n), int(k), _s(stream))


def q8GemmSimt(a, q, s, c, m, n, k, epilogue=EPI_NONE, aux=None, stream=None):
    call("logos_q8_gemm_simt", a.handle, q.handle, s.handle, c.handle, int(m), int(n), int(k), int(epilogue),
         _h(aux), _s(stream))


def ropeTable(l_max, d, theta):
    out = np.empty((l_max, d // 2, 2), np.float32)
    call("logos_rope_table", _host_ptr(out), int(l_max), int(d), float(theta))
    return out


def kvAppendRope(k_cache, v_cache, k_new, v_new, rope_table, seq_len, b, h_kv, d, l_max, stream=None):
    call("logos_kv_append_rope", k_cache.handle, v_cache.handle, k_new.handle, v_new.handle, rope_table.handle,
         seq_len.handle, int(b), int(h_kv), int(d), int(l_max), _s(stream))


def gqaDecodeAttn(q, k_cache, v_cache, seq_len, o, b, h_q, h_kv, d, l_max, softmax_scale, stream=None):
    call("logos_gqa_decode_attn", q.handle, k_cache.handle, v_cache.handle, seq_len.handle, o.handle, int(b),
         int(h_q), int(h_kv), int(d), int(l_max), float(softmax_scale), _s(stream))


def gqaDecodeAttnFixedScratch(q, k_cache, v_cache, seq_len, o, b, h_q, h_kv, d, l_max, softmax_scale, stream=None):
    """gqaDecodeAttn for hosts that cannot let an operator allocate device memory: the split-KV partials use a
    fixed 16 MiB array inside the library; larger shapes raise LogosError (OutOfBounds)."""
    call("logos_gqa_decode_attn_fixed_scratch", q.handle, k_cache.handle, v_cache.handle, seq_len.handle, o.handle,
         int(b), int(h_q), int(h_kv), int(d), int(l_max), float(softmax_scale), _s(stream))


def gqaDecodeAttnFused(q_raw, k_new, v_new, k_cache, v_cache, rope_table, seq_len, o, b, h_q, h_kv, d, l_max,
                       softmax_scale, stream=None):
    call("logos_gqa_decode_attn_fused", q_raw.handle, k_new.handle, v_new.handle, k_cache.handle, v_cache.handle,
         rope_table.handle, seq_len.handle, o.handle, int(b), int(h_q), int(h_kv), int(d), int(l_max),
         float(softmax_scale), _s(stream))


def rmsNorm(x, g, y, rows, h, eps, stream=None):
    call("logos_rmsnorm", x.handle, g.handle, y.handle, int(rows), int(h), float(eps), _s(stream))


def swiGlu(gate, up, y, count, stream=None):
    call("logos_swiglu", gate.handle, up.handle, y.handle, int(count), _s(stream))


# ---------------------------------------------------------------- host-buffer forms
# The call a host program makes when its data lives in host memory: copy in,
# run, copy out.  These are what the end-to-end numbers time.
def q8GemvHost(q, s, x, device=0):
    n, k = q.shape
    dq, ds, dx = (DeviceBuffer.from_host(a, device) for a in (q, s, np.asarray(x, np.float32)))
    dy = DeviceBuffer(n * 4, device)
    q8Gemv(dq, ds, dx, dy, n, k)
    y = dy.download(np.float32, (n,))
    for b in (dq, ds, dx, dy):
        b.free()
    return y


def q8GemmHost(a_bf16, q, s, epilogue=EPI_NONE, aux=None, device=0, simt=False):
    m, k = a_bf16.shape
    n = q.shape[0]
    n_out = n // 2 if epilogue == EPI_SWIGLU else n
    da, dq, ds = (DeviceBuffer.from_host(t, device) for t in (a_bf16, q, s))
    dx = DeviceBuffer.from_host(aux, device) if aux is not None else None
    dc = DeviceBuffer(m * n_out * 2, device)
    (q8GemmSimt if simt else q8Gemm)(da, dq, ds, dc, m, n, k, epilogue, dx)
    c = dc.download(np.uint16, (m, n_out))
    for b in (da, dq, ds, dc, dx):
        if b is not None:
            b.free()
    return c


def q8GemmF32Host(a_f32, q, s, device=0):
    m, k = a_f32.shape
    n = q.shape[0]
    da, dq, ds = (DeviceBuffer.from_host(t, device) for t in (np.asarray(a_f32, np.float32), q, s))
    dc = DeviceBuffer(m * n * 4, device)
    q8GemmF32(da, dq, ds, dc, m, n, k)
    c = dc.download(np.float32, (m, n))
    for b in (da, dq, ds, dc):
        b.free()
    return c


# ---------------------------------------------------------------- model level
def tpUniqueId():
    buf = (C.c_uint8 * 128)()
    call("logos_tp_unique_id", C.cast(buf, C.c_void_p))
    return bytes(buf)


class Llm:
    """llmCreate / llmPrefill / llmDecodeStep / llmFree over one model handle."""

    def __init__(self, nccl_unique_id=None, **cfg):
        defaults = dict(rms_eps=1e-6, rope_theta=1e6, tied_embeddings=1, tp_degree=1, tp_rank=0, device=0,
                        act_dtype=F32, seed=0, init_std=0.02, qkv_bias=0)
        defaults.update(cfg)
        self.cfg = LlmConfig(**defaults)
        h = _lib.H()
        idbuf = None
        if nccl_unique_id is not None:
            idbuf = (C.c_uint8 * 128).from_buffer_copy(nccl_unique_id)
        call("logos_llm_create", C.byref(self.cfg), C.cast(idbuf, C.c_void_p) if idbuf is not None else None,
             C.byref(h))
        self.handle = h

    def prefill(self, tokens):
        tokens = np.ascontiguousarray(tokens, np.int32)
        assert tokens.shape[0] == self.cfg.batch
        call("logos_llm_prefill", self.handle, _host_ptr(tokens), int(tokens.shape[1]))

    def prefillRagged(self, tokens, lens):
        """tokens [B][t_max]; sequence b consumes tokens[b, :lens[b]] (0 <= lens[b] <= t_max);
        lens[b] == -1 keeps sequence b as it is while other slots take new prompts."""
        tokens = np.ascontiguousarray(tokens, np.int32)
        lens = np.ascontiguousarray(lens, np.int32)
        assert tokens.shape[0] == self.cfg.batch and lens.shape == (self.cfg.batch,)
        call("logos_llm_prefill_ragged", self.handle, _host_ptr(tokens), int(tokens.shape[1]), _host_ptr(lens))

    def synthKv(self, t, seed=0):
        call("logos_llm_synth_kv", self.handle, int(t), int(seed))

    def setTokens(self, tokens):
        tokens = np.ascontiguousarray(tokens, np.int32)
        call("logos_llm_set_tokens", self.handle, _host_ptr(tokens))

    def decodeStep(self):
        out = np.empty(self.cfg.batch, np.int32)
        call("logos_llm_decode_step", self.handle, _host_ptr(out))
        return out

    def decodeSteps(self, steps, read_back=True):
        out = np.empty((steps, self.cfg.batch), np.int32) if read_back else None
        call("logos_llm_decode_steps", self.handle, int(steps), _host_ptr(out) if read_back else None)
        return out

    def readKv(self, layer):
        c = self.cfg
        shape = (c.batch, c.h_kv // c.tp_degree, c.l_max, c.head_dim)
        k = np.empty(shape, np.uint16)
        v = np.empty(shape, np.uint16)
        call("logos_llm_read_kv", self.handle, int(layer), _host_ptr(k), _host_ptr(v))
        return k, v

    def readLogits(self):
        out = np.empty((self.cfg.batch, self.cfg.vocab), np.float32)
        call("logos_llm_read_logits", self.handle, _host_ptr(out))
        return out

    def readSeqLen(self):
        out = np.empty(self.cfg.batch, np.int32)
        call("logos_llm_read_seq_len", self.handle, _host_ptr(out))
        return out

    def setSeqLen(self, t):
        call("logos_llm_set_seq_len", self.handle, int(t))

    def setSampling(self, temperature, seed=0, top_k=0):
        """Temperature sampling by Gumbel-max on the seeded generator, over the top_k largest logits
        when top_k > 0; temperature 0 is greedy."""
        call("logos_llm_set_sampling", self.handle, float(temperature), int(top_k), int(seed))

    def lastTiming(self):
        ms = C.c_double()
        launches = C.c_int64()
        call("logos_llm_last_timing", self.handle, C.byref(ms), C.byref(launches))
        return ms.value, launches.value

    def config(self):
        """The logos_llm_config_t the model was created with, as a dict."""
        cfg = LlmConfig()
        call("logos_llm_get_config", self.handle, C.byref(cfg))
        return {name: getattr(cfg, name) for name, _ in LlmConfig._fields_}

    def tpExchange(self):
        """0 = no TP group, 1 = NCCL all-reduce, 2 = exchange folded into residual + RMSNorm over peer memory."""
        mode = C.c_int32()
        call("logos_llm_tp_exchange", self.handle, C.byref(mode))
        return mode.value

    def loadWeights(self, path):
        """Replace weights and norm gains with this rank's part of a weight file (weights.py)."""
        call("logos_llm_load_weights", self.handle, str(path).encode())

    def saveWeights(self, path):
        """Write the model's weights and gains as a weight file (tp_degree 1 only)."""
        call("logos_llm_save_weights", self.handle, str(path).encode())

    def profileStep(self):
        """One step with per-class device timing: ms for (gemm, attention, elementwise, exchange)."""
        ms = (C.c_double * 4)()
        call("logos_llm_profile_step", self.handle, ms)
        return dict(zip(("q8_gemm", "attention", "elementwise", "exchange"), (float(v) for v in ms)))

    def free(self):
        if self.handle is not None:
            call("logos_llm_free", self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def llmCreate(**cfg):
    return Llm(**cfg)


def llmPrefill(model, tokens):
    model.prefill(tokens)


def llmDecodeStep(model):
    return model.decodeStep()


def llmDecodeSteps(model, steps):
    return model.decodeSteps(steps)


def llmLoadWeights(model, path):
    model.loadWeights(path)


def llmFree(model):
    model.free()
