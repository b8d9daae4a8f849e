"""Loader and ctypes signatures for liblogos_b200.so (include/logos_b200.h).

There is no fallback: if the shared library is missing the import of any
operator raises, and if it is present but no CUDA device is visible every
compute call returns an error status that is raised as LogosError.
"""
import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
# LOGOS_B200_LIBRARY names another build of the same library (same header), e.g. one compiled with other flags
LIB_PATH = os.environ.get("LOGOS_B200_LIBRARY") or os.path.join(_HERE, "liblogos_b200.so")
HEADER_PATH = os.path.join(_HERE, "..", "include", "logos_b200.h")

# LogosStatus (crates/logicaffeine_compile/src/codegen/ffi.rs:196-209)
STATUS_NAMES = {
    0: "Ok", 1: "Error", 2: "RefinementViolation", 3: "NullPointer", 4: "OutOfBounds",
    5: "DeserializationFailed", 6: "InvalidHandle", 7: "ContainsNullByte", 8: "ThreadPanic",
    9: "MemoryExhausted",
}

F32, F16, BF16, I8, I32 = 0, 1, 2, 3, 4


class LogosError(RuntimeError):
    def __init__(self, status, message):
        self.status = status
        self.status_name = STATUS_NAMES.get(status, str(status))
        super().__init__("LogosStatus::%s: %s" % (self.status_name, message))


class LlmConfig(C.Structure):
    """logos_llm_config_t"""
    _fields_ = [
        ("layers", C.c_int64), ("hidden", C.c_int64), ("h_q", C.c_int64), ("h_kv", C.c_int64),
        ("head_dim", C.c_int64), ("ffn", C.c_int64), ("vocab", C.c_int64), ("l_max", C.c_int64),
        ("batch", C.c_int64),
        ("rms_eps", C.c_float), ("rope_theta", C.c_float),
        ("tied_embeddings", C.c_int32), ("tp_degree", C.c_int32), ("tp_rank", C.c_int32),
        ("device", C.c_int32), ("act_dtype", C.c_int32),
        ("seed", C.c_uint64), ("init_std", C.c_float), ("qkv_bias", C.c_int32),
    ]


H = C.c_void_p   # logos_handle_t
I64 = C.c_int64
I32c = C.c_int32
U64 = C.c_uint64
FLT = C.c_float
PTR = C.c_void_p

# name -> (restype, argtypes); restype None means logos_status_t
_SIGNATURES = {
    "logos_b200_last_error": (C.c_char_p, []),
    "logos_b200_get_last_error": (C.c_char_p, []),
    "logos_b200_clear_error": (None.__class__, []),
    "logos_b200_free_string": (None.__class__, [C.c_char_p]),
    "logos_b200_abi_version": (C.c_uint32, []),
    "logos_b200_version": (C.c_char_p, []),
    "logos_free_string": (None.__class__, [C.c_char_p]),
    "logos_last_error": (C.c_char_p, []),
    "logos_get_last_error": (C.c_char_p, []),
    "logos_clear_error": (None.__class__, []),
    "logos_abi_version": (C.c_uint32, []),
    "logos_version": (C.c_char_p, []),
    "logos_device_count": (C.c_int32, []),
    "logos_dev_alloc": (None, [I64, I32c, C.POINTER(H)]),
    "logos_dev_upload": (None, [H, I64, PTR, I64]),
    "logos_dev_download": (None, [PTR, H, I64, I64]),
    "logos_dev_memset": (None, [H, I32c, I64]),
    "logos_dev_ptr": (None, [H, C.POINTER(PTR), C.POINTER(I64)]),
    "logos_dev_sync": (None, [I32c]),
    "logos_dev_mem_info": (None, [I32c, C.POINTER(I64), C.POINTER(I64)]),
    "logos_dev_free": (None, [H]),
    "logos_kernel_status": (None, [I32c, C.POINTER(I32c)]),
    "logos_launch_counts": (None, [C.POINTER(I64)]),
    "logos_synth_fill": (None, [H, I64, I32c, I32c, U64, U64, I64, I64, FLT, FLT, PTR]),
    "logos_q8_quantize": (None, [H, H, H, I64, I64, PTR]),
    "logos_q8_synth_weights": (None, [H, H, I64, I64, I64, U64, U64, FLT, PTR]),
    "logos_q8_gemv": (None, [H, H, H, H, I64, I64, PTR]),
    "logos_q8_gemm": (None, [H, H, H, H, I64, I64, I64, I32c, H, PTR]),
    "logos_q8_gemm_f32": (None, [H, H, H, H, I64, I64, I64, PTR]),
    "logos_q8_gemm_simt": (None, [H, H, H, H, I64, I64, I64, I32c, H, PTR]),
    "logos_rope_table": (None, [PTR, I64, I64, C.c_double]),
    "logos_kv_append_rope": (None, [H, H, H, H, H, H, I64, I64, I64, I64, PTR]),
    "logos_gqa_decode_attn": (None, [H, H, H, H, H, I64, I64, I64, I64, I64, FLT, PTR]),
    "logos_gqa_decode_attn_fixed_scratch": (None, [H, H, H, H, H, I64, I64, I64, I64, I64, FLT, PTR]),
    "logos_gqa_decode_attn_fused": (None, [H, H, H, H, H, H, H, H, I64, I64, I64, I64, I64, FLT, PTR]),
    "logos_rmsnorm": (None, [H, H, H, I64, I64, FLT, PTR]),
    "logos_swiglu": (None, [H, H, H, I64, PTR]),
    "logos_tp_unique_id": (None, [PTR]),
    "logos_llm_create": (None, [C.POINTER(LlmConfig), PTR, C.POINTER(H)]),
    "logos_llm_get_config": (None, [H, C.POINTER(LlmConfig)]),
    "logos_llm_prefill": (None, [H, PTR, I64]),
    "logos_llm_prefill_ragged": (None, [H, PTR, I64, PTR]),
    "logos_llm_synth_kv": (None, [H, I64, U64]),
    "logos_llm_set_tokens": (None, [H, PTR]),
    "logos_llm_decode_step": (None, [H, PTR]),
    "logos_llm_decode_steps": (None, [H, I64, PTR]),
    "logos_llm_read_kv": (None, [H, I64, PTR, PTR]),
    "logos_llm_read_logits": (None, [H, PTR]),
    "logos_llm_read_seq_len": (None, [H, PTR]),
    "logos_llm_set_seq_len": (None, [H, I64]),
    "logos_llm_set_sampling": (None, [H, FLT, I64, U64]),
    "logos_llm_last_timing": (None, [H, C.POINTER(C.c_double), C.POINTER(I64)]),
    "logos_llm_tp_exchange": (None, [H, C.POINTER(C.c_int32)]),
    "logos_dependent_launch_scope": (None, [C.c_int32, C.POINTER(C.c_int32)]),
    "logos_llm_profile_step": (None, [H, C.POINTER(C.c_double)]),
    "logos_llm_weights_file_bytes": (None, [C.POINTER(LlmConfig), C.POINTER(I64)]),
    "logos_llm_weights_span": (None, [C.POINTER(LlmConfig), I64, I32c, C.POINTER(I64), C.POINTER(I64), C.POINTER(I64),
                               C.POINTER(I64)]),
    "logos_llm_weights_header": (None, [C.POINTER(LlmConfig), PTR]),
    "logos_llm_weights_check": (None, [C.c_char_p, C.POINTER(LlmConfig)]),
    "logos_llm_weights_read_shard": (None, [C.c_char_p, I32c, I32c, I64, I32c, PTR, I64, PTR, I64, C.POINTER(I64),
                                     C.POINTER(I64)]),
    "logos_llm_load_weights": (None, [H, C.c_char_p]),
    "logos_llm_save_weights": (None, [H, C.c_char_p]),
    "logos_llm_free": (None, [H]),
}


def header_symbols():
    """Every function the public header declares."""
    with open(HEADER_PATH) as f:
        text = f.read()
    return sorted(set(re.findall(r"LOGOS_API[^;(]*?\b(logos_[a-z0-9_]+)\s*\(", text)))


_lib = None


def load():
    """Load the shared library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "liblogos_b200.so is missing: build it with `python -m logicaffeine_b200.build` "
            "(there is no CPU or PyTorch fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        if res is None:
            fn.restype = C.c_int
        elif res is type(None):
            fn.restype = None
        else:
            fn.restype = res
    _lib = lib
    return lib


def check(status):
    if status != 0:
        msg = load().logos_b200_last_error()
        raise LogosError(status, msg.decode() if msg else "(no message)")


def call(name, *args):
    """Call a status-returning entry point and raise LogosError on failure."""
    check(getattr(load(), name)(*args))
