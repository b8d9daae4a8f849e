"""The C-ABI library without a GPU: it loads, exports every symbol the public
header declares, follows the reference's status / last-error / handle
conventions (crates/logicaffeine_compile/src/codegen/ffi.rs:196-264,288-324),
and refuses compute loudly instead of falling back to a CPU path."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from logicaffeine_b200 import _lib


def test_library_exports_every_declared_symbol(llm):
    lib = _lib.load()
    names = _lib.header_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), "header declares %s but the library does not export it" % n
    assert set(names) == set(_lib._SIGNATURES), "ctypes table and header differ"


def test_only_logos_symbols_are_exported():
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True).stdout
    syms = [l.split()[-1] for l in out.splitlines() if " T " in l]
    assert syms and all(s.startswith("logos_") for s in syms), [s for s in syms if not s.startswith("logos_")][:5]


def test_status_codes_match_the_reference_enum():
    text = open(_lib.HEADER_PATH).read()
    want = {"OK": 0, "ERROR": 1, "REFINEMENT_VIOLATION": 2, "NULL_POINTER": 3, "OUT_OF_BOUNDS": 4,
            "DESERIALIZATION_FAILED": 5, "INVALID_HANDLE": 6, "CONTAINS_NULL_BYTE": 7, "THREAD_PANIC": 8,
            "MEMORY_EXHAUSTED": 9}
    # the enumerator spelling of the C header the reference generates
    # (crates/logicaffeine_compile/src/codegen/ffi.rs:1364-1375): LOGOS_STATUS_<NAME> = <code>
    for k, v in want.items():
        assert re.search(r"\bLOGOS_STATUS_%s\s*=\s*%d\b" % (k, v), text), k
        assert re.search(r"#define\s+LOGOS_%s\s+LOGOS_STATUS_%s\b" % (k, k), text), k
    assert re.search(r"typedef\s+void\s*\*\s*logos_handle_t\s*;", text)
    assert re.search(r"#define\s+LOGOS_ABI_VERSION\s+1\b", text)


def test_runtime_names_of_the_reference_preamble_and_the_library_prefix(llm):
    """The preamble names of ffi.rs:1377-1384 are exported (weak) next to the library's own
    logos_b200_ copies; both read the same per-thread store; logos_free_string takes NULL."""
    import subprocess
    lib = _lib.load()
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True).stdout
    kinds = {l.split()[-1]: l.split()[-2] for l in out.splitlines() if len(l.split()) >= 3}
    for n in ("last_error", "get_last_error", "clear_error", "free_string", "abi_version", "version"):
        assert kinds.get("logos_" + n) == "W", (n, kinds.get("logos_" + n))
        assert kinds.get("logos_b200_" + n) == "T", (n, kinds.get("logos_b200_" + n))
    assert lib.logos_dev_alloc(16, 0, None) == 3
    assert lib.logos_b200_last_error() == lib.logos_last_error() == lib.logos_b200_get_last_error()
    lib.logos_b200_clear_error()
    assert lib.logos_last_error() is None and lib.logos_b200_last_error() is None
    lib.logos_free_string(None)
    lib.logos_b200_free_string(None)
    assert lib.logos_b200_abi_version() == lib.logos_abi_version() == 1


def test_version_and_abi(llm):
    assert llm.abiVersion() == 1
    assert _lib.load().logos_version().decode().startswith("0.")


def test_config_struct_layout_matches_header():
    # 9 int64, 2 float, 5 int32, pad, uint64, float, int32
    assert C.sizeof(_lib.LlmConfig) == 9 * 8 + 2 * 4 + 5 * 4 + 4 + 8 + 4 + 4
    assert _lib.LlmConfig.seed.offset == 104 and _lib.LlmConfig.init_std.offset == 112


def test_null_and_invalid_handles(llm):
    lib = _lib.load()
    assert lib.logos_dev_alloc(16, 0, None) == 3  # NullPointer before any work
    assert b"null" in lib.logos_last_error()
    lib.logos_clear_error()
    assert lib.logos_last_error() is None
    assert lib.logos_dev_free(C.c_void_p(12345)) == 6  # InvalidHandle, not UB
    assert lib.logos_dev_free(None) == 3
    assert lib.logos_llm_free(C.c_void_p(777)) == 6
    assert lib.logos_q8_gemv(C.c_void_p(1), C.c_void_p(2), C.c_void_p(3), C.c_void_p(4), 4, 32, None) == 6
    assert lib.logos_q8_gemv(None, None, None, None, 4, 32, None) == 3
    assert lib.logos_q8_gemv(None, None, None, None, 4, 33, None) == 4  # K not a multiple of 32
    assert lib.logos_llm_create(None, None, None) == 3
    # model-level entry points added later: the handle is checked before anything else
    for call in (lambda h: lib.logos_llm_load_weights(h, b"/nonexistent"),
                 lambda h: lib.logos_llm_save_weights(h, b"/nonexistent"),
                 lambda h: lib.logos_llm_set_sampling(h, 1.0, 0, 0),
                 lambda h: lib.logos_llm_prefill_ragged(h, None, 1, None)):
        assert call(None) == 3
        assert call(C.c_void_p(777)) == 6
    assert lib.logos_llm_weights_check(None, None) == 3
    assert lib.logos_llm_weights_file_bytes(None, None) == 3
    assert lib.logos_llm_weights_header(None, None) == 3
    assert lib.logos_llm_weights_read_shard(None, 1, 0, 0, 1, None, 0, None, 0, None, None) == 3
    assert lib.logos_get_last_error() == lib.logos_last_error()


def test_error_state_is_per_thread(llm):
    import threading
    lib = _lib.load()
    lib.logos_clear_error()
    seen = {}

    def worker():
        lib.logos_dev_free(C.c_void_p(999))
        seen["worker"] = lib.logos_last_error()

    t = threading.Thread(target=worker)
    t.start()
    t.join()
    assert seen["worker"] is not None
    assert lib.logos_last_error() is None


def test_rope_table_is_host_side_and_matches_the_oracle(llm, oracle):
    tab = llm.ropeTable(33, 128, 1e6)
    assert np.array_equal(tab.view(np.uint32), oracle.rope_table(33, 128, 1e6).view(np.uint32))


@pytest.mark.skipif(_lib.load().logos_device_count() > 0, reason="checks the no-GPU behaviour")
def test_no_cpu_fallback(llm):
    with pytest.raises(llm.LogosError) as e:
        llm.DeviceBuffer(64)
    assert e.value.status == 1 and "no CUDA device" in str(e.value)
    with pytest.raises(llm.LogosError):
        llm.Llm(layers=1, hidden=64, h_q=2, h_kv=1, head_dim=64, ffn=64, vocab=64, l_max=8, batch=1)


def test_bad_model_config_is_rejected_before_any_device_work(llm):
    base = dict(layers=1, hidden=64, h_q=2, h_kv=1, head_dim=64, ffn=64, vocab=64, l_max=8, batch=1)
    for bad in (dict(head_dim=48), dict(h_q=3, h_kv=2), dict(hidden=48), dict(tp_degree=2), dict(layers=0),
                dict(act_dtype=llm.I8)):
        cfg = dict(base)
        cfg.update(bad)
        with pytest.raises(llm.LogosError) as e:
            llm.Llm(**cfg)
        assert e.value.status in (1, 4), bad


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        _lib.load()


def test_ctypes_signatures_have_the_headers_arity():
    """Every prototype in the public header against the ctypes table: same set of names, same
    number of parameters (a mismatch would corrupt the call, not fail it)."""
    import re
    with open(_lib.HEADER_PATH) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    protos = dict(re.findall(r"LOGOS_API[^;(]*?\b(logos_[a-z0-9_]+)\s*\(([^;]*?)\)\s*;", text, flags=re.S))
    assert set(protos) == set(_lib._SIGNATURES)
    for name, params in protos.items():
        params = " ".join(params.split())
        n = 0 if params in ("", "void") else params.count(",") + 1
        assert n == len(_lib._SIGNATURES[name][1]), (name, params)
