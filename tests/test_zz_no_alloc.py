"""The attention entry point that allocates nothing.

Some hosts cannot afford a device allocation inside an operator call: a server that gave
the whole GPU to its own arena at start-up, or a decode loop whose latency budget has no
room for the device-wide synchronisation an allocation implies.  For them
logos_gqa_decode_attn_fixed_scratch keeps the partial results of the (sequence, KV head)
pairs its persistent grid cuts in a fixed 6 MiB array inside the library.  It runs the same kernels as logos_gqa_decode_attn, so on the
same inputs the two must agree bit for bit, call after call (the array keeps the previous
call's contents), and a call beyond the stated maximum must be refused, not truncated.

This file sorts last on purpose: if it fails under `pytest -x`, every other test has
already run."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _inputs(O, b, hq, hkv, d, lmax, lens, seed):
    kc = O.synth_fill(O.F16, 2, seed, 20, 0, b * hkv * lmax * d, 0.0, 1.0).reshape(b, hkv, lmax, d)
    vc = O.synth_fill(O.F16, 2, seed, 21, 0, b * hkv * lmax * d, 0.0, 1.0).reshape(b, hkv, lmax, d)
    q = O.synth_fill(O.F16, 2, seed, 22, 0, b * hq * d, 0.0, 1.0).reshape(b, hq, d)
    return q, kc, vc, np.asarray(lens, np.int32)


def test_fixed_scratch_attention_matches_the_allocating_entry_point_twice(llm, oracle):
    O = oracle
    # two different shapes back to back: the second call finds the first call's partials in the array
    cases = [(4, 28, 4, 128, 700, [1, 64, 65, 699], 3), (3, 14, 2, 64, 300, [299, 130, 7], 4)]
    for b, hq, hkv, d, lmax, lens, seed in cases:
        q, kc, vc, seq = _inputs(O, b, hq, hkv, d, lmax, lens, seed)
        scale = 1.0 / np.sqrt(d)
        dq, dkc, dvc, dseq = (llm.DeviceBuffer.from_host(x) for x in (q, kc, vc, seq))
        want_buf = llm.DeviceBuffer(b * hq * d * 2)
        got_buf = llm.DeviceBuffer(b * hq * d * 2)
        llm.gqaDecodeAttn(dq, dkc, dvc, dseq, want_buf, b, hq, hkv, d, lmax, scale)
        want = want_buf.download(np.uint16, (b, hq, d))
        assert llm.kernelStatus() == 0   # also the status reader's own one-off allocation, before memory is measured
        for call in range(2):
            got_buf.memset(0xFF)
            llm.devSync()
            free_before, _ = llm.devMemInfo()
            llm.gqaDecodeAttnFixedScratch(dq, dkc, dvc, dseq, got_buf, b, hq, hkv, d, lmax, scale)
            llm.devSync()
            free_after, _ = llm.devMemInfo()
            # the very first call on a device may load the kernels' module; every later call must
            # not lower the driver's free-memory figure: no allocation, no growth
            if call == 1:
                assert free_after >= free_before, (free_before, free_after)
            got = got_buf.download(np.uint16, (b, hq, d))
            assert np.array_equal(got, want), "call %d differs from logos_gqa_decode_attn" % call
            # reads the fixed-scratch path's own status word (and the per-device one): a bounded
            # wait that gave up inside these kernels would show here
            assert llm.kernelStatus() == 0
        ref = O.gqa_decode_attn(q, kc, vc, seq, scale)
        a, r = O.f16_to_f32(want), O.f16_to_f32(ref)
        assert np.linalg.norm(a - r) / np.linalg.norm(r) < 1e-3   # and both agree with the oracle
        assert llm.kernelStatus() == 0


def test_fixed_scratch_refuses_what_does_not_fit(llm):
    # the most sequences one call takes is 2048 (a CTA keeps one tile count per sequence in shared memory)
    b, hq, hkv, d, lmax = 2049, 2, 1, 64, 64
    q = llm.DeviceBuffer(b * hq * d * 2)
    cache = llm.DeviceBuffer(b * hkv * lmax * d * 2)
    seq = llm.DeviceBuffer(b * 4)
    seq.memset(0)
    with pytest.raises(llm.LogosError) as e:
        llm.gqaDecodeAttnFixedScratch(q, cache, cache, seq, q, b, hq, hkv, d, lmax, 0.1)
    assert e.value.status == 4 and "2048" in str(e.value)
    for x in (q, cache, seq):
        x.free()
