"""Weight file without a GPU: the library's layout arithmetic against the Python restatement,
header validation and its status codes, and the rectangles a tensor-parallel rank takes out of
the whole matrices (against the seeded generator's own row / column slices)."""
import os

import numpy as np
import pytest

from logicaffeine_b200 import weights as W
from logicaffeine_b200._lib import LogosError

ARCH = dict(layers=2, hidden=128, h_q=4, h_kv=2, head_dim=64, ffn=256, vocab=320, tied_embeddings=0)
MODEL = dict(ARCH, l_max=16, batch=2, rms_eps=1e-6, rope_theta=1e6, seed=21, init_std=0.02)


def _oracle_model(O, **over):
    return O.Llm(tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, **dict(MODEL, **over))


def _write_from(model, path, cfg, gains=None):
    def get(layer, kind):
        if kind in W.GAINS:
            return None if gains is None else gains[(layer, kind)]
        return model.get_tensor(layer, kind)
    return W.writeWeightsFile(path, cfg, get)


@pytest.mark.parametrize("cfg", [ARCH, dict(ARCH, tied_embeddings=1, layers=3, hidden=96, ffn=160, vocab=77),
                                 dict(layers=64, hidden=5120, h_q=64, h_kv=8, head_dim=128, ffn=27648, vocab=152064,
                                      tied_embeddings=0),
                                 dict(ARCH, qkv_bias=1), dict(ARCH, qkv_bias=1, tied_embeddings=1, layers=5)])
def test_layout_of_the_library_equals_the_python_restatement(cfg):
    spans, total = W.layout(cfg)
    assert W.weightsFileBytes(cfg) == total
    assert W.weightsHeader(cfg) == W.header(cfg)
    for (layer, kind), span in list(spans.items())[:40] + list(spans.items())[-12:]:
        assert W.weightsSpan(cfg, layer, kind) == span, (layer, W.TENSOR_NAMES[kind])
    # regions are aligned, ordered and do not overlap
    ends = 256
    for (layer, kind), (q_off, q_bytes, s_off, s_bytes) in spans.items():
        assert q_off % 256 == 0 and s_off % 256 == 0 and q_off >= ends
        ends = max(q_off + q_bytes, s_off + s_bytes)
    assert total >= ends and total % 256 == 0


def test_the_32b_shaped_file_is_the_q8_weight_bytes_plus_gains_and_padding():
    cfg = dict(layers=64, hidden=5120, h_q=64, h_kv=8, head_dim=128, ffn=27648, vocab=152064, tied_embeddings=0)
    params = 64 * (5120 * (8192 + 2 * 1024) + 8192 * 5120 + 3 * 5120 * 27648) + 2 * 152064 * 5120
    payload = params * 9 // 8 + (2 * 64 + 1) * 5120 * 4        # 1 byte + 4/32 bytes per weight, f32 gains
    total = W.weightsFileBytes(cfg)
    assert 0 <= total - 256 - payload < 256 * (64 * 16 + 8)      # only alignment gaps on top


def test_span_and_size_reject_bad_arguments():
    with pytest.raises(LogosError) as e:
        W.weightsSpan(ARCH, 2, W.Q)                  # layer out of range
    assert e.value.status == 4
    with pytest.raises(LogosError) as e:
        W.weightsSpan(ARCH, 0, 15)                   # no such tensor
    assert e.value.status == 4
    with pytest.raises(LogosError) as e:
        W.weightsSpan(ARCH, 0, W.Q_BIAS)             # this architecture has no biases
    assert e.value.status == 1
    with pytest.raises(LogosError) as e:
        W.weightsSpan(dict(ARCH, tied_embeddings=1), 0, W.HEAD)
    assert e.value.status == 1
    with pytest.raises(LogosError) as e:
        W.weightsFileBytes(dict(ARCH, hidden=100))   # not a multiple of the Q8 block
    assert e.value.status == 1
    with pytest.raises(LogosError) as e:
        W.weightsFileBytes(dict(ARCH, layers=0))
    assert e.value.status == 4


def test_written_file_checks_out_and_shards_are_the_generator_slices(oracle, tmp_path):
    O = oracle
    ref = _oracle_model(O)
    path = tmp_path / "model.q8w"
    rng = np.random.default_rng(3)
    gains = {(l, k): rng.uniform(0.5, 1.5, ARCH["hidden"]).astype(np.float32)
             for l in range(ARCH["layers"]) for k in (W.ATTN_NORM, W.MLP_NORM)}
    gains[(0, W.FINAL_NORM)] = rng.uniform(0.5, 1.5, ARCH["hidden"]).astype(np.float32)
    total = _write_from(ref, path, ARCH, gains)
    assert os.path.getsize(path) == total == W.weightsFileBytes(ARCH)
    assert W.weightsCheck(path) == dict(ARCH, qkv_bias=0)
    H, D, F = ARCH["hidden"], ARCH["head_dim"], ARCH["ffn"]
    nq, nkv = ARCH["h_q"] * D, ARCH["h_kv"] * D
    std, seed = MODEL["init_std"], MODEL["seed"]
    for layer in range(ARCH["layers"]):
        st = layer * 16
        for g in (1, 2):
            for r in range(g):
                # row shards: q, k, v, gate, up; column shards: o, down (the model's own sharding plan)
                want = {
                    W.Q: O.q8_synth_weights(nq // g, H, seed, st + 0, std, row0=r * (nq // g)),
                    W.K: O.q8_synth_weights(nkv // g, H, seed, st + 1, std, row0=r * (nkv // g)),
                    W.V: O.q8_synth_weights(nkv // g, H, seed, st + 2, std, row0=r * (nkv // g)),
                    W.O: O.q8_synth_weights(H, nq // g, seed, st + 3, std, col0=r * (nq // g), k_total=nq),
                    W.GATE: O.q8_synth_weights(F // g, H, seed, st + 4, std, row0=r * (F // g)),
                    W.UP: O.q8_synth_weights(F // g, H, seed, st + 5, std, row0=r * (F // g)),
                    W.DOWN: O.q8_synth_weights(H, F // g, seed, st + 6, std, col0=r * (F // g), k_total=F),
                }
                for kind, (wq, ws) in want.items():
                    q, s = W.weightsReadShard(path, layer, kind, g, r)
                    assert np.array_equal(q, wq) and np.array_equal(s.view(np.uint32), ws.view(np.uint32)), \
                        (layer, W.TENSOR_NAMES[kind], g, r)
        for kind in (W.ATTN_NORM, W.MLP_NORM):
            assert np.array_equal(W.weightsReadShard(path, layer, kind, 2, 1), gains[(layer, kind)])
    assert np.array_equal(W.weightsReadShard(path, 0, W.FINAL_NORM), gains[(0, W.FINAL_NORM)])
    for kind in (W.EMBED, W.HEAD):          # replicated on every rank
        q, s = W.weightsReadShard(path, 0, kind, 2, 1)
        wq, ws = ref.get_tensor(0, kind)
        assert np.array_equal(q, wq) and np.array_equal(s, ws)
    with pytest.raises(LogosError) as e:
        W.weightsReadShard(path, 0, W.Q, 3, 0)       # heads do not divide by 3
    assert e.value.status == 1
    with pytest.raises(LogosError) as e:
        W.weightsReadShard(path, 0, W.Q, 2, 2)       # rank outside the group
    assert e.value.status == 4
    ref.close()


def test_malformed_files_are_told_apart(oracle, tmp_path):
    O = oracle
    ref = _oracle_model(O)
    good = tmp_path / "good.q8w"
    total = _write_from(ref, good, ARCH)
    ref.close()
    data = good.read_bytes()

    def status_of(blob, name):
        p = tmp_path / name
        p.write_bytes(blob)
        with pytest.raises(LogosError) as e:
            W.weightsCheck(p)
        return e.value.status, str(e.value)

    with pytest.raises(LogosError) as e:
        W.weightsCheck(tmp_path / "absent.q8w")
    assert e.value.status == 1 and "cannot open" in str(e.value)                     # Error: unreadable
    assert status_of(data[:100], "short")[0] == 5                                   # DeserializationFailed from here on
    assert status_of(b"NOTLOGOS" + data[8:], "magic")[0] == 5
    assert status_of(data[:8] + (2).to_bytes(4, "little") + data[12:], "version")[0] == 5
    st, msg = status_of(data[:total - 300], "truncated")
    assert st == 5 and "truncated" in msg
    bad_len = data[:80] + (total + 256).to_bytes(8, "little") + data[88:]            # file_bytes field
    assert status_of(bad_len, "length")[0] == 5
    bad_arch = data[:24] + (100).to_bytes(8, "little") + data[32:]                   # hidden = 100
    assert status_of(bad_arch, "arch")[0] == 5
    W.weightsCheck(good)                                                             # the good one still passes


def test_oracle_tensors_round_trip_and_gains_are_used(oracle):
    O = oracle
    toks = O.synth_fill(O.I32, 3, 1, 999, 0, MODEL["batch"] * 4, 0.0, float(MODEL["vocab"])).reshape(MODEL["batch"], 4)
    a = _oracle_model(O)
    b = _oracle_model(O, seed=22)                   # other weights ...
    for layer, kind in W.tensors(ARCH):             # ... replaced by a's, tensor by tensor
        got = a.get_tensor(layer, kind)
        if kind in W.GAINS:
            assert np.array_equal(got, np.ones(ARCH["hidden"], np.float32))
            b.set_tensor(layer, kind, got)
        else:
            b.set_tensor(layer, kind, *got)
    a.prefill(toks)
    b.prefill(toks)
    assert np.array_equal(a.read_logits(), b.read_logits())
    c = _oracle_model(O)
    c.set_tensor(0, W.FINAL_NORM, np.full(ARCH["hidden"], 2.0, np.float32))
    c.prefill(toks)
    # a gain of 2 on the final norm doubles every logit (x * inv * 2 is exact in binary)
    assert np.array_equal(c.read_logits(), 2.0 * a.read_logits())
    with pytest.raises(KeyError):
        a.get_tensor(5, W.Q)
    for m in (a, b, c):
        m.close()


def test_host_quantiser_equals_the_oracle_bit_for_bit(oracle):
    O = oracle
    w = O.synth_fill(O.F32, 2, 7, 1, 0, 96 * 256, 0.0, 0.02).reshape(96, 256)
    w[5, 32:64] = 0.0                       # an all-zero block
    w[6, 0] = 3.0                           # an outlier that sets its block's scale
    w[7, :32] = np.float32(1e-30)           # tiny values: the scale is subnormal-free but small
    q, s = W.q8QuantizeHost(w)
    q0, s0 = O.q8_quantize(w)
    assert np.array_equal(q, q0)
    assert np.array_equal(s.view(np.uint32), s0.view(np.uint32))
    with pytest.raises(ValueError):
        W.q8QuantizeHost(np.zeros((2, 40), np.float32))


def test_bias_vectors_in_the_file_and_their_shards(oracle, tmp_path):
    O = oracle
    arch = dict(ARCH, qkv_bias=1)
    ref = _oracle_model(O, qkv_bias=1)
    plain = _oracle_model(O)
    path = tmp_path / "biased.q8w"
    W.writeWeightsFile(path, arch, lambda l, k: None if k in W.GAINS else ref.get_tensor(l, k))
    assert W.weightsCheck(path) == arch
    assert os.path.getsize(path) > W.weightsFileBytes(ARCH)
    nq, nkv = ARCH["h_q"] * ARCH["head_dim"], ARCH["h_kv"] * ARCH["head_dim"]
    for layer in range(ARCH["layers"]):
        for kind, n, stream in ((W.Q_BIAS, nq, 7), (W.K_BIAS, nkv, 8), (W.V_BIAS, nkv, 9)):
            whole = O.synth_fill(O.F32, 2, MODEL["seed"], layer * 16 + stream, 0, n, 0.0, MODEL["init_std"])
            assert np.array_equal(ref.get_tensor(layer, kind), whole)
            assert np.array_equal(W.weightsReadShard(path, layer, kind), whole)
            for r in range(2):       # a rank's slice = the generator started at the rank's first row
                part = O.synth_fill(O.F32, 2, MODEL["seed"], layer * 16 + stream, r * (n // 2), n // 2, 0.0, MODEL["init_std"])
                assert np.array_equal(W.weightsReadShard(path, layer, kind, 2, r), part)
        # the matrices sit where the layout says, biases in between
        q, s = W.weightsReadShard(path, layer, W.O)
        wq, ws = ref.get_tensor(layer, W.O)
        assert np.array_equal(q, wq) and np.array_equal(s, ws)
    with pytest.raises(KeyError):
        plain.get_tensor(0, W.Q_BIAS)
    # the biases are used: same weights, other logits
    toks = O.synth_fill(O.I32, 3, 1, 999, 0, MODEL["batch"] * 4, 0.0, float(MODEL["vocab"])).reshape(MODEL["batch"], 4)
    ref.prefill(toks)
    plain.prefill(toks)
    assert not np.array_equal(ref.read_logits(), plain.read_logits())
    # zero biases = no biases, bit for bit
    for layer in range(ARCH["layers"]):
        for kind, n in ((W.Q_BIAS, nq), (W.K_BIAS, nkv), (W.V_BIAS, nkv)):
            ref.set_tensor(layer, kind, np.zeros(n, np.float32))
    ref.prefill(toks)
    assert np.array_equal(ref.read_logits(), plain.read_logits())
    # unknown header flags are refused
    data = bytearray(path.read_bytes())
    data[88] |= 2
    (tmp_path / "flags.q8w").write_bytes(bytes(data))
    with pytest.raises(LogosError) as e:
        W.weightsCheck(tmp_path / "flags.q8w")
    assert e.value.status == 5
    ref.close()
    plain.close()


def test_layout_property_random_architectures():
    """Random architectures: the library's spans equal the Python restatement's for every tensor,
    regions are aligned, ordered and disjoint, and the file ends within one alignment unit of the last."""
    from hypothesis import given, settings, strategies as stg

    @settings(max_examples=40, deadline=None)
    @given(layers=stg.integers(1, 4), hb=stg.integers(1, 6), hkv=stg.sampled_from([1, 2, 4]), grp=stg.integers(1, 4),
           d=stg.sampled_from([64, 128]), fb=stg.integers(1, 9), vocab=stg.integers(1, 500), tied=stg.booleans(),
           bias=stg.booleans())
    def check(layers, hb, hkv, grp, d, fb, vocab, tied, bias):
        cfg = dict(layers=layers, hidden=32 * hb, h_q=hkv * grp, h_kv=hkv, head_dim=d, ffn=32 * hkv * fb, vocab=vocab,
                   tied_embeddings=int(tied), qkv_bias=int(bias))
        spans, total = W.layout(cfg)
        assert W.weightsFileBytes(cfg) == total
        end = 256
        for (layer, kind), span in spans.items():
            assert W.weightsSpan(cfg, layer, kind) == span
            q_off, q_bytes, s_off, s_bytes = span
            assert q_off % 256 == 0 and q_off >= end and (s_bytes == 0 or (s_off % 256 == 0 and s_off >= q_off + q_bytes))
            end = max(q_off + q_bytes, s_off + s_bytes)
        assert end <= total < end + 256
    check()
