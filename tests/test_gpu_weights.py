"""Weight file on the GPU: a saved model is byte for byte the file the Python writer makes from
the oracle's tensors; a model that loads a file (other weights than it was created with, norm
gains that are not 1) decodes the oracle's tokens; a second load under an already captured step
takes effect; mismatches are refused and leave the model usable."""
import numpy as np
import pytest

from conftest import rel_l2
from logicaffeine_b200 import weights as W
from logicaffeine_b200._lib import LogosError

pytestmark = pytest.mark.gpu

CFG = dict(layers=3, hidden=256, h_q=4, h_kv=2, head_dim=64, ffn=512, vocab=1024, l_max=64, batch=4,
           rms_eps=1e-6, rope_theta=1e6, tied_embeddings=0, seed=31, init_std=0.02)


def _oracle(O, **over):
    return O.Llm(tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, **dict(CFG, **over))


def _gains(seed):
    rng = np.random.default_rng(seed)
    g = {(l, k): rng.uniform(0.5, 1.5, CFG["hidden"]).astype(np.float32)
         for l in range(CFG["layers"]) for k in (W.ATTN_NORM, W.MLP_NORM)}
    g[(0, W.FINAL_NORM)] = rng.uniform(0.5, 1.5, CFG["hidden"]).astype(np.float32)
    return g


def _write(ref, path, cfg, gains=None):
    def get(layer, kind):
        if kind in W.GAINS:
            return None if gains is None else gains[(layer, kind)]
        return ref.get_tensor(layer, kind)
    W.writeWeightsFile(path, cfg, get)
    for key, g in (gains or {}).items():
        ref.set_tensor(key[0], key[1], g)


def _prompt(O, t):
    return O.synth_fill(O.I32, 3, 4, 999, 0, CFG["batch"] * t, 0.0, float(CFG["vocab"])).reshape(CFG["batch"], t)


@pytest.mark.parametrize("tied", [0, 1])
def test_saved_model_is_the_writers_file(llm, oracle, tmp_path, tied):
    O = oracle
    cfg = dict(CFG, tied_embeddings=tied)
    ref = _oracle(O, tied_embeddings=tied)
    _write(ref, tmp_path / "want.q8w", cfg)
    gpu = llm.Llm(**cfg)
    gpu.saveWeights(tmp_path / "got.q8w")
    want, got = (tmp_path / "want.q8w").read_bytes(), (tmp_path / "got.q8w").read_bytes()
    assert len(got) == len(want) == W.weightsFileBytes(cfg)
    assert got == want
    assert W.weightsCheck(tmp_path / "got.q8w")["tied_embeddings"] == tied
    gpu.free()
    ref.close()


def test_loaded_weights_and_gains_decode_like_the_oracle(llm, oracle, tmp_path):
    O = oracle
    t, steps = 6, 16
    toks = _prompt(O, t)
    ref = _oracle(O)                                   # seed 31 and gains that are not 1
    _write(ref, tmp_path / "a.q8w", CFG, _gains(1))
    gpu = llm.Llm(**dict(CFG, seed=77))                # created with other weights
    gpu.loadWeights(tmp_path / "a.q8w")
    ref.prefill(toks)
    gpu.prefill(toks)
    assert rel_l2(gpu.readLogits(), ref.read_logits()) < 1e-4
    want = np.array([ref.decode_step().copy() for _ in range(steps)])
    got = gpu.decodeSteps(steps)                        # the step is captured as a graph in here
    assert np.array_equal(got, want)

    # a second file under the captured step: the graph reads the new bytes
    ref2 = _oracle(O, seed=32)
    _write(ref2, tmp_path / "b.q8w", CFG, _gains(2))
    gpu.loadWeights(tmp_path / "b.q8w")
    ref2.prefill(toks)
    gpu.prefill(toks)
    want2 = np.array([ref2.decode_step().copy() for _ in range(steps)])
    got2 = gpu.decodeSteps(steps)
    assert np.array_equal(got2, want2)
    assert not np.array_equal(got2, got)

    # what was loaded is what a save writes
    gpu.saveWeights(tmp_path / "b_again.q8w")
    assert (tmp_path / "b_again.q8w").read_bytes() == (tmp_path / "b.q8w").read_bytes()
    gpu.free()
    ref.close()
    ref2.close()


def test_mismatched_and_unreadable_files_are_refused(llm, oracle, tmp_path):
    O = oracle
    other = dict(CFG, ffn=768)
    ref = _oracle(O, ffn=768)
    _write(ref, tmp_path / "other.q8w", other)
    ref.close()
    gpu = llm.Llm(**CFG)
    toks = _prompt(O, 3)
    gpu.prefill(toks)
    before = gpu.decodeSteps(4)
    with pytest.raises(LogosError) as e:
        gpu.loadWeights(tmp_path / "other.q8w")
    assert e.value.status == 1 and "ffn 768" in str(e.value)
    with pytest.raises(LogosError) as e:
        gpu.loadWeights(tmp_path / "absent.q8w")
    assert e.value.status == 1
    (tmp_path / "junk.q8w").write_bytes(b"\0" * 4096)
    with pytest.raises(LogosError) as e:
        gpu.loadWeights(tmp_path / "junk.q8w")
    assert e.value.status == 5
    with pytest.raises(LogosError) as e:
        gpu.saveWeights(tmp_path / "no_such_dir" / "x.q8w")
    assert e.value.status == 1
    gpu.prefill(toks)                                   # untouched by the refused loads
    assert np.array_equal(gpu.decodeSteps(4), before)
    gpu.free()


def test_biased_model_saves_loads_and_decodes(llm, oracle, tmp_path):
    """q/k/v bias vectors (Qwen2): the seeded biases of a created model are the oracle's, they sit
    in the file between v and o, and a model that loads other biases decodes the oracle's tokens
    (the attention kernel adds them where it stages q and the new k/v row)."""
    O = oracle
    cfg = dict(CFG, qkv_bias=1)
    t, steps = 6, 16
    toks = _prompt(O, t)
    ref = _oracle(O, qkv_bias=1)
    W.writeWeightsFile(tmp_path / "want.q8w", cfg, lambda l, k: None if k in W.GAINS else ref.get_tensor(l, k))
    gpu = llm.Llm(**cfg)
    gpu.saveWeights(tmp_path / "got.q8w")
    assert (tmp_path / "got.q8w").read_bytes() == (tmp_path / "want.q8w").read_bytes()
    ref.prefill(toks)
    gpu.prefill(toks)
    want = np.array([ref.decode_step().copy() for _ in range(steps)])
    assert np.array_equal(gpu.decodeSteps(steps), want)
    plain = llm.Llm(**CFG)                     # the biases matter
    plain.prefill(toks)
    assert not np.array_equal(plain.decodeSteps(steps), want)
    with pytest.raises(LogosError) as e:       # a file with biases does not fit a model without
        plain.loadWeights(tmp_path / "want.q8w")
    assert e.value.status == 1 and "qkv_bias" in str(e.value)
    plain.free()

    rng = np.random.default_rng(5)
    nq, nkv = CFG["h_q"] * CFG["head_dim"], CFG["h_kv"] * CFG["head_dim"]
    for layer in range(CFG["layers"]):
        for kind, n in ((W.Q_BIAS, nq), (W.K_BIAS, nkv), (W.V_BIAS, nkv)):
            ref.set_tensor(layer, kind, rng.uniform(-0.5, 0.5, n).astype(np.float32))
    W.writeWeightsFile(tmp_path / "other.q8w", cfg, lambda l, k: None if k in W.GAINS else ref.get_tensor(l, k))
    gpu.loadWeights(tmp_path / "other.q8w")
    ref.prefill(toks)
    gpu.prefill(toks)
    want2 = np.array([ref.decode_step().copy() for _ in range(steps)])
    got2 = gpu.decodeSteps(steps)
    assert np.array_equal(got2, want2) and not np.array_equal(want2, want)
    k, _ = gpu.readKv(0)
    kr, _ = ref.read_kv(0)
    assert rel_l2(O.f16_to_f32(k), O.f16_to_f32(kr)) < 2e-4
    gpu.free()
    ref.close()
