"""Tensor parallelism on two GPUs of one node: every rank (its own process, as under
torchrun) builds its shard of the seeded weights, the only exchange is the sum of the partial
products after o_proj and down_proj - folded into the residual + RMSNorm kernel over
peer-mapped memory (the default), or as an NCCL all-reduce (LOGOS_B200_TP_FUSED=0) - and the greedy tokens
must equal the oracle's (unsharded) ones.  Skipped when fewer than two GPUs are visible."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _env(fused):
    env = dict(os.environ)
    env.pop("LOGOS_B200_TP_FUSED", None)
    if fused != "default":
        env["LOGOS_B200_TP_FUSED"] = fused
    return env


def _run_ranks(tmp_path, steps, t, fused, extra=()):
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), str(r), "2", str(tmp_path),
                               str(steps), str(t)] + list(extra), stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True, env=_env(fused))
             for r in range(2)]
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=170)[0])
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for r, p in enumerate(procs):
        assert p.returncode == 0, "rank %d failed:\n%s" % (r, outs[r][-2000:] if r < len(outs) else "")
    return tuple(np.load(tmp_path / ("r%d.npz" % i)) for i in range(2))


@pytest.mark.timeout(300)
def test_tp2_ranks_load_their_shards_from_one_file(llm, oracle, tmp_path):
    """The ranks are created from another seed and take their rows / columns out of one file
    of whole matrices; tokens equal the oracle's run on the file's weights and gains."""
    if llm.deviceCount() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, HERE)
    from tp_worker import CFG
    from logicaffeine_b200 import weights as W
    O = oracle
    steps, t = 12, 5
    ref = O.Llm(tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, **CFG)
    rng = np.random.default_rng(11)
    gains = {key: rng.uniform(0.5, 1.5, CFG["hidden"]).astype(np.float32)
             for key in W.tensors(CFG) if key[1] in W.GAINS}
    path = tmp_path / "model.q8w"
    W.writeWeightsFile(path, CFG, lambda l, k: gains[(l, k)] if k in W.GAINS else ref.get_tensor(l, k))
    for (l, k), g in gains.items():
        ref.set_tensor(l, k, g)
    r0, r1 = _run_ranks(tmp_path, steps, t, "default", [str(path)])
    toks = O.synth_fill(O.I32, 3, 9, 999, 0, CFG["batch"] * t, 0.0, float(CFG["vocab"])).reshape(CFG["batch"], t)
    ref.prefill(toks)
    want = np.array([ref.decode_step().copy() for _ in range(steps)])
    assert np.array_equal(r0["tokens"], want) and np.array_equal(r1["tokens"], want)
    ref.close()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("fused", ["default", "0"])
def test_tp2_tokens_match_the_oracle(llm, oracle, tmp_path, fused):
    if llm.deviceCount() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, HERE)
    from tp_worker import CFG
    O = oracle
    steps, t = 16, 7
    r0, r1 = _run_ranks(tmp_path, steps, t, fused)
    toks = O.synth_fill(O.I32, 3, 9, 999, 0, CFG["batch"] * t, 0.0, float(CFG["vocab"])).reshape(CFG["batch"], t)
    ref = O.Llm(tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, **CFG)
    ref.prefill(toks)
    want = np.array([ref.decode_step().copy() for _ in range(steps)])
    assert int(r0["exchange"]) == int(r1["exchange"]) == (1 if fused == "0" else 2)   # no silent fall-back
    assert np.array_equal(r0["tokens"], want) and np.array_equal(r1["tokens"], want)
    assert np.array_equal(r0["logits"], r1["logits"])           # replicated lm_head on identical inputs
    # each rank holds its own KV heads: rank r's head 0 is the oracle's head r
    kr, vr = ref.read_kv(0)
    n = t + steps
    for r, z in enumerate((r0, r1)):
        same = np.mean(z["k"][:, 0, :n] == kr[:, r, :n])
        assert same > 0.98, same
    ref.close()
