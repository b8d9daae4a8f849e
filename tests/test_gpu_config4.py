"""BASELINE.json's config 4 at its own shapes: a Qwen2.5-32B-shaped model (hidden 5120, 64 query /
8 KV heads of 128, FFN 27648, vocabulary 152064, batch 64) at reduced depth, so the CPU oracle
can step it.  Greedy tokens and logits of the unsharded GPU model equal the oracle's, and the
same model under tensor parallelism on 2, 4 and 8 GPUs (one process per rank, both ways of
exchanging the partial sums) decodes the same tokens.  The multi-GPU cases skip when fewer GPUs
are visible."""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

PROMPT, STEPS = 3, 16


@pytest.fixture(scope="module")
def expected(oracle):
    """The oracle's run, computed once for every case of this file."""
    from tp_worker import CFG4, prompt_tokens
    O = oracle
    ref = O.Llm(tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, **CFG4)
    ref.prefill(prompt_tokens(CFG4, PROMPT))
    first = ref.read_logits().copy()
    tokens = np.array([ref.decode_step().copy() for _ in range(STEPS)])
    last = ref.read_logits().copy()
    ref.close()
    return dict(tokens=tokens, first_logits=first, last_logits=last)


@pytest.mark.timeout(900)
def test_config4_shapes_tokens_and_logits_on_one_gpu(llm, expected):
    from tp_worker import CFG4, prompt_tokens
    gpu = llm.Llm(**CFG4)
    gpu.prefill(prompt_tokens(CFG4, PROMPT))
    assert rel_l2(gpu.readLogits(), expected["first_logits"]) < 1e-4
    got = gpu.decodeSteps(STEPS)
    assert llm.kernelStatus() == 0
    mism = [(int(np.argmax(got[:, j] != expected["tokens"][:, j])), j) for j in range(CFG4["batch"])
            if (got[:, j] != expected["tokens"][:, j]).any()]
    assert not mism, "first mismatching (step, sequence): %s" % mism[:4]
    assert rel_l2(gpu.readLogits(), expected["last_logits"]) < 1e-4
    gpu.free()


def _run_ranks(world, tmp_path, fused):
    env = dict(os.environ)
    env.pop("LOGOS_B200_TP_FUSED", None)
    if fused != "default":
        env["LOGOS_B200_TP_FUSED"] = fused
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), str(r), str(world), str(tmp_path),
                               str(STEPS), str(PROMPT), "cfg=cfg4"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True, env=env)
             for r in range(world)]
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
    return [np.load(tmp_path / ("r%d.npz" % i)) for i in range(world)]


@pytest.mark.timeout(900)
@pytest.mark.parametrize("fused", ["default", "0"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_config4_shapes_tensor_parallel_tokens_equal_the_unsharded_oracle(llm, expected, tmp_path, world, fused):
    if llm.deviceCount() < world:
        pytest.skip("needs %d GPUs" % world)
    ranks = _run_ranks(world, tmp_path, fused)
    for r, z in enumerate(ranks):
        assert int(z["exchange"]) == (1 if fused == "0" else 2), "rank %d fell back silently" % r
        assert int(z["status"]) == 0
        assert np.array_equal(z["tokens"], expected["tokens"]), "rank %d" % r
        assert np.array_equal(z["logits"], ranks[0]["logits"])      # every rank ends with the same logits
    assert rel_l2(ranks[0]["logits"], expected["last_logits"]) < 1e-4
