"""Tensor parallelism on two GPUs of one node: every rank builds its shard of the
seeded weights, the only exchange is the NCCL sum all-reduce after o_proj and
down_proj, and the greedy tokens must equal the oracle's (unsharded) ones.
Skipped when fewer than two GPUs are visible."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = dict(layers=3, hidden=256, h_q=8, h_kv=2, head_dim=64, ffn=512, vocab=1024, l_max=64, batch=4,
           rms_eps=1e-6, rope_theta=1e6, tied_embeddings=0, seed=9, init_std=0.02)


def _rank(rank, world, uid, toks, steps, out_dir):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    sys.path.insert(0, ROOT)
    from logicaffeine_b200 import llm
    m = llm.Llm(nccl_unique_id=uid, tp_degree=world, tp_rank=rank, device=rank, **CFG)
    m.prefill(toks)
    got = m.decodeSteps(steps)
    k, v = m.readKv(0)
    np.savez(os.path.join(out_dir, "r%d.npz" % rank), tokens=got, k=k, v=v, logits=m.readLogits())
    m.free()


def test_tp2_tokens_match_the_oracle(llm, oracle, tmp_path):
    if llm.deviceCount() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    O = oracle
    steps, t = 16, 7
    toks = O.synth_fill(O.I32, 3, 9, 999, 0, CFG["batch"] * t, 0.0, float(CFG["vocab"])).reshape(CFG["batch"], t)
    uid = llm.tpUniqueId()
    mp.spawn(_rank, args=(2, uid, toks, steps, str(tmp_path)), nprocs=2, join=True)
    ref = O.Llm(tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, **CFG)
    ref.prefill(toks)
    want = np.array([ref.decode_step().copy() for _ in range(steps)])
    r0, r1 = (np.load(tmp_path / ("r%d.npz" % i)) for i in range(2))
    assert np.array_equal(r0["tokens"], want) and np.array_equal(r1["tokens"], want)
    assert np.array_equal(r0["logits"], r1["logits"])           # replicated lm_head on identical inputs
    # each rank holds its own KV heads: rank r's head 0 is the oracle's head r
    kr, vr = ref.read_kv(0)
    n = t + steps
    for r, z in enumerate((r0, r1)):
        same = np.mean(z["k"][:, 0, :n] == kr[:, r, :n])
        assert same > 0.98, same
    ref.close()
