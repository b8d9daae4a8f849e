"""One tensor-parallel rank as its own process (used by test_gpu_tp.py):
    python tests/tp_worker.py RANK WORLD OUT_DIR STEPS PROMPT_LEN [WEIGHT_FILE]
With WEIGHT_FILE the model is created from another seed and every rank loads its shard of the file.
Rank 0 makes the NCCL id and publishes it in OUT_DIR; every rank writes its tokens, its
first layer's KV cache and the last logits to OUT_DIR/rRANK.npz."""
import faulthandler
import os
import sys
import time

faulthandler.dump_traceback_later(150, exit=True)  # never outlive the test that started us
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402,F401  (first, so every rank resolves the libnccl.so.2 a torchrun job would)

from logicaffeine_b200 import llm  # noqa: E402
from oracle import oracle as O  # noqa: E402  (inputs only: the seeded prompt generator)

CFG = dict(layers=3, hidden=256, h_q=8, h_kv=2, head_dim=64, ffn=512, vocab=1024, l_max=64, batch=4,
           rms_eps=1e-6, rope_theta=1e6, tied_embeddings=0, seed=9, init_std=0.02)


def main():
    rank, world, out_dir, steps, t = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], int(sys.argv[4]), int(sys.argv[5])
    id_path = os.path.join(out_dir, "nccl_id.bin")
    if rank == 0:
        with open(id_path + ".tmp", "wb") as f:
            f.write(llm.tpUniqueId())
        os.replace(id_path + ".tmp", id_path)
    t0 = time.time()
    while not os.path.exists(id_path):
        if time.time() - t0 > 60:
            raise RuntimeError("rank 0 never published the NCCL id")
        time.sleep(0.05)
    with open(id_path, "rb") as f:
        uid = f.read()
    toks = O.synth_fill(O.I32, 3, 9, 999, 0, CFG["batch"] * t, 0.0, float(CFG["vocab"])).reshape(CFG["batch"], t)
    weight_file = sys.argv[6] if len(sys.argv) > 6 else None
    cfg = dict(CFG, seed=CFG["seed"] + 100) if weight_file else CFG
    m = llm.Llm(nccl_unique_id=uid, tp_degree=world, tp_rank=rank, device=rank, **cfg)
    if weight_file:
        m.loadWeights(weight_file)
    m.prefill(toks)
    got = m.decodeSteps(steps)
    k, v = m.readKv(0)
    np.savez(os.path.join(out_dir, "r%d.npz" % rank), tokens=got, k=k, v=v, logits=m.readLogits(), exchange=m.tpExchange())
    print("rank", rank, "done", flush=True)


if __name__ == "__main__":
    main()
