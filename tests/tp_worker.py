"""One tensor-parallel rank as its own process (used by test_gpu_tp.py and test_gpu_config4.py):
    python tests/tp_worker.py RANK WORLD OUT_DIR STEPS PROMPT_LEN [cfg=NAME] [force=NPZ] [WEIGHT_FILE]
With WEIGHT_FILE the model is created from another seed and every rank loads its shard of the file;
cfg=NAME picks one of CONFIGS (default "toy"); force=NPZ names a file whose array "inputs" [STEPS][B]
holds the token every step consumes (teacher forcing: a near-tie that flips one argmax then does
not change what the later steps are compared on).
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


# BASELINE.json's config 4 (Qwen2.5-32B-shaped, batch 64) at reduced depth and a short context: every GEMM
# shape of the real model (N = 55296 gate/up, K = 27648 down with split-K, the 1188-tile lm_head, 80-tile qkv),
# 8 sequences per rank at 8 ranks, in a model the CPU oracle steps in a few seconds
CFG4 = dict(layers=2, hidden=5120, h_q=64, h_kv=8, head_dim=128, ffn=27648, vocab=152064, l_max=32, batch=64,
            rms_eps=1e-6, rope_theta=1e6, tied_embeddings=0, seed=4, init_std=0.02)
CONFIGS = {"toy": CFG, "cfg4": CFG4}


def prompt_tokens(cfg, t):
    return O.synth_fill(O.I32, 3, cfg["seed"], 999, 0, cfg["batch"] * t, 0.0, float(cfg["vocab"])).reshape(cfg["batch"], t)


def main():
    global CFG
    rank, world, out_dir, steps, t = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], int(sys.argv[4]), int(sys.argv[5])
    forced = None
    while len(sys.argv) > 6 and "=" in sys.argv[6]:
        key, val = sys.argv.pop(6).split("=", 1)
        if key == "cfg":
            CFG = CONFIGS[val]
        elif key == "force":
            forced = np.load(val)["inputs"]
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
    toks = prompt_tokens(CFG, t)
    weight_file = sys.argv[6] if len(sys.argv) > 6 else None
    cfg = dict(CFG, seed=CFG["seed"] + 100) if weight_file else CFG
    m = llm.Llm(nccl_unique_id=uid, tp_degree=world, tp_rank=rank, device=rank, **cfg)
    if weight_file:
        m.loadWeights(weight_file)
    m.prefill(toks)
    if forced is None:
        got = m.decodeSteps(steps)
    else:
        got = np.zeros((steps, CFG["batch"]), np.int32)
        for i in range(steps):
            m.setTokens(forced[i])
            got[i] = m.decodeStep()
    k, v = m.readKv(0)
    np.savez(os.path.join(out_dir, "r%d.npz" % rank), tokens=got, k=k, v=v, logits=m.readLogits(), exchange=m.tpExchange(),
             status=llm.kernelStatus(rank))
    print("rank", rank, "done", flush=True)


if __name__ == "__main__":
    main()
