"""The tensor-parallel sharding plan on two CPU ranks (gloo): each rank builds
its shard of the seeded weights the way the library does (rows of q/k/v/gate/up,
columns of o_proj/down_proj, indexed in the logical matrix), runs the oracle's
GEMMs on its shard, and the only exchange is a sum all-reduce after o_proj and
after down_proj.  The result must match the unsharded oracle."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    O.set_threads(1)
    H, D, HQ, HKV, F, B, seed, std = 128, 32, 8, 2, 256, 3, 11, 0.02
    nq, nkv, f = HQ * D // world, HKV * D // world, F // world
    x = O.synth_fill(O.F32, 2, seed, 500, 0, B * H, 0.0, 1.0).reshape(B, H)

    def mat(n, k, stream, row0=0, col0=0, k_total=None):
        return O.q8_synth_weights(n, k, seed, stream, std, row0=row0, col0=col0, k_total=k_total)

    # row-sharded projections: this rank's slice of the output columns
    q_loc = O.q8_gemm_f32(x, O.F32, *mat(nq, H, 0, row0=rank * nq))
    k_loc = O.q8_gemm_f32(x, O.F32, *mat(nkv, H, 1, row0=rank * nkv))
    g_loc = O.q8_gemm_f32(x, O.F32, *mat(f, H, 4, row0=rank * f))
    u_loc = O.q8_gemm_f32(x, O.F32, *mat(f, H, 5, row0=rank * f))
    act_loc = O.swiglu(g_loc, u_loc)
    # column-sharded projections: partial sums, then the exchange
    o_part = O.q8_gemm_f32(q_loc, O.F32, *mat(H, nq, 3, col0=rank * nq, k_total=HQ * D))
    d_part = O.q8_gemm_f32(act_loc, O.F32, *mat(H, f, 6, col0=rank * f, k_total=F))
    o_sum = torch.from_numpy(o_part.copy())
    d_sum = torch.from_numpy(d_part.copy())
    dist.all_reduce(o_sum)
    dist.all_reduce(d_sum)
    gathered = [torch.zeros(B, nq) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(q_loc.copy()))
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), o=o_sum.numpy(), d=d_sum.numpy(),
             q=torch.cat(gathered, 1).numpy(), k=k_loc)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_sharding_matches_unsharded(oracle, tmp_path):
    import torch.multiprocessing as mp
    O = oracle
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    H, D, HQ, HKV, F, B, seed, std = 128, 32, 8, 2, 256, 3, 11, 0.02
    x = O.synth_fill(O.F32, 2, seed, 500, 0, B * H, 0.0, 1.0).reshape(B, H)
    full = lambda n, k, st: O.q8_synth_weights(n, k, seed, st, std)
    q = O.q8_gemm_f32(x, O.F32, *full(HQ * D, H, 0))
    kk = O.q8_gemm_f32(x, O.F32, *full(HKV * D, H, 1))
    act = O.swiglu(O.q8_gemm_f32(x, O.F32, *full(F, H, 4)), O.q8_gemm_f32(x, O.F32, *full(F, H, 5)))
    o = O.q8_gemm_f32(q, O.F32, *full(H, HQ * D, 3))
    d = O.q8_gemm_f32(act, O.F32, *full(H, F, 6))
    r = [np.load(tmp_path / ("rank%d.npz" % i)) for i in range(world)]
    # every rank holds the same reduced result, bit for bit
    assert np.array_equal(r[0]["o"], r[1]["o"]) and np.array_equal(r[0]["d"], r[1]["d"])
    # row shards are exact slices; column shards agree up to the f32 order of the split sum
    assert np.array_equal(r[0]["q"], q)
    nkv = HKV * D // world
    assert np.array_equal(r[1]["k"], kk[:, nkv:2 * nkv])
    rel = lambda a, b: np.linalg.norm(a - b) / np.linalg.norm(b)
    assert rel(r[0]["o"], o) < 1e-6 and rel(r[0]["d"], d) < 1e-6


def test_bench_byte_model_matches_the_survey_figures():
    sys.path.insert(0, ROOT)
    import bench
    w = dict(bench.WORKLOADS["qwen32b-b64"])
    assert bench.gemm_weight_bytes(w, 1) == 38247137280.0          # 1.125 B per weight, config 4
    assert bench.kv_bytes(w, 1, 2048) == 34359738368                # 262144 B x 64 sequences x 2048
    # tensor parallel: layer weights divide, the replicated lm_head does not
    head = w["vocab"] * w["hidden"] * 1.125
    assert abs(bench.gemm_weight_bytes(w, 8) - ((38247137280.0 - head) / 8 + head)) < 1.0
    w0 = dict(bench.WORKLOADS["qwen0.5b-b16"])
    layer = (14 * 64 + 2 * 2 * 64) * 896 + 896 * 14 * 64 + 3 * 4864 * 896
    assert bench.gemm_weight_bytes(w0, 1) == (24 * layer + 151936 * 896) * 1.125
