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
    # the rank's slice of the projection's bias: the generator's window at the rank's first row
    q_loc = (q_loc + O.synth_fill(O.F32, 2, seed, 7, rank * nq, nq, 0.0, std)).astype(np.float32)
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
    q = (q + O.synth_fill(O.F32, 2, seed, 7, 0, HQ * D, 0.0, std)).astype(np.float32)
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


def test_bench_byte_model_matches_the_workload_arithmetic():
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


def _slot_words(values_u32, epoch):
    """The wire format of the folded exchange: 16-byte slots {word, epoch, word, epoch}."""
    v = np.asarray(values_u32, np.uint32).reshape(-1, 2)
    out = np.empty((v.shape[0], 4), np.uint32)
    out[:, 0], out[:, 2] = v[:, 0], v[:, 1]
    out[:, 1] = out[:, 3] = epoch
    return out


def _exchange_worker(rank, world, port, out_dir):
    """The folded exchange on CPU ranks: push partial rows to the row's owner, the owner folds
    them in rank order into its slice of the residual stream and normalises, pushes the packed
    activation words to everybody, everybody unpacks.  send/recv stand in for the NVLink pushes."""
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, H, eps, epoch = 4, 64, 1e-6, 7
    rows_own = B // world
    h = O.synth_fill(O.F32, 2, 3, 700, 0, B * H, 0.0, 1.0).reshape(B, H)            # same on every rank
    part = O.synth_fill(O.F32, 2, 3, 710 + rank, 0, B * H, 0.0, 0.1).reshape(B, H)   # this rank's partial sums
    # A: push to owners (slot format), including to oneself
    inbox = np.zeros((world, rows_own, H // 2, 4), np.uint32)
    pending = []
    for owner in range(world):
        rows = slice(owner * rows_own, (owner + 1) * rows_own)
        msg = _slot_words(part[rows].view(np.uint32), epoch).reshape(rows_own, H // 2, 4)
        if owner == rank:
            inbox[rank] = msg
        else:
            pending.append(dist.isend(torch.from_numpy(msg.view(np.int32).copy()), owner))
    for src in range(world):
        if src != rank:
            t = torch.zeros(rows_own, H // 2, 4, dtype=torch.int32)
            dist.recv(t, src)
            inbox[src] = t.numpy().view(np.uint32)
    for w in pending:
        w.wait()
    assert np.all(inbox[:, :, :, 1] == epoch) and np.all(inbox[:, :, :, 3] == epoch)
    # B: the owner folds in rank order, normalises, packs hi | lo << 16
    mine = slice(rank * rows_own, (rank + 1) * rows_own)
    hv = h[mine].copy()
    for src in range(world):
        vals = inbox[src][:, :, [0, 2]].reshape(rows_own, H).view(np.float32)
        hv = (hv + vals).astype(np.float32)
    inv = (np.float32(1.0) / np.sqrt((np.sum(hv.astype(np.float64) ** 2, 1) / H + eps))).astype(np.float32)
    xn = (hv * inv[:, None]).astype(np.float32)
    hi = xn.astype(np.float16)
    lo = ((xn - hi.astype(np.float32)) * np.float32(2048.0)).astype(np.float16)
    packed = hi.view(np.uint16).astype(np.uint32) | (lo.view(np.uint16).astype(np.uint32) << 16)
    msg = torch.from_numpy(_slot_words(packed, epoch).view(np.int32).copy())
    rows_words = [torch.zeros_like(msg) for _ in range(world)]
    dist.all_gather(rows_words, msg)
    # C: unpack every owner's rows into plain planes
    words = np.concatenate([w.numpy().view(np.uint32)[:, [0, 2]].reshape(rows_own, H) for w in rows_words], 0)
    hi_all = (words & 0xffff).astype(np.uint16).view(np.float16)
    lo_all = (words >> 16).astype(np.uint16).view(np.float16)
    np.savez(os.path.join(out_dir, "x%d.npz" % rank), hi=hi_all, lo=lo_all, h_own=hv, part=part)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_folded_exchange_scheme_equals_allreduce_then_norm(oracle, tmp_path):
    import torch.multiprocessing as mp
    O = oracle
    world, B, H, eps = 2, 4, 64, 1e-6
    mp.spawn(_exchange_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r = [np.load(tmp_path / ("x%d.npz" % i)) for i in range(world)]
    h = O.synth_fill(O.F32, 2, 3, 700, 0, B * H, 0.0, 1.0).reshape(B, H)
    total = h.copy()
    for i in range(world):
        total = (total + r[i]["part"]).astype(np.float32)           # rank order, as the owner adds
    inv = (np.float32(1.0) / np.sqrt((np.sum(total.astype(np.float64) ** 2, 1) / H + eps))).astype(np.float32)
    xn = (total * inv[:, None]).astype(np.float32)
    hi = xn.astype(np.float16)
    lo = ((xn - hi.astype(np.float32)) * np.float32(2048.0)).astype(np.float16)
    for i in range(world):
        assert np.array_equal(r[i]["hi"].view(np.uint16), hi.view(np.uint16))   # every rank holds every row
        assert np.array_equal(r[i]["lo"].view(np.uint16), lo.view(np.uint16))
        assert np.array_equal(r[i]["h_own"], total[i * (B // world):(i + 1) * (B // world)])  # only the owner's rows of h
