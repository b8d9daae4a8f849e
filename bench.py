#!/usr/bin/env python
"""Decode throughput of the Q8 hot path on N B200s of one node.

    python bench.py --gpus 1 --steps 64 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...     # the CPU arm: the oracle on the host cores

Workload (default): Qwen2.5-32B-shaped batch-64 greedy decode at context 2048,
random-init Q8 weights, fp16 KV cache, tensor parallel over the N ranks.  A
step is one decode step of all 64 sequences.  One JSON line on rank 0.

value      tokens/s with everything resident in HBM, K steps issued by one
           library call, device time from CUDA events on the model's stream,
           max over ranks
e2e        the same K steps through the per-step host API: each step copies
           its input token ids from pinned host memory and reads its output
           token ids back, wall clock around the loop
roofline   all Q8 GEMM launches of a step: algorithmic weight bytes / device
           time of those launches (CUDA events inside the library)
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # BASELINE.json configs[4]
    "qwen32b-b64": dict(layers=64, hidden=5120, h_q=64, h_kv=8, head_dim=128, ffn=27648, vocab=152064, batch=64,
                        tied_embeddings=0, ctx=2048),
    # BASELINE.json configs[3]
    "qwen0.5b-b16": dict(layers=24, hidden=896, h_q=14, h_kv=2, head_dim=64, ffn=4864, vocab=151936, batch=16,
                         tied_embeddings=1, ctx=128),
    # a small shape for quick checks of the script itself
    "tiny": dict(layers=4, hidden=1024, h_q=8, h_kv=2, head_dim=128, ffn=2048, vocab=4096, batch=16,
                 tied_embeddings=1, ctx=256),
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def gemm_weight_bytes(w, tp):
    """Algorithmic bytes of the Q8 GEMM launches of one step on one rank: 1.125 B per weight."""
    H, D = w["hidden"], w["head_dim"]
    nq, nkv, F = w["h_q"] * D // tp, w["h_kv"] * D // tp, w["ffn"] // tp
    per_layer = (nq + 2 * nkv) * H + H * nq + 2 * F * H + H * F
    params = w["layers"] * per_layer + w["vocab"] * H
    return params * 1.125


def kv_bytes(w, tp, length):
    return 2 * w["batch"] * (w["h_kv"] // tp) * length * w["head_dim"] * 2 * w["layers"]


class ClockSampler:
    """Samples nvidia-smi clocks while the timed region runs."""

    def __init__(self, index):
        self.rows = []
        self.proc = None
        self.index = index

    def start(self):
        q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown," \
            "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown," \
            "clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                for n, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_sample(w, ctx, reps, threads=None):
    """The oracle on one decoder layer of the workload, one step at context `ctx`;
    returns (tokens/s extrapolated to the full depth, seconds per layer-step, threads)."""
    from oracle import oracle as O
    if threads:
        O.set_threads(threads)
    m = O.Llm(layers=1, hidden=w["hidden"], h_q=w["h_q"], h_kv=w["h_kv"], head_dim=w["head_dim"], ffn=w["ffn"],
              vocab=1024, l_max=ctx + reps + 2, batch=w["batch"], rms_eps=1e-6, rope_theta=1e6, tied_embeddings=1,
              tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, seed=0, init_std=0.02)
    m.synth_kv(ctx, 1)
    m.set_tokens(np.arange(w["batch"], dtype=np.int32) % 1024)
    m.decode_step()  # warm
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        m.decode_step()
        times.append(time.perf_counter() - t0)
    m.close()
    t_layer = float(np.median(times))
    return w["batch"] / (t_layer * w["layers"]), t_layer, O.threads()


def run_reference(args, w, rank):
    """CPU arm: the oracle (a port: the reference holds no implementation of this path)."""
    if rank != 0:
        return
    reps = max(1, args.steps)
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_sample(w, w["ctx"], 1)
    t0 = time.perf_counter()
    tps, t_layer, threads = cpu_sample(w, w["ctx"], reps)
    sample = "1 of %d decoder layers x 1 decode step at context %d, batch %d, per timed step; scaled by the layer " \
             "count; lm_head (2%% of the weights) not in the sample" % (w["layers"], w["ctx"], w["batch"])
    line = {
        "impl": "reference", "metric": "Q8 decode tokens/s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": reps, "warmup": args.warmup, "ms_per_step": t_layer * w["layers"] * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 weights x f32 activations, f32 accumulate",
        "data": "synthetic", "config": {"workload": args.workload, "batch": w["batch"], "context": w["ctx"]},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


def gemv_probe(llm, torch, device):
    """Config 0 (4096x4096 Q8 GEMV) over 12 rotating weight copies (227 MB > L2), one CUDA graph of 120 launches."""
    n = k = 4096
    copies, launches = 12, 120
    qs, ss = [], []
    for c in range(copies):
        q = llm.DeviceBuffer(n * k, device)
        s = llm.DeviceBuffer(n * (k // 32) * 4, device)
        llm.synthFill(q, llm.I8, 0, 0, 100 + c, 0, n * k)
        llm.synthFill(s, llm.F32, 1, 0, 200 + c, 0, n * (k // 32), 1e-3, 1e-2)
        qs.append(q)
        ss.append(s)
    x = llm.DeviceBuffer(k * 4, device)
    y = llm.DeviceBuffer(n * 4, device)
    llm.synthFill(x, llm.F32, 2, 0, 3, 0, k, 0.0, 1.0)
    llm.devSync(device)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        sp = stream.cuda_stream
        for c in range(copies):
            llm.q8Gemv(qs[c], ss[c], x, y, n, k, stream=sp)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        # a chain of GEMVs as a batch-1 decode would issue them: the weights of a launch are
        # fetched while the previous launch finishes (dependent-launch scope), x and y wait
        prev = llm.dependentLaunchScope(True)
        try:
            with torch.cuda.graph(graph, stream=stream):
                for i in range(launches):
                    llm.q8Gemv(qs[i % copies], ss[i % copies], x, y, n, k, stream=stream.cuda_stream)
        finally:
            llm.dependentLaunchScope(prev)
        for _ in range(3):
            graph.replay()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = 1e9
        for _ in range(5):
            e0.record(stream)
            graph.replay()
            e1.record(stream)
            stream.synchronize()
            best = min(best, e0.elapsed_time(e1))
    us = best * 1e3 / launches
    nbytes = n * k + n * (k // 32) * 4 + k * 4 + n * 4
    for b in qs + ss + [x, y]:
        b.free()
    return {"shape": "4096x4096", "us_per_launch": us, "algorithmic_bytes": nbytes, "gbs": nbytes / us / 1e3,
            "timing": "CUDA graph of %d dependent launches (dependent-launch scope: a launch fetches its weights while "
                      "the previous one finishes) over %d rotating weight copies (> L2)" % (launches, copies)}


def op_probe(args):
    """Single-operator timing (used for ncu captures and kernel work): one JSON line."""
    import torch
    from logicaffeine_b200 import llm
    dev = 0
    torch.cuda.set_device(dev)
    peak, peak_kind = peaks()
    stream = torch.cuda.Stream()
    sp = stream.cuda_stream
    m, n, k, reps, copies = args.m, args.n, args.k, args.reps, args.copies
    if args.op == "weights":
        # weight file: save the workload's model (seeded weights), then time loading the file back
        # (host wall clock around the call; the file was just written, so it comes from the page cache)
        import tempfile
        from logicaffeine_b200 import weights as W
        cfg = {k: v for k, v in WORKLOADS[args.workload].items() if k != "ctx"}
        cfg.update(batch=1, l_max=64, seed=0, init_std=0.02)
        model = llm.Llm(**cfg)
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, "model.q8w")
            t0 = time.perf_counter()
            model.saveWeights(path)
            t_save = time.perf_counter() - t0
            size = os.path.getsize(path)
            assert size == W.weightsFileBytes(cfg)
            loads = []
            for _ in range(3):
                t0 = time.perf_counter()
                model.loadWeights(path)
                loads.append(time.perf_counter() - t0)
        model.free()
        print(json.dumps({"op": "weights", "workload": args.workload, "file_bytes": size, "save_s": t_save,
                          "load_s": loads, "load_gbs": size / min(loads) / 1e9,
                          "how": "mmap + two pinned 32 MiB staging buffers + cudaMemcpy2DAsync, page cache hot"}),
              flush=True)
        return
    if args.op == "q8_gemm":
        a = llm.DeviceBuffer(m * k * 4, dev)
        c = llm.DeviceBuffer(m * n * 4, dev)
        llm.synthFill(a, llm.F32, 2, 0, 1, 0, m * k, 0.0, 1.0)
        qs, ss = [], []
        for i in range(copies):
            q = llm.DeviceBuffer(n * k, dev)
            s_ = llm.DeviceBuffer(n * (k // 32) * 4, dev)
            llm.synthFill(q, llm.I8, 0, 0, 10 + i, 0, n * k)
            llm.synthFill(s_, llm.F32, 1, 0, 50 + i, 0, n * (k // 32), 1e-3, 1e-2)
            qs.append(q)
            ss.append(s_)
        run = lambda i: llm.q8GemmF32(a, qs[i % copies], ss[i % copies], c, m, n, k, stream=sp)
        nbytes = n * k * 1.125
    elif args.op == "q8_gemv":
        x = llm.DeviceBuffer(k * 4, dev)
        y = llm.DeviceBuffer(n * 4, dev)
        llm.synthFill(x, llm.F32, 2, 0, 1, 0, k, 0.0, 1.0)
        qs, ss = [], []
        for i in range(copies):
            q = llm.DeviceBuffer(n * k, dev)
            s_ = llm.DeviceBuffer(n * (k // 32) * 4, dev)
            llm.synthFill(q, llm.I8, 0, 0, 10 + i, 0, n * k)
            llm.synthFill(s_, llm.F32, 1, 0, 50 + i, 0, n * (k // 32), 1e-3, 1e-2)
            qs.append(q)
            ss.append(s_)
        run = lambda i: llm.q8Gemv(qs[i % copies], ss[i % copies], x, y, n, k, stream=sp)
        nbytes = n * k * 1.125 + k * 4 + n * 4
    else:  # attention: b = m sequences, n = context, config-2 heads unless overridden
        b, ctx, hq, hkv, d = m, n, args.hq, args.hkv, args.d
        lmax = ctx + 1
        kc = llm.DeviceBuffer(b * hkv * lmax * d * 2, dev)
        vc = llm.DeviceBuffer(b * hkv * lmax * d * 2, dev)
        llm.synthFill(kc, llm.F16, 2, 0, 1, 0, b * hkv * lmax * d, 0.0, 1.0)
        llm.synthFill(vc, llm.F16, 2, 0, 2, 0, b * hkv * lmax * d, 0.0, 1.0)
        qb, kn, vn = (llm.DeviceBuffer(b * h * d * 2, dev) for h in (hq, hkv, hkv))
        for j, (buf, h) in enumerate(((qb, hq), (kn, hkv), (vn, hkv))):
            llm.synthFill(buf, llm.F16, 2, 0, 3 + j, 0, b * h * d, 0.0, 1.0)
        tab = llm.DeviceBuffer.from_host(llm.ropeTable(lmax, d, 1e6), dev)
        ob = llm.DeviceBuffer(b * hq * d * 2, dev)
        lens = np.full(b, ctx, np.int32)
        seq = llm.DeviceBuffer.from_host(lens, dev)

        def run(i):
            seq.upload(lens)  # the fused call bumps the lengths; rewind so every launch sees the same work
            llm.gqaDecodeAttnFused(qb, kn, vn, kc, vc, tab, seq, ob, b, hq, hkv, d, lmax, 1.0 / np.sqrt(d), stream=sp)
        nbytes = 2 * b * hkv * (ctx + 1) * d * 2 + 2 * b * hq * d * 2
    llm.devSync(dev)
    with torch.cuda.stream(stream):
        for i in range(3):
            run(i)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        times = []
        for i in range(reps):
            e0.record(stream)
            run(i)
            e1.record(stream)
            stream.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)
    us = float(np.median(times))
    print(json.dumps({"op": args.op, "m": m, "n": n, "k": k, "us_median": us, "us_min": float(min(times)),
                      "algorithmic_bytes": nbytes, "gbs": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak,
                      "peak_kind": "of " + peak_kind, "status": llm.kernelStatus(dev),
                      "timing": "CUDA events around single launches (includes launch latency), %d rotating weight "
                                "copies" % copies}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qwen32b-b64", choices=sorted(WORKLOADS))
    ap.add_argument("--prefill", default="synthetic-kv", choices=["synthetic-kv", "prompt"])
    ap.add_argument("--act", default="f32", choices=["f32", "f16", "bf16"])
    ap.add_argument("--no-extras", action="store_true", help="skip the CPU baseline and the GEMV probe")
    ap.add_argument("--op", default="decode", choices=["decode", "q8_gemm", "q8_gemv", "attention", "weights"],
                    help="time one operator instead of the decode loop (attention: --m sequences, --n context)")
    ap.add_argument("--m", type=int, default=64)
    ap.add_argument("--n", type=int, default=18944)
    ap.add_argument("--k", type=int, default=3584)
    ap.add_argument("--hq", type=int, default=28)
    ap.add_argument("--hkv", type=int, default=4)
    ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--copies", type=int, default=3)
    args = ap.parse_args()
    if args.op != "decode":
        op_probe(args)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    w = dict(WORKLOADS[args.workload])
    if args.impl == "reference":
        run_reference(args, w, rank)
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    from logicaffeine_b200 import llm

    if not torch.cuda.is_available() or llm.deviceCount() == 0:
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    tp = world
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(llm.tpUniqueId()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        uid_bytes = bytes(uid.cpu().numpy().tobytes())
    else:
        uid_bytes = None

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ctx, B, K, W = w.pop("ctx"), w["batch"], args.steps, args.warmup
    act = {"f32": llm.F32, "f16": llm.F16, "bf16": llm.BF16}[args.act]
    t_setup = time.perf_counter()
    model = llm.Llm(nccl_unique_id=uid_bytes, tp_degree=tp, tp_rank=rank, device=local_rank, act_dtype=act,
                    l_max=ctx + K + 8, rms_eps=1e-6, rope_theta=1e6, seed=0, init_std=0.02, **w)
    tok_pinned = torch.empty(B, dtype=torch.int32).pin_memory()
    out_pinned = torch.empty(B, dtype=torch.int32).pin_memory()
    rng = np.random.default_rng(0)
    first_tokens = rng.integers(0, w["vocab"], B).astype(np.int32)
    if args.prefill == "prompt":
        prompts = rng.integers(0, w["vocab"], (B, ctx)).astype(np.int32)
        model.prefill(prompts)
        first_tokens = model.decodeStep()
        ctx = ctx + 1
    else:
        model.synthKv(ctx, 1)
    setup_s = time.perf_counter() - t_setup

    def rewind():
        model.setSeqLen(ctx)
        model.setTokens(first_tokens)

    # ---- warm-up, then the timed region: K steps, inputs resident, one library call
    rewind()
    model.decodeSteps(W, read_back=False)
    rewind()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    model.decodeSteps(K, read_back=False)
    barrier()
    ms, launches_per_step = model.lastTiming()
    ms = max_over_ranks(ms)
    clocks = sampler.stop() if rank == 0 else None
    value = B * K / (ms / 1e3)

    # ---- end to end: per-step host API, token ids in from pinned memory and out again every step
    rewind()
    tok_np, out_np = tok_pinned.numpy(), out_pinned.numpy()
    tok_np[:] = first_tokens
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        model.setTokens(tok_np)
        out_np[:] = model.decodeStep()
        tok_np[:] = out_np
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e = {"value": B * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": int(B * 4),
           "d2h_bytes_per_step": int(B * 4)}

    # ---- per-class device time of a step (events inside the library), mid-run context
    rewind()
    model.decodeSteps(max(1, K // 2), read_back=False)
    prof = [model.profileStep() for _ in range(3)]
    cls = {k: float(np.median([p[k] for p in prof])) for k in prof[0]}
    peak, peak_kind = peaks()
    gb = gemm_weight_bytes(dict(w, **{"ctx": ctx}), tp)
    gemm_gbs = gb / (cls["q8_gemm"] * 1e-3) / 1e9 if cls["q8_gemm"] > 0 else 0.0
    mid_len = ctx + max(1, K // 2) + 1
    attn_gbs = kv_bytes(w, tp, mid_len) / (cls["attention"] * 1e-3) / 1e9 if cls["attention"] > 0 else 0.0
    traffic = None
    tfile = os.path.join(ROOT, "profiles", "q8_gemm_traffic.json")
    if os.path.exists(tfile):
        with open(tfile) as f:
            traffic = json.load(f).get("dram_bytes_per_algorithmic_byte")
    n_gemm = 4 * w["layers"] + 1
    roofline = {"bound": "hbm", "kernel": "q8_gemm_tc_kernel (all %d launches of a step)" % n_gemm,
                "achieved": gemm_gbs, "peak": peak, "peak_kind": "of " + peak_kind, "unit": "GB/s",
                "frac": gemm_gbs / peak, "frac_of_8000_nominal": gemm_gbs / 8000.0,
                "algorithmic_bytes_per_step": gb,
                "traffic": (traffic * gb / n_gemm) if traffic else None}

    line = {
        "metric": "Q8 decode tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 weights x fp16 activation planes (f32-class), f32 accumulate, fp16 KV" if args.act == "f32"
                 else "int8 weights x %s activations, f32 accumulate, fp16 KV" % args.act,
        "data": "synthetic",
        "config": {"workload": args.workload, "batch": B, "context": ctx, "parallelism": "tp%d" % tp,
                   "kv": "seeded N(0,1) fp16 fill" if args.prefill == "synthetic-kv" else "prompt prefill",
                   "l2": "per-step working set (weights + KV, %.1f GB per rank) is far larger than L2" %
                         ((gb + kv_bytes(w, tp, ctx)) / 1e9)},
        "e2e": e2e, "gpu_launches": int(launches_per_step * K), "launches_per_step": int(launches_per_step),
        "roofline": roofline,
        "kernels_ms_per_step": cls,
        "attention": {"achieved": attn_gbs, "unit": "GB/s", "frac": attn_gbs / peak, "context": mid_len},
        "clocks": clocks, "setup_s": setup_s, "launch_counts": llm.launchCounts(),
    }

    if rank == 0 and world == 1 and not args.no_extras:
        try:
            line["q8_gemv"] = gemv_probe(llm, torch, local_rank)
            line["q8_gemv"]["frac"] = line["q8_gemv"]["gbs"] / peak
            line["q8_gemv"]["frac_of_8000_nominal"] = line["q8_gemv"]["gbs"] / 8000.0
        except Exception as e:  # the probe is an extra; the headline stands without it
            line["q8_gemv"] = {"error": str(e)}
        tps, t_layer, threads = cpu_sample(dict(w), ctx, 5)
        line["cpu_baseline"] = {
            "value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": "oracle on 1 of %d decoder layers x 1 decode step at context %d, batch %d, median of 5; scaled "
                      "by the layer count; lm_head not in the sample" % (w["layers"], ctx, B)}
    model.free()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
