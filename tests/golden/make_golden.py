"""Independent numpy restatement of the Q8 decode arithmetic -> golden vectors.

    python tests/golden/make_golden.py        # rewrites tests/golden/golden.npz

The reference holds no vectors for this path, so these pin the C oracle
(oracle/logos_oracle.c) against a second implementation written separately:
float64 for sums whose f32 order is free, explicit float32 steps where the
result is defined bit for bit (generator, Q8 block rule, rotary embedding and
the fp16 KV rows).  Inputs come from numpy's own generator, not from the code
under test.  Nothing here imports the oracle or the CUDA library.
"""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
f32 = np.float32
M64 = (1 << 64) - 1


# ------------------------------------------------------------------ generator
def mix64(z):
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & M64
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & M64
    z ^= z >> 31
    return z


def ctr_hash(seed, stream, idx):
    G = 0x9E3779B97F4A7C15
    return mix64((mix64((seed + G * (stream + 1)) & M64) + G * (idx + 1)) & M64)


def gen_i8(seed, stream, idx):
    return int((ctr_hash(seed, stream, idx) >> 32) % 255) - 127


def gen_uniform(seed, stream, idx, a, b):
    r = ctr_hash(seed, stream, idx) >> 40
    u = f32(r) * f32(5.9604644775390625e-08)
    return f32(f32(a) + f32(u * f32(f32(b) - f32(a))))


def gen_normal(seed, stream, idx):
    h = ctr_hash(seed, stream, idx >> 1)
    k1 = h >> 40
    k2 = (h >> 16) & 0xFFFFFF
    v = k1 + 1
    e = v.bit_length() - 1
    m = f32(f32(v) * f32(2.0 ** (-e)))
    if m > f32(1.41421354):
        m = f32(m * f32(0.5))
        e += 1
    t = f32(f32(m - f32(1.0)) / f32(m + f32(1.0)))
    t2 = f32(t * t)
    p = f32(0.111111111)
    for c in (0.142857143, 0.2, 0.333333343, 1.0):
        p = f32(f32(p * t2) + f32(c))
    ln_m = f32(f32(f32(2.0) * t) * p)
    ln_u = f32(ln_m + f32(f32(e - 24) * f32(0.693147182)))
    r = np.sqrt(f32(f32(-2.0) * ln_u), dtype=f32)
    quad = k2 >> 22
    fr = f32(f32(k2 & 0x3FFFFF) * f32(2.384185791015625e-07))
    x = f32(fr * f32(1.57079637))
    x2 = f32(x * x)
    c = f32(2.08767570e-09)
    for k in (-2.75573192e-07, 2.48015873e-05, -1.38888889e-03, 4.16666667e-02, -0.5, 1.0):
        c = f32(f32(c * x2) + f32(k))
    s = f32(1.60590438e-10)
    for k in (-2.50521084e-08, 2.75573192e-06, -1.98412698e-04, 8.33333333e-03, -1.66666667e-01, 1.0):
        s = f32(f32(s * x2) + f32(k))
    s = f32(s * x)
    cq, sq = [(c, s), (-s, c), (-c, -s), (s, -c)][quad]
    return f32(r * (sq if idx & 1 else cq))


def ln_pos(x):
    """ln of a positive normal float32: exponent by bits, atanh series on the mantissa."""
    bits = int(np.array([x], f32).view(np.uint32)[0])
    e = (bits >> 23) - 127
    m = np.array([(bits & 0x007FFFFF) | 0x3F800000], np.uint32).view(f32)[0]
    if m > f32(1.41421354):
        m = f32(m * f32(0.5))
        e += 1
    t = f32(f32(m - f32(1.0)) / f32(m + f32(1.0)))
    t2 = f32(t * t)
    p = f32(0.111111111)
    for c in (0.142857143, 0.2, 0.333333343, 1.0):
        p = f32(f32(p * t2) + f32(c))
    ln_m = f32(f32(f32(2.0) * t) * p)
    return f32(ln_m + f32(f32(e) * f32(0.693147182)))


def gen_gumbel(seed, stream, idx):
    """-ln(-ln u), u = (2k+1) * 2^-24 from the top 23 bits of the hash."""
    k = ctr_hash(seed, stream, idx) >> 41
    u = f32(f32(2 * k + 1) * f32(5.9604644775390625e-08))
    return f32(-ln_pos(f32(-ln_pos(u))))


def sample_rows(logits, inv_t, top_k, seed, positions):
    """Gumbel-max over the logits that reach the row's top_k-th largest (0: all of them)."""
    rows, vocab = logits.shape
    out = np.zeros(rows, np.int32)
    for i in range(rows):
        least = -np.inf
        if 0 < top_k < vocab:
            least = np.sort(logits[i])[::-1][top_k - 1]
        best, best_v = -1, None
        for v in range(vocab):
            if logits[i, v] < least:
                continue
            x = f32(f32(logits[i, v] * inv_t) + gen_gumbel(seed, i, int(positions[i]) * vocab + v))
            if best < 0 or x > best_v:
                best, best_v = v, x
        out[i] = best
    return out


# ------------------------------------------------------------------ 16-bit floats
def to_bf16_bits(a):
    u = np.ascontiguousarray(a, f32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(f32)


# ------------------------------------------------------------------ operators
def q8_quantize(w):
    n, k = w.shape
    wb = w.reshape(n, k // 32, 32).astype(f32)
    amax = np.abs(wb).max(axis=2)
    s = (amax / f32(127.0)).astype(f32)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = (wb / s[:, :, None]).astype(f32)
    q = np.where(amax[:, :, None] > 0, np.clip(np.rint(r), -127, 127), 0).astype(np.int8)
    return q.reshape(n, k), s


def dequant64(q, s):
    n, k = q.shape
    return (q.reshape(n, k // 32, 32).astype(np.float64) * s.astype(np.float64)[:, :, None]).reshape(n, k)


def rope_table(l_max, d, theta):
    i = np.arange(d // 2, dtype=np.float64)
    inv = np.array([theta ** (-2.0 * x / d) for x in i])
    ang = np.arange(l_max, dtype=np.float64)[:, None] * inv[None, :]
    return np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(f32)


def rope_f16(x, tab_pos):
    """x f32 [d] -> fp16 bits; every product and sum rounded to f32."""
    d = x.shape[-1]
    h = d // 2
    c, s = tab_pos[:, 0], tab_pos[:, 1]
    x1, x2 = x[:h].astype(f32), x[h:].astype(f32)
    o1 = (x1 * c).astype(f32) - (x2 * s).astype(f32)
    o2 = (x2 * c).astype(f32) + (x1 * s).astype(f32)
    return np.concatenate([o1.astype(f32), o2.astype(f32)]).astype(np.float16).view(np.uint16)


def attention64(q16, kc16, vc16, seq_len, scale):
    """q16 [B][Hq][D] fp16 bits, caches [B][Hkv][L][D] fp16 bits -> f64 [B][Hq][D]."""
    b, hq, d = q16.shape
    hkv = kc16.shape[1]
    g = hq // hkv
    out = np.zeros((b, hq, d))
    qf = q16.view(np.float16).astype(np.float64)
    kf = kc16.view(np.float16).astype(np.float64)
    vf = vc16.view(np.float16).astype(np.float64)
    for i in range(b):
        n = int(seq_len[i])
        if n == 0:
            continue
        for h in range(hq):
            sc = kf[i, h // g, :n] @ qf[i, h] * float(f32(scale))
            p = np.exp(sc - sc.max())
            out[i, h] = (p[:, None] * vf[i, h // g, :n]).sum(0) / p.sum()
    return out


# ------------------------------------------------------------------ the decode model, in float64
def synth_matrix(n, k, seed, stream, std):
    """Q8 blocks of the seeded N(0, std) matrix: element (r, c) is value r * k + c of its stream."""
    w = np.array([[f32(f32(std) * gen_normal(seed, stream, r * k + c)) for c in range(k)] for r in range(n)], f32)
    return q8_quantize(w)


def synth_vector(n, seed, stream, std):
    return np.array([f32(f32(std) * gen_normal(seed, stream, i)) for i in range(n)], f32)


class Model64:
    """The batched greedy decode step restated with float64 sums: f32 residual stream values are
    kept in float64 here, the KV cache and the rotated query are rounded to fp16 exactly as the
    arithmetic defines them.  Weight streams per layer l: 16 l + {0 q, 1 k, 2 v, 3 o, 4 gate,
    5 up, 6 down, 7 q_bias, 8 k_bias, 9 v_bias}; embedding 1 << 20 (tied lm_head)."""

    def __init__(self, cfg, gains):
        self.c = c = dict(cfg)
        H, D = c["hidden"], c["head_dim"]
        nq, nkv, F = c["h_q"] * D, c["h_kv"] * D, c["ffn"]
        mat = lambda n, k, st: dequant64(*synth_matrix(n, k, c["seed"], st, c["init_std"]))
        self.layers = []
        for l in range(c["layers"]):
            st = 16 * l
            L = dict(q=mat(nq, H, st), k=mat(nkv, H, st + 1), v=mat(nkv, H, st + 2), o=mat(H, nq, st + 3),
                     g=mat(F, H, st + 4), u=mat(F, H, st + 5), d=mat(H, F, st + 6))
            for j, (name, n) in enumerate((("bq", nq), ("bk", nkv), ("bv", nkv))):
                L[name] = synth_vector(n, c["seed"], st + 7 + j, c["init_std"]).astype(np.float64)
            self.layers.append(L)
        eq, es = synth_matrix(c["vocab"], H, c["seed"], 1 << 20, c["init_std"])
        self.embed_f32 = (eq.reshape(c["vocab"], H // 32, 32).astype(f32) * es[:, :, None]).astype(f32).reshape(c["vocab"], H)
        self.head = dequant64(eq, es)
        self.gains = gains.astype(np.float64)            # [2 layers + 1][hidden]
        self.tab = rope_table(c["l_max"], D, c["rope_theta"])
        B = c["batch"]
        self.kc = np.zeros((c["layers"], B, c["h_kv"], c["l_max"], D), np.uint16)
        self.vc = np.zeros_like(self.kc)
        self.len = np.zeros(B, np.int64)

    def norm(self, h, g):
        return h / np.sqrt((h ** 2).mean(1, keepdims=True) + float(f32(self.c["rms_eps"]))) * g

    def step(self, tokens):
        c = self.c
        B, D, hq, hkv = c["batch"], c["head_dim"], c["h_q"], c["h_kv"]
        h = self.embed_f32[tokens].astype(np.float64)
        scale = f32(1.0) / np.sqrt(f32(D))
        for l, L in enumerate(self.layers):
            x = self.norm(h, self.gains[2 * l])
            q = x @ L["q"].T + L["bq"]
            k = x @ L["k"].T + L["bk"]
            v = x @ L["v"].T + L["bv"]
            q16 = np.zeros((B, hq, D), np.uint16)
            for i in range(B):
                pos = int(self.len[i])
                for j in range(hq):
                    q16[i, j] = rope_f16(q[i, j * D:(j + 1) * D].astype(f32), self.tab[pos])
                for j in range(hkv):
                    self.kc[l, i, j, pos] = rope_f16(k[i, j * D:(j + 1) * D].astype(f32), self.tab[pos])
                    self.vc[l, i, j, pos] = v[i, j * D:(j + 1) * D].astype(f32).astype(np.float16).view(np.uint16)
            att = attention64(q16, self.kc[l], self.vc[l], self.len + 1, scale).reshape(B, hq * D)
            h = h + att @ L["o"].T
            x = self.norm(h, self.gains[2 * l + 1])
            g, u = x @ L["g"].T, x @ L["u"].T
            h = h + (g / (1.0 + np.exp(-g)) * u) @ L["d"].T
        self.len += 1
        logits = self.norm(h, self.gains[2 * c["layers"]]) @ self.head.T
        return logits


def main():
    rng = np.random.default_rng(20240607)
    out = {}

    # generator spot values
    idx = np.array([0, 1, 2, 3, 17, 1000, 123456789, (1 << 40) + 5], dtype=np.uint64)
    out["gen_idx"] = idx
    out["gen_i8"] = np.array([gen_i8(7, 3, int(i)) for i in idx], np.int8)
    out["gen_uniform"] = np.array([gen_uniform(7, 3, int(i), 1e-3, 1e-2) for i in idx], f32)
    out["gen_normal"] = np.array([gen_normal(7, 3, int(i)) for i in idx], f32)
    out["gen_normal_run"] = np.array([gen_normal(0, 11, i) for i in range(256)], f32)

    # Q8 block rule (with an all-zero block and a tie at .5)
    w = rng.normal(0, 0.02, (6, 96)).astype(f32)
    w[2, 32:64] = 0.0
    w[4, 0:32] = np.arange(32, dtype=f32) - f32(15.5)
    qq, ss = q8_quantize(w)
    out["quant_w"], out["quant_q"], out["quant_s"] = w, qq, ss

    # GEMV
    n, k = 48, 160
    q = rng.integers(-127, 128, (n, k)).astype(np.int8)
    s = rng.uniform(1e-3, 1e-2, (n, k // 32)).astype(f32)
    x = rng.normal(0, 1, k).astype(f32)
    out["gemv_q"], out["gemv_s"], out["gemv_x"] = q, s, x
    out["gemv_y"] = dequant64(q, s) @ x.astype(np.float64)

    # GEMM (bf16 activations), all three epilogues
    m, n, k = 5, 64, 128
    a = to_bf16_bits(rng.normal(0, 1, (m, k)).astype(f32))
    q = rng.integers(-127, 128, (n, k)).astype(np.int8)
    s = rng.uniform(1e-3, 1e-2, (n, k // 32)).astype(f32)
    aux = to_bf16_bits(rng.normal(0, 1, (m, n)).astype(f32))
    acc = from_bf16_bits(a).astype(np.float64) @ dequant64(q, s).T
    out["gemm_a"], out["gemm_q"], out["gemm_s"], out["gemm_aux"] = a, q, s, aux
    out["gemm_acc"] = acc
    out["gemm_res"] = acc + from_bf16_bits(aux).astype(np.float64)
    g, u = acc[:, 0::2], acc[:, 1::2]
    out["gemm_swiglu"] = g / (1.0 + np.exp(-g)) * u

    # rotary table, append (bit exact) and attention
    b, hq, hkv, d, lmax = 3, 6, 2, 64, 40
    tab = rope_table(lmax, d, 1e6)
    out["rope_tab"] = tab
    seq = np.array([0, 17, 39], np.int32)
    kc = rng.normal(0, 1, (b, hkv, lmax, d)).astype(np.float16).view(np.uint16)
    vc = rng.normal(0, 1, (b, hkv, lmax, d)).astype(np.float16).view(np.uint16)
    kn = rng.normal(0, 1, (b, hkv, d)).astype(np.float16).view(np.uint16)
    vn = rng.normal(0, 1, (b, hkv, d)).astype(np.float16).view(np.uint16)
    qr = rng.normal(0, 1, (b, hq, d)).astype(np.float16).view(np.uint16)
    out["att_seq"], out["att_kc"], out["att_vc"] = seq, kc, vc
    out["att_kn"], out["att_vn"], out["att_q"] = kn, vn, qr
    kc2, vc2 = kc.copy(), vc.copy()
    qrot = np.zeros_like(qr)
    for i in range(b):
        for h in range(hkv):
            kc2[i, h, seq[i]] = rope_f16(kn[i, h].view(np.float16).astype(f32), tab[seq[i]])
            vc2[i, h, seq[i]] = vn[i, h]
        for h in range(hq):
            qrot[i, h] = rope_f16(qr[i, h].view(np.float16).astype(f32), tab[seq[i]])
    out["att_kc_after"], out["att_vc_after"], out["att_q_rot"] = kc2, vc2, qrot
    scale = 1.0 / np.sqrt(d)
    out["att_scale"] = np.array([scale], f32)
    out["att_o_plain"] = attention64(qr, kc, vc, seq, scale)           # unfused: q as given, old lengths
    out["att_o_fused"] = attention64(qrot, kc2, vc2, seq + 1, scale)   # fused: rotated q, appended row

    # RMSNorm, SwiGLU
    xx = rng.normal(0, 2, (4, 96)).astype(f32)
    gg = rng.normal(1, 0.1, 96).astype(f32)
    x64 = xx.astype(np.float64)
    out["norm_x"], out["norm_g"] = xx, gg
    out["norm_y"] = x64 / np.sqrt((x64 ** 2).mean(1, keepdims=True) + 1e-6) * gg.astype(np.float64)
    ga = rng.normal(0, 2, 200).astype(f32)
    ub = rng.normal(0, 2, 200).astype(f32)
    out["swi_g"], out["swi_u"] = ga, ub
    out["swi_y"] = ga.astype(np.float64) / (1.0 + np.exp(-ga.astype(np.float64))) * ub.astype(np.float64)

    # Gumbel variate and Gumbel-max sampling (its own generator: the arrays above stay as they were)
    rng2 = np.random.default_rng(20240608)
    out["gen_gumbel"] = np.array([gen_gumbel(7, 3, int(i)) for i in idx], f32)
    out["gen_gumbel_run"] = np.array([gen_gumbel(0, 12, i) for i in range(256)], f32)
    lg = (rng2.normal(0, 2, (5, 40))).astype(f32)
    lg[3, 7] = lg[3, 9]                                   # a tie inside the row
    pos = np.array([0, 1, 33, 4096, 12], np.int32)
    inv_t = f32(f32(1.0) / f32(0.7))
    out["samp_logits"], out["samp_pos"], out["samp_temperature"] = lg, pos, np.array([0.7], f32)
    out["samp_tokens"] = sample_rows(lg, inv_t, 0, 21, pos)
    out["samp_tokens_top4"] = sample_rows(lg, inv_t, 4, 21, pos)
    out["samp_tokens_top1"] = sample_rows(lg, inv_t, 1, 21, pos)

    # a tiny decode model end to end: seeded weights and biases, gains that are not 1, a 3-token
    # prompt per sequence, then 5 greedy steps
    cfg = dict(layers=2, hidden=64, h_q=2, h_kv=1, head_dim=64, ffn=96, vocab=48, l_max=10, batch=2, rms_eps=1e-6,
               rope_theta=1e6, seed=13, init_std=0.05)
    gains = rng2.uniform(0.5, 1.5, (2 * cfg["layers"] + 1, cfg["hidden"])).astype(f32)
    prompt = rng2.integers(0, cfg["vocab"], (cfg["batch"], 3)).astype(np.int32)
    m = Model64(cfg, gains)
    for p in range(3):
        logits = m.step(prompt[:, p])
    toks = []
    for _ in range(5):
        nxt = logits.argmax(1).astype(np.int32)
        toks.append(nxt)
        logits = m.step(nxt)
    out["model_cfg"] = np.array([cfg[k] for k in ("layers", "hidden", "h_q", "h_kv", "head_dim", "ffn", "vocab", "l_max",
                                                  "batch", "seed")], np.int64)
    out["model_std"] = np.array([cfg["init_std"]], f32)
    out["model_gains"], out["model_prompt"] = gains, prompt
    out["model_tokens"] = np.array(toks, np.int32)                 # [5][B]: the tokens steps 1..5 consume
    out["model_logits"] = logits                                    # after the 5th of them
    out["model_k0"], out["model_v0"] = m.kc[0], m.vc[0]             # layer 0 cache, fp16 bits
    sl = np.sort(logits, 1)
    out["model_margin"] = sl[:, -1] - sl[:, -2]

    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print("wrote golden.npz with", len(out), "arrays")


if __name__ == "__main__":
    main()
