"""The C oracle against the committed golden vectors (numpy restatement,
tests/golden/make_golden.py).  Integer and bit-defined results must be equal;
f32-accumulated results must sit within f32 rounding of the float64 values."""
import numpy as np

from conftest import rel_l2


def test_generator_bits(oracle, golden):
    O = oracle
    idx = golden["gen_idx"]
    for j, i in enumerate(idx):
        i = int(i)
        assert O.synth_fill(O.I8, 0, 7, 3, i, 1)[0] == golden["gen_i8"][j]
        u = O.synth_fill(O.F32, 1, 7, 3, i, 1, 1e-3, 1e-2)[0]
        assert u.view(np.uint32) == golden["gen_uniform"][j].view(np.uint32)
        z = O.synth_fill(O.F32, 2, 7, 3, i, 1, 0.0, 1.0)[0]
        assert z.view(np.uint32) == golden["gen_normal"][j].view(np.uint32)
    run = O.synth_fill(O.F32, 2, 0, 11, 0, 256, 0.0, 1.0)
    assert np.array_equal(run.view(np.uint32), golden["gen_normal_run"].view(np.uint32))


def test_generator_distribution(oracle):
    O = oracle
    z = O.synth_fill(O.F32, 2, 5, 1, 0, 400_000, 0.0, 1.0)
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1.0) < 0.01
    kurt = ((z - z.mean()) ** 4).mean() / z.var() ** 2
    assert abs(kurt - 3.0) < 0.05
    q = O.synth_fill(O.I8, 0, 5, 2, 0, 400_000)
    assert q.min() == -127 and q.max() == 127
    u = O.synth_fill(O.F32, 1, 5, 3, 0, 100_000, 1e-3, 1e-2)
    assert u.min() >= 1e-3 and u.max() < 1e-2


def test_quantize_bit_exact(oracle, golden):
    q, s = oracle.q8_quantize(golden["quant_w"])
    assert np.array_equal(q, golden["quant_q"])
    assert np.array_equal(s.view(np.uint32), golden["quant_s"].view(np.uint32))
    assert (q[2, 32:64] == 0).all() and s[2, 1] == 0.0  # all-zero block


def test_synth_weights_match_fill_then_quantize(oracle):
    O = oracle
    n, k = 8, 96
    z = O.synth_fill(O.F32, 2, 9, 4, 0, n * k, 0.0, 1.0).reshape(n, k)
    w = (np.float32(0.02) * z).astype(np.float32)
    q0, s0 = O.q8_quantize(w)
    q1, s1 = O.q8_synth_weights(n, k, 9, 4, 0.02)
    assert np.array_equal(q0, q1) and np.array_equal(s0.view(np.uint32), s1.view(np.uint32))
    # shards are slices of the logical matrix
    q2, s2 = O.q8_synth_weights(3, k, 9, 4, 0.02, row0=2)
    assert np.array_equal(q2, q1[2:5]) and np.array_equal(s2, s1[2:5])
    q3, s3 = O.q8_synth_weights(n, 32, 9, 4, 0.02, col0=64, k_total=k)
    assert np.array_equal(q3, q1[:, 64:96]) and np.array_equal(s3, s1[:, 2:3])


def test_gemv(oracle, golden):
    y = oracle.q8_gemv(golden["gemv_q"], golden["gemv_s"], golden["gemv_x"])
    assert rel_l2(y, golden["gemv_y"]) < 2e-6


def test_gemv_hand_cases(oracle):
    O = oracle
    # one block, scale 1, one-hot x picks a weight column
    q = np.arange(-16, 16, dtype=np.int8).reshape(1, 32)
    s = np.ones((1, 1), np.float32)
    for j in (0, 13, 31):
        x = np.zeros(32, np.float32)
        x[j] = 1.0
        assert O.q8_gemv(q, s, x)[0] == float(q[0, j])
    # all ones
    assert O.q8_gemv(np.ones((2, 64), np.int8), np.full((2, 2), 0.5, np.float32), np.ones(64, np.float32))[1] == 32.0


def test_gemm_epilogues(oracle, golden):
    O = oracle
    a, q, s = golden["gemm_a"], golden["gemm_q"], golden["gemm_s"]
    acc = O.q8_gemm_f32(a, O.BF16, q, s)
    assert rel_l2(acc, golden["gemm_acc"]) < 2e-6
    bf = lambda x: O.bf16_to_f32(O.f32_to_bf16(np.asarray(x, np.float32)))
    c0 = O.bf16_to_f32(O.q8_gemm(a, q, s, 0))
    assert rel_l2(c0, bf(golden["gemm_acc"])) < 2e-3 and np.mean(c0 != bf(golden["gemm_acc"])) < 0.01
    c1 = O.bf16_to_f32(O.q8_gemm(a, q, s, 1, golden["gemm_aux"]))
    assert np.mean(c1 != bf(golden["gemm_res"])) < 0.01
    c2 = O.bf16_to_f32(O.q8_gemm(a, q, s, 2))
    assert c2.shape == (a.shape[0], q.shape[0] // 2)
    assert rel_l2(c2, golden["gemm_swiglu"]) < 5e-3


def test_gemm_m1_equals_gemv(oracle):
    O = oracle
    rng = np.random.default_rng(3)
    q = rng.integers(-127, 128, (40, 96)).astype(np.int8)
    s = rng.uniform(1e-3, 1e-2, (40, 3)).astype(np.float32)
    x = rng.normal(0, 1, 96).astype(np.float32)
    y = O.q8_gemv(q, s, x)
    c = O.q8_gemm_f32(x.reshape(1, -1), O.F32, q, s)
    assert np.array_equal(y.view(np.uint32), c.ravel().view(np.uint32))


def test_rope_table_and_append_bits(oracle, golden):
    O = oracle
    tab = O.rope_table(40, 64, 1e6)
    assert np.array_equal(tab.view(np.uint32), golden["rope_tab"].view(np.uint32))
    assert (tab[0, :, 0] == 1.0).all() and (tab[0, :, 1] == 0.0).all()  # position 0 is the identity
    kc, vc = golden["att_kc"].copy(), golden["att_vc"].copy()
    seq = golden["att_seq"].copy()
    O.kv_append_rope(kc, vc, golden["att_kn"], golden["att_vn"], tab, seq)
    assert np.array_equal(kc, golden["att_kc_after"]) and np.array_equal(vc, golden["att_vc_after"])
    assert np.array_equal(seq, golden["att_seq"] + 1)


def test_append_to_full_sequence_is_a_no_op(oracle, golden):
    O = oracle
    tab = golden["rope_tab"]
    kc, vc = golden["att_kc"].copy(), golden["att_vc"].copy()
    seq = np.array([40, 40, 40], np.int32)
    O.kv_append_rope(kc, vc, golden["att_kn"], golden["att_vn"], tab, seq)
    assert np.array_equal(kc, golden["att_kc"]) and (seq == 40).all()


def test_attention(oracle, golden):
    O = oracle
    scale = float(golden["att_scale"][0])
    o = O.f16_to_f32(O.gqa_decode_attn(golden["att_q"], golden["att_kc"], golden["att_vc"], golden["att_seq"], scale))
    ref = golden["att_o_plain"]
    assert (o[0] == 0).all()  # empty sequence
    assert rel_l2(o, ref) < 1e-3
    kc, vc, seq = golden["att_kc"].copy(), golden["att_vc"].copy(), golden["att_seq"].copy()
    of = O.f16_to_f32(O.gqa_decode_attn_fused(golden["att_q"], golden["att_kn"], golden["att_vn"], kc, vc,
                                              golden["rope_tab"], seq, scale))
    assert np.array_equal(kc, golden["att_kc_after"]) and np.array_equal(vc, golden["att_vc_after"])
    assert rel_l2(of, golden["att_o_fused"]) < 1e-3
    # a sequence of length one attends to its only row: o == v
    assert np.array_equal(O.f32_to_f16(of[0, 0]), golden["att_vn"][0, 0])


def test_norm_and_swiglu(oracle, golden):
    O = oracle
    assert rel_l2(O.rmsnorm(golden["norm_x"], golden["norm_g"], 1e-6), golden["norm_y"]) < 1e-6
    assert rel_l2(O.swiglu(golden["swi_g"], golden["swi_u"]), golden["swi_y"]) < 1e-6


def test_model_is_deterministic_and_kv_grows(oracle):
    O = oracle
    cfg = dict(layers=2, hidden=64, h_q=4, h_kv=2, head_dim=64, ffn=128, vocab=300, l_max=16, batch=2, rms_eps=1e-6,
               rope_theta=1e6, tied_embeddings=0, tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, seed=3,
               init_std=0.02)
    toks = np.array([[1, 2, 3], [4, 5, 6]], np.int32)
    runs = []
    for _ in range(2):
        m = O.Llm(**cfg)
        m.prefill(toks)
        out = [m.decode_step().copy() for _ in range(4)]
        k, v = m.read_kv(1)
        assert (m.read_seq_len() == 7).all()
        assert k[:, :, :7].any() and not k[:, :, 7:].any()
        runs.append((np.array(out), k, v))
        m.close()
    assert np.array_equal(runs[0][0], runs[1][0]) and np.array_equal(runs[0][1], runs[1][1])


def test_gumbel_bits_and_sampled_tokens(oracle, golden):
    """The sampler's noise and its choices against the independent numpy restatement: the Gumbel
    variate bit for bit, and the chosen token per row with all logits, the top 4 and the top 1."""
    O = oracle
    for j, i in enumerate(golden["gen_idx"]):
        g = O.synth_fill(O.F32, 4, 7, 3, int(i), 1)[0]
        assert g.view(np.uint32) == golden["gen_gumbel"][j].view(np.uint32)
    run = O.synth_fill(O.F32, 4, 0, 12, 0, 256)
    assert np.array_equal(run.view(np.uint32), golden["gen_gumbel_run"].view(np.uint32))
    lg, pos, t = golden["samp_logits"], golden["samp_pos"], float(golden["samp_temperature"][0])
    assert np.array_equal(O.sample_rows(lg, t, 21, pos), golden["samp_tokens"])
    assert np.array_equal(O.sample_rows(lg, t, 21, pos, top_k=4), golden["samp_tokens_top4"])
    assert np.array_equal(O.sample_rows(lg, t, 21, pos, top_k=1), golden["samp_tokens_top1"])
    # top 1 is the row's largest logit whatever the noise (lowest index on the tie in row 3)
    assert np.array_equal(golden["samp_tokens_top1"], lg.argmax(1))


def test_decode_model_against_the_float64_restatement(oracle, golden):
    """The whole model (seeded Q8 weights and q/k/v biases, gains that are not 1, RoPE positions,
    fp16 KV append, GQA attention, SwiGLU, residuals, tied lm_head, greedy choice) against the
    numpy model of tests/golden/make_golden.py, which shares no code with the oracle."""
    O = oracle
    names = ("layers", "hidden", "h_q", "h_kv", "head_dim", "ffn", "vocab", "l_max", "batch", "seed")
    cfg = {k: int(v) for k, v in zip(names, golden["model_cfg"])}
    m = O.Llm(tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, rms_eps=1e-6, rope_theta=1e6, tied_embeddings=1,
              init_std=float(golden["model_std"][0]), qkv_bias=1, **cfg)
    gains = golden["model_gains"]
    for l in range(cfg["layers"]):
        m.set_tensor(l, 0, gains[2 * l])
        m.set_tensor(l, 5, gains[2 * l + 1])
    m.set_tensor(0, 9, gains[2 * cfg["layers"]])
    m.prefill(golden["model_prompt"])
    want = golden["model_tokens"]                       # [5][B]: the tokens steps 1..5 consume
    assert np.array_equal(m.read_logits().argmax(1), want[0])
    outs = np.array([m.decode_step().copy() for _ in range(5)])
    assert np.array_equal(outs[:4], want[1:])
    assert np.array_equal(outs[4], golden["model_logits"].argmax(1))
    assert rel_l2(m.read_logits(), golden["model_logits"]) < 1e-4
    assert golden["model_margin"].min() > 1e-2          # the choices above were not near ties
    k, v = m.read_kv(0)
    n = 3 + 5
    assert m.read_seq_len().tolist() == [n] * cfg["batch"]
    for got, ref in ((k, golden["model_k0"]), (v, golden["model_v0"])):
        assert not got[:, :, n:].any() and not ref[:, :, n:].any()
        assert np.mean(got[:, :, :n] != ref[:, :, :n]) < 0.02        # fp16 values on a rounding boundary may flip
        assert rel_l2(O.f16_to_f32(got), O.f16_to_f32(ref)) < 1e-3
    m.close()
