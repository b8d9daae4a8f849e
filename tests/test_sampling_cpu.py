"""Temperature sampling in the oracle: the Gumbel variate of the seeded generator has the right
distribution, Gumbel-max draws follow softmax(logits / T), temperature 0 is the plain argmax,
and a draw depends on (seed, row, position) only."""
import numpy as np


def test_gumbel_variate_moments_and_range(oracle):
    O = oracle
    g = O.synth_fill(O.F32, 4, 12, 3, 0, 400000)
    assert np.isfinite(g).all()
    # u = (2k+1) * 2^-24 lies strictly inside (0,1): -ln(-ln u) is bounded on both sides
    assert g.min() > -3.0 and g.max() < 17.0
    assert abs(g.mean() - 0.5772157) < 0.01                    # Euler-Mascheroni
    assert abs(g.var() - np.pi ** 2 / 6) < 0.03
    again = O.synth_fill(O.F32, 4, 12, 3, 0, 400000)
    assert np.array_equal(g, again)
    other = O.synth_fill(O.F32, 4, 12, 4, 0, 1000)
    assert not np.array_equal(g[:1000], other)
    # a window of the same stream is the same values
    assert np.array_equal(O.synth_fill(O.F32, 4, 12, 3, 1000, 500), g[1000:1500])


def test_gumbel_max_draws_follow_the_softmax(oracle):
    O = oracle
    logits = np.array([0.0, 1.0, 2.0, -1.0, 0.5, 2.5, -3.0, 1.5], np.float32)
    n = 40000
    for temperature in (1.0, 0.5, 2.0):
        rows = np.tile(logits, (n, 1))
        # every row its own stream, every row its own position: n independent draws
        tok = O.sample_rows(rows, temperature, seed=9, positions=np.arange(n) % 1000)
        freq = np.bincount(tok, minlength=8) / n
        p = np.exp(logits.astype(np.float64) / temperature)
        p /= p.sum()
        sigma = np.sqrt(p * (1 - p) / n)
        assert np.all(np.abs(freq - p) < 5 * sigma + 1e-4), (temperature, freq, p)


def test_temperature_zero_is_argmax_with_lowest_index_on_ties(oracle):
    O = oracle
    x = np.array([[1.0, 3.0, 3.0, 2.0], [5.0, 5.0, 5.0, 5.0], [-1.0, -2.0, -0.5, -0.5]], np.float32)
    assert O.sample_rows(x, 0.0, seed=1, positions=[0, 0, 0]).tolist() == [1, 0, 2]


def test_a_draw_depends_on_seed_row_and_position_only(oracle):
    O = oracle
    rng = np.random.default_rng(0)
    x = rng.normal(size=(6, 512)).astype(np.float32)
    pos = np.array([3, 4, 5, 6, 7, 8], np.int32)
    a = O.sample_rows(x, 1.0, 5, pos)
    assert np.array_equal(a, O.sample_rows(x, 1.0, 5, pos))
    # the same logits in the same row at the same position give the same token whatever the other rows hold
    y = x.copy()
    y[1:] = rng.normal(size=(5, 512)).astype(np.float32)
    assert O.sample_rows(y, 1.0, 5, pos)[0] == a[0]
    # another seed or other positions move the draws
    assert not np.array_equal(a, O.sample_rows(x, 1.0, 6, pos))
    assert not np.array_equal(a, O.sample_rows(x, 1.0, 5, pos + 1))


def test_oracle_model_samples_reproducibly(oracle):
    O = oracle
    cfg = dict(layers=2, hidden=128, h_q=4, h_kv=2, head_dim=64, ffn=256, vocab=320, l_max=32, batch=3,
               rms_eps=1e-6, rope_theta=1e6, tied_embeddings=1, seed=2, init_std=0.02)
    toks = O.synth_fill(O.I32, 3, 2, 999, 0, 3 * 4, 0.0, 320.0).reshape(3, 4)

    def run(temperature, seed):
        m = O.Llm(tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, **cfg)
        m.set_sampling(temperature, seed)
        m.prefill(toks)
        out = np.array([m.decode_step().copy() for _ in range(8)])
        m.close()
        return out

    greedy, a, b, c = run(0.0, 1), run(1.0, 1), run(1.0, 1), run(1.0, 2)
    assert np.array_equal(a, b)
    assert not np.array_equal(a, greedy) and not np.array_equal(a, c)


def test_oracle_ragged_prompts_equal_each_sequence_alone(oracle):
    """Sequences of a batch do not interact: a ragged batch gives every sequence the tokens it
    gets when it is run alone with its own prompt; equal lengths equal the plain prefill."""
    O = oracle
    cfg = dict(layers=2, hidden=128, h_q=4, h_kv=2, head_dim=64, ffn=256, vocab=320, l_max=32,
               rms_eps=1e-6, rope_theta=1e6, tied_embeddings=1, seed=2, init_std=0.02)
    lens = np.array([6, 1, 3, 0], np.int32)
    toks = O.synth_fill(O.I32, 3, 2, 999, 0, 4 * 6, 0.0, 320.0).reshape(4, 6)

    def decode(m, n):
        return np.array([m.decode_step().copy() for _ in range(n)])

    m = O.Llm(tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, batch=4, **cfg)
    m.prefill_ragged(toks, lens)
    assert np.array_equal(m.read_seq_len(), lens)
    batch = decode(m, 6)
    assert np.array_equal(m.read_seq_len(), lens + 6)
    for b in range(4):
        one = O.Llm(tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, batch=1, **cfg)
        if lens[b]:
            one.prefill(toks[b:b + 1, :lens[b]])
        else:
            one.set_tokens(np.zeros(1, np.int32))            # an empty prompt starts from token 0
        assert np.array_equal(decode(one, 6)[:, 0], batch[:, b]), b
        one.close()
    # a slot takes a new prompt in a running batch: the others carry on as if nothing happened
    m.prefill_ragged(toks, lens)
    head = decode(m, 3)
    fresh = np.zeros((4, 6), np.int32)
    fresh[1, :2] = [7, 300]
    m.prefill_ragged(fresh, np.array([-1, 2, -1, -1], np.int32))
    assert np.array_equal(m.read_seq_len(), [lens[0] + 3, 2, lens[2] + 3, lens[3] + 3])
    tail = decode(m, 3)
    for b in (0, 2, 3):
        assert np.array_equal(np.concatenate([head[:, b], tail[:, b]]), batch[:, b]), b
    one = O.Llm(tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, batch=1, **cfg)
    one.prefill(fresh[1:2, :2])
    assert np.array_equal(decode(one, 3)[:, 0], tail[:, 1])
    one.close()
    m.prefill_ragged(toks, np.full(4, 6, np.int32))
    same = decode(m, 4)
    m.prefill(toks)
    assert np.array_equal(decode(m, 4), same)
    m.close()


def test_top_k_restricts_the_draw_to_the_k_largest_with_ties(oracle):
    O = oracle
    logits = np.array([0.0, 1.0, 2.0, -1.0, 0.5, 2.5, -3.0, 1.5], np.float32)
    n = 30000
    rows = np.tile(logits, (n, 1))
    tok = O.sample_rows(rows, 1.0, seed=3, positions=np.arange(n) % 997, top_k=3)
    assert set(np.unique(tok)) == {2, 5, 7}                       # 2.0, 2.5, 1.5
    p = np.exp(logits[[2, 5, 7]].astype(np.float64))
    p /= p.sum()
    freq = np.array([(tok == i).mean() for i in (2, 5, 7)])
    assert np.all(np.abs(freq - p) < 5 * np.sqrt(p * (1 - p) / n) + 1e-4)
    # ties at the k-th largest value are all candidates; k = 1 is the argmax whatever the noise
    tied = np.tile(np.array([1.0, 3.0, 2.0, 2.0, 0.0], np.float32), (4000, 1))
    assert set(np.unique(O.sample_rows(tied, 1.0, 5, np.arange(4000), top_k=2))) == {1, 2, 3}
    assert set(np.unique(O.sample_rows(tied, 5.0, 5, np.arange(4000), top_k=1))) == {1}
    # k >= vocabulary or 0: no filter, the same draws
    base = O.sample_rows(rows[:500], 1.0, 3, np.arange(500))
    assert np.array_equal(O.sample_rows(rows[:500], 1.0, 3, np.arange(500), top_k=8), base)
    assert np.array_equal(O.sample_rows(rows[:500], 1.0, 3, np.arange(500), top_k=100), base)
    # temperature 0 ignores top_k
    assert O.sample_rows(rows[:3], 0.0, 3, [0, 0, 0], top_k=3).tolist() == [5, 5, 5]


def test_oracle_steps_past_a_full_cache(oracle):
    O = oracle
    cfg = dict(layers=2, hidden=128, h_q=4, h_kv=2, head_dim=64, ffn=256, vocab=320, l_max=8, batch=2,
               rms_eps=1e-6, rope_theta=1e6, tied_embeddings=1, seed=2, init_std=0.02)
    toks = O.synth_fill(O.I32, 3, 2, 999, 0, 2 * 6, 0.0, 320.0).reshape(2, 6)
    m = O.Llm(tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, **cfg)
    m.prefill_ragged(toks, np.array([6, 2], np.int32))
    k_before = None
    for step in range(7):
        m.decode_step()
        if step == 1:                                   # sequence 0 is full now (6 + 2)
            k_before = m.read_kv(0)[0][0].copy()
    assert m.read_seq_len().tolist() == [8, 8]
    assert np.array_equal(m.read_kv(0)[0][0], k_before)   # a full sequence's cache is not written again
    m.close()
