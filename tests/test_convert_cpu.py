"""Float checkpoint -> weight file (logicaffeine_b200.convert) on a synthetic checkpoint in the
published Qwen2 layout: bf16 tensors over two safetensors files and a config.json.  Every tensor
in the file is the host quantiser's output for the checkpoint's tensor (the quantiser itself is
held against the oracle in test_weights_cpu.py), gains and biases arrive unchanged, and the
oracle runs on what was converted."""
import json

import numpy as np
import pytest

from logicaffeine_b200 import convert
from logicaffeine_b200 import weights as W

torch = pytest.importorskip("torch")
st = pytest.importorskip("safetensors.torch")

HF = dict(model_type="qwen2", num_hidden_layers=2, hidden_size=128, num_attention_heads=4, num_key_value_heads=2,
          intermediate_size=256, vocab_size=320, tie_word_embeddings=False, rms_norm_eps=1e-6, rope_theta=1000000.0)


def _checkpoint(path, hf, with_bias=True, with_head=True):
    g = torch.Generator().manual_seed(1)
    H, D = hf["hidden_size"], hf["hidden_size"] // hf["num_attention_heads"]
    nq, nkv, F, V = hf["num_attention_heads"] * D, hf["num_key_value_heads"] * D, hf["intermediate_size"], hf["vocab_size"]
    rnd = lambda *shape: (torch.randn(*shape, generator=g) * 0.05).to(torch.bfloat16)
    tensors = {"model.embed_tokens.weight": rnd(V, H), "model.norm.weight": (1 + rnd(H)).to(torch.bfloat16)}
    if with_head:
        tensors["lm_head.weight"] = rnd(V, H)
    for l in range(hf["num_hidden_layers"]):
        p = "model.layers.%d." % l
        tensors[p + "input_layernorm.weight"] = (1 + rnd(H)).to(torch.bfloat16)
        tensors[p + "post_attention_layernorm.weight"] = (1 + rnd(H)).to(torch.bfloat16)
        for name, n, k in (("self_attn.q_proj", nq, H), ("self_attn.k_proj", nkv, H), ("self_attn.v_proj", nkv, H),
                           ("self_attn.o_proj", H, nq), ("mlp.gate_proj", F, H), ("mlp.up_proj", F, H),
                           ("mlp.down_proj", H, F)):
            tensors[p + name + ".weight"] = rnd(n, k)
        if with_bias:
            for name, n in (("q_proj", nq), ("k_proj", nkv), ("v_proj", nkv)):
                tensors[p + "self_attn." + name + ".bias"] = rnd(n)
    names = sorted(tensors)
    half = len(names) // 2
    path.mkdir()
    st.save_file({n: tensors[n] for n in names[:half]}, str(path / "model-00001-of-00002.safetensors"))
    st.save_file({n: tensors[n] for n in names[half:]}, str(path / "model-00002-of-00002.safetensors"))
    (path / "config.json").write_text(json.dumps(hf))
    return {n: t.float().numpy() for n, t in tensors.items()}


def test_converted_file_holds_the_quantised_checkpoint(oracle, tmp_path):
    O = oracle
    src = _checkpoint(tmp_path / "ckpt", HF)
    cfg = convert.convertCheckpoint(tmp_path / "ckpt", tmp_path / "model.q8w")
    assert cfg == dict(layers=2, hidden=128, h_q=4, h_kv=2, head_dim=32, ffn=256, vocab=320, tied_embeddings=0,
                       rms_eps=1e-6, rope_theta=1e6, qkv_bias=1)
    arch = W.weightsCheck(tmp_path / "model.q8w")
    assert all(arch[k] == cfg[k] for k in arch)
    for layer, kind in W.tensors(cfg):
        name = convert.tensorName(layer, kind)
        got = W.weightsReadShard(tmp_path / "model.q8w", layer, kind)
        if kind in W.VECTORS:
            assert np.array_equal(got, src[name]), name
        else:
            q, s = O.q8_quantize(src[name])
            assert np.array_equal(got[0], q) and np.array_equal(got[1].view(np.uint32), s.view(np.uint32)), name
    # a rank of a group of two takes its rows of q_proj and its columns of down_proj
    q, s = O.q8_quantize(src["model.layers.1.self_attn.q_proj.weight"])
    gq, gs = W.weightsReadShard(tmp_path / "model.q8w", 1, W.Q, 2, 1)
    assert np.array_equal(gq, q[64:]) and np.array_equal(gs, s[64:])
    q, s = O.q8_quantize(src["model.layers.0.mlp.down_proj.weight"])
    gq, gs = W.weightsReadShard(tmp_path / "model.q8w", 0, W.DOWN, 2, 1)
    assert np.array_equal(gq, q[:, 128:]) and np.array_equal(gs, s[:, 4:])


def test_oracle_runs_on_a_converted_checkpoint(oracle, tmp_path):
    """head_dim 64 (what the library's attention takes): convert, put every tensor of the file
    into the oracle's model, and check its first logits against float64 matrix algebra on the
    dequantised weights for a one-token prompt (position 0: the rotary embedding is the identity,
    attention over one position returns v)."""
    O = oracle
    hf = dict(HF, num_attention_heads=2, num_key_value_heads=1, num_hidden_layers=1)
    _checkpoint(tmp_path / "ckpt", hf)
    cfg = convert.convertCheckpoint(tmp_path / "ckpt", tmp_path / "m.q8w")
    assert cfg["head_dim"] == 64
    m = O.Llm(tp_degree=1, tp_rank=0, device=0, act_dtype=O.F32, l_max=8, batch=1, seed=0, init_std=0.02, **cfg)
    f = tmp_path / "m.q8w"
    deq = {}
    for layer, kind in W.tensors(cfg):
        t = W.weightsReadShard(f, layer, kind)
        if kind in W.VECTORS:
            m.set_tensor(layer, kind, t)
            deq[kind] = t.astype(np.float64)
        else:
            m.set_tensor(layer, kind, *t)
            deq[kind] = (t[0].reshape(t[0].shape[0], -1, 32).astype(np.float64) * t[1][:, :, None]).reshape(t[0].shape)
    tok = 17
    m.prefill(np.array([[tok]], np.int32))
    norm = lambda x, g: x / np.sqrt((x ** 2).mean() + 1e-6) * g
    h = deq[W.EMBED][tok]
    x = norm(h, deq[W.ATTN_NORM])
    v = deq[W.V] @ x + deq[W.V_BIAS]
    v = v.astype(np.float32).astype(np.float16).astype(np.float64)        # the cache holds fp16
    att = np.concatenate([v, v])                                          # both query heads share the KV head
    h = h + deq[W.O] @ att
    x = norm(h, deq[W.MLP_NORM])
    g, u = deq[W.GATE] @ x, deq[W.UP] @ x
    h = h + deq[W.DOWN] @ (g / (1 + np.exp(-g)) * u)
    logits = deq[W.HEAD] @ norm(h, deq[W.FINAL_NORM])
    got = m.read_logits()[0].astype(np.float64)
    # f32 against float64 sums, and fp16 cache values that sit on a rounding boundary may differ by one place
    assert np.linalg.norm(got - logits) / np.linalg.norm(logits) < 5e-4
    m.close()


def test_checkpoint_without_biases_or_head_and_bad_shapes(tmp_path):
    hf = dict(HF, tie_word_embeddings=True)
    _checkpoint(tmp_path / "plain", hf, with_bias=False, with_head=False)
    cfg = convert.convertCheckpoint(tmp_path / "plain", tmp_path / "plain.q8w")
    assert cfg["qkv_bias"] == 0 and cfg["tied_embeddings"] == 1
    assert W.weightsCheck(tmp_path / "plain.q8w")["qkv_bias"] == 0
    # the config promises another ffn than the tensors have
    _checkpoint(tmp_path / "bad", HF)
    (tmp_path / "bad" / "config.json").write_text(json.dumps(dict(HF, intermediate_size=512)))
    with pytest.raises(ValueError) as e:
        convert.convertCheckpoint(tmp_path / "bad", tmp_path / "bad.q8w")
    assert "gate_proj" in str(e.value)
    with pytest.raises(FileNotFoundError):
        convert._Checkpoint(tmp_path)
