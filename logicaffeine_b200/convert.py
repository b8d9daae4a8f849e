"""Float checkpoint -> weight file.

    python -m logicaffeine_b200.convert CHECKPOINT_DIR OUT.q8w

CHECKPOINT_DIR holds a `config.json` and one or more `*.safetensors` files in the
layout the Qwen2 family is published in (tensor names `model.embed_tokens.weight`,
`model.layers.N.self_attn.q_proj.weight` / `.bias`, `...mlp.gate_proj.weight`,
`model.norm.weight`, `lm_head.weight`, ...).  Every projection matrix is quantised
to Q8 blocks of 32 along its input dimension with `weights.q8QuantizeHost` (the
library's own rule, bit for bit) and written with `weights.writeWeightsFile`; norm
gains and q/k/v biases are stored as f32.  One tensor is in memory at a time.

The decode model's conventions match that layout: rotary pairs are (i, i + D/2),
RMSNorm multiplies by its weight after normalising, gate and up are separate
matrices (the library interleaves them when it loads the file).
"""
import glob
import json
import os
import sys

import numpy as np

from . import weights as W

_LAYER_NAMES = {
    W.ATTN_NORM: "input_layernorm.weight", W.MLP_NORM: "post_attention_layernorm.weight",
    W.Q: "self_attn.q_proj.weight", W.K: "self_attn.k_proj.weight", W.V: "self_attn.v_proj.weight",
    W.O: "self_attn.o_proj.weight", W.GATE: "mlp.gate_proj.weight", W.UP: "mlp.up_proj.weight",
    W.DOWN: "mlp.down_proj.weight", W.Q_BIAS: "self_attn.q_proj.bias", W.K_BIAS: "self_attn.k_proj.bias",
    W.V_BIAS: "self_attn.v_proj.bias",
}


def tensorName(layer, kind):
    """Name of a weight-file tensor in the checkpoint."""
    if kind == W.FINAL_NORM:
        return "model.norm.weight"
    if kind == W.EMBED:
        return "model.embed_tokens.weight"
    if kind == W.HEAD:
        return "lm_head.weight"
    return "model.layers.%d.%s" % (layer, _LAYER_NAMES[kind])


def configFromCheckpoint(ckpt_dir):
    """Architecture (and rms_eps / rope_theta) as keyword arguments of llm.Llm, from config.json."""
    with open(os.path.join(ckpt_dir, "config.json")) as f:
        c = json.load(f)
    heads = int(c["num_attention_heads"])
    hidden = int(c["hidden_size"])
    cfg = dict(layers=int(c["num_hidden_layers"]), hidden=hidden, h_q=heads,
               h_kv=int(c.get("num_key_value_heads", heads)), head_dim=int(c.get("head_dim", hidden // heads)),
               ffn=int(c["intermediate_size"]), vocab=int(c["vocab_size"]),
               tied_embeddings=1 if c.get("tie_word_embeddings", False) else 0,
               rms_eps=float(c.get("rms_norm_eps", 1e-6)), rope_theta=float(c.get("rope_theta", 1e6)))
    cfg["qkv_bias"] = 1 if c.get("attention_bias", c.get("model_type") == "qwen2") else 0
    return cfg


class _Checkpoint:
    """Tensor name -> file, over every *.safetensors of a directory; tensors load one at a time."""

    def __init__(self, ckpt_dir):
        from safetensors import safe_open
        self._open = safe_open
        self.where = {}
        files = sorted(glob.glob(os.path.join(ckpt_dir, "*.safetensors")))
        if not files:
            raise FileNotFoundError("no *.safetensors in %s" % ckpt_dir)
        for path in files:
            with safe_open(path, framework="pt") as f:
                for name in f.keys():
                    self.where[name] = path

    def __contains__(self, name):
        return name in self.where

    def get(self, name):
        if name not in self.where:
            raise KeyError("the checkpoint has no tensor '%s'" % name)
        with self._open(self.where[name], framework="pt") as f:
            return f.get_tensor(name).float().numpy()      # bf16 / fp16 / f32 -> f32, exactly


def convertCheckpoint(ckpt_dir, out_path, progress=None):
    """Write OUT as the weight file of the checkpoint in CKPT_DIR; returns the llm.Llm keyword
    arguments that fit it.  Raises if a tensor is missing or its shape is not the architecture's."""
    cfg = configFromCheckpoint(ckpt_dir)
    ck = _Checkpoint(ckpt_dir)
    if cfg["qkv_bias"] and tensorName(0, W.Q_BIAS) not in ck:
        cfg["qkv_bias"] = 0                                 # the config allows biases, the files hold none
    if not cfg["tied_embeddings"] and tensorName(0, W.HEAD) not in ck:
        cfg["tied_embeddings"] = 1                          # no separate lm_head stored: it is the embedding

    def get(layer, kind):
        name = tensorName(layer, kind)
        if progress:
            progress(name)
        t = ck.get(name)
        n, k = W.shape(cfg, kind)
        if kind in W.VECTORS:
            if t.shape != (k,):
                raise ValueError("%s: shape %s, the architecture needs (%d,)" % (name, t.shape, k))
            return t
        if t.shape != (n, k):
            raise ValueError("%s: shape %s, the architecture needs (%d, %d)" % (name, t.shape, n, k))
        return W.q8QuantizeHost(t)

    W.writeWeightsFile(out_path, cfg, get)
    return cfg


def main(argv):
    if len(argv) != 3:
        sys.stderr.write(__doc__)
        return 2
    cfg = convertCheckpoint(argv[1], argv[2], progress=lambda name: sys.stderr.write("  %s\n" % name))
    print(json.dumps({"file": argv[2], "bytes": os.path.getsize(argv[2]), "config": cfg}))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
