"""Seeded synthetic Gemma-2 encoder weights for the tests (names as
crates/cortiq-engine/src/textenc.rs:172-216 resolves them) and a container builder that quantizes
them with the CPU oracle's encoders."""
import numpy as np

from cmf_b200.container import CmfWriter
from oracle.nextdit import QWeight

TINY = dict(hidden_size=256, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
            intermediate_size=1024, vocab_size=512, query_pre_attn_scalar=64, attn_logit_softcapping=50.0,
            rope_theta=10000.0, rms_norm_eps=1e-6, sliding_window=4096)
# a cap low enough to bend logits of the synthetic weights (tanh far from linear)
TINY_CAP = dict(TINY, attn_logit_softcapping=2.0)
# Gemma-2-2B geometry (head_dim 256, GQA 8/4, GeGLU 9216) with a reduced depth and vocabulary
GEMMA_GEOM = dict(hidden_size=2304, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=4, head_dim=256,
                  intermediate_size=9216, vocab_size=1024, query_pre_attn_scalar=256, attn_logit_softcapping=50.0,
                  rope_theta=10000.0, rms_norm_eps=1e-6, sliding_window=4096)


def make_tensors(cfg, seed=0, std=0.02):
    rng = np.random.default_rng(seed)
    hs, nh, nkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    inter = cfg["intermediate_size"]
    t = {"te.embed_tokens.weight": (rng.standard_normal((cfg["vocab_size"], hs)) / np.sqrt(hs)).astype(np.float32)}

    def mat(r, c):
        return (rng.standard_normal((r, c)) * std).astype(np.float32)

    def norm():
        return (0.1 * rng.standard_normal(hs)).astype(np.float32)

    for l in range(cfg["num_hidden_layers"]):
        p = f"te.layers.{l}"
        t[p + ".input_layernorm.weight"] = norm()
        # logits of standard deviation ~2.5 whatever the geometry (sigma_w^2 * hidden with q_pre_attn = head_dim)
        qk = np.float32(np.sqrt(2.5 / hs) / std)
        t[p + ".self_attn.q_proj.weight"] = mat(nh * hd, hs) * qk
        t[p + ".self_attn.k_proj.weight"] = mat(nkv * hd, hs) * qk
        t[p + ".self_attn.v_proj.weight"] = mat(nkv * hd, hs)
        t[p + ".self_attn.o_proj.weight"] = mat(hs, nh * hd)
        t[p + ".post_attention_layernorm.weight"] = norm()
        t[p + ".pre_feedforward_layernorm.weight"] = norm()
        t[p + ".mlp.gate_proj.weight"] = mat(inter, hs) * 2
        t[p + ".mlp.up_proj.weight"] = mat(inter, hs)
        t[p + ".mlp.down_proj.weight"] = mat(hs, inter)
        t[p + ".post_feedforward_layernorm.weight"] = norm()
    t["te.norm.weight"] = norm()
    return t


def build(cfg, path, level, seed=0):
    """Write a container (embedding q8_row, ``*_proj`` at ``level``, norms f32) and return the tensor
    dict the oracle consumes (QWeight for every quantized tensor)."""
    t = make_tensors(cfg, seed)
    w = CmfWriter(arch={"arch_name": "gemma2-encoder-synth", "hidden_size": cfg["hidden_size"],
                        "num_layers": cfg["num_hidden_layers"], "vocab_size": cfg["vocab_size"]})
    out = {}
    for name, arr in t.items():
        dt = 3 if name == "te.embed_tokens.weight" else (level if name.endswith("_proj.weight") else None)
        if dt is None:
            w.add_f32(name, arr)
            out[name] = arr
        else:
            q = QWeight.quantize(dt, arr)
            w.add(name, dt, arr.shape, q.payload)
            out[name] = q
    w.add_json("te.config_json", cfg)
    w.write(path)
    return out
