"""CPU restatement of the Gemma-2 prompt encoder.  TEST INFRASTRUCTURE: only tests, the smoke check
and the benchmark's CPU-baseline leg may import this module; the product never does.

Follows crates/cortiq-engine/src/textenc.rs (rms_norm_gemma :59-68, gelu_tanh :70-73, encode
:222-336), whose own parity reference is python/gemma_ref.py.  Pinned against outputs of
python/gemma_ref.py's functions on seeded synthetic f32 weights (tests/golden/make_gemma_ref.py).

Linears go through oracle.nextdit.matmat (exact dequant of q8_row / q4_tiled / q4tp, f32 products);
norm statistics in float64, RoPE angles and attention in float32 as the engine computes them.
"""
import numpy as np

from .nextdit import QWeight, matmat


def rms_norm_gemma(x, w, eps):
    """textenc.rs:59-68: f32(v * inv) * (1 + w) with f64 mean of squares."""
    x = np.asarray(x, np.float32)
    ss = (x.astype(np.float64) ** 2).mean(-1, keepdims=True)
    inv = 1.0 / np.sqrt(ss + eps)
    return (x.astype(np.float64) * inv).astype(np.float32) * (np.float32(1.0) + np.asarray(w, np.float32))


def gelu_tanh(v):
    """textenc.rs:70-73."""
    v = np.asarray(v, np.float32)
    c = np.float32(0.7978846)
    return np.float32(0.5) * v * (np.float32(1.0) + np.tanh(c * (v + np.float32(0.044715) * v * v * v)))


def rope_half(x, theta):
    """textenc.rs:271-286: pairs (i, i + hd/2), f32 frequencies / angles / sin / cos."""
    n, heads, hd = x.shape
    i = np.arange(hd // 2, dtype=np.float32)
    freq = (np.float32(1.0) / np.power(np.float32(theta), np.float32(2.0) * i / np.float32(hd))).astype(np.float32)
    ang = (np.arange(n, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32)
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    a, b = x[..., : hd // 2], x[..., hd // 2:]
    return np.concatenate([a * cos[:, None, :] - b * sin[:, None, :], a * sin[:, None, :] + b * cos[:, None, :]],
                          axis=-1).astype(np.float32)


class GemmaOracle:
    """t: {name: f32 array or QWeight} with the container's ``te.`` names; cfg: te.config_json."""

    def __init__(self, t, cfg):
        self.t, self.cfg = t, cfg
        self.hs, self.nl = cfg["hidden_size"], cfg["num_hidden_layers"]
        self.nh, self.nkv, self.hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        self.scale = np.float32(1.0) / np.sqrt(np.float32(cfg.get("query_pre_attn_scalar", 256.0)))
        self.softcap = np.float32(cfg.get("attn_logit_softcapping", 0.0) or 0.0)
        self.theta = np.float32(cfg.get("rope_theta", 10000.0))
        self.eps = float(cfg.get("rms_norm_eps", 1e-6))
        self.window = int(cfg.get("sliding_window", 4096))

    def embed(self, ids):
        """textenc.rs:237-246: dequantized rows times sqrt(hidden)."""
        e = self.t["te.embed_tokens.weight"]
        ids = np.asarray(ids, np.int64)
        if isinstance(e, QWeight):
            assert e.dtype == 3, "the packer stores the embedding table as q8_row"
            q = e.payload[: e.rows * e.cols].view(np.int8).reshape(e.rows, e.cols)[ids].astype(np.float32)
            sc = e.payload[e.rows * e.cols:].view(np.float16)[ids].astype(np.float32)
            rows = q * sc[:, None]
        else:
            rows = np.asarray(e, np.float32)[ids]
        return (rows * np.sqrt(np.float32(self.hs))).astype(np.float32)

    def attention(self, q, k, v):
        """textenc.rs:287-323: causal, GQA, soft-capped logits, f32."""
        n = q.shape[0]
        hpk = self.nh // self.nkv
        out = np.zeros((n, self.nh, self.hd), np.float32)
        mask = np.triu(np.full((n, n), -np.inf, np.float32), 1)
        for h in range(self.nh):
            kv = h // hpk
            s = (q[:, h] @ k[:, kv].T).astype(np.float32) * self.scale
            if self.softcap > 0:
                s = self.softcap * np.tanh(s / self.softcap)
            s = s + mask
            s = s - s.max(-1, keepdims=True)
            e = np.exp(s).astype(np.float32)
            a = e * (np.float32(1.0) / e.sum(-1, keepdims=True, dtype=np.float32))
            out[:, h] = a @ v[:, kv]
        return out.reshape(n, self.nh * self.hd)

    def encode(self, ids, keep_layer_inputs=False):
        """textenc.rs:222-336 -> (final-normed hidden [n, hidden], streams)."""
        n = len(ids)
        assert n < self.window
        t = self.t
        h = self.embed(ids)
        streams = []
        for l in range(self.nl):
            p = f"te.layers.{l}"
            if keep_layer_inputs:
                streams.append(h.copy())
            xn = rms_norm_gemma(h, t[f"{p}.input_layernorm.weight"], self.eps)
            q = matmat(t[f"{p}.self_attn.q_proj.weight"], xn).reshape(n, self.nh, self.hd)
            k = matmat(t[f"{p}.self_attn.k_proj.weight"], xn).reshape(n, self.nkv, self.hd)
            v = matmat(t[f"{p}.self_attn.v_proj.weight"], xn).reshape(n, self.nkv, self.hd)
            q, k = rope_half(q, self.theta), rope_half(k, self.theta)
            proj = matmat(t[f"{p}.self_attn.o_proj.weight"], self.attention(q, k, v))
            h = h + rms_norm_gemma(proj, t[f"{p}.post_attention_layernorm.weight"], self.eps)
            xn = rms_norm_gemma(h, t[f"{p}.pre_feedforward_layernorm.weight"], self.eps)
            g = matmat(t[f"{p}.mlp.gate_proj.weight"], xn)
            u = matmat(t[f"{p}.mlp.up_proj.weight"], xn)
            d = matmat(t[f"{p}.mlp.down_proj.weight"], (gelu_tanh(g) * u).astype(np.float32))
            h = (h + rms_norm_gemma(d, t[f"{p}.post_feedforward_layernorm.weight"], self.eps)).astype(np.float32)
        if keep_layer_inputs:
            streams.append(h.copy())
        return rms_norm_gemma(h, t["te.norm.weight"], self.eps), streams
