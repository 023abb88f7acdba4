"""Generate tests/golden/gemma_ref_*.npz by running the reference's own numpy encoder functions
(python/gemma_ref.py, imported from the reference checkout) on seeded synthetic f32 weights.

Run in the build container only:  python tests/golden/make_gemma_ref.py /path/to/reference
The fixtures hold the weights' seed, the token ids and the reference's hidden states; the oracle
(oracle/gemma.py) must reproduce them.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from tests import gemma_model  # noqa: E402

CASES = {"tiny": (gemma_model.TINY, 5, [2, 106, 45, 108, 317, 385, 23, 107, 9, 500, 77]),
         "tiny_long": (gemma_model.TINY, 6, list(np.random.default_rng(1).integers(0, 512, 40)))}


def run_reference(ref, cfg, t, ids):
    """The body of gemma_ref.main() after its file loading (python/gemma_ref.py:84-121), also
    keeping the stream that enters every layer."""
    t = {k.replace("te.", "model.", 1): v for k, v in t.items()}
    hs, nh, nkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps, cap = cfg["rms_norm_eps"], cfg["attn_logit_softcapping"]
    scale = 1.0 / np.sqrt(cfg["query_pre_attn_scalar"])
    ids = np.array(ids, dtype=np.uint32)
    n = len(ids)
    h = t["model.embed_tokens.weight"][ids] * np.sqrt(np.float32(hs))
    streams = []
    for l in range(cfg["num_hidden_layers"]):
        streams.append(h.copy())
        p = f"model.layers.{l}"
        xn = ref.rms_norm(h, t[f"{p}.input_layernorm.weight"], eps)
        q = (xn @ t[f"{p}.self_attn.q_proj.weight"].T).reshape(n, nh, hd)
        k = (xn @ t[f"{p}.self_attn.k_proj.weight"].T).reshape(n, nkv, hd)
        v = (xn @ t[f"{p}.self_attn.v_proj.weight"].T).reshape(n, nkv, hd)
        q, k = ref.rope(q, cfg["rope_theta"]), ref.rope(k, cfg["rope_theta"])
        hpk = nh // nkv
        outs = np.zeros((n, nh, hd), dtype=np.float32)
        for hh in range(nh):
            kv = hh // hpk
            s = (q[:, hh] @ k[:, kv].T) * scale
            s = cap * np.tanh(s / cap)
            s = s + np.triu(np.full((n, n), -np.inf), 1)
            s -= s.max(-1, keepdims=True)
            e = np.exp(s)
            a = e / e.sum(-1, keepdims=True)
            outs[:, hh] = a @ v[:, kv]
        proj = outs.reshape(n, nh * hd) @ t[f"{p}.self_attn.o_proj.weight"].T
        h = h + ref.rms_norm(proj, t[f"{p}.post_attention_layernorm.weight"], eps)
        xn = ref.rms_norm(h, t[f"{p}.pre_feedforward_layernorm.weight"], eps)
        g = xn @ t[f"{p}.mlp.gate_proj.weight"].T
        u = xn @ t[f"{p}.mlp.up_proj.weight"].T
        dn = (ref.gelu_tanh(g) * u) @ t[f"{p}.mlp.down_proj.weight"].T
        h = h + ref.rms_norm(dn, t[f"{p}.post_feedforward_layernorm.weight"], eps)
    streams.append(h.copy())
    return ref.rms_norm(h, t["model.norm.weight"], eps).astype(np.float32), streams


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    root = sys.argv[1]
    sys.path.insert(0, os.path.join(root, "python"))
    import gemma_ref as ref
    for name, (cfg, wseed, ids) in CASES.items():
        t = gemma_model.make_tensors(cfg, wseed)
        out, streams = run_reference(ref, cfg, t, ids)
        np.savez_compressed(os.path.join(HERE, f"gemma_ref_{name}.npz"), weight_seed=wseed,
                            ids=np.array(ids, np.uint32), out=out, penultimate=streams[-2].astype(np.float32),
                            last_stream=streams[-1].astype(np.float32))
        print(name, "ids", len(ids), "-> hidden", out.shape, "mean |h|", float(np.abs(out).mean()))


if __name__ == "__main__":
    main()
