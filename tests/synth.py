"""Seeded synthetic NextDiT weights for the tests (names as the reference's loader expects,
crates/cortiq-engine/src/dit.rs:510-589)."""
import numpy as np

TINY = dict(hidden_size=256, num_layers=2, num_refiner_layers=2, num_attention_heads=4,
            num_kv_heads=4, in_channels=16, patch_size=2, axes_dim_rope=[32, 16, 16],
            norm_eps=1e-5, inter=1024, cap_feat=256)

# Lumina-2 geometry with a reduced layer count: same head_dim 96, GQA 24/8, SwiGLU 9216.
LUMINA_GEOM = dict(hidden_size=2304, num_layers=2, num_refiner_layers=1, num_attention_heads=24,
                   num_kv_heads=8, in_channels=16, patch_size=2, axes_dim_rope=[32, 32, 32],
                   norm_eps=1e-5, inter=9216, cap_feat=2304)


def block_names(pfx, modulated):
    names = [f"{pfx}.attn.to_q.weight", f"{pfx}.attn.to_k.weight", f"{pfx}.attn.to_v.weight",
             f"{pfx}.attn.to_out.0.weight", f"{pfx}.feed_forward.linear_1.weight",
             f"{pfx}.feed_forward.linear_3.weight", f"{pfx}.feed_forward.linear_2.weight"]
    return names


def make_tensors(cfg, seed=0, norm_jitter=0.0, std=0.02):
    """dict name -> f32 array.  2-D weights and biases ~ N(0, std); norm weights 1 (+ jitter)."""
    rng = np.random.default_rng(seed)
    hs, nh, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_kv_heads"]
    hd = hs // nh
    inter, cap_feat = cfg["inter"], cfg["cap_feat"]
    pv = cfg["patch_size"] ** 2 * cfg["in_channels"]
    temb = min(hs, 1024)
    t = {}

    def mat(r, c):
        return (rng.standard_normal((r, c)) * std).astype(np.float32)

    def vec(n):
        return (rng.standard_normal(n) * std).astype(np.float32)

    def norm(n):
        return (1.0 + norm_jitter * rng.standard_normal(n)).astype(np.float32)

    t["dit.x_embedder.weight"] = mat(hs, pv)
    t["dit.x_embedder.bias"] = vec(hs)
    pre = "dit.time_caption_embed."
    t[pre + "timestep_embedder.linear_1.weight"] = mat(temb, 256)
    t[pre + "timestep_embedder.linear_1.bias"] = vec(temb)
    t[pre + "timestep_embedder.linear_2.weight"] = mat(temb, temb)
    t[pre + "timestep_embedder.linear_2.bias"] = vec(temb)
    t[pre + "caption_embedder.0.weight"] = norm(cap_feat)
    t[pre + "caption_embedder.1.weight"] = mat(hs, cap_feat)
    t[pre + "caption_embedder.1.bias"] = vec(hs)
    for group, count, modulated in (("context_refiner", cfg["num_refiner_layers"], False),
                                    ("noise_refiner", cfg["num_refiner_layers"], True),
                                    ("layers", cfg["num_layers"], True)):
        for l in range(count):
            p = f"dit.{group}.{l}"
            if modulated:
                t[p + ".norm1.linear.weight"] = mat(4 * hs, temb)
                t[p + ".norm1.linear.bias"] = vec(4 * hs)
                t[p + ".norm1.norm.weight"] = norm(hs)
            else:
                t[p + ".norm1.weight"] = norm(hs)
            t[p + ".attn.to_q.weight"] = mat(nh * hd, hs)
            t[p + ".attn.to_k.weight"] = mat(nkv * hd, hs)
            t[p + ".attn.to_v.weight"] = mat(nkv * hd, hs)
            t[p + ".attn.to_out.0.weight"] = mat(hs, nh * hd)
            t[p + ".attn.norm_q.weight"] = norm(hd)
            t[p + ".attn.norm_k.weight"] = norm(hd)
            t[p + ".norm2.weight"] = norm(hs)
            t[p + ".ffn_norm1.weight"] = norm(hs)
            t[p + ".feed_forward.linear_1.weight"] = mat(inter, hs)
            t[p + ".feed_forward.linear_3.weight"] = mat(inter, hs)
            t[p + ".feed_forward.linear_2.weight"] = mat(hs, inter)
            t[p + ".ffn_norm2.weight"] = norm(hs)
    t["dit.norm_out.linear_1.weight"] = mat(hs, temb)
    t["dit.norm_out.linear_1.bias"] = vec(hs)
    t["dit.norm_out.linear_2.weight"] = mat(pv, hs)
    t["dit.norm_out.linear_2.bias"] = vec(pv)
    return t


def quant_plan(cfg, attn, ffn, mod=3, cap=None):
    """name -> dtype id for the projections a packer would quantize
    (crates/cortiq-cli/src/imagepack.rs:164-177 quantizes the modulation linear to q8_row
    always, and attention / feed-forward / caption projections to the chosen level)."""
    plan = {}
    for group, count, modulated in (("context_refiner", cfg["num_refiner_layers"], False),
                                    ("noise_refiner", cfg["num_refiner_layers"], True),
                                    ("layers", cfg["num_layers"], True)):
        for l in range(count):
            p = f"dit.{group}.{l}"
            if modulated:
                plan[p + ".norm1.linear.weight"] = mod
            for s in (".attn.to_q.weight", ".attn.to_k.weight", ".attn.to_v.weight", ".attn.to_out.0.weight"):
                plan[p + s] = attn
            for s in (".feed_forward.linear_1.weight", ".feed_forward.linear_3.weight", ".feed_forward.linear_2.weight"):
                plan[p + s] = ffn
    plan["dit.time_caption_embed.caption_embedder.1.weight"] = cap if cap is not None else attn
    return plan
