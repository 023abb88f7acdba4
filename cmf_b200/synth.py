"""Synthetic NextDiT containers for benchmarks and demos: random-init weights N(0, std) are
generated AND quantized on the device (byte-identical to the reference encoders), then written
as a regular .cmf file that the library memory-maps like any packed model."""
import os

import numpy as np

from . import gpu
from .container import CmfWriter, DT_F32, DT_Q4TP, DT_Q4_TILED, DT_Q8_ROW

# Lumina-Image-2.0 geometry (2.6 B parameters)
LUMINA2 = dict(hidden_size=2304, num_layers=26, num_refiner_layers=2, num_attention_heads=24, num_kv_heads=8,
               in_channels=16, patch_size=2, axes_dim_rope=[32, 32, 32], norm_eps=1e-5, inter=9216, cap_feat=2304)
TINY = dict(hidden_size=256, num_layers=2, num_refiner_layers=2, num_attention_heads=4, num_kv_heads=4,
            in_channels=16, patch_size=2, axes_dim_rope=[32, 16, 16], norm_eps=1e-5, inter=1024, cap_feat=256)

CODECS = {"q8": DT_Q8_ROW, "q4t": DT_Q4_TILED, "q4tp": DT_Q4TP, "f32": DT_F32}


def tensor_list(cfg, attn, ffn):
    """[(name, dtype id, shape, kind)] in the order the reference's packer would emit
    (crates/cortiq-cli/src/imagepack.rs:156-178): modulation linears q8_row, attention / FFN /
    caption projections at the chosen level, everything else f32.  kind: 'w' weight ~N(0,std),
    'b' bias ~N(0,std), 'n' norm weight (ones)."""
    hs, nh, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_kv_heads"]
    hd = hs // nh
    inter, cap_feat = cfg["inter"], cfg["cap_feat"]
    pv = cfg["patch_size"] ** 2 * cfg["in_channels"]
    temb = min(hs, 1024)
    out = [("dit.x_embedder.weight", DT_F32, (hs, pv), "w"), ("dit.x_embedder.bias", DT_F32, (hs,), "b")]
    p = "dit.time_caption_embed."
    out += [(p + "timestep_embedder.linear_1.weight", DT_F32, (temb, 256), "w"),
            (p + "timestep_embedder.linear_1.bias", DT_F32, (temb,), "b"),
            (p + "timestep_embedder.linear_2.weight", DT_F32, (temb, temb), "w"),
            (p + "timestep_embedder.linear_2.bias", DT_F32, (temb,), "b"),
            (p + "caption_embedder.0.weight", DT_F32, (cap_feat,), "n"),
            (p + "caption_embedder.1.weight", attn, (hs, cap_feat), "w"),
            (p + "caption_embedder.1.bias", DT_F32, (hs,), "b")]
    for group, count, modulated in (("context_refiner", cfg["num_refiner_layers"], False),
                                    ("noise_refiner", cfg["num_refiner_layers"], True),
                                    ("layers", cfg["num_layers"], True)):
        for l in range(count):
            b = f"dit.{group}.{l}"
            if modulated:
                out += [(b + ".norm1.linear.weight", DT_Q8_ROW, (4 * hs, temb), "w"),
                        (b + ".norm1.linear.bias", DT_F32, (4 * hs,), "b"),
                        (b + ".norm1.norm.weight", DT_F32, (hs,), "n")]
            else:
                out += [(b + ".norm1.weight", DT_F32, (hs,), "n")]
            out += [(b + ".attn.to_q.weight", attn, (nh * hd, hs), "w"), (b + ".attn.to_k.weight", attn, (nkv * hd, hs), "w"),
                    (b + ".attn.to_v.weight", attn, (nkv * hd, hs), "w"), (b + ".attn.to_out.0.weight", attn, (hs, nh * hd), "w"),
                    (b + ".attn.norm_q.weight", DT_F32, (hd,), "n"), (b + ".attn.norm_k.weight", DT_F32, (hd,), "n"),
                    (b + ".norm2.weight", DT_F32, (hs,), "n"), (b + ".ffn_norm1.weight", DT_F32, (hs,), "n"),
                    (b + ".feed_forward.linear_1.weight", ffn, (inter, hs), "w"),
                    (b + ".feed_forward.linear_3.weight", ffn, (inter, hs), "w"),
                    (b + ".feed_forward.linear_2.weight", ffn, (hs, inter), "w"),
                    (b + ".ffn_norm2.weight", DT_F32, (hs,), "n")]
    out += [("dit.norm_out.linear_1.weight", DT_F32, (hs, temb), "w"), ("dit.norm_out.linear_1.bias", DT_F32, (hs,), "b"),
            ("dit.norm_out.linear_2.weight", DT_F32, (pv, hs), "w"), ("dit.norm_out.linear_2.bias", DT_F32, (pv,), "b")]
    return out


def write_model(path, cfg, attn="q8", ffn="q8", seed=0, std=0.02):
    """Write a synthetic model; every tensor's values are a pure function of (seed, position in
    the list), so two ranks writing the same arguments produce identical files."""
    attn, ffn = CODECS[attn], CODECS[ffn]
    w = CmfWriter(arch={"arch_name": "nextdit-synth", "hidden_size": cfg["hidden_size"],
                        "num_layers": cfg["num_layers"], "vocab_size": 0}, quant_type="mixed")
    for i, (name, dt, shape, kind) in enumerate(tensor_list(cfg, attn, ffn)):
        if kind == "n":
            w.add_f32(name, np.ones(shape, np.float32))
            continue
        rows, cols = (shape[0], shape[1]) if len(shape) == 2 else (1, shape[0])
        payload = gpu.encode_random(dt, seed * 100003 + i + 1, std, rows, cols)
        w.add(name, dt, shape, payload)
    cj = {k: cfg[k] for k in ("hidden_size", "num_layers", "num_refiner_layers", "num_attention_heads",
                              "num_kv_heads", "in_channels", "patch_size", "axes_dim_rope", "norm_eps")}
    w.add_json("dit.config_json", cj)
    tmp = path + f".tmp{os.getpid()}"
    w.write(tmp, hash_tensors=False)
    os.replace(tmp, path)
    return path


# ---------------------------------------------------------------------------------------------
# Synthetic FLUX-class VAE decoder (diffusers AutoencoderKL naming, crates/cortiq-engine/src/vae.rs
# from_tensors :549-633).  Host numpy only: about 50 M parameters at full size.
FLUX_VAE = dict(block_out_channels=[128, 256, 512, 512], layers_per_block=2, latent_channels=16, norm_num_groups=32,
                scaling_factor=0.3611, shift_factor=0.1159, out_channels=3)
TINY_VAE = dict(block_out_channels=[32, 64], layers_per_block=1, latent_channels=16, norm_num_groups=32,
                scaling_factor=0.3611, shift_factor=0.1159, out_channels=3)


def vae_tensor_list(cfg):
    """[(name without the 'vae.' prefix, shape, kind)]; kind 'k' conv kernel, 'l' linear weight,
    'b' bias, 'g' norm gain, 'h' norm shift."""
    rev = list(reversed(cfg["block_out_channels"]))
    out = []

    def conv(n, oc, ic, k):
        out.append((n + ".weight", (oc, ic, k, k), "k"))
        out.append((n + ".bias", (oc,), "b"))

    def norm(n, c):
        out.append((n + ".weight", (c,), "g"))
        out.append((n + ".bias", (c,), "h"))

    def resnet(n, cin, cout):
        norm(n + ".norm1", cin)
        conv(n + ".conv1", cout, cin, 3)
        norm(n + ".norm2", cout)
        conv(n + ".conv2", cout, cout, 3)
        if cin != cout:
            conv(n + ".conv_shortcut", cout, cin, 1)

    c0 = rev[0]
    conv("decoder.conv_in", c0, cfg["latent_channels"], 3)
    resnet("decoder.mid_block.resnets.0", c0, c0)
    a = "decoder.mid_block.attentions.0"
    norm(a + ".group_norm", c0)
    for p in ("to_q", "to_k", "to_v", "to_out.0"):
        out.append((f"{a}.{p}.weight", (c0, c0), "l"))
        out.append((f"{a}.{p}.bias", (c0,), "b"))
    resnet("decoder.mid_block.resnets.1", c0, c0)
    prev = c0
    for b, ch in enumerate(rev):
        for r in range(cfg["layers_per_block"] + 1):
            resnet(f"decoder.up_blocks.{b}.resnets.{r}", prev if r == 0 else ch, ch)
        prev = ch
        if b != len(rev) - 1:
            conv(f"decoder.up_blocks.{b}.upsamplers.0.conv", ch, ch, 3)
    norm("decoder.conv_norm_out", prev)
    conv("decoder.conv_out", cfg["out_channels"], prev, 3)
    return out


def vae_tensors(cfg, seed=0):
    """{name: f32 array} of a synthetic decoder.  Conv kernels are rounded to f16 values (the
    packer stores them as f16, crates/cortiq-cli/src/imagepack.rs:181-205), scaled so that
    activations keep unit order of magnitude through the stack."""
    rng = np.random.default_rng(seed * 7919 + 17)
    t = {}
    for name, shape, kind in vae_tensor_list(cfg):
        if kind == "k":
            fan_in = shape[1] * shape[2] * shape[3]
            a = rng.standard_normal(shape, np.float32) * np.float32(1.0 / np.sqrt(fan_in))
            a = a.astype(np.float16).astype(np.float32)
        elif kind == "l":
            a = rng.standard_normal(shape, np.float32) * np.float32(1.0 / np.sqrt(shape[1]))
        elif kind == "g":
            a = 1.0 + 0.1 * rng.standard_normal(shape, np.float32)
        else:
            a = 0.05 * rng.standard_normal(shape, np.float32)
        t[name] = a.astype(np.float32)
    return t


def vae_config_json(cfg):
    return {k: cfg[k] for k in ("block_out_channels", "layers_per_block", "latent_channels", "norm_num_groups",
                                "scaling_factor", "shift_factor", "out_channels")}


def add_vae(writer, cfg, seed=0):
    """Append vae.* tensors and vae.config_json to a CmfWriter: 4-D kernels as f16, the rest f32."""
    from .container import DT_F16
    for name, a in vae_tensors(cfg, seed).items():
        if a.ndim == 4:
            h = np.ascontiguousarray(a.astype(np.float16))
            writer.add("vae." + name, DT_F16, a.shape, h.view(np.uint8).reshape(-1))
        else:
            writer.add_f32("vae." + name, a)
    writer.add_json("vae.config_json", vae_config_json(cfg))


def write_vae_model(path, cfg, seed=0):
    w = CmfWriter(arch={"arch_name": "flux-vae-synth", "hidden_size": 0, "num_layers": 0, "vocab_size": 0},
                  quant_type="f16")
    add_vae(w, cfg, seed)
    tmp = path + f".tmp{os.getpid()}"
    w.write(tmp, hash_tensors=False)
    os.replace(tmp, path)
    return path


# ---------------------------------------------------------------------------------------------
# Synthetic Gemma-2 prompt encoder (te.* names of crates/cortiq-engine/src/textenc.rs:172-216;
# packing rules of crates/cortiq-cli/src/imagepack.rs:129-152: embedding q8_row, *_proj weights
# at the chosen level, norms f32).
GEMMA2_2B = dict(hidden_size=2304, num_hidden_layers=26, num_attention_heads=8, num_key_value_heads=4, head_dim=256,
                 intermediate_size=9216, vocab_size=256000, query_pre_attn_scalar=256, attn_logit_softcapping=50.0,
                 rope_theta=10000.0, rms_norm_eps=1e-6, sliding_window=4096)
TINY_GEMMA = dict(hidden_size=256, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                  intermediate_size=1024, vocab_size=512, query_pre_attn_scalar=64, attn_logit_softcapping=50.0,
                  rope_theta=10000.0, rms_norm_eps=1e-6, sliding_window=4096)


def gemma_tensor_list(cfg, level):
    """[(name, dtype id, shape, kind)]; kind 'w' projection ~N(0, std), 'e' embedding, 'n' norm weight."""
    hs, nh, nkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    inter = cfg["intermediate_size"]
    out = [("te.embed_tokens.weight", DT_Q8_ROW, (cfg["vocab_size"], hs), "e")]
    for l in range(cfg["num_hidden_layers"]):
        p = f"te.layers.{l}"
        out += [(p + ".input_layernorm.weight", DT_F32, (hs,), "n"),
                (p + ".self_attn.q_proj.weight", level, (nh * hd, hs), "w"),
                (p + ".self_attn.k_proj.weight", level, (nkv * hd, hs), "w"),
                (p + ".self_attn.v_proj.weight", level, (nkv * hd, hs), "w"),
                (p + ".self_attn.o_proj.weight", level, (hs, nh * hd), "w"),
                (p + ".post_attention_layernorm.weight", DT_F32, (hs,), "n"),
                (p + ".pre_feedforward_layernorm.weight", DT_F32, (hs,), "n"),
                (p + ".mlp.gate_proj.weight", level, (inter, hs), "w"),
                (p + ".mlp.up_proj.weight", level, (inter, hs), "w"),
                (p + ".mlp.down_proj.weight", level, (hs, inter), "w"),
                (p + ".post_feedforward_layernorm.weight", DT_F32, (hs,), "n")]
    out.append(("te.norm.weight", DT_F32, (hs,), "n"))
    return out


def add_gemma(writer, cfg, level="q4t", seed=0, std=0.02):
    """Append te.* tensors (random-init, quantized on the device) and te.config_json."""
    lvl = CODECS[level]
    for i, (name, dt, shape, kind) in enumerate(gemma_tensor_list(cfg, lvl)):
        if kind == "n":
            rng = np.random.default_rng(seed * 7907 + i)
            writer.add_f32(name, (0.1 * rng.standard_normal(shape)).astype(np.float32))
            continue
        s = std if kind == "w" else 1.0 / np.sqrt(cfg["hidden_size"])
        writer.add(name, dt, shape, gpu.encode_random(dt, seed * 100019 + i + 1, float(s), shape[0], shape[1]))
    writer.add_json("te.config_json", {k: cfg[k] for k in (
        "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim", "intermediate_size",
        "vocab_size", "query_pre_attn_scalar", "attn_logit_softcapping", "rope_theta", "rms_norm_eps", "sliding_window")})


def write_gemma_model(path, cfg, level="q4t", seed=0):
    w = CmfWriter(arch={"arch_name": "gemma2-encoder-synth", "hidden_size": cfg["hidden_size"],
                        "num_layers": cfg["num_hidden_layers"], "vocab_size": cfg["vocab_size"]}, quant_type="mixed")
    add_gemma(w, cfg, level, seed)
    tmp = path + f".tmp{os.getpid()}"
    w.write(tmp, hash_tensors=False)
    os.replace(tmp, path)
    return path
