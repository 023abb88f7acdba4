"""CPU restatement of the FLUX-class VAE decoder.  TEST INFRASTRUCTURE: only tests, the smoke
check and the benchmark's CPU-baseline leg may import this module; the product never does.

Follows crates/cortiq-engine/src/vae.rs (Conv2d::apply :153-250, GroupNorm::apply :270-294, silu
:297-311, upsample2x :314-327, ResnetBlock::apply :337-400, AttnBlock::apply :415-489,
VaeDecoder::decode :637-690), whose own parity reference is python/vae_ref.py.  Pinned against
outputs of python/vae_ref.py on synthetic weights (tests/golden/make_vae_ref.py) and against the
known-answer tests of vae.rs:700-755.

Tensors are NCHW float32; matrix products accumulate in float64 (vae_ref.py:47, a superset of the
engine's f32 accumulation) and are rounded to float32 once.
"""
import numpy as np


def conv2d(x, w, b):
    """x [ic, h, w], w [oc, ic, k, k], b [oc] -> [oc, h, w]; zero padding k // 2 (vae.rs:153)."""
    oc, ic, k, _ = w.shape
    c, h, ww = x.shape
    assert c == ic
    pad = k // 2
    xp = np.pad(x.astype(np.float64), ((0, 0), (pad, pad), (pad, pad)))
    y = np.zeros((oc, h * ww), np.float64)
    w64 = w.astype(np.float64)
    for ky in range(k):
        for kx in range(k):
            y += w64[:, :, ky, kx] @ xp[:, ky:ky + h, kx:kx + ww].reshape(ic, -1)
    return (y + b.astype(np.float64)[:, None]).reshape(oc, h, ww).astype(np.float32)


def group_norm(x, w, b, groups=32):
    """vae.rs:270-294: f64 mean / variance per group, eps 1e-6; the normalized value is rounded
    to f32 before the f32 affine."""
    c, h, ww = x.shape
    per = c // groups
    y = x.reshape(groups, per * h * ww).astype(np.float64)
    mean = y.mean(axis=1, keepdims=True)
    var = ((y - mean) ** 2).mean(axis=1, keepdims=True)
    inv = 1.0 / np.sqrt(var + 1e-6)
    n = ((y - mean) * inv).astype(np.float32).reshape(c, h, ww)
    return n * w.astype(np.float32)[:, None, None] + b.astype(np.float32)[:, None, None]


def silu(x):
    """vae.rs:297: v / (1 + exp(-v)) in f32."""
    x = x.astype(np.float32)
    with np.errstate(over="ignore"):
        return (x / (np.float32(1.0) + np.exp(-x))).astype(np.float32)


def upsample2x(x):
    """vae.rs:314: nearest neighbour."""
    return np.repeat(np.repeat(x, 2, axis=1), 2, axis=2)


def resnet(t, n, x, groups=32):
    """vae.rs:337-400."""
    h = conv2d(silu(group_norm(x, t[f"{n}.norm1.weight"], t[f"{n}.norm1.bias"], groups)),
               t[f"{n}.conv1.weight"], t[f"{n}.conv1.bias"])
    h = conv2d(silu(group_norm(h, t[f"{n}.norm2.weight"], t[f"{n}.norm2.bias"], groups)),
               t[f"{n}.conv2.weight"], t[f"{n}.conv2.bias"])
    if f"{n}.conv_shortcut.weight" in t:
        x = conv2d(x, t[f"{n}.conv_shortcut.weight"], t[f"{n}.conv_shortcut.bias"])
    return (x + h).astype(np.float32)


def attention(t, n, x, groups=32):
    """vae.rs:415-489: one head over the h*w tokens, head dimension = channels."""
    c, h, ww = x.shape
    hw = h * ww
    xn = group_norm(x, t[f"{n}.group_norm.weight"], t[f"{n}.group_norm.bias"], groups)
    tok = xn.reshape(c, hw).T.astype(np.float64)                       # [hw, c]

    def proj(p, a):
        return (a @ t[f"{n}.{p}.weight"].astype(np.float64).T + t[f"{n}.{p}.bias"].astype(np.float64)).astype(np.float32)

    q, k, v = proj("to_q", tok), proj("to_k", tok), proj("to_v", tok)
    scale = np.float32(1.0) / np.sqrt(np.float32(c))
    s = ((q.astype(np.float64) @ k.astype(np.float64).T) * np.float64(scale)).astype(np.float32)
    s = s - s.max(axis=1, keepdims=True)
    e = np.exp(s).astype(np.float32)
    p = e * (np.float32(1.0) / e.sum(axis=1, keepdims=True, dtype=np.float32))
    o = (p.astype(np.float64) @ v.astype(np.float64)).astype(np.float32)  # [hw, c]
    o = proj("to_out.0", o.astype(np.float64))
    return (x + o.T.reshape(c, h, ww)).astype(np.float32)


def decode(t, cfg, z, taps=None):
    """vae.rs:637-690.  t: {name: array} without the 'vae.' prefix; z [latent_channels, h, w] at
    model scale.  ``taps`` (a list) receives the activation after every stage."""
    g = int(cfg.get("norm_num_groups", 32))
    x = (z.astype(np.float32) / np.float32(cfg.get("scaling_factor", 1.0)) + np.float32(cfg.get("shift_factor", 0.0)))
    x = conv2d(x.astype(np.float32), t["decoder.conv_in.weight"], t["decoder.conv_in.bias"])
    note = (lambda name, a: taps.append((name, a))) if taps is not None else (lambda name, a: None)
    note("conv_in", x)
    x = resnet(t, "decoder.mid_block.resnets.0", x, g)
    note("mid_res1", x)
    x = attention(t, "decoder.mid_block.attentions.0", x, g)
    note("mid_attn", x)
    x = resnet(t, "decoder.mid_block.resnets.1", x, g)
    note("mid_res2", x)
    b = 0
    while f"decoder.up_blocks.{b}.resnets.0.conv1.weight" in t:
        r = 0
        while f"decoder.up_blocks.{b}.resnets.{r}.conv1.weight" in t:
            x = resnet(t, f"decoder.up_blocks.{b}.resnets.{r}", x, g)
            r += 1
        up = f"decoder.up_blocks.{b}.upsamplers.0.conv"
        if f"{up}.weight" in t:
            x = conv2d(upsample2x(x), t[f"{up}.weight"], t[f"{up}.bias"])
        note(f"up{b}", x)
        b += 1
    x = silu(group_norm(x, t["decoder.conv_norm_out.weight"], t["decoder.conv_norm_out.bias"], g))
    return conv2d(x, t["decoder.conv_out.weight"], t["decoder.conv_out.bias"])
