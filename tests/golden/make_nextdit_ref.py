"""Generate tests/golden/nextdit_ref_*.npz by running the reference's own numpy forward
(python/nextdit_ref.py, imported from the reference checkout) on seeded synthetic weights.

Run in the build container only:  python tests/golden/make_nextdit_ref.py /path/to/reference
The fixtures hold the inputs' seeds and the reference's output; the oracle must reproduce it.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from tests import synth  # noqa: E402


def run_reference(ref, cfg, tensors, latent, cap, t):
    """The body of nextdit_ref.main() with its module constants overridden for `cfg`."""
    hs = cfg["hidden_size"]
    ref.HID, ref.NH, ref.NKV = hs, cfg["num_attention_heads"], cfg["num_kv_heads"]
    ref.HD = hs // ref.NH
    ref.AXES_DIM = tuple(cfg["axes_dim_rope"])
    ref.EPS = cfg["norm_eps"]
    tt = {k[len("dit."):]: v for k, v in tensors.items()}
    C, H, W = latent.shape
    P = cfg["patch_size"]
    hp, wp = H // P, W // P
    cap_n = cap.shape[0]
    half = 128
    freqs = np.exp(-np.log(10000.0) * np.arange(half, dtype=np.float64) / half)
    ang = t * freqs
    emb = np.concatenate([np.cos(ang), np.sin(ang)]).astype(np.float32)
    pre = "time_caption_embed.timestep_embedder."
    temb = emb @ tt[pre + "linear_1.weight"].T + tt[pre + "linear_1.bias"]
    temb = ref.silu(temb) @ tt[pre + "linear_2.weight"].T + tt[pre + "linear_2.bias"]
    cap_e = ref.rms(cap, tt["time_caption_embed.caption_embedder.0.weight"]) \
        @ tt["time_caption_embed.caption_embedder.1.weight"].T + tt["time_caption_embed.caption_embedder.1.bias"]
    tok = latent.reshape(C, hp, P, wp, P).transpose(1, 3, 2, 4, 0).reshape(hp * wp, P * P * C)
    img = tok @ tt["x_embedder.weight"].T + tt["x_embedder.bias"]
    cap_ids = np.stack([np.arange(cap_n), np.zeros(cap_n), np.zeros(cap_n)], 1).astype(np.int32)
    rr, cc = np.divmod(np.arange(hp * wp), wp)
    img_ids = np.stack([np.full(hp * wp, cap_n), rr, cc], 1).astype(np.int32)
    cap_tab, img_tab = ref.rope_table(cap_ids), ref.rope_table(img_ids)
    for l in range(cfg["num_refiner_layers"]):
        cap_e = ref.block(tt, cap_e, f"context_refiner.{l}", cap_tab)
    for l in range(cfg["num_refiner_layers"]):
        img = ref.block(tt, img, f"noise_refiner.{l}", img_tab, temb)
    x = np.concatenate([cap_e, img], 0)
    tab = np.concatenate([cap_tab, img_tab], 0)
    taps = []
    for l in range(cfg["num_layers"]):
        x = ref.block(tt, x, f"layers.{l}", tab, temb)
        taps.append(x.astype(np.float32))
    scale = ref.silu(temb) @ tt["norm_out.linear_1.weight"].T + tt["norm_out.linear_1.bias"]
    x64 = x.astype(np.float64)
    xn = ((x64 - x64.mean(-1, keepdims=True)) / np.sqrt(x64.var(-1, keepdims=True) + 1e-6)).astype(np.float32)
    out = (xn * (1.0 + scale)) @ tt["norm_out.linear_2.weight"].T + tt["norm_out.linear_2.bias"]
    pred = out[cap_n:].reshape(hp, wp, P, P, C).transpose(4, 0, 2, 1, 3).reshape(C, H, W)
    return pred.astype(np.float32), taps


CASES = {
    # name: (cfg, weight seed, norm jitter, weight std, input seed, H, W, cap_n, t)
    "tiny": (synth.TINY, 0, 0.0, 0.02, 0, 32, 32, 32, 0.5),
    "tiny_ragged": (synth.TINY, 3, 0.1, 0.05, 4, 12, 20, 7, 0.7),
}


def inputs(cfg, seed, H, W, cap_n):
    rng = np.random.default_rng(seed)
    latent = rng.standard_normal((cfg["in_channels"], H, W)).astype(np.float32)
    cap = rng.standard_normal((cap_n, cfg["cap_feat"])).astype(np.float32)
    return latent, cap


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    refroot = sys.argv[1]
    sys.path.insert(0, os.path.join(refroot, "python"))
    import nextdit_ref as ref
    for name, (cfg, wseed, jit, std, iseed, H, W, cap_n, t) in CASES.items():
        tensors = synth.make_tensors(cfg, wseed, jit, std)
        latent, cap = inputs(cfg, iseed, H, W, cap_n)
        pred, taps = run_reference(ref, cfg, tensors, latent, cap, t)
        np.savez_compressed(os.path.join(HERE, f"nextdit_ref_{name}.npz"), pred=pred,
                            last_block=taps[-1], first_block=taps[0])
        print(name, pred.shape, float(np.abs(pred).mean()))


if __name__ == "__main__":
    main()
