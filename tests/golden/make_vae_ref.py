"""Generate tests/golden/vae_ref_*.npz by running the reference's own numpy decoder
(python/vae_ref.py, imported from the reference checkout) on seeded synthetic weights.

Run in the build container only:  python tests/golden/make_vae_ref.py /path/to/reference
The fixtures hold the weights' seed, the latent and the reference's activations; the oracle
(oracle/vae.py) must reproduce them.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from cmf_b200 import synth  # noqa: E402

CASES = {
    # name: (config, weight seed, latent h, latent w, latent seed)
    "tiny": (synth.TINY_VAE, 3, 8, 8, 7),
    "tiny_ragged": (synth.TINY_VAE, 4, 6, 10, 8),
}


def run_reference(ref, cfg, t, z):
    """The body of vae_ref.main() after its file loading (python/vae_ref.py:107-127)."""
    taps = {}
    x = z / cfg["scaling_factor"] + cfg["shift_factor"]
    x = ref.conv2d(x, t["decoder.conv_in.weight"], t["decoder.conv_in.bias"])
    taps["conv_in"] = x
    x = ref.resnet(t, "decoder.mid_block.resnets.0", x)
    taps["mid_res1"] = x
    x = ref.attn(t, "decoder.mid_block.attentions.0", x)
    taps["mid_attn"] = x
    x = ref.resnet(t, "decoder.mid_block.resnets.1", x)
    b = 0
    while f"decoder.up_blocks.{b}.resnets.0.conv1.weight" in t:
        r = 0
        while f"decoder.up_blocks.{b}.resnets.{r}.conv1.weight" in t:
            x = ref.resnet(t, f"decoder.up_blocks.{b}.resnets.{r}", x)
            r += 1
        upn = f"decoder.up_blocks.{b}.upsamplers.0.conv"
        if f"{upn}.weight" in t:
            x = ref.conv2d(ref.upsample2x(x), t[f"{upn}.weight"], t[f"{upn}.bias"])
        taps[f"up{b}"] = x
        b += 1
    x = ref.silu(ref.group_norm(x, t["decoder.conv_norm_out.weight"], t["decoder.conv_norm_out.bias"]))
    x = ref.conv2d(x, t["decoder.conv_out.weight"], t["decoder.conv_out.bias"])
    return x.astype(np.float32), taps


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    root = sys.argv[1]
    sys.path.insert(0, os.path.join(root, "python"))
    import vae_ref as ref
    for name, (cfg, wseed, h, w, zseed) in CASES.items():
        t = synth.vae_tensors(cfg, wseed)
        z = np.random.default_rng(zseed).standard_normal((cfg["latent_channels"], h, w)).astype(np.float32)
        out, taps = run_reference(ref, cfg, t, z)
        np.savez_compressed(os.path.join(HERE, f"vae_ref_{name}.npz"), weight_seed=wseed, z=z, out=out,
                            **{"tap_" + k: v.astype(np.float32) for k, v in taps.items()})
        print(name, "latent", z.shape, "->", out.shape, "range", float(out.min()), float(out.max()))


if __name__ == "__main__":
    main()
