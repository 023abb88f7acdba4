"""The VAE oracle (oracle/vae.py) against the fixtures generated from the reference's numpy
decoder (tests/golden/make_vae_ref.py) and the known-answer tests of
crates/cortiq-engine/src/vae.rs:700-755.  No GPU."""
import os

import numpy as np
import pytest

from cmf_b200 import synth
from oracle import vae as ovae

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("case", ["tiny", "tiny_ragged"])
def test_oracle_matches_reference_decoder(case):
    g = np.load(os.path.join(GOLD, f"vae_ref_{case}.npz"))
    t = synth.vae_tensors(synth.TINY_VAE, int(g["weight_seed"]))
    taps = []
    out = ovae.decode(t, synth.TINY_VAE, g["z"], taps=taps)
    for name, a in taps:
        key = "tap_" + name
        if key in g.files:
            assert np.abs(a - g[key]).max() < 2e-5, name
    assert out.shape == g["out"].shape
    # the reference test's own bar is 2e-3 (crates/cortiq-engine/tests/vae_parity.rs:46)
    assert np.abs(out - g["out"]).max() < 2e-5


def test_conv2d_known_answer():
    # vae.rs:701-719
    w = np.ones((1, 1, 3, 3), np.float32)
    b = np.array([0.5], np.float32)
    x = np.arange(1, 10, dtype=np.float32).reshape(1, 3, 3)
    y = ovae.conv2d(x, w, b).reshape(-1)
    assert y[4] == 45.5 and y[0] == 12.5 and y[8] == 5 + 6 + 8 + 9 + 0.5


def test_group_norm_known_answer():
    # vae.rs:722-736
    x = np.array([1, 3, 5, 7, 10, 10, 10, 10], np.float32).reshape(2, 2, 2)
    y = ovae.group_norm(x, np.array([2.0, 1.0], np.float32), np.array([0.0, 3.0], np.float32), groups=2).reshape(-1)
    assert abs(float(y[0]) - (-3.0 / np.sqrt(5.0) * 2.0)) < 1e-5
    assert abs(float(y[4]) - 3.0) < 1e-4


def test_upsample_known_answer():
    # vae.rs:739-750
    y = ovae.upsample2x(np.array([1, 2, 3, 4], np.float32).reshape(1, 2, 2)).reshape(-1)
    assert y.tolist() == [1, 1, 2, 2, 1, 1, 2, 2, 3, 3, 4, 4, 3, 3, 4, 4]


def test_synthetic_decoder_lists_the_tensors_the_loader_wants():
    # names resolved by VaeDecoder::from_tensors (vae.rs:549-633)
    names = {n for n, _, _ in synth.vae_tensor_list(synth.FLUX_VAE)}
    for n in ("decoder.conv_in.weight", "decoder.mid_block.attentions.0.to_out.0.bias",
              "decoder.up_blocks.2.resnets.0.conv_shortcut.weight", "decoder.up_blocks.2.upsamplers.0.conv.weight",
              "decoder.up_blocks.3.resnets.2.conv2.weight", "decoder.conv_norm_out.weight", "decoder.conv_out.bias"):
        assert n in names
    assert "decoder.up_blocks.3.upsamplers.0.conv.weight" not in names
    assert "decoder.up_blocks.0.resnets.0.conv_shortcut.weight" not in names
    n_params = sum(int(np.prod(s)) for _, s, _ in synth.vae_tensor_list(synth.FLUX_VAE))
    assert 45e6 < n_params < 55e6
