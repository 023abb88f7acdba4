"""VAE decoder on the device against the CPU oracle (oracle/vae.py) and the fixtures generated
from the reference's numpy decoder: the facade's stand-alone convolutions, the whole decoder at
tiny and FLUX channel widths, and size-independent properties at 1024x1024."""
import os

import numpy as np
import pytest

from oracle import vae as ovae
from tests.modelfile import rel_l2

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# The decoder is an f32 network: operands travel as f16 hi + lo planes (22 significand bits) and
# accumulate in f32, so the device differs from the f64-accumulating oracle by f32 rounding only.
CONV_TOL = 2e-5          # rel-L2 of one convolution: the tensor core's f32 accumulation over up to 4608 terms
PARITY_MAX_ABS = 2e-3    # the reference's own bar, crates/cortiq-engine/tests/vae_parity.rs:46


@pytest.mark.parametrize("ic,oc,h,w,k", [(32, 64, 8, 8, 3), (16, 32, 12, 20, 3), (64, 3, 16, 16, 3), (128, 130, 33, 17, 1),
                                          (96, 64, 40, 24, 3), (1, 1, 3, 3, 3), (512, 512, 16, 16, 3)])
def test_conv2d_matches_oracle(ic, oc, h, w, k):
    from cmf_b200 import vae
    rng = np.random.default_rng(ic * 1000 + oc)
    wt = (rng.standard_normal((oc, ic, k, k)) / np.sqrt(ic * k * k)).astype(np.float32)
    b = rng.standard_normal(oc).astype(np.float32)
    x = rng.standard_normal((ic, h, w)).astype(np.float32)
    got = vae.conv2d(wt, b, x, ic, oc, h, w, k)
    want = ovae.conv2d(x, wt, b)
    assert got.shape == want.shape
    assert rel_l2(got, want) < CONV_TOL
    assert np.abs(got - want).max() < 1e-4


def test_conv2d_known_answer():
    # crates/cortiq-engine/src/vae.rs:701-719
    from cmf_b200 import vae
    y = vae.conv2d(np.ones((1, 1, 3, 3), np.float32), np.array([0.5], np.float32),
                   np.arange(1, 10, dtype=np.float32).reshape(1, 3, 3), 1, 1, 3, 3, 3).reshape(-1)
    assert y[4] == 45.5 and y[0] == 12.5 and y[8] == 5 + 6 + 8 + 9 + 0.5


def test_conv2d_rejects_bad_arguments():
    from cmf_b200 import CmfCudaError, vae
    with pytest.raises(CmfCudaError):
        vae.conv2d(np.zeros((1, 1, 5, 5), np.float32), np.zeros(1, np.float32), np.zeros((1, 4, 4), np.float32), 1, 1, 4, 4, 5)
    with pytest.raises(CmfCudaError):
        vae.upsample_conv(np.zeros((8, 8, 3, 3), np.float32), np.zeros(8, np.float32), np.zeros((8, 4, 4), np.float32), 8, 8, 4, 4, 3)


@pytest.mark.parametrize("ic,oc,h,w", [(32, 32, 8, 8), (64, 96, 10, 6)])
def test_upsample_conv_matches_oracle(ic, oc, h, w):
    from cmf_b200 import vae
    rng = np.random.default_rng(5)
    wt = (rng.standard_normal((oc, ic, 3, 3)) / np.sqrt(ic * 9)).astype(np.float32)
    b = rng.standard_normal(oc).astype(np.float32)
    x = rng.standard_normal((ic, h, w)).astype(np.float32)
    got = vae.upsample_conv(wt, b, x, ic, oc, h, w, 3)
    want = ovae.conv2d(ovae.upsample2x(x), wt, b)
    assert rel_l2(got, want) < CONV_TOL


@pytest.mark.parametrize("case", ["tiny", "tiny_ragged"])
def test_decoder_matches_reference_fixture(tmp_path, case):
    from cmf_b200 import Model, VaeDecoder, synth
    g = np.load(os.path.join(GOLD, f"vae_ref_{case}.npz"))
    path = str(tmp_path / "vae.cmf")
    synth.write_vae_model(path, synth.TINY_VAE, int(g["weight_seed"]))
    z = g["z"]
    with Model(path) as m:
        dec = VaeDecoder(m)
        assert dec.latent_channels == 16 and dec.upscale == 2
        assert abs(dec.scaling_factor - 0.3611) < 1e-6 and abs(dec.shift_factor - 0.1159) < 1e-6
        out = dec.decode(z, z.shape[1], z.shape[2])
        again = dec.decode(z, z.shape[1], z.shape[2])
        dec.close()
    assert out.shape == g["out"].shape
    assert np.array_equal(out, again)
    assert np.abs(out - g["out"]).max() < PARITY_MAX_ABS
    assert rel_l2(out, g["out"]) < 1e-4


def test_decoder_flux_widths_matches_oracle(tmp_path):
    """Real channel widths (128/256/512/512, 3 upsamplers, 512-wide attention) on an 8x6 latent."""
    from cmf_b200 import Model, VaeDecoder, synth
    path = str(tmp_path / "vae.cmf")
    synth.write_vae_model(path, synth.FLUX_VAE, 1)
    t = synth.vae_tensors(synth.FLUX_VAE, 1)
    z = np.random.default_rng(2).standard_normal((16, 8, 6)).astype(np.float32)
    want = ovae.decode(t, synth.FLUX_VAE, z)
    with Model(path) as m:
        dec = VaeDecoder(m)
        assert dec.upscale == 8
        out = dec.decode(z, 8, 6)
        dec.close()
    assert out.shape == (3, 64, 48)
    assert np.abs(out - want).max() < PARITY_MAX_ABS
    assert rel_l2(out, want) < 1e-4


def test_decoder_rejects_a_container_without_vae(tmp_path):
    from cmf_b200 import CmfCudaError, CmfWriter, Model, VaeDecoder
    path = str(tmp_path / "empty.cmf")
    w = CmfWriter(arch={"arch_name": "none"})
    w.add_f32("x", np.zeros((2, 2), np.float32))
    w.write(path)
    with Model(path) as m:
        with pytest.raises(CmfCudaError):
            VaeDecoder(m)


def test_conv2d_full_size_linearity_and_samples():
    """The largest convolution of a 1024x1024 decode (128 -> 128 channels, 3x3, 1024 x 1024):
    linear in x, and equal to a direct f64 dot product at sampled outputs."""
    from cmf_b200 import vae
    ic = oc = 128
    h = w = 1024
    rng = np.random.default_rng(11)
    wt = (rng.standard_normal((oc, ic, 3, 3)) / np.sqrt(ic * 9)).astype(np.float16).astype(np.float32)
    b = rng.standard_normal(oc).astype(np.float32)
    x1 = rng.standard_normal((ic, h, w), np.float32)
    x2 = rng.standard_normal((ic, h, w), np.float32)
    y1 = vae.conv2d(wt, b, x1, ic, oc, h, w, 3)
    y2 = vae.conv2d(wt, b, x2, ic, oc, h, w, 3)
    y12 = vae.conv2d(wt, b, x1 + x2, ic, oc, h, w, 3)
    assert np.isfinite(y12).all()
    assert rel_l2(y1 + y2 - b[:, None, None], y12) < 1e-5
    xp = np.pad(x1, ((0, 0), (1, 1), (1, 1))).astype(np.float64)
    w64 = wt.astype(np.float64)
    for (o, yy, xx) in [(0, 0, 0), (127, 1023, 1023), (5, 0, 1023), (64, 511, 512), (17, 1023, 0), (99, 255, 256), (31, 16, 15)]:
        want = float((w64[o] * xp[:, yy:yy + 3, xx:xx + 3]).sum() + b[o])
        assert abs(float(y1[o, yy, xx]) - want) < 2e-5


def test_decoder_1024_runs_and_is_deterministic(tmp_path):
    """Full FLUX decoder on a 128x128 latent (1024x1024 image, 16384-token attention)."""
    from cmf_b200 import Model, VaeDecoder, synth
    path = str(tmp_path / "vae.cmf")
    synth.write_vae_model(path, synth.FLUX_VAE, 0)
    z = np.random.default_rng(3).standard_normal((16, 128, 128)).astype(np.float32)
    with Model(path) as m:
        dec = VaeDecoder(m)
        a = dec.decode(z, 128, 128)
        b = dec.decode(z, 128, 128)
        # the top-left of the image depends on the rest only through GroupNorm statistics and the
        # attention block: a latent with a different bottom-right corner changes it, but little
        z2 = z.copy()
        z2[:, 100:, 100:] += 0.5
        c = dec.decode(z2, 128, 128)
        dec.close()
    assert a.shape == (3, 1024, 1024) and np.isfinite(a).all()
    assert np.array_equal(a, b)
    assert not np.array_equal(a[:, :256, :256], c[:, :256, :256])
    assert a.std() > 1e-3


@pytest.mark.parametrize("n,c", [(256, 512), (100, 512), (64, 160)])
def test_dit_attention_single_wide_head(n, c):
    """gpu::dit_attention as the VAE's attention block calls it (crates/cortiq-engine/src/vae.rs:438):
    one head whose dimension is the channel count, f32 in and out."""
    from cmf_b200 import gpu
    rng = np.random.default_rng(n + c)
    q, k, v = (rng.standard_normal((n, c)).astype(np.float32) for _ in range(3))
    scale = 1.0 / np.sqrt(np.float32(c))
    out = np.empty((n, c), np.float32)
    assert gpu.dit_attention(q, k, v, 1, 1, n, c, float(scale), out)
    s = (q.astype(np.float64) @ k.astype(np.float64).T) * float(scale)
    s -= s.max(axis=1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=1, keepdims=True)
    want = (p @ v.astype(np.float64)).astype(np.float32)
    assert rel_l2(out, want) < 2e-5


def test_decoder_2048_runs(tmp_path):
    """A 256 x 256 latent (2048 x 2048 image): the 65536-token attention block no longer fits a score
    row in shared memory and takes the three-pass softmax; the largest activation is 4.3 GB."""
    from cmf_b200 import Model, VaeDecoder, synth
    path = str(tmp_path / "vae.cmf")
    synth.write_vae_model(path, synth.FLUX_VAE, 0)
    z = np.random.default_rng(4).standard_normal((16, 256, 256)).astype(np.float32)
    with Model(path) as m:
        dec = VaeDecoder(m)
        a = dec.decode(z, 256, 256)
        # same weights, the top-left quarter of the latent alone: GroupNorm statistics and attention
        # see different context, so only the order of magnitude is comparable
        b = dec.decode(z[:, :128, :128], 128, 128)
        dec.close()
    assert a.shape == (3, 2048, 2048) and np.isfinite(a).all()
    assert 0.5 < a.std() / b.std() < 2.0
