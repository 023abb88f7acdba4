"""Depth and step count at Lumina width against the CPU oracle: error growth of the hidden state
through all 26 joint blocks of a Lumina-2-size model, and of the latents through a 30-step Euler
loop.  Tolerance: relative L2 <= 1e-2 per block output, per velocity and per denoised latent (the
bar of crates/cortiq-engine/tests/dit_parity.rs:44-55 is a whole-forward comparison; the loop is
crates/cortiq-engine/src/imagegen.rs:143-217).

The 2.6 B-parameter model is generated and quantized on the device (byte-identical to the oracle's
encoders, tests/test_gpu_codecs.py) and read back from the container for the oracle, which
dequantizes each projection when it uses it."""
import os

import numpy as np
import pytest

from oracle import codecs as oc
from oracle import nextdit as nd
from tests import synth as tsynth
from tests.modelfile import build, load_for_oracle, rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.mark.parametrize("attn,ffn", [("q4t", "q4t"), ("q8", "q4tp")])
def test_lumina_full_depth_per_block_and_velocity(tmp_path, attn, ffn):
    """All 26 joint + 2 + 2 refiner layers at hidden 2304, a 32x32 latent (256 image tokens) with 40
    / 9 caption tokens: x after every joint block and both predicted velocities."""
    from cmf_b200 import Model, NextDit, synth
    path = os.path.join(str(tmp_path), "lumina.cmf")
    synth.write_model(path, synth.LUMINA2, attn=attn, ffn=ffn, seed=0)
    tensors, cfg = load_for_oracle(path, cache=False)
    assert cfg["num_layers"] == 26 and cfg["num_refiner_layers"] == 2
    orc = nd.NextDitOracle(tensors, cfg)
    rng = np.random.default_rng(0)
    h = w = 32
    latent = rng.standard_normal((16, h, w)).astype(np.float32)
    cap = rng.standard_normal((40, 2304)).astype(np.float32)
    cap_u = rng.standard_normal((9, 2304)).astype(np.float32)
    wc, wu = orc.refine_caption(cap), orc.refine_caption(cap_u)
    orc.block_taps = []
    oc_, ou_ = orc.forward_cfg_pair(latent, h, w, wc, wu, 0.5)
    joint = [x for p, x in orc.block_taps if p.startswith("dit.layers")]
    assert len(joint) == 26
    with Model(path) as m:
        dit = NextDit(m)
        cc = dit.refine_caption(cap)
        pc, pu, taps = dit.forward_cfg_pair(latent, h, w, wc, 40, wu, 9, 0.5, taps=True)
        dit.close()
    errs = [rel_l2(taps[l], joint[l]) for l in range(26)]
    print(f"\n[{attn} attention / {ffn} FFN] rel-L2 of x after joint block 1..26: "
          + " ".join(f"{e:.2e}" for e in errs))
    print(f"  refine_caption {rel_l2(cc, wc):.2e}; velocity cond {rel_l2(pc, oc_):.2e}, uncond {rel_l2(pu, ou_):.2e}")
    assert rel_l2(cc, wc) < TOL
    assert max(errs) < TOL, errs
    assert rel_l2(pc, oc_) < TOL and rel_l2(pu, ou_) < TOL, (rel_l2(pc, oc_), rel_l2(pu, ou_))


def test_euler_30_steps_tiny(tmp_path):
    """The engine's default 30 steps with CFG on the tiny model: final latent against the oracle's
    loop, and the error after every step (it must not build up beyond the bar)."""
    from cmf_b200 import GenParams, Model, NextDit
    cfg = tsynth.TINY
    path = str(tmp_path / "m.cmf")
    tensors, _ = build(cfg, path, tsynth.quant_plan(cfg, oc.Q8_ROW, oc.Q4TP), seed=1)
    rng = np.random.default_rng(8)
    h = w = 16
    lat = nd.gauss_latent(16 * h * w, 42).reshape(1, 16, h, w)
    cap = rng.standard_normal((1, 12, 256)).astype(np.float32)
    cap_u = rng.standard_normal((1, 5, 256)).astype(np.float32)
    orc = nd.NextDitOracle(tensors, cfg)
    want_steps = []
    want = nd.denoise(orc, lat[0], h, w, cap[0], cap_u[0], steps=30, gs=4.0, on_step=lambda i, x: want_steps.append(x.copy()))
    errs = []
    with Model(path) as m:
        dit = NextDit(m)
        dit.denoise_begin(lat, cap, cap_u, 30, 4.0, GenParams())
        for i in range(30):
            dit.denoise_step(i)
            errs.append(rel_l2(dit.denoise_end()[0], want_steps[i]))
        got = dit.denoise_end()
        dit.close()
    print("\nrel-L2 of the latent after Euler step 1..30: " + " ".join(f"{e:.1e}" for e in errs))
    assert max(errs) < TOL, errs
    assert rel_l2(got[0], want) < TOL


@pytest.mark.parametrize("prologue", ["0", "1"])
def test_euler_8_steps_lumina_width_4_layers(tmp_path, monkeypatch, prologue):
    """Eight CFG Euler steps at hidden 2304 (4 joint + 1 + 1 refiner layers, q4_tiled), 32x32 latent;
    with the separate qk-norm + RoPE pass and with Q rotated in the attention prologue (head_dim 96)."""
    from cmf_b200 import GenParams, Model, NextDit, denoise, synth
    monkeypatch.setenv("CMFC_ROPE_PROLOGUE", prologue)
    cfg = dict(synth.LUMINA2, num_layers=4, num_refiner_layers=1)
    path = os.path.join(str(tmp_path), "l4.cmf")
    synth.write_model(path, cfg, attn="q4t", ffn="q4t", seed=3)
    tensors, cj = load_for_oracle(path, cache=True)
    orc = nd.NextDitOracle(tensors, cj)
    rng = np.random.default_rng(5)
    h = w = 32
    lat = nd.gauss_latent(16 * h * w, 7).reshape(1, 16, h, w)
    cap = rng.standard_normal((1, 40, 2304)).astype(np.float32)
    cap_u = rng.standard_normal((1, 9, 2304)).astype(np.float32)
    want = nd.denoise(orc, lat[0], h, w, cap[0], cap_u[0], steps=8, gs=4.0)
    with Model(path) as m:
        dit = NextDit(m)
        got = denoise(dit, lat, cap, cap_u, GenParams(steps=8, guidance_scale=4.0))
        dit.close()
    err = rel_l2(got[0], want)
    print(f"\nLumina width, 4 layers, 8 Euler steps: latent rel-L2 {err:.2e}")
    assert err < TOL


@pytest.mark.parametrize("ratio,norm", [(0.5, True), (1.0, False), (0.34, False), (0.0, True)])
def test_cfg_truncation_and_normalization_switch(tmp_path, ratio, norm):
    """GenParams::cfg_trunc_ratio / cfg_normalization (crates/cortiq-engine/src/imagegen.rs:31-34,
    :164, :192): past the ratio only the cond branch runs, through the single-sequence forward; the
    per-row norm rescale is optional.  Six steps, batch of two, against the oracle per prompt."""
    from cmf_b200 import GenParams, Model, NextDit, denoise
    cfg = tsynth.TINY
    path = str(tmp_path / "m.cmf")
    tensors, _ = build(cfg, path, tsynth.quant_plan(cfg, oc.Q8_ROW, oc.Q8_ROW), seed=4)
    rng = np.random.default_rng(9)
    B, h, w = 2, 16, 16
    lat = np.stack([nd.gauss_latent(16 * h * w, s).reshape(16, h, w) for s in range(B)])
    cap = rng.standard_normal((B, 12, 256)).astype(np.float32)
    cap_u = rng.standard_normal((B, 5, 256)).astype(np.float32)
    orc = nd.NextDitOracle(tensors, cfg)
    p = GenParams(steps=6, guidance_scale=4.0, cfg_trunc_ratio=ratio, cfg_normalization=norm)
    with Model(path) as m:
        dit = NextDit(m)
        got = denoise(dit, lat, cap, cap_u, p)
        again = denoise(dit, lat, cap, cap_u, p)          # second run replays both captured step graphs
        default = denoise(dit, lat, cap, cap_u, GenParams(steps=6, guidance_scale=4.0))
        dit.close()
    assert np.array_equal(got, again)
    for b in range(B):
        want = nd.denoise(orc, lat[b], h, w, cap[b], cap_u[b], steps=6, gs=4.0, cfg_trunc_ratio=ratio,
                          cfg_normalization=norm)
        assert rel_l2(got[b], want) < TOL, (b, rel_l2(got[b], want))
    assert rel_l2(got, default) > 1e-3      # the switches really change the trajectory
