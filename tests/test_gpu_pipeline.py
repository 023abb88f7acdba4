"""The whole image pipeline of a packaged container (crates/cortiq-engine/src/imagegen.rs:225-297):
prompt ids -> Gemma-2 caption features -> CFG Euler loop -> VAE decode -> RGB, against the same
chain of CPU oracles on a tiny te + dit + vae container."""
import numpy as np
import pytest

from oracle import codecs as oc
from oracle import gemma as og
from oracle import nextdit as nd
from oracle import vae as ovae
from oracle.nextdit import QWeight
from tests import gemma_model, synth
from tests.modelfile import rel_l2

pytestmark = pytest.mark.gpu


def build_pipeline(path, seed=0):
    """te.* (q8 embedding, q4_tiled projections), dit.* (q8 modulation + attention, q4tp FFN), vae.*"""
    from cmf_b200 import synth as psynth
    from cmf_b200.container import CmfWriter
    w = CmfWriter(arch={"arch_name": "lumina2-image", "hidden_size": 256, "num_layers": 3, "vocab_size": 512})
    te_cfg, dit_cfg, vae_cfg = gemma_model.TINY, synth.TINY, psynth.TINY_VAE
    te, dit = {}, {}
    for name, arr in gemma_model.make_tensors(te_cfg, seed).items():
        dt = 3 if name == "te.embed_tokens.weight" else (oc.Q4_TILED if name.endswith("_proj.weight") else None)
        if dt is None:
            w.add_f32(name, arr)
            te[name] = arr
        else:
            te[name] = QWeight.quantize(dt, arr)
            w.add(name, dt, arr.shape, te[name].payload)
    w.add_json("te.config_json", te_cfg)
    plan = synth.quant_plan(dit_cfg, oc.Q8_ROW, oc.Q4TP)
    for name, arr in synth.make_tensors(dit_cfg, seed + 1, 0.05).items():
        dt = plan.get(name)
        if dt is None or arr.ndim != 2:
            w.add_f32(name, arr)
            dit[name] = arr
        else:
            dit[name] = QWeight.quantize(dt, arr)
            w.add(name, dt, arr.shape, dit[name].payload)
    w.add_json("dit.config_json", {k: dit_cfg[k] for k in (
        "hidden_size", "num_layers", "num_refiner_layers", "num_attention_heads", "num_kv_heads", "in_channels",
        "patch_size", "axes_dim_rope", "norm_eps")})
    psynth.add_vae(w, vae_cfg, seed + 2)
    w.write(path)
    return (te, te_cfg), (dit, dit_cfg), (psynth.vae_tensors(vae_cfg, seed + 2), vae_cfg)


@pytest.mark.parametrize("guidance", [4.0, 1.0])
def test_generate_matches_the_chain_of_oracles(tmp_path, guidance):
    from cmf_b200 import GenParams, Model, Pipeline
    path = str(tmp_path / "pipe.cmf")
    (te, te_cfg), (dit, dit_cfg), (vae, vae_cfg) = build_pipeline(path)
    ids = np.array([2, 17, 300, 45, 9, 128, 77, 5, 410, 33, 12], np.uint32)
    uncond = np.array([2], np.uint32)
    # the tiny VAE has one upsampler: latent 16 x 16 -> 32 x 32 pixels; GenParams counts in FLUX's 8x
    p = GenParams(steps=4, guidance_scale=guidance, seed=7, height=128, width=128)
    stages = {}
    with Model(path) as m:
        pipe = Pipeline(m)
        rgb = pipe.generate(ids, uncond, p, stages=stages)
        again = pipe.generate(ids, uncond, p)
        pipe.close()
    lh = lw = 16
    enc = og.GemmaOracle(te, te_cfg)
    cap = enc.encode(ids, keep_layer_inputs=True)[1][-2]
    cap_u = enc.encode(uncond, keep_layer_inputs=True)[1][-2] if guidance > 1.0 else None
    lat0 = nd.gauss_latent(16 * lh * lw, 7).reshape(16, lh, lw)
    lat = nd.denoise(nd.NextDitOracle(dit, dit_cfg), lat0, lh, lw, cap, cap_u, steps=4, gs=guidance)
    want = np.clip(ovae.decode(vae, vae_cfg, lat) / 2 + 0.5, 0, 1)
    assert rgb.shape == want.shape == (3, 32, 32)
    assert rgb.min() >= 0.0 and rgb.max() <= 1.0 and np.array_equal(rgb, again)
    assert set(stages) == {"text encode", "denoise", "vae decode"}
    assert rel_l2(rgb, want) < 2e-2
    assert np.abs(rgb - want).max() < 5e-2


def test_generate_rejects_bad_sizes(tmp_path):
    from cmf_b200 import GenParams, Model, Pipeline
    path = str(tmp_path / "pipe.cmf")
    build_pipeline(path)
    with Model(path) as m:
        pipe = Pipeline(m)
        with pytest.raises(ValueError):
            pipe.generate([2, 3], [2], GenParams(steps=1, height=120, width=128))
        pipe.close()
