"""GPU parity of one block (facade dit_block_seg), of the whole forward and of the Euler loop
against the CPU oracle.  Tolerance: relative L2 <= 1e-2 per block output and per latent."""
import numpy as np
import pytest

from oracle import codecs as oc
from oracle import nextdit as nd
from tests import synth
from tests.modelfile import build, rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _inputs(cfg, seed, h, w, cap_n, cap_u_n):
    rng = np.random.default_rng(seed)
    latent = rng.standard_normal((cfg["in_channels"], h, w)).astype(np.float32)
    cap = rng.standard_normal((cap_n, cfg["cap_feat"])).astype(np.float32)
    cap_u = rng.standard_normal((cap_u_n, cfg["cap_feat"])).astype(np.float32)
    return latent, cap, cap_u


def _block_args(gpu, m, tensors, cfg, pfx, n, rope, mods):
    hs, nh, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_kv_heads"]
    t = tensors
    s_msa = g_msa = s_mlp = g_mlp = None
    if mods is not None:
        s_msa, g_msa, s_mlp, g_mlp = mods
    norm1 = t[pfx + (".norm1.norm.weight" if mods is not None else ".norm1.weight")]
    return gpu.DitBlockArgs(
        n=n, hidden=hs, inter=cfg["inter"], nh=nh, nkv=nkv, hd=hs // nh, eps=cfg["norm_eps"],
        rope_cos=rope[0].astype(np.float32), rope_sin=rope[1].astype(np.float32),
        norm1=norm1, norm2=t[pfx + ".norm2.weight"], ffn_norm1=t[pfx + ".ffn_norm1.weight"],
        ffn_norm2=t[pfx + ".ffn_norm2.weight"], norm_q=t[pfx + ".attn.norm_q.weight"],
        norm_k=t[pfx + ".attn.norm_k.weight"], s_msa=s_msa, gate_msa=g_msa, s_mlp=s_mlp, gate_mlp=g_mlp,
        wq=m.index(pfx + ".attn.to_q.weight"), wk=m.index(pfx + ".attn.to_k.weight"),
        wv=m.index(pfx + ".attn.to_v.weight"), wo=m.index(pfx + ".attn.to_out.0.weight"),
        w1=m.index(pfx + ".feed_forward.linear_1.weight"), w3=m.index(pfx + ".feed_forward.linear_3.weight"),
        w2=m.index(pfx + ".feed_forward.linear_2.weight"))


@pytest.mark.parametrize("attn,ffn", [(oc.Q8_ROW, oc.Q8_ROW), (oc.Q8_ROW, oc.Q4TP), (oc.Q4_TILED, oc.Q4_TILED)])
def test_block_seg_facade(tmp_path, attn, ffn):
    from cmf_b200 import Model, gpu
    cfg = synth.TINY
    path = str(tmp_path / "m.cmf")
    tensors, _ = build(cfg, path, synth.quant_plan(cfg, attn, ffn), seed=2, norm_jitter=0.1, std=0.05)
    orc = nd.NextDitOracle(tensors, cfg)
    rng = np.random.default_rng(3)
    segs = [150, 67, 131]           # ragged, the middle one starts off any 8-token boundary
    n = sum(segs)
    x0 = rng.standard_normal((n, cfg["hidden_size"])).astype(np.float32)
    ids = np.concatenate([np.stack([np.arange(s), np.arange(s) // 7, np.arange(s) % 7], 1) for s in segs])
    rope = nd.rope_table(ids, cfg["axes_dim_rope"])
    temb = rng.standard_normal(256).astype(np.float32)
    with Model(path) as m:
        # modulated block, then an unmodulated one chained on the device
        pfx = "dit.layers.0"
        mods = orc.modulation(pfx, temb)
        a = _block_args(gpu, m, tensors, cfg, pfx, n, rope, mods)
        x = x0.copy()
        gpu.dit_block_seg(m, a, segs, x)
        want = orc.block_forward_seg(pfx, x0, rope, temb, segs)
        assert rel_l2(x, want) < TOL, rel_l2(x, want)
        # chain: block 0 (resident_out) -> context refiner block (resident_in), read back once
        a.resident_out = True
        x = x0.copy()
        gpu.dit_block_seg(m, a, segs, x)
        assert np.array_equal(x, x0)            # nothing copied back
        assert gpu.dit_chain_supported() and not gpu.fused_dit_block_available()
        b = _block_args(gpu, m, tensors, cfg, "dit.context_refiner.0", n, rope, None)
        b.resident_in = True
        gpu.dit_block_seg(m, b, segs, x)
        want2 = orc.block_forward_seg("dit.context_refiner.0", want, rope, None, segs)
        assert rel_l2(x, want2) < TOL
        y = np.empty_like(x)
        gpu.dit_state_fetch(y)
        assert np.array_equal(x, y)


def test_block_seg_rejects_bad_segments(tmp_path):
    from cmf_b200 import CmfCudaError, Model, gpu
    cfg = synth.TINY
    path = str(tmp_path / "m.cmf")
    tensors, _ = build(cfg, path, synth.quant_plan(cfg, oc.Q8_ROW, oc.Q8_ROW))
    n = 64
    rope = nd.rope_table(np.zeros((n, 3), np.int64), cfg["axes_dim_rope"])
    x = np.zeros((n, 256), np.float32)
    with Model(path) as m:
        a = _block_args(gpu, m, tensors, cfg, "dit.context_refiner.0", n, rope, None)
        with pytest.raises(CmfCudaError) as e:
            gpu.dit_block_seg(m, a, [30, 30], x)
        assert e.value.code == -1
        a.resident_in = True
        with pytest.raises(CmfCudaError):
            gpu.dit_block_seg(m, a, [n], None)


@pytest.mark.parametrize("plan_name", ["q8", "q4tp_ffn_q8_attn", "q4t"])
def test_tiny_forward_pair_per_block_and_latent(tmp_path, plan_name):
    """The tiny CPU-runnable denoiser (2 layers, hidden 256, q8 per-row weights, 32x32 latent, 32 caption
    tokens, batch 1, t = 0.5, seed 0) plus the mixed-codec variants."""
    from cmf_b200 import Model, NextDit
    cfg = synth.TINY
    attn, ffn = {"q8": (oc.Q8_ROW, oc.Q8_ROW), "q4tp_ffn_q8_attn": (oc.Q8_ROW, oc.Q4TP),
                 "q4t": (oc.Q4_TILED, oc.Q4_TILED)}[plan_name]
    path = str(tmp_path / "m.cmf")
    tensors, _ = build(cfg, path, synth.quant_plan(cfg, attn, ffn), seed=0)
    latent, cap, cap_u = _inputs(cfg, 0, 32, 32, 32, 32)
    orc = nd.NextDitOracle(tensors, cfg)
    with Model(path) as m:
        # every quantized tensor dequantizes bit-exactly on the device
        for name, q in tensors.items():
            if isinstance(q, nd.QWeight):
                got = m.dequant(m.index(name))
                assert np.array_equal(got.view(np.uint32), q.dense().view(np.uint32)), name
        dit = NextDit(m)
        cc, cu = dit.refine_caption(cap), dit.refine_caption(cap_u)
        wc, wu = orc.refine_caption(cap), orc.refine_caption(cap_u)
        # refine_caption chains three stages (embed + two refiner blocks); each block is held to
        # TOL on its own in test_block_seg_facade, the chain to 2 * TOL
        assert rel_l2(cc, wc) < 2 * TOL and rel_l2(cu, wu) < 2 * TOL, (rel_l2(cc, wc), rel_l2(cu, wu))
        pc, pu, taps = dit.forward_cfg_pair(latent, 32, 32, wc, 32, wu, 32, 0.5, taps=True)
        orc.block_taps = []
        oc_, ou_ = orc.forward_cfg_pair(latent, 32, 32, wc, wu, 0.5)
        joint = [x for p, x in orc.block_taps if p.startswith("dit.layers")]
        for l, want in enumerate(joint):
            assert rel_l2(taps[l], want) < TOL, (l, rel_l2(taps[l], want))
        assert rel_l2(pc, oc_) < TOL and rel_l2(pu, ou_) < TOL, (rel_l2(pc, oc_), rel_l2(pu, ou_))
        single = dit.forward_with_cap(latent, 32, 32, wc, 32, 0.5)
        assert rel_l2(single, orc.forward_with_cap(latent, 32, 32, wc, 0.5)) < TOL
        dit.close()


@pytest.mark.parametrize("prologue", ["0", "1"])
def test_ragged_forward(tmp_path, monkeypatch, prologue):
    """Ragged latent and caption lengths; once with the separate qk-norm + RoPE pass for Q and K, once
    with Q normalised and rotated in the attention kernel's prologue (CMFC_ROPE_PROLOGUE=1)."""
    from cmf_b200 import Model, NextDit
    monkeypatch.setenv("CMFC_ROPE_PROLOGUE", prologue)
    cfg = synth.TINY
    path = str(tmp_path / "m.cmf")
    tensors, _ = build(cfg, path, synth.quant_plan(cfg, oc.Q8_ROW, oc.Q4TP), seed=5, norm_jitter=0.1, std=0.05)
    latent, cap, cap_u = _inputs(cfg, 6, 12, 20, 7, 3)
    orc = nd.NextDitOracle(tensors, cfg)
    wc, wu = orc.refine_caption(cap), orc.refine_caption(cap_u)
    with Model(path) as m:
        dit = NextDit(m)
        pc, pu = dit.forward_cfg_pair(latent, 12, 20, wc, 7, wu, 3, 0.7)
        oc_, ou_ = orc.forward_cfg_pair(latent, 12, 20, wc, wu, 0.7)
        assert rel_l2(pc, oc_) < TOL and rel_l2(pu, ou_) < TOL
        dit.close()


def test_denoise_loop_batch(tmp_path):
    """Euler loop with CFG over a batch of two prompts: latents after 4 steps against the oracle
    run per prompt, and the batch result equal to the per-prompt results."""
    from cmf_b200 import GenParams, Model, NextDit, denoise
    cfg = synth.TINY
    path = str(tmp_path / "m.cmf")
    tensors, _ = build(cfg, path, synth.quant_plan(cfg, oc.Q8_ROW, oc.Q4TP), seed=1)
    rng = np.random.default_rng(8)
    B, h, w, cap_n, cap_u_n = 2, 16, 16, 12, 5
    lat = np.stack([nd.gauss_latent(16 * h * w, s).reshape(16, h, w) for s in range(B)])
    cap = rng.standard_normal((B, cap_n, 256)).astype(np.float32)
    cap_u = rng.standard_normal((B, cap_u_n, 256)).astype(np.float32)
    orc = nd.NextDitOracle(tensors, cfg)
    p = GenParams(steps=4, guidance_scale=4.0)
    with Model(path) as m:
        dit = NextDit(m)
        got = denoise(dit, lat, cap, cap_u, p)
        one = denoise(dit, lat[1:2], cap[1:2], cap_u[1:2], p)
        nocfg = denoise(dit, lat[:1], cap[:1], None, p)
        dit.close()
    for b in range(B):
        want = nd.denoise(orc, lat[b], h, w, cap[b], cap_u[b], steps=4, gs=4.0)
        assert rel_l2(got[b], want) < TOL, (b, rel_l2(got[b], want))
    assert rel_l2(one[0], got[1]) < 1e-5          # batching does not change a prompt's result
    want = nd.denoise(orc, lat[0], h, w, cap[0], None, steps=4)
    assert rel_l2(nocfg[0], want) < TOL


def test_lumina_geometry_two_layers(tmp_path):
    """Lumina-2 geometry (hidden 2304, 24/8 heads of 96, FFN 9216) with 2 joint layers, q4tp FFN +
    q8 attention, a 32x32 latent and 40 caption tokens: per-block and per-latent parity."""
    from cmf_b200 import Model, NextDit
    cfg = synth.LUMINA_GEOM
    path = str(tmp_path / "m.cmf")
    tensors, _ = build(cfg, path, synth.quant_plan(cfg, oc.Q8_ROW, oc.Q4TP), seed=0)
    latent, cap, cap_u = _inputs(cfg, 0, 32, 32, 40, 9)
    orc = nd.NextDitOracle(tensors, cfg)
    wc, wu = orc.refine_caption(cap), orc.refine_caption(cap_u)
    with Model(path) as m:
        dit = NextDit(m)
        assert rel_l2(dit.refine_caption(cap), wc) < TOL
        pc, pu, taps = dit.forward_cfg_pair(latent, 32, 32, wc, 40, wu, 9, 0.5, taps=True)
        dit.close()
    orc.block_taps = []
    oc_, ou_ = orc.forward_cfg_pair(latent, 32, 32, wc, wu, 0.5)
    joint = [x for p, x in orc.block_taps if p.startswith("dit.layers")]
    for l, want in enumerate(joint):
        assert rel_l2(taps[l], want) < TOL, (l, rel_l2(taps[l], want))
    assert rel_l2(pc, oc_) < TOL and rel_l2(pu, ou_) < TOL


def test_captured_step_after_many_segmentations(tmp_path):
    """The device copies of the segment tables are cached per segmentation, least recently used first
    out.  Forty different attention shapes fill and turn over that cache; the denoise loop that
    follows (a warm-up step, then captured steps that may not upload anything) must still find every
    table its warm-up step used."""
    from cmf_b200 import GenParams, Model, NextDit, denoise, gpu
    rng = np.random.default_rng(2)
    for n in range(130, 170):
        q = rng.standard_normal((2, n, 64)).astype(np.float32)
        out = np.empty((n, 128), np.float32)
        gpu.dit_attention(q, q, q, 2, 2, n, 64, 0.125, out)
    cfg = synth.TINY
    path = str(tmp_path / "m.cmf")
    tensors, _ = build(cfg, path, synth.quant_plan(cfg, oc.Q8_ROW, oc.Q8_ROW), seed=1)
    lat = nd.gauss_latent(16 * 16 * 16, 0).reshape(1, 16, 16, 16)
    cap = rng.standard_normal((1, 12, 256)).astype(np.float32)
    cap_u = rng.standard_normal((1, 5, 256)).astype(np.float32)
    with Model(path) as m:
        dit = NextDit(m)
        got = denoise(dit, lat, cap, cap_u, GenParams(steps=3, guidance_scale=4.0))
        dit.close()
    want = nd.denoise(nd.NextDitOracle(tensors, cfg), lat[0], 16, 16, cap[0], cap_u[0], steps=3, gs=4.0)
    assert rel_l2(got[0], want) < TOL


def test_forward_with_tracking_attention_matches_bounded(tmp_path, monkeypatch):
    """A block's attention normally takes the bounded form (the head norm bounds every score);
    CMFC_ATTN_FIXED_REF=0 makes it track the running row maximum instead, the form used when the
    norm gains put the bound out of range.  Both against the oracle and against each other, with
    jittered norm weights so the gains are not all one."""
    from cmf_b200 import Model, NextDit
    cfg = synth.TINY
    path = str(tmp_path / "m.cmf")
    tensors, _ = build(cfg, path, synth.quant_plan(cfg, oc.Q8_ROW, oc.Q8_ROW), seed=2, norm_jitter=0.2)
    latent, cap, cap_u = _inputs(cfg, 3, 32, 32, 40, 9)
    orc = nd.NextDitOracle(tensors, cfg)
    wc, wu = orc.refine_caption(cap), orc.refine_caption(cap_u)
    want_c, want_u = orc.forward_cfg_pair(latent, 32, 32, wc, wu, 0.3)
    got = {}
    with Model(path) as m:
        dit = NextDit(m)
        for env in ("1", "0"):
            monkeypatch.setenv("CMFC_ATTN_FIXED_REF", env)
            got[env] = dit.forward_cfg_pair(latent, 32, 32, wc, 40, wu, 9, 0.3)
        dit.close()
    for env in ("1", "0"):
        assert rel_l2(got[env][0], want_c) < TOL and rel_l2(got[env][1], want_u) < TOL, env
    assert 0 < rel_l2(got["0"][0], got["1"][0]) < 5e-3


@pytest.mark.parametrize("case", ["one_large_gain", "all_gains_large"])
def test_forward_with_norm_gains_beyond_the_weight_bound(tmp_path, monkeypatch, case):
    """Head-norm gains so large that the worst case they allow (a whole row's weight on the largest gain)
    exceeds the bounded attention form's range.  The qk-norm + RoPE pass then measures the finished
    heads and attention decides on the device: with ONE gain of 5 in the query norm and one in the key norm
    (worst-case bound 294 log2 units) real rows measure about 50 and the bounded form runs; with ALL gains
    3.5 they measure 144 and the tracking form runs.  Either way the result
    must equal the forced tracking form; against the oracle the tolerance is wider than elsewhere
    because logits this large amplify the bf16 rounding of Q and K."""
    from cmf_b200 import Model, NextDit
    cfg = synth.TINY

    def mutate(t):
        for name in t:
            if name.endswith("attn.norm_q.weight") or name.endswith("attn.norm_k.weight"):
                if case == "one_large_gain":
                    t[name][3 if name.endswith("norm_q.weight") else 5] = 5.0
                else:
                    t[name] *= 3.5

    path = str(tmp_path / "m.cmf")
    tensors, _ = build(cfg, path, synth.quant_plan(cfg, oc.Q8_ROW, oc.Q8_ROW), seed=5, mutate=mutate)
    latent, cap, cap_u = _inputs(cfg, 4, 32, 32, 40, 9)
    orc = nd.NextDitOracle(tensors, cfg)
    wc, wu = orc.refine_caption(cap), orc.refine_caption(cap_u)
    want_c, _ = orc.forward_cfg_pair(latent, 32, 32, wc, wu, 0.4)
    got = {}
    with Model(path) as m:
        dit = NextDit(m)
        for env in ("1", "0"):
            monkeypatch.setenv("CMFC_ATTN_FIXED_REF", env)
            got[env] = dit.forward_cfg_pair(latent, 32, 32, wc, 40, wu, 9, 0.4)[0]
        dit.close()
    assert np.isfinite(got["1"]).all()
    assert rel_l2(got["1"], got["0"]) < 5e-3, rel_l2(got["1"], got["0"])
    assert rel_l2(got["1"], want_c) < 5e-2, rel_l2(got["1"], want_c)
    # the same through the captured step (the measurement's memset and both launches are graph nodes)
    from cmf_b200 import GenParams, denoise
    lat = nd.gauss_latent(16 * 16 * 16, 1).reshape(1, 16, 16, 16)
    loops = {}
    with Model(path) as m:
        dit = NextDit(m)
        for env in ("1", "0"):
            monkeypatch.setenv("CMFC_ATTN_FIXED_REF", env)
            loops[env] = denoise(dit, lat, cap[None], cap_u[None], GenParams(steps=4, guidance_scale=4.0))
        dit.close()
    # four guided steps (guidance scale 4) on logits this large amplify the different bf16 rounding of
    # the queries (pre-scaled here, unscaled in the forced form): a wider tolerance than for one forward
    assert np.isfinite(loops["1"]).all()
    assert rel_l2(loops["1"], loops["0"]) < 3e-2, rel_l2(loops["1"], loops["0"])
