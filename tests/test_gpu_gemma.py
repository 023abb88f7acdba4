"""Gemma-2 prompt encoder on the device against the CPU oracle (oracle/gemma.py): tiny models in
the three codecs, Gemma-2-2B head geometry, ragged prompt lengths, error behaviour."""
import os

import numpy as np
import pytest

from oracle import codecs as oc
from oracle import gemma as og
from tests import gemma_model
from tests.modelfile import rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-2   # relative L2, the tolerance of the denoiser path (bf16 GEMM operands, f32 accumulation)


@pytest.mark.parametrize("level", [oc.Q8_ROW, oc.Q4_TILED, oc.Q4TP])
@pytest.mark.parametrize("n", [1, 11, 40, 130])
def test_tiny_encoder_matches_oracle(tmp_path, level, n):
    from cmf_b200 import GemmaEncoder, Model
    cfg = gemma_model.TINY
    path = str(tmp_path / "te.cmf")
    t = gemma_model.build(cfg, path, level, seed=2)
    ids = np.random.default_rng(n).integers(0, cfg["vocab_size"], n).astype(np.uint32)
    want, want_streams = og.GemmaOracle(t, cfg).encode(ids, keep_layer_inputs=True)
    with Model(path) as m:
        enc = GemmaEncoder(m)
        assert (enc.hidden, enc.num_layers, enc.nh, enc.nkv, enc.head_dim) == (256, 3, 4, 2, 64)
        out, streams = enc.encode(ids, keep_layer_inputs=True)
        only_final, none = enc.encode(ids)
        cap = enc.caption_features(ids)
        enc.close()
    assert len(streams) == cfg["num_hidden_layers"] + 1 and none == []
    assert np.array_equal(streams[0], want_streams[0])            # embedding rows * sqrt(hidden): exact
    for got, ref in zip(streams, want_streams):
        assert rel_l2(got, ref) < TOL
    assert rel_l2(out, want) < TOL
    assert np.array_equal(out, only_final) and np.array_equal(cap, streams[-2])


def test_soft_cap_bends_the_logits(tmp_path):
    """attn_logit_softcapping = 2 against logits of deviation ~2.5: the tanh is far from linear."""
    from cmf_b200 import GemmaEncoder, Model
    cfg = gemma_model.TINY_CAP
    path = str(tmp_path / "te.cmf")
    t = gemma_model.build(cfg, path, oc.Q8_ROW, seed=7)
    ids = np.random.default_rng(3).integers(0, cfg["vocab_size"], 50).astype(np.uint32)
    want, _ = og.GemmaOracle(t, cfg).encode(ids)
    uncapped, _ = og.GemmaOracle(t, dict(cfg, attn_logit_softcapping=0.0)).encode(ids)
    with Model(path) as m:
        enc = GemmaEncoder(m)
        out, _ = enc.encode(ids)
        enc.close()
    assert rel_l2(out, want) < TOL
    assert rel_l2(uncapped, want) > 3 * TOL      # the cap matters for this input


def test_gemma2_head_geometry_matches_oracle(tmp_path):
    """hidden 2304, head_dim 256 (nh * hd != hidden), GQA 8/4, GeGLU 9216, q4_tiled, 77 tokens."""
    from cmf_b200 import GemmaEncoder, Model
    cfg = gemma_model.GEMMA_GEOM
    path = str(tmp_path / "te.cmf")
    t = gemma_model.build(cfg, path, oc.Q4_TILED, seed=3)
    ids = np.random.default_rng(0).integers(0, cfg["vocab_size"], 77).astype(np.uint32)
    want, want_streams = og.GemmaOracle(t, cfg).encode(ids, keep_layer_inputs=True)
    with Model(path) as m:
        enc = GemmaEncoder(m)
        out, streams = enc.encode(ids, keep_layer_inputs=True)
        enc.close()
    for got, ref in zip(streams, want_streams):
        assert rel_l2(got, ref) < TOL
    assert rel_l2(out, want) < TOL


@pytest.mark.parametrize("level,tol", [("q8", 1e-4), ("q4t", TOL)])
def test_full_depth_gemma2_2b(tmp_path, level, tol):
    """All 26 layers at Gemma-2-2B sizes (2.6 B parameters, device-quantized synthetic weights; the
    vocabulary is cut to 4096 rows, which the forward never notices), 77 tokens.  q8 weights are
    exact in the GEMM operand, so only f32 summation order separates device and oracle."""
    from cmf_b200 import GemmaEncoder, Model, synth
    from tests.modelfile import load_for_oracle
    cfg = dict(synth.GEMMA2_2B, vocab_size=4096)
    path = str(tmp_path / "te.cmf")
    synth.write_gemma_model(path, cfg, level, seed=1)
    t, _ = load_for_oracle(path, cache=False)
    ids = np.random.default_rng(0).integers(0, cfg["vocab_size"], 77).astype(np.uint32)
    want, want_streams = og.GemmaOracle(t, cfg).encode(ids, keep_layer_inputs=True)
    with Model(path) as m:
        enc = GemmaEncoder(m)
        assert (enc.hidden, enc.num_layers, enc.head_dim, enc.inter) == (2304, 26, 256, 9216)
        out, streams = enc.encode(ids, keep_layer_inputs=True)
        enc.close()
    for got, ref in zip(streams, want_streams):
        assert rel_l2(got, ref) < tol
    assert rel_l2(out, want) < tol


def test_prefix_independence(tmp_path):
    """Causal: the states of a prefix do not depend on what follows it."""
    from cmf_b200 import GemmaEncoder, Model
    cfg = gemma_model.TINY
    path = str(tmp_path / "te.cmf")
    gemma_model.build(cfg, path, oc.Q8_ROW, seed=4)
    a = np.arange(3, 36, dtype=np.uint32)
    b = a.copy()
    b[20:] = 7
    with Model(path) as m:
        enc = GemmaEncoder(m)
        ha, _ = enc.encode(a)
        hb, _ = enc.encode(b)
        enc.close()
    assert rel_l2(ha[:20], hb[:20]) < 1e-6 and rel_l2(ha[20:], hb[20:]) > 1e-3


def test_errors(tmp_path):
    from cmf_b200 import CmfCudaError, CmfWriter, GemmaEncoder, Model
    cfg = gemma_model.TINY
    path = str(tmp_path / "te.cmf")
    gemma_model.build(cfg, path, oc.Q8_ROW, seed=4)
    with Model(path) as m:
        enc = GemmaEncoder(m)
        with pytest.raises(CmfCudaError):
            enc.encode(np.array([1, 2, cfg["vocab_size"]], np.uint32))    # id outside the vocabulary
        with pytest.raises(CmfCudaError):
            enc.encode(np.zeros(0, np.uint32))                            # empty prompt
        with pytest.raises(CmfCudaError):
            enc.encode(np.zeros(cfg["sliding_window"], np.uint32))        # textenc.rs:224-229
        ok, _ = enc.encode(np.array([1, 2, 3], np.uint32))                # the handle survives the errors
        assert np.isfinite(ok).all()
        enc.close()
    empty = str(tmp_path / "none.cmf")
    w = CmfWriter(arch={"arch_name": "none"})
    w.add_f32("x", np.zeros((2, 2), np.float32))
    w.write(empty)
    with Model(empty) as m:
        with pytest.raises(CmfCudaError):
            GemmaEncoder(m)
