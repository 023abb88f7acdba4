"""The Gemma-2 encoder oracle (oracle/gemma.py) against the fixtures generated from the reference's
numpy functions (tests/golden/make_gemma_ref.py).  No GPU."""
import os

import numpy as np
import pytest

from oracle import gemma as og
from tests import gemma_model
from tests.modelfile import rel_l2

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("case", ["tiny", "tiny_long"])
def test_oracle_matches_reference_encoder(case):
    g = np.load(os.path.join(GOLD, f"gemma_ref_{case}.npz"))
    t = gemma_model.make_tensors(gemma_model.TINY, int(g["weight_seed"]))
    out, streams = og.GemmaOracle(t, gemma_model.TINY).encode(g["ids"], keep_layer_inputs=True)
    assert len(streams) == gemma_model.TINY["num_hidden_layers"] + 1
    # the reference test's own bar is 1e-3 relative (crates/cortiq-engine/tests/textenc_parity.rs:36-48)
    assert rel_l2(streams[-2], g["penultimate"]) < 1e-5
    assert rel_l2(streams[-1], g["last_stream"]) < 1e-5
    rel = np.abs(out - g["out"]) / np.maximum(np.abs(g["out"]), 1.0)
    assert rel.max() < 1e-4


def test_norm_and_gelu_forms():
    # textenc.rs:59-73
    x = np.array([[3.0, 4.0]], np.float32)
    y = og.rms_norm_gemma(x, np.array([0.0, 1.0], np.float32), 0.0)
    assert np.allclose(y, [[3.0 / np.sqrt(12.5), 2 * 4.0 / np.sqrt(12.5)]], atol=1e-6)
    assert abs(float(og.gelu_tanh(np.float32(1.0))) - 0.841192) < 1e-5
    assert float(og.gelu_tanh(np.float32(0.0))) == 0.0


def test_rope_half_rotates_pairs_i_and_i_plus_half():
    # textenc.rs:271-286: position 0 is the identity; norms of the (i, i + hd/2) pairs are kept
    x = np.random.default_rng(0).standard_normal((5, 2, 8)).astype(np.float32)
    y = og.rope_half(x, 10000.0)
    assert np.array_equal(y[0], x[0])
    assert np.allclose(x[..., :4] ** 2 + x[..., 4:] ** 2, y[..., :4] ** 2 + y[..., 4:] ** 2, atol=1e-5)


def test_causality():
    t = gemma_model.make_tensors(gemma_model.TINY, 1)
    orc = og.GemmaOracle(t, gemma_model.TINY)
    a, _ = orc.encode([2, 5, 9, 11, 13])
    b, _ = orc.encode([2, 5, 9, 400, 401])
    assert np.array_equal(a[:3], b[:3]) and not np.array_equal(a[3:], b[3:])
