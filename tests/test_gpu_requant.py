"""q4_tiled -> q4tp recoding on the device (crates/cortiq-cli/src/requant.rs, Mode::FullQ4tp):
byte-identical to the oracle's encoder over the oracle's dequant, everything else verbatim, and
the recoded model still runs through the denoiser within tolerance of the original."""
import numpy as np
import pytest

from oracle import codecs as oc
from tests import synth
from tests.modelfile import build as build_model, load_for_oracle, rel_l2

pytestmark = pytest.mark.gpu


def test_requant_q4tp_matches_oracle_and_runs(tmp_path):
    from cmf_b200 import Model, NextDit
    from cmf_b200.requant import read_header, requant_q4tp
    cfg = synth.TINY
    src, dst = str(tmp_path / "a.cmf"), str(tmp_path / "b.cmf")
    build_model(cfg, src, synth.quant_plan(cfg, oc.Q8_ROW, oc.Q4_TILED), seed=1)
    n, before, after = requant_q4tp(src, dst)
    assert n > 0 and after < before
    assert read_header(dst)["arch"] == read_header(src)["arch"]
    a, _ = load_for_oracle(src)
    b, _ = load_for_oracle(dst)
    assert set(a) == set(b)
    recoded = 0
    for name, ta in a.items():
        tb = b[name]
        if hasattr(ta, "dtype") and not isinstance(ta, np.ndarray) and ta.dtype == oc.Q4_TILED:
            assert tb.dtype == oc.Q4TP
            want = oc.encode(oc.Q4TP, oc.dequant(oc.Q4_TILED, ta.payload, ta.rows, ta.cols))
            assert np.array_equal(np.asarray(tb.payload), np.asarray(want)), name
            recoded += 1
        elif isinstance(ta, np.ndarray):
            assert np.array_equal(ta, tb)
        else:
            assert ta.dtype == tb.dtype and np.array_equal(ta.payload, tb.payload)
    assert recoded == n
    rng = np.random.default_rng(0)
    lat = rng.standard_normal((16, 16, 16)).astype(np.float32)
    cap = rng.standard_normal((12, 256)).astype(np.float32)
    outs = []
    for path in (src, dst):
        with Model(path) as m:
            dit = NextDit(m)
            outs.append(dit.forward(lat, 16, 16, cap, 12, 0.4))
            dit.close()
    assert rel_l2(outs[1], outs[0]) < 0.1 and not np.array_equal(outs[0], outs[1])   # the ladder moves scales by a few percent
