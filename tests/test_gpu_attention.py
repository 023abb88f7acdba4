"""GPU parity of the flash attention kernel through the facade's dit_attention."""
import numpy as np
import pytest

from oracle import codecs as oc
from oracle.nextdit import attention_seq
from tests.modelfile import rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nh,nkv,hd,n", [(4, 4, 64, 288), (6, 2, 96, 128), (6, 2, 96, 67), (24, 8, 96, 1100),
                                          (2, 1, 128, 513), (2, 2, 32, 300)])
def test_attention_matches_oracle(nh, nkv, hd, n):
    from cmf_b200 import gpu
    rng = np.random.default_rng(nh * 1000 + n)
    q = oc.bf16_round(rng.standard_normal((n, nh, hd)).astype(np.float32))
    k = oc.bf16_round(rng.standard_normal((n, nkv, hd)).astype(np.float32))
    v = oc.bf16_round(rng.standard_normal((n, nkv, hd)).astype(np.float32))
    out = np.empty((n, nh * hd), np.float32)
    scale = 1.0 / np.sqrt(hd)
    gpu.dit_attention(q.transpose(1, 0, 2), k.transpose(1, 0, 2), v.transpose(1, 0, 2), nh, nkv, n, hd, scale, out)
    want = attention_seq(q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), nh, nkv, hd)
    assert np.isfinite(out).all()
    assert rel_l2(out, want) < 6e-3, rel_l2(out, want)


def test_attention_sharp_and_flat_rows():
    """Rows with one dominant key (max tracking) and rows with identical keys (uniform P)."""
    from cmf_b200 import gpu
    nh, nkv, hd, n = 2, 2, 64, 400
    rng = np.random.default_rng(0)
    q = rng.standard_normal((n, nh, hd)).astype(np.float32)
    k = rng.standard_normal((n, nkv, hd)).astype(np.float32)
    k[300] = q[5] * 4.0          # key 300 dominates query 5, found only in the third key tile
    k[:, 1] = k[0:1, 1]          # head 1: all keys equal -> uniform attention
    q, k = oc.bf16_round(q), oc.bf16_round(k)
    v = oc.bf16_round(rng.standard_normal((n, nkv, hd)).astype(np.float32))
    out = np.empty((n, nh * hd), np.float32)
    gpu.dit_attention(q.transpose(1, 0, 2), k.transpose(1, 0, 2), v.transpose(1, 0, 2), nh, nkv, n, hd, 0.125, out)
    want = attention_seq(q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), nh, nkv, hd)
    assert rel_l2(out, want) < 6e-3
    assert rel_l2(out.reshape(n, nh, hd)[:, 1], np.broadcast_to(v[:, 1].mean(0), (n, hd))) < 6e-3


def test_attention_rising_scores_wide_range():
    """Scores that rise by ~30 log2 units per key tile: the running maximum moves on every tile (O is
    rescaled each time) and the early keys end up more than 2^-126 below the final maximum, which is
    where the exponentials computed without the special-function unit clamp their argument."""
    from cmf_b200 import gpu
    nh, nkv, hd, n = 6, 2, 96, 700
    rng = np.random.default_rng(11)
    q = rng.standard_normal((n, nh, hd)).astype(np.float32)
    k = rng.standard_normal((n, nkv, hd)).astype(np.float32)
    q[:, :, 0] = 4.0
    k[:, :, 0] = 300.0 * np.arange(n, dtype=np.float32)[:, None] / n
    q, k = oc.bf16_round(q), oc.bf16_round(k)
    v = oc.bf16_round(rng.standard_normal((n, nkv, hd)).astype(np.float32))
    out = np.empty((n, nh * hd), np.float32)
    scale = 1.0 / np.sqrt(hd)
    gpu.dit_attention(q.transpose(1, 0, 2), k.transpose(1, 0, 2), v.transpose(1, 0, 2), nh, nkv, n, hd, scale, out)
    want = attention_seq(q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), nh, nkv, hd)
    assert np.isfinite(out).all()
    assert rel_l2(out, want) < 6e-3, rel_l2(out, want)


def _score_bound_log2(q, k, scale):
    """max |q_i| * max |k_j| * scale * log2(e): what the entry measures on the device to decide between the
    bounded form (at most 96: P = exp2 of the pre-scaled score, no reference at all) and the form that
    follows the running row maximum."""
    qn = np.sqrt((q.astype(np.float64) ** 2).sum(-1)).max()
    kn = np.sqrt((k.astype(np.float64) ** 2).sum(-1)).max()
    return qn * kn * scale * 1.4426950408889634


def test_attention_bounded_form_equals_running_maximum(monkeypatch):
    """The same bounded input through both softmax forms: the bounded one (default when the bound allows)
    and the running row maximum (CMFC_ATTN_FIXED_REF=0)."""
    from cmf_b200 import gpu
    nh, nkv, hd, n = 6, 2, 96, 900
    rng = np.random.default_rng(21)
    q = oc.bf16_round(rng.standard_normal((n, nh, hd)).astype(np.float32))
    k = oc.bf16_round(rng.standard_normal((n, nkv, hd)).astype(np.float32))
    v = oc.bf16_round(rng.standard_normal((n, nkv, hd)).astype(np.float32))
    scale = 1.0 / np.sqrt(hd)
    assert _score_bound_log2(q, k, scale) < 40
    outs = []
    for env in (None, "0"):
        if env is None:
            monkeypatch.delenv("CMFC_ATTN_FIXED_REF", raising=False)
        else:
            monkeypatch.setenv("CMFC_ATTN_FIXED_REF", env)
        out = np.empty((n, nh * hd), np.float32)
        gpu.dit_attention(q.transpose(1, 0, 2), k.transpose(1, 0, 2), v.transpose(1, 0, 2), nh, nkv, n, hd, scale, out)
        outs.append(out)
    want = attention_seq(q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), nh, nkv, hd)
    assert rel_l2(outs[0], want) < 6e-3 and rel_l2(outs[1], want) < 6e-3
    assert rel_l2(outs[0], outs[1]) < 4e-3


@pytest.mark.parametrize("sign,qa,ka,lo,hi", [(-1.0, 15.0, 14.0, 30, 47), (-1.0, 22.0, 21.0, 75, 95), (1.0, 22.0, 21.0, 75, 95)])
def test_attention_bounded_form_scores_at_the_edge_of_the_bound(sign, qa, ka, lo, hi):
    """Every key points away from (or along) every query, so all scores of a row sit near minus (plus) the
    bound: the exponentials are around 2^-85 (2^85), still normal numbers in f32 and bf16, and the result
    must not lose accuracy."""
    from cmf_b200 import gpu
    nh, nkv, hd, n = 2, 2, 64, 300
    rng = np.random.default_rng(5)
    u = rng.standard_normal(hd).astype(np.float32)
    u /= np.linalg.norm(u)
    q = np.broadcast_to(qa * u, (n, nh, hd)).astype(np.float32) + 0.05 * rng.standard_normal((n, nh, hd)).astype(np.float32)
    k = np.broadcast_to(sign * ka * u, (n, nkv, hd)).astype(np.float32) + 0.3 * rng.standard_normal((n, nkv, hd)).astype(np.float32)
    q, k = oc.bf16_round(q), oc.bf16_round(k)
    v = oc.bf16_round(rng.standard_normal((n, nkv, hd)).astype(np.float32))
    scale = 1.0 / np.sqrt(hd)
    b = _score_bound_log2(q, k, scale)
    assert lo < b < hi, b
    out = np.empty((n, nh * hd), np.float32)
    gpu.dit_attention(q.transpose(1, 0, 2), k.transpose(1, 0, 2), v.transpose(1, 0, 2), nh, nkv, n, hd, scale, out)
    want = attention_seq(q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), nh, nkv, hd)
    assert np.isfinite(out).all()
    assert rel_l2(out, want) < 6e-3, rel_l2(out, want)
