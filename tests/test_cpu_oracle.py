"""CPU tests: the oracle against the reference's golden vectors and known-answer values, the
container writer/reader, and the C ABI's symbol table.  No GPU work."""
import ctypes
import importlib.util
import os
import re

import numpy as np
import pytest

from oracle import codecs as oc
from oracle import nextdit as nd
from tests import synth
from tests.modelfile import rel_l2

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "golden")


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


# ---- f16: crates/cortiq-core/src/quant.rs:871-891 known answers ----
def test_f16_known_answers():
    assert oc.f16_to_f32(0x0001) == 2.0 ** -24          # smallest subnormal
    assert oc.f16_to_f32(0x03FF) == 1023 * 2.0 ** -24   # largest subnormal
    assert oc.f16_to_f32(0x0400) == 2.0 ** -14          # smallest normal
    assert oc.f16_to_f32(0x812B) == -(0x12B) * 2.0 ** -24
    for h in (0x0001, 0x03FF, 0x0400, 0x812B, 0x3C00, 0x7BFF, 0xFBFF, 0x0000, 0x8000, 0x3555):
        assert oc.f32_to_f16(oc.f16_to_f32(h)) == h


def test_f16_matches_ieee_everywhere():
    hs = np.arange(65536, dtype=np.uint16)
    want = hs.view(np.float16).astype(np.float32)
    got = np.array([oc.f16_to_f32(int(h)) for h in hs], np.float32)
    ok = ~np.isnan(want)
    assert np.array_equal(got.view(np.uint32)[ok], want.view(np.uint32)[ok])
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(4000) * np.exp(rng.uniform(-9, 9, 4000))).astype(np.float32)
    x = x[np.abs(x) > 6.2e-5]  # normal halves: round-to-nearest-even, as IEEE
    got = np.array([oc.f32_to_f16(float(v)) for v in x], np.uint16)
    assert np.array_equal(got, x.astype(np.float16).view(np.uint16))


# ---- encoders / dequantizers against the reference's numpy implementation ----
def test_codecs_match_reference_python():
    g = np.load(os.path.join(GOLD, "codecs_ref.npz"))
    cases = _load(os.path.join(GOLD, "make_codecs_ref.py"), "mk").inputs()
    for k, w in cases.items():
        assert np.array_equal(oc.encode(oc.Q8_ROW, w), g[k + "_q8"]), k
        assert np.array_equal(oc.encode_q4_block(w), g[k + "_q4block"]), k
        assert np.array_equal(oc.dequant(oc.Q8_ROW, g[k + "_q8"], *w.shape), g[k + "_q8_deq"]), k
        tiled = oc.encode(oc.Q4_TILED, w)
        assert np.array_equal(oc.dequant(oc.Q4_TILED, tiled, *w.shape), g[k + "_q4t_deq"]), k
        # q4_tiled == q4_block values, scale moved to the head of each tile (qtensor.rs:11154)
        blk = g[k + "_q4block"]
        n = w.size // 32
        assert np.array_equal(tiled.reshape(n, 18)[:, 2:].reshape(-1), blk[:n * 16])
        assert np.array_equal(tiled.reshape(n, 18)[:, :2].reshape(-1), blk[n * 16:])


def test_hash64_matches_reference():
    from cmf_b200.container import hash64
    g = np.load(os.path.join(GOLD, "codecs_ref.npz"))
    for k in ("w0", "w1", "w2"):
        assert hash64(g[k + "_q8"].tobytes()) == int(g[k + "_hash"][0])


def _tile_spread_rows(rows, cols, spread, seed=3):
    """Rows whose per-tile amplitude spreads over `spread` powers of two, row amplitudes over six
    decades: the axis a per-row scale ladder has to cope with (the shape of the reference's
    q4tp test inputs, crates/cortiq-cli/src/convert.rs:4070-4095)."""
    rng = np.random.default_rng(seed)
    amp = 10.0 ** ((np.arange(rows) % 7) - 3.0)
    tilt = np.exp2(np.abs(rng.uniform(-1, 1, (rows, cols // 32))) * spread)
    v = rng.uniform(-1, 1, (rows, cols // 32, 32)) * amp[:, None, None] * tilt[:, :, None]
    return v.reshape(rows, cols).astype(np.float32)


def test_q4tp_payload_length():  # convert.rs:4413-4424
    for rows, cols in ((1, 32), (7, 64), (16, 2048), (2048, 512)):
        w = _tile_spread_rows(rows, cols, 1.27)
        gpr = cols // 32
        assert oc.encode(oc.Q4TP, w).size == rows * gpr * 16 + rows * 4 + rows * ((gpr * 5 + 7) // 8)


def test_q4tp_code_packing_every_offset():  # convert.rs:4426-4440
    gpr = 37
    want = [(g * 7 + 3) % 32 for g in range(gpr)]
    stride = (gpr * 5 + 7) // 8
    buf = np.zeros(stride, np.uint8)
    for g, c in enumerate(want):
        bit = g * 5
        buf[bit // 8] |= (c << (bit % 8)) & 0xFF
        if bit % 8 > 3:
            buf[bit // 8 + 1] |= c >> (8 - bit % 8)
    got = [oc.lib().orc_q4tp_code(buf.ctypes.data, stride, g) for g in range(gpr)]
    assert got == want


def test_q4tp_error_budget_vs_q4t():  # convert.rs:4442-4463
    rows, cols = 256, 2048
    for spread, budget in ((0.0, 1.02), (1.27, 1.02), (1.89, 1.03), (3.70, 1.06)):
        w = _tile_spread_rows(rows, cols, spread)
        a = oc.dequant(oc.Q4_TILED, oc.encode(oc.Q4_TILED, w), rows, cols)
        b = oc.dequant(oc.Q4TP, oc.encode(oc.Q4TP, w), rows, cols)
        assert rel_l2(b, w) <= rel_l2(a, w) * budget, spread


def test_q4tp_dead_tile_stays_zero():  # convert.rs:4465-4484
    w = _tile_spread_rows(4, 128, 1.27)
    w[1, :32] = 0.0
    out = oc.dequant(oc.Q4TP, oc.encode(oc.Q4TP, w), 4, 128)
    assert np.all(out[1, :32] == 0.0)
    assert rel_l2(out[1, 32:], w[1, 32:]) < 0.15


def test_q4tp_ladder_is_iterated():  # quant.rs:396-411: one exp2 then 31 multiplies
    t = oc.q4tp_ladder(oc.f32_to_f16(-9.37), oc.f32_to_f16(0.113))
    r = np.exp2(np.float32(oc.f16_to_f32(oc.f32_to_f16(0.113)))).astype(np.float32)
    x = np.float32(np.exp2(np.float32(oc.f16_to_f32(oc.f32_to_f16(-9.37)))))
    for c in range(32):
        assert abs(t[c] - x) <= 2e-7 * x  # libm exp2f vs numpy exp2 may differ in the last bit
        x = np.float32(x * r)


def test_exact_matmat_equals_dense_product():  # qtensor.rs:10702: exact path == dequant then dot
    rng = np.random.default_rng(2)
    w = (rng.standard_normal((64, 256)) * 0.02).astype(np.float32)
    x = rng.standard_normal((5, 256)).astype(np.float32)
    for dt in (oc.Q8_ROW, oc.Q4_TILED, oc.Q4TP):
        p = oc.encode(dt, w)
        y = oc.matmat_exact(dt, p, 64, 256, x)
        ref = x.astype(np.float64) @ oc.dequant(dt, p, 64, 256).astype(np.float64).T
        assert rel_l2(y, ref) < 2e-6


# ---- the forward against the reference's numpy forward ----
@pytest.mark.parametrize("case", ["tiny", "tiny_ragged"])
@pytest.mark.parametrize("exact", [False, True])
def test_oracle_forward_matches_reference_numpy(case, exact):
    mk = _load(os.path.join(GOLD, "make_nextdit_ref.py"), "mkref")
    cfg, wseed, jit, std, iseed, H, W, cap_n, t = mk.CASES[case]
    gold = np.load(os.path.join(GOLD, f"nextdit_ref_{case}.npz"))
    tensors = synth.make_tensors(cfg, wseed, jit, std)
    latent, cap = mk.inputs(cfg, iseed, H, W, cap_n)
    m = nd.NextDitOracle(tensors, cfg, exact=exact)
    m.block_taps = []
    pred = m.forward_with_cap(latent, H, W, m.refine_caption(cap), t)
    joint = [x for p, x in m.block_taps if p.startswith("dit.layers")]
    # the reference's own parity bar: max |got - want| / max(|want|, 1) < 1e-3 (tests/dit_parity.rs:44-55)
    assert np.max(np.abs(pred - gold["pred"]) / np.maximum(np.abs(gold["pred"]), 1.0)) < 1e-4
    assert rel_l2(joint[0], gold["first_block"]) < 1e-5
    assert rel_l2(joint[-1], gold["last_block"]) < 1e-5


def test_cfg_pair_equals_two_single_forwards():
    cfg = synth.TINY
    tensors = synth.make_tensors(cfg, 1, 0.1, 0.05)
    rng = np.random.default_rng(7)
    latent = rng.standard_normal((16, 8, 12)).astype(np.float32)
    m = nd.NextDitOracle(tensors, cfg)
    c1 = m.refine_caption(rng.standard_normal((9, 256)).astype(np.float32))
    c2 = m.refine_caption(rng.standard_normal((3, 256)).astype(np.float32))
    pc, pu = m.forward_cfg_pair(latent, 8, 12, c1, c2, 0.3)
    assert rel_l2(pc, m.forward_with_cap(latent, 8, 12, c1, 0.3)) < 1e-5
    assert rel_l2(pu, m.forward_with_cap(latent, 8, 12, c2, 0.3)) < 1e-5


def test_sigmas_and_loop_pieces():
    sg = nd.sigmas(30)
    assert len(sg) == 31 and sg[0] == 1.0 and sg[-1] == 0.0
    assert all(a > b for a, b in zip(sg, sg[1:]))
    assert abs(sg[29] - 6.0 * (1 / 30) / (1 + 5.0 / 30)) < 1e-15
    z = nd.gauss_latent(4096, 42)
    assert z.dtype == np.float32 and abs(float(z.mean())) < 0.06 and abs(float(z.std()) - 1) < 0.05
    assert np.array_equal(z, nd.gauss_latent(4096, 42)) and not np.array_equal(z, nd.gauss_latent(4096, 43))
    c = np.ones((2, 4), np.float32)
    u = np.zeros((2, 4), np.float32)
    comb = nd.cfg_combine(c, u, 4.0, 4)
    assert np.allclose(np.linalg.norm(comb, axis=1), np.linalg.norm(c, axis=1))


# ---- container ----
def test_container_roundtrip_and_validation(tmp_path):
    import cmf_b200
    from cmf_b200.container import CmfWriter, Model
    from cmf_b200._lib import CmfCudaError
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((128, 64)) * 0.02).astype(np.float32)
    wr = CmfWriter(arch={"arch_name": "t", "hidden_size": 64, "num_layers": 0, "vocab_size": 0})
    wr.add("a.q8", oc.Q8_ROW, w.shape, oc.encode(oc.Q8_ROW, w))
    wr.add("a.q4t", oc.Q4_TILED, w.shape, oc.encode(oc.Q4_TILED, w))
    wr.add("a.q4tp", oc.Q4TP, w.shape, oc.encode(oc.Q4TP, w))
    wr.add_f32("a.f32", w)
    big = rng.standard_normal((64, 128)).astype(np.float32)  # 32 KiB: must land 4096-aligned
    wr.add_f32("big", big)
    wr.add_json("dit.config_json", {"hidden_size": 64})
    path = str(tmp_path / "t.cmf")
    wr.write(path)
    with Model(path) as m:
        assert len(m) == 6
        for name, dt in (("a.q8", 3), ("a.q4t", 11), ("a.q4tp", 15), ("a.f32", 0), ("big", 0)):
            i = m.index(name)
            d, shape, nb = m.info(i)
            assert d == dt and nb == oc.nbytes(dt, *shape) and shape == ((128, 64) if name != "big" else (64, 128))
        assert np.array_equal(m.tensor_bytes(m.index("a.q4tp")), oc.encode(oc.Q4TP, w))
        assert np.array_equal(m.tensor_bytes(m.index("big")).view(np.float32).reshape(64, 128), big)
        with pytest.raises(CmfCudaError) as e:
            m.index("nope")
        assert e.value.code == -9
    raw = bytearray(open(path, "rb").read())
    for mutate, frag in ((lambda b: b.__setitem__(0, 0x58), "magic"),
                         (lambda b: b.__setitem__(4, 3), "version"),
                         (lambda b: b.__setitem__(130, b[130] ^ 1), "header hash"),
                         (lambda b: b.__setitem__(12, 0x80), "feature")):
        bad = bytearray(raw)
        mutate(bad)
        p2 = str(tmp_path / "bad.cmf")
        open(p2, "wb").write(bad)
        with pytest.raises(CmfCudaError) as e:
            Model(p2)
        assert e.value.code == -8 and frag in str(e.value)
    open(str(tmp_path / "short.cmf"), "wb").write(raw[:100])
    with pytest.raises(CmfCudaError):
        Model(str(tmp_path / "short.cmf"))
    with pytest.raises(CmfCudaError) as e:
        Model(str(tmp_path / "missing.cmf"))
    assert e.value.code == -7


def test_reader_rejects_wrapping_offsets_and_unimplemented_features(tmp_path):
    """Offsets, lengths and counts of an untrusted file must not wrap the reader's bounds checks
    (the reference uses checked arithmetic, crates/cortiq-core/src/format.rs:700-712), and a file
    that REQUIRES a feature this backend does not implement (binary masks, two-factor quantization)
    is refused instead of being run with the feature ignored."""
    import struct
    from cmf_b200 import CmfCudaError, Model
    from cmf_b200.container import CmfWriter, hash64
    w = (np.random.default_rng(0).standard_normal((128, 64)) * 0.02).astype(np.float32)
    wr = CmfWriter(arch={"arch_name": "t", "hidden_size": 64, "num_layers": 1, "vocab_size": 0})
    wr.add("a.q8", oc.Q8_ROW, w.shape, oc.encode(oc.Q8_ROW, w))
    wr.add_f32("a.f32", w)
    path = str(tmp_path / "t.cmf")
    wr.write(path)
    raw = bytearray(open(path, "rb").read())
    with Model(path) as m:
        assert len(m) == 2
    dir_off, dir_len = struct.unpack_from("<QQ", raw, 0x20)
    TOP = (1 << 64) - 8

    def reseal(b):      # a forged directory still carries a matching directory hash
        struct.pack_into("<Q", b, 0x78, hash64(bytes(b[dir_off:dir_off + dir_len])))

    def mut_env(at, value):
        def f(b):
            struct.pack_into("<Q", b, at, value)
        return f

    def mut_dir(at, fmt, value):
        def f(b):
            struct.pack_into(fmt, b, dir_off + at, value)
            reseal(b)
        return f
    cases = [
        (mut_env(0x10, TOP), "section"),                       # hdr_off + hdr_len wraps
        (mut_env(0x18, TOP), "section"),                       # hdr_len huge
        (mut_env(0x20, TOP), "section"),                       # dir_off wraps
        (mut_env(0x28, (1 << 64) - 1), "section"),             # dir_len huge
        (mut_env(0x30, TOP - (TOP % 4096)), "section"),        # data_off wraps
        (mut_env(0x38, (1 << 64) - 1), "section"),             # data_len huge
        (mut_dir(0, "<Q", (1 << 64) // 56 + 1), "directory"),  # count * 56 wraps to a small number
        (mut_dir(8, "<Q", (1 << 63)), "directory"),            # pool_off beyond the section
        (mut_dir(16 + 0, "<I", 0xFFFFFFF0), "name"),           # name_off far past the pool
        (mut_dir(16 + 32, "<Q", TOP - (TOP % 64)), "data section"),   # tensor off + nbytes wraps
        (mut_dir(16 + 40, "<Q", (1 << 64) - 64), "data section"),     # tensor nbytes huge
    ]
    for k, (mutate, frag) in enumerate(cases):
        bad = bytearray(raw)
        mutate(bad)
        p2 = str(tmp_path / f"bad{k}.cmf")
        open(p2, "wb").write(bad)
        with pytest.raises(CmfCudaError) as e:
            Model(p2)
        assert e.value.code == -8 and frag in str(e.value), (k, str(e.value))
    for required in (1 | 2, 1 | 4, 2, 4):   # FEAT_BINARY_MASKS, FEAT_QUANT_2F (format.rs required_features)
        bad = bytearray(raw)
        struct.pack_into("<I", bad, 12, required)
        p2 = str(tmp_path / f"feat{required}.cmf")
        open(p2, "wb").write(bad)
        with pytest.raises(CmfCudaError) as e:
            Model(p2)
        assert e.value.code == -8 and "feature" in str(e.value)


def test_reader_opens_a_container_written_by_the_reference_writer():
    """tests/golden/container_ref_q8.cmf was produced by the reference's own Python writer
    (converter/convert_dtgma_to_cmf.py _write_cmf / encode_directory:1095-1116; generator
    tests/golden/make_container_ref.py).  Its directory starts right after the header JSON (no
    64-byte rounding), 1-D tensors are f16 and every record carries a tensor hash."""
    from cmf_b200 import Model
    from cmf_b200.container import hash64
    want = np.load(os.path.join(GOLD, "container_ref_q8.npz"))
    with Model(os.path.join(GOLD, "container_ref_q8.cmf")) as m:
        assert len(m) == len(want.files)
        # canonical order of the reference writer: final norm, lm_head, then layers by index
        assert [m.name(i) for i in range(len(m))] == ["model.norm.weight", "lm_head.weight",
                                                      "model.layers.0.self_attn.q_proj.weight",
                                                      "model.layers.1.mlp.down_proj.weight"]
        for name in want.files:
            w = want[name]
            i = m.index(name)
            dt, shape, nb = m.info(i)
            raw = np.array(m.tensor_bytes(i), copy=True)
            assert shape == w.shape
            if w.ndim == 1:
                assert dt == 1 and np.array_equal(raw.view(np.float16), w.astype(np.float16))
            else:
                # the reference's numpy encode_q8_row and the oracle's restatement emit the same bytes
                assert dt == oc.Q8_ROW and np.array_equal(raw, oc.encode(oc.Q8_ROW, w))
                assert np.array_equal(oc.dequant(oc.Q8_ROW, raw, *w.shape), oc.dequant(oc.Q8_ROW, oc.encode(oc.Q8_ROW, w), *w.shape))
            assert nb == raw.size and hash64(raw.tobytes()) != 0


def test_container_is_readable_by_reference_reader(tmp_path):
    """Cross-check the writer with the reference's standalone reader where the reference checkout
    is available (CMF_REFERENCE=<checkout>); elsewhere this is covered by the library's own reader."""
    ref = os.environ.get("CMF_REFERENCE", "")
    if not ref or not os.path.exists(os.path.join(ref, "python", "cmf_reader.py")):
        pytest.skip("reference checkout not mounted")
    rd = _load(os.path.join(ref, "python", "cmf_reader.py"), "cmf_reader_ref")
    from cmf_b200.container import CmfWriter
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((32, 64)) * 0.02).astype(np.float32)
    wr = CmfWriter(arch={"arch_name": "t", "hidden_size": 64, "num_layers": 1, "vocab_size": 0})
    wr.add("w.q8", oc.Q8_ROW, w.shape, oc.encode(oc.Q8_ROW, w))
    wr.add("w.q4t", oc.Q4_TILED, w.shape, oc.encode(oc.Q4_TILED, w))
    wr.add_f32("w.f32", w)
    path = str(tmp_path / "x.cmf")
    wr.write(path)
    r = rd.CmfReader(path)
    assert r.verify() == []
    assert np.array_equal(r.tensor("w.f32"), w)
    assert np.array_equal(r.tensor("w.q8"), oc.dequant(oc.Q8_ROW, oc.encode(oc.Q8_ROW, w), 32, 64))
    assert np.array_equal(r.tensor("w.q4t"), oc.dequant(oc.Q4_TILED, oc.encode(oc.Q4_TILED, w), 32, 64))
    r.close()


# ---- C ABI ----
def test_library_exports_every_declared_symbol():
    import cmf_b200
    from cmf_b200._lib import SYMBOLS
    hdr = open(os.path.join(os.path.dirname(HERE), "include", "cmf_cuda.h")).read()
    declared = set(re.findall(r"\b(cmfc_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations parsed"
    L = ctypes.CDLL(cmf_b200.library_path())
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} is declared in include/cmf_cuda.h but not exported"
    assert declared == set(SYMBOLS), declared ^ set(SYMBOLS)


def test_bad_arguments_never_reach_a_launch():
    import cmf_b200
    L = cmf_b200.lib()
    assert L.cmfc_model_open(None, None) == -1
    assert L.cmfc_model_find(None, b"x") == -1
    assert L.cmfc_payload_nbytes(3, 4, 8) == 4 * 8 + 8
    assert L.cmfc_payload_nbytes(11, 4, 64) == 4 * 2 * 18
    assert L.cmfc_payload_nbytes(15, 7, 64) == 7 * 2 * 16 + 7 * 4 + 7 * 2
    assert b"null" in L.cmfc_last_error()


def test_product_gauss_latent_equals_oracle():
    """cmf_b200.imagegen.gauss_latent (vectorised) against the scalar restatement of
    crates/cortiq-engine/src/imagegen.rs:75-108."""
    from cmf_b200.imagegen import gauss_latent, to_rgb01
    from oracle.nextdit import gauss_latent as ref
    for n, seed in ((1, 0), (7, 42), (1001, 1), (4096, 2 ** 63 + 5)):
        assert np.array_equal(gauss_latent(n, seed), ref(n, seed))
    assert to_rgb01(np.array([-3.0, -1.0, 0.0, 1.0, 3.0], np.float32)).tolist() == [0.0, 0.0, 0.5, 1.0, 1.0]
