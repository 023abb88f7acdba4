"""GPU parity of the dequant-fused GEMM through the facade entries q8_matmat / q4t_matmat /
q4tp_matmat, dit_qkv and the fused FFN, against the strict CPU kernels of the oracle."""
import numpy as np
import pytest

from oracle import codecs as oc
from tests.modelfile import rel_l2, single_weight_file

pytestmark = pytest.mark.gpu

TOL = 1e-2  # relative L2 on Y (north-star tolerance), inputs rounded to bf16 on the device


def _call(gpu, dt, m, idx, x, rows, cols):
    out = np.empty((x.shape[0], rows), np.float32)
    if dt == oc.Q8_ROW:
        gpu.q8_matmat(m, idx, None, x, x.shape[0], rows, cols, out)
    elif dt == oc.Q4_TILED:
        gpu.q4t_matmat(m, idx, x, x.shape[0], rows, cols, out)
    else:
        gpu.q4tp_matmat(m, idx, x, x.shape[0], rows, cols, out)
    return out


@pytest.mark.parametrize("dt", [oc.Q8_ROW, oc.Q4_TILED, oc.Q4TP])
@pytest.mark.parametrize("shape", [(128, 64, 1), (128, 64, 256), (256, 256, 288), (384, 2304, 700), (2304, 1024, 33)])
def test_matmat_small(tmp_path, dt, shape):
    from cmf_b200 import Model, gpu
    rows, cols, b = shape
    rng = np.random.default_rng(rows + cols + b)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    x = oc.bf16_round(rng.standard_normal((b, cols)).astype(np.float32))
    path = str(tmp_path / "w.cmf")
    q = single_weight_file(path, [("w", dt, w)])["w"]
    with Model(path) as m:
        got = _call(gpu, dt, m, m.index("w"), x, rows, cols)
        # twice: the second call runs against resident weights and reused workspaces
        got2 = _call(gpu, dt, m, m.index("w"), x, rows, cols)
    want = oc.matmat_exact(dt, q.payload, rows, cols, x)
    assert np.array_equal(got, got2)
    err = rel_l2(got, want)
    # q8 levels are exact in bf16 and x is bf16-exact: only f32 summation order differs
    assert err < (2e-5 if dt == oc.Q8_ROW else 4e-3), err
    assert err < TOL


_SWEEP_X = {}


def _sweep_x(M, K):
    """X ~ N(0, 1) rounded to bf16, seed 1, one array per (M, K) shared by the codecs and widths."""
    if (M, K) not in _SWEEP_X:
        _SWEEP_X.clear()                                  # one resident array at a time (up to 640 MB)
        rng = np.random.default_rng(1)
        _SWEEP_X[(M, K)] = oc.bf16_round(rng.standard_normal((M, K), dtype=np.float32))
    return _SWEEP_X[(M, K)]


def _sample_rows(M, rng):
    """First and last token, both sides of a few 256-token tile edges, and random tokens."""
    rows = {0, M - 1}
    edges = np.arange(256, M, 256)
    for e in (rng.choice(edges, min(6, edges.size), replace=False) if edges.size else []):
        rows.update((int(e) - 1, int(e)))
    rows.update(int(r) for r in rng.choice(M, 10, replace=False))
    return np.array(sorted(rows))


@pytest.mark.parametrize("codec", ["q8", "q4t", "q4tp"])
@pytest.mark.parametrize("K,N", [(2304, 2304), (2304, 6912), (2304, 9216), (9216, 2304)])
@pytest.mark.parametrize("M", [256, 4352, 17408])
def test_matmat_op_sweep(tmp_path, M, K, N, codec):
    """The op-level sweep Y[M, N] = X[M, K] . W^T: W ~ N(0, 0.02) quantized by the (byte-identical)
    device encoder from seed 1, X ~ N(0, 1) in bf16 from seed 1, every (K, N) x M x codec point
    against the strict CPU kernels (crates/cortiq-engine/src/qtensor.rs:3533-3546, :4418-4432,
    :4647-4661) on sampled token rows.  M = 256 is served by the single-CTA kernel (fewer tiles
    than SM pairs), the larger M by the CTA-pair kernel."""
    from cmf_b200 import Model, gpu, synth
    from cmf_b200.container import CmfWriter
    dt = synth.CODECS[codec]
    path = str(tmp_path / "w.cmf")
    wr = CmfWriter(arch={"arch_name": "sweep"})
    payload = gpu.encode_random(dt, 1, 0.02, N, K)
    wr.add("w", dt, (N, K), payload)
    wr.write(path, hash_tensors=False)
    x = _sweep_x(M, K)
    with Model(path) as m:
        got = _call(gpu, dt, m, 0, x, N, K)
    assert np.isfinite(got).all()
    pick = _sample_rows(M, np.random.default_rng(M + K + N))
    want = oc.matmat_exact(dt, payload, N, K, x[pick])
    err = rel_l2(got[pick], want)
    assert err < (2e-5 if codec == "q8" else 4e-3), (M, K, N, codec, err)
    assert err < TOL


@pytest.mark.parametrize("dt", [oc.Q8_ROW, oc.Q4_TILED, oc.Q4TP])
def test_gemm_operand_is_the_rounded_reference_dequant(tmp_path, dt):
    """One-hot activations read the tensor-core A operand back: Y[k, n] = operand[n, k].  For the
    4-bit codecs it must be RN_bf16(reference f32 dequant) bit for bit; for q8 the integer level
    is the operand and the f32 row scale is applied after, which reproduces the dequant exactly."""
    from cmf_b200 import Model, gpu
    rows, cols = 256, 256
    rng = np.random.default_rng(77)
    w = (rng.standard_normal((rows, cols)) * np.exp(rng.uniform(-6, 3, (rows, 1)))).astype(np.float32)
    w[5, 40] = 900.0
    path = str(tmp_path / "w.cmf")
    q = single_weight_file(path, [("w", dt, w)])["w"]
    x = np.eye(cols, dtype=np.float32)
    with Model(path) as m:
        got = _call(gpu, dt, m, m.index("w"), x, rows, cols)   # [cols, rows]
    dense = oc.dequant(dt, q.payload, rows, cols)
    want = dense.T if dt == oc.Q8_ROW else oc.bf16_round(dense).T
    assert np.array_equal(got.view(np.uint32), np.ascontiguousarray(want).view(np.uint32))


def test_matmat_rejects_wrong_codec_and_shape(tmp_path):
    from cmf_b200 import CmfCudaError, Model, gpu
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((128, 64)) * 0.02).astype(np.float32)
    path = str(tmp_path / "w.cmf")
    single_weight_file(path, [("w", oc.Q8_ROW, w), ("odd", oc.Q8_ROW, w[:100])])
    x = np.zeros((4, 64), np.float32)
    out = np.empty((4, 128), np.float32)
    with Model(path) as m:
        with pytest.raises(CmfCudaError) as e:
            gpu.q4t_matmat(m, m.index("w"), x, 4, 128, 64, out)
        assert e.value.code == -2
        with pytest.raises(CmfCudaError) as e:
            gpu.q8_matmat(m, m.index("w"), None, np.zeros((4, 128), np.float32), 4, 64, 128, np.empty((4, 64), np.float32))
        assert e.value.code == -3
        with pytest.raises(CmfCudaError) as e:  # 100 rows: not a multiple of the 128-row tile
            gpu.q8_matmat(m, m.index("odd"), None, x, 4, 100, 64, np.empty((4, 100), np.float32))
        assert e.value.code == -3
        with pytest.raises(CmfCudaError):
            gpu.q8_matmat(m, 99, None, x, 4, 128, 64, out)


@pytest.mark.parametrize("codecs", [(oc.Q8_ROW, oc.Q8_ROW), (oc.Q4TP, oc.Q4_TILED), (oc.Q4_TILED, oc.Q4TP)])
def test_qkv_and_ffn(tmp_path, codecs):
    from cmf_b200 import Model, gpu
    from oracle.nextdit import silu
    hs, inter, nq, nkv, b = 256, 1024, 256, 128, 300
    rng = np.random.default_rng(4)
    mats = {"q": (nq, hs), "k": (nkv, hs), "v": (nkv, hs), "w1": (inter, hs), "w3": (inter, hs), "w2": (hs, inter)}
    ws = {k: (rng.standard_normal(s) * 0.05).astype(np.float32) for k, s in mats.items()}
    a, f = codecs
    entries = [(k, a if k in "qkv" else f, v) for k, v in ws.items()]
    path = str(tmp_path / "w.cmf")
    qs = single_weight_file(path, entries)
    x = oc.bf16_round(rng.standard_normal((b, hs)).astype(np.float32))
    with Model(path) as m:
        qo, ko, vo = (np.empty((b, nq), np.float32), np.empty((b, nkv), np.float32), np.empty((b, nkv), np.float32))
        gpu.dit_qkv(m, m.index("q"), m.index("k"), m.index("v"), x, b, hs, nq, nkv, qo, ko, vo)
        out = np.empty((b, hs), np.float32)
        gpu.q4t_ffn(m, m.index("w1"), m.index("w3"), m.index("w2"), x, b, hs, inter, out)
    for got, k in ((qo, "q"), (ko, "k"), (vo, "v")):
        want = oc.matmat_exact(qs[k].dtype, qs[k].payload, *mats[k], x)
        assert rel_l2(got, want) < 4e-3, k
    g = oc.matmat_exact(qs["w1"].dtype, qs["w1"].payload, inter, hs, x)
    u = oc.matmat_exact(qs["w3"].dtype, qs["w3"].payload, inter, hs, x)
    want = oc.matmat_exact(qs["w2"].dtype, qs["w2"].payload, hs, inter, silu(g) * u)
    assert rel_l2(out, want) < TOL


@pytest.mark.parametrize("dt", [oc.Q8_ROW, oc.Q4_TILED, oc.Q4TP])
@pytest.mark.parametrize("M", [4352, 2700])
def test_pair_kernel_equals_single_cta_kernel(tmp_path, monkeypatch, dt, M):
    """The CTA-pair GEMM (2-SM MMA, 256 x 256 tiles) and the single-CTA GEMM (128 x 256 tiles) feed
    the tensor core the same operands in the same k order: same bits out (with the K split of the
    last partial wave off, which adds partial sums in another order).  M = 2700 leaves a ragged
    last token tile whose second half is entirely out of range."""
    from cmf_b200 import Model, gpu
    rng = np.random.default_rng(3)
    K, N = 2304, 9216                                   # 36 row pairs x 11 or 17 token tiles: the pair path
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = oc.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    path = str(tmp_path / "w.cmf")
    single_weight_file(path, [("w", dt, w)])
    with Model(path) as m:
        monkeypatch.setenv("CMFC_GEMM_PAIR", "1")
        monkeypatch.setenv("CMFC_GEMM_SPLITK", "0")
        a = _call(gpu, dt, m, m.index("w"), x, N, K)
        monkeypatch.setenv("CMFC_GEMM_PAIR", "0")
        b = _call(gpu, dt, m, m.index("w"), x, N, K)
    assert np.isfinite(a).all()
    assert np.array_equal(a, b)


@pytest.mark.parametrize("dt", [oc.Q8_ROW, oc.Q4_TILED, oc.Q4TP])
@pytest.mark.parametrize("M,K,N", [(8704, 9216, 2304), (4352, 4096, 4608), (2700, 8192, 2304)])
def test_pair_kernel_k_split_of_last_wave(tmp_path, monkeypatch, dt, M, K, N):
    """These shapes (K of 4096 or more) leave a last wave of tiles that fills less than half of the 74
    CTA pairs (10, 10 and 25 tiles); the kernel cuts those tiles along K into slices for all pairs and a
    second kernel adds the slices in order.  Same result as the unsplit kernel up to the f32 summation
    order, identical from run to run, and every tile outside the last wave bit-identical."""
    from cmf_b200 import Model, gpu
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = oc.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    path = str(tmp_path / "w.cmf")
    single_weight_file(path, [("w", dt, w)])
    with Model(path) as m:
        monkeypatch.setenv("CMFC_GEMM_PAIR", "1")
        monkeypatch.setenv("CMFC_GEMM_SPLITK", "1")
        a = _call(gpu, dt, m, m.index("w"), x, N, K)
        a2 = _call(gpu, dt, m, m.index("w"), x, N, K)
        monkeypatch.setenv("CMFC_GEMM_SPLITK", "0")
        b = _call(gpu, dt, m, m.index("w"), x, N, K)
    assert np.isfinite(a).all()
    assert np.array_equal(a, a2)
    # the tensor core accumulates a tile's K = 2304 ... 9216 products in f32 inside the MMA; adding seven
    # shorter partial sums afterwards changes the split tiles by a few 1e-6 relative (measured 1.4e-6
    # over the whole output for K = 9216, where 10 of 306 tiles are split)
    assert rel_l2(a, b) < 5e-6, rel_l2(a, b)
    tiles_n, tiles_m = N // 256, (M + 255) // 256
    full = (tiles_n * tiles_m) // 74 * 74
    assert full < tiles_n * tiles_m
    differs = 0
    for tile in range(tiles_n * tiles_m):
        n0, m0 = (tile % tiles_n) * 256, (tile // tiles_n) * 256
        same = np.array_equal(a[m0:m0 + 256, n0:n0 + 256], b[m0:m0 + 256, n0:n0 + 256])
        if tile < full:
            assert same, tile
        else:
            differs += not same
    assert differs > 0      # the split path really ran


@pytest.mark.parametrize("dt", [oc.Q4_TILED, oc.Q4TP])
def test_k_split_planned_per_prompt_is_batch_independent(tmp_path, monkeypatch, dt):
    """Inside a forward the K split is planned per prompt (period): the last 10 of the 306 tiles of
    EVERY 8704-token prompt are cut, whatever the number of prompts in the launch.  A stack of two
    prompts therefore gives each prompt the bits it gets alone, while the split tiles differ from the
    unsplit kernel in the f32 summation order only."""
    from cmf_b200 import Model, gpu
    K, N, T = 9216, 2304, 8704
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = oc.bf16_round(rng.standard_normal((2 * T, K)).astype(np.float32))
    path = str(tmp_path / "w.cmf")
    single_weight_file(path, [("w", dt, w)])
    with Model(path) as m:
        monkeypatch.setenv("CMFC_GEMM_SPLITK", str(T))
        both = _call(gpu, dt, m, m.index("w"), x, N, K)
        first = _call(gpu, dt, m, m.index("w"), x[:T], N, K)
        second = _call(gpu, dt, m, m.index("w"), x[T:], N, K)
        monkeypatch.setenv("CMFC_GEMM_SPLITK", "0")
        plain = _call(gpu, dt, m, m.index("w"), x, N, K)
    assert np.array_equal(both[:T], first) and np.array_equal(both[T:], second)
    assert rel_l2(both, plain) < 5e-6
    tiles_n, per = N // 256, (T // 256) * (N // 256)
    differs = 0
    for tile in range(2 * per):
        n0, m0 = (tile % tiles_n) * 256, (tile // tiles_n) * 256
        same = np.array_equal(both[m0:m0 + 256, n0:n0 + 256], plain[m0:m0 + 256, n0:n0 + 256])
        if tile % per < per // 74 * 74:
            assert same, tile                     # whole tiles: bit-identical to the unsplit kernel
        else:
            differs += not same
    assert differs > 0                            # the split path really ran, in both prompts
