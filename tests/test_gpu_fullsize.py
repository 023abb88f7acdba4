"""Full-size cases (the largest sweep GEMM, the 2.6 B model at 1024x1024) checked through
size-independent properties, since the CPU oracle cannot run them in seconds: linearity and
row-sampled parity of the largest sweep GEMM; equality of the batched CFG pair with two single
forwards, and of a batch with its prompts run alone."""
import os

import numpy as np
import pytest

from oracle import codecs as oc
from tests.modelfile import rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("codec", ["q4t", "q4tp", "q8"])
def test_sweep_gemm_largest_shape_linearity_and_samples(tmp_path, codec):
    from cmf_b200 import Model, gpu, synth
    from cmf_b200.container import CmfWriter
    N, K, M = 9216, 2304, 17408
    dt = synth.CODECS[codec]
    path = str(tmp_path / "w.cmf")
    w = CmfWriter(arch={"arch_name": "sweep"})
    payload = gpu.encode_random(dt, 1, 0.02, N, K)       # W ~ N(0, 0.02), seed 1, quantized on the device
    w.add("w", dt, (N, K), payload)
    w.write(path, hash_tensors=False)
    rng = np.random.default_rng(1)
    x1 = rng.integers(-3, 4, (M, K)).astype(np.float32)   # small integers: exact in bf16, and so is x1 + x2
    x2 = rng.integers(-3, 4, (M, K)).astype(np.float32)
    call = {"q8": lambda m, x, o: gpu.q8_matmat(m, 0, None, x, M, N, K, o), "q4t": lambda m, x, o: gpu.q4t_matmat(m, 0, x, M, N, K, o),
            "q4tp": lambda m, x, o: gpu.q4tp_matmat(m, 0, x, M, N, K, o)}[codec]
    with Model(path) as m:
        y1, y2, y12 = (np.empty((M, N), np.float32) for _ in range(3))
        call(m, x1, y1)
        call(m, x2, y2)
        call(m, x1 + x2, y12)
    assert np.isfinite(y12).all()
    assert rel_l2(y1 + y2, y12) < 1e-5                     # linear up to f32 summation order
    pick = np.array([0, 255, 256, 4351, 8703, 17407])
    want = oc.matmat_exact(dt, payload, N, K, x1[pick])
    assert rel_l2(y1[pick], want) < (2e-5 if codec == "q8" else 4e-3)


def test_lumina_1024_pair_single_and_batch_consistency(tmp_path, monkeypatch):
    """The 2.6 B model with q4tp feed-forward and q8 attention weights at 1024x1024, 256 caption tokens."""
    from cmf_b200 import GenParams, Model, NextDit, denoise, synth
    path = os.path.join(str(tmp_path), "lumina.cmf")
    synth.write_model(path, synth.LUMINA2, attn="q8", ffn="q4tp", seed=0)
    rng = np.random.default_rng(0)
    lat = rng.standard_normal((2, 16, 128, 128)).astype(np.float32)
    cap = rng.standard_normal((2, 256, 2304)).astype(np.float32)
    cap_u = rng.standard_normal((2, 256, 2304)).astype(np.float32)
    with Model(path) as m:
        dit = NextDit(m)
        cc, cu = dit.refine_caption(cap[0]), dit.refine_caption(cap_u[0])
        pc, pu = dit.forward_cfg_pair(lat[0], 128, 128, cc, 256, cu, 256, 0.5)
        sc = dit.forward_with_cap(lat[0], 128, 128, cc, 256, 0.5)
        su = dit.forward_with_cap(lat[0], 128, 128, cu, 256, 0.5)
        assert np.isfinite(pc).all() and np.isfinite(pu).all()
        # the pair path batches two segments and shares the image branch; per sequence it is the
        # same function as the single forward (bf16 operand rounding may flip, hence a tolerance)
        assert rel_l2(pc, sc) < 5e-3 and rel_l2(pu, su) < 5e-3, (rel_l2(pc, sc), rel_l2(pu, su))
        assert rel_l2(pc, pu) > 1e-2   # the two branches really differ
        p = GenParams(steps=2, guidance_scale=4.0)
        both = denoise(dit, lat, cap, cap_u, p)
        one = denoise(dit, lat[1:2], cap[1:2], cap_u[1:2], p)
        assert rel_l2(one[0], both[1]) < 1e-5                # a prompt's result does not depend on its batch
        # The feed-forward down projection (K = 9216; 153 tiles per 4352-token sequence on 74 CTA pairs)
        # runs with the last 5 tiles of EVERY sequence cut along K; the plan depends on the position
        # inside the sequence only, which is what keeps the line above true.  Without the split: one
        # launch less per down projection (the kernel that adds the slices), the same result up to f32
        # summation order.  The forward walks the joint layers as two side-by-side chains (one per
        # sequence here), so there are 2 x 26 down projections; as one chain (CMFC_STREAMS=1) 26 --
        # and the very same bits, since no kernel's arithmetic depends on how the batch is cut.
        from cmf_b200 import gpu
        gpu.launch_count(reset=True)
        pc2, pu2 = dit.forward_cfg_pair(lat[0], 128, 128, cc, 256, cu, 256, 0.5)
        with_split = gpu.launch_count(reset=True)
        monkeypatch.setenv("CMFC_GEMM_SPLITK", "0")
        pc3, _ = dit.forward_cfg_pair(lat[0], 128, 128, cc, 256, cu, 256, 0.5)
        without = gpu.launch_count(reset=True)
        monkeypatch.delenv("CMFC_GEMM_SPLITK")
        assert np.array_equal(pc, pc2)
        assert with_split - without == 52, (with_split, without)
        # (last-bit differences of one GEMM grow through 26 blocks of bf16 operand rounding; the pair
        # path against two single forwards, above, is held to the same 5e-3)
        assert 0 < rel_l2(pc2, pc3) < 5e-3, rel_l2(pc2, pc3)
        monkeypatch.setenv("CMFC_STREAMS", "1")
        pc4, pu4 = dit.forward_cfg_pair(lat[0], 128, 128, cc, 256, cu, 256, 0.5)
        one_chain = gpu.launch_count(reset=True)
        monkeypatch.setenv("CMFC_GEMM_SPLITK", "0")
        dit.forward_cfg_pair(lat[0], 128, 128, cc, 256, cu, 256, 0.5)
        assert one_chain - gpu.launch_count(reset=True) == 26
        monkeypatch.delenv("CMFC_GEMM_SPLITK")
        monkeypatch.delenv("CMFC_STREAMS")
        assert np.array_equal(pc2, pc4) and np.array_equal(pu2, pu4)
        dit.close()
