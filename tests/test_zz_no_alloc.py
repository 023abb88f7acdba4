"""The allocation-free linear entry (cmfc_matmat_device_noalloc) against the regular entry.

Collected last on purpose: a run that stops at the first failure has then already executed every
other test.  Serves hosts that cannot call cudaMalloc when the linear runs (a foreign memory pool
owns the device memory, or the call sits on a path where allocating is not allowed), so the
activation staging buffer is a fixed array inside the library instead of a workspace."""
import numpy as np
import pytest

from oracle import codecs as oc
from tests.modelfile import rel_l2, single_weight_file

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dt", [oc.Q8_ROW, oc.Q4TP])
def test_noalloc_matches_regular_entry_twice(tmp_path, dt):
    import torch
    from cmf_b200 import CmfCudaError, Model, gpu
    rows, cols = 384, 2304
    rng = np.random.default_rng(21)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    path = str(tmp_path / "w.cmf")
    single_weight_file(path, [("w", dt, w)])
    gpu.set_current_device(0)
    with Model(path) as m:
        idx = m.index("w")
        for call, b in enumerate((700, 130)):   # two calls in a row; the second reuses the scratch
            x = rng.standard_normal((b, cols)).astype(np.float32)
            want = np.empty((b, rows), np.float32)
            if dt == oc.Q8_ROW:
                gpu.q8_matmat(m, idx, None, x, b, rows, cols, want)   # also makes the tensor resident
            else:
                gpu.q4tp_matmat(m, idx, x, b, rows, cols, want)
            assert gpu.weight_is_resident(m, idx)
            dx = torch.from_numpy(x).cuda()
            dy = torch.full((b, rows), float("nan"), device="cuda", dtype=torch.float32)
            torch.cuda.synchronize()
            gpu.matmat_device_noalloc(m, idx, dx.data_ptr(), b, dy.data_ptr())
            got = dy.cpu().numpy()
            assert np.isfinite(got).all()
            assert rel_l2(got, want) < 1e-6, (call, rel_l2(got, want))   # same kernels, same operands
        # beyond the fixed scratch: rejected with a clear status, nothing launched
        too_many = gpu.noalloc_max_elements() // cols + 1
        with pytest.raises(CmfCudaError) as e:
            gpu.matmat_device_noalloc(m, idx, dx.data_ptr(), too_many, dy.data_ptr())
        assert e.value.code == -3 and "scratch" in str(e.value)


def test_noalloc_needs_a_resident_tensor(tmp_path):
    import torch
    from cmf_b200 import CmfCudaError, Model, gpu
    rng = np.random.default_rng(2)
    w = (rng.standard_normal((128, 64)) * 0.02).astype(np.float32)
    path = str(tmp_path / "w.cmf")
    single_weight_file(path, [("w", oc.Q8_ROW, w)])
    gpu.set_current_device(0)
    with Model(path) as m:
        dx = torch.zeros((4, 64), device="cuda")
        dy = torch.zeros((4, 128), device="cuda")
        with pytest.raises(CmfCudaError) as e:
            gpu.matmat_device_noalloc(m, m.index("w"), dx.data_ptr(), 4, dy.data_ptr())
        assert e.value.code == -9
