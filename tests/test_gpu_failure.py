"""Failure path of the bounded device waits, without a GPU fault: a kernel waits on a barrier that
nobody arrives on, runs out of its (small) poll budget, records the site and exits normally; the
host reports CMFC_ERR_DEVICE_WAIT and the same context then computes correctly."""
import numpy as np
import pytest

from oracle import codecs as oc
from tests.modelfile import rel_l2, single_weight_file

pytestmark = pytest.mark.gpu


def test_a_bounded_wait_runs_out_and_the_context_stays_usable(tmp_path):
    from cmf_b200 import CmfCudaError, Model, gpu
    gpu.set_current_device(0)
    rows, cols, b = 256, 512, 300
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    x = oc.bf16_round(rng.standard_normal((b, cols)).astype(np.float32))
    path = str(tmp_path / "w.cmf")
    q = single_weight_file(path, [("w", oc.Q4_TILED, w)])["w"]
    want = oc.matmat_exact(oc.Q4_TILED, q.payload, rows, cols, x)
    with Model(path) as m:
        out = np.empty((b, rows), np.float32)
        gpu.q4t_matmat(m, m.index("w"), x, b, rows, cols, out)
        assert rel_l2(out, want) < 4e-3
        for polls in (64, 2048):
            with pytest.raises(CmfCudaError) as e:
                gpu.selftest_wait_timeout(polls)
            assert e.value.code == -5 and "bounded wait" in str(e.value)
        gpu.synchronize()                        # the status word was cleared: no stale error
        out2 = np.empty((b, rows), np.float32)
        gpu.q4t_matmat(m, m.index("w"), x, b, rows, cols, out2)
        assert np.array_equal(out, out2)
    with pytest.raises(CmfCudaError) as e:
        gpu.selftest_wait_timeout(0)
    assert e.value.code == -1
