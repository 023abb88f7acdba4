"""The allocation-free linear entry (cmfc_matmat_device_noalloc) against the regular entry and the
CPU oracle.

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
    q = single_weight_file(path, [("w", dt, w)])["w"]
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
            free_before = torch.cuda.mem_get_info()[0]
            gpu.matmat_device_noalloc(m, idx, dx.data_ptr(), b, dy.data_ptr())
            free_after = torch.cuda.mem_get_info()[0]
            if call > 0:
                # the property the entry exists for: no device memory is taken or returned by the call
                # (the first call on a device may load the library's module image; later ones may not)
                assert free_after == free_before, (free_before, free_after)
            got = dy.cpu().numpy()
            assert np.isfinite(got).all()
            assert rel_l2(got, want) < 1e-6, (call, rel_l2(got, want))   # same kernels, same operands
            # and against the strict CPU kernel of the oracle, on bf16-rounded activations as the device sees them
            exact = oc.matmat_exact(dt, q.payload, rows, cols, oc.bf16_round(x))
            assert rel_l2(got, exact) < (2e-5 if dt == oc.Q8_ROW else 4e-3), rel_l2(got, exact)
        # beyond the fixed scratch: rejected with a clear status, nothing launched
        too_many = gpu.noalloc_max_elements() // cols + 1
        with pytest.raises(CmfCudaError) as e:
            gpu.matmat_device_noalloc(m, idx, dx.data_ptr(), too_many, dy.data_ptr())
        assert e.value.code == -3 and "scratch" in str(e.value)


def test_noalloc_input_ordered_by_an_event_not_a_device_sync(tmp_path):
    """The entry runs on the library's own stream, which is ordered after nothing else: a caller
    that fills d_x on another stream makes the library's stream wait on an event it recorded there
    (cmfc_stream_handle), instead of synchronizing the device."""
    import torch
    from cmf_b200 import Model, gpu
    rows, cols, b = 256, 2304, 1500
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    path = str(tmp_path / "w.cmf")
    q = single_weight_file(path, [("w", oc.Q8_ROW, w)])["w"]
    gpu.set_current_device(0)
    x = rng.standard_normal((b, cols)).astype(np.float32)
    with Model(path) as m:
        idx = m.index("w")
        warm = np.empty((4, rows), np.float32)
        gpu.q8_matmat(m, idx, None, x[:4], 4, rows, cols, warm)           # makes the tensor resident
        lib_stream = torch.cuda.ExternalStream(gpu.stream_handle(), device=torch.device("cuda", 0))
        producer = torch.cuda.Stream()
        hx = torch.from_numpy(x).pin_memory()
        dx = torch.empty((b, cols), device="cuda", dtype=torch.float32)
        dy = torch.full((b, rows), float("nan"), device="cuda", dtype=torch.float32)
        junk = torch.empty((64, 1024, 1024), device="cuda")
        torch.cuda.synchronize()
        with torch.cuda.stream(producer):
            for _ in range(20):
                junk.normal_()                      # keeps the producer stream busy before the copy
            dx.copy_(hx, non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(producer)
        lib_stream.wait_event(ready)                # no device-wide synchronize
        gpu.matmat_device_noalloc(m, idx, dx.data_ptr(), b, dy.data_ptr())
        got = dy.cpu().numpy()
    exact = oc.matmat_exact(oc.Q8_ROW, q.payload, rows, cols, oc.bf16_round(x))
    assert rel_l2(got, exact) < 2e-5, rel_l2(got, exact)


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
