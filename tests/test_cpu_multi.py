"""world_size-2 gloo tests of the multi-GPU host logic (sharding, final gather, a rank that
never arrives).  The per-rank "denoiser" is the CPU oracle on the tiny config, so the test
checks that sharded + gathered results equal the single-process result."""
import multiprocessing as mp
import socket

import numpy as np
import pytest

from cmf_b200.shard import shard_range


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _inputs(n_prompts):
    from oracle import nextdit as nd
    rng = np.random.default_rng(3)
    lat = np.stack([nd.gauss_latent(16 * 8 * 8, s).reshape(16, 8, 8) for s in range(n_prompts)])
    cap = rng.standard_normal((n_prompts, 6, 256)).astype(np.float32)
    cap_u = rng.standard_normal((n_prompts, 3, 256)).astype(np.float32)
    return lat, cap, cap_u


def _denoise_shard(lo, hi):
    from oracle import nextdit as nd
    from tests import synth
    cfg = dict(synth.TINY, num_layers=1, num_refiner_layers=1)
    orc = nd.NextDitOracle(synth.make_tensors(cfg, 0), cfg)
    lat, cap, cap_u = _inputs(3)
    return np.stack([nd.denoise(orc, lat[i], 8, 8, cap[i], cap_u[i], steps=2) for i in range(lo, hi)]) \
        if hi > lo else np.zeros((0, 16, 8, 8), np.float32)


def _oracle_denoise(dit, lat, cap, cap_u, params):
    """Stand-in for the device loop with the package's ``denoise`` signature: the CPU oracle."""
    from oracle import nextdit as nd
    from tests import synth
    cfg = dict(synth.TINY, num_layers=1, num_refiner_layers=1)
    orc = nd.NextDitOracle(synth.make_tensors(cfg, 0), cfg)
    return np.stack([nd.denoise(orc, lat[i], 8, 8, cap[i], cap_u[i], steps=params["steps"]) for i in range(lat.shape[0])])


def _worker(rank, world, port, q, absent, sharded=False):
    try:
        import torch.distributed as dist
        from cmf_b200.shard import denoise_sharded, gather_latents, init_cpu_group
        if rank in absent:
            return  # this rank never joins: the others must fail cleanly, not hang
        init_cpu_group(rank, world, port, timeout_s=6.0)
        if sharded:
            # the product entry: every rank passes the full batch, the shard is taken inside
            lat, cap, cap_u = _inputs(3)
            out = denoise_sharded(None, lat, cap, cap_u, {"steps": 2}, denoise_fn=_oracle_denoise)
        else:
            lo, hi = shard_range(3, world, rank)
            out = gather_latents(_denoise_shard(lo, hi), 3)
        q.put((rank, "ok", out))
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        q.put((rank, "error", repr(e)))


def _run(world, absent=(), sharded=False):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_worker, args=(r, world, port, q, absent, sharded)) for r in range(world)]
    for p in ps:
        p.start()
    res = {}
    for _ in range(world - len(absent)):
        r, status, payload = q.get(timeout=120)
        res[r] = (status, payload)
    for p in ps:
        p.join(timeout=30)
    return res


def test_shard_range_is_a_partition():
    for n in (0, 1, 7, 8, 16):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def test_two_ranks_match_single_process():
    res = _run(2)
    assert res[0][0] == "ok" and res[1][0] == "ok", res
    assert res[1][1] is None
    want = _denoise_shard(0, 3)
    assert res[0][1].shape == want.shape
    assert np.array_equal(res[0][1], want)  # same arithmetic, ragged split 2 + 1


def test_denoise_sharded_two_ranks_match_single_process():
    res = _run(2, sharded=True)
    assert res[0][0] == "ok" and res[1][0] == "ok", res
    assert res[1][1] is None
    assert np.array_equal(res[0][1], _denoise_shard(0, 3))


def test_denoise_sharded_without_a_group_is_plain_denoise():
    from cmf_b200.shard import denoise_sharded
    lat, cap, cap_u = _inputs(2)
    got = denoise_sharded(None, lat, cap, cap_u, {"steps": 1}, denoise_fn=lambda d, a, b, c, p: a * 2.0)
    assert np.array_equal(got, lat * 2.0)


def test_missing_rank_is_an_error_not_a_hang():
    res = _run(2, absent=(1,))
    assert res[0][0] == "error", res
