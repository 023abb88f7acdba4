"""Multi-GPU plumbing of the denoise path: replicas, prompts sharded, one gather at the end.

Every prompt's cond/uncond pair is an independent trajectory (segments never attend to each
other, crates/cortiq-engine/src/dit.rs:1112-1131), so ranks share nothing per step.  Each rank
memory-maps the container and uploads its own weight copy; the only exchange is the gather of
the final latents (1 MiB per 1024x1024 image) over torch.distributed (NCCL on GPUs, gloo on CPU).
"""
import datetime

import numpy as np


def shard_range(n_items, world, rank):
    """Contiguous, balanced shard [lo, hi) of n_items for `rank` of `world`; a prompt's CFG pair
    is one item, so a pair never straddles ranks."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    base, extra = divmod(n_items, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def gather_latents(local, n_total, group=None, device=None, dst=0):
    """Gather per-rank latents [n_local, c, h, w] (numpy f32) on rank `dst` in prompt order.
    Returns the full array on `dst`, None elsewhere.  Ranks may hold different counts."""
    import torch
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    shape = tuple(local.shape[1:])
    per = max(shard_range(n_total, world, r)[1] - shard_range(n_total, world, r)[0] for r in range(world))
    buf = np.zeros((per,) + shape, np.float32)
    buf[:local.shape[0]] = local
    t = torch.from_numpy(buf)
    if device is not None:
        t = t.to(device)
    out = [torch.empty_like(t) for _ in range(world)] if rank == dst else None
    dist.gather(t, out, dst=dst, group=group)
    if rank != dst:
        return None
    parts = []
    for r in range(world):
        lo, hi = shard_range(n_total, world, r)
        parts.append(out[r][:hi - lo].cpu().numpy())
    return np.concatenate(parts, 0)


def denoise_sharded(dit, latents, cap, cap_u, params, group=None, device=None, denoise_fn=None):
    """``denoise`` for a batch of prompts split over the ranks of a torch.distributed group.

    Every rank passes the SAME full host arrays (``latents`` [n, c, h, w], ``cap`` [n, cap_n, feat],
    ``cap_u`` [n, cap_u_n, feat] or None); rank r denoises prompts ``shard_range(n, world, r)`` on
    its own GPU (a prompt's cond/uncond pair never straddles ranks, so CFG combine and the Euler
    update of crates/cortiq-engine/src/imagegen.rs:186-205 stay rank-local and nothing is exchanged
    per step) and one gather brings the final latents to rank 0 in prompt order.  Returns the full
    [n, c, h, w] array on rank 0 and None on the others; without a process group (or with one
    rank) it is plain ``denoise``.  ``denoise_fn`` replaces the device loop in host-logic tests."""
    import torch.distributed as dist
    if denoise_fn is None:
        from .dit import denoise as denoise_fn
    n = latents.shape[0]
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return denoise_fn(dit, latents, cap, cap_u, params)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    lo, hi = shard_range(n, world, rank)
    if hi > lo:
        local = denoise_fn(dit, latents[lo:hi], cap[lo:hi], None if cap_u is None else cap_u[lo:hi], params)
    else:
        local = np.zeros((0,) + tuple(latents.shape[1:]), np.float32)
    return gather_latents(np.ascontiguousarray(local, np.float32), n, group=group, device=device)


def init_cpu_group(rank, world, port, timeout_s=30.0):
    """gloo process group on 127.0.0.1 (host-side tests of the sharding logic)."""
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s))
