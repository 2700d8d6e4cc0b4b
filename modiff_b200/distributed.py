"""Data-parallel sampling over the image batch: one process per GPU, every rank samples its
own shard with its own noise seed, and a single all-gather at the end assembles the samples.
The reference is single-process (its only multi-GPU switch raises NotImplementedError,
qdiff/layer_recon.py:102-105); images are independent given their x_T, so nothing is
exchanged inside the sampling loop.

Per-tensor dynamic activation scales couple the images of one shard (the scale is the maximum
over the whole batch tensor, qdiff/quant_layer.py:197-206), so a rank's samples equal a
single-process run on exactly that shard, not a slice of one big batch.
"""
import datetime
import os

import torch
import torch.distributed as dist

from ._lib import ModiffError


def env_world():
    """(rank, local_rank, world_size) from the torchrun environment (1 process -> 0, 0, 1)."""
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


def init(backend=None):
    """Initialise the default process group when launched by torchrun; no-op otherwise."""
    rank, local_rank, world = env_world()
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kw)
    return rank, local_rank, world


def shard_bounds(total, rank, world):
    """Contiguous shard [lo, hi) of `total` images for `rank`; the first `total % world` ranks
    hold one image more."""
    base, rem = divmod(total, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def rank_seed(base_seed, rank):
    """Noise seed of a rank's shard (rank r uses base + r)."""
    return int(base_seed) + int(rank)


def shard_noise(shape, base_seed, rank, device):
    """x_T ~ N(0, 1) of one shard, drawn on the host from the rank's seed so that a
    single-process run can re-create any shard exactly."""
    g = torch.Generator().manual_seed(rank_seed(base_seed, rank))
    return torch.randn(shape, generator=g).to(device)


def gather_samples(local, group=None):
    """All-gather equal-sized shards along dim 0 in rank order (one collective)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local
    world = dist.get_world_size(group)
    local = local.contiguous()
    out = torch.empty((world * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype,
                      device=local.device)
    dist.all_gather_into_tensor(out, local, group=group)
    return out


def gather_ragged(local, total, group=None):
    """All-gather shards produced by `shard_bounds` (sizes may differ by one): pads to the
    largest shard, gathers once, and drops the padding."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local
    world = dist.get_world_size(group)
    sizes = [shard_bounds(total, r, world) for r in range(world)]
    biggest = max(hi - lo for lo, hi in sizes)
    pad = biggest - local.shape[0]
    if pad:
        local = torch.cat([local, local.new_zeros((pad,) + tuple(local.shape[1:]))], dim=0)
    full = gather_samples(local, group).view((world, biggest) + tuple(local.shape[1:]))
    return torch.cat([full[r, :hi - lo] for r, (lo, hi) in enumerate(sizes)], dim=0)


def await_peers(tag, timeout_s=30.0, group=None):
    """Host-side check, between sampling passes, that every rank has reached the gather named
    `tag`: each rank posts a key in the process group's store and waits for the others' keys.
    A rank that raised, exited or never arrived makes the wait run out, and the survivors get a
    `ModiffError` naming the missing ranks before they launch a collective that could not
    complete.  Nothing runs on the device here, so no kernel or collective is in flight when a
    rank is found missing.  The reference has no counterpart (single process,
    qdiff/layer_recon.py:102-105)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    store = dist.distributed_c10d._get_default_store()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    store.set(f"modiff/{tag}/{rank}", b"1")
    missing = []
    deadline = datetime.timedelta(seconds=float(timeout_s))
    for r in range(world):
        if r == rank:
            continue
        try:
            store.wait([f"modiff/{tag}/{r}"], deadline)
        except Exception:       # the store raises its own timeout type
            missing.append(r)
    if missing:
        raise ModiffError(f"rank(s) {missing} did not reach '{tag}' within {timeout_s:.0f} s: "
                          "not gathering (their shards are lost; restart the pass)")


def gather_samples_checked(local, tag, timeout_s=30.0, group=None):
    """`gather_samples` behind `await_peers`: raises instead of blocking when a rank is gone."""
    await_peers(tag, timeout_s, group)
    return gather_samples(local, group)
