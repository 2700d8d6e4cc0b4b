"""World-size-2 gloo test (CPU) of the data-parallel plumbing: shard bounds, per-rank seeds and
the order / raggedness of the final all-gather."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, out_dir):
    sys.path.insert(0, ROOT)
    from modiff_b200 import distributed as D
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    r, lr, w = D.init(backend="gloo")
    assert (r, w) == (rank, world)
    # equal shards: every rank draws its shard from its own seed
    local = D.shard_noise((4, 3, 8, 8), base_seed=7, rank=rank, device="cpu")
    full = D.gather_samples(local)
    # ragged shards of `total` images
    lo, hi = D.shard_bounds(total, rank, world)
    ragged = torch.arange(lo, hi, dtype=torch.float32).view(-1, 1).repeat(1, 3)
    full_ragged = D.gather_ragged(ragged, total)
    torch.save((full, full_ragged), os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gather(tmp_path):
    world, total = 2, 7
    port = _free_port()
    mp.spawn(_worker, args=(world, port, total, str(tmp_path)), nprocs=world, join=True)
    from modiff_b200 import distributed as D
    expect = torch.cat([D.shard_noise((4, 3, 8, 8), 7, r, "cpu") for r in range(world)], dim=0)
    for r in range(world):
        full, ragged = torch.load(os.path.join(tmp_path, f"r{r}.pt"))
        assert torch.equal(full, expect)                     # rank order, bit-identical shards
        assert torch.equal(ragged[:, 0], torch.arange(total, dtype=torch.float32))


def test_shard_bounds_cover_the_batch():
    from modiff_b200 import distributed as D
    for total in (1, 7, 8, 2048, 2050):
        for world in (1, 2, 4, 8):
            spans = [D.shard_bounds(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    assert D.rank_seed(1, 3) == 4
    assert D.env_world() == (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
                             int(os.environ.get("WORLD_SIZE", 1)))


def _leaver(rank, world, port, out_dir):
    """Rank 1 finishes the first pass and leaves (between passes, nothing in flight); rank 0
    goes on to a second pass and must learn on the host that its peer is gone."""
    sys.path.insert(0, ROOT)
    import time
    from modiff_b200 import distributed as D
    from modiff_b200._lib import ModiffError
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    D.init(backend="gloo")
    local = D.shard_noise((2, 3, 4, 4), base_seed=3, rank=rank, device="cpu")
    first = D.gather_samples_checked(local, "pass0", timeout_s=20.0)
    assert first.shape[0] == 2 * world
    if rank == 1:
        os._exit(0)                       # leaves without a word
    t0 = time.time()
    try:
        D.gather_samples_checked(local, "pass1", timeout_s=2.0)
        outcome = "gathered"
    except ModiffError as e:
        outcome = f"raised after {time.time() - t0:.1f}s: {e}"
    with open(os.path.join(out_dir, "r0.txt"), "w") as fh:
        fh.write(outcome)
    os._exit(0)                           # no collective teardown with a dead peer


def test_rank_leaving_between_passes_is_detected_on_the_host(tmp_path):
    """Failure detection without touching a device: a rank that exits between two sampling
    passes makes the survivor's next gather raise within its timeout instead of blocking."""
    world = 2
    port = _free_port()
    ctx = mp.spawn(_leaver, args=(world, port, str(tmp_path)), nprocs=world, join=False)
    ok = ctx.join(timeout=90)
    while not ok:
        ok = ctx.join(timeout=90)
    text = open(os.path.join(tmp_path, "r0.txt")).read()
    assert text.startswith("raised after"), text
    assert "rank(s) [1]" in text and "pass1" in text
    assert float(text.split()[2][:-2]) < 15.0
