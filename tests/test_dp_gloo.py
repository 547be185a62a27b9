"""World-size-2 gloo test of the data-parallel host logic (no GPU)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from spion_b200 import dp
    assert dp.world_size() == 1                                   # before the group exists
    r, w = dp.init_from_env("gloo", timeout_s=60)
    assert (r, w) == (rank, world) and dp.world_size() == world
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 3))
    bucket = dp.FlatGradBucket(model.parameters())
    g = torch.Generator().manual_seed(1)
    X = torch.randn(8, 8, generator=g); y = torch.randint(0, 3, (8,), generator=g)
    lo, hi = dp.shard_range(8, rank, world)
    bucket.zero()
    torch.nn.functional.cross_entropy(model(X[lo:hi]), y[lo:hi]).backward()
    bucket.allreduce_mean()
    # mask agreement: rank 0 decides, everyone receives
    local = [torch.full((4, 4), float(rank + 1))]
    masks = dp.agree_on_masks(local, lambda A: (A > 0.5).to(torch.uint8) * (torch.eye(4, dtype=torch.uint8) + 0))
    avg = dp.average_map(torch.full((2, 2), float(rank)))
    if rank == 0:
        torch.save({"flat": bucket.flat.clone(), "mask": masks[0], "avg": avg}, out)
    else:
        torch.save({"mask": masks[0]}, out + ".1")
    dist.barrier()
    dist.destroy_process_group()


def test_flat_bucket_allreduce_and_mask_broadcast(tmp_path):
    out = str(tmp_path / "r0.pt")
    port = 29000 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    got = torch.load(out)
    other = torch.load(out + ".1")
    # single-process full-batch gradient == mean of the two shard gradients
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 3))
    g = torch.Generator().manual_seed(1)
    X = torch.randn(8, 8, generator=g); y = torch.randint(0, 3, (8,), generator=g)
    torch.nn.functional.cross_entropy(model(X), y).backward()
    want = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
    torch.testing.assert_close(got["flat"], want, rtol=1e-5, atol=1e-6)
    assert torch.equal(got["mask"], other["mask"]) and torch.equal(got["mask"], torch.eye(4, dtype=torch.uint8))
    assert torch.allclose(got["avg"], torch.full((2, 2), 0.5))


def test_shard_range_rejects_uneven():
    from spion_b200 import dp
    assert dp.shard_range(64, 3, 8) == (24, 32)
    with pytest.raises(ValueError):
        dp.shard_range(10, 0, 4)
