"""The N>1 path on CPU ranks: two gloo processes shard a batched problem, each computes its
shard (with the oracle standing in for the kernel), writes it into its slice of the full
buffer, and the in-place gather completes the output on both ranks."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, extent, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from heron_b200.multi import gather_output, partition, shard_slice
        from oracle import np_oracle as npo
        rng = np.random.default_rng(123)  # same stream on every rank: shards are slices of one tensor
        a = rng.integers(-128, 128, (extent, 16, 32)).astype(np.int8)
        b = rng.integers(-128, 128, (extent, 8, 32)).astype(np.int8)
        start, count = partition(extent, world)[rank]
        full = torch.full((extent, 16, 8), -1, dtype=torch.int32)
        mine = shard_slice(full, rank, world)
        assert mine.shape[0] == count and mine.data_ptr() == full[start:].data_ptr() if count else True
        if count:
            mine.copy_(torch.from_numpy(npo.bmm_int(a[start:start + count], b[start:start + count])))
        gather_output(full, rank, world)
        want = torch.from_numpy(npo.bmm_int(a, b))
        q.put((rank, bool(torch.equal(full, want))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("extent", [6, 5])  # equal shards (one all-gather) and ragged shards
def test_two_rank_shard_and_gather(extent):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + extent) % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, extent, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
