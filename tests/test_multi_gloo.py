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


def _mismatch_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from heron_b200.multi import ShardMismatch, gather_output
        # rank 1 was handed a wrong total (5 units instead of 6)
        full = torch.zeros((6 if rank == 0 else 5, 4), dtype=torch.int32)
        try:
            gather_output(full, rank, world, check=True)
            q.put((rank, "no error"))
        except ShardMismatch:
            q.put((rank, "mismatch"))
    finally:
        dist.destroy_process_group()


def test_wrong_shard_size_is_caught_on_the_host():
    """Failure injection on the host: a rank with a wrong extent is reported by every rank before
    any data moves."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + 77) % 2000
    procs = [ctx.Process(target=_mismatch_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert results == [(0, "mismatch"), (1, "mismatch")]


def _absent_worker(rank, world, port, q):
    import datetime
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        q.put((rank, "left"))  # leaves between steps, nothing in flight
        return
    from heron_b200.multi import gather_output
    full = torch.zeros((6, 4), dtype=torch.int32)
    try:
        gather_output(full, rank, world)
        q.put((rank, "no error"))
    except Exception as exc:  # the short process-group timeout ends the collective with an error
        q.put((rank, "error:" + type(exc).__name__))


def test_rank_that_leaves_ends_the_collective_with_an_error():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + 191) % 2000
    procs = [ctx.Process(target=_absent_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    assert results[1] == "left"
    assert results[0].startswith("error:")


def _chunked_worker(rank, world, port, extent, chunks, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from heron_b200.multi import ChunkedGather
        from oracle import np_oracle as npo
        rng = np.random.default_rng(321)
        a = rng.integers(-128, 128, (extent, 16, 32)).astype(np.int8)
        b = rng.integers(-128, 128, (extent, 8, 32)).astype(np.int8)
        full = torch.full((extent, 16, 8), -1, dtype=torch.int32)
        cg = ChunkedGather(extent, rank, world, chunks)

        def kernel_for(start, count):
            def run():  # the oracle stands in for the kernel bound to this slice of `full`
                if count:
                    full[start:start + count].copy_(torch.from_numpy(npo.bmm_int(a[start:start + count],
                                                                                 b[start:start + count])))
            return run

        cg.run([kernel_for(s, n) for (s, n) in cg.parts], full)
        q.put((rank, bool(torch.equal(full, torch.from_numpy(npo.bmm_int(a, b)))), len(cg.parts)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("extent,chunks", [(8, 2), (12, 3), (7, 2), (9, 4), (3, 4)])
def test_two_rank_chunked_gather(extent, chunks):
    """The overlapped form: the leading dimension cut into super-chunks, each split over the ranks
    and gathered by itself (equal and ragged splits; more chunks than units)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + 300 + 10 * extent + chunks) % 2000
    procs = [ctx.Process(target=_chunked_worker, args=(r, 2, port, extent, chunks, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[:2] for r in results) == [(0, True), (1, True)]


def test_chunked_partition_covers_the_extent_once():
    sys.path.insert(0, ROOT)
    from heron_b200.multi import partition_chunked
    for extent, world, chunks in [(1024, 8, 4), (192, 8, 2), (10, 4, 3), (5, 8, 2), (1, 2, 1)]:
        seen = []
        for r in range(world):
            mine, supers = partition_chunked(extent, r, world, chunks)
            assert len(mine) == len(supers)
            for (s, n), (c0, cn) in zip(mine, supers):
                assert c0 <= s and s + n <= c0 + cn
                seen.extend(range(s, s + n))
        assert sorted(seen) == list(range(extent))
