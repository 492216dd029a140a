"""Body of the multi-GPU check, one process per GPU (launched by tests/test_gpu_multi.py under
torch.distributed.run).  Each rank computes its shard of a batched GEMM and of an NHWC conv with
the sm_100a kernels, writing straight into its slice of a full-size output buffer; one in-place
NCCL all-gather completes the buffer; every rank compares the whole result with the oracle.  Then
the form without a collective: each rank's kernel stores its shard into every rank's buffer."""
import os
import sys

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # (before torch is imported)

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from heron_b200 import _lib, kernels as K
    from heron_b200.multi import gather_output, partition, shard_case, shard_slice
    from oracle import np_oracle as npo

    rng = np.random.default_rng(4242)  # same stream on every rank
    ok = True

    # batched GEMM, batch 12 (equal shards) and 7 (ragged shards over 2 ranks)
    for batch in (12, 7):
        a = rng.integers(-128, 128, (batch, 192, 64)).astype(np.int8)
        b = rng.integers(-128, 128, (batch, 160, 64)).astype(np.int8)
        args, (start, count) = shard_case("bmm", [batch, 192, 64, 160], rank, world)
        full = torch.full((batch, 192, 160), -1, dtype=torch.int32, device=dev)
        mine = shard_slice(full, rank, world)
        assert mine.shape[0] == count == args[0]
        if count:
            K.bmm(torch.from_numpy(a[start:start + count]).to(dev), torch.from_numpy(b[start:start + count]).to(dev),
                  out=mine)
        gather_output(full, rank, world)
        ok &= bool(np.array_equal(full.cpu().numpy(), npo.bmm_int(a, b)))

    # NHWC conv, 16 images
    x = rng.integers(0, 256, (16, 7, 7, 64), dtype=np.uint8)
    w = rng.integers(-128, 128, (3, 3, 64, 128)).astype(np.int8)
    start, count = partition(16, world)[rank]
    full = torch.full((16, 7, 7, 128), -1, dtype=torch.int32, device=dev)
    K.conv2d_nhwc(torch.from_numpy(x[start:start + count]).to(dev), torch.from_numpy(w).to(dev), 1, 1, 1,
                  out=shard_slice(full, rank, world))
    gather_output(full, rank, world)
    ok &= bool(np.array_equal(full.cpu().numpy(), npo.conv2d_nhwc_int(x, w, 1, 1, 1)))

    # the overlapped form: two super-chunks, the gather of the first behind the kernel of the second
    from heron_b200.multi import ChunkedGather
    for chunks in (2, 3):
        cg = ChunkedGather(16, rank, world, chunks)
        full = torch.full((16, 7, 7, 128), -1, dtype=torch.int32, device=dev)
        wd = torch.from_numpy(w).to(dev)
        plans = [K.plan_conv2d_nhwc(torch.from_numpy(x[s:s + n]).to(dev), wd, 1, 1, 1, out=full[s:s + n])
                 for (s, n) in cg.parts if n]
        if len(plans) == len(cg.parts):
            cg.run(plans, full)
            torch.cuda.synchronize(dev)
            ok &= bool(np.array_equal(full.cpu().numpy(), npo.conv2d_nhwc_int(x, w, 1, 1, 1)))

    # no collective at all: every rank's kernel stores its shard into every rank's buffer
    from heron_b200.multi import PeerStoreOutput
    for batch in (12, 7):
        a = rng.integers(-128, 128, (batch, 192, 64)).astype(np.int8)
        b = rng.integers(-128, 128, (batch, 160, 64)).astype(np.int8)
        start, count = partition(batch, world)[rank]
        po = PeerStoreOutput((batch, 192, 160), torch.int32, dev)
        po.full.fill_(-1)
        po.barrier()
        if count:
            plan = K.plan_bmm(torch.from_numpy(a[start:start + count]).to(dev),
                              torch.from_numpy(b[start:start + count]).to(dev), out=po.mine(start, count))
            po.attach(plan, start, count)
            plan.launch()
            plan.launch()  # (a second launch stores the same bits again)
        po.barrier()
        torch.cuda.synchronize(dev)
        ok &= bool(np.array_equal(po.full.cpu().numpy(), npo.bmm_int(a, b)))
        po.barrier()
    start, count = partition(16, world)[rank]
    po = PeerStoreOutput((16, 7, 7, 128), torch.int32, dev)
    po.full.fill_(-1)
    po.barrier()
    plan = K.plan_conv2d_nhwc(torch.from_numpy(x[start:start + count]).to(dev), torch.from_numpy(w).to(dev), 1, 1, 1,
                              out=po.mine(start, count), knobs=dict(conv_algo=1))
    po.attach(plan, start, count)
    plan.launch()
    po.barrier()
    torch.cuda.synchronize(dev)
    ok &= bool(np.array_equal(po.full.cpu().numpy(), npo.conv2d_nhwc_int(x, w, 1, 1, 1)))
    po.barrier()
    # (the strip kernels and the direct-store epilogue have no such outputs: refused, not ignored)
    try:
        K.plan_conv2d_nhwc(torch.from_numpy(x[start:start + count]).to(dev), torch.from_numpy(w).to(dev), 1, 1, 1,
                           out=po.mine(start, count), knobs=dict(conv_algo=1, epilogue=2)).set_peer_outputs(
                               [po.mine(start, count)])
        ok = False
    except _lib.HeronB200Error as e:
        ok &= e.status == _lib.HB_ERR_KNOB

    ok &= _lib.last_status() == 0
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    if rank == 0:
        print("MULTI_RANK_CHECK", "PASS" if int(flag) == 1 else "FAIL", "world", world)
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
