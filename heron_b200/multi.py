"""multi.py — two things under the reference's module name.

1. ``Job``: the reference's helper that runs a function in a forked child with a timeout and
   kills the child's process tree afterwards (multi.py:11-49); the tuners use it for sampling.
2. The batch-parallel partitioner that the B200 build adds: batched GEMM shards its batch and
   NHWC conv shards its images over the GPUs of one box, one process per GPU.  Shards are
   independent (no exchange during compute); where a caller wants the whole output, every rank's
   kernel writes its shard straight into its slice of a full-size buffer and one in-place
   all-gather over that buffer (NCCL over NVLink, or gloo on CPU ranks) completes it.
"""
import multiprocessing as _multi
import signal

multi = _multi.get_context("fork")


class Job:
    def __init__(self, func, attach_info, timeout=10):
        self.func = func
        self.attach_info = attach_info
        self.timeout = timeout

    def start(self, inputs):
        self.queue = multi.Queue(2)
        self.process = multi.Process(target=exec, args=(self.func, self.queue, inputs))
        self.process.start()

    def get(self):
        try:
            res = self.queue.get(block=True, timeout=self.timeout)
        except Exception:
            res = 0
        if self.process.is_alive():
            kill_child_processes(self.process.pid)
            self.process.terminate()
        self.process.join()
        self.queue.close()
        self.queue.join_thread()
        del self.process
        del self.queue
        return res


def exec(func, queue, args):
    queue.put(func(*args))


def kill_child_processes(parent_pid, sig=signal.SIGTERM):
    import psutil
    try:
        parent = psutil.Process(parent_pid)
    except psutil.NoSuchProcess:
        return
    for process in parent.children(recursive=True):
        try:
            process.send_signal(sig)
        except psutil.NoSuchProcess:
            return


# ---- batch-parallel partitioning --------------------------------------------------------------

# Position of the sharded leading dimension in each operator's case arguments
# (gemm [M,K,N] does not shard; bmm [batch,M,K,N]; conv [N,H,W,CI,CO,KH,KW,stride,pad,dil,...]).
# The image-parallel operators next to them (dil, c1d, c3d, t2d) lead with N as well.
SHARD_ARG = {"bmm": 0, "c2d_nhwc": 0, "c2d": 0, "dil": 0, "c1d": 0, "c3d": 0, "t2d": 0}


def partition(extent, world):
    """Contiguous split of ``extent`` units over ``world`` ranks: [(start, count)] per rank.
    The first ``extent % world`` ranks get one extra unit."""
    if world <= 0 or extent < 0:
        raise ValueError("need world > 0 and extent >= 0")
    base, extra = divmod(extent, world)
    out, start = [], 0
    for r in range(world):
        cnt = base + (1 if r < extra else 0)
        out.append((start, cnt))
        start += cnt
    return out


def shard_case(op_name, case_args, rank, world):
    """Case arguments of rank ``rank``'s shard, plus (start, count) of its units."""
    if op_name not in SHARD_ARG:
        raise ValueError("operator %r has no batch-like dimension to shard: run replicas" % op_name)
    pos = SHARD_ARG[op_name]
    start, count = partition(int(case_args[pos]), world)[rank]
    args = list(case_args)
    args[pos] = count
    return args, (start, count)


def shard_slice(full, rank, world):
    """View of rank ``rank``'s slice of a tensor whose leading dimension is the sharded one."""
    start, count = partition(full.shape[0], world)[rank]
    return full[start:start + count]


class ShardMismatch(RuntimeError):
    """Ranks disagree on the extent or layout of the tensor they are about to gather."""


def check_same_extent(full, world, group=None):
    """Host-side guard (one small all-reduce): every rank must hold a full buffer of the same
    shape, otherwise the in-place gather would write past a smaller rank's slices."""
    import torch
    import torch.distributed as dist
    dims = list(full.shape) + [0] * (8 - full.dim())
    lo = torch.tensor(dims, dtype=torch.int64, device=full.device)
    hi = lo.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
    if not torch.equal(lo, hi):
        raise ShardMismatch("ranks hold full buffers of different shapes: min %s max %s"
                            % (lo.tolist()[:full.dim()], hi.tolist()[:full.dim()]))


def gather_output(full, rank, world, group=None, check=False):
    """Completes ``full`` on every rank: each rank has already written its own slice.

    Equal shards use one in-place ``all_gather_into_tensor``; ragged shards (extent not a
    multiple of world) fall back to one broadcast per rank.  No copy precedes the collective.
    """
    import torch.distributed as dist
    if world == 1:
        return full
    if check:
        check_same_extent(full, world, group)
    parts = partition(full.shape[0], world)
    if len({c for _, c in parts}) == 1:
        dist.all_gather_into_tensor(full, shard_slice(full, rank, world), group=group)
    else:
        for r, (start, count) in enumerate(parts):
            if count:
                dist.broadcast(full[start:start + count], src=r, group=group)
    return full


def partition_chunked(extent, rank, world, chunks):
    """This rank's slices when the leading dimension is first cut into ``chunks`` super-chunks and
    every super-chunk is split over the ranks: [(start, count)] per super-chunk, plus the
    super-chunks' own (start, count).  With ``chunks == 1`` this is ``partition``.  Each
    super-chunk is a contiguous range whose rank slices lie in rank order, so it can be completed
    by one in-place all-gather while the kernels of the next super-chunk run."""
    if chunks <= 0:
        raise ValueError("need chunks > 0")
    supers = [sc for sc in partition(extent, chunks) if sc[1] > 0]
    mine = []
    for (c0, cn) in supers:
        s, n = partition(cn, world)[rank]
        mine.append((c0 + s, n))
    return mine, supers


class ChunkedGather:
    """Compute + gather of a sharded operator's whole output with the two overlapped.

    ``parts`` lists this rank's (start, count) slices of the leading dimension, one per
    super-chunk.  ``run(plans, full)`` launches ``plans[c]`` (a kernel bound to
    ``full[start:start+count]`` of slice c) on the current stream and, on a second stream, gathers
    super-chunk c - 1 in place while it runs; when it returns, the current stream waits for the
    last gather.  No kernel of this library is handed another GPU's memory: the exchange is the
    collective library's (NCCL over NVLink on GPUs, gloo on CPU ranks)."""

    def __init__(self, extent, rank, world, chunks=1, group=None):
        self.rank, self.world, self.group = rank, world, group
        self.parts, self.supers = partition_chunked(extent, rank, world, chunks)
        self._comm = None

    def _comm_stream(self, device):
        import torch
        if self._comm is None:
            self._comm = torch.cuda.Stream(device=device)
        return self._comm

    def gather_super(self, full, c):
        c0, cn = self.supers[c]
        gather_output(full[c0:c0 + cn], self.rank, self.world, group=self.group)

    def run(self, plans, full):
        if len(plans) != len(self.parts):
            raise ValueError("one plan per super-chunk")
        if not full.is_cuda:
            for c, plan in enumerate(plans):  # CPU ranks (tests): no streams to overlap
                plan()
                self.gather_super(full, c)
            return full
        import torch
        cur = torch.cuda.current_stream(full.device)
        comm = self._comm_stream(full.device)
        comm.wait_stream(cur)  # earlier users of `full` on the compute stream
        for c, plan in enumerate(plans):
            plan.launch()
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(comm):
                comm.wait_event(done)
                self.gather_super(full, c)
        cur.wait_stream(comm)
        return full


class PeerStoreOutput:
    """The whole output of a sharded operator on every GPU of one box with no collective at all:
    each rank's kernel stores its tiles into its slice of EVERY rank's output buffer (TMA stores
    from the kernel's staging buffer, over NVLink for the other GPUs), so the transfer rides on
    the kernel's own epilogue.

    The buffer is symmetric memory (torch.distributed._symmetric_memory: the same allocation on
    every rank, each rank's copy mapped into all processes).  ``attach(plan, start, count)`` hands
    the plan this rank's slice of the other ranks' buffers (`hb_plan_set_peer_outputs`); the plan
    itself must have been built on ``mine(start, count)``.  After every rank's launch,
    ``barrier()`` says on the current stream that all slices have arrived: a one-element all-reduce
    of the collective library, ordered behind this rank's kernel, which completes only when every
    rank's kernel (and with it its stores into this rank's buffer) has.  A rank that never arrives
    ends that collective through the process group's timeout with an error on the host; the
    symmetric-memory library's own device-side barrier would spin on the GPU instead.
    Only plain stores cross NVLink; nothing in the kernel waits on another GPU.  NVLink multicast
    is switched off for the allocation (a rank that dies while its memory is bound to a multicast
    object disturbs the other GPUs of the box)."""

    def __init__(self, shape, dtype, device, group=None):
        import os
        import torch.distributed as dist
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.shape, self.dtype = tuple(shape), dtype
        self.full = symm_mem.empty(*self.shape, dtype=dtype, device=device)
        self._hdl = symm_mem.rendezvous(self.full, self.group)
        self._peers = [self._hdl.get_buffer(r, self.shape, dtype) for r in range(self.world) if r != self.rank]
        import torch
        self._token = torch.zeros(1, dtype=torch.int32, device=device)

    def mine(self, start, count):
        return self.full[start:start + count]

    def attach(self, plan, start, count):
        plan.set_peer_outputs([p[start:start + count] for p in self._peers])
        return plan

    def barrier(self):
        import torch.distributed as dist
        dist.all_reduce(self._token, group=self.group)
