"""Host-buffer execution of a built kernel: the call a user of the reference makes when tensors
live in host memory (numpy -> device array -> built function -> ``asnumpy``,
tests/quick_start/dlboost/run.py:52-62), as a three-stage pipeline.

Each step copies that step's inputs from pinned host memory to the device, launches the kernel
and copies the output back to pinned host memory.  With ``depth`` buffer sets the three stages
of consecutive steps overlap on three streams (upload, compute, download), so the sustained rate
is that of the slowest stage; the copies still happen for every step.
"""
import numpy as np


class HostPipeline:
    def __init__(self, handle, args, depth=2, device_id=0, resident=()):
        """``resident``: indices of inputs that are uploaded once and reused by every step (the
        filter of a conv); all other inputs are uploaded per step."""
        import torch
        from ..kernels import TORCH_DTYPES
        self.torch = torch
        self.device = torch.device("cuda", device_id)
        self.args = args
        self.depth = depth
        self.resident = tuple(resident)
        self.n_in = len(args) - 1
        with torch.cuda.device(self.device):
            self.s_up, self.s_run, self.s_down = (torch.cuda.Stream() for _ in range(3))
            self.dev = [[torch.empty(a.shape, dtype=TORCH_DTYPES[a.dtype], device=self.device) for a in args]
                        for _ in range(depth)]
            for d in self.dev[1:]:
                for i in self.resident:
                    d[i] = self.dev[0][i]
            self.host_out = [torch.empty(args[-1].shape, dtype=TORCH_DTYPES[args[-1].dtype]).pin_memory()
                             for _ in range(depth)]
            self.plans = [handle.plan(*d) for d in self.dev]
            self.up_done = [torch.cuda.Event() for _ in range(depth)]
            self.run_done = [torch.cuda.Event() for _ in range(depth)]
            self.down_done = [torch.cuda.Event() for _ in range(depth)]
        self.h2d_bytes_per_step = sum(int(np.prod(a.shape)) * self.dev[0][i].element_size()
                                      for i, a in enumerate(args[:-1]) if i not in self.resident)
        self.d2h_bytes_per_step = int(np.prod(args[-1].shape)) * self.dev[0][-1].element_size()
        self._step = 0

    def upload_resident(self, host_inputs):
        for i in self.resident:
            self.dev[0][i].copy_(host_inputs[i], non_blocking=False)

    def submit(self, host_inputs):
        """Enqueues one step on pinned host inputs; returns the slot whose ``host_out`` will hold
        the result after ``wait(slot)``."""
        torch = self.torch
        slot = self._step % self.depth
        self._step += 1
        with torch.cuda.stream(self.s_up):
            # the previous user of this slot must have finished computing before inputs change
            self.s_up.wait_event(self.run_done[slot])
            for i in range(self.n_in):
                if i not in self.resident:
                    self.dev[slot][i].copy_(host_inputs[i], non_blocking=True)
            self.up_done[slot].record(self.s_up)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.up_done[slot])
            self.s_run.wait_event(self.down_done[slot])  # output buffer of this slot drained
            self.plans[slot].launch(self.s_run.cuda_stream)
            self.run_done[slot].record(self.s_run)
        with torch.cuda.stream(self.s_down):
            self.s_down.wait_event(self.run_done[slot])
            self.host_out[slot].copy_(self.dev[slot][-1], non_blocking=True)
            self.down_done[slot].record(self.s_down)
        return slot

    def wait(self, slot):
        self.down_done[slot].synchronize()
        return self.host_out[slot]

    def drain(self):
        for s in (self.s_up, self.s_run, self.s_down):
            s.synchronize()
