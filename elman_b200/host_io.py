"""E1 cell forward + backward for callers whose tensors live in HOST memory.

`E1HostPipeline.submit()` takes pinned host tensors (x, z, d_output), runs the cell on
the GPU and leaves output, dx, dz, dW_x, dW_h, db in pinned host buffers.  Uploads,
kernels and downloads run on three CUDA streams over `depth` device slots (default 3), so the
upload of call i+1 and the download of call i-1 overlap the kernels of call i: with
PCIe moving about as many bytes per call as the kernels take time for, a stream of
calls runs at the speed of the slowest of the three instead of their sum.  The
arithmetic is that of hasty_pytorch_lib.mamba_gated_elman_forward / _backward
(elman/cuda/pytorch/elman_ladder.cc:161-281 in the reference); the reference has no
host-buffer entry point, its callers hold CUDA tensors.
"""
import torch

from . import hasty_pytorch_lib as H


class _Slot:
    pass


class E1HostPipeline:
    def __init__(self, T, B, d, W_x, W_h, b, h0=None, dtype=torch.bfloat16, device=None, depth=3):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None \
            else torch.device(device)
        self.T, self.B, self.d, self.dtype = T, B, d, dtype
        dev = self.device
        self.W_x = W_x.to(dev, dtype).contiguous()
        self.W_h = W_h.to(dev, dtype).contiguous()
        self.b = b.to(dev, dtype).contiguous()
        self.h0 = (torch.zeros(B, d, device=dev, dtype=dtype) if h0 is None
                   else h0.to(dev, dtype).contiguous())
        self.up = torch.cuda.Stream(device=dev)
        self.comp = torch.cuda.Stream(device=dev)
        self.down = torch.cuda.Stream(device=dev)
        self.slots = []
        for _ in range(depth):
            s = _Slot()
            s.x, s.z, s.r = (torch.empty(T, B, d, device=dev, dtype=dtype) for _ in range(3))
            s.host = {k: torch.empty(T, B, d, dtype=dtype).pin_memory()
                      for k in ("output", "dx", "dz")}
            s.host.update({k: torch.empty(d, d, dtype=dtype).pin_memory()
                           for k in ("dW_x", "dW_h")})
            s.host["db"] = torch.empty(d, dtype=dtype).pin_memory()
            s.uploaded, s.computed, s.downloaded = (torch.cuda.Event() for _ in range(3))
            s.busy = False
            self.slots.append(s)
        self.calls = 0
        self.pre_compute = None   # optional callable run on the compute stream before each call
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(dev))
        for st in (self.up, self.comp, self.down):
            st.wait_event(ready)

    def submit(self, x, z, d_output):
        """Enqueues one call; returns the slot's dict of pinned host result buffers, valid
        after wait() (or after the returned dict's "done" event has completed).

        The buffers belong to one of `depth` ring slots and are REUSED: the submission numbered
        `valid_until_call` (also in the dict; calls are counted from 0) writes into the same
        host memory.  Consume or copy the results before making that submission; the pipeline
        cannot know when the caller is done reading, so it only orders the device side (the
        slot's previous kernels finish before its inputs are replaced, and downloads into one slot
        are ordered on one stream)."""
        for name, t in (("x", x), ("z", z), ("d_output", d_output)):
            if t.is_cuda or not t.is_pinned():
                raise RuntimeError(f"E1HostPipeline.submit: {name} must be a pinned host tensor")
        s = self.slots[self.calls % len(self.slots)]
        self.calls += 1
        if s.busy:  # the slot's device input buffers are free once its previous kernels are done
            self.up.wait_event(s.computed)
        with torch.cuda.stream(self.up):
            s.x.copy_(x, non_blocking=True)
            s.z.copy_(z, non_blocking=True)
            s.r.copy_(d_output, non_blocking=True)
            s.uploaded.record(self.up)
        with torch.cuda.stream(self.comp):
            self.comp.wait_event(s.uploaded)
            if self.pre_compute is not None:
                self.pre_compute()
            h, out, v = H.mamba_gated_elman_forward(True, s.x, s.z, self.h0, self.W_x, self.W_h,
                                                    self.b)
            dx, dz, dWx, dWh, db = H.mamba_gated_elman_backward(self.W_x, self.W_h, s.x, s.z, h, v,
                                                                s.r)
            s.computed.record(self.comp)
        results = {"output": out, "dx": dx, "dz": dz, "dW_x": dWx, "dW_h": dWh, "db": db}
        with torch.cuda.stream(self.down):
            self.down.wait_event(s.computed)
            for k, t in results.items():
                t.record_stream(self.down)
                s.host[k].copy_(t, non_blocking=True)
            s.downloaded.record(self.down)
        s.busy = True
        res = dict(s.host)
        res["done"] = s.downloaded
        res["valid_until_call"] = self.calls - 1 + len(self.slots)
        return res

    def wait(self):
        """Blocks until every submitted call has delivered its results to host memory."""
        self.down.synchronize()
        self.comp.synchronize()

    def bytes_per_call(self):
        e = torch.empty(0, dtype=self.dtype).element_size()
        n = self.T * self.B * self.d
        return 3 * n * e, (3 * n + 2 * self.d * self.d + self.d) * e
