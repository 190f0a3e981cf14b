"""A whole training step (forward, loss, backward, gradient clipping, optimizer)
captured once into a CUDA graph and replayed.

The layer/time pipeline of LadderLM issues a few thousand small launches per step
on several streams; issued from Python they are bound by the host.  Captured, the
streams' fork/join structure becomes graph dependencies and a step costs one
launch.  The reference trains eagerly (train_ladder.py); this is an addition on
the caller's side and changes no arithmetic.

Requirements: fixed token shape; an optimizer constructed with capturable=True;
no host synchronisation inside the model (LadderLM has none).
"""
import torch


def raise_on_device_timeout(where="a replayed step"):
    """Bounded device-side waits that give up are reported through a host-mapped status
    word.  The library's entry points read it when they are called, but a graph replay calls
    none of them: read it here (a plain host load, no synchronisation) and raise, so that the
    optimizer never keeps stepping on the results of a launch that gave up."""
    from . import _lib
    code, detail = _lib.device_status()
    if code != 0:
        raise _lib.ElmanB200Error(
            f"{where}: an earlier launch gave up a bounded device-side wait "
            f"(kernel {(detail >> 24) & 0xFF}, step {detail & 0xFFFFFF}); its results, and every "
            "step replayed since, are invalid")


class GraphedTrainStep:
    def __init__(self, net, optimizer, example_tokens, max_grad_norm=1.0, autocast_dtype=None,
                 warmup_steps=3, after_backward=None):
        """`after_backward(params)`, if given, runs between backward and clipping, inside
        the captured step: the place for a data-parallel gradient all-reduce."""
        self.net, self.opt = net, optimizer
        self.after_backward = after_backward
        self.max_grad_norm = max_grad_norm
        self.autocast_dtype = autocast_dtype
        self.tokens = example_tokens.clone()
        self.params = [p for g in optimizer.param_groups for p in g["params"]]
        side = torch.cuda.Stream(device=self.tokens.device)
        side.wait_stream(torch.cuda.current_stream(self.tokens.device))
        with torch.cuda.stream(side):
            for _ in range(warmup_steps):  # eager: creates optimizer state, library handles, streams
                self._eager_step()
        torch.cuda.current_stream(self.tokens.device).wait_stream(side)
        torch.cuda.synchronize(self.tokens.device)
        self.graph = torch.cuda.CUDAGraph()
        self.opt.zero_grad(set_to_none=True)
        from . import _lib
        before = _lib.launch_count()
        with torch.cuda.graph(self.graph):
            self.loss = self._eager_step(zero=False)
        # kernels of the CUDA library inside one captured step (each replay runs them again)
        self.library_launches_per_step = _lib.launch_count() - before

    def _eager_step(self, zero=True):
        if zero:
            self.opt.zero_grad(set_to_none=True)
        if self.autocast_dtype is not None:
            with torch.autocast(device_type="cuda", dtype=self.autocast_dtype):
                loss = self.net(self.tokens, return_loss=True)
        else:
            loss = self.net(self.tokens, return_loss=True)
        loss.backward()
        if self.after_backward is not None:
            self.after_backward(self.params)
        if self.max_grad_norm:
            torch.nn.utils.clip_grad_norm_(self.params, self.max_grad_norm)
        self.opt.step()
        return loss.detach()

    def __call__(self, tokens):
        """Copies `tokens` (host or device) into the captured input and replays the step.
        Returns the captured loss tensor (valid until the next call)."""
        raise_on_device_timeout("GraphedTrainStep")   # covers every replay up to the last one
        self.tokens.copy_(tokens, non_blocking=True)
        self.graph.replay()
        return self.loss

    def loss_value(self):
        """The last step's loss on the host; raises if any launch of it gave up a wait."""
        value = float(self.loss)          # synchronises with the replay
        raise_on_device_timeout("GraphedTrainStep.loss_value")
        return value


def allreduce_gradients(params, group=None):
    """Mean of the gradients over the ranks of `group` with one NCCL all-reduce over a
    flat buffer (capturable: no host synchronisation, fixed shapes)."""
    import torch.distributed as dist
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return
    flat = torch.cat([g.reshape(-1) for g in grads])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    flat.div_(dist.get_world_size(group))
    offset = 0
    for g in grads:
        n = g.numel()
        g.copy_(flat[offset:offset + n].view_as(g))
        offset += n
