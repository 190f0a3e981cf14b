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
                 warmup_steps=3, after_backward=None, reducer=None):
        """`reducer` (a FlatGradients, optional): the gradients live in its flat buffer; it
        zeroes them, all-reduces them bucket by bucket while backward still runs (N > 1) and
        clips them.  `after_backward(params)` (the older hook), if given, runs between
        backward and clipping, inside the captured step."""
        self.net, self.opt = net, optimizer
        self.after_backward = after_backward
        self.reducer = reducer
        self.max_grad_norm = max_grad_norm
        self.autocast_dtype = autocast_dtype
        self.tokens = example_tokens.clone()
        self.params = [p for g in optimizer.param_groups for p in g["params"]]
        side = torch.cuda.Stream(device=self.tokens.device)
        side.wait_stream(torch.cuda.current_stream(self.tokens.device))
        with torch.cuda.stream(side):
            self.warmup_losses = []
            for _ in range(warmup_steps):  # eager: creates optimizer state, library handles, streams
                self.warmup_losses.append(self._eager_step())
        torch.cuda.current_stream(self.tokens.device).wait_stream(side)
        torch.cuda.synchronize(self.tokens.device)
        self.graph = torch.cuda.CUDAGraph()
        if self.reducer is None:
            self.opt.zero_grad(set_to_none=True)
        from . import _lib
        before = _lib.launch_count()
        with torch.cuda.graph(self.graph):
            self.loss = self._eager_step(zero=False)
        # kernels of the CUDA library inside one captured step (each replay runs them again)
        self.library_launches_per_step = _lib.launch_count() - before

    def _eager_step(self, zero=True):
        if self.reducer is not None:
            self.reducer.zero()          # also inside the captured step: one memset
        elif zero:
            self.opt.zero_grad(set_to_none=True)
        if self.autocast_dtype is not None:
            with torch.autocast(device_type="cuda", dtype=self.autocast_dtype):
                loss = self.net(self.tokens, return_loss=True)
        else:
            loss = self.net(self.tokens, return_loss=True)
        loss.backward()
        if self.reducer is not None:
            self.reducer.finish()
        if self.after_backward is not None:
            self.after_backward(self.params)
        if isinstance(self.opt, FlatAdamW) and self.reducer is not None:
            # clipping folded into the update: the factor is applied as the gradients are read
            coef = self.reducer.clip_coef(self.max_grad_norm)[0] if self.max_grad_norm else None
            self.opt.step(grad_scale=coef)
            return loss.detach()
        if self.max_grad_norm:
            if self.reducer is not None:
                self.reducer.clip_(self.max_grad_norm)
            else:
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


class FlatGradients:
    """Every gradient of a model as a view into ONE pre-allocated flat buffer, cut into
    buckets, and — for data-parallel training — one all-reduce per bucket that starts as
    soon as that bucket's gradients are final, on a communication stream of its own, while
    the backward pass of the remaining layers still runs.

    This is what DistributedDataParallel does for the reference (bucketed NCCL all-reduce
    overlapped with autograd, train_ladder.py:306-307), without its copies: gradients are
    accumulated by autograd straight into the buffer the collective reads, nothing is
    concatenated before or copied back after.  Capturable into a CUDA graph (fixed
    addresses, no host synchronisation); the cross-stream edges become graph edges.

      buckets        list of lists of parameters, in the order their gradients become final
                     (last layer first); every parameter in exactly one bucket
      group / world  process group and its size; world 1 (or no initialised group) means no
                     collective — the flat buffer still serves zeroing and clipping

    Per step: zero() -> forward/backward -> finish() -> clip_() -> optimizer.
    """

    def __init__(self, buckets, group=None, direct=(), bucket_groups=None):
        """`direct`: parameters whose gradient the library's GEMMs accumulate straight into
        this buffer through a fused_ops.GradSink (installed here) instead of autograd;
        `bucket_groups[i]`: the sink's unit group (layer index) that completes bucket i."""
        import torch.distributed as dist
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        params = [p for b in buckets for p in b]
        if len({id(p) for p in params}) != len(params):
            raise ValueError("a parameter appears in more than one bucket")
        if not params:
            raise ValueError("no parameters")
        dtype, device = params[0].dtype, params[0].device
        for p in params:
            if p.dtype != dtype or p.device != device:
                raise ValueError("all parameters must share one dtype and device")
        total = 0
        self._slices = []
        for b in buckets:      # 256-byte aligned buckets
            start = total
            for p in b:
                total += p.numel()
            total = (total + 127) // 128 * 128
            self._slices.append((start, total))
        self.flat = torch.zeros(total, dtype=dtype, device=device)
        self.bucket_views = [self.flat[a:b] for a, b in self._slices]
        self.params = params
        self._pending = []
        self._bucket_of = {}
        self._hooks = []
        for bi, (b, (start, _)) in enumerate(zip(buckets, self._slices)):
            off = start
            for p in b:
                p.grad = self.flat[off:off + p.numel()].view_as(p)
                off += p.numel()
                self._bucket_of[id(p)] = bi
                if self.world > 1 and id(p) not in {id(q) for q in direct}:
                    self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad_final))
            self._pending.append(len(b))
        self.sink = None
        direct_ids = {id(p) for p in direct}
        if direct_ids:
            from . import fused_ops
            self.sink = fused_ops.GradSink()
            for p in params:
                if id(p) in direct_ids:
                    self.sink.register(p, p.grad)
            self.sink.on_group_done = self._on_group_done
            fused_ops.set_grad_sink(self.sink)
            # a bucket with direct parameters is complete when its remaining parameters' hooks
            # have fired AND the sink reports its group done (one extra pending count)
            groups = list(bucket_groups) if bucket_groups is not None else [None] * len(buckets)
            self._group_bucket = {}
            for bi, b in enumerate(buckets):
                n_direct = sum(1 for p in b if id(p) in direct_ids)
                if n_direct:
                    self._pending[bi] += 1 - n_direct
                    if groups[bi] is not None:
                        self._group_bucket[groups[bi]] = bi
        self._direct_ids = direct_ids
        self._sizes = list(self._pending)
        self.comm_stream = torch.cuda.Stream(device=device) if (device.type == "cuda" and self.world > 1) else None
        self._launched = 0

    def close(self):
        """Removes this object's gradient sink from the autograd nodes (they return their weight
        gradients to autograd again) and its hooks."""
        from . import fused_ops
        if self.sink is not None and fused_ops.get_grad_sink() is self.sink:
            fused_ops.set_grad_sink(None)
        for h in self._hooks:
            h.remove()
        self._hooks = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def describe(self):
        if self.world == 1:
            return "none (one rank); gradients in one flat buffer"
        mb = [round((b - a) * self.flat.element_size() / 1e6, 1) for a, b in self._slices]
        return (f"NCCL all-reduce of {len(mb)} buckets {mb} MB, each released on a communication "
                "stream when its gradients are final, overlapped with the rest of backward, "
                "inside the step graph; gradients are views into one flat buffer (no cat, no copy-back)")

    def zero(self):
        self.flat.zero_()
        self._pending = list(self._sizes)
        self._launched = 0

    def _on_grad_final(self, p):
        # autograd accumulated in place into the view; a replaced .grad would break the scheme
        bi = self._bucket_of[id(p)]
        self._pending[bi] -= 1
        if self._pending[bi] == 0:
            self._reduce_bucket(bi)

    def _on_group_done(self, group):
        bi = getattr(self, "_group_bucket", {}).get(group)
        if bi is None or self.world == 1:
            return
        self._pending[bi] -= 1
        if self._pending[bi] == 0:
            self._reduce_bucket(bi)

    def _reduce_bucket(self, bi):
        import torch.distributed as dist
        self._launched += 1
        view = self.bucket_views[bi]
        if self.comm_stream is None:
            dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group)
            return
        here = torch.cuda.current_stream(view.device)   # the stream this gradient became final on
        ready = torch.cuda.Event()
        ready.record(here)
        self.comm_stream.wait_event(ready)
        if self.sink is not None:      # ... and the weight-gradient GEMMs on their side streams
            self.sink.join(self.comm_stream)
        with torch.cuda.stream(self.comm_stream):
            dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group)

    def finish(self):
        """After backward: buckets whose hooks did not all fire (a parameter without a
        gradient this step) are reduced now; the caller's stream then waits for the
        communication stream and the sums become means."""
        if self.sink is not None:
            self.sink.join(final=True)   # the caller's stream waits for the accumulating GEMMs
        if self.world == 1:
            return
        for bi, left in enumerate(self._pending):
            if left > 0:
                self._pending[bi] = 0
                self._reduce_bucket(bi)
        if self.comm_stream is not None:
            torch.cuda.current_stream(self.flat.device).wait_stream(self.comm_stream)
        self.flat.mul_(1.0 / self.world)

    def clip_coef(self, max_norm, eps=1e-6):
        """(factor, norm): the factor clip_grad_norm_ would scale the gradients by —
        min(1, max_norm / (|g| + eps)) — as a 0-dim fp32 device tensor, gradients untouched.
        FlatAdamW applies it while it reads them."""
        total = torch.linalg.vector_norm(self.flat, 2, dtype=torch.float32)
        return torch.clamp(max_norm / (total + eps), max=1.0), total

    def flatten_parameters(self):
        """Moves the parameters themselves into one flat buffer with the layout of the
        gradient buffer (every parameter becomes a view of it) and returns that buffer."""
        if getattr(self, "flat_params", None) is None:
            flat = torch.zeros_like(self.flat)
            lo = self.flat.data_ptr()
            with torch.no_grad():
                for p in self.params:
                    off = (p.grad.data_ptr() - lo) // self.flat.element_size()
                    view = flat[off:off + p.numel()].view_as(p)
                    view.copy_(p.data)
                    p.data = view
            self.flat_params = flat
            if self.sink is not None:     # the sink finds a weight by its address: re-register
                self.sink.targets.clear()
                for p in self.params:
                    if id(p) in self._direct_ids:
                        self.sink.register(p, p.grad)
        return self.flat_params

    def clip_(self, max_norm, eps=1e-6):
        """torch.nn.utils.clip_grad_norm_ (train_ladder.py:542-543 of the reference) on the
        flat buffer: one norm, one scale, no host synchronisation.  Returns the norm."""
        total = torch.linalg.vector_norm(self.flat, 2, dtype=torch.float32)
        coef = torch.clamp(max_norm / (total + eps), max=1.0)
        self.flat.mul_(coef.to(self.flat.dtype))   # same dtype: the vectorised kernel
        return total

    def check_views(self):
        """True while every parameter's .grad still is its view into the flat buffer."""
        lo = self.flat.data_ptr()
        hi = lo + self.flat.numel() * self.flat.element_size()
        return all(p.grad is not None and lo <= p.grad.data_ptr() < hi for p in self.params)


class FlatAdamW:
    """AdamW (torch.optim.AdamW's update rule; train_ladder.py:360-365 of the reference) over
    the flat parameter / gradient buffers of a FlatGradients: one kernel launch per step
    (elman_adamw_step) instead of the per-tensor launches of the framework optimizer, with
    the clipping factor applied while the gradients are read.  Moment estimates are kept in
    the parameters' dtype, as torch.optim.AdamW keeps them.  The step counter lives on the
    device, so a captured step advances it on every replay."""

    def __init__(self, grads, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        if not grads.flat.is_cuda:
            raise RuntimeError("FlatAdamW runs on CUDA buffers only (no CPU fallback)")
        self.grads = grads
        self.flat_params = grads.flatten_parameters()
        self.exp_avg = torch.zeros_like(grads.flat)
        self.exp_avg_sq = torch.zeros_like(grads.flat)
        self.step_count = torch.zeros(1, dtype=torch.float32, device=grads.flat.device)
        self.defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        self.param_groups = [dict(params=list(grads.params), **self.defaults)]

    def zero_grad(self, set_to_none=False):
        self.grads.zero()

    def step(self, grad_scale=None):
        from . import _lib
        from . import hasty_pytorch_lib as H
        g = self.param_groups[0]
        flat = self.flat_params
        if grad_scale is not None and (grad_scale.dtype != torch.float32 or not grad_scale.is_cuda):
            raise RuntimeError("FlatAdamW.step: grad_scale must be a float32 CUDA tensor")
        with torch.cuda.device(flat.device):
            rc = _lib.load().elman_adamw_step(
                H._DT[flat.dtype], flat.numel(), flat.data_ptr(), self.grads.flat.data_ptr(),
                self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(), float(g["lr"]),
                float(g["betas"][0]), float(g["betas"][1]), float(g["eps"]),
                float(g["weight_decay"]), self.step_count.data_ptr(),
                None if grad_scale is None else grad_scale.data_ptr(),
                torch.cuda.current_stream(flat.device).cuda_stream)
            _lib.check(rc, "elman_adamw_step")

    def state_dict(self):
        return {"step": self.step_count.clone(), "exp_avg": self.exp_avg.clone(),
                "exp_avg_sq": self.exp_avg_sq.clone(), "param_groups": [
                    {k: v for k, v in self.param_groups[0].items() if k != "params"}]}

    def load_state_dict(self, sd):
        self.step_count.copy_(sd["step"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.param_groups[0].update(sd["param_groups"][0])


def ladder_buckets(model):
    """Buckets for a LadderLM in the order backward completes them: the last layer (with its
    pre-norm) first, the embedding / final norm last.  Other modules: one bucket."""
    layers = getattr(model, "layers", None)
    norms = getattr(model, "layer_norms", None)
    if layers is None or norms is None:
        return [[p for p in model.parameters() if p.requires_grad]]
    seen, buckets = set(), []
    for i in reversed(range(len(layers))):
        b = [p for p in list(layers[i].parameters()) + list(norms[i].parameters())
             if p.requires_grad and id(p) not in seen]
        seen.update(id(p) for p in b)
        if b:
            buckets.append(b)
    rest = [p for p in model.parameters() if p.requires_grad and id(p) not in seen]
    if rest:
        buckets.append(rest)
    return buckets


def direct_weights(model):
    """Weights of a LadderLM whose gradient contributions the library's GEMMs can accumulate
    in place: the layers' projection matrices reached only through this package's autograd
    nodes (not the tied embedding / head weight, which also receives an autograd gradient)."""
    out = []
    for layer in getattr(model, "layers", []):
        if not getattr(layer, "fused", True) or getattr(layer, "use_conv", False):
            continue
        for name in ("in_proj", "out_proj"):
            lin = getattr(layer, name, None)
            if lin is not None and getattr(lin, "bias", None) is None:
                out.append(lin.weight)
        cell = getattr(layer, "cell", None)
        if cell is not None and hasattr(cell, "W_x") and hasattr(layer, "in_proj"):
            out.append(cell.W_x)
            if getattr(cell, "w_h_mode", "none") in ("none", "free") and hasattr(cell, "W_h"):
                out.append(cell.W_h)
            if hasattr(cell, "W_gate"):
                out.append(cell.W_gate)
    return out


def make_gradient_reducer(model, group=None, direct=True):
    buckets = ladder_buckets(model)
    layers = getattr(model, "layers", None)
    groups = None
    if layers is not None and len(buckets) >= len(layers):
        groups = [len(layers) - 1 - bi if bi < len(layers) else None for bi in range(len(buckets))]
    use_direct = direct and getattr(model, "fused_ops", False) and next(model.parameters()).is_cuda
    return FlatGradients(buckets, group=group, direct=direct_weights(model) if use_direct else (),
                         bucket_groups=groups)
