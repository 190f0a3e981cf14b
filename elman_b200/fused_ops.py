"""Autograd nodes for the time-parallel ops around the cell, each backed by one kernel (or
one GEMM) of the CUDA library instead of a chain of framework ops:

  AddRMSNormFunction      residual add + RMSNorm, fp32 residual stream
                          (elman/models/ladder_lm.py:986-1003, :1013-1026 of the reference)
  InProjSplitSiluFunction the layer's input projection with split + silu in the GEMM epilogue
                          (elman/models/mamba_gated_elman.py:283-297)
  linear()                out_proj / lm_head through the library's GEMMs
                          (mamba_gated_elman.py:306, ladder_lm.py:929-933, :1062)

They change no arithmetic beyond rounding order and are used by the layers' fused paths and
by LadderLM; CPU tensors are refused like everywhere else in the package.
"""
import torch

from . import hasty_pytorch_lib


class GradSink:
    """Weight gradients written by the GEMM that produces them straight into pre-allocated
    buffers (C += A^T B), on side streams, instead of being returned to autograd.

    Why: in the (layer, time chunk) pipeline every weight receives one gradient contribution
    per chunk.  Returned to autograd, each contribution costs an extra add kernel, and the
    weight-gradient GEMMs sit on the streams that carry the chain of data gradients from layer
    to layer.  With a sink the autograd nodes return None for those weights and only the
    data-gradient GEMMs stay on the chain (the same idea as gradient-accumulation fusion in
    large-model trainers; the reference, which runs whole sequences layer by layer, has no
    counterpart).  Contributions to one weight always come from the same compute stream, so
    they are serialised on that stream's companion; `join()` makes a stream wait for all of
    them.  The owner (FlatGradients) registers the targets and joins before it reads them.
    """

    def __init__(self):
        self.targets = {}       # data_ptr of the weight -> gradient buffer shaped like it
        self.streams = {}       # compute stream id -> companion stream
        self.used = []          # companions that carry work since the last complete join
        self.units_expected = {}
        self.units_done = {}
        self.on_group_done = None   # callback(group) once all units of a group ran backward

    def register(self, weight, grad):
        self.targets[weight.data_ptr()] = grad

    def target(self, weight):
        return self.targets.get(weight.data_ptr())

    def _companion(self, device):
        cur = torch.cuda.current_stream(device)
        side = self.streams.get(cur.cuda_stream)
        if side is None:
            side = self.streams[cur.cuda_stream] = torch.cuda.Stream(device=device)
        return cur, side

    def accumulate_tn(self, grad, A, B):
        """grad += A^T B (A [K,M], B [K,N]) on the companion of the current stream."""
        H = hasty_pytorch_lib
        if not A.is_cuda:                       # (test stand-ins) no streams to use
            grad.add_(H.gemm(H.GEMM_TN, A, B))
            return
        cur, side = self._companion(A.device)
        ready = torch.cuda.Event()
        ready.record(cur)
        side.wait_event(ready)
        if side not in self.used:
            self.used.append(side)
        A.record_stream(side)
        B.record_stream(side)
        with torch.cuda.stream(side):
            H.gemm(H.GEMM_TN, A, B, out=grad, accumulate=True)

    def join(self, stream=None, final=False):
        """Makes `stream` (default: the current one) wait for every accumulation issued since
        the last final join.  Only companions that carry such work are touched: under stream
        capture an idle companion is not part of the capture and must not be waited on."""
        for side in self.used:
            target = stream or torch.cuda.current_stream(side.device)
            done = torch.cuda.Event()
            done.record(side)
            target.wait_event(done)
        if final:
            self.used = []

    # units: a group (one layer) is complete once all of its (layer, chunk) units have issued
    # their backward work; the owner then may start reducing that group's gradients
    def begin_pass(self):
        self.units_expected.clear()
        self.units_done.clear()

    def expect_unit(self, group):
        self.units_expected[group] = self.units_expected.get(group, 0) + 1

    def unit_done(self, group):
        self.units_done[group] = self.units_done.get(group, 0) + 1
        if self.units_done[group] == self.units_expected.get(group, 0) and self.on_group_done:
            self.on_group_done(group)


_sink = None


def set_grad_sink(sink):
    """Installs (or, with None, removes) the process-wide GradSink the autograd nodes of this
    package consult; returns the previous one."""
    global _sink
    old, _sink = _sink, sink
    return old


def get_grad_sink():
    return _sink


def weight_grad_tn(weight, A, B):
    """dW = A^T B for `weight`: returned — or, if a sink holds a buffer for this weight and
    gradients are being taken for it, accumulated there and None returned."""
    sink = _sink
    tgt = sink.target(weight) if (sink is not None and weight.requires_grad) else None
    if tgt is not None:
        # only if the buffer still IS this weight's gradient (an entry left behind by an
        # earlier owner whose memory was reused must never divert a gradient)
        g = getattr(weight, "grad", None)
        if g is None or g.data_ptr() != tgt.data_ptr() or g.shape != tgt.shape:
            tgt = None
    if tgt is None:
        return hasty_pytorch_lib.gemm(hasty_pytorch_lib.GEMM_TN, A, B)
    sink.accumulate_tn(tgt, A, B)
    return None


def rmsnorm_eps(norm_module, dtype):
    """nn.RMSNorm's effective epsilon: its own if set, else the machine epsilon of the type
    torch.rms_norm computes in — float32 for bfloat16 and float32 inputs (the documented
    "finfo(input.dtype).eps" is not what the kernels use for 16-bit inputs)."""
    eps = getattr(norm_module, "eps", None)
    if eps is not None:
        return float(eps)
    return float(torch.finfo(torch.float64 if dtype == torch.float64 else torch.float32).eps)


class AddRMSNormFunction(torch.autograd.Function):
    """forward(x, residual_in | None, weight, eps) -> (y, residual_out):
    residual_out = x + residual_in in fp32, y = RMSNorm(residual_out cast to x's dtype)."""

    @staticmethod
    def forward(ctx, x, residual_in, weight, eps, unit_group=None):
        H = hasty_pytorch_lib
        ctx.unit_group = unit_group   # this op opens a (layer, chunk) unit: its backward closes it
        xs = x.contiguous()
        y, res_out, rstd = H.add_rmsnorm_forward(
            xs, None if residual_in is None else residual_in.contiguous(), weight.contiguous(), eps)
        ctx.save_for_backward(res_out, rstd, weight)
        ctx.has_residual = residual_in is not None
        ctx.set_materialize_grads(False)
        ctx.mark_non_differentiable(rstd)
        return y, res_out

    @staticmethod
    def backward(ctx, dy, dres_out):
        res_out, rstd, weight = ctx.saved_tensors
        H = hasty_pytorch_lib
        if dy is None:
            dy = torch.zeros(res_out.shape, dtype=weight.dtype, device=res_out.device)
        if dres_out is not None and dres_out.dtype != torch.float32:
            dres_out = dres_out.float()
        here = torch.cuda.current_stream(dy.device) if dy.device.type == "cuda" else None
        if here is not None:
            dy.record_stream(here)
            if dres_out is not None:
                dres_out.record_stream(here)
        dres_in, dx, dw = H.add_rmsnorm_backward(
            dy.contiguous(), None if dres_out is None else dres_out.contiguous(), res_out, rstd,
            weight.contiguous(), want_dres_in=ctx.has_residual, want_dx=True)
        if ctx.unit_group is not None and _sink is not None:
            _sink.unit_done(ctx.unit_group)
        return dx, dres_in, dw, None, None


class InProjSplitSiluFunction(torch.autograd.Function):
    """forward(u [..., K], W_in [2d, K]) -> (x_act [..., d], z [..., d]) with
    x_act = silu((u W_in^T)[..., :d]) and z = (u W_in^T)[..., d:]."""

    @staticmethod
    def forward(ctx, u, W_in):
        H = hasty_pytorch_lib
        u2 = u.contiguous().view(-1, u.shape[-1])
        x_raw, x_act, z = H.in_proj_split_silu(u2, W_in.contiguous())
        ctx.save_for_backward(u2, W_in, x_raw)
        ctx.lead = u.shape[:-1]
        ctx.set_materialize_grads(False)
        d = x_act.shape[-1]
        return x_act.view(*ctx.lead, d), z.view(*ctx.lead, d)

    @staticmethod
    def backward(ctx, d_act, dz):
        u2, W_in, x_raw = ctx.saved_tensors
        H = hasty_pytorch_lib
        M, d = x_raw.shape
        if d_act is None:
            d_act = torch.zeros_like(x_raw)
        if dz is None:
            dz = torch.zeros_like(x_raw)
        here = torch.cuda.current_stream(x_raw.device) if x_raw.device.type == "cuda" else None
        if here is not None:
            d_act.record_stream(here)
            dz.record_stream(here)
        dxz = H.silu_backward_concat(d_act.contiguous().view(M, d), x_raw, dz.contiguous().view(M, d))
        du = H.gemm(H.GEMM_NN, dxz, W_in.contiguous())
        dW = weight_grad_tn(W_in, dxz, u2)
        return du.view(*ctx.lead, u2.shape[-1]), dW


EMBEDDING_ONE_HOT_MAX_VOCAB = 4096


class EmbeddingRowsFunction(torch.autograd.Function):
    """forward(tokens [...], weight [V, D]) -> weight[tokens].  The backward pass forms the
    weight gradient as a GEMM, onehot(tokens)^T · d_rows, through `weight_grad_tn`: dense and
    deterministic, and with a gradient sink it accumulates beside the data path instead of
    running ATen's sort-and-segment kernels at the very end of the backward pass.  Meant for
    byte-level vocabularies (`embedding_rows` falls back to nn.functional.embedding above
    EMBEDDING_ONE_HOT_MAX_VOCAB rows)."""

    @staticmethod
    def forward(ctx, tokens, weight):
        ctx.save_for_backward(tokens, weight)
        return torch.nn.functional.embedding(tokens, weight)

    @staticmethod
    def backward(ctx, d_rows):
        tokens, weight = ctx.saved_tensors
        n = tokens.numel()
        onehot = torch.zeros(n, weight.size(0), dtype=weight.dtype, device=weight.device)
        onehot.scatter_(1, tokens.reshape(n, 1), 1.0)
        d2 = d_rows.contiguous().view(n, weight.size(1))
        if d2.dtype != weight.dtype:
            d2 = d2.to(weight.dtype)
        return None, weight_grad_tn(weight, onehot, d2)


def embedding_rows(tokens, weight):
    """weight[tokens], with the one-hot GEMM backward where the library handles the weight."""
    if library_handles(weight) and weight.size(0) <= EMBEDDING_ONE_HOT_MAX_VOCAB \
            and torch.is_grad_enabled() and weight.requires_grad:
        return EmbeddingRowsFunction.apply(tokens, weight)
    return torch.nn.functional.embedding(tokens, weight)


def linear(x, weight, bias=None):
    """y = x W^T (+ b) over the last dimension through the library's GEMMs."""
    from .mamba_gated_elman import LinearFunction
    return LinearFunction.apply(x, weight, bias)


def library_handles(x):
    """True when `x` can go through the library's layer ops (CUDA, fp32 or bf16)."""
    return x.is_cuda and x.dtype in (torch.float32, torch.bfloat16)
