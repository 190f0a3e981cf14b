"""E1 — gated Elman layer with a Mamba2-style split input projection.

    x, z = split(in_proj(u));  x = silu(conv1d(x) if use_conv else x)
    h_t  = tanh(W_x x_t + W_h h_{t-1} + b)
    y_t  = h_t * silu(z_t);    out = out_proj(y)

Class names, constructor arguments, tensor layouts and parameter names follow
the reference (elman/models/mamba_gated_elman.py:30-311) so checkpoints and
callers carry over.  The cell always runs the CUDA library; a CPU tensor is an
error, not a fallback.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import fused_ops, hasty_pytorch_lib
from ._spectral import spectrally_normalised


class MambaGatedElmanFunction(torch.autograd.Function):
    """forward(training, x, z, h0, W_x, W_h, b) -> (h[T+1,B,d], output[T,B,d]).

    The backward pass takes only the gradient of `output`; the gradient of the
    returned h is dropped, exactly as the reference Function does (:42-47).
    """

    @staticmethod
    def forward(ctx, training, x, z, h0, W_x, W_h, b):
        h, output, v = hasty_pytorch_lib.mamba_gated_elman_forward(training, x, z, h0, W_x, W_h, b)
        ctx.save_for_backward(W_x, W_h, x, z, h, v)
        return h, output

    @staticmethod
    def backward(ctx, _dh, d_output):
        W_x, W_h, x, z, h, v = ctx.saved_tensors
        if v.numel() == 0:
            raise RuntimeError("backward needs the pre-activations: run forward with training=True")
        dx, dz, dW_x, dW_h, db = hasty_pytorch_lib.mamba_gated_elman_backward(
            W_x, W_h, x, z, h, v, d_output.contiguous())
        return None, dx, dz, None, dW_x, dW_h, db


class MambaGatedElmanHXFunction(torch.autograd.Function):
    """E1 with the output gate on [h_t ; x_t] — an extension: the reference has no such class;
    the formula is the one in its README (README.md:25-29),

        y_t = h_t * silu(W_g [h_t ; x_t] + b_g),   W_g = [W_gh | W_gx].

    forward(training, x, z, h0, W_x, W_h, b, W_gh) -> (h, output) with z = W_gx x + b_g the
    caller's time-parallel gate projection, exactly the `z` input of MambaGatedElmanFunction.
    The gradient of the returned h is dropped, as there."""

    @staticmethod
    def forward(ctx, training, x, z, h0, W_x, W_h, b, W_gh):
        h, output, v, zg = hasty_pytorch_lib.mamba_gated_elman_hx_forward(
            training, x, z, h0, W_x, W_h, b, W_gh)
        ctx.save_for_backward(W_x, W_h, W_gh, x, zg, h, v)
        return h, output

    @staticmethod
    def backward(ctx, _dh, d_output):
        W_x, W_h, W_gh, x, zg, h, v = ctx.saved_tensors
        if v.numel() == 0:
            raise RuntimeError("backward needs the pre-activations: run forward with training=True")
        dx, dz, dW_x, dW_h, db, dW_gh = hasty_pytorch_lib.mamba_gated_elman_hx_backward(
            W_x, W_h, W_gh, x, zg, h, v, d_output.contiguous())
        return None, dx, dz, None, dW_x, dW_h, db, dW_gh


def e1_hx_gate_cell(x, h0, W_x, W_h, b, W_g, b_g, training=True):
    """The whole README cell on time-major x [T,B,d]: gate projection z = W_gx x + b_g through
    the library's GEMM (bias in its epilogue), then MambaGatedElmanHXFunction.
    W_g: [d, 2d] = [W_gh | W_gx].  Returns (output [T,B,d], h [T+1,B,d])."""
    d = x.shape[-1]
    W_gh, W_gx = W_g[:, :d].contiguous(), W_g[:, d:].contiguous()
    z = LinearFunction.apply(x, W_gx, b_g)
    h, output = MambaGatedElmanHXFunction.apply(training, x.contiguous(), z.contiguous(),
                                                h0.contiguous(), W_x.contiguous(),
                                                W_h.contiguous(), b.contiguous(), W_gh)
    return output, h


class MambaGatedElmanChunkFunction(torch.autograd.Function):
    """One time chunk of a longer sequence (no counterpart in the reference).

    forward(x, z, h0, W_x, W_h, b) -> (output [T,B,d], h_last [B,d]).  Chunks are
    chained by passing h_last as the next chunk's h0.  Between two chained chunks
    the "gradient" that autograd carries along the h_last -> h0 edge is NOT
    dL/dh: it is the pre-activation gradient dv of the later chunk's first step,
    which is what the backward kernel takes as its state from the future
    (dL/dh would be dv W_h, one more matrix product the kernel does anyway).
    h_last must therefore only ever feed another chunk's h0 (or be detached), and
    the h0 of the first chunk gets no gradient, like the reference's Function.
    """

    @staticmethod
    def forward(ctx, x, z, h0, W_x, W_h, b, flags=0):
        h, output, v = hasty_pytorch_lib.mamba_gated_elman_forward(True, x, z, h0, W_x, W_h, b,
                                                                   flags)
        ctx.save_for_backward(W_x, W_h, x, z, h, v)
        ctx.set_materialize_grads(False)
        ctx.flags = flags
        return output, h[-1].clone()

    @staticmethod
    def backward(ctx, d_output, dv_in):
        W_x, W_h, x, z, h, v = ctx.saved_tensors
        if d_output is None:
            d_output = torch.zeros_like(x)
        dx, dz, dW_x, dW_h, db, dv_out = hasty_pytorch_lib.mamba_gated_elman_backward_carry(
            W_x, W_h, x, z, h, v, d_output.contiguous(),
            None if dv_in is None else dv_in.contiguous(), ctx.flags)
        return dx, dz, dv_out, dW_x, dW_h, db, None


class ChunkLink:
    """Carries the hidden states (and the bias gradient) of one chunk from its recurrence
    node to its projection node, whose backward pass needs them for dW_h."""
    __slots__ = ("h", "db")

    def __init__(self):
        self.h = None
        self.db = None


class E1ChunkProjectionFunction(torch.autograd.Function):
    """The time-parallel half of one chunk: forward(x, W_x, b, W_h, link) -> pre = x W_x^T + b.

    Its backward receives d(pre), which is the pre-activation gradient dv of the chunk's
    recurrence, and computes every GEMM of the cell's backward pass from it: dx = dv W_x,
    dW_x = dv^T x and — with the hidden states the recurrence node left in `link` —
    dW_h = dv^T h[0:T].  W_h is an input only so that this node can return that gradient;
    the forward pass does not read it.  Split from E1ChunkRecurrenceFunction so that the two
    halves can run on different CUDA streams (no counterpart in the reference).
    """

    @staticmethod
    def forward(ctx, x, W_x, b, W_h, link):
        T, B, d = x.shape
        pre = hasty_pytorch_lib.gemm(hasty_pytorch_lib.GEMM_NT, x.view(T * B, d), W_x, b)
        ctx.save_for_backward(x, W_x)
        ctx.link = link
        ctx.W_h_key = W_h     # only its identity is used: where its gradient goes
        return pre.view(T, B, d)

    @staticmethod
    def backward(ctx, dpre):
        x, W_x = ctx.saved_tensors
        T, B, d = x.shape
        link, ctx.link = ctx.link, None
        here = torch.cuda.current_stream(x.device) if x.is_cuda else None
        dv = dpre.contiguous().view(T * B, d)
        h, db = link.h, link.db
        if here is not None:   # produced on the recurrence's stream, read on this one
            for t in (dpre, h, db):
                t.record_stream(here)
        G = hasty_pytorch_lib
        dx = G.gemm(G.GEMM_NN, dv, W_x).view(T, B, d)
        # weight gradients: into the gradient sink's buffers on a side stream when one is
        # installed (only dx stays on the chain that the preceding layer waits for)
        dW_x = fused_ops.weight_grad_tn(W_x, dv, x.view(T * B, d))
        dW_h = fused_ops.weight_grad_tn(ctx.W_h_key, dv, h[:T].view(T * B, d))
        link.h = link.db = None
        return dx, dW_x, db, dW_h, None


class LinearFunction(torch.autograd.Function):
    """y = x W^T + b over the last dimension through the library's GEMMs (elman_gemm);
    backward: dx = dy W, dW = dy^T x, db = column sums of dy."""

    @staticmethod
    def forward(ctx, x, W, b):
        ctx.save_for_backward(x, W)
        ctx.has_bias = b is not None
        x2 = x.reshape(-1, x.shape[-1])
        return hasty_pytorch_lib.gemm(hasty_pytorch_lib.GEMM_NT, x2, W, b).view(*x.shape[:-1],
                                                                              W.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, W = ctx.saved_tensors
        G = hasty_pytorch_lib
        dy2 = dy.contiguous().view(-1, W.shape[0])
        dx = G.gemm(G.GEMM_NN, dy2, W).view(x.shape)
        dW = fused_ops.weight_grad_tn(W, dy2, x.reshape(-1, x.shape[-1]))
        return dx, dW, (G.column_sum(dy2) if ctx.has_bias else None)


class E1ChunkRecurrenceFunction(torch.autograd.Function):
    """The sequential half of one chunk: forward(pre, z, h0, W_h, link, flags) ->
    (output [T,B,d], h_last [B,d]).  The h_last -> next chunk's h0 edge carries the
    pre-activation gradient backward, exactly as in MambaGatedElmanChunkFunction; the
    gradient of W_h is produced by the projection node."""

    @staticmethod
    def forward(ctx, pre, z, h0, W_h, link, flags=0, W_h_T=None):
        h, output, v = hasty_pytorch_lib.e1_recurrence_forward(True, pre, z, h0, W_h, flags)
        link.h = h
        ctx.link = link
        ctx.W_h_T = W_h_T    # optional transposed copy shared by all chunks of a pass
        ctx.save_for_backward(W_h, z, h, v)
        ctx.set_materialize_grads(False)
        ctx.flags = flags
        return output, h[-1].clone()

    @staticmethod
    def backward(ctx, d_output, dv_in):
        W_h, z, h, v = ctx.saved_tensors
        T = z.shape[0]
        if d_output is None:
            d_output = torch.zeros_like(z)
        if z.is_cuda:
            here = torch.cuda.current_stream(z.device)
            d_output.record_stream(here)
            if dv_in is not None:
                dv_in.record_stream(here)
        dv, dz, db = hasty_pytorch_lib.e1_recurrence_backward(
            W_h, z, h, v, d_output.contiguous(), None if dv_in is None else dv_in.contiguous(),
            ctx.flags, ctx.W_h_T)
        ctx.link.db = db
        ctx.link = ctx.W_h_T = None
        return dv[:T], dz, dv[0], None, None, None, None


class MambaGatedElmanCell(nn.Module):
    """Weights of the recurrence and the dispatch into the CUDA library."""

    def __init__(self, dim, w_h_mode="none", w_h_init_gain=1.0, mamba2_init=False):
        super().__init__()
        self.dim = dim
        self.w_h_mode = w_h_mode
        self.mamba2_init = mamba2_init
        self.W_x = nn.Parameter(torch.empty(dim, dim))
        self.W_h = nn.Parameter(torch.empty(dim, dim))
        self.b = nn.Parameter(torch.zeros(dim))
        self._init_weights(w_h_init_gain)

    def _init_weights(self, gain):
        if self.mamba2_init == "s4d":
            nn.init.normal_(self.W_x, std=0.02)
            q = torch.empty(self.dim, self.dim, dtype=torch.float32)
            nn.init.orthogonal_(q)
            radii = torch.linspace(0.99, 0.9999, self.dim)
            with torch.no_grad():
                self.W_h.copy_((q @ torch.diag(radii) @ q.T).to(self.W_h.dtype))
            nn.init.zeros_(self.b)
        elif self.mamba2_init:
            nn.init.normal_(self.W_x, std=0.02)
            w = torch.empty(self.dim, self.dim, dtype=torch.float32)
            nn.init.orthogonal_(w)
            with torch.no_grad():
                self.W_h.copy_((w * 0.999).to(self.W_h.dtype))
            nn.init.zeros_(self.b)
        else:
            nn.init.xavier_uniform_(self.W_x)
            nn.init.xavier_uniform_(self.W_h, gain=gain)

    def get_W_h(self):
        if self.w_h_mode == "spectral_norm":
            return spectrally_normalised(self, self.W_h)
        return self.W_h

    def forward(self, x, z, h0=None):
        """x, z: [T,B,dim]; h0: [B,dim] -> (output [T,B,dim], h [T+1,B,dim])."""
        T, B, D = x.shape
        if not x.is_cuda:
            raise RuntimeError("elman_b200 runs on CUDA tensors only (no CPU fallback)")
        if h0 is None:
            h0 = torch.zeros(B, D, device=x.device, dtype=x.dtype)
        W_h = self.get_W_h()
        h, output = MambaGatedElmanFunction.apply(
            self.training, x.contiguous(), z.contiguous(), h0.contiguous(),
            self.W_x.contiguous(), W_h.contiguous(), self.b.contiguous())
        return output, h


class MambaGatedElman(nn.Module):
    """The E1 layer: in_proj -> (conv) -> silu -> cell -> out_proj, batch-major in and out."""

    def __init__(self, dim, expansion=1.0, dropout=0.0, r_h_mode="none", r_h_init_gain=1.0,
                 use_conv=False, d_conv=4, mamba2_init=False, **kwargs):
        super().__init__()
        self.dim = dim
        self.d_inner = int(dim * expansion)
        self.use_conv = use_conv
        self.mamba2_init = mamba2_init
        self.in_proj = nn.Linear(dim, 2 * self.d_inner, bias=False)
        if use_conv:
            self.conv1d = nn.Conv1d(self.d_inner, self.d_inner, kernel_size=d_conv,
                                    padding=d_conv - 1, groups=self.d_inner, bias=True)
        self.cell = MambaGatedElmanCell(self.d_inner, w_h_mode=r_h_mode,
                                        w_h_init_gain=r_h_init_gain, mamba2_init=mamba2_init)
        self.out_proj = nn.Linear(self.d_inner, dim, bias=False)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        # projections and their elementwise tails through the library's own kernels (False:
        # nn.Linear / framework ops, the reference's op-by-op form; same arithmetic)
        self.fused = True
        self._init_weights()

    def _init_weights(self):
        if self.mamba2_init:
            nn.init.normal_(self.in_proj.weight, std=0.02)
            nn.init.normal_(self.out_proj.weight, std=0.02)
        else:
            nn.init.xavier_uniform_(self.in_proj.weight)
            nn.init.xavier_uniform_(self.out_proj.weight)

    def forward(self, x, h0=None, **kwargs):
        """x: [B,T,dim] -> (output [B,T,dim], h_final [B,d_inner])."""
        B, T, D = x.shape
        if self.fused and not self.use_conv and fused_ops.library_handles(x):
            return self.forward_fused(x, h0)
        x_proj, z = self.in_proj(x).chunk(2, dim=-1)
        if self.use_conv:
            x_proj = self.conv1d(x_proj.transpose(1, 2))[:, :, :T].transpose(1, 2)
        x_proj = F.silu(x_proj)
        x_rnn = x_proj.permute(1, 0, 2).contiguous()
        z_rnn = z.permute(1, 0, 2).contiguous()
        cell_out, h_all = self.cell(x_rnn, z_rnn, h0)
        y = self.dropout(cell_out.permute(1, 0, 2).contiguous())
        return self.out_proj(y), h_all[-1]

    def forward_fused(self, x, h0=None, time_major=False):
        """forward() with every op on the library's kernels: one transposing copy of the input
        to the cell's time-major layout, in_proj with split + silu in its GEMM epilogue, the
        cell, out_proj as a library GEMM, one transposing copy back (none with time_major)."""
        xt = x if time_major else x.transpose(0, 1).contiguous()
        x_act, z = fused_ops.InProjSplitSiluFunction.apply(xt, self.in_proj.weight)
        cell_out, h_all = self.cell(x_act, z, h0)
        y = fused_ops.linear(self.dropout(cell_out), self.out_proj.weight)
        return (y if time_major else y.transpose(0, 1).contiguous()), h_all[-1]

    def _in_proj_act(self, x):
        """(silu(x half), gate half) of in_proj(x), contiguous, for time-major x."""
        if self.fused and fused_ops.library_handles(x):
            return fused_ops.InProjSplitSiluFunction.apply(x, self.in_proj.weight)
        x_proj, z = self.in_proj(x).chunk(2, dim=-1)
        return F.silu(x_proj).contiguous(), z.contiguous()

    def _out_proj(self, y):
        if self.fused and fused_ops.library_handles(y):
            return fused_ops.linear(y, self.out_proj.weight)
        return self.out_proj(y)

    # ---- time-chunked execution (used by LadderLM's layer/time pipeline) ----
    @property
    def supports_time_chunks(self):
        return not self.use_conv  # the causal conv would need its own carry

    def chunk_recurrence_blocks(self, dtype, T, B, flags=0):
        """Thread blocks one recurrence launch of this layer keeps resident (0: cooperative)."""
        return hasty_pytorch_lib.recurrence_blocks(dtype, T, B, self.d_inner, flags)

    def chunk_weights(self):
        """What every chunk of one forward pass shares: the effective W_h, computed once
        (the spectral-norm power iteration advances once per pass, as in forward())."""
        return self.cell.get_W_h().contiguous()

    def forward_chunk(self, x, h0, W_h, flags=0, time_major=False):
        """x: [B,Tc,dim] ([Tc,B,dim] with time_major), h0: [B,d_inner] (last state of the
        preceding chunk) -> (output in the layout of x, h_last).  Chained over the chunks of
        a sequence this equals forward() on the whole sequence.  Time-major callers skip the
        three layout copies around the cell: every other op of the layer is per token."""
        if time_major:
            x_rnn, z_rnn = self._in_proj_act(x)
        else:
            x_proj, z = self.in_proj(x).chunk(2, dim=-1)
            x_rnn = F.silu(x_proj).permute(1, 0, 2).contiguous()
            z_rnn = z.permute(1, 0, 2).contiguous()
        cell = self.cell
        cell_out, h_last = MambaGatedElmanChunkFunction.apply(
            x_rnn, z_rnn, h0.contiguous(), cell.W_x.contiguous(), W_h, cell.b.contiguous(), flags)
        y = cell_out if time_major else cell_out.permute(1, 0, 2).contiguous()
        return self._out_proj(self.dropout(y)), h_last

    # The same chunk in three pieces, for callers that put them on different streams:
    # chunk_pre (time-parallel, up to the projected inputs), chunk_rec (the recurrence
    # alone) and chunk_post (output projection).  All time-major [Tc,B,*].
    def chunk_pre(self, x, W_h, link):
        x_act, z = self._in_proj_act(x)
        cell = self.cell
        pre = E1ChunkProjectionFunction.apply(x_act, cell.W_x.contiguous(), cell.b.contiguous(),
                                              W_h, link)
        return pre, z

    def chunk_rec(self, pre, z, h0, W_h, link, flags=0, W_h_T=None):
        return E1ChunkRecurrenceFunction.apply(pre, z, h0.contiguous(), W_h, link, flags, W_h_T)

    def chunk_post(self, cell_out):
        return self._out_proj(self.dropout(cell_out))

    def extra_repr(self):
        return f"dim={self.dim}, d_inner={self.d_inner}, use_conv={self.use_conv}, LEVEL=1_MAMBA_GATED"
