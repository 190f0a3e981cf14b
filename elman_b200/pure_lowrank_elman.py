"""E5 — pure low-rank Elman layer: every matrix is a rank-r product U V, no projections.

    h_t = tanh(U_h (V_h h_{t-1}) + U_x (V_x x_t) + b);   y_t = h_t * silu(U_z (V_z x_t))

Mirrors the reference interface (elman/models/pure_lowrank_elman.py:28-307).
`use_fused` and `use_cuda_graph` are accepted for compatibility; the CUDA path
here is a single persistent launch per call, so neither changes what runs.
"""
import torch
import torch.nn as nn

from . import hasty_pytorch_lib


class PureLowRankElmanFunction(torch.autograd.Function):
    """forward(x, h0, U_h, V_h, U_x, V_x, U_z, V_z, b, training) -> (output, h)."""

    @staticmethod
    def forward(ctx, x, h0, U_h, V_h, U_x, V_x, U_z, V_z, b, training):
        h, output, v = hasty_pytorch_lib.pure_lowrank_elman_forward(
            training, x, h0, U_h, V_h, U_x, V_x, U_z, V_z, b)
        if training:
            ctx.save_for_backward(U_h, V_h, U_x, V_x, U_z, V_z, x, h, v)
        return output, h

    @staticmethod
    def backward(ctx, grad_output, _grad_h):
        U_h, V_h, U_x, V_x, U_z, V_z, x, h, v = ctx.saved_tensors
        dx, dU_h, dV_h, dU_x, dV_x, dU_z, dV_z, db = hasty_pytorch_lib.pure_lowrank_elman_backward(
            U_h, V_h, U_x, V_x, U_z, V_z, x, h, v, grad_output.contiguous())
        return dx, None, dU_h, dV_h, dU_x, dV_x, dU_z, dV_z, db, None


# Same computation under the reference's second name.
PureLowRankElmanFusedFunction = PureLowRankElmanFunction


class PureLowRankElmanChunkFunction(torch.autograd.Function):
    """One time chunk of a longer sequence (no counterpart in the reference):
    forward(x, h0, U_h, V_h, U_x, V_x, U_z, V_z, b) -> (output [T,B,d], h_last [B,d]).
    As with the E1 chunk nodes, the h_last -> next chunk's h0 edge carries the
    pre-activation gradient of the later chunk's first step backward, not dL/dh."""

    @staticmethod
    def forward(ctx, x, h0, U_h, V_h, U_x, V_x, U_z, V_z, b):
        h, output, v = hasty_pytorch_lib.pure_lowrank_elman_forward(
            True, x, h0, U_h, V_h, U_x, V_x, U_z, V_z, b)
        ctx.save_for_backward(U_h, V_h, U_x, V_x, U_z, V_z, x, h, v)
        ctx.set_materialize_grads(False)
        return output, h[-1].clone()

    @staticmethod
    def backward(ctx, grad_output, dv_in):
        U_h, V_h, U_x, V_x, U_z, V_z, x, h, v = ctx.saved_tensors
        if grad_output is None:
            grad_output = torch.zeros_like(x)
        if x.is_cuda:
            here = torch.cuda.current_stream(x.device)
            grad_output.record_stream(here)
            if dv_in is not None:
                dv_in.record_stream(here)
        r = hasty_pytorch_lib.pure_lowrank_elman_backward_carry(
            U_h, V_h, U_x, V_x, U_z, V_z, x, h, v, grad_output.contiguous(),
            None if dv_in is None else dv_in.contiguous())
        dx, dU_h, dV_h, dU_x, dV_x, dU_z, dV_z, db, dv_out = r
        return dx, dv_out, dU_h, dV_h, dU_x, dV_x, dU_z, dV_z, db


class PureLowRankElmanCell(nn.Module):
    def __init__(self, dim, rank=64, use_fused=True, use_cuda_graph=False):
        super().__init__()
        self.dim = dim
        self.rank = rank
        self.use_fused = use_fused
        self.use_cuda_graph = use_cuda_graph
        for name in ("h", "x", "z"):
            setattr(self, "U_" + name, nn.Parameter(torch.empty(dim, rank)))
            setattr(self, "V_" + name, nn.Parameter(torch.empty(rank, dim)))
        self.b = nn.Parameter(torch.zeros(dim))
        self._init_weights()

    def _init_weights(self):
        with torch.no_grad():
            for name in ("h", "x", "z"):
                U, V = getattr(self, "U_" + name), getattr(self, "V_" + name)
                nn.init.orthogonal_(U)
                nn.init.orthogonal_(V)
                U.mul_(0.5)
                V.mul_(0.5)

    def forward(self, x, h0=None):
        """x: [T,B,dim] -> (output [T,B,dim], h [T+1,B,dim])."""
        T, B, D = x.shape
        if not x.is_cuda:
            raise RuntimeError("elman_b200 runs on CUDA tensors only (no CPU fallback)")
        if h0 is None:
            h0 = torch.zeros(B, D, device=x.device, dtype=x.dtype)
        args = [t.contiguous() for t in (x, h0, self.U_h, self.V_h, self.U_x, self.V_x, self.U_z,
                                         self.V_z, self.b)]
        return PureLowRankElmanFunction.apply(*args, self.training)


class PureLowRankElman(nn.Module):
    def __init__(self, dim, rank=None, dropout=0.0, use_fused=True, use_cuda_graph=False, **kwargs):
        super().__init__()
        self.dim = dim
        self.d_inner = dim
        self.use_fused = use_fused
        self.use_cuda_graph = use_cuda_graph
        self.rank = max(16, dim // 8) if rank is None else rank
        self.cell = PureLowRankElmanCell(dim, rank=self.rank, use_fused=use_fused,
                                         use_cuda_graph=use_cuda_graph)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    def forward(self, x, h0=None, **kwargs):
        """x: [B,T,dim] -> (output [B,T,dim], h_final [B,dim])."""
        cell_out, h_all = self.cell(x.permute(1, 0, 2).contiguous(), h0)
        return self.dropout(cell_out.permute(1, 0, 2).contiguous()), h_all[-1]

    # ---- time-chunked execution (LadderLM's layer/time pipeline), time-major [Tc,B,dim] ----
    # The layer is the cell: nothing runs before the recurrence call (which contains the
    # low-rank projections) and only dropout after it.
    supports_time_chunks = True

    def chunk_weights(self):
        return None

    def chunk_recurrence_blocks(self, dtype, T, B, flags=0):
        return hasty_pytorch_lib.lowrank_blocks(dtype, T, B, self.dim, self.rank)

    def chunk_pre(self, x, W_h, link):
        return x.contiguous(), None

    def chunk_rec(self, pre, z, h0, W_h, link, flags=0, W_h_T=None):
        c = self.cell
        return PureLowRankElmanChunkFunction.apply(
            pre, h0.contiguous(), c.U_h.contiguous(), c.V_h.contiguous(), c.U_x.contiguous(),
            c.V_x.contiguous(), c.U_z.contiguous(), c.V_z.contiguous(), c.b.contiguous())

    def chunk_post(self, cell_out):
        return self.dropout(cell_out)

    def extra_repr(self):
        return (f"dim={self.dim}, rank={self.rank}, fused={self.use_fused}, "
                f"cuda_graph={self.use_cuda_graph}, LEVEL=5")
