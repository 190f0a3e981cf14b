"""Siblings of E1 that run on the same recurrence kernels — the reference's ladder levels
4, 32, 33, 57 and the multi-head E1H.  Class names, constructor arguments, parameter names and forward contracts
follow the reference files so that checkpoints and callers carry over:

  E32NoPresilu      E1 without the silu on the recurrence input
                    (elman/models/e32_no_presilu.py:196-302; its cell calls the E1 extension
                    functions, :30-47)
  E33SelfGate       y_t = h_t * silu(h_t), in_proj to d_inner only
                    (elman/models/e33_self_gate.py:30-50, :52-193, :196-296)
  LowRankElman      (E4) E1 whose recurrent matrix is U V, rank r; the recurrence runs on the
                    low-rank (E5) kernel (elman/models/lowrank_elman.py:28-46, :49-160, :163-254)
  E1MultiHead       (E1H) H independent heads of size n_state, run as one block-diagonal
                    recurrence (elman/models/e1_multihead.py:43-115, :118-283)
  E57LearnedRadius  E1 whose W_h is rescaled to a LEARNED spectral radius
                    sigmoid(log_radius) * max_radius (elman/models/e57_learned_radius.py:25-148,
                    :151-254; reuses the E1 autograd Function, :118-121)

As everywhere in this package the cells run the CUDA library only (CPU tensors raise).
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import fused_ops, hasty_pytorch_lib
from .mamba_gated_elman import MambaGatedElman, MambaGatedElmanCell, MambaGatedElmanFunction


class E32NoPresilu(MambaGatedElman):
    """E1 with the pre-activation removed: the recurrence input is the raw first half of
    in_proj(x).  The reference's default r_h_mode for this level is spectral normalisation."""

    def __init__(self, dim, expansion=1.0, dropout=0.0, r_h_mode="spectral_norm", r_h_init_gain=1.0,
                 use_conv=False, d_conv=4, mamba2_init=False, **kwargs):
        super().__init__(dim, expansion=expansion, dropout=dropout, r_h_mode=r_h_mode,
                         r_h_init_gain=r_h_init_gain, use_conv=use_conv, d_conv=d_conv,
                         mamba2_init=mamba2_init, **kwargs)

    def forward(self, x, h0=None, **kwargs):
        B, T, D = x.shape
        x_proj, z = self.in_proj(x).chunk(2, dim=-1)
        if self.use_conv:
            x_proj = self.conv1d(x_proj.transpose(1, 2))[:, :, :T].transpose(1, 2)
        x_rnn = x_proj.permute(1, 0, 2).contiguous()      # no silu here
        z_rnn = z.permute(1, 0, 2).contiguous()
        cell_out, h_all = self.cell(x_rnn, z_rnn, h0)
        y = self.dropout(cell_out.permute(1, 0, 2).contiguous())
        return self._out_proj(y), h_all[-1]

    def _in_proj_act(self, x):     # the time-chunked path: same split, no activation
        x_proj, z = self.in_proj(x).chunk(2, dim=-1)
        return x_proj.contiguous(), z.contiguous()

    def forward_fused(self, x, h0=None, time_major=False):
        raise NotImplementedError("E32 has no fused whole-layer path; use forward()")

    def extra_repr(self):
        return f"dim={self.dim}, d_inner={self.d_inner}, LEVEL=32_NO_PRESILU"


class E33SelfGateFunction(torch.autograd.Function):
    """forward(training, x, h0, W_x, W_h, b) -> (h, output); the gradient of h is dropped."""

    @staticmethod
    def forward(ctx, training, x, h0, W_x, W_h, b):
        h, output, v = hasty_pytorch_lib.e33_self_gate_forward(training, x, h0, W_x, W_h, b)
        ctx.save_for_backward(W_x, W_h, x, h, v)
        return h, output

    @staticmethod
    def backward(ctx, _dh, d_output):
        W_x, W_h, x, h, v = ctx.saved_tensors
        if v.numel() == 0:
            raise RuntimeError("backward needs the pre-activations: run forward with training=True")
        dx, dW_x, dW_h, db = hasty_pytorch_lib.e33_self_gate_backward(
            W_x, W_h, x, h, v, d_output.contiguous())
        return None, dx, None, dW_x, dW_h, db


class E33SelfGateCell(MambaGatedElmanCell):
    """E1's weights and W_h handling; the output gate is the state itself."""

    def forward(self, x, z=None, h0=None):
        T, B, D = x.shape
        if not x.is_cuda:
            raise RuntimeError("elman_b200 runs on CUDA tensors only (no CPU fallback)")
        if h0 is None:
            h0 = torch.zeros(B, D, device=x.device, dtype=x.dtype)
        h, output = E33SelfGateFunction.apply(self.training, x.contiguous(), h0.contiguous(),
                                              self.W_x.contiguous(), self.get_W_h().contiguous(),
                                              self.b.contiguous())
        return output, h


class E33SelfGate(nn.Module):
    def __init__(self, dim, expansion=1.0, dropout=0.0, r_h_mode="none", r_h_init_gain=1.0,
                 use_conv=False, d_conv=4, mamba2_init=False, **kwargs):
        super().__init__()
        self.dim = dim
        self.d_inner = int(dim * expansion)
        self.use_conv = use_conv
        self.mamba2_init = mamba2_init
        self.in_proj = nn.Linear(dim, self.d_inner, bias=False)
        if use_conv:
            self.conv1d = nn.Conv1d(self.d_inner, self.d_inner, kernel_size=d_conv,
                                    padding=d_conv - 1, groups=self.d_inner, bias=True)
        self.cell = E33SelfGateCell(self.d_inner, w_h_mode=r_h_mode, w_h_init_gain=r_h_init_gain,
                                    mamba2_init=mamba2_init)
        self.out_proj = nn.Linear(self.d_inner, dim, bias=False)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        if mamba2_init:
            nn.init.normal_(self.in_proj.weight, std=0.02)
            nn.init.normal_(self.out_proj.weight, std=0.02)
        else:
            nn.init.xavier_uniform_(self.in_proj.weight)
            nn.init.xavier_uniform_(self.out_proj.weight)

    def forward(self, x, h0=None, **kwargs):
        """x: [B,T,dim] -> (output [B,T,dim], h_final [B,d_inner])."""
        B, T, D = x.shape
        x_proj = self.in_proj(x)
        if self.use_conv:
            x_proj = self.conv1d(x_proj.transpose(1, 2))[:, :, :T].transpose(1, 2)
        x_rnn = F.silu(x_proj).permute(1, 0, 2).contiguous()
        cell_out, h_all = self.cell(x_rnn, None, h0)
        y = self.dropout(cell_out.permute(1, 0, 2).contiguous())
        out = fused_ops.linear(y, self.out_proj.weight) if fused_ops.library_handles(y) \
            else self.out_proj(y)
        return out, h_all[-1]

    def extra_repr(self):
        return f"dim={self.dim}, d_inner={self.d_inner}, LEVEL=33_SELF_GATE"


class E57LearnedRadiusCell(nn.Module):
    """E1 cell whose recurrent matrix is rescaled to sigmoid(log_radius) * max_radius."""

    def __init__(self, dim, max_radius=0.999, init_radius=0.99, mamba2_init=False):
        super().__init__()
        self.dim = dim
        self.max_radius = max_radius
        self.mamba2_init = mamba2_init
        self.W_x = nn.Parameter(torch.empty(dim, dim))
        self.W_h = nn.Parameter(torch.empty(dim, dim))
        self.b = nn.Parameter(torch.zeros(dim))
        init_logit = torch.logit(torch.tensor(init_radius / max_radius))
        self.log_radius = nn.Parameter(torch.full((1,), init_logit.item()))
        if mamba2_init:
            nn.init.normal_(self.W_x, std=0.02)
            w = torch.empty(dim, dim, dtype=torch.float32)
            nn.init.orthogonal_(w)
            with torch.no_grad():
                self.W_h.copy_(w.to(self.W_h.dtype))
            nn.init.constant_(self.b, 0.0)
        else:
            nn.init.xavier_uniform_(self.W_x)
            nn.init.xavier_uniform_(self.W_h)

    @property
    def target_radius(self):
        return torch.sigmoid(self.log_radius) * self.max_radius

    def get_W_h(self):
        """Three power-iteration steps (no gradient) from a persistent vector, then
        W_h * target / (|u^T W_h v| + 1e-8); gradients reach W_h and log_radius."""
        W = self.W_h
        u = getattr(self, "_spectral_u", None)
        if u is None or u.shape[0] != self.dim:
            u = torch.randn(self.dim, device=W.device, dtype=W.dtype)
            u = u / u.norm()
        with torch.no_grad():
            for _ in range(3):
                v = W.T @ u
                v = v / (v.norm() + 1e-8)
                u = W @ v
                u = u / (u.norm() + 1e-8)
            self._spectral_u = u
        sigma = (u @ W @ v).abs()
        return W * (self.target_radius / (sigma + 1e-8))

    def forward(self, x, z, h0=None):
        T, B, D = x.shape
        if not x.is_cuda:
            raise RuntimeError("elman_b200 runs on CUDA tensors only (no CPU fallback)")
        if h0 is None:
            h0 = torch.zeros(B, D, device=x.device, dtype=x.dtype)
        h, output = MambaGatedElmanFunction.apply(
            self.training, x.contiguous(), z.contiguous(), h0.contiguous(), self.W_x.contiguous(),
            self.get_W_h().contiguous(), self.b.contiguous())
        return output, h


class E57LearnedRadius(nn.Module):
    def __init__(self, dim, expansion=2.0, dropout=0.0, r_h_mode="learned", r_h_init_gain=1.0,
                 use_conv=False, d_conv=4, mamba2_init=False, max_radius=0.999, init_radius=0.99,
                 **kwargs):
        super().__init__()
        self.dim = dim
        self.d_inner = int(dim * expansion)
        self.use_conv = use_conv
        self.mamba2_init = mamba2_init
        self.in_proj = nn.Linear(dim, 2 * self.d_inner, bias=False)
        if use_conv:
            self.conv1d = nn.Conv1d(self.d_inner, self.d_inner, kernel_size=d_conv,
                                    padding=d_conv - 1, groups=self.d_inner, bias=True)
        self.cell = E57LearnedRadiusCell(self.d_inner, max_radius=max_radius,
                                         init_radius=init_radius, mamba2_init=mamba2_init)
        self.out_proj = nn.Linear(self.d_inner, dim, bias=False)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        if mamba2_init:
            nn.init.normal_(self.in_proj.weight, std=0.02)
            nn.init.normal_(self.out_proj.weight, std=0.02)
        else:
            nn.init.xavier_uniform_(self.in_proj.weight)
            nn.init.xavier_uniform_(self.out_proj.weight)

    def forward(self, x, h0=None, **kwargs):
        B, T, D = x.shape
        if not self.use_conv and fused_ops.library_handles(x):
            xt = x.transpose(0, 1).contiguous()
            x_act, z = fused_ops.InProjSplitSiluFunction.apply(xt, self.in_proj.weight)
            cell_out, h_all = self.cell(x_act, z, h0)
            y = fused_ops.linear(self.dropout(cell_out), self.out_proj.weight)
            return y.transpose(0, 1).contiguous(), h_all[-1]
        x_proj, z = self.in_proj(x).chunk(2, dim=-1)
        if self.use_conv:
            x_proj = self.conv1d(x_proj.transpose(1, 2))[:, :, :T].transpose(1, 2)
        x_rnn = F.silu(x_proj).permute(1, 0, 2).contiguous()
        z_rnn = z.permute(1, 0, 2).contiguous()
        cell_out, h_all = self.cell(x_rnn, z_rnn, h0)
        y = self.dropout(cell_out.permute(1, 0, 2).contiguous())
        return self.out_proj(y), h_all[-1]

    def extra_repr(self):
        return f"dim={self.dim}, d_inner={self.d_inner}, LEVEL=57_LEARNED_RADIUS"


class LowRankElmanFunction(torch.autograd.Function):
    """forward(x, z, h0, W_x, U, V, b, training) -> (output, h); the gradient of h is dropped
    (elman/models/lowrank_elman.py:28-46)."""

    @staticmethod
    def forward(ctx, x, z, h0, W_x, U, V, b, training):
        h, output, v = hasty_pytorch_lib.lowrank_elman_forward(training, x, z, h0, W_x, U, V, b)
        ctx.save_for_backward(W_x, U, V, x, z, h, v)
        return output, h

    @staticmethod
    def backward(ctx, grad_output, _grad_h):
        W_x, U, V, x, z, h, v = ctx.saved_tensors
        if v.numel() == 0:
            raise RuntimeError("backward needs the pre-activations: run forward with training=True")
        dx, dz, dW_x, dU, dV, db = hasty_pytorch_lib.lowrank_elman_backward(
            W_x, U, V, x, z, h, v, grad_output.contiguous())
        return dx, dz, None, dW_x, dU, dV, db, None


class LowRankElmanCell(nn.Module):
    """E4 cell: W_x [dim, dim], U [dim, rank], V [rank, dim], b; U V rescaled to the given
    spectral radius by a three-step power iteration on the product, both factors taking the
    square root of the scale (elman/models/lowrank_elman.py:49-108)."""

    def __init__(self, dim, rank=64, spectral_radius=0.95):
        super().__init__()
        self.dim, self.rank, self.spectral_radius = dim, rank, spectral_radius
        self.W_x = nn.Parameter(torch.empty(dim, dim))
        self.U = nn.Parameter(torch.empty(dim, rank))
        self.V = nn.Parameter(torch.empty(rank, dim))
        self.b = nn.Parameter(torch.zeros(dim))
        nn.init.xavier_uniform_(self.W_x)
        nn.init.orthogonal_(self.U)
        nn.init.orthogonal_(self.V)
        with torch.no_grad():
            self.U.mul_(0.3)
            self.V.mul_(0.3)

    def get_UV(self):
        u = getattr(self, "_spectral_u", None)
        if u is None or u.shape[0] != self.dim:
            u = torch.randn(self.dim, device=self.U.device, dtype=self.U.dtype)
            u = u / u.norm()
        UV = self.U @ self.V
        with torch.no_grad():
            for _ in range(3):
                v = UV.T @ u
                v = v / (v.norm() + 1e-8)
                u = UV @ v
                u = u / (u.norm() + 1e-8)
            self._spectral_u = u
        sigma = (u @ UV @ v).abs()
        scale = self.spectral_radius / (sigma + 1e-8)
        return self.U * scale.sqrt(), self.V * scale.sqrt()

    def forward(self, x, z, h0=None):
        """x, z: [T, B, dim] -> (output [T, B, dim], h [T+1, B, dim])."""
        T, B, D = x.shape
        if not x.is_cuda:
            raise RuntimeError("elman_b200 runs on CUDA tensors only (no CPU fallback)")
        if h0 is None:
            h0 = torch.zeros(B, D, device=x.device, dtype=x.dtype)
        U, V = self.get_UV()
        return LowRankElmanFunction.apply(x.contiguous(), z.contiguous(), h0.contiguous(),
                                          self.W_x.contiguous(), U.contiguous(), V.contiguous(),
                                          self.b.contiguous(), self.training)


class LowRankElman(nn.Module):
    """E4 layer: x, z = split(in_proj(x)); x = silu(x); cell; out_proj
    (elman/models/lowrank_elman.py:163-254; rank defaults to dim / (2 expansion), floor 16)."""

    def __init__(self, dim, expansion=1.0, rank=None, spectral_radius=0.95, dropout=0.0, **kwargs):
        super().__init__()
        self.dim = dim
        self.d_inner = int(dim * expansion)
        if rank is None:
            rank = max(16, int(dim / (2 * expansion)))
        self.rank = rank
        self.in_proj = nn.Linear(dim, 2 * self.d_inner, bias=False)
        self.cell = LowRankElmanCell(self.d_inner, rank=rank, spectral_radius=spectral_radius)
        self.out_proj = nn.Linear(self.d_inner, dim, bias=False)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        nn.init.xavier_uniform_(self.in_proj.weight)
        nn.init.xavier_uniform_(self.out_proj.weight)

    def forward(self, x, h0=None, **kwargs):
        """x: [B,T,dim] -> (output [B,T,dim], h_final [B,d_inner])."""
        x_proj, z = self.in_proj(x).chunk(2, dim=-1)
        x_rnn = F.silu(x_proj).permute(1, 0, 2).contiguous()
        z_rnn = z.permute(1, 0, 2).contiguous()
        cell_out, h_all = self.cell(x_rnn, z_rnn, h0)
        y = self.dropout(cell_out.permute(1, 0, 2).contiguous())
        out = fused_ops.linear(y, self.out_proj.weight) if fused_ops.library_handles(y) \
            else self.out_proj(y)
        return out, h_all[-1]

    def extra_repr(self):
        return f"dim={self.dim}, d_inner={self.d_inner}, rank={self.rank}, LEVEL=4"


class E1HFunction(torch.autograd.Function):
    """forward(training, pre_x [B,T,H,N], z, h0 [B,H,N], W_h [H,N,N], b_h [H,N]) -> (output
    [B,T,H,N], h_final); the gradients of h0 and h_final are dropped
    (elman/models/e1_multihead.py:43-115)."""

    @staticmethod
    def forward(ctx, training, pre_x, z, h0, W_h, b_h):
        pre_x_t = pre_x.permute(1, 0, 2, 3).contiguous()
        z_t = z.permute(1, 0, 2, 3).contiguous()
        h_final, output_t, saved = hasty_pytorch_lib.e1h_forward(training, pre_x_t, z_t, h0, W_h, b_h)
        ctx.save_for_backward(pre_x_t, z_t, W_h, b_h, saved)
        return output_t.permute(1, 0, 2, 3).contiguous(), h_final

    @staticmethod
    def backward(ctx, d_output, _d_h_final):
        pre_x_t, z_t, W_h, b_h, saved = ctx.saved_tensors
        if saved.numel() == 0:
            raise RuntimeError("backward needs the saved states: run forward with training=True")
        d_pre, d_z, dW_rows, db_rows = hasty_pytorch_lib.e1h_backward(
            pre_x_t, z_t, W_h, b_h, saved, d_output.permute(1, 0, 2, 3).contiguous())
        return (None, d_pre.permute(1, 0, 2, 3).contiguous(), d_z.permute(1, 0, 2, 3).contiguous(),
                None, dW_rows.sum(dim=0).to(W_h.dtype), db_rows.sum(dim=0).to(b_h.dtype))


class E1MultiHead(nn.Module):
    """E1H layer: x, z = split(in_proj(x)); x = silu(x); per-head W_x; H independent Elman
    recurrences of size n_state with per-head W_h and b; gate silu(z); out_proj
    (elman/models/e1_multihead.py:118-283).  Unlike the reference's kernel (bf16, training mode
    only) the recurrence here runs for fp32 and bf16, training or not."""

    def __init__(self, dim, n_heads=16, n_state=32, expansion=1.0, dropout=0.0, mamba2_init=False,
                 **kwargs):
        super().__init__()
        self.dim, self.n_heads, self.n_state = dim, n_heads, n_state
        self.d_inner = n_heads * n_state
        self.in_proj = nn.Linear(dim, 2 * self.d_inner, bias=False)
        self.W_x = nn.Parameter(torch.empty(n_heads, n_state, n_state))
        self.W_h = nn.Parameter(torch.empty(n_heads, n_state, n_state))
        self.b = nn.Parameter(torch.zeros(n_heads, n_state))
        self.out_proj = nn.Linear(self.d_inner, dim, bias=False)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        if mamba2_init:
            nn.init.normal_(self.in_proj.weight, std=0.02)
            nn.init.normal_(self.out_proj.weight, std=0.02)
            nn.init.normal_(self.W_x, std=0.02)
        else:
            nn.init.xavier_uniform_(self.in_proj.weight)
            nn.init.xavier_uniform_(self.out_proj.weight)
        with torch.no_grad():
            for k in range(n_heads):
                w = torch.empty(n_state, n_state, dtype=torch.float32)
                nn.init.orthogonal_(w)
                self.W_h.data[k].copy_(w * (0.999 if mamba2_init else 0.9))
                if not mamba2_init:
                    nn.init.xavier_uniform_(self.W_x.data[k])

    def forward(self, x, h0=None, **kwargs):
        """x: [B,T,dim] -> (output [B,T,dim], h_final [B,H,n_state])."""
        B, T, D = x.shape
        Hh, N = self.n_heads, self.n_state
        if not x.is_cuda:
            raise RuntimeError("elman_b200 runs on CUDA tensors only (no CPU fallback)")
        x_proj, z = self.in_proj(x).chunk(2, dim=-1)
        x_proj = F.silu(x_proj).view(B, T, Hh, N)
        pre_x = torch.einsum("bthi,hij->bthj", x_proj, self.W_x)
        if h0 is None:
            h0 = torch.zeros(B, Hh, N, device=x.device, dtype=x.dtype)
        out, h_final = E1HFunction.apply(self.training, pre_x, z.reshape(B, T, Hh, N).contiguous(),
                                         h0.contiguous(), self.W_h, self.b)
        y = self.dropout(out.reshape(B, T, self.d_inner))
        proj = fused_ops.linear(y, self.out_proj.weight) if fused_ops.library_handles(y) \
            else self.out_proj(y)
        return proj, h_final

    def extra_repr(self):
        return (f"dim={self.dim}, n_heads={self.n_heads}, n_state={self.n_state}, "
                f"d_inner={self.d_inner}, LEVEL=E1H_MULTIHEAD")
