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

from . import hasty_pytorch_lib
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
        x_proj, z = self.in_proj(x).chunk(2, dim=-1)
        if self.use_conv:
            x_proj = self.conv1d(x_proj.transpose(1, 2))[:, :, :T].transpose(1, 2)
        x_proj = F.silu(x_proj)
        x_rnn = x_proj.permute(1, 0, 2).contiguous()
        z_rnn = z.permute(1, 0, 2).contiguous()
        cell_out, h_all = self.cell(x_rnn, z_rnn, h0)
        y = self.dropout(cell_out.permute(1, 0, 2).contiguous())
        return self.out_proj(y), h_all[-1]

    def extra_repr(self):
        return f"dim={self.dim}, d_inner={self.d_inner}, use_conv={self.use_conv}, LEVEL=1_MAMBA_GATED"
