"""E0 — stock Elman layer with a learned, x-only output gate.

    h_t = tanh(W_x x_t + W_h h_{t-1} + b);   y_t = h_t * silu(W_gate x_t + b_gate)

Mirrors the reference interface (elman/models/stock_elman.py:29-271).
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import hasty_pytorch_lib
from ._spectral import spectrally_normalised


class StockElmanFunction(torch.autograd.Function):
    """forward(training, x, h0, W_x, W_h, W_gate, b, b_gate) -> (output, h)."""

    @staticmethod
    def forward(ctx, training, x, h0, W_x, W_h, W_gate, b, b_gate):
        h, output, v, gate_cache = hasty_pytorch_lib.stock_elman_forward(
            training, x.contiguous(), h0.contiguous(), W_x.contiguous(), W_h.contiguous(),
            W_gate.contiguous(), b.contiguous(), b_gate.contiguous())
        if training:
            ctx.save_for_backward(x, W_x, W_h, W_gate, b_gate, h, v, gate_cache)
        return output, h

    @staticmethod
    def backward(ctx, d_output, _dh):
        x, W_x, W_h, W_gate, b_gate, h, v, gate_cache = ctx.saved_tensors
        dx, dW_x, dW_h, dW_gate, db, db_gate = hasty_pytorch_lib.stock_elman_backward(
            W_x, W_h, W_gate, x.contiguous(), h, v, gate_cache, d_output.contiguous())
        return None, dx, None, dW_x, dW_h, dW_gate, db, db_gate


class StockElmanCell(nn.Module):
    """w_h_mode: 'free', 'spectral_norm' (default) or 'scaled_orthogonal'."""

    def __init__(self, dim, w_h_mode="spectral_norm", w_h_init_gain=1.0):
        super().__init__()
        self.dim = dim
        self.w_h_mode = w_h_mode
        self.w_h_init_gain = w_h_init_gain
        self.W_x = nn.Parameter(torch.empty(dim, dim))
        self.b = nn.Parameter(torch.zeros(dim))
        self.W_gate = nn.Parameter(torch.empty(dim, dim))
        self.b_gate = nn.Parameter(torch.zeros(dim))
        if w_h_mode == "scaled_orthogonal":
            self.register_buffer("W_h_base", torch.empty(dim, dim))
            self.w_h_log_scale = nn.Parameter(torch.tensor(-0.01))
        else:
            self.W_h = nn.Parameter(torch.empty(dim, dim))
        self._init_weights()

    def _init_weights(self):
        nn.init.xavier_uniform_(self.W_x)
        nn.init.xavier_uniform_(self.W_gate)
        if self.w_h_mode == "scaled_orthogonal":
            nn.init.orthogonal_(self.W_h_base)
        else:
            nn.init.xavier_uniform_(self.W_h, gain=self.w_h_init_gain)

    def get_W_h(self):
        if self.w_h_mode == "scaled_orthogonal":
            return torch.sigmoid(self.w_h_log_scale) * self.W_h_base
        if self.w_h_mode == "spectral_norm":
            return spectrally_normalised(self, self.W_h)
        return self.W_h

    def forward(self, x, h0=None):
        """x: [T,B,dim] -> (output [T,B,dim], h [T+1,B,dim])."""
        T, B, D = x.shape
        if not x.is_cuda:
            raise RuntimeError("elman_b200 runs on CUDA tensors only (no CPU fallback)")
        if h0 is None:
            h0 = torch.zeros(B, self.dim, device=x.device, dtype=x.dtype)
        return StockElmanFunction.apply(self.training, x, h0, self.W_x, self.get_W_h(),
                                        self.W_gate, self.b, self.b_gate)


class StockElman(nn.Module):
    """in_proj -> (conv + silu) -> cell -> out_proj."""

    def __init__(self, dim, expansion=1.0, dropout=0.0, r_h_mode="spectral_norm",
                 r_h_init_gain=1.0, use_conv=False, d_conv=4, **kwargs):
        super().__init__()
        self.dim = dim
        self.d_inner = int(dim * expansion)
        self.r_h_mode = r_h_mode
        self.use_conv = use_conv
        self.in_proj = nn.Linear(dim, self.d_inner, bias=False)
        if use_conv:
            self.conv1d = nn.Conv1d(self.d_inner, self.d_inner, kernel_size=d_conv,
                                    padding=d_conv - 1, groups=self.d_inner, bias=True)
        else:
            self.conv1d = None
        self.cell = StockElmanCell(self.d_inner, w_h_mode=r_h_mode, w_h_init_gain=r_h_init_gain)
        self.out_proj = nn.Linear(self.d_inner, dim, bias=False)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        nn.init.xavier_uniform_(self.in_proj.weight)
        nn.init.xavier_uniform_(self.out_proj.weight)

    def forward(self, x, h0=None, **kwargs):
        B, T, D = x.shape
        x_proj = self.in_proj(x)
        if self.use_conv and self.conv1d is not None:
            x_proj = F.silu(self.conv1d(x_proj.transpose(1, 2))[:, :, :T].transpose(1, 2))
        cell_out, h_all = self.cell(x_proj.permute(1, 0, 2).contiguous(), h0)
        y = self.dropout(cell_out.permute(1, 0, 2).contiguous())
        return self.out_proj(y), h_all[-1]

    # ---- time-chunked execution (LadderLM's layer/time pipeline), time-major [Tc,B,*] ----
    # E0 differs from E1 only in where the gate pre-activation comes from, so the chunk
    # pieces reuse E1's projection and recurrence nodes: pre = W_x x + b and the gate
    # g = W_gate x + b_gate are both time-parallel projections, and the recurrence
    # h_t = tanh(pre_t + W_h h_{t-1}), y_t = h_t silu(g_t) is the same kernel.
    @property
    def supports_time_chunks(self):
        return not self.use_conv

    def chunk_recurrence_blocks(self, dtype, T, B, flags=0):
        """Thread blocks one recurrence launch of this layer keeps resident (0: cooperative)."""
        return hasty_pytorch_lib.recurrence_blocks(dtype, T, B, self.d_inner, flags)

    def chunk_weights(self):
        return self.cell.get_W_h().contiguous()

    def chunk_pre(self, x, W_h, link):
        from . import fused_ops
        from .mamba_gated_elman import E1ChunkProjectionFunction, LinearFunction
        cell = self.cell
        x_proj = (fused_ops.linear(x.contiguous(), self.in_proj.weight)
                  if fused_ops.library_handles(x) else self.in_proj(x).contiguous())
        pre = E1ChunkProjectionFunction.apply(x_proj, cell.W_x.contiguous(), cell.b.contiguous(),
                                              W_h, link)
        gate = LinearFunction.apply(x_proj, cell.W_gate.contiguous(), cell.b_gate.contiguous())
        return pre, gate

    def chunk_rec(self, pre, gate, h0, W_h, link, flags=0, W_h_T=None):
        from .mamba_gated_elman import E1ChunkRecurrenceFunction
        return E1ChunkRecurrenceFunction.apply(pre, gate, h0.contiguous(), W_h, link, flags, W_h_T)

    def chunk_post(self, cell_out):
        from . import fused_ops
        y = self.dropout(cell_out)
        return (fused_ops.linear(y, self.out_proj.weight) if fused_ops.library_handles(y)
                else self.out_proj(y))

    def extra_repr(self):
        return f"dim={self.dim}, d_inner={self.d_inner}, LEVEL=0_STOCK"
