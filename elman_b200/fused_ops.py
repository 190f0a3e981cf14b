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
    def forward(ctx, x, residual_in, weight, eps):
        H = hasty_pytorch_lib
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
        return dx, dres_in, dw, None


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
        dW = H.gemm(H.GEMM_TN, dxz, u2)
        return du.view(*ctx.lead, u2.shape[-1]), dW


def linear(x, weight, bias=None):
    """y = x W^T (+ b) over the last dimension through the library's GEMMs."""
    from .mamba_gated_elman import LinearFunction
    return LinearFunction.apply(x, weight, bias)


def library_handles(x):
    """True when `x` can go through the library's layer ops (CUDA, fp32 or bf16)."""
    return x.is_cuda and x.dtype in (torch.float32, torch.bfloat16)
