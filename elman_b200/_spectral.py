"""Spectral normalisation of the recurrent matrix, shared by the E0 and E1 cells.

Same arithmetic as the reference cells' get_W_h
(elman/models/mamba_gated_elman.py:123-146, elman/models/stock_elman.py:104-125):
three power-iteration steps without gradient from a persistent vector u, then
W_h * (0.99 / (|u^T W_h v| + 1e-8)) with the gradient flowing through sigma.

On CUDA tensors the whole of it is ONE kernel of the library per direction
(elman_spectral_norm_forward / _backward: a thread-block cluster per matrix, fp32 arithmetic)
behind an autograd node; `FUSED = False` (or a tensor the library does not take) selects the
same steps as framework ops.
"""
import torch

from . import hasty_pytorch_lib

TARGET_RADIUS = 0.99
POWER_ITERS = 3
EPS = 1e-8
FUSED = True


class SpectralNormFunction(torch.autograd.Function):
    """forward(W, u) -> W_eff; u is advanced in place.  backward: the gradient of W with u and v
    held constant (the reference runs its iteration under no_grad and differentiates
    |u^T W v| only through W)."""

    @staticmethod
    def forward(ctx, W, u):
        W_eff, v, sigma = hasty_pytorch_lib.spectral_norm_forward(W.contiguous(), u, TARGET_RADIUS,
                                                                  EPS, POWER_ITERS)
        ctx.save_for_backward(W, v, sigma, u.clone())   # u as this pass left it
        return W_eff

    @staticmethod
    def backward(ctx, dW_eff):
        W, v, sigma, u = ctx.saved_tensors
        dW = hasty_pytorch_lib.spectral_norm_backward(W.contiguous(), u, v, sigma,
                                                      dW_eff.contiguous(), TARGET_RADIUS, EPS)
        return dW, None


def _library_takes(W_h: torch.Tensor) -> bool:
    return (FUSED and W_h.device.type == "cuda" and W_h.dim() == 2
            and W_h.dtype in (torch.float32, torch.bfloat16))


def spectrally_normalised(module, W_h: torch.Tensor) -> torch.Tensor:
    dim = W_h.shape[0]
    u = getattr(module, "_spectral_u", None)
    if u is None or u.shape[0] != dim:
        u = torch.randn(dim, device=W_h.device, dtype=W_h.dtype)
        u = u / u.norm()
    if _library_takes(W_h):
        # keep the vector in place once it exists: a captured CUDA graph then reads and
        # advances the same buffer on every replay
        if u.device != W_h.device or u.dtype != W_h.dtype or not u.is_contiguous():
            u = u.to(device=W_h.device, dtype=W_h.dtype).contiguous()
        module._spectral_u = u
        return SpectralNormFunction.apply(W_h, u)
    with torch.no_grad():
        for _ in range(POWER_ITERS):
            v = W_h.T @ u
            v = v / (v.norm() + EPS)
            u = W_h @ v
            u = u / (u.norm() + EPS)
        if getattr(module, "_spectral_u", None) is not None and module._spectral_u.shape == u.shape \
                and module._spectral_u.device == u.device and module._spectral_u.dtype == u.dtype:
            module._spectral_u.copy_(u)
            u = module._spectral_u
        else:
            module._spectral_u = u
    sigma = (u @ W_h @ v).abs()
    return W_h * (TARGET_RADIUS / (sigma + EPS))
