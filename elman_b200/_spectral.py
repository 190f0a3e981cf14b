"""Spectral normalisation of the recurrent matrix, shared by the E0 and E1 cells.

Same arithmetic as the reference cells' get_W_h
(elman/models/mamba_gated_elman.py:123-146, elman/models/stock_elman.py:104-125):
three power-iteration steps without gradient from a persistent vector u, then
W_h * (0.99 / (|u^T W_h v| + 1e-8)) with the gradient flowing through sigma.
"""
import torch

TARGET_RADIUS = 0.99
POWER_ITERS = 3
EPS = 1e-8


def spectrally_normalised(module, W_h: torch.Tensor) -> torch.Tensor:
    dim = W_h.shape[0]
    u = getattr(module, "_spectral_u", None)
    if u is None or u.shape[0] != dim:
        u = torch.randn(dim, device=W_h.device, dtype=W_h.dtype)
        u = u / u.norm()
    with torch.no_grad():
        for _ in range(POWER_ITERS):
            v = W_h.T @ u
            v = v / (v.norm() + EPS)
            u = W_h @ v
            u = u / (u.norm() + EPS)
        # keep the vector in place once it exists: a captured CUDA graph then reads
        # and advances the same buffer on every replay
        if getattr(module, "_spectral_u", None) is not None and module._spectral_u.shape == u.shape \
                and module._spectral_u.device == u.device and module._spectral_u.dtype == u.dtype:
            module._spectral_u.copy_(u)
            u = module._spectral_u
        else:
            module._spectral_u = u
    sigma = (u @ W_h @ v).abs()
    return W_h * (TARGET_RADIUS / (sigma + EPS))
