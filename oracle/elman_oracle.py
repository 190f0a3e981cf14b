"""CPU oracle for the E0 / E1 / E5 Elman-layer recurrence (TEST INFRASTRUCTURE ONLY).

This module restates, in plain PyTorch on the CPU, the algorithm the reference
implements for the three layer cells on the hot path.  It is the checker the
GPU kernels are compared with; it is never part of the shipped compute path.
Only the test-suite, the smoke entry point and the benchmark's CPU-baseline leg
import it.

Parity status: PINNED.  `tests/golden/make_golden.py` runs the reference's own
Python cells (imported from a checkout of the reference) on seeded inputs and
stores their outputs and gradients; `tests/test_oracle_golden.py` checks every
function here against those files.

Reference lines each function follows (paths relative to the reference repo):

* E1 forward  : elman/models/mamba_gated_elman.py:180-199 (Python loop) and
                elman/cuda/lib/mamba_gated_elman_gpu.cu.cc:440-473 (GEMM + fused
                tanh/gate kernel, same math).
* E1 backward : elman/cuda/lib/mamba_gated_elman_gpu.cu.cc:527-592 (BPTT loop and
                the three batch GEMMs); the autograd.Function drops the gradient
                of the returned h (elman/models/mamba_gated_elman.py:42-47).
* E0 forward  : elman/models/stock_elman.py:157-180; backward
                elman/cuda/lib/stock_elman_gpu.cu.cc:322-472.
* E5 forward  : elman/models/pure_lowrank_elman.py:214-248; backward
                elman/cuda/lib/pure_lowrank_elman_fused_gpu.cu.cc:295-505.
* E33 forward : elman/models/e33_self_gate.py:170-193 (self gate y = h silu(h)); backward
                by the chain rule of that loop (its CUDA pair: elman_ladder.cc:444-557).

All functions take time-major tensors x[T,B,d] and return dictionaries of
tensors in the dtype they were given (use float64 inputs for error bars).
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch

Tensor = torch.Tensor


# ----------------------------------------------------------------------------
# elementwise pieces
# ----------------------------------------------------------------------------

def silu(z: Tensor) -> Tensor:
    return z * torch.sigmoid(z)


def dsilu(z: Tensor) -> Tensor:
    """d/dz silu(z) = s(z)·(1 + z·(1 − s(z))); mamba_gated_elman_gpu.cu.cc:321-323."""
    s = torch.sigmoid(z)
    return s * (1.0 + z * (1.0 - s))


# ----------------------------------------------------------------------------
# E1 : h_t = tanh(W_x x_t + W_h h_{t-1} + b),  y_t = h_t · silu(z_t)
# ----------------------------------------------------------------------------

def e1_forward(x: Tensor, z: Tensor, h0: Tensor, W_x: Tensor, W_h: Tensor,
               b: Tensor) -> Dict[str, Tensor]:
    """Returns h[T+1,B,d] (h[0]=h0), output[T,B,d], v[T,B,d] (pre-activation)."""
    T = x.shape[0]
    h = [h0]
    ys, vs = [], []
    for t in range(T):
        raw = x[t] @ W_x.T + h[-1] @ W_h.T + b
        hn = torch.tanh(raw)
        h.append(hn)
        vs.append(raw)
        ys.append(hn * silu(z[t]))
    return {"h": torch.stack(h), "output": torch.stack(ys), "v": torch.stack(vs)}


def e1_backward(W_x: Tensor, W_h: Tensor, x: Tensor, z: Tensor, h: Tensor,
                v: Tensor, d_output: Tensor, dv_in: Tensor = None) -> Dict[str, Tensor]:
    """Explicit BPTT in the order of the reference's backward Run().

    The gradient of the returned hidden-state sequence is not an input: the
    reference Function ignores it.  `dv_in` ([B,d], optional) is not part of the
    reference either: when a sequence is processed in time chunks it carries the
    pre-activation gradient of the first step of the following chunk, which is
    all the loop below needs from the future (dh_rec = dv_{t+1} W_h); the
    result's "dv0" is what the preceding chunk takes as its `dv_in`.
    """
    T, B, d = x.shape
    dv_all = torch.zeros_like(x)
    dz = torch.zeros_like(z)
    dh_rec = torch.zeros(B, d, dtype=x.dtype) if dv_in is None else dv_in @ W_h
    for t in range(T - 1, -1, -1):
        h_t = h[t + 1]
        dh = d_output[t] * silu(z[t]) + dh_rec
        dz[t] = d_output[t] * h_t * dsilu(z[t])
        th = torch.tanh(v[t])
        dv = dh * (1.0 - th * th)
        dv_all[t] = dv
        dh_rec = dv @ W_h
    dv2 = dv_all.reshape(T * B, d)
    return {
        "dx": (dv2 @ W_x).reshape(T, B, d),
        "dz": dz,
        "dW_x": dv2.T @ x.reshape(T * B, d),
        "dW_h": dv2.T @ h[:T].reshape(T * B, d),
        "db": dv2.sum(0),
        "dv0": dv_all[0] if T > 0 else dv_in,
    }


# ----------------------------------------------------------------------------
# E0 : h_t as E1,  y_t = h_t · silu(W_gate x_t + b_gate)
# ----------------------------------------------------------------------------

def e0_forward(x: Tensor, h0: Tensor, W_x: Tensor, W_h: Tensor, W_gate: Tensor,
               b: Tensor, b_gate: Tensor) -> Dict[str, Tensor]:
    T = x.shape[0]
    h = [h0]
    ys, vs, gs = [], [], []
    for t in range(T):
        raw = x[t] @ W_x.T + h[-1] @ W_h.T + b
        hn = torch.tanh(raw)
        h.append(hn)
        vs.append(raw)
        g = x[t] @ W_gate.T + b_gate
        gs.append(g)
        ys.append(hn * silu(g))
    return {"h": torch.stack(h), "output": torch.stack(ys), "v": torch.stack(vs),
            "gate_cache": torch.stack(gs)}


def e0_backward(W_x: Tensor, W_h: Tensor, W_gate: Tensor, x: Tensor, h: Tensor,
                v: Tensor, gate_cache: Tensor, d_output: Tensor) -> Dict[str, Tensor]:
    T, B, d = x.shape
    dv_all = torch.zeros_like(x)
    dg_all = torch.zeros_like(x)
    dh_rec = torch.zeros(B, d, dtype=x.dtype)
    for t in range(T - 1, -1, -1):
        g = gate_cache[t]
        dh = d_output[t] * silu(g) + dh_rec
        dg_all[t] = d_output[t] * h[t + 1] * dsilu(g)
        th = torch.tanh(v[t])
        dv = dh * (1.0 - th * th)
        dv_all[t] = dv
        dh_rec = dv @ W_h
    dv2 = dv_all.reshape(T * B, d)
    dg2 = dg_all.reshape(T * B, d)
    x2 = x.reshape(T * B, d)
    return {
        "dx": (dv2 @ W_x + dg2 @ W_gate).reshape(T, B, d),
        "dW_x": dv2.T @ x2,
        "dW_h": dv2.T @ h[:T].reshape(T * B, d),
        "dW_gate": dg2.T @ x2,
        "db": dv2.sum(0),
        "db_gate": dg2.sum(0),
    }


# ----------------------------------------------------------------------------
# E5 : h_t = tanh(U_h V_h h_{t-1} + U_x V_x x_t + b),  y_t = h_t · silu(U_z V_z x_t)
# ----------------------------------------------------------------------------

def e5_forward(x: Tensor, h0: Tensor, U_h: Tensor, V_h: Tensor, U_x: Tensor,
               V_x: Tensor, U_z: Tensor, V_z: Tensor, b: Tensor) -> Dict[str, Tensor]:
    T = x.shape[0]
    h = [h0]
    ys, vs = [], []
    for t in range(T):
        Uh = (h[-1] @ V_h.T) @ U_h.T
        Ux = (x[t] @ V_x.T) @ U_x.T
        pre = Uh + Ux + b
        hn = torch.tanh(pre)
        h.append(hn)
        vs.append(pre)
        Uz = (x[t] @ V_z.T) @ U_z.T
        ys.append(hn * silu(Uz))
    return {"h": torch.stack(h), "output": torch.stack(ys), "v": torch.stack(vs)}


def e5_backward(U_h: Tensor, V_h: Tensor, U_x: Tensor, V_x: Tensor, U_z: Tensor,
                V_z: Tensor, x: Tensor, h: Tensor, v: Tensor,
                d_output: Tensor, dv_in: Tensor = None) -> Dict[str, Tensor]:
    """BPTT with the weight gradients taken as batched products over all steps
    (the reference accumulates the same sums one step at a time).  `dv_in` / "dv0":
    the time-chunk carry, as in e1_backward (not part of the reference)."""
    T, B, d = x.shape
    x2 = x.reshape(T * B, d)
    Vz = x2 @ V_z.T                      # [TB, r]
    UVz = (Vz @ U_z.T).reshape(T, B, d)   # gate pre-activation, recomputed
    dv_all = torch.zeros_like(x)
    dg_all = torch.zeros_like(x)
    dh_rec = torch.zeros(B, d, dtype=x.dtype) if dv_in is None else (dv_in @ U_h) @ V_h
    for t in range(T - 1, -1, -1):
        g = UVz[t]
        dh = d_output[t] * silu(g) + dh_rec
        dg_all[t] = d_output[t] * h[t + 1] * dsilu(g)
        th = torch.tanh(v[t])
        dv = dh * (1.0 - th * th)
        dv_all[t] = dv
        dh_rec = (dv @ U_h) @ V_h
    dv2 = dv_all.reshape(T * B, d)
    dg2 = dg_all.reshape(T * B, d)
    hp = h[:T].reshape(T * B, d)
    Vx = x2 @ V_x.T
    Vh = hp @ V_h.T
    dVx = dv2 @ U_x                      # [TB, r]
    dVz = dg2 @ U_z
    dVh = dv2 @ U_h
    return {
        "dx": (dVx @ V_x + dVz @ V_z).reshape(T, B, d),
        "dU_h": dv2.T @ Vh,
        "dV_h": dVh.T @ hp,
        "dU_x": dv2.T @ Vx,
        "dV_x": dVx.T @ x2,
        "dU_z": dg2.T @ Vz,
        "dV_z": dVz.T @ x2,
        "db": dv2.sum(0),
        "dv0": dv_all[0] if T > 0 else dv_in,
    }


# ----------------------------------------------------------------------------
# E33 : h_t as E1,  y_t = h_t · silu(h_t)   (elman/models/e33_self_gate.py:144-193;
#       its CUDA pair e33_self_gate_forward/backward, elman_ladder.cc:444-557)
# ----------------------------------------------------------------------------

def e33_forward(x: Tensor, h0: Tensor, W_x: Tensor, W_h: Tensor, b: Tensor) -> Dict[str, Tensor]:
    T = x.shape[0]
    h = [h0]
    ys, vs = [], []
    for t in range(T):
        raw = x[t] @ W_x.T + h[-1] @ W_h.T + b
        hn = torch.tanh(raw)
        h.append(hn)
        vs.append(raw)
        ys.append(hn * silu(hn))
    return {"h": torch.stack(h), "output": torch.stack(ys), "v": torch.stack(vs)}


def e33_backward(W_x: Tensor, W_h: Tensor, x: Tensor, h: Tensor, v: Tensor,
                 d_output: Tensor) -> Dict[str, Tensor]:
    T, B, d = x.shape
    dv_all = torch.zeros_like(x)
    dh_rec = torch.zeros(B, d, dtype=x.dtype)
    for t in range(T - 1, -1, -1):
        h_t = h[t + 1]
        dh = d_output[t] * (silu(h_t) + h_t * dsilu(h_t)) + dh_rec
        th = torch.tanh(v[t])
        dv = dh * (1.0 - th * th)
        dv_all[t] = dv
        dh_rec = dv @ W_h
    dv2 = dv_all.reshape(T * B, d)
    return {"dx": (dv2 @ W_x).reshape(T, B, d), "dW_x": dv2.T @ x.reshape(T * B, d),
            "dW_h": dv2.T @ h[:T].reshape(T * B, d), "db": dv2.sum(0)}


# ----------------------------------------------------------------------------
# E4: E1 with a low-rank recurrent matrix W_h = U V
# (elman/models/lowrank_elman.py:134-160 of the reference, the Python time loop; the
#  backward is the BPTT its CUDA pair lowrank_elman_forward/backward implements,
#  elman_ladder.cc:2665-2800)
# ----------------------------------------------------------------------------

def e4_forward(x: Tensor, z: Tensor, h0: Tensor, W_x: Tensor, U: Tensor, V: Tensor,
               b: Tensor) -> Dict[str, Tensor]:
    T = x.shape[0]
    h = [h0]
    ys, vs = [], []
    for t in range(T):
        raw = x[t] @ W_x.T + (h[-1] @ V.T) @ U.T + b
        hn = torch.tanh(raw)
        h.append(hn)
        vs.append(raw)
        ys.append(hn * silu(z[t]))
    return {"h": torch.stack(h), "output": torch.stack(ys), "v": torch.stack(vs)}


def e4_backward(W_x: Tensor, U: Tensor, V: Tensor, x: Tensor, z: Tensor, h: Tensor, v: Tensor,
                d_output: Tensor) -> Dict[str, Tensor]:
    T, B, d = x.shape
    dv_all = torch.zeros_like(x)
    dz = torch.zeros_like(x)
    dh_rec = torch.zeros(B, d, dtype=x.dtype)
    for t in range(T - 1, -1, -1):
        h_t = h[t + 1]
        dz[t] = d_output[t] * h_t * dsilu(z[t])
        dh = d_output[t] * silu(z[t]) + dh_rec
        th = torch.tanh(v[t])
        dv = dh * (1.0 - th * th)
        dv_all[t] = dv
        dh_rec = (dv @ U) @ V
    dv2 = dv_all.reshape(T * B, d)
    hp = h[:T].reshape(T * B, d)
    return {"dx": (dv2 @ W_x).reshape(T, B, d), "dz": dz, "dW_x": dv2.T @ x.reshape(T * B, d),
            "dU": dv2.T @ (hp @ V.T), "dV": (dv2 @ U).T @ hp, "db": dv2.sum(0)}


# ----------------------------------------------------------------------------
# E1H: H independent heads of size N (elman/models/e1_multihead.py:204-211 of the reference,
# the Python time loop: wh = einsum('bhi,hij->bhj', h_prev, W_h); the backward is the BPTT of
# its CUDA pair e1h_forward/backward, elman_ladder.cc:14610-14730)
# ----------------------------------------------------------------------------

def e1h_forward(pre_x: Tensor, z: Tensor, h0: Tensor, W_h: Tensor, b: Tensor) -> Dict[str, Tensor]:
    """pre_x, z: [T,B,H,N]; h0: [B,H,N]; W_h: [H,N,N]; b: [H,N]."""
    T = pre_x.shape[0]
    h = [h0]
    ys, vs = [], []
    for t in range(T):
        raw = pre_x[t] + torch.einsum("bhi,hij->bhj", h[-1], W_h) + b
        hn = torch.tanh(raw)
        h.append(hn)
        vs.append(raw)
        ys.append(hn * silu(z[t]))
    return {"h": torch.stack(h), "output": torch.stack(ys), "v": torch.stack(vs)}


def e1h_backward(z: Tensor, W_h: Tensor, h: Tensor, v: Tensor, d_output: Tensor) -> Dict[str, Tensor]:
    T = z.shape[0]
    d_pre = torch.zeros_like(z)
    dz = torch.zeros_like(z)
    dh_rec = torch.zeros_like(h[0])
    dW = torch.zeros_like(W_h)
    for t in range(T - 1, -1, -1):
        h_t = h[t + 1]
        dz[t] = d_output[t] * h_t * dsilu(z[t])
        dh = d_output[t] * silu(z[t]) + dh_rec
        th = torch.tanh(v[t])
        dv = dh * (1.0 - th * th)
        d_pre[t] = dv
        dW += torch.einsum("bhi,bhj->hij", h[t], dv)
        dh_rec = torch.einsum("bhj,hij->bhi", dv, W_h)
    return {"d_pre_x": d_pre, "dz": dz, "dW_h": dW, "db": d_pre.sum((0, 1))}


# ----------------------------------------------------------------------------
# E1 with the README's gate  y_t = h_t · silu(W_g [h_t ; x_t] + b_g)
# (README.md:25-29 of the reference; no class in the reference implements it,
#  so this one function is "parity unpinned" by reference code.)
# ----------------------------------------------------------------------------

def e1_hx_gate_forward(x: Tensor, h0: Tensor, W_x: Tensor, W_h: Tensor, b: Tensor,
                       W_g: Tensor, b_g: Tensor) -> Dict[str, Tensor]:
    T, B, d = x.shape
    W_gh, W_gx = W_g[:, :d], W_g[:, d:]
    h = [h0]
    ys, vs, zs = [], [], []
    for t in range(T):
        raw = x[t] @ W_x.T + h[-1] @ W_h.T + b
        hn = torch.tanh(raw)
        h.append(hn)
        vs.append(raw)
        zz = hn @ W_gh.T + x[t] @ W_gx.T + b_g
        zs.append(zz)
        ys.append(hn * silu(zz))
    return {"h": torch.stack(h), "output": torch.stack(ys), "v": torch.stack(vs),
            "z": torch.stack(zs)}


# ----------------------------------------------------------------------------
# autograd cross-check helpers (the reference's CPU path uses autograd for BPTT)
# ----------------------------------------------------------------------------

def e1_autograd(x, z, h0, W_x, W_h, b, d_output) -> Dict[str, Tensor]:
    leaves = [t.detach().clone().requires_grad_(True) for t in (x, z, W_x, W_h, b)]
    xx, zz, wx, wh, bb = leaves
    out = e1_forward(xx, zz, h0, wx, wh, bb)
    (out["output"] * d_output).sum().backward()
    return {"h": out["h"].detach(), "output": out["output"].detach(), "v": out["v"].detach(),
            "dx": xx.grad, "dz": zz.grad, "dW_x": wx.grad, "dW_h": wh.grad, "db": bb.grad}


def e0_autograd(x, h0, W_x, W_h, W_gate, b, b_gate, d_output) -> Dict[str, Tensor]:
    leaves = [t.detach().clone().requires_grad_(True) for t in (x, W_x, W_h, W_gate, b, b_gate)]
    xx, wx, wh, wg, bb, bg = leaves
    out = e0_forward(xx, h0, wx, wh, wg, bb, bg)
    (out["output"] * d_output).sum().backward()
    return {"h": out["h"].detach(), "output": out["output"].detach(), "v": out["v"].detach(),
            "gate_cache": out["gate_cache"].detach(),
            "dx": xx.grad, "dW_x": wx.grad, "dW_h": wh.grad, "dW_gate": wg.grad,
            "db": bb.grad, "db_gate": bg.grad}


def e5_autograd(x, h0, U_h, V_h, U_x, V_x, U_z, V_z, b, d_output) -> Dict[str, Tensor]:
    leaves = [t.detach().clone().requires_grad_(True)
              for t in (x, U_h, V_h, U_x, V_x, U_z, V_z, b)]
    xx, uh, vh, ux, vx, uz, vz, bb = leaves
    out = e5_forward(xx, h0, uh, vh, ux, vx, uz, vz, bb)
    (out["output"] * d_output).sum().backward()
    return {"h": out["h"].detach(), "output": out["output"].detach(), "v": out["v"].detach(),
            "dx": xx.grad, "dU_h": uh.grad, "dV_h": vh.grad, "dU_x": ux.grad,
            "dV_x": vx.grad, "dU_z": uz.grad, "dV_z": vz.grad, "db": bb.grad}


# ----------------------------------------------------------------------------
# seeded synthetic inputs (the benchmark's shapes and value distributions)
# ----------------------------------------------------------------------------

def _spectral_radius(W: Tensor) -> float:
    return float(torch.linalg.eigvals(W.double()).abs().max())


def make_e1_inputs(T: int, B: int, d: int, seed: int = 1234,
                   dtype: torch.dtype = torch.float32,
                   radius: float = 0.9) -> Dict[str, Tensor]:
    """x~N(0,1); W_x,W_h~N(0,1/d) with W_h rescaled to spectral radius `radius`;
    b=0; gate weights W_g[d,2d]~N(0,1/(2d)), b_g=0; z = x·W_gxᵀ + b_g; h0=0;
    d_output r~N(0,1).  For bf16 every tensor is rounded to bf16 first."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, B, d, generator=g)
    W_x = torch.randn(d, d, generator=g) / math.sqrt(d)
    W_h = torch.randn(d, d, generator=g) / math.sqrt(d)
    W_h = W_h * (radius / _spectral_radius(W_h))
    b = torch.zeros(d)
    W_g = torch.randn(d, 2 * d, generator=g) / math.sqrt(2 * d)
    b_g = torch.zeros(d)
    r = torch.randn(T, B, d, generator=g)
    h0 = torch.zeros(B, d)
    z = (x.reshape(T * B, d) @ W_g[:, d:].T + b_g).reshape(T, B, d)
    out = {"x": x, "z": z, "h0": h0, "W_x": W_x, "W_h": W_h, "b": b,
           "W_g": W_g, "b_g": b_g, "d_output": r}
    return {k: v.to(dtype) for k, v in out.items()}


def make_e0_inputs(T: int, B: int, d: int, seed: int = 1234,
                   dtype: torch.dtype = torch.float32) -> Dict[str, Tensor]:
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, B, d, generator=g)
    W_x = torch.randn(d, d, generator=g) / math.sqrt(d)
    W_h = torch.randn(d, d, generator=g) / math.sqrt(d)
    W_h = W_h * (0.9 / _spectral_radius(W_h))
    W_gate = torch.randn(d, d, generator=g) / math.sqrt(d)
    b = 0.1 * torch.randn(d, generator=g)
    b_gate = 0.1 * torch.randn(d, generator=g)
    r = torch.randn(T, B, d, generator=g)
    out = {"x": x, "h0": torch.zeros(B, d), "W_x": W_x, "W_h": W_h, "W_gate": W_gate,
           "b": b, "b_gate": b_gate, "d_output": r}
    return {k: v.to(dtype) for k, v in out.items()}


def make_e5_inputs(T: int, B: int, d: int, rank: int, seed: int = 1234,
                   dtype: torch.dtype = torch.float32) -> Dict[str, Tensor]:
    """U[d,r], V[r,d] ~ N(0, 1/sqrt(d·r)); U_h, V_h each scaled by
    sqrt(0.9/rho(V_h U_h)) so that U_h V_h has spectral radius 0.9."""
    g = torch.Generator().manual_seed(seed)
    s = (d * rank) ** -0.25
    x = torch.randn(T, B, d, generator=g)
    mats = {}
    for name in ("h", "x", "z"):
        mats["U_" + name] = torch.randn(d, rank, generator=g) * s
        mats["V_" + name] = torch.randn(rank, d, generator=g) * s
    rho = _spectral_radius(mats["V_h"] @ mats["U_h"])
    sc = math.sqrt(0.9 / rho)
    mats["U_h"] = mats["U_h"] * sc
    mats["V_h"] = mats["V_h"] * sc
    b = torch.zeros(d)
    r = torch.randn(T, B, d, generator=g)
    out = {"x": x, "h0": torch.zeros(B, d), **mats, "b": b, "d_output": r}
    return {k: v.to(dtype) for k, v in out.items()}


def rel_err(a: Tensor, ref: Tensor) -> float:
    """Norm-wise relative error ||a-ref||_2 / ||ref||_2 (in float64)."""
    a = a.detach().double().cpu()
    ref = ref.detach().double().cpu()
    den = float(ref.norm())
    if den == 0.0:
        return float((a - ref).norm())
    return float((a - ref).norm() / den)
