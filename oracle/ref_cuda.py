"""TEST INFRASTRUCTURE ONLY — the reference's own CUDA kernels, callable from Python.

Loads oracle/_ref/libelman_ref_cuda.so (built by oracle/build_ref.py from the
reference's unmodified sources) and exposes the six hot-path entry points with
the tensor allocation the reference's pybind11 layer performs
(elman/cuda/pytorch/elman_ladder.cc:22-281, :2956-3103): outputs from
torch.empty, weight gradients from torch.zeros, h[0] = h0, and workspaces of the
sizes computed there.  Used by the GPU tests as a second oracle (the reference's
bf16 rounding points) and by `bench.py --impl reference_cuda`.
"""
from __future__ import annotations

import ctypes
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "libelman_ref_cuda.so")
_lib = None
_DT = {torch.float32: 0, torch.bfloat16: 1}


def available() -> bool:
    return os.path.exists(LIB_PATH)


def load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIB_PATH)
        for name in ("ref_e1_forward", "ref_e1_backward", "ref_e0_forward", "ref_e0_backward",
                     "ref_e5_forward", "ref_e5_backward"):
            getattr(_lib, name).restype = None
    return _lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None and t.numel() else 0)


def _st(x):
    return ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)


def e1_forward(training, x, z, h0, W_x, W_h, b):
    T, B, d = x.shape
    o = dict(dtype=x.dtype, device=x.device)
    h = torch.empty(T + 1, B, d, **o); out = torch.empty(T, B, d, **o)
    v = torch.empty(T, B, d, **o) if training else torch.empty(0, **o)
    ws = torch.empty(T * B * d + B * d, **o)
    h[0] = h0
    load().ref_e1_forward(_DT[x.dtype], int(training), T, B, d, _p(W_x), _p(W_h), _p(b), _p(x),
                          _p(z), _p(h), _p(out), _p(v), _p(ws), _st(x))
    return h, out, v, ws


def e1_backward(W_x, W_h, x, z, h, v, dy):
    T, B, d = x.shape
    o = dict(dtype=x.dtype, device=x.device)
    dx = torch.empty_like(x); dz = torch.empty_like(z)
    dWx = torch.zeros(d, d, **o); dWh = torch.zeros(d, d, **o); db = torch.zeros(d, **o)
    ws = torch.empty((T + 2) * B * d + 2 * d, **o)
    load().ref_e1_backward(_DT[x.dtype], T, B, d, _p(W_x), _p(W_h), _p(x), _p(z), _p(h), _p(v),
                           _p(dy), _p(dx), _p(dz), _p(dWx), _p(dWh), _p(db), _p(ws), _st(x))
    return dx, dz, dWx, dWh, db, ws


def e0_forward(training, x, h0, W_x, W_h, W_gate, b, b_gate):
    T, B, d = x.shape
    o = dict(dtype=x.dtype, device=x.device)
    h = torch.empty(T + 1, B, d, **o); out = torch.empty(T, B, d, **o)
    v = torch.empty(T, B, d, **o); gc = torch.empty(T, B, d, **o)
    ws = torch.empty(2 * T * B * d + B * d, **o)
    h[0] = h0
    load().ref_e0_forward(_DT[x.dtype], int(training), T, B, d, _p(W_x), _p(W_h), _p(W_gate), _p(b),
                          _p(b_gate), _p(x), _p(h), _p(out), _p(v), _p(gc), _p(ws), _st(x))
    return h, out, v, gc, ws


def e0_backward(W_x, W_h, W_gate, x, h, v, gc, dy):
    T, B, d = x.shape
    o = dict(dtype=x.dtype, device=x.device)
    dx = torch.empty_like(x)
    dWx, dWh, dWg = (torch.zeros(d, d, **o) for _ in range(3))
    db, dbg = (torch.zeros(d, **o) for _ in range(2))
    ws = torch.empty((2 * T + 2) * B * d + 4 * d, **o)
    load().ref_e0_backward(_DT[x.dtype], T, B, d, _p(W_x), _p(W_h), _p(W_gate), _p(x), _p(h), _p(v),
                           _p(gc), _p(dy), _p(dx), _p(dWx), _p(dWh), _p(dWg), _p(db), _p(dbg),
                           _p(ws), _st(x))
    return dx, dWx, dWh, dWg, db, dbg, ws


def e5_forward(training, x, h0, U_h, V_h, U_x, V_x, U_z, V_z, b):
    T, B, d = x.shape
    r = U_h.shape[1]
    o = dict(dtype=x.dtype, device=x.device)
    h = torch.empty(T + 1, B, d, **o); out = torch.empty(T, B, d, **o)
    v = torch.empty(T, B, d, **o)
    ws = torch.empty(2 * T * B * r + 2 * T * B * d + B * r + B * d, **o)
    h[0] = h0
    load().ref_e5_forward(_DT[x.dtype], int(training), T, B, d, r, _p(U_h), _p(V_h), _p(U_x),
                          _p(V_x), _p(U_z), _p(V_z), _p(b), _p(x), _p(h), _p(out), _p(v), _p(ws),
                          _st(x))
    return h, out, v, ws


def e5_backward(U_h, V_h, U_x, V_x, U_z, V_z, x, h, v, dy):
    T, B, d = x.shape
    r = U_h.shape[1]
    o = dict(dtype=x.dtype, device=x.device)
    dx = torch.empty_like(x)
    dU = [torch.zeros(d, r, **o) for _ in range(3)]
    dV = [torch.zeros(r, d, **o) for _ in range(3)]
    db = torch.zeros(d, **o)
    ws = torch.empty(5 * B * d + 7 * B * r + 2 * d, **o)
    load().ref_e5_backward(_DT[x.dtype], T, B, d, r, _p(U_h), _p(V_h), _p(U_x), _p(V_x), _p(U_z),
                           _p(V_z), _p(x), _p(h), _p(v), _p(dy), _p(dx), _p(dU[0]), _p(dV[0]),
                           _p(dU[1]), _p(dV[1]), _p(dU[2]), _p(dV[2]), _p(db), _p(ws), _st(x))
    return dx, dU[0], dV[0], dU[1], dV[1], dU[2], dV[2], db, ws
