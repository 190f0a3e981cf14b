"""Drop-in for the reference's `hasty_pytorch_lib` extension module (E0 / E1 / E5 only).

Same function names, positional arguments and return lists as the pybind11
functions of the reference (elman/cuda/pytorch/elman_ladder.cc:22-281 and
:2802-3103, registered at :16539-16591).  Each function allocates its outputs
and scratch with PyTorch's caching allocator, as the reference does with
torch::empty, and enqueues the work of libelman_b200 on PyTorch's current CUDA
stream.  Inputs must be CUDA and contiguous (the reference's CHECK_INPUT,
support.h:21-23); shapes and dtypes are cross-checked as well, which the
reference does not do.  fp32 and bf16 are accepted; fp16/fp64 raise.

Use `elman_b200.install_as_hasty()` to make `import hasty_pytorch_lib` resolve
to this module, so the reference's model files pick it up unchanged.
"""
from __future__ import annotations

import torch

from . import _lib

_DT = {torch.float32: _lib.ELMAN_F32, torch.bfloat16: _lib.ELMAN_BF16}


def _check_inputs(fn, ref, **tensors):
    for name, t in tensors.items():
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{fn}: {name} must be a Tensor")
        if not t.is_cuda:
            raise RuntimeError(f"{fn}: {name} must be a CUDA tensor")
        if not t.is_contiguous():
            raise RuntimeError(f"{fn}: {name} must be contiguous")
        if t.dtype != ref.dtype:
            raise RuntimeError(f"{fn}: {name} has dtype {t.dtype}, expected {ref.dtype}")
        if t.device != ref.device:
            raise RuntimeError(f"{fn}: {name} is on {t.device}, expected {ref.device}")
    if ref.dtype not in _DT:
        raise RuntimeError(f"{fn}: dtype {ref.dtype} is not supported (float32 and bfloat16 are)")
    return _DT[ref.dtype]


def _shape(fn, t, shape, name):
    if tuple(t.shape) != tuple(shape):
        raise RuntimeError(f"{fn}: {name} has shape {tuple(t.shape)}, expected {tuple(shape)}")


def _ptr(t):
    return None if t is None or t.numel() == 0 else t.data_ptr()


def _workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def _stream(device):
    return torch.cuda.current_stream(device).cuda_stream


# --------------------------------------------------------------------------- E1

FLAG_COMPACT = 1   # ELMAN_FLAG_COMPACT: smallest-footprint recurrence launch


def mamba_gated_elman_forward(training, x, z, h0, W_x, W_h, b, flags=0):
    """-> [h[T+1,B,d], output[T,B,d], v[T,B,d] (empty if not training)]

    `flags` is not a reference argument (see elman_e1_forward_flags)."""
    fn = "mamba_gated_elman_forward"
    dt = _check_inputs(fn, x, x=x, z=z, h0=h0, W_x=W_x, W_h=W_h, b=b)
    if x.dim() != 3:
        raise RuntimeError(f"{fn}: x must be [T, B, dim]")
    T, B, d = x.shape
    _shape(fn, z, (T, B, d), "z"); _shape(fn, h0, (B, d), "h0")
    _shape(fn, W_x, (d, d), "W_x"); _shape(fn, W_h, (d, d), "W_h"); _shape(fn, b, (d,), "b")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        h = torch.empty(T + 1, B, d, dtype=x.dtype, device=x.device)
        out = torch.empty(T, B, d, dtype=x.dtype, device=x.device)
        v = torch.empty((T, B, d) if training else (0,), dtype=x.dtype, device=x.device)
        nws = lib.elman_e1_forward_workspace(dt, T, B, d)
        ws = _workspace(nws, x.device)
        rc = lib.elman_e1_forward_flags(dt, int(flags), 1 if training else 0, T, B, d, _ptr(x),
                                        _ptr(z), _ptr(h0), _ptr(W_x), _ptr(W_h), _ptr(b), _ptr(h),
                                        _ptr(out), _ptr(v), ws.data_ptr(), ws.numel(),
                                        _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [h, out, v]


def mamba_gated_elman_backward(W_x, W_h, x, z, h, v, d_output):
    """-> [dx, dz, dW_x, dW_h, db]"""
    fn = "mamba_gated_elman_backward"
    dt = _check_inputs(fn, x, W_x=W_x, W_h=W_h, x=x, z=z, h=h, v=v, d_output=d_output)
    T, B, d = x.shape
    _shape(fn, z, (T, B, d), "z"); _shape(fn, h, (T + 1, B, d), "h")
    _shape(fn, v, (T, B, d), "v"); _shape(fn, d_output, (T, B, d), "d_output")
    _shape(fn, W_x, (d, d), "W_x"); _shape(fn, W_h, (d, d), "W_h")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        dx = torch.empty_like(x)
        dz = torch.empty_like(z)
        dW_x = torch.empty(d, d, dtype=x.dtype, device=x.device)
        dW_h = torch.empty(d, d, dtype=x.dtype, device=x.device)
        db = torch.empty(d, dtype=x.dtype, device=x.device)
        ws = _workspace(lib.elman_e1_backward_workspace(dt, T, B, d), x.device)
        rc = lib.elman_e1_backward(dt, T, B, d, _ptr(W_x), _ptr(W_h), _ptr(x), _ptr(z), _ptr(h),
                                   _ptr(v), _ptr(d_output), _ptr(dx), _ptr(dz), _ptr(dW_x),
                                   _ptr(dW_h), _ptr(db), ws.data_ptr(), ws.numel(),
                                   _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [dx, dz, dW_x, dW_h, db]


def mamba_gated_elman_backward_carry(W_x, W_h, x, z, h, v, d_output, dv_in=None, flags=0):
    """Backward over one time chunk -> [dx, dz, dW_x, dW_h, db, dv_out].

    An extension with no counterpart in the reference: `dv_in` [B,d] is the
    `dv_out` of the chunk that follows in time (None for the last chunk) and
    `dv_out` [B,d] goes to the chunk that precedes.  With dv_in=None the first
    five results equal mamba_gated_elman_backward's.
    """
    fn = "mamba_gated_elman_backward_carry"
    tensors = dict(W_x=W_x, W_h=W_h, x=x, z=z, h=h, v=v, d_output=d_output)
    if dv_in is not None:
        tensors["dv_in"] = dv_in
    dt = _check_inputs(fn, x, **tensors)
    T, B, d = x.shape
    _shape(fn, z, (T, B, d), "z"); _shape(fn, h, (T + 1, B, d), "h")
    _shape(fn, v, (T, B, d), "v"); _shape(fn, d_output, (T, B, d), "d_output")
    _shape(fn, W_x, (d, d), "W_x"); _shape(fn, W_h, (d, d), "W_h")
    if dv_in is not None:
        _shape(fn, dv_in, (B, d), "dv_in")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        dx = torch.empty_like(x)
        dz = torch.empty_like(z)
        dW_x = torch.empty(d, d, dtype=x.dtype, device=x.device)
        dW_h = torch.empty(d, d, dtype=x.dtype, device=x.device)
        db = torch.empty(d, dtype=x.dtype, device=x.device)
        dv_out = torch.empty(B, d, dtype=x.dtype, device=x.device)
        ws = _workspace(lib.elman_e1_backward_workspace(dt, T, B, d), x.device)
        rc = lib.elman_e1_backward_carry(dt, int(flags), T, B, d, _ptr(W_x), _ptr(W_h), _ptr(x), _ptr(z),
                                         _ptr(h), _ptr(v), _ptr(d_output), _ptr(dv_in), _ptr(dx),
                                         _ptr(dz), _ptr(dW_x), _ptr(dW_h), _ptr(db), _ptr(dv_out),
                                         ws.data_ptr(), ws.numel(), _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [dx, dz, dW_x, dW_h, db, dv_out]


def recurrence_blocks(dtype, T, B, d, flags=0):
    """Thread blocks one E1/E0 recurrence launch of this shape keeps resident (0 when the
    shape takes a cooperative-launch kernel); see elman_b200_recurrence_blocks."""
    if dtype not in _DT:
        raise RuntimeError(f"recurrence_blocks: dtype {dtype} is not supported")
    return int(_lib.load().elman_b200_recurrence_blocks(_DT[dtype], int(flags), int(T), int(B),
                                                        int(d)))


# ------------------------------------------- the phases of an E1 call, one by one
# (extensions of the C ABI: elman_gemm, elman_column_sum, elman_e1_recurrence_*)

GEMM_NT, GEMM_NN, GEMM_TN = 0, 1, 2


def gemm(op, A, B, bias=None, out=None, accumulate=False):
    """Dense row-major GEMM through elman_gemm:
    GEMM_NT out[M,N] = A[M,K] B[N,K]^T (+bias), GEMM_NN A[M,K] B[K,N], GEMM_TN A[K,M]^T B[K,N]."""
    fn = "gemm"
    tensors = dict(A=A, B=B)
    if bias is not None:
        tensors["bias"] = bias
    dt = _check_inputs(fn, A, **tensors)
    if A.dim() != 2 or B.dim() != 2:
        raise RuntimeError(f"{fn}: A and B must be matrices")
    if op == GEMM_NT:
        (M, K), (N, K2) = A.shape, B.shape
    elif op == GEMM_NN:
        (M, K), (K2, N) = A.shape, B.shape
    elif op == GEMM_TN:
        (K, M), (K2, N) = A.shape, B.shape
    else:
        raise RuntimeError(f"{fn}: unknown form {op}")
    if K != K2:
        raise RuntimeError(f"{fn}: inner extents differ ({K} vs {K2})")
    if out is None:
        out = torch.empty(M, N, dtype=A.dtype, device=A.device)
        accumulate = False
    else:
        _shape(fn, out, (M, N), "out")
    with torch.cuda.device(A.device):
        rc = _lib.load().elman_gemm(dt, op, M, N, K, _ptr(A), _ptr(B), _ptr(bias), _ptr(out),
                                    1 if accumulate else 0, _stream(A.device))
        _lib.check(rc, fn)
    return out


def column_sum(x):
    """out[N] = sum over the rows of x[M,N] (deterministic) through elman_column_sum."""
    fn = "column_sum"
    dt = _check_inputs(fn, x, x=x)
    M, N = x.shape
    lib = _lib.load()
    with torch.cuda.device(x.device):
        out = torch.empty(N, dtype=x.dtype, device=x.device)
        ws = _workspace(lib.elman_column_sum_workspace(N), x.device)
        rc = lib.elman_column_sum(dt, M, N, _ptr(x), _ptr(out), ws.data_ptr(), ws.numel(),
                                  _stream(x.device))
        _lib.check(rc, fn)
    return out


def e1_recurrence_forward(training, pre, z, h0, W_h, flags=0):
    """The recurrence of the E1 cell alone, on already projected inputs pre = W_x x + b:
    -> [h[T+1,B,d], output[T,B,d], v[T,B,d] (empty if not training)]."""
    fn = "e1_recurrence_forward"
    dt = _check_inputs(fn, pre, pre=pre, z=z, h0=h0, W_h=W_h)
    if pre.dim() != 3:
        raise RuntimeError(f"{fn}: pre must be [T, B, dim]")
    T, B, d = pre.shape
    _shape(fn, z, (T, B, d), "z"); _shape(fn, h0, (B, d), "h0"); _shape(fn, W_h, (d, d), "W_h")
    lib = _lib.load()
    with torch.cuda.device(pre.device):
        h = torch.empty(T + 1, B, d, dtype=pre.dtype, device=pre.device)
        out = torch.empty(T, B, d, dtype=pre.dtype, device=pre.device)
        v = torch.empty((T, B, d) if training else (0,), dtype=pre.dtype, device=pre.device)
        ws = _workspace(lib.elman_e1_recurrence_workspace(dt, d), pre.device)
        rc = lib.elman_e1_recurrence_forward(dt, int(flags), 1 if training else 0, T, B, d,
                                             _ptr(pre), _ptr(z), _ptr(h0), _ptr(W_h), _ptr(h),
                                             _ptr(out), _ptr(v), ws.data_ptr(), ws.numel(),
                                             _stream(pre.device))
        _lib.check(rc, fn)
    return [h, out, v]


def e1_recurrence_backward(W_h, z, h, v, d_output, dv_in=None, flags=0, W_h_T=None):
    """BPTT of the recurrence alone -> [dv[T+1,B,d], dz[T,B,d], db[d]].  dv[:T] is the
    gradient of `pre`; dv[0] is what the preceding time chunk takes as its dv_in; slot T
    holds a copy of this call's dv_in (zeros if None)."""
    fn = "e1_recurrence_backward"
    tensors = dict(W_h=W_h, z=z, h=h, v=v, d_output=d_output)
    if dv_in is not None:
        tensors["dv_in"] = dv_in
    dt = _check_inputs(fn, z, **tensors)
    T, B, d = z.shape
    _shape(fn, h, (T + 1, B, d), "h"); _shape(fn, v, (T, B, d), "v")
    _shape(fn, d_output, (T, B, d), "d_output"); _shape(fn, W_h, (d, d), "W_h")
    if dv_in is not None:
        _shape(fn, dv_in, (B, d), "dv_in")
    if W_h_T is not None:
        _check_inputs(fn, z, W_h_T=W_h_T)
        _shape(fn, W_h_T, (d, d), "W_h_T")
    lib = _lib.load()
    with torch.cuda.device(z.device):
        dv = torch.empty(T + 1, B, d, dtype=z.dtype, device=z.device)
        dz = torch.empty_like(z)
        db = torch.empty(d, dtype=z.dtype, device=z.device)
        ws = _workspace(lib.elman_e1_recurrence_workspace(dt, d), z.device)
        rc = lib.elman_e1_recurrence_backward(dt, int(flags), T, B, d, _ptr(W_h), _ptr(z), _ptr(h),
                                              _ptr(v), _ptr(d_output), _ptr(dv_in), _ptr(W_h_T),
                                              _ptr(dv),
                                              _ptr(dz), _ptr(db), ws.data_ptr(), ws.numel(),
                                              _stream(z.device))
        _lib.check(rc, fn)
    return [dv, dz, db]


# --------------------------------------------------------------------------- E0

def stock_elman_forward(training, x, h0, W_x, W_h, W_gate, b, b_gate):
    """-> [h, output, v, gate_cache] (v, gate_cache empty if not training)"""
    fn = "stock_elman_forward"
    dt = _check_inputs(fn, x, x=x, h0=h0, W_x=W_x, W_h=W_h, W_gate=W_gate, b=b, b_gate=b_gate)
    if x.dim() != 3:
        raise RuntimeError(f"{fn}: x must be [T, B, dim]")
    T, B, d = x.shape
    _shape(fn, h0, (B, d), "h0")
    for name, w in (("W_x", W_x), ("W_h", W_h), ("W_gate", W_gate)):
        _shape(fn, w, (d, d), name)
    _shape(fn, b, (d,), "b"); _shape(fn, b_gate, (d,), "b_gate")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        h = torch.empty(T + 1, B, d, dtype=x.dtype, device=x.device)
        out = torch.empty(T, B, d, dtype=x.dtype, device=x.device)
        v = torch.empty((T, B, d) if training else (0,), dtype=x.dtype, device=x.device)
        gc = torch.empty((T, B, d) if training else (0,), dtype=x.dtype, device=x.device)
        ws = _workspace(lib.elman_e0_forward_workspace(dt, T, B, d), x.device)
        rc = lib.elman_e0_forward(dt, 1 if training else 0, T, B, d, _ptr(x), _ptr(h0), _ptr(W_x),
                                  _ptr(W_h), _ptr(W_gate), _ptr(b), _ptr(b_gate), _ptr(h),
                                  _ptr(out), _ptr(v), _ptr(gc), ws.data_ptr(), ws.numel(),
                                  _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [h, out, v, gc]


def stock_elman_backward(W_x, W_h, W_gate, x, h, v, gate_cache, d_output):
    """-> [dx, dW_x, dW_h, dW_gate, db, db_gate]"""
    fn = "stock_elman_backward"
    dt = _check_inputs(fn, x, W_x=W_x, W_h=W_h, W_gate=W_gate, x=x, h=h, v=v,
                       gate_cache=gate_cache, d_output=d_output)
    T, B, d = x.shape
    _shape(fn, h, (T + 1, B, d), "h"); _shape(fn, v, (T, B, d), "v")
    _shape(fn, gate_cache, (T, B, d), "gate_cache"); _shape(fn, d_output, (T, B, d), "d_output")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        dx = torch.empty_like(x)
        dW_x, dW_h, dW_gate = (torch.empty(d, d, dtype=x.dtype, device=x.device) for _ in range(3))
        db, db_gate = (torch.empty(d, dtype=x.dtype, device=x.device) for _ in range(2))
        ws = _workspace(lib.elman_e0_backward_workspace(dt, T, B, d), x.device)
        rc = lib.elman_e0_backward(dt, T, B, d, _ptr(W_x), _ptr(W_h), _ptr(W_gate), _ptr(x),
                                   _ptr(h), _ptr(v), _ptr(gate_cache), _ptr(d_output), _ptr(dx),
                                   _ptr(dW_x), _ptr(dW_h), _ptr(dW_gate), _ptr(db), _ptr(db_gate),
                                   ws.data_ptr(), ws.numel(), _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [dx, dW_x, dW_h, dW_gate, db, db_gate]


# --------------------------------------------------------------------------- E5

def pure_lowrank_elman_forward(training, x, h0, U_h, V_h, U_x, V_x, U_z, V_z, b):
    """-> [h, output, v]"""
    fn = "pure_lowrank_elman_forward"
    dt = _check_inputs(fn, x, x=x, h0=h0, U_h=U_h, V_h=V_h, U_x=U_x, V_x=V_x, U_z=U_z, V_z=V_z,
                       b=b)
    if x.dim() != 3:
        raise RuntimeError(f"{fn}: x must be [T, B, dim]")
    T, B, d = x.shape
    r = U_h.shape[1] if U_h.dim() == 2 else -1
    for name, u in (("U_h", U_h), ("U_x", U_x), ("U_z", U_z)):
        _shape(fn, u, (d, r), name)
    for name, vv in (("V_h", V_h), ("V_x", V_x), ("V_z", V_z)):
        _shape(fn, vv, (r, d), name)
    _shape(fn, h0, (B, d), "h0"); _shape(fn, b, (d,), "b")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        h = torch.empty(T + 1, B, d, dtype=x.dtype, device=x.device)
        out = torch.empty(T, B, d, dtype=x.dtype, device=x.device)
        v = torch.empty((T, B, d) if training else (0,), dtype=x.dtype, device=x.device)
        ws = _workspace(lib.elman_e5_forward_workspace(dt, T, B, d, r), x.device)
        rc = lib.elman_e5_forward(dt, 1 if training else 0, T, B, d, r, _ptr(x), _ptr(h0),
                                  _ptr(U_h), _ptr(V_h), _ptr(U_x), _ptr(V_x), _ptr(U_z), _ptr(V_z),
                                  _ptr(b), _ptr(h), _ptr(out), _ptr(v), ws.data_ptr(), ws.numel(),
                                  _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [h, out, v]


def pure_lowrank_elman_backward(U_h, V_h, U_x, V_x, U_z, V_z, x, h, v, d_output):
    """-> [dx, dU_h, dV_h, dU_x, dV_x, dU_z, dV_z, db]"""
    fn = "pure_lowrank_elman_backward"
    dt = _check_inputs(fn, x, U_h=U_h, V_h=V_h, U_x=U_x, V_x=V_x, U_z=U_z, V_z=V_z, x=x, h=h, v=v,
                       d_output=d_output)
    T, B, d = x.shape
    r = U_h.shape[1]
    _shape(fn, h, (T + 1, B, d), "h"); _shape(fn, v, (T, B, d), "v")
    _shape(fn, d_output, (T, B, d), "d_output")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        dx = torch.empty_like(x)
        dU = [torch.empty(d, r, dtype=x.dtype, device=x.device) for _ in range(3)]
        dV = [torch.empty(r, d, dtype=x.dtype, device=x.device) for _ in range(3)]
        db = torch.empty(d, dtype=x.dtype, device=x.device)
        ws = _workspace(lib.elman_e5_backward_workspace(dt, T, B, d, r), x.device)
        rc = lib.elman_e5_backward(dt, T, B, d, r, _ptr(U_h), _ptr(V_h), _ptr(U_x), _ptr(V_x),
                                   _ptr(U_z), _ptr(V_z), _ptr(x), _ptr(h), _ptr(v), _ptr(d_output),
                                   _ptr(dx), _ptr(dU[0]), _ptr(dV[0]), _ptr(dU[1]), _ptr(dV[1]),
                                   _ptr(dU[2]), _ptr(dV[2]), _ptr(db), ws.data_ptr(), ws.numel(),
                                   _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [dx, dU[0], dV[0], dU[1], dV[1], dU[2], dV[2], db]


def pure_lowrank_elman_backward_carry(U_h, V_h, U_x, V_x, U_z, V_z, x, h, v, d_output, dv_in=None):
    """Backward over one time chunk -> [dx, dU_h, dV_h, dU_x, dV_x, dU_z, dV_z, db, dv_out]
    (an extension, as mamba_gated_elman_backward_carry)."""
    fn = "pure_lowrank_elman_backward_carry"
    tensors = dict(U_h=U_h, V_h=V_h, U_x=U_x, V_x=V_x, U_z=U_z, V_z=V_z, x=x, h=h, v=v,
                   d_output=d_output)
    if dv_in is not None:
        tensors["dv_in"] = dv_in
    dt = _check_inputs(fn, x, **tensors)
    T, B, d = x.shape
    r = U_h.shape[1]
    _shape(fn, h, (T + 1, B, d), "h"); _shape(fn, v, (T, B, d), "v")
    _shape(fn, d_output, (T, B, d), "d_output")
    if dv_in is not None:
        _shape(fn, dv_in, (B, d), "dv_in")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        dx = torch.empty_like(x)
        dU = [torch.empty(d, r, dtype=x.dtype, device=x.device) for _ in range(3)]
        dV = [torch.empty(r, d, dtype=x.dtype, device=x.device) for _ in range(3)]
        db = torch.empty(d, dtype=x.dtype, device=x.device)
        dv_out = torch.empty(B, d, dtype=x.dtype, device=x.device)
        ws = _workspace(lib.elman_e5_backward_workspace(dt, T, B, d, r), x.device)
        rc = lib.elman_e5_backward_carry(dt, T, B, d, r, _ptr(U_h), _ptr(V_h), _ptr(U_x), _ptr(V_x),
                                         _ptr(U_z), _ptr(V_z), _ptr(x), _ptr(h), _ptr(v),
                                         _ptr(d_output), _ptr(dv_in), _ptr(dx), _ptr(dU[0]),
                                         _ptr(dV[0]), _ptr(dU[1]), _ptr(dV[1]), _ptr(dU[2]),
                                         _ptr(dV[2]), _ptr(db), _ptr(dv_out), ws.data_ptr(),
                                         ws.numel(), _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [dx, dU[0], dV[0], dU[1], dV[1], dU[2], dV[2], db, dv_out]


def lowrank_blocks(dtype, T, B, d, r):
    """Thread blocks one E5 recurrence launch keeps resident (0: cooperative-launch kernel)."""
    if dtype not in _DT:
        raise RuntimeError(f"lowrank_blocks: dtype {dtype} is not supported")
    return int(_lib.load().elman_b200_lowrank_blocks(_DT[dtype], int(T), int(B), int(d), int(r)))


# The reference exposes the fused E5 kernels under separate names; here both
# names run the same (already fused) path.
pure_lowrank_elman_forward_fused = pure_lowrank_elman_forward
pure_lowrank_elman_backward_fused = pure_lowrank_elman_backward
# The reference's back-to-back-GEMM variant of E5 (V_h h and U_h (.) fused with the rank-r
# intermediate kept on chip; elman/cuda/pytorch/elman_ladder.cc:3111-3178, :3180-3250, whose
# kernel is a stub restricted to rank 64/128/256) has the same signature; here every E5 call is
# that fusion (the single-cluster low-rank kernel), for any rank.
b2b_lowrank_elman_forward = pure_lowrank_elman_forward
b2b_lowrank_elman_backward = pure_lowrank_elman_backward


# ------------------------------------------------------------------ projection

def projection(A, W, bias=None, out=None, accumulate=False):
    """out[M,N] = A[M,K] @ W[N,K]^T (+ bias) (+ out) through elman_projection."""
    fn = "projection"
    tensors = dict(A=A, W=W)
    if bias is not None:
        tensors["bias"] = bias
    dt = _check_inputs(fn, A, **tensors)
    M, K = A.shape
    N = W.shape[0]
    _shape(fn, W, (N, K), "W")
    if out is None:
        out = torch.empty(M, N, dtype=A.dtype, device=A.device)
        accumulate = False
    lib = _lib.load()
    with torch.cuda.device(A.device):
        rc = lib.elman_projection(dt, M, N, K, _ptr(A), K, _ptr(W), K, _ptr(bias), _ptr(out), N,
                                  1 if accumulate else 0, _stream(A.device))
        _lib.check(rc, fn)
    return out


# ------------------------------ layer ops around the cell (extensions of the C ABI)

def spectral_norm_forward(W, u, target_radius, eps, iterations):
    """Power iteration from u (advanced in place) and rescaling of W in one kernel
    -> (W_eff like W, v fp32 [d], sigma fp32 [1]) through elman_spectral_norm_forward."""
    fn = "spectral_norm_forward"
    dt = _check_inputs(fn, W, W=W, u=u)
    if W.dim() != 2 or W.shape[0] != W.shape[1]:
        raise RuntimeError(f"{fn}: W must be square")
    d = W.shape[0]
    _shape(fn, u, (d,), "u")
    with torch.cuda.device(W.device):
        W_eff = torch.empty_like(W)
        v = torch.empty(d, dtype=torch.float32, device=W.device)
        sigma = torch.empty(1, dtype=torch.float32, device=W.device)
        rc = _lib.load().elman_spectral_norm_forward(dt, d, _ptr(W), _ptr(u), _ptr(v), _ptr(sigma),
                                                     _ptr(W_eff), float(target_radius), float(eps),
                                                     int(iterations), _stream(W.device))
        _lib.check(rc, fn)
    return W_eff, v, sigma


def spectral_norm_backward(W, u, v, sigma, dW_eff, target_radius, eps, out=None):
    """Gradient of W from the gradient of W_eff (u, v constant) -> dW like W; with `out` the
    result is ADDED into it."""
    fn = "spectral_norm_backward"
    dt = _check_inputs(fn, W, W=W, u=u, dW_eff=dW_eff)
    d = W.shape[0]
    _shape(fn, dW_eff, (d, d), "dW_eff"); _shape(fn, u, (d,), "u")
    for name, t, n in (("v", v, d), ("sigma", sigma, 1)):
        if t.dtype != torch.float32 or t.numel() != n or t.device != W.device or not t.is_contiguous():
            raise RuntimeError(f"{fn}: {name} must be a contiguous float32 tensor of {n} elements")
    with torch.cuda.device(W.device):
        accumulate = out is not None
        if out is None:
            out = torch.empty_like(W)
        else:
            _check_inputs(fn, W, out=out)
            _shape(fn, out, (d, d), "out")
        rc = _lib.load().elman_spectral_norm_backward(dt, d, _ptr(W), _ptr(u), _ptr(v), _ptr(sigma),
                                                      _ptr(dW_eff), _ptr(out), 1 if accumulate else 0,
                                                      float(target_radius), float(eps),
                                                      _stream(W.device))
        _lib.check(rc, fn)
    return out


def add_rmsnorm_forward(x, residual_in, weight, eps):
    """x [..., D] (+ residual_in fp32, or None) -> (y like x, residual_out fp32, rstd fp32 [rows])
    through elman_add_rmsnorm_forward."""
    fn = "add_rmsnorm_forward"
    dt = _check_inputs(fn, x, x=x, weight=weight)
    D = x.shape[-1]
    M = x.numel() // max(D, 1)
    _shape(fn, weight, (D,), "weight")
    if residual_in is not None:
        if residual_in.dtype != torch.float32 or not residual_in.is_contiguous() or \
                residual_in.shape != x.shape or residual_in.device != x.device:
            raise RuntimeError(f"{fn}: residual_in must be a contiguous float32 tensor shaped like x")
    with torch.cuda.device(x.device):
        res_out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        y = torch.empty_like(x)
        rstd = torch.empty(M, dtype=torch.float32, device=x.device)
        rc = _lib.load().elman_add_rmsnorm_forward(dt, M, D, _ptr(x), _ptr(residual_in), _ptr(weight),
                                                   float(eps), _ptr(res_out), _ptr(y), _ptr(rstd),
                                                   _stream(x.device))
        _lib.check(rc, fn)
    return y, res_out, rstd


def add_rmsnorm_backward(dy, dres_out, res_out, rstd, weight, want_dres_in, want_dx):
    """-> (dres_in fp32 or None, dx like dy or None, dweight [D]) through
    elman_add_rmsnorm_backward."""
    fn = "add_rmsnorm_backward"
    dt = _check_inputs(fn, dy, dy=dy, weight=weight)
    D = dy.shape[-1]
    M = dy.numel() // max(D, 1)
    for name, t in (("dres_out", dres_out), ("res_out", res_out), ("rstd", rstd)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or not t.is_cuda):
            raise RuntimeError(f"{fn}: {name} must be a contiguous float32 CUDA tensor")
    lib = _lib.load()
    with torch.cuda.device(dy.device):
        dres_in = torch.empty(dy.shape, dtype=torch.float32, device=dy.device) if want_dres_in else None
        dx = torch.empty_like(dy) if want_dx else None
        dw = torch.empty(D, dtype=dy.dtype, device=dy.device)
        ws = _workspace(lib.elman_add_rmsnorm_backward_workspace(D), dy.device)
        rc = lib.elman_add_rmsnorm_backward(dt, M, D, _ptr(dy), _ptr(dres_out), _ptr(res_out),
                                            _ptr(rstd), _ptr(weight), _ptr(dres_in), _ptr(dx),
                                            _ptr(dw), ws.data_ptr(), ws.numel(), _stream(dy.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(dy.device))
    return dres_in, dx, dw


def in_proj_split_silu(u, W_in):
    """u [M,K], W_in [2*d,K] -> (x_raw, x_act = silu(x_raw), z), each [M,d], through
    elman_in_proj_split_silu (split and silu in the GEMM epilogue on the bf16 path)."""
    fn = "in_proj_split_silu"
    dt = _check_inputs(fn, u, u=u, W_in=W_in)
    M, K = u.shape
    if W_in.dim() != 2 or W_in.shape[1] != K or W_in.shape[0] % 2:
        raise RuntimeError(f"{fn}: W_in must be [2*d_inner, {K}]")
    d = W_in.shape[0] // 2
    lib = _lib.load()
    with torch.cuda.device(u.device):
        x_raw, x_act, z = (torch.empty(M, d, dtype=u.dtype, device=u.device) for _ in range(3))
        need = 0 if (dt == _lib.ELMAN_BF16 and d % 32 == 0 and K % 8 == 0
                     and _lib.get_option("force_generic") == 0) else lib.elman_in_proj_workspace(dt, M, d)
        ws = _workspace(need, u.device)
        rc = lib.elman_in_proj_split_silu(dt, M, d, K, _ptr(u), _ptr(W_in), _ptr(x_raw), _ptr(x_act),
                                          _ptr(z), ws.data_ptr(), ws.numel() if need else 0,
                                          _stream(u.device))
        if rc == 4 and not need:   # the library chose the two-pass form after all
            ws = _workspace(lib.elman_in_proj_workspace(dt, M, d), u.device)
            rc = lib.elman_in_proj_split_silu(dt, M, d, K, _ptr(u), _ptr(W_in), _ptr(x_raw),
                                              _ptr(x_act), _ptr(z), ws.data_ptr(), ws.numel(),
                                              _stream(u.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(u.device))
    return x_raw, x_act, z


def silu_backward_concat(d_act, x_raw, dz):
    """-> dxz [M, 2*d] = [d_act * silu'(x_raw) | dz] through elman_silu_backward_concat."""
    fn = "silu_backward_concat"
    dt = _check_inputs(fn, d_act, d_act=d_act, x_raw=x_raw, dz=dz)
    M, d = d_act.shape
    _shape(fn, x_raw, (M, d), "x_raw"); _shape(fn, dz, (M, d), "dz")
    with torch.cuda.device(d_act.device):
        dxz = torch.empty(M, 2 * d, dtype=d_act.dtype, device=d_act.device)
        rc = _lib.load().elman_silu_backward_concat(dt, M, d, _ptr(d_act), _ptr(x_raw), _ptr(dz),
                                                    _ptr(dxz), _stream(d_act.device))
        _lib.check(rc, fn)
    return dxz


# ------------------------- E1 with the gate on [h; x] (extension; README formula of the reference)

def mamba_gated_elman_hx_forward(training, x, z, h0, W_x, W_h, b, W_gh):
    """y_t = h_t * silu(z_t + W_gh h_t) -> [h[T+1,B,d], output, v (empty if not training), z_gate]
    through elman_e1_hx_forward.  Not a function of the reference's extension module."""
    fn = "mamba_gated_elman_hx_forward"
    dt = _check_inputs(fn, x, x=x, z=z, h0=h0, W_x=W_x, W_h=W_h, b=b, W_gh=W_gh)
    if x.dim() != 3:
        raise RuntimeError(f"{fn}: x must be [T, B, dim]")
    T, B, d = x.shape
    _shape(fn, z, (T, B, d), "z"); _shape(fn, h0, (B, d), "h0"); _shape(fn, b, (d,), "b")
    for name, w in (("W_x", W_x), ("W_h", W_h), ("W_gh", W_gh)):
        _shape(fn, w, (d, d), name)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        h = torch.empty(T + 1, B, d, dtype=x.dtype, device=x.device)
        out = torch.empty(T, B, d, dtype=x.dtype, device=x.device)
        zg = torch.empty(T, B, d, dtype=x.dtype, device=x.device)
        v = torch.empty((T, B, d) if training else (0,), dtype=x.dtype, device=x.device)
        ws = _workspace(lib.elman_e1_hx_forward_workspace(dt, T, B, d), x.device)
        rc = lib.elman_e1_hx_forward(dt, 1 if training else 0, T, B, d, _ptr(x), _ptr(z), _ptr(h0),
                                     _ptr(W_x), _ptr(W_h), _ptr(b), _ptr(W_gh), _ptr(h), _ptr(out),
                                     _ptr(v), _ptr(zg), ws.data_ptr(), ws.numel(), _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [h, out, v, zg]


def mamba_gated_elman_hx_backward(W_x, W_h, W_gh, x, z_gate, h, v, d_output):
    """-> [dx, dz, dW_x, dW_h, db, dW_gh] through elman_e1_hx_backward."""
    fn = "mamba_gated_elman_hx_backward"
    dt = _check_inputs(fn, x, W_x=W_x, W_h=W_h, W_gh=W_gh, x=x, z_gate=z_gate, h=h, v=v,
                       d_output=d_output)
    T, B, d = x.shape
    _shape(fn, z_gate, (T, B, d), "z_gate"); _shape(fn, h, (T + 1, B, d), "h")
    _shape(fn, v, (T, B, d), "v"); _shape(fn, d_output, (T, B, d), "d_output")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        dx = torch.empty_like(x)
        dz = torch.empty_like(x)
        dW_x, dW_h, dW_gh = (torch.empty(d, d, dtype=x.dtype, device=x.device) for _ in range(3))
        db = torch.empty(d, dtype=x.dtype, device=x.device)
        ws = _workspace(lib.elman_e1_hx_backward_workspace(dt, T, B, d), x.device)
        rc = lib.elman_e1_hx_backward(dt, T, B, d, _ptr(W_x), _ptr(W_h), _ptr(W_gh), _ptr(x),
                                      _ptr(z_gate), _ptr(h), _ptr(v), _ptr(d_output), _ptr(dx),
                                      _ptr(dz), _ptr(dW_x), _ptr(dW_h), _ptr(db), _ptr(dW_gh),
                                      ws.data_ptr(), ws.numel(), _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [dx, dz, dW_x, dW_h, db, dW_gh]


# --------------------------------------------------------------------------- E33

def lowrank_elman_forward(training, x, z, h0, W_x, U, V, b):
    """E4: h_t = tanh(W_x x_t + U (V h_{t-1}) + b), y_t = h_t * silu(z_t) -> [h, output, v];
    the reference's lowrank_elman_forward (elman/cuda/pytorch/elman_ladder.cc:2665-2726)."""
    fn = "lowrank_elman_forward"
    dt = _check_inputs(fn, x, x=x, z=z, h0=h0, W_x=W_x, U=U, V=V, b=b)
    if x.dim() != 3:
        raise RuntimeError(f"{fn}: x must be [T, B, dim]")
    T, B, d = x.shape
    if U.dim() != 2 or U.shape[0] != d:
        raise RuntimeError(f"{fn}: U must be [dim, rank]")
    r = U.shape[1]
    _shape(fn, z, (T, B, d), "z"); _shape(fn, h0, (B, d), "h0"); _shape(fn, W_x, (d, d), "W_x")
    _shape(fn, V, (r, d), "V"); _shape(fn, b, (d,), "b")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        h = torch.empty(T + 1, B, d, dtype=x.dtype, device=x.device)
        out = torch.empty(T, B, d, dtype=x.dtype, device=x.device)
        v = torch.empty((T, B, d) if training else (0,), dtype=x.dtype, device=x.device)
        ws = _workspace(lib.elman_e4_forward_workspace(dt, T, B, d, r), x.device)
        rc = lib.elman_e4_forward(dt, 1 if training else 0, T, B, d, r, _ptr(x), _ptr(z), _ptr(h0),
                                  _ptr(W_x), _ptr(U), _ptr(V), _ptr(b), _ptr(h), _ptr(out), _ptr(v),
                                  ws.data_ptr(), ws.numel(), _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [h, out, v]


def lowrank_elman_backward(W_x, U, V, x, z, h, v, d_output):
    """-> [dx, dz, dW_x, dU, dV, db]; the reference's lowrank_elman_backward (:2728-2800)."""
    fn = "lowrank_elman_backward"
    dt = _check_inputs(fn, x, W_x=W_x, U=U, V=V, x=x, z=z, h=h, v=v, d_output=d_output)
    T, B, d = x.shape
    r = U.shape[1]
    _shape(fn, V, (r, d), "V"); _shape(fn, z, (T, B, d), "z"); _shape(fn, h, (T + 1, B, d), "h")
    _shape(fn, v, (T, B, d), "v"); _shape(fn, d_output, (T, B, d), "d_output")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        dx, dz = torch.empty_like(x), torch.empty_like(x)
        dW_x = torch.empty(d, d, dtype=x.dtype, device=x.device)
        dU = torch.empty(d, r, dtype=x.dtype, device=x.device)
        dV = torch.empty(r, d, dtype=x.dtype, device=x.device)
        db = torch.empty(d, dtype=x.dtype, device=x.device)
        ws = _workspace(lib.elman_e4_backward_workspace(dt, T, B, d, r), x.device)
        rc = lib.elman_e4_backward(dt, T, B, d, r, _ptr(W_x), _ptr(U), _ptr(V), _ptr(x), _ptr(z),
                                   _ptr(h), _ptr(v), _ptr(d_output), _ptr(dx), _ptr(dz), _ptr(dW_x),
                                   _ptr(dU), _ptr(dV), _ptr(db), ws.data_ptr(), ws.numel(),
                                   _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [dx, dz, dW_x, dU, dV, db]


def _e1h_dense_weight(W_h):
    """[H, N, N] per-head weights, used as h_prev @ W_h[k] by the reference's einsum
    'bhi,hij->bhj', as ONE block-diagonal [H N, H N] matrix in the W h convention of the dense
    recurrence (block k = W_h[k] transposed)."""
    return torch.block_diag(*W_h.transpose(1, 2).unbind(0)).contiguous()


def e1h_forward(training, pre_x, z, h0, W_h, b_h):
    """E1H, H independent heads of size N: h_t = tanh(pre_x_t + h_{t-1} W_h + b) per head,
    y_t = h_t * silu(z_t).  pre_x, z: [T, B, H, N]; h0: [B, H, N]; W_h: [H, N, N]; b_h: [H, N]
    -> [h_final [B,H,N], output [T,B,H,N], saved state for e1h_backward]; the reference's
    e1h_forward (elman/cuda/pytorch/elman_ladder.cc:14610-14666; its kernel,
    elman/cuda/lib/e1h_multihead_gpu.cu.cc, keeps every 16th state and recomputes).

    Here the heads run as one dense recurrence with a block-diagonal weight on the tensor-core
    recurrence kernel — the step is bound by its dependency chain, not by the multiplications, so
    the zero blocks cost nothing that matters; the third return value holds all states and
    pre-activations ([2T+1, B, H, N]) instead of checkpoints and is opaque to the caller, as
    it is in the reference."""
    fn = "e1h_forward"
    _check_inputs(fn, pre_x, pre_x=pre_x, z=z, h0=h0, W_h=W_h, b_h=b_h)
    if pre_x.dim() != 4:
        raise RuntimeError(f"{fn}: pre_x must be [T, B, H, N]")
    T, B, Hh, N = pre_x.shape
    d = Hh * N
    _shape(fn, z, (T, B, Hh, N), "z"); _shape(fn, h0, (B, Hh, N), "h0")
    _shape(fn, W_h, (Hh, N, N), "W_h"); _shape(fn, b_h, (Hh, N), "b_h")
    pre = (pre_x.reshape(T, B, d) + b_h.reshape(d)).contiguous()
    h, out, v = e1_recurrence_forward(training, pre, z.reshape(T, B, d), h0.reshape(B, d),
                                      _e1h_dense_weight(W_h))
    saved = torch.cat([h, v]).reshape(2 * T + 1, B, Hh, N) if training else pre_x.new_empty(0)
    return [h[T].reshape(B, Hh, N).clone(), out.reshape(T, B, Hh, N), saved]


def e1h_backward(pre_x, z, W_h, b_h, saved, d_output):
    """-> [d_pre_x [T,B,H,N], d_z [T,B,H,N], d_W_h [B,H,N,N] fp32, d_b [B,H,N] fp32]; the
    reference's e1h_backward (:14668-14730).  The reference returns per-batch-row partial
    weight gradients that its caller sums over the first axis; here the sums are formed on the
    device by one GEMM and returned in row 0, the other rows are zero."""
    fn = "e1h_backward"
    _check_inputs(fn, pre_x, pre_x=pre_x, z=z, W_h=W_h, b_h=b_h, saved=saved, d_output=d_output)
    T, B, Hh, N = pre_x.shape
    d = Hh * N
    _shape(fn, saved, (2 * T + 1, B, Hh, N), "saved"); _shape(fn, d_output, (T, B, Hh, N), "d_output")
    flat = saved.reshape(2 * T + 1, B, d)
    h, v = flat[:T + 1], flat[T + 1:]
    dv, dz, db = e1_recurrence_backward(_e1h_dense_weight(W_h), z.reshape(T, B, d), h, v,
                                        d_output.reshape(T, B, d).contiguous())
    dvf = dv[:T].reshape(T * B, d)
    dWd = gemm(GEMM_TN, dvf, h[:T].reshape(T * B, d))        # [d, d]: sum_t dv_t h_{t-1}^T
    blocks = dWd.reshape(Hh, N, Hh, N)
    idx = torch.arange(Hh, device=dWd.device)
    dW = blocks[idx, :, idx, :].transpose(1, 2).float()       # per head, back to h_prev @ W form
    dW_rows = torch.zeros(B, Hh, N, N, dtype=torch.float32, device=dWd.device)
    db_rows = torch.zeros(B, Hh, N, dtype=torch.float32, device=dWd.device)
    dW_rows[0] = dW
    db_rows[0] = db.float().reshape(Hh, N)
    return [dv[:T].reshape(T, B, Hh, N), dz.reshape(T, B, Hh, N), dW_rows, db_rows]


def e33_self_gate_forward(training, x, h0, W_x, W_h, b):
    """y_t = h_t * silu(h_t) -> [h, output, v (empty if not training)]; the reference's
    e33_self_gate_forward (elman/cuda/pytorch/elman_ladder.cc:444-497)."""
    fn = "e33_self_gate_forward"
    dt = _check_inputs(fn, x, x=x, h0=h0, W_x=W_x, W_h=W_h, b=b)
    if x.dim() != 3:
        raise RuntimeError(f"{fn}: x must be [T, B, dim]")
    T, B, d = x.shape
    _shape(fn, h0, (B, d), "h0"); _shape(fn, W_x, (d, d), "W_x"); _shape(fn, W_h, (d, d), "W_h")
    _shape(fn, b, (d,), "b")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        h = torch.empty(T + 1, B, d, dtype=x.dtype, device=x.device)
        out = torch.empty(T, B, d, dtype=x.dtype, device=x.device)
        v = torch.empty((T, B, d) if training else (0,), dtype=x.dtype, device=x.device)
        ws = _workspace(lib.elman_e33_forward_workspace(dt, T, B, d), x.device)
        rc = lib.elman_e33_forward(dt, 1 if training else 0, T, B, d, _ptr(x), _ptr(h0), _ptr(W_x),
                                   _ptr(W_h), _ptr(b), _ptr(h), _ptr(out), _ptr(v), ws.data_ptr(),
                                   ws.numel(), _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [h, out, v]


def e33_self_gate_backward(W_x, W_h, x, h, v, d_output):
    """-> [dx, dW_x, dW_h, db]; the reference's e33_self_gate_backward (:499-557)."""
    fn = "e33_self_gate_backward"
    dt = _check_inputs(fn, x, W_x=W_x, W_h=W_h, x=x, h=h, v=v, d_output=d_output)
    T, B, d = x.shape
    _shape(fn, h, (T + 1, B, d), "h"); _shape(fn, v, (T, B, d), "v")
    _shape(fn, d_output, (T, B, d), "d_output")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        dx = torch.empty_like(x)
        dW_x, dW_h = (torch.empty(d, d, dtype=x.dtype, device=x.device) for _ in range(2))
        db = torch.empty(d, dtype=x.dtype, device=x.device)
        ws = _workspace(lib.elman_e33_backward_workspace(dt, T, B, d), x.device)
        rc = lib.elman_e33_backward(dt, T, B, d, _ptr(W_x), _ptr(W_h), _ptr(x), _ptr(h), _ptr(v),
                                    _ptr(d_output), _ptr(dx), _ptr(dW_x), _ptr(dW_h), _ptr(db),
                                    ws.data_ptr(), ws.numel(), _stream(x.device))
        _lib.check(rc, fn)
        ws.record_stream(torch.cuda.current_stream(x.device))
    return [dx, dW_x, dW_h, db]
