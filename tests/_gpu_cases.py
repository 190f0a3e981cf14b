"""Helpers shared by the GPU parity tests: run one cell through the CUDA library
(via the extension-module functions, i.e. through the C ABI) and through the CPU
oracle on the same seeded inputs, and return per-tensor norm-wise relative errors."""
import contextlib

import torch

from elman_b200 import _lib
from elman_b200 import hasty_pytorch_lib as H
from oracle import elman_oracle as orc

# tolerances stated by the task: fp32 within 1e-4 relative, bf16 within 2e-2 relative
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


@contextlib.contextmanager
def option(name, value):
    old = _lib.get_option(name)
    _lib.set_option(name, value)
    try:
        yield
    finally:
        _lib.set_option(name, old)


def round_inputs(inp, dtype):
    """Round every input to `dtype` first; the oracle gets the rounded values in fp32."""
    dev = {k: v.to(dtype).cuda().contiguous() for k, v in inp.items()}
    ref = {k: v.to(dtype).float() for k, v in inp.items()}
    return dev, ref


def errors(got, want):
    return {k: orc.rel_err(got[k].float().cpu(), want[k]) for k in want if k in got}


def assert_close(errs, tol, what=""):
    bad = {k: e for k, e in errs.items() if not (e < tol)}
    assert not bad, f"{what} rel errors above {tol}: {bad} (all: {errs})"


def run_e1(inp, dtype, training=True):
    dev, ref = round_inputs(inp, dtype)
    h, out, v = H.mamba_gated_elman_forward(training, dev["x"], dev["z"], dev["h0"], dev["W_x"],
                                            dev["W_h"], dev["b"])
    got = {"h": h, "output": out, "v": v}
    if training:
        dx, dz, dWx, dWh, db = H.mamba_gated_elman_backward(dev["W_x"], dev["W_h"], dev["x"],
                                                            dev["z"], h, v, dev["d_output"])
        got.update(dx=dx, dz=dz, dW_x=dWx, dW_h=dWh, db=db)
    torch.cuda.synchronize()
    return got, ref


def oracle_e1(ref):
    f = orc.e1_forward(ref["x"], ref["z"], ref["h0"], ref["W_x"], ref["W_h"], ref["b"])
    g = orc.e1_backward(ref["W_x"], ref["W_h"], ref["x"], ref["z"], f["h"], f["v"], ref["d_output"])
    return {**f, **g}


def run_e0(inp, dtype, training=True):
    dev, ref = round_inputs(inp, dtype)
    h, out, v, gc = H.stock_elman_forward(training, dev["x"], dev["h0"], dev["W_x"], dev["W_h"],
                                          dev["W_gate"], dev["b"], dev["b_gate"])
    got = {"h": h, "output": out, "v": v, "gate_cache": gc}
    if training:
        r = H.stock_elman_backward(dev["W_x"], dev["W_h"], dev["W_gate"], dev["x"], h, v, gc,
                                   dev["d_output"])
        got.update(dict(zip(("dx", "dW_x", "dW_h", "dW_gate", "db", "db_gate"), r)))
    torch.cuda.synchronize()
    return got, ref


def oracle_e0(ref):
    f = orc.e0_forward(ref["x"], ref["h0"], ref["W_x"], ref["W_h"], ref["W_gate"], ref["b"],
                       ref["b_gate"])
    g = orc.e0_backward(ref["W_x"], ref["W_h"], ref["W_gate"], ref["x"], f["h"], f["v"],
                        f["gate_cache"], ref["d_output"])
    return {**f, **g}


E5W = ("U_h", "V_h", "U_x", "V_x", "U_z", "V_z")


def run_e5(inp, dtype, training=True):
    dev, ref = round_inputs(inp, dtype)
    w = [dev[k] for k in E5W]
    h, out, v = H.pure_lowrank_elman_forward(training, dev["x"], dev["h0"], *w, dev["b"])
    got = {"h": h, "output": out, "v": v}
    if training:
        r = H.pure_lowrank_elman_backward(*w, dev["x"], h, v, dev["d_output"])
        got.update(dict(zip(("dx", "dU_h", "dV_h", "dU_x", "dV_x", "dU_z", "dV_z", "db"), r)))
    torch.cuda.synchronize()
    return got, ref


def oracle_e5(ref):
    w = [ref[k] for k in E5W]
    f = orc.e5_forward(ref["x"], ref["h0"], *w, ref["b"])
    g = orc.e5_backward(*w, ref["x"], f["h"], f["v"], ref["d_output"])
    return {**f, **g}
