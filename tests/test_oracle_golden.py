"""The CPU oracle against the fixtures produced by the reference's own code."""
import os

import numpy as np
import pytest
import torch

from oracle import elman_oracle as orc

TOL = 2e-5  # fp32 CPU vs fp32 CPU, different summation order only


def load(golden_dir, name):
    d = np.load(os.path.join(golden_dir, name + ".npz"))
    inp = {k[3:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("in_")}
    out = {k[4:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("out_")}
    return inp, out, d["meta"]


def check(got, want, keys, tol=TOL):
    for k in keys:
        err = orc.rel_err(got[k], want[k])
        assert err < tol, f"{k}: rel err {err:.3e}"


E1_KEYS = ["output", "h", "dx", "dz", "dW_x", "dW_h", "db"]


@pytest.mark.parametrize("name", ["e1_small", "e1_h0"])
def test_e1_matches_reference(golden_dir, name):
    inp, want, _ = load(golden_dir, name)
    fwd = orc.e1_forward(inp["x"], inp["z"], inp["h0"], inp["W_x"], inp["W_h"], inp["b"])
    bwd = orc.e1_backward(inp["W_x"], inp["W_h"], inp["x"], inp["z"], fwd["h"], fwd["v"],
                          inp["d_output"])
    check({**fwd, **bwd}, want, E1_KEYS)
    ag = orc.e1_autograd(inp["x"], inp["z"], inp["h0"], inp["W_x"], inp["W_h"], inp["b"],
                         inp["d_output"])
    check(ag, want, E1_KEYS)


def test_e1_config0_matches_reference(golden_dir):
    _, want, meta = load(golden_dir, "e1_c0")
    T, B, d, seed = (int(v) for v in meta)
    inp = orc.make_e1_inputs(T, B, d, seed=seed)
    chk = np.load(os.path.join(golden_dir, "e1_c0.npz"))["in_checksum"]
    mine = np.array([float(v.double().abs().sum()) for v in inp.values()])
    assert np.allclose(mine, chk, rtol=1e-12), "seeded input generator drifted"
    fwd = orc.e1_forward(inp["x"], inp["z"], inp["h0"], inp["W_x"], inp["W_h"], inp["b"])
    bwd = orc.e1_backward(inp["W_x"], inp["W_h"], inp["x"], inp["z"], fwd["h"], fwd["v"],
                          inp["d_output"])
    check({**fwd, **bwd}, want, ["output", "dx", "dz", "dW_x", "dW_h", "db"], tol=1e-4)


@pytest.mark.parametrize("name", ["e0_small", "e0_mid"])
def test_e0_matches_reference(golden_dir, name):
    inp, want, _ = load(golden_dir, name)
    fwd = orc.e0_forward(inp["x"], inp["h0"], inp["W_x"], inp["W_h"], inp["W_gate"], inp["b"],
                         inp["b_gate"])
    bwd = orc.e0_backward(inp["W_x"], inp["W_h"], inp["W_gate"], inp["x"], fwd["h"], fwd["v"],
                          fwd["gate_cache"], inp["d_output"])
    keys = ["output", "h", "dx", "dW_x", "dW_h", "dW_gate", "db", "db_gate"]
    check({**fwd, **bwd}, want, keys)
    ag = orc.e0_autograd(inp["x"], inp["h0"], inp["W_x"], inp["W_h"], inp["W_gate"], inp["b"],
                         inp["b_gate"], inp["d_output"])
    check(ag, want, keys)


@pytest.mark.parametrize("name", ["e5_small", "e5_mid"])
def test_e5_matches_reference(golden_dir, name):
    inp, want, _ = load(golden_dir, name)
    w = [inp[k] for k in ("U_h", "V_h", "U_x", "V_x", "U_z", "V_z")]
    fwd = orc.e5_forward(inp["x"], inp["h0"], *w, inp["b"])
    bwd = orc.e5_backward(*w, inp["x"], fwd["h"], fwd["v"], inp["d_output"])
    keys = ["output", "h", "dx", "dU_h", "dV_h", "dU_x", "dV_x", "dU_z", "dV_z", "db"]
    check({**fwd, **bwd}, want, keys)
    ag = orc.e5_autograd(inp["x"], inp["h0"], *w, inp["b"], inp["d_output"])
    check(ag, want, keys)


def test_fp64_error_bar():
    """fp32 oracle vs its own fp64 run: the floor under every fp32 tolerance."""
    inp = orc.make_e1_inputs(64, 4, 128, seed=5)
    a = orc.e1_autograd(inp["x"], inp["z"], inp["h0"], inp["W_x"], inp["W_h"], inp["b"],
                        inp["d_output"])
    i64 = {k: v.double() for k, v in inp.items()}
    b = orc.e1_autograd(i64["x"], i64["z"], i64["h0"], i64["W_x"], i64["W_h"], i64["b"],
                        i64["d_output"])
    for k in E1_KEYS:
        assert orc.rel_err(a[k], b[k]) < 1e-5


def test_hx_gate_reduces_to_e1_when_h_block_is_zero():
    inp = orc.make_e1_inputs(5, 2, 16, seed=9)
    Wg = inp["W_g"].clone()
    Wg[:, :16] = 0
    a = orc.e1_hx_gate_forward(inp["x"], inp["h0"], inp["W_x"], inp["W_h"], inp["b"], Wg,
                               inp["b_g"])
    b = orc.e1_forward(inp["x"], inp["z"], inp["h0"], inp["W_x"], inp["W_h"], inp["b"])
    assert orc.rel_err(a["output"], b["output"]) < 1e-6
