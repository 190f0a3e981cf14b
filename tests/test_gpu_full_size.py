"""Full-size parity: outputs AND all gradients at the benchmark's own shapes.

configs[1] (E1, bf16, d=1280, B=32, T=512), the same shape for E0, and configs[3]
(E5, bf16, d=1536, rank 270, B=32, T=512) run through the C ABI and are compared,
tensor by tensor (norm-wise relative error, 2e-2 for bf16), with

  * one fp32 pass of the CPU oracle on the same bf16-rounded inputs, and
  * the reference's own CUDA kernels (oracle/_ref, rebuilt for sm_100) when that
    library is present.

512 steps of bf16 BPTT is where accumulated rounding would show; the small-shape
tests cannot see it.  The reference kernels round to bf16 at every intermediate
(and E5 accumulates its weight gradients in bf16 once per step), so their own
distance to the fp32 result is reported beside ours.
"""
import pytest
import torch

from elman_b200 import _lib
from oracle import elman_oracle as orc
from oracle import ref_cuda
from tests._gpu_cases import (E5W, TOL, assert_close, errors, oracle_e0, oracle_e1, oracle_e5,
                              round_inputs, run_e0, run_e1, run_e5)

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def rel(a, b):
    return orc.rel_err(a.float().cpu(), b.float().cpu())


def _versus_reference_cuda(mine, theirs, truth, what):
    """Ours against the reference kernels: within tolerance of them wherever they are
    themselves within tolerance of the fp32 result; never further from the fp32 result
    than they are by more than the tolerance."""
    tol = TOL[BF16]
    report = {}
    for k in theirs:
        e_mine, e_ref, e_pair = rel(mine[k], truth[k]), rel(theirs[k], truth[k]), rel(mine[k], theirs[k])
        report[k] = (e_mine, e_ref, e_pair)
        assert e_mine < e_ref + tol, f"{what} {k}: ours {e_mine:.3e}, reference kernels {e_ref:.3e}"
        assert e_pair < tol + e_ref, f"{what} {k}: vs reference kernels {e_pair:.3e} (their own error {e_ref:.3e})"
    return report


def test_e1_config1_full_size_outputs_and_gradients():
    T, B, d = 512, 32, 1280
    inp = orc.make_e1_inputs(T, B, d, seed=1235)
    before = _lib.tc_launch_count()
    got, ref = run_e1(inp, BF16)
    # two recurrences, the projection, dx, and the two weight gradients in one dual launch
    assert _lib.tc_launch_count() >= before + 5, "recurrences and GEMMs must take the tcgen05 kernels"
    assert _lib.device_status()[0] == 0
    truth = oracle_e1(ref)                       # one fp32 CPU pass, a few seconds
    keys = ("h", "output", "v", "dx", "dz", "dW_x", "dW_h", "db")
    assert_close({k: rel(got[k], truth[k]) for k in keys}, TOL[BF16], "E1 configs[1] vs fp32 oracle")
    if ref_cuda.available():
        dev, _ = round_inputs(inp, BF16)
        rh, rout, rv, _ws = ref_cuda.e1_forward(True, dev["x"], dev["z"], dev["h0"], dev["W_x"],
                                                dev["W_h"], dev["b"])
        rr = ref_cuda.e1_backward(dev["W_x"], dev["W_h"], dev["x"], dev["z"], rh, rv, dev["d_output"])
        torch.cuda.synchronize()
        theirs = dict(zip(("dx", "dz", "dW_x", "dW_h", "db"), rr[:5]))
        theirs.update(h=rh, output=rout, v=rv)
        _versus_reference_cuda(got, theirs, truth, "E1 configs[1]")


def test_e0_config1_shape_outputs_and_gradients():
    T, B, d = 512, 32, 1280
    inp = orc.make_e0_inputs(T, B, d, seed=1236)
    got, ref = run_e0(inp, BF16)
    assert _lib.device_status()[0] == 0
    truth = oracle_e0(ref)
    assert_close(errors(got, truth), TOL[BF16], "E0 d1280 B32 T512 vs fp32 oracle")
    if ref_cuda.available():
        dev, _ = round_inputs(inp, BF16)
        rh, rout, rv, rgc, _ws = ref_cuda.e0_forward(True, dev["x"], dev["h0"], dev["W_x"], dev["W_h"],
                                                     dev["W_gate"], dev["b"], dev["b_gate"])
        rr = ref_cuda.e0_backward(dev["W_x"], dev["W_h"], dev["W_gate"], dev["x"], rh, rv, rgc,
                                  dev["d_output"])
        torch.cuda.synchronize()
        theirs = dict(zip(("dx", "dW_x", "dW_h", "dW_gate", "db", "db_gate"), rr[:6]))
        theirs.update(h=rh, output=rout, v=rv, gate_cache=rgc)
        _versus_reference_cuda(got, theirs, truth, "E0 d1280")


def test_e5_config3_full_size_outputs_and_gradients():
    T, B, d, r = 512, 32, 1536, 270
    inp = orc.make_e5_inputs(T, B, d, r, seed=1237)
    before = _lib.tc_launch_count()
    got, ref = run_e5(inp, BF16)
    assert _lib.tc_launch_count() >= before + 2, "the low-rank tensor-core kernel was not used"
    assert _lib.device_status()[0] == 0
    truth = oracle_e5(ref)
    assert_close(errors(got, truth), TOL[BF16], "E5 configs[3] vs fp32 oracle")
    if ref_cuda.available():
        dev, _ = round_inputs(inp, BF16)
        w = [dev[k] for k in E5W]
        rh, rout, rv, _ws = ref_cuda.e5_forward(True, dev["x"], dev["h0"], *w, dev["b"])
        rr = ref_cuda.e5_backward(*w, dev["x"], rh, rv, dev["d_output"])
        torch.cuda.synchronize()
        theirs = dict(zip(("dx", "dU_h", "dV_h", "dU_x", "dV_x", "dU_z", "dV_z", "db"), rr[:8]))
        theirs.update(h=rh, output=rout, v=rv)
        # the reference adds its weight gradients in bf16 once per step: graded against the
        # fp32 result, with the reference's own distance as the allowance
        tol = TOL[BF16]
        for k in theirs:
            e_mine, e_ref = rel(got[k], truth[k]), rel(theirs[k], truth[k])
            assert e_mine < e_ref + tol, (k, e_mine, e_ref)


def test_e1_config4_shape_backward_matches_oracle():
    """d=2048, B=256 (configs[4] is forward-only; its backward runs the same plan family):
    a short sequence, every tensor against the fp32 oracle."""
    T, B, d = 12, 256, 2048
    inp = orc.make_e1_inputs(T, B, d, seed=1239)
    got, ref = run_e1(inp, BF16)
    assert _lib.device_status()[0] == 0
    assert_close(errors(got, oracle_e1(ref)), TOL[BF16], "E1 d2048 B256 vs fp32 oracle")
