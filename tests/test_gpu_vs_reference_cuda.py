"""The CUDA library against the REFERENCE's own CUDA kernels on the same GPU.

oracle/_ref/libelman_ref_cuda.so is the reference's unmodified kernel sources
compiled for sm_100 (oracle/build_ref.py).  Both implementations are also compared
with the fp32 CPU oracle: the reference rounds to bf16 at every intermediate, so
its own distance to the fp32 truth is the yardstick for "matches the reference".
"""
import pytest
import torch

from elman_b200 import hasty_pytorch_lib as H
from oracle import elman_oracle as orc
from oracle import ref_cuda
from tests._gpu_cases import TOL, oracle_e0, oracle_e1, oracle_e5, round_inputs

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_cuda.available(),
                                 reason="oracle/_ref/libelman_ref_cuda.so was not built")]


def rel(a, b):
    return orc.rel_err(a.float().cpu(), b.float().cpu())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,B,d", [(16, 4, 128), (48, 32, 256)])
def test_e1_matches_reference_cuda(dtype, T, B, d):
    inp = orc.make_e1_inputs(T, B, d, seed=800 + d)
    dev, ref = round_inputs(inp, dtype)
    h, out, v = H.mamba_gated_elman_forward(True, dev["x"], dev["z"], dev["h0"], dev["W_x"],
                                            dev["W_h"], dev["b"])
    mine = dict(zip(("dx", "dz", "dW_x", "dW_h", "db"),
                    H.mamba_gated_elman_backward(dev["W_x"], dev["W_h"], dev["x"], dev["z"], h, v,
                                                 dev["d_output"])))
    mine.update(h=h, output=out)
    rh, rout, rv, _ = ref_cuda.e1_forward(True, dev["x"], dev["z"], dev["h0"], dev["W_x"],
                                          dev["W_h"], dev["b"])
    rr = ref_cuda.e1_backward(dev["W_x"], dev["W_h"], dev["x"], dev["z"], rh, rv, dev["d_output"])
    theirs = dict(zip(("dx", "dz", "dW_x", "dW_h", "db"), rr[:5]))
    theirs.update(h=rh, output=rout)
    torch.cuda.synchronize()
    truth = oracle_e1(ref)
    for k in mine:
        e_mine, e_ref = rel(mine[k], truth[k]), rel(theirs[k], truth[k])
        assert rel(mine[k], theirs[k]) < TOL[dtype], f"{k}: vs reference CUDA"
        # never further from the fp32 truth than the tolerance, and not worse than the
        # reference's own rounding by more than that tolerance
        assert e_mine < TOL[dtype] and e_mine < e_ref + TOL[dtype], (k, e_mine, e_ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_e0_matches_reference_cuda(dtype):
    T, B, d = 24, 16, 128
    inp = orc.make_e0_inputs(T, B, d, seed=810)
    dev, ref = round_inputs(inp, dtype)
    h, out, v, gc = H.stock_elman_forward(True, dev["x"], dev["h0"], dev["W_x"], dev["W_h"],
                                          dev["W_gate"], dev["b"], dev["b_gate"])
    names = ("dx", "dW_x", "dW_h", "dW_gate", "db", "db_gate")
    mine = dict(zip(names, H.stock_elman_backward(dev["W_x"], dev["W_h"], dev["W_gate"], dev["x"],
                                                  h, v, gc, dev["d_output"])))
    mine.update(h=h, output=out)
    rh, rout, rv, rgc, _ = ref_cuda.e0_forward(True, dev["x"], dev["h0"], dev["W_x"], dev["W_h"],
                                               dev["W_gate"], dev["b"], dev["b_gate"])
    rr = ref_cuda.e0_backward(dev["W_x"], dev["W_h"], dev["W_gate"], dev["x"], rh, rv, rgc,
                              dev["d_output"])
    theirs = dict(zip(names, rr[:6]))
    theirs.update(h=rh, output=rout)
    torch.cuda.synchronize()
    truth = oracle_e0(ref)
    for k in mine:
        assert rel(mine[k], theirs[k]) < TOL[dtype], f"{k}: vs reference CUDA"
        assert rel(mine[k], truth[k]) < TOL[dtype], k


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_e5_matches_reference_cuda(dtype):
    T, B, d, r = 16, 8, 128, 24
    inp = orc.make_e5_inputs(T, B, d, r, seed=820)
    dev, ref = round_inputs(inp, dtype)
    w = [dev[k] for k in ("U_h", "V_h", "U_x", "V_x", "U_z", "V_z")]
    h, out, v = H.pure_lowrank_elman_forward(True, dev["x"], dev["h0"], *w, dev["b"])
    names = ("dx", "dU_h", "dV_h", "dU_x", "dV_x", "dU_z", "dV_z", "db")
    mine = dict(zip(names, H.pure_lowrank_elman_backward(*w, dev["x"], h, v, dev["d_output"])))
    mine.update(h=h, output=out)
    rh, rout, rv, _ = ref_cuda.e5_forward(True, dev["x"], dev["h0"], *w, dev["b"])
    rr = ref_cuda.e5_backward(*w, dev["x"], rh, rv, dev["d_output"])
    theirs = dict(zip(names, rr[:8]))
    theirs.update(h=rh, output=rout)
    torch.cuda.synchronize()
    truth = oracle_e5(ref)
    for k in mine:
        e_mine, e_ref = rel(mine[k], truth[k]), rel(theirs[k], truth[k])
        # the reference accumulates dU/dV in bf16 once per step; grade against the fp32 truth
        assert e_mine < TOL[dtype], (k, e_mine)
        assert e_mine < e_ref + TOL[dtype], (k, e_mine, e_ref)
