"""Bounded device-side waits: a wait that cannot be satisfied gives up, records a
status the host reads, and leaves the context usable.  The failure is made on the
host side (a flag nothing sets); no kernel faults, traps or spins without a limit."""
import pytest
import torch

from elman_b200 import _lib
from elman_b200 import hasty_pytorch_lib as H

pytestmark = pytest.mark.gpu


def test_wait_probe_times_out_and_context_survives():
    lib = _lib.load()
    _lib.device_status(clear=True)
    scratch = torch.zeros(2, dtype=torch.int32, device="cuda")
    rc = lib.elman_b200_wait_probe(20000, scratch.data_ptr(),
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(scratch[1]) == 1, "the probe should have given up"
    code, detail = _lib.device_status()
    assert code == 3 and (detail >> 24) == 6
    # compute entry points refuse to run while the status word is set ...
    A = torch.randn(8, 8, device="cuda")
    with pytest.raises(_lib.ElmanB200Error, match="bounded"):
        H.projection(A, A)
    # ... and work again once it is cleared: the context is intact
    _lib.device_status(clear=True)
    out = H.projection(A, A)
    torch.cuda.synchronize()
    assert torch.allclose(out.cpu(), (A @ A.T).cpu(), atol=1e-4)


# ---------------------------------------------------------------------------
# The give-up paths of the kernels that carry the waits.  Option "test_stall_step"
# makes thread block 0 of the next tensor-core launch wait, at one step, for something
# nothing delivers; with a small "spin_limit" that wait — and then every other block's
# wait for block 0 — runs out within milliseconds.  Each kernel must return (abort word,
# drain, cluster barrier, tensor memory freed), the status word must name it, the next
# entry point must refuse, and after clearing the same call must match the oracle.
# ---------------------------------------------------------------------------
from oracle import elman_oracle as orc  # noqa: E402
from tests._gpu_cases import TOL, assert_close, errors, option, oracle_e1, oracle_e5  # noqa: E402
from tests._gpu_cases import round_inputs, run_e1, run_e5  # noqa: E402

KID_REC_TC_FWD, KID_REC_TC_BWD, KID_GEMM_TC, KID_LOWRANK_TC = 2, 3, 4, 7


def _expect_timeout(kernel_id):
    torch.cuda.synchronize()          # the launch returned: nothing hangs
    code, detail = _lib.device_status()
    assert code == 3, "the stalled launch should have recorded ELMAN_ERR_TIMEOUT"
    assert (detail >> 24) & 0xFF == kernel_id, f"status names kernel {(detail >> 24) & 0xFF}"
    A = torch.randn(8, 8, device="cuda")
    with pytest.raises(_lib.ElmanB200Error, match="bounded"):
        H.projection(A, A)            # entry points refuse while the word is set
    _lib.device_status(clear=True)


def test_recurrence_kernels_give_up_when_a_block_stalls_and_recover():
    T, B, d = 8, 16, 256
    inp = orc.make_e1_inputs(T, B, d, seed=41)
    dev, ref = round_inputs(inp, torch.bfloat16)
    _lib.device_status(clear=True)
    before = _lib.tc_launch_count()
    with option("spin_limit", 5000), option("test_stall_step", 5):
        H.mamba_gated_elman_forward(True, dev["x"], dev["z"], dev["h0"], dev["W_x"], dev["W_h"],
                                    dev["b"])
        _expect_timeout(KID_REC_TC_FWD)
    assert _lib.tc_launch_count() > before
    # a clean forward gives the states the backward needs; then stall the backward kernel
    h, out, v = H.mamba_gated_elman_forward(True, dev["x"], dev["z"], dev["h0"], dev["W_x"],
                                            dev["W_h"], dev["b"])
    with option("spin_limit", 5000), option("test_stall_step", 5):
        H.mamba_gated_elman_backward(dev["W_x"], dev["W_h"], dev["x"], dev["z"], h, v,
                                     dev["d_output"])
        _expect_timeout(KID_REC_TC_BWD)
    # the context is intact and the same calls are right again
    got, ref = run_e1(inp, torch.bfloat16)
    assert _lib.device_status()[0] == 0
    assert_close(errors(got, oracle_e1(ref)), TOL[torch.bfloat16], "after the give-up")


def test_lowrank_kernel_gives_up_when_a_block_withholds_its_share_and_recovers():
    T, B, d, r = 8, 16, 256, 64
    inp = orc.make_e5_inputs(T, B, d, r, seed=42)
    dev, _ = round_inputs(inp, torch.bfloat16)
    w = [dev[k] for k in ("U_h", "V_h", "U_x", "V_x", "U_z", "V_z")]
    _lib.device_status(clear=True)
    with option("spin_limit", 5000), option("test_stall_step", 5):
        H.pure_lowrank_elman_forward(True, dev["x"], dev["h0"], *w, dev["b"])
        _expect_timeout(KID_LOWRANK_TC)
    got, ref = run_e5(inp, torch.bfloat16)
    assert _lib.device_status()[0] == 0
    assert_close(errors(got, oracle_e5(ref)), TOL[torch.bfloat16], "after the give-up")


@pytest.mark.parametrize("pair", [1, 2])
@pytest.mark.parametrize("persistent", [1, 2])
def test_projection_gemm_gives_up_when_a_stage_never_lands_and_recovers(persistent, pair):
    M, N, K = 256, 256, 1024
    g = torch.Generator().manual_seed(43)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    W = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    _lib.device_status(clear=True)
    # persistent 1: one tile per block, 2: persistent kernel; pair 2: the CTA-pair kernel, where
    # the even CTA's stage barrier never completes and both CTAs must end
    with option("gemm_persistent", persistent), option("gemm_pair", pair):
        with option("spin_limit", 5000), option("test_stall_step", 5):
            H.gemm(H.GEMM_NT, A, W)
            _expect_timeout(KID_GEMM_TC)
        out = H.gemm(H.GEMM_NT, A, W)
    torch.cuda.synchronize()
    assert _lib.device_status()[0] == 0
    want = A.float() @ W.float().T
    assert orc.rel_err(out.float().cpu(), want.cpu()) < TOL[torch.bfloat16]
