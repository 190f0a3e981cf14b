"""elman_e1_forward_static: the E1 forward pass for callers that cannot allocate.

Some users of the library cannot call cudaMalloc where they need the forward
pass: a plugin inside a host application that owns every byte of device memory,
code running in a section where an allocation (which may synchronise the
device) is not allowed, or a bare C caller without a workspace to hand in.  For
them the library carries its scratch in a built-in device array.  This test
calls that entry point through the C ABI, twice in a row on different inputs
(the array keeps the first call's contents, so the second call proves the
re-initialisation), and checks the outputs against the regular entry point.

It is collected last on purpose: should it fail, a run that stops at the first
failure has already executed every other test.
"""
import pytest
import torch

from elman_b200 import _lib
from oracle import elman_oracle as orc

pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2  # the tolerance the other bf16 parity tests use


def _device_inputs(T, B, d, seed):
    inp = orc.make_e1_inputs(T, B, d, seed=seed)
    return {k: v.to(torch.bfloat16).cuda().contiguous() for k, v in inp.items()}


def _forward(lib, static, dev, T, B, d):
    h = torch.empty(T + 1, B, d, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(T, B, d, dtype=torch.bfloat16, device="cuda")
    v = torch.empty(T, B, d, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    args = [_lib.ELMAN_BF16, 1, T, B, d, dev["x"].data_ptr(), dev["z"].data_ptr(),
            dev["h0"].data_ptr(), dev["W_x"].data_ptr(), dev["W_h"].data_ptr(),
            dev["b"].data_ptr(), h.data_ptr(), out.data_ptr(), v.data_ptr()]
    if static:
        rc = lib.elman_e1_forward_static(*args, stream)
        _lib.check(rc, "elman_e1_forward_static")
    else:
        nws = lib.elman_e1_forward_workspace(_lib.ELMAN_BF16, T, B, d)
        ws = torch.empty(nws, dtype=torch.uint8, device="cuda")
        rc = lib.elman_e1_forward(*args, ws.data_ptr(), ws.numel(), stream)
        _lib.check(rc, "elman_e1_forward")
        torch.cuda.synchronize()  # keep `ws` alive until the work is done
    torch.cuda.synchronize()
    return {"h": h, "output": out, "v": v}


def test_static_scratch_entry_point_matches_regular_one_twice_in_a_row():
    lib = _lib.load()
    T, B, d = 24, 32, 256
    assert lib.elman_e1_forward_workspace(_lib.ELMAN_BF16, T, B, d) <= \
        lib.elman_e1_forward_static_scratch_bytes()
    # the first call on a device looks up the array's address; do it before measuring
    _forward(lib, True, _device_inputs(T, B, d, 900), T, B, d)
    for seed in (901, 902):  # two calls in a row, different data
        dev = _device_inputs(T, B, d, seed)
        want = _forward(lib, False, dev, T, B, d)
        # device memory as the driver sees it (cudaMemGetInfo): an allocation made inside
        # the library, behind PyTorch's allocator, would show up here
        h = torch.empty(T + 1, B, d, dtype=torch.bfloat16, device="cuda")
        out = torch.empty(T, B, d, dtype=torch.bfloat16, device="cuda")
        v = torch.empty(T, B, d, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc = lib.elman_e1_forward_static(
            _lib.ELMAN_BF16, 1, T, B, d, dev["x"].data_ptr(), dev["z"].data_ptr(),
            dev["h0"].data_ptr(), dev["W_x"].data_ptr(), dev["W_h"].data_ptr(),
            dev["b"].data_ptr(), h.data_ptr(), out.data_ptr(), v.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "elman_e1_forward_static")
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before, "the call allocated device memory"
        assert _lib.device_status()[0] == 0
        got = {"h": h, "output": out, "v": v}
        # same kernels, same plan, same inputs: the results are the regular entry point's
        # bit for bit (tolerance 0; the bf16 parity tolerance applies against the oracle)
        for k in ("h", "output", "v"):
            assert torch.equal(got[k], want[k]), f"seed {seed}, {k} differs from elman_e1_forward"
        ref = {k: t.float().cpu() for k, t in dev.items()}
        o = orc.e1_forward(ref["x"], ref["z"], ref["h0"], ref["W_x"], ref["W_h"], ref["b"])
        for k in ("h", "output", "v"):
            err = orc.rel_err(got[k].float().cpu(), o[k])
            assert err < BF16_TOL, f"seed {seed}, {k}: rel err {err:.3e} vs the CPU oracle"


def test_static_scratch_entry_point_rejects_sizes_beyond_its_array():
    lib = _lib.load()
    T, B, d = 512, 32, 1280  # needs ~42 MB of scratch, the array holds 16 MiB
    assert lib.elman_e1_forward_workspace(_lib.ELMAN_BF16, T, B, d) > \
        lib.elman_e1_forward_static_scratch_bytes()
    one = torch.zeros(1, dtype=torch.bfloat16, device="cuda")
    p = one.data_ptr()
    rc = lib.elman_e1_forward_static(_lib.ELMAN_BF16, 1, T, B, d, p, p, p, p, p, p, p, p, p, None)
    assert rc == 4  # ELMAN_ERR_WORKSPACE, nothing was launched
    msg = lib.elman_b200_last_error().decode()
    assert "built-in array" in msg and "elman_e1_forward with a workspace" in msg
