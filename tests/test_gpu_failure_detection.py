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
