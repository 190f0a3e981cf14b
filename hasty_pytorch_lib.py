"""`import hasty_pytorch_lib` — the module name the reference's model files probe for
(elman/models/mamba_gated_elman.py:23-27, stock_elman.py:18-24,
pure_lowrank_elman.py:21-25; the reference builds it with
elman/cuda/setup.py:67-77).  This top-level module re-exports the functions of
elman_b200.hasty_pytorch_lib under that name, so that a checkout of the reference finds
this library without any edit once the package is installed (or this directory is on
sys.path): its `hasattr(hasty_pytorch_lib, '<fn>')` probes succeed and its autograd
Functions call straight into libelman_b200.

Importing it loads the CUDA library; a missing build raises ImportError here, which
the reference's `try: import hasty_pytorch_lib` turns into its own Python fallback —
there is no fallback inside this package.
"""
from elman_b200 import _lib as _elman_lib
from elman_b200.hasty_pytorch_lib import *  # noqa: F401,F403
from elman_b200.hasty_pytorch_lib import (  # noqa: F401  (names without __all__)
    b2b_lowrank_elman_backward, b2b_lowrank_elman_forward, e1h_backward, e1h_forward,
    e33_self_gate_backward, e33_self_gate_forward, lowrank_elman_backward,
    lowrank_elman_forward,
    mamba_gated_elman_backward, mamba_gated_elman_forward, pure_lowrank_elman_backward,
    pure_lowrank_elman_backward_fused, pure_lowrank_elman_forward,
    pure_lowrank_elman_forward_fused, stock_elman_backward, stock_elman_forward)

_elman_lib.load()   # fail at import time, not at the first call, when the .so is missing
