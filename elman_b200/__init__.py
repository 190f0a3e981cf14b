"""elman_b200 — B200 (sm_100a) implementation of the E0 / E1 / E5 Elman-layer hot path.

Layout:
  csrc/                    CUDA kernels and the C ABI (include/elman_b200.h)
  hasty_pytorch_lib.py     the reference's extension-module functions on top of the C ABI
  mamba_gated_elman.py     E1: autograd Function, cell, layer (same API as the reference)
  stock_elman.py           E0
  pure_lowrank_elman.py    E5
  ladder_lm.py             the byte-level LM wrapper that calls the layers (caller of the path)
"""
import sys

__version__ = "0.1.0"


def install_as_hasty() -> None:
    """Make `import hasty_pytorch_lib` resolve to elman_b200.hasty_pytorch_lib.

    Call before importing the reference's `elman.models.*` modules; their
    `try: import hasty_pytorch_lib` probes then find this implementation and
    their autograd Functions call into it unchanged.
    """
    from . import hasty_pytorch_lib as mod
    sys.modules["hasty_pytorch_lib"] = mod
