"""The drop-in contract: `import hasty_pytorch_lib` resolves to this library, and the
reference's own, unmodified model files run on top of it.

The CPU tests check the module name, the function names, arities and return lengths the
reference's callers rely on (elman/cuda/pytorch/elman_ladder.cc:22-30, :86-94, :161-168,
:219-226, :2802-2812, :2871-2881, registered at :16539-16591).  The tests that load the
reference's `elman/models/*.py` need a checkout of the reference (ELMAN_REFERENCE_DIR);
they are skipped where there is none, e.g. on a GPU-only box.
"""
import importlib
import importlib.util
import inspect
import os
import sys

import pytest
import torch

from oracle import build_ref

REF_MODELS = os.path.join(build_ref.REFERENCE_DIR, "elman", "models")
needs_reference = pytest.mark.skipif(not os.path.isdir(REF_MODELS),
                                     reason="no checkout of the reference on this machine")

# name -> (positional parameters the reference's binding takes, length of the returned list)
REFERENCE_FUNCTIONS = {
    "stock_elman_forward": (8, 4), "stock_elman_backward": (8, 6),
    "mamba_gated_elman_forward": (7, 3), "mamba_gated_elman_backward": (7, 5),
    "pure_lowrank_elman_forward": (10, 3), "pure_lowrank_elman_backward": (10, 8),
    "pure_lowrank_elman_forward_fused": (10, 3), "pure_lowrank_elman_backward_fused": (10, 8),
    "b2b_lowrank_elman_forward": (10, 3), "b2b_lowrank_elman_backward": (10, 8),
    "e33_self_gate_forward": (6, 3), "e33_self_gate_backward": (6, 4),
    "lowrank_elman_forward": (8, 3), "lowrank_elman_backward": (8, 6),
    "e1h_forward": (6, 3), "e1h_backward": (6, 4),
}


def test_top_level_module_resolves_and_exports_the_reference_names():
    sys.modules.pop("hasty_pytorch_lib", None)
    mod = importlib.import_module("hasty_pytorch_lib")
    assert os.path.basename(mod.__file__) == "hasty_pytorch_lib.py"
    for name, (nargs, _) in REFERENCE_FUNCTIONS.items():
        assert hasattr(mod, name), name        # the reference probes with hasattr
        params = [p for p in inspect.signature(getattr(mod, name)).parameters.values()
                  if p.default is inspect.Parameter.empty]
        assert len(params) == nargs, f"{name} takes {len(params)} required arguments, not {nargs}"


def test_packaging_names_the_module_and_the_build_step():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "pyproject.toml")).read()
    assert 'py-modules = ["hasty_pytorch_lib"]' in text and 'packages = ["elman_b200"]' in text
    assert "nvcc_build.build" in open(os.path.join(root, "setup.py")).read()


def _load_reference(name):
    sys.modules.pop("hasty_pytorch_lib", None)
    spec = importlib.util.spec_from_file_location("reference_" + name,
                                                  os.path.join(REF_MODELS, name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@needs_reference
def test_reference_model_files_find_the_extension_unchanged():
    """Their `try: import hasty_pytorch_lib` probes succeed with nothing installed by hand."""
    assert _load_reference("mamba_gated_elman").MAMBA_CUDA_AVAILABLE is True
    assert _load_reference("stock_elman").HASTE_AVAILABLE is True
    assert _load_reference("pure_lowrank_elman").HASTY_AVAILABLE is True
    # siblings that run on the same functions (E32, E57: the E1 pair; E33: its own pair)
    assert _load_reference("e32_no_presilu").MAMBA_CUDA_AVAILABLE is True
    assert _load_reference("e33_self_gate").E33_CUDA_AVAILABLE is True
    assert _load_reference("lowrank_elman").HASTY_AVAILABLE is True       # E4
    assert _load_reference("e1_multihead").HAS_CUDA is True               # E1H


@needs_reference
@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_reference_cells_on_cuda_match_their_own_cpu_fallback(dtype, tol):
    """The reference's classes, loaded from its files: on CUDA they dispatch into this
    library, on the CPU they run their own Python loop.  Same weights, same inputs."""
    from oracle import elman_oracle as orc
    from elman_b200 import _lib
    T, B, d, r = 12, 4, 128, 24
    torch.manual_seed(11)
    cases = []
    m1 = _load_reference("mamba_gated_elman")
    cases.append((m1.MambaGatedElmanCell(d), lambda cell, x: cell(x, x.flip(0) * 0.5)))
    m0 = _load_reference("stock_elman")
    cases.append((m0.StockElmanCell(d, w_h_mode="free"), lambda cell, x: cell(x)))
    m5 = _load_reference("pure_lowrank_elman")
    cases.append((m5.PureLowRankElmanCell(d, rank=r), lambda cell, x: cell(x)))
    m4 = _load_reference("lowrank_elman")
    u0 = torch.randn(d)
    u0 = u0 / u0.norm()

    def call_e4(cell, x):    # its power iteration starts from a stored vector: pin it per pass
        cell._spectral_u = u0.to(x.device, x.dtype)
        return cell(x, x.flip(0) * 0.5)
    cases.append((m4.LowRankElmanCell(d, rank=r), call_e4))
    for cell, call in cases:
        cell = cell.to(dtype)
        x_cpu = torch.randn(T, B, d).to(dtype)
        r_cpu = torch.randn(T, B, d).to(dtype)
        ref_cell = cell.float()                       # their CPU loop, in fp32
        xc = x_cpu.float().requires_grad_(True)
        out_c, h_c = call(ref_cell, xc)
        (out_c * r_cpu.float()).sum().backward()
        want = {n: p.grad.clone() for n, p in ref_cell.named_parameters()}
        want_dx = xc.grad.clone()
        ref_cell.zero_grad()
        gpu_cell = ref_cell.to(dtype).cuda()
        xg = x_cpu.cuda().requires_grad_(True)
        before = _lib.launch_count()
        out_g, h_g = call(gpu_cell, xg)
        (out_g.float() * r_cpu.cuda().float()).sum().backward()
        torch.cuda.synchronize()
        assert _lib.launch_count() > before, "the reference class did not reach the CUDA library"
        assert orc.rel_err(out_g.float().cpu(), out_c.detach()) < tol
        assert orc.rel_err(h_g.float().cpu(), h_c.detach()) < tol
        assert orc.rel_err(xg.grad.float().cpu(), want_dx) < tol
        for n, p in gpu_cell.named_parameters():
            if want[n].abs().sum() > 0:
                assert orc.rel_err(p.grad.float().cpu(), want[n]) < tol, n
