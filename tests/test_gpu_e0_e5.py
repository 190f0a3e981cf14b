"""E0 and E5 parity on the GPU: CUDA library (through the C ABI) vs the CPU oracle
and the fixtures the reference produced."""
import os

import numpy as np
import pytest
import torch

from oracle import elman_oracle as orc
from tests._gpu_cases import (TOL, assert_close, errors, option, oracle_e0, oracle_e5, run_e0,
                              run_e5)

pytestmark = pytest.mark.gpu


def fixture(golden_dir, name):
    d = np.load(os.path.join(golden_dir, name + ".npz"))
    inp = {k[3:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("in_")}
    want = {k[4:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("out_")}
    return inp, want


@pytest.mark.parametrize("name", ["e0_small", "e0_mid"])
def test_e0_fp32_reference_fixtures(golden_dir, name):
    inp, want = fixture(golden_dir, name)
    got, _ = run_e0(inp, torch.float32)
    assert_close(errors(got, want), TOL[torch.float32], name)


@pytest.mark.parametrize("T,B,d", [(3, 2, 17), (20, 4, 96)])
def test_e0_fp32_matches_oracle(T, B, d):
    inp = orc.make_e0_inputs(T, B, d, seed=400 + d)
    got, ref = run_e0(inp, torch.float32)
    assert_close(errors(got, oracle_e0(ref)), TOL[torch.float32], f"E0 fp32 {T},{B},{d}")


@pytest.mark.parametrize("T,B,d,generic", [(12, 16, 128, 1), (12, 16, 128, 0), (24, 32, 256, 0)])
def test_e0_bf16_matches_oracle(T, B, d, generic):
    inp = orc.make_e0_inputs(T, B, d, seed=500 + d)
    with option("force_generic", generic):
        got, ref = run_e0(inp, torch.bfloat16)
    assert_close(errors(got, oracle_e0(ref)), TOL[torch.bfloat16], f"E0 bf16 generic={generic}")


def test_e0_inference_mode():
    inp = orc.make_e0_inputs(6, 16, 128, seed=1)
    a, _ = run_e0(inp, torch.bfloat16, training=True)
    b, _ = run_e0(inp, torch.bfloat16, training=False)
    assert b["v"].numel() == 0 and b["gate_cache"].numel() == 0
    assert torch.equal(a["output"], b["output"])


@pytest.mark.parametrize("name", ["e5_small", "e5_mid"])
def test_e5_fp32_reference_fixtures(golden_dir, name):
    inp, want = fixture(golden_dir, name)
    got, _ = run_e5(inp, torch.float32)
    assert_close(errors(got, want), TOL[torch.float32], name)


@pytest.mark.parametrize("T,B,d,r", [(4, 2, 24, 5), (16, 4, 96, 20)])
def test_e5_fp32_matches_oracle(T, B, d, r):
    inp = orc.make_e5_inputs(T, B, d, r, seed=600 + d)
    got, ref = run_e5(inp, torch.float32)
    assert_close(errors(got, oracle_e5(ref)), TOL[torch.float32], f"E5 fp32 {T},{B},{d},{r}")


@pytest.mark.parametrize("T,B,d,r", [(12, 16, 128, 24), (16, 32, 256, 30), (8, 32, 1536, 270)])
def test_e5_bf16_matches_oracle(T, B, d, r):
    inp = orc.make_e5_inputs(T, B, d, r, seed=700 + d)
    got, ref = run_e5(inp, torch.bfloat16)
    assert_close(errors(got, oracle_e5(ref)), TOL[torch.bfloat16], f"E5 bf16 {T},{B},{d},{r}")


@pytest.mark.parametrize("T,B,d,r", [(16, 32, 256, 30), (20, 16, 512, 100), (10, 32, 1024, 200),
                                     (8, 32, 1536, 270), (9, 8, 256, 64)])
def test_e5_bf16_tensor_core_cluster_kernel_matches_oracle(T, B, d, r):
    """Shapes the single-cluster tcgen05 kernel takes (d/128 CTAs, rank chunks <= CTAs)."""
    from elman_b200 import _lib
    inp = orc.make_e5_inputs(T, B, d, r, seed=900 + d + r)
    before = _lib.tc_launch_count()
    got, ref = run_e5(inp, torch.bfloat16)
    # forward and backward recurrences plus tensor-core GEMMs where K allows it
    assert _lib.tc_launch_count() >= before + 2, "the low-rank tensor-core kernel was not used"
    assert _lib.device_status()[0] == 0
    assert_close(errors(got, oracle_e5(ref)), TOL[torch.bfloat16], f"E5 tcgen05 {T},{B},{d},{r}")
    with option("force_generic", 1):
        gen, _ = run_e5(inp, torch.bfloat16)
    assert_close({k: orc.rel_err(got[k].float().cpu(), gen[k].float().cpu()) for k in got
                  if got[k].numel()}, TOL[torch.bfloat16], "tcgen05 vs CUDA-core path")


def test_e5_bf16_results_are_bit_reproducible():
    inp = orc.make_e5_inputs(12, 32, 512, 96, seed=5)
    a, _ = run_e5(inp, torch.bfloat16)
    b, _ = run_e5(inp, torch.bfloat16)
    for k in a:
        assert torch.equal(a[k], b[k]), k
