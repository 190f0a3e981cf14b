"""E1 parity on the GPU: CUDA library (through the C ABI) vs the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from elman_b200 import _lib
from elman_b200 import hasty_pytorch_lib as H
from oracle import elman_oracle as orc
from tests._gpu_cases import TOL, assert_close, errors, option, oracle_e1, run_e1

pytestmark = pytest.mark.gpu

FWD_BWD_KEYS = ["h", "output", "v", "dx", "dz", "dW_x", "dW_h", "db"]


@pytest.mark.parametrize("T,B,d", [(1, 1, 8), (5, 3, 33), (16, 4, 64), (12, 9, 130), (40, 2, 256)])
def test_fp32_matches_oracle(T, B, d):
    inp = orc.make_e1_inputs(T, B, d, seed=100 + d)
    got, ref = run_e1(inp, torch.float32)
    assert_close(errors(got, oracle_e1(ref)), TOL[torch.float32], f"fp32 T{T} B{B} d{d}")


def test_fp32_config0_matches_reference_fixture(golden_dir):
    """configs[0]: fp32, B=4, T=128, d=256 against the reference's own outputs."""
    d = np.load(os.path.join(golden_dir, "e1_c0.npz"))
    T, B, dim, seed = (int(v) for v in d["meta"])
    inp = orc.make_e1_inputs(T, B, dim, seed=seed)
    got, _ = run_e1(inp, torch.float32)
    want = {k[4:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("out_")}
    assert_close(errors(got, want), TOL[torch.float32], "config0 vs reference fixture")


@pytest.mark.parametrize("name", ["e1_small", "e1_h0"])
def test_fp32_small_reference_fixtures(golden_dir, name):
    d = np.load(os.path.join(golden_dir, name + ".npz"))
    inp = {k[3:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("in_")}
    want = {k[4:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("out_")}
    got, _ = run_e1(inp, torch.float32)
    assert_close(errors(got, want), TOL[torch.float32], name)


@pytest.mark.parametrize("T,B,d", [(7, 3, 40), (24, 16, 128), (16, 32, 256)])
def test_bf16_cuda_core_path_matches_oracle(T, B, d):
    inp = orc.make_e1_inputs(T, B, d, seed=200 + d)
    with option("force_generic", 1):
        got, ref = run_e1(inp, torch.bfloat16)
    assert_close(errors(got, oracle_e1(ref)), TOL[torch.bfloat16], f"bf16 generic T{T} B{B} d{d}")


@pytest.mark.parametrize("T,B,d,ksplit", [(6, 16, 128, 1), (6, 16, 128, 2), (20, 32, 256, 4),
                                          (20, 32, 256, 2), (9, 16, 384, 2), (33, 32, 512, 8),
                                          (12, 64, 256, 4), (10, 48, 256, 4), (8, 8, 128, 2)])
def test_bf16_tensor_core_path_matches_oracle(T, B, d, ksplit):
    inp = orc.make_e1_inputs(T, B, d, seed=300 + d + ksplit)
    before = _lib.tc_launch_count()
    with option("rec_ksplit", ksplit):
        got, ref = run_e1(inp, torch.bfloat16)
    assert _lib.tc_launch_count() > before, "tensor-core kernels were not used"
    assert _lib.device_status()[0] == 0
    assert_close(errors(got, oracle_e1(ref)), TOL[torch.bfloat16],
                 f"bf16 tcgen05 T{T} B{B} d{d} S{ksplit}")


def test_bf16_batch_groups_pipeline_matches_oracle():
    inp = orc.make_e1_inputs(16, 64, 256, seed=77)
    for groups in (1, 2, 4):
        with option("rec_groups", groups), option("rec_ksplit", 4):
            got, ref = run_e1(inp, torch.bfloat16)
        assert_close(errors(got, oracle_e1(ref)), TOL[torch.bfloat16], f"groups={groups}")


def test_inference_mode_returns_empty_v_and_same_output():
    inp = orc.make_e1_inputs(10, 16, 128, seed=5)
    got_t, _ = run_e1(inp, torch.bfloat16, training=True)
    got_i, _ = run_e1(inp, torch.bfloat16, training=False)
    assert got_i["v"].numel() == 0
    assert torch.equal(got_t["output"], got_i["output"])
    assert torch.equal(got_t["h"], got_i["h"])


def test_nonzero_h0_and_bias():
    inp = orc.make_e1_inputs(9, 16, 128, seed=6)
    g = torch.Generator().manual_seed(1)
    inp["h0"] = 0.5 * torch.randn(16, 128, generator=g)
    inp["b"] = 0.2 * torch.randn(128, generator=g)
    for dtype in (torch.float32, torch.bfloat16):
        got, ref = run_e1(inp, dtype)
        assert_close(errors(got, oracle_e1(ref)), TOL[dtype], f"h0/bias {dtype}")


def test_results_are_bit_reproducible():
    """No float atomics anywhere: two runs give identical bits (the reference's db is not)."""
    inp = orc.make_e1_inputs(32, 32, 256, seed=8)
    a, _ = run_e1(inp, torch.bfloat16)
    b, _ = run_e1(inp, torch.bfloat16)
    for k in FWD_BWD_KEYS:
        assert torch.equal(a[k], b[k]), k


def test_config1_full_size_properties():
    """configs[1] (bf16, d=1280, B=32, T=512): size-independent properties at full size,
    plus the CPU oracle on a prefix of the sequence."""
    T, B, d = 512, 32, 1280
    inp = orc.make_e1_inputs(T, B, d, seed=1235)
    got, ref = run_e1(inp, torch.bfloat16)
    assert _lib.device_status()[0] == 0
    for k in FWD_BWD_KEYS:
        assert torch.isfinite(got[k].float()).all(), k
    # (1) tensor-core path agrees with the CUDA-core path of the same library
    with option("force_generic", 1):
        gen, _ = run_e1(inp, torch.bfloat16)
    assert_close({k: orc.rel_err(got[k].float().cpu(), gen[k].float().cpu()) for k in FWD_BWD_KEYS},
                 TOL[torch.bfloat16], "tcgen05 vs CUDA-core at config1")
    # (2) batch independence: rows 0..15 alone give the same forward result
    sub = {k: (v[:, :16].contiguous() if v.dim() == 3 else v) for k, v in inp.items()}
    sub["h0"] = inp["h0"][:16].contiguous()
    gsub, _ = run_e1(sub, torch.bfloat16, training=False)
    assert orc.rel_err(gsub["output"].float().cpu(), got["output"][:, :16].float().cpu()) < 1e-2
    # (3) causality + oracle: the first 24 steps match the CPU oracle on the same prefix
    Tp = 24
    pref = {k: (v[:Tp].contiguous() if v.dim() == 3 else v) for k, v in ref.items()}
    o = orc.e1_forward(pref["x"], pref["z"], pref["h0"], pref["W_x"], pref["W_h"], pref["b"])
    assert orc.rel_err(got["output"][:Tp].float().cpu(), o["output"]) < TOL[torch.bfloat16]
    assert orc.rel_err(got["h"][:Tp + 1].float().cpu(), o["h"]) < TOL[torch.bfloat16]
    # (4) backward is linear in d_output: grads(2r) = 2 grads(r)
    dev = {k: v.to(torch.bfloat16).cuda() for k, v in inp.items()}
    r2 = (dev["d_output"].float() * 2).to(torch.bfloat16)
    dx2, dz2, dWx2, dWh2, db2 = H.mamba_gated_elman_backward(
        dev["W_x"], dev["W_h"], dev["x"], dev["z"], got["h"], got["v"], r2)
    assert orc.rel_err(dx2.float().cpu(), 2 * got["dx"].float().cpu()) < 1e-2
    assert orc.rel_err(dWh2.float().cpu(), 2 * got["dW_h"].float().cpu()) < 1e-2


def test_argument_checks_raise():
    x = torch.zeros(4, 2, 8, device="cuda")
    W = torch.zeros(8, 8, device="cuda")
    b = torch.zeros(8, device="cuda")
    h0 = torch.zeros(2, 8, device="cuda")
    with pytest.raises(RuntimeError, match="CUDA"):
        H.mamba_gated_elman_forward(True, x.cpu(), x, h0, W, W, b)
    with pytest.raises(RuntimeError, match="contiguous"):
        H.mamba_gated_elman_forward(True, x.transpose(0, 1), x, h0, W, W, b)
    with pytest.raises(RuntimeError, match="shape"):
        H.mamba_gated_elman_forward(True, x, x, h0, W[:4], W, b)
    with pytest.raises(RuntimeError, match="dtype"):
        H.mamba_gated_elman_forward(True, x, x.half(), h0, W, W, b)
    with pytest.raises(RuntimeError, match="not supported"):
        H.mamba_gated_elman_forward(True, x.double(), x.double(), h0.double(), W.double(),
                                    W.double(), b.double())


def test_empty_sequence_and_empty_batch():
    W = torch.randn(8, 8, device="cuda")
    b = torch.zeros(8, device="cuda")
    h0 = torch.randn(2, 8, device="cuda")
    x = torch.zeros(0, 2, 8, device="cuda")
    h, out, v = H.mamba_gated_elman_forward(True, x, x, h0, W, W, b)
    assert h.shape == (1, 2, 8) and out.shape == (0, 2, 8)
    assert torch.equal(h[0], h0)
    dx, dz, dWx, dWh, db = H.mamba_gated_elman_backward(W, W, x, x, h, v, out)
    assert float(dWx.abs().sum()) == 0 and float(db.abs().sum()) == 0
    x0 = torch.zeros(3, 0, 8, device="cuda")
    h, out, v = H.mamba_gated_elman_forward(True, x0, x0, torch.zeros(0, 8, device="cuda"), W, W, b)
    assert out.shape == (3, 0, 8)


def test_wide_large_batch_forward_shape_of_config4():
    """configs[4] is forward-only bf16 d=2048, B=256, T=2048; same d and B here with a short T
    (the recurrence is the same program for any T): tensor-core path with 16 pipelined batch
    groups, against the CPU oracle on a prefix and against the CUDA-core path."""
    T, B, d = 24, 256, 2048
    inp = orc.make_e1_inputs(T, B, d, seed=1238)
    before = _lib.tc_launch_count()
    got, ref = run_e1(inp, torch.bfloat16, training=False)
    assert _lib.tc_launch_count() >= before + 2
    assert _lib.device_status()[0] == 0
    Tp = 6
    pref = {k: (v[:Tp].contiguous() if v.dim() == 3 else v) for k, v in ref.items()}
    o = orc.e1_forward(pref["x"], pref["z"], pref["h0"], pref["W_x"], pref["W_h"], pref["b"])
    assert orc.rel_err(got["output"][:Tp].float().cpu(), o["output"]) < TOL[torch.bfloat16]
    with option("force_generic", 1):
        gen, _ = run_e1(inp, torch.bfloat16, training=False)
    assert orc.rel_err(got["output"].float().cpu(), gen["output"].float().cpu()) < TOL[torch.bfloat16]
    assert orc.rel_err(got["h"].float().cpu(), gen["h"].float().cpu()) < TOL[torch.bfloat16]


@pytest.mark.parametrize("mode", [1, 2])
def test_both_publication_modes_give_identical_results(mode):
    inp = orc.make_e1_inputs(20, 32, 512, seed=31)
    a, _ = run_e1(inp, torch.bfloat16)
    with option("rec_direct_publish", mode):
        b, _ = run_e1(inp, torch.bfloat16)
    for k in FWD_BWD_KEYS:
        assert torch.equal(a[k], b[k]), k


def test_weights_in_tensor_memory_variant_is_bit_identical():
    """The recurrent weight tile as the MMAs' A operand from tensor memory (1, also the default
    where it fits) or from shared memory (2)."""
    inp = orc.make_e1_inputs(20, 32, 512, seed=32)
    default, _ = run_e1(inp, torch.bfloat16)
    with option("rec_w_tmem", 1):
        a, _ = run_e1(inp, torch.bfloat16)
    with option("rec_w_tmem", 2):
        b, _ = run_e1(inp, torch.bfloat16)
    for k in FWD_BWD_KEYS:
        assert torch.equal(a[k], b[k]) and torch.equal(default[k], b[k]), k


def test_host_pipeline_delivers_the_device_results():
    """E1HostPipeline (pinned host buffers in and out, three overlapping streams) returns bit
    for bit what the device-tensor functions return, for several calls in flight."""
    from elman_b200.host_io import E1HostPipeline
    T, B, d = 24, 32, 256
    calls = []
    for k in range(5):
        inp = orc.make_e1_inputs(T, B, d, seed=300 + k)
        calls.append({n: v.to(torch.bfloat16).contiguous().pin_memory() for n, v in inp.items()})
    w = {n: calls[0][n].cuda() for n in ("W_x", "W_h", "b", "h0")}
    pipe = E1HostPipeline(T, B, d, w["W_x"], w["W_h"], w["b"], w["h0"], depth=2)
    got = []
    for k, c in enumerate(calls):
        res = pipe.submit(c["x"], c["z"], c["d_output"])
        assert res["valid_until_call"] == k + 2   # the slot's host buffers are reused two calls later
        res["done"].synchronize()
        got.append({n: res[n].clone() for n in ("output", "dx", "dz", "dW_x", "dW_h", "db")})
    pipe.wait()
    for c, g in zip(calls, got):
        x, z, r = (c[n].cuda() for n in ("x", "z", "d_output"))
        h, out, v = H.mamba_gated_elman_forward(True, x, z, w["h0"], w["W_x"], w["W_h"], w["b"])
        dx, dz, dWx, dWh, db = H.mamba_gated_elman_backward(w["W_x"], w["W_h"], x, z, h, v, r)
        for n, t in (("output", out), ("dx", dx), ("dz", dz), ("dW_x", dWx), ("dW_h", dWh), ("db", db)):
            assert torch.equal(g[n], t.cpu()), n
    with pytest.raises(RuntimeError, match="pinned"):
        pipe.submit(calls[0]["x"].cuda(), calls[0]["z"], calls[0]["d_output"])


def test_weight_gradients_dual_launch_and_split_k_match_oracle():
    """T*B large against d: the dW GEMMs have few output tiles and a long K.  By default dW_x and
    dW_h (same first operand dv) run as ONE launch of the CTA-pair kernel; with the pair kernel
    off each is cut into K ranges with fp32 partial sums (deterministic reduce); with the
    persistent kernel off as well, one tile per block over the whole K."""
    inp = orc.make_e1_inputs(80, 32, 256, seed=77)
    got, ref = run_e1(inp, torch.bfloat16)
    assert_close(errors(got, oracle_e1(ref)), TOL[torch.bfloat16], "dual dW launch vs oracle")
    again, _ = run_e1(inp, torch.bfloat16)
    for k in ("dW_x", "dW_h", "dx"):
        assert torch.equal(got[k], again[k]), k
    with option("gemm_pair", 1):            # split-K through the persistent 128x256 kernel
        split, _ = run_e1(inp, torch.bfloat16)
        assert_close(errors(split, oracle_e1(ref)), TOL[torch.bfloat16], "split-K dW vs oracle")
        with option("gemm_persistent", 1):  # the 128x128 kernel, no K split
            plain, _ = run_e1(inp, torch.bfloat16)
    for k in ("dW_x", "dW_h"):
        assert orc.rel_err(got[k].float().cpu(), plain[k].float().cpu()) < 5e-3, k
        assert orc.rel_err(split[k].float().cpu(), plain[k].float().cpu()) < 5e-3, k


@pytest.mark.parametrize("T,B,d", [(6, 48, 256), (5, 64, 256), (4, 96, 384), (5, 128, 512),
                                   (3, 256, 512), (4, 160, 256), (3, 512, 256)])
def test_large_batch_plans_match_oracle(T, B, d):
    """Batches over 32 take the throughput plan (wide batch groups pipelined through the
    resident weight tile, publisher warp, W in tensor memory when needed): forward and
    backward against the oracle, and against the latency plan."""
    inp = orc.make_e1_inputs(T, B, d, seed=B + d)
    before = _lib.tc_launch_count()
    got, ref = run_e1(inp, torch.bfloat16)
    assert _lib.tc_launch_count() - before >= 2, "the recurrences must take the tcgen05 kernel"
    assert _lib.device_status()[0] == 0
    assert_close(errors(got, oracle_e1(ref)), TOL[torch.bfloat16], "throughput plan vs oracle")
    with option("rec_large_batch", 0):
        other, _ = run_e1(inp, torch.bfloat16)
    for k in ("h", "output", "dx", "dz"):
        assert orc.rel_err(got[k].float().cpu(), other[k].float().cpu()) < 1e-2, k


@pytest.mark.parametrize("T,B,d", [(5, 128, 512), (4, 256, 256), (3, 192, 384), (6, 256, 2048)])
def test_batch_replicas_of_the_grid_change_nothing(T, B, d):
    """Large batches run several independent copies of the recurrence grid, each on its own
    share of the batch groups (option rec_replicas).  Every sequence is computed by the same
    program either way: outputs and data gradients are bit-identical to the single-copy
    launch, weight gradients too, the bias gradient up to its order of summation."""
    inp = orc.make_e1_inputs(T, B, d, seed=B + d + 1)
    with option("rec_replicas", 1):
        one, ref = run_e1(inp, torch.bfloat16)
    many, _ = run_e1(inp, torch.bfloat16)          # default: as many copies as fit
    assert _lib.device_status()[0] == 0
    for k in ("h", "output", "v", "dx", "dz", "dW_x", "dW_h"):
        assert torch.equal(one[k], many[k]), k
    assert orc.rel_err(many["db"].float().cpu(), one["db"].float().cpu()) < 1e-2
    assert_close(errors(many, oracle_e1(ref)), TOL[torch.bfloat16], "replicated grid vs oracle")
    blocks_one = None
    with option("rec_replicas", 1):
        blocks_one = H.recurrence_blocks(torch.bfloat16, T, B, d)
    assert H.recurrence_blocks(torch.bfloat16, T, B, d) >= 2 * blocks_one, "replicas were not used"
