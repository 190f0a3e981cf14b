"""Host-side mirror classes (autograd Functions, cells, layers) on the CPU.

The CUDA library is replaced, in these tests only, by stand-ins built from the
CPU oracle, so that the Python plumbing (argument order, saved tensors, spectral
normalisation, the layer's projections and permutes) is checked against the
fixtures the reference produced.  The shipped classes themselves refuse CPU
tensors; the stand-ins lift that by patching `is_cuda` away from the call path.
"""
import os

import numpy as np
import pytest
import torch

from elman_b200 import mamba_gated_elman as e1mod
from elman_b200 import pure_lowrank_elman as e5mod
from elman_b200 import stock_elman as e0mod
from oracle import elman_oracle as orc


class OracleBackend:
    """Oracle-backed stand-in with the extension module's function names."""

    @staticmethod
    def mamba_gated_elman_forward(training, x, z, h0, W_x, W_h, b, flags=0):
        o = orc.e1_forward(x, z, h0, W_x, W_h, b)
        return [o["h"], o["output"], o["v"] if training else x.new_empty(0)]

    @staticmethod
    def mamba_gated_elman_backward(W_x, W_h, x, z, h, v, d_output):
        g = orc.e1_backward(W_x, W_h, x, z, h, v, d_output)
        return [g["dx"], g["dz"], g["dW_x"], g["dW_h"], g["db"]]

    @staticmethod
    def mamba_gated_elman_backward_carry(W_x, W_h, x, z, h, v, d_output, dv_in=None, flags=0):
        g = orc.e1_backward(W_x, W_h, x, z, h, v, d_output, dv_in)
        return [g["dx"], g["dz"], g["dW_x"], g["dW_h"], g["db"], g["dv0"]]

    GEMM_NT, GEMM_NN, GEMM_TN = 0, 1, 2

    @staticmethod
    def gemm(op, A, B, bias=None, out=None, accumulate=False):
        r = {0: lambda: A @ B.T, 1: lambda: A @ B, 2: lambda: A.T @ B}[op]()
        return r if bias is None else r + bias

    @staticmethod
    def column_sum(x):
        return x.sum(0)

    @staticmethod
    def in_proj_split_silu(u, W_in):
        xz = u @ W_in.T
        d = W_in.shape[0] // 2
        x_raw, z = xz[:, :d].contiguous(), xz[:, d:].contiguous()
        return x_raw, orc.silu(x_raw), z

    @staticmethod
    def silu_backward_concat(d_act, x_raw, dz):
        return torch.cat([d_act * orc.dsilu(x_raw), dz], dim=1)

    @staticmethod
    def add_rmsnorm_forward(x, residual_in, weight, eps):
        res = x.float() if residual_in is None else x.float() + residual_in
        v = res.to(x.dtype).float()
        rstd = torch.rsqrt(v.pow(2).mean(-1) + eps)
        y = (v * rstd[..., None] * weight.float()).to(x.dtype)
        return y, res, rstd.reshape(-1)

    @staticmethod
    def add_rmsnorm_backward(dy, dres_out, res_out, rstd, weight, want_dres_in, want_dx):
        D = dy.shape[-1]
        xh = res_out.to(dy.dtype).float() * rstd.reshape(*dy.shape[:-1], 1)
        g = dy.float() * weight.float()
        dxn = rstd.reshape(*dy.shape[:-1], 1) * (g - xh * (g * xh).mean(-1, keepdim=True))
        total = dxn if dres_out is None else dxn + dres_out
        dw = (dy.float() * xh).reshape(-1, D).sum(0).to(dy.dtype)
        return (total if want_dres_in else None), (total.to(dy.dtype) if want_dx else None), dw

    @staticmethod
    def e1_recurrence_forward(training, pre, z, h0, W_h, flags=0):
        d = pre.shape[-1]   # the recurrence alone = the cell with W_x = I, b = 0
        o = orc.e1_forward(pre, z, h0, torch.eye(d, dtype=pre.dtype), W_h, torch.zeros(d, dtype=pre.dtype))
        return [o["h"], o["output"], o["v"] if training else pre.new_empty(0)]

    @staticmethod
    def e1_recurrence_backward(W_h, z, h, v, d_output, dv_in=None, flags=0, W_h_T=None):
        T, B, d = z.shape
        g = orc.e1_backward(torch.eye(d, dtype=z.dtype), W_h, torch.zeros_like(z), z, h, v,
                            d_output, dv_in)
        carry = torch.zeros(1, B, d, dtype=z.dtype) if dv_in is None else dv_in[None]
        return [torch.cat([g["dx"], carry]), g["dz"], g["db"]]

    @staticmethod
    def e33_self_gate_forward(training, x, h0, W_x, W_h, b):
        o = orc.e33_forward(x, h0, W_x, W_h, b)
        return [o["h"], o["output"], o["v"] if training else x.new_empty(0)]

    @staticmethod
    def e33_self_gate_backward(W_x, W_h, x, h, v, d_output):
        g = orc.e33_backward(W_x, W_h, x, h, v, d_output)
        return [g["dx"], g["dW_x"], g["dW_h"], g["db"]]

    @staticmethod
    def e1h_forward(training, pre_x, z, h0, W_h, b_h):
        o = orc.e1h_forward(pre_x, z, h0, W_h, b_h)
        T = pre_x.shape[0]
        saved = torch.cat([o["h"], o["v"]]) if training else pre_x.new_empty(0)
        return [o["h"][T].clone(), o["output"], saved]

    @staticmethod
    def e1h_backward(pre_x, z, W_h, b_h, saved, d_output):
        T, B = pre_x.shape[:2]
        g = orc.e1h_backward(z, W_h, saved[:T + 1], saved[T + 1:], d_output)
        dW = torch.zeros((B,) + tuple(W_h.shape)); db = torch.zeros((B,) + tuple(b_h.shape))
        dW[0], db[0] = g["dW_h"], g["db"]
        return [g["d_pre_x"], g["dz"], dW, db]

    @staticmethod
    def lowrank_elman_forward(training, x, z, h0, W_x, U, V, b):
        o = orc.e4_forward(x, z, h0, W_x, U, V, b)
        return [o["h"], o["output"], o["v"] if training else x.new_empty(0)]

    @staticmethod
    def lowrank_elman_backward(W_x, U, V, x, z, h, v, d_output):
        g = orc.e4_backward(W_x, U, V, x, z, h, v, d_output)
        return [g[k] for k in ("dx", "dz", "dW_x", "dU", "dV", "db")]

    @staticmethod
    def stock_elman_forward(training, x, h0, W_x, W_h, W_gate, b, b_gate):
        o = orc.e0_forward(x, h0, W_x, W_h, W_gate, b, b_gate)
        e = x.new_empty(0)
        return [o["h"], o["output"], o["v"] if training else e, o["gate_cache"] if training else e]

    @staticmethod
    def stock_elman_backward(W_x, W_h, W_gate, x, h, v, gate_cache, d_output):
        g = orc.e0_backward(W_x, W_h, W_gate, x, h, v, gate_cache, d_output)
        return [g[k] for k in ("dx", "dW_x", "dW_h", "dW_gate", "db", "db_gate")]

    @staticmethod
    def pure_lowrank_elman_forward(training, x, h0, U_h, V_h, U_x, V_x, U_z, V_z, b):
        o = orc.e5_forward(x, h0, U_h, V_h, U_x, V_x, U_z, V_z, b)
        return [o["h"], o["output"], o["v"] if training else x.new_empty(0)]

    @staticmethod
    def pure_lowrank_elman_backward(U_h, V_h, U_x, V_x, U_z, V_z, x, h, v, d_output):
        g = orc.e5_backward(U_h, V_h, U_x, V_x, U_z, V_z, x, h, v, d_output)
        return [g[k] for k in ("dx", "dU_h", "dV_h", "dU_x", "dV_x", "dU_z", "dV_z", "db")]


def _e5_backward_carry(U_h, V_h, U_x, V_x, U_z, V_z, x, h, v, d_output, dv_in=None):
    g = orc.e5_backward(U_h, V_h, U_x, V_x, U_z, V_z, x, h, v, d_output, dv_in)
    return [g[k] for k in ("dx", "dU_h", "dV_h", "dU_x", "dV_x", "dU_z", "dV_z", "db", "dv0")]


OracleBackend.pure_lowrank_elman_backward_carry = staticmethod(_e5_backward_carry)


class _CpuAsCuda(torch.Tensor):
    """A CPU tensor that answers is_cuda=True so the cells' device check passes."""

    @property
    def is_cuda(self):
        return True


def as_fake_cuda(t):
    return t.as_subclass(_CpuAsCuda)


@pytest.fixture()
def oracle_backend(monkeypatch):
    from elman_b200 import fused_ops, siblings
    for mod in (e1mod, e0mod, e5mod, fused_ops, siblings):
        monkeypatch.setattr(mod, "hasty_pytorch_lib", OracleBackend)


def load(golden_dir, name):
    d = np.load(os.path.join(golden_dir, name + ".npz"))
    inp = {k[3:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("in_")}
    out = {k[4:]: torch.from_numpy(d[k]) for k in d.files if k.startswith("out_")}
    return inp, out


def test_cells_refuse_cpu_tensors():
    cell = e1mod.MambaGatedElmanCell(8)
    with pytest.raises(RuntimeError, match="CUDA"):
        cell(torch.zeros(2, 1, 8), torch.zeros(2, 1, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        e0mod.StockElmanCell(8)(torch.zeros(2, 1, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        e5mod.PureLowRankElmanCell(8, rank=2)(torch.zeros(2, 1, 8))


@pytest.mark.parametrize("name,spectral", [("e1_small", False), ("e1_h0", False),
                                           ("e1_spectral", True)])
def test_e1_cell_against_reference_fixture(golden_dir, oracle_backend, name, spectral):
    inp, want = load(golden_dir, name)
    d = inp["W_x"].shape[0]
    cell = e1mod.MambaGatedElmanCell(d, w_h_mode="spectral_norm" if spectral else "none")
    with torch.no_grad():
        cell.W_x.copy_(inp["W_x"]); cell.W_h.copy_(inp["W_h"]); cell.b.copy_(inp["b"])
    if spectral:
        cell._spectral_u = inp["spectral_u"].clone()
    x = as_fake_cuda(inp["x"].clone()).requires_grad_(True)
    z = as_fake_cuda(inp["z"].clone()).requires_grad_(True)
    out, h = cell(x, z, inp["h0"])
    (out * inp["d_output"]).sum().backward()
    got = {"output": out, "h": h, "dx": x.grad, "dz": z.grad, "dW_x": cell.W_x.grad,
           "dW_h": cell.W_h.grad, "db": cell.b.grad}
    for k, vref in want.items():
        assert orc.rel_err(got[k], vref) < 2e-5, k


def test_e1_layer_against_reference_fixture(golden_dir, oracle_backend):
    inp, want = load(golden_dir, "e1_layer")
    dim = inp["x"].shape[-1]
    layer = e1mod.MambaGatedElman(dim, expansion=1.0)
    sd = {k[2:]: v for k, v in inp.items() if k.startswith("p_")}
    assert set(sd) == set(layer.state_dict()), "parameter names differ from the reference's"
    layer.load_state_dict(sd)
    x = as_fake_cuda(inp["x"].clone()).requires_grad_(True)
    out, h_final = layer(x)
    (out * inp["d_output"]).sum().backward()
    assert orc.rel_err(out, want["output"]) < 2e-5
    assert orc.rel_err(h_final, want["h_final"]) < 2e-5
    assert orc.rel_err(x.grad, want["dx"]) < 2e-5
    for k, p in layer.named_parameters():
        assert orc.rel_err(p.grad, want["g_" + k]) < 5e-5, k


def test_e0_cell_against_reference_fixture(golden_dir, oracle_backend):
    inp, want = load(golden_dir, "e0_small")
    d = inp["W_x"].shape[0]
    cell = e0mod.StockElmanCell(d, w_h_mode="free")
    with torch.no_grad():
        for k in ("W_x", "W_h", "W_gate", "b", "b_gate"):
            getattr(cell, k).copy_(inp[k])
    x = as_fake_cuda(inp["x"].clone()).requires_grad_(True)
    out, h = cell(x, inp["h0"])
    (out * inp["d_output"]).sum().backward()
    got = {"output": out, "h": h, "dx": x.grad, "dW_x": cell.W_x.grad, "dW_h": cell.W_h.grad,
           "dW_gate": cell.W_gate.grad, "db": cell.b.grad, "db_gate": cell.b_gate.grad}
    for k, vref in want.items():
        assert orc.rel_err(got[k], vref) < 2e-5, k


def test_e5_cell_against_reference_fixture(golden_dir, oracle_backend):
    inp, want = load(golden_dir, "e5_small")
    d, r = inp["U_h"].shape
    cell = e5mod.PureLowRankElmanCell(d, rank=r)
    with torch.no_grad():
        for k in ("U_h", "V_h", "U_x", "V_x", "U_z", "V_z", "b"):
            getattr(cell, k).copy_(inp[k])
    x = as_fake_cuda(inp["x"].clone()).requires_grad_(True)
    out, h = cell(x, inp["h0"])
    (out * inp["d_output"]).sum().backward()
    got = {"output": out, "h": h, "dx": x.grad, "db": cell.b.grad}
    for k in ("U_h", "V_h", "U_x", "V_x", "U_z", "V_z"):
        got["d" + k] = getattr(cell, k).grad
    for k, vref in want.items():
        assert orc.rel_err(got[k], vref) < 2e-5, k


def test_state_dict_names_match_reference_layout():
    assert set(e0mod.StockElman(16).state_dict()) == {
        "in_proj.weight", "cell.W_x", "cell.b", "cell.W_gate", "cell.b_gate", "cell.W_h",
        "out_proj.weight"}
    assert set(e5mod.PureLowRankElman(16, rank=4).state_dict()) == {
        "cell.U_h", "cell.V_h", "cell.U_x", "cell.V_x", "cell.U_z", "cell.V_z", "cell.b"}


@pytest.mark.parametrize("cuts", [(0, 3, 5), (0, 1), (0,)])
def test_e1_layer_in_time_chunks_equals_reference_fixture(golden_dir, oracle_backend, cuts):
    """forward_chunk chained over time chunks (state forward, pre-activation gradient
    backward) reproduces the reference layer's whole-sequence output and gradients."""
    inp, want = load(golden_dir, "e1_layer")
    dim = inp["x"].shape[-1]
    layer = e1mod.MambaGatedElman(dim, expansion=1.0)
    layer.load_state_dict({k[2:]: v for k, v in inp.items() if k.startswith("p_")})
    x = inp["x"].clone().requires_grad_(True)
    B, T, _ = x.shape
    edges = list(cuts) + [T]
    W_h = layer.chunk_weights()
    state = torch.zeros(B, layer.d_inner)
    outs = []
    for t0, t1 in zip(edges[:-1], edges[1:]):
        out, state = layer.forward_chunk(x[:, t0:t1], state, W_h)
        outs.append(out)
    out = torch.cat(outs, dim=1)
    (out * inp["d_output"]).sum().backward()
    got = {"output": out, "h_final": state, "dx": x.grad}
    for n, p_ in layer.named_parameters():
        got["g_" + n] = p_.grad
    checked = 0
    for k, vref in want.items():
        if k in got:
            assert orc.rel_err(got[k], vref) < 2e-5, k
            checked += 1
    assert checked >= 4


@pytest.mark.parametrize("cuts", [(0, 3, 5), (0,)])
def test_e1_layer_split_chunk_pieces_equal_reference_fixture(golden_dir, oracle_backend, cuts):
    """chunk_pre / chunk_rec / chunk_post (time-major, the projection node returning dW_h
    from the states the recurrence node leaves in the link) reproduce the reference layer."""
    inp, want = load(golden_dir, "e1_layer")
    dim = inp["x"].shape[-1]
    layer = e1mod.MambaGatedElman(dim, expansion=1.0)
    layer.load_state_dict({k[2:]: v for k, v in inp.items() if k.startswith("p_")})
    x = inp["x"].clone().requires_grad_(True)
    B, T, _ = x.shape
    edges = list(cuts) + [T]
    W_h = layer.chunk_weights()
    state = torch.zeros(B, layer.d_inner)
    outs = []
    for t0, t1 in zip(edges[:-1], edges[1:]):
        link = e1mod.ChunkLink()
        pre, z = layer.chunk_pre(x[:, t0:t1].transpose(0, 1).contiguous(), W_h, link)
        cell_out, state = layer.chunk_rec(pre, z, state, W_h, link)
        outs.append(layer.chunk_post(cell_out).transpose(0, 1))
    out = torch.cat(outs, dim=1)
    (out * inp["d_output"]).sum().backward()
    got = {"output": out, "h_final": state, "dx": x.grad}
    for n, p_ in layer.named_parameters():
        got["g_" + n] = p_.grad
    checked = 0
    for k, vref in want.items():
        if k in got:
            assert orc.rel_err(got[k], vref) < 2e-5, k
            checked += 1
    assert checked >= 7


def test_e0_layer_chunk_pieces_equal_whole_layer(oracle_backend):
    """StockElman's chunk_pre / chunk_rec / chunk_post (E1's projection and recurrence nodes
    with the gate from a second projection) reproduce its own whole-sequence forward()."""
    torch.manual_seed(3)
    dim, B, T = 24, 2, 7
    layer = e0mod.StockElman(dim, expansion=1.0, r_h_mode="free")
    x1 = as_fake_cuda(torch.randn(B, T, dim)).requires_grad_(True)
    d_out = torch.randn(B, T, dim)
    out1, h1 = layer(x1)
    (out1 * d_out).sum().backward()
    want = {n: p_.grad.clone() for n, p_ in layer.named_parameters()}
    want_dx = x1.grad.clone()
    layer.zero_grad()
    x2 = torch.Tensor(x1.detach().clone()).requires_grad_(True)
    W_h = layer.chunk_weights()
    state = torch.zeros(B, layer.d_inner)
    outs = []
    for t0, t1 in ((0, 3), (3, 4), (4, 7)):
        link = e1mod.ChunkLink()
        pre, gate = layer.chunk_pre(x2[:, t0:t1].transpose(0, 1).contiguous(), W_h, link)
        cell_out, state = layer.chunk_rec(pre, gate, state, W_h, link)
        outs.append(layer.chunk_post(cell_out).transpose(0, 1))
    out2 = torch.cat(outs, dim=1)
    (out2 * d_out).sum().backward()
    assert orc.rel_err(out2, torch.Tensor(out1.detach())) < 1e-5
    assert orc.rel_err(state, torch.Tensor(h1.detach())) < 1e-5
    assert orc.rel_err(x2.grad, torch.Tensor(want_dx)) < 1e-5
    for n, p_ in layer.named_parameters():
        assert orc.rel_err(p_.grad, want[n]) < 1e-5, n


def test_e5_layer_chunk_pieces_equal_whole_layer(oracle_backend):
    """PureLowRankElman in time chunks (state forward, pre-activation gradient backward)
    reproduces its own whole-sequence forward() and gradients."""
    torch.manual_seed(4)
    dim, B, T = 24, 2, 7
    layer = e5mod.PureLowRankElman(dim, rank=5)
    x1 = as_fake_cuda(torch.randn(B, T, dim)).requires_grad_(True)
    d_out = torch.randn(B, T, dim)
    out1, h1 = layer(x1)
    (out1 * d_out).sum().backward()
    want = {n: p_.grad.clone() for n, p_ in layer.named_parameters()}
    want_dx = x1.grad.clone()
    layer.zero_grad()
    x2 = torch.Tensor(x1.detach().clone()).requires_grad_(True)
    state = torch.zeros(B, dim)
    outs = []
    for t0, t1 in ((0, 2), (2, 3), (3, 7)):
        pre, z = layer.chunk_pre(x2[:, t0:t1].transpose(0, 1), None, None)
        cell_out, state = layer.chunk_rec(pre, z, state, None, None)
        outs.append(layer.chunk_post(cell_out).transpose(0, 1))
    out2 = torch.cat(outs, dim=1)
    (out2 * d_out).sum().backward()
    assert orc.rel_err(out2, torch.Tensor(out1.detach())) < 1e-5
    assert orc.rel_err(state, torch.Tensor(h1.detach())) < 1e-5
    assert orc.rel_err(x2.grad, torch.Tensor(want_dx)) < 1e-5
    for n, p_ in layer.named_parameters():
        assert orc.rel_err(p_.grad, want[n]) < 1e-5, n


def test_graphed_step_raises_when_the_status_word_reports_a_timeout(monkeypatch):
    """A graph replay calls no library entry point, so nothing else would look at the status
    word: the step wrapper reads it and raises."""
    from elman_b200 import _lib, train_step
    monkeypatch.setattr(_lib, "device_status", lambda clear=False: (0, 0))
    train_step.raise_on_device_timeout()          # clean: no exception
    monkeypatch.setattr(_lib, "device_status", lambda clear=False: (3, (3 << 24) | 17))
    with pytest.raises(_lib.ElmanB200Error, match="kernel 3, step 17"):
        train_step.raise_on_device_timeout()

    class _Graph:
        replays = 0

        def replay(self):
            self.replays += 1

    step = train_step.GraphedTrainStep.__new__(train_step.GraphedTrainStep)
    step.tokens, step.graph, step.loss = torch.zeros(2), _Graph(), torch.tensor(1.0)
    with pytest.raises(_lib.ElmanB200Error):
        step(torch.ones(2))
    assert step.graph.replays == 0                # the poisoned step was not replayed
    monkeypatch.setattr(_lib, "device_status", lambda clear=False: (0, 0))
    step(torch.ones(2))
    assert step.graph.replays == 1 and step.loss_value() == 1.0


@pytest.mark.parametrize("name,cls,kw", [("e32_layer", "E32NoPresilu", {}),
                                         ("e33_layer", "E33SelfGate", {"r_h_mode": "spectral_norm"}),
                                         ("e57_layer", "E57LearnedRadius", {"expansion": 1.0}),
                                         ("e4_layer", "LowRankElman", {"rank": 24})])
def test_sibling_layers_against_reference_fixtures(golden_dir, oracle_backend, name, cls, kw):
    """E4 / E32 / E33 / E57 (the reference's ladder levels that run on the E1 and E5 recurrences) against
    what the reference's own files computed: outputs, state, every parameter gradient."""
    from elman_b200 import siblings
    inp, want = load(golden_dir, name)
    layer = getattr(siblings, cls)(inp["x"].shape[-1], **kw)
    sd = {k[2:]: v for k, v in inp.items() if k.startswith("p_")}
    assert set(sd) == set(layer.state_dict()), "parameter names differ from the reference's"
    layer.load_state_dict(sd)
    layer.cell._spectral_u = inp["spectral_u"].clone()
    x = as_fake_cuda(inp["x"].clone()).requires_grad_(True)
    out, h_final = layer(x)
    (out * inp["d_output"]).sum().backward()
    assert orc.rel_err(out, want["output"]) < 2e-5
    assert orc.rel_err(h_final, want["h_final"]) < 2e-5
    assert orc.rel_err(x.grad, want["dx"]) < 2e-5
    for k, p in layer.named_parameters():
        assert orc.rel_err(p.grad, want["g_" + k]) < 5e-5, k


def test_e1h_layer_against_reference_fixture(golden_dir, oracle_backend):
    """The multi-head E1 layer against what the reference's own file computed (its PyTorch
    loop): output, final state, every parameter gradient; same parameter names."""
    from elman_b200 import siblings
    inp, want = load(golden_dir, "e1h_layer")
    layer = siblings.E1MultiHead(64, n_heads=4, n_state=16)
    sd = {k[2:]: v for k, v in inp.items() if k.startswith("p_")}
    assert set(sd) == set(layer.state_dict()), "parameter names differ from the reference's"
    layer.load_state_dict(sd)
    x = as_fake_cuda(inp["x"].clone()).requires_grad_(True)
    out, h_final = layer(x)
    (out * inp["d_output"]).sum().backward()
    assert orc.rel_err(out, want["output"]) < 2e-5
    assert orc.rel_err(h_final, want["h_final"]) < 2e-5
    assert orc.rel_err(x.grad, want["dx"]) < 2e-5
    for k, p in layer.named_parameters():
        assert orc.rel_err(p.grad, want["g_" + k]) < 5e-5, k


def test_oracle_e1h_explicit_backward_equals_autograd():
    g0 = torch.Generator().manual_seed(8)
    T, B, Hh, N = 6, 3, 4, 8
    px, z, dy = (torch.randn(T, B, Hh, N, generator=g0) for _ in range(3))
    h0 = 0.1 * torch.randn(B, Hh, N, generator=g0)
    W, b = 0.3 * torch.randn(Hh, N, N, generator=g0), 0.1 * torch.randn(Hh, N, generator=g0)
    f = orc.e1h_forward(px, z, h0, W, b)
    g = orc.e1h_backward(z, W, f["h"], f["v"], dy)
    leaves = [t.clone().requires_grad_(True) for t in (px, z, W, b)]
    o = orc.e1h_forward(leaves[0], leaves[1], h0, leaves[2], leaves[3])
    (o["output"] * dy).sum().backward()
    for k, t in zip(("d_pre_x", "dz", "dW_h", "db"), leaves):
        assert orc.rel_err(g[k], t.grad) < 1e-5, k


def test_oracle_e4_explicit_backward_equals_autograd():
    inp = orc.make_e1_inputs(7, 3, 24, seed=5)
    g0 = torch.Generator().manual_seed(6)
    U, V = 0.3 * torch.randn(24, 5, generator=g0), 0.3 * torch.randn(5, 24, generator=g0)
    f = orc.e4_forward(inp["x"], inp["z"], inp["h0"], inp["W_x"], U, V, inp["b"])
    g = orc.e4_backward(inp["W_x"], U, V, inp["x"], inp["z"], f["h"], f["v"], inp["d_output"])
    leaves = [t.clone().requires_grad_(True) for t in (inp["x"], inp["z"], inp["W_x"], U, V, inp["b"])]
    o = orc.e4_forward(leaves[0], leaves[1], inp["h0"], *leaves[2:])
    (o["output"] * inp["d_output"]).sum().backward()
    for k, t in zip(("dx", "dz", "dW_x", "dU", "dV", "db"), leaves):
        assert orc.rel_err(g[k], t.grad) < 1e-5, k


def test_oracle_e33_explicit_backward_equals_autograd():
    inp = orc.make_e1_inputs(7, 3, 24, seed=4)
    f = orc.e33_forward(inp["x"], inp["h0"], inp["W_x"], inp["W_h"], inp["b"])
    g = orc.e33_backward(inp["W_x"], inp["W_h"], inp["x"], f["h"], f["v"], inp["d_output"])
    leaves = [inp[k].clone().requires_grad_(True) for k in ("x", "W_x", "W_h", "b")]
    o = orc.e33_forward(leaves[0], inp["h0"], leaves[1], leaves[2], leaves[3])
    (o["output"] * inp["d_output"]).sum().backward()
    for k, t in zip(("dx", "dW_x", "dW_h", "db"), leaves):
        assert orc.rel_err(g[k], t.grad) < 1e-5, k
