"""Generate the golden fixtures in this directory from the REFERENCE's own code.

Run once, in a container that has a checkout of the reference:

    python tests/golden/make_golden.py --reference /path/to/reference

It loads the reference's three model files directly (without importing the
whole `elman.models` package), builds its cells, overwrites their parameters
with seeded values, runs the cells' Python forward loops on the CPU with
autograd for the backward pass, and stores inputs, outputs and gradients as
`.npz` files.  The fixtures are what pins `oracle/elman_oracle.py` and the
host-side mirror classes to the reference; the test-suite never needs the
reference checkout itself.
"""

from __future__ import annotations

import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from oracle.elman_oracle import make_e0_inputs, make_e1_inputs, make_e5_inputs  # noqa: E402


def load_ref(root: str, name: str):
    path = os.path.join(root, "elman", "models", name + ".py")
    spec = importlib.util.spec_from_file_location("reference_" + name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def to_np(d):
    return {k: v.detach().cpu().numpy() for k, v in d.items()}


def save(name, store_inputs, inputs, outputs, meta):
    payload = {}
    if store_inputs:
        payload.update({"in_" + k: v for k, v in to_np(inputs).items()})
    else:
        # inputs are regenerated from the seed; keep a checksum to catch RNG drift
        payload["in_checksum"] = np.array(
            [float(v.double().abs().sum()) for v in inputs.values()], dtype=np.float64)
    payload.update({"out_" + k: v for k, v in to_np(outputs).items()})
    payload["meta"] = np.array(meta, dtype=np.int64)
    np.savez(os.path.join(HERE, name + ".npz"), **payload)
    print("wrote", name, {k: v.shape for k, v in payload.items()})


def run_e1(mod, T, B, d, seed, h0_random=False, spectral=False):
    inp = make_e1_inputs(T, B, d, seed=seed)
    if h0_random:
        g = torch.Generator().manual_seed(seed + 77)
        inp["h0"] = 0.5 * torch.randn(B, d, generator=g)
    cell = mod.MambaGatedElmanCell(d, w_h_mode="spectral_norm" if spectral else "none")
    with torch.no_grad():
        cell.W_x.copy_(inp["W_x"])
        cell.W_h.copy_(inp["W_h"])
        cell.b.copy_(inp["b"])
    if spectral:
        g = torch.Generator().manual_seed(seed + 5)
        u = torch.randn(d, generator=g)
        cell._spectral_u = u / u.norm()
        inp["spectral_u"] = cell._spectral_u.clone()
    x = inp["x"].clone().requires_grad_(True)
    z = inp["z"].clone().requires_grad_(True)
    out, h = cell(x, z, inp["h0"])
    (out * inp["d_output"]).sum().backward()
    res = {"output": out, "h": h, "dx": x.grad, "dz": z.grad, "dW_x": cell.W_x.grad,
           "dW_h": cell.W_h.grad, "db": cell.b.grad}
    return inp, res


def run_e0(mod, T, B, d, seed):
    inp = make_e0_inputs(T, B, d, seed=seed)
    cell = mod.StockElmanCell(d, w_h_mode="free")
    with torch.no_grad():
        cell.W_x.copy_(inp["W_x"])
        cell.W_h.copy_(inp["W_h"])
        cell.W_gate.copy_(inp["W_gate"])
        cell.b.copy_(inp["b"])
        cell.b_gate.copy_(inp["b_gate"])
    x = inp["x"].clone().requires_grad_(True)
    out, h = cell(x, inp["h0"])
    (out * inp["d_output"]).sum().backward()
    res = {"output": out, "h": h, "dx": x.grad, "dW_x": cell.W_x.grad, "dW_h": cell.W_h.grad,
           "dW_gate": cell.W_gate.grad, "db": cell.b.grad, "db_gate": cell.b_gate.grad}
    return inp, res


def run_e5(mod, T, B, d, r, seed):
    inp = make_e5_inputs(T, B, d, r, seed=seed)
    cell = mod.PureLowRankElmanCell(d, rank=r)
    with torch.no_grad():
        for k in ("U_h", "V_h", "U_x", "V_x", "U_z", "V_z", "b"):
            getattr(cell, k).copy_(inp[k])
    x = inp["x"].clone().requires_grad_(True)
    out, h = cell(x, inp["h0"])
    (out * inp["d_output"]).sum().backward()
    res = {"output": out, "h": h, "dx": x.grad, "db": cell.b.grad}
    for k in ("U_h", "V_h", "U_x", "V_x", "U_z", "V_z"):
        res["d" + k] = getattr(cell, k).grad
    return inp, res


def run_e1_layer(mod, B, T, dim, seed):
    """The whole E1 layer (in_proj, silu, cell, out_proj) with its default init."""
    torch.manual_seed(seed)
    layer = mod.MambaGatedElman(dim, expansion=1.0)
    g = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(B, T, dim, generator=g)
    r = torch.randn(B, T, dim, generator=g)
    xin = x.clone().requires_grad_(True)
    out, h_final = layer(xin)
    (out * r).sum().backward()
    inp = {"x": x, "d_output": r}
    inp.update({"p_" + k: v.detach().clone() for k, v in layer.state_dict().items()})
    res = {"output": out, "h_final": h_final, "dx": xin.grad}
    res.update({"g_" + k: p.grad for k, p in layer.named_parameters()})
    return inp, res


def run_sibling_layer(mod, cls_name, B, T, dim, seed, **kw):
    """A whole sibling layer of E1 (E32 / E33 / E57) from the reference's own file, default
    init, power-iteration start vector pinned where the cell normalises W_h."""
    torch.manual_seed(seed)
    layer = getattr(mod, cls_name)(dim, **kw)
    g = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(B, T, dim, generator=g)
    r = torch.randn(B, T, dim, generator=g)
    u = torch.randn(layer.d_inner, generator=g)
    layer.cell._spectral_u = u / u.norm()
    inp = {"x": x, "d_output": r, "spectral_u": layer.cell._spectral_u.clone()}
    inp.update({"p_" + k: v.detach().clone() for k, v in layer.state_dict().items()})
    xin = x.clone().requires_grad_(True)
    out, h_final = layer(xin)
    (out * r).sum().backward()
    res = {"output": out, "h_final": h_final, "dx": xin.grad}
    res.update({"g_" + k: p.grad for k, p in layer.named_parameters()})
    return inp, res


def run_e1h_layer(mod, B, T, dim, seed, **kw):
    """The reference's multi-head E1 layer (elman/models/e1_multihead.py) through its own
    PyTorch loop (`_forward_pytorch`, the path it takes off CUDA), default init."""
    torch.manual_seed(seed)
    layer = mod.E1MultiHead(dim, **kw)
    g = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(B, T, dim, generator=g)
    r = torch.randn(B, T, dim, generator=g)
    inp = {"x": x, "d_output": r}
    inp.update({"p_" + k: v.detach().clone() for k, v in layer.state_dict().items()})
    xin = x.clone().requires_grad_(True)
    out, h_final = layer(xin)
    (out * r).sum().backward()
    res = {"output": out, "h_final": h_final, "dx": xin.grad}
    res.update({"g_" + k: p.grad for k, p in layer.named_parameters()})
    return inp, res


def run_ladder_lm(reference_root, seed):
    """The reference's LadderLM (level 1, spectral-norm W_h as it defaults to) on seeded
    token ids: loss and every parameter gradient.  Importing it pulls in the whole
    `elman.models` package (slow, tens of seconds)."""
    sys.path.insert(0, reference_root)
    from elman.models.ladder_lm import LadderLM  # noqa: E402
    torch.manual_seed(seed)
    model = LadderLM(vocab_size=256, dim=32, depth=2, level=1, expansion=1.0)
    g = torch.Generator().manual_seed(seed + 1)
    tokens = torch.randint(0, 256, (3, 13), generator=g)
    us = {}
    for i, layer in enumerate(model.layers):  # pin the power-iteration start vectors
        u = torch.randn(32, generator=g)
        layer.cell._spectral_u = u / u.norm()
        us[f"spectral_u_{i}"] = layer.cell._spectral_u.clone()
    inp = {"tokens": tokens, **us}
    inp.update({"p_" + k: v.detach().clone() for k, v in model.state_dict().items()})
    loss = model(tokens, return_loss=True)
    loss.backward()
    res = {"loss": loss.detach().reshape(1)}
    res.update({"g_" + k: p.grad for k, p in model.named_parameters()})
    return inp, res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference",
                    default=os.environ.get("ELMAN_REFERENCE_DIR", os.path.join(os.sep, "root", "reference")))
    ap.add_argument("--only-lm", action="store_true")
    ap.add_argument("--only-siblings", action="store_true")
    args = ap.parse_args()
    if args.only_siblings:
        for name, cls, seed, kw in (("e32_no_presilu", "E32NoPresilu", 61, {}),
                                    ("e33_self_gate", "E33SelfGate", 62, {"r_h_mode": "spectral_norm"}),
                                    ("e57_learned_radius", "E57LearnedRadius", 63, {"expansion": 1.0})):
            mod = load_ref(args.reference, name)
            inp, res = run_sibling_layer(mod, cls, 2, 8, 64, seed, **kw)
            save(name.split("_")[0] + "_layer", True, inp, res, [2, 8, 64, seed])
        mod = load_ref(args.reference, "lowrank_elman")       # E4: rank 24 of 64
        inp, res = run_sibling_layer(mod, "LowRankElman", 2, 8, 64, 64, rank=24)
        save("e4_layer", True, inp, res, [2, 8, 64, 64])
        mod = load_ref(args.reference, "e1_multihead")        # E1H: 4 heads of 16
        inp, res = run_e1h_layer(mod, 2, 8, 64, 65, n_heads=4, n_state=16)
        save("e1h_layer", True, inp, res, [2, 8, 64, 65])
        return
    if args.only_lm:
        inp, res = run_ladder_lm(args.reference, seed=51)
        save("ladder_lm", True, inp, res, [3, 12, 32, 51])
        return
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    torch.manual_seed(0)

    m1 = load_ref(args.reference, "mamba_gated_elman")
    m0 = load_ref(args.reference, "stock_elman")
    m5 = load_ref(args.reference, "pure_lowrank_elman")
    assert not m1.MAMBA_CUDA_AVAILABLE and not m0.HASTE_AVAILABLE

    inp, res = run_e1(m1, 6, 3, 32, seed=11)
    save("e1_small", True, inp, res, [6, 3, 32, 11])
    inp, res = run_e1(m1, 9, 2, 48, seed=12, h0_random=True)
    save("e1_h0", True, inp, res, [9, 2, 48, 12])
    inp, res = run_e1(m1, 7, 2, 32, seed=13, spectral=True)
    save("e1_spectral", True, inp, res, [7, 2, 32, 13])
    # configs[0] of the benchmark: fp32, B=4, T=128, d=256, seed 1234
    inp, res = run_e1(m1, 128, 4, 256, seed=1234)
    res.pop("h")  # large: [129,4,256]; output and gradients pin it
    cell_in = make_e1_inputs(128, 4, 256, seed=1234)
    save("e1_c0", False, cell_in, res, [128, 4, 256, 1234])

    inp, res = run_e0(m0, 6, 3, 32, seed=21)
    save("e0_small", True, inp, res, [6, 3, 32, 21])
    inp, res = run_e0(m0, 24, 4, 128, seed=22)
    save("e0_mid", True, inp, res, [24, 4, 128, 22])

    inp, res = run_e5(m5, 6, 3, 32, 8, seed=31)
    save("e5_small", True, inp, res, [6, 3, 32, 8, 31])
    inp, res = run_e5(m5, 24, 4, 128, 24, seed=32)
    save("e5_mid", True, inp, res, [24, 4, 128, 24, 32])

    inp, res = run_e1_layer(m1, 2, 8, 64, seed=41)
    save("e1_layer", True, inp, res, [2, 8, 64, 41])

    inp, res = run_ladder_lm(args.reference, seed=51)
    save("ladder_lm", True, inp, res, [3, 12, 32, 51])

    for name, cls, seed, kw in (("e32_no_presilu", "E32NoPresilu", 61, {}),
                                ("e33_self_gate", "E33SelfGate", 62, {"r_h_mode": "spectral_norm"}),
                                ("e57_learned_radius", "E57LearnedRadius", 63, {"expansion": 1.0})):
        mod = load_ref(args.reference, name)
        inp, res = run_sibling_layer(mod, cls, 2, 8, 64, seed, **kw)
        save(name.split("_")[0] + "_layer", True, inp, res, [2, 8, 64, seed])
    mod = load_ref(args.reference, "lowrank_elman")
    inp, res = run_sibling_layer(mod, "LowRankElman", 2, 8, 64, 64, rank=24)
    save("e4_layer", True, inp, res, [2, 8, 64, 64])
    mod = load_ref(args.reference, "e1_multihead")
    inp, res = run_e1h_layer(mod, 2, 8, 64, 65, n_heads=4, n_state=16)
    save("e1h_layer", True, inp, res, [2, 8, 64, 65])


if __name__ == "__main__":
    main()
