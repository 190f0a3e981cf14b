"""The layer's time-parallel ops (residual add + RMSNorm, in_proj with split + silu, their
backward passes) through the C ABI against the same math in plain PyTorch fp32 — the ops the
reference runs as separate framework passes (elman/models/ladder_lm.py:986-1003,
elman/models/mamba_gated_elman.py:283-297)."""
import pytest
import torch
import torch.nn.functional as F

from elman_b200 import _lib, fused_ops
from elman_b200 import hasty_pytorch_lib as H
from oracle import elman_oracle as orc
from tests._gpu_cases import TOL, option

pytestmark = pytest.mark.gpu


def rel(a, b):
    return orc.rel_err(a.float().cpu(), b.float().cpu())


def _ref_add_norm(x, res_in, w, eps):
    """fp32 reference with the rounding point of the op-by-op form (norm input in x's dtype)."""
    res = x.float() if res_in is None else x.float() + res_in
    v = res.to(x.dtype).float()
    y = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y, res


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,D,with_res", [((3, 5), 33, True), ((64, 32), 1280, True),
                                             ((7,), 2560, False), ((4, 2), 128, False)])
def test_add_rmsnorm_forward_and_backward_match_pytorch(dtype, rows, D, with_res):
    g = torch.Generator().manual_seed(D + len(rows))
    x = torch.randn(*rows, D, generator=g).to(dtype).cuda()
    res_in = (2 * torch.randn(*rows, D, generator=g)).cuda() if with_res else None
    w = (1 + 0.2 * torch.randn(D, generator=g)).to(dtype).cuda()
    dy = torch.randn(*rows, D, generator=g).to(dtype).cuda()
    dres = torch.randn(*rows, D, generator=g).cuda()
    eps = fused_ops.rmsnorm_eps(torch.nn.RMSNorm(D), dtype)
    # reference: autograd through the fp32 math (straight-through the rounding of the input)
    xr = x.detach().float().clone().requires_grad_(True)
    rr = res_in.clone().requires_grad_(True) if with_res else None
    wr = w.detach().float().clone().requires_grad_(True)
    res = xr if rr is None else xr + rr
    v = res + (res.to(dtype).float() - res).detach()
    y_ref = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * wr
    (y_ref * dy.float()).sum().backward(retain_graph=True)
    (res * dres).sum().backward()
    # library
    xq = x.detach().clone().requires_grad_(True)
    rq = res_in.clone().requires_grad_(True) if with_res else None
    wq = w.detach().clone().requires_grad_(True)
    y, res_out = fused_ops.AddRMSNormFunction.apply(xq, rq, wq, eps)
    ((y.float() * dy.float()).sum() + (res_out * dres).sum()).backward()
    torch.cuda.synchronize()
    tol = TOL[dtype]
    assert rel(y, y_ref) < tol and rel(res_out, res) < 1e-6
    assert rel(xq.grad, xr.grad) < tol
    assert rel(wq.grad, wr.grad) < tol
    if with_res:
        assert rq.grad.dtype == torch.float32 and rel(rq.grad, rr.grad) < (1e-5 if dtype == torch.float32 else tol)
    # against nn.RMSNorm itself (the module the reference's fallback path calls)
    ref_mod = torch.nn.RMSNorm(D).to("cuda", dtype)
    with torch.no_grad():
        ref_mod.weight.copy_(w)
    base = x.float() if res_in is None else x.float() + res_in
    assert rel(y, ref_mod(base.to(dtype))) < tol
    # ... also where the mean square is far below the 16-bit machine epsilon (embedding-sized
    # activations): the default epsilon must be the one nn.RMSNorm really uses
    small = (0.02 * x.float()).to(dtype)
    ys, _ = fused_ops.AddRMSNormFunction.apply(small, None, w, fused_ops.rmsnorm_eps(ref_mod, dtype))
    assert rel(ys, ref_mod(small)) < tol


@pytest.mark.parametrize("M,d,K,generic", [(2048, 1280, 1280, 0), (192, 64, 64, 0), (50, 96, 40, 0),
                                          (2048, 1280, 1280, 1), (37, 24, 16, 0)])
def test_in_proj_split_silu_matches_pytorch(M, d, K, generic):
    """bf16: split + silu in the tcgen05 GEMM's epilogue (d % 32 == 0) and the two-pass form."""
    g = torch.Generator().manual_seed(M + d)
    u = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    W = (torch.randn(2 * d, K, generator=g) / K ** 0.5).to(torch.bfloat16).cuda()
    before = _lib.tc_launch_count()
    with option("force_generic", generic):
        x_raw, x_act, z = H.in_proj_split_silu(u, W)
    torch.cuda.synchronize()
    if not generic and d % 32 == 0 and K % 8 == 0:
        assert _lib.tc_launch_count() == before + 1, "expected ONE tensor-core launch, no extra pass"
    xz = u.float() @ W.float().T
    assert rel(x_raw, xz[:, :d]) < TOL[torch.bfloat16]
    assert rel(z, xz[:, d:]) < TOL[torch.bfloat16]
    assert rel(x_act, F.silu(xz[:, :d])) < TOL[torch.bfloat16]
    # the activation is the silu of the value as stored
    assert rel(x_act, F.silu(x_raw.float())) < 5e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("lead,d,K", [((6, 4), 64, 64), ((5, 3), 24, 20), ((64, 32), 1280, 1280)])
def test_in_proj_function_gradients_match_pytorch(dtype, lead, d, K):
    g = torch.Generator().manual_seed(d + K)
    u = torch.randn(*lead, K, generator=g).to(dtype).cuda()
    W = (torch.randn(2 * d, K, generator=g) / K ** 0.5).to(dtype).cuda()
    da = torch.randn(*lead, d, generator=g).to(dtype).cuda()
    dzz = torch.randn(*lead, d, generator=g).to(dtype).cuda()
    ur = u.detach().float().clone().requires_grad_(True)
    Wr = W.detach().float().clone().requires_grad_(True)
    xz = ur @ Wr.T
    (F.silu(xz[..., :d]) * da.float() + xz[..., d:] * dzz.float()).sum().backward()
    uq, Wq = u.detach().clone().requires_grad_(True), W.detach().clone().requires_grad_(True)
    xa, z = fused_ops.InProjSplitSiluFunction.apply(uq, Wq)
    (xa.float() * da.float() + z.float() * dzz.float()).sum().backward()
    torch.cuda.synchronize()
    tol = TOL[dtype]
    assert rel(xa, F.silu(xz[..., :d])) < tol and rel(z, xz[..., d:]) < tol
    assert rel(uq.grad, ur.grad) < tol and rel(Wq.grad, Wr.grad) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,d", [(2048, 1280), (33, 20), (16, 8)])
def test_silu_backward_concat_matches_pytorch(dtype, M, d):
    g = torch.Generator().manual_seed(M)
    da, xr, dz = (torch.randn(M, d, generator=g).to(dtype).cuda() for _ in range(3))
    got = H.silu_backward_concat(da, xr, dz)
    torch.cuda.synchronize()
    s = torch.sigmoid(xr.float())
    want = torch.cat([da.float() * s * (1 + xr.float() * (1 - s)), dz.float()], dim=1)
    assert rel(got, want) < (1e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("d", [7, 32, 50, 72, 256, 1280])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1.5e-2)])
def test_spectral_norm_kernel_matches_the_framework_ops(d, dtype, tol):
    """elman_spectral_norm_forward/backward (one cluster kernel per direction) against the same
    steps as framework ops in fp32: the rescaled matrix, the advanced vector u, and the
    gradient of W through sigma = |u^T W v| with u, v constant."""
    from elman_b200 import _spectral
    from oracle.elman_oracle import rel_err
    g = torch.Generator().manual_seed(d)
    W = (torch.randn(d, d, generator=g) * d ** -0.5).to(dtype)
    u0 = torch.randn(d, generator=g)
    u0 = (u0 / u0.norm()).to(dtype)
    G = torch.randn(d, d, generator=g).to(dtype)

    class Holder:
        pass
    ref, got = Holder(), Holder()
    ref._spectral_u = u0.float().clone()
    Wr = W.float().clone().requires_grad_(True)
    old = _spectral.FUSED
    _spectral.FUSED = False
    try:
        We_ref = _spectral.spectrally_normalised(ref, Wr)
    finally:
        _spectral.FUSED = old
    (We_ref * G.float()).sum().backward()

    got._spectral_u = u0.clone().cuda()
    Wg = W.clone().cuda().requires_grad_(True)
    before = _lib.launch_count()
    We = _spectral.spectrally_normalised(got, Wg)
    (We.float() * G.cuda().float()).sum().backward()
    torch.cuda.synchronize()
    assert _lib.launch_count() - before == 2, "one kernel forward, one backward"
    assert _lib.device_status()[0] == 0
    assert rel_err(We.float().cpu(), We_ref.detach()) < tol
    assert rel_err(got._spectral_u.float().cpu(), ref._spectral_u) < tol
    assert rel_err(Wg.grad.float().cpu(), Wr.grad) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_embedding_rows_gradient_matches_the_framework_embedding(dtype, tol):
    """The one-hot GEMM backward of `embedding_rows` gives nn.functional.embedding's weight
    gradient (tokens repeat many times: vocabulary 256, 51 x 32 tokens)."""
    torch.manual_seed(5)
    V, D, Tc, B = 256, 320, 51, 32
    tokens = torch.randint(0, V, (Tc, B), device="cuda")
    tokens[0, :8] = 7                       # a row hit many times, and rows never hit
    w_ref = (torch.randn(V, D, device="cuda") * 0.1).to(dtype).requires_grad_(True)
    w_lib = w_ref.detach().clone().requires_grad_(True)
    dy = torch.randn(Tc, B, D, device="cuda").to(dtype)
    y_ref = F.embedding(tokens, w_ref)
    y_lib = fused_ops.embedding_rows(tokens, w_lib)
    assert y_lib.grad_fn is not None and "EmbeddingRows" in type(y_lib.grad_fn).__name__
    assert torch.equal(y_ref, y_lib)
    y_ref.backward(dy)
    y_lib.backward(dy)
    ref = w_ref.grad.float()
    err = (w_lib.grad.float() - ref).norm() / ref.norm()
    assert err < tol, err
    never = torch.ones(V, dtype=torch.bool, device="cuda")
    never[tokens.unique()] = False
    assert torch.count_nonzero(w_lib.grad[never]) == 0
