"""The projection GEMM (TMA + tcgen05 for bf16, CUDA cores for fp32) vs a torch fp32 matmul."""
import pytest
import torch

from elman_b200 import _lib
from elman_b200 import hasty_pytorch_lib as H
from oracle.elman_oracle import rel_err
from tests._gpu_cases import option

pytestmark = pytest.mark.gpu


def ref_proj(A, W, bias, C0):
    r = A.float().cpu() @ W.float().cpu().T
    if bias is not None:
        r = r + bias.float().cpu()
    if C0 is not None:
        r = r + C0.float().cpu()
    return r


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 128, 128), (100, 72, 40), (1, 8, 8),
                                   (384, 1280, 1280), (130, 250, 72), (2048, 256, 1024)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_bf16_tensor_core_gemm(M, N, K, with_bias):
    g = torch.Generator().manual_seed(M + N + K)
    A = torch.randn(M, K, generator=g).bfloat16().cuda()
    W = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16().cuda()
    bias = torch.randn(N, generator=g).bfloat16().cuda() if with_bias else None
    before = _lib.tc_launch_count()
    out = H.projection(A, W, bias)
    torch.cuda.synchronize()
    assert _lib.tc_launch_count() == before + 1, "tcgen05 GEMM was not used"
    assert _lib.device_status()[0] == 0
    # bf16 output: one rounding of an fp32-accumulated result
    assert rel_err(out, ref_proj(A, W, bias, None)) < 4e-3


def test_bf16_accumulate_into_existing_output():
    g = torch.Generator().manual_seed(3)
    A = torch.randn(256, 128, generator=g).bfloat16().cuda()
    W = (torch.randn(192, 128, generator=g) / 11).bfloat16().cuda()
    C0 = torch.randn(256, 192, generator=g).bfloat16().cuda()
    out = C0.clone()
    H.projection(A, W, None, out=out, accumulate=True)
    torch.cuda.synchronize()
    assert rel_err(out, ref_proj(A, W, None, C0)) < 4e-3


@pytest.mark.parametrize("M,N,K", [(64, 64, 16), (100, 72, 41), (5, 3, 7)])
def test_fp32_cuda_core_gemm(M, N, K):
    g = torch.Generator().manual_seed(M * N)
    A = torch.randn(M, K, generator=g).cuda()
    W = torch.randn(N, K, generator=g).cuda()
    bias = torch.randn(N, generator=g).cuda()
    out = H.projection(A, W, bias)
    torch.cuda.synchronize()
    assert rel_err(out, ref_proj(A, W, bias, None)) < 1e-5


def test_bf16_odd_k_falls_back_to_cuda_cores_and_matches():
    g = torch.Generator().manual_seed(9)
    A = torch.randn(64, 270, generator=g).bfloat16().cuda()
    W = (torch.randn(96, 270, generator=g) / 16).bfloat16().cuda()
    before = _lib.tc_launch_count()
    out = H.projection(A, W)
    torch.cuda.synchronize()
    assert _lib.tc_launch_count() == before
    assert rel_err(out, ref_proj(A, W, None, None)) < 4e-3


def test_tensor_core_and_cuda_core_paths_agree():
    g = torch.Generator().manual_seed(10)
    A = torch.randn(512, 256, generator=g).bfloat16().cuda()
    W = (torch.randn(384, 256, generator=g) / 16).bfloat16().cuda()
    a = H.projection(A, W)
    with option("force_generic", 1):
        b = H.projection(A, W)
    torch.cuda.synchronize()
    assert rel_err(a, b.float().cpu()) < 4e-3


KERNELS = {"tile": (1, 1), "persistent": (1, 2), "pair": (2, 0)}


@pytest.fixture()
def gemm_kernel_choice():
    """Force one of the three tcgen05 GEMM kernels: 128x128 tiles, persistent 128x256 tiles, and the
    CTA-pair kernel (persistent, 256x256 tiles over two CTAs)."""
    old = _lib.get_option("gemm_pair"), _lib.get_option("gemm_persistent")

    def choose(name):
        pair, persistent = KERNELS[name]
        _lib.set_option("gemm_pair", pair)
        _lib.set_option("gemm_persistent", persistent)
    yield choose
    _lib.set_option("gemm_pair", old[0])
    _lib.set_option("gemm_persistent", old[1])


def test_all_gemm_kernels_agree_bit_for_bit(gemm_kernel_choice):
    """Every output element is accumulated over K in the same order by all three kernels."""
    g = torch.Generator().manual_seed(99)
    A = torch.randn(1000, 520, generator=g).bfloat16().cuda()
    W = (torch.randn(1304, 520, generator=g) / 22).bfloat16().cuda()
    At = torch.randn(520, 1000, generator=g).bfloat16().cuda()
    Bn = (torch.randn(520, 1304, generator=g) / 22).bfloat16().cuda()
    bias = torch.randn(1304, generator=g).bfloat16().cuda()
    outs = []
    for choice in KERNELS:
        gemm_kernel_choice(choice)
        outs.append((H.gemm(H.GEMM_NT, A, W, bias), H.gemm(H.GEMM_NN, A, Bn),
                     H.gemm(H.GEMM_TN, At, Bn)))
    torch.cuda.synchronize()
    assert _lib.device_status()[0] == 0
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert torch.equal(a, b)


@pytest.mark.parametrize("kernel", list(KERNELS))
@pytest.mark.parametrize("M,N,K", [(512, 512, 128), (304, 520, 136), (1280, 1280, 2048),
                                   (2048, 1280, 1280), (384, 392, 64), (8, 16, 8),
                                   (4096, 2560, 320), (136, 264, 72)])
def test_every_gemm_form(M, N, K, kernel, request):
    """NT (+bias, +accumulate), NN and TN through elman_gemm: K-major and MN-major operands of
    all three tcgen05 kernels (forced here for every shape they can take), ragged tile edges,
    against fp32 matmuls."""
    request.getfixturevalue("gemm_kernel_choice")(kernel)
    g = torch.Generator().manual_seed(7 * M + 3 * N + K)
    s = K ** -0.5
    A = torch.randn(M, K, generator=g).bfloat16().cuda()
    Bnt = (torch.randn(N, K, generator=g) * s).bfloat16().cuda()
    Bnn = (torch.randn(K, N, generator=g) * s).bfloat16().cuda()
    At = torch.randn(K, M, generator=g).bfloat16().cuda()
    bias = torch.randn(N, generator=g).bfloat16().cuda()
    C0 = torch.randn(M, N, generator=g).bfloat16().cuda()
    f = lambda t: t.float().cpu()
    before = _lib.tc_launch_count()
    nt = H.gemm(H.GEMM_NT, A, Bnt, bias)
    acc = H.gemm(H.GEMM_NT, A, Bnt, None, out=C0.clone(), accumulate=True)
    nn = H.gemm(H.GEMM_NN, A, Bnn)
    tn = H.gemm(H.GEMM_TN, At, Bnn)
    torch.cuda.synchronize()
    assert _lib.tc_launch_count() - before == 4, "all four must take the tcgen05 kernel"
    assert _lib.device_status()[0] == 0
    assert rel_err(f(nt), f(A) @ f(Bnt).T + f(bias)) < 1e-2
    assert rel_err(f(acc), f(A) @ f(Bnt).T + f(C0)) < 1e-2
    assert rel_err(f(nn), f(A) @ f(Bnn)) < 1e-2
    assert rel_err(f(tn), f(At).T @ f(Bnn)) < 1e-2
