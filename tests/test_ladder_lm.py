"""The LM wrapper (the caller of the hot path) on the CPU, against the fixture the
reference's LadderLM produced, and its data-parallel training step on two gloo ranks.
The CUDA library is replaced by the oracle-backed stand-in of test_host_logic (test only)."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from elman_b200 import ladder_lm
from elman_b200 import mamba_gated_elman as e1mod
from oracle import elman_oracle as orc
from tests.test_host_logic import OracleBackend

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


class _FakeCudaLayer(e1mod.MambaGatedElman):
    """E1 layer whose cell input answers is_cuda=True, so the CPU stand-in can run."""

    def forward(self, x, h0=None, **kw):
        from tests.test_host_logic import as_fake_cuda
        return super().forward(as_fake_cuda(x), h0, **kw)


def _build(fix, monkeypatch_fn):
    from elman_b200 import fused_ops
    monkeypatch_fn(e1mod, "hasty_pytorch_lib", OracleBackend)
    monkeypatch_fn(fused_ops, "hasty_pytorch_lib", OracleBackend)
    monkeypatch_fn(ladder_lm, "_LEVELS", {**ladder_lm._LEVELS, 1: _FakeCudaLayer})
    model = ladder_lm.LadderLM(vocab_size=256, dim=32, depth=2, level=1, expansion=1.0)
    sd = {k[5:]: torch.from_numpy(fix[k]) for k in fix.files if k.startswith("in_p_")}
    assert set(sd) == set(model.state_dict()), "parameter names differ from the reference's"
    model.load_state_dict(sd)
    for i, layer in enumerate(model.layers):
        layer.cell._spectral_u = torch.from_numpy(fix[f"in_spectral_u_{i}"]).clone()
    return model


def test_lm_loss_and_gradients_match_reference_fixture(monkeypatch):
    fix = np.load(os.path.join(GOLDEN, "ladder_lm.npz"))
    model = _build(fix, monkeypatch.setattr)
    tokens = torch.from_numpy(fix["in_tokens"])
    loss = model(tokens, return_loss=True)
    loss.backward()
    assert abs(float(loss) - float(fix["out_loss"][0])) < 1e-5
    for k, p in model.named_parameters():
        want = torch.from_numpy(fix["out_g_" + k])
        assert orc.rel_err(p.grad, want) < 1e-4, k


def test_lm_interfaces():
    model = ladder_lm.LadderLM(vocab_size=256, dim=1280, depth=6, level=1, expansion=1.0)
    assert model.get_num_params() == 49_496_320  # the "~50M" model of the benchmark
    with pytest.raises(ValueError):
        ladder_lm.get_ladder_level(7)
    tok = ladder_lm.zipf_tokens(4, 33, seed=1)
    assert tok.shape == (4, 33) and int(tok.min()) >= 0 and int(tok.max()) < 256
    assert torch.equal(tok, ladder_lm.zipf_tokens(4, 33, seed=1))


def _ddp_worker(rank, world, port, out):
    torch.set_num_threads(1)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fix = np.load(os.path.join(GOLDEN, "ladder_lm.npz"))

        def setattr_(obj, name, val):
            setattr(obj, name, val)
        model = _build(fix, setattr_)
        ddp = torch.nn.parallel.DistributedDataParallel(model)
        tokens = ladder_lm.zipf_tokens(2, 9, seed=100 + rank)   # each rank its own shard
        loss = ddp(tokens, return_loss=True)
        loss.backward()
        if rank == 0:
            torch.save({k: p.grad.clone() for k, p in model.named_parameters()}, out)
    finally:
        dist.destroy_process_group()


def test_data_parallel_step_on_two_gloo_ranks_averages_shard_gradients(tmp_path, monkeypatch):
    """world_size 2 on CPU: DDP's gradient equals the mean of the two shards' gradients."""
    out = str(tmp_path / "grads.pt")
    port = 29500 + (os.getpid() % 400)
    mp.start_processes(_ddp_worker, args=(2, port, out), nprocs=2, join=True, start_method="spawn")
    got = torch.load(out)
    fix = np.load(os.path.join(GOLDEN, "ladder_lm.npz"))
    ref = {}
    for r in range(2):
        model = _build(fix, monkeypatch.setattr)
        model(ladder_lm.zipf_tokens(2, 9, seed=100 + r), return_loss=True).backward()
        for k, p in model.named_parameters():
            ref[k] = ref.get(k, 0) + p.grad / 2
    for k in ref:
        assert orc.rel_err(got[k], ref[k]) < 1e-5, k


def _allreduce_worker(rank, world, port, out):
    import torch.distributed as dist
    from elman_b200.train_step import allreduce_gradients
    torch.set_num_threads(1)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                            world_size=world)
    a = torch.nn.Parameter(torch.zeros(3, 2))
    b = torch.nn.Parameter(torch.zeros(5))
    c = torch.nn.Parameter(torch.zeros(2))          # never gets a gradient
    a.grad = torch.full((3, 2), float(rank + 1))
    b.grad = torch.arange(5.0) * (rank + 1)
    allreduce_gradients([a, b, c])
    out.put((rank, a.grad.clone(), b.grad.clone(), c.grad is None))
    dist.barrier()
    dist.destroy_process_group()


def test_allreduce_gradients_averages_over_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + os.getpid() % 200
    procs = [ctx.Process(target=_allreduce_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ga, gb, none_c in got:
        assert torch.allclose(ga, torch.full((3, 2), 1.5))
        assert torch.allclose(gb, torch.arange(5.0) * 1.5)
        assert none_c


def _flat_worker(rank, world, port, out):
    import torch.distributed as dist
    from elman_b200.train_step import FlatGradients
    torch.set_num_threads(1)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                            world_size=world)
    torch.manual_seed(5)                       # same weights on both ranks
    net = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.Tanh(), torch.nn.Linear(8, 3))
    unused = torch.nn.Parameter(torch.zeros(4))        # gets no gradient: its bucket is still reduced
    fg = FlatGradients([list(net[2].parameters()), list(net[0].parameters()) + [unused]])
    x = torch.randn(5, 6, generator=torch.Generator().manual_seed(100 + rank))
    results = []
    for _ in range(2):                         # two steps: the buffer is reused
        fg.zero()
        net(x).pow(2).sum().backward()
        launched_by_hooks = fg._launched
        fg.finish()
        results.append(([p.grad.clone() for p in net.parameters()], launched_by_hooks,
                        fg.check_views(), float(unused.grad.abs().sum())))
    out.put((rank, results))
    dist.barrier()
    dist.destroy_process_group()


def test_flat_gradient_buckets_are_averaged_over_two_gloo_ranks_as_they_complete():
    """FlatGradients on two CPU ranks: each bucket is all-reduced from the hook of its last
    gradient (the layer that finishes backward first goes first), gradients stay views into
    the flat buffer, and the result is the mean of the two ranks' gradients."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29850 + os.getpid() % 100
    procs = [ctx.Process(target=_flat_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    torch.manual_seed(5)
    net = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.Tanh(), torch.nn.Linear(8, 3))
    want = None
    for r in range(2):
        net.zero_grad()
        x = torch.randn(5, 6, generator=torch.Generator().manual_seed(100 + r))
        net(x).pow(2).sum().backward()
        g = [p.grad.clone() / 2 for p in net.parameters()]
        want = g if want is None else [a + b for a, b in zip(want, g)]
    for rank in (0, 1):
        for grads, by_hooks, views_ok, unused_sum in got[rank]:
            assert by_hooks == 1       # the complete bucket went from its hook, during backward
            assert views_ok and unused_sum == 0.0
            for a, b in zip(grads, want):
                assert torch.allclose(a, b, atol=1e-6)


def test_lm_gradients_with_the_gradient_sink_match_reference_fixture(monkeypatch):
    """Weight gradients accumulated in place by the nodes that produce them (GradSink, through
    FlatGradients(direct=...)) instead of returned to autograd: same loss, same gradients as
    the reference fixture, for the whole sequence and for chained time chunks."""
    from elman_b200 import fused_ops
    from elman_b200.train_step import FlatGradients, direct_weights, ladder_buckets
    fix = np.load(os.path.join(GOLDEN, "ladder_lm.npz"))
    model = _build(fix, monkeypatch.setattr)
    direct = direct_weights(model)
    assert len(direct) == 3 * model.depth          # in_proj, out_proj, W_x (W_h is spectral-normed)
    fg = FlatGradients(ladder_buckets(model), direct=direct)
    try:
        assert fused_ops.get_grad_sink() is fg.sink
        tokens = torch.from_numpy(fix["in_tokens"])
        for _ in range(2):                          # twice: zero() must reset the sums
            for i, layer in enumerate(model.layers):    # the power iteration advances its vector
                layer.cell._spectral_u = torch.from_numpy(fix[f"in_spectral_u_{i}"]).clone()
            fg.zero()
            loss = model(tokens, return_loss=True)
            loss.backward()
            fg.finish()
            assert abs(float(loss) - float(fix["out_loss"][0])) < 1e-5
            assert fg.check_views()
            for k, p in model.named_parameters():
                want = torch.from_numpy(fix["out_g_" + k])
                assert orc.rel_err(p.grad, want) < 1e-4, k
    finally:
        fg.close()
    assert fused_ops.get_grad_sink() is None
