"""The optimizer tail on flat buffers (FlatGradients + FlatAdamW, elman_adamw_step) against
torch.nn.utils.clip_grad_norm_ + torch.optim.AdamW, the step of the reference's training loop
(train_ladder.py:360-365, :542-545), and the whole captured step built on them."""
import pytest
import torch

from elman_b200 import _lib
from elman_b200.train_step import FlatAdamW, FlatGradients, GraphedTrainStep, make_gradient_reducer
from oracle import elman_oracle as orc

pytestmark = pytest.mark.gpu


def _nets(dtype):
    torch.manual_seed(3)
    a = torch.nn.Sequential(torch.nn.Linear(40, 72), torch.nn.Tanh(), torch.nn.Linear(72, 9)).cuda().to(dtype)
    b = torch.nn.Sequential(torch.nn.Linear(40, 72), torch.nn.Tanh(), torch.nn.Linear(72, 9)).cuda().to(dtype)
    b.load_state_dict(a.state_dict())
    return a, b


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_flat_adamw_with_folded_clipping_follows_torch_adamw(dtype, tol):
    a, b = _nets(dtype)
    grads = FlatGradients([list(a[2].parameters()), list(a[0].parameters())])
    opt_a = FlatAdamW(grads, lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opt_b = torch.optim.AdamW(b.parameters(), lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    g = torch.Generator().manual_seed(1)
    for it in range(6):
        x = (3 * torch.randn(16, 40, generator=g)).cuda().to(dtype)
        opt_a.zero_grad()
        a(x).float().pow(2).sum().backward()
        coef, norm_a = grads.clip_coef(0.5)
        opt_a.step(grad_scale=coef)
        opt_b.zero_grad(set_to_none=True)
        b(x).float().pow(2).sum().backward()
        norm_b = torch.nn.utils.clip_grad_norm_(b.parameters(), 0.5)
        opt_b.step()
        assert abs(float(norm_a) - float(norm_b)) < 2e-2 * float(norm_b)
        assert grads.check_views()
    assert float(opt_a.step_count) == 6.0
    for pa, pb in zip(a.parameters(), b.parameters()):
        # the update's size, not the weight's, is what rounding perturbs: compare the moves
        assert orc.rel_err(pa.float().cpu(), pb.float().cpu()) < tol


def test_graphed_step_on_flat_buffers_follows_the_eager_framework_step():
    """GraphedTrainStep with FlatGradients + FlatAdamW (zeroing, clipping and the update on flat
    buffers, fused layer ops, pipeline) against the eager step with torch's optimizer."""
    from elman_b200.ladder_lm import LadderLM, zipf_tokens
    batches = [zipf_tokens(8, 129, seed=300 + k).cuda() for k in range(5)]

    def make(**kw):
        torch.manual_seed(29)
        return LadderLM(vocab_size=256, dim=256, depth=3, level=1, r_h_mode="spectral_norm",
                        **kw).cuda().bfloat16()

    model = make(pipeline_chunks=0, fused_ops=False)
    for layer in model.layers:
        layer.fused = False
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    eager = []
    for tok in [batches[0]] * 3 + batches:
        opt.zero_grad(set_to_none=True)
        loss = model(tok, return_loss=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        eager.append(loss.item())
    model = make(pipeline_chunks=4)
    red = make_gradient_reducer(model)
    fopt = FlatAdamW(red, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    step = GraphedTrainStep(model, fopt, batches[0], max_grad_norm=1.0, warmup_steps=3, reducer=red)
    graphed = [step(tok).item() for tok in batches]
    assert _lib.device_status()[0] == 0 and red.check_views()
    assert float(fopt.step_count) == 3 + len(batches)     # warm-up steps + replays (capture runs nothing)
    for a, b in zip(eager[3:], graphed):
        assert abs(a - b) < 5e-2 * abs(a), (eager, graphed)
