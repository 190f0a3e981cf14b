"""Time-chunked execution on the GPU: the chunk-carry backward entry point of the C
ABI, and LadderLM's (layer, time chunk) pipeline over several CUDA streams."""
import pytest
import torch

from _gpu_cases import TOL, assert_close, errors, oracle_e1, option, round_inputs, run_e1
from elman_b200 import hasty_pytorch_lib as H
from oracle import elman_oracle as orc

pytestmark = pytest.mark.gpu


def run_e1_chunked(inp, dtype, edges):
    """Forward per chunk with the state carried, backward per chunk in reverse with the
    pre-activation gradient carried; weight gradients summed over chunks in fp32."""
    dev, ref = round_inputs(inp, dtype)
    state = dev["h0"]
    fwd = []
    for t0, t1 in zip(edges[:-1], edges[1:]):
        x, z = dev["x"][t0:t1].contiguous(), dev["z"][t0:t1].contiguous()
        h, out, v = H.mamba_gated_elman_forward(True, x, z, state, dev["W_x"], dev["W_h"], dev["b"])
        fwd.append((x, z, h, out, v))
        state = h[-1].contiguous()
    got = {"output": torch.cat([f[3] for f in fwd]),
           "h": torch.cat([fwd[0][2][:1]] + [f[2][1:] for f in fwd])}
    carry = None
    dxs, dzs = [], []
    sums = None
    for (x, z, h, out, v), t0, t1 in reversed(list(zip(fwd, edges[:-1], edges[1:]))):
        dx, dz, dWx, dWh, db, carry = H.mamba_gated_elman_backward_carry(
            dev["W_x"], dev["W_h"], x, z, h, v, dev["d_output"][t0:t1].contiguous(), carry)
        dxs.insert(0, dx); dzs.insert(0, dz)
        parts = [dWx.float(), dWh.float(), db.float()]
        sums = parts if sums is None else [a + b for a, b in zip(sums, parts)]
    got.update(dx=torch.cat(dxs), dz=torch.cat(dzs), dW_x=sums[0], dW_h=sums[1], db=sums[2])
    torch.cuda.synchronize()
    return got, ref


@pytest.mark.parametrize("dtype,T,B,d,edges", [
    (torch.float32, 12, 3, 40, (0, 5, 6, 12)),
    (torch.float32, 9, 2, 64, (0, 9)),
    (torch.bfloat16, 24, 16, 128, (0, 8, 24)),      # tensor-core kernels
    (torch.bfloat16, 40, 32, 256, (0, 16, 17, 40)),
    (torch.bfloat16, 10, 3, 40, (0, 4, 10)),        # CUDA-core bf16 kernels
])
def test_chained_chunks_match_oracle_and_whole_sequence(dtype, T, B, d, edges):
    inp = orc.make_e1_inputs(T, B, d, seed=91)
    got, ref = run_e1_chunked(inp, dtype, edges)
    assert_close(errors(got, oracle_e1(ref)), TOL[dtype], "chunked vs oracle")
    whole, _ = run_e1(inp, dtype)
    # the per-step arithmetic is the same kernel code on the same values
    for k in ("output", "h", "dx", "dz"):
        assert torch.equal(got[k], whole[k]), k
    for k in ("dW_x", "dW_h", "db"):
        assert orc.rel_err(got[k].cpu(), whole[k].float().cpu()) < TOL[dtype], k


@pytest.mark.parametrize("T,B,d", [(12, 32, 256), (10, 16, 1280), (6, 64, 512)])
def test_compact_launch_flag_matches_oracle(T, B, d):
    """ELMAN_FLAG_COMPACT changes the launch plan (smaller K split, W in tensor memory
    where needed), not the result beyond the summation order."""
    inp = orc.make_e1_inputs(T, B, d, seed=17)
    dev, ref = round_inputs(inp, torch.bfloat16)
    h, out, v = H.mamba_gated_elman_forward(True, dev["x"], dev["z"], dev["h0"], dev["W_x"],
                                            dev["W_h"], dev["b"], H.FLAG_COMPACT)
    dx, dz, dWx, dWh, db, dv0 = H.mamba_gated_elman_backward_carry(
        dev["W_x"], dev["W_h"], dev["x"], dev["z"], h, v, dev["d_output"], None, H.FLAG_COMPACT)
    torch.cuda.synchronize()
    got = {"h": h, "output": out, "v": v, "dx": dx, "dz": dz, "dW_x": dWx, "dW_h": dWh, "db": db}
    assert_close(errors(got, oracle_e1(ref)), TOL[torch.bfloat16], "compact plan vs oracle")


def test_carry_entry_point_with_no_carry_equals_plain_backward():
    inp = orc.make_e1_inputs(20, 32, 256, seed=5)
    dev, _ = round_inputs(inp, torch.bfloat16)
    h, out, v = H.mamba_gated_elman_forward(True, dev["x"], dev["z"], dev["h0"], dev["W_x"],
                                            dev["W_h"], dev["b"])
    a = H.mamba_gated_elman_backward(dev["W_x"], dev["W_h"], dev["x"], dev["z"], h, v,
                                     dev["d_output"])
    b = H.mamba_gated_elman_backward_carry(dev["W_x"], dev["W_h"], dev["x"], dev["z"], h, v,
                                           dev["d_output"], None)
    for ta, tb in zip(a, b[:5]):
        assert torch.equal(ta, tb)
    assert b[5].shape == (32, 256) and torch.isfinite(b[5].float()).all()


def test_recurrence_blocks_query():
    fast = H.recurrence_blocks(torch.bfloat16, 128, 32, 1280)
    compact = H.recurrence_blocks(torch.bfloat16, 128, 32, 1280, H.FLAG_COMPACT)
    assert fast in (10, 20, 40, 80) and 0 < compact <= fast
    assert H.recurrence_blocks(torch.float32, 128, 32, 1280) == 0
    assert H.recurrence_blocks(torch.bfloat16, 16, 3, 40) == 0


def _lm_step(model, tokens):
    model.zero_grad(set_to_none=True)
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=False):
        loss = model(tokens, return_loss=True)
    loss.backward()
    torch.cuda.synchronize()
    return loss.detach().float().item(), {n: p.grad.detach().float().clone()
                                          for n, p in model.named_parameters()}


@pytest.mark.parametrize("chunks,streams", [(4, 0), (3, 2), (8, 3)])
def test_pipelined_ladder_lm_matches_sequential(chunks, streams):
    from elman_b200.ladder_lm import LadderLM, zipf_tokens
    torch.manual_seed(7)
    model = LadderLM(vocab_size=256, dim=256, depth=4, level=1, r_h_mode="none").cuda().bfloat16()
    tokens = zipf_tokens(8, 97, seed=3).cuda()
    loss_seq, g_seq = _lm_step(model, tokens)
    model.pipeline_chunks, model.pipeline_streams = chunks, streams
    for _ in range(3):  # repeated: a cross-stream ordering bug would not show every time
        loss_pipe, g_pipe = _lm_step(model, tokens)
        assert abs(loss_pipe - loss_seq) < 2e-2 * abs(loss_seq)
        for n in g_seq:
            assert orc.rel_err(g_pipe[n].cpu(), g_seq[n].cpu()) < TOL[torch.bfloat16], n


def test_pipelined_ladder_lm_trains_like_sequential():
    """Several optimizer steps with and without the pipeline from the same start."""
    from elman_b200.ladder_lm import LadderLM, zipf_tokens
    losses = {}
    for chunks in (0, 4):
        torch.manual_seed(11)
        model = LadderLM(vocab_size=256, dim=256, depth=3, level=1, r_h_mode="spectral_norm",
                         pipeline_chunks=chunks).cuda().bfloat16()
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
        out = []
        for step in range(6):
            tokens = zipf_tokens(8, 129, seed=100 + step).cuda()
            opt.zero_grad(set_to_none=True)
            loss = model(tokens, return_loss=True)
            loss.backward()
            opt.step()
            out.append(loss.item())
        losses[chunks] = out
    for a, b in zip(losses[0], losses[4]):
        assert abs(a - b) < 3e-2 * abs(a), losses
    assert losses[4][-1] < losses[4][0]


def test_graphed_train_step_matches_eager_steps():
    """The whole step captured in a CUDA graph (pipeline streams included) follows the same
    loss trajectory as eager steps from the same start on the same tokens."""
    from elman_b200.ladder_lm import LadderLM, zipf_tokens
    from elman_b200.train_step import GraphedTrainStep
    batches = [zipf_tokens(8, 129, seed=200 + k).cuda() for k in range(5)]

    def make():
        torch.manual_seed(23)
        model = LadderLM(vocab_size=256, dim=256, depth=3, level=1, r_h_mode="spectral_norm",
                         pipeline_chunks=4).cuda().bfloat16()
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, capturable=True)
        return model, opt

    model, opt = make()
    eager = []
    for tok in [batches[0]] * 3 + batches:       # the graphed arm warms up 3 times on batch 0
        opt.zero_grad(set_to_none=True)
        loss = model(tok, return_loss=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        eager.append(loss.item())
    model, opt = make()
    step = GraphedTrainStep(model, opt, batches[0], max_grad_norm=1.0, warmup_steps=3)
    assert step.library_launches_per_step > 0
    graphed = [step(tok).item() for tok in batches]
    for a, b in zip(eager[3:], graphed):
        assert abs(a - b) < 3e-2 * abs(a), (eager, graphed)


def test_full_size_pipelined_step_keeps_every_wait_satisfied():
    """configs[2] at full size (d1280 x 6, B32, T512, bf16), eager and pipelined over 8 chunks: six
    recurrence launches whose blocks wait on one another run beside the device-wide GEMMs of the
    other streams.  Nothing may time out (status word stays clear), the loss is finite, and the
    gradients agree with the layer-by-layer pass."""
    from elman_b200 import _lib
    from elman_b200.ladder_lm import LadderLM, zipf_tokens
    torch.manual_seed(5)
    model = LadderLM(vocab_size=256, dim=1280, depth=6, level=1, r_h_mode="none",
                     pipeline_chunks=0).cuda().bfloat16()
    tokens = zipf_tokens(32, 513, seed=9).cuda()
    _lib.device_status(clear=True)
    loss_seq, g_seq = _lm_step(model, tokens)
    model.pipeline_chunks = 8
    for _ in range(3):
        loss_pipe, g_pipe = _lm_step(model, tokens)
        assert _lib.device_status()[0] == 0, _lib.device_status()
        assert loss_pipe == loss_pipe and abs(loss_pipe - loss_seq) < 2e-2 * abs(loss_seq)
    for n in g_seq:
        assert orc.rel_err(g_pipe[n].cpu(), g_seq[n].cpu()) < 2 * TOL[torch.bfloat16], n


@pytest.mark.parametrize("dtype,T,B,d", [(torch.float32, 7, 3, 40), (torch.bfloat16, 16, 32, 256),
                                         (torch.bfloat16, 9, 5, 72)])
def test_phase_entry_points_compose_to_the_whole_call(dtype, T, B, d):
    """elman_gemm + elman_e1_recurrence_forward/backward + elman_column_sum, chained by
    hand, give bit for bit what elman_e1_forward / elman_e1_backward give."""
    inp = orc.make_e1_inputs(T, B, d, seed=41)
    dev, ref = round_inputs(inp, dtype)
    whole, _ = run_e1(inp, dtype)
    x2 = dev["x"].view(T * B, d)
    pre = H.gemm(H.GEMM_NT, x2, dev["W_x"], dev["b"]).view(T, B, d)
    h, out, v = H.e1_recurrence_forward(True, pre, dev["z"], dev["h0"], dev["W_h"])
    dv, dz, db = H.e1_recurrence_backward(dev["W_h"], dev["z"], h, v, dev["d_output"])
    dv2 = dv[:T].view(T * B, d)
    got = {"h": h, "output": out, "v": v, "dz": dz, "db": db,
           "dx": H.gemm(H.GEMM_NN, dv2, dev["W_x"]).view(T, B, d),
           "dW_x": H.gemm(H.GEMM_TN, dv2, x2),
           "dW_h": H.gemm(H.GEMM_TN, dv2, h[:T].view(T * B, d))}
    torch.cuda.synchronize()
    for k, t in got.items():
        assert torch.equal(t, whole[k]), k
    assert_close(errors(got, oracle_e1(ref)), TOL[dtype], "phases vs oracle")
    cs = H.column_sum(dv2)
    assert orc.rel_err(cs.float().cpu(), whole["db"].float().cpu()) < TOL[dtype]
    # accumulate and the carried gradient
    acc = H.gemm(H.GEMM_NN, dv2, dev["W_x"], out=got["dx"].view(T * B, d).clone(), accumulate=True)
    assert orc.rel_err(acc.float().cpu(), 2 * got["dx"].view(T * B, d).float().cpu()) < 1e-2
    with pytest.raises(Exception):
        H.gemm(7, dv2, dev["W_x"])


@pytest.mark.parametrize("dtype,batch,dim", [(torch.float32, 3, 72), (torch.bfloat16, 5, 136)])
def test_pipelined_ladder_lm_on_the_cuda_core_kernels(dtype, batch, dim):
    """Shapes the tensor-core recurrence does not take (fp32; odd sizes) run the pipeline on
    the cooperative CUDA-core kernels: same results as layer by layer."""
    from elman_b200.ladder_lm import LadderLM, zipf_tokens
    torch.manual_seed(5)
    model = LadderLM(vocab_size=256, dim=dim, depth=3, level=1, r_h_mode="none").cuda().to(dtype)
    tokens = zipf_tokens(batch, 41, seed=9).cuda()
    loss_seq, g_seq = _lm_step(model, tokens)
    model.pipeline_chunks = 3
    loss_pipe, g_pipe = _lm_step(model, tokens)
    tol = TOL[dtype] * (50 if dtype == torch.float32 else 1)   # fp32: sums reordered over chunks
    assert abs(loss_pipe - loss_seq) < tol * abs(loss_seq)
    for n in g_seq:
        assert orc.rel_err(g_pipe[n].cpu(), g_seq[n].cpu()) < tol, n


def test_pipelined_ladder_lm_level0_matches_sequential():
    """The E0 layer runs the same pipeline (E1's projection/recurrence nodes, gate from a
    second projection)."""
    from elman_b200.ladder_lm import LadderLM, zipf_tokens
    torch.manual_seed(8)
    model = LadderLM(vocab_size=256, dim=256, depth=3, level=0, r_h_mode="free").cuda().bfloat16()
    with torch.no_grad():       # keep the free recurrent matrices contractive
        for layer in model.layers:
            layer.cell.W_h.mul_(0.5)
    tokens = zipf_tokens(8, 65, seed=4).cuda()
    loss_seq, g_seq = _lm_step(model, tokens)
    model.pipeline_chunks = 4
    for _ in range(2):
        loss_pipe, g_pipe = _lm_step(model, tokens)
        assert abs(loss_pipe - loss_seq) < 2e-2 * abs(loss_seq)
        for n in g_seq:
            assert orc.rel_err(g_pipe[n].cpu(), g_seq[n].cpu()) < TOL[torch.bfloat16], n


@pytest.mark.parametrize("dtype,T,B,d,r,edges", [
    (torch.float32, 10, 3, 40, 6, (0, 4, 10)),
    (torch.bfloat16, 24, 16, 256, 32, (0, 8, 9, 24)),     # single-cluster tcgen05 kernel
    (torch.bfloat16, 12, 32, 384, 48, (0, 5, 12)),
    (torch.bfloat16, 9, 3, 72, 10, (0, 3, 9)),            # CUDA-core bf16 kernel
])
def test_e5_chained_chunks_match_oracle_and_whole_sequence(dtype, T, B, d, r, edges):
    from _gpu_cases import E5W, oracle_e5, run_e5
    inp = orc.make_e5_inputs(T, B, d, r, seed=61)
    dev, ref = round_inputs(inp, dtype)
    w = [dev[k] for k in E5W]
    state, fwd = dev["h0"], []
    for t0, t1 in zip(edges[:-1], edges[1:]):
        x = dev["x"][t0:t1].contiguous()
        h, out, v = H.pure_lowrank_elman_forward(True, x, state, *w, dev["b"])
        fwd.append((x, h, out, v))
        state = h[-1].contiguous()
    carry, dxs, sums = None, [], None
    for (x, h, out, v), t0, t1 in reversed(list(zip(fwd, edges[:-1], edges[1:]))):
        res = H.pure_lowrank_elman_backward_carry(*w, x, h, v, dev["d_output"][t0:t1].contiguous(),
                                                  carry)
        carry = res[8]
        dxs.insert(0, res[0])
        parts = [t.float() for t in res[1:8]]
        sums = parts if sums is None else [a + b for a, b in zip(sums, parts)]
    torch.cuda.synchronize()
    got = {"output": torch.cat([f[2] for f in fwd]),
           "h": torch.cat([fwd[0][1][:1]] + [f[1][1:] for f in fwd]), "dx": torch.cat(dxs)}
    got.update(dict(zip(("dU_h", "dV_h", "dU_x", "dV_x", "dU_z", "dV_z", "db"), sums)))
    assert_close(errors(got, oracle_e5(ref)), TOL[dtype], "E5 chunked vs oracle")
    whole, _ = run_e5(inp, dtype)
    for k in ("output", "h", "dx"):
        assert torch.equal(got[k], whole[k]), k


def test_pipelined_ladder_lm_level5_matches_sequential():
    from elman_b200.ladder_lm import LadderLM, zipf_tokens
    torch.manual_seed(12)
    model = LadderLM(vocab_size=256, dim=256, depth=3, level=5, rank=32).cuda().bfloat16()
    tokens = zipf_tokens(8, 65, seed=6).cuda()
    loss_seq, g_seq = _lm_step(model, tokens)
    model.pipeline_chunks = 4
    for _ in range(2):
        loss_pipe, g_pipe = _lm_step(model, tokens)
        assert abs(loss_pipe - loss_seq) < 2e-2 * abs(loss_seq)
        for n in g_seq:
            assert orc.rel_err(g_pipe[n].cpu(), g_seq[n].cpu()) < TOL[torch.bfloat16], n
