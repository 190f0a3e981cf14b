"""Data, checkpoint and hidden-carry plumbing around the hot path (CPU): the byte-stream
datasets against a direct restatement of the reference classes' behaviour
(elman/data/dataset.py:19-150, :156-256) on a synthetic file, the checkpoint dictionary of
train_ladder.py:596-613, and the TBPTT carry of :456-475, :516-528."""
import os

import numpy as np
import torch

from elman_b200 import data as D


def _corpus(tmp_path, n=20000, seed=0):
    rng = np.random.RandomState(seed)
    raw = rng.randint(32, 127, size=n).astype(np.uint8)
    raw[rng.choice(n, size=40, replace=False)] = D.DOC_DELIMITER
    path = os.path.join(tmp_path, "corpus.bin")
    raw.tofile(path)
    return path, raw


def _ref_scan(raw, pos):
    n = len(raw)
    while pos < n and raw[pos] != D.DOC_DELIMITER:
        pos += 1
    return pos + 1 if pos < n else 0


def test_document_stream_serves_the_file_in_order_and_wraps(tmp_path):
    path, raw = _corpus(str(tmp_path))
    ds = D.DocumentStreamDataset(path, chunk_size=777, rank=3, world_size=8, seed=42)
    start = _ref_scan(raw, int(np.random.RandomState(42 + 3).randint(0, len(raw) - 1000)))
    if start >= len(raw):
        start = 0
    pos = start
    for _ in range(60):                           # 46 620 bytes: wraps the 20 000-byte file twice
        chunk, is_end, length = ds[0]
        want = np.take(raw, np.arange(pos, pos + 777) % len(raw))
        assert torch.equal(chunk, torch.from_numpy(want.astype(np.int64)))
        assert is_end is False and length == 777 and chunk.dtype == torch.long
        pos = (pos + 777) % len(raw)
    assert ds.get_stats()["wraps"] == 2 and ds.get_stats()["chunks_served"] == 60
    chunks, ends, lens = ds.get_batch(4)
    assert chunks.shape == (4, 777) and not ends.any() and int(lens[0]) == 777


def test_batched_streams_continue_per_element_and_differ_per_rank(tmp_path):
    path, raw = _corpus(str(tmp_path))
    a = D.BatchedStreamDataset(path, batch_size=4, chunk_size=100, rank=0, world_size=2, seed=7)
    b = D.BatchedStreamDataset(path, batch_size=4, chunk_size=100, rank=1, world_size=2, seed=7)
    first, _ = a.get_batch()
    second, ends = a.get_batch()
    assert first.shape == (4, 100) and ends.dtype == torch.bool
    for i in range(4):                            # chunk i continues where chunk i stopped
        s = a.positions[i] - 200
        want = np.take(raw, np.arange(s, s + 200) % len(raw))
        got = torch.cat([first[i], second[i]]).numpy()
        assert np.array_equal(got, want)
        assert raw[(s - 1) % len(raw)] == D.DOC_DELIMITER      # started on a document boundary
    assert not torch.equal(first, b.get_batch()[0])             # other rank, other streams
    # start positions as the reference spreads them
    rng = np.random.RandomState(7)
    for i in range(4):
        base = i * len(raw) // 8
        jitter = int(rng.randint(0, max(1, len(raw) // 80)))
        assert a.positions[i] - 200 == _ref_scan(raw, (base + jitter) % len(raw))


def test_hidden_carry_detaches_and_resets_at_document_ends():
    h = [torch.randn(3, 5, requires_grad=True) * 2, None, (torch.ones(3, 2), torch.ones(3, 2))]
    c = D.carry_hidden(h)
    assert not c[0].requires_grad and c[1] is None and isinstance(c[2], tuple)
    r = D.reset_hidden(c, torch.tensor([False, True, False]))
    assert float(r[0][1].abs().sum()) == 0 and torch.equal(r[0][0], c[0][0])
    assert float(r[2][0][1].sum()) == 0 and float(r[2][0][2].sum()) == 2


def test_checkpoint_dictionary_and_latest_link(tmp_path):
    net = torch.nn.Linear(4, 3)
    opt = torch.optim.AdamW(net.parameters(), lr=1e-3)
    net(torch.randn(2, 4)).sum().backward()
    opt.step()
    path = D.save_checkpoint(str(tmp_path), net, opt, step=1000, loss=1.4321, tokens_seen=5,
                             args={"level": 1}, level=1)
    assert os.path.basename(path) == "level1_step001000_loss1.4321.pt"
    latest = os.path.join(str(tmp_path), "latest.pt")
    assert os.path.islink(latest) and os.readlink(latest) == os.path.basename(path)
    ckpt = torch.load(latest, weights_only=False)
    assert set(ckpt) == {"step", "model_state_dict", "optimizer_state_dict", "loss", "tokens_seen", "args"}
    net2 = torch.nn.Linear(4, 3)
    opt2 = torch.optim.AdamW(net2.parameters(), lr=1e-3)
    rest = D.load_checkpoint(latest, net2, opt2)
    assert rest["step"] == 1000 and rest["tokens_seen"] == 5
    assert torch.equal(net2.weight, net.weight)
    D.save_checkpoint(str(tmp_path), net, opt, step=2000, loss=1.2, tokens_seen=9)
    assert os.readlink(latest).startswith("level1_step002000")
