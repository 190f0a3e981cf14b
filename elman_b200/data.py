"""Byte-stream data, checkpoints and hidden-state carry for the training loop — the plumbing
either side of the hot path in the reference's trainer.

  DocumentStreamDataset   one stream of raw bytes per rank, 0x1e-delimited documents
                          (elman/data/dataset.py:19-150 of the reference)
  BatchedStreamDataset    batch_size independent streams that persist across calls, as
                          truncated BPTT needs (elman/data/dataset.py:156-256)
  save_checkpoint / load_checkpoint
                          the dict and the `latest.pt` link of train_ladder.py:596-613
  carry_hidden / reset_hidden
                          detach the layers' final states for the next chunk and zero them at
                          document ends (train_ladder.py:456-475, :516-528)

Same constructor arguments, start positions (seeded per rank), return tuples and wrap-around
behaviour as the reference classes; the bytes are served from a read-only numpy memmap in
slices instead of Python lists of ints, and batches go out through pinned buffers.  Vocabulary
is the byte (0..255); every byte, the delimiter included, is a token.
"""
import os

import numpy as np
import torch

DOC_DELIMITER = 0x1E


def _open(path):
    data = np.memmap(path, dtype=np.uint8, mode="r")
    if data.shape[0] == 0:
        raise ValueError(f"{path} is empty")
    return data


def _next_document(data, pos):
    """Index just after the next delimiter at or after `pos` (0 if there is none: wrap)."""
    n = data.shape[0]
    step = 1 << 16
    while pos < n:
        hit = np.flatnonzero(data[pos:pos + step] == DOC_DELIMITER)
        if hit.size:
            nxt = pos + int(hit[0]) + 1
            return (nxt if nxt < n else 0), nxt >= n
        pos += step
    return 0, True


def _read(data, pos, count):
    """`count` bytes from `pos`, wrapping at the end of the file -> (array, new pos, wraps)."""
    n = data.shape[0]
    out = np.empty(count, dtype=np.uint8)
    done, wraps = 0, 0
    while done < count:
        if pos >= n:
            pos = 0
            wraps += 1
        take = min(count - done, n - pos)
        out[done:done + take] = data[pos:pos + take]
        done += take
        pos += take
    return out, pos, wraps


class DocumentStreamDataset(torch.utils.data.Dataset):
    """One sequential byte stream; every __getitem__ returns the next chunk_size bytes as
    (chunk int64 [chunk_size], False, chunk_size)."""

    def __init__(self, data_path, chunk_size, rank=0, world_size=1, seed=42):
        self.chunk_size = chunk_size
        self.rank, self.world_size = rank, world_size
        self.data = _open(data_path)
        self.file_size = int(self.data.shape[0])
        rng = np.random.RandomState(seed + rank)
        self.position = int(rng.randint(0, max(1, self.file_size - 1000)))
        self.chunks_served = self.docs_completed = self.bytes_processed = self.wraps = 0
        self.position, wrapped = _next_document(self.data, self.position)
        self.wraps += int(wrapped)

    def __len__(self):
        return 1_000_000_000

    def __getitem__(self, idx):
        raw, self.position, wraps = _read(self.data, self.position, self.chunk_size)
        self.wraps += wraps
        self.bytes_processed += self.chunk_size
        self.chunks_served += 1
        return torch.from_numpy(raw.astype(np.int64)), False, self.chunk_size

    def get_stats(self):
        return {"chunks_served": self.chunks_served, "docs_completed": self.docs_completed,
                "bytes_processed": self.bytes_processed, "wraps": self.wraps,
                "position": self.position}

    def get_batch(self, batch_size, device=None):
        """-> (chunks [batch_size, chunk_size] int64, is_doc_end [batch_size] bool,
        actual_lengths [batch_size] int64); staged in pinned memory when a device is given."""
        pin = device is not None and torch.cuda.is_available()
        if getattr(self, "_chunks", None) is None or self._chunks.shape[0] != batch_size:
            self._chunks = torch.empty(batch_size, self.chunk_size, dtype=torch.long, pin_memory=pin)
            self._ends = torch.zeros(batch_size, dtype=torch.bool, pin_memory=pin)
            self._lens = torch.full((batch_size,), self.chunk_size, dtype=torch.long, pin_memory=pin)
        for i in range(batch_size):
            self._chunks[i] = self[0][0]
        if device is not None:
            return (self._chunks.to(device, non_blocking=True), self._ends.to(device, non_blocking=True),
                    self._lens.to(device, non_blocking=True))
        return self._chunks.clone(), self._ends.clone(), self._lens.clone()


class BatchedStreamDataset:
    """batch_size streams, stream i of rank r starting near (r*batch_size + i)/(total streams) of
    the file (plus a seeded jitter, then forward to the next document); chunk i of one call
    continues chunk i of the previous call."""

    def __init__(self, data_path, batch_size, chunk_size, rank=0, world_size=1, seed=42):
        self.batch_size, self.chunk_size = batch_size, chunk_size
        self.data = _open(data_path)
        self.file_size = int(self.data.shape[0])
        rng = np.random.RandomState(seed + rank * 1000)
        total = batch_size * world_size
        self.positions = []
        for i in range(batch_size):
            base = (rank * batch_size + i) * self.file_size // total
            jitter = int(rng.randint(0, max(1, self.file_size // (total * 10))))
            pos, _ = _next_document(self.data, (base + jitter) % self.file_size)
            self.positions.append(pos)
        pin = torch.cuda.is_available()
        self._chunks = torch.empty(batch_size, chunk_size, dtype=torch.long, pin_memory=pin)
        self._ends = torch.zeros(batch_size, dtype=torch.bool, pin_memory=pin)

    def get_batch(self, device=None):
        """-> (chunks [batch_size, chunk_size] int64, is_doc_end [batch_size] bool)."""
        for i in range(self.batch_size):
            raw, self.positions[i], _ = _read(self.data, self.positions[i], self.chunk_size)
            self._chunks[i] = torch.from_numpy(raw.astype(np.int64))
        if device is not None:
            return self._chunks.to(device, non_blocking=True), self._ends.to(device, non_blocking=True)
        return self._chunks.clone(), self._ends.clone()


# ------------------------------------------------------------------ hidden-state carry

def carry_hidden(next_hidden):
    """The layers' final states, detached, as the next chunk's prev_hiddens (lists and tuples
    of states are walked, None passes through)."""
    def detach(h):
        if h is None:
            return None
        if isinstance(h, (list, tuple)):
            return type(h)(detach(e) for e in h)
        return h.detach()
    return None if next_hidden is None else [detach(h) for h in next_hidden]


def reset_hidden(hidden_state, is_doc_end):
    """Zeroes the state of every sequence whose last chunk ended a document."""
    def reset(h):
        if h is None:
            return None
        if isinstance(h, (list, tuple)):
            return type(h)(reset(e) for e in h)
        keep = ~is_doc_end.view(-1, *([1] * (h.dim() - 1)))
        return h * keep.to(h.dtype)
    return None if hidden_state is None else [reset(h) for h in hidden_state]


# ------------------------------------------------------------------------ checkpoints

def save_checkpoint(output_dir, model, optimizer, step, loss, tokens_seen, args=None, level=1):
    """Writes level{L}_step{S}_loss{X}.pt with the reference's keys and re-points latest.pt."""
    os.makedirs(output_dir, exist_ok=True)
    name = f"level{level}_step{step:06d}_loss{loss:.4f}.pt"
    path = os.path.join(output_dir, name)
    torch.save({"step": step, "model_state_dict": model.state_dict(),
                "optimizer_state_dict": optimizer.state_dict(), "loss": loss,
                "tokens_seen": tokens_seen, "args": dict(args or {})}, path)
    latest = os.path.join(output_dir, "latest.pt")
    if os.path.islink(latest) or os.path.exists(latest):
        os.unlink(latest)
    os.symlink(name, latest)
    return path


def load_checkpoint(path, model, optimizer=None, map_location=None):
    """Restores model (and optimizer) from a checkpoint of this package or of the reference
    (same parameter names); returns the remaining entries (step, loss, tokens_seen, args)."""
    ckpt = torch.load(path, map_location=map_location, weights_only=False)
    model.load_state_dict(ckpt["model_state_dict"])
    if optimizer is not None and "optimizer_state_dict" in ckpt:
        optimizer.load_state_dict(ckpt["optimizer_state_dict"])
    return {k: v for k, v in ckpt.items() if k not in ("model_state_dict", "optimizer_state_dict")}
