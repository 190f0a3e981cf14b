"""Byte-level language model around the E0 / E1 / E5 layers — the caller of the hot path.

Same structure and forward contract as the reference's LadderLM
(elman/models/ladder_lm.py:793-1070) for the three levels this package
implements: token embedding -> depth x (residual add + pre-RMSNorm with an fp32
residual stream -> Elman layer) -> final add + norm -> tied linear head ->
(cross-entropy).  Parameter names match (`embedding`, `layer_norms.i`,
`layers.i.*`, `norm`, `lm_head`), so checkpoints carry over.  Constructor
arguments that only concern other levels of the reference are accepted and
ignored.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .mamba_gated_elman import MambaGatedElman
from .pure_lowrank_elman import PureLowRankElman
from .stock_elman import StockElman

_LEVELS = {0: StockElman, 1: MambaGatedElman, 5: PureLowRankElman}


def get_ladder_level(level):
    """Layer class of an ablation-ladder level (0 = E0, 1 = E1, 5 = E5)."""
    try:
        return _LEVELS[int(level)]
    except (KeyError, ValueError):
        raise ValueError(f"level {level!r} is not implemented here (available: 0, 1, 5)")


class LadderLM(nn.Module):
    def __init__(self, vocab_size=256, dim=512, depth=12, level=0, expansion=1.0, rank=None,
                 dropout=0.0, r_h_mode="spectral_norm", r_h_init_gain=0.1, mamba2_init=False,
                 use_conv=False, d_conv=4, loss_chunk_size=0, **unused):
        super().__init__()
        self.vocab_size = vocab_size
        self.dim = dim
        self.depth = depth
        self.level = level
        self.rank = rank
        self.r_h_mode = r_h_mode
        self.loss_chunk_size = loss_chunk_size
        self.residual_in_fp32 = True
        layer_cls = get_ladder_level(level)
        self.embedding = nn.Embedding(vocab_size, dim)
        self.layer_norms = nn.ModuleList([nn.RMSNorm(dim) for _ in range(depth)])
        self.layers = nn.ModuleList([
            layer_cls(dim=dim, expansion=expansion, rank=rank, dropout=dropout, r_h_mode=r_h_mode,
                      r_h_init_gain=r_h_init_gain, mamba2_init=mamba2_init, use_conv=use_conv,
                      d_conv=d_conv)
            for _ in range(depth)])
        self.norm = nn.RMSNorm(dim)
        self.lm_head = nn.Linear(dim, vocab_size, bias=False)
        self.lm_head.weight = self.embedding.weight  # tied
        nn.init.normal_(self.embedding.weight, std=0.02)

    def forward(self, x, return_loss=False, return_prev_hiddens=False, prev_hiddens=None,
                prev_conv_buffers=None, actual_length=None, doc_boundaries=None):
        """x: [B,T] token ids ([B,T+1] with return_loss: inputs and shifted targets)."""
        if return_loss:
            inp, target = x[:, :-1], x[:, 1:]
        else:
            inp = x
        h = self.embedding(inp)
        if prev_hiddens is None:
            prev_hiddens = [None] * self.depth
        new_hiddens = []
        residual = None
        for i, (ln, layer) in enumerate(zip(self.layer_norms, self.layers)):
            residual = (h + residual) if residual is not None else h
            h = ln(residual.to(dtype=ln.weight.dtype))
            if self.residual_in_fp32:
                residual = residual.to(torch.float32)
            h, h_final = layer(h, prev_hiddens[i])
            new_hiddens.append(h_final)
        h = self.norm((h + residual).to(dtype=self.norm.weight.dtype))
        if not return_loss:
            logits = self.lm_head(h)
            return (logits, (new_hiddens, None)) if return_prev_hiddens else logits
        if actual_length is not None:
            positions = torch.arange(target.size(1), device=h.device).unsqueeze(0)
            target = target.clone()
            target[~(positions < (actual_length.unsqueeze(1) - 1))] = -100
        T_total = h.size(1)
        if self.loss_chunk_size > 0 and T_total > self.loss_chunk_size:
            total, count = h.new_zeros(()), 0
            for t0 in range(0, T_total, self.loss_chunk_size):
                t1 = min(t0 + self.loss_chunk_size, T_total)
                tc = target[:, t0:t1]
                total = total + F.cross_entropy(self.lm_head(h[:, t0:t1]).reshape(-1, self.vocab_size),
                                                tc.reshape(-1), ignore_index=-100, reduction="sum")
                count = count + (tc != -100).sum()
            loss = total / count.clamp(min=1)
        else:
            loss = F.cross_entropy(self.lm_head(h).view(-1, self.vocab_size), target.reshape(-1),
                                   ignore_index=-100)
        return (loss, (new_hiddens, None)) if return_prev_hiddens else loss

    def get_num_params(self):
        return sum(p.numel() for p in self.parameters())


def zipf_tokens(batch, length, seed, vocab=256, s=1.1):
    """Seeded i.i.d. Zipf(s) token ids over `vocab` symbols with a fixed random
    assignment of ranks to byte values: the synthetic stand-in for byte-level text."""
    g = torch.Generator().manual_seed(seed)
    p = torch.arange(1, vocab + 1, dtype=torch.float64) ** (-s)
    perm = torch.randperm(vocab, generator=torch.Generator().manual_seed(4321))
    ranks = torch.multinomial(p / p.sum(), batch * length, replacement=True, generator=g)
    return perm[ranks].reshape(batch, length)
