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

from . import fused_ops
from .mamba_gated_elman import MambaGatedElman
from .pure_lowrank_elman import PureLowRankElman
from .siblings import E32NoPresilu, E33SelfGate, E57LearnedRadius, LowRankElman
from .stock_elman import StockElman

_LEVELS = {0: StockElman, 1: MambaGatedElman, 4: LowRankElman, 5: PureLowRankElman,
           32: E32NoPresilu, 33: E33SelfGate, 57: E57LearnedRadius}


def get_ladder_level(level):
    """Layer class of an ablation-ladder level (0 = E0, 1 = E1, 4 = E1 with a low-rank recurrent
    matrix, 5 = E5, 32 / 33 / 57 = the E1 siblings without pre-silu, with a self gate, with a
    learned spectral radius)."""
    try:
        return _LEVELS[int(level)]
    except (KeyError, ValueError):
        raise ValueError(f"level {level!r} is not implemented here "
                         f"(available: {sorted(_LEVELS)})")


class LadderLM(nn.Module):
    def __init__(self, vocab_size=256, dim=512, depth=12, level=0, expansion=1.0, rank=None,
                 dropout=0.0, r_h_mode="spectral_norm", r_h_init_gain=0.1, mamba2_init=False,
                 use_conv=False, d_conv=4, loss_chunk_size=0, pipeline_chunks=0,
                 pipeline_streams=0, fused_ops=True, **unused):
        super().__init__()
        # fused_ops (not a reference argument): residual add + RMSNorm as one kernel each way
        # and the head as a library GEMM (the reference's fused_add_norm switch, ladder_lm.py
        # :986-1003, selects a Triton kernel for the same purpose); False = framework ops
        self.fused_ops = bool(fused_ops)
        # pipeline_chunks > 1 (not a reference argument): run the layer stack as a
        # wavefront over (layer, time chunk) on several CUDA streams, see _pipelined_layers
        self.pipeline_chunks = int(pipeline_chunks)
        self.pipeline_streams = int(pipeline_streams)
        # overlapped recurrences run with their smallest footprint (ELMAN_FLAG_COMPACT)
        self.pipeline_flags = 1
        self._streams = {}
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
        if prev_hiddens is None:
            prev_hiddens = [None] * self.depth
        sink = fused_ops.get_grad_sink()
        if sink is not None and torch.is_grad_enabled():
            sink.begin_pass()
        if return_loss and actual_length is not None:
            positions = torch.arange(target.size(1), device=target.device).unsqueeze(0)
            target = target.clone()
            target[~(positions < (actual_length.unsqueeze(1) - 1))] = -100
        time_major = False
        if self._can_pipeline(inp) and return_loss and self.loss_chunk_size == 0:
            # Pipeline with the loss: final norm, head and cross-entropy run per time chunk as
            # soon as the last layer has produced it — beside the rest of the wavefront instead
            # of after it on the whole sequence, and in the backward pass the last chunk's head
            # gradient is all the first recurrence waits for.  The mean over tokens is the sum
            # of the chunks' sums over the number of counted targets.
            target_tm = target.t().contiguous()          # [T,B]: the small integer side transposed

            def chunk_loss(c, hc, rc, t0, t1):
                hn, _ = self._add_norm(self.norm, hc, rc, last=True)
                return F.cross_entropy(self._head(hn).view(-1, self.vocab_size),
                                       target_tm[t0:t1].reshape(-1), ignore_index=-100,
                                       reduction="sum")
            sums, _, new_hiddens = self._pipelined_layers(self._embed_chunks(inp), prev_hiddens,
                                                          per_chunk=chunk_loss)
            count = target.numel() if actual_length is None else (target != -100).sum().clamp(min=1)
            loss = torch.stack(sums).sum() / count
            return (loss, (new_hiddens, None)) if return_prev_hiddens else loss
        if self._can_pipeline(inp):
            h, residual, new_hiddens = self._pipelined_layers(self._embed_chunks(inp), prev_hiddens)
            time_major = True
        else:
            h = self.embedding(inp)
            new_hiddens = []
            residual = None
            for i, (ln, layer) in enumerate(zip(self.layer_norms, self.layers)):
                h, residual = self._add_norm(ln, h, residual, group=i)
                h, h_final = layer(h, prev_hiddens[i])
                new_hiddens.append(h_final)
        h, _ = self._add_norm(self.norm, h, residual, last=True)
        if time_major and (not return_loss or self.loss_chunk_size > 0):
            h = h.transpose(0, 1).contiguous()   # back to [B,T,D] for the callers below
            time_major = False
        if not return_loss:
            logits = self._head(h)
            return (logits, (new_hiddens, None)) if return_prev_hiddens else logits
        if time_major:
            # the mean over tokens does not care about their order: transpose the small
            # integer targets instead of the activations
            target = target.transpose(0, 1)
        T_total = h.size(1)
        if self.loss_chunk_size > 0 and T_total > self.loss_chunk_size:
            total, count = h.new_zeros(()), 0
            for t0 in range(0, T_total, self.loss_chunk_size):
                t1 = min(t0 + self.loss_chunk_size, T_total)
                tc = target[:, t0:t1]
                total = total + F.cross_entropy(self._head(h[:, t0:t1]).reshape(-1, self.vocab_size),
                                                tc.reshape(-1), ignore_index=-100, reduction="sum")
                count = count + (tc != -100).sum()
            loss = total / count.clamp(min=1)
        else:
            loss = F.cross_entropy(self._head(h).view(-1, self.vocab_size), target.reshape(-1),
                                   ignore_index=-100)
        return (loss, (new_hiddens, None)) if return_prev_hiddens else loss

    def _add_norm(self, norm, h, residual, last=False, group=None):
        """residual = h + residual (fp32 stream); h = norm(residual in the layer's dtype).
        Returns (h, residual); with `last` the residual is not needed any more.  `group`: the
        layer whose (layer, chunk) unit this op opens (told to the gradient sink, if any)."""
        if self.fused_ops and self.residual_in_fp32 and fused_ops.library_handles(h) \
                and h.dtype == norm.weight.dtype:
            sink = fused_ops.get_grad_sink()
            if group is not None and sink is not None and torch.is_grad_enabled():
                sink.expect_unit(group)
            else:
                group = None
            return fused_ops.AddRMSNormFunction.apply(
                h, residual, norm.weight, fused_ops.rmsnorm_eps(norm, h.dtype), group)
        residual = (h + residual) if residual is not None else h
        h = norm(residual.to(dtype=norm.weight.dtype))
        if self.residual_in_fp32 and not last:
            residual = residual.to(torch.float32)
        return h, residual

    def _head(self, h):
        if self.fused_ops and fused_ops.library_handles(h) and h.dtype == self.lm_head.weight.dtype:
            return fused_ops.linear(h.contiguous(), self.lm_head.weight)
        return self.lm_head(h)

    # ------------------------------------------------------------------ pipeline
    #
    # A recurrence launch is a chain of T dependent steps that keeps only a
    # fraction of the GPU's SMs busy, and layer l+1 at time t needs layer l only
    # up to time t.  Cutting the sequence into C time chunks turns the depth x C
    # (layer, chunk) units into a wavefront: unit (l, c) needs (l-1, c) for its
    # input and (l, c-1) for its initial state.  Each layer's recurrences run back to
    # back on a stream of their own while the time-parallel ops before and after them
    # (norms, projections, weight-gradient GEMMs) run on two further streams per layer,
    # so up to `depth` recurrences overlap each other and everything else.  Autograd runs every backward op on
    # the stream of its forward op, so the backward pass forms the mirrored
    # wavefront by itself.  Chained chunks reproduce the unchunked layer exactly
    # (state carried forward, pre-activation gradient carried backward).

    def _can_pipeline(self, inp):
        h = inp
        return (self.pipeline_chunks > 1 and h.is_cuda and h.size(1) >= 2 * self.pipeline_chunks
                and all(getattr(layer, "supports_time_chunks", False) for layer in self.layers))

    def _pipeline_streams(self, device, n_rec):
        """Per layer one stream for the ops before the recurrence and one for those after it;
        `n_rec` streams for the recurrences themselves, dealt to the layers round-robin."""
        key = (device, n_rec)
        if key not in self._streams:
            # From the pool of high-priority streams: the framework hands out streams from a
            # fixed pool per priority and starts over when it is used up, and the gradient
            # sink, the host pipeline, graph capture and the communication stream draw from the
            # default pool — two logical streams on one CUDA stream would serialise units
            # that are meant to overlap.  (The priority itself changes nothing measurable.)
            mk = lambda n: [torch.cuda.Stream(device=device, priority=-1) for _ in range(n)]
            self._streams[key] = (mk(self.depth), mk(n_rec), mk(self.depth))
        return self._streams[key]

    def _recurrence_stream_count(self, h, chunk_len):
        """Recurrence launches that may be in flight at once.  The thread blocks of one
        launch wait for one another, so every set of launches that can run together must
        fit on the device together: one stream per layer while that holds."""
        if self.pipeline_streams > 0:
            return self.pipeline_streams
        # layers may differ in width and plan: the widest launch decides
        blocks = max(layer.chunk_recurrence_blocks(h.dtype, chunk_len, h.size(1),
                                                   self.pipeline_flags) for layer in self.layers)
        sms = torch.cuda.get_device_properties(h.device).multi_processor_count
        n = sms // blocks if blocks > 0 else 2
        return max(1, min(n, self.depth))

    def _chunk_edges(self, T):
        """Time-chunk boundaries.  `pipeline_sizes` (a list of chunk lengths summing to T)
        overrides the uniform cut into `pipeline_chunks` chunks.  (Tapered schedules — short
        chunks at both ends to shorten the wavefront's ramp — measured no better than the
        uniform cut at depth 6, T = 512: the step is bound by total SM time, not by the ramp.)"""
        sizes = getattr(self, "pipeline_sizes", None)
        if sizes and sum(sizes) == T and all(n > 0 for n in sizes):
            edges = [0]
            for n in sizes:
                edges.append(edges[-1] + int(n))
            return edges
        C = self.pipeline_chunks
        return [(T * c) // C for c in range(C + 1)]

    def _embed_chunks(self, inp):
        """Embedding rows of inp [B,T] for the pipeline, which is time-major throughout: one
        [T,B,D] tensor — or, with the fused ops, one tensor per time chunk, so that a chunk's
        share of the embedding gradient is formed (as a one-hot GEMM) as soon as the backward
        wavefront has left layer 0's unit of that chunk rather than after the whole pass."""
        tokens = inp.t()
        if self.fused_ops and fused_ops.library_handles(self.embedding.weight):
            tokens = tokens.contiguous()
            edges = self._chunk_edges(tokens.size(0))
            return [fused_ops.embedding_rows(tokens[edges[c]:edges[c + 1]], self.embedding.weight)
                    for c in range(len(edges) - 1)]
        return self.embedding(tokens)

    def _pipelined_layers(self, h, prev_hiddens, per_chunk=None):
        """h: [T,B,D] time-major (or its time chunks as a list, cut at `_chunk_edges`)
        -> (h, residual, final states), both outputs [T,B,D]; with
        `per_chunk(c, h_c, residual_c, t0, t1)` the last layer's chunks are handed to it one by
        one on the caller's stream as they become ready, and its results are returned as a
        list in place of h (residual None)."""
        from .mamba_gated_elman import ChunkLink
        given = list(h) if isinstance(h, (list, tuple)) else None
        if given is not None:
            h = given[0]
        T = h.size(0) if given is None else sum(x.size(0) for x in given)
        B = h.size(1)              # time-major [T,B,D]
        edges = self._chunk_edges(T)
        C = len(edges) - 1
        main = torch.cuda.current_stream(h.device)
        pre_streams, rec_streams, post_streams = self._pipeline_streams(
            h.device, self._recurrence_stream_count(h, edges[1] - edges[0]))
        shared, shared_t = [None] * self.depth, [None] * self.depth
        # time-major chunks [Tc,B,D]: the cell's own layout, so no layer transposes anything;
        # slices along the leading dimension are contiguous views, nothing is copied
        h_chunks = given if given is not None else [h[edges[c]:edges[c + 1]] for c in range(C)]
        start = torch.cuda.Event()   # everything the side streams read is enqueued before this
        start.record(main)
        for s in pre_streams + rec_streams + post_streams:
            s.wait_event(start)
        res_chunks = [None] * C
        states = []
        post_done = [[None] * C for _ in range(self.depth)]

        def record(stream):
            ev = torch.cuda.Event()
            ev.record(stream)
            return ev

        for i, (ln, layer) in enumerate(zip(self.layer_norms, self.layers)):
            sp, sr, sq = pre_streams[i], rec_streams[i % len(rec_streams)], post_streams[i]
            with torch.cuda.stream(sp):
                # what all chunks of this layer share, on the layer's own stream: the effective
                # W_h (the spectral-norm power iteration) of layer i is needed only when the
                # wavefront reaches layer i, so the six of them overlap instead of queueing up
                # in front of the first recurrence; likewise their backward passes
                shared[i] = layer.chunk_weights()
                # one transposed copy per layer and pass for the backward recurrences of all chunks
                shared_t[i] = (shared[i].detach().t().contiguous()
                               if (shared[i] is not None and torch.is_grad_enabled()) else None)
            d_inner = getattr(layer, "d_inner", self.dim)
            state = prev_hiddens[i]
            state = (torch.zeros(B, d_inner, device=h.device, dtype=h.dtype) if state is None
                     else state.detach())
            state.record_stream(sr)
            if shared[i] is not None:
                shared[i].record_stream(sr)
            if shared_t[i] is not None:
                shared_t[i].record_stream(sr)

            def issue_pre(c):
                # residual add, norm, input projections: everything up to the recurrence
                with torch.cuda.stream(sp):
                    if i > 0:
                        sp.wait_event(post_done[i - 1][c])
                    hin, rin = h_chunks[c], res_chunks[c]
                    hin.record_stream(sp)
                    if rin is not None:
                        rin.record_stream(sp)
                    hn, residual = self._add_norm(ln, hin, rin, group=i)
                    link = ChunkLink()
                    pre, z = layer.chunk_pre(hn, shared[i], link)
                    return pre, z, link, residual, record(sp)

            ahead = issue_pre(0)
            for c in range(C):
                pre, z, link, residual, pre_ev = ahead
                with torch.cuda.stream(sr):
                    sr.wait_event(pre_ev)
                    pre.record_stream(sr)
                    if z is not None:
                        z.record_stream(sr)
                    cell_out, state = layer.chunk_rec(pre, z, state, shared[i], link,
                                                      self.pipeline_flags, shared_t[i])
                    rec_ev = record(sr)
                if c + 1 < C:   # enqueued before this chunk's post ops: the next recurrence
                    ahead = issue_pre(c + 1)    # of this layer never waits behind them
                with torch.cuda.stream(sq):
                    sq.wait_event(rec_ev)
                    cell_out.record_stream(sq)
                    out = layer.chunk_post(cell_out)
                    post_done[i][c] = record(sq)
                h_chunks[c], res_chunks[c] = out, residual
            states.append(state)
        results = []
        for c in range(C):
            main.wait_event(post_done[-1][c])
            h_chunks[c].record_stream(main)
            res_chunks[c].record_stream(main)
            if per_chunk is not None:
                results.append(per_chunk(c, h_chunks[c], res_chunks[c], edges[c], edges[c + 1]))
        for st in states:
            st.record_stream(main)
        for s in pre_streams + rec_streams + post_streams:
            main.wait_event(record(s))   # every stream rejoins (required under graph capture)
        if per_chunk is not None:
            return results, None, [st.detach() for st in states]
        # both still time-major [T,B,D]
        return torch.cat(h_chunks, dim=0), torch.cat(res_chunks, dim=0), [st.detach() for st in states]

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
